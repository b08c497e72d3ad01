"""Pins the numpy oracle: golden vectors made by the reference's PyTorch module
(tests/golden/make_golden.py) and the closed-form known-answer tests of the reference's
tests/test_kernels.cu (:91-120 causal softmax, :210-284 tiled attention)."""
import math

import numpy as np
import pytest

import os

from conftest import GOLDEN_DIR, golden_names, load_golden
from oracle import attention_oracle as orc

TOL = 1e-5  # the FP32 parity gate of the path (max-abs)


@pytest.mark.parametrize("name", golden_names())
def test_core_matches_reference_module(name):
    g = load_golden(name)
    B, T, C, H = (int(x) for x in g["shape"])
    d = C // H
    scale = 1.0 / math.sqrt(d)
    out, m, l = orc.attention_forward(g["q"], g["k"], g["v"], scale)
    assert orc.compute_metrics(out, g["out"])["max_abs"] <= TOL
    assert orc.compute_metrics(m, g["m"])["max_abs"] <= TOL
    assert orc.compute_metrics(l / g["l"], np.ones_like(l))["max_abs"] <= TOL
    dq, dk, dv = orc.attention_backward(g["q"], g["k"], g["v"], g["out"], g["dout"], g["m"], g["l"], scale)
    for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert orc.compute_metrics(got, g[key])["max_abs"] <= TOL, key


@pytest.mark.parametrize("name", [n for n in golden_names() if n.startswith(("config1", "paritygate"))])
def test_layout_ops_match_reference_module(name):
    g = load_golden(name)
    B, T, C, H = (int(x) for x in g["shape"])
    d = C // H
    q, k, v = orc.qkv_split_transpose_forward(g["qkv"], B, T, H, d)
    assert np.array_equal(q, g["q"]) and np.array_equal(k, g["k"]) and np.array_equal(v, g["v"])
    assert np.array_equal(orc.qkv_split_transpose_backward(g["dq"], g["dk"], g["dv"]), g["dqkv"])
    assert np.array_equal(orc.head_merge_transpose_forward(g["out"]), g["merged"])
    assert np.array_equal(orc.head_merge_transpose_backward(g["dmerged"], H), g["dout"])


@pytest.mark.parametrize("name", [n for n in golden_names() if n.startswith(("config1", "paritygate"))])
def test_block_matches_reference_module(name):
    g = load_golden(name)
    B, T, C, H = (int(x) for x in g["shape"])
    r = orc.mha_block_forward_backward(g["x"], g["w_qkv"], g["b_qkv"], g["w_proj"], g["b_proj"], g["dY"], H)
    for key in ("y", "dx", "dw_qkv", "db_qkv", "dw_proj", "db_proj", "qkv", "dqkv"):
        assert orc.compute_metrics(r[key], g[key])["max_abs"] <= TOL, key


def test_causal_softmax_known_answer():
    # tests/test_kernels.cu:91-120: all-ones 4x4 scores, scale 1
    T = 4
    p = orc.causal_softmax_forward(np.ones((T, T), np.float32), 1, 1, T, 1.0).reshape(T, T)
    assert abs(p[0, 0] - 1.0) < 1e-5 and abs(p[0, 1]) < 1e-5
    assert abs(p[1, 0] - 0.5) < 1e-4 and abs(p[1, 1] - 0.5) < 1e-4 and abs(p[1, 2]) < 1e-5
    assert np.all(np.triu(p, 1) == 0)


def test_tiled_attention_known_answer():
    # tests/test_kernels.cu:210-284: B=H=1, T=8, d=32, q=k=0.1, v=1, dO=0.5 -> every O element is 1
    T, d = 8, 32
    q = np.full((1, 1, T, d), 0.1, np.float32)
    v = np.ones((1, 1, T, d), np.float32)
    dO = np.full((1, 1, T, d), 0.5, np.float32)
    r = orc.attention_forward_backward(q, q.copy(), v, dO, 1.0 / math.sqrt(d))
    assert np.all(np.abs(r["out"] - 1.0) < 1e-3)
    for key in ("dq", "dk", "dv"):
        assert np.all(np.isfinite(r[key]))
    # uniform probabilities: row i attends to i+1 keys with weight 1/(i+1)
    assert np.allclose(r["l"].ravel(), np.arange(1, T + 1))


def test_softmax_backward_is_gradient_of_forward():
    rng = np.random.default_rng(0)
    B, H, T, scale = 1, 2, 9, 0.37
    s = rng.standard_normal((B * H * T, T))
    dp = rng.standard_normal((B * H * T, T))
    p = orc.causal_softmax_forward(s, B, H, T, scale)
    ds = orc.causal_softmax_backward(dp, p, B, H, T, scale)
    eps = 1e-6
    idx = (5, 2)
    s2 = s.copy(); s2[idx] += eps
    num = ((orc.causal_softmax_forward(s2, B, H, T, scale) - p) * dp).sum() / eps
    assert abs(num - ds[idx]) < 1e-5
    assert np.all(ds.reshape(B * H, T, T)[:, np.triu_indices(T, 1)[0], np.triu_indices(T, 1)[1]] == 0)


def test_bf16_round_matches_torch():
    import torch
    x = np.random.default_rng(1).standard_normal(4096).astype(np.float32) * 3
    want = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(orc.bf16_round(x), want)


def test_torch_port_agrees_with_numpy_oracle():
    import torch
    from oracle import torch_port
    rng = np.random.default_rng(5)
    q, k, v, dO = (rng.standard_normal((3, 70, 32)).astype(np.float32) for _ in range(4))
    scale = 1 / math.sqrt(32)
    out, dq, dk, dv = torch_port.forward_backward(*(torch.from_numpy(a) for a in (q, k, v, dO)), scale)
    ref = orc.attention_forward_backward(q, k, v, dO, scale)
    for got, key in ((out, "out"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert orc.compute_metrics(got.numpy(), ref[key])["max_abs"] <= TOL, key


@pytest.mark.parametrize("case", ["parity_audit", "parity_audit_d64"])
def test_gpt_port_matches_the_reference_generator(case):
    """oracle/torch_gpt_port.py (the CPU baseline of the full training step) against the files the reference's own
    golden generator wrote from PyTorchGPT (pytorch_src/utils.py:167-240): logits, loss and the flat gradient in the
    CUDA blob order, at the gates of scripts/compare_parity.py:108-117."""
    import torch
    from oracle import torch_gpt_port as gpt
    d = os.path.join(GOLDEN_DIR, case)
    B, T, C, L, H, V = (int(x) for x in open(os.path.join(d, "config.txt")).read().split())
    load = lambda n, dt=np.float32: np.fromfile(os.path.join(d, n), dtype=dt)
    flat = torch.from_numpy(load("pytorch_params.bin")).clone().requires_grad_(True)
    assert flat.numel() == gpt.num_parameters(V, T, C, L)
    idx = torch.from_numpy(load("inputs.bin", np.int32).astype(np.int64)).view(B, T)
    tgt = torch.from_numpy(load("targets.bin", np.int32).astype(np.int64)).view(B, T)
    logits, loss = gpt.gpt_forward(flat, idx, tgt, V, T, C, L, H)
    loss.backward()
    assert np.abs(logits.detach().numpy().ravel() - load("pytorch_logits.bin")).max() <= 1e-5
    assert abs(float(loss) - float(load("pytorch_loss.bin")[0])) <= 1e-5
    assert np.abs(flat.grad.numpy() - load("pytorch_grads.bin")).max() <= 5e-5


@pytest.mark.parametrize("case", ["parity_audit", "parity_audit_d64"])
def test_cross_entropy_oracle_matches_the_reference_generator(case):
    """oracle/cross_entropy_oracle.py against the reference generator's own files: its loss from its logits and
    targets (1e-5, the gate of scripts/compare_parity.py:108-117), and d_logits against autograd of
    F.cross_entropy, the loss of pytorch_src/model.py:118-121."""
    import torch
    from oracle import cross_entropy_oracle as ce
    d = os.path.join(GOLDEN_DIR, case)
    B, T, C, L, H, V = (int(x) for x in open(os.path.join(d, "config.txt")).read().split())
    logits = np.fromfile(os.path.join(d, "pytorch_logits.bin"), dtype=np.float32).reshape(B * T, V)
    targets = np.fromfile(os.path.join(d, "targets.bin"), dtype=np.int32)
    dlogits, loss = ce.cross_entropy_forward_backward(logits, targets)
    assert abs(loss - float(np.fromfile(os.path.join(d, "pytorch_loss.bin"), dtype=np.float32)[0])) <= 1e-5
    lt = torch.from_numpy(logits.astype(np.float64)).requires_grad_(True)
    torch.nn.functional.cross_entropy(lt, torch.from_numpy(targets.astype(np.int64))).backward()
    assert np.abs(dlogits - lt.grad.numpy()).max() <= 1e-9
    # float32 arithmetic, as the reference kernel runs it, stays within the same gate
    d32, loss32 = ce.cross_entropy_forward_backward(logits, targets, dtype=np.float32)
    assert abs(loss32 - loss) <= 1e-5 and np.abs(d32 - dlogits).max() <= 1e-7
