"""GPU parity of the FP32 launch API (through the C ABI) against the golden vectors made by the
reference's PyTorch module and against the numpy oracle. Gate: max-abs <= 1e-5 (FP32 mode);
layout launchers must be bit-exact."""
import math

import numpy as np
import pytest
import torch

from conftest import golden_names, load_golden
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.fixture(scope="module")
def ops(pkg):
    pkg.ops.set_math_mode("fp32")
    return pkg.ops


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.float().cpu().numpy()


def max_abs(a, b):
    return orc.compute_metrics(a, b)["max_abs"]


@pytest.mark.parametrize("name", golden_names())
def test_attention_core_vs_golden(ops, name):
    g = load_golden(name)
    B, T, C, H = (int(x) for x in g["shape"])
    d = C // H
    scale = 1.0 / math.sqrt(d)
    q, k, v, dout = dev(g["q"]), dev(g["k"]), dev(g["v"]), dev(g["dout"])
    out, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
    m, l, ws = (torch.empty(B, H, T, device="cuda") for _ in range(3))
    ops.tiled_causal_attention_forward(q, k, v, out, B, H, T, d, scale, m, l)
    assert max_abs(host(out), g["out"]) <= TOL
    assert max_abs(host(m), g["m"]) <= TOL
    assert max_abs(host(l) / g["l"], np.ones_like(g["l"])) <= TOL  # l grows with T: relative
    ops.tiled_causal_attention_backward(q, k, v, out, dout, m, l, dq, dk, dv, ws, B, H, T, d, scale)
    assert max_abs(host(ws), orc.attention_precompute_dot_do_o(g["dout"], g["out"])) <= TOL
    for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert max_abs(host(got), g[key]) <= TOL, key
    # statistics are optional, as in the reference (m_out = l_out = nullptr)
    out2 = torch.empty_like(q)
    ops.tiled_causal_attention_forward(q, k, v, out2, B, H, T, d, scale)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("name", [n for n in golden_names() if n.startswith(("config1", "paritygate"))])
def test_layout_launchers_vs_golden_bit_exact(ops, name):
    g = load_golden(name)
    B, T, C, H = (int(x) for x in g["shape"])
    d = C // H
    q, k, v = (torch.empty(B, H, T, d, device="cuda") for _ in range(3))
    ops.qkv_split_transpose_forward(dev(g["qkv"]), q, k, v, B, T, H, d)
    assert np.array_equal(host(q), g["q"]) and np.array_equal(host(k), g["k"]) and np.array_equal(host(v), g["v"])
    dqkv = torch.empty(B, T, 3 * C, device="cuda")
    ops.qkv_split_transpose_backward(dev(g["dq"]), dev(g["dk"]), dev(g["dv"]), dqkv, B, T, H, d)
    assert np.array_equal(host(dqkv), g["dqkv"])
    merged = torch.empty(B, T, C, device="cuda")
    ops.head_merge_transpose_forward(dev(g["out"]), merged, B, H, T, d)
    assert np.array_equal(host(merged), g["merged"])
    dout = torch.empty(B, H, T, d, device="cuda")
    ops.head_merge_transpose_backward(dev(g["dmerged"]), dout, B, H, T, d)
    assert np.array_equal(host(dout), g["dout"])


def test_layout_scalar_path_when_d_is_odd(ops):
    """d % 4 != 0 takes the element-wise path (the reference's scalar kernels, attention.cu:54,115,326,363)."""
    B, T, H, d = 2, 5, 3, 6
    rng = np.random.default_rng(3)
    qkv = rng.standard_normal((B, T, 3 * H * d)).astype(np.float32)
    q, k, v = (torch.empty(B, H, T, d, device="cuda") for _ in range(3))
    ops.qkv_split_transpose_forward(dev(qkv), q, k, v, B, T, H, d)
    rq, rk, rv = orc.qkv_split_transpose_forward(qkv, B, T, H, d)
    assert np.array_equal(host(q), rq) and np.array_equal(host(k), rk) and np.array_equal(host(v), rv)
    back = torch.empty(B, T, 3 * H * d, device="cuda")
    ops.qkv_split_transpose_backward(q, k, v, back, B, T, H, d)
    assert np.array_equal(host(back), qkv)
    merged = torch.empty(B, T, H * d, device="cuda")
    ops.head_merge_transpose_forward(q, merged, B, H, T, d)
    assert np.array_equal(host(merged), orc.head_merge_transpose_forward(rq))
    again = torch.empty(B, H, T, d, device="cuda")
    ops.head_merge_transpose_backward(merged, again, B, H, T, d)
    assert torch.equal(again, q)


@pytest.mark.parametrize("T", [1, 7, 8, 63, 64, 65, 127, 128, 129, 257])
@pytest.mark.parametrize("d", [32, 64, 128])
def test_attention_core_edge_lengths(ops, T, d):
    B, H = 1, 2
    scale = 1.0 / math.sqrt(d)
    rng = np.random.default_rng(T * 1000 + d)
    q, k, v, dO = (rng.standard_normal((B, H, T, d)).astype(np.float32) for _ in range(4))
    ref = orc.attention_forward_backward(q, k, v, dO, scale)
    tq, tk, tv, tdo = dev(q), dev(k), dev(v), dev(dO)
    out, dq, dk, dv = (torch.empty_like(tq) for _ in range(4))
    m, l, ws = (torch.empty(B, H, T, device="cuda") for _ in range(3))
    ops.tiled_causal_attention_forward(tq, tk, tv, out, B, H, T, d, scale, m, l)
    ops.tiled_causal_attention_backward(tq, tk, tv, out, tdo, m, l, dq, dk, dv, ws, B, H, T, d, scale)
    for got, key in ((out, "out"), (m, "m"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert max_abs(host(got), ref[key]) <= TOL, key


def test_known_answers_of_reference_kernel_tests(ops):
    # tests/test_kernels.cu:91-120
    T = 4
    probs = torch.zeros(T, T, device="cuda")
    ops.causal_softmax_forward(torch.ones(T, T, device="cuda"), probs, 1, 1, T, 1.0)
    p = host(probs)
    assert abs(p[0, 0] - 1) < 1e-5 and abs(p[0, 1]) < 1e-5
    assert abs(p[1, 0] - 0.5) < 1e-4 and abs(p[1, 1] - 0.5) < 1e-4 and abs(p[1, 2]) < 1e-5
    # tests/test_kernels.cu:210-284
    B = H = 1
    T, d = 8, 32
    scale = 1.0 / math.sqrt(d)
    q = torch.full((B, H, T, d), 0.1, device="cuda")
    k = q.clone()
    v = torch.ones_like(q)
    dO = torch.full_like(q, 0.5)
    out, dq, dk, dv = (torch.zeros_like(q) for _ in range(4))
    m, l, ws = (torch.empty(B, H, T, device="cuda") for _ in range(3))
    ops.tiled_causal_attention_forward(q, k, v, out, B, H, T, d, scale, m, l)
    assert torch.all((out - 1.0).abs() < 1e-3)
    ops.tiled_causal_attention_backward(q, k, v, out, dO, m, l, dq, dk, dv, ws, B, H, T, d, scale)
    for t in (dq, dk, dv):
        assert torch.isfinite(t).all()


@pytest.mark.parametrize("T", [4, 33, 200, 1030])
def test_causal_softmax_vs_oracle(ops, T):
    B, H, scale = 2, 2, 0.3
    rng = np.random.default_rng(T)
    s = rng.standard_normal((B * H * T, T)).astype(np.float32) * 3
    dp = rng.standard_normal((B * H * T, T)).astype(np.float32)
    probs = torch.full((B * H * T, T), -7.0, device="cuda")  # poisoned: zeros above the diagonal must be written
    ops.causal_softmax_forward(dev(s), probs, B, H, T, scale)
    ref = orc.causal_softmax_forward(s, B, H, T, scale)
    assert max_abs(host(probs), ref) <= TOL
    iu = np.triu_indices(T, 1)
    assert np.all(host(probs).reshape(B * H, T, T)[:, iu[0], iu[1]] == 0)
    ds = torch.full((B * H * T, T), -7.0, device="cuda")
    ops.causal_softmax_backward(dev(dp), probs, ds, B, H, T, scale)
    assert max_abs(host(ds), orc.causal_softmax_backward(dp, host(probs), B, H, T, scale)) <= TOL
    assert np.all(host(ds).reshape(B * H, T, T)[:, iu[0], iu[1]] == 0)


def test_non_tiled_branch_composes_to_the_tiled_one(ops):
    """model.cu:314-332 / :618-650: scores GEMM -> causal_softmax -> PV GEMM equals the tiled launcher."""
    B, H, T, d = 1, 3, 96, 32
    scale = 1.0 / math.sqrt(d)
    torch.backends.cuda.matmul.allow_tf32 = False
    q, k, v = (torch.randn(B, H, T, d, device="cuda") for _ in range(3))
    scores = (q @ k.transpose(-1, -2)).reshape(B * H * T, T).contiguous()
    probs = torch.empty_like(scores)
    ops.causal_softmax_forward(scores, probs, B, H, T, scale)
    composed = probs.view(B, H, T, T) @ v
    out = torch.empty_like(q)
    ops.tiled_causal_attention_forward(q, k, v, out, B, H, T, d, scale)
    assert (composed - out).abs().max().item() <= TOL


@pytest.mark.parametrize("name", [n for n in golden_names() if n.startswith(("config1", "paritygate"))])
def test_block_forward_backward_vs_golden(pkg, ops, name):
    """Config 1: LayerNorm(gamma=1,beta=0) -> QKV projection -> engine -> output projection; y, dx, dW."""
    g = load_golden(name)
    B, T, C, H = (int(x) for x in g["shape"])
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    attn = pkg.mha.CausalSelfAttention(d_model=C, num_heads=H, max_seq_len=T, math="fp32").cuda()
    ln = torch.nn.LayerNorm(C, eps=1e-5).cuda()
    with torch.no_grad():
        attn.qkv_proj.weight.copy_(dev(g["w_qkv"]).t())
        attn.qkv_proj.bias.copy_(dev(g["b_qkv"]))
        attn.out_proj.weight.copy_(dev(g["w_proj"]).t())
        attn.out_proj.bias.copy_(dev(g["b_proj"]))
    x = dev(g["x"]).requires_grad_(True)
    y = attn(ln(x))
    y.backward(dev(g["dY"]))
    assert max_abs(host(y.detach()), g["y"]) <= TOL
    assert max_abs(host(x.grad), g["dx"]) <= TOL
    assert max_abs(host(attn.qkv_proj.weight.grad.t()), g["dw_qkv"]) <= TOL
    assert max_abs(host(attn.out_proj.weight.grad.t()), g["dw_proj"]) <= TOL
    assert max_abs(host(attn.qkv_proj.bias.grad), g["db_qkv"]) <= TOL
    assert max_abs(host(attn.out_proj.bias.grad), g["db_proj"]) <= TOL


def test_forward_is_bitwise_repeatable(ops):
    B, H, T, d = 2, 2, 300, 64
    q, k, v = (torch.randn(B, H, T, d, device="cuda") for _ in range(3))
    a, b = torch.empty_like(q), torch.empty_like(q)
    ops.tiled_causal_attention_forward(q, k, v, a, B, H, T, d, 0.125)
    ops.tiled_causal_attention_forward(q, k, v, b, B, H, T, d, 0.125)
    assert torch.equal(a, b)
