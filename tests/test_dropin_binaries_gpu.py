"""The reference's own executables, compiled from its unmodified sources against this engine
(oracle/Makefile -> oracle/_ref/), run on the GPU:

  * tests/test_kernels.cu of the reference (its assert-based kernel tests) must pass as they are;
  * src/parity_audit.cu + src/model.cu of the reference, fed the golden files its own PyTorch
    generator wrote (tests/golden/parity_audit*/), must meet the gates of scripts/compare_parity.py:108-117:
    logits and loss max-abs <= 1e-5, gradients <= 5e-5 - with the tiled launchers (--tiled_attn) and with
    the materialised-softmax branch, whose split/softmax/merge launchers also come from this engine.

The binaries are prebuilt where the reference checkout exists; where they are absent the tests skip."""
import os
import shutil
import subprocess

import numpy as np
import pytest

from conftest import GOLDEN_DIR, ROOT

pytestmark = pytest.mark.gpu
REF_BIN = os.path.join(ROOT, "oracle", "_ref")


def _binary(name):
    path = os.path.join(REF_BIN, name)
    if not os.path.exists(path):
        pytest.skip(f"{path} not built (needs the reference checkout: make -C oracle REFERENCE=...)")
    return path


def test_reference_kernel_test_suite_passes_unchanged():
    res = subprocess.run([_binary("test_kernels")], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "All isolated kernel tests passed" in res.stdout
    assert "[b200attn]" not in res.stderr  # no launcher reported a failure


def _max_abs(a, b):
    return float(np.abs(a.astype(np.float64) - b.astype(np.float64)).max())


@pytest.mark.parametrize("case", ["parity_audit", "parity_audit_d64"])
@pytest.mark.parametrize("tiled", [True, False])
def test_reference_model_meets_its_parity_gate(tmp_path, case, tiled):
    exe = _binary("parity_audit")
    work = tmp_path / case
    shutil.copytree(os.path.join(GOLDEN_DIR, case), work)
    cmd = [exe, str(work)] + (["--tiled_attn"] if tiled else [])
    env = dict(os.environ, B200ATTN_MATH="fp32")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "[b200attn]" not in res.stderr
    load = lambda n: np.fromfile(os.path.join(work, n), dtype=np.float32)
    assert _max_abs(load("cuda_logits.bin"), load("pytorch_logits.bin")) <= 1e-5
    assert _max_abs(load("cuda_loss.bin"), load("pytorch_loss.bin")) <= 1e-5
    assert _max_abs(load("cuda_grads.bin"), load("pytorch_grads.bin")) <= 5e-5


@pytest.mark.parametrize("fused", ["0", "1"])
def test_reference_model_through_the_tensor_cores(tmp_path, fused):
    """Same model binary, d_head = 64, attention routed to the tcgen05 kernels by B200ATTN_MATH=bf16 - with one
    conversion pass per operand, and with the BF16 copies written by the layout launchers (B200ATTN_FUSED_CONVERT=1).
    BF16 operands cannot meet the FP32 gate; the whole-model error stays within the BF16 gates."""
    exe = _binary("parity_audit")
    work = tmp_path / "bf16"
    shutil.copytree(os.path.join(GOLDEN_DIR, "parity_audit_d64"), work)
    env = dict(os.environ, B200ATTN_MATH="bf16", B200ATTN_FUSED_CONVERT=fused)
    res = subprocess.run([exe, str(work), "--tiled_attn"], capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "[b200attn]" not in res.stderr
    load = lambda n: np.fromfile(os.path.join(work, n), dtype=np.float32)
    ref, got = load("pytorch_grads.bin"), load("cuda_grads.bin")
    assert _max_abs(load("cuda_logits.bin"), load("pytorch_logits.bin")) <= 2e-2
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) <= 5e-3
    assert _max_abs(got, ref) <= 2e-2


@pytest.mark.parametrize("case", ["parity_audit", "parity_audit_d64"])
def test_gemm_dropin_meets_the_reference_gate_in_fp32(tmp_path, case):
    """The reference model with BOTH its attention kernels and its GEMM wrappers (src/kernels/matmul.cu)
    replaced - oracle/_ref/parity_audit_gemm links transformer-cuda_b200/gemm/matmul_dropin.cu behind the
    unchanged declarations of include/kernels/matmul.cuh. In the default FP32 arithmetic the whole model
    still meets the gates of scripts/compare_parity.py:108-117."""
    exe = _binary("parity_audit_gemm")
    work = tmp_path / case
    shutil.copytree(os.path.join(GOLDEN_DIR, case), work)
    env = dict(os.environ, B200ATTN_MATH="fp32", B200GEMM_MATH="fp32")
    res = subprocess.run([exe, str(work), "--tiled_attn"], capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "[b200attn]" not in res.stderr and "b200gemm:" not in res.stderr
    load = lambda n: np.fromfile(os.path.join(work, n), dtype=np.float32)
    assert _max_abs(load("cuda_logits.bin"), load("pytorch_logits.bin")) <= 1e-5
    assert _max_abs(load("cuda_loss.bin"), load("pytorch_loss.bin")) <= 1e-5
    assert _max_abs(load("cuda_grads.bin"), load("pytorch_grads.bin")) <= 5e-5


def test_gemm_dropin_on_the_tensor_cores(tmp_path):
    """B200GEMM_MATH=bf16: every GEMM of the model rounds its operands to BF16 (FP32 accumulation, FP32
    buffers), attention on the tcgen05 kernels as well. The whole-model error stays within the BF16 gates
    used for the attention path (max-abs 2e-2 on logits, relative-L2 5e-3 and max-abs 2e-2 on gradients)."""
    exe = _binary("parity_audit_gemm")
    work = tmp_path / "bf16"
    shutil.copytree(os.path.join(GOLDEN_DIR, "parity_audit_d64"), work)
    env = dict(os.environ, B200ATTN_MATH="bf16", B200GEMM_MATH="bf16")
    res = subprocess.run([exe, str(work), "--tiled_attn"], capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "[b200attn]" not in res.stderr and "b200gemm:" not in res.stderr
    load = lambda n: np.fromfile(os.path.join(work, n), dtype=np.float32)
    ref, got = load("pytorch_grads.bin"), load("cuda_grads.bin")
    assert _max_abs(load("cuda_logits.bin"), load("pytorch_logits.bin")) <= 2e-2
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) <= 5e-3
    assert _max_abs(got, ref) <= 2e-2


@pytest.mark.parametrize("mode,tol,kernel", [("fp32", "1e-4", "library"), ("bf16", "2e-2", "library"), ("bf16", "2e-2", "tcgen05"), ("bf16", "2e-2", "auto")])
def test_gemm_wrappers_against_host_fp64(mode, tol, kernel):
    """oracle/_ref/gemm_check: every wrapper of include/kernels/matmul.cuh on seeded inputs against an FP64 host
    computation, including the language-model-head shapes (V = 50257: leading dimensions that are not a
    multiple of 16 bytes), which in BF16 arithmetic take the staged path (padded BF16 operands, padded FP32
    result copied into place), or - B200GEMM_KERNEL=tcgen05 - the hand-written tcgen05 kernel of gemm/gemm_tc.cu, which
    writes the unaligned result in place; large products in all four operand layouts, ragged sizes included."""
    res = subprocess.run([_binary("gemm_check"), tol], capture_output=True, text=True, timeout=900,
                         env=dict(os.environ, B200GEMM_MATH=mode, B200GEMM_KERNEL=kernel))
    assert res.returncode == 0, res.stdout + res.stderr
    assert "b200gemm:" not in res.stderr
    assert res.stdout.count('"ok": true') == 15 and '"ok": false' not in res.stdout, res.stdout
    import json
    tail = json.loads(res.stdout.strip().splitlines()[-1])
    assert tail["device_fault"] == 0
    # seven of the cases are large enough for the hand-written kernel; "library" never runs it
    assert tail["tcgen05_kernel_launches"] == {"tcgen05": 7, "auto": 3, "library": 0}[kernel], tail


def test_staged_operand_reuse_between_the_backward_pair():
    """B200GEMM_REUSE_STAGED=1: dW = X^T dY followed by dX = dY W^T converts dY once; dX still agrees with the FP64 host
    result (the last case of gemm_check), and without the switch nothing is reused."""
    import json
    for flag, want in (("1", 1), ("0", 0)):
        res = subprocess.run([_binary("gemm_check"), "2e-2"], capture_output=True, text=True, timeout=900,
                             env=dict(os.environ, B200GEMM_MATH="bf16", B200GEMM_REUSE_STAGED=flag))
        assert res.returncode == 0, res.stdout + res.stderr
        pair = [json.loads(l) for l in res.stdout.splitlines() if "backward_pair_dx" in l][0]
        assert pair["ok"] and pair["staged_reuses"] == want, pair


def test_weights_inside_a_flat_buffer_are_read_from_its_bf16_twin():
    """B200GEMM_TWINS=1: a matrix that starts inside a registered flat buffer (b200gemm_bf16_twin_range - what the AdamW
    drop-in keeps of the parameters) at a multiple of 128 elements is read from the twin - gemm_check fills the twin with
    twice the FP32 values, so the product doubles - and one at any other offset is converted as usual; without the switch
    no twin is handed out."""
    import json
    for flag, want in (("1", "on"), ("0", "off")):
        res = subprocess.run([_binary("gemm_check"), "2e-2"], capture_output=True, text=True, timeout=900,
                             env=dict(os.environ, B200GEMM_MATH="bf16", B200GEMM_TWINS=flag))
        assert res.returncode == 0, res.stdout + res.stderr
        line = [json.loads(l) for l in res.stdout.splitlines() if "range_twin" in l][0]
        assert line["ok"] and line["twins"] == want, line


@pytest.mark.parametrize("case", ["parity_audit", "parity_audit_d64"])
def test_loss_dropin_meets_the_reference_gate_in_fp32(tmp_path, case):
    """oracle/_ref/parity_audit_all: the reference model with its attention kernels, its GEMM wrappers, its loss
    launcher (src/kernels/loss.cu), its LayerNorm launchers (src/kernels/layernorm.cu) AND its GELU launchers
    (src/kernels/ffn.cu) replaced - libb200loss, libb200norm and libb200ffn behind the unchanged declarations of
    include/kernels/loss.cuh, layernorm.cuh and ffn.cuh. Loss, logits and
    every gradient (all of which flow from d_logits, through five LayerNorms) still meet the gates of
    scripts/compare_parity.py:108-117."""
    exe = _binary("parity_audit_all")
    work = tmp_path / case
    shutil.copytree(os.path.join(GOLDEN_DIR, case), work)
    env = dict(os.environ, B200ATTN_MATH="fp32", B200GEMM_MATH="fp32")
    res = subprocess.run([exe, str(work), "--tiled_attn"], capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stdout + res.stderr
    for tag in ("[b200attn]", "b200gemm:", "[b200loss]", "[b200norm]", "[b200ffn]"):
        assert tag not in res.stderr
    load = lambda n: np.fromfile(os.path.join(work, n), dtype=np.float32)
    assert _max_abs(load("cuda_logits.bin"), load("pytorch_logits.bin")) <= 1e-5
    assert _max_abs(load("cuda_loss.bin"), load("pytorch_loss.bin")) <= 1e-5
    assert _max_abs(load("cuda_grads.bin"), load("pytorch_grads.bin")) <= 5e-5


def test_adamw_dropin_against_host_restatement():
    """oracle/_ref/optimizer_check: transformer-cuda_b200/optim/adamw_dropin.cu (class AdamW of the reference's
    include/optimizer.h) over five steps - fused_step with and without the clip taking effect, then the
    clip_grad_norm + step + zero_grad form - against a double-precision restatement of src/optimizer.cu on a
    parameter count that is not a multiple of four: parameters within 2e-6, gradients left exactly zero."""
    import json
    res = subprocess.run([_binary("optimizer_check")], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "[b200opt]" not in res.stderr
    rep = json.loads(res.stdout.strip().splitlines()[-1])
    assert rep["ok"] and rep["max_abs_param_error"] <= 2e-6 and rep["max_abs_leftover_grad"] == 0.0


def test_reference_kernel_test_suite_with_the_layernorm_dropin():
    """tests/test_kernels.cu of the reference, unchanged, with src/kernels/layernorm.cu replaced by libb200norm and
    src/kernels/ffn.cu by libb200ffn as well as attention.cu by libb200attn: its LayerNorm test (:13-89), its GELU test
    and every other test pass."""
    res = subprocess.run([_binary("test_kernels_all")], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "All isolated kernel tests passed" in res.stdout
    assert "[b200norm]" not in res.stderr and "[b200attn]" not in res.stderr


def test_layernorm_dropin_against_host_restatement():
    """oracle/_ref/layernorm_check: both launchers of include/kernels/layernorm.cuh against a double-precision
    restatement of src/kernels/layernorm.cu - register path (C = 128 k) and generic path, with and without gamma /
    beta, residual_add and accumulate, dgamma / dbeta added to non-zero buffers."""
    import json
    res = subprocess.run([_binary("layernorm_check")], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "[b200norm]" not in res.stderr
    cases = [json.loads(l) for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(cases) == 7 and all(c["ok"] for c in cases), res.stdout
