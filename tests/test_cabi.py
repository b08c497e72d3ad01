"""CPU-side checks of the drop-in boundary: the shared library loads, exports every symbol that
include/b200attn.h declares, keeps the nine launcher signatures of the reference header, and rejects
bad arguments before touching the GPU. No compute call is made here."""
import ctypes
import os
import re
import subprocess

import pytest

from conftest import ROOT


@pytest.fixture(scope="module")
def lib(pkg):
    import __graft_entry__ as entry
    if not os.path.exists(pkg.lib.SO_PATH):
        entry.build()
    return pkg.lib


def test_every_declared_symbol_is_exported(lib):
    so = lib.load()
    names = lib.declared_symbols()
    assert len(names) >= 24
    for n in names:
        assert hasattr(so, n), n
    # and the binding covers exactly the header
    assert sorted(lib._SIGNATURES) == names


def test_cpp_launchers_are_exported(lib):
    """The nine C++ launchers of include/kernels/attention.cuh must be present (mangled) in the library."""
    out = subprocess.run(["nm", "-D", "--defined-only", "-C", lib.SO_PATH], capture_output=True, text=True, check=True).stdout
    for name in ("qkv_split_transpose_forward", "qkv_split_transpose_backward", "causal_softmax_forward",
                 "tiled_causal_attention_forward", "attention_precompute_dot_do_o", "tiled_causal_attention_backward",
                 "causal_softmax_backward", "head_merge_transpose_forward", "head_merge_transpose_backward"):
        assert re.search(rf"\b{name}\(", out), name


def test_header_keeps_reference_signatures():
    """Parameter lists as in the reference's include/kernels/attention.cuh:6-105 (types and defaults)."""
    with open(os.path.join(ROOT, "include", "kernels", "attention.cuh")) as f:
        text = re.sub(r"\s+", " ", f.read())
    expect = [
        "void qkv_split_transpose_forward(const float* qkv, float* q, float* k, float* v, int B, int T, int H, int d_head, cudaStream_t stream = 0);",
        "void qkv_split_transpose_backward(const float* dq, const float* dk, const float* dv, float* dqkv, int B, int T, int H, int d_head, cudaStream_t stream = 0);",
        "void causal_softmax_forward(const float* scores, float* probs, int B, int H, int T, float scale, cudaStream_t stream = 0);",
        "void tiled_causal_attention_forward(const float* q, const float* k, const float* v, float* out, int B, int H, int T, int d_head, float scale, float* m_out = nullptr, float* l_out = nullptr, cudaStream_t stream = 0);",
        "void attention_precompute_dot_do_o(const float* dO, const float* O, float* D, int B, int H, int T, int d_head, cudaStream_t stream = 0);",
        "void tiled_causal_attention_backward(const float* q, const float* k, const float* v, const float* o, const float* do_ptr, const float* m_ptr, const float* l_ptr, float* dq, float* dk, float* dv, float* d_workspace, int B, int H, int T, int d_head, float scale, cudaStream_t stream = 0);",
        "void causal_softmax_backward(const float* dprobs, const float* probs, float* dscores, int B, int H, int T, float scale, cudaStream_t stream = 0);",
        "void head_merge_transpose_forward(const float* in, float* out, int B, int H, int T, int d_head, cudaStream_t stream = 0);",
        "void head_merge_transpose_backward(const float* dout, float* din, int B, int H, int T, int d_head, cudaStream_t stream = 0);",
    ]
    for sig in expect:
        assert sig in text, sig


def test_argument_errors_need_no_gpu(lib):
    so = lib.load()
    assert so.b200attn_version() >= 100
    assert so.b200attn_set_math_mode(7) == lib.ERR_INVALID_ARGUMENT
    assert b"unknown mode" in so.b200attn_last_error()
    assert so.b200attn_set_math_mode(lib.MATH_FP32) == lib.OK
    # null pointers and negative sizes are rejected before any CUDA call
    rc = so.b200attn_fwd_f32(None, None, None, None, 1, 1, 8, 32, 1.0, None, None, None)
    assert rc == lib.ERR_INVALID_ARGUMENT and b"NULL" in so.b200attn_last_error()
    rc = so.b200attn_qkv_split_f32(None, None, None, None, -1, 1, 1, 32, None)
    assert rc == lib.ERR_INVALID_ARGUMENT
    # empty problems are a no-op, as in the reference (grid of zero blocks)
    assert so.b200attn_fwd_f32(None, None, None, None, 0, 4, 16, 32, 1.0, None, None, None) == lib.OK
    assert so.b200attn_merge_heads_f32(None, None, 2, 2, 0, 32, None) == lib.OK
    with pytest.raises(lib.B200AttnError):
        lib.call("b200attn_fill_normal_f32", None, ctypes.c_longlong(-1), ctypes.c_ulonglong(0), ctypes.c_longlong(0), None)


def test_python_launchers_reject_cpu_tensors(pkg):
    import torch
    x = torch.zeros(1, 1, 8, 32)
    with pytest.raises(pkg.lib.B200AttnError):
        pkg.ops.tiled_causal_attention_forward(x, x, x, x, 1, 1, 8, 32, 1.0)


def test_loss_library_exports_its_header(pkg):
    """libb200loss.so: every symbol of include/b200loss.h is exported and bound, the C++ launcher with the
    reference's signature (include/kernels/loss.cuh:8-15) is present, and bad arguments fail before any CUDA call."""
    import importlib
    import __graft_entry__ as entry
    loss_ops = importlib.import_module(pkg.__name__ + ".loss_ops")
    if not os.path.exists(loss_ops.SO_PATH):
        entry.build()
    so = loss_ops.load()
    names = loss_ops.declared_symbols()
    assert sorted(loss_ops._SIGNATURES) == names
    for n in names:
        assert hasattr(so, n), n
    out = subprocess.run(["nm", "-D", "--defined-only", "-C", loss_ops.SO_PATH], capture_output=True, text=True, check=True).stdout
    assert re.search(r"\bcross_entropy_forward_backward\(float const\*, int const\*, float\*, float\*, int, int, int, CUstream_st\*\)", out)
    assert re.search(r"\bcross_entropy_forward_backward_device\(", out)
    with open(os.path.join(ROOT, "include", "kernels", "loss.cuh")) as f:
        text = re.sub(r"\s+", " ", f.read())
    assert ("void cross_entropy_forward_backward(const float* logits, const int* targets, float* dlogits, float* host_loss, "
            "int B, int T, int V, cudaStream_t stream = 0);") in text
    assert so.b200loss_cross_entropy(None, None, None, None, 1, 1, 8, None) == -1
    assert b"NULL" in so.b200loss_last_error()
    assert so.b200loss_max_resident_vocab() >= 50257


def test_caller_dropin_headers_keep_reference_signatures():
    """The headers of the callers' drop-ins declare the reference's launchers verbatim (names, parameter order, types,
    default arguments: include/kernels/layernorm.cuh:9-36, ffn.cuh:7-33, matmul.cuh:10-81 of the reference), so its
    model.cu compiles against them unchanged; and the static libraries define them."""
    def text(name):
        with open(os.path.join(ROOT, "include", "kernels", name)) as f:
            return re.sub(r"\s+", " ", f.read())
    expect = {
        "layernorm.cuh": [
            "void layernorm_forward(const float* x, const float* gamma, const float* beta, float* out, float* mean, float* rstd, int N, int C, float eps, cudaStream_t stream = 0);",
            "void layernorm_backward(const float* dout, const float* x, const float* gamma, const float* mean, const float* rstd, float* dx, float* dgamma, float* dbeta, int N, int C, const float* residual_add = nullptr, bool accumulate = false, cudaStream_t stream = 0);",
        ],
        "ffn.cuh": [
            "void gelu_forward(const float* x, float* y, int N, cudaStream_t stream = 0);",
            "void add_bias_gelu_forward(const float* x, const float* bias, float* y, int M, int N, cudaStream_t stream = 0);",
            "void gelu_backward(const float* dy, const float* x, float* dx, int N, cudaStream_t stream = 0);",
        ],
        "matmul.cuh": [
            "void matmul_forward(cublasHandle_t handle, const float* A, const float* B, float* C, int M, int N, int K, bool transA = false, bool transB = false, float alpha = 1.0f, float beta = 0.0f, cudaStream_t stream = 0);",
            "void add_bias(float* Y, const float* bias, int M, int N, cudaStream_t stream = 0);",
        ],
    }
    for header, sigs in expect.items():
        t = text(header)
        for sig in sigs:
            assert sig in t, (header, sig)
    libdir = os.path.join(ROOT, "transformer-cuda_b200", "lib")
    if not os.path.exists(os.path.join(libdir, "libb200norm.a")):
        import __graft_entry__ as entry
        entry.build()
    defined = {"libb200norm.a": ["layernorm_forward(", "layernorm_backward(", "b200norm_set_backward_hook"],
               "libb200ffn.a": ["gelu_forward(", "add_bias_gelu_forward(", "gelu_backward("],
               "libb200gemm.a": ["matmul_forward(", "matmul_cublaslt(", "bias_backward(", "b200gemm_bf16_twin", "b200gemm::tc_gemm_bf16("],
               "libb200loss.a": ["cross_entropy_forward_backward(", "b200loss_cross_entropy"]}
    for lib, names in defined.items():
        out = subprocess.run(["nm", "--defined-only", "-C", os.path.join(libdir, lib)], capture_output=True, text=True, check=True).stdout
        for n in names:
            assert n in out, (lib, n)
    # every extern "C" extension a drop-in header declares is defined by its library
    for header, lib in (("matmul.cuh", "libb200gemm.a"), ("layernorm.cuh", "libb200norm.a")):
        declared = re.findall(r'extern "C" [\w \*]*?\b(b200\w+)\(', text(header))
        assert declared, header
        out = subprocess.run(["nm", "--defined-only", os.path.join(libdir, lib)], capture_output=True, text=True, check=True).stdout
        symbols = {line.split()[-1] for line in out.splitlines() if line.strip()}
        for name in declared:
            assert name in symbols, (lib, name)
