"""The attention launch API on torch CUDA tensors.

The first nine functions carry the names, argument order and meaning of the launchers declared in
the reference's include/kernels/attention.cuh (lines 6-105), so a test written against that header
reads the same here; tensors replace raw pointers and the current torch stream replaces the
`cudaStream_t` argument. The remaining functions expose the BF16 tensor-core entry points.
PyTorch only provides device memory and the stream: all arithmetic happens in libb200attn.so.
Errors are raised as `lib.B200AttnError`; nothing falls back to PyTorch or the CPU.
"""
import ctypes

import torch

from . import lib as _lib


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t, dtype, name):
    if t is None:
        return None
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise _lib.B200AttnError(_lib.ERR_INVALID_ARGUMENT, f"{name}: expected a CUDA tensor")
    if t.dtype != dtype:
        raise _lib.B200AttnError(_lib.ERR_INVALID_ARGUMENT, f"{name}: expected dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise _lib.B200AttnError(_lib.ERR_INVALID_ARGUMENT, f"{name}: tensor must be contiguous")
    return ctypes.c_void_p(t.data_ptr())


def _need(t, numel, name):
    if t.numel() < numel:
        raise _lib.B200AttnError(_lib.ERR_INVALID_ARGUMENT, f"{name}: needs {numel} elements, has {t.numel()}")


F32, BF16 = torch.float32, torch.bfloat16


# ------------------------------------------------------------------ the nine reference launchers
def qkv_split_transpose_forward(qkv, q, k, v, B, T, H, d_head):
    """attention.cuh:6 - (B,T,3*H*d) -> q,k,v (B,H,T,d)."""
    n = B * T * H * d_head
    _need(qkv, 3 * n, "qkv"); _need(q, n, "q"); _need(k, n, "k"); _need(v, n, "v")
    _lib.call("b200attn_qkv_split_f32", _ptr(qkv, F32, "qkv"), _ptr(q, F32, "q"), _ptr(k, F32, "k"), _ptr(v, F32, "v"),
              B, T, H, d_head, _stream())


def qkv_split_transpose_backward(dq, dk, dv, dqkv, B, T, H, d_head):
    """attention.cuh:14 - dq,dk,dv (B,H,T,d) -> dqkv (B,T,3*H*d)."""
    n = B * T * H * d_head
    _need(dqkv, 3 * n, "dqkv"); _need(dq, n, "dq"); _need(dk, n, "dk"); _need(dv, n, "dv")
    _lib.call("b200attn_qkv_merge_grad_f32", _ptr(dq, F32, "dq"), _ptr(dk, F32, "dk"), _ptr(dv, F32, "dv"),
              _ptr(dqkv, F32, "dqkv"), B, T, H, d_head, _stream())


def causal_softmax_forward(scores, probs, B, H, T, scale):
    """attention.cuh:25 - probs = causal softmax(scale * scores), rows (B*H*T, T)."""
    _need(scores, B * H * T * T, "scores"); _need(probs, B * H * T * T, "probs")
    _lib.call("b200attn_causal_softmax_fwd_f32", _ptr(scores, F32, "scores"), _ptr(probs, F32, "probs"), B, H, T,
              float(scale), _stream())


def tiled_causal_attention_forward(q, k, v, out, B, H, T, d_head, scale, m_out=None, l_out=None):
    """attention.cuh:39 - out = softmax(scale*q k^T + causal) v, optional statistics m, l (B,H,T)."""
    n = B * H * T * d_head
    for t, nm in ((q, "q"), (k, "k"), (v, "v"), (out, "out")):
        _need(t, n, nm)
    for t, nm in ((m_out, "m_out"), (l_out, "l_out")):
        if t is not None:
            _need(t, B * H * T, nm)
    _lib.call("b200attn_fwd_f32", _ptr(q, F32, "q"), _ptr(k, F32, "k"), _ptr(v, F32, "v"), _ptr(out, F32, "out"),
              B, H, T, d_head, float(scale), _ptr(m_out, F32, "m_out"), _ptr(l_out, F32, "l_out"), _stream())


def attention_precompute_dot_do_o(dO, O, D, B, H, T, d_head):
    """attention.cuh:52 - D[row] = sum_e dO*O."""
    _need(dO, B * H * T * d_head, "dO"); _need(O, B * H * T * d_head, "O"); _need(D, B * H * T, "D")
    _lib.call("b200attn_dot_do_o_f32", _ptr(dO, F32, "dO"), _ptr(O, F32, "O"), _ptr(D, F32, "D"), B, H, T, d_head,
              _stream())


def tiled_causal_attention_backward(q, k, v, o, do_ptr, m_ptr, l_ptr, dq, dk, dv, d_workspace, B, H, T, d_head, scale):
    """attention.cuh:63 - dq,dk,dv (overwritten) from q,k,v,o,dO and the saved m,l; d_workspace: B*H*T floats."""
    n = B * H * T * d_head
    for t, nm in ((q, "q"), (k, "k"), (v, "v"), (o, "o"), (do_ptr, "do_ptr"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        _need(t, n, nm)
    for t, nm in ((m_ptr, "m_ptr"), (l_ptr, "l_ptr"), (d_workspace, "d_workspace")):
        _need(t, B * H * T, nm)
    _lib.call("b200attn_bwd_f32", _ptr(q, F32, "q"), _ptr(k, F32, "k"), _ptr(v, F32, "v"), _ptr(o, F32, "o"),
              _ptr(do_ptr, F32, "do_ptr"), _ptr(m_ptr, F32, "m_ptr"), _ptr(l_ptr, F32, "l_ptr"), _ptr(dq, F32, "dq"),
              _ptr(dk, F32, "dk"), _ptr(dv, F32, "dv"), _ptr(d_workspace, F32, "d_workspace"), B, H, T, d_head,
              float(scale), _stream())


def causal_softmax_backward(dprobs, probs, dscores, B, H, T, scale):
    """attention.cuh:82 - dscores = scale * p * (dp - sum(dp*p)), zeros above the diagonal."""
    for t, nm in ((dprobs, "dprobs"), (probs, "probs"), (dscores, "dscores")):
        _need(t, B * H * T * T, nm)
    _lib.call("b200attn_causal_softmax_bwd_f32", _ptr(dprobs, F32, "dprobs"), _ptr(probs, F32, "probs"),
              _ptr(dscores, F32, "dscores"), B, H, T, float(scale), _stream())


def head_merge_transpose_forward(inp, out, B, H, T, d_head):
    """attention.cuh:92 - (B,H,T,d) -> (B,T,H*d)."""
    _need(inp, B * H * T * d_head, "in"); _need(out, B * H * T * d_head, "out")
    _lib.call("b200attn_merge_heads_f32", _ptr(inp, F32, "in"), _ptr(out, F32, "out"), B, H, T, d_head, _stream())


def head_merge_transpose_backward(dout, din, B, H, T, d_head):
    """attention.cuh:100 - (B,T,H*d) -> (B,H,T,d)."""
    _need(dout, B * H * T * d_head, "dout"); _need(din, B * H * T * d_head, "din")
    _lib.call("b200attn_split_heads_f32", _ptr(dout, F32, "dout"), _ptr(din, F32, "din"), B, H, T, d_head, _stream())


# ------------------------------------------------------------------ BF16 tensor-core entry points
def _slab_dims(q, others, stats):
    """(BH, T, d) of q (..., T, d); every tensor of `others` must hold BH*T*d elements and every one of
    `stats` BH*T, so that no tile store or reduction of the kernels can run past a caller's buffer."""
    if q.dim() < 2:
        raise _lib.B200AttnError(_lib.ERR_INVALID_ARGUMENT, "q: expected (..., T, d)")
    T, d = q.shape[-2], q.shape[-1]
    BH = q.numel() // (T * d) if T * d else 0
    for t, nm in others:
        if t.numel() != q.numel():
            raise _lib.B200AttnError(_lib.ERR_INVALID_ARGUMENT, f"{nm}: has {t.numel()} elements, q has {q.numel()}")
    for t, nm in stats:
        _need(t, BH * T, nm)
    return BH, T, d


def _packed_dims(qkv, H):
    """(B, T, d) of qkv (B, T, 3*H*d); a width that 3*H does not divide is an error, not a truncation."""
    if qkv.dim() != 3 or H <= 0 or qkv.shape[2] % (3 * H) != 0:
        raise _lib.B200AttnError(_lib.ERR_INVALID_ARGUMENT, f"qkv: expected (B, T, 3*H*d) with H={H}, got {tuple(qkv.shape)}")
    return qkv.shape[0], qkv.shape[1], qkv.shape[2] // (3 * H)


def _exact(t, numel, name):
    if t.numel() != numel:
        raise _lib.B200AttnError(_lib.ERR_INVALID_ARGUMENT, f"{name}: has {t.numel()} elements, needs {numel}")


def attention_forward_bf16(q, k, v, scale, out=None, lse=None):
    """q,k,v: BF16 (..., T, d) with any leading (batch, head) dims; returns (out BF16, lse FP32 (..., T))."""
    if out is None:
        out = torch.empty_like(q)
    if lse is None:
        lse = torch.empty(q.shape[:-1], dtype=F32, device=q.device)
    BH, T, d = _slab_dims(q, ((k, "k"), (v, "v"), (out, "out")), ((lse, "lse"),))
    _lib.call("b200attn_fwd_bf16", _ptr(q, BF16, "q"), _ptr(k, BF16, "k"), _ptr(v, BF16, "v"), _ptr(out, BF16, "out"),
              _ptr(lse, F32, "lse"), BH, T, d, float(scale), _stream())
    return out, lse


def attention_backward_bf16(q, k, v, o, dO, lse, scale, dq=None, dk=None, dv=None):
    """BF16 backward; returns (dq, dk, dv) BF16, overwritten."""
    dq = torch.empty_like(q) if dq is None else dq
    dk = torch.empty_like(k) if dk is None else dk
    dv = torch.empty_like(v) if dv is None else dv
    BH, T, d = _slab_dims(q, ((k, "k"), (v, "v"), (o, "o"), (dO, "dO"), (dq, "dq"), (dk, "dk"), (dv, "dv")), ((lse, "lse"),))
    _lib.call("b200attn_bwd_bf16", _ptr(q, BF16, "q"), _ptr(k, BF16, "k"), _ptr(v, BF16, "v"), _ptr(o, BF16, "o"),
              _ptr(dO, BF16, "dO"), _ptr(lse, F32, "lse"), _ptr(dq, BF16, "dq"), _ptr(dk, BF16, "dk"),
              _ptr(dv, BF16, "dv"), BH, T, d, float(scale), _stream())
    return dq, dk, dv


def attention_backward_bf16_noalloc(q, k, v, o, dO, lse, scale, dq, dk, dv):
    """The BF16 backward through the entry point that takes its scratch from the library's static
    device array instead of allocating (see include/b200attn.h for who needs it and its size limit).
    Output tensors are passed in, so this wrapper allocates nothing either."""
    BH, T, d = _slab_dims(q, ((k, "k"), (v, "v"), (o, "o"), (dO, "dO"), (dq, "dq"), (dk, "dk"), (dv, "dv")), ((lse, "lse"),))
    _lib.call("b200attn_bwd_bf16_noalloc", _ptr(q, BF16, "q"), _ptr(k, BF16, "k"), _ptr(v, BF16, "v"),
              _ptr(o, BF16, "o"), _ptr(dO, BF16, "dO"), _ptr(lse, F32, "lse"), _ptr(dq, BF16, "dq"),
              _ptr(dk, BF16, "dk"), _ptr(dv, BF16, "dv"), BH, T, d, float(scale), _stream())
    return dq, dk, dv


def attention_forward_bf16_packed(qkv, H, scale, out=None, lse=None):
    """Attention straight on the projection output: qkv BF16 (B, T, 3*H*d) with inner order
    [Q heads | K heads | V heads]; returns (out BF16 (B, T, H*d), lse FP32 (B, H, T)). No split or merge pass."""
    B, T, d = _packed_dims(qkv, H)
    out = torch.empty(B, T, H * d, device=qkv.device, dtype=BF16) if out is None else out
    lse = torch.empty(B, H, T, device=qkv.device, dtype=F32) if lse is None else lse
    _exact(out, B * T * H * d, "out"); _need(lse, B * H * T, "lse")
    _lib.call("b200attn_fwd_bf16_packed", _ptr(qkv, BF16, "qkv"), _ptr(out, BF16, "out"), _ptr(lse, F32, "lse"),
              B, T, H, d, float(scale), _stream())
    return out, lse


def attention_backward_bf16_packed(qkv, out, dout, lse, H, scale, dqkv=None):
    """Backward of attention_forward_bf16_packed: dout BF16 (B, T, H*d) -> dqkv BF16 (B, T, 3*H*d), overwritten."""
    B, T, d = _packed_dims(qkv, H)
    dqkv = torch.empty_like(qkv) if dqkv is None else dqkv
    _exact(out, B * T * H * d, "out"); _exact(dout, B * T * H * d, "dout"); _exact(dqkv, qkv.numel(), "dqkv")
    _need(lse, B * H * T, "lse")
    _lib.call("b200attn_bwd_bf16_packed", _ptr(qkv, BF16, "qkv"), _ptr(out, BF16, "out"), _ptr(dout, BF16, "dout"),
              _ptr(lse, F32, "lse"), _ptr(dqkv, BF16, "dqkv"), B, T, H, d, float(scale), _stream())
    return dqkv


def qkv_split_transpose_forward_bf16(qkv, q, k, v, B, T, H, d_head):
    """FP32 (B,T,3*H*d) -> BF16 q,k,v (B,H,T,d)."""
    _lib.call("b200attn_qkv_split_bf16", _ptr(qkv, F32, "qkv"), _ptr(q, BF16, "q"), _ptr(k, BF16, "k"),
              _ptr(v, BF16, "v"), B, T, H, d_head, _stream())


def qkv_split_transpose_backward_bf16(dq, dk, dv, dqkv, B, T, H, d_head):
    """BF16 dq,dk,dv (B,H,T,d) -> FP32 dqkv (B,T,3*H*d)."""
    _lib.call("b200attn_qkv_merge_grad_bf16", _ptr(dq, BF16, "dq"), _ptr(dk, BF16, "dk"), _ptr(dv, BF16, "dv"),
              _ptr(dqkv, F32, "dqkv"), B, T, H, d_head, _stream())


def head_merge_transpose_forward_bf16(inp, out, B, H, T, d_head):
    """BF16 (B,H,T,d) -> FP32 (B,T,H*d)."""
    _lib.call("b200attn_merge_heads_bf16", _ptr(inp, BF16, "in"), _ptr(out, F32, "out"), B, H, T, d_head, _stream())


def head_merge_transpose_backward_bf16(dout, din, B, H, T, d_head):
    """FP32 (B,T,H*d) -> BF16 (B,H,T,d)."""
    _lib.call("b200attn_split_heads_bf16", _ptr(dout, F32, "dout"), _ptr(din, BF16, "din"), B, H, T, d_head, _stream())


# ------------------------------------------------------------------ library state and synthetic inputs
def set_math_mode(mode):
    """'fp32' (SIMT, exact; default) or 'bf16' (tensor cores) for the float32 attention launchers."""
    code = {"fp32": _lib.MATH_FP32, "bf16": _lib.MATH_BF16}.get(mode, mode)
    _lib.call("b200attn_set_math_mode", int(code))


def get_math_mode():
    return "bf16" if _lib.load().b200attn_get_math_mode() == _lib.MATH_BF16 else "fp32"


def set_fused_convert(on):
    """BF16 copies of q, k, v / dO written by the FP32 layout launchers and reused by the FP32 attention launchers in
    BF16 math mode (see include/b200attn.h)."""
    _lib.call("b200attn_set_fused_convert", 1 if on else 0)


def fused_convert_hits():
    return int(_lib.load().b200attn_fused_convert_hits())


def reserve(BH, T, d):
    _lib.call("b200attn_reserve", int(BH), int(T), int(d))


def release():
    """Free the library-owned scratch of the current device (synchronises it)."""
    _lib.call("b200attn_release")


def check_device_fault():
    """Synchronise and raise if a kernel's bounded wait ran out."""
    code = ctypes.c_uint(0)
    _lib.check(_lib.load().b200attn_check_device_fault(ctypes.byref(code)))


def fill_normal_(t, seed, offset=0):
    """Fill a contiguous FP32 or BF16 CUDA tensor with N(0,1) samples offset..offset+numel of stream `seed`."""
    if t.dtype == F32:
        _lib.call("b200attn_fill_normal_f32", _ptr(t, F32, "dst"), t.numel(), int(seed), int(offset), _stream())
    else:
        _lib.call("b200attn_fill_normal_bf16", _ptr(t, BF16, "dst"), t.numel(), int(seed), int(offset), _stream())
    return t


def kernel_timing(enable, every=1):
    """Start (True) or stop (False) event timing of the tensor-core kernels, on every `every`-th launch of
    each kernel; clears records."""
    _lib.call("b200attn_kernel_timing", int(every) if enable else 0)


def kernel_times():
    """Summed durations and launch counts recorded since kernel_timing(True):
    dict(fwd_ms, fwd_launches, bwd_ms, bwd_launches)."""
    f, b = ctypes.c_double(0), ctypes.c_double(0)
    nf, nb = ctypes.c_int(0), ctypes.c_int(0)
    _lib.call("b200attn_kernel_times", ctypes.byref(f), ctypes.byref(nf), ctypes.byref(b), ctypes.byref(nb))
    return dict(fwd_ms=f.value, fwd_launches=nf.value, bwd_ms=b.value, bwd_launches=nb.value)


def kernel_time_samples(backward):
    """The single launch durations (ms, launch order) of the forward (False) or backward (True) kernel recorded since
    kernel_timing(True)."""
    n = ctypes.c_int(0)
    _lib.call("b200attn_kernel_time_samples", int(bool(backward)), None, 0, ctypes.byref(n))
    if n.value == 0:
        return []
    buf = (ctypes.c_float * n.value)()
    _lib.call("b200attn_kernel_time_samples", int(bool(backward)), buf, n.value, ctypes.byref(n))
    return list(buf)
