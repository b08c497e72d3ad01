"""CPU oracle for the causal multi-head self-attention path (numpy).

TEST INFRASTRUCTURE ONLY. This module is the checker that the CUDA engine is compared
against; nothing in the product path imports it. Only tests/, the smoke check and the
CPU-baseline leg of bench.py may import it.

Every function restates, in plain numpy, what the reference computes for one step of the
path, and cites the reference file:line it follows (paths are relative to the root of
sarimahsan/transformer-cuda):

    pytorch_src/model.py:31-58         CausalSelfAttention.forward (the arithmetic truth)
    src/kernels/attention.cu           the CUDA launchers whose buffers and statistics
                                       (m, l, D, zeros above the diagonal) the drop-in keeps
    scripts/compare_parity.py:11-26    the error metrics of the parity gate

Parity of this oracle is pinned: tests/test_oracle_golden.py checks it against golden
vectors produced by importing the reference's own PyTorch module (tests/golden/make_golden.py)
and against the closed-form known-answer tests of the reference's tests/test_kernels.cu.

Arithmetic is float64 by default (so the oracle's own rounding stays far below the 1e-5 gate);
pass dtype=np.float32 to mimic the reference's precision.
"""
from __future__ import annotations

import math

import numpy as np

# 1e-12 is added to the softmax denominator by the reference's CUDA kernels
# (src/kernels/attention.cu:189, :616, :787). It is far below FP32 resolution of a
# denominator that is always >= 1, so the oracle omits it; the golden-vector tests
# confirm agreement with the PyTorch module, which has no such term.


# --------------------------------------------------------------------------- layout
def qkv_split_transpose_forward(qkv: np.ndarray, B: int, T: int, H: int, d: int):
    """(B, T, 3*H*d) -> q, k, v each (B, H, T, d).

    Inner order of the last axis is [Q heads | K heads | V heads]
    (pytorch_src/model.py:36-41 chunk + view + transpose; src/kernels/attention.cu:24-83).
    """
    x = np.asarray(qkv).reshape(B, T, 3, H, d)
    q = np.ascontiguousarray(x[:, :, 0].transpose(0, 2, 1, 3))
    k = np.ascontiguousarray(x[:, :, 1].transpose(0, 2, 1, 3))
    v = np.ascontiguousarray(x[:, :, 2].transpose(0, 2, 1, 3))
    return q, k, v


def qkv_split_transpose_backward(dq: np.ndarray, dk: np.ndarray, dv: np.ndarray):
    """Inverse scatter: three (B, H, T, d) -> (B, T, 3*H*d), every element overwritten
    (src/kernels/attention.cu:85-143)."""
    B, H, T, d = dq.shape
    out = np.empty((B, T, 3, H, d), dtype=dq.dtype)
    out[:, :, 0] = dq.transpose(0, 2, 1, 3)
    out[:, :, 1] = dk.transpose(0, 2, 1, 3)
    out[:, :, 2] = dv.transpose(0, 2, 1, 3)
    return out.reshape(B, T, 3 * H * d)


def head_merge_transpose_forward(x: np.ndarray):
    """(B, H, T, d) -> (B, T, H*d) (pytorch_src/model.py:55; src/kernels/attention.cu:308-343)."""
    B, H, T, d = x.shape
    return np.ascontiguousarray(x.transpose(0, 2, 1, 3)).reshape(B, T, H * d)


def head_merge_transpose_backward(dy: np.ndarray, H: int):
    """(B, T, H*d) -> (B, H, T, d) (src/kernels/attention.cu:345-379)."""
    B, T, C = dy.shape
    return np.ascontiguousarray(dy.reshape(B, T, H, C // H).transpose(0, 2, 1, 3))


# --------------------------------------------------------------------------- non-tiled softmax
def causal_softmax_forward(scores: np.ndarray, B: int, H: int, T: int, scale: float, dtype=np.float64):
    """scores (B*H*T, T) -> probs: softmax over j <= i of scale*scores, exact zeros for j > i
    (pytorch_src/model.py:45-51; src/kernels/attention.cu:147-238)."""
    s = np.asarray(scores, dtype=dtype).reshape(B * H, T, T) * dtype(scale)
    keep = np.tril(np.ones((T, T), dtype=bool))
    s = np.where(keep, s, -np.inf)
    m = s.max(axis=-1, keepdims=True)
    e = np.exp(s - m)
    p = e / e.sum(axis=-1, keepdims=True)
    return p.reshape(B * H * T, T)


def causal_softmax_backward(dprobs: np.ndarray, probs: np.ndarray, B: int, H: int, T: int, scale: float,
                            dtype=np.float64):
    """dscores = scale * p * (dp - sum_j dp*p) for j <= i, zeros above the diagonal
    (src/kernels/attention.cu:242-306)."""
    p = np.asarray(probs, dtype=dtype).reshape(B * H, T, T)
    dp = np.asarray(dprobs, dtype=dtype).reshape(B * H, T, T)
    keep = np.tril(np.ones((T, T), dtype=bool))
    p = np.where(keep, p, 0)
    dp = np.where(keep, dp, 0)
    dot = (p * dp).sum(axis=-1, keepdims=True)
    ds = dtype(scale) * p * (dp - dot)
    return ds.reshape(B * H * T, T)


# --------------------------------------------------------------------------- attention core
def _bh_view(x: np.ndarray, dtype):
    x = np.asarray(x, dtype=dtype)
    if x.ndim == 4:
        B, H, T, d = x.shape
        return x.reshape(B * H, T, d)
    return x


def attention_forward(q, k, v, scale: float, dtype=np.float64):
    """O = softmax(scale * Q K^T + causal mask) V per (b, h) slab
    (pytorch_src/model.py:44-52; src/kernels/attention.cu:518-624).

    Returns (out, m, l): out has q's shape; m = row maximum of the scaled, masked scores and
    l = sum_j exp(s_ij - m_i) (un-normalised), the statistics the reference's tiled kernel
    exports (src/kernels/attention.cu:619-620). log-sum-exp = m + log(l).
    """
    shape = np.asarray(q).shape
    qf, kf, vf = _bh_view(q, dtype), _bh_view(k, dtype), _bh_view(v, dtype)
    BH, T, d = qf.shape
    out = np.empty_like(qf)
    m = np.empty((BH, T), dtype=dtype)
    l = np.empty((BH, T), dtype=dtype)
    keep = np.tril(np.ones((T, T), dtype=bool))
    for i in range(BH):
        s = (qf[i] @ kf[i].T) * dtype(scale)
        s = np.where(keep, s, -np.inf)
        mi = s.max(axis=-1)
        e = np.exp(s - mi[:, None])
        li = e.sum(axis=-1)
        out[i] = (e @ vf[i]) / li[:, None]
        m[i], l[i] = mi, li
    return out.reshape(shape), m.reshape(shape[:-1]), l.reshape(shape[:-1])


def attention_precompute_dot_do_o(dO, O, dtype=np.float64):
    """D[row] = sum_e dO[row, e] * O[row, e] (src/kernels/attention.cu:659-691)."""
    return (np.asarray(dO, dtype=dtype) * np.asarray(O, dtype=dtype)).sum(axis=-1)


def attention_backward(q, k, v, o, dO, m, l, scale: float, dtype=np.float64):
    """dQ, dK, dV of the causal attention core from the saved statistics
    (src/kernels/attention.cu:697-1011; equals autograd of pytorch_src/model.py:44-52):

        P  = exp(S - m) / l            S = scale * Q K^T (causal)
        dV = P^T dO
        dP = dO V^T
        dS = scale * P * (dP - D)      D = rowsum(dO * O)
        dQ = dS K,  dK = dS^T Q
    """
    shape = np.asarray(q).shape
    qf, kf, vf = _bh_view(q, dtype), _bh_view(k, dtype), _bh_view(v, dtype)
    of, dof = _bh_view(o, dtype), _bh_view(dO, dtype)
    BH, T, d = qf.shape
    mf = np.asarray(m, dtype=dtype).reshape(BH, T)
    lf = np.asarray(l, dtype=dtype).reshape(BH, T)
    D = attention_precompute_dot_do_o(dof, of, dtype)
    dq, dk, dv = np.empty_like(qf), np.empty_like(kf), np.empty_like(vf)
    keep = np.tril(np.ones((T, T), dtype=bool))
    for i in range(BH):
        s = (qf[i] @ kf[i].T) * dtype(scale)
        p = np.where(keep, np.exp(np.where(keep, s, 0) - mf[i][:, None]) / lf[i][:, None], 0)
        dv[i] = p.T @ dof[i]
        dp = dof[i] @ vf[i].T
        ds = dtype(scale) * p * (dp - D[i][:, None])
        dq[i] = ds @ kf[i]
        dk[i] = ds.T @ qf[i]
    return dq.reshape(shape), dk.reshape(shape), dv.reshape(shape)


def attention_forward_backward(q, k, v, dO, scale: float, dtype=np.float64):
    """Convenience: forward then backward; returns dict(out, m, l, dq, dk, dv)."""
    out, m, l = attention_forward(q, k, v, scale, dtype)
    dq, dk, dv = attention_backward(q, k, v, out, dO, m, l, scale, dtype)
    return dict(out=out, m=m, l=l, dq=dq, dk=dk, dv=dv)


# --------------------------------------------------------------------------- whole MHA block (config 1)
def layernorm_forward(x, eps=1e-5, dtype=np.float64):
    """LayerNorm with gamma = 1, beta = 0 (pytorch_src/model.py:68; nn.LayerNorm, biased variance)."""
    x = np.asarray(x, dtype=dtype)
    mu = x.mean(axis=-1, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=-1, keepdims=True)
    rstd = 1.0 / np.sqrt(var + eps)
    return (x - mu) * rstd, rstd


def layernorm_backward(dy, xhat, rstd):
    """Gradient of layernorm_forward with respect to its input (gamma = 1)."""
    C = dy.shape[-1]
    return rstd * (dy - dy.mean(axis=-1, keepdims=True) - xhat * (dy * xhat).sum(axis=-1, keepdims=True) / C)


def mha_block_forward_backward(x, w_qkv, b_qkv, w_proj, b_proj, dY, H: int, apply_layernorm=True,
                               dtype=np.float64):
    """LayerNorm (gamma=1, beta=0) -> QKV projection -> split -> causal attention -> merge -> output
    projection, forward and backward (pytorch_src/model.py:31-58 preceded by :74's ln_1).

    Weights are stored (in, out) row-major as the CUDA parameter blob does (include/model.h:14,16),
    i.e. y = x @ W + b. Returns a dict with y, dx, dw_qkv, db_qkv, dw_proj, db_proj and the
    intermediates qkv, q, k, v, out, m, l, dq, dk, dv.
    """
    x = np.asarray(x, dtype=dtype)
    B, T, C = x.shape
    d = C // H
    scale = 1.0 / math.sqrt(d)
    w_qkv, w_proj = np.asarray(w_qkv, dtype=dtype), np.asarray(w_proj, dtype=dtype)
    if apply_layernorm:
        h, rstd = layernorm_forward(x, dtype=dtype)
    else:
        h, rstd = x, None
    qkv = h @ w_qkv + np.asarray(b_qkv, dtype=dtype)
    q, k, v = qkv_split_transpose_forward(qkv, B, T, H, d)
    out, m, l = attention_forward(q, k, v, scale, dtype)
    merged = head_merge_transpose_forward(out)
    y = merged @ w_proj + np.asarray(b_proj, dtype=dtype)

    dY = np.asarray(dY, dtype=dtype)
    dw_proj = merged.reshape(-1, C).T @ dY.reshape(-1, C)
    db_proj = dY.reshape(-1, C).sum(axis=0)
    dmerged = dY @ w_proj.T
    dout = head_merge_transpose_backward(dmerged, H)
    dq, dk, dv = attention_backward(q, k, v, out, dout, m, l, scale, dtype)
    dqkv = qkv_split_transpose_backward(dq, dk, dv)
    dw_qkv = h.reshape(-1, C).T @ dqkv.reshape(-1, 3 * C)
    db_qkv = dqkv.reshape(-1, 3 * C).sum(axis=0)
    dh = dqkv @ w_qkv.T
    dx = layernorm_backward(dh, h, rstd) if apply_layernorm else dh
    return dict(y=y, dx=dx, dw_qkv=dw_qkv, db_qkv=db_qkv, dw_proj=dw_proj, db_proj=db_proj, qkv=qkv, q=q, k=k, v=v,
                out=out, m=m, l=l, dout=dout, dq=dq, dk=dk, dv=dv, dqkv=dqkv)


# --------------------------------------------------------------------------- metrics
def compute_metrics(test: np.ndarray, ref: np.ndarray):
    """max-abs, RMS and relative-L2 error as the parity gate defines them
    (scripts/compare_parity.py:11-26: rel_l2 = ||test - ref||_2 / ||ref||_2)."""
    a = np.asarray(test, dtype=np.float64).ravel()
    b = np.asarray(ref, dtype=np.float64).ravel()
    diff = a - b
    nb = float(np.linalg.norm(b))
    return dict(max_abs=float(np.abs(diff).max()) if diff.size else 0.0,
                rms=float(np.sqrt((diff ** 2).mean())) if diff.size else 0.0,
                rel_l2=float(np.linalg.norm(diff) / nb) if nb > 0 else float(np.linalg.norm(diff)))


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round float32 values to the nearest bfloat16 (ties to even) and return them as float32;
    used so that BF16 runs are compared with the oracle evaluated on the same quantised inputs."""
    a = np.ascontiguousarray(x, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return rounded.astype(np.uint32).view(np.float32).reshape(a.shape)


def attention_flops(B: int, H: int, T: int, d: int):
    """Algorithmic FLOP count with causal pairs counted as half the square:
    forward 2*B*H*T^2*d (two GEMMs), backward 5*B*H*T^2*d (five GEMMs)."""
    f = 2.0 * B * H * T * T * d
    return dict(fwd=f, bwd=2.5 * f, total=3.5 * f)
