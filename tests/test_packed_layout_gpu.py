"""GPU parity of the interleaved-layout entry points (b200attn_fwd_bf16_packed / b200attn_bwd_bf16_packed):
attention straight on the (B, T, 3*H*d) projection buffer with the output merged as (B, T, H*d), i.e. the
chain qkv_split_transpose_forward -> tiled_causal_attention_forward -> head_merge_transpose_forward of the
reference (src/model.cu:305-336) and its backward (src/model.cu:602-653) without the layout passes.

Checked three ways: against the oracle's split -> attention -> merge composition (BF16 gates:
max-abs <= 2e-2, relative-L2 <= 5e-3), bit-exactly against the (B, H, T, d) entry points for everything
that is deterministic (O, lse, dK, dV), and that bytes outside the tensors are never written."""
import math

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
MAX_ABS, REL_L2 = 2e-2, 5e-3
BF16 = torch.bfloat16


@pytest.fixture(scope="module")
def ops(pkg):
    return pkg.ops


def host(t):
    return t.float().cpu().numpy()


def gate(got, ref, what):
    m = orc.compute_metrics(got, ref)
    assert m["max_abs"] <= MAX_ABS and m["rel_l2"] <= REL_L2, f"{what}: {m}"


def split(qkv, B, T, H, d):
    """(B, T, 3*H*d) -> three contiguous (B, H, T, d) tensors, by torch indexing."""
    x = qkv.view(B, T, 3, H, d).permute(2, 0, 3, 1, 4).contiguous()
    return x[0], x[1], x[2]


def merge(x):
    """(B, H, T, d) -> (B, T, H*d)."""
    B, H, T, d = x.shape
    return x.permute(0, 2, 1, 3).reshape(B, T, H * d).contiguous()


# the last case is long enough (d = 128, T > 4096) for the one-CTA-per-SM forward kernel, at a ragged length
CASES = [(2, 300, 3, 64), (1, 1024, 2, 128), (3, 100, 2, 64), (1, 129, 5, 128), (2, 1, 2, 64), (1, 4200, 2, 128)]


@pytest.mark.parametrize("B,T,H,d", CASES)
def test_packed_forward_backward(ops, B, T, H, d):
    scale = 1.0 / math.sqrt(d)
    C = H * d
    qkv = ops.fill_normal_(torch.empty(B, T, 3 * C, device="cuda", dtype=BF16), seed=1000 + T + d)
    dout = ops.fill_normal_(torch.empty(B, T, C, device="cuda", dtype=BF16), seed=2000 + T + d)

    out, lse = ops.attention_forward_bf16_packed(qkv, H, scale)
    dqkv = ops.attention_backward_bf16_packed(qkv, out, dout, lse, H, scale)
    ops.check_device_fault()
    assert out.shape == (B, T, C) and lse.shape == (B, H, T) and dqkv.shape == qkv.shape

    # oracle: split -> attention -> merge on the BF16-rounded inputs
    q, k, v = orc.qkv_split_transpose_forward(host(qkv), B, T, H, d)
    dO = orc.head_merge_transpose_backward(host(dout), H)
    ref = orc.attention_forward_backward(q, k, v, dO, scale)
    gate(host(out), orc.head_merge_transpose_forward(ref["out"]), "out")
    assert np.abs(host(lse) - (ref["m"] + np.log(ref["l"])).reshape(B, H, T)).max() <= 1e-4
    ref_dqkv = orc.qkv_split_transpose_backward(ref["dq"], ref["dk"], ref["dv"])
    got = host(dqkv).reshape(B, T, 3, C)
    want = np.asarray(ref_dqkv).reshape(B, T, 3, C)
    for i, name in enumerate(("dq", "dk", "dv")):
        gate(got[:, :, i], want[:, :, i], name)

    # the (B, H, T, d) entry points on the same values: identical tiles, identical arithmetic
    qs, ks, vs = split(qkv, B, T, H, d)
    out_s, lse_s = ops.attention_forward_bf16(qs, ks, vs, scale)
    assert torch.equal(merge(out_s.view(B, H, T, d)), out)
    assert torch.equal(lse_s.view(B, H, T), lse)
    dos = dout.view(B, T, H, d).permute(0, 2, 1, 3).contiguous()
    dq_s, dk_s, dv_s = ops.attention_backward_bf16(qs, ks, vs, out_s, dos, lse_s, scale)
    g = dqkv.view(B, T, 3, H, d)
    assert torch.equal(g[:, :, 1].permute(0, 2, 1, 3), dk_s.view(B, H, T, d))
    assert torch.equal(g[:, :, 2].permute(0, 2, 1, 3), dv_s.view(B, H, T, d))
    # dQ is summed with floating-point reductions in both paths: equal up to summation order
    diff = (g[:, :, 0].permute(0, 2, 1, 3).float() - dq_s.view(B, H, T, d).float()).abs().max().item()
    assert diff <= 2.0 ** -6 * max(1.0, dq_s.float().abs().max().item())


def test_packed_writes_stay_inside(ops):
    """T is not a multiple of the 128-row tile: tile stores of the last rows must be clipped per (b, h), so
    neither the next batch entry nor guard bytes after the buffers change."""
    B, T, H, d = 2, 130, 2, 64
    C = H * d
    scale = 1.0 / math.sqrt(d)
    guard = 4096
    qkv = ops.fill_normal_(torch.empty(B, T, 3 * C, device="cuda", dtype=BF16), seed=7)
    dout = ops.fill_normal_(torch.empty(B, T, C, device="cuda", dtype=BF16), seed=8)
    out_buf = torch.full((B * T * C + guard,), 7.0, device="cuda", dtype=BF16)
    g_buf = torch.full((B * T * 3 * C + guard,), 7.0, device="cuda", dtype=BF16)
    out = out_buf[: B * T * C].view(B, T, C)
    dqkv = g_buf[: B * T * 3 * C].view(B, T, 3 * C)
    _, lse = ops.attention_forward_bf16_packed(qkv, H, scale, out=out)
    ops.attention_backward_bf16_packed(qkv, out, dout, lse, H, scale, dqkv=dqkv)
    ops.check_device_fault()
    assert torch.all(out_buf[B * T * C:] == 7.0) and torch.all(g_buf[B * T * 3 * C:] == 7.0)
    # every element inside was produced (7.0 would be an unlikely exact value everywhere)
    assert (out == 7.0).float().mean().item() < 0.01 and (dqkv == 7.0).float().mean().item() < 0.01
    # and batch entry 1 does not depend on batch entry 0 having been processed before or after it
    out1, lse1 = ops.attention_forward_bf16_packed(qkv[1:].contiguous(), H, scale)
    assert torch.equal(out1[0], out[1])
