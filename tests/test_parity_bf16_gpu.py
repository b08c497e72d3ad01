"""GPU parity of the BF16 tensor-core path (tcgen05) through the C ABI. The oracle is evaluated on
the BF16-rounded inputs, so input quantisation is not charged. Gates (outputs and gradients):
max-abs <= 2e-2 and relative-L2 <= 5e-3. Full benchmark sizes are covered by checking a subset of
(batch, head) slabs against the oracle plus size-independent properties."""
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


def make_inputs(ops, BH, T, d, seed):
    return [ops.fill_normal_(torch.empty(BH, T, d, device="cuda", dtype=BF16), seed=seed + i) for i in range(4)]


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("T", [1, 8, 100, 128, 129, 255, 256, 300, 640])
def test_forward_backward_vs_oracle(ops, T, d):
    BH = 3
    scale = 1.0 / math.sqrt(d)
    q, k, v, dO = make_inputs(ops, BH, T, d, seed=11 * T + d)
    ref = orc.attention_forward_backward(host(q), host(k), host(v), host(dO), scale)
    out, lse = ops.attention_forward_bf16(q, k, v, scale)
    dq, dk, dv = ops.attention_backward_bf16(q, k, v, out, dO, lse, scale)
    ops.check_device_fault()
    gate(host(out), ref["out"], "out")
    assert np.abs(host(lse) - (ref["m"] + np.log(ref["l"]))).max() <= 1e-4
    gate(host(dq), ref["dq"], "dq")
    gate(host(dk), ref["dk"], "dk")
    gate(host(dv), ref["dv"], "dv")


@pytest.mark.parametrize("d", [64, 128])
def test_float_api_in_bf16_mode(ops, d):
    """tiled_causal_attention_forward/backward with FP32 buffers routed through the tensor cores."""
    B, H, T = 2, 2, 200
    scale = 1.0 / math.sqrt(d)
    qb, kb, vb, dob = make_inputs(ops, B * H, T, d, seed=5)
    q, k, v, dO = (t.float().view(B, H, T, d).contiguous() for t in (qb, kb, vb, dob))
    ref = orc.attention_forward_backward(host(q), host(k), host(v), host(dO), scale)
    out, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
    m, l, ws = (torch.empty(B, H, T, device="cuda") for _ in range(3))
    ops.set_math_mode("bf16")
    try:
        ops.tiled_causal_attention_forward(q, k, v, out, B, H, T, d, scale, m, l)
        ops.tiled_causal_attention_backward(q, k, v, out, dO, m, l, dq, dk, dv, ws, B, H, T, d, scale)
        ops.check_device_fault()
    finally:
        ops.set_math_mode("fp32")
    gate(host(out), ref["out"], "out")
    assert np.abs(host(m) - ref["m"]).max() <= 1e-4
    assert np.abs(host(l) / ref["l"] - 1).max() <= 1e-4
    for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        gate(host(got), ref[key], key)


def test_unsupported_head_dim_is_an_error_not_a_noop(pkg, ops):
    """The reference silently skips the backward for d not in {32,64} (attention.cu:1009-1011);
    here an unsupported shape fails loudly."""
    q = torch.zeros(1, 16, 32, device="cuda", dtype=BF16)
    with pytest.raises(pkg.lib.B200AttnError) as e:
        ops.attention_forward_bf16(q, q, q, 1.0)
    assert e.value.code == pkg.lib.ERR_UNSUPPORTED


def test_config2_gpt2_small_shape(ops):
    """B=8, H=12, T=1024, d=64: every slab against the oracle."""
    B, H, T, d = 8, 12, 1024, 64
    scale = 1.0 / math.sqrt(d)
    q, k, v, dO = make_inputs(ops, B * H, T, d, seed=2024)
    out, lse = ops.attention_forward_bf16(q, k, v, scale)
    dq, dk, dv = ops.attention_backward_bf16(q, k, v, out, dO, lse, scale)
    ops.check_device_fault()
    ref = orc.attention_forward_backward(host(q), host(k), host(v), host(dO), scale, dtype=np.float32)
    for got, key in ((out, "out"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        gate(host(got), ref[key], key)


@pytest.mark.parametrize("BH,T,d,check", [(32, 8192, 128, (0, 17, 31)), (64, 16384, 128, (5,))])
def test_long_context_shapes_on_a_slab_subset(ops, BH, T, d, check):
    """Config 3 (B=2,H=16,T=8192,d=128) and the longest sweep point (T=16384): the kernels run on the
    whole problem; a fixed subset of slabs is compared with the oracle (a T x T FP32 matrix per slab)."""
    if BH * T * d > 2 ** 27:
        BH = 2 ** 27 // (T * d)  # keep device memory modest; slabs are independent
        check = tuple(c for c in check if c < BH) or (BH - 1,)
    scale = 1.0 / math.sqrt(d)
    q, k, v, dO = make_inputs(ops, BH, T, d, seed=77)
    out, lse = ops.attention_forward_bf16(q, k, v, scale)
    dq, dk, dv = ops.attention_backward_bf16(q, k, v, out, dO, lse, scale)
    ops.check_device_fault()
    for s in check:
        sl = slice(s, s + 1)
        ref = orc.attention_forward_backward(host(q[sl]), host(k[sl]), host(v[sl]), host(dO[sl]), scale, dtype=np.float32)
        for got, key in ((out, "out"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
            gate(host(got[sl]), ref[key], f"slab {s} {key}")


@pytest.mark.parametrize("BH,T", [(2, 4097), (1, 4224), (2, 5000)])
def test_long_forward_kernel_at_ragged_lengths(ops, BH, T):
    """d = 128 beyond T = 4096 runs the one-CTA-per-SM forward (eight softmax warps, three score buffers);
    lengths that are no multiple of 128 exercise its zero-filled loads and clipped stores. Every slab is
    compared with the oracle (a T x T FP32 matrix per slab), backward included."""
    d = 128
    scale = 1.0 / math.sqrt(d)
    q, k, v, dO = make_inputs(ops, BH, T, d, seed=3 * T)
    out, lse = ops.attention_forward_bf16(q, k, v, scale)
    dq, dk, dv = ops.attention_backward_bf16(q, k, v, out, dO, lse, scale)
    ops.check_device_fault()
    for s in range(BH):
        sl = slice(s, s + 1)
        ref = orc.attention_forward_backward(host(q[sl]), host(k[sl]), host(v[sl]), host(dO[sl]), scale, dtype=np.float32)
        assert np.abs(host(lse[sl]) - (ref["m"] + np.log(ref["l"]))).max() <= 1e-3
        for got, key in ((out, "out"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
            gate(host(got[sl]), ref[key], f"T={T} slab {s} {key}")


@pytest.mark.parametrize("B,T", [(64, 512), (32, 1024), (16, 2048), (8, 4096)])
def test_scaling_sweep_shapes_on_a_slab_subset(ops, B, T):
    """The sweep points H=32, d=128 with T = 512 ... 4096 at their full (B, T): the kernels run on the whole
    problem (B*32 slabs), the first and the last slab are compared with the oracle."""
    H, d = 32, 128
    BH = B * H
    scale = 1.0 / math.sqrt(d)
    q, k, v, dO = make_inputs(ops, BH, T, d, seed=31 + T)
    out, lse = ops.attention_forward_bf16(q, k, v, scale)
    dq, dk, dv = ops.attention_backward_bf16(q, k, v, out, dO, lse, scale)
    ops.check_device_fault()
    for s in (0, BH - 1):
        sl = slice(s, s + 1)
        ref = orc.attention_forward_backward(host(q[sl]), host(k[sl]), host(v[sl]), host(dO[sl]), scale, dtype=np.float32)
        for got, key in ((out, "out"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
            gate(host(got[sl]), ref[key], f"B={B} T={T} slab {s} {key}")


def test_size_independent_properties_at_full_size(ops):
    """Properties that need no oracle, at config-3 size: V = 1 gives O = 1 (rows of P sum to one);
    the forward is bitwise repeatable; O is linear in V; a (batch, head) shard reproduces the bits of
    the full run; dV is linear in dO."""
    BH, T, d = 32, 8192, 128
    scale = 1.0 / math.sqrt(d)
    q, k, v, dO = make_inputs(ops, BH, T, d, seed=9)
    ones = torch.ones_like(v)
    o1, _ = ops.attention_forward_bf16(q, k, ones, scale)
    assert (o1.float() - 1).abs().max().item() <= 2 ** -7
    out, lse = ops.attention_forward_bf16(q, k, v, scale)
    out_again, lse_again = ops.attention_forward_bf16(q, k, v, scale)
    assert torch.equal(out, out_again) and torch.equal(lse, lse_again)
    o2, _ = ops.attention_forward_bf16(q, k, (v.float() * 2).to(BF16), scale)
    assert torch.equal(o2, (out.float() * 2).to(BF16))  # scaling by 2 is exact in BF16
    sl = slice(12, 20)  # what rank 3 of 4 would own... any contiguous slab range
    o_sh, lse_sh = ops.attention_forward_bf16(q[sl], k[sl], v[sl], scale)
    assert torch.equal(o_sh, out[sl]) and torch.equal(lse_sh, lse[sl])
    dq, dk, dv = ops.attention_backward_bf16(q, k, v, out, dO, lse, scale)
    _, dk_sh, dv_sh = ops.attention_backward_bf16(q[sl], k[sl], v[sl], out[sl], dO[sl], lse[sl], scale)
    assert torch.equal(dk_sh, dk[sl]) and torch.equal(dv_sh, dv[sl])  # dK, dV do not depend on atomics order
    _, _, dv2 = ops.attention_backward_bf16(q, k, v, out, (dO.float() * 2).to(BF16), lse, scale)
    assert torch.equal(dv2, (dv.float() * 2).to(BF16))
    ops.check_device_fault()
    assert torch.isfinite(dq.float()).all()


def test_split_and_merge_with_conversion(ops):
    B, T, H, d = 2, 50, 3, 64
    C = H * d
    qkv = torch.randn(B, T, 3 * C, device="cuda")
    q, k, v = (torch.empty(B, H, T, d, device="cuda", dtype=BF16) for _ in range(3))
    ops.qkv_split_transpose_forward_bf16(qkv, q, k, v, B, T, H, d)
    rq, rk, rv = orc.qkv_split_transpose_forward(host(qkv), B, T, H, d)
    assert np.array_equal(host(q), orc.bf16_round(rq)) and np.array_equal(host(k), orc.bf16_round(rk))
    assert np.array_equal(host(v), orc.bf16_round(rv))
    dqkv = torch.empty(B, T, 3 * C, device="cuda")
    ops.qkv_split_transpose_backward_bf16(q, k, v, dqkv, B, T, H, d)
    assert np.array_equal(host(dqkv), orc.bf16_round(host(qkv)))
    merged = torch.empty(B, T, C, device="cuda")
    ops.head_merge_transpose_forward_bf16(q, merged, B, H, T, d)
    assert np.array_equal(host(merged), orc.head_merge_transpose_forward(host(q)))
    back = torch.empty(B, H, T, d, device="cuda", dtype=BF16)
    ops.head_merge_transpose_backward_bf16(merged, back, B, H, T, d)
    assert torch.equal(back, q)


def test_seeded_fill_is_shard_consistent(ops):
    """A shard generates exactly its part of the full tensor (counter-based stream)."""
    n = 100_003
    full = ops.fill_normal_(torch.empty(n, device="cuda", dtype=BF16), seed=42)
    part = ops.fill_normal_(torch.empty(5000, device="cuda", dtype=BF16), seed=42, offset=12345)
    assert torch.equal(part, full[12345:17345])
    f32 = ops.fill_normal_(torch.empty(1 << 20, device="cuda"), seed=7)
    assert abs(f32.mean().item()) < 5e-3 and abs(f32.std().item() - 1) < 5e-3


def test_module_bf16_mode_matches_fp32_mode(pkg):
    """The mha module in BF16 mode stays within the BF16 gates of its FP32 mode (config-1-like block, d=64)."""
    torch.manual_seed(0)
    B, T, C, H = 2, 96, 256, 4
    a32 = pkg.mha.CausalSelfAttention(C, H, T, math="fp32").cuda()
    a16 = pkg.mha.CausalSelfAttention(C, H, T, math="bf16").cuda()
    a16.load_state_dict(a32.state_dict())
    x = torch.randn(B, T, C, device="cuda")
    dY = torch.randn(B, T, C, device="cuda")
    res = []
    for mod in (a32, a16):
        xi = x.clone().requires_grad_(True)
        y = mod(xi)
        y.backward(dY)
        res.append((y.detach(), xi.grad, mod.qkv_proj.weight.grad))
    for a, b in zip(res[0], res[1]):
        m = orc.compute_metrics(host(b), host(a))
        assert m["rel_l2"] <= 2e-2, m


def test_fused_conversion_in_the_layout_launchers(pkg, ops):
    """FP32 launch API in BF16 math mode with b200attn_set_fused_convert(1): the split / head-split launchers leave
    BF16 copies of q, k, v and dO, the attention launchers pick them up (7 operand conversions skipped per layer pass)
    and every result is bit-identical to the path that converts operand by operand; dK, dV and O exactly, dQ up to the
    order of its floating-point reductions. A tensor that did not come from a layout launcher is converted as before."""
    B, T, H, d = 2, 192, 3, 64
    C, scale = H * d, 1.0 / math.sqrt(d)
    qkv = ops.fill_normal_(torch.empty(B, T, 3 * C, device="cuda"), seed=61)
    dmerged = ops.fill_normal_(torch.empty(B, T, C, device="cuda"), seed=62)

    def run(fused):
        ops.set_fused_convert(fused)
        q, k, v, out, dO, dq, dk, dv = (torch.empty(B, H, T, d, device="cuda") for _ in range(8))
        m, l, ws = (torch.empty(B, H, T, device="cuda") for _ in range(3))
        ops.qkv_split_transpose_forward(qkv, q, k, v, B, T, H, d)
        ops.tiled_causal_attention_forward(q, k, v, out, B, H, T, d, scale, m, l)
        ops.head_merge_transpose_backward(dmerged, dO, B, H, T, d)
        ops.tiled_causal_attention_backward(q, k, v, out, dO, m, l, dq, dk, dv, ws, B, H, T, d, scale)
        ops.check_device_fault()
        return q, k, v, out, dO, dq, dk, dv

    ops.set_math_mode("bf16")
    try:
        plain = run(False)
        hits0 = ops.fused_convert_hits()
        fused = run(True)
        assert ops.fused_convert_hits() - hits0 == 7  # q, k, v (forward) + q, k, v, dO (backward)
        # tensors the layout launchers never saw: converted as before, no new hits
        other = [t.clone() for t in plain[:3]]
        out2, m2, l2 = torch.empty_like(other[0]), torch.empty(B, H, T, device="cuda"), torch.empty(B, H, T, device="cuda")
        ops.tiled_causal_attention_forward(other[0], other[1], other[2], out2, B, H, T, d, scale, m2, l2)
        assert ops.fused_convert_hits() - hits0 == 7 and torch.equal(out2, plain[3])
    finally:
        ops.set_fused_convert(False)
        ops.set_math_mode("fp32")
    for i, name in enumerate(("q", "k", "v", "out", "dO")):
        assert torch.equal(plain[i], fused[i]), name
    assert torch.equal(plain[6], fused[6]) and torch.equal(plain[7], fused[7])  # dK, dV
    diff = (plain[5] - fused[5]).abs().max().item()
    assert diff <= 2.0 ** -6 * max(1.0, plain[5].abs().max().item())
