"""The launchers are capture-safe, as the reference's benchmark --cuda_graph path requires
(src/benchmark.cu:158-175 captures forward + backward + optimizer on one stream and replays it):
once scratch is reserved, a captured sequence allocates nothing, and replays give the eager results.
Without a reservation a call that would have to grow scratch during capture fails with
B200ATTN_ERR_SCRATCH instead of allocating."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _inputs(ops, BH, T, d, dtype, seed):
    return [ops.fill_normal_(torch.empty(BH, T, d, device="cuda", dtype=dtype), seed=seed + i) for i in range(4)]


def test_bf16_forward_backward_in_a_cuda_graph(pkg):
    ops = pkg.ops
    BH, T, d = 6, 384, 64
    scale = 1.0 / math.sqrt(d)
    q, k, v, dO = _inputs(ops, BH, T, d, BF16, 900)
    o, lse = torch.empty_like(q), torch.empty(BH, T, device="cuda")
    dq, dk, dv = (torch.empty_like(q) for _ in range(3))
    ops.reserve(BH, T, d)
    ops.attention_forward_bf16(q, k, v, scale, o, lse)  # eager reference run (also warms up module loading)
    ops.attention_backward_bf16(q, k, v, o, dO, lse, scale, dq, dk, dv)
    torch.cuda.synchronize()
    want = [t.clone() for t in (o, lse, dk, dv)]
    want_dq = dq.clone()
    for t in (o, lse, dq, dk, dv):
        t.zero_()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        ops.attention_forward_bf16(q, k, v, scale, o, lse)
        ops.attention_backward_bf16(q, k, v, o, dO, lse, scale, dq, dk, dv)
    for _ in range(2):
        for t in (o, lse, dq, dk, dv):
            t.zero_()
        g.replay()
        torch.cuda.synchronize()
        for got, ref in zip((o, lse, dk, dv), want):
            assert torch.equal(got, ref)
        assert (dq.float() - want_dq.float()).abs().max().item() <= 2e-2  # dQ partials meet in atomics
    ops.check_device_fault()


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
def test_float_launch_api_in_a_cuda_graph(pkg, mode):
    ops = pkg.ops
    B, H, T, d = 2, 2, 160, 64
    scale = 1.0 / math.sqrt(d)
    q, k, v, dO = (t.view(B, H, T, d) for t in _inputs(ops, B * H, T, d, torch.float32, 910))
    out, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
    m, l, ws = (torch.empty(B, H, T, device="cuda") for _ in range(3))
    ops.set_math_mode(mode)
    try:
        ops.reserve(B * H, T, d)

        def run():
            ops.tiled_causal_attention_forward(q, k, v, out, B, H, T, d, scale, m, l)
            ops.tiled_causal_attention_backward(q, k, v, out, dO, m, l, dq, dk, dv, ws, B, H, T, d, scale)

        run()
        torch.cuda.synchronize()
        want = [t.clone() for t in (out, m, l, dq, dk, dv)]
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            run()
        for t in (out, dq, dk, dv):
            t.zero_()
        g.replay()
        torch.cuda.synchronize()
        for got, ref in zip((out, m, l, dq, dk, dv), want):
            assert (got - ref).abs().max().item() <= (1e-6 if mode == "fp32" else 2e-2)
    finally:
        ops.set_math_mode("fp32")


def test_growing_scratch_during_capture_is_refused(pkg):
    ops, lib = pkg.ops, pkg.lib
    lib.call("b200attn_release")  # drop the reservation so that the next backward would have to allocate
    BH, T, d = 2, 256, 128
    q, k, v, dO = _inputs(ops, BH, T, d, BF16, 920)
    o, lse = ops.attention_forward_bf16(q, k, v, 0.1)
    dq, dk, dv = (torch.empty_like(q) for _ in range(3))
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with pytest.raises(lib.B200AttnError) as e:
        with torch.cuda.graph(g):
            ops.attention_backward_bf16(q, k, v, o, dO, lse, 0.1, dq, dk, dv)
    assert e.value.code == lib.ERR_SCRATCH
    torch.cuda.synchronize()
    ops.attention_backward_bf16(q, k, v, o, dO, lse, 0.1, dq, dk, dv)  # outside capture it simply grows
    torch.cuda.synchronize()
