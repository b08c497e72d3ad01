"""The library's per-launch timing of its two tensor-core kernels (b200attn_kernel_timing, b200attn_kernel_times,
b200attn_kernel_time_samples - what bench.py's roofline durations come from): every N-th launch of each kernel is
sampled, the single durations add up to the reported sums, enabling again clears the records, and the results of the
sampled launches are the results of the unsampled ones."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def test_every_second_launch_is_sampled_and_the_samples_add_up(pkg):
    ops = pkg.ops
    BH, T, d = 4, 384, 64
    scale = 1.0 / math.sqrt(d)
    q, k, v, dO = (ops.fill_normal_(torch.empty(BH, T, d, device="cuda", dtype=BF16), seed=700 + i) for i in range(4))
    out0, lse0 = ops.attention_forward_bf16(q, k, v, scale)
    dq0, dk0, dv0 = ops.attention_backward_bf16(q, k, v, out0, dO, lse0, scale)
    torch.cuda.synchronize()
    try:
        ops.kernel_timing(True, every=2)
        for _ in range(5):
            out, lse = ops.attention_forward_bf16(q, k, v, scale)
            dq, dk, dv = ops.attention_backward_bf16(q, k, v, out, dO, lse, scale)
        kt = ops.kernel_times()
        fwd, bwd = ops.kernel_time_samples(False), ops.kernel_time_samples(True)
        assert kt["fwd_launches"] == 3 and kt["bwd_launches"] == 3      # launches 0, 2 and 4 of five
        assert len(fwd) == 3 and len(bwd) == 3
        assert all(0.0 < x < 50.0 for x in fwd + bwd)
        assert sum(fwd) == pytest.approx(kt["fwd_ms"], rel=1e-4) and sum(bwd) == pytest.approx(kt["bwd_ms"], rel=1e-4)
        # forward and statistics are deterministic: sampled or not, the same bits (dQ is summed with atomics)
        assert torch.equal(out, out0) and torch.equal(lse, lse0) and torch.equal(dk, dk0) and torch.equal(dv, dv0)
        assert (dq.float() - dq0.float()).abs().max().item() <= 2e-2
        ops.kernel_timing(True, every=1)                                   # enabling again clears the records
        assert ops.kernel_time_samples(True) == [] and ops.kernel_times()["fwd_launches"] == 0
        ops.attention_forward_bf16(q, k, v, scale)
        assert len(ops.kernel_time_samples(False)) == 1 and ops.kernel_time_samples(True) == []
    finally:
        ops.kernel_timing(False)
    assert ops.kernel_times()["fwd_launches"] == 0
    ops.check_device_fault()
