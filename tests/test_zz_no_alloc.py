"""b200attn_bwd_bf16_noalloc: the backward for callers that cannot allocate device memory (their
pool owns the GPU, or cudaMalloc's implicit synchronisation is not allowed where they run).

It takes its scratch from a static device array, so it must give what b200attn_bwd_bf16 gives. The
test calls it through the C ABI twice in a row with different data and shapes - the array keeps the
previous call's contents, so the second call shows that stale sums are cleared - and compares each
result with the allocating entry point within the BF16 gates of the other tests (max-abs <= 2e-2,
relative-L2 <= 5e-3): the two entry points may run different kernel variants (at head dim 64 the
allocating one uses the persistent kernel, whose extra scratch is not part of the static array's
documented budget), and dQ is reduced with atomics in both.
After each call the device fault word is polled (the entry point keeps its own word inside the static
array). A third test checks what the entry point exists for: with the allocating path's scratch released,
a call leaves the device's free memory where it was. This file sorts last so that a run that stops at the
first failure has already run everything else; it also passes alone in a fresh process, where its first
call performs the per-device set-up."""
import math

import pytest
import torch

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _inputs(ops, BH, T, d, seed):
    return [ops.fill_normal_(torch.empty(BH, T, d, device="cuda", dtype=BF16), seed=seed + i) for i in range(4)]


def test_two_calls_in_a_row_match_the_allocating_entry_point(pkg):
    ops = pkg.ops
    for BH, T, d, seed in ((6, 700, 64, 300), (3, 260, 128, 400)):  # second call: smaller, other head dim, other data
        scale = 1.0 / math.sqrt(d)
        q, k, v, dO = _inputs(ops, BH, T, d, seed)
        out, lse = ops.attention_forward_bf16(q, k, v, scale)
        want_dq, want_dk, want_dv = ops.attention_backward_bf16(q, k, v, out, dO, lse, scale)
        dq, dk, dv = (torch.full_like(q, float("nan")) for _ in range(3))
        ops.attention_backward_bf16_noalloc(q, k, v, out, dO, lse, scale, dq, dk, dv)
        ops.check_device_fault()  # synchronises; raises if a bounded wait of the no-alloc kernels ran out
        for got, want, name in ((dq, want_dq, "dq"), (dk, want_dk, "dk"), (dv, want_dv, "dv")):
            m = orc.compute_metrics(got.float().cpu().numpy(), want.float().cpu().numpy())
            assert m["max_abs"] <= 2e-2 and m["rel_l2"] <= 5e-3, (name, m)


def test_shapes_beyond_the_static_array_are_rejected(pkg):
    lib = pkg.lib
    BH, T, d = 64, 4096, 128  # 128 MiB of dQ accumulator: does not fit in 32 MiB
    assert 4 * BH * T * d > lib.NOALLOC_SCRATCH_BYTES
    x = torch.empty(1, device="cuda", dtype=BF16)  # never touched: the size check comes first
    f = torch.empty(1, device="cuda")
    rc = lib.load().b200attn_bwd_bf16_noalloc(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(),
                                              f.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), BH, T, d, 1.0, None)
    assert rc == lib.ERR_UNSUPPORTED
    text = lib.load().b200attn_last_error().decode()
    assert "b200attn_bwd_bf16_noalloc" in text and str(lib.NOALLOC_SCRATCH_BYTES) in text, text
    # a row count whose byte size would wrap 64 bits is rejected by the same check, not by a later failure
    rc = lib.load().b200attn_bwd_bf16_noalloc(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(),
                                              f.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), 2**31 - 1, 2**31 - 1, 128,
                                              1.0, None)
    assert rc == lib.ERR_UNSUPPORTED


def test_a_call_leaves_free_device_memory_unchanged(pkg):
    ops = pkg.ops
    BH, T, d = 4, 384, 64
    scale = 1.0 / math.sqrt(d)
    q, k, v, dO = _inputs(ops, BH, T, d, 500)
    out, lse = ops.attention_forward_bf16(q, k, v, scale)
    dq, dk, dv = (torch.empty_like(q) for _ in range(3))
    # first call: module load and per-device set-up happen here, and the kernels get loaded
    ops.attention_backward_bf16_noalloc(q, k, v, out, dO, lse, scale, dq, dk, dv)
    torch.cuda.synchronize()
    ops.release()  # drop the allocating path's scratch so that it cannot mask an allocation
    free_before = torch.cuda.mem_get_info()[0]
    ops.attention_backward_bf16_noalloc(q, k, v, out, dO, lse, scale, dq, dk, dv)
    ops.check_device_fault()
    free_after = torch.cuda.mem_get_info()[0]
    assert free_after >= free_before, (free_before, free_after)
