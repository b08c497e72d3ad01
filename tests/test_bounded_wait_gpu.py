"""A bounded wait that runs out, on a healthy GPU: the library's self-test kernel waits - with a limit of a few
thousand polls - on a barrier that nothing signals. Nothing traps, faults or hangs: the wait gives up, the kernel
ends normally, the fault word names the wait, b200attn_check_device_fault reports and clears it, and the same
context then runs a correct forward + backward."""
import ctypes
import math

import pytest
import torch

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def test_a_wait_that_runs_out_is_reported_and_the_context_stays_usable(pkg):
    lib, ops = pkg.lib, pkg.ops
    ops.check_device_fault()  # clean start
    report = torch.zeros(2, device="cuda", dtype=torch.int32)
    lib.call("b200attn_selftest_bounded_wait", ctypes.c_void_p(report.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    code = ctypes.c_uint(0)
    rc = lib.load().b200attn_check_device_fault(ctypes.byref(code))
    assert rc == lib.ERR_DEVICE_FAULT
    assert code.value == 0x57410000 | 0x7E57, hex(code.value)   # "WA" | identifier of the wait that gave up
    assert "0x57417e57" in lib.load().b200attn_last_error().decode().lower()
    flag, second_wait_kcycles = report.cpu().tolist()
    assert flag == 1                      # the CTA's abort flag was set by the wait that gave up
    assert second_wait_kcycles < 20000    # the next wait left after at most 1024 polls instead of 2^20
    # the word was cleared by the check, and nothing is left behind
    code = ctypes.c_uint(123)
    assert lib.load().b200attn_check_device_fault(ctypes.byref(code)) == lib.OK and code.value == 0

    # the context is intact: a normal forward + backward is still right
    BH, T, d = 2, 200, 64
    scale = 1.0 / math.sqrt(d)
    q, k, v, dO = (ops.fill_normal_(torch.empty(BH, T, d, device="cuda", dtype=BF16), seed=900 + i) for i in range(4))
    out, lse = ops.attention_forward_bf16(q, k, v, scale)
    dq, dk, dv = ops.attention_backward_bf16(q, k, v, out, dO, lse, scale)
    ops.check_device_fault()
    f = lambda t: t.float().cpu().numpy()
    ref = orc.attention_forward_backward(f(q), f(k), f(v), f(dO), scale)
    for got, key in ((out, "out"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        m = orc.compute_metrics(f(got), ref[key])
        assert m["max_abs"] <= 2e-2 and m["rel_l2"] <= 5e-3, (key, m)
