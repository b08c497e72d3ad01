"""CPU restatement of the reference's attention math with the library the reference itself uses.

TEST / BASELINE INFRASTRUCTURE ONLY (see attention_oracle.py): used as the timed CPU baseline by
bench.py and as a cross-check of the numpy oracle in tests; never on the product path.

`attention_core` repeats, op for op, steps 3-5 of CausalSelfAttention.forward in the reference
(pytorch_src/model.py:44-52: scaled q @ k^T, masked_fill with -inf below a tril mask, softmax, @ v);
the backward is PyTorch autograd, as in the reference's training loop (pytorch_src/train.py).
The reference module cannot be imported on the benchmark machine (its checkout is not there), which
is why this port exists; tests/test_oracle_golden.py pins the same math against vectors produced by
the real module.
"""
import math
import time

import torch
import torch.nn.functional as F


def attention_core(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    """q, k, v: (..., T, d) FP32 -> (..., T, d). pytorch_src/model.py:44-52."""
    T = q.shape[-2]
    att = (q @ k.transpose(-2, -1)) * scale
    mask = torch.tril(torch.ones(T, T, device=q.device))
    att = att.masked_fill(mask == 0, float("-inf"))
    probs = F.softmax(att, dim=-1)
    return probs @ v


def forward_backward(q, k, v, dO, scale):
    """One forward + autograd backward of the core; returns (out, dq, dk, dv)."""
    q, k, v = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    out = attention_core(q, k, v, scale)
    out.backward(dO)
    return out.detach(), q.grad, k.grad, v.grad


def time_forward_backward(BH: int, T: int, d: int, budget_s: float = 15.0, max_slabs_per_call: int = 8, seed: int = 0):
    """Time the core forward+backward on the host CPU with every thread torch has, on (batch, head)
    slabs of the given shape, until about `budget_s` seconds of work are done (at least one call after
    one warm-up call). Slabs are processed `max_slabs_per_call` at a time so the T x T matrices fit in RAM
    (for T >= 4096 one slab per call). Returns dict(seconds_per_slab, slabs_timed, threads, calls)."""
    g = torch.Generator().manual_seed(seed)
    per_call = max(1, min(max_slabs_per_call, BH, (1 << 28) // max(1, T * T)))
    q, k, v, dO = (torch.randn(per_call, T, d, generator=g) for _ in range(4))
    scale = 1.0 / math.sqrt(d)
    forward_backward(q, k, v, dO, scale)  # warm-up
    calls, t0 = 0, time.perf_counter()
    while True:
        forward_backward(q, k, v, dO, scale)
        calls += 1
        el = time.perf_counter() - t0
        if el >= budget_s or calls * per_call >= 4 * BH:
            break
    return dict(seconds_per_slab=el / (calls * per_call), slabs_timed=calls * per_call, threads=torch.get_num_threads(),
                calls=calls, slabs_per_call=per_call)
