"""CPU oracle for the fused softmax cross-entropy that opens the model's backward pass (numpy).

TEST INFRASTRUCTURE ONLY: the checker the CUDA loss kernels are compared against; nothing in the product path
imports it. Only tests/ and the smoke check may import it.

Restates cross_entropy_kernel and its launcher of sarimahsan/transformer-cuda (src/kernels/loss.cu:24-95 and
:97-125) row by row:

    max_i   = max_v logits[i, v]                                   loss.cu:42-59
    sum_i   = sum_v exp(logits[i, v] - max_i)                      loss.cu:62-74
    loss_i  = log(sum_i) - (logits[i, target_i] - max_i)           loss.cu:78-84
    dlogits[i, v] = (exp(logits[i, v] - max_i) / (sum_i + 1e-12) - [v == target_i]) / rows      loss.cu:87-91
    loss    = (sum_i loss_i) / rows                                loss.cu:120-122 (summed on the host)

Parity of this oracle is pinned: tests/test_oracle_golden.py checks its loss against the logits, targets and loss
files the reference's own PyTorch generator wrote (tests/golden/parity_audit*/, pytorch_src/utils.py:167-240) and
its dlogits against autograd of torch.nn.functional.cross_entropy, the loss the reference's PyTorch model uses
(pytorch_src/model.py:118-121). Arithmetic is float64 unless dtype says otherwise.
"""
from __future__ import annotations

import numpy as np

SUM_EPS = 1e-12  # src/kernels/loss.cu:77


def cross_entropy_forward_backward(logits, targets, dtype=np.float64):
    """logits (rows, V) or (B, T, V), targets with rows integers in [0, V) -> (dlogits like logits, mean loss)."""
    shape = np.shape(logits)
    x = np.asarray(logits, dtype=dtype).reshape(-1, shape[-1])
    t = np.asarray(targets).reshape(-1).astype(np.int64)
    rows = x.shape[0]
    assert t.shape[0] == rows
    mx = x.max(axis=1, keepdims=True)
    e = np.exp(x - mx)
    s = e.sum(axis=1, keepdims=True)
    row_loss = np.log(s[:, 0]) - (x[np.arange(rows), t] - mx[:, 0])
    d = e / (s + dtype(SUM_EPS))
    d[np.arange(rows), t] -= 1
    d /= rows
    return d.reshape(shape), float(row_loss.sum() / rows)
