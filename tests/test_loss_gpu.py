"""Parity of the fused softmax cross-entropy (libb200loss, drop-in for cross_entropy_forward_backward of
sarimahsan/transformer-cuda, src/kernels/loss.cu:97-125) against the CPU oracle, through the C ABI.

Gates: the reference's own parity gate is 1e-5 on the loss (scripts/compare_parity.py:108-117); d_logits are
probabilities / rows, so they are compared after multiplying by rows, max-abs <= 5e-6 (FP32 exponentials)."""
import os

import numpy as np
import pytest

from conftest import GOLDEN_DIR

pytestmark = pytest.mark.gpu
PROB_TOL = 5e-6
LOSS_TOL = 1e-5


@pytest.fixture(scope="module")
def loss_ops(pkg):
    import importlib
    return importlib.import_module(pkg.__name__ + ".loss_ops")


def _case(rows, V, seed, spread=3.0):
    rng = np.random.default_rng(seed)
    logits = (rng.standard_normal((rows, V)) * spread).astype(np.float32)
    targets = rng.integers(0, V, size=rows).astype(np.int32)
    return logits, targets


def _run(loss_ops, logits, targets, in_place=False, misalign=False):
    import torch
    rows, V = logits.shape
    if misalign:  # a view that starts 4 bytes into an allocation: not 16-byte aligned
        store = torch.empty(rows * V + 1, dtype=torch.float32, device="cuda")
        lt = store[1:].view(1, rows, V)
        lt.copy_(torch.from_numpy(logits).view(1, rows, V))
    else:
        lt = torch.from_numpy(logits).cuda().view(1, rows, V)
    tt = torch.from_numpy(targets).cuda()
    out = lt if in_place else (torch.empty_like(lt) if not misalign else lt)
    path = loss_ops.kernel_path(lt, out)
    d, loss = loss_ops.cross_entropy_forward_backward(lt, tt, dlogits=out)
    loss_ops.check_device_fault()
    return d.cpu().numpy().reshape(rows, V), float(loss), path


# (rows, V): the reference's test shape; all four 4-byte phases of a row start; one chunk more or less from row to row
# (V = 8197); the GPT-2 vocabulary; the largest resident row; rows that exceed shared memory; V below 8
RESIDENT = [(64, 65), (37, 1000), (301, 5003), (450, 8197), (6, 50257), (3, 57344)]
STREAMING = [(3, 57345), (5, 70001), (9, 7), (4, 1)]


@pytest.mark.parametrize("rows,V", RESIDENT + STREAMING)
def test_matches_the_oracle(loss_ops, rows, V):
    from oracle import cross_entropy_oracle as ce
    logits, targets = _case(rows, V, seed=rows * 7919 + V)
    got, loss, path = _run(loss_ops, logits, targets)
    assert path == (0 if (rows, V) in RESIDENT else 1)
    want, want_loss = ce.cross_entropy_forward_backward(logits, targets)
    assert np.abs(got.astype(np.float64) - want).max() * rows <= PROB_TOL
    assert abs(loss - want_loss) <= LOSS_TOL
    assert np.abs(got.sum(axis=1, dtype=np.float64)).max() * rows <= 1e-4  # softmax - onehot sums to zero


def test_in_place_and_unaligned_buffers(loss_ops):
    from oracle import cross_entropy_oracle as ce
    logits, targets = _case(200, 5003, seed=11)
    want, want_loss = ce.cross_entropy_forward_backward(logits, targets)
    for kw, path_want in ((dict(in_place=True), 0), (dict(misalign=True), 1)):
        got, loss, path = _run(loss_ops, logits, targets, **kw)
        assert path == path_want
        assert np.abs(got.astype(np.float64) - want).max() * 200 <= PROB_TOL
        assert abs(loss - want_loss) <= LOSS_TOL


def test_loss_of_the_reference_generator_files(loss_ops):
    """Logits and targets written by the reference's PyTorch generator -> its loss file, at its own 1e-5 gate."""
    for case in ("parity_audit", "parity_audit_d64"):
        d = os.path.join(GOLDEN_DIR, case)
        B, T, C, L, H, V = (int(x) for x in open(os.path.join(d, "config.txt")).read().split())
        logits = np.fromfile(os.path.join(d, "pytorch_logits.bin"), dtype=np.float32).reshape(B * T, V)
        targets = np.fromfile(os.path.join(d, "targets.bin"), dtype=np.int32)
        _, loss, _ = _run(loss_ops, logits, targets)
        assert abs(loss - float(np.fromfile(os.path.join(d, "pytorch_loss.bin"), dtype=np.float32)[0])) <= LOSS_TOL


def test_loss_is_reproducible_and_optional(loss_ops):
    import torch
    logits, targets = _case(700, 8197, seed=3)
    lt, tt = torch.from_numpy(logits).cuda().view(1, 700, 8197), torch.from_numpy(targets).cuda()
    d1, l1 = loss_ops.cross_entropy_forward_backward(lt, tt)
    d2, l2 = loss_ops.cross_entropy_forward_backward(lt, tt)
    d3, l3 = loss_ops.cross_entropy_forward_backward(lt, tt, want_loss=False)
    assert l3 is None
    assert torch.equal(d1, d2) and torch.equal(d1, d3)
    assert l1.item() == l2.item()  # fixed summation order: bit-identical from run to run


def test_full_size_vocabulary_by_properties(loss_ops):
    """The shape of the GPT step (16 x 1024 rows of 50257 logits, 3.3 GB each way): every row of d_logits sums to
    zero, the loss agrees with a float64 logsumexp on the device, and 48 sampled rows agree with the oracle."""
    import torch
    from oracle import cross_entropy_oracle as ce
    B, T, V = 16, 1024, 50257
    g = torch.Generator(device="cuda").manual_seed(4)
    logits = torch.randn(B, T, V, device="cuda", generator=g) * 2.0
    targets = torch.randint(0, V, (B * T,), device="cuda", generator=g, dtype=torch.int32)
    d, loss = loss_ops.cross_entropy_forward_backward(logits, targets)
    loss_ops.check_device_fault()
    rows = B * T
    flat, dflat = logits.view(rows, V), d.view(rows, V)
    assert float(dflat.sum(dim=1, dtype=torch.float64).abs().max()) * rows <= 1e-4
    want = 0.0
    for lo in range(0, rows, 2048):
        blk = flat[lo:lo + 2048].double()
        tgt = targets[lo:lo + 2048].long()
        want += float((torch.logsumexp(blk, dim=1) - blk.gather(1, tgt[:, None])[:, 0]).sum())
    assert abs(float(loss) - want / rows) <= LOSS_TOL
    pick = torch.arange(0, rows, rows // 48, device="cuda")[:48]
    sub, _ = ce.cross_entropy_forward_backward(flat[pick].cpu().numpy(), targets[pick].cpu().numpy())
    assert np.abs(dflat[pick].cpu().numpy().astype(np.float64) * rows - sub * 48).max() <= PROB_TOL
