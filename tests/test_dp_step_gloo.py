"""The data-parallel training step's gradient exchange (config 4) on CPU with two gloo ranks: each rank computes
gradients of the same seeded model on its OWN data, the flat gradient buffer is averaged across ranks
(dist.average_gradients_, the host-side statement of the harness's ncclAllReduce(avg)), and every rank applies the
same clip + AdamW update. Checked: the replicas are bit-identical after the steps, and they match a single process
that sees both ranks' data in one batch (mean loss), i.e. the exchange is a mean and happens before clip/AdamW."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from conftest import ROOT

LR, BETAS, WD, CLIP, STEPS = 3e-4, (0.9, 0.95), 0.1, 1.0, 3


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _model():
    torch.manual_seed(42)  # identical initial weights on every rank, as in the harness
    return torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.GELU(), torch.nn.Linear(32, 8))


def _data(rank, step):
    g = torch.Generator().manual_seed(1000 * (rank + 1) + step)  # distinct data per rank
    return torch.randn(12, 16, generator=g), torch.randn(12, 8, generator=g)


def _flat_grads(model):
    return torch.cat([p.grad.reshape(-1) for p in model.parameters()])


def _set_grads(model, flat):
    o = 0
    for p in model.parameters():
        p.grad.copy_(flat[o:o + p.numel()].view_as(p))
        o += p.numel()


def _worker(rank, world, port, out_dir):
    import sys
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import __graft_entry__ as entry
    entry.load_package()
    from transformer_cuda_b200 import dist as pdist
    pdist.init(backend="gloo")
    torch.set_num_threads(1)
    model = _model()
    opt = torch.optim.AdamW(model.parameters(), lr=LR, betas=BETAS, weight_decay=WD)
    for step in range(STEPS):
        x, y = _data(rank, step)
        opt.zero_grad()
        torch.nn.functional.mse_loss(model(x), y).backward()
        flat = _flat_grads(model)
        if step % 2 == 0:
            flat = pdist.average_gradients_(flat)                 # the exchange: once, on the finished buffer
        else:                                                     # ... or part by part, in the order the harness uses
            n = flat.numel()
            flat = pdist.average_gradients_in_parts_(flat, pdist.gradient_parts(2, n // 4, n // 4, n - 3 * (n // 4)))
        _set_grads(model, flat)
        torch.nn.utils.clip_grad_norm_(model.parameters(), CLIP)  # global-norm clip sees the AVERAGED gradient
        opt.step()
    np.save(os.path.join(out_dir, f"params_{rank}.npy"), torch.cat([p.detach().reshape(-1) for p in model.parameters()]).numpy())
    torch.distributed.destroy_process_group()


@pytest.mark.timeout(180)
def test_replicas_stay_identical_and_match_one_big_batch(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    p0, p1 = (np.load(tmp_path / f"params_{r}.npy") for r in range(world))
    assert np.array_equal(p0, p1)  # bit-identical replicas

    # one process, both ranks' data in one batch: the mean over 24 rows equals the mean of the two 12-row means
    torch.set_num_threads(1)
    model = _model()
    opt = torch.optim.AdamW(model.parameters(), lr=LR, betas=BETAS, weight_decay=WD)
    for step in range(STEPS):
        xs, ys = zip(*(_data(r, step) for r in range(world)))
        opt.zero_grad()
        torch.nn.functional.mse_loss(model(torch.cat(xs)), torch.cat(ys)).backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), CLIP)
        opt.step()
    single = torch.cat([p.detach().reshape(-1) for p in model.parameters()]).numpy()
    assert np.abs(p0 - single).max() <= 1e-6


def test_single_rank_is_a_no_op(pkg):
    from transformer_cuda_b200 import dist as pdist
    g = torch.arange(5, dtype=torch.float32)
    assert torch.equal(pdist.average_gradients_(g.clone()), g)


def test_gradient_parts_tile_the_buffer_in_backward_order(pkg):
    from transformer_cuda_b200 import dist as pdist
    # GPT-2 small: embeddings 38 597 376 + 786 432, twelve layers of 7 087 872, final LayerNorm + head 1 536 + 38 597 376
    parts = pdist.gradient_parts(12, 7087872, 38597376 + 786432, 1536 + 38597376)
    assert len(parts) == 14 and sum(c for _, c in parts) == 163037184
    assert parts[0] == (163037184 - 38598912, 38598912) and parts[-1] == (0, 39383808)
    assert [o for o, _ in parts[1:13]] == [39383808 + l * 7087872 for l in range(11, -1, -1)]
    g = torch.arange(10, dtype=torch.float32)
    assert torch.equal(pdist.average_gradients_in_parts_(g.clone(), pdist.gradient_parts(2, 3, 2, 2)), g)
    with pytest.raises(ValueError):
        pdist.average_gradients_in_parts_(g.clone(), [(0, 4), (5, 5)])
