"""Host logic of the multi-GPU path on CPU: slab partitioning, and a world_size-2 gloo run in which
every rank processes only its (batch, head) slabs (the oracle stands in for the device) and the
gathered result, and the max-over-ranks time, match a single-process run."""
import math
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from conftest import ROOT


def test_slab_range_partitions(pkg):
    sr = pkg.shard.slab_range
    for total in (0, 1, 5, 32, 96, 2048):
        for world in (1, 2, 3, 4, 8):
            parts = [sr(total, r, world) for r in range(world)]
            assert parts[0].start == 0 and parts[-1].stop == total
            assert all(a.stop == b.start for a, b in zip(parts, parts[1:]))
            counts = [p.count for p in parts]
            assert max(counts) - min(counts) <= 1
    assert pkg.shard.element_offset(sr(96, 3, 8), 1024, 64) == 36 * 1024 * 64
    with pytest.raises(ValueError):
        sr(8, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total_slabs, T, d, out_path):
    import sys
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    import __graft_entry__ as entry
    from oracle import attention_oracle as orc
    pkg = entry.load_package()
    from transformer_cuda_b200 import dist as pdist
    pdist.init(backend="gloo")
    rng = np.random.default_rng(0)  # every rank derives the same full tensors, then takes its slabs
    q, k, v = (rng.standard_normal((total_slabs, T, d)).astype(np.float32) for _ in range(3))
    mine = pdist.my_slabs(total_slabs)
    sl = slice(mine.start, mine.stop)
    out, _, _ = orc.attention_forward(q[sl], k[sl], v[sl], 1 / math.sqrt(d))
    full = pdist.gather_slabs(torch.from_numpy(np.ascontiguousarray(out.astype(np.float32))), total_slabs)
    pdist.barrier()
    slowest = pdist.max_over_ranks(10.0 + rank)
    total = pdist.sum_over_ranks(float(mine.count))
    if rank == 0:
        np.savez(out_path, full=full.numpy(), slowest=slowest, total=total)
    torch.distributed.destroy_process_group()


@pytest.mark.timeout(180)
def test_two_rank_sharded_run_matches_single_process(tmp_path, pkg):
    from oracle import attention_oracle as orc
    total_slabs, T, d, world = 5, 48, 32, 2
    out_path = str(tmp_path / "gathered.npz")
    mp.spawn(_worker, args=(world, _free_port(), total_slabs, T, d, out_path), nprocs=world, join=True)
    got = np.load(out_path)
    rng = np.random.default_rng(0)
    q, k, v = (rng.standard_normal((total_slabs, T, d)).astype(np.float32) for _ in range(3))
    want, _, _ = orc.attention_forward(q, k, v, 1 / math.sqrt(d))
    assert np.array_equal(got["full"], want.astype(np.float32))
    assert float(got["slowest"]) == 11.0 and float(got["total"]) == total_slabs
