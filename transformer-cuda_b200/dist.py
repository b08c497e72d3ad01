"""Process-level plumbing for running the (batch, head)-sharded path on several GPUs of one box:
rank discovery from the torchrun environment, the barrier + max-over-ranks timing reduction the
benchmark uses, and a gather of per-shard results for tests. The attention path itself exchanges
nothing between ranks; the only collectives here carry timings and test data."""
import os

import torch
import torch.distributed as dist

from .shard import slab_range


def env_rank_world():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def init(backend=None):
    """Join the process group described by RANK / WORLD_SIZE / MASTER_* (no-op for a single process)."""
    rank, world, local = env_rank_world()
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kwargs = {}
        if backend == "nccl":
            kwargs["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kwargs)
    return rank, world, local


def barrier():
    if dist.is_initialized():
        dist.barrier()


def max_over_ranks(value: float, device="cpu") -> float:
    """The slowest rank's value: multi-GPU times are reported as the maximum over ranks."""
    if not dist.is_initialized():
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, device="cpu") -> float:
    if not dist.is_initialized():
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def my_slabs(total_slabs: int):
    rank, world, _ = env_rank_world()
    if dist.is_initialized():
        rank, world = dist.get_rank(), dist.get_world_size()
    return slab_range(total_slabs, rank, world)


def gather_slabs(local: torch.Tensor, total_slabs: int) -> torch.Tensor:
    """Concatenate per-rank (count_r, ...) tensors into the full (total_slabs, ...) tensor on every rank."""
    if not dist.is_initialized():
        return local
    world = dist.get_world_size()
    tail = tuple(local.shape[1:])
    counts = [slab_range(total_slabs, r, world).count for r in range(world)]
    width = max(counts)  # all_gather wants equal shapes: pad every shard to the largest one
    padded = torch.zeros((width,) + tail, dtype=local.dtype, device=local.device)
    padded[: local.shape[0]] = local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded)
    return torch.cat([p[:c] for p, c in zip(parts, counts)], dim=0)


def average_gradients_(flat_grads: torch.Tensor) -> torch.Tensor:
    """The gradient exchange of the data-parallel training step (config 4), in place on one flat buffer: sum over
    ranks, then multiply by 1/world (what ncclAllReduce(avg) does in transformer-cuda_b200/harness/gpt_step_dp.cu).
    It runs once per step on the finished buffer, before the optimizer: the reference's fused_step computes the
    global gradient norm and clears the buffer (src/optimizer.cu:225-249), so every rank must see the averaged
    gradient first. Every rank then applies the identical update and the replicas stay bit-identical."""
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(flat_grads, op=dist.ReduceOp.SUM)
        flat_grads.mul_(1.0 / dist.get_world_size())
    return flat_grads



def gradient_parts(num_layers: int, per_layer: int, embeddings: int, tail: int):
    """The order in which the parts of the flat gradient buffer [embeddings | layer 0 ... layer L-1 | final LayerNorm +
    head] become final during the reference model's backward pass (src/model.cu:431-704), as (offset, count) pairs:
    the tail first (after the final LayerNorm's backward), then the layers from the last to the first (after each
    layer's LN1 backward), the embeddings last. transformer-cuda_b200/harness/gpt_step_dp.cu all-reduces them in this
    order on a second stream while the pass still runs; every rank must use the same order."""
    total = embeddings + num_layers * per_layer + tail
    parts = [(total - tail, tail)]
    for layer in range(num_layers - 1, -1, -1):
        parts.append((embeddings + layer * per_layer, per_layer))
    parts.append((0, embeddings))
    return [(o, c) for o, c in parts if c > 0]


def average_gradients_in_parts_(flat_grads: torch.Tensor, parts) -> torch.Tensor:
    """average_gradients_ issued part by part (the harness's overlapped form): the same result, as long as the parts
    tile the buffer exactly once."""
    covered = sorted(parts)
    if sum(c for _, c in covered) != flat_grads.numel() or any(covered[i][0] + covered[i][1] != covered[i + 1][0]
                                                                for i in range(len(covered) - 1)) or covered[0][0] != 0:
        raise ValueError("the parts must tile the gradient buffer exactly once")
    if dist.is_initialized() and dist.get_world_size() > 1:
        for offset, count in parts:
            piece = flat_grads[offset:offset + count]
            dist.all_reduce(piece, op=dist.ReduceOp.SUM)
            piece.mul_(1.0 / dist.get_world_size())
    return flat_grads
