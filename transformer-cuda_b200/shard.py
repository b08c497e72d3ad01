"""(batch, head) partitioning of the attention path across the GPUs of one box.

Every (b, h) pair is an independent attention problem and, in the (B, H, T, d) layout, one contiguous
T*d slab (src/kernels/attention.cu:534-538 of the reference indexes slabs by `bh * T * d`). A shard is
therefore a contiguous range of slab indices and a pointer offset; ranks exchange nothing.
"""
from dataclasses import dataclass


@dataclass(frozen=True)
class SlabRange:
    start: int  # first (b*H + h) slab owned by the rank
    count: int  # number of slabs owned

    @property
    def stop(self):
        return self.start + self.count


def slab_range(total_slabs: int, rank: int, world_size: int) -> SlabRange:
    """Contiguous, balanced split of `total_slabs` = B*H over `world_size` ranks; the first
    `total_slabs % world_size` ranks get one extra slab. Ranks beyond the slab count get an empty range."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank/world_size {rank}/{world_size}")
    if total_slabs < 0:
        raise ValueError("total_slabs must be >= 0")
    base, extra = divmod(total_slabs, world_size)
    start = rank * base + min(rank, extra)
    return SlabRange(start, base + (1 if rank < extra else 0))


def element_offset(r: SlabRange, T: int, d: int) -> int:
    """Index of the shard's first element inside the full (B*H, T, d) tensor (also its offset in the
    counter-based random streams, so a shard reproduces its part of the 1-GPU tensor)."""
    return r.start * T * d
