"""Sharding a cache over the GPUs of one box, and the only communication the codec needs.

Every vector (per-vector methods) and every (segment, token group) (per-channel keys) is
independent, so the cache splits by layer, or by (layer, KV head), with no exchange step:
each rank encodes and decodes its own segments in its own memory.  The one collective is an
all-gather of a few 64-bit verification checksums and timings after the work is done
(NCCL between GPUs; gloo works the same for CPU ranks in tests).
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Shard:
    rank: int
    world: int
    first_segment: int     # index into the layer-major list of (layer, kv_head) segments
    segments: int

    @property
    def segment_range(self) -> range:
        return range(self.first_segment, self.first_segment + self.segments)


def shard_segments(layers: int, kv_heads: int, world: int, rank: int, by: str = "layer") -> Shard:
    """Contiguous block of segments for ``rank``.  ``by="layer"`` keeps the KV heads of a layer
    together (layers must divide evenly: 24 layers -> 24/12/6/3 per rank at 1/2/4/8);
    ``by="segment"`` splits the layers x kv_heads list itself (640 -> 80 per rank at 8), giving the
    first ``total % world`` ranks one extra segment when it does not divide."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} is outside a world of {world}")
    if by == "layer":
        if layers % world:
            raise ValueError(f"{layers} layers do not divide over {world} ranks")
        per = layers // world
        return Shard(rank, world, rank * per * kv_heads, per * kv_heads)
    if by == "segment":
        total = layers * kv_heads
        base, extra = divmod(total, world)
        first = rank * base + min(rank, extra)
        return Shard(rank, world, first, base + (1 if rank < extra else 0))
    raise ValueError(f"unknown sharding {by!r}")


def gather_int64(values, device=None, group=None):
    """All-gathers a short list of 64-bit integers (checksums, counters, microseconds) from every
    rank; returns ``world`` lists.  Unsigned values are carried as their two's-complement bit
    patterns.  Without an initialised process group it returns ``[values]``."""
    import torch
    import torch.distributed as dist
    vals = [int(v) & 0xFFFFFFFFFFFFFFFF for v in values]
    if not (dist.is_available() and dist.is_initialized()):
        return [vals]
    signed = [v - (1 << 64) if v >= (1 << 63) else v for v in vals]
    if device is None:
        device = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    mine = torch.tensor(signed, dtype=torch.int64, device=device)
    out = [torch.empty_like(mine) for _ in range(dist.get_world_size(group))]
    dist.all_gather(out, mine, group=group)
    return [[int(v) & 0xFFFFFFFFFFFFFFFF for v in t.cpu().tolist()] for t in out]
