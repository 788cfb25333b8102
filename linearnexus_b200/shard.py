"""Sharding of the (batch x head) units of a delta-rule call over the ranks of one node.

Every op of this package is independent across (batch, head) pairs, so a multi-GPU run is one
process per GPU, each working on a contiguous block of batch rows (or of flattened batch*head
units when there are fewer batch rows than ranks), with no collective on the data path.
``torch.distributed`` is used only to put results together for checking and reporting.
"""

from __future__ import annotations

from typing import List, Tuple

import torch


def unit_range(n_units: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous [lo, hi) block of ``n_units`` for ``rank``; block sizes differ by at most one."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(n_units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_inputs(tensors: dict, world: int, rank: int) -> Tuple[dict, str]:
    """Slice every tensor of ``tensors`` ([B,H,...] each, None allowed) for ``rank``.

    Shards the batch axis when B >= world, otherwise flattens (B,H) -> (B*H, 1) units first (the
    case of KDA B=4 on 8 GPUs).  Returns the shard and the axis mode ("batch" or "unit")."""
    some = next(t for t in tensors.values() if t is not None)
    B, H = some.shape[0], some.shape[1]
    if B >= world:
        lo, hi = unit_range(B, world, rank)
        return {k: (None if t is None else t[lo:hi]) for k, t in tensors.items()}, "batch"
    lo, hi = unit_range(B * H, world, rank)
    out = {}
    for k, t in tensors.items():
        out[k] = None if t is None else t.reshape(B * H, 1, *t.shape[2:])[lo:hi]
    return out, "unit"


def gather_outputs(local: torch.Tensor, sizes: List[int]) -> torch.Tensor:
    """all_gather shards of different leading size (``sizes[r]`` rows on rank r) and concatenate them."""
    import torch.distributed as dist
    world = dist.get_world_size()
    pad = max(sizes)
    buf = local.new_zeros((pad,) + tuple(local.shape[1:]))
    buf[: local.shape[0]] = local
    parts = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(parts, buf)
    return torch.cat([p[:n] for p, n in zip(parts, sizes)], dim=0)
