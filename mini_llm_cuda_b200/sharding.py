"""Host-side sharding of independent sequences over the GPUs of one box.

Decode has no cross-sequence dependency: every GPU holds a full weight replica and its own
slice of the sequences (their KV pages and delta-net state), so the token path needs no
collective. torch.distributed is used only around it: a barrier before timing, the max of the
per-rank device times, and a gather of the generated ids to rank 0. The reference has no
multi-GPU code at all (it never calls cudaSetDevice)."""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np


def shard_range(n_items: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous block of items for `rank`; the first n_items % world ranks get one more."""
    if world < 1 or not (0 <= rank < world) or n_items < 0:
        raise ValueError("bad shard arguments")
    base, extra = divmod(n_items, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def max_over_ranks(value: float, device=None) -> float:
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_tokens(local: np.ndarray, n_total: int, device=None) -> Optional[np.ndarray]:
    """local: int32 [n_local, T] ids of this rank's sequences (its shard_range of n_total).
    Returns [n_total, T] in sequence order on rank 0, None elsewhere."""
    import torch
    import torch.distributed as dist
    local = np.ascontiguousarray(local, dtype=np.int32)
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        assert local.shape[0] == n_total
        return local
    world, rank = dist.get_world_size(), dist.get_rank()
    T = local.shape[1]
    per = -(-n_total // world)                       # padded rows per rank
    pad = np.full((per, T), -1, dtype=np.int32)
    pad[:local.shape[0]] = local
    mine = torch.from_numpy(pad).to(device) if device is not None else torch.from_numpy(pad)
    parts = [torch.empty_like(mine) for _ in range(world)] if rank == 0 else None
    dist.gather(mine, parts, dst=0)
    if rank != 0:
        return None
    out = np.empty((n_total, T), dtype=np.int32)
    for r in range(world):
        a, b = shard_range(n_total, world, r)
        out[a:b] = parts[r].cpu().numpy()[:b - a]
    return out
