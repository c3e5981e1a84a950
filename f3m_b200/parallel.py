"""Multi-GPU product: one process per GPU, torch.distributed for the plumbing.

The reference's multi-GPU mode is one independent process per block of K with no communication
(par_FFM_block, experiments/FFM_classes.py:128-211; experiment_utils/scalability_analysis.sh).  Here
every rank holds a shard of the points and of b:

  1. all-gather the shards of X and b (NCCL over NVLink): every rank holds all sources;
  2. every rank builds the same tree and interaction lists (cheap next to the sums);
  3. the boxes are split into contiguous slices of the sorted order, one per rank; each rank computes
     the finest-level moments of its slice of the SOURCE boxes (f3m_plan_moments_range), the moment
     arrays are summed with an all-reduce, and each rank computes the far and near field of its slice
     of the TARGET boxes (f3m_plan_apply_range_moments);
  4. the slices are combined with an all-reduce, so every rank ends with the whole product
     (rows outside a rank's slice are zero before the sum).
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch
import torch.distributed as dist


def shard_bounds(n: int, world: int) -> List[int]:
    """Row boundaries of an even split: rank r owns [bounds[r], bounds[r+1])."""
    return [r * n // world for r in range(world + 1)]


def gather_shards(x_shard: torch.Tensor, counts: List[int], group=None) -> torch.Tensor:
    """All-gather row shards into one (sum(counts), cols) tensor.  Equal shards are gathered in place;
    unequal ones are padded to the longest shard first (collectives want equal sizes)."""
    x_shard = x_shard.contiguous()
    if len(set(counts)) == 1:
        full = torch.empty(sum(counts), *x_shard.shape[1:], dtype=x_shard.dtype, device=x_shard.device)
        dist.all_gather(list(full.split(counts)), x_shard, group=group)
        return full
    mx = max(counts)
    padded = torch.zeros(mx, *x_shard.shape[1:], dtype=x_shard.dtype, device=x_shard.device)
    padded[:x_shard.shape[0]] = x_shard
    buf = torch.empty(len(counts), mx, *x_shard.shape[1:], dtype=x_shard.dtype, device=x_shard.device)
    dist.all_gather(list(buf.unbind(0)), padded, group=group)
    return torch.cat([buf[r, :c] for r, c in enumerate(counts)], 0)


def distributed_kmvm(x_shard: torch.Tensor, b_shard: torch.Tensor, params, group=None,
                     compute: Optional[Callable] = None) -> torch.Tensor:
    """K(X, X) b with X and b sharded by rows over the ranks of `group`; returns the full (N, R) product
    on every rank.  `compute(X, b, lo, hi)` must return an (N, R) tensor holding the rows of the slice
    [lo, hi) of its own ordering and zeros elsewhere; the default runs the CUDA engine."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    n_local = torch.tensor([x_shard.shape[0]], device=x_shard.device, dtype=torch.int64)
    all_n = [torch.zeros_like(n_local) for _ in range(world)]
    dist.all_gather(all_n, n_local, group=group)
    counts = [int(t.item()) for t in all_n]
    N = sum(counts)
    X = gather_shards(x_shard, counts, group)
    b = gather_shards(b_shard, counts, group)
    bounds = shard_bounds(N, world)
    lo, hi = bounds[rank], bounds[rank + 1]
    if compute is None:
        from . import engine
        plan = engine.Plan(X, None, params)
        if plan.moments_size(b.shape[1]) > 0:
            # each rank interpolates the sources of its own slice onto the finest-level nodes; the moment
            # arrays (zero outside the slice) are summed over NVLink, so nobody passes over all sources
            mom = plan.moments(b, (lo, hi))
            dist.all_reduce(mom, group=group)
            out = plan.apply(b, row_range=(lo, hi), moments=mom)
        else:
            out = plan.apply(b, row_range=(lo, hi))
        plan.close()
    else:
        out = compute(X, b, lo, hi)
    dist.all_reduce(out, group=group)
    return out
