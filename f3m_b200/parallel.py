"""Multi-GPU product: one process per GPU, torch.distributed for the plumbing.

The reference's multi-GPU mode is one independent process per block of K with no communication
(par_FFM_block, experiments/FFM_classes.py:128-211; experiment_utils/scalability_analysis.sh).  Here every rank
holds a shard of the points and of b and gets back the rows of the product that belong to its shard:

  1. all-gather the shards of X (NCCL over NVLink); the all-gather of b runs while the tree is built;
  2. every rank builds the same tree and interaction lists (a few milliseconds next to the sums);
  3. the sorted target rows are cut into one slice per rank of equal estimated work (f3m_plan_partition_rows);
  4. each rank interpolates an equal share of the source boxes onto the finest-level nodes; the moment slices are
     all-gathered while the rank computes the direct sums of its slice (it packs only the source boxes its own
     lists name: its slice plus a halo);
  5. far field of the slice from the gathered moments; nothing but the rank's own rows is written;
  6. the sorted slices are all-gathered and each rank takes the rows of its own shard, in input order.

No kernel reads another GPU's memory: remote data always lands in local HBM through NCCL first.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist


def shard_bounds(n: int, world: int) -> List[int]:
    """Row boundaries of an even split: rank r owns [bounds[r], bounds[r+1])."""
    return [r * n // world for r in range(world + 1)]


def _all_gather_equal(full: torch.Tensor, piece: torch.Tensor, group, async_op: bool):
    """All-gather of equal pieces into `full` (piece r at rows [r m, (r+1) m)); `piece` may be full's own part.  On
    CUDA tensors this is one flat NCCL all-gather without staging copies; elsewhere the list form."""
    if full.is_cuda:
        return dist.all_gather_into_tensor(full, piece, group=group, async_op=async_op)
    return dist.all_gather(list(full.split(piece.shape[0])), piece, group=group, async_op=async_op)


def gather_shards(x_shard: torch.Tensor, counts: List[int], group=None, async_op: bool = False):
    """All-gather row shards into one (sum(counts), cols) tensor.  Equal shards are gathered in place;
    unequal ones are padded to the longest shard first (collectives want equal sizes).  With async_op the
    result is a function that waits for the collective and returns the tensor."""
    x_shard = x_shard.contiguous()
    if len(set(counts)) == 1:
        full = torch.empty(sum(counts), *x_shard.shape[1:], dtype=x_shard.dtype, device=x_shard.device)
        work = _all_gather_equal(full, x_shard, group, async_op)

        def finish_even():
            work.wait()
            return full
        return finish_even if async_op else full
    mx = max(counts)
    padded = torch.zeros(mx, *x_shard.shape[1:], dtype=x_shard.dtype, device=x_shard.device)
    padded[:x_shard.shape[0]] = x_shard
    buf = torch.empty(len(counts), mx, *x_shard.shape[1:], dtype=x_shard.dtype, device=x_shard.device)
    work = _all_gather_equal(buf.view(len(counts) * mx, *x_shard.shape[1:]), padded, group, async_op)

    def finish():
        if async_op:
            work.wait()
        return torch.cat([buf[r, :c] for r, c in enumerate(counts)], 0)
    return finish if async_op else finish()


class EngineBackend:
    """The CUDA engine behind the phases of distributed_kmvm (a test may pass a stand-in with the same methods)."""

    def plan(self, X: torch.Tensor, params):
        from . import engine
        return engine.Plan(X, None, params)


class _Clock:
    """Device time between marks on the current CUDA stream (nothing on CPU tensors)."""

    def __init__(self, device, stats: Optional[Dict]):
        self.on = stats is not None and device.type == "cuda"
        self.stats, self.marks = stats, []
        self.mark("start")

    def mark(self, name):
        if self.on:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.marks.append((name, ev))

    def finish(self):
        if not self.on:
            return
        torch.cuda.synchronize()
        for (_, a), (name, b) in zip(self.marks[:-1], self.marks[1:]):
            self.stats[name] = self.stats.get(name, 0.0) + a.elapsed_time(b)


def distributed_kmvm(x_shard: torch.Tensor, b_shard: torch.Tensor, params, group=None, backend=None,
                     stats: Optional[Dict] = None) -> torch.Tensor:
    """K(X, X) b with X and b sharded by rows over the ranks of `group`: returns the (n_local, R) rows of the
    product that belong to this rank's shard.  `stats` (a dict) receives the device milliseconds of the phases."""
    backend = backend or EngineBackend()
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    dev = x_shard.device
    clock = _Clock(dev, stats)
    if b_shard.dim() == 1:
        b_shard = b_shard[:, None]
    n_local = torch.tensor([x_shard.shape[0]], device=dev, dtype=torch.int64)
    all_n = [torch.zeros_like(n_local) for _ in range(world)]
    dist.all_gather(all_n, n_local, group=group)
    counts = [int(t.item()) for t in all_n]
    N = sum(counts)
    in_lo = sum(counts[:rank])
    in_hi = in_lo + counts[rank]
    R = b_shard.shape[1]

    X = gather_shards(x_shard, counts, group)
    b_wait = gather_shards(b_shard, counts, group, async_op=True)    # lands while the tree is built
    clock.mark("gather_points")
    plan = backend.plan(X, params)
    clock.mark("tree_lists")
    bounds = plan.partition_rows(R, world)
    rb, re = bounds[rank], bounds[rank + 1]
    msize = plan.moments_size(R)
    _, nby = plan.finest_boxes()
    exchange = msize > 0 and world > 1
    mom_full = mom_slice = None
    box_range = (0, 0)
    if exchange:
        per_box = msize // nby
        cb = -(-nby // world)                                      # source boxes per rank, the last share may be short
        mom_full = torch.empty(world * cb * per_box, device=dev, dtype=torch.float32)
        mom_slice = mom_full[rank * cb * per_box:(rank + 1) * cb * per_box]
        box_range = (min(nby, rank * cb), min(nby, (rank + 1) * cb))
    b = b_wait()
    clock.mark("partition")
    plan.shard_begin(b, (rb, re), box_range, mom_slice)
    clock.mark("sources_moments")
    mom_work = None
    if exchange:
        # every rank's slice sits at its own place of mom_full: an in-place all-gather, overlapped with the direct sums
        mom_work = _all_gather_equal(mom_full, mom_slice, group, True)
    acc = torch.empty(N, R, device=dev, dtype=torch.float32)        # sorted row order; this rank fills [rb, re)
    plan.shard_near(acc)
    clock.mark("direct_sums")
    if mom_work is not None:
        mom_work.wait()
    plan.shard_far(mom_full, acc)
    plan.shard_end()
    clock.mark("far_field")
    if world > 1:
        acc = gather_shards(acc[rb:re], [bounds[r + 1] - bounds[r] for r in range(world)], group)
    clock.mark("gather_result")
    out = plan.rows_to_input_order(acc, in_lo, in_hi)
    clock.mark("own_rows")
    if stats is not None:
        stats["slice_rows"] = re - rb
        if hasattr(plan, "timings"):
            stats["engine_ms"] = plan.timings()
    plan.close()
    clock.finish()
    return out
