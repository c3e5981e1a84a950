"""Multi-GPU product: one process per GPU, torch.distributed for the plumbing.

The reference's multi-GPU mode is one independent process per block of K with no communication
(par_FFM_block, experiments/FFM_classes.py:128-211; experiment_utils/scalability_analysis.sh).  Here every rank
holds a shard of the points and of b and gets back the rows of the product that belong to its shard:

  1. every rank sorts its own shard of the points inside the global bounding cube; the sorted runs are all-gathered
     (NCCL over NVLink) and merged, cell by cell, into the same sorted arrays on every rank; the all-gather of b runs
     meanwhile (strongly clustered sets, whose tree goes deeper than the shards are sorted: all-gather of the points
     and a sort on every rank);
  2. every rank builds the same levels and interaction lists (about two milliseconds);
  3. the sorted target rows are cut into one slice per rank of equal estimated work (f3m_plan_partition_rows);
  4. each rank interpolates an equal share of the source boxes onto the finest-level nodes; the moment slices are
     all-gathered while the rank computes the direct sums of its slice (it packs only the source boxes its own
     lists name: its slice plus a halo);
  5. far field of the slice from the gathered moments; nothing but the rank's own rows is written;
  6. all-to-all: every computed row goes to the rank that owns its input row, which puts it in input order.

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


_UNEVEN_ALL_GATHER = {"ok": None}   # does this backend's all_gather take pieces of different lengths?


def _gather_slices_in_place(acc: torch.Tensor, bounds: List[int], rank: int, group):
    """Every rank's slice acc[bounds[r]:bounds[r+1]] to every rank.  On CUDA tensors the list form of all_gather takes
    the slices as they lie in acc (NCCL: one grouped broadcast per rank, no staging copy); backends that want equal
    pieces get the padded form."""
    world = len(bounds) - 1
    mine = acc[bounds[rank]:bounds[rank + 1]]
    if acc.is_cuda and _UNEVEN_ALL_GATHER["ok"] is not False:
        try:
            dist.all_gather([acc[bounds[r]:bounds[r + 1]] for r in range(world)], mine, group=group)
            _UNEVEN_ALL_GATHER["ok"] = True
            return acc
        except (RuntimeError, ValueError):   # raised at argument checking, on every rank alike
            if _UNEVEN_ALL_GATHER["ok"]:
                raise
            _UNEVEN_ALL_GATHER["ok"] = False
    return gather_shards(mine, [bounds[r + 1] - bounds[r] for r in range(world)], group)


def gather_runs(t_shard: torch.Tensor, counts: List[int], group=None, async_op: bool = False):
    """All-gather row shards WITHOUT closing the gaps: rank r's rows start at row r * max(counts) of the result.
    Returns (buffer, stride) -- with async_op a function that waits and returns them."""
    mx = max(counts)
    t_shard = t_shard.contiguous()
    if t_shard.shape[0] != mx:
        padded = torch.zeros(mx, *t_shard.shape[1:], dtype=t_shard.dtype, device=t_shard.device)
        padded[:t_shard.shape[0]] = t_shard
        t_shard = padded
    buf = torch.empty(len(counts) * mx, *t_shard.shape[1:], dtype=t_shard.dtype, device=t_shard.device)
    work = _all_gather_equal(buf, t_shard, group, async_op)

    def finish():
        work.wait()
        return buf, mx
    return finish if async_op else (buf, mx)


_TOO_DEEP = set()   # (N, d, min_points) of point sets whose tree went deeper than the shards are sorted: skip the attempt


class EngineBackend:
    """The CUDA engine behind the phases of distributed_kmvm (a test may pass a stand-in with the same methods)."""

    def plan(self, X: torch.Tensor, params):
        from . import engine
        return engine.Plan(X, None, params)

    def bounding_box(self, x_shard: torch.Tensor):
        from . import engine
        return engine.bounding_box(x_shard)

    def plan_from_shards(self, x_shard: torch.Tensor, counts: List[int], rank: int, params, group, origin, top, clock=None):
        """The plan of all points with the sort shared by the ranks: inside the global bounding cube (origin, top: the
        per-dimension extremes over all ranks) every rank sorts its shard, levels and lists are built from the gathered
        cell counts while the sorted runs travel, and the runs are merged in.  None when that form does not apply (the
        level loop would need more levels than the shards were sorted to): the caller gathers the points instead."""
        import numpy as np
        from . import engine
        from ._lib import F3MError
        dev, d, N = x_shard.device, x_shard.shape[1], sum(counts)
        if min(counts) < 1 or (N, d, float(params.min_points)) in _TOO_DEEP:
            return None
        origin, top = np.asarray(origin, dtype=np.float32), np.asarray(top, dtype=np.float32)
        edge0 = float(np.float32((top - origin).max()) * np.float32(1.01))     # calculate_edge_X, float32
        if not (np.isfinite(edge0) and edge0 > 0):
            return None    # the single-GPU path reports degenerate or non-finite point sets
        depth = engine.sort_depth(N, d, params.min_points)
        if d * depth > 22:
            return None
        if clock:
            clock.mark("cube")
        recs, cells = engine.sort_shard(x_shard, sum(counts[:rank]), origin, edge0, params.math_mode, depth)
        if clock:
            clock.mark("sort_shard")
        cells_all = torch.empty(len(counts) * cells.shape[0], device=dev, dtype=torch.int32)
        _all_gather_equal(cells_all, cells, group, False)
        recs_wait = gather_runs(recs, counts, group, async_op=True)      # the records travel while the lists are built
        try:
            plan = engine.Plan.from_cell_counts(cells_all.view(len(counts), -1), d, origin, edge0, depth, params)
            if clock:
                clock.mark("levels_lists")
            recs_all, stride = recs_wait()
            plan.attach_runs(recs_all, stride)
            if clock:
                clock.mark("merge_runs")
            return plan
        except F3MError as e:
            recs_wait()
            if e.status == 5:     # F3M_ERR_UNSUPPORTED: deeper than the shards were sorted (the same on every rank)
                _TOO_DEEP.add((N, d, float(params.min_points)))
                return None
            raise


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
    # one small all-gather brings the shard sizes and, for the shared sort, the shards' bounding boxes
    d = x_shard.shape[1]
    use_shards = world > 1 and hasattr(backend, "plan_from_shards") and x_shard.shape[0] > 0
    head = [float(x_shard.shape[0])]
    if hasattr(backend, "plan_from_shards"):
        lo, hi = backend.bounding_box(x_shard) if x_shard.shape[0] > 0 else ([float("inf")] * d, [float("-inf")] * d)
        head += list(lo) + list(hi)
    mine = torch.tensor(head, device=dev, dtype=torch.float64)
    table = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(table, mine, group=group)
    table = torch.stack(table).cpu()
    counts = [int(v) for v in table[:, 0].tolist()]
    N = sum(counts)
    in_lo = sum(counts[:rank])
    in_hi = in_lo + counts[rank]
    R = b_shard.shape[1]

    b_wait = gather_shards(b_shard, counts, group, async_op=True)    # lands while the tree is built
    plan = X = None
    if use_shards and min(counts) > 0:
        origin = table[:, 1:1 + d].min(0).values.float().numpy()
        top = table[:, 1 + d:1 + 2 * d].max(0).values.float().numpy()
        plan = backend.plan_from_shards(x_shard, counts, rank, params, group, origin, top, clock)
    if plan is None:
        X = gather_shards(x_shard, counts, group)
        clock.mark("gather_points")
        plan = backend.plan(X, params)
    clock.mark("tree_lists")
    if dev.type == "cuda" and float(N) * (x_shard.shape[1] + R) * 4 > 4e9:
        # Very large sets: what was only needed to build the plan (the gathered points or runs in torch's pool, the
        # sort's buffers in the library's) goes back to the driver before the product's own arrays are sized.
        X = None
        if hasattr(plan, "X"):
            plan.X = plan.Y = None
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        from . import engine as _engine
        _engine.release_cached_memory()
    bounds = plan.partition_rows(R, world)
    if world > 1:
        # every rank computes the same cuts from the same plan; rank 0's copy is the one used, so that a difference
        # between the ranks could never leave a row without an owner
        cuts = torch.tensor(bounds, device=dev, dtype=torch.int64)
        dist.broadcast(cuts, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        bounds = [int(v) for v in cuts.tolist()]
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
    if world > 1 and R <= 2 and hasattr(plan, "gathered_rows_to_input_order"):
        # few columns: one all-gather of the slices (padded to the longest, left where they land), then every rank
        # picks the rows of its own shard -- NCCL's all-gather moves these few hundred megabytes faster than an
        # all-to-all moves an eighth of them
        gathered, stride = gather_runs(acc[rb:re], [bounds[r + 1] - bounds[r] for r in range(world)], group)
        clock.mark("exchange_rows")
        out = plan.gathered_rows_to_input_order(gathered, bounds, stride, in_lo, in_hi)
    elif world > 1:
        # all-to-all: every row of the slice goes to the rank that owns its input row, with the row number beside it
        in_bounds = [sum(counts[:r]) for r in range(world + 1)]
        send, send_counts = plan.rows_by_owner(acc, (rb, re), in_bounds)
        clock.mark("pack_rows")
        mine = torch.tensor(send_counts, device=dev, dtype=torch.int64)
        table = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(table, mine, group=group)
        recv_counts = torch.stack(table)[:, rank].tolist()
        assert sum(recv_counts) == in_hi - in_lo, "rows received do not add up to this rank's shard"
        recv = torch.empty(in_hi - in_lo, R + 1, device=dev, dtype=torch.float32)
        dist.all_to_all_single(recv, send, output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
        clock.mark("exchange_rows")
        out = plan.place_rows(recv, in_lo, in_hi)
    else:
        clock.mark("exchange_rows")
        out = plan.rows_to_input_order(acc, in_lo, in_hi)
    clock.mark("own_rows")
    if stats is not None:
        stats["slice_rows"] = re - rb
        if hasattr(plan, "timings"):
            stats["engine_ms"] = plan.timings()
    plan.close()
    clock.finish()
    return out
