"""Thin Python layer over the C ABI: plans, products, introspection.  torch supplies device
memory and the current stream; all arithmetic happens in libf3m.so."""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional

import numpy as np
import torch

from . import _lib
from ._lib import Params, LevelInfo, PlanStats, check


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _as_f32(t: torch.Tensor) -> torch.Tensor:
    if t.dtype != torch.float32 or not t.is_contiguous():
        t = t.float().contiguous()
    return t


def is_shared(X: torch.Tensor, Y: Optional[torch.Tensor]) -> bool:
    """True when Y is the same point set as X: no Y, or the same storage address AND the same shape.  The address
    alone is not enough: a leading slice X[:k] starts at X's address but is a different (smaller) point set."""
    return Y is None or (Y.data_ptr() == X.data_ptr() and tuple(Y.shape) == tuple(X.shape))


def _check_product_shapes(X, Y, b):
    if X.dim() != 2 or Y.dim() != 2 or Y.shape[1] != X.shape[1]:
        raise AssertionError(f"X {tuple(X.shape)} and Y {tuple(Y.shape)} must be (n, d) arrays of one dimension d")
    if b.shape[0] != Y.shape[0]:
        raise AssertionError(f"b has {b.shape[0]} rows, Y has {Y.shape[0]}")


def make_params(ls, min_points, nr_of_interpolation, var_compression, eff_var_limit, small_field_points,
                math_mode=_lib.MATH_FASTMATH, flags=0) -> Params:
    return Params(float(ls), float(min_points), int(nr_of_interpolation), int(bool(var_compression)),
                  float(eff_var_limit), int(small_field_points), int(math_mode), int(flags))


def bounding_box(X: torch.Tensor):
    """Per-dimension minimum and maximum of the points (two lists of d floats; f3m_bounding_box_f32)."""
    X = _as_f32(X)
    d = X.shape[1]
    lo, hi = (C.c_float * d)(), (C.c_float * d)()
    with torch.cuda.device(X.device):
        check(_lib.lib().f3m_bounding_box_f32(X.data_ptr(), X.shape[0], d, lo, hi, _stream_ptr(X.device)), "f3m_bounding_box_f32")
    return list(lo), list(hi)


def sort_depth(n_total: int, d: int, min_points: float) -> int:
    return int(_lib.lib().f3m_sort_depth(int(n_total), int(d), float(min_points)))


def sort_shard(X: torch.Tensor, row_offset: int, origin, edge0: float, math_mode: int, depth: int):
    """One rank's share of a sort done by several GPUs (f3m_sort_shard_f32): the sorted records (n, words) and the
    number of points in every cell of the sorted depth (2^(d depth) int32)."""
    X = _as_f32(X)
    n, d = X.shape
    words = int(_lib.lib().f3m_record_words(d))
    recs = torch.empty(n, words, device=X.device, dtype=torch.int32)
    cells = torch.empty(1 << (d * depth), device=X.device, dtype=torch.int32)
    org = (C.c_float * d)(*[float(v) for v in origin])
    with torch.cuda.device(X.device):
        check(_lib.lib().f3m_sort_shard_f32(X.data_ptr(), n, int(row_offset), d, org, C.c_float(edge0), int(math_mode), int(depth),
                                            recs.data_ptr(), cells.data_ptr(), _stream_ptr(X.device)), "f3m_sort_shard_f32")
    return recs, cells


class Plan:
    """Tree and interaction lists of one (X, Y) pair (f3m_plan); apply() multiplies by any b."""

    @classmethod
    def from_cell_counts(cls, cell_counts: torch.Tensor, d: int, origin, edge0: float, depth: int, params: Params) -> "Plan":
        """Levels and lists of all points (Y = X) from the cell counts of runs sorted on several GPUs, row r = run r
        (f3m_plan_create_from_cell_counts).  attach_runs() must follow before any product."""
        self = cls.__new__(cls)
        self.X = self.Y = None
        self.same = True
        self.params = params
        self.device = cell_counts.device
        self.d = d
        self._h = C.c_void_p()
        cell_counts = cell_counts.contiguous()
        org = (C.c_float * d)(*[float(v) for v in origin])
        with torch.cuda.device(self.device):
            st = _lib.lib().f3m_plan_create_from_cell_counts(C.byref(self._h), cell_counts.data_ptr(), cell_counts.shape[0], d, org,
                                                             C.c_float(edge0), int(depth), C.byref(params), _stream_ptr(self.device))
        check(st, "f3m_plan_create_from_cell_counts")
        self.N = self.M = int(cell_counts.sum().item())
        return self

    def attach_runs(self, recs: torch.Tensor, run_stride: int):
        """The gathered sorted runs (run r at record r * run_stride) are merged into the plan (f3m_plan_attach_runs)."""
        with torch.cuda.device(self.device):
            check(_lib.lib().f3m_plan_attach_runs(self._h, recs.data_ptr(), int(run_stride), _stream_ptr(self.device)),
                  "f3m_plan_attach_runs")

    def __init__(self, X: torch.Tensor, Y: Optional[torch.Tensor], params: Params):
        if not X.is_cuda:
            raise ValueError("Plan needs CUDA tensors: the engine has no CPU path")
        self.X = _as_f32(X)
        self.same = is_shared(X, Y)
        self.Y = self.X if self.same else _as_f32(Y)
        if self.Y.dim() != 2 or self.X.dim() != 2 or self.Y.shape[1] != self.X.shape[1]:
            raise AssertionError(f"X {tuple(X.shape)} and Y {tuple(self.Y.shape)} must be (n, d) arrays of one dimension d")
        if self.Y.device != self.X.device:
            raise ValueError("X and Y must be on the same device")
        self.params = params
        self.device = self.X.device
        self.N, self.d = self.X.shape
        self.M = self.Y.shape[0]
        self._h = C.c_void_p()
        with torch.cuda.device(self.device):
            st = _lib.lib().f3m_plan_create(C.byref(self._h), self.X.data_ptr(), self.N, self.Y.data_ptr(), self.M,
                                            self.d, C.byref(self.params), _stream_ptr(self.device))
        check(st, "f3m_plan_create")

    def moments_size(self, R: int) -> int:
        """Floats of the finest-level moment array if this plan can exchange moments between ranks, else 0."""
        n = C.c_int64()
        check(_lib.lib().f3m_plan_moments_size(self._h, int(R), C.byref(n)), "f3m_plan_moments_size")
        return int(n.value)

    def moments(self, b: torch.Tensor, src_range) -> torch.Tensor:
        """Finest-level moments of the source boxes starting inside src_range of the sorted order (zero elsewhere)."""
        b = _as_f32(b.to(self.device))
        if b.dim() == 1:
            b = b[:, None]
        if b.shape[0] != self.M:
            raise AssertionError(f"b has {b.shape[0]} rows, Y has {self.M}")
        mom = torch.empty(self.moments_size(b.shape[1]), device=self.device, dtype=torch.float32)
        with torch.cuda.device(self.device):
            st = _lib.lib().f3m_plan_moments_range(self._h, b.data_ptr(), b.shape[1], int(src_range[0]), int(src_range[1]),
                                                   mom.data_ptr(), _stream_ptr(self.device))
        check(st, "f3m_plan_moments_range")
        return mom

    def apply(self, b: torch.Tensor, row_range=None, moments: Optional[torch.Tensor] = None) -> torch.Tensor:
        b = _as_f32(b.to(self.device))
        if b.dim() == 1:
            b = b[:, None]
        if b.shape[0] != self.M:
            raise AssertionError(f"b has {b.shape[0]} rows, Y has {self.M}")
        out = torch.empty(self.N, b.shape[1], device=self.device, dtype=torch.float32)
        with torch.cuda.device(self.device):
            if moments is not None:
                if (not moments.is_cuda or moments.dtype != torch.float32 or not moments.is_contiguous()
                        or moments.numel() != self.moments_size(b.shape[1])):
                    raise ValueError("moments must be the contiguous float32 CUDA array of moments_size(R) floats that moments() returns")
                rr = (0, self.N) if row_range is None else row_range
                st = _lib.lib().f3m_plan_apply_range_moments(self._h, b.data_ptr(), b.shape[1], out.data_ptr(), int(rr[0]),
                                                             int(rr[1]), moments.data_ptr(), _stream_ptr(self.device))
            elif row_range is None:
                st = _lib.lib().f3m_plan_apply(self._h, b.data_ptr(), b.shape[1], out.data_ptr(), _stream_ptr(self.device))
            else:
                st = _lib.lib().f3m_plan_apply_range(self._h, b.data_ptr(), b.shape[1], out.data_ptr(), int(row_range[0]),
                                                     int(row_range[1]), _stream_ptr(self.device))
        check(st, "f3m_plan_apply")
        return out

    # ---- one product shared by several GPUs, in phases (see include/f3m.h) --------------------
    def partition_rows(self, R: int, nparts: int):
        """Cuts of the sorted target rows into nparts slices of equal estimated work (list of nparts + 1 ints)."""
        bounds = (C.c_int64 * (nparts + 1))()
        with torch.cuda.device(self.device):
            check(_lib.lib().f3m_plan_partition_rows(self._h, int(R), int(nparts), bounds, _stream_ptr(self.device)),
                  "f3m_plan_partition_rows")
        return [int(v) for v in bounds]

    def shard_begin(self, b: torch.Tensor, row_range, box_range=None, mom_slice: Optional[torch.Tensor] = None):
        b = _as_f32(b)
        if b.dim() == 1:
            b = b[:, None]
        if b.shape[0] != self.M or not b.is_cuda:
            raise AssertionError(f"b must be a CUDA tensor with {self.M} rows")
        self._shard_b = b      # kept alive until shard_end
        box_range = (0, 0) if box_range is None else box_range
        with torch.cuda.device(self.device):
            st = _lib.lib().f3m_plan_shard_begin(self._h, b.data_ptr(), b.shape[1], int(row_range[0]), int(row_range[1]),
                                                 int(box_range[0]), int(box_range[1]),
                                                 None if mom_slice is None else mom_slice.data_ptr(), _stream_ptr(self.device))
        check(st, "f3m_plan_shard_begin")

    def shard_near(self, acc_sorted: torch.Tensor):
        with torch.cuda.device(self.device):
            check(_lib.lib().f3m_plan_shard_near(self._h, acc_sorted.data_ptr(), _stream_ptr(self.device)), "f3m_plan_shard_near")

    def shard_far(self, mom: Optional[torch.Tensor], acc_sorted: torch.Tensor):
        with torch.cuda.device(self.device):
            check(_lib.lib().f3m_plan_shard_far(self._h, None if mom is None else mom.data_ptr(), acc_sorted.data_ptr(),
                                                _stream_ptr(self.device)), "f3m_plan_shard_far")

    def shard_end(self):
        check(_lib.lib().f3m_plan_shard_end(self._h), "f3m_plan_shard_end")
        self._shard_b = None

    def rows_to_input_order(self, acc_sorted: torch.Tensor, in_lo: int, in_hi: int) -> torch.Tensor:
        """Rows in_lo..in_hi of the product in input order, taken from the sorted result acc_sorted (N, R)."""
        R = acc_sorted.shape[1]
        out = torch.empty(in_hi - in_lo, R, device=self.device, dtype=torch.float32)
        with torch.cuda.device(self.device):
            check(_lib.lib().f3m_plan_rows_to_input_order(self._h, acc_sorted.data_ptr(), R, int(in_lo), int(in_hi), out.data_ptr(),
                                                          _stream_ptr(self.device)), "f3m_plan_rows_to_input_order")
        return out

    def gathered_rows_to_input_order(self, gathered: torch.Tensor, slice_bounds, stride: int, in_lo: int, in_hi: int) -> torch.Tensor:
        """Rows in_lo..in_hi of the product in input order from the all-gathered slices (slice g at row g * stride)."""
        R = gathered.shape[1]
        nr = len(slice_bounds) - 1
        cuts = (C.c_int64 * (nr + 1))(*[int(v) for v in slice_bounds])
        out = torch.empty(in_hi - in_lo, R, device=self.device, dtype=torch.float32)
        with torch.cuda.device(self.device):
            check(_lib.lib().f3m_plan_gathered_rows_to_input_order(self._h, gathered.data_ptr(), R, cuts, nr, int(stride), int(in_lo),
                                                                   int(in_hi), out.data_ptr(), _stream_ptr(self.device)),
                  "f3m_plan_gathered_rows_to_input_order")
        return out

    def rows_by_owner(self, acc_sorted: torch.Tensor, row_range, in_bounds):
        """The rows [row_range) of the sorted result as records [values, input row] grouped by the rank that owns the
        input row (rank g owns input rows in_bounds[g]..in_bounds[g+1]): (send buffer (rows, R + 1), counts per rank)."""
        nr = len(in_bounds) - 1
        R = acc_sorted.shape[1]
        cuts = (C.c_int64 * (nr + 1))(*[int(v) for v in in_bounds])
        counts = (C.c_int64 * nr)()
        rb, re = int(row_range[0]), int(row_range[1])
        with torch.cuda.device(self.device):
            check(_lib.lib().f3m_plan_count_rows_by_owner(self._h, rb, re, cuts, nr, counts, _stream_ptr(self.device)),
                  "f3m_plan_count_rows_by_owner")
            send = torch.empty(re - rb, R + 1, device=self.device, dtype=torch.float32)
            if re > rb:
                check(_lib.lib().f3m_plan_pack_rows_by_owner(self._h, acc_sorted.data_ptr(), R, rb, re, cuts, nr, counts, send.data_ptr(),
                                                             _stream_ptr(self.device)), "f3m_plan_pack_rows_by_owner")
        return send, [int(v) for v in counts]

    def place_rows(self, records: torch.Tensor, in_lo: int, in_hi: int) -> torch.Tensor:
        """Received records [values, input row] -> the rows in_lo..in_hi of the product in input order."""
        R = records.shape[1] - 1
        out = torch.empty(in_hi - in_lo, R, device=self.device, dtype=torch.float32)
        if records.shape[0] == 0:
            return out
        with torch.cuda.device(self.device):
            check(_lib.lib().f3m_plan_place_rows(self._h, records.data_ptr(), records.shape[0], R, int(in_lo), int(in_hi), out.data_ptr(),
                                                 _stream_ptr(self.device)), "f3m_plan_place_rows")
        return out

    def finest_boxes(self):
        """(target boxes, source boxes) at the finest level (1, 1 when no level was built)."""
        L = self.stats()["levels"]
        if L == 0:
            return 1, 1
        info = self.level(L)
        return info["boxes_x"], info["boxes_y"]

    # ---- introspection ---------------------------------------------------------------------
    def stats(self) -> Dict:
        s = PlanStats()
        check(_lib.lib().f3m_plan_get_stats(self._h, C.byref(s)), "f3m_plan_get_stats")
        return {k: getattr(s, k) for k, _ in PlanStats._fields_}

    def level(self, level: int) -> Dict:
        s = LevelInfo()
        check(_lib.lib().f3m_plan_get_level(self._h, level, C.byref(s)), "f3m_plan_get_level")
        return {k: getattr(s, k) for k, _ in LevelInfo._fields_}

    def timings(self) -> Dict:
        ms = (C.c_float * 8)()
        check(_lib.lib().f3m_plan_last_timings(self._h, ms), "f3m_plan_last_timings")
        names = ["permute", "direct", "p2m", "m2l", "l2p", "unpermute", "total", "build"]
        d = {n: float(ms[i]) for i, n in enumerate(names)}
        d["direct_launches"] = int(_lib.lib().f3m_plan_last_direct_launches(self._h))
        return d

    def direct_variants(self) -> Dict:
        """Direct-sum launches of the last apply() by kernel form (f3m_plan_last_direct_variants)."""
        c = (C.c_int32 * 6)()
        check(_lib.lib().f3m_plan_last_direct_variants(self._h, c), "f3m_plan_last_direct_variants")
        return dict(zip(("mufu", "poly2", "poly3", "direct", "moments", "tensor"), (int(v) for v in c)))

    def array(self, level: int, tree: int, what: int) -> np.ndarray:
        info = self.level(level) if level >= 1 else None
        nb = (info["boxes_x"] if tree == 0 else info["boxes_y"]) if info else 1
        nbx = info["boxes_x"] if info else 1
        if what == _lib.ARR_SORTED_INDEX:
            shape, dt = ((self.N if tree == 0 else self.M),), np.int32
        elif what == _lib.ARR_BOX_OFFSETS:
            shape, dt = (nb + 1,), np.int32
        elif what == _lib.ARR_BOX_CENTERS:
            shape, dt = (nb, self.d), np.float32
        elif what == _lib.ARR_BOX_CODES:
            shape, dt = (nb,), np.uint32
        elif what in (_lib.ARR_FAR_PTR, _lib.ARR_SMALL_PTR, _lib.ARR_KEEP_PTR):
            shape, dt = (nbx + 1,), np.int32
        else:
            key = {_lib.ARR_FAR_IDX: "n_far", _lib.ARR_SMALL_IDX: "n_small", _lib.ARR_KEEP_IDX: "n_keep"}[what]
            shape, dt = ((info[key] if info else 1),), np.int32
        out = np.empty(shape, dtype=dt)
        check(_lib.lib().f3m_plan_copy_array(self._h, level, tree, what, out.ctypes.data_as(C.c_void_p), out.nbytes),
              "f3m_plan_copy_array")
        return out

    def pairs(self, level: int, cls: str) -> np.ndarray:
        """(n,2) int array of (target box, source box) of one class ('far', 'small', 'keep'), sorted."""
        pid, iid = {"far": (_lib.ARR_FAR_PTR, _lib.ARR_FAR_IDX), "small": (_lib.ARR_SMALL_PTR, _lib.ARR_SMALL_IDX),
                    "keep": (_lib.ARR_KEEP_PTR, _lib.ARR_KEEP_IDX)}[cls]
        ptr, idx = self.array(level, 0, pid), self.array(level, 0, iid)
        left = np.repeat(np.arange(ptr.size - 1), np.diff(ptr))
        return np.stack([left, idx], 1).astype(np.int64)

    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            _lib.lib().f3m_plan_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def kmvm(X, Y, b, params: Params) -> torch.Tensor:
    """One-shot product through f3m_kmvm_f32 (tree built and dropped inside the call)."""
    same = is_shared(X, Y)
    X = _as_f32(X)
    Y = X if same else _as_f32(Y)
    b = _as_f32(b)
    if b.dim() == 1:
        b = b[:, None]
    _check_product_shapes(X, Y, b)
    if not (X.is_cuda and Y.is_cuda and b.is_cuda):
        raise ValueError("kmvm needs CUDA tensors: the engine has no CPU path (use kmvm_host for host buffers)")
    out = torch.empty(X.shape[0], b.shape[1], device=X.device, dtype=torch.float32)
    with torch.cuda.device(X.device):
        st = _lib.lib().f3m_kmvm_f32(X.data_ptr(), X.shape[0], Y.data_ptr(), Y.shape[0], b.data_ptr(), b.shape[1],
                                     X.shape[1], C.byref(params), out.data_ptr(), _stream_ptr(X.device))
    check(st, "f3m_kmvm_f32")
    return out


def workspace_bytes(N: int, M: int, R: int, d: int, params: Params) -> int:
    """Estimated bytes of temporaries of one product (f3m_workspace_bytes)."""
    return int(_lib.lib().f3m_workspace_bytes(int(N), int(M), int(R), int(d), C.byref(params)))


def kmvm_ws(X, Y, b, params: Params, workspace: torch.Tensor) -> torch.Tensor:
    """One-shot product whose temporaries all come out of `workspace`, a CUDA tensor the caller owns
    (f3m_kmvm_ws_f32): the library requests nothing from the driver during the call."""
    same = is_shared(X, Y)
    X = _as_f32(X)
    Y = X if same else _as_f32(Y)
    b = _as_f32(b)
    if b.dim() == 1:
        b = b[:, None]
    _check_product_shapes(X, Y, b)
    if not (X.is_cuda and Y.is_cuda and b.is_cuda and workspace.is_cuda and workspace.is_contiguous()):
        raise ValueError("kmvm_ws needs CUDA tensors and a contiguous CUDA workspace")
    out = torch.empty(X.shape[0], b.shape[1], device=X.device, dtype=torch.float32)
    with torch.cuda.device(X.device):
        st = _lib.lib().f3m_kmvm_ws_f32(X.data_ptr(), X.shape[0], Y.data_ptr(), Y.shape[0], b.data_ptr(), b.shape[1],
                                        X.shape[1], C.byref(params), out.data_ptr(), workspace.data_ptr(),
                                        workspace.numel() * workspace.element_size(), _stream_ptr(X.device))
    check(st, "f3m_kmvm_ws_f32")
    return out


def last_workspace_peak() -> int:
    return int(_lib.lib().f3m_last_workspace_peak())


def kmvm_host(X, Y, b, params: Params, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Product with HOST tensors through f3m_kmvm_host_f32: H2D copies, product, D2H copy in one call."""
    same = is_shared(X, Y)
    X = _as_f32(X)
    Y = X if same else _as_f32(Y)
    b = _as_f32(b)
    if b.dim() == 1:
        b = b[:, None]
    _check_product_shapes(X, Y, b)
    if X.is_cuda or Y.is_cuda or b.is_cuda:
        raise ValueError("kmvm_host takes CPU tensors")
    if out is None:
        out = torch.empty(X.shape[0], b.shape[1], dtype=torch.float32)
    st = _lib.lib().f3m_kmvm_host_f32(X.data_ptr(), X.shape[0], Y.data_ptr(), Y.shape[0], b.data_ptr(), b.shape[1],
                                      X.shape[1], C.byref(params), out.data_ptr())
    check(st, "f3m_kmvm_host_f32")
    return out


def rbf_dense(X, Y, b, ls: float, grad: bool = False) -> torch.Tensor:
    """Exact dense product (f3m_rbf_dense_f32 / _f64 / _grad_f32), dtype taken from X."""
    if not X.is_cuda:
        raise ValueError("rbf_dense needs CUDA tensors")
    dt = X.dtype
    if dt not in (torch.float32, torch.float64):
        X, dt = X.float(), torch.float32
    X, Y, b = X.contiguous(), Y.to(dt).contiguous(), b.to(dt).contiguous()
    if b.dim() == 1:
        b = b[:, None]
    assert Y.shape[1] == X.shape[1] and Y.shape[0] == b.shape[0]
    out = torch.empty(X.shape[0], b.shape[1], device=X.device, dtype=dt)
    L = _lib.lib()
    with torch.cuda.device(X.device):
        if dt == torch.float64:
            if grad:
                raise NotImplementedError("the gradient op exists in float32 only")
            st = L.f3m_rbf_dense_f64(X.data_ptr(), X.shape[0], Y.data_ptr(), Y.shape[0], b.data_ptr(), b.shape[1],
                                     X.shape[1], float(ls), out.data_ptr(), _stream_ptr(X.device))
        else:
            fn = L.f3m_rbf_dense_grad_f32 if grad else L.f3m_rbf_dense_f32
            st = fn(X.data_ptr(), X.shape[0], Y.data_ptr(), Y.shape[0], b.data_ptr(), b.shape[1], X.shape[1], float(ls),
                    out.data_ptr(), _stream_ptr(X.device))
    check(st, "f3m_rbf_dense")
    return out


def measure_peaks(device=None) -> Dict:
    """Measured exponential (MUFU.EX2) and FP32 FMA issue peaks of the current GPU, in G ops/s."""
    a, b = C.c_double(), C.c_double()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        check(_lib.lib().f3m_measure_peaks(C.byref(a), C.byref(b), _stream_ptr(dev)), "f3m_measure_peaks")
    return {"gexp_per_s": a.value, "gfma_per_s": b.value}


def release_cached_memory():
    """Returns the device blocks the library keeps for reuse to the driver (f3m_release_cached_memory)."""
    check(_lib.lib().f3m_release_cached_memory(), "f3m_release_cached_memory")


def launch_count() -> int:
    return int(_lib.lib().f3m_launch_count())
