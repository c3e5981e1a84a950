"""CPU tests (no GPU): the oracle against the exact product and against the golden fixtures produced by
the reference itself, the host-side logic, and the C-ABI library's symbol table."""
import ctypes
import glob
import os
import re
import sys

import numpy as np
import pytest
import torch

from cases import CASES, make_case, oracle_kwargs, rel_l2

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")


# ---------------------------------------------------------------------------------------------
# C ABI
# ---------------------------------------------------------------------------------------------
def declared_symbols():
    text = open(os.path.join(ROOT, "include", "f3m.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(f3m_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from f3m_b200 import _lib
    handle = ctypes.CDLL(_lib.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(handle, n), f"{n} is declared in include/f3m.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert _lib.lib().f3m_version() >= 100
    assert _lib.lib().f3m_status_string(0) == b"ok"


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU error path")
def test_no_gpu_is_an_error_not_a_fallback():
    from f3m_b200 import _lib, engine
    a, b = ctypes.c_double(), ctypes.c_double()
    st = _lib.lib().f3m_measure_peaks(ctypes.byref(a), ctypes.byref(b), None)
    assert st == 2      # F3M_ERR_CUDA
    assert b"failed" in _lib.lib().f3m_last_error()
    with pytest.raises(ValueError):
        engine.Plan(torch.rand(10, 3), None, engine.make_params(1.0, 1000, 64, False, 0.15, 64))
    with pytest.raises(_lib.F3MError):
        engine.kmvm_host(torch.rand(10, 3), None, torch.rand(10, 1), engine.make_params(1.0, 1000, 64, False, 0.15, 64))


def test_argument_checks_without_gpu():
    from f3m_b200 import _lib
    L = _lib.lib()
    prm = _lib.Params(1.0, 1000.0, 64, 0, 0.15, 64, 0, 0)
    plan = ctypes.c_void_p()
    buf = (ctypes.c_float * 30)()
    assert L.f3m_plan_create(ctypes.byref(plan), buf, 10, buf, 10, 7, ctypes.byref(prm), None) == 1   # bad dimension
    assert L.f3m_plan_create(ctypes.byref(plan), buf, 0, buf, 0, 3, ctypes.byref(prm), None) == 1    # empty input
    assert L.f3m_plan_create(ctypes.byref(plan), None, 10, buf, 10, 3, ctypes.byref(prm), None) == 1  # null pointer
    assert L.f3m_plan_apply(None, buf, 1, buf, None) == 1
    assert L.f3m_plan_destroy(None) == 0


# ---------------------------------------------------------------------------------------------
# oracle vs exact product
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name,tol", [("u3_default", 2e-5), ("u3_xy", 2e-3), ("u2_shared", 1e-4), ("u1_shared", 1e-5),
                                      ("tiny", 1e-6), ("dup_points", 1e-3)])
def test_oracle_against_float64_dense(name, tol):
    from oracle.f3m_oracle import f3m_kmvm, dense_kmvm_f64
    c = make_case(name)
    out = f3m_kmvm(c["X"], c["Y"], c["b"], **oracle_kwargs(c))
    Y = c["X"] if c["Y"] is None else c["Y"]
    rows = torch.arange(min(c["N"], 2000))
    exact = dense_kmvm_f64(c["X"], Y, c["b"], c["ls"], rows=rows)
    assert rel_l2(out[rows], exact) <= tol


def test_oracle_node_rule_and_grid():
    from oracle.f3m_oracle import node_list, cheb_nodes_weights, tensor_grid, lagrange_basis_1d
    assert node_list(3, 64) == [4, 4, 4] and node_list(3, 125) == [5, 5, 5] and node_list(3, 216) == [6, 6, 6]
    assert node_list(4, 81) == [3, 3, 3, 3] and node_list(5, 3125) == [5] * 5 and node_list(2, 36) == [6, 6]
    nodes, w = cheb_nodes_weights(5)
    assert np.allclose(nodes.numpy(), np.cos((2 * np.arange(5) + 1) * np.pi / 10), atol=1e-6)
    idx, grid = tensor_grid([nodes, nodes, nodes])
    assert idx[1].tolist() == [1, 0, 0] and idx[5].tolist() == [0, 1, 0]      # dimension 0 fastest
    t = torch.tensor([-0.9, 0.1, 0.77, float(nodes[2])])
    L = lagrange_basis_1d(t, nodes, w)
    assert np.allclose(L.sum(1).numpy(), 1.0, atol=1e-5)                       # partition of unity
    assert L[3].tolist() == [0, 0, 1, 0, 0]                                    # exact node hit
    poly = lambda x: 3 * x ** 4 - x ** 2 + 0.5
    assert np.allclose((L @ poly(nodes)).numpy(), poly(t).numpy(), atol=1e-5)  # degree p-1 is reproduced


# ---------------------------------------------------------------------------------------------
# oracle vs fixtures produced by the reference itself on a B200 (tests/golden/make_golden.py)
# ---------------------------------------------------------------------------------------------
def golden_files():
    return sorted(glob.glob(os.path.join(GOLDEN, "*.npz")))


def test_golden_fixtures_present():
    assert len(golden_files()) >= 4, "golden fixtures missing: run tests/golden/make_golden.py on a GPU box"


@pytest.mark.parametrize("path", golden_files(), ids=lambda p: os.path.basename(p)[:-4])
def test_oracle_against_reference_golden(path):
    """Box structure and pair lists of the oracle equal the reference's except where the reference's
    fast-math divide/sqrt put a point or a pair on the other side of a boundary; the product agrees to
    the tolerance of north_star (rel-L2 1e-5) plus the effect of those few differences."""
    from oracle.f3m_oracle import f3m_kmvm
    name = os.path.basename(path)[:-4]
    g = np.load(path)
    c = make_case(name)
    trace = []
    ties = []

    def reference_decision(level, tie_pairs):
        # pairs within a few ulp of the far threshold (exact ties of whole offset families in 4-D and 5-D): take the
        # reference's own far / not-far decision from the fixture, everything else is the restatement's
        far = set(map(tuple, g[f"l{level}_far"].tolist()))
        ties.append(int(tie_pairs.shape[0]))
        return torch.tensor([tuple(p) in far for p in tie_pairs.tolist()], dtype=torch.bool)

    out = f3m_kmvm(c["X"], c["Y"], c["b"], trace=trace, near_tie_far=reference_decision if c["d"] >= 4 else None,
                   **oracle_kwargs(c))
    if c["d"] >= 4:
        print(f"{name}: {sum(ties)} pairs on the far threshold took the reference's decision")
    levels = [t for t in trace if "far" in t]
    assert len(levels) == int(g["levels"])
    moved_total = 0
    for t in levels:
        l = t["level"]
        for key in ("x", "y"):
            ref_off = g[f"l{l}_{key}_offsets"]
            mine = t[key]["offsets"].numpy()
            assert mine.size == ref_off.size, f"level {l}: {mine.size - 1} boxes vs reference {ref_off.size - 1}"
            moved = int(np.abs(np.diff(mine) - np.diff(ref_off)).sum())
            moved_total += moved
            assert moved <= max(2, c["N"] // 2000), f"level {l}: {moved} points in different boxes"
            assert np.allclose(t[key]["centers"].numpy(), g[f"l{l}_{key}_centers"], rtol=0, atol=1e-6 * float(g[f"l{l}_{key}_edge"]) * 2 ** l)
        for cls in ("far", "small", "keep"):
            a = set(map(tuple, t[cls].numpy().tolist()))
            b = set(map(tuple, g[f"l{l}_{cls}"].tolist()))
            diff = len(a ^ b)
            assert diff <= (0 if moved_total == 0 else 8 + 4 * moved_total), f"level {l} {cls}: {diff} pairs differ"
    err = rel_l2(out.numpy(), g["out"])
    assert err <= (1e-5 if moved_total == 0 else 1e-4), f"rel-L2 vs reference product {err:.3e}"


# ---------------------------------------------------------------------------------------------
# multi-rank host logic on CPU (gloo, world size 2)
# ---------------------------------------------------------------------------------------------
class _FakePlan:
    """Stand-in for engine.Plan in the multi-rank host logic: same phase methods, dense float64 arithmetic on the CPU.
    "Sorted order" is a fixed permutation, "boxes" are runs of 37 sorted rows, the near part of the product is the
    dense kernel product and the far part is a made-up term that needs every box's moment in the right order, so that
    a moment slice that is lost, misplaced or taken from the wrong rank changes the result."""
    BOX = 37

    def __init__(self, X, ls):
        from oracle.f3m_oracle import dense_kmvm_f64
        self._dense = dense_kmvm_f64
        self.X, self.ls = X, ls
        self.N = X.shape[0]
        g = torch.Generator().manual_seed(99)
        self.perm = torch.randperm(self.N, generator=g)            # sorted position -> input row
        self.nb = -(-self.N // self.BOX)

    def partition_rows(self, R, nparts):
        cuts = [0] + [min(self.N, self.BOX * ((self.nb * k) // nparts + (k % 2))) for k in range(1, nparts)] + [self.N]
        return cuts                                                 # uneven on purpose, at box starts

    def moments_size(self, R):
        return self.nb * R

    def finest_boxes(self):
        return self.nb, self.nb

    def shard_begin(self, b, row_range, box_range, mom_slice):
        self.b, self.rows, self.R = b, row_range, b.shape[1]
        bs = b[self.perm]
        for j in range(box_range[0], box_range[1]):                # "moment" of a box: the sum of its rows of b
            mom_slice.view(-1, self.R)[j - box_range[0]] = bs[j * self.BOX:(j + 1) * self.BOX].sum(0)

    def shard_near(self, acc):
        rb, re = self.rows
        rows = self.perm[rb:re]
        acc[rb:re] = self._dense(self.X[rows], self.X, self.b, self.ls).float()

    def shard_far(self, mom, acc):
        rb, re = self.rows
        m = mom.view(-1, self.R)[:self.nb]
        w = torch.arange(1, self.nb + 1, dtype=torch.float32)[:, None]
        acc[rb:re] += 1e-3 * (w * m).sum(0)

    def shard_end(self):
        pass

    def rows_by_owner(self, acc, row_range, in_bounds):
        rb, re = row_range
        rows = self.perm[rb:re]
        owner = torch.bucketize(rows, torch.tensor(in_bounds[1:-1]), right=True)
        order = torch.argsort(owner, stable=True)
        send = torch.cat([acc[rb:re][order], rows[order, None].int().view(torch.float32)], 1)
        return send.contiguous(), torch.bincount(owner, minlength=len(in_bounds) - 1).tolist()

    def place_rows(self, recs, lo, hi):
        out = torch.full((hi - lo, recs.shape[1] - 1), float("nan"))
        out[recs[:, -1].contiguous().view(torch.int32).long() - lo] = recs[:, :-1]
        return out

    def rows_to_input_order(self, acc, lo, hi):
        out = torch.empty(self.N, acc.shape[1])
        out[self.perm] = acc
        return out[lo:hi].clone()

    def close(self):
        pass


class _FakePlanGather(_FakePlan):
    """With the all-gather form of the result exchange (what the engine's plan offers for one or two columns)."""

    def gathered_rows_to_input_order(self, gathered, slice_bounds, stride, lo, hi):
        acc = torch.cat([gathered[g * stride:g * stride + slice_bounds[g + 1] - slice_bounds[g]] for g in range(len(slice_bounds) - 1)])
        return self.rows_to_input_order(acc, lo, hi)


class _FakeBackend:
    def __init__(self, gather_form):
        self.cls = _FakePlanGather if gather_form else _FakePlan

    def plan(self, X, params):
        return self.cls(X, params)


def _rank_main(rank, world, port, q):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from f3m_b200.parallel import distributed_kmvm
    from oracle.f3m_oracle import dense_kmvm_f64
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(3)
    X, b = torch.rand(1001, 3, generator=g), torch.randn(1001, 2, generator=g)
    cuts = [0, 377, 1001] if world == 2 else [0, 200, 377, 1001]    # uneven shards
    lo, hi = cuts[rank], cuts[rank + 1]
    out = distributed_kmvm(X[lo:hi], b[lo:hi], 0.5, backend=_FakeBackend(gather_form=(world == 2)))
    plan = _FakePlan(X, 0.5)
    bs = b[plan.perm]
    mom = torch.stack([bs[j * plan.BOX:(j + 1) * plan.BOX].sum(0) for j in range(plan.nb)])
    far = 1e-3 * (torch.arange(1, plan.nb + 1, dtype=torch.float32)[:, None] * mom).sum(0)
    exact = dense_kmvm_f64(X, X, b, 0.5).float() + far
    q.put((rank, tuple(out.shape), rel_l2(out, exact[lo:hi])))
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_distributed_host_logic_gloo(world):
    """The phases of f3m_b200.parallel.distributed_kmvm on CPU ranks (gloo): shards of unequal size, slices of unequal
    size, moment slices gathered in box order, every rank gets exactly the rows of its own shard."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + 7 * world) % 2000
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(30)
        assert p.exitcode == 0
    sizes = {2: [377, 624], 3: [200, 177, 624]}[world]
    for rank, shape, err in res:
        assert shape == (sizes[rank], 2)
        assert err <= 1e-6, res
