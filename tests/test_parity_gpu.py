"""GPU parity tests: the CUDA engine (through the C ABI) against the CPU oracle on seeded inputs.

Bit-exact: per-level box offsets / counts, box centres, far / small / keep pair lists (engine in
IEEE mode vs the oracle's IEEE float32 arithmetic).  Floating point: KMVM output within rel-L2
1e-5 of the oracle's output and no worse than the oracle against the exact float64 product
(rel-L2 1e-5 against the reference algorithm at equal nodes and leaf size is the tolerance this engine is specified to)."""
import numpy as np
import pytest
import torch

from cases import CASES, make_case, oracle_kwargs, random_cases, rel_l2

pytestmark = pytest.mark.gpu

TOL_VS_ORACLE = 1e-5


def _run_engine(c, dev, math_mode):
    from f3m_b200 import engine, _lib
    prm = engine.make_params(c["ls"], c["min_points"], c["P"], c["var_comp"], c["eff"], c["small"], math_mode)
    X = c["X"].to(dev)
    Y = None if c["Y"] is None else c["Y"].to(dev)
    plan = engine.Plan(X, Y, prm)
    out = plan.apply(c["b"].to(dev))
    return plan, out


RANDOM_CASES = random_cases(24)


@pytest.mark.parametrize("name", list(RANDOM_CASES))
def test_engine_matches_oracle_random_configs(name, cuda):
    """Randomized sweep over the parameter space (seeded): same checks as the named cases."""
    _check_against_oracle(make_case(name, RANDOM_CASES), cuda)


@pytest.mark.parametrize("name", list(CASES))
def test_engine_matches_oracle(name, cuda):
    _check_against_oracle(make_case(name), cuda)


def _check_against_oracle(c, cuda):
    from f3m_b200 import _lib
    from oracle.f3m_oracle import f3m_kmvm, dense_kmvm_f64
    trace, stats = [], {}
    ref = f3m_kmvm(c["X"], c["Y"], c["b"], trace=trace, stats=stats, **oracle_kwargs(c))
    plan, out = _run_engine(c, cuda, _lib.MATH_IEEE)
    st = plan.stats()
    levels = [t for t in trace if "far" in t]
    assert st["levels"] == len(levels)
    # ---- box assignment and interaction lists: bit-exact ------------------------------------
    for t in levels:
        l = t["level"]
        for tree, key in ((0, "x"), (1, "y")):
            off = plan.array(l, tree, _lib.ARR_BOX_OFFSETS)
            assert np.array_equal(off, t[key]["offsets"].numpy().astype(np.int32)), f"box offsets differ at level {l}"
            ctr = plan.array(l, tree, _lib.ARR_BOX_CENTERS)
            assert np.array_equal(ctr, t[key]["centers"].numpy()), f"box centres differ at level {l}"
            perm = plan.array(l, tree, _lib.ARR_SORTED_INDEX).astype(np.int64)
            box_of_sorted = np.repeat(np.arange(off.size - 1), np.diff(off))
            box_of_point = np.empty_like(box_of_sorted)
            box_of_point[perm] = box_of_sorted
            assert np.array_equal(box_of_point, t[key]["box_of_point"].numpy()), f"box of point differs at level {l}"
        for cls in ("far", "small", "keep"):
            assert np.array_equal(plan.pairs(l, cls), t[cls].numpy()), f"{cls} list differs at level {l}"
    assert st["direct_pairs"] == stats.get("direct_pairs", 0)
    assert st["node_pairs"] == stats.get("node_pairs", 0)
    # ---- output -------------------------------------------------------------------------------
    out = out.cpu()
    err_ref = rel_l2(out, ref)
    assert err_ref <= TOL_VS_ORACLE, f"rel-L2 vs oracle {err_ref:.3e}"
    rows = torch.arange(min(c["N"], 3000))
    Ysrc = c["X"] if c["Y"] is None else c["Y"]
    exact = dense_kmvm_f64(c["X"], Ysrc, c["b"], c["ls"], rows=rows)
    e_engine, e_oracle = rel_l2(out[rows], exact), rel_l2(ref[rows], exact)
    assert e_engine <= max(1.2 * e_oracle, e_oracle + 2e-6), f"engine {e_engine:.3e} vs oracle {e_oracle:.3e} against float64"


def _golden_names():
    import glob, os
    here = os.path.dirname(os.path.abspath(__file__))
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(here, "golden", "*.npz")))


@pytest.mark.parametrize("name", _golden_names())
def test_engine_matches_reference_golden(name, cuda):
    """Default (fast-math) mode against fixtures produced by the reference itself on a B200
    (tests/golden/make_golden.py): box offsets, box of every point, centres and the far / small / keep
    lists bit-exact; product within rel-L2 1e-5 of the reference's."""
    import os
    from f3m_b200 import _lib
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", name + ".npz"))
    c = make_case(name)
    plan, out = _run_engine(c, cuda, _lib.MATH_FASTMATH)
    L = int(g["levels"])
    assert plan.stats()["levels"] == L
    for l in range(1, L + 1):
        for tree, key in ((0, "x"), (1, "y")):
            assert np.array_equal(plan.array(l, tree, _lib.ARR_BOX_OFFSETS), g[f"l{l}_{key}_offsets"]), f"offsets, level {l}"
            assert np.array_equal(plan.array(l, tree, _lib.ARR_BOX_CENTERS), g[f"l{l}_{key}_centers"]), f"centres, level {l}"
        for cls in ("far", "small", "keep"):
            assert np.array_equal(plan.pairs(l, cls), g[f"l{l}_{cls}"].astype(np.int64)), f"{cls} list, level {l}"
    for tree, key in ((0, "x"), (1, "y")):
        off = plan.array(L, tree, _lib.ARR_BOX_OFFSETS)
        perm = plan.array(L, tree, _lib.ARR_SORTED_INDEX).astype(np.int64)
        box_of_point = np.empty(perm.size, dtype=np.int64)
        box_of_point[perm] = np.repeat(np.arange(off.size - 1), np.diff(off))
        assert np.array_equal(box_of_point, g[f"{key}_box_of_point_finest"]), "box of point at the finest level"
    err = rel_l2(out.cpu(), g["out"])
    assert err <= TOL_VS_ORACLE, f"rel-L2 vs reference product {err:.3e}"
    # the reference's own exact dense op (rbf_float_d, F3M_src/pybinder_setup.cu:40-50) on the first rows, stored in the
    # fixture, against this engine's dense op: both are float32 sums with an approximate exponential
    from f3m_b200 import engine
    ref_rows = g["dense_ref_rows"]
    X = c["X"].to(cuda)
    Y = X if c["Y"] is None else c["Y"].to(cuda)
    dense = engine.rbf_dense(X[:ref_rows.shape[0]].contiguous(), Y, c["b"].to(cuda), c["ls"]).cpu()
    assert rel_l2(dense, ref_rows) <= 5e-6, f"dense op vs the reference's dense op {rel_l2(dense, ref_rows):.3e}"


@pytest.mark.parametrize("name", ["u3_shared", "u3_xy", "n4_r8"])
def test_fastmath_mode_close_to_ieee(name, cuda):
    """The default (fast-math) box index / far test differs from IEEE only for points within a few
    ulp of a cell face or pairs on the distance threshold: box counts differ by a handful of points."""
    from f3m_b200 import _lib
    c = make_case(name)
    p0, o0 = _run_engine(c, cuda, _lib.MATH_IEEE)
    p1, o1 = _run_engine(c, cuda, _lib.MATH_FASTMATH)
    assert p0.stats()["levels"] == p1.stats()["levels"]
    for l in range(1, p0.stats()["levels"] + 1):
        a, b = p0.array(l, 0, _lib.ARR_BOX_OFFSETS), p1.array(l, 0, _lib.ARR_BOX_OFFSETS)
        assert a.size == b.size
        assert np.abs(np.diff(a) - np.diff(b)).sum() <= max(4, c["N"] // 5000)
    # in 4-D the corner-touching boxes sit exactly on the far threshold (distance 2*edge), so the two
    # modes may classify whole families of pairs differently; the outputs then differ by the
    # interpolation error of those pairs, not by rounding
    assert rel_l2(o1.cpu(), o0.cpu()) <= (1e-4 if c["d"] <= 3 else 5e-2)


def test_one_shot_and_plan_agree(cuda):
    from f3m_b200 import engine, _lib
    c = make_case("u3_shared")
    prm = engine.make_params(c["ls"], c["min_points"], c["P"], c["var_comp"], c["eff"], c["small"])
    X, b = c["X"].to(cuda), c["b"].to(cuda)
    a = engine.kmvm(X, None, b, prm)
    plan = engine.Plan(X, None, prm)
    b1 = plan.apply(b)
    b2 = plan.apply(b)
    assert rel_l2(a.cpu(), b1.cpu()) <= 2e-6
    assert rel_l2(b2.cpu(), b1.cpu()) <= 2e-6
    host = engine.kmvm_host(c["X"], None, c["b"], prm)
    assert rel_l2(host, b1.cpu()) <= 2e-6


def test_row_range_shards_sum_to_full(cuda):
    """Target boxes sharded over row ranges (the multi-GPU split) add up to the full product."""
    from f3m_b200 import engine
    c = make_case("u3_shared")
    prm = engine.make_params(c["ls"], c["min_points"], c["P"], c["var_comp"], c["eff"], c["small"])
    plan = engine.Plan(c["X"].to(cuda), None, prm)
    b = c["b"].to(cuda)
    full = plan.apply(b)
    N = c["N"]
    cuts = [0, N // 3, N // 2, N]
    parts = sum(plan.apply(b, row_range=(cuts[i], cuts[i + 1])) for i in range(3))
    assert rel_l2(parts.cpu(), full.cpu()) <= 1e-6


@pytest.mark.parametrize("name", ["u3_shared", "n4_r8", "u3_xy"])
def test_sharded_moments_and_rows_sum_to_full(name, cuda):
    """The multi-GPU decomposition on one GPU: two "ranks" each interpolate their slice of the sources onto
    the finest-level nodes, the moment arrays are added (the all-reduce), and each computes its slice of the
    target boxes from the summed moments; the two outputs add up to the full product."""
    from f3m_b200 import engine
    c = make_case(name)
    prm = engine.make_params(c["ls"], c["min_points"], c["P"], c["var_comp"], c["eff"], c["small"])
    X = c["X"].to(cuda)
    Y = None if c["Y"] is None else c["Y"].to(cuda)
    plan = engine.Plan(X, Y, prm)
    b = c["b"].to(cuda)
    full = plan.apply(b)
    assert plan.moments_size(c["R"]) > 0
    N, M = plan.N, plan.M
    mom = plan.moments(b, (0, M // 3)) + plan.moments(b, (M // 3, M))
    parts = plan.apply(b, row_range=(0, N // 2), moments=mom) + plan.apply(b, row_range=(N // 2, N), moments=mom)
    assert rel_l2(parts.cpu(), full.cpu()) <= 2e-6


@pytest.mark.parametrize("d,ls,R", [(3, 3.0, 1), (3, 1.2, 2), (2, 2.0, 1), (4, 4.0, 3)])
def test_near_moments_flag(d, ls, R, cuda):
    """Optional moment form of the near field: with boxes much smaller than the lengthscale the near sums are
    evaluated from 2nd/3rd-order box moments; the result must agree with the direct sums to the size of the
    ex2.approx error, and the accuracy against float64 must not get worse."""
    from f3m_b200 import engine, _lib
    from oracle.f3m_oracle import dense_kmvm_f64
    g = torch.Generator().manual_seed(100 + d)
    X = torch.rand(40000, d, generator=g)
    b = torch.randn(40000, R, generator=g)
    P = {2: 36, 3: 64, 4: 81}[d]
    outs = {}
    for flags in (0, _lib.FLAG_NEAR_MOMENTS):
        prm = engine.make_params(ls, 300.0, P, False, 0.15, P, flags=flags)
        plan = engine.Plan(X.to(cuda), None, prm)
        outs[flags] = plan.apply(b.to(cuda)).cpu()
        assert plan.stats()["direct_pairs"] > 0
    assert rel_l2(outs[_lib.FLAG_NEAR_MOMENTS], outs[0]) <= 3e-6
    rows = torch.arange(2000)
    exact = dense_kmvm_f64(X, X, b, ls, rows=rows)
    e0, e1 = rel_l2(outs[0][rows], exact), rel_l2(outs[_lib.FLAG_NEAR_MOMENTS][rows], exact)
    assert e1 <= max(1.2 * e0, e0 + 2e-6)
    # a lengthscale for which the exponent bound is too large: the flag must change nothing
    prm0 = engine.make_params(0.05, 300.0, P, False, 0.15, P)
    prm1 = engine.make_params(0.05, 300.0, P, False, 0.15, P, flags=_lib.FLAG_NEAR_MOMENTS)
    a0 = engine.kmvm(X.to(cuda), None, b.to(cuda), prm0).cpu()
    a1 = engine.kmvm(X.to(cuda), None, b.to(cuda), prm1).cpu()
    assert rel_l2(a1, a0) <= 1e-7


@pytest.mark.parametrize("d,ls,n,xy", [(3, 3.0, 40000, False), (3, 0.8, 60000, False), (2, 2.0, 30000, False),
                                       (1, 1.0, 20000, False), (4, 4.0, 30000, False), (5, 6.0, 20000, False),
                                       (3, 2.0, 30000, True)])
def test_near_tensor_cores_flag(d, ls, n, xy, cuda):
    """Optional tcgen05 form of the direct near sums: the exponent matrix of a target tile against a source tile
    is a TF32 matrix product of split operands (exact to FP32 rounding).  It computes the same sums as the CUDA-core
    kernels, so the two must agree to FP32 rounding and share the accuracy against float64."""
    from f3m_b200 import engine, _lib
    from oracle.f3m_oracle import dense_kmvm_f64
    g = torch.Generator().manual_seed(200 + d)
    X = torch.rand(n, d, generator=g)
    Y = torch.rand(n // 2, d, generator=g) * 0.9 + 0.05 if xy else None
    b = torch.randn(Y.shape[0] if xy else n, 1, generator=g)
    P = {1: 6, 2: 36, 3: 64, 4: 81, 5: 32}[d]
    outs = {}
    for flags in (0, _lib.FLAG_NEAR_TENSOR_CORES):
        prm = engine.make_params(ls, 300.0, P, False, 0.15, P, flags=flags)
        plan = engine.Plan(X.to(cuda), None if Y is None else Y.to(cuda), prm)
        outs[flags] = plan.apply(b.to(cuda)).cpu()
        again = plan.apply(b.to(cuda)).cpu()
        assert rel_l2(again, outs[flags]) <= 5e-6   # summation order of the far field may differ between runs
        assert plan.stats()["direct_pairs"] > 0
    assert rel_l2(outs[_lib.FLAG_NEAR_TENSOR_CORES], outs[0]) <= 5e-6
    rows = torch.arange(1500)
    exact = dense_kmvm_f64(X, X if Y is None else Y, b, ls, rows=rows)
    e0, e1 = rel_l2(outs[0][rows], exact), rel_l2(outs[_lib.FLAG_NEAR_TENSOR_CORES][rows], exact)
    assert e1 <= max(1.2 * e0, e0 + 2e-6)


@pytest.mark.parametrize("p", [2, 3, 4, 5, 6, 7, 8])
def test_far_field_node_counts_d3(p, cuda):
    """Every node count of the fast far-field path in three dimensions (P2M/L2P register tiling, nested M2L) against
    the CPU restatement, and the interpolation error against float64 must fall with the node count."""
    from f3m_b200 import engine, _lib
    from oracle.f3m_oracle import f3m_kmvm, dense_kmvm_f64
    g = torch.Generator().manual_seed(300 + p)
    n = 12000
    X = torch.rand(n, 3, generator=g) * 3.0
    b = torch.randn(n, 1, generator=g)
    P = p ** 3
    prm = engine.make_params(1.0, 100.0, P, False, 0.15, 20, math_mode=_lib.MATH_IEEE)
    out = engine.kmvm(X.to(cuda), None, b.to(cuda), prm).cpu()
    ref = f3m_kmvm(X, None, b, 1.0, min_points=100.0, nr_of_interpolation=P, small_field_points=20)
    exact = dense_kmvm_f64(X, X, b, 1.0)
    e_ref, e_out = rel_l2(ref, exact), rel_l2(out, exact)
    print(f"p={p}: error of the restatement {e_ref:.3e}, of the engine {e_out:.3e}, between them {rel_l2(out, ref):.3e}")
    assert rel_l2(out, ref) <= max(1e-5, 0.2 * e_ref)       # same algorithm, different summation order
    assert e_out <= 1.2 * e_ref + 2e-6
    assert e_out <= {2: 0.5, 3: 0.2, 4: 5e-2, 5: 1e-2, 6: 3e-3, 7: 6e-4, 8: 2e-4}[p]


def test_failed_call_leaves_library_usable(cuda):
    """A call that fails (one point: no bounding cube) must not poison the next one: status and message for the
    failure, then a correct product from the same process.  Degenerate but valid inputs work: two points, points on a
    line, far-apart clusters, large offsets, extreme lengthscales, leaf size 1."""
    from f3m_b200 import engine
    g = torch.Generator().manual_seed(77)

    def product(X, b, ls=1.0, mp=100., P=27):
        prm = engine.make_params(ls, mp, P, False, 0.15, P)
        out = engine.kmvm(X.to(cuda), None, b.to(cuda), prm).cpu()
        exact = engine.rbf_dense(X.double().to(cuda), X.double().to(cuda), b.double().to(cuda), ls).cpu()
        return rel_l2(out, exact)

    with pytest.raises(RuntimeError, match="bounding cube"):
        product(torch.rand(1, 3, generator=g), torch.randn(1, 1, generator=g))
    with pytest.raises(RuntimeError, match="bounding cube"):
        product(torch.ones(500, 3) * 0.3, torch.randn(500, 1, generator=g))
    bad = torch.rand(3000, 3, generator=g)
    bad[17, 1] = float("nan")
    with pytest.raises(RuntimeError, match="bounding cube"):
        product(bad, torch.randn(3000, 1, generator=g))
    bad[17, 1] = float("inf")
    with pytest.raises(RuntimeError, match="bounding cube"):
        product(bad, torch.randn(3000, 1, generator=g))
    assert product(torch.rand(2, 3, generator=g), torch.randn(2, 1, generator=g)) <= 1e-5
    assert product(torch.rand(4000, 3, generator=g), torch.randn(4000, 1, generator=g)) <= 5e-3
    line = torch.cat([torch.rand(5000, 1, generator=g), torch.zeros(5000, 2)], 1)
    assert product(line, torch.randn(5000, 1, generator=g)) <= 5e-3
    far = torch.cat([torch.rand(3000, 3, generator=g) * 0.05, torch.rand(3000, 3, generator=g) * 0.05 + 10.0])
    assert product(far, torch.randn(6000, 1, generator=g)) <= 5e-3
    # clusters 1e5 times smaller than their distance need more levels than a 30-bit cell index holds: a clean error
    too_deep = torch.cat([torch.rand(3000, 3, generator=g) * 1e-3, torch.rand(3000, 3, generator=g) * 1e-3 + 100.0])
    with pytest.raises(RuntimeError, match="level"):
        product(too_deep, torch.randn(6000, 1, generator=g))
    assert product(torch.rand(5000, 3, generator=g) + 1e3, torch.randn(5000, 1, generator=g)) <= 5e-3
    assert product(torch.rand(5000, 3, generator=g), torch.randn(5000, 1, generator=g), ls=1e-3) <= 1e-4
    assert product(torch.rand(5000, 3, generator=g), torch.randn(5000, 1, generator=g), ls=1e3) <= 1e-4
    assert product(torch.rand(3000, 3, generator=g), torch.randn(3000, 1, generator=g), mp=1.) <= 5e-3


def test_dense_ops(cuda):
    from f3m_b200 import engine
    from oracle.f3m_oracle import dense_kmvm_f64
    g = torch.Generator().manual_seed(5)
    for d in (1, 2, 3, 4, 5):
        X, Y = torch.rand(700, d, generator=g), torch.rand(900, d, generator=g)
        b = torch.randn(900, 3, generator=g)
        exact = dense_kmvm_f64(X, Y, b, 0.6)
        out32 = engine.rbf_dense(X.to(cuda), Y.to(cuda), b.to(cuda), 0.6).cpu()
        out64 = engine.rbf_dense(X.double().to(cuda), Y.double().to(cuda), b.double().to(cuda), 0.6).cpu()
        assert rel_l2(out32, exact) <= 5e-6
        assert rel_l2(out64, exact) <= 1e-13
        # gradient op: ls^-3 sum r^2 exp(-r^2/(2 ls^2)) b   (n_tree.cu:213-241)
        r2 = torch.cdist(X.double(), Y.double()) ** 2
        gexact = (r2 * torch.exp(-r2 / (2 * 0.6 ** 2))) @ b.double() / 0.6 ** 3
        gout = engine.rbf_dense(X.to(cuda), Y.to(cuda), b.to(cuda), 0.6, grad=True).cpu()
        assert rel_l2(gout, gexact) <= 1e-5


def test_operator_surface(cuda):
    """FFM(X, ...) @ b, forward, chunked products and the ffm_3d_float function table."""
    import ffm_3d_float
    from F3M_src.FFM_classes import FFM, benchmark_matmul, benchmark_matmul_double
    torch.manual_seed(0)
    X = torch.rand(20000, 3)
    Y = torch.rand(6000, 3)
    b = torch.randn(20000, 1)
    op = FFM(X, ls=1.0, min_points=500, nr_of_interpolation=64, small_field_points=64, device="cuda:0")
    res = op @ b
    assert res.shape == (20000, 1) and res.is_cuda
    exact = benchmark_matmul_double(X[:2000], X, ls=1.0, device="cuda:0") @ b
    assert rel_l2(res[:2000].cpu(), exact.cpu()) <= 1e-4
    exact32 = benchmark_matmul(X[:2000], X, ls=1.0, device="cuda:0") @ b
    assert rel_l2(exact32.cpu(), exact.cpu()) <= 5e-6
    res2 = ffm_3d_float.FFM_XY_FLOAT_3(op.X, op.X, b.to("cuda:0"), "cuda:0", 1.0, 500.0, 64, False, 0.15, 64)
    assert rel_l2(res2.cpu(), res.cpu()) <= 2e-6
    opxy = FFM(X, Y, ls=1.0, min_points=500, nr_of_interpolation=64, small_field_points=64, device="cuda:0")
    by = torch.randn(6000, 2)
    full = opxy @ by
    chunked = opxy.chunk_forward_example(by, chunks=3)
    assert rel_l2(chunked.cpu(), full.cpu()) <= 1e-4
    # blocked products (block_FFM_matmul, par_FFM_block) against the single product
    from F3M_src.FFM_classes import block_FFM_matmul, par_FFM_block
    blk = block_FFM_matmul(X, ls=1.0, min_points=500, nr_of_interpolation=64, small_field_points=64, device="cuda:0", blocks_X=2)
    assert rel_l2(blk @ b, res.cpu()) <= 1e-4
    blkxy = block_FFM_matmul(X, Y, ls=1.0, min_points=500, nr_of_interpolation=64, small_field_points=64, device="cuda:0",
                             blocks_X=2, blocks_Y=3)
    assert rel_l2(blkxy @ by, full.cpu()) <= 1e-4
    par = par_FFM_block(X, b, ls=1.0, min_points=500, nr_of_interpolation=64, small_field_points=64, devices=[0, 0])
    parts = par()
    assert len(parts) == 4
    top = parts[0].cpu() + parts[2].cpu()          # row block 0: source blocks 0 and 1
    assert rel_l2(top, res[:top.shape[0]].cpu()) <= 1e-4
    with pytest.raises(AssertionError):
        opxy.forward(opxy.X, opxy.Y, torch.randn(5, 1, device="cuda:0"))
    with pytest.raises(AssertionError):
        op.forward(op.X.cpu(), op.X.cpu(), b)


def _load_reference_build():
    import importlib.util, os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "f3m_ref_d3.so")
    if not os.path.exists(path):
        pytest.skip("reference GPU build (oracle/_ref/f3m_ref_d3.so) not present")
    spec = importlib.util.spec_from_file_location("f3m_ref_d3", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("n,m,ls,P,var_comp", [(400000, None, 0.04, 64, False),      # box edge ~ lengthscale at the far levels
                                               (300000, None, 1.0, 216, False),
                                               (200000, 150000, 0.3, 125, False),
                                               (300000, None, 0.5, 64, True)])
def test_engine_vs_reference_live(n, m, ls, P, var_comp, cuda):
    """The engine against the UNMODIFIED reference running on the same GPU (checker only), at sizes the
    fixtures do not cover: product within rel-L2 1e-5 (north_star's tolerance), and the engine no worse
    than the reference against the float64 dense product."""
    from f3m_b200 import engine
    ref = _load_reference_build()
    g = torch.Generator().manual_seed(n + (m or 0))
    X = torch.rand(n, 3, generator=g).to(cuda)
    Y = X if m is None else (torch.rand(m, 3, generator=g) * 0.8 + 0.1).to(cuda)
    b = torch.randn(Y.shape[0], 1, generator=g).to(cuda)
    out_ref = ref.FFM_XY_FLOAT(X, Y, b, "cuda:0", float(ls), 1000.0, int(P), bool(var_comp), 0.3, int(P))
    torch.cuda.synchronize()
    prm = engine.make_params(ls, 1000.0, P, var_comp, 0.3, P)
    out = engine.kmvm(X, None if m is None else Y, b, prm)
    # box offsets and the three pair lists of every level, bit for bit, at a size the fixtures do not reach
    trace = ref.field_trace(X, Y, "cuda:0", float(ls), 1000.0, int(P), bool(var_comp), 0.3, int(P))
    torch.cuda.synchronize()
    plan = engine.Plan(X, None if m is None else Y, prm)
    assert plan.stats()["levels"] == len(trace)
    from f3m_b200 import _lib

    def canon(t):
        p_ = t.cpu().numpy().astype(np.int64).reshape(-1, 2)
        return p_[np.lexsort((p_[:, 1], p_[:, 0]))]

    for l, t in enumerate(trace, start=1):
        for cls, ref_pairs in zip(("far", "small", "keep"), t[:3]):
            assert np.array_equal(plan.pairs(l, cls), canon(ref_pairs)), f"{cls} list differs from the reference at level {l}"
        assert np.array_equal(plan.array(l, 0, _lib.ARR_BOX_OFFSETS), t[5].cpu().numpy().astype(np.int32)), f"target box offsets, level {l}"
        assert np.array_equal(plan.array(l, 1, _lib.ARR_BOX_OFFSETS), t[10].cpu().numpy().astype(np.int32)), f"source box offsets, level {l}"
    plan.close()
    err = rel_l2(out.cpu(), out_ref.cpu())
    rows = torch.arange(2000, device=cuda)
    exact = engine.rbf_dense(X[rows].double(), Y.double(), b.double(), ls).cpu()
    e_engine, e_ref = rel_l2(out[rows].cpu(), exact), rel_l2(out_ref[rows].cpu(), exact)
    assert e_engine <= max(1.2 * e_ref, e_ref + 2e-6), f"engine {e_engine:.3e} vs reference {e_ref:.3e} against float64"
    print(f"n={n} ls={ls} P={P}: engine-vs-reference {err:.3e}, engine-vs-f64 {e_engine:.3e}, reference-vs-f64 {e_ref:.3e}")
    # 1e-5 of the reference, unless the reference itself is further than that from the exact product: then the
    # engine cannot be closer to the reference than the reference is to the truth, and must beat it instead
    assert err <= max(TOL_VS_ORACLE, 1.1 * e_ref), f"rel-L2 vs reference {err:.3e} (reference's own error vs float64 {e_ref:.3e})"
    if err > TOL_VS_ORACLE:
        # The relaxed bound above was used.  Show where the gap comes from: evaluate the reference ALGORITHM (same
        # float32 tree and lists, per-level P2M -> M2L -> L2P, direct sums) in float64.  The engine must be within
        # 1e-5 of that, and the reference's distance from it -- its own float32 rounding -- must account for the gap.
        from oracle.f3m_oracle import f3m_kmvm
        alg64 = f3m_kmvm(X.cpu(), None if m is None else Y.cpu(), b.cpu(), ls, min_points=1000.0, nr_of_interpolation=P,
                         var_compression=var_comp, eff_var_limit=0.3, small_field_points=P, dtype=torch.float64)
        e_alg, r_alg = rel_l2(out.cpu(), alg64), rel_l2(out_ref.cpu(), alg64)
        print(f"   reference algorithm in float64: engine {e_alg:.3e}, reference {r_alg:.3e}")
        assert e_alg <= TOL_VS_ORACLE, f"engine vs the reference algorithm in float64 {e_alg:.3e}"
        assert r_alg >= 0.8 * err and abs(r_alg - err) <= 0.5 * err, \
            f"gap to the reference {err:.3e} is not explained by the reference's rounding {r_alg:.3e}"


def test_reference_algorithm_in_float64_p216(cuda):
    """At 216 nodes the reference's float32 rounding (atomic float32 P2M sums, exp of float32 node distances) is larger
    than 1e-5 of the product.  The engine is compared with the reference ALGORITHM evaluated in float64 (same float32 tree
    and lists): within 1e-5, and closer to it than the float32 restatement of the same algorithm is."""
    from f3m_b200 import engine, _lib
    from oracle.f3m_oracle import f3m_kmvm
    g = torch.Generator().manual_seed(216)
    n = 60000
    X = torch.rand(n, 3, generator=g)
    b = torch.randn(n, 1, generator=g)
    kw = dict(ls=1.0, min_points=400.0, nr_of_interpolation=216, var_compression=False, eff_var_limit=0.15, small_field_points=216)
    alg32 = f3m_kmvm(X, None, b, **kw)
    alg64 = f3m_kmvm(X, None, b, dtype=torch.float64, **kw)
    prm = engine.make_params(1.0, 400.0, 216, False, 0.15, 216, math_mode=_lib.MATH_IEEE)
    out = engine.kmvm(X.to(cuda), None, b.to(cuda), prm).cpu()
    e_engine, e_alg32 = rel_l2(out, alg64), rel_l2(alg32, alg64)
    print(f"P=216: engine vs algorithm-in-float64 {e_engine:.3e}; float32 restatement vs the same {e_alg32:.3e}")
    assert e_engine <= TOL_VS_ORACLE
    assert e_engine <= max(e_alg32, 2e-6)


def test_polynomial_exponent_variants_run(cuda):
    """Which form of the direct-sum kernel a list takes depends on (scaled box edge)^2: the all-MUFU form, the form
    that evaluates 2/5 of the exponentials by a degree-2 polynomial, and the degree-3 form must each run for the
    lengthscales chosen here, and each must agree with the CPU restatement of the same algorithm to 1e-5."""
    from f3m_b200 import engine, _lib
    from oracle.f3m_oracle import f3m_kmvm
    g = torch.Generator().manual_seed(31)
    n = 40000
    X = torch.rand(n, 3, generator=g)
    b = torch.randn(n, 1, generator=g)
    seen = {}
    for ls in (0.2, 1.6, 4.0):
        prm = engine.make_params(ls, 300.0, 64, False, 0.15, 64, math_mode=_lib.MATH_IEEE)
        plan = engine.Plan(X.to(cuda), None, prm)
        out = plan.apply(b.to(cuda)).cpu()
        v = plan.direct_variants()
        ref = f3m_kmvm(X, None, b, ls, min_points=300.0, nr_of_interpolation=64, small_field_points=64)
        err = rel_l2(out, ref)
        print(f"ls={ls}: variants {v}, rel-L2 vs the restatement {err:.3e}")
        assert err <= TOL_VS_ORACLE
        for k, c in v.items():
            seen[k] = seen.get(k, 0) + c
    assert seen["mufu"] > 0 and seen["poly2"] > 0 and seen["poly3"] > 0, seen


def test_two_separate_point_sets_level1_reach(cuda):
    """X and Y in two small cubes a few lengthscales apart: the level-1 boxes hold fewer than 2P points, so every
    level-1 pair is "small" whatever its distance (size is tested before distance, 1_d_conv.cu:916-920) and the
    direct sums see targets far outside the usual reach of a source box.  The result must match the float64 dense
    product; 150 lengthscales apart it must be finite and (numerically) zero."""
    from f3m_b200 import engine
    g = torch.Generator().manual_seed(41)
    for edge, sep, tol in ((0.1, 1.4, 2e-5), (0.15, 2.5, 2e-5), (0.2, 4.0, 1e-4), (1.0, 150.0, None)):
        X = torch.rand(300, 3, generator=g) * edge
        Y = torch.rand(250, 3, generator=g) * edge + sep
        b = torch.randn(250, 2, generator=g)
        prm = engine.make_params(1.0, 20.0, 64, False, 0.15, 64)
        plan = engine.Plan(X.to(cuda), Y.to(cuda), prm)
        out = plan.apply(b.to(cuda)).cpu()
        st = plan.stats()
        assert st["levels"] >= 1 and plan.level(1)["n_small"] > 0
        assert torch.isfinite(out).all()
        exact = engine.rbf_dense(X.double().to(cuda), Y.double().to(cuda), b.double().to(cuda), 1.0).cpu()
        if tol is None:
            assert float(out.abs().max()) <= 1e-30 and float(exact.abs().max()) <= 1e-30
        else:
            err = rel_l2(out, exact)
            print(f"edge {edge} separation {sep}: variants {plan.direct_variants()}, rel-L2 vs float64 {err:.3e}")
            assert err <= tol


def test_leading_slice_is_not_the_shared_tree(cuda):
    """Y = X[:k] starts at X's address but is another point set: it must not be taken for the shared-tree case
    (which would read N rows of a k-row b)."""
    from f3m_b200 import engine
    from F3M_src.FFM_classes import FFM
    g = torch.Generator().manual_seed(51)
    X = torch.rand(9000, 3, generator=g).to(cuda)
    b = torch.randn(9000, 1, generator=g).to(cuda)
    k = 2500
    prm = engine.make_params(1.0, 300.0, 64, False, 0.15, 64)
    out = engine.kmvm(X, X[:k], b[:k], prm)
    exact = engine.rbf_dense(X.double(), X[:k].double(), b[:k].double(), 1.0)
    assert rel_l2(out.cpu(), exact.cpu()) <= 1e-4
    with pytest.raises(AssertionError):
        engine.kmvm(X, X[:k], b, prm)                       # b has N rows, Y has k
    op = FFM(X, ls=1.0, min_points=300, nr_of_interpolation=64, small_field_points=64, device="cuda:0")
    full = op @ b
    chunked = op.chunk_forward_example(b, chunks=3)        # first chunk of Y is a leading slice of X
    assert rel_l2(chunked.cpu(), full.cpu()) <= 1e-4
    plan = engine.Plan(X, X[:k], prm)
    assert not plan.same and plan.M == k


@pytest.mark.parametrize("name,world", [("u3_shared", 3), ("clustered3", 4), ("n4_r8", 2), ("u3_xy", 2), ("u3_varcomp", 3), ("tiny", 2)])
def test_sharded_phases_equal_full_product(name, world, cuda):
    """The phases a multi-GPU product runs (slices of equal estimated work, moments of a share of the source boxes,
    direct sums that pack only the sources the slice's lists name, far field from the gathered moments), carried out
    for every "rank" in turn on one GPU: the assembled sorted result, put back into input order, must equal the
    single-call product."""
    from f3m_b200 import engine
    c = make_case(name)
    prm = engine.make_params(c["ls"], c["min_points"], c["P"], c["var_comp"], c["eff"], c["small"])
    X = c["X"].to(cuda)
    Y = None if c["Y"] is None else c["Y"].to(cuda)
    plan = engine.Plan(X, Y, prm)
    b = c["b"].to(cuda)
    R = b.shape[1]
    full = plan.apply(b)
    bounds = plan.partition_rows(R, world)
    assert bounds[0] == 0 and bounds[-1] == plan.N and all(a <= b_ for a, b_ in zip(bounds, bounds[1:]))
    L = plan.stats()["levels"]
    if L > 0:   # cuts lie on finest-level box starts
        starts = set(plan.array(L, 0, 1).tolist())      # F3M_ARR_BOX_OFFSETS of the target tree
        assert all(v in starts for v in bounds)
    msize = plan.moments_size(R)
    _, nby = plan.finest_boxes()
    mom_full, per_box, cb = None, 0, 0
    if msize > 0:
        per_box, cb = msize // nby, -(-nby // world)
        mom_full = torch.full((world * cb * per_box,), float("nan"), device=cuda)
        for r in range(world):      # what the all-gather delivers: every rank's slice at its place
            box_range = (min(nby, r * cb), min(nby, (r + 1) * cb))
            plan.shard_begin(b, (bounds[r], bounds[r + 1]), box_range, mom_full[r * cb * per_box:(r + 1) * cb * per_box])
            plan.shard_end()
        assert torch.isfinite(mom_full[:nby * per_box]).all()
        assert rel_l2(mom_full[:nby * per_box].cpu(), plan.moments(b, (0, plan.M)).cpu()) <= 1e-6
    acc = torch.full((plan.N, R), float("nan"), device=cuda)
    for r in range(world):
        box_range = (min(nby, r * cb), min(nby, (r + 1) * cb)) if msize > 0 else (0, 0)
        scratch = None if msize == 0 else torch.empty(cb * per_box, device=cuda)
        plan.shard_begin(b, (bounds[r], bounds[r + 1]), box_range, scratch)
        plan.shard_near(acc)
        plan.shard_far(mom_full, acc)
        plan.shard_end()
    assert torch.isfinite(acc).all()
    cut = plan.N // 3
    out = torch.cat([plan.rows_to_input_order(acc, 0, cut), plan.rows_to_input_order(acc, cut, plan.N)])
    assert rel_l2(out.cpu(), full.cpu()) <= 2e-6
    # the all-gather form: slices at a fixed stride, as the collective leaves them
    stride = max(bounds[r + 1] - bounds[r] for r in range(world))
    gathered = torch.full((world * stride, R), float("nan"), device=cuda)
    for r in range(world):
        gathered[r * stride:r * stride + bounds[r + 1] - bounds[r]] = acc[bounds[r]:bounds[r + 1]]
    assert torch.equal(plan.gathered_rows_to_input_order(gathered, bounds, stride, cut, plan.N), out[cut:])
    # the all-to-all form of the same step: every slice's rows grouped by the owner of the input row, then placed
    in_bounds = [0, plan.N // 5, plan.N // 2, plan.N][:world + 1] if world >= 3 else [0, plan.N // 3, plan.N]
    owners = len(in_bounds) - 1
    chunks = [[] for _ in range(owners)]
    for r in range(world):
        send, counts = plan.rows_by_owner(acc, (bounds[r], bounds[r + 1]), in_bounds)
        assert sum(counts) == bounds[r + 1] - bounds[r] == send.shape[0]
        pos = 0
        for q, c_ in enumerate(counts):
            chunks[q].append(send[pos:pos + c_])
            pos += c_
    for q in range(owners):
        recv = torch.cat(chunks[q]).contiguous()
        assert recv.shape[0] == in_bounds[q + 1] - in_bounds[q]
        placed = plan.place_rows(recv, in_bounds[q], in_bounds[q + 1])
        assert torch.equal(placed, out[in_bounds[q]:in_bounds[q + 1]])


def test_plan_is_deterministic(cuda):
    """Two plans of the same points hold the same permutation, bit for bit: ranks that build the plan on different GPUs
    exchange slices of the SORTED result, so the order inside a box must not depend on the run."""
    from f3m_b200 import engine, _lib
    g = torch.Generator().manual_seed(61)
    X = (torch.rand(400000, 3, generator=g) * 3).to(cuda)
    prm = engine.make_params(1.0, 200.0, 64, False, 0.15, 64)
    perms = []
    for _ in range(3):
        plan = engine.Plan(X, None, prm)
        perms.append(plan.array(0, 0, _lib.ARR_SORTED_INDEX))
        plan.close()
    assert np.array_equal(perms[0], perms[1]) and np.array_equal(perms[0], perms[2])
    assert np.array_equal(np.sort(perms[0]), np.arange(X.shape[0]))


@pytest.mark.parametrize("name", ["u3_shared", "n4_r8", "u2_shared", "clustered3"])
def test_plan_from_sorted_runs(name, cuda):
    """The sort shared by several ranks, carried out on one GPU: three uneven shards are sorted separately inside the
    global bounding cube, laid out as an all-gather would leave them (runs at a fixed stride, the short ones padded) and
    merged.  Boxes, centres and interaction lists must equal those of the plan built from all points at once, and so
    must the product (the two plans order the points inside a box differently)."""
    import numpy as np
    from f3m_b200 import engine, _lib
    c = make_case(name)
    prm = engine.make_params(c["ls"], c["min_points"], c["P"], c["var_comp"], c["eff"], c["small"])
    X = c["X"].to(cuda)
    b = c["b"].to(cuda)
    N, d = X.shape
    ref = engine.Plan(X, None, prm)
    full = ref.apply(b)
    cuts = [0, N // 5, N // 5 + N // 2, N]
    counts = [cuts[i + 1] - cuts[i] for i in range(3)]
    los, his = zip(*[engine.bounding_box(X[cuts[i]:cuts[i + 1]]) for i in range(3)])
    origin = np.min(np.array(los, dtype=np.float32), 0)
    top = np.max(np.array(his, dtype=np.float32), 0)
    edge0 = float(np.float32((top - origin).max()) * np.float32(1.01))
    assert abs(edge0 - ref.stats()["edge0"]) == 0.0
    depth = engine.sort_depth(N, d, c["min_points"])
    stride = max(counts)
    words = _lib.lib().f3m_record_words(d)
    recs_all = torch.zeros(3 * stride, words, device=cuda, dtype=torch.int32)
    cells = []
    for i in range(3):
        r, cnt = engine.sort_shard(X[cuts[i]:cuts[i + 1]], cuts[i], origin, edge0, prm.math_mode, depth)
        recs_all[i * stride:i * stride + counts[i]] = r
        assert int(cnt.sum()) == counts[i]
        cells.append(cnt)
    try:
        plan = engine.Plan.from_cell_counts(torch.stack(cells), d, origin, edge0, depth, prm)
    except _lib.F3MError as e:
        assert e.status == 5 and ref.stats()["levels"] > depth     # deeper than the estimate: the documented refusal
        return
    with pytest.raises(RuntimeError, match="sorted runs"):          # no product before the points are there
        plan.apply(b)
    plan.attach_runs(recs_all, stride)
    L = ref.stats()["levels"]
    assert plan.stats()["levels"] == L and plan.stats()["direct_pairs"] == ref.stats()["direct_pairs"]
    for l in range(1, L + 1):
        for what in (_lib.ARR_BOX_OFFSETS, _lib.ARR_BOX_CENTERS, _lib.ARR_BOX_CODES):
            assert np.array_equal(plan.array(l, 0, what), ref.array(l, 0, what))
        for cls in ("far", "small", "keep"):
            assert np.array_equal(plan.pairs(l, cls), ref.pairs(l, cls))
    perm = plan.array(0, 0, _lib.ARR_SORTED_INDEX)
    assert np.array_equal(np.sort(perm), np.arange(N))
    assert rel_l2(plan.apply(b).cpu(), full.cpu()) <= 2e-6


def test_product_in_a_caller_owned_workspace(cuda):
    """f3m_kmvm_ws_f32: every temporary comes out of a tensor the caller owns.  Same result as the allocating entry
    point; the driver's free memory does not move during the call; a workspace that is too small is a clean error; the
    size estimate covers evenly spread points, and the reported peak says how much was really used."""
    from f3m_b200 import engine, _lib
    g = torch.Generator().manual_seed(71)
    for (n, m, d, R, P) in ((300000, None, 3, 1, 64), (60000, 40000, 2, 3, 36), (50000, None, 4, 8, 81)):
        X = torch.rand(n, d, generator=g).to(cuda)
        Y = None if m is None else torch.rand(m, d, generator=g).to(cuda)
        b = torch.randn(n if m is None else m, R, generator=g).to(cuda)
        prm = engine.make_params(0.7, 300.0, P, False, 0.15, P)
        ref = engine.kmvm(X, Y, b, prm)
        need = engine.workspace_bytes(n, m or n, R, d, prm)
        ws = torch.empty(need, dtype=torch.uint8, device=cuda)
        engine.kmvm_ws(X, Y, b, prm, ws)                      # first use of the device may create the per-device slot
        torch.cuda.synchronize()
        free0 = torch.cuda.mem_get_info()[0]
        out = engine.kmvm_ws(X, Y, b, prm, ws)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free0           # nothing taken from or given back to the driver
        assert rel_l2(out.cpu(), ref.cpu()) <= 2e-6
        peak = engine.last_workspace_peak()
        assert 0 < peak <= need
        print(f"n={n} d={d} R={R}: workspace estimate {need / 1e6:.1f} MB, peak used {peak / 1e6:.1f} MB")
        small = torch.empty(max(4096, peak // 3), dtype=torch.uint8, device=cuda)
        with pytest.raises(_lib.F3MError) as e:
            engine.kmvm_ws(X, Y, b, prm, small)
        assert e.value.status == 7 and "workspace" in str(e.value)
        again = engine.kmvm_ws(X, Y, b, prm, ws)                # the failed call left nothing behind
        assert rel_l2(again.cpu(), ref.cpu()) <= 2e-6
