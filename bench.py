#!/usr/bin/env python
"""Benchmark of the F3M Gaussian KMVM hot path.

    python bench.py [--gpus N --steps K --warmup W] [--impl reference] [--workload c2|c3|c4]

One "step" is one complete kernel matrix-vector product out = K(X,X) b (bounding cube, sort, box
division, interaction lists, far field, near field).  Headline workload (c2, the default):
N = M = 1e8 points i.i.d. Uniform[0, sqrt(12)]^3 (float32, seed 1), b ~ N(0,1) with one column,
lengthscale 1, 216 interpolation nodes (6 per dimension), min_points 1000, small_field_points 216.
The data are synthetic (the reference's own sweeps draw the same distributions,
experiments/experiments.py:41-66).  Other workloads, not run by default: c3 = 10-component Gaussian
mixture (means U[-5,5]^3, std U[0.3,1]), lengthscale 0.5, 216 nodes (benchs_sparse/sparse_datasets.py:58-65
draws clustered data of this kind); c4 = N(0, I_d) in 4 or 5 dimensions with 8 columns.

Prints ONE JSON line.  `value` = N*M / seconds with inputs resident in HBM; `e2e` = the same through the
host-buffer path (host->device copies of X and b, device->host copy of the result inside the timed region).
N > 1 GPUs (torchrun): every rank starts with its 1/N shard of X and b and ends with the rows of the
product that belong to its shard (f3m_b200/parallel.py: all-gather of the points, tree on every rank,
slices of equal estimated work, moment exchange overlapped with the direct sums, all-to-all of the computed
rows to their owners); the time is the max over ranks.

--impl reference: the reference has no CPU implementation (its operator calls CUDA unconditionally,
experiments/FFM_classes.py:98-126); this arm times the CPU restatement of the reference algorithm
(oracle/f3m_oracle.py, PyTorch CPU ops on all host threads) on a bounded sample of the same workload.
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "gaussian_kmvm_interactions_per_s"
UNIT = "interactions/s"
SQRT12 = 12 ** 0.5


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c2", "c3", "c4"])
    ap.add_argument("--n", "--points", dest="n", type=float, default=None,
                    help="points (default: 1e8 for c2 and c3, 1e7 for c4); under torchrun write --points (its own parser claims --n)")
    ap.add_argument("--ls", type=float, default=None)
    ap.add_argument("--nodes", type=int, default=None, help="interpolation nodes per box (p^d)")
    ap.add_argument("--dim", type=int, default=None, help="c4: 4 or 5")
    ap.add_argument("--min-points", type=float, default=1000.)
    ap.add_argument("--cpu-sample", type=float, default=2e5, help="points of the CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the optional near-field modes and the reference GPU build")
    ap.add_argument("--check-rows", type=int, default=5000)
    a = ap.parse_args()
    w = a.workload
    a.d = {"c2": 3, "c3": 3, "c4": a.dim or 5}[w]
    a.R = 8 if w == "c4" else 1
    a.n = a.n if a.n is not None else (1e7 if w == "c4" else 1e8)
    a.ls = a.ls if a.ls is not None else {"c2": 1.0, "c3": 0.5, "c4": 1.0}[w]
    a.nodes = a.nodes if a.nodes is not None else {"c2": 216, "c3": 216, "c4": 3 ** a.d}[w]
    return a


def workload_name(a):
    if a.workload == "c2":
        return (f"C2: 3-D Gaussian KMVM X=Y, N=M={int(a.n):.0e} U[0,sqrt12]^3 f32, ls={a.ls:g}, "
                f"{a.nodes} nodes, min_points={a.min_points:g}, small_field_points={a.nodes}, var_compression=False")
    if a.workload == "c3":
        return (f"C3: 3-D clustered Gaussian KMVM X=Y, N=M={int(a.n):.0e} from a 10-component mixture (means U[-5,5]^3, std U[0.3,1]) f32, "
                f"ls={a.ls:g}, {a.nodes} nodes, min_points={a.min_points:g}, small_field_points={a.nodes}, var_compression=False")
    return (f"C4: {a.d}-D Gaussian KMVM X=Y, N=M={int(a.n):.0e} N(0,I) f32, {a.R} columns, ls={a.ls:g}, {a.nodes} nodes, "
            f"min_points={a.min_points:g}, small_field_points={a.nodes}, var_compression=False")


def draw_points(a, n, device, generator):
    """n points of the workload's distribution (and the same stream of random numbers on every rank)."""
    import torch
    if a.workload == "c2":
        return torch.empty(n, 3, device=device).uniform_(0, SQRT12, generator=generator)
    if a.workload == "c4":
        return torch.randn(n, a.d, device=device, generator=generator)
    gm = torch.Generator().manual_seed(7)     # the mixture itself is the same for every rank and every sample
    means = (torch.rand(10, 3, generator=gm) * 10 - 5).to(device)
    std = (torch.rand(10, generator=gm) * 0.7 + 0.3).to(device)
    comp = torch.randint(0, 10, (n,), device=device, generator=generator)
    X = torch.randn(n, 3, device=device, generator=generator)
    X.mul_(std[comp, None]).add_(means[comp])
    return X


# ------------------------------------------------------------------------------------------------
# CPU arm (checker code timed as the baseline; never on the product path)
# ------------------------------------------------------------------------------------------------
def cpu_sample_run(a, steps, warmup):
    import torch
    from oracle.f3m_oracle import f3m_kmvm
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    ns = int(a.cpu_sample)
    g = torch.Generator().manual_seed(1)
    X = draw_points(a, ns, "cpu", g)
    b = torch.randn(ns, a.R, generator=g)
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        f3m_kmvm(X, None, b, a.ls, a.min_points, a.nodes, False, 0.15, a.nodes)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    t = statistics.median(times)
    n_full = float(a.n)
    # the treecode is O(N) at fixed leaf occupancy: time for the full workload ~ t * N/ns
    value = n_full * n_full * a.R / (t * n_full / ns)
    return dict(value=value, unit=UNIT, cores=cores, kind="port",
                sample=(f"oracle/f3m_oracle.py (PyTorch CPU, {cores} threads) on {ns} points of the same distribution and "
                        f"parameters: {t:.2f} s per product = {ns * ns * a.R / t:.3e} interactions/s on the sample; value is "
                        f"extrapolated linearly in N to the {int(n_full):.0e}-point workload")), t


def reference_gpu_run(n=1e7, nodes=216):
    """The UNMODIFIED reference built for sm_100a (oracle/_ref/f3m_ref_d3.so), timed on this GPU in a child process at
    the size it is known to complete at.  Checker code: runs outside every timed region, never on the product path."""
    so = os.path.join(ROOT, "oracle", "_ref", "f3m_ref_d3.so")
    if not os.path.exists(so):
        return {"skipped": "oracle/_ref/f3m_ref_d3.so is not built on this machine"}
    try:
        p = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "time_reference_gpu.py"), str(n), "--nodes", str(nodes),
                            "--reps", "2"], capture_output=True, text=True, timeout=600)
        for line in p.stdout.splitlines():
            if line.startswith("{"):
                r = json.loads(line)
                return {"n": r["N"], "nodes": nodes, "s_per_kmvm": r["s_per_kmvm"], "interactions_per_s": r["interactions_per_s"],
                        "what": "unmodified reference sources compiled for sm_100a, FFM_XY<float,3>, same distribution and parameters"}
        return {"skipped": "the reference build printed no result: " + (p.stderr or p.stdout)[-300:].replace("\n", " ")}
    except Exception as e:   # noqa: BLE001 - a checker that cannot run is reported, not fatal
        return {"skipped": f"{type(e).__name__}: {e}"}


def run_reference_arm(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, min(a.steps, 3)), min(a.warmup, 1)
    cb, t = cpu_sample_run(a, steps, warmup)
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": a.gpus, "steps": steps,
            "warmup": warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(a),
                       "sample": f"each step runs the CPU restatement on {int(a.cpu_sample)} points of the workload; "
                                 f"value is that rate extrapolated linearly in N to {int(a.n):.0e} points"},
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
            "note": "reference has no CPU path; CPU restatement of its algorithm timed on a bounded sample"}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                       "-i", str(gpu_index)], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        if self.p is None:
            return None
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        for line in self.f.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.f.name)
        if not sm:
            return None
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def rel_l2_on_sample(out_rows, X_rows, X_all, b_all, ls, engine):
    """(sum of squared differences, sum of squares) of out_rows against the float64 dense product of those rows."""
    exact = engine.rbf_dense(X_rows.double(), X_all.double(), b_all.double(), ls)
    return float((out_rows.double() - exact).pow(2).sum()), float(exact.pow(2).sum())


def main():
    a = parse()
    if a.impl == "reference":
        run_reference_arm(a)
        return
    import torch
    import torch.distributed as dist
    from f3m_b200 import engine
    from f3m_b200.parallel import distributed_kmvm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    N, d, R = int(a.n), a.d, a.R
    prm = engine.make_params(a.ls, a.min_points, a.nodes, False, 0.15, a.nodes)

    # synthetic workload: rank r draws shard r of the same data set at every world size (seed = f(r, world) would change
    # the data with N; instead the whole set is drawn shard by shard from one seeded stream and only the own shard is kept)
    g = torch.Generator(device=dev).manual_seed(1)
    lo, hi = rank * N // world, (rank + 1) * N // world
    if world == 1 or N * (d + R) * 4 <= 8e9:
        X = draw_points(a, N, dev, g)
        b = torch.randn(N, R, device=dev, generator=g)
        Xs, bs = X[lo:hi].clone(), b[lo:hi].clone()
        if world > 1:
            del X, b
    else:   # too large to draw whole on every rank: per-rank streams (the set then depends on the world size)
        g = torch.Generator(device=dev).manual_seed(1 + rank)
        Xs = draw_points(a, hi - lo, dev, g)
        bs = torch.randn(hi - lo, R, device=dev, generator=g)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    state = {}

    def step(stats=None):
        if world == 1:
            state["out"] = engine.kmvm(Xs, None, bs, prm)
        else:
            state["out"] = distributed_kmvm(Xs, bs, prm, stats=stats)

    for _ in range(a.warmup):
        step()
    barrier()
    launches0 = engine.launch_count()
    sampler = ClockSampler(local) if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(a.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler else None
    launches = engine.launch_count() - launches0
    tmax = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    ms = float(tmax.item())
    ms_per_step = ms / a.steps
    value = float(N) * float(N) * R / (ms_per_step * 1e-3)

    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": workload_name(a), "l2": f"inputs ({N * (d + R) * 4 / 1e9:.1f} GB) larger than L2; no flush needed",
                       "parallelism": "1 GPU" if world == 1 else
                       f"{world} GPUs: all-gather of the points, tree on every rank, target rows cut into slices of equal estimated "
                       f"work, moment exchange overlapped with the direct sums, every rank ends with the rows of its own shard"},
            "gpu_launches": int(launches), "clocks": clocks}

    if world > 1:
        # ---- one more product outside the timed region: phase times (max over ranks), balance, error on sampled rows ----
        stats = {}
        step(stats)
        names = ["cube", "sort_shard", "levels_lists", "merge_runs", "gather_points", "tree_lists", "partition", "sources_moments", "direct_sums", "far_field", "pack_rows", "exchange_rows", "own_rows"]
        t = torch.tensor([stats.get(k, 0.0) for k in names], device=dev, dtype=torch.float64)
        tm = t.clone()
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        line["stages_ms"] = {k: round(float(v), 3) for k, v in zip(names, tm)}
        line["stages_note"] = ("device time between marks on each rank's stream, max over ranks; the moment all-gather runs beside "
                               "direct_sums, the all-gather of b beside tree_lists")
        work = torch.tensor([stats.get("direct_sums", 0.0) + stats.get("far_field", 0.0)], device=dev, dtype=torch.float64)
        wmax, wsum = work.clone(), work.clone()
        dist.all_reduce(wmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(wsum, op=dist.ReduceOp.SUM)
        line["imbalance_max_over_mean"] = round(float(wmax) / (float(wsum) / world), 4)
        rows_t = torch.tensor([float(stats.get("slice_rows", 0))], device=dev, dtype=torch.float64)
        rows_all = [torch.zeros_like(rows_t) for _ in range(world)]
        dist.all_gather(rows_all, rows_t)
        line["slice_rows"] = [int(v.item()) for v in rows_all]
        # error: every rank checks check_rows / world rows of its own shard against the float64 dense product
        n_check = max(1, a.check_rows // world)
        torch.cuda.empty_cache()
        engine.release_cached_memory()
        Xall = torch.empty(N, d, device=dev)
        ball = torch.empty(N, R, device=dev)
        counts = [(r + 1) * N // world - r * N // world for r in range(world)]
        dist.all_gather(list(Xall.split(counts)), Xs)
        dist.all_gather(list(ball.split(counts)), bs)
        rows = torch.randperm(hi - lo, device=dev, generator=g)[:n_check]
        num, den = rel_l2_on_sample(state["out"][rows], Xs[rows], Xall, ball, a.ls, engine)
        nd = torch.tensor([num, den], device=dev, dtype=torch.float64)
        dist.all_reduce(nd)
        line["rel_l2_vs_f64"] = float((nd[0] / nd[1]).sqrt())
        line["rel_l2_rows"] = n_check * world
        del Xall, ball

    if rank == 0 and world == 1:
        # ---- stage times, roofline of the dominant kernel (direct sums), accuracy ------------------------------
        plan = engine.Plan(Xs, None, prm)
        out = plan.apply(bs)
        st, tm = plan.stats(), plan.timings()
        tms = [tm]
        for _ in range(2):
            plan.apply(bs)
            tms.append(plan.timings())
        direct_ms = statistics.median(t["direct"] for t in tms)
        variants = plan.direct_variants()
        peaks = engine.measure_peaks(dev)
        flop_per_pair = 3 * d + 2 * R                      # 3d + 2R
        # The direct-sum kernel (near_kernel_x2) spends per pair d multiply-adds on the inner product, R on the
        # accumulation and either one exponential (MUFU) or a degree-DEG polynomial (DEG multiply-adds) -- the share of
        # polynomial pairs and the degree follow the rule in near.cu (direct_impl): same bound on the exponent here.
        Lv = st["levels"]
        edge = plan.level(Lv)["edge"] if Lv else 0.0
        se = math.sqrt(math.log2(math.e) / (2.0 * a.ls * a.ls)) * edge
        h = d * 2.5 * se * se * math.log(2.0)
        deg, share = (2, 2 / 5) if h ** 3 / 24 <= 3e-7 else ((3, 1 / 3) if h ** 4 / 192 <= 3e-7 else (0, 0.0))
        fma_per_pair = d + R + share * deg
        exp_per_pair = 1.0 - share
        peak_pairs = min(peaks["gfma_per_s"] / fma_per_pair, peaks["gexp_per_s"] / exp_per_pair) * 1e9
        achieved_pairs = st["direct_pairs"] / (direct_ms * 1e-3)
        sm_mhz = (clocks or {}).get("sm_mhz") or 1965.0
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        roof = {"bound": "fp32-fma+sfu", "bound_note": "not hbm, not tensor in the default path: inner product + exponential per pair; a source row is reused by every target of a tile",
                "achieved": achieved_pairs * flop_per_pair / 1e12, "peak": peak_pairs * flop_per_pair / 1e12,
                "unit": "TFLOP/s", "frac": achieved_pairs / peak_pairs,
                "kernel": f"near_kernel_x2<{d},{R if R == 1 else 8},{deg},..> (all direct-sum launches of one product; packed f32x2 arithmetic over source pairs; "
                          f"{share:.2f} of the pairs evaluate 2^t by a degree-{deg} polynomial on the FMA pipe)",
                "pairs": st["direct_pairs"], "ms": direct_ms, "launches": tm["direct_launches"], "kernel_forms": variants,
                "peak_source": f"measured in this run by register-only probes: {peaks['gexp_per_s']:.0f} Gexp/s, "
                               f"{peaks['gfma_per_s']:.0f} Gfma/s; peak = min(fma/{fma_per_pair:.2f}, exp/{exp_per_pair:.2f}) pairs/s x {flop_per_pair} flop",
                # the probe reads a little under lanes x SMs x clock; with that number as the FMA peak the fraction is:
                "fma_peak_theoretical_gfma": 128 * sms * sm_mhz * 1e-3,
                "frac_vs_theoretical_fma": achieved_pairs / (min(128 * sms * sm_mhz * 1e-3 / fma_per_pair,
                                                                  peaks["gexp_per_s"] / exp_per_pair) * 1e9)}
        if a.workload == "c2":
            # DRAM bytes per launch from an ncu capture of this kernel at N=1e7 (profiles/near_kernel_x2_c2_1e7.md), scaled by
            # N: the traffic is per point (packed sources, targets, output)
            roof["traffic"] = 37.7 * N
            roof["traffic_note"] = "37.7 B/point from the ncu capture at N=1e7, scaled to N; algorithmic minimum 36 B/point"
        else:
            roof["traffic"] = None
        line["roofline"] = roof
        line["stages_ms"] = {k: round(v, 3) for k, v in tm.items() if k != "direct_launches"}
        # ---- per-stage rooflines from the algorithmic work (bytes against the measured copy bandwidth, multiply-adds
        # against the FMA peak measured above); the slower of the two is the stage's bound ------------------------------
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
                hbm_gbs, hbm_src = float(json.load(fh)["hbm_gbs"]), "of measured"
        except Exception:
            hbm_gbs, hbm_src = 6650.0, "of fallback"
        if Lv:
            nb_leaf = plan.level(Lv)["boxes_x"]
            pd = plan.level(Lv)["nodes_per_dim"]
            Pn = pd ** d
            fma_s = peaks["gfma_per_s"] * 1e9

            def stage_roof(ms_, nbytes, fmas):
                t_b, t_f = nbytes / (hbm_gbs * 1e9) * 1e3, fmas / fma_s * 1e3
                return {"ms": round(ms_, 3), "hbm_roof_ms": round(t_b, 3), "fma_roof_ms": round(t_f, 3),
                        "frac": round(max(t_b, t_f) / ms_, 3) if ms_ > 0 else None}
            line["stages_roofline"] = {
                "hbm_peak_gbs": hbm_gbs, "hbm_peak": hbm_src,
                "tree+lists": stage_roof(tm["build"], N * (2 * 4 * d + 2 * 4 * R + 8), 0),   # sort traffic: 40 B/point at d=3, R=1
                "p2m": stage_roof(tm["p2m"], N * (4 * d + 4 * R) + nb_leaf * Pn * R * 4, N * Pn * R),
                "m2l": stage_roof(tm["m2l"], 2 * nb_leaf * Pn * R * 4, st["far_box_pairs"] * d * pd * Pn * R),
                "l2p": stage_roof(tm["l2p"], N * (4 * d + 8 * R) + nb_leaf * Pn * R * 4, N * Pn * R),
                "direct": {"ms": round(direct_ms, 3), "frac": round(achieved_pairs / peak_pairs, 3)},
                "note": "m2l multiply-adds counted in the per-pair form (d axis transforms per far pair); the nested kernel does fewer"}
        line["work"] = {"levels": st["levels"], "direct_pairs": st["direct_pairs"], "far_box_pairs": st["far_box_pairs"],
                        "node_pairs_reference_form": st["node_pairs"]}
        rows = torch.randperm(N, device=dev, generator=g)[:a.check_rows]
        num, den = rel_l2_on_sample(out[rows], Xs[rows], Xs, bs, a.ls, engine)
        line["rel_l2_vs_f64"] = math.sqrt(num / den)
        plan.close()
        if not a.no_extras and a.workload == "c2":
            exact = engine.rbf_dense(Xs[rows].double(), Xs.double(), bs.double(), a.ls)
            from f3m_b200 import _lib as f3m_lib

            def mode_run(flags):
                prm_m = engine.make_params(a.ls, a.min_points, a.nodes, False, 0.15, a.nodes, flags=flags)
                for _ in range(2):
                    out_m = engine.kmvm(Xs, None, bs, prm_m)
                torch.cuda.synchronize()
                e0.record()
                for _ in range(a.steps):
                    out_m = engine.kmvm(Xs, None, bs, prm_m)
                e1.record()
                torch.cuda.synchronize()
                ms_m = e0.elapsed_time(e1) / a.steps
                return {"ms_per_step": ms_m, "value": float(N) * float(N) * R / (ms_m * 1e-3), "unit": UNIT,
                        "rel_l2_vs_f64": float((out_m[rows].double() - exact).norm() / exact.norm())}
            # ---- the same product with the optional forms of the near field (not the headline: `value` above is the
            # default path, whose near field is the direct sum on the CUDA cores) ----------------------------------------
            line["near_moments_mode"] = dict(mode_run(f3m_lib.FLAG_NEAR_MOMENTS),
                                             note="F3M_FLAG_NEAR_MOMENTS: near sums from 2nd/3rd-order box moments where the exponent "
                                                  "is provably tiny; same pair lists; optional, off by default")
            line["near_tensor_cores_mode"] = dict(mode_run(f3m_lib.FLAG_NEAR_TENSOR_CORES),
                                                  note="F3M_FLAG_NEAR_TENSOR_CORES: exponent tiles as TF32 tcgen05 products of split operands "
                                                       "(TMEM accumulators, bulk copies, mbarrier pipeline); optional, off by default")
            del exact
        # ---- end to end through the host-buffer entry point ------------------------------------------------------
        Xh = torch.empty(N, d, pin_memory=True).copy_(Xs)
        bh = torch.empty(N, R, pin_memory=True).copy_(bs)
        oh = torch.empty(N, R, pin_memory=True)
        del Xs, bs, out
        torch.cuda.empty_cache()
        for _ in range(1):
            engine.kmvm_host(Xh, None, bh, prm, out=oh)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        e0.record()
        for _ in range(a.steps):
            engine.kmvm_host(Xh, None, bh, prm, out=oh)
        e1.record()
        torch.cuda.synchronize()
        e2e_ms = max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3) / a.steps
        line["e2e"] = {"value": float(N) * float(N) * R / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                       "h2d_bytes_per_step": N * d * 4 + N * R * 4, "d2h_bytes_per_step": N * R * 4,
                       "api": "f3m_kmvm_host_f32 (pinned host tensors)"}
        del Xh, bh, oh
        if not a.no_extras and a.workload == "c2":
            # the reference's own CUDA code on this GPU, at the size it is known to complete at, and this engine at that size
            ref_gpu = reference_gpu_run(1e7, a.nodes)
            if "s_per_kmvm" in ref_gpu:
                n7 = int(ref_gpu["n"])
                g7 = torch.Generator(device=dev).manual_seed(1)
                X7 = torch.empty(n7, 3, device=dev).uniform_(0, SQRT12, generator=g7)
                b7 = torch.randn(n7, 1, device=dev, generator=g7)
                for _ in range(2):
                    engine.kmvm(X7, None, b7, prm)
                torch.cuda.synchronize()
                e0.record()
                for _ in range(5):
                    engine.kmvm(X7, None, b7, prm)
                e1.record()
                torch.cuda.synchronize()
                ref_gpu["engine_s_same_n"] = e0.elapsed_time(e1) / 5 * 1e-3
                ref_gpu["engine_over_reference"] = ref_gpu["s_per_kmvm"] / ref_gpu["engine_s_same_n"]
            line["reference_gpu"] = ref_gpu
        if not a.no_cpu_baseline:
            line["cpu_baseline"], _ = cpu_sample_run(a, 1, 0)
    if world > 1:
        # ---- end to end at N GPUs: host shard -> device, product, own rows -> host, every step --------------------
        Xh = torch.empty(hi - lo, d, pin_memory=True).copy_(Xs)
        bh = torch.empty(hi - lo, R, pin_memory=True).copy_(bs)
        oh = torch.empty(hi - lo, R, pin_memory=True)

        def e2e_step():
            xd = Xh.to(dev, non_blocking=True)
            bd = bh.to(dev, non_blocking=True)
            out = distributed_kmvm(xd, bd, prm)
            oh.copy_(out, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        e2e_step()
        barrier()
        e0.record()
        for _ in range(a.steps):
            e2e_step()
        e1.record()
        barrier()
        t2 = torch.tensor([e0.elapsed_time(e1)], device=dev)
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        e2e_ms = float(t2.item()) / a.steps
        line["e2e"] = {"value": float(N) * float(N) * R / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                       "h2d_bytes_per_step": N * d * 4 + N * R * 4, "d2h_bytes_per_step": N * R * 4,
                       "api": "pinned host shards -> f3m_b200.parallel.distributed_kmvm -> pinned host rows of the shard (bytes summed over ranks)"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
