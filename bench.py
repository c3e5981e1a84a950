#!/usr/bin/env python
"""Benchmark of the F3M Gaussian KMVM hot path.

    python bench.py [--gpus N --steps K --warmup W] [--impl reference]

One "step" is one complete kernel matrix-vector product out = K(X,X) b (bounding cube, sort, box
division, interaction lists, far field, near field) on the headline workload:
N = M = 1e8 points i.i.d. Uniform[0, sqrt(12)]^3 (float32, seed 1), b ~ N(0,1) with one column,
lengthscale 1, 216 interpolation nodes (6 per dimension), min_points 1000, small_field_points 216.
The data are synthetic (the reference's own sweeps draw the same distributions,
experiments/experiments.py:41-66).

Prints ONE JSON line.  `value` = N*M*R / seconds with inputs resident in HBM; `e2e` = the same through
the host-buffer C-ABI call (host->device copies of X and b, device->host copy of the result inside the
timed region).  N > 1 GPUs (torchrun): every rank starts with its 1/N shard of X and b, the shards are
all-gathered over NCCL, every rank builds the tree and computes the target boxes of its slice of the
sorted order, and the output slices are summed with an all-reduce; the time is the max over ranks.

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
    ap.add_argument("--n", type=float, default=1e8, help="points (default: the headline 1e8)")
    ap.add_argument("--ls", type=float, default=1.0)
    ap.add_argument("--nodes", type=int, default=216, help="interpolation nodes per box (p^3)")
    ap.add_argument("--min-points", type=float, default=1000.)
    ap.add_argument("--cpu-sample", type=float, default=2e5, help="points of the CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--check-rows", type=int, default=5000)
    return ap.parse_args()


def workload_name(a):
    return (f"C2: 3-D Gaussian KMVM X=Y, N=M={int(a.n):.0e} U[0,sqrt12]^3 f32, ls={a.ls:g}, "
            f"{a.nodes} nodes, min_points={a.min_points:g}, small_field_points={a.nodes}, var_compression=False")


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
    X = torch.rand(ns, 3, generator=g) * SQRT12
    b = torch.randn(ns, 1, generator=g)
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
    value = n_full * n_full / (t * n_full / ns)
    return dict(value=value, unit=UNIT, cores=cores, kind="port",
                sample=(f"oracle/f3m_oracle.py (PyTorch CPU, {cores} threads) on {ns} points of the same distribution and "
                        f"parameters: {t:.2f} s per product = {ns * ns / t:.3e} interactions/s on the sample; value is "
                        f"extrapolated linearly in N to the {int(n_full):.0e}-point workload")), t


def run_reference_arm(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, min(a.steps, 3)), min(a.warmup, 1)
    cb, t = cpu_sample_run(a, steps, warmup)
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": a.gpus, "steps": steps,
            "warmup": warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": workload_name(a)}, "cpu_baseline": cb,
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
    N = int(a.n)
    prm = engine.make_params(a.ls, a.min_points, a.nodes, False, 0.15, a.nodes)

    # synthetic workload: every rank draws the same full arrays from the seed and keeps its shard
    g = torch.Generator(device=dev).manual_seed(1)
    X = torch.empty(N, 3, device=dev).uniform_(0, SQRT12, generator=g)
    b = torch.randn(N, 1, device=dev, generator=g)
    lo, hi = rank * N // world, (rank + 1) * N // world
    Xs, bs = X[lo:hi].clone(), b[lo:hi].clone()
    if world > 1:
        del X, b

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    state = {}

    def step():
        if world == 1:
            out = engine.kmvm(Xs, None, bs, prm)
            state["out"] = out
            return
        # all-gather sources over NVLink, build the tree, compute the target boxes of this rank's slice of
        # the sorted order, all-reduce the output slices (f3m_b200/parallel.py)
        state["out"] = distributed_kmvm(Xs, bs, prm)

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
    value = float(N) * float(N) / (ms_per_step * 1e-3)

    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": workload_name(a), "l2": "inputs (1.6 GB) larger than L2; no flush needed",
                       "parallelism": "1 GPU" if world == 1 else f"{world} GPUs: all-gather sources, target boxes sharded by sorted row range, all-reduce output"},
            "gpu_launches": int(launches), "clocks": clocks}

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
        peaks = engine.measure_peaks(dev)
        d_ = 3
        flop_per_pair = 3 * d_ + 2 * 1                      # 3d + 2R
        # The direct-sum kernel (near_kernel_x2) spends per pair d multiply-adds on the inner product, one on the
        # accumulation and either one exponential (MUFU) or a degree-DEG polynomial (DEG multiply-adds) -- the share of
        # polynomial pairs and the degree follow the rule in near.cu (direct_impl): same bound on the exponent here.
        edge = plan.level(st["levels"])["edge"]
        se = math.sqrt(math.log2(math.e) / (2.0 * a.ls * a.ls)) * edge
        h = d_ * 2.5 * se * se * math.log(2.0)
        deg, share = (2, 2 / 5) if h ** 3 / 24 <= 3e-7 else ((3, 1 / 3) if h ** 4 / 192 <= 3e-7 else (0, 0.0))
        fma_per_pair = d_ + 1 + share * deg
        exp_per_pair = 1.0 - share
        peak_pairs = min(peaks["gfma_per_s"] / fma_per_pair, peaks["gexp_per_s"] / exp_per_pair) * 1e9
        achieved_pairs = st["direct_pairs"] / (direct_ms * 1e-3)
        line["roofline"] = {"bound": "fp32-fma+sfu", "bound_note": "not hbm, not tensor in the default path: inner product + exponential per pair; a source row is reused by every target of a tile",
                            "achieved": achieved_pairs * flop_per_pair / 1e12, "peak": peak_pairs * flop_per_pair / 1e12,
                            "unit": "TFLOP/s", "frac": achieved_pairs / peak_pairs,
                            # DRAM bytes per launch from an ncu capture of this kernel at N=1e7, scaled by N: the traffic is
                            # per point (packed sources, targets, output)
                            "traffic": 37.7 * N, "traffic_note": "37.7 B/point from the ncu capture at N=1e7, scaled to N; algorithmic minimum 36 B/point",
                            "kernel": f"near_kernel_x2<3,1,{deg},..> (all direct-sum launches of one product; packed f32x2 arithmetic over source pairs; "
                                      f"{share:.2f} of the pairs evaluate 2^t by a degree-{deg} polynomial on the FMA pipe)",
                            "pairs": st["direct_pairs"], "ms": direct_ms, "launches": tm["direct_launches"],
                            "peak_source": f"measured in this run by register-only probes: {peaks['gexp_per_s']:.0f} Gexp/s, "
                                           f"{peaks['gfma_per_s']:.0f} Gfma/s; peak = min(fma/{fma_per_pair:.2f}, exp/{exp_per_pair:.2f}) pairs/s x {flop_per_pair} flop"}
        line["stages_ms"] = {k: round(v, 3) for k, v in tm.items() if k != "direct_launches"}
        # ---- per-stage rooflines from the algorithmic work (bytes against the measured copy bandwidth, multiply-adds
        # against the FMA peak measured above); the slower of the two is the stage's bound ------------------------------
        try:
            with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")) as fh:
                hbm_gbs, hbm_src = float(json.load(fh)["hbm_gbs"]), "of measured"
        except Exception:
            hbm_gbs, hbm_src = 6650.0, "of fallback"
        nb_leaf = plan.level(st["levels"])["boxes_x"]
        Pn = plan.level(st["levels"])["nodes_per_dim"] ** d_
        fma_s = peaks["gfma_per_s"] * 1e9
        def stage_roof(ms, nbytes, fmas):
            t_b, t_f = nbytes / (hbm_gbs * 1e9) * 1e3, fmas / fma_s * 1e3
            return {"ms": round(ms, 3), "hbm_roof_ms": round(t_b, 3), "fma_roof_ms": round(t_f, 3), "frac": round(max(t_b, t_f) / ms, 3)}
        line["stages_roofline"] = {
            "hbm_peak_gbs": hbm_gbs, "hbm_peak": hbm_src,
            "tree+lists": stage_roof(tm["build"], N * (2 * 4 * d_ + 2 * 4 + 8), 0),        # sort traffic: 40 B/point at d=3, R=1
            "p2m": stage_roof(tm["p2m"], N * (4 * d_ + 4) + nb_leaf * Pn * 4, N * Pn),
            "m2l": stage_roof(tm["m2l"], 2 * nb_leaf * Pn * 4, st["far_box_pairs"] * d_ * plan.level(st["levels"])["nodes_per_dim"] * Pn),
            "l2p": stage_roof(tm["l2p"], N * (4 * d_ + 8) + nb_leaf * Pn * 4, N * Pn),
            "direct": {"ms": round(direct_ms, 3), "frac": round(achieved_pairs / peak_pairs, 3)},
            "note": "m2l multiply-adds counted in the per-pair form (d axis transforms per far pair); the nested kernel does fewer"}
        line["work"] = {"levels": st["levels"], "direct_pairs": st["direct_pairs"], "far_box_pairs": st["far_box_pairs"],
                        "node_pairs_reference_form": st["node_pairs"]}
        rows = torch.randperm(N, device=dev, generator=g)[:a.check_rows]
        exact = engine.rbf_dense(Xs[rows].double(), Xs.double(), bs.double(), a.ls)
        line["rel_l2_vs_f64"] = float((out[rows].double() - exact).norm() / exact.norm())
        plan.close()
        # ---- the same product with the optional moment form of the near field (not the headline: `value` above is
        # the default path, whose near field is the direct sum) ---------------------------------------------------
        from f3m_b200 import _lib as f3m_lib
        prm_m = engine.make_params(a.ls, a.min_points, a.nodes, False, 0.15, a.nodes, flags=f3m_lib.FLAG_NEAR_MOMENTS)
        for _ in range(2):
            out_m = engine.kmvm(Xs, None, bs, prm_m)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(a.steps):
            out_m = engine.kmvm(Xs, None, bs, prm_m)
        e1.record()
        torch.cuda.synchronize()
        ms_m = e0.elapsed_time(e1) / a.steps
        line["near_moments_mode"] = {"ms_per_step": ms_m, "value": float(N) * float(N) / (ms_m * 1e-3), "unit": UNIT,
                                     "rel_l2_vs_f64": float((out_m[rows].double() - exact).norm() / exact.norm()),
                                     "note": "F3M_FLAG_NEAR_MOMENTS: near sums from 2nd/3rd-order box moments where the exponent "
                                             "is provably tiny; same pair lists; optional, off by default"}
        # ---- and with the optional tcgen05 form of the near sums (same sums, exponent tiles from the tensor cores) -----
        prm_t = engine.make_params(a.ls, a.min_points, a.nodes, False, 0.15, a.nodes, flags=f3m_lib.FLAG_NEAR_TENSOR_CORES)
        for _ in range(2):
            out_t = engine.kmvm(Xs, None, bs, prm_t)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(a.steps):
            out_t = engine.kmvm(Xs, None, bs, prm_t)
        e1.record()
        torch.cuda.synchronize()
        ms_t = e0.elapsed_time(e1) / a.steps
        line["near_tensor_cores_mode"] = {"ms_per_step": ms_t, "value": float(N) * float(N) / (ms_t * 1e-3), "unit": UNIT,
                                          "rel_l2_vs_f64": float((out_t[rows].double() - exact).norm() / exact.norm()),
                                          "note": "F3M_FLAG_NEAR_TENSOR_CORES: exponent tiles as TF32 tcgen05 products of split operands "
                                                  "(TMEM accumulators, bulk copies, mbarrier pipeline); optional, off by default"}
        del exact, out_m, out_t
        # ---- end to end through the host-buffer entry point ------------------------------------------------------
        Xh = torch.empty(N, 3, pin_memory=True).copy_(Xs)
        bh = torch.empty(N, 1, pin_memory=True).copy_(bs)
        oh = torch.empty(N, 1, pin_memory=True)
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
        line["e2e"] = {"value": float(N) * float(N) / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                       "h2d_bytes_per_step": N * 3 * 4 + N * 4, "d2h_bytes_per_step": N * 4,
                       "api": "f3m_kmvm_host_f32 (pinned host tensors)"}
        if not a.no_cpu_baseline:
            line["cpu_baseline"], _ = cpu_sample_run(a, 1, 0)
    if world > 1:
        # ---- end to end at N GPUs: host shard -> device, product, own output slice -> host, every step ------------
        Xh = torch.empty(hi - lo, 3, pin_memory=True).copy_(Xs)
        bh = torch.empty(hi - lo, 1, pin_memory=True).copy_(bs)
        oh = torch.empty(hi - lo, 1, pin_memory=True)

        def e2e_step():
            xd = Xh.to(dev, non_blocking=True)
            bd = bh.to(dev, non_blocking=True)
            out = distributed_kmvm(xd, bd, prm)
            oh.copy_(out[lo:hi], non_blocking=True)
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
        line["e2e"] = {"value": float(N) * float(N) / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                       "h2d_bytes_per_step": N * 3 * 4 + N * 4, "d2h_bytes_per_step": N * 4,
                       "api": "pinned host shards -> f3m_b200.parallel.distributed_kmvm -> pinned host slice (bytes summed over ranks)"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
