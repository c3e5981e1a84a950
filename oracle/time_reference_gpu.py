"""TEST INFRASTRUCTURE ONLY.  Times the UNMODIFIED reference (oracle/_ref/f3m_ref_d3.so, built by
oracle/Makefile from the reference's own sources for sm_100a) on the GPU of this machine, on the
benchmark's distribution, and prints one JSON line per size.  Used to put the reference's own GPU
speed on a B200 beside the engine's; nothing in the product imports this.

    python oracle/time_reference_gpu.py [N ...]  [--nodes 216] [--min-points 1000]
"""
import argparse
import importlib.util
import json
import os
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_reference(d=3):
    path = os.path.join(ROOT, "oracle", "_ref", f"f3m_ref_d{d}.so")
    spec = importlib.util.spec_from_file_location(f"f3m_ref_d{d}", path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    return ref


def time_reference(n, nodes=216, min_points=1000., ls=1.0, reps=3, dev="cuda:0"):
    """Median seconds of FFM_XY<float,3> (F3M_src/n_tree.cu:1056-1125) on n points of the benchmark's distribution."""
    ref = load_reference(3)
    n = int(n)
    g = torch.Generator(device=dev).manual_seed(1)
    X = torch.empty(n, 3, device=dev).uniform_(0, 12 ** 0.5, generator=g)
    b = torch.randn(n, 1, device=dev, generator=g)
    times = []
    for it in range(reps + 1):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = ref.FFM_XY_FLOAT(X, X, b, dev, ls, min_points, nodes, False, 0.15, nodes)
        torch.cuda.synchronize()
        if it:
            times.append(time.perf_counter() - t0)
    t = sorted(times)[len(times) // 2]
    return {"impl": "reference build for sm_100a (GPU)", "N": n, "nodes": nodes, "min_points": min_points, "ls": ls,
            "s_per_kmvm": t, "interactions_per_s": float(n) * n / t, "checksum": float(out.double().sum())}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("n", nargs="*", type=float, default=[1e6])
    ap.add_argument("--nodes", type=int, default=216)
    ap.add_argument("--min-points", type=float, default=1000.)
    ap.add_argument("--ls", type=float, default=1.0)
    ap.add_argument("--reps", type=int, default=3)
    a = ap.parse_args()
    for n in a.n:
        print(json.dumps(time_reference(n, a.nodes, a.min_points, a.ls, a.reps)), flush=True)
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
