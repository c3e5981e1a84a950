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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("n", nargs="*", type=float, default=[1e6])
    ap.add_argument("--nodes", type=int, default=216)
    ap.add_argument("--min-points", type=float, default=1000.)
    ap.add_argument("--ls", type=float, default=1.0)
    ap.add_argument("--reps", type=int, default=3)
    a = ap.parse_args()
    path = os.path.join(ROOT, "oracle", "_ref", "f3m_ref_d3.so")
    spec = importlib.util.spec_from_file_location("f3m_ref_d3", path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    dev = "cuda:0"
    for n in a.n:
        n = int(n)
        g = torch.Generator(device=dev).manual_seed(1)
        X = torch.empty(n, 3, device=dev).uniform_(0, 12 ** 0.5, generator=g)
        b = torch.randn(n, 1, device=dev, generator=g)
        times = []
        for it in range(a.reps + 1):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            out = ref.FFM_XY_FLOAT(X, X, b, dev, a.ls, a.min_points, a.nodes, False, 0.15, a.nodes)
            torch.cuda.synchronize()
            if it:
                times.append(time.perf_counter() - t0)
        t = sorted(times)[len(times) // 2]
        print(json.dumps({"impl": "reference build for sm_100a (GPU)", "N": n, "nodes": a.nodes, "min_points": a.min_points,
                          "ls": a.ls, "s_per_kmvm": t, "interactions_per_s": float(n) * n / t,
                          "checksum": float(out.double().sum())}), flush=True)
        del X, b, out
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
