"""Generates the golden fixtures in this folder by running the UNMODIFIED reference (MrHuff/F3M) on a GPU.

The reference has no CPU path, so it cannot run where it is built: oracle/Makefile compiles it for
sm_100a from the reference's own sources into oracle/_ref/f3m_ref_d{3,4,5}.so (one module per dimension),
and this script is run on a machine with a B200:

    python tests/golden/make_golden.py [out_dir] [case ...]   # default out_dir: ./golden_out, default: all cases;
                                                              # copy the files here afterwards

For every seeded case of tests/cases.py listed in GOLDEN_CASES it stores, per level, the reference's
box offsets (unique_counts_cum_reindexed), box centres, the box of every point at the finest level,
the far / small / keep pair lists (get_field), and the product FFM_XY<float,d>(X, Y, b); plus the
reference's own dense product on the first rows.  Files are small .npz archives.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "tests"))
from cases import make_case  # noqa: E402

GOLDEN_CASES = ["u3_default", "u3_shared", "u3_sqrt12_ls01", "u3_xy", "u3_varcomp", "clustered3", "dup_points", "n3_p125_r3",
                "n4_r8", "u4_shared", "n5_r8"]


def load_ref(d=3):
    path = os.path.join(ROOT, "oracle", "_ref", f"f3m_ref_d{d}.so")
    spec = importlib.util.spec_from_file_location(f"f3m_ref_d{d}", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def box_of_point(sorted_index, cum):
    sorted_index, cum = sorted_index.cpu().numpy().astype(np.int64), cum.cpu().numpy().astype(np.int64)
    box_sorted = np.repeat(np.arange(cum.size - 1), np.diff(cum))
    out = np.empty_like(box_sorted)
    out[sorted_index] = box_sorted
    return out


def canon(pairs):
    p = pairs.cpu().numpy().astype(np.int64).reshape(-1, 2)
    return p[np.lexsort((p[:, 1], p[:, 0]))].astype(np.int32)


def main():
    out_dir = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "golden_out")
    os.makedirs(out_dir, exist_ok=True)
    names = sys.argv[2:] or GOLDEN_CASES
    refs = {}
    dev = "cuda:0"
    for name in names:
        c = make_case(name)
        if c["d"] not in refs:
            refs[c["d"]] = load_ref(c["d"])
        ref = refs[c["d"]]
        X = c["X"].to(dev)
        Y = X if c["Y"] is None else c["Y"].to(dev)
        b = c["b"].to(dev)
        trace = ref.field_trace(X, Y, dev, float(c["ls"]), float(c["min_points"]), int(c["P"]), bool(c["var_comp"]),
                                float(c["eff"]), int(c["small"]))
        torch.cuda.synchronize()
        rec = {"levels": np.int32(len(trace))}
        for l, t in enumerate(trace, start=1):
            far, small, keep = t[0], t[1], t[2]
            xs, ys = t[3:8], t[8:13]
            rec[f"l{l}_far"], rec[f"l{l}_small"], rec[f"l{l}_keep"] = canon(far), canon(small), canon(keep)
            for key, snap in (("x", xs), ("y", ys)):
                sidx, counts, cum, centers, edge = snap
                rec[f"l{l}_{key}_offsets"] = cum.cpu().numpy().astype(np.int32)
                rec[f"l{l}_{key}_centers"] = centers.cpu().numpy().astype(np.float32)
                rec[f"l{l}_{key}_edge"] = np.float32(edge.item())
                if l == len(trace):
                    rec[f"{key}_box_of_point_finest"] = box_of_point(sidx, cum).astype(np.int32)
        out = ref.FFM_XY_FLOAT(X, Y, b, dev, float(c["ls"]), float(c["min_points"]), int(c["P"]), bool(c["var_comp"]),
                               float(c["eff"]), int(c["small"]))
        torch.cuda.synchronize()
        rec["out"] = out.cpu().numpy().astype(np.float32)
        rows = min(2000, X.shape[0])
        Xr = X[:rows].contiguous()
        rec["dense_ref_rows"] = ref.rbf_float(Xr, Y, b, float(c["ls"]), True).cpu().numpy().astype(np.float32)
        np.savez_compressed(os.path.join(out_dir, f"{name}.npz"), **rec)
        print(name, "levels", len(trace), "out", rec["out"].shape, flush=True)


if __name__ == "__main__":
    main()
