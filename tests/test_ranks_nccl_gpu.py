"""A product computed by real NCCL ranks (one process per GPU): needs at least two visible GPUs, skipped otherwise.

Each rank starts with its shard of X and b, runs f3m_b200.parallel.distributed_kmvm and gets the rows of its shard;
they are checked against the float64 dense product and against the single-GPU product of the same engine."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

RANK_CODE = r'''
import os, sys, json, torch, torch.distributed as dist
sys.path.insert(0, os.environ["F3M_ROOT"])
from f3m_b200 import engine
from f3m_b200.parallel import distributed_kmvm
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
res = {}
for name, n, d, R, ls, P, dist_kind in (("uniform", 300001, 3, 1, 1.0, 64, "u"), ("clustered", 200000, 3, 2, 0.5, 64, "c"),
                                        ("normal4", 60000, 4, 8, 1.0, 81, "n")):
    g = torch.Generator().manual_seed(5)
    if dist_kind == "u":
        X = torch.rand(n, d, generator=g) * 12 ** 0.5
    elif dist_kind == "n":
        X = torch.randn(n, d, generator=g)
    else:
        means = torch.rand(10, d, generator=g) * 10 - 5
        comp = torch.randint(0, 10, (n,), generator=g)
        X = means[comp] + (torch.rand(10, generator=g) * 0.7 + 0.3)[comp, None] * torch.randn(n, d, generator=g)
    b = torch.randn(n, R, generator=g)
    cuts = [0] + sorted(torch.randint(1, n, (world - 1,), generator=g).tolist()) + [n]     # uneven shards
    lo, hi = cuts[rank], cuts[rank + 1]
    prm = engine.make_params(ls, 500.0, P, False, 0.15, P)
    stats = {}
    out = distributed_kmvm(X[lo:hi].to(dev), b[lo:hi].to(dev), prm, stats=stats)
    assert out.shape == (hi - lo, R)
    Xd, bd = X.to(dev), b.to(dev)
    single = engine.kmvm(Xd, None, bd, prm)[lo:hi]
    rows = torch.arange(lo, min(hi, lo + 1500), device=dev)
    exact = engine.rbf_dense(Xd[rows].double(), Xd.double(), bd.double(), ls)
    e_dist = float((out[:rows.numel()].double() - exact).norm() / exact.norm())
    e_single = float((single[:rows.numel()].double() - exact).norm() / exact.norm())
    diff = float((out - single).norm() / single.norm())
    res[name] = dict(e_dist=e_dist, e_single=e_single, diff=diff, slice_rows=stats["slice_rows"])
with open(os.path.join(os.environ["F3M_OUT"], f"result_{rank}.json"), "w") as fh:
    json.dump(dict(rank=rank, res=res), fh)
dist.barrier()
dist.destroy_process_group()
'''


@pytest.mark.parametrize("world", [2, 4])
def test_product_on_nccl_ranks(world, tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import json
    script = tmp_path / "rank.py"
    script.write_text(RANK_CODE)
    env = dict(os.environ, F3M_ROOT=ROOT, F3M_OUT=str(tmp_path), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29600 + world), str(script)]
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    lines = [json.load(open(tmp_path / f"result_{r}.json")) for r in range(world)]
    for rec in lines:
        for name, r in rec["res"].items():
            assert r["diff"] <= 5e-6, (name, rec)                       # same engine, other summation order of the far field
            assert r["e_dist"] <= max(1.2 * r["e_single"], r["e_single"] + 2e-6), (name, rec)
