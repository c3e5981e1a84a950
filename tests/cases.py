"""Seeded parity cases shared by the CPU and GPU tests and by the golden-fixture generator."""
import numpy as np
import torch

# name -> dict(d, N, M (None: shared tree), dist, ls, min_points, P, small, var_comp, eff, R, seed)
CASES = {
    "u3_shared": dict(d=3, N=30000, M=None, dist="uniform", ls=1.0, min_points=600., P=64, small=64, var_comp=False, eff=0.15, R=1, seed=0),
    "u3_default": dict(d=3, N=20000, M=None, dist="uniform", ls=1.0, min_points=1000., P=64, small=1000, var_comp=False, eff=0.15, R=1, seed=1),
    "u3_sqrt12_ls01": dict(d=3, N=30000, M=None, dist="uniform_sqrt12", ls=0.1, min_points=500., P=64, small=64, var_comp=False, eff=0.15, R=1, seed=2),
    "u3_xy": dict(d=3, N=20000, M=15000, dist="uniform", ls=0.7, min_points=400., P=27, small=27, var_comp=False, eff=0.15, R=1, seed=3),
    "n3_p125_r3": dict(d=3, N=25000, M=None, dist="normal", ls=1.5, min_points=300., P=125, small=125, var_comp=False, eff=0.15, R=3, seed=4),
    "u3_varcomp": dict(d=3, N=30000, M=None, dist="uniform_sqrt12", ls=1.0, min_points=400., P=64, small=64, var_comp=True, eff=0.9, R=1, seed=5),
    "u2_shared": dict(d=2, N=20000, M=None, dist="uniform", ls=0.5, min_points=200., P=36, small=36, var_comp=False, eff=0.15, R=2, seed=6),
    "u1_shared": dict(d=1, N=8000, M=None, dist="uniform", ls=0.2, min_points=200., P=8, small=8, var_comp=False, eff=0.15, R=1, seed=7),
    "n4_r8": dict(d=4, N=20000, M=None, dist="normal", ls=1.0, min_points=500., P=81, small=81, var_comp=False, eff=0.15, R=8, seed=8),
    "n5_r8": dict(d=5, N=12000, M=None, dist="normal", ls=1.5, min_points=1000., P=32, small=32, var_comp=False, eff=0.15, R=8, seed=9),
    # 4-D uniform with few nodes: at level 2 the list holds whole families of pairs exactly on the far threshold
    # (offsets (+-2,0,0,0) and (+-1,+-1,+-1,+-1): centre distance = 2 edges), the ties of 1_d_conv.cu:903-953
    "u4_shared": dict(d=4, N=30000, M=None, dist="uniform", ls=0.8, min_points=100., P=16, small=16, var_comp=False, eff=0.15, R=1, seed=18),
    "clustered3": dict(d=3, N=30000, M=None, dist="clustered", ls=0.5, min_points=300., P=64, small=64, var_comp=False, eff=0.15, R=1, seed=10),
    # per-level far path (more than 8 nodes per dimension, or node counts that change between levels)
    "u2_p10": dict(d=2, N=20000, M=None, dist="uniform", ls=0.5, min_points=300., P=100, small=100, var_comp=False, eff=0.15, R=1, seed=13),
    "u1_p32": dict(d=1, N=20000, M=None, dist="uniform", ls=0.1, min_points=300., P=32, small=32, var_comp=False, eff=0.15, R=2, seed=14),
    "u3_vc_mixed_p": dict(d=3, N=60000, M=None, dist="uniform", ls=1.03, min_points=150., P=64, small=64, var_comp=True, eff=0.001, R=1, seed=15),
    # two point sets whose cubes do not overlap: every level-1 pair is far
    "xy_far_apart": dict(d=3, N=15000, M=12000, dist="uniform", ls=2.0, min_points=500., P=64, small=64, var_comp=False, eff=0.15, R=1, seed=16, y_shift=4.0),
    "u3_r10": dict(d=3, N=15000, M=None, dist="uniform", ls=1.0, min_points=400., P=27, small=27, var_comp=False, eff=0.15, R=10, seed=17),
    "tiny": dict(d=3, N=50, M=None, dist="uniform", ls=1.0, min_points=1000., P=64, small=1000, var_comp=False, eff=0.15, R=1, seed=11),
    "dup_points": dict(d=3, N=5000, M=None, dist="duplicates", ls=1.0, min_points=100., P=27, small=27, var_comp=False, eff=0.15, R=1, seed=12),
}


def _draw(dist, n, d, g):
    if dist == "uniform":
        return torch.rand(n, d, generator=g)
    if dist == "uniform_sqrt12":
        return torch.rand(n, d, generator=g) * 12 ** 0.5
    if dist == "normal":
        return torch.randn(n, d, generator=g)
    if dist == "clustered":   # 10-component Gaussian mixture, means U[-5,5], std U[0.3,1]
        means = torch.rand(10, d, generator=g) * 10 - 5
        std = torch.rand(10, generator=g) * 0.7 + 0.3
        comp = torch.randint(0, 10, (n,), generator=g)
        return means[comp] + std[comp, None] * torch.randn(n, d, generator=g)
    if dist == "duplicates":  # many repeated points: boxes that cannot be split
        base = torch.rand(n // 10, d, generator=g)
        return base[torch.randint(0, n // 10, (n,), generator=g)]
    raise ValueError(dist)


def random_cases(count, seed=2024):
    """Seeded random configurations (dimension, sizes, distribution, lengthscale, leaf size, node count, list
    thresholds, variance compression, columns) for the randomized parity sweep."""
    rng = np.random.RandomState(seed)
    out = {}
    for i in range(count):
        d = int(rng.randint(1, 6))
        p = int(rng.randint(2, {1: 9, 2: 7, 3: 6, 4: 4, 5: 4}[d]))
        P = p ** d
        n = int(rng.randint(300, 7000))
        xy = rng.rand() < 0.35
        out[f"rand{i:02d}"] = dict(
            d=d, N=n, M=int(rng.randint(200, 5000)) if xy else None,
            dist=["uniform", "uniform_sqrt12", "normal", "clustered", "duplicates"][int(rng.randint(0, 5))],
            ls=float(np.exp(rng.uniform(np.log(0.08), np.log(4.0)))), min_points=float([20, 50, 100, 300][int(rng.randint(0, 4))]),
            P=P, small=int([P, 2 * P, 30, 1000][int(rng.randint(0, 4))]), var_comp=bool(rng.rand() < 0.3),
            eff=float([0.15, 0.3, 0.9, 0.001][int(rng.randint(0, 4))]), R=int([1, 1, 2, 3, 8][int(rng.randint(0, 5))]),
            seed=1000 + i)
    return out


def make_case(name, table=None):
    c = dict((table or CASES)[name])
    g = torch.Generator().manual_seed(c["seed"])
    X = _draw(c["dist"], c["N"], c["d"], g).float().contiguous()
    Y = None if c["M"] is None else (_draw(c["dist"], c["M"], c["d"], g) * 0.9 + 0.05 + c.get("y_shift", 0.0)).float().contiguous()
    b = torch.randn(c["N"] if Y is None else c["M"], c["R"], generator=g).float().contiguous()
    c.update(X=X, Y=Y, b=b)
    return c


def oracle_kwargs(c):
    return dict(ls=c["ls"], min_points=c["min_points"], nr_of_interpolation=c["P"], var_compression=c["var_comp"],
                eff_var_limit=c["eff"], small_field_points=c["small"])


def rel_l2(a, ref):
    a, ref = np.asarray(a, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    return float(np.linalg.norm(a - ref) / max(np.linalg.norm(ref), 1e-300))
