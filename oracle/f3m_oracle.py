"""CPU restatement of the reference F3M algorithm (MrHuff/F3M) -- TEST INFRASTRUCTURE ONLY.

This file is the checker and the timed CPU baseline.  It is never imported by the product
package: only the tests, the smoke check and the CPU legs of the benchmark may use it.

The reference has no CPU path (its operator dispatches straight into a CUDA extension,
experiments/FFM_classes.py:98-126), so this is a stage-by-stage restatement of the reference's
algorithm with PyTorch CPU tensor ops in float32, batched per level.  Each function cites the
reference lines it follows (paths are relative to the reference repository).

Parity pin: the restatement is checked against outputs of the reference itself (built for sm_100a
from its own sources and run on a B200) stored as fixtures under tests/golden/ -- box
assignments, far/small/near lists and KMVM outputs.  Arithmetic that the reference evaluates
with fast-math GPU instructions (approximate divide in the box index, approximate sqrt in the far
test) is evaluated here with IEEE float32 operations; the engine has a matching "ieee" mode and a
"fastmath" mode, and the tests state which is compared with what.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np
import torch

F32 = torch.float32
I64 = torch.int64


# --------------------------------------------------------------------------------------
# exact dense product (accuracy oracle)
# --------------------------------------------------------------------------------------
def dense_kmvm_f64(X: torch.Tensor, Y: torch.Tensor, b: torch.Tensor, ls: float,
                   rows: Optional[torch.Tensor] = None, chunk: int = 2048) -> torch.Tensor:
    """out[i] = sum_j exp(-|x_i-y_j|^2/(2 ls^2)) b_j in float64.

    The op of rbf_call (F3M_src/n_tree.cu:185-211, kernel F3M_src/1_d_conv.cu:171-214) with a
    true double-precision exponential.
    """
    Xd = X.double() if rows is None else X[rows].double()
    Yd, bd = Y.double(), b.double()
    lcs = 1.0 / (2.0 * float(ls) * float(ls))
    out = torch.empty(Xd.shape[0], bd.shape[1], dtype=torch.float64)
    for s in range(0, Xd.shape[0], chunk):
        d2 = torch.cdist(Xd[s:s + chunk], Yd, compute_mode="donot_use_mm_for_euclid_dist").pow_(2)
        out[s:s + chunk] = torch.exp_(d2.mul_(-lcs)) @ bd
    return out


# --------------------------------------------------------------------------------------
# interpolation nodes
# --------------------------------------------------------------------------------------
def node_list(nd: int, max_nodes: int) -> List[int]:
    """Nodes per dimension (F3M_src/n_tree.cu:328-349).

    The reference finishes with a random permutation of the dimensions (n_tree.cu:347); it is the
    identity whenever max_nodes is a perfect nd-th power, which is the only case pinned here.  For
    other values this restatement keeps the un-permuted order.
    """
    ref_val = np.float32(math.pow(max_nodes, float(np.float32(1.0) / np.float32(nd))))
    hi, lo = int(math.ceil(ref_val)), int(math.floor(ref_val))
    acc, out = 1, []
    for i in range(nd):
        future = acc * int(math.pow(lo, nd - (i + 1))) * hi
        if future <= max_nodes:
            out.append(hi)
            acc *= hi
        else:
            out.append(lo)
            acc *= lo
    return out


def cheb_nodes_weights(p: int, dtype=F32):
    """First-kind Chebyshev nodes and barycentric weights (n_tree.cu:265-285), float32 as in the reference
    (float64 when the algorithm is evaluated in float64: see the `dtype` argument of f3m_kmvm)."""
    if dtype == torch.float64:
        k = torch.arange(0, p, dtype=torch.float64)
        ang = (2. * k + 1.) * math.pi / (2. * p)
        return torch.cos(ang), torch.where(k.long() % 2 == 0, 1.0, -1.0) * torch.sin(ang)
    pi32 = float(np.float32(math.atan(1.0) * 4.0))
    k = torch.arange(0, p).to(F32)
    nodes = torch.cos((k * 2. + 1.) * pi32 / (2 * (p - 1) + 2))
    w = torch.tensor([math.pow(-1.0, i) * math.sin(((2. * float(np.float32(i)) + 1.) * pi32)
                                                 / (2. * float(np.float32(p - 1.0)) + 2.))
                      for i in range(p)], dtype=torch.float64).to(F32)
    return nodes, w


def tensor_grid(nodes_1d: List[torch.Tensor]):
    """Multi-index of every grid node, dimension 0 fastest (1_d_conv.cu:850-884)."""
    ps = [int(n.numel()) for n in nodes_1d]
    P = int(np.prod(ps))
    m = torch.arange(P)
    idx, stride = [], 1
    for p in ps:
        idx.append((m // stride) % p)
        stride *= p
    idx = torch.stack(idx, 1)                                   # (P, d) int64
    coords = torch.stack([nodes_1d[k][idx[:, k]] for k in range(len(ps))], 1)   # (P, d) f32
    return idx, coords


def lagrange_basis_1d(t: torch.Tensor, nodes: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Barycentric basis L_j(t) for every t (n,) -> (n, p), float32.

    Follows lagrange_data_load + calculate_barycentric_lagrange (1_d_conv.cu:217-238, 418-448):
    L_j = (1/sum_l w_l/(t-t_l)) * w_j/(t-t_j); a coordinate that hits a node exactly gets the
    indicator of that node.
    """
    diff = t[:, None] - nodes[None, :]
    hit = diff == 0
    safe = torch.where(hit, torch.ones_like(diff), diff)
    terms = w[None, :] / safe
    lx = 1.0 / terms.sum(1, keepdim=True)
    L = (lx * w[None, :]) / safe
    anyhit = hit.any(1)
    if bool(anyhit.any()):
        L[anyhit] = hit[anyhit].to(L.dtype)
    return L


def full_basis(T: torch.Tensor, nodes_1d, w_1d) -> torch.Tensor:
    """(n, d) scaled coordinates -> (n, P) product basis, dimension 0 fastest."""
    B = lagrange_basis_1d(T[:, 0], nodes_1d[0], w_1d[0])
    for k in range(1, T.shape[1]):
        Lk = lagrange_basis_1d(T[:, k], nodes_1d[k], w_1d[k])
        B = (Lk[:, :, None] * B[:, None, :]).reshape(T.shape[0], -1)
    return B


# --------------------------------------------------------------------------------------
# tree
# --------------------------------------------------------------------------------------
class Tree:
    """State of n_tree_cuda (n_tree.cu:50-180) restated with Morton prefixes.

    The reference numbers the boxes of a level as children of the compacted parents
    (natural id = 2^d * compact(parent) + child code, child code bit k = upper half in dimension k,
    1_d_conv.cu:887-899) and then removes the empty ones (n_tree.cu:162-177,
    transpose_to_existing_only_tree 1_d_conv.cu:1056-1077).  That is the rank of the point's
    level-l Morton prefix (dimension 0 in the least significant bit of each group) among the
    occupied prefixes, which is how it is computed here.
    """

    def __init__(self, data: torch.Tensor, edge0: torch.Tensor, xmin: torch.Tensor):
        self.data = data
        self.n, self.d = data.shape
        self.edge0 = edge0.to(F32)                      # edge_og
        self.edge = self.edge0.clone()
        self.xmin = xmin.to(F32)
        self.depth = 0
        self.centers = (self.xmin + 0.5 * self.edge).unsqueeze(0)        # n_tree.cu:93
        self.keys = torch.zeros(1, dtype=I64)           # occupied Morton prefixes, sorted
        self.box_of_point = torch.zeros(self.n, dtype=I64)
        self.counts = torch.tensor([self.n], dtype=I64)
        self.max_count = float(self.n)                  # "avg_nr_points" (n_tree.cu:87,169)
        self.parent = torch.zeros(1, dtype=I64)
        self._update_offsets()

    def _update_offsets(self):
        self.offsets = torch.zeros(self.counts.numel() + 1, dtype=I64)
        self.offsets[1:] = torch.cumsum(self.counts, 0)
        self.sorted_index = torch.argsort(self.box_of_point, stable=True)

    def cell_coords(self, depth: int) -> torch.Tensor:
        """floor(2^l (x - xmin)/edge_og) in float32 (1_d_conv.cu:1143); IEEE divide here."""
        side = torch.tensor(2.0, dtype=F32).pow(depth)
        q = torch.floor(side * (self.data - self.xmin) / self.edge0).to(I64)
        return q.clamp_(0, 2 ** depth - 1)

    def divide(self):
        d = self.d
        self.depth += 1
        q = self.cell_coords(self.depth)
        key = torch.zeros(self.n, dtype=I64)
        for lvl in range(1, self.depth + 1):                      # coarsest level most significant
            sh = self.depth - lvl
            for k in range(d):
                key |= ((q[:, k] >> sh) & 1) << (d * sh + k)
        keys, inv, counts = torch.unique(key, sorted=True, return_inverse=True, return_counts=True)
        parent_keys = keys >> d
        parent = torch.searchsorted(self.keys, parent_keys)
        assert bool((self.keys[parent] == parent_keys).all()), "child cell outside an occupied parent"
        code = keys & (2 ** d - 1)
        sign = torch.stack([((code >> k) & 1) * 2 - 1 for k in range(d)], 1).to(F32)
        # natural_center_divide (n_tree.cu:98-104): centre = parent centre + (0.25*edge_parent)*(+-1)
        self.centers = self.centers[parent] + (0.25 * self.edge) * sign
        self.edge = self.edge * 0.5
        self.parent, self.keys, self.box_of_point, self.counts = parent, keys, inv, counts
        self.max_count = float(counts.max())
        # first child (compact id) of every parent box; children of a parent are contiguous
        nparent = int(parent.max()) + 1 if parent.numel() else 0
        self.child_start = torch.searchsorted(parent, torch.arange(nparent + 1))
        self._update_offsets()


def bounding_cube(X: torch.Tensor, Y: Optional[torch.Tensor]):
    """calculate_edge_X / calculate_edge (n_tree.cu:25-46): edge = 1.01 * largest coordinate range."""
    xmin, xmax = X.min(0).values, X.max(0).values
    if Y is None:
        return (xmax - xmin).max() * 1.01, xmin, None
    ymin, ymax = Y.min(0).values, Y.max(0).values
    edge = torch.stack([(xmax - xmin).max(), (ymax - ymin).max()]).max() * 1.01
    return edge, xmin, ymin


# --------------------------------------------------------------------------------------
# interaction lists
# --------------------------------------------------------------------------------------
def candidate_pairs(near: torch.Tensor, tx: Tree, ty: Tree) -> torch.Tensor:
    """All child pairs of the surviving near pairs with both children occupied, in compact ids.

    get_new_interactions (n_tree.cu:594-641; repeat_within / repeat_add 1_d_conv.cu:1080-1125)
    followed by filter_out_interactions (n_tree.cu:788-811).  Returned sorted by (left, right),
    which is the order the reference produces.
    """
    out = []
    csx, csy = tx.child_start, ty.child_start
    for s in range(0, near.shape[0], 1 << 16):
        blk = near[s:s + (1 << 16)]
        nx = csx[blk[:, 0] + 1] - csx[blk[:, 0]]
        ny = csy[blk[:, 1] + 1] - csy[blk[:, 1]]
        per = nx * ny
        tot = int(per.sum())
        pid = torch.repeat_interleave(torch.arange(blk.shape[0]), per)
        start = torch.cumsum(per, 0) - per
        r = torch.arange(tot) - start[pid]
        left = csx[blk[pid, 0]] + r // ny[pid]
        right = csy[blk[pid, 1]] + r % ny[pid]
        out.append(torch.stack([left, right], 1))
    pairs = torch.cat(out, 0) if out else torch.zeros(0, 2, dtype=I64)
    order = np.lexsort((pairs[:, 1].numpy(), pairs[:, 0].numpy()))
    return pairs[torch.from_numpy(order)]


def classify_pairs(pairs, tx: Tree, ty: Tree, lcs: float, P: int, small_field: int,
                   var_comp: bool, eff_var_limit: float, near_tie_far=None):
    """far / small / keep masks (separate_interactions n_tree.cu:701-787; kernels 1_d_conv.cu:903-1029).

    near_tie_far: optional callable(level, tie_pairs) -> bool tensor.  Pairs whose centre distance is within a few
    float32 ulp of the far threshold 2*edge (in 4 and more dimensions whole families of box offsets sit exactly on it)
    are classified by the reference with sqrt.approx and a fused sum, whose last-bit behaviour no CPU arithmetic
    reproduces; a test that knows the reference's decision for those pairs passes it in here, and every other
    decision stays the restatement's own."""
    d = tx.d
    bx, by = pairs[:, 0], pairs[:, 1]
    size = tx.counts[bx] + ty.counts[by]
    edge = tx.edge
    e = float(edge)
    square_edge = float(np.float32(np.float32(e) * np.float32(e)) * np.float32(lcs))
    do_init = (square_edge <= 5) if var_comp else True
    dist = ty.centers[by] - tx.centers[bx]
    acc = torch.zeros(pairs.shape[0], dtype=F32)
    for k in range(d):                               # get_2_norm (1_d_conv.cu:242-250), k order
        acc = acc + dist[:, k] * dist[:, k]
    norm = torch.sqrt(acc)
    undecided = torch.ones(pairs.shape[0], dtype=torch.bool)
    small = torch.zeros_like(undecided)
    far = torch.zeros_like(undecided)
    if do_init:
        m = size < 2 * P
        small |= m
        undecided &= ~m
    is_far = norm >= edge * 2
    if near_tie_far is not None:
        thr = float(edge * 2)
        tie = undecided & ((norm - thr).abs() <= 8 * float(np.spacing(np.float32(thr))))
        if bool(tie.any()):
            is_far = is_far.clone()
            is_far[tie] = near_tie_far(tx.depth, pairs[tie])
    m = undecided & is_far
    if do_init:
        far |= m
    undecided &= ~m                                   # var_comp with q>5: pair is dropped
    if var_comp:
        lcs32 = np.float32(lcs)
        enable_pair = (d * square_edge / 4) <= eff_var_limit
        enable_all = (d * square_edge / 4) <= (eff_var_limit / 2)
        crit = float(np.float32(math.sqrt(eff_var_limit * 2 / (d * float(lcs32)))))
        if enable_pair:
            m = undecided & ((norm * norm * float(lcs32)) <= 1e-2)
            far |= m
            undecided &= ~m
        if enable_all:
            m = undecided & (norm <= crit)
            far |= m
            undecided &= ~m
    m = undecided & (size < 2 * small_field)
    small |= m
    undecided &= ~m
    return far, small, undecided


# --------------------------------------------------------------------------------------
# numerical stages
# --------------------------------------------------------------------------------------
def direct_sums(pairs, tx: Tree, ty: Tree, b, lcs: float, out):
    """near_field_run (n_tree.cu:831-902) + skip_conv_1d_shared (1_d_conv.cu:255-335).  Arithmetic in out.dtype."""
    if pairs.shape[0] == 0:
        return 0
    dt = out.dtype
    X, Y = tx.data.to(dt), ty.data.to(dt)
    left = pairs[:, 0]
    ub, cnt = torch.unique_consecutive(left, return_counts=True)
    starts = torch.cumsum(cnt, 0) - cnt
    npairs = 0
    for u, s, c in zip(ub.tolist(), starts.tolist(), cnt.tolist()):
        xi = tx.sorted_index[tx.offsets[u]:tx.offsets[u + 1]]
        rights = pairs[s:s + c, 1]
        yj = torch.cat([ty.sorted_index[ty.offsets[r]:ty.offsets[r + 1]] for r in rights.tolist()])
        xs, ys = X[xi], Y[yj]
        d2 = torch.zeros(xs.shape[0], ys.shape[0], dtype=dt)
        for k in range(X.shape[1]):
            diff = xs[:, k, None] - ys[None, :, k]
            d2 += diff * diff
        out[xi] += torch.exp(-d2 * lcs) @ b[yj]
        npairs += xs.shape[0] * ys.shape[0]
    return npairs


def far_field(far, tx: Tree, ty: Tree, b, lcs: float, P: int, out, stats):
    """far_field_compute_v2 (n_tree.cu:489-593): P2M -> node-to-node sums -> L2P.  Arithmetic in out.dtype."""
    d = tx.d
    dt = out.dtype
    ps = node_list(d, P)
    nodes_1d, w_1d = zip(*[cheb_nodes_weights(p, dt) for p in ps])
    _, grid = tensor_grid(list(nodes_1d))                      # (P, d) in [-1,1]
    Pn = grid.shape[0]
    edge = tx.edge.to(dt)
    xdata, ydata, xctr, yctr = tx.data.to(dt), ty.data.to(dt), tx.centers.to(dt), ty.centers.to(dt)
    R = b.shape[1]
    uy = torch.unique(far[:, 1])
    ux = torch.unique(far[:, 0])
    factor = 2 / edge                                          # 1_d_conv.cu:473
    # P2M (lagrange_shared, 1_d_conv.cu:451-552)
    mom = torch.zeros(ty.counts.numel(), Pn, R, dtype=dt)
    needed = torch.zeros(ty.counts.numel(), dtype=torch.bool)
    needed[uy] = True
    idx = ty.sorted_index[needed[ty.box_of_point[ty.sorted_index]]]
    for s in range(0, idx.numel(), 1 << 15):
        ii = idx[s:s + (1 << 15)]
        bx = ty.box_of_point[ii]
        T = factor * (ydata[ii] - yctr[bx])
        B = full_basis(T, nodes_1d, w_1d)
        mom.index_add_(0, bx, B[:, :, None] * b[ii][:, None, :])
    # M2L (setup_skip_conv n_tree.cu:433-486; skip_conv_far_boxes_opt 1_d_conv.cu:741-817)
    g = grid * edge / 2. + edge / 2.                           # n_tree.cu:510
    loc = torch.zeros(tx.counts.numel(), Pn, R, dtype=dt)
    chunk = max(1, (1 << 24) // (Pn * Pn))
    for s in range(0, far.shape[0], chunk):
        blk = far[s:s + chunk]
        xi = g[None, :, :] + xctr[blk[:, 0]][:, None, :]
        yj = g[None, :, :] + yctr[blk[:, 1]][:, None, :]
        d2 = torch.zeros(blk.shape[0], Pn, Pn, dtype=dt)
        for k in range(d):
            diff = xi[:, :, None, k] - yj[:, None, :, k]
            d2 += diff * diff
        loc.index_add_(0, blk[:, 0], torch.bmm(torch.exp(-d2 * lcs), mom[blk[:, 1]]))
    stats["node_pairs"] = stats.get("node_pairs", 0) + int(far.shape[0]) * Pn * Pn
    # L2P (laplace_shared_transpose, 1_d_conv.cu:554-659)
    neededx = torch.zeros(tx.counts.numel(), dtype=torch.bool)
    neededx[ux] = True
    idx = tx.sorted_index[neededx[tx.box_of_point[tx.sorted_index]]]
    for s in range(0, idx.numel(), 1 << 15):
        ii = idx[s:s + (1 << 15)]
        bx = tx.box_of_point[ii]
        T = factor * (xdata[ii] - xctr[bx])
        B = full_basis(T, nodes_1d, w_1d)
        out[ii] += torch.einsum("np,npr->nr", B, loc[bx])


# --------------------------------------------------------------------------------------
# top level
# --------------------------------------------------------------------------------------
def f3m_kmvm(X: torch.Tensor, Y: Optional[torch.Tensor], b: torch.Tensor, ls: float,
             min_points: float = 1000., nr_of_interpolation: int = 64, var_compression: bool = False,
             eff_var_limit: float = 0.15, small_field_points: int = 1000,
             trace: Optional[List[Dict]] = None, lists_only: bool = False,
             stats: Optional[Dict] = None, dtype=F32, near_tie_far=None) -> Optional[torch.Tensor]:
    """FFM_XY<float,d> (n_tree.cu:1056-1125).  Y=None means the shared-tree case X is Y.

    dtype=torch.float64 evaluates the SAME algorithm -- the float32 tree, box assignment and interaction lists of
    the reference, per-level P2M -> M2L -> L2P and the direct sums -- with all arithmetic on b in float64.  Its
    distance from the float32 result is the reference algorithm's own rounding error, which is what separates
    "differs from the reference" from "differs from what the reference computes up to its rounding"."""
    X = X.to(F32).contiguous()
    b = b.to(dtype).contiguous()
    same = Y is None
    stats = stats if stats is not None else {}
    lcs = float(np.float32(1) / (np.float32(2) * np.float32(ls) * np.float32(ls)))   # n_tree.cu:1060
    out = torch.zeros(X.shape[0], b.shape[1], dtype=dtype)
    edge, xmin, ymin = bounding_cube(X, None if same else Y.to(F32))
    tx = Tree(X, edge, xmin)
    ty = tx if same else Tree(Y.to(F32).contiguous(), edge, ymin)
    near = torch.zeros(1, 2, dtype=I64)
    d = X.shape[1]

    def go_on():
        if near.shape[0] == 0:
            return False
        if same:
            return tx.max_count > min_points
        return tx.max_count > min_points and ty.max_count > min_points

    while go_on():
        tx.divide()
        if not same:
            ty.divide()
        pairs = candidate_pairs(near, tx, ty)
        P_level = nr_of_interpolation
        far_m, small_m, keep_m = classify_pairs(pairs, tx, ty, lcs, nr_of_interpolation,
                                                small_field_points, var_compression, eff_var_limit, near_tie_far)
        far, small, near = pairs[far_m], pairs[small_m], pairs[keep_m]
        if var_compression:                      # get_interpolation_rule (n_tree.cu:971-978,1022-1028)
            e = np.float32(float(tx.edge))
            if float(e * e * np.float32(lcs)) < 0.01:
                P_level = min(3 ** d, nr_of_interpolation)
        if trace is not None:
            rec = dict(level=tx.depth, far=far.clone(), small=small.clone(), keep=near.clone(),
                       edge=float(tx.edge), P=P_level)
            for name, t in (("x", tx), ("y", ty)):
                rec[name] = dict(box_of_point=t.box_of_point.clone(), counts=t.counts.clone(),
                                 offsets=t.offsets.clone(), centers=t.centers.clone(),
                                 sorted_index=t.sorted_index.clone())
            trace.append(rec)
        if lists_only:
            continue
        if small.shape[0] > 0:
            stats["direct_pairs"] = stats.get("direct_pairs", 0) + direct_sums(small, tx, ty, b, lcs, out)
        if far.shape[0] > 0:
            far_field(far, tx, ty, b, lcs, P_level, out, stats)
    if trace is not None:
        trace.append(dict(level=tx.depth, final_near=near.clone()))
    if lists_only:
        return None
    if near.shape[0] > 0:
        stats["direct_pairs"] = stats.get("direct_pairs", 0) + direct_sums(near, tx, ty, b, lcs, out)
    return out
