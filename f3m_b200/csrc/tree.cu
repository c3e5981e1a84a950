// Box division, second half (per-level boxes read off the sorted keys) and interaction lists.
//
// Replaces n_tree_cuda::divide (F3M_src/n_tree.cu:105-179), get_new_interactions (n_tree.cu:594-641),
// filter_out_interactions (n_tree.cu:788-811) and separate_interactions (n_tree.cu:701-787) with
// their kernels (F3M_src/1_d_conv.cu:903-1125).  The reference materialises all 4^d child pairs of
// every surviving pair, masks them three times and rebuilds CSR rows with sorts and hash tables; here
// one warp per target box walks its parent's row, classifies the child pairs in registers and writes
// the three lists directly as CSR rows (count pass, scan, write pass).  Box ids are dense ranks, so
// no hash table is needed anywhere.
#include <algorithm>
#include "common.cuh"

namespace f3m {

// ---------------------------------------------------------------------------------------------
// Boxes of a level = runs of equal key prefix in the sorted key array.  A point starts a box at level l and at
// every deeper level when its key differs from its predecessor's in a bit of level l or above, so ONE pass over
// the keys finds the box starts of a whole batch of levels: count per tile and level, scan per level over the
// tiles, write offsets and prefixes.
// ---------------------------------------------------------------------------------------------
constexpr int HT = 256, HI = 8, HTILE = HT * HI;
constexpr int HB = 8;   // levels per batch

// coarsest level at which point i starts a box (lmax + 1: at none of the levels the key holds)
__device__ __forceinline__ int first_head_level(uint32_t key, uint32_t prev, bool first, int d, int lmax) {
    if (first) return 1;
    const uint32_t x = key ^ prev;
    if (!x) return lmax + 1;
    // bit h belongs to the d-bit group of level lmax - h / d; h < 32 and d <= 5, so h / d = (h * ceil(2^16 / d)) >> 16
    const int h = 31 - __clz(x);
    return lmax - ((h * ((65536 + d - 1) / d)) >> 16);
}

// the HI consecutive keys of a thread and the one before them
__device__ __forceinline__ void load_head_levels(const uint32_t *__restrict__ keys, int64_t n, int64_t base, int d, int lmax,
                                                 int (&l0)[8]) {
    uint32_t k[9];
    k[0] = (base > 0 && base - 1 < n) ? keys[base - 1] : 0u;
#pragma unroll
    for (int q = 0; q < 8; q++) k[q + 1] = (base + q < n) ? keys[base + q] : 0u;
#pragma unroll
    for (int q = 0; q < 8; q++) l0[q] = (base + q < n) ? first_head_level(k[q + 1], k[q], base + q == 0, d, lmax) : lmax + 1;
}

// part[v * nt + tile] = boxes of level l_first + v that start inside the tile
__global__ void __launch_bounds__(HT) heads_count(const uint32_t *__restrict__ keys, int64_t n, int d, int lmax, int l_first,
                                                 int nlev, int nt, int *part) {
    __shared__ int tot[HB];
    if (threadIdx.x < HB) tot[threadIdx.x] = 0;
    __syncthreads();
    const int64_t base = (int64_t)blockIdx.x * HTILE + (int64_t)threadIdx.x * HI;
    int l0[HI], c[HB];
    load_head_levels(keys, n, base, d, lmax, l0);
    int deepest = lmax + 1;
#pragma unroll
    for (int k = 0; k < HI; k++) deepest = min(deepest, l0[k]);
    // most warps hold no box start at any level of the batch (a box has hundreds of points)
    if (!__any_sync(0xffffffffu, deepest <= l_first + nlev - 1)) deepest = lmax + 1;
#pragma unroll
    for (int v = 0; v < HB; v++) c[v] = 0;
    if (deepest <= l_first + nlev - 1) {
#pragma unroll
        for (int k = 0; k < HI; k++)
#pragma unroll
            for (int v = 0; v < HB; v++) c[v] += (l0[k] <= l_first + v);
    }
#pragma unroll
    for (int v = 0; v < HB; v++) {
        if (v < nlev && __any_sync(0xffffffffu, c[v] > 0)) {
            int x = c[v];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
            if ((threadIdx.x & 31) == 0 && x) atomicAdd(&tot[v], x);
        }
    }
    __syncthreads();
    if (threadIdx.x < nlev) part[(size_t)threadIdx.x * nt + blockIdx.x] = tot[threadIdx.x];
}

// one block per level of the batch: exclusive scan of the level's tile counts, total -> totals[level]
__global__ void __launch_bounds__(1024) heads_scan(int *part, int nt, int *totals) {
    __shared__ int sm[33];
    int *row = part + (size_t)blockIdx.x * nt;
    int carry = 0;
    for (int base = 0; base < nt; base += 1024) {
        const int i = base + threadIdx.x;
        const int v = i < nt ? row[i] : 0;
        int total;
        const int ex = block_exclusive_scan(v, &total, sm);
        if (i < nt) row[i] = ex + carry;
        carry += total;
    }
    if (threadIdx.x == 0) totals[blockIdx.x] = carry;
}

struct HeadsOut {
    int *off[HB];
    uint32_t *code[HB];
    int nb[HB];
};

__global__ void __launch_bounds__(HT) heads_write(const uint32_t *__restrict__ keys, int64_t n, int d, int lmax, int l_first,
                                                 int nlev, int nt, const int *__restrict__ part, HeadsOut out) {
    __shared__ int wtot[HB][HT / 32];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int64_t base = (int64_t)blockIdx.x * HTILE + (int64_t)threadIdx.x * HI;
    int l0[HI], c[HB];
    load_head_levels(keys, n, base, d, lmax, l0);
#pragma unroll
    for (int v = 0; v < HB; v++) c[v] = 0;
#pragma unroll
    for (int k = 0; k < HI; k++)
#pragma unroll
        for (int v = 0; v < HB; v++) c[v] += (l0[k] <= l_first + v);
    int ex[HB];   // boxes of the level that start before this thread's keys, inside the warp
#pragma unroll
    for (int v = 0; v < HB; v++) {
        int inc = c[v];
        if (v < nlev && __any_sync(0xffffffffu, inc > 0)) {   // warp-uniform: most warps hold no box start
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += t;
            }
        }
        ex[v] = inc - c[v];
        if (lane == 31) wtot[v][w] = inc;
    }
    __syncthreads();
#pragma unroll
    for (int v = 0; v < HB; v++) {
        if (v >= nlev || c[v] == 0) continue;
        int r = part[(size_t)v * nt + blockIdx.x] + ex[v];
        for (int ww = 0; ww < w; ww++) r += wtot[v][ww];
        const int shift = d * (lmax - (l_first + v));
#pragma unroll
        for (int k = 0; k < HI; k++)
            if (l0[k] <= l_first + v) {
                out.off[v][r] = (int)(base + k);
                out.code[v][r] = keys[base + k] >> shift;
                r++;
            }
        if (blockIdx.x == 0 && threadIdx.x == 0) out.off[v][out.nb[v]] = (int)n;
    }
}

template <int D>
__global__ void __launch_bounds__(256) level_links(int nb, const uint32_t *__restrict__ code, const int *__restrict__ off,
                                                  int nbp, const uint32_t *__restrict__ pcode,
                                                  const float *__restrict__ pctr, float quarter_edge, int *parent,
                                                  float *ctr, int *maxcount, int *err) {
    int b = blockIdx.x * blockDim.x + threadIdx.x;
    int cnt = 0;
    if (b < nb) {
        uint32_t c = code[b], pc = c >> D;
        int lo = 0, hi = nbp;   // lower_bound of pc in pcode
        while (lo < hi) {
            int mid = (lo + hi) >> 1;
            if (pcode[mid] < pc) lo = mid + 1; else hi = mid;
        }
        if (lo >= nbp || pcode[lo] != pc) { atomicExch(err, 1); lo = 0; }
        parent[b] = lo;
        // natural_center_divide (n_tree.cu:98-104): centre = parent centre + (0.25*parent edge)*(+-1),
        // one float32 addition per coordinate
#pragma unroll
        for (int k = 0; k < D; k++) {
            float sgn = ((c >> k) & 1u) ? quarter_edge : -quarter_edge;
            ctr[b * D + k] = __fadd_rn(pctr[lo * D + k], sgn);
        }
        cnt = off[b + 1] - off[b];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cnt = max(cnt, __shfl_xor_sync(0xffffffffu, cnt, o));
    if ((threadIdx.x & 31) == 0 && cnt > 0) atomicMax(maxcount, cnt);
}

// child_start[p] = first child of parent p: the child whose point range starts where p's does
__global__ void __launch_bounds__(256) child_starts(int nbp, const int *__restrict__ poff, int nb,
                                                   const int *__restrict__ off, int *child_start) {
    int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p > nbp) return;
    if (p == nbp) { child_start[p] = nb; return; }
    int target = poff[p], lo = 0, hi = nb;
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (off[mid] < target) lo = mid + 1; else hi = mid;
    }
    child_start[p] = lo;
}

void build_root(Tree &t, cudaStream_t s) {
    t.levels.clear();
    t.levels.emplace_back();
    Level &L = t.levels.back();
    L.nb = 1;
    L.edge = t.edge0;
    L.max_count = (int)t.n;
    L.off.alloc(2, s); L.code.alloc(1, s); L.parent.alloc(1, s); L.ctr.alloc(t.d, s);
    int off[2] = {0, (int)t.n};
    float c[MAXD];
    float half = 0.5f * t.edge0;                       // exact
    for (int k = 0; k < t.d; k++) c[k] = t.origin[k] + half;   // n_tree.cu:93, float32 add
    F3M_CUDA(cudaMemcpyAsync(L.off.p, off, sizeof(off), cudaMemcpyHostToDevice, s));
    F3M_CUDA(cudaMemsetAsync(L.code.p, 0, 4, s));
    F3M_CUDA(cudaMemsetAsync(L.parent.p, 0, 4, s));
    F3M_CUDA(cudaMemcpyAsync(L.ctr.p, c, sizeof(float) * t.d, cudaMemcpyHostToDevice, s));
    F3M_CUDA(cudaStreamSynchronize(s));   // host arrays above go out of scope
}

// Appends the levels after the last one built, up to l_last, in batches of HB levels: two host synchronisations
// per batch (box counts before the arrays are sized, largest boxes after the links).
__global__ void __launch_bounds__(256) remap_offsets_kernel(int count, int *off, const int *__restrict__ fine_off) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) off[i] = fine_off[off[i]];
}

void build_levels(Tree &t, int l_last, f3m_plan *pl, cudaStream_t s) {
    F3M_REQUIRE(l_last <= t.sorted_depth, F3M_ERR_INTERNAL, "level %d requested, keys are sorted to level %d", l_last, t.sorted_depth);
    // a tree that waits for its sorted runs: one pseudo key per occupied finest cell stands for the cell's points, and
    // the box starts found among them are translated into offsets of the merged order
    const bool from_cells = t.runs.pending;
    const uint32_t *keys = from_cells ? t.runs.pkeys.p : t.keys.p;
    const int64_t n = from_cells ? t.runs.nocc : t.n;
    const int nt = (int)((n + HTILE - 1) / HTILE);
    int *d_err = pl->d_flags + FL_ERR, *d_tot = pl->d_flags + FL_LVTOT, *d_max = pl->d_flags + FL_LVMAX;
    while ((int)t.levels.size() <= l_last) {
        const int l_first = (int)t.levels.size();
        const int nlev = std::min(HB, l_last - l_first + 1);
        DevBuf<int> part;
        part.alloc((size_t)nlev * nt, s);
        heads_count<<<nt, HT, 0, s>>>(keys, n, t.d, t.lmax, l_first, nlev, nt, part.p);
        F3M_LAUNCH_CHECK();
        heads_scan<<<nlev, 1024, 0, s>>>(part.p, nt, d_tot);
        F3M_LAUNCH_CHECK();
        F3M_CUDA(cudaMemcpyAsync(pl->h_pinned + FL_LVTOT, d_tot, nlev * sizeof(int), cudaMemcpyDeviceToHost, s));
        F3M_CUDA(cudaStreamSynchronize(s));
        HeadsOut ho{};
        for (int v = 0; v < nlev; v++) {
            const int nb = pl->h_pinned[FL_LVTOT + v];
            t.levels.emplace_back();
            Level &L = t.levels.back();
            L.nb = nb;
            L.edge = t.levels[l_first + v - 1].edge * 0.5f;
            L.off.alloc((size_t)nb + 1, s); L.code.alloc(nb, s); L.parent.alloc(nb, s); L.ctr.alloc((size_t)nb * t.d, s);
            ho.off[v] = L.off.p; ho.code[v] = L.code.p; ho.nb[v] = nb;
        }
        heads_write<<<nt, HT, 0, s>>>(keys, n, t.d, t.lmax, l_first, nlev, nt, part.p, ho);
        F3M_LAUNCH_CHECK();
        if (from_cells)
            for (int v = 0; v < nlev; v++) {
                remap_offsets_kernel<<<(unsigned)((ho.nb[v] + 1 + 255) / 256), 256, 0, s>>>(ho.nb[v] + 1, ho.off[v], t.runs.fine_off.p);
                F3M_LAUNCH_CHECK();
            }
        F3M_CUDA(cudaMemsetAsync(d_max, 0, nlev * sizeof(int), s));
        for (int v = 0; v < nlev; v++) {
            Level &L = t.levels[l_first + v], &P = t.levels[l_first + v - 1];
            const int nb = L.nb;
            const float q = 0.25f * P.edge;
            const unsigned g = (unsigned)((nb + 255) / 256);
            switch (t.d) {
                case 1: level_links<1><<<g, 256, 0, s>>>(nb, L.code.p, L.off.p, P.nb, P.code.p, P.ctr.p, q, L.parent.p, L.ctr.p, d_max + v, d_err); break;
                case 2: level_links<2><<<g, 256, 0, s>>>(nb, L.code.p, L.off.p, P.nb, P.code.p, P.ctr.p, q, L.parent.p, L.ctr.p, d_max + v, d_err); break;
                case 3: level_links<3><<<g, 256, 0, s>>>(nb, L.code.p, L.off.p, P.nb, P.code.p, P.ctr.p, q, L.parent.p, L.ctr.p, d_max + v, d_err); break;
                case 4: level_links<4><<<g, 256, 0, s>>>(nb, L.code.p, L.off.p, P.nb, P.code.p, P.ctr.p, q, L.parent.p, L.ctr.p, d_max + v, d_err); break;
                default: level_links<5><<<g, 256, 0, s>>>(nb, L.code.p, L.off.p, P.nb, P.code.p, P.ctr.p, q, L.parent.p, L.ctr.p, d_max + v, d_err); break;
            }
            F3M_LAUNCH_CHECK();
            P.child_start.alloc((size_t)P.nb + 1, s);
            child_starts<<<(unsigned)((P.nb + 1 + 255) / 256), 256, 0, s>>>(P.nb, P.off.p, nb, L.off.p, P.child_start.p);
            F3M_LAUNCH_CHECK();
        }
        F3M_CUDA(cudaMemcpyAsync(pl->h_pinned + FL_LVMAX, d_max, nlev * sizeof(int), cudaMemcpyDeviceToHost, s));
        F3M_CUDA(cudaMemcpyAsync(pl->h_pinned + FL_ERR, d_err, sizeof(int), cudaMemcpyDeviceToHost, s));
        F3M_CUDA(cudaStreamSynchronize(s));
        F3M_REQUIRE(pl->h_pinned[FL_ERR] == 0, F3M_ERR_INTERNAL, "a box of levels %d..%d has no parent one level up", l_first,
                    l_first + nlev - 1);
        for (int v = 0; v < nlev; v++) t.levels[l_first + v].max_count = pl->h_pinned[FL_LVMAX + v];
    }
}

// ---------------------------------------------------------------------------------------------
// interaction lists
// ---------------------------------------------------------------------------------------------
struct ClassifyParams {
    int two_p;          // 2 * interpolation nodes
    int two_small;      // 2 * small_field_points
    float edge2;        // 2 * box edge
    int do_init;        // n_tree.cu:729-734
    int var_comp;
    int enable_pair, enable_all;   // n_tree.cu:738-739
    float crit, lcs;               // n_tree.cu:740
    int ieee;
};
enum { CLS_KEEP = 0, CLS_FAR = 1, CLS_SMALL = 2, CLS_DROP = 3 };

// boolean_separate_interactions_small / _var_comp (1_d_conv.cu:903-1029), same order of tests
template <int D>
__device__ __forceinline__ int classify(int size, const float *cx, const float *cy, const ClassifyParams &cp) {
    if (cp.do_init && size < cp.two_p) return CLS_SMALL;
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < D; k++) {
        float dk = __fsub_rn(cy[k], cx[k]);
        acc = cp.ieee ? __fadd_rn(acc, __fmul_rn(dk, dk)) : __fmaf_rn(dk, dk, acc);
    }
    float nrm;
    if (cp.ieee) nrm = __fsqrt_rn(acc);
    else asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(nrm) : "f"(acc));
    if (nrm >= cp.edge2) return cp.do_init ? CLS_FAR : CLS_DROP;
    if (cp.var_comp) {
        if (cp.enable_pair && (double)__fmul_rn(__fmul_rn(nrm, nrm), cp.lcs) <= 1e-2) return CLS_FAR;
        if (cp.enable_all && nrm <= cp.crit) return CLS_FAR;
    }
    if (size < cp.two_small) return CLS_SMALL;
    return CLS_KEEP;
}

// One warp per target box of the new level.  pass 0: count per class; pass 1: write source ids.
template <int D>
__global__ void __launch_bounds__(256) lists_kernel(int pass, int nbx, const int *__restrict__ parent_x,
                                                   const int *__restrict__ kptr, const int *__restrict__ kidx,
                                                   const int *__restrict__ cs_y, const int *__restrict__ off_x,
                                                   const int *__restrict__ off_y, const float *__restrict__ ctr_x,
                                                   const float *__restrict__ ctr_y, ClassifyParams cp, int *far_ptr,
                                                   int *small_ptr, int *keep_ptr, int *far_idx, int *small_idx,
                                                   int *keep_idx) {
    constexpr int NCH = 1 << D;
    constexpr int EPW = 32 / NCH;
    const int lane = threadIdx.x & 31;
    const int box = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (box >= nbx) return;
    const int px = parent_x[box];
    const int e0 = kptr[px], e1 = kptr[px + 1];
    const int nx = off_x[box + 1] - off_x[box];
    float cx[D];
#pragma unroll
    for (int k = 0; k < D; k++) cx[k] = ctr_x[box * D + k];
    int nf = 0, ns = 0, nk = 0;
    if (pass == 1) { nf = far_ptr[box]; ns = small_ptr[box]; nk = keep_ptr[box]; }
    const unsigned lt = (1u << lane) - 1;
    const int sub = lane / NCH, ch = lane % NCH;
    for (int it = e0; it < e1; it += EPW) {
        int e = it + sub;
        int cls = -1, by = 0;
        if (e < e1) {
            int py = kidx[e];
            int c0 = cs_y[py], c1 = cs_y[py + 1];
            by = c0 + ch;
            if (by < c1) {
                float cy[D];
#pragma unroll
                for (int k = 0; k < D; k++) cy[k] = ctr_y[by * D + k];
                cls = classify<D>(nx + off_y[by + 1] - off_y[by], cx, cy, cp);
            }
        }
        unsigned mf = __ballot_sync(0xffffffffu, cls == CLS_FAR);
        unsigned ms = __ballot_sync(0xffffffffu, cls == CLS_SMALL);
        unsigned mk = __ballot_sync(0xffffffffu, cls == CLS_KEEP);
        if (pass == 1) {
            if (cls == CLS_FAR) far_idx[nf + __popc(mf & lt)] = by;
            if (cls == CLS_SMALL) small_idx[ns + __popc(ms & lt)] = by;
            if (cls == CLS_KEEP) keep_idx[nk + __popc(mk & lt)] = by;
        }
        nf += __popc(mf); ns += __popc(ms); nk += __popc(mk);
    }
    if (pass == 0 && lane == 0) { far_ptr[box] = nf; small_ptr[box] = ns; keep_ptr[box] = nk; }
}

// sum over the rows of a CSR list of n_x * sum n_y  (work accounting only)
__global__ void __launch_bounds__(256) pair_work_kernel(int nbx, const int *__restrict__ ptr, const int *__restrict__ idx,
                                                       const int *__restrict__ off_x, const int *__restrict__ off_y,
                                                       unsigned long long *total) {
    const int lane = threadIdx.x & 31;
    const int box = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (box >= nbx) return;
    long long s = 0;
    for (int e = ptr[box] + lane; e < ptr[box + 1]; e += 32) { int by = idx[e]; s += off_y[by + 1] - off_y[by]; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0 && s) atomicAdd(total, (unsigned long long)(s * (long long)(off_x[box + 1] - off_x[box])));
}

// adds the list's pair work to the plan's device-side total, which the host reads once when the plan is complete
void accumulate_pair_work(f3m_plan *pl, int level, const PairCSR &csr, cudaStream_t s) {
    if (csr.count == 0) return;
    Level &lx = pl->tx.levels[level], &ly = pl->ty->levels[level];
    unsigned long long *d_tot = reinterpret_cast<unsigned long long *>(pl->d_flags + FL_PAIRWORK);
    pair_work_kernel<<<(unsigned)(((int64_t)lx.nb * 32 + 255) / 256), 256, 0, s>>>(lx.nb, csr.ptr.p, csr.idx.p, lx.off.p,
                                                                                   ly.off.p, d_tot);
    F3M_LAUNCH_CHECK();
}

void build_level_lists(f3m_plan *pl, int level, cudaStream_t s) {
    Tree &tx = pl->tx, &ty = *pl->ty;
    Level &lx = tx.levels[level], &ly = ty.levels[level];
    Level &py = ty.levels[level - 1];
    LevelLists &prev = pl->lists[level - 1];
    LevelLists &cur = pl->lists[level];
    const f3m_params &prm = pl->prm;
    const int d = pl->d;
    const int nbx = lx.nb;

    ClassifyParams cp{};
    cp.two_p = 2 * prm.nr_interpolation;
    cp.two_small = 2 * prm.small_field_points;
    cp.edge2 = lx.edge * 2.f;
    cp.ieee = prm.math_mode == F3M_MATH_IEEE;
    cp.var_comp = prm.var_compression != 0;
    cp.lcs = pl->lcs;
    float square_edge = lx.edge * lx.edge * pl->lcs;          // n_tree.cu:728
    cp.do_init = cp.var_comp ? (square_edge <= 5) : 1;
    if (cp.var_comp) {
        cp.enable_pair = (d * square_edge / 4) <= prm.eff_var_limit;
        cp.enable_all = (d * square_edge / 4) <= (prm.eff_var_limit / 2);
        cp.crit = sqrtf(prm.eff_var_limit * 2 / (d * pl->lcs));
    }
    cur.far.ptr.alloc((size_t)nbx + 1, s); cur.small.ptr.alloc((size_t)nbx + 1, s); cur.keep.ptr.alloc((size_t)nbx + 1, s);
    cur.far.ptr.zero(); cur.small.ptr.zero(); cur.keep.ptr.zero();
    unsigned grid = (unsigned)(((int64_t)nbx * 32 + 255) / 256);
#define F3M_LISTS(PASS)                                                                                              \
    switch (d) {                                                                                                     \
        case 1: lists_kernel<1><<<grid, 256, 0, s>>>(PASS, nbx, lx.parent.p, prev.keep.ptr.p, prev.keep.idx.p, py.child_start.p, lx.off.p, ly.off.p, lx.ctr.p, ly.ctr.p, cp, cur.far.ptr.p, cur.small.ptr.p, cur.keep.ptr.p, cur.far.idx.p, cur.small.idx.p, cur.keep.idx.p); break; \
        case 2: lists_kernel<2><<<grid, 256, 0, s>>>(PASS, nbx, lx.parent.p, prev.keep.ptr.p, prev.keep.idx.p, py.child_start.p, lx.off.p, ly.off.p, lx.ctr.p, ly.ctr.p, cp, cur.far.ptr.p, cur.small.ptr.p, cur.keep.ptr.p, cur.far.idx.p, cur.small.idx.p, cur.keep.idx.p); break; \
        case 3: lists_kernel<3><<<grid, 256, 0, s>>>(PASS, nbx, lx.parent.p, prev.keep.ptr.p, prev.keep.idx.p, py.child_start.p, lx.off.p, ly.off.p, lx.ctr.p, ly.ctr.p, cp, cur.far.ptr.p, cur.small.ptr.p, cur.keep.ptr.p, cur.far.idx.p, cur.small.idx.p, cur.keep.idx.p); break; \
        case 4: lists_kernel<4><<<grid, 256, 0, s>>>(PASS, nbx, lx.parent.p, prev.keep.ptr.p, prev.keep.idx.p, py.child_start.p, lx.off.p, ly.off.p, lx.ctr.p, ly.ctr.p, cp, cur.far.ptr.p, cur.small.ptr.p, cur.keep.ptr.p, cur.far.idx.p, cur.small.idx.p, cur.keep.idx.p); break; \
        default: lists_kernel<5><<<grid, 256, 0, s>>>(PASS, nbx, lx.parent.p, prev.keep.ptr.p, prev.keep.idx.p, py.child_start.p, lx.off.p, ly.off.p, lx.ctr.p, ly.ctr.p, cp, cur.far.ptr.p, cur.small.ptr.p, cur.keep.ptr.p, cur.far.idx.p, cur.small.idx.p, cur.keep.idx.p); break; \
    }                                                                                                                \
    F3M_LAUNCH_CHECK();
    F3M_LISTS(0)
    int *ptrs[3] = {cur.far.ptr.p, cur.small.ptr.p, cur.keep.ptr.p};
    long long *d_tot = reinterpret_cast<long long *>(pl->d_flags + FL_LISTTOT);
    exclusive_scan_multi(ptrs, 3, (int64_t)nbx + 1, d_tot, s);
    long long *h = reinterpret_cast<long long *>(pl->h_pinned + FL_LISTTOT);
    F3M_CUDA(cudaMemcpyAsync(h, d_tot, 3 * sizeof(long long), cudaMemcpyDeviceToHost, s));
    F3M_CUDA(cudaStreamSynchronize(s));
    F3M_REQUIRE(h[0] <= 0x7fffffffLL && h[1] <= 0x7fffffffLL && h[2] <= 0x7fffffffLL, F3M_ERR_OVERFLOW,
                "interaction list of level %d exceeds 2^31 pairs (far %lld, small %lld, kept %lld)", level, h[0], h[1], h[2]);
    cur.far.count = h[0]; cur.small.count = h[1]; cur.keep.count = h[2];
    cur.far.idx.alloc((size_t)h[0], s); cur.small.idx.alloc((size_t)h[1], s); cur.keep.idx.alloc((size_t)h[2], s);
    F3M_LISTS(1)
#undef F3M_LISTS
}

}  // namespace f3m
