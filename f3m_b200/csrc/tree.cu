// Box division, second half (per-level boxes read off the sorted keys) and interaction lists.
//
// Replaces n_tree_cuda::divide (F3M_src/n_tree.cu:105-179), get_new_interactions (n_tree.cu:594-641),
// filter_out_interactions (n_tree.cu:788-811) and separate_interactions (n_tree.cu:701-787) with
// their kernels (F3M_src/1_d_conv.cu:903-1125).  The reference materialises all 4^d child pairs of
// every surviving pair, masks them three times and rebuilds CSR rows with sorts and hash tables; here
// one warp per target box walks its parent's row, classifies the child pairs in registers and writes
// the three lists directly as CSR rows (count pass, scan, write pass).  Box ids are dense ranks, so
// no hash table is needed anywhere.
#include "common.cuh"

namespace f3m {

// ---------------------------------------------------------------------------------------------
// boxes of one level = runs of equal key prefix in the sorted key array
// ---------------------------------------------------------------------------------------------
constexpr int HT = 256, HI = 8, HTILE = HT * HI;

__device__ __forceinline__ int block_scan_excl(int v, int *total, int *sm) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) sm[wid] = inc;
    __syncthreads();
    if (wid == 0) {
        int w = lane < nw ? sm[lane] : 0, winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int t = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += t;
        }
        sm[lane] = winc - w;
        if (lane == 31) sm[32] = winc;
    }
    __syncthreads();
    int r = sm[wid] + inc - v;
    if (total) *total = sm[32];
    __syncthreads();
    return r;
}

__device__ __forceinline__ bool is_head(const uint32_t *keys, int64_t i, int shift) {
    return i == 0 || (keys[i] >> shift) != (keys[i - 1] >> shift);
}

__global__ void __launch_bounds__(HT) head_count(const uint32_t *__restrict__ keys, int64_t n, int shift, int *part) {
    __shared__ int sm[33];
    int64_t base = (int64_t)blockIdx.x * HTILE + (int64_t)threadIdx.x * HI;
    int c = 0;
#pragma unroll
    for (int k = 0; k < HI; k++)
        if (base + k < n) c += is_head(keys, base + k, shift);
    int total;
    block_scan_excl(c, &total, sm);
    if (threadIdx.x == 0) part[blockIdx.x] = total;
}

__global__ void scan_partials_total(int *part, int nparts, int *total_out) {
    __shared__ int sm[33];
    int carry = 0;
    for (int base = 0; base < nparts; base += blockDim.x) {
        int i = base + threadIdx.x;
        int v = i < nparts ? part[i] : 0;
        int total;
        int ex = block_scan_excl(v, &total, sm);
        if (i < nparts) part[i] = ex + carry;
        carry += total;
    }
    if (threadIdx.x == 0) *total_out = carry;
}

__global__ void __launch_bounds__(HT) head_write(const uint32_t *__restrict__ keys, int64_t n, int shift,
                                                const int *__restrict__ part, int *off, uint32_t *code, int nb) {
    __shared__ int sm[33];
    int64_t base = (int64_t)blockIdx.x * HTILE + (int64_t)threadIdx.x * HI;
    bool h[HI];
    int c = 0;
#pragma unroll
    for (int k = 0; k < HI; k++) {
        h[k] = (base + k < n) && is_head(keys, base + k, shift);
        c += h[k];
    }
    int r = block_scan_excl(c, nullptr, sm) + part[blockIdx.x];
#pragma unroll
    for (int k = 0; k < HI; k++)
        if (h[k]) {
            off[r] = (int)(base + k);
            code[r] = keys[base + k] >> shift;
            r++;
        }
    if (blockIdx.x == 0 && threadIdx.x == 0) off[nb] = (int)n;
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

void build_next_level(Tree &t, f3m_plan *pl, cudaStream_t s) {
    const int lvl = (int)t.levels.size();
    F3M_REQUIRE(lvl <= t.lmax, F3M_ERR_DEPTH,
                "tree needs level %d but a 30-bit cell index holds %d levels in %d dimensions", lvl, t.lmax, t.d);
    const int shift = t.d * (t.lmax - lvl);
    const int64_t n = t.n;
    int nt = (int)((n + HTILE - 1) / HTILE);
    DevBuf<int> part;
    part.alloc(nt, s);
    int *d_total = pl->d_flags + 1, *d_max = pl->d_flags + 2, *d_err = pl->d_flags + 0;
    head_count<<<nt, HT, 0, s>>>(t.keys.p, n, shift, part.p);
    F3M_LAUNCH_CHECK();
    scan_partials_total<<<1, 1024, 0, s>>>(part.p, nt, d_total);
    F3M_LAUNCH_CHECK();
    F3M_CUDA(cudaMemcpyAsync(pl->h_pinned, d_total, sizeof(int), cudaMemcpyDeviceToHost, s));
    F3M_CUDA(cudaStreamSynchronize(s));
    const int nb = pl->h_pinned[0];
    t.levels.emplace_back();
    Level &L = t.levels[lvl];
    Level &P = t.levels[lvl - 1];
    L.nb = nb;
    L.edge = P.edge * 0.5f;
    L.off.alloc((size_t)nb + 1, s); L.code.alloc(nb, s); L.parent.alloc(nb, s); L.ctr.alloc((size_t)nb * t.d, s);
    head_write<<<nt, HT, 0, s>>>(t.keys.p, n, shift, part.p, L.off.p, L.code.p, nb);
    F3M_LAUNCH_CHECK();
    F3M_CUDA(cudaMemsetAsync(d_max, 0, sizeof(int), s));
    const float q = 0.25f * P.edge;
    unsigned g = (unsigned)((nb + 255) / 256);
    switch (t.d) {
        case 1: level_links<1><<<g, 256, 0, s>>>(nb, L.code.p, L.off.p, P.nb, P.code.p, P.ctr.p, q, L.parent.p, L.ctr.p, d_max, d_err); break;
        case 2: level_links<2><<<g, 256, 0, s>>>(nb, L.code.p, L.off.p, P.nb, P.code.p, P.ctr.p, q, L.parent.p, L.ctr.p, d_max, d_err); break;
        case 3: level_links<3><<<g, 256, 0, s>>>(nb, L.code.p, L.off.p, P.nb, P.code.p, P.ctr.p, q, L.parent.p, L.ctr.p, d_max, d_err); break;
        case 4: level_links<4><<<g, 256, 0, s>>>(nb, L.code.p, L.off.p, P.nb, P.code.p, P.ctr.p, q, L.parent.p, L.ctr.p, d_max, d_err); break;
        default: level_links<5><<<g, 256, 0, s>>>(nb, L.code.p, L.off.p, P.nb, P.code.p, P.ctr.p, q, L.parent.p, L.ctr.p, d_max, d_err); break;
    }
    F3M_LAUNCH_CHECK();
    P.child_start.alloc((size_t)P.nb + 1, s);
    child_starts<<<(unsigned)((P.nb + 1 + 255) / 256), 256, 0, s>>>(P.nb, P.off.p, nb, L.off.p, P.child_start.p);
    F3M_LAUNCH_CHECK();
    F3M_CUDA(cudaMemcpyAsync(pl->h_pinned, pl->d_flags, 4 * sizeof(int), cudaMemcpyDeviceToHost, s));
    F3M_CUDA(cudaStreamSynchronize(s));
    F3M_REQUIRE(pl->h_pinned[0] == 0, F3M_ERR_INTERNAL, "box of level %d has no parent at level %d", lvl, lvl - 1);
    L.max_count = pl->h_pinned[2];
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

void accumulate_pair_work(f3m_plan *pl, int level, const PairCSR &csr, int64_t *h_pairs, cudaStream_t s) {
    if (csr.count == 0) return;
    Level &lx = pl->tx.levels[level], &ly = pl->ty->levels[level];
    unsigned long long *d_tot = reinterpret_cast<unsigned long long *>(pl->d_flags + 8);
    F3M_CUDA(cudaMemsetAsync(d_tot, 0, 8, s));
    pair_work_kernel<<<(unsigned)(((int64_t)lx.nb * 32 + 255) / 256), 256, 0, s>>>(lx.nb, csr.ptr.p, csr.idx.p, lx.off.p,
                                                                                   ly.off.p, d_tot);
    F3M_LAUNCH_CHECK();
    F3M_CUDA(cudaMemcpyAsync(pl->h_pinned, d_tot, 8, cudaMemcpyDeviceToHost, s));
    F3M_CUDA(cudaStreamSynchronize(s));
    *h_pairs += *reinterpret_cast<long long *>(pl->h_pinned);
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
    exclusive_scan_i32(cur.far.ptr.p, cur.far.ptr.p, (int64_t)nbx + 1, s);
    exclusive_scan_i32(cur.small.ptr.p, cur.small.ptr.p, (int64_t)nbx + 1, s);
    exclusive_scan_i32(cur.keep.ptr.p, cur.keep.ptr.p, (int64_t)nbx + 1, s);
    int *h = pl->h_pinned;
    F3M_CUDA(cudaMemcpyAsync(h + 0, cur.far.ptr.p + nbx, 4, cudaMemcpyDeviceToHost, s));
    F3M_CUDA(cudaMemcpyAsync(h + 1, cur.small.ptr.p + nbx, 4, cudaMemcpyDeviceToHost, s));
    F3M_CUDA(cudaMemcpyAsync(h + 2, cur.keep.ptr.p + nbx, 4, cudaMemcpyDeviceToHost, s));
    F3M_CUDA(cudaStreamSynchronize(s));
    F3M_REQUIRE(h[0] >= 0 && h[1] >= 0 && h[2] >= 0, F3M_ERR_OVERFLOW, "interaction list of level %d exceeds 2^31 pairs", level);
    cur.far.count = h[0]; cur.small.count = h[1]; cur.keep.count = h[2];
    cur.far.idx.alloc((size_t)h[0], s); cur.small.idx.alloc((size_t)h[1], s); cur.keep.idx.alloc((size_t)h[2], s);
    F3M_LISTS(1)
#undef F3M_LISTS
}

}  // namespace f3m
