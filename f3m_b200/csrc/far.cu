// Far field of one level: P2M (anterpolation) -> node-to-node sums -> L2P (interpolation).
//
// Replaces far_field_compute_v2 (F3M_src/n_tree.cu:489-593) and its kernels lagrange_shared,
// skip_conv_far_boxes_opt and laplace_shared_transpose (F3M_src/1_d_conv.cu:451-659, 741-817).
//
//  * P2M: the reference issues one global atomicAdd per (point, node, column).  Here a CTA takes a
//    chunk of the sorted source points, keeps the 1-D Lagrange bases of the chunk in shared memory,
//    reduces every box segment of the chunk in registers (one thread per node) and adds one partial
//    moment vector per segment.  HBM-bound: the points are read once per level.
//  * node-to-node: the reference evaluates P^2 exponentials per box pair.  The interpolation nodes
//    form a tensor grid and the Gaussian is a product over dimensions, so the P x P block between two
//    boxes is the Kronecker product of d small p x p matrices that depend only on the integer offset
//    of the two boxes in that dimension.  Those matrices are tabulated once per level (a few KB) and
//    each pair costs d*p*P multiply-adds and no exponential.
//  * L2P: one thread per target point, sum-factorised over the fastest dimension.
#include <math.h>
#include "common.cuh"

namespace f3m {

// get_node_list (F3M_src/n_tree.cu:328-349) for the uniform case; the same float rounding of the d-th root.
int nodes_per_dim(int d, int nr_interpolation) {
    float ref_val = (float)pow((double)nr_interpolation, (double)(1.0f / (float)d));
    int hi = (int)ceilf(ref_val), lo = (int)floorf(ref_val);
    // the reference keeps `hi` in a dimension only if the product stays within nr_interpolation
    long prod = 1;
    for (int i = 0; i < d; i++) prod *= hi;
    int p = (prod <= nr_interpolation) ? hi : lo;
    return p < 1 ? 1 : p;
}

struct NodeTab {
    int p;
    float node[MAXP];
    float w[MAXP];
};

static NodeTab make_nodes(int p) {
    NodeTab t{};
    t.p = p;
    cheb_nodes_weights(p, t.node, t.w);
    return t;
}

constexpr int CH = 256;   // points per CTA chunk in P2M / L2P

// Barycentric Lagrange basis of one coordinate (lagrange_data_load + calculate_barycentric_lagrange,
// 1_d_conv.cu:217-238, 418-448).  Writes p values with stride `stride`.
__device__ __forceinline__ void lagrange_1d(float t, const NodeTab &nt, float *dst, int stride) {
    const int p = nt.p;
    int hit = -1;
    float sum = 0.f;
    for (int i = 0; i < p; i++) {
        float diff = t - nt.node[i];
        if (diff == 0.f) hit = i;
        else sum += nt.w[i] / diff;
    }
    if (hit >= 0) {
        for (int i = 0; i < p; i++) dst[i * stride] = (i == hit) ? 1.f : 0.f;
    } else {
        float lx = 1.f / sum;
        for (int i = 0; i < p; i++) dst[i * stride] = (lx * nt.w[i]) / (t - nt.node[i]);
    }
}


__global__ void __launch_bounds__(256) mark_sources(const int *__restrict__ idx, int64_t n, unsigned char *need) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) need[idx[i]] = 1;
}

// ---------------------------------------------------------------------------------------------
// P2M
// ---------------------------------------------------------------------------------------------
template <int D, int RB>
__global__ void __launch_bounds__(CH) p2m_kernel(const float *__restrict__ pts, int n, const float *__restrict__ bs, int R,
                                                int r0, const int *__restrict__ off, int nb,
                                                const float *__restrict__ ctr, float factor, NodeTab nt,
                                                const unsigned char *__restrict__ need, int P, float *mom) {
    extern __shared__ float sm[];
    const int p = nt.p;
    float *Ls = sm;                              // [D*p][CH+1]
    float *bsm = Ls + D * p * (CH + 1);          // [CH][RB]
    __shared__ int s_box[CH];
    const int c0 = blockIdx.x * CH;
    const int j = threadIdx.x, i = c0 + j;
    int mybox = -1;
    if (i < n) {
        mybox = box_of_row(off, nb, i);
        if (!need[mybox]) mybox = -1;
    }
    s_box[j] = mybox;
    if (mybox >= 0) {
#pragma unroll
        for (int k = 0; k < D; k++) {
            float t = factor * (pts[(size_t)k * n + i] - ctr[mybox * D + k]);
            lagrange_1d(t, nt, Ls + (k * p) * (CH + 1) + j, CH + 1);
        }
#pragma unroll
        for (int r = 0; r < RB; r++) bsm[j * RB + r] = (r0 + r < R) ? bs[(size_t)i * R + r0 + r] : 0.f;
    }
    __syncthreads();
    const int last = min(n - c0, CH) - 1;
    const int box_first = box_of_row(off, nb, c0), box_last = box_of_row(off, nb, c0 + last);
    // thread -> (node, point group)
    int groups = CH / P;
    if (groups < 1) groups = 1;
    const int g = (P >= CH) ? 0 : j / P;
    const bool active = (P >= CH) || (g < groups);
    for (int bb = box_first; bb <= box_last; bb++) {
        if (!need[bb]) continue;
        const int j0 = max(off[bb], c0) - c0, j1 = min(off[bb + 1], c0 + CH) - c0;
        if (!active) continue;
        for (int m = (P >= CH) ? j : j % P; m < P; m += CH) {
            const float *lp[D];
            int rem = m;
#pragma unroll
            for (int k = 0; k < D; k++) {
                lp[k] = Ls + (k * p + rem % p) * (CH + 1);
                rem /= p;
            }
            float acc[RB];
#pragma unroll
            for (int r = 0; r < RB; r++) acc[r] = 0.f;
            for (int jj = j0 + g; jj < j1; jj += groups) {
                float prod = lp[0][jj];
#pragma unroll
                for (int k = 1; k < D; k++) prod *= lp[k][jj];
#pragma unroll
                for (int r = 0; r < RB; r++) acc[r] = fmaf(prod, bsm[jj * RB + r], acc[r]);
            }
#pragma unroll
            for (int r = 0; r < RB; r++)
                if (r0 + r < R && j0 + g < j1) atomicAdd(&mom[((size_t)bb * P + m) * R + r0 + r], acc[r]);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// node-to-node tables and sums
// ---------------------------------------------------------------------------------------------
constexpr int NOFF = 16;   // tabulated integer box offsets per dimension

struct M2LGeom {
    int dqmin[MAXD];       // smallest tabulated offset per dimension
    double shift[MAXD];    // source-tree origin minus target-tree origin
};

// T[k][o][i][j] = exp(-lcs * (g_i - g_j - delta)^2), delta = (o + dqmin_k) * edge + shift_k,
// g = node * edge / 2 (the constant +edge/2 of n_tree.cu:510 cancels in the difference)
__global__ void m2l_table_kernel(NodeTab nt, int d, double edge, double lcs, M2LGeom geo, float *T) {
    const int p = nt.p;
    const int tot = d * NOFF * p * p;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < tot; e += gridDim.x * blockDim.x) {
        int jn = e % p, in = (e / p) % p, o = (e / (p * p)) % NOFF, k = e / (p * p * NOFF);
        double delta = (double)(o + geo.dqmin[k]) * edge + geo.shift[k];
        double diff = ((double)nt.node[in] - (double)nt.node[jn]) * edge * 0.5 - delta;
        T[e] = (float)exp(-lcs * diff * diff);
    }
}

template <int D>
__device__ __forceinline__ void decode_cell(uint32_t code, int level, int *q) {
#pragma unroll
    for (int k = 0; k < D; k++) q[k] = 0;
    for (int jb = 0; jb < level; jb++)
#pragma unroll
        for (int k = 0; k < D; k++) q[k] |= (int)((code >> (D * jb + k)) & 1u) << jb;
}

// One CTA per target box with a non-empty far row; threads own output entries (node, column).
template <int D, int RB, int EPT>
__global__ void m2l_kernel(int nbx, int level, const int *__restrict__ fptr, const int *__restrict__ fidx,
                           const uint32_t *__restrict__ code_x, const uint32_t *__restrict__ code_y,
                           const int *__restrict__ off_x, int row_begin, int row_end, const float *__restrict__ T,
                           M2LGeom geo, int p, int P, int R, int r0, const float *__restrict__ mom, float *loc,
                           int *err) {
    extern __shared__ float sm[];
    const int bx = blockIdx.x;
    const int e0 = fptr[bx], e1 = fptr[bx + 1];
    if (e0 == e1) return;
    { int o = off_x[bx]; if (o < row_begin || o >= row_end) return; }
    const int PR = P * RB;
    float *buf0 = sm, *buf1 = sm + PR;
    int qx[D];
    decode_cell<D>(code_x[bx], level, qx);
    float acc[EPT];
#pragma unroll
    for (int u = 0; u < EPT; u++) acc[u] = 0.f;
    int stride[D];
    { int s = 1;
#pragma unroll
      for (int k = 0; k < D; k++) { stride[k] = s; s *= p; } }
    for (int e = e0; e < e1; e++) {
        const int by = fidx[e];
        int qy[D];
        decode_cell<D>(code_y[by], level, qy);
        const float *Tk[D];
        bool ok = true;
#pragma unroll
        for (int k = 0; k < D; k++) {
            int o = qy[k] - qx[k] - geo.dqmin[k];
            if (o < 0 || o >= NOFF) { ok = false; o = 0; }
            Tk[k] = T + (size_t)(k * NOFF + o) * p * p;
        }
        if (!ok) { if (threadIdx.x == 0) atomicExch(err, 2); continue; }
        // load the source moments
        for (int q = threadIdx.x; q < PR; q += blockDim.x) {
            int m = q / RB, r = q - m * RB;
            buf0[q] = (r0 + r < R) ? mom[((size_t)by * P + m) * R + r0 + r] : 0.f;
        }
        __syncthreads();
        float *in = buf0, *out = buf1;
#pragma unroll
        for (int k = 0; k < D; k++) {
            const float *Tm = Tk[k];
            const int st = stride[k];
#pragma unroll
            for (int u = 0; u < EPT; u++) {
                int q = threadIdx.x + u * blockDim.x;
                if (q < PR) {
                    int m = q / RB, r = q - m * RB;
                    int mk = (m / st) % p;
                    const float *src = in + (size_t)(m - mk * st) * RB + r;
                    const float *trow = Tm + mk * p;
                    float s = 0.f;
                    for (int jn = 0; jn < p; jn++) s = fmaf(__ldg(trow + jn), src[(size_t)jn * st * RB], s);
                    if (k == D - 1) acc[u] += s; else out[q] = s;
                }
            }
            __syncthreads();
            float *tmp = in; in = out; out = tmp;
        }
    }
#pragma unroll
    for (int u = 0; u < EPT; u++) {
        int q = threadIdx.x + u * blockDim.x;
        if (q < PR) {
            int m = q / RB, r = q - m * RB;
            if (r0 + r < R) loc[((size_t)bx * P + m) * R + r0 + r] = acc[u];
        }
    }
}

// ---------------------------------------------------------------------------------------------
// L2P
// ---------------------------------------------------------------------------------------------
template <int D, int RB>
__global__ void __launch_bounds__(CH) l2p_kernel(const float *__restrict__ pts, int n, const int *__restrict__ off, int nb,
                                                const float *__restrict__ ctr, float factor, NodeTab nt,
                                                const int *__restrict__ fptr, int row_begin, int row_end, int P, int R,
                                                int r0, const float *__restrict__ loc, float *out) {
    extern __shared__ float sm[];
    const int p = nt.p;
    float *Ls = sm;   // [D*p][CH]
    const int j = threadIdx.x, i = blockIdx.x * CH + j;
    if (i >= n) return;
    const int box = box_of_row(off, nb, i);
    if (fptr[box + 1] == fptr[box]) return;
    { int o = off[box]; if (o < row_begin || o >= row_end) return; }
#pragma unroll
    for (int k = 0; k < D; k++) {
        float t = factor * (pts[(size_t)k * n + i] - ctr[box * D + k]);
        lagrange_1d(t, nt, Ls + (k * p) * CH + j, CH);
    }
    const float *lb = loc + (size_t)box * P * R + r0;
    float acc[RB];
#pragma unroll
    for (int r = 0; r < RB; r++) acc[r] = 0.f;
    const int outer = P / p;
    for (int o = 0; o < outer; o++) {
        float wgt = 1.f;
        int rem = o;
#pragma unroll
        for (int k = 1; k < D; k++) {
            wgt *= Ls[(k * p + rem % p) * CH + j];
            rem /= p;
        }
        float s[RB];
#pragma unroll
        for (int r = 0; r < RB; r++) s[r] = 0.f;
        for (int i0 = 0; i0 < p; i0++) {
            float l0 = Ls[i0 * CH + j];
            const float *lp = lb + (size_t)(o * p + i0) * R;
#pragma unroll
            for (int r = 0; r < RB; r++)
                if (r0 + r < R) s[r] = fmaf(l0, __ldg(lp + r), s[r]);
        }
#pragma unroll
        for (int r = 0; r < RB; r++) acc[r] = fmaf(wgt, s[r], acc[r]);
    }
#pragma unroll
    for (int r = 0; r < RB; r++)
        if (r0 + r < R) out[(size_t)i * R + r0 + r] += acc[r];
}

// ---------------------------------------------------------------------------------------------
// host driver for one level
// ---------------------------------------------------------------------------------------------
template <int D, int RB>
static void far_level_impl(f3m_plan *pl, int level, const float *bs, int R, int r0, float *out, int row_begin,
                           int row_end, cudaStream_t s) {
    Tree &tx = pl->tx, &ty = *pl->ty;
    Level &lx = tx.levels[level], &ly = ty.levels[level];
    LevelLists &ll = pl->lists[level];
    const int p = ll.p;
    int P = 1;
    for (int k = 0; k < D; k++) P *= p;
    NodeTab nt = make_nodes(p);
    const float factor = 2.f / lx.edge;
    const int n_y = (int)ty.n, n_x = (int)tx.n;

    // source boxes that appear in the far list
    DevBuf<unsigned char> need;
    need.alloc(ly.nb, s);
    need.zero();
    mark_sources<<<(unsigned)((ll.far.count + 255) / 256), 256, 0, s>>>(ll.far.idx.p, ll.far.count, need.p);
    F3M_LAUNCH_CHECK();

    DevBuf<float> mom, loc, T;
    mom.alloc((size_t)ly.nb * P * R, s);
    mom.zero();
    loc.alloc((size_t)lx.nb * P * R, s);
    pl->last.begin(ST_P2M, s);
    {
        size_t smem = ((size_t)D * p * (CH + 1) + (size_t)CH * RB) * sizeof(float);
        F3M_CUDA(cudaFuncSetAttribute(p2m_kernel<D, RB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        p2m_kernel<D, RB><<<(unsigned)((n_y + CH - 1) / CH), CH, smem, s>>>(ty.pts.p, n_y, bs, R, r0, ly.off.p, ly.nb, ly.ctr.p,
                                                                          factor, nt, need.p, P, mom.p);
        F3M_LAUNCH_CHECK();
    }
    pl->last.end(s);
    pl->last.begin(ST_M2L, s);
    {
        M2LGeom geo{};
        for (int k = 0; k < D; k++) {
            double sh = pl->same ? 0.0 : (double)ty.origin[k] - (double)tx.origin[k];
            geo.shift[k] = sh;
            // pairs of level >= 2 descend from parent pairs closer than two parent edges, so their
            // offset lies within a few boxes of -shift/edge; level-1 pairs are children of the root
            // pair, with offsets -1, 0, 1 wherever the two cubes are
            geo.dqmin[k] = (level == 1 ? 0 : (int)floor(-sh / (double)lx.edge)) - NOFF / 2 + 1;
        }
        T.alloc((size_t)D * NOFF * p * p, s);
        m2l_table_kernel<<<8, 256, 0, s>>>(nt, D, (double)lx.edge, (double)pl->lcs, geo, T.p);
        F3M_LAUNCH_CHECK();
        const int PR = P * RB;
        int threads = ((PR + 31) / 32) * 32;
        if (threads < 64) threads = 64;
        if (threads > 256) threads = 256;
        int ept = (PR + threads - 1) / threads;
        if (ept > 4 && threads < 1024) { threads = 1024; ept = (PR + threads - 1) / threads; }
        size_t smem = (size_t)2 * PR * sizeof(float);
        F3M_REQUIRE(ept <= 32 && smem <= 200 * 1024, F3M_ERR_UNSUPPORTED,
                    "%d interpolation nodes x %d columns exceed the node-to-node kernel's capacity", P, RB);
        int *d_err = pl->d_flags + FL_ERR;
#define F3M_M2L(E)                                                                                                   \
    {                                                                                                                \
        F3M_CUDA(cudaFuncSetAttribute(m2l_kernel<D, RB, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        m2l_kernel<D, RB, E><<<lx.nb, threads, smem, s>>>(lx.nb, level, ll.far.ptr.p, ll.far.idx.p, lx.code.p, ly.code.p, \
                                                          lx.off.p, row_begin, row_end, T.p, geo, p, P, R, r0, mom.p,   \
                                                          loc.p, d_err);                                               \
    }
        if (ept <= 1) F3M_M2L(1)
        else if (ept <= 2) F3M_M2L(2)
        else if (ept <= 4) F3M_M2L(4)
        else if (ept <= 8) F3M_M2L(8)
        else if (ept <= 16) F3M_M2L(16)
        else F3M_M2L(32)
#undef F3M_M2L
        F3M_LAUNCH_CHECK();
    }
    pl->last.end(s);
    pl->last.begin(ST_L2P, s);
    {
        size_t smem = (size_t)D * p * CH * sizeof(float);
        F3M_CUDA(cudaFuncSetAttribute(l2p_kernel<D, RB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        l2p_kernel<D, RB><<<(unsigned)((n_x + CH - 1) / CH), CH, smem, s>>>(tx.pts.p, n_x, lx.off.p, lx.nb, lx.ctr.p, factor, nt,
                                                                          ll.far.ptr.p, row_begin, row_end, P, R, r0,
                                                                          loc.p, out);
        F3M_LAUNCH_CHECK();
    }
    pl->last.end(s);
}

template <int D>
static void far_level_d(f3m_plan *pl, int level, const float *bs, int R, float *out, int rb, int re, cudaStream_t s) {
    // columns are processed in blocks of 1, 4 or 8
    int p = pl->lists[level].p, P = 1;
    for (int k = 0; k < D; k++) P *= p;
    for (int r0 = 0; r0 < R;) {
        int left = R - r0;
        if (left >= 8 && (size_t)P * 8 * 8 <= 200 * 1024) { far_level_impl<D, 8>(pl, level, bs, R, r0, out, rb, re, s); r0 += 8; }
        else if (left >= 2) { far_level_impl<D, 4>(pl, level, bs, R, r0, out, rb, re, s); r0 += 4; }
        else { far_level_impl<D, 1>(pl, level, bs, R, r0, out, rb, re, s); r0 += 1; }
    }
}

void far_field_level(f3m_plan *pl, int level, const float *b_sorted, int R, float *out_sorted, int64_t row_begin,
                     int64_t row_end, cudaStream_t s) {
    if (pl->lists[level].far.count == 0) return;
    F3M_REQUIRE(pl->lists[level].p <= MAXP, F3M_ERR_UNSUPPORTED, "%d nodes per dimension exceed the limit of %d",
                pl->lists[level].p, MAXP);
    switch (pl->d) {
        case 1: far_level_d<1>(pl, level, b_sorted, R, out_sorted, (int)row_begin, (int)row_end, s); break;
        case 2: far_level_d<2>(pl, level, b_sorted, R, out_sorted, (int)row_begin, (int)row_end, s); break;
        case 3: far_level_d<3>(pl, level, b_sorted, R, out_sorted, (int)row_begin, (int)row_end, s); break;
        case 4: far_level_d<4>(pl, level, b_sorted, R, out_sorted, (int)row_begin, (int)row_end, s); break;
        default: far_level_d<5>(pl, level, b_sorted, R, out_sorted, (int)row_begin, (int)row_end, s); break;
    }
}

}  // namespace f3m
