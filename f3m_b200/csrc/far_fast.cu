// Far field, fast path: one pass over the points, box-to-box translations in between.
//
// The reference interpolates every level directly from and to the points: P2M and L2P touch all N
// points at every level, and the node-to-node step evaluates P^2 exponentials per box pair
// (far_field_compute_v2, F3M_src/n_tree.cu:489-593; kernels F3M_src/1_d_conv.cu:451-659, 741-817).
// Here, with p nodes per dimension and P = p^d:
//
//   P2M   only at the finest level (one CTA per box, no atomics);
//   M2M   moments of a box = sum over its children of (A_s0 x A_s1 x ..) child moments, where
//         A_s[i][j] = L_i(s/2 + t_j/2) is the parent's 1-D Lagrange basis at the child's nodes.  A
//         parent basis function restricted to a child is a polynomial of degree p-1 per dimension, so
//         interpolating it on the child's p nodes is exact: these are the moments the reference
//         computes from the points, up to rounding;
//   M2L   per far pair the P x P Gaussian block is the Kronecker product of d tabulated p x p
//         matrices that depend only on the integer box offset per dimension: d*p*P multiply-adds and
//         no exponential per pair;
//   L2L   the transpose of M2M, pushing local expansions down to the finest level;
//   L2P   only at the finest level.
//
// All three translations are "apply d small matrices along the d axes of a p^d array"; a warp does
// that for one box (pair) at a time with the array in its own shared-memory buffers.  Every kernel
// here is bound by shared-memory / L2 bandwidth and FP32 issue, not HBM: the moment arrays of the
// finest level (boxes * P floats) are read a few times from L2/HBM, the points once.
#include <math.h>
#include <algorithm>
#include <vector>
#include "common.cuh"

namespace f3m {

constexpr int NOFF2 = 16;     // tabulated box offsets per dimension
constexpr int PMAX_FAST = 8;  // nodes per dimension handled by this path

struct NodeTab2 {
    int p;
    float node[PMAX_FAST];
    float w[PMAX_FAST];
};

struct Geom2 {
    int dqmin[MAXD];
    double shift[MAXD];
};

__host__ __device__ constexpr int mat_stride(int p) { return (p * p + 3) / 4 * 4; }

static NodeTab2 make_nodes2(int p) {
    NodeTab2 t{};
    t.p = p;
    cheb_nodes_weights(p, t.node, t.w);
    return t;
}

// ---------------------------------------------------------------------------------------------
// tables
// ---------------------------------------------------------------------------------------------
// T[k][o][i*p+j] = exp(-lcs (g_i - g_j - delta)^2), delta = (o + dqmin_k) edge + shift_k, g = node*edge/2
// (setup_skip_conv n_tree.cu:433-486 adds the centres to the scaled nodes; the +edge/2 of n_tree.cu:510 cancels)
__global__ void m2l_table2(NodeTab2 nt, int d, double edge, double lcs, Geom2 geo, float *T) {
    const int p = nt.p, MS = mat_stride(p);
    const int tot = d * NOFF2 * MS;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < tot; e += gridDim.x * blockDim.x) {
        int q = e % MS, o = (e / MS) % NOFF2, k = e / (MS * NOFF2);
        float v = 0.f;
        if (q < p * p) {
            int in = q / p, jn = q % p;
            double delta = (double)(o + geo.dqmin[k]) * edge + geo.shift[k];
            double diff = ((double)nt.node[in] - (double)nt.node[jn]) * edge * 0.5 - delta;
            v = (float)exp(-lcs * diff * diff);
        }
        T[e] = v;
    }
}

// A[s][i*p+j] = L_i(xi), xi = (s ? +0.5 : -0.5) + 0.5 t_j ; AT is its transpose.  Exact Lagrange products in double.
static void make_shift_tables(const NodeTab2 &nt, std::vector<float> &A, std::vector<float> &AT) {
    const int p = nt.p, MS = mat_stride(p);
    A.assign(2 * MS, 0.f);
    AT.assign(2 * MS, 0.f);
    for (int s = 0; s < 2; s++)
        for (int j = 0; j < p; j++) {
            double xi = (s ? 0.5 : -0.5) + 0.5 * (double)nt.node[j];
            for (int i = 0; i < p; i++) {
                double L = 1.0;
                for (int l = 0; l < p; l++)
                    if (l != i) L *= (xi - (double)nt.node[l]) / ((double)nt.node[i] - (double)nt.node[l]);
                A[s * MS + i * p + j] = (float)L;
                AT[s * MS + j * p + i] = (float)L;
            }
        }
}

// ---------------------------------------------------------------------------------------------
// warp-level "apply d matrices along the d axes"
// Array layout: index = m*RB + r, m = sum_k m_k p^k (dimension 0 fastest), r the column.
// Stage k transforms axis k: out[.., i, ..] = sum_j M_k[i][j] in[.., j, ..].  The last stage adds into acc.
// ---------------------------------------------------------------------------------------------
struct KronCfg {
    int d, RB, P, nf;        // nf = (P/p)*RB fibres per stage
    int st[MAXD];            // element stride of axis k: RB * p^k
    float inv_st[MAXD];
};

static KronCfg make_kron_cfg(int d, int p, int RB) {
    KronCfg c{};
    c.d = d; c.RB = RB;
    c.P = 1;
    for (int k = 0; k < d; k++) c.P *= p;
    c.nf = (c.P / p) * RB;
    int st = RB;
    for (int k = 0; k < MAXD; k++) {
        c.st[k] = st;
        c.inv_st[k] = 1.0f / (float)st;
        if (k < d) st *= p;
    }
    return c;
}

// A lane owns whole fibres (p consecutive entries along the axis being transformed): it loads the p x p
// matrix of the stage into registers once, then p inputs -> p outputs per fibre.  With ACC_REG the
// outputs of the last stage are accumulated in registers (possible when a stage has at most 64 fibres,
// i.e. two rounds per lane); otherwise in the warp's shared-memory accumulator.
__host__ __device__ constexpr int cpow(int b, int e) { return e <= 0 ? 1 : b * cpow(b, e - 1); }

// DD > 0: dimension known at compile time and one column (RB = 1): every stride is a constant, so the
// index arithmetic folds into immediate offsets.  DD = 0: dimension and column block taken from cfg.
template <int PP, bool ACC_REG, int DD>
__device__ __forceinline__ void warp_kron(const float *src0, float *bufA, float *bufB, float *acc_sm,
                                          float (&acc_reg)[2][PP], float &acc_left, const float *const (&mats)[MAXD],
                                          const KronCfg &cfg, int lane) {
    constexpr int MS = mat_stride(PP);
    const float *src = src0;
    float *dst = bufA;
    const int nf = DD ? cpow(PP, DD - 1) : cfg.nf;
    const int dd = DD ? DD : cfg.d;
#pragma unroll
    for (int k = 0; k < MAXD; k++) {
        if (k < dd) {
            const bool last = (k == dd - 1);
            const int st = DD ? cpow(PP, k) : cfg.st[k];
            const float inv = DD ? 1.0f / (float)cpow(PP, k) : cfg.inv_st[k];
            float M[MS];
            const float4 *M4 = reinterpret_cast<const float4 *>(mats[k]);
#pragma unroll
            for (int q = 0; q < MS / 4; q++) {
                float4 v = M4[q];
                M[4 * q] = v.x; M[4 * q + 1] = v.y; M[4 * q + 2] = v.z; M[4 * q + 3] = v.w;
            }
            auto fibre = [&](int f, float *areg) {
                const int hi = last ? 0 : (DD ? f / st : __float2int_rz(((float)f + 0.5f) * inv));
                const int base = hi * st * PP + (f - hi * st);
                float v[PP];
#pragma unroll
                for (int j = 0; j < PP; j++) v[j] = src[base + j * st];
#pragma unroll
                for (int i = 0; i < PP; i++) {
                    float o = 0.f;
#pragma unroll
                    for (int j = 0; j < PP; j++) o = fmaf(M[i * PP + j], v[j], o);
                    if (!last) dst[base + i * st] = o;
                    else if (ACC_REG) areg[i] += o;
                    else acc_sm[base + i * st] += o;
                }
            };
            if (ACC_REG) {   // at most two rounds, register accumulators indexed statically
                if (lane < nf) fibre(lane, acc_reg[0]);
                const int left = nf - 32;
                if (left > 0 && left * PP <= 32) {
                    // a short second round (e.g. 36 fibres): one OUTPUT per lane instead of one fibre per lane
                    if (lane < left * PP) {
                        const int lf = lane / PP, i = lane - lf * PP, f = 32 + lf;
                        const int hi = last ? 0 : (DD ? f / st : __float2int_rz(((float)f + 0.5f) * inv));
                        const int base = hi * st * PP + (f - hi * st);
                        const float *mrow = mats[k] + i * PP;
                        float o = 0.f;
#pragma unroll
                        for (int j = 0; j < PP; j++) o = fmaf(mrow[j], src[base + j * st], o);
                        if (!last) dst[base + i * st] = o;
                        else acc_left += o;
                    }
                } else if (lane + 32 < nf) fibre(lane + 32, acc_reg[1]);
            } else {
                for (int f = lane; f < nf; f += 32) fibre(f, acc_reg[0]);
            }
            __syncwarp();
            src = dst;
            dst = (dst == bufA) ? bufB : bufA;
        }
    }
}

// after the last pair: registers -> the warp's shared-memory accumulator (layout of the last stage: base = fibre)
template <int PP>
__device__ __forceinline__ void flush_acc(float (&acc_reg)[2][PP], float acc_left, float *acc_sm, const KronCfg &cfg,
                                          int lane) {
    const int st = cfg.st[cfg.d - 1];   // for one column this equals the number of fibres
    const int left = cfg.nf - 32;
    const bool short_round = left > 0 && left * PP <= 32;
#pragma unroll
    for (int rnd = 0; rnd < 2; rnd++) {
        const int f = lane + rnd * 32;
        if (f < cfg.nf && !(rnd == 1 && short_round))
#pragma unroll
            for (int i = 0; i < PP; i++) acc_sm[f + i * st] = acc_reg[rnd][i];
    }
    if (short_round && lane < left * PP) {
        const int lf = lane / PP, i = lane - lf * PP;
        acc_sm[32 + lf + i * st] = acc_left;
    }
}

__global__ void __launch_bounds__(256) decode_cells_kernel(int nb, int level, int d, const uint32_t *__restrict__ code, int *cell) {
    int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nb) return;
    const uint32_t c = code[b];
    for (int k = 0; k < d; k++) {
        int q = 0;
        for (int jb = 0; jb < level; jb++) q |= (int)((c >> (d * jb + k)) & 1u) << jb;
        cell[b * d + k] = q;
    }
}

__device__ __forceinline__ void decode_cell2(uint32_t code, int level, int d, int *q) {
    for (int k = 0; k < d; k++) q[k] = 0;
    for (int jb = 0; jb < level; jb++)
        for (int k = 0; k < d; k++) q[k] |= (int)((code >> (d * jb + k)) & 1u) << jb;
}

// ---------------------------------------------------------------------------------------------
// M2L: one CTA per target box, its warps share the far row
// ---------------------------------------------------------------------------------------------
template <int PP, bool ACC_REG, int DD>
__global__ void __launch_bounds__(128, 5) m2l_fast(int nbx, int d, const int *__restrict__ fptr, const int *__restrict__ fidx,
                                               const int *__restrict__ cell_x, const int *__restrict__ cell_y,
                                               const int *__restrict__ off_x, int row_begin, int row_end,
                                               const float *__restrict__ T, Geom2 geo, KronCfg cfg,
                                               const float *__restrict__ mom, float *loc, int *err) {
    extern __shared__ __align__(16) float sm[];
    constexpr int MS = mat_stride(PP);
    const int bx = blockIdx.x;
    const int e0 = fptr[bx], e1 = fptr[bx + 1];
    if (e0 == e1) return;
    if (off_x[bx + 1] <= row_begin || off_x[bx] >= row_end) return;   // box has no point in this rank's slice
    const int nw = blockDim.x >> 5, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int PR = cfg.P * cfg.RB, ntab = d * NOFF2 * MS;
    float *Tsm = sm;
    float *wbuf = sm + ntab + (size_t)w * 3 * PR;
    float *bufA = wbuf, *bufB = wbuf + PR, *acc = wbuf + 2 * PR;
    for (int q = threadIdx.x; q < ntab; q += blockDim.x) Tsm[q] = T[q];
    for (int q = lane; q < PR; q += 32) acc[q] = 0.f;
    float acc_reg[2][PP], acc_left = 0.f;
#pragma unroll
    for (int a = 0; a < 2; a++)
#pragma unroll
        for (int i = 0; i < PP; i++) acc_reg[a][i] = 0.f;
    __syncthreads();
    int qx[MAXD];
#pragma unroll
    for (int k = 0; k < MAXD; k++) qx[k] = k < d ? cell_x[bx * d + k] : 0;
    for (int e = e0 + w; e < e1; e += nw) {
        const int by = fidx[e];
        const float *mats[MAXD];
        bool ok = true;
#pragma unroll
        for (int k = 0; k < MAXD; k++) {
            int o = 0;
            if (k < d) {
                o = cell_y[by * d + k] - qx[k] - geo.dqmin[k];
                if (o < 0 || o >= NOFF2) { ok = false; o = 0; }
            }
            mats[k] = Tsm + (k * NOFF2 + o) * MS;
        }
        if (!ok) { if (lane == 0) atomicExch(err, 2); continue; }
        warp_kron<PP, ACC_REG, DD>(mom + (size_t)by * PR, bufA, bufB, acc, acc_reg, acc_left, mats, cfg, lane);
    }
    if (ACC_REG) flush_acc<PP>(acc_reg, acc_left, acc, cfg, lane);
    __syncthreads();
    for (int q = threadIdx.x; q < PR; q += blockDim.x) {
        float s = 0.f;
        for (int ww = 0; ww < nw; ww++) s += sm[ntab + (size_t)ww * 3 * PR + 2 * PR + q];
        loc[(size_t)bx * PR + q] = s;
    }
}

// ---------------------------------------------------------------------------------------------
// M2L, nested form (d = 2, 3, one column).  T(pair) = T_{d-1}(o_{d-1}) x .. x T_0(o_0) and the sum over the
// far pairs of a target box can be taken axis by axis:
//     loc = sum_{o0} T0(o0) [ sum_{o1} T1(o1) [ sum_{o2} T2(o2) mom(o0,o1,o2) ] ]
// With the row ordered by (o0, o1, o2) only the last-axis transform is applied per pair; the axis-1 transform
// once per (o0,o1) group and the axis-0 transform once per o0 group: ~240 instead of 567 stage applications
// for the 189 far pairs of an interior box.  Any order is correct (a group is flushed whenever the higher
// offsets change), ordering only increases the sharing.
// ---------------------------------------------------------------------------------------------
// One warp per target box: packed offsets of its far pairs (axis 0 most significant) and the row in
// ascending order of them.  The source boxes of one row have distinct cells, hence distinct keys below
// 16^3: the rank of a key is the number of set bits below it in a bitmap of the row.
// In four and five dimensions the rank key is the base-8 number of the offsets counted from the lowest one
// that can occur (tabulated offset 4): 8^4 and 8^5 keys.  An offset outside that window is clamped; if two
// pairs of a row then share a rank key the row keeps its list order (every order is correct, see above).
template <int WPL>   // bitmap words per lane: 4 -> 4096 rank keys, 32 -> 32768
__global__ void __launch_bounds__(128) far_order_kernel(int nbx, int d, const int *__restrict__ fptr, const int *__restrict__ fidx,
                                                       const int *__restrict__ cell_x, const int *__restrict__ cell_y,
                                                       Geom2 geo, uint32_t *okey, int *oidx, int *err,
                                                       const int *__restrict__ off_x, int row_begin, int row_end) {
    constexpr int ORD_WORDS = 32 * WPL;
    __shared__ uint32_t bits[4][ORD_WORDS];
    __shared__ int below[4][ORD_WORDS];
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bx = blockIdx.x * 4 + w;
    if (bx >= nbx) return;
    if (off_x[bx + 1] <= row_begin || off_x[bx] >= row_end) return;   // no row of this box in the slice being computed
    const int e0 = fptr[bx], n = fptr[bx + 1] - e0;
    if (n == 0) return;
    const bool compact = d > 3;
    // key: one nibble per axis, last axis lowest, axis 0 on top; rkey: what the row is ordered by
    auto key_of = [&](int by, uint32_t &rkey) {
        uint32_t key = 0;
        rkey = 0;
        for (int k = 0; k < d; k++) {
            int o = cell_y[by * d + k] - cell_x[bx * d + k] - geo.dqmin[k];
            if (o < 0 || o >= NOFF2) { atomicExch(err, 2); o = 0; }
            key |= (uint32_t)o << (4 * (d - 1 - k));
            rkey = rkey * 8u + (uint32_t)min(max(o - 4, 0), 7);
        }
        if (!compact) rkey = key;
        return key;
    };
    for (int q = lane; q < ORD_WORDS; q += 32) bits[w][q] = 0u;
    __syncwarp();
    for (int i = lane; i < n; i += 32) {
        uint32_t rkey;
        key_of(fidx[e0 + i], rkey);
        atomicOr(&bits[w][rkey >> 5], 1u << (rkey & 31u));
    }
    __syncwarp();
    // exclusive prefix of the word populations: WPL words per lane, then a warp scan
    int tot = 0;
#pragma unroll 4
    for (int q = 0; q < WPL; q++) tot += __popc(bits[w][lane * WPL + q]);
    int incl = tot;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { int v = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += v; }
    int run = incl - tot;
#pragma unroll 4
    for (int q = 0; q < WPL; q++) { below[w][lane * WPL + q] = run; run += __popc(bits[w][lane * WPL + q]); }
    const int distinct = __shfl_sync(0xffffffffu, incl, 31);
    __syncwarp();
    if (distinct != n) {   // cannot happen for d <= 3 (boxes of one level have distinct cells); keep the list order
        if (lane == 0 && !compact) atomicExch(err, 2);
        for (int i = lane; i < n; i += 32) { int by = fidx[e0 + i]; uint32_t rk; okey[e0 + i] = key_of(by, rk); oidx[e0 + i] = by; }
        return;
    }
    for (int i = lane; i < n; i += 32) {
        const int by = fidx[e0 + i];
        uint32_t rkey;
        const uint32_t key = key_of(by, rkey);
        const int rank = below[w][rkey >> 5] + __popc(bits[w][rkey >> 5] & ((1u << (rkey & 31u)) - 1u));
        okey[e0 + rank] = key;
        oidx[e0 + rank] = by;
    }
}

// Accumulators of one lane for one buffer of the nested transform: the fibres lane and lane+32 of the
// axis that produced it, or (when only a few fibres are left after the first 32) one output of a fibre
// beyond 32 per lane.
template <int PP>
struct FibreAcc {
    float r0[PP], r1[PP], left;
    __device__ __forceinline__ void clear() {
#pragma unroll
        for (int i = 0; i < PP; i++) r0[i] = r1[i] = 0.f;
        left = 0.f;
    }
};

template <int PP, int DD>
struct NestGeom {
    static constexpr int MS = mat_stride(PP);
    static constexpr int P = cpow(PP, DD);
    static constexpr int nf = cpow(PP, DD - 1);
    static constexpr int left = nf - 32;
    static constexpr bool short_round = left > 0 && left * PP <= 32;
    static constexpr bool second_round = left > 0 && !short_round;
    template <int K>
    static __device__ __forceinline__ int base(int f) {
        constexpr int st = cpow(PP, K);
        const int hi = f / st;
        return hi * st * PP + (f - hi * st);
    }
};

// inputs of one lane for one application along axis K
template <int PP>
struct FibreIn {
    float v0[PP], v1[PP];
};

template <int PP, int K, int DD, bool GLOBAL>
__device__ __forceinline__ void nest_load(const float *src, FibreIn<PP> &in, int lane) {
    using G = NestGeom<PP, DD>;
    constexpr int st = cpow(PP, K);
    if (lane < G::nf) {
        const int base = G::template base<K>(lane);
#pragma unroll
        for (int j = 0; j < PP; j++) in.v0[j] = GLOBAL ? __ldg(src + base + j * st) : src[base + j * st];
    }
    if (G::short_round) {
        if (lane < G::left * PP) {
            const int base = G::template base<K>(32 + lane / PP);
#pragma unroll
            for (int j = 0; j < PP; j++) in.v1[j] = GLOBAL ? __ldg(src + base + j * st) : src[base + j * st];
        }
    } else if (G::second_round) {
        if (lane + 32 < G::nf) {
            const int base = G::template base<K>(lane + 32);
#pragma unroll
            for (int j = 0; j < PP; j++) in.v1[j] = GLOBAL ? __ldg(src + base + j * st) : src[base + j * st];
        }
    }
}

// out += M_k applied along the axis to the loaded fibres
template <int PP, int DD>
__device__ __forceinline__ void nest_apply(const FibreIn<PP> &in, const float *Mk, FibreAcc<PP> &out, int lane) {
    using G = NestGeom<PP, DD>;
    float M[G::MS];
    const float4 *M4 = reinterpret_cast<const float4 *>(Mk);
#pragma unroll
    for (int q = 0; q < G::MS / 4; q++) {
        float4 v = M4[q];
        M[4 * q] = v.x; M[4 * q + 1] = v.y; M[4 * q + 2] = v.z; M[4 * q + 3] = v.w;
    }
    if (lane < G::nf) {
#pragma unroll
        for (int i = 0; i < PP; i++) {
            float o = 0.f;
#pragma unroll
            for (int j = 0; j < PP; j++) o = fmaf(M[i * PP + j], in.v0[j], o);
            out.r0[i] += o;
        }
    }
    if (G::short_round) {
        if (lane < G::left * PP) {
            const float *mrow = Mk + (lane % PP) * PP;
            float o = 0.f;
#pragma unroll
            for (int j = 0; j < PP; j++) o = fmaf(mrow[j], in.v1[j], o);
            out.left += o;
        }
    } else if (G::second_round) {
        if (lane + 32 < G::nf) {
#pragma unroll
            for (int i = 0; i < PP; i++) {
                float o = 0.f;
#pragma unroll
                for (int j = 0; j < PP; j++) o = fmaf(M[i * PP + j], in.v1[j], o);
                out.r1[i] += o;
            }
        }
    }
}

// registers -> shared memory in the layout of axis K (the axis that produced them), then clear
template <int PP, int K, int DD>
__device__ __forceinline__ void nest_spill(FibreAcc<PP> &a, float *dst, int lane) {
    using G = NestGeom<PP, DD>;
    constexpr int st = cpow(PP, K);
    if (lane < G::nf) {
        const int base = G::template base<K>(lane);
#pragma unroll
        for (int i = 0; i < PP; i++) dst[base + i * st] = a.r0[i];
    }
    if (G::short_round) {
        if (lane < G::left * PP) dst[G::template base<K>(32 + lane / PP) + (lane % PP) * st] = a.left;
    } else if (G::second_round) {
        if (lane + 32 < G::nf) {
            const int base = G::template base<K>(lane + 32);
#pragma unroll
            for (int i = 0; i < PP; i++) dst[base + i * st] = a.r1[i];
        }
    }
    a.clear();
}

// The per-pair transform runs along the LAST axis (its fibres are strided by the number of fibres, so a
// warp reads 32 consecutive floats per load); the packed key of a pair holds the offset of that axis in
// its lowest 4 bits, the next axis above it, axis 0 on top.
template <int PP, int DD>
__global__ void __launch_bounds__(128, PP <= 6 ? 4 : 2) m2l_nested(int nbx, const int *__restrict__ fptr,
                                                                   const uint32_t *__restrict__ okey, const int *__restrict__ oidx,
                                                                   const int *__restrict__ off_x, int row_begin, int row_end,
                                                                   const float *__restrict__ T, const float *__restrict__ mom,
                                                                   float *loc) {
    extern __shared__ __align__(16) float sm[];
    using G = NestGeom<PP, DD>;
    constexpr int MS = G::MS, P = G::P;
    constexpr int KA = DD - 1;               // axis applied per pair
    const int bx = blockIdx.x;
    const int e0 = fptr[bx], e1 = fptr[bx + 1];
    if (e0 == e1) return;
    if (off_x[bx + 1] <= row_begin || off_x[bx] >= row_end) return;
    const int nw = blockDim.x >> 5, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int ntab = DD * NOFF2 * MS;
    float *Tsm = sm;
    float *buf = sm + ntab + (size_t)w * P;  // one transpose buffer per warp
    for (int q = threadIdx.x; q < ntab; q += blockDim.x) Tsm[q] = T[q];
    FibreAcc<PP> V, U, A;
    V.clear(); U.clear(); A.clear();
    __syncthreads();
    const int len = e1 - e0;
    const int cb = e0 + (int)(((long long)len * w) / nw), ce = e0 + (int)(((long long)len * (w + 1)) / nw);
    // matrix of axis k for the offset stored in nibble (DD-1-k) of the key
    auto mat = [&](int k, uint32_t key) { return Tsm + (k * NOFF2 + ((key >> (4 * (DD - 1 - k))) & 15u)) * MS; };
    auto close_groups = [&](uint32_t key, bool all) {
        FibreIn<PP> in;
        nest_spill<PP, KA, DD>(V, buf, lane);
        __syncwarp();
        if (DD == 3) {
            nest_load<PP, 1, DD, false>(buf, in, lane);
            nest_apply<PP, DD>(in, mat(1, key), U, lane);
            __syncwarp();
            if (all) {
                nest_spill<PP, 1, DD>(U, buf, lane);
                __syncwarp();
                nest_load<PP, 0, DD, false>(buf, in, lane);
                nest_apply<PP, DD>(in, mat(0, key), A, lane);
                __syncwarp();
            }
        } else {
            nest_load<PP, 0, DD, false>(buf, in, lane);
            nest_apply<PP, DD>(in, mat(0, key), A, lane);
            __syncwarp();
        }
    };
    uint32_t prev = 0xffffffffu;
    for (int c = cb; c < ce; c += 32) {
        const int cn = min(32, ce - c);
        uint32_t mykey = 0;
        int myidx = 0;
        if (lane < cn) { mykey = okey[c + lane]; myidx = oidx[c + lane]; }
        FibreIn<PP> cur;
        nest_load<PP, KA, DD, true>(mom + (size_t)__shfl_sync(0xffffffffu, myidx, 0) * P, cur, lane);
        for (int t = 0; t < cn; t++) {
            const uint32_t key = __shfl_sync(0xffffffffu, mykey, t);
            FibreIn<PP> nxt;
            const int tn = min(t + 1, cn - 1);   // the last one re-reads itself: no branch around the loads
            nest_load<PP, KA, DD, true>(mom + (size_t)__shfl_sync(0xffffffffu, myidx, tn) * P, nxt, lane);
            if (prev != 0xffffffffu && (key >> 4) != (prev >> 4)) close_groups(prev, DD == 3 ? (key >> 8) != (prev >> 8) : true);
            nest_apply<PP, DD>(cur, mat(KA, key), V, lane);
            prev = key;
            cur = nxt;
        }
    }
    if (prev != 0xffffffffu) close_groups(prev, true);
    // layout of axis 0: the lane's fibre is PP consecutive entries
    float *accw = sm + ntab + (size_t)w * P;
    nest_spill<PP, 0, DD>(A, accw, lane);
    __syncthreads();
    for (int q = threadIdx.x; q < P; q += blockDim.x) {
        float s = 0.f;
        for (int ww = 0; ww < nw; ww++) s += sm[ntab + (size_t)ww * P + q];
        loc[(size_t)bx * P + q] = s;
    }
}

// ---------------------------------------------------------------------------------------------
// M2L, nested form for several columns and for d = 4, 5: one CTA per target box, every thread owns FPT
// fibres of each axis and keeps the partial sums of ALL nesting levels in registers.  A far pair costs one
// coalesced read of the source box's moments and the last-axis transform, with no shared-memory traffic;
// shared memory is only used to re-lay the sums out for the next axis when a group of offsets closes.
// ---------------------------------------------------------------------------------------------
template <int PP, int DD, int RBB>
struct RowCfg {
    static constexpr int MS = mat_stride(PP);
    static constexpr int P = cpow(PP, DD), PR = P * RBB, NF = PR / PP;
    static constexpr int MAX_ACC = 64;   // accumulator registers of a thread over all levels
    static constexpr int pick_threads() {
        int best = 0;
        long best_u = -1;
        for (int nt = 32; nt <= 256; nt += 32) {
            const int fpt = (NF + nt - 1) / nt;
            if (DD * fpt * PP > MAX_ACC) continue;
            const long u = (long)NF * 1000000 / ((long)fpt * nt);   // share of fibre slots that hold a fibre
            if (u >= best_u) { best_u = u; best = nt; }
        }
        return best;
    }
    static constexpr int NT = pick_threads();
    static constexpr int FPT = NT ? (NF + NT - 1) / NT : 1;
    static constexpr int DEPTH = FPT * PP * 4 <= 40 ? 4 : 2;   // source boxes in flight per CTA (divides 32)
    static constexpr size_t smem = ((size_t)DD * NOFF2 * MS + (size_t)PR) * sizeof(float);
    static constexpr bool ok = NT > 0 && smem <= 160 * 1024;
    template <int K>
    static __device__ __forceinline__ int base(int f) {
        constexpr int st = RBB * cpow(PP, K);
        const int hi = f / st;
        return hi * st * PP + (f - hi * st);
    }
};

template <int PP>
__device__ __forceinline__ void load_matrix(const float *Mk, float (&M)[mat_stride(PP)]) {
    const float4 *M4 = reinterpret_cast<const float4 *>(Mk);
#pragma unroll
    for (int q = 0; q < mat_stride(PP) / 4; q++) {
        float4 v = M4[q];
        M[4 * q] = v.x; M[4 * q + 1] = v.y; M[4 * q + 2] = v.z; M[4 * q + 3] = v.w;
    }
}

// Closes nesting level K: the sums over the last offsets (axes K..DD-1 already applied) go through shared memory
// into the layout of axis K-1, that axis' matrix for the group's offset is applied, and the result is added to
// level K-1; level K-1 closes too when the offsets above it change.
template <int PP, int DD, int RBB, int K>
__device__ __forceinline__ void rows_close(float (&acc)[DD][RowCfg<PP, DD, RBB>::FPT][PP], float *buf, const float *Tsm,
                                           uint32_t prev, uint32_t key, bool final, int tid) {
    using C = RowCfg<PP, DD, RBB>;
    if constexpr (K >= 1) {
        constexpr int stK = RBB * cpow(PP, K), stL = RBB * cpow(PP, K - 1);
#pragma unroll
        for (int r = 0; r < C::FPT; r++) {
            const int f = tid + r * C::NT;
            if (f < C::NF) {
                const int base = C::template base<K>(f);
#pragma unroll
                for (int i = 0; i < PP; i++) { buf[base + i * stK] = acc[K][r][i]; acc[K][r][i] = 0.f; }
            }
        }
        __syncthreads();
        float M[C::MS];
        load_matrix<PP>(Tsm + ((K - 1) * NOFF2 + ((prev >> (4 * (DD - K))) & 15u)) * C::MS, M);
#pragma unroll
        for (int r = 0; r < C::FPT; r++) {
            const int f = tid + r * C::NT;
            if (f < C::NF) {
                const int base = C::template base<K - 1>(f);
                float v[PP];
#pragma unroll
                for (int j = 0; j < PP; j++) v[j] = buf[base + j * stL];
#pragma unroll
                for (int i = 0; i < PP; i++) {
                    float o = 0.f;
#pragma unroll
                    for (int j = 0; j < PP; j++) o = fmaf(M[i * PP + j], v[j], o);
                    acc[K - 1][r][i] += o;
                }
            }
        }
        __syncthreads();
        if constexpr (K >= 2) {
            constexpr int sh = 4 * (DD - K + 1);   // nibbles of the axes K-1..DD-1
            if (final || (key >> sh) != (prev >> sh)) rows_close<PP, DD, RBB, K - 1>(acc, buf, Tsm, prev, key, final, tid);
        }
    }
}

template <int PP, int DD, int RBB>
__global__ void __launch_bounds__(RowCfg<PP, DD, RBB>::NT ? RowCfg<PP, DD, RBB>::NT : 32)
m2l_rows(int nbx, const int *__restrict__ fptr, const uint32_t *__restrict__ okey, const int *__restrict__ oidx,
         const int *__restrict__ off_x, int row_begin, int row_end, const float *__restrict__ T,
         const float *__restrict__ mom, float *loc) {
    using C = RowCfg<PP, DD, RBB>;
    constexpr int MS = C::MS, PR = C::PR, NF = C::NF, NT = C::NT ? C::NT : 32, FPT = C::FPT;
    constexpr int KA = DD - 1;   // axis applied per pair: its fibres are strided by NF, fibre f starts at element f
    extern __shared__ __align__(16) float sm[];
    const int bx = blockIdx.x, tid = threadIdx.x, lane = tid & 31;
    const int e0 = fptr[bx], e1 = fptr[bx + 1];
    if (e0 == e1) return;
    if (off_x[bx + 1] <= row_begin || off_x[bx] >= row_end) return;
    constexpr int ntab = DD * NOFF2 * MS;
    float *Tsm = sm, *buf = sm + ntab;
    for (int q = tid; q < ntab; q += NT) Tsm[q] = T[q];
    float acc[DD][FPT][PP];
#pragma unroll
    for (int k = 0; k < DD; k++)
#pragma unroll
        for (int r = 0; r < FPT; r++)
#pragma unroll
            for (int i = 0; i < PP; i++) acc[k][r][i] = 0.f;
    __syncthreads();
    auto fetch = [&](int by, float (&v)[FPT][PP]) {
        const float *src = mom + (size_t)by * PR;
#pragma unroll
        for (int r = 0; r < FPT; r++) {
            const int f = tid + r * NT;
#pragma unroll
            for (int j = 0; j < PP; j++) v[r][j] = f < NF ? __ldg(src + f + j * NF) : 0.f;
        }
    };
    // DEPTH source boxes are on their way while one is consumed; the row's keys and boxes are read 32 at a time, one
    // per lane, the next 32 a chunk ahead (entries past the end of the row repeat its last pair and are never consumed)
    constexpr int DEPTH = C::DEPTH;
    float pre[DEPTH][FPT][PP];
    uint32_t prev = 0xffffffffu;
    int nxtidx = oidx[min(e0 + lane, e1 - 1)];
    uint32_t nxtkey = okey[min(e0 + lane, e1 - 1)];
#pragma unroll
    for (int u = 0; u < DEPTH; u++) fetch(__shfl_sync(0xffffffffu, nxtidx, u), pre[u]);
    for (int c = e0; c < e1; c += 32) {
        const int cn = min(32, e1 - c);
        const uint32_t mykey = nxtkey;
        const int myidx = nxtidx;
        nxtidx = oidx[min(c + 32 + lane, e1 - 1)];
        nxtkey = okey[min(c + 32 + lane, e1 - 1)];
        for (int t0 = 0; t0 < cn; t0 += DEPTH) {
#pragma unroll
            for (int u = 0; u < DEPTH; u++) {
                const int t = t0 + u;
                if (t < cn) {
                    const uint32_t key = __shfl_sync(0xffffffffu, mykey, t);
                    if (prev != 0xffffffffu && (key >> 4) != (prev >> 4))
                        rows_close<PP, DD, RBB, KA>(acc, buf, Tsm, prev, key, false, tid);
                    float M[MS];
                    load_matrix<PP>(Tsm + (KA * NOFF2 + (key & 15u)) * MS, M);
#pragma unroll
                    for (int r = 0; r < FPT; r++)
#pragma unroll
                        for (int i = 0; i < PP; i++) {
                            float o = 0.f;
#pragma unroll
                            for (int j = 0; j < PP; j++) o = fmaf(M[i * PP + j], pre[u][r][j], o);
                            acc[KA][r][i] += o;
                        }
                    prev = key;
                    const int ahead = t + DEPTH;
                    const int a0 = __shfl_sync(0xffffffffu, myidx, ahead & 31), a1 = __shfl_sync(0xffffffffu, nxtidx, ahead & 31);
                    fetch(ahead < 32 ? a0 : a1, pre[u]);
                }
            }
        }
    }
    rows_close<PP, DD, RBB, KA>(acc, buf, Tsm, prev, prev, true, tid);
    // level 0 holds the box's local expansion in the layout of axis 0
    float *dst = loc + (size_t)bx * PR;
#pragma unroll
    for (int r = 0; r < FPT; r++) {
        const int f = tid + r * NT;
        if (f < NF) {
            const int base = C::template base<0>(f);
#pragma unroll
            for (int i = 0; i < PP; i++) dst[base + i * RBB] = acc[0][r][i];
        }
    }
}

// Host side of m2l_rows: the kernel exists for the (nodes, dimension, columns) whose accumulators fit the registers.
template <int PP, int DD, int RBB>
static bool m2l_rows_launch_one(bool probe, int nbx, const int *fptr, const uint32_t *okey, const int *oidx, const int *offx, int rb,
                                int re, const float *T, const float *mom, float *loc, cudaStream_t s) {
    using C = RowCfg<PP, DD, RBB>;
    if constexpr (C::ok) {
        if (probe) return true;
        F3M_CUDA(cudaFuncSetAttribute(m2l_rows<PP, DD, RBB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::smem));
        m2l_rows<PP, DD, RBB><<<nbx, C::NT, C::smem, s>>>(nbx, fptr, okey, oidx, offx, rb, re, T, mom, loc);
        return true;
    } else
        return false;
}

template <int PP, int RBB>
static bool m2l_rows_dispatch(bool probe, int d, int nbx, const int *fptr, const uint32_t *okey, const int *oidx, const int *offx,
                              int rb, int re, const float *T, const float *mom, float *loc, cudaStream_t s) {
    switch (d) {
    case 2: return m2l_rows_launch_one<PP, 2, RBB>(probe, nbx, fptr, okey, oidx, offx, rb, re, T, mom, loc, s);
    case 3: return m2l_rows_launch_one<PP, 3, RBB>(probe, nbx, fptr, okey, oidx, offx, rb, re, T, mom, loc, s);
    case 4: return m2l_rows_launch_one<PP, 4, RBB>(probe, nbx, fptr, okey, oidx, offx, rb, re, T, mom, loc, s);
    case 5: return m2l_rows_launch_one<PP, 5, RBB>(probe, nbx, fptr, okey, oidx, offx, rb, re, T, mom, loc, s);
    default: return false;
    }
}

template <int PP, int RBB>
static bool rows_form_available(int d) {
    return m2l_rows_dispatch<PP, RBB>(true, d, 0, nullptr, nullptr, nullptr, nullptr, 0, 0, nullptr, nullptr, nullptr, nullptr);
}

template <int PP, int RBB>
static void launch_m2l_rows(int d, int nbx, const int *fptr, const uint32_t *okey, const int *oidx, const int *offx, int rb, int re,
                            const float *T, const float *mom, float *loc, cudaStream_t s) {
    m2l_rows_dispatch<PP, RBB>(false, d, nbx, fptr, okey, oidx, offx, rb, re, T, mom, loc, s);
}

// M2M: one CTA per parent box, warps share the children
template <int PP>
__global__ void __launch_bounds__(128) m2m_fast(int nbp, int d, const int *__restrict__ child_start,
                                               const uint32_t *__restrict__ code_child, const float *__restrict__ A,
                                               KronCfg cfg, const float *__restrict__ mom_child, float *mom_parent) {
    extern __shared__ __align__(16) float sm[];
    constexpr int MS = mat_stride(PP);
    const int pb = blockIdx.x;
    const int nw = blockDim.x >> 5, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int PR = cfg.P * cfg.RB, ntab = 2 * MS;
    float *Asm = sm;
    float *wbuf = sm + ntab + (size_t)w * 3 * PR;
    float *bufA = wbuf, *bufB = wbuf + PR, *acc = wbuf + 2 * PR;
    for (int q = threadIdx.x; q < ntab; q += blockDim.x) Asm[q] = A[q];
    for (int q = lane; q < PR; q += 32) acc[q] = 0.f;
    float acc_reg[2][PP], acc_left = 0.f;
    __syncthreads();
    const int c0 = child_start[pb], c1 = child_start[pb + 1];
    for (int c = c0 + w; c < c1; c += nw) {
        const uint32_t code = code_child[c];
        const float *mats[MAXD];
#pragma unroll
        for (int k = 0; k < MAXD; k++) mats[k] = Asm + ((code >> k) & 1u) * MS;
        warp_kron<PP, false, 0>(mom_child + (size_t)c * PR, bufA, bufB, acc, acc_reg, acc_left, mats, cfg, lane);
    }
    __syncthreads();
    for (int q = threadIdx.x; q < PR; q += blockDim.x) {
        float s = 0.f;
        for (int ww = 0; ww < nw; ww++) s += sm[ntab + (size_t)ww * 3 * PR + 2 * PR + q];
        mom_parent[(size_t)pb * PR + q] = s;
    }
}

// L2L: one warp per child box
template <int PP>
__global__ void __launch_bounds__(128) l2l_fast(int nbc, int d, const int *__restrict__ parent,
                                               const uint32_t *__restrict__ code_child, const int *__restrict__ off_c,
                                               int row_begin, int row_end, const float *__restrict__ AT, KronCfg cfg,
                                               const float *__restrict__ loc_parent, float *loc_child) {
    extern __shared__ __align__(16) float sm[];
    constexpr int MS = mat_stride(PP);
    const int nw = blockDim.x >> 5, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int PR = cfg.P * cfg.RB, ntab = 2 * MS;
    float *Asm = sm;
    float *wbuf = sm + ntab + (size_t)w * 3 * PR;
    float *bufA = wbuf, *bufB = wbuf + PR, *acc = wbuf + 2 * PR;
    for (int q = threadIdx.x; q < ntab; q += blockDim.x) Asm[q] = AT[q];
    __syncthreads();
    const int c = blockIdx.x * nw + w;
    if (c >= nbc) return;
    if (off_c[c + 1] <= row_begin || off_c[c] >= row_end) return;
    for (int q = lane; q < PR; q += 32) acc[q] = 0.f;
    __syncwarp();
    const uint32_t code = code_child[c];
    const float *mats[MAXD];
#pragma unroll
    for (int k = 0; k < MAXD; k++) mats[k] = Asm + ((code >> k) & 1u) * MS;
    float acc_reg[2][PP], acc_left = 0.f;
    warp_kron<PP, false, 0>(loc_parent + (size_t)parent[c] * PR, bufA, bufB, acc, acc_reg, acc_left, mats, cfg, lane);
    for (int q = lane; q < PR; q += 32) loc_child[(size_t)c * PR + q] += acc[q];
}

// ---------------------------------------------------------------------------------------------
// P2M / L2P at the finest level: one CTA per (box, split)
// ---------------------------------------------------------------------------------------------
// Barycentric Lagrange basis (lagrange_data_load + calculate_barycentric_lagrange, 1_d_conv.cu:217-238, 418-448)
template <int PP>
__device__ __forceinline__ void lagrange_pp(float t, const NodeTab2 &nt, float *L) {
    // q_i = w_i / (t - t_i) with the fast reciprocal (2 ulp): L_i = q_i / sum_l q_l.  The reference's kernels are
    // built with --use_fast_math, so their divisions are the approximate ones too.
    int hit = -1;
    float sum = 0.f;
    float q[PP];
#pragma unroll
    for (int i = 0; i < PP; i++) {
        const float diff = t - nt.node[i];
        if (diff == 0.f) hit = i;
        q[i] = __fdividef(nt.w[i], diff);
        sum += q[i];
    }
    if (hit >= 0) {
#pragma unroll
        for (int i = 0; i < PP; i++) L[i] = (i == hit) ? 1.f : 0.f;
    } else {
        const float lx = __fdividef(1.f, sum);
#pragma unroll
        for (int i = 0; i < PP; i++) L[i] = lx * q[i];
    }
}

// P2M.  A thread owns one combination (m_1 .. m_{d-1}) of the slower node indices and all p values of
// the fastest one: per point it forms w = b * prod_{k>=1} L_k[m_k] once and adds w * L_0[i] to p
// accumulators, so a (point, node) pair costs about one shared-memory read and one multiply-add.
// Threads beyond the number of combinations form further groups that take every G-th point.
template <int PP, int RB>
__global__ void __launch_bounds__(256) p2m_leaf(const float *__restrict__ pts, int n, int d, const float *__restrict__ bs, int R,
                                               int r0, const int *__restrict__ off, const float *__restrict__ ctr,
                                               float factor, NodeTab2 nt, int P, int nsplit, int src_begin, int src_end,
                                               float *mom) {
    extern __shared__ __align__(16) float sm[];
    constexpr int TP = 128, NTH = 256, LS = TP + 1;
    float *Ls = sm;                                   // [d*PP][TP+1]
    float *bsm = Ls + (size_t)d * PP * LS;            // [TP][RB]
    float *accsm = bsm + (size_t)TP * RB;             // [P][RB]
    const int box = blockIdx.x;
    const int a = off[box], b = off[box + 1];
    if (a < src_begin || a >= src_end) return;      // only the boxes of this slice of the sorted sources
    const int len = b - a;
    const int s0 = a + (int)(((long long)len * blockIdx.y) / nsplit), s1 = a + (int)(((long long)len * (blockIdx.y + 1)) / nsplit);
    if (s0 >= s1) return;
    const int PR = P * RB, C = P / PP;
    // the PP x RB block of one combination starts an odd number of floats after the previous one: the lanes of a
    // warp (consecutive combinations) then add to different banks
    constexpr int CS = (PP * RB) | 1;
    for (int q = threadIdx.x; q < C * CS; q += NTH) accsm[q] = 0.f;
    float c[MAXD];
    for (int k = 0; k < d; k++) c[k] = ctr[box * d + k];
    const int G = C >= NTH ? 1 : NTH / C;             // point groups
    const int g = C >= NTH ? 0 : threadIdx.x / C;
    for (int base = s0; base < s1; base += TP) {
        const int cnt = min(TP, s1 - base);
        __syncthreads();
        if ((int)threadIdx.x < cnt) {
            const int i = base + threadIdx.x;
            for (int k = 0; k < d; k++) {
                float L[PP];
                lagrange_pp<PP>(factor * (pts[(size_t)k * n + i] - c[k]), nt, L);
#pragma unroll
                for (int q = 0; q < PP; q++) Ls[(k * PP + q) * LS + threadIdx.x] = L[q];
            }
#pragma unroll
            for (int r = 0; r < RB; r++) bsm[threadIdx.x * RB + r] = (r0 + r < R) ? bs[(size_t)i * R + r0 + r] : 0.f;
        }
        __syncthreads();
        if (g < G) {
            for (int cc = (C >= NTH ? (int)threadIdx.x : (int)threadIdx.x - g * C); cc < C; cc += NTH) {
                const float *lp[MAXD];
                int rem = cc;
#pragma unroll
                for (int k = 1; k < MAXD; k++) {
                    lp[k] = Ls;
                    if (k < d) { lp[k] = Ls + (size_t)(k * PP + rem % PP) * LS; rem /= PP; }
                }
                float acc[PP][RB];
#pragma unroll
                for (int i = 0; i < PP; i++)
#pragma unroll
                    for (int r = 0; r < RB; r++) acc[i][r] = 0.f;
                for (int j = g; j < cnt; j += G) {
                    float w = 1.f;
#pragma unroll
                    for (int k = 1; k < MAXD; k++)
                        if (k < d) w *= lp[k][j];
                    float wb[RB];
#pragma unroll
                    for (int r = 0; r < RB; r++) wb[r] = w * bsm[j * RB + r];
#pragma unroll
                    for (int i = 0; i < PP; i++) {
                        const float l0 = Ls[i * LS + j];
#pragma unroll
                        for (int r = 0; r < RB; r++) acc[i][r] = fmaf(l0, wb[r], acc[i][r]);
                    }
                }
#pragma unroll
                for (int i = 0; i < PP; i++)
#pragma unroll
                    for (int r = 0; r < RB; r++) atomicAdd(&accsm[cc * CS + i * RB + r], acc[i][r]);
            }
        }
    }
    __syncthreads();
    float *dst = mom + (size_t)box * PR;
    constexpr int BLK = PP * RB;
    if (nsplit == 1) for (int q = threadIdx.x; q < PR; q += NTH) dst[q] = accsm[q + (q / BLK) * (CS - BLK)];
    else for (int q = threadIdx.x; q < PR; q += NTH) atomicAdd(dst + q, accsm[q + (q / BLK) * (CS - BLK)]);
}

template <int PP, int RB>
__global__ void __launch_bounds__(128) l2p_leaf(const float *__restrict__ pts, int n, int d, const int *__restrict__ off,
                                               const float *__restrict__ ctr, float factor, NodeTab2 nt, int P, int nsplit,
                                               int row_begin, int row_end, const float *__restrict__ loc, int R, int r0,
                                               float *out) {
    extern __shared__ __align__(16) float sm[];
    constexpr int TP = 128;
    const int PR = P * RB;
    float *locsm = sm;                 // [P][RB]
    float *Ls = sm + PR;               // [(d-1)*PP][TP]
    const int box = blockIdx.x;
    const int a = off[box], b = off[box + 1];
    if (a < row_begin || a >= row_end) return;    // finest-level boxes belong to the slice their first point is in
    const int len = b - a;
    const int s0 = a + (int)(((long long)len * blockIdx.y) / nsplit), s1 = a + (int)(((long long)len * (blockIdx.y + 1)) / nsplit);
    if (s0 >= s1) return;
    for (int q = threadIdx.x; q < PR; q += TP) locsm[q] = loc[(size_t)box * PR + q];
    __syncthreads();
    float c[MAXD];
    for (int k = 0; k < d; k++) c[k] = ctr[box * d + k];
    const int outer = P / PP;
    for (int i = s0 + threadIdx.x; i < s1; i += TP) {
        float l0[PP];
        lagrange_pp<PP>(factor * (pts[i] - c[0]), nt, l0);
        for (int k = 1; k < d; k++) {
            float L[PP];
            lagrange_pp<PP>(factor * (pts[(size_t)k * n + i] - c[k]), nt, L);
#pragma unroll
            for (int q = 0; q < PP; q++) Ls[((k - 1) * PP + q) * TP + threadIdx.x] = L[q];
        }
        float acc[RB];
#pragma unroll
        for (int r = 0; r < RB; r++) acc[r] = 0.f;
        for (int o = 0; o < outer; o++) {
            float wgt = 1.f;
            int rem = o;
            for (int k = 1; k < d; k++) {
                wgt *= Ls[((k - 1) * PP + rem % PP) * TP + threadIdx.x];
                rem /= PP;
            }
            float sacc[RB];
#pragma unroll
            for (int r = 0; r < RB; r++) sacc[r] = 0.f;
            const float *lp = locsm + (size_t)o * PP * RB;
#pragma unroll
            for (int i0 = 0; i0 < PP; i0++)
#pragma unroll
                for (int r = 0; r < RB; r++) sacc[r] = fmaf(l0[i0], lp[i0 * RB + r], sacc[r]);
#pragma unroll
            for (int r = 0; r < RB; r++) acc[r] = fmaf(wgt, sacc[r], acc[r]);
        }
#pragma unroll
        for (int r = 0; r < RB; r++)
            if (r0 + r < R) out[(size_t)i * R + r0 + r] += acc[r];
    }
}

// ---------------------------------------------------------------------------------------------
// P2M / L2P for d = 3 and one column, register-tiled.  A lane is (point stream, m2): it keeps the PP x PP block
// (m0, m1) of the box's moments (or local expansion) for its m2 in registers, so a point costs the lane PP
// multiplies and PP^2 multiply-adds against 4 broadcast 16-byte loads and one 4-byte load of the point's Lagrange
// rows -- the multiply-add rate, not shared memory, is the limit.  32 / PP streams per warp, 4 warps per CTA, one box
// per CTA (blockIdx.y splits very large boxes).  The rows [L0 (8) | L1 (8) | L2 (8) | pad (4)] are 28 floats apart,
// which puts the rows of the streams of one warp on different banks.
// ---------------------------------------------------------------------------------------------
constexpr int L3_RS = 28;
template <int PP>
struct Leaf3 {
    static constexpr int SUB = 32 / PP;              // point streams per warp
    static constexpr int NSTREAM = 4 * SUB;          // per CTA
    static constexpr int TP = NSTREAM * (128 / NSTREAM);   // points per chunk
};

template <int PP>
__device__ __forceinline__ void leaf3_rows(const float *__restrict__ pts, int n, int i, const float (&c)[3], float factor,
                                           const NodeTab2 &nt, float scale2, float *row) {
    float L[PP];
#pragma unroll
    for (int k = 0; k < 3; k++) {
        lagrange_pp<PP>(factor * (pts[(size_t)k * n + i] - c[k]), nt, L);
#pragma unroll
        for (int q = 0; q < PP; q++) row[8 * k + q] = (k == 2) ? scale2 * L[q] : L[q];
    }
}

// the same from coordinates already in registers (the loads of a chunk are issued while the previous chunk is consumed)
template <int PP>
__device__ __forceinline__ void leaf3_rows_xyz(const float (&x)[3], const float (&c)[3], float factor, const NodeTab2 &nt,
                                               float scale2, float *row) {
    float L[PP];
#pragma unroll
    for (int k = 0; k < 3; k++) {
        lagrange_pp<PP>(factor * (x[k] - c[k]), nt, L);
#pragma unroll
        for (int q = 0; q < PP; q++) row[8 * k + q] = (k == 2) ? scale2 * L[q] : L[q];
    }
}

template <int PP>
__global__ void __launch_bounds__(128) p2m_leaf3(const float *__restrict__ pts, int n, const float *__restrict__ bs, int R, int r0,
                                                const int *__restrict__ off, const float *__restrict__ ctr, float factor,
                                                NodeTab2 nt, int nsplit, int src_begin, int src_end, float *mom,
                                                const int *__restrict__ box_list) {
    using G = Leaf3<PP>;
    constexpr int P = PP * PP * PP;
    // the Lagrange rows of a chunk; after the last chunk the same memory holds one partial moment array per stream
    constexpr int NSCR = (G::TP * L3_RS > G::NSTREAM * P) ? G::TP * L3_RS : G::NSTREAM * P;
    __shared__ __align__(16) float rows[NSCR];
    const int box = box_list ? box_list[blockIdx.x] : (int)blockIdx.x;
    const int a = off[box], b = off[box + 1];
    if (a < src_begin || a >= src_end) return;      // only the boxes of this slice of the sorted sources
    const int len = b - a;
    const int s0 = a + (int)(((long long)len * blockIdx.y) / nsplit), s1 = a + (int)(((long long)len * (blockIdx.y + 1)) / nsplit);
    if (s0 >= s1) return;
    const float c[3] = {ctr[box * 3], ctr[box * 3 + 1], ctr[box * 3 + 2]};
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane / PP, m2 = lane - sub * PP;
    const bool active = sub < G::SUB;
    const int stream = warp * G::SUB + sub;
    float acc[PP][PP];
#pragma unroll
    for (int i = 0; i < PP; i++)
#pragma unroll
        for (int j = 0; j < PP; j++) acc[i][j] = 0.f;
    // the point of the next chunk is fetched while the streams consume the current one
    float px[3] = {0.f, 0.f, 0.f}, pb = 0.f;
    auto fetch = [&](int base) {
        const int i = base + (int)threadIdx.x;
        if (i < s1) {
            px[0] = pts[i]; px[1] = pts[(size_t)n + i]; px[2] = pts[(size_t)2 * n + i];
            pb = bs[(size_t)i * R + r0];
        }
    };
    fetch(s0);
    for (int base = s0; base < s1; base += G::TP) {
        const int cnt = min(G::TP, s1 - base);
        __syncthreads();
        if ((int)threadIdx.x < cnt)   // the column value rides on the L2 row
            leaf3_rows_xyz<PP>(px, c, factor, nt, pb, rows + threadIdx.x * L3_RS);
        fetch(base + G::TP);
        __syncthreads();
        if (active)
            for (int j = stream; j < cnt; j += G::NSTREAM) {
                const float *row = rows + j * L3_RS;
                const float4 a0 = *reinterpret_cast<const float4 *>(row), a1 = *reinterpret_cast<const float4 *>(row + 4);
                const float4 b0 = *reinterpret_cast<const float4 *>(row + 8), b1 = *reinterpret_cast<const float4 *>(row + 12);
                const float l0[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                const float l1[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
                const float w2 = row[16 + m2];
#pragma unroll
                for (int i1 = 0; i1 < PP; i1++) {
                    const float u = w2 * l1[i1];
#pragma unroll
                    for (int i0 = 0; i0 < PP; i0++) acc[i1][i0] = fmaf(u, l0[i0], acc[i1][i0]);
                }
            }
    }
    __syncthreads();
    if (active) {
        float *mine = rows + stream * P + PP * PP * m2;
#pragma unroll
        for (int i1 = 0; i1 < PP; i1++)
#pragma unroll
            for (int i0 = 0; i0 < PP; i0++) mine[i0 + PP * i1] = acc[i1][i0];
    }
    __syncthreads();
    float *dst = mom + (size_t)box * P;
    for (int q = threadIdx.x; q < P; q += 128) {
        float v = 0.f;
#pragma unroll
        for (int st = 0; st < G::NSTREAM; st++) v += rows[st * P + q];
        if (nsplit == 1) dst[q] = v;
        else atomicAdd(dst + q, v);
    }
}

template <int PP>
__global__ void __launch_bounds__(128) l2p_leaf3(const float *__restrict__ pts, int n, const int *__restrict__ off,
                                                const float *__restrict__ ctr, float factor, NodeTab2 nt, int nsplit,
                                                int row_begin, int row_end, const float *__restrict__ loc, int R, int r0,
                                                float *out, const int *__restrict__ box_list) {
    using G = Leaf3<PP>;
    constexpr int P = PP * PP * PP;
    __shared__ __align__(16) float rows[G::TP * L3_RS];
    __shared__ float part[G::TP * 8];   // per point: the PP partial sums over m2
    const int box = box_list ? box_list[blockIdx.x] : (int)blockIdx.x;
    const int a = off[box], b = off[box + 1];
    if (a < row_begin || a >= row_end) return;    // finest-level boxes belong to the slice their first point is in
    const int len = b - a;
    const int s0 = a + (int)(((long long)len * blockIdx.y) / nsplit), s1 = a + (int)(((long long)len * (blockIdx.y + 1)) / nsplit);
    if (s0 >= s1) return;
    const float c[3] = {ctr[box * 3], ctr[box * 3 + 1], ctr[box * 3 + 2]};
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane / PP, m2 = lane - sub * PP;
    const bool active = sub < G::SUB;
    const int stream = warp * G::SUB + sub;
    float lc[PP][PP];   // loc[m0][m1][m2] of this lane's m2
#pragma unroll
    for (int i1 = 0; i1 < PP; i1++)
#pragma unroll
        for (int i0 = 0; i0 < PP; i0++) lc[i1][i0] = active ? __ldg(loc + (size_t)box * P + i0 + PP * i1 + PP * PP * m2) : 0.f;
    float px[3] = {0.f, 0.f, 0.f};
    auto fetch = [&](int base) {
        const int i = base + (int)threadIdx.x;
        if (i < s1) { px[0] = pts[i]; px[1] = pts[(size_t)n + i]; px[2] = pts[(size_t)2 * n + i]; }
    };
    fetch(s0);
    for (int base = s0; base < s1; base += G::TP) {
        const int cnt = min(G::TP, s1 - base);
        __syncthreads();
        if ((int)threadIdx.x < cnt) leaf3_rows_xyz<PP>(px, c, factor, nt, 1.f, rows + threadIdx.x * L3_RS);
        fetch(base + G::TP);   // the next chunk's point, while the streams consume this one
        __syncthreads();
        if (active)
            for (int j = stream; j < cnt; j += G::NSTREAM) {
                const float *row = rows + j * L3_RS;
                const float4 a0 = *reinterpret_cast<const float4 *>(row), a1 = *reinterpret_cast<const float4 *>(row + 4);
                const float4 b0 = *reinterpret_cast<const float4 *>(row + 8), b1 = *reinterpret_cast<const float4 *>(row + 12);
                const float l0[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                const float l1[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
                float sacc = 0.f;
#pragma unroll
                for (int i1 = 0; i1 < PP; i1++) {
                    float t = 0.f;
#pragma unroll
                    for (int i0 = 0; i0 < PP; i0++) t = fmaf(l0[i0], lc[i1][i0], t);
                    sacc = fmaf(l1[i1], t, sacc);
                }
                part[j * 8 + m2] = row[16 + m2] * sacc;
            }
        __syncthreads();
        if ((int)threadIdx.x < cnt) {
            float v = 0.f;
#pragma unroll
            for (int q = 0; q < PP; q++) v += part[threadIdx.x * 8 + q];
            out[(size_t)(base + threadIdx.x) * R + r0] += v;
        }
    }
}

// Small finest-level boxes (clustered data leaves millions of boxes with a handful of points): one warp per box, so
// that a box costs a few hundred instructions instead of a CTA's launch, barriers and reductions.
constexpr int LEAF_SMALL = 32;

__global__ void __launch_bounds__(256) split_leaf_boxes(int nb, const int *__restrict__ off, int *small_list, int *big_list, int *counts) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nb) return;
    const int len = off[b + 1] - off[b];
    if (len <= LEAF_SMALL) small_list[atomicAdd(counts, 1)] = b;
    else big_list[atomicAdd(counts + 1, 1)] = b;
}

// P2M: lanes = nodes (ceil(P / 32) per lane), points in turn; the points' Lagrange rows go through shared memory
template <int PP>
__global__ void __launch_bounds__(128) p2m_small3(const float *__restrict__ pts, int n, const float *__restrict__ bs, int R, int r0,
                                                 const int *__restrict__ off, const float *__restrict__ ctr, float factor,
                                                 NodeTab2 nt, int src_begin, int src_end, float *mom,
                                                 const int *__restrict__ box_list, int nlist) {
    constexpr int P = PP * PP * PP, NPL = (P + 31) / 32;
    __shared__ __align__(16) float rows_s[4][LEAF_SMALL * L3_RS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int li = blockIdx.x * 4 + warp;
    if (li >= nlist) return;
    const int box = box_list[li];
    const int a = off[box], len = off[box + 1] - a;
    if (a < src_begin || a >= src_end) return;
    const float c[3] = {ctr[box * 3], ctr[box * 3 + 1], ctr[box * 3 + 2]};
    float *rows = rows_s[warp];
    if (lane < len) leaf3_rows<PP>(pts, n, a + lane, c, factor, nt, bs[(size_t)(a + lane) * R + r0], rows + lane * L3_RS);
    __syncwarp();
    float acc[NPL];
    int o0[NPL], o1[NPL], o2[NPL];
#pragma unroll
    for (int q = 0; q < NPL; q++) {
        const int m = min(lane + 32 * q, P - 1);
        acc[q] = 0.f;
        o0[q] = m % PP; o1[q] = 8 + (m / PP) % PP; o2[q] = 16 + m / (PP * PP);
    }
    for (int j = 0; j < len; j++) {
        const float *row = rows + j * L3_RS;
#pragma unroll
        for (int q = 0; q < NPL; q++) acc[q] = fmaf(row[o2[q]] * row[o1[q]], row[o0[q]], acc[q]);
    }
#pragma unroll
    for (int q = 0; q < NPL; q++)
        if (lane + 32 * q < P) mom[(size_t)box * P + lane + 32 * q] = acc[q];
}

// L2P: lanes = points; the box's local expansion is staged in shared memory and read by every lane
template <int PP>
__global__ void __launch_bounds__(128) l2p_small3(const float *__restrict__ pts, int n, const int *__restrict__ off,
                                                 const float *__restrict__ ctr, float factor, NodeTab2 nt, int row_begin,
                                                 int row_end, const float *__restrict__ loc, int R, int r0, float *out,
                                                 const int *__restrict__ box_list, int nlist) {
    constexpr int P = PP * PP * PP;
    __shared__ float loc_s[4][P];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int li = blockIdx.x * 4 + warp;
    if (li >= nlist) return;
    const int box = box_list[li];
    const int a = off[box], len = off[box + 1] - a;
    if (a < row_begin || a >= row_end) return;
    for (int q = lane; q < P; q += 32) loc_s[warp][q] = __ldg(loc + (size_t)box * P + q);
    __syncwarp();
    if (lane >= len) return;
    const float c[3] = {ctr[box * 3], ctr[box * 3 + 1], ctr[box * 3 + 2]};
    float row[24];
    leaf3_rows<PP>(pts, n, a + lane, c, factor, nt, 1.f, row);
    float v = 0.f;
#pragma unroll
    for (int i2 = 0; i2 < PP; i2++) {
        float s2 = 0.f;
#pragma unroll
        for (int i1 = 0; i1 < PP; i1++) {
            float s1 = 0.f;
#pragma unroll
            for (int i0 = 0; i0 < PP; i0++) s1 = fmaf(row[i0], loc_s[warp][i0 + PP * i1 + PP * PP * i2], s1);
            s2 = fmaf(row[8 + i1], s1, s2);
        }
        v = fmaf(row[16 + i2], s2, v);
    }
    out[(size_t)(a + lane) * R + r0] += v;
}

// lists of the small and the large finest-level boxes of one tree (0: targets, 1: sources), built once per plan
static void ensure_leaf_split(f3m_plan *pl, int which, Level &lv, cudaStream_t s) {
    if (pl->leaf_split[which]) return;
    pl->leaf_small[which].alloc((size_t)lv.nb, s);
    pl->leaf_big[which].alloc((size_t)lv.nb, s);
    int *counts = pl->d_flags + FL_LEAF;
    F3M_CUDA(cudaMemsetAsync(counts, 0, 2 * sizeof(int), s));
    split_leaf_boxes<<<(lv.nb + 255) / 256, 256, 0, s>>>(lv.nb, lv.off.p, pl->leaf_small[which].p, pl->leaf_big[which].p, counts);
    F3M_LAUNCH_CHECK();
    F3M_CUDA(cudaMemcpyAsync(pl->h_pinned, counts, 2 * sizeof(int), cudaMemcpyDeviceToHost, s));
    F3M_CUDA(cudaStreamSynchronize(s));
    pl->n_leaf_small[which] = pl->h_pinned[0];
    pl->n_leaf_big[which] = pl->h_pinned[1];
    pl->leaf_split[which] = true;
}

// ---------------------------------------------------------------------------------------------
// host driver
// ---------------------------------------------------------------------------------------------
template <int PP, int RB>
static void far_fast_block(f3m_plan *pl, const float *bs, int R, int r0, float *out, int rb, int re, int lmin,
                           cudaStream_t s) {
    Tree &tx = pl->tx, &ty = *pl->ty;
    const int d = pl->d, L = pl->levels;
    int P = 1;
    for (int k = 0; k < d; k++) P *= PP;
    const int PR = P * RB;
    constexpr int MS = mat_stride(PP);
    NodeTab2 nt = make_nodes2(PP);
    const KronCfg cfg = make_kron_cfg(d, PP, RB);
    const int n_x = (int)tx.n, n_y = (int)ty.n;
    if (RB == 1 && d == 3) {
        ensure_leaf_split(pl, 0, tx.levels[L], s);
        if (!pl->same) ensure_leaf_split(pl, 1, ty.levels[L], s);
    }

    if (pl->moments_out) {
        // sharded P2M: finest-level moments of the source boxes that start in [mom_begin, mom_end), zero elsewhere
        Level &ly = ty.levels[L];
        if (pl->mom_box_end >= 0)   // the caller's array holds the boxes [mom_box_begin, mom_box_end) only
            F3M_CUDA(cudaMemsetAsync(pl->moments_out + pl->mom_box_begin * PR, 0,
                                     (size_t)(pl->mom_box_end - pl->mom_box_begin) * PR * sizeof(float), s));
        else
            F3M_CUDA(cudaMemsetAsync(pl->moments_out, 0, (size_t)ly.nb * PR * sizeof(float), s));
        int nsplit = std::max(1, std::min(64, (ly.max_count + 8191) / 8192));
        size_t smem = ((size_t)d * PP * 129 + (size_t)128 * RB + (size_t)PR + (size_t)(P / PP)) * sizeof(float);
        F3M_CUDA(cudaFuncSetAttribute(p2m_leaf<PP, RB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        pl->last.begin(ST_P2M, s);
        if (RB == 1 && d == 3) {
            const int wy = pl->same ? 0 : 1;
            if (pl->n_leaf_big[wy])
                p2m_leaf3<PP><<<dim3(pl->n_leaf_big[wy], nsplit), 128, 0, s>>>(ty.pts.p, n_y, bs, R, r0, ly.off.p, ly.ctr.p, 2.f / ly.edge, nt,
                                                                             nsplit > 1 ? nsplit : 1, (int)pl->mom_begin, (int)pl->mom_end,
                                                                             pl->moments_out, pl->leaf_big[wy].p);
            if (pl->n_leaf_small[wy])
                p2m_small3<PP><<<(pl->n_leaf_small[wy] + 3) / 4, 128, 0, s>>>(ty.pts.p, n_y, bs, R, r0, ly.off.p, ly.ctr.p, 2.f / ly.edge, nt,
                                                                            (int)pl->mom_begin, (int)pl->mom_end, pl->moments_out,
                                                                            pl->leaf_small[wy].p, pl->n_leaf_small[wy]);
        } else
        p2m_leaf<PP, RB><<<dim3(ly.nb, nsplit), 256, smem, s>>>(ty.pts.p, n_y, d, bs, R, r0, ly.off.p, ly.ctr.p, 2.f / ly.edge, nt, P,
                                                              nsplit > 1 ? nsplit : 1, (int)pl->mom_begin, (int)pl->mom_end,
                                                              pl->moments_out);
        pl->last.end(s);
        F3M_LAUNCH_CHECK();
        return;
    }
    std::vector<DevBuf<float>> mom(L + 1), loc(L + 1);
    std::vector<const float *> momp(L + 1, nullptr);
    for (int l = lmin; l <= L; l++) {
        if (!(l == L && pl->ext_mom)) mom[l].alloc((size_t)ty.levels[l].nb * PR, s);
        momp[l] = (l == L && pl->ext_mom) ? pl->ext_mom : mom[l].p;
        loc[l].alloc((size_t)tx.levels[l].nb * PR, s);
        loc[l].zero();
    }
    std::vector<float> hA, hAT;
    make_shift_tables(nt, hA, hAT);
    DevBuf<float> A, AT;
    A.alloc(hA.size(), s); AT.alloc(hAT.size(), s);
    F3M_CUDA(cudaMemcpyAsync(A.p, hA.data(), hA.size() * sizeof(float), cudaMemcpyHostToDevice, s));
    F3M_CUDA(cudaMemcpyAsync(AT.p, hAT.data(), hAT.size() * sizeof(float), cudaMemcpyHostToDevice, s));
    F3M_CUDA(cudaStreamSynchronize(s));   // hA / hAT are pageable host vectors

    // warps per CTA of the translation kernels, limited by shared memory
    const size_t per_warp = (size_t)3 * PR * sizeof(float);
    auto warps_for = [&](size_t table_bytes) {
        size_t avail = 200 * 1024 - table_bytes;
        int nw = (int)std::min<size_t>(4, avail / per_warp);
        return nw;
    };

    // ---- P2M at the finest level, M2M upwards ---------------------------------------------------
    pl->last.begin(ST_P2M, s);
    {
        Level &ly = ty.levels[L];
        const float factor = 2.f / ly.edge;          // 1_d_conv.cu:473
        if (!pl->ext_mom) {
            int nsplit = std::max(1, std::min(64, (ly.max_count + 8191) / 8192));
            if (nsplit > 1) mom[L].zero();
            size_t smem = ((size_t)d * PP * 129 + (size_t)128 * RB + (size_t)PR + (size_t)(P / PP)) * sizeof(float);
            F3M_CUDA(cudaFuncSetAttribute(p2m_leaf<PP, RB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            if (RB == 1 && d == 3) {
                const int wy = pl->same ? 0 : 1;
                if (pl->n_leaf_big[wy])
                    p2m_leaf3<PP><<<dim3(pl->n_leaf_big[wy], nsplit), 128, 0, s>>>(ty.pts.p, n_y, bs, R, r0, ly.off.p, ly.ctr.p, factor, nt,
                                                                                 nsplit, 0, n_y, mom[L].p, pl->leaf_big[wy].p);
                if (pl->n_leaf_small[wy])
                    p2m_small3<PP><<<(pl->n_leaf_small[wy] + 3) / 4, 128, 0, s>>>(ty.pts.p, n_y, bs, R, r0, ly.off.p, ly.ctr.p, factor, nt, 0,
                                                                                n_y, mom[L].p, pl->leaf_small[wy].p, pl->n_leaf_small[wy]);
            } else
            p2m_leaf<PP, RB><<<dim3(ly.nb, nsplit), 256, smem, s>>>(ty.pts.p, n_y, d, bs, R, r0, ly.off.p, ly.ctr.p, factor, nt, P,
                                                                  nsplit, 0, n_y, mom[L].p);
            F3M_LAUNCH_CHECK();
        }
        const int nw = warps_for(2 * MS * sizeof(float));
        size_t sm2 = (size_t)2 * MS * sizeof(float) + nw * per_warp;
        F3M_CUDA(cudaFuncSetAttribute(m2m_fast<PP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm2));
        for (int l = L - 1; l >= lmin; l--) {
            Level &lp = ty.levels[l], &lc = ty.levels[l + 1];
            m2m_fast<PP><<<lp.nb, 32 * nw, sm2, s>>>(lp.nb, d, lp.child_start.p, lc.code.p, A.p, cfg, momp[l + 1], mom[l].p);
            F3M_LAUNCH_CHECK();
        }
    }
    pl->last.end(s);
    // ---- M2L at every level that has far pairs -------------------------------------------------
    pl->last.begin(ST_M2L, s);
    {
        DevBuf<float> T;
        T.alloc((size_t)d * NOFF2 * MS, s);
        const size_t tab = (size_t)d * NOFF2 * MS * sizeof(float);
        const int nw = warps_for(tab);
        size_t smem = tab + nw * per_warp;
        const bool acc_reg = cfg.nf <= 64;
        // launcher: static strides for d = 2, 3 with one column, runtime strides otherwise
        auto launch_m2l = [&](int nbx, const int *fptr, const int *fidx, const int *cx, const int *cy, const int *offx,
                              const Geom2 &geo, const float *momL, float *locL) {
#define F3M_M2L_CALL(ACC_, DD_)                                                                                          \
    {                                                                                                                    \
        F3M_CUDA(cudaFuncSetAttribute(m2l_fast<PP, ACC_, DD_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        m2l_fast<PP, ACC_, DD_><<<nbx, 32 * nw, smem, s>>>(nbx, d, fptr, fidx, cx, cy, offx, rb, re, T.p, geo, cfg, momL,  \
                                                          locL, pl->d_flags);                                            \
    }
            if (RB == 1 && d == 3) { if (acc_reg) F3M_M2L_CALL(true, 3) else F3M_M2L_CALL(false, 3) }
            else if (RB == 1 && d == 2) { if (acc_reg) F3M_M2L_CALL(true, 2) else F3M_M2L_CALL(false, 2) }
            else { if (acc_reg) F3M_M2L_CALL(true, 0) else F3M_M2L_CALL(false, 0) }
#undef F3M_M2L_CALL
        };
        DevBuf<int> cellx, celly;
        for (int l = lmin; l <= L; l++) {
            LevelLists &ll = pl->lists[l];
            if (ll.far.count == 0) continue;
            Level &lx = tx.levels[l], &ly = ty.levels[l];
            Geom2 geo{};
            for (int k = 0; k < d; k++) {
                double sh = pl->same ? 0.0 : (double)ty.origin[k] - (double)tx.origin[k];
                geo.shift[k] = sh;
                // pairs of level >= 2 descend from parent pairs closer than two parent edges, so their offset lies
                // within a few boxes of -shift/edge; level-1 pairs are children of the root pair: offsets -1, 0, 1
                geo.dqmin[k] = (l == 1 ? 0 : (int)floor(-sh / (double)lx.edge)) - NOFF2 / 2 + 1;
            }
            m2l_table2<<<8, 256, 0, s>>>(nt, d, (double)lx.edge, (double)pl->lcs, geo, T.p);
            F3M_LAUNCH_CHECK();
            cellx.alloc((size_t)lx.nb * d, s);
            decode_cells_kernel<<<(lx.nb + 255) / 256, 256, 0, s>>>(lx.nb, l, d, lx.code.p, cellx.p);
            F3M_LAUNCH_CHECK();
            const int *cy = cellx.p;
            if (!pl->same) {
                celly.alloc((size_t)ly.nb * d, s);
                decode_cells_kernel<<<(ly.nb + 255) / 256, 256, 0, s>>>(ly.nb, l, d, ly.code.p, celly.p);
                F3M_LAUNCH_CHECK();
                cy = celly.p;
            }
            const bool nested = RB == 1 && (d == 2 || d == 3) && cfg.nf <= 64;
            const bool rows = !nested && rows_form_available<PP, RB>(d);
            if (nested || rows) {
                if (!ll.far_ordered) {
                    ll.far_okey.alloc((size_t)ll.far.count, s);
                    ll.far_oidx.alloc((size_t)ll.far.count, s);
                    if (d <= 4)
                        far_order_kernel<4><<<(lx.nb + 3) / 4, 128, 0, s>>>(lx.nb, d, ll.far.ptr.p, ll.far.idx.p, cellx.p, cy, geo,
                                                                           ll.far_okey.p, ll.far_oidx.p, pl->d_flags, lx.off.p, rb, re);
                    else
                        far_order_kernel<32><<<(lx.nb + 3) / 4, 128, 0, s>>>(lx.nb, d, ll.far.ptr.p, ll.far.idx.p, cellx.p, cy, geo,
                                                                            ll.far_okey.p, ll.far_oidx.p, pl->d_flags, lx.off.p, rb, re);
                    F3M_LAUNCH_CHECK();
                    // kept for later products of this plan only when every box was ordered
                    ll.far_ordered = rb <= 0 && re >= n_x;
                }
            }
            if (rows) {
                launch_m2l_rows<PP, RB>(d, lx.nb, ll.far.ptr.p, ll.far_okey.p, ll.far_oidx.p, lx.off.p, rb, re, T.p, momp[l], loc[l].p, s);
            } else if (nested) {
                const size_t smem_n = tab + (size_t)4 * P * sizeof(float);   // tables + one buffer per warp
                if (d == 3) {
                    F3M_CUDA(cudaFuncSetAttribute(m2l_nested<PP, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_n));
                    m2l_nested<PP, 3><<<lx.nb, 128, smem_n, s>>>(lx.nb, ll.far.ptr.p, ll.far_okey.p, ll.far_oidx.p, lx.off.p, rb, re,
                                                                  T.p, momp[l], loc[l].p);
                } else {
                    F3M_CUDA(cudaFuncSetAttribute(m2l_nested<PP, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_n));
                    m2l_nested<PP, 2><<<lx.nb, 128, smem_n, s>>>(lx.nb, ll.far.ptr.p, ll.far_okey.p, ll.far_oidx.p, lx.off.p, rb, re,
                                                                  T.p, momp[l], loc[l].p);
                }
            } else
                launch_m2l(lx.nb, ll.far.ptr.p, ll.far.idx.p, cellx.p, cy, lx.off.p, geo, momp[l], loc[l].p);
            F3M_LAUNCH_CHECK();
        }
    }
    pl->last.end(s);
    // ---- L2L downwards, L2P at the finest level -------------------------------------------------
    pl->last.begin(ST_L2P, s);
    {
        const int nw = warps_for(2 * MS * sizeof(float));
        size_t sm2 = (size_t)2 * MS * sizeof(float) + nw * per_warp;
        F3M_CUDA(cudaFuncSetAttribute(l2l_fast<PP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm2));
        for (int l = lmin; l < L; l++) {
            Level &lc = tx.levels[l + 1];
            l2l_fast<PP><<<(lc.nb + nw - 1) / nw, 32 * nw, sm2, s>>>(lc.nb, d, lc.parent.p, lc.code.p, lc.off.p, rb, re, AT.p, cfg,
                                                                    loc[l].p, loc[l + 1].p);
            F3M_LAUNCH_CHECK();
        }
        Level &lx = tx.levels[L];
        const float factor = 2.f / lx.edge;
        int nsplit = std::max(1, std::min(64, (lx.max_count + 8191) / 8192));
        size_t smem = ((size_t)PR + (size_t)std::max(1, d - 1) * PP * 128) * sizeof(float);
        F3M_CUDA(cudaFuncSetAttribute(l2p_leaf<PP, RB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (RB == 1 && d == 3) {
            if (pl->n_leaf_big[0])
                l2p_leaf3<PP><<<dim3(pl->n_leaf_big[0], nsplit), 128, 0, s>>>(tx.pts.p, n_x, lx.off.p, lx.ctr.p, factor, nt, nsplit, rb, re,
                                                                            loc[L].p, R, r0, out, pl->leaf_big[0].p);
            if (pl->n_leaf_small[0])
                l2p_small3<PP><<<(pl->n_leaf_small[0] + 3) / 4, 128, 0, s>>>(tx.pts.p, n_x, lx.off.p, lx.ctr.p, factor, nt, rb, re, loc[L].p,
                                                                           R, r0, out, pl->leaf_small[0].p, pl->n_leaf_small[0]);
        } else
        l2p_leaf<PP, RB><<<dim3(lx.nb, nsplit), 128, smem, s>>>(tx.pts.p, n_x, d, lx.off.p, lx.ctr.p, factor, nt, P, nsplit, rb, re,
                                                               loc[L].p, R, r0, out);
        F3M_LAUNCH_CHECK();
    }
    pl->last.end(s);
}

template <int PP>
static void far_fast_p(f3m_plan *pl, const float *bs, int R, float *out, int rb, int re, int lmin, cudaStream_t s) {
    int P = 1;
    for (int k = 0; k < pl->d; k++) P *= PP;
    // 8 columns at a time when the three per-warp buffers of the translation kernels fit, else one
    const bool wide = R > 1 && (size_t)3 * P * 8 * sizeof(float) + (size_t)pl->d * NOFF2 * mat_stride(PP) * sizeof(float) <= 200 * 1024;
    for (int r0 = 0; r0 < R;) {
        if (wide) { far_fast_block<PP, 8>(pl, bs, R, r0, out, rb, re, lmin, s); r0 += 8; }
        else { far_fast_block<PP, 1>(pl, bs, R, r0, out, rb, re, lmin, s); r0 += 1; }
    }
}

// Number of floats of the finest-level moment array when the far field of (plan, R) runs as one column block on
// the single-pass path, else 0 (then moments cannot be exchanged between ranks and every rank computes its own).
int64_t far_moments_size(const f3m_plan *pl, int R) {
    const int L = pl->levels;
    int lmin = 0, p = 0;
    bool uniform = true;
    for (int l = 1; l <= L; l++) {
        if (pl->lists[l].far.count == 0) continue;
        if (!lmin) { lmin = l; p = pl->lists[l].p; }
        else if (pl->lists[l].p != p) uniform = false;
    }
    if (!lmin || !uniform || p > PMAX_FAST || p < 2) return 0;
    int P = 1;
    for (int k = 0; k < pl->d; k++) P *= p;
    const size_t tab = (size_t)pl->d * NOFF2 * mat_stride(p) * sizeof(float);
    if ((size_t)3 * P * sizeof(float) + tab > 200 * 1024) return 0;
    int RB = 1;
    if (R > 1) {
        if (R > 8 || (size_t)3 * P * 8 * sizeof(float) + tab > 200 * 1024) return 0;
        RB = 8;
    }
    return (int64_t)pl->ty->levels[L].nb * P * RB;
}

// Far field of the whole product.  Fast path when every level with far pairs uses the same p <= 8;
// otherwise (var_compression switching node counts between levels, or more nodes per dimension) the
// per-level path of far.cu.
void far_field(f3m_plan *pl, const float *b_sorted, int R, float *out_sorted, int64_t row_begin, int64_t row_end,
               cudaStream_t s) {
    const int L = pl->levels;
    int lmin = 0, p = 0;
    bool uniform = true;
    for (int l = 1; l <= L; l++) {
        if (pl->lists[l].far.count == 0) continue;
        if (!lmin) { lmin = l; p = pl->lists[l].p; }
        else if (pl->lists[l].p != p) uniform = false;
    }
    if (!lmin) return;
    int P = 1;
    for (int k = 0; k < pl->d; k++) P *= p;
    const bool fits = (size_t)3 * P * sizeof(float) + (size_t)pl->d * NOFF2 * mat_stride(p) * sizeof(float) <= 200 * 1024;
    if (!uniform || p > PMAX_FAST || p < 2 || !fits) {
        for (int l = lmin; l <= L; l++) far_field_level(pl, l, b_sorted, R, out_sorted, row_begin, row_end, s);
        return;
    }
    const int rb = (int)row_begin, re = (int)row_end;
    switch (p) {
        case 2: far_fast_p<2>(pl, b_sorted, R, out_sorted, rb, re, lmin, s); break;
        case 3: far_fast_p<3>(pl, b_sorted, R, out_sorted, rb, re, lmin, s); break;
        case 4: far_fast_p<4>(pl, b_sorted, R, out_sorted, rb, re, lmin, s); break;
        case 5: far_fast_p<5>(pl, b_sorted, R, out_sorted, rb, re, lmin, s); break;
        case 6: far_fast_p<6>(pl, b_sorted, R, out_sorted, rb, re, lmin, s); break;
        case 7: far_fast_p<7>(pl, b_sorted, R, out_sorted, rb, re, lmin, s); break;
        default: far_fast_p<8>(pl, b_sorted, R, out_sorted, rb, re, lmin, s); break;
    }
}

}  // namespace f3m
