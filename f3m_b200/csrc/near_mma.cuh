// Near field on the 5th-generation tensor cores (tcgen05, sm_100a).  Included by near.cu.
//
// The pair term of the direct sum is 2^(-s^2 |x_i - y_j|^2) b_j (s^2 = log2(e)/(2 ls^2)).  About the centre c
// of the SOURCE box, with u = s (x - c) and v = s (y - c),
//     -s^2 |x - y|^2 = -|u|^2 + t_ij ,   t_ij = 2 u_i . v_j - |v_j|^2 ,
// so the sum over a source box is 2^(-|u_i|^2) * sum_j 2^(t_ij) b_j and t is an inner product of two short
// rows: a 128 x 128 x K matrix product per (target tile, source tile).  The tensor core takes TF32 operands
// (10-bit mantissa), so every number is split into a TF32 head and a TF32 tail (x = xh + xl up to 2^-22 |x|):
//     B row (source, packed once per product):  [ vh | vl | nvh nvl ]          nv = -|v|^2     (2 d + 2 slots)
//     A1 row (target, per source box):          [ 2uh | 2uh | 1   1   ]
//     A2 row                                    [ 2ul | 2ul | 0   0   ]
// and t = A1.B + A2.B, two accumulating MMAs on the same B tile.  Products of TF32 numbers are exact in the
// FP32 accumulator, so t has FP32 accuracy.  The B tiles are fetched with bulk copies (cp.async.bulk) that
// complete on an mbarrier; the exponent tile lands in tensor memory; eight warps read it back (tcgen05.ld),
// evaluate 2^t in packed pairs -- part of the column pairs on the MUFU pipe, part as a polynomial on the FMA
// pipe when t is provably small -- and accumulate e * b_j per target row.
//
// Two CTAs per SM (256 TMEM columns each = two 128 x 128 accumulator tiles), 8 consumer warps + 1 producer
// warp, coupled only through mbarriers: threads r and r + 128 own target row r and take alternate 32-column
// chunks of a tile.  The producer thread keeps the bulk copies MM_SLOTS-1 tiles ahead and issues the MMAs of
// tile k as soon as tile k-2 (same TMEM buffer) has been consumed; a consumer warp waits for tile k's
// accumulator, builds the target rows of a source box two tiles before its first tile, consumes its chunks
// and signals the tile's barrier.  Every wait is bounded: on expiry the CTA records an error
// code, stops taking work, frees its tensor memory and returns.
#pragma once

namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// whole warp; writes the TMEM base address to shared memory
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], TF32 inputs, FP32 accumulator; issued by ONE thread
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// the mbarrier receives one arrival when every MMA issued so far by this thread has completed
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 consecutive FP32 columns of the calling thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
// The registers of a tcgen05.ld hold their values only after this wait; passing them through the statement
// keeps the compiler from scheduling their uses above it.
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                   "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]),
                   "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]),
                   "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}

// Shared-memory operand descriptor, K-major, no swizzle: the operand is stored as 8-row x 16-byte core
// matrices; lbo = byte distance between core matrices that are neighbours along K, sbo = between
// neighbours along the row (M or N) direction.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3ffffu) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;   // descriptor version of this architecture
    return d;                 // base offset 0, no swizzle
}
// instruction descriptor: FP32 accumulator, TF32 x TF32, both operands K-major, M x N tile
__host__ __device__ constexpr uint32_t idesc_tf32(int M, int N) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// global -> shared bulk copy (16-byte aligned addresses, size a multiple of 16) that signals the mbarrier
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ float tf32_head(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }

}   // namespace tc

constexpr int MM_M = 128, MM_N = 128, MM_BUFS = 2, MM_AR = MM_BUFS, MM_CONSUMERS = 256, MM_THREADS = MM_CONSUMERS + 64, MM_ROWCHUNK = 256, MM_SLOTS = 8;
constexpr int MM_PRODUCER = MM_CONSUMERS;      // first lane of the first extra warp: issues the MMAs
constexpr int MM_COPIER = MM_CONSUMERS + 32;   // first lane of the second extra warp: starts the bulk copies

template <int D>
struct MmaShape {
    static constexpr int used = 2 * D + 2;
    static constexpr int K = (used + 7) / 8 * 8;
    static constexpr int KC = K / 4;   // 16-byte chunks per row
    static constexpr int KS = K / 8;   // MMA steps per operand pair
};

// dynamic shared memory of the kernel; at least 100 KB so that exactly two CTAs (2 x 256 TMEM columns) share an SM
template <int D>
constexpr int mm_smem_bytes() {
    constexpr int KC = MmaShape<D>::KC;
    constexpr int need = (MM_AR * 2 * KC * MM_M + MM_SLOTS * KC * MM_N) * 16 + MM_SLOTS * MM_N * 4 + 2 * MM_ROWCHUNK * 4 +
                         MM_ROWCHUNK * D * 4 + MM_M * 4 + 256;
    return need > 100 * 1024 ? need : 100 * 1024;
}

// Packed source rows: box b starts at row mm_row_start(off[b], b) and is padded to a multiple of 32 rows
// with rows of zero weight, so every tile is a whole number of 32-column chunks and 16-byte aligned.
__host__ __device__ __forceinline__ int mm_row_start(int off, int box) { return ((off + 31) & ~31) + 32 * box; }
static inline size_t mm_rows_total(int64_t n, int nb) { return (size_t)((n + 31) & ~(int64_t)31) + 32 * ((size_t)nb + 1); }

template <int D>
__global__ void __launch_bounds__(256) pack_split_rows(const float *__restrict__ pts, int n, const float *__restrict__ bs, int R,
                                                      int r0, float scale, const int *__restrict__ off_y, int nby,
                                                      const float *__restrict__ ctr_y, float4 *Bc, size_t rows, float *Gb) {
    using S = MmaShape<D>;
    int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    const int by = box_of_row(off_y, nby, j);
    const int s0 = off_y[by], s1 = off_y[by + 1];
    float vh[D], vl[D], nv = 0.f;
#pragma unroll
    for (int k = 0; k < D; k++) {
        const float v = scale * (pts[(size_t)k * n + j] - ctr_y[by * D + k]);
        nv = fmaf(-v, v, nv);
        vh[k] = tc::tf32_head(v);
        vl[k] = tc::tf32_head(v - vh[k]);
    }
    const float nvh = tc::tf32_head(nv), nvl = tc::tf32_head(nv - nvh);
    float o[S::K];
    int q = 0;
#pragma unroll
    for (int k = 0; k < D; k++) o[q++] = vh[k];
#pragma unroll
    for (int k = 0; k < D; k++) o[q++] = vl[k];
    o[q++] = nvh; o[q++] = nvl;
#pragma unroll
    for (; q < S::K; q++) o[q] = 0.f;
    const int rs = mm_row_start(s0, by);
    const int pos = rs + (j - s0);
#pragma unroll
    for (int kc = 0; kc < S::KC; kc++) Bc[(size_t)kc * rows + pos] = make_float4(o[4 * kc], o[4 * kc + 1], o[4 * kc + 2], o[4 * kc + 3]);
    Gb[pos] = bs[(size_t)j * R + r0];
    if (j == s1 - 1) {   // padding rows of this box
        const int end = rs + ((s1 - s0 + 31) & ~31);
        for (int pp = pos + 1; pp < end; pp++) {
#pragma unroll
            for (int kc = 0; kc < S::KC; kc++) Bc[(size_t)kc * rows + pp] = make_float4(0.f, 0.f, 0.f, 0.f);
            Gb[pp] = 0.f;
        }
    }
}

// 32 exponent columns of one target row, two columns per instruction; NPOLY8 of every 8 column pairs use the
// polynomial c0 + c1 t + c2 t^2 (+ c3 t^3) instead of the MUFU pipe
template <int DEG, int NPOLY8>
__device__ __forceinline__ void mm_consume32(const uint32_t (&r)[32], const float *bs, f32x2 (&acc)[2], f32x2 c0, f32x2 c1,
                                             f32x2 c2, f32x2 c3) {
#pragma unroll
    for (int q = 0; q < 8; q++) {
        const ulonglong2 bb = *reinterpret_cast<const ulonglong2 *>(bs + 4 * q);
#pragma unroll
        for (int jj = 0; jj < 2; jj++) {
            const int pr = (2 * q + jj) % 8;
            const bool poly = DEG > 0 && ((pr + 1) * NPOLY8 / 8 != (pr * NPOLY8) / 8);
            const float ta = __uint_as_float(r[4 * q + 2 * jj]), tb = __uint_as_float(r[4 * q + 2 * jj + 1]);
            f32x2 e;
            if (poly) {
                const f32x2 t = pack2(ta, tb);
                e = (DEG == 2) ? fma2(fma2(c2, t, c1), t, c0) : fma2(fma2(fma2(c3, t, c2), t, c1), t, c0);
            } else {
                e = pack2(ex2_approx(ta), ex2_approx(tb));
            }
            acc[jj] = fma2(e, jj ? bb.y : bb.x, acc[jj]);
        }
    }
}


struct MmCursor {
    int e, base;   // near box within the row chunk, first source row of the tile within that box
    int par;       // which of the two A buffers holds the target rows about that box's centre
};

template <int D, int DEG, int NPOLY8>
__global__ void __launch_bounds__(MM_THREADS, 2)
near_mma_kernel(const float *__restrict__ xpts, int n_x, const int *__restrict__ off_x, int nbx, const int *__restrict__ tile_off,
                int n_items, const int *__restrict__ ptr, const int *__restrict__ idx, const int *__restrict__ off_y,
                const float *__restrict__ ctr_y, const float4 *__restrict__ Bc, size_t rows, const float *__restrict__ Gb,
                float scale, int R, int r0, float *out, int *counter, int *err, float pc0, float pc1, float pc2, float pc3,
                int row_begin, int row_end) {
    using S = MmaShape<D>;
    constexpr int KC = S::KC;
    constexpr int A_ONE = 2 * KC * MM_M;   // float4 per A buffer (A1 and A2)
    constexpr int B_ONE = KC * MM_N;       // float4 per B slot
    extern __shared__ __align__(128) unsigned char smraw[];
    float4 *Asm = reinterpret_cast<float4 *>(smraw);                   // [MM_AR][2][KC][128]
    float4 *Bsm = Asm + MM_AR * A_ONE;                                     // [MM_SLOTS][KC][128]
    float *bsm = reinterpret_cast<float *>(Bsm + MM_SLOTS * B_ONE);    // [MM_SLOTS][128]
    int *rowst = reinterpret_cast<int *>(bsm + MM_SLOTS * MM_N);       // [MM_ROWCHUNK] first packed row of the box
    int *cntp = rowst + MM_ROWCHUNK;                                   // [MM_ROWCHUNK] padded source count
    float *cen = reinterpret_cast<float *>(cntp + MM_ROWCHUNK);        // [MM_ROWCHUNK][D] source box centres
    float *comb = cen + MM_ROWCHUNK * D;                               // [128]
    // copies landed (per slot, tx count) | accumulator ready (per TMEM buffer) | accumulator read back (per TMEM
    // buffer, 8 warps) | slot's b values no longer needed (per slot, 8 warps)
    __shared__ __align__(8) uint64_t mbar[2 * MM_SLOTS + 2 * MM_BUFS];
    __shared__ uint32_t tmem_base_s;
    __shared__ int item_s;
    __shared__ volatile int abort_s;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, row = tid & (MM_M - 1), half = tid >> 7;   // half 2: producer warp
    const bool consumer = tid < MM_CONSUMERS;
    if (warp == 0) tc::tmem_alloc(tc::smem_u32(&tmem_base_s), MM_BUFS * MM_N);
    if (tid == 0) {
        for (int i = 0; i < MM_SLOTS + MM_BUFS; i++) tc::mbar_init(tc::smem_u32(&mbar[i]), 1);
        for (int i = 0; i < MM_SLOTS + MM_BUFS; i++) tc::mbar_init(tc::smem_u32(&mbar[MM_SLOTS + MM_BUFS + i]), MM_CONSUMERS / 32);
        tc::fence_mbar_init();
        abort_s = 0;
    }
    // stale rows of a slot take part in the MMA (their columns are never read): keep them finite
    for (int q = tid; q < MM_SLOTS * B_ONE; q += MM_THREADS) Bsm[q] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int q = tid; q < MM_SLOTS * MM_N; q += MM_THREADS) bsm[q] = 0.f;
    tc::fence_async_smem();
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = tmem_base_s;
    const uint32_t bar_copy = tc::smem_u32(&mbar[0]), bar_acc = tc::smem_u32(&mbar[MM_SLOTS]),
                   bar_read = tc::smem_u32(&mbar[MM_SLOTS + MM_BUFS]), bar_late = tc::smem_u32(&mbar[MM_SLOTS + 2 * MM_BUFS]);
    constexpr uint32_t IDESC = tc::idesc_tf32(MM_M, MM_N);
    const uint32_t a_addr = tc::smem_u32(Asm), b_addr = tc::smem_u32(Bsm), bs_addr = tc::smem_u32(bsm);
    const f32x2 c0 = pack2(pc0, pc0), c1 = pack2(pc1, pc1), c2 = pack2(pc2, pc2), c3 = pack2(pc3, pc3);

    // Tiles are numbered over the life of the CTA: tile k uses copy slot k % MM_SLOTS (its k / MM_SLOTS-th use) and
    // TMEM buffer k % MM_BUFS (its k / MM_BUFS-th use), which gives the parity every wait needs.
    unsigned gk = 0;
    int bad = 0;          // set by a thread whose wait expired; the barriers between row chunks OR it over the CTA
    bool aborted = false;
    auto bounded_wait = [&](uint32_t bar, uint32_t par) {
        int tries = 0;
        while (!tc::mbar_try_wait(bar, par)) {
            __nanosleep(20);
            if (++tries > 400000 || ((tries & 1023) == 0 && abort_s)) { atomicExch(err, 8); bad = 1; abort_s = 1; break; }
        }
    };

    for (;;) {
        if (tid == MM_PRODUCER) item_s = atomicAdd(counter, 1);
        aborted = aborted || __syncthreads_or(bad);
        const int item = item_s;
        if (item >= n_items || aborted) break;
        // item -> (target box, 128 consecutive targets of it)
        int box;
        {
            int lo = 0, hi = nbx;
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (tile_off[mid] <= item) lo = mid; else hi = mid;
            }
            box = lo;
        }
        // only the rows inside [row_begin, row_end): the others belong to another slice of the targets
        const int t0 = max(off_x[box], row_begin) + MM_M * (item - tile_off[box]);
        const int nrows = min(MM_M, min(off_x[box + 1], row_end) - t0);
        const bool row_ok = consumer && row < nrows;
        const bool warp_rows = 32 * (warp & 3) < nrows;   // does this warp hold any target
        float x[D];
#pragma unroll
        for (int k = 0; k < D; k++) x[k] = row_ok ? xpts[(size_t)k * n_x + t0 + row] : 0.f;
        float tot = 0.f;
        const int e0 = ptr[box], e1 = ptr[box + 1];
        for (int ec = e0; ec < e1 && !aborted; ec += MM_ROWCHUNK) {
            const int nbc = min(MM_ROWCHUNK, e1 - ec);
            if (tid < nbc) {
                const int by = idx[ec + tid];
                const int so = off_y[by];
                rowst[tid] = mm_row_start(so, by);
                cntp[tid] = (off_y[by + 1] - so + 31) & ~31;
#pragma unroll
                for (int k = 0; k < D; k++) cen[tid * D + k] = ctr_y[by * D + k];
            }
            __syncthreads();
            auto valid = [&](const MmCursor &c) { return c.e < nbc; };
            auto skip_empty = [&](MmCursor &c) {
                while (c.e < nbc && cntp[c.e] == 0) c.e++;
            };
            auto advance = [&](MmCursor c) {
                c.base += MM_N;
                if (c.base >= cntp[c.e]) { c.e++; c.base = 0; c.par = (c.par + 1) % MM_AR; skip_empty(c); }
                return c;
            };
            // A1 / A2 rows of this thread's target about the centre of near box e (threads 0..127)
            auto build_a = [&](int e, int par) {
                float Uh[D], Ul[D];
#pragma unroll
                for (int k = 0; k < D; k++) {
                    const float u2 = row_ok ? 2.f * scale * (x[k] - cen[e * D + k]) : 0.f;
                    Uh[k] = tc::tf32_head(u2);
                    Ul[k] = tc::tf32_head(u2 - Uh[k]);
                }
                float o1[S::K], o2[S::K];
                int q = 0;
#pragma unroll
                for (int k = 0; k < D; k++) { o1[q] = Uh[k]; o2[q] = Ul[k]; q++; }
#pragma unroll
                for (int k = 0; k < D; k++) { o1[q] = Uh[k]; o2[q] = Ul[k]; q++; }
                o1[q] = 1.f; o2[q] = 0.f; q++;
                o1[q] = 1.f; o2[q] = 0.f; q++;
#pragma unroll
                for (; q < S::K; q++) { o1[q] = 0.f; o2[q] = 0.f; }
                float4 *dst = Asm + par * A_ONE;
#pragma unroll
                for (int kc = 0; kc < KC; kc++) {
                    dst[kc * MM_M + row] = make_float4(o1[4 * kc], o1[4 * kc + 1], o1[4 * kc + 2], o1[4 * kc + 3]);
                    dst[(KC + kc) * MM_M + row] = make_float4(o2[4 * kc], o2[4 * kc + 1], o2[4 * kc + 2], o2[4 * kc + 3]);
                }
            };
            MmCursor first{0, 0, 0};
            skip_empty(first);
            if (valid(first)) {
                // target rows of the boxes that start within the first MM_BUFS tiles; later boxes are built MM_BUFS
                // tiles ahead by the consumers (the ring of MM_AR A buffers covers one box per tile in flight)
                MmCursor look0 = first;
                for (int a = 0; a < MM_BUFS && valid(look0); a++) {
                    if (tid < MM_M && look0.base == 0) build_a(look0.e, look0.par);
                    look0 = advance(look0);
                }
                tc::fence_async_smem();
                __syncthreads();
                if (tid == MM_COPIER) {
                    // ---- copy thread: runs as far ahead as the MM_SLOTS slots allow; a slot is free once the tile that
                    // used it before has been consumed ----
                    MmCursor cp = first;
                    for (unsigned kp = gk; valid(cp) && !abort_s; kp++, cp = advance(cp)) {
                        if (kp >= MM_SLOTS) bounded_wait(bar_late + 8u * (kp % MM_SLOTS), ((kp - MM_SLOTS) / MM_SLOTS) & 1u);
                        const unsigned slot = kp % MM_SLOTS;
                        const uint32_t ncols = (uint32_t)min(MM_N, cntp[cp.e] - cp.base);
                        const size_t g = (size_t)rowst[cp.e] + cp.base;
                        const uint32_t bar = bar_copy + 8u * slot;
                        tc::mbar_expect_tx(bar, ncols * (16u * KC + 4u));
#pragma unroll
                        for (int kc = 0; kc < KC; kc++)
                            tc::bulk_g2s(b_addr + (slot * B_ONE + kc * MM_N) * 16u, Bc + (size_t)kc * rows + g, ncols * 16u, bar);
                        tc::bulk_g2s(bs_addr + slot * MM_N * 4u, Gb + g, ncols * 4u, bar);
                    }
                } else if (tid == MM_PRODUCER) {
                    // ---- MMA thread: tile km as soon as its copies have landed and TMEM buffer km % MM_BUFS has been read ----
                    // descriptors of the A buffers (ring position x {A1, A2} x K step) and of slot 0 of B
                    uint64_t adesc[MM_AR][2][S::KS], bdesc0[S::KS];
#pragma unroll
                    for (int r = 0; r < MM_AR; r++)
#pragma unroll
                        for (int m = 0; m < 2; m++)
#pragma unroll
                            for (int ks = 0; ks < S::KS; ks++)
                                adesc[r][m][ks] = tc::smem_desc(a_addr + (uint32_t)r * A_ONE * 16u + (m * KC + 2 * ks) * (MM_M * 16), MM_M * 16, 128);
#pragma unroll
                    for (int ks = 0; ks < S::KS; ks++) bdesc0[ks] = tc::smem_desc(b_addr + 2 * ks * (MM_N * 16), MM_N * 16, 128);
                    MmCursor cm = first;
                    for (unsigned km = gk; valid(cm) && !abort_s; km++, cm = advance(cm)) {
                        bounded_wait(bar_copy + 8u * (km % MM_SLOTS), (km / MM_SLOTS) & 1u);
                        if (km >= MM_BUFS) bounded_wait(bar_read + 8u * (km % MM_BUFS), ((km - MM_BUFS) / MM_BUFS) & 1u);   // buffer read back, A rows built
                        tc::fence_after_sync();
                        const uint32_t d_tmem = tmem + (km % MM_BUFS) * MM_N;
                        const uint64_t bslot = (uint64_t)(((km % MM_SLOTS) * B_ONE * 16u) >> 4);   // start-address field counts 16-byte units
#pragma unroll
                        for (int m = 0; m < 2; m++)
#pragma unroll
                            for (int ks = 0; ks < S::KS; ks++) {
                                uint64_t ad = adesc[0][m][ks];
#pragma unroll
                                for (int r = 1; r < MM_AR; r++)
                                    if (cm.par == r) ad = adesc[r][m][ks];
                                tc::mma_tf32(d_tmem, ad, bdesc0[ks] + bslot, IDESC, (m | ks) ? 1u : 0u);
                            }
                        tc::mma_commit(bar_acc + 8u * (km % MM_BUFS));
                    }
                } else if (consumer) {
                    // ---- consumers ----
                    MmCursor cur = first, look = look0;   // look: tile k + MM_BUFS
                    unsigned k = gk;
                    float fx = 0.f;
                    f32x2 acc[2] = {pack2(0.f, 0.f), pack2(0.f, 0.f)};
                    auto close_box = [&]() {
                        float a, b, c, d;
                        unpack2(acc[0], a, b);
                        unpack2(acc[1], c, d);
                        tot = fmaf(fx, (a + b) + (c + d), tot);
                        acc[0] = acc[1] = pack2(0.f, 0.f);
                    };
                    while (valid(cur) && !abort_s) {
                        if (cur.base == 0) {   // first tile of a source box: close the previous box, new row factor
                            close_box();
                            float nu = 0.f;
#pragma unroll
                            for (int q = 0; q < D; q++) {
                                const float u = scale * (x[q] - cen[cur.e * D + q]);
                                nu = fmaf(-u, u, nu);
                            }
                            fx = ex2_approx(nu);
                        }
                        bounded_wait(bar_copy + 8u * (k % MM_SLOTS), (k / MM_SLOTS) & 1u);   // the tile's b values landed
                        bounded_wait(bar_acc + 8u * (k % MM_BUFS), (k / MM_BUFS) & 1u);      // its exponents are in TMEM
                        tc::fence_after_sync();
                        // every MMA up to tile k is done: the ring buffer of the box that starts at tile k + MM_BUFS is free
                        if (tid < MM_M && valid(look) && look.base == 0) {
                            build_a(look.e, look.par);
                            tc::fence_async_smem();
                        }
                        const int ncols = min(MM_N, cntp[cur.e] - cur.base);
                        // this warp's chunks of the tile: half, half + 2, ...; the TMEM buffer is released after the last read
                        const uint32_t taddr = tmem + ((uint32_t)(32 * (warp & 3)) << 16) + (k % MM_BUFS) * MM_N;
                        const float *bs = bsm + (k % MM_SLOTS) * MM_N;
                        uint32_t ra[32];
                        int ch = half;
                        if (warp_rows)
                            for (; 32 * (ch + 2) < ncols; ch += 2) {
                                tc::tmem_ld32(taddr + 32 * ch, ra);
                                tc::tmem_ld_wait(ra);
                                mm_consume32<DEG, NPOLY8>(ra, bs + 32 * ch, acc, c0, c1, c2, c3);
                            }
                        const bool work = warp_rows && 32 * ch < ncols;
                        if (work) {
                            tc::tmem_ld32(taddr + 32 * ch, ra);
                            tc::tmem_ld_wait(ra);
                        }
                        tc::fence_before_sync();
                        __syncwarp();
                        if (lane == 0) tc::mbar_arrive(bar_read + 8u * (k % MM_BUFS));   // the TMEM buffer may be overwritten
                        if (work) mm_consume32<DEG, NPOLY8>(ra, bs + 32 * ch, acc, c0, c1, c2, c3);
                        __syncwarp();
                        if (lane == 0) tc::mbar_arrive(bar_late + 8u * (k % MM_SLOTS));        // the slot's b values are no longer needed
                        k++;
                        cur = advance(cur);
                        if (valid(look)) look = advance(look);
                    }
                    close_box();
                }
                // every thread counts the tiles of the chunk the same way
                for (MmCursor c = first; valid(c); c = advance(c)) gk++;
            }
            tc::fence_before_sync();
            aborted = __syncthreads_or(bad) || aborted;   // the row chunk's tables and buffers are reused
        }
        if (half == 1) comb[row] = tot;
        __syncthreads();
        if (half == 0 && row_ok) out[(size_t)(t0 + row) * R + r0] += tot + comb[row];
    }
    if (aborted)   // give an operation that may still be in flight time to drain before the tensor memory goes back
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem, MM_BUFS * MM_N);
}
