// Near field on the 5th-generation tensor cores (tcgen05, sm_100a).  Included by near.cu.
//
// The pair term of the direct sum is 2^(t_ij) b_j with t_ij = -s^2 |x_i - y_j|^2 (s^2 = log2(e)/(2 ls^2)).
// With u = s (x - c), v = s (y - c) about the centre c of the TARGET box,
//     t_ij = -|u_i|^2 + 2 u_i . v_j - |v_j|^2
// is an inner product of two short rows, i.e. a 128 x 256 x K matrix product per (target tile, source tile).
// The tensor core takes TF32 operands (10-bit mantissa), so every number is split into a TF32 head and a
// TF32 tail (x = xh + xl exactly up to 2^-22 |x|) and the four cross products are spread over the K slots:
//     A row (target):  [ 2uh | 2ul | 2uh | 2ul | 1   1   nuh nul ]      nu = -|u|^2
//     B row (source):  [  vh |  vh |  vl |  vl | nvh nvl 1   1   ]      nv = -|v|^2
// 4 d + 4 slots, rounded up to a multiple of 8 (one tcgen05.mma step has K = 8 for TF32).  Products of two
// TF32 numbers are exact in the FP32 accumulator, so the exponent comes out with FP32 accuracy.
// The exponent tile lands in tensor memory; eight warps read it back (tcgen05.ld), evaluate 2^t -- part of
// the columns on the MUFU pipe, part as a polynomial on the FMA pipe when |t| is provably small -- and
// accumulate e * b_j per target row.  Per pair that is ~2-4 issue slots instead of 5-7 on the CUDA cores.
//
// One persistent CTA per SM (512 TMEM columns = two 128 x 256 accumulator tiles), 256 threads:
// thread r and thread r+128 own target row r and split the 256 columns of a tile between them.
// Pipeline per source tile k: pack tile k+1 into shared memory (all threads) -> barrier -> one thread issues
// the MMAs of tile k+1 into the other TMEM buffer -> everyone waits for tile k's mbarrier and consumes it.
// Every wait is bounded: on expiry the CTA records an error code, stops taking work, frees its tensor
// memory and returns.
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

__device__ __forceinline__ float tf32_head(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }

}   // namespace tc

constexpr int MM_M = 128, MM_N = 256, MM_THREADS = 256, MM_ROWCHUNK = 256;
constexpr int MM_SMEM_BYTES = 120 * 1024;   // more than half of an SM's shared memory: one CTA per SM

template <int D>
struct MmaShape {
    static constexpr int used = 4 * D + 4;
    static constexpr int K = (used + 7) / 8 * 8;
    static constexpr int KC = K / 4;   // 16-byte chunks per row
};

// 2^t for small |t|, Taylor polynomial in t ln2 of degree DEG (3 or 4)
template <int DEG>
__device__ __forceinline__ float exp2_poly_mm(float t) {
    constexpr float C1 = 0.69314718056f, C2 = 0.24022650696f, C3 = 0.05550410866f, C4 = 0.00961812911f;
    if (DEG == 2) return fmaf(fmaf(C2, t, C1), t, 1.f);
    if (DEG == 3) return fmaf(fmaf(fmaf(C3, t, C2), t, C1), t, 1.f);
    return fmaf(fmaf(fmaf(fmaf(C4, t, C3), t, C2), t, C1), t, 1.f);
}

// 32 exponent columns of one target row -> acc[0..3]
template <int DEG, int NPOLY8>
__device__ __forceinline__ void mm_consume32(const uint32_t (&r)[32], const float *bs, float (&acc)[4]) {
#pragma unroll
    for (int q = 0; q < 8; q++) {
        const float4 bb = *reinterpret_cast<const float4 *>(bs + 4 * q);
        const float bv[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int col = 4 * q + j;
            // NPOLY8 of every 8 columns go to the FMA pipe, spread evenly
            const bool poly = DEG > 0 && (((col % 8) + 1) * NPOLY8 / 8 != ((col % 8) * NPOLY8) / 8);
            const float t = __uint_as_float(r[col]);
            const float e = poly ? exp2_poly_mm<DEG ? DEG : 3>(t) : ex2_approx(t);
            acc[j] = fmaf(e, bv[j], acc[j]);
        }
    }
}

template <int D, int DEG, int NPOLY8>
__global__ void __launch_bounds__(MM_THREADS, 1)
near_mma_kernel(const float *__restrict__ xpts, int n_x, const int *__restrict__ off_x, const float *__restrict__ ctr_x, int nbx,
                const int *__restrict__ tile_off, int n_items, const int *__restrict__ ptr, const int *__restrict__ idx,
                const int *__restrict__ off_y, const float *__restrict__ packed, float scale, int R, int r0, float *out,
                int *counter, int *err) {
    using S = MmaShape<D>;
    constexpr int KC = S::KC;
    constexpr int W = row_width(D, 1);
    extern __shared__ __align__(128) unsigned char smraw[];
    float4 *Asm = reinterpret_cast<float4 *>(smraw);              // [KC][128]
    float4 *Bsm = Asm + KC * MM_M;                                // [2][KC][256]
    float *bsm = reinterpret_cast<float *>(Bsm + 2 * KC * MM_N);  // [3][256]
    int *pref = reinterpret_cast<int *>(bsm + 3 * MM_N);          // [MM_ROWCHUNK + 1] (+ padding)
    int *srcoff = pref + MM_ROWCHUNK + 4;                         // [MM_ROWCHUNK]
    float *comb = reinterpret_cast<float *>(srcoff + MM_ROWCHUNK);   // [128]
    int *wsum = reinterpret_cast<int *>(comb + MM_M);             // [8]
    __shared__ __align__(8) uint64_t mbar[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int item_s;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (warp == 0) tc::tmem_alloc(tc::smem_u32(&tmem_base_s), 512);
    if (tid == 0) {
        tc::mbar_init(tc::smem_u32(&mbar[0]), 1);
        tc::mbar_init(tc::smem_u32(&mbar[1]), 1);
        tc::fence_mbar_init();
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = tmem_base_s;
    const uint32_t bar0 = tc::smem_u32(&mbar[0]);   // barrier of TMEM buffer b at bar0 + 8 b
    uint32_t parity = 0u;                          // bit b: phase to wait for next on buffer b
    constexpr uint32_t IDESC = tc::idesc_tf32(MM_M, MM_N);
    const uint32_t a_addr = tc::smem_u32(Asm), b_addr = tc::smem_u32(Bsm);

    // B row of one source (or of a padding column) -> shared memory
    auto pack_b = [&](const float (&row)[W], bool valid, const float (&c)[D], int buf, int slot3) {
        float vh[D], vl[D], nv = 0.f;
#pragma unroll
        for (int k = 0; k < D; k++) {
            const float v = valid ? scale * (row[k] - c[k]) : 0.f;
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
        for (int k = 0; k < D; k++) o[q++] = vh[k];
#pragma unroll
        for (int k = 0; k < D; k++) o[q++] = vl[k];
#pragma unroll
        for (int k = 0; k < D; k++) o[q++] = vl[k];
        o[q++] = nvh; o[q++] = nvl; o[q++] = 1.f; o[q++] = 1.f;
#pragma unroll
        for (; q < S::K; q++) o[q] = 0.f;
        float4 *dst = Bsm + (size_t)buf * KC * MM_N;
#pragma unroll
        for (int kc = 0; kc < KC; kc++) dst[kc * MM_N + tid] = make_float4(o[4 * kc], o[4 * kc + 1], o[4 * kc + 2], o[4 * kc + 3]);
        bsm[slot3 * MM_N + tid] = valid ? row[D] : 0.f;
    };
    // the MMAs of one source tile: K/8 steps, the first overwrites the accumulator
    auto issue_mma = [&](int buf) {
        tc::fence_after_sync();
        const uint32_t d_tmem = tmem + (uint32_t)buf * MM_N;
#pragma unroll
        for (int ks = 0; ks < S::K / 8; ks++) {
            const uint64_t ad = tc::smem_desc(a_addr + ks * 2 * (MM_M * 16), MM_M * 16, 128);
            const uint64_t bd = tc::smem_desc(b_addr + buf * (KC * MM_N * 16) + ks * 2 * (MM_N * 16), MM_N * 16, 128);
            tc::mma_tf32(d_tmem, ad, bd, IDESC, ks > 0 ? 1u : 0u);
        }
        tc::mma_commit(bar0 + 8u * (uint32_t)buf);
    };

    // `bad` is set by a thread whose wait expired; every barrier below ORs it over the CTA, so all threads
    // leave the loops at the same point
    int bad = 0;
    bool aborted = false;
    for (;;) {
        if (tid == 0) item_s = atomicAdd(counter, 1);
        aborted = aborted || __syncthreads_or(bad);
        const int item = item_s;
        if (item >= n_items || aborted) break;
        int box, t0, t1;
        item_to_tile(item, tile_off, nbx, off_x, box, t0, t1);
        float c[D];
#pragma unroll
        for (int k = 0; k < D; k++) c[k] = __ldg(ctr_x + box * D + k);
        if (tid < MM_M) {   // A row of target t0 + tid
            const int ti = t0 + tid;
            float Uh[D], Ul[D], nu = 0.f;
#pragma unroll
            for (int k = 0; k < D; k++) {
                const float u = ti < t1 ? scale * (xpts[(size_t)k * n_x + ti] - c[k]) : 0.f;
                nu = fmaf(-u, u, nu);
                Uh[k] = tc::tf32_head(2.f * u);
                Ul[k] = tc::tf32_head(2.f * u - Uh[k]);
            }
            const float nuh = tc::tf32_head(nu), nul = tc::tf32_head(nu - nuh);
            float o[S::K];
            int q = 0;
#pragma unroll
            for (int k = 0; k < D; k++) o[q++] = Uh[k];
#pragma unroll
            for (int k = 0; k < D; k++) o[q++] = Ul[k];
#pragma unroll
            for (int k = 0; k < D; k++) o[q++] = Uh[k];
#pragma unroll
            for (int k = 0; k < D; k++) o[q++] = Ul[k];
            o[q++] = 1.f; o[q++] = 1.f; o[q++] = nuh; o[q++] = nul;
#pragma unroll
            for (; q < S::K; q++) o[q] = 0.f;
#pragma unroll
            for (int kc = 0; kc < KC; kc++) Asm[kc * MM_M + tid] = make_float4(o[4 * kc], o[4 * kc + 1], o[4 * kc + 2], o[4 * kc + 3]);
        }
        float tot = 0.f;
        const int e0 = ptr[box], e1 = ptr[box + 1];
        for (int ec = e0; ec < e1 && !aborted; ec += MM_ROWCHUNK) {
            const int nbc = min(MM_ROWCHUNK, e1 - ec);
            // sources of this chunk of the row, as one concatenated list: pref[e] = first position of box e
            int cnt = 0, so = 0;
            if (tid < nbc) {
                const int by = idx[ec + tid];
                so = off_y[by];
                cnt = off_y[by + 1] - so;
            }
            int incl = cnt;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            if (lane == 31) wsum[warp] = incl;
            __syncthreads();
            int before = 0;
#pragma unroll
            for (int w = 0; w < MM_THREADS / 32; w++) before += (w < warp) ? wsum[w] : 0;
            pref[tid + 1] = before + incl;
            if (tid == 0) pref[0] = 0;
            srcoff[tid] = so;
            __syncthreads();
            const int total = pref[nbc];
            const int T = (total + MM_N - 1) / MM_N;
            if (T > 0) {
                int eb = 0;   // near box that holds this thread's current position (positions only grow)
                auto fetch = [&](int k, float (&row)[W], bool &valid) {
                    const int p = k * MM_N + tid;
                    valid = p < total;
                    if (valid) {
                        while (p >= pref[eb + 1]) eb++;
                        const float4 *src = reinterpret_cast<const float4 *>(packed + (size_t)(srcoff[eb] + p - pref[eb]) * W);
#pragma unroll
                        for (int q = 0; q < W / 4; q++) {
                            const float4 v = __ldg(src + q);
                            row[4 * q] = v.x; row[4 * q + 1] = v.y; row[4 * q + 2] = v.z; row[4 * q + 3] = v.w;
                        }
                    }
                };
                float nxt[W];
                bool nvalid;
                fetch(0, nxt, nvalid);
                pack_b(nxt, nvalid, c, 0, 0);
                if (T > 1) fetch(1, nxt, nvalid);
                tc::fence_async_smem();
                __syncthreads();
                if (tid == 0) issue_mma(0);
                for (int k = 0; k < T; k++) {
                    if (k + 1 < T) {
                        pack_b(nxt, nvalid, c, (k + 1) & 1, (k + 1) % 3);
                        if (k + 2 < T) fetch(k + 2, nxt, nvalid);
                    }
                    tc::fence_async_smem();
                    tc::fence_before_sync();
                    if (__syncthreads_or(bad)) { aborted = true; break; }
                    if (tid == 0 && k + 1 < T) issue_mma((k + 1) & 1);
                    const int buf = k & 1;
                    {   // bounded wait for the accumulator of tile k
                        int tries = 0;
                        while (!tc::mbar_try_wait(bar0 + 8u * (uint32_t)buf, (parity >> buf) & 1u)) {
                            if (++tries > 400000) { atomicExch(err, 8); bad = 1; break; }
                        }
                        parity ^= 1u << buf;
                    }
                    tc::fence_after_sync();
                    const uint32_t taddr = tmem + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)(buf * MM_N + (warp >> 2) * 128);
                    const float *bs = bsm + (k % 3) * MM_N + (warp >> 2) * 128;
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
                    uint32_t ra[32], rb[32];
                    tc::tmem_ld32(taddr, ra);
                    tc::tmem_ld_wait(ra);
                    tc::tmem_ld32(taddr + 32, rb);
                    mm_consume32<DEG, NPOLY8>(ra, bs, acc);
                    tc::tmem_ld_wait(rb);
                    tc::tmem_ld32(taddr + 64, ra);
                    mm_consume32<DEG, NPOLY8>(rb, bs + 32, acc);
                    tc::tmem_ld_wait(ra);
                    tc::tmem_ld32(taddr + 96, rb);
                    mm_consume32<DEG, NPOLY8>(ra, bs + 64, acc);
                    tc::tmem_ld_wait(rb);
                    mm_consume32<DEG, NPOLY8>(rb, bs + 96, acc);
                    tot += (acc[0] + acc[1]) + (acc[2] + acc[3]);
                }
            }
            tc::fence_before_sync();
            aborted = __syncthreads_or(bad) || aborted;   // the row chunk's tables and buffers are reused
        }
        if (warp >= 4) comb[tid - MM_M] = tot;
        __syncthreads();
        if (tid < MM_M && t0 + tid < t1) out[(size_t)(t0 + tid) * R + r0] += tot + comb[tid];
    }
    if (aborted)   // give an operation that may still be in flight time to drain before the tensor memory goes back
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem, 512);
}
