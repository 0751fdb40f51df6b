// y[M,N] = act(x)[M,K] . W[N,K]^T for a handful of rows (M <= 64): the matrix products of a
// decode step, which are bound by streaming W from HBM once.
//
// The weight rows sit on the M axis of mma.sync m16n8k16 and the batch on its N axis.
// A CTA of 8 warps owns 16 rows of W (one m16 tile); each warp takes an equal share of K and
// the partial tiles are added in shared memory in warp order, so the result does not depend
// on timing. What bounds the kernel is how many bytes of W are on their way from HBM at any
// moment, so a thread keeps two small sets of weight registers and loads one while it
// multiplies the other; the sets are small enough (80 registers a thread) for three CTAs on
// an SM. MEASURED on B200, Qwen3-8B layer shapes at 8 rows, the four products of a layer:
// one set of 8 loads, 92 us; two sets of 8 (110 registers, two CTAs), 100 us; two sets of 4,
// 83 us (and 82 with sets of 8 for the matrices of 4096 rows only: see gs_launch); 16 warps a CTA for the narrow matrices, 89 us; W through TMA boxes of 16 rows x 128
// bytes into per-warp rings, 92-121 us (the vocabulary product fell from 5.8 to 3.2 TB/s). Both operands go from global memory straight into fragments with
// 16-byte loads: the sum over k may run in any order as long as W and x agree on it, so a
// thread's eight consecutive k values serve as the (2t, 2t+1) and (2t+8, 2t+9) pairs of two
// k-steps. W is read with a no-allocate hint (each byte is used once); x stays cached.
//
// Input: x bfloat16 [M,K]. (In this form, taking the float32 residual stream and a gain
// instead, RMSNorm folded into the product, was measured slower at every batch size: each of
// up to 1536 CTAs re-reads the stream and the gain. The persistent form further down, with one
// CTA an SM, does fold it.)
//
// Two forms. This one, a CTA a 16-row tile of W, takes up to 64 rows of x and any sizes. The
// persistent one (gemm_stream_kernel) takes at most 8 rows and the sizes gp_takes() names; in
// a decode step of the 8B shapes it is 0.6 % (8 rows) to 5.6 % (2 rows) faster, with the two
// norms of a layer folded into the q/k/v and gate/up products. The two cut K differently (8 and
// 16 warps), so their results differ in the last bits.
// Output forms:  bfloat16 or float32 [M,N];  added into a float32 [M,N] (the residual);  or,
// for a gate/up matrix whose rows are interleaved in eights (8 gate rows, the 8 matching up
// rows, ...), silu(gate) * up as bfloat16 [M, N/2].
#include "common.cuh"

#ifndef GS_UNROLL
#define GS_UNROLL 2             // 16-byte loads per row half in one register set
#endif
#ifndef GS_NARROW_UNROLL
#define GS_NARROW_UNROLL 4      // the same for a matrix with too few rows to fill the GPU
#endif

#define GS_OUT_BF16 0
#define GS_OUT_F32 1
#define GS_OUT_ADD_F32 2
#define GS_OUT_SWIGLU 3

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(uint32_t*)&v;
}

__device__ __forceinline__ uint4 load_x(const bf16* __restrict__ x, int m, int M, int K, int kk,
                                        bool valid_k) {
    if (m >= M || !valid_k) return make_uint4(0u, 0u, 0u, 0u);
    return *(const uint4*)(x + (size_t)m * K + kk);
}

template <int MT, int OMODE, int GS_WARPS, int UNROLL>
__global__ void __launch_bounds__(GS_WARPS * 32)
gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, void* __restrict__ y,
                   int M, int N, int K) {
    __shared__ float red[GS_WARPS][16][MT * 8 + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * 16;
    int slice = (K + GS_WARPS - 1) / GS_WARPS;
    slice = (slice + 31) / 32 * 32;
    const int k_begin = warp * slice;
    const int k_end = k_begin + slice < K ? k_begin + slice : K;
    const int row_lo = n0 + g, row_hi = n0 + g + 8;
    const bf16* w_lo = w + (size_t)(row_lo < N ? row_lo : 0) * K;
    const bf16* w_hi = w + (size_t)(row_hi < N ? row_hi : 0) * K;
    const bool ok_lo = row_lo < N, ok_hi = row_hi < N;
    constexpr int STEP = 32 * UNROLL;

    float acc[MT][4];
#pragma unroll
    for (int j = 0; j < MT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

    uint4 a_lo[UNROLL], a_hi[UNROLL], b_lo[UNROLL], b_hi[UNROLL];
    auto load_w = [&](uint4 (&lo)[UNROLL], uint4 (&hi)[UNROLL], int k) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int kk = k + u * 32 + 8 * t;
            const bool v = kk < k_end;
            lo[u] = (v && ok_lo) ? ldg_stream(w_lo + kk) : make_uint4(0u, 0u, 0u, 0u);
            hi[u] = (v && ok_hi) ? ldg_stream(w_hi + kk) : make_uint4(0u, 0u, 0u, 0u);
        }
    };
    auto multiply = [&](const uint4 (&lo)[UNROLL], const uint4 (&hi)[UNROLL], int k) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int kk = k + u * 32 + 8 * t;
            const bool v = kk < k_end;
#pragma unroll
            for (int j = 0; j < MT; ++j) {
                const uint4 b = load_x(x, j * 8 + g, M, K, kk, v);
                mma_bf16_16816(acc[j], lo[u].x, hi[u].x, lo[u].y, hi[u].y, b.x, b.y);
                mma_bf16_16816(acc[j], lo[u].z, hi[u].z, lo[u].w, hi[u].w, b.z, b.w);
            }
        }
    };
    // The weights depend on no earlier kernel: the first loads go out before this kernel
    // waits for the one that makes x, so the stream from HBM is already running when it ends.
    load_w(a_lo, a_hi, k_begin);
    load_w(b_lo, b_hi, k_begin + STEP);
    pdl_wait();
    for (int k = k_begin; k < k_end; k += 2 * STEP) {
        multiply(a_lo, a_hi, k);
        load_w(a_lo, a_hi, k + 2 * STEP);
        if (k + STEP < k_end) multiply(b_lo, b_hi, k + STEP);
        load_w(b_lo, b_hi, k + 3 * STEP);
    }
    pdl_launch_late();
    // partial tiles -> shared memory: [warp][row of W][batch row]
#pragma unroll
    for (int j = 0; j < MT; ++j) {
        red[warp][g][j * 8 + 2 * t] = acc[j][0];
        red[warp][g][j * 8 + 2 * t + 1] = acc[j][1];
        red[warp][g + 8][j * 8 + 2 * t] = acc[j][2];
        red[warp][g + 8][j * 8 + 2 * t + 1] = acc[j][3];
    }
    __syncthreads();
    if (OMODE == GS_OUT_SWIGLU) {
        // rows 0..7 of the tile are gate columns n0/2 .. n0/2+7, rows 8..15 the matching up
        for (int i = threadIdx.x; i < 8 * MT * 8; i += GS_WARPS * 32) {
            const int r = i & 7, m = i >> 3;
            const int col = n0 / 2 + r;
            if (m >= M || col >= N / 2) continue;
            float gt = 0.f, up = 0.f;
#pragma unroll
            for (int wv = 0; wv < GS_WARPS; ++wv) { gt += red[wv][r][m]; up += red[wv][r + 8][m]; }
            // the gate and up values pass through bfloat16 as they do when the product is
            // stored before the gate is applied
            gt = __bfloat162float(__float2bfloat16_rn(gt));
            up = __bfloat162float(__float2bfloat16_rn(up));
            ((bf16*)y)[(size_t)m * (N / 2) + col] = __float2bfloat16_rn(gt / (1.f + expf(-gt)) * up);
        }
        return;
    }
    // 16 x (MT*8) outputs; consecutive threads take consecutive rows of W (contiguous in y)
    for (int i = threadIdx.x; i < 16 * MT * 8; i += GS_WARPS * 32) {
        const int r = i & 15, m = i >> 4;
        const int n = n0 + r;
        if (m >= M || n >= N) continue;
        float s = 0.f;
#pragma unroll
        for (int wv = 0; wv < GS_WARPS; ++wv) s += red[wv][r][m];
        const size_t at = (size_t)m * N + n;
        if (OMODE == GS_OUT_BF16) ((bf16*)y)[at] = __float2bfloat16_rn(s);
        else if (OMODE == GS_OUT_F32) ((float*)y)[at] = s;
        else ((float*)y)[at] += s;
    }
}

template <int MT, int WARPS, int UNROLL>
static int gs_launch_o(const bf16* x, const bf16* w, void* y, int M, int N, int K, int omode,
                       cudaStream_t s) {
    const dim3 grid((N + 15) / 16), block(WARPS * 32);
    switch (omode) {
        case GS_OUT_BF16:
            return tgo_launch_pdl(gemm_skinny_kernel<MT, GS_OUT_BF16, WARPS, UNROLL>, grid, block, 0, s,
                                  x, w, y, M, N, K);
        case GS_OUT_F32:
            return tgo_launch_pdl(gemm_skinny_kernel<MT, GS_OUT_F32, WARPS, UNROLL>, grid, block, 0, s,
                                  x, w, y, M, N, K);
        case GS_OUT_ADD_F32:
            return tgo_launch_pdl(gemm_skinny_kernel<MT, GS_OUT_ADD_F32, WARPS, UNROLL>, grid, block, 0,
                                  s, x, w, y, M, N, K);
        default:
            return tgo_launch_pdl(gemm_skinny_kernel<MT, GS_OUT_SWIGLU, WARPS, UNROLL>, grid, block, 0,
                                  s, x, w, y, M, N, K);
    }
}

// A CTA has 2 x UNROLL x 2 loads of 16 bytes a thread on their way, 32 KB with UNROLL 2, and
// what bounds the kernel is how many bytes the whole GPU has on their way (about 15 MB hide
// the latency of HBM at its full rate). A matrix of 4096 rows is only 256 CTAs: 8 MB. For
// such a matrix (its CTAs all fit on the GPU at two an SM) each thread keeps twice the loads
// in flight, at 110 registers; where there are more CTAs than that, three an SM with the
// smaller sets are better.
template <int MT>
static int gs_launch(const bf16* x, const bf16* w, void* y, int M, int N, int K, int omode,
                     cudaStream_t s) {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    const bool narrow = MT == 1 && GS_NARROW_UNROLL != GS_UNROLL && (N + 15) / 16 <= 2 * sms && K >= 2048;
    if constexpr (MT == 1) {        // only this one is built with the larger sets
        if (narrow) return gs_launch_o<MT, 8, GS_NARROW_UNROLL>(x, w, y, M, N, K, omode, s);
    }
    return gs_launch_o<MT, 8, GS_UNROLL>(x, w, y, M, N, K, omode, s);
}

// ------------------------------------------------------------------ the persistent form
// For at most 8 rows of x. One CTA per SM for the whole product: CTA c owns a contiguous
// range of the rows of W, about N / gridDim.x of them, and walks it in tiles of 16 rows. Its
// 16 warps each take a sixteenth of K of every tile, so a warp always needs the same columns
// of x: each warp stages its columns of x once in shared memory. The two register sets run
// over the flat sequence of (tile, k step) of the CTA, so the loads of the next tile are on their way while this
// tile's partial sums are added, and nothing starts or drains between tiles. The partial
// tiles of the 16 warps meet in one of GP_NB buffers in shared memory; the warps only arrive
// at a named barrier and go on loading, and one warp (tile mod 16) waits for all, adds them
// in warp order and stores. A buffer is written again only after its reducer has given it
// back through a second barrier.
// MEASURED on B200 with the global timer, inside a decode step of the 8B shapes at 8 rows: the
// gate/up product (201 MB) takes 36 us, its loop 27.6 us (6.6 TB/s); q/k/v 11.6 us with a loop
// of 5.9; o 9.6 with a loop of 3.8: between a kernel's start and its first product lie 4 us
// (index arithmetic and first instructions 0.9, x and the first weights 2 to 3) whatever the
// form, and that, 13 kernels a layer, is what holds a decode step at 0.63 of the HBM rate.
#define GP_WARPS 16
#define GP_UNROLL 4
#define GP_SET_K (32 * GP_UNROLL)
#define GP_NB 3
#define GP_RED_LD 9
#define GP_X_PAD 32             // elements between rows of x in shared memory beyond K: 64 bytes,
                                // so that the 16-byte reads of a quarter warp touch every bank once
#define GP_RED_BYTES (GP_NB * GP_WARPS * 16 * GP_RED_LD * 4)
#define GP_SSQ_BYTES (8 * GP_WARPS * 4)

__device__ __forceinline__ void named_arrive(int id) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(GP_WARPS * 32) : "memory");
}
__device__ __forceinline__ void named_sync(int id) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(GP_WARPS * 32) : "memory");
}

// With NORM_IN, x is not given: the rows are RMSNorm(hsrc) with `gain`, made here from the
// float32 stream while they are staged (each CTA for itself: 148 times 128 KB from the L2
// instead of a kernel of its own between two products).
template <int OMODE, bool NORM_IN>
__global__ void __launch_bounds__(GP_WARPS * 32, 1)
gemm_stream_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, void* __restrict__ y,
                   int M, int N, int K, int unit, const float* __restrict__ hsrc,
                   const float* __restrict__ gain, float eps) {
    extern __shared__ __align__(16) unsigned char gp_smem[];
    float* red = (float*)gp_smem;
    float* ssq = (float*)(gp_smem + GP_RED_BYTES);            // [8][GP_WARPS]
    bf16* xs = (bf16*)(gp_smem + GP_RED_BYTES + GP_SSQ_BYTES);
    const int xs_ld = K + GP_X_PAD;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    // the rows of W of this CTA: whole units (16 rows for a gated pair of eights, else 8)
    const int n_units = (N + unit - 1) / unit;
    const unsigned u0 = blockIdx.x * (unsigned)n_units / gridDim.x;      // the launch keeps these
    const unsigned u1 = (blockIdx.x + 1) * (unsigned)n_units / gridDim.x;  // products below 2^32
    const int r0 = (int)(u0 * unit);
    const int r1 = (int)(u1 * unit) < N ? (int)(u1 * unit) : N;
    const int n_tiles = r1 > r0 ? (r1 - r0 + 15) / 16 : 0;

    int slice = (K + GP_WARPS - 1) / GP_WARPS;
    slice = (slice + 31) / 32 * 32;
    const int k_begin = warp * slice;
    const int k_end = k_begin + slice < K ? k_begin + slice : K;
    const int n_sets = (slice + GP_SET_K - 1) / GP_SET_K;
    const int total = n_tiles * n_sets;

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    uint4 a_lo[GP_UNROLL], a_hi[GP_UNROLL], b_lo[GP_UNROLL], b_hi[GP_UNROLL];

    int ld_tile = 0, ld_set = 0;
    auto load_w = [&](uint4 (&lo)[GP_UNROLL], uint4 (&hi)[GP_UNROLL]) {
        if (ld_tile < n_tiles) {
            const int row_lo = r0 + ld_tile * 16 + g, row_hi = row_lo + 8;
            const bool ok_lo = row_lo < r1, ok_hi = row_hi < r1;
            const bf16* p_lo = w + (size_t)(ok_lo ? row_lo : 0) * K;
            const bf16* p_hi = w + (size_t)(ok_hi ? row_hi : 0) * K;
#pragma unroll
            for (int u = 0; u < GP_UNROLL; ++u) {
                const int kk = k_begin + ld_set * GP_SET_K + u * 32 + 8 * t;
                const bool v = kk < k_end;
                lo[u] = (v && ok_lo) ? ldg_stream(p_lo + kk) : make_uint4(0u, 0u, 0u, 0u);
                hi[u] = (v && ok_hi) ? ldg_stream(p_hi + kk) : make_uint4(0u, 0u, 0u, 0u);
            }
        }
        if (++ld_set == n_sets) { ld_set = 0; ++ld_tile; }
    };

    auto reduce_and_store = [&](int tile, int buf) {
        const float* rb = red + (size_t)buf * GP_WARPS * 16 * GP_RED_LD;
        const int row0 = r0 + tile * 16;
        if (OMODE == GS_OUT_SWIGLU) {
            // rows 0..7 of the tile are gate columns row0/2 .. row0/2+7, rows 8..15 the matching up
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const int o = lane + 32 * q, r = o & 7, m = o >> 3;
                const int col = row0 / 2 + r;
                if (m >= M || row0 + r >= r1) continue;        // N is a multiple of 16: whole tiles
                float gt = 0.f, up = 0.f;
#pragma unroll
                for (int wv = 0; wv < GP_WARPS; ++wv) {
                    gt += rb[(wv * 16 + r) * GP_RED_LD + m];
                    up += rb[(wv * 16 + r + 8) * GP_RED_LD + m];
                }
                gt = __bfloat162float(__float2bfloat16_rn(gt));
                up = __bfloat162float(__float2bfloat16_rn(up));
                ((bf16*)y)[(size_t)m * (N / 2) + col] = __float2bfloat16_rn(gt / (1.f + expf(-gt)) * up);
            }
            return;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int o = lane + 32 * q, r = o & 15, m = o >> 4;
            const int n = row0 + r;
            if (m >= M || n >= r1) continue;
            float s = 0.f;
#pragma unroll
            for (int wv = 0; wv < GP_WARPS; ++wv) s += rb[(wv * 16 + r) * GP_RED_LD + m];
            const size_t at = (size_t)m * N + n;
            if (OMODE == GS_OUT_BF16) ((bf16*)y)[at] = __float2bfloat16_rn(s);
            else if (OMODE == GS_OUT_F32) ((float*)y)[at] = s;
            else ((float*)y)[at] += s;
        }
    };

    // barriers 1..GP_NB: a buffer's partial tiles are all there; GP_NB+1..2*GP_NB: it is free again
    auto flush = [&](int tile) {
        const int buf = tile % GP_NB;
        if (tile >= GP_NB && warp != (tile - GP_NB) % GP_WARPS) named_sync(1 + GP_NB + buf);
        float* rb = red + ((size_t)(buf * GP_WARPS + warp) * 16) * GP_RED_LD;
        rb[g * GP_RED_LD + 2 * t] = acc[0];
        rb[g * GP_RED_LD + 2 * t + 1] = acc[1];
        rb[(g + 8) * GP_RED_LD + 2 * t] = acc[2];
        rb[(g + 8) * GP_RED_LD + 2 * t + 1] = acc[3];
        acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
        __threadfence_block();
        if (warp == tile % GP_WARPS) {
            named_sync(1 + buf);
            reduce_and_store(tile, buf);
            if (tile + GP_NB < n_tiles) {
                __threadfence_block();
                named_arrive(1 + GP_NB + buf);
            }
        } else {
            named_arrive(1 + buf);
        }
    };

    int c_tile = 0, c_set = 0;
    auto multiply = [&](const uint4 (&lo)[GP_UNROLL], const uint4 (&hi)[GP_UNROLL]) {
#pragma unroll
        for (int u = 0; u < GP_UNROLL; ++u) {
            const int kk = k_begin + c_set * GP_SET_K + u * 32 + 8 * t;
            uint4 b = make_uint4(0u, 0u, 0u, 0u);
            if (g < M && kk < k_end) b = *(const uint4*)(xs + (size_t)g * xs_ld + kk);
            mma_bf16_16816(acc, lo[u].x, hi[u].x, lo[u].y, hi[u].y, b.x, b.y);
            mma_bf16_16816(acc, lo[u].z, hi[u].z, lo[u].w, hi[u].w, b.z, b.w);
        }
        if (++c_set == n_sets) { c_set = 0; flush(c_tile); ++c_tile; }
    };

    // The first weights before the wait for the kernel that makes x: they depend on nothing.
    // Where the rows are made here from the float32 stream this matters most: every CTA reads
    // the same 128 KB of it from the L2, 4.4 us during which HBM would stand idle (a decode step
    // went from 3.43 to 3.29 ms at batch 1 and from 3.91 to 3.86 at batch 8); for rows given
    // as bfloat16 the copies of x then queue behind the weights (2.7 us instead of 1.9), but the
    // step still gains (3.29 to 3.27, 3.85 to 3.84).
    load_w(a_lo, a_hi);
    load_w(b_lo, b_hi);
    pdl_wait();
    if (NORM_IN && k_end - k_begin <= 256) {
        // four rows' pieces in registers at a time (both sets of weights are on their way):
        // the sums of squares first, then the rows again (from the L1 now) to scale them
        const int cols4 = k_end > k_begin ? (k_end - k_begin) / 4 : 0;
        auto load4 = [&](float4 (&v)[4][2], int m0) {
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int c = lane + 32 * q, m = m0 + r;
                    v[r][q] = (m < M && c < cols4) ? *(const float4*)(hsrc + (size_t)m * K + k_begin + 4 * c)
                                                   : make_float4(0.f, 0.f, 0.f, 0.f);
                }
        };
        for (int m0 = 0; m0 < M; m0 += 4) {
            float4 v[4][2];
            load4(v, m0);
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                float ss = 0.f;
#pragma unroll
                for (int q = 0; q < 2; ++q)
                    ss += v[r][q].x * v[r][q].x + v[r][q].y * v[r][q].y + v[r][q].z * v[r][q].z + v[r][q].w * v[r][q].w;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (lane == 0) ssq[(m0 + r) * GP_WARPS + warp] = ss;
            }
        }
        __syncthreads();
        float4 gn[2];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int c = lane + 32 * q;
            gn[q] = c < cols4 ? *(const float4*)(gain + k_begin + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        for (int m0 = 0; m0 < M; m0 += 4) {
            float4 v[4][2];
            load4(v, m0);
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int m = m0 + r;
                if (m >= M) break;
                float total = 0.f;
#pragma unroll
                for (int wv = 0; wv < GP_WARPS; ++wv) total += ssq[m * GP_WARPS + wv];
                const float scale = rsqrtf(total / (float)K + eps);
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int c = lane + 32 * q;
                    if (c >= cols4) continue;
                    __nv_bfloat162 lo2 = __floats2bfloat162_rn((v[r][q].x * scale) * gn[q].x, (v[r][q].y * scale) * gn[q].y);
                    __nv_bfloat162 hi2 = __floats2bfloat162_rn((v[r][q].z * scale) * gn[q].z, (v[r][q].w * scale) * gn[q].w);
                    uint2 pk;
                    pk.x = *(uint32_t*)&lo2;
                    pk.y = *(uint32_t*)&hi2;
                    *(uint2*)(xs + (size_t)m * xs_ld + k_begin + 4 * c) = pk;
                }
            }
        }
    } else if (NORM_IN) {
        const int cols4 = k_end > k_begin ? (k_end - k_begin) / 4 : 0;
        for (int m = 0; m < M; ++m) {
            const float* hr = hsrc + (size_t)m * K + k_begin;
            float ss = 0.f;
            for (int c = lane; c < cols4; c += 32) {
                const float4 v = *(const float4*)(hr + 4 * c);
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) ssq[m * GP_WARPS + warp] = ss;
        }
        __syncthreads();
        for (int m = 0; m < M; ++m) {
            float total = 0.f;
#pragma unroll
            for (int wv = 0; wv < GP_WARPS; ++wv) total += ssq[m * GP_WARPS + wv];
            const float scale = rsqrtf(total / (float)K + eps);
            const float* hr = hsrc + (size_t)m * K + k_begin;
            for (int c = lane; c < cols4; c += 32) {
                const float4 v = *(const float4*)(hr + 4 * c);
                const float4 gn = *(const float4*)(gain + k_begin + 4 * c);
                __nv_bfloat162 lo2 = __floats2bfloat162_rn((v.x * scale) * gn.x, (v.y * scale) * gn.y);
                __nv_bfloat162 hi2 = __floats2bfloat162_rn((v.z * scale) * gn.z, (v.w * scale) * gn.w);
                uint2 pk;
                pk.x = *(uint32_t*)&lo2;
                pk.y = *(uint32_t*)&hi2;
                *(uint2*)(xs + (size_t)m * xs_ld + k_begin + 4 * c) = pk;
            }
        }
    } else {
        // Each warp stages the columns of x that it alone reads. Every CTA copies the same x,
        // so each starts at another place: the requests of the moment then spread over x,
        // and over the L2, instead of all asking for one line.
        const int cols = k_end > k_begin ? (k_end - k_begin) / 8 : 0;      // 16-byte pieces a row
        const int n = M * cols;
        const int rot = n > 0 ? (int)((blockIdx.x * 37u) % (unsigned)n) : 0;
        for (int i = lane; i < n; i += 32) {
            int j = i + rot;
            if (j >= n) j -= n;
            const int m = j / cols, c = j - m * cols;
            const unsigned dst = (unsigned)__cvta_generic_to_shared(xs + (size_t)m * xs_ld + k_begin + c * 8);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst),
                         "l"(x + (size_t)m * K + k_begin + c * 8) : "memory");
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    }
    if (!NORM_IN) asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncwarp();
    for (int s = 0; s < total; s += 2) {
        multiply(a_lo, a_hi);
        load_w(a_lo, a_hi);
        if (s + 1 < total) {
            multiply(b_lo, b_hi);
            load_w(b_lo, b_hi);
        }
    }
    pdl_launch_late();
}

// Shared memory the persistent form needs; it is taken for at most 8 rows when that fits.
static size_t gp_smem_bytes(int M, int K) {
    return (size_t)GP_RED_BYTES + GP_SSQ_BYTES + (size_t)M * (K + GP_X_PAD) * sizeof(bf16);
}

template <int OMODE, bool NORM_IN>
static int gp_launch_o(const bf16* x, const bf16* w, void* y, int M, int N, int K, int grid,
                       size_t smem, const float* hsrc, const float* gain, float eps, cudaStream_t s) {
    static size_t allowed = 0;          // grows to the most any call has asked for
    if (smem > allowed) {
        const cudaError_t e = cudaFuncSetAttribute(
            gemm_stream_kernel<OMODE, NORM_IN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return (int)e;
        }
        allowed = smem;
    }
    return tgo_launch_pdl(gemm_stream_kernel<OMODE, NORM_IN>, dim3(grid), dim3(GP_WARPS * 32), smem, s,
                          x, w, y, M, N, K, OMODE == GS_OUT_SWIGLU ? 16 : 8, hsrc, gain, eps);
}

#ifndef GS_STREAM
#define GS_STREAM 1
#endif
#ifndef GP_MAX_ROWS
#define GP_MAX_ROWS 8
#endif
#ifndef GP_MAX_SMEM
#define GP_MAX_SMEM (128 * 1024)
#endif

// Whether the persistent form takes a product of these sizes: few rows; enough rows of W to
// give every warp of a CTA something to reduce; a K that gives each warp whole register sets
// (with 5120, two and a half sets a warp, it was 5-8 % behind the other form in a decode step
// of the 14B and 32B shapes); and rows of x that leave most of the SM's shared memory to the
// L1 (with 197 KB of x, the 8 x 12288 rows of a down projection, the loads in flight were held
// to a third and the product took 44 us instead of 22).
static bool gp_takes(int M, int N, int K) {
    return GS_STREAM && M <= GP_MAX_ROWS && N >= 16 * GP_WARPS && N < (1 << 24) &&
           K % (GP_WARPS * GP_SET_K) == 0 && gp_smem_bytes(M, K) <= GP_MAX_SMEM;
}

// 1: done by the persistent form; 0: not taken (the caller goes on to the other form); < 0: error
static int gp_try(const bf16* x, const bf16* w, void* y, int M, int N, int K, int omode,
                  cudaStream_t s, const float* hsrc = nullptr, const float* gain = nullptr,
                  float eps = 0.f) {
    if (!gp_takes(M, N, K)) return 0;
    const size_t smem = gp_smem_bytes(M, K);
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    const int tiles = (N + 15) / 16;
    const int grid = tiles < sms ? tiles : sms;
    int rc;
    if (hsrc) {
        switch (omode) {
            case GS_OUT_BF16: rc = gp_launch_o<GS_OUT_BF16, true>(x, w, y, M, N, K, grid, smem, hsrc, gain, eps, s); break;
            case GS_OUT_F32: rc = gp_launch_o<GS_OUT_F32, true>(x, w, y, M, N, K, grid, smem, hsrc, gain, eps, s); break;
            case GS_OUT_SWIGLU: rc = gp_launch_o<GS_OUT_SWIGLU, true>(x, w, y, M, N, K, grid, smem, hsrc, gain, eps, s); break;
            default: return 0;
        }
        return rc ? -rc : 1;
    }
    switch (omode) {
        case GS_OUT_BF16: rc = gp_launch_o<GS_OUT_BF16, false>(x, w, y, M, N, K, grid, smem, nullptr, nullptr, 0.f, s); break;
        case GS_OUT_F32: rc = gp_launch_o<GS_OUT_F32, false>(x, w, y, M, N, K, grid, smem, nullptr, nullptr, 0.f, s); break;
        case GS_OUT_ADD_F32: rc = gp_launch_o<GS_OUT_ADD_F32, false>(x, w, y, M, N, K, grid, smem, nullptr, nullptr, 0.f, s); break;
        default: rc = gp_launch_o<GS_OUT_SWIGLU, false>(x, w, y, M, N, K, grid, smem, nullptr, nullptr, 0.f, s); break;
    }
    return rc ? -rc : 1;
}

// Most rows this kernel takes; K must be a multiple of 8 (16-byte loads).
TGO_API int tgo_gemm_skinny_max_rows() { return 64; }

// Whether tgo_gemm_skinny_normed takes these sizes.
TGO_API int tgo_gemm_skinny_folds_norm(int M, int N, int K) { return gp_takes(M, N, K) ? 1 : 0; }

// y = RMSNorm(h; gain, eps) . W^T for at most 8 rows, the norm folded into the persistent
// form's staging of its rows. Returns TGO_E_BAD_ARG where that form does not take the sizes
// (the caller then norms with a kernel of its own).
TGO_API int tgo_gemm_skinny_normed(const float* h, const float* gain, float eps, const void* w,
                                   void* y, int M, int N, int K, int omode, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || M > 8 || omode < 0 || omode > 3 || omode == GS_OUT_ADD_F32 ||
        (omode == GS_OUT_SWIGLU && N % 16) || ((uintptr_t)h % 16) || ((uintptr_t)gain % 16))
        return TGO_E_BAD_ARG;
    const int rc = gp_try(nullptr, (const bf16*)w, y, M, N, K, omode, stream, h, gain, eps);
    return rc > 0 ? 0 : rc < 0 ? -rc : TGO_E_BAD_ARG;
}

TGO_API int tgo_gemm_skinny(const void* x, const void* w, void* y, int M, int N, int K, int omode,
                            cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || M > 64 || omode < 0 || omode > 3 || (omode == GS_OUT_SWIGLU && N % 16))
        return TGO_E_BAD_ARG;
    const bf16 *xp = (const bf16*)x, *wp = (const bf16*)w;
    if (M <= 8) {
        const int rc = gp_try(xp, wp, y, M, N, K, omode, stream);
        if (rc) return rc > 0 ? 0 : -rc;
        return gs_launch<1>(xp, wp, y, M, N, K, omode, stream);
    }
    if (M <= 16) return gs_launch<2>(xp, wp, y, M, N, K, omode, stream);
    if (M <= 32) return gs_launch<4>(xp, wp, y, M, N, K, omode, stream);
    return gs_launch<8>(xp, wp, y, M, N, K, omode, stream);
}
