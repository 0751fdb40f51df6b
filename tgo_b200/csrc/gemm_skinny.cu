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
// Input: x bfloat16 [M,K]. (Taking the float32 residual stream and a gain instead, RMSNorm
// folded into the product, was measured slower at every batch size: every CTA re-reads the
// stream and the gain.)
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

// Most rows this kernel takes; K must be a multiple of 8 (16-byte loads).
TGO_API int tgo_gemm_skinny_max_rows() { return 64; }

TGO_API int tgo_gemm_skinny(const void* x, const void* w, void* y, int M, int N, int K, int omode,
                            cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || M > 64 || omode < 0 || omode > 3 || (omode == GS_OUT_SWIGLU && N % 16))
        return TGO_E_BAD_ARG;
    const bf16 *xp = (const bf16*)x, *wp = (const bf16*)w;
    if (M <= 8) return gs_launch<1>(xp, wp, y, M, N, K, omode, stream);
    if (M <= 16) return gs_launch<2>(xp, wp, y, M, N, K, omode, stream);
    if (M <= 32) return gs_launch<4>(xp, wp, y, M, N, K, omode, stream);
    return gs_launch<8>(xp, wp, y, M, N, K, omode, stream);
}
