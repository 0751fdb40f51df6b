// A chain of small-batch matrix products in ONE persistent kernel (at most 8 rows: a decode
// step). The phases of a chain run back to back in the same resident CTAs: a grid-wide barrier
// stands where the kernel boundary was, and before a CTA waits at it, it issues the first
// weight loads of the next phase, so HBM keeps streaming through the barrier.
//
// MEASURED, Qwen3-8B layer shapes, 8 rows, B200: the four products of a layer take 171 us as
// one chain and 105 us as separate dependent launches; a whole decode step takes 7.0 ms with
// chains and 4.4 ms without. One CTA per SM leaves fewer loads in flight than two resident
// CTAs of the separate kernel, 16-row tiles dealt to 148 CTAs leave the last wave 27% empty
// for a 4096-row matrix, and every CTA stages the whole of x again in every phase. The
// engine therefore does not use this kernel unless ops.USE_CHAINS is set; it stays built and
// tested so that the comparison can be repeated.
//
// A phase is  y = epilogue( act(x) . W^T ):
//   x   rows of the float32 residual stream h, normalised on the way in: bf16(h * rsqrt(mean
//       h^2 + eps) * gain) (RMSNorm needs no kernel of its own), or a bfloat16 matrix;
//   W   [N, K] bfloat16, streamed once with 16-byte loads straight into mma.sync m16n8k16
//       fragments (weight rows on the M axis, the batch on N; see gemm_skinny.cu);
//   y   bfloat16 [M, N]; added into the float32 stream h [M, N]; or, for a gate/up matrix
//       with rows interleaved in eights, silu(gate) * up as bfloat16 [M, N / 2].
// x is staged once per CTA in shared memory (padded rows, conflict-free fragment reads).
// 16-row tiles of W are dealt round-robin to the CTAs; the 16 warps of a CTA split K and their
// partial tiles are added in warp order, so results do not depend on timing.
//
// The grid is one CTA per SM, launched cooperatively (all CTAs resident). The barrier is a
// counter and a generation in global memory that reset themselves, so a captured graph may
// replay the kernel. A wait that lasts two seconds sets *err and is not repeated.
#include <cooperative_groups.h>

#include "common.cuh"

#define GC_WARPS 16
#define GC_THREADS (GC_WARPS * 32)
#define GC_UNROLL 4
#define GC_MAX_PHASES 4
#define GC_WAIT_CYCLES 4000000000ll

#define GC_X_NORM 0          // x = float32 stream with gain
#define GC_X_BF16 1
#define GC_OUT_BF16 0
#define GC_OUT_ADD_F32 2
#define GC_OUT_SWIGLU 3

struct GcPhase {
    const void* x;           // float32 [M, K] (GC_X_NORM) or bfloat16 [M, K]
    const float* gain;       // [K] for GC_X_NORM
    const bf16* w;           // [N, K]
    void* y;
    float eps;
    int x_kind, out_kind, N, K;
};

struct GcArgs {
    GcPhase phase[GC_MAX_PHASES];
    int n_phases, M;
    int* barrier;            // [2]: arrivals, generation
    int* err;
};

__device__ __forceinline__ uint4 gc_ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void gc_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// All CTAs of the grid meet here. Arrivals are counted; the last one resets the count and
// moves the generation on, which the others watch. Returns false after a time-out (or if an
// earlier one was recorded), and the caller goes on without waiting again.
__device__ bool gc_grid_barrier(int* bar, int* err) {
    __shared__ int s_ok;
    __syncthreads();
    if (threadIdx.x == 0) {
        int ok = 1;
        if (*(volatile int*)err != 0) {
            ok = 0;
        } else {
            const int gen = *(volatile int*)(bar + 1);
            __threadfence();
            if (atomicAdd(bar, 1) == (int)gridDim.x - 1) {
                *(volatile int*)bar = 0;
                __threadfence();
                atomicAdd(bar + 1, 1);
            } else {
                const long long start = clock64();
                while (*(volatile int*)(bar + 1) == gen) {
                    if (clock64() - start > GC_WAIT_CYCLES) {
                        atomicExch(err, 7);
                        ok = 0;
                        break;
                    }
                }
            }
            __threadfence();
        }
        s_ok = ok;
    }
    __syncthreads();
    return s_ok != 0;
}

// x of one phase -> shared memory as bfloat16 [M][ldx] (rows beyond M are zeros).
__device__ void gc_stage_x(const GcPhase& p, int M, bf16* x_s, int ldx, float* scale_s) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int K = p.K;
    if (p.x_kind == GC_X_NORM) {
        const float* h = (const float*)p.x;
        for (int m = warp; m < 8; m += GC_WARPS) {
            float ss = 0.f;
            if (m < M)
                for (int k = 4 * lane; k < K; k += 128) {
                    const float4 v = *(const float4*)(h + (size_t)m * K + k);
                    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                }
            ss = warp_sum(ss);
            if (lane == 0) scale_s[m] = rsqrtf(ss / (float)K + p.eps);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < 8 * (K / 4); i += GC_THREADS) {
            const int m = i / (K / 4), k = 4 * (i % (K / 4));
            uint2 pk = make_uint2(0u, 0u);
            if (m < M) {
                const float4 v = *(const float4*)(h + (size_t)m * K + k);
                const float4 g = *(const float4*)(p.gain + k);
                const float s = scale_s[m];
                __nv_bfloat162 a = __floats2bfloat162_rn((v.x * s) * g.x, (v.y * s) * g.y);
                __nv_bfloat162 b = __floats2bfloat162_rn((v.z * s) * g.z, (v.w * s) * g.w);
                pk.x = *(uint32_t*)&a;
                pk.y = *(uint32_t*)&b;
            }
            *(uint2*)(x_s + (size_t)m * ldx + k) = pk;
        }
    } else {
        const bf16* x = (const bf16*)p.x;
        for (int i = threadIdx.x; i < 8 * (K / 8); i += GC_THREADS) {
            const int m = i / (K / 8), k = 8 * (i % (K / 8));
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (m < M) v = *(const uint4*)(x + (size_t)m * K + k);
            *(uint4*)(x_s + (size_t)m * ldx + k) = v;
        }
    }
    __syncthreads();
}

__device__ __forceinline__ float gc_bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__global__ void __launch_bounds__(GC_THREADS, 1) gemm_chain_kernel(const GcArgs a) {
    extern __shared__ __align__(16) unsigned char gc_smem[];
    __shared__ float red[2][GC_WARPS][16][9];
    __shared__ float scale_s[8];
    bf16* x_s = (bf16*)gc_smem;
    pdl_wait();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int M = a.M;
    bool alive = true;

    for (int ph = 0; ph < a.n_phases; ++ph) {
        const GcPhase& p = a.phase[ph];
        const int K = p.K, N = p.N;
        const int ldx = K + 8;                             // padded: fragment reads hit distinct banks
        int slice = (K + GC_WARPS - 1) / GC_WARPS;
        slice = (slice + 31) / 32 * 32;
        const int k_begin = warp * slice;
        const int k_end = k_begin + slice < K ? k_begin + slice : K;
        const int n_tiles = (N + 15) / 16;

        // The work of this CTA in this phase is a sequence of steps (tile, k-step). Weight loads
        // run a step ahead of the products in two register sets used in turn (no copies, so a
        // set is only waited for when it is multiplied): loads stay in flight across k-steps,
        // across the reduction and store of a tile, and across the barrier before the phase,
        // since a phase's weights depend on nothing the previous phase wrote.
        const int iters = k_end > k_begin ? (k_end - k_begin + 32 * GC_UNROLL - 1) / (32 * GC_UNROLL) : 0;
        int iters_max = (slice + 32 * GC_UNROLL - 1) / (32 * GC_UNROLL);     // the same for every warp
        if (iters_max < 1) iters_max = 1;
        const int my_tiles = (int)blockIdx.x < n_tiles ? (n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
        const int steps = my_tiles * iters_max;
        uint4 a_lo[GC_UNROLL], a_hi[GC_UNROLL], b_lo[GC_UNROLL], b_hi[GC_UNROLL];
        auto load_w = [&](uint4 (&lo)[GC_UNROLL], uint4 (&hi)[GC_UNROLL], int step) {
            const int tile = (int)blockIdx.x + (step / iters_max) * (int)gridDim.x;
            const int k = k_begin + (step % iters_max) * 32 * GC_UNROLL;
            const int row_lo = tile * 16 + g, row_hi = row_lo + 8;
            const bool in = step < steps;
            const bool ok_lo = in && row_lo < N, ok_hi = in && row_hi < N;
            const bf16* w_lo = p.w + (size_t)(ok_lo ? row_lo : 0) * K;
            const bf16* w_hi = p.w + (size_t)(ok_hi ? row_hi : 0) * K;
#pragma unroll
            for (int u = 0; u < GC_UNROLL; ++u) {
                const int kk = k + u * 32 + 8 * t;
                const bool v = kk < k_end;
                lo[u] = (v && ok_lo) ? gc_ldg_stream(w_lo + kk) : make_uint4(0u, 0u, 0u, 0u);
                hi[u] = (v && ok_hi) ? gc_ldg_stream(w_hi + kk) : make_uint4(0u, 0u, 0u, 0u);
            }
        };
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        auto compute = [&](const uint4 (&lo)[GC_UNROLL], const uint4 (&hi)[GC_UNROLL], int step) {
            const int tile = (int)blockIdx.x + (step / iters_max) * (int)gridDim.x;
            const int it = step % iters_max;
            const int k = k_begin + it * 32 * GC_UNROLL;
            if (it == 0) { acc[0] = acc[1] = acc[2] = acc[3] = 0.f; }
#pragma unroll
            for (int u = 0; u < GC_UNROLL; ++u) {
                const int kk = k + u * 32 + 8 * t;
                uint4 xb = make_uint4(0u, 0u, 0u, 0u);
                if (kk < k_end) xb = *(const uint4*)(x_s + (size_t)g * ldx + kk);
                gc_mma(acc, lo[u].x, hi[u].x, lo[u].y, hi[u].y, xb.x, xb.y);
                gc_mma(acc, lo[u].z, hi[u].z, lo[u].w, hi[u].w, xb.z, xb.w);
            }
            if (it != iters_max - 1) return;
            // the tile is complete: partial tiles -> shared memory [warp][row of W][batch row],
            // then summed in warp order by the threads that store
            float (*rd)[16][9] = red[(step / iters_max) & 1];
            rd[warp][g][2 * t] = acc[0];
            rd[warp][g][2 * t + 1] = acc[1];
            rd[warp][g + 8][2 * t] = acc[2];
            rd[warp][g + 8][2 * t + 1] = acc[3];
            __syncthreads();
            if (p.out_kind == GC_OUT_SWIGLU) {
                if (threadIdx.x < 64) {
                    const int r = threadIdx.x & 7, m = threadIdx.x >> 3;
                    const int col = tile * 8 + r;
                    if (m < M && col < N / 2) {
                        float gt = 0.f, up = 0.f;
#pragma unroll
                        for (int wv = 0; wv < GC_WARPS; ++wv) { gt += rd[wv][r][m]; up += rd[wv][r + 8][m]; }
                        gt = gc_bf16_round(gt);
                        up = gc_bf16_round(up);
                        ((bf16*)p.y)[(size_t)m * (N / 2) + col] = __float2bfloat16_rn(gt / (1.f + expf(-gt)) * up);
                    }
                }
            } else if (threadIdx.x < 128) {
                const int r = threadIdx.x & 15, m = threadIdx.x >> 4;
                const int n = tile * 16 + r;
                if (m < M && n < N) {
                    float sum = 0.f;
#pragma unroll
                    for (int wv = 0; wv < GC_WARPS; ++wv) sum += rd[wv][r][m];
                    const size_t at = (size_t)m * N + n;
                    if (p.out_kind == GC_OUT_BF16) ((bf16*)p.y)[at] = __float2bfloat16_rn(sum);
                    else ((float*)p.y)[at] += sum;
                }
            }
            // no second barrier: the next tile writes the other half of `red`, and the tile
            // after that comes behind the next tile's barrier
        };
        (void)iters;
        load_w(a_lo, a_hi, 0);
        if (ph > 0 && alive) alive = gc_grid_barrier(a.barrier, a.err);
        gc_stage_x(p, M, x_s, ldx, scale_s);
        for (int step = 0; step < steps; step += 2) {
            load_w(b_lo, b_hi, step + 1);
            compute(a_lo, a_hi, step);
            load_w(a_lo, a_hi, step + 2);
            if (step + 1 < steps) compute(b_lo, b_hi, step + 1);
        }
        __syncthreads();
    }
    pdl_launch_late();
}

// Bytes of shared memory the chain needs for its widest x: 8 rows of (K + 8) bfloat16.
static size_t gc_smem_bytes(const GcArgs& a) {
    int kmax = 0;
    for (int i = 0; i < a.n_phases; ++i) kmax = a.phase[i].K > kmax ? a.phase[i].K : kmax;
    return (size_t)8 * (kmax + 8) * sizeof(bf16);
}

// phases: n_phases records of 9 values each, as 64-bit integers:
//   x pointer, gain pointer, w pointer, y pointer, eps (float bits), x_kind, out_kind, N, K
// barrier: int32[2] that starts at zero and is left to the kernel; err: int32[1].
TGO_API int tgo_gemm_chain(const long long* phases, int n_phases, int M, int* barrier, int* err,
                           cudaStream_t stream) {
    if (n_phases <= 0) return 0;
    if (n_phases > GC_MAX_PHASES || M <= 0 || M > 8 || !barrier || !err) return TGO_E_BAD_ARG;
    GcArgs a;
    a.n_phases = n_phases;
    a.M = M;
    a.barrier = barrier;
    a.err = err;
    for (int i = 0; i < n_phases; ++i) {
        const long long* r = phases + 9 * i;
        GcPhase& p = a.phase[i];
        p.x = (const void*)r[0];
        p.gain = (const float*)r[1];
        p.w = (const bf16*)r[2];
        p.y = (void*)r[3];
        const uint32_t bits = (uint32_t)r[4];
        memcpy(&p.eps, &bits, 4);
        p.x_kind = (int)r[5];
        p.out_kind = (int)r[6];
        p.N = (int)r[7];
        p.K = (int)r[8];
        if (p.N <= 0 || p.K <= 0 || p.K % 8 || !p.x || !p.w || !p.y || ((uintptr_t)p.x & 15) ||
            ((uintptr_t)p.w & 15) || (p.x_kind == GC_X_NORM && (!p.gain || p.K % 4)) ||
            (p.x_kind != GC_X_NORM && p.x_kind != GC_X_BF16) ||
            (p.out_kind != GC_OUT_BF16 && p.out_kind != GC_OUT_ADD_F32 && p.out_kind != GC_OUT_SWIGLU) ||
            (p.out_kind == GC_OUT_SWIGLU && p.N % 16))
            return TGO_E_BAD_ARG;
    }
    const size_t smem = gc_smem_bytes(a);
    if (smem > 200 * 1024) return TGO_E_BAD_ARG;
    cudaError_t e = cudaFuncSetAttribute(gemm_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    int dev = 0, sms = 0;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return (int)e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemm_chain_kernel, GC_THREADS, smem);
    if (e != cudaSuccess) return (int)e;
    if (per_sm < 1) return TGO_E_BAD_ARG;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sms);
    cfg.blockDim = dim3(GC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, gemm_chain_kernel, a);
}
