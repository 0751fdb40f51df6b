// D = A . B^T on the 5th-generation tensor cores: bfloat16 operands, both K-major (row-major
// with K contiguous, as activations [rows, K] and checkpoint weights [out, K] are), float32
// accumulation in tensor memory.
//
// One CTA computes one 128 x BN tile of D. Six warps, three roles:
//   warp 0, one lane   producer: TMA tile loads (128-byte swizzle) of A [128 x 64] and
//                      B [BN x 64] into a ring of shared-memory stages, completion counted
//                      on each stage's `full` mbarrier;
//   warp 1, one lane   issuer: tcgen05.mma (UMMA 128 x BN x 16, four per stage) from
//                      shared-memory descriptors into a TMEM accumulator; tcgen05.commit
//                      releases the stage (`empty`) and, after the last one, hands the
//                      accumulator over (`acc_full`). Warp 1 also allocates and frees TMEM;
//   warps 2..5         epilogue: tcgen05.ld of their 32-lane quarter of the accumulator,
//                      32 columns at a time, then the stores.
// Rows of A are rows of D and TMEM lanes; rows of B are columns of D and TMEM columns.
// `transpose_out` stores D^T instead: with the weight matrix as A and a few activation rows
// as B this is the decode orientation (weights on the 128-wide M axis, batch on N).
// `splits` > 1 cuts K over gridDim.z CTAs, each writing a float32 partial tile; a second
// kernel adds the partials in split order and applies the output form.
//
// Tails: TMA fills out-of-range rows and K with zeros; stores are guarded. K % 8 == 0.
// No cluster, no multicast. Every mbarrier wait gives up after about two seconds, records
// where in *err and lets the CTA run to its end (TMEM is freed on every path).
#include <cuda.h>

#include "common.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192
#define TC_WAIT_CYCLES 4000000000ll

#define TC_OUT_BF16 0
#define TC_OUT_F32 1
#define TC_OUT_ADD_F32 2
#define TC_OUT_PARTIAL 3      // float32 partial tile of a K split

__device__ __forceinline__ uint32_t tc_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tc_smem(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tc_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(tc_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Wait with a time limit. Returns false, and records `code`, if the phase never completed.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err, int code) {
    if (mbar_try(bar, parity)) return true;
    const long long start = clock64();
    while (!mbar_try(bar, parity)) {
        if (clock64() - start > TC_WAIT_CYCLES) {
            if (err) atomicExch(err, code);
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(tc_smem(dst)), "l"(map), "r"(tc_smem(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tc_smem(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major operand tile in shared memory, rows of 64 bf16 (128 bytes) with the 128-byte
// swizzle that TMA wrote: start address / 16, leading offset 1 (unused), stride between
// groups of eight rows 1024 bytes, descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc(const void* tile) {
    uint64_t d = (uint64_t)((tc_smem(tile) & 0x3ffff) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

template <int BN>
struct TcSmem {
    static constexpr int A_BYTES = TC_BM * TC_BK * 2;
    static constexpr int B_BYTES = BN * TC_BK * 2;
    static constexpr int STAGE = A_BYTES + B_BYTES;
    static constexpr int STAGES = (200 * 1024) / STAGE < 8 ? (200 * 1024) / STAGE : 8;
    static constexpr size_t TOTAL = (size_t)STAGES * STAGE + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

template <int BN, int OMODE, bool TRANSPOSE>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               void* __restrict__ out, int rows_a, int rows_b, int K, long long ld_out,
               int kb_per_split, int* __restrict__ err) {
    using L = TcSmem<BN>;
    constexpr int STAGES = L::STAGES;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(base + (size_t)STAGES * L::STAGE);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * TC_BM, n0 = blockIdx.x * BN;
    const int kb_total = (K + TC_BK - 1) / TC_BK;
    const int kb_lo = blockIdx.z * kb_per_split;
    const int kb_hi = kb_lo + kb_per_split < kb_total ? kb_lo + kb_per_split : kb_total;
    const int n_kb = kb_hi > kb_lo ? kb_hi - kb_lo : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(tc_smem(tmem_slot)), "r"((uint32_t)BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int i = 0; i < n_kb; ++i) {
                const int s = i % STAGES;
                const uint32_t round = (uint32_t)(i / STAGES);
                if (!mbar_wait(&empty[s], (round & 1) ^ 1, err, 1)) break;
                mbar_expect_tx(&full[s], L::STAGE);
                unsigned char* st = base + (size_t)s * L::STAGE;
                tma_load_2d(st, &map_a, (kb_lo + i) * TC_BK, m0, &full[s]);
                tma_load_2d(st + L::A_BYTES, &map_b, (kb_lo + i) * TC_BK, n0, &full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: float32 accumulate, bf16 x bf16, both K-major, N, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                   ((uint32_t)(TC_BM >> 4) << 24);
            bool ok = true;
            for (int i = 0; i < n_kb && ok; ++i) {
                const int s = i % STAGES;
                const uint32_t round = (uint32_t)(i / STAGES);
                ok = mbar_wait(&full[s], round & 1, err, 2);
                if (!ok) break;
                tc_fence_after();
                unsigned char* st = base + (size_t)s * L::STAGE;
                const uint64_t da = umma_desc(st), db = umma_desc(st + L::A_BYTES);
#pragma unroll
                for (int k = 0; k < TC_BK / 16; ++k)        // 16 bf16 = 32 bytes = 2 descriptor units
                    umma_bf16(tmem_base, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                              (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(&empty[s]);
            }
            umma_commit(acc_full);          // arrives once every MMA issued above has finished
        }
    } else {
        const int quarter = warp & 3;                       // TMEM lanes this warp may read
        const bool ok = mbar_wait(acc_full, 0, err, 3);
        tc_fence_after();
        const int row = quarter * 32 + lane;                // row of the tile = TMEM lane
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 32);
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                  "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
                  "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
                  "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
                  "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                : "r"(taddr));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (!ok || n_kb == 0) continue;
            const int gm = m0 + row;                        // row of A
            if (gm >= rows_a) continue;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const int gn = n0 + c * 32 + j;             // row of B
                if (gn >= rows_b) break;
                const float v = __uint_as_float(r[j]);
                size_t at;
                if (OMODE == TC_OUT_PARTIAL)
                    at = ((size_t)blockIdx.z * (TRANSPOSE ? rows_b : rows_a) + (TRANSPOSE ? gn : gm)) * ld_out +
                         (TRANSPOSE ? gm : gn);
                else
                    at = TRANSPOSE ? (size_t)gn * ld_out + gm : (size_t)gm * ld_out + gn;
                if (OMODE == TC_OUT_BF16) ((bf16*)out)[at] = __float2bfloat16_rn(v);
                else if (OMODE == TC_OUT_ADD_F32) ((float*)out)[at] += v;
                else ((float*)out)[at] = v;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
    }
}

// out = sum over splits of partial[s] (in split order), in the wanted output form.
template <int OMODE>
__global__ void gemm_tc_reduce_kernel(const float* __restrict__ partial, void* __restrict__ out,
                                      long long n, int splits) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        float s = 0.f;
        for (int k = 0; k < splits; ++k) s += partial[(size_t)k * n + i];
        if (OMODE == TC_OUT_BF16) ((bf16*)out)[i] = __float2bfloat16_rn(s);
        else if (OMODE == TC_OUT_ADD_F32) ((float*)out)[i] += s;
        else ((float*)out)[i] = s;
    }
}

// ------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// A [rows, K] bf16 row-major -> tiles of box_rows x 64 with the 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return TGO_E_BAD_ARG;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                          box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 2000 + (int)r;
}

template <int BN, int OMODE, bool TRANSPOSE>
static int tc_launch(const CUtensorMap& ma, const CUtensorMap& mb, void* out, int rows_a, int rows_b, int K,
                     long long ld_out, int splits, int kb_per_split, int* err, cudaStream_t stream) {
    auto kern = gemm_tc_kernel<BN, OMODE, TRANSPOSE>;
    const size_t smem = TcSmem<BN>::TOTAL;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const dim3 grid((rows_b + BN - 1) / BN, (rows_a + TC_BM - 1) / TC_BM, splits);
    kern<<<grid, TC_THREADS, smem, stream>>>(ma, mb, out, rows_a, rows_b, K, ld_out, kb_per_split, err);
    return launch_status();
}

template <int BN, bool TRANSPOSE>
static int tc_dispatch(const CUtensorMap& ma, const CUtensorMap& mb, void* out, int rows_a, int rows_b, int K,
                       long long ld_out, int omode, int splits, int kb_per_split, int* err, cudaStream_t s) {
    switch (omode) {
        case TC_OUT_BF16: return tc_launch<BN, TC_OUT_BF16, TRANSPOSE>(ma, mb, out, rows_a, rows_b, K, ld_out, splits, kb_per_split, err, s);
        case TC_OUT_F32: return tc_launch<BN, TC_OUT_F32, TRANSPOSE>(ma, mb, out, rows_a, rows_b, K, ld_out, splits, kb_per_split, err, s);
        case TC_OUT_ADD_F32: return tc_launch<BN, TC_OUT_ADD_F32, TRANSPOSE>(ma, mb, out, rows_a, rows_b, K, ld_out, splits, kb_per_split, err, s);
        default: return tc_launch<BN, TC_OUT_PARTIAL, TRANSPOSE>(ma, mb, out, rows_a, rows_b, K, ld_out, splits, kb_per_split, err, s);
    }
}

// out[M, N] (row-major, leading dimension N) = x[M, K] . w[N, K]^T.
//   transpose == 0: x is the A operand (rows on the 128-wide axis): prefill, many rows.
//   transpose == 1: w is the A operand and x the B operand (M <= 256 rows padded to a
//                   multiple of 16): decode, few rows; the tile is stored transposed.
// omode: 0 bfloat16, 1 float32, 2 add into float32. splits > 1: K is cut; `workspace` must
// hold splits * M * N floats. err: one int on the device that a timed-out wait sets.
TGO_API int tgo_gemm_tc(const void* x, const void* w, void* out, int M, int N, int K, int omode,
                        int transpose, int splits, float* workspace, int* err, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || omode < 0 || omode > 2 || splits < 1 || (splits > 1 && !workspace) ||
        ((uintptr_t)x & 15) || ((uintptr_t)w & 15))
        return TGO_E_BAD_ARG;
    const int kb_total = (K + TC_BK - 1) / TC_BK;
    if (splits > kb_total) splits = kb_total;
    const int kb_per_split = (kb_total + splits - 1) / splits;
    splits = (kb_total + kb_per_split - 1) / kb_per_split;
    const int om = splits > 1 ? TC_OUT_PARTIAL : omode;
    void* dst = splits > 1 ? (void*)workspace : out;
    CUtensorMap ma, mb;
    int rc;
    if (!transpose) {
        const int bn = N >= 256 ? 256 : 128;
        if ((rc = make_map(&ma, x, M, K, TC_BM))) return rc;
        if ((rc = make_map(&mb, w, N, K, bn))) return rc;
        rc = bn == 256 ? tc_dispatch<256, false>(ma, mb, dst, M, N, K, N, om, splits, kb_per_split, err, stream)
                       : tc_dispatch<128, false>(ma, mb, dst, M, N, K, N, om, splits, kb_per_split, err, stream);
    } else {
        if (M > 256) return TGO_E_BAD_ARG;
        const int bn = M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
        if ((rc = make_map(&ma, w, N, K, TC_BM))) return rc;
        if ((rc = make_map(&mb, x, M, K, bn))) return rc;
        // A = w (N rows), B = x (M rows); D^T is stored: out[m, n], leading dimension N
        switch (bn) {
            case 32: rc = tc_dispatch<32, true>(ma, mb, dst, N, M, K, N, om, splits, kb_per_split, err, stream); break;
            case 64: rc = tc_dispatch<64, true>(ma, mb, dst, N, M, K, N, om, splits, kb_per_split, err, stream); break;
            case 128: rc = tc_dispatch<128, true>(ma, mb, dst, N, M, K, N, om, splits, kb_per_split, err, stream); break;
            default: rc = tc_dispatch<256, true>(ma, mb, dst, N, M, K, N, om, splits, kb_per_split, err, stream); break;
        }
    }
    if (rc || splits == 1) return rc;
    const long long n = (long long)M * N;
    const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    if (omode == TC_OUT_BF16) gemm_tc_reduce_kernel<TC_OUT_BF16><<<blocks, 256, 0, stream>>>(workspace, out, n, splits);
    else if (omode == TC_OUT_F32) gemm_tc_reduce_kernel<TC_OUT_F32><<<blocks, 256, 0, stream>>>(workspace, out, n, splits);
    else gemm_tc_reduce_kernel<TC_OUT_ADD_F32><<<blocks, 256, 0, stream>>>(workspace, out, n, splits);
    return launch_status();
}
