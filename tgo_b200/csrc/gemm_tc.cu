// D = A . B^T on the 5th-generation tensor cores: bfloat16 operands, both K-major (row-major
// with K contiguous, as activations [rows, K] and checkpoint weights [out, K] are), float32
// accumulation in tensor memory.
//
// One CTA computes one 128 x BN tile of D at a time (BN, the tile's width, is a run-time
// argument: a multiple of 16 up to 256, chosen by the host per product). Six warps, three
// roles:
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
// (The decode orientation, weights as A and a few activation rows as B with D stored
// transposed, was built and measured for 9 to 64 rows: 104-124 us a layer of the 8B shape
// against the library's 80-83, with K splits and a reduce kernel 3-8 % behind it in the
// running model. It is not kept.)
//
// A second form of the kernel (DUAL) gives a CTA 256 rows: two accumulators fed by two A
// tiles and one shared B tile per k-block, and four more epilogue warps. Per product it
// brings a third fewer operand bytes into the SM, which is what bounds a 128 x 256 tile.
//
// The last round. CTAs walk whole tiles in rounds of gridDim.x; what is left for the last,
// partial round (or all there is, when there are fewer tiles than SMs) is cut along K over
// the CTAs that would otherwise idle (`tail_splits` > 1): split 0 of a tile keeps its part in
// its accumulator; the others write theirs as float32 into a workspace and count up the
// tile's flag; split 0 waits for the count (with a time limit), adds the parts in split
// order while it reads its accumulator, stores the tile and sets the flag back to zero. No
// CTA waits before its own products are done, so the wait needs no co-residency. One
// workspace per device: products of one device must not run at the same time.
//
// Tails: TMA fills out-of-range rows and K with zeros; stores are guarded. K % 8 == 0.
// No cluster, no multicast. Every mbarrier wait gives up after about two seconds, records
// where in *err and lets the CTA run to its end (TMEM is freed on every path).
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192
#define TC_GROUP_M 16
#define TC_WAIT_CYCLES 4000000000ll

#define TC_OUT_BF16 0
#define TC_OUT_F32 1
#define TC_OUT_ADD_F32 2
#define TC_OUT_SWIGLU 4       // silu(gate) * up of a gate/up matrix interleaved in eights, bfloat16

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

// Shared and tensor memory of a CTA for tiles `bn` wide (a value at run time: the host picks
// the width that wastes the least of the GPU for the shape at hand).
#define TC_A_BYTES (TC_BM * TC_BK * 2)
#define TC_RING_BYTES (200 * 1024)
#define TC_STAGE_OUT_BYTES 2048            // per epilogue warp: 32 rows x 64 bytes of output on their way out
#define TC_SMEM_TOTAL ((size_t)TC_RING_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + 8 * TC_STAGE_OUT_BYTES)
__host__ __device__ __forceinline__ int tc_stage_bytes(int bn, bool dual = false) {
    return (dual ? 2 : 1) * TC_A_BYTES + bn * TC_BK * 2;
}
__host__ __device__ __forceinline__ int tc_stages(int bn, bool dual = false) {
    const int n = TC_RING_BYTES / tc_stage_bytes(bn, dual);
    return n < 8 ? n : 8;
}
// columns of tensor memory per accumulator: a power of two (an allocation has to be)
__host__ __device__ __forceinline__ int tc_acc_cols(int bn) { return bn <= 32 ? 32 : bn <= 64 ? 64 : bn <= 128 ? 128 : 256; }

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc_smem(bar)) : "memory");
}
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float silu_mul(float g, float u) {
    g = bf16_round(g);      // as when the product is stored before the gate is applied
    u = bf16_round(u);
    // 2^x and 1/x of the special-function unit (relative error about 2^-22; the result is
    // rounded to bfloat16): the library routines cost ten times the instructions, and a
    // 256 x 224 tile has 28672 of these
    return __fdividef(g, 1.f + __expf(-g)) * u;
}

__device__ __forceinline__ void tc_tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
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
}
__device__ __forceinline__ void tc_tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t tc_pack(uint32_t lo, uint32_t hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(lo), __uint_as_float(hi));
    return *(uint32_t*)&v;
}

// A warp's 32 rows x 64 bytes of bfloat16 output (each lane holds its row's four 16-byte
// pieces) -> memory through the warp's staging buffer, so that a store instruction writes 8
// rows x 64 contiguous bytes instead of 32 rows x 16: a quarter of the cache lines per
// instruction. (Each thread storing its own row, a 256 x 192 tile took 5.8 us to leave, a
// seventh of the tile's time, with the tensor core idle: measured with the global timer.)
// dst: the warp's first row at the pieces' first column; rows_ok rows of the warp exist.
__device__ __forceinline__ void tc_store_staged(unsigned char* stage, const uint4 (&v)[4], bf16* dst,
                                                long long ld_out, int rows_ok, int lane) {
    const uint32_t sbase = tc_smem(stage);
    const int swz = (lane >> 1) & 3;
#pragma unroll
    for (int q = 0; q < 4; ++q)
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(sbase + (uint32_t)(lane * 64 + ((q ^ swz) << 4))),
                     "r"(v[q].x), "r"(v[q].y), "r"(v[q].z), "r"(v[q].w) : "memory");
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int e = i * 32 + lane, row = e >> 2, q = e & 3;
        uint4 x;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(x.x), "=r"(x.y), "=r"(x.z), "=r"(x.w)
                     : "r"(sbase + (uint32_t)(row * 64 + ((q ^ ((row >> 1) & 3)) << 4))) : "memory");
        if (row < rows_ok) *(uint4*)(dst + (size_t)row * ld_out + q * 8) = x;
    }
    __syncwarp();
}

// One thread's 32 consecutive accumulator columns (row `gm` of A, rows gn0.. of B) -> memory.
template <int OMODE>
__device__ __forceinline__ void tc_store(const uint32_t (&r)[32], void* __restrict__ out, int gm, int gn0,
                                         int rows_a, int rows_b, long long ld_out) {
    if (OMODE == TC_OUT_SWIGLU) {
        // columns come as 8 gate, 8 up, 8 gate, 8 up: 16 outputs at column gn0 / 2
        if (gm >= rows_a) return;
        bf16* dst = (bf16*)out + (size_t)gm * ld_out + gn0 / 2;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if (gn0 + 16 * h + 16 > rows_b) break;
            uint32_t pk[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float a = silu_mul(__uint_as_float(r[16 * h + 2 * j]), __uint_as_float(r[16 * h + 8 + 2 * j]));
                const float b = silu_mul(__uint_as_float(r[16 * h + 2 * j + 1]), __uint_as_float(r[16 * h + 9 + 2 * j]));
                __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
                pk[j] = *(uint32_t*)&v;
            }
            if ((ld_out & 7) == 0) *(uint4*)(dst + 8 * h) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            else
#pragma unroll
                for (int j = 0; j < 4; ++j) *(uint32_t*)(dst + 8 * h + 2 * j) = pk[j];
        }
        return;
    }
    if (gm >= rows_a) return;
    if (gn0 + 32 <= rows_b && (ld_out & 7) == 0) {
        if (OMODE == TC_OUT_BF16) {
            uint4* dst = (uint4*)((bf16*)out + (size_t)gm * ld_out + gn0);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                uint4 pk;
                __nv_bfloat162 h;
                h = __floats2bfloat162_rn(__uint_as_float(r[8 * v]), __uint_as_float(r[8 * v + 1]));
                pk.x = *(uint32_t*)&h;
                h = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
                pk.y = *(uint32_t*)&h;
                h = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
                pk.z = *(uint32_t*)&h;
                h = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
                pk.w = *(uint32_t*)&h;
                dst[v] = pk;
            }
        } else {
            float4* dst = (float4*)((float*)out + (size_t)gm * ld_out + gn0);
#pragma unroll
            for (int v = 0; v < 8; ++v) {
                float4 x = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                       __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                if (OMODE == TC_OUT_ADD_F32) {
                    const float4 y = dst[v];
                    x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w;
                }
                dst[v] = x;
            }
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const int gn = gn0 + j;
        if (gn >= rows_b) break;
        const float v = __uint_as_float(r[j]);
        const size_t at = (size_t)gm * ld_out + gn;
        if (OMODE == TC_OUT_BF16) ((bf16*)out)[at] = __float2bfloat16_rn(v);
        else if (OMODE == TC_OUT_ADD_F32) ((float*)out)[at] += v;
        else ((float*)out)[at] = v;
    }
}

// Persistent: the grid is at most one CTA per SM and each CTA walks tiles blockIdx.x,
// blockIdx.x + gridDim.x, ... The accumulator is double-buffered in TMEM (2 x BN columns), so
// the epilogue of one tile runs while the next tile's products are issued.
template <int OMODE, bool DUAL>
__global__ void __launch_bounds__(DUAL ? TC_THREADS + 128 : TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               void* __restrict__ out, int rows_a, int rows_b, int K, long long ld_out,
               int* __restrict__ err, int BN, int tail_splits,
               float* __restrict__ tail_ws, int* __restrict__ tail_flags) {
    // DUAL: a CTA's tile is 256 rows, two 128-row halves that share every B tile in shared
    // memory (a third fewer operand bytes per product: one SM cannot be fed the 48 KB that a
    // 128 x 256 tile wants every 512 tensor cycles); the two accumulators fill the 512
    // columns of tensor memory, so the next tile waits for the epilogue of this one, which
    // two warpgroups run, one per half.
    constexpr int ROWS = DUAL ? 2 * TC_BM : TC_BM;
    const int STAGES = tc_stages(BN, DUAL), STAGE = tc_stage_bytes(BN, DUAL);
    const int ACC_COLS = tc_acc_cols(BN), TMEM_COLS = DUAL ? 512 : 2 * ACC_COLS;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(base + TC_RING_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;       // [2]
    uint64_t* acc_empty = acc_full + 2;        // [2]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    unsigned char* stage_out = base + TC_RING_BYTES + 256;      // [8 epilogue warps][TC_STAGE_OUT_BYTES]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Tile order: the A-row tiles of one group of TC_GROUP_M run first over a B tile, so the
    // CTAs that are resident together share B tiles (and a small set of A tiles) in L2 instead
    // of streaming all of B once per row of tiles.
    const int tiles_m = (rows_a + ROWS - 1) / ROWS;
    const int tiles_n = (rows_b + BN - 1) / BN;
    const int n_tiles = tiles_m * tiles_n;
    const int per_group = TC_GROUP_M * tiles_n;
    const int kb_total = (K + TC_BK - 1) / TC_BK;
    // whole tiles in full rounds, then the tiles of the last round cut tail_splits ways
    const int whole = tail_splits > 1 ? n_tiles / (int)gridDim.x * (int)gridDim.x : n_tiles;
    const int n_tail = n_tiles - whole;
    const int total = tail_splits > 1 ? whole + n_tail * tail_splits : n_tiles;
    constexpr int EPI_WARPS = DUAL ? 8 : 4;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], DUAL ? 8 : 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(tc_smem(tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // work item w -> (split, m0, n0, k-block range)
    // tail: -1, or which tile of the last round this is, `split` then being its part of K
    auto locate = [&](int w, int& split, int& m0, int& n0, int& kb_lo, int& n_kb, int& tail) {
        int tile, kb_hi;
        if (tail_splits > 1 && w >= whole) {
            tail = (w - whole) % n_tail;
            split = (w - whole) / n_tail;
            tile = whole + tail;
            kb_lo = (int)((long long)split * kb_total / tail_splits);
            kb_hi = (int)((long long)(split + 1) * kb_total / tail_splits);
        } else {
            tail = -1;
            split = 0;
            tile = w;
            kb_lo = 0;
            kb_hi = kb_total;
        }
        const int group = tile / per_group, within = tile % per_group;
        const int group_m = tiles_m - group * TC_GROUP_M < TC_GROUP_M ? tiles_m - group * TC_GROUP_M : TC_GROUP_M;
        m0 = (group * TC_GROUP_M + within % group_m) * ROWS;
        n0 = (within / group_m) * BN;
        n_kb = kb_hi > kb_lo ? kb_hi - kb_lo : 0;
    };

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;                                    // stage uses so far, over all tiles
            bool ok = true;
            for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
                int split, m0, n0, kb_lo, n_kb, tail;
                locate(w, split, m0, n0, kb_lo, n_kb, tail);
                for (int i = 0; i < n_kb; ++i, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, err, 1);
                    if (!ok) break;
                    mbar_expect_tx(&full[s], (uint32_t)STAGE);
                    unsigned char* st = base + (size_t)s * STAGE;
                    const int kb = kb_lo + i;
                    tma_load_2d(st, &map_a, kb * TC_BK, m0, &full[s]);
                    if (DUAL) tma_load_2d(st + TC_A_BYTES, &map_a, kb * TC_BK, m0 + TC_BM, &full[s]);
                    tma_load_2d(st + (DUAL ? 2 : 1) * TC_A_BYTES, &map_b, kb * TC_BK, n0, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: float32 accumulate, bf16 x bf16, both K-major, N, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                   ((uint32_t)(TC_BM >> 4) << 24);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total && ok; w += gridDim.x, ++local) {
                int split, m0, n0, kb_lo, n_kb, tail;
                locate(w, split, m0, n0, kb_lo, n_kb, tail);
                // two accumulators in turn, or (DUAL) the one pair there is
                const uint32_t buf = DUAL ? 0u : (local & 1);
                const uint32_t use = DUAL ? local : (local >> 1);
                ok = mbar_wait(&acc_empty[buf], (use & 1) ^ 1, err, 4);   // epilogue let go of it
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * ACC_COLS;
                for (int i = 0; i < n_kb; ++i, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(&full[s], (it / STAGES) & 1, err, 2);
                    if (!ok) break;
                    tc_fence_after();
                    unsigned char* st = base + (size_t)s * STAGE;
                    const uint64_t da = umma_desc(st), db = umma_desc(st + (DUAL ? 2 : 1) * TC_A_BYTES);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k) {  // 16 bf16 = 32 bytes = 2 descriptor units
                        umma_bf16(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                                  (i > 0 || k > 0) ? 1u : 0u);
                        if (DUAL)       // the lower 128 rows: the next A tile, accumulator columns 256..
                            umma_bf16(d_tmem + 256u, da + (uint64_t)(TC_A_BYTES >> 4) + (uint64_t)(2 * k),
                                      db + (uint64_t)(2 * k), idesc, (i > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty[s]);
                }
                umma_commit(&acc_full[buf]);    // arrives once every MMA issued above has finished
            }
        }
    } else {
        const int quarter = warp & 3;                           // TMEM lanes this warp may read
        const int half = DUAL ? (warp - 2) >> 2 : 0;            // DUAL: warps 2-5 the upper rows, 6-9 the lower
        const int row = half * TC_BM + quarter * 32 + lane;     // row of the tile (TMEM lane, + 128)
        uint32_t local = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < total; w += gridDim.x, ++local) {
            int split, m0, n0, kb_lo, n_kb, tail;
            locate(w, split, m0, n0, kb_lo, n_kb, tail);
            const uint32_t buf = DUAL ? 0u : (local & 1);
            const uint32_t use = DUAL ? local : (local >> 1);
            if (ok) ok = mbar_wait(&acc_full[buf], use & 1, err, 3);
            tc_fence_after();
            const bool gathers = tail >= 0 && split == 0, gives = tail >= 0 && split > 0;
            if (gathers && ok) {
                // every epilogue warp of the tile's other parts has counted up
                int seen = 0;
                if (lane == 0) {
                    const int want = (tail_splits - 1) * EPI_WARPS;
                    const long long start = clock64();
                    for (;;) {
                        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(tail_flags + tail) : "memory");
                        if (seen >= want) break;
                        if (clock64() - start > TC_WAIT_CYCLES) {
                            if (err) atomicExch(err, 5);
                            seen = -1;
                            break;
                        }
                    }
                }
                ok = __shfl_sync(0xffffffffu, seen, 0) >= 0;
            }
            // a part of a tile: [tile of the last round][part - 1][group of 4 columns][row] as
            // float4, so that the 32 lanes of a warp (32 rows) write and read 512 bytes in a row
            float4* part = tail < 0 ? nullptr : (float4*)tail_ws + ((size_t)tail * (tail_splits - 1)) * ROWS * (BN / 4) + row;
            // a tile that is not a multiple of 32 wide: its last group of columns is cut at the
            // tile's edge (what lies beyond belongs to the next tile)
            const int n_edge = n0 + BN < rows_b ? n0 + BN : rows_b;
            const uint32_t tacc = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * ACC_COLS + (uint32_t)(half * 256);
            // The usual tile (whole, bfloat16 or gated output, rows of the output 16-byte
            // aligned): the loads from tensor memory run one group of columns ahead of the
            // stores, and the stores go through the warp's staging buffer. MEASURED (global
            // timer, 2048 rows of the 8B shapes): a 256 x 192 tile's way out 5.8 -> 3.1 us of
            // its 42, a gated 256 x 224 tile's 9.8 -> 6.0 us of its 48 (a 256-row tile fills
            // tensor memory, so the tensor core idles meanwhile, and every SM writes its tile
            // at the same moment: 14 MB at once). Tried and not kept: copying the whole slice
            // out of tensor memory into registers (rounded to bfloat16: up to 128 registers a
            // thread), giving tensor memory back at once and storing while the next tile runs;
            // the kernel then spills (its ten warps get 168 registers each, and with three
            // warpgroups and setmaxnreg the compiler spilled more), and was slower: q/k/v
            // 92.8 us against 85.9, gate/up 320 against 285.
            if ((OMODE == TC_OUT_BF16 || OMODE == TC_OUT_SWIGLU) && tail < 0 && (ld_out & 7) == 0 && ok && n_kb > 0) {
                unsigned char* stage = stage_out + (warp - 2) * TC_STAGE_OUT_BYTES;
                const int row0 = m0 + half * TC_BM + quarter * 32;             // the warp's first row
                const int rows_ok = rows_a - row0 < 32 ? rows_a - row0 : 32;   // may be <= 0
                const int n_chunks = (BN + 31) / 32;
                uint32_t ra[32], rb[32];
                if (OMODE == TC_OUT_BF16) {
                    tc_tmem_ld32(tacc, ra);
#pragma unroll 1
                    for (int c = 0; c < n_chunks; c += 2) {
                        tc_tmem_wait_ld();
                        if (c + 1 < n_chunks) tc_tmem_ld32(tacc + (uint32_t)((c + 1) * 32), rb);
                        {
                            const int gn0 = n0 + c * 32;
                            if (gn0 + 32 <= n_edge) {
                                uint4 v[4];
#pragma unroll
                                for (int q = 0; q < 4; ++q)
                                    v[q] = make_uint4(tc_pack(ra[8 * q], ra[8 * q + 1]), tc_pack(ra[8 * q + 2], ra[8 * q + 3]),
                                                      tc_pack(ra[8 * q + 4], ra[8 * q + 5]), tc_pack(ra[8 * q + 6], ra[8 * q + 7]));
                                tc_store_staged(stage, v, (bf16*)out + (size_t)row0 * ld_out + gn0, ld_out, rows_ok, lane);
                            } else {
                                tc_store<OMODE>(ra, out, m0 + row, gn0, rows_a, n_edge, ld_out);
                            }
                        }
                        if (c + 1 < n_chunks) {
                            tc_tmem_wait_ld();
                            if (c + 2 < n_chunks) tc_tmem_ld32(tacc + (uint32_t)((c + 2) * 32), ra);
                            const int gn0 = n0 + (c + 1) * 32;
                            if (gn0 + 32 <= n_edge) {
                                uint4 v[4];
#pragma unroll
                                for (int q = 0; q < 4; ++q)
                                    v[q] = make_uint4(tc_pack(rb[8 * q], rb[8 * q + 1]), tc_pack(rb[8 * q + 2], rb[8 * q + 3]),
                                                      tc_pack(rb[8 * q + 4], rb[8 * q + 5]), tc_pack(rb[8 * q + 6], rb[8 * q + 7]));
                                tc_store_staged(stage, v, (bf16*)out + (size_t)row0 * ld_out + gn0, ld_out, rows_ok, lane);
                            } else {
                                tc_store<OMODE>(rb, out, m0 + row, gn0, rows_a, n_edge, ld_out);
                            }
                        }
                    }
                } else {
                    // gated: two groups of 32 accumulator columns (8 gate, 8 up, ...) make 32
                    // outputs, 64 bytes a row; the next two groups are loaded while these leave
                    tc_tmem_ld32(tacc, ra);
                    if (n_chunks > 1) tc_tmem_ld32(tacc + 32u, rb);
#pragma unroll 1
                    for (int c = 0; c < n_chunks; c += 2) {
                        tc_tmem_wait_ld();
                        const int gn0 = n0 + c * 32;
                        const bool pair = c + 1 < n_chunks && gn0 + 64 <= n_edge;
                        uint4 v[4];
                        if (pair) {
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                uint32_t pk[4];
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const float a = silu_mul(__uint_as_float(ra[16 * h + 2 * j]), __uint_as_float(ra[16 * h + 8 + 2 * j]));
                                    const float b = silu_mul(__uint_as_float(ra[16 * h + 2 * j + 1]), __uint_as_float(ra[16 * h + 9 + 2 * j]));
                                    __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
                                    pk[j] = *(uint32_t*)&t;
                                }
                                v[h] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                            }
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                uint32_t pk[4];
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const float a = silu_mul(__uint_as_float(rb[16 * h + 2 * j]), __uint_as_float(rb[16 * h + 8 + 2 * j]));
                                    const float b = silu_mul(__uint_as_float(rb[16 * h + 2 * j + 1]), __uint_as_float(rb[16 * h + 9 + 2 * j]));
                                    __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
                                    pk[j] = *(uint32_t*)&t;
                                }
                                v[2 + h] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                            }
                        } else {
                            tc_store<OMODE>(ra, out, m0 + row, gn0, rows_a, n_edge, ld_out);
                            if (c + 1 < n_chunks) tc_store<OMODE>(rb, out, m0 + row, gn0 + 32, rows_a, n_edge, ld_out);
                        }
                        if (c + 2 < n_chunks) tc_tmem_ld32(tacc + (uint32_t)((c + 2) * 32), ra);
                        if (c + 3 < n_chunks) tc_tmem_ld32(tacc + (uint32_t)((c + 3) * 32), rb);
                        if (pair)
                            tc_store_staged(stage, v, (bf16*)out + (size_t)row0 * ld_out + gn0 / 2, ld_out, rows_ok, lane);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[buf]);
                continue;
            }
#pragma unroll 1
            for (int c = 0; c < (BN + 31) / 32; ++c) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * ACC_COLS + (uint32_t)(half * 256) + (uint32_t)(c * 32);
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
                const int cols = BN - c * 32 < 32 ? BN - c * 32 : 32;        // 32 or 16
                if (gives) {
                    float4* dst = part + ((size_t)(split - 1) * (BN / 4) + c * 8) * ROWS;
#pragma unroll
                    for (int v = 0; v < 8; ++v)
                        if (4 * v < cols)
                            dst[(size_t)v * ROWS] = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                                 __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                    continue;
                }
                if (gathers && ok) {
                    for (int p = 0; p < tail_splits - 1; ++p) {
                        const float4* src = part + ((size_t)p * (BN / 4) + c * 8) * ROWS;
#pragma unroll
                        for (int v = 0; v < 8; ++v)
                            if (4 * v < cols) {
                                const float4 y = __ldcg(src + (size_t)v * ROWS);    // written by another SM: not through L1
                                r[4 * v] = __float_as_uint(__uint_as_float(r[4 * v]) + y.x);
                                r[4 * v + 1] = __float_as_uint(__uint_as_float(r[4 * v + 1]) + y.y);
                                r[4 * v + 2] = __float_as_uint(__uint_as_float(r[4 * v + 2]) + y.z);
                                r[4 * v + 3] = __float_as_uint(__uint_as_float(r[4 * v + 3]) + y.w);
                            }
                    }
                }
                if (ok && n_kb > 0)
                    tc_store<OMODE>(r, out, m0 + row, n0 + c * 32, rows_a, n_edge, ld_out);
            }
            // the accumulator may be overwritten: one arrival per epilogue warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
            if (gives) {
                // this warp's rows of the part are written: make them visible, then count
                __threadfence();
                __syncwarp();
                if (lane == 0) atomicAdd(tail_flags + tail, 1);
            }
            if (gathers) {
                // all epilogue warps have seen the count: the flag goes back to zero for the
                // next launch
                asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory");
                if (warp == 2 && lane == 0) tail_flags[tail] = 0;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
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

// A [rows, K] bf16 row-major -> tiles of box_rows x 64 with the 128-byte swizzle. Maps are kept
// by (address, shape, box): a weight's map is made once, and activations come back to the same
// addresses step after step (a map describes memory, not its contents).
static int make_map_uncached(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows);
static int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
    struct Key {
        const void* ptr; int rows, K, box;
        bool operator==(const Key& o) const { return ptr == o.ptr && rows == o.rows && K == o.K && box == o.box; }
    };
    struct Hash {
        size_t operator()(const Key& k) const {
            return (size_t)(uintptr_t)k.ptr * 0x9e3779b97f4a7c15ull ^ ((size_t)k.rows << 40) ^ ((size_t)k.K << 16) ^ (size_t)k.box;
        }
    };
    static std::mutex lock;
    static std::unordered_map<Key, CUtensorMap, Hash> maps;
    std::lock_guard<std::mutex> hold(lock);
    const Key key{ptr, rows, K, box_rows};
    auto it = maps.find(key);
    if (it != maps.end()) { *map = it->second; return 0; }
    const int rc = make_map_uncached(map, ptr, rows, K, box_rows);
    if (rc) return rc;
    if (maps.size() > 8192) maps.clear();
    maps.emplace(key, *map);
    return 0;
}
static int make_map_uncached(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
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

static int tc_sms() {
    int dev = 0;
    static int cached[64] = {};
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) {
        if (!cached[dev]) cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev);
        if (cached[dev] > 0) return cached[dev];
    }
    return 148;
}

template <int OMODE, bool DUAL>
static int tc_launch(int BN, const CUtensorMap& ma, const CUtensorMap& mb, void* out, int rows_a, int rows_b, int K,
                     long long ld_out, int* err, cudaStream_t stream, int tail_splits, float* tail_ws,
                     int* tail_flags) {
    auto kern = gemm_tc_kernel<OMODE, DUAL>;
    const size_t smem = TC_SMEM_TOTAL;
    static bool sized = false;            // per instance of this template
    if (!sized) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        sized = true;
    }
    const int total = ((rows_b + BN - 1) / BN) * ((rows_a + (DUAL ? 2 : 1) * TC_BM - 1) / ((DUAL ? 2 : 1) * TC_BM));
    const int sms = tc_sms();
    // with a cut last round the kernel derives the rounds from the grid: it has to be `sms`
    const dim3 grid(tail_splits > 1 ? sms : total < sms ? total : sms);
    kern<<<grid, DUAL ? TC_THREADS + 128 : TC_THREADS, smem, stream>>>(ma, mb, out, rows_a, rows_b, K, ld_out, err, BN,
                                                                       tail_splits, tail_ws, tail_flags);
    return launch_status();
}

template <bool DUAL>
static int tc_dispatch(int BN, const CUtensorMap& ma, const CUtensorMap& mb, void* out, int rows_a, int rows_b, int K,
                       long long ld_out, int omode, int* err, cudaStream_t s, int tail_splits, float* tail_ws,
                       int* tail_flags) {
#define TC_CASE(mode) \
    return tc_launch<mode, DUAL>(BN, ma, mb, out, rows_a, rows_b, K, ld_out, err, s, tail_splits, tail_ws, tail_flags)
    switch (omode) {
        case TC_OUT_BF16: TC_CASE(TC_OUT_BF16);
        case TC_OUT_F32: TC_CASE(TC_OUT_F32);
        case TC_OUT_ADD_F32: TC_CASE(TC_OUT_ADD_F32);
        default: TC_CASE(TC_OUT_SWIGLU);
    }
#undef TC_CASE
}

// For tests and tuning: the tile of the product is rows x width instead of
// the cost model's choice (rows 128 or 256; 0 gives the choice back). The width has to be
// one the instruction takes with 128 rows: a multiple of 16 from 16 to 256. tail: 0 leaves
// the cut of the last round to the shape, 1 forbids it. Not for use while other threads
// launch products.
static int g_forced_rows = 0, g_forced_width = 0, g_forced_tail = 0;
TGO_API int tgo_gemm_tc_force_tile(int rows, int width, int tail) {
    g_forced_tail = tail;
    if (rows == 0) { g_forced_rows = g_forced_width = 0; return 0; }
    if ((rows != 128 && rows != 256) || width < 16 || width > 256 || width % 16)
        return TGO_E_BAD_ARG;
    g_forced_rows = rows;
    g_forced_width = width;
    return 0;
}

// What the last product of this process ran as (one thread at a time launches products): rows and width of its tiles and the number
// of parts its last round's tiles were cut into.
static int g_last_rows = 0, g_last_width = 0, g_last_cut = 0;
TGO_API void tgo_gemm_tc_last_plan(int* rows, int* width, int* cut) {
    *rows = g_last_rows; *width = g_last_width; *cut = g_last_cut;
}

#define TC_TAIL_MIN_KB 8        // k-blocks a part of a cut tile has at least
// Floats of workspace and flags that a cut last round may use: every CTA but one writes a
// part of the largest tile.
TGO_API long long tgo_gemm_tc_tail_floats() { return (long long)(tc_sms() - 1) * 2 * TC_BM * 256; }
TGO_API int tgo_gemm_tc_tail_flags() { return tc_sms(); }

// How many ways the tiles of the last round are cut along K (1: not at all).
static int tc_tail_splits(long long tiles, int kb_total, int sms) {
    const int left = (int)(tiles % sms);
    if (!left) return 1;
    int s = sms / left;
    if (s > kb_total / TC_TAIL_MIN_KB) s = kb_total / TC_TAIL_MIN_KB;
    return s < 2 ? 1 : s;
}

// out[M, N] (row-major, leading dimension N) = x[M, K] . w[N, K]^T; x is the A operand (its
// rows on the 128-wide axis): prompt portions, many rows.
// omode: 0 bfloat16, 1 float32, 2 add into float32, 4 w is a gate/up matrix with rows
// interleaved in eights and out is silu(gate) * up, bfloat16 [M, N / 2].
// tail_ws, tail_flags: tgo_gemm_tc_tail_floats() floats and tgo_gemm_tc_tail_flags() zeroed
// ints of this device for the cut of the last round; without them the last round is not cut.
// The kernel leaves the flags zero. One product at a time per device may use them.
// err: one int on the device that a timed-out wait sets.
TGO_API int tgo_gemm_tc(const void* x, const void* w, void* out, int M, int N, int K, int omode,
                        float* tail_ws, int* tail_flags, int* err, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || omode < 0 || omode == 3 || omode > TC_OUT_SWIGLU ||
        (omode == TC_OUT_SWIGLU && N % 16) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15))
        return TGO_E_BAD_ARG;
    const long long ld = omode == TC_OUT_SWIGLU ? N / 2 : N;
    const int kb_total = (K + TC_BK - 1) / TC_BK;
    CUtensorMap ma, mb;
    int rc;
    // Tile shape. The CTAs walk the tiles in rounds, and a round lasts as long as a whole
    // tile however few tiles it has, unless it is the last and its tiles are cut along K.
    // A k-block of a tile costs the larger of its products (2 cycles a column for 128
    // rows) and of bringing its operands in (an SM is fed about 70 bytes a cycle:
    // measured, a 128 x 256 tile's 48 KB keep the tensor pipe at 73 %). A tile of 256
    // rows (two accumulators over one B tile) needs a third fewer bytes per product.
    // Among 128 or 256 rows and widths in multiples of 32 (the kernel takes multiples of
    // 16, but a sweep over twelve products of three model sizes at 512 to 4096 rows found
    // the widths between to cost as much as the next multiple of 32 or more), the
    // cheapest by this count wins.
    const int sms = tc_sms();
    const bool may_cut = tail_ws && tail_flags && g_forced_tail != 1;
    int bn = N >= 256 ? 256 : 128;
    bool dual = false;
    if (g_forced_rows) {
        bn = g_forced_width;
        dual = g_forced_rows == 256;
    } else if (N >= 256) {
        double best = -1.0;
        for (int rows = 128; rows <= 256; rows += 128) {
            if (rows == 256 && M <= 128) break;
            const long long tiles_m = (M + rows - 1) / rows;
            for (int width = 256; width >= 64; width -= 32) {
                const long long tiles = tiles_m * ((N + width - 1) / width);
                const double math = 2.0 * width * (rows / 128);
                const double feed = ((rows / 128) * 16384.0 + 128.0 * width) / 70.0;
                const double per_kb = math > feed ? math : feed;
                // + the epilogue, which a 256-row tile cannot hide behind the next tile
                const double fixed = (rows == 256 ? 12.0 * width : 0.0) + 2000.0;
                const int cut = may_cut ? tc_tail_splits(tiles, kb_total, sms) : 1;
                double cost;
                if (cut > 1)        // + the parts' way through the workspace: written, waited for,
                                    // read (fitted to measured differences between cut and uncut)
                    cost = (double)(tiles / sms) * (per_kb * kb_total + fixed) +
                           per_kb * ((kb_total + cut - 1) / cut) + fixed + cut * rows * width * 4.0 / 35.0 + 8000.0;
                else
                    cost = (double)((tiles + sms - 1) / sms) * (per_kb * kb_total + fixed);
                if (best < 0 || cost < best) { best = cost; bn = width; dual = rows == 256; }
            }
        }
    }
    const long long tiles = (long long)((M + (dual ? 2 : 1) * TC_BM - 1) / ((dual ? 2 : 1) * TC_BM)) * ((N + bn - 1) / bn);
    const int cut = may_cut ? tc_tail_splits(tiles, kb_total, sms) : 1;
    g_last_rows = dual ? 256 : 128; g_last_width = bn; g_last_cut = cut;
    if ((rc = make_map(&ma, x, M, K, TC_BM))) return rc;
    if ((rc = make_map(&mb, w, N, K, bn))) return rc;
    return dual ? tc_dispatch<true>(bn, ma, mb, out, M, N, K, ld, omode, err, stream, cut, tail_ws, tail_flags)
                : tc_dispatch<false>(bn, ma, mb, out, M, N, K, ld, omode, err, stream, cut, tail_ws, tail_flags);
}
