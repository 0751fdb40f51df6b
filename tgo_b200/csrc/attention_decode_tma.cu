// Decode attention (one token per request) with the cache pages brought in by TMA: the same
// arithmetic as flash_decode_kernel (attention_flash.cu: mma.sync m16n8k16, the G query heads
// of a kv head as the rows of one m16 tile, 64 keys a tile, four warps with 16 keys each,
// float32 softmax state, partial results per key split for flash_combine_kernel), for head
// size 128 and pages of 8, 16, 32 or 64 tokens. What changes is who moves the data: a fifth
// warp asks the tensor memory accelerator for the pages of the next tiles (two boxes of
// page_size rows x 64 columns per page and per K / V, 128-byte swizzle) into a ring of two
// stages with an mbarrier each, so the four computing warps issue no copies and no addresses
// for them: that kernel is bound by instruction issue, not by the bandwidth it asks for.
//
// Rows of a tile that no query may read (past the request's last key, before its window) are
// not masked in V by the copy as cp.async's zero fill did: the warp that owns such keys
// writes zeros over its V rows before it multiplies (P is zero there, the cache may hold NaN).
//
// Fused form (DtFuse): the kernel also does what a kernel before it did for a decode step: it
// takes the raw q rows, norms and rotates them into shared memory itself, and the one CTA of a
// (token, kv head) whose keys include the token's own position norms and rotates the new k,
// writes it and the new v to their row of the cache, and lays both over that row of the tile
// that TMA brought (a stale row of the page). The arithmetic is that of
// qk_norm_rope_cache_dh128_kernel, operation for operation, so both ways give the same bits.
//
// Every mbarrier wait has a time limit (about two seconds), after which a flag is set and the
// CTA runs to its end without waiting again.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "mma_sync.cuh"

#define DT_BN 64
#define DT_DH 128
#ifndef DT_STAGES
#define DT_STAGES 2
#endif
#ifndef DT_MIN_BLOCKS
#define DT_MIN_BLOCKS 3
#endif
#define DT_HALF_BYTES (DT_BN * 128)            // 64 keys x 64 columns of bf16
#define DT_TILE_BYTES (2 * DT_HALF_BYTES)      // K or V of one tile
#define DT_STAGE_BYTES (2 * DT_TILE_BYTES)     // K and V
#define DT_THREADS 160
#define DT_PAGES_CAP 1024
#ifndef DT_KEYS_ON_M_MAX_GROUP
#define DT_KEYS_ON_M_MAX_GROUP 8      // up to this many query heads a kv head: the keys take the M axis
#endif
#define DT_WAIT_CYCLES 4000000000ll

__device__ int dt_error_flag = 0;

__device__ __forceinline__ bool dt_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool dt_wait(uint32_t bar, uint32_t parity) {
    if (dt_try(bar, parity)) return true;
    const long long start = clock64();
    while (!dt_try(bar, parity)) {
        if (clock64() - start > DT_WAIT_CYCLES) {
            atomicExch(&dt_error_flag, 1);
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ void dt_tma(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// byte offset of 16-byte piece `c` (0..15) of row `r` in a tile of two swizzled halves
__device__ __forceinline__ uint32_t dt_at(int r, int c) {
    return (uint32_t)((c >> 3) * DT_HALF_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4));
}

struct DtFuse {
    const bf16* k_new;          // this step's raw k rows [T, k_stride] and v rows, by token
    long long k_stride;
    const bf16* v_new;
    long long v_stride;
    const float* q_gain;        // per-head RMSNorm gains [128], or null for no norm
    const float* k_gain;
    float eps;
    const float* rope;          // [T, 128]: 64 cosines then 64 sines of each token, or null
    const int* slots;           // cache row (page * page_size + offset) of each token; < 0: none
    bf16* k_cache;              // null: not fused, q comes normed and rotated, the cache written
    bf16* v_cache;
};

// One head vector of 128 channels by a warp, lane l holding channels 4l .. 4l+3: RMSNorm with
// `gain` (if given), then the half-split rotation by the token's cosines and sines (if given),
// the partner channel i +- 64 sitting 16 lanes away. Returns the four values as bfloat16.
__device__ __forceinline__ uint2 dt_norm_rope(const bf16* __restrict__ vec, const float* __restrict__ gain,
                                              float eps, const float* __restrict__ cs, int lane) {
    const uint2 raw = *(const uint2*)(vec + 4 * lane);
    const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&raw.x);
    const float2 b = __bfloat1622float2(*(const __nv_bfloat162*)&raw.y);
    float x[4] = {a.x, a.y, b.x, b.y};
    if (gain) {
        float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
        ss = warp_sum(ss);
        const float scale = rsqrtf(ss / 128.f + eps);
        const float4 g = *(const float4*)(gain + 4 * lane);
        x[0] = (x[0] * scale) * g.x; x[1] = (x[1] * scale) * g.y;
        x[2] = (x[2] * scale) * g.z; x[3] = (x[3] * scale) * g.w;
    }
    if (cs) {
        const int i0 = 4 * (lane & 15);
        const float4 c = *(const float4*)(cs + i0), sn = *(const float4*)(cs + 64 + i0);
        const float cc[4] = {c.x, c.y, c.z, c.w}, sv[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float other = __shfl_xor_sync(0xffffffffu, x[e], 16);
            x[e] = lane < 16 ? x[e] * cc[e] - other * sv[e] : other * sv[e] + x[e] * cc[e];
        }
    }
    const __nv_bfloat162 lo = __floats2bfloat162_rn(x[0], x[1]), hi = __floats2bfloat162_rn(x[2], x[3]);
    uint2 out;
    out.x = *(const uint32_t*)&lo;
    out.y = *(const uint32_t*)&hi;
    return out;
}

template <bool KEYS_ON_M>
__global__ void __launch_bounds__(DT_THREADS, DT_MIN_BLOCKS)
flash_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out,
                        long long out_stride, int page_size, int page_shift,
                        const int* __restrict__ block_tables, int max_blocks,
                        const int* __restrict__ positions, const int* __restrict__ seq_ids, int H,
                        int Hkv, float scale_log2, int window, int n_splits,
                        float* __restrict__ part_o, float* __restrict__ part_ml,
                        const int* __restrict__ tok_list, const DtFuse fz) {
    constexpr int DH = DT_DH, KS = DH / 16, CH = DH / 8, LDQ = DH + 8;
    extern __shared__ unsigned char dt_raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)dt_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* ring = base;                                      // [stage][K | V][2 halves][64][128 B]
    uint64_t* bars = (uint64_t*)(ring + DT_STAGES * DT_STAGE_BYTES); // K full[S], empty[S], V full[S]
    bf16* sq = (bf16*)(bars + 3 * DT_STAGES);                        // [16][LDQ]
    float* s_ml = (float*)(sq + 16 * LDQ);                           // [4][16][2]
    int* s_pages = (int*)(s_ml + 4 * 16 * 2);                        // [DT_PAGES_CAP]
    pdl_wait();

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // the tokens of the step this launch takes: all of them, or those a list names (the
    // single tokens of a step that also holds prompt portions); partial results are kept by
    // place in the list
    const int slot = blockIdx.x;
    const int tok = tok_list ? tok_list[slot] : slot, kvh = blockIdx.y, split = blockIdx.z;
    const int G = H / Hkv;
    const int p = positions[tok];
    if (p < 0) {                               // a request that brings nothing: zeros out
        if (split == 0)
            for (int i = tid; i < G * DH; i += DT_THREADS)
                out[(size_t)tok * out_stride + (size_t)(kvh * G) * DH + i] = __float2bfloat16_rn(0.f);
        if (n_splits > 1)
            for (int r = tid; r < G; r += DT_THREADS) {
                const size_t at = ((size_t)slot * H + kvh * G + r) * n_splits + split;
                part_ml[at * 2] = -INFINITY;
                part_ml[at * 2 + 1] = 0.f;
            }
        return;
    }
    const int* bt = block_tables + (size_t)seq_ids[tok] * max_blocks;
    const int key_lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int key_hi = p + 1;
    const int t_first = key_lo / DT_BN, t_end = (key_hi + DT_BN - 1) / DT_BN;
    int t_lo = t_first, t_hi = t_end;
    if (n_splits > 1) {
        const int per = (t_end - t_first + n_splits - 1) / n_splits;
        t_lo = t_first + split * per;
        t_hi = t_lo + per < t_end ? t_lo + per : t_end;
    }
    const int n_it = t_hi > t_lo ? t_hi - t_lo : 0;
    const int pages_per_tile = DT_BN >> page_shift;
    const int pg_lo = t_lo * pages_per_tile;
    {
        int pg_hi = t_hi * pages_per_tile;
        if (pg_hi > max_blocks) pg_hi = max_blocks;
        if (pg_hi - pg_lo > DT_PAGES_CAP) pg_hi = pg_lo + DT_PAGES_CAP;
        for (int i = pg_lo + tid; i < pg_hi; i += DT_THREADS) s_pages[i - pg_lo] = bt[i];
    }
    if (tid == 0) {
        for (int s = 0; s < DT_STAGES; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bars[s])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 4;" ::"r"(smem_u32(&bars[DT_STAGES + s])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bars[2 * DT_STAGES + s])));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();          // the pages and the barriers are there: the producer may start
    // fused form: the iteration and the warp that hold the token's own key, and its new row
    int it_own = -1, warp_own = -1;
    uint2 k_own = make_uint2(0u, 0u), v_own = make_uint2(0u, 0u);
    // The four computing warps stage q (and in the fused form make it) while the fifth already
    // asks for the first tiles; they meet at a barrier of their own.
    if (warp == 4) {
    } else if (fz.k_cache) {
        const float* cs = fz.rope ? fz.rope + (size_t)tok * DH : nullptr;
        if (warp < 4) {
            for (int r = warp; r < 16; r += 4) {
                uint2 row = make_uint2(0u, 0u);
                if (r < G)
                    row = dt_norm_rope(q + (size_t)tok * q_stride + (size_t)(kvh * G + r) * DH, fz.q_gain,
                                       fz.eps, cs, lane);
                *(uint2*)(sq + r * LDQ + 4 * lane) = row;
            }
            if (n_it > 0 && p >= t_lo * DT_BN && p < t_hi * DT_BN) {
                it_own = p / DT_BN - t_lo;
                warp_own = (p & (DT_BN - 1)) >> 4;
                if (warp == warp_own) {
                    k_own = dt_norm_rope(fz.k_new + (size_t)tok * fz.k_stride + (size_t)kvh * DH, fz.k_gain,
                                         fz.eps, cs, lane);
                    v_own = *(const uint2*)(fz.v_new + (size_t)tok * fz.v_stride + (size_t)kvh * DH + 4 * lane);
                    const int row = fz.slots[tok];
                    if (row >= 0) {
                        const int page = row >> page_shift, off = row - (page << page_shift);
                        const size_t at = (((size_t)page * Hkv + kvh) * page_size + off) * DH + 4 * lane;
                        *(uint2*)(fz.k_cache + at) = k_own;
                        *(uint2*)(fz.v_cache + at) = v_own;
                    }
                }
            }
        }
    } else {
        for (int i = tid; i < 16 * CH; i += 128) {
            const int r = i / CH, c = i % CH;
            const bool ok = r < G;
            cp_async16(sq + r * LDQ + c * 8,
                       ok ? q + (size_t)tok * q_stride + (size_t)(kvh * G + r) * DH + c * 8 : q, ok);
        }
        cp_async_commit();
        cp_async_wait<0>();
    }
    if (warp < 4) asm volatile("bar.sync 1, 128;" ::: "memory");
    // the token's own key and value over the row of the tile that the copy brought
    auto lay_own = [&](uint32_t tile, uint2 row) {
        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(tile + dt_at(p & (DT_BN - 1), lane >> 1) + (lane & 1) * 8),
                     "r"(row.x), "r"(row.y) : "memory");
        __syncwarp();
    };

    if (warp == 4) {
        // ------------------------------------------------------------- producer
        auto page_of = [&](int pi) { return pi - pg_lo < DT_PAGES_CAP ? s_pages[pi - pg_lo] : bt[pi]; };
        bool ok = true;
        for (int it = 0; it < n_it; ++it) {
            const int s = it % DT_STAGES;
            const uint32_t ph = (uint32_t)(it / DT_STAGES) & 1u;
            const int j = t_lo + it;
            int first = j * pages_per_tile, last = first + pages_per_tile;      // pages with a readable key
            while (first < last && (first + 1) * page_size <= key_lo) ++first;
            while (last > first && (last - 1) * page_size >= key_hi) --last;
            ok = __all_sync(0xffffffffu, ok && dt_wait(smem_u32(&bars[DT_STAGES + s]), ph ^ 1u));
            if (!ok) break;
            // K and V of a tile have a barrier each: Q K^T starts when K is there
            const uint32_t k_full = smem_u32(&bars[s]), v_full = smem_u32(&bars[2 * DT_STAGES + s]);
            if (lane == 0) {
                const uint32_t bytes = (uint32_t)(last - first) * (uint32_t)page_size * 256u;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(k_full), "r"(bytes) : "memory");
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(v_full), "r"(bytes) : "memory");
            }
            __syncwarp();
            for (int pi = first + lane; pi < last; pi += 32) {
                const int row = (page_of(pi) * Hkv + kvh) * page_size;
                const uint32_t dst = smem_u32(ring + s * DT_STAGE_BYTES) + (uint32_t)((pi - j * pages_per_tile) * page_size * 128);
                dt_tma(dst, &map_k, 0, row, k_full);
                dt_tma(dst + DT_HALF_BYTES, &map_k, 64, row, k_full);
            }
            for (int pi = first + lane; pi < last; pi += 32) {
                const int row = (page_of(pi) * Hkv + kvh) * page_size;
                const uint32_t dst = smem_u32(ring + s * DT_STAGE_BYTES) + (uint32_t)((pi - j * pages_per_tile) * page_size * 128);
                dt_tma(dst + DT_TILE_BYTES, &map_v, 0, row, v_full);
                dt_tma(dst + DT_TILE_BYTES + DT_HALF_BYTES, &map_v, 64, row, v_full);
            }
        }
        // the producer takes no part in the sums below, but in the barriers
    }

    // Two forms of the arithmetic. With at most 8 query heads a kv head the keys take the M
    // axis of the products and the heads the N axis (S^T = K Q^T, O^T += V^T P^T): a 16-key
    // tile of a warp costs 8 + 8 products, 4 exponentials a lane and 32 accumulators to
    // rescale, where the heads on the M axis (up to 16 of them) cost twice that with three
    // quarters of the rows empty for a group of four.
    float o[KEYS_ON_M ? DH / 16 : DH / 8][4];
#pragma unroll
    for (int i = 0; i < (KEYS_ON_M ? DH / 16 : DH / 8); ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;      // KEYS_ON_M: heads 2t and 2t+1
    const int r_lo = lane >> 2, r_hi = r_lo + 8;
    const bool row_lo_ok = r_lo < G, row_hi_ok = r_hi < G;

    if constexpr (KEYS_ON_M) {
      if (warp < 4) {
        const int g = lane >> 2, t = lane & 3;
        const bool q0_ok = 2 * t < G, q1_ok = 2 * t + 1 < G;
        // Q^T as the B operand: for k-steps 2j and 2j+1, b0 and b1 of each
        uint32_t qb[KS / 2][4];
#pragma unroll
        for (int j = 0; j < KS / 2; ++j)
            ldmatrix_x4(qb[j], sq + (lane & 7) * LDQ + j * 32 + (lane >> 3) * 8);
        bool ok = true;
        for (int it = 0; it < n_it; ++it) {
            const int s = it % DT_STAGES;
            const uint32_t ph = (uint32_t)(it / DT_STAGES) & 1u;
            const int tile = t_lo + it;
            if (ok) ok = dt_wait(smem_u32(&bars[s]), ph);           // K
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const uint32_t kt = smem_u32(ring + s * DT_STAGE_BYTES);
            const uint32_t vt = kt + DT_TILE_BYTES;
            const int my_key0 = tile * DT_BN + warp * 16;
            if (it == it_own && warp == warp_own) lay_own(kt, k_own);
            float sc[4] = {0.f, 0.f, 0.f, 0.f};       // keys g, g+8 x heads 2t, 2t+1
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t ka[4];
                const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = ks * 2 + (lane >> 4);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(ka[0]), "=r"(ka[1]), "=r"(ka[2]), "=r"(ka[3]) : "r"(kt + dt_at(r, c)));
                mma_bf16(sc, ka, qb[ks >> 1][(ks & 1) * 2], qb[ks >> 1][(ks & 1) * 2 + 1]);
            }
            const int key_a = my_key0 + g, key_b = key_a + 8;
            const bool vis_a = key_a >= key_lo && key_a < key_hi, vis_b = key_b >= key_lo && key_b < key_hi;
            sc[0] = (vis_a && q0_ok) ? sc[0] * scale_log2 : -INFINITY;
            sc[1] = (vis_a && q1_ok) ? sc[1] * scale_log2 : -INFINITY;
            sc[2] = (vis_b && q0_ok) ? sc[2] * scale_log2 : -INFINITY;
            sc[3] = (vis_b && q1_ok) ? sc[3] * scale_log2 : -INFINITY;
            float mx0 = fmaxf(sc[0], sc[2]), mx1 = fmaxf(sc[1], sc[3]);
#pragma unroll
            for (int off = 4; off <= 16; off <<= 1) {             // over the keys: lanes of equal t
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
            }
            const float mn0 = fmaxf(m_lo, mx0), mn1 = fmaxf(m_hi, mx1);
            const float base0 = mn0 == -INFINITY ? 0.f : mn0, base1 = mn1 == -INFINITY ? 0.f : mn1;
            const float corr0 = exp2f(m_lo - base0), corr1 = exp2f(m_hi - base1);
            m_lo = mn0;
            m_hi = mn1;
            sc[0] = exp2f(sc[0] - base0); sc[1] = exp2f(sc[1] - base1);
            sc[2] = exp2f(sc[2] - base0); sc[3] = exp2f(sc[3] - base1);
            l_lo = l_lo * corr0 + sc[0] + sc[2];
            l_hi = l_hi * corr1 + sc[1] + sc[3];
            if (ok) ok = dt_wait(smem_u32(&bars[2 * DT_STAGES + s]), ph);        // V
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (it == it_own && warp == warp_own) lay_own(vt, v_own);
            if (my_key0 + 16 > key_hi || my_key0 < key_lo) {       // V rows nobody may read: zeros
                for (int i = lane; i < 16 * 16; i += 32) {
                    const int r = i >> 4, c = i & 15;
                    const int key = my_key0 + r;
                    if (key >= key_hi || key < key_lo)
                        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(vt + dt_at(warp * 16 + r, c)), "r"(0u) : "memory");
                }
                __syncwarp();
            }
            // P^T as the B operand: the two 8 x 8 blocks (keys x heads) transposed
            uint32_t pb0, pb1;
            {
                const uint32_t blk_a = pack_bf16(sc[0], sc[1]), blk_b = pack_bf16(sc[2], sc[3]);
                asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(pb0) : "r"(blk_a));
                asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(pb1) : "r"(blk_b));
            }
#pragma unroll
            for (int dt = 0; dt < DH / 16; ++dt) {
                uint32_t va[4];
                const int r = warp * 16 + (lane & 7) + (lane >> 4) * 8, c = dt * 2 + ((lane >> 3) & 1);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(va[0]), "=r"(va[1]), "=r"(va[2]), "=r"(va[3]) : "r"(vt + dt_at(r, c)));
                o[dt][0] *= corr0; o[dt][1] *= corr1; o[dt][2] *= corr0; o[dt][3] *= corr1;
                mma_bf16(o[dt], va, pb0, pb1);
            }
            __syncwarp();                      // every lane has read the stage
            if (lane == 0)
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&bars[DT_STAGES + s])) : "memory");
        }
      }
    } else {
    if (warp < 4) {
        uint32_t qa[KS][4];
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
            ldmatrix_x4(qa[ks], sq + ((lane & 7) + ((lane >> 3) & 1) * 8) * LDQ + ks * 16 + (lane >> 4) * 8);
        bool ok = true;
        for (int it = 0; it < n_it; ++it) {
            const int s = it % DT_STAGES;
            const uint32_t ph = (uint32_t)(it / DT_STAGES) & 1u;
            const int t = t_lo + it;
            if (ok) ok = dt_wait(smem_u32(&bars[s]), ph) && dt_wait(smem_u32(&bars[2 * DT_STAGES + s]), ph);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const uint32_t kt = smem_u32(ring + s * DT_STAGE_BYTES);
            const uint32_t vt = kt + DT_TILE_BYTES;
            const int my_key0 = t * DT_BN + warp * 16;
            if (it == it_own && warp == warp_own) {
                lay_own(kt, k_own);
                lay_own(vt, v_own);
            }
            // this warp's V rows that nobody may read: zeros (P is zero there; the page may hold anything)
            if (my_key0 + 16 > key_hi || my_key0 < key_lo) {
                for (int i = lane; i < 16 * 16; i += 32) {
                    const int r = i >> 4, c = i & 15;
                    const int key = my_key0 + r;
                    if (key >= key_hi || key < key_lo)
                        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(vt + dt_at(warp * 16 + r, c)), "r"(0u) : "memory");
                }
                __syncwarp();
            }
            float sc[2][4];
            sc[0][0] = sc[0][1] = sc[0][2] = sc[0][3] = 0.f;
            sc[1][0] = sc[1][1] = sc[1][2] = sc[1][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t kb[4];
                const int r = warp * 16 + (lane & 7) + (lane >> 4) * 8, c = ks * 2 + ((lane >> 3) & 1);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(kb[0]), "=r"(kb[1]), "=r"(kb[2]), "=r"(kb[3]) : "r"(kt + dt_at(r, c)));
                mma_bf16(sc[0], qa[ks], kb[0], kb[1]);
                mma_bf16(sc[1], qa[ks], kb[2], kb[3]);
            }
            const int kbase = my_key0 + (lane & 3) * 2;
            float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = kbase + i * 8 + e;
                    const bool vis = j >= key_lo && j < key_hi;
                    sc[i][e] = (vis && row_lo_ok) ? sc[i][e] * scale_log2 : -INFINITY;
                    sc[i][2 + e] = (vis && row_hi_ok) ? sc[i][2 + e] * scale_log2 : -INFINITY;
                    mx_lo = fmaxf(mx_lo, sc[i][e]);
                    mx_hi = fmaxf(mx_hi, sc[i][2 + e]);
                }
            }
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
            const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
            const float base_lo = mn_lo == -INFINITY ? 0.f : mn_lo;
            const float base_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
            const float corr_lo = exp2f(m_lo - base_lo), corr_hi = exp2f(m_hi - base_hi);
            m_lo = mn_lo;
            m_hi = mn_hi;
            float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                sc[i][0] = exp2f(sc[i][0] - base_lo);
                sc[i][1] = exp2f(sc[i][1] - base_lo);
                sc[i][2] = exp2f(sc[i][2] - base_hi);
                sc[i][3] = exp2f(sc[i][3] - base_hi);
                sum_lo += sc[i][0] + sc[i][1];
                sum_hi += sc[i][2] + sc[i][3];
            }
            l_lo = l_lo * corr_lo + sum_lo;
            l_hi = l_hi * corr_hi + sum_hi;
            uint32_t pa[4];
            pa[0] = pack_bf16(sc[0][0], sc[0][1]);
            pa[1] = pack_bf16(sc[0][2], sc[0][3]);
            pa[2] = pack_bf16(sc[1][0], sc[1][1]);
            pa[3] = pack_bf16(sc[1][2], sc[1][3]);
#pragma unroll
            for (int dp = 0; dp < DH / 16; ++dp) {
                uint32_t vb[4];
                const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = dp * 2 + (lane >> 4);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(vb[0]), "=r"(vb[1]), "=r"(vb[2]), "=r"(vb[3]) : "r"(vt + dt_at(r, c)));
                o[2 * dp][0] *= corr_lo; o[2 * dp][1] *= corr_lo;
                o[2 * dp][2] *= corr_hi; o[2 * dp][3] *= corr_hi;
                o[2 * dp + 1][0] *= corr_lo; o[2 * dp + 1][1] *= corr_lo;
                o[2 * dp + 1][2] *= corr_hi; o[2 * dp + 1][3] *= corr_hi;
                mma_bf16(o[2 * dp], pa, vb[0], vb[1]);
                mma_bf16(o[2 * dp + 1], pa, vb[2], vb[3]);
            }
            __syncwarp();                      // every lane has read the stage
            if (lane == 0)
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&bars[DT_STAGES + s])) : "memory");
        }
    }
    }
    __syncthreads();                           // all tiles read: the ring is free for the join
    pdl_launch_late();
    float* so = (float*)ring;                  // [4][16][DH]
    if constexpr (KEYS_ON_M) {
      if (warp < 4) {
        const int g = lane >> 2, t = lane & 3;
#pragma unroll
        for (int off = 4; off <= 16; off <<= 1) {
            l_lo += __shfl_xor_sync(0xffffffffu, l_lo, off);
            l_hi += __shfl_xor_sync(0xffffffffu, l_hi, off);
        }
        // O^T: lane (g, t) holds rows dt*16 + g (+8) of heads 2t and 2t+1
#pragma unroll
        for (int dt = 0; dt < DH / 16; ++dt) {
            so[((size_t)warp * 16 + 2 * t) * DH + dt * 16 + g] = o[dt][0];
            so[((size_t)warp * 16 + 2 * t + 1) * DH + dt * 16 + g] = o[dt][1];
            so[((size_t)warp * 16 + 2 * t) * DH + dt * 16 + g + 8] = o[dt][2];
            so[((size_t)warp * 16 + 2 * t + 1) * DH + dt * 16 + g + 8] = o[dt][3];
        }
        if (g == 0) {
            s_ml[(warp * 16 + 2 * t) * 2] = m_lo; s_ml[(warp * 16 + 2 * t) * 2 + 1] = l_lo;
            s_ml[(warp * 16 + 2 * t + 1) * 2] = m_hi; s_ml[(warp * 16 + 2 * t + 1) * 2 + 1] = l_hi;
        }
      }
    } else {
    if (warp < 4) {
        l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
        l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
        l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
        l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
        const int col = (lane & 3) * 2;
#pragma unroll
        for (int i = 0; i < DH / 8; ++i) {
            *(float2*)(so + ((size_t)warp * 16 + r_lo) * DH + i * 8 + col) = make_float2(o[i][0], o[i][1]);
            *(float2*)(so + ((size_t)warp * 16 + r_hi) * DH + i * 8 + col) = make_float2(o[i][2], o[i][3]);
        }
        if ((lane & 3) == 0) {
            s_ml[(warp * 16 + r_lo) * 2] = m_lo; s_ml[(warp * 16 + r_lo) * 2 + 1] = l_lo;
            s_ml[(warp * 16 + r_hi) * 2] = m_hi; s_ml[(warp * 16 + r_hi) * 2 + 1] = l_hi;
        }
    }
    }
    __syncthreads();
    for (int i = tid; i < G * DH; i += DT_THREADS) {
        const int r = i / DH, d = i % DH;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, s_ml[(w * 16 + r) * 2]);
        float l = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = s_ml[(w * 16 + r) * 2];
            if (mw != -INFINITY) {
                const float f = exp2f(mw - m);
                l += s_ml[(w * 16 + r) * 2 + 1] * f;
                acc += so[((size_t)w * 16 + r) * DH + d] * f;
            }
        }
        const int head = kvh * G + r;
        if (n_splits == 1) {
            out[(size_t)tok * out_stride + (size_t)head * DH + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
        } else {
            const size_t at = ((size_t)slot * H + head) * n_splits + split;
            part_o[at * DH + d] = acc;
            if (d == 0) { part_ml[at * 2] = m; part_ml[at * 2 + 1] = l; }
        }
    }
}

// ------------------------------------------------------------------------------ host
typedef CUresult (*DtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                               CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                               CUtensorMapFloatOOBfill);

// The tensor map of one layer's K or V pages, [rows, 128] bf16 in boxes of page_size x 64;
// made once per (address, rows, page size) and kept.
static const CUtensorMap* dt_map_of(const void* pages, long long rows, int page_size) {
    static std::mutex lock;
    static std::unordered_map<uint64_t, CUtensorMap> maps;
    static DtEncodeFn encode = nullptr;
    std::lock_guard<std::mutex> hold(lock);
    if (!encode) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) != cudaSuccess ||
            qr != cudaDriverEntryPointSuccess)
            return nullptr;
        encode = (DtEncodeFn)p;
    }
    const uint64_t key = (uint64_t)(uintptr_t)pages ^ ((uint64_t)rows * 0x9e3779b97f4a7c15ull) ^ ((uint64_t)page_size << 56);
    auto it = maps.find(key);
    if (it != maps.end()) return &it->second;
    CUtensorMap map;
    const cuuint64_t dims[2] = {DT_DH, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {DT_DH * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)page_size};
    const cuuint32_t elem[2] = {1, 1};
    if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return nullptr;
    return &maps.emplace(key, map).first->second;
}

// 1 if this kernel takes the shape: head size 128, at most 16 query heads a kv head, pages of
// 8, 16, 32 or 64 tokens.
TGO_API int tgo_attention_decode_tma_supports(int dh, int group, int page_size) {
    return dh == DT_DH && group >= 1 && group <= 16 &&
           (page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64);
}

// Reads (and waits for the device to reach) the flag a wait that ran out sets; 0: none did.
TGO_API int tgo_attention_decode_tma_error(int* value) {
    return (int)cudaMemcpyFromSymbol(value, dt_error_flag, sizeof(int));
}

// tok_list: null, or T indices into the step's tokens: those are taken instead of 0 .. T-1
// (q, out, positions and seq_ids are indexed by them; the partial results by 0 .. T-1).
// One token per request (token t is request seq_ids[t] at positions[t]); n_splits CTAs per
// (token, kv head) write partial results to part_o [T, H, n_splits, 128] and part_ml
// [T, H, n_splits, 2] for flash_combine_kernel when n_splits > 1.
static int dt_launch(const void* q, long long q_stride, void* out, long long out_stride,
                     const void* k_cache, const void* v_cache, int n_pages, int page_size,
                     const int* block_tables, int max_blocks, const int* positions,
                     const int* seq_ids, int T, int H, int Hkv, int dh, float scale,
                     int window, int n_splits, float* part_o, float* part_ml,
                     const int* tok_list, const DtFuse& fz, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || H % Hkv || !tgo_attention_decode_tma_supports(dh, H / Hkv, page_size) ||
        n_pages <= 0 || max_blocks <= 0 || window < 0 || n_splits < 1 || n_splits > 65535 || Hkv > 65535 ||
        (n_splits > 1 && (!part_o || !part_ml)) || q_stride % 8 || ((uintptr_t)q % 16) ||
        ((uintptr_t)k_cache % 128) || ((uintptr_t)v_cache % 128))
        return TGO_E_BAD_ARG;
    const long long rows = (long long)n_pages * Hkv * page_size;
    if (rows > 0x7fffffffll) return TGO_E_BAD_ARG;
    const CUtensorMap* mk = dt_map_of(k_cache, rows, page_size);
    const CUtensorMap* mv = dt_map_of(v_cache, rows, page_size);
    if (!mk || !mv) return TGO_E_BAD_ARG;
    constexpr size_t ring = (size_t)DT_STAGES * DT_STAGE_BYTES;
    static_assert(ring >= (size_t)4 * 16 * DT_DH * sizeof(float), "the join of the four warps reuses the ring");
    constexpr size_t smem = 1024 + ring + 3 * DT_STAGES * 8 + 16 * (DT_DH + 8) * sizeof(bf16) +
                            4 * 16 * 2 * sizeof(float) + DT_PAGES_CAP * sizeof(int);
    static bool once = false;
    if (!once) {
        cudaError_t e = cudaFuncSetAttribute(flash_decode_tma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(flash_decode_tma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        once = true;
    }
    int shift = 0;
    while ((1 << shift) < page_size) ++shift;
    if (H / Hkv <= DT_KEYS_ON_M_MAX_GROUP)
        return tgo_launch_pdl(flash_decode_tma_kernel<true>, dim3(T, Hkv, n_splits), dim3(DT_THREADS), smem, stream,
                              *mk, *mv, (const bf16*)q, q_stride, (bf16*)out, out_stride, page_size, shift,
                              block_tables, max_blocks, positions, seq_ids, H, Hkv, scale * 1.4426950408889634f,
                              window, n_splits, part_o, part_ml, tok_list, fz);
    return tgo_launch_pdl(flash_decode_tma_kernel<false>, dim3(T, Hkv, n_splits), dim3(DT_THREADS), smem, stream,
                          *mk, *mv, (const bf16*)q, q_stride, (bf16*)out, out_stride, page_size, shift,
                          block_tables, max_blocks, positions, seq_ids, H, Hkv, scale * 1.4426950408889634f,
                          window, n_splits, part_o, part_ml, tok_list, fz);
}

TGO_API int tgo_attention_decode_tma(const void* q, long long q_stride, void* out, long long out_stride,
                                     const void* k_cache, const void* v_cache, int n_pages, int page_size,
                                     const int* block_tables, int max_blocks, const int* positions,
                                     const int* seq_ids, int T, int H, int Hkv, int dh, float scale,
                                     int window, int n_splits, float* part_o, float* part_ml,
                                     const int* tok_list, cudaStream_t stream) {
    DtFuse none = {};
    return dt_launch(q, q_stride, out, out_stride, k_cache, v_cache, n_pages, page_size, block_tables,
                     max_blocks, positions, seq_ids, T, H, Hkv, dh, scale, window, n_splits, part_o,
                     part_ml, tok_list, none, stream);
}

// The fused form: q holds the raw query rows of the step's T tokens (every token, no list);
// k_new and v_new their raw key and value rows; the kernel norms (gains of 128 floats, or
// null for none) and rotates (rope [T, 128], cosines then sines, or null) q and k, writes k and
// v to the cache rows slots[t], and attends over the cache including that row.
TGO_API int tgo_attention_decode_tma_fused(const void* q, long long q_stride, void* out, long long out_stride,
                                           void* k_cache, void* v_cache, int n_pages, int page_size,
                                           const int* block_tables, int max_blocks, const int* positions,
                                           const int* seq_ids, int T, int H, int Hkv, int dh, float scale,
                                           int window, int n_splits, float* part_o, float* part_ml,
                                           const void* k_new, long long k_stride, const void* v_new,
                                           long long v_stride, const float* q_gain, const float* k_gain,
                                           float eps, const float* rope, const int* slots,
                                           cudaStream_t stream) {
    if (!k_new || !v_new || !slots || !k_cache || !v_cache || k_stride % 4 || v_stride % 4 ||
        ((uintptr_t)k_new % 8) || ((uintptr_t)v_new % 8) || q_stride % 4 || ((uintptr_t)q % 8) ||
        (q_gain && (uintptr_t)q_gain % 16) || (k_gain && (uintptr_t)k_gain % 16) ||
        (rope && (uintptr_t)rope % 16))
        return TGO_E_BAD_ARG;
    DtFuse fz;
    fz.k_new = (const bf16*)k_new; fz.k_stride = k_stride;
    fz.v_new = (const bf16*)v_new; fz.v_stride = v_stride;
    fz.q_gain = q_gain; fz.k_gain = k_gain; fz.eps = eps;
    fz.rope = rope; fz.slots = slots;
    fz.k_cache = (bf16*)k_cache; fz.v_cache = (bf16*)v_cache;
    return dt_launch(q, q_stride, out, out_stride, k_cache, v_cache, n_pages, page_size, block_tables,
                     max_blocks, positions, seq_ids, T, H, Hkv, dh, scale, window, n_splits, part_o,
                     part_ml, nullptr, fz, stream);
}
