// Paged causal attention on the tensor cores for bfloat16 storage, prefill and decode.
//
// One CTA takes a tile of query rows of one request and one kv head: the rows are the
// (token, query head of the group) pairs of up to 128/G consecutive tokens, G = H/Hkv,
// so every row of the tile reads the same keys and values. Keys and values come from the
// paged cache [page][kv_head][offset][DH] through the request's block table, 64 at a time,
// by cp.async into shared memory (two buffers: the next tile loads while this one is
// computed). S = Q K^T and O += P V are mma.sync m16n8k16 with float32 accumulators; the
// running maximum, the sum of exponentials and the rescaling are float32 in registers.
// A query at position p reads keys max(0, p - window + 1) .. p (window 0: from 0).
//
// Decode steps may cut each request's keys into `n_splits` ranges, one CTA each; the
// partial results (unnormalised O, maximum, sum) go to scratch and `flash_combine_kernel`
// joins them. Tiles are given by arrays (first token, token count) or, when those are
// null, tile t is the single token t (decode).
//
// mma.sync is the legacy tensor path on sm_100a; attention is a few percent of the
// model's flops, and this kernel is bound by the cache's bandwidth in decode.
#include "common.cuh"

#define FL_BN 64                 // keys per tile
#define FL_PAD 8                 // bf16 of padding per shared-memory row (keeps ldmatrix conflict-free)

#include "mma_sync.cuh"

#define FP_WARPS 4
#define FP_RW 2                  // m16 row tiles per warp
#define FP_BM (16 * FP_WARPS * FP_RW)

// Prefill: a tile of up to FP_BM query rows (consecutive tokens of one request x the G heads
// of one kv head). Each warp owns FP_RW m16 tiles, so every key and value fragment it loads
// from shared memory feeds FP_RW products.
template <int DH>
__global__ void __launch_bounds__(FP_WARPS * 32)
flash_prefill_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out,
                     long long out_stride, const bf16* __restrict__ k_cache,
                     const bf16* __restrict__ v_cache, int page_size, int page_shift,
                     const int* __restrict__ block_tables, int max_blocks,
                     const int* __restrict__ positions, const int* __restrict__ seq_ids,
                     const int* __restrict__ tile_tok0, const int* __restrict__ tile_ntok, int H,
                     int Hkv, float scale_log2, int window, int pages_cap) {
    constexpr int LD = DH + FL_PAD;            // shared-memory row stride in bf16
    constexpr int KS = DH / 16;                // k-steps of Q K^T
    constexpr int CH = DH / 8;                 // 16-byte chunks per row
    constexpr int THREADS = FP_WARPS * 32;
    constexpr int ROWS_PER_IT = THREADS / CH;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sq = (bf16*)smem_raw;                // [FP_BM][LD]
    bf16* sk = sq + FP_BM * LD;                // [2][FL_BN][LD]
    bf16* sv = sk + 2 * FL_BN * LD;            // [2][FL_BN][LD]
    int* s_pages = (int*)(sv + 2 * FL_BN * LD);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // later tiles of a request read more keys: they are started first, so that the kernel
    // does not end on a few long CTAs
    const int tile = gridDim.x - 1 - blockIdx.x, kvh = blockIdx.y;
    const int G = H / Hkv;
    const int tok0 = tile_tok0[tile], ntok = tile_ntok[tile];
    const int n_rows = ntok * G;
    const int p0 = positions[tok0];            // position of the tile's first token
    if (p0 < 0) {                              // a request that brings nothing: zeros out
        for (int i = tid; i < n_rows * DH; i += THREADS) {
            const int r = i / DH, d = i % DH;
            out[(size_t)(tok0 + r / G) * out_stride + (size_t)(kvh * G + r % G) * DH + d] =
                __float2bfloat16_rn(0.f);
        }
        return;
    }
    const int* bt = block_tables + (size_t)seq_ids[tok0] * max_blocks;
    const int p_last = p0 + ntok - 1;
    // keys any row of the tile may read: [key_lo, key_hi)
    const int key_lo = (window > 0 && p0 - window + 1 > 0) ? p0 - window + 1 : 0;
    const int key_hi = p_last + 1;
    const int t_lo = key_lo / FL_BN, t_hi = (key_hi + FL_BN - 1) / FL_BN;

    // the tile's slice of the block table -> shared memory
    const int pg_lo = (t_lo * FL_BN) / page_size;
    {
        int pg_hi = (t_hi * FL_BN + page_size - 1) / page_size;
        if (pg_hi > max_blocks) pg_hi = max_blocks;
        if (pg_hi - pg_lo > pages_cap) pg_hi = pg_lo + pages_cap;
        for (int i = pg_lo + tid; i < pg_hi; i += THREADS) s_pages[i - pg_lo] = bt[i];
    }
    for (int i = tid; i < FP_BM * CH; i += THREADS) {
        const int r = i / CH, c = i % CH;
        const bool ok = r < n_rows;
        const bf16* src = ok ? q + (size_t)(tok0 + r / G) * q_stride + (size_t)(kvh * G + r % G) * DH + c * 8 : q;
        cp_async16(sq + r * LD + c * 8, src, ok);
    }
    __syncthreads();
    auto page_of = [&](int pi) { return pi - pg_lo < pages_cap ? s_pages[pi - pg_lo] : bt[pi]; };
    const int c_mine = tid % CH, r_mine = tid / CH;
    auto load_kv = [&](int t, int buf) {
        bf16* dk = sk + buf * FL_BN * LD + c_mine * 8;
        bf16* dv = sv + buf * FL_BN * LD + c_mine * 8;
#pragma unroll
        for (int r = r_mine; r < FL_BN; r += ROWS_PER_IT) {
            const int j = t * FL_BN + r;
            const bool ok = j >= key_lo && j < key_hi;
            size_t off = 0;
            if (ok) {
                const int pi = page_shift >= 0 ? j >> page_shift : j / page_size;
                const int po = j - pi * page_size;
                off = (((size_t)page_of(pi) * Hkv + kvh) * page_size + po) * DH + c_mine * 8;
            }
            cp_async16(dk + r * LD, k_cache + off, ok);
            cp_async16(dv + r * LD, v_cache + off, ok);
        }
    };
    load_kv(t_lo, 0);
    cp_async_commit();

    float o[FP_RW][DH / 8][4];
    float m_run[FP_RW][2], l_run[FP_RW][2];
    int pos_row[FP_RW][2], vis_row[FP_RW][2];
#pragma unroll
    for (int rw = 0; rw < FP_RW; ++rw) {
#pragma unroll
        for (int i = 0; i < DH / 8; ++i) { o[rw][i][0] = o[rw][i][1] = o[rw][i][2] = o[rw][i][3] = 0.f; }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = (warp * FP_RW + rw) * 16 + (lane >> 2) + 8 * h;
            m_run[rw][h] = -INFINITY;
            l_run[rw][h] = 0.f;
            pos_row[rw][h] = r < n_rows ? p0 + r / G : -1;      // rows beyond the tile read nothing
            vis_row[rw][h] = (window > 0 && pos_row[rw][h] - window + 1 > 0) ? pos_row[rw][h] - window + 1 : 0;
        }
    }
    const bool warp_active = warp * FP_RW * 16 < n_rows;

    for (int t = t_lo; t < t_hi; ++t) {
        const int buf = (t - t_lo) & 1;
        if (t + 1 < t_hi) load_kv(t + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (warp_active) {
            const bf16* kt = sk + buf * FL_BN * LD;
            const bf16* vt = sv + buf * FL_BN * LD;
            float s[FP_RW][FL_BN / 8][4];
#pragma unroll
            for (int rw = 0; rw < FP_RW; ++rw)
#pragma unroll
                for (int i = 0; i < FL_BN / 8; ++i) { s[rw][i][0] = s[rw][i][1] = s[rw][i][2] = s[rw][i][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t qa[FP_RW][4];
#pragma unroll
                for (int rw = 0; rw < FP_RW; ++rw)
                    ldmatrix_x4(qa[rw], sq + ((warp * FP_RW + rw) * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD +
                                            ks * 16 + (lane >> 4) * 8);
#pragma unroll
                for (int np = 0; np < FL_BN / 16; ++np) {       // two n-tiles (16 keys) at a time
                    uint32_t kb[4];
                    ldmatrix_x4(kb, kt + (np * 16 + (lane & 7) + (lane >> 4) * 8) * LD + ks * 16 +
                                        ((lane >> 3) & 1) * 8);
#pragma unroll
                    for (int rw = 0; rw < FP_RW; ++rw) {
                        mma_bf16(s[rw][2 * np], qa[rw], kb[0], kb[1]);
                        mma_bf16(s[rw][2 * np + 1], qa[rw], kb[2], kb[3]);
                    }
                }
            }
            // a tile that lies wholly inside every row's range needs no mask
            const int first_row_pos = p0 + (warp * FP_RW * 16) / G;
            const bool full = (t + 1) * FL_BN - 1 <= first_row_pos && t * FL_BN >= key_lo &&
                              (window == 0 || t * FL_BN >= p_last - window + 1) &&
                              (warp * FP_RW + FP_RW) * 16 <= n_rows;
            const int kbase = t * FL_BN + (lane & 3) * 2;
            uint32_t pa[FP_RW][FL_BN / 16][4];
#pragma unroll
            for (int rw = 0; rw < FP_RW; ++rw) {
                float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int i = 0; i < FL_BN / 8; ++i) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int j = kbase + i * 8 + e;
                        const bool a = full || (j <= pos_row[rw][0] && j >= vis_row[rw][0]);
                        const bool c = full || (j <= pos_row[rw][1] && j >= vis_row[rw][1]);
                        s[rw][i][e] = a ? s[rw][i][e] * scale_log2 : -INFINITY;
                        s[rw][i][2 + e] = c ? s[rw][i][2 + e] * scale_log2 : -INFINITY;
                        mx[0] = fmaxf(mx[0], s[rw][i][e]);
                        mx[1] = fmaxf(mx[1], s[rw][i][2 + e]);
                    }
                }
                float corr[2], base[2], sum[2] = {0.f, 0.f};
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                    const float mn = fmaxf(m_run[rw][h], mx[h]);
                    // a row that has seen no key yet keeps base 0 so that exp2(-inf - 0) = 0
                    base[h] = mn == -INFINITY ? 0.f : mn;
                    corr[h] = exp2f(m_run[rw][h] - base[h]);
                    m_run[rw][h] = mn;
                }
#pragma unroll
                for (int i = 0; i < FL_BN / 8; ++i) {
                    s[rw][i][0] = exp2f(s[rw][i][0] - base[0]);
                    s[rw][i][1] = exp2f(s[rw][i][1] - base[0]);
                    s[rw][i][2] = exp2f(s[rw][i][2] - base[1]);
                    s[rw][i][3] = exp2f(s[rw][i][3] - base[1]);
                    sum[0] += s[rw][i][0] + s[rw][i][1];
                    sum[1] += s[rw][i][2] + s[rw][i][3];
                }
                l_run[rw][0] = l_run[rw][0] * corr[0] + sum[0];     // per-lane partial sums
                l_run[rw][1] = l_run[rw][1] * corr[1] + sum[1];
#pragma unroll
                for (int i = 0; i < DH / 8; ++i) {
                    o[rw][i][0] *= corr[0]; o[rw][i][1] *= corr[0];
                    o[rw][i][2] *= corr[1]; o[rw][i][3] *= corr[1];
                }
#pragma unroll
                for (int kk = 0; kk < FL_BN / 16; ++kk) {
                    pa[rw][kk][0] = pack_bf16(s[rw][2 * kk][0], s[rw][2 * kk][1]);
                    pa[rw][kk][1] = pack_bf16(s[rw][2 * kk][2], s[rw][2 * kk][3]);
                    pa[rw][kk][2] = pack_bf16(s[rw][2 * kk + 1][0], s[rw][2 * kk + 1][1]);
                    pa[rw][kk][3] = pack_bf16(s[rw][2 * kk + 1][2], s[rw][2 * kk + 1][3]);
                }
            }
            // O += P V
#pragma unroll
            for (int kk = 0; kk < FL_BN / 16; ++kk) {
#pragma unroll
                for (int dp = 0; dp < DH / 16; ++dp) {          // two n-tiles (16 dims) at a time
                    uint32_t vb[4];
                    ldmatrix_x4_trans(vb, vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD +
                                              dp * 16 + (lane >> 4) * 8);
#pragma unroll
                    for (int rw = 0; rw < FP_RW; ++rw) {
                        mma_bf16(o[rw][2 * dp], pa[rw][kk], vb[0], vb[1]);
                        mma_bf16(o[rw][2 * dp + 1], pa[rw][kk], vb[2], vb[3]);
                    }
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    if (!warp_active) return;
    const int col = (lane & 3) * 2;
#pragma unroll
    for (int rw = 0; rw < FP_RW; ++rw) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float l = l_run[rw][h];
            l += __shfl_xor_sync(0xffffffffu, l, 1);
            l += __shfl_xor_sync(0xffffffffu, l, 2);
            const int r = (warp * FP_RW + rw) * 16 + (lane >> 2) + 8 * h;
            if (r >= n_rows) continue;
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* dst = out + (size_t)(tok0 + r / G) * out_stride + (size_t)(kvh * G + r % G) * DH + col;
#pragma unroll
            for (int i = 0; i < DH / 8; ++i)
                *(uint32_t*)(dst + i * 8) = pack_bf16(o[rw][i][2 * h] * inv, o[rw][i][2 * h + 1] * inv);
        }
    }
}

// Decode: one token per request. The G query heads that share a kv head are the (up to 16)
// rows of one m16 tile, which all four warps hold; each 64-key tile is loaded by the whole
// CTA and warp w takes its keys 16w .. 16w+15, keeping its own maximum, sum and O. At the
// end the four partial states are joined through shared memory in warp order. With
// n_splits > 1 the CTA covers one range of the request's key tiles and writes a partial
// state for flash_combine_kernel. (Joining the splits inside this kernel, by letting the
// last CTA to finish do it, was measured slower than the separate small kernel.)
template <int DH>
__global__ void __launch_bounds__(128)
flash_decode_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out,
                    long long out_stride, const bf16* __restrict__ k_cache,
                    const bf16* __restrict__ v_cache, int page_size, int page_shift,
                    const int* __restrict__ block_tables, int max_blocks,
                    const int* __restrict__ positions, const int* __restrict__ seq_ids, int H,
                    int Hkv, float scale_log2, int window, int n_splits,
                    float* __restrict__ part_o, float* __restrict__ part_ml, int pages_cap) {
    constexpr int LD = DH + FL_PAD;
    constexpr int KS = DH / 16;
    constexpr int CH = DH / 8;
    constexpr int ROWS_PER_IT = 128 / CH;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sq = (bf16*)smem_raw;                // [16][LD]
    bf16* sk = sq + 16 * LD;                   // [2][64][LD]
    bf16* sv = sk + 2 * FL_BN * LD;            // [2][64][LD]
    __shared__ float s_ml[4][16][2];
    pdl_wait();

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tok = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int G = H / Hkv;
    const int p = positions[tok];
    if (p < 0) {                               // a request that brings nothing: zeros out
        if (split == 0)
            for (int i = tid; i < G * DH; i += 128)
                out[(size_t)tok * out_stride + (size_t)(kvh * G) * DH + i] = __float2bfloat16_rn(0.f);
        if (n_splits > 1)
            for (int r = tid; r < G; r += 128) {
                const size_t at = ((size_t)tok * H + kvh * G + r) * n_splits + split;
                part_ml[at * 2] = -INFINITY;
                part_ml[at * 2 + 1] = 0.f;
            }
        return;
    }
    const int* bt = block_tables + (size_t)seq_ids[tok] * max_blocks;
    const int key_lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int key_hi = p + 1;
    const int t_first = key_lo / FL_BN, t_end = (key_hi + FL_BN - 1) / FL_BN;
    int t_lo = t_first, t_hi = t_end;
    if (n_splits > 1) {
        const int per = (t_end - t_first + n_splits - 1) / n_splits;
        t_lo = t_first + split * per;
        t_hi = t_lo + per < t_end ? t_lo + per : t_end;
    }
    // this CTA's slice of the block table -> shared memory, so that the address of a row is
    // not a chain of two global loads
    int* s_pages = (int*)(sv + 2 * FL_BN * LD);
    const int pg_lo = (t_lo * FL_BN) / page_size;
    {
        int pg_hi = (t_hi * FL_BN + page_size - 1) / page_size;
        if (pg_hi > max_blocks) pg_hi = max_blocks;
        if (pg_hi - pg_lo > pages_cap) pg_hi = pg_lo + pages_cap;
        for (int i = pg_lo + tid; i < pg_hi; i += 128) s_pages[i - pg_lo] = bt[i];
    }
    __syncthreads();
    auto page_of = [&](int pi) { return pi - pg_lo < pages_cap ? s_pages[pi - pg_lo] : bt[pi]; };
    for (int i = tid; i < 16 * CH; i += 128) {
        const int r = i / CH, c = i % CH;
        const bool ok = r < G;
        cp_async16(sq + r * LD + c * 8,
                   ok ? q + (size_t)tok * q_stride + (size_t)(kvh * G + r) * DH + c * 8 : q, ok);
    }
    const int c_mine = tid % CH, r_mine = tid / CH;
    auto load_kv = [&](int t, int buf) {
        bf16* dk = sk + buf * FL_BN * LD + c_mine * 8;
        bf16* dv = sv + buf * FL_BN * LD + c_mine * 8;
#pragma unroll
        for (int r = r_mine; r < FL_BN; r += ROWS_PER_IT) {
            const int j = t * FL_BN + r;
            const bool ok = j >= key_lo && j < key_hi;
            size_t off = 0;
            if (ok) {
                const int pi = page_shift >= 0 ? j >> page_shift : j / page_size;
                const int po = j - pi * page_size;
                off = (((size_t)page_of(pi) * Hkv + kvh) * page_size + po) * DH + c_mine * 8;
            }
            cp_async16(dk + r * LD, k_cache + off, ok);
            cp_async16(dv + r * LD, v_cache + off, ok);
        }
    };
    if (t_lo < t_hi) load_kv(t_lo, 0);
    cp_async_commit();

    float o[DH / 8][4];
#pragma unroll
    for (int i = 0; i < DH / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    const int r_lo = lane >> 2, r_hi = r_lo + 8;
    const bool row_lo_ok = r_lo < G, row_hi_ok = r_hi < G;
    uint32_t qa[KS][4];

    for (int t = t_lo; t < t_hi; ++t) {
        const int buf = (t - t_lo) & 1;
        if (t + 1 < t_hi) load_kv(t + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (t == t_lo) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks)
                ldmatrix_x4(qa[ks], sq + ((lane & 7) + ((lane >> 3) & 1) * 8) * LD + ks * 16 +
                                        (lane >> 4) * 8);
        }
        const bf16* kt = sk + buf * FL_BN * LD + warp * 16 * LD;
        const bf16* vt = sv + buf * FL_BN * LD + warp * 16 * LD;
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = 0.f;
        s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t kb[4];
            ldmatrix_x4(kb, kt + ((lane & 7) + (lane >> 4) * 8) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
            mma_bf16(s[0], qa[ks], kb[0], kb[1]);
            mma_bf16(s[1], qa[ks], kb[2], kb[3]);
        }
        const int kbase = t * FL_BN + warp * 16 + (lane & 3) * 2;
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = kbase + i * 8 + e;
                const bool vis = j >= key_lo && j < key_hi;
                s[i][e] = (vis && row_lo_ok) ? s[i][e] * scale_log2 : -INFINITY;
                s[i][2 + e] = (vis && row_hi_ok) ? s[i][2 + e] * scale_log2 : -INFINITY;
                mx_lo = fmaxf(mx_lo, s[i][e]);
                mx_hi = fmaxf(mx_hi, s[i][2 + e]);
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
            s[i][0] = exp2f(s[i][0] - base_lo);
            s[i][1] = exp2f(s[i][1] - base_lo);
            s[i][2] = exp2f(s[i][2] - base_hi);
            s[i][3] = exp2f(s[i][3] - base_hi);
            sum_lo += s[i][0] + s[i][1];
            sum_hi += s[i][2] + s[i][3];
        }
        l_lo = l_lo * corr_lo + sum_lo;
        l_hi = l_hi * corr_hi + sum_hi;
        uint32_t pa[4];
        pa[0] = pack_bf16(s[0][0], s[0][1]);
        pa[1] = pack_bf16(s[0][2], s[0][3]);
        pa[2] = pack_bf16(s[1][0], s[1][1]);
        pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int dp = 0; dp < DH / 16; ++dp) {
            uint32_t vb[4];
            ldmatrix_x4_trans(vb, vt + ((lane & 7) + ((lane >> 3) & 1) * 8) * LD + dp * 16 +
                                      (lane >> 4) * 8);
            o[2 * dp][0] *= corr_lo; o[2 * dp][1] *= corr_lo;
            o[2 * dp][2] *= corr_hi; o[2 * dp][3] *= corr_hi;
            o[2 * dp + 1][0] *= corr_lo; o[2 * dp + 1][1] *= corr_lo;
            o[2 * dp + 1][2] *= corr_hi; o[2 * dp + 1][3] *= corr_hi;
            mma_bf16(o[2 * dp], pa, vb[0], vb[1]);
            mma_bf16(o[2 * dp + 1], pa, vb[2], vb[3]);
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    __syncthreads();
    pdl_launch_late();
    // join the four warps' states: O through the (now free) key/value buffers
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    float* so = (float*)sk;                    // [4][16][DH]
    const int col = (lane & 3) * 2;
#pragma unroll
    for (int i = 0; i < DH / 8; ++i) {
        *(float2*)(so + ((size_t)warp * 16 + r_lo) * DH + i * 8 + col) = make_float2(o[i][0], o[i][1]);
        *(float2*)(so + ((size_t)warp * 16 + r_hi) * DH + i * 8 + col) = make_float2(o[i][2], o[i][3]);
    }
    if ((lane & 3) == 0) {
        s_ml[warp][r_lo][0] = m_lo; s_ml[warp][r_lo][1] = l_lo;
        s_ml[warp][r_hi][0] = m_hi; s_ml[warp][r_hi][1] = l_hi;
    }
    __syncthreads();
    for (int i = tid; i < G * DH; i += 128) {
        const int r = i / DH, d = i % DH;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, s_ml[w][r][0]);
        float l = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = s_ml[w][r][0];
            if (mw != -INFINITY) {
                const float f = exp2f(mw - m);
                l += s_ml[w][r][1] * f;
                acc += so[((size_t)w * 16 + r) * DH + d] * f;
            }
        }
        const int head = kvh * G + r;
        if (n_splits == 1) {
            out[(size_t)tok * out_stride + (size_t)head * DH + d] =
                __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
        } else {
            const size_t at = ((size_t)tok * H + head) * n_splits + split;
            part_o[at * DH + d] = acc;
            if (d == 0) { part_ml[at * 2] = m; part_ml[at * 2 + 1] = l; }
        }
    }
}

// out[t, h, :] = sum_s O_s 2^(m_s - m) / sum_s l_s 2^(m_s - m), m = max_s m_s.
// A split that saw no key has m = -inf, l = 0 and its O is not read.
__global__ void flash_combine_kernel(const float* __restrict__ part_o,
                                     const float* __restrict__ part_ml, bf16* __restrict__ out,
                                     long long out_stride, int H, int DH, int n_splits,
                                     const int* __restrict__ tok_list) {
    pdl_wait();
    pdl_launch();
    // partial results lie by place in the launch; the output row is the token the list names
    const int h = blockIdx.y;
    const int t = tok_list ? tok_list[blockIdx.x] : blockIdx.x;
    const size_t base = ((size_t)blockIdx.x * H + h) * n_splits;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, part_ml[(base + s) * 2]);
    float l = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = part_ml[(base + s) * 2];
        if (ms != -INFINITY) l += part_ml[(base + s) * 2 + 1] * exp2f(ms - m);
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    for (int d = threadIdx.x; d < DH; d += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = part_ml[(base + s) * 2];
            if (ms != -INFINITY) acc += part_o[(base + s) * DH + d] * exp2f(ms - m);
        }
        out[(size_t)t * out_stride + (size_t)h * DH + d] = __float2bfloat16_rn(acc * inv);
    }
}

template <int DH>
static int prefill_launch(const bf16* q, long long q_stride, bf16* out, long long out_stride,
                          const bf16* k_cache, const bf16* v_cache, int page_size,
                          const int* block_tables, int max_blocks, const int* positions,
                          const int* seq_ids, const int* tile_tok0, const int* tile_ntok, int n_tiles,
                          int H, int Hkv, float scale, int window, cudaStream_t stream) {
    constexpr int LD = DH + FL_PAD;
    const int pages_cap = max_blocks < 4096 ? max_blocks : 4096;
    const size_t smem = (size_t)(FP_BM + 4 * FL_BN) * LD * sizeof(bf16) + (size_t)pages_cap * sizeof(int);
    auto kern = flash_prefill_kernel<DH>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    int shift = -1;
    for (int sft = 0; sft < 31; ++sft) if ((1 << sft) == page_size) shift = sft;
    kern<<<dim3(n_tiles, Hkv), FP_WARPS * 32, smem, stream>>>(
        q, q_stride, out, out_stride, k_cache, v_cache, page_size, shift, block_tables, max_blocks,
        positions, seq_ids, tile_tok0, tile_ntok, H, Hkv, scale * 1.4426950408889634f, window, pages_cap);
    return launch_status();
}

template <int DH>
static int decode_launch(const bf16* q, long long q_stride, bf16* out, long long out_stride,
                         const bf16* k_cache, const bf16* v_cache, int page_size,
                         const int* block_tables, int max_blocks, const int* positions,
                         const int* seq_ids, int T, int H, int Hkv, float scale, int window,
                         int n_splits, float* part_o, float* part_ml, cudaStream_t stream) {
    constexpr int LD = DH + FL_PAD;
    size_t smem = (size_t)(16 + 4 * FL_BN) * LD * sizeof(bf16);
    const size_t merge = (size_t)4 * 16 * DH * sizeof(float) + (size_t)16 * LD * sizeof(bf16);
    if (merge > smem) smem = merge;
    int pages_cap = max_blocks < 2048 ? max_blocks : 2048;     // block-table entries kept on chip
    smem += (size_t)pages_cap * sizeof(int);
    auto kern = flash_decode_kernel<DH>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    int shift = -1;
    for (int sft = 0; sft < 31; ++sft) if ((1 << sft) == page_size) shift = sft;
    return tgo_launch_pdl(kern, dim3(T, Hkv, n_splits), dim3(128), smem, stream, q, q_stride, out,
                          out_stride, k_cache, v_cache, page_size, shift, block_tables, max_blocks,
                          positions, seq_ids, H, Hkv, scale * 1.4426950408889634f, window, n_splits,
                          part_o, part_ml, pages_cap);
}

// head sizes with a tensor-core instance; others are refused and the caller falls back
TGO_API int tgo_attention_flash_supports(int dh, int group) {
    return (dh == 16 || dh == 32 || dh == 64 || dh == 128) && group >= 1 && group <= 16;
}

// Query rows (token x head of the group) one prefill tile holds: a tile takes
// tgo_attention_flash_tile_rows() / group consecutive tokens of one request.
TGO_API int tgo_attention_flash_tile_rows() { return FP_BM; }

// With tile arrays: the prefill kernel (n_splits must be 1). Without: every token is a tile
// of its own and the decode kernel runs, with n_splits CTAs per (token, kv head).
TGO_API int tgo_attention_flash(const void* q, long long q_stride, void* out, long long out_stride,
                                const void* k_cache, const void* v_cache, int page_size,
                                const int* block_tables, int max_blocks, const int* positions,
                                const int* seq_ids, const int* tile_tok0, const int* tile_ntok,
                                int n_tiles, int H, int Hkv, int dh, float scale, int window,
                                int n_splits, float* part_o, float* part_ml,
                                cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || H % Hkv || !tgo_attention_flash_supports(dh, H / Hkv) ||
        page_size <= 0 || max_blocks <= 0 || window < 0 || n_splits < 1 || Hkv > 65535 ||
        n_splits > 65535 || (n_splits > 1 && (!part_o || !part_ml || tile_tok0)) ||
        (tile_tok0 && !tile_ntok))
        return TGO_E_BAD_ARG;
    const bf16* qp = (const bf16*)q;
    const bf16* kp = (const bf16*)k_cache;
    const bf16* vp = (const bf16*)v_cache;
    bf16* op = (bf16*)out;
#define FA_CASE(D)                                                                                  \
    case D:                                                                                         \
        return tile_tok0 ? prefill_launch<D>(qp, q_stride, op, out_stride, kp, vp, page_size,        \
                                             block_tables, max_blocks, positions, seq_ids, tile_tok0, \
                                             tile_ntok, n_tiles, H, Hkv, scale, window, stream)      \
                         : decode_launch<D>(qp, q_stride, op, out_stride, kp, vp, page_size,         \
                                            block_tables, max_blocks, positions, seq_ids, n_tiles, H, \
                                            Hkv, scale, window, n_splits, part_o, part_ml, stream);
    switch (dh) {
        FA_CASE(16)
        FA_CASE(32)
        FA_CASE(64)
        FA_CASE(128)
    }
#undef FA_CASE
    return TGO_E_BAD_ARG;
}

static int combine_launch(const float* part_o, const float* part_ml, void* out, long long out_stride,
                          int T, int H, int dh, int n_splits, const int* tok_list, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H > 65535) return TGO_E_BAD_ARG;
    return tgo_launch_pdl(flash_combine_kernel, dim3(T, H),
                          dim3(dh < 128 ? 32 * ((dh + 31) / 32) : 128), 0, stream, part_o, part_ml,
                          (bf16*)out, out_stride, H, dh, n_splits, tok_list);
}

// The same for the T tokens that tok_list names (partial results by place in the list).
TGO_API int tgo_attention_flash_combine_listed(const float* part_o, const float* part_ml, void* out,
                                               long long out_stride, int T, int H, int dh, int n_splits,
                                               const int* tok_list, cudaStream_t stream) {
    return combine_launch(part_o, part_ml, out, out_stride, T, H, dh, n_splits, tok_list, stream);
}

TGO_API int tgo_attention_flash_combine(const float* part_o, const float* part_ml, void* out,
                                        long long out_stride, int T, int H, int dh, int n_splits,
                                        cudaStream_t stream) {
    return combine_launch(part_o, part_ml, out, out_stride, T, H, dh, n_splits, nullptr, stream);
}


// ------------------------------------------------------------ no-allocation entry point
// See attention_decode_static.h: the same decode kernels, with the partial outputs of the
// key splits in an array that is part of the library image instead of caller memory.
#include "attention_decode_static.h"

#include <mutex>

static __device__ __align__(256) float tgo_decode_static_scratch[TGO_DECODE_STATIC_SCRATCH_FLOATS];

#define TGO_STATIC_MAX_DEVICES 64

// Device address of the array on the current device. In host code the array's name is only
// a handle for the runtime, not an address a kernel could use; the address comes from
// cudaGetSymbolAddress, once per device, with that device current.
static int decode_static_scratch(float** ptr) {
    static std::mutex lock;
    static float* known[TGO_STATIC_MAX_DEVICES] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= TGO_STATIC_MAX_DEVICES) return TGO_E_BAD_ARG;
    std::lock_guard<std::mutex> guard(lock);
    if (!known[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, tgo_decode_static_scratch);
        if (e != cudaSuccess) return (int)e;
        known[dev] = (float*)p;
    }
    *ptr = known[dev];
    return 0;
}

int tgo_attention_decode_static(const void* q, long long q_stride, void* out, long long out_stride,
                                const void* k_cache, const void* v_cache, int page_size,
                                const int* block_tables, int max_blocks, const int* positions,
                                const int* seq_ids, int T, int H, int Hkv, int dh, float scale,
                                int window, int n_splits, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || H % Hkv || !tgo_attention_flash_supports(dh, H / Hkv) ||
        page_size <= 0 || max_blocks <= 0 || window < 0 || n_splits < 1 || n_splits > 65535 ||
        Hkv > 65535)
        return TGO_E_BAD_ARG;
    float* part_o = nullptr;
    float* part_ml = nullptr;
    if (n_splits > 1) {
        const size_t n_o = (size_t)T * H * n_splits * dh, n_ml = (size_t)T * H * n_splits * 2;
        if (n_o + n_ml > (size_t)TGO_DECODE_STATIC_SCRATCH_FLOATS) return TGO_E_SCRATCH_TOO_SMALL;
        float* base = nullptr;
        const int rc = decode_static_scratch(&base);
        if (rc) return rc;
        part_o = base;
        part_ml = base + n_o;
    }
    int rc = TGO_E_BAD_ARG;
#define FS_CASE(D)                                                                                   \
    case D:                                                                                          \
        rc = decode_launch<D>((const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)k_cache, \
                              (const bf16*)v_cache, page_size, block_tables, max_blocks, positions,  \
                              seq_ids, T, H, Hkv, scale, window, n_splits, part_o, part_ml, stream); \
        break;
    switch (dh) {
        FS_CASE(16)
        FS_CASE(32)
        FS_CASE(64)
        FS_CASE(128)
    }
#undef FS_CASE
    if (rc || n_splits == 1) return rc;
    return tgo_attention_flash_combine(part_o, part_ml, out, out_stride, T, H, dh, n_splits, stream);
}
