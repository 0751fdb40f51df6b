// Sampling on the device, one block per row of float32 logits, so that a step reads back
// token ids instead of [rows, vocab] floats.
//
// The order of the stages is the reference's (sample/sample.go:16-24, sample/stages.go:
// 74-146): bias -> penalties -> (temperature 0: argmax, ties to the lowest id) -> divide by
// the temperature -> top-k on the softmax weights by (weight, lower id) -> top-p (smallest
// prefix of the descending candidates whose weight reaches p of the total; at most 128
// candidates) -> walk the kept ids in ascending order and return the first whose running
// sum exceeds u * total, or the last kept id if rounding never gets there.
//
// Sums over the vocabulary are formed per thread over a contiguous range and then over the
// threads in order, which is not the reference's single ascending sum: totals can differ
// in their last bits and so can a draw that lands within rounding of a boundary.
#include "common.cuh"

#define SM_THREADS 1024
#define SM_MAXC 128          // most candidates a truncation stage keeps (sample.go:47)

// ---------------------------------------------------------------- bias and penalties
// Sparse edits of one row: logits[bias_ids[i]] += bias[i]; then for each distinct history
// token (ids, counts): repetition (divide a positive logit, multiply otherwise), then
// subtract presence + frequency * count (sample/stages.go:152-190).
__global__ void adjust_kernel(float* __restrict__ row, const int* __restrict__ bias_ids,
                              const float* __restrict__ bias, int n_bias,
                              const int* __restrict__ ids, const int* __restrict__ counts, int n_ids,
                              float rep, float presence, float frequency, int V) {
    for (int i = threadIdx.x; i < n_bias; i += blockDim.x)
        if (bias_ids[i] >= 0 && bias_ids[i] < V) row[bias_ids[i]] += bias[i];
    __syncthreads();
    const bool use_rep = rep != 0.f && rep != 1.f;
    const bool use_add = presence != 0.f || frequency != 0.f;
    for (int i = threadIdx.x; i < n_ids; i += blockDim.x) {
        const int id = ids[i];
        if (id < 0 || id >= V) continue;
        float x = row[id];
        if (use_rep) x = x > 0.f ? x / rep : x * rep;
        if (use_add) x -= presence + frequency * (float)counts[i];
        row[id] = x;
    }
}

TGO_API int tgo_logits_adjust(float* row, const int* bias_ids, const float* bias, int n_bias,
                              const int* ids, const int* counts, int n_ids, float rep,
                              float presence, float frequency, int V, cudaStream_t stream) {
    if (n_bias <= 0 && n_ids <= 0) return 0;
    adjust_kernel<<<1, 256, 0, stream>>>(row, bias_ids, bias, n_bias, ids, counts, n_ids, rep,
                                         presence, frequency, V);
    return launch_status();
}

// ------------------------------------------------------------------------- helpers
struct Best { float v; int i; };

__device__ __forceinline__ Best better(Best a, Best b) {   // larger value, then lower id
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

// argmax of f(row[i]) over the row with the lowest-id tie rule; every thread gets it.
__device__ Best block_argmax(const float* __restrict__ row, int V, float inv_t, Best* scratch) {
    Best b = {-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = inv_t == 1.f ? row[i] : row[i] / inv_t;
        if (v > b.v || (v == b.v && i < b.i)) { b.v = v; b.i = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other;
        other.v = __shfl_xor_sync(0xffffffffu, b.v, o);
        other.i = __shfl_xor_sync(0xffffffffu, b.i, o);
        b = better(b, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = b;
    __syncthreads();
    if (warp == 0) {
        Best t = lane < (blockDim.x >> 5) ? scratch[lane] : Best{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best other;
            other.v = __shfl_xor_sync(0xffffffffu, t.v, o);
            other.i = __shfl_xor_sync(0xffffffffu, t.i, o);
            t = better(t, other);
        }
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// argmax in two passes so that a handful of rows still fills the GPU: AM_PARTS blocks per row
// each reduce a contiguous slice to (value, id); one warp per row then reduces the parts.
// Ties go to the lowest id at every level.
#define AM_PARTS 32
#define AM_THREADS 256

__global__ void __launch_bounds__(AM_THREADS)
argmax_part_kernel(const float* __restrict__ logits, long long stride, int V,
                   float* __restrict__ part_v, int* __restrict__ part_i) {
    __shared__ Best scratch[33];
    pdl_wait();
    pdl_launch();
    const int r = blockIdx.y, part = blockIdx.x;
    const int per = (V + AM_PARTS - 1) / AM_PARTS;
    const int lo = part * per, hi = lo + per < V ? lo + per : V;
    const float* row = logits + (size_t)r * stride;
    Best b = {-INFINITY, 0x7fffffff};
    for (int i = lo + threadIdx.x; i < hi; i += AM_THREADS) {
        const float v = row[i];
        if (v > b.v || (v == b.v && i < b.i)) { b.v = v; b.i = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other;
        other.v = __shfl_xor_sync(0xffffffffu, b.v, o);
        other.i = __shfl_xor_sync(0xffffffffu, b.i, o);
        b = better(b, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) scratch[warp] = b;
    __syncthreads();
    if (warp == 0) {
        Best t = lane < AM_THREADS / 32 ? scratch[lane] : Best{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best other;
            other.v = __shfl_xor_sync(0xffffffffu, t.v, o);
            other.i = __shfl_xor_sync(0xffffffffu, t.i, o);
            t = better(t, other);
        }
        if (lane == 0) { part_v[r * AM_PARTS + part] = t.v; part_i[r * AM_PARTS + part] = t.i; }
    }
}

__global__ void argmax_final_kernel(const float* __restrict__ part_v,
                                    const int* __restrict__ part_i, int* __restrict__ out) {
    pdl_wait();
    pdl_launch();
    const int r = blockIdx.x, lane = threadIdx.x;
    Best b = {part_v[r * AM_PARTS + lane], part_i[r * AM_PARTS + lane]};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other;
        other.v = __shfl_xor_sync(0xffffffffu, b.v, o);
        other.i = __shfl_xor_sync(0xffffffffu, b.i, o);
        b = better(b, other);
    }
    if (lane == 0) out[r] = b.i == 0x7fffffff ? 0 : b.i;
}

// scratch: n * 32 floats and n * 32 ints
TGO_API int tgo_argmax(const float* logits, long long stride, int n, int V, int* out,
                       float* part_v, int* part_i, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (V <= 0 || n > 65535 || !part_v || !part_i) return TGO_E_BAD_ARG;
    const int rc = tgo_launch_pdl(argmax_part_kernel, dim3(AM_PARTS, n), dim3(AM_THREADS), 0, stream,
                                  logits, stride, V, part_v, part_i);
    if (rc) return rc;
    return tgo_launch_pdl(argmax_final_kernel, dim3(n), dim3(32), 0, stream,
                          (const float*)part_v, (const int*)part_i, out);
}

// Exclusive prefix of per-thread values (float), in thread order; total in *total.
// part[] has blockDim.x + 1 floats of shared memory. The order of additions is fixed.
__device__ void block_prefix_f(float mine, float* part, float* seg, float* total) {
    const int t = threadIdx.x;
    part[t] = mine;
    __syncthreads();
    if (t < 32) {
        float s = 0.f;
        for (int j = 0; j < 32; ++j) s += part[t * 32 + j];
        seg[t] = s;
    }
    __syncthreads();
    if (t == 0) {
        float s = 0.f;
        for (int j = 0; j < 32; ++j) { const float x = seg[j]; seg[j] = s; s += x; }
        *total = s;
    }
    __syncthreads();
    if (t < 32) {
        float s = seg[t];
        for (int j = 0; j < 32; ++j) { const float x = part[t * 32 + j]; part[t * 32 + j] = s; s += x; }
    }
    __syncthreads();
}

__device__ void block_prefix_i(int mine, int* part, int* seg, int* total) {
    const int t = threadIdx.x;
    part[t] = mine;
    __syncthreads();
    if (t < 32) {
        int s = 0;
        for (int j = 0; j < 32; ++j) s += part[t * 32 + j];
        seg[t] = s;
    }
    __syncthreads();
    if (t == 0) {
        int s = 0;
        for (int j = 0; j < 32; ++j) { const int x = seg[j]; seg[j] = s; s += x; }
        *total = s;
    }
    __syncthreads();
    if (t < 32) {
        int s = seg[t];
        for (int j = 0; j < 32; ++j) { const int x = part[t * 32 + j]; part[t * 32 + j] = s; s += x; }
    }
    __syncthreads();
}

// Entries have..want-1 of a row's alternatives: the lowest ids that are not among
// listed[0..n_listed), each with -inf. These are tokens the policy gave no chance; among
// equal shares the lower id comes first (decode.go:293-318). Ids below 2 * SM_MAXC suffice,
// since at most SM_MAXC are listed and at most SM_MAXC are wanted. Every thread calls it.
__device__ void fill_masked(int have, int want, const int* listed, int n_listed, int V,
                            int* ipart, int* iseg, int* itotal,
                            int* __restrict__ ids_out, float* __restrict__ lp_out) {
    const int t = threadIdx.x;
    int open_id = 0;
    if (t < 2 * SM_MAXC && t < V) {
        open_id = 1;
        for (int j = 0; j < n_listed; ++j)
            if (listed[j] == t) { open_id = 0; break; }
    }
    block_prefix_i(open_id, ipart, iseg, itotal);
    if (open_id) {
        const int at = have + ipart[t];
        if (at < want) { ids_out[at] = t; lp_out[at] = -INFINITY; }
    }
}

// ------------------------------------------------------------------------- sampler
// With lp_n given, a row r with lp_n[r] >= 0 also reports the distribution it was drawn
// from, after every stage of the policy (decode.go:263-318, sample/sample.go:155-176):
// lp_out[r] = ln of the drawn token's share of the kept weights, and the lp_n[r] (at most
// top_stride) most likely tokens, descending by (share, lower id), in top_ids / top_lp;
// a token outside the kept set has -inf, and at temperature 0 every token but the argmax.
// The draw is the same with and without the report.
__global__ void __launch_bounds__(SM_THREADS)
sample_kernel(const float* __restrict__ logits, long long stride, int V,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ draws,
              int* __restrict__ out, const int* __restrict__ lp_n, float* __restrict__ lp_out,
              int* __restrict__ top_ids, float* __restrict__ top_lp, int top_stride) {
    __shared__ Best bscratch[33];
    __shared__ float part[SM_THREADS];
    __shared__ float seg[32];
    __shared__ int ipart[SM_THREADS];
    __shared__ int iseg[32];
    __shared__ float total_s;
    __shared__ int itotal_s;
    __shared__ int result_s;
    __shared__ unsigned hist[256];
    __shared__ unsigned sel_prefix, sel_remaining;
    __shared__ float cw[SM_MAXC], sw[SM_MAXC];
    __shared__ int cid[SM_MAXC], sid[SM_MAXC];
    __shared__ int n_cand, n_kept;
    __shared__ int single_s;

    const int r = blockIdx.x, t = threadIdx.x;
    const float* row = logits + (size_t)r * stride;
    const float T = temperature[r];
    const float u = draws[r];
    int want = lp_n ? lp_n[r] : -1;           // < 0: no report for this row
    if (want > top_stride) want = top_stride;
    if (want > V) want = V;
    int* const alt_ids = top_ids ? top_ids + (size_t)r * top_stride : nullptr;
    float* const alt_lp = top_lp ? top_lp + (size_t)r * top_stride : nullptr;
    if (T == 0.f) {
        const Best b = block_argmax(row, V, 1.f, bscratch);
        if (t == 0) {
            out[r] = b.i;
            if (want >= 0) lp_out[r] = 0.f;
            if (want > 0) { alt_ids[0] = b.i; alt_lp[0] = 0.f; }
            single_s = b.i;
        }
        if (want > 1) {
            __syncthreads();
            fill_masked(1, want, &single_s, 1, V, ipart, iseg, &itotal_s, alt_ids, alt_lp);
        }
        return;
    }
    const float m = block_argmax(row, V, T, bscratch).v;     // max of logits / T
    const int chunk = (V + SM_THREADS - 1) / SM_THREADS;
    const int c0 = t * chunk < V ? t * chunk : V;
    const int c1 = c0 + chunk < V ? c0 + chunk : V;
    const int k_req = top_k[r];
    const float p_req = top_p[r];

    // total of exp(l/T - m) over the vocabulary, ascending within a thread, threads in order
    float mine = 0.f;
    for (int i = c0; i < c1; ++i) mine += expf(row[i] / T - m);
    block_prefix_f(mine, part, seg, &total_s);
    const float total_all = total_s;

    const bool all_kept = k_req <= 0 && p_req <= 0.f;
    if (all_kept) {
        if (t == 0) result_s = V - 1;
        __syncthreads();
        const float target = u * total_all;
        const float before = part[t];
        const float after = t + 1 < SM_THREADS ? part[t + 1] : total_all;
        if (c0 < c1 && before <= target && after > target) {
            float acc = before;
            int pick = c1 - 1;
            for (int i = c0; i < c1; ++i) {
                acc += expf(row[i] / T - m);
                if (acc > target) { pick = i; break; }
            }
            result_s = pick;
        }
        __syncthreads();
        if (t == 0) {
            out[r] = result_s;
            if (want >= 0) lp_out[r] = logf(expf(row[result_s] / T - m) / total_all);
        }
        if (want <= 0) return;
        // the alternatives are the `want` largest of the whole vocabulary: selected below
    }

    // ---- the k largest weights by (weight, lower id): radix select on the float bits
    const int k = all_kept ? want
                : k_req > 0 ? (k_req < V ? k_req : V) : (SM_MAXC < V ? SM_MAXC : V);
    if (t == 0) { sel_prefix = 0u; sel_remaining = (unsigned)k; }
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        for (int i = t; i < 256; i += SM_THREADS) hist[i] = 0u;
        __syncthreads();
        const unsigned prefix = sel_prefix;
        for (int i = t; i < V; i += SM_THREADS) {
            const unsigned bits = __float_as_uint(expf(row[i] / T - m));
            if (pass == 0 || (bits >> (shift + 8)) == (prefix >> (shift + 8)))
                atomicAdd(&hist[(bits >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (t == 0) {
            unsigned rem = sel_remaining;
            int b = 255;
            for (; b > 0; --b) {
                if (hist[b] >= rem) break;
                rem -= hist[b];
            }
            sel_prefix = prefix | ((unsigned)b << shift);
            sel_remaining = rem;
        }
        __syncthreads();
    }
    const unsigned thr = sel_prefix;            // bits of the k-th largest weight
    const int need_equal = (int)sel_remaining;  // how many of the ties at thr are kept
    if (t == 0) n_cand = 0;
    __syncthreads();
    int eq = 0;
    for (int i = c0; i < c1; ++i) {
        const float w = expf(row[i] / T - m);
        const unsigned bits = __float_as_uint(w);
        if (bits > thr) {
            const int at = atomicAdd(&n_cand, 1);
            if (at < SM_MAXC) { cw[at] = w; cid[at] = i; }
        } else if (bits == thr) {
            ++eq;
        }
    }
    block_prefix_i(eq, ipart, iseg, &itotal_s);
    {
        int rank = ipart[t];                    // ties before this thread's range, by id
        for (int i = c0; i < c1 && rank < need_equal; ++i) {
            const float w = expf(row[i] / T - m);
            if (__float_as_uint(w) == thr) {
                const int at = atomicAdd(&n_cand, 1);
                if (at < SM_MAXC) { cw[at] = w; cid[at] = i; }
                ++rank;
            }
        }
    }
    __syncthreads();
    const int nc = n_cand < SM_MAXC ? n_cand : SM_MAXC;
    // descending by (weight, lower id)
    if (t < nc) {
        int rank = 0;
        for (int j = 0; j < nc; ++j)
            if (cw[j] > cw[t] || (cw[j] == cw[t] && cid[j] < cid[t])) ++rank;
        sw[rank] = cw[t];
        sid[rank] = cid[t];
    }
    __syncthreads();
    if (all_kept) {
        if (t < nc && t < want) { alt_ids[t] = sid[t]; alt_lp[t] = logf(sw[t] / total_all); }
        return;
    }
    if (t == 0) {
        float total;
        if (k_req > 0) {
            total = 0.f;
            for (int j = 0; j < nc; ++j) total += sw[j];
        } else {
            total = total_all;
        }
        int kept = nc;
        if (p_req > 0.f) {
            const float target = total * p_req;
            float acc = 0.f;
            kept = 0;
            while (kept < nc && acc < target) { acc += sw[kept]; ++kept; }
            total = acc;
        }
        n_kept = kept;
        total_s = total;
    }
    __syncthreads();
    const int kept = n_kept;
    if (want > 0) {
        if (t < kept && t < want) { alt_ids[t] = sid[t]; alt_lp[t] = logf(sw[t] / total_s); }
        if (want > kept)
            fill_masked(kept, want, sid, kept, V, ipart, iseg, &itotal_s, alt_ids, alt_lp);
    }
    // ascending by id
    if (t < kept) {
        int rank = 0;
        for (int j = 0; j < kept; ++j)
            if (sid[j] < sid[t]) ++rank;
        cw[rank] = sw[t];
        cid[rank] = sid[t];
    }
    __syncthreads();
    if (t == 0) {
        const float target = u * total_s;
        float acc = 0.f;
        int pick = kept > 0 ? cid[kept - 1] : 0;
        float w_pick = kept > 0 ? cw[kept - 1] : 0.f;
        for (int j = 0; j < kept; ++j) {
            acc += cw[j];
            if (acc > target) { pick = cid[j]; w_pick = cw[j]; break; }
        }
        out[r] = pick;
        if (want >= 0) lp_out[r] = logf(w_pick / total_s);
    }
}

// lp_n null: no row reports. Else lp_out has n floats and, if top_stride > 0, top_ids and
// top_lp have n * top_stride entries (top_stride at most 128).
TGO_API int tgo_sample(const float* logits, long long stride, int n, int V,
                       const float* temperature, const int* top_k, const float* top_p,
                       const float* draws, int* out, const int* lp_n, float* lp_out,
                       int* top_ids, float* top_lp, int top_stride, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (V <= 0) return TGO_E_BAD_ARG;
    if (lp_n && (!lp_out || top_stride < 0 || top_stride > SM_MAXC ||
                 (top_stride > 0 && (!top_ids || !top_lp)))) return TGO_E_BAD_ARG;
    sample_kernel<<<n, SM_THREADS, 0, stream>>>(logits, stride, V, temperature, top_k, top_p,
                                                draws, out, lp_n, lp_out, top_ids, top_lp,
                                                lp_n ? top_stride : 0);
    return launch_status();
}
