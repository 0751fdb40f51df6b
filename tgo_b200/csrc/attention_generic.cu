// Paged causal attention, one warp per (token, head), any head size up to 256 and any
// storage type. It is the float32 path's attention and the fallback of the bfloat16
// path for head sizes that the tensor-core kernels do not take.
//
// The query at position p of request b reads keys lo..p, lo = max(0, p - window + 1)
// (window 0: lo = 0), through the request's block table. Keys are taken 32 at a time
// starting at lo, so the order of every sum depends on (p, window) alone: the result
// for a position is bit-identical however the tokens were cut into steps or batched.
#include "common.cuh"

#define AG_MAX_DH 256
#define AG_WARPS 4

template <typename T>
__global__ void attention_generic_kernel(
    const T* __restrict__ q, long long q_stride, T* __restrict__ out, long long out_stride,
    int H, int Hkv, int dh, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
    int page_size, const int* __restrict__ block_tables, int max_blocks,
    const int* __restrict__ seq_ids, const int* __restrict__ positions, float scale, int window) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int h = blockIdx.y * AG_WARPS + warp;
    if (h >= H) return;
    float* qs = smem + warp * dh;
    const int p = positions[t];
    const int b = p >= 0 ? seq_ids[t] : 0;
    const int kvh = h / (H / Hkv);
    const int* bt = block_tables + (size_t)b * max_blocks;
    const T* qv = q + (size_t)t * q_stride + (size_t)h * dh;
    for (int i = lane; i < dh; i += 32) qs[i] = to_f32(qv[i]);
    __syncwarp();

    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    float m = -INFINITY, l = 0.f;
    float acc[AG_MAX_DH / 32];
#pragma unroll
    for (int i = 0; i < AG_MAX_DH / 32; ++i) acc[i] = 0.f;

    for (int base = lo; base <= p; base += 32) {
        const int j = base + lane;
        const int nvalid = (p - base + 1) < 32 ? (p - base + 1) : 32;
        float s = -INFINITY;
        if (j <= p) {
            const int page = bt[j / page_size];
            const T* kr = k_cache + (((size_t)page * Hkv + kvh) * page_size + (j % page_size)) * dh;
            float a = 0.f;
            for (int d = 0; d < dh; ++d) a += qs[d] * to_f32(kr[d]);
            s = a * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = expf(m - m_new);          // m = -inf the first time: corr = 0
        const float w = j <= p ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(w);
#pragma unroll
        for (int i = 0; i < AG_MAX_DH / 32; ++i) acc[i] *= corr;
        for (int jj = 0; jj < nvalid; ++jj) {
            const float wj = __shfl_sync(0xffffffffu, w, jj);
            const int kj = base + jj;
            const int page = bt[kj / page_size];
            const T* vr = v_cache + (((size_t)page * Hkv + kvh) * page_size + (kj % page_size)) * dh;
#pragma unroll
            for (int i = 0; i < AG_MAX_DH / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < dh) acc[i] += wj * to_f32(vr[d]);
            }
        }
        m = m_new;
    }
    T* o = out + (size_t)t * out_stride + (size_t)h * dh;
    const float inv = l > 0.f ? 1.f / l : 0.f;     // position < 0: no keys, zeros out
#pragma unroll
    for (int i = 0; i < AG_MAX_DH / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < dh) o[d] = from_f32<T>(acc[i] * inv);
    }
}

TGO_API int tgo_attention_generic(const void* q, long long q_stride, void* out,
                                  long long out_stride, int dtype, int T, int H, int Hkv, int dh,
                                  const void* k_cache, const void* v_cache, int page_size,
                                  const int* block_tables, int max_blocks, const int* seq_ids,
                                  const int* positions, float scale, int window,
                                  cudaStream_t stream) {
    if (T <= 0) return 0;
    if (dh <= 0 || dh > AG_MAX_DH || H <= 0 || Hkv <= 0 || H % Hkv || page_size <= 0 ||
        max_blocks <= 0 || window < 0)
        return TGO_E_BAD_ARG;
    const dim3 grid(T, (H + AG_WARPS - 1) / AG_WARPS);
    const size_t smem = (size_t)AG_WARPS * dh * sizeof(float);
    if (dtype == TGO_BF16)
        attention_generic_kernel<bf16><<<grid, AG_WARPS * 32, smem, stream>>>(
            (const bf16*)q, q_stride, (bf16*)out, out_stride, H, Hkv, dh, (const bf16*)k_cache,
            (const bf16*)v_cache, page_size, block_tables, max_blocks, seq_ids, positions, scale,
            window);
    else if (dtype == TGO_F32)
        attention_generic_kernel<float><<<grid, AG_WARPS * 32, smem, stream>>>(
            (const float*)q, q_stride, (float*)out, out_stride, H, Hkv, dh, (const float*)k_cache,
            (const float*)v_cache, page_size, block_tables, max_blocks, seq_ids, positions, scale,
            window);
    else
        return TGO_E_BAD_ARG;
    return launch_status();
}
