// Memory-bound kernels between the matrix products: embedding gather, residual add
// fused with RMSNorm (and with the row selection before the head), the SiLU gate, and
// per-head q/k RMSNorm fused with the rotation and the write into the paged cache.
// Sums of squares, the rotation and the residual are float32 whatever the storage.
#include "common.cuh"

// ------------------------------------------------------------------ embedding
// out[t, :] = table[ids[t], :] widened to float32 (the residual stream's type).
// An id outside [0, V) writes zeros; the host refuses such ids before the launch.
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ out, int d, int V) {
    pdl_wait();
    pdl_launch();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < V;
    const T* row = table + (size_t)(ok ? id : 0) * d;
    float* o = out + (size_t)t * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = ok ? to_f32(row[i]) : 0.f;
}

TGO_API int tgo_embed(const void* table, int dtype, const int* ids, float* out, int T, int d,
                      int V, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int threads = d >= 1024 ? 256 : 128;
    if (dtype == TGO_BF16)
        return tgo_launch_pdl(embed_kernel<bf16>, dim3(T), dim3(threads), 0, stream,
                              (const bf16*)table, ids, out, d, V);
    else if (dtype == TGO_F32)
        return tgo_launch_pdl(embed_kernel<float>, dim3(T), dim3(threads), 0, stream,
                              (const float*)table, ids, out, d, V);
    else
        return TGO_E_BAD_ARG;
    return launch_status();
}

// ------------------------------------------------------- residual add + RMSNorm
// For output row i: r = rows ? rows[i] : i;  x = h[r] (+ delta[r]);  if rows is null the
// sum is written back to h (the residual stream moves on);  out[i] = x * rsqrt(mean x^2
// + eps) * gain, computed as (x * scale) * gain.  One block per row; the row is held in
// registers when it fits (d <= blockDim * 4 * CHUNKS), else read a second time.
template <typename TD, typename TO, int CHUNKS>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                   const float* __restrict__ gain, float eps,
                                   TO* __restrict__ out, const int* __restrict__ rows, int d) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch();
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float* hr = h + (size_t)r * d;
    const TD* dr = delta ? delta + (size_t)r * d : nullptr;
    TO* o = out + (size_t)i * d;
    float x[CHUNKS > 0 ? CHUNKS : 1];
    float ss = 0.f;
    if (CHUNKS > 0) {
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            const int j = threadIdx.x + c * blockDim.x;
            float v = 0.f;
            if (j < d) {
                v = hr[j];
                if (dr) v += to_f32(dr[j]);
                if (dr && !rows) hr[j] = v;
            }
            x[c] = v;
            ss += v * v;
        }
    } else {
        for (int j = threadIdx.x; j < d; j += blockDim.x) {
            float v = hr[j];
            if (dr) v += to_f32(dr[j]);
            if (dr && !rows) hr[j] = v;
            ss += v * v;
        }
    }
    const float total = block_sum(ss, scratch);
    const float scale = rsqrtf(total / (float)d + eps);
    if (CHUNKS > 0) {
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            const int j = threadIdx.x + c * blockDim.x;
            if (j < d) o[j] = from_f32<TO>((x[c] * scale) * gain[j]);
        }
    } else {
        for (int j = threadIdx.x; j < d; j += blockDim.x) {
            float v = hr[j];
            if (dr && rows) v += to_f32(dr[j]);
            o[j] = from_f32<TO>((v * scale) * gain[j]);
        }
    }
}

// The same with four consecutive elements per thread and 16-byte accesses, for d % 4 == 0
// and rows that fit 4 * CH4 * blockDim registers.
template <typename TD> struct Delta4;
template <> struct Delta4<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 v = *(const uint2*)p;
        const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&v.x);
        const float2 b = __bfloat1622float2(*(const __nv_bfloat162*)&v.y);
        return make_float4(a.x, a.y, b.x, b.y);
    }
};
template <> struct Delta4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *(const float4*)p; }
};
template <typename TO> struct Out4;
template <> struct Out4<bf16> {
    static __device__ __forceinline__ void store(bf16* p, float4 x) {
        __nv_bfloat162 a = __floats2bfloat162_rn(x.x, x.y), b = __floats2bfloat162_rn(x.z, x.w);
        uint2 v;
        v.x = *(uint32_t*)&a;
        v.y = *(uint32_t*)&b;
        *(uint2*)p = v;
    }
};
template <> struct Out4<float> {
    static __device__ __forceinline__ void store(float* p, float4 x) { *(float4*)p = x; }
};

template <typename TD, typename TO, int CH4>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                       const float* __restrict__ gain, float eps,
                                       TO* __restrict__ out, const int* __restrict__ rows, int d) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch();
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float* hr = h + (size_t)r * d;
    const TD* dr = delta ? delta + (size_t)r * d : nullptr;
    TO* o = out + (size_t)i * d;
    float4 x[CH4];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < CH4; ++c) {
        const int j = 4 * (threadIdx.x + c * blockDim.x);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (j < d) {
            v = *(const float4*)(hr + j);
            if (dr) {
                const float4 dl = Delta4<TD>::load(dr + j);
                v.x += dl.x; v.y += dl.y; v.z += dl.z; v.w += dl.w;
                if (!rows) *(float4*)(hr + j) = v;
            }
        }
        x[c] = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    const float total = block_sum(ss, scratch);
    const float scale = rsqrtf(total / (float)d + eps);
#pragma unroll
    for (int c = 0; c < CH4; ++c) {
        const int j = 4 * (threadIdx.x + c * blockDim.x);
        if (j < d) {
            const float4 g = *(const float4*)(gain + j);
            Out4<TO>::store(o + j, make_float4((x[c].x * scale) * g.x, (x[c].y * scale) * g.y,
                                               (x[c].z * scale) * g.z, (x[c].w * scale) * g.w));
        }
    }
}

template <typename TD, typename TO>
static int add_rmsnorm_launch(float* h, const void* delta, const float* gain, float eps, void* out,
                              const int* rows, int n, int d, cudaStream_t s) {
    const TD* dl = (const TD*)delta;
    TO* o = (TO*)out;
    if (d % 4 == 0 && d <= 16384 && ((uintptr_t)h % 16 == 0) && ((uintptr_t)out % 16 == 0) &&
        ((uintptr_t)gain % 16 == 0) && (!delta || (uintptr_t)delta % 16 == 0)) {
        const int quads = d / 4;
        const int vt = quads <= 256 ? 128 : quads <= 1024 ? 256 : 512;
        const int ch = (quads + vt - 1) / vt;
        if (ch <= 1) return tgo_launch_pdl(add_rmsnorm_vec_kernel<TD, TO, 1>, dim3(n), dim3(vt), 0, s, h, dl, gain, eps, o, rows, d);
        if (ch <= 2) return tgo_launch_pdl(add_rmsnorm_vec_kernel<TD, TO, 2>, dim3(n), dim3(vt), 0, s, h, dl, gain, eps, o, rows, d);
        if (ch <= 4) return tgo_launch_pdl(add_rmsnorm_vec_kernel<TD, TO, 4>, dim3(n), dim3(vt), 0, s, h, dl, gain, eps, o, rows, d);
        return tgo_launch_pdl(add_rmsnorm_vec_kernel<TD, TO, 8>, dim3(n), dim3(vt), 0, s, h, dl, gain, eps, o, rows, d);
    }
    int threads = 256;
    if (d > 2048) threads = 512;
    if (d > 4096) threads = 1024;
    const int chunks = (d + threads - 1) / threads;
    if (chunks <= 4)
        return tgo_launch_pdl(add_rmsnorm_kernel<TD, TO, 4>, dim3(n), dim3(threads), 0, s, h, dl,
                              gain, eps, o, rows, d);
    else if (chunks <= 8)
        return tgo_launch_pdl(add_rmsnorm_kernel<TD, TO, 8>, dim3(n), dim3(threads), 0, s, h, dl,
                              gain, eps, o, rows, d);
    else if (chunks <= 16)
        return tgo_launch_pdl(add_rmsnorm_kernel<TD, TO, 16>, dim3(n), dim3(threads), 0, s, h, dl,
                              gain, eps, o, rows, d);
    else
        return tgo_launch_pdl(add_rmsnorm_kernel<TD, TO, 0>, dim3(n), dim3(threads), 0, s, h, dl,
                              gain, eps, o, rows, d);
}

TGO_API int tgo_add_rmsnorm(float* h, const void* delta, int delta_dtype, const float* gain,
                            float eps, void* out, int out_dtype, const int* rows, int n, int d,
                            cudaStream_t stream) {
    if (n <= 0) return 0;
    if (d <= 0) return TGO_E_BAD_ARG;
    if (out_dtype == TGO_BF16 && (delta_dtype == TGO_BF16 || !delta))
        return add_rmsnorm_launch<bf16, bf16>(h, delta, gain, eps, out, rows, n, d, stream);
    if (out_dtype == TGO_F32 && (delta_dtype == TGO_F32 || !delta))
        return add_rmsnorm_launch<float, float>(h, delta, gain, eps, out, rows, n, d, stream);
    if (out_dtype == TGO_BF16 && delta_dtype == TGO_F32)
        return add_rmsnorm_launch<float, bf16>(h, delta, gain, eps, out, rows, n, d, stream);
    if (out_dtype == TGO_F32 && delta_dtype == TGO_BF16)
        return add_rmsnorm_launch<bf16, float>(h, delta, gain, eps, out, rows, n, d, stream);
    return TGO_E_BAD_ARG;
}

// h[r] += delta[r] for every row, nothing else (the add a block leaves pending when
// no norm follows it).
template <typename TD>
__global__ void residual_add_kernel(float* __restrict__ h, const TD* __restrict__ delta, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) h[i] += to_f32(delta[i]);
}

TGO_API int tgo_residual_add(float* h, const void* delta, int dtype, long long n,
                             cudaStream_t stream) {
    if (n <= 0) return 0;
    const int threads = 256;
    const int blocks = (int)((n + threads - 1) / threads < 65535 ? (n + threads - 1) / threads : 65535);
    if (dtype == TGO_BF16)
        residual_add_kernel<bf16><<<blocks, threads, 0, stream>>>(h, (const bf16*)delta, (size_t)n);
    else if (dtype == TGO_F32)
        residual_add_kernel<float><<<blocks, threads, 0, stream>>>(h, (const float*)delta, (size_t)n);
    else
        return TGO_E_BAD_ARG;
    return launch_status();
}

// ------------------------------------------------------------------- SiLU gate
// out[t, j] = silu(gate_j) * up_j over gu [T, 2f]. Two column layouts of gu:
//   plain        gate_j = gu[t, j],                      up_j = gu[t, f + j]
//   interleaved  gate_j = gu[t, 16 * (j / 8) + j % 8],   up_j = gu[t, 16 * (j / 8) + 8 + j % 8]
// (eight gate columns, then the eight matching up columns: the row order in which a joined
// gate/up matrix is kept so that one CTA of the weight-streaming product holds both).
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int f, int interleaved) {
    pdl_wait();
    pdl_launch();
    const size_t t = blockIdx.y;
    const T* row = gu + t * 2 * (size_t)f;
    T* o = out + t * (size_t)f;
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < f; j += gridDim.x * blockDim.x) {
        const int gi = interleaved ? 16 * (j / 8) + j % 8 : j;
        const int ui = interleaved ? gi + 8 : f + j;
        const float a = to_f32(row[gi]);
        const float s = a / (1.f + expf(-a));
        o[j] = from_f32<T>(s * to_f32(row[ui]));
    }
}

// bf16, 8 values per thread when f is a multiple of 8 (16-byte loads and stores).
__global__ void swiglu_bf16x8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int f,
                                     int interleaved) {
    pdl_wait();
    pdl_launch();
    const size_t t = blockIdx.y;
    const uint4* row = (const uint4*)(gu + t * 2 * (size_t)f);
    uint4* o = (uint4*)(out + t * (size_t)f);
    const int n8 = f / 8;
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < n8; j += gridDim.x * blockDim.x) {
        uint4 gv = row[interleaved ? 2 * j : j], uv = row[interleaved ? 2 * j + 1 : n8 + j], ov;
        const __nv_bfloat162* gp = (const __nv_bfloat162*)&gv;
        const __nv_bfloat162* up = (const __nv_bfloat162*)&uv;
        __nv_bfloat162* op = (__nv_bfloat162*)&ov;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 a = __bfloat1622float2(gp[k]);
            const float2 b = __bfloat1622float2(up[k]);
            float2 r;
            r.x = a.x / (1.f + expf(-a.x)) * b.x;
            r.y = a.y / (1.f + expf(-a.y)) * b.y;
            op[k] = __float22bfloat162_rn(r);
        }
        o[j] = ov;
    }
}

TGO_API int tgo_swiglu(const void* gate_up, void* out, int dtype, int T, int f, int interleaved,
                       cudaStream_t stream) {
    if (T <= 0) return 0;
    if (f <= 0 || (interleaved && f % 8)) return TGO_E_BAD_ARG;
    // grid.y is limited to 65535 rows: larger batches go in slices.
    for (int t0 = 0; t0 < T; t0 += 65535) {
        const int rows = T - t0 < 65535 ? T - t0 : 65535;
        int rc;
        if (dtype == TGO_BF16 && f % 8 == 0) {
            rc = tgo_launch_pdl(swiglu_bf16x8_kernel, dim3((f / 8 + 255) / 256, rows), dim3(256), 0,
                                stream, (const bf16*)gate_up + (size_t)t0 * 2 * f,
                                (bf16*)out + (size_t)t0 * f, f, interleaved);
        } else if (dtype == TGO_BF16) {
            rc = tgo_launch_pdl(swiglu_kernel<bf16>, dim3((f + 255) / 256, rows), dim3(256), 0,
                                stream, (const bf16*)gate_up + (size_t)t0 * 2 * f,
                                (bf16*)out + (size_t)t0 * f, f, interleaved);
        } else if (dtype == TGO_F32) {
            rc = tgo_launch_pdl(swiglu_kernel<float>, dim3((f + 255) / 256, rows), dim3(256), 0,
                                stream, (const float*)gate_up + (size_t)t0 * 2 * f,
                                (float*)out + (size_t)t0 * f, f, interleaved);
        } else {
            return TGO_E_BAD_ARG;
        }
        if (rc) return rc;
    }
    return 0;
}

// ------------------------------------------------------------ rotation table
// table[t, i] = cos(pos_t * inv_freq[i]), table[t, half + i] = sin(...), the angle and its
// sine and cosine evaluated in float64 and rounded once to float32. Made once per step and
// read by every layer that rotates with the same frequencies.
__global__ void rope_table_kernel(const int* __restrict__ positions,
                                  const double* __restrict__ inv_freq, float* __restrict__ table,
                                  int half) {
    pdl_wait();
    pdl_launch();
    const int t = blockIdx.x;
    const double pos = (double)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        double s, c;
        sincos(pos * inv_freq[i], &s, &c);
        table[(size_t)t * 2 * half + i] = (float)c;
        table[(size_t)t * 2 * half + half + i] = (float)s;
    }
}

TGO_API int tgo_rope_table(const int* positions, const double* inv_freq, float* table, int T,
                           int half, cudaStream_t stream) {
    if (T <= 0 || half <= 0) return 0;
    return tgo_launch_pdl(rope_table_kernel, dim3(T), dim3(half < 64 ? 32 : 64), 0, stream,
                          positions, inv_freq, table, half);
}

// --------------------------------- per-head q/k RMSNorm + rotation + cache write
// One block per token. Heads of q are normalised (if q_gain), rotated (if a rotation table
// is given) and written back in place; heads of k likewise and then stored at the token's
// slot of the paged cache; v is copied to its slot. The rotation pairs channel i with
// i + rot/2 (half-split) and is done in float32 with the table's cosines and sines.
// slot < 0 stores nothing. k or v may be null (a layer that reads another layer's cache
// computes q only); with k given and k_cache null, k is written back in place like q (used
// when another position encoding runs between the norm and the store).
//
// Cache layout of one layer: [page][kv_head][offset in page][head_dim]; slot = page *
// page_size + offset.
#define QKR_MAX_DH 512
#define QKR_WARPS 4
// grid (tokens, ceil((H + 2 Hkv) / QKR_WARPS)): one warp per head vector; the warps past the
// q and k heads copy the v heads.
template <typename T>
__global__ void qk_norm_rope_cache_kernel(
    T* __restrict__ q, long long q_stride, T* __restrict__ k, long long k_stride,
    const T* __restrict__ v, long long v_stride, int H, int Hkv, int dh,
    const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps,
    const float* __restrict__ rope, int rot,
    const int* __restrict__ slots, T* __restrict__ k_cache, T* __restrict__ v_cache,
    int page_size) {
    extern __shared__ float smem[];
    pdl_wait();
    pdl_launch();
    const int t = blockIdx.x;
    const int half = rot / 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hh = blockIdx.y * QKR_WARPS + warp;
    const int nk = k ? Hkv : 0, nv = v ? Hkv : 0;
    if (hh >= H + nk + nv) return;
    float* buf = smem + warp * dh;
    const float* cs = rope ? rope + (size_t)t * rot : nullptr;   // [half] cos, [half] sin
    const int slot = slots ? slots[t] : -1;
    const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
    if (hh >= H + nk) {                                          // a v head: copy to its slot
        const int head = hh - H - nk;
        if (slot < 0) return;
        const T* src = v + (size_t)t * v_stride + (size_t)head * dh;
        T* dst = v_cache + (((size_t)page * Hkv + head) * page_size + off) * dh;
        for (int i = lane; i < dh; i += 32) dst[i] = src[i];
        return;
    }
    const bool is_q = hh < H;
    const int head = is_q ? hh : hh - H;
    T* vec = is_q ? q + (size_t)t * q_stride + (size_t)head * dh
                  : k + (size_t)t * k_stride + (size_t)head * dh;
    const float* gain = is_q ? q_gain : k_gain;
    float ss = 0.f;
    for (int i = lane; i < dh; i += 32) {
        const float x = to_f32(vec[i]);
        buf[i] = x;
        ss += x * x;
    }
    if (gain) {
        ss = warp_sum(ss);
        const float scale = rsqrtf(ss / (float)dh + eps);
        for (int i = lane; i < dh; i += 32) buf[i] = (buf[i] * scale) * gain[i];
    }
    __syncwarp();
    T* dst = vec;
    if (!is_q && k_cache) {
        dst = slot >= 0 ? k_cache + (((size_t)page * Hkv + head) * page_size + off) * dh : nullptr;
    }
    if (!dst) return;
    for (int i = lane; i < dh; i += 32) {
        float y;
        if (cs && i < half)
            y = buf[i] * cs[i] - buf[i + half] * cs[half + i];
        else if (cs && i < rot)
            y = buf[i - half] * cs[i] + buf[i] * cs[i - half];
        else
            y = buf[i];
        dst[i] = from_f32<T>(y);
    }
}

// The same for head_dim 128 with the whole head rotated (or none of it): each lane holds four
// consecutive channels (one 8- or 16-byte access), the partner channel i +- 64 sits in lane
// +- 16, and nothing goes through shared memory.
template <typename T> struct Vec4;
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float (&x)[4]) {
        const uint2 v = *(const uint2*)p;
        const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&v.x);
        const float2 b = __bfloat1622float2(*(const __nv_bfloat162*)&v.y);
        x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&x)[4]) {
        __nv_bfloat162 a = __floats2bfloat162_rn(x[0], x[1]), b = __floats2bfloat162_rn(x[2], x[3]);
        uint2 v;
        v.x = *(uint32_t*)&a;
        v.y = *(uint32_t*)&b;
        *(uint2*)p = v;
    }
};
template <> struct Vec4<float> {
    static __device__ __forceinline__ void load(const float* p, float (&x)[4]) {
        const float4 v = *(const float4*)p;
        x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&x)[4]) {
        *(float4*)p = make_float4(x[0], x[1], x[2], x[3]);
    }
};

template <typename T>
__global__ void qk_norm_rope_cache_dh128_kernel(
    T* __restrict__ q, long long q_stride, T* __restrict__ k, long long k_stride,
    const T* __restrict__ v, long long v_stride, int H, int Hkv,
    const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps,
    const float* __restrict__ rope, const int* __restrict__ slots, T* __restrict__ k_cache,
    T* __restrict__ v_cache, int page_size) {
    constexpr int dh = 128;
    pdl_wait();
    pdl_launch();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hh = blockIdx.y * QKR_WARPS + warp;
    const int nk = k ? Hkv : 0, nv = v ? Hkv : 0;
    if (hh >= H + nk + nv) return;
    const int slot = slots ? slots[t] : -1;
    const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
    float x[4];
    if (hh >= H + nk) {
        const int head = hh - H - nk;
        if (slot < 0) return;
        Vec4<T>::load(v + (size_t)t * v_stride + (size_t)head * dh + 4 * lane, x);
        Vec4<T>::store(v_cache + (((size_t)page * Hkv + head) * page_size + off) * dh + 4 * lane, x);
        return;
    }
    const bool is_q = hh < H;
    const int head = is_q ? hh : hh - H;
    T* vec = is_q ? q + (size_t)t * q_stride + (size_t)head * dh : k + (size_t)t * k_stride + (size_t)head * dh;
    const float* gain = is_q ? q_gain : k_gain;
    Vec4<T>::load(vec + 4 * lane, x);
    if (gain) {
        float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
        ss = warp_sum(ss);
        const float scale = rsqrtf(ss / (float)dh + eps);
        const float4 g = *(const float4*)(gain + 4 * lane);
        x[0] = (x[0] * scale) * g.x; x[1] = (x[1] * scale) * g.y;
        x[2] = (x[2] * scale) * g.z; x[3] = (x[3] * scale) * g.w;
    }
    if (rope) {
        // channels 4*lane .. +3; lanes 0..15 hold the low half, their partners are 16 lanes on
        const float* cs = rope + (size_t)t * dh;              // [64] cos, [64] sin
        const int i0 = 4 * (lane & 15);
        const float4 c = *(const float4*)(cs + i0), sn = *(const float4*)(cs + 64 + i0);
        const float cc[4] = {c.x, c.y, c.z, c.w}, sv[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float other = __shfl_xor_sync(0xffffffffu, x[e], 16);
            x[e] = lane < 16 ? x[e] * cc[e] - other * sv[e] : other * sv[e] + x[e] * cc[e];
        }
    }
    T* dst = vec;
    if (!is_q && k_cache)
        dst = slot >= 0 ? k_cache + (((size_t)page * Hkv + head) * page_size + off) * dh : nullptr;
    if (dst) Vec4<T>::store(dst + 4 * lane, x);
}

// The same for many tokens of bfloat16 with head size 128 (a prompt portion): one CTA per
// token, half a warp per head vector with 16-byte accesses (lane l of the half holds channels
// 8l .. 8l+7, its rotation partner is 8 lanes on), the CTA's 16 half-warps walk the token's
// q, k and v heads.
#define QKW_WARPS 8
__global__ void __launch_bounds__(QKW_WARPS * 32)
qk_norm_rope_cache_dh128_wide_kernel(
    bf16* __restrict__ q, long long q_stride, bf16* __restrict__ k, long long k_stride,
    const bf16* __restrict__ v, long long v_stride, int H, int Hkv,
    const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps,
    const float* __restrict__ rope, const int* __restrict__ slots, bf16* __restrict__ k_cache,
    bf16* __restrict__ v_cache, int page_size) {
    constexpr int dh = 128;
    pdl_wait();
    pdl_launch();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, hl = lane & 15;
    const int half_id = threadIdx.x >> 4;                    // 0 .. 15
    const int nk = k ? Hkv : 0, nv = v ? Hkv : 0;
    const int total = H + nk + nv;
    const int slot = slots ? slots[t] : -1;
    const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
    // the token's cos and sin for this lane's channels (the low and the high half share them)
    float cc[8], sv[8];
    if (rope) {
        const float* cs = rope + (size_t)t * dh;              // [64] cos, [64] sin
        const int i0 = 8 * (hl & 7);
        const float4 c0 = *(const float4*)(cs + i0), c1 = *(const float4*)(cs + i0 + 4);
        const float4 s0 = *(const float4*)(cs + 64 + i0), s1 = *(const float4*)(cs + 64 + i0 + 4);
        cc[0] = c0.x; cc[1] = c0.y; cc[2] = c0.z; cc[3] = c0.w; cc[4] = c1.x; cc[5] = c1.y; cc[6] = c1.z; cc[7] = c1.w;
        sv[0] = s0.x; sv[1] = s0.y; sv[2] = s0.z; sv[3] = s0.w; sv[4] = s1.x; sv[5] = s1.y; sv[6] = s1.z; sv[7] = s1.w;
    }
    // every half-warp runs the same number of rounds, so that the shuffles below are complete
    const int rounds = (total + 15) / 16;
    // the vector of round r for this half-warp: read one round ahead of its use
    auto fetch = [&](int r) {
        const int hh = r * 16 + half_id;
        if (hh >= total) return make_uint4(0u, 0u, 0u, 0u);
        const bf16* src = hh < H ? q + (size_t)t * q_stride + (size_t)hh * dh
                          : hh >= H + nk ? v + (size_t)t * v_stride + (size_t)(hh - H - nk) * dh
                                         : k + (size_t)t * k_stride + (size_t)(hh - H) * dh;
        return *(const uint4*)(src + 8 * hl);
    };
    uint4 ahead = fetch(0);
    for (int r = 0; r < rounds; ++r) {
        const int hh = r * 16 + half_id;
        const bool live = hh < total;
        const bool is_v = live && hh >= H + nk;
        const bool is_q = live && hh < H;
        const int head = !live ? 0 : is_q ? hh : is_v ? hh - H - nk : hh - H;
        const uint4 raw = ahead;
        if (r + 1 < rounds) ahead = fetch(r + 1);
        if (is_v) {
            if (slot >= 0) *(uint4*)(v_cache + (((size_t)page * Hkv + head) * page_size + off) * dh + 8 * hl) = raw;
            continue;                                        // no shuffles on this path ...
        }
        // ... but a half-warp of v and a half-warp of q or k may share a warp: the shuffles
        // below stay inside the half-warp and name only its lanes
        const unsigned mask = 0xffffu << (lane & 16);
        float x[8];
        {
            const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&raw.x), b = __bfloat1622float2(*(const __nv_bfloat162*)&raw.y);
            const float2 c = __bfloat1622float2(*(const __nv_bfloat162*)&raw.z), d = __bfloat1622float2(*(const __nv_bfloat162*)&raw.w);
            x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y; x[4] = c.x; x[5] = c.y; x[6] = d.x; x[7] = d.y;
        }
        const float* gain = is_q ? q_gain : k_gain;
        if (gain) {
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(mask, ss, o);      // within the half-warp
            const float scale = rsqrtf(ss / (float)dh + eps);
            const float4 g0 = *(const float4*)(gain + 8 * hl), g1 = *(const float4*)(gain + 8 * hl + 4);
            x[0] = (x[0] * scale) * g0.x; x[1] = (x[1] * scale) * g0.y; x[2] = (x[2] * scale) * g0.z; x[3] = (x[3] * scale) * g0.w;
            x[4] = (x[4] * scale) * g1.x; x[5] = (x[5] * scale) * g1.y; x[6] = (x[6] * scale) * g1.z; x[7] = (x[7] * scale) * g1.w;
        }
        if (rope) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float other = __shfl_xor_sync(mask, x[e], 8);
                x[e] = hl < 8 ? x[e] * cc[e] - other * sv[e] : other * sv[e] + x[e] * cc[e];
            }
        }
        if (!live) continue;
        uint4 o4;
        { __nv_bfloat162 p0 = __floats2bfloat162_rn(x[0], x[1]), p1 = __floats2bfloat162_rn(x[2], x[3]);
          __nv_bfloat162 p2 = __floats2bfloat162_rn(x[4], x[5]), p3 = __floats2bfloat162_rn(x[6], x[7]);
          o4.x = *(uint32_t*)&p0; o4.y = *(uint32_t*)&p1; o4.z = *(uint32_t*)&p2; o4.w = *(uint32_t*)&p3; }
        bf16* dst = is_q ? q + (size_t)t * q_stride + (size_t)head * dh : k + (size_t)t * k_stride + (size_t)head * dh;
        if (!is_q && k_cache)
            dst = slot >= 0 ? k_cache + (((size_t)page * Hkv + head) * page_size + off) * dh : nullptr;
        if (dst) *(uint4*)(dst + 8 * hl) = o4;
    }
}

TGO_API int tgo_qk_norm_rope_cache(void* q, long long q_stride, void* k, long long k_stride,
                                   const void* v, long long v_stride, int dtype, int T, int H,
                                   int Hkv, int dh, const float* q_gain, const float* k_gain,
                                   float eps, const float* rope, int rot, const int* slots,
                                   void* k_cache, void* v_cache, int page_size,
                                   cudaStream_t stream) {
    if (T <= 0) return 0;
    if (dh <= 0 || dh > QKR_MAX_DH || rot < 0 || rot > dh || (rot & 1) || H <= 0) return TGO_E_BAD_ARG;
    if ((k || v) && Hkv <= 0) return TGO_E_BAD_ARG;
    if ((k_cache || v) && (page_size <= 0 || !slots)) return TGO_E_BAD_ARG;
    if ((v && !v_cache) || (k_cache && !k)) return TGO_E_BAD_ARG;
    const int warps = QKR_WARPS;
    const size_t smem = (size_t)(warps * dh) * sizeof(float);
    const int vectors = H + (k ? Hkv : 0) + (v ? Hkv : 0);
    const dim3 grid(T, (vectors + warps - 1) / warps);
    const int esz = dtype == TGO_BF16 ? 2 : 4;
    const bool aligned = ((uintptr_t)q * 1 % 16 == 0) && (q_stride * esz) % 16 == 0 &&
                         (!k || (((uintptr_t)k % 16 == 0) && (k_stride * esz) % 16 == 0)) &&
                         (!v || (((uintptr_t)v % 16 == 0) && (v_stride * esz) % 16 == 0));
    if (dh == 128 && (rot == 128 || !rope) && aligned && dtype == TGO_BF16 && T >= 64)
        return tgo_launch_pdl(qk_norm_rope_cache_dh128_wide_kernel, dim3(T), dim3(QKW_WARPS * 32), 0, stream,
                              (bf16*)q, q_stride, (bf16*)k, k_stride, (const bf16*)v, v_stride, H, Hkv,
                              q_gain, k_gain, eps, rope, slots, (bf16*)k_cache, (bf16*)v_cache, page_size);
    if (dh == 128 && (rot == 128 || !rope) && aligned && (dtype == TGO_BF16 || dtype == TGO_F32)) {
        if (dtype == TGO_BF16)
            return tgo_launch_pdl(qk_norm_rope_cache_dh128_kernel<bf16>, grid, dim3(warps * 32), 0, stream,
                                  (bf16*)q, q_stride, (bf16*)k, k_stride, (const bf16*)v, v_stride, H, Hkv,
                                  q_gain, k_gain, eps, rope, slots, (bf16*)k_cache, (bf16*)v_cache, page_size);
        return tgo_launch_pdl(qk_norm_rope_cache_dh128_kernel<float>, grid, dim3(warps * 32), 0, stream,
                              (float*)q, q_stride, (float*)k, k_stride, (const float*)v, v_stride, H, Hkv,
                              q_gain, k_gain, eps, rope, slots, (float*)k_cache, (float*)v_cache, page_size);
    }
    if (dtype == TGO_BF16)
        return tgo_launch_pdl(qk_norm_rope_cache_kernel<bf16>, grid, dim3(warps * 32), smem, stream,
            (bf16*)q, q_stride, (bf16*)k, k_stride, (const bf16*)v, v_stride, H, Hkv, dh, q_gain,
            k_gain, eps, rope, rot, slots, (bf16*)k_cache, (bf16*)v_cache, page_size);
    else if (dtype == TGO_F32)
        return tgo_launch_pdl(qk_norm_rope_cache_kernel<float>, grid, dim3(warps * 32), smem, stream,
            (float*)q, q_stride, (float*)k, k_stride, (const float*)v, v_stride, H, Hkv, dh,
            q_gain, k_gain, eps, rope, rot, slots, (float*)k_cache, (float*)v_cache, page_size);
    else
        return TGO_E_BAD_ARG;
    return launch_status();
}
