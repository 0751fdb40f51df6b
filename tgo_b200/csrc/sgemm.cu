// y[M,N] = x[M,K] . w[N,K]^T in true float32: plain FMA, no tensor cores, no reduced-
// precision mode. Every output element is one running sum over k = 0..K-1 in that order,
// whatever tile it falls in, so a row's result does not depend on which other rows are in
// the batch. This is the matrix product of the float32 path of the whole model.
#include "common.cuh"

#define SG_BM 64
#define SG_BN 64
#define SG_BK 16

__global__ void __launch_bounds__(256)
sgemm_tn_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y,
                int M, int N, int K) {
    __shared__ float xs[SG_BK][SG_BM + 4];
    __shared__ float ws[SG_BK][SG_BN + 4];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int m0 = blockIdx.y * SG_BM, n0 = blockIdx.x * SG_BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += SG_BK) {
        // 64 rows x 16 k per operand = 1024 values, 4 per thread
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int idx = threadIdx.x + r * 256;
            const int row = idx / SG_BK, kk = idx % SG_BK;
            const int gm = m0 + row, gn = n0 + row, gk = k0 + kk;
            xs[kk][row] = (gm < M && gk < K) ? x[(size_t)gm * K + gk] : 0.f;
            ws[kk][row] = (gn < N && gk < K) ? w[(size_t)gn * K + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < SG_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) y[(size_t)gm * N + gn] = acc[i][j];
        }
    }
}

TGO_API int tgo_sgemm_tn(const float* x, const float* w, float* y, int M, int N, int K,
                         cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return TGO_E_BAD_ARG;
    const dim3 grid((N + SG_BN - 1) / SG_BN, (M + SG_BM - 1) / SG_BM);
    if (grid.y > 65535) return TGO_E_BAD_ARG;
    sgemm_tn_kernel<<<grid, 256, 0, stream>>>(x, w, y, M, N, K);
    return launch_status();
}
