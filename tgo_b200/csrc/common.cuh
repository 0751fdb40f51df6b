// Shared helpers of the sm_100a kernels: storage types, warp and block reductions.
// Every kernel entry point is extern "C", takes raw device pointers and a stream,
// and returns the cudaError_t of its launch as an int; nothing here allocates.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define TGO_API extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python side
#define TGO_F32 0
#define TGO_BF16 1

#define TGO_E_BAD_ARG 1000   // returned (not a CUDA code) when a size is refused

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(bf16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` is 33 floats of shared memory. The order of the additions depends only
// on the block size, never on the data, so equal inputs give equal sums.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

static inline int launch_status() { return (int)cudaGetLastError(); }

// ---- programmatic dependent launch
// Kernels of a decode step are short; launched this way the next kernel's blocks are
// scheduled while the previous kernel drains, and wait at pdl_wait() until it has completed
// and its writes are visible. Every kernel launched through tgo_launch_pdl calls pdl_wait()
// first thing, in every thread, before it reads or writes global memory, so the chain of
// dependencies stays what stream order would give. TGO_NO_PDL=1 turns the attribute off.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Letting dependents launch from the top of a kernel (pdl_launch) was measured slower on
// B200 in every variant tried (all kernels; only the small ones): it is compiled out unless
// TGO_PDL_TRIGGER=1. Kernels that fill the GPU call pdl_launch_late() once a block has
// finished its streaming loop. What does help: a matrix product issues its first weight
// loads, which depend on nothing, before its pdl_wait().
#ifndef TGO_PDL_TRIGGER
#define TGO_PDL_TRIGGER 0
#endif
#ifndef TGO_PDL_TRIGGER_LATE
#define TGO_PDL_TRIGGER_LATE 1
#endif
__device__ __forceinline__ void pdl_launch() {
#if TGO_PDL_TRIGGER
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}
__device__ __forceinline__ void pdl_launch_late() {
#if TGO_PDL_TRIGGER_LATE
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}

#include <stdlib.h>
static inline bool tgo_pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("TGO_NO_PDL");
        on = (e && e[0] == '1') ? 0 : 1;
    }
    return on == 1;
}

template <typename... KArgs, typename... Args>
static inline int tgo_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tgo_pdl_enabled() ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
