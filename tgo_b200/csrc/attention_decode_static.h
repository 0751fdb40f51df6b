// tgo_attention_decode_static: split-key decode attention that allocates nothing.
//
// This entry point has no counterpart in the reference (latere-ai/tgo has no device code
// and leaves scratch memory to its external tensor runtime).
//
// Who it is for. The ordinary entry point, tgo_attention_flash, takes its scratch buffers
// (the partial outputs of the key splits) from the caller, and the Python wrapper gets
// them from torch's allocator on every call. Some callers cannot do that:
//   * a host program that has handed the whole device to another memory manager, or runs
//     under a fixed memory budget, so that cudaMalloc after start-up fails or is forbidden;
//   * a latency-bound serving loop: cudaMalloc and cudaFree synchronise the whole device,
//     which stalls every stream for the sake of a few megabytes;
//   * code that links this library from C and has no tensor allocator at all.
// For them the scratch lives in a file-scope `static __device__` array inside the library,
// TGO_DECODE_STATIC_SCRATCH_FLOATS floats (8 MiB) on every GPU that loads the library, held
// until the process exits. The caller still passes inputs and outputs.
//
// Rules.
//   * Sizes: tokens * heads * n_splits * (head_dim + 2) floats must fit the array; a larger
//     request is refused with TGO_E_SCRATCH_TOO_SMALL (1001) and nothing is launched.
//     Unsupported head sizes or groups are refused with 1000, as by tgo_attention_flash.
//   * The first call on a device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and remembers it. Make that first
//     call outside any stream capture.
//   * It calls no cudaMalloc, cudaFree or other allocating routine.
//   * All calls share the one array and it keeps what the last call left there. Nothing in
//     it has to start at zero: every slot that is read was written earlier in the same call.
//     Two calls whose kernels overlap on the GPU (different streams) race on it; issue
//     calls on one stream, or order them yourself.
#pragma once
#include <cuda_runtime.h>

#define TGO_DECODE_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define TGO_E_SCRATCH_TOO_SMALL 1001

#ifdef __cplusplus
extern "C" {
#endif

// One token per request (decode). q: [T, >= H*dh] bfloat16 rows of stride q_stride elements;
// out likewise; k_cache, v_cache: one layer's pages [page][kv_head][page_size][dh] bfloat16;
// block_tables: int32 [requests, max_blocks]; positions, seq_ids: int32 [T] (position < 0:
// the row reads nothing and its output is zero). window 0: every earlier key. n_splits >= 1
// CTAs share each request's keys. Returns 0, a cudaError_t, 1000 or 1001.
__attribute__((visibility("default")))
int tgo_attention_decode_static(const void* q, long long q_stride, void* out, long long out_stride,
                                const void* k_cache, const void* v_cache, int page_size,
                                const int* block_tables, int max_blocks, const int* positions,
                                const int* seq_ids, int T, int H, int Hkv, int dh, float scale,
                                int window, int n_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
