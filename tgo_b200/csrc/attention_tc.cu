// Paged causal attention for prompt portions on the tcgen05 tensor cores (head size 128,
// bfloat16): S = Q K^T and O += P V are tcgen05.mma with the accumulators in tensor memory,
// Q, K and V come in by TMA, and the softmax runs in registers between the two products.
//
// A work item is one tile of 128 query rows and one kv head: the G query heads that share the
// kv head, for 128 / G consecutive tokens of one request (row r = token r / G, head r % G), so
// K and V are read once for the whole group. An item walks the request's keys in tiles of 128.
// One persistent CTA per SM draws items from a counter (see the kernel below for its warps).
//
// The softmax: two threads per row, one for keys 0..63 of the tile and one for keys 64..127.
// Each reads its half row of S (64 float32), masks, takes the maximum, swaps it with its
// partner through shared memory, writes P = exp2(S * scale - m) as bfloat16 over the first
// half of the S buffer, and keeps its part of the row sum. The running maximum is only moved
// when some row of the warp has grown by more than 2^8 since it was set; then the rows of O
// in tensor memory are rescaled. (The result is the same: the factor cancels in O / l; only
// the range of P changes, and 2^8 is far from overflow.)
//
// Rows of V that no query may read (past the request's end in its last page, before the
// window) are zeroed in shared memory before P V: P is zero there, but the cache may hold
// anything, NaN included. Keys of K in such rows give S values that the mask replaces.
//
// MEASURED on B200, 2048-token prompt of 32/8 heads (CUDA events, warm): 262 us for the
// mma.sync kernel this replaced; 136 us for one CTA per item with two S buffers and one softmax
// thread per row; 100 us with two threads per row; 91 us with two such CTAs per SM; 78 us
// persistent with everything double-buffered; 74.5 us with items drawn only when there is
// room for them; 65 us with Q by TMA (529 TFLOP/s; an 8192-token prompt 608 us, 904 TFLOP/s).
// Timed inside the kernel with the global timer on that prompt: a key tile takes 1.45 us
// (the special-function unit alone needs 1024 cycles, 0.53 us, for a tile's 128 x 128
// exponentials, as long as its two products take), an item 2.5 us more (0.4 us to its first
// S, 0.5 us for its last product, 1.6 us to scale and store O). Tried and not kept: a cubic
// on the FMA pipe for every second or fourth exponential (issue-bound: 81.5 and 76.9 us
// against 77.6); two softmax groups of four warps with an S and an O each (107 us); three S
// buffers and one O buffer, so that Q K^T may run two key tiles ahead (66.5 us against 65.6,
// 614 us against 614 at 8192 tokens: the softmax threads do not wait for the products); four
// softmax threads a row, 32 keys each, sixteen softmax warps (68.5 us against 66.2, 651 against
// 612 at 8192 tokens: nor do they lack warps to hide their own latency).
//
// Every wait has a time limit (about two seconds): it records a code, the CTA stops issuing,
// frees its tensor memory and returns. No cluster, no multicast.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

#define AT_BM 128
#define AT_BN 128
#define AT_DH 128
#define AT_WAIT_CYCLES 4000000000ll
#define AT_BLOCK_BYTES (128 * 64 * 2)          // 128 rows x 64 columns of bf16
#define AT_TILE_BYTES (2 * AT_BLOCK_BYTES)     // a Q, K or V tile: two column halves
#define AT_PAGES_CAP 1024
#ifndef AP_PV_N
#define AP_PV_N 128      // output columns of one P V product: 128, or 64 (two products a k-step)
#endif
#ifndef AP_LBO_BYTES
#define AP_LBO_BYTES AT_BLOCK_BYTES
#endif

__device__ int at_error_flag = 0;

__device__ __forceinline__ uint32_t at_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void at_mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(at_smem(bar)), "r"(count));
}
__device__ __forceinline__ void at_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(at_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void at_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(at_smem(bar)) : "memory");
}
__device__ __forceinline__ bool at_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(at_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool at_wait(uint64_t* bar, uint32_t parity, int code) {
    if (at_try(bar, parity)) return true;
    const long long start = clock64();
    while (!at_try(bar, parity)) {
        if (clock64() - start > AT_WAIT_CYCLES) {
            atomicExch(&at_error_flag, code);
            return false;
        }
    }
    return true;
}
// A box of the query rows: coordinates (column in the half, half, head, token)
__device__ __forceinline__ void at_tma_4d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(at_smem(dst)), "l"(map), "r"(at_smem(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void at_tma_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(at_smem(dst)), "l"(map), "r"(at_smem(bar)), "r"(x), "r"(y) : "memory");
}
// operands in shared memory -> accumulator in tensor memory
__device__ __forceinline__ void at_mma_ss(uint32_t d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
// A in tensor memory, B in shared memory
__device__ __forceinline__ void at_mma_ts(uint32_t d, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void at_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(at_smem(bar)) : "memory");
}
__device__ __forceinline__ void at_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void at_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory operand descriptor, rows of 128 bytes with the 128-byte swizzle, groups of 8
// rows 1024 bytes apart. For a K-major operand the rows are the M or N index; for an MN-major
// one (V) the rows are the k index and the 64 columns one block of N. Both offsets hold the
// distance between 8-row groups: whichever the unit takes for that direction, it is right,
// and the other direction has extent one.
__device__ __forceinline__ uint64_t at_desc(const void* tile) {
    uint64_t d = (uint64_t)((at_smem(tile) & 0x3ffff) >> 4);
    d |= (uint64_t)(1024 >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// The same for V when one product spans both 64-column blocks: the second block of columns
// lies AP_LBO_BYTES after the first.
__device__ __forceinline__ uint64_t at_desc_mn(const void* tile) {
    uint64_t d = (uint64_t)((at_smem(tile) & 0x3ffff) >> 4);
    d |= (uint64_t)((AP_PV_N == 128 ? AP_LBO_BYTES : 1024) >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ void at_tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
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
__device__ __forceinline__ void at_tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
          "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
          "r"(r[30]), "r"(r[31]), "r"(taddr)
        : "memory");
}
// Barrier 1 of the 256 softmax threads; every thread gets the OR of the predicates.
__device__ __forceinline__ bool at_bar_or(bool pred) {
    uint32_t r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\t"
                 "bar.red.or.pred q, 1, 256, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                 : "=r"(r) : "r"((uint32_t)pred) : "memory");
    return r != 0;
}
// 2^x on the special-function unit; -inf gives 0
__device__ __forceinline__ float at_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t at_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(uint32_t*)&v;
}

// ------------------------------------------------------------------ persistent form
// One CTA per SM walks work items (query tile, kv head) that it draws from a counter, longest
// first. Inside the CTA everything is double-buffered, so the parts of neighbouring key tiles
// and of neighbouring items overlap:
//   tensor memory (512 columns)  S0, S1 (128 each; P lies over S) and O0, O1 (128 each): the
//                 issuer runs Q K^T one key tile ahead of the softmax, and starts the next
//                 item while the softmax threads still write the last one's O out;
//   shared memory  two Q tiles, two K tiles, two V tiles (192 KB);
//   warp 0   draws an item when a Q buffer is free, reads its sizes, asks TMA for its Q rows
//            (two boxes) and publishes a record of the item in a ring of four;
//   warps 12 and 10  follow the records and ask TMA for the K and for the V pages, a warp
//            each, so that K runs ahead of V and neither waits for the next item's Q;
//   warps 1 and 11  issue S = Q K^T and O += P V, a thread each (a thread starts a product
//            about every 80 cycles); warps 2-9 softmax, two threads a row, as above.
// The counter is a global of this library (one per device): launches of this kernel on one
// device must not overlap (the engine issues them on one stream).
// A record (and its Q buffer) is only replaced when every reader has seen it: the products
// with the item's Q have run, and the second issuer, the K and V warps and the eight softmax
// warps have each read the record; so no waiter ever falls two phases behind a barrier.
#define AP_THREADS 416

struct ApItem {          // what warp 0 tells the others about an item
    int valid;           // 0: no more items
    int tok0, n_rows, p0, n_it, t_lo, key_lo, key_hi, seq, kvh;
    int pad[6];
};

// The counter the CTAs draw items from, and the count of CTAs that have finished: the last
// CTA of a launch to finish sets both back to zero for the next launch (every CTA reaches its
// end, whatever its waits did).
__device__ unsigned int ap_ticket = 0;
__device__ unsigned int ap_finished = 0;

__global__ void __launch_bounds__(AP_THREADS, 1)
attention_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                               const __grid_constant__ CUtensorMap map_q, bf16* __restrict__ out,
                               long long out_stride, int page_size, int page_shift,
                               const int* __restrict__ block_tables, int max_blocks,
                               const int* __restrict__ positions, const int* __restrict__ seq_ids,
                               const int* __restrict__ tile_tok0, const int* __restrict__ tile_ntok,
                               int n_tiles, int H, int Hkv, float scale_log2, int window) {
    extern __shared__ unsigned char at_raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)at_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* sQ = base;                                   // [2][2 halves][128 rows][128 B]
    unsigned char* sK = sQ + 2 * AT_TILE_BYTES;                 // [2 stages]
    unsigned char* sV = sK + 2 * AT_TILE_BYTES;                 // [2 stages]
    uint64_t* bars = (uint64_t*)(sV + 2 * AT_TILE_BYTES);
    uint64_t* q_full = bars;            // [2]
    uint64_t* q_empty = bars + 2;       // [2]
    uint64_t* k_full = bars + 4;        // [2]
    uint64_t* k_empty = bars + 6;       // [2]
    uint64_t* v_full = bars + 8;        // [2]
    uint64_t* v_empty = bars + 10;      // [2]
    uint64_t* s_full = bars + 12;       // [2]
    uint64_t* p_full = bars + 14;       // [2]
    uint64_t* o_free = bars + 16;       // [2]
    uint64_t* o_done = bars + 18;       // [1]
    uint64_t* p_free = bars + 19;       // [2]
    uint32_t* tmem_slot = (uint32_t*)(bars + 21);
    ApItem* ring = (ApItem*)(bars + 22);                        // [4]
    float* s_xm = (float*)(ring + 4);   // [2][2 halves][128 rows]
    float* s_xl = s_xm + 512;           // [2 halves][128 rows]
    int* s_pages_k = (int*)(s_xl + 256);          // [AT_PAGES_CAP]
    int* s_pages_v = s_pages_k + AT_PAGES_CAP;    // [AT_PAGES_CAP]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = H / Hkv;
    const int n_items = n_tiles * Hkv;
    const int pages_per_tile = AT_BN >> page_shift;
    const int q_box_rows = (AT_BM / G) * G;       // rows of a Q box: the tokens of a full tile x G heads
    // rows of the Q buffers that no box writes (128 is no multiple of G) must not hold NaN
    // bit patterns by chance: zero both buffers once
    for (int i = tid; i < 2 * AT_TILE_BYTES / 16; i += AP_THREADS) ((uint4*)sQ)[i] = make_uint4(0u, 0u, 0u, 0u);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");

    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            at_mbar_init(&q_full[i], 1); at_mbar_init(&q_empty[i], 12);
            at_mbar_init(&k_full[i], 1); at_mbar_init(&k_empty[i], 1);
            at_mbar_init(&v_full[i], 1); at_mbar_init(&v_empty[i], 1);
            at_mbar_init(&s_full[i], 1); at_mbar_init(&p_full[i], 8);
            at_mbar_init(&o_free[i], 8); at_mbar_init(&p_free[i], 1);
        }
        at_mbar_init(o_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(at_smem(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    at_fence_before();
    __syncthreads();
    at_fence_after();
    const uint32_t tmem = *tmem_slot;

    // pages of key tile j that hold a key some row of the item may read: [first, last)
    auto page_range = [&](int j, int key_lo, int key_hi, int& first, int& last) {
        first = j * pages_per_tile;
        last = first + pages_per_tile;
        while (first < last && (first + 1) * page_size <= key_lo) ++first;
        while (last > first && (last - 1) * page_size >= key_hi) --last;
    };

    if (warp == 0) {
        // ---------------------------------------------------------- items and Q
        bool ok = true;
        auto draw = [&](int& item, int& tok0, int& ntok) {
            item = 0;
            if (lane == 0) item = (int)atomicAdd(&ap_ticket, 1u);
            item = __shfl_sync(0xffffffffu, item, 0);
            tok0 = ntok = 0;
            if (item < n_items) {
                const int tile = n_tiles - 1 - item / Hkv;      // longest first: later tiles read more keys
                tok0 = tile_tok0[tile];
                ntok = tile_ntok[tile];
            }
        };
        int item, tok0, ntok;
        for (uint32_t n = 0; ok; ++n) {
            ApItem* rec = &ring[n & 3];
            const uint32_t qb = n & 1u, qph = (n >> 1) & 1u;
            // the Q buffer (and with it the turn to publish) is free once the products of the
            // item two back have run and everybody has read its record
            ok = __all_sync(0xffffffffu, at_wait(&q_empty[qb], qph ^ 1u, 1));
            if (!ok) break;
            // An item is drawn only now, when the CTA has room for it: the CTA then holds the
            // item it computes and the one it loads, and no third. (Drawn one turn earlier, as
            // this kernel did at first, two items lay reserved behind the running one; with
            // three or four items a CTA on a 2048-token prompt that is nearly a fixed share
            // each: the CTAs' loads ranged from 24 to 35 key tiles, and the last CTA ended
            // 11 us after the median one, of 61.)
            draw(item, tok0, ntok);
            if (item >= n_items) {
                if (lane == 0) {
                    rec->valid = 0;
                    at_arrive(&q_full[qb]);
                }
                break;
            }
            const int kvh = item % Hkv;
            const int n_rows = ntok * G;
            const int p0 = positions[tok0], seq = seq_ids[tok0];
            const int q_tok0 = tok0;
            const int p_last = p0 + ntok - 1;
            const int key_lo = (window > 0 && p0 - window + 1 > 0) ? p0 - window + 1 : 0;
            const int key_hi = p_last + 1;
            const int t_lo = key_lo / AT_BN, t_hi = (key_hi + AT_BN - 1) / AT_BN;
            const int n_it = p0 < 0 ? 0 : t_hi - t_lo;
            if (lane == 0) {
                rec->valid = 1; rec->tok0 = q_tok0; rec->n_rows = n_rows; rec->p0 = p0; rec->n_it = n_it;
                rec->t_lo = t_lo; rec->key_lo = key_lo; rec->key_hi = key_hi; rec->seq = seq; rec->kvh = kvh;
                if (n_it > 0) {
                    // The item's Q rows by TMA: two boxes (the two 64-column halves of the head
                    // size) of G heads x the tile's tokens, which land in row order token * G +
                    // head with the 128-byte swizzle the products read. A box always spans a full
                    // tile's tokens: tokens past this tile's are other tokens' rows (their results
                    // are never stored; rows are independent), tokens past the last are zeros.
                    // (Copied by this warp with 2048 16-byte cp.async, the rows of the first item
                    // took 8 us to arrive and those of later items 13 us, competing with the
                    // softmax warps for issue slots: measured with the global timer.)
                    unsigned char* dq = sQ + qb * AT_TILE_BYTES;
                    at_expect_tx(&q_full[qb], 2u * (uint32_t)q_box_rows * 128u);
                    at_tma_4d(dq, &map_q, 0, 0, kvh * G, q_tok0, &q_full[qb]);
                    at_tma_4d(dq + AT_BLOCK_BYTES, &map_q, 0, 1, kvh * G, q_tok0, &q_full[qb]);
                } else {
                    at_arrive(&q_full[qb]);
                }
            }
        }
    } else if (warp == 10 || warp == 12) {
        // ---------------------------------------------------------- V (warp 10), K (warp 12)
        const bool is_k = warp == 12;
        int* s_pages = is_k ? s_pages_k : s_pages_v;
        unsigned char* tiles = is_k ? sK : sV;
        uint64_t* full = is_k ? k_full : v_full;
        uint64_t* empty = is_k ? k_empty : v_empty;
        const CUtensorMap* map = is_k ? &map_k : &map_v;
        bool ok = true;
        uint32_t g = 0;
        for (uint32_t n = 0; ok; ++n) {
            const uint32_t qb = n & 1u, qph = (n >> 1) & 1u;
            ok = __all_sync(0xffffffffu, at_wait(&q_full[qb], qph, 1));
            if (!ok) break;
            const ApItem rec = ring[n & 3];
            if (!rec.valid) break;
            __syncwarp();
            if (lane == 0) at_arrive(&q_empty[qb]);
            const int* bt = block_tables + (size_t)rec.seq * max_blocks;
            const int pg_lo = rec.t_lo * pages_per_tile;
            if (rec.n_it > 0) {
                int pg_hi = (rec.t_lo + rec.n_it) * pages_per_tile;
                if (pg_hi > max_blocks) pg_hi = max_blocks;
                if (pg_hi - pg_lo > AT_PAGES_CAP) pg_hi = pg_lo + AT_PAGES_CAP;
                for (int i = pg_lo + lane; i < pg_hi; i += 32) s_pages[i - pg_lo] = bt[i];
            }
            __syncwarp();
            auto page_of = [&](int pi) { return pi - pg_lo < AT_PAGES_CAP ? s_pages[pi - pg_lo] : bt[pi]; };
            for (int it = 0; it < rec.n_it; ++it, ++g) {
                const uint32_t s = g & 1u, ph = (g >> 1) & 1u;
                const int j = rec.t_lo + it;
                int first, last;
                page_range(j, rec.key_lo, rec.key_hi, first, last);
                ok = __all_sync(0xffffffffu, at_wait(&empty[s], ph ^ 1u, 1));
                if (!ok) break;
                if (lane == 0) at_expect_tx(&full[s], (uint32_t)(last - first) * (uint32_t)page_size * 256u);
                __syncwarp();
                for (int pi = first + lane; pi < last; pi += 32) {
                    const int row = (page_of(pi) * Hkv + rec.kvh) * page_size;
                    unsigned char* dst = tiles + s * AT_TILE_BYTES + (pi - j * pages_per_tile) * page_size * 128;
                    at_tma_2d(dst, map, 0, row, &full[s]);
                    at_tma_2d(dst + AT_BLOCK_BYTES, map, 64, row, &full[s]);
                }
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------- issuer of S = Q K^T
        // (a thread can start a product about every 80 cycles, so the two kinds of product
        // have a thread each)
        if (lane == 0) {
            const uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 3) << 17) |
                                      ((uint32_t)(128 >> 4) << 24);
            uint32_t g = 0;
            bool ok = true;
            for (uint32_t n = 0; ok; ++n) {
                const uint32_t qb = n & 1u;
                if (!at_wait(&q_full[qb], (n >> 1) & 1u, 2)) break;
                const ApItem* rec = &ring[n & 3];
                if (!rec->valid) break;
                const int n_it = rec->n_it;
                const unsigned char* qt = sQ + qb * AT_TILE_BYTES;
                const uint64_t dq0 = at_desc(qt), dq1 = at_desc(qt + AT_BLOCK_BYTES);
                for (int it = 0; it < n_it; ++it, ++g) {
                    const uint32_t s = g & 1u, ph = (g >> 1) & 1u;
                    // K has landed, and the P that lay in this S buffer has been multiplied
                    ok = at_wait(&k_full[s], ph, 2) && at_wait(&p_free[s], ph ^ 1u, 2);
                    if (!ok) break;
                    at_fence_after();
                    const uint64_t dk0 = at_desc(sK + s * AT_TILE_BYTES), dk1 = at_desc(sK + s * AT_TILE_BYTES + AT_BLOCK_BYTES);
#pragma unroll
                    for (int k = 0; k < 4; ++k) at_mma_ss(tmem + 128u * s, dq0 + 2 * k, dk0 + 2 * k, idesc_qk, k > 0 ? 1u : 0u);
#pragma unroll
                    for (int k = 0; k < 4; ++k) at_mma_ss(tmem + 128u * s, dq1 + 2 * k, dk1 + 2 * k, idesc_qk, 1u);
                    at_commit(&k_empty[s]);
                    at_commit(&s_full[s]);
                }
                at_commit(&q_empty[qb]);               // the item's products with Q have run
            }
        }
    } else if (warp == 11) {
        // ---------------------------------------------------------- issuer of O += P V
        if (lane == 0) {
            const uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                                      ((uint32_t)(AP_PV_N >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
            uint32_t g = 0;
            bool ok = true;
            for (uint32_t n = 0; ok; ++n) {
                if (!at_wait(&q_full[n & 1u], (n >> 1) & 1u, 2)) break;
                const ApItem* rec = &ring[n & 3];
                if (!rec->valid) break;
                const int n_it = rec->n_it;
                at_arrive(&q_empty[n & 1u]);
                const uint32_t ob = n & 1u;
                const uint32_t tm_o = tmem + 256u + 128u * ob;
                for (int it = 0; it < n_it && ok; ++it, ++g) {
                    const uint32_t s = g & 1u, ph = (g >> 1) & 1u;
                    if (it == 0) ok = at_wait(&o_free[ob], ((n >> 1) & 1u) ^ 1u, 2);    // item n-2's O is out
                    ok = ok && at_wait(&p_full[s], ph, 2) && at_wait(&v_full[s], ph, 2);
                    if (!ok) break;
                    at_fence_after();
#pragma unroll
                    for (int h = 0; h < 128 / AP_PV_N; ++h) {
                        const uint64_t dv = at_desc_mn(sV + s * AT_TILE_BYTES + h * AT_BLOCK_BYTES);
#pragma unroll
                        for (int k = 0; k < 8; ++k)           // 16 keys = 2 groups of 8 rows = 2048 bytes
                            at_mma_ts(tm_o + 64u * h, tmem + 128u * s + 8u * k, dv + (uint64_t)(128 * k), idesc_pv,
                                      (it > 0 || k > 0) ? 1u : 0u);
                    }
                    at_commit(&v_empty[s]);
                    at_commit(&p_free[s]);
                    at_commit(o_done);
                }
            }
        }
    } else {
        // ---------------------------------------------------------- softmax
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const int row = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        bool ok = true;
        uint32_t g = 0;
        for (uint32_t n = 0;; ++n) {
            if (ok) ok = at_wait(&q_full[n & 1u], (n >> 1) & 1u, 3);
            if (at_bar_or(!ok)) break;             // a wait ran out somewhere: all 256 leave together
            const ApItem rec = ring[n & 3];
            if (!rec.valid) break;
            __syncwarp();
            if (lane == 0) at_arrive(&q_empty[n & 1u]);
            const uint32_t ob = n & 1u;
            const uint32_t tm_o = tmem + 256u + 128u * ob;
            const int n_rows = rec.n_rows, p0 = rec.p0, n_it = rec.n_it, key_lo = rec.key_lo, key_hi = rec.key_hi;
            const bool row_ok = row < n_rows;
            bf16* dst = out + (size_t)(rec.tok0 + (row_ok ? row : 0) / G) * out_stride +
                        (size_t)(rec.kvh * G + (row_ok ? row : 0) % G) * AT_DH + 64 * half;
            if (n_it == 0) {                       // a request that brings nothing: zeros out
                if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) *(uint4*)(dst + i * 8) = make_uint4(0u, 0u, 0u, 0u);
                }
                __syncwarp();
                if (lane == 0) at_arrive(&o_free[ob]);
                continue;
            }
            const int pos = row_ok ? p0 + row / G : -1;
            const int vis_lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
            const int warp_first = quarter * 32, warp_last = quarter * 32 + 31;
            const bool warp_rows_ok = warp_last < n_rows;
            const int warp_pos_min = p0 + warp_first / G;
            const int warp_pos_max = p0 + (warp_last < n_rows ? warp_last : n_rows - 1) / G;
            const int warp_vis_max = (window > 0 && warp_pos_max - window + 1 > 0) ? warp_pos_max - window + 1 : 0;
            float m_used = -INFINITY, l = 0.f;
            for (int it = 0; it < n_it; ++it, ++g) {
                const uint32_t s = g & 1u, ph = (g >> 1) & 1u;
                const uint32_t tm_s = tmem + 128u * s;
                const int tile_lo = (rec.t_lo + it) * AT_BN;
                const int kbase = tile_lo + 64 * half;
                if (ok) ok = at_wait(&s_full[s], ph, 3);
                at_fence_after();
                float sc[64];
                {
                    uint32_t r0[32], r1[32];
                    at_tmem_ld32(tm_s + lane_base + 64u * half, r0);
                    at_tmem_ld32(tm_s + lane_base + 64u * half + 32u, r1);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 32; ++i) { sc[i] = __uint_as_float(r0[i]); sc[32 + i] = __uint_as_float(r1[i]); }
                }
                const bool full = warp_rows_ok && kbase + 63 <= warp_pos_min && kbase >= warp_vis_max;
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                if (full) {
#pragma unroll
                    for (int i = 0; i < 64; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], sc[i]);
                } else {
#pragma unroll
                    for (int i = 0; i < 64; ++i) {
                        const int key = kbase + i;
                        sc[i] = (key <= pos && key >= vis_lo) ? sc[i] : -INFINITY;
                        mx4[i & 3] = fmaxf(mx4[i & 3], sc[i]);
                    }
                }
                float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
                float* xm = s_xm + (g & 1u) * 256;
                xm[half * 128 + row] = mx;
                // the barrier: both halves have read their S (P is written over it below), and
                // whether any thread's wait ran out, so that all leave together
                if (at_bar_or(!ok)) { ok = false; break; }
                mx = fmaxf(mx, xm[(half ^ 1) * 128 + row]);
                const float m_new = fmaxf(m_used, mx);
                const bool grow = m_new > m_used + 8.f || (m_used == -INFINITY && m_new != -INFINITY);
                const bool rescale = __any_sync(0xffffffffu, grow);
                float corr = 1.f;
                if (rescale) {
                    corr = m_new == -INFINITY ? 1.f : exp2f(m_used - m_new);
                    m_used = m_new;
                }
                const float base_m = m_used == -INFINITY ? 0.f : m_used;
                float sum4[4] = {0.f, 0.f, 0.f, 0.f};
                {
                    uint32_t r[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const float a = at_ex2(fmaf(sc[2 * i], scale_log2, -base_m));
                        const float b = at_ex2(fmaf(sc[2 * i + 1], scale_log2, -base_m));
                        sum4[i & 3] += a + b;
                        r[i] = at_pack(a, b);
                    }
                    at_tmem_st32(tm_s + lane_base + 32u * half, r);
                }
                l = l * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
                if (tile_lo + AT_BN > key_hi || tile_lo < key_lo) {     // rows of V that nobody may read
                    if (ok) ok = at_wait(&v_full[s], ph, 3);
                    const int key = tile_lo + row;
                    if (key >= key_hi || key < key_lo) {
                        unsigned char* vrow = sV + s * AT_TILE_BYTES + half * AT_BLOCK_BYTES + row * 128;
#pragma unroll
                        for (int c = 0; c < 8; ++c) *(uint4*)(vrow + c * 16) = make_uint4(0u, 0u, 0u, 0u);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                if (it > 0) {
                    if (ok) ok = at_wait(o_done, (g - 1u) & 1u, 3);         // the previous P V is in O
                    at_fence_after();
                    if (rescale) {
                        uint32_t r[32];
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            at_tmem_ld32(tm_o + lane_base + 64u * half + 32u * c, r);
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * corr);
                            at_tmem_st32(tm_o + lane_base + 64u * half + 32u * c, r);
                        }
                    }
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                at_fence_before();
                const bool warp_ok = __all_sync(0xffffffffu, ok);
                if (lane == 0 && warp_ok) at_arrive(&p_full[s]);
            }
            if (!ok) break;                        // decided at a barrier: the same for all 256
            ok = at_wait(o_done, (g - 1u) & 1u, 3);                         // the item's last P V
            at_fence_after();
            s_xl[half * 128 + row] = l;
            if (at_bar_or(!ok)) break;
            l += s_xl[(half ^ 1) * 128 + row];
            {
                const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t r[32];
                    at_tmem_ld32(tm_o + lane_base + 64u * half + 32u * c, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (row_ok) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint4 v;
                            v.x = at_pack(__uint_as_float(r[8 * i]) * inv, __uint_as_float(r[8 * i + 1]) * inv);
                            v.y = at_pack(__uint_as_float(r[8 * i + 2]) * inv, __uint_as_float(r[8 * i + 3]) * inv);
                            v.z = at_pack(__uint_as_float(r[8 * i + 4]) * inv, __uint_as_float(r[8 * i + 5]) * inv);
                            v.w = at_pack(__uint_as_float(r[8 * i + 6]) * inv, __uint_as_float(r[8 * i + 7]) * inv);
                            *(uint4*)(dst + c * 32 + i * 8) = v;
                        }
                    }
                }
                at_fence_before();
                __syncwarp();
                if (lane == 0) at_arrive(&o_free[ob]);
            }
        }
    }
    at_fence_before();
    __syncthreads();
    if (warp == 1) {
        at_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
    if (tid == 0 && atomicAdd(&ap_finished, 1u) == gridDim.x - 1u) {
        ap_ticket = 0;              // nobody draws any more: every CTA has seen the end of the items
        ap_finished = 0;
        __threadfence();
    }
}

// ------------------------------------------------------------------------------ host
typedef CUresult (*AtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                               CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                               CUtensorMapFloatOOBfill);

// The tensor map of one layer's K or V pages, [rows, 128] bf16 in boxes of page_size x 64;
// made once per (address, rows, page size) and kept.
static const CUtensorMap* at_map_of(const void* pages, long long rows, int page_size) {
    static std::mutex lock;
    static std::unordered_map<uint64_t, CUtensorMap> maps;
    static AtEncodeFn encode = nullptr;
    std::lock_guard<std::mutex> hold(lock);
    if (!encode) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) != cudaSuccess ||
            qr != cudaDriverEntryPointSuccess)
            return nullptr;
        encode = (AtEncodeFn)p;
    }
    const uint64_t key = (uint64_t)(uintptr_t)pages ^ ((uint64_t)rows * 0x9e3779b97f4a7c15ull) ^ ((uint64_t)page_size << 56);
    auto it = maps.find(key);
    if (it != maps.end()) return &it->second;
    CUtensorMap map;
    const cuuint64_t dims[2] = {AT_DH, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {AT_DH * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)page_size};
    const cuuint32_t elem[2] = {1, 1};
    if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return nullptr;
    return &maps.emplace(key, map).first->second;
}

// The tensor map of a step's query rows, q [tokens, >= H * 128] bf16 with a row stride, seen
// as (64 columns, 2 halves, H heads, tokens): a box is one half of G heads of a tile's tokens.
// Kept by (address, stride, tokens, heads, group): a step's activations come back to the same
// addresses step after step.
static const CUtensorMap* at_map_q(const void* q, long long q_stride, int tokens, int H, int G) {
    struct Key {
        const void* q; long long stride; int tokens, H, G;
        bool operator==(const Key& o) const {
            return q == o.q && stride == o.stride && tokens == o.tokens && H == o.H && G == o.G;
        }
    };
    struct Hash {
        size_t operator()(const Key& k) const {
            return (size_t)(uintptr_t)k.q * 0x9e3779b97f4a7c15ull ^ ((size_t)k.stride << 32) ^ ((size_t)k.tokens << 12) ^
                   ((size_t)k.H << 6) ^ (size_t)k.G;
        }
    };
    static std::mutex lock;
    static std::unordered_map<Key, CUtensorMap, Hash> maps;
    static AtEncodeFn encode = nullptr;
    std::lock_guard<std::mutex> hold(lock);
    if (!encode) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) != cudaSuccess ||
            qr != cudaDriverEntryPointSuccess)
            return nullptr;
        encode = (AtEncodeFn)p;
    }
    const Key key{q, q_stride, tokens, H, G};
    auto it = maps.find(key);
    if (it != maps.end()) return &it->second;
    CUtensorMap map;
    const cuuint64_t dims[4] = {64, 2, (cuuint64_t)H, (cuuint64_t)tokens};
    const cuuint64_t strides[3] = {128, 256, (cuuint64_t)q_stride * 2};
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)G, (cuuint32_t)(AT_BM / G)};
    const cuuint32_t elem[4] = {1, 1, 1, 1};
    if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(q), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return nullptr;
    if (maps.size() > 4096) maps.clear();
    return &maps.emplace(key, map).first->second;
}

// 1 if this kernel takes the shape: head size 128, up to 16 query heads a kv head (a tile then
// holds 128 / group tokens, rounded down), pages of 8, 16, 32, 64 or 128 tokens.
TGO_API int tgo_attention_tc_supports(int dh, int group, int page_size) {
    const bool g_ok = group >= 1 && group <= 16;
    const bool p_ok = page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128;
    return dh == AT_DH && g_ok && p_ok;
}


// Reads (and waits for the device to reach) the code a wait that ran out left; 0: none did.
TGO_API int tgo_attention_tc_error(int* value) {
    return (int)cudaMemcpyFromSymbol(value, at_error_flag, sizeof(int));
}

// Prompt portions: tiles of up to 128 / group consecutive tokens of one request each
// (tile_tok0, tile_ntok); q has n_tokens rows of q_stride elements, its first H * 128 columns
// the heads. k_cache and v_cache: [n_pages, Hkv, page_size, 128] bf16.
// One CTA per SM draws (tile, kv head) items from a counter.
TGO_API int tgo_attention_tc_prefill(const void* q, long long q_stride, int n_tokens, void* out, long long out_stride,
                                     const void* k_cache, const void* v_cache, int n_pages, int page_size,
                                     const int* block_tables, int max_blocks, const int* positions,
                                     const int* seq_ids, const int* tile_tok0, const int* tile_ntok,
                                     int n_tiles, int H, int Hkv, int dh, float scale, int window,
                                     cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (n_tokens <= 0 || H <= 0 || Hkv <= 0 || H % Hkv || !tgo_attention_tc_supports(dh, H / Hkv, page_size) || n_pages <= 0 ||
        max_blocks <= 0 || window < 0 || Hkv > 65535 || !tile_tok0 || !tile_ntok || q_stride % 8 ||
        out_stride % 8 || ((uintptr_t)q % 16) || ((uintptr_t)out % 16) || ((uintptr_t)k_cache % 128) ||
        ((uintptr_t)v_cache % 128))
        return TGO_E_BAD_ARG;
    const long long rows = (long long)n_pages * Hkv * page_size;
    if (rows > 0x7fffffffll || (long long)n_tiles * Hkv > 0x7fffffffll) return TGO_E_BAD_ARG;
    const CUtensorMap* mk = at_map_of(k_cache, rows, page_size);
    const CUtensorMap* mv = at_map_of(v_cache, rows, page_size);
    const CUtensorMap* mq = at_map_q(q, q_stride, n_tokens, H, H / Hkv);
    if (!mk || !mv || !mq) return TGO_E_BAD_ARG;
    int shift = 0;
    while ((1 << shift) < page_size) ++shift;
    const float scale_log2 = scale * 1.4426950408889634f;
    {
        constexpr size_t smem = 1024 + 6 * (size_t)AT_TILE_BYTES + 22 * 8 + 4 * sizeof(ApItem) +
                                768 * sizeof(float) + 2 * AT_PAGES_CAP * sizeof(int);
        // per device: its SM count, and whether this kernel's attribute is set there
        static int sms_of[64] = {};
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return (int)e;
        if (dev < 0 || dev >= 64) return TGO_E_BAD_ARG;
        if (!sms_of[dev]) {
            e = cudaFuncSetAttribute(attention_tc_persistent_kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            int n = 0;
            if ((e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
            sms_of[dev] = n;
        }
        const int sms = sms_of[dev];
        const int items = n_tiles * Hkv;
        attention_tc_persistent_kernel<<<dim3(items < sms ? items : sms), AP_THREADS, smem, stream>>>(
            *mk, *mv, *mq, (bf16*)out, out_stride, page_size, shift, block_tables, max_blocks,
            positions, seq_ids, tile_tok0, tile_ntok, n_tiles, H, Hkv, scale_log2, window);
        return launch_status();
    }
}
