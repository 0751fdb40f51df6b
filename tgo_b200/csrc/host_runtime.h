// C interface of the host runtime (host_runtime.cpp): the books of cache pages and request
// slots, the three calls of a step (grow, pack, commit) and the scheduler's policy. Plain C
// types only, no CUDA; every function that returns int returns one of the codes below unless
// its comment says otherwise, and tgo_cache_last_error tells what went wrong.
#ifndef TGO_HOST_RUNTIME_H
#define TGO_HOST_RUNTIME_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum tgo_host_code {
    TGO_HOST_OK = 0,
    TGO_HOST_PAGES_EXHAUSTED = 1,  /* info: group, pages needed, pages free; nothing was taken */
    TGO_HOST_SLOTS_EXHAUSTED = 2,
    TGO_HOST_ALREADY_LIVE = 3,
    TGO_HOST_NOT_LIVE = 4,
    TGO_HOST_BAD_ARGUMENT = 5,
    TGO_HOST_NO_PAGE = 6,          /* info: group, position, entry of the step */
    TGO_HOST_PAGE_MISUSE = 7,      /* a page given back twice, or not one of the pool's */
    TGO_HOST_BUFFER_SMALL = 8,     /* info[0]: ints needed */
    TGO_HOST_BROKEN_BOOKS = 9      /* tgo_cache_check found a fault */
};

/* kinds[g]: 0 the group keeps every key, 1 a window of windows[g] keys. NULL on bad sizes. */
void* tgo_cache_create(int n_groups, const int* kinds, const int* windows, int page_size,
                       const int* pages_per_group, int num_slots);
void tgo_cache_destroy(void* cache);
const char* tgo_cache_last_error(void* cache, long long info[3]);

int tgo_cache_admit(void* cache, long long handle, long long reserve_tokens, int* slot);
int tgo_cache_grow(void* cache, long long handle, long long upto);
int tgo_cache_commit(void* cache, long long handle, long long new_length, int* released_pairs, int cap,
                     int* n_released);
int tgo_cache_finish(void* cache, long long handle, int* released_pairs, int cap, int* n_released);

/* what: 0 length, 1 slot, 2 version, 3 live (1 or 0); -1 for a request that is not live */
long long tgo_cache_request(void* cache, long long handle, int what);
/* the table's length; its first `cap` entries into `out` */
int tgo_cache_table(void* cache, long long handle, int group, int* out, int cap);
/* what: 0 free pages, 1 held, 2 in all, 3 taken so far, 4 given back so far */
long long tgo_cache_pool(void* cache, int group, int what);
int tgo_cache_page_is_held(void* cache, int group, int page);
int tgo_cache_free_slots(void* cache);
int tgo_cache_live_requests(void* cache);
int tgo_cache_can_hold(void* cache, long long n_tokens, long long step_tokens);   /* 1 or 0 */
long long tgo_cache_slot_of(void* cache, long long handle, int group, long long position); /* row, or -1 */
int tgo_cache_check(void* cache);

int tgo_step_grow(void* cache, int n, const long long* handles, const int* extents, int* refused,
                  int* widest_table);
int tgo_step_commit(void* cache, int n, const long long* handles, const int* extents);
int tgo_step_widest_table(void* cache, int n, const long long* handles);   /* a length, or -1 */
/* out: ids[T] pos[T] seq[T] q_start[B+1] ctx[B] state_slot[B] rows[n_rows], then per group
   slots[T] table[B * width]. meta: T, B, n_rows, largest context, ints written, the width of
   each group, the length before the step of each entry (5 + groups + n ints). */
int tgo_step_pack(void* cache, int n, const long long* handles, const int* extents, const int* tokens_flat,
                  const int* n_want, const int* want_flat, int pad_to, int width_quantum, int all_rows,
                  int32_t* out, long long cap, int* meta);

/* the number of work items (slot, token count, 1 prompt tokens / 0 the fed token), in slot
   order; -1 for a chunk or budget that is not positive */
int tgo_schedule_next_step(int n_slots, const int* live, const long long* prompt_len,
                           const long long* prefilled, const int* has_feed, long long chunk,
                           long long budget, int* out_slot, long long* out_count, int* out_prefill);
/* the slot to evict, or -1 */
int tgo_schedule_victim(int n_slots, const int* live, const int* in_prompt, const long long* arrived);

#ifdef __cplusplus
}
#endif
#endif
