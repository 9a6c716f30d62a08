/* Paged attention with split keys for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference engine; it exists for users of this
 * library only.
 *
 * fsie_attn_generic() splits a long key range over several thread blocks and needs two
 * float buffers for the partial results, which its caller allocates.  Some callers cannot
 * do that: a serving process that handed every free byte of the GPU to its page pool at
 * start-up and has nothing left to ask cudaMalloc for; a step loop that must not take the
 * device-wide synchronisation that cudaMalloc and cudaFree imply; a plain C program that
 * links this library without torch and plans all of its device memory before it starts.
 * For them this variant keeps the partial results in a fixed array inside the library
 * (FSIE_STATIC_SCRATCH_FLOATS floats, 4 MiB, held by every GPU that loads the library until
 * the process exits).  Inputs and outputs are still the caller's.
 *
 *  - It calls no cudaMalloc, cudaFree or any allocating routine.
 *  - The first call on a device looks the array's device address up and sets the kernel's
 *    shared-memory limit; make that first call outside any stream capture, and from one host
 *    thread: the looked-up address is kept per device without a lock (two threads racing
 *    through their first calls would both store the same value, but nothing orders them).
 *  - It needs nsplit * tokens * heads * (head_dim + 2) floats; a launch that needs more than
 *    FSIE_STATIC_SCRATCH_FLOATS is refused with FSIE_ERR_SCRATCH_TOO_SMALL and nothing runs.
 *    fsie_attn_static_scratch_floats() tells the need beforehand (anything above the limit is
 *    reported as limit + 1: the product is cut off before it could overflow; negative sizes
 *    give -1 and the launch is refused as a bad argument).
 *  - Nothing in the array has to start at zero: every (split, token, head) slot that a tile
 *    covers is written by the launch before its merge reads it.  The array keeps the last
 *    call's contents, so the tiles must cover every one of the `tokens` rows: with
 *    nsplit > 1 the merge runs over all `tokens`, and a row that no tile covers is merged
 *    from whatever an earlier call left there - its row of `out` is undefined.
 *  - All calls share the one array.  Calls that overlap on the GPU (two streams, two
 *    threads, two processes' worth of launches on one context) race on it; keep calls on one
 *    stream or order them yourself.
 *
 * Arguments are those of fsie_attn_generic() without part_o and part_ml; the result in
 * `out` is the same up to the rounding of the merge.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FSIE_STATIC_SCRATCH_FLOATS (1u << 20)
#define FSIE_ERR_SCRATCH_TOO_SMALL (-3)
#define FSIE_ERR_SCRATCH_SETUP (-4)

/* floats of scratch a launch with these sizes needs */
long long fsie_attn_static_scratch_floats(int tokens, int heads, int head_dim, int nsplit);

/* text for a negative return code of fsie_attn_generic_static_scratch */
const char* fsie_attn_static_scratch_error(int code);

int fsie_attn_generic_static_scratch(
    const void* q, int q_ld, const void* k_pages, const void* v_pages, long long page_stride,
    int page_size, const int* block_tables, int bt_stride, const int* tile_item,
    const int* tile_row0, int tiles, const int* item_qstart, const int* item_qlen,
    const int* item_pos0, void* out, int out_ld, int tokens, int heads, int kv_heads,
    int head_dim, int window, int nsplit, float scale, int dtype, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
