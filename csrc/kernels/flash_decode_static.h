// iris_flash_decode_static: paged GQA flash-decode over ONE GPU's KV cache for callers that
// cannot allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for embedders of this library
// that are not allowed to call cudaMalloc (or any allocating routine, torch's caching allocator
// included) at the point where they decode: for example a serving loop that runs under a fixed
// memory budget handed out at start-up, or a plugin called from a host application that owns all
// device memory. Such a caller still passes its inputs (q, the paged K/V cache, the block table,
// the lengths) and its output buffer; what it cannot provide is the scratch the split-K kernel
// needs for its per-split partial results. Here that scratch is a fixed array that lives inside
// the library itself.
//
// Properties a caller has to know:
//  * The scratch is a file-scope device array of IRIS_DECODE_STATIC_SCRATCH_BYTES (8 MiB). Every
//    GPU on which the library is loaded carries it from load to process exit, used or not.
//  * A call needs batch * q_heads * splits * (head_dim + 1) floats. Larger problems are refused
//    with IRIS_DECODE_STATIC_TOO_LARGE and a message in `err`; nothing is launched. Lower `splits`
//    (it trades parallelism for scratch) or use iris_flash_decode with a buffer of your own.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress,
//    with that device current). That look-up is not a stream operation: make the first call on a
//    device outside any stream capture.
//  * All calls on a device share the one array, and it keeps whatever the previous call left in
//    it. Every slot a call reads is written by that same call first, so nothing needs clearing;
//    but two calls whose kernels overlap on the GPU (different streams) race on the array. Order
//    them on one stream or with events.
//  * No cudaMalloc, cudaFree or allocating library routine is called, on any path.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define IRIS_DECODE_STATIC_SCRATCH_BYTES (8u << 20)
#define IRIS_DECODE_STATIC_TOO_LARGE (-100)

// q [B, Hq, 128], k_cache / v_cache [num_blocks, page, Hkv, 128], block_table int32 [B, max_blocks],
// kv_lens int32 [B], out [B, Hq, 128]; dtype: 0 fp16, 1 bf16 (IrisDType). Device pointers, all
// contiguous. Launches on `stream` and returns without synchronising. Returns 0, a negative
// launch/argument code, or IRIS_DECODE_STATIC_TOO_LARGE. `err` (may be null) receives a message.
int iris_flash_decode_static(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                             const int32_t* kv_lens, void* out, int32_t B, int32_t Hq, int32_t Hkv, int32_t D,
                             int32_t page, int32_t max_blocks, int32_t splits, float sm_scale, float soft_cap,
                             int32_t dtype, void* stream, char* err, int32_t errlen);

// Floats of scratch the given problem needs (to size `splits` against the limit).
uint64_t iris_flash_decode_static_scratch_needed(int32_t B, int32_t Hq, int32_t splits, int32_t D);

#ifdef __cplusplus
}
#endif
