// Paged attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference runtime.  It exists for hosts that drive the
// kernel library directly through its C symbols from a context where cudaMalloc is off the table: a
// plug-in loaded into another process whose memory pool it does not own, a latency-critical serving
// thread that must never take the allocator lock, or a caller running under a fixed device-memory
// budget that was handed out before this library was loaded.  `ogb_paged_attention` with
// kv splits > 1 needs fp32 scratch for the per-split partial results and expects the caller to
// provide it; `ogb_paged_attention_noalloc` computes exactly the same thing but keeps that scratch in
// a fixed array inside the library's device image.
//
// Contract
//   * Inputs and outputs are still the caller's buffers; nothing is allocated or freed here
//     (no cudaMalloc / cudaFree / cudaMallocAsync, no framework allocator).
//   * The scratch is OGB_NOALLOC_SCRATCH_BYTES of device memory that every GPU holding the
//     library keeps until the process exits.  A call whose split-KV partials need more than that
//     (total_tokens * Hq * (D + 2) * splits * 4 bytes) is refused with OGB_ERR_NOALLOC_TOO_LARGE
//     and launches nothing; `ogb_paged_attention_noalloc_required_bytes` tells the size beforehand.
//   * The first call on a device looks up the device address of the array (the array's name in
//     host code is only a host-side handle, not a device pointer) with that device current, and
//     caches it.  Make that first call during set-up, before any stream capture.
//   * All calls on a device share the one array and it keeps the previous call's contents: the
//     kernel overwrites every element it later reads, so nothing needs clearing, but two calls
//     whose executions overlap on the GPU (different streams) race on it.  Issue them on one
//     stream, or order them yourself.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OGB_NOALLOC_SCRATCH_BYTES (8ll << 20)
#define OGB_ERR_NOALLOC_TOO_LARGE (-7)
#define OGB_ERR_NOALLOC_SETUP (-8)

long long ogb_paged_attention_noalloc_required_bytes(int total_tokens, int Hq, int D, int splits);

// Same arguments as ogb_paged_attention without the scratch pair.  Returns 0, one of the launcher's
// negative codes, OGB_ERR_NOALLOC_TOO_LARGE (request needs more scratch than the library holds) or
// OGB_ERR_NOALLOC_SETUP (the device address of the scratch could not be obtained).
int ogb_paged_attention_noalloc(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int32_t* cu_seqlens,
                                const int32_t* past_lens, const int32_t* block_table, int table_cols, int block_size, void* out,
                                int out_stride, const float* sinks, float scale, float softcap, int window, int B,
                                int total_tokens, int max_q_len, int Hq, int Hkv, int D, int splits, void* stream);

#ifdef __cplusplus
}
#endif
