// Paged decode attention through a C entry point that never allocates.
//
// This entry point has no counterpart in the reference project.  It exists for callers that hold raw device
// pointers and must not allocate on the request path: a C or C++ serving host that hands out all of its device
// memory from one arena at start-up, or a caller inside a region where a call into an allocator could
// synchronise the device or fail under memory pressure.  The split-KV partials that the regular entry points
// (`mmb_paged_decode` + `mmb_decode_merge`, api.h) take from the caller live here in a fixed array of device
// memory that is part of the loaded module.
//
// Limits (see also mmb_paged_attention_noalloc_limits):
//   B * Hq * splits * dv  <= 2 Mi floats   (8 MiB of partial outputs)
//   B * Hq * splits       <= 16 Ki rows    (128 KiB of running max / sum pairs)
// A call beyond either limit is rejected with MMB_NOALLOC_TOO_LARGE and launches nothing.
//
// The first call on a device looks up the address of the scratch array for that device (one runtime query, with
// that device current) and should therefore come before any stream capture.  The scratch is one array per
// device: two calls that overlap in time on the same device (different streams or threads) race on it; calls on
// one stream are ordered and safe.
//
// The kernels are launched with the programmatic-dependent-launch attribute and request K tiles before they wait
// for the preceding kernel of the stream.  Every cached KV row other than the one at position ctx - 1 must
// therefore be complete in memory before this call is enqueued (the usual case: older rows were written by
// earlier steps); a caller whose preceding kernel still writes older rows sets MMB200_PDL=0 in the environment.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif
#define MMB_NOALLOC_EXPORT __attribute__((visibility("default")))

enum {
  MMB_NOALLOC_OK = 0,
  MMB_NOALLOC_TOO_LARGE = -1,     // the partials do not fit the built-in scratch
  MMB_NOALLOC_BAD_ARGUMENT = -2,  // null pointer, non-positive size, unsupported head shape
  MMB_NOALLOC_SETUP_FAILED = -3   // the scratch address could not be obtained on the current device
  // positive values are cudaError_t codes from the launches
};

// Inputs and outputs are the caller's (all on the current device):
//   q            bf16 [B, Hq, dqk]
//   k_pool       bf16 [num_slots, Hkv, dqk]
//   v_pool       bf16 [num_slots, Hkv, dv], or null when V is the first dv columns of K (MLA latent cache)
//   block_tables int32 [B, max_blocks], ctx_lens int32 [B]
//   w_uv         optional bf16 [Hq, dvo, dv] per-head up projection (pass null and dvo = dv without it)
//   out          bf16 [B, Hq, dvo]
MMB_NOALLOC_EXPORT int mmb_paged_attention_noalloc(const void* q, const void* k_pool, const void* v_pool, const int* block_tables,
                                const int* ctx_lens, const void* w_uv, void* out, int B, int Hq, int Hkv, int dqk,
                                int dv, int dvo, int block_size, int max_blocks, int splits, float scale, int window,
                                cudaStream_t stream);

// Capacity of the scratch: floats for the partial outputs and rows (B * Hq * splits) for the max / sum pairs.
MMB_NOALLOC_EXPORT void mmb_paged_attention_noalloc_limits(long long* max_partial_floats, long long* max_rows);

// Text of the last error this thread got from mmb_paged_attention_noalloc ("" after a successful call).
MMB_NOALLOC_EXPORT const char* mmb_paged_attention_noalloc_error(void);

#ifdef __cplusplus
}
#endif
