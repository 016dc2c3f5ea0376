// Declaration of the one entry point of this library that allocates nothing.
// It has no counterpart in the reference: the reference's decode attention always takes its
// split workspace from its backend's allocator.
//
// Who needs it.  Some programs that embed this library decide their device-memory budget once,
// at start-up, and hand everything that is left to a pool of their own; for them a later
// cudaMalloc can fail, can stall the device while it runs, or simply breaks the rule that the
// host process owns every byte.  Other callers sit on a path where latency matters and an
// allocator call (with its implicit synchronisation) is not acceptable between two launches.
// Such callers cannot provide, or let us allocate, the scratch that the split-KV decode
// attention needs for its per-split partial results.  For them the scratch lives inside the
// library image, in a file-scope device array of fixed size.
//
// Cost and limit.  The array holds LEONE_STATIC_SCRATCH_FLOATS floats (4 MiB).  Every GPU that
// loads the library keeps that much memory until the process exits, whether or not the entry
// point is ever called.  A call needs n_seqs * n_q * splits * (head_dim + 2) floats when
// splits > 1 (nothing when splits == 1); a call that needs more is refused with
// LEONE_STATIC_TOO_LARGE and a message, and nothing is launched.
//
// Sharing.  All calls in the process share the one array, and it keeps whatever the last call
// left in it.  This kernel pair writes every partial it later reads, so nothing has to be
// cleared between calls.  Two calls whose kernels overlap on the GPU (different streams, or
// threads launching at once) race on the array; keep calls on one stream or order them yourself.
//
// First call.  The first call on a device looks up the array's device address
// (cudaGetSymbolAddress, once per device, with that device current).  Make that first call
// before any stream capture begins.
#pragma once
#include <cuda_runtime.h>

#define LEONE_STATIC_SCRATCH_FLOATS (1 << 20)
#define LEONE_STATIC_TOO_LARGE (-4)
#define LEONE_STATIC_SETUP_FAILED (-5)

#ifdef __cplusplus
extern "C" {
#endif

// Split-KV decode attention over the paged cache, bf16, exactly as leone_attention_decode, but
// with the split scratch in the library's own static device array.  The caller passes inputs and
// outputs only.  Returns 0 when launched, a negative code when refused (then `error`, if not
// null, receives a zero-terminated message of at most error_len bytes), or a positive
// cudaError_t from the launch.
int leone_attention_decode_static(const void* qkv, int row_stride, void* out, int out_stride,
                                  const void* k_pool, const void* v_pool, const int* block_table,
                                  int table_width, const int* q_start, const int* ctx_len,
                                  int n_seqs, int n_q, int n_kv, int d, float scale, int window,
                                  int page_tokens, int num_pages, int splits, int* status,
                                  char* error, int error_len, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
