// Allocation-free entry point for paged decode attention.
//
// This entry point has no counterpart in the reference engine; it exists for callers of this library
// that are not allowed to allocate device memory around the call:
//   * code running while a stream is being captured, or between two captures, where an allocation
//     would change what the capture records or move a buffer that an earlier graph baked in;
//   * a serving loop that has handed all remaining device memory to its KV page pool, so that any
//     further allocation can fail or stall on a free;
//   * hosts that call the library through its C symbols with no tensor framework (and therefore no
//     caching allocator) behind them.
//
// he_attn_decode() wants the caller to supply `partial`, a scratch buffer of
// R * H * max_splits * (D + 2) floats.  he_attn_decode_noalloc() is the same computation with the scratch
// taken from a fixed array that lives in the library's own device image, so neither the caller nor the
// library allocates anything: no cudaMalloc / cudaFree, no allocating library routine, no framework
// allocator.  The caller still passes every input and output; `args->partial` is ignored.
//
// Limits and rules
//   * The built-in scratch holds HE_ATTN_NOALLOC_MAX_FLOATS floats (8 MiB).  A call that needs more
//     returns -HE_ERR_BAD_ARG (-3) and launches nothing; he_attn_decode_noalloc_capacity() reports the
//     limit so a caller can size R / max_splits against it beforehand.
//   * The first call on each device looks the array's address up (cudaGetSymbolAddress, with that
//     device current) and remembers it.  Make that first call before starting any stream capture;
//     later calls on the same device only launch kernels.
//     Two first calls on the same device from different host threads only repeat the look-up (both
//     store the same address), but do not rely on that: make the first call from one thread.
//   * Every row's context must fit the split grid: ctx_len[r] (or the window, when one is set)
//     <= split_len * max_splits.  A longer context is reduced over the first max_splits splits only.
//   * Nothing in the scratch has to start at zero: every value the reduce kernel reads was written by
//     the split kernel of the same call.
//   * There is ONE array per device, shared by every call.  Two calls whose kernels can overlap
//     (different streams, or different host threads on different streams) race on it; issue calls on
//     one stream, or order them with events.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HE_ATTN_NOALLOC_MAX_FLOATS (2u * 1024u * 1024u)

struct AttnDecArgs;  // same argument block as he_attn_decode (see attn_decode.cu)

// Returns 0 on success, -3 for a shape beyond the scratch capacity or otherwise unsupported, a positive
// cudaError_t value if the address look-up or a launch failed.
int he_attn_decode_noalloc(const struct AttnDecArgs* args, cudaStream_t stream);

// Capacity of the built-in scratch in floats.
long long he_attn_decode_noalloc_capacity(void);

#ifdef __cplusplus
}
#endif
