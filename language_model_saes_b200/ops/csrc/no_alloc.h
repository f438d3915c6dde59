// Allocation-free C entry point for grouping sparse codes by feature.
//
// This entry point has no counterpart in the reference project. It exists for callers that must not allocate
// device memory while they run: code that executes inside a fixed memory budget (an inference server that has
// handed all remaining memory to its own pools), code running under an allocator that cannot be re-entered
// from where the call is made, or plain C / C++ hosts that link this library without PyTorch's caching
// allocator. The regular entry point (`csc_build`, reached through the Python bindings) expects its caller to
// pass scratch tensors; this one keeps its scratch inside the library.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest feature count the built-in scratch can serve. The scratch (two int arrays of this length plus a few
// hundred block totals, about 8 MiB) lives in a static device array: every GPU that loads this library holds
// it until the process exits.
#define LMSAE_NOALLOC_MAX_FEATURES (1 << 20)

// Groups the n = rows * k entries of `idx` (feature id per (row, slot), -1 = empty slot) by feature:
//   offsets[f] .. offsets[f+1]  delimit feature f's entries (offsets has F + 1 ints),
//   entries[...]                hold the flat positions (row * k + slot) of those entries (n ints).
// `idx`, `offsets` and `entries` are device pointers owned by the caller; the work is enqueued on `stream`.
//
// Returns 0 on success, otherwise a cudaError_t value (cudaErrorInvalidValue when F exceeds
// LMSAE_NOALLOC_MAX_FEATURES, when n exceeds INT_MAX (entry positions are 32-bit) or an argument is null /
// negative). It never calls cudaMalloc, cudaFree or any allocating library routine.
//
// The first call on a device looks up the device address of the scratch array (cudaGetSymbolAddress, with
// that device current); make that first call outside of any stream capture. Two host threads may make their first
// call at the same time: the look-up is idempotent and its result is published atomically. All calls share the one scratch
// array, which still holds the previous call's counters when a call starts: the function clears what it needs,
// but two calls that overlap on the same GPU (different streams, different threads) race on it and must be
// serialised by the caller.
int lmsae_csc_build_noalloc(const int* idx, long long n, int F, int* offsets, int* entries, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
