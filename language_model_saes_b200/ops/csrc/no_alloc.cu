// Implementation of the allocation-free entry point declared in no_alloc.h.
#include "no_alloc.h"

#include <atomic>
#include <climits>

#include "kernels.h"

namespace {

constexpr int kBlockSums = LMSAE_NOALLOC_MAX_FEATURES / 4096 + 1;
constexpr int kScratchInts = 2 * LMSAE_NOALLOC_MAX_FEATURES + kBlockSums;

// Scratch of the counting sort: [counts | cursor | block totals]. In host code this name is only a handle
// for cudaGetSymbolAddress, never a pointer that a kernel may be given.
static __device__ __align__(256) int g_csc_scratch[kScratchInts];

constexpr int kMaxDevices = 64;
// One slot per device. Atomic, so that two host threads that make their first call on a device at the same moment
// do not race in the C++ sense: both may look the address up, both obtain the same value, and either store wins.
std::atomic<int*> g_scratch_addr[kMaxDevices];

// Device address of the scratch array on the current device, resolved once per device.
cudaError_t scratch_for_current_device(int** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  int* ptr = g_scratch_addr[dev].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_csc_scratch);
    if (e != cudaSuccess) return e;
    if (ptr == nullptr) return cudaErrorInvalidSymbol;
    g_scratch_addr[dev].store(ptr, std::memory_order_release);
  }
  *out = ptr;
  return cudaSuccess;
}

}  // namespace

extern "C" int lmsae_csc_build_noalloc(const int* idx, long long n, int F, int* offsets, int* entries,
                                       cudaStream_t stream) {
  if (idx == nullptr || offsets == nullptr || entries == nullptr || n < 0 || F <= 0) return (int)cudaErrorInvalidValue;
  if (F > LMSAE_NOALLOC_MAX_FEATURES) return (int)cudaErrorInvalidValue;
  if (n > (long long)INT_MAX) return (int)cudaErrorInvalidValue;  // entry positions are stored as 32-bit ints
  int* scratch = nullptr;
  cudaError_t e = scratch_for_current_device(&scratch);
  if (e != cudaSuccess) return (int)e;
  int* counts = scratch;
  int* cursor = scratch + LMSAE_NOALLOC_MAX_FEATURES;
  int* block_sums = scratch + 2 * LMSAE_NOALLOC_MAX_FEATURES;
  // csc_build_launch zeroes the counters it uses (cudaMemsetAsync on `stream`) before counting, so the
  // leftovers of the previous call do not matter; cursor and block totals are fully overwritten.
  return lmsae::csc_build_launch(idx, n, F, counts, offsets, cursor, entries, block_sums, stream);
}
