// Shared device helpers for the sm_100a kernels: mbarrier, TMA, tcgen05/TMEM wrappers, bounded
// waits and the error-status word that every waiting kernel reports through.
//
// Conventions
//   * Every spin on an mbarrier or on a flag written by another CTA / GPU is bounded. When the bound
//     runs out the waiter records {code, detail} in the status word, sets a CTA-wide abort flag where
//     one exists and leaves through the kernel's normal tear-down (TMEM is freed, no trap).
//   * No TMA load here carries a cluster-multicast qualifier.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lmsae {

// ---- status word -----------------------------------------------------------------------------
// status[0] = first error code (0 = ok), status[1] = detail, status[2] = block index, status[3] = aux
enum StatusCode : int {
  kOk = 0,
  kTimeoutFullBarrier = 1,
  kTimeoutEmptyBarrier = 2,
  kTimeoutTmemFull = 3,
  kTimeoutTmemEmpty = 4,
  kTimeoutPeerFlag = 5,
  kBadArgument = 6,
  kCapacityOverflow = 7,
};

__device__ __forceinline__ void report_status(int* status, int code, int detail, int aux = 0) {
  if (status == nullptr) return;
  if (atomicCAS(status, 0, code) == 0) {
    status[1] = detail;
    status[2] = (int)blockIdx.x;
    status[3] = aux;
  }
}

// ---- bounds-checked debug build ---------------------------------------------------------------
// Compiled with -DLMSAE_BOUNDS_CHECK (ops/native.py: build(debug=True), loaded with LMSAE_NATIVE_CHECKED=1), every
// data-dependent index that goes through LMSAE_IDX(index, limit) is compared with its limit first. A violation is
// RECORDED (source line, offending index, limit, number of violations; one record per translation unit, read back by
// the extension's bounds_report()) and the index is clamped into range, so the access that follows is legal: nothing
// traps and the context stays usable. In the regular build the macro is the index itself.
#ifdef LMSAE_BOUNDS_CHECK
static __device__ int g_lmsae_bounds[4];
__device__ __forceinline__ long long lmsae_checked_index(long long i, long long n, int line) {
  if (i >= 0 && i < n) return i;
  if (atomicAdd(&g_lmsae_bounds[3], 1) == 0) {
    g_lmsae_bounds[0] = line;
    g_lmsae_bounds[1] = (int)i;
    g_lmsae_bounds[2] = (int)n;
  }
  return i < 0 ? 0 : (n > 0 ? n - 1 : 0);
}
#define LMSAE_IDX(i, n) lmsae_checked_index((long long)(i), (long long)(n), __LINE__)
// Host accessor of this translation unit's record: out = {line, index, limit, count}; clears the record.
#define LMSAE_DEFINE_BOUNDS_FETCH(name)                                              \
  int name(int* out) {                                                               \
    cudaError_t e = cudaMemcpyFromSymbol(out, g_lmsae_bounds, 4 * sizeof(int));      \
    if (e != cudaSuccess) return (int)e;                                             \
    const int zero[4] = {0, 0, 0, 0};                                                \
    return (int)cudaMemcpyToSymbol(g_lmsae_bounds, zero, 4 * sizeof(int));           \
  }
#else
#define LMSAE_IDX(i, n) (i)
#define LMSAE_DEFINE_BOUNDS_FETCH(name) \
  int name(int* out) {                  \
    out[0] = out[1] = out[2] = out[3] = 0; \
    return 0;                           \
  }
#endif

// ---- small PTX wrappers ----------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P1;\n\t"
      "elect.sync _|P1, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P1;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred P1;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P1;\n\t"
      "}\n"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Roughly one to two seconds at B200 clocks; a healthy pipeline wait lasts microseconds.
constexpr long long kWaitBudgetCycles = 3000000000LL;

// Bounded wait. Returns true when the phase completed, false when the budget ran out or another
// role of this CTA already aborted (abort_flag != 0).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0x3ff) == 0) {
      if (abort_flag != nullptr && *abort_flag != 0) return false;
      if (clock64() - t0 > kWaitBudgetCycles) return false;
    }
  }
}

// ---- TMA -------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// 2-D tiled load global -> shared (this CTA only), completion counted in bytes on `bar`.
// c0 is the innermost coordinate; c0 * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int c0,
                                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

// ---- tcgen05 / TMEM --------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]^T, bf16 inputs, fp32 accumulate, issued by ONE thread.
__device__ __forceinline__ void umma_bf16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Makes `bar` observe completion of all tcgen05.mma issued so far by this thread.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ---- thread-block clusters and CTA pairs (tcgen05 cta_group::2) ---------------------------------
// A CTA pair is a cluster of two CTAs on neighbouring SMs that issue ONE tensor-core instruction over both
// SMs: rank 0 (the leader) issues it, each CTA supplies its half of A (M rows) and of B (N rows) from its own
// shared memory at the same offsets, and each CTA's TMEM receives its half of the accumulator rows.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// All threads of all CTAs of the cluster.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in CTA `rank` of the cluster (shared::cluster window).
__device__ __forceinline__ uint32_t mapa_u32(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Load into THIS CTA's shared memory; the byte count completes on a barrier that may live in the peer CTA
// (`bar_cluster_addr` is a shared::cluster address). No multicast: every CTA fetches its own tile.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* tmap, uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
// TMEM management for a CTA pair: one warp of EACH CTA executes these, with the same arguments.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A * B^T over the CTA pair (M = 256 rows: 128 per CTA), issued by ONE thread of
// the leader CTA. The eight zero words are the "disable output lane" mask.
__device__ __forceinline__ void umma_bf16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                  uint32_t accumulate) {
  const uint32_t z = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(z)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in every CTA of `cta_mask` once all tensor-core work
// issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(cta_mask)
      : "memory");
}

// 32 lanes x 32 consecutive fp32 columns -> 32 registers per thread (thread i of the warp = lane i of
// the warp's TMEM quarter).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// The reverse of tmem_ld_32x32b_x32: 32 registers per thread -> 32 lanes x 32 consecutive fp32 columns of TMEM.
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for a K-major bf16 tile stored by TMA with the 128-byte swizzle:
// rows are 128 bytes (64 bf16) apart inside an 8-row, 1024-byte swizzle atom; atoms follow each other
// every 1024 bytes along M/N. The tile base must be 1024-byte aligned; stepping K by 16 elements inside
// the 64-wide stage advances the start address by 32 bytes.
__device__ __forceinline__ uint64_t make_sw128_kmajor_desc(uint32_t smem_addr) {
  uint64_t desc = 0;
  desc |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);  // start address, bits [0,14)
  desc |= (uint64_t)1 << 16;                        // leading byte offset (unused for swizzled K-major)
  desc |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset: 8 rows * 128 B
  desc |= (uint64_t)1 << 46;                        // descriptor version for sm_100
  desc |= (uint64_t)2 << 61;                        // SWIZZLE_128B
  return desc;
}

// Instruction descriptor: bf16 x bf16 -> fp32, both operands K-major, dense.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N) {
  return (1u << 4)                     // accumulator format: f32
         | (1u << 7)                   // A format: bf16
         | (1u << 10)                  // B format: bf16
         | ((uint32_t)(N >> 3) << 17)  // N / 8
         | ((uint32_t)(M >> 4) << 24); // M / 16
}

// ---- misc ------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Acquire / release accessors for flags shared across CTAs (gpu scope) or GPUs (sys scope).
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Debug build only: a pseudo-random pause of up to ~8 us (different per block and per call), placed in front of every
// flag publication and flag wait and at the start of the communicating kernels. It perturbs the order in which blocks
// and ranks reach their synchronisation points, so that a protocol that only works for one lucky interleaving fails in
// the small-case tests instead of in a long run.
__device__ __forceinline__ void lmsae_jitter() {
#ifdef LMSAE_BOUNDS_CHECK
  const unsigned long long t = (unsigned long long)clock64();
  const unsigned ns = (unsigned)(((t ^ (t >> 13)) * 2654435761ull + (unsigned long long)blockIdx.x * 40503ull) >> 5) & 0x1fffu;
  __nanosleep(ns);
#endif
}

// Bounded spin until *flag >= target (flags only grow). Returns false when the budget ran out.
__device__ __forceinline__ bool wait_flag_sys(const uint32_t* flag, uint32_t target) {
  if (ld_acquire_sys(flag) >= target) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    if (ld_acquire_sys(flag) >= target) return true;
    if ((++spins & 0xff) == 0) {
      if (clock64() - t0 > kWaitBudgetCycles) return false;
      __nanosleep(64);
    }
  }
}

}  // namespace lmsae
