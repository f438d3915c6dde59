// Device helpers shared by the kernels that move data between GPUs through peer mappings of symmetric buffers:
// epoch flags (one writer per word, st.release.sys / bounded ld.acquire.sys), the "last block signals" epilogue,
// the accounting of exposed waiting time, and the NVSwitch multicast (multimem) accessors.
//
// Every wait is bounded and reports through the status word; nothing here traps or spins without a limit.
#pragma once
#include "common.cuh"
#include "kernels.h"

namespace lmsae {

__device__ __forceinline__ void bf16x8_to_float_c(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ uint4 float8_to_bf16x8(const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16x2(f[0], f[1]);
  o.y = pack_bf16x2(f[2], f[3]);
  o.z = pack_bf16x2(f[4], f[5]);
  o.w = pack_bf16x2(f[6], f[7]);
  return o;
}

__device__ __forceinline__ uint32_t* flag_slot(const PeerTable& pt, int on_rank, int phase, int src) {
  return reinterpret_cast<uint32_t*>(pt.base[on_rank] + pt.flags_off) + phase * kMaxPeers + src;
}

// After all of this grid's stores: the last block to arrive publishes `epoch` in every peer's flag slot.
// Returns true in the block that signalled (uniformly over its threads).
__device__ __forceinline__ bool signal_peers_when_grid_done(const PeerTable& pt, int phase, uint32_t epoch,
                                                            unsigned* done_counter) {
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    lmsae_jitter();
    const unsigned prev = atomicAdd(done_counter, 1u);
    s_last = (prev == gridDim.x - 1);
    if (s_last) *done_counter = 0;
  }
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if ((int)threadIdx.x < pt.world) st_release_sys(flag_slot(pt, threadIdx.x, phase, pt.rank), epoch);
  }
  return s_last != 0;
}

// Block-wide bounded wait until every source rank has published `epoch` for `phase` in OUR flag slots.
// Returns false (uniformly) on expiry. Block 0 adds the cycles it spent here to the rank's exposed-wait
// counters (pt.stats: one {cycles, calls} pair of 64-bit words per phase), which is how the time a step
// spends waiting for its peers is measured without a profiler (`record_always`: for kernels in which one block only
// waits, whichever it is).
__device__ __forceinline__ bool wait_all_sources(const PeerTable& pt, int phase, uint32_t epoch, int* status,
                                                 bool record_always = false) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < 32) {
    long long waited = 0;
    if ((int)threadIdx.x < pt.world) {
      lmsae_jitter();
      const long long t0 = clock64();
      if (!wait_flag_sys(flag_slot(pt, pt.rank, phase, threadIdx.x), epoch)) {
        report_status(status, kTimeoutPeerFlag, phase, (int)threadIdx.x);
        s_ok = 0;
      }
      waited = clock64() - t0;
    }
    if ((blockIdx.x == 0 || record_always) && pt.stats != nullptr) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const long long other = __shfl_xor_sync(0xffffffffu, waited, o);
        waited = other > waited ? other : waited;
      }
      if (threadIdx.x == 0) {
        atomicAdd(pt.stats + 2 * phase, (unsigned long long)waited);
        atomicAdd(pt.stats + 2 * phase + 1, 1ull);
      }
    }
  }
  __syncthreads();
  return s_ok != 0;
}

// ---- NVSwitch multicast (NVLS) accessors ---------------------------------------------------------------
// `mc` is an address inside the multicast mapping of the group's symmetric buffers: a load-reduce returns the
// element-wise sum of the 16 bytes at that offset in EVERY rank's buffer (added inside the switch, fp32
// accumulation for bf16 data), a store writes the 16 bytes into every rank's buffer with one message.
__device__ __forceinline__ uint4 multimem_ld_reduce_add_bf16x8(const void* mc) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(mc)
               : "memory");
  return r;
}
__device__ __forceinline__ void multimem_st_16B(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

}  // namespace lmsae
