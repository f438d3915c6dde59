// Fused compute + collective kernels over NVLink peer memory for the feature-sharded ("model" parallel) step.
//
// Every rank owns one symmetric buffer (allocated and exchanged by the host side, parallel/symm.py) whose
// peer mappings are plain device pointers here. All transfers are ordinary stores / loads through those
// pointers (no TMA on peer memory, no multicast); completion is signalled with monotonically growing epoch
// flags written with st.release.sys and awaited with bounded ld.acquire.sys spins that report a status code
// on expiry instead of hanging.
//
//   push_candidates_kernel     all-gather of the per-rank top-k candidates (k (value, column) pairs per row):
//                              each rank stores its pairs straight into every peer's merge input
//   sparse_decode_scatter      gather-GEMM decode whose epilogue IS the reduce-scatter: every finished row of
//                              the partial reconstruction is stored into the symmetric buffer of the rank that
//                              owns that row, while other rows are still being computed
//   reduce_loss_push_kernel    the row owner sums the tp partials (+ bias), evaluates the MSE loss and its
//                              gradient, and all-gathers the bf16 gradient rows by storing them into every peer
//   wait_flags_kernel          bounded wait for one phase of one epoch (consumers run after it in stream order)
//
// They replace: the all-reduces of the reference's distributed top-k (utils/distributed/ops.py:226-250) and
// the Partial->Replicate all-reduce after its decoder matmul (models/sae.py:374-375).
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

// After all of this grid's stores: the last block to arrive publishes `epoch` in every peer's flag slot.
__device__ __forceinline__ void signal_peers_when_grid_done(const PeerTable& pt, int phase, uint32_t epoch,
                                                            unsigned* done_counter) {
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(done_counter, 1u);
    s_last = (prev == gridDim.x - 1);
    if (s_last) *done_counter = 0;
  }
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if ((int)threadIdx.x < pt.world) {
      uint32_t* flag = reinterpret_cast<uint32_t*>(pt.base[threadIdx.x] + pt.flags_off) + phase * kMaxPeers + pt.rank;
      st_release_sys(flag, epoch);
    }
  }
}

// Block-wide bounded wait until every source rank has published `epoch` for `phase` in OUR flag slots.
// Returns false (uniformly) on expiry.
__device__ __forceinline__ bool wait_all_sources(const PeerTable& pt, int phase, uint32_t epoch, int* status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < pt.world) {
    const uint32_t* flag =
        reinterpret_cast<const uint32_t*>(pt.base[pt.rank] + pt.flags_off) + phase * kMaxPeers + threadIdx.x;
    if (!wait_flag_sys(flag, epoch)) {
      report_status(status, kTimeoutPeerFlag, phase, (int)threadIdx.x);
      s_ok = 0;
    }
  }
  __syncthreads();
  return s_ok != 0;
}

// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
push_candidates_kernel(const PeerTable pt, const float* __restrict__ val, const int* __restrict__ idx, int B, int k,
                       uint32_t epoch, unsigned* done_counter) {
  // peer layout: val [B][world * k] floats at cand_val_off, idx likewise at cand_idx_off; our segment = rank
  const long long n = (long long)B * k;
  for (int p = 0; p < pt.world; ++p) {
    float* dv = reinterpret_cast<float*>(pt.base[p] + pt.cand_val_off);
    int* di = reinterpret_cast<int*>(pt.base[p] + pt.cand_idx_off);
    for (long long i = blockIdx.x * 256LL + threadIdx.x; i < n; i += (long long)gridDim.x * 256) {
      const long long row = i / k, j = i - row * k;
      const long long o = row * ((long long)pt.world * k) + (long long)pt.rank * k + j;
      dv[o] = val[i];
      di[o] = idx[i];
    }
  }
  signal_peers_when_grid_done(pt, kPhaseCand, epoch, done_counter);
}

__global__ void wait_flags_kernel(const PeerTable pt, int phase, uint32_t epoch, int* status) {
  wait_all_sources(pt, phase, epoch, status);
}

// ---------------------------------------------------------------------------------------------
constexpr int SC_THREADS = 512;
constexpr int SC_MAX_VEC = 2;

__global__ void __launch_bounds__(SC_THREADS)
sparse_decode_scatter_kernel(const PeerTable pt, const int* __restrict__ idx, const float* __restrict__ val, int B, int k,
                             int d, const __nv_bfloat16* __restrict__ W, uint32_t epoch, unsigned* done_counter) {
  extern __shared__ uint8_t smem_raw[];
  int* s_idx = reinterpret_cast<int*>(smem_raw);
  float* s_val = reinterpret_cast<float*>(smem_raw) + k;
  const int nvec = d / 8;
  const int rows_per_rank = B / pt.world;
  for (int row = blockIdx.x; row < B; row += gridDim.x) {
    __syncthreads();
    for (int j = threadIdx.x; j < k; j += SC_THREADS) {
      s_idx[j] = idx[(size_t)row * k + j];
      s_val[j] = val[(size_t)row * k + j];
    }
    __syncthreads();
    float acc[SC_MAX_VEC][8];
#pragma unroll
    for (int u = 0; u < SC_MAX_VEC; ++u)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[u][i] = 0.0f;
    for (int j = 0; j < k; ++j) {
      const int f = s_idx[j];
      if (f < 0) continue;
      const float a = s_val[j];
      const uint4* wrow = reinterpret_cast<const uint4*>(W + (size_t)f * d);
#pragma unroll
      for (int u = 0; u < SC_MAX_VEC; ++u) {
        const int v = threadIdx.x + u * SC_THREADS;
        if (v < nvec) {
          float w[8];
          bf16x8_to_float_c(__ldg(wrow + v), w);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[u][i] = fmaf(a, w[i], acc[u][i]);
        }
      }
    }
    // epilogue = reduce-scatter: this row belongs to rank `owner`; our partial goes to slot [rank] there
    const int owner = row / rows_per_rank;
    const int lrow = row - owner * rows_per_rank;
    float* dst = reinterpret_cast<float*>(pt.base[owner] + pt.partial_off) +
                 ((size_t)pt.rank * rows_per_rank + lrow) * d;
#pragma unroll
    for (int u = 0; u < SC_MAX_VEC; ++u) {
      const int v = threadIdx.x + u * SC_THREADS;
      if (v < nvec) {
        float4* o = reinterpret_cast<float4*>(dst + v * 8);
        o[0] = make_float4(acc[u][0], acc[u][1], acc[u][2], acc[u][3]);
        o[1] = make_float4(acc[u][4], acc[u][5], acc[u][6], acc[u][7]);
      }
    }
  }
  signal_peers_when_grid_done(pt, kPhasePartial, epoch, done_counter);
}

// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
reduce_loss_push_kernel(const PeerTable pt, int B, int d, const __nv_bfloat16* __restrict__ label,
                        const float* __restrict__ bias, const float* __restrict__ row_weight, float grad_scale,
                        float* __restrict__ loss_sum, float* __restrict__ xhat_out, uint32_t epoch,
                        unsigned* done_counter, int* status) {
  __shared__ float s_red[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows_per_rank = B / pt.world;
  const bool ok = wait_all_sources(pt, kPhasePartial, epoch, status);
  if (ok) {
    const float* partial = reinterpret_cast<const float*>(pt.base[pt.rank] + pt.partial_off);
    const int nvec = d / 8;
    for (int lrow = blockIdx.x; lrow < rows_per_rank; lrow += gridDim.x) {
      const int row = pt.rank * rows_per_rank + lrow;
      const float rw = row_weight != nullptr ? row_weight[row] : 1.0f;
      float sq = 0.0f;
      for (int v = threadIdx.x; v < nvec; v += 256) {
        float x[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = bias != nullptr ? bias[v * 8 + i] : 0.0f;
        for (int s = 0; s < pt.world; ++s) {
          const float4* src = reinterpret_cast<const float4*>(partial + ((size_t)s * rows_per_rank + lrow) * d + v * 8);
          const float4 a = src[0], b = src[1];
          x[0] += a.x; x[1] += a.y; x[2] += a.z; x[3] += a.w;
          x[4] += b.x; x[5] += b.y; x[6] += b.z; x[7] += b.w;
        }
        if (xhat_out != nullptr) {
          float4* o = reinterpret_cast<float4*>(xhat_out + (size_t)row * d + v * 8);
          o[0] = make_float4(x[0], x[1], x[2], x[3]);
          o[1] = make_float4(x[4], x[5], x[6], x[7]);
        }
        float y[8];
        bf16x8_to_float_c(__ldg(reinterpret_cast<const uint4*>(label + (size_t)row * d) + v), y);
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          e[i] = x[i] - y[i];
          sq = fmaf(e[i], e[i], sq);
          e[i] *= grad_scale * rw;
        }
        uint4 o;
        o.x = pack_bf16x2(e[0], e[1]);
        o.y = pack_bf16x2(e[2], e[3]);
        o.z = pack_bf16x2(e[4], e[5]);
        o.w = pack_bf16x2(e[6], e[7]);
        // all-gather of the gradient rows: store into every rank's full [B, d] gradient buffer
        for (int p = 0; p < pt.world; ++p) {
          uint4* dst = reinterpret_cast<uint4*>(pt.base[p] + pt.dxhat_off) + ((size_t)row * d) / 8 + v;
          *dst = o;
        }
      }
      sq = warp_sum(sq);
      __syncthreads();
      if (lane == 0) s_red[warp] = sq;
      __syncthreads();
      if (warp == 0) {
        float t = lane < 8 ? s_red[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) atomicAdd(loss_sum, t * rw);
      }
    }
  }
  // signal even after a failed wait so that peers do not pile further timeouts on top of the first one
  signal_peers_when_grid_done(pt, kPhaseDxhat, epoch, done_counter);
}

// ---- launchers ----------------------------------------------------------------------------------
// ---------------------------------------------------------------------------------------------
// Row all-to-all for the activation shuffle: local row i goes to global position dest[i] of the logical
// [world * rows_per_rank] array, i.e. to slot dest[i] % rows_per_rank of rank dest[i] / rows_per_rank. Every CTA
// copies whole rows with 16-byte peer stores (a row of d_model 4096 bf16 values is 8 KB); the last CTA to finish
// publishes the epoch in every peer's flag slot. `dest` restricted to one rank is injective, and the union over
// ranks is a permutation, so no two stores touch the same bytes.
__global__ void __launch_bounds__(256)
shuffle_rows_kernel(const PeerTable pt, const uint4* __restrict__ src, const long long* __restrict__ dest, int n_local,
                    int rows_per_rank, int vec_per_row, long long recv_off, int phase, uint32_t epoch,
                    unsigned* done_counter) {
  for (int i = blockIdx.x; i < n_local; i += gridDim.x) {
    const long long g = dest[i];
    const int r = (int)(g / rows_per_rank);
    const long long slot = g - (long long)r * rows_per_rank;
    if (r < 0 || r >= pt.world) continue;  // never for a valid permutation; keeps a bad index off the wire
    uint4* dst = reinterpret_cast<uint4*>(pt.base[r] + recv_off) + slot * vec_per_row;
    const uint4* s = src + (long long)i * vec_per_row;
    for (int v = threadIdx.x; v < vec_per_row; v += 256) dst[v] = __ldg(s + v);
  }
  signal_peers_when_grid_done(pt, phase, epoch, done_counter);
}

int shuffle_rows_launch(const PeerTable& pt, const void* src, const long long* dest, int n_local, int rows_per_rank,
                        int row_bytes, long long recv_off, int phase, uint32_t epoch, unsigned* done_counter,
                        cudaStream_t stream) {
  if (row_bytes % 16 != 0 || n_local > rows_per_rank || phase < 0 || phase >= kNumPhases) return (int)cudaErrorInvalidValue;
  int blocks = n_local < 148 * 4 ? (n_local > 0 ? n_local : 1) : 148 * 4;
  shuffle_rows_kernel<<<blocks, 256, 0, stream>>>(pt, reinterpret_cast<const uint4*>(src), dest, n_local, rows_per_rank,
                                                  row_bytes / 16, recv_off, phase, epoch, done_counter);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Broadcast of (optionally masked and cast) rows from one rank to every rank of the group: the rank that read a chunk of
// cached activations from disk drops the masked-out token rows, casts to the training dtype and stores the result
// straight into every peer's landing zone, one read of the source for `world` NVLink writes. Replaces a boolean index,
// a dtype cast and a broadcast collective (activation/processors/cached_activation.py:301-320 and the loader-side
// redistribute of the reference project). `pos` = exclusive prefix sum of `keep` (both nullptr: keep every row).
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
bcast_rows_cast_kernel(const PeerTable pt, const TI* __restrict__ src, const int* __restrict__ keep,
                       const int* __restrict__ pos, long long n, int d, long long recv_off, long long cap_rows, int phase,
                       uint32_t epoch, unsigned* done_counter) {
  for (long long i = blockIdx.x; i < n; i += gridDim.x) {
    if (keep != nullptr && keep[i] == 0) continue;
    const long long o = pos != nullptr ? pos[i] : i;
    if (o < 0 || o >= cap_rows) continue;  // never written past the landing zone
    const TI* s = src + (size_t)i * d;
    for (int c = threadIdx.x * 8; c < d; c += 256 * 8) {
      float f[8];
      if constexpr (sizeof(TI) == 4) {
        const float4 a = __ldcs(reinterpret_cast<const float4*>(s + c)), b = __ldcs(reinterpret_cast<const float4*>(s + c) + 1);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
      } else {
        bf16x8_to_float_c(__ldcs(reinterpret_cast<const uint4*>(s + c)), f);
      }
      for (int p = 0; p < pt.world; ++p) {
        TO* dst = reinterpret_cast<TO*>(pt.base[p] + recv_off) + (size_t)o * d + c;
        if constexpr (sizeof(TO) == 4) {
          reinterpret_cast<float4*>(dst)[0] = make_float4(f[0], f[1], f[2], f[3]);
          reinterpret_cast<float4*>(dst)[1] = make_float4(f[4], f[5], f[6], f[7]);
        } else {
          uint4 u;
          u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]); u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
          *reinterpret_cast<uint4*>(dst) = u;
        }
      }
    }
  }
  signal_peers_when_grid_done(pt, phase, epoch, done_counter);
}

int bcast_rows_cast_launch(const PeerTable& pt, int in_dtype, int out_dtype, const void* src, const int* keep, const int* pos,
                           long long n, int d, long long recv_off, long long cap_rows, int phase, uint32_t epoch,
                           unsigned* done_counter, cudaStream_t stream) {
  if (d % 8 != 0 || recv_off % 16 != 0 || phase < 0 || phase >= kNumPhases) return (int)cudaErrorInvalidValue;
  const int blocks = (int)(n < 148LL * 8 ? (n > 0 ? n : 1) : 148LL * 8);
  using bf = __nv_bfloat16;
#define LMSAE_BCAST(TI, TO)                                                                                              \
  bcast_rows_cast_kernel<TI, TO><<<blocks, 256, 0, stream>>>(pt, static_cast<const TI*>(src), keep, pos, n, d, recv_off, \
                                                             cap_rows, phase, epoch, done_counter)
  if (in_dtype == 0 && out_dtype == 0) LMSAE_BCAST(float, float);
  else if (in_dtype == 0 && out_dtype == 1) LMSAE_BCAST(float, bf);
  else if (in_dtype == 1 && out_dtype == 0) LMSAE_BCAST(bf, float);
  else if (in_dtype == 1 && out_dtype == 1) LMSAE_BCAST(bf, bf);
  else return (int)cudaErrorInvalidValue;
#undef LMSAE_BCAST
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Second half of the head-summed encoder: after every rank's GEMM epilogue has added its partial pre-activations into
// the column slab this rank owns (reduce-scatter by vector reductions over NVLink, encoder_gemm.cu), the owner reads
// its fp32 slab [B, cols] once, stores the sums into every rank's full [B, world * cols] output (all-gather by peer
// stores) and clears the slab for the call after next. Replaces the all-reduce of a [batch, d_sae] tensor per step
// in models/crosscoder.py:350-375 of the reference project.
template <typename TO>
__global__ void __launch_bounds__(256)
headsum_gather_kernel(const PeerTable pt, long long slab_off, long long out_off, int B, int cols, int phase_in,
                      int phase_out, uint32_t epoch, unsigned* done_counter, int* status) {
  const bool ok = wait_all_sources(pt, phase_in, epoch, status);
  if (ok) {
    float* slab = reinterpret_cast<float*>(pt.base[pt.rank] + slab_off);
    const int N = cols * pt.world;
    const int vec_per_row = cols / 8;
    for (long long i = blockIdx.x * 256LL + threadIdx.x; i < (long long)B * vec_per_row; i += (long long)gridDim.x * 256) {
      const long long row = i / vec_per_row;
      const int c = (int)(i - row * vec_per_row) * 8;
      float4* sp = reinterpret_cast<float4*>(slab + row * cols + c);
      const float4 a = sp[0], b = sp[1];
      sp[0] = make_float4(0.f, 0.f, 0.f, 0.f);
      sp[1] = make_float4(0.f, 0.f, 0.f, 0.f);
      const long long o = row * N + (long long)pt.rank * cols + c;
      for (int p = 0; p < pt.world; ++p) {
        TO* dst = reinterpret_cast<TO*>(pt.base[p] + out_off) + o;
        if constexpr (sizeof(TO) == 4) {
          reinterpret_cast<float4*>(dst)[0] = a;
          reinterpret_cast<float4*>(dst)[1] = b;
        } else {
          uint4 u;
          u.x = pack_bf16x2(a.x, a.y); u.y = pack_bf16x2(a.z, a.w); u.z = pack_bf16x2(b.x, b.y); u.w = pack_bf16x2(b.z, b.w);
          *reinterpret_cast<uint4*>(dst) = u;
        }
      }
    }
  }
  // signal even after a failed wait so that peers do not pile further timeouts on top of the first one
  signal_peers_when_grid_done(pt, phase_out, epoch, done_counter);
}

int headsum_gather_launch(const PeerTable& pt, long long slab_off, long long out_off, int B, int cols, int out_dtype,
                          int phase_in, int phase_out, uint32_t epoch, unsigned* done_counter, int* status,
                          cudaStream_t stream) {
  if (cols % 8 != 0 || slab_off % 16 != 0 || out_off % 16 != 0) return (int)cudaErrorInvalidValue;
  if (phase_in < 0 || phase_in >= kNumPhases || phase_out < 0 || phase_out >= kNumPhases) return (int)cudaErrorInvalidValue;
  const long long work = (long long)B * (cols / 8);
  int blocks = (int)((work + 255) / 256);
  if (blocks > 148 * 4) blocks = 148 * 4;
  if (blocks < 1) blocks = 1;
  if (out_dtype == 0)
    headsum_gather_kernel<float><<<blocks, 256, 0, stream>>>(pt, slab_off, out_off, B, cols, phase_in, phase_out, epoch,
                                                            done_counter, status);
  else
    headsum_gather_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(pt, slab_off, out_off, B, cols, phase_in, phase_out,
                                                                    epoch, done_counter, status);
  return (int)cudaGetLastError();
}

// One warp publishes `epoch` for `phase` in every peer's flag slot (an acknowledgement: "I have consumed epoch").
__global__ void signal_flags_kernel(const PeerTable pt, int phase, uint32_t epoch) {
  __threadfence_system();
  if ((int)threadIdx.x < pt.world) {
    uint32_t* flag = reinterpret_cast<uint32_t*>(pt.base[threadIdx.x] + pt.flags_off) + phase * kMaxPeers + pt.rank;
    st_release_sys(flag, epoch);
  }
}

int signal_flags_launch(const PeerTable& pt, int phase, uint32_t epoch, cudaStream_t stream) {
  if (phase < 0 || phase >= kNumPhases) return (int)cudaErrorInvalidValue;
  signal_flags_kernel<<<1, 32, 0, stream>>>(pt, phase, epoch);
  return (int)cudaGetLastError();
}

// Bounded wait for ONE source rank's flag.
__global__ void wait_flag_src_kernel(const PeerTable pt, int phase, uint32_t epoch, int src, int* status) {
  if (threadIdx.x == 0) {
    const uint32_t* flag = reinterpret_cast<const uint32_t*>(pt.base[pt.rank] + pt.flags_off) + phase * kMaxPeers + src;
    if (!wait_flag_sys(flag, epoch)) report_status(status, kTimeoutPeerFlag, phase, src);
  }
}

int wait_flag_src_launch(const PeerTable& pt, int phase, uint32_t epoch, int src, int* status, cudaStream_t stream) {
  if (phase < 0 || phase >= kNumPhases || src < 0 || src >= pt.world) return (int)cudaErrorInvalidValue;
  wait_flag_src_kernel<<<1, 32, 0, stream>>>(pt, phase, epoch, src, status);
  return (int)cudaGetLastError();
}

int push_candidates_launch(const PeerTable& pt, const float* val, const int* idx, int B, int k, uint32_t epoch,
                           unsigned* done_counter, cudaStream_t stream) {
  int blocks = (int)(((long long)B * k + 255) / 256);
  if (blocks > 148 * 2) blocks = 148 * 2;
  push_candidates_kernel<<<blocks, 256, 0, stream>>>(pt, val, idx, B, k, epoch, done_counter);
  return (int)cudaGetLastError();
}

int wait_flags_launch(const PeerTable& pt, int phase, uint32_t epoch, int* status, cudaStream_t stream) {
  wait_flags_kernel<<<1, 32, 0, stream>>>(pt, phase, epoch, status);
  return (int)cudaGetLastError();
}

int sparse_decode_scatter_launch(const PeerTable& pt, const int* idx, const float* val, int B, int k, int d,
                                 const __nv_bfloat16* W, uint32_t epoch, unsigned* done_counter, cudaStream_t stream) {
  if (d % 8 != 0 || d > SC_THREADS * SC_MAX_VEC * 8 || B % pt.world != 0) return (int)cudaErrorInvalidValue;
  int blocks = B < 148 * 4 ? B : 148 * 4;
  sparse_decode_scatter_kernel<<<blocks, SC_THREADS, (size_t)k * 8, stream>>>(pt, idx, val, B, k, d, W, epoch,
                                                                              done_counter);
  return (int)cudaGetLastError();
}

int reduce_loss_push_launch(const PeerTable& pt, int B, int d, const __nv_bfloat16* label, const float* bias,
                            const float* row_weight, float grad_scale, float* loss_sum, float* xhat_out, uint32_t epoch,
                            unsigned* done_counter, int* status, cudaStream_t stream) {
  if (d % 8 != 0 || B % pt.world != 0) return (int)cudaErrorInvalidValue;
  const int rows = B / pt.world;
  int blocks = rows < 148 * 4 ? rows : 148 * 4;
  reduce_loss_push_kernel<<<blocks, 256, 0, stream>>>(pt, B, d, label, bias, row_weight, grad_scale, loss_sum, xhat_out,
                                                      epoch, done_counter, status);
  return (int)cudaGetLastError();
}

}  // namespace lmsae
