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
#include "comm_common.cuh"

namespace lmsae {

LMSAE_DEFINE_BOUNDS_FETCH(bounds_fetch_comm_ops)

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
// Sparse decode of this shard's codes whose epilogue is the reduce-scatter of the partial reconstruction.
//   PT       element type of the partial rows on the wire: float, or __nv_bfloat16 (half the NVLink bytes; what a
//            bf16 all-reduce of the decoder output moves)
//   LOCAL    false: each finished row is stored into slot [rank] of the landing zone of the rank that OWNS the row
//            (peer store); true: rows stay in this rank's own buffer as [B][d] and the owner pulls the sum of all
//            ranks' copies through the switch (multimem.ld_reduce in reduce_loss_push_kernel)
// `compact`: codes of a row are packed from slot 0 on (what the merge kernel writes), so the slot loop stops at the
// first empty one; under feature sharding a row holds about k / world codes.
// ---------------------------------------------------------------------------------------------
constexpr int SC_THREADS = 512;
constexpr int SC_MAX_VEC = 2;
constexpr int SC_UNROLL = 4;

template <typename PT, bool LOCAL>
__global__ void __launch_bounds__(SC_THREADS)
sparse_decode_scatter_kernel(const PeerTable pt, const int* __restrict__ idx, const float* __restrict__ val, int B, int k,
                             int d, int F, const __nv_bfloat16* __restrict__ W, int compact, uint32_t epoch,
                             unsigned* done_counter) {
#ifdef LMSAE_BOUNDS_CHECK
  if (threadIdx.x == 0) lmsae_jitter();  // debug build: blocks start their stores at perturbed times
  __syncthreads();
#endif
  const int nvec = d / 8;
  const int rows_per_rank = B / pt.world;
  for (int row = blockIdx.x; row < B; row += gridDim.x) {
    const int* ridx = idx + (size_t)row * k;
    const float* rval = val + (size_t)row * k;
    float acc[SC_MAX_VEC][8];
#pragma unroll
    for (int u = 0; u < SC_MAX_VEC; ++u)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[u][i] = 0.0f;
    for (int j0 = 0; j0 < k; j0 += SC_UNROLL) {
      // the codes of a row are the same for every thread: these loads are broadcasts served by L1
      int f[SC_UNROLL];
      float a[SC_UNROLL];
#pragma unroll
      for (int t = 0; t < SC_UNROLL; ++t) {
        const int j = j0 + t;
        f[t] = j < k ? __ldg(ridx + j) : -1;
        a[t] = j < k ? __ldg(rval + j) : 0.0f;
      }
      if (compact && f[0] < 0) break;
      // all gathers of the group are issued before the first is used
      uint4 w[SC_UNROLL][SC_MAX_VEC];
#pragma unroll
      for (int t = 0; t < SC_UNROLL; ++t) {
        const uint4* wrow = reinterpret_cast<const uint4*>(W + (size_t)(f[t] < 0 ? 0 : LMSAE_IDX(f[t], F)) * d);
#pragma unroll
        for (int u = 0; u < SC_MAX_VEC; ++u) {
          const int v = threadIdx.x + u * SC_THREADS;
          w[t][u] = (f[t] >= 0 && v < nvec) ? __ldg(wrow + v) : make_uint4(0u, 0u, 0u, 0u);
        }
      }
#pragma unroll
      for (int t = 0; t < SC_UNROLL; ++t)
#pragma unroll
        for (int u = 0; u < SC_MAX_VEC; ++u) {
          float wf[8];
          bf16x8_to_float_c(w[t][u], wf);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[u][i] = fmaf(a[t], wf[i], acc[u][i]);
        }
    }
    // epilogue = reduce-scatter
    const int owner = row / rows_per_rank;
    const int lrow = row - owner * rows_per_rank;
    PT* dst = LOCAL ? reinterpret_cast<PT*>(pt.base[pt.rank] + pt.partial_off) + (size_t)row * d
                    : reinterpret_cast<PT*>(pt.base[owner] + pt.partial_off) + ((size_t)pt.rank * rows_per_rank + lrow) * d;
#pragma unroll
    for (int u = 0; u < SC_MAX_VEC; ++u) {
      const int v = threadIdx.x + u * SC_THREADS;
      if (v < nvec) {
        if constexpr (sizeof(PT) == 4) {
          float4* o = reinterpret_cast<float4*>(dst + v * 8);
          o[0] = make_float4(acc[u][0], acc[u][1], acc[u][2], acc[u][3]);
          o[1] = make_float4(acc[u][4], acc[u][5], acc[u][6], acc[u][7]);
        } else {
          *reinterpret_cast<uint4*>(dst + v * 8) = float8_to_bf16x8(acc[u]);
        }
      }
    }
  }
  signal_peers_when_grid_done(pt, kPhasePartial, epoch, done_counter);
}

// ---------------------------------------------------------------------------------------------
// The owner of a block of rows sums the partial reconstructions of all shards (+ bias), evaluates the loss and its
// gradient and all-gathers the bf16 gradient rows into every rank's [B][d] buffer.
//   MC = false  partials are read from the `world` slots of this rank's landing zone; the gradient row is stored into
//               every peer (world peer stores per 16 bytes)
//   MC = true   one multimem.ld_reduce per 16 bytes returns the sum over all ranks' [B][d] buffers (added inside the
//               NVSwitch), one multimem.st publishes the gradient to every rank
// ---------------------------------------------------------------------------------------------
template <typename PT, bool MC>
__global__ void __launch_bounds__(256)
reduce_loss_push_kernel(const PeerTable pt, int B, int d, const __nv_bfloat16* __restrict__ label,
                        const float* __restrict__ bias, const float* __restrict__ row_weight, float grad_scale,
                        float* __restrict__ loss_sum, float* __restrict__ xhat_out, uint32_t epoch_in, uint32_t epoch_out,
                        unsigned* done_counter, int* status) {
  __shared__ float s_red[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows_per_rank = B / pt.world;
  const bool ok = wait_all_sources(pt, kPhasePartial, epoch_in, status);
  if (ok) {
    const PT* partial = reinterpret_cast<const PT*>(pt.base[pt.rank] + pt.partial_off);
    const int nvec = d / 8;
    for (int lrow = blockIdx.x; lrow < rows_per_rank; lrow += gridDim.x) {
      const int row = pt.rank * rows_per_rank + lrow;
      const float rw = row_weight != nullptr ? row_weight[row] : 1.0f;
      float sq = 0.0f;
      for (int v = threadIdx.x; v < nvec; v += 256) {
        float x[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = bias != nullptr ? bias[v * 8 + i] : 0.0f;
        if constexpr (MC) {
          const char* mc = pt.mc_base + pt.partial_off + ((size_t)row * d + (size_t)v * 8) * sizeof(__nv_bfloat16);
          float t[8];
          bf16x8_to_float_c(multimem_ld_reduce_add_bf16x8(mc), t);
#pragma unroll
          for (int i = 0; i < 8; ++i) x[i] += t[i];
        } else if constexpr (sizeof(PT) == 4) {
          for (int s = 0; s < pt.world; ++s) {
            const float4* src = reinterpret_cast<const float4*>(partial + ((size_t)s * rows_per_rank + lrow) * d + v * 8);
            const float4 a = src[0], b = src[1];
            x[0] += a.x; x[1] += a.y; x[2] += a.z; x[3] += a.w;
            x[4] += b.x; x[5] += b.y; x[6] += b.z; x[7] += b.w;
          }
        } else {
          // issue the loads of all slots before the first conversion (world <= 8)
          uint4 raw[kMaxPeers];
#pragma unroll
          for (int s = 0; s < kMaxPeers; ++s)
            if (s < pt.world)
              raw[s] = *(reinterpret_cast<const uint4*>(partial + ((size_t)s * rows_per_rank + lrow) * d) + v);
#pragma unroll
          for (int s = 0; s < kMaxPeers; ++s)
            if (s < pt.world) {
              float t[8];
              bf16x8_to_float_c(raw[s], t);
#pragma unroll
              for (int i = 0; i < 8; ++i) x[i] += t[i];
            }
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
        const uint4 o = float8_to_bf16x8(e);
        const size_t off16 = ((size_t)row * d) / 8 + v;
        if constexpr (MC) {
          multimem_st_16B(reinterpret_cast<uint4*>(pt.mc_base + pt.dxhat_off) + off16, o);
        } else {
          // all-gather of the gradient rows: store into every rank's full [B, d] gradient buffer
          for (int p = 0; p < pt.world; ++p) *(reinterpret_cast<uint4*>(pt.base[p] + pt.dxhat_off) + off16) = o;
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
  signal_peers_when_grid_done(pt, kPhaseDxhat, epoch_out, done_counter);
}

// ---------------------------------------------------------------------------------------------
// All-gather of several row-sharded tensors over a (data-parallel) group in ONE kernel: every rank stores its part of
// each tensor at offset rank * nbytes of the gathered tensor in every rank's buffer (its own included), the last block
// publishes the epoch and then waits (bounded) for the other ranks' flags, so that the kernels after this one in the
// stream find every rank's rows in place. Replaces one collective per tensor (x, d x_hat and the three code tensors of
// a data-parallel step).
//
// MC: one multimem.st per 16 bytes through the multicast mapping; the switch replicates it into every rank's buffer,
// so a rank sends its rows over its link once instead of once per peer.
template <bool MC>
__global__ void __launch_bounds__(256)
exchange_rows_kernel(const PeerTable pt, const RowExchange ex, uint32_t epoch, unsigned* done_counter, int* status) {
#ifdef LMSAE_BOUNDS_CHECK
  if (threadIdx.x == 0) lmsae_jitter();  // debug build: blocks start their stores at perturbed times
  __syncthreads();
#endif
  for (int i = 0; i < ex.n; ++i) {
    const uint4* s = reinterpret_cast<const uint4*>(ex.src[i]);
    const long long nvec = ex.nbytes[i] / 16;
    const long long off = ex.dst_off[i] + (long long)pt.rank * ex.nbytes[i];
    if constexpr (MC) {
      uint4* dst = reinterpret_cast<uint4*>(pt.mc_base + off);
      for (long long v = blockIdx.x * 256LL + threadIdx.x; v < nvec; v += (long long)gridDim.x * 256)
        multimem_st_16B(dst + v, __ldg(s + v));
    } else {
      for (int p = 0; p < pt.world; ++p) {
        uint4* dst = reinterpret_cast<uint4*>(pt.base[p] + off);
        for (long long v = blockIdx.x * 256LL + threadIdx.x; v < nvec; v += (long long)gridDim.x * 256) dst[v] = __ldg(s + v);
      }
    }
  }
  const bool last = signal_peers_when_grid_done(pt, kPhaseRows, epoch, done_counter);
  if (last) wait_all_sources(pt, kPhaseRows, epoch, status, /*record_always=*/true);
}

int exchange_rows_launch(const PeerTable& pt, const RowExchange& ex, uint32_t epoch, unsigned* done_counter, int* status,
                         bool use_multicast, cudaStream_t stream) {
  if (ex.n < 1 || ex.n > 8) return (int)cudaErrorInvalidValue;
  if (use_multicast && pt.mc_base == nullptr) return (int)cudaErrorInvalidValue;
  long long total = 0;
  for (int i = 0; i < ex.n; ++i) total += ex.nbytes[i] / 16;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  if (blocks < 1) blocks = 1;
  if (use_multicast) exchange_rows_kernel<true><<<(int)blocks, 256, 0, stream>>>(pt, ex, epoch, done_counter, status);
  else exchange_rows_kernel<false><<<(int)blocks, 256, 0, stream>>>(pt, ex, epoch, done_counter, status);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// In-place all-reduce (sum) of a bf16 array that every rank holds at the same offset of its symmetric buffer, in one
// kernel: the crosscoder's sum of encoder pre-activations over head ranks (models/crosscoder.py:350-375 of the
// reference project all-reduces that [batch, d_sae] tensor with NCCL). Protocol:
//   1. block 0 publishes "my array is written" (phase_in) to every rank; every block waits for all ranks' flags
//   2. rank r owns the r-th share of the 16-byte vectors. MC: one multimem.ld_reduce returns the sum over all ranks'
//      copies (added inside the NVSwitch, fp32 accumulation) and one multimem.st writes it back into every rank's copy.
//      Without a multicast mapping the same is done with `world` peer loads and `world` peer stores.
//      No element is read after its owner has overwritten it: only the owner reads it at all.
//   3. the last block publishes "my share is reduced everywhere" (phase_out) and waits for the other ranks' flags, so
//      that the kernels behind this one in the stream find the complete sums.
// ---------------------------------------------------------------------------------------------
template <bool MC>
__global__ void __launch_bounds__(512)
allreduce_bf16_inplace_kernel(const PeerTable pt, long long off, long long n16, int phase_in, int phase_out, uint32_t epoch,
                              unsigned* done_counter, int* status) {
  if (blockIdx.x == 0) {
    __threadfence_system();
    if ((int)threadIdx.x < pt.world) st_release_sys(flag_slot(pt, threadIdx.x, phase_in, pt.rank), epoch);
  }
  const bool ok = wait_all_sources(pt, phase_in, epoch, status);
  if (ok) {
    const long long per = (n16 + pt.world - 1) / pt.world;
    const long long lo = per * pt.rank, hi = lo + per < n16 ? lo + per : n16;
    constexpr int U = 4;  // vectors per thread and round: their loads are all in flight before the first store
    const long long stride = (long long)gridDim.x * 512;
    for (long long v0 = lo + blockIdx.x * 512LL + threadIdx.x; v0 < hi; v0 += stride * U) {
      if constexpr (MC) {
        uint4 r[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long v = v0 + u * stride;
          if (v < hi) r[u] = multimem_ld_reduce_add_bf16x8(pt.mc_base + off + v * 16);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long v = v0 + u * stride;
          if (v < hi) multimem_st_16B(pt.mc_base + off + v * 16, r[u]);
        }
      } else {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long v = v0 + u * stride;
          if (v >= hi) break;
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          uint4 raw[kMaxPeers];
#pragma unroll
          for (int s = 0; s < kMaxPeers; ++s)
            if (s < pt.world) raw[s] = *(reinterpret_cast<const uint4*>(pt.base[s] + off) + v);
#pragma unroll
          for (int s = 0; s < kMaxPeers; ++s)
            if (s < pt.world) {
              float t[8];
              bf16x8_to_float_c(raw[s], t);
#pragma unroll
              for (int i = 0; i < 8; ++i) acc[i] += t[i];
            }
          const uint4 o = float8_to_bf16x8(acc);
          for (int s = 0; s < pt.world; ++s) *(reinterpret_cast<uint4*>(pt.base[s] + off) + v) = o;
        }
      }
    }
  }
  const bool last = signal_peers_when_grid_done(pt, phase_out, epoch, done_counter);
  if (last) wait_all_sources(pt, phase_out, epoch, status, /*record_always=*/true);
}

int allreduce_bf16_launch(const PeerTable& pt, long long off, long long n16, int phase_in, int phase_out, uint32_t epoch,
                          int use_multicast, unsigned* done_counter, int* status, cudaStream_t stream) {
  if (phase_in < 0 || phase_in >= kNumPhases || phase_out < 0 || phase_out >= kNumPhases || phase_in == phase_out)
    return (int)cudaErrorInvalidValue;
  if (use_multicast && pt.mc_base == nullptr) return (int)cudaErrorInvalidValue;
  // every block waits at the start: the grid must be resident at once (one CTA of 512 threads per SM at most two)
  const int blocks = 148 * 2;
  if (use_multicast)
    allreduce_bf16_inplace_kernel<true><<<blocks, 512, 0, stream>>>(pt, off, n16, phase_in, phase_out, epoch, done_counter, status);
  else
    allreduce_bf16_inplace_kernel<false><<<blocks, 512, 0, stream>>>(pt, off, n16, phase_in, phase_out, epoch, done_counter, status);
  return (int)cudaGetLastError();
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
// MC: the stores go through the NVSwitch multicast mapping (multimem.st), one message for all ranks.
template <typename TI, typename TO, bool MC>
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
      if constexpr (MC) {
        TO* dst = reinterpret_cast<TO*>(pt.mc_base + recv_off) + (size_t)o * d + c;
        if constexpr (sizeof(TO) == 4) {
          uint4 lo, hi;
          lo.x = __float_as_uint(f[0]); lo.y = __float_as_uint(f[1]); lo.z = __float_as_uint(f[2]); lo.w = __float_as_uint(f[3]);
          hi.x = __float_as_uint(f[4]); hi.y = __float_as_uint(f[5]); hi.z = __float_as_uint(f[6]); hi.w = __float_as_uint(f[7]);
          multimem_st_16B(dst, lo);
          multimem_st_16B(dst + 4, hi);
        } else {
          multimem_st_16B(dst, float8_to_bf16x8(f));
        }
      } else {
        for (int p = 0; p < pt.world; ++p) {
          TO* dst = reinterpret_cast<TO*>(pt.base[p] + recv_off) + (size_t)o * d + c;
          if constexpr (sizeof(TO) == 4) {
            reinterpret_cast<float4*>(dst)[0] = make_float4(f[0], f[1], f[2], f[3]);
            reinterpret_cast<float4*>(dst)[1] = make_float4(f[4], f[5], f[6], f[7]);
          } else {
            *reinterpret_cast<uint4*>(dst) = float8_to_bf16x8(f);
          }
        }
      }
    }
  }
  signal_peers_when_grid_done(pt, phase, epoch, done_counter);
}

int bcast_rows_cast_launch(const PeerTable& pt, int in_dtype, int out_dtype, const void* src, const int* keep, const int* pos,
                           long long n, int d, long long recv_off, long long cap_rows, int phase, uint32_t epoch,
                           unsigned* done_counter, bool use_multicast, cudaStream_t stream) {
  if (d % 8 != 0 || recv_off % 16 != 0 || phase < 0 || phase >= kNumPhases) return (int)cudaErrorInvalidValue;
  if (use_multicast && pt.mc_base == nullptr) return (int)cudaErrorInvalidValue;
  const int blocks = (int)(n < 148LL * 8 ? (n > 0 ? n : 1) : 148LL * 8);
  using bf = __nv_bfloat16;
#define LMSAE_BCAST(TI, TO)                                                                                             \
  do {                                                                                                                  \
    if (use_multicast)                                                                                                  \
      bcast_rows_cast_kernel<TI, TO, true><<<blocks, 256, 0, stream>>>(pt, static_cast<const TI*>(src), keep, pos, n, d, \
                                                                       recv_off, cap_rows, phase, epoch, done_counter); \
    else                                                                                                                \
      bcast_rows_cast_kernel<TI, TO, false><<<blocks, 256, 0, stream>>>(pt, static_cast<const TI*>(src), keep, pos, n, \
                                                                        d, recv_off, cap_rows, phase, epoch,            \
                                                                        done_counter);                                  \
  } while (0)
  if (in_dtype == 0 && out_dtype == 0) LMSAE_BCAST(float, float);
  else if (in_dtype == 0 && out_dtype == 1) LMSAE_BCAST(float, bf);
  else if (in_dtype == 1 && out_dtype == 0) LMSAE_BCAST(bf, float);
  else if (in_dtype == 1 && out_dtype == 1) LMSAE_BCAST(bf, bf);
  else return (int)cudaErrorInvalidValue;
#undef LMSAE_BCAST
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

int sparse_decode_scatter_launch(const PeerTable& pt, const int* idx, const float* val, int B, int k, int d, int F,
                                 const __nv_bfloat16* W, int partial_dtype, int use_multicast, int compact_codes,
                                 uint32_t epoch, unsigned* done_counter, cudaStream_t stream) {
  if (d % 8 != 0 || d > SC_THREADS * SC_MAX_VEC * 8 || B % pt.world != 0) return (int)cudaErrorInvalidValue;
  if (use_multicast && (partial_dtype != 1 || pt.mc_base == nullptr)) return (int)cudaErrorInvalidValue;
  int blocks = B < 148 * 4 ? B : 148 * 4;
  using bf = __nv_bfloat16;
#define LMSAE_SCATTER(PT, LOCAL) \
  sparse_decode_scatter_kernel<PT, LOCAL><<<blocks, SC_THREADS, 0, stream>>>(pt, idx, val, B, k, d, F, W, compact_codes, epoch, done_counter)
  if (use_multicast) LMSAE_SCATTER(bf, true);
  else if (partial_dtype == 1) LMSAE_SCATTER(bf, false);
  else LMSAE_SCATTER(float, false);
#undef LMSAE_SCATTER
  return (int)cudaGetLastError();
}

int reduce_loss_push_launch(const PeerTable& pt, int B, int d, const __nv_bfloat16* label, const float* bias,
                            const float* row_weight, float grad_scale, float* loss_sum, float* xhat_out,
                            int partial_dtype, int use_multicast, uint32_t epoch_in, uint32_t epoch_out,
                            unsigned* done_counter, int* status, cudaStream_t stream) {
  if (d % 8 != 0 || B % pt.world != 0) return (int)cudaErrorInvalidValue;
  if (use_multicast && (partial_dtype != 1 || pt.mc_base == nullptr)) return (int)cudaErrorInvalidValue;
  const int rows = B / pt.world;
  int blocks = rows < 148 * 4 ? rows : 148 * 4;
  using bf = __nv_bfloat16;
#define LMSAE_REDUCE(PT, MC)                                                                                         \
  reduce_loss_push_kernel<PT, MC><<<blocks, 256, 0, stream>>>(pt, B, d, label, bias, row_weight, grad_scale, loss_sum, \
                                                              xhat_out, epoch_in, epoch_out, done_counter, status)
  if (use_multicast) LMSAE_REDUCE(bf, true);
  else if (partial_dtype == 1) LMSAE_REDUCE(bf, false);
  else LMSAE_REDUCE(float, false);
#undef LMSAE_REDUCE
  return (int)cudaGetLastError();
}

}  // namespace lmsae
