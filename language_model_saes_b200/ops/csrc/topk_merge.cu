// Exact top-k merge of per-range candidate lists.
//
// The encoder GEMM emits, for every row, C = (number of ranges) * KS candidates (gated value, column or
// -1). This kernel keeps the k best (value descending, ties by position). Under feature
// sharding it runs twice: once per rank on its own ranges (emit_gated = 1, output = k (g, local column)
// pairs that are exchanged between the shards), and once on the gathered lists of all shards, where only
// candidates in [own_lo, own_hi) -- this shard's segment -- are written out; positions won by other
// shards stay (-1, 0). That reproduces a global per-row TopK over the sharded feature axis (the job of
// distributed_topk in utils/distributed/ops.py:158-266 of the reference) with one exchange instead of
// an iterative threshold search.
#include "comm_common.cuh"

namespace lmsae {

constexpr int MERGE_WARPS = 4;

// One warp per row. Positive floats order like their bit patterns, so the k-th largest candidate is found by a
// descent over the 31 value bits (count(key >= t) per trial, one warp reduction each) instead of ranking every
// candidate against every other one; candidates equal to the threshold get the remaining places in slot order. The
// (at most k) winners are compacted into shared memory and ranked among themselves. Only winners whose candidate
// slot lies in [own_lo, own_hi) are written, in value-descending order FROM SLOT 0 ON (the rest of the row is
// (-1, 0)): consumers of a shard's codes may stop at the first empty slot.
//
// comm.mode selects what surrounds the merge under feature sharding:
//   kMergeLocal  nothing (single GPU, or lists that are exchanged by other means)
//   kMergePush   the row's k (value, column) pairs are not written to out_* but stored straight into segment
//                [rank * k, (rank + 1) * k) of EVERY rank's merge input (the all-gather of the candidate lists by
//                peer stores, fused into the kernel that produces them); the last block publishes the epoch
//   kMergeWait   the kernel first waits (bounded) until every rank has published the epoch for the candidate
//                phase, then merges the gathered lists it finds in this rank's own buffer
__global__ void __launch_bounds__(MERGE_WARPS * 32)
topk_merge_kernel(const float* cand_val, const int* cand_idx, int M, int C, int k,  // may be peer-written: no read-only path
                  const float* __restrict__ gate, int own_lo, int own_hi, int emit_gated,
                  int* __restrict__ out_idx, float* __restrict__ out_val, const MergeComm comm) {
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned lt_mask = (1u << lane) - 1u;
  // per warp: keys[C], ids[C], winner keys[k], winner slots[k], staged output ids[k] and values[k]
  uint32_t* skey = reinterpret_cast<uint32_t*>(smem_raw) + (size_t)warp * (2 * C + 4 * k);
  int* sidx = reinterpret_cast<int*>(skey + C);
  uint32_t* wkey = reinterpret_cast<uint32_t*>(sidx + C);
  int* wslot = reinterpret_cast<int*>(wkey + k);
  int* oidx = wslot + k;
  float* oval = reinterpret_cast<float*>(oidx + k);

  bool inputs_ok = true;
  if (comm.mode == kMergeWait) inputs_ok = wait_all_sources(comm.pt, kPhaseCand, comm.epoch, comm.status);

  for (int row = blockIdx.x * MERGE_WARPS + warp; row < M; row += gridDim.x * MERGE_WARPS) {
    for (int i = lane; i < k; i += 32) {
      oidx[i] = -1;
      oval[i] = 0.0f;
    }
    if (inputs_ok) {
      const float* cv = cand_val + (size_t)row * C;
      const int* ci = cand_idx + (size_t)row * C;
      for (int i = lane; i < C; i += 32) {
        const int id = ci[i];
        const float v = cv[i];
        sidx[i] = id;
        skey[i] = (id >= 0 && v > 0.0f) ? __float_as_uint(v) : 0u;  // only positive candidates compete
      }
      __syncwarp();
      // threshold: the largest t with count(key >= t) >= k (0 when fewer than k candidates are positive)
      uint32_t t = 0;
      for (int bit = 30; bit >= 0; --bit) {
        const uint32_t trial = t | (1u << bit);
        int c = 0;
        for (int i = lane; i < C; i += 32) c += skey[i] >= trial;
        if (__reduce_add_sync(0xffffffffu, c) >= k) t = trial;
      }
      int above = 0;
      for (int i = lane; i < C; i += 32) above += skey[i] > t;
      above = __reduce_add_sync(0xffffffffu, above);
      const int ties_wanted = (t == 0u) ? 0 : k - above;  // t == 0: every positive candidate is in, nothing equals t
      // compaction of the winners in slot order
      int n_win = 0, ties_seen = 0;
      for (int base = 0; base < C; base += 32) {
        const int i = base + lane;
        const uint32_t key = i < C ? skey[i] : 0u;
        const bool eq = t != 0u && key == t;
        const unsigned eq_ballot = __ballot_sync(0xffffffffu, eq);
        const bool win = key > t || (eq && ties_seen + __popc(eq_ballot & lt_mask) < ties_wanted);
        const unsigned win_ballot = __ballot_sync(0xffffffffu, win);
        if (win) {
          const int pos = n_win + __popc(win_ballot & lt_mask);
          wkey[pos] = key;
          wslot[pos] = i;
        }
        n_win += __popc(win_ballot);
        ties_seen += __popc(eq_ballot);
      }
      __syncwarp();
      // place of each of this shard's winners among this shard's winners (value descending, earlier slot first
      // among equals)
      for (int w = lane; w < n_win; w += 32) {
        const int slot = wslot[w];
        if (slot < own_lo || slot >= own_hi) continue;
        const uint32_t key = wkey[w];
        int place = 0;
        for (int j = 0; j < n_win; ++j) {
          const uint32_t u = wkey[j];
          const int sj = wslot[j];
          place += (sj >= own_lo && sj < own_hi) && ((u > key) || (u == key && sj < slot));
        }
        const int id = sidx[slot];
        const float v = __uint_as_float(key);
        oidx[place] = id;
        oval[place] = (!emit_gated && gate != nullptr) ? v / gate[id] : v;
      }
    }
    __syncwarp();
    if (comm.mode == kMergePush) {
      const size_t o = (size_t)row * ((size_t)comm.pt.world * k) + (size_t)comm.pt.rank * k;
      for (int p = 0; p < comm.pt.world; ++p) {
        float* dv = reinterpret_cast<float*>(comm.pt.base[p] + comm.pt.cand_val_off) + o;
        int* di = reinterpret_cast<int*>(comm.pt.base[p] + comm.pt.cand_idx_off) + o;
        for (int i = lane; i < k; i += 32) {
          dv[i] = oval[i];
          di[i] = oidx[i];
        }
      }
    } else {
      for (int i = lane; i < k; i += 32) {
        out_idx[(size_t)row * k + i] = oidx[i];
        out_val[(size_t)row * k + i] = oval[i];
      }
    }
    __syncwarp();
  }
  if (comm.mode == kMergePush) signal_peers_when_grid_done(comm.pt, kPhaseCand, comm.epoch, comm.done_counter);
}

int topk_merge_launch(const float* cand_val, const int* cand_idx, int M, int C, int k, const float* gate,
                      int own_lo, int own_hi, int emit_gated, int* out_idx, float* out_val, const MergeComm& comm,
                      cudaStream_t stream) {
  const size_t smem = (size_t)MERGE_WARPS * (2 * (size_t)C + 4 * (size_t)k) * 4;
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (comm.mode != kMergePush && (out_idx == nullptr || out_val == nullptr)) return (int)cudaErrorInvalidValue;
  cudaError_t e = cudaFuncSetAttribute(topk_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  int blocks = (M + MERGE_WARPS - 1) / MERGE_WARPS;
  if (blocks > 148 * 8) blocks = 148 * 8;
  topk_merge_kernel<<<blocks, MERGE_WARPS * 32, smem, stream>>>(cand_val, cand_idx, M, C, k, gate, own_lo, own_hi,
                                                               emit_gated, out_idx, out_val, comm);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// Row top-k over a materialised bf16 matrix H[M, N] (used when k is larger than the fused epilogue
// supports, for Aux-K over dead features and for the generic autograd path).
// One CTA per row. Pass 1 finds the k-th largest gated value by a radix descent over the fp32 bit pattern
// (4 passes of 8 bits, 256-bin histogram in shared memory); pass 2 writes the survivors.
// value = H * gate (gate optional) * alive (alive optional byte mask: only features with alive != 0
// compete); only values > 0 compete.
// ------------------------------------------------------------------------------------------------
constexpr int RT_THREADS = 512;

__device__ __forceinline__ float gated_value(const __nv_bfloat16* __restrict__ hrow, const float* __restrict__ gate,
                                             const uint8_t* __restrict__ alive, int c) {
  float v = __bfloat162float(hrow[c]);
  if (gate != nullptr) v *= gate[c];
  if (alive != nullptr && alive[c] == 0) v = 0.0f;
  return v;
}

__global__ void __launch_bounds__(RT_THREADS)
row_topk_kernel(const __nv_bfloat16* __restrict__ H, long long ldh, int M, int N, int k,
                const float* __restrict__ gate, const uint8_t* __restrict__ alive, int* __restrict__ out_idx,
                float* __restrict__ out_val) {
  __shared__ unsigned hist[256];
  __shared__ unsigned s_prefix, s_remaining, s_count_gt, s_cursor_gt, s_cursor_eq;
  const int row = blockIdx.x;
  if (row >= M) return;
  const __nv_bfloat16* hrow = H + (long long)row * ldh;

  unsigned prefix = 0;     // bits decided so far (from the top)
  unsigned remaining = k;  // how many of the top-k are still inside the undecided bucket
  bool fewer_than_k = false;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = threadIdx.x; i < 256; i += RT_THREADS) hist[i] = 0;
    __syncthreads();
    const unsigned hi_mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int c = threadIdx.x; c < N; c += RT_THREADS) {
      const float v = gated_value(hrow, gate, alive, c);
      if (v > 0.0f) {
        const unsigned b = __float_as_uint(v);
        if ((b & hi_mask) == prefix) atomicAdd(&hist[(b >> shift) & 0xff], 1u);
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned acc = 0;
      int bin = 255;
      for (; bin >= 0; --bin) {
        if (acc + hist[bin] >= remaining) break;
        acc += hist[bin];
      }
      if (bin < 0) {  // fewer than `remaining` positive values in this bucket: keep them all
        s_prefix = 0xffffffffu;
        s_remaining = 0;
      } else {
        s_prefix = prefix | ((unsigned)bin << shift);
        s_remaining = remaining - acc;
      }
    }
    __syncthreads();
    if (s_prefix == 0xffffffffu) {
      fewer_than_k = true;
      break;
    }
    prefix = s_prefix;
    remaining = s_remaining;
    __syncthreads();
  }
  // threshold bit pattern = prefix (exact k-th value); `remaining` = how many equal to it to keep
  const unsigned thr = fewer_than_k ? 0u : prefix;
  if (threadIdx.x == 0) {
    s_cursor_gt = 0;
    s_cursor_eq = 0;
    s_count_gt = fewer_than_k ? 0u : (unsigned)k - remaining;
  }
  for (int i = threadIdx.x; i < k; i += RT_THREADS) {
    out_idx[(size_t)row * k + i] = -1;
    out_val[(size_t)row * k + i] = 0.0f;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < N; c += RT_THREADS) {
    const float v = gated_value(hrow, gate, alive, c);
    if (v > 0.0f) {
      const unsigned b = __float_as_uint(v);
      int pos = -1;
      if (fewer_than_k || b > thr) {
        pos = (int)atomicAdd(&s_cursor_gt, 1u);
      } else if (b == thr) {
        const unsigned e = atomicAdd(&s_cursor_eq, 1u);
        if (e < remaining) pos = (int)(s_count_gt + e);
      }
      if (pos >= 0 && pos < k) {
        out_idx[(size_t)row * k + pos] = c;
        out_val[(size_t)row * k + pos] = (gate != nullptr) ? v / gate[c] : v;
      }
    }
  }
}

int row_topk_launch(const __nv_bfloat16* H, long long ldh, int M, int N, int k, const float* gate,
                    const uint8_t* alive, int* out_idx, float* out_val, cudaStream_t stream) {
  row_topk_kernel<<<M, RT_THREADS, 0, stream>>>(H, ldh, M, N, k, gate, alive, out_idx, out_val);
  return (int)cudaGetLastError();
}

}  // namespace lmsae
