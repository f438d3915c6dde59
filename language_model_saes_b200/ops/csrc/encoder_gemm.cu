// Encoder GEMM for sparse dictionaries on sm_100a:
//
//     H[m, n] = sum_k X[m, k] * W[n, k] + bias[n]          (X, W bf16 K-major; fp32 accumulate)
//
// with two optional epilogues that run while the next tile's MMAs are in flight:
//   * WRITE_H : store H as bf16 (the "hidden_pre" tensor of the reference encoder,
//               models/sae.py:323-331 in the reference project); with a gate and no top-k, H * gate[n] is stored;
//   * TOPK    : keep, per row, the k largest *gated* values g = H * gate[n] (gate = decoder row norm when
//               sparsity_include_decoder_norm is set, models/sae.py:333-341) that are > 0, without ever
//               writing the dense pre-activation matrix. Each CTA sweeps a contiguous range of N-tiles for
//               one 128-row panel, so the running top-k state lives in shared memory for the whole sweep;
//               at the end it emits k (value, column) candidates per row for its range. A small merge
//               kernel (topk_merge.cu) combines the ranges (and, under feature sharding, the ranks).
//
// Structure (one CTA per SM, 256 threads):
//   warp 0    : TMA producer (one elected lane) -> STAGES-deep ring of {A 128x64, B 256x64} bf16 tiles,
//               128-byte swizzle, no cluster multicast
//   warp 1    : tcgen05.mma issuer (one elected lane), UMMA 128x256x16, accumulators in TMEM,
//               two 256-column accumulator buffers so the epilogue of tile i overlaps the MMAs of tile i+1
//   warp 2    : TMEM allocation / release
//   warps 4-7 : epilogue; thread r of the warpgroup owns accumulator row r (TMEM lane r)
// Every mbarrier wait is bounded; on expiry the CTA records a status code, raises a CTA-wide abort flag,
// drains and frees its TMEM.
//
// PAIR variant (tcgen05 cta_group::2): two CTAs on neighbouring SMs form a cluster and work on two adjacent
// 128-row panels with ONE 256x256x16 instruction stream issued by the leader (cluster rank 0). Each CTA loads
// its own A tile and only HALF of the B tile (128 of the 256 dictionary rows), so a stage is 32 KB instead of
// 48 KB per CTA: B crosses L2 -> shared memory once per pair, and the ring is 5-6 stages deep even with the
// 64-slot top-k state resident. Both producers complete their bytes on the LEADER's "full" barrier; the
// leader's commits arrive on the "empty" / "accumulator full" barriers of BOTH CTAs; both epilogues release an
// accumulator buffer on the leader's "accumulator empty" barrier. Each CTA's epilogue is unchanged: it reads
// its own 128 TMEM lanes (its panel's rows) x 256 columns.
#include "common.cuh"
#include "kernels.h"

namespace lmsae {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KB
constexpr int TMEM_COLS = 512;
constexpr int NUM_THREADS = 256;

template <int STAGES, int KS, bool PAIR>
struct SmemLayout {
  static constexpr int kBRows = PAIR ? BN / 2 : BN;       // dictionary rows of a B tile held by one CTA
  static constexpr int kBStageBytes = kBRows * BK * 2;    // 16 KB (pair) / 32 KB
  static constexpr int kStageBytes = A_STAGE_BYTES + kBStageBytes;
  static constexpr int kStageOff = 0;
  static constexpr int kSlotValOff = STAGES * kStageBytes;
  static constexpr int kSlotIdxOff = kSlotValOff + BM * KS * 4;
  static constexpr int kBarOff = kSlotIdxOff + BM * KS * 4;
  static constexpr int kNumBars = 2 * STAGES + 4;
  static constexpr int kTmemPtrOff = kBarOff + kNumBars * 8;
  static constexpr int kAbortOff = kTmemPtrOff + 4;
  static constexpr int kTotal = kAbortOff + 4;
  static constexpr int kDynamicBytes = kTotal + 1024;  // slack for manual 1024-byte alignment
};

// v[j] for a run-time j without spilling the register array: a 5-level tree of selects.
__device__ __forceinline__ float select32(const float (&v)[32], int j) {
  float a[16], b[8], c[4];
#pragma unroll
  for (int i = 0; i < 16; ++i) a[i] = (j & 1) ? v[2 * i + 1] : v[2 * i];
#pragma unroll
  for (int i = 0; i < 8; ++i) b[i] = (j & 2) ? a[2 * i + 1] : a[2 * i];
#pragma unroll
  for (int i = 0; i < 4; ++i) c[i] = (j & 4) ? b[2 * i + 1] : b[2 * i];
  const float d0 = (j & 8) ? c[1] : c[0];
  const float d1 = (j & 8) ? c[3] : c[2];
  return (j & 16) ? d1 : d0;
}

template <bool WRITE_H, bool TOPK, int STAGES, int KS, bool PAIR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
enc_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const EncGemmParams p) {
  using L = SmemLayout<STAGES, KS, PAIR>;
  constexpr int STAGE_BYTES = L::kStageBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full_bar = empty_bar + STAGES;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem + L::kTmemPtrOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);
  float* slot_val = reinterpret_cast<float*>(smem + L::kSlotValOff);
  int* slot_idx = reinterpret_cast<int*>(smem + L::kSlotIdxOff);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // work unit = one CTA (one panel) or one CTA pair (two adjacent panels); units of a split are consecutive
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0;
  const int unit = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int units_per_split = PAIR ? p.num_panels / 2 : p.num_panels;
  // ragged deal (p.units != 0): the first `extra` panel units get base + 1 column ranges, the others base; units of one
  // range index are consecutive within their group, so the CTAs that run together sweep the same B tiles
  int panel_unit, split, my_splits;
  if (p.units == 0) {
    panel_unit = unit % units_per_split;
    split = unit / units_per_split;
    my_splits = p.num_splits;
  } else {
    const int base = p.units / units_per_split, extra = p.units % units_per_split;
    const int first = extra * (base + 1);
    if (unit < first) {
      panel_unit = unit % extra;
      split = unit / extra;
      my_splits = base + 1;
    } else {
      const int rest = units_per_split - extra;
      panel_unit = extra + (unit - first) % rest;
      split = (unit - first) / rest;
      my_splits = base;
    }
  }
  const int panel = PAIR ? panel_unit * 2 + (int)cta_rank : panel_unit;
  const int num_n_tiles = (p.N + BN - 1) / BN;
  const int tile_begin = (int)(((long long)split * num_n_tiles) / my_splits);
  const int tile_end = (int)(((long long)(split + 1) * num_n_tiles) / my_splits);
  const int num_k_stages = (p.K + BK - 1) / BK;
  const int m0 = panel * BM;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    mbar_init(&tmem_full_bar[0], 1);
    mbar_init(&tmem_full_bar[1], 1);
    mbar_init(&tmem_empty_bar[0], PAIR ? 8 : 4);  // epilogue warps of the CTA (of both CTAs of a pair)
    mbar_init(&tmem_empty_bar[1], PAIR ? 8 : 4);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 2) {
    if constexpr (PAIR) {
      tmem_alloc_pair(tmem_ptr_smem, TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_ptr_smem, TMEM_COLS);
      tmem_relinquish();
    }
  }
  if constexpr (TOPK) {
    // slots are stored slot-major, [KS][128 rows], so that the thread owning a row reads and writes its
    // slots without bank conflicts. The first k slots hold (0, -1) = "empty, any positive value beats
    // it"; the rest hold +inf so they are never the minimum and never replaced.
    for (int i = threadIdx.x; i < BM * KS; i += NUM_THREADS) {
      const int s = i / BM;
      float v = (s < p.k) ? 0.0f : __int_as_float(0x7f800000);
      int ix = -1;
      if (p.resume_topk && s < p.k) {
        // continue the sweep of an earlier launch: its result for (row, this column range) is the state
        const int r = m0 + (i - s * BM);
        if (r < p.M) {
          const long long o = (long long)r * ((long long)p.num_splits * KS) + (long long)split * KS + s;
          v = p.cand_val[o];
          ix = p.cand_idx[o];
        }
      }
      slot_val[i] = v;
      slot_idx[i] = ix;
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      const int k_stages_per_head = p.heads > 1 ? num_k_stages / p.heads : num_k_stages;
      for (int tile = tile_begin; tile < tile_end && ok; ++tile) {
        const int n0 = tile * BN;
        for (int ks = 0; ks < num_k_stages; ++ks, ++it) {
          const int s = it % STAGES;
          const uint32_t parity = ((it / STAGES) & 1) ^ 1;
          // head-summed encoders: K block ks belongs to head h and reads that head's rows of the weight map
          const int head = ks / k_stages_per_head;
          const int bk = (ks - head * k_stages_per_head) * BK;
          const int brow = n0 + head * p.b_rows_per_head;
          if (!mbar_wait_bounded(&empty_bar[s], parity, abort_flag)) {
            report_status(p.status, kTimeoutEmptyBarrier, (int)it);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + L::kStageOff + s * STAGE_BYTES;
          uint8_t* b_dst = a_dst + A_STAGE_BYTES;
          if constexpr (PAIR) {
            // the leader's barrier counts the bytes of both CTAs; bytes landing before the leader has
            // announced them only make the pending count negative for a moment
            if (leader) mbar_arrive_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
            const uint32_t bar = mapa_u32(smem_u32(&full_bar[s]), 0);
            tma_load_2d_pair(a_dst, &tmap_a, bar, ks * BK, m0);
            tma_load_2d_pair(b_dst, &tmap_b, bar, bk, brow + (int)cta_rank * L::kBRows);
          } else {
            mbar_arrive_expect_tx(&full_bar[s], STAGE_BYTES);
            tma_load_2d(a_dst, &tmap_a, &full_bar[s], ks * BK, m0);
            tma_load_2d(b_dst, &tmap_b, &full_bar[s], bk, brow);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (pair: leader CTA only)
    if ((!PAIR || leader) && elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(PAIR ? 2 * BM : BM, BN);
      uint32_t it = 0;
      bool ok = true;
      int lt = 0;
      for (int tile = tile_begin; tile < tile_end && ok; ++tile, ++lt) {
        const int buf = lt & 1;
        const uint32_t acc_parity = ((lt >> 1) & 1) ^ 1;
        if (!mbar_wait_bounded(&tmem_empty_bar[buf], acc_parity, abort_flag)) {
          report_status(p.status, kTimeoutTmemEmpty, lt);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        for (int ks = 0; ks < num_k_stages; ++ks, ++it) {
          const int s = it % STAGES;
          const uint32_t parity = (it / STAGES) & 1;
          if (!mbar_wait_bounded(&full_bar[s], parity, abort_flag)) {
            report_status(p.status, kTimeoutFullBarrier, (int)it);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + L::kStageOff + s * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_STAGE_BYTES;
          const uint64_t a_desc = make_sw128_kmajor_desc(a_addr);
          const uint64_t b_desc = make_sw128_kmajor_desc(b_addr);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            // +32 bytes per 16-element K step: the start-address field is in 16-byte units
            const uint32_t acc = (ks > 0 || kk > 0) ? 1u : 0u;
            if constexpr (PAIR) {
              umma_bf16_ss_pair(tmem_d, a_desc + (uint64_t)(kk * 2), b_desc + (uint64_t)(kk * 2), idesc, acc);
            } else {
              umma_bf16_ss(tmem_d, a_desc + (uint64_t)(kk * 2), b_desc + (uint64_t)(kk * 2), idesc, acc);
            }
          }
          // stage reusable (in both CTAs of a pair) once these MMAs have read it
          if constexpr (PAIR) umma_commit_pair(&empty_bar[s], 3); else umma_commit(&empty_bar[s]);
        }
        if (ok) {
          if constexpr (PAIR) umma_commit_pair(&tmem_full_bar[buf], 3); else umma_commit(&tmem_full_bar[buf]);
        }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue
    const int q = warp - 4;             // TMEM lane quarter of this warp
    const int row_in_tile = q * 32 + lane;
    const int row = m0 + row_in_tile;
    const bool row_ok = row < p.M;
    // Running top-k of this thread's row. The KS slots form groups of 8; gmin[g] caches the smallest
    // value of group g in a register, tau = min(gmin) is the value a candidate has to beat. An insert
    // touches one group only: 8 shared-memory reads, 2 writes.
    constexpr int NG = KS > 0 ? KS / 8 : 1;
    float gmin[NG];
    float tau = 0.0f;
    float* my_slot_val = slot_val + row_in_tile;
    int* my_slot_idx = slot_idx + row_in_tile;
    if constexpr (TOPK) {
      // (the slot arrays were filled before the CTA-wide barrier above)
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        float m = __int_as_float(0x7f800000);
        if (p.resume_topk) {
#pragma unroll
          for (int t = 0; t < 8; ++t) m = fminf(m, my_slot_val[(g * 8 + t) * BM]);
        } else if (g * 8 < p.k) {
          m = 0.0f;
        }
        gmin[g] = m;
        tau = (g == 0) ? m : fminf(tau, m);
      }
    }
    int lt = 0;
    bool ok = true;
    for (int tile = tile_begin; tile < tile_end && ok; ++tile, ++lt) {
      const int buf = lt & 1;
      const uint32_t parity = (lt >> 1) & 1;
      if (!mbar_wait_bounded(&tmem_full_bar[buf], parity, abort_flag)) {
        if (lane == 0) report_status(p.status, kTimeoutTmemFull, lt);
        *abort_flag = 1;
        ok = false;
        break;
      }
      tc_fence_after();
      const int n0 = tile * BN;
      const uint32_t taddr_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
#pragma unroll 1
      for (int chunk = 0; chunk < BN / 32; ++chunk) {
        const int c0 = n0 + chunk * 32;
        if (c0 >= p.N) break;  // uniform across the CTA
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr_row + (uint32_t)(chunk * 32), r);
        tmem_wait_ld();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        const bool full_chunk = (c0 + 32 <= p.N);
        if (p.bias != nullptr) {
          if (full_chunk) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const float4 b4 = __ldg(reinterpret_cast<const float4*>(p.bias + c0 + j));
              v[j] += b4.x; v[j + 1] += b4.y; v[j + 2] += b4.z; v[j + 3] += b4.w;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) if (c0 + j < p.N) v[j] += __ldg(p.bias + c0 + j);
          }
        }
        if constexpr (WRITE_H && !TOPK) {
          // plain store variants: an optional per-column gate (decoder row norm) is applied to the stored value
          if (p.gate != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) if (full_chunk || c0 + j < p.N) v[j] *= __ldg(p.gate + c0 + j);
          }
        }
        if constexpr (WRITE_H) {
          if (row_ok) {
            __nv_bfloat16* dst = p.H + (long long)row * p.ldh + c0;
            if (full_chunk) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 o;
                o.x = pack_bf16x2(v[j], v[j + 1]);
                o.y = pack_bf16x2(v[j + 2], v[j + 3]);
                o.z = pack_bf16x2(v[j + 4], v[j + 5]);
                o.w = pack_bf16x2(v[j + 6], v[j + 7]);
                *reinterpret_cast<uint4*>(dst + j) = o;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) if (c0 + j < p.N) dst[j] = __float2bfloat16(v[j]);
            }
          }
        }
        if constexpr (TOPK) {
          if (p.gate != nullptr) {
            if (full_chunk) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                const float4 g4 = __ldg(reinterpret_cast<const float4*>(p.gate + c0 + j));
                v[j] *= g4.x; v[j + 1] *= g4.y; v[j + 2] *= g4.z; v[j + 3] *= g4.w;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) if (c0 + j < p.N) v[j] *= __ldg(p.gate + c0 + j);
            }
          }
          if (!row_ok) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = -1.0f;
          }
          // Which of this row's 32 values beat the current threshold? Usually none. The rare inserts run
          // in a per-thread loop (one copy of the insert code; lanes work on different columns at once).
          uint32_t pending = 0;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const bool in_range = full_chunk || (c0 + j < p.N);
            pending |= (in_range && v[j] > tau) ? (1u << j) : 0u;
          }
          while (pending != 0) {
            const int j = __ffs(pending) - 1;
            pending &= pending - 1;
            const float g = select32(v, j);
            if (g > tau) {
              int gi = 0;
              float gm = gmin[0];
#pragma unroll
              for (int t = 1; t < NG; ++t) {
                if (gmin[t] < gm) { gm = gmin[t]; gi = t; }
              }
              float* gv = my_slot_val + gi * 8 * BM;
              float sv[8];
#pragma unroll
              for (int t = 0; t < 8; ++t) sv[t] = gv[t * BM];
              int sel = 0;
#pragma unroll
              for (int t = 7; t >= 0; --t) sel = (sv[t] == gm) ? t : sel;
              gv[sel * BM] = g;
              my_slot_idx[(gi * 8 + sel) * BM] = p.n_index_offset + c0 + j;
              float nm = g;
#pragma unroll
              for (int t = 0; t < 8; ++t) nm = fminf(nm, (t == sel) ? g : sv[t]);
              float nt = nm;
#pragma unroll
              for (int t = 0; t < NG; ++t) {
                gmin[t] = (t == gi) ? nm : gmin[t];
                nt = fminf(nt, gmin[t]);
              }
              tau = nt;
            }
          }
        }
      }
      // release this accumulator buffer to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (PAIR) mbar_arrive_cluster(mapa_u32(smem_u32(&tmem_empty_bar[buf]), 0));
        else mbar_arrive(&tmem_empty_bar[buf]);
      }
    }
    if constexpr (TOPK) if (ok && row_ok) {
      // emit this sweep's candidates: [row][split * KS + slot]
      const long long o = (long long)row * ((long long)p.num_splits * KS) + (long long)split * KS;
      for (int s = 0; s < KS; ++s) {
        const bool valid = s < p.k;
        p.cand_val[o + s] = valid ? my_slot_val[s * BM] : 0.0f;
        p.cand_idx[o + s] = valid ? my_slot_idx[s * BM] : -1;
      }
      // a panel with fewer ranges than the lists have room for: its last range also marks the unused lists empty
      if (split == my_splits - 1) {
        for (int s = my_splits * KS; s < p.num_splits * KS; ++s) {
          const long long e = (long long)row * ((long long)p.num_splits * KS) + s;
          p.cand_val[e] = 0.0f;
          p.cand_idx[e] = -1;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    // let copies that may still be in flight land before shared memory and TMEM go away
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  // pair: neither CTA may free TMEM or leave while the other can still touch its barriers, shared memory or
  // accumulator rows
  if constexpr (PAIR) cluster_sync_all();
  if (warp == 2) {
    tc_fence_after();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, TMEM_COLS); else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- host side -------------------------------------------------------------------------------
template <bool WRITE_H, bool TOPK, int STAGES, int KS, bool PAIR>
static cudaError_t launch_variant(const CUtensorMap& ta, const CUtensorMap& tb, const EncGemmParams& p,
                                  cudaStream_t stream) {
  using L = SmemLayout<STAGES, KS, PAIR>;
  static_assert(L::kDynamicBytes <= 232448, "shared memory of one CTA exceeds 227 KB");
  auto kern = enc_gemm_kernel<WRITE_H, TOPK, STAGES, KS, PAIR>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.units != 0 ? p.units * (PAIR ? 2 : 1) : p.num_panels * p.num_splits);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = L::kDynamicBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = PAIR ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, ta, tb, p);
}

// mode: bit 0 = WRITE_H, bit 1 = TOPK, bit 2 = 3-stage ring for the plain single-CTA variant (a tuning probe),
// bit 3 = CTA-pair variant (needs an even number of panels; `tb` must then have a 128-row box),
// bit 4 = with bit 3 and TOPK: a 4-stage ring (under 200 KB of shared memory), which leaves room on the SM for
//         CTAs of a bandwidth-bound kernel running at the same time on another stream.
// Returns a CUDA error code (0 = launched).
int enc_gemm_launch(const CUtensorMap& ta, const CUtensorMap& tb, const EncGemmParams& p, int mode,
                    cudaStream_t stream) {
  const bool wh = mode & 1, tk = mode & 2, pair = mode & 8, compact = mode & 16;
  if (pair && (p.num_panels % 2 != 0)) return (int)cudaErrorInvalidValue;
  if (p.heads > 1 && (p.K % (p.heads * BK) != 0 || p.b_rows_per_head < p.N)) return (int)cudaErrorInvalidValue;
  if (p.units != 0) {  // ragged deal: every panel unit gets at least one range, none more ranges than there are tiles
    const int panel_units = pair ? p.num_panels / 2 : p.num_panels;
    const int base = p.units / panel_units, extra = p.units % panel_units;
    if (base < 1 || base + (extra > 0 ? 1 : 0) != p.num_splits || p.num_splits > (p.N + BN - 1) / BN)
      return (int)cudaErrorInvalidValue;
  }
  cudaError_t e;
  if (!tk) {
    if (pair) e = launch_variant<true, false, 6, 0, true>(ta, tb, p, stream);
    else e = (mode & 4) ? launch_variant<true, false, 3, 0, false>(ta, tb, p, stream)
                        : launch_variant<true, false, 4, 0, false>(ta, tb, p, stream);
  } else if (p.k <= 32) {
    if (pair && compact && !wh) e = launch_variant<false, true, 4, 32, true>(ta, tb, p, stream);
    else if (pair) e = wh ? launch_variant<true, true, 6, 32, true>(ta, tb, p, stream) : launch_variant<false, true, 6, 32, true>(ta, tb, p, stream);
    else e = wh ? launch_variant<true, true, 4, 32, false>(ta, tb, p, stream) : launch_variant<false, true, 4, 32, false>(ta, tb, p, stream);
  } else {
    if (pair && compact && !wh) e = launch_variant<false, true, 4, 64, true>(ta, tb, p, stream);
    else if (pair) e = wh ? launch_variant<true, true, 5, 64, true>(ta, tb, p, stream) : launch_variant<false, true, 5, 64, true>(ta, tb, p, stream);
    else e = wh ? launch_variant<true, true, 3, 64, false>(ta, tb, p, stream) : launch_variant<false, true, 3, 64, false>(ta, tb, p, stream);
  }
  return (int)e;
}

int enc_gemm_slots_for_k(int k) { return k <= 32 ? 32 : 64; }

}  // namespace lmsae
