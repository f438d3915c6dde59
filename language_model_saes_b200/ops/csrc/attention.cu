// Causal attention with separate query/key and value widths on sm_100a tensor cores (tcgen05 + TMEM + TMA).
//
// Low-rank sparse attention dictionaries (models/lorsa.py:642-661,714-725,864-904 of the reference project) run one
// attention per QK head whose value / output width is the head's OV group: q, k are [batch, seq, heads, d_qk] and
// v is [batch, seq, heads, d_v] with d_v != d_qk in general, which the flash kernels of the usual libraries do not take.
//
// Forward (attn_fwd_kernel): one CTA per (128-query block, head, value chunk of DV columns, batch element), 128 threads,
// thread r owns query row r (= TMEM lane r).
//   per 128-key block (causal: only blocks up to the diagonal):
//     TMA      K block [128 x DQK] and V^T block [DV x 128] (both K-major, 128-byte swizzle) -> shared memory
//     tcgen05  S = Q K^T            (128 x 128 x DQK, accumulator in TMEM columns [0, 128))
//     threads  read their S row from TMEM, online softmax in the exp2 domain, write P as bf16 into shared memory in the
//              swizzled K-major layout the tensor core reads
//     tcgen05  O_blk = P V          (128 x DV x 128, TMEM columns [128, 128 + DV))
//     threads  O = O * alpha + O_blk in registers
//   epilogue: O / l as bf16, log-sum-exp per row for the backward pass.
// V is consumed as V^T [batch, heads, d_v, seq] so that both operands of P V are K-major (keys contiguous).
// Every mbarrier wait is bounded; on expiry the CTA records a status code, stops issuing work and frees its TMEM.
#include "common.cuh"
#include "kernels.h"

namespace lmsae {

namespace {

constexpr int ATT_BM = 128;  // queries per CTA
constexpr int ATT_BN = 128;  // keys per block
constexpr int ATT_THREADS = 128;
constexpr int ATOM_BYTES_128 = 128 * 128;  // 128 rows x 64 bf16

template <int DQK, int DV>
struct AttnSmem {
  static constexpr int kQOff = 0;
  static constexpr int kQBytes = (DQK / 64) * ATOM_BYTES_128;
  static constexpr int kKOff = kQOff + kQBytes;
  static constexpr int kVOff = kKOff + kQBytes;
  static constexpr int kVAtomBytes = DV * 128;  // DV rows x 64 keys
  static constexpr int kVBytes = 2 * kVAtomBytes;
  static constexpr int kPOff = kVOff + kVBytes;
  static constexpr int kPBytes = 2 * ATOM_BYTES_128;
  static constexpr int kBarOff = kPOff + kPBytes;
  static constexpr int kTmemPtrOff = kBarOff + 4 * 8;
  static constexpr int kAbortOff = kTmemPtrOff + 4;
  static constexpr int kTotal = kAbortOff + 4;
  static constexpr int kDynamicBytes = kTotal + 1024;
};

// byte offset of the 16-byte chunk `chunk` (0..7) of row `row` inside a 128-byte-swizzled K-major atom
__device__ __forceinline__ uint32_t sw128_chunk_off(int row, int chunk) {
  return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4));
}

}  // namespace

template <int DQK, int DV>
__global__ void __launch_bounds__(ATT_THREADS)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_vt, const AttnParams p) {
  using L = AttnSmem<DQK, DV>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bar_q = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* bar_kv = bar_q + 1;
  uint64_t* bar_s = bar_q + 2;
  uint64_t* bar_o = bar_q + 3;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem + L::kTmemPtrOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qblocks = (p.seq + ATT_BM - 1) / ATT_BM;
  const int qblk = n_qblocks - 1 - (int)blockIdx.x;  // longest rows first
  const int dv_chunks = p.dv / DV;
  const int head = (int)blockIdx.y / dv_chunks;
  const int dv0 = ((int)blockIdx.y - head * dv_chunks) * DV;
  const int batch = (int)blockIdx.z;
  const int q0 = qblk * ATT_BM;
  const int row = (int)threadIdx.x;
  const int qpos = q0 + row;
  const bool row_ok = qpos < p.seq;

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_kv, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmap_q);
    prefetch_tensormap(&tmap_k);
    prefetch_tensormap(&tmap_vt);
  }
  if (warp == 0) {
    tmem_alloc(tmem_ptr_smem, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const uint32_t tmem_s = tmem_base;
  const uint32_t tmem_o = tmem_base + ATT_BN;
  const uint32_t lane_off = (uint32_t)(warp * 32) << 16;

  if (threadIdx.x == 0) {
    mbar_arrive_expect_tx(bar_q, L::kQBytes);
#pragma unroll
    for (int a = 0; a < DQK / 64; ++a)
      tma_load_2d(smem + L::kQOff + a * ATOM_BYTES_128, &tmap_q, bar_q, head * DQK + a * 64, batch * p.seq + q0);
  }

  float o_acc[DV];
#pragma unroll
  for (int i = 0; i < DV; ++i) o_acc[i] = 0.0f;
  float m_run = -INFINITY, l_run = 0.0f;
  const float sc = p.scale_log2;

  const int n_kblocks = qblk + 1;  // causal: key blocks 0 .. diagonal
  bool ok = true;
  for (int kb = 0; kb < n_kblocks && ok; ++kb) {
    const int k0 = kb * ATT_BN;
    const uint32_t parity = kb & 1;
    if (threadIdx.x == 0) {
      mbar_arrive_expect_tx(bar_kv, L::kQBytes + L::kVBytes);
#pragma unroll
      for (int a = 0; a < DQK / 64; ++a)
        tma_load_2d(smem + L::kKOff + a * ATOM_BYTES_128, &tmap_k, bar_kv, head * DQK + a * 64, batch * p.seq + k0);
#pragma unroll
      for (int a = 0; a < 2; ++a)
        tma_load_2d(smem + L::kVOff + a * L::kVAtomBytes, &tmap_vt, bar_kv, k0 + a * 64,
                    (batch * p.heads + head) * p.dv + dv0);
      bool got = true;
      if (kb == 0) got = mbar_wait_bounded(bar_q, 0, abort_flag);
      got = got && mbar_wait_bounded(bar_kv, parity, abort_flag);
      if (!got) {
        report_status(p.status, kTimeoutFullBarrier, kb);
        *abort_flag = 1;
      } else {
        tc_fence_after();
        constexpr uint32_t idesc_s = make_idesc_bf16(ATT_BM, ATT_BN);
#pragma unroll
        for (int kk = 0; kk < DQK / 16; ++kk) {
          const uint32_t qa = smem_u32(smem + L::kQOff + (kk / 4) * ATOM_BYTES_128);
          const uint32_t ka = smem_u32(smem + L::kKOff + (kk / 4) * ATOM_BYTES_128);
          umma_bf16_ss(tmem_s, make_sw128_kmajor_desc(qa) + (uint64_t)((kk % 4) * 2),
                       make_sw128_kmajor_desc(ka) + (uint64_t)((kk % 4) * 2), idesc_s, kk > 0 ? 1u : 0u);
        }
      }
      umma_commit(bar_s);  // also after an abort, so that the waiters below leave promptly
    }
    if (!mbar_wait_bounded(bar_s, parity, abort_flag) || *abort_flag != 0) {
      if (*abort_flag == 0) report_status(p.status, kTimeoutTmemFull, kb);
      *abort_flag = 1;
      ok = false;
    }
    // (every thread takes the same branches from here on: abort_flag is re-read after a CTA-wide barrier)
    __syncthreads();
    ok = (*abort_flag == 0);
    if (!ok) break;
    tc_fence_after();

    // ---- pass 1: row maximum of the scaled, masked scores
    float m_blk = -INFINITY;
#pragma unroll 1
    for (int c = 0; c < ATT_BN / 32; ++c) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(tmem_s + lane_off + (uint32_t)(c * 32), r);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int kpos = k0 + c * 32 + j;
        const float s = (kpos <= qpos && kpos < p.seq) ? __uint_as_float(r[j]) * sc : -INFINITY;
        m_blk = fmaxf(m_blk, s);
      }
    }
    const float m_new = fmaxf(m_run, m_blk);
    const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;  // a fully masked row keeps exp2(-inf) = 0 everywhere
    const float alpha = exp2f(m_run - m_use);                 // m_run = -inf on the first block: alpha = 0
    float l_blk = 0.0f;
    // ---- pass 2: probabilities -> bf16 in shared memory (swizzled K-major, two 64-key atoms)
#pragma unroll 1
    for (int c = 0; c < ATT_BN / 32; ++c) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(tmem_s + lane_off + (uint32_t)(c * 32), r);
      tmem_wait_ld();
      float pv[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int kpos = k0 + c * 32 + j;
        const float s = (kpos <= qpos && kpos < p.seq) ? __uint_as_float(r[j]) * sc : -INFINITY;
        pv[j] = exp2f(s - m_use);
      }
      uint8_t* atom = smem + L::kPOff + (c / 2) * ATOM_BYTES_128;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 u;
        u.x = pack_bf16x2(pv[g * 8 + 0], pv[g * 8 + 1]);
        u.y = pack_bf16x2(pv[g * 8 + 2], pv[g * 8 + 3]);
        u.z = pack_bf16x2(pv[g * 8 + 4], pv[g * 8 + 5]);
        u.w = pack_bf16x2(pv[g * 8 + 6], pv[g * 8 + 7]);
        // the sum uses the rounded values, so that O / l is an exact convex combination of the V rows seen by the MMA
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float2 f = __bfloat1622float2(h[t]);
          l_blk += f.x + f.y;
        }
        *reinterpret_cast<uint4*>(atom + sw128_chunk_off(row, (c % 2) * 4 + g)) = u;
      }
    }
    l_run = l_run * alpha + l_blk;
    m_run = m_new;
#pragma unroll
    for (int i = 0; i < DV; ++i) o_acc[i] *= alpha;

    fence_proxy_async();  // the generic-proxy stores of P must be visible to the tensor core's reads
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) {
      tc_fence_after();
      constexpr uint32_t idesc_o = make_idesc_bf16(ATT_BM, DV);
#pragma unroll
      for (int kk = 0; kk < ATT_BN / 16; ++kk) {
        const uint32_t pa = smem_u32(smem + L::kPOff + (kk / 4) * ATOM_BYTES_128);
        const uint32_t va = smem_u32(smem + L::kVOff + (kk / 4) * L::kVAtomBytes);
        umma_bf16_ss(tmem_o, make_sw128_kmajor_desc(pa) + (uint64_t)((kk % 4) * 2),
                     make_sw128_kmajor_desc(va) + (uint64_t)((kk % 4) * 2), idesc_o, kk > 0 ? 1u : 0u);
      }
      umma_commit(bar_o);
    }
    if (!mbar_wait_bounded(bar_o, parity, abort_flag)) {
      report_status(p.status, kTimeoutTmemFull, 1000 + kb);
      *abort_flag = 1;
    }
    __syncthreads();
    ok = (*abort_flag == 0);
    if (!ok) break;
    tc_fence_after();
#pragma unroll
    for (int c = 0; c < DV / 32; ++c) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(tmem_o + lane_off + (uint32_t)(c * 32), r);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j) o_acc[c * 32 + j] += __uint_as_float(r[j]);
    }
    // the next block's TMA and MMAs overwrite K, V, P and both accumulators: everyone must be done reading
    tc_fence_before();
    __syncthreads();
  }

  if (ok && row_ok) {
    const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
    __nv_bfloat16* dst = p.out + (((size_t)batch * p.seq + qpos) * p.heads + head) * p.dv + dv0;
#pragma unroll
    for (int i = 0; i < DV; i += 8) {
      uint4 u;
      u.x = pack_bf16x2(o_acc[i] * inv, o_acc[i + 1] * inv);
      u.y = pack_bf16x2(o_acc[i + 2] * inv, o_acc[i + 3] * inv);
      u.z = pack_bf16x2(o_acc[i + 4] * inv, o_acc[i + 5] * inv);
      u.w = pack_bf16x2(o_acc[i + 6] * inv, o_acc[i + 7] * inv);
      *reinterpret_cast<uint4*>(dst + i) = u;
    }
    if (p.lse != nullptr && dv0 == 0)
      p.lse[((size_t)batch * p.heads + head) * p.seq + qpos] = m_run * 0.6931471805599453f + __logf(l_run);
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);  // copies that may still be in flight land first
    __syncthreads();
  }
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

template <int DQK, int DV>
static cudaError_t attn_fwd_variant(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tvt,
                                    const AttnParams& p, cudaStream_t stream) {
  using L = AttnSmem<DQK, DV>;
  auto kern = attn_fwd_kernel<DQK, DV>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
  if (e != cudaSuccess) return e;
  dim3 grid((p.seq + ATT_BM - 1) / ATT_BM, p.heads * (p.dv / DV), p.batch);
  kern<<<grid, ATT_THREADS, L::kDynamicBytes, stream>>>(tq, tk, tvt, p);
  return cudaGetLastError();
}

int attn_value_chunk(int dv) { return dv % 128 == 0 ? 128 : (dv % 64 == 0 ? 64 : 0); }

int attn_fwd_launch(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tvt, const AttnParams& p,
                    cudaStream_t stream) {
  const int dvc = attn_value_chunk(p.dv);
  if (dvc == 0 || (p.dqk != 64 && p.dqk != 128) || p.seq % 8 != 0 || p.batch > 65535 || p.heads * (p.dv / dvc) > 65535)
    return (int)cudaErrorInvalidValue;
  cudaError_t e;
  if (p.dqk == 64) e = dvc == 128 ? attn_fwd_variant<64, 128>(tq, tk, tvt, p, stream) : attn_fwd_variant<64, 64>(tq, tk, tvt, p, stream);
  else e = dvc == 128 ? attn_fwd_variant<128, 128>(tq, tk, tvt, p, stream) : attn_fwd_variant<128, 64>(tq, tk, tvt, p, stream);
  return (int)e;
}

}  // namespace lmsae
