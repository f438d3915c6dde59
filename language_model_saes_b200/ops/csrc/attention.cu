// Causal attention with separate query/key and value widths on sm_100a tensor cores (tcgen05 + TMEM + TMA).
//
// Low-rank sparse attention dictionaries (models/lorsa.py:642-661,714-725,864-904 of the reference project) run one
// attention per QK head whose value / output width is the head's OV group: q, k are [batch, seq, heads, d_qk] and
// v is [batch, seq, heads, d_v] with d_v != d_qk in general, which the flash kernels of the usual libraries do not take.
//
// Forward (attn_fwd_kernel): one CTA per (128-query block, head, value chunk of DV columns, batch element); four warps
// whose thread r owns query row r (= TMEM lane r) and a fifth warp that issues the TMA loads and the MMAs.
//   per 128-key block (causal: only blocks up to the diagonal):
//     TMA      K block [128 x DQK] and V^T block [DV x 128] (both K-major, 128-byte swizzle) -> shared memory
//     tcgen05  S = Q K^T            (128 x 128 x DQK, accumulator in TMEM columns [0, 128))
//     threads  read their S row from TMEM, online softmax in the exp2 domain, write P as bf16 into shared memory in the
//              swizzled K-major layout the tensor core reads
//     tcgen05  O += P V             (128 x DV x 128, TMEM columns [128, 128 + DV))
//              (accumulating in TMEM; the rows rescale it in place only when their maximum has grown a lot)
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
  static constexpr int kKOff = kQOff + kQBytes;        // two K buffers
  static constexpr int kVOff = kKOff + 2 * kQBytes;    // two V^T buffers
  static constexpr int kVAtomBytes = DV * 128;         // DV rows x 64 keys
  static constexpr int kVBytes = 2 * kVAtomBytes;
  static constexpr int kPOff = kVOff + 2 * kVBytes;    // two P buffers
  static constexpr int kPBytes = 2 * ATOM_BYTES_128;
  static constexpr int kXchOff = kPOff + 2 * kPBytes;  // float [2][4][128]: row statistics exchanged between column quarters
  static constexpr int kBarOff = kXchOff + 2 * 4 * 128 * 4;
  static constexpr int kNumBars = 15;
  static constexpr int kTmemPtrOff = kBarOff + kNumBars * 8;
  static constexpr int kAbortOff = kTmemPtrOff + 4;
  static constexpr int kTotal = kAbortOff + 4;
  static constexpr int kDynamicBytes = kTotal + 1024;
};

// Two-element fp32 arithmetic (one instruction for a pair): d = a * b + c and d = a + b on (lo, hi) pairs.
__device__ __forceinline__ void fma_f32x2(float& d0, float& d1, float a0, float a1, float b, float c) {
  asm("{\n\t"
      ".reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rb, {%4, %4};\n\t"
      "mov.b64 rc, {%5, %5};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t"
      "}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
// max of three in one instruction
__device__ __forceinline__ float max3_f32(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ void add_f32x2(float& d0, float& d1, float a0, float a1) {
  asm("{\n\t"
      ".reg .b64 ra, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rd, {%0, %1};\n\t"
      "add.rn.f32x2 rd, rd, ra;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t"
      "}"
      : "+f"(d0), "+f"(d1)
      : "f"(a0), "f"(a1));
}

// byte offset of the 16-byte chunk `chunk` (0..7) of row `row` inside a 128-byte-swizzled K-major atom
__device__ __forceinline__ uint32_t sw128_chunk_off(int row, int chunk) {
  return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4));
}

}  // namespace

constexpr int FWD_ROW_WARPS = 16;      // warp w works on query rows 32 (w % 4) .. + 31 and key columns 32 (w / 4) .. + 31
constexpr int FWD_ROW_THREADS = FWD_ROW_WARPS * 32;
constexpr int FWD_THREADS = FWD_ROW_THREADS + 32;  // + the last warp: TMA + MMA issue
constexpr float kRescaleSlack = 8.0f;  // log2 units the running reference may lag behind the true row maximum

// Persistent: one CTA per SM walks a list of tiles (query block, head, value chunk, batch element), longest first, so
// that the loads and first MMAs of the next tile run while the softmax warps finish and store the current one.
// K, V^T, P (shared memory) and S (TMEM) are double-buffered over the sequence of key blocks of ALL tiles of the CTA:
// the g-th key block uses buffer g & 1 and completes phase g >> 1 of that buffer's barriers. The output accumulator is
// double-buffered over tiles (tile t uses buffer t & 1). Roles and hand-offs (mbarriers and 64-thread named barriers; no
// CTA-wide barrier inside the loops):
//   issuer   loads two key blocks ahead inside a tile; S(g+1) is computed while the rows work on S(g); P V (g) as soon
//            as P(g) is written; a K / V^T buffer is refilled when S / P V of its previous block has consumed it.
//   rows     four threads per query row, one per quarter of the 128 keys of a block (sixteen warps: the softmax work is
//            latency-bound, so the warps are there to hide each other's TMEM loads and barrier polls): S(g) TMEM -> 32
//            registers, release the S buffer; the four exchange their maxima through shared memory; the output accumulator stays in TMEM
//            and is only rescaled when the maximum has grown by more than 2^8 since the reference was set (rarely
//            after the first blocks), which keeps p <= 256 and the sums well inside fp32 / bf16 range; exponentials ->
//            P (bf16, swizzled K-major, two 64-key atoms) -> signal. After a tile's last block: O / l
//            to global memory, release the accumulator buffer.
template <int DQK, int DV>
__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_vt, const AttnParams p) {
  using L = AttnSmem<DQK, DV>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* bar_q = bars + 0;
  uint64_t* bar_k = bars + 1;        // [2]
  uint64_t* bar_v = bars + 3;        // [2]
  uint64_t* bar_s_full = bars + 5;   // [2]
  uint64_t* bar_s_free = bars + 7;   // [2]
  uint64_t* bar_p_full = bars + 9;   // [2]
  uint64_t* bar_pv_done = bars + 11; // [2]
  uint64_t* bar_o_free = bars + 13;  // [2]
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem + L::kTmemPtrOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);

  const int warp = threadIdx.x >> 5;
  const int n_qblocks = (p.seq + ATT_BM - 1) / ATT_BM;
  const int dv_chunks = p.dv / DV;
  const int per_qblock = p.heads * dv_chunks * p.batch;  // tiles that share a query block index (same length)
  const int n_tiles = n_qblocks * per_qblock;

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_k[i], 1);
      mbar_init(&bar_v[i], 1);
      mbar_init(&bar_s_full[i], 1);
      // (one arrival per softmax warp: hundreds of arrivals on one shared-memory word per key block would serialise)
      mbar_init(&bar_s_free[i], FWD_ROW_WARPS);
      mbar_init(&bar_p_full[i], FWD_ROW_WARPS);
      mbar_init(&bar_pv_done[i], 1);
      mbar_init(&bar_o_free[i], FWD_ROW_WARPS);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == FWD_ROW_WARPS) {
    tmem_alloc(tmem_ptr_smem, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;  // S buffers at columns [0, 128) and [128, 256), O buffers at 256 and 384

  // tile w of the global list (longest query blocks first): query block, then (batch, head, value chunk)
  auto decode_tile = [&](int w, int& qblk, int& head, int& dv0, int& batch) {
    qblk = n_qblocks - 1 - w / per_qblock;
    int r = w % per_qblock;
    batch = r / (p.heads * dv_chunks);
    r -= batch * (p.heads * dv_chunks);
    head = r / dv_chunks;
    dv0 = (r - head * dv_chunks) * DV;
  };

  if (warp == FWD_ROW_WARPS) {
    // ------------------------------------------------------------------ TMA + MMA issuer
    if (elect_one()) {
      bool ok = true;
      int where = 0;
      uint32_t g0 = 0;  // key blocks issued by this CTA before the current tile
      int t = 0;
      for (int w = (int)blockIdx.x; w < n_tiles && ok; w += (int)gridDim.x, ++t) {
        int qblk, head, dv0, batch;
        decode_tile(w, qblk, head, dv0, batch);
        const int q0 = qblk * ATT_BM;
        const int n_kblocks = qblk + 1;  // causal: key blocks 0 .. diagonal
        const uint32_t tmem_o = tmem_base + 2 * ATT_BN + (uint32_t)((t & 1) * DV);
        auto load_k = [&](int kb) {
          const int u = (g0 + kb) & 1;
          mbar_arrive_expect_tx(&bar_k[u], L::kQBytes);
          for (int a = 0; a < DQK / 64; ++a)
            tma_load_2d(smem + L::kKOff + u * L::kQBytes + a * ATOM_BYTES_128, &tmap_k, &bar_k[u], head * DQK + a * 64,
                        batch * p.seq + kb * ATT_BN);
        };
        auto load_v = [&](int kb) -> bool {
          const uint32_t g = g0 + kb;
          const int u = g & 1;
          // the buffer's previous block is g - 2: its P V must have read it
          if (g >= 2 && !mbar_wait_bounded(&bar_pv_done[u], ((g - 2) >> 1) & 1, abort_flag)) return false;
          mbar_arrive_expect_tx(&bar_v[u], L::kVBytes);
          for (int a = 0; a < 2; ++a)
            tma_load_2d(smem + L::kVOff + u * L::kVBytes + a * L::kVAtomBytes, &tmap_vt, &bar_v[u], kb * ATT_BN + a * 64,
                        (batch * p.heads + head) * p.dv + dv0);
          return true;
        };
        auto issue_s = [&](int kb) {
          const int u = (g0 + kb) & 1;
          constexpr uint32_t idesc_s = make_idesc_bf16(ATT_BM, ATT_BN);
#pragma unroll
          for (int kk = 0; kk < DQK / 16; ++kk) {
            const uint32_t qa = smem_u32(smem + L::kQOff + (kk / 4) * ATOM_BYTES_128);
            const uint32_t ka = smem_u32(smem + L::kKOff + u * L::kQBytes + (kk / 4) * ATOM_BYTES_128);
            umma_bf16_ss(tmem_base + (uint32_t)(u * ATT_BN), make_sw128_kmajor_desc(qa) + (uint64_t)((kk % 4) * 2),
                         make_sw128_kmajor_desc(ka) + (uint64_t)((kk % 4) * 2), idesc_s, kk > 0 ? 1u : 0u);
          }
          umma_commit(&bar_s_full[u]);
        };
        // The previous tile's S MMAs have all completed (their barriers were waited for below), so Q and the K buffers
        // are free; V buffers are checked in load_v.
        where = 1;
        mbar_arrive_expect_tx(bar_q, L::kQBytes);
        for (int a = 0; a < DQK / 64; ++a)
          tma_load_2d(smem + L::kQOff + a * ATOM_BYTES_128, &tmap_q, bar_q, head * DQK + a * 64, batch * p.seq + q0);
        load_k(0);
        if (n_kblocks > 1) load_k(1);
        ok = load_v(0);
        // S(0): Q and K(0) landed; the S buffer's previous block (g0 - 2) was read by the rows
        ok = ok && mbar_wait_bounded(bar_q, t & 1, abort_flag) && mbar_wait_bounded(&bar_k[g0 & 1], (g0 >> 1) & 1, abort_flag);
        if (ok && g0 >= 2) ok = mbar_wait_bounded(&bar_s_free[g0 & 1], ((g0 - 2) >> 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        issue_s(0);
        // V(1) goes into the buffer that the previous tile's LAST block used: this wait is the one place where the
        // issuer depends on the rows having finished that tile's last softmax, so it comes after S(0) is under way
        where = 2;
        if (n_kblocks > 1) ok = load_v(1);
        // the accumulator buffer of this tile was last used by tile t - 2: its rows must have stored their outputs
        if (ok && t >= 2) ok = mbar_wait_bounded(&bar_o_free[t & 1], ((t - 2) >> 1) & 1, abort_flag);
        for (int kb = 0; kb < n_kblocks && ok; ++kb) {
          const uint32_t g = g0 + kb;
          const int u = g & 1;
          const uint32_t ph = (g >> 1) & 1;  // phase of this block's use of buffer u
          const bool more = kb + 1 < n_kblocks;
          if (more) {
            // S(kb+1): its K block has landed and the rows have released the S buffer it overwrites (block g - 1)
            where = 10 * kb + 3;
            ok = mbar_wait_bounded(&bar_k[u ^ 1], ((g + 1) >> 1) & 1, abort_flag);
            if (ok && g >= 1) ok = mbar_wait_bounded(&bar_s_free[u ^ 1], ((g - 1) >> 1) & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            issue_s(kb + 1);
          }
          // K buffer u is free once S(kb) has been computed: fetch block kb + 2 into it
          where = 10 * kb + 4;
          ok = mbar_wait_bounded(&bar_s_full[u], ph, abort_flag);
          if (!ok) break;
          if (kb + 2 < n_kblocks) load_k(kb + 2);
          // P V (kb)
          where = 10 * kb + 5;
          ok = mbar_wait_bounded(&bar_p_full[u], ph, abort_flag) && mbar_wait_bounded(&bar_v[u], ph, abort_flag);
          if (!ok) break;
          tc_fence_after();
          constexpr uint32_t idesc_o = make_idesc_bf16(ATT_BM, DV);
#pragma unroll
          for (int kk = 0; kk < ATT_BN / 16; ++kk) {
            const uint32_t pa = smem_u32(smem + L::kPOff + u * L::kPBytes + (kk / 4) * ATOM_BYTES_128);
            const uint32_t va = smem_u32(smem + L::kVOff + u * L::kVBytes + (kk / 4) * L::kVAtomBytes);
            umma_bf16_ss(tmem_o, make_sw128_kmajor_desc(pa) + (uint64_t)((kk % 4) * 2),
                         make_sw128_kmajor_desc(va) + (uint64_t)((kk % 4) * 2), idesc_o, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&bar_pv_done[u]);
          // the V buffer of the previous block is free once its P V has completed (it ran before this one): refill it
          if (kb >= 1 && more) {
            where = 10 * kb + 6;
            ok = load_v(kb + 1);
          }
        }
        g0 += (uint32_t)n_kblocks;
      }
      if (!ok) {
        report_status(p.status, kTimeoutFullBarrier, where);
        *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax rows
    const int quarter = warp & 3, cq = warp >> 2, lane = (int)threadIdx.x & 31;
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t s_col = (uint32_t)(cq * 32);
    // output columns of this thread (rescale and final store): a quarter of DV, at least one 32-column TMEM load
    constexpr int O_W = DV / 4 >= 32 ? DV / 4 : 32;
    const bool o_active = cq * O_W < DV;
    const uint32_t o_col = (uint32_t)(cq * O_W);
    float* xch = reinterpret_cast<float*>(smem + L::kXchOff);  // [2 parities][4 column quarters][128 rows]
    const float sc = p.scale_log2;
    bool ok = true;
    uint32_t g0 = 0;
    int t = 0;
    for (int w = (int)blockIdx.x; w < n_tiles && ok; w += (int)gridDim.x, ++t) {
      int qblk, head, dv0, batch;
      decode_tile(w, qblk, head, dv0, batch);
      const int q0 = qblk * ATT_BM;
      const int n_kblocks = qblk + 1;
      const int qpos = q0 + row;
      const bool row_ok = qpos < p.seq;
      const uint32_t tmem_o = tmem_base + 2 * ATT_BN + (uint32_t)((t & 1) * DV);
      float m_ref = -INFINITY, l_run = 0.0f;
      for (int kb = 0; kb < n_kblocks && ok; ++kb) {
        const uint32_t g = g0 + kb;
        const int u = g & 1;
        const uint32_t ph = (g >> 1) & 1;
        const int k0 = kb * ATT_BN + (int)s_col;
        // (a failed wait ends the loops for the whole warp: the TMEM accesses and votes below are warp-wide)
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&bar_s_full[u], ph, abort_flag))) { ok = false; break; }
        tc_fence_after();
        uint32_t s[32];
        tmem_ld_32x32b_x32(tmem_base + (uint32_t)(u * ATT_BN) + lane_off + s_col, s);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_s_free[u]);
        // masked raw scores and their maximum (only the diagonal and the last block have anything to mask)
        // (warp-uniform branch: the common, unmasked case costs one maximum per element and nothing else)
        const int last_ok = min(qpos, p.seq - 1) - k0;  // columns 0 .. last_ok of this thread's 32 are visible
        float m_raw = -INFINITY;
        if (__any_sync(0xffffffffu, last_ok < 31)) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (j > last_ok) s[j] = 0xff800000u;  // -inf
            m_raw = fmaxf(m_raw, __uint_as_float(s[j]));
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; j += 2) m_raw = max3_f32(m_raw, __uint_as_float(s[j]), __uint_as_float(s[j + 1]));
        }
        // the other three quarters of the row: exchange through shared memory, 128-thread barrier of the four warps
        // that share these 32 rows
        float* xr = xch + (u * 4) * ATT_BM + row;
        xr[cq * ATT_BM] = m_raw;
        asm volatile("bar.sync %0, 128;" ::"r"(1 + quarter) : "memory");
        const float m_blk = fmaxf(fmaxf(xr[0], xr[ATT_BM]), fmaxf(xr[2 * ATT_BM], xr[3 * ATT_BM])) * sc;  // sc > 0
        float alpha = 1.0f;
        bool rescale = false;
        if (m_blk > m_ref + kRescaleSlack || m_ref == -INFINITY) {
          const float m_new = fmaxf(m_ref, m_blk);
          if (m_new != -INFINITY) {
            alpha = exp2f(m_ref - m_new);  // 0 when nothing was accumulated under the old reference
            rescale = kb > 0;
            m_ref = m_new;
          }
        }
        const float m_use = (m_ref == -INFINITY) ? 0.0f : m_ref;
        if (__any_sync(0xffffffffu, rescale)) {  // this warp's share of the output columns
          // the accumulator belongs to the tensor core until P V (g - 1) has completed
          if (!__all_sync(0xffffffffu, mbar_wait_bounded(&bar_pv_done[u ^ 1], ((g - 1) >> 1) & 1, abort_flag))) { ok = false; break; }
          tc_fence_after();
          if (o_active) {
#pragma unroll 1
            for (int c = 0; c < O_W / 32; ++c) {
              uint32_t r[32];
              tmem_ld_32x32b_x32(tmem_o + lane_off + o_col + (uint32_t)(c * 32), r);
              tmem_wait_ld();
#pragma unroll
              for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * alpha);
              tmem_st_32x32b_x32(tmem_o + lane_off + o_col + (uint32_t)(c * 32), r);
            }
            tmem_wait_st();
          }
        }
        if (g >= 2) {
          // P buffer u was read by P V (g - 2)
          if (!__all_sync(0xffffffffu, mbar_wait_bounded(&bar_pv_done[u], ((g - 2) >> 1) & 1, abort_flag))) { ok = false; break; }
        }
        l_run *= alpha;
        float l_blk = 0.0f, l_blk1 = 0.0f;
        // this quarter's 32 keys are half of a 64-key swizzle atom: 16-byte chunks (cq % 2) * 4 .. + 3 of atom cq / 2
        uint8_t* atom = smem + L::kPOff + u * L::kPBytes + (cq >> 1) * ATOM_BYTES_128;
        const float neg_m = -m_use;
#pragma unroll
        for (int gq = 0; gq < 4; ++gq) {
          float pv[8];
#pragma unroll
          for (int i = 0; i < 8; i += 2) {
            // exponent arguments and the running sums two elements per instruction; the exponentials one by one
            float a0, a1;
            fma_f32x2(a0, a1, __uint_as_float(s[gq * 8 + i]), __uint_as_float(s[gq * 8 + i + 1]), sc, neg_m);
            pv[i] = exp2f(a0);
            pv[i + 1] = exp2f(a1);
            add_f32x2(l_blk, l_blk1, pv[i], pv[i + 1]);
          }
          uint4 wv;
          wv.x = pack_bf16x2(pv[0], pv[1]);
          wv.y = pack_bf16x2(pv[2], pv[3]);
          wv.z = pack_bf16x2(pv[4], pv[5]);
          wv.w = pack_bf16x2(pv[6], pv[7]);
          *reinterpret_cast<uint4*>(atom + sw128_chunk_off(row, (cq & 1) * 4 + gq)) = wv;
        }
        l_run += l_blk + l_blk1;
        fence_proxy_async();  // the generic-proxy stores of P must be visible to the tensor core's reads
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_p_full[u]);
      }
      // ---- the tile's epilogue
      const uint32_t g_last = g0 + (uint32_t)n_kblocks - 1;
      ok = __all_sync(0xffffffffu, ok && mbar_wait_bounded(&bar_pv_done[g_last & 1], (g_last >> 1) & 1, abort_flag));
      if (!ok) break;
      tc_fence_after();
      // total of the four partial sums; slot parity continues the per-block sequence (block g_last used g_last & 1)
      float* xl = xch + (int)((g_last + 1) & 1) * 4 * ATT_BM + row;
      xl[cq * ATT_BM] = l_run;
      asm volatile("bar.sync %0, 128;" ::"r"(1 + quarter) : "memory");
      const float l_tot = (xl[0] + xl[ATT_BM]) + (xl[2 * ATT_BM] + xl[3 * ATT_BM]);
      const float inv = l_tot > 0.0f ? 1.0f / l_tot : 0.0f;
      if (o_active) {
        __nv_bfloat16* dst = p.out + (((size_t)batch * p.seq + (row_ok ? qpos : 0)) * p.heads + head) * p.dv + dv0 + o_col;
#pragma unroll 1
        for (int c = 0; c < O_W / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_o + lane_off + o_col + (uint32_t)(c * 32), r);
          tmem_wait_ld();
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 wv;
              wv.x = pack_bf16x2(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
              wv.y = pack_bf16x2(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
              wv.z = pack_bf16x2(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
              wv.w = pack_bf16x2(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + c * 32 + i) = wv;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_o_free[t & 1]);
      if (row_ok && cq == 0 && p.lse != nullptr && dv0 == 0)
        p.lse[((size_t)batch * p.heads + head) * p.seq + qpos] = m_ref * 0.6931471805599453f + __logf(l_tot);
      // keep the four warps of a row quarter together across tiles: the sum exchange above and the next maximum exchange
      // use the same slots
      asm volatile("bar.sync %0, 128;" ::"r"(1 + quarter) : "memory");
      g0 += (uint32_t)n_kblocks;
    }
    if (!ok) {
      report_status(p.status, kTimeoutTmemFull, row);
      *abort_flag = 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);  // copies that may still be in flight land first
    __syncthreads();
  }
  if (warp == FWD_ROW_WARPS) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int DQK, int DV>
static cudaError_t attn_fwd_variant(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tvt,
                                    const AttnParams& p, cudaStream_t stream) {
  using L = AttnSmem<DQK, DV>;
  static_assert(L::kDynamicBytes <= 232448, "shared memory of one CTA exceeds 227 KB");
  auto kern = attn_fwd_kernel<DQK, DV>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
  if (e != cudaSuccess) return e;
  static int num_sms = 0;  // persistent grid: one CTA per SM
  if (num_sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      num_sms = 148;
  }
  const long long tiles = (long long)((p.seq + ATT_BM - 1) / ATT_BM) * p.heads * (p.dv / DV) * p.batch;
  if (tiles <= 0 || tiles > 2147483647LL) return cudaErrorInvalidValue;
  const int grid = (int)(tiles < num_sms ? tiles : num_sms);
  kern<<<grid, FWD_THREADS, L::kDynamicBytes, stream>>>(tq, tk, tvt, p);
  return cudaGetLastError();
}

int attn_value_chunk(int dv) { return dv % 128 == 0 ? 128 : (dv % 64 == 0 ? 64 : 0); }

// =============================================================================================================
// Backward. With P = softmax(scale * Q K^T) (causal), O = P V, D = rowsum(dO * O):
//   dV = P^T dO,   dP = dO V^T,   dS = P * (dP - D) * scale,   dQ = dS K,   dK = dS^T Q.
// Two kernels, both built from the same pieces as the forward pass and with every MMA operand K-major (the host
// passes transposed copies K^T, Q^T, dO^T [batch, heads, width, seq] where a product contracts over positions):
//   attn_bwd_dq_kernel   one CTA per query block; per key block: S and dP on the tensor cores (dP contracts over
//                        the FULL value width, streamed through a two-stage ring of 64-column atoms), the threads
//                        (one query row each) form dS, and dQ += dS K accumulates in TMEM over the key blocks.
//   attn_bwd_dkv_kernel  one CTA per key block (and value chunk); per query block: S^T = K Q^T and dP^T = V dO^T, the
//                        threads (one key row each) form P^T and dS^T, and dV += P^T dO, dK += dS^T Q accumulate in
//                        TMEM over the query blocks.
// =============================================================================================================
namespace {

// D[tmem] (+)= A * B^T over K = 16 * steps, both tiles made of 64-column swizzle atoms `a_atom` / `b_atom` bytes apart.
__device__ __forceinline__ void issue_mma_atoms(uint32_t tmem_d, uint32_t a_base, uint32_t a_atom, uint32_t b_base,
                                                uint32_t b_atom, int steps, uint32_t idesc, bool accumulate) {
  for (int kk = 0; kk < steps; ++kk) {
    const uint64_t da = make_sw128_kmajor_desc(a_base + (uint32_t)(kk / 4) * a_atom) + (uint64_t)((kk % 4) * 2);
    const uint64_t db = make_sw128_kmajor_desc(b_base + (uint32_t)(kk / 4) * b_atom) + (uint64_t)((kk % 4) * 2);
    umma_bf16_ss(tmem_d, da, db, idesc, (accumulate || kk > 0) ? 1u : 0u);
  }
}

template <int DQK>
struct BwdDqSmem {
  // with 64-wide queries there is room for two K / K^T buffers: the next key block's tiles (and the first dO / V atom)
  // are fetched while the threads work on the current one
  static constexpr bool kDouble = DQK == 64;
  static constexpr int kKBufs = kDouble ? 2 : 1;
  static constexpr int kQBytes = (DQK / 64) * ATOM_BYTES_128;
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQOff + kQBytes;
  static constexpr int kKtAtomBytes = DQK * 128;
  static constexpr int kKtOff = kKOff + kKBufs * kQBytes;
  static constexpr int kDsOff = kKtOff + kKBufs * 2 * kKtAtomBytes;
  static constexpr int kRingOff = kDsOff + 2 * ATOM_BYTES_128;  // 2 stages x {dO atom, V atom}
  static constexpr int kBarOff = kRingOff + 4 * ATOM_BYTES_128;
  static constexpr int kNumBars = 9;
  static constexpr int kTmemPtrOff = kBarOff + kNumBars * 8;
  static constexpr int kAbortOff = kTmemPtrOff + 4;
  static constexpr int kDynamicBytes = kAbortOff + 4 + 1024;
};

template <int DQK, int DVC>
struct BwdDkvSmem {
  // with 64-wide queries there is room for two Q buffers: the next query block's Q tile (and the first V / dO atom) are
  // fetched while the threads work on the current one
  static constexpr bool kDouble = DQK == 64;
  static constexpr int kQBufs = kDouble ? 2 : 1;
  static constexpr int kKBytes = (DQK / 64) * ATOM_BYTES_128;
  static constexpr int kKOff = 0;
  static constexpr int kQOff = kKOff + kKBytes;              // Q_i, later Q_i^T (same size), per buffer
  static constexpr int kQtAtomBytes = DQK * 128;
  static constexpr int kRingOff = kQOff + kQBufs * kKBytes;  // 2 stages x {V atom, dO atom}; later dO^T chunk
  static constexpr int kDotAtomBytes = DVC * 128;
  static constexpr int kPtOff = kRingOff + 4 * ATOM_BYTES_128;
  static constexpr int kDstOff = kPtOff + 2 * ATOM_BYTES_128;
  static constexpr int kLseOff = kDstOff + 2 * ATOM_BYTES_128;
  static constexpr int kDeltaOff = kLseOff + 128 * 4;
  static constexpr int kBarOff = kDeltaOff + 128 * 4;
  static constexpr int kNumBars = 10;
  static constexpr int kTmemPtrOff = kBarOff + kNumBars * 8;
  static constexpr int kAbortOff = kTmemPtrOff + 4;
  static constexpr int kDynamicBytes = kAbortOff + 4 + 1024;
};

}  // namespace

template <int DQK>
__global__ void __launch_bounds__(ATT_THREADS)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_kt, const __grid_constant__ CUtensorMap tmap_do,
                   const __grid_constant__ CUtensorMap tmap_v, const AttnBwdParams p) {
  using L = BwdDqSmem<DQK>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* bar_q = bars + 0;
  uint64_t* bar_k = bars + 1;      // [2]
  uint64_t* bar_mma1 = bars + 3;
  uint64_t* bar_mma2 = bars + 4;
  uint64_t* ring_full = bars + 5;  // [2]
  uint64_t* ring_free = bars + 7;  // [2]
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem + L::kTmemPtrOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);

  const int warp = threadIdx.x >> 5;
  const int n_qblocks = (p.seq + ATT_BM - 1) / ATT_BM;
  const int qblk = n_qblocks - 1 - (int)blockIdx.x;
  const int head = (int)blockIdx.y, batch = (int)blockIdx.z;
  const int q0 = qblk * ATT_BM;
  const int row = (int)threadIdx.x;
  const int qpos = q0 + row;
  const bool row_ok = qpos < p.seq;
  const int dv_atoms = p.dv / 64;

  if (threadIdx.x == 0) {
    for (int i = 0; i < L::kNumBars; ++i) mbar_init(&bars[i], 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_ptr_smem, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const uint32_t tmem_s = tmem_base, tmem_dp = tmem_base + 128, tmem_dq = tmem_base + 256;
  const uint32_t lane_off = (uint32_t)(warp * 32) << 16;

  const size_t stat = ((size_t)batch * p.heads + head) * p.seq + (row_ok ? qpos : 0);
  const float lse2 = row_ok ? p.lse[stat] * 1.4426950408889634f : INFINITY;  // +inf: every probability of the row is 0
  const float delta = row_ok ? p.delta[stat] : 0.0f;

  if (threadIdx.x == 0) {
    mbar_arrive_expect_tx(bar_q, L::kQBytes);
    for (int a = 0; a < DQK / 64; ++a)
      tma_load_2d(smem + L::kQOff + a * ATOM_BYTES_128, &tmap_q, bar_q, head * DQK + a * 64, batch * p.seq + q0);
  }

  const int n_kblocks = qblk + 1;
  uint32_t ring_n = 0;  // atom steps issued so far (thread 0 only)
  bool ok = true;
  for (int kb = 0; kb < n_kblocks && ok; ++kb) {
    const int k0 = kb * ATT_BN;
    const uint32_t parity = kb & 1;
    const int ub = L::kDouble ? (kb & 1) : 0;  // K / K^T buffer of this key block
    if (threadIdx.x == 0) {
      bool got = true;
      auto load_block = [&](int blk) {
        const int u = L::kDouble ? (blk & 1) : 0;
        mbar_arrive_expect_tx(&bar_k[u], L::kQBytes + 2 * L::kKtAtomBytes);
        for (int a = 0; a < DQK / 64; ++a)
          tma_load_2d(smem + L::kKOff + u * L::kQBytes + a * ATOM_BYTES_128, &tmap_k, &bar_k[u], head * DQK + a * 64,
                      batch * p.seq + blk * ATT_BN);
        for (int a = 0; a < 2; ++a)
          tma_load_2d(smem + L::kKtOff + (u * 2 + a) * L::kKtAtomBytes, &tmap_kt, &bar_k[u], blk * ATT_BN + a * 64,
                      (batch * p.heads + head) * DQK);
      };
      // dP = dO V^T over the whole value width: atoms through a two-stage ring, the next load in flight during the MMAs
      auto load_atom = [&](uint32_t n, int a, int blk) -> bool {
        const int st = n & 1;
        if (!mbar_wait_bounded(&ring_free[st], ((n >> 1) & 1) ^ 1, abort_flag)) return false;
        uint8_t* base = smem + L::kRingOff + st * 2 * ATOM_BYTES_128;
        mbar_arrive_expect_tx(&ring_full[st], 2 * ATOM_BYTES_128);
        tma_load_2d(base, &tmap_do, &ring_full[st], head * p.dv + a * 64, batch * p.seq + q0);
        tma_load_2d(base + ATOM_BYTES_128, &tmap_v, &ring_full[st], head * p.dv + a * 64, batch * p.seq + blk * ATT_BN);
        return true;
      };
      if (kb == 0 || !L::kDouble) {  // (double-buffered: issued during the previous block, see below)
        load_block(kb);
        got = load_atom(ring_n, 0, kb);
      }
      if (kb == 0) got = got && mbar_wait_bounded(bar_q, 0, abort_flag);
      got = got && mbar_wait_bounded(&bar_k[ub], L::kDouble ? ((kb >> 1) & 1) : parity, abort_flag);
      if (got) {
        tc_fence_after();
        issue_mma_atoms(tmem_s, smem_u32(smem + L::kQOff), ATOM_BYTES_128, smem_u32(smem + L::kKOff + ub * L::kQBytes),
                        ATOM_BYTES_128, DQK / 16, make_idesc_bf16(ATT_BM, ATT_BN), false);
        for (int a = 0; a < dv_atoms && got; ++a) {
          const uint32_t n = ring_n + a;
          if (a + 1 < dv_atoms) got = load_atom(n + 1, a + 1, kb);
          got = got && mbar_wait_bounded(&ring_full[n & 1], (n >> 1) & 1, abort_flag);
          if (!got) break;
          tc_fence_after();
          const uint32_t base = smem_u32(smem + L::kRingOff + (n & 1) * 2 * ATOM_BYTES_128);
          issue_mma_atoms(tmem_dp, base, 0, base + ATOM_BYTES_128, 0, 4, make_idesc_bf16(ATT_BM, ATT_BN), a > 0);
          umma_commit(&ring_free[n & 1]);
        }
        ring_n += dv_atoms;
      }
      if (!got) {
        report_status(p.status, kTimeoutFullBarrier, kb);
        *abort_flag = 1;
      }
      umma_commit(bar_mma1);
      if (L::kDouble && got && kb + 1 < n_kblocks) {
        // next key block: its K / K^T buffer was last read by the MMAs of block kb - 1 (complete); the ring stage
        // frees up when this block's last dP MMAs have read it
        load_block(kb + 1);
        if (!load_atom(ring_n, 0, kb + 1)) {
          report_status(p.status, kTimeoutEmptyBarrier, kb);
          *abort_flag = 1;
        }
      }
    }
    if (!mbar_wait_bounded(bar_mma1, parity, abort_flag)) {
      report_status(p.status, kTimeoutTmemFull, kb);
      *abort_flag = 1;
    }
    __syncthreads();
    ok = (*abort_flag == 0);
    if (!ok) break;
    tc_fence_after();

#pragma unroll 1
    for (int c = 0; c < ATT_BN / 32; ++c) {
      uint32_t rs[32], rp[32];
      tmem_ld_32x32b_x32(tmem_s + lane_off + (uint32_t)(c * 32), rs);
      tmem_ld_32x32b_x32(tmem_dp + lane_off + (uint32_t)(c * 32), rp);
      tmem_wait_ld();
      float ds[32];
      if (kb < qblk && k0 + ATT_BN <= p.seq) {
        // a block below the diagonal and inside the sequence: nothing to mask (uniform over the CTA)
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float pr = exp2f(fmaf(__uint_as_float(rs[j]), p.scale_log2, -lse2));
          ds[j] = pr * (__uint_as_float(rp[j]) - delta) * p.scale;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int kpos = k0 + c * 32 + j;
          const bool valid = kpos <= qpos && kpos < p.seq;
          const float pr = valid ? exp2f(fmaf(__uint_as_float(rs[j]), p.scale_log2, -lse2)) : 0.0f;
          ds[j] = pr * (__uint_as_float(rp[j]) - delta) * p.scale;
        }
      }
      uint8_t* atom = smem + L::kDsOff + (c / 2) * ATOM_BYTES_128;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 u;
        u.x = pack_bf16x2(ds[g * 8 + 0], ds[g * 8 + 1]);
        u.y = pack_bf16x2(ds[g * 8 + 2], ds[g * 8 + 3]);
        u.z = pack_bf16x2(ds[g * 8 + 4], ds[g * 8 + 5]);
        u.w = pack_bf16x2(ds[g * 8 + 6], ds[g * 8 + 7]);
        *reinterpret_cast<uint4*>(atom + sw128_chunk_off(row, (c % 2) * 4 + g)) = u;
      }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) {
      tc_fence_after();
      // dQ += dS [128 q x 128 keys] * (K^T [DQK x 128 keys])^T
      issue_mma_atoms(tmem_dq, smem_u32(smem + L::kDsOff), ATOM_BYTES_128,
                      smem_u32(smem + L::kKtOff + ub * 2 * L::kKtAtomBytes), L::kKtAtomBytes, ATT_BN / 16,
                      make_idesc_bf16(ATT_BM, DQK), kb > 0);
      umma_commit(bar_mma2);
    }
    if (!mbar_wait_bounded(bar_mma2, parity, abort_flag)) {
      report_status(p.status, kTimeoutTmemFull, 1000 + kb);
      *abort_flag = 1;
    }
    tc_fence_before();
    __syncthreads();
    ok = (*abort_flag == 0);
  }

  if (ok) {
    tc_fence_after();
#pragma unroll 1
    for (int c = 0; c < DQK / 32; ++c) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(tmem_dq + lane_off + (uint32_t)(c * 32), r);
      tmem_wait_ld();
      if (row_ok) {
        float* dst = p.dq + (((size_t)batch * p.seq + qpos) * p.heads + head) * DQK + c * 32;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                            __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int DQK, int DVC>
__global__ void __launch_bounds__(ATT_THREADS)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_q,
                    const __grid_constant__ CUtensorMap tmap_qt, const __grid_constant__ CUtensorMap tmap_v,
                    const __grid_constant__ CUtensorMap tmap_do, const __grid_constant__ CUtensorMap tmap_dot,
                    const AttnBwdParams p) {
  using L = BwdDkvSmem<DQK, DVC>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* bar_k = bars + 0;
  uint64_t* bar_q = bars + 1;      // [2] Q_i loads, one per buffer
  uint64_t* bar_t = bars + 3;      // Q_i^T / dO_i^T loads
  uint64_t* bar_mma1 = bars + 4;
  uint64_t* bar_mma2 = bars + 5;
  uint64_t* ring_full = bars + 6;  // [2]
  uint64_t* ring_free = bars + 8;  // [2]
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem + L::kTmemPtrOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);
  float* s_lse = reinterpret_cast<float*>(smem + L::kLseOff);
  float* s_delta = reinterpret_cast<float*>(smem + L::kDeltaOff);

  const int warp = threadIdx.x >> 5;
  const int n_blocks = (p.seq + ATT_BM - 1) / ATT_BM;
  const int kblk = (int)blockIdx.x;  // key block 0 meets every query block: longest first
  const int dv_chunks = p.dv / DVC;
  const int head = (int)blockIdx.y / dv_chunks;
  const int chunk = (int)blockIdx.y - head * dv_chunks;
  const int dv0 = chunk * DVC;
  const bool do_dk = chunk == 0;
  const int batch = (int)blockIdx.z;
  const int k0 = kblk * ATT_BN;
  const int row = (int)threadIdx.x;
  const int kpos = k0 + row;
  const bool row_ok = kpos < p.seq;
  const int dv_atoms = p.dv / 64;

  if (threadIdx.x == 0) {
    for (int i = 0; i < L::kNumBars; ++i) mbar_init(&bars[i], 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_ptr_smem, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const uint32_t tmem_st = tmem_base, tmem_dpt = tmem_base + 128, tmem_dv = tmem_base + 256, tmem_dk = tmem_base + 384;
  const uint32_t lane_off = (uint32_t)(warp * 32) << 16;

  if (threadIdx.x == 0) {
    mbar_arrive_expect_tx(bar_k, L::kKBytes);
    for (int a = 0; a < DQK / 64; ++a)
      tma_load_2d(smem + L::kKOff + a * ATOM_BYTES_128, &tmap_k, bar_k, head * DQK + a * 64, batch * p.seq + k0);
  }

  uint32_t ring_n = 0;
  bool ok = true;
  int it = 0;
  for (int qb = kblk; qb < n_blocks && ok; ++qb, ++it) {
    const int q0 = qb * ATT_BM;
    const uint32_t parity = it & 1;
    {
      // statistics of this query block's rows (columns of S^T)
      const int qp = q0 + row;
      const size_t o = ((size_t)batch * p.heads + head) * p.seq + (qp < p.seq ? qp : 0);
      s_lse[row] = qp < p.seq ? p.lse[o] * 1.4426950408889634f : INFINITY;
      s_delta[row] = qp < p.seq ? p.delta[o] : 0.0f;
    }
    const int uq = L::kDouble ? (it & 1) : 0;  // Q buffer of this query block
    auto load_q = [&](int blk, int u) {
      mbar_arrive_expect_tx(&bar_q[u], L::kKBytes);
      for (int a = 0; a < DQK / 64; ++a)
        tma_load_2d(smem + L::kQOff + u * L::kKBytes + a * ATOM_BYTES_128, &tmap_q, &bar_q[u], head * DQK + a * 64,
                    batch * p.seq + blk * ATT_BM);
    };
    auto load_atom = [&](uint32_t n, int a, int blk) -> bool {
      const int st = n & 1;
      if (!mbar_wait_bounded(&ring_free[st], ((n >> 1) & 1) ^ 1, abort_flag)) return false;
      uint8_t* base = smem + L::kRingOff + st * 2 * ATOM_BYTES_128;
      mbar_arrive_expect_tx(&ring_full[st], 2 * ATOM_BYTES_128);
      tma_load_2d(base, &tmap_v, &ring_full[st], head * p.dv + a * 64, batch * p.seq + k0);
      tma_load_2d(base + ATOM_BYTES_128, &tmap_do, &ring_full[st], head * p.dv + a * 64, batch * p.seq + blk * ATT_BM);
      return true;
    };
    if (threadIdx.x == 0) {
      bool got = true;
      if (it == 0 || !L::kDouble) {  // (double-buffered: issued during the previous block, see below)
        load_q(qb, uq);
        got = load_atom(ring_n, 0, qb);
      }
      if (it == 0) got = got && mbar_wait_bounded(bar_k, 0, abort_flag);
      got = got && mbar_wait_bounded(&bar_q[uq], L::kDouble ? ((it >> 1) & 1) : parity, abort_flag);
      if (got) {
        tc_fence_after();
        // S^T = K_j Q_i^T
        issue_mma_atoms(tmem_st, smem_u32(smem + L::kKOff), ATOM_BYTES_128, smem_u32(smem + L::kQOff + uq * L::kKBytes),
                        ATOM_BYTES_128, DQK / 16, make_idesc_bf16(ATT_BM, ATT_BN), false);
        // dP^T = V_j dO_i^T over the whole value width
        for (int a = 0; a < dv_atoms && got; ++a) {
          const uint32_t n = ring_n + a;
          if (a + 1 < dv_atoms) got = load_atom(n + 1, a + 1, qb);
          got = got && mbar_wait_bounded(&ring_full[n & 1], (n >> 1) & 1, abort_flag);
          if (!got) break;
          tc_fence_after();
          const uint32_t base = smem_u32(smem + L::kRingOff + (n & 1) * 2 * ATOM_BYTES_128);
          issue_mma_atoms(tmem_dpt, base, 0, base + ATOM_BYTES_128, 0, 4, make_idesc_bf16(ATT_BM, ATT_BN), a > 0);
          umma_commit(&ring_free[n & 1]);
        }
        ring_n += dv_atoms;
      }
      if (!got) {
        report_status(p.status, kTimeoutFullBarrier, it);
        *abort_flag = 1;
      }
      umma_commit(bar_mma1);
    }
    if (!mbar_wait_bounded(bar_mma1, parity, abort_flag)) {
      report_status(p.status, kTimeoutTmemFull, it);
      *abort_flag = 1;
    }
    __syncthreads();  // also publishes s_lse / s_delta
    ok = (*abort_flag == 0);
    if (!ok) break;
    tc_fence_after();

    // Q_i and the ring are free now (their MMAs completed): fetch Q_i^T and the dO_i^T chunk while the threads work. The
    // chunk goes into the ring stage that the NEXT query block's first atom does not use, so that atom (and the next Q
    // tile, into the other Q buffer) can be fetched now as well.
    const int dot_stage = L::kDouble ? (int)((ring_n & 1) ^ 1) : 0;
    if (threadIdx.x == 0) {
      // both ring stages must be idle before anything overwrites them (their last MMAs were committed above)
      bool got = mbar_wait_bounded(&ring_free[0], (((ring_n + 1) >> 1) & 1) ^ 1, abort_flag) &&
                 mbar_wait_bounded(&ring_free[1], ((ring_n >> 1) & 1) ^ 1, abort_flag);
      if (got) {
        mbar_arrive_expect_tx(bar_t, (do_dk ? 2 * L::kQtAtomBytes : 0) + 2 * L::kDotAtomBytes);
        if (do_dk)
          for (int a = 0; a < 2; ++a)
            tma_load_2d(smem + L::kQOff + uq * L::kKBytes + a * L::kQtAtomBytes, &tmap_qt, bar_t, q0 + a * 64,
                        (batch * p.heads + head) * DQK);
        for (int a = 0; a < 2; ++a)
          tma_load_2d(smem + L::kRingOff + dot_stage * 2 * ATOM_BYTES_128 + a * L::kDotAtomBytes, &tmap_dot, bar_t,
                      q0 + a * 64, (batch * p.heads + head) * p.dv + dv0);
        if (L::kDouble && qb + 1 < n_blocks) {
          load_q(qb + 1, uq ^ 1);  // that buffer held Q^T of block qb - 1, read by MMAs that have completed
          got = load_atom(ring_n, 0, qb + 1);
        }
      }
      if (!got) {
        report_status(p.status, kTimeoutEmptyBarrier, it);
        *abort_flag = 1;
      }
    }
    __syncwarp();  // warp 0 is whole again before its warp-wide TMEM loads

#pragma unroll 1
    for (int c = 0; c < ATT_BM / 32; ++c) {
      uint32_t rs[32], rp[32];
      tmem_ld_32x32b_x32(tmem_st + lane_off + (uint32_t)(c * 32), rs);
      tmem_ld_32x32b_x32(tmem_dpt + lane_off + (uint32_t)(c * 32), rp);
      tmem_wait_ld();
      float pt[32], ds[32];
      if (qb > kblk && q0 + ATT_BM <= p.seq && k0 + ATT_BN <= p.seq) {
        // a query block above the diagonal, both blocks inside the sequence: nothing to mask (uniform over the CTA)
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int col = c * 32 + j;
          pt[j] = exp2f(fmaf(__uint_as_float(rs[j]), p.scale_log2, -s_lse[col]));
          ds[j] = pt[j] * (__uint_as_float(rp[j]) - s_delta[col]) * p.scale;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int col = c * 32 + j;
          const int qp = q0 + col;
          const bool valid = row_ok && kpos <= qp && qp < p.seq;
          pt[j] = valid ? exp2f(fmaf(__uint_as_float(rs[j]), p.scale_log2, -s_lse[col])) : 0.0f;
          ds[j] = pt[j] * (__uint_as_float(rp[j]) - s_delta[col]) * p.scale;
        }
      }
      uint8_t* atom_p = smem + L::kPtOff + (c / 2) * ATOM_BYTES_128;
      uint8_t* atom_d = smem + L::kDstOff + (c / 2) * ATOM_BYTES_128;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 u, w;
        u.x = pack_bf16x2(pt[g * 8 + 0], pt[g * 8 + 1]);
        u.y = pack_bf16x2(pt[g * 8 + 2], pt[g * 8 + 3]);
        u.z = pack_bf16x2(pt[g * 8 + 4], pt[g * 8 + 5]);
        u.w = pack_bf16x2(pt[g * 8 + 6], pt[g * 8 + 7]);
        w.x = pack_bf16x2(ds[g * 8 + 0], ds[g * 8 + 1]);
        w.y = pack_bf16x2(ds[g * 8 + 2], ds[g * 8 + 3]);
        w.z = pack_bf16x2(ds[g * 8 + 4], ds[g * 8 + 5]);
        w.w = pack_bf16x2(ds[g * 8 + 6], ds[g * 8 + 7]);
        const uint32_t off = sw128_chunk_off(row, (c % 2) * 4 + g);
        *reinterpret_cast<uint4*>(atom_p + off) = u;
        *reinterpret_cast<uint4*>(atom_d + off) = w;
      }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) {
      bool got = (*abort_flag == 0) && mbar_wait_bounded(bar_t, parity, abort_flag);
      if (got) {
        tc_fence_after();
        // dV += P^T [128 keys x 128 q] * (dO^T chunk [DVC x 128 q])^T
        issue_mma_atoms(tmem_dv, smem_u32(smem + L::kPtOff), ATOM_BYTES_128,
                        smem_u32(smem + L::kRingOff + dot_stage * 2 * ATOM_BYTES_128), L::kDotAtomBytes, ATT_BM / 16,
                        make_idesc_bf16(ATT_BM, DVC), it > 0);
        // dK += dS^T [128 keys x 128 q] * (Q^T [DQK x 128 q])^T
        if (do_dk)
          issue_mma_atoms(tmem_dk, smem_u32(smem + L::kDstOff), ATOM_BYTES_128, smem_u32(smem + L::kQOff + uq * L::kKBytes),
                          L::kQtAtomBytes, ATT_BM / 16, make_idesc_bf16(ATT_BM, DQK), it > 0);
      } else {
        report_status(p.status, kTimeoutFullBarrier, 2000 + it);
        *abort_flag = 1;
      }
      umma_commit(bar_mma2);
    }
    if (!mbar_wait_bounded(bar_mma2, parity, abort_flag)) {
      report_status(p.status, kTimeoutTmemFull, 1000 + it);
      *abort_flag = 1;
    }
    tc_fence_before();
    __syncthreads();
    ok = (*abort_flag == 0);
  }

  if (ok) {
    tc_fence_after();
#pragma unroll 1
    for (int c = 0; c < DVC / 32; ++c) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(tmem_dv + lane_off + (uint32_t)(c * 32), r);
      tmem_wait_ld();
      if (row_ok) {
        float* dst = p.dv_out + (((size_t)batch * p.seq + kpos) * p.heads + head) * p.dv + dv0 + c * 32;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                            __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
      }
    }
    if (do_dk) {
#pragma unroll 1
      for (int c = 0; c < DQK / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_dk + lane_off + (uint32_t)(c * 32), r);
        tmem_wait_ld();
        if (row_ok) {
          float* dst = p.dk + (((size_t)batch * p.seq + kpos) * p.heads + head) * DQK + c * 32;
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                              __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int DQK>
static cudaError_t attn_bwd_dq_variant(const CUtensorMap* maps, const AttnBwdParams& p, cudaStream_t stream) {
  using L = BwdDqSmem<DQK>;
  static_assert(L::kDynamicBytes <= 232448, "shared memory of one CTA exceeds 227 KB");
  auto kern = attn_bwd_dq_kernel<DQK>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
  if (e != cudaSuccess) return e;
  dim3 grid((p.seq + ATT_BM - 1) / ATT_BM, p.heads, p.batch);
  kern<<<grid, ATT_THREADS, L::kDynamicBytes, stream>>>(maps[0], maps[1], maps[2], maps[3], maps[4], p);
  return cudaGetLastError();
}

template <int DQK, int DVC>
static cudaError_t attn_bwd_dkv_variant(const CUtensorMap* maps, const AttnBwdParams& p, cudaStream_t stream) {
  using L = BwdDkvSmem<DQK, DVC>;
  static_assert(L::kDynamicBytes <= 232448, "shared memory of one CTA exceeds 227 KB");
  auto kern = attn_bwd_dkv_kernel<DQK, DVC>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
  if (e != cudaSuccess) return e;
  dim3 grid((p.seq + ATT_BM - 1) / ATT_BM, p.heads * (p.dv / DVC), p.batch);
  kern<<<grid, ATT_THREADS, L::kDynamicBytes, stream>>>(maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], p);
  return cudaGetLastError();
}

// maps_dq = {q, k, k^T, dO, v}; maps_dkv = {k, q, q^T, v, dO, dO^T}
int attn_bwd_launch(const CUtensorMap* maps_dq, const CUtensorMap* maps_dkv, const AttnBwdParams& p, cudaStream_t stream) {
  const int dvc = attn_value_chunk(p.dv);
  if (dvc == 0 || (p.dqk != 64 && p.dqk != 128) || p.seq % 8 != 0 || p.batch > 65535 || p.heads * (p.dv / dvc) > 65535)
    return (int)cudaErrorInvalidValue;
  cudaError_t e = p.dqk == 64 ? attn_bwd_dq_variant<64>(maps_dq, p, stream) : attn_bwd_dq_variant<128>(maps_dq, p, stream);
  if (e != cudaSuccess) return (int)e;
  if (p.dqk == 64) e = dvc == 128 ? attn_bwd_dkv_variant<64, 128>(maps_dkv, p, stream) : attn_bwd_dkv_variant<64, 64>(maps_dkv, p, stream);
  else e = dvc == 128 ? attn_bwd_dkv_variant<128, 128>(maps_dkv, p, stream) : attn_bwd_dkv_variant<128, 64>(maps_dkv, p, stream);
  return (int)e;
}


// Value columns per CTA of the forward kernel: with 128-wide queries the double-buffered tiles only fit for 64.
int attn_fwd_value_chunk(int dqk, int dv) {
  const int c = attn_value_chunk(dv);
  return (dqk == 128 && c == 128) ? 64 : c;
}

int attn_fwd_launch(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tvt, const AttnParams& p,
                    cudaStream_t stream) {
  const int dvc = attn_fwd_value_chunk(p.dqk, p.dv);
  if (dvc == 0 || (p.dqk != 64 && p.dqk != 128) || p.seq % 8 != 0 || p.batch > 65535 || p.heads * (p.dv / dvc) > 65535)
    return (int)cudaErrorInvalidValue;
  cudaError_t e;
  if (p.dqk == 64) e = dvc == 128 ? attn_fwd_variant<64, 128>(tq, tk, tvt, p, stream) : attn_fwd_variant<64, 64>(tq, tk, tvt, p, stream);
  else e = attn_fwd_variant<128, 64>(tq, tk, tvt, p, stream);
  return (int)e;
}

}  // namespace lmsae
