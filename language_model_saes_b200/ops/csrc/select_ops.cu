// Selection and compaction kernels (sm_100a, streaming SIMT kernels: one or two passes over the data at HBM speed).
//
//  radix_hist_hi / radix_hist_lo / radix_pick
//        exact k-th largest POSITIVE value of a big tensor by a two-level radix select on the float bit pattern
//        (positive IEEE floats order like their bits): a 32,640-bin shared-memory histogram of the upper 16 bits, one
//        CTA picks the bin that holds the k-th value, a second pass histograms the lower 16 bits of that bin's members.
//        This is the batch-level top-k ("BatchTopK": keep the k * batch largest pre-activations of the whole batch,
//        models/sparse_dictionary.py:775-788 and utils/distributed/ops.py:158-266 of the reference project, which sorts
//        or bisects with one all-reduce per iteration). Feature- or data-sharded callers sum the histograms across ranks
//        between a histogram and its pick, so the whole exchange is two small all-reduces.
//  row_nnz / row_compact
//        dense [B, N] activations -> padded sparse (column, value) lists in ascending column order.
//  gather_rows_cast
//        out[pos[i], :] = cast(src[i, :]) for rows with keep[i] != 0: token-mask compaction of cached activations
//        (activation/processors/cached_activation.py:301-320, activation/processors/activation.py:277-285).
#include "common.cuh"
#include "kernels.h"

namespace lmsae {

namespace {

constexpr int kHiBins = 0x7F80;  // upper 16 bits of positive finite floats and +inf: 0 .. 0x7F80 - 1 (+inf = 0x7F80 clipped)
constexpr int HIST_THREADS = 1024;

template <typename T>
__device__ __forceinline__ uint32_t positive_bits(T v);
template <>
__device__ __forceinline__ uint32_t positive_bits<float>(float v) {
  return v > 0.0f ? __float_as_uint(v) : 0u;
}
template <>
__device__ __forceinline__ uint32_t positive_bits<__nv_bfloat16>(__nv_bfloat16 v) {
  const float f = __bfloat162float(v);
  return f > 0.0f ? __float_as_uint(f) : 0u;
}

__device__ __forceinline__ float to_float_any(float v) { return v; }
__device__ __forceinline__ float to_float_any(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_float_any(float v);
template <>
__device__ __forceinline__ float from_float_any<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float_any<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

template <typename T>
struct Vec;
template <>
struct Vec<float> {
  static constexpr int N = 4;
  __device__ static bool all_below(const uint4&, uint32_t) { return false; }
  __device__ static void decode(const uint4& v, uint32_t (&b)[4]) {
    b[0] = positive_bits(__uint_as_float(v.x)); b[1] = positive_bits(__uint_as_float(v.y));
    b[2] = positive_bits(__uint_as_float(v.z)); b[3] = positive_bits(__uint_as_float(v.w));
  }
};
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  // floor2: a positive bf16 pattern in both halves of a word (0: none). True when none of the eight elements reaches it
  // (as signed 16-bit integers positive floats order like their patterns, negative floats sort below all of them).
  __device__ static bool all_below(const uint4& v, uint32_t floor2) {
    return floor2 != 0u &&
           (__vcmpges2(v.x, floor2) | __vcmpges2(v.y, floor2) | __vcmpges2(v.z, floor2) | __vcmpges2(v.w, floor2)) == 0u;
  }
  __device__ static void decode(const uint4& v, uint32_t (&b)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // a bf16 is the upper half of the float with the same value; sign bit set or zero = not positive
      const uint32_t lo = w[i] << 16, hi = w[i] & 0xFFFF0000u;
      b[2 * i] = (lo & 0x80000000u) || (lo & 0x7FFFFFFFu) > 0x7F800000u ? 0u : lo;
      b[2 * i + 1] = (hi & 0x80000000u) || (hi & 0x7FFFFFFFu) > 0x7F800000u ? 0u : hi;
    }
  }
};

// x is a contiguous [A, S, N] array; the selection runs over all (a, n) of segment s: A rows of N contiguous elements.
// `visit(bits)` is called for every positive element whose float bits are at least `floor_bits` (0: every positive
// element). Rows are cut into chunks of threads x 16 bytes; 16-bit vectors without any element at the floor are
// rejected with four packed comparisons.
template <typename T, int THREADS, typename Fn>
__device__ __forceinline__ void for_each_positive(const T* __restrict__ x, long long A, long long S, long long N,
                                                  long long s, uint32_t floor_bits, Fn visit) {
  constexpr int V = Vec<T>::N;
  const long long chunk = (long long)THREADS * V;
  const long long chunks_per_row = (N + chunk - 1) / chunk;
  const bool vec_ok = (N % V == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0);
  const uint32_t floor2 = (floor_bits >> 16) * 0x10001u;  // the floor rounded down to 16 bits, in both halves
  const long long total = A * chunks_per_row;
  if (vec_ok) {
    // four chunks per round, all four loads issued before the first is looked at (one CTA of 1024 threads per SM has
    // no other way to keep enough bytes in flight)
    constexpr int U = 4;
    for (long long item0 = blockIdx.x; item0 < total; item0 += (long long)gridDim.x * U) {
      uint4 raw[U];
      bool have[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long item = item0 + (long long)u * gridDim.x;
        have[u] = false;
        if (item < total) {
          const long long a = item / chunks_per_row, ch = item - a * chunks_per_row;
          const long long e = ch * chunk + (long long)threadIdx.x * V;
          if (e < N) {
            raw[u] = __ldcs(reinterpret_cast<const uint4*>(x + (a * S + s) * N + e));
            have[u] = true;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (!have[u] || Vec<T>::all_below(raw[u], floor2)) continue;
        uint32_t b[V];
        Vec<T>::decode(raw[u], b);
#pragma unroll
        for (int i = 0; i < V; ++i)
          if (b[i] != 0 && b[i] >= floor_bits) visit(b[i]);
      }
    }
    return;
  }
  for (long long item = blockIdx.x; item < total; item += gridDim.x) {
    const long long a = item / chunks_per_row, ch = item - a * chunks_per_row;
    const T* row = x + (a * S + s) * N;
    const long long e = ch * chunk + (long long)threadIdx.x * V;
    if (e >= N) continue;
    for (int i = 0; i < V && e + i < N; ++i) {
      const uint32_t b = positive_bits<T>(row[e + i]);
      if (b != 0 && b >= floor_bits) visit(b);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(HIST_THREADS)
radix_hist_hi_kernel(const T* __restrict__ x, long long A, long long S, long long N, long long s,
                     unsigned* __restrict__ hist, const float* __restrict__ floor, const long long* __restrict__ need) {
  // `floor`: only values of at least *floor are counted (a caller that knows a lower bound of the value it is looking
  // for saves nearly all of the shared-memory atomics). `need`: the pass runs only if need[3] != 0 (the repeat without
  // a floor, for the case that the floor turned out to lie above the value sought).
  if (need != nullptr && need[3] == 0) return;
  extern __shared__ unsigned s_hist[];  // [kHiBins]
  for (int i = threadIdx.x; i < kHiBins; i += HIST_THREADS) s_hist[i] = 0;
  __syncthreads();
  const float fl = floor != nullptr ? *floor : 0.0f;
  const uint32_t floor_bits = fl > 0.0f ? __float_as_uint(fl) : 0u;
  for_each_positive<T, HIST_THREADS>(x, A, S, N, s, floor_bits, [&](uint32_t b) {
    uint32_t bin = b >> 16;
    if (bin >= (uint32_t)kHiBins) bin = kHiBins - 1;
    atomicAdd(&s_hist[bin], 1u);
  });
  __syncthreads();
  for (int i = threadIdx.x; i < kHiBins; i += HIST_THREADS) {
    const unsigned c = s_hist[i];
    if (c != 0) atomicAdd(&hist[i], c);
  }
}

// second level: members of the bin sel[0] only (a small fraction of the data), straight to global memory
template <typename T>
__global__ void __launch_bounds__(256)
radix_hist_lo_kernel(const T* __restrict__ x, long long A, long long S, long long N, long long s,
                     const long long* __restrict__ sel, unsigned* __restrict__ hist) {
  const uint32_t want = (uint32_t)sel[0];
  for_each_positive<T, 256>(x, A, S, N, s, 0u, [&](uint32_t b) {
    uint32_t bin = b >> 16;
    if (bin >= (uint32_t)kHiBins) bin = kHiBins - 1;
    if (bin == want) atomicAdd(&hist[b & 0xFFFFu], 1u);
  });
}

// One CTA: the largest bin b with  count(bins >= b) >= k.  sel_out = {b, k - count(bins > b), count(all bins)}.
// With fewer than k members in total the pick is bin 0 (everything positive passes). `level` 0 = upper bits, 1 = lower
// bits: level 1 takes k from sel_in[1], and writes the threshold  float((sel_in[0] << 16) | b)  to thr.
__global__ void __launch_bounds__(1024)
radix_pick_kernel(const unsigned* __restrict__ hist, int nbins, long long k, const long long* __restrict__ sel_in,
                  int level, long long* __restrict__ sel_out, float* __restrict__ thr, const long long* __restrict__ need) {
  // sel_out[3] = 1 when the histogram held fewer than k members (with a floored histogram: the floor was too high).
  // `need`: the pick runs only if need[3] != 0 (read by every thread before anything is written: need may be sel_out).
  const bool run_it = need == nullptr || need[3] != 0;
  __shared__ long long s_part[1024];
  __syncthreads();
  if (!run_it) return;
  __shared__ long long s_above;  // count in the chunks above the chosen chunk
  __shared__ int s_chunk;
  if (level == 1) k = sel_in[1];
  const bool take_all = k <= 0;  // fewer than k positive values overall: every positive value passes
  const int per = (nbins + 1023) / 1024;
  // thread i owns bins [hi - per, hi) counted from the top, so that a scan over threads walks downwards
  const int hi = nbins - (int)threadIdx.x * per;
  long long mine = 0;
  for (int b = hi - 1; b >= hi - per && b >= 0; --b) mine += hist[b];
  s_part[threadIdx.x] = mine;
  if (threadIdx.x == 0) { s_chunk = -1; s_above = 0; }
  __syncthreads();
  if (threadIdx.x == 0) {
    long long run = 0;
    for (int i = 0; i < 1024; ++i) {
      if (run + s_part[i] >= k && s_chunk < 0) { s_chunk = i; s_above = run; }
      run += s_part[i];
    }
    sel_out[2] = run;
    sel_out[3] = (level == 0 && run < k) ? 1 : 0;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    long long bin = 0, remaining = k;
    if (s_chunk >= 0) {
      long long run = s_above;
      const int top = nbins - s_chunk * per;
      for (int b = top - 1; b >= top - per && b >= 0; --b) {
        const long long c = hist[b];
        if (run + c >= k) { bin = b; remaining = k - run; break; }
        run += c;
      }
    } else {
      remaining = 0;  // fewer than k positive values: keep them all
    }
    if (take_all) { bin = 0; remaining = 0; }
    sel_out[0] = bin;
    sel_out[1] = remaining;
    if (level == 1 && thr != nullptr) {
      const uint32_t bits = ((uint32_t)sel_in[0] << 16) | (uint32_t)bin;
      // bin 0 of both levels = "everything positive": the smallest positive float keeps x > 0 as the rule
      *thr = bits == 0 ? __uint_as_float(1u) : __uint_as_float(bits);
    }
    if (level == 0 && thr != nullptr) {
      const uint32_t bits = (uint32_t)bin << 16;  // bf16 data: the upper half IS the value
      *thr = bits == 0 ? __uint_as_float(1u) : __uint_as_float(bits);
    }
  }
}

// out = x where x >= thr[segment] (thr > 0, so non-positive entries never pass), else 0; x is [A, S, N] contiguous.
template <typename T>
__global__ void __launch_bounds__(256)
threshold_mask_kernel(const T* __restrict__ x, const float* __restrict__ thr, long long rows, long long S, long long N,
                      T* __restrict__ out) {
  constexpr int V = Vec<T>::N;
  const bool vec_ok = (N % V == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (reinterpret_cast<uintptr_t>(out) % 16 == 0);
  const long long chunk = 256LL * V;
  const long long chunks_per_row = (N + chunk - 1) / chunk;
  for (long long item = blockIdx.x; item < rows * chunks_per_row; item += gridDim.x) {
    const long long r = item / chunks_per_row, ch = item - r * chunks_per_row;
    const float t = thr[r % S];
    const long long e = ch * chunk + (long long)threadIdx.x * V;
    if (e >= N) continue;
    const T* src = x + r * N + e;
    T* dst = out + r * N + e;
    if (vec_ok) {
      if constexpr (sizeof(T) == 4) {
        float4 v = __ldcs(reinterpret_cast<const float4*>(src));
        v.x = v.x >= t ? v.x : 0.f; v.y = v.y >= t ? v.y : 0.f; v.z = v.z >= t ? v.z : 0.f; v.w = v.w >= t ? v.w : 0.f;
        __stcs(reinterpret_cast<float4*>(dst), v);
      } else {
        uint4 u = __ldcs(reinterpret_cast<const uint4*>(src));
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 f = __bfloat1622float2(h[i]);
          f.x = f.x >= t ? f.x : 0.f;
          f.y = f.y >= t ? f.y : 0.f;
          h[i] = __floats2bfloat162_rn(f.x, f.y);
        }
        __stcs(reinterpret_cast<uint4*>(dst), u);
      }
    } else {
      for (int i = 0; i < V && e + i < N; ++i) {
        const float f = to_float_any(src[i]);
        dst[i] = f >= t ? src[i] : from_float_any<T>(0.f);
      }
    }
  }
}

// ---- dense rows -> padded sparse lists --------------------------------------------------------------
constexpr int RC_THREADS = 256;

// 16 bytes of a row as raw words: V elements of type T; element i as a float, and a scalar fall-back loader that packs
// the in-range elements of an unaligned or ragged vector (zeros elsewhere).
template <typename T>
struct RowVec;
template <>
struct RowVec<float> {
  static constexpr int V = 4;
  __device__ static float get(const uint4& u, int i) {
    return __uint_as_float(i == 0 ? u.x : i == 1 ? u.y : i == 2 ? u.z : u.w);
  }
  __device__ static uint4 gather(const float* p, long long n_valid) {
    uint4 u = make_uint4(0u, 0u, 0u, 0u);
    if (n_valid > 0) u.x = __float_as_uint(p[0]);
    if (n_valid > 1) u.y = __float_as_uint(p[1]);
    if (n_valid > 2) u.z = __float_as_uint(p[2]);
    if (n_valid > 3) u.w = __float_as_uint(p[3]);
    return u;
  }
};
template <>
struct RowVec<__nv_bfloat16> {
  static constexpr int V = 8;
  __device__ static float get(const uint4& u, int i) {
    const unsigned w = (i >> 1) == 0 ? u.x : (i >> 1) == 1 ? u.y : (i >> 1) == 2 ? u.z : u.w;
    return __uint_as_float((i & 1) ? (w & 0xffff0000u) : (w << 16));
  }
  __device__ static uint4 gather(const __nv_bfloat16* p, long long n_valid) {
    unsigned w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < n_valid) w[i >> 1] |= (unsigned)__bfloat16_as_ushort(p[i]) << ((i & 1) * 16);
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// One CTA per row (grid-stride). Every warp owns one contiguous eighth of the row and streams it with RC_U 16-byte
// loads in flight per lane; nothing in the streaming loops synchronises the block.
//   Without thr an entry is kept when x != 0. With thr (> 0): entries above *thr are kept; entries EQUAL to it are
//   kept too, unless tie_quota is given, in which case only the first tie_quota[row] of them (in column order) are:
//   that is how a caller keeps an exact number of entries when the threshold value repeats.
//   A counting call (idx == nullptr) is one streaming pass; with `ties` it reports the two kinds separately
//   (nnz = entries above the threshold, ties = entries equal to it); with `seg_counts` it also stores every warp
//   segment's two counts ([B, 8, 2]).
//   A compacting call needs those per-segment counts to know where a warp's entries start in the list: it takes them
//   from `seg_counts` when a counting call of the same matrix and threshold left them there, and counts them itself
//   in a first pass over the row otherwise. The second pass finds an entry's slot with warp-level scans (lanes hold
//   consecutive columns, warps consecutive segments), so the list comes out in ascending column order.
//   With col_div the stored value is x / col_div[column] (gated pre-activation back to the activation).
//   With col_thr (one threshold per column, instead of thr) an entry is kept when x > col_thr[column]: the JumpReLU
//   selection of pre-activations against per-feature thresholds.
constexpr int RC_U = 4;

struct RowPredicate {
  bool has_thr, split_ties;
  float t;
  const float* col_thr;
  // bf16 rows against a positive threshold that is itself a bf16 value: the comparison runs on the raw 16-bit patterns,
  // two elements per instruction (as signed integers, positive floats order like their patterns and every negative
  // float sorts below them)
  bool raw16;
  unsigned t2;  // the threshold's pattern in both halves of a word
  bool raw16_nonzero;  // bf16 rows, "keep what is not zero": a packed test of the 15 magnitude bits
};

// bit i of the two masks: element c + i is kept outright / equals the threshold
template <typename T>
__device__ __forceinline__ void rc_classify(const uint4& u, long long c, long long end, const RowPredicate& q,
                                            unsigned& m_strict, unsigned& m_tie) {
  constexpr int V = RowVec<T>::V;
  m_strict = m_tie = 0;
  if constexpr (V == 8) {
    if (q.raw16_nonzero) {  // (+0 and -0 are both "zero"; elements past the end of the row were loaded as zeros)
      const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const unsigned g = __vcmpne2(w[j] & 0x7fff7fffu, 0u);
        m_strict |= ((g & 1u) | ((g >> 15) & 2u)) << (2 * j);
      }
      return;
    }
    if (q.raw16) {  // (elements past the end of the row were loaded as zeros: never above or equal to a positive threshold)
      const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const unsigned g = q.split_ties ? __vcmpgts2(w[j], q.t2) : __vcmpges2(w[j], q.t2);
        m_strict |= ((g & 1u) | ((g >> 15) & 2u)) << (2 * j);
        if (q.split_ties) {
          const unsigned e = __vcmpeq2(w[j], q.t2);
          m_tie |= ((e & 1u) | ((e >> 15) & 2u)) << (2 * j);
        }
      }
      return;
    }
  }
  if (q.col_thr != nullptr && c + V <= end && (c & 3) == 0) {
    // a whole vector against its columns' thresholds, fetched four at a time
    float th[V];
#pragma unroll
    for (int j = 0; j < V / 4; ++j) {
      const float4 t4 = __ldg(reinterpret_cast<const float4*>(q.col_thr + c) + j);
      th[4 * j] = t4.x; th[4 * j + 1] = t4.y; th[4 * j + 2] = t4.z; th[4 * j + 3] = t4.w;
    }
#pragma unroll
    for (int i = 0; i < V; ++i) m_strict |= (unsigned)(RowVec<T>::get(u, i) > th[i]) << i;
    return;
  }
#pragma unroll
  for (int i = 0; i < V; ++i) {
    const bool in = c + i < end;
    const float f = RowVec<T>::get(u, i);
    if (q.split_ties) {
      m_strict |= (unsigned)(in && f > q.t) << i;
      m_tie |= (unsigned)(in && f == q.t) << i;
    } else if (q.col_thr != nullptr) {
      m_strict |= (unsigned)(in && f > q.col_thr[in ? c + i : 0]) << i;
    } else {
      m_strict |= (unsigned)(in && (q.has_thr ? (f >= q.t) : (f != 0.0f))) << i;
    }
  }
}

template <typename T>
__device__ __forceinline__ uint4 rc_load(const T* xr, long long c, long long end, bool vec_ok) {
  if (c >= end) return make_uint4(0u, 0u, 0u, 0u);
  if (vec_ok) return __ldcs(reinterpret_cast<const uint4*>(xr + c));
  return RowVec<T>::gather(xr + c, end - c);
}

template <typename T>
__global__ void __launch_bounds__(RC_THREADS, 3)
row_compact_kernel(const T* __restrict__ x, int B, long long N, int cap, int* __restrict__ idx, float* __restrict__ val,
                   int* __restrict__ nnz, const float* __restrict__ thr, const float* __restrict__ col_div,
                   int* __restrict__ ties, const int* __restrict__ tie_quota, const float* __restrict__ col_thr,
                   int* __restrict__ seg_counts) {
  constexpr int V = RowVec<T>::V;
  constexpr int NW = RC_THREADS / 32;
  RowPredicate q;
  q.has_thr = thr != nullptr;
  q.t = q.has_thr ? *thr : 0.0f;
  q.split_ties = q.has_thr && (ties != nullptr || tie_quota != nullptr);
  q.col_thr = col_thr;
  q.raw16 = false;
  q.t2 = 0u;
  q.raw16_nonzero = V == 8 && !q.has_thr && col_thr == nullptr;
  if constexpr (V == 8) {
    const __nv_bfloat16 tb = __float2bfloat16(q.t);
    q.raw16 = q.has_thr && q.t > 0.0f && __bfloat162float(tb) == q.t;
    q.t2 = (unsigned)__bfloat16_as_ushort(tb) * 0x10001u;
  }
  const bool vec_ok = (N % V == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0);
  __shared__ int s_a[NW], s_b[NW];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // a warp's segment: an eighth of the row, rounded up to whole vectors
  const long long seg_len = (((N + NW - 1) / NW) + V - 1) / V * V;
  const long long s0 = min(N, (long long)warp * seg_len), s1 = min(N, s0 + seg_len);
  const long long stride = 32LL * V * RC_U;
  const bool counting = idx == nullptr;

  for (int row = blockIdx.x; row < B; row += gridDim.x) {
    const T* xr = x + (size_t)row * N;
    int n_s = 0, n_t = 0;
    if (counting || seg_counts == nullptr) {
      // ---- pass 1: this segment's counts
      for (long long c0 = s0; c0 < s1; c0 += stride) {
        uint4 raw[RC_U];
#pragma unroll
        for (int u = 0; u < RC_U; ++u) raw[u] = rc_load<T>(xr, c0 + ((long long)u * 32 + lane) * V, s1, vec_ok);
#pragma unroll
        for (int u = 0; u < RC_U; ++u) {
          unsigned ms, mt;
          rc_classify<T>(raw[u], c0 + ((long long)u * 32 + lane) * V, s1, q, ms, mt);
          n_s += __popc(ms);
          n_t += __popc(mt);
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        n_s += __shfl_xor_sync(0xffffffffu, n_s, o);
        n_t += __shfl_xor_sync(0xffffffffu, n_t, o);
      }
      if (counting && seg_counts != nullptr && lane == 0) {
        seg_counts[((size_t)row * NW + warp) * 2] = n_s;
        seg_counts[((size_t)row * NW + warp) * 2 + 1] = n_t;
      }
    } else {
      n_s = seg_counts[((size_t)row * NW + warp) * 2];
      n_t = seg_counts[((size_t)row * NW + warp) * 2 + 1];
    }
    __syncthreads();  // (the previous row's readers of s_a / s_b are done)
    if (lane == 0) { s_a[warp] = n_s; s_b[warp] = n_t; }
    __syncthreads();
    int s_before = 0, t_before = 0, s_total = 0, t_total = 0;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      if (w < warp) { s_before += s_a[w]; t_before += s_b[w]; }
      s_total += s_a[w];
      t_total += s_b[w];
    }
    if (counting) {
      if (threadIdx.x == 0) {
        if (nnz != nullptr) nnz[row] = s_total;
        if (ties != nullptr) ties[row] = t_total;
      }
      continue;
    }
    // ---- pass 2: compaction of this segment; S_seen / T_seen: strict entries and ties of the row before the next vector
    const int quota = tie_quota != nullptr ? tie_quota[row] : 0x7fffffff;
    int S_seen = s_before, T_seen = t_before;
    if (n_s + n_t > 0) {
      for (long long c0 = s0; c0 < s1; c0 += stride) {
        uint4 raw[RC_U];
#pragma unroll
        for (int u = 0; u < RC_U; ++u) raw[u] = rc_load<T>(xr, c0 + ((long long)u * 32 + lane) * V, s1, vec_ok);
#pragma unroll
        for (int u = 0; u < RC_U; ++u) {
          const long long c = c0 + ((long long)u * 32 + lane) * V;
          unsigned ms, mt;
          rc_classify<T>(raw[u], c, s1, q, ms, mt);
          if (__ballot_sync(0xffffffffu, (ms | mt) != 0u) == 0u) continue;  // nothing kept in these 32 vectors
          const int mine = __popc(ms) | (__popc(mt) << 16);  // both counts in one word (at most 256 each per warp)
          int inc = mine;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const int a = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += a;
          }
          const int tot = __shfl_sync(0xffffffffu, inc, 31);
          const int exc = inc - mine;
          int tie_rank = T_seen + (exc >> 16);
          int slot = S_seen + (exc & 0xffff) + min(tie_rank, quota);
#pragma unroll
          for (int i = 0; i < V; ++i) {
            const bool strict = (ms >> i) & 1u, tie = (mt >> i) & 1u;
            const bool keep = strict || (tie && tie_rank < quota);
            tie_rank += tie;
            if (keep) {
              if (slot < cap) {
                idx[(size_t)row * cap + slot] = (int)(c + i);
                const float f = RowVec<T>::get(raw[u], i);
                val[(size_t)row * cap + slot] = col_div != nullptr ? f / col_div[c + i] : f;
              }
              ++slot;
            }
          }
          S_seen += tot & 0xffff;
          T_seen += tot >> 16;
        }
      }
    }
    const int count = s_total + min(t_total, quota);
    if (threadIdx.x == 0 && nnz != nullptr) nnz[row] = count;
    for (int j = count + threadIdx.x; j < cap; j += RC_THREADS) {
      idx[(size_t)row * cap + j] = -1;
      val[(size_t)row * cap + j] = 0.0f;
    }
  }
}

// ---- masked row gather with a dtype cast ------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&f)[8]) {
  const float4 a = __ldcs(reinterpret_cast<const float4*>(p)), b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = __ldcs(reinterpret_cast<const uint4*>(p));
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&f)[8]);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&f)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]); o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = o;
}

// pos = exclusive prefix sum of keep; rows with keep != 0 land at out[pos[i], :]. d % 8 == 0; 8 elements per thread step
// (fp32 -> bf16 rounds to nearest even; the other three combinations are exact).
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
gather_rows_cast_kernel(const TI* __restrict__ src, const int* __restrict__ keep, const int* __restrict__ pos, long long n,
                        int d, TO* __restrict__ out, long long out_rows) {
  for (long long i = blockIdx.x; i < n; i += gridDim.x) {
    if (keep[i] == 0 || pos[i] < 0 || pos[i] >= out_rows) continue;  // a row that does not fit is dropped, never written
    const TI* s = src + (size_t)i * d;
    TO* o = out + (size_t)pos[i] * d;
    for (int c = threadIdx.x * 8; c < d; c += 256 * 8) {
      float f[8];
      load8<TI>(s + c, f);
      store8<TO>(o + c, f);
    }
  }
}

}  // namespace

int radix_hist_launch(int dtype, const void* x, long long A, long long S, long long N, long long s, int level,
                      const long long* sel, unsigned* hist, const float* floor, const long long* need,
                      cudaStream_t stream) {
  if (A <= 0 || N <= 0 || s < 0 || s >= S) return (int)cudaErrorInvalidValue;
  if (level == 0) {
    const size_t smem = (size_t)kHiBins * 4;
    cudaError_t e;
    if (dtype == 0) {
      e = cudaFuncSetAttribute(radix_hist_hi_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      radix_hist_hi_kernel<float><<<148, HIST_THREADS, smem, stream>>>(static_cast<const float*>(x), A, S, N, s, hist, floor, need);
    } else {
      e = cudaFuncSetAttribute(radix_hist_hi_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      radix_hist_hi_kernel<__nv_bfloat16>
          <<<148, HIST_THREADS, smem, stream>>>(static_cast<const __nv_bfloat16*>(x), A, S, N, s, hist, floor, need);
    }
  } else {
    if (dtype == 0)
      radix_hist_lo_kernel<float><<<148 * 8, 256, 0, stream>>>(static_cast<const float*>(x), A, S, N, s, sel, hist);
    else
      radix_hist_lo_kernel<__nv_bfloat16>
          <<<148 * 8, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), A, S, N, s, sel, hist);
  }
  return (int)cudaGetLastError();
}

int radix_hi_bins() { return kHiBins; }

int radix_pick_launch(const unsigned* hist, int nbins, long long k, const long long* sel_in, int level, long long* sel_out,
                      float* thr, const long long* need, cudaStream_t stream) {
  if (nbins <= 0 || nbins > 65536 || (level == 1 && sel_in == nullptr)) return (int)cudaErrorInvalidValue;
  radix_pick_kernel<<<1, 1024, 0, stream>>>(hist, nbins, k, sel_in, level, sel_out, thr, need);
  return (int)cudaGetLastError();
}

int threshold_mask_launch(int dtype, const void* x, const float* thr, long long A, long long S, long long N, void* out,
                          cudaStream_t stream) {
  const long long rows = A * S;
  if (rows <= 0 || N <= 0) return 0;
  if (dtype == 0)
    threshold_mask_kernel<float><<<148 * 8, 256, 0, stream>>>(static_cast<const float*>(x), thr, rows, S, N, static_cast<float*>(out));
  else
    threshold_mask_kernel<__nv_bfloat16><<<148 * 8, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), thr, rows, S, N,
                                                                     static_cast<__nv_bfloat16*>(out));
  return (int)cudaGetLastError();
}

int row_compact_launch(int dtype, const void* x, int B, long long N, int cap, int* idx, float* val, int* nnz,
                       const float* thr, const float* col_div, int* ties, const int* tie_quota, const float* col_thr,
                       int* seg_counts, cudaStream_t stream) {
  if (col_thr != nullptr && (thr != nullptr || ties != nullptr || tie_quota != nullptr)) return (int)cudaErrorInvalidValue;
  if (B <= 0) return 0;
  if (N > 2147483647LL) return (int)cudaErrorInvalidValue;
  const int blocks = B < 148 * 8 ? B : 148 * 8;
  if (dtype == 0)
    row_compact_kernel<float><<<blocks, RC_THREADS, 0, stream>>>(static_cast<const float*>(x), B, N, cap, idx, val, nnz, thr, col_div, ties,
                                                                 tie_quota, col_thr, seg_counts);
  else
    row_compact_kernel<__nv_bfloat16>
        <<<blocks, RC_THREADS, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), B, N, cap, idx, val, nnz, thr, col_div, ties,
                                            tie_quota, col_thr, seg_counts);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------------------
// JumpReLU threshold gradient of one crosscoder head from dense matrices: G[b, f] = d loss / d a[b, f] (reconstruction
// part, = d x_hat[b, :] . W_D[f, :]) and S[b, f] = summed pre-activation, both bf16 [B, F]; n[f] = decoder norm of the
// head, theta[f] = threshold. With x = S n:  d theta[f] += sum_b (G / n) * (-theta / w) * 1[|x - theta| < w / 2 and x > 0]
// (activation_functions.py:15-64 of the reference project: rectangle window of width w around the threshold).
// `add_per_hit` is added to G / n at every entry inside the window (a loss term whose derivative with respect to the
// JumpReLU output is the same constant at every entry, e.g. a tanh penalty at zero activation). Each thread owns eight
// consecutive columns and walks a chunk of rows; partial column sums go to fp32 atomics.
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
jumprelu_window_grad_kernel(const __nv_bfloat16* __restrict__ G, const __nv_bfloat16* __restrict__ S, int B, int F,
                            const float* __restrict__ n, const float* __restrict__ theta, float window, float add_per_hit,
                            int rows_per_block, float* __restrict__ dtheta) {
  const int c = (blockIdx.x * 256 + threadIdx.x) * 8;
  if (c >= F) return;
  const int r0 = blockIdx.y * rows_per_block, r1 = min(B, r0 + rows_per_block);
  float nn[8], th[8], acc[8], hits[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    nn[i] = n[c + i];
    th[i] = theta[c + i];
    acc[i] = hits[i] = 0.0f;
  }
  const float half_w = 0.5f * window;
  for (int r = r0; r < r1; ++r) {
    float g[8], s[8];
    load8<__nv_bfloat16>(G + (size_t)r * F + c, g);
    load8<__nv_bfloat16>(S + (size_t)r * F + c, s);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float x = s[i] * nn[i];
      if (x > 0.0f && fabsf(x - th[i]) < half_w) {
        acc[i] += g[i];
        hits[i] += 1.0f;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i)
    if (hits[i] != 0.0f) atomicAdd(dtheta + c + i, (acc[i] / nn[i] + add_per_hit * hits[i]) * (-th[i] / window));
}

int jumprelu_window_grad_launch(const __nv_bfloat16* G, const __nv_bfloat16* S, int B, int F, const float* n,
                                const float* theta, float window, float add_per_hit, float* dtheta, cudaStream_t stream) {
  if (F % 8 != 0 || B <= 0) return (int)cudaErrorInvalidValue;
  const int rows_per_block = 128;
  dim3 grid((F / 8 + 255) / 256, (B + rows_per_block - 1) / rows_per_block);
  jumprelu_window_grad_kernel<<<grid, 256, 0, stream>>>(G, S, B, F, n, theta, window, add_per_hit, rows_per_block, dtheta);
  return (int)cudaGetLastError();
}

int gather_rows_cast_launch(int in_dtype, int out_dtype, const void* src, const int* keep, const int* pos, long long n,
                            int d, void* out, long long out_rows, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (d % 8 != 0) return (int)cudaErrorInvalidValue;
  const int blocks = (int)(n < 148LL * 16 ? n : 148LL * 16);
  using bf = __nv_bfloat16;
  if (in_dtype == 0 && out_dtype == 0)
    gather_rows_cast_kernel<float, float><<<blocks, 256, 0, stream>>>((const float*)src, keep, pos, n, d, (float*)out, out_rows);
  else if (in_dtype == 0 && out_dtype == 1)
    gather_rows_cast_kernel<float, bf><<<blocks, 256, 0, stream>>>((const float*)src, keep, pos, n, d, (bf*)out, out_rows);
  else if (in_dtype == 1 && out_dtype == 0)
    gather_rows_cast_kernel<bf, float><<<blocks, 256, 0, stream>>>((const bf*)src, keep, pos, n, d, (float*)out, out_rows);
  else if (in_dtype == 1 && out_dtype == 1)
    gather_rows_cast_kernel<bf, bf><<<blocks, 256, 0, stream>>>((const bf*)src, keep, pos, n, d, (bf*)out, out_rows);
  else
    return (int)cudaErrorInvalidValue;
  return (int)cudaGetLastError();
}

}  // namespace lmsae
