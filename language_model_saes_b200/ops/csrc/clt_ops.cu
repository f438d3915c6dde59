// Cross-layer transcoder decoder fan-out on sparse codes (sm_100a, SIMT gather kernels: HBM/L2-bound).
//
// A cross-layer transcoder decodes the features of source layer s into every target layer t >= s:
//   y[t, b, :] = b_D[t] + sum_{s <= t} sum_f a[b, s, f] * W_D[t][s, f, :]
// (models/clt.py:629-709 of the reference project, which runs one dense or CSR product per (s, t) pair and one
// all-reduce per target layer). Here the codes of a token are one padded list of (c = s * F + f, value) pairs, and
//
//   clt_decode_kernel   one CTA per (token, target layer) gathers the rows W_D[t][s, f, :] of that token's codes with
//                       s <= t and accumulates them in registers: every target layer in one launch, no dense product;
//   clt_dact_kernel     d a[b, j] = sum_{t >= s} d y[t, b, :] . W_D[t][s, f, :]   (one CTA per token, a warp per code);
//   clt_wgrad_kernel    d W_D[t][s, f, :] = sum_{b in rows(c)} a[b, c] * d y[t, b, :] for every t >= s from the
//                       by-feature lists of a counting sort: one CTA per active (s, f), no atomics; rows of features
//                       that did not fire are not touched (the caller hands in zero-filled gradients).
//
// W_D[t] is its own allocation of shape [t + 1, F, d] (bf16); the kernels take the table of base pointers by value.
#include "common.cuh"
#include "kernels.h"

namespace lmsae {

namespace {

__device__ __forceinline__ void bf16x8_unpack(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

constexpr int CLT_MAX_VEC = 2;  // 16-byte chunks of a row owned by one thread

}  // namespace

// ---------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(512)
clt_decode_kernel(const CltTable tab, const int* __restrict__ idx, const float* __restrict__ val, int B, int K, int L,
                  int F, int d, const float* __restrict__ bias, float* __restrict__ out_f32,
                  __nv_bfloat16* __restrict__ out_bf16) {
  extern __shared__ uint8_t smem_raw[];
  int* s_idx = reinterpret_cast<int*>(smem_raw);            // [K]
  float* s_val = reinterpret_cast<float*>(smem_raw) + K;    // [K]
  const int nvec = d / 8;
  const long long items = (long long)B * L;
  for (long long w = blockIdx.x; w < items; w += gridDim.x) {
    const int row = (int)(w / L);
    const int t = L - 1 - (int)(w % L);  // deepest target (longest list) first
    __syncthreads();
    for (int j = threadIdx.x; j < K; j += blockDim.x) {
      s_idx[j] = idx[(size_t)row * K + j];
      s_val[j] = val[(size_t)row * K + j];
    }
    __syncthreads();
    const __nv_bfloat16* Wt = tab.W[t];
    const long long limit = (long long)(t + 1) * F;  // codes c < limit come from source layers s <= t
    float acc[CLT_MAX_VEC][8];
#pragma unroll
    for (int u = 0; u < CLT_MAX_VEC; ++u)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[u][i] = 0.0f;
    for (int j = 0; j < K; ++j) {
      const int c = s_idx[j];
      if (c < 0 || c >= limit) continue;
      const float a = s_val[j];
      const uint4* wrow = reinterpret_cast<const uint4*>(Wt + (size_t)c * d);
#pragma unroll
      for (int u = 0; u < CLT_MAX_VEC; ++u) {
        const int v = threadIdx.x + u * blockDim.x;
        if (v < nvec) {
          float wv[8];
          bf16x8_unpack(__ldg(wrow + v), wv);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[u][i] = fmaf(a, wv[i], acc[u][i]);
        }
      }
    }
    const size_t obase = ((size_t)t * B + row) * d;
#pragma unroll
    for (int u = 0; u < CLT_MAX_VEC; ++u) {
      const int v = threadIdx.x + u * blockDim.x;
      if (v < nvec) {
        const int c0 = v * 8;
        if (bias != nullptr) {
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[u][i] += bias[(size_t)t * d + c0 + i];
        }
        if (out_f32 != nullptr) {
          float4* o = reinterpret_cast<float4*>(out_f32 + obase + c0);
          o[0] = make_float4(acc[u][0], acc[u][1], acc[u][2], acc[u][3]);
          o[1] = make_float4(acc[u][4], acc[u][5], acc[u][6], acc[u][7]);
        }
        if (out_bf16 != nullptr) {
          uint4 o;
          o.x = pack_bf16x2(acc[u][0], acc[u][1]);
          o.y = pack_bf16x2(acc[u][2], acc[u][3]);
          o.z = pack_bf16x2(acc[u][4], acc[u][5]);
          o.w = pack_bf16x2(acc[u][6], acc[u][7]);
          *reinterpret_cast<uint4*>(out_bf16 + obase + c0) = o;
        }
      }
    }
  }
}

static int clt_threads_for(int d) {
  int t = ((d / 8 + 31) / 32) * 32;
  if (t > 512) t = ((d / 16 + 31) / 32) * 32;  // two chunks per thread
  return t < 32 ? 32 : t;
}

int clt_decode_launch(const CltTable& tab, const int* idx, const float* val, int B, int K, int L, int F, int d,
                      const float* bias, float* out_f32, __nv_bfloat16* out_bf16, cudaStream_t stream) {
  if (d % 8 != 0 || d > 512 * CLT_MAX_VEC * 8 || L < 1 || L > kMaxCltLayers) return (int)cudaErrorInvalidValue;
  if ((long long)L * F > 2147483647LL) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)K * 8;
  if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
  const int threads = clt_threads_for(d);
  if (threads > 512) return (int)cudaErrorInvalidValue;
  long long items = (long long)B * L;
  if (items <= 0) return 0;
  const int blocks = (int)(items < 148LL * 32 ? items : 148LL * 32);
  clt_decode_kernel<<<blocks, threads, smem, stream>>>(tab, idx, val, B, K, L, F, d, bias, out_f32, out_bf16);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// gradient of the codes
// ---------------------------------------------------------------------------------------------
constexpr int CLT_DACT_THREADS = 256;

__global__ void __launch_bounds__(CLT_DACT_THREADS)
clt_dact_kernel(const CltTable tab, const int* __restrict__ idx, int B, int K, int L, int F, int d,
                const __nv_bfloat16* __restrict__ dy, float* __restrict__ dval) {
  extern __shared__ uint8_t smem_raw[];
  float* s_dy = reinterpret_cast<float*>(smem_raw);          // [d]
  float* s_acc = s_dy + d;                                   // [K]
  int* s_idx = reinterpret_cast<int*>(s_acc + K);            // [K]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = d / 8;
  for (int row = blockIdx.x; row < B; row += gridDim.x) {
    __syncthreads();
    for (int j = threadIdx.x; j < K; j += CLT_DACT_THREADS) {
      s_idx[j] = idx[(size_t)row * K + j];
      s_acc[j] = 0.0f;
    }
    __syncthreads();
    for (int t = 0; t < L; ++t) {
      const long long limit = (long long)(t + 1) * F;
      __syncthreads();
      for (int v = threadIdx.x; v < nvec; v += CLT_DACT_THREADS) {
        float f[8];
        bf16x8_unpack(__ldg(reinterpret_cast<const uint4*>(dy + ((size_t)t * B + row) * d) + v), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) s_dy[v * 8 + i] = f[i];
      }
      __syncthreads();
      const __nv_bfloat16* Wt = tab.W[t];
      // code j always belongs to warp j % 8, so its accumulator has one writer
      for (int j = warp; j < K; j += CLT_DACT_THREADS / 32) {
        const int c = s_idx[j];
        if (c < 0 || c >= limit) continue;
        const uint4* wrow = reinterpret_cast<const uint4*>(Wt + (size_t)c * d);
        float dot = 0.0f;
        for (int v = lane; v < nvec; v += 32) {
          float wv[8];
          bf16x8_unpack(__ldg(wrow + v), wv);
          const float* g = s_dy + v * 8;
#pragma unroll
          for (int i = 0; i < 8; ++i) dot = fmaf(wv[i], g[i], dot);
        }
        dot = warp_sum(dot);
        if (lane == 0) s_acc[j] += dot;
      }
    }
    __syncthreads();
    for (int j = threadIdx.x; j < K; j += CLT_DACT_THREADS) dval[(size_t)row * K + j] = s_acc[j];
  }
}

int clt_dact_launch(const CltTable& tab, const int* idx, int B, int K, int L, int F, int d, const __nv_bfloat16* dy,
                    float* dval, cudaStream_t stream) {
  if (d % 8 != 0 || L < 1 || L > kMaxCltLayers) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)d * 4 + (size_t)K * 8;
  if (smem > 160 * 1024) return (int)cudaErrorInvalidValue;
  cudaError_t e = cudaFuncSetAttribute(clt_dact_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
  if (e != cudaSuccess) return (int)e;
  if (B <= 0) return 0;
  const int blocks = B < 148 * 8 ? B : 148 * 8;
  clt_dact_kernel<<<blocks, CLT_DACT_THREADS, smem, stream>>>(tab, idx, B, K, L, F, d, dy, dval);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// gradient of the decoders
// ---------------------------------------------------------------------------------------------
constexpr int CLT_WG_THREADS = 256;

__global__ void __launch_bounds__(CLT_WG_THREADS)
clt_wgrad_kernel(const CltGradTable tab, const int* __restrict__ offsets, const int* __restrict__ entries,
                 const float* __restrict__ act, int B, int K, int L, int F, int d,
                 const __nv_bfloat16* __restrict__ dy) {
  const long long n_codes = (long long)L * F;
  for (long long c = blockIdx.x; c < n_codes; c += gridDim.x) {
    const int e0 = offsets[c], e1 = offsets[c + 1];
    if (e0 == e1) continue;
    const int s = (int)(c / F);
    for (int t = s; t < L; ++t) {
      float* grow = tab.G[t] + (size_t)c * d;
      const __nv_bfloat16* dyt = dy + (size_t)t * B * d;
      for (int c0 = threadIdx.x * 4; c0 < d; c0 += CLT_WG_THREADS * 4) {
        float g[4] = {0.f, 0.f, 0.f, 0.f};
        for (int e = e0; e < e1; ++e) {
          const int ent = entries[e];
          const int row = ent / K;
          const float a = act[ent];
          const uint2 u = __ldg(reinterpret_cast<const uint2*>(dyt + (size_t)row * d + c0));
          const float2 d01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
          const float2 d23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
          g[0] = fmaf(a, d01.x, g[0]); g[1] = fmaf(a, d01.y, g[1]);
          g[2] = fmaf(a, d23.x, g[2]); g[3] = fmaf(a, d23.y, g[3]);
        }
        *reinterpret_cast<float4*>(grow + c0) = make_float4(g[0], g[1], g[2], g[3]);
      }
    }
  }
}

int clt_wgrad_launch(const CltGradTable& tab, const int* offsets, const int* entries, const float* act, int B, int K,
                     int L, int F, int d, const __nv_bfloat16* dy, cudaStream_t stream) {
  if (d % 4 != 0 || L < 1 || L > kMaxCltLayers) return (int)cudaErrorInvalidValue;
  const long long n_codes = (long long)L * F;
  if (n_codes <= 0 || n_codes > 2147483647LL) return (int)cudaErrorInvalidValue;
  const int blocks = (int)(n_codes < 148LL * 16 ? n_codes : 148LL * 16);
  clt_wgrad_kernel<<<blocks, CLT_WG_THREADS, 0, stream>>>(tab, offsets, entries, act, B, K, L, F, d, dy);
  return (int)cudaGetLastError();
}

}  // namespace lmsae
