// Rotary position embedding of the query and key projections of a low-rank sparse attention dictionary, both tensors
// in one launch (semantics of models/lorsa.py:666-712 in the reference project):
//
//   out[c] = x[c] * cos[pos, c] + turned(x)[c] * sin[pos, c]      for the first rd channels of every head,
//   out[c] = x[c]                                                 for the others,
//
// with turned(x)[2j] = -x[2j+1], turned(x)[2j+1] = x[2j] for adjacent pairs and turned(x)[j] = -x[j+rd/2],
// turned(x)[j+rd/2] = x[j] for the half-split layout. With sin_sign = -1 the same kernel is the inverse rotation,
// which is also the backward pass of the forward one (the map is orthogonal on every channel pair as long as both
// channels of a pair share their angle, which is how the tables are built).
//
// x is [tokens, heads, width] bf16 with tokens = batch x seq and pos = token % seq; the tables are fp32 [>= seq, rd].
// One thread owns eight consecutive channels of one (token, head) (one 16-byte load and store per tensor) and, in the
// half-split layout, fetches the partner block rd/2 channels away (rd/2 is a multiple of 8, checked by the caller).
// Arithmetic in fp32, one rounding to bf16 on the way out.
#include "common.cuh"
#include "kernels.h"

namespace lmsae {

namespace {

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 u;
  u.x = pack_bf16x2(v[0], v[1]);
  u.y = pack_bf16x2(v[2], v[3]);
  u.z = pack_bf16x2(v[4], v[5]);
  u.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

__device__ __forceinline__ void load8f(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

template <bool ADJACENT>
__global__ void __launch_bounds__(256)
rotary_pair_kernel(const __nv_bfloat16* __restrict__ xa, const __nv_bfloat16* __restrict__ xb, __nv_bfloat16* __restrict__ oa,
                   __nv_bfloat16* __restrict__ ob, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                   long long n_blocks, int seq, int heads, int width, int rd, float sin_sign) {
  const int per_head = width / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < 2 * n_blocks; i += (long long)gridDim.x * blockDim.x) {
    const bool second = i >= n_blocks;
    const long long j = second ? i - n_blocks : i;
    const __nv_bfloat16* x = second ? xb : xa;
    __nv_bfloat16* o = second ? ob : oa;
    const int c0 = (int)(j % per_head) * 8;           // first channel of this thread's block
    const long long th = j / per_head;                // token x head
    const int pos = (int)((th / heads) % seq);
    const long long base = th * width;
    float v[8], r[8];
    load8(x + base + c0, v);
    if (c0 >= rd) {  // channels past the rotated ones pass through
      store8(o + base + c0, v);
      continue;
    }
    float cs[8], sn[8];
    load8f(cos_t + (long long)pos * rd + c0, cs);
    load8f(sin_t + (long long)pos * rd + c0, sn);
    if constexpr (ADJACENT) {
#pragma unroll
      for (int p = 0; p < 8; p += 2) {
        r[p] = v[p] * cs[p] - sin_sign * v[p + 1] * sn[p];
        r[p + 1] = v[p + 1] * cs[p + 1] + sin_sign * v[p] * sn[p + 1];
      }
    } else {
      const int half = rd / 2;
      const bool low = c0 < half;
      float w[8];
      load8(x + base + (low ? c0 + half : c0 - half), w);
      const float sgn = low ? -sin_sign : sin_sign;
#pragma unroll
      for (int p = 0; p < 8; ++p) r[p] = v[p] * cs[p] + sgn * w[p] * sn[p];
    }
    store8(o + base + c0, r);
  }
}

}  // namespace

int rotary_pair_launch(const __nv_bfloat16* xa, const __nv_bfloat16* xb, __nv_bfloat16* oa, __nv_bfloat16* ob, const float* cos_t,
                       const float* sin_t, long long tokens, int seq, int heads, int width, int rd, int adjacent, float sin_sign,
                       cudaStream_t stream) {
  const long long n_blocks = tokens * heads * (width / 8);
  if (n_blocks == 0) return (int)cudaSuccess;
  const int threads = 256;
  const long long want = (2 * n_blocks + threads - 1) / threads;
  const int grid = (int)(want < 148LL * 16 ? want : 148LL * 16);
  if (adjacent)
    rotary_pair_kernel<true><<<grid, threads, 0, stream>>>(xa, xb, oa, ob, cos_t, sin_t, n_blocks, seq, heads, width, rd, sin_sign);
  else
    rotary_pair_kernel<false><<<grid, threads, 0, stream>>>(xa, xb, oa, ob, cos_t, sin_t, n_blocks, seq, heads, width, rd, sin_sign);
  return (int)cudaGetLastError();
}

}  // namespace lmsae
