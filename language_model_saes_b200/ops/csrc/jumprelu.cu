// JumpReLU with its straight-through threshold gradient as two streaming kernels
// (semantics of activation_functions.py:15-64 in the reference project):
//
//   forward   y  = x * 1[x > theta],           theta = exp(log_theta)
//   backward  dx = dy * 1[x > theta]
//             d log_theta[p] = sum_rows dy * (-theta^2 / w) * 1[|x - theta| < w/2 and x > 0]
//
// x is viewed as [rows, P] with P = number of thresholds (the trailing dimensions of x). Both kernels are pure
// streaming: the backward reads x and dy once and writes dx once; hits of the rectangle window are rare (a
// fraction ~ w * density(theta) of the elements), so they go straight to fp32 atomics on a [P] buffer instead
// of a second reduction pass. exp() is evaluated per element from the L1-resident log_theta row.
#include "common.cuh"
#include "kernels.h"

namespace lmsae {

template <typename T> struct Vec4;
template <> struct Vec4<float> {
  using type = float4;
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
  static __device__ __forceinline__ float round(float x) { return x; }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4]) {
    uint2 u;
    u.x = pack_bf16x2(v[0], v[1]);
    u.y = pack_bf16x2(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = u;
  }
  // thresholds are compared in the tensor's own precision, as an eager exp() in bf16 would produce them
  static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16(x)); }
};

template <typename T, bool BWD>
__global__ void __launch_bounds__(256)
jumprelu_kernel(const T* __restrict__ x, const T* __restrict__ log_theta, const T* __restrict__ dy, T* __restrict__ out,
                float* __restrict__ dlog, long long n_vec, int P, float window) {
  const float half_w = Vec4<T>::round(0.5f * window);
  const float inv_w = 1.0f / window;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (long long)gridDim.x * blockDim.x) {
    const long long e = i * 4;
    const int p = (int)(e % P);  // P % 4 == 0: the four elements share a row
    float xv[4], lt[4], o[4], g[4];
    Vec4<T>::load(x + e, xv);
    Vec4<T>::load(log_theta + p, lt);
    if constexpr (BWD) Vec4<T>::load(dy + e, g);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float theta = Vec4<T>::round(expf(lt[j]));
      const bool on = xv[j] > theta;
      if constexpr (BWD) {
        o[j] = on ? g[j] : 0.0f;
        if (fabsf(Vec4<T>::round(xv[j] - theta)) < half_w && xv[j] > 0.0f && g[j] != 0.0f) {
          atomicAdd(dlog + p + j, -g[j] * theta * theta * inv_w);
        }
      } else {
        o[j] = on ? xv[j] : 0.0f;
      }
    }
    Vec4<T>::store(out + e, o);
  }
}

template <typename T>
static int launch(const void* x, const void* log_theta, const void* dy, void* out, float* dlog, long long n, int P,
                  float window, bool bwd, cudaStream_t stream) {
  if (P % 4 != 0 || n % P != 0) return (int)cudaErrorInvalidValue;
  const long long n_vec = n / 4;
  if (n_vec == 0) return 0;
  long long blocks = (n_vec + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (bwd) {
    jumprelu_kernel<T, true><<<(int)blocks, 256, 0, stream>>>((const T*)x, (const T*)log_theta, (const T*)dy, (T*)out, dlog, n_vec, P, window);
  } else {
    jumprelu_kernel<T, false><<<(int)blocks, 256, 0, stream>>>((const T*)x, (const T*)log_theta, nullptr, (T*)out, nullptr, n_vec, P, window);
  }
  return (int)cudaGetLastError();
}

// dtype: 0 = fp32, 1 = bf16. `dlog` (fp32 [P], zeroed by the caller) is used by the backward only.
int jumprelu_launch(int dtype, const void* x, const void* log_theta, const void* dy, void* out, float* dlog, long long n,
                    int P, float window, int backward, cudaStream_t stream) {
  if (dtype == 0) return launch<float>(x, log_theta, dy, out, dlog, n, P, window, backward != 0, stream);
  if (dtype == 1) return launch<__nv_bfloat16>(x, log_theta, dy, out, dlog, n, P, window, backward != 0, stream);
  return (int)cudaErrorInvalidValue;
}

}  // namespace lmsae
