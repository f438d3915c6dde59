// Sparse decoder forward / backward and the fused gradient + Adam update (sm_100a, plain SIMT kernels:
// these ops are gather- and HBM-bound, not tensor-core work).
//
// Layouts: W_D and W_E^T are both stored feature-major [F, d] (row f contiguous), with an fp32 master
// copy and a bf16 shadow used by the forward kernels. Sparse codes are [B, k] (idx int32, -1 = empty).
//
//  sparse_decode_kernel   x_hat[b,:] = sum_j val[b,j] * W[idx[b,j],:] (+ bias); optional fused MSE loss,
//                         d(x_hat) and d(val) (decoder math of models/sae.py:347-377, loss of
//                         models/sparse_dictionary.py:880-886, gather-GEMM of kernels/kernels.py:383-436
//                         in the reference project)
//  sparse_dact_kernel     d val[b,j] = d x_hat[b,:] . W[idx[b,j],:]           (kernels/kernels.py:327-379)
//  csc_* kernels          group the (row, slot) pairs by feature (counting sort)
//  sparse_grad_adam_kernel  for every feature row f: rebuild dW_D[f,:] = sum act * d x_hat[b,:] and
//                         dW_E^T[f,:] = sum d h * x[b,:] in registers from the feature's entry list and
//                         apply Adam to both rows in the same pass -- the dense gradient is never written
//                         (replaces kernels/kernels.py:137-225 + torch.optim.Adam in the reference).
#include "comm_common.cuh"

namespace lmsae {

LMSAE_DEFINE_BOUNDS_FETCH(bounds_fetch_sparse_ops)

// ---------------------------------------------------------------------------------------------
// decode (+ loss, + dact)
// ---------------------------------------------------------------------------------------------
constexpr int DEC_THREADS = 512;
constexpr int DEC_MAX_VEC = 2;  // each thread owns up to 2 chunks of 8 columns -> d <= 8192


__device__ __forceinline__ void bf16x8_to_float(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__global__ void __launch_bounds__(DEC_THREADS)
sparse_decode_kernel(const DecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  int* s_idx = reinterpret_cast<int*>(smem_raw);                 // [k]
  float* s_val = reinterpret_cast<float*>(smem_raw) + p.k;       // [k]
  float* s_dx = reinterpret_cast<float*>(smem_raw) + 2 * p.k;    // [d] (dval only)
  __shared__ float s_red[DEC_THREADS / 32];
  const int nvec = p.d / 8;  // d % 8 == 0
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  for (int row = blockIdx.x; row < p.B; row += gridDim.x) {
    __syncthreads();
    for (int j = threadIdx.x; j < p.k; j += DEC_THREADS) {
      s_idx[j] = p.idx[(size_t)row * p.k + j];
      s_val[j] = p.val[(size_t)row * p.k + j];
    }
    __syncthreads();

    float acc[DEC_MAX_VEC][8];
#pragma unroll
    for (int u = 0; u < DEC_MAX_VEC; ++u)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[u][i] = 0.0f;

    for (int j = 0; j < p.k; ++j) {
      const int f = s_idx[j];
      if (f < 0) continue;
      const float a = s_val[j];
      const uint4* wrow = reinterpret_cast<const uint4*>(p.W + (size_t)LMSAE_IDX(f, p.F) * p.d);
#pragma unroll
      for (int u = 0; u < DEC_MAX_VEC; ++u) {
        const int v = threadIdx.x + u * DEC_THREADS;
        if (v < nvec) {
          float w[8];
          bf16x8_to_float(__ldg(wrow + v), w);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[u][i] = fmaf(a, w[i], acc[u][i]);
        }
      }
    }

    float local_sq = 0.0f;
    const float rw = (p.row_weight != nullptr) ? p.row_weight[row] : 1.0f;
#pragma unroll
    for (int u = 0; u < DEC_MAX_VEC; ++u) {
      const int v = threadIdx.x + u * DEC_THREADS;
      if (v < nvec) {
        const int c = v * 8;
        if (p.bias != nullptr) {
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[u][i] += p.bias[c + i];
        }
        if (p.xhat_f32 != nullptr) {
          float4* o = reinterpret_cast<float4*>(p.xhat_f32 + (size_t)row * p.d + c);
          o[0] = make_float4(acc[u][0], acc[u][1], acc[u][2], acc[u][3]);
          o[1] = make_float4(acc[u][4], acc[u][5], acc[u][6], acc[u][7]);
        }
        if (p.xhat_bf16 != nullptr) {
          uint4 o;
          o.x = pack_bf16x2(acc[u][0], acc[u][1]);
          o.y = pack_bf16x2(acc[u][2], acc[u][3]);
          o.z = pack_bf16x2(acc[u][4], acc[u][5]);
          o.w = pack_bf16x2(acc[u][6], acc[u][7]);
          *reinterpret_cast<uint4*>(p.xhat_bf16 + (size_t)row * p.d + c) = o;
        }
        if (p.label != nullptr) {
          float y[8];
          bf16x8_to_float(__ldg(reinterpret_cast<const uint4*>(p.label + (size_t)row * p.d) + v), y);
          float e[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            e[i] = acc[u][i] - y[i];
            local_sq = fmaf(e[i], e[i], local_sq);
            e[i] *= p.grad_scale * rw;
          }
          uint4 o;
          o.x = pack_bf16x2(e[0], e[1]);
          o.y = pack_bf16x2(e[2], e[3]);
          o.z = pack_bf16x2(e[4], e[5]);
          o.w = pack_bf16x2(e[6], e[7]);
          *reinterpret_cast<uint4*>(p.dxhat + (size_t)row * p.d + c) = o;
          if (p.dval != nullptr) {
            // keep the bf16-rounded gradient so that every consumer sees the same d x_hat
            float er[8];
            bf16x8_to_float(o, er);
#pragma unroll
            for (int i = 0; i < 8; ++i) s_dx[c + i] = er[i];
          }
        }
      }
    }
    if (p.label != nullptr) {
      local_sq = warp_sum(local_sq);
      if (lane == 0) s_red[warp] = local_sq;
      __syncthreads();
      if (warp == 0) {
        float t = (lane < DEC_THREADS / 32) ? s_red[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) {
          if (p.row_loss != nullptr) p.row_loss[row] = t;
          atomicAdd(p.loss_sum, t * rw);
        }
      }
      if (p.dval != nullptr) {
        // second pass over the same (L2-resident) decoder rows: d val[j] = d x_hat . W[idx[j], :]
        __syncthreads();
        for (int j = warp; j < p.k; j += DEC_THREADS / 32) {
          const int f = s_idx[j];
          float dot = 0.0f;
          if (f >= 0) {
            const uint4* wrow = reinterpret_cast<const uint4*>(p.W + (size_t)LMSAE_IDX(f, p.F) * p.d);
            for (int v = lane; v < nvec; v += 32) {
              float w[8];
              bf16x8_to_float(__ldg(wrow + v), w);
              const float* dx = s_dx + v * 8;
#pragma unroll
              for (int i = 0; i < 8; ++i) dot = fmaf(w[i], dx[i], dot);
            }
          }
          dot = warp_sum(dot);
          if (lane == 0) p.dval[(size_t)row * p.k + j] = dot;
        }
      }
    }
  }
}

int sparse_decode_launch(const DecodeParams& p, cudaStream_t stream) {
  if (p.d % 8 != 0 || p.d > DEC_THREADS * DEC_MAX_VEC * 8) return (int)cudaErrorInvalidValue;
  size_t smem = (size_t)p.k * 8 + (p.dval != nullptr ? (size_t)p.d * 4 : 0);
  cudaError_t e = cudaFuncSetAttribute(sparse_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  if (e != cudaSuccess) return (int)e;
  if (smem > 100 * 1024) return (int)cudaErrorInvalidValue;
  int blocks = p.B < 148 * 16 ? p.B : 148 * 16;
  sparse_decode_kernel<<<blocks, DEC_THREADS, smem, stream>>>(p);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// d val[b,j] = d x_hat[b,:] . W[idx[b,j],:]    (stand-alone, for the feature-sharded path where
// d x_hat only exists after the cross-shard reduction)
// ---------------------------------------------------------------------------------------------
constexpr int DACT_THREADS = 256;

// `wait_pt.world > 0`: d x_hat is the gradient buffer of the fused feature-sharded step, filled by the row owners'
// peer stores; the kernel then waits (bounded) for every owner's flag of `epoch` itself instead of relying on a
// separate wait launch before it.
__global__ void __launch_bounds__(DACT_THREADS)
sparse_dact_kernel(const int* __restrict__ idx, int B, int k, int d, int F, const __nv_bfloat16* __restrict__ W,
                   const __nv_bfloat16* dxhat /* may be peer-written: no read-only path */, float* __restrict__ dval, const PeerTable wait_pt,
                   uint32_t epoch, int* status) {
  extern __shared__ float s_dx[];  // [d]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = d / 8;
  if (wait_pt.world > 0 && !wait_all_sources(wait_pt, kPhaseDxhat, epoch, status)) {
    // the gradient rows never arrived: leave zeros so that nothing downstream consumes stale data
    for (long long i = blockIdx.x * (long long)DACT_THREADS + threadIdx.x; i < (long long)B * k;
         i += (long long)gridDim.x * DACT_THREADS)
      dval[i] = 0.0f;
    return;
  }
  for (int row = blockIdx.x; row < B; row += gridDim.x) {
    __syncthreads();
    for (int v = threadIdx.x; v < nvec; v += DACT_THREADS) {
      float f[8];
      bf16x8_to_float(*(reinterpret_cast<const uint4*>(dxhat + (size_t)row * d) + v), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) s_dx[v * 8 + i] = f[i];
    }
    __syncthreads();
    for (int j = warp; j < k; j += DACT_THREADS / 32) {
      const int f = idx[(size_t)row * k + j];
      float dot = 0.0f;
      if (f >= 0) {
        const uint4* wrow = reinterpret_cast<const uint4*>(W + (size_t)LMSAE_IDX(f, F) * d);
#pragma unroll 4
        for (int v = lane; v < nvec; v += 32) {
          float w[8];
          bf16x8_to_float(__ldg(wrow + v), w);
          const float* dx = s_dx + v * 8;
#pragma unroll
          for (int i = 0; i < 8; ++i) dot = fmaf(w[i], dx[i], dot);
        }
      }
      dot = warp_sum(dot);
      if (lane == 0) dval[(size_t)row * k + j] = dot;
    }
  }
}

int sparse_dact_launch(const int* idx, int B, int k, int d, int F, const __nv_bfloat16* W, const __nv_bfloat16* dxhat,
                       float* dval, const PeerTable* wait, uint32_t epoch, int* status, cudaStream_t stream) {
  if (d % 8 != 0 || (size_t)d * 4 > 160 * 1024) return (int)cudaErrorInvalidValue;
  cudaError_t e = cudaFuncSetAttribute(sparse_dact_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
  if (e != cudaSuccess) return (int)e;
  int blocks = B < 148 * 8 ? B : 148 * 8;
  PeerTable pt{};
  if (wait != nullptr) pt = *wait;
  sparse_dact_kernel<<<blocks, DACT_THREADS, (size_t)d * 4, stream>>>(idx, B, k, d, F, W, dxhat, dval, pt, epoch, status);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// MSE loss + gradient on dense rows (feature-sharded path: x_hat arrives from the cross-shard reduce)
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
mse_loss_grad_kernel(const float* __restrict__ xhat, const __nv_bfloat16* __restrict__ label,
                     const float* __restrict__ bias, const float* __restrict__ row_weight, int rows, int d,
                     float grad_scale, __nv_bfloat16* __restrict__ dxhat, float* __restrict__ loss_sum,
                     float* __restrict__ row_loss) {
  __shared__ float s_red[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rw = row_weight != nullptr ? row_weight[row] : 1.0f;
    float sq = 0.0f;
    for (int c = threadIdx.x; c < d; c += 256) {
      float xh = xhat[(size_t)row * d + c];
      if (bias != nullptr) xh += bias[c];
      const float e = xh - __bfloat162float(label[(size_t)row * d + c]);
      sq = fmaf(e, e, sq);
      dxhat[(size_t)row * d + c] = __float2bfloat16(e * grad_scale * rw);
    }
    sq = warp_sum(sq);
    __syncthreads();
    if (lane == 0) s_red[warp] = sq;
    __syncthreads();
    if (warp == 0) {
      float t = lane < 8 ? s_red[lane] : 0.0f;
      t = warp_sum(t);
      if (lane == 0) {
        if (row_loss != nullptr) row_loss[row] = t;
        atomicAdd(loss_sum, t * rw);
      }
    }
  }
}

int mse_loss_grad_launch(const float* xhat, const __nv_bfloat16* label, const float* bias, const float* row_weight,
                         int rows, int d, float grad_scale, __nv_bfloat16* dxhat, float* loss_sum, float* row_loss,
                         cudaStream_t stream) {
  int blocks = rows < 148 * 8 ? rows : 148 * 8;
  mse_loss_grad_kernel<<<blocks, 256, 0, stream>>>(xhat, label, bias, row_weight, rows, d, grad_scale, dxhat,
                                                   loss_sum, row_loss);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Aux-K: losses and gradients of   l = |e|^2 + alpha |e - e_aux|^2   per row, with e = label - x_hat (x_hat from
// the main codes) and e_aux the reconstruction of the residual from dead features
// (models/sparse_dictionary.py:941-991 of the reference project; e is NOT detached there, so the auxiliary term
// also pulls on x_hat). Outputs, per row scaled by grad_scale * row_weight:
//   g_main = d l / d x_hat = (x_hat - label) - alpha * r,      g_aux = d l / d e_aux = -alpha * r,   r = e - e_aux
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
auxk_loss_grad_kernel(const float* __restrict__ xhat, const float* __restrict__ aux_rec,
                      const __nv_bfloat16* __restrict__ label, const float* __restrict__ bias,
                      const float* __restrict__ row_weight, int rows, int d, float grad_scale, float alpha_host,
                      const float* __restrict__ alpha_factor, __nv_bfloat16* __restrict__ g_main,
                      __nv_bfloat16* __restrict__ g_aux, float* __restrict__ loss_sum, float* __restrict__ aux_sum) {
  __shared__ float s_red[2][8];
  // alpha_factor (one device float, optional): 0 switches the auxiliary term off without the host knowing, e.g. in a step
  // that has no dead feature
  const float alpha = alpha_factor != nullptr ? alpha_host * *alpha_factor : alpha_host;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rw = row_weight != nullptr ? row_weight[row] : 1.0f;
    const float sc = grad_scale * rw;
    float sq = 0.0f, sq_aux = 0.0f;
    for (int c = threadIdx.x; c < d; c += 256) {
      const size_t o = (size_t)row * d + c;
      float xh = xhat[o];
      if (bias != nullptr) xh += bias[c];
      const float e = __bfloat162float(label[o]) - xh;
      const float r = e - aux_rec[o];
      sq = fmaf(e, e, sq);
      sq_aux = fmaf(r, r, sq_aux);
      g_main[o] = __float2bfloat16(-(e + alpha * r) * sc);
      g_aux[o] = __float2bfloat16(-alpha * r * sc);
    }
    sq = warp_sum(sq);
    sq_aux = warp_sum(sq_aux);
    __syncthreads();
    if (lane == 0) { s_red[0][warp] = sq; s_red[1][warp] = sq_aux; }
    __syncthreads();
    if (warp == 0) {
      float t = lane < 8 ? s_red[0][lane] : 0.0f, u = lane < 8 ? s_red[1][lane] : 0.0f;
      t = warp_sum(t);
      u = warp_sum(u);
      if (lane == 0) {
        atomicAdd(loss_sum, t * rw);
        atomicAdd(aux_sum, alpha * u * rw);
      }
    }
  }
}

int auxk_loss_grad_launch(const float* xhat, const float* aux_rec, const __nv_bfloat16* label, const float* bias,
                          const float* row_weight, int rows, int d, float grad_scale, float alpha,
                          const float* alpha_factor, __nv_bfloat16* g_main, __nv_bfloat16* g_aux, float* loss_sum,
                          float* aux_sum, cudaStream_t stream) {
  int blocks = rows < 148 * 8 ? rows : 148 * 8;
  if (blocks <= 0) return 0;
  auxk_loss_grad_kernel<<<blocks, 256, 0, stream>>>(xhat, aux_rec, label, bias, row_weight, rows, d, grad_scale, alpha,
                                                    alpha_factor, g_main, g_aux, loss_sum, aux_sum);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// group (row, slot) pairs by feature: counts -> offsets (exclusive scan) -> entries
// ---------------------------------------------------------------------------------------------
__global__ void csc_count_kernel(const int* __restrict__ idx, long long n, int F, int* __restrict__ counts) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int f = idx[i];
    if (f >= 0 && f < F) atomicAdd(&counts[f], 1);
  }
}

// Exclusive scan of counts[F] in three small launches: per-block scan of 4096 elements (coalesced int4
// loads) + block totals, scan of the totals by one block, then add-back while writing offsets and cursors.
constexpr int SCAN_THREADS = 1024;
constexpr int SCAN_ELEMS = SCAN_THREADS * 4;

__device__ __forceinline__ int block_exclusive_scan_1024(int v, int* s_warp, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) s_warp[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = s_warp[lane];
    int winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += t;
    }
    s_warp[lane] = winc - w;  // exclusive prefix of the warp totals
    if (lane == 31) s_warp[32] = winc;
  }
  __syncthreads();
  total = s_warp[32];
  return s_warp[warp] + inc - v;
}

__global__ void __launch_bounds__(SCAN_THREADS)
csc_scan_local_kernel(const int* __restrict__ counts, int F, int* __restrict__ offsets, int* __restrict__ block_sums) {
  __shared__ int s_warp[33];
  const int base = blockIdx.x * SCAN_ELEMS + threadIdx.x * 4;
  int c[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) c[i] = (base + i < F) ? counts[base + i] : 0;
  const int mine = c[0] + c[1] + c[2] + c[3];
  int total;
  int run = block_exclusive_scan_1024(mine, s_warp, total);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (base + i < F) offsets[base + i] = run;
    run += c[i];
  }
  if (threadIdx.x == 0) block_sums[blockIdx.x] = total;
}

__global__ void __launch_bounds__(SCAN_THREADS)
csc_scan_sums_kernel(int* __restrict__ block_sums, int nblocks, int* __restrict__ offsets, int F) {
  __shared__ int s_warp[33];
  __shared__ int s_carry;
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();
  for (int b0 = 0; b0 < nblocks; b0 += SCAN_THREADS) {
    const int i = b0 + threadIdx.x;
    const int v = i < nblocks ? block_sums[i] : 0;
    int total;
    const int ex = block_exclusive_scan_1024(v, s_warp, total);
    const int carry = s_carry;
    if (i < nblocks) block_sums[i] = carry + ex;
    __syncthreads();
    if (threadIdx.x == 0) s_carry = carry + total;
    __syncthreads();
  }
  if (threadIdx.x == 0) offsets[F] = s_carry;
}

__global__ void __launch_bounds__(SCAN_THREADS)
csc_scan_add_kernel(const int* __restrict__ block_sums, int F, int* __restrict__ offsets, int* __restrict__ cursor) {
  const int add = block_sums[blockIdx.x];
  const int base = blockIdx.x * SCAN_ELEMS + threadIdx.x * 4;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (base + i < F) {
      const int o = offsets[base + i] + add;
      offsets[base + i] = o;
      if (cursor != nullptr) cursor[base + i] = o;
    }
  }
}

__global__ void csc_fill_kernel(const int* __restrict__ idx, long long n, int F, int* __restrict__ cursor,
                                int* __restrict__ entries) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int f = idx[i];
    if (f >= 0 && f < F) {
      const int pos = atomicAdd(&cursor[f], 1);
      entries[pos] = (int)i;
    }
  }
}

int csc_build_launch(const int* idx, long long n, int F, int* counts, int* offsets, int* cursor, int* entries,
                     int* block_sums_buf, cudaStream_t stream) {
  if (n < 0 || n > 2147483647LL || F <= 0) return (int)cudaErrorInvalidValue;  // positions are stored as 32-bit ints
  cudaError_t e = cudaMemsetAsync(counts, 0, (size_t)F * sizeof(int), stream);
  if (e != cudaSuccess) return (int)e;
  const int threads = 256;
  int blocks = (int)((n + threads - 1) / threads);
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  csc_count_kernel<<<blocks, threads, 0, stream>>>(idx, n, F, counts);
  // `block_sums_buf` holds one int per 4096 features
  const int nblocks = (F + SCAN_ELEMS - 1) / SCAN_ELEMS;
  int* block_sums = block_sums_buf;
  csc_scan_local_kernel<<<nblocks, SCAN_THREADS, 0, stream>>>(counts, F, offsets, block_sums);
  csc_scan_sums_kernel<<<1, SCAN_THREADS, 0, stream>>>(block_sums, nblocks, offsets, F);
  csc_scan_add_kernel<<<nblocks, SCAN_THREADS, 0, stream>>>(block_sums, F, offsets, cursor);
  csc_fill_kernel<<<blocks, threads, 0, stream>>>(idx, n, F, cursor, entries);
  return (int)cudaGetLastError();
}

// offsets[0..n] = exclusive prefix sum of counts[0..n-1] (offsets[n] = total); `block_sums_buf`: one int per 4096 counts
int exclusive_scan_launch(const int* counts, int n, int* offsets, int* block_sums_buf, cudaStream_t stream) {
  if (n <= 0) return (int)cudaErrorInvalidValue;
  const int nblocks = (n + SCAN_ELEMS - 1) / SCAN_ELEMS;
  csc_scan_local_kernel<<<nblocks, SCAN_THREADS, 0, stream>>>(counts, n, offsets, block_sums_buf);
  csc_scan_sums_kernel<<<1, SCAN_THREADS, 0, stream>>>(block_sums_buf, nblocks, offsets, n);
  csc_scan_add_kernel<<<nblocks, SCAN_THREADS, 0, stream>>>(block_sums_buf, n, offsets, nullptr);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// fused sparse gradient + Adam over feature rows
// ---------------------------------------------------------------------------------------------


constexpr int GA_THREADS = 256;

__device__ __forceinline__ float4 ldcs4(const float* p) { return __ldcs(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ void stcs4(float* p, const float4& v) { __stcs(reinterpret_cast<float4*>(p), v); }

__device__ __forceinline__ void adam_elem(float& p, float& m, float& v, float g, const AdamHyper& h) {
  m = h.beta1 * m + (1.0f - h.beta1) * g;
  v = h.beta2 * v + (1.0f - h.beta2) * g * g;
  const float denom = sqrtf(v) / h.bias_correction2_sqrt + h.eps;
  p -= (h.lr / h.bias_correction1) * (m / denom);
}

// One CTA walks feature rows (grid-stride). For a row it first rebuilds the two gradient rows from the
// feature's entry list (gathers of x / d x_hat rows, normally L2 hits), then streams p, m, v once.
// VEC = float4 groups per thread and chunk step. VEC 1 with four CTAs per SM is the stand-alone form (most warps to
// hide latency). VEC 2 with two CTAs per SM keeps the same number of bytes in flight per SM (twelve 16-byte loads per
// thread) with half the warps and registers-per-SM to spare: the form that shares the SMs with a concurrently running
// encoder GEMM of the next step.
// SIDES: 3 = both matrices, 1 = decoder side only, 2 = encoder side only (compile-time, so a one-sided launch carries no
// registers for the other side). One-sided launches serve dictionaries with short rows and several decoder matrices per
// encoder (cross-layer transcoders): a row is then one chunk, and what bounds the kernel is the chain offsets -> entries
// -> codes -> gathered rows -> parameters per row. There the parameter and moment loads are issued BEFORE the entry loop
// (EARLY), so that their trip to HBM overlaps the gathers, which mostly hit L2.
template <int VEC, int MIN_CTAS, int SIDES>
__global__ void __launch_bounds__(GA_THREADS, MIN_CTAS)
sparse_grad_adam_kernel(const GradAdamParams p) {
  constexpr bool doD = (SIDES & 1) != 0, doE = (SIDES & 2) != 0;
  constexpr bool EARLY = SIDES != 3;
  __shared__ float s_red[GA_THREADS / 32];
  __shared__ float s_gsq[GA_THREADS / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float gmul = p.grad_mul != nullptr ? *p.grad_mul : 1.0f;
  float gsq_local = 0.0f;
  // An earlier kernel of this step gave up on a bounded wait (its inputs never arrived): the codes and gradient rows
  // this kernel would consume are stale, so the parameters and moments stay as they are until the host has seen the
  // status word.
  const bool skip = p.status != nullptr && *reinterpret_cast<const volatile int*>(p.status) != 0;

  for (int f = p.f_begin + blockIdx.x; f < p.f_end && !skip; f += gridDim.x) {
    const int e0 = p.offsets[f], e1 = p.offsets[f + 1];
    const int xr = p.extra_row != nullptr ? p.extra_row[f] : -1;
    const float self_scale = p.wd_self_scale != nullptr ? p.wd_self_scale[f] * gmul : 0.0f;
    float bias_g = (xr >= 0 && p.extra_gb != nullptr) ? p.extra_gb[xr] : 0.0f;
    float norm_sq = 0.0f;
    for (int c0 = 0; c0 < p.d; c0 += GA_THREADS * 4 * VEC) {
      int c[VEC];
      bool in[VEC];
      size_t o[VEC], os[VEC];
      float gD[VEC][4], gE[VEC][4];
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
        c[v] = c0 + v * GA_THREADS * 4 + threadIdx.x * 4;
        in[v] = c[v] < p.d;  // d % 4 == 0
        o[v] = (size_t)f * p.d + (in[v] ? c[v] : 0);                  // parameters, shadows, dense gradient outputs
        os[v] = (size_t)(f - p.state_f0) * p.d + (in[v] ? c[v] : 0);  // moments
#pragma unroll
        for (int i = 0; i < 4; ++i) gD[v][i] = gE[v][i] = 0.0f;
        if (xr >= 0 && in[v]) {
          if (doD && p.extra_gD != nullptr) {
            const float4 a = *reinterpret_cast<const float4*>(p.extra_gD + (size_t)xr * p.d + c[v]);
            gD[v][0] = a.x; gD[v][1] = a.y; gD[v][2] = a.z; gD[v][3] = a.w;
          }
          if (doE && p.extra_gE != nullptr) {
            const float4 b = *reinterpret_cast<const float4*>(p.extra_gE + (size_t)xr * p.d + c[v]);
            gE[v][0] = b.x; gE[v][1] = b.y; gE[v][2] = b.z; gE[v][3] = b.w;
          }
        }
      }
      float4 w[VEC], m[VEC], vv[VEC], we[VEC], me[VEC], ve[VEC];
      if constexpr (EARLY) {
        if (p.update) {
#pragma unroll
          for (int v = 0; v < VEC; ++v) {
            if (in[v]) {
              if constexpr (doD) { w[v] = ldcs4(p.WD + o[v]); m[v] = ldcs4(p.mD + os[v]); vv[v] = ldcs4(p.vD + os[v]); }
              if constexpr (doE) { we[v] = ldcs4(p.WE + o[v]); me[v] = ldcs4(p.mE + os[v]); ve[v] = ldcs4(p.vE + os[v]); }
            }
          }
        }
      }
      // The entries' metadata (position, token row, code, code gradient) is fetched 32 entries at a time, one entry per
      // lane, and handed round by shuffles: one coalesced load and one integer division per entry and warp instead of
      // three dependent broadcast loads and a division per entry and THREAD, and the row gathers of successive entries
      // no longer wait for index loads in between.
      for (int eb = e0; eb < e1; eb += 32) {
        const int n_e = min(32, e1 - eb);
        int row_l = 0, aux_l = 0;
        float a_l = 0.0f, da_l = 0.0f;
        if (lane < n_e) {
          const int ent = (int)LMSAE_IDX(p.entries[eb + lane], p.n_codes);
          row_l = (int)LMSAE_IDX(ent / p.k, p.n_rows);
          a_l = p.act[ent];
          da_l = p.dact[ent];
          // codes beyond the first k_main slots of a row (auxiliary codes) multiply the auxiliary output gradient
          aux_l = (p.dxhat_aux != nullptr && ent - row_l * p.k >= p.k_main) ? 1 : 0;
        }
        for (int j = 0; j < n_e; ++j) {
          const int row = __shfl_sync(0xffffffffu, row_l, j);
          const float a = __shfl_sync(0xffffffffu, a_l, j);
          const float da = __shfl_sync(0xffffffffu, da_l, j);
          const __nv_bfloat16* gmat = __shfl_sync(0xffffffffu, aux_l, j) ? p.dxhat_aux : p.dxhat;
          if (c0 == 0 && threadIdx.x == 0) bias_g += da;
#pragma unroll
          for (int v = 0; v < VEC; ++v) {
            if (in[v]) {
              if constexpr (doD) {
                const uint2 ud = __ldg(reinterpret_cast<const uint2*>(gmat + (size_t)row * p.d + c[v]));
                const float2 d01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ud.x));
                const float2 d23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ud.y));
                gD[v][0] = fmaf(a, d01.x, gD[v][0]); gD[v][1] = fmaf(a, d01.y, gD[v][1]);
                gD[v][2] = fmaf(a, d23.x, gD[v][2]); gD[v][3] = fmaf(a, d23.y, gD[v][3]);
              }
              if constexpr (doE) {
                const uint2 ux = __ldg(reinterpret_cast<const uint2*>(p.x + (size_t)row * p.d + c[v]));
                const float2 x01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ux.x));
                const float2 x23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ux.y));
                gE[v][0] = fmaf(da, x01.x, gE[v][0]); gE[v][1] = fmaf(da, x01.y, gE[v][1]);
                gE[v][2] = fmaf(da, x23.x, gE[v][2]); gE[v][3] = fmaf(da, x23.y, gE[v][3]);
              }
            }
          }
        }
      }
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
        if (!in[v]) continue;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          gD[v][i] *= gmul;
          gE[v][i] *= gmul;
          gsq_local += gD[v][i] * gD[v][i] + gE[v][i] * gE[v][i];
        }
        if (p.gD_out != nullptr) *reinterpret_cast<float4*>(p.gD_out + o[v]) = make_float4(gD[v][0], gD[v][1], gD[v][2], gD[v][3]);
        if (p.gE_out != nullptr) *reinterpret_cast<float4*>(p.gE_out + o[v]) = make_float4(gE[v][0], gE[v][1], gE[v][2], gE[v][3]);
      }
      if (p.update) {
        // all streams of this chunk step are requested before the first is used (96 bytes in flight per thread and VEC)
        if constexpr (!EARLY) {
#pragma unroll
          for (int v = 0; v < VEC; ++v) {
            if (in[v]) {
              if constexpr (doD) { w[v] = ldcs4(p.WD + o[v]); m[v] = ldcs4(p.mD + os[v]); vv[v] = ldcs4(p.vD + os[v]); }
              if constexpr (doE) { we[v] = ldcs4(p.WE + o[v]); me[v] = ldcs4(p.mE + os[v]); ve[v] = ldcs4(p.vE + os[v]); }
            }
          }
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
          if (!in[v]) continue;
          if constexpr (doD) {
            if (self_scale != 0.0f) {  // (not part of the squared-norm accumulation above: a penalty term's share is small)
              gD[v][0] = fmaf(self_scale, w[v].x, gD[v][0]); gD[v][1] = fmaf(self_scale, w[v].y, gD[v][1]);
              gD[v][2] = fmaf(self_scale, w[v].z, gD[v][2]); gD[v][3] = fmaf(self_scale, w[v].w, gD[v][3]);
            }
            adam_elem(w[v].x, m[v].x, vv[v].x, gD[v][0], p.h); adam_elem(w[v].y, m[v].y, vv[v].y, gD[v][1], p.h);
            adam_elem(w[v].z, m[v].z, vv[v].z, gD[v][2], p.h); adam_elem(w[v].w, m[v].w, vv[v].w, gD[v][3], p.h);
            stcs4(p.WD + o[v], w[v]); stcs4(p.mD + os[v], m[v]); stcs4(p.vD + os[v], vv[v]);
            norm_sq += w[v].x * w[v].x + w[v].y * w[v].y + w[v].z * w[v].z + w[v].w * w[v].w;
            uint2 sh; sh.x = pack_bf16x2(w[v].x, w[v].y); sh.y = pack_bf16x2(w[v].z, w[v].w);
            if (SIDES == 3 && p.n_pub > 0) {
              for (int q = 0; q < p.n_pub; ++q)
                *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.pub.base[q] + p.pub_wd_off) + o[v]) = sh;
            } else {
              *reinterpret_cast<uint2*>(p.WD_bf16 + o[v]) = sh;
            }
          }
          if constexpr (doE) {
            adam_elem(we[v].x, me[v].x, ve[v].x, gE[v][0], p.h); adam_elem(we[v].y, me[v].y, ve[v].y, gE[v][1], p.h);
            adam_elem(we[v].z, me[v].z, ve[v].z, gE[v][2], p.h); adam_elem(we[v].w, me[v].w, ve[v].w, gE[v][3], p.h);
            stcs4(p.WE + o[v], we[v]); stcs4(p.mE + os[v], me[v]); stcs4(p.vE + os[v], ve[v]);
            uint2 sh; sh.x = pack_bf16x2(we[v].x, we[v].y); sh.y = pack_bf16x2(we[v].z, we[v].w);
            if (SIDES == 3 && p.n_pub > 0) {
              for (int q = 0; q < p.n_pub; ++q)
                *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.pub.base[q] + p.pub_we_off) + o[v]) = sh;
            } else {
              *reinterpret_cast<uint2*>(p.WE_bf16 + o[v]) = sh;
            }
          }
        }
      }
    }
    if (threadIdx.x == 0) {
      bias_g *= gmul;
      gsq_local += bias_g * bias_g;
      if (p.update && p.bE != nullptr && doE) {
        float b = p.bE[f], m = p.mbE[f - p.state_f0], v = p.vbE[f - p.state_f0];
        adam_elem(b, m, v, bias_g, p.h);
        p.mbE[f - p.state_f0] = m; p.vbE[f - p.state_f0] = v;
        if (SIDES == 3 && p.n_pub > 0) {
          for (int q = 0; q < p.n_pub; ++q) reinterpret_cast<float*>(p.pub.base[q] + p.pub_be_off)[f] = b;
        } else {
          p.bE[f] = b;
        }
      }
    }
    if (p.update && doD && (p.dec_norm != nullptr || p.norm_sq_accum != nullptr)) {
      norm_sq = warp_sum(norm_sq);
      __syncthreads();
      if (lane == 0) s_red[warp] = norm_sq;
      __syncthreads();
      if (warp == 0) {
        float t = lane < GA_THREADS / 32 ? s_red[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) {
          if (p.norm_sq_accum != nullptr) {
            p.norm_sq_accum[f] += t;  // one CTA per row and launch: the squared norms of several matrices add up here
          } else if (SIDES == 3 && p.n_pub > 0) {
            for (int q = 0; q < p.n_pub; ++q) reinterpret_cast<float*>(p.pub.base[q] + p.pub_norm_off)[f] = sqrtf(t);
          } else {
            p.dec_norm[f] = sqrtf(t);
          }
        }
      }
    }
  }
  if (p.grad_sq_sum != nullptr) {
    gsq_local = warp_sum(gsq_local);
    if (lane == 0) s_gsq[warp] = gsq_local;
    __syncthreads();
    if (warp == 0) {
      float t = lane < GA_THREADS / 32 ? s_gsq[lane] : 0.0f;
      t = warp_sum(t);
      if (lane == 0) atomicAdd(p.grad_sq_sum, t);
    }
  }
  // published even when the update was skipped, so that the replicas waiting for this rank's rows do not time out too
  if constexpr (SIDES == 3) {
    if (p.n_pub > 0 && p.update) signal_peers_when_grid_done(p.pub, kPhaseParams, p.pub_epoch, p.pub_done);
  }
}

// ---------------------------------------------------------------------------------------------
// Short rows (d <= 1024, a multiple of 128): one WARP per feature row. With rows of 3 KB a CTA per row spends its time in
// the dependent chain offsets -> entries -> codes -> gathered rows -> parameters, and a block barrier per row for the
// norm; here sixteen rows are in flight per SM (eight warps per CTA, two CTAs), a lane owns four consecutive columns of
// every 128-column chunk, the row norm is a warp reduction, and nothing synchronises the block. A two-sided update
// runs as two launches, one per side. Not supported here (the CTA-per-row kernel
// takes those launches): extra dense rows, publication to replicas, dense gradient outputs.
// ---------------------------------------------------------------------------------------------
constexpr int RW_MAX_CHUNKS = 8;  // d <= 1024
constexpr int RW_GROUP = 4;       // parameter chunks loaded together (12 x 16 bytes in flight per lane)

// One side of one row. G: gather source (d x_hat for the decoder side, x for the encoder side); coef_l: this lane's
// entry's coefficient (code for the decoder side, code gradient for the encoder side), row_l / aux_l likewise.
template <bool IS_D>
__device__ __forceinline__ void rowwarp_side(const GradAdamParams& p, int f, int e0, int e1, int lane, int nch, float gmul,
                                             float& gsq_local) {
  float* W = IS_D ? p.WD : p.WE;
  float* M1 = IS_D ? p.mD : p.mE;
  float* M2 = IS_D ? p.vD : p.vE;
  __nv_bfloat16* SH = IS_D ? p.WD_bf16 : p.WE_bf16;
  const __nv_bfloat16* G = IS_D ? p.dxhat : p.x;
  float g[RW_MAX_CHUNKS][4];
#pragma unroll
  for (int c = 0; c < RW_MAX_CHUNKS; ++c) g[c][0] = g[c][1] = g[c][2] = g[c][3] = 0.0f;
  float bias_g = 0.0f;
  for (int eb = e0; eb < e1; eb += 32) {
    const int n_e = min(32, e1 - eb);
    int row_l = 0, aux_l = 0;
    float coef_l = 0.0f;
    if (lane < n_e) {
      const int ent = (int)LMSAE_IDX(p.entries[eb + lane], p.n_codes);
      row_l = (int)LMSAE_IDX(ent / p.k, p.n_rows);
      coef_l = IS_D ? p.act[ent] : p.dact[ent];
      aux_l = (IS_D && p.dxhat_aux != nullptr && ent - row_l * p.k >= p.k_main) ? 1 : 0;
    }
    if (!IS_D) bias_g += coef_l;  // summed over the lanes below
    for (int j = 0; j < n_e; ++j) {
      const int row = __shfl_sync(0xffffffffu, row_l, j);
      const float a = __shfl_sync(0xffffffffu, coef_l, j);
      const __nv_bfloat16* src = (IS_D && __shfl_sync(0xffffffffu, aux_l, j)) ? p.dxhat_aux : G;
      const __nv_bfloat16* gr = src + (size_t)row * p.d + lane * 4;
#pragma unroll
      for (int c = 0; c < RW_MAX_CHUNKS; ++c) {
        if (c < nch) {
          const uint2 u = __ldg(reinterpret_cast<const uint2*>(gr + c * 128));
          const float2 v01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
          const float2 v23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
          g[c][0] = fmaf(a, v01.x, g[c][0]); g[c][1] = fmaf(a, v01.y, g[c][1]);
          g[c][2] = fmaf(a, v23.x, g[c][2]); g[c][3] = fmaf(a, v23.y, g[c][3]);
        }
      }
    }
  }
#pragma unroll
  for (int c = 0; c < RW_MAX_CHUNKS; ++c) {
    if (c < nch) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        g[c][i] *= gmul;
        gsq_local += g[c][i] * g[c][i];
      }
    }
  }
  if (!IS_D) {
    bias_g = warp_sum(bias_g) * gmul;
    if (lane == 0) gsq_local += bias_g * bias_g;
  }
  if (!p.update) return;
  const float self_scale = (IS_D && p.wd_self_scale != nullptr) ? p.wd_self_scale[f] * gmul : 0.0f;
  float norm_sq = 0.0f;
  const size_t o0 = (size_t)f * p.d + lane * 4, os0 = (size_t)(f - p.state_f0) * p.d + lane * 4;
#pragma unroll
  for (int c0 = 0; c0 < RW_MAX_CHUNKS; c0 += RW_GROUP) {
    if (c0 >= nch) break;
    float4 w[RW_GROUP], m[RW_GROUP], v[RW_GROUP];
#pragma unroll
    for (int q = 0; q < RW_GROUP; ++q) {
      if (c0 + q < nch) {
        w[q] = ldcs4(W + o0 + (c0 + q) * 128);
        m[q] = ldcs4(M1 + os0 + (c0 + q) * 128);
        v[q] = ldcs4(M2 + os0 + (c0 + q) * 128);
      }
    }
#pragma unroll
    for (int q = 0; q < RW_GROUP; ++q) {
      if (c0 + q < nch) {
        float* gg = g[c0 + q];
        if (IS_D && self_scale != 0.0f) {
          gg[0] = fmaf(self_scale, w[q].x, gg[0]); gg[1] = fmaf(self_scale, w[q].y, gg[1]);
          gg[2] = fmaf(self_scale, w[q].z, gg[2]); gg[3] = fmaf(self_scale, w[q].w, gg[3]);
        }
        adam_elem(w[q].x, m[q].x, v[q].x, gg[0], p.h); adam_elem(w[q].y, m[q].y, v[q].y, gg[1], p.h);
        adam_elem(w[q].z, m[q].z, v[q].z, gg[2], p.h); adam_elem(w[q].w, m[q].w, v[q].w, gg[3], p.h);
        stcs4(W + o0 + (c0 + q) * 128, w[q]);
        stcs4(M1 + os0 + (c0 + q) * 128, m[q]);
        stcs4(M2 + os0 + (c0 + q) * 128, v[q]);
        if (IS_D) norm_sq += w[q].x * w[q].x + w[q].y * w[q].y + w[q].z * w[q].z + w[q].w * w[q].w;
        uint2 sh;
        sh.x = pack_bf16x2(w[q].x, w[q].y);
        sh.y = pack_bf16x2(w[q].z, w[q].w);
        *reinterpret_cast<uint2*>(SH + o0 + (c0 + q) * 128) = sh;
      }
    }
  }
  if (IS_D) {
    if (p.dec_norm != nullptr || p.norm_sq_accum != nullptr) {
      norm_sq = warp_sum(norm_sq);
      if (lane == 0) {
        if (p.norm_sq_accum != nullptr) p.norm_sq_accum[f] += norm_sq;  // one warp per row and launch
        else p.dec_norm[f] = sqrtf(norm_sq);
      }
    }
  } else if (lane == 0 && p.bE != nullptr) {
    float b = p.bE[f], m = p.mbE[f - p.state_f0], v = p.vbE[f - p.state_f0];
    adam_elem(b, m, v, bias_g, p.h);
    p.mbE[f - p.state_f0] = m;
    p.vbE[f - p.state_f0] = v;
    p.bE[f] = b;
  }
}

template <int SIDES>
__global__ void __launch_bounds__(GA_THREADS, 2)
sparse_grad_adam_rowwarp_kernel(const GradAdamParams p) {
  __shared__ float s_gsq[GA_THREADS / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float gmul = p.grad_mul != nullptr ? *p.grad_mul : 1.0f;
  const bool skip = p.status != nullptr && *reinterpret_cast<const volatile int*>(p.status) != 0;  // see the kernel above
  const int nch = p.d / 128;
  float gsq_local = 0.0f;
  const int warps = gridDim.x * (GA_THREADS / 32);
  for (int f = p.f_begin + blockIdx.x * (GA_THREADS / 32) + warp; f < p.f_end && !skip; f += warps) {
    const int e0 = p.offsets[f], e1 = p.offsets[f + 1];
    if constexpr ((SIDES & 1) != 0) rowwarp_side<true>(p, f, e0, e1, lane, nch, gmul, gsq_local);
    if constexpr ((SIDES & 2) != 0) rowwarp_side<false>(p, f, e0, e1, lane, nch, gmul, gsq_local);
  }
  if (p.grad_sq_sum != nullptr) {
    gsq_local = warp_sum(gsq_local);
    if (lane == 0) s_gsq[warp] = gsq_local;
    __syncthreads();
    if (warp == 0) {
      float t = lane < GA_THREADS / 32 ? s_gsq[lane] : 0.0f;
      t = warp_sum(t);
      if (lane == 0) atomicAdd(p.grad_sq_sum, t);
    }
  }
}

int sparse_grad_adam_launch(const GradAdamParams& p, cudaStream_t stream) {
  if (p.d % 4 != 0) return (int)cudaErrorInvalidValue;
  const int rows = p.f_end - p.f_begin;
  if (rows <= 0) return 0;
  // CTAs are persistent (grid-stride over feature rows): the grid size sets how many share an SM
  if (p.n_pub < 0 || p.n_pub > kMaxPeers || (p.n_pub > 0 && p.n_pub != p.pub.world)) return (int)cudaErrorInvalidValue;
  if (p.state_f0 < 0 || p.state_f0 > p.f_begin) return (int)cudaErrorInvalidValue;
  const int cap = (p.ctas_per_sm >= 1 && p.ctas_per_sm <= 4) ? 148 * p.ctas_per_sm : 148 * 8;
  int blocks = rows < cap ? rows : cap;
  const bool doD = p.WD != nullptr, doE = p.WE != nullptr;
  if (!doD && !doE) return (int)cudaErrorInvalidValue;
  if (!(doD && doE) && p.n_pub > 0) return (int)cudaErrorInvalidValue;  // rows are published by two-sided launches only
  if (p.d <= 128 * RW_MAX_CHUNKS && p.d % 128 == 0 && p.extra_row == nullptr && p.n_pub == 0 && p.gD_out == nullptr &&
      p.gE_out == nullptr && p.ctas_per_sm == 0 && p.use_rowwarp != 0) {
    // short rows: a warp per row
    const int per_cta = GA_THREADS / 32;
    int rw_blocks = (rows + per_cta - 1) / per_cta;
    if (rw_blocks > 148 * 2) rw_blocks = 148 * 2;
    // (a two-sided update is two launches: both sides in one kernel do not fit the register budget of two CTAs per SM)
    if (doD) sparse_grad_adam_rowwarp_kernel<1><<<rw_blocks, GA_THREADS, 0, stream>>>(p);
    if (doE) sparse_grad_adam_rowwarp_kernel<2><<<rw_blocks, GA_THREADS, 0, stream>>>(p);
    return (int)cudaGetLastError();
  }
  if (doD && doE) {
    if (p.ctas_per_sm >= 1 && p.ctas_per_sm <= 2)
      sparse_grad_adam_kernel<2, 2, 3><<<blocks, GA_THREADS, 0, stream>>>(p);
    else
      sparse_grad_adam_kernel<1, 4, 3><<<blocks, GA_THREADS, 0, stream>>>(p);
  } else {
    // one-sided: fewer registers; the encoder side fits five CTAs (rows in flight) per SM, the decoder side (row norms,
    // norm penalty) four without spilling
    const int per_sm = doD ? 4 : 5;
    if (p.ctas_per_sm < 1 || p.ctas_per_sm > per_sm) blocks = rows < 148 * per_sm ? rows : 148 * per_sm;
    if (doD) sparse_grad_adam_kernel<1, 4, 1><<<blocks, GA_THREADS, 0, stream>>>(p);
    else sparse_grad_adam_kernel<1, 5, 2><<<blocks, GA_THREADS, 0, stream>>>(p);
  }
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// dense helpers: column sum of a bf16 matrix, and a flat Adam step with an explicit gradient
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
colsum_bf16_kernel(const __nv_bfloat16* __restrict__ a, int rows, int d, int rows_per_block, float* __restrict__ out) {
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(rows, r0 + rows_per_block);
  for (int c = blockIdx.x * 256 + threadIdx.x; c < d; c += gridDim.x * 256) {
    float s = 0.0f;
    for (int r = r0; r < r1; ++r) s += __bfloat162float(a[(size_t)r * d + c]);
    atomicAdd(out + c, s);
  }
}

int colsum_bf16_launch(const __nv_bfloat16* a, int rows, int d, float* out, cudaStream_t stream) {
  cudaError_t e = cudaMemsetAsync(out, 0, (size_t)d * sizeof(float), stream);
  if (e != cudaSuccess) return (int)e;
  const int rows_per_block = 64;
  dim3 grid((d + 255) / 256, (rows + rows_per_block - 1) / rows_per_block);
  colsum_bf16_kernel<<<grid, 256, 0, stream>>>(a, rows, d, rows_per_block, out);
  return (int)cudaGetLastError();
}

// Flat Adam (torch.optim.Adam semantics without weight decay / amsgrad), optional bf16 shadow and
// squared-gradient accumulation. Used for small dense parameters (b_D, thresholds) and by the generic
// multi-tensor optimizer.
__global__ void __launch_bounds__(256)
adam_flat_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                 long long n, AdamHyper h, const float* __restrict__ grad_mul, __nv_bfloat16* __restrict__ shadow,
                 float* __restrict__ grad_sq_sum, int update, const int* __restrict__ status) {
  __shared__ float s_gsq[8];
  if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) return;  // see sparse_grad_adam_kernel
  const float gmul = grad_mul != nullptr ? *grad_mul : 1.0f;
  float gsq = 0.0f;
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < n; i += (long long)gridDim.x * 256) {
    const float gi = g[i] * gmul;
    gsq += gi * gi;
    if (update) {
      float pi = p[i], mi = m[i], vi = v[i];
      adam_elem(pi, mi, vi, gi, h);
      p[i] = pi; m[i] = mi; v[i] = vi;
      if (shadow != nullptr) shadow[i] = __float2bfloat16(pi);
    }
  }
  if (grad_sq_sum != nullptr) {
    gsq = warp_sum(gsq);
    if ((threadIdx.x & 31) == 0) s_gsq[threadIdx.x >> 5] = gsq;
    __syncthreads();
    if (threadIdx.x < 32) {
      float t = threadIdx.x < 8 ? s_gsq[threadIdx.x] : 0.0f;
      t = warp_sum(t);
      if (threadIdx.x == 0) atomicAdd(grad_sq_sum, t);
    }
  }
}

int adam_flat_launch(float* p, const float* g, float* m, float* v, long long n, AdamHyper h, const float* grad_mul,
                     __nv_bfloat16* shadow, float* grad_sq_sum, int update, const int* status, cudaStream_t stream) {
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  adam_flat_kernel<<<(int)blocks, 256, 0, stream>>>(p, g, m, v, n, h, grad_mul, shadow, grad_sq_sum, update, status);
  return (int)cudaGetLastError();
}

// Row L2 norms of an fp32 [F, d] matrix (+ optional bf16 shadow refresh): used at set-up and after
// loading weights so that dec_norm / shadows agree with the master copy.
__global__ void __launch_bounds__(256)
row_norm_shadow_kernel(const float* __restrict__ W, int F, int d, float* __restrict__ norm,
                       __nv_bfloat16* __restrict__ shadow) {
  __shared__ float s_red[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int f = blockIdx.x; f < F; f += gridDim.x) {
    float s = 0.0f;
    for (int c = threadIdx.x; c < d; c += 256) {
      const float w = W[(size_t)f * d + c];
      s = fmaf(w, w, s);
      if (shadow != nullptr) shadow[(size_t)f * d + c] = __float2bfloat16(w);
    }
    s = warp_sum(s);
    __syncthreads();
    if (lane == 0) s_red[warp] = s;
    __syncthreads();
    if (warp == 0) {
      float t = lane < 8 ? s_red[lane] : 0.0f;
      t = warp_sum(t);
      if (lane == 0 && norm != nullptr) norm[f] = sqrtf(t);
    }
  }
}

int row_norm_shadow_launch(const float* W, int F, int d, float* norm, __nv_bfloat16* shadow, cudaStream_t stream) {
  int blocks = F < 148 * 16 ? F : 148 * 16;
  row_norm_shadow_kernel<<<blocks, 256, 0, stream>>>(W, F, d, norm, shadow);
  return (int)cudaGetLastError();
}

}  // namespace lmsae
