// Python bindings (torch extension) for the sm_100a kernels. Tensors are checked for device, dtype and
// contiguity here; the kernels assume what these checks guarantee.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <torch/extension.h>

#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

#include "kernels.h"

namespace {

using torch::Tensor;

void check_cuda(int code, const char* what) {
  TORCH_CHECK(code == 0, what, " failed: ", cudaGetErrorString(static_cast<cudaError_t>(code)));
}

#define CHECK_T(t, dt)                                                       \
  TORCH_CHECK((t).is_cuda(), #t " must be a CUDA tensor");                   \
  TORCH_CHECK((t).scalar_type() == (dt), #t " has the wrong dtype");         \
  TORCH_CHECK((t).is_contiguous(), #t " must be contiguous")

template <typename T>
T* opt_ptr(const c10::optional<Tensor>& t) {
  return t.has_value() ? reinterpret_cast<T*>(t->data_ptr()) : nullptr;
}

// ---- peer tables -----------------------------------------------------------------------------------
// `table` = [world, rank, flags_off, cand_val_off, cand_idx_off, partial_off, dxhat_off, multicast base pointer (0: none),
//            pointer to the exposed-wait counters (0: none), ptr_0 .. ptr_{world-1}]
constexpr int kPeerTableHeader = 9;
lmsae::PeerTable make_peer_table(const std::vector<int64_t>& table) {
  TORCH_CHECK((int)table.size() >= kPeerTableHeader + 1, "peer table too short");
  lmsae::PeerTable pt{};
  pt.world = (int)table[0];
  pt.rank = (int)table[1];
  TORCH_CHECK(pt.world >= 1 && pt.world <= lmsae::kMaxPeers && pt.rank >= 0 && pt.rank < pt.world, "bad world/rank");
  TORCH_CHECK((int)table.size() == kPeerTableHeader + pt.world, "peer table needs one pointer per rank");
  pt.flags_off = table[2];
  pt.cand_val_off = table[3];
  pt.cand_idx_off = table[4];
  pt.partial_off = table[5];
  pt.dxhat_off = table[6];
  pt.mc_base = reinterpret_cast<char*>(static_cast<uintptr_t>(table[7]));
  pt.stats = reinterpret_cast<unsigned long long*>(static_cast<uintptr_t>(table[8]));
  for (int i = 0; i < pt.world; ++i) pt.base[i] = reinterpret_cast<char*>(static_cast<uintptr_t>(table[kPeerTableHeader + i]));
  return pt;
}

// ---- tensor maps -----------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    TORCH_CHECK(e == cudaSuccess && p != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 2-D bf16 row-major [rows, cols] tensor, box = {64 columns, box_rows}, 128-byte swizzle.
CUtensorMap make_bf16_tile_map(const void* base, int64_t rows, int64_t cols, int box_rows) {
  TORCH_CHECK(reinterpret_cast<uintptr_t>(base) % 16 == 0, "TMA base address must be 16-byte aligned");
  TORCH_CHECK((cols * 2) % 16 == 0, "TMA row pitch must be a multiple of 16 bytes (K % 8 == 0)");
  CUtensorMap m;
  cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estride[2] = {1, 1};
  CUresult r = get_encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box,
                               estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", (int)r);
  return m;
}

// ---- encoder GEMM ----------------------------------------------------------------------------------
// mode bit 0: write H (bf16 [M, N]); bit 1: fused per-row top-k candidates.
// Returns the number of candidate slots per range (KS) so that callers can size / interpret the buffers.
int64_t encoder_gemm(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& bias,
                     const c10::optional<Tensor>& gate, int64_t mode, int64_t k, int64_t num_splits,
                     const c10::optional<Tensor>& H, const c10::optional<Tensor>& cand_val,
                     const c10::optional<Tensor>& cand_idx, const Tensor& status, int64_t n_index_offset,
                     bool resume_topk, int64_t units) {
  CHECK_T(x, torch::kBFloat16);
  CHECK_T(w, torch::kBFloat16);
  CHECK_T(status, torch::kInt32);
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && x.size(1) == w.size(1), "x [M,K] and w [N,K] must share K");
  const c10::cuda::CUDAGuard guard(x.device());
  lmsae::EncGemmParams p{};
  p.M = (int)x.size(0);
  p.K = (int)x.size(1);
  p.N = (int)w.size(0);
  TORCH_CHECK(p.K % 8 == 0 && p.N % 8 == 0, "K and N must be multiples of 8");
  p.num_panels = (p.M + 127) / 128;
  p.num_splits = (int)num_splits;
  p.units = (int)units;  // 0: num_splits ranges for every panel (pair); else that many work units dealt out raggedly
  const int n_tiles = (p.N + 255) / 256;
  TORCH_CHECK(p.num_splits >= 1 && p.num_splits <= n_tiles, "num_splits must be in [1, number of N tiles]");
  if (bias.has_value()) { CHECK_T(*bias, torch::kFloat32); TORCH_CHECK(bias->numel() == p.N); }
  if (gate.has_value()) { CHECK_T(*gate, torch::kFloat32); TORCH_CHECK(gate->numel() == p.N); }
  p.bias = opt_ptr<const float>(bias);
  p.gate = opt_ptr<const float>(gate);
  p.status = status.data_ptr<int>();
  p.k = (int)k;
  p.n_index_offset = (int)n_index_offset;
  p.resume_topk = resume_topk ? 1 : 0;
  int ks = 0;
  if (mode & 1) {
    TORCH_CHECK(H.has_value(), "mode bit 0 needs H");
    CHECK_T(*H, torch::kBFloat16);
    TORCH_CHECK(H->size(0) == p.M && H->size(1) == p.N);
    p.H = reinterpret_cast<__nv_bfloat16*>(H->data_ptr());
    p.ldh = p.N;
  }
  if (mode & 2) {
    TORCH_CHECK(k >= 1 && k <= 64, "fused top-k supports 1 <= k <= 64");
    ks = lmsae::enc_gemm_slots_for_k((int)k);
    TORCH_CHECK(cand_val.has_value() && cand_idx.has_value());
    CHECK_T(*cand_val, torch::kFloat32);
    CHECK_T(*cand_idx, torch::kInt32);
    TORCH_CHECK(cand_val->numel() >= (int64_t)p.M * p.num_splits * ks && cand_idx->numel() >= (int64_t)p.M * p.num_splits * ks,
                "candidate buffers too small");
    p.cand_val = cand_val->data_ptr<float>();
    p.cand_idx = cand_idx->data_ptr<int>();
  }
  TORCH_CHECK(mode & 3, "mode must request H and/or top-k");
  // bit 3 asks for the CTA-pair kernel; it needs whole pairs of 128-row panels, otherwise the single-CTA kernel runs
  if ((mode & 8) && (p.num_panels % 2 != 0)) {
    mode &= ~(int64_t)8;
    p.units = 0;  // (a ragged deal was sized for pairs)
  }
  const CUtensorMap ta = make_bf16_tile_map(x.data_ptr(), p.M, p.K, 128);
  const CUtensorMap tb = make_bf16_tile_map(w.data_ptr(), p.N, p.K, (mode & 8) ? 128 : 256);
  check_cuda(lmsae::enc_gemm_launch(ta, tb, p, (int)mode, at::cuda::getCurrentCUDAStream()), "encoder_gemm launch");
  return ks;
}

// comm_mode 0: plain merge. 1: the k winners of every row are stored into every rank's merge input (`table`, candidate
// offsets already pointing at the buffer of this exchange) instead of out_idx / out_val, and the epoch is published.
// 2: wait for every rank's candidate flag of `epoch` first; cand_val / cand_idx are views of this rank's buffer.
void topk_merge(const Tensor& cand_val, const Tensor& cand_idx, int64_t M, int64_t C, int64_t k,
                const c10::optional<Tensor>& gate, int64_t own_lo, int64_t own_hi, bool emit_gated,
                const c10::optional<Tensor>& out_idx, const c10::optional<Tensor>& out_val, int64_t comm_mode,
                const std::vector<int64_t>& table, int64_t epoch, const c10::optional<Tensor>& done_counter,
                const c10::optional<Tensor>& status) {
  CHECK_T(cand_val, torch::kFloat32);
  CHECK_T(cand_idx, torch::kInt32);
  TORCH_CHECK(cand_val.numel() >= M * C && cand_idx.numel() >= M * C);
  TORCH_CHECK(0 <= own_lo && own_lo <= own_hi && own_hi <= C);
  lmsae::MergeComm comm{};
  comm.mode = (int)comm_mode;
  TORCH_CHECK(comm_mode >= 0 && comm_mode <= 2, "comm_mode must be 0, 1 or 2");
  if (comm_mode != lmsae::kMergePush) {
    TORCH_CHECK(out_idx.has_value() && out_val.has_value());
    CHECK_T(*out_idx, torch::kInt32);
    CHECK_T(*out_val, torch::kFloat32);
    TORCH_CHECK(out_idx->numel() >= M * k && out_val->numel() >= M * k);
  }
  if (comm_mode != lmsae::kMergeLocal) {
    comm.pt = make_peer_table(table);
    comm.epoch = (uint32_t)epoch;
    TORCH_CHECK(status.has_value());
    CHECK_T(*status, torch::kInt32);
    comm.status = status->data_ptr<int>();
    if (comm_mode == lmsae::kMergePush) {
      TORCH_CHECK(done_counter.has_value());
      CHECK_T(*done_counter, torch::kInt32);
      comm.done_counter = reinterpret_cast<unsigned*>(done_counter->data_ptr<int>());
    }
  }
  const c10::cuda::CUDAGuard guard(cand_val.device());
  check_cuda(lmsae::topk_merge_launch(cand_val.data_ptr<float>(), cand_idx.data_ptr<int>(), (int)M, (int)C, (int)k,
                                      opt_ptr<const float>(gate), (int)own_lo, (int)own_hi, emit_gated ? 1 : 0,
                                      opt_ptr<int>(out_idx), opt_ptr<float>(out_val), comm,
                                      at::cuda::getCurrentCUDAStream()),
             "topk_merge launch");
}

void row_topk(const Tensor& H, int64_t k, const c10::optional<Tensor>& gate, const c10::optional<Tensor>& alive,
              const Tensor& out_idx, const Tensor& out_val) {
  CHECK_T(H, torch::kBFloat16);
  CHECK_T(out_idx, torch::kInt32);
  CHECK_T(out_val, torch::kFloat32);
  TORCH_CHECK(H.dim() == 2 && out_idx.numel() >= H.size(0) * k && out_val.numel() >= H.size(0) * k);
  if (alive.has_value()) { CHECK_T(*alive, torch::kUInt8); TORCH_CHECK(alive->numel() == H.size(1)); }
  if (gate.has_value()) { CHECK_T(*gate, torch::kFloat32); TORCH_CHECK(gate->numel() == H.size(1)); }
  const c10::cuda::CUDAGuard guard(H.device());
  check_cuda(lmsae::row_topk_launch(reinterpret_cast<const __nv_bfloat16*>(H.data_ptr()), H.size(1), (int)H.size(0),
                                    (int)H.size(1), (int)k, opt_ptr<const float>(gate), opt_ptr<const uint8_t>(alive),
                                    out_idx.data_ptr<int>(), out_val.data_ptr<float>(),
                                    at::cuda::getCurrentCUDAStream()),
             "row_topk launch");
}

// x_hat = decode(idx, val); optional outputs and fused loss as described in sparse_ops.cu.
void sparse_decode(const Tensor& idx, const Tensor& val, const Tensor& W, const c10::optional<Tensor>& bias,
                   const c10::optional<Tensor>& xhat_f32, const c10::optional<Tensor>& xhat_bf16,
                   const c10::optional<Tensor>& label, const c10::optional<Tensor>& row_weight, double grad_scale,
                   const c10::optional<Tensor>& dxhat, const c10::optional<Tensor>& loss_sum,
                   const c10::optional<Tensor>& row_loss, const c10::optional<Tensor>& dval) {
  CHECK_T(idx, torch::kInt32);
  CHECK_T(val, torch::kFloat32);
  CHECK_T(W, torch::kBFloat16);
  TORCH_CHECK(idx.dim() == 2 && val.sizes() == idx.sizes() && W.dim() == 2);
  const c10::cuda::CUDAGuard guard(idx.device());
  lmsae::DecodeParams p{};
  p.idx = idx.data_ptr<int>();
  p.val = val.data_ptr<float>();
  p.B = (int)idx.size(0);
  p.k = (int)idx.size(1);
  p.d = (int)W.size(1);
  p.F = (int)W.size(0);
  p.W = reinterpret_cast<const __nv_bfloat16*>(W.data_ptr());
  if (bias.has_value()) { CHECK_T(*bias, torch::kFloat32); TORCH_CHECK(bias->numel() == p.d); }
  p.bias = opt_ptr<const float>(bias);
  if (xhat_f32.has_value()) { CHECK_T(*xhat_f32, torch::kFloat32); TORCH_CHECK(xhat_f32->numel() == (int64_t)p.B * p.d); }
  if (xhat_bf16.has_value()) { CHECK_T(*xhat_bf16, torch::kBFloat16); TORCH_CHECK(xhat_bf16->numel() == (int64_t)p.B * p.d); }
  p.xhat_f32 = opt_ptr<float>(xhat_f32);
  p.xhat_bf16 = opt_ptr<__nv_bfloat16>(xhat_bf16);
  if (label.has_value()) {
    CHECK_T(*label, torch::kBFloat16);
    TORCH_CHECK(label->numel() == (int64_t)p.B * p.d);
    TORCH_CHECK(dxhat.has_value() && loss_sum.has_value(), "fused loss needs dxhat and loss_sum");
    CHECK_T(*dxhat, torch::kBFloat16);
    CHECK_T(*loss_sum, torch::kFloat32);
    TORCH_CHECK(dxhat->numel() == (int64_t)p.B * p.d);
    if (row_weight.has_value()) { CHECK_T(*row_weight, torch::kFloat32); TORCH_CHECK(row_weight->numel() == p.B); }
    if (row_loss.has_value()) { CHECK_T(*row_loss, torch::kFloat32); TORCH_CHECK(row_loss->numel() == p.B); }
    if (dval.has_value()) { CHECK_T(*dval, torch::kFloat32); TORCH_CHECK(dval->numel() == (int64_t)p.B * p.k); }
    p.label = reinterpret_cast<const __nv_bfloat16*>(label->data_ptr());
    p.row_weight = opt_ptr<const float>(row_weight);
    p.grad_scale = (float)grad_scale;
    p.dxhat = opt_ptr<__nv_bfloat16>(dxhat);
    p.loss_sum = opt_ptr<float>(loss_sum);
    p.row_loss = opt_ptr<float>(row_loss);
    p.dval = opt_ptr<float>(dval);
  }
  check_cuda(lmsae::sparse_decode_launch(p, at::cuda::getCurrentCUDAStream()), "sparse_decode launch");
}

// `table` non-empty: dxhat is the gradient buffer of the fused feature-sharded step; the kernel waits for the row owners'
// flags of `epoch` before reading it.
void sparse_dact(const Tensor& idx, const Tensor& W, const Tensor& dxhat, const Tensor& dval,
                 const std::vector<int64_t>& table, int64_t epoch, const c10::optional<Tensor>& status) {
  CHECK_T(idx, torch::kInt32);
  CHECK_T(W, torch::kBFloat16);
  CHECK_T(dxhat, torch::kBFloat16);
  CHECK_T(dval, torch::kFloat32);
  TORCH_CHECK(idx.dim() == 2 && dval.numel() == idx.numel() && dxhat.numel() == idx.size(0) * W.size(1));
  const c10::cuda::CUDAGuard guard(idx.device());
  lmsae::PeerTable pt{};
  if (!table.empty()) {
    pt = make_peer_table(table);
    TORCH_CHECK(status.has_value());
    CHECK_T(*status, torch::kInt32);
  }
  check_cuda(lmsae::sparse_dact_launch(idx.data_ptr<int>(), (int)idx.size(0), (int)idx.size(1), (int)W.size(1), (int)W.size(0),
                                       reinterpret_cast<const __nv_bfloat16*>(W.data_ptr()),
                                       reinterpret_cast<const __nv_bfloat16*>(dxhat.data_ptr()),
                                       dval.data_ptr<float>(), table.empty() ? nullptr : &pt, (uint32_t)epoch,
                                       opt_ptr<int>(status), at::cuda::getCurrentCUDAStream()),
             "sparse_dact launch");
}

void mse_loss_grad(const Tensor& xhat, const Tensor& label, const c10::optional<Tensor>& bias,
                   const c10::optional<Tensor>& row_weight, double grad_scale, const Tensor& dxhat,
                   const Tensor& loss_sum, const c10::optional<Tensor>& row_loss) {
  CHECK_T(xhat, torch::kFloat32);
  CHECK_T(label, torch::kBFloat16);
  CHECK_T(dxhat, torch::kBFloat16);
  CHECK_T(loss_sum, torch::kFloat32);
  TORCH_CHECK(xhat.dim() == 2 && label.numel() == xhat.numel() && dxhat.numel() == xhat.numel());
  const c10::cuda::CUDAGuard guard(xhat.device());
  check_cuda(lmsae::mse_loss_grad_launch(xhat.data_ptr<float>(), reinterpret_cast<const __nv_bfloat16*>(label.data_ptr()),
                                         opt_ptr<const float>(bias), opt_ptr<const float>(row_weight),
                                         (int)xhat.size(0), (int)xhat.size(1), (float)grad_scale,
                                         reinterpret_cast<__nv_bfloat16*>(dxhat.data_ptr()), loss_sum.data_ptr<float>(),
                                         opt_ptr<float>(row_loss), at::cuda::getCurrentCUDAStream()),
             "mse_loss_grad launch");
}

void auxk_loss_grad(const Tensor& xhat, const Tensor& aux_rec, const Tensor& label, const c10::optional<Tensor>& bias,
                    const c10::optional<Tensor>& row_weight, double grad_scale, double alpha, const Tensor& g_main,
                    const Tensor& g_aux, const Tensor& loss_sum, const Tensor& aux_sum,
                    const c10::optional<Tensor>& alpha_factor) {
  if (alpha_factor.has_value()) { CHECK_T(*alpha_factor, torch::kFloat32); TORCH_CHECK(alpha_factor->numel() == 1); }
  CHECK_T(xhat, torch::kFloat32);
  CHECK_T(aux_rec, torch::kFloat32);
  CHECK_T(label, torch::kBFloat16);
  CHECK_T(g_main, torch::kBFloat16);
  CHECK_T(g_aux, torch::kBFloat16);
  CHECK_T(loss_sum, torch::kFloat32);
  CHECK_T(aux_sum, torch::kFloat32);
  TORCH_CHECK(xhat.dim() == 2 && aux_rec.sizes() == xhat.sizes() && label.numel() == xhat.numel() &&
              g_main.numel() == xhat.numel() && g_aux.numel() == xhat.numel());
  const c10::cuda::CUDAGuard guard(xhat.device());
  check_cuda(lmsae::auxk_loss_grad_launch(xhat.data_ptr<float>(), aux_rec.data_ptr<float>(),
                                          reinterpret_cast<const __nv_bfloat16*>(label.data_ptr()), opt_ptr<const float>(bias),
                                          opt_ptr<const float>(row_weight), (int)xhat.size(0), (int)xhat.size(1),
                                          (float)grad_scale, (float)alpha, opt_ptr<const float>(alpha_factor),
                                          reinterpret_cast<__nv_bfloat16*>(g_main.data_ptr()),
                                          reinterpret_cast<__nv_bfloat16*>(g_aux.data_ptr()), loss_sum.data_ptr<float>(),
                                          aux_sum.data_ptr<float>(), at::cuda::getCurrentCUDAStream()),
             "auxk_loss_grad launch");
}

void csc_build(const Tensor& idx, int64_t F, const Tensor& counts, const Tensor& offsets, const Tensor& cursor,
               const Tensor& entries, const Tensor& block_sums) {
  CHECK_T(idx, torch::kInt32);
  CHECK_T(counts, torch::kInt32);
  CHECK_T(offsets, torch::kInt32);
  CHECK_T(cursor, torch::kInt32);
  CHECK_T(entries, torch::kInt32);
  CHECK_T(block_sums, torch::kInt32);
  TORCH_CHECK(counts.numel() >= F && offsets.numel() >= F + 1 && cursor.numel() >= F && entries.numel() >= idx.numel());
  TORCH_CHECK(block_sums.numel() >= (F + 4095) / 4096, "block_sums needs one int per 4096 features");
  const c10::cuda::CUDAGuard guard(idx.device());
  check_cuda(lmsae::csc_build_launch(idx.data_ptr<int>(), idx.numel(), (int)F, counts.data_ptr<int>(),
                                     offsets.data_ptr<int>(), cursor.data_ptr<int>(), entries.data_ptr<int>(),
                                     block_sums.data_ptr<int>(), at::cuda::getCurrentCUDAStream()),
             "csc_build launch");
}

lmsae::AdamHyper make_hyper(double lr, double beta1, double beta2, double eps, int64_t step) {
  lmsae::AdamHyper h;
  h.lr = (float)lr;
  h.beta1 = (float)beta1;
  h.beta2 = (float)beta2;
  h.eps = (float)eps;
  h.bias_correction1 = (float)(1.0 - std::pow(beta1, (double)step));
  h.bias_correction2_sqrt = (float)std::sqrt(1.0 - std::pow(beta2, (double)step));
  return h;
}

void sparse_grad_adam(const Tensor& offsets, const Tensor& entries, const Tensor& act, const Tensor& dact,
                      const Tensor& x, const Tensor& dxhat, const c10::optional<Tensor>& WD_o, const c10::optional<Tensor>& mD_o,
                      const c10::optional<Tensor>& vD_o, const c10::optional<Tensor>& WD_bf16_o,
                      const c10::optional<Tensor>& WE_o, const c10::optional<Tensor>& mE_o, const c10::optional<Tensor>& vE_o,
                      const c10::optional<Tensor>& WE_bf16_o, const c10::optional<Tensor>& bE, const c10::optional<Tensor>& mbE,
                      const c10::optional<Tensor>& vbE, const c10::optional<Tensor>& dec_norm,
                      const c10::optional<Tensor>& grad_mul, const c10::optional<Tensor>& grad_sq_sum, double lr,
                      double beta1, double beta2, double eps, int64_t step, bool update, int64_t f_begin,
                      int64_t f_end, int64_t ctas_per_sm, const c10::optional<Tensor>& dxhat_aux, int64_t k_main,
                      const c10::optional<Tensor>& gD_out, const c10::optional<Tensor>& gE_out,
                      const c10::optional<Tensor>& status, int64_t state_f0, const std::vector<int64_t>& pub_table,
                      const std::vector<int64_t>& pub_offsets, int64_t pub_epoch,
                      const c10::optional<Tensor>& pub_done, const c10::optional<Tensor>& extra_row,
                      const c10::optional<Tensor>& extra_gD, const c10::optional<Tensor>& extra_gE,
                      const c10::optional<Tensor>& extra_gb, const c10::optional<Tensor>& wd_self_scale,
                      const c10::optional<Tensor>& norm_sq_accum) {
  // one-sided launches: the decoder group (WD, mD, vD, WD_bf16) or the encoder group (WE, mE, vE, WE_bf16) may be absent
  const bool has_d = WD_o.has_value(), has_e = WE_o.has_value();
  TORCH_CHECK(has_d || has_e, "at least one of the decoder / encoder groups must be given");
  TORCH_CHECK(!has_d || (mD_o.has_value() && vD_o.has_value() && WD_bf16_o.has_value()), "decoder group incomplete");
  TORCH_CHECK(!has_e || (mE_o.has_value() && vE_o.has_value() && WE_bf16_o.has_value()), "encoder group incomplete");
  const Tensor& any_w = has_d ? *WD_o : *WE_o;
  const Tensor& WD = has_d ? *WD_o : any_w; const Tensor& mD = has_d ? *mD_o : any_w; const Tensor& vD = has_d ? *vD_o : any_w;
  const Tensor& WE = has_e ? *WE_o : any_w; const Tensor& mE = has_e ? *mE_o : any_w; const Tensor& vE = has_e ? *vE_o : any_w;
  const Tensor& WD_bf16 = has_d ? *WD_bf16_o : *WE_bf16_o;
  const Tensor& WE_bf16 = has_e ? *WE_bf16_o : *WD_bf16_o;
  CHECK_T(offsets, torch::kInt32);
  CHECK_T(entries, torch::kInt32);
  CHECK_T(act, torch::kFloat32);
  CHECK_T(dact, torch::kFloat32);
  CHECK_T(x, torch::kBFloat16);
  CHECK_T(dxhat, torch::kBFloat16);
  CHECK_T(WD, torch::kFloat32); CHECK_T(mD, torch::kFloat32); CHECK_T(vD, torch::kFloat32); CHECK_T(WD_bf16, torch::kBFloat16);
  CHECK_T(WE, torch::kFloat32); CHECK_T(mE, torch::kFloat32); CHECK_T(vE, torch::kFloat32); CHECK_T(WE_bf16, torch::kBFloat16);
  TORCH_CHECK(WD.dim() == 2 && WE.sizes() == WD.sizes() && act.dim() == 2 && dact.sizes() == act.sizes());
  const c10::cuda::CUDAGuard guard(WD.device());
  lmsae::GradAdamParams p{};
  p.F = (int)WD.size(0);
  p.d = (int)WD.size(1);
  p.k = (int)act.size(1);
  p.n_rows = (int)x.size(0);
  p.n_codes = act.numel();
  TORCH_CHECK(offsets.numel() >= p.F + 1 && x.size(1) == p.d && dxhat.sizes() == x.sizes());
  p.f_begin = (int)f_begin;
  p.f_end = f_end < 0 ? p.F : (int)f_end;
  TORCH_CHECK(0 <= p.f_begin && p.f_begin <= p.f_end && p.f_end <= p.F, "feature range out of bounds");
  p.state_f0 = (int)state_f0;
  TORCH_CHECK(0 <= p.state_f0 && p.state_f0 <= p.f_begin, "state_f0 must not exceed the first updated row");
  // state and shadow tensors are only touched when the update is applied; with state_f0 > 0 the moments cover rows
  // [state_f0, f_end) at least
  if (update) {
    for (const Tensor* t : {&WD_bf16, &WE_bf16}) TORCH_CHECK(t->numel() == WD.numel());
    for (const Tensor* t : {&mD, &vD, &mE, &vE})
      TORCH_CHECK(t->numel() >= (int64_t)(p.f_end - p.state_f0) * p.d, "moment arrays too small for the updated rows");
  }
  p.offsets = offsets.data_ptr<int>();
  p.entries = entries.data_ptr<int>();
  p.act = act.data_ptr<float>();
  p.dact = dact.data_ptr<float>();
  p.x = reinterpret_cast<const __nv_bfloat16*>(x.data_ptr());
  p.dxhat = reinterpret_cast<const __nv_bfloat16*>(dxhat.data_ptr());
  if (has_d) {
    p.WD = WD.data_ptr<float>(); p.mD = mD.data_ptr<float>(); p.vD = vD.data_ptr<float>();
    p.WD_bf16 = reinterpret_cast<__nv_bfloat16*>(WD_bf16.data_ptr());
  }
  if (has_e) {
    p.WE = WE.data_ptr<float>(); p.mE = mE.data_ptr<float>(); p.vE = vE.data_ptr<float>();
    p.WE_bf16 = reinterpret_cast<__nv_bfloat16*>(WE_bf16.data_ptr());
  }
  if (norm_sq_accum.has_value()) { CHECK_T(*norm_sq_accum, torch::kFloat32); TORCH_CHECK(norm_sq_accum->numel() == WD.size(0)); }
  p.norm_sq_accum = opt_ptr<float>(norm_sq_accum);
  if (bE.has_value()) {
    TORCH_CHECK(mbE.has_value() && vbE.has_value());
    CHECK_T(*bE, torch::kFloat32); CHECK_T(*mbE, torch::kFloat32); CHECK_T(*vbE, torch::kFloat32);
    TORCH_CHECK(bE->numel() == p.F && mbE->numel() >= p.f_end - p.state_f0 && vbE->numel() >= p.f_end - p.state_f0);
  }
  p.bE = opt_ptr<float>(bE); p.mbE = opt_ptr<float>(mbE); p.vbE = opt_ptr<float>(vbE);
  if (dec_norm.has_value()) { CHECK_T(*dec_norm, torch::kFloat32); TORCH_CHECK(dec_norm->numel() == p.F); }
  p.dec_norm = opt_ptr<float>(dec_norm);
  p.grad_mul = opt_ptr<const float>(grad_mul);
  p.grad_sq_sum = opt_ptr<float>(grad_sq_sum);
  p.h = make_hyper(lr, beta1, beta2, eps, step);
  p.update = update ? 1 : 0;
  p.ctas_per_sm = (int)ctas_per_sm;
  // warp-per-row kernel for short rows unless LMSAE_ADAM_ROWWARP=0 (read once)
  static const int rowwarp = [] { const char* e = std::getenv("LMSAE_ADAM_ROWWARP"); return (e != nullptr && e[0] == '0') ? 0 : 1; }();
  p.use_rowwarp = rowwarp;
  if (status.has_value()) { CHECK_T(*status, torch::kInt32); }
  p.status = opt_ptr<const int>(status);
  if (wd_self_scale.has_value()) { CHECK_T(*wd_self_scale, torch::kFloat32); TORCH_CHECK(wd_self_scale->numel() == p.F); }
  p.wd_self_scale = opt_ptr<const float>(wd_self_scale);
  if (extra_row.has_value()) {
    // dense gradient rows for one or both matrices (a side without rows passes nothing)
    TORCH_CHECK(extra_gD.has_value() || extra_gE.has_value(), "extra gradient rows need at least one matrix");
    CHECK_T(*extra_row, torch::kInt32);
    TORCH_CHECK(extra_row->numel() == p.F, "extra_row: one entry per feature");
    int64_t n_extra = -1;
    for (const auto* g : {&extra_gD, &extra_gE}) {
      if (!g->has_value()) continue;
      CHECK_T(**g, torch::kFloat32);
      TORCH_CHECK((*g)->dim() == 2 && (*g)->size(1) == p.d && (n_extra < 0 || (*g)->size(0) == n_extra), "extra gradient rows must be [rows, d]");
      n_extra = (*g)->size(0);
    }
    p.extra_row = extra_row->data_ptr<int>();
    p.extra_gD = opt_ptr<const float>(extra_gD);
    p.extra_gE = opt_ptr<const float>(extra_gE);
    if (extra_gb.has_value()) { CHECK_T(*extra_gb, torch::kFloat32); TORCH_CHECK(extra_gb->numel() == n_extra); }
    p.extra_gb = opt_ptr<const float>(extra_gb);
  }
  if (!pub_table.empty()) {
    p.pub = make_peer_table(pub_table);
    p.n_pub = p.pub.world;
    TORCH_CHECK(pub_offsets.size() == 4 && pub_done.has_value(), "publication needs four offsets and a counter");
    CHECK_T(*pub_done, torch::kInt32);
    p.pub_wd_off = pub_offsets[0]; p.pub_we_off = pub_offsets[1]; p.pub_norm_off = pub_offsets[2]; p.pub_be_off = pub_offsets[3];
    for (int64_t o : pub_offsets) TORCH_CHECK(o % 16 == 0, "publication offsets must be 16-byte aligned");
    p.pub_epoch = (uint32_t)pub_epoch;
    p.pub_done = reinterpret_cast<unsigned*>(pub_done->data_ptr<int>());
  }
  if (dxhat_aux.has_value()) { CHECK_T(*dxhat_aux, torch::kBFloat16); TORCH_CHECK(dxhat_aux->sizes() == dxhat.sizes()); }
  p.dxhat_aux = dxhat_aux.has_value() ? reinterpret_cast<const __nv_bfloat16*>(dxhat_aux->data_ptr()) : nullptr;
  p.k_main = (int)k_main;
  for (const auto* t : {&gD_out, &gE_out}) {
    if (t->has_value()) { CHECK_T(**t, torch::kFloat32); TORCH_CHECK((*t)->numel() == WD.numel()); }
  }
  p.gD_out = opt_ptr<float>(gD_out);
  p.gE_out = opt_ptr<float>(gE_out);
  check_cuda(lmsae::sparse_grad_adam_launch(p, at::cuda::getCurrentCUDAStream()), "sparse_grad_adam launch");
}

void colsum_bf16(const Tensor& a, const Tensor& out) {
  CHECK_T(a, torch::kBFloat16);
  CHECK_T(out, torch::kFloat32);
  TORCH_CHECK(a.dim() == 2 && out.numel() == a.size(1));
  const c10::cuda::CUDAGuard guard(a.device());
  check_cuda(lmsae::colsum_bf16_launch(reinterpret_cast<const __nv_bfloat16*>(a.data_ptr()), (int)a.size(0),
                                       (int)a.size(1), out.data_ptr<float>(), at::cuda::getCurrentCUDAStream()),
             "colsum_bf16 launch");
}

void adam_flat(const Tensor& p, const Tensor& g, const Tensor& m, const Tensor& v, const c10::optional<Tensor>& grad_mul,
               const c10::optional<Tensor>& shadow, const c10::optional<Tensor>& grad_sq_sum, double lr, double beta1,
               double beta2, double eps, int64_t step, bool update, const c10::optional<Tensor>& status) {
  CHECK_T(p, torch::kFloat32); CHECK_T(g, torch::kFloat32); CHECK_T(m, torch::kFloat32); CHECK_T(v, torch::kFloat32);
  TORCH_CHECK(g.numel() == p.numel() && m.numel() == p.numel() && v.numel() == p.numel());
  if (shadow.has_value()) { CHECK_T(*shadow, torch::kBFloat16); TORCH_CHECK(shadow->numel() == p.numel()); }
  const c10::cuda::CUDAGuard guard(p.device());
  check_cuda(lmsae::adam_flat_launch(p.data_ptr<float>(), g.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
                                     p.numel(), make_hyper(lr, beta1, beta2, eps, step), opt_ptr<const float>(grad_mul),
                                     opt_ptr<__nv_bfloat16>(shadow), opt_ptr<float>(grad_sq_sum), update ? 1 : 0,
                                     opt_ptr<const int>(status), at::cuda::getCurrentCUDAStream()),
             "adam_flat launch");
}

void row_norm_shadow(const Tensor& W, const c10::optional<Tensor>& norm, const c10::optional<Tensor>& shadow) {
  CHECK_T(W, torch::kFloat32);
  TORCH_CHECK(W.dim() == 2);
  if (norm.has_value()) { CHECK_T(*norm, torch::kFloat32); TORCH_CHECK(norm->numel() == W.size(0)); }
  if (shadow.has_value()) { CHECK_T(*shadow, torch::kBFloat16); TORCH_CHECK(shadow->numel() == W.numel()); }
  const c10::cuda::CUDAGuard guard(W.device());
  check_cuda(lmsae::row_norm_shadow_launch(W.data_ptr<float>(), (int)W.size(0), (int)W.size(1), opt_ptr<float>(norm),
                                           opt_ptr<__nv_bfloat16>(shadow), at::cuda::getCurrentCUDAStream()),
             "row_norm_shadow launch");
}

// ---- JumpReLU --------------------------------------------------------------------------------------
// forward: returns y; backward (dy given): returns dx and accumulates d log_theta into `dlog` (fp32 [P], zeroed here).
Tensor jumprelu(const Tensor& x, const Tensor& log_theta, const c10::optional<Tensor>& dy, const c10::optional<Tensor>& dlog,
                double window) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && log_theta.is_contiguous(), "jumprelu needs contiguous CUDA tensors");
  TORCH_CHECK(x.scalar_type() == log_theta.scalar_type(), "x and log_theta must share a dtype");
  const int dtype = x.scalar_type() == torch::kFloat32 ? 0 : (x.scalar_type() == torch::kBFloat16 ? 1 : -1);
  TORCH_CHECK(dtype >= 0, "jumprelu supports fp32 and bf16");
  const int64_t P = log_theta.numel();
  TORCH_CHECK(P > 0 && P % 4 == 0 && x.numel() % P == 0, "thresholds must cover the trailing dimensions of x (multiple of 4)");
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor out = torch::empty_like(x);
  const bool bwd = dy.has_value();
  float* dlog_ptr = nullptr;
  if (bwd) {
    TORCH_CHECK(dy->is_contiguous() && dy->scalar_type() == x.scalar_type() && dy->numel() == x.numel());
    TORCH_CHECK(dlog.has_value() && dlog->scalar_type() == torch::kFloat32 && dlog->numel() == P && dlog->is_contiguous());
    dlog_ptr = dlog->data_ptr<float>();
  }
  check_cuda(lmsae::jumprelu_launch(dtype, x.data_ptr(), log_theta.data_ptr(), bwd ? dy->data_ptr() : nullptr, out.data_ptr(),
                                    dlog_ptr, x.numel(), (int)P, (float)window, bwd ? 1 : 0, at::cuda::getCurrentCUDAStream()),
             "jumprelu launch");
  return out;
}

// ---- attention ---------------------------------------------------------------------------------------------
// q, k: bf16 [batch, seq, heads, d_qk]; vt: bf16 [batch, heads, d_v, seq] (values transposed, keys contiguous);
// out: bf16 [batch, seq, heads, d_v]; lse: fp32 [batch, heads, seq] or absent. Causal.
void attn_fwd(const Tensor& q, const Tensor& k, const Tensor& vt, const Tensor& out, const c10::optional<Tensor>& lse,
              double scale, const Tensor& status) {
  CHECK_T(q, torch::kBFloat16);
  CHECK_T(k, torch::kBFloat16);
  CHECK_T(vt, torch::kBFloat16);
  CHECK_T(out, torch::kBFloat16);
  CHECK_T(status, torch::kInt32);
  TORCH_CHECK(q.dim() == 4 && k.sizes() == q.sizes() && vt.dim() == 4, "q, k [b, s, h, dqk]; vt [b, h, dv, s]");
  lmsae::AttnParams p{};
  p.batch = (int)q.size(0);
  p.seq = (int)q.size(1);
  p.heads = (int)q.size(2);
  p.dqk = (int)q.size(3);
  p.dv = (int)vt.size(2);
  TORCH_CHECK(vt.size(0) == p.batch && vt.size(1) == p.heads && vt.size(3) == p.seq, "vt must be [b, h, dv, s]");
  TORCH_CHECK(out.dim() == 4 && out.size(0) == p.batch && out.size(1) == p.seq && out.size(2) == p.heads && out.size(3) == p.dv,
              "out must be [b, s, h, dv]");
  const int dvc = lmsae::attn_fwd_value_chunk(p.dqk, p.dv);
  TORCH_CHECK(dvc != 0 && (p.dqk == 64 || p.dqk == 128) && p.seq % 8 == 0, "attn_fwd: d_qk in {64, 128}, d_v % 64 == 0, seq % 8 == 0");
  if (lse.has_value()) {
    CHECK_T(*lse, torch::kFloat32);
    TORCH_CHECK(lse->numel() == (int64_t)p.batch * p.heads * p.seq, "lse must be [b, h, s]");
  }
  p.scale_log2 = (float)(scale * 1.4426950408889634);
  p.out = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  p.lse = opt_ptr<float>(lse);
  p.status = status.data_ptr<int>();
  const c10::cuda::CUDAGuard guard(q.device());
  const CUtensorMap tq = make_bf16_tile_map(q.data_ptr(), (int64_t)p.batch * p.seq, (int64_t)p.heads * p.dqk, 128);
  const CUtensorMap tk = make_bf16_tile_map(k.data_ptr(), (int64_t)p.batch * p.seq, (int64_t)p.heads * p.dqk, 128);
  const CUtensorMap tvt = make_bf16_tile_map(vt.data_ptr(), (int64_t)p.batch * p.heads * p.dv, p.seq, dvc);
  check_cuda(lmsae::attn_fwd_launch(tq, tk, tvt, p, at::cuda::getCurrentCUDAStream()), "attn_fwd launch");
}

// q, k, v, dout: bf16 [b, s, h, *]; kt, qt: bf16 [b, h, dqk, s]; dot: bf16 [b, h, dv, s]; lse, delta: fp32 [b, h, s];
// dq, dk: fp32 [b, s, h, dqk]; dv: fp32 [b, s, h, dv].
void attn_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& dout, const Tensor& qt, const Tensor& kt,
              const Tensor& dot, const Tensor& lse, const Tensor& delta, const Tensor& dq, const Tensor& dk, const Tensor& dv,
              double scale, const Tensor& status) {
  for (const Tensor* t : {&q, &k, &v, &dout, &qt, &kt, &dot}) { CHECK_T(*t, torch::kBFloat16); }
  for (const Tensor* t : {&lse, &delta, &dq, &dk, &dv}) { CHECK_T(*t, torch::kFloat32); }
  CHECK_T(status, torch::kInt32);
  lmsae::AttnBwdParams p{};
  p.batch = (int)q.size(0);
  p.seq = (int)q.size(1);
  p.heads = (int)q.size(2);
  p.dqk = (int)q.size(3);
  p.dv = (int)v.size(3);
  const int64_t bs = (int64_t)p.batch * p.seq, bh = (int64_t)p.batch * p.heads;
  TORCH_CHECK(k.sizes() == q.sizes() && dq.sizes() == q.sizes() && dk.sizes() == q.sizes(), "q, k, dq, dk: [b, s, h, dqk]");
  TORCH_CHECK(v.size(0) == p.batch && v.size(1) == p.seq && v.size(2) == p.heads && dout.sizes() == v.sizes() && dv.sizes() == v.sizes(),
              "v, dout, dv: [b, s, h, dv]");
  TORCH_CHECK(qt.numel() == q.numel() && kt.numel() == q.numel() && qt.size(3) == p.seq && kt.size(3) == p.seq &&
                  dot.numel() == v.numel() && dot.size(3) == p.seq, "qt, kt: [b, h, dqk, s]; dot: [b, h, dv, s]");
  TORCH_CHECK(lse.numel() == bh * p.seq && delta.numel() == bh * p.seq, "lse, delta: [b, h, s]");
  const int dvc = lmsae::attn_value_chunk(p.dv);
  TORCH_CHECK(dvc != 0 && (p.dqk == 64 || p.dqk == 128) && p.seq % 8 == 0, "attn_bwd: d_qk in {64, 128}, d_v % 64 == 0, seq % 8 == 0");
  p.scale = (float)scale;
  p.scale_log2 = (float)(scale * 1.4426950408889634);
  p.lse = lse.data_ptr<float>();
  p.delta = delta.data_ptr<float>();
  p.dq = dq.data_ptr<float>();
  p.dk = dk.data_ptr<float>();
  p.dv_out = dv.data_ptr<float>();
  p.status = status.data_ptr<int>();
  const c10::cuda::CUDAGuard guard(q.device());
  const CUtensorMap mq = make_bf16_tile_map(q.data_ptr(), bs, (int64_t)p.heads * p.dqk, 128);
  const CUtensorMap mk = make_bf16_tile_map(k.data_ptr(), bs, (int64_t)p.heads * p.dqk, 128);
  const CUtensorMap mv = make_bf16_tile_map(v.data_ptr(), bs, (int64_t)p.heads * p.dv, 128);
  const CUtensorMap mdo = make_bf16_tile_map(dout.data_ptr(), bs, (int64_t)p.heads * p.dv, 128);
  const CUtensorMap mqt = make_bf16_tile_map(qt.data_ptr(), bh * p.dqk, p.seq, p.dqk);
  const CUtensorMap mkt = make_bf16_tile_map(kt.data_ptr(), bh * p.dqk, p.seq, p.dqk);
  const CUtensorMap mdot = make_bf16_tile_map(dot.data_ptr(), bh * p.dv, p.seq, dvc);
  const CUtensorMap maps_dq[5] = {mq, mk, mkt, mdo, mv};
  const CUtensorMap maps_dkv[6] = {mk, mq, mqt, mv, mdo, mdot};
  check_cuda(lmsae::attn_bwd_launch(maps_dq, maps_dkv, p, at::cuda::getCurrentCUDAStream()), "attn_bwd launch");
}

// ---- selection / compaction ----------------------------------------------------------------------------
int dtype_code(const Tensor& t) {
  if (t.scalar_type() == torch::kFloat32) return 0;
  if (t.scalar_type() == torch::kBFloat16) return 1;
  TORCH_CHECK(false, "fp32 or bf16 expected");
  return -1;
}

int64_t radix_hi_bins() { return lmsae::radix_hi_bins(); }

// x: contiguous, viewed as [A, S, N]; level 0 fills hist[radix_hi_bins()], level 1 fills hist[65536] with the members of
// bin sel[0]. hist is uint32 storage handed in as int32.
// floor (fp32, one element, level 0 only): count only values of at least *floor. need (int64 [4]): run only if need[3] != 0.
void radix_hist(const Tensor& x, int64_t A, int64_t S, int64_t N, int64_t s, int64_t level, const c10::optional<Tensor>& sel,
                const Tensor& hist, const c10::optional<Tensor>& floor, const c10::optional<Tensor>& need) {
  if (floor.has_value()) { CHECK_T(*floor, torch::kFloat32); TORCH_CHECK(level == 0 && floor->numel() >= 1, "floor: one fp32 value, first level only"); }
  if (need.has_value()) { CHECK_T(*need, torch::kInt64); TORCH_CHECK(need->numel() >= 4, "need: int64 [4]"); }
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.numel() == A * S * N, "x must be a contiguous [A, S, N] array");
  CHECK_T(hist, torch::kInt32);
  TORCH_CHECK(hist.numel() >= (level == 0 ? lmsae::radix_hi_bins() : 65536), "histogram too small");
  if (level == 1) {
    TORCH_CHECK(sel.has_value(), "level 1 needs the level-0 pick");
    CHECK_T(*sel, torch::kInt64);
  }
  const c10::cuda::CUDAGuard guard(x.device());
  check_cuda(lmsae::radix_hist_launch(dtype_code(x), x.data_ptr(), A, S, N, s, (int)level,
                                      level == 1 ? reinterpret_cast<const long long*>(sel->data_ptr<int64_t>()) : nullptr,
                                      reinterpret_cast<unsigned*>(hist.data_ptr<int>()), opt_ptr<float>(floor),
                                      need.has_value() ? reinterpret_cast<const long long*>(need->data_ptr<int64_t>()) : nullptr,
                                      at::cuda::getCurrentCUDAStream()),
             "radix_hist launch");
}

void radix_pick(const Tensor& hist, int64_t nbins, int64_t k, const c10::optional<Tensor>& sel_in, int64_t level,
                const Tensor& sel_out, const c10::optional<Tensor>& thr, const c10::optional<Tensor>& need) {
  CHECK_T(hist, torch::kInt32);
  CHECK_T(sel_out, torch::kInt64);
  TORCH_CHECK(hist.numel() >= nbins && sel_out.numel() >= 4, "radix_pick: buffers too small");
  if (need.has_value()) { CHECK_T(*need, torch::kInt64); TORCH_CHECK(need->numel() >= 4, "need: int64 [4]"); }
  if (thr.has_value()) { CHECK_T(*thr, torch::kFloat32); }
  if (sel_in.has_value()) { CHECK_T(*sel_in, torch::kInt64); }
  const c10::cuda::CUDAGuard guard(hist.device());
  check_cuda(lmsae::radix_pick_launch(reinterpret_cast<const unsigned*>(hist.data_ptr<int>()), (int)nbins, k,
                                      sel_in.has_value() ? reinterpret_cast<const long long*>(sel_in->data_ptr<int64_t>()) : nullptr,
                                      (int)level, reinterpret_cast<long long*>(sel_out.data_ptr<int64_t>()),
                                      opt_ptr<float>(thr),
                                      need.has_value() ? reinterpret_cast<const long long*>(need->data_ptr<int64_t>()) : nullptr,
                                      at::cuda::getCurrentCUDAStream()),
             "radix_pick launch");
}

// out = where(x >= thr[segment], x, 0) for x viewed as [A, S, N]
Tensor threshold_mask(const Tensor& x, const Tensor& thr, int64_t A, int64_t S, int64_t N) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.numel() == A * S * N, "x must be a contiguous [A, S, N] array");
  CHECK_T(thr, torch::kFloat32);
  TORCH_CHECK(thr.numel() == S, "one threshold per segment");
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor out = torch::empty_like(x);
  check_cuda(lmsae::threshold_mask_launch(dtype_code(x), x.data_ptr(), thr.data_ptr<float>(), A, S, N, out.data_ptr(),
                                          at::cuda::getCurrentCUDAStream()),
             "threshold_mask launch");
  return out;
}

// x [B, N] -> idx / val [B, cap] (both optional: count only) and nnz [B] (optional). seg_counts int32 [B, 8, 2]
// (optional): written by a counting call, read by a compacting call of the same matrix and thresholds, which then
// skips its own counting pass.
void row_compact(const Tensor& x, const c10::optional<Tensor>& idx, const c10::optional<Tensor>& val,
                 const c10::optional<Tensor>& nnz, const c10::optional<Tensor>& thr, const c10::optional<Tensor>& col_div,
                 const c10::optional<Tensor>& ties, const c10::optional<Tensor>& tie_quota,
                 const c10::optional<Tensor>& col_thr, const c10::optional<Tensor>& seg_counts) {
  if (seg_counts.has_value()) { CHECK_T(*seg_counts, torch::kInt32); TORCH_CHECK(seg_counts->numel() == x.size(0) * 16, "seg_counts must be [B, 8, 2]"); }
  if (col_thr.has_value()) { CHECK_T(*col_thr, torch::kFloat32); TORCH_CHECK(col_thr->numel() == x.size(1) && !thr.has_value(), "col_thr: one per column, instead of thr"); }
  if (ties.has_value()) { CHECK_T(*ties, torch::kInt32); TORCH_CHECK(ties->numel() == x.size(0) && thr.has_value(), "ties: [B], with thr"); }
  if (tie_quota.has_value()) { CHECK_T(*tie_quota, torch::kInt32); TORCH_CHECK(tie_quota->numel() == x.size(0) && thr.has_value(), "tie_quota: [B], with thr"); }
  if (thr.has_value()) { CHECK_T(*thr, torch::kFloat32); TORCH_CHECK(thr->numel() >= 1); }
  if (col_div.has_value()) { CHECK_T(*col_div, torch::kFloat32); TORCH_CHECK(col_div->numel() == x.size(1), "one divisor per column"); }
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.dim() == 2, "x must be a contiguous CUDA matrix");
  int cap = 0;
  if (idx.has_value()) {
    CHECK_T(*idx, torch::kInt32);
    TORCH_CHECK(val.has_value(), "idx and val come together");
    CHECK_T(*val, torch::kFloat32);
    TORCH_CHECK(idx->dim() == 2 && idx->size(0) == x.size(0) && val->sizes() == idx->sizes(), "idx / val must be [B, cap]");
    cap = (int)idx->size(1);
  }
  if (nnz.has_value()) {
    CHECK_T(*nnz, torch::kInt32);
    TORCH_CHECK(nnz->numel() == x.size(0), "nnz must be [B]");
  }
  const c10::cuda::CUDAGuard guard(x.device());
  check_cuda(lmsae::row_compact_launch(dtype_code(x), x.data_ptr(), (int)x.size(0), x.size(1), cap, opt_ptr<int>(idx),
                                       opt_ptr<float>(val), opt_ptr<int>(nnz), opt_ptr<float>(thr), opt_ptr<float>(col_div),
                                       opt_ptr<int>(ties), opt_ptr<int>(tie_quota), opt_ptr<float>(col_thr),
                                       opt_ptr<int>(seg_counts), at::cuda::getCurrentCUDAStream()),
             "row_compact launch");
}

// d theta[f] += window-weighted column sums of G / n (see select_ops.cu); G, S bf16 [B, F], n / theta / dtheta fp32 [F].
void jumprelu_window_grad(const Tensor& G, const Tensor& S, const Tensor& n, const Tensor& theta, double window,
                          double add_per_hit, const Tensor& dtheta) {
  CHECK_T(G, torch::kBFloat16);
  CHECK_T(S, torch::kBFloat16);
  CHECK_T(n, torch::kFloat32);
  CHECK_T(theta, torch::kFloat32);
  CHECK_T(dtheta, torch::kFloat32);
  TORCH_CHECK(G.dim() == 2 && S.sizes() == G.sizes() && n.numel() == G.size(1) && theta.numel() == G.size(1) && dtheta.numel() == G.size(1));
  const c10::cuda::CUDAGuard guard(G.device());
  check_cuda(lmsae::jumprelu_window_grad_launch(reinterpret_cast<const __nv_bfloat16*>(G.data_ptr()),
                                                reinterpret_cast<const __nv_bfloat16*>(S.data_ptr()), (int)G.size(0), (int)G.size(1),
                                                n.data_ptr<float>(), theta.data_ptr<float>(), (float)window, (float)add_per_hit, dtheta.data_ptr<float>(),
                                                at::cuda::getCurrentCUDAStream()),
             "jumprelu_window_grad launch");
}

// Rotary embedding (sin_sign = 1) or its inverse (-1) of xa and xb [batch x seq, heads, width] bf16 into oa and ob;
// cos / sin fp32 [>= seq, rd] (see rotary.cu).
void rotary_pair(const Tensor& xa, const Tensor& xb, const Tensor& oa, const Tensor& ob, const Tensor& cos_t, const Tensor& sin_t,
                 int64_t seq, bool adjacent, double sin_sign) {
  CHECK_T(xa, torch::kBFloat16);
  CHECK_T(xb, torch::kBFloat16);
  CHECK_T(oa, torch::kBFloat16);
  CHECK_T(ob, torch::kBFloat16);
  CHECK_T(cos_t, torch::kFloat32);
  CHECK_T(sin_t, torch::kFloat32);
  TORCH_CHECK(xa.dim() == 3 && xb.sizes() == xa.sizes() && oa.sizes() == xa.sizes() && ob.sizes() == xa.sizes(), "rotary: shapes differ");
  TORCH_CHECK(cos_t.dim() == 2 && sin_t.sizes() == cos_t.sizes() && cos_t.size(0) >= seq, "rotary: tables must be [>= seq, rd]");
  const int64_t tokens = xa.size(0), heads = xa.size(1), width = xa.size(2), rd = cos_t.size(1);
  TORCH_CHECK(seq >= 1 && tokens % seq == 0, "rotary: tokens must be batch x seq");
  TORCH_CHECK(width % 8 == 0 && rd <= width && rd % (adjacent ? 8 : 16) == 0, "rotary: head width / rotary width not aligned");
  const c10::cuda::CUDAGuard guard(xa.device());
  check_cuda(lmsae::rotary_pair_launch(reinterpret_cast<const __nv_bfloat16*>(xa.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(xb.data_ptr()),
                                       reinterpret_cast<__nv_bfloat16*>(oa.data_ptr()), reinterpret_cast<__nv_bfloat16*>(ob.data_ptr()),
                                       cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), tokens, (int)seq, (int)heads, (int)width, (int)rd,
                                       adjacent ? 1 : 0, (float)sin_sign, at::cuda::getCurrentCUDAStream()),
             "rotary_pair launch");
}

void exclusive_scan(const Tensor& counts, const Tensor& offsets, const Tensor& block_sums) {
  CHECK_T(counts, torch::kInt32);
  CHECK_T(offsets, torch::kInt32);
  CHECK_T(block_sums, torch::kInt32);
  const int64_t n = counts.numel();
  TORCH_CHECK(offsets.numel() == n + 1 && block_sums.numel() >= (n + 4095) / 4096 && n < 2147483647LL, "exclusive_scan: sizes");
  const c10::cuda::CUDAGuard guard(counts.device());
  check_cuda(lmsae::exclusive_scan_launch(counts.data_ptr<int>(), (int)n, offsets.data_ptr<int>(), block_sums.data_ptr<int>(),
                                          at::cuda::getCurrentCUDAStream()),
             "exclusive_scan launch");
}

// out[pos[i], :] = cast(src[i, :]) where keep[i] != 0
void gather_rows_cast(const Tensor& src, const Tensor& keep, const Tensor& pos, const Tensor& out) {
  TORCH_CHECK(src.is_cuda() && src.is_contiguous() && src.dim() == 2 && out.is_cuda() && out.is_contiguous() && out.dim() == 2,
              "src / out must be contiguous CUDA matrices");
  CHECK_T(keep, torch::kInt32);
  CHECK_T(pos, torch::kInt32);
  TORCH_CHECK(keep.numel() == src.size(0) && pos.numel() >= src.size(0) && out.size(1) == src.size(1), "gather_rows_cast: sizes");
  const c10::cuda::CUDAGuard guard(src.device());
  check_cuda(lmsae::gather_rows_cast_launch(dtype_code(src), dtype_code(out), src.data_ptr(), keep.data_ptr<int>(),
                                            pos.data_ptr<int>(), src.size(0), (int)src.size(1), out.data_ptr(), out.size(0),
                                            at::cuda::getCurrentCUDAStream()),
             "gather_rows_cast launch");
}

// ---- cross-layer transcoder decoder fan-out ----------------------------------------------------------
// `weights[t]`: bf16 [t + 1, F, d]. idx / val: [B, K] codes c = s * F + f (-1 = empty).
lmsae::CltTable make_clt_table(const std::vector<Tensor>& weights, int64_t F, int64_t d) {
  TORCH_CHECK(!weights.empty() && (int)weights.size() <= lmsae::kMaxCltLayers, "1..64 target layers");
  lmsae::CltTable tab{};
  for (size_t t = 0; t < weights.size(); ++t) {
    const Tensor& w = weights[t];
    CHECK_T(w, torch::kBFloat16);
    TORCH_CHECK(w.dim() == 3 && w.size(0) == (int64_t)t + 1 && w.size(1) == F && w.size(2) == d,
                "decoder of target layer t must be [t + 1, F, d]");
    tab.W[t] = reinterpret_cast<const __nv_bfloat16*>(w.data_ptr());
  }
  return tab;
}

void clt_decode(const Tensor& idx, const Tensor& val, const std::vector<Tensor>& weights, const c10::optional<Tensor>& bias,
                const Tensor& out) {
  CHECK_T(idx, torch::kInt32);
  CHECK_T(val, torch::kFloat32);
  TORCH_CHECK(idx.dim() == 2 && val.sizes() == idx.sizes(), "idx / val must be [B, K]");
  const int64_t B = idx.size(0), K = idx.size(1), L = (int64_t)weights.size();
  const int64_t F = weights[0].size(1), d = weights[0].size(2);
  const c10::cuda::CUDAGuard guard(idx.device());
  const lmsae::CltTable tab = make_clt_table(weights, F, d);
  TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.numel() == L * B * d, "out must be [L, B, d]");
  float* o32 = nullptr;
  __nv_bfloat16* o16 = nullptr;
  if (out.scalar_type() == torch::kFloat32) o32 = out.data_ptr<float>();
  else if (out.scalar_type() == torch::kBFloat16) o16 = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  else TORCH_CHECK(false, "out must be fp32 or bf16");
  if (bias.has_value()) {
    CHECK_T(*bias, torch::kFloat32);
    TORCH_CHECK(bias->numel() == L * d, "bias must be [L, d]");
  }
  check_cuda(lmsae::clt_decode_launch(tab, idx.data_ptr<int>(), val.data_ptr<float>(), (int)B, (int)K, (int)L, (int)F, (int)d,
                                      opt_ptr<float>(bias), o32, o16, at::cuda::getCurrentCUDAStream()),
             "clt_decode launch");
}

void clt_dact(const Tensor& idx, const std::vector<Tensor>& weights, const Tensor& dy, const Tensor& dval) {
  CHECK_T(idx, torch::kInt32);
  CHECK_T(dy, torch::kBFloat16);
  CHECK_T(dval, torch::kFloat32);
  const int64_t B = idx.size(0), K = idx.size(1), L = (int64_t)weights.size();
  const int64_t F = weights[0].size(1), d = weights[0].size(2);
  TORCH_CHECK(dy.numel() == L * B * d && dval.numel() == B * K, "dy must be [L, B, d], dval [B, K]");
  const c10::cuda::CUDAGuard guard(idx.device());
  const lmsae::CltTable tab = make_clt_table(weights, F, d);
  check_cuda(lmsae::clt_dact_launch(tab, idx.data_ptr<int>(), (int)B, (int)K, (int)L, (int)F, (int)d,
                                    reinterpret_cast<const __nv_bfloat16*>(dy.data_ptr()), dval.data_ptr<float>(),
                                    at::cuda::getCurrentCUDAStream()),
             "clt_dact launch");
}

// `grads[t]`: fp32 [t + 1, F, d], zero-filled by the caller; rows of the codes that occur are overwritten.
void clt_wgrad(const Tensor& offsets, const Tensor& entries, const Tensor& act, const Tensor& dy,
               const std::vector<Tensor>& grads, int64_t B, int64_t K) {
  CHECK_T(offsets, torch::kInt32);
  CHECK_T(entries, torch::kInt32);
  CHECK_T(act, torch::kFloat32);
  CHECK_T(dy, torch::kBFloat16);
  const int64_t L = (int64_t)grads.size();
  TORCH_CHECK(L >= 1 && L <= lmsae::kMaxCltLayers, "1..64 target layers");
  const int64_t F = grads[0].size(1), d = grads[0].size(2);
  lmsae::CltGradTable tab{};
  for (int64_t t = 0; t < L; ++t) {
    const Tensor& g = grads[t];
    CHECK_T(g, torch::kFloat32);
    TORCH_CHECK(g.dim() == 3 && g.size(0) == t + 1 && g.size(1) == F && g.size(2) == d, "gradient of target layer t must be [t + 1, F, d]");
    tab.G[t] = g.data_ptr<float>();
  }
  TORCH_CHECK(offsets.numel() == L * F + 1 && act.numel() == B * K && entries.numel() >= B * K && dy.numel() == L * B * d,
              "clt_wgrad: inconsistent sizes");
  const c10::cuda::CUDAGuard guard(dy.device());
  check_cuda(lmsae::clt_wgrad_launch(tab, offsets.data_ptr<int>(), entries.data_ptr<int>(), act.data_ptr<float>(), (int)B, (int)K,
                                     (int)L, (int)F, (int)d, reinterpret_cast<const __nv_bfloat16*>(dy.data_ptr()),
                                     at::cuda::getCurrentCUDAStream()),
             "clt_wgrad launch");
}

// ---- peer-memory collectives -----------------------------------------------------------------------
void comm_push_candidates(const std::vector<int64_t>& table, const Tensor& val, const Tensor& idx, int64_t epoch,
                          const Tensor& done_counter) {
  CHECK_T(val, torch::kFloat32);
  CHECK_T(idx, torch::kInt32);
  CHECK_T(done_counter, torch::kInt32);
  TORCH_CHECK(val.dim() == 2 && idx.sizes() == val.sizes());
  const c10::cuda::CUDAGuard guard(val.device());
  check_cuda(lmsae::push_candidates_launch(make_peer_table(table), val.data_ptr<float>(), idx.data_ptr<int>(),
                                           (int)val.size(0), (int)val.size(1), (uint32_t)epoch,
                                           reinterpret_cast<unsigned*>(done_counter.data_ptr<int>()),
                                           at::cuda::getCurrentCUDAStream()),
             "push_candidates launch");
}

// Row all-to-all: `src` [n_local, row_bytes] (any dtype, contiguous), `dest` int64 [n_local] global positions.
void comm_shuffle_rows(const std::vector<int64_t>& table, const Tensor& src, const Tensor& dest, int64_t rows_per_rank,
                       int64_t recv_off, int64_t phase, int64_t epoch, const Tensor& done_counter) {
  CHECK_T(dest, torch::kInt64);
  CHECK_T(done_counter, torch::kInt32);
  TORCH_CHECK(src.is_cuda() && src.is_contiguous() && src.dim() >= 1 && dest.numel() == src.size(0));
  const int64_t row_bytes = src.size(0) > 0 ? (int64_t)(src.numel() / src.size(0)) * (int64_t)src.element_size() : 16;
  TORCH_CHECK(row_bytes % 16 == 0, "rows must be a multiple of 16 bytes");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(src.data_ptr()) % 16 == 0 && recv_off % 16 == 0, "16-byte alignment");
  const c10::cuda::CUDAGuard guard(src.device());
  check_cuda(lmsae::shuffle_rows_launch(make_peer_table(table), src.data_ptr(), reinterpret_cast<const long long*>(dest.data_ptr<int64_t>()),
                                        (int)src.size(0), (int)rows_per_rank, (int)row_bytes, (long long)recv_off, (int)phase,
                                        (uint32_t)epoch, reinterpret_cast<unsigned*>(done_counter.data_ptr<int>()),
                                        at::cuda::getCurrentCUDAStream()),
             "shuffle_rows launch");
}

// src [n, d] (fp32 / bf16) on the sending rank; keep / pos int32 [n] / [n + 1] or absent; the landing zone at
// `recv_off` holds `cap_rows` rows of d elements of `out_dtype` (0 = fp32, 1 = bf16).
void comm_bcast_rows(const std::vector<int64_t>& table, const Tensor& src, const c10::optional<Tensor>& keep,
                     const c10::optional<Tensor>& pos, int64_t out_dtype, int64_t recv_off, int64_t cap_rows, int64_t phase,
                     int64_t epoch, const Tensor& done_counter, bool use_multicast) {
  TORCH_CHECK(src.is_cuda() && src.is_contiguous() && src.dim() == 2, "src must be a contiguous CUDA matrix");
  CHECK_T(done_counter, torch::kInt32);
  if (keep.has_value()) {
    CHECK_T(*keep, torch::kInt32);
    TORCH_CHECK(pos.has_value() && keep->numel() == src.size(0), "keep and pos come together");
    CHECK_T(*pos, torch::kInt32);
    TORCH_CHECK(pos->numel() >= src.size(0), "pos too short");
  }
  const c10::cuda::CUDAGuard guard(src.device());
  lmsae::PeerTable pt = make_peer_table(table);
  check_cuda(lmsae::bcast_rows_cast_launch(pt, dtype_code(src), (int)out_dtype, src.data_ptr(), opt_ptr<int>(keep), opt_ptr<int>(pos),
                                           src.size(0), (int)src.size(1), recv_off, cap_rows, (int)phase, (uint32_t)epoch,
                                           reinterpret_cast<unsigned*>(done_counter.data_ptr<int>()), use_multicast,
                                           at::cuda::getCurrentCUDAStream()),
             "comm_bcast_rows launch");
}

// Head-summed encoder GEMM: x [M, heads * d] bf16, w [heads * rows_per_head, d] bf16 (head h's rows start at
// h * rows_per_head; the first N of them are used), bias fp32 [N] or absent. One accumulation over K = heads * d sums
// x_h . W_h^T over the local heads; the result (+ bias) is stored as bf16 into H_out [M, N], which may be a view of a
// symmetric buffer that an all-reduce kernel then sums over the head ranks in place.
void head_sum_gemm(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& bias, int64_t heads, int64_t rows_per_head,
                   int64_t N, bool pair, const Tensor& status, const Tensor& H_out) {
  CHECK_T(x, torch::kBFloat16);
  CHECK_T(w, torch::kBFloat16);
  CHECK_T(status, torch::kInt32);
  CHECK_T(H_out, torch::kBFloat16);
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && heads >= 1 && x.size(1) == heads * w.size(1), "x [M, heads*d], w [heads*rows, d]");
  TORCH_CHECK(w.size(0) == heads * rows_per_head && N <= rows_per_head, "w must hold `heads` blocks of rows_per_head rows");
  TORCH_CHECK(H_out.dim() == 2 && H_out.size(0) == x.size(0) && H_out.size(1) == N, "H_out must be [M, N]");
  TORCH_CHECK(w.size(1) % 64 == 0, "d must be a multiple of 64");
  const c10::cuda::CUDAGuard guard(x.device());
  lmsae::EncGemmParams p{};
  p.M = (int)x.size(0);
  p.K = (int)x.size(1);
  p.N = (int)N;
  p.num_panels = (p.M + 127) / 128;
  const int n_tiles = (p.N + 255) / 256;
  // as many column ranges as fill the GPU (one CTA per panel and range)
  int splits = 148 / p.num_panels;
  if (splits < 1) splits = 1;
  if (splits > n_tiles) splits = n_tiles;
  p.num_splits = splits;
  if (bias.has_value()) { CHECK_T(*bias, torch::kFloat32); TORCH_CHECK(bias->numel() == p.N); }
  p.bias = opt_ptr<const float>(bias);
  p.status = status.data_ptr<int>();
  p.heads = (int)heads;
  p.b_rows_per_head = (int)rows_per_head;
  p.H = reinterpret_cast<__nv_bfloat16*>(H_out.data_ptr());
  p.ldh = p.N;
  int mode = 1;
  if (pair && p.num_panels % 2 == 0) mode |= 8;
  const CUtensorMap ta = make_bf16_tile_map(x.data_ptr(), p.M, p.K, 128);
  const CUtensorMap tb = make_bf16_tile_map(w.data_ptr(), w.size(0), w.size(1), (mode & 8) ? 128 : 256);
  check_cuda(lmsae::enc_gemm_launch(ta, tb, p, mode, at::cuda::getCurrentCUDAStream()), "head_sum_gemm launch");
}

// In-place sum over the ranks of `table` of the bf16 array at byte offset `off` (n16 16-byte vectors) of every rank's
// symmetric buffer; see allreduce_bf16_inplace_kernel.
void comm_allreduce_bf16(const std::vector<int64_t>& table, int64_t off, int64_t n16, int64_t phase_in, int64_t phase_out,
                         int64_t epoch, bool use_multicast, const Tensor& done_counter, const Tensor& status) {
  CHECK_T(done_counter, torch::kInt32);
  CHECK_T(status, torch::kInt32);
  TORCH_CHECK(off % 16 == 0 && n16 >= 0);
  const c10::cuda::CUDAGuard guard(status.device());
  check_cuda(lmsae::allreduce_bf16_launch(make_peer_table(table), off, n16, (int)phase_in, (int)phase_out, (uint32_t)epoch,
                                          use_multicast ? 1 : 0, reinterpret_cast<unsigned*>(done_counter.data_ptr<int>()),
                                          status.data_ptr<int>(), at::cuda::getCurrentCUDAStream()),
             "allreduce_bf16 launch");
}

void comm_signal(const std::vector<int64_t>& table, int64_t phase, int64_t epoch) {
  lmsae::PeerTable pt = make_peer_table(table);
  check_cuda(lmsae::signal_flags_launch(pt, (int)phase, (uint32_t)epoch, at::cuda::getCurrentCUDAStream()), "comm_signal launch");
}

void comm_wait_src(const std::vector<int64_t>& table, int64_t phase, int64_t epoch, int64_t src, const Tensor& status) {
  CHECK_T(status, torch::kInt32);
  lmsae::PeerTable pt = make_peer_table(table);
  check_cuda(lmsae::wait_flag_src_launch(pt, (int)phase, (uint32_t)epoch, (int)src, status.data_ptr<int>(),
                                         at::cuda::getCurrentCUDAStream()),
             "comm_wait_src launch");
}

void comm_wait(const std::vector<int64_t>& table, int64_t phase, int64_t epoch, const Tensor& status) {
  CHECK_T(status, torch::kInt32);
  const c10::cuda::CUDAGuard guard(status.device());
  check_cuda(lmsae::wait_flags_launch(make_peer_table(table), (int)phase, (uint32_t)epoch, status.data_ptr<int>(),
                                      at::cuda::getCurrentCUDAStream()),
             "wait_flags launch");
}

// partial_dtype: 0 = fp32, 1 = bf16 partial rows; use_multicast: keep the rows local and let the owner sum them through the
// switch; compact_codes: the codes of a row are packed from slot 0 on.
void comm_decode_scatter(const std::vector<int64_t>& table, const Tensor& idx, const Tensor& val, const Tensor& W,
                         int64_t partial_dtype, bool use_multicast, bool compact_codes, int64_t epoch,
                         const Tensor& done_counter) {
  CHECK_T(idx, torch::kInt32);
  CHECK_T(val, torch::kFloat32);
  CHECK_T(W, torch::kBFloat16);
  CHECK_T(done_counter, torch::kInt32);
  TORCH_CHECK(idx.dim() == 2 && val.sizes() == idx.sizes() && W.dim() == 2);
  const c10::cuda::CUDAGuard guard(idx.device());
  check_cuda(lmsae::sparse_decode_scatter_launch(make_peer_table(table), idx.data_ptr<int>(), val.data_ptr<float>(),
                                                 (int)idx.size(0), (int)idx.size(1), (int)W.size(1), (int)W.size(0),
                                                 reinterpret_cast<const __nv_bfloat16*>(W.data_ptr()), (int)partial_dtype,
                                                 use_multicast ? 1 : 0, compact_codes ? 1 : 0, (uint32_t)epoch,
                                                 reinterpret_cast<unsigned*>(done_counter.data_ptr<int>()),
                                                 at::cuda::getCurrentCUDAStream()),
             "sparse_decode_scatter launch");
}

void comm_reduce_loss_push(const std::vector<int64_t>& table, int64_t B, int64_t d, const Tensor& label,
                           const c10::optional<Tensor>& bias, const c10::optional<Tensor>& row_weight,
                           double grad_scale, const Tensor& loss_sum, const c10::optional<Tensor>& xhat_out,
                           int64_t partial_dtype, bool use_multicast, int64_t epoch_in, int64_t epoch_out,
                           const Tensor& done_counter, const Tensor& status) {
  CHECK_T(label, torch::kBFloat16);
  CHECK_T(loss_sum, torch::kFloat32);
  CHECK_T(done_counter, torch::kInt32);
  CHECK_T(status, torch::kInt32);
  TORCH_CHECK(label.numel() == B * d);
  if (bias.has_value()) { CHECK_T(*bias, torch::kFloat32); TORCH_CHECK(bias->numel() == d); }
  if (row_weight.has_value()) { CHECK_T(*row_weight, torch::kFloat32); TORCH_CHECK(row_weight->numel() == B); }
  if (xhat_out.has_value()) { CHECK_T(*xhat_out, torch::kFloat32); TORCH_CHECK(xhat_out->numel() == B * d); }
  const c10::cuda::CUDAGuard guard(label.device());
  check_cuda(lmsae::reduce_loss_push_launch(make_peer_table(table), (int)B, (int)d,
                                            reinterpret_cast<const __nv_bfloat16*>(label.data_ptr()),
                                            opt_ptr<const float>(bias), opt_ptr<const float>(row_weight),
                                            (float)grad_scale, loss_sum.data_ptr<float>(), opt_ptr<float>(xhat_out),
                                            (int)partial_dtype, use_multicast ? 1 : 0, (uint32_t)epoch_in,
                                            (uint32_t)epoch_out, reinterpret_cast<unsigned*>(done_counter.data_ptr<int>()),
                                            status.data_ptr<int>(), at::cuda::getCurrentCUDAStream()),
             "reduce_loss_push launch");
}

// All-gather of up to eight row-sharded tensors over the ranks of `table` by peer stores, in one kernel: tensor i (any
// dtype, contiguous, the same byte size on every rank) lands at byte offset dst_offsets[i] + rank * nbytes_i of every
// rank's buffer; the kernel returns once every rank's rows have arrived here (bounded wait by its last block).
void comm_exchange_rows(const std::vector<int64_t>& table, const std::vector<Tensor>& src,
                        const std::vector<int64_t>& dst_offsets, int64_t epoch, const Tensor& done_counter,
                        const Tensor& status, bool use_multicast) {
  CHECK_T(done_counter, torch::kInt32);
  CHECK_T(status, torch::kInt32);
  TORCH_CHECK(!src.empty() && src.size() <= 8 && src.size() == dst_offsets.size(), "one offset per tensor, at most eight");
  lmsae::RowExchange ex{};
  ex.n = (int)src.size();
  for (int i = 0; i < ex.n; ++i) {
    TORCH_CHECK(src[i].is_cuda() && src[i].is_contiguous(), "exchange tensors must be contiguous CUDA tensors");
    ex.src[i] = src[i].data_ptr();
    ex.nbytes[i] = (long long)src[i].numel() * (long long)src[i].element_size();
    ex.dst_off[i] = dst_offsets[i];
    TORCH_CHECK(ex.nbytes[i] % 16 == 0 && ex.dst_off[i] % 16 == 0 && reinterpret_cast<uintptr_t>(ex.src[i]) % 16 == 0,
                "exchange tensors must be multiples of 16 bytes at 16-byte aligned addresses");
  }
  const c10::cuda::CUDAGuard guard(src[0].device());
  check_cuda(lmsae::exchange_rows_launch(make_peer_table(table), ex, (uint32_t)epoch,
                                         reinterpret_cast<unsigned*>(done_counter.data_ptr<int>()), status.data_ptr<int>(),
                                         use_multicast, at::cuda::getCurrentCUDAStream()),
             "exchange_rows launch");
}

// Records of the bounds-checked debug build: {translation unit: [source line, offending index, limit, number of
// violations]} since the last call (all zero in the regular build); reading clears them.
std::map<std::string, std::vector<int64_t>> bounds_report() {
  std::map<std::string, std::vector<int64_t>> out;
  int rec[4];
  check_cuda(lmsae::bounds_fetch_sparse_ops(rec), "bounds_fetch_sparse_ops");
  out["sparse_ops.cu"] = {rec[0], rec[1], rec[2], rec[3]};
  check_cuda(lmsae::bounds_fetch_comm_ops(rec), "bounds_fetch_comm_ops");
  out["comm_ops.cu"] = {rec[0], rec[1], rec[2], rec[3]};
  return out;
}

bool bounds_checked_build() {
#ifdef LMSAE_BOUNDS_CHECK
  return true;
#else
  return false;
#endif
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("bounds_report", &bounds_report);
  m.def("bounds_checked_build", &bounds_checked_build);
  m.def("comm_push_candidates", &comm_push_candidates);
  m.def("comm_exchange_rows", &comm_exchange_rows);
  m.def("comm_wait", &comm_wait);
  m.def("comm_bcast_rows", &comm_bcast_rows);
  m.def("comm_signal", &comm_signal);
  m.def("comm_allreduce_bf16", &comm_allreduce_bf16);
  m.def("head_sum_gemm", &head_sum_gemm);
  m.def("comm_wait_src", &comm_wait_src);
  m.def("comm_shuffle_rows", &comm_shuffle_rows);
  m.def("comm_decode_scatter", &comm_decode_scatter);
  m.def("comm_reduce_loss_push", &comm_reduce_loss_push);
  m.doc() = "sm_100a kernels for sparse-dictionary training";
  m.def("encoder_gemm", &encoder_gemm);
  m.def("jumprelu", &jumprelu);
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_bwd", &attn_bwd);
  m.def("radix_hi_bins", &radix_hi_bins);
  m.def("radix_hist", &radix_hist);
  m.def("radix_pick", &radix_pick);
  m.def("threshold_mask", &threshold_mask);
  m.def("row_compact", &row_compact);
  m.def("jumprelu_window_grad", &jumprelu_window_grad);
  m.def("rotary_pair", &rotary_pair);
  m.def("exclusive_scan", &exclusive_scan);
  m.def("gather_rows_cast", &gather_rows_cast);
  m.def("clt_decode", &clt_decode);
  m.def("clt_dact", &clt_dact);
  m.def("clt_wgrad", &clt_wgrad);
  m.def("topk_merge", &topk_merge);
  m.def("row_topk", &row_topk);
  m.def("sparse_decode", &sparse_decode);
  m.def("sparse_dact", &sparse_dact);
  m.def("mse_loss_grad", &mse_loss_grad);
  m.def("csc_build", &csc_build);
  m.def("auxk_loss_grad", &auxk_loss_grad);
  m.def("sparse_grad_adam", &sparse_grad_adam);
  m.def("colsum_bf16", &colsum_bf16);
  m.def("adam_flat", &adam_flat);
  m.def("row_norm_shadow", &row_norm_shadow);
}
