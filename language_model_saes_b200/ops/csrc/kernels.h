// Parameter blocks and host launchers of the sm_100a kernels, shared by the .cu files and the bindings.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lmsae {

struct EncGemmParams {
  int M, N, K;
  int num_panels;
  int num_splits;
  // Work units (one CTA, or one CTA pair = two adjacent panels) launched: 0 = num_splits per panel unit. Otherwise the
  // units are dealt out raggedly, units / panel_units to every panel unit and one more to the first units % panel_units
  // of them (num_splits is then the larger count and sizes the candidate lists), so that a batch whose panel count does
  // not divide the SM count still occupies every SM.
  int units;
  const float* bias;
  const float* gate;
  __nv_bfloat16* H;
  long long ldh;
  int k;
  float* cand_val;
  int* cand_idx;
  int* status;
  // Sweeping the dictionary in several launches (one per feature chunk): this launch covers columns
  // [n_index_offset, n_index_offset + N) of the whole dictionary (W, bias and gate already point at the chunk),
  // writes global column indices, and when resume_topk != 0 continues the running top-k that the previous
  // chunk's launch left in cand_val / cand_idx instead of starting empty.
  int n_index_offset;
  int resume_topk;
  // Head-summed encoders (crosscoders): the K dimension is `heads` blocks of K / heads columns; block h of A pairs with
  // rows [h * b_rows_per_head, h * b_rows_per_head + N) of the B tensor map, so one accumulation sums
  // x_h . W_h^T over the heads. heads <= 1: a plain GEMM.
  int heads;
  int b_rows_per_head;
};
int enc_gemm_launch(const CUtensorMap& ta, const CUtensorMap& tb, const EncGemmParams& p, int mode, cudaStream_t stream);
int enc_gemm_slots_for_k(int k);

// ---- peer-memory collectives (comm_ops.cu) -------------------------------------------------------
constexpr int kMaxPeers = 8;
// Flag words of a symmetric buffer: flag[phase][src] = last epoch that rank `src` published for `phase`. Every
// communicator object owns its buffer and therefore its own set of phases; the names below are those of the fused
// training step (model group) and of the data-parallel row exchange / parameter publication (data group).
enum CommPhase : int {
  kPhaseCand = 0, kPhasePartial = 1, kPhaseDxhat = 2, kPhaseAux = 3, kPhaseRows = 4, kPhaseParams = 5, kNumPhases = 8
};

// Peer mappings of every rank's symmetric buffer plus the byte offsets of its regions (same on all ranks).
struct PeerTable {
  char* base[kMaxPeers];
  int world, rank;
  long long flags_off;     // uint32 [kNumPhases][kMaxPeers]
  long long cand_val_off;  // float [B][world * k]   (the host alternates between two such buffers)
  long long cand_idx_off;  // int   [B][world * k]
  long long partial_off;   // partial reconstruction rows: [world][B / world][d] (peer stores) or [B][d] (multicast reads)
  long long dxhat_off;     // bf16  [B][d]
  char* mc_base;           // multicast (NVLS) mapping of the same buffers, nullptr when the group has none
  unsigned long long* stats;  // exposed-wait accounting: {cycles, calls} per phase, local device memory or nullptr
};

enum MergeCommMode : int { kMergeLocal = 0, kMergePush = 1, kMergeWait = 2 };
struct MergeComm {
  PeerTable pt;
  int mode;
  uint32_t epoch;
  unsigned* done_counter;
  int* status;
};

int topk_merge_launch(const float* cand_val, const int* cand_idx, int M, int C, int k, const float* gate, int own_lo,
                      int own_hi, int emit_gated, int* out_idx, float* out_val, const MergeComm& comm, cudaStream_t stream);
int row_topk_launch(const __nv_bfloat16* H, long long ldh, int M, int N, int k, const float* gate,
                    const uint8_t* alive, int* out_idx, float* out_val, cudaStream_t stream);

// Records of the bounds-checked debug build, one per translation unit (all zero in the regular build).
int bounds_fetch_sparse_ops(int* out);
int bounds_fetch_comm_ops(int* out);

struct DecodeParams {
  const int* idx;
  const float* val;
  int B, k, d;
  int F;  // rows of W (the limit of the codes' feature indices; checked in the debug build)
  const __nv_bfloat16* W;
  const float* bias;
  float* xhat_f32;
  __nv_bfloat16* xhat_bf16;
  const __nv_bfloat16* label;
  const float* row_weight;
  float grad_scale;
  __nv_bfloat16* dxhat;
  float* loss_sum;
  float* row_loss;
  float* dval;
};
int sparse_decode_launch(const DecodeParams& p, cudaStream_t stream);
// `wait`: optional (pt.world > 0) bounded wait for the gradient rows of the fused step (phase kPhaseDxhat) at kernel entry
int sparse_dact_launch(const int* idx, int B, int k, int d, int F, const __nv_bfloat16* W, const __nv_bfloat16* dxhat,
                       float* dval, const PeerTable* wait, uint32_t epoch, int* status, cudaStream_t stream);
int mse_loss_grad_launch(const float* xhat, const __nv_bfloat16* label, const float* bias, const float* row_weight,
                         int rows, int d, float grad_scale, __nv_bfloat16* dxhat, float* loss_sum, float* row_loss,
                         cudaStream_t stream);
int csc_build_launch(const int* idx, long long n, int F, int* counts, int* offsets, int* cursor, int* entries,
                     int* block_sums_buf, cudaStream_t stream);

struct AdamHyper {
  float lr, beta1, beta2, eps;
  float bias_correction1, bias_correction2_sqrt;
};
struct GradAdamParams {
  int F, d, k;
  int n_rows;        // rows of x / dxhat and
  long long n_codes; // elements of act / dact: limits of the entry lists' positions (checked in the debug build)
  const int* offsets;
  const int* entries;
  const float* act;
  const float* dact;
  const __nv_bfloat16* x;
  const __nv_bfloat16* dxhat;
  float* WD; float* mD; float* vD; __nv_bfloat16* WD_bf16;
  float* WE; float* mE; float* vE; __nv_bfloat16* WE_bf16;
  float* bE; float* mbE; float* vbE;
  float* dec_norm;
  const float* grad_mul;
  float* grad_sq_sum;
  AdamHyper h;
  int update;
  int f_begin, f_end;  // feature rows handled by this launch
  int ctas_per_sm;     // 0 = fill the GPU (4 per SM); 1..4 = leave registers free for a concurrently running kernel
  int use_rowwarp;     // != 0: rows of at most 1024 columns (a multiple of 128) take the warp-per-row kernel
  const int* status;   // kernels' status word: a recorded error turns the update into a no-op (nullptr: not checked)
  // Dense gradient rows for a subset of the features, added to the rows rebuilt from the entry lists: feature f takes
  // row extra_row[f] (when >= 0) of the fp32 matrices extra_gD / extra_gE [rows, d] and element extra_row[f] of extra_gb.
  const int* extra_row;
  const float* extra_gD; const float* extra_gE; const float* extra_gb;
  // Gradient that reaches a decoder row through its own norm (a sparsity penalty on a * ||W_D row||): the row's gradient
  // gets wd_self_scale[f] * W_D[f, :] added, with the row read in the same pass that updates it (nullptr: none).
  const float* wd_self_scale;
  // Instead of writing dec_norm[f] = ||new W_D row||, add the squared norm to norm_sq_accum[f] (nullptr: off): a feature
  // whose gate is the norm over SEVERAL decoder matrices collects it over one launch per matrix.
  float* norm_sq_accum;
  const __nv_bfloat16* dxhat_aux;  // output gradient seen by the code slots >= k_main of every row (nullptr: none)
  int k_main;
  float* gD_out;  // optional dense [F, d] outputs of the rebuilt gradient rows (for autograd callers)
  float* gE_out;
  // Optimizer state sharded by feature row over data-parallel replicas: this launch owns rows [f_begin, f_end); its
  // moments are arrays of (f_end - state_f0) rows that start at row state_f0 of the dictionary (0: full-size arrays).
  int state_f0;
  // Publication of the updated rows to the other replicas (n_pub > 0): the bf16 shadows, decoder norms and encoder
  // biases are stored at byte offsets pub_*_off of EVERY rank's symmetric buffer in pub (this rank's own included, the
  // local WD_bf16 / WE_bf16 / dec_norm / bE pointers above are then views of that buffer), and the last block
  // publishes pub_epoch for phase kPhaseParams.
  int n_pub;
  PeerTable pub;
  long long pub_wd_off, pub_we_off, pub_norm_off, pub_be_off;
  uint32_t pub_epoch;
  unsigned* pub_done;
};
int auxk_loss_grad_launch(const float* xhat, const float* aux_rec, const __nv_bfloat16* label, const float* bias,
                          const float* row_weight, int rows, int d, float grad_scale, float alpha,
                          const float* alpha_factor, __nv_bfloat16* g_main, __nv_bfloat16* g_aux, float* loss_sum,
                          float* aux_sum, cudaStream_t stream);
int sparse_grad_adam_launch(const GradAdamParams& p, cudaStream_t stream);
int colsum_bf16_launch(const __nv_bfloat16* a, int rows, int d, float* out, cudaStream_t stream);
int adam_flat_launch(float* p, const float* g, float* m, float* v, long long n, AdamHyper h, const float* grad_mul,
                     __nv_bfloat16* shadow, float* grad_sq_sum, int update, const int* status, cudaStream_t stream);
int row_norm_shadow_launch(const float* W, int F, int d, float* norm, __nv_bfloat16* shadow, cudaStream_t stream);

// ---- cross-layer transcoder decoder fan-out (clt_ops.cu) --------------------------------------------
constexpr int kMaxCltLayers = 64;
struct CltTable { const __nv_bfloat16* W[kMaxCltLayers]; };  // W[t]: bf16 [t + 1, F, d], one allocation per target layer
struct CltGradTable { float* G[kMaxCltLayers]; };            // G[t]: fp32 [t + 1, F, d]
int clt_decode_launch(const CltTable& tab, const int* idx, const float* val, int B, int K, int L, int F, int d,
                      const float* bias, float* out_f32, __nv_bfloat16* out_bf16, cudaStream_t stream);
int clt_dact_launch(const CltTable& tab, const int* idx, int B, int K, int L, int F, int d, const __nv_bfloat16* dy,
                    float* dval, cudaStream_t stream);
int clt_wgrad_launch(const CltGradTable& tab, const int* offsets, const int* entries, const float* act, int B, int K,
                     int L, int F, int d, const __nv_bfloat16* dy, cudaStream_t stream);

// ---- selection / compaction (select_ops.cu) --------------------------------------------------------
// dtype: 0 = fp32, 1 = bf16. x is a contiguous [A, S, N] array and the selection covers segment s.
int radix_hi_bins();
int radix_hist_launch(int dtype, const void* x, long long A, long long S, long long N, long long s, int level,
                      const long long* sel, unsigned* hist, const float* floor, const long long* need,
                      cudaStream_t stream);
int radix_pick_launch(const unsigned* hist, int nbins, long long k, const long long* sel_in, int level, long long* sel_out,
                      float* thr, const long long* need, cudaStream_t stream);
int threshold_mask_launch(int dtype, const void* x, const float* thr, long long A, long long S, long long N, void* out,
                          cudaStream_t stream);
int row_compact_launch(int dtype, const void* x, int B, long long N, int cap, int* idx, float* val, int* nnz,
                       const float* thr, const float* col_div, int* ties, const int* tie_quota, const float* col_thr,
                       int* seg_counts, cudaStream_t stream);
int jumprelu_window_grad_launch(const __nv_bfloat16* G, const __nv_bfloat16* S, int B, int F, const float* n,
                                const float* theta, float window, float add_per_hit, float* dtheta, cudaStream_t stream);
int gather_rows_cast_launch(int in_dtype, int out_dtype, const void* src, const int* keep, const int* pos, long long n,
                            int d, void* out, long long out_rows, cudaStream_t stream);
int exclusive_scan_launch(const int* counts, int n, int* offsets, int* block_sums_buf, cudaStream_t stream);

// ---- rotary embedding of two [tokens, heads, width] bf16 tensors in one launch (rotary.cu) ----------------------
int rotary_pair_launch(const __nv_bfloat16* xa, const __nv_bfloat16* xb, __nv_bfloat16* oa, __nv_bfloat16* ob, const float* cos_t,
                       const float* sin_t, long long tokens, int seq, int heads, int width, int rd, int adjacent, float sin_sign,
                       cudaStream_t stream);

// ---- causal attention with d_v != d_qk (attention.cu) ------------------------------------------------
struct AttnParams {
  int batch, seq, heads, dqk, dv;
  float scale_log2;       // softmax scale * log2(e)
  __nv_bfloat16* out;     // [batch, seq, heads, dv]
  float* lse;             // [batch, heads, seq] natural-log sum of exponentials (nullptr: not wanted)
  int* status;
};
struct AttnBwdParams {
  int batch, seq, heads, dqk, dv;
  float scale, scale_log2;
  const float* lse;    // [batch, heads, seq] from the forward pass
  const float* delta;  // [batch, heads, seq] rowsum(dO * O)
  float* dq;           // [batch, seq, heads, dqk]
  float* dk;           // [batch, seq, heads, dqk]
  float* dv_out;       // [batch, seq, heads, dv]
  int* status;
};
int attn_bwd_launch(const CUtensorMap* maps_dq, const CUtensorMap* maps_dkv, const AttnBwdParams& p, cudaStream_t stream);
int attn_value_chunk(int dv);
int attn_fwd_value_chunk(int dqk, int dv);
int attn_fwd_launch(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tvt, const AttnParams& p,
                    cudaStream_t stream);

// ---- elementwise (jumprelu.cu) ---------------------------------------------------------------------
int jumprelu_launch(int dtype, const void* x, const void* log_theta, const void* dy, void* out, float* dlog, long long n,
                    int P, float window, int backward, cudaStream_t stream);

// All-gather of several row-sharded tensors in one kernel (comm_ops.cu::exchange_rows_kernel).
struct RowExchange {
  const void* src[8];
  long long nbytes[8];   // bytes of this rank's part (the same on every rank), multiples of 16
  long long dst_off[8];  // byte offset of the gathered tensor in every rank's buffer
  int n;
};
int exchange_rows_launch(const PeerTable& pt, const RowExchange& ex, uint32_t epoch, unsigned* done_counter, int* status,
                         bool use_multicast, cudaStream_t stream);
int push_candidates_launch(const PeerTable& pt, const float* val, const int* idx, int B, int k, uint32_t epoch,
                           unsigned* done_counter, cudaStream_t stream);
int shuffle_rows_launch(const PeerTable& pt, const void* src, const long long* dest, int n_local, int rows_per_rank,
                        int row_bytes, long long recv_off, int phase, uint32_t epoch, unsigned* done_counter,
                        cudaStream_t stream);
int bcast_rows_cast_launch(const PeerTable& pt, int in_dtype, int out_dtype, const void* src, const int* keep, const int* pos,
                           long long n, int d, long long recv_off, long long cap_rows, int phase, uint32_t epoch,
                           unsigned* done_counter, bool use_multicast, cudaStream_t stream);
int allreduce_bf16_launch(const PeerTable& pt, long long off, long long n16, int phase_in, int phase_out, uint32_t epoch,
                          int use_multicast, unsigned* done_counter, int* status, cudaStream_t stream);
int signal_flags_launch(const PeerTable& pt, int phase, uint32_t epoch, cudaStream_t stream);
int wait_flag_src_launch(const PeerTable& pt, int phase, uint32_t epoch, int src, int* status, cudaStream_t stream);
int wait_flags_launch(const PeerTable& pt, int phase, uint32_t epoch, int* status, cudaStream_t stream);
// partial_dtype: 0 = fp32, 1 = bf16 partial rows. use_multicast: partial rows stay in the producer's own buffer ([B][d])
// and the owner sums them with multimem.ld_reduce; the gradient rows are published with multimem.st (needs pt.mc_base,
// bf16 partials).
int sparse_decode_scatter_launch(const PeerTable& pt, const int* idx, const float* val, int B, int k, int d, int F,
                                 const __nv_bfloat16* W, int partial_dtype, int use_multicast, int compact_codes,
                                 uint32_t epoch, unsigned* done_counter, cudaStream_t stream);
int reduce_loss_push_launch(const PeerTable& pt, int B, int d, const __nv_bfloat16* label, const float* bias,
                            const float* row_weight, float grad_scale, float* loss_sum, float* xhat_out,
                            int partial_dtype, int use_multicast, uint32_t epoch_in, uint32_t epoch_out,
                            unsigned* done_counter, int* status, cudaStream_t stream);

}  // namespace lmsae
