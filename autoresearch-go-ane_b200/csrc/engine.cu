// Training-step engine: device-resident model state plus the orchestration of one
// Step / EvalLogits / EvalLoss, mirroring ane.Engine (ane/engine.go) over CUDA kernels.
//
// Data layout in HBM
//   parameters   one flat fp32 buffer P (master), with same-shaped G (accumulated gradients),
//                Adam m and v; a bf16 shadow of the GEMM operands (matrices + embedding) that the
//                optimizer kernel rewrites, so no separate weight-refresh pass exists
//                (the reference restages weights after every update, ane/runtime.go:25-94).
//   activations  token-major [M = batch*seq, C]; residual stream fp32, GEMM operands in T
//                (bf16 on the tensor-core path, float in fp32 parity mode).
//   per layer    Wqkv [(H+2KV)*hd, D] (Wq|Wk|Wv rows), Wo [D, H*hd], W13 [Hd or 2Hd, D] (W1|W3), W2 [D, Hd].
#include "engine.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <thread>

#include "common.cuh"
#include "dp.h"
#include "gemm.h"
#include "kernels.h"

namespace ane {

// Window sampler of Engine.Step (ane/engine.go:395-404) over the drand48 generator
// (ane/engine.go:873-880), extended to data parallelism: every rank advances the one global
// stream by batch*world draws per step and keeps draws rank, rank+world, ...  Host-only.
void sample_windows(uint64_t* rng, uint64_t n_tokens, uint32_t seq, uint32_t batch, uint32_t rank, uint32_t world,
                    uint64_t* out_pos) {
  constexpr uint64_t kMul = 0x5DEECE66Dull, kAdd = 0xBull, kMask = (1ull << 48) - 1;
  if (world == 0) world = 1;
  const uint64_t limit = n_tokens > (uint64_t)seq + 1 ? n_tokens - seq - 1 : 0;
  for (uint32_t i = 0; i < batch * world; ++i) {
    *rng = (kMul * (*rng) + kAdd) & kMask;
    const double u = (double)(*rng) / (double)(1ull << 48);
    uint64_t pos = 0;
    if (limit > 0) {
      pos = (uint64_t)(u * (double)limit);
      if (pos >= limit) pos = limit - 1;
    }
    if (i % world == rank) out_pos[i / world] = pos;
  }
}

namespace {

inline int64_t now_ns() {
  return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch())
      .count();
}


template <typename T>
struct Act {  // saved activations of one layer (ane/train_full.go:12-37)
  float* x2 = nullptr;
  T* xn = nullptr;
  void* qkv = nullptr;    // packed q|k|v: fp32 when the engine keeps attention operands in fp32, else T
  void* qkpre = nullptr;  // rotated pre-norm q|k (reference architecture), same type as qkv
  T* att = nullptr;
  T* att_lo = nullptr;    // bf16 engines on the tensor-core attention: what rounding att to bf16 dropped (for delta)
  T* x2n = nullptr;
  T* h13 = nullptr;
  T* gate = nullptr;
  float* rstd1 = nullptr;
  float* rstd2 = nullptr;
  float* lse = nullptr;
  float* ve_act = nullptr;
  // debug gradient taps (fp32), only with debug_taps
  float* t_dout = nullptr;
  float* t_dx2 = nullptr;
  float* t_dqkv = nullptr;
  float* t_dh13 = nullptr;
};

__global__ void gather_windows_kernel(const uint16_t* __restrict__ tokens, const uint64_t* __restrict__ pos,
                                      uint16_t* __restrict__ in, uint16_t* __restrict__ tgt, int B, int seq) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B * seq) return;
  const int b = i / seq, t = i - b * seq;
  const uint64_t p = pos[b] + (uint64_t)t;
  in[i] = tokens[p];
  tgt[i] = tokens[p + 1];
}

// out[(b*ncols + c)*seq + t] = src[(b*seq+t)*ld + col0 + c]   (token-major -> the reference's [C][seq])
// il != 0: tap column c lives at source column (c/32)*64 + c%32 + col0 (the interleaved h1 | h3 layout).
template <typename TS>
__global__ void export_tap_kernel(const TS* __restrict__ src, int ld, int col0, int ncols, int M, int seq, int il,
                                  float* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)M * ncols) return;
  const int m = (int)(i / ncols), c = (int)(i - (long long)m * ncols);
  const int b = m / seq, t = m - b * seq;
  const int sc = il ? ((c >> 5) << 6) + (c & 31) + col0 : col0 + c;
  out[((size_t)b * ncols + c) * seq + t] = to_f<TS>(src[(size_t)m * ld + sc]);
}

// next-token targets inside each window for the evaluation loss: tgt[b,t] = tok[b,t+1], last = invalid.
__global__ void shift_targets_kernel(const uint16_t* __restrict__ tok, uint16_t* __restrict__ tgt, int B, int seq) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B * seq) return;
  const int t = i % seq;
  tgt[i] = (t + 1 < seq) ? tok[i + 1] : (uint16_t)0xFFFF;
}

template <typename TS>
__global__ void to_f32_kernel(const TS* __restrict__ src, float* __restrict__ dst, uint64_t n) {
  uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) dst[i] = to_f<TS>(src[i]);
}
template <typename TD>
__global__ void from_f32_kernel(const float* __restrict__ src, TD* __restrict__ dst, uint64_t n) {
  uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) dst[i] = from_f<TD>(src[i]);
}
inline unsigned ew_grid(uint64_t n) {
  uint64_t g = (n + 255) / 256;
  if (g > 148ull * 16) g = 148ull * 16;
  return (unsigned)(g < 1 ? 1 : g);
}

struct Slot {
  size_t off = 0, n = 0;
};

template <typename T>
class EngineT final : public EngineBase {
 public:
  ~EngineT() override { destroy(); }

  int open(const ane_options& o, const uint16_t* tokens, uint64_t n_tokens, const uint8_t* dp_id) override;
  int step(const uint16_t* input, const uint16_t* target, uint32_t n_seq, ane_step_result* out) override;
  int flush(double* refresh_ms) override;
  int eval_logits(const uint16_t* tokens, uint32_t n_seq, float* out, uint64_t cap, uint32_t layout) override;
  int eval_loss(const uint16_t* tokens, uint32_t n_seq, double* loss_sum, uint64_t* n_pos) override;
  int decode(const uint16_t* prompts, uint32_t n_seq, uint32_t prompt_len, uint32_t n_new, float temperature,
             const double* uniforms, uint16_t* out) override;
  int set_lr(float lr) override;
  float get_lr() override { return lr_; }
  int get_state(ane_state* s) override;
  int set_state(const ane_state* s) override;
  int reseed(int64_t seed) override;
  int64_t tensor_size(uint32_t id, uint32_t layer) override;
  int import_tensor(uint32_t id, uint32_t layer, uint32_t which, const float* buf, uint64_t n) override;
  int export_tensor(uint32_t id, uint32_t layer, uint32_t which, float* buf, uint64_t n) override;
  int64_t get_tap(uint32_t tap, uint32_t layer, float* buf, uint64_t cap) override;
  int profile_gemm(int enable) override;
  int profile_read(double* gemm_ms, double* gemm_flops, uint64_t* gemm_launches) override;
  int timer_begin() override;
  int timer_end(float* ms) override;

 private:
  static constexpr bool kIsF32 = sizeof(T) == 4;

  int fail(int code, const std::string& msg) {
    err_ = msg;
    return code;
  }
  int cuda_check(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return 0;
    return fail(ANE_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
  }
  template <typename U>
  int dalloc(U** p, size_t count) {
    void* q = nullptr;
    cudaError_t e = cudaMalloc(&q, std::max<size_t>(count, 1) * sizeof(U));
    if (e != cudaSuccess) return cuda_check(e, "cudaMalloc");
    allocs_.push_back(q);
    *p = reinterpret_cast<U*>(q);
    return 0;
  }
  void destroy();
  bool is_ve_layer(int i) const { return isN_ && (i % 2 == (L_ - 1) % 2); }  // ane/stories/weights.go:22
  const T* wop(size_t off) const {
    if constexpr (kIsF32) return P_ + off;
    else return Sh_ + off;
  }
  int gemm(const GemmDesc& d, cudaStream_t on = nullptr) {
    int rc;
    cudaStream_t st = on ? on : stream_;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (profiling_) {
      cudaEventCreate(&e0);
      cudaEventCreate(&e1);
      cudaEventRecord(e0, st);
    }
    if constexpr (kIsF32) rc = x3_ ? gemm_bf16x3(d, &split_, d_status_, st) : gemm_f32(d, st);
    else rc = gemm_bf16(d, d_status_, st);
    if (profiling_) {
      cudaEventRecord(e1, st);
      prof_events_.push_back({e0, e1});
      prof_shapes_.push_back({d.M, d.N, d.K, (d.a_mn ? 1 : 0) | (d.b_mn ? 2 : 0) | (d.out << 2) | (d.res1 ? 16 : 0)});
      // the recomputed classifier product of the logit-free head is time spent, not algorithmic work
      if (d.out != GEMM_OUT_CE_GRAD) prof_flops_ += 2.0 * (double)d.M * (double)d.N * (double)d.K;
    }
    if (rc != 0) return fail(ANE_ERR_KERNEL, gemm_last_error());
    return 0;
  }
  // The weight-gradient products of layer `l` as one grouped launch (bf16 engines).
  int gemm_group(const GemmDesc* ds, int n, int l, cudaStream_t st) {
    if constexpr (kIsF32) {
      return fail(ANE_ERR_STATE, "storiesane step: grouped products run on bf16 engines");
    } else {
      cudaEvent_t e0 = nullptr, e1 = nullptr;
      if (profiling_) {
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        cudaEventRecord(e0, st);
      }
      bool built = group_built_[l] != 0;
      const int rc = gemm_bf16_grouped(ds, n, d_groups_ + (size_t)l * gemm_group_slot_bytes(), &built, d_status_, st);
      group_built_[l] = built ? 1 : 0;
      if (profiling_) {
        cudaEventRecord(e1, st);
        prof_events_.push_back({e0, e1});
        prof_shapes_.push_back({0, 0, ds[0].K, 3 | (GEMM_OUT_ACCUM << 2)});
        for (int p = 0; p < n; ++p) prof_flops_ += 2.0 * (double)ds[p].M * (double)ds[p].N * (double)ds[p].K;
      }
      if (rc != 0) return fail(ANE_ERR_KERNEL, gemm_last_error());
      return 0;
    }
  }
  // T-typed view of an fp32 buffer: in fp32 mode the buffer itself, else a separately written copy.
  T* tview(float* f32buf, T* tbuf) const {
    if constexpr (kIsF32) return f32buf;
    else return tbuf;
  }
  T* tcopy_arg(T* tbuf) const {  // what to pass as "also write a T copy" output
    if constexpr (kIsF32) return nullptr;
    else return tbuf;
  }
  void cast_to_t(const float* src, T* dst, uint64_t n) {
    if constexpr (!kIsF32) {
      count_launch();
      from_f32_kernel<T><<<ew_grid(n), 256, 0, stream_>>>(src, dst, n);
    }
  }
  int layout_params();
  int alloc_buffers();
  int refresh_shadow();
  int forward(const uint16_t* d_tok, int B, int Tl, int pos0);
  int head_and_backward(int B);
  int head_eval_loss(int B, double* loss_sum, uint64_t* n_pos);
  int backward_layers(int B);
  int do_flush();
  int check_device_status(int* out_status);
  Slot slot_of(uint32_t id, uint32_t layer, bool* ok) const;

  // ---- configuration
  ane_options o_{};
  int D_ = 0, Hd_ = 0, L_ = 0, H_ = 0, KV_ = 0, hd_ = 0, V_ = 0, S_ = 0, B_ = 0, M_ = 0;
  int QD_ = 0, KVD_ = 0, QKVD_ = 0, N13_ = 0;
  bool isN_ = false, quirks_ = false;
  // The reference architecture's backward recomputes attention with unscaled scores
  // (ane/train_full.go:268-269), which amplifies operand rounding; its q/k/v stay in fp32.
  bool qkv_f32_ = false;
  bool att_tc_ = false;  // tensor-core attention kernels (bf16 operands, head_dim 64)
  bool x3_ = false;      // fp32 engine whose GEMMs run as three bf16 tensor-core products (ANE_DTYPE_BF16X3)
  SplitScratch split_;   // its operand halves (one stream at a time: no side stream in this mode)
  bool decoding_ = false;  // forward() runs one KV-cached decode step
  std::vector<T*> kcache_, vcache_;  // [B, S_, KV*hd] per layer, allocated by the first decode
  int32_t* d_argmax_ = nullptr;
  double* d_dec_u_ = nullptr;  // uniform draws of a sampling decode, [n_new][n_seq]
  uint16_t *d_dec_tok_ = nullptr, *d_dec_out_ = nullptr;
  float* h_logits_ = nullptr;  // pinned staging for EvalLogits downloads
  float* att_delta_ = nullptr;
  // fp32 q|k|v (reference arch) on the tcgen05 attention kernels: bf16 hi / lo copies, the backward's own
  // log-sum-exp, raw bf16 gradients
  bool att_split_ = false;
  bf16 *qkvh_ = nullptr, *qkvl_ = nullptr, *dqkv_raw_ = nullptr;
  float* att_lse_b_ = nullptr;
  float lr_ = 0, embed_lr_ = 0, scalar_lr_ = 0, lambda_lr_ = 0;
  int ce_rows_ = 0;
  // ---- parameters
  std::vector<Slot> s_qkv_, s_wo_, s_w13_, s_w2_, s_ve_embed_, s_ve_gate_, s_rms_att_, s_rms_ffn_;
  Slot s_embed_, s_rms_final_, s_resid_, s_x0l_, s_smear_gate_, s_smear_l_, s_backout_l_;
  size_t n_params_ = 0, shadow_n_ = 0;
  size_t r_mat0_ = 0, r_mat1_ = 0, r_ve0_ = 0, r_ve1_ = 0, r_veg0_ = 0, r_veg1_ = 0, r_rms0_ = 0, r_rms1_ = 0,
         r_lam0_ = 0, r_lam1_ = 0;
  float *P_ = nullptr, *G_ = nullptr, *Mo_ = nullptr, *Vo_ = nullptr;
  bf16* Sh_ = nullptr;
  float* d_one_ = nullptr;   // device constant 1.0f
  float* d_zero_ = nullptr;  // device constant 0.0f
  // ---- activations / work buffers
  std::vector<float*> xs_;
  std::vector<Act<T>> acts_;
  float *x0_ = nullptr, *xraw_ = nullptr, *gate_pre_ = nullptr, *gx0_ = nullptr, *gmid_ = nullptr, *dgp_ = nullptr,
        *dxs_ = nullptr, *dxs2_ = nullptr;
  T *x0_t_ = nullptr, *dgp_t_ = nullptr;
  // Backward operands that the weight-gradient GEMMs read are double-buffered by layer parity, so those
  // GEMMs can trail the main chain on their own stream by up to two layers.
  float *dcur_[2] = {nullptr, nullptr}, *dxn_ = nullptr, *dy_ = nullptr, *dx2_[2] = {nullptr, nullptr},
        *dqkv_f32_[2] = {nullptr, nullptr};
  T *dcur_t_[2] = {nullptr, nullptr}, *dx2_t_[2] = {nullptr, nullptr}, *dgate_ = nullptr, *dh13_[2] = {nullptr, nullptr},
    *datt_ = nullptr, *dqkv_[2] = {nullptr, nullptr}, *xnf_ = nullptr;
  cudaStream_t dw_stream_ = nullptr;       // weight-gradient GEMMs (the reference's async dW workers,
                                           // ane/train_full.go:969-992, become a second stream)
  std::vector<cudaEvent_t> ev_dw_done_;    // per layer: its four dW GEMMs have finished
  cudaEvent_t ev_dw_in_ = nullptr;
  bool dw_overlap_ = true;
  float *rstdf_ = nullptr, *logits_ = nullptr, *loss_rows_ = nullptr, *inv_valid_ = nullptr, *d_loss_ = nullptr;
  float* tgt_logit_ = nullptr;             // fp32 logit of every row's target (bf16-logits cross-entropy)
  // Classifier head that keeps no logits (bf16 engines): statistics of pass 1 per 256-column tile and row, the
  // rows' log2-sum-exp and gradient coefficients, and the gradient block [M, head_cols_] that pass 2 writes and
  // the dX / dEmbed products read while it is still in L2.
  // bf16 engines with ANE_B200_GROUP_DW=1: the four weight-gradient products of a layer leave as one grouped
  // stream-K launch on the side stream once the layer's main chain is done (one start-up and about one exposed
  // epilogue per CTA instead of four of each).  One descriptor slot per layer, filled at its first use.  Off by
  // default: the products' own time falls (6.79 -> 6.52 ms per step summed) but the step gets slower (8.83 ->
  // 8.97 ms), because one persistent launch holds every SM for ~95 us while the main chain waits for SMs.
  bool group_dw_ = false;
  uint8_t* d_groups_ = nullptr;
  std::vector<char> group_built_;
  bool head_fused_ = false;
  int head_cols_ = 0;
  float *ce_stats_ = nullptr, *ce_lse2_ = nullptr, *ce_coef_ = nullptr;
  bf16* dl_block_ = nullptr;
  int fused_head(int B);
  T* dlogits_ = nullptr;
  T* dlogits2_ = nullptr;                  // second chunk buffer: the classifier dW GEMM of chunk c runs on the
  cudaEvent_t ev_cls_ce_[2] = {nullptr, nullptr};  // side stream while chunk c+1 is computed
  cudaEvent_t ev_cls_dw_[2] = {nullptr, nullptr};
  cudaEvent_t ev_logits_[64] = {};          // EvalLogits: one per downloaded piece
  float *rope_cos_ = nullptr, *rope_sin_ = nullptr;
  float* rope_chunks_ = nullptr;  // the same tables by 16-byte chunk, for the one-CTA-per-head attention backward
  double* d_acc_ = nullptr;
  float *d_scales_ = nullptr, *d_norm_ = nullptr;
  int* d_status_ = nullptr;
  float* tap_tmp_ = nullptr;
  size_t tap_tmp_n_ = 0;
  // ---- tokens / sampler
  uint16_t *d_tokens_ = nullptr, *d_in_ = nullptr, *d_tgt_ = nullptr;
  uint16_t *h_in_ = nullptr, *h_tgt_ = nullptr;  // pinned
  uint64_t *d_pos_ = nullptr, *h_pos_ = nullptr;
  float* h_loss_ = nullptr;  // pinned
  uint64_t n_tokens_ = 0, rng_ = 0;
  // ---- state
  ane_state st_{};
  uint32_t pending_seqs_ = 0, micro_steps_ = 0;
  int64_t t_open_ns_ = 0;
  int last_B_ = 0;
  cudaStream_t stream_ = nullptr;
  cudaEvent_t ev0_ = nullptr, ev1_ = nullptr, ev_adam0_ = nullptr, ev_adam1_ = nullptr;
  DataParallel dp_;
  cudaStream_t comm_stream_ = nullptr;   // gradient all-reduce, overlapped with backward
  cudaEvent_t ev_bucket_ = nullptr, ev_comm_done_ = nullptr;
  // Sharded optimizer (world_size > 1): the layer matrices' gradients are reduce-scattered per bucket of
  // bucket_layers_ layers, each rank updates its slice of every bucket (fp32 weights and Adam moments of the
  // other slices are not touched), and the updated fp32 weights are all-gathered bucket by bucket on the
  // communication stream while the next pass already runs; a layer waits for its bucket.  Embedding, norm
  // weights and scalars stay replicated (all-reduce + full update): the embedding is read in fp32.
  bool shard_opt_ = false;
  int bucket_layers_ = 1;
  std::vector<cudaEvent_t> ev_gather_;    // per bucket: weights (and bf16 copies) complete on this rank
  cudaEvent_t ev_opt_done_ = nullptr, ev_norm_in_ = nullptr, ev_norm_out_ = nullptr;
  bool gather_pending_ = false;
  bool moments_current_ = true;           // the non-owned slices of the Adam moments match their owners'
  int n_buckets() const { return (L_ + bucket_layers_ - 1) / bucket_layers_; }
  size_t bucket_lo(int b) const { return s_qkv_[b * bucket_layers_].off; }
  size_t bucket_hi(int b) const { return (b + 1) * bucket_layers_ < L_ ? s_qkv_[(b + 1) * bucket_layers_].off : r_mat1_; }
  size_t bucket_slice(int b) const { return (bucket_hi(b) - bucket_lo(b)) / (size_t)o_.world_size; }
  void wait_bucket(int b) { if (gather_pending_) cudaStreamWaitEvent(stream_, ev_gather_[b], 0); }
  void wait_all_buckets() { if (gather_pending_) cudaStreamWaitEvent(stream_, ev_gather_.back(), 0); }
  int reduce_bucket(int b);
  int gather_moments();
  bool overlap_reduce_ = false;           // this micro-step is the last before the optimizer update
  size_t reduced_lo_ = 0;                 // G_[reduced_lo_, r_mat1_) has already been handed to the all-reduce
  std::vector<void*> allocs_;
  bool profiling_ = false;
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> prof_events_;
  struct ProfShape { int M, N, K, flags; };
  std::vector<ProfShape> prof_shapes_;
  double prof_flops_ = 0.0;
  cudaEvent_t ev_t0_ = nullptr, ev_t1_ = nullptr;
};

template <typename T>
void EngineT<T>::destroy() {
  if (stream_) cudaStreamSynchronize(stream_);
  if (comm_stream_) cudaStreamSynchronize(comm_stream_);  // weight gathers of the last update may still run
  dp_.shutdown();
  split_.release();
  for (void* p : allocs_) cudaFree(p);
  allocs_.clear();
  if (h_in_) cudaFreeHost(h_in_);
  if (h_tgt_) cudaFreeHost(h_tgt_);
  if (h_pos_) cudaFreeHost(h_pos_);
  if (h_loss_) cudaFreeHost(h_loss_);
  if (h_logits_) cudaFreeHost(h_logits_);
  h_logits_ = nullptr;
  h_in_ = h_tgt_ = nullptr;
  h_pos_ = nullptr;
  h_loss_ = nullptr;
  profile_gemm(0);
  for (cudaEvent_t* e : {&ev0_, &ev1_, &ev_adam0_, &ev_adam1_, &ev_t0_, &ev_t1_})
    if (*e) {
      cudaEventDestroy(*e);
      *e = nullptr;
    }
  for (auto& ev : ev_dw_done_)
    if (ev) cudaEventDestroy(ev);
  ev_dw_done_.clear();
  if (dw_stream_) {
    cudaStreamSynchronize(dw_stream_);
    cudaStreamDestroy(dw_stream_);
    dw_stream_ = nullptr;
  }
  for (cudaEvent_t* e : {&ev_bucket_, &ev_comm_done_, &ev_dw_in_, &ev_cls_ce_[0], &ev_cls_ce_[1], &ev_cls_dw_[0], &ev_cls_dw_[1]})
    if (*e) {
      cudaEventDestroy(*e);
      *e = nullptr;
    }
  for (auto& e : ev_logits_)
    if (e) {
      cudaEventDestroy(e);
      e = nullptr;
    }
  if (comm_stream_) {
    cudaStreamSynchronize(comm_stream_);
    cudaStreamDestroy(comm_stream_);
    comm_stream_ = nullptr;
  }
  for (cudaEvent_t* ev : {&ev_opt_done_, &ev_norm_in_, &ev_norm_out_})
    if (*ev) {
      cudaEventDestroy(*ev);
      *ev = nullptr;
    }
  for (auto& ev : ev_gather_)
    if (ev) cudaEventDestroy(ev);
  ev_gather_.clear();
  gather_pending_ = false;
  if (stream_) {
    cudaStreamDestroy(stream_);
    stream_ = nullptr;
  }
}

// Parameter layout: groups are contiguous so the optimizer needs one launch per group and the
// gradient all-reduce sees one flat buffer.
template <typename T>
int EngineT<T>::layout_params() {
  size_t off = 0;
  auto take = [&](size_t n) {
    Slot s;
    s.off = off;
    s.n = n;
    off += (n + 127) / 128 * 128;
    return s;
  };
  s_qkv_.resize(L_); s_wo_.resize(L_); s_w13_.resize(L_); s_w2_.resize(L_);
  s_ve_embed_.assign(L_, Slot()); s_ve_gate_.assign(L_, Slot());
  s_rms_att_.assign(L_, Slot()); s_rms_ffn_.assign(L_, Slot());
  r_mat0_ = off;
  for (int l = 0; l < L_; ++l) {
    s_qkv_[l] = take((size_t)QKVD_ * D_);
    s_wo_[l] = take((size_t)D_ * QD_);
    s_w13_[l] = take((size_t)N13_ * D_);
    s_w2_[l] = take((size_t)D_ * Hd_);
  }
  r_mat1_ = off;
  if (isN_) s_smear_gate_ = take((size_t)D_ * D_);
  s_embed_ = take((size_t)V_ * D_);
  shadow_n_ = off;  // bf16 shadow covers matrices, smear gate and the embedding
  r_ve0_ = off;
  for (int l = 0; l < L_; ++l)
    if (is_ve_layer(l)) s_ve_embed_[l] = take((size_t)V_ * D_);
  r_ve1_ = off;
  r_veg0_ = off;
  for (int l = 0; l < L_; ++l)
    if (is_ve_layer(l)) s_ve_gate_[l] = take((size_t)H_ * 12);
  r_veg1_ = off;
  r_rms0_ = off;
  if (!isN_) {
    for (int l = 0; l < L_; ++l) {
      s_rms_att_[l] = take(D_);
      s_rms_ffn_[l] = take(D_);
    }
    s_rms_final_ = take(D_);
  }
  r_rms1_ = off;
  if (isN_) {
    s_smear_l_ = take(1);
    s_backout_l_ = take(1);
    r_lam0_ = off;
    s_resid_ = take(L_);
    s_x0l_ = take(L_);
    r_lam1_ = off;
  }
  n_params_ = off;
  return 0;
}

template <typename T>
Slot EngineT<T>::slot_of(uint32_t id, uint32_t layer, bool* ok) const {
  *ok = true;
  Slot s;
  const bool per_layer = (id >= ANE_T_WQ && id <= ANE_T_RMS_FFN) || id == ANE_T_VE_EMBED || id == ANE_T_VE_GATE;
  if (per_layer && layer >= (uint32_t)L_) {
    *ok = false;
    return s;
  }
  switch (id) {
    case ANE_T_EMBED: return s_embed_;
    case ANE_T_WQ: s.off = s_qkv_[layer].off; s.n = (size_t)QD_ * D_; return s;
    case ANE_T_WK: s.off = s_qkv_[layer].off + (size_t)QD_ * D_; s.n = (size_t)KVD_ * D_; return s;
    case ANE_T_WV: s.off = s_qkv_[layer].off + (size_t)(QD_ + KVD_) * D_; s.n = (size_t)KVD_ * D_; return s;
    case ANE_T_WO: return s_wo_[layer];
    case ANE_T_W1: s.off = s_w13_[layer].off; s.n = (size_t)Hd_ * D_; return s;
    case ANE_T_W3:
      if (isN_) return s;
      s.off = s_w13_[layer].off + (size_t)Hd_ * D_; s.n = (size_t)Hd_ * D_; return s;
    case ANE_T_W2: return s_w2_[layer];
    case ANE_T_RMS_ATT: return s_rms_att_[layer];
    case ANE_T_RMS_FFN: return s_rms_ffn_[layer];
    case ANE_T_RMS_FINAL: return s_rms_final_;
    case ANE_T_VE_EMBED: return s_ve_embed_[layer];
    case ANE_T_VE_GATE: return s_ve_gate_[layer];
    case ANE_T_RESID_LAMBDAS: return s_resid_;
    case ANE_T_X0_LAMBDAS: return s_x0l_;
    case ANE_T_SMEAR_GATE: return s_smear_gate_;
    case ANE_T_SMEAR_LAMBDA: return s_smear_l_;
    case ANE_T_BACKOUT_LAMBDA: return s_backout_l_;
    default: *ok = false; return s;
  }
}

template <typename T>
int EngineT<T>::alloc_buffers() {
  const size_t MD = (size_t)M_ * D_;
  int rc = 0;
#define A(ptr, n)                        \
  do {                                   \
    if ((rc = dalloc(&(ptr), (n))) != 0) return rc; \
  } while (0)
  A(P_, n_params_); A(G_, n_params_); A(Mo_, n_params_); A(Vo_, n_params_);
  if (!kIsF32) A(Sh_, shadow_n_);
  A(d_one_, 1); A(d_zero_, 1);
  xs_.assign(L_ + 1, nullptr);
  for (int l = 0; l <= L_; ++l) A(xs_[l], MD);
  acts_.assign(L_, Act<T>());
  for (int l = 0; l < L_; ++l) {
    Act<T>& a = acts_[l];
    A(a.x2, MD); A(a.xn, MD); A(a.att, (size_t)M_ * QD_); A(a.x2n, MD);
    // ANE_B200_ATT_NO_LO=1 leaves the remainder out (delta from the bf16 output alone; for comparisons)
    if (!kIsF32 && !qkv_f32_ && attention_tc_supported(hd_) && getenv("ANE_B200_ATT_NO_LO") == nullptr)
      A(a.att_lo, (size_t)M_ * QD_);
    {
      uint8_t* raw = nullptr;
      A(raw, (size_t)M_ * QKVD_ * (qkv_f32_ ? 4 : sizeof(T)));
      a.qkv = raw;
    }
    A(a.h13, (size_t)M_ * N13_); A(a.gate, (size_t)M_ * Hd_);
    A(a.rstd1, M_); A(a.rstd2, M_); A(a.lse, (size_t)B_ * H_ * S_);
    if (isN_) {
      uint8_t* raw = nullptr;
      A(raw, (size_t)M_ * (QD_ + KVD_) * (qkv_f32_ ? 4 : sizeof(T)));
      a.qkpre = raw;
    }
    if (is_ve_layer(l)) A(a.ve_act, (size_t)M_ * H_);
    if (o_.debug_taps) {
      A(a.t_dout, MD); A(a.t_dx2, MD); A(a.t_dqkv, (size_t)M_ * QKVD_); A(a.t_dh13, (size_t)M_ * N13_);
    }
  }
  if (isN_) {
    A(x0_, MD); A(xraw_, MD); A(gate_pre_, MD); A(gx0_, MD); A(gmid_, MD); A(dgp_, MD); A(dxs_, MD); A(dxs2_, MD);
    if (!kIsF32) { A(x0_t_, MD); A(dgp_t_, MD); }
  }
  A(dcur_[0], MD); A(dcur_[1], MD); A(dxn_, MD); A(dy_, MD); A(dx2_[0], MD); A(dx2_[1], MD);
  A(dqkv_f32_[0], (size_t)M_ * QKVD_); A(dqkv_f32_[1], (size_t)M_ * QKVD_);
  if (!kIsF32) {
    A(dcur_t_[0], MD); A(dcur_t_[1], MD); A(dx2_t_[0], MD); A(dx2_t_[1], MD);
    A(dqkv_[0], (size_t)M_ * QKVD_); A(dqkv_[1], (size_t)M_ * QKVD_);
  }
  A(dgate_, (size_t)M_ * Hd_); A(dh13_[0], (size_t)M_ * N13_); A(dh13_[1], (size_t)M_ * N13_); A(datt_, (size_t)M_ * QD_);
  A(xnf_, MD); A(rstdf_, M_); A(att_delta_, (size_t)B_ * H_ * S_);
  if (att_split_) {
    A(qkvh_, (size_t)M_ * QKVD_); A(qkvl_, (size_t)M_ * QKVD_); A(dqkv_raw_, (size_t)M_ * QKVD_);
    A(att_lse_b_, (size_t)B_ * H_ * S_);
  }
  A(logits_, (size_t)ce_rows_ * V_);
  if (head_fused_) {
    A(ce_stats_, (size_t)2 * ((V_ + 255) / 256) * M_); A(ce_lse2_, M_); A(ce_coef_, M_);
    A(dl_block_, (size_t)M_ * head_cols_);
  } else {
    A(dlogits_, (size_t)ce_rows_ * V_); A(dlogits2_, (size_t)ce_rows_ * V_);
  }
  A(loss_rows_, M_); A(inv_valid_, B_); A(d_loss_, 4); A(tgt_logit_, M_);
  A(rope_cos_, (size_t)S_ * (hd_ / 2)); A(rope_sin_, (size_t)S_ * (hd_ / 2));
  if (hd_ == 64) A(rope_chunks_, (size_t)S_ * 64);
  A(d_acc_, 2); A(d_scales_, 4); A(d_norm_, 2); A(d_status_, 1);
  A(d_in_, M_); A(d_tgt_, M_); A(d_pos_, B_);
  if (group_dw_) {
    A(d_groups_, (size_t)L_ * gemm_group_slot_bytes());
    group_built_.assign(L_, 0);
  }
  tap_tmp_n_ = std::max((size_t)M_ * std::max({QKVD_, N13_, D_}), (size_t)V_ * S_);
  A(tap_tmp_, tap_tmp_n_);
#undef A
  return 0;
}

template <typename T>
int EngineT<T>::open(const ane_options& opts, const uint16_t* tokens, uint64_t n_tokens, const uint8_t* dp_id) {
  o_ = opts;
  // ---- defaults (ane/engine.go:188-239, ane/stories/config.go:3-18)
  if (o_.dim <= 0) o_.dim = 768;
  if (o_.hidden <= 0) o_.hidden = 2048;
  if (o_.n_layers <= 0) o_.n_layers = 12;
  if (o_.n_heads <= 0) o_.n_heads = 12;
  if (o_.n_kv_heads <= 0) o_.n_kv_heads = o_.n_heads;
  if (o_.vocab <= 0) o_.vocab = 32000;
  if (o_.seq <= 0) o_.seq = 256;
  if (o_.batch <= 0) o_.batch = 1;
  if (o_.lr <= 0) o_.lr = 3e-4f;
  if (o_.accum_steps <= 0) o_.accum_steps = 1;
  if (o_.seed == 0) o_.seed = 42;
  if (o_.adam_beta1 <= 0) o_.adam_beta1 = 0.9f;
  if (o_.adam_beta2 <= 0) o_.adam_beta2 = 0.999f;
  if (o_.adam_eps <= 0) o_.adam_eps = 1e-8f;
  if (o_.grad_clip < 0) o_.grad_clip = 0;
  if (o_.loss_scale < 0) o_.loss_scale = 0;
  if (o_.loss_scale == 0) o_.loss_scale = 256;
  if (o_.embed_lr_mult <= 0) o_.embed_lr_mult = 1.0f;
  if (o_.scalar_lr_mult <= 0) o_.scalar_lr_mult = 1.0f;
  if (o_.lambda_lr_mult <= 0) o_.lambda_lr_mult = 0.01f;
  if (o_.lambda_beta1 <= 0) o_.lambda_beta1 = o_.adam_beta1;
  if (o_.lambda_beta2 <= 0) o_.lambda_beta2 = o_.adam_beta2;
  if (o_.world_size <= 0) o_.world_size = 1;
  isN_ = o_.arch == ANE_ARCH_REFERENCE;
  quirks_ = isN_ && o_.quirks != 0;
  qkv_f32_ = kIsF32 || isN_;
  if (o_.rope_theta <= 0) o_.rope_theta = isN_ ? 100000.f : 10000.f;
  D_ = o_.dim; Hd_ = o_.hidden; L_ = o_.n_layers; H_ = o_.n_heads; KV_ = o_.n_kv_heads; V_ = o_.vocab; S_ = o_.seq;
  B_ = o_.batch;
  if (D_ % H_ != 0) return fail(ANE_ERR_ARG, "storiesane open: dim must be a multiple of n_heads");
  hd_ = D_ / H_;
  if (H_ % KV_ != 0) return fail(ANE_ERR_ARG, "storiesane open: n_heads must be a multiple of n_kv_heads");
  if (isN_ && KV_ != H_) return fail(ANE_ERR_ARG, "storiesane open: the reference architecture has no shared KV heads");
  if ((hd_ & 1) || hd_ > 128) return fail(ANE_ERR_ARG, "storiesane open: head_dim must be even and <= 128");
  if (D_ % 8 || Hd_ % 8 || (hd_ % 8)) return fail(ANE_ERR_ARG, "storiesane open: dim, hidden and head_dim must be multiples of 8");
  if (!isN_ && Hd_ % 32) return fail(ANE_ERR_ARG, "storiesane open: hidden must be a multiple of 32 (SwiGLU layout)");
  if (V_ > 65535) return fail(ANE_ERR_ARG, "storiesane open: vocab must fit uint16 token ids");
  if (V_ % 8) return fail(ANE_ERR_ARG, "storiesane open: vocab must be a multiple of 8");
  if (isN_ && D_ < 12) return fail(ANE_ERR_ARG, "storiesane open: dim too small for the value-embedding gate");
  if (n_tokens > 0 && n_tokens < (uint64_t)S_ + 1)
    return fail(ANE_ERR_ARG, "storiesane open: not enough tokens for seq");  // ane/engine.go:192-194
  M_ = B_ * S_;
  QD_ = H_ * hd_; KVD_ = KV_ * hd_; QKVD_ = QD_ + 2 * KVD_;
  N13_ = isN_ ? Hd_ : 2 * Hd_;
  att_tc_ = !qkv_f32_ && attention_tc_supported(hd_);
  att_split_ = !kIsF32 && qkv_f32_ && attention_tcgen05_supported(hd_, S_) && getenv("ANE_B200_ATT_SIMT") == nullptr;
  // bf16 engines: the training head keeps no logits (two passes over the classifier product, the gradient formed
  // per block of vocabulary columns).  ANE_B200_HEAD_UNFUSED=1 keeps the chunked logits -> cross-entropy form.
  head_fused_ = !kIsF32 && getenv("ANE_B200_HEAD_UNFUSED") == nullptr;
  if (head_fused_) {
    // gradient block [M, cols] in bf16: sized to stay in L2 between its producer and its two consumers (<= 64 MB)
    int cols = o_.ce_chunk_cols > 0 ? o_.ce_chunk_cols : (int)std::min<size_t>(65536, ((size_t)64 << 20) / ((size_t)2 * B_ * S_));
    cols = std::max(256, cols / 256 * 256);
    head_cols_ = std::min(cols, (V_ + 255) / 256 * 256);
  }
  // rows per logits chunk where logits still exist: the unfused head (8192 x 32000 bf16 = 524 MB) and the
  // evaluation paths (fp32 logits, 1024 rows at a time when the training head keeps none)
  ce_rows_ = o_.ce_chunk_rows > 0 ? o_.ce_chunk_rows : (head_fused_ ? 1024 : 8192);
  if (ce_rows_ > M_) ce_rows_ = M_;
  ce_rows_ = std::max(ce_rows_, std::min(M_, S_));  // eval logits uses one sequence per chunk
  ce_rows_ = std::max(ce_rows_, std::min(M_, B_));  // decoding: one row of logits per sequence
  lr_ = o_.lr;
  set_lr(lr_);

  int rc;
  if ((rc = cuda_check(cudaSetDevice(o_.device), "cudaSetDevice")) != 0) return rc;
  // ANE_B200_STREAM_PRIO=1: the main chain's stream above the weight-gradient stream, so that freed SMs go to the
  // critical path first (measurement switch)
  int prio_lo = 0, prio_hi = 0;
  cudaDeviceGetStreamPriorityRange(&prio_lo, &prio_hi);
  const char* spe = getenv("ANE_B200_STREAM_PRIO");
  const bool stream_prio = spe && spe[0] == '1';
  if ((rc = cuda_check(cudaStreamCreateWithPriority(&stream_, cudaStreamNonBlocking, stream_prio ? prio_hi : 0), "cudaStreamCreate")) != 0) return rc;
  for (cudaEvent_t* e : {&ev0_, &ev1_, &ev_adam0_, &ev_adam1_})
    if ((rc = cuda_check(cudaEventCreate(e), "cudaEventCreate")) != 0) return rc;
  if ((rc = cuda_check(cudaStreamCreateWithPriority(&dw_stream_, cudaStreamNonBlocking, stream_prio ? prio_lo : 0), "cudaStreamCreate")) != 0) return rc;
  if ((rc = cuda_check(cudaEventCreateWithFlags(&ev_dw_in_, cudaEventDisableTiming), "cudaEventCreate")) != 0) return rc;
  for (cudaEvent_t* e : {&ev_cls_ce_[0], &ev_cls_ce_[1], &ev_cls_dw_[0], &ev_cls_dw_[1]})
    if ((rc = cuda_check(cudaEventCreateWithFlags(e, cudaEventDisableTiming), "cudaEventCreate")) != 0) return rc;
  for (auto& e : ev_logits_)
    if ((rc = cuda_check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate")) != 0) return rc;
  ev_dw_done_.assign(o_.n_layers, nullptr);
  for (auto& ev : ev_dw_done_)
    if ((rc = cuda_check(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreate")) != 0) return rc;
  {
    const char* env = getenv("ANE_B200_DW_OVERLAP");
    dw_overlap_ = !(env && env[0] == '0');
    x3_ = kIsF32 && o_.compute_dtype == ANE_DTYPE_BF16X3;
    {
      const char* ge = getenv("ANE_B200_GROUP_DW");
      group_dw_ = !kIsF32 && ge && ge[0] == '1';
    }
    if (x3_) dw_overlap_ = false;  // the split scratch serves one stream
  }
  layout_params();
  if ((rc = alloc_buffers()) != 0) return rc;
  if ((rc = cuda_check(cudaMallocHost(&h_in_, sizeof(uint16_t) * M_), "cudaMallocHost")) != 0) return rc;
  if ((rc = cuda_check(cudaMallocHost(&h_tgt_, sizeof(uint16_t) * M_), "cudaMallocHost")) != 0) return rc;
  if ((rc = cuda_check(cudaMallocHost(&h_pos_, sizeof(uint64_t) * B_), "cudaMallocHost")) != 0) return rc;
  if ((rc = cuda_check(cudaMallocHost(&h_loss_, sizeof(float) * 4), "cudaMallocHost")) != 0) return rc;
  if ((rc = cuda_check(cudaMallocHost(&h_logits_, sizeof(float) * (size_t)V_ * S_), "cudaMallocHost")) != 0) return rc;
  for (float* p : {P_, G_, Mo_, Vo_})
    if ((rc = cuda_check(cudaMemsetAsync(p, 0, sizeof(float) * n_params_, stream_), "memset")) != 0) return rc;
  cudaMemsetAsync(d_status_, 0, sizeof(int), stream_);
  const float one = 1.f, zero = 0.f;
  cudaMemcpyAsync(d_one_, &one, sizeof(float), cudaMemcpyHostToDevice, stream_);
  cudaMemcpyAsync(d_zero_, &zero, sizeof(float), cudaMemcpyHostToDevice, stream_);
  // defaults: residual lambdas and norm weights start at 1 (ane/stories/weights.go:155-162)
  {
    std::vector<float> ones((size_t)std::max(D_, L_), 1.0f);
    if (isN_) cudaMemcpyAsync(P_ + s_resid_.off, ones.data(), sizeof(float) * L_, cudaMemcpyHostToDevice, stream_);
    else {
      for (int l = 0; l < L_; ++l) {
        cudaMemcpyAsync(P_ + s_rms_att_[l].off, ones.data(), sizeof(float) * D_, cudaMemcpyHostToDevice, stream_);
        cudaMemcpyAsync(P_ + s_rms_ffn_[l].off, ones.data(), sizeof(float) * D_, cudaMemcpyHostToDevice, stream_);
      }
      cudaMemcpyAsync(P_ + s_rms_final_.off, ones.data(), sizeof(float) * D_, cudaMemcpyHostToDevice, stream_);
    }
    cudaStreamSynchronize(stream_);
  }
  count_launch();
  build_rope_tables(rope_cos_, rope_sin_, S_, hd_, (double)o_.rope_theta, stream_);
  if (rope_chunks_ != nullptr) attention_rope_chunk_tables(rope_cos_, rope_sin_, rope_chunks_, S_, stream_);
  if ((rc = refresh_shadow()) != 0) return rc;
  if (n_tokens > 0 && tokens) {
    n_tokens_ = n_tokens;
    if ((rc = dalloc(&d_tokens_, n_tokens)) != 0) return rc;
    if ((rc = cuda_check(cudaMemcpyAsync(d_tokens_, tokens, sizeof(uint16_t) * n_tokens, cudaMemcpyHostToDevice, stream_),
                         "token upload")) != 0)
      return rc;
  }
  rng_ = (((uint64_t)o_.seed & 0xffffffffull) << 16) | 0x330Eull;  // ane/engine.go:873
  if (o_.world_size > 1) {
    if (!dp_id) return fail(ANE_ERR_ARG, "storiesane open: world_size > 1 needs a bootstrap id");
    if ((rc = dp_.init(o_.rank, o_.world_size, dp_id, o_.device)) != 0) return fail(ANE_ERR_NCCL, dp_.last_error());
    int lo_prio = 0, hi_prio = 0;
    cudaDeviceGetStreamPriorityRange(&lo_prio, &hi_prio);
    if ((rc = cuda_check(cudaStreamCreateWithPriority(&comm_stream_, cudaStreamNonBlocking, hi_prio), "comm stream")) != 0)
      return rc;
    if ((rc = cuda_check(cudaEventCreateWithFlags(&ev_bucket_, cudaEventDisableTiming), "event")) != 0) return rc;
    if ((rc = cuda_check(cudaEventCreateWithFlags(&ev_comm_done_, cudaEventDisableTiming), "event")) != 0) return rc;
    const char* e = getenv("ANE_B200_DP_LAYERS_PER_BUCKET");  // layers per gradient bucket (default 1)
    bucket_layers_ = e && atoi(e) > 0 ? atoi(e) : 1;
    const char* se = getenv("ANE_B200_DP_SHARD_OPTIMIZER");   // 0: replicated update on every rank
    shard_opt_ = !(se && se[0] == '0');
    for (int b = 0; b < n_buckets(); ++b)  // slices must keep 16-byte alignment
      if ((bucket_hi(b) - bucket_lo(b)) % ((size_t)o_.world_size * 4) != 0) shard_opt_ = false;
    for (cudaEvent_t* ev : {&ev_opt_done_, &ev_norm_in_, &ev_norm_out_})
      if ((rc = cuda_check(cudaEventCreateWithFlags(ev, cudaEventDisableTiming), "event")) != 0) return rc;
    ev_gather_.assign(n_buckets(), nullptr);
    for (auto& ev : ev_gather_)
      if ((rc = cuda_check(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "event")) != 0) return rc;
  }
  if ((rc = cuda_check(cudaStreamSynchronize(stream_), "open sync")) != 0) return rc;
  t_open_ns_ = now_ns();
  st_.struct_size = sizeof(ane_state);
  return 0;
}

template <typename T>
int EngineT<T>::refresh_shadow() {
  if constexpr (!kIsF32) {
    wait_all_buckets();
    count_launch();
    cast_f32_to_bf16(P_, Sh_, shadow_n_, stream_);
  }
  return 0;
}

template <typename T>
int EngineT<T>::set_lr(float lr) {  // ane/engine.go:366-378
  if (lr <= 0) return fail(ANE_ERR_ARG, "storiesane set lr: lr must be > 0");
  lr_ = lr;
  embed_lr_ = lr * o_.embed_lr_mult;
  scalar_lr_ = lr * o_.scalar_lr_mult;
  lambda_lr_ = lr * o_.scalar_lr_mult * o_.lambda_lr_mult;
  return 0;
}

// ------------------------------------------------------------------------------------------------
// Forward (ane/train_full.go:383-453; eval path ane/engine.go:954-1038 performs the same arithmetic)
// ------------------------------------------------------------------------------------------------
template <typename T>
int EngineT<T>::forward(const uint16_t* d_tok, int B, int Tl, int pos0) {
  // Tl = tokens per sequence in this pass (S_ for training/eval, the prompt length for prefill, 1 for a
  // decode step); pos0 = position of the first token (non-zero only while decoding).
  const int M = B * Tl;
  int rc;
  const float att_scale = (float)(1.0 / sqrt((double)hd_));
  if (isN_) {
    count_launch();
    embed_forward(d_tok, P_ + s_embed_.off, x0_, xraw_, M, D_, V_, true, stream_);
    cast_to_t(x0_, x0_t_, (uint64_t)M * D_);
    GemmDesc g;
    g.A = tview(x0_, x0_t_); g.B = wop(s_smear_gate_.off); g.C = gate_pre_;
    g.M = M; g.N = D_; g.K = D_; g.lda = D_; g.ldb = D_; g.ldc = D_; g.out = GEMM_OUT_F32;
    count_launch();
    if ((rc = gemm(g)) != 0) return rc;
    count_launch();
    smear_forward(x0_, gate_pre_, P_ + s_smear_l_.off, xs_[0], M, Tl, D_, stream_);
  } else {
    count_launch();
    embed_forward(d_tok, P_ + s_embed_.off, xs_[0], nullptr, M, D_, V_, false, stream_);
  }
  for (int l = 0; l < L_; ++l) {
    Act<T>& a = acts_[l];
    const float* w_att = isN_ ? nullptr : P_ + s_rms_att_[l].off;
    const float* w_ffn = isN_ ? nullptr : P_ + s_rms_ffn_[l].off;
    const float* rl = isN_ ? P_ + s_resid_.off + l : d_one_;
    const float* xl = isN_ ? P_ + s_x0l_.off + l : nullptr;
    if (l % bucket_layers_ == 0) wait_bucket(l / bucket_layers_);
    count_launch();
    rmsnorm_forward<T>(xs_[l], w_att, a.xn, a.rstd1, M, D_, stream_);
    // llama arch, bf16, head_dim 64: the rotation of q and k happens on the fp32 accumulators in the epilogue
    static const bool no_fuse_rope = getenv("ANE_B200_NO_FUSE_ROPE") != nullptr;  // A/B measurements
    const bool fused_rope = !kIsF32 && !qkv_f32_ && !isN_ && hd_ == 64 && !no_fuse_rope;
    {
      GemmDesc g;
      g.A = a.xn; g.B = wop(s_qkv_[l].off); g.C = a.qkv;
      g.M = M; g.N = QKVD_; g.K = D_; g.lda = D_; g.ldb = D_; g.ldc = QKVD_;
      g.out = qkv_f32_ ? GEMM_OUT_F32 : GEMM_OUT_BF16;
      if (fused_rope) {
        g.out = GEMM_OUT_BF16_ROPE;
        g.rope_cos = rope_cos_;
        g.rope_sin = rope_sin_;
        g.rope_seq = Tl;
        g.rope_pos0 = pos0;
        g.rope_cols = (H_ + KV_) * hd_;
      }
      count_launch();
      if ((rc = gemm(g)) != 0) return rc;
    }
    // bf16 engine with fp32 q|k|v on the split-precision tensor-core attention: the rotation kernel also writes the
    // bf16 copy that the attention forward reads.  The value embedding only touches v and does not read q or k,
    // so it goes first and its result is part of that copy.
    bool hi_ready = false;
    bool fuse_hi = false;
    if constexpr (!kIsF32) fuse_hi = !fused_rope && qkv_f32_ && att_split_ && Tl == S_ && !decoding_ && hd_ == 64;
    if (fuse_hi && is_ve_layer(l)) {
      count_launch();
      ve_forward<float>((float*)a.qkv, xs_[l], d_tok, P_ + s_ve_embed_[l].off, P_ + s_ve_gate_[l].off, a.ve_act, M, D_,
                        H_, KV_, hd_, V_, stream_);
    }
    if (!fused_rope) {
      count_launch();
      if (fuse_hi) {
        rope_qknorm_forward_hd64((float*)a.qkv, (float*)a.qkpre, rope_cos_, rope_sin_, M, Tl, H_, KV_, isN_, pos0, qkvh_, stream_);
        hi_ready = true;
      } else if (qkv_f32_)
        rope_qknorm_forward<float>((float*)a.qkv, (float*)a.qkpre, rope_cos_, rope_sin_, M, Tl, H_, KV_, hd_, isN_, pos0, stream_);
      else
        rope_qknorm_forward<T>((T*)a.qkv, (T*)a.qkpre, rope_cos_, rope_sin_, M, Tl, H_, KV_, hd_, isN_, pos0, stream_);
    }
    if (!fuse_hi && is_ve_layer(l)) {  // reference architecture only, so qkv is fp32 here
      count_launch();
      ve_forward<float>((float*)a.qkv, xs_[l], d_tok, P_ + s_ve_embed_[l].off, P_ + s_ve_gate_[l].off, a.ve_act, M, D_,
                        H_, KV_, hd_, V_, stream_);
    }
    count_launch();
    if (decoding_) {
      // one new token per sequence: append its k|v to the cache and attend over positions 0..pos0
      kv_cache_append<T>((const T*)a.qkv, kcache_[l], vcache_[l], B, S_, pos0, H_, KV_, hd_, stream_);
      count_launch();
      attention_decode_simt<T>((const T*)a.qkv, kcache_[l], vcache_[l], a.att, B, S_, pos0, H_, KV_, hd_, att_scale,
                               stream_);
    } else if (qkv_f32_) {
      bool done = false;
      if constexpr (!kIsF32) {
        if (att_split_ && Tl == S_) {  // scaled scores are not amplified: the bf16 hi part suffices in the forward
          if (!hi_ready) {
            count_launch();
            cast_f32_to_bf16((const float*)a.qkv, qkvh_, (uint64_t)M * QKVD_, stream_);
          }
          done = attention_forward_tcgen05(qkvh_, a.att, nullptr, a.lse, B, Tl, H_, KV_, att_scale, d_status_, stream_) == 0;
        }
      }
      if (!done)
        attention_forward_simt<float, T>((const float*)a.qkv, a.att, a.lse, B, Tl, H_, KV_, hd_, att_scale, stream_);
    } else if constexpr (!kIsF32) {
      if (att_tc_)
        attention_forward_tc((const bf16*)a.qkv, a.att, (bf16*)a.att_lo, a.lse, B, Tl, H_, KV_, att_scale, d_status_, stream_);
      else
        attention_forward_simt<T, T>((const T*)a.qkv, a.att, a.lse, B, Tl, H_, KV_, hd_, att_scale, stream_);
    }
    {
      GemmDesc g;  // x2 = rl*x + Wo*att (+ xl*x0)   ane/train_full.go:414-426
      g.A = a.att; g.B = wop(s_wo_[l].off); g.C = a.x2;
      g.M = M; g.N = D_; g.K = QD_; g.lda = QD_; g.ldb = QD_; g.ldc = D_; g.out = GEMM_OUT_F32;
      g.res1 = xs_[l]; g.s1 = rl; g.ldres = D_;
      if (isN_) { g.res2 = x0_; g.s2 = xl; }
      count_launch();
      if ((rc = gemm(g)) != 0) return rc;
    }
    count_launch();
    rmsnorm_forward<T>(a.x2, w_ffn, a.x2n, a.rstd2, M, D_, stream_);
    {
      GemmDesc g;
      g.A = a.x2n; g.B = wop(s_w13_[l].off); g.C = a.h13;
      g.M = M; g.N = N13_; g.K = D_; g.lda = D_; g.ldb = D_; g.ldc = N13_;
      g.out = kIsF32 ? GEMM_OUT_F32 : GEMM_OUT_BF16;
      // llama arch, bf16: the GEMM epilogue also writes gate = silu(h1) * h3 (W1 | W3 rows are interleaved in
      // 32-row blocks, so every 64-column piece of h13 holds matching h1 and h3 columns).
      static const bool no_fuse_gate = getenv("ANE_B200_NO_FUSE_SWIGLU") != nullptr;  // A/B measurements
      const bool fused_gate = !kIsF32 && !isN_ && !no_fuse_gate && Hd_ % 64 == 0;
      // reference arch, bf16: gate = max(h1, 0)^2 from the same epilogue
      static const bool no_fuse_relu2 = getenv("ANE_B200_NO_FUSE_RELU2") != nullptr;  // A/B measurements
      const bool fused_relu2 = !kIsF32 && isN_ && !no_fuse_relu2 && Hd_ % 8 == 0;
      if (fused_gate) {
        g.out = GEMM_OUT_BF16_SWIGLU;
        g.aux = a.gate;
        g.ldaux = Hd_;
      } else if (fused_relu2) {
        g.out = GEMM_OUT_BF16_RELU2;
        g.aux = a.gate;
        g.ldaux = Hd_;
      }
      count_launch();
      if ((rc = gemm(g)) != 0) return rc;
      if (!fused_gate && !fused_relu2) {
        count_launch();
        if (isN_) relu2_forward<T>(a.h13, a.gate, (uint64_t)M * Hd_, stream_);
        else swiglu_forward<T>(a.h13, a.gate, M, Hd_, stream_);
      }
    }
    {
      GemmDesc g;  // out = rl*x2 + W2*gate (+ xl*x0)   ane/train_full.go:434-445
      g.A = a.gate; g.B = wop(s_w2_[l].off); g.C = xs_[l + 1];
      g.M = M; g.N = D_; g.K = Hd_; g.lda = Hd_; g.ldb = Hd_; g.ldc = D_; g.out = GEMM_OUT_F32;
      g.res1 = a.x2; g.s1 = rl; g.ldres = D_;
      if (isN_) { g.res2 = x0_; g.s2 = xl; }
      count_launch();
      if ((rc = gemm(g)) != 0) return rc;
    }
  }
  if (isN_) {  // backout: final -= lambda_b * x_mid   ane/common.go:385-389
    count_launch();
    axpy_dev(xs_[L_], xs_[L_ / 2], P_ + s_backout_l_.off, -1.f, (uint64_t)M * D_, false, stream_);
  }
  const float* w_final = isN_ ? nullptr : P_ + s_rms_final_.off;
  count_launch();
  rmsnorm_forward<T>(xs_[L_], w_final, xnf_, rstdf_, M, D_, stream_);
  last_B_ = B;
  return 0;
}

// ------------------------------------------------------------------------------------------------
// Final head (ane/train_full.go:480-558): classifier GEMM + softcap + cross-entropy in token chunks,
// so only ce_rows x vocab logits exist at any time; then dy and the classifier weight gradient.
// ------------------------------------------------------------------------------------------------
template <typename T>
int EngineT<T>::head_and_backward(int B) {
  const int M = B * S_;
  int rc;
  count_launch();
  count_valid_targets(d_tgt_, inv_valid_, B, S_, V_, stream_);
  if (head_fused_) {
    if ((rc = fused_head(B)) != 0) return rc;
    count_launch();
    reduce_loss(loss_rows_, inv_valid_, d_loss_, B, S_, stream_);
    const float* w_fin = isN_ ? nullptr : P_ + s_rms_final_.off;
    count_launch();
    rmsnorm_backward<T>(dy_, xs_[L_], w_fin, rstdf_, nullptr, nullptr, dcur_[0], tcopy_arg(dcur_t_[0]),
                        isN_ ? nullptr : G_ + s_rms_final_.off, M, D_, stream_);
    return backward_layers(B);
  }
  // The dEmbed GEMM of a chunk runs on the side stream (it only feeds the optimizer); the two dlogits
  // buffers alternate so that the next chunk's cross-entropy does not overwrite its operand.
  cudaStream_t dws = (dw_overlap_ && !profiling_) ? dw_stream_ : stream_;
  int chunk = 0;
  for (int r0 = 0; r0 < M; r0 += ce_rows_, ++chunk) {
    const int rows = std::min(ce_rows_, M - r0);
    const int cb = chunk & 1;
    T* dlogits = cb ? dlogits2_ : dlogits_;
    if (dws != stream_ && chunk >= 2) cudaStreamWaitEvent(stream_, ev_cls_dw_[cb], 0);
    GemmDesc g;
    g.A = xnf_ + (size_t)r0 * D_; g.B = wop(s_embed_.off); g.C = logits_;
    g.M = rows; g.N = V_; g.K = D_; g.lda = D_; g.ldb = D_; g.ldc = V_; g.out = GEMM_OUT_F32;
    if constexpr (!kIsF32) {
      // bf16 logits (half the traffic of the chunk) plus the target logit of every row in fp32; the buffer is
      // the fp32 one, half used
      g.out = GEMM_OUT_BF16_TGT;
      g.tgt = d_tgt_;
      g.tgt_out = tgt_logit_;
      g.tgt_row0 = r0;
    }
    count_launch();
    if ((rc = gemm(g)) != 0) return rc;
    count_launch();
    if constexpr (!kIsF32)
      cross_entropy_rows_bf16(reinterpret_cast<const bf16*>(logits_), d_tgt_, inv_valid_, tgt_logit_, dlogits, loss_rows_,
                              rows, r0, S_, V_, isN_, o_.loss_scale, stream_);
    else
      cross_entropy_rows<T>(logits_, d_tgt_, inv_valid_, dlogits, loss_rows_, rows, r0, S_, V_, isN_, o_.loss_scale,
                            stream_);
    if (dws != stream_) {
      cudaEventRecord(ev_cls_ce_[cb], stream_);
      cudaStreamWaitEvent(dws, ev_cls_ce_[cb], 0);
    }
    GemmDesc gx;  // dy = dlogits * Embed   (ane/stories/cpu.go:333-360)
    gx.A = dlogits; gx.B = wop(s_embed_.off); gx.C = dy_ + (size_t)r0 * D_;
    gx.M = rows; gx.N = D_; gx.K = V_; gx.lda = V_; gx.ldb = D_; gx.ldc = D_; gx.b_mn = true; gx.out = GEMM_OUT_F32;
    count_launch();
    if ((rc = gemm(gx)) != 0) return rc;
    GemmDesc gw;  // gEmbed += dlogits^T * xn   (ane/stories/cpu.go:366-385)
    gw.A = dlogits; gw.B = xnf_ + (size_t)r0 * D_; gw.C = G_ + s_embed_.off;
    gw.M = V_; gw.N = D_; gw.K = rows; gw.lda = V_; gw.ldb = D_; gw.ldc = D_; gw.a_mn = true; gw.b_mn = true;
    gw.out = GEMM_OUT_ACCUM;
    count_launch();
    if ((rc = gemm(gw, dws)) != 0) return rc;
    if (dws != stream_) cudaEventRecord(ev_cls_dw_[cb], dws);
  }
  count_launch();
  reduce_loss(loss_rows_, inv_valid_, d_loss_, B, S_, stream_);
  const float* w_final = isN_ ? nullptr : P_ + s_rms_final_.off;
  count_launch();
  rmsnorm_backward<T>(dy_, xs_[L_], w_final, rstdf_, nullptr, nullptr, dcur_[0], tcopy_arg(dcur_t_[0]),
                      isN_ ? nullptr : G_ + s_rms_final_.off, M, D_, stream_);
  return backward_layers(B);
}

// ------------------------------------------------------------------------------------------------
// The same head without logits in memory (bf16 engines).  Pass 1: the classifier product with an epilogue
// that keeps, per row and 256-column tile, only the maximum and the sum of exponentials, plus the row's
// target logit; a small kernel merges them into the row's log-sum-exp, loss and gradient coefficient.
// Pass 2, per block of vocabulary columns: the product again, its epilogue writing
// coef * (softmax - onehot) in bf16 into a block that stays in L2, then dy (+)= block * Embed[block] and
// gEmbed[block] += block^T * xn.  One more product than the stored-logits form in exchange for ~2 GB less
// HBM traffic per step and no [tokens, vocab] buffer.
// ------------------------------------------------------------------------------------------------
template <typename T>
int EngineT<T>::fused_head(int B) {
  if constexpr (kIsF32) {
    return fail(ANE_ERR_STATE, "storiesane step: the logit-free head runs on bf16 engines");
  } else {
    const int M = B * S_;
    int rc;
    GemmDesc g;
    g.A = xnf_; g.B = wop(s_embed_.off); g.C = nullptr;
    g.M = M; g.N = V_; g.K = D_; g.lda = D_; g.ldb = D_; g.ldc = V_;
    g.out = GEMM_OUT_CE_STATS;
    g.tgt = d_tgt_; g.tgt_out = tgt_logit_; g.tgt_row0 = 0;
    g.ce_stats = ce_stats_; g.ce_rows = M; g.ce_softcap = isN_;
    count_launch();
    if ((rc = gemm(g)) != 0) return rc;
    count_launch();
    ce_merge_stats(ce_stats_, (V_ + 255) / 256, M, tgt_logit_, d_tgt_, inv_valid_, S_, V_, isN_, o_.loss_scale, ce_lse2_,
                   ce_coef_, loss_rows_, stream_);
    for (int v0 = 0; v0 < V_; v0 += head_cols_) {
      const int nc = std::min(head_cols_, V_ - v0);
      GemmDesc p2 = g;  // logits of columns [v0, v0 + nc) again, turned into their gradient
      p2.B = wop(s_embed_.off + (size_t)v0 * D_); p2.C = dl_block_;
      p2.N = nc; p2.ldc = head_cols_;
      p2.out = GEMM_OUT_CE_GRAD;
      p2.tgt_out = nullptr; p2.ce_stats = nullptr;
      p2.ce_lse2 = ce_lse2_; p2.ce_coef = ce_coef_; p2.ce_col0 = v0;
      count_launch();
      if ((rc = gemm(p2)) != 0) return rc;
      GemmDesc gx;  // dy (+)= block * Embed[v0 : v0 + nc]   (ane/stories/cpu.go:333-360)
      gx.A = dl_block_; gx.B = wop(s_embed_.off + (size_t)v0 * D_); gx.C = dy_;
      gx.M = M; gx.N = D_; gx.K = nc; gx.lda = head_cols_; gx.ldb = D_; gx.ldc = D_; gx.b_mn = true; gx.out = GEMM_OUT_F32;
      if (v0 > 0) { gx.res1 = dy_; gx.s1 = d_one_; gx.ldres = D_; }  // in place: every piece is read before it is written
      count_launch();
      if ((rc = gemm(gx)) != 0) return rc;
      GemmDesc gw;  // gEmbed[v0 : v0 + nc] += block^T * xn   (ane/stories/cpu.go:366-385)
      gw.A = dl_block_; gw.B = xnf_; gw.C = G_ + s_embed_.off + (size_t)v0 * D_;
      gw.M = nc; gw.N = D_; gw.K = M; gw.lda = head_cols_; gw.ldb = D_; gw.ldc = D_; gw.a_mn = true; gw.b_mn = true;
      gw.out = GEMM_OUT_ACCUM;
      count_launch();
      if ((rc = gemm(gw)) != 0) return rc;
    }
    return 0;
  }
}

// ------------------------------------------------------------------------------------------------
// Layer backward (ane/train_full.go:691-820 with the CPU layer functions :592-601, :644-675).
// ------------------------------------------------------------------------------------------------
template <typename T>
int EngineT<T>::backward_layers(int B) {
  const int M = B * S_;
  const uint64_t MD = (uint64_t)M * D_;
  int rc;
  int cur = 0;
  const float att_scale_bwd = quirks_ ? 1.0f : (float)(1.0 / sqrt((double)hd_));
  if (isN_) {
    // backout backward (ane/common.go:393-403): d lambda_b = -sum(dOut * xMid); stash -lambda_b * dOut
    count_launch();
    dot_accumulate(dcur_[cur], xs_[L_ / 2], MD, -1.f, G_ + s_backout_l_.off, stream_);
    count_launch();
    axpy_dev(gmid_, dcur_[cur], P_ + s_backout_l_.off, -1.f, MD, true, stream_);
    cudaMemsetAsync(gx0_, 0, sizeof(float) * MD, stream_);
  }
  for (int l = L_ - 1; l >= 0; --l) {
    Act<T>& a = acts_[l];
    const float* w_att = isN_ ? nullptr : P_ + s_rms_att_[l].off;
    const float* w_ffn = isN_ ? nullptr : P_ + s_rms_ffn_[l].off;
    const float* rl = isN_ ? P_ + s_resid_.off + l : d_one_;
    const float* xl = isN_ ? P_ + s_x0l_.off + l : nullptr;
    float* dcur = dcur_[cur];
    T* dcur_t = tview(dcur_[cur], dcur_t_[cur]);
    float* dprev = dcur_[cur ^ 1];
    T* dprev_t = tview(dcur_[cur ^ 1], dcur_t_[cur ^ 1]);
    const int pb = l & 1;  // buffer parity of this layer
    float* dx2 = dx2_[pb];
    T* dx2_t = tview(dx2_[pb], dx2_t_[pb]);
    T* dh13 = dh13_[pb];
    float* dqkv_f32 = dqkv_f32_[pb];
    // Side stream for this layer's weight-gradient GEMMs (main stream when overlap is off or while
    // per-GEMM profiling wants a serial timeline).
    cudaStream_t dws = (dw_overlap_ && !profiling_) ? dw_stream_ : stream_;
    // The parity buffers were last read by the dW GEMMs of layer l+2.
    if (dws != stream_ && l + 2 < L_) cudaStreamWaitEvent(stream_, ev_dw_done_[l + 2], 0);
    if (o_.debug_taps) cudaMemcpyAsync(a.t_dout, dcur, sizeof(float) * MD, cudaMemcpyDeviceToDevice, stream_);
    // ---- FFN backward
    {
      GemmDesc g;  // dgate = dOut * W2
      g.A = dcur_t; g.B = wop(s_w2_[l].off); g.C = dgate_;
      g.M = M; g.N = Hd_; g.K = D_; g.lda = D_; g.ldb = Hd_; g.ldc = Hd_; g.b_mn = true;
      g.out = kIsF32 ? GEMM_OUT_F32 : GEMM_OUT_BF16;
      // llama arch, bf16: the SwiGLU backward runs on the accumulators in the epilogue (d h13 written directly,
      // d gate never stored)
      static const bool no_fuse_dswiglu = getenv("ANE_B200_NO_FUSE_DSWIGLU") != nullptr;  // A/B measurements
      const bool fused_dswiglu = !kIsF32 && !isN_ && !no_fuse_dswiglu && Hd_ % 32 == 0;
      // reference arch, bf16: likewise the ReLU^2 backward, d h = d gate * 2 max(h, 0)
      const bool fused_drelu2 = !kIsF32 && isN_ && !no_fuse_dswiglu && Hd_ % 64 == 0;
      if (fused_dswiglu) {
        g.out = GEMM_OUT_DSWIGLU;
        g.C = dh13; g.ldc = N13_;
        g.aux = a.h13; g.ldaux = N13_;
      } else if (fused_drelu2) {
        g.out = GEMM_OUT_DRELU2;
        g.C = dh13; g.ldc = N13_;
        g.aux = a.h13; g.ldaux = N13_;
      }
      count_launch();
      if ((rc = gemm(g)) != 0) return rc;
      if (!fused_dswiglu && !fused_drelu2) {
        count_launch();
        if (isN_) relu2_backward<T>(dgate_, a.h13, dh13, (uint64_t)M * Hd_, stream_);
        else swiglu_backward<T>(dgate_, a.h13, dh13, M, Hd_, stream_);
      }
    }
    if (o_.debug_taps) {
      count_launch();
      to_f32_kernel<T><<<ew_grid((uint64_t)M * N13_), 256, 0, stream_>>>(dh13, a.t_dh13, (uint64_t)M * N13_);
    }
    {
      GemmDesc g;  // dx2n = dh13 * W13
      g.A = dh13; g.B = wop(s_w13_[l].off); g.C = dxn_;
      g.M = M; g.N = D_; g.K = N13_; g.lda = N13_; g.ldb = D_; g.ldc = D_; g.b_mn = true; g.out = GEMM_OUT_F32;
      count_launch();
      if ((rc = gemm(g)) != 0) return rc;
    }
    // dx2 = rl*dOut + rms_bwd(dx2n; x2)
    count_launch();
    rmsnorm_backward<T>(dxn_, a.x2, w_ffn, a.rstd2, dcur, rl, dx2, tcopy_arg(dx2_t_[pb]),
                        isN_ ? nullptr : G_ + s_rms_ffn_[l].off, M, D_, stream_);
    if (o_.debug_taps) cudaMemcpyAsync(a.t_dx2, dx2, sizeof(float) * MD, cudaMemcpyDeviceToDevice, stream_);
    GemmDesc dw[4];  // this layer's weight-gradient products: dW2, dW13, dWo, dWqkv
    const bool grouped = group_dw_ && M == M_;
    {
      GemmDesc& g = dw[0];  // dW2 += dOut^T * gate
      g.A = dcur_t; g.B = a.gate; g.C = G_ + s_w2_[l].off;
      g.M = D_; g.N = Hd_; g.K = M; g.lda = D_; g.ldb = Hd_; g.ldc = Hd_; g.a_mn = true; g.b_mn = true;
      g.out = GEMM_OUT_ACCUM;
      GemmDesc& g2 = dw[1];  // dW13 += dh13^T * x2n
      g2.A = dh13; g2.B = a.x2n; g2.C = G_ + s_w13_[l].off;
      g2.M = N13_; g2.N = D_; g2.K = M; g2.lda = N13_; g2.ldb = D_; g2.ldc = D_; g2.a_mn = true; g2.b_mn = true;
      g2.out = GEMM_OUT_ACCUM;
      if (!grouped) {
        if (dws != stream_) {  // operands (dOut copy, gate, dh13, x2n) are ready at this point of the main stream
          cudaEventRecord(ev_dw_in_, stream_);
          cudaStreamWaitEvent(dws, ev_dw_in_, 0);
        }
        count_launch();
        if ((rc = gemm(g, dws)) != 0) return rc;
        count_launch();
        if ((rc = gemm(g2, dws)) != 0) return rc;
      }
    }
    if (isN_) {  // lambda gradients, FFN residual (ane/train_full.go:732-748)
      count_launch(3);
      if (MD % 4 == 0) {
        lambda_grads(dcur, a.x2, x0_, gx0_, xl, MD, G_ + s_resid_.off + l, G_ + s_x0l_.off + l, stream_);
      } else {
        dot_accumulate(dcur, a.x2, MD, 1.f, G_ + s_resid_.off + l, stream_);
        dot_accumulate(dcur, x0_, MD, 1.f, G_ + s_x0l_.off + l, stream_);
        axpy_dev(gx0_, dcur, xl, 1.f, MD, false, stream_);
      }
    }
    // ---- attention backward
    {
      GemmDesc g;  // datt = dx2 * Wo
      g.A = dx2_t; g.B = wop(s_wo_[l].off); g.C = datt_;
      g.M = M; g.N = QD_; g.K = D_; g.lda = D_; g.ldb = QD_; g.ldc = QD_; g.b_mn = true;
      g.out = kIsF32 ? GEMM_OUT_F32 : GEMM_OUT_BF16;
      count_launch();
      if ((rc = gemm(g)) != 0) return rc;
    }
    T* dqkv = tview(dqkv_f32, dqkv_[pb]);
    bool dqkv_ready = false;  // true once dqkv holds the final GEMM operand
    bool dq_is_bf16 = false;  // attention gradient left in dqkv_raw_ (bf16) instead of dqkv_f32
    if (qkv_f32_) {
      bool done = false;
      if constexpr (!kIsF32) {
        if (att_split_) {
          count_launch(5);
          split_f32_to_bf16x2((const float*)a.qkv, qkvh_, qkvl_, (uint64_t)M * QKVD_, stream_);
          done = attention_backward_tcgen05_split(qkvh_, qkvl_, datt_, att_lse_b_, att_delta_, dqkv_raw_, B, S_, H_, KV_,
                                                  att_scale_bwd, d_status_, stream_) == 0;
          // head size 64 (the only one these kernels take): the next kernel reads the bf16 gradient directly
          dq_is_bf16 = done;
        }
      }
      if (!done) {
        cudaMemsetAsync(dqkv_f32, 0, sizeof(float) * (size_t)M * QKVD_, stream_);
        count_launch();
        attention_backward_simt<float, T>((const float*)a.qkv, datt_, dqkv_f32, B, S_, H_, KV_, hd_, att_scale_bwd, stream_);
      }
    } else if constexpr (!kIsF32) {
      if (att_tc_) {
        // Tensor-core path: the kernels undo the rotation and emit bf16 operands directly.
        count_launch(attention_backward_tc((const bf16*)a.qkv, a.att, (const bf16*)a.att_lo, datt_, a.lse, att_delta_, dqkv_[pb], rope_cos_, rope_sin_, rope_chunks_, B, S_,
                                           H_, KV_, att_scale_bwd, d_status_, stream_));
        dqkv_ready = true;
        if (o_.debug_taps) {
          count_launch();
          to_f32_kernel<T><<<ew_grid((uint64_t)M * QKVD_), 256, 0, stream_>>>(dqkv_[pb], a.t_dqkv, (uint64_t)M * QKVD_);
        }
      } else {
        cudaMemsetAsync(dqkv_f32, 0, sizeof(float) * (size_t)M * QKVD_, stream_);
        count_launch();
        attention_backward_simt<T, T>((const T*)a.qkv, datt_, dqkv_f32, B, S_, H_, KV_, hd_, att_scale_bwd, stream_);
      }
    }
    if (!dqkv_ready) {
      // QK-norm / rotation backward in fp32 and, fused, the one rounding to the GEMM operand type.
      // The fp32 result is kept when something still reads it (value-embedding backward, taps).
      const bool keep_f32 = kIsF32 || is_ve_layer(l) || o_.debug_taps;
      count_launch();
      bool fast = false;
      if constexpr (!kIsF32) {
        if (dq_is_bf16) {
          rope_qknorm_backward_hd64<bf16, T>(dqkv_raw_, keep_f32 ? dqkv_f32 : nullptr, (const float*)a.qkpre, rope_cos_,
                                             rope_sin_, M, S_, H_, KV_, isN_, quirks_, quirks_, tcopy_arg(dqkv_[pb]), stream_);
          fast = true;
        }
      }
      if (!fast && hd_ == 64) {
        rope_qknorm_backward_hd64<float, T>(dqkv_f32, keep_f32 ? dqkv_f32 : nullptr, (const float*)a.qkpre, rope_cos_,
                                            rope_sin_, M, S_, H_, KV_, isN_, quirks_, quirks_, tcopy_arg(dqkv_[pb]), stream_);
        fast = true;
      }
      if (!fast)
        rope_qknorm_backward<float, T>(dqkv_f32, (const float*)a.qkpre, rope_cos_, rope_sin_, M, S_, H_, KV_, hd_, isN_,
                                       quirks_, quirks_, tcopy_arg(dqkv_[pb]), keep_f32, stream_);
      if (o_.debug_taps)
        cudaMemcpyAsync(a.t_dqkv, dqkv_f32, sizeof(float) * (size_t)M * QKVD_, cudaMemcpyDeviceToDevice, stream_);
    }
    {
      GemmDesc g;  // dxn = dq*Wq + dk*Wk + dv*Wv   (ane/train_full.go:650-665)
      g.A = dqkv; g.B = wop(s_qkv_[l].off); g.C = dxn_;
      g.M = M; g.N = D_; g.K = QKVD_; g.lda = QKVD_; g.ldb = D_; g.ldc = D_; g.b_mn = true; g.out = GEMM_OUT_F32;
      count_launch();
      if ((rc = gemm(g)) != 0) return rc;
    }
    // dprev = rms_bwd(dxn; x) + rl*dx2  (+ value-embedding gate path, + mid-layer backout gradient)
    const bool post_fix = is_ve_layer(l) || (isN_ && l == L_ / 2);
    // dprev's buffers were read (as that layer's dOut) by the dW2 GEMM of layer l+1.
    if (dws != stream_ && l + 1 < L_) cudaStreamWaitEvent(stream_, ev_dw_done_[l + 1], 0);
    count_launch();
    rmsnorm_backward<T>(dxn_, xs_[l], w_att, a.rstd1, dx2, rl, dprev, post_fix ? nullptr : tcopy_arg(dcur_t_[cur ^ 1]),
                        isN_ ? nullptr : G_ + s_rms_att_[l].off, M, D_, stream_);
    if (is_ve_layer(l)) {
      count_launch();
      ve_backward<float>(dqkv_f32, xs_[l], d_in_, P_ + s_ve_embed_[l].off, P_ + s_ve_gate_[l].off, a.ve_act,
                         G_ + s_ve_embed_[l].off, G_ + s_ve_gate_[l].off, dprev, M, D_, H_, KV_, hd_, V_, stream_);
    }
    {
      GemmDesc& g = dw[2];  // dWo += dx2^T * att
      g.A = dx2_t; g.B = a.att; g.C = G_ + s_wo_[l].off;
      g.M = D_; g.N = QD_; g.K = M; g.lda = D_; g.ldb = QD_; g.ldc = QD_; g.a_mn = true; g.b_mn = true;
      g.out = GEMM_OUT_ACCUM;
      GemmDesc& g2 = dw[3];  // dWqkv += dqkv^T * xn
      g2.A = dqkv; g2.B = a.xn; g2.C = G_ + s_qkv_[l].off;
      g2.M = QKVD_; g2.N = D_; g2.K = M; g2.lda = QKVD_; g2.ldb = D_; g2.ldc = D_; g2.a_mn = true; g2.b_mn = true;
      g2.out = GEMM_OUT_ACCUM;
      if (dws != stream_) {
        cudaEventRecord(ev_dw_in_, stream_);
        cudaStreamWaitEvent(dws, ev_dw_in_, 0);
      }
      if (grouped) {
        count_launch();
        if ((rc = gemm_group(dw, 4, l, dws)) != 0) return rc;
      } else {
        count_launch();
        if ((rc = gemm(g, dws)) != 0) return rc;
        count_launch();
        if ((rc = gemm(g2, dws)) != 0) return rc;
      }
      if (dws != stream_) cudaEventRecord(ev_dw_done_[l], dws);
    }
    if (isN_) {  // lambda gradients, attention residual (ane/train_full.go:770-782)
      count_launch(3);
      if (MD % 4 == 0) {
        lambda_grads(dx2, xs_[l], x0_, gx0_, xl, MD, G_ + s_resid_.off + l, G_ + s_x0l_.off + l, stream_);
      } else {
        dot_accumulate(dx2, xs_[l], MD, 1.f, G_ + s_resid_.off + l, stream_);
        dot_accumulate(dx2, x0_, MD, 1.f, G_ + s_x0l_.off + l, stream_);
        axpy_dev(gx0_, dx2, xl, 1.f, MD, false, stream_);
      }
      if (l == L_ / 2) {  // gradient of the backout term joins at the output of layer L/2-1
        count_launch();
        add_inplace(dprev, gmid_, MD, stream_);
      }
    }
    if (post_fix) cast_to_t(dprev, dcur_t_[cur ^ 1], MD);
    (void)dprev_t;
    if (overlap_reduce_ && l % bucket_layers_ == 0) {
      // The matrix gradients of this bucket's layers are final: hand them to the reduction on the
      // communication stream while the layers below are still being differentiated.
      cudaEventRecord(ev_bucket_, stream_);
      cudaStreamWaitEvent(comm_stream_, ev_bucket_, 0);
      if (dws != stream_) cudaStreamWaitEvent(comm_stream_, ev_dw_done_[l], 0);
      if ((rc = reduce_bucket(l / bucket_layers_)) != 0) return rc;
      reduced_lo_ = s_qkv_[l].off;
    }
    cur ^= 1;
  }
  if (dw_overlap_ && !profiling_) cudaStreamWaitEvent(stream_, ev_dw_done_[0], 0);  // joins every dW GEMM (in-order stream)
  float* dcur = dcur_[cur];
  if (isN_) {
    if (quirks_) {  // reference order: x0 gradient joins before the smear backward (ane/train_full.go:789-798)
      count_launch();
      add_inplace(dcur, gx0_, MD, stream_);
    }
    count_launch();
    smear_backward(dcur, x0_, gate_pre_, P_ + s_smear_l_.off, dgp_, dxs_, G_ + s_smear_l_.off, M, S_, D_, stream_);
    cast_to_t(dgp_, dgp_t_, MD);
    T* dgp_t = tview(dgp_, dgp_t_);
    T* x0_t = tview(x0_, x0_t_);
    GemmDesc g;  // gSmearGate += dGatePre^T * xPre   (ane/common.go:373)
    g.A = dgp_t; g.B = x0_t; g.C = G_ + s_smear_gate_.off;
    g.M = D_; g.N = D_; g.K = M; g.lda = D_; g.ldb = D_; g.ldc = D_; g.a_mn = true; g.b_mn = true; g.out = GEMM_OUT_ACCUM;
    count_launch();
    if ((rc = gemm(g)) != 0) return rc;
    GemmDesc g2;  // dxPre += SmearGate^T * dGatePre   (ane/common.go:377-381)
    g2.A = dgp_t; g2.B = wop(s_smear_gate_.off); g2.C = dxs2_;
    g2.M = M; g2.N = D_; g2.K = D_; g2.lda = D_; g2.ldb = D_; g2.ldc = D_; g2.b_mn = true; g2.out = GEMM_OUT_F32;
    g2.res1 = dxs_; g2.s1 = d_one_; g2.ldres = D_;
    count_launch();
    if ((rc = gemm(g2)) != 0) return rc;
    if (!quirks_) {
      count_launch();
      add_inplace(dxs2_, gx0_, MD, stream_);
    }
    // embedding-norm backward (ane/train_full.go:800-802)
    count_launch();
    rmsnorm_backward<T>(dxs2_, xraw_, nullptr, nullptr, nullptr, nullptr, dxs_, nullptr, nullptr, M, D_, stream_);
    dcur = dxs_;
  }
  count_launch();
  embed_backward(d_in_, dcur, G_ + s_embed_.off, M, D_, V_, stream_);
  return 0;
}

// ------------------------------------------------------------------------------------------------
// Gradient exchange of one bucket of layers on the communication stream: all-reduce, or (sharded optimizer)
// reduce-scatter, after which the slices this rank does not own are cleared so that later micro-steps
// accumulate onto zeros (the update clears the owned slice).
// ------------------------------------------------------------------------------------------------
template <typename T>
int EngineT<T>::reduce_bucket(int b) {
  const size_t lo = bucket_lo(b), hi = bucket_hi(b);
  if (!shard_opt_) {
    if (dp_.all_reduce_sum(G_ + lo, hi - lo, comm_stream_) != 0) return fail(ANE_ERR_NCCL, dp_.last_error());
    return 0;
  }
  const size_t sl = bucket_slice(b), mine = lo + (size_t)o_.rank * sl;
  if (dp_.reduce_scatter_sum(G_ + lo, sl, comm_stream_) != 0) return fail(ANE_ERR_NCCL, dp_.last_error());
  if (mine > lo) cudaMemsetAsync(G_ + lo, 0, (mine - lo) * sizeof(float), comm_stream_);
  if (mine + sl < hi) cudaMemsetAsync(G_ + mine + sl, 0, (hi - mine - sl) * sizeof(float), comm_stream_);
  return 0;
}

// Brings the Adam moments of every slice to every rank (collective; after it the moments are current until the
// next update).
template <typename T>
int EngineT<T>::gather_moments() {
  if (!dp_.active() || !shard_opt_ || moments_current_) return 0;
  cudaEventRecord(ev_bucket_, stream_);
  cudaStreamWaitEvent(comm_stream_, ev_bucket_, 0);
  for (int b = 0; b < n_buckets(); ++b)
    for (float* base : {Mo_, Vo_})
      if (dp_.all_gather_bytes(base + bucket_lo(b), bucket_slice(b) * sizeof(float), comm_stream_) != 0)
        return fail(ANE_ERR_NCCL, dp_.last_error());
  cudaEventRecord(ev_comm_done_, comm_stream_);
  cudaStreamWaitEvent(stream_, ev_comm_done_, 0);
  moments_current_ = true;
  return 0;
}

// ------------------------------------------------------------------------------------------------
// Optimizer update (ane/engine.go:646-682).
// ------------------------------------------------------------------------------------------------
template <typename T>
int EngineT<T>::do_flush() {
  if (pending_seqs_ == 0) return 0;
  int rc;
  uint32_t global_pending = pending_seqs_ * (uint32_t)o_.world_size;
  const bool shard = dp_.active() && shard_opt_;
  if (dp_.active()) {
    // matrices not yet reduced during backward (all of them when the update was not foreseen), bucket by
    // bucket from the top; then the rest (embedding, norms, ...)
    if (!overlap_reduce_) reduced_lo_ = r_mat1_;
    cudaEventRecord(ev_bucket_, stream_);
    cudaStreamWaitEvent(comm_stream_, ev_bucket_, 0);
    if (dw_overlap_) cudaStreamWaitEvent(comm_stream_, ev_dw_done_[0], 0);
    for (int b = n_buckets() - 1; b >= 0; --b)
      if (bucket_lo(b) < reduced_lo_ && (rc = reduce_bucket(b)) != 0) return rc;
    reduced_lo_ = r_mat0_;
    if (dp_.all_reduce_sum(G_ + r_mat1_, n_params_ - r_mat1_, comm_stream_) != 0)
      return fail(ANE_ERR_NCCL, dp_.last_error());
    cudaEventRecord(ev_comm_done_, comm_stream_);
    cudaStreamWaitEvent(stream_, ev_comm_done_, 0);
    overlap_reduce_ = false;
  }
  cudaEventRecord(ev_adam0_, stream_);
  float pre_scale = (float)(1.0 / (double)global_pending);
  if (o_.loss_scale > 0) pre_scale /= o_.loss_scale;
  cudaMemsetAsync(d_acc_, 0, sizeof(double) * 2, stream_);
  if (o_.grad_clip > 0) {
    // layer tensors + embedding (+ value embeddings and gates); the llama arch clips over every parameter.
    if (shard) {
      // this rank's slices of the matrices, summed over ranks; the replicated groups are added afterwards
      for (int b = 0; b < n_buckets(); ++b) {
        count_launch();
        sumsq_accumulate(G_ + bucket_lo(b) + (size_t)o_.rank * bucket_slice(b), bucket_slice(b), pre_scale, d_acc_, stream_);
      }
      cudaEventRecord(ev_norm_in_, stream_);
      cudaStreamWaitEvent(comm_stream_, ev_norm_in_, 0);
      if (dp_.all_reduce_sum_f64(d_acc_, 1, comm_stream_) != 0) return fail(ANE_ERR_NCCL, dp_.last_error());
      cudaEventRecord(ev_norm_out_, comm_stream_);
      cudaStreamWaitEvent(stream_, ev_norm_out_, 0);
    } else {
      count_launch();
      sumsq_accumulate(G_ + r_mat0_, r_mat1_ - r_mat0_, pre_scale, d_acc_, stream_);
    }
    count_launch();
    sumsq_accumulate(G_ + s_embed_.off, r_veg1_ - s_embed_.off, pre_scale, d_acc_, stream_);
    if (!isN_) {
      count_launch();
      sumsq_accumulate(G_ + r_rms0_, r_rms1_ - r_rms0_, pre_scale, d_acc_, stream_);
    }
  }
  count_launch();
  finalize_clip(d_acc_, pre_scale, o_.grad_clip, d_scales_, d_norm_, stream_);
  st_.adam_t++;
  const int t = (int)st_.adam_t;
  auto hyper = [&](float lr, float b1, float b2, float wd) {
    AdamHyper h;
    h.lr = lr; h.b1 = b1; h.b2 = b2; h.eps = o_.adam_eps; h.wd = wd;
    const float bc1 = (float)(1.0 - pow((double)b1, (double)t));  // ane/train_full.go:1107-1111
    const float bc2 = (float)(1.0 - pow((double)b2, (double)t));
    h.inv_bc1 = 1 / bc1;
    h.inv_bc2 = 1 / bc2;
    return h;
  };
  const float b1 = o_.adam_beta1, b2 = o_.adam_beta2;
  const float* clip_s = d_scales_ + 1;
  const float* pre_s = d_scales_;
  auto run = [&](size_t off, size_t n, AdamHyper h, const float* gs, bool shadow) {
    if (!n) return;
    count_launch();
    adam_update(P_ + off, G_ + off, Mo_ + off, Vo_ + off, (shadow && !kIsF32) ? Sh_ + off : nullptr, n, h, gs, stream_);
  };
  if (shard) {
    for (int b = 0; b < n_buckets(); ++b)
      run(bucket_lo(b) + (size_t)o_.rank * bucket_slice(b), bucket_slice(b), hyper(lr_, b1, b2, o_.weight_decay), clip_s, true);
  } else {
    run(r_mat0_, r_mat1_ - r_mat0_, hyper(lr_, b1, b2, o_.weight_decay), clip_s, true);
  }
  if (isN_) run(s_smear_gate_.off, s_embed_.off - s_smear_gate_.off, hyper(lr_, b1, b2, o_.weight_decay), pre_s, true);
  run(s_embed_.off, r_ve0_ - s_embed_.off, hyper(embed_lr_, b1, b2, 0.f), clip_s, true);
  run(r_ve0_, r_ve1_ - r_ve0_, hyper(embed_lr_, b1, b2, 0.f), clip_s, false);
  run(r_veg0_, r_veg1_ - r_veg0_, hyper(scalar_lr_, b1, b2, 0.f), clip_s, false);
  run(r_rms0_, r_rms1_ - r_rms0_, hyper(lr_, b1, b2, 0.f), clip_s, false);
  if (isN_) {
    run(s_smear_l_.off, r_lam0_ - s_smear_l_.off, hyper(scalar_lr_, b1, b2, 0.f), pre_s, false);
    run(r_lam0_, r_lam1_ - r_lam0_, hyper(lambda_lr_, o_.lambda_beta1, o_.lambda_beta2, 0.f), pre_s, false);
  }
  cudaEventRecord(ev_adam1_, stream_);
  if (shard) {
    // every rank's updated slices -> everyone, in the order the next pass reads them
    cudaEventRecord(ev_opt_done_, stream_);
    cudaStreamWaitEvent(comm_stream_, ev_opt_done_, 0);
    for (int b = 0; b < n_buckets(); ++b) {
      if (dp_.all_gather_bytes(P_ + bucket_lo(b), bucket_slice(b) * sizeof(float), comm_stream_) != 0)
        return fail(ANE_ERR_NCCL, dp_.last_error());
      if constexpr (!kIsF32) {
        count_launch();
        cast_f32_to_bf16(P_ + bucket_lo(b), Sh_ + bucket_lo(b), bucket_hi(b) - bucket_lo(b), comm_stream_);
      }
      cudaEventRecord(ev_gather_[b], comm_stream_);
    }
    gather_pending_ = true;
    moments_current_ = false;
  }
  pending_seqs_ = 0;
  micro_steps_ = 0;
  st_.pending_steps = 0;
  st_.cum_batches++;
  return 0;
}

template <typename T>
int EngineT<T>::flush(double* refresh_ms) {
  int rc = do_flush();
  if (rc != 0) return rc;
  wait_all_buckets();
  if ((rc = cuda_check(cudaStreamSynchronize(stream_), "flush sync")) != 0) return rc;
  if (refresh_ms) *refresh_ms = 0.0;
  return 0;
}

template <typename T>
int EngineT<T>::check_device_status(int* out_status) {
  int v = 0;
  cudaError_t e = cudaMemcpyAsync(&v, d_status_, sizeof(int), cudaMemcpyDeviceToHost, stream_);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream_);
  if (e != cudaSuccess) return cuda_check(e, "device status read");
  if (out_status) *out_status = v;
  if (v != 0) {
    cudaMemsetAsync(d_status_, 0, sizeof(int), stream_);
    char buf[96];
    snprintf(buf, sizeof buf, "storiesane step: device pipeline wait timed out (status %d)", v);
    return fail(ANE_ERR_DEVICE, buf);
  }
  return 0;
}

// ------------------------------------------------------------------------------------------------
// Step (ane/engine.go:381-442)
// ------------------------------------------------------------------------------------------------
template <typename T>
int EngineT<T>::step(const uint16_t* input, const uint16_t* target, uint32_t n_seq, ane_step_result* out) {
  const int64_t t0 = now_ns();
  int rc;
  if ((rc = cuda_check(cudaSetDevice(o_.device), "cudaSetDevice")) != 0) return rc;
  cudaEventRecord(ev0_, stream_);
  if (input) {
    if ((int)n_seq != B_) return fail(ANE_ERR_ARG, "storiesane step: n_seq must equal the engine batch");
    memcpy(h_in_, input, sizeof(uint16_t) * M_);
    memcpy(h_tgt_, target, sizeof(uint16_t) * M_);
    cudaMemcpyAsync(d_in_, h_in_, sizeof(uint16_t) * M_, cudaMemcpyHostToDevice, stream_);
    cudaMemcpyAsync(d_tgt_, h_tgt_, sizeof(uint16_t) * M_, cudaMemcpyHostToDevice, stream_);
  } else {
    if (n_tokens_ < (uint64_t)S_ + 1) return fail(ANE_ERR_STATE, "storiesane step: not enough tokens");
    // One global drand48 stream; rank r takes draws r, r+world, ... of each step (ane/engine.go:395-404).
    sample_windows(&rng_, n_tokens_, (uint32_t)S_, (uint32_t)B_, (uint32_t)o_.rank, (uint32_t)o_.world_size, h_pos_);
    st_.token_pos = h_pos_[B_ - 1] + (uint64_t)S_;
    cudaMemcpyAsync(d_pos_, h_pos_, sizeof(uint64_t) * B_, cudaMemcpyHostToDevice, stream_);
    count_launch();
    gather_windows_kernel<<<(M_ + 255) / 256, 256, 0, stream_>>>(d_tokens_, d_pos_, d_in_, d_tgt_, B_, S_);
  }
  overlap_reduce_ = dp_.active() && (int)micro_steps_ + 1 >= o_.accum_steps;
  reduced_lo_ = r_mat1_;
  if ((rc = forward(d_in_, B_, S_, 0)) != 0) return rc;
  if ((rc = head_and_backward(B_)) != 0) return rc;
  cudaMemcpyAsync(h_loss_, d_loss_, sizeof(float), cudaMemcpyDeviceToHost, stream_);
  pending_seqs_ += (uint32_t)B_;
  micro_steps_++;
  st_.pending_steps = micro_steps_;
  bool flushed = false;
  if ((int)micro_steps_ >= o_.accum_steps) {
    if ((rc = do_flush()) != 0) return rc;
    flushed = true;
  }
  cudaEventRecord(ev1_, stream_);
  int dev_status = 0;
  if ((rc = check_device_status(&dev_status)) != 0) {
    if (out) out->device_status = dev_status;
    return rc;
  }
  if ((rc = cuda_check(cudaGetLastError(), "step")) != 0) return rc;
  float ms = 0.f, adam_ms = 0.f;
  cudaEventElapsedTime(&ms, ev0_, ev1_);
  if (flushed) cudaEventElapsedTime(&adam_ms, ev_adam0_, ev_adam1_);
  const int64_t dur = now_ns() - t0;
  st_.last_loss = h_loss_[0];
  st_.cum_steps++;
  st_.cum_train_ms += (double)dur / 1e6;
  st_.cum_wall_ms = (double)(now_ns() - t_open_ns_) / 1e6;
  if (out) {
    const uint32_t sz = out->struct_size;
    memset(out, 0, sizeof(*out));
    out->struct_size = sz;
    out->loss = h_loss_[0];
    out->step_ns = dur;
    out->device_eval_ns = (int64_t)((double)ms * 1e6);
    out->cpu_work_ns = std::max<int64_t>(0, dur - out->device_eval_ns);
    out->adam_ns = (int64_t)((double)adam_ms * 1e6);
    out->flushed = flushed ? 1 : 0;
    out->device_status = dev_status;
  }
  return 0;
}

// ------------------------------------------------------------------------------------------------
// EvalLogits (ane/engine.go:449-462, :954-1038): one classifier GEMM per sequence straight into the
// reference's [vocab][seq] order (C[v, t] = Embed[v,:] . xn[t,:]).
// ------------------------------------------------------------------------------------------------
template <typename T>
int EngineT<T>::eval_logits(const uint16_t* tokens, uint32_t n_seq, float* out, uint64_t cap, uint32_t layout) {
  int rc;
  if ((rc = cuda_check(cudaSetDevice(o_.device), "cudaSetDevice")) != 0) return rc;
  const uint64_t per_seq = (uint64_t)V_ * S_;
  if (cap < per_seq * n_seq) return fail(ANE_ERR_ARG, "storiesane eval logits: output buffer too small");
  for (uint32_t s0 = 0; s0 < n_seq; s0 += (uint32_t)B_) {
    const int nb = (int)std::min<uint32_t>((uint32_t)B_, n_seq - s0);
    const int M = nb * S_;
    memcpy(h_in_, tokens + (size_t)s0 * S_, sizeof(uint16_t) * M);
    cudaMemcpyAsync(d_in_, h_in_, sizeof(uint16_t) * M, cudaMemcpyHostToDevice, stream_);
    if ((rc = forward(d_in_, nb, S_, 0)) != 0) return rc;
    for (int b = 0; b < nb; ++b) {
      GemmDesc g;
      if (layout == 0) {  // [V][seq]
        g.A = wop(s_embed_.off); g.B = xnf_ + (size_t)b * S_ * D_; g.C = logits_;
        g.M = V_; g.N = S_; g.K = D_; g.lda = D_; g.ldb = D_; g.ldc = S_;
      } else {  // [seq][V]
        g.A = xnf_ + (size_t)b * S_ * D_; g.B = wop(s_embed_.off); g.C = logits_;
        g.M = S_; g.N = V_; g.K = D_; g.lda = D_; g.ldb = D_; g.ldc = V_;
      }
      g.out = GEMM_OUT_F32;
      count_launch();
      if ((rc = gemm(g)) != 0) return rc;
      if (isN_) {
        count_launch();
        softcap_inplace(logits_, per_seq, stream_);
      }
      // device -> pinned staging (full PCIe rate) -> caller's buffer, in pieces: the host copies piece i
      // out of the staging buffer while pieces i+1.. are still crossing PCIe.  One core copies ~10 GB/s, a
      // fifth of the PCIe rate (32.8 MB cross in 0.6-0.7 ms), so the pieces are dealt to several threads
      // (ANE_B200_EVAL_COPY_THREADS; default: the host's cores, at most 16) - measured per call with 2 / 4 / 8 /
      // 12 / 16 threads: 2.54 / 2.10 / 1.99 / 1.91 / 1.75 ms, of which 0.83 ms is the forward pass.
      float* dst = out + (size_t)(s0 + b) * per_seq;
      {
        // A page-locked destination (ane_host_malloc, or memory the caller registered) takes the copy directly.
        cudaPointerAttributes pa;
        if (cudaPointerGetAttributes(&pa, dst) == cudaSuccess && pa.type == cudaMemoryTypeHost) {
          if ((rc = cuda_check(cudaMemcpyAsync(dst, logits_, sizeof(float) * per_seq, cudaMemcpyDeviceToHost, stream_),
                               "logits download")) != 0)
            return rc;
          if ((rc = cuda_check(cudaStreamSynchronize(stream_), "logits sync")) != 0) return rc;
          continue;
        }
        cudaGetLastError();  // an ordinary pointer may leave an error code behind on older drivers
      }
      static const int kPieces = [] {
        const char* e = getenv("ANE_B200_EVAL_PIECES");
        const int v = e ? atoi(e) : 32;
        return v < 1 ? 1 : (v > 64 ? 64 : v);
      }();
      const uint64_t piece = (per_seq + kPieces - 1) / kPieces;
      int n_pieces = 0;
      for (int pi = 0; pi < kPieces; ++pi) {
        const uint64_t off = (uint64_t)pi * piece;
        if (off >= per_seq) break;
        const uint64_t n = std::min(piece, per_seq - off);
        if ((rc = cuda_check(cudaMemcpyAsync(h_logits_ + off, logits_ + off, sizeof(float) * n, cudaMemcpyDeviceToHost,
                                             stream_), "logits download")) != 0)
          return rc;
        cudaEventRecord(ev_logits_[pi], stream_);
        ++n_pieces;
      }
      static const int copy_threads = [] {
        const char* e = getenv("ANE_B200_EVAL_COPY_THREADS");
        const unsigned hw = std::thread::hardware_concurrency();
        const int v = e ? atoi(e) : (hw == 0 ? 4 : (int)hw);
        return v < 1 ? 1 : (v > 16 ? 16 : v);
      }();
      // small outputs (under 1 MiB) are not worth a thread start
      const int use_threads = per_seq * sizeof(float) < (1u << 20) ? 1 : copy_threads;
      std::atomic<int> copy_err{0};
      auto copy_share = [&](int t) {  // pieces t, t + threads, ...: every thread's last piece is a late one
        if (t > 0 && cudaSetDevice(o_.device) != cudaSuccess) {
          copy_err.store(1);
          return;
        }
        for (int pi = t; pi < n_pieces; pi += use_threads) {
          const uint64_t off = (uint64_t)pi * piece;
          const uint64_t n = std::min(piece, per_seq - off);
          if (cudaEventSynchronize(ev_logits_[pi]) != cudaSuccess) {
            copy_err.store(1);
            return;
          }
          memcpy(dst + off, h_logits_ + off, sizeof(float) * n);
        }
      };
      std::vector<std::thread> helpers;
      for (int t = 1; t < use_threads && t < n_pieces; ++t) helpers.emplace_back(copy_share, t);
      copy_share(0);
      for (auto& h : helpers) h.join();
      if (copy_err.load() != 0) return cuda_check(cudaErrorUnknown, "logits sync");
    }
  }
  return check_device_status(nullptr);
}

// Fused evaluation loss: classifier chunk + cross-entropy on the device, only the scalar comes back.
template <typename T>
int EngineT<T>::eval_loss(const uint16_t* tokens, uint32_t n_seq, double* loss_sum, uint64_t* n_pos) {
  int rc;
  if ((rc = cuda_check(cudaSetDevice(o_.device), "cudaSetDevice")) != 0) return rc;
  double total = 0.0;
  uint64_t count = 0;
  for (uint32_t s0 = 0; s0 < n_seq; s0 += (uint32_t)B_) {
    const int nb = (int)std::min<uint32_t>((uint32_t)B_, n_seq - s0);
    const int M = nb * S_;
    memcpy(h_in_, tokens + (size_t)s0 * S_, sizeof(uint16_t) * M);
    cudaMemcpyAsync(d_in_, h_in_, sizeof(uint16_t) * M, cudaMemcpyHostToDevice, stream_);
    count_launch();
    shift_targets_kernel<<<(M + 255) / 256, 256, 0, stream_>>>(d_in_, d_tgt_, nb, S_);
    if ((rc = forward(d_in_, nb, S_, 0)) != 0) return rc;
    cudaMemsetAsync(loss_rows_, 0, sizeof(float) * M, stream_);
    bool fused_done = false;
    if constexpr (!kIsF32) {
      if (head_fused_) {  // pass 1 of the logit-free head is all the loss needs: statistics, target logits, merge
        GemmDesc g;
        g.A = xnf_; g.B = wop(s_embed_.off); g.C = nullptr;
        g.M = M; g.N = V_; g.K = D_; g.lda = D_; g.ldb = D_; g.ldc = V_;
        g.out = GEMM_OUT_CE_STATS;
        g.tgt = d_tgt_; g.tgt_out = tgt_logit_; g.tgt_row0 = 0;
        g.ce_stats = ce_stats_; g.ce_rows = M; g.ce_softcap = isN_;
        count_launch();
        if ((rc = gemm(g)) != 0) return rc;
        count_launch();
        ce_merge_stats(ce_stats_, (V_ + 255) / 256, M, tgt_logit_, d_tgt_, nullptr, S_, V_, isN_, 0.f, ce_lse2_, ce_coef_,
                       loss_rows_, stream_);
        fused_done = true;
      }
    }
    for (int r0 = 0; r0 < M && !fused_done; r0 += ce_rows_) {
      const int rows = std::min(ce_rows_, M - r0);
      GemmDesc g;
      g.A = xnf_ + (size_t)r0 * D_; g.B = wop(s_embed_.off); g.C = logits_;
      g.M = rows; g.N = V_; g.K = D_; g.lda = D_; g.ldb = D_; g.ldc = V_; g.out = GEMM_OUT_F32;
      count_launch();
      if ((rc = gemm(g)) != 0) return rc;
      count_launch();
      cross_entropy_rows<T>(logits_, d_tgt_, d_one_ - 0, (T*)nullptr, loss_rows_, rows, r0, M + 1, V_, isN_, 0.f, stream_);
    }
    std::vector<float> rows_host(M);
    if ((rc = cuda_check(cudaMemcpyAsync(rows_host.data(), loss_rows_, sizeof(float) * M, cudaMemcpyDeviceToHost, stream_),
                         "loss rows")) != 0)
      return rc;
    if ((rc = cuda_check(cudaStreamSynchronize(stream_), "eval loss sync")) != 0) return rc;
    for (int i = 0; i < M; ++i) {
      const int t = i % S_;
      if (t + 1 >= S_) continue;
      if (h_in_[i + 1] >= V_) continue;
      total += (double)rows_host[i];
      count++;
    }
  }
  if (loss_sum) *loss_sum = total;
  if (n_pos) *n_pos = count;
  return check_device_status(nullptr);
}

// ------------------------------------------------------------------------------------------------
// Greedy decoding with a KV cache (llama-style architecture).  Prefill runs the ordinary forward over the
// prompt, k|v of every layer are copied into the cache, then each step runs the layer stack on one
// token per sequence.  Tokens stay on the device until the end; argmax follows ane/train_full.go:344-354
// (lowest index wins ties).  The reference has no KV cache (its Llama2Config.NKVHeads is parsed and
// ignored, ane/stories/config.go:20-28); the check is the full-recompute forward.
// ------------------------------------------------------------------------------------------------
__global__ void store_tokens_kernel(const int32_t* __restrict__ arg, uint16_t* __restrict__ next_tok,
                                    uint16_t* __restrict__ out, int B, int n_new, int step) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const uint16_t t = (uint16_t)arg[b];
  next_tok[b] = t;
  out[(size_t)b * n_new + step] = t;
}

template <typename T>
int EngineT<T>::decode(const uint16_t* prompts, uint32_t n_seq, uint32_t prompt_len, uint32_t n_new,
                       float temperature, const double* uniforms, uint16_t* out) {
  int rc;
  const bool sampling = temperature > 1e-6f;  // ane/train_full.go:319
  if (sampling && !uniforms) return fail(ANE_ERR_ARG, "storiesane decode: sampling needs one uniform draw per token");
  if (isN_) return fail(ANE_ERR_STATE, "storiesane decode: KV-cache decoding is built for the llama-style architecture");
  if (n_seq == 0 || (int)n_seq > B_) return fail(ANE_ERR_ARG, "storiesane decode: n_seq must be in [1, batch]");
  if (prompt_len == 0 || n_new == 0 || (int)(prompt_len + n_new) > S_)
    return fail(ANE_ERR_ARG, "storiesane decode: prompt_len + n_new must fit the engine's seq");
  if ((rc = cuda_check(cudaSetDevice(o_.device), "cudaSetDevice")) != 0) return rc;
  const int B = (int)n_seq, P = (int)prompt_len;
  if (kcache_.empty()) {
    kcache_.assign(L_, nullptr);
    vcache_.assign(L_, nullptr);
    for (int l = 0; l < L_; ++l) {
      if ((rc = dalloc(&kcache_[l], (size_t)B_ * S_ * KVD_)) != 0) return rc;
      if ((rc = dalloc(&vcache_[l], (size_t)B_ * S_ * KVD_)) != 0) return rc;
    }
    if ((rc = dalloc(&d_argmax_, B_)) != 0) return rc;
    if ((rc = dalloc(&d_dec_tok_, B_)) != 0) return rc;
    if ((rc = dalloc(&d_dec_out_, (size_t)B_ * S_)) != 0) return rc;
    if ((rc = dalloc(&d_dec_u_, (size_t)B_ * S_)) != 0) return rc;
  }
  if (sampling)  // [n_new][n_seq]: the draws of one step are contiguous
    cudaMemcpyAsync(d_dec_u_, uniforms, sizeof(double) * (size_t)n_seq * n_new, cudaMemcpyHostToDevice, stream_);
  // The prompt does not fit the pinned window buffer in general (B*P <= B_*S_ does hold).
  memcpy(h_in_, prompts, sizeof(uint16_t) * (size_t)B * P);
  cudaMemcpyAsync(d_in_, h_in_, sizeof(uint16_t) * (size_t)B * P, cudaMemcpyHostToDevice, stream_);
  decoding_ = false;
  if ((rc = forward(d_in_, B, P, 0)) != 0) return rc;
  for (int l = 0; l < L_; ++l) {
    count_launch();
    kv_cache_fill<T>((const T*)acts_[l].qkv, kcache_[l], vcache_[l], B, P, S_, H_, KV_, hd_, stream_);
  }
  auto next_token = [&](int rows_per_seq, int step) -> int {
    // logits of the last position of every sequence -> argmax or sampled index -> token
    GemmDesc g;
    g.A = xnf_ + (size_t)(rows_per_seq - 1) * D_; g.B = wop(s_embed_.off); g.C = logits_;
    g.M = B; g.N = V_; g.K = D_; g.lda = rows_per_seq * D_; g.ldb = D_; g.ldc = V_; g.out = GEMM_OUT_F32;
    count_launch();
    int r = gemm(g);
    if (r != 0) return r;
    count_launch(2);
    sample_rows(logits_, d_dec_u_ + (size_t)step * B, sampling ? temperature : 0.f, d_argmax_, B, V_, stream_);
    store_tokens_kernel<<<(B + 127) / 128, 128, 0, stream_>>>(d_argmax_, d_dec_tok_, d_dec_out_, B, (int)n_new, step);
    return 0;
  };
  if ((rc = next_token(P, 0)) != 0) return rc;
  decoding_ = true;
  for (int step = 1; step < (int)n_new; ++step) {
    const int pos = P + step - 1;  // position of the token generated in the previous step
    if ((rc = forward(d_dec_tok_, B, 1, pos)) != 0) {
      decoding_ = false;
      return rc;
    }
    if ((rc = next_token(1, step)) != 0) {
      decoding_ = false;
      return rc;
    }
  }
  decoding_ = false;
  if ((rc = cuda_check(cudaMemcpyAsync(out, d_dec_out_, sizeof(uint16_t) * (size_t)B * n_new, cudaMemcpyDeviceToHost,
                                       stream_),
                       "decode download")) != 0)
    return rc;
  return check_device_status(nullptr);
}

template <typename T>
int EngineT<T>::get_state(ane_state* s) {
  if (!s) return fail(ANE_ERR_ARG, "storiesane state: null");
  const uint32_t sz = s->struct_size;
  *s = st_;
  s->struct_size = sz ? sz : (uint32_t)sizeof(ane_state);
  return 0;
}
template <typename T>
int EngineT<T>::set_state(const ane_state* s) {  // ane/engine.go:506-512
  if (!s) return fail(ANE_ERR_ARG, "storiesane load state: null");
  st_ = *s;
  micro_steps_ = s->pending_steps;
  pending_seqs_ = s->pending_steps * (uint32_t)B_;
  // the wall clock continues from the restored total (ane/engine.go:560: start = now - CumWall)
  t_open_ns_ = now_ns() - (int64_t)(s->cum_wall_ms * 1e6);
  return 0;
}
template <typename T>
int EngineT<T>::reseed(int64_t seed) {  // drand48Seed, ane/engine.go:873
  rng_ = (((uint64_t)seed & 0xffffffffull) << 16) | 0x330Eull;
  return 0;
}

template <typename T>
int64_t EngineT<T>::tensor_size(uint32_t id, uint32_t layer) {
  bool ok;
  Slot s = slot_of(id, layer, &ok);
  if (!ok) return -1;
  return (int64_t)s.n;
}

template <typename T>
int EngineT<T>::import_tensor(uint32_t id, uint32_t layer, uint32_t which, const float* buf, uint64_t n) {
  bool ok;
  Slot s = slot_of(id, layer, &ok);
  if (!ok || which > 3) return fail(ANE_ERR_ARG, "storiesane import: unknown tensor");
  if (s.n == 0) return fail(ANE_ERR_ARG, "storiesane import: tensor not present in this architecture");
  if (n != s.n) return fail(ANE_ERR_ARG, "storiesane import: element count mismatch");
  float* base = which == 0 ? P_ : which == 1 ? G_ : which == 2 ? Mo_ : Vo_;
  int rc;
  wait_all_buckets();
  if (!isN_ && (id == ANE_T_W1 || id == ANE_T_W3)) {
    // W1 and W3 share the fused W13 matrix in blocks of 32 rows: [W1 rows 0..31 | W3 rows 0..31 | W1 rows 32..63 | ...]
    const size_t blk = (size_t)32 * D_ * sizeof(float);
    float* dst = base + s_w13_[layer].off + (id == ANE_T_W3 ? (size_t)32 * D_ : 0);
    rc = cuda_check(cudaMemcpy2DAsync(dst, 2 * blk, buf, blk, blk, (size_t)Hd_ / 32, cudaMemcpyHostToDevice, stream_), "import");
    if (rc) return rc;
    if (which == 0 && !kIsF32) {
      count_launch();
      cast_f32_to_bf16(P_ + s_w13_[layer].off, Sh_ + s_w13_[layer].off, s_w13_[layer].n, stream_);
    }
    return cuda_check(cudaStreamSynchronize(stream_), "import sync");
  }
  rc = cuda_check(cudaMemcpyAsync(base + s.off, buf, sizeof(float) * n, cudaMemcpyHostToDevice, stream_), "import");
  if (rc) return rc;
  if (which == 0 && !kIsF32 && s.off < shadow_n_) {
    count_launch();
    cast_f32_to_bf16(P_ + s.off, Sh_ + s.off, s.n, stream_);
  }
  return cuda_check(cudaStreamSynchronize(stream_), "import sync");
}

template <typename T>
int EngineT<T>::export_tensor(uint32_t id, uint32_t layer, uint32_t which, float* buf, uint64_t n) {
  bool ok;
  Slot s = slot_of(id, layer, &ok);
  if (!ok || which > 3) return fail(ANE_ERR_ARG, "storiesane export: unknown tensor");
  if (n != s.n) return fail(ANE_ERR_ARG, "storiesane export: element count mismatch");
  if (n == 0) return 0;
  const float* base = which == 0 ? P_ : which == 1 ? G_ : which == 2 ? Mo_ : Vo_;
  int rc;
  wait_all_buckets();
  // Adam moments of the layer matrices live on the rank that owns the slice: reading them is a collective
  // call (every rank must export), which brings all slices up to date once per update.
  if (which >= 2 && s.off >= r_mat0_ && s.off < r_mat1_ && (rc = gather_moments()) != 0) return rc;
  if (!isN_ && (id == ANE_T_W1 || id == ANE_T_W3)) {  // de-interleave the 32-row blocks (see import_tensor)
    const size_t blk = (size_t)32 * D_ * sizeof(float);
    const float* src = base + s_w13_[layer].off + (id == ANE_T_W3 ? (size_t)32 * D_ : 0);
    rc = cuda_check(cudaMemcpy2DAsync(buf, blk, src, 2 * blk, blk, (size_t)Hd_ / 32, cudaMemcpyDeviceToHost, stream_), "export");
  } else {
    rc = cuda_check(cudaMemcpyAsync(buf, base + s.off, sizeof(float) * n, cudaMemcpyDeviceToHost, stream_), "export");
  }
  if (rc) return rc;
  return cuda_check(cudaStreamSynchronize(stream_), "export sync");
}

template <typename T>
int64_t EngineT<T>::get_tap(uint32_t tap, uint32_t layer, float* buf, uint64_t cap) {
  const int B = last_B_;
  if (B <= 0) {
    fail(ANE_ERR_STATE, "storiesane tap: no step has run");
    return -1;
  }
  const int M = B * S_;
  const void* src = nullptr;
  bool src_f32 = true;
  int ld = 0, col0 = 0, ncols = 0, il = 0;
  if (tap < 32 && layer >= (uint32_t)L_) {
    fail(ANE_ERR_ARG, "storiesane tap: bad layer");
    return -1;
  }
  const bool tf = kIsF32;
  if (tap < 32) {
    Act<T>& a = acts_[layer];
    switch (tap) {
      case ANE_TAP_X: src = xs_[layer]; ld = D_; ncols = D_; break;
      case ANE_TAP_XNORM: src = a.xn; src_f32 = tf; ld = D_; ncols = D_; break;
      case ANE_TAP_Q: src = a.qkv; src_f32 = qkv_f32_; ld = QKVD_; ncols = QD_; break;
      case ANE_TAP_K: src = a.qkv; src_f32 = qkv_f32_; ld = QKVD_; col0 = QD_; ncols = KVD_; break;
      case ANE_TAP_V: src = a.qkv; src_f32 = qkv_f32_; ld = QKVD_; col0 = QD_ + KVD_; ncols = KVD_; break;
      case ANE_TAP_ATT: src = a.att; src_f32 = tf; ld = QD_; ncols = QD_; break;
      case ANE_TAP_X2: src = a.x2; ld = D_; ncols = D_; break;
      case ANE_TAP_X2NORM: src = a.x2n; src_f32 = tf; ld = D_; ncols = D_; break;
      case ANE_TAP_H1: src = a.h13; src_f32 = tf; ld = N13_; ncols = Hd_; il = !isN_; break;
      case ANE_TAP_H3: if (!isN_) { src = a.h13; src_f32 = tf; ld = N13_; col0 = 32; ncols = Hd_; il = 1; } break;
      case ANE_TAP_GATE: src = a.gate; src_f32 = tf; ld = Hd_; ncols = Hd_; break;
      case ANE_TAP_QPRE: if (isN_) { src = a.qkpre; src_f32 = qkv_f32_; ld = QD_ + KVD_; ncols = QD_; } break;
      case ANE_TAP_KPRE: if (isN_) { src = a.qkpre; src_f32 = qkv_f32_; ld = QD_ + KVD_; col0 = QD_; ncols = KVD_; } break;
      case ANE_TAP_DOUT: src = a.t_dout; ld = D_; ncols = D_; break;
      case ANE_TAP_DX2: src = a.t_dx2; ld = D_; ncols = D_; break;
      case ANE_TAP_DH1: src = a.t_dh13; ld = N13_; ncols = Hd_; il = !isN_; break;
      case ANE_TAP_DH3: if (!isN_) { src = a.t_dh13; ld = N13_; col0 = 32; ncols = Hd_; il = 1; } break;
      case ANE_TAP_DQ: src = a.t_dqkv; ld = QKVD_; ncols = QD_; break;
      case ANE_TAP_DK: src = a.t_dqkv; ld = QKVD_; col0 = QD_; ncols = KVD_; break;
      case ANE_TAP_DV: src = a.t_dqkv; ld = QKVD_; col0 = QD_ + KVD_; ncols = KVD_; break;
      default: break;
    }
  } else {
    switch (tap) {
      case ANE_TAP_X0: if (isN_) { src = x0_; ld = D_; ncols = D_; } break;
      case ANE_TAP_XMID: if (isN_) { src = xs_[L_ / 2]; ld = D_; ncols = D_; } break;
      case ANE_TAP_FINAL: src = xs_[L_]; ld = D_; ncols = D_; break;
      case ANE_TAP_FINAL_NORM: src = xnf_; src_f32 = tf; ld = D_; ncols = D_; break;
      default: break;
    }
  }
  if (!src || ncols == 0) return 0;
  const uint64_t n = (uint64_t)M * ncols;
  if (cap < n) {
    fail(ANE_ERR_ARG, "storiesane tap: buffer too small");
    return -1;
  }
  if (n > tap_tmp_n_) {
    fail(ANE_ERR_ARG, "storiesane tap: internal buffer too small");
    return -1;
  }
  const unsigned grid = (unsigned)((n + 255) / 256);
  count_launch();
  if (src_f32)
    export_tap_kernel<float><<<grid, 256, 0, stream_>>>(reinterpret_cast<const float*>(src), ld, col0, ncols, M, S_, il, tap_tmp_);
  else
    export_tap_kernel<T><<<grid, 256, 0, stream_>>>(reinterpret_cast<const T*>(src), ld, col0, ncols, M, S_, il, tap_tmp_);
  if (cuda_check(cudaMemcpyAsync(buf, tap_tmp_, sizeof(float) * n, cudaMemcpyDeviceToHost, stream_), "tap") != 0) return -1;
  if (cuda_check(cudaStreamSynchronize(stream_), "tap sync") != 0) return -1;
  return (int64_t)n;
}

template <typename T>
int EngineT<T>::profile_gemm(int enable) {
  cudaStreamSynchronize(stream_);
  for (auto& pr : prof_events_) {
    cudaEventDestroy(pr.first);
    cudaEventDestroy(pr.second);
  }
  prof_events_.clear();
  prof_shapes_.clear();
  prof_flops_ = 0.0;
  profiling_ = enable != 0;
  return 0;
}

template <typename T>
int EngineT<T>::profile_read(double* gemm_ms, double* gemm_flops, uint64_t* gemm_launches) {
  int rc = cuda_check(cudaStreamSynchronize(stream_), "profile sync");
  if (rc) return rc;
  double total = 0.0;
  // ANE_B200_GEMM_TABLE=1 prints one line per distinct GEMM shape to stderr (launches, time, TFLOP/s).
  const bool table = getenv("ANE_B200_GEMM_TABLE") != nullptr;
  struct Row { ProfShape s; int n; double ms; };
  std::vector<Row> rows;
  for (size_t i = 0; i < prof_events_.size(); ++i) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, prof_events_[i].first, prof_events_[i].second) != cudaSuccess) continue;
    total += ms;
    if (!table) continue;
    const ProfShape& s = prof_shapes_[i];
    bool found = false;
    for (auto& r : rows)
      if (r.s.M == s.M && r.s.N == s.N && r.s.K == s.K && r.s.flags == s.flags) {
        r.n++;
        r.ms += ms;
        found = true;
        break;
      }
    if (!found) rows.push_back({s, 1, (double)ms});
  }
  for (auto& r : rows) {
    const double fl = 2.0 * r.s.M * r.s.N * r.s.K * r.n;
    fprintf(stderr, "gemm M=%d N=%d K=%d a_mn=%d b_mn=%d out=%d res=%d  n=%d  %.1f us/launch  %.0f TFLOP/s\n", r.s.M, r.s.N,
            r.s.K, r.s.flags & 1, (r.s.flags >> 1) & 1, (r.s.flags >> 2) & 3, (r.s.flags >> 4) & 1, r.n,
            1e3 * r.ms / r.n, fl / (r.ms * 1e-3) / 1e12);
  }
  if (gemm_ms) *gemm_ms = total;
  if (gemm_flops) *gemm_flops = prof_flops_;
  if (gemm_launches) *gemm_launches = prof_events_.size();
  return 0;
}

template <typename T>
int EngineT<T>::timer_begin() {
  if (!ev_t0_) {
    int rc = cuda_check(cudaEventCreate(&ev_t0_), "cudaEventCreate");
    if (rc) return rc;
    if ((rc = cuda_check(cudaEventCreate(&ev_t1_), "cudaEventCreate")) != 0) return rc;
  }
  return cuda_check(cudaEventRecord(ev_t0_, stream_), "timer begin");
}

template <typename T>
int EngineT<T>::timer_end(float* ms) {
  if (!ev_t0_) return fail(ANE_ERR_STATE, "storiesane timer: end without begin");
  wait_all_buckets();
  int rc = cuda_check(cudaEventRecord(ev_t1_, stream_), "timer end");
  if (rc) return rc;
  if ((rc = cuda_check(cudaEventSynchronize(ev_t1_), "timer sync")) != 0) return rc;
  float v = 0.f;
  if ((rc = cuda_check(cudaEventElapsedTime(&v, ev_t0_, ev_t1_), "timer elapsed")) != 0) return rc;
  if (ms) *ms = v;
  return 0;
}

}  // namespace

EngineBase* create_engine(int compute_dtype) {
  if (compute_dtype == ANE_DTYPE_F32 || compute_dtype == ANE_DTYPE_BF16X3) return new EngineT<float>();
  return new EngineT<bf16>();
}

}  // namespace ane
