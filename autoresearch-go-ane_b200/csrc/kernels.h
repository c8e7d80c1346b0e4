// Host-callable launchers for the non-GEMM kernels of the training step.
//
// Layout convention: activations are token-major [M, C] with M = batch*seq rows
// (row = b*seq + t); the reference keeps them channel-first [C, seq] per sequence
// (ane/common.go:91-105).  "T" is the activation storage type: bf16 in the
// tensor-core path, float in the fp32 parity path.  Residual-stream tensors and
// every reduction are fp32.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ane {

typedef __nv_bfloat16 bf16;

void cast_f32_to_bf16(const float* src, bf16* dst, uint64_t n, cudaStream_t s);
// hi = bf16(x), lo = bf16(x - hi); n % 4 == 0, 16-byte aligned pointers.
void split_f32_to_bf16x2(const float* src, bf16* hi, bf16* lo, uint64_t n, cudaStream_t s);
void cast_bf16_to_f32(const bf16* src, float* dst, uint64_t n, cudaStream_t s);

// x[m,:] = embed[tok[m],:] (zeros for ids >= vocab), ane/stories/cpu.go:41-72.
// If embed_norm: x_raw keeps the gathered row and x = rms(x_raw) (ane/train_full.go:384-388).
void embed_forward(const uint16_t* tok, const float* embed, float* x, float* x_raw, int M, int D, int vocab,
                   bool embed_norm, cudaStream_t s);
// g_embed[tok[m],:] += dx[m,:], ane/stories/cpu.go:74-95.
void embed_backward(const uint16_t* tok, const float* dx, float* g_embed, int M, int D, int vocab, cudaStream_t s);

// y = x * rstd (* w); rstd = (mean(x^2)+1e-5)^-1/2.  ane/common.go:107-174, ane/stories/cpu.go:97-127.
template <typename T>
void rmsnorm_forward(const float* x, const float* w, T* y, float* rstd, int M, int D, cudaStream_t s);
// dx = rms_bwd(dy; x, w) + res_scale * res   (ane/common.go:176-197; ane/stories/cpu.go:129-150)
//   dy: fp32 [M,D];  res/res_scale optional;  dx_f32 and dx_t outputs (dx_t optional copy in T);
//   dw (optional, weighted norm): dw[i] += sum_m dy*x*rstd.
template <typename T>
void rmsnorm_backward(const float* dy, const float* x, const float* w, const float* rstd, const float* res,
                      const float* res_scale, float* dx_f32, T* dx_t, float* dw, int M, int D, cudaStream_t s);

// In-place interleaved-pair RoPE (ane/train_util.go:204-224) on the q and k column blocks of a packed
// [M, (H+2KV)*hd] buffer, followed (qk_norm) by the per-head 1.2*rms norm (ane/common.go:199-227);
// qk_pre, if given, receives the rotated pre-norm q|k ([M, (H+KV)*hd]).
// Row m holds position pos0 + (m % seq).
template <typename T>
void rope_qknorm_forward(T* qkv, T* qk_pre, const float* cosb, const float* sinb, int M, int seq, int H, int KV,
                         int hd, bool qk_norm, int pos0, cudaStream_t s);
// Backward of the above on dq|dk in a packed dqkv buffer: QK-norm backward (ane/common.go:229-270;
// reference_coeff reproduces its qkScale^2 factor) then inverse rotation unless skip_rope.
// out_t (optional) receives the whole packed dq|dk|dv row converted to TO (the v columns pass through);
// write_back = also store the transformed dq|dk in place.
template <typename T, typename TO>
void rope_qknorm_backward(T* dqkv, const T* qk_pre, const float* cosb, const float* sinb, int M, int seq, int H,
                          int KV, int hd, bool qk_norm, bool reference_coeff, bool skip_rope, TO* out_t,
                          bool write_back, cudaStream_t s);
// Head size 64, fp32 q|k|v: rotation (+ QK-norm) in place, and with `hi_out` the bf16 copy of all of q|k|v in the
// same pass (elementwise.cu).
void rope_qknorm_forward_hd64(float* qkv, float* qk_pre, const float* cosb, const float* sinb, int M, int seq, int H, int KV,
                              bool qk_norm, int pos0, bf16* hi_out, cudaStream_t s);
// Head size 64 with fp32 pre-norm q|k; the incoming gradient may be bf16, the fp32 output is optional and may
// be the input itself (elementwise.cu).
template <typename TI, typename TO>
void rope_qknorm_backward_hd64(const TI* din, float* out_f32, const float* qk_pre, const float* cosb, const float* sinb,
                               int M, int seq, int H, int KV, bool qk_norm, bool reference_coeff, bool skip_rope, TO* out_t,
                               cudaStream_t s);
void build_rope_tables(float* cosb, float* sinb, int seq, int hd, double theta, cudaStream_t s);

// FFN activations.  relu2: g = max(h,0)^2 (ane/common.go:146).  swiglu: g = silu(h1)*h3 with h13 = [M, 2*Hd].
template <typename T>
void relu2_forward(const T* h1, T* gate, uint64_t n, cudaStream_t s);
template <typename T>
void relu2_backward(const T* dgate, const T* h1, T* dh1, uint64_t n, cudaStream_t s);  // ane/accel_stub.go:21-29
template <typename T>
void swiglu_forward(const T* h13, T* gate, int M, int Hd, cudaStream_t s);
template <typename T>
void swiglu_backward(const T* dgate, const T* h13, T* dh13, int M, int Hd, cudaStream_t s);

// Causal attention, SIMT reference-precision path (any head_dim <= 128; fp32 math).
//   q,k,v live in one packed buffer [M, ld] at column offsets 0, H*hd, (H+KV)*hd.
//   out [M, H*hd]; lse [B*H*seq] = log-sum-exp of the scaled scores.
// Forward: ane/common.go:61-89.  Backward: ane/train_full.go:261-316 with `scale` explicit.
template <typename T, typename TO>
void attention_forward_simt(const T* qkv, TO* out, float* lse, int B, int seq, int H, int KV, int hd, float scale,
                            cudaStream_t s);
// dq,dk,dv accumulate into fp32 [M, (H+2KV)*hd] (must be zeroed by the caller).
template <typename T, typename TD>
void attention_backward_simt(const T* qkv, const TD* d_out, float* dqkv_f32, int B, int seq, int H, int KV, int hd,
                             float scale, cudaStream_t s);

// KV cache (decode): caches are [B, max_seq, KV*hd]; qkv rows are packed q|k|v as above.
template <typename T>
void kv_cache_fill(const T* qkv, T* kcache, T* vcache, int B, int seq, int max_seq, int H, int KV, int hd,
                   cudaStream_t s);
template <typename T>
void kv_cache_append(const T* qkv, T* kcache, T* vcache, int B, int max_seq, int pos, int H, int KV, int hd,
                     cudaStream_t s);
// One query row per sequence (qkv [B, ld]) against cache positions 0..pos.
template <typename T>
void attention_decode_simt(const T* qkv, const T* kcache, const T* vcache, T* out, int B, int max_seq, int pos, int H,
                           int KV, int hd, float scale, cudaStream_t s);

// Tensor-core causal attention (bf16 operands, head_dim 64 only; see attention_tc.cu).
bool attention_tc_supported(int hd);
// `out_lo` (optional, [M, H*64] like `out`) receives bf16(O - bf16(O)): given to the backward as well, it makes
// delta = rowsum(dO * O) as accurate as an fp32 O would (with bf16 O alone that rounding is the largest
// error of dQ).
void attention_forward_tc(const bf16* qkv, bf16* out, bf16* out_lo, float* lse, int B, int seq, int H, int KV, float scale,
                          int* d_status, cudaStream_t s);
int attention_forward_tcgen05(const bf16* qkv, bf16* out, bf16* out_lo, float* lse, int B, int seq, int H, int KV,
                              float scale, int* d_status, cudaStream_t s);
// Writes every element of dq|dk|dv (bf16, packed like qkv); with cos/sin tables the rotation of q and k
// is undone in the epilogue (pass nullptr to skip).  `delta` is scratch [B*H*seq].
// With head_dim 64 and seq % 128 == 0 the tcgen05 kernels (attention_tcgen05.cu) run, else mma.sync ones;
// `d_status` is the device status word their bounded waits report through.
// Returns the number of kernels it launched.
// `rope_chunks` (optional): the tables as attention_rope_chunk_tables() lays them out, for the seq-256 backward.
int attention_backward_tc(const bf16* qkv, const bf16* out, const bf16* out_lo, const bf16* d_out, const float* lse, float* delta,
                          bf16* dqkv, const float* cosb, const float* sinb, const float* rope_chunks, int B, int seq, int H,
                          int KV, float scale, int* d_status, cudaStream_t s);
void attention_rope_chunk_tables(const float* cosb, const float* sinb, float* out, int seq, cudaStream_t s);
bool attention_tcgen05_supported(int hd, int seq);
// Backward for q|k|v kept in fp32 and given as bf16 (hi, lo) pairs: scores at split precision, own row
// statistics for the backward's `scale` (lse, delta: scratch [B*H*seq]), dq|dk|dv out as bf16, no rotation.
int attention_backward_tcgen05_split(const bf16* qkv_hi, const bf16* qkv_lo, const bf16* d_out, float* lse, float* delta,
                                     bf16* dqkv, int B, int seq, int H, int KV, float scale, int* d_status,
                                     cudaStream_t s);
// `delta` is scratch [B*H*seq] (rowsum(dO * O), produced by the dQ kernel, or by the one-CTA-per-head kernel that
// sequences of 256 without grouped heads take).  Returns the number of kernels launched or a negative error code.
int attention_backward_tcgen05(const bf16* qkv, const bf16* out, const bf16* out_lo, const bf16* d_out, const float* lse, float* delta,
                               bf16* dqkv,
                               const float* cosb, const float* sinb, const float* rope_chunks, int B, int seq, int H, int KV,
                               float scale, int* d_status, cudaStream_t s);

// Cross-entropy over token-major logits [rows, V] (fp32), ane/stories/cpu.go:212-292 with the
// soft cap of ane/common.go:272-287 folded in:
//   z = softcap ? 15*tanh(x/15) : x;  p = softmax(z);  loss_row = -log(max(p[tgt],1e-10))
//   dlogits = grad_scale * inv_valid[row's sequence] * (p - onehot) * (softcap ? 1-tanh^2 : 1)
// Rows with target >= V give a zero gradient row and loss_row = 0 (not counted).
template <typename TO>
void cross_entropy_rows(const float* logits, const uint16_t* targets, const float* inv_valid, TO* dlogits,
                        float* loss_rows, int rows, int row0, int seq, int V, bool softcap, float grad_scale,
                        cudaStream_t s);
// The same from bf16 logits, with the (raw) target logit of every row supplied in fp32.
void cross_entropy_rows_bf16(const bf16* logits, const uint16_t* targets, const float* inv_valid, const float* tgt_logit,
                             bf16* dlogits, float* loss_rows, int rows, int row0, int seq, int V, bool softcap,
                             float grad_scale, cudaStream_t s);
// Between the two passes of the classifier head that keeps no logits: per-tile (max, sum) pairs [n_tiles][rows]
// (log2 domain) -> lse2[row], coef[row] = grad_scale * inv_valid[row / seq] (0 without a target) and loss_rows[row].
void ce_merge_stats(const float* stats, int n_tiles, int rows, const float* tgt_logit, const uint16_t* targets,
                    const float* inv_valid, int seq, int V, bool softcap, float grad_scale, float* lse2, float* coef,
                    float* loss_rows, cudaStream_t s);
void softcap_inplace(float* logits, uint64_t n, cudaStream_t s);
// inv_valid[b] = 1/count(targets[b,:] < V) (0 when none); ane/stories/cpu.go:276-279.
void count_valid_targets(const uint16_t* targets, float* inv_valid, int B, int seq, int V, cudaStream_t s);
// loss_out[0] = mean over sequences of (sum_t loss_rows * inv_valid[b])
void reduce_loss(const float* loss_rows, const float* inv_valid, float* loss_out, int B, int seq, cudaStream_t s);

// Gradient norm and optimizer -------------------------------------------------------------------
// acc[0] += sum (g*pre_scale)^2 in double (ane/train_full.go:167-196, ane/accel_stub.go:88-95).
void sumsq_accumulate(const float* g, uint64_t n, float pre_scale, double* acc, cudaStream_t s);
// scales[0] = pre_scale; scales[1] = pre_scale * (clip>0 && norm>clip ? clip/norm : 1)
void finalize_clip(const double* acc, float pre_scale, float clip, float* scales, float* norm_out, cudaStream_t s);
struct AdamHyper {
  float lr, b1, b2, eps, wd, inv_bc1, inv_bc2;
};
// ane/train_full.go:1113-1150.  g_eff = g * (*gscale);  writes w, m, v, optional bf16 shadow, zeroes g.
void adam_update(float* w, float* g, float* m, float* v, bf16* shadow, uint64_t n, AdamHyper h, const float* gscale,
                 cudaStream_t s);

// Reference-architecture extras ---------------------------------------------------------------------
// Smear: x[m,:] = x_pre[m,:] + lambda * sigmoid(gate_pre[m,:]) * x_pre[m-1,:] (0 at t=0), ane/common.go:324-339.
void smear_forward(const float* x_pre, const float* gate_pre, const float* lambda, float* x, int M, int seq, int D,
                   cudaStream_t s);
// ane/common.go:343-370 (element-wise part): d_gate_pre, dx (pre-GEMM part), d_lambda accumulation.
void smear_backward(const float* d_out, const float* x_pre, const float* gate_pre, const float* lambda,
                    float* d_gate_pre, float* dx, float* g_lambda, int M, int seq, int D, cudaStream_t s);
// out[0] += alpha * sum(a*b)  (double accumulation; ane/train_full.go:733-782, ane/common.go:396-400)
// out_a += sum(d*a), out_b += sum(d*b), y += *alpha * d in one pass (n % 4 == 0, 16-byte aligned buffers).
void lambda_grads(const float* d, const float* a, const float* b, float* y, const float* alpha, uint64_t n, float* out_a,
                  float* out_b, cudaStream_t s);
void dot_accumulate(const float* a, const float* b, uint64_t n, float alpha, float* out, cudaStream_t s);
// y += (*alpha) * x  and  y = (*alpha) * x   (alpha is a device scalar; sign flips it)
void axpy_dev(float* y, const float* x, const float* alpha, float sign, uint64_t n, bool assign, cudaStream_t s);
void add_inplace(float* y, const float* x, uint64_t n, cudaStream_t s);
// Value embeddings, ane/train_full.go:1035-1086 (gate over the first 12 channels of the layer input).
template <typename T>
void ve_forward(T* qkv, const float* x, const uint16_t* tok, const float* ve_embed, const float* ve_gate,
                float* gate_act, int M, int D, int H, int KV, int hd, int vocab, cudaStream_t s);
template <typename T>
void ve_backward(const T* dqkv, const float* x, const uint16_t* tok, const float* ve_embed, const float* ve_gate,
                 const float* gate_act, float* g_ve_embed, float* g_ve_gate, float* d_prev, int M, int D, int H,
                 int KV, int hd, int vocab, cudaStream_t s);

// [rows, cols] fp32 -> [cols, rows] fp32 (tap export in the reference's channel-first layout).
void transpose_f32(const float* in, float* out, int rows, int cols, cudaStream_t s);
// Greedy argmax per row, lowest index wins ties (ane/train_full.go:344-354).
void argmax_rows(const float* logits, int32_t* out, int rows, int V, cudaStream_t s);
// Temperature sampling per row with one caller-supplied uniform draw u[row] in [0,1) (ane/train_full.go:318-342);
// temperature <= 1e-6 is the argmax.
void sample_rows(const float* logits, const double* u, float temperature, int32_t* out, int rows, int V,
                 cudaStream_t s);

}  // namespace ane
