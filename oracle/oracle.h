/*
 * CPU oracle for the training step -- TEST INFRASTRUCTURE ONLY.
 *
 * A restatement, in plain C++, of the reference's Go CPU step
 * (ane/train_full.go, ane/common.go, ane/train_util.go, ane/stories/cpu.go,
 * ane/engine.go).  Only tests/, the smoke check and the cpu_baseline /
 * reference legs of bench.py may load this library; the product library never
 * links or calls it.
 *
 * PARITY UNPINNED: the reference ships no golden vectors, known-answer tests or
 * fixtures for this path and cannot be built here (no Go toolchain), so this
 * restatement is pinned only by line-by-line traceability to the cited Go
 * sources plus self-consistency checks (finite differences, invariants) and an
 * independent fp64 torch-autograd statement of both networks (tests/test_oracle.py).
 */
#ifndef ANE_ORACLE_H_
#define ANE_ORACLE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Architecture switches. ARCH_N = the network the reference trains
 * (ane/train_full.go:383-453); ARCH_L = the Llama2-style network of the
 * benchmark configs (weighted RMSNorm, SwiGLU, optional GQA, theta 10000). */
#define ORC_ARCH_N 0
#define ORC_ARCH_L 1

typedef struct orc_config {
  int32_t dim, hidden, heads, kv_heads, layers, vocab, seq;
  int32_t arch;        /* ORC_ARCH_N / ORC_ARCH_L */
  int32_t quirks;      /* 1 = reproduce the reference's backward exactly (ARCH_N only) */
  float rope_theta;    /* <=0: 100000 (N) / 10000 (L) */
  int32_t accum_steps; /* <=0: 1 */
  float lr, beta1, beta2, eps, weight_decay, grad_clip, loss_scale;
  float embed_lr_mult, scalar_lr_mult, lambda_lr_mult, lambda_beta1, lambda_beta2;
} orc_config;

/* Tensor ids (shared with the GPU library's import/export). */
enum {
  ORC_T_EMBED = 0,
  ORC_T_WQ = 1, ORC_T_WK = 2, ORC_T_WV = 3, ORC_T_WO = 4, ORC_T_W1 = 5, ORC_T_W2 = 6, ORC_T_W3 = 7,
  ORC_T_RMS_ATT = 8, ORC_T_RMS_FFN = 9, ORC_T_RMS_FINAL = 10,
  ORC_T_VE_EMBED = 11, ORC_T_VE_GATE = 12,
  ORC_T_RESID_LAMBDAS = 13, ORC_T_X0_LAMBDAS = 14,
  ORC_T_SMEAR_GATE = 15, ORC_T_SMEAR_LAMBDA = 16, ORC_T_BACKOUT_LAMBDA = 17,
  ORC_T_COUNT = 18
};
/* which */
enum { ORC_W = 0, ORC_G = 1, ORC_M = 2, ORC_V = 3 };

/* Activation taps, reference layout [channels][seq] (ane/train_full.go:12-37). */
enum {
  ORC_TAP_X = 0, ORC_TAP_XNORM, ORC_TAP_Q, ORC_TAP_K, ORC_TAP_V, ORC_TAP_ATT, ORC_TAP_X2, ORC_TAP_X2NORM,
  ORC_TAP_H1, ORC_TAP_GATE, ORC_TAP_FFN_OUT, ORC_TAP_QPRE, ORC_TAP_KPRE, ORC_TAP_H3,
  ORC_TAP_DOUT, ORC_TAP_DH1, ORC_TAP_DX2, ORC_TAP_DQ, ORC_TAP_DK, ORC_TAP_DV, ORC_TAP_DH3,
  /* global taps (layer ignored) */
  ORC_TAP_X0 = 32, ORC_TAP_XMID, ORC_TAP_FINAL, ORC_TAP_FINAL_NORM, ORC_TAP_LOGITS_PRE, ORC_TAP_LOGITS,
  ORC_TAP_DLOGITS, ORC_TAP_DFINAL
};

typedef struct orc_model orc_model;

orc_model* orc_create(const orc_config* cfg);
void orc_destroy(orc_model* m);
/* Effective configuration after defaults (ane/engine.go:188-239). */
void orc_get_config(const orc_model* m, orc_config* out);
/* Pointer into the oracle's own storage; *n receives the element count (0 if absent). */
float* orc_tensor(orc_model* m, int32_t tensor_id, int32_t layer, int32_t which, uint64_t* n);
float* orc_tap(orc_model* m, int32_t tap_id, int32_t layer, uint64_t* n);

/* One reference Step without the sampler: forward, head, backward, gradient
 * accumulation (ane/engine.go:405-414).  Flushes (Adam) after accum_steps calls,
 * like backwardAndAccumulate (ane/train_full.go:815-818).  Returns the loss. */
float orc_step(orc_model* m, const uint16_t* input, const uint16_t* target);
/* Forward + head + backward only; gradients are added to the accumulators and no
 * optimizer update happens until orc_flush. */
float orc_accumulate(orc_model* m, const uint16_t* input, const uint16_t* target);
/* flushPending (ane/engine.go:646-682). */
void orc_flush(orc_model* m);
uint32_t orc_pending(const orc_model* m);
uint32_t orc_adam_t(const orc_model* m);
void orc_set_lr(orc_model* m, float lr);

/* evalLogitsCPUInto (ane/engine.go:954-1038): logits[v*seq + t]. */
void orc_eval_logits(orc_model* m, const uint16_t* tokens, float* logits_vt);
/* Correctly indexed restatement of harness.go:46-89 for one window:
 * sum over t < seq-1 of -log softmax(logits[:,t])[tokens[t+1]] (float64). */
double orc_eval_loss_window(orc_model* m, const uint16_t* tokens, int32_t* n_positions);

/* Forward loss only (no gradients), for finite-difference checks. */
double orc_loss_only(orc_model* m, const uint16_t* input, const uint16_t* target);

/* drand48 sampler of the engine (ane/engine.go:873-880, :395-404). */
uint64_t orc_drand48_seed(int64_t seed);
uint64_t orc_sample_pos(uint64_t* rng_state, uint64_t n_tokens, uint32_t seq);

/* Primitive entry points used by the per-kernel parity tests (all [C][seq]). */
void orc_rmsnorm(float* out, const float* x, const float* w_or_null, int32_t dim, int32_t seq);
void orc_rmsnorm_final(float* out, const float* x, const float* w_or_null, int32_t dim, int32_t seq);
void orc_rmsnorm_bwd(float* dx, float* dw_or_null, const float* dy, const float* x, const float* w_or_null,
                     int32_t dim, int32_t seq);
void orc_linear(float* out, const float* w, const float* in, int32_t out_ch, int32_t in_ch, int32_t seq);
void orc_linear_dx(float* dx, const float* w, const float* dy, int32_t out_ch, int32_t in_ch, int32_t seq);
void orc_linear_dw(float* dw, const float* dy, const float* x, int32_t out_ch, int32_t in_ch, int32_t seq);
void orc_rope(float* x, int32_t heads, int32_t head_dim, int32_t seq, float theta, int32_t inverse);
void orc_qknorm(float* q, float* k, int32_t dim, int32_t heads, int32_t seq);
void orc_attention(float* out, const float* q, const float* k, const float* v, int32_t heads, int32_t kv_heads,
                   int32_t head_dim, int32_t seq);
void orc_attention_bwd(float* dq, float* dk, float* dv, const float* d_out, const float* q, const float* k,
                       const float* v, int32_t heads, int32_t kv_heads, int32_t head_dim, int32_t seq, float scale);
float orc_cross_entropy(float* dlogits, const float* logits, const uint16_t* targets, int32_t vocab, int32_t seq);
void orc_softcap(float* logits, uint64_t n);
void orc_adam(float* w, const float* g, float* m, float* v, uint64_t n, int32_t t, float lr, float b1, float b2,
              float eps, float wd);
int32_t orc_argmax(const float* v, int32_t n);
int32_t orc_sample(const float* logits, int32_t n, float temperature, double u);

/* Threading: 1 = only the loops the reference runs through parallelFor*
 * (norms, CE, classifier GEMMs, Adam) plus dW jobs; 0 (default) = every loop whose
 * arithmetic is independent across iterations. Arithmetic is identical either way. */
void orc_set_reference_threading(int32_t on);
int32_t orc_num_threads(void);
void orc_set_num_threads(int32_t n);

#ifdef __cplusplus
}
#endif
#endif
