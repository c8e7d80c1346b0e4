/*
 * libane_b200 -- C ABI of the B200 training-step library.
 *
 * The library stands in for the step math behind the reference's Go `ane`
 * package (ane/engine.go: Open :184, Step :381, EvalLogits :449, Flush :484,
 * State :498, LoadState :506, LR/SetLR :358-378, Close :567).  A Go host binds
 * these symbols with purego (Dlopen + RegisterLibFunc), so every entry point
 * takes only integers and pointers, returns an int32 status (0 = ok, negative =
 * error class) and never keeps a caller pointer after it returns.
 *
 * Pointers named d_* are device pointers (from ane_dev_malloc); all others are
 * host pointers.
 */
#ifndef ANE_B200_H_
#define ANE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ---------------------------------------------------------- */
#define ANE_OK 0
#define ANE_ERR_ARG (-1)     /* bad argument / closed engine              */
#define ANE_ERR_CUDA (-2)    /* a CUDA runtime call failed                 */
#define ANE_ERR_KERNEL (-3)  /* a kernel launch was rejected               */
#define ANE_ERR_DEVICE (-4)  /* a kernel reported a device-side status     */
#define ANE_ERR_NCCL (-5)    /* NCCL setup or collective failed            */
#define ANE_ERR_STATE (-6)   /* call not valid in the current engine state */

#define ANE_DTYPE_BF16 0
#define ANE_DTYPE_F32 1
/* fp32 storage everywhere like ANE_DTYPE_F32, but every GEMM runs on the tensor cores as three bf16
 * products of (hi, lo) operand pairs (Ah*Bh + Ah*Bl + Al*Bh, fp32 accumulation): near-fp32 results at
 * tensor-core speed, for parity with the reference's fp32 CPU step where bf16 operands are too coarse
 * (its backward recomputes the softmax from unscaled scores, ane/train_full.go:268-269). */
#define ANE_DTYPE_BF16X3 2

/* ---- device buffers and timing (test / measurement seams) ------------------- */
int32_t ane_device_count(void);
int32_t ane_dev_set(int32_t device);
void* ane_dev_malloc(uint64_t bytes);
int32_t ane_dev_free(void* d_ptr);
int32_t ane_dev_h2d(void* d_dst, const void* h_src, uint64_t bytes);
int32_t ane_dev_d2h(void* h_dst, const void* d_src, uint64_t bytes);
int32_t ane_dev_memset(void* d_ptr, int32_t value, uint64_t bytes);
/* Page-locked host memory.  ane_eval_logits copies into such a buffer straight from the device; into ordinary
 * (pageable) memory the logits go through the engine's own page-locked staging buffer and a host copy.  The
 * reference has no counterpart: its EvalLogits returns a fresh Go slice (ane/engine.go:954-1038). */
void* ane_host_malloc(uint64_t bytes);
int32_t ane_host_free(void* h_ptr);
int32_t ane_dev_sync(void);
int32_t ane_timer_begin(void);
int32_t ane_timer_end(float* out_ms);
const char* ane_ops_last_error(void);
int32_t ane_ops_device_status(int32_t* out_status);

int32_t ane_op_cast_f32_to_bf16(const float* d_src, void* d_dst, uint64_t n);
int32_t ane_op_cast_bf16_to_f32(const void* d_src, float* d_dst, uint64_t n);
/* sampleFromLogits (ane/train_full.go:318-342) for `rows` rows of `vocab` fp32 logits: d_out[r] = sampled
 * index of row r for the uniform draw d_u[r]; temperature <= 1e-6 gives argmax (ane/train_full.go:344-354).
 * All three pointers are device pointers. */
int32_t ane_op_sample_rows(const float* d_logits, const double* d_u, float temperature, int32_t* d_out, int32_t rows,
                           int32_t vocab);

/* Squared gradient norm, *d_out = sum (g*pre_scale)^2 accumulated in double: the first half of
 * clipLayerGradients (ane/train_full.go:167-196; sumSquaresGrad, ane/accel_stub.go:88-95).
 * d_g and d_out are device pointers.  Allocates a device accumulator for the call. */
int32_t ane_op_sumsq(const float* d_g, uint64_t n, float pre_scale, double* d_out);
/* Same result without allocating anything: the working storage is a fixed 32 KiB array inside the
 * library, so n is limited to 2^28 elements (larger n returns ANE_ERR_ARG).  For hosts that own all
 * device memory themselves or must not trigger an allocation in a latency-critical loop.  No
 * counterpart in the reference.  The first call on a device resolves the array's address (do it
 * before any stream capture); calls share the array, so overlapping calls race.  Unlike ane_op_sumsq,
 * which waits for the device, this call only queues its two kernels on the default stream and returns:
 * *d_out is ready once that stream has caught up (ane_dev_sync, or any later work on the same stream). */
int32_t ane_op_sumsq_noalloc(const float* d_g, uint64_t n, float pre_scale, double* d_out);
const char* ane_op_sumsq_noalloc_last_error(void);

/*
 * Dense contraction C[M,N] (op)= alpha*A*B (+ s1*res1 + s2*res2).
 * Replaces cblas_sgemm at ane/accel_darwin.go:74,94,124-138,163-175,207 and
 * ane/stories/gemm_accel_darwin.go:15,35,55 (pure-Go equivalents:
 * ane/common.go:91, ane/train_full.go:213,242, ane/stories/cpu.go:303-385).
 *   a_mn = 0: A stored [M,K];  a_mn = 1: A stored [K,M]
 *   b_mn = 0: B stored [N,K];  b_mn = 1: B stored [K,N]
 *   out_mode 0: store bf16, 1: store fp32, 2: C += (fp32, beta = 1),
 *            7: SwiGLU backward fused into the product (dX form, bf16 operands): A*B is d gate [m, n]; d_aux = h13
 *               [m, 2n] bf16 with h1 | h3 interleaved in blocks of 32 columns; d_c receives d h13 [m, 2n] bf16 in the
 *               same layout (ldc its pitch): d h1 = d gate * h3 * silu'(h1), d h3 = d gate * silu(h1)
 *               (the reference's FFN is ReLU^2, ane/common.go:146; this is the llama-style counterpart)
 *           10: ReLU^2 backward fused into the product (dX form, bf16 operands, n % 64 == 0): A*B is d gate [m, n];
 *               d_aux = h [m, n] bf16; d_c receives d h = d gate * 2 max(h, 0) in bf16 (ane/common.go:146 differentiated)
 */
typedef struct ane_gemm_args {
  uint32_t struct_size;
  int32_t dtype; /* operands: ANE_DTYPE_BF16 (tcgen05), ANE_DTYPE_F32 (SIMT), ANE_DTYPE_BF16X3 (fp32 in, split tcgen05) */
  const void* d_a;
  const void* d_b;
  void* d_c;
  int32_t m, n, k;
  int32_t lda, ldb, ldc;
  int32_t a_mn, b_mn;
  int32_t out_mode;
  float alpha;
  const float* d_res1;
  const float* d_s1; /* device scalar or NULL (=1) */
  const float* d_res2;
  const float* d_s2;
  int32_t ldres;
  int32_t split_k; /* 0 = library chooses */
  const void* d_aux; /* out_mode 7: h13; out_mode 10: h */
  int32_t ldaux;
  int32_t pad_;
} ane_gemm_args;
int32_t ane_op_gemm(const ane_gemm_args* args);


/* ============================================================================
 * Engine: the drop-in surface behind ane.Engine (ane/engine.go).
 * ========================================================================== */

#define ANE_ARCH_REFERENCE 0 /* the network ane/train_full.go:383-453 trains           */
#define ANE_ARCH_LLAMA 1     /* weighted RMSNorm, SwiGLU (W1/W3/W2), optional GQA        */

/* Mirrors ane.Options (ane/engine.go:14-40); zero / negative values take the defaults
 * of ane.Open (ane/engine.go:188-239).  Model dimensions are runtime fields here (the
 * reference fixes them in ane/stories/config.go:3-18); zero means the reference value. */
typedef struct ane_options {
  uint32_t struct_size;
  int32_t dim, hidden, n_layers, n_heads, n_kv_heads, vocab; /* 768, 2048, 12, 12, =n_heads, 32000 */
  int32_t seq;                                                /* 256 */
  int32_t batch;          /* sequences per ane_step call (reference: 1) */
  int32_t arch;           /* ANE_ARCH_*                                  */
  int32_t quirks;         /* 1: reproduce the reference's backward exactly (ANE_ARCH_REFERENCE only) */
  int32_t compute_dtype;  /* ANE_DTYPE_BF16 (tensor cores), ANE_DTYPE_F32 (SIMT parity mode) or ANE_DTYPE_BF16X3 */
  float rope_theta;       /* 0: 100000 (reference arch) / 10000 (llama arch) */
  int32_t accum_steps;    /* ane_step calls per optimizer update */
  float lr;
  int64_t seed;
  float adam_beta1, adam_beta2, adam_eps, weight_decay, grad_clip, loss_scale;
  float embed_lr_mult, scalar_lr_mult, lambda_lr_mult, lambda_beta1, lambda_beta2;
  int32_t use_ane;         /* accepted and ignored: the GPU path is always on */
  int32_t hybrid_backward; /* accepted and ignored */
  int32_t device;          /* CUDA device ordinal */
  int32_t rank, world_size;/* data-parallel rank / size (world_size <= 1: single GPU) */
  int32_t debug_taps;      /* 1: keep per-layer gradient taps for ane_get_tap */
  int32_t ce_chunk_rows;   /* token rows per logits chunk where logits exist (evaluation; fp32 heads) (0: library chooses) */
  int32_t ce_chunk_cols;   /* vocabulary columns per gradient block of the logit-free training head (0: library chooses) */
  int32_t reserved[5];
} ane_options;

/* Mirrors ane.StepResult (ane/engine.go:55-69); durations in nanoseconds. */
typedef struct ane_step_result {
  uint32_t struct_size;
  float loss;
  int64_t step_ns;
  int64_t compile_ns;          /* always 0: nothing is compiled at run time */
  int64_t startup_compile_ns;  /* always 0 */
  int64_t device_eval_ns;      /* GPU time of the step (the reference's ANEEvalDuration slot) */
  int64_t cpu_work_ns;         /* host time not overlapped with the device */
  int64_t weight_refresh_ns;   /* always 0: the bf16 shadow weights are written by the optimizer kernel */
  int64_t final_head_ns, embed_grad_ns, rms_dw_ns, dw_gemm_ns, dw_wait_ns, adam_ns;
  int32_t flushed;             /* 1 if this call ran the optimizer update */
  int32_t device_status;       /* 0, or the code a kernel's bounded wait reported */
} ane_step_result;

/* Mirrors ane.State (ane/engine.go:43-52). */
typedef struct ane_state {
  uint32_t struct_size;
  uint32_t cum_steps, cum_batches, adam_t, pending_steps;
  uint64_t token_pos;
  float last_loss;
  float pad_;
  double cum_train_ms, cum_wall_ms;
} ane_state;

typedef struct ane_engine ane_engine;

/* 128-byte NCCL bootstrap id: rank 0 calls ane_dp_unique_id and shares the bytes with the
 * other ranks (any out-of-band channel) before every rank calls ane_open with it. */
int32_t ane_dp_unique_id(uint8_t out_id[128]);

/* ane.Open (ane/engine.go:184).  tokens may be NULL/0 for an evaluation-only engine.
 * dp_id is NULL unless opts->world_size > 1.  Weights start at zero (norm weights and
 * residual lambdas at 1); load them with ane_import_tensor. */
int32_t ane_open(const ane_options* opts, const uint16_t* tokens, uint64_t n_tokens, const uint8_t* dp_id,
                 ane_engine** out);
int32_t ane_close(ane_engine* e);              /* ane/engine.go:567 */
const char* ane_last_error(ane_engine* e);     /* message for the last non-zero status (e may be NULL) */
uint32_t ane_version(void);

/* The window sampler Engine.Step uses, exposed for hosts and tests (pure host code, no GPU):
 * ane_sampler_seed = drand48Seed (ane/engine.go:873); ane_sample_windows advances the generator by
 * batch*world draws (ane/engine.go:877-880, :395-404) and returns this rank's `batch` window starts
 * (draws rank, rank+world, ...), so all ranks together consume one reference sample stream. */
uint64_t ane_sampler_seed(int64_t seed);
int32_t ane_sample_windows(uint64_t* rng_state, uint64_t n_tokens, uint32_t seq, uint32_t batch, uint32_t rank,
                           uint32_t world, uint64_t* out_pos);

/* Engine.Step (ane/engine.go:381): samples `batch` windows with the drand48 sampler
 * (ane/engine.go:395-404, :873-880), runs forward, head, backward; every accum_steps calls it
 * applies the optimizer update (ane/engine.go:646-682). */
int32_t ane_step(ane_engine* e, ane_step_result* out);
/* Same step on caller-provided windows: input/target are [n_seq][seq] host arrays, n_seq == batch. */
int32_t ane_step_tokens(ane_engine* e, const uint16_t* input, const uint16_t* target, uint32_t n_seq,
                        ane_step_result* out);
/* Engine.Flush (ane/engine.go:484): apply pending accumulated gradients now. */
int32_t ane_flush(ane_engine* e, double* refresh_ms);
/* Engine.EvalLogits (ane/engine.go:449).  tokens: [n_seq][seq].  layout 0 = the reference's
 * [n_seq][vocab][seq] (logits[v*seq+t]); layout 1 = [n_seq*seq][vocab].  out_cap in floats. */
int32_t ane_eval_logits(ane_engine* e, const uint16_t* tokens, uint32_t n_seq, float* out, uint64_t out_cap,
                        uint32_t layout);
/* Fused evaluation loss (no logits leave the device): per window, sum over t < seq-1 of
 * -log softmax(logits[:,t])[tokens[t+1]], the loop of harness.go:46-89 with correct indexing. */
int32_t ane_eval_loss(ane_engine* e, const uint16_t* tokens, uint32_t n_seq, double* loss_sum, uint64_t* n_positions);
/* Greedy generation with a KV cache (llama-style architecture): prompts [n_seq][prompt_len] ->
 * out [n_seq][n_new]; prompt_len + n_new <= seq, n_seq <= batch.  Token choice is the reference's argmax
 * (ane/train_full.go:344-354: first index of the maximum).  The reference itself has no KV cache. */
int32_t ane_decode_greedy(ane_engine* e, const uint16_t* prompts, uint32_t n_seq, uint32_t prompt_len, uint32_t n_new,
                          uint16_t* out);
/* The same generation loop with the reference's temperature sampler in place of the argmax
 * (sampleFromLogits, ane/train_full.go:318-342: total = sum exp((l - max)/T) in double, first index whose
 * running sum reaches u*total).  The reference draws u from Go's math/rand, which is not reproduced: the
 * caller supplies the draws, uniforms[step*n_seq + b] in [0,1), one per generated token.  temperature
 * <= 1e-6 is the argmax and ignores uniforms. */
int32_t ane_decode_sample(ane_engine* e, const uint16_t* prompts, uint32_t n_seq, uint32_t prompt_len, uint32_t n_new,
                          float temperature, const double* uniforms, uint16_t* out);
int32_t ane_set_lr(ane_engine* e, float lr);   /* ane/engine.go:366 */
float ane_get_lr(ane_engine* e);               /* ane/engine.go:358 */
int32_t ane_get_state(ane_engine* e, ane_state* out);       /* ane/engine.go:498 */
/* LoadState (ane/engine.go:506).  The engine's wall clock continues from in->cum_wall_ms
 * (ane/engine.go:560: start = now - CumWall). */
int32_t ane_set_state(ane_engine* e, const ane_state* in);
/* Restarts the window sampler from drand48Seed(seed) (ane/engine.go:873): what LoadCheckpoint does with
 * seed + meta.Step after a resume (ane/engine.go:559), so that the resumed run does not replay the
 * windows of the run that wrote the file. */
int32_t ane_reseed(ane_engine* e, int64_t seed);

/* Weights / gradients / optimizer moments by tensor id, as row-major fp32 in the reference's
 * shapes (ane/stories/weights.go:13-42), so a host can read and write checkpoints
 * (ane/stories/ckpt.go:77-269).  which: 0 weight, 1 accumulated gradient, 2 Adam m, 3 Adam v. */
enum {
  ANE_T_EMBED = 0, ANE_T_WQ = 1, ANE_T_WK = 2, ANE_T_WV = 3, ANE_T_WO = 4, ANE_T_W1 = 5, ANE_T_W2 = 6, ANE_T_W3 = 7,
  ANE_T_RMS_ATT = 8, ANE_T_RMS_FFN = 9, ANE_T_RMS_FINAL = 10, ANE_T_VE_EMBED = 11, ANE_T_VE_GATE = 12,
  ANE_T_RESID_LAMBDAS = 13, ANE_T_X0_LAMBDAS = 14, ANE_T_SMEAR_GATE = 15, ANE_T_SMEAR_LAMBDA = 16,
  ANE_T_BACKOUT_LAMBDA = 17, ANE_T_COUNT = 18
};
int64_t ane_tensor_size(ane_engine* e, uint32_t tensor_id, uint32_t layer); /* elements; 0 if absent; <0 error */
int32_t ane_import_tensor(ane_engine* e, uint32_t tensor_id, uint32_t layer, uint32_t which, const float* buf,
                          uint64_t n);
/* With world_size > 1 the Adam moments (which 2, 3) of the layer matrices are kept by the rank that owns each
 * slice: exporting them is a collective call (every rank must make it); weights and gradients export locally. */
int32_t ane_export_tensor(ane_engine* e, uint32_t tensor_id, uint32_t layer, uint32_t which, float* buf, uint64_t n);

/* Activation taps of the last step, reference layout [n_seq][channels][seq] (ane/train_full.go:12-37). */
enum {
  ANE_TAP_X = 0, ANE_TAP_XNORM, ANE_TAP_Q, ANE_TAP_K, ANE_TAP_V, ANE_TAP_ATT, ANE_TAP_X2, ANE_TAP_X2NORM,
  ANE_TAP_H1, ANE_TAP_GATE, ANE_TAP_FFN_OUT, ANE_TAP_QPRE, ANE_TAP_KPRE, ANE_TAP_H3,
  ANE_TAP_DOUT, ANE_TAP_DH1, ANE_TAP_DX2, ANE_TAP_DQ, ANE_TAP_DK, ANE_TAP_DV, ANE_TAP_DH3,
  ANE_TAP_X0 = 32, ANE_TAP_XMID, ANE_TAP_FINAL, ANE_TAP_FINAL_NORM
};
int64_t ane_get_tap(ane_engine* e, uint32_t tap_id, uint32_t layer, float* buf, uint64_t cap); /* returns floats written */

/* Measurement seams (no counterpart in the reference, whose StepResult timers are host clocks,
 * ane/metrics.go:13-43): CUDA-event timer on the engine's stream, and per-GEMM device time /
 * algorithmic FLOPs accumulated while profiling is enabled. */
int32_t ane_engine_timer_begin(ane_engine* e);
int32_t ane_engine_timer_end(ane_engine* e, float* out_ms);
int32_t ane_profile_gemm(ane_engine* e, int32_t enable);
int32_t ane_profile_read(ane_engine* e, double* gemm_ms, double* gemm_flops, uint64_t* gemm_launches);

/* Kernel launches issued by this library since the engine was opened (for measurement reports). */
uint64_t ane_launch_count(ane_engine* e);

#ifdef __cplusplus
}
#endif
#endif /* ANE_B200_H_ */
