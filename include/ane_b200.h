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

/* ---- device buffers and timing (test / measurement seams) ------------------- */
int32_t ane_device_count(void);
int32_t ane_dev_set(int32_t device);
void* ane_dev_malloc(uint64_t bytes);
int32_t ane_dev_free(void* d_ptr);
int32_t ane_dev_h2d(void* d_dst, const void* h_src, uint64_t bytes);
int32_t ane_dev_d2h(void* h_dst, const void* d_src, uint64_t bytes);
int32_t ane_dev_memset(void* d_ptr, int32_t value, uint64_t bytes);
int32_t ane_dev_sync(void);
int32_t ane_timer_begin(void);
int32_t ane_timer_end(float* out_ms);
const char* ane_ops_last_error(void);
int32_t ane_ops_device_status(int32_t* out_status);

int32_t ane_op_cast_f32_to_bf16(const float* d_src, void* d_dst, uint64_t n);
int32_t ane_op_cast_bf16_to_f32(const void* d_src, float* d_dst, uint64_t n);

/*
 * Dense contraction C[M,N] (op)= alpha*A*B (+ s1*res1 + s2*res2).
 * Replaces cblas_sgemm at ane/accel_darwin.go:74,94,124-138,163-175,207 and
 * ane/stories/gemm_accel_darwin.go:15,35,55 (pure-Go equivalents:
 * ane/common.go:91, ane/train_full.go:213,242, ane/stories/cpu.go:303-385).
 *   a_mn = 0: A stored [M,K];  a_mn = 1: A stored [K,M]
 *   b_mn = 0: B stored [N,K];  b_mn = 1: B stored [K,N]
 *   out_mode 0: store bf16, 1: store fp32, 2: C += (fp32, beta = 1)
 */
typedef struct ane_gemm_args {
  uint32_t struct_size;
  int32_t dtype; /* ANE_DTYPE_BF16 (tcgen05) or ANE_DTYPE_F32 (SIMT) operands */
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
} ane_gemm_args;
int32_t ane_op_gemm(const ane_gemm_args* args);

#ifdef __cplusplus
}
#endif
#endif /* ANE_B200_H_ */
