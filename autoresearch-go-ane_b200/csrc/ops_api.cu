// C-ABI entry points for device buffers and single kernels ("ops").
//
// These are the seams the parity tests and per-kernel roofline measurements call
// through: every argument is a plain pointer or integer, pointers named d_* are
// device pointers obtained from ane_dev_malloc. All ops run on the legacy default
// stream of the current device.
#include <stdio.h>
#include <string.h>

#include <string>

#include "../../include/ane_b200.h"
#include "common.cuh"
#include "gemm.h"
#include "kernels.h"

using namespace ane;

static thread_local std::string g_ops_err;
// One device status word and one timer event pair per device: a kernel launched on device d must be handed
// device-d memory, and events belong to the device that was current when they were made.
static constexpr int kMaxDevices = 64;
static int* g_ops_status_dev[kMaxDevices] = {nullptr};
static cudaEvent_t g_ev0_dev[kMaxDevices] = {nullptr}, g_ev1_dev[kMaxDevices] = {nullptr};

static int set_err(int code, const std::string& msg) {
  g_ops_err = msg;
  return code;
}
static int cuda_fail(cudaError_t e, const char* what) {
  return set_err(ANE_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}
#define CK(call)                                    \
  do {                                              \
    cudaError_t _e = (call);                        \
    if (_e != cudaSuccess) return cuda_fail(_e, #call); \
  } while (0)

static int current_device(int* dev) {
  CK(cudaGetDevice(dev));
  if (*dev < 0 || *dev >= kMaxDevices) return set_err(ANE_ERR_ARG, "device ordinal out of range");
  return 0;
}
// The status word of the current device (allocated on first use there).
static int ensure_status(int** out) {
  int dev = 0;
  if (int rc = current_device(&dev)) return rc;
  if (!g_ops_status_dev[dev]) {
    int* p = nullptr;
    CK(cudaMalloc(&p, sizeof(int)));
    cudaError_t e = cudaMemset(p, 0, sizeof(int));
    if (e != cudaSuccess) {
      cudaFree(p);
      return cuda_fail(e, "cudaMemset");
    }
    g_ops_status_dev[dev] = p;
  }
  *out = g_ops_status_dev[dev];
  return 0;
}

extern "C" {

const char* ane_ops_last_error(void) { return g_ops_err.c_str(); }

int32_t ane_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) return 0;
  return n;
}

int32_t ane_dev_set(int32_t device) {
  CK(cudaSetDevice(device));
  return 0;
}

void* ane_dev_malloc(uint64_t bytes) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes ? bytes : 1);
  if (e != cudaSuccess) {
    cuda_fail(e, "cudaMalloc");
    return nullptr;
  }
  return p;
}
int32_t ane_dev_free(void* d_ptr) {
  CK(cudaFree(d_ptr));
  return 0;
}
void* ane_host_malloc(uint64_t bytes) {
  void* p = nullptr;
  cudaError_t e = cudaMallocHost(&p, bytes ? bytes : 1);
  if (e != cudaSuccess) {
    cuda_fail(e, "cudaMallocHost");
    return nullptr;
  }
  return p;
}
int32_t ane_host_free(void* h_ptr) {
  CK(cudaFreeHost(h_ptr));
  return 0;
}
int32_t ane_dev_h2d(void* d_dst, const void* h_src, uint64_t bytes) {
  CK(cudaMemcpy(d_dst, h_src, bytes, cudaMemcpyHostToDevice));
  return 0;
}
int32_t ane_dev_d2h(void* h_dst, const void* d_src, uint64_t bytes) {
  CK(cudaMemcpy(h_dst, d_src, bytes, cudaMemcpyDeviceToHost));
  return 0;
}
int32_t ane_dev_memset(void* d_ptr, int32_t value, uint64_t bytes) {
  CK(cudaMemset(d_ptr, value, bytes));
  return 0;
}
int32_t ane_dev_sync(void) {
  CK(cudaDeviceSynchronize());
  return 0;
}

// Reads and clears the device status word the op kernels report into
// (0 = ok; 101..103 = a bounded pipeline wait gave up).
int32_t ane_ops_device_status(int32_t* out_status) {
  int* status = nullptr;
  if (ensure_status(&status)) return ANE_ERR_CUDA;
  int v = 0;
  CK(cudaMemcpy(&v, status, sizeof(int), cudaMemcpyDeviceToHost));
  CK(cudaMemset(status, 0, sizeof(int)));
  if (out_status) *out_status = v;
  return 0;
}

// Times `fn`-style regions: begin/end record CUDA events on the default stream.
int32_t ane_timer_begin(void) {
  int dev = 0;
  if (int rc = current_device(&dev)) return rc;
  if (!g_ev0_dev[dev]) {
    CK(cudaEventCreate(&g_ev0_dev[dev]));
    CK(cudaEventCreate(&g_ev1_dev[dev]));
  }
  CK(cudaEventRecord(g_ev0_dev[dev], 0));
  return 0;
}
int32_t ane_timer_end(float* out_ms) {
  int dev = 0;
  if (int rc = current_device(&dev)) return rc;
  if (!g_ev0_dev[dev] || !g_ev1_dev[dev]) return set_err(ANE_ERR_ARG, "ane_timer_end without ane_timer_begin on this device");
  CK(cudaEventRecord(g_ev1_dev[dev], 0));
  CK(cudaEventSynchronize(g_ev1_dev[dev]));
  float ms = 0.f;
  CK(cudaEventElapsedTime(&ms, g_ev0_dev[dev], g_ev1_dev[dev]));
  if (out_ms) *out_ms = ms;
  return 0;
}

int32_t ane_op_cast_f32_to_bf16(const float* d_src, void* d_dst, uint64_t n) {
  cast_f32_to_bf16(d_src, reinterpret_cast<bf16*>(d_dst), n, 0);
  CK(cudaGetLastError());
  return 0;
}
int32_t ane_op_cast_bf16_to_f32(const void* d_src, float* d_dst, uint64_t n) {
  cast_bf16_to_f32(reinterpret_cast<const bf16*>(d_src), d_dst, n, 0);
  CK(cudaGetLastError());
  return 0;
}

// Squared norm of a gradient buffer: *d_out = sum (g*pre_scale)^2 in double
// (ane/train_full.go:167-196 with ane/accel_stub.go:88-95).  The accumulator the kernel reduces
// into is device scratch allocated here for the duration of the call.
int32_t ane_op_sumsq(const float* d_g, uint64_t n, float pre_scale, double* d_out) {
  if (!d_g || !d_out) return set_err(ANE_ERR_ARG, "ane_op_sumsq: null pointer");
  double* acc = nullptr;
  CK(cudaMalloc(&acc, sizeof(double)));
  cudaError_t e = cudaMemsetAsync(acc, 0, sizeof(double), 0);
  if (e == cudaSuccess) {
    sumsq_accumulate(d_g, n, pre_scale, acc, 0);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaMemcpyAsync(d_out, acc, sizeof(double), cudaMemcpyDeviceToDevice, 0);
  if (e == cudaSuccess) e = cudaStreamSynchronize(0);
  const cudaError_t ef = cudaFree(acc);  // the accumulator is released on every path
  if (e != cudaSuccess) return cuda_fail(e, "ane_op_sumsq");
  if (ef != cudaSuccess) return cuda_fail(ef, "cudaFree");
  return 0;
}

int32_t ane_op_sample_rows(const float* d_logits, const double* d_u, float temperature, int32_t* d_out, int32_t rows,
                           int32_t vocab) {
  if (!d_logits || !d_out || (temperature > 1e-6f && !d_u)) return set_err(ANE_ERR_ARG, "ane_op_sample_rows: null pointer");
  if (rows < 0 || vocab <= 0) return set_err(ANE_ERR_ARG, "ane_op_sample_rows: bad dimensions");
  sample_rows(d_logits, d_u, temperature, d_out, rows, vocab, 0);
  CK(cudaGetLastError());
  CK(cudaStreamSynchronize(0));
  return 0;
}

int32_t ane_op_gemm(const ane_gemm_args* a) {
  if (!a || a->struct_size != sizeof(ane_gemm_args)) return set_err(ANE_ERR_ARG, "ane_op_gemm: bad struct_size");
  if (!a->d_a || !a->d_b || !a->d_c) return set_err(ANE_ERR_ARG, "ane_op_gemm: null operand pointer");
  if (a->m < 0 || a->n < 0 || a->k < 0 || a->lda <= 0 || a->ldb <= 0 || a->ldc <= 0)
    return set_err(ANE_ERR_ARG, "ane_op_gemm: bad dimensions");
  if ((a->d_res1 || a->d_res2) && a->ldres <= 0) return set_err(ANE_ERR_ARG, "ane_op_gemm: ldres missing");
  int* status = nullptr;
  if (ensure_status(&status)) return ANE_ERR_CUDA;
  GemmDesc d;
  d.A = a->d_a; d.B = a->d_b; d.C = a->d_c;
  d.M = a->m; d.N = a->n; d.K = a->k;
  d.lda = a->lda; d.ldb = a->ldb; d.ldc = a->ldc;
  d.a_mn = a->a_mn != 0; d.b_mn = a->b_mn != 0;
  d.out = a->out_mode;
  d.alpha = a->alpha;
  d.res1 = a->d_res1; d.s1 = a->d_s1; d.res2 = a->d_res2; d.s2 = a->d_s2;
  d.ldres = a->ldres;
  d.split_k = a->split_k;
  d.aux = const_cast<void*>(a->d_aux);
  d.ldaux = a->ldaux;
  int rc;
  if (a->dtype == ANE_DTYPE_BF16X3) {
    SplitScratch sc;  // operand halves for this call only
    rc = gemm_bf16x3(d, &sc, status, 0);
    cudaStreamSynchronize(0);
    sc.release();
  } else {
    rc = (a->dtype == ANE_DTYPE_F32) ? gemm_f32(d, 0) : gemm_bf16(d, status, 0);
  }
  if (rc != 0) return set_err(ANE_ERR_KERNEL, gemm_last_error());
  return 0;
}

}  // extern "C"
