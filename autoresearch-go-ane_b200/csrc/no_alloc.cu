// Gradient sum-of-squares without any allocation.
//
// Who needs this: a host that has already given all device memory to its own arena, or that sits
// in a latency-critical loop where a cudaMalloc/cudaFree would stall the whole device, cannot let a
// library allocate behind its back.  For such callers this entry point computes the same quantity
// as ane_op_sumsq (the squared gradient norm that clipping starts from) but keeps its working
// storage in a fixed array that is part of the library image: no cudaMalloc, no cudaFree, no
// allocating library routine.  Every GPU that loads the library holds that array (32 KiB) until
// the process exits.
//
// Limits and rules
//   * at most kMaxElems input elements (one partial sum per kChunk elements, kMaxChunks partials);
//     larger inputs are rejected with ANE_ERR_ARG and a message;
//   * the first call on each device looks up the array's device address; make that first call
//     before starting any stream capture;
//   * all calls share the one array and it keeps whatever the previous call left in it.  Each call
//     overwrites exactly the partials it later reads, so nothing needs clearing, but two calls that
//     run on the GPU at the same time race on it: serialise them.
#include <string>

#include "../../include/ane_b200.h"
#include "common.cuh"

namespace {

constexpr unsigned long long kChunk = 1ull << 16;   // elements per partial sum
constexpr int kMaxChunks = 4096;                    // 4096 doubles = 32 KiB of scratch
constexpr unsigned long long kMaxElems = kChunk * kMaxChunks;  // 2^28 elements (1 GiB of fp32)

// Scratch: one partial sum per chunk.  In host code this name is only a handle for
// cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) double g_sumsq_partials[kMaxChunks];

// One block per chunk: partial[c] = sum over the chunk of (g*pre_scale)^2, accumulated in double.
__global__ void __launch_bounds__(256)
sumsq_partials_kernel(const float* __restrict__ g, unsigned long long n, float pre_scale, double* __restrict__ partials) {
  const unsigned long long begin = (unsigned long long)blockIdx.x * kChunk;
  unsigned long long end = begin + kChunk;
  if (end > n) end = n;
  double local = 0.0;
  for (unsigned long long i = begin + threadIdx.x; i < end; i += blockDim.x) {
    const float v = g[i] * pre_scale;
    local += (double)v * (double)v;
  }
  local = ane::warp_sum_d(local);
  __shared__ double s_p[8];
  if ((threadIdx.x & 31) == 0) s_p[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    double tot = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += s_p[w];
    partials[blockIdx.x] = tot;
  }
}

// Single block: out[0] = sum of the first n_chunks partials, in a fixed order.
__global__ void __launch_bounds__(256)
sumsq_final_kernel(const double* __restrict__ partials, int n_chunks, double* __restrict__ out) {
  double local = 0.0;
  for (int i = threadIdx.x; i < n_chunks; i += blockDim.x) local += partials[i];
  local = ane::warp_sum_d(local);
  __shared__ double s_p[8];
  if ((threadIdx.x & 31) == 0) s_p[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    double tot = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += s_p[w];
    out[0] = tot;
  }
}

constexpr int kMaxDevices = 64;
double* g_partials_addr[kMaxDevices] = {nullptr};  // device address of the scratch, per device
thread_local std::string g_noalloc_err;

}  // namespace

extern "C" {

const char* ane_op_sumsq_noalloc_last_error(void) { return g_noalloc_err.c_str(); }

int32_t ane_op_sumsq_noalloc(const float* d_g, uint64_t n, float pre_scale, double* d_out) {
  if (!d_g || !d_out) {
    g_noalloc_err = "ane_op_sumsq_noalloc: null pointer";
    return ANE_ERR_ARG;
  }
  if (n > kMaxElems) {
    g_noalloc_err = "ane_op_sumsq_noalloc: n exceeds the fixed scratch (limit 268435456 elements); "
                    "split the buffer or use ane_op_sumsq";
    return ANE_ERR_ARG;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    g_noalloc_err = std::string("ane_op_sumsq_noalloc: cudaGetDevice: ") + cudaGetErrorString(e);
    return ANE_ERR_CUDA;
  }
  if (!g_partials_addr[dev]) {
    // First call on this device (the device is current): resolve the array's device address.
    double* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_sumsq_partials);
    if (e != cudaSuccess || !p) {
      g_noalloc_err = std::string("ane_op_sumsq_noalloc: cudaGetSymbolAddress: ") + cudaGetErrorString(e);
      return ANE_ERR_CUDA;
    }
    g_partials_addr[dev] = p;
  }
  double* partials = g_partials_addr[dev];
  const int n_chunks = (int)((n + kChunk - 1) / kChunk);
  if (n_chunks > 0) sumsq_partials_kernel<<<n_chunks, 256, 0, 0>>>(d_g, n, pre_scale, partials);
  sumsq_final_kernel<<<1, 256, 0, 0>>>(partials, n_chunks, d_out);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    g_noalloc_err = std::string("ane_op_sumsq_noalloc: launch: ") + cudaGetErrorString(e);
    return ANE_ERR_CUDA;
  }
  return 0;
}

}  // extern "C"
