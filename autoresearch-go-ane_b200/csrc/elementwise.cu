// Element-wise kernels: dtype casts.
#include "common.cuh"
#include "kernels.h"

namespace ane {

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ src, bf16* __restrict__ dst, uint64_t n) {
  uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) dst[i] = __float2bfloat16_rn(src[i]);
}
__global__ void cast_bf16_to_f32_kernel(const bf16* __restrict__ src, float* __restrict__ dst, uint64_t n) {
  uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) dst[i] = __bfloat162float(src[i]);
}

static inline int grid_for(uint64_t n, int block) {
  uint64_t g = (n + block - 1) / block;
  if (g > 148ull * 16) g = 148ull * 16;
  if (g < 1) g = 1;
  return (int)g;
}

void cast_f32_to_bf16(const float* src, bf16* dst, uint64_t n, cudaStream_t s) {
  if (!n) return;
  cast_f32_to_bf16_kernel<<<grid_for(n, 256), 256, 0, s>>>(src, dst, n);
}
void cast_bf16_to_f32(const bf16* src, float* dst, uint64_t n, cudaStream_t s) {
  if (!n) return;
  cast_bf16_to_f32_kernel<<<grid_for(n, 256), 256, 0, s>>>(src, dst, n);
}

}  // namespace ane
