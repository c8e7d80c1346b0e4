// Host-callable launchers for the non-GEMM kernels of the training step.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ane {

typedef __nv_bfloat16 bf16;

void cast_f32_to_bf16(const float* src, bf16* dst, uint64_t n, cudaStream_t s);
void cast_bf16_to_f32(const bf16* src, float* dst, uint64_t n, cudaStream_t s);

}  // namespace ane
