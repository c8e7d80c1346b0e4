// Embedding gather/scatter and RMSNorm forward/backward (HBM-bound kernels).
#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace ane {

static constexpr int kWarpsPerBlock = 8;

// ------------------------------------------------------------------------------------------
// Embedding (ane/stories/cpu.go:41-95) with the optional parameterless embed-norm
// (ane/train_full.go:384-388).  One warp per token row.
// ------------------------------------------------------------------------------------------
__global__ void embed_forward_kernel(const uint16_t* __restrict__ tok, const float* __restrict__ embed,
                                     float* __restrict__ x, float* __restrict__ x_raw, int M, int D, int vocab,
                                     int embed_norm) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  const int t = tok[row];
  const bool valid = t < vocab;
  const float* src = embed + (size_t)(valid ? t : 0) * D;
  float* dst = x + (size_t)row * D;
  float ss = 0.f;
  for (int i = lane; i < D; i += 32) {
    float v = valid ? src[i] : 0.f;
    if (x_raw) x_raw[(size_t)row * D + i] = v;
    ss += v * v;
    if (!embed_norm) dst[i] = v;
  }
  if (embed_norm) {
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)D + 1e-5f);
    for (int i = lane; i < D; i += 32) {
      float v = valid ? src[i] : 0.f;
      dst[i] = v * r;
    }
  }
}

void embed_forward(const uint16_t* tok, const float* embed, float* x, float* x_raw, int M, int D, int vocab,
                   bool embed_norm, cudaStream_t s) {
  if (M <= 0) return;
  const int blocks = (M + kWarpsPerBlock - 1) / kWarpsPerBlock;
  launch_pdl(embed_forward_kernel, dim3(blocks), dim3(kWarpsPerBlock * 32), 0, s, tok, embed, x, x_raw, M, D, vocab, embed_norm ? 1 : 0);
}

__global__ void embed_backward_kernel(const uint16_t* __restrict__ tok, const float* __restrict__ dx,
                                      float* __restrict__ g_embed, int M, int D, int vocab) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  const int t = tok[row];
  if (t >= vocab) return;
  float* dst = g_embed + (size_t)t * D;
  const float* src = dx + (size_t)row * D;
  for (int i = lane; i < D; i += 32) atomicAdd(dst + i, src[i]);
}

void embed_backward(const uint16_t* tok, const float* dx, float* g_embed, int M, int D, int vocab, cudaStream_t s) {
  if (M <= 0) return;
  const int blocks = (M + kWarpsPerBlock - 1) / kWarpsPerBlock;
  launch_pdl(embed_backward_kernel, dim3(blocks), dim3(kWarpsPerBlock * 32), 0, s, tok, dx, g_embed, M, D, vocab);
}

// ------------------------------------------------------------------------------------------
// RMSNorm forward: one warp per row, float4 loads, fp32 statistics.
// ------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void store4(T* p, float a, float b, float c, float d);
template <>
__device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <>
__device__ __forceinline__ void store4<bf16>(bf16* p, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&lo);
  u.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}

template <typename T>
__global__ void rmsnorm_forward_kernel(const float* __restrict__ x, const float* __restrict__ w, T* __restrict__ y,
                                       float* __restrict__ rstd, int M, int D) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)row * D);
  const float4* wr = reinterpret_cast<const float4*>(w);
  const int n4 = D >> 2;
  float ss = 0.f;
  for (int i = lane; i < n4; i += 32) {
    float4 v = xr[i];
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = warp_sum(ss);
  const float r = 1.0f / sqrtf(ss / (float)D + 1e-5f);
  if (lane == 0 && rstd) rstd[row] = r;
  T* yr = y + (size_t)row * D;
  for (int i = lane; i < n4; i += 32) {
    float4 v = xr[i];
    float4 ww = w ? wr[i] : make_float4(1.f, 1.f, 1.f, 1.f);
    store4<T>(yr + 4 * i, v.x * r * ww.x, v.y * r * ww.y, v.z * r * ww.z, v.w * r * ww.w);
  }
}

// Register-resident variant for D = 128*NV: a few resident blocks per SM deal the rows round-robin and
// each warp requests its next row before it reduces the current one.
static constexpr int kRmsFwdWarps = 16;
template <typename T, int NV>
__global__ void __launch_bounds__(kRmsFwdWarps * 32)
rmsnorm_forward_reg_kernel(const float* __restrict__ x, const float* __restrict__ w, T* __restrict__ y,
                           float* __restrict__ rstd, int M) {
  pdl_trigger();
  pdl_wait();
  constexpr int D = 128 * NV;
  const int lane = threadIdx.x & 31;
  const int stride = gridDim.x * kRmsFwdWarps;
  int row = blockIdx.x * kRmsFwdWarps + (threadIdx.x >> 5);
  if (row >= M) return;
  float4 wv[NV], nxt[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    wv[k] = w ? reinterpret_cast<const float4*>(w)[lane + 32 * k] : make_float4(1.f, 1.f, 1.f, 1.f);
    nxt[k] = reinterpret_cast<const float4*>(x + (size_t)row * D)[lane + 32 * k];
  }
  for (; row < M; row += stride) {
    float4 v[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) v[k] = nxt[k];
    if (row + stride < M) {
      const float4* xn = reinterpret_cast<const float4*>(x + (size_t)(row + stride) * D);
#pragma unroll
      for (int k = 0; k < NV; ++k) nxt[k] = xn[lane + 32 * k];
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)D + 1e-5f);
    if (lane == 0 && rstd) rstd[row] = r;
    T* yr = y + (size_t)row * D;
#pragma unroll
    for (int k = 0; k < NV; ++k)
      store4<T>(yr + 4 * (lane + 32 * k), v[k].x * r * wv[k].x, v[k].y * r * wv[k].y, v[k].z * r * wv[k].z,
                v[k].w * r * wv[k].w);
  }
}

template <typename T>
void rmsnorm_forward(const float* x, const float* w, T* y, float* rstd, int M, int D, cudaStream_t s) {
  if (M <= 0) return;
  if (D % 128 == 0 && D <= 1024) {
    const int rb = std::min((M + kRmsFwdWarps - 1) / kRmsFwdWarps, 148 * 2);
#define ANE_RMS_FWD_CASE(NV)                                                                                     \
  case NV:                                                                                                        \
    launch_pdl(rmsnorm_forward_reg_kernel<T, NV>, dim3(rb), dim3(kRmsFwdWarps * 32), 0, s, x, w, y, rstd, M);    \
    return;
    switch (D / 128) {
      ANE_RMS_FWD_CASE(1)
      ANE_RMS_FWD_CASE(2)
      ANE_RMS_FWD_CASE(3)
      ANE_RMS_FWD_CASE(4)
      ANE_RMS_FWD_CASE(5)
      ANE_RMS_FWD_CASE(6)
      ANE_RMS_FWD_CASE(7)
      ANE_RMS_FWD_CASE(8)
    }
#undef ANE_RMS_FWD_CASE
  }
  const int blocks = (M + kWarpsPerBlock - 1) / kWarpsPerBlock;
  launch_pdl(rmsnorm_forward_kernel<T>, dim3(blocks), dim3(kWarpsPerBlock * 32), 0, s, x, w, y, rstd, M, D);
}
template void rmsnorm_forward<float>(const float*, const float*, float*, float*, int, int, cudaStream_t);
template void rmsnorm_forward<bf16>(const float*, const float*, bf16*, float*, int, int, cudaStream_t);

// ------------------------------------------------------------------------------------------
// RMSNorm backward (+ residual blend, + optional weight gradient).
//   g = dy*w;  dot = sum(g*x);  dx = g*r - x*dot*r^3/D + res_scale*res
//   dw[i] += sum_rows dy*x*r    (block-local shared accumulation, then global atomics)
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void rmsnorm_backward_kernel(const float* __restrict__ dy, const float* __restrict__ x,
                                        const float* __restrict__ w, const float* __restrict__ rstd,
                                        const float* __restrict__ res, const float* __restrict__ res_scale,
                                        float* __restrict__ dx_f32, T* __restrict__ dx_t, float* __restrict__ dw,
                                        int M, int D) {
  extern __shared__ float s_dw[];  // [D] when dw != nullptr
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  if (dw) {
    for (int i = threadIdx.x; i < D; i += blockDim.x) s_dw[i] = 0.f;
    __syncthreads();
  }
  const float rs = res ? (res_scale ? *res_scale : 1.f) : 0.f;
  const int n4 = D >> 2;
  const float inv_d = 1.0f / (float)D;
  for (int row = blockIdx.x * kWarpsPerBlock + warp; row < M; row += gridDim.x * kWarpsPerBlock) {
    const float4* dyr = reinterpret_cast<const float4*>(dy + (size_t)row * D);
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)row * D);
    const float4* wr = reinterpret_cast<const float4*>(w);
    float r;
    if (rstd) {
      r = rstd[row];
    } else {
      float ss = 0.f;
      for (int i = lane; i < n4; i += 32) {
        float4 v = xr[i];
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
      ss = warp_sum(ss);
      r = 1.0f / sqrtf(ss * inv_d + 1e-5f);
    }
    float dot = 0.f;
    for (int i = lane; i < n4; i += 32) {
      float4 g = dyr[i], v = xr[i];
      if (w) {
        float4 ww = wr[i];
        g.x *= ww.x; g.y *= ww.y; g.z *= ww.z; g.w *= ww.w;
      }
      dot += g.x * v.x + g.y * v.y + g.z * v.z + g.w * v.w;
    }
    dot = warp_sum(dot);
    const float coeff = dot * r * r * r * inv_d;
    const float4* rr = res ? reinterpret_cast<const float4*>(res + (size_t)row * D) : nullptr;
    for (int i = lane; i < n4; i += 32) {
      float4 g = dyr[i], v = xr[i];
      if (dw) {
        atomicAdd(&s_dw[4 * i + 0], g.x * v.x * r);
        atomicAdd(&s_dw[4 * i + 1], g.y * v.y * r);
        atomicAdd(&s_dw[4 * i + 2], g.z * v.z * r);
        atomicAdd(&s_dw[4 * i + 3], g.w * v.w * r);
      }
      if (w) {
        float4 ww = wr[i];
        g.x *= ww.x; g.y *= ww.y; g.z *= ww.z; g.w *= ww.w;
      }
      float4 o;
      o.x = g.x * r - coeff * v.x;
      o.y = g.y * r - coeff * v.y;
      o.z = g.z * r - coeff * v.z;
      o.w = g.w * r - coeff * v.w;
      if (rr) {
        float4 q = rr[i];
        o.x += rs * q.x; o.y += rs * q.y; o.z += rs * q.z; o.w += rs * q.w;
      }
      if (dx_f32) *reinterpret_cast<float4*>(dx_f32 + (size_t)row * D + 4 * i) = o;
      if (dx_t) store4<T>(dx_t + (size_t)row * D + 4 * i, o.x, o.y, o.z, o.w);
    }
  }
  if (dw) {
    __syncthreads();
    for (int i = threadIdx.x; i < D; i += blockDim.x) atomicAdd(dw + i, s_dw[i]);
  }
}

// Register-resident variant for D = 128*NV (NV float4 per lane): each row is read once, and all three
// inputs of a row (dy, x, residual) are requested before anything is computed, so a row costs one memory
// round trip.  One block of twelve warps per SM, rows dealt round-robin.
static constexpr int kRmsBwdWarps = 12;
template <typename T, int NV>
__global__ void __launch_bounds__(kRmsBwdWarps * 32)
rmsnorm_backward_reg_kernel(const float* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ w,
                            const float* __restrict__ rstd, const float* __restrict__ res,
                            const float* __restrict__ res_scale, float* __restrict__ dx_f32, T* __restrict__ dx_t,
                            float* __restrict__ dw, int M) {
  pdl_trigger();
  pdl_wait();
  constexpr int D = 128 * NV;
  __shared__ float s_dw[kRmsBwdWarps][D > 1024 ? 1 : D];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const float rs = res ? (res_scale ? *res_scale : 1.f) : 0.f;
  const float inv_d = 1.0f / (float)D;
  float4 wv[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k)
    wv[k] = w ? reinterpret_cast<const float4*>(w)[lane + 32 * k] : make_float4(1.f, 1.f, 1.f, 1.f);
  float4 dwacc[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k) dwacc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int row = blockIdx.x * kRmsBwdWarps + warp; row < M; row += gridDim.x * kRmsBwdWarps) {
    const float4* dyr = reinterpret_cast<const float4*>(dy + (size_t)row * D);
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)row * D);
    const float4* rr = res ? reinterpret_cast<const float4*>(res + (size_t)row * D) : nullptr;
    float4 g[NV], v[NV], q[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      g[k] = dyr[lane + 32 * k];
      v[k] = xr[lane + 32 * k];
      q[k] = rr ? rr[lane + 32 * k] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float r;
    if (rstd) {
      r = rstd[row];
    } else {
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < NV; ++k) ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
      ss = warp_sum(ss);
      r = 1.0f / sqrtf(ss * inv_d + 1e-5f);
    }
    if (dw) {
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        dwacc[k].x += g[k].x * v[k].x * r;
        dwacc[k].y += g[k].y * v[k].y * r;
        dwacc[k].z += g[k].z * v[k].z * r;
        dwacc[k].w += g[k].w * v[k].w * r;
      }
    }
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      g[k].x *= wv[k].x; g[k].y *= wv[k].y; g[k].z *= wv[k].z; g[k].w *= wv[k].w;
      dot += g[k].x * v[k].x + g[k].y * v[k].y + g[k].z * v[k].z + g[k].w * v[k].w;
    }
    dot = warp_sum(dot);
    const float coeff = dot * r * r * r * inv_d;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      float4 o;
      o.x = g[k].x * r - coeff * v[k].x;
      o.y = g[k].y * r - coeff * v[k].y;
      o.z = g[k].z * r - coeff * v[k].z;
      o.w = g[k].w * r - coeff * v[k].w;
      o.x += rs * q[k].x; o.y += rs * q[k].y; o.z += rs * q[k].z; o.w += rs * q[k].w;
      if (dx_f32) reinterpret_cast<float4*>(dx_f32 + (size_t)row * D)[lane + 32 * k] = o;
      if (dx_t) store4<T>(dx_t + (size_t)row * D + 4 * (lane + 32 * k), o.x, o.y, o.z, o.w);
    }
  }
  if (dw) {
    if constexpr (D <= 1024) {
#pragma unroll
      for (int k = 0; k < NV; ++k) reinterpret_cast<float4*>(&s_dw[warp][0])[lane + 32 * k] = dwacc[k];
      __syncthreads();
      for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float t = 0.f;
#pragma unroll
        for (int wq = 0; wq < kRmsBwdWarps; ++wq) t += s_dw[wq][i];
        atomicAdd(dw + i, t);
      }
    }
  }
}

template <typename T>
void rmsnorm_backward(const float* dy, const float* x, const float* w, const float* rstd, const float* res,
                      const float* res_scale, float* dx_f32, T* dx_t, float* dw, int M, int D, cudaStream_t s) {
  if (M <= 0) return;
  int blocks = (M + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if (D % 128 == 0 && D <= 1024) {
    const int rb = std::min((M + kRmsBwdWarps - 1) / kRmsBwdWarps, 148);
#define ANE_RMS_BWD_CASE(NV)                                                                                      \
  case NV:                                                                                                         \
    launch_pdl(rmsnorm_backward_reg_kernel<T, NV>, dim3(rb), dim3(kRmsBwdWarps * 32), 0, s, dy, x, w, rstd, res,    \
               res_scale, dx_f32, dx_t, dw, M);                                                                    \
    return;
    switch (D / 128) {
      ANE_RMS_BWD_CASE(1)
      ANE_RMS_BWD_CASE(2)
      ANE_RMS_BWD_CASE(3)
      ANE_RMS_BWD_CASE(4)
      ANE_RMS_BWD_CASE(5)
      ANE_RMS_BWD_CASE(6)
      ANE_RMS_BWD_CASE(7)
      ANE_RMS_BWD_CASE(8)
    }
#undef ANE_RMS_BWD_CASE
  }
  if (dw && blocks > 148 * 2) blocks = 148 * 2;  // bound the number of global atomic passes
  const size_t smem = dw ? sizeof(float) * (size_t)D : 0;
  // dx_t may alias dx_f32 only when T == float; callers pass nullptr instead.
  rmsnorm_backward_kernel<T><<<blocks, kWarpsPerBlock * 32, smem, s>>>(dy, x, w, rstd, res, res_scale, dx_f32, dx_t,
                                                                         dw, M, D);
}
template void rmsnorm_backward<float>(const float*, const float*, const float*, const float*, const float*,
                                      const float*, float*, float*, float*, int, int, cudaStream_t);
template void rmsnorm_backward<bf16>(const float*, const float*, const float*, const float*, const float*,
                                     const float*, float*, bf16*, float*, int, int, cudaStream_t);

}  // namespace ane
