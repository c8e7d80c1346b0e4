// Element-wise kernels: dtype casts, RoPE + QK-norm, FFN activations, and the small
// reference-architecture ops (smear, value embeddings, lambda reductions).
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

// 16-byte vectors of T: 8 bf16 or 4 floats.
template <typename T>
struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};

static inline int grid_for(uint64_t n, int block) {
  uint64_t g = (n + block - 1) / block;
  if (g > 148ull * 16) g = 148ull * 16;
  if (g < 1) g = 1;
  return (int)g;
}

// hi = bf16(x), lo = bf16(x - hi): two bf16 tensors that together carry ~16 mantissa bits of x.
__global__ void split_f32_to_bf16x2_kernel(const float* __restrict__ src, bf16* __restrict__ hi, bf16* __restrict__ lo,
                                           uint64_t n4) {
  uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (; i < n4; i += stride) {
    const float4 v = reinterpret_cast<const float4*>(src)[i];
    const float x[4] = {v.x, v.y, v.z, v.w};
    bf16 h[4], l[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      h[k] = __float2bfloat16_rn(x[k]);
      l[k] = __float2bfloat16_rn(x[k] - __bfloat162float(h[k]));
    }
    reinterpret_cast<uint2*>(hi)[i] = *reinterpret_cast<const uint2*>(h);
    reinterpret_cast<uint2*>(lo)[i] = *reinterpret_cast<const uint2*>(l);
  }
}
void split_f32_to_bf16x2(const float* src, bf16* hi, bf16* lo, uint64_t n, cudaStream_t s) {
  if (!n) return;  // n must be a multiple of 4
  split_f32_to_bf16x2_kernel<<<grid_for(n / 4, 256), 256, 0, s>>>(src, hi, lo, n / 4);
}

void cast_f32_to_bf16(const float* src, bf16* dst, uint64_t n, cudaStream_t s) {
  if (!n) return;
  cast_f32_to_bf16_kernel<<<grid_for(n, 256), 256, 0, s>>>(src, dst, n);
}
void cast_bf16_to_f32(const bf16* src, float* dst, uint64_t n, cudaStream_t s) {
  if (!n) return;
  cast_bf16_to_f32_kernel<<<grid_for(n, 256), 256, 0, s>>>(src, dst, n);
}


// ------------------------------------------------------------------------------------------
// RoPE tables (ane/train_util.go:183-202): cos/sin of pos / theta^(2i/hd), computed in double.
// ------------------------------------------------------------------------------------------
__global__ void rope_table_kernel(float* cosb, float* sinb, int seq, int half, int hd, double theta) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= seq * half) return;
  const int pos = idx / half, i = idx - pos * half;
  const double freq = (double)pos / pow(theta, (double)(2 * i) / (double)hd);
  cosb[idx] = (float)cos(freq);
  sinb[idx] = (float)sin(freq);
}
void build_rope_tables(float* cosb, float* sinb, int seq, int hd, double theta, cudaStream_t s) {
  const int half = hd / 2, n = seq * half;
  if (n <= 0) return;
  rope_table_kernel<<<(n + 255) / 256, 256, 0, s>>>(cosb, sinb, seq, half, hd, theta);
}

// ------------------------------------------------------------------------------------------
// RoPE (+ QK-norm) forward / backward: one warp per (token, head) over the q and k heads of a
// packed [M, (H+2KV)*hd] buffer.  Pairs (2i, 2i+1) rotate together (ane/train_util.go:204-224).
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_qknorm_forward_kernel(T* __restrict__ qkv, T* __restrict__ qk_pre,
                                           const float* __restrict__ cosb, const float* __restrict__ sinb, int M,
                                           int seq, int H, int KV, int hd, int qk_norm, int pos0) {
  const int heads = H + KV;
  const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)M * heads) return;
  const int m = (int)(wid / heads), head = (int)(wid - (long long)m * heads);
  const int t = pos0 + m % seq;
  const int half = hd >> 1;
  const int ld = (H + 2 * KV) * hd;
  T* p = qkv + (size_t)m * ld + (size_t)head * hd;  // q heads then k heads are contiguous
  float ss = 0.f;
  float e_[2], o_[2];  // up to hd = 128
  int cnt = 0;
  for (int i = lane; i < half; i += 32, ++cnt) {
    const float c = cosb[t * half + i], s = sinb[t * half + i];
    const float e = to_f<T>(p[2 * i]), o = to_f<T>(p[2 * i + 1]);
    const float e2 = e * c - o * s, o2 = o * c + e * s;
    e_[cnt] = e2;
    o_[cnt] = o2;
    ss += e2 * e2 + o2 * o2;
  }
  if (qk_norm) {
    ss = warp_sum(ss);
    const float scale = 1.2f / sqrtf(ss / (float)hd + 1e-5f);
    T* pre = qk_pre ? qk_pre + (size_t)m * (heads * hd) + (size_t)head * hd : nullptr;
    cnt = 0;
    for (int i = lane; i < half; i += 32, ++cnt) {
      if (pre) {
        pre[2 * i] = from_f<T>(e_[cnt]);
        pre[2 * i + 1] = from_f<T>(o_[cnt]);
      }
      // Normalise the value that was saved (rounded to T), as the reference normalises its saved copy.
      const float e2 = pre ? to_f<T>(pre[2 * i]) : e_[cnt];
      const float o2 = pre ? to_f<T>(pre[2 * i + 1]) : o_[cnt];
      p[2 * i] = from_f<T>(e2 * scale);
      p[2 * i + 1] = from_f<T>(o2 * scale);
    }
  } else {
    cnt = 0;
    for (int i = lane; i < half; i += 32, ++cnt) {
      p[2 * i] = from_f<T>(e_[cnt]);
      p[2 * i + 1] = from_f<T>(o_[cnt]);
    }
  }
}

// Rotation only (no QK-norm): element-wise over the q|k columns, 16 bytes per thread.
template <typename T>
__global__ void rope_only_forward_kernel(T* __restrict__ qkv, const float* __restrict__ cosb,
                                         const float* __restrict__ sinb, int M, int seq, int H, int KV, int hd, int pos0) {
  pdl_trigger();
  pdl_wait();
  constexpr int VN = Vec16<T>::N;
  const int qk_cols = (H + KV) * hd;
  const int vec_per_row = qk_cols / VN;
  const int ld = (H + 2 * KV) * hd;
  const int half = hd >> 1;
  uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t n = (uint64_t)M * vec_per_row, stride = (uint64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    const int m = (int)(i / vec_per_row);
    const int col = (int)(i - (uint64_t)m * vec_per_row) * VN;
    const int t = pos0 + m % seq;
    const int pair0 = (col % hd) >> 1;
    T* p = qkv + (size_t)m * ld + col;
    uint4 u = *reinterpret_cast<const uint4*>(p);
    T* e = reinterpret_cast<T*>(&u);
#pragma unroll
    for (int q = 0; q < VN / 2; ++q) {
      const float c = cosb[t * half + pair0 + q], sn = sinb[t * half + pair0 + q];
      const float a = to_f<T>(e[2 * q]), b = to_f<T>(e[2 * q + 1]);
      e[2 * q] = from_f<T>(a * c - b * sn);
      e[2 * q + 1] = from_f<T>(b * c + a * sn);
    }
    *reinterpret_cast<uint4*>(p) = u;
  }
}

template <typename T>
void rope_qknorm_forward(T* qkv, T* qk_pre, const float* cosb, const float* sinb, int M, int seq, int H, int KV,
                         int hd, bool qk_norm, int pos0, cudaStream_t s) {
  if (!qk_norm) {
    const uint64_t n = (uint64_t)M * (H + KV) * hd / Vec16<T>::N;
    if (!n) return;
    launch_pdl(rope_only_forward_kernel<T>, dim3(grid_for(n, 256)), dim3(256), 0, s, qkv, cosb, sinb, M, seq, H, KV, hd, pos0);
    return;
  }
  const long long warps = (long long)M * (H + KV);
  if (warps <= 0) return;
  const int wpb = 8;
  rope_qknorm_forward_kernel<T><<<(unsigned)((warps + wpb - 1) / wpb), wpb * 32, 0, s>>>(
      qkv, qk_pre, cosb, sinb, M, seq, H, KV, hd, qk_norm, pos0);
}
template void rope_qknorm_forward<float>(float*, float*, const float*, const float*, int, int, int, int, int, bool, int,
                                         cudaStream_t);
template void rope_qknorm_forward<bf16>(bf16*, bf16*, const float*, const float*, int, int, int, int, int, bool, int,
                                        cudaStream_t);

template <typename T, typename TO>
__global__ void rope_qknorm_backward_kernel(T* __restrict__ dqkv, const T* __restrict__ qk_pre,
                                            const float* __restrict__ cosb, const float* __restrict__ sinb, int M,
                                            int seq, int H, int KV, int hd, int qk_norm, int reference_coeff,
                                            int skip_rope, TO* __restrict__ out_t, int write_back) {
  const int heads = H + KV;
  const int slots = out_t ? H + 2 * KV : heads;  // with a typed copy, the v heads are converted too
  const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)M * slots) return;
  const int m = (int)(wid / slots), head = (int)(wid - (long long)m * slots);
  if (head >= heads) {  // v head: conversion only
    const size_t off = (size_t)m * ((H + 2 * KV) * hd) + (size_t)head * hd;
    for (int i = lane; i < hd; i += 32) out_t[off + i] = from_f<TO>(to_f<T>(dqkv[off + i]));
    return;
  }
  const int t = m % seq;
  const int half = hd >> 1;
  const int ld = (H + 2 * KV) * hd;
  T* p = dqkv + (size_t)m * ld + (size_t)head * hd;
  float ge[2], go[2];
  int cnt = 0;
  for (int i = lane; i < half; i += 32, ++cnt) {
    ge[cnt] = to_f<T>(p[2 * i]);
    go[cnt] = to_f<T>(p[2 * i + 1]);
  }
  if (qk_norm) {
    const T* pre = qk_pre + (size_t)m * (heads * hd) + (size_t)head * hd;
    float xe[2], xo[2];
    float ss = 0.f, dot = 0.f;
    cnt = 0;
    for (int i = lane; i < half; i += 32, ++cnt) {
      xe[cnt] = to_f<T>(pre[2 * i]);
      xo[cnt] = to_f<T>(pre[2 * i + 1]);
      ss += xe[cnt] * xe[cnt] + xo[cnt] * xo[cnt];
      dot += ge[cnt] * xe[cnt] + go[cnt] * xo[cnt];
    }
    ss = warp_sum(ss);
    dot = warp_sum(dot);
    const float qs = 1.2f;
    const float r = 1.0f / sqrtf(ss / (float)hd + 1e-5f);
    float coeff = dot * r * r * r / (float)hd * qs;
    if (reference_coeff) coeff *= qs;
    cnt = 0;
    for (int i = lane; i < half; i += 32, ++cnt) {
      ge[cnt] = ge[cnt] * r * qs - coeff * xe[cnt];
      go[cnt] = go[cnt] * r * qs - coeff * xo[cnt];
    }
  }
  cnt = 0;
  for (int i = lane; i < half; i += 32, ++cnt) {
    float e = ge[cnt], o = go[cnt];
    if (!skip_rope) {
      const float c = cosb[t * half + i], s = sinb[t * half + i];
      const float e2 = e * c + o * s, o2 = o * c - e * s;
      e = e2;
      o = o2;
    }
    if (write_back) {
      p[2 * i] = from_f<T>(e);
      p[2 * i + 1] = from_f<T>(o);
    }
    if (out_t) {
      TO* po = out_t + (size_t)m * ld + (size_t)head * hd;
      po[2 * i] = from_f<TO>(e);
      po[2 * i + 1] = from_f<TO>(o);
    }
  }
}

template <typename T, typename TO>
void rope_qknorm_backward(T* dqkv, const T* qk_pre, const float* cosb, const float* sinb, int M, int seq, int H,
                          int KV, int hd, bool qk_norm, bool reference_coeff, bool skip_rope, TO* out_t,
                          bool write_back, cudaStream_t s) {
  const long long warps = (long long)M * (out_t ? H + 2 * KV : H + KV);
  if (warps <= 0) return;
  const int wpb = 8;
  rope_qknorm_backward_kernel<T, TO><<<(unsigned)((warps + wpb - 1) / wpb), wpb * 32, 0, s>>>(
      dqkv, qk_pre, cosb, sinb, M, seq, H, KV, hd, qk_norm, reference_coeff, skip_rope, out_t, write_back ? 1 : 0);
}
template void rope_qknorm_backward<float, float>(float*, const float*, const float*, const float*, int, int, int, int,
                                                 int, bool, bool, bool, float*, bool, cudaStream_t);
template void rope_qknorm_backward<float, bf16>(float*, const float*, const float*, const float*, int, int, int, int,
                                                int, bool, bool, bool, bf16*, bool, cudaStream_t);

// Head size 64, fp32 pre-norm q|k: the same backward with one (even, odd) pair per lane, so a head is one
// 8-byte (fp32) or 4-byte (bf16) access per lane, and four heads per warp whose loads are all issued
// before the first reduction.  The incoming gradient may be bf16 (the tensor-core attention backward
// writes bf16), which removes the conversion pass in front of this kernel; the fp32 result is written
// only when out_f32 is given (it may be the fp32 input itself), the GEMM operand copy when out_t is.
template <typename TI>
__device__ __forceinline__ float2 load_pair(const TI* p);
template <>
__device__ __forceinline__ float2 load_pair<float>(const float* p) { return *reinterpret_cast<const float2*>(p); }
template <>
__device__ __forceinline__ float2 load_pair<bf16>(const bf16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
template <typename TO>
__device__ __forceinline__ void store_pair(TO* p, float e, float o);
template <>
__device__ __forceinline__ void store_pair<float>(float* p, float e, float o) { *reinterpret_cast<float2*>(p) = make_float2(e, o); }
template <>
__device__ __forceinline__ void store_pair<bf16>(bf16* p, float e, float o) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(e, o);
}

// Forward counterpart for fp32 q|k|v with head size 64: rotation and QK-norm of four heads per warp (one pair
// per lane), fp32 results in place, the pre-norm copy for the backward, and in the same pass the bf16 copy of
// all of q|k|v that the tensor-core attention reads (otherwise a separate conversion pass over the tensor).
__global__ void __launch_bounds__(256)
rope_qknorm_forward_hd64_kernel(float* qkv, float* __restrict__ qk_pre, const float* __restrict__ cosb,
                                const float* __restrict__ sinb, int M, int seq, int H, int KV, int qk_norm, int pos0,
                                bf16* __restrict__ hi_out) {
  constexpr int HD = 64, G = 4;
  const int heads = H + KV, slots = H + 2 * KV;
  const int groups = (slots + G - 1) / G;
  const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)M * groups) return;
  const int m = (int)(wid / groups), h0 = (int)(wid - (long long)m * groups) * G;
  const int t = pos0 + m % seq;
  const size_t row = (size_t)m * slots * HD;
  float2 v[G];
#pragma unroll
  for (int q = 0; q < G; ++q) {
    const int head = h0 + q;
    v[q] = head < slots ? *reinterpret_cast<const float2*>(qkv + row + (size_t)head * HD + 2 * lane) : make_float2(0.f, 0.f);
  }
  const float c = cosb[t * (HD / 2) + lane], s = sinb[t * (HD / 2) + lane];
#pragma unroll
  for (int q = 0; q < G; ++q) {
    const int head = h0 + q;
    if (head >= slots) break;
    float e = v[q].x, o = v[q].y;
    const size_t off = row + (size_t)head * HD + 2 * lane;
    if (head < heads) {
      const float e2 = e * c - o * s, o2 = o * c + e * s;
      e = e2;
      o = o2;
      if (qk_norm) {
        const float ss = warp_sum(e * e + o * o);
        const float scale = 1.2f / sqrtf(ss / (float)HD + 1e-5f);
        if (qk_pre) store_pair<float>(qk_pre + (size_t)m * heads * HD + (size_t)head * HD + 2 * lane, e, o);
        e *= scale;
        o *= scale;
      }
      store_pair<float>(qkv + off, e, o);
    }
    if (hi_out) store_pair<bf16>(hi_out + off, e, o);
  }
}

void rope_qknorm_forward_hd64(float* qkv, float* qk_pre, const float* cosb, const float* sinb, int M, int seq, int H, int KV,
                              bool qk_norm, int pos0, bf16* hi_out, cudaStream_t s) {
  const long long warps = (long long)M * ((H + 2 * KV + 3) / 4);
  if (warps <= 0) return;
  const int wpb = 8;
  rope_qknorm_forward_hd64_kernel<<<(unsigned)((warps + wpb - 1) / wpb), wpb * 32, 0, s>>>(qkv, qk_pre, cosb, sinb, M, seq, H,
                                                                                         KV, qk_norm, pos0, hi_out);
}

// Eight values of a row as fp32, from 16 bytes of bf16 or 32 bytes of fp32, and back.
template <typename TI>
__device__ __forceinline__ void load8(const TI* p, float* v);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float* v) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<bf16>(const bf16* p, float* v) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = __bfloat1622float2(h[k]);
    v[2 * k] = f.x;
    v[2 * k + 1] = f.y;
  }
}
template <typename TO>
__device__ __forceinline__ void store8(TO* p, const float* v);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float* v) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8<bf16>(bf16* p, const float* v) {
  uint4 u;
  __nv_bfloat162 t;
  t = __floats2bfloat162_rn(v[0], v[1]); u.x = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(v[2], v[3]); u.y = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(v[4], v[5]); u.z = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(v[6], v[7]); u.w = *reinterpret_cast<uint32_t*>(&t);
  *reinterpret_cast<uint4*>(p) = u;
}

// A warp takes four consecutive heads of one token; eight lanes share a head, each with eight consecutive
// elements (four rotation pairs), so the two per-head sums of the QK-norm backward are three-step
// reductions over eight lanes and every access is 16 or 32 bytes wide.
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
rope_qknorm_backward_hd64_kernel(const TI* din, float* out_f32, const float* __restrict__ qk_pre,
                                 const float* __restrict__ cosb, const float* __restrict__ sinb, int M, int seq, int H,
                                 int KV, int qk_norm, int reference_coeff, int skip_rope, TO* __restrict__ out_t) {
  constexpr int HD = 64, G = 4;
  const int heads = H + KV, slots = H + 2 * KV;
  const int groups = (slots + G - 1) / G;
  const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)M * groups) return;
  const int m = (int)(wid / groups);
  const int head = (int)(wid - (long long)m * groups) * G + (lane >> 3);
  const int part = lane & 7;  // elements [8 * part, 8 * part + 8) of the head
  const int t = m % seq;
  const bool live = head < slots, qk = head < heads;
  const size_t off = (size_t)m * slots * HD + (size_t)head * HD + 8 * part;
  float g[8], x[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) g[k] = x[k] = 0.f;
  if (live) load8<TI>(din + off, g);
  if (qk && qk_norm) load8<float>(qk_pre + (size_t)m * heads * HD + (size_t)head * HD + 8 * part, x);
  if (qk_norm) {  // warp-uniform: lanes of v heads and of missing heads add zeros
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      ss += x[k] * x[k];
      dot += g[k] * x[k];
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
      ss += __shfl_xor_sync(0xffffffffu, ss, o);
      dot += __shfl_xor_sync(0xffffffffu, dot, o);
    }
    if (qk) {
      const float qs = 1.2f;
      const float r = 1.0f / sqrtf(ss / (float)HD + 1e-5f);
      float coeff = dot * r * r * r / (float)HD * qs;
      if (reference_coeff) coeff *= qs;
#pragma unroll
      for (int k = 0; k < 8; ++k) g[k] = g[k] * r * qs - coeff * x[k];
    }
  }
  if (!live) return;
  if (qk && !skip_rope) {
    const float4 c4 = *reinterpret_cast<const float4*>(cosb + t * (HD / 2) + 4 * part);
    const float4 s4 = *reinterpret_cast<const float4*>(sinb + t * (HD / 2) + 4 * part);
    const float c[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const float e = g[2 * p], o = g[2 * p + 1];
      g[2 * p] = e * c[p] + o * sn[p];
      g[2 * p + 1] = o * c[p] - e * sn[p];
    }
  }
  // v heads pass through unchanged: nothing to write when the fp32 output is the input itself
  if (out_f32 && (qk || (const void*)out_f32 != (const void*)din)) store8<float>(out_f32 + off, g);
  if (out_t) store8<TO>(out_t + off, g);
}

template <typename TI, typename TO>
void rope_qknorm_backward_hd64(const TI* din, float* out_f32, const float* qk_pre, const float* cosb, const float* sinb,
                               int M, int seq, int H, int KV, bool qk_norm, bool reference_coeff, bool skip_rope, TO* out_t,
                               cudaStream_t s) {
  const long long warps = (long long)M * ((H + 2 * KV + 3) / 4);
  if (warps <= 0) return;
  const int wpb = 8;
  rope_qknorm_backward_hd64_kernel<TI, TO><<<(unsigned)((warps + wpb - 1) / wpb), wpb * 32, 0, s>>>(
      din, out_f32, qk_pre, cosb, sinb, M, seq, H, KV, qk_norm, reference_coeff, skip_rope, out_t);
}
template void rope_qknorm_backward_hd64<float, float>(const float*, float*, const float*, const float*, const float*, int,
                                                      int, int, int, bool, bool, bool, float*, cudaStream_t);
template void rope_qknorm_backward_hd64<float, bf16>(const float*, float*, const float*, const float*, const float*, int, int,
                                                     int, int, bool, bool, bool, bf16*, cudaStream_t);
template void rope_qknorm_backward_hd64<bf16, bf16>(const bf16*, float*, const float*, const float*, const float*, int, int,
                                                    int, int, bool, bool, bool, bf16*, cudaStream_t);

// ------------------------------------------------------------------------------------------
// FFN activations
// ------------------------------------------------------------------------------------------
// 16 bytes per access (8 bf16 or 4 floats) over the aligned body, element-wise over the tail.
template <typename T>
__global__ void relu2_forward_kernel(const T* __restrict__ h1, T* __restrict__ gate, uint64_t n) {
  constexpr int VN = Vec16<T>::N;
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(h1) | reinterpret_cast<uintptr_t>(gate)) & 15) == 0;
  const uint64_t nv = vec_ok ? n / VN : 0;
  for (uint64_t i = tid; i < nv; i += stride) {
    const uint4 a = reinterpret_cast<const uint4*>(h1)[i];
    const T* x = reinterpret_cast<const T*>(&a);
    uint4 o;
    T* g = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int q = 0; q < VN; ++q) {
      const float h = to_f<T>(x[q]);
      g[q] = from_f<T>(h <= 0.f ? 0.f : h * h);
    }
    reinterpret_cast<uint4*>(gate)[i] = o;
  }
  for (uint64_t i = nv * VN + tid; i < n; i += stride) {
    const float h = to_f<T>(h1[i]);
    gate[i] = from_f<T>(h <= 0.f ? 0.f : h * h);
  }
}
template <typename T>
__global__ void relu2_backward_kernel(const T* __restrict__ dgate, const T* __restrict__ h1, T* __restrict__ dh1,
                                      uint64_t n) {
  constexpr int VN = Vec16<T>::N;
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  const bool vec_ok =
      ((reinterpret_cast<uintptr_t>(h1) | reinterpret_cast<uintptr_t>(dgate) | reinterpret_cast<uintptr_t>(dh1)) & 15) == 0;
  const uint64_t nv = vec_ok ? n / VN : 0;
  for (uint64_t i = tid; i < nv; i += stride) {
    const uint4 a = reinterpret_cast<const uint4*>(h1)[i];
    const uint4 b = reinterpret_cast<const uint4*>(dgate)[i];
    const T* x = reinterpret_cast<const T*>(&a);
    const T* d = reinterpret_cast<const T*>(&b);
    uint4 o;
    T* r = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int q = 0; q < VN; ++q) {
      float h = to_f<T>(x[q]);
      if (h < 0.f) h = 0.f;
      r[q] = from_f<T>(to_f<T>(d[q]) * 2.f * h);
    }
    reinterpret_cast<uint4*>(dh1)[i] = o;
  }
  for (uint64_t i = nv * VN + tid; i < n; i += stride) {
    float h = to_f<T>(h1[i]);
    if (h < 0.f) h = 0.f;
    dh1[i] = from_f<T>(to_f<T>(dgate[i]) * 2.f * h);
  }
}
// SwiGLU on the interleaved FFN layout: h13 [M, 2*Hd] holds, per 64 columns, 32 columns of h1 = x W1^T
// followed by the matching 32 columns of h3 = x W3^T (the rows of W1 and W3 are interleaved the same way
// in the fused W13 matrix), so that one GEMM tile carries both factors of gate = silu(h1) * h3.
__host__ __device__ __forceinline__ uint64_t h1_col(uint64_t j) { return ((j >> 5) << 6) + (j & 31); }

template <typename T>
__global__ void swiglu_forward_kernel(const T* __restrict__ h13, T* __restrict__ gate, int M, int Hd) {
  pdl_trigger();
  pdl_wait();
  constexpr int VN = Vec16<T>::N;
  const int vec_per_row = Hd / VN;
  uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t n = (uint64_t)M * vec_per_row, stride = (uint64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    const uint64_t m = i / vec_per_row, j = (i - m * vec_per_row) * VN;
    const uint4 a = *reinterpret_cast<const uint4*>(h13 + m * 2 * Hd + h1_col(j));
    const uint4 b = *reinterpret_cast<const uint4*>(h13 + m * 2 * Hd + h1_col(j) + 32);
    const T* h1 = reinterpret_cast<const T*>(&a);
    const T* h3 = reinterpret_cast<const T*>(&b);
    uint4 o;
    T* g = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int q = 0; q < VN; ++q) {
      const float x = to_f<T>(h1[q]);
      const float sg = 1.f / (1.f + __expf(-x));
      g[q] = from_f<T>(x * sg * to_f<T>(h3[q]));
    }
    *reinterpret_cast<uint4*>(gate + m * Hd + j) = o;
  }
}
template <typename T>
__global__ void swiglu_backward_kernel(const T* __restrict__ dgate, const T* __restrict__ h13, T* __restrict__ dh13,
                                       int M, int Hd) {
  pdl_trigger();
  pdl_wait();
  constexpr int VN = Vec16<T>::N;
  const int vec_per_row = Hd / VN;
  uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t n = (uint64_t)M * vec_per_row, stride = (uint64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    const uint64_t m = i / vec_per_row, j = (i - m * vec_per_row) * VN;
    const uint4 a = *reinterpret_cast<const uint4*>(h13 + m * 2 * Hd + h1_col(j));
    const uint4 b = *reinterpret_cast<const uint4*>(h13 + m * 2 * Hd + h1_col(j) + 32);
    const uint4 c = *reinterpret_cast<const uint4*>(dgate + m * Hd + j);
    const T* h1 = reinterpret_cast<const T*>(&a);
    const T* h3 = reinterpret_cast<const T*>(&b);
    const T* dgv = reinterpret_cast<const T*>(&c);
    uint4 o1, o3;
    T* d1 = reinterpret_cast<T*>(&o1);
    T* d3 = reinterpret_cast<T*>(&o3);
#pragma unroll
    for (int q = 0; q < VN; ++q) {
      const float x = to_f<T>(h1[q]);
      const float dg = to_f<T>(dgv[q]);
      const float sg = 1.f / (1.f + __expf(-x));
      const float silu = x * sg;
      const float dsilu = sg * (1.f + x * (1.f - sg));
      d1[q] = from_f<T>(dg * to_f<T>(h3[q]) * dsilu);
      d3[q] = from_f<T>(dg * silu);
    }
    *reinterpret_cast<uint4*>(dh13 + m * 2 * Hd + h1_col(j)) = o1;
    *reinterpret_cast<uint4*>(dh13 + m * 2 * Hd + h1_col(j) + 32) = o3;
  }
}

template <typename T>
void relu2_forward(const T* h1, T* gate, uint64_t n, cudaStream_t s) {
  if (!n) return;
  relu2_forward_kernel<T><<<grid_for((n + Vec16<T>::N - 1) / Vec16<T>::N, 256), 256, 0, s>>>(h1, gate, n);
}
template <typename T>
void relu2_backward(const T* dgate, const T* h1, T* dh1, uint64_t n, cudaStream_t s) {
  if (!n) return;
  relu2_backward_kernel<T><<<grid_for((n + Vec16<T>::N - 1) / Vec16<T>::N, 256), 256, 0, s>>>(dgate, h1, dh1, n);
}
template <typename T>
void swiglu_forward(const T* h13, T* gate, int M, int Hd, cudaStream_t s) {
  const uint64_t n = (uint64_t)M * Hd / Vec16<T>::N;
  if (!n) return;
  launch_pdl(swiglu_forward_kernel<T>, dim3(grid_for(n, 256)), dim3(256), 0, s, h13, gate, M, Hd);
}
template <typename T>
void swiglu_backward(const T* dgate, const T* h13, T* dh13, int M, int Hd, cudaStream_t s) {
  const uint64_t n = (uint64_t)M * Hd / Vec16<T>::N;
  if (!n) return;
  launch_pdl(swiglu_backward_kernel<T>, dim3(grid_for(n, 256)), dim3(256), 0, s, dgate, h13, dh13, M, Hd);
}
template void relu2_forward<float>(const float*, float*, uint64_t, cudaStream_t);
template void relu2_forward<bf16>(const bf16*, bf16*, uint64_t, cudaStream_t);
template void relu2_backward<float>(const float*, const float*, float*, uint64_t, cudaStream_t);
template void relu2_backward<bf16>(const bf16*, const bf16*, bf16*, uint64_t, cudaStream_t);
template void swiglu_forward<float>(const float*, float*, int, int, cudaStream_t);
template void swiglu_forward<bf16>(const bf16*, bf16*, int, int, cudaStream_t);
template void swiglu_backward<float>(const float*, const float*, float*, int, int, cudaStream_t);
template void swiglu_backward<bf16>(const bf16*, const bf16*, bf16*, int, int, cudaStream_t);

// ------------------------------------------------------------------------------------------
// Smear (ane/common.go:324-382), element-wise parts.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

__global__ void smear_forward_kernel(const float* __restrict__ x_pre, const float* __restrict__ gate_pre,
                                     const float* __restrict__ lambda, float* __restrict__ x, int M, int seq, int D) {
  uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t n = (uint64_t)M * D, stride = (uint64_t)gridDim.x * blockDim.x;
  const float lam = *lambda;
  for (; i < n; i += stride) {
    const int m = (int)(i / D);
    const int t = m % seq;
    const float shifted = t == 0 ? 0.f : x_pre[i - D];
    x[i] = x_pre[i] + lam * sigmoidf_(gate_pre[i]) * shifted;
  }
}
void smear_forward(const float* x_pre, const float* gate_pre, const float* lambda, float* x, int M, int seq, int D,
                   cudaStream_t s) {
  const uint64_t n = (uint64_t)M * D;
  if (!n) return;
  smear_forward_kernel<<<grid_for(n, 256), 256, 0, s>>>(x_pre, gate_pre, lambda, x, M, seq, D);
}

__global__ void smear_backward_kernel(const float* __restrict__ d_out, const float* __restrict__ x_pre,
                                      const float* __restrict__ gate_pre, const float* __restrict__ lambda,
                                      float* __restrict__ d_gate_pre, float* __restrict__ dx,
                                      float* __restrict__ g_lambda, int M, int seq, int D) {
  uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t n = (uint64_t)M * D, stride = (uint64_t)gridDim.x * blockDim.x;
  const float lam = *lambda;
  double local = 0.0;
  for (; i < n; i += stride) {
    const int m = (int)(i / D);
    const int t = m % seq;
    const float g = sigmoidf_(gate_pre[i]);
    const float sh = t == 0 ? 0.f : x_pre[i - D];
    const float dy = d_out[i];
    local += (double)(dy * g * sh);
    d_gate_pre[i] = dy * lam * sh * g * (1.f - g);
    float v = dy;
    if (t + 1 < seq) v += d_out[i + D] * lam * sigmoidf_(gate_pre[i + D]);
    dx[i] = v;
  }
  local = warp_sum_d(local);
  __shared__ double s_part[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) s_part[warp] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    double tot = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += s_part[w];
    atomicAdd(g_lambda, (float)tot);
  }
}
void smear_backward(const float* d_out, const float* x_pre, const float* gate_pre, const float* lambda,
                    float* d_gate_pre, float* dx, float* g_lambda, int M, int seq, int D, cudaStream_t s) {
  const uint64_t n = (uint64_t)M * D;
  if (!n) return;
  smear_backward_kernel<<<grid_for(n, 256), 256, 0, s>>>(d_out, x_pre, gate_pre, lambda, d_gate_pre, dx, g_lambda, M,
                                                         seq, D);
}

// ------------------------------------------------------------------------------------------
// Small reductions / vector ops
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
dot_accumulate_kernel(const float* __restrict__ a, const float* __restrict__ b, uint64_t n, float alpha,
                      float* __restrict__ out) {
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  double local = 0.0;
  // 16-byte loads, two per operand in flight, when both buffers are aligned; products are rounded to fp32
  // before the double sum, as in the reference's loops (ane/train_full.go:733-782)
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0;
  const uint64_t n4 = vec_ok ? n / 4 : 0;
  const float4* a4 = reinterpret_cast<const float4*>(a);
  const float4* b4 = reinterpret_cast<const float4*>(b);
  uint64_t i = tid;
  for (; i + stride < n4; i += 2 * stride) {
    const float4 x0 = a4[i], y0 = b4[i], x1 = a4[i + stride], y1 = b4[i + stride];
    local += (double)(x0.x * y0.x) + (double)(x0.y * y0.y) + (double)(x0.z * y0.z) + (double)(x0.w * y0.w);
    local += (double)(x1.x * y1.x) + (double)(x1.y * y1.y) + (double)(x1.z * y1.z) + (double)(x1.w * y1.w);
  }
  for (; i < n4; i += stride) {
    const float4 x0 = a4[i], y0 = b4[i];
    local += (double)(x0.x * y0.x) + (double)(x0.y * y0.y) + (double)(x0.z * y0.z) + (double)(x0.w * y0.w);
  }
  for (uint64_t j = n4 * 4 + tid; j < n; j += stride) local += (double)(a[j] * b[j]);
  local = warp_sum_d(local);
  __shared__ double s_part[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) s_part[warp] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    double tot = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += s_part[w];
    atomicAdd(out, alpha * (float)tot);
  }
}
void dot_accumulate(const float* a, const float* b, uint64_t n, float alpha, float* out, cudaStream_t s) {
  if (!n) return;
  int grid = grid_for((n + 3) / 4, 256);
  if (grid > 148 * 8) grid = 148 * 8;
  dot_accumulate_kernel<<<grid, 256, 0, s>>>(a, b, n, alpha, out);
}

// The three passes of one residual's lambda gradients in one (ane/train_full.go:733-782):
//   out_a += sum(d * a),  out_b += sum(d * b)  (products rounded to fp32, summed in double),  y += *alpha * d.
// d is read once instead of three times: 5 instead of 7 tensor passes over HBM, one launch instead of three.
__global__ void __launch_bounds__(256)
lambda_grads_kernel(const float* __restrict__ d, const float* __restrict__ a, const float* __restrict__ b,
                    float* __restrict__ y, const float* __restrict__ alpha, uint64_t n4, float* __restrict__ out_a,
                    float* __restrict__ out_b) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  const float al = *alpha;
  double sa = 0.0, sb = 0.0;
  const float4* d4 = reinterpret_cast<const float4*>(d);
  const float4* a4 = reinterpret_cast<const float4*>(a);
  const float4* b4 = reinterpret_cast<const float4*>(b);
  float4* y4 = reinterpret_cast<float4*>(y);
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 dv = d4[i], av = a4[i], bv = b4[i];
    float4 yv = y4[i];
    sa += (double)(dv.x * av.x) + (double)(dv.y * av.y) + (double)(dv.z * av.z) + (double)(dv.w * av.w);
    sb += (double)(dv.x * bv.x) + (double)(dv.y * bv.y) + (double)(dv.z * bv.z) + (double)(dv.w * bv.w);
    yv.x += al * dv.x; yv.y += al * dv.y; yv.z += al * dv.z; yv.w += al * dv.w;
    y4[i] = yv;
  }
  sa = warp_sum_d(sa);
  sb = warp_sum_d(sb);
  __shared__ double s_a[8], s_b[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    s_a[warp] = sa;
    s_b[warp] = sb;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    double ta = 0, tb = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
      ta += s_a[w];
      tb += s_b[w];
    }
    atomicAdd(out_a, (float)ta);
    atomicAdd(out_b, (float)tb);
  }
}
// n must be a multiple of 4 and the buffers 16-byte aligned (token-major activations are).
void lambda_grads(const float* d, const float* a, const float* b, float* y, const float* alpha, uint64_t n, float* out_a,
                  float* out_b, cudaStream_t s) {
  if (!n) return;
  int grid = grid_for(n / 4, 256);
  if (grid > 148 * 8) grid = 148 * 8;
  lambda_grads_kernel<<<grid, 256, 0, s>>>(d, a, b, y, alpha, n / 4, out_a, out_b);
}

__global__ void axpy_dev_kernel(float* __restrict__ y, const float* __restrict__ x, const float* __restrict__ alpha,
                                float sign, uint64_t n, int assign) {
  uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  const float a = sign * (alpha ? *alpha : 1.f);
  for (; i < n; i += stride) y[i] = assign ? a * x[i] : y[i] + a * x[i];
}
void axpy_dev(float* y, const float* x, const float* alpha, float sign, uint64_t n, bool assign, cudaStream_t s) {
  if (!n) return;
  axpy_dev_kernel<<<grid_for(n, 256), 256, 0, s>>>(y, x, alpha, sign, n, assign ? 1 : 0);
}
void add_inplace(float* y, const float* x, uint64_t n, cudaStream_t s) { axpy_dev(y, x, nullptr, 1.f, n, false, s); }

// ------------------------------------------------------------------------------------------
// Value embeddings (ane/train_full.go:1035-1086): one warp per (token, head).
// ------------------------------------------------------------------------------------------
static constexpr int kVEGateChannels = 12;  // ane/stories/weights.go:28

template <typename T>
__global__ void ve_forward_kernel(T* __restrict__ qkv, const float* __restrict__ x, const uint16_t* __restrict__ tok,
                                  const float* __restrict__ ve_embed, const float* __restrict__ ve_gate,
                                  float* __restrict__ gate_act, int M, int D, int H, int KV, int hd, int vocab) {
  const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)M * H) return;
  const int m = (int)(wid / H), h = (int)(wid - (long long)m * H);
  float gp = 0.f;
  for (int c = 0; c < kVEGateChannels; ++c) gp += ve_gate[h * kVEGateChannels + c] * x[(size_t)m * D + c];
  const float act = 1.0f / (1.0f + expf(-gp));
  if (lane == 0) gate_act[(size_t)m * H + h] = act;
  const float gate = 3.0f * act;
  const int t = tok[m];
  if (t >= vocab) return;
  const int ld = (H + 2 * KV) * hd;
  T* v = qkv + (size_t)m * ld + (size_t)(H + KV) * hd + (size_t)h * hd;
  const float* ve = ve_embed + (size_t)t * D + (size_t)h * hd;
  for (int d = lane; d < hd; d += 32) v[d] = from_f<T>(to_f<T>(v[d]) + gate * ve[d]);
}
template <typename T>
void ve_forward(T* qkv, const float* x, const uint16_t* tok, const float* ve_embed, const float* ve_gate,
                float* gate_act, int M, int D, int H, int KV, int hd, int vocab, cudaStream_t s) {
  const long long warps = (long long)M * H;
  if (warps <= 0) return;
  ve_forward_kernel<T><<<(unsigned)((warps + 7) / 8), 256, 0, s>>>(qkv, x, tok, ve_embed, ve_gate, gate_act, M, D, H,
                                                                    KV, hd, vocab);
}
template void ve_forward<float>(float*, const float*, const uint16_t*, const float*, const float*, float*, int, int,
                                int, int, int, int, cudaStream_t);
template void ve_forward<bf16>(bf16*, const float*, const uint16_t*, const float*, const float*, float*, int, int, int,
                               int, int, int, cudaStream_t);

// Blocks stride over the (token, head) pairs and keep the gate-weight gradient (H x 12 sums that every pair
// adds to) in shared memory, flushed once per block: the global atomics on those few addresses were the
// bulk of this kernel's time.
template <typename T>
__global__ void ve_backward_kernel(const T* __restrict__ dqkv, const float* __restrict__ x,
                                   const uint16_t* __restrict__ tok, const float* __restrict__ ve_embed,
                                   const float* __restrict__ ve_gate, const float* __restrict__ gate_act,
                                   float* __restrict__ g_ve_embed, float* __restrict__ g_ve_gate,
                                   float* __restrict__ d_prev, int M, int D, int H, int KV, int hd, int vocab) {
  extern __shared__ float s_gate[];  // [H][kVEGateChannels]
  for (int i = threadIdx.x; i < H * kVEGateChannels; i += blockDim.x) s_gate[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long total = (long long)M * H;
  const long long step = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); wid < total; wid += step) {
    const int m = (int)(wid / H), h = (int)(wid - (long long)m * H);
    const int t = tok[m];
    if (t >= vocab) continue;
    const float act = gate_act[(size_t)m * H + h];
    const float gate = 3.0f * act;
    const int ld = (H + 2 * KV) * hd;
    const T* dv = dqkv + (size_t)m * ld + (size_t)(H + KV) * hd + (size_t)h * hd;
    const float* ve = ve_embed + (size_t)t * D + (size_t)h * hd;
    float* gve = g_ve_embed + (size_t)t * D + (size_t)h * hd;
    float d_gate = 0.f;
    for (int d = lane; d < hd; d += 32) {
      const float g = to_f<T>(dv[d]);
      atomicAdd(gve + d, g * gate);
      d_gate += g * ve[d];
    }
    d_gate = warp_sum(d_gate);
    const float d_gate_pre = d_gate * 3.0f * act * (1.f - act);
    if (lane < kVEGateChannels) {
      atomicAdd(&s_gate[h * kVEGateChannels + lane], d_gate_pre * x[(size_t)m * D + lane]);
      atomicAdd(d_prev + (size_t)m * D + lane, d_gate_pre * ve_gate[h * kVEGateChannels + lane]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < H * kVEGateChannels; i += blockDim.x)
    if (s_gate[i] != 0.f) atomicAdd(g_ve_gate + i, s_gate[i]);
}
template <typename T>
void ve_backward(const T* dqkv, const float* x, const uint16_t* tok, const float* ve_embed, const float* ve_gate,
                 const float* gate_act, float* g_ve_embed, float* g_ve_gate, float* d_prev, int M, int D, int H,
                 int KV, int hd, int vocab, cudaStream_t s) {
  const long long warps = (long long)M * H;
  if (warps <= 0) return;
  long long blocks = (warps + 7) / 8;
  if (blocks > 148 * 4) blocks = 148 * 4;
  ve_backward_kernel<T><<<(unsigned)blocks, 256, sizeof(float) * H * kVEGateChannels, s>>>(
      dqkv, x, tok, ve_embed, ve_gate, gate_act, g_ve_embed, g_ve_gate, d_prev, M, D, H, KV, hd, vocab);
}
template void ve_backward<float>(const float*, const float*, const uint16_t*, const float*, const float*,
                                 const float*, float*, float*, float*, int, int, int, int, int, int, cudaStream_t);
template void ve_backward<bf16>(const bf16*, const float*, const uint16_t*, const float*, const float*, const float*,
                                float*, float*, float*, int, int, int, int, int, int, cudaStream_t);

// ------------------------------------------------------------------------------------------
// Transpose and argmax
// ------------------------------------------------------------------------------------------
__global__ void transpose_f32_kernel(const float* __restrict__ in, float* __restrict__ out, int rows, int cols) {
  __shared__ float tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int r = r0 + j, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = in[(size_t)r * cols + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int c = c0 + j, r = r0 + threadIdx.x;
    if (r < rows && c < cols) out[(size_t)c * rows + r] = tile[threadIdx.x][j];
  }
}
void transpose_f32(const float* in, float* out, int rows, int cols, cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return;
  dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
  transpose_f32_kernel<<<grid, block, 0, s>>>(in, out, rows, cols);
}

__global__ void argmax_rows_kernel(const float* __restrict__ logits, int32_t* __restrict__ out, int rows, int V) {
  const int row = blockIdx.x;
  if (row >= rows) return;
  const float* p = logits + (size_t)row * V;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = p[i];
    if (v > best || (v == best && i < best_i)) {
      best = v;
      best_i = i;
    }
  }
  __shared__ float s_v[256];
  __shared__ int s_i[256];
  s_v[threadIdx.x] = best;
  s_i[threadIdx.x] = best_i;
  __syncthreads();
  for (int o = blockDim.x >> 1; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) {
      const float v = s_v[threadIdx.x + o];
      const int i = s_i[threadIdx.x + o];
      if (v > s_v[threadIdx.x] || (v == s_v[threadIdx.x] && i < s_i[threadIdx.x])) {
        s_v[threadIdx.x] = v;
        s_i[threadIdx.x] = i;
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) out[row] = s_i[0] == 0x7fffffff ? 0 : s_i[0];
}
void argmax_rows(const float* logits, int32_t* out, int rows, int V, cudaStream_t s) {
  if (rows <= 0) return;
  argmax_rows_kernel<<<rows, 256, 0, s>>>(logits, out, rows, V);
}

// Temperature sampling (ane/train_full.go:318-342): total = sum_i exp((l_i - max) / T) in double, target = u * total,
// result = first i whose running sum reaches target.  One block per row: every thread owns a contiguous chunk and
// sums it in index order, thread 0 scans the 256 chunk sums in order, and the thread whose chunk straddles the
// target walks it again.  The running sum therefore groups the additions by chunk; the index can differ from the
// reference's single serial sum only when target lies within double rounding of a prefix boundary.
__global__ void __launch_bounds__(256)
sample_rows_kernel(const float* __restrict__ logits, const double* __restrict__ u, float temperature,
                   int32_t* __restrict__ out, int rows, int V) {
  const int row = blockIdx.x;
  if (row >= rows) return;
  const float* p = logits + (size_t)row * V;
  __shared__ float s_max[256];
  __shared__ double s_sum[256];
  __shared__ double s_target;
  __shared__ int s_pick;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, p[i]);
  s_max[threadIdx.x] = mx;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) s_max[threadIdx.x] = fmaxf(s_max[threadIdx.x], s_max[threadIdx.x + o]);
    __syncthreads();
  }
  const double maxv = (double)s_max[0];
  const double inv_temp = (double)(1.0f / temperature);
  const int per = (V + 255) / 256;
  const int i0 = min((int)threadIdx.x * per, V), i1 = min(i0 + per, V);
  double part = 0.0;
  for (int i = i0; i < i1; ++i) part += exp(((double)p[i] - maxv) * inv_temp);
  s_sum[threadIdx.x] = part;
  __syncthreads();
  if (threadIdx.x == 0) {
    double acc = 0.0;
    for (int t = 0; t < 256; ++t) {  // s_sum[t] becomes the sum of all chunks before t
      const double v = s_sum[t];
      s_sum[t] = acc;
      acc += v;
    }
    s_target = u[row] * acc;
    s_pick = V - 1;  // the reference's answer when the running sum never reaches target
  }
  __syncthreads();
  const double target = s_target;
  const double before = s_sum[threadIdx.x];
  const double through = before + part;
  // exactly one chunk has before < target <= through, except at target == 0 (the first element wins)
  if (i1 > i0 && through >= target && (before < target || threadIdx.x == 0)) {
    double acc = before;
    int pick = i1 - 1;
    for (int i = i0; i < i1; ++i) {
      acc += exp(((double)p[i] - maxv) * inv_temp);
      if (acc >= target) {
        pick = i;
        break;
      }
    }
    atomicMin(&s_pick, pick);
  }
  __syncthreads();
  if (threadIdx.x == 0) out[row] = s_pick;
}
void sample_rows(const float* logits, const double* u, float temperature, int32_t* out, int rows, int V,
                 cudaStream_t s) {
  if (rows <= 0) return;
  if (temperature <= 1e-6f) argmax_rows_kernel<<<rows, 256, 0, s>>>(logits, out, rows, V);
  else sample_rows_kernel<<<rows, 256, 0, s>>>(logits, u, temperature, out, rows, V);
}

}  // namespace ane
