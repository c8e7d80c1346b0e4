// Cross-entropy over logit rows, gradient-norm reduction and the fused AdamW update.
#include <cstdlib>
#include "common.cuh"
#include "kernels.h"

namespace ane {

// ------------------------------------------------------------------------------------------
// Cross entropy (ane/stories/cpu.go:212-292) with the soft cap (ane/common.go:272-287) folded in.
// One block per token row of fp32 logits [rows, V]; two passes (online max/sum, then gradient).
// The launch asks for enough (unused) dynamic shared memory to hold residency at three blocks per SM:
// the rows in flight (3 x 148 x V x 4 B = 57 MB at V = 32000) then fit the 126 MB L2 and the second
// pass is served from there instead of from HBM.
// ------------------------------------------------------------------------------------------
static constexpr int kCEThreads = 512;
static constexpr int kCEResidencySmem = 64 * 1024;

__device__ __forceinline__ float softcap_f(float x) { return 15.0f * tanhf(x * (1.0f / 15.0f)); }
// tanh through one exp and one fast division (absolute error ~1e-7): for the bf16-logits kernel, whose
// inputs are already rounded to 3 decimal digits.
__device__ __forceinline__ float fast_tanh(float y) { return 1.0f - __fdividef(2.0f, __expf(2.0f * y) + 1.0f); }

template <typename TO>
__global__ void __launch_bounds__(kCEThreads)
cross_entropy_rows_kernel(const float* __restrict__ logits, const uint16_t* __restrict__ targets,
                          const float* __restrict__ inv_valid, TO* __restrict__ dlogits,
                          float* __restrict__ loss_rows, int rows, int row0, int seq, int V, int softcap,
                          float grad_scale) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  if (r >= rows) return;
  const int grow = row0 + r;  // global token row
  const float* x = logits + (size_t)r * V;
  TO* dl = dlogits ? dlogits + (size_t)r * V : nullptr;
  const int tgt = targets[grow];
  __shared__ float s_m[kCEThreads / 32], s_l[kCEThreads / 32];
  __shared__ float s_bm, s_bl;
  if (tgt >= V) {  // invalid target: zero gradient row, not counted (cpu.go:253-258)
    if (dl)
      for (int i = threadIdx.x; i < V; i += kCEThreads) dl[i] = from_f<TO>(0.f);
    if (threadIdx.x == 0 && loss_rows) loss_rows[grow] = 0.f;
    return;
  }
  float m = -INFINITY, l = 0.f;
  const int V4 = V >> 2;  // V is a multiple of 4 (checked when the engine opens)
  const float4* x4 = reinterpret_cast<const float4*>(x);
#pragma unroll 2
  for (int i = threadIdx.x; i < V4; i += kCEThreads) {
    const float4 q = x4[i];
    float z[4] = {q.x, q.y, q.z, q.w};
    if (softcap) {
#pragma unroll
      for (int k = 0; k < 4; ++k) z[k] = softcap_f(z[k]);
    }
    const float zm = fmaxf(fmaxf(z[0], z[1]), fmaxf(z[2], z[3]));
    if (zm > m) {
      l *= __expf(m - zm);
      m = zm;
    }
    l += __expf(z[0] - m) + __expf(z[1] - m) + __expf(z[2] - m) + __expf(z[3] - m);
  }
  // warp then block combine of (m, l)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), l2 = __shfl_xor_sync(0xffffffffu, l, o);
    const float mn = fmaxf(m, m2);
    l = (m == -INFINITY ? 0.f : l * __expf(m - mn)) + (m2 == -INFINITY ? 0.f : l2 * __expf(m2 - mn));
    m = mn;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    s_m[warp] = m;
    s_l[warp] = l;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float bm = s_m[0], bl = s_l[0];
    for (int w = 1; w < kCEThreads / 32; ++w) {
      const float mn = fmaxf(bm, s_m[w]);
      bl = (bm == -INFINITY ? 0.f : bl * __expf(bm - mn)) + (s_m[w] == -INFINITY ? 0.f : s_l[w] * __expf(s_m[w] - mn));
      bm = mn;
    }
    s_bm = bm;
    s_bl = bl;
  }
  __syncthreads();
  const float bm = s_bm;
  const float inv_sum = 1.0f / s_bl;
  const float gs = grad_scale * inv_valid[grow / seq];
  for (int i = threadIdx.x; i < V4; i += kCEThreads) {
    const float4 q = x4[i];
    const float raw[4] = {q.x, q.y, q.z, q.w};
    float outv[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float z = raw[k], dcap = 1.f;
      if (softcap) {
        const float th = tanhf(raw[k] * (1.0f / 15.0f));
        z = 15.0f * th;
        dcap = 1.f - th * th;
      }
      const float p = __expf(z - bm) * inv_sum;
      const int idx = 4 * i + k;
      if (idx == tgt && loss_rows) loss_rows[grow] = -logf(fmaxf(expf(z - bm) * inv_sum, 1e-10f));
      outv[k] = gs * (p - (idx == tgt ? 1.f : 0.f)) * dcap;
    }
    if (dl) {
      if constexpr (sizeof(TO) == 4) {
        *reinterpret_cast<float4*>(dl + 4 * i) = make_float4(outv[0], outv[1], outv[2], outv[3]);
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(outv[0], outv[1]), hi = __floats2bfloat162_rn(outv[2], outv[3]);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&lo);
        u.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(dl + 4 * i) = u;
      }
    }
  }
}

// Same loss and gradient from bf16 logits (16-byte loads of 8), with the target logit supplied in fp32
// (tgt_logit[row], written by the classifier GEMM epilogue): the log-sum-exp of rounded logits errs by a
// probability-weighted mean of zero-mean rounding errors, while the target term, which would carry its
// rounding error into the loss one to one, stays exact.
__global__ void __launch_bounds__(kCEThreads)
cross_entropy_rows_bf16_kernel(const bf16* __restrict__ logits, const uint16_t* __restrict__ targets,
                               const float* __restrict__ inv_valid, const float* __restrict__ tgt_logit,
                               bf16* __restrict__ dlogits, float* __restrict__ loss_rows, int rows, int row0, int seq,
                               int V, int softcap, float grad_scale) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  if (r >= rows) return;
  const int grow = row0 + r;
  const uint4* x8 = reinterpret_cast<const uint4*>(logits + (size_t)r * V);
  uint4* d8 = dlogits ? reinterpret_cast<uint4*>(dlogits + (size_t)r * V) : nullptr;
  const int tgt = targets[grow];
  const int V8 = V >> 3;  // V is a multiple of 8 (checked when the engine opens)
  __shared__ float s_m[kCEThreads / 32], s_l[kCEThreads / 32];
  __shared__ float s_bm, s_bl;
  if (tgt >= V) {  // invalid target: zero gradient row, not counted (cpu.go:253-258)
    if (d8)
      for (int i = threadIdx.x; i < V8; i += kCEThreads) d8[i] = make_uint4(0u, 0u, 0u, 0u);
    if (threadIdx.x == 0 && loss_rows) loss_rows[grow] = 0.f;
    return;
  }
  float m = -INFINITY, l = 0.f;
#pragma unroll 2
  for (int i = threadIdx.x; i < V8; i += kCEThreads) {
    const uint4 q = x8[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
    float z[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      z[2 * k] = softcap ? 15.0f * fast_tanh(f.x * (1.0f / 15.0f)) : f.x;
      z[2 * k + 1] = softcap ? 15.0f * fast_tanh(f.y * (1.0f / 15.0f)) : f.y;
    }
    float zm = z[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) zm = fmaxf(zm, z[k]);
    if (zm > m) {
      l *= __expf(m - zm);
      m = zm;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) l += __expf(z[k] - m);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), l2 = __shfl_xor_sync(0xffffffffu, l, o);
    const float mn = fmaxf(m, m2);
    l = (m == -INFINITY ? 0.f : l * __expf(m - mn)) + (m2 == -INFINITY ? 0.f : l2 * __expf(m2 - mn));
    m = mn;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    s_m[warp] = m;
    s_l[warp] = l;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float bm = s_m[0], bl = s_l[0];
    for (int w = 1; w < kCEThreads / 32; ++w) {
      const float mn = fmaxf(bm, s_m[w]);
      bl = (bm == -INFINITY ? 0.f : bl * __expf(bm - mn)) + (s_m[w] == -INFINITY ? 0.f : s_l[w] * __expf(s_m[w] - mn));
      bm = mn;
    }
    s_bm = bm;
    s_bl = bl;
    if (loss_rows) {
      float zt = tgt_logit[grow];
      if (softcap) zt = softcap_f(zt);
      loss_rows[grow] = -logf(fmaxf(expf(zt - bm) / bl, 1e-10f));
    }
  }
  __syncthreads();
  if (!d8) return;
  const float bm = s_bm;
  const float inv_sum = 1.0f / s_bl;
  const float gs = grad_scale * inv_valid[grow / seq];
  for (int i = threadIdx.x; i < V8; i += kCEThreads) {
    const uint4 q = x8[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
    float outv[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float2 f = __bfloat1622float2(h[k >> 1]);
      const float raw = (k & 1) ? f.y : f.x;
      float z = raw, dcap = 1.f;
      if (softcap) {
        const float th = fast_tanh(raw * (1.0f / 15.0f));
        z = 15.0f * th;
        dcap = 1.f - th * th;
      }
      const float p = __expf(z - bm) * inv_sum;
      outv[k] = gs * (p - ((8 * i + k) == tgt ? 1.f : 0.f)) * dcap;
    }
    uint4 u;
    __nv_bfloat162 t;
    t = __floats2bfloat162_rn(outv[0], outv[1]); u.x = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(outv[2], outv[3]); u.y = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(outv[4], outv[5]); u.z = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(outv[6], outv[7]); u.w = *reinterpret_cast<uint32_t*>(&t);
    d8[i] = u;
  }
}

// Register-resident form for rows of up to threads x slots x 8 = 32768 logits: the block reads its
// row once, 16 bytes per load with every load of a thread in flight together, and keeps it packed in
// registers (two blocks per SM hold two 64 KB rows: 512 threads x 8 pieces or 256 threads x 16 pieces).  Three sweeps over the registers:
// packed bf16 maxima, sum of exponentials, gradient.  Per logit that is about ten instructions and two
// MUFU operations, against ~29 issued instructions of the streaming kernel above, which is bound by
// instruction issue and not by memory.  The target's one-hot term is patched into the single 16-byte
// piece that holds it, outside the per-element work.

__device__ __forceinline__ float ex2_fast(float x) {  // one MUFU.EX2, denormal results flushed to zero
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));  // volatile: keeps the sweeps in source order (register pressure)
  return y;
}
__device__ __forceinline__ float bf16_lo_f(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi_f(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&t);
}
__device__ __forceinline__ uint32_t bf16x2_max(uint32_t a, uint32_t b) {
  const __nv_bfloat162 r = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}

template <bool SOFTCAP, int kCERegThreads, int kCERegSlots>
__global__ void __launch_bounds__(kCERegThreads, 2)
cross_entropy_rows_bf16_reg_kernel(const bf16* __restrict__ logits, const uint16_t* __restrict__ targets,
                                   const float* __restrict__ inv_valid, const float* __restrict__ tgt_logit,
                                   bf16* __restrict__ dlogits, float* __restrict__ loss_rows, int rows, int row0,
                                   int seq, int V, float grad_scale) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  if (r >= rows) return;
  const int grow = row0 + r;
  const uint4* x8 = reinterpret_cast<const uint4*>(logits + (size_t)r * V);
  uint4* d8 = dlogits ? reinterpret_cast<uint4*>(dlogits + (size_t)r * V) : nullptr;
  const int tgt = targets[grow];
  const int V8 = V >> 3;
  const int tid = threadIdx.x;
  __shared__ float s_m[kCERegThreads / 32], s_l[kCERegThreads / 32];
  if (tgt >= V) {  // invalid target: zero gradient row, not counted (cpu.go:253-258)
    if (d8)
      for (int i = tid; i < V8; i += kCERegThreads) d8[i] = make_uint4(0u, 0u, 0u, 0u);
    if (tid == 0 && loss_rows) loss_rows[grow] = 0.f;
    return;
  }
  constexpr uint32_t kNegInf2 = 0xff80ff80u;  // two bf16 -inf: contributes nothing to maximum or sum
  uint4 q[kCERegSlots];
#pragma unroll
  for (int j = 0; j < kCERegSlots; ++j) {
    const int i = tid + j * kCERegThreads;
    q[j] = i < V8 ? x8[i] : make_uint4(kNegInf2, kNegInf2, kNegInf2, kNegInf2);
  }
  // sweep 1: row maximum of the raw logits (the soft cap is monotonic, so it is applied to the maximum)
  uint32_t mx = kNegInf2;
#pragma unroll
  for (int j = 0; j < kCERegSlots; ++j)
    mx = bf16x2_max(mx, bf16x2_max(bf16x2_max(q[j].x, q[j].y), bf16x2_max(q[j].z, q[j].w)));
  float m = fmaxf(bf16_lo_f(mx), bf16_hi_f(mx));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  const int lane = tid & 31, warp = tid >> 5;
  if (lane == 0) s_m[warp] = m;
  __syncthreads();
  m = s_m[lane & (kCERegThreads / 32 - 1)];
#pragma unroll
  for (int o = kCERegThreads / 64; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  const float bm = SOFTCAP ? 15.0f * fast_tanh(m * (1.0f / 15.0f)) : m;
  constexpr float kLog2e = 1.4426950408889634f;
  const float mb = bm * kLog2e;
  // sweep 2: sum of exp(z - max)
  float l = 0.f;
#pragma unroll
  for (int j = 0; j < kCERegSlots; ++j) {
    const uint32_t w[4] = {q[j].x, q[j].y, q[j].z, q[j].w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float a = bf16_lo_f(w[k]), b = bf16_hi_f(w[k]);
      if (SOFTCAP) {
        a = 15.0f * fast_tanh(a * (1.0f / 15.0f));
        b = 15.0f * fast_tanh(b * (1.0f / 15.0f));
      }
      l += ex2_fast(fmaf(a, kLog2e, -mb)) + ex2_fast(fmaf(b, kLog2e, -mb));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
  if (lane == 0) s_l[warp] = l;
  __syncthreads();
  l = s_l[lane & (kCERegThreads / 32 - 1)];
#pragma unroll
  for (int o = kCERegThreads / 64; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
  if (tid == 0 && loss_rows) {
    float zt = tgt_logit[grow];
    if (SOFTCAP) zt = softcap_f(zt);
    loss_rows[grow] = -logf(fmaxf(expf(zt - bm) / l, 1e-10f));
  }
  if (!d8) return;
  // sweep 3: gradient gs * (softmax - onehot) [* d softcap], written in the logits' own format
  const float gs = grad_scale * inv_valid[grow / seq];
  const float sc = gs / l;
#pragma unroll
  for (int j = 0; j < kCERegSlots; ++j) {
    const int i = tid + j * kCERegThreads;
    const uint32_t w[4] = {q[j].x, q[j].y, q[j].z, q[j].w};
    float o[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float a = bf16_lo_f(w[k]), b = bf16_hi_f(w[k]);
      if (SOFTCAP) {
        const float ta = fast_tanh(a * (1.0f / 15.0f)), tb = fast_tanh(b * (1.0f / 15.0f));
        o[2 * k] = ex2_fast(fmaf(15.0f * ta, kLog2e, -mb)) * sc * (1.f - ta * ta);
        o[2 * k + 1] = ex2_fast(fmaf(15.0f * tb, kLog2e, -mb)) * sc * (1.f - tb * tb);
      } else {
        o[2 * k] = ex2_fast(fmaf(a, kLog2e, -mb)) * sc;
        o[2 * k + 1] = ex2_fast(fmaf(b, kLog2e, -mb)) * sc;
      }
    }
    if (i < V8)
      d8[i] = make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]), pack_bf16x2(o[4], o[5]), pack_bf16x2(o[6], o[7]));
  }
  // The target's one-hot term: the thread that stored the piece holding the target rewrites that one
  // element afterwards (same thread, same address: program order), which keeps the sweep free of it.
  if (tid == ((tgt >> 3) & (kCERegThreads - 1))) {
    float z = __bfloat162float(logits[(size_t)r * V + tgt]), dcap = 1.f;
    if (SOFTCAP) {
      const float th = fast_tanh(z * (1.0f / 15.0f));
      z = 15.0f * th;
      dcap = 1.f - th * th;
    }
    dlogits[(size_t)r * V + tgt] = __float2bfloat16_rn((ex2_fast(fmaf(z, kLog2e, -mb)) * sc - gs) * dcap);
  }
}

// Set ANE_B200_CE_STREAMING=1 to keep every row on the streaming kernel (for comparisons).
static bool ce_force_streaming() {
  static const bool v = [] {
    const char* e = getenv("ANE_B200_CE_STREAMING");
    return e && e[0] == '1';
  }();
  return v;
}

// ANE_B200_CE_REG_THREADS=256 selects 256 threads x 16 pieces for the register-resident kernel (default 512 x 8).
static int ce_reg_threads() {
  static const int v = [] {
    const char* e = getenv("ANE_B200_CE_REG_THREADS");
    return (e && atoi(e) == 256) ? 256 : 512;
  }();
  return v;
}

void cross_entropy_rows_bf16(const bf16* logits, const uint16_t* targets, const float* inv_valid, const float* tgt_logit,
                             bf16* dlogits, float* loss_rows, int rows, int row0, int seq, int V, bool softcap,
                             float grad_scale, cudaStream_t s) {
  if (rows <= 0) return;
  if ((V >> 3) <= 4096 && !ce_force_streaming()) {
    auto go = [&](auto kernel, int threads) {
      launch_pdl(kernel, dim3(rows), dim3(threads), 0, s, logits, targets, inv_valid, tgt_logit, dlogits, loss_rows, rows,
                 row0, seq, V, grad_scale);
    };
    if (ce_reg_threads() == 256) {
      if (softcap) go(cross_entropy_rows_bf16_reg_kernel<true, 256, 16>, 256);
      else go(cross_entropy_rows_bf16_reg_kernel<false, 256, 16>, 256);
    } else {
      if (softcap) go(cross_entropy_rows_bf16_reg_kernel<true, 512, 8>, 512);
      else go(cross_entropy_rows_bf16_reg_kernel<false, 512, 8>, 512);
    }
    return;
  }
  static bool attr_done = false;
  if (!attr_done) {
    if (cudaFuncSetAttribute(cross_entropy_rows_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kCEResidencySmem) != cudaSuccess)
      return;
    attr_done = true;
  }
  launch_pdl(cross_entropy_rows_bf16_kernel, dim3(rows), dim3(kCEThreads), kCEResidencySmem, s, logits, targets, inv_valid,
             tgt_logit, dlogits, loss_rows, rows, row0, seq, V, softcap ? 1 : 0, grad_scale);
}

template <typename TO>
void cross_entropy_rows(const float* logits, const uint16_t* targets, const float* inv_valid, TO* dlogits,
                        float* loss_rows, int rows, int row0, int seq, int V, bool softcap, float grad_scale,
                        cudaStream_t s) {
  if (rows <= 0) return;
  static bool attr_done = false;  // per instantiation (TO)
  if (!attr_done) {
    if (cudaFuncSetAttribute(cross_entropy_rows_kernel<TO>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kCEResidencySmem) != cudaSuccess)
      return;
    attr_done = true;
  }
  launch_pdl(cross_entropy_rows_kernel<TO>, dim3(rows), dim3(kCEThreads), kCEResidencySmem, s, logits, targets, inv_valid, dlogits, loss_rows,
             rows, row0, seq, V, softcap ? 1 : 0, grad_scale);
}
template void cross_entropy_rows<float>(const float*, const uint16_t*, const float*, float*, float*, int, int, int,
                                        int, bool, float, cudaStream_t);
template void cross_entropy_rows<bf16>(const float*, const uint16_t*, const float*, bf16*, float*, int, int, int, int,
                                       bool, float, cudaStream_t);

// Classifier head without logits in memory, between its two passes: the per-tile (maximum, sum) pairs of a row
// (log2 domain) combine to the row's log2-sum-exp; the loss of the row follows from its target logit
// (ane/stories/cpu.go:212-292: -log(max(p[target], 1e-10)); rows whose target lies outside the vocabulary
// count nothing and get a zero gradient row), and coef = grad_scale * inv_valid[sequence] is what pass 2
// multiplies (softmax - onehot) by.  One thread per row; stats is [n_tiles][rows].
__global__ void ce_merge_stats_kernel(const float2* __restrict__ stats, int n_tiles, int rows, const float* __restrict__ tgt_logit,
                                      const uint16_t* __restrict__ targets, const float* __restrict__ inv_valid, int seq, int V,
                                      int softcap, float grad_scale, float* __restrict__ lse2, float* __restrict__ coef,
                                      float* __restrict__ loss_rows) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float m = -INFINITY, s = 0.f;
  for (int t = 0; t < n_tiles; ++t) {
    const float2 v = stats[(size_t)t * rows + r];
    const float mn = fmaxf(m, v.x);
    s = s * exp2f(m - mn) + v.y * exp2f(v.x - mn);
    m = mn;
  }
  const float l2 = m + log2f(s);
  lse2[r] = l2;
  const int tgt = targets[r];
  if (tgt >= V) {
    coef[r] = 0.f;
    if (loss_rows) loss_rows[r] = 0.f;
    return;
  }
  coef[r] = inv_valid ? grad_scale * inv_valid[r / seq] : 0.f;
  if (loss_rows) {
    float zt = tgt_logit[r];
    if (softcap) zt = softcap_f(zt);
    loss_rows[r] = -logf(fmaxf(exp2f(zt * 1.4426950408889634f - l2), 1e-10f));
  }
}
void ce_merge_stats(const float* stats, int n_tiles, int rows, const float* tgt_logit, const uint16_t* targets,
                    const float* inv_valid, int seq, int V, bool softcap, float grad_scale, float* lse2, float* coef,
                    float* loss_rows, cudaStream_t s) {
  if (rows <= 0) return;
  launch_pdl(ce_merge_stats_kernel, dim3((rows + 127) / 128), dim3(128), 0, s, reinterpret_cast<const float2*>(stats), n_tiles,
             rows, tgt_logit, targets, inv_valid, seq, V, softcap ? 1 : 0, grad_scale, lse2, coef, loss_rows);
}

__global__ void softcap_inplace_kernel(float* __restrict__ logits, uint64_t n) {
  uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) logits[i] = softcap_f(logits[i]);
}
void softcap_inplace(float* logits, uint64_t n, cudaStream_t s) {
  if (!n) return;
  uint64_t g = (n + 255) / 256;
  if (g > 148ull * 16) g = 148ull * 16;
  softcap_inplace_kernel<<<(unsigned)g, 256, 0, s>>>(logits, n);
}

__global__ void count_valid_targets_kernel(const uint16_t* __restrict__ targets, float* __restrict__ inv_valid, int B,
                                           int seq, int V) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x;
  if (b >= B) return;
  int c = 0;
  for (int t = threadIdx.x; t < seq; t += blockDim.x) c += targets[(size_t)b * seq + t] < V ? 1 : 0;
  __shared__ int s_c[32];
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) s_c[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int tot = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += s_c[w];
    inv_valid[b] = tot > 0 ? (float)(1.0 / (double)tot) : 0.f;
  }
}
void count_valid_targets(const uint16_t* targets, float* inv_valid, int B, int seq, int V, cudaStream_t s) {
  if (B <= 0) return;
  launch_pdl(count_valid_targets_kernel, dim3(B), dim3(128), 0, s, targets, inv_valid, B, seq, V);
}

// loss_out[0] = (1/B) * sum_b inv_valid[b] * sum_t loss_rows[b,t]   (single block, double accumulation)
__global__ void reduce_loss_kernel(const float* __restrict__ loss_rows, const float* __restrict__ inv_valid,
                                   float* __restrict__ loss_out, int B, int seq) {
  pdl_trigger();
  pdl_wait();
  double local = 0.0;
  const int n = B * seq;
  for (int i = threadIdx.x; i < n; i += blockDim.x) local += (double)loss_rows[i] * (double)inv_valid[i / seq];
  local = warp_sum_d(local);
  __shared__ double s_p[32];
  if ((threadIdx.x & 31) == 0) s_p[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    double tot = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += s_p[w];
    loss_out[0] = (float)(tot / (double)B);
  }
}
void reduce_loss(const float* loss_rows, const float* inv_valid, float* loss_out, int B, int seq, cudaStream_t s) {
  if (B <= 0) return;
  launch_pdl(reduce_loss_kernel, dim3(1), dim3(1024), 0, s, loss_rows, inv_valid, loss_out, B, seq);
}

// ------------------------------------------------------------------------------------------
// Gradient norm (ane/train_full.go:167-196): sum of squares in double.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
sumsq_kernel(const float* __restrict__ g, uint64_t n, float pre_scale, double* __restrict__ acc) {
  pdl_trigger();
  pdl_wait();
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  double local = 0.0;
  // 16-byte loads, two in flight per thread, when the buffer is aligned; scalar head/tail otherwise.
  const bool vec_ok = (reinterpret_cast<uintptr_t>(g) & 15) == 0;
  const uint64_t n4 = vec_ok ? n / 4 : 0;
  const float4* g4 = reinterpret_cast<const float4*>(g);
  uint64_t i = tid;
  for (; i + stride < n4; i += 2 * stride) {
    const float4 a = __ldg(g4 + i);
    const float4 b = __ldg(g4 + i + stride);
    const float a0 = a.x * pre_scale, a1 = a.y * pre_scale, a2 = a.z * pre_scale, a3 = a.w * pre_scale;
    const float b0 = b.x * pre_scale, b1 = b.y * pre_scale, b2 = b.z * pre_scale, b3 = b.w * pre_scale;
    local += (double)a0 * a0 + (double)a1 * a1 + (double)a2 * a2 + (double)a3 * a3;
    local += (double)b0 * b0 + (double)b1 * b1 + (double)b2 * b2 + (double)b3 * b3;
  }
  for (; i < n4; i += stride) {
    const float4 a = __ldg(g4 + i);
    const float a0 = a.x * pre_scale, a1 = a.y * pre_scale, a2 = a.z * pre_scale, a3 = a.w * pre_scale;
    local += (double)a0 * a0 + (double)a1 * a1 + (double)a2 * a2 + (double)a3 * a3;
  }
  for (uint64_t j = n4 * 4 + tid; j < n; j += stride) {
    const float v = g[j] * pre_scale;
    local += (double)v * (double)v;
  }
  local = warp_sum_d(local);
  __shared__ double s_p[8];
  if ((threadIdx.x & 31) == 0) s_p[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    double tot = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += s_p[w];
    atomicAdd(acc, tot);
  }
}
void sumsq_accumulate(const float* g, uint64_t n, float pre_scale, double* acc, cudaStream_t s) {
  if (!n) return;
  uint64_t grid = (n + 255) / 256;
  if (grid > 148ull * 8) grid = 148ull * 8;
  launch_pdl(sumsq_kernel, dim3((unsigned)grid), dim3(256), 0, s, g, n, pre_scale, acc);
}

__global__ void finalize_clip_kernel(const double* __restrict__ acc, float pre_scale, float clip,
                                     float* __restrict__ scales, float* __restrict__ norm_out) {
  pdl_trigger();
  pdl_wait();
  const double norm2 = acc[0];
  float s = 1.f;
  const float norm = (float)sqrt(norm2);
  if (clip > 0.f && norm2 > 0.0 && norm > clip) s = clip / norm;
  scales[0] = pre_scale;
  scales[1] = pre_scale * s;
  if (norm_out) norm_out[0] = norm;
}
void finalize_clip(const double* acc, float pre_scale, float clip, float* scales, float* norm_out, cudaStream_t s) {
  launch_pdl(finalize_clip_kernel, dim3(1), dim3(1), 0, s, acc, pre_scale, clip, scales, norm_out);
}

// ------------------------------------------------------------------------------------------
// AdamW (ane/train_full.go:1113-1150).  28 B/param of fp32 state traffic + 2 B bf16 shadow.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void adam_one(float& w, float g, float& m, float& v, const AdamHyper& h) {
  m = h.b1 * m + (1.f - h.b1) * g;
  v = h.b2 * v + (1.f - h.b2) * g * g;
  const float mh = m * h.inv_bc1;
  const float vh = v * h.inv_bc2;
  float update = mh / (sqrtf(vh) + h.eps);
  if (h.wd != 0.f) update += h.wd * w;
  w -= h.lr * update;
}

__global__ void __launch_bounds__(256)
adam_kernel(float* __restrict__ w, float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
            bf16* __restrict__ shadow, uint64_t n, AdamHyper h, const float* __restrict__ gscale, int vec_ok) {
  pdl_trigger();
  pdl_wait();
  const float gs = gscale ? *gscale : 1.f;
  const uint64_t n4 = vec_ok ? (n >> 2) : 0;
  uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  float4* w4 = reinterpret_cast<float4*>(w);
  float4* g4 = reinterpret_cast<float4*>(g);
  float4* m4 = reinterpret_cast<float4*>(m);
  float4* v4 = reinterpret_cast<float4*>(v);
  for (uint64_t k = i; k < n4; k += stride) {
    float4 ww = w4[k], gg = g4[k], mm = m4[k], vv = v4[k];
    adam_one(ww.x, gg.x * gs, mm.x, vv.x, h);
    adam_one(ww.y, gg.y * gs, mm.y, vv.y, h);
    adam_one(ww.z, gg.z * gs, mm.z, vv.z, h);
    adam_one(ww.w, gg.w * gs, mm.w, vv.w, h);
    w4[k] = ww;
    m4[k] = mm;
    v4[k] = vv;
    g4[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (shadow) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(ww.x, ww.y), hi = __floats2bfloat162_rn(ww.z, ww.w);
      uint2 u;
      u.x = *reinterpret_cast<uint32_t*>(&lo);
      u.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(shadow)[k] = u;
    }
  }
  for (uint64_t k = (n4 << 2) + i; k < n; k += stride) {
    float ww = w[k], mm = m[k], vv = v[k];
    adam_one(ww, g[k] * gs, mm, vv, h);
    w[k] = ww;
    m[k] = mm;
    v[k] = vv;
    g[k] = 0.f;
    if (shadow) shadow[k] = __float2bfloat16_rn(ww);
  }
}

void adam_update(float* w, float* g, float* m, float* v, bf16* shadow, uint64_t n, AdamHyper h, const float* gscale,
                 cudaStream_t s) {
  if (!n) return;
  uint64_t grid = ((n >> 2) + 255) / 256;
  if (grid > 148ull * 8) grid = 148ull * 8;
  if (grid < 1) grid = 1;
  auto al = [](const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; };
  const int vec_ok = al(w, 16) && al(g, 16) && al(m, 16) && al(v, 16) && (!shadow || al(shadow, 8));
  launch_pdl(adam_kernel, dim3((unsigned)grid), dim3(256), 0, s, w, g, m, v, shadow, n, h, gscale, vec_ok);
}

}  // namespace ane
