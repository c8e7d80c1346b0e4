// Causal attention, SIMT path: fp32 math on CUDA cores, any head_dim <= 128, GQA-aware.
// It serves the fp32 parity mode and head sizes the tensor-core kernels do not cover.
//
// Forward restates ane/common.go:61-89 (scores * scale, causal mask, softmax, P*V);
// backward restates ane/train_full.go:261-316 with the score scale as an argument
// (the reference hard-codes 1.0 there).
#include "common.cuh"
#include "kernels.h"

namespace ane {

static constexpr int kAttWarps = 4;
static constexpr int kMaxHdPerLane = 4;  // head_dim <= 128

// One warp per query row (b, h, t).  Dynamic smem: kAttWarps * hd floats (query vectors).
template <typename T, typename TO>
__global__ void attention_forward_simt_kernel(const T* __restrict__ qkv, TO* __restrict__ out,
                                              float* __restrict__ lse, int B, int seq, int H, int KV, int hd,
                                              float scale) {
  extern __shared__ float s_q[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long wid = (long long)blockIdx.x * kAttWarps + warp;
  const long long total = (long long)B * H * seq;
  if (wid >= total) return;
  const int t = (int)(wid % seq);
  const int h = (int)((wid / seq) % H);
  const int b = (int)(wid / ((long long)seq * H));
  const int kvh = h / (H / KV);
  const int ld = (H + 2 * KV) * hd;
  const size_t row0 = (size_t)b * seq;
  float* q = s_q + warp * hd;
  const T* qp = qkv + (row0 + t) * ld + (size_t)h * hd;
  for (int d = lane; d < hd; d += 32) q[d] = to_f<T>(qp[d]);
  __syncwarp();
  const T* kbase = qkv + row0 * ld + (size_t)(H + kvh) * hd;
  const T* vbase = qkv + row0 * ld + (size_t)(H + KV + kvh) * hd;
  float m_run = -INFINITY, l_run = 0.f;
  float acc[kMaxHdPerLane] = {0.f, 0.f, 0.f, 0.f};
  for (int j0 = 0; j0 <= t; j0 += 32) {
    const int j = j0 + lane;
    float s = -INFINITY;
    if (j <= t) {
      const T* kp = kbase + (size_t)j * ld;
      float dot = 0.f;
      for (int d = 0; d < hd; ++d) dot += q[d] * to_f<T>(kp[d]);
      s = dot * scale;
    }
    const float m_new = fmaxf(m_run, warp_max(s));
    const float corr = __expf(m_run - m_new);  // exp(-inf) = 0 on the first chunk
    const float p = (j <= t) ? __expf(s - m_new) : 0.f;
    l_run = l_run * corr + warp_sum(p);
#pragma unroll
    for (int c = 0; c < kMaxHdPerLane; ++c) acc[c] *= corr;
    const int lim = min(32, t - j0 + 1);
    for (int jj = 0; jj < lim; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const T* vp = vbase + (size_t)(j0 + jj) * ld;
#pragma unroll
      for (int c = 0; c < kMaxHdPerLane; ++c) {
        const int d = lane + 32 * c;
        if (d < hd) acc[c] += pj * to_f<T>(vp[d]);
      }
    }
    m_run = m_new;
  }
  const float inv = 1.0f / l_run;
  TO* op = out + (row0 + t) * (size_t)(H * hd) + (size_t)h * hd;
#pragma unroll
  for (int c = 0; c < kMaxHdPerLane; ++c) {
    const int d = lane + 32 * c;
    if (d < hd) op[d] = from_f<TO>(acc[c] * inv);
  }
  if (lane == 0 && lse) lse[((size_t)b * H + h) * seq + t] = m_run + logf(l_run);
}

template <typename T, typename TO>
void attention_forward_simt(const T* qkv, TO* out, float* lse, int B, int seq, int H, int KV, int hd, float scale,
                            cudaStream_t s) {
  const long long total = (long long)B * H * seq;
  if (total <= 0) return;
  const unsigned blocks = (unsigned)((total + kAttWarps - 1) / kAttWarps);
  attention_forward_simt_kernel<T, TO><<<blocks, kAttWarps * 32, kAttWarps * hd * sizeof(float), s>>>(qkv, out, lse, B, seq,
                                                                                                   H, KV, hd, scale);
}
template void attention_forward_simt<float, float>(const float*, float*, float*, int, int, int, int, int, float,
                                                   cudaStream_t);
template void attention_forward_simt<bf16, bf16>(const bf16*, bf16*, float*, int, int, int, int, int, float,
                                                 cudaStream_t);
template void attention_forward_simt<float, bf16>(const float*, bf16*, float*, int, int, int, int, int, float,
                                                  cudaStream_t);

// Backward: one warp per query row.  Dynamic smem per warp: 2*hd (q, dO) + 2*seq (scores, dP) floats.
// dq/dk/dv accumulate into a zero-initialised fp32 [M, (H+2KV)*hd] buffer with atomics.
template <typename T, typename TD>
__global__ void attention_backward_simt_kernel(const T* __restrict__ qkv, const TD* __restrict__ d_out,
                                               float* __restrict__ dqkv, int B, int seq, int H, int KV, int hd,
                                               float scale) {
  extern __shared__ float s_mem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long wid = (long long)blockIdx.x * kAttWarps + warp;
  const long long total = (long long)B * H * seq;
  if (wid >= total) return;
  const int t = (int)(wid % seq);
  const int h = (int)((wid / seq) % H);
  const int b = (int)(wid / ((long long)seq * H));
  const int kvh = h / (H / KV);
  const int ld = (H + 2 * KV) * hd;
  const size_t row0 = (size_t)b * seq;
  float* base = s_mem + (size_t)warp * (2 * hd + 2 * seq);
  float* q = base;
  float* dO = base + hd;
  float* sc = base + 2 * hd;
  float* dP = sc + seq;
  const T* qp = qkv + (row0 + t) * ld + (size_t)h * hd;
  const TD* dop = d_out + (row0 + t) * (size_t)(H * hd) + (size_t)h * hd;
  for (int d = lane; d < hd; d += 32) {
    q[d] = to_f<T>(qp[d]);
    dO[d] = to_f<TD>(dop[d]);
  }
  __syncwarp();
  const T* kbase = qkv + row0 * ld + (size_t)(H + kvh) * hd;
  const T* vbase = qkv + row0 * ld + (size_t)(H + KV + kvh) * hd;
  float mx = -INFINITY;
  for (int j = lane; j <= t; j += 32) {
    const T* kp = kbase + (size_t)j * ld;
    const T* vp = vbase + (size_t)j * ld;
    float dot = 0.f, dp = 0.f;
    for (int d = 0; d < hd; ++d) {
      dot += q[d] * to_f<T>(kp[d]);
      dp += dO[d] * to_f<T>(vp[d]);
    }
    sc[j] = dot * scale;
    dP[j] = dp;
    mx = fmaxf(mx, dot * scale);
  }
  mx = warp_max(mx);
  float tot = 0.f;
  for (int j = lane; j <= t; j += 32) {
    const float e = expf(sc[j] - mx);
    sc[j] = e;
    tot += e;
  }
  tot = warp_sum(tot);
  const float inv = 1.0f / tot;
  float ds_sum = 0.f;
  for (int j = lane; j <= t; j += 32) {
    const float p = sc[j] * inv;
    sc[j] = p;
    ds_sum += p * dP[j];
  }
  ds_sum = warp_sum(ds_sum);
  __syncwarp();
  float dq_acc[kMaxHdPerLane] = {0.f, 0.f, 0.f, 0.f};
  float* dkb = dqkv + row0 * ld + (size_t)(H + kvh) * hd;
  float* dvb = dqkv + row0 * ld + (size_t)(H + KV + kvh) * hd;
  for (int j = 0; j <= t; ++j) {
    const float p = sc[j];
    const float ds = p * (dP[j] - ds_sum) * scale;
    const T* kp = kbase + (size_t)j * ld;
#pragma unroll
    for (int c = 0; c < kMaxHdPerLane; ++c) {
      const int d = lane + 32 * c;
      if (d < hd) {
        dq_acc[c] += ds * to_f<T>(kp[d]);
        atomicAdd(dkb + (size_t)j * ld + d, ds * q[d]);
        atomicAdd(dvb + (size_t)j * ld + d, p * dO[d]);
      }
    }
  }
  float* dqp = dqkv + (row0 + t) * ld + (size_t)h * hd;
#pragma unroll
  for (int c = 0; c < kMaxHdPerLane; ++c) {
    const int d = lane + 32 * c;
    if (d < hd) dqp[d] = dq_acc[c];  // each (row, head) is owned by exactly one warp
  }
}

template <typename T, typename TD>
void attention_backward_simt(const T* qkv, const TD* d_out, float* dqkv_f32, int B, int seq, int H, int KV, int hd,
                             float scale, cudaStream_t s) {
  const long long total = (long long)B * H * seq;
  if (total <= 0) return;
  const unsigned blocks = (unsigned)((total + kAttWarps - 1) / kAttWarps);
  const size_t smem = sizeof(float) * (size_t)kAttWarps * (2 * hd + 2 * seq);
  static bool attr_done = false;  // one flag per template instantiation
  if (!attr_done && smem > 48 * 1024) {
    cudaFuncSetAttribute(attention_backward_simt_kernel<T, TD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         200 * 1024);
    attr_done = true;
  }
  attention_backward_simt_kernel<T, TD><<<blocks, kAttWarps * 32, smem, s>>>(qkv, d_out, dqkv_f32, B, seq, H, KV, hd,
                                                                         scale);
}
template void attention_backward_simt<float, float>(const float*, const float*, float*, int, int, int, int, int, float,
                                                    cudaStream_t);
template void attention_backward_simt<bf16, bf16>(const bf16*, const bf16*, float*, int, int, int, int, int, float,
                                                  cudaStream_t);
template void attention_backward_simt<float, bf16>(const float*, const bf16*, float*, int, int, int, int, int, float,
                                                   cudaStream_t);


// ------------------------------------------------------------------------------------------------
// KV cache for decoding: caches are [B, max_seq, KV*hd].
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void kv_cache_copy_kernel(const T* __restrict__ qkv, T* __restrict__ kcache, T* __restrict__ vcache, int B,
                                     int seq, int max_seq, int pos0, int H, int KV, int hd) {
  const int kvd = KV * hd;
  const int ld = (H + 2 * KV) * hd;
  const long long n = (long long)B * seq * kvd;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % kvd);
    const long long m = i / kvd;
    const int b = (int)(m / seq), t = (int)(m - (long long)b * seq);
    const size_t dst = ((size_t)b * max_seq + pos0 + t) * kvd + c;
    kcache[dst] = qkv[(size_t)m * ld + (size_t)H * hd + c];
    vcache[dst] = qkv[(size_t)m * ld + (size_t)(H + KV) * hd + c];
  }
}
template <typename T>
void kv_cache_fill(const T* qkv, T* kcache, T* vcache, int B, int seq, int max_seq, int H, int KV, int hd,
                   cudaStream_t s) {
  const long long n = (long long)B * seq * KV * hd;
  if (n <= 0) return;
  long long g = (n + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  kv_cache_copy_kernel<T><<<(unsigned)g, 256, 0, s>>>(qkv, kcache, vcache, B, seq, max_seq, 0, H, KV, hd);
}
template <typename T>
void kv_cache_append(const T* qkv, T* kcache, T* vcache, int B, int max_seq, int pos, int H, int KV, int hd,
                     cudaStream_t s) {
  const long long n = (long long)B * KV * hd;
  if (n <= 0) return;
  kv_cache_copy_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(qkv, kcache, vcache, B, 1, max_seq, pos, H, KV, hd);
}
template void kv_cache_fill<float>(const float*, float*, float*, int, int, int, int, int, int, cudaStream_t);
template void kv_cache_fill<bf16>(const bf16*, bf16*, bf16*, int, int, int, int, int, int, cudaStream_t);
template void kv_cache_append<float>(const float*, float*, float*, int, int, int, int, int, int, cudaStream_t);
template void kv_cache_append<bf16>(const bf16*, bf16*, bf16*, int, int, int, int, int, int, cudaStream_t);

// One warp per (sequence, head): the single query row attends to cache positions 0..pos.
// One block per (sequence, query head); its warps split the cached positions (warp w takes the 32-key
// chunks w, w + kDecWarps, ...), each keeps a running (max, sum, P*V) and the block merges them at the end.
// Key rows are read with 16-byte loads, value rows as one coalesced 128-byte row per key.
static constexpr int kDecWarps = 8;

template <typename T>
__device__ __forceinline__ float dot_row(const float* q, const T* kp, int hd) {
  float dot = 0.f;
  if constexpr (sizeof(T) == 2) {
    for (int d = 0; d < hd; d += 8) {  // hd % 8 == 0 (checked when the engine opens)
      const uint4 u = *reinterpret_cast<const uint4*>(kp + d);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h2[e]);
        dot += q[d + 2 * e] * f.x + q[d + 2 * e + 1] * f.y;
      }
    }
  } else {
    for (int d = 0; d < hd; d += 4) {
      const float4 f = *reinterpret_cast<const float4*>(kp + d);
      dot += q[d] * f.x + q[d + 1] * f.y + q[d + 2] * f.z + q[d + 3] * f.w;
    }
  }
  return dot;
}

template <typename T>
__global__ void __launch_bounds__(kDecWarps * 32)
attention_decode_simt_kernel(const T* __restrict__ qkv, const T* __restrict__ kcache, const T* __restrict__ vcache,
                             T* __restrict__ out, int B, int max_seq, int pos, int H, int KV, int hd, float scale) {
  extern __shared__ float s_dec[];  // q[hd] | per warp: m, l | per warp: acc[hd]
  float* q = s_dec;
  float* s_m = q + hd;
  float* s_l = s_m + kDecWarps;
  float* s_acc = s_l + kDecWarps;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x / H, h = blockIdx.x - b * H;
  const int kvh = h / (H / KV);
  const int kvd = KV * hd;
  const int ld = (H + 2 * KV) * hd;
  const T* qp = qkv + (size_t)b * ld + (size_t)h * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) q[d] = to_f<T>(qp[d]);
  __syncthreads();
  const T* kbase = kcache + (size_t)b * max_seq * kvd + (size_t)kvh * hd;
  const T* vbase = vcache + (size_t)b * max_seq * kvd + (size_t)kvh * hd;
  float m_run = -INFINITY, l_run = 0.f;
  float acc[kMaxHdPerLane] = {0.f, 0.f, 0.f, 0.f};
  for (int j0 = warp * 32; j0 <= pos; j0 += kDecWarps * 32) {
    const int j = j0 + lane;
    float sc = -INFINITY;
    if (j <= pos) sc = dot_row<T>(q, kbase + (size_t)j * kvd, hd) * scale;
    const float m_new = fmaxf(m_run, warp_max(sc));  // finite: this chunk has at least key j0
    const float corr = __expf(m_run - m_new);
    const float p = (j <= pos) ? __expf(sc - m_new) : 0.f;
    l_run = l_run * corr + warp_sum(p);
#pragma unroll
    for (int c = 0; c < kMaxHdPerLane; ++c) acc[c] *= corr;
    const int lim = min(32, pos - j0 + 1);
    for (int jj = 0; jj < lim; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const T* vp = vbase + (size_t)(j0 + jj) * kvd;
#pragma unroll
      for (int c = 0; c < kMaxHdPerLane; ++c) {
        const int d = lane + 32 * c;
        if (d < hd) acc[c] += pj * to_f<T>(vp[d]);
      }
    }
    m_run = m_new;
  }
  if (lane == 0) {
    s_m[warp] = m_run;
    s_l[warp] = l_run;
  }
#pragma unroll
  for (int c = 0; c < kMaxHdPerLane; ++c) {
    const int d = lane + 32 * c;
    if (d < hd) s_acc[warp * hd + d] = acc[c];
  }
  __syncthreads();
  // merge: warps without any key have m = -inf, l = 0 and drop out
  float m = -INFINITY;
  for (int w = 0; w < kDecWarps; ++w) m = fmaxf(m, s_m[w]);
  float l = 0.f;
  for (int w = 0; w < kDecWarps; ++w) l += s_l[w] * __expf(s_m[w] - m);
  T* op = out + (size_t)b * (H * hd) + (size_t)h * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float o = 0.f;
    for (int w = 0; w < kDecWarps; ++w) o += s_acc[w * hd + d] * __expf(s_m[w] - m);
    op[d] = from_f<T>(o / l);
  }
}
// head_dim 64, bf16 cache: every lane owns whole keys for BOTH products (its key's score, then p * its value
// row into a private 64-wide accumulator), so a chunk of 32 keys costs sixteen 16-byte loads per lane and
// no shuffles; the lanes' accumulators are summed once at the end.  The query heads that share a KV head
// are handled by separate blocks (their K/V rows then come from L2).
__global__ void __launch_bounds__(kDecWarps * 32, 2)
attention_decode_hd64_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                             bf16* __restrict__ out, int B, int max_seq, int pos, int H, int KV, float scale) {
  constexpr int hd = 64;
  __shared__ float q[hd];
  __shared__ float s_m[kDecWarps], s_l[kDecWarps];
  __shared__ float s_acc[kDecWarps][hd];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x / H, h = blockIdx.x - b * H;
  const int kvh = h / (H / KV);
  const int kvd = KV * hd;
  const int ld = (H + 2 * KV) * hd;
  if (threadIdx.x < hd) q[threadIdx.x] = __bfloat162float(qkv[(size_t)b * ld + (size_t)h * hd + threadIdx.x]);
  __syncthreads();
  const bf16* kbase = kcache + (size_t)b * max_seq * kvd + (size_t)kvh * hd;
  const bf16* vbase = vcache + (size_t)b * max_seq * kvd + (size_t)kvh * hd;
  float m_run = -INFINITY, l_lane = 0.f;
  float acc[hd];
#pragma unroll
  for (int d = 0; d < hd; ++d) acc[d] = 0.f;
  for (int j0 = warp * 32; j0 <= pos; j0 += kDecWarps * 32) {
    const int j = j0 + lane;
    const bool valid = j <= pos;
    float sc = -INFINITY;
    if (valid) {
      uint4 kr[8];
      const uint4* kp = reinterpret_cast<const uint4*>(kbase + (size_t)j * kvd);
#pragma unroll
      for (int c = 0; c < 8; ++c) kr[c] = kp[c];
      float dot = 0.f;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&kr[c]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h2[e]);
          dot += q[8 * c + 2 * e] * f.x + q[8 * c + 2 * e + 1] * f.y;
        }
      }
      sc = dot * scale;
    }
    const float m_new = fmaxf(m_run, warp_max(sc));  // finite: this chunk has at least key j0
    const float corr = __expf(m_run - m_new);
    const float p = valid ? __expf(sc - m_new) : 0.f;
    l_lane = l_lane * corr + p;
    if (valid) {
      uint4 vr[8];
      const uint4* vp = reinterpret_cast<const uint4*>(vbase + (size_t)j * kvd);
#pragma unroll
      for (int c = 0; c < 8; ++c) vr[c] = vp[c];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&vr[c]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h2[e]);
          acc[8 * c + 2 * e] = acc[8 * c + 2 * e] * corr + p * f.x;
          acc[8 * c + 2 * e + 1] = acc[8 * c + 2 * e + 1] * corr + p * f.y;
        }
      }
    } else {
#pragma unroll
      for (int d = 0; d < hd; ++d) acc[d] *= corr;
    }
    m_run = m_new;
  }
  // sum the lanes' partial results (they share m_run), then merge the warps
  const float l_warp = warp_sum(l_lane);
#pragma unroll
  for (int d = 0; d < hd; ++d) {
    const float t = warp_sum(acc[d]);
    if (lane == (d & 31)) s_acc[warp][d] = t;
  }
  if (lane == 0) {
    s_m[warp] = m_run;
    s_l[warp] = l_warp;
  }
  __syncthreads();
  if (threadIdx.x < hd) {
    float m = -INFINITY;
    for (int w = 0; w < kDecWarps; ++w) m = fmaxf(m, s_m[w]);
    float l = 0.f, o = 0.f;
    for (int w = 0; w < kDecWarps; ++w) {
      const float f = __expf(s_m[w] - m);  // warps without any key: exp(-inf) = 0
      l += s_l[w] * f;
      o += s_acc[w][threadIdx.x] * f;
    }
    out[(size_t)b * (H * hd) + (size_t)h * hd + threadIdx.x] = __float2bfloat16_rn(o / l);
  }
}

template <typename T>
void attention_decode_simt(const T* qkv, const T* kcache, const T* vcache, T* out, int B, int max_seq, int pos, int H,
                           int KV, int hd, float scale, cudaStream_t s) {
  const int total = B * H;
  if (total <= 0) return;
  if constexpr (sizeof(T) == 2) {
    if (hd == 64) {
      attention_decode_hd64_kernel<<<total, kDecWarps * 32, 0, s>>>(qkv, kcache, vcache, out, B, max_seq, pos, H, KV, scale);
      return;
    }
  }
  const size_t smem = sizeof(float) * (size_t)(hd + 2 * kDecWarps + kDecWarps * hd);
  attention_decode_simt_kernel<T><<<total, kDecWarps * 32, smem, s>>>(qkv, kcache, vcache, out, B, max_seq, pos, H, KV, hd,
                                                                       scale);
}
template void attention_decode_simt<float>(const float*, const float*, const float*, float*, int, int, int, int, int,
                                           int, float, cudaStream_t);
template void attention_decode_simt<bf16>(const bf16*, const bf16*, const bf16*, bf16*, int, int, int, int, int, int,
                                          float, cudaStream_t);

}  // namespace ane
