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

}  // namespace ane
