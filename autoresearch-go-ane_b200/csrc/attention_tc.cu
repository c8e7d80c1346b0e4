// Causal flash-style attention on tensor cores (bf16 operands, fp32 softmax and accumulation),
// head_dim 64, GQA-aware.  Probabilities are never written to memory: the forward keeps a running
// (max, sum) per query row, the backward recomputes each 64x64 score tile from Q, K and the saved
// log-sum-exp.
//
// Forward restates ane/common.go:61-89; backward restates ane/train_full.go:261-316 (with the
// score scale of the forward).  The reference's ANE graphs materialise [heads, seq, seq]
// probabilities (ane/mil_stories.go:383-432); these kernels replace them.
//
// Layout: q|k|v packed token-major [M, (H+2KV)*64]; out [M, H*64]; lse, delta [B, H, seq].
#include "common.cuh"
#include "kernels.h"

namespace ane {

namespace {

constexpr int HD = 64;
constexpr int BT = 64;          // query / key tile
constexpr int LDS = HD + 8;     // padded smem row (144 B: 16-B aligned rows, conflict-free ldmatrix)
constexpr int ATT_THREADS = 128;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const bf16* p) {
  const uint32_t a = smem_u32(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const bf16* p) {
  const uint32_t a = smem_u32(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Copies a [64 x 64] bf16 tile (rows row0.., row pitch ld) into padded smem; rows >= rows_valid are zero.
__device__ __forceinline__ void load_tile(bf16* dst, const bf16* src, int ld, int rows_valid) {
  for (int i = threadIdx.x; i < BT * (HD / 8); i += ATT_THREADS) {
    const int r = i >> 3, c = (i & 7) * 8;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < rows_valid) v = *reinterpret_cast<const uint4*>(src + (size_t)r * ld + c);
    *reinterpret_cast<uint4*>(dst + r * LDS + c) = v;
  }
}

// acc[nt][.] (16 x 64) += A(16 rows of `a_tile` starting at a_row0; K = HD) * B^T, with B stored [n][k] in b_tile.
__device__ __forceinline__ void gemm_a_smem_b_nk(float (&acc)[8][4], const bf16* a_tile, int a_row0, const bf16* b_tile,
                                                 int lane) {
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk) {
    uint32_t a[4];
    ldsm_x4(a, a_tile + (a_row0 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDS + kk * 16 + (lane >> 4) * 8);
#pragma unroll
    for (int np = 0; np < 4; ++np) {
      uint32_t b[4];
      ldsm_x4(b, b_tile + (np * 16 + (lane & 7) + (lane >> 4) * 8) * LDS + kk * 16 + ((lane >> 3) & 1) * 8);
      mma_bf16(acc[2 * np], a, b[0], b[1]);
      mma_bf16(acc[2 * np + 1], a, b[2], b[3]);
    }
  }
}

// acc (16 x 64) += P (16 x 64 in registers, accumulator layout `p`, converted to bf16) * B, with B stored [k][n].
__device__ __forceinline__ void gemm_a_regs_b_kn(float (&acc)[8][4], const float (&p)[8][4], const bf16* b_tile,
                                                 int lane) {
#pragma unroll
  for (int kk = 0; kk < BT / 16; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(p[2 * kk][0], p[2 * kk][1]);
    a[1] = pack_bf16(p[2 * kk][2], p[2 * kk][3]);
    a[2] = pack_bf16(p[2 * kk + 1][0], p[2 * kk + 1][1]);
    a[3] = pack_bf16(p[2 * kk + 1][2], p[2 * kk + 1][3]);
#pragma unroll
    for (int np = 0; np < HD / 16; ++np) {
      uint32_t b[4];
      ldsm_x4_t(b, b_tile + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDS + np * 16 + (lane >> 4) * 8);
      mma_bf16(acc[2 * np], a, b[0], b[1]);
      mma_bf16(acc[2 * np + 1], a, b[2], b[3]);
    }
  }
}

__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// ------------------------------------------------------------------------------------------------
// Forward: grid (q tiles, B*H); 4 warps x 16 query rows.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(ATT_THREADS)
attention_fwd_tc_kernel(const bf16* __restrict__ qkv, bf16* __restrict__ out, float* __restrict__ lse, int T, int H,
                        int KV, float scale) {
  __shared__ __align__(16) bf16 Qs[BT * LDS];
  __shared__ __align__(16) bf16 Ks[BT * LDS];
  __shared__ __align__(16) bf16 Vs[BT * LDS];
  const int qt = blockIdx.x, bh = blockIdx.y;
  const int b = bh / H, h = bh - b * H, kvh = h / (H / KV);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  const int ld = (H + 2 * KV) * HD;
  const size_t row0 = (size_t)b * T;
  const int q0 = qt * BT;
  load_tile(Qs, qkv + (row0 + q0) * ld + (size_t)h * HD, ld, min(BT, T - q0));
  float o[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
  float m_i[2] = {-INFINITY, -INFINITY}, l_i[2] = {0.f, 0.f};
  const float sl2 = scale * kLog2e;
  for (int j = 0; j <= qt; ++j) {
    __syncthreads();
    const int k0 = j * BT;
    load_tile(Ks, qkv + (row0 + k0) * ld + (size_t)(H + kvh) * HD, ld, min(BT, T - k0));
    load_tile(Vs, qkv + (row0 + k0) * ld + (size_t)(H + KV + kvh) * HD, ld, min(BT, T - k0));
    __syncthreads();
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[i][e] = 0.f;
    gemm_a_smem_b_nk(s, Qs, warp * 16, Ks, lane);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = q0 + warp * 16 + g + (e >> 1) * 8;
        const int col = k0 + nt * 8 + 2 * t4 + (e & 1);
        float v = s[nt][e] * sl2;
        if (col > row || col >= T) v = -INFINITY;
        s[nt][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    float corr[2], m_new[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = quad_max(mx[r]);
      m_new[r] = fmaxf(m_i[r], mx[r]);
      const float m_use = (m_new[r] == -INFINITY) ? 0.f : m_new[r];  // rows past the sequence end
      corr[r] = exp2f(m_i[r] - m_use);
      m_i[r] = m_new[r];
      m_new[r] = m_use;
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = exp2f(s[nt][e] - m_new[e >> 1]);
        s[nt][e] = p;
        rs[e >> 1] += p;
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) l_i[r] = l_i[r] * corr[r] + rs[r];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[nt][e] *= corr[e >> 1];
    gemm_a_regs_b_kn(o, s, Vs, lane);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_i[r] = quad_sum(l_i[r]);
    const int row = q0 + warp * 16 + g + r * 8;
    if (row < T) {
      const float inv = 1.0f / l_i[r];
      bf16* op = out + (row0 + row) * (size_t)(H * HD) + (size_t)h * HD;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        __nv_bfloat162 v = __floats2bfloat162_rn(o[nt][2 * r] * inv, o[nt][2 * r + 1] * inv);
        *reinterpret_cast<__nv_bfloat162*>(op + nt * 8 + 2 * t4) = v;
      }
      if (t4 == 0) lse[((size_t)b * H + h) * T + row] = m_i[r] / kLog2e + logf(l_i[r]);
    }
  }
}

// delta[b,h,t] = sum_d dO * O  (one warp per (token, head))
__global__ void attention_delta_kernel(const bf16* __restrict__ d_out, const bf16* __restrict__ out,
                                       float* __restrict__ delta, int B, int T, int H) {
  const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)B * T * H) return;
  const int h = (int)(wid % H);
  const long long m = wid / H;
  const int b = (int)(m / T), t = (int)(m - (long long)b * T);
  const size_t off = (size_t)m * (H * HD) + (size_t)h * HD + 2 * lane;
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(d_out + off);
  const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162*>(out + off);
  float v = __bfloat162float(a.x) * __bfloat162float(c.x) + __bfloat162float(a.y) * __bfloat162float(c.y);
  v = warp_sum(v);
  if (lane == 0) delta[((size_t)b * H + h) * T + t] = v;
}

// ------------------------------------------------------------------------------------------------
// Backward, dQ: grid (q tiles, B*H); 4 warps x 16 query rows; loops over key tiles <= q tile.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(ATT_THREADS)
attention_bwd_dq_tc_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ d_out, const float* __restrict__ lse,
                           const float* __restrict__ delta, float* __restrict__ dqkv, int T, int H, int KV,
                           float scale) {
  __shared__ __align__(16) bf16 Qs[BT * LDS];
  __shared__ __align__(16) bf16 dOs[BT * LDS];
  __shared__ __align__(16) bf16 Ks[BT * LDS];
  __shared__ __align__(16) bf16 Vs[BT * LDS];
  const int qt = blockIdx.x, bh = blockIdx.y;
  const int b = bh / H, h = bh - b * H, kvh = h / (H / KV);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  const int ld = (H + 2 * KV) * HD;
  const size_t row0 = (size_t)b * T;
  const int q0 = qt * BT;
  const int q_valid = min(BT, T - q0);
  load_tile(Qs, qkv + (row0 + q0) * ld + (size_t)h * HD, ld, q_valid);
  load_tile(dOs, d_out + (row0 + q0) * (size_t)(H * HD) + (size_t)h * HD, H * HD, q_valid);
  float lse_r[2], del_r[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = q0 + warp * 16 + g + r * 8;
    const bool ok = row < T;
    lse_r[r] = ok ? lse[((size_t)b * H + h) * T + row] * kLog2e : 0.f;
    del_r[r] = ok ? delta[((size_t)b * H + h) * T + row] : 0.f;
  }
  float dq[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) dq[i][e] = 0.f;
  const float sl2 = scale * kLog2e;
  for (int j = 0; j <= qt; ++j) {
    __syncthreads();
    const int k0 = j * BT;
    load_tile(Ks, qkv + (row0 + k0) * ld + (size_t)(H + kvh) * HD, ld, min(BT, T - k0));
    load_tile(Vs, qkv + (row0 + k0) * ld + (size_t)(H + KV + kvh) * HD, ld, min(BT, T - k0));
    __syncthreads();
    float s[8][4], dp[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        s[i][e] = 0.f;
        dp[i][e] = 0.f;
      }
    gemm_a_smem_b_nk(s, Qs, warp * 16, Ks, lane);
    gemm_a_smem_b_nk(dp, dOs, warp * 16, Vs, lane);
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = q0 + warp * 16 + g + (e >> 1) * 8;
        const int col = k0 + nt * 8 + 2 * t4 + (e & 1);
        float p = 0.f;
        if (col <= row && row < T) p = exp2f(s[nt][e] * sl2 - lse_r[e >> 1]);
        s[nt][e] = p * (dp[nt][e] - del_r[e >> 1]) * scale;  // dS
      }
    gemm_a_regs_b_kn(dq, s, Ks, lane);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = q0 + warp * 16 + g + r * 8;
    if (row < T) {
      float* p = dqkv + (row0 + row) * ld + (size_t)h * HD;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
        *reinterpret_cast<float2*>(p + nt * 8 + 2 * t4) = make_float2(dq[nt][2 * r], dq[nt][2 * r + 1]);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Backward, dK/dV: grid (key tiles, B*KV); 4 warps x 16 key rows; loops over the query heads that
// share this KV head and over query tiles >= key tile, so no atomics are needed.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(ATT_THREADS)
attention_bwd_dkv_tc_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ d_out,
                            const float* __restrict__ lse, const float* __restrict__ delta, float* __restrict__ dqkv,
                            int T, int H, int KV, float scale) {
  __shared__ __align__(16) bf16 Qs[BT * LDS];
  __shared__ __align__(16) bf16 dOs[BT * LDS];
  __shared__ __align__(16) bf16 Ks[BT * LDS];
  __shared__ __align__(16) bf16 Vs[BT * LDS];
  __shared__ float lse_s[BT], del_s[BT];
  const int kt = blockIdx.x, bk = blockIdx.y;
  const int b = bk / KV, kvh = bk - b * KV;
  const int group = H / KV;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  const int ld = (H + 2 * KV) * HD;
  const size_t row0 = (size_t)b * T;
  const int k0 = kt * BT;
  load_tile(Ks, qkv + (row0 + k0) * ld + (size_t)(H + kvh) * HD, ld, min(BT, T - k0));
  load_tile(Vs, qkv + (row0 + k0) * ld + (size_t)(H + KV + kvh) * HD, ld, min(BT, T - k0));
  float dk[8][4], dv[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      dk[i][e] = 0.f;
      dv[i][e] = 0.f;
    }
  const float sl2 = scale * kLog2e;
  const int n_qt = (T + BT - 1) / BT;
  for (int hq = kvh * group; hq < (kvh + 1) * group; ++hq) {
    for (int i = kt; i < n_qt; ++i) {
      __syncthreads();
      const int q0 = i * BT;
      const int q_valid = min(BT, T - q0);
      load_tile(Qs, qkv + (row0 + q0) * ld + (size_t)hq * HD, ld, q_valid);
      load_tile(dOs, d_out + (row0 + q0) * (size_t)(H * HD) + (size_t)hq * HD, H * HD, q_valid);
      if (threadIdx.x < BT) {
        const int row = q0 + threadIdx.x;
        const bool ok = row < T;
        lse_s[threadIdx.x] = ok ? lse[((size_t)b * H + hq) * T + row] * kLog2e : 0.f;
        del_s[threadIdx.x] = ok ? delta[((size_t)b * H + hq) * T + row] : 0.f;
      }
      __syncthreads();
      float st[8][4], dpt[8][4];
#pragma unroll
      for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          st[a][e] = 0.f;
          dpt[a][e] = 0.f;
        }
      gemm_a_smem_b_nk(st, Ks, warp * 16, Qs, lane);     // S^T  = K  Q^T
      gemm_a_smem_b_nk(dpt, Vs, warp * 16, dOs, lane);   // dP^T = V dO^T
      float pt[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int krow = k0 + warp * 16 + g + (e >> 1) * 8;   // key index
          const int qc = nt * 8 + 2 * t4 + (e & 1);              // query index inside the tile
          const int qrow = q0 + qc;
          float p = 0.f;
          if (krow <= qrow && qrow < T) p = exp2f(st[nt][e] * sl2 - lse_s[qc]);
          pt[nt][e] = p;
          st[nt][e] = p * (dpt[nt][e] - del_s[qc]) * scale;     // dS^T
        }
      gemm_a_regs_b_kn(dv, pt, dOs, lane);   // dV += P^T dO
      gemm_a_regs_b_kn(dk, st, Qs, lane);    // dK += dS^T Q
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = k0 + warp * 16 + g + r * 8;
    if (row < T) {
      float* pk = dqkv + (row0 + row) * ld + (size_t)(H + kvh) * HD;
      float* pv = dqkv + (row0 + row) * ld + (size_t)(H + KV + kvh) * HD;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        *reinterpret_cast<float2*>(pk + nt * 8 + 2 * t4) = make_float2(dk[nt][2 * r], dk[nt][2 * r + 1]);
        *reinterpret_cast<float2*>(pv + nt * 8 + 2 * t4) = make_float2(dv[nt][2 * r], dv[nt][2 * r + 1]);
      }
    }
  }
}

}  // namespace

bool attention_tc_supported(int hd) { return hd == HD; }

void attention_forward_tc(const bf16* qkv, bf16* out, float* lse, int B, int seq, int H, int KV, float scale,
                          cudaStream_t s) {
  if (B <= 0 || seq <= 0) return;
  dim3 grid((seq + BT - 1) / BT, B * H);
  attention_fwd_tc_kernel<<<grid, ATT_THREADS, 0, s>>>(qkv, out, lse, seq, H, KV, scale);
}

void attention_backward_tc(const bf16* qkv, const bf16* out, const bf16* d_out, const float* lse, float* delta,
                           float* dqkv_f32, int B, int seq, int H, int KV, float scale, cudaStream_t s) {
  if (B <= 0 || seq <= 0) return;
  const long long warps = (long long)B * seq * H;
  attention_delta_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, s>>>(d_out, out, delta, B, seq, H);
  dim3 gq((seq + BT - 1) / BT, B * H);
  attention_bwd_dq_tc_kernel<<<gq, ATT_THREADS, 0, s>>>(qkv, d_out, lse, delta, dqkv_f32, seq, H, KV, scale);
  dim3 gk((seq + BT - 1) / BT, B * KV);
  attention_bwd_dkv_tc_kernel<<<gk, ATT_THREADS, 0, s>>>(qkv, d_out, lse, delta, dqkv_f32, seq, H, KV, scale);
}

}  // namespace ane
