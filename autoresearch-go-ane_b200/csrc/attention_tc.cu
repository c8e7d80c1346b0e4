// Causal flash-style attention on tensor cores (bf16 operands, fp32 softmax and accumulation),
// head_dim 64, GQA-aware.  Probabilities are never written to memory: the forward keeps a running
// (max, sum) per query row, the backward recomputes each score tile from Q, K and the saved
// log-sum-exp.  Key/value (forward, dQ) or query/dO (dK/dV) tiles stream through a two-stage
// cp.async ring so loads overlap the MMAs.
//
// Forward restates ane/common.go:61-89; backward restates ane/train_full.go:261-316 (with the
// score scale of the forward) and, fused into its epilogue, the inverse of the rotation of
// ane/train_util.go:204-224, so dq|dk|dv leave the kernel as bf16 GEMM operands.  The reference's
// ANE graphs materialise [heads, seq, seq] probabilities (ane/mil_stories.go:383-432); these
// kernels replace them.
//
// Layout: q|k|v packed token-major [M, (H+2KV)*64]; out [M, H*64]; lse, delta [B, H, seq].
#include <stdlib.h>

#include "common.cuh"
#include "kernels.h"

namespace ane {

namespace {

constexpr int HD = 64;
constexpr int KT = 64;           // streamed tile (keys in fwd/dQ, queries in dK/dV)
constexpr int BR = 128;          // resident tile rows per block (8 warps x 16 rows)
constexpr int LDS = HD + 8;      // padded smem row (144 B: 16-B aligned rows, conflict-free ldmatrix)
constexpr int ATT_THREADS = 256;
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
__device__ __forceinline__ void cp_async_16(bf16* dst, const bf16* src, bool valid) {
  const uint32_t d = smem_u32(dst);
  const int bytes = valid ? 16 : 0;  // 0 => the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Asynchronously copies an [nrows x 64] bf16 tile (row pitch ld) into padded smem; rows >= rows_valid
// are zero-filled.  rows_valid >= 1.
__device__ __forceinline__ void load_tile_async(bf16* dst, const bf16* src, int ld, int nrows, int rows_valid) {
  for (int i = threadIdx.x; i < nrows * (HD / 8); i += ATT_THREADS) {
    const int r = i >> 3, c = (i & 7) * 8;
    const bool ok = r < rows_valid;
    cp_async_16(dst + r * LDS + c, src + (size_t)(ok ? r : 0) * ld + c, ok);
  }
}

// acc (16 x 64) += A(16 rows of a_tile from a_row0; K = HD) * B^T, with B stored [n][k] in b_tile (64 rows).
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

// acc (16 x 64) += P (16 x 64 in registers, accumulator layout, rounded to bf16) * B, with B stored [k][n] (64 rows).
__device__ __forceinline__ void gemm_a_regs_b_kn(float (&acc)[8][4], const float (&p)[8][4], const bf16* b_tile,
                                                 int lane) {
#pragma unroll
  for (int kk = 0; kk < KT / 16; ++kk) {
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
__device__ __forceinline__ void zero_acc(float (&a)[8][4]) {
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) a[i][e] = 0.f;
}

// Writes one accumulator (16 rows x 64 cols per warp) as bf16 into a packed gradient row, optionally
// undoing the pair rotation first (each thread holds whole (even, odd) pairs).
__device__ __forceinline__ void store_grad_bf16(bf16* base, int ld, int row_lo, int T, size_t row0,
                                                const float (&acc)[8][4], const float* cosb, const float* sinb,
                                                int g, int t4) {
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = row_lo + g + r * 8;
    if (row >= T) continue;
    bf16* p = base + (row0 + row) * ld;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      float e = acc[nt][2 * r], o = acc[nt][2 * r + 1];
      if (cosb) {
        const int pair = nt * 4 + t4;
        const float c = cosb[row * (HD / 2) + pair], s = sinb[row * (HD / 2) + pair];
        const float e2 = e * c + o * s, o2 = o * c - e * s;
        e = e2;
        o = o2;
      }
      *reinterpret_cast<__nv_bfloat162*>(p + nt * 8 + 2 * t4) = __floats2bfloat162_rn(e, o);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Forward: grid (query tiles of 128, B*H); 8 warps x 16 query rows; key/value tiles of 64 streamed.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(ATT_THREADS)
attention_fwd_tc_kernel(const bf16* __restrict__ qkv, bf16* __restrict__ out, bf16* __restrict__ out_lo,
                        float* __restrict__ lse, int T, int H, int KV, float scale) {
  extern __shared__ __align__(16) uint8_t att_smem[];
  bf16* Qs = reinterpret_cast<bf16*>(att_smem);   // [BR][LDS]
  bf16* Ks = Qs + BR * LDS;                       // [2][KT][LDS]
  bf16* Vs = Ks + 2 * KT * LDS;                   // [2][KT][LDS]
  const int qt = blockIdx.x, bh = blockIdx.y;
  const int b = bh / H, h = bh - b * H, kvh = h / (H / KV);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  const int ld = (H + 2 * KV) * HD;
  const size_t row0 = (size_t)b * T;
  const int q0 = qt * BR;
  const int q_last = min(q0 + BR, T) - 1;
  const int n_kv = q_last / KT + 1;
  const bf16* kbase = qkv + row0 * ld + (size_t)(H + kvh) * HD;
  const bf16* vbase = qkv + row0 * ld + (size_t)(H + KV + kvh) * HD;
  load_tile_async(Qs, qkv + (row0 + q0) * ld + (size_t)h * HD, ld, BR, min(BR, T - q0));
  load_tile_async(Ks, kbase, ld, KT, min(KT, T));
  load_tile_async(Vs, vbase, ld, KT, min(KT, T));
  cp_async_commit();
  float o[8][4];
  zero_acc(o);
  float m_i[2] = {-INFINITY, -INFINITY}, l_i[2] = {0.f, 0.f};
  const float sl2 = scale * kLog2e;
  const int r_lo = q0 + warp * 16;
  for (int j = 0; j < n_kv; ++j) {
    const int k0 = j * KT;
    if (j + 1 < n_kv) {
      const int kn = k0 + KT;
      load_tile_async(Ks + ((j + 1) & 1) * KT * LDS, kbase + (size_t)kn * ld, ld, KT, min(KT, T - kn));
      load_tile_async(Vs + ((j + 1) & 1) * KT * LDS, vbase + (size_t)kn * ld, ld, KT, min(KT, T - kn));
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (k0 <= r_lo + 15 && r_lo < T) {  // warp-uniform: skip tiles entirely above the diagonal
      const bf16* Kc = Ks + (j & 1) * KT * LDS;
      const bf16* Vc = Vs + (j & 1) * KT * LDS;
      float s[8][4];
      zero_acc(s);
      gemm_a_smem_b_nk(s, Qs, warp * 16, Kc, lane);
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int row = r_lo + g + (e >> 1) * 8;
          const int col = k0 + nt * 8 + 2 * t4 + (e & 1);
          float v = s[nt][e] * sl2;
          if (col > row || col >= T) v = -INFINITY;
          s[nt][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      float corr[2], m_use[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = quad_max(mx[r]);
        const float m_new = fmaxf(m_i[r], mx[r]);
        m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;  // rows with nothing visible yet
        corr[r] = exp2f(m_i[r] - m_use[r]);
        m_i[r] = m_new;
      }
      float rs[2] = {0.f, 0.f};
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p = exp2f(s[nt][e] - m_use[e >> 1]);
          s[nt][e] = p;
          rs[e >> 1] += p;
        }
#pragma unroll
      for (int r = 0; r < 2; ++r) l_i[r] = l_i[r] * corr[r] + rs[r];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[nt][e] *= corr[e >> 1];
      gemm_a_regs_b_kn(o, s, Vc, lane);
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_i[r] = quad_sum(l_i[r]);
    const int row = r_lo + g + r * 8;
    if (row < T) {
      const float inv = 1.0f / l_i[r];
      bf16* op = out + (row0 + row) * (size_t)(H * HD) + (size_t)h * HD;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const float ox = o[nt][2 * r] * inv, oy = o[nt][2 * r + 1] * inv;
        const __nv_bfloat162 hi = __floats2bfloat162_rn(ox, oy);
        *reinterpret_cast<__nv_bfloat162*>(op + nt * 8 + 2 * t4) = hi;
        if (out_lo)  // what the rounding dropped, for the backward's delta
          *reinterpret_cast<__nv_bfloat162*>(out_lo + (op - out) + nt * 8 + 2 * t4) =
              __floats2bfloat162_rn(ox - __bfloat162float(hi.x), oy - __bfloat162float(hi.y));
      }
      if (t4 == 0) lse[((size_t)b * H + h) * T + row] = m_i[r] / kLog2e + logf(l_i[r]);
    }
  }
}

// delta[b,h,t] = sum_d dO * O  (one warp per (token, head))
__global__ void attention_delta_kernel(const bf16* __restrict__ d_out, const bf16* __restrict__ out,
                                       const bf16* __restrict__ out_lo, float* __restrict__ delta, int B, int T, int H) {
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
  if (out_lo) {
    const __nv_bfloat162 d = *reinterpret_cast<const __nv_bfloat162*>(out_lo + off);
    v += __bfloat162float(a.x) * __bfloat162float(d.x) + __bfloat162float(a.y) * __bfloat162float(d.y);
  }
  v = warp_sum(v);
  if (lane == 0) delta[((size_t)b * H + h) * T + t] = v;
}

// ------------------------------------------------------------------------------------------------
// Backward, dQ: grid (query tiles of 128, B*H); key/value tiles streamed.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(ATT_THREADS)
attention_bwd_dq_tc_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ d_out, const float* __restrict__ lse,
                           const float* __restrict__ delta, bf16* __restrict__ dqkv, const float* __restrict__ cosb,
                           const float* __restrict__ sinb, int T, int H, int KV, float scale) {
  extern __shared__ __align__(16) uint8_t att_smem[];
  bf16* Qs = reinterpret_cast<bf16*>(att_smem);   // [BR][LDS]
  bf16* dOs = Qs + BR * LDS;                      // [BR][LDS]
  bf16* Ks = dOs + BR * LDS;                      // [2][KT][LDS]
  bf16* Vs = Ks + 2 * KT * LDS;                   // [2][KT][LDS]
  const int qt = blockIdx.x, bh = blockIdx.y;
  const int b = bh / H, h = bh - b * H, kvh = h / (H / KV);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  const int ld = (H + 2 * KV) * HD;
  const size_t row0 = (size_t)b * T;
  const int q0 = qt * BR;
  const int q_valid = min(BR, T - q0);
  const int n_kv = (q0 + q_valid - 1) / KT + 1;
  const bf16* kbase = qkv + row0 * ld + (size_t)(H + kvh) * HD;
  const bf16* vbase = qkv + row0 * ld + (size_t)(H + KV + kvh) * HD;
  load_tile_async(Qs, qkv + (row0 + q0) * ld + (size_t)h * HD, ld, BR, q_valid);
  load_tile_async(dOs, d_out + (row0 + q0) * (size_t)(H * HD) + (size_t)h * HD, H * HD, BR, q_valid);
  load_tile_async(Ks, kbase, ld, KT, min(KT, T));
  load_tile_async(Vs, vbase, ld, KT, min(KT, T));
  cp_async_commit();
  const int r_lo = q0 + warp * 16;
  float lse_r[2], del_r[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = r_lo + g + r * 8;
    const bool ok = row < T;
    lse_r[r] = ok ? lse[((size_t)b * H + h) * T + row] * kLog2e : 0.f;
    del_r[r] = ok ? delta[((size_t)b * H + h) * T + row] : 0.f;
  }
  float dq[8][4];
  zero_acc(dq);
  const float sl2 = scale * kLog2e;
  for (int j = 0; j < n_kv; ++j) {
    const int k0 = j * KT;
    if (j + 1 < n_kv) {
      const int kn = k0 + KT;
      load_tile_async(Ks + ((j + 1) & 1) * KT * LDS, kbase + (size_t)kn * ld, ld, KT, min(KT, T - kn));
      load_tile_async(Vs + ((j + 1) & 1) * KT * LDS, vbase + (size_t)kn * ld, ld, KT, min(KT, T - kn));
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (k0 <= r_lo + 15 && r_lo < T) {
      const bf16* Kc = Ks + (j & 1) * KT * LDS;
      const bf16* Vc = Vs + (j & 1) * KT * LDS;
      float s[8][4], dp[8][4];
      zero_acc(s);
      zero_acc(dp);
      gemm_a_smem_b_nk(s, Qs, warp * 16, Kc, lane);
      gemm_a_smem_b_nk(dp, dOs, warp * 16, Vc, lane);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int row = r_lo + g + (e >> 1) * 8;
          const int col = k0 + nt * 8 + 2 * t4 + (e & 1);
          float p = 0.f;
          if (col <= row && row < T) p = exp2f(s[nt][e] * sl2 - lse_r[e >> 1]);
          s[nt][e] = p * (dp[nt][e] - del_r[e >> 1]) * scale;  // dS
        }
      gemm_a_regs_b_kn(dq, s, Kc, lane);
    }
    __syncthreads();
  }
  store_grad_bf16(dqkv + (size_t)h * HD, ld, r_lo, T, row0, dq, cosb, sinb, g, t4);
}

// ------------------------------------------------------------------------------------------------
// Backward, dK/dV: grid (key tiles of 128, B*KV); 8 warps x 16 key rows; streams the query/dO tiles
// of every query head that shares this KV head, so no atomics are needed.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(ATT_THREADS, 2)
attention_bwd_dkv_tc_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ d_out,
                            const float* __restrict__ lse, const float* __restrict__ delta, bf16* __restrict__ dqkv,
                            const float* __restrict__ cosb, const float* __restrict__ sinb, int T, int H, int KV,
                            float scale) {
  extern __shared__ __align__(16) uint8_t att_smem[];
  bf16* Ks = reinterpret_cast<bf16*>(att_smem);   // [BR][LDS]
  bf16* Vs = Ks + BR * LDS;                       // [BR][LDS]
  bf16* Qs = Vs + BR * LDS;                       // [2][KT][LDS]
  bf16* dOs = Qs + 2 * KT * LDS;                  // [2][KT][LDS]
  float* lse_s = reinterpret_cast<float*>(dOs + 2 * KT * LDS);  // [2][KT]
  float* del_s = lse_s + 2 * KT;                                // [2][KT]
  const int kt = blockIdx.x, bk = blockIdx.y;
  const int b = bk / KV, kvh = bk - b * KV;
  const int group = H / KV;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  const int ld = (H + 2 * KV) * HD;
  const size_t row0 = (size_t)b * T;
  const int k0 = kt * BR;
  const int k_valid = min(BR, T - k0);
  const int n_qt = (T + KT - 1) / KT;
  const int i0 = k0 / KT;                 // first query tile that can see these keys
  const int per_head = n_qt - i0;
  const int n_it = group * per_head;
  auto issue = [&](int it) {
    const int hq = kvh * group + it / per_head;
    const int q0 = (i0 + it % per_head) * KT;
    const int q_valid = min(KT, T - q0);
    const int bufi = it & 1;
    load_tile_async(Qs + bufi * KT * LDS, qkv + (row0 + q0) * ld + (size_t)hq * HD, ld, KT, q_valid);
    load_tile_async(dOs + bufi * KT * LDS, d_out + (row0 + q0) * (size_t)(H * HD) + (size_t)hq * HD, H * HD, KT,
                    q_valid);
    if (threadIdx.x < KT) {
      const int row = q0 + threadIdx.x;
      const bool ok = row < T;
      lse_s[bufi * KT + threadIdx.x] = ok ? lse[((size_t)b * H + hq) * T + row] * kLog2e : 0.f;
      del_s[bufi * KT + threadIdx.x] = ok ? delta[((size_t)b * H + hq) * T + row] : 0.f;
    }
  };
  load_tile_async(Ks, qkv + (row0 + k0) * ld + (size_t)(H + kvh) * HD, ld, BR, k_valid);
  load_tile_async(Vs, qkv + (row0 + k0) * ld + (size_t)(H + KV + kvh) * HD, ld, BR, k_valid);
  issue(0);
  cp_async_commit();
  float dk[8][4], dv[8][4];
  zero_acc(dk);
  zero_acc(dv);
  const float sl2 = scale * kLog2e;
  const int kr_lo = k0 + warp * 16;
  for (int it = 0; it < n_it; ++it) {
    if (it + 1 < n_it) {
      issue(it + 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int q0 = (i0 + it % per_head) * KT;
    if (q0 + KT - 1 >= kr_lo && kr_lo < T) {  // warp-uniform: some query of this tile sees some key of this warp
      const bf16* Qc = Qs + (it & 1) * KT * LDS;
      const bf16* dOc = dOs + (it & 1) * KT * LDS;
      const float* lse_c = lse_s + (it & 1) * KT;
      const float* del_c = del_s + (it & 1) * KT;
      float st[8][4], dpt[8][4];
      zero_acc(st);
      zero_acc(dpt);
      gemm_a_smem_b_nk(st, Ks, warp * 16, Qc, lane);     // S^T  = K  Q^T
      gemm_a_smem_b_nk(dpt, Vs, warp * 16, dOc, lane);   // dP^T = V dO^T
      // st becomes P^T in place; after dV it becomes dS^T in place, so only two 16x64 temporaries live.
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int krow = kr_lo + g + (e >> 1) * 8;          // key index
          const int qc = nt * 8 + 2 * t4 + (e & 1);            // query index inside the tile
          const int qrow = q0 + qc;
          float p = 0.f;
          if (krow <= qrow && qrow < T) p = exp2f(st[nt][e] * sl2 - lse_c[qc]);
          st[nt][e] = p;
        }
      gemm_a_regs_b_kn(dv, st, dOc, lane);   // dV += P^T dO
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int qc = nt * 8 + 2 * t4 + (e & 1);
          st[nt][e] = st[nt][e] * (dpt[nt][e] - del_c[qc]) * scale;   // dS^T
        }
      gemm_a_regs_b_kn(dk, st, Qc, lane);    // dK += dS^T Q
    }
    __syncthreads();
  }
  store_grad_bf16(dqkv + (size_t)(H + kvh) * HD, ld, kr_lo, T, row0, dk, cosb, sinb, g, t4);
  store_grad_bf16(dqkv + (size_t)(H + KV + kvh) * HD, ld, kr_lo, T, row0, dv, nullptr, nullptr, g, t4);
}

constexpr size_t kFwdSmem = (size_t)(BR + 4 * KT) * LDS * sizeof(bf16);
constexpr size_t kDqSmem = (size_t)(2 * BR + 4 * KT) * LDS * sizeof(bf16);
constexpr size_t kDkvSmem = (size_t)(2 * BR + 4 * KT) * LDS * sizeof(bf16) + 4 * KT * sizeof(float);

bool g_attr_done = false;
bool ensure_attrs() {
  if (g_attr_done) return true;
  if (cudaFuncSetAttribute(attention_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFwdSmem) !=
          cudaSuccess ||
      cudaFuncSetAttribute(attention_bwd_dq_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDqSmem) !=
          cudaSuccess ||
      cudaFuncSetAttribute(attention_bwd_dkv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDkvSmem) !=
          cudaSuccess)
    return false;
  g_attr_done = true;
  return true;
}

}  // namespace

bool attention_tc_supported(int hd) { return hd == HD; }

void attention_forward_tc(const bf16* qkv, bf16* out, bf16* out_lo, float* lse, int B, int seq, int H, int KV, float scale,
                          int* d_status, cudaStream_t s) {
  if (B <= 0 || seq <= 0 || !ensure_attrs()) return;
  static const bool legacy = getenv("ANE_B200_ATT_LEGACY") != nullptr;
  if (!legacy && attention_tcgen05_supported(HD, seq) &&
      attention_forward_tcgen05(qkv, out, out_lo, lse, B, seq, H, KV, scale, d_status, s) == 0)
    return;
  dim3 grid((seq + BR - 1) / BR, B * H);
  attention_fwd_tc_kernel<<<grid, ATT_THREADS, kFwdSmem, s>>>(qkv, out, out_lo, lse, seq, H, KV, scale);
}

int attention_backward_tc(const bf16* qkv, const bf16* out, const bf16* out_lo, const bf16* d_out, const float* lse, float* delta,
                          bf16* dqkv, const float* cosb, const float* sinb, const float* rope_chunks, int B, int seq, int H,
                          int KV, float scale, int* d_status, cudaStream_t s) {
  if (B <= 0 || seq <= 0 || !ensure_attrs()) return 0;
  // ANE_B200_ATT_LEGACY=1 keeps the mma.sync kernels (A/B measurements).
  static const bool legacy = getenv("ANE_B200_ATT_LEGACY") != nullptr;
  if (!legacy && attention_tcgen05_supported(HD, seq)) {
    const int n = attention_backward_tcgen05(qkv, out, out_lo, d_out, lse, delta, dqkv, cosb, sinb, rope_chunks, B, seq, H, KV, scale,
                                             d_status, s);
    if (n > 0) return n;
  }
  const long long warps = (long long)B * seq * H;
  attention_delta_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, s>>>(d_out, out, out_lo, delta, B, seq, H);
  dim3 gq((seq + BR - 1) / BR, B * H);
  attention_bwd_dq_tc_kernel<<<gq, ATT_THREADS, kDqSmem, s>>>(qkv, d_out, lse, delta, dqkv, cosb, sinb, seq, H, KV,
                                                               scale);
  dim3 gk((seq + BR - 1) / BR, B * KV);
  attention_bwd_dkv_tc_kernel<<<gk, ATT_THREADS, kDkvSmem, s>>>(qkv, d_out, lse, delta, dqkv, cosb, sinb, seq, H, KV,
                                                                 scale);
  return 3;
}

}  // namespace ane
