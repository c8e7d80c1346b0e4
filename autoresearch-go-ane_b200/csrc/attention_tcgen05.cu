// Causal attention on the tcgen05 tensor cores (bf16 operands, fp32 accumulation in tensor memory),
// head_dim 64, sequence length a multiple of 128, GQA-aware.
//
// All three kernels share one shape: a RESIDENT pair of 128-row tiles (R1, R2) stays in shared memory
// for the life of the CTA, a STREAMED pair of 64-row tiles (X1, X2) arrives through a two-stage TMA
// ring, and every iteration is
//
//     MMA 1 :  S' = R1 X1^T   (and dP' = R2 X2^T in the backward)      128 x 64, K = head_dim
//     SIMT  :  one thread per row of S' reads it from tensor memory, applies mask / softmax algebra
//              and writes bf16 operand tiles (128B-swizzled, K-major) back to shared memory
//     MMA 2 :  accumulators (+)= operand tile * X          128 x 64, K = 64 streamed rows
//
//   forward :  R1 = Q_i            X = (K_j, V_j)    O_i  = sum_j P_ij V_j         (online softmax)
//   dK/dV   :  R  = (K_j, V_j)     X = (Q_i, dO_i)   dV_j += P^T dO_i,  dK_j += dS^T Q_i
//   dQ      :  R  = (Q_i, dO_i)    X = (K_j, V_j)    dQ_i += dS K_j
//
// Probabilities never reach global memory; the backward recomputes them from the saved log-sum-exp.
// The rotation of q and k is undone in the dQ / dK epilogues, so dq|dk|dv leave as bf16 GEMM operands.
// Every mbarrier wait is bounded and reports through the status word (see common.cuh).
//
// Forward restates ane/common.go:61-89, backward ane/train_full.go:261-316 (score scale explicit),
// the inverse rotation ane/train_util.go:204-224.
#include "common.cuh"
#include "gemm.h"
#include "gemm_tc.cuh"
#include "kernels.h"

namespace ane {

namespace {

constexpr int A5_THREADS = 320;              // warp 0: TMA, warp 1: MMA, warps 2-9: two threads per tile row
constexpr int A5_COMPUTE = 256;              // (each takes 32 of the 64 columns of its row)
constexpr uint32_t kTileR = 128 * 128;       // resident tile: 128 rows x 128 B
constexpr uint32_t kTileX = 64 * 128;        // streamed tile:  64 rows x 128 B
constexpr float kLog2e = 1.4426950408889634f;

enum Attn5Mode : int { A5_DKV = 1, A5_DQ = 2 };

struct Attn5Params {
  const float* lse;    // [B, H, T] natural-log sum-exp of the scaled scores
  float* delta;        // [B, H, T] rowsum(dO * O): written by the dQ kernel, read by the dK/dV kernel
  bf16* dqkv;          // packed like qkv
  const float* cosb;   // [T, 32] rotation tables or nullptr
  const float* sinb;
  int T, H, KV;
  float scale;
  int* status;
  int o_lo;            // dQ: tm_o_lo holds bf16(O - bf16(O)) from the forward; delta = rowsum(dO * (O + O_lo))
};

// Instruction descriptor: bf16 x bf16 -> fp32, M = 128, N = 64; operand majors selectable.
__host__ __device__ constexpr uint32_t a5_idesc(bool a_mn, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

__device__ __forceinline__ float fast_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void named_bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// Stores 8 consecutive values of a row as one 16-byte chunk of a 128B-swizzled K-major operand tile.
__device__ __forceinline__ void st_chunk(uint8_t* tile, int row, int chunk, const float* v) {
  uint4 u;
  u.x = pack2_bf16(v[0], v[1]);
  u.y = pack2_bf16(v[2], v[3]);
  u.z = pack2_bf16(v[4], v[5]);
  u.w = pack2_bf16(v[6], v[7]);
  *reinterpret_cast<uint4*>(tile + row * 128 + ((chunk ^ (row & 7)) << 4)) = u;
}

// ------------------------------------------------------------------------------------------------
// Backward.  MODE A5_DKV: grid (B*KV, key tiles of 128), streams the (Q, dO) 64-row tiles of every
// query head sharing the KV head (no atomics).  MODE A5_DQ: grid (B*H, query tiles of 128), streams
// the (K, V) 64-row tiles up to the diagonal.  Two CTAs per SM: 256 TMEM columns and < 100 KB each.
// ------------------------------------------------------------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(A5_THREADS, 2)
attn5_bwd_kernel(const __grid_constant__ CUtensorMap tm_qkv_r, const __grid_constant__ CUtensorMap tm_qkv_x,
                 const __grid_constant__ CUtensorMap tm_do_r, const __grid_constant__ CUtensorMap tm_do_x,
                 const __grid_constant__ CUtensorMap tm_o_r, const __grid_constant__ CUtensorMap tm_o_lo,
                 const __grid_constant__ CUtensorMap tm_dqkv,
                 const __grid_constant__ CUtensorMap tm_cos, const __grid_constant__ CUtensorMap tm_sin, Attn5Params p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[2];
  __shared__ __align__(8) uint64_t bar_empty[2];
  __shared__ __align__(8) uint64_t bar_r, bar_s1, bar_s2, bar_p1, bar_p2, bar_acc, bar_cs;
  __shared__ uint32_t tmem_slot;
  __shared__ __align__(16) float ld_s[2][128];  // dK/dV: per streamed query [0,64) lse*log2e, [64,128) delta
  __shared__ float xd[2][128];                  // dQ: partial rowsum(dO * O) per column half

  int* status = p.status;
  if (status != nullptr && *reinterpret_cast<volatile int*>(status) != DEV_OK) return;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sR1 = smem_base, sR2 = sR1 + kTileR;
  const uint32_t sX1 = sR2 + kTileR;           // [2 stages]
  const uint32_t sX2 = sX1 + 2 * kTileX;       // [2 stages]
  const uint32_t sDS = sX2 + 2 * kTileX;       // dS' operand tile
  const uint32_t sP = sDS + kTileR;            // P' operand tile (dK/dV only)
  uint8_t* pR1 = smem_al;
  uint8_t* pR2 = smem_al + kTileR;
  uint8_t* pDS = smem_al + (sDS - smem_base);
  uint8_t* pP = smem_al + (sP - smem_base);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int T = p.T, H = p.H, KV = p.KV, group = H / KV;
  const int nT = T / 128;
  int rt, b, h = 0, kvh, n_per = 1, n_it;
  if constexpr (MODE == A5_DKV) {
    rt = blockIdx.y;  // grid (B*KV, tiles): every heaviest key tile (most visible queries) is scheduled first
    b = blockIdx.x / KV;
    kvh = blockIdx.x - b * KV;
    n_per = T / 64 - 2 * rt;
    n_it = group * n_per;
  } else {
    rt = nT - 1 - blockIdx.y;  // grid (B*H, tiles): heaviest query tiles first
    b = blockIdx.x / H;
    h = blockIdx.x - b * H;
    kvh = h / group;
    n_it = 2 * rt + 2;
  }
  const int row0 = b * T;
  const bool rope = p.cosb != nullptr;

  // Streamed tiles of iteration `it` into ring stage it & 1 (the caller has made sure the stage is free).
  auto issue_x = [&](int it) {
    const int s = it & 1;
    const uint32_t full = smem_u32(&bar_full[s]);
    mbar_expect_tx(full, 2 * kTileX);
    if constexpr (MODE == A5_DKV) {
      const int g = it / n_per;
      const int qh = 2 * rt + (it - g * n_per);
      const int hq = kvh * group + g;
      tma_load_2d(sX1 + s * kTileX, &tm_qkv_x, full, hq * 64, row0 + qh * 64);
      tma_load_2d(sX2 + s * kTileX, &tm_do_x, full, hq * 64, row0 + qh * 64);
    } else {
      tma_load_2d(sX1 + s * kTileX, &tm_qkv_x, full, (H + kvh) * 64, row0 + it * 64);
      tma_load_2d(sX2 + s * kTileX, &tm_qkv_x, full, (H + KV + kvh) * 64, row0 + it * 64);
    }
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    mbar_init(smem_u32(&bar_r), 1);
    mbar_init(smem_u32(&bar_s1), 1);
    mbar_init(smem_u32(&bar_s2), 1);
    mbar_init(smem_u32(&bar_p1), 8);
    mbar_init(smem_u32(&bar_p2), 8);
    mbar_init(smem_u32(&bar_acc), 1);
    mbar_init(smem_u32(&bar_cs), 1);
    fence_mbar_init();
    pdl_wait();  // everything read below was written by earlier kernels
    // The first loads leave before the CTA-wide set-up barrier: their latency overlaps the TMEM allocation.
    const uint32_t rbar = smem_u32(&bar_r);
    mbar_expect_tx(rbar, (MODE == A5_DKV ? 2 : (p.o_lo ? 4 : 3)) * kTileR);
    if constexpr (MODE == A5_DKV) {
      tma_load_2d(sR1, &tm_qkv_r, rbar, (H + kvh) * 64, row0 + rt * 128);
      tma_load_2d(sR2, &tm_qkv_r, rbar, (H + KV + kvh) * 64, row0 + rt * 128);
    } else {
      // The attention output tile O_i rides along (into the still idle dS' buffer) for delta = rowsum(dO * O).
      tma_load_2d(sR1, &tm_qkv_r, rbar, h * 64, row0 + rt * 128);
      tma_load_2d(sR2, &tm_do_r, rbar, h * 64, row0 + rt * 128);
      tma_load_2d(sDS, &tm_o_r, rbar, h * 64, row0 + rt * 128);
      if (p.o_lo) tma_load_2d(sP, &tm_o_lo, rbar, h * 64, row0 + rt * 128);  // P' is not an operand of dQ: its tile is free
    }
    issue_x(0);
    issue_x(1);  // n_it >= 2 always
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), 256);
    tmem_relinquish();
  }
  pdl_trigger();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  const uint32_t tmem_base = tmem_slot;
  const uint32_t tS = tmem_base, tDP = tmem_base + 64, tA1 = tmem_base + 128, tA2 = tmem_base + 192;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      for (int it = 2; it < n_it; ++it) {
        const int s = it & 1;
        const uint32_t ph = (uint32_t)(it >> 1) & 1u;
        if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, status, DEV_MBAR_TIMEOUT_PRODUCER)) break;
        issue_x(it);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_kk = a5_idesc(false, false);  // both operands K-major
      constexpr uint32_t idesc_kn = a5_idesc(false, true);   // B stored [k][n]
      bool ok = mbar_wait(smem_u32(&bar_r), 0, status, DEV_MBAR_TIMEOUT_MMA);
      for (int it = 0; ok && it < n_it; ++it) {
        const int s = it & 1;
        const uint32_t ph = (uint32_t)(it >> 1) & 1u;
        if (!mbar_wait(smem_u32(&bar_full[s]), ph, status, DEV_MBAR_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t x1 = sX1 + s * kTileX, x2 = sX2 + s * kTileX;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tc_mma_bf16(tS, make_smem_desc(sR1 + k * 32, 16, 1024), make_smem_desc(x1 + k * 32, 16, 1024), idesc_kk,
                      k > 0 ? 1u : 0u);
        tc_commit(smem_u32(&bar_s1));  // the row threads turn S' into P' while dP' is still being computed
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tc_mma_bf16(tDP, make_smem_desc(sR2 + k * 32, 16, 1024), make_smem_desc(x2 + k * 32, 16, 1024), idesc_kk,
                      k > 0 ? 1u : 0u);
        tc_commit(smem_u32(&bar_s2));
        const uint32_t par = (uint32_t)it & 1u;
        if constexpr (MODE == A5_DKV) {
          if (!mbar_wait(smem_u32(&bar_p1), par, status, DEV_MBAR_TIMEOUT_MMA)) break;
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < 4; ++k)  // dV += P^T dO, while the row threads still work on dS'
            tc_mma_bf16(tA1, make_smem_desc(sP + k * 32, 16, 1024), make_smem_desc(x2 + k * 2048, 8192, 1024),
                        idesc_kn, (it > 0 || k > 0) ? 1u : 0u);
        }
        if (!mbar_wait(smem_u32(&bar_p2), par, status, DEV_MBAR_TIMEOUT_MMA)) break;
        tc_fence_after();
        if (it == n_it - 1 && rope) {
          // The resident tiles have been read for the last time (the row threads saw this iteration's
          // S' and dP' before arriving): their space takes the rotation tables of these 128 positions.
          const uint32_t cbar = smem_u32(&bar_cs);
          mbar_expect_tx(cbar, 2 * kTileR);
          tma_load_2d(sR1, &tm_cos, cbar, 0, rt * 128);
          tma_load_2d(sR2, &tm_sin, cbar, 0, rt * 128);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k)  // dK += dS^T Q   |   dQ += dS K
          tc_mma_bf16(MODE == A5_DKV ? tA2 : tA1, make_smem_desc(sDS + k * 32, 16, 1024),
                      make_smem_desc(x1 + k * 2048, 8192, 1024), idesc_kn, (it > 0 || k > 0) ? 1u : 0u);
        tc_commit(smem_u32(&bar_empty[s]));
        if (it == n_it - 1) tc_commit(smem_u32(&bar_acc));
      }
    }
  } else {
    // ------------------------------ two threads per tile row ------------------------------
    const int lane_group = warp & 3;                 // TMEM lanes this warp may read
    const int half = (warp - 2) >> 2;                // which 32 of the 64 columns
    const int r = lane_group * 32 + lane;            // row of the resident tile = TMEM lane
    const int ct = threadIdx.x - 64;                 // 0..255 within the compute group
    const uint32_t lane_off = ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(half * 32);
    const float sl2 = p.scale * kLog2e;
    const int rpos = rt * 128 + r;                   // position of this row inside its sequence
    float lse_r = 0.f, del_r = 0.f;
    bool ok = true;
    if constexpr (MODE == A5_DQ) {
      lse_r = p.lse[((size_t)b * H + h) * T + rpos] * kLog2e;
      // delta for these 128 queries, from the dO and O tiles in shared memory; the dK/dV kernel that
      // follows in the stream reads it from global memory.
      ok = mbar_wait(smem_u32(&bar_r), 0, status, DEV_MBAR_TIMEOUT_EPILOGUE);
      float part = 0.f, part_lo = 0.f;
      if (ok) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int off = r * 128 + (((half * 4 + q) ^ (r & 7)) << 4);
          const uint4 a = *reinterpret_cast<const uint4*>(pR2 + off);
          const uint4 c = *reinterpret_cast<const uint4*>(pDS + off);
          const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
          const __nv_bfloat162* c2 = reinterpret_cast<const __nv_bfloat162*>(&c);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 af = __bfloat1622float2(a2[e]), cf = __bfloat1622float2(c2[e]);
            part += af.x * cf.x + af.y * cf.y;
          }
          if (p.o_lo) {
            const uint4 d = *reinterpret_cast<const uint4*>(pP + off);
            const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&d);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 af = __bfloat1622float2(a2[e]), df = __bfloat1622float2(d2[e]);
              part_lo += af.x * df.x + af.y * df.y;
            }
          }
        }
      }
      part += part_lo;
      xd[half][r] = part;
      named_bar_sync(1, A5_COMPUTE);  // also: every read of O is done before dS' is written over it
      del_r = part + xd[half ^ 1][r];
      if (half == 0) p.delta[((size_t)b * H + h) * T + rpos] = del_r;
    }
    for (int it = 0; ok && it < n_it; ++it) {
      const int s = it & 1;
      int xpos0;  // sequence position of the first streamed row
      if constexpr (MODE == A5_DKV) {
        const int g = it / n_per;
        const int qh = 2 * rt + (it - g * n_per);
        const int hq = kvh * group + g;
        xpos0 = qh * 64;
        const size_t base = ((size_t)b * H + hq) * T + xpos0;
        if (ct < 128) ld_s[s][ct] = (ct < 64) ? p.lse[base + ct] * kLog2e : p.delta[base + ct - 64];
        named_bar_sync(1, A5_COMPUTE);
      } else {
        xpos0 = it * 64;
      }
      const uint32_t par = (uint32_t)it & 1u;
      if (!mbar_wait(smem_u32(&bar_s1), par, status, DEV_MBAR_TIMEOUT_EPILOGUE)) {
        ok = false;
        break;
      }
      tc_fence_after();
      float sv[32];
      tmem_ld_32x32(tS + lane_off, sv);
      tmem_ld_wait();
      // Mask only where the tile touches the diagonal (warp-uniform test).
      bool diag;
      if constexpr (MODE == A5_DKV) diag = xpos0 < rt * 128 + 127;
      else diag = xpos0 + 63 > rt * 128;
      const int c0 = xpos0 + half * 32;  // sequence position of this thread's first column
      if constexpr (MODE == A5_DKV) {
        const float4* l4 = reinterpret_cast<const float4*>(&ld_s[s][half * 32]);
#pragma unroll
        for (int e4 = 0; e4 < 8; ++e4) {
          const float4 l = l4[e4];
          const float lv[4] = {l.x, l.y, l.z, l.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int e = e4 * 4 + k;
            float pr = fast_ex2(sv[e] * sl2 - lv[k]);
            if (diag && rpos > c0 + e) pr = 0.f;  // key after query
            sv[e] = pr;
          }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) st_chunk(pP, r, half * 4 + q, sv + 8 * q);
        tc_fence_before();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_p1));
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          float pr = fast_ex2(sv[e] * sl2 - lse_r);
          if (diag && c0 + e > rpos) pr = 0.f;
          sv[e] = pr;
        }
      }
      if (!mbar_wait(smem_u32(&bar_s2), par, status, DEV_MBAR_TIMEOUT_EPILOGUE)) {
        ok = false;
        break;
      }
      tc_fence_after();
      float dv[32];
      tmem_ld_32x32(tDP + lane_off, dv);
      tmem_ld_wait();
      // dS' without the score scale: the accumulators fed by dS' are scaled once in the epilogue.
      if constexpr (MODE == A5_DKV) {
        const float4* d4 = reinterpret_cast<const float4*>(&ld_s[s][64 + half * 32]);
#pragma unroll
        for (int e4 = 0; e4 < 8; ++e4) {
          const float4 d = d4[e4];
          dv[e4 * 4 + 0] = sv[e4 * 4 + 0] * (dv[e4 * 4 + 0] - d.x);
          dv[e4 * 4 + 1] = sv[e4 * 4 + 1] * (dv[e4 * 4 + 1] - d.y);
          dv[e4 * 4 + 2] = sv[e4 * 4 + 2] * (dv[e4 * 4 + 2] - d.z);
          dv[e4 * 4 + 3] = sv[e4 * 4 + 3] * (dv[e4 * 4 + 3] - d.w);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) dv[e] = sv[e] * (dv[e] - del_r);
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) st_chunk(pDS, r, half * 4 + q, dv + 8 * q);
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_p2));
    }
    // Epilogue: accumulators -> bf16 tiles in the (now idle) operand buffers -> TMA stores.  The inverse
    // rotation reads its cos/sin rows from the swizzled tiles the MMA thread fetched over R1 / R2.
    ok = ok && mbar_wait(smem_u32(&bar_acc), 0, status, DEV_MBAR_TIMEOUT_EPILOGUE);
    if (ok && rope) ok = mbar_wait(smem_u32(&bar_cs), 0, status, DEV_MBAR_TIMEOUT_EPILOGUE);
    if (ok) {
      tc_fence_after();
      float a[32];
      auto unrotate = [&]() {
        if (!rope) return;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int off = r * 128 + (((half * 4 + q) ^ (r & 7)) << 4);
          const float4 c = *reinterpret_cast<const float4*>(pR1 + off);
          const float4 s = *reinterpret_cast<const float4*>(pR2 + off);
          const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float ev = a[8 * q + 2 * e], ov = a[8 * q + 2 * e + 1];
            a[8 * q + 2 * e] = ev * cc[e] + ov * ss[e];
            a[8 * q + 2 * e + 1] = ov * cc[e] - ev * ss[e];
          }
        }
      };
      tmem_ld_32x32(tA1 + lane_off, a);
      tmem_ld_wait();
      if constexpr (MODE == A5_DQ) {
#pragma unroll
        for (int e = 0; e < 32; ++e) a[e] *= p.scale;
        unrotate();
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) st_chunk(MODE == A5_DKV ? pP : pDS, r, half * 4 + q, a + 8 * q);  // dV | dQ
      if constexpr (MODE == A5_DKV) {
        tmem_ld_32x32(tA2 + lane_off, a);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) a[e] *= p.scale;
        unrotate();
#pragma unroll
        for (int q = 0; q < 4; ++q) st_chunk(pDS, r, half * 4 + q, a + 8 * q);  // dK
      }
      fence_proxy_async_smem();
    }
    named_bar_sync(1, A5_COMPUTE);
    if (ok && ct == 0) {
      if constexpr (MODE == A5_DKV) {
        tma_store_2d(&tm_dqkv, sP, (H + KV + kvh) * 64, row0 + rt * 128);
        tma_store_2d(&tm_dqkv, sDS, (H + kvh) * 64, row0 + rt * 128);
      } else {
        tma_store_2d(&tm_dqkv, sDS, h * 64, row0 + rt * 128);
      }
      tma_store_commit();
      tma_store_wait_read<0>();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}


// ------------------------------------------------------------------------------------------------
// Forward: grid (B*H, query tiles of 128).  Score tiles are double-buffered in tensor memory so the
// MMA of key block j+1 overlaps the softmax of block j; each P V product lands in its own TMEM
// buffer and is folded into the register-resident output row (with the running-max correction)
// one iteration later, off the critical path.
// ------------------------------------------------------------------------------------------------
struct Attn5FwdParams {
  bf16* out;    // [M, H*64]
  float* lse;   // [B, H, T]
  int T, H, KV;
  float scale;
  int* status;
  int write_lo;  // also store out_lo = bf16(O - bf16(O)) through tm_out_lo (for the backward's delta)
};

__global__ void __launch_bounds__(A5_THREADS, 2)
attn5_fwd_kernel(const __grid_constant__ CUtensorMap tm_qkv_r, const __grid_constant__ CUtensorMap tm_qkv_x,
                 const __grid_constant__ CUtensorMap tm_out, const __grid_constant__ CUtensorMap tm_out_lo,
                 Attn5FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[2];
  __shared__ __align__(8) uint64_t bar_empty[2];
  __shared__ __align__(8) uint64_t bar_s[2];
  __shared__ __align__(8) uint64_t bar_p[2];
  __shared__ __align__(8) uint64_t bar_o[2];
  __shared__ __align__(8) uint64_t bar_r;
  __shared__ uint32_t tmem_slot;
  __shared__ float xmax[2][2][128];  // [block parity][column half][row] partial row maxima

  int* status = p.status;
  if (status != nullptr && *reinterpret_cast<volatile int*>(status) != DEV_OK) return;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sR1 = smem_base;
  const uint32_t sX1 = sR1 + kTileR;           // K blocks [2 stages]
  const uint32_t sX2 = sX1 + 2 * kTileX;       // V blocks [2 stages]
  const uint32_t sP = sX2 + 2 * kTileX;        // P operand tiles [2]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int T = p.T, H = p.H, KV = p.KV, group = H / KV;
  const int rt = T / 128 - 1 - blockIdx.y;     // grid (B*H, tiles): heaviest query tiles first
  const int b = blockIdx.x / H, h = blockIdx.x - b * H, kvh = h / group;
  const int n_it = 2 * rt + 2;
  const int row0 = b * T;

  // K and V blocks of iteration `it` into ring stage it & 1 (the caller has made sure the stage is free).
  auto issue_x = [&](int it) {
    const int s = it & 1;
    const uint32_t full = smem_u32(&bar_full[s]);
    mbar_expect_tx(full, 2 * kTileX);
    tma_load_2d(sX1 + s * kTileX, &tm_qkv_x, full, (H + kvh) * 64, row0 + it * 64);
    tma_load_2d(sX2 + s * kTileX, &tm_qkv_x, full, (H + KV + kvh) * 64, row0 + it * 64);
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
      mbar_init(smem_u32(&bar_s[s]), 1);
      mbar_init(smem_u32(&bar_p[s]), 8);
      mbar_init(smem_u32(&bar_o[s]), 1);
    }
    mbar_init(smem_u32(&bar_r), 1);
    fence_mbar_init();
    pdl_wait();  // q|k|v were written by earlier kernels
    // The first loads leave before the CTA-wide set-up barrier: their latency overlaps the TMEM allocation.
    const uint32_t rbar = smem_u32(&bar_r);
    mbar_expect_tx(rbar, kTileR);
    tma_load_2d(sR1, &tm_qkv_r, rbar, h * 64, row0 + rt * 128);
    issue_x(0);
    issue_x(1);  // n_it >= 2 always
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), 256);
    tmem_relinquish();
  }
  pdl_trigger();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  const uint32_t tmem_base = tmem_slot;  // S[0] S[1] O[0] O[1], 64 columns each

  if (warp == 0) {
    if (lane == 0) {
      for (int it = 2; it < n_it; ++it) {
        const int s = it & 1;
        const uint32_t ph = (uint32_t)(it >> 1) & 1u;
        if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, status, DEV_MBAR_TIMEOUT_PRODUCER)) break;
        issue_x(it);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_kk = a5_idesc(false, false);
      constexpr uint32_t idesc_kn = a5_idesc(false, true);
      auto issue_scores = [&](int it) -> bool {
        const int s = it & 1;
        if (!mbar_wait(smem_u32(&bar_full[s]), (uint32_t)(it >> 1) & 1u, status, DEV_MBAR_TIMEOUT_MMA)) return false;
        tc_fence_after();
        const uint32_t x1 = sX1 + s * kTileX;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tc_mma_bf16(tmem_base + (uint32_t)(s * 64), make_smem_desc(sR1 + k * 32, 16, 1024),
                      make_smem_desc(x1 + k * 32, 16, 1024), idesc_kk, k > 0 ? 1u : 0u);
        tc_commit(smem_u32(&bar_s[s]));
        return true;
      };
      bool ok = mbar_wait(smem_u32(&bar_r), 0, status, DEV_MBAR_TIMEOUT_MMA);
      ok = ok && issue_scores(0);
      for (int it = 0; ok && it < n_it; ++it) {
        const int s = it & 1;
        if (it + 1 < n_it && !issue_scores(it + 1)) break;
        if (!mbar_wait(smem_u32(&bar_p[s]), (uint32_t)(it >> 1) & 1u, status, DEV_MBAR_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t x2 = sX2 + s * kTileX, pt = sP + s * kTileR;
#pragma unroll
        for (int k = 0; k < 4; ++k)  // O_part = P V
          tc_mma_bf16(tmem_base + 128u + (uint32_t)(s * 64), make_smem_desc(pt + k * 32, 16, 1024),
                      make_smem_desc(x2 + k * 2048, 8192, 1024), idesc_kn, k > 0 ? 1u : 0u);
        tc_commit(smem_u32(&bar_o[s]));
        tc_commit(smem_u32(&bar_empty[s]));
      }
    }
  } else {
    // Two threads per query row: each owns 32 of the 64 key columns of a block and 32 of the 64
    // output columns.  Partial row maxima are exchanged through shared memory; row sums stay partial
    // (same running maximum on both sides) and are combined once at the end.
    const int lane_group = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = lane_group * 32 + lane;
    const uint32_t lane_off = ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(half * 32);
    const float sl2 = p.scale * kLog2e;
    const int rpos = rt * 128 + r;
    float o[32];
#pragma unroll
    for (int e = 0; e < 32; ++e) o[e] = 0.f;
    float m_run = -INFINITY, l_part = 0.f, corr_pending = 0.f;
    bool ok = true;
    // o = o * corr + O_part(it), read from tensor memory once its MMA has retired.
    auto fold = [&](int it, float corr) -> bool {
      const int s = it & 1;
      if (!mbar_wait(smem_u32(&bar_o[s]), (uint32_t)(it >> 1) & 1u, status, DEV_MBAR_TIMEOUT_EPILOGUE)) return false;
      tc_fence_after();
      float part[32];
      tmem_ld_32x32(tmem_base + 128u + (uint32_t)(s * 64) + lane_off, part);
      tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 32; ++e) o[e] = o[e] * corr + part[e];
      return true;
    };
    for (int it = 0; it < n_it; ++it) {
      const int s = it & 1;
      const int c0 = it * 64 + half * 32;  // sequence position of this thread's first key
      if (!mbar_wait(smem_u32(&bar_s[s]), (uint32_t)(it >> 1) & 1u, status, DEV_MBAR_TIMEOUT_EPILOGUE)) {
        ok = false;
        break;
      }
      tc_fence_after();
      float sv[32];
      tmem_ld_32x32(tmem_base + (uint32_t)(s * 64) + lane_off, sv);
      tmem_ld_wait();
      const bool diag = it * 64 + 63 > rt * 128;  // warp-uniform
      float mx = -INFINITY;
      if (diag) {
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          sv[e] = (c0 + e <= rpos) ? sv[e] * sl2 : -INFINITY;
          mx = fmaxf(mx, sv[e]);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          sv[e] *= sl2;
          mx = fmaxf(mx, sv[e]);
        }
      }
      xmax[s][half][r] = mx;
      named_bar_sync(1, A5_COMPUTE);
      mx = fmaxf(mx, xmax[s][half ^ 1][r]);
      const float m_new = fmaxf(m_run, mx);  // finite: key 0 is visible to every query
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = fast_ex2(m_run - m_use);
      float rs = 0.f;
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        sv[e] = fast_ex2(sv[e] - m_use);
        rs += sv[e];
      }
      uint8_t* pP = smem_al + (sP - smem_base) + s * kTileR;
#pragma unroll
      for (int q = 0; q < 4; ++q) st_chunk(pP, r, half * 4 + q, sv + 8 * q);
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_p[s]));
      l_part = l_part * corr + rs;
      m_run = m_new;
      // Fold the previous block's P V (its MMA ran while this block's softmax did).
      if (it > 0 && !fold(it - 1, corr_pending)) {
        ok = false;
        break;
      }
      corr_pending = corr;
    }
    ok = ok && fold(n_it - 1, corr_pending);
    float l_run = 1.f;
    if (ok) xmax[0][half][r] = l_part;  // xmax[0] last held maxima at least two barriers ago
    named_bar_sync(1, A5_COMPUTE);
    if (ok) {
      l_run = l_part + xmax[0][half ^ 1][r];
      const float inv = 1.0f / l_run;
#pragma unroll
      for (int e = 0; e < 32; ++e) o[e] *= inv;
      // The output tile is staged in the P buffer that the last P V product did not use (n_it is even,
      // so that is buffer 0; its last reader retired before the previous fold) and leaves by TMA.
      uint8_t* pO = smem_al + (sP - smem_base);
#pragma unroll
      for (int q = 0; q < 4; ++q) st_chunk(pO, r, half * 4 + q, o + 8 * q);
      if (p.write_lo) {
        // What bf16 rounding took away from O, as a second bf16 tile in the other P buffer (its last reader,
        // the final P V product, has been folded above).  The backward forms delta = rowsum(dO * O) from
        // O + O_lo: with O alone, delta's rounding error is the largest error of dQ and dK.
#pragma unroll
        for (int e = 0; e < 32; ++e) o[e] -= __bfloat162float(__float2bfloat16_rn(o[e]));
#pragma unroll
        for (int q = 0; q < 4; ++q) st_chunk(pO + kTileR, r, half * 4 + q, o + 8 * q);
      }
      fence_proxy_async_smem();
      if (half == 0) p.lse[((size_t)b * H + h) * T + rpos] = m_run / kLog2e + logf(l_run);
    }
    named_bar_sync(1, A5_COMPUTE);
    if (ok && threadIdx.x == 64) {
      tma_store_2d(&tm_out, sP, h * 64, row0 + rt * 128);
      if (p.write_lo) tma_store_2d(&tm_out_lo, sP + kTileR, h * 64, row0 + rt * 128);
      tma_store_commit();
      tma_store_wait_read<0>();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

constexpr size_t kFwdSmem5 = kTileR + 4 * kTileX + 2 * kTileR + 1024;

// ------------------------------------------------------------------------------------------------
// Persistent forms.  A work unit is one (sequence, head, 128-row tile); units are numbered heaviest
// first (the tile with the most visible keys of every head, then the next tile, ...) and dealt to the
// grid in boustrophedon order (round 0 left to right, round 1 right to left, ...), which gives every
// CTA the same amount of work to within one unit without a shared counter.  Every warp role walks the
// same list, so nothing about a unit has to be passed between them.
// ------------------------------------------------------------------------------------------------
struct A5Units {
  int n_units;  // B * heads * tiles
  int per_tile; // B * heads: units that share a tile rank
  int heads;    // heads per sequence in this kernel's numbering (H, or KV for the dK/dV kernel)
  int tiles;    // T / 128
  int last_tile_heaviest;  // 1: query tiles (the last sees the most keys); 0: key tiles (the first is seen by the most queries)
};

__device__ __forceinline__ bool a5_unit_at(const A5Units& w, int k, int& rt, int& b, int& h) {
  const int G = (int)gridDim.x, cta = (int)blockIdx.x;
  const int u = (k & 1) ? k * G + (G - 1 - cta) : k * G + cta;
  if (u >= w.n_units) return false;  // rounds only grow: no later unit exists for this CTA either
  const int rank = u / w.per_tile, bh = u - rank * w.per_tile;
  b = bh / w.heads;
  h = bh - b * w.heads;
  rt = w.last_tile_heaviest ? w.tiles - 1 - rank : rank;
  return true;
}

// Persistent forward: grid = min(units, 2 per SM).  One query tile, a THREE-stage ring of (K, V) blocks
// that runs on across unit boundaries, score / P / partial-output buffers alternating with the global
// block counter.  The next unit's Q is fetched as soon as the last score product of the current unit has
// retired, under that unit's last softmax and its epilogue; barriers and tensor memory are set up once.
__global__ void __launch_bounds__(A5_THREADS, 2)
attn5_fwd_persist_kernel(const __grid_constant__ CUtensorMap tm_qkv_r, const __grid_constant__ CUtensorMap tm_qkv_x,
                         const __grid_constant__ CUtensorMap tm_out, const __grid_constant__ CUtensorMap tm_out_lo,
                         Attn5FwdParams p, A5Units w) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[3];
  __shared__ __align__(8) uint64_t bar_empty[3];
  __shared__ __align__(8) uint64_t bar_s[2];
  __shared__ __align__(8) uint64_t bar_p[2];
  __shared__ __align__(8) uint64_t bar_o[2];
  __shared__ __align__(8) uint64_t bar_q, bar_qfree;
  __shared__ uint32_t tmem_slot;
  __shared__ float xmax[2][2][128];  // [block parity][column half][row] partial row maxima

  int* status = p.status;
  if (status != nullptr && *reinterpret_cast<volatile int*>(status) != DEV_OK) return;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base;
  const uint32_t sX1 = sQ + kTileR;            // K blocks [3 stages]
  const uint32_t sX2 = sX1 + 3 * kTileX;       // V blocks [3 stages]
  const uint32_t sP = sX2 + 3 * kTileX;        // P operand tiles [2]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int T = p.T, H = p.H, KV = p.KV, group = H / KV;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 3; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&bar_s[s]), 1);
      mbar_init(smem_u32(&bar_p[s]), 8);
      mbar_init(smem_u32(&bar_o[s]), 1);
    }
    mbar_init(smem_u32(&bar_q), 1);
    mbar_init(smem_u32(&bar_qfree), 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), 256);
    tmem_relinquish();
  }
  pdl_trigger();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();  // q|k|v were written by earlier kernels
  const uint32_t tmem_base = tmem_slot;  // S[0] S[1] O[0] O[1], 64 columns each

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int g = 0;  // blocks issued so far, over all units
      bool ok = true;
      for (int k = 0; ok; ++k) {
        int rt, b, h;
        if (!a5_unit_at(w, k, rt, b, h)) break;
        const int kvh = h / group, row0 = b * T, n_it = 2 * rt + 2;
        for (int it = 0; it < n_it; ++it, ++g) {
          const int s = g % 3;
          if (g >= 3 && !mbar_wait(smem_u32(&bar_empty[s]), ((uint32_t)(g / 3) & 1u) ^ 1u, status,
                                   DEV_MBAR_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&bar_full[s]);
          mbar_expect_tx(full, 2 * kTileX);
          tma_load_2d(sX1 + s * kTileX, &tm_qkv_x, full, (H + kvh) * 64, row0 + it * 64);
          tma_load_2d(sX2 + s * kTileX, &tm_qkv_x, full, (H + KV + kvh) * 64, row0 + it * 64);
          if (it == 0) {
            // The query tile's buffer is free once every score product of the previous unit has retired.
            if (k > 0 && !mbar_wait(smem_u32(&bar_qfree), (uint32_t)(k - 1) & 1u, status, DEV_MBAR_TIMEOUT_PRODUCER)) {
              ok = false;
              break;
            }
            const uint32_t qb = smem_u32(&bar_q);
            mbar_expect_tx(qb, kTileR);
            tma_load_2d(sQ, &tm_qkv_r, qb, h * 64, row0 + rt * 128);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_kk = a5_idesc(false, false);
      constexpr uint32_t idesc_kn = a5_idesc(false, true);
      auto issue_scores = [&](int gg) -> bool {
        const int s3 = gg % 3;
        if (!mbar_wait(smem_u32(&bar_full[s3]), (uint32_t)(gg / 3) & 1u, status, DEV_MBAR_TIMEOUT_MMA)) return false;
        tc_fence_after();
        const uint32_t x1 = sX1 + s3 * kTileX;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tc_mma_bf16(tmem_base + (uint32_t)((gg & 1) * 64), make_smem_desc(sQ + k * 32, 16, 1024),
                      make_smem_desc(x1 + k * 32, 16, 1024), idesc_kk, k > 0 ? 1u : 0u);
        tc_commit(smem_u32(&bar_s[gg & 1]));
        return true;
      };
      int g = 0;
      bool ok = true;
      for (int k = 0; ok; ++k) {
        int rt, b, h;
        if (!a5_unit_at(w, k, rt, b, h)) break;
        const int n_it = 2 * rt + 2;
        ok = mbar_wait(smem_u32(&bar_q), (uint32_t)k & 1u, status, DEV_MBAR_TIMEOUT_MMA);
        ok = ok && issue_scores(g);
        for (int it = 0; ok && it < n_it; ++it, ++g) {
          if (it + 1 < n_it) {
            // The next block's scores run under this block's softmax.  (Not across a unit boundary: the
            // next unit's Q may still be on its way, and waiting for it here would hold back this P V.)
            if (!issue_scores(g + 1)) {
              ok = false;
              break;
            }
            if (it + 2 == n_it) tc_commit(smem_u32(&bar_qfree));  // this unit's last use of Q
          }
          const int s = g & 1, s3 = g % 3;
          if (!mbar_wait(smem_u32(&bar_p[s]), (uint32_t)(g >> 1) & 1u, status, DEV_MBAR_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t x2 = sX2 + s3 * kTileX, pt = sP + s * kTileR;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)  // O_part = P V
            tc_mma_bf16(tmem_base + 128u + (uint32_t)(s * 64), make_smem_desc(pt + kk * 32, 16, 1024),
                        make_smem_desc(x2 + kk * 2048, 8192, 1024), idesc_kn, kk > 0 ? 1u : 0u);
          tc_commit(smem_u32(&bar_o[s]));
          tc_commit(smem_u32(&bar_empty[s3]));
        }
      }
    }
  } else {
    // Two threads per query row, as in the one-unit kernel.
    const int lane_group = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = lane_group * 32 + lane;
    const uint32_t lane_off = ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(half * 32);
    const float sl2 = p.scale * kLog2e;
    uint8_t* pP0 = smem_al + (sP - smem_base);
    int g = 0;
    bool ok = true;
    float o[32];
    // o = o * corr + O_part(block gg), read from tensor memory once its MMA has retired.
    auto fold = [&](int gg, float corr) -> bool {
      const int s = gg & 1;
      if (!mbar_wait(smem_u32(&bar_o[s]), (uint32_t)(gg >> 1) & 1u, status, DEV_MBAR_TIMEOUT_EPILOGUE)) return false;
      tc_fence_after();
      float part[32];
      tmem_ld_32x32(tmem_base + 128u + (uint32_t)(s * 64) + lane_off, part);
      tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 32; ++e) o[e] = o[e] * corr + part[e];
      return true;
    };
    for (int k = 0; ok; ++k) {
      int rt, b, h;
      if (!a5_unit_at(w, k, rt, b, h)) break;
      const int n_it = 2 * rt + 2, row0 = b * T, rpos = rt * 128 + r;
#pragma unroll
      for (int e = 0; e < 32; ++e) o[e] = 0.f;
      float m_run = -INFINITY, l_part = 0.f, corr_pending = 0.f;
      for (int it = 0; it < n_it; ++it, ++g) {
        const int s = g & 1;
        const int c0 = it * 64 + half * 32;  // sequence position of this thread's first key
        if (!mbar_wait(smem_u32(&bar_s[s]), (uint32_t)(g >> 1) & 1u, status, DEV_MBAR_TIMEOUT_EPILOGUE)) {
          ok = false;
          break;
        }
        tc_fence_after();
        float sv[32];
        tmem_ld_32x32(tmem_base + (uint32_t)(s * 64) + lane_off, sv);
        tmem_ld_wait();
        const bool diag = it * 64 + 63 > rt * 128;  // warp-uniform
        float mx = -INFINITY;
        if (diag) {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            sv[e] = (c0 + e <= rpos) ? sv[e] * sl2 : -INFINITY;
            mx = fmaxf(mx, sv[e]);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            sv[e] *= sl2;
            mx = fmaxf(mx, sv[e]);
          }
        }
        xmax[s][half][r] = mx;
        // The previous unit's output left through the two P buffers: its store must have read them
        // before this unit writes probabilities there (the barrier below publishes that to everyone).
        if (it == 0 && k > 0 && threadIdx.x == 64) tma_store_wait_read<0>();
        named_bar_sync(1, A5_COMPUTE);
        mx = fmaxf(mx, xmax[s][half ^ 1][r]);
        const float m_new = fmaxf(m_run, mx);  // finite: key 0 is visible to every query
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float corr = fast_ex2(m_run - m_use);
        float rs = 0.f;
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          sv[e] = fast_ex2(sv[e] - m_use);
          rs += sv[e];
        }
        uint8_t* pP = pP0 + s * kTileR;
#pragma unroll
        for (int q = 0; q < 4; ++q) st_chunk(pP, r, half * 4 + q, sv + 8 * q);
        tc_fence_before();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_p[s]));
        l_part = l_part * corr + rs;
        m_run = m_new;
        if (it > 0 && !fold(g - 1, corr_pending)) {
          ok = false;
          break;
        }
        corr_pending = corr;
      }
      ok = ok && fold(g - 1, corr_pending);
      float l_run = 1.f;
      if (ok) xmax[0][half][r] = l_part;  // xmax[0] last held maxima at least two barriers ago
      named_bar_sync(1, A5_COMPUTE);
      if (ok) {
        l_run = l_part + xmax[0][half ^ 1][r];
        const float inv = 1.0f / l_run;
#pragma unroll
        for (int e = 0; e < 32; ++e) o[e] *= inv;
        // Staged in the two P buffers: both P V products that read them were folded above.
#pragma unroll
        for (int q = 0; q < 4; ++q) st_chunk(pP0, r, half * 4 + q, o + 8 * q);
        if (p.write_lo) {
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] -= __bfloat162float(__float2bfloat16_rn(o[e]));
#pragma unroll
          for (int q = 0; q < 4; ++q) st_chunk(pP0 + kTileR, r, half * 4 + q, o + 8 * q);
        }
        fence_proxy_async_smem();
        if (half == 0) p.lse[((size_t)b * H + h) * T + rpos] = m_run / kLog2e + logf(l_run);
      }
      named_bar_sync(1, A5_COMPUTE);
      if (ok && threadIdx.x == 64) {
        tma_store_2d(&tm_out, sP, h * 64, row0 + rt * 128);
        if (p.write_lo) tma_store_2d(&tm_out_lo, sP + kTileR, h * 64, row0 + rt * 128);
        tma_store_commit();
      }
    }
    if (threadIdx.x == 64) tma_store_wait_read<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

constexpr size_t kFwdPersistSmem = kTileR + 6 * kTileX + 2 * kTileR + 1024;

// ------------------------------------------------------------------------------------------------
// Backward with one CTA per (sequence, head), for seq = 256 without grouped heads: the head's Q, K, V
// and dO (eight 128-row tiles) stay in shared memory, and its three visible 128 x 128 blocks
// (q0 k0), (q1 k0), (q1 k1) are walked once.  Per block
//
//     MMA   :  S = Q_i K_j^T,  dP = dO_i V_j^T                         128 x 128, K = head_dim
//     SIMT  :  two threads per query row: P = 2^(S scale log2e - lse),  dS = P (dP - delta)  -> bf16 tiles
//     MMA   :  dV_j += P^T dO_i,  dK_j += dS^T Q_i  (A read M-major from the same tile),  dQ_i += dS K_j
//
// so probabilities and both score products are formed once per block, where the two-kernel form above
// forms them twice, and the five accumulators (dQ_0, dQ_1, dK_j, dV_j next to S and dP: all 512
// columns of tensor memory) never leave the SM.  The next block's S is issued as soon as the row
// threads have copied the current one to registers, its dP likewise, so the row threads run back to back.
// Finished accumulators (dQ_0, dK_0, dV_0 after the second block, the others after the third) are staged in
// two spare tiles and in V0 / K1 / V1, dead by then, and sent out by the producer thread.  The same thread
// fetches the NEXT head's tiles, each group as soon as its tiles are free: Q0 and dO0 when the first block's
// MMAs have retired, K0 after the second block's, V0 when the store of dV_0 has read it, Q1 and dO1 after the
// third block's, K1 and V1 after their stores - so a head's first block finds its operands waiting.  delta is
// rowsum(P dP) for the first query tile (its one block holds whole rows) and rowsum(dO (O + O_lo)) for the
// second, from O tiles parked in the spare tiles while those are idle.
// ------------------------------------------------------------------------------------------------
__host__ __device__ constexpr uint32_t a5_idesc_n(bool a_mn, bool b_mn, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

struct Attn5HeadParams {
  const float* lse;    // [B, H, T] natural-log sum-exp of the scaled scores
  float* delta;        // [B, H, T] rowsum(dO * O), written for inspection
  const bf16* o;       // [M, H*64] attention output (read through its tensor map)
  const bf16* o_lo;    // bf16(O - bf16(O)) or nullptr: whether the second tensor map is read as well
  bf16* dqkv;          // [M, 3*H*64] dq | dk | dv
  const float4* rope;  // rotation tables by 16-byte chunk: [cos chunk 0..7 | sin chunk 0..7][T] (see
                       // attention_rope_chunk_tables), or nullptr for no rotation
  int H;
  float scale;
  int* status;
  int n_units;         // B * H
  uint32_t smem_bytes; // dynamic shared memory of the launch
};

__global__ void __launch_bounds__(A5_THREADS, 1)
attn5_bwd_head_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_do,
                      const __grid_constant__ CUtensorMap tm_o, const __grid_constant__ CUtensorMap tm_o_lo,
                      const __grid_constant__ CUtensorMap tm_dqkv, Attn5HeadParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_ldq0, bar_ldk0, bar_ldv0, bar_ldq1, bar_ldkv1, bar_ldo, bar_stage0, bar_stage1, bar_stfree;
  __shared__ __align__(8) uint64_t bar_s, bar_dp, bar_sfree, bar_dpfree, bar_p1, bar_p2, bar_pfree, bar_dsfree;
  __shared__ __align__(8) uint64_t bar_acc0, bar_acc1, bar_acc2, bar_kvdr, bar_findr;
  __shared__ uint32_t tmem_slot;
  __shared__ float xd[2][2][128];  // [query tile][column half][row] partial rowsum(dO * O)

  int* status = p.status;
  if (status != nullptr && *reinterpret_cast<volatile int*>(status) != DEV_OK) return;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  // tiles: Q0 Q1 K0 K1 V0 V1 dO0 dO1, then P (two 64-key halves), dS (two halves) and two staging tiles
  const uint32_t sQ = smem_base, sK = sQ + 2 * kTileR, sV = sK + 2 * kTileR, sDO = sV + 2 * kTileR;
  const uint32_t sP = sDO + 2 * kTileR, sDS = sP + 2 * kTileR, sT = sDS + 2 * kTileR;
  if (sT + 2 * kTileR > smem_u32(smem_raw) + p.smem_bytes) {  // the launch did not get the room this layout needs
    if (threadIdx.x == 0 && status != nullptr) atomicCAS(status, DEV_OK, DEV_MBAR_TIMEOUT_PRODUCER);
    return;
  }
  auto ptr = [&](uint32_t a) { return smem_al + (a - smem_base); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int T = 256;
  const int H = p.H, n_units = p.n_units;
  const bool rope = p.rope != nullptr;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar_ldq0), 1);
    mbar_init(smem_u32(&bar_ldk0), 1);
    mbar_init(smem_u32(&bar_ldv0), 1);
    mbar_init(smem_u32(&bar_ldq1), 1);
    mbar_init(smem_u32(&bar_ldkv1), 1);
    mbar_init(smem_u32(&bar_ldo), 1);
    mbar_init(smem_u32(&bar_stage0), 8);
    mbar_init(smem_u32(&bar_stage1), 8);
    mbar_init(smem_u32(&bar_stfree), 1);
    mbar_init(smem_u32(&bar_s), 1);
    mbar_init(smem_u32(&bar_dp), 1);
    mbar_init(smem_u32(&bar_sfree), 8);
    mbar_init(smem_u32(&bar_dpfree), 8);
    mbar_init(smem_u32(&bar_p1), 8);
    mbar_init(smem_u32(&bar_p2), 8);
    mbar_init(smem_u32(&bar_pfree), 1);
    mbar_init(smem_u32(&bar_dsfree), 1);
    mbar_init(smem_u32(&bar_acc0), 1);
    mbar_init(smem_u32(&bar_acc1), 1);
    mbar_init(smem_u32(&bar_acc2), 1);
    mbar_init(smem_u32(&bar_kvdr), 8);
    mbar_init(smem_u32(&bar_findr), 8);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), 512);
    tmem_relinquish();
  }
  pdl_trigger();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();  // everything read below was written by earlier kernels
  const uint32_t tmem_base = tmem_slot;
  const uint32_t tS = tmem_base, tDP = tmem_base + 128, tDQ0 = tmem_base + 256, tDQ1 = tmem_base + 320,
                 tDK = tmem_base + 384, tDV = tmem_base + 448;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      bool ok = true;
      auto load = [&](uint32_t dst, const CUtensorMap* tm, uint32_t bar, int col, int row) {
        tma_load_2d(dst, tm, bar, col, row);
      };
      // The five load groups of unit u, in the order their tiles fall free in the previous head.
      auto load_q0 = [&](int u) {  // Q0, dO0: free when the first block's MMAs have retired
        const int b = u / H, h = u - b * H, row = b * T;
        const uint32_t l = smem_u32(&bar_ldq0);
        mbar_expect_tx(l, 2u * kTileR);
        load(sQ, &tm_qkv, l, h * 64, row);
        load(sDO, &tm_do, l, h * 64, row);
      };
      auto load_k0 = [&](int u) {  // K0: free when the second block's MMAs have retired
        const int b = u / H, h = u - b * H, row = b * T;
        const uint32_t l = smem_u32(&bar_ldk0);
        mbar_expect_tx(l, kTileR);
        load(sK, &tm_qkv, l, (H + h) * 64, row);
      };
      auto load_v0 = [&](int u) {  // V0: staged dV_0
        const int b = u / H, h = u - b * H, row = b * T;
        const uint32_t l = smem_u32(&bar_ldv0);
        mbar_expect_tx(l, kTileR);
        load(sV, &tm_qkv, l, (2 * H + h) * 64, row);
      };
      auto load_q1 = [&](int u) {  // Q1, dO1: free when the third block's MMAs have retired
        const int b = u / H, h = u - b * H, row = b * T + 128;
        const uint32_t l = smem_u32(&bar_ldq1);
        mbar_expect_tx(l, 2u * kTileR);
        load(sQ + kTileR, &tm_qkv, l, h * 64, row);
        load(sDO + kTileR, &tm_do, l, h * 64, row);
      };
      auto load_kv1 = [&](int u) {  // K1, V1: staged dK_1, dV_1
        const int b = u / H, h = u - b * H, row = b * T + 128;
        const uint32_t l = smem_u32(&bar_ldkv1);
        mbar_expect_tx(l, 2u * kTileR);
        load(sK + kTileR, &tm_qkv, l, (H + h) * 64, row);
        load(sV + kTileR, &tm_qkv, l, (2 * H + h) * 64, row);
      };
      auto load_o1 = [&](int u) {  // O and O_lo of query tile 1 into the two spare tiles, idle until the first drain
        const int b = u / H, h = u - b * H, row = b * T + 128;
        const uint32_t l = smem_u32(&bar_ldo);
        mbar_expect_tx(l, (p.o_lo != nullptr ? 2u : 1u) * kTileR);
        load(sT, &tm_o, l, h * 64, row);
        if (p.o_lo != nullptr) load(sT + kTileR, &tm_o_lo, l, h * 64, row);
      };
      // dQ_t, dK_t, dV_t as the row threads staged them: out by TMA; once the stores have read their
      // tiles those are free (for the next drain, or for the next head's data).
      auto store_group = [&](int u, int t, uint32_t s_dq, uint32_t s_dk, uint32_t s_dv, uint64_t* staged, uint32_t parity) {
        ok = ok && mbar_wait(smem_u32(staged), parity, status, DEV_MBAR_TIMEOUT_PRODUCER);
        const int b = u / H, h = u - b * H, row = b * T + t * 128;
        if (ok) {
          tma_store_2d(&tm_dqkv, s_dq, h * 64, row);
          tma_store_2d(&tm_dqkv, s_dk, (H + h) * 64, row);
          tma_store_2d(&tm_dqkv, s_dv, (2 * H + h) * 64, row);
        }
        tma_store_commit();
        tma_store_wait_read<0>();
        mbar_arrive(smem_u32(&bar_stfree));
      };
      if ((int)blockIdx.x < n_units) {
        load_q0(blockIdx.x);
        load_k0(blockIdx.x);
        load_v0(blockIdx.x);
        load_q1(blockIdx.x);
        load_o1(blockIdx.x);
        load_kv1(blockIdx.x);
      }
      int k = 0;
      for (int u = blockIdx.x; u < n_units; u += gridDim.x, ++k) {
        const int un = u + (int)gridDim.x;
        const bool more = un < n_units;
        const uint32_t kp = (uint32_t)k & 1u;
        ok = ok && mbar_wait(smem_u32(&bar_acc0), kp, status, DEV_MBAR_TIMEOUT_PRODUCER);
        if (more) load_q0(un);
        ok = ok && mbar_wait(smem_u32(&bar_acc1), kp, status, DEV_MBAR_TIMEOUT_PRODUCER);
        if (more) load_k0(un);
        store_group(u, 0, sT, sT + kTileR, sV, &bar_stage0, kp);
        if (more) load_v0(un);
        ok = ok && mbar_wait(smem_u32(&bar_acc2), kp, status, DEV_MBAR_TIMEOUT_PRODUCER);
        if (more) load_q1(un);
        store_group(u, 1, sT, sK + kTileR, sV + kTileR, &bar_stage1, kp);
        if (more) load_o1(un);
        if (more) load_kv1(un);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------
    if (lane == 0) {
      constexpr uint32_t id_s = a5_idesc_n(false, false, 128);  // S, dP: both operands K-major, N = 128 keys
      constexpr uint32_t id_t = a5_idesc_n(true, true, 64);     // dV, dK: A = P^T / dS^T read M-major, B stored [k][n]
      constexpr uint32_t id_q = a5_idesc_n(false, true, 64);    // dQ: A = dS K-major, B = K stored [k][n]
      auto scores = [&](int i, int j) {  // S = Q_i K_j^T
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          tc_mma_bf16(tS, make_smem_desc(sQ + i * kTileR + kk * 32, 16, 1024),
                      make_smem_desc(sK + j * kTileR + kk * 32, 16, 1024), id_s, kk > 0 ? 1u : 0u);
        tc_commit(smem_u32(&bar_s));
      };
      auto dprobs = [&](int i, int j) {  // dP = dO_i V_j^T
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          tc_mma_bf16(tDP, make_smem_desc(sDO + i * kTileR + kk * 32, 16, 1024),
                      make_smem_desc(sV + j * kTileR + kk * 32, 16, 1024), id_s, kk > 0 ? 1u : 0u);
        tc_commit(smem_u32(&bar_dp));
      };
      // acc[128 keys x 64] (+)= X^T B_i with X = P or dS ([128 queries x 128 keys] in two 64-key halves)
      auto transposed = [&](uint32_t acc, uint32_t x, uint32_t bt, bool accumulate) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)  // 16 queries per step
          tc_mma_bf16(acc, make_smem_desc(x + kk * 2048, kTileR, 1024), make_smem_desc(bt + kk * 2048, 8192, 1024), id_t,
                      (accumulate || kk > 0) ? 1u : 0u);
      };
      auto dq = [&](uint32_t acc, int j, bool accumulate) {  // dQ_i (+)= dS K_j
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)  // 16 keys per step: half kk / 4 of the dS tile
          tc_mma_bf16(acc, make_smem_desc(sDS + (kk >> 2) * kTileR + (kk & 3) * 32, 16, 1024),
                      make_smem_desc(sK + j * kTileR + kk * 2048, 8192, 1024), id_q, (accumulate || kk > 0) ? 1u : 0u);
      };
      bool ok = true;
      uint32_t c = 0;  // blocks so far
      int k = 0;
      for (int u = blockIdx.x; u < n_units; u += gridDim.x, ++k, c += 3) {
        const uint32_t kp = (uint32_t)k & 1u;
        ok = ok && mbar_wait(smem_u32(&bar_ldq0), kp, status, DEV_MBAR_TIMEOUT_MMA);
        ok = ok && mbar_wait(smem_u32(&bar_ldk0), kp, status, DEV_MBAR_TIMEOUT_MMA);
        if (c > 0) {
          ok = ok && mbar_wait(smem_u32(&bar_sfree), (c - 1) & 1u, status, DEV_MBAR_TIMEOUT_MMA);
          ok = ok && mbar_wait(smem_u32(&bar_dpfree), (c - 1) & 1u, status, DEV_MBAR_TIMEOUT_MMA);
        }
        tc_fence_after();
        scores(0, 0);
        ok = ok && mbar_wait(smem_u32(&bar_ldv0), kp, status, DEV_MBAR_TIMEOUT_MMA);
        tc_fence_after();
        dprobs(0, 0);
        // A block's S is reissued for the next block as soon as the row threads hold the current one in
        // registers, its dP likewise: the waits below come in the order the row threads arrive.
        ok = ok && mbar_wait(smem_u32(&bar_ldq1), kp, status, DEV_MBAR_TIMEOUT_MMA);
        ok = ok && mbar_wait(smem_u32(&bar_sfree), c & 1u, status, DEV_MBAR_TIMEOUT_MMA);
        tc_fence_after();
        scores(1, 0);
        // block 0: (q0, k0)
        if (k > 0) ok = ok && mbar_wait(smem_u32(&bar_findr), (uint32_t)(k - 1) & 1u, status, DEV_MBAR_TIMEOUT_MMA);
        ok = ok && mbar_wait(smem_u32(&bar_p1), c & 1u, status, DEV_MBAR_TIMEOUT_MMA);
        tc_fence_after();
        transposed(tDV, sP, sDO, false);
        tc_commit(smem_u32(&bar_pfree));
        ok = ok && mbar_wait(smem_u32(&bar_dpfree), c & 1u, status, DEV_MBAR_TIMEOUT_MMA);
        tc_fence_after();
        dprobs(1, 0);
        ok = ok && mbar_wait(smem_u32(&bar_p2), c & 1u, status, DEV_MBAR_TIMEOUT_MMA);
        tc_fence_after();
        transposed(tDK, sDS, sQ, false);
        dq(tDQ0, 0, false);
        tc_commit(smem_u32(&bar_dsfree));
        tc_commit(smem_u32(&bar_acc0));  // Q0 and dO0 are dead
        // block 1: (q1, k0)
        ok = ok && mbar_wait(smem_u32(&bar_ldkv1), kp, status, DEV_MBAR_TIMEOUT_MMA);
        ok = ok && mbar_wait(smem_u32(&bar_sfree), (c + 1) & 1u, status, DEV_MBAR_TIMEOUT_MMA);
        tc_fence_after();
        scores(1, 1);
        ok = ok && mbar_wait(smem_u32(&bar_p1), (c + 1) & 1u, status, DEV_MBAR_TIMEOUT_MMA);
        tc_fence_after();
        transposed(tDV, sP, sDO + kTileR, true);
        tc_commit(smem_u32(&bar_pfree));
        ok = ok && mbar_wait(smem_u32(&bar_dpfree), (c + 1) & 1u, status, DEV_MBAR_TIMEOUT_MMA);
        tc_fence_after();
        dprobs(1, 1);
        ok = ok && mbar_wait(smem_u32(&bar_p2), (c + 1) & 1u, status, DEV_MBAR_TIMEOUT_MMA);
        tc_fence_after();
        transposed(tDK, sDS, sQ + kTileR, true);
        dq(tDQ1, 0, false);
        tc_commit(smem_u32(&bar_dsfree));
        tc_commit(smem_u32(&bar_acc1));  // dK_0, dV_0, dQ_0 are final; Q0 / K0 / V0 / dO0 are dead
        // block 2: (q1, k1), into dK / dV once the row threads have drained the first key tile's
        ok = ok && mbar_wait(smem_u32(&bar_p1), (c + 2) & 1u, status, DEV_MBAR_TIMEOUT_MMA);
        ok = ok && mbar_wait(smem_u32(&bar_kvdr), kp, status, DEV_MBAR_TIMEOUT_MMA);
        tc_fence_after();
        transposed(tDV, sP, sDO + kTileR, false);
        tc_commit(smem_u32(&bar_pfree));
        ok = ok && mbar_wait(smem_u32(&bar_p2), (c + 2) & 1u, status, DEV_MBAR_TIMEOUT_MMA);
        tc_fence_after();
        transposed(tDK, sDS, sQ + kTileR, false);
        dq(tDQ1, 1, true);
        tc_commit(smem_u32(&bar_dsfree));
        tc_commit(smem_u32(&bar_acc2));
      }
    }
  } else {
    // ------------------------------ two threads per query row ------------------------------
    const int lane_group = warp & 3;
    const int half = (warp - 2) >> 2;                // which 64 of a block's 128 keys / which 32 of 64 output columns
    const int r = lane_group * 32 + lane;
    const uint32_t lane_base = (uint32_t)(lane_group * 32) << 16;
    const float sl2 = p.scale * kLog2e;
    bool ok = true;
    uint32_t c = 0;
    int k = 0;
    // delta of query tile 1 = rowsum(dO (O + O_lo)) from the dO tile and the O / O_lo tiles parked in the two
    // spare tiles.  (Tile 0 needs neither: its only block holds the whole row, so delta = rowsum(P dP) there.)
    auto delta_tile1 = [&]() -> float {
      float part = 0.f, part_lo = 0.f;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int so = r * 128 + (((half * 4 + q) ^ (r & 7)) << 4);
        const uint4 a = *reinterpret_cast<const uint4*>(ptr(sDO + kTileR) + so);
        const uint4 o = *reinterpret_cast<const uint4*>(ptr(sT) + so);
        const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 af = __bfloat1622float2(a2[e]), of = __bfloat1622float2(o2[e]);
          part += af.x * of.x + af.y * of.y;
        }
        if (p.o_lo != nullptr) {
          const uint4 d = *reinterpret_cast<const uint4*>(ptr(sT + kTileR) + so);
          const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&d);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 af = __bfloat1622float2(a2[e]), df = __bfloat1622float2(d2[e]);
            part_lo += af.x * df.x + af.y * df.y;
          }
        }
      }
      return part + part_lo;
    };
    auto load_lse = [&](int u, float* l2) {
      const int b = u / H, h = u - b * H;
      const size_t stat0 = ((size_t)b * H + h) * T;
      l2[0] = p.lse[stat0 + r];  // (scaled where it is used: the loads stay in flight until then)
      l2[1] = p.lse[stat0 + 128 + r];
    };
    float lse_n[2] = {0.f, 0.f};
    if ((int)blockIdx.x < n_units) load_lse(blockIdx.x, lse_n);
    for (int u = blockIdx.x; u < n_units; u += gridDim.x, ++k, c += 3) {
      const int b = u / H, h = u - b * H;
      const uint32_t kp = (uint32_t)k & 1u;
      const size_t stat0 = ((size_t)b * H + h) * T;
      float lse_r[2], del_r[2] = {0.f, 0.f};
      lse_r[0] = lse_n[0] * kLog2e;
      lse_r[1] = lse_n[1] * kLog2e;

      // One 128 x 128 block, this thread's query row and 64 keys, in two parts: probabilities to registers ...
      auto probs = [&](int i, bool diag, uint32_t cc, float* sv) {
        ok = ok && mbar_wait(smem_u32(&bar_s), cc & 1u, status, DEV_MBAR_TIMEOUT_EPILOGUE);
        tc_fence_after();
        tmem_ld_32x32(tS + lane_base + (uint32_t)(half * 64), sv);
        tmem_ld_32x32(tS + lane_base + (uint32_t)(half * 64 + 32), sv + 32);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_sfree));  // the next block's S may be issued
        const float ls = lse_r[i];
#pragma unroll
        for (int e = 0; e < 64; ++e) {
          float pr = fast_ex2(fmaf(sv[e], sl2, -ls));
          if (diag && half * 64 + e > r) pr = 0.f;  // key after query
          sv[e] = pr;
        }
      };
      // ... then P and dS = P (dP - delta) to their operand tiles
      auto finish = [&](int i, uint32_t cc, const float* sv, bool own_delta) {
        if (cc > 0) ok = ok && mbar_wait(smem_u32(&bar_pfree), (cc - 1) & 1u, status, DEV_MBAR_TIMEOUT_EPILOGUE);
        uint8_t* pP = ptr(sP + half * kTileR);
#pragma unroll
        for (int q = 0; q < 8; ++q) st_chunk(pP, r, q, sv + 8 * q);
        tc_fence_before();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_p1));
        // dS without the score scale: the accumulators fed by dS are scaled once when they are drained.
        ok = ok && mbar_wait(smem_u32(&bar_dp), cc & 1u, status, DEV_MBAR_TIMEOUT_EPILOGUE);
        tc_fence_after();
        if (cc > 0) ok = ok && mbar_wait(smem_u32(&bar_dsfree), (cc - 1) & 1u, status, DEV_MBAR_TIMEOUT_EPILOGUE);
        uint8_t* pD = ptr(sDS + half * kTileR);
        if (own_delta) {
          // The block holds the whole row: delta = rowsum(P dP), its two halves meeting through shared memory.
          float dv[64];
          tmem_ld_32x32(tDP + lane_base + (uint32_t)(half * 64), dv);
          tmem_ld_32x32(tDP + lane_base + (uint32_t)(half * 64 + 32), dv + 32);
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bar_dpfree));
          float ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int e = 0; e < 64; ++e) ps[e & 3] = fmaf(sv[e], dv[e], ps[e & 3]);
          float dl = (ps[0] + ps[1]) + (ps[2] + ps[3]);
          xd[0][half][r] = dl;
          named_bar_sync(1, A5_COMPUTE);
          dl += xd[0][half ^ 1][r];
          del_r[i] = dl;
#pragma unroll
          for (int e = 0; e < 64; ++e) dv[e] = sv[e] * (dv[e] - dl);
#pragma unroll
          for (int q = 0; q < 8; ++q) st_chunk(pD, r, q, dv + 8 * q);
        } else {
        const float dl = del_r[i];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          float dv[32];
          tmem_ld_32x32(tDP + lane_base + (uint32_t)(half * 64 + hh * 32), dv);
          tmem_ld_wait();
          if (hh == 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_dpfree));  // the next block's dP may be issued
          }
#pragma unroll
          for (int e = 0; e < 32; ++e) dv[e] = sv[hh * 32 + e] * (dv[e] - dl);
#pragma unroll
          for (int q = 0; q < 4; ++q) st_chunk(pD, r, hh * 4 + q, dv + 8 * q);
        }
        }
        tc_fence_before();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_p2));
      };
      // dV_t, dK_t, dQ_t of 128-row tile t: tensor memory -> bf16 in staging tiles (dQ always in the first
      // spare tile, so that Q_t is free at once; dK_0 in the second spare tile, the rest in their own dead
      // operand tiles); the producer thread sends them out and refills the tiles.
      auto drain = [&](int t, uint32_t tdq, uint64_t* drained, uint64_t* staged) {
        // chunk q of this thread's 16 (cos, sin) pairs: consecutive rows are consecutive float4s
        // chunk q of this thread's 16 (cos, sin) pairs: consecutive rows are consecutive float4s
        const float4* c4 = p.rope + (size_t)(half * 4) * T + (t * 128 + r);
        const uint32_t col = (uint32_t)(half * 32);
        // one accumulator at a time (dV as it is; dK and dQ scaled and rotated back)
#pragma unroll
        for (int which = 0; which < 3; ++which) {
          float a[32];
          tmem_ld_32x32((which == 0 ? tDV : which == 1 ? tDK : tdq) + lane_base + col, a);
          tmem_ld_wait();
          if (which == 2) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(drained));
          }
          if (which > 0) {
#pragma unroll
            for (int e = 0; e < 32; ++e) a[e] *= p.scale;
            if (rope) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float4 cv = __ldg(c4 + q * T), sv4 = __ldg(c4 + (8 + q) * T);  // (L1 hits for dQ after dK)
                const float cs[4] = {cv.x, cv.y, cv.z, cv.w}, sn[4] = {sv4.x, sv4.y, sv4.z, sv4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float ev = a[8 * q + 2 * e], ov = a[8 * q + 2 * e + 1];
                  a[8 * q + 2 * e] = ev * cs[e] + ov * sn[e];
                  a[8 * q + 2 * e + 1] = ov * cs[e] - ev * sn[e];
                }
              }
            }
          }
          uint8_t* dst = ptr(which == 0 ? sV + t * kTileR : which == 1 ? (t == 0 ? sT + kTileR : sK + kTileR) : sT);
#pragma unroll
          for (int q = 0; q < 4; ++q) st_chunk(dst, r, half * 4 + q, a + 8 * q);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(staged));
      };

      // The rotation chunks a drain reads are asked into L1 one phase ahead (no registers held meanwhile).
      auto prefetch_rope = [&](int t) {
        if (!rope) return;
        const float4* c4 = p.rope + (size_t)(half * 4) * T + (t * 128 + r);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          asm volatile("prefetch.global.L1 [%0];" ::"l"(c4 + q * T));
          asm volatile("prefetch.global.L1 [%0];" ::"l"(c4 + (8 + q) * T));
        }
      };
      float sv[64];
      probs(0, true, c, sv);
      finish(0, c, sv, true);
      if (half == 0) p.delta[stat0 + r] = del_r[0];
      probs(1, false, c + 1, sv);
      // delta of the second query tile, as late as it can be (its O tiles were the last loads to go out)
      ok = ok && mbar_wait(smem_u32(&bar_ldq1), kp, status, DEV_MBAR_TIMEOUT_EPILOGUE);
      ok = ok && mbar_wait(smem_u32(&bar_ldo), kp, status, DEV_MBAR_TIMEOUT_EPILOGUE);
      del_r[1] = delta_tile1();
      xd[1][half][r] = del_r[1];
      named_bar_sync(1, A5_COMPUTE);  // also: the spare tiles have been read before the first drain writes them
      del_r[1] += xd[1][half ^ 1][r];
      if (half == 0) p.delta[stat0 + 128 + r] = del_r[1];
      finish(1, c + 1, sv, false);
      // The third block's probabilities are formed while the second block's MMAs retire.
      prefetch_rope(0);
      probs(1, true, c + 2, sv);
      ok = ok && mbar_wait(smem_u32(&bar_acc1), kp, status, DEV_MBAR_TIMEOUT_EPILOGUE);
      tc_fence_after();
      // the spare tiles: the previous head's last stores have read them (store groups complete in order)
      if (k > 0) ok = ok && mbar_wait(smem_u32(&bar_stfree), 1u, status, DEV_MBAR_TIMEOUT_EPILOGUE);
      drain(0, tDQ0, &bar_kvdr, &bar_stage0);
      prefetch_rope(1);
      finish(1, c + 2, sv, false);
      if (u + (int)gridDim.x < n_units) load_lse(u + gridDim.x, lse_n);
      ok = ok && mbar_wait(smem_u32(&bar_acc2), kp, status, DEV_MBAR_TIMEOUT_EPILOGUE);
      tc_fence_after();
      ok = ok && mbar_wait(smem_u32(&bar_stfree), 0u, status, DEV_MBAR_TIMEOUT_EPILOGUE);  // this head's first stores
      drain(1, tDQ1, &bar_findr, &bar_stage1);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

constexpr size_t kBwdHeadTiles = 14 * kTileR;  // plus what aligning the first tile to 1024 bytes takes

// ------------------------------------------------------------------------------------------------
// Split-precision backward for q|k|v kept in fp32 (the reference architecture).  The reference's
// backward recomputes its probabilities from UNSCALED scores (ane/train_full.go:268-269), whose
// magnitude (up to ~1.4 * head_dim) turns the bf16 rounding of q and k into percent-level errors of
// P.  Here q and k arrive as two bf16 tensors each (hi = bf16(x), lo = bf16(x - hi)) and the score
// product is issued as three accumulating MMAs, q_hi k_hi + q_hi k_lo + q_lo k_hi, which restores
// ~16 mantissa bits; every other product (dO V^T, P^T dO, dS^T Q, dS K) is not amplified and uses
// the hi parts alone.  Because the backward softmax has its own scale, its row statistics come from
// a statistics pass (MODE A5_STATS: lse and delta = sum_j P dP, accumulated online), not from the
// forward.  Gradients leave as bf16 without any rotation (the caller's QK-norm / rotation backward
// follows in fp32).  One CTA per SM (112-128 KB of shared memory).
// ------------------------------------------------------------------------------------------------
enum : int { A5_STATS = 3 };

struct Attn5SplitParams {
  float* lse;      // [B, H, T] log-sum-exp of scale * scores (written by STATS, read by the others)
  float* delta;    // [B, H, T] sum_j P dP                      (written by STATS, read by the others)
  int T, H, KV;
  float scale;
  int* status;
};

template <int MODE>
__global__ void __launch_bounds__(A5_THREADS, 1)
attn5_bwd_split_kernel(const __grid_constant__ CUtensorMap tm_hi_r, const __grid_constant__ CUtensorMap tm_hi_x,
                       const __grid_constant__ CUtensorMap tm_lo_r, const __grid_constant__ CUtensorMap tm_lo_x,
                       const __grid_constant__ CUtensorMap tm_do_r, const __grid_constant__ CUtensorMap tm_do_x,
                       const __grid_constant__ CUtensorMap tm_dqkv, Attn5SplitParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[2];
  __shared__ __align__(8) uint64_t bar_empty[2];
  __shared__ __align__(8) uint64_t bar_r, bar_s1, bar_s2, bar_p1, bar_p2, bar_acc;
  __shared__ uint32_t tmem_slot;
  __shared__ __align__(16) float ld_s[2][128];  // dK/dV: per streamed query [0,64) lse*log2e, [64,128) delta
  __shared__ float xs[3][2][128];               // STATS: (m, l, acc) per column half and row

  int* status = p.status;
  if (status != nullptr && *reinterpret_cast<volatile int*>(status) != DEV_OK) return;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sR1h = smem_base, sR1l = sR1h + kTileR, sR2 = sR1l + kTileR;  // resident: hi, lo, second operand
  const uint32_t sX = sR2 + kTileR;                                           // [2 stages][X1 hi | X1 lo | X2]
  const uint32_t sDS = sX + 2 * 3 * kTileX;                                   // dS' operand tile
  const uint32_t sP = sDS + kTileR;                                           // P' operand tile (dK/dV only)
  uint8_t* pDS = smem_al + (sDS - smem_base);
  uint8_t* pP = smem_al + (sP - smem_base);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int T = p.T, H = p.H, KV = p.KV, group = H / KV;
  const int nT = T / 128;
  int rt, b, h = 0, kvh, n_per = 1, n_it;
  if constexpr (MODE == A5_DKV) {
    rt = blockIdx.y;
    b = blockIdx.x / KV;
    kvh = blockIdx.x - b * KV;
    n_per = T / 64 - 2 * rt;
    n_it = group * n_per;
  } else {
    rt = nT - 1 - blockIdx.y;
    b = blockIdx.x / H;
    h = blockIdx.x - b * H;
    kvh = h / group;
    n_it = 2 * rt + 2;
  }
  const int row0 = b * T;

  auto issue_x = [&](int it) {
    const int s = it & 1;
    const uint32_t full = smem_u32(&bar_full[s]);
    const uint32_t x1h = sX + s * 3 * kTileX, x1l = x1h + kTileX, x2 = x1l + kTileX;
    mbar_expect_tx(full, 3 * kTileX);
    if constexpr (MODE == A5_DKV) {
      const int g = it / n_per;
      const int qh = 2 * rt + (it - g * n_per);
      const int hq = kvh * group + g;
      tma_load_2d(x1h, &tm_hi_x, full, hq * 64, row0 + qh * 64);
      tma_load_2d(x1l, &tm_lo_x, full, hq * 64, row0 + qh * 64);
      tma_load_2d(x2, &tm_do_x, full, hq * 64, row0 + qh * 64);
    } else {
      tma_load_2d(x1h, &tm_hi_x, full, (H + kvh) * 64, row0 + it * 64);
      tma_load_2d(x1l, &tm_lo_x, full, (H + kvh) * 64, row0 + it * 64);
      tma_load_2d(x2, &tm_hi_x, full, (H + KV + kvh) * 64, row0 + it * 64);
    }
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    mbar_init(smem_u32(&bar_r), 1);
    mbar_init(smem_u32(&bar_s1), 1);
    mbar_init(smem_u32(&bar_s2), 1);
    mbar_init(smem_u32(&bar_p1), 8);
    mbar_init(smem_u32(&bar_p2), 8);
    mbar_init(smem_u32(&bar_acc), 1);
    fence_mbar_init();
    pdl_wait();
    const uint32_t rbar = smem_u32(&bar_r);
    mbar_expect_tx(rbar, 3 * kTileR);
    if constexpr (MODE == A5_DKV) {
      tma_load_2d(sR1h, &tm_hi_r, rbar, (H + kvh) * 64, row0 + rt * 128);
      tma_load_2d(sR1l, &tm_lo_r, rbar, (H + kvh) * 64, row0 + rt * 128);
      tma_load_2d(sR2, &tm_hi_r, rbar, (H + KV + kvh) * 64, row0 + rt * 128);
    } else {
      tma_load_2d(sR1h, &tm_hi_r, rbar, h * 64, row0 + rt * 128);
      tma_load_2d(sR1l, &tm_lo_r, rbar, h * 64, row0 + rt * 128);
      tma_load_2d(sR2, &tm_do_r, rbar, h * 64, row0 + rt * 128);
    }
    issue_x(0);
    issue_x(1);  // n_it >= 2 always
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), 256);
    tmem_relinquish();
  }
  pdl_trigger();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  const uint32_t tmem_base = tmem_slot;
  const uint32_t tS = tmem_base, tDP = tmem_base + 64, tA1 = tmem_base + 128, tA2 = tmem_base + 192;

  if (warp == 0) {
    if (lane == 0) {
      for (int it = 2; it < n_it; ++it) {
        const int s = it & 1;
        const uint32_t ph = (uint32_t)(it >> 1) & 1u;
        if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, status, DEV_MBAR_TIMEOUT_PRODUCER)) break;
        issue_x(it);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_kk = a5_idesc(false, false);
      constexpr uint32_t idesc_kn = a5_idesc(false, true);
      bool ok = mbar_wait(smem_u32(&bar_r), 0, status, DEV_MBAR_TIMEOUT_MMA);
      for (int it = 0; ok && it < n_it; ++it) {
        const int s = it & 1;
        const uint32_t ph = (uint32_t)(it >> 1) & 1u;
        if (!mbar_wait(smem_u32(&bar_full[s]), ph, status, DEV_MBAR_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t x1h = sX + s * 3 * kTileX, x1l = x1h + kTileX, x2 = x1l + kTileX;
        // S' = R1 X1^T at split precision: hi hi + lo hi + hi lo
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tc_mma_bf16(tS, make_smem_desc(sR1h + k * 32, 16, 1024), make_smem_desc(x1h + k * 32, 16, 1024), idesc_kk,
                      k > 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tc_mma_bf16(tS, make_smem_desc(sR1l + k * 32, 16, 1024), make_smem_desc(x1h + k * 32, 16, 1024), idesc_kk, 1u);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tc_mma_bf16(tS, make_smem_desc(sR1h + k * 32, 16, 1024), make_smem_desc(x1l + k * 32, 16, 1024), idesc_kk, 1u);
        tc_commit(smem_u32(&bar_s1));
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tc_mma_bf16(tDP, make_smem_desc(sR2 + k * 32, 16, 1024), make_smem_desc(x2 + k * 32, 16, 1024), idesc_kk,
                      k > 0 ? 1u : 0u);
        tc_commit(smem_u32(&bar_s2));
        const uint32_t par = (uint32_t)it & 1u;
        if constexpr (MODE == A5_DKV) {
          if (!mbar_wait(smem_u32(&bar_p1), par, status, DEV_MBAR_TIMEOUT_MMA)) break;
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < 4; ++k)  // dV += P^T dO
            tc_mma_bf16(tA1, make_smem_desc(sP + k * 32, 16, 1024), make_smem_desc(x2 + k * 2048, 8192, 1024),
                        idesc_kn, (it > 0 || k > 0) ? 1u : 0u);
        }
        if (!mbar_wait(smem_u32(&bar_p2), par, status, DEV_MBAR_TIMEOUT_MMA)) break;
        tc_fence_after();
        if constexpr (MODE != A5_STATS) {
#pragma unroll
          for (int k = 0; k < 4; ++k)  // dK += dS^T Q_hi   |   dQ += dS K_hi
            tc_mma_bf16(MODE == A5_DKV ? tA2 : tA1, make_smem_desc(sDS + k * 32, 16, 1024),
                        make_smem_desc(x1h + k * 2048, 8192, 1024), idesc_kn, (it > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(smem_u32(&bar_empty[s]));
        if (it == n_it - 1) tc_commit(smem_u32(&bar_acc));
      }
    }
  } else {
    const int lane_group = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = lane_group * 32 + lane;
    const int ct = threadIdx.x - 64;
    const uint32_t lane_off = ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(half * 32);
    const float sl2 = p.scale * kLog2e;
    const int rpos = rt * 128 + r;
    float lse_r = 0.f, del_r = 0.f;
    if constexpr (MODE == A5_DQ) {
      lse_r = p.lse[((size_t)b * H + h) * T + rpos] * kLog2e;
      del_r = p.delta[((size_t)b * H + h) * T + rpos];
    }
    float m_run = -INFINITY, l_run = 0.f, a_run = 0.f;  // STATS: online max / sum-exp / sum exp*dP (log2 domain)
    bool ok = true;
    for (int it = 0; ok && it < n_it; ++it) {
      const int s = it & 1;
      int xpos0;
      if constexpr (MODE == A5_DKV) {
        const int g = it / n_per;
        const int qh = 2 * rt + (it - g * n_per);
        const int hq = kvh * group + g;
        xpos0 = qh * 64;
        const size_t base = ((size_t)b * H + hq) * T + xpos0;
        if (ct < 128) ld_s[s][ct] = (ct < 64) ? p.lse[base + ct] * kLog2e : p.delta[base + ct - 64];
        named_bar_sync(1, A5_COMPUTE);
      } else {
        xpos0 = it * 64;
      }
      const uint32_t par = (uint32_t)it & 1u;
      if (!mbar_wait(smem_u32(&bar_s1), par, status, DEV_MBAR_TIMEOUT_EPILOGUE)) {
        ok = false;
        break;
      }
      tc_fence_after();
      float sv[32];
      tmem_ld_32x32(tS + lane_off, sv);
      tmem_ld_wait();
      bool diag;
      if constexpr (MODE == A5_DKV) diag = xpos0 < rt * 128 + 127;
      else diag = xpos0 + 63 > rt * 128;
      const int c0 = xpos0 + half * 32;
      float m_new = m_run;
      if constexpr (MODE == A5_DKV) {
        const float4* l4 = reinterpret_cast<const float4*>(&ld_s[s][half * 32]);
#pragma unroll
        for (int e4 = 0; e4 < 8; ++e4) {
          const float4 l = l4[e4];
          const float lv[4] = {l.x, l.y, l.z, l.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int e = e4 * 4 + k;
            float pr = fast_ex2(sv[e] * sl2 - lv[k]);
            if (diag && rpos > c0 + e) pr = 0.f;
            sv[e] = pr;
          }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) st_chunk(pP, r, half * 4 + q, sv + 8 * q);
        tc_fence_before();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_p1));
      } else if constexpr (MODE == A5_DQ) {
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          float pr = fast_ex2(sv[e] * sl2 - lse_r);
          if (diag && c0 + e > rpos) pr = 0.f;
          sv[e] = pr;
        }
      } else {  // STATS: scaled scores in the log2 domain, running maximum
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          sv[e] = (diag && c0 + e > rpos) ? -INFINITY : sv[e] * sl2;
          m_new = fmaxf(m_new, sv[e]);
        }
      }
      if (!mbar_wait(smem_u32(&bar_s2), par, status, DEV_MBAR_TIMEOUT_EPILOGUE)) {
        ok = false;
        break;
      }
      tc_fence_after();
      float dv[32];
      tmem_ld_32x32(tDP + lane_off, dv);
      tmem_ld_wait();
      if constexpr (MODE == A5_STATS) {
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float corr = fast_ex2(m_run - m_use);
        float ls = 0.f, as = 0.f;
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const float pr = fast_ex2(sv[e] - m_use);
          ls += pr;
          as += pr * dv[e];
        }
        l_run = l_run * corr + ls;
        a_run = a_run * corr + as;
        m_run = m_new;
      } else {
        if constexpr (MODE == A5_DKV) {
          const float4* d4 = reinterpret_cast<const float4*>(&ld_s[s][64 + half * 32]);
#pragma unroll
          for (int e4 = 0; e4 < 8; ++e4) {
            const float4 d = d4[e4];
            dv[e4 * 4 + 0] = sv[e4 * 4 + 0] * (dv[e4 * 4 + 0] - d.x);
            dv[e4 * 4 + 1] = sv[e4 * 4 + 1] * (dv[e4 * 4 + 1] - d.y);
            dv[e4 * 4 + 2] = sv[e4 * 4 + 2] * (dv[e4 * 4 + 2] - d.z);
            dv[e4 * 4 + 3] = sv[e4 * 4 + 3] * (dv[e4 * 4 + 3] - d.w);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) dv[e] = sv[e] * (dv[e] - del_r);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) st_chunk(pDS, r, half * 4 + q, dv + 8 * q);
        fence_proxy_async_smem();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_p2));
    }
    ok = ok && mbar_wait(smem_u32(&bar_acc), 0, status, DEV_MBAR_TIMEOUT_EPILOGUE);
    if constexpr (MODE == A5_STATS) {
      // merge the two column halves of every row: (m, l, acc) -> lse (natural log), delta = acc / l
      xs[0][half][r] = m_run;
      xs[1][half][r] = l_run;
      xs[2][half][r] = a_run;
      named_bar_sync(1, A5_COMPUTE);
      if (ok && half == 0) {
        const float m2 = xs[0][1][r], l2 = xs[1][1][r], a2 = xs[2][1][r];
        const float m = fmaxf(m_run, m2);  // finite: key 0 is visible to every query
        const float c1 = fast_ex2(m_run - m), c2 = fast_ex2(m2 - m);
        const float l = l_run * c1 + l2 * c2;
        const float a = a_run * c1 + a2 * c2;
        const size_t o = ((size_t)b * H + h) * T + rpos;
        p.lse[o] = (m + log2f(l)) / kLog2e;
        p.delta[o] = a / l;
      }
    } else {
      if (ok) {
        tc_fence_after();
        float a[32];
        tmem_ld_32x32(tA1 + lane_off, a);
        tmem_ld_wait();
        if constexpr (MODE == A5_DQ) {
#pragma unroll
          for (int e = 0; e < 32; ++e) a[e] *= p.scale;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) st_chunk(MODE == A5_DKV ? pP : pDS, r, half * 4 + q, a + 8 * q);  // dV | dQ
        if constexpr (MODE == A5_DKV) {
          tmem_ld_32x32(tA2 + lane_off, a);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) a[e] *= p.scale;
#pragma unroll
          for (int q = 0; q < 4; ++q) st_chunk(pDS, r, half * 4 + q, a + 8 * q);  // dK
        }
        fence_proxy_async_smem();
      }
      named_bar_sync(1, A5_COMPUTE);
      if (ok && ct == 0) {
        if constexpr (MODE == A5_DKV) {
          tma_store_2d(&tm_dqkv, sP, (H + KV + kvh) * 64, row0 + rt * 128);
          tma_store_2d(&tm_dqkv, sDS, (H + kvh) * 64, row0 + rt * 128);
        } else {
          tma_store_2d(&tm_dqkv, sDS, h * 64, row0 + rt * 128);
        }
        tma_store_commit();
        tma_store_wait_read<0>();
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

constexpr size_t kSplitSmem = 3 * kTileR + 6 * kTileX + 2 * kTileR + 1024;

constexpr size_t kDkvSmem5 = 2 * kTileR + 4 * kTileX + 2 * kTileR + 1024;
constexpr size_t kDqSmem5 = 2 * kTileR + 4 * kTileX + 2 * kTileR + 1024;  // dS' tile + the O_lo tile for delta

// Persistent grids (two CTAs per SM walking a unit list) unless ANE_B200_ATTN_PERSIST=0 asks for one CTA per unit.
bool attn_persistent() {
  static const bool on = [] {
    const char* e = getenv("ANE_B200_ATTN_PERSIST");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}

// Sequences of 256 without grouped heads take the one-CTA-per-head backward unless ANE_B200_ATTN_BWD_HEAD=0.
bool attn_bwd_whole_head() {
  static const bool on = [] {
    const char* e = getenv("ANE_B200_ATTN_BWD_HEAD");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}

// Dynamic shared memory for the one-CTA-per-head backward: everything a block may have, less the kernel's
// static part (0 = the layout does not fit and the two-kernel form runs instead).
size_t g_bwd_head_smem = 0;
void setup_bwd_head_smem() {
  cudaFuncAttributes fa;
  int dev = 0, optin = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaFuncGetAttributes(&fa, attn5_bwd_head_kernel) != cudaSuccess ||
      cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess)
    return;
  const size_t stat = fa.sharedSizeBytes, pad = (1024 - stat % 1024) % 1024;
  if ((size_t)optin < stat + pad + kBwdHeadTiles) return;
  const size_t dyn = (size_t)optin - stat;
  if (cudaFuncSetAttribute(attn5_bwd_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn) != cudaSuccess) {
    cudaGetLastError();
    return;
  }
  g_bwd_head_smem = dyn;
}

bool g_attr5_done = false;
bool ensure_attrs5() {
  if (g_attr5_done) return true;
  setup_bwd_head_smem();
  if (cudaFuncSetAttribute(attn5_bwd_kernel<A5_DKV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDkvSmem5) !=
          cudaSuccess ||
      cudaFuncSetAttribute(attn5_bwd_kernel<A5_DQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDqSmem5) !=
          cudaSuccess ||
      cudaFuncSetAttribute(attn5_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFwdSmem5) != cudaSuccess ||
      cudaFuncSetAttribute(attn5_fwd_persist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFwdPersistSmem) !=
          cudaSuccess ||
      cudaFuncSetAttribute(attn5_bwd_split_kernel<A5_STATS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)kSplitSmem) != cudaSuccess ||
      cudaFuncSetAttribute(attn5_bwd_split_kernel<A5_DQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSplitSmem) !=
          cudaSuccess ||
      cudaFuncSetAttribute(attn5_bwd_split_kernel<A5_DKV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSplitSmem) !=
          cudaSuccess)
    return false;
  g_attr5_done = true;
  return true;
}

}  // namespace

namespace {
__global__ void rope_chunk_tables_kernel(const float* __restrict__ cosb, const float* __restrict__ sinb,
                                         float4* __restrict__ out, int seq) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;  // (table, chunk, position)
  if (i >= 16 * seq) return;
  const int pos = i % seq, chunk = (i / seq) & 7;
  const float* src = (i / seq >= 8 ? sinb : cosb) + (size_t)pos * 32 + chunk * 4;
  out[i] = make_float4(src[0], src[1], src[2], src[3]);
}
}  // namespace

// The [seq, 32] cos / sin tables regrouped for the one-CTA-per-head backward, whose threads own one row each:
// out[(table * 8 + chunk) * seq + pos] = the four values pos * 32 + chunk * 4 .. + 3 of cos (table 0) or sin
// (table 1), so a warp's 32 rows read 512 consecutive bytes.  `out` holds 64 * seq floats.
void attention_rope_chunk_tables(const float* cosb, const float* sinb, float* out, int seq, cudaStream_t s) {
  rope_chunk_tables_kernel<<<(16 * seq + 255) / 256, 256, 0, s>>>(cosb, sinb, reinterpret_cast<float4*>(out), seq);
}

bool attention_tcgen05_supported(int hd, int seq) { return hd == 64 && seq > 0 && seq % 128 == 0; }

int attention_forward_tcgen05(const bf16* qkv, bf16* out, bf16* out_lo, float* lse, int B, int seq, int H, int KV,
                              float scale, int* d_status, cudaStream_t s) {
  if (B <= 0) return 0;
  if (!attention_tcgen05_supported(64, seq) || H % KV != 0 || !ensure_attrs5()) return -1;
  const uint64_t M = (uint64_t)B * seq;
  const uint64_t ld = (uint64_t)(H + 2 * KV) * 64;
  CUtensorMap tm_qkv_r, tm_qkv_x, tm_out, tm_out_lo;
  if (!make_tmap_2d(&tm_qkv_r, qkv, ld, M, ld, 64, 128, false) || !make_tmap_2d(&tm_qkv_x, qkv, ld, M, ld, 64, 64, false) ||
      !make_tmap_2d(&tm_out, out, (uint64_t)H * 64, M, (uint64_t)H * 64, 64, 128, false) ||
      !make_tmap_2d(&tm_out_lo, out_lo ? out_lo : out, (uint64_t)H * 64, M, (uint64_t)H * 64, 64, 128, false))
    return -2;
  Attn5FwdParams p{out, lse, seq, H, KV, scale, d_status, out_lo ? 1 : 0};
  if (attn_persistent()) {
    const A5Units w{B * H * (seq / 128), B * H, H, seq / 128, 1};
    const int slots = 2 * gemm_num_sms();
    return launch_pdl(attn5_fwd_persist_kernel, dim3(w.n_units < slots ? w.n_units : slots), dim3(A5_THREADS),
                      kFwdPersistSmem, s, tm_qkv_r, tm_qkv_x, tm_out, tm_out_lo, p, w) == cudaSuccess
               ? 0
               : -4;
  }
  dim3 grid(B * H, seq / 128);
  return launch_pdl(attn5_fwd_kernel, grid, dim3(A5_THREADS), kFwdSmem5, s, tm_qkv_r, tm_qkv_x, tm_out, tm_out_lo, p) ==
                 cudaSuccess
             ? 0
             : -4;
}

int attention_backward_tcgen05(const bf16* qkv, const bf16* out, const bf16* out_lo, const bf16* d_out, const float* lse, float* delta,
                               bf16* dqkv,
                               const float* cosb, const float* sinb, const float* rope_chunks, int B, int seq, int H, int KV,
                               float scale, int* d_status, cudaStream_t s) {
  if (B <= 0) return 0;  // returns the number of kernels launched, negative on failure
  if (!attention_tcgen05_supported(64, seq) || H % KV != 0 || !ensure_attrs5()) return -1;
  const uint64_t M = (uint64_t)B * seq;
  const uint64_t ld = (uint64_t)(H + 2 * KV) * 64;
  CUtensorMap tm_qkv_r, tm_qkv_x, tm_do_r, tm_do_x, tm_o_r, tm_o_lo, tm_dqkv, tm_cos, tm_sin;
  if (!make_tmap_2d(&tm_qkv_r, qkv, ld, M, ld, 64, 128, false) || !make_tmap_2d(&tm_qkv_x, qkv, ld, M, ld, 64, 64, false) ||
      !make_tmap_2d(&tm_do_r, d_out, (uint64_t)H * 64, M, (uint64_t)H * 64, 64, 128, false) ||
      !make_tmap_2d(&tm_do_x, d_out, (uint64_t)H * 64, M, (uint64_t)H * 64, 64, 64, false) ||
      !make_tmap_2d(&tm_o_r, out, (uint64_t)H * 64, M, (uint64_t)H * 64, 64, 128, false) ||
      !make_tmap_2d(&tm_o_lo, out_lo ? out_lo : out, (uint64_t)H * 64, M, (uint64_t)H * 64, 64, 128, false) ||
      !make_tmap_2d(&tm_dqkv, dqkv, ld, M, ld, 64, 128, false))
    return -2;
  if (cosb != nullptr && sinb != nullptr) {  // [seq, 32] fp32 tables, one 128-byte row per position
    if (!make_tmap_2d(&tm_cos, cosb, 32, (uint64_t)seq, 32, 32, 128, true) ||
        !make_tmap_2d(&tm_sin, sinb, 32, (uint64_t)seq, 32, 32, 128, true))
      return -2;
  } else {
    cosb = sinb = nullptr;
    tm_cos = tm_sin = tm_dqkv;  // never dereferenced
  }
  Attn5Params p{lse, delta, dqkv, cosb, sinb, seq, H, KV, scale, d_status, out_lo ? 1 : 0};
  if (seq == 256 && H == KV && g_bwd_head_smem != 0 && (cosb == nullptr || rope_chunks != nullptr) && attn_bwd_whole_head()) {
    const int n_units = B * H, sms = gemm_num_sms();
    Attn5HeadParams hp{lse,   delta, out,      out_lo,  dqkv, cosb != nullptr ? reinterpret_cast<const float4*>(rope_chunks) : nullptr,
                       H,     scale, d_status, n_units, (uint32_t)g_bwd_head_smem};
    return launch_pdl(attn5_bwd_head_kernel, dim3(n_units < sms ? n_units : sms), dim3(A5_THREADS), g_bwd_head_smem, s, tm_qkv_r,
                      tm_do_r, tm_o_r, tm_o_lo, tm_dqkv, hp) == cudaSuccess
               ? 1
               : -4;
  }
  // dQ first: it also produces delta, which the dK/dV kernel consumes.
  dim3 gq(B * H, seq / 128);
  if (launch_pdl(attn5_bwd_kernel<A5_DQ>, gq, dim3(A5_THREADS), kDqSmem5, s, tm_qkv_r, tm_qkv_x, tm_do_r, tm_do_x, tm_o_r,
                 tm_o_lo, tm_dqkv, tm_cos, tm_sin, p) != cudaSuccess)
    return -4;
  dim3 gk(B * KV, seq / 128);
  if (launch_pdl(attn5_bwd_kernel<A5_DKV>, gk, dim3(A5_THREADS), kDkvSmem5, s, tm_qkv_r, tm_qkv_x, tm_do_r, tm_do_x, tm_o_r,
                 tm_o_lo, tm_dqkv, tm_cos, tm_sin, p) != cudaSuccess)
    return -4;
  return cudaGetLastError() == cudaSuccess ? 2 : -4;
}

int attention_backward_tcgen05_split(const bf16* qkv_hi, const bf16* qkv_lo, const bf16* d_out, float* lse, float* delta,
                                     bf16* dqkv, int B, int seq, int H, int KV, float scale, int* d_status,
                                     cudaStream_t s) {
  if (B <= 0) return 0;
  if (!attention_tcgen05_supported(64, seq) || H % KV != 0 || !ensure_attrs5()) return -1;
  const uint64_t M = (uint64_t)B * seq;
  const uint64_t ld = (uint64_t)(H + 2 * KV) * 64;
  CUtensorMap hi_r, hi_x, lo_r, lo_x, do_r, do_x, out_r;
  if (!make_tmap_2d(&hi_r, qkv_hi, ld, M, ld, 64, 128, false) || !make_tmap_2d(&hi_x, qkv_hi, ld, M, ld, 64, 64, false) ||
      !make_tmap_2d(&lo_r, qkv_lo, ld, M, ld, 64, 128, false) || !make_tmap_2d(&lo_x, qkv_lo, ld, M, ld, 64, 64, false) ||
      !make_tmap_2d(&do_r, d_out, (uint64_t)H * 64, M, (uint64_t)H * 64, 64, 128, false) ||
      !make_tmap_2d(&do_x, d_out, (uint64_t)H * 64, M, (uint64_t)H * 64, 64, 64, false) ||
      !make_tmap_2d(&out_r, dqkv, ld, M, ld, 64, 128, false))
    return -2;
  Attn5SplitParams p{lse, delta, seq, H, KV, scale, d_status};
  dim3 gq(B * H, seq / 128), gk(B * KV, seq / 128);
  if (launch_pdl(attn5_bwd_split_kernel<A5_STATS>, gq, dim3(A5_THREADS), kSplitSmem, s, hi_r, hi_x, lo_r, lo_x, do_r, do_x,
                 out_r, p) != cudaSuccess ||
      launch_pdl(attn5_bwd_split_kernel<A5_DQ>, gq, dim3(A5_THREADS), kSplitSmem, s, hi_r, hi_x, lo_r, lo_x, do_r, do_x,
                 out_r, p) != cudaSuccess ||
      launch_pdl(attn5_bwd_split_kernel<A5_DKV>, gk, dim3(A5_THREADS), kSplitSmem, s, hi_r, hi_x, lo_r, lo_x, do_r, do_x,
                 out_r, p) != cudaSuccess)
    return -4;
  return 0;
}

}  // namespace ane
