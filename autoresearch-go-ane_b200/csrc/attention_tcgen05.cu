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

bool g_attr5_done = false;
bool ensure_attrs5() {
  if (g_attr5_done) return true;
  if (cudaFuncSetAttribute(attn5_bwd_kernel<A5_DKV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDkvSmem5) !=
          cudaSuccess ||
      cudaFuncSetAttribute(attn5_bwd_kernel<A5_DQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDqSmem5) !=
          cudaSuccess ||
      cudaFuncSetAttribute(attn5_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFwdSmem5) != cudaSuccess ||
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
  dim3 grid(B * H, seq / 128);
  return launch_pdl(attn5_fwd_kernel, grid, dim3(A5_THREADS), kFwdSmem5, s, tm_qkv_r, tm_qkv_x, tm_out, tm_out_lo, p) ==
                 cudaSuccess
             ? 0
             : -4;
}

int attention_backward_tcgen05(const bf16* qkv, const bf16* out, const bf16* out_lo, const bf16* d_out, const float* lse, float* delta,
                               bf16* dqkv,
                               const float* cosb, const float* sinb, int B, int seq, int H, int KV, float scale,
                               int* d_status, cudaStream_t s) {
  if (B <= 0) return 0;
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
  // dQ first: it also produces delta, which the dK/dV kernel consumes.
  dim3 gq(B * H, seq / 128);
  if (launch_pdl(attn5_bwd_kernel<A5_DQ>, gq, dim3(A5_THREADS), kDqSmem5, s, tm_qkv_r, tm_qkv_x, tm_do_r, tm_do_x, tm_o_r,
                 tm_o_lo, tm_dqkv, tm_cos, tm_sin, p) != cudaSuccess)
    return -4;
  dim3 gk(B * KV, seq / 128);
  if (launch_pdl(attn5_bwd_kernel<A5_DKV>, gk, dim3(A5_THREADS), kDkvSmem5, s, tm_qkv_r, tm_qkv_x, tm_do_r, tm_do_x, tm_o_r,
                 tm_o_lo, tm_dqkv, tm_cos, tm_sin, p) != cudaSuccess)
    return -4;
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
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
