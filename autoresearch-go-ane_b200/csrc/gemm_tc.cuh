// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   C[M,N] (op)= A * B      bf16 operands, fp32 accumulation in tensor memory
//
// Operand storage (both row-major buffers of bf16):
//   A_MN == false : A is [M, K] (K contiguous, "K-major")
//   A_MN == true  : A is [K, M] (M contiguous, "MN-major")   -- used by dW = dY^T X
//   B_MN == false : B is [N, K] (K contiguous)               -- used by y = x W^T
//   B_MN == true  : B is [K, N] (N contiguous)               -- used by dx = dy W
//
// Pipeline: warp 0 issues TMA loads (128B-swizzled tiles) into a shared-memory
// ring; warp 1 issues tcgen05.mma (M=128, N=BN, K=16) into one of two TMEM
// accumulators; warps 2..5 drain the other accumulator with tcgen05.ld and run
// the epilogue functor. No cluster launch, no multicast.
//
// This replaces the nine cblas_sgemm call sites of the reference
// (ane/accel_darwin.go:74-207, ane/stories/gemm_accel_darwin.go:15-55) and the
// naive loops they shadow (ane/common.go:91-105, ane/train_full.go:213-259,
// ane/stories/cpu.go:303-385).
#pragma once

#include "common.cuh"

namespace ane {

static constexpr int GEMM_BM = 128;
static constexpr int GEMM_BK = 64;
static constexpr int GEMM_THREADS = 192;

template <int BN>
struct GemmCfg {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr uint32_t A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr uint32_t B_BYTES = BN * GEMM_BK * 2;
  static constexpr uint32_t SMEM_BYTES = STAGES * (A_BYTES + B_BYTES) + 1024;  // +1024: manual alignment
  static constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512)));
};

// 64-bit shared-memory matrix descriptor (sm_100 format, version field = 1).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);            // start address, bits [0,14)
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;   // leading byte offset, bits [16,30)
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;   // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                              // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                              // layout type: 128-byte swizzle
  return d;
}

// Plain store / blend epilogue:  C = alpha*acc + s1*res1 + s2*res2
template <typename OutT>
struct EpiStore {
  OutT* C;
  int ldc;
  float alpha;
  const float* res1;  // optional fp32 [M, ldres]
  const float* s1;    // optional device scalar (nullptr => 1)
  const float* res2;
  const float* s2;
  int ldres;
  struct State {};
  __device__ __forceinline__ void tile_begin(State&, int, int) const {}
  __device__ __forceinline__ void tile_end(State&, int, int, int, int) const {}
  __device__ __forceinline__ void chunk(State&, int m, int n0, float* acc, int M, int N) const {
    if (m >= M) return;
    float a1 = 0.f, a2 = 0.f;
    if (res1) a1 = s1 ? *s1 : 1.f;
    if (res2) a2 = s2 ? *s2 : 1.f;
    OutT* crow = C + (size_t)m * ldc + n0;
    const float* r1 = res1 ? res1 + (size_t)m * ldres + n0 : nullptr;
    const float* r2 = res2 ? res2 + (size_t)m * ldres + n0 : nullptr;
    if (n0 + 32 <= N) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float v[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) v[q] = alpha * acc[j + q];
        if (r1) {
          float4 t = *reinterpret_cast<const float4*>(r1 + j);
          v[0] += a1 * t.x; v[1] += a1 * t.y; v[2] += a1 * t.z; v[3] += a1 * t.w;
        }
        if (r2) {
          float4 t = *reinterpret_cast<const float4*>(r2 + j);
          v[0] += a2 * t.x; v[1] += a2 * t.y; v[2] += a2 * t.z; v[3] += a2 * t.w;
        }
        if constexpr (sizeof(OutT) == 4) {
          *reinterpret_cast<float4*>(crow + j) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
          __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0], v[1]);
          __nv_bfloat162 p1 = __floats2bfloat162_rn(v[2], v[3]);
          uint2 u;
          u.x = *reinterpret_cast<uint32_t*>(&p0);
          u.y = *reinterpret_cast<uint32_t*>(&p1);
          *reinterpret_cast<uint2*>(crow + j) = u;
        }
      }
    } else {
      for (int j = 0; j < 32 && n0 + j < N; ++j) {
        float v = alpha * acc[j];
        if (r1) v += a1 * r1[j];
        if (r2) v += a2 * r2[j];
        crow[j] = from_f<OutT>(v);
      }
    }
  }
};

// Accumulating epilogue (beta = 1): C += alpha*acc, via fp32 reductions so that
// split-K work items may target the same output tile.
struct EpiAtomicAdd {
  float* C;
  int ldc;
  float alpha;
  struct State {};
  __device__ __forceinline__ void tile_begin(State&, int, int) const {}
  __device__ __forceinline__ void tile_end(State&, int, int, int, int) const {}
  __device__ __forceinline__ void chunk(State&, int m, int n0, float* acc, int M, int N) const {
    if (m >= M) return;
    float* crow = C + (size_t)m * ldc + n0;
    int lim = N - n0 < 32 ? N - n0 : 32;
    for (int j = 0; j < lim; ++j) atomicAdd(crow + j, alpha * acc[j]);
  }
};

template <int BN, bool A_MN, bool B_MN, class Epi>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               Epi epi, int M, int N, int K, int split_k, int* status) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int BM = GEMM_BM, BK = GEMM_BK;

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[STAGES];
  __shared__ __align__(8) uint64_t bar_empty[STAGES];
  __shared__ __align__(8) uint64_t bar_tfull[2];
  __shared__ __align__(8) uint64_t bar_tempty[2];
  __shared__ uint32_t tmem_slot;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_a0 = smem_base;
  const uint32_t smem_b0 = smem_base + STAGES * Cfg::A_BYTES;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // A pipeline wait that gave up earlier in this stream poisons the status word: later launches
  // return at once instead of each running into its own time-out.
  if (status != nullptr && *reinterpret_cast<volatile int*>(status) != DEV_OK) return;

  const int tiles_m = (M + BM - 1) / BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int kblocks = (K + BK - 1) / BK;
  const int kb_per_split = (kblocks + split_k - 1) / split_k;
  const int total_work = tiles_m * tiles_n * split_k;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_tfull[b]), 1);
      mbar_init(smem_u32(&bar_tempty[b]), 4);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        const int split = w / (tiles_m * tiles_n);
        const int rem = w - split * (tiles_m * tiles_n);
        const int tn = rem / tiles_m, tm = rem - tn * tiles_m;
        const int kb0 = split * kb_per_split;
        const int kb1 = min(kb0 + kb_per_split, kblocks);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, status, DEV_MBAR_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&bar_full[stage]);
          mbar_expect_tx(full, Cfg::A_BYTES + Cfg::B_BYTES);
          const uint32_t sa = smem_a0 + stage * Cfg::A_BYTES;
          const uint32_t sb = smem_b0 + stage * Cfg::B_BYTES;
          if constexpr (!A_MN) {
            tma_load_2d(sa, &tmA, full, kb * BK, tm * BM);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * (64 * BK * 2), &tmA, full, tm * BM + j * 64, kb * BK);
          }
          if constexpr (!B_MN) {
            tma_load_2d(sb, &tmB, full, kb * BK, tn * BN);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (64 * BK * 2), &tmB, full, tn * BN + j * 64, kb * BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) |
                                 ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) |
                                 ((uint32_t)(BM >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        const int split = w / (tiles_m * tiles_n);
        const int kb0 = split * kb_per_split;
        const int kb1 = min(kb0 + kb_per_split, kblocks);
        if (kb1 <= kb0) continue;
        const int buf = local & 1;
        const uint32_t tphase = (uint32_t)(local >> 1) & 1u;
        if (!mbar_wait(smem_u32(&bar_tempty[buf]), tphase ^ 1u, status, DEV_MBAR_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(smem_u32(&bar_full[stage]), phase, status, DEV_MBAR_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_a0 + stage * Cfg::A_BYTES;
          const uint32_t sb = smem_b0 + stage * Cfg::B_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            uint64_t adesc, bdesc;
            if constexpr (!A_MN) adesc = make_smem_desc(sa + k * 32, 16, 1024);
            else                 adesc = make_smem_desc(sa + k * 2048, 64 * BK * 2, 1024);
            if constexpr (!B_MN) bdesc = make_smem_desc(sb + k * 32, 16, 1024);
            else                 bdesc = make_smem_desc(sb + k * 2048, 64 * BK * 2, 1024);
            tc_mma_bf16(tmem_d, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tc_commit(smem_u32(&bar_empty[stage]));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(smem_u32(&bar_tfull[buf]));
        ++local;
      }
    }
  } else {
    // ------------------------------ epilogue warps ------------------------------
    const int lane_group = warp & 3;  // TMEM lanes [32*lane_group, 32*lane_group+32)
    int local = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
      const int split = w / (tiles_m * tiles_n);
      const int rem = w - split * (tiles_m * tiles_n);
      const int tn = rem / tiles_m, tm = rem - tn * tiles_m;
      const int kb0 = split * kb_per_split;
      const int kb1 = min(kb0 + kb_per_split, kblocks);
      if (kb1 <= kb0) continue;
      const int buf = local & 1;
      const uint32_t tphase = (uint32_t)(local >> 1) & 1u;
      if (!mbar_wait(smem_u32(&bar_tfull[buf]), tphase, status, DEV_MBAR_TIMEOUT_EPILOGUE)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int m = tm * BM + lane_group * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(buf * BN);
      typename Epi::State st;
      epi.tile_begin(st, m, tn * BN);
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        if (tn * BN + c >= N) break;  // warp-uniform
        float acc[32];
        __syncwarp();
        tmem_ld_32x32(taddr + (uint32_t)c, acc);
        tmem_ld_wait();
        epi.chunk(st, m, tn * BN + c, acc, M, N);
      }
      epi.tile_end(st, m, tn, M, N);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[buf]));
      ++local;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace ane
