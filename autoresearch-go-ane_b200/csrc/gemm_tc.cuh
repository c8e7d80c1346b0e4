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
// the epilogue functor.  MT == GEMM_MT_PAIR runs the same pipeline on a cluster of two CTAs that share one
// 256 x BN tile through tcgen05.mma.cta_group::2: each CTA loads its 128 rows of A and half of the B tile, so the
// shared-memory fill per FLOP drops without giving up the second accumulator set.  Every load still writes a
// single CTA's shared memory.
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
static constexpr int GEMM_THREADS = 192;  // TMA warp, MMA warp, four epilogue warps (kernels with eight: 320)
#ifndef ANE_B200_GEMM_EW8
#define ANE_B200_GEMM_EW8 0  // 1: the SwiGLU epilogues of the 256-column CTA-pair kernels run on eight epilogue warps
#endif

// MT = number of 128-row A sub-tiles per output tile.  MT = 2 (256 x BN tiles) shares every B tile between
// two MMAs, so the shared-memory fill per FLOP drops by a third; its MT*BN accumulator columns leave no
// room for a second TMEM buffer when BN > 128, so the epilogue of a tile then does not overlap the next
// tile's main loop -- it pays for long K, not for short K.
// MT = GEMM_MT_PAIR / GEMM_MT_PAIR2: a cluster of two CTAs works on one tile through cta_group::2 MMAs
// (M = 256: 128 rows from each CTA, half of the B tile from each CTA).  PAIR keeps one 128-row sub-tile per
// CTA and both accumulator sets (short K); PAIR2 gives each CTA two sub-tiles (512 x BN tiles, one
// accumulator set): the least fill per FLOP, for long K with few columns.
static constexpr int GEMM_MT_PAIR = 4;
static constexpr int GEMM_MT_PAIR2 = 5;
static constexpr uint32_t GEMM_TMARES_BYTES = 4 * 2 * 4096;
static constexpr uint32_t GEMM_SMEM_LIMIT = 232448u;
template <int BN, int MT>
struct GemmCfg {
  static constexpr bool PAIR = MT >= GEMM_MT_PAIR;
  static constexpr int SUBS = MT == GEMM_MT_PAIR ? 1 : (MT == GEMM_MT_PAIR2 ? 2 : MT);  // 128-row sub-tiles per CTA
  static constexpr int BM_TILE = (PAIR ? 2 : 1) * SUBS * GEMM_BM;       // rows of a scheduled tile
  static constexpr uint32_t A_BYTES = SUBS * GEMM_BM * GEMM_BK * 2;     // per CTA and stage
  // a CTA of a pair holds half of the tile's B rows, rounded up to whole 64-column chunks (an MN-major half of
  // 96 columns is loaded as two chunks, the second half used)
  static constexpr int B_ROWS = PAIR ? ((BN / 2 + 63) / 64) * 64 : BN;
  static constexpr uint32_t B_BYTES = B_ROWS * GEMM_BK * 2;
  // Staged output pieces per epilogue warp (a buffer is reused once its TMA store has read it; four buffers
  // measured no faster than two and cost a pipeline stage).
  static constexpr int SBUF = 2;
  static constexpr uint32_t STAGING_BYTES = 4 * SBUF * 4096;  // 4 epilogue warps x SBUF buffers x (32 rows x 128 B)
  // Epilogue warps.  The epilogues that do arithmetic per element and move more than one piece per 64 accumulator
  // columns (SwiGLU forward: h13 + gate; SwiGLU backward: h13 in, d h13 out) take longer than the 12-k-block main
  // loop of their products with four warps (one per scheduler, ~750 cycles of fixed cost per piece).  With eight,
  // two warps share each TMEM lane group and split the tile's columns (256-column CTA-pair tiles only).  Measured
  // with ANE_B200_GEMM_EW8=1: the two warps of a scheduler then share its exponential unit and the pipeline drops
  // to three stages, W2-dX 51 -> 46 us, W1|W3 forward 51 -> 56 us, the step unchanged; hence off by default.
  __host__ __device__ static constexpr int epi_warps(int epi_kind) {
    return (ANE_B200_GEMM_EW8 && PAIR && SUBS == 1 && BN == 256 && (epi_kind == 3 || epi_kind == 8)) ? 8 : 4;
  }
  __host__ __device__ static constexpr uint32_t staging_bytes(int ew) { return (uint32_t)ew * SBUF * 4096; }
  // Pipeline depth.  Single-CTA kernels take what fits beside the staging buffers and use the TMA-fed residual
  // epilogue only if its buffers still fit; pair kernels give up stages for them instead.
  // `room`: also a single-CTA kernel gives up stages for the TMA-fed input pieces (an epilogue that cannot do without them)
  // `depth`: input pieces each epilogue warp keeps in flight; `ew`: epilogue warps
  __host__ __device__ static constexpr int stages(bool tma_res, bool room = false, int depth = 2, int ew = 4) {
    const uint32_t res = (uint32_t)(ew * depth) * 4096u;
    const uint32_t avail = GEMM_SMEM_LIMIT - 1024u - staging_bytes(ew) - (((PAIR || room) && tma_res) ? res : 0u);
    const int n = (int)(avail / (A_BYTES + B_BYTES));
    return n > 6 ? 6 : n;
  }
  __host__ __device__ static constexpr uint32_t smem_bytes(bool tma_res, bool room = false, int depth = 2, int ew = 4) {  // +1024: alignment
    return stages(tma_res, room, depth, ew) * (A_BYTES + B_BYTES) + staging_bytes(ew) + 1024 +
           (tma_res ? (uint32_t)(ew * depth) * 4096u : 0u);
  }
  // Input pieces (residual, h13) each epilogue warp keeps in flight.  Four instead of two measured no faster for the
  // SwiGLU backward (its pieces arrive in time; the epilogue is bound by its arithmetic), so two everywhere.
  __host__ __device__ static constexpr int res_depth(int) { return 2; }
  static constexpr int ACC_COLS = SUBS * BN;                     // one accumulator set
  static constexpr int NBUF = (2 * ACC_COLS <= 512) ? 2 : 1;     // TMEM accumulator sets
  static constexpr uint32_t TMEM_COLS = (NBUF * ACC_COLS <= 256) ? 256 : 512;
};

// 64-bit shared-memory matrix descriptor (sm_100 format, version field = 1).
__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);            // start address, bits [0,14)
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;   // leading byte offset, bits [16,30)
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;   // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                              // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                              // layout type: 128-byte swizzle
  return d;
}

// Epilogue kinds.  Every kind stages 32-row x 128-byte pieces of the accumulator in 128B-swizzled
// shared memory and hands them to TMA, so global writes are full lines and edge tiles are clipped by
// the tensor map instead of by per-thread bounds checks.
enum EpiKind : int {
  EPI_STORE_BF16 = 0,   // C(bf16) = alpha*acc
  EPI_STORE_F32 = 1,    // C(fp32) = alpha*acc + s1*res1 + s2*res2
  EPI_REDUCE_F32 = 2,   // C(fp32) += alpha*acc  (TMA reduce-add; split-K safe)
  // EPI_STORE_BF16 plus gate = silu(h1) * h3 from the fp32 accumulators: every 64-column piece holds 32
  // columns of h1 and the matching 32 of h3; the gate piece goes straight to global memory.
  EPI_STORE_BF16_SWIGLU = 3,
  // EPI_STORE_BF16 with the rotary embedding applied to the fp32 accumulators of the q|k heads (one
  // 64-column piece = one head); each epilogue thread keeps the cos/sin row of its token in registers.
  EPI_STORE_BF16_ROPE = 4,
  // C(fp32) = alpha*acc + s1*res1 with the residual pieces fetched by TMA (two 32-row x 128-byte buffers
  // per epilogue warp, two pieces ahead) instead of by per-thread row loads: the residual read then costs
  // one bulk copy per piece.  Needs GEMM_TMARES_BYTES of shared memory beside the pipeline stages.
  EPI_STORE_F32_TMARES = 5,
  // EPI_STORE_BF16 that also writes the accumulator of each row's target column in fp32.
  EPI_STORE_BF16_TGT = 6,
  // EPI_STORE_BF16 plus gate = max(h, 0)^2 of every 64-column piece, staged as one more piece (tmD: gate [M, N]).
  EPI_STORE_BF16_RELU2 = 7,
  // SwiGLU backward on the accumulators: acc = d gate [M, N]; tmD = h13 [M, 2N] (bf16, h1 | h3 interleaved in blocks
  // of 32 columns), tmC = d h13 [M, 2N] in the same layout.  A piece is 32 accumulator columns: its h1 | h3 columns
  // are one 64-column bf16 piece of h13, fetched by TMA like the residual pieces of EPI_STORE_F32_TMARES, and its
  // d h1 | d h3 columns one 64-column piece of the output.  d gate itself is never written.
  EPI_DSWIGLU = 8,
  // Classifier head without logits in memory, pass 1: acc = logits tile.  Every row's maximum and sum of
  // exponentials over the tile's columns (log2 domain, after the optional soft cap) go to ce_stats[tile_n][row];
  // the row's target logit, if its column falls into the tile, to tgt_out (fp32, before the soft cap).  Nothing
  // else is stored.
  EPI_CE_STATS = 9,
  // Pass 2 (logits recomputed for a block of vocabulary columns): C(bf16) = coef[row] * (softmax - onehot)
  // [* d softcap] with the row's log2-sum-exp from pass 1; the gradient of the loss with respect to the logits.
  EPI_CE_GRAD = 10,
  // d h = d gate * 2 max(h, 0) on the accumulators of d gate = A*B, with h [M, N] (bf16) fed by TMA through the D
  // map, one 32-row x 64-column piece per output piece: the ReLU^2 backward (ane/common.go:146) in the W2-dX epilogue.
  EPI_DRELU2 = 11,
};
__device__ __forceinline__ float epi_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// tanh by one ex2 and one fast reciprocal: 1 - 2 / (1 + 2^(2 u log2 e))
__device__ __forceinline__ float epi_tanh(float u) {
  return 1.f - __fdividef(2.f, 1.f + epi_ex2(2.885390081777927f * u));
}
// sigmoid(x) = 0.5 + 0.5 tanh(x / 2) on the hardware tanh (relative error ~2^-11, below the bf16 rounding of
// everything it feeds): one special-function instruction where ex2 + reciprocal take two, and the SwiGLU
// epilogues are bound by that unit (16 results per clock per SM).
__device__ __forceinline__ float epi_sigmoid(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  return fmaf(0.5f, t, 0.5f);
}
struct EpiParams {
  float alpha;
  const float* res1;  // optional fp32 [M, ldres]
  const float* s1;    // optional device scalar (nullptr => 1)
  const float* res2;
  const float* s2;
  int ldres;
  bf16* aux;   // EPI_STORE_BF16_SWIGLU: gate [M, N/2]; EPI_STORE_BF16_RELU2: gate [M, N]
  int ldaux;
  const float* rope_cos;  // EPI_STORE_BF16_ROPE: [positions, 32]
  const float* rope_sin;
  int rope_seq, rope_pos0, rope_cols;
  const uint16_t* tgt;  // EPI_STORE_BF16_TGT, EPI_CE_STATS, EPI_CE_GRAD
  float* tgt_out;
  int tgt_row0;
  float* ce_stats;       // EPI_CE_STATS: [tiles_n][ce_rows] pairs (max, sum of 2^(z - max)), z in the log2 domain
  const float* ce_lse2;  // EPI_CE_GRAD: per row log2-sum-exp
  const float* ce_coef;  // EPI_CE_GRAD: per row gradient coefficient (0: row without a target)
  int ce_rows;           // row count of the statistics buffer
  int ce_col0;           // vocabulary column of this product's column 0
  int ce_softcap;        // z = 15 tanh(logit / 15) (ane/common.go:272-287)
};

// Several accumulating products with one contraction length, run by one launch (the four weight gradients of a
// layer: dW = dY^T X with K = tokens for all of them).  Lives in device memory; the tile lists of the problems
// are concatenated and dealt out stream-K, so the launch pays one start-up and each CTA about one exposed
// epilogue where four launches paid four of each.
struct alignas(64) GemmGroup {
  CUtensorMap a[4], b[4], c[4];
  int M[4], N[4];
  int tile0[5];  // first tile of each problem in the concatenated list; tile0[n] = all tiles
  int n;
};

// Work scheduler shared by the three warp roles (each role walks the same sequence).
//   split_k > 0 : classic persistent schedule, work item = (k split, tile), stride gridDim.x.
//   split_k == 0: stream-K.  The tiles x k-blocks units are dealt out in equal contiguous ranges, one per
//                 CTA; a range is cut into segments at tile boundaries and every segment ends in a
//                 reduce-add, so it needs an accumulating epilogue.  Removes the partial last wave.
struct GemmSched {
  int tiles_m, tiles, kblocks, split_k, kb_per_split, total_work, w;
  long long u, u1;
  int bid, nblk;  // this CTA's (or CTA pair's) index and the number of them
  const GemmGroup* grp;  // grouped launch: tiles index the concatenated list
  int bm_tile, prob;     // prob = problem of the segment returned last
  __device__ __forceinline__ void init(int M, int N, int K, int BM_TILE, int BN, int split, int bid_, int nblk_,
                                       const GemmGroup* g = nullptr) {
    bid = bid_;
    nblk = nblk_;
    grp = g;
    bm_tile = BM_TILE;
    prob = 0;
    tiles_m = (M + BM_TILE - 1) / BM_TILE;
    const int tiles_n = (N + BN - 1) / BN;
    tiles = g ? g->tile0[g->n] : tiles_m * tiles_n;
    kblocks = (K + GEMM_BK - 1) / GEMM_BK;
    split_k = split;
    if (split_k > 0) {
      kb_per_split = (kblocks + split_k - 1) / split_k;
      total_work = tiles * split_k;
      w = bid;
    } else {
      const long long units = (long long)tiles * kblocks;
      u = units * bid / nblk;
      u1 = units * (bid + 1) / nblk;
    }
  }
  // Next non-empty segment: tile (tm, tn) and k-block range [kb0, kb1).
  __device__ __forceinline__ bool next(int& tm, int& tn, int& kb0, int& kb1) {
    if (split_k > 0) {
      while (w < total_work) {
        const int split = w / tiles;
        const int rem = w - split * tiles;
        w += nblk;
        kb0 = split * kb_per_split;
        kb1 = min(kb0 + kb_per_split, kblocks);
        if (kb1 <= kb0) continue;
        place(rem, tm, tn);
        return true;
      }
      return false;
    }
    if (u >= u1) return false;
    const int tile = (int)(u / kblocks);
    kb0 = (int)(u - (long long)tile * kblocks);
    const long long left = u1 - u;
    kb1 = (left < (long long)(kblocks - kb0)) ? kb0 + (int)left : kblocks;
    u += kb1 - kb0;
    place(tile, tm, tn);
    return true;
  }
  // tile index -> (tm, tn), and for a grouped launch the problem it belongs to
  __device__ __forceinline__ void place(int tile, int& tm, int& tn) {
    int tmn = tiles_m;
    if (grp) {
      int p = 0;
      while (p + 1 < grp->n && tile >= grp->tile0[p + 1]) ++p;
      prob = p;
      tile -= grp->tile0[p];
      tmn = (grp->M[p] + bm_tile - 1) / bm_tile;
    }
    tn = tile / tmn;
    tm = tile - tn * tmn;
  }
};

template <int BN, int MT, bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(64 + 32 * GemmCfg<BN, MT>::epi_warps(EPI), 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmD, EpiParams epi, int M0,
               int N0, int K, int split_k, int* status, const GemmGroup* group) {
  using Cfg = GemmCfg<BN, MT>;
  // grouped launches exist for the accumulating weight-gradient form on single-CTA tiles only
  constexpr bool kGroup = A_MN && B_MN && EPI == EPI_REDUCE_F32 && MT < GEMM_MT_PAIR;
  const GemmGroup* grp = kGroup ? group : nullptr;
  int M = M0, N = N0;  // the epilogue of a grouped launch sets them per tile
  constexpr bool kTmaRes = (EPI == EPI_STORE_F32_TMARES || EPI == EPI_DSWIGLU || EPI == EPI_DRELU2);  // an input piece per output piece, by TMA
  constexpr int RD = Cfg::res_depth(EPI);  // input pieces in flight per epilogue warp
  constexpr int EW = Cfg::epi_warps(EPI);  // epilogue warps: 4, or 8 (two per TMEM lane group, half of the columns each)
  constexpr int STAGES = Cfg::stages(kTmaRes, EPI == EPI_DSWIGLU || EPI == EPI_DRELU2, RD, EW);
  constexpr int BM = Cfg::BM_TILE, BK = GEMM_BK;
  constexpr int NBUF = Cfg::NBUF;
  constexpr bool PAIR = Cfg::PAIR;
  constexpr int SUBS = Cfg::SUBS;
  static_assert(!PAIR || BN % 32 == 0, "each CTA of a pair supplies BN/2 columns of B");
  // bytes one CTA's loads of a stage deliver
  constexpr uint32_t STAGE_TX = Cfg::A_BYTES + (PAIR ? (B_MN ? Cfg::B_BYTES : (uint32_t)(BN / 2) * BK * 2) : Cfg::B_BYTES);

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[STAGES];
  __shared__ __align__(8) uint64_t bar_empty[STAGES];
  __shared__ __align__(8) uint64_t bar_tfull[NBUF];
  __shared__ __align__(8) uint64_t bar_tempty[NBUF];
  __shared__ uint32_t tmem_slot;
  __shared__ __align__(8) uint64_t bar_res[8][4];  // TMA-fed input pieces (residual, h13): piece landed

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_a0 = smem_base;
  const uint32_t smem_b0 = smem_base + STAGES * Cfg::A_BYTES;
  const uint32_t smem_stage0 = smem_b0 + STAGES * Cfg::B_BYTES;  // epilogue staging, 1024-B aligned

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // A pipeline wait that gave up earlier in this stream poisons the status word: later launches
  // return at once instead of each running into its own time-out.
  // (a pair always runs through: its two CTAs must take the same path, and every wait below is bounded)
  if (!PAIR && status != nullptr && *reinterpret_cast<volatile int*>(status) != DEV_OK) return;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;  // 0 = the CTA that issues the MMAs
  const int sched_id = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int sched_n = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  // rows of this CTA's sub-tile i inside the tile: a pair's MMA i covers 256 consecutive rows, 128 per CTA
  auto sub_row = [&](int i) { return PAIR ? i * 2 * GEMM_BM + (int)rank * GEMM_BM : i * GEMM_BM; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    if constexpr (kTmaRes) {
      for (int w = 0; w < EW; ++w)
        for (int b = 0; b < RD; ++b) mbar_init(smem_u32(&bar_res[w][b]), 1);
      tma_prefetch_desc(&tmD);
    }
    for (int b = 0; b < NBUF; ++b) {
      mbar_init(smem_u32(&bar_tfull[b]), 1);
      mbar_init(smem_u32(&bar_tempty[b]), (PAIR ? 2 : 1) * EW);  // the epilogue warps of both CTAs
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      tmem_alloc_pair(smem_u32(&tmem_slot), Cfg::TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(&tmem_slot), Cfg::TMEM_COLS);
      tmem_relinquish();
    }
  }
  pdl_trigger();
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  pdl_wait();  // operands, residuals and C belong to earlier kernels: nothing above touched them

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      GemmSched sched;
      sched.init(M, N, K, BM, BN, split_k, sched_id, sched_n, grp);
      int tm, tn, kb0, kb1;
      while (ok && sched.next(tm, tn, kb0, kb1)) {
        const CUtensorMap* pA = grp ? &grp->a[sched.prob] : &tmA;
        const CUtensorMap* pB = grp ? &grp->b[sched.prob] : &tmB;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, status, DEV_MBAR_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          const uint32_t sa = smem_a0 + stage * Cfg::A_BYTES;
          const uint32_t sb = smem_b0 + stage * Cfg::B_BYTES;
          if constexpr (PAIR) {
            // both CTAs' bytes complete on the leader's barrier, which expects the sum
            const uint32_t full = map_to_cta(smem_u32(&bar_full[stage]), 0);
            if (rank == 0) mbar_expect_tx(smem_u32(&bar_full[stage]), 2 * STAGE_TX);
            const int n0 = tn * BN + (int)rank * (BN / 2);
#pragma unroll
            for (int i = 0; i < SUBS; ++i) {
              const int m0 = tm * BM + sub_row(i);
              const uint32_t sai = sa + i * (GEMM_BM * BK * 2);
              if constexpr (!A_MN) {
                tma_load_2d_pair(sai, &tmA, full, kb * BK, m0);
              } else {
#pragma unroll
                for (int j = 0; j < GEMM_BM / 64; ++j)
                  tma_load_2d_pair(sai + j * (64 * BK * 2), &tmA, full, m0 + j * 64, kb * BK);
              }
            }
            if constexpr (!B_MN) {
              tma_load_2d_pair(sb, &tmB, full, kb * BK, n0);  // box of BN/2 rows
            } else {
#pragma unroll
              for (int j = 0; j < Cfg::B_ROWS / 64; ++j)  // the last chunk may reach past this CTA's half: unused columns
                tma_load_2d_pair(sb + j * (64 * BK * 2), &tmB, full, n0 + j * 64, kb * BK);
            }
          } else {
          const uint32_t full = smem_u32(&bar_full[stage]);
          mbar_expect_tx(full, STAGE_TX);
          if constexpr (!A_MN) {
#pragma unroll
            for (int i = 0; i < SUBS; ++i)
              tma_load_2d(sa + i * (GEMM_BM * BK * 2), pA, full, kb * BK, tm * BM + i * GEMM_BM);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * (64 * BK * 2), pA, full, tm * BM + j * 64, kb * BK);
          }
          if constexpr (!B_MN) {
            tma_load_2d(sb, pB, full, kb * BK, tn * BN);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (64 * BK * 2), pB, full, tn * BN + j * 64, kb * BK);
          }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) |
                                 ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) |
                                 ((uint32_t)((PAIR ? 2 * GEMM_BM : GEMM_BM) >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      GemmSched sched;
      sched.init(M, N, K, BM, BN, split_k, sched_id, sched_n, grp);
      int tm, tn, kb0, kb1;
      while (ok && sched.next(tm, tn, kb0, kb1)) {
        const int buf = local % NBUF;
        const uint32_t tphase = (uint32_t)(local / NBUF) & 1u;
        if (!mbar_wait(smem_u32(&bar_tempty[buf]), tphase ^ 1u, status, DEV_MBAR_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * Cfg::ACC_COLS);
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
            uint64_t bdesc;
            if constexpr (!B_MN) bdesc = make_smem_desc(sb + k * 32, 16, 1024);
            else                 bdesc = make_smem_desc(sb + k * 2048, 64 * BK * 2, 1024);
#pragma unroll
            for (int i = 0; i < SUBS; ++i) {  // the A sub-tiles share this B tile
              uint64_t adesc;
              const uint32_t sai = sa + i * (GEMM_BM * BK * 2);
              if constexpr (!A_MN) adesc = make_smem_desc(sai + k * 32, 16, 1024);
              else                 adesc = make_smem_desc(sai + k * 2048, 64 * BK * 2, 1024);
              if constexpr (PAIR) tc_mma_bf16_pair(tmem_d + (uint32_t)(i * BN), adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
              else tc_mma_bf16(tmem_d + (uint32_t)(i * BN), adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            }
          }
          if constexpr (PAIR) tc_commit_pair(smem_u32(&bar_empty[stage]));  // frees the stage in both CTAs
          else tc_commit(smem_u32(&bar_empty[stage]));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if constexpr (PAIR) tc_commit_pair(smem_u32(&bar_tfull[buf]));
        else tc_commit(smem_u32(&bar_tfull[buf]));
        ++local;
      }
    }
  } else {
    // ------------------------------ epilogue warps ------------------------------
    const int lane_group = warp & 3;  // TMEM lanes [32*lane_group, 32*lane_group+32)
    // Columns per staged piece: 128 bytes of output per row.
    constexpr bool kBf16Out = (EPI == EPI_STORE_BF16 || EPI == EPI_STORE_BF16_SWIGLU || EPI == EPI_STORE_BF16_ROPE ||
                               EPI == EPI_STORE_BF16_TGT || EPI == EPI_STORE_BF16_RELU2 || EPI == EPI_CE_STATS ||
                               EPI == EPI_CE_GRAD || EPI == EPI_DRELU2);
    constexpr int CW = kBf16Out ? 64 : 32;
    constexpr int SBUF = Cfg::SBUF;
    const uint32_t stage_base = smem_stage0 + (uint32_t)(warp - 2) * (uint32_t)(SBUF * 4096);
    uint8_t* stage_ptr = smem_raw + (stage_base - smem_u32(smem_raw));
    int local = 0;
    int sbuf = 0;
    bool ok = true;
    float a1 = 0.f, a2 = 0.f;
    if constexpr (EPI == EPI_STORE_F32 || EPI == EPI_STORE_F32_TMARES) {
      if (epi.res1) a1 = epi.s1 ? *epi.s1 : 1.f;
      if (epi.res2) a2 = epi.s2 ? *epi.s2 : 1.f;
    }
    // EPI_STORE_F32_TMARES: this warp's two residual buffers, behind the store staging of all four warps
    const uint32_t res_base = smem_stage0 + Cfg::staging_bytes(EW) + (uint32_t)(warp - 2) * (uint32_t)(RD * 4096);
    // with eight warps, warps 2-5 take the first half of the tile's columns and warps 6-9 the second
    constexpr int CSPAN = BN / (EW / 4);
    const int c_begin = ((warp - 2) >> 2) * CSPAN, c_end = c_begin + CSPAN;
    const uint8_t* res_ptr = smem_raw + (res_base - smem_u32(smem_raw));
    uint32_t res_uses = 0;  // pieces consumed so far (buffer = uses % RD, phase = (uses / RD) & 1)
    GemmSched sched;
    sched.init(M, N, K, BM, BN, split_k, sched_id, sched_n, grp);
    int tm, tn, kb0, kb1;
    while (ok && sched.next(tm, tn, kb0, kb1)) {
      const CUtensorMap* pC = &tmC;
      if (grp) {  // this tile's problem: its output map and bounds
        pC = &grp->c[sched.prob];
        M = grp->M[sched.prob];
        N = grp->N[sched.prob];
      }
      const int buf = local % NBUF;
      const uint32_t tphase = (uint32_t)(local / NBUF) & 1u;
      // Residual rows are fetched one 32-column piece ahead (the first piece while the MMAs of this
      // tile are still running), so their latency is off the epilogue's critical path.
      float4 pre[8];
      bool pre_ok = false;
      auto prefetch_first = [&](int m) {
        if constexpr (EPI == EPI_STORE_F32) {
          pre_ok = false;
          if (epi.res1 && m < M && tn * BN + c_begin + 32 <= N) {
            const float4* rp = reinterpret_cast<const float4*>(epi.res1 + (size_t)m * epi.ldres + tn * BN + c_begin);
#pragma unroll
            for (int q = 0; q < 8; ++q) pre[q] = rp[q];
            pre_ok = true;
          }
        }
      };
      prefetch_first(tm * BM + sub_row(0) + lane_group * 32 + lane);
      // Residual piece `piece` (counted over the whole kernel) of the current (tile, sub): same validity test as
      // the consuming loop, so every issued piece is consumed.
      uint32_t res_issued = res_uses;
      auto issue_res = [&](int m_w, int n0r) {
        if constexpr (kTmaRes) {
          if (n0r < N && n0r < tn * BN + c_end && m_w < M) {
            if (lane == 0) {
              const uint32_t b = res_issued % (uint32_t)RD;
              const uint32_t bar = smem_u32(&bar_res[warp - 2][b]);
              mbar_expect_tx(bar, 4096);
              tma_load_2d(res_base + b * 4096u, &tmD, bar, EPI == EPI_DSWIGLU ? 2 * n0r : n0r, m_w);
            }
            ++res_issued;
          }
        }
      };
      if constexpr (kTmaRes) {  // first two pieces of sub-tile 0, while the MMAs still run
#pragma unroll
        for (int k = 0; k < RD; ++k) issue_res(tm * BM + sub_row(0) + lane_group * 32, tn * BN + c_begin + k * CW);
      }
      if (!mbar_wait(smem_u32(&bar_tfull[buf]), tphase, status, DEV_MBAR_TIMEOUT_EPILOGUE)) {
        ok = false;
        break;
      }
      tc_fence_after();
#pragma unroll 1
      for (int sub = 0; sub < SUBS; ++sub) {
      const int m_warp = tm * BM + sub_row(sub) + lane_group * 32;
      const int m = m_warp + lane;
      if (sub > 0) {
        prefetch_first(m);
        if constexpr (kTmaRes) {
#pragma unroll
          for (int k = 0; k < RD; ++k) issue_res(m_warp, tn * BN + c_begin + k * CW);
        }
      }
      int tgt_col = -1;        // EPI_STORE_BF16_TGT: this row's target column
      if constexpr (EPI == EPI_STORE_BF16_TGT || EPI == EPI_CE_STATS || EPI == EPI_CE_GRAD) {
        if (m < M) tgt_col = (int)epi.tgt[epi.tgt_row0 + m];
      }
      float ce_m = -INFINITY, ce_s = 0.f;  // EPI_CE_STATS: this row's running maximum / sum over the tile's pieces
      float ce_l = 0.f, ce_c = 0.f;        // EPI_CE_GRAD: this row's log2-sum-exp and coefficient
      if constexpr (EPI == EPI_CE_GRAD) {
        if (m < M) {
          ce_l = epi.ce_lse2[m];
          ce_c = epi.ce_coef[m];
        }
      }
      uint32_t gate_even[16];  // EPI_STORE_BF16_SWIGLU: the even piece's half of a gate row
      float4 rc4[8], rs4[8];   // EPI_STORE_BF16_ROPE: cos / sin of this thread's token, 32 pairs
      if constexpr (EPI == EPI_STORE_BF16_ROPE) {
        if (tn * BN < epi.rope_cols && m < M) {
          const size_t pos = (size_t)(epi.rope_pos0 + m % epi.rope_seq) * 32;
          const float4* cp = reinterpret_cast<const float4*>(epi.rope_cos + pos);
          const float4* sp = reinterpret_cast<const float4*>(epi.rope_sin + pos);
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            rc4[q] = cp[q];
            rs4[q] = sp[q];
          }
        }
      }
      const uint32_t taddr = tmem_base + ((uint32_t)(lane_group * 32) << 16) +
                             (uint32_t)(buf * Cfg::ACC_COLS + sub * BN);
#pragma unroll 1
      for (int c = c_begin; c < c_end; c += CW) {
        const int n0 = tn * BN + c;
        if (n0 >= N || m_warp >= M) break;  // warp-uniform
        float acc[CW];
        __syncwarp();
        tmem_ld_32x32(taddr + (uint32_t)c, acc);
        if constexpr (CW == 64) tmem_ld_32x32(taddr + (uint32_t)c + 32u, acc + 32);
        float4 cur[8];
        bool cur_ok = false;
        if constexpr (EPI == EPI_STORE_F32) {
          cur_ok = pre_ok;
#pragma unroll
          for (int q = 0; q < 8; ++q) cur[q] = pre[q];
          pre_ok = false;
          const int nn = n0 + CW;
          if (epi.res1 && m < M && c + CW < c_end && nn + 32 <= N) {
            const float4* rp = reinterpret_cast<const float4*>(epi.res1 + (size_t)m * epi.ldres + nn);
#pragma unroll
            for (int q = 0; q < 8; ++q) pre[q] = rp[q];
            pre_ok = true;
          }
        }
        tmem_ld_wait();
        if constexpr (EPI == EPI_CE_STATS) {
          constexpr float kL2e = 1.4426950408889634f;
          const int t = tgt_col - epi.ce_col0 - n0;
          if (t >= 0 && t < CW) {  // one piece per row at most
            float v = 0.f;
#pragma unroll
            for (int e = 0; e < CW; ++e) v = (e == t) ? acc[e] : v;
            epi.tgt_out[epi.tgt_row0 + m] = epi.alpha * v;
          }
          const int nvalid = N - n0;  // columns past the matrix hold zeros: they must not count
          // Four independent chains for the maximum and for the sum: one warp per scheduler has only its own
          // instruction-level parallelism to hide the latency of the adds and of the exponentials.
          float pm[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
          float ps[4] = {0.f, 0.f, 0.f, 0.f};
          if (!epi.ce_softcap && nvalid >= CW) {  // the common case: 2^(acc * a2 - max) straight from the accumulators
            const float a2 = epi.alpha * kL2e;    // alpha > 0: the maximum of the raw values is the maximum of the scaled ones
#pragma unroll
            for (int e = 0; e < CW; e += 4) {
              pm[0] = fmaxf(pm[0], acc[e]); pm[1] = fmaxf(pm[1], acc[e + 1]);
              pm[2] = fmaxf(pm[2], acc[e + 2]); pm[3] = fmaxf(pm[3], acc[e + 3]);
            }
            const float mn = fmaxf(ce_m, a2 * fmaxf(fmaxf(pm[0], pm[1]), fmaxf(pm[2], pm[3])));
#pragma unroll
            for (int e = 0; e < CW; e += 4) {
              ps[0] += epi_ex2(fmaf(acc[e], a2, -mn)); ps[1] += epi_ex2(fmaf(acc[e + 1], a2, -mn));
              ps[2] += epi_ex2(fmaf(acc[e + 2], a2, -mn)); ps[3] += epi_ex2(fmaf(acc[e + 3], a2, -mn));
            }
            ce_s = ce_s * epi_ex2(ce_m - mn) + ((ps[0] + ps[1]) + (ps[2] + ps[3]));
            ce_m = mn;
          } else {
#pragma unroll
            for (int e = 0; e < CW; ++e) {
              float v = epi.alpha * acc[e];
              if (epi.ce_softcap) v = 15.f * epi_tanh(v * (1.f / 15.f));
              v = (e < nvalid) ? v * kL2e : -INFINITY;
              acc[e] = v;
              pm[e & 3] = fmaxf(pm[e & 3], v);
            }
            const float mn = fmaxf(ce_m, fmaxf(fmaxf(pm[0], pm[1]), fmaxf(pm[2], pm[3])));
#pragma unroll
            for (int e = 0; e < CW; ++e) ps[e & 3] += epi_ex2(acc[e] - mn);
            ce_s = ce_s * epi_ex2(ce_m - mn) + ((ps[0] + ps[1]) + (ps[2] + ps[3]));
            ce_m = mn;
          }
          continue;  // nothing is staged or stored
        }
        // The piece staged SBUF iterations ago must have been read by its TMA store before its
        // buffer is rewritten.
        if (lane == 0) tma_store_wait_read<SBUF - 1>();
        __syncwarp();
        uint8_t* row_ptr = stage_ptr + sbuf * 4096 + lane * 128;
        if constexpr (EPI == EPI_CE_GRAD) {
          constexpr float kL2e = 1.4426950408889634f;
          const int t = tgt_col - epi.ce_col0 - n0;
          // The one-hot term touches one element of one piece per row: it is taken out of the sweep.  A row whose
          // target falls into this piece first fetches that raw value, then corrects the element after the sweep.
          float corr = 0.f;
          const bool has_t = t >= 0 && t < CW;
          if (has_t) {
            float v = 0.f;
#pragma unroll
            for (int e = 0; e < CW; ++e) v = (e == t) ? acc[e] : v;
            v *= epi.alpha;
            float dcap = 1.f;
            if (epi.ce_softcap) {
              const float th = epi_tanh(v * (1.f / 15.f));
              dcap = 1.f - th * th;
            }
            corr = ce_c * dcap;
          }
          if (!epi.ce_softcap) {
            const float a2 = epi.alpha * kL2e;
#pragma unroll
            for (int e = 0; e < CW; ++e) acc[e] = ce_c * epi_ex2(fmaf(acc[e], a2, -ce_l));
          } else {
#pragma unroll
            for (int e = 0; e < CW; ++e) {
              const float th = epi_tanh(epi.alpha * acc[e] * (1.f / 15.f));
              acc[e] = ce_c * epi_ex2(fmaf(15.f * th, kL2e, -ce_l)) * (1.f - th * th);
            }
          }
          if (has_t) {
#pragma unroll
            for (int e = 0; e < CW; ++e) acc[e] = (e == t) ? acc[e] - corr : acc[e];
          }
#pragma unroll
          for (int q = 0; q < 8; ++q)
            *reinterpret_cast<uint4*>(row_ptr + ((q ^ (lane & 7)) << 4)) =
                make_uint4(pack2_bf16(acc[8 * q], acc[8 * q + 1]), pack2_bf16(acc[8 * q + 2], acc[8 * q + 3]),
                           pack2_bf16(acc[8 * q + 4], acc[8 * q + 5]), pack2_bf16(acc[8 * q + 6], acc[8 * q + 7]));
        } else if constexpr (EPI == EPI_DSWIGLU) {
          const uint32_t b = res_uses % (uint32_t)RD;
          if (!mbar_wait(smem_u32(&bar_res[warp - 2][b]), (res_uses / (uint32_t)RD) & 1u, status, DEV_MBAR_TIMEOUT_EPILOGUE)) {
            ok = false;
            break;
          }
          // this row's 64 bf16 of h13: 16-byte chunks 0-3 = h1 of the piece's 32 gate columns, 4-7 = h3
          const uint8_t* hrow = res_ptr + b * 4096u + lane * 128;
          uint4 hraw[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) hraw[q] = *reinterpret_cast<const uint4*>(hrow + ((q ^ (lane & 7)) << 4));
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const __nv_bfloat162* h1p = reinterpret_cast<const __nv_bfloat162*>(&hraw[q]);
            const __nv_bfloat162* h3p = reinterpret_cast<const __nv_bfloat162*>(&hraw[q + 4]);
            uint32_t o1[4], o3[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 x = __bfloat1622float2(h1p[e]), h = __bfloat1622float2(h3p[e]);
              const float dg0 = epi.alpha * acc[8 * q + 2 * e], dg1 = epi.alpha * acc[8 * q + 2 * e + 1];
              // d silu = s (1 + x (1 - s)) with s = sigmoid(x)
              const float s0 = epi_sigmoid(x.x), s1 = epi_sigmoid(x.y);
              o1[e] = pack2_bf16(dg0 * h.x * s0 * (1.f + x.x * (1.f - s0)), dg1 * h.y * s1 * (1.f + x.y * (1.f - s1)));
              o3[e] = pack2_bf16(dg0 * x.x * s0, dg1 * x.y * s1);
            }
            *reinterpret_cast<uint4*>(row_ptr + ((q ^ (lane & 7)) << 4)) = make_uint4(o1[0], o1[1], o1[2], o1[3]);
            *reinterpret_cast<uint4*>(row_ptr + (((q + 4) ^ (lane & 7)) << 4)) = make_uint4(o3[0], o3[1], o3[2], o3[3]);
          }
        } else if constexpr (EPI == EPI_DRELU2) {
          const uint32_t b = res_uses % (uint32_t)RD;
          if (!mbar_wait(smem_u32(&bar_res[warp - 2][b]), (res_uses / (uint32_t)RD) & 1u, status, DEV_MBAR_TIMEOUT_EPILOGUE)) {
            ok = false;
            break;
          }
          const uint8_t* hrow = res_ptr + b * 4096u + lane * 128;  // this row's 64 bf16 of h
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const uint4 hraw = *reinterpret_cast<const uint4*>(hrow + ((q ^ (lane & 7)) << 4));
            const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&hraw);
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 h = __bfloat1622float2(hp[e]);
              const float two_a = 2.f * epi.alpha;
              o[e] = pack2_bf16(two_a * acc[8 * q + 2 * e] * fmaxf(h.x, 0.f), two_a * acc[8 * q + 2 * e + 1] * fmaxf(h.y, 0.f));
            }
            *reinterpret_cast<uint4*>(row_ptr + ((q ^ (lane & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        } else if constexpr (kBf16Out) {
          if constexpr (EPI == EPI_STORE_BF16_TGT) {
            const int t = tgt_col - n0;
            if (t >= 0 && t < CW) {  // one piece per row at most
              float v = 0.f;
#pragma unroll
              for (int e = 0; e < CW; ++e) v = (e == t) ? acc[e] : v;
              epi.tgt_out[epi.tgt_row0 + m] = epi.alpha * v;
            }
          }
          if constexpr (EPI == EPI_STORE_BF16_ROPE) {
            if (n0 < epi.rope_cols && m < M) {  // pairs (2p, 2p+1) of this head
              const float* rc = reinterpret_cast<const float*>(rc4);
              const float* rs = reinterpret_cast<const float*>(rs4);
#pragma unroll
              for (int pr = 0; pr < 32; ++pr) {
                const float a = acc[2 * pr], b = acc[2 * pr + 1];
                acc[2 * pr] = a * rc[pr] - b * rs[pr];
                acc[2 * pr + 1] = b * rc[pr] + a * rs[pr];
              }
            }
          }
          if constexpr (EPI == EPI_STORE_BF16_SWIGLU) {
            // gate = silu(h1) * h3 for the 32 gate columns of this piece.  Two consecutive pieces make one
            // 128-byte gate row: the even piece parks its half in registers, the odd piece stages the row
            // as one more piece of the two-buffer rotation (it takes this buffer, h13 takes the other).
            uint32_t gcur[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              // silu(x) * h = x * h * sigmoid(x) (the epilogue has four warps per SM, so instruction count
              // matters here)
              const float x0 = epi.alpha * acc[2 * e], x1 = epi.alpha * acc[2 * e + 1];
              const float h0 = epi.alpha * acc[32 + 2 * e], h1 = epi.alpha * acc[32 + 2 * e + 1];
              gcur[e] = pack2_bf16(x0 * h0 * epi_sigmoid(x0), x1 * h1 * epi_sigmoid(x1));
            }
            if (((c / CW) & 1) == 0) {
#pragma unroll
              for (int e = 0; e < 16; ++e) gate_even[e] = gcur[e];
            } else {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                *reinterpret_cast<uint4*>(row_ptr + ((q ^ (lane & 7)) << 4)) =
                    make_uint4(gate_even[4 * q], gate_even[4 * q + 1], gate_even[4 * q + 2], gate_even[4 * q + 3]);
                *reinterpret_cast<uint4*>(row_ptr + (((q + 4) ^ (lane & 7)) << 4)) =
                    make_uint4(gcur[4 * q], gcur[4 * q + 1], gcur[4 * q + 2], gcur[4 * q + 3]);
              }
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_2d(&tmD, stage_base + (uint32_t)sbuf * 4096u, (n0 - CW) >> 1, m_warp);
                tma_store_commit();
                tma_store_wait_read<SBUF - 1>();  // the next buffer in the rotation is free again
              }
              sbuf = (sbuf + 1) % SBUF;
              __syncwarp();
              row_ptr = stage_ptr + sbuf * 4096 + lane * 128;
            }
          }
          if constexpr (EPI == EPI_STORE_BF16_RELU2) {
            // gate piece first (this buffer), then the h piece takes the next buffer of the rotation
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              float g[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const float h = fmaxf(epi.alpha * acc[8 * q + e], 0.f);
                g[e] = h * h;
              }
              *reinterpret_cast<uint4*>(row_ptr + ((q ^ (lane & 7)) << 4)) =
                  make_uint4(pack2_bf16(g[0], g[1]), pack2_bf16(g[2], g[3]), pack2_bf16(g[4], g[5]), pack2_bf16(g[6], g[7]));
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmD, stage_base + (uint32_t)sbuf * 4096u, n0, m_warp);
              tma_store_commit();
              tma_store_wait_read<SBUF - 1>();  // the next buffer in the rotation is free again
            }
            sbuf = (sbuf + 1) % SBUF;
            __syncwarp();
            row_ptr = stage_ptr + sbuf * 4096 + lane * 128;
          }
#pragma unroll
          for (int q = 0; q < 8; ++q) {  // 8 chunks of 8 bf16
            uint4 u;
            u.x = pack2_bf16(epi.alpha * acc[8 * q + 0], epi.alpha * acc[8 * q + 1]);
            u.y = pack2_bf16(epi.alpha * acc[8 * q + 2], epi.alpha * acc[8 * q + 3]);
            u.z = pack2_bf16(epi.alpha * acc[8 * q + 4], epi.alpha * acc[8 * q + 5]);
            u.w = pack2_bf16(epi.alpha * acc[8 * q + 6], epi.alpha * acc[8 * q + 7]);
            *reinterpret_cast<uint4*>(row_ptr + ((q ^ (lane & 7)) << 4)) = u;
          }
        } else {
          const bool in_rows = m < M;
          const float* r1 = (EPI == EPI_STORE_F32 && epi.res1 && in_rows) ? epi.res1 + (size_t)m * epi.ldres + n0 : nullptr;
          const float* r2 = (EPI == EPI_STORE_F32 && epi.res2 && in_rows) ? epi.res2 + (size_t)m * epi.ldres + n0 : nullptr;
          const bool full = n0 + 32 <= N;
          const uint8_t* res_row = nullptr;
          float4 rres[8];  // the residual piece, read before any staging store (the compiler cannot tell the two apart)
          if constexpr (EPI == EPI_STORE_F32_TMARES) {
            const uint32_t b = res_uses % (uint32_t)RD;
            if (!mbar_wait(smem_u32(&bar_res[warp - 2][b]), (res_uses / (uint32_t)RD) & 1u, status, DEV_MBAR_TIMEOUT_EPILOGUE)) {
              ok = false;
              break;
            }
            res_row = res_ptr + b * 4096u + lane * 128;
#pragma unroll
            for (int q = 0; q < 8; ++q) rres[q] = *reinterpret_cast<const float4*>(res_row + ((q ^ (lane & 7)) << 4));
          }
#pragma unroll
          for (int q = 0; q < 8; ++q) {  // 8 chunks of 4 fp32
            float4 v = make_float4(epi.alpha * acc[4 * q], epi.alpha * acc[4 * q + 1], epi.alpha * acc[4 * q + 2],
                                   epi.alpha * acc[4 * q + 3]);
            if constexpr (EPI == EPI_STORE_F32_TMARES) {  // rows / columns outside the tensor arrive as zeros
              const float4 t = rres[q];
              v.x += a1 * t.x; v.y += a1 * t.y; v.z += a1 * t.z; v.w += a1 * t.w;
            }
            if constexpr (EPI == EPI_STORE_F32) {
              if (r1) {
                if (cur_ok) {
                  const float4 t = cur[q];
                  v.x += a1 * t.x; v.y += a1 * t.y; v.z += a1 * t.z; v.w += a1 * t.w;
                } else if (full) {
                  const float4 t = *reinterpret_cast<const float4*>(r1 + 4 * q);
                  v.x += a1 * t.x; v.y += a1 * t.y; v.z += a1 * t.z; v.w += a1 * t.w;
                } else {
                  if (n0 + 4 * q + 0 < N) v.x += a1 * r1[4 * q + 0];
                  if (n0 + 4 * q + 1 < N) v.y += a1 * r1[4 * q + 1];
                  if (n0 + 4 * q + 2 < N) v.z += a1 * r1[4 * q + 2];
                  if (n0 + 4 * q + 3 < N) v.w += a1 * r1[4 * q + 3];
                }
              }
              if (r2) {
                if (full) {
                  const float4 t = *reinterpret_cast<const float4*>(r2 + 4 * q);
                  v.x += a2 * t.x; v.y += a2 * t.y; v.z += a2 * t.z; v.w += a2 * t.w;
                } else {
                  if (n0 + 4 * q + 0 < N) v.x += a2 * r2[4 * q + 0];
                  if (n0 + 4 * q + 1 < N) v.y += a2 * r2[4 * q + 1];
                  if (n0 + 4 * q + 2 < N) v.z += a2 * r2[4 * q + 2];
                  if (n0 + 4 * q + 3 < N) v.w += a2 * r2[4 * q + 3];
                }
              }
            }
            *reinterpret_cast<float4*>(row_ptr + ((q ^ (lane & 7)) << 4)) = v;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if constexpr (kTmaRes) {  // this residual buffer is free: fetch the piece after next
          ++res_uses;
          issue_res(m_warp, n0 + RD * CW);
        }
        if (lane == 0) {
          const uint32_t src = stage_base + (uint32_t)sbuf * 4096u;
          if constexpr (EPI == EPI_REDUCE_F32) tma_reduce_add_2d(pC, src, n0, m_warp);
          else if constexpr (EPI == EPI_DSWIGLU) tma_store_2d(&tmC, src, 2 * n0, m_warp);
          else tma_store_2d(&tmC, src, n0, m_warp);
          tma_store_commit();
        }
        sbuf = (sbuf + 1) % SBUF;
      }
      if constexpr (EPI == EPI_CE_STATS) {
        if (m < M && m_warp < M && tn * BN < N)
          reinterpret_cast<float2*>(epi.ce_stats)[(size_t)tn * epi.ce_rows + m] = make_float2(ce_m, ce_s);
      }
      }  // sub
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR && rank != 0) mbar_arrive_cluster(map_to_cta(smem_u32(&bar_tempty[buf]), 0));
        else mbar_arrive(smem_u32(&bar_tempty[buf]));
      }
      ++local;
    }
    if (lane == 0) tma_store_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();  // the peer has drained its accumulators and its last loads have landed
  if (warp == 1) {
    tc_fence_after();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
    else tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace ane
