// GEMM launchers: tcgen05 bf16 path (gemm_tc.cuh) and the fp32 SIMT path.
#include "gemm.h"

#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <mutex>
#include <string>
#include <tuple>

#include "gemm_tc.cuh"

namespace ane {

static thread_local std::string g_gemm_err;
const char* gemm_last_error() { return g_gemm_err.c_str(); }

bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("ANE_B200_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

int gemm_num_sms() {
  static int sms[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (sms[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    // ANE_B200_GEMM_SMS caps the persistent grids (e.g. to leave SMs to a communication kernel).
    const char* e = getenv("ANE_B200_GEMM_SMS");
    if (e && atoi(e) > 0 && atoi(e) < n) n = atoi(e);
    sms[dev] = n;
  }
  return sms[dev];
}

// ------------------------------------------------------------------------------------------
// Tensor maps
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 2-D tensor [outer, inner] with row pitch ld (elements); box = [box_outer, box_inner]; 128B swizzle.
static bool make_tmap(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer, bool is_f32 = false) {
  typedef std::tuple<int, const void*, uint64_t, uint64_t, uint64_t, uint32_t, uint32_t, bool> Key;
  static std::map<Key, CUtensorMap> cache;
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  Key key(dev, ptr, inner, outer, ld, box_inner, box_outer, is_f32);
  const uint64_t esz = is_f32 ? 4 : 2;
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return true;
  }
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    g_gemm_err = "cuTensorMapEncodeTiled entry point not available";
    return false;
  }
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || (ld * esz) % 16 != 0) {
    g_gemm_err = "TMA operand must be 16-byte aligned with a 16-byte multiple row pitch";
    return false;
  }
  cuuint64_t gdim[2] = {inner, outer};
  cuuint64_t gstride[1] = {ld * esz};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap tm;
  CUresult r = fn(&tm, is_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[160];
    snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled failed (%d) inner=%llu outer=%llu ld=%llu", (int)r,
             (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)ld);
    g_gemm_err = buf;
    return false;
  }
  cache[key] = tm;
  *out = tm;
  return true;
}

bool make_tmap_2d(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                  uint32_t box_outer, bool is_f32) {
  return make_tmap(out, ptr, inner, outer, ld, box_inner, box_outer, is_f32);
}

template <int BN, int MT, bool A_MN, bool B_MN, int EPI>
static int launch_tc(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& td,
                     const EpiParams& epi,
                     const GemmDesc& d, int split_k, int* d_status, cudaStream_t stream) {
  auto kern = gemm_tc_kernel<BN, MT, A_MN, B_MN, EPI>;
  constexpr bool tma_res = (EPI == EPI_STORE_F32_TMARES || EPI == EPI_DSWIGLU || EPI == EPI_DRELU2);
  constexpr int depth = GemmCfg<BN, MT>::res_depth(EPI);
  constexpr int ew = GemmCfg<BN, MT>::epi_warps(EPI);
  constexpr int threads = 64 + 32 * ew;
  constexpr uint32_t smem_bytes = GemmCfg<BN, MT>::smem_bytes(tma_res, EPI == EPI_DSWIGLU || EPI == EPI_DRELU2, depth, ew);
  static_assert(smem_bytes <= GEMM_SMEM_LIMIT && GemmCfg<BN, MT>::stages(tma_res, EPI == EPI_DSWIGLU || EPI == EPI_DRELU2, depth, ew) >= 3, "pipeline does not fit");
  static bool attr_set = false;  // per template instantiation
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes);
    if (e != cudaSuccess) {
      g_gemm_err = std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e);
      return -3;
    }
    attr_set = true;
  }
  constexpr int BM_TILE = GemmCfg<BN, MT>::BM_TILE;
  const int base_tiles = ((d.M + BM_TILE - 1) / BM_TILE) * ((d.N + BN - 1) / BN);
  if constexpr (GemmCfg<BN, MT>::PAIR) {
    // one cluster of two CTAs per tile; as many clusters as the device keeps resident at once
    static int max_pairs = 0;  // per template instantiation
    if (max_pairs == 0) {
      cudaLaunchConfig_t q = {};
      q.gridDim = dim3(2 * 74);
      q.blockDim = dim3(threads);
      q.dynamicSmemBytes = smem_bytes;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = 2;
      at[0].val.clusterDim.y = 1;
      at[0].val.clusterDim.z = 1;
      q.attrs = at;
      q.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &q) != cudaSuccess || n <= 0) n = gemm_num_sms() / 2;
      if (n > gemm_num_sms() / 2) n = gemm_num_sms() / 2;
      max_pairs = n;
    }
    const int work = base_tiles * (split_k > 0 ? split_k : 1);
    const int pairs = work < max_pairs ? work : max_pairs;
    cudaError_t e = launch_pdl_cluster(kern, dim3(2 * (pairs < 1 ? 1 : pairs)), dim3(threads), smem_bytes, stream, 2u,
                                       ta, tb, tc, td, epi, d.M, d.N, d.K, split_k > 0 ? split_k : 1, d_status,
                                       (const GemmGroup*)nullptr);
    if (e != cudaSuccess) {
      g_gemm_err = std::string("gemm_tc pair launch: ") + cudaGetErrorString(e);
      return -4;
    }
    return 0;
  }
  int grid;
  if (split_k > 0) {
    const int tiles = base_tiles * split_k;
    grid = tiles < gemm_num_sms() ? tiles : gemm_num_sms();
  } else {  // stream-K: equal shares of the tile x k-block units, at least 8 k-blocks per CTA
    const long long units = (long long)base_tiles * ((d.K + GEMM_BK - 1) / GEMM_BK);
    long long g = units / 8;
    if (g > gemm_num_sms()) g = gemm_num_sms();
    grid = (int)g;
  }
  if (grid < 1) grid = 1;
  cudaError_t e = launch_pdl(kern, dim3(grid), dim3(threads), smem_bytes, stream, ta, tb, tc, td, epi, d.M, d.N,
                             d.K, split_k, d_status, (const GemmGroup*)nullptr);
  if (e != cudaSuccess) {
    g_gemm_err = std::string("gemm_tc launch: ") + cudaGetErrorString(e);
    return -4;
  }
  return 0;
}

template <int BN, int MT, bool A_MN, bool B_MN>
static int dispatch_epi(const CUtensorMap& ta, const CUtensorMap& tb, const GemmDesc& d, int split_k,
                        int* d_status, cudaStream_t stream) {
  EpiParams epi{d.alpha, d.res1, d.s1, d.res2, d.s2, d.ldres, reinterpret_cast<bf16*>(d.aux), d.ldaux,
                d.rope_cos, d.rope_sin, d.rope_seq, d.rope_pos0, d.rope_cols, d.tgt, d.tgt_out, d.tgt_row0,
                d.ce_stats, d.ce_lse2, d.ce_coef, d.ce_rows, d.ce_col0, d.ce_softcap ? 1 : 0};
  CUtensorMap tc;
  if (d.out == GEMM_OUT_BF16) {
    if (!make_tmap(&tc, d.C, d.N, d.M, d.ldc, 64, 32, false)) return -2;
    return launch_tc<BN, MT, A_MN, B_MN, EPI_STORE_BF16>(ta, tb, tc, tc, epi, d, 1, d_status, stream);
  }
  if (d.out == GEMM_OUT_BF16_TGT) {
    if constexpr (!A_MN && !B_MN) {
      if (d.tgt == nullptr || d.tgt_out == nullptr) {
        g_gemm_err = "target-logit epilogue: missing target pointers";
        return -2;
      }
      if (!make_tmap(&tc, d.C, d.N, d.M, d.ldc, 64, 32, false)) return -2;
      return launch_tc<BN, MT, A_MN, B_MN, EPI_STORE_BF16_TGT>(ta, tb, tc, tc, epi, d, 1, d_status, stream);
    } else {
      g_gemm_err = "the target-logit epilogue takes K-major operands only";
      return -2;
    }
  }
  if (d.out == GEMM_OUT_BF16_ROPE) {
    if constexpr (!A_MN && !B_MN) {
      if (!make_tmap(&tc, d.C, d.N, d.M, d.ldc, 64, 32, false)) return -2;
      return launch_tc<BN, MT, A_MN, B_MN, EPI_STORE_BF16_ROPE>(ta, tb, tc, tc, epi, d, 1, d_status, stream);
    } else {
      g_gemm_err = "the rotary epilogue takes K-major operands only";
      return -2;
    }
  }
  if (d.out == GEMM_OUT_BF16_SWIGLU) {
    if constexpr (!A_MN && !B_MN) {
      CUtensorMap td;  // gate [M, N/2]: pieces of 32 rows x 64 columns
      if (!make_tmap(&tc, d.C, d.N, d.M, d.ldc, 64, 32, false) ||
          !make_tmap(&td, d.aux, d.N / 2, d.M, d.ldaux, 64, 32, false))
        return -2;
      return launch_tc<BN, MT, A_MN, B_MN, EPI_STORE_BF16_SWIGLU>(ta, tb, tc, td, epi, d, 1, d_status, stream);
    } else {
      g_gemm_err = "the SwiGLU epilogue takes K-major operands only";
      return -2;
    }
  }
  if (d.out == GEMM_OUT_BF16_RELU2) {
    if constexpr (!A_MN && !B_MN) {
      CUtensorMap td;  // gate [M, N], same pieces as C
      if (!make_tmap(&tc, d.C, d.N, d.M, d.ldc, 64, 32, false) || !make_tmap(&td, d.aux, d.N, d.M, d.ldaux, 64, 32, false))
        return -2;
      return launch_tc<BN, MT, A_MN, B_MN, EPI_STORE_BF16_RELU2>(ta, tb, tc, td, epi, d, 1, d_status, stream);
    } else {
      g_gemm_err = "the ReLU^2 epilogue takes K-major operands only";
      return -2;
    }
  }
  if (d.out == GEMM_OUT_CE_STATS || d.out == GEMM_OUT_CE_GRAD) {
    if constexpr (!A_MN && !B_MN && BN == 256 && (MT == 1 || MT == GEMM_MT_PAIR)) {
      if (d.out == GEMM_OUT_CE_STATS)  // no output tensor: the A map stands in for the unused descriptors
        return launch_tc<BN, MT, A_MN, B_MN, EPI_CE_STATS>(ta, tb, ta, ta, epi, d, 1, d_status, stream);
      if (!make_tmap(&tc, d.C, d.N, d.M, d.ldc, 64, 32, false)) return -2;
      return launch_tc<BN, MT, A_MN, B_MN, EPI_CE_GRAD>(ta, tb, tc, tc, epi, d, 1, d_status, stream);
    } else {
      g_gemm_err = "the classifier-head epilogues take K-major operands on 256-column tiles";
      return -2;
    }
  }
  if (d.out == GEMM_OUT_DSWIGLU) {
    if constexpr (!A_MN && B_MN && BN == 256 && (MT == 1 || MT == GEMM_MT_PAIR)) {
      CUtensorMap td;  // h13 in, d h13 out: [M, 2N] bf16, pieces of 32 rows x 64 columns
      if (!make_tmap(&tc, d.C, 2 * (uint64_t)d.N, d.M, d.ldc, 64, 32, false) ||
          !make_tmap(&td, d.aux, 2 * (uint64_t)d.N, d.M, d.ldaux, 64, 32, false))
        return -2;
      return launch_tc<BN, MT, A_MN, B_MN, EPI_DSWIGLU>(ta, tb, tc, td, epi, d, 1, d_status, stream);
    } else {
      g_gemm_err = "the SwiGLU-backward epilogue takes the dX form (A K-major, B MN-major) on 256-column tiles";
      return -2;
    }
  }
  if (d.out == GEMM_OUT_DRELU2) {
    if constexpr (!A_MN && B_MN && BN == 256 && (MT == 1 || MT == GEMM_MT_PAIR)) {
      CUtensorMap td;  // h in, d h out: [M, N] bf16, pieces of 32 rows x 64 columns
      if (!make_tmap(&tc, d.C, d.N, d.M, d.ldc, 64, 32, false) || !make_tmap(&td, d.aux, d.N, d.M, d.ldaux, 64, 32, false))
        return -2;
      return launch_tc<BN, MT, A_MN, B_MN, EPI_DRELU2>(ta, tb, tc, td, epi, d, 1, d_status, stream);
    } else {
      g_gemm_err = "the ReLU^2-backward epilogue takes the dX form (A K-major, B MN-major) on 256-column tiles";
      return -2;
    }
  }
  if (!make_tmap(&tc, d.C, d.N, d.M, d.ldc, 32, 32, true)) return -2;
  if (d.out == GEMM_OUT_F32) {
    // One residual, K-major operands and room for the residual buffers: let TMA fetch the residual pieces.
    if constexpr (!A_MN && !B_MN && GemmCfg<BN, MT>::smem_bytes(true) <= GEMM_SMEM_LIMIT && GemmCfg<BN, MT>::stages(true) >= 3) {
      static const bool no_tma_res = getenv("ANE_B200_NO_TMA_RES") != nullptr;  // A/B measurements
      if (d.res1 != nullptr && d.res2 == nullptr && !no_tma_res) {
        CUtensorMap td;
        if (!make_tmap(&td, d.res1, d.N, d.M, d.ldres, 32, 32, true)) return -2;
        return launch_tc<BN, MT, A_MN, B_MN, EPI_STORE_F32_TMARES>(ta, tb, tc, td, epi, d, 1, d_status, stream);
      }
    }
    return launch_tc<BN, MT, A_MN, B_MN, EPI_STORE_F32>(ta, tb, tc, tc, epi, d, 1, d_status, stream);
  }
  if constexpr (GemmCfg<BN, MT>::PAIR) {
    g_gemm_err = "CTA-pair tiles are built for the non-accumulating epilogues";
    return -2;
  } else {
    return launch_tc<BN, MT, A_MN, B_MN, EPI_REDUCE_F32>(ta, tb, tc, tc, epi, d, split_k, d_status, stream);
  }
}

template <int BN, int MT>
static int dispatch_layout(const GemmDesc& d, int split_k, int* d_status, cudaStream_t stream) {
  CUtensorMap ta, tb;
  bool ok;
  if (!d.a_mn) ok = make_tmap(&ta, d.A, d.K, d.M, d.lda, GEMM_BK, GEMM_BM);
  else         ok = make_tmap(&ta, d.A, d.M, d.K, d.lda, 64, GEMM_BK);
  if (!ok) return -2;
  // K-major B: one box per CTA and stage (a CTA of a pair loads half of the tile's rows)
  if (!d.b_mn) ok = make_tmap(&tb, d.B, d.K, d.N, d.ldb, GEMM_BK, GemmCfg<BN, MT>::PAIR ? BN / 2 : BN);
  else         ok = make_tmap(&tb, d.B, d.N, d.K, d.ldb, 64, GEMM_BK);
  if (!ok) return -2;
  if constexpr (GemmCfg<BN, MT>::PAIR) {  // forward and dX forms only (A K-major)
    if (!d.a_mn && !d.b_mn) return dispatch_epi<BN, MT, false, false>(ta, tb, d, split_k, d_status, stream);
    if (!d.a_mn && d.b_mn) return dispatch_epi<BN, MT, false, true>(ta, tb, d, split_k, d_status, stream);
    g_gemm_err = "CTA-pair tiles: unsupported operand layout";
    return -2;
  } else {
  if (!d.a_mn && !d.b_mn) return dispatch_epi<BN, MT, false, false>(ta, tb, d, split_k, d_status, stream);
  if (!d.a_mn && d.b_mn) return dispatch_epi<BN, MT, false, true>(ta, tb, d, split_k, d_status, stream);
  if (d.a_mn && d.b_mn) return dispatch_epi<BN, MT, true, true>(ta, tb, d, split_k, d_status, stream);
  return dispatch_epi<BN, MT, true, false>(ta, tb, d, split_k, d_status, stream);
  }
}

// ------------------------------------------------------------------------------------------
// Tile / schedule selection.
//   128-row tiles: width by a waves x width cost (wider tiles win unless they leave the last wave
//   mostly empty; 128-wide tiles stall on shared-memory fill); accumulating GEMMs take the width that
//   pads N least and classic split-K when it fills whole waves, else stream-K.
//   256-row tiles (two A sub-tiles share each B tile: a third less shared-memory fill per FLOP, but
//   no second TMEM accumulator set, so the epilogue is not hidden): measured faster by 5-15 % when
//   the main loop is long (K >= 2048), the 256-row tiles still cover most SMs and the epilogue is
//   short (no residual; M >= 2048 for weight gradients); slower otherwise.
// ------------------------------------------------------------------------------------------
struct GemmPlan {
  int bn = 256, mt = 1, sched = 1;  // sched > 0: classic persistent with that split-K; 0: stream-K
};

static GemmPlan plan_gemm(const GemmDesc& d, int sms) {
  const int kblocks = (d.K + GEMM_BK - 1) / GEMM_BK;
  static const int force_mt = [] {
    const char* e = getenv("ANE_B200_GEMM_MT");  // 1 or 2 pins the tile height (measurements)
    return e ? atoi(e) : 0;
  }();
  GemmPlan p;
  const bool accum = d.out == GEMM_OUT_ACCUM;
  // ---- 256-row tiles
  if (force_mt != 1 && d.M > 128 && (kblocks >= 32 || force_mt == 2)) {
    const int tiles_m2 = (d.M + 255) / 256;
    int bn2 = 256;
    long pad_best = -1;
    for (int bn : {256, 192}) {  // least padding of N, ties to the wider tile
      const long pad = (long)((d.N + bn - 1) / bn) * bn;
      if (pad_best < 0 || pad < pad_best) {
        pad_best = pad;
        bn2 = bn;
      }
    }
    const long tiles2 = (long)tiles_m2 * ((d.N + bn2 - 1) / bn2);
    if (accum && d.split_k <= 0 && (d.M >= 2048 || force_mt == 2)) {
      p.mt = 2;
      p.bn = bn2;
      int split = (int)(sms / tiles2);
      int max_split = kblocks / 4;
      if (max_split < 1) max_split = 1;
      if (split > max_split) split = max_split;
      if (split < 1) split = 1;
      const long waves = (tiles2 * split + sms - 1) / sms;
      const long classic_cost = waves * ((kblocks + split - 1) / split);
      const long streamk_cost = (tiles2 * kblocks + sms - 1) / sms + 8;
      p.sched = (streamk_cost < classic_cost && tiles2 * kblocks >= 8L * sms) ? 0 : split;
      return p;
    }
    if (!accum && ((d.res1 == nullptr && d.res2 == nullptr) || force_mt == 2)) {
      // whole waves only: a last wave that is mostly empty costs more than the fill saves; and no
      // residual epilogue, which is long and would no longer hide behind the next tile
      double best_eff = 0.0;
      int best_bn = 256;
      for (int bn : {256, 192}) {
        const long t = (long)tiles_m2 * ((d.N + bn - 1) / bn);
        const long waves = (t + sms - 1) / sms;
        const double eff = (double)t / (double)(waves * sms) * ((double)d.N / (double)(((d.N + bn - 1) / bn) * bn));
        if (eff > best_eff + 1e-9) {
          best_eff = eff;
          best_bn = bn;
        }
      }
      if (force_mt == 2 || best_eff >= 0.8) {
        p.mt = 2;
        p.bn = best_bn;
        p.sched = 1;
        return p;
      }
    }
  }
  // ---- 128-row tiles
  const int tiles_m = (d.M + GEMM_BM - 1) / GEMM_BM;
  if (accum && d.split_k <= 0) {
    int best_bn = 256;
    long best_pad = -1;
    for (int bn : {256, 192, 128}) {
      const long pad = (long)((d.N + bn - 1) / bn) * bn;
      if (best_pad < 0 || pad < best_pad) {
        best_pad = pad;
        best_bn = bn;
      }
    }
    const int tiles = tiles_m * ((d.N + best_bn - 1) / best_bn);
    int split = sms / tiles;
    int max_split = kblocks / 4;
    if (max_split < 1) max_split = 1;
    if (split > max_split) split = max_split;
    if (split < 1) split = 1;
    const long waves = ((long)tiles * split + sms - 1) / sms;
    const long classic_cost = waves * ((kblocks + split - 1) / split);
    const long streamk_cost = ((long)tiles * kblocks + sms - 1) / sms + 8;
    p.bn = best_bn;
    p.sched = (streamk_cost < classic_cost) ? 0 : split;
    return p;
  }
  long best_cost = -1;
  for (int bn : {256, 192, 128}) {
    const int tiles = tiles_m * ((d.N + bn - 1) / bn);
    const int split_k = accum ? d.split_k : 1;
    const long waves = ((long)tiles * split_k + sms - 1) / sms;
    const long kb = (kblocks + split_k - 1) / split_k;
    long cost = waves * kb * bn;
    if (bn == 128) cost += cost / 3;   // fill-rate penalty of the narrow tile
    if (bn == 192) cost += cost / 10;  // a narrower tile must win clearly
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      p.bn = bn;
      p.sched = split_k;
    }
  }
  return p;
}

int gemm_bf16(const GemmDesc& d, int* d_status, cudaStream_t stream) {
  if (d.M <= 0 || d.N <= 0 || d.K <= 0) return 0;
  if (d.out == GEMM_OUT_F32 && (d.res1 || d.res2) && (d.ldres % 4 != 0 ||
      (reinterpret_cast<uintptr_t>(d.res1) & 15) != 0 || (reinterpret_cast<uintptr_t>(d.res2) & 15) != 0)) {
    g_gemm_err = "fp32 residual operands must be 16-byte aligned with ldres % 4 == 0";
    return -2;
  }
  if (d.out == GEMM_OUT_BF16_SWIGLU && (d.aux == nullptr || d.N % 128 != 0 || d.ldaux % 8 != 0 ||
                                        (reinterpret_cast<uintptr_t>(d.aux) & 15) != 0)) {
    g_gemm_err = "SwiGLU epilogue: N must be a multiple of 128 and the gate buffer 16-byte aligned with ldaux % 8 == 0";
    return -2;
  }
  if (d.out == GEMM_OUT_BF16_RELU2 && (d.aux == nullptr || d.ldaux % 8 != 0 || (reinterpret_cast<uintptr_t>(d.aux) & 15) != 0)) {
    g_gemm_err = "ReLU^2 epilogue: the gate buffer must be 16-byte aligned with ldaux % 8 == 0";
    return -2;
  }
  if (d.out == GEMM_OUT_BF16_ROPE &&
      (d.rope_cos == nullptr || d.rope_sin == nullptr || d.rope_seq <= 0 || d.rope_cols % 64 != 0 || d.alpha != 1.f ||
       (reinterpret_cast<uintptr_t>(d.rope_cos) & 15) != 0 || (reinterpret_cast<uintptr_t>(d.rope_sin) & 15) != 0)) {
    g_gemm_err = "rotary epilogue: needs 16-byte aligned cos/sin tables, rope_seq > 0, rope_cols % 64 == 0 and alpha == 1";
    return -2;
  }
  if (d.out == GEMM_OUT_DSWIGLU || d.out == GEMM_OUT_DRELU2) {
    if (d.aux == nullptr || d.a_mn || !d.b_mn || d.N % (d.out == GEMM_OUT_DRELU2 ? 64 : 32) != 0 || d.ldaux % 8 != 0 ||
        d.ldc % 8 != 0 || (reinterpret_cast<uintptr_t>(d.aux) & 15) != 0) {
      g_gemm_err = "SwiGLU / ReLU^2 backward epilogue: dX form only, N % 32 == 0 (ReLU^2: % 64), the saved activations and the "
                   "output 16-byte aligned with pitches % 8 == 0";
      return -2;
    }
    // 256-column tiles: CTA pairs when they fill their waves (the step's shape), else one CTA per tile
    const int pairs = gemm_num_sms() / 2;
    const long tiles = (long)((d.M + 255) / 256) * ((d.N + 255) / 256);
    const long waves = (tiles + pairs - 1) / pairs;
    const double eff = (double)tiles / (double)(waves * pairs);
    static const bool no_pair = [] { const char* e = getenv("ANE_B200_GEMM_PAIR"); return e && atoi(e) == 0; }();
    if (!no_pair && d.M >= 256 && eff >= 0.8) return dispatch_layout<256, GEMM_MT_PAIR>(d, 1, d_status, stream);
    return dispatch_layout<256, 1>(d, 1, d_status, stream);
  }
  if (d.out == GEMM_OUT_CE_STATS || d.out == GEMM_OUT_CE_GRAD) {
    const bool stats = d.out == GEMM_OUT_CE_STATS;
    if (d.a_mn || d.b_mn || d.tgt == nullptr || (stats && (d.ce_stats == nullptr || d.tgt_out == nullptr || d.ce_rows < d.M)) ||
        (!stats && (d.ce_lse2 == nullptr || d.ce_coef == nullptr || d.C == nullptr))) {
      g_gemm_err = "classifier-head epilogue: K-major operands, targets and the statistics / per-row buffers are required";
      return -2;
    }
    const int pairs = gemm_num_sms() / 2;
    const long tiles = (long)((d.M + 255) / 256) * ((d.N + 255) / 256);
    const long waves = (tiles + pairs - 1) / pairs;
    const double eff = (double)tiles / (double)(waves * pairs);
    static const bool no_pair = [] { const char* e = getenv("ANE_B200_GEMM_PAIR"); return e && atoi(e) == 0; }();
    if (!no_pair && d.M >= 256 && eff >= 0.8) return dispatch_layout<256, GEMM_MT_PAIR>(d, 1, d_status, stream);
    return dispatch_layout<256, 1>(d, 1, d_status, stream);
  }
  GemmPlan p = plan_gemm(d, gemm_num_sms());
  if (d.out == GEMM_OUT_BF16_SWIGLU && p.bn == 192) p.bn = 256;  // gate rows pair up two 64-column pieces
  // CTA-pair tiles (256 x 256 per two SMs, half of the B tile per CTA): measured faster than both single-CTA
  // forms when K is short (the 256-row single-CTA tile cannot hide its epilogue there) and the tiles fill the
  // pairs' waves; slower for N = 768 (96 tiles on 74 pairs) and for long K.
  static const int pair_env = [] {
    // 0: off; 128 | 192 | 256: 256-row pair tiles of that width, 512: 512 x 192 pair tiles, wherever pairs apply
    const char* e = getenv("ANE_B200_GEMM_PAIR");
    return e ? atoi(e) : -1;
  }();
  if (pair_env != 0 && d.out != GEMM_OUT_ACCUM && !d.a_mn && d.M >= 256) {
    int bn = 0;
    if (pair_env > 0) {
      bn = pair_env;
      if (bn == 192 && d.out == GEMM_OUT_BF16_SWIGLU) bn = 256;
    } else {
      const int pairs = gemm_num_sms() / 2;
      const long tiles = (long)((d.M + 255) / 256) * ((d.N + 255) / 256);
      const long waves = (tiles + pairs - 1) / pairs;
      const double eff = (double)tiles / (double)(waves * pairs) * ((double)d.N / (double)(((d.N + 255) / 256) * 256));
      const int kblocks = (d.K + GEMM_BK - 1) / GEMM_BK;
      if (kblocks < 32 && eff >= 0.85) {
        bn = 256;
      } else if (d.out != GEMM_OUT_BF16_SWIGLU) {
        // 512 x 192 tiles (two sub-tiles per CTA, one accumulator set): the least fill per FLOP.  For the
        // N = 768 shapes they make one wave of 64 tiles; measured faster than the single-CTA 256-row tile for
        // K >= 2048 and for the short-K bf16 store, slower for the short-K residual epilogue (which is exposed).
        const long tiles2 = (long)((d.M + 511) / 512) * ((d.N + 191) / 192);
        const long waves2 = (tiles2 + pairs - 1) / pairs;
        const double eff2 =
            (double)tiles2 / (double)(waves2 * pairs) * ((double)d.N / (double)(((d.N + 191) / 192) * 192));
        const bool exposed_residual = kblocks < 32 && (d.res1 != nullptr || d.res2 != nullptr);
        if (eff2 >= 0.85 && !exposed_residual) bn = 512;
      }
    }
    if (bn == 512 && d.out != GEMM_OUT_BF16_SWIGLU) return dispatch_layout<192, GEMM_MT_PAIR2>(d, 1, d_status, stream);
    if (bn == 256) return dispatch_layout<256, GEMM_MT_PAIR>(d, 1, d_status, stream);
    if (bn == 192) return dispatch_layout<192, GEMM_MT_PAIR>(d, 1, d_status, stream);
    if (bn == 128) return dispatch_layout<128, GEMM_MT_PAIR>(d, 1, d_status, stream);
  }
  if (p.mt == 2) {
    if (p.bn == 256) return dispatch_layout<256, 2>(d, p.sched, d_status, stream);
    return dispatch_layout<192, 2>(d, p.sched, d_status, stream);
  }
  if (p.bn == 256) return dispatch_layout<256, 1>(d, p.sched, d_status, stream);
  if (p.bn == 192) return dispatch_layout<192, 1>(d, p.sched, d_status, stream);
  return dispatch_layout<128, 1>(d, p.sched, d_status, stream);
}

// ------------------------------------------------------------------------------------------
// Grouped accumulating products: C_p += A_p^T B_p for up to four problems with one contraction length, both
// operands stored [K, .] (the weight gradients of a layer), one stream-K launch over the concatenated tiles
// of 256 x 256.  `slot` is device memory for the group's descriptors; it is filled on the first call for a
// given slot (`*built`) and reused afterwards -- the operands of a layer never move.
// ------------------------------------------------------------------------------------------
int gemm_bf16_grouped(const GemmDesc* ds, int n, void* slot, bool* built, int* d_status, cudaStream_t stream) {
  if (n < 1 || n > 4 || slot == nullptr || built == nullptr) {
    g_gemm_err = "grouped GEMM: one to four problems and a descriptor slot are required";
    return -2;
  }
  constexpr int BN = 256, MT = 2;
  constexpr int BM_TILE = GemmCfg<BN, MT>::BM_TILE;
  int K = ds[0].K;
  long tiles = 0;
  for (int p = 0; p < n; ++p) {
    const GemmDesc& d = ds[p];
    if (!d.a_mn || !d.b_mn || d.out != GEMM_OUT_ACCUM || d.K != K || d.alpha != 1.f || d.M <= 0 || d.N <= 0) {
      g_gemm_err = "grouped GEMM: every problem must be C += A^T B with MN-major operands, alpha 1 and the same K";
      return -2;
    }
    tiles += (long)((d.M + BM_TILE - 1) / BM_TILE) * ((d.N + BN - 1) / BN);
  }
  if (!*built) {
    GemmGroup g;
    memset(&g, 0, sizeof g);
    g.n = n;
    int t0 = 0;
    for (int p = 0; p < n; ++p) {
      const GemmDesc& d = ds[p];
      if (!make_tmap(&g.a[p], d.A, d.M, d.K, d.lda, 64, GEMM_BK) || !make_tmap(&g.b[p], d.B, d.N, d.K, d.ldb, 64, GEMM_BK) ||
          !make_tmap(&g.c[p], d.C, d.N, d.M, d.ldc, 32, 32, true))
        return -2;
      g.M[p] = d.M;
      g.N[p] = d.N;
      g.tile0[p] = t0;
      t0 += ((d.M + BM_TILE - 1) / BM_TILE) * ((d.N + BN - 1) / BN);
    }
    g.tile0[n] = t0;
    // synchronous copy: the descriptors must be in place before the launch below and the source is on the stack
    if (cudaMemcpy(slot, &g, sizeof g, cudaMemcpyHostToDevice) != cudaSuccess) {
      g_gemm_err = "grouped GEMM: descriptor upload failed";
      return -3;
    }
    *built = true;
  }
  auto kern = gemm_tc_kernel<BN, MT, true, true, EPI_REDUCE_F32>;
  constexpr uint32_t smem_bytes = GemmCfg<BN, MT>::smem_bytes(false);
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes) != cudaSuccess) {
      g_gemm_err = "grouped GEMM: cudaFuncSetAttribute failed";
      return -3;
    }
    attr_set = true;
  }
  const long long units = (long long)tiles * ((K + GEMM_BK - 1) / GEMM_BK);
  long long grid = units / 8;
  if (grid > gemm_num_sms()) grid = gemm_num_sms();
  if (grid < 1) grid = 1;
  CUtensorMap ta, tb, tc;  // the kernel's own map parameters are not used by a grouped launch; any valid maps do
  const GemmDesc& d0 = ds[0];
  if (!make_tmap(&ta, d0.A, d0.M, d0.K, d0.lda, 64, GEMM_BK) || !make_tmap(&tb, d0.B, d0.N, d0.K, d0.ldb, 64, GEMM_BK) ||
      !make_tmap(&tc, d0.C, d0.N, d0.M, d0.ldc, 32, 32, true))
    return -2;
  EpiParams epi{};
  epi.alpha = 1.f;
  cudaError_t e = launch_pdl(kern, dim3((unsigned)grid), dim3(GEMM_THREADS), smem_bytes, stream, ta, tb, tc, tc, epi, d0.M, d0.N,
                             K, 0, d_status, reinterpret_cast<const GemmGroup*>(slot));
  if (e != cudaSuccess) {
    g_gemm_err = std::string("grouped GEMM launch: ") + cudaGetErrorString(e);
    return -4;
  }
  return 0;
}
size_t gemm_group_slot_bytes() { return sizeof(GemmGroup); }

// ------------------------------------------------------------------------------------------
// Split-precision GEMM: fp32 operands as bf16 (hi, lo) pairs, three tensor-core products.
// ------------------------------------------------------------------------------------------
// src [rows, cols] fp32 with row pitch ld  ->  hi, lo [rows, ldo] bf16 (ldo >= cols, a multiple of 8)
__global__ void split_rows_kernel(const float* __restrict__ src, bf16* __restrict__ hi, bf16* __restrict__ lo, int rows,
                                  int cols, long long ld, int ldo) {
  const long long total = (long long)rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / cols), c = (int)(i - (long long)r * cols);
    const float x = src[(size_t)r * ld + c];
    const bf16 h = __float2bfloat16_rn(x);
    hi[(size_t)r * ldo + c] = h;
    lo[(size_t)r * ldo + c] = __float2bfloat16_rn(x - __bfloat162float(h));
  }
}

void SplitScratch::release() {
  for (int i = 0; i < 4; ++i) {
    if (buf[i]) cudaFree(buf[i]);
    buf[i] = nullptr;
    cap[i] = 0;
  }
}

int gemm_bf16x3(const GemmDesc& d, SplitScratch* sc, int* d_status, cudaStream_t stream) {
  if (d.M <= 0 || d.N <= 0 || d.K <= 0) return 0;
  if (d.out != GEMM_OUT_F32 && d.out != GEMM_OUT_ACCUM) {
    g_gemm_err = "split-precision GEMM writes fp32 (store or accumulate) only";
    return -2;
  }
  // stored shapes of the operands
  const int a_rows = d.a_mn ? d.K : d.M, a_cols = d.a_mn ? d.M : d.K;
  const int b_rows = d.b_mn ? d.K : d.N, b_cols = d.b_mn ? d.N : d.K;
  const int lda = (a_cols + 7) / 8 * 8, ldb = (b_cols + 7) / 8 * 8;
  const size_t need[4] = {(size_t)a_rows * lda * 2, (size_t)a_rows * lda * 2, (size_t)b_rows * ldb * 2, (size_t)b_rows * ldb * 2};
  for (int i = 0; i < 4; ++i) {
    if (sc->cap[i] >= need[i]) continue;
    // the previous, smaller buffer may still be read by GEMMs in flight on this stream
    if (sc->buf[i]) {
      cudaStreamSynchronize(stream);
      cudaFree(sc->buf[i]);
      sc->buf[i] = nullptr;
      sc->cap[i] = 0;
    }
    const size_t bytes = need[i] + need[i] / 4 + 256;
    if (cudaMalloc(&sc->buf[i], bytes) != cudaSuccess) {
      g_gemm_err = "split-precision GEMM: out of memory for the operand halves";
      return -3;
    }
    sc->cap[i] = bytes;
  }
  bf16* ah = reinterpret_cast<bf16*>(sc->buf[0]);
  bf16* al = reinterpret_cast<bf16*>(sc->buf[1]);
  bf16* bh = reinterpret_cast<bf16*>(sc->buf[2]);
  bf16* bl = reinterpret_cast<bf16*>(sc->buf[3]);
  auto grid = [](long long n) {
    long long g = (n + 255) / 256;
    return (unsigned)(g > 148LL * 16 ? 148LL * 16 : (g < 1 ? 1 : g));
  };
  split_rows_kernel<<<grid((long long)a_rows * a_cols), 256, 0, stream>>>(reinterpret_cast<const float*>(d.A), ah, al, a_rows,
                                                                          a_cols, d.lda, lda);
  split_rows_kernel<<<grid((long long)b_rows * b_cols), 256, 0, stream>>>(reinterpret_cast<const float*>(d.B), bh, bl, b_rows,
                                                                          b_cols, d.ldb, ldb);
  if (cudaGetLastError() != cudaSuccess) {
    g_gemm_err = "split-precision GEMM: operand split launch failed";
    return -4;
  }
  GemmDesc g = d;  // the large term keeps the output kind (store with residuals, or accumulate)
  g.A = ah; g.B = bh; g.lda = lda; g.ldb = ldb;
  int rc = gemm_bf16(g, d_status, stream);
  if (rc != 0) return rc;
  GemmDesc c = g;  // the two cross terms accumulate on top
  c.out = GEMM_OUT_ACCUM;
  c.res1 = c.res2 = nullptr;
  c.s1 = c.s2 = nullptr;
  c.split_k = 0;
  c.B = bl;
  if ((rc = gemm_bf16(c, d_status, stream)) != 0) return rc;
  c.A = al;
  c.B = bh;
  return gemm_bf16(c, d_status, stream);
}

// ------------------------------------------------------------------------------------------
// fp32 SIMT GEMM (parity mode).  64x64x16 tiles, 256 threads, 4x4 micro-tiles.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M, int N,
                int K, int lda, int ldb, int ldc, int a_mn, int b_mn, int out, float alpha,
                const float* __restrict__ res1, const float* __restrict__ s1, const float* __restrict__ res2,
                const float* __restrict__ s2, int ldres) {
  __shared__ float As[16][65];
  __shared__ float Bs[16][65];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int idx = threadIdx.x; idx < 64 * 16; idx += 256) {
      int kk, mm;
      if (a_mn) { mm = idx & 63; kk = idx >> 6; } else { kk = idx & 15; mm = idx >> 4; }
      const int gm = m0 + mm, gk = k0 + kk;
      float v = 0.f;
      if (gm < M && gk < K) v = a_mn ? A[(size_t)gk * lda + gm] : A[(size_t)gm * lda + gk];
      As[kk][mm] = v;
      int nn;
      if (b_mn) { nn = idx & 63; kk = idx >> 6; } else { kk = idx & 15; nn = idx >> 4; }
      const int gn = n0 + nn;
      const int gk2 = k0 + kk;
      v = 0.f;
      if (gn < N && gk2 < K) v = b_mn ? B[(size_t)gk2 * ldb + gn] : B[(size_t)gn * ldb + gk2];
      Bs[kk][nn] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  float a1 = 0.f, a2 = 0.f;
  if (res1) a1 = s1 ? *s1 : 1.f;
  if (res2) a2 = s2 ? *s2 : 1.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = alpha * acc[i][j];
      if (out == GEMM_OUT_ACCUM) {
        C[(size_t)m * ldc + n] += v;
      } else {
        if (res1) v += a1 * res1[(size_t)m * ldres + n];
        if (res2) v += a2 * res2[(size_t)m * ldres + n];
        C[(size_t)m * ldc + n] = v;
      }
    }
  }
}

int gemm_f32(const GemmDesc& d, cudaStream_t stream) {
  if (d.M <= 0 || d.N <= 0 || d.K <= 0) return 0;
  if (d.out == GEMM_OUT_BF16) {
    g_gemm_err = "fp32 GEMM cannot write bf16";
    return -2;
  }
  dim3 grid((d.N + 63) / 64, (d.M + 63) / 64);
  gemm_f32_kernel<<<grid, 256, 0, stream>>>(
      reinterpret_cast<const float*>(d.A), reinterpret_cast<const float*>(d.B), reinterpret_cast<float*>(d.C),
      d.M, d.N, d.K, d.lda, d.ldb, d.ldc, d.a_mn ? 1 : 0, d.b_mn ? 1 : 0, d.out, d.alpha, d.res1, d.s1, d.res2,
      d.s2, d.ldres);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    g_gemm_err = std::string("gemm_f32 launch: ") + cudaGetErrorString(e);
    return -4;
  }
  return 0;
}

}  // namespace ane
