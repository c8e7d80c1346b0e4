// Host-side GEMM dispatch used by the engine.
//
// One descriptor covers every dense contraction of the training step:
//   C[M,N] (op)= alpha * A*B (+ s1*res1 + s2*res2)
// with A stored [M,K] (a_mn=false) or [K,M] (a_mn=true) and B stored [N,K]
// (b_mn=false) or [K,N] (b_mn=true).  Shapes follow the reference's call sites:
// linearCF (ane/common.go:91), linearBackwardDXCF (ane/train_full.go:242),
// accumLinearGradCF (ane/train_full.go:213) and the three classifier GEMMs
// (ane/stories/cpu.go:303-385).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ane {

enum GemmOut : int {
  GEMM_OUT_BF16 = 0,    // store bf16 (bf16 path only)
  GEMM_OUT_F32 = 1,     // store fp32, optional residual blend
  GEMM_OUT_ACCUM = 2,   // C += alpha*A*B in fp32 (beta = 1)
  // store bf16 and, for C = [h1 | h3] interleaved in 32-column blocks, also gate = silu(h1) * h3 into
  // `aux` [M, N/2] (bf16, row pitch ldaux); K-major operands only, N % 64 == 0
  GEMM_OUT_BF16_SWIGLU = 3,
  // store bf16 after rotating the (even, odd) column pairs of every 64-column head below column
  // `rope_cols` by the angle of the row's position (rope_pos0 + row % rope_seq): the q|k part of a packed
  // q|k|v projection with head_dim 64.  cos/sin tables are [positions, 32] fp32.  K-major operands only.
  GEMM_OUT_BF16_ROPE = 4,
  // store bf16 and, for every row whose target column (tgt[tgt_row0 + row]) falls inside the matrix, also
  // that one element in fp32 into tgt_out[tgt_row0 + row]: classifier logits for the cross-entropy, which
  // then reads bf16 logits but takes the target logit at full precision.  K-major operands only.
  GEMM_OUT_BF16_TGT = 5,
  // store bf16 (h) and also gate = max(h, 0)^2, taken from the fp32 accumulators, into `aux` [M, N] (bf16, row
  // pitch ldaux): the reference architecture's FFN activation (ane/common.go:146).  K-major operands only.
  GEMM_OUT_BF16_RELU2 = 6,
  // SwiGLU backward fused into the product d gate = A*B [M, N]: with `aux` = h13 [M, 2N] (bf16, h1 | h3 interleaved
  // in blocks of 32 columns, row pitch ldaux) the kernel writes C = d h13 [M, 2N] in the same layout (row pitch ldc),
  //   d h1 = d gate * h3 * silu'(h1),  d h3 = d gate * silu(h1),
  // from the fp32 accumulators; d gate itself is not stored.  A K-major, B MN-major (the dX form), N % 32 == 0.
  GEMM_OUT_DSWIGLU = 7,
  // Classifier head that keeps no logits (both K-major operands, 256-column tiles).
  // CE_STATS: nothing is stored but, per row and 256-column tile, the maximum and the sum of exponentials of the
  //   (optionally soft-capped) logits in the log2 domain -> ce_stats[tile][row] (float2, ce_rows rows per tile), and
  //   the row's target logit -> tgt_out (like GEMM_OUT_BF16_TGT).
  // CE_GRAD: the product is recomputed for the vocabulary columns [ce_col0, ce_col0 + N) and
  //   C(bf16)[row, col] = ce_coef[row] * (2^(z log2e - ce_lse2[row]) - [col is the row's target]) (* d softcap).
  GEMM_OUT_CE_STATS = 8,
  GEMM_OUT_CE_GRAD = 9,
  // ReLU^2 backward fused into the product d gate = A*B [M, N]: with `aux` = h [M, N] (bf16, row pitch ldaux) the
  // kernel writes C = d h = d gate * 2 max(h, 0) (bf16, row pitch ldc) from the fp32 accumulators; d gate itself is
  // not stored (ane/common.go:146 differentiated).  A K-major, B MN-major (the dX form), N % 64 == 0.
  GEMM_OUT_DRELU2 = 10,
};

struct GemmDesc {
  const void* A = nullptr;
  const void* B = nullptr;
  void* C = nullptr;
  int M = 0, N = 0, K = 0;
  int lda = 0, ldb = 0, ldc = 0;
  bool a_mn = false, b_mn = false;
  int out = GEMM_OUT_F32;
  float alpha = 1.f;
  const float* res1 = nullptr;
  const float* s1 = nullptr;  // device scalar, nullptr => 1
  const float* res2 = nullptr;
  const float* s2 = nullptr;
  int ldres = 0;
  void* aux = nullptr;  // GEMM_OUT_BF16_SWIGLU, GEMM_OUT_BF16_RELU2: gate output
  int ldaux = 0;
  const float* rope_cos = nullptr;  // GEMM_OUT_BF16_ROPE
  const float* rope_sin = nullptr;
  int rope_seq = 0, rope_pos0 = 0, rope_cols = 0;
  const uint16_t* tgt = nullptr;  // GEMM_OUT_BF16_TGT
  float* tgt_out = nullptr;
  int tgt_row0 = 0;
  float* ce_stats = nullptr;       // GEMM_OUT_CE_STATS
  const float* ce_lse2 = nullptr;  // GEMM_OUT_CE_GRAD
  const float* ce_coef = nullptr;
  int ce_rows = 0, ce_col0 = 0;
  bool ce_softcap = false;
  int split_k = 0;  // 0 => choose
};

// bf16 operands, tcgen05 tensor cores.  Returns 0 or a negative error code.
int gemm_bf16(const GemmDesc& d, int* d_status, cudaStream_t stream);
// fp32 operands, SIMT FMA (the fp32 parity mode).
int gemm_f32(const GemmDesc& d, cudaStream_t stream);

// fp32 operands at split precision on the tensor cores: A and B are each cut into a bf16 (hi, lo) pair
// (hi = bf16(x), lo = bf16(x - hi): together ~16 significand bits) and the product is formed as the three
// bf16 GEMMs Ah*Bh + Ah*Bl + Al*Bh accumulated in fp32 (the dropped Al*Bl term is ~2^-18 relative).  Output
// kinds GEMM_OUT_F32 (with residuals) and GEMM_OUT_ACCUM.  The scratch holds the four operand halves and
// grows on demand; one scratch serves one stream at a time.
struct SplitScratch {
  void* buf[4] = {nullptr, nullptr, nullptr, nullptr};  // A hi, A lo, B hi, B lo
  size_t cap[4] = {0, 0, 0, 0};                         // bytes
  void release();
};
int gemm_bf16x3(const GemmDesc& d, SplitScratch* scratch, int* d_status, cudaStream_t stream);

// Up to four accumulating products C_p += A_p^T B_p (both operands stored [K, .], the same K: the weight gradients of
// one layer) in one stream-K launch.  `slot` = gemm_group_slot_bytes() of device memory (64-byte aligned) that keeps
// the group's descriptors; `*built` says whether it already holds them (the operands of a slot must not change).
int gemm_bf16_grouped(const GemmDesc* ds, int n, void* slot, bool* built, int* d_status, cudaStream_t stream);
size_t gemm_group_slot_bytes();

int gemm_num_sms();
// 2-D tensor map over a row-major [outer, inner] buffer (row pitch ld elements) of bf16 (or fp32) with a
// 128B-swizzled [box_outer, box_inner] box; cached per (device, arguments).  False + gemm_last_error() on failure.
bool make_tmap_2d(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                  uint32_t box_outer, bool is_f32);
const char* gemm_last_error();

}  // namespace ane
