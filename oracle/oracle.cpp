// CPU oracle for the training step -- TEST INFRASTRUCTURE ONLY (see oracle.h).
//
// Every function cites the reference source it restates.  Arithmetic types and
// per-element summation order follow the pure-Go path that runs when the
// accelerator hooks return false (ane/accel_stub.go, ane/stories/gemm_stub.go):
// float32 sums in the GEMM loops, float64 inside norm / softmax / lambda
// reductions.  Loops are re-nested so the inner loop runs over the contiguous
// `seq` axis where that leaves each output's summation order unchanged.
//
// PARITY UNPINNED: no golden vectors exist in the reference for this path.
#include "oracle.h"

#include <math.h>
#include <omp.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <vector>

namespace {

typedef std::vector<float> vecf;

int g_ref_threading = 0;
int g_threads = 1;  // set by orc_set_num_threads; 1 until the host side picks a count

// Loops the reference itself spreads over cores (parallelFor / parallelForCF /
// compileParallel) are always parallel; the others only when not imitating the
// reference's threading.
#define PAR_REF _Pragma("omp parallel for schedule(static) num_threads(g_threads)")
#define PAR_ALL _Pragma("omp parallel for schedule(static) num_threads(g_ref_threading ? 1 : g_threads)")
#define PAR_DW _Pragma("omp parallel for schedule(static) num_threads(g_ref_threading ? std::min(4, g_threads) : g_threads)")

// ---------------------------------------------------------------------------------------------
// Primitives
// ---------------------------------------------------------------------------------------------

// ane/stories/cpu.go:41-72 EmbedLookup: out-of-range token ids give a zero column.
void embed_lookup(float* out, const float* embed, const uint16_t* tokens, int vocab, int dim, int seq) {
  PAR_REF
  for (int t = 0; t < seq; ++t) {
    int tok = tokens[t];
    if (tok < 0 || tok >= vocab) {
      for (int d = 0; d < dim; ++d) out[(size_t)d * seq + t] = 0.f;
      continue;
    }
    const float* row = embed + (size_t)tok * dim;
    for (int d = 0; d < dim; ++d) out[(size_t)d * seq + t] = row[d];
  }
}

// ane/stories/cpu.go:74-95 EmbedBackward: serial scatter-add in token order.
void embed_backward(float* d_embed, const float* dx, const uint16_t* tokens, int vocab, int dim, int seq) {
  for (int t = 0; t < seq; ++t) {
    int tok = tokens[t];
    if (tok < 0 || tok >= vocab) continue;
    float* row = d_embed + (size_t)tok * dim;
    for (int d = 0; d < dim; ++d) row[d] += dx[(size_t)d * seq + t];
  }
}

// ane/common.go:107-128 rmsNormCF (weighted) and :153-174 rmsNormNoWeightCF:
// sum of squares in float64, scale cast to float32, float32 multiplies.
void rmsnorm_cf(float* out, const float* x, const float* w, int dim, int seq) {
  PAR_REF
  for (int t = 0; t < seq; ++t) {
    double sum = 0.0;
    for (int i = 0; i < dim; ++i) {
      double v = (double)x[(size_t)i * seq + t];
      sum += v * v;
    }
    float scale = (float)(1.0 / sqrt(sum / (double)dim + 1e-5));
    if (w) {
      for (int i = 0; i < dim; ++i) out[(size_t)i * seq + t] = x[(size_t)i * seq + t] * scale * w[i];
    } else {
      for (int i = 0; i < dim; ++i) out[(size_t)i * seq + t] = x[(size_t)i * seq + t] * scale;
    }
  }
}

// ane/stories/cpu.go:97-111 RMSNorm and :113-127 RMSNormNoWeight (used for the
// final norm): multiply in float64, cast once.
void rmsnorm_final(float* out, const float* x, const float* w, int dim, int seq) {
  PAR_REF
  for (int t = 0; t < seq; ++t) {
    double sum = 0.0;
    for (int i = 0; i < dim; ++i) {
      double v = (double)x[(size_t)i * seq + t];
      sum += v * v;
    }
    double rrms = 1.0 / sqrt(sum / (double)dim + 1e-5);
    if (w) {
      for (int i = 0; i < dim; ++i)
        out[(size_t)i * seq + t] = (float)((double)x[(size_t)i * seq + t] * rrms * (double)w[i]);
    } else {
      for (int i = 0; i < dim; ++i) out[(size_t)i * seq + t] = (float)((double)x[(size_t)i * seq + t] * rrms);
    }
  }
}

// ane/common.go:176-197 rmsNormNoWeightBackwardCF == ane/stories/cpu.go:129-150:
// everything in float64, one cast at the store.
// With weights (Llama-style configs) this is the exact gradient of y = x*rrms*w:
//   dx = rrms*(w*dy) - x * rrms^3/D * sum(w*dy*x);  dw += dy*x*rrms.
// The reference's own weighted variant (ane/stories/cpu.go:152-210) multiplies the
// second term by w as well, which is not the gradient of its forward; it is unused
// by the reference's training path and is not reproduced.
void rmsnorm_bwd(float* dx, float* dw, const float* dy, const float* x, const float* w, int dim, int seq) {
  const double inv_d = 1.0 / (double)dim;
  PAR_REF
  for (int t = 0; t < seq; ++t) {
    double sum = 0.0;
    for (int i = 0; i < dim; ++i) {
      double v = (double)x[(size_t)i * seq + t];
      sum += v * v;
    }
    double rrms = 1.0 / sqrt(sum * inv_d + 1e-5);
    double dot = 0.0;
    if (w) {
      for (int i = 0; i < dim; ++i)
        dot += (double)dy[(size_t)i * seq + t] * (double)w[i] * (double)x[(size_t)i * seq + t];
    } else {
      for (int i = 0; i < dim; ++i) dot += (double)dy[(size_t)i * seq + t] * (double)x[(size_t)i * seq + t];
    }
    double coeff = dot * rrms * rrms * rrms * inv_d;
    for (int i = 0; i < dim; ++i) {
      size_t idx = (size_t)i * seq + t;
      double g = (double)dy[idx];
      if (w) g *= (double)w[i];
      dx[idx] = (float)(g * rrms - coeff * (double)x[idx]);
    }
  }
  if (w && dw) {
    // dw[i] += sum_t dy*x*rrms, float64 per channel.
    PAR_ALL
    for (int i = 0; i < dim; ++i) {
      double acc = 0.0;
      for (int t = 0; t < seq; ++t) {
        double s = 0.0;
        for (int j = 0; j < dim; ++j) {
          double v = (double)x[(size_t)j * seq + t];
          s += v * v;
        }
        double rrms = 1.0 / sqrt(s * inv_d + 1e-5);
        acc += (double)dy[(size_t)i * seq + t] * (double)x[(size_t)i * seq + t] * rrms;
      }
      dw[i] += (float)acc;
    }
  }
}

// Faster dw path used by the model (rrms per token computed once); same values as above.
void rmsnorm_bwd_model(float* dx, float* dw, const float* dy, const float* x, const float* w, int dim, int seq) {
  rmsnorm_bwd(dx, nullptr, dy, x, w, dim, seq);
  if (!(w && dw)) return;
  const double inv_d = 1.0 / (double)dim;
  std::vector<double> rr(seq);
  for (int t = 0; t < seq; ++t) {
    double s = 0.0;
    for (int j = 0; j < dim; ++j) {
      double v = (double)x[(size_t)j * seq + t];
      s += v * v;
    }
    rr[t] = 1.0 / sqrt(s * inv_d + 1e-5);
  }
  PAR_ALL
  for (int i = 0; i < dim; ++i) {
    double acc = 0.0;
    for (int t = 0; t < seq; ++t) acc += (double)dy[(size_t)i * seq + t] * (double)x[(size_t)i * seq + t] * rr[t];
    dw[i] += (float)acc;
  }
}

// ane/common.go:91-105 linearCF: out[o,t] = sum_i W[o,i]*in[i,t], float32 sum, i ascending.
void linear_cf(float* out, const float* w, const float* in, int out_ch, int in_ch, int seq) {
  PAR_ALL
  for (int o = 0; o < out_ch; ++o) {
    const float* row = w + (size_t)o * in_ch;
    float* acc = out + (size_t)o * seq;
    for (int t = 0; t < seq; ++t) acc[t] = 0.f;
    for (int i = 0; i < in_ch; ++i) {
      const float wi = row[i];
      const float* xi = in + (size_t)i * seq;
      for (int t = 0; t < seq; ++t) acc[t] += wi * xi[t];
    }
  }
}

// ane/train_full.go:242-259 linearBackwardDXCF: dx[i,t] = sum_o W[o,i]*dy[o,t], o ascending.
void linear_dx_cf(float* dx, const float* w, const float* dy, int out_ch, int in_ch, int seq) {
  PAR_ALL
  for (int i = 0; i < in_ch; ++i) {
    float* row = dx + (size_t)i * seq;
    for (int t = 0; t < seq; ++t) row[t] = 0.f;
    for (int o = 0; o < out_ch; ++o) {
      const float weight = w[(size_t)o * in_ch + i];
      const float* dy_row = dy + (size_t)o * seq;
      for (int t = 0; t < seq; ++t) row[t] += weight * dy_row[t];
    }
  }
}

// ane/train_full.go:213-229 accumLinearGradCF: dW[o,i] += sum_t dy[o,t]*x[i,t] (float32 local sum).
void linear_dw_cf(float* dw, const float* dy, const float* x, int out_ch, int in_ch, int seq) {
  PAR_DW
  for (int o = 0; o < out_ch; ++o) {
    float* row = dw + (size_t)o * in_ch;
    const float* dy_row = dy + (size_t)o * seq;
    for (int i = 0; i < in_ch; ++i) {
      const float* x_row = x + (size_t)i * seq;
      float sum = 0.f;
      for (int t = 0; t < seq; ++t) sum += dy_row[t] * x_row[t];
      row[i] += sum;
    }
  }
}

// ane/train_util.go:183-202 buildRoPETables (theta is 100000 there; a parameter here).
void build_rope(vecf& c, vecf& s, int seq, int head_dim, double theta) {
  int half = head_dim / 2;
  c.assign((size_t)seq * half, 0.f);
  s.assign((size_t)seq * half, 0.f);
  for (int pos = 0; pos < seq; ++pos)
    for (int i = 0; i < half; ++i) {
      double freq = (double)pos / pow(theta, (double)(2 * i) / (double)head_dim);
      c[(size_t)pos * half + i] = (float)cos(freq);
      s[(size_t)pos * half + i] = (float)sin(freq);
    }
}

// ane/train_util.go:204-224 applyRoPECFInPlace: interleaved pairs (2i, 2i+1).
// inverse = rotate by -angle (the exact backward of the rotation; the reference has none).
void rope_cf(float* x, int heads, int head_dim, int seq, const float* rc, const float* rs, bool inverse) {
  int half = head_dim / 2;
  PAR_ALL
  for (int h = 0; h < heads; ++h) {
    int head_base = h * head_dim;
    for (int i = 0; i < half; ++i) {
      size_t even = (size_t)(head_base + 2 * i) * seq;
      size_t odd = even + seq;
      for (int t = 0; t < seq; ++t) {
        float c = rc[(size_t)t * half + i];
        float s = rs[(size_t)t * half + i];
        if (inverse) s = -s;
        float e = x[even + t];
        float o = x[odd + t];
        x[even + t] = e * c - o * s;
        x[odd + t] = o * c + e * s;
      }
    }
  }
}

// ane/common.go:199-227 qkNormCF (one tensor at a time; q and k are independent there).
void qknorm_one(float* q, int heads, int head_dim, int seq) {
  const double qk_scale = 1.2;
  PAR_ALL
  for (int h = 0; h < heads; ++h) {
    int base = h * head_dim;
    for (int t = 0; t < seq; ++t) {
      double sum = 0.0;
      for (int i = 0; i < head_dim; ++i) {
        double v = (double)q[(size_t)(base + i) * seq + t];
        sum += v * v;
      }
      float scale = (float)(qk_scale / sqrt(sum / (double)head_dim + 1e-5));
      for (int i = 0; i < head_dim; ++i) q[(size_t)(base + i) * seq + t] *= scale;
    }
  }
}

// ane/common.go:229-270 qkNormBackwardCF (one tensor at a time).
// The reference scales the projection term by qkScale^2 (:247,:263); the exact gradient of
// y = qkScale*x*rrms has a single qkScale there.  reference_coeff selects which.
void qknorm_bwd_one(float* dq, const float* q_pre, int heads, int head_dim, int seq, bool reference_coeff) {
  const double qk_scale = 1.2;
  const double inv_hd = 1.0 / (double)head_dim;
  PAR_ALL
  for (int h = 0; h < heads; ++h) {
    int base = h * head_dim;
    for (int t = 0; t < seq; ++t) {
      double sum = 0.0;
      for (int i = 0; i < head_dim; ++i) {
        double v = (double)q_pre[(size_t)(base + i) * seq + t];
        sum += v * v;
      }
      double rrms = 1.0 / sqrt(sum * inv_hd + 1e-5);
      double dot = 0.0;
      for (int i = 0; i < head_dim; ++i)
        dot += (double)dq[(size_t)(base + i) * seq + t] * (double)q_pre[(size_t)(base + i) * seq + t];
      double coeff = dot * rrms * rrms * rrms * inv_hd * qk_scale;
      if (reference_coeff) coeff = dot * rrms * rrms * rrms * inv_hd * qk_scale * qk_scale;
      for (int i = 0; i < head_dim; ++i) {
        size_t idx = (size_t)(base + i) * seq + t;
        dq[idx] = (float)((double)dq[idx] * rrms * qk_scale - coeff * (double)q_pre[idx]);
      }
    }
  }
}

// ane/accel_stub.go:31-48 softmaxRowAccel.
void softmax_row(float* out, const float* in, int n) {
  float maxv = in[0];
  for (int i = 1; i < n; ++i)
    if (in[i] > maxv) maxv = in[i];
  double sum = 0.0;
  for (int i = 0; i < n; ++i) {
    double e = exp((double)(in[i] - maxv));
    out[i] = (float)e;
    sum += e;
  }
  float inv = (float)(1.0 / sum);
  for (int i = 0; i < n; ++i) out[i] *= inv;
}

// ane/common.go:61-89 causalAttentionCF, extended with shared KV heads (query head h
// reads KV head h / (heads/kv_heads)); kv_heads == heads is the reference.
void attention_cf(float* out, const float* qf, const float* kf, const float* vf, int heads, int kv_heads,
                  int head_dim, int seq) {
  const float scale = (float)(1.0 / sqrt((double)head_dim));
  const int group = heads / kv_heads;
  PAR_ALL
  for (int h = 0; h < heads; ++h) {
    vecf scores(seq), probs(seq);
    int base = h * head_dim;
    int kbase = (h / group) * head_dim;
    for (int t = 0; t < seq; ++t) {
      for (int j = 0; j <= t; ++j) scores[j] = 0.f;
      for (int i = 0; i < head_dim; ++i) {
        const float qv = qf[(size_t)(base + i) * seq + t];
        const float* krow = kf + (size_t)(kbase + i) * seq;
        for (int j = 0; j <= t; ++j) scores[j] += qv * krow[j];
      }
      for (int j = 0; j <= t; ++j) scores[j] = scores[j] * scale;
      for (int j = t + 1; j < seq; ++j) scores[j] = -65504.f;
      softmax_row(probs.data(), scores.data(), seq);
      for (int i = 0; i < head_dim; ++i) {
        const float* vrow = vf + (size_t)(kbase + i) * seq;
        float sum = 0.f;
        for (int j = 0; j < seq; ++j) sum += probs[j] * vrow[j];
        out[(size_t)(base + i) * seq + t] = sum;
      }
    }
  }
}

// ane/train_full.go:261-316 causalAttentionBackwardCF with the score scale as a
// parameter (the reference hard-codes 1.0 there while its forward uses 1/sqrt(hd)).
// Parallel over KV heads so that every dk/dv element keeps its (h, t, s) update order.
void attention_bwd_cf(float* dq, float* dk, float* dv, const float* d_out, const float* q, const float* k,
                      const float* v, int heads, int kv_heads, int head_dim, int seq, float scale) {
  memset(dq, 0, sizeof(float) * (size_t)heads * head_dim * seq);
  memset(dk, 0, sizeof(float) * (size_t)kv_heads * head_dim * seq);
  memset(dv, 0, sizeof(float) * (size_t)kv_heads * head_dim * seq);
  const int group = heads / kv_heads;
  PAR_ALL
  for (int kh = 0; kh < kv_heads; ++kh) {
    vecf scores(seq), probs(seq), d_scores(seq);
    for (int h = kh * group; h < (kh + 1) * group; ++h) {
      int base = h * head_dim;
      int kbase = kh * head_dim;
      for (int t = 0; t < seq; ++t) {
        float maxv = -INFINITY;
        for (int s = 0; s <= t; ++s) scores[s] = 0.f;
        for (int i = 0; i < head_dim; ++i) {
          const float qv = q[(size_t)(base + i) * seq + t];
          const float* krow = k + (size_t)(kbase + i) * seq;
          for (int s = 0; s <= t; ++s) scores[s] += qv * krow[s];
        }
        for (int s = 0; s <= t; ++s) {
          scores[s] = scores[s] * scale;
          if (scores[s] > maxv) maxv = scores[s];
        }
        double total = 0.0;
        for (int s = 0; s <= t; ++s) {
          double e = exp((double)(scores[s] - maxv));
          probs[s] = (float)e;
          total += e;
        }
        float inv_total = (float)(1.0 / total);
        for (int s = 0; s <= t; ++s) probs[s] *= inv_total;

        for (int s = 0; s <= t; ++s) d_scores[s] = 0.f;
        for (int i = 0; i < head_dim; ++i) {
          const float dov = d_out[(size_t)(base + i) * seq + t];
          const float* vrow = v + (size_t)(kbase + i) * seq;
          for (int s = 0; s <= t; ++s) d_scores[s] += dov * vrow[s];
        }
        float ds_sum = 0.f;
        for (int s = 0; s <= t; ++s) ds_sum += probs[s] * d_scores[s];

        for (int s = 0; s <= t; ++s) {
          float ds = probs[s] * (d_scores[s] - ds_sum) * scale;
          for (int i = 0; i < head_dim; ++i) {
            size_t q_idx = (size_t)(base + i) * seq;
            size_t k_idx = (size_t)(kbase + i) * seq;
            dq[q_idx + t] += ds * k[k_idx + s];
            dk[k_idx + s] += ds * q[q_idx + t];
            dv[k_idx + s] += probs[s] * d_out[q_idx + t];
          }
        }
      }
    }
  }
}

// ane/common.go:272-287 logitSoftcap / logitSoftcapBackward.
void softcap(float* logits, size_t n) {
  const double cap = 15.0, inv_cap = 1.0 / 15.0;
  PAR_ALL
  for (size_t i = 0; i < n; ++i) logits[i] = (float)cap * (float)tanh((double)logits[i] * inv_cap);
}
void softcap_bwd(float* grad, const float* pre, size_t n) {
  const double inv_cap = 1.0 / 15.0;
  PAR_ALL
  for (size_t i = 0; i < n; ++i) {
    double t = tanh((double)pre[i] * inv_cap);
    grad[i] = grad[i] * (float)(1 - t * t);
  }
}

// ane/common.go:301-303 sigmoid32.
inline float sigmoid32(float x) { return 1.0f / (1 + (float)exp((double)(-x))); }

// ane/stories/cpu.go:212-292 CrossEntropyLoss (dLogits may alias logits).
float cross_entropy(float* d_logits, const float* logits, const uint16_t* targets, int v, int s) {
  double loss = 0.0;
  int valid = 0;
  std::vector<double> losses(s, 0.0);
  std::vector<int> valids(s, 0);
  PAR_REF
  for (int t = 0; t < s; ++t) {
    float mx = logits[t];
    for (int i = 1; i < v; ++i) {
      float val = logits[(size_t)i * s + t];
      if (val > mx) mx = val;
    }
    double sum = 0.0;
    for (int i = 0; i < v; ++i) {
      float e = (float)exp((double)(logits[(size_t)i * s + t] - mx));
      d_logits[(size_t)i * s + t] = e;
      sum += (double)e;
    }
    float inv = (float)(1.0 / sum);
    int tgt = targets[t];
    for (int i = 0; i < v; ++i) d_logits[(size_t)i * s + t] *= inv;
    if (tgt < 0 || tgt >= v) {
      for (int i = 0; i < v; ++i) d_logits[(size_t)i * s + t] = 0.f;
      continue;
    }
    float p = d_logits[(size_t)tgt * s + t];
    if (p < 1e-10f) p = 1e-10f;
    losses[t] = -log((double)p);
    d_logits[(size_t)tgt * s + t] -= 1.f;
    valids[t] = 1;
  }
  for (int t = 0; t < s; ++t) {
    loss += losses[t];
    valid += valids[t];
  }
  if (valid == 0) return 0.f;
  float inv_valid = (float)(1.0 / (double)valid);
  PAR_REF
  for (int t = 0; t < s; ++t) {
    int tgt = targets[t];
    if (tgt < 0 || tgt >= v) continue;
    for (int i = 0; i < v; ++i) d_logits[(size_t)i * s + t] *= inv_valid;
  }
  return (float)(loss / (double)valid);
}

// ane/stories/cpu.go:303-327 MatMulVocabSeq.
void matmul_vocab_seq(float* logits, const float* embed, const float* x, int vocab, int dim, int seq) {
  PAR_REF
  for (int v = 0; v < vocab; ++v) {
    const float* eb = embed + (size_t)v * dim;
    float* out = logits + (size_t)v * seq;
    for (int t = 0; t < seq; ++t) out[t] = 0.f;
    for (int d = 0; d < dim; ++d) {
      const float w = eb[d];
      const float* xd = x + (size_t)d * seq;
      for (int t = 0; t < seq; ++t) out[t] += w * xd[t];
    }
  }
}

// ane/stories/cpu.go:333-360 MatMulEmbedTScale.
void matmul_embed_t_scale(float* dx, const float* embed, const float* d_logits, int vocab, int dim, int seq,
                          float scale) {
  if (scale == 0.f) {
    memset(dx, 0, sizeof(float) * (size_t)dim * seq);
    return;
  }
  PAR_REF
  for (int d = 0; d < dim; ++d) {
    vecf acc(seq, 0.f);
    for (int v = 0; v < vocab; ++v) {
      const float w = embed[(size_t)v * dim + d];
      const float* dlv = d_logits + (size_t)v * seq;
      for (int t = 0; t < seq; ++t) acc[t] += w * dlv[t];
    }
    float* out = dx + (size_t)d * seq;
    for (int t = 0; t < seq; ++t) out[t] = acc[t] * scale;
  }
}

// ane/stories/cpu.go:366-385 MatMulGradEmbedScale (overwrites dEmbed).
void matmul_grad_embed_scale(float* d_embed, const float* d_logits, const float* x, int vocab, int dim, int seq,
                             float scale) {
  if (scale == 0.f) {
    memset(d_embed, 0, sizeof(float) * (size_t)vocab * dim);
    return;
  }
  PAR_REF
  for (int v = 0; v < vocab; ++v) {
    const float* dl = d_logits + (size_t)v * seq;
    for (int d = 0; d < dim; ++d) {
      const float* xd = x + (size_t)d * seq;
      float sum = 0.f;
      for (int t = 0; t < seq; ++t) sum += dl[t] * xd[t];
      d_embed[(size_t)v * dim + d] = sum * scale;
    }
  }
}

// ane/train_full.go:1107-1111 adamBiasCorrectionInv.
void adam_bc_inv(int t, float b1, float b2, float* inv1, float* inv2) {
  float bc1 = (float)(1.0 - pow((double)b1, (double)t));
  float bc2 = (float)(1.0 - pow((double)b2, (double)t));
  *inv1 = 1 / bc1;
  *inv2 = 1 / bc2;
}

// ane/train_full.go:1113-1150 adamUpdateCFWithInv (element order is irrelevant: elementwise).
void adam_update(float* w, const float* g, float* m, float* v, size_t n, float lr, float b1, float b2, float eps,
                 float wd, float inv_bc1, float inv_bc2) {
  PAR_REF
  for (size_t i = 0; i < n; ++i) {
    m[i] = b1 * m[i] + (1 - b1) * g[i];
    v[i] = b2 * v[i] + (1 - b2) * g[i] * g[i];
    float mh = m[i] * inv_bc1;
    float vh = v[i] * inv_bc2;
    float update = mh / ((float)sqrt((double)vh) + eps);
    if (wd != 0) update += wd * w[i];
    w[i] -= lr * update;
  }
}

// ane/accel_stub.go:88-95 sumSquaresGrad.
double sum_squares(const vecf& v) {
  double s = 0;
  for (float x : v) {
    double f = (double)x;
    s += f * f;
  }
  return s;
}
void scale_vec(vecf& v, float s) {
  for (auto& x : v) x *= s;
}
void add_vec(vecf& d, const vecf& s) {
  for (size_t i = 0; i < d.size(); ++i) d[i] += s[i];
}

// ---------------------------------------------------------------------------------------------
// Model
// ---------------------------------------------------------------------------------------------
struct LayerCache {  // ane/train_full.go:12-37
  vecf x, x_norm, q, k, v, att_out, x2, x2_norm, h1, gate, pre_mix, q_pre, k_pre, h3;
  vecf d_out, dh1, dx2, dq, dk, dv, dh3;
  vecf ve, ve_gate_act;
};

}  // namespace

struct orc_model {
  orc_config c;
  int hd, qdim, kvdim;
  bool is_n, quirks;
  // tensors[which][layer][id]; global tensors live at layer 0.
  std::vector<std::vector<vecf>> ten[4];
  std::vector<LayerCache> caches;
  vecf rope_cos, rope_sin;
  // engine scratch (ane/engine.go:118-170)
  vecf x, x0, x_pre_embed_norm, tmp_hidden, x_norm, logits, logits_pre, logits_post, dy, dx, g_embed, g_x0, x_mid,
      x_mid_fwd, final_hidden;
  vecf grad_gate, grad_h1, grad_h3, grad_x_norm, grad_x2, grad_att, grad_q, grad_k, grad_v, grad_prev;
  vecf smear_x_pre, smear_gate_pre, smear_shifted, smear_gate_act, g_smear_gate, g_smear_lambda, g_backout_lambda;
  uint32_t pending = 0, adam_t = 0;
  float lr, embed_lr, scalar_lr, lambda_lr;

  vecf& T(int which, int id, int layer = 0) { return ten[which][layer][id]; }
  bool is_ve_layer(int i) const { return is_n && (i % 2 == (c.layers - 1) % 2); }  // ane/stories/weights.go:22
};

namespace {

bool layer_tensor(int id) {
  return (id >= ORC_T_WQ && id <= ORC_T_RMS_FFN) || id == ORC_T_VE_EMBED || id == ORC_T_VE_GATE;
}

size_t tensor_size(const orc_model& m, int id, int layer) {
  const orc_config& c = m.c;
  switch (id) {
    case ORC_T_EMBED: return (size_t)c.vocab * c.dim;
    case ORC_T_WQ: return (size_t)m.qdim * c.dim;
    case ORC_T_WK: return (size_t)m.kvdim * c.dim;
    case ORC_T_WV: return (size_t)m.kvdim * c.dim;
    case ORC_T_WO: return (size_t)c.dim * m.qdim;
    case ORC_T_W1: return (size_t)c.hidden * c.dim;
    case ORC_T_W2: return (size_t)c.dim * c.hidden;
    case ORC_T_W3: return m.is_n ? 0 : (size_t)c.hidden * c.dim;
    case ORC_T_RMS_ATT: return m.is_n ? 0 : c.dim;
    case ORC_T_RMS_FFN: return m.is_n ? 0 : c.dim;
    case ORC_T_RMS_FINAL: return m.is_n ? 0 : c.dim;
    case ORC_T_VE_EMBED: return m.is_ve_layer(layer) ? (size_t)c.vocab * c.dim : 0;
    case ORC_T_VE_GATE: return m.is_ve_layer(layer) ? (size_t)c.heads * 12 : 0;  // VEGateChannels = 12
    case ORC_T_RESID_LAMBDAS: return m.is_n ? c.layers : 0;
    case ORC_T_X0_LAMBDAS: return m.is_n ? c.layers : 0;
    case ORC_T_SMEAR_GATE: return m.is_n ? (size_t)c.dim * c.dim : 0;
    case ORC_T_SMEAR_LAMBDA: return m.is_n ? 1 : 0;
    case ORC_T_BACKOUT_LAMBDA: return m.is_n ? 1 : 0;
  }
  return 0;
}

// ane/common.go:324-339 smearForwardWithSaveCF.
void smear_forward_save(orc_model& m, float* x) {
  const int dim = m.c.dim, seq = m.c.seq;
  const float lambda = m.T(ORC_W, ORC_T_SMEAR_LAMBDA)[0];
  memcpy(m.smear_x_pre.data(), x, sizeof(float) * (size_t)dim * seq);
  linear_cf(m.smear_gate_pre.data(), m.T(ORC_W, ORC_T_SMEAR_GATE).data(), m.smear_x_pre.data(), dim, dim, seq);
  for (int d = 0; d < dim; ++d)
    for (int t = 0; t < seq; ++t) {
      size_t i = (size_t)d * seq + t;
      m.smear_gate_act[i] = sigmoid32(m.smear_gate_pre[i]);
      m.smear_shifted[i] = (t == 0) ? 0.f : m.smear_x_pre[i - 1];
      x[i] += lambda * m.smear_gate_act[i] * m.smear_shifted[i];
    }
}

// ane/common.go:343-382 smearBackwardCF.
void smear_backward(orc_model& m, float* d_out) {
  const int dim = m.c.dim, seq = m.c.seq;
  const float lambda = m.T(ORC_W, ORC_T_SMEAR_LAMBDA)[0];
  double d_lambda = 0;
  vecf d_gate_pre((size_t)dim * seq);
  for (int d = 0; d < dim; ++d)
    for (int t = 0; t < seq; ++t) {
      size_t i = (size_t)d * seq + t;
      float g = m.smear_gate_act[i];
      float s = m.smear_shifted[i];
      float dy = d_out[i];
      d_lambda += (double)(dy * g * s);
      d_gate_pre[i] = dy * lambda * s * g * (1 - g);
      float d_shifted = dy * lambda * g;
      if (t > 0) d_out[i - 1] += d_shifted;
    }
  m.g_smear_lambda[0] += (float)d_lambda;
  linear_dw_cf(m.g_smear_gate.data(), d_gate_pre.data(), m.smear_x_pre.data(), dim, dim, seq);
  vecf dx_from_gate((size_t)dim * seq);
  linear_dx_cf(dx_from_gate.data(), m.T(ORC_W, ORC_T_SMEAR_GATE).data(), d_gate_pre.data(), dim, dim, seq);
  for (size_t i = 0; i < dx_from_gate.size(); ++i) d_out[i] += dx_from_gate[i];
}

// ane/train_full.go:1035-1059 veForwardCF.
void ve_forward(orc_model& m, int layer, LayerCache& cache, const uint16_t* input) {
  const int dim = m.c.dim, seq = m.c.seq, heads = m.c.heads, hd = m.hd, gc = 12;
  const vecf& ve_embed = m.T(ORC_W, ORC_T_VE_EMBED, layer);
  const vecf& ve_gate = m.T(ORC_W, ORC_T_VE_GATE, layer);
  for (int t = 0; t < seq; ++t) {
    int tok = input[t];
    // The reference indexes veEmbed[tok*dim+d] unchecked (a Go index panic for tok >= vocab); here an
    // out-of-range token reads a zero row, matching EmbedLookup's treatment (ane/stories/cpu.go:60-65).
    const bool tok_ok = tok < m.c.vocab;
    for (int d = 0; d < dim; ++d) cache.ve[(size_t)d * seq + t] = tok_ok ? ve_embed[(size_t)tok * dim + d] : 0.f;
    for (int h = 0; h < heads; ++h) {
      float gate_pre = 0.f;
      for (int cidx = 0; cidx < gc; ++cidx) gate_pre += ve_gate[h * gc + cidx] * cache.x[(size_t)cidx * seq + t];
      float act = (float)(1.0 / (1.0 + exp(-(double)gate_pre)));
      cache.ve_gate_act[(size_t)h * seq + t] = act;
      float gate = 3.0f * act;
      for (int d = h * hd; d < (h + 1) * hd; ++d) cache.v[(size_t)d * seq + t] += gate * cache.ve[(size_t)d * seq + t];
    }
  }
}

// ane/train_full.go:1062-1086 veBackwardCF.
void ve_backward(orc_model& m, int layer, LayerCache& cache, float* d_prev, const float* dv, const uint16_t* input) {
  const int dim = m.c.dim, seq = m.c.seq, heads = m.c.heads, hd = m.hd, gc = 12;
  vecf& d_ve_embed = m.T(ORC_G, ORC_T_VE_EMBED, layer);
  vecf& d_ve_gate = m.T(ORC_G, ORC_T_VE_GATE, layer);
  const vecf& ve_gate = m.T(ORC_W, ORC_T_VE_GATE, layer);
  for (int t = 0; t < seq; ++t) {
    int tok = input[t];
    for (int h = 0; h < heads; ++h) {
      float act = cache.ve_gate_act[(size_t)h * seq + t];
      float gate = 3.0f * act;
      float d_gate = 0.f;
      for (int d = h * hd; d < (h + 1) * hd; ++d) {
        float dvdt = dv[(size_t)d * seq + t];
        if (tok < m.c.vocab) d_ve_embed[(size_t)tok * dim + d] += dvdt * gate;
        d_gate += dvdt * cache.ve[(size_t)d * seq + t];
      }
      float d_gate_pre = d_gate * 3.0f * act * (1 - act);
      for (int cidx = 0; cidx < gc; ++cidx) {
        d_ve_gate[h * gc + cidx] += d_gate_pre * cache.x[(size_t)cidx * seq + t];
        d_prev[(size_t)cidx * seq + t] += d_gate_pre * ve_gate[h * gc + cidx];
      }
    }
  }
}

inline float silu32(float x) { return x * (float)(1.0 / (1.0 + exp(-(double)x))); }

// ane/train_full.go:383-453 forwardTrainingCPU (ARCH_N); the ARCH_L branches restate the
// Llama-style block from its definition with the same primitives.
float* forward_training(orc_model& m, const uint16_t* input) {
  const orc_config& c = m.c;
  const int dim = c.dim, seq = c.seq, hidden = c.hidden;
  const size_t ds = (size_t)dim * seq;
  embed_lookup(m.x.data(), m.T(ORC_W, ORC_T_EMBED).data(), input, c.vocab, dim, seq);
  if (m.is_n) {
    m.x_pre_embed_norm = m.x;
    rmsnorm_cf(m.x.data(), m.x.data(), nullptr, dim, seq);
    m.x0 = m.x;
    smear_forward_save(m, m.x.data());
  }
  float* cur = m.x.data();
  float* next = m.tmp_hidden.data();
  const int mid_layer = c.layers / 2;
  for (int i = 0; i < c.layers; ++i) {
    LayerCache& cache = m.caches[i];
    memcpy(cache.x.data(), cur, sizeof(float) * ds);
    const float* w_att = m.is_n ? nullptr : m.T(ORC_W, ORC_T_RMS_ATT, i).data();
    const float* w_ffn = m.is_n ? nullptr : m.T(ORC_W, ORC_T_RMS_FFN, i).data();
    rmsnorm_cf(cache.x_norm.data(), cache.x.data(), w_att, dim, seq);
    linear_cf(cache.q.data(), m.T(ORC_W, ORC_T_WQ, i).data(), cache.x_norm.data(), m.qdim, dim, seq);
    linear_cf(cache.k.data(), m.T(ORC_W, ORC_T_WK, i).data(), cache.x_norm.data(), m.kvdim, dim, seq);
    rope_cf(cache.q.data(), c.heads, m.hd, seq, m.rope_cos.data(), m.rope_sin.data(), false);
    rope_cf(cache.k.data(), c.kv_heads, m.hd, seq, m.rope_cos.data(), m.rope_sin.data(), false);
    if (m.is_n) {
      cache.q_pre = cache.q;
      cache.k_pre = cache.k;
      qknorm_one(cache.q.data(), c.heads, m.hd, seq);
      qknorm_one(cache.k.data(), c.kv_heads, m.hd, seq);
    }
    linear_cf(cache.v.data(), m.T(ORC_W, ORC_T_WV, i).data(), cache.x_norm.data(), m.kvdim, dim, seq);
    if (m.is_ve_layer(i)) ve_forward(m, i, cache, input);
    attention_cf(cache.att_out.data(), cache.q.data(), cache.k.data(), cache.v.data(), c.heads, c.kv_heads, m.hd, seq);
    linear_cf(next, m.T(ORC_W, ORC_T_WO, i).data(), cache.att_out.data(), dim, m.qdim, seq);
    const float rl = m.is_n ? m.T(ORC_W, ORC_T_RESID_LAMBDAS)[i] : 1.0f;
    const float xl = m.is_n ? m.T(ORC_W, ORC_T_X0_LAMBDAS)[i] : 0.0f;
    for (size_t j = 0; j < ds; ++j) cache.x2[j] = rl * cache.x[j] + next[j];
    if (xl != 0)
      for (size_t j = 0; j < ds; ++j) cache.x2[j] += xl * m.x0[j];
    rmsnorm_cf(cache.x2_norm.data(), cache.x2.data(), w_ffn, dim, seq);
    linear_cf(cache.h1.data(), m.T(ORC_W, ORC_T_W1, i).data(), cache.x2_norm.data(), hidden, dim, seq);
    if (m.is_n) {
      for (size_t j = 0; j < cache.gate.size(); ++j) {  // ane/common.go:146 reluSquared32
        float h = cache.h1[j];
        cache.gate[j] = h <= 0 ? 0.f : h * h;
      }
    } else {
      linear_cf(cache.h3.data(), m.T(ORC_W, ORC_T_W3, i).data(), cache.x2_norm.data(), hidden, dim, seq);
      for (size_t j = 0; j < cache.gate.size(); ++j) cache.gate[j] = silu32(cache.h1[j]) * cache.h3[j];
    }
    linear_cf(next, m.T(ORC_W, ORC_T_W2, i).data(), cache.gate.data(), dim, hidden, seq);
    memcpy(cache.pre_mix.data(), next, sizeof(float) * ds);
    for (size_t j = 0; j < ds; ++j) next[j] = rl * cache.x2[j] + next[j];
    if (xl != 0)
      for (size_t j = 0; j < ds; ++j) next[j] += xl * m.x0[j];
    std::swap(cur, next);
    if (m.is_n && i == mid_layer - 1) {
      memcpy(m.x_mid.data(), cur, sizeof(float) * ds);
      m.x_mid_fwd = m.x_mid;
    }
  }
  if (m.is_n) {  // ane/common.go:385-389 backoutForwardCF
    const float bl = m.T(ORC_W, ORC_T_BACKOUT_LAMBDA)[0];
    for (size_t j = 0; j < ds; ++j) cur[j] -= bl * m.x_mid[j];
  }
  memcpy(m.final_hidden.data(), cur, sizeof(float) * ds);
  return cur;
}

// ane/train_full.go:480-558 runFinalHead (CPU branches).
float run_final_head(orc_model& m, const float* final_hidden, const uint16_t* target, bool backward) {
  const orc_config& c = m.c;
  const int dim = c.dim, seq = c.seq, vocab = c.vocab;
  const float* w_final = m.is_n ? nullptr : m.T(ORC_W, ORC_T_RMS_FINAL).data();
  rmsnorm_final(m.x_norm.data(), final_hidden, w_final, dim, seq);
  matmul_vocab_seq(m.logits.data(), m.T(ORC_W, ORC_T_EMBED).data(), m.x_norm.data(), vocab, dim, seq);
  m.logits_pre = m.logits;
  if (m.is_n) softcap(m.logits.data(), m.logits.size());
  m.logits_post = m.logits;
  float loss = cross_entropy(m.logits.data(), m.logits.data(), target, vocab, seq);
  if (!backward) return loss;
  const float grad_scale = 1.0f * c.loss_scale;
  if (m.is_n) softcap_bwd(m.logits.data(), m.logits_pre.data(), m.logits.size());
  if (grad_scale == 0) std::fill(m.dy.begin(), m.dy.end(), 0.f);
  else matmul_embed_t_scale(m.dy.data(), m.T(ORC_W, ORC_T_EMBED).data(), m.logits.data(), vocab, dim, seq, grad_scale);
  matmul_grad_embed_scale(m.g_embed.data(), m.logits.data(), m.x_norm.data(), vocab, dim, seq, grad_scale);
  float* dw = m.is_n ? nullptr : m.T(ORC_G, ORC_T_RMS_FINAL).data();
  rmsnorm_bwd_model(m.dx.data(), dw, m.dy.data(), final_hidden, w_final, dim, seq);
  return loss;
}

// ane/train_full.go:691-820 backwardAndAccumulate with the CPU layer backward
// (:592-601 backwardFFNCPU, :644-675 backwardAttentionCPU).
void backward_accumulate(orc_model& m, const uint16_t* input) {
  const orc_config& c = m.c;
  const int dim = c.dim, seq = c.seq, hidden = c.hidden;
  const size_t ds = (size_t)dim * seq;
  float* d_cur = m.dx.data();
  float* d_prev = m.grad_prev.data();
  if (m.is_n) {
    // ane/common.go:393-403 backoutBackwardCF
    std::fill(m.g_backout_lambda.begin(), m.g_backout_lambda.end(), 0.f);
    double d_lambda = 0;
    for (size_t i = 0; i < ds; ++i) d_lambda -= (double)(d_cur[i] * m.x_mid[i]);
    m.g_backout_lambda[0] += (float)d_lambda;
    const float bl = m.T(ORC_W, ORC_T_BACKOUT_LAMBDA)[0];
    for (size_t i = 0; i < ds; ++i) m.x_mid[i] = -bl * d_cur[i];
    std::fill(m.g_x0.begin(), m.g_x0.end(), 0.f);
  }
  const int mid_layer = c.layers / 2;
  const float att_bwd_scale = (m.is_n && m.quirks) ? 1.0f : (float)(1.0 / sqrt((double)m.hd));
  for (int l = c.layers - 1; l >= 0; --l) {
    LayerCache& cache = m.caches[l];
    const float rl = m.is_n ? m.T(ORC_W, ORC_T_RESID_LAMBDAS)[l] : 1.0f;
    const float* w_att = m.is_n ? nullptr : m.T(ORC_W, ORC_T_RMS_ATT, l).data();
    const float* w_ffn = m.is_n ? nullptr : m.T(ORC_W, ORC_T_RMS_FFN, l).data();
    memcpy(cache.d_out.data(), d_cur, sizeof(float) * ds);
    for (size_t j = 0; j < ds; ++j) m.grad_x2[j] = d_cur[j] * rl;  // copy + scaleSlice
    // ---- FFN backward
    linear_dx_cf(m.grad_gate.data(), m.T(ORC_W, ORC_T_W2, l).data(), cache.d_out.data(), dim, hidden, seq);
    if (m.is_n) {
      for (size_t j = 0; j < m.grad_h1.size(); ++j) {  // ane/accel_stub.go:21-29
        float r = cache.h1[j];
        if (r < 0) r = 0;
        m.grad_h1[j] = m.grad_gate[j] * 2 * r;
      }
      linear_dx_cf(m.grad_x_norm.data(), m.T(ORC_W, ORC_T_W1, l).data(), m.grad_h1.data(), hidden, dim, seq);
    } else {
      for (size_t j = 0; j < m.grad_h1.size(); ++j) {
        float h = cache.h1[j];
        float sg = (float)(1.0 / (1.0 + exp(-(double)h)));
        float silu = h * sg;
        float dsilu = sg * (1.0f + h * (1.0f - sg));
        m.grad_h1[j] = m.grad_gate[j] * cache.h3[j] * dsilu;
        m.grad_h3[j] = m.grad_gate[j] * silu;
      }
      linear_dx_cf(m.grad_x_norm.data(), m.T(ORC_W, ORC_T_W1, l).data(), m.grad_h1.data(), hidden, dim, seq);
      linear_dx_cf(d_prev, m.T(ORC_W, ORC_T_W3, l).data(), m.grad_h3.data(), hidden, dim, seq);
      for (size_t j = 0; j < ds; ++j) m.grad_x_norm[j] += d_prev[j];
      cache.dh3 = m.grad_h3;
    }
    rmsnorm_bwd_model(d_prev, m.is_n ? nullptr : m.T(ORC_G, ORC_T_RMS_FFN, l).data(), m.grad_x_norm.data(),
                      cache.x2.data(), w_ffn, dim, seq);
    for (size_t j = 0; j < ds; ++j) m.grad_x2[j] += d_prev[j];
    cache.dh1 = m.grad_h1;
    cache.dx2 = m.grad_x2;
    linear_dw_cf(m.T(ORC_G, ORC_T_W2, l).data(), cache.d_out.data(), cache.gate.data(), dim, hidden, seq);
    linear_dw_cf(m.T(ORC_G, ORC_T_W1, l).data(), cache.dh1.data(), cache.x2_norm.data(), hidden, dim, seq);
    if (!m.is_n) linear_dw_cf(m.T(ORC_G, ORC_T_W3, l).data(), cache.dh3.data(), cache.x2_norm.data(), hidden, dim, seq);

    double d_rl = 0, d_xl = 0;
    float xl = 0;
    if (m.is_n) {
      for (size_t j = 0; j < ds; ++j) d_rl += (double)(d_cur[j] * cache.x2[j]);
      xl = m.T(ORC_W, ORC_T_X0_LAMBDAS)[l];
      for (size_t j = 0; j < ds; ++j) d_xl += (double)(d_cur[j] * m.x0[j]);
      for (size_t j = 0; j < ds; ++j) m.g_x0[j] += xl * d_cur[j];
    }
    // ---- attention backward
    const float* att_dx2 = cache.dx2.data();
    linear_dx_cf(m.grad_att.data(), m.T(ORC_W, ORC_T_WO, l).data(), att_dx2, dim, m.qdim, seq);
    attention_bwd_cf(m.grad_q.data(), m.grad_k.data(), m.grad_v.data(), m.grad_att.data(), cache.q.data(),
                     cache.k.data(), cache.v.data(), c.heads, c.kv_heads, m.hd, seq, att_bwd_scale);
    if (m.is_n) {
      qknorm_bwd_one(m.grad_q.data(), cache.q_pre.data(), c.heads, m.hd, seq, m.quirks);
      qknorm_bwd_one(m.grad_k.data(), cache.k_pre.data(), c.kv_heads, m.hd, seq, m.quirks);
    }
    if (!(m.is_n && m.quirks)) {  // exact backward of the rotation; absent from the reference
      rope_cf(m.grad_q.data(), c.heads, m.hd, seq, m.rope_cos.data(), m.rope_sin.data(), true);
      rope_cf(m.grad_k.data(), c.kv_heads, m.hd, seq, m.rope_cos.data(), m.rope_sin.data(), true);
    }
    linear_dx_cf(m.grad_x_norm.data(), m.T(ORC_W, ORC_T_WQ, l).data(), m.grad_q.data(), m.qdim, dim, seq);
    linear_dx_cf(d_prev, m.T(ORC_W, ORC_T_WK, l).data(), m.grad_k.data(), m.kvdim, dim, seq);
    for (size_t j = 0; j < ds; ++j) m.grad_x_norm[j] += d_prev[j];
    linear_dx_cf(d_prev, m.T(ORC_W, ORC_T_WV, l).data(), m.grad_v.data(), m.kvdim, dim, seq);
    for (size_t j = 0; j < ds; ++j) m.grad_x_norm[j] += d_prev[j];
    rmsnorm_bwd_model(d_prev, m.is_n ? nullptr : m.T(ORC_G, ORC_T_RMS_ATT, l).data(), m.grad_x_norm.data(),
                      cache.x.data(), w_att, dim, seq);
    if (m.is_ve_layer(l)) ve_backward(m, l, cache, d_prev, m.grad_v.data(), input);
    for (size_t j = 0; j < ds; ++j) d_prev[j] += rl * att_dx2[j];
    cache.dq = m.grad_q;
    cache.dk = m.grad_k;
    cache.dv = m.grad_v;
    linear_dw_cf(m.T(ORC_G, ORC_T_WO, l).data(), att_dx2, cache.att_out.data(), dim, m.qdim, seq);
    linear_dw_cf(m.T(ORC_G, ORC_T_WQ, l).data(), cache.dq.data(), cache.x_norm.data(), m.qdim, dim, seq);
    linear_dw_cf(m.T(ORC_G, ORC_T_WK, l).data(), cache.dk.data(), cache.x_norm.data(), m.kvdim, dim, seq);
    linear_dw_cf(m.T(ORC_G, ORC_T_WV, l).data(), cache.dv.data(), cache.x_norm.data(), m.kvdim, dim, seq);
    if (m.is_n) {
      for (size_t j = 0; j < ds; ++j) d_rl += (double)(att_dx2[j] * cache.x[j]);
      for (size_t j = 0; j < ds; ++j) d_xl += (double)(att_dx2[j] * m.x0[j]);
      for (size_t j = 0; j < ds; ++j) m.g_x0[j] += xl * att_dx2[j];
      m.T(ORC_G, ORC_T_RESID_LAMBDAS)[l] += (float)d_rl;
      m.T(ORC_G, ORC_T_X0_LAMBDAS)[l] += (float)d_xl;
    }
    std::swap(d_cur, d_prev);
    if (m.is_n && l == mid_layer)
      for (size_t j = 0; j < ds; ++j) d_cur[j] += m.x_mid[j];
  }
  if (m.is_n) {
    if (m.quirks) {
      // Reference order (ane/train_full.go:789-798): x0 gradient joins before smear backward.
      for (size_t j = 0; j < ds; ++j) d_cur[j] += m.g_x0[j];
    }
    std::fill(m.g_smear_gate.begin(), m.g_smear_gate.end(), 0.f);
    std::fill(m.g_smear_lambda.begin(), m.g_smear_lambda.end(), 0.f);
    smear_backward(m, d_cur);
    if (!m.quirks) {
      // x0 was taken before the smear (ane/train_full.go:390-392): exact order.
      for (size_t j = 0; j < ds; ++j) d_cur[j] += m.g_x0[j];
    }
    rmsnorm_bwd(d_prev, nullptr, d_cur, m.x_pre_embed_norm.data(), nullptr, dim, seq);
    memcpy(d_cur, d_prev, sizeof(float) * ds);
  }
  embed_backward(m.g_embed.data(), d_cur, input, c.vocab, dim, seq);
  add_vec(m.T(ORC_G, ORC_T_EMBED), m.g_embed);
  if (m.is_n) {
    add_vec(m.T(ORC_G, ORC_T_SMEAR_GATE), m.g_smear_gate);
    add_vec(m.T(ORC_G, ORC_T_SMEAR_LAMBDA), m.g_smear_lambda);
    add_vec(m.T(ORC_G, ORC_T_BACKOUT_LAMBDA), m.g_backout_lambda);
  }
  m.pending++;
}

void adam_tensor(orc_model& m, int id, int layer, float lr, float b1, float b2, float wd, float i1, float i2) {
  vecf& w = m.T(ORC_W, id, layer);
  if (w.empty()) return;
  adam_update(w.data(), m.T(ORC_G, id, layer).data(), m.T(ORC_M, id, layer).data(), m.T(ORC_V, id, layer).data(),
              w.size(), lr, b1, b2, m.c.eps, wd, i1, i2);
}

// ane/engine.go:646-682 flushPending, with ane/train_full.go:167-196 clipLayerGradients and
// :1088-1100 applyLayerAdam.  ARCH_L adds W3 and the norm weights (base LR, no decay) and
// clips over every parameter.
void flush_pending(orc_model& m) {
  const orc_config& c = m.c;
  if (m.pending == 0) return;
  float scale = (float)(1.0 / (double)m.pending);
  if (c.loss_scale > 0) scale /= c.loss_scale;
  for (int which_layer = 0; which_layer < c.layers; ++which_layer)
    for (int id = 0; id < ORC_T_COUNT; ++id)
      if (layer_tensor(id)) scale_vec(m.T(ORC_G, id, which_layer), scale);
  for (int id = 0; id < ORC_T_COUNT; ++id)
    if (!layer_tensor(id)) scale_vec(m.T(ORC_G, id, 0), scale);
  if (c.grad_clip > 0) {
    double norm2 = 0;
    for (int l = 0; l < c.layers; ++l)
      for (int id : {ORC_T_WQ, ORC_T_WK, ORC_T_WV, ORC_T_WO, ORC_T_W1, ORC_T_W2, ORC_T_VE_EMBED, ORC_T_VE_GATE,
                     ORC_T_W3, ORC_T_RMS_ATT, ORC_T_RMS_FFN})
        norm2 += sum_squares(m.T(ORC_G, id, l));
    norm2 += sum_squares(m.T(ORC_G, ORC_T_EMBED));
    norm2 += sum_squares(m.T(ORC_G, ORC_T_RMS_FINAL));
    if (norm2 > 0) {
      float norm = (float)sqrt(norm2);
      if (norm > c.grad_clip) {
        float s = c.grad_clip / norm;
        for (int l = 0; l < c.layers; ++l)
          for (int id : {ORC_T_WQ, ORC_T_WK, ORC_T_WV, ORC_T_WO, ORC_T_W1, ORC_T_W2, ORC_T_VE_EMBED, ORC_T_VE_GATE,
                         ORC_T_W3, ORC_T_RMS_ATT, ORC_T_RMS_FFN})
            scale_vec(m.T(ORC_G, id, l), s);
        scale_vec(m.T(ORC_G, ORC_T_EMBED), s);
        scale_vec(m.T(ORC_G, ORC_T_RMS_FINAL), s);
      }
    }
  }
  m.adam_t++;
  int t = (int)m.adam_t;
  float i1, i2;
  adam_bc_inv(t, c.beta1, c.beta2, &i1, &i2);
  for (int l = 0; l < c.layers; ++l) {
    for (int id : {ORC_T_WQ, ORC_T_WK, ORC_T_WV, ORC_T_WO, ORC_T_W1, ORC_T_W2, ORC_T_W3})
      adam_tensor(m, id, l, m.lr, c.beta1, c.beta2, c.weight_decay, i1, i2);
    adam_tensor(m, ORC_T_RMS_ATT, l, m.lr, c.beta1, c.beta2, 0, i1, i2);
    adam_tensor(m, ORC_T_RMS_FFN, l, m.lr, c.beta1, c.beta2, 0, i1, i2);
    adam_tensor(m, ORC_T_VE_EMBED, l, m.embed_lr, c.beta1, c.beta2, 0, i1, i2);
    adam_tensor(m, ORC_T_VE_GATE, l, m.scalar_lr, c.beta1, c.beta2, 0, i1, i2);
  }
  adam_tensor(m, ORC_T_RMS_FINAL, 0, m.lr, c.beta1, c.beta2, 0, i1, i2);
  adam_tensor(m, ORC_T_SMEAR_GATE, 0, m.lr, c.beta1, c.beta2, c.weight_decay, i1, i2);
  adam_tensor(m, ORC_T_EMBED, 0, m.embed_lr, c.beta1, c.beta2, 0, i1, i2);
  adam_tensor(m, ORC_T_SMEAR_LAMBDA, 0, m.scalar_lr, c.beta1, c.beta2, 0, i1, i2);
  adam_tensor(m, ORC_T_BACKOUT_LAMBDA, 0, m.scalar_lr, c.beta1, c.beta2, 0, i1, i2);
  float l1, l2;
  adam_bc_inv(t, c.lambda_beta1, c.lambda_beta2, &l1, &l2);
  adam_tensor(m, ORC_T_RESID_LAMBDAS, 0, m.lambda_lr, c.lambda_beta1, c.lambda_beta2, 0, l1, l2);
  adam_tensor(m, ORC_T_X0_LAMBDAS, 0, m.lambda_lr, c.lambda_beta1, c.lambda_beta2, 0, l1, l2);
  for (int l = 0; l < c.layers; ++l)
    for (auto& v : m.ten[ORC_G][l]) std::fill(v.begin(), v.end(), 0.f);
  m.pending = 0;
}

void set_lr(orc_model& m, float lr) {  // ane/engine.go:366-378 SetLR
  m.lr = lr;
  m.embed_lr = lr * m.c.embed_lr_mult;
  m.scalar_lr = lr * m.c.scalar_lr_mult;
  m.lambda_lr = lr * m.c.scalar_lr_mult * m.c.lambda_lr_mult;
}

}  // namespace

extern "C" {

orc_model* orc_create(const orc_config* cfg) {
  if (!cfg) return nullptr;
  orc_config c = *cfg;
  if (c.dim <= 0 || c.heads <= 0 || c.layers <= 0 || c.vocab <= 0 || c.hidden <= 0) return nullptr;
  if (c.kv_heads <= 0) c.kv_heads = c.heads;
  if (c.dim % c.heads != 0 || c.heads % c.kv_heads != 0 || ((c.dim / c.heads) & 1)) return nullptr;
  // ane/engine.go:188-239 defaults
  if (c.seq <= 0) c.seq = 256;
  if (c.lr <= 0) c.lr = 3e-4f;
  if (c.accum_steps <= 0) c.accum_steps = 1;
  if (c.beta1 <= 0) c.beta1 = 0.9f;
  if (c.beta2 <= 0) c.beta2 = 0.999f;
  if (c.eps <= 0) c.eps = 1e-8f;
  if (c.grad_clip < 0) c.grad_clip = 0;
  if (c.loss_scale < 0) c.loss_scale = 0;
  if (c.loss_scale == 0) c.loss_scale = 256;
  if (c.embed_lr_mult <= 0) c.embed_lr_mult = 1.0f;
  if (c.scalar_lr_mult <= 0) c.scalar_lr_mult = 1.0f;
  if (c.lambda_lr_mult <= 0) c.lambda_lr_mult = 0.01f;
  if (c.lambda_beta1 <= 0) c.lambda_beta1 = c.beta1;
  if (c.lambda_beta2 <= 0) c.lambda_beta2 = c.beta2;
  if (c.rope_theta <= 0) c.rope_theta = (c.arch == ORC_ARCH_N) ? 100000.f : 10000.f;
  orc_model* m = new orc_model();
  m->c = c;
  m->is_n = c.arch == ORC_ARCH_N;
  m->quirks = c.quirks != 0;
  if (m->is_n && c.kv_heads != c.heads) {
    delete m;
    return nullptr;
  }
  m->hd = c.dim / c.heads;
  m->qdim = c.heads * m->hd;
  m->kvdim = c.kv_heads * m->hd;
  for (int w = 0; w < 4; ++w) {
    m->ten[w].resize(c.layers);
    for (int l = 0; l < c.layers; ++l) {
      m->ten[w][l].resize(ORC_T_COUNT);
      for (int id = 0; id < ORC_T_COUNT; ++id) {
        if (!layer_tensor(id) && l != 0) continue;
        m->ten[w][l][id].assign(tensor_size(*m, id, l), 0.f);
      }
    }
  }
  if (m->is_n) {  // ane/stories/weights.go:155-162 initLambdasDefault
    for (auto& v : m->T(ORC_W, ORC_T_RESID_LAMBDAS)) v = 1.0f;
  } else {
    for (int l = 0; l < c.layers; ++l) {
      for (auto& v : m->T(ORC_W, ORC_T_RMS_ATT, l)) v = 1.0f;
      for (auto& v : m->T(ORC_W, ORC_T_RMS_FFN, l)) v = 1.0f;
    }
    for (auto& v : m->T(ORC_W, ORC_T_RMS_FINAL)) v = 1.0f;
  }
  const size_t ds = (size_t)c.dim * c.seq, hs = (size_t)c.hidden * c.seq, vs = (size_t)c.vocab * c.seq;
  const size_t qs = (size_t)m->qdim * c.seq, ks = (size_t)m->kvdim * c.seq;
  m->caches.resize(c.layers);
  for (int l = 0; l < c.layers; ++l) {
    LayerCache& lc = m->caches[l];
    for (vecf* v : {&lc.x, &lc.x_norm, &lc.att_out, &lc.x2, &lc.x2_norm, &lc.pre_mix, &lc.d_out, &lc.dx2}) v->assign(ds, 0.f);
    for (vecf* v : {&lc.q, &lc.q_pre, &lc.dq}) v->assign(qs, 0.f);
    for (vecf* v : {&lc.k, &lc.v, &lc.k_pre, &lc.dk, &lc.dv}) v->assign(ks, 0.f);
    for (vecf* v : {&lc.h1, &lc.gate, &lc.dh1, &lc.h3, &lc.dh3}) v->assign(hs, 0.f);
    if (m->is_ve_layer(l)) {
      lc.ve.assign(ds, 0.f);
      lc.ve_gate_act.assign((size_t)c.heads * c.seq, 0.f);
    }
  }
  build_rope(m->rope_cos, m->rope_sin, c.seq, m->hd, (double)c.rope_theta);
  for (vecf* v : {&m->x, &m->x0, &m->x_pre_embed_norm, &m->tmp_hidden, &m->x_norm, &m->dy, &m->dx, &m->g_x0, &m->x_mid,
                  &m->x_mid_fwd, &m->final_hidden, &m->grad_x_norm, &m->grad_x2, &m->grad_prev, &m->smear_x_pre,
                  &m->smear_gate_pre, &m->smear_shifted, &m->smear_gate_act})
    v->assign(ds, 0.f);
  m->grad_att.assign(qs, 0.f);
  m->grad_q.assign(qs, 0.f);
  m->grad_k.assign(ks, 0.f);
  m->grad_v.assign(ks, 0.f);
  for (vecf* v : {&m->grad_gate, &m->grad_h1, &m->grad_h3}) v->assign(hs, 0.f);
  for (vecf* v : {&m->logits, &m->logits_pre, &m->logits_post}) v->assign(vs, 0.f);
  m->g_embed.assign((size_t)c.vocab * c.dim, 0.f);
  m->g_smear_gate.assign(m->is_n ? (size_t)c.dim * c.dim : 0, 0.f);
  m->g_smear_lambda.assign(1, 0.f);
  m->g_backout_lambda.assign(1, 0.f);
  set_lr(*m, c.lr);
  return m;
}

void orc_destroy(orc_model* m) { delete m; }
void orc_get_config(const orc_model* m, orc_config* out) {
  if (m && out) *out = m->c;
}

float* orc_tensor(orc_model* m, int32_t id, int32_t layer, int32_t which, uint64_t* n) {
  if (n) *n = 0;
  if (!m || id < 0 || id >= ORC_T_COUNT || which < 0 || which > 3) return nullptr;
  if (!layer_tensor(id)) layer = 0;
  if (layer < 0 || layer >= m->c.layers) return nullptr;
  vecf& v = m->T(which, id, layer);
  if (n) *n = v.size();
  return v.empty() ? nullptr : v.data();
}

float* orc_tap(orc_model* m, int32_t tap, int32_t layer, uint64_t* n) {
  if (n) *n = 0;
  if (!m) return nullptr;
  vecf* v = nullptr;
  if (tap < 32) {
    if (layer < 0 || layer >= m->c.layers) return nullptr;
    LayerCache& lc = m->caches[layer];
    switch (tap) {
      case ORC_TAP_X: v = &lc.x; break;
      case ORC_TAP_XNORM: v = &lc.x_norm; break;
      case ORC_TAP_Q: v = &lc.q; break;
      case ORC_TAP_K: v = &lc.k; break;
      case ORC_TAP_V: v = &lc.v; break;
      case ORC_TAP_ATT: v = &lc.att_out; break;
      case ORC_TAP_X2: v = &lc.x2; break;
      case ORC_TAP_X2NORM: v = &lc.x2_norm; break;
      case ORC_TAP_H1: v = &lc.h1; break;
      case ORC_TAP_GATE: v = &lc.gate; break;
      case ORC_TAP_FFN_OUT: v = &lc.pre_mix; break;
      case ORC_TAP_QPRE: v = &lc.q_pre; break;
      case ORC_TAP_KPRE: v = &lc.k_pre; break;
      case ORC_TAP_H3: v = &lc.h3; break;
      case ORC_TAP_DOUT: v = &lc.d_out; break;
      case ORC_TAP_DH1: v = &lc.dh1; break;
      case ORC_TAP_DX2: v = &lc.dx2; break;
      case ORC_TAP_DQ: v = &lc.dq; break;
      case ORC_TAP_DK: v = &lc.dk; break;
      case ORC_TAP_DV: v = &lc.dv; break;
      case ORC_TAP_DH3: v = &lc.dh3; break;
    }
  } else {
    switch (tap) {
      case ORC_TAP_X0: v = &m->x0; break;
      case ORC_TAP_XMID: v = &m->x_mid_fwd; break;
      case ORC_TAP_FINAL: v = &m->final_hidden; break;
      case ORC_TAP_FINAL_NORM: v = &m->x_norm; break;
      case ORC_TAP_LOGITS_PRE: v = &m->logits_pre; break;
      case ORC_TAP_LOGITS: v = &m->logits_post; break;
      case ORC_TAP_DLOGITS: v = &m->logits; break;
      case ORC_TAP_DFINAL: v = &m->dx; break;
    }
  }
  if (!v || v->empty()) return nullptr;
  if (n) *n = v->size();
  return v->data();
}

float orc_accumulate(orc_model* m, const uint16_t* input, const uint16_t* target) {
  float* fin = forward_training(*m, input);
  float loss = run_final_head(*m, fin, target, true);
  backward_accumulate(*m, input);
  return loss;
}

void orc_flush(orc_model* m) { flush_pending(*m); }

float orc_step(orc_model* m, const uint16_t* input, const uint16_t* target) {
  float loss = orc_accumulate(m, input, target);
  if ((int)m->pending >= m->c.accum_steps) flush_pending(*m);
  return loss;
}

uint32_t orc_pending(const orc_model* m) { return m->pending; }
uint32_t orc_adam_t(const orc_model* m) { return m->adam_t; }
void orc_set_lr(orc_model* m, float lr) { set_lr(*m, lr); }

double orc_loss_only(orc_model* m, const uint16_t* input, const uint16_t* target) {
  // float64 log-softmax over the forward logits, so finite differences are not limited
  // by the float32 loss accumulation of the training path.
  float* fin = forward_training(*m, input);
  run_final_head(*m, fin, target, false);
  const int v = m->c.vocab, s = m->c.seq;
  double loss = 0;
  int valid = 0;
  for (int t = 0; t < s; ++t) {
    int tgt = target[t];
    if (tgt < 0 || tgt >= v) continue;
    double mx = -1e300;
    for (int i = 0; i < v; ++i) mx = std::max(mx, (double)m->logits_post[(size_t)i * s + t]);
    double sum = 0;
    for (int i = 0; i < v; ++i) sum += exp((double)m->logits_post[(size_t)i * s + t] - mx);
    loss -= (double)m->logits_post[(size_t)tgt * s + t] - mx - log(sum);
    valid++;
  }
  return valid ? loss / valid : 0.0;
}

// ane/engine.go:954-1038 evalLogitsCPUInto: the training forward without saves.  The two
// paths perform the same arithmetic (the eval path folds rl*cur + x2 in the other operand
// order, which is commutative in IEEE arithmetic), so the training forward is reused.
void orc_eval_logits(orc_model* m, const uint16_t* tokens, float* logits_vt) {
  float* fin = forward_training(*m, tokens);
  const orc_config& c = m->c;
  const float* w_final = m->is_n ? nullptr : m->T(ORC_W, ORC_T_RMS_FINAL).data();
  rmsnorm_final(m->x_norm.data(), fin, w_final, c.dim, c.seq);
  matmul_vocab_seq(logits_vt, m->T(ORC_W, ORC_T_EMBED).data(), m->x_norm.data(), c.vocab, c.dim, c.seq);
  if (m->is_n) softcap(logits_vt, (size_t)c.vocab * c.seq);
}

// harness.go:46-89 evalLoss for one window, with logits read as [v*seq+t] (the layout the
// engine produces) instead of the harness's [t*vocab+v].
double orc_eval_loss_window(orc_model* m, const uint16_t* tokens, int32_t* n_positions) {
  const int v = m->c.vocab, s = m->c.seq;
  vecf logits((size_t)v * s);
  orc_eval_logits(m, tokens, logits.data());
  double total = 0;
  int count = 0;
  for (int i = 0; i < s - 1; ++i) {
    int tgt = tokens[i + 1];
    if (tgt >= v) continue;
    float maxv = logits[i];
    for (int j = 1; j < v; ++j) maxv = std::max(maxv, logits[(size_t)j * s + i]);
    double sum = 0;
    for (int j = 0; j < v; ++j) sum += exp((double)(logits[(size_t)j * s + i] - maxv));
    double log_prob = (double)(logits[(size_t)tgt * s + i] - maxv) - log(sum);
    total -= log_prob;
    count++;
  }
  if (n_positions) *n_positions = count;
  return total;
}

// ane/engine.go:873-880 drand48Seed / nextFloat64 and :395-404 window sampling.
uint64_t orc_drand48_seed(int64_t seed) { return (((uint64_t)seed & 0xffffffffull) << 16) | 0x330Eull; }
uint64_t orc_sample_pos(uint64_t* rng, uint64_t n_tokens, uint32_t seq) {
  *rng = (0x5DEECE66Dull * (*rng) + 0xBull) & ((1ull << 48) - 1);
  double u = (double)(*rng) / (double)(1ull << 48);
  if (n_tokens < (uint64_t)seq + 1) return 0;
  uint64_t limit = n_tokens - seq - 1;
  uint64_t pos = 0;
  if (limit > 0) {
    pos = (uint64_t)(u * (double)limit);
    if (pos >= limit) pos = limit - 1;
  }
  return pos;
}

void orc_rmsnorm(float* out, const float* x, const float* w, int32_t dim, int32_t seq) { rmsnorm_cf(out, x, w, dim, seq); }
void orc_rmsnorm_final(float* out, const float* x, const float* w, int32_t dim, int32_t seq) {
  rmsnorm_final(out, x, w, dim, seq);
}
void orc_rmsnorm_bwd(float* dx, float* dw, const float* dy, const float* x, const float* w, int32_t dim, int32_t seq) {
  rmsnorm_bwd(dx, dw, dy, x, w, dim, seq);
}
void orc_linear(float* out, const float* w, const float* in, int32_t oc, int32_t ic, int32_t seq) {
  linear_cf(out, w, in, oc, ic, seq);
}
void orc_linear_dx(float* dx, const float* w, const float* dy, int32_t oc, int32_t ic, int32_t seq) {
  linear_dx_cf(dx, w, dy, oc, ic, seq);
}
void orc_linear_dw(float* dw, const float* dy, const float* x, int32_t oc, int32_t ic, int32_t seq) {
  linear_dw_cf(dw, dy, x, oc, ic, seq);
}
void orc_rope(float* x, int32_t heads, int32_t head_dim, int32_t seq, float theta, int32_t inverse) {
  vecf c, s;
  build_rope(c, s, seq, head_dim, (double)theta);
  rope_cf(x, heads, head_dim, seq, c.data(), s.data(), inverse != 0);
}
void orc_qknorm(float* q, float* k, int32_t dim, int32_t heads, int32_t seq) {
  qknorm_one(q, heads, dim / heads, seq);
  qknorm_one(k, heads, dim / heads, seq);
}
void orc_attention(float* out, const float* q, const float* k, const float* v, int32_t heads, int32_t kv_heads,
                   int32_t head_dim, int32_t seq) {
  attention_cf(out, q, k, v, heads, kv_heads, head_dim, seq);
}
void orc_attention_bwd(float* dq, float* dk, float* dv, const float* d_out, const float* q, const float* k,
                       const float* v, int32_t heads, int32_t kv_heads, int32_t head_dim, int32_t seq, float scale) {
  attention_bwd_cf(dq, dk, dv, d_out, q, k, v, heads, kv_heads, head_dim, seq, scale);
}
float orc_cross_entropy(float* dlogits, const float* logits, const uint16_t* targets, int32_t vocab, int32_t seq) {
  return cross_entropy(dlogits, logits, targets, vocab, seq);
}
void orc_softcap(float* logits, uint64_t n) { softcap(logits, n); }
void orc_adam(float* w, const float* g, float* m, float* v, uint64_t n, int32_t t, float lr, float b1, float b2,
              float eps, float wd) {
  float i1, i2;
  adam_bc_inv(t, b1, b2, &i1, &i2);
  adam_update(w, g, m, v, n, lr, b1, b2, eps, wd, i1, i2);
}
// ane/train_full.go:344-354 argmax: first index of the strict maximum.
int32_t orc_argmax(const float* v, int32_t n) {
  int best = 0;
  float best_val = v[0];
  for (int i = 1; i < n; ++i)
    if (v[i] > best_val) {
      best_val = v[i];
      best = i;
    }
  return best;
}

// ane/train_full.go:318-342 sampleFromLogits, with the uniform draw supplied by the caller (the reference
// takes it from Go's math/rand, which is not restated).
int32_t orc_sample(const float* logits, int32_t n, float temperature, double u) {
  if (temperature <= 1e-6f) return orc_argmax(logits, n);
  float maxv = logits[0];
  for (int i = 1; i < n; ++i)
    if (logits[i] > maxv) maxv = logits[i];
  const double inv_temp = (double)(1 / temperature);
  double total = 0.0;
  for (int i = 0; i < n; ++i) total += exp(((double)logits[i] - (double)maxv) * inv_temp);
  const double target = u * total;
  double acc = 0.0;
  for (int i = 0; i < n; ++i) {
    acc += exp(((double)logits[i] - (double)maxv) * inv_temp);
    if (acc >= target) return i;
  }
  return n - 1;
}

void orc_set_reference_threading(int32_t on) { g_ref_threading = on ? 1 : 0; }
int32_t orc_num_threads(void) { return g_threads; }
void orc_set_num_threads(int32_t n) { g_threads = n < 1 ? 1 : n; }

}  // extern "C"
