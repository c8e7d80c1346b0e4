// Engine interface behind the C ABI (one implementation per compute dtype).
#pragma once

#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/ane_b200.h"

namespace ane {

class EngineBase {
 public:
  virtual ~EngineBase() {}
  virtual int open(const ane_options& o, const uint16_t* tokens, uint64_t n_tokens, const uint8_t* dp_id) = 0;
  // input == nullptr: sample windows with the engine's drand48 sampler.
  virtual int step(const uint16_t* input, const uint16_t* target, uint32_t n_seq, ane_step_result* out) = 0;
  virtual int flush(double* refresh_ms) = 0;
  virtual int eval_logits(const uint16_t* tokens, uint32_t n_seq, float* out, uint64_t cap, uint32_t layout) = 0;
  virtual int eval_loss(const uint16_t* tokens, uint32_t n_seq, double* loss_sum, uint64_t* n_pos) = 0;
  virtual int decode(const uint16_t* prompts, uint32_t n_seq, uint32_t prompt_len, uint32_t n_new, float temperature,
                     const double* uniforms, uint16_t* out) = 0;
  virtual int set_lr(float lr) = 0;
  virtual float get_lr() = 0;
  virtual int get_state(ane_state* s) = 0;
  virtual int set_state(const ane_state* s) = 0;
  virtual int reseed(int64_t seed) = 0;
  virtual int64_t tensor_size(uint32_t id, uint32_t layer) = 0;
  virtual int import_tensor(uint32_t id, uint32_t layer, uint32_t which, const float* buf, uint64_t n) = 0;
  virtual int export_tensor(uint32_t id, uint32_t layer, uint32_t which, float* buf, uint64_t n) = 0;
  virtual int64_t get_tap(uint32_t tap, uint32_t layer, float* buf, uint64_t cap) = 0;
  // Per-GEMM device timing (CUDA events around every GEMM launch) for roofline reports.
  virtual int profile_gemm(int enable) = 0;
  virtual int profile_read(double* gemm_ms, double* gemm_flops, uint64_t* gemm_launches) = 0;
  // CUDA-event timer on the engine's own stream.
  virtual int timer_begin() = 0;
  virtual int timer_end(float* ms) = 0;

  const std::string& last_error() const { return err_; }
  uint64_t launches() const { return launches_; }

 protected:
  void count_launch(int n = 1) { launches_ += (uint64_t)n; }
  std::string err_;
  uint64_t launches_ = 0;
};

EngineBase* create_engine(int compute_dtype);

void sample_windows(uint64_t* rng, uint64_t n_tokens, uint32_t seq, uint32_t batch, uint32_t rank, uint32_t world,
                    uint64_t* out_pos);

}  // namespace ane
