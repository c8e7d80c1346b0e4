// extern "C" surface of the engine (see include/ane_b200.h for the reference citations).
#include <string.h>

#include <string>

#include "dp.h"
#include "engine.h"

struct ane_engine {
  ane::EngineBase* impl = nullptr;
};

// The Go and Python bindings mirror these layouts field by field.
static_assert(sizeof(ane_options) == 168, "ane_options layout changed: update the bindings");
static_assert(sizeof(ane_step_result) == 112, "ane_step_result layout changed: update the bindings");
static_assert(sizeof(ane_state) == 56, "ane_state layout changed: update the bindings");

static thread_local std::string g_api_err;

extern "C" {

uint32_t ane_version(void) { return 100; }

uint64_t ane_sampler_seed(int64_t seed) { return (((uint64_t)seed & 0xffffffffull) << 16) | 0x330Eull; }

int32_t ane_sample_windows(uint64_t* rng_state, uint64_t n_tokens, uint32_t seq, uint32_t batch, uint32_t rank,
                           uint32_t world, uint64_t* out_pos) {
  if (!rng_state || !out_pos || batch == 0 || rank >= (world ? world : 1)) return ANE_ERR_ARG;
  ane::sample_windows(rng_state, n_tokens, seq, batch, rank, world, out_pos);
  return 0;
}

const char* ane_last_error(ane_engine* e) {
  if (e && e->impl) return e->impl->last_error().c_str();
  return g_api_err.c_str();
}

int32_t ane_dp_unique_id(uint8_t out_id[128]) {
  if (!out_id) return ANE_ERR_ARG;
  std::string err;
  if (ane::DataParallel::unique_id(out_id, &err) != 0) {
    g_api_err = err;
    return ANE_ERR_NCCL;
  }
  return 0;
}

int32_t ane_open(const ane_options* opts, const uint16_t* tokens, uint64_t n_tokens, const uint8_t* dp_id,
                 ane_engine** out) {
  if (!opts || !out) {
    g_api_err = "storiesane open: null argument";
    return ANE_ERR_ARG;
  }
  if (opts->struct_size != sizeof(ane_options)) {
    g_api_err = "storiesane open: ane_options.struct_size mismatch";
    return ANE_ERR_ARG;
  }
  *out = nullptr;
  ane::EngineBase* impl = ane::create_engine(opts->compute_dtype);
  int rc = impl->open(*opts, tokens, n_tokens, dp_id);
  if (rc != 0) {
    g_api_err = impl->last_error();
    delete impl;
    return rc;
  }
  ane_engine* e = new ane_engine();
  e->impl = impl;
  *out = e;
  return 0;
}

int32_t ane_close(ane_engine* e) {
  if (!e) return 0;
  delete e->impl;
  e->impl = nullptr;
  delete e;
  return 0;
}

#define ENGINE_OR_FAIL(e, what)                                \
  if (!(e) || !(e)->impl) {                                    \
    g_api_err = "storiesane " what ": engine is closed";       \
    return ANE_ERR_ARG;                                        \
  }

int32_t ane_step(ane_engine* e, ane_step_result* out) {
  ENGINE_OR_FAIL(e, "step");
  return e->impl->step(nullptr, nullptr, 0, out);
}
int32_t ane_step_tokens(ane_engine* e, const uint16_t* input, const uint16_t* target, uint32_t n_seq,
                        ane_step_result* out) {
  ENGINE_OR_FAIL(e, "step");
  if (!input || !target) {
    g_api_err = "storiesane step: null token buffers";
    return ANE_ERR_ARG;
  }
  return e->impl->step(input, target, n_seq, out);
}
int32_t ane_flush(ane_engine* e, double* refresh_ms) {
  ENGINE_OR_FAIL(e, "flush");
  return e->impl->flush(refresh_ms);
}
int32_t ane_eval_logits(ane_engine* e, const uint16_t* tokens, uint32_t n_seq, float* out, uint64_t out_cap,
                        uint32_t layout) {
  ENGINE_OR_FAIL(e, "eval logits");
  if (!tokens || !out) {
    g_api_err = "storiesane eval logits: null buffer";
    return ANE_ERR_ARG;
  }
  return e->impl->eval_logits(tokens, n_seq, out, out_cap, layout);
}
int32_t ane_eval_loss(ane_engine* e, const uint16_t* tokens, uint32_t n_seq, double* loss_sum, uint64_t* n_positions) {
  ENGINE_OR_FAIL(e, "eval loss");
  if (!tokens) {
    g_api_err = "storiesane eval loss: null buffer";
    return ANE_ERR_ARG;
  }
  return e->impl->eval_loss(tokens, n_seq, loss_sum, n_positions);
}
int32_t ane_decode_greedy(ane_engine* e, const uint16_t* prompts, uint32_t n_seq, uint32_t prompt_len, uint32_t n_new,
                          uint16_t* out) {
  ENGINE_OR_FAIL(e, "decode");
  if (!prompts || !out) {
    g_api_err = "storiesane decode: null buffer";
    return ANE_ERR_ARG;
  }
  return e->impl->decode(prompts, n_seq, prompt_len, n_new, 0.f, nullptr, out);
}

int32_t ane_decode_sample(ane_engine* e, const uint16_t* prompts, uint32_t n_seq, uint32_t prompt_len, uint32_t n_new,
                          float temperature, const double* uniforms, uint16_t* out) {
  ENGINE_OR_FAIL(e, "decode");
  if (!prompts || !out) {
    g_api_err = "storiesane decode: null buffer";
    return ANE_ERR_ARG;
  }
  return e->impl->decode(prompts, n_seq, prompt_len, n_new, temperature, uniforms, out);
}
int32_t ane_set_lr(ane_engine* e, float lr) {
  ENGINE_OR_FAIL(e, "set lr");
  return e->impl->set_lr(lr);
}
float ane_get_lr(ane_engine* e) {
  if (!e || !e->impl) return 0.f;
  return e->impl->get_lr();
}
int32_t ane_get_state(ane_engine* e, ane_state* out) {
  ENGINE_OR_FAIL(e, "state");
  return e->impl->get_state(out);
}
int32_t ane_set_state(ane_engine* e, const ane_state* in) {
  ENGINE_OR_FAIL(e, "load state");
  return e->impl->set_state(in);
}
int32_t ane_reseed(ane_engine* e, int64_t seed) {
  ENGINE_OR_FAIL(e, "reseed");
  return e->impl->reseed(seed);
}
int64_t ane_tensor_size(ane_engine* e, uint32_t tensor_id, uint32_t layer) {
  if (!e || !e->impl) return -1;
  return e->impl->tensor_size(tensor_id, layer);
}
int32_t ane_import_tensor(ane_engine* e, uint32_t tensor_id, uint32_t layer, uint32_t which, const float* buf,
                          uint64_t n) {
  ENGINE_OR_FAIL(e, "import");
  if (!buf) return ANE_ERR_ARG;
  return e->impl->import_tensor(tensor_id, layer, which, buf, n);
}
int32_t ane_export_tensor(ane_engine* e, uint32_t tensor_id, uint32_t layer, uint32_t which, float* buf, uint64_t n) {
  ENGINE_OR_FAIL(e, "export");
  if (!buf && n) return ANE_ERR_ARG;
  return e->impl->export_tensor(tensor_id, layer, which, buf, n);
}
int64_t ane_get_tap(ane_engine* e, uint32_t tap_id, uint32_t layer, float* buf, uint64_t cap) {
  if (!e || !e->impl || !buf) return -1;
  return e->impl->get_tap(tap_id, layer, buf, cap);
}
int32_t ane_profile_gemm(ane_engine* e, int32_t enable) {
  ENGINE_OR_FAIL(e, "profile");
  return e->impl->profile_gemm(enable);
}
int32_t ane_profile_read(ane_engine* e, double* gemm_ms, double* gemm_flops, uint64_t* gemm_launches) {
  ENGINE_OR_FAIL(e, "profile");
  return e->impl->profile_read(gemm_ms, gemm_flops, gemm_launches);
}
int32_t ane_engine_timer_begin(ane_engine* e) {
  ENGINE_OR_FAIL(e, "timer");
  return e->impl->timer_begin();
}
int32_t ane_engine_timer_end(ane_engine* e, float* out_ms) {
  ENGINE_OR_FAIL(e, "timer");
  return e->impl->timer_end(out_ms);
}
uint64_t ane_launch_count(ane_engine* e) {
  if (!e || !e->impl) return 0;
  return e->impl->launches();
}

}  // extern "C"
