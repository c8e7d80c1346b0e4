// Data-parallel gradient exchange: one process per GPU, NCCL all-reduce of the flat fp32
// gradient buffer.  NCCL is loaded lazily with dlopen so single-GPU use has no NCCL dependency.
// The reference has no multi-device path; the reduction it mirrors is the sum over AccumSteps
// sequences that precedes one optimizer update (ane/train_full.go:811-818, ane/engine.go:650-654).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace ane {

class DataParallel {
 public:
  static int unique_id(uint8_t out[128], std::string* err);
  int init(int rank, int world, const uint8_t id[128], int device);
  bool active() const { return comm_ != nullptr; }
  // In-place sum over ranks, issued in buckets on `stream`.
  int all_reduce_sum(float* buf, size_t n, cudaStream_t stream);
  // Sum of n doubles over ranks, in place (the squared gradient norm of a sharded optimizer).
  int all_reduce_sum_f64(double* buf, size_t n, cudaStream_t stream);
  // In-place reduce-scatter: buf holds world * n_per_rank floats; afterwards rank r's slice
  // [r * n_per_rank, (r + 1) * n_per_rank) holds the sum over ranks (the other slices are unspecified).
  int reduce_scatter_sum(float* buf, size_t n_per_rank, cudaStream_t stream);
  // In-place all-gather: rank r contributes bytes [r * bytes_per_rank, (r + 1) * bytes_per_rank) of buf.
  int all_gather_bytes(void* buf, size_t bytes_per_rank, cudaStream_t stream);
  int rank() const { return rank_; }
  void shutdown();
  const char* last_error() const { return err_.c_str(); }
  int world() const { return world_; }

 private:
  void* comm_ = nullptr;
  int world_ = 1, rank_ = 0;
  std::string err_;
};

}  // namespace ane
