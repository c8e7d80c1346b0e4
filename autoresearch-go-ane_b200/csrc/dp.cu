#include "dp.h"

#include <dlfcn.h>
#include <string.h>

#include <mutex>

namespace ane {

namespace {

struct NcclId {
  char internal[128];
};
typedef int (*GetUniqueIdFn)(NcclId*);
typedef int (*CommInitRankFn)(void**, int, NcclId, int);
typedef int (*AllReduceFn)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef int (*ReduceScatterFn)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef int (*AllGatherFn)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef int (*CommDestroyFn)(void*);
typedef const char* (*GetErrorStringFn)(int);

struct NcclApi {
  void* handle = nullptr;
  GetUniqueIdFn get_unique_id = nullptr;
  CommInitRankFn comm_init_rank = nullptr;
  AllReduceFn all_reduce = nullptr;
  ReduceScatterFn reduce_scatter = nullptr;
  AllGatherFn all_gather = nullptr;
  CommDestroyFn comm_destroy = nullptr;
  GetErrorStringFn get_error_string = nullptr;
  std::string err;
};

NcclApi* nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (api.handle) break;
    }
    if (!api.handle) {
      api.err = "libnccl.so.2 not found";
      return;
    }
    api.get_unique_id = (GetUniqueIdFn)dlsym(api.handle, "ncclGetUniqueId");
    api.comm_init_rank = (CommInitRankFn)dlsym(api.handle, "ncclCommInitRank");
    api.all_reduce = (AllReduceFn)dlsym(api.handle, "ncclAllReduce");
    api.reduce_scatter = (ReduceScatterFn)dlsym(api.handle, "ncclReduceScatter");
    api.all_gather = (AllGatherFn)dlsym(api.handle, "ncclAllGather");
    api.comm_destroy = (CommDestroyFn)dlsym(api.handle, "ncclCommDestroy");
    api.get_error_string = (GetErrorStringFn)dlsym(api.handle, "ncclGetErrorString");
    if (!api.get_unique_id || !api.comm_init_rank || !api.all_reduce || !api.comm_destroy || !api.reduce_scatter ||
        !api.all_gather)
      api.err = "NCCL symbols missing";
  });
  return &api;
}

constexpr int kNcclFloat = 7;  // ncclFloat32
constexpr int kNcclSum = 0;    // ncclSum
constexpr int kNcclDouble = 8; // ncclFloat64
constexpr int kNcclInt8 = 0;   // ncclInt8
// ~32 MiB buckets: large enough to run at link bandwidth, small enough to pipeline.
constexpr size_t kBucketElems = 8u << 20;

}  // namespace

int DataParallel::unique_id(uint8_t out[128], std::string* err) {
  NcclApi* a = nccl();
  if (!a->err.empty()) {
    if (err) *err = a->err;
    return -1;
  }
  NcclId id;
  memset(&id, 0, sizeof id);
  int r = a->get_unique_id(&id);
  if (r != 0) {
    if (err) *err = std::string("ncclGetUniqueId: ") + (a->get_error_string ? a->get_error_string(r) : "error");
    return -1;
  }
  memcpy(out, id.internal, 128);
  return 0;
}

int DataParallel::init(int rank, int world, const uint8_t id[128], int device) {
  NcclApi* a = nccl();
  if (!a->err.empty()) {
    err_ = a->err;
    return -1;
  }
  if (rank < 0 || rank >= world) {
    err_ = "bad rank";
    return -1;
  }
  cudaSetDevice(device);
  NcclId nid;
  memcpy(nid.internal, id, 128);
  void* comm = nullptr;
  int r = a->comm_init_rank(&comm, world, nid, rank);
  if (r != 0) {
    err_ = std::string("ncclCommInitRank: ") + (a->get_error_string ? a->get_error_string(r) : "error");
    return -1;
  }
  comm_ = comm;
  world_ = world;
  rank_ = rank;
  return 0;
}

int DataParallel::all_reduce_sum(float* buf, size_t n, cudaStream_t stream) {
  if (!comm_) return 0;
  NcclApi* a = nccl();
  for (size_t off = 0; off < n; off += kBucketElems) {
    const size_t cnt = n - off < kBucketElems ? n - off : kBucketElems;
    int r = a->all_reduce(buf + off, buf + off, cnt, kNcclFloat, kNcclSum, comm_, stream);
    if (r != 0) {
      err_ = std::string("ncclAllReduce: ") + (a->get_error_string ? a->get_error_string(r) : "error");
      return -1;
    }
  }
  return 0;
}

int DataParallel::all_reduce_sum_f64(double* buf, size_t n, cudaStream_t stream) {
  if (!comm_ || n == 0) return 0;
  NcclApi* a = nccl();
  int r = a->all_reduce(buf, buf, n, kNcclDouble, kNcclSum, comm_, stream);
  if (r != 0) {
    err_ = std::string("ncclAllReduce: ") + (a->get_error_string ? a->get_error_string(r) : "error");
    return -1;
  }
  return 0;
}

int DataParallel::reduce_scatter_sum(float* buf, size_t n_per_rank, cudaStream_t stream) {
  if (!comm_ || n_per_rank == 0) return 0;
  NcclApi* a = nccl();
  int r = a->reduce_scatter(buf, buf + (size_t)rank_ * n_per_rank, n_per_rank, kNcclFloat, kNcclSum, comm_, stream);
  if (r != 0) {
    err_ = std::string("ncclReduceScatter: ") + (a->get_error_string ? a->get_error_string(r) : "error");
    return -1;
  }
  return 0;
}

int DataParallel::all_gather_bytes(void* buf, size_t bytes_per_rank, cudaStream_t stream) {
  if (!comm_ || bytes_per_rank == 0) return 0;
  NcclApi* a = nccl();
  int r = a->all_gather(static_cast<char*>(buf) + (size_t)rank_ * bytes_per_rank, buf, bytes_per_rank, kNcclInt8, comm_,
                        stream);
  if (r != 0) {
    err_ = std::string("ncclAllGather: ") + (a->get_error_string ? a->get_error_string(r) : "error");
    return -1;
  }
  return 0;
}

void DataParallel::shutdown() {
  if (comm_) {
    NcclApi* a = nccl();
    if (a->comm_destroy) a->comm_destroy(comm_);
    comm_ = nullptr;
  }
}

}  // namespace ane
