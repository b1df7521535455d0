#include "tensor_parallel.h"

#include <dlfcn.h>

#include <mutex>

namespace etc {

namespace {

// The handful of NCCL entry points used, declared here so that no NCCL header is needed at build time.
struct UniqueId { char internal[128]; };
using Comm = void*;
using GetUniqueIdFn = int (*)(UniqueId*);
using CommInitRankFn = int (*)(Comm*, int, UniqueId, int);
using AllReduceFn = int (*)(const void*, void*, size_t, int, int, Comm, cudaStream_t);
using CommDestroyFn = int (*)(Comm);
using GetErrorStringFn = const char* (*)(int);
constexpr int kNcclFloat32 = 7, kNcclSum = 0;

struct Api {
  void* lib = nullptr;
  GetUniqueIdFn get_unique_id = nullptr;
  CommInitRankFn comm_init_rank = nullptr;
  AllReduceFn all_reduce = nullptr;
  CommDestroyFn comm_destroy = nullptr;
  GetErrorStringFn get_error_string = nullptr;
  std::string error;
};

Api& api() {
  static Api a;
  static std::once_flag once;
  std::call_once(once, [] {
    // prefer the copy that is already mapped into this process: two NCCL instances would not share anything
    a.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!a.lib) a.lib = dlopen("libnccl.so.2", RTLD_NOW);
    if (!a.lib) {
      a.error = std::string("libnccl.so.2 cannot be loaded: ") + (dlerror() ? dlerror() : "unknown error");
      return;
    }
    a.get_unique_id = (GetUniqueIdFn)dlsym(a.lib, "ncclGetUniqueId");
    a.comm_init_rank = (CommInitRankFn)dlsym(a.lib, "ncclCommInitRank");
    a.all_reduce = (AllReduceFn)dlsym(a.lib, "ncclAllReduce");
    a.comm_destroy = (CommDestroyFn)dlsym(a.lib, "ncclCommDestroy");
    a.get_error_string = (GetErrorStringFn)dlsym(a.lib, "ncclGetErrorString");
    if (!a.get_unique_id || !a.comm_init_rank || !a.all_reduce || !a.comm_destroy || !a.get_error_string)
      a.error = "libnccl.so.2 lacks one of ncclGetUniqueId, ncclCommInitRank, ncclAllReduce, ncclCommDestroy, ncclGetErrorString";
  });
  return a;
}

bool check(int rc, const char* what, std::string* error) {
  if (rc == 0) return true;
  if (error) *error = std::string(what) + ": " + api().get_error_string(rc);
  return false;
}

}  // namespace

struct TpComm {
  Comm comm = nullptr;
  int rank = 0, world = 1;
};

bool tp_unique_id(unsigned char out[128], std::string* error) {
  Api& a = api();
  if (!a.error.empty()) { if (error) *error = a.error; return false; }
  UniqueId id;
  if (!check(a.get_unique_id(&id), "ncclGetUniqueId", error)) return false;
  for (int i = 0; i < 128; ++i) out[i] = (unsigned char)id.internal[i];
  return true;
}

TpComm* tp_comm_create(int rank, int world, const unsigned char id_bytes[128], std::string* error) {
  Api& a = api();
  if (!a.error.empty()) { if (error) *error = a.error; return nullptr; }
  UniqueId id;
  for (int i = 0; i < 128; ++i) id.internal[i] = (char)id_bytes[i];
  TpComm* c = new TpComm();
  c->rank = rank;
  c->world = world;
  if (!check(a.comm_init_rank(&c->comm, world, id, rank), "ncclCommInitRank", error)) {
    delete c;
    return nullptr;
  }
  return c;
}

void tp_comm_destroy(TpComm* comm) {
  if (!comm) return;
  if (comm->comm) api().comm_destroy(comm->comm);
  delete comm;
}

bool tp_allreduce_sum(TpComm* comm, float* data, size_t count, cudaStream_t stream, std::string* error) {
  return check(api().all_reduce(data, data, count, kNcclFloat32, kNcclSum, comm->comm, stream), "ncclAllReduce", error);
}

}  // namespace etc
