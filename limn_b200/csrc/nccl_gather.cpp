// The one collective of the path, for hosts that do not bring a communication library of their own: the gather of
// the (batch, head) shards' outputs over NCCL. The attention problems of a batch are independent, so a sharded run
// needs no communication while it computes; afterwards every rank's slice of O (or of dQ, dK, dV) is gathered
// into one tensor on each GPU. NCCL is loaded at run time (libnccl.so.2), so the library has no link-time
// dependency on it and a single-GPU host never touches it. The reference has nothing here: limn is single-GPU
// (limn/backend_cuda.py:283 takes device 0).
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.h"

namespace limn_b200 {
namespace {

struct UniqueId {
  char bytes[LIMN_B200_NCCL_ID_BYTES];
};
typedef struct ncclComm* Comm;
typedef int (*GetUniqueIdFn)(UniqueId*);
typedef int (*CommInitRankFn)(Comm*, int, UniqueId, int);
typedef int (*AllGatherFn)(const void*, void*, size_t, int, Comm, cudaStream_t);
typedef int (*CommDestroyFn)(Comm);
typedef const char* (*GetErrorStringFn)(int);

struct Nccl {
  void* handle = nullptr;
  GetUniqueIdFn get_unique_id = nullptr;
  CommInitRankFn comm_init_rank = nullptr;
  AllGatherFn all_gather = nullptr;
  CommDestroyFn comm_destroy = nullptr;
  GetErrorStringFn get_error_string = nullptr;
  Comm comm = nullptr;
  int rank = -1, world = 0;
};
Nccl g_nccl;
std::mutex g_nccl_mutex;

// Loads NCCL on first use. LIMN_B200_NCCL_LIBRARY names the file to load instead of the default search.
int load(Nccl& n) {
  if (n.handle != nullptr) return LIMN_B200_OK;
  const char* named = getenv("LIMN_B200_NCCL_LIBRARY");
  const char* candidates[] = {named, "libnccl.so.2", "libnccl.so"};
  void* handle = nullptr;
  for (const char* name : candidates) {
    if (name == nullptr || name[0] == '\0') continue;
    handle = dlopen(name, RTLD_NOW | RTLD_LOCAL);
    if (handle != nullptr || name == named) break;  // a named library that does not load is an error, not a hint
  }
  if (handle == nullptr) {
    const char* why = dlerror();
    return fail(LIMN_B200_UNSUPPORTED, "nccl: cannot load %s: %s", named && named[0] ? named : "libnccl.so.2", why ? why : "not found");
  }
  n.get_unique_id = reinterpret_cast<GetUniqueIdFn>(dlsym(handle, "ncclGetUniqueId"));
  n.comm_init_rank = reinterpret_cast<CommInitRankFn>(dlsym(handle, "ncclCommInitRank"));
  n.all_gather = reinterpret_cast<AllGatherFn>(dlsym(handle, "ncclAllGather"));
  n.comm_destroy = reinterpret_cast<CommDestroyFn>(dlsym(handle, "ncclCommDestroy"));
  n.get_error_string = reinterpret_cast<GetErrorStringFn>(dlsym(handle, "ncclGetErrorString"));
  if (!n.get_unique_id || !n.comm_init_rank || !n.all_gather || !n.comm_destroy || !n.get_error_string) {
    dlclose(handle);
    return fail(LIMN_B200_UNSUPPORTED, "nccl: the loaded library lacks one of ncclGetUniqueId, ncclCommInitRank, ncclAllGather, ncclCommDestroy, ncclGetErrorString");
  }
  n.handle = handle;
  return LIMN_B200_OK;
}

int nccl_fail(const Nccl& n, int result, const char* doing) {
  return fail(LIMN_B200_CUDA_ERROR, "nccl: %s: %s", doing, n.get_error_string ? n.get_error_string(result) : "error");
}

}  // namespace
}  // namespace limn_b200

using namespace limn_b200;

extern "C" {

int limn_b200_nccl_unique_id(void* id_out) {
  clear_error();
  if (id_out == nullptr) return fail(LIMN_B200_BAD_ARGUMENT, "nccl_unique_id: null result pointer");
  std::lock_guard<std::mutex> lock(g_nccl_mutex);
  if (int rc = load(g_nccl)) return rc;
  UniqueId id;
  if (int res = g_nccl.get_unique_id(&id)) return nccl_fail(g_nccl, res, "making a unique id");
  memcpy(id_out, id.bytes, sizeof(id.bytes));
  return LIMN_B200_OK;
}

int limn_b200_nccl_init(int rank, int world, const void* id) {
  clear_error();
  if (id == nullptr) return fail(LIMN_B200_BAD_ARGUMENT, "nccl_init: null id");
  if (world <= 0 || rank < 0 || rank >= world)
    return fail(LIMN_B200_BAD_ARGUMENT, "nccl_init: rank %d is not one of %d ranks", rank, world);
  std::lock_guard<std::mutex> lock(g_nccl_mutex);
  if (g_nccl.comm != nullptr) return fail(LIMN_B200_BAD_ARGUMENT, "nccl_init: this process already holds a communicator; destroy it first");
  if (int rc = load(g_nccl)) return rc;
  UniqueId copy;
  memcpy(copy.bytes, id, sizeof(copy.bytes));
  Comm comm = nullptr;
  if (int res = g_nccl.comm_init_rank(&comm, world, copy, rank)) return nccl_fail(g_nccl, res, "creating the communicator");
  g_nccl.comm = comm, g_nccl.rank = rank, g_nccl.world = world;
  return LIMN_B200_OK;
}

int limn_b200_nccl_all_gather(const void* send, void* recv, unsigned long long bytes_per_rank, void* stream) {
  clear_error();
  if (send == nullptr || recv == nullptr) return fail(LIMN_B200_BAD_ARGUMENT, "nccl_all_gather: a required pointer is null");
  std::lock_guard<std::mutex> lock(g_nccl_mutex);
  if (g_nccl.comm == nullptr) return fail(LIMN_B200_BAD_ARGUMENT, "nccl_all_gather: no communicator; call limn_b200_nccl_init first");
  if (bytes_per_rank == 0) return LIMN_B200_OK;
  constexpr int kNcclInt8 = 0;  // ncclInt8 / ncclChar: the gather moves bytes, whatever the storage dtype
  if (int res = g_nccl.all_gather(send, recv, static_cast<size_t>(bytes_per_rank), kNcclInt8, g_nccl.comm, static_cast<cudaStream_t>(stream)))
    return nccl_fail(g_nccl, res, "enqueueing the all-gather");
  return LIMN_B200_OK;
}

int limn_b200_nccl_destroy(void) {
  clear_error();
  std::lock_guard<std::mutex> lock(g_nccl_mutex);
  if (g_nccl.comm == nullptr) return LIMN_B200_OK;
  const int res = g_nccl.comm_destroy(g_nccl.comm);
  g_nccl.comm = nullptr, g_nccl.rank = -1, g_nccl.world = 0;
  if (res) return nccl_fail(g_nccl, res, "destroying the communicator");
  return LIMN_B200_OK;
}

}  // extern "C"
