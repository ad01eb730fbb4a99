// Data-parallel gradient exchange: one NCCL communicator per process (one
// process per GPU), sum all-reduce of a flat gradient buffer on the caller's
// stream.  The reference has no multi-GPU code at all (its only concurrency
// primitive is several streams on one device, src/core/utils.zig:39-71); this is
// the single collective the data-parallel training configuration needs.  The
// 1/world_size scaling is folded into the optimizer step (grad_scale of
// launch_adam), not done here.
//
// NCCL is resolved at run time (dlopen of libnccl.so.2: the copy already in the
// process is reused), so the library loads on machines without it.
#include "mp_common.cuh"
#include "../../include/mp_comm.h"

#include <dlfcn.h>
#include <string.h>

#include <mutex>

namespace {

struct NcclId { char internal[128]; };
typedef void* NcclComm;

struct NcclApi {
  void* lib = nullptr;
  int (*getUniqueId)(NcclId*) = nullptr;
  int (*commInitRank)(NcclComm*, int, NcclId, int) = nullptr;
  int (*commDestroy)(NcclComm) = nullptr;
  int (*allReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  const char* (*getErrorString)(int) = nullptr;
};

NcclApi* nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, []() {
    const char* names[] = {"libnccl.so.2", "libnccl.so", "/usr/lib/x86_64-linux-gnu/libnccl.so.2"};
    for (const char* nm : names) {
      api.lib = dlopen(nm, RTLD_NOW | RTLD_GLOBAL);
      if (api.lib != nullptr) break;
    }
    if (api.lib == nullptr) return;
    api.getUniqueId = reinterpret_cast<decltype(api.getUniqueId)>(dlsym(api.lib, "ncclGetUniqueId"));
    api.commInitRank = reinterpret_cast<decltype(api.commInitRank)>(dlsym(api.lib, "ncclCommInitRank"));
    api.commDestroy = reinterpret_cast<decltype(api.commDestroy)>(dlsym(api.lib, "ncclCommDestroy"));
    api.allReduce = reinterpret_cast<decltype(api.allReduce)>(dlsym(api.lib, "ncclAllReduce"));
    api.getErrorString = reinterpret_cast<decltype(api.getErrorString)>(dlsym(api.lib, "ncclGetErrorString"));
  });
  if (api.lib == nullptr || api.allReduce == nullptr) MP_FATAL("NCCL (libnccl.so.2) could not be loaded");
  return &api;
}

#define MP_NCCL_CHECK(expr)                                                                  \
  do {                                                                                       \
    const int mp_rc__ = (expr);                                                              \
    if (mp_rc__ != 0) {                                                                      \
      printf("NCCL error %d (%s) in %s at line %d\n", mp_rc__,                               \
             nccl()->getErrorString ? nccl()->getErrorString(mp_rc__) : "?", __FILE__, __LINE__); \
      fflush(stdout);                                                                        \
      exit(EXIT_FAILURE);                                                                    \
    }                                                                                        \
  } while (0)

struct MpComm {
  uint64_t magic;
  NcclComm comm;
  int world, rank;
};
constexpr uint64_t COMM_MAGIC = 0x4d50434f4d4d3031ull;

}  // namespace

extern "C" void mpCommGetUniqueId(void* out128) {
  NcclId id;
  MP_NCCL_CHECK(nccl()->getUniqueId(&id));
  memcpy(out128, &id, sizeof(id));
}

extern "C" void* mpCommInit(const void* unique_id128, uint32_t world_size, uint32_t rank) {
  NcclId id;
  memcpy(&id, unique_id128, sizeof(id));
  MpComm* c = new MpComm();
  c->magic = COMM_MAGIC;
  c->world = static_cast<int>(world_size);
  c->rank = static_cast<int>(rank);
  MP_NCCL_CHECK(nccl()->commInitRank(&c->comm, c->world, id, c->rank));
  return c;
}

extern "C" void mpCommDestroy(void* comm) {
  MpComm* c = static_cast<MpComm*>(comm);
  if (c == nullptr || c->magic != COMM_MAGIC) MP_FATAL("not a handle from mpCommInit");
  MP_NCCL_CHECK(nccl()->commDestroy(c->comm));
  c->magic = 0;
  delete c;
}

extern "C" uint32_t mpCommWorldSize(void* comm) { return static_cast<uint32_t>(static_cast<MpComm*>(comm)->world); }

extern "C" void mpAllReduceSum(void* comm, void* buffer, len_t count, uint32_t dtype_key, StreamContext ctx) {
  MpComm* c = static_cast<MpComm*>(comm);
  if (c == nullptr || c->magic != COMM_MAGIC) MP_FATAL("not a handle from mpCommInit");
  if (dtype_key > 2) MP_FATAL("mpAllReduceSum: bad dtype key %u", dtype_key);
  if (count == 0) return;
  const int nccl_type[3] = {6 /* ncclFloat16 */, 7 /* ncclFloat32 */, 8 /* ncclFloat64 */};
  MP_NCCL_CHECK(nccl()->allReduce(buffer, buffer, count, nccl_type[dtype_key], 0 /* ncclSum */, c->comm, mp_stream(ctx)));
}
