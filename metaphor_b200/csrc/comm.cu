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
//
// Failure detection is host-side only: every call has a variant that returns a
// status instead of exiting, mpCommPoll waits for the stream with a host
// time-out while polling ncclCommGetAsyncError, mpCommAbort tears a stuck
// communicator down, and mpSetFailPoint makes a named entry point report an
// error without doing anything (for tests of the recovery path).  Nothing here
// waits on the device without a limit.
#include "mp_common.cuh"
#include "../../include/mp_comm.h"

#include <dlfcn.h>
#include <string.h>

#include <chrono>
#include <map>
#include <mutex>
#include <string>
#include <thread>

namespace {

struct NcclId { char internal[128]; };
typedef void* NcclComm;

struct NcclApi {
  void* lib = nullptr;
  int (*getUniqueId)(NcclId*) = nullptr;
  int (*commInitRank)(NcclComm*, int, NcclId, int) = nullptr;
  int (*commDestroy)(NcclComm) = nullptr;
  int (*commAbort)(NcclComm) = nullptr;
  int (*commGetAsyncError)(NcclComm, int*) = nullptr;
  int (*allReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  const char* (*getErrorString)(int) = nullptr;
};

NcclApi* nccl_or_null() {
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
    api.commAbort = reinterpret_cast<decltype(api.commAbort)>(dlsym(api.lib, "ncclCommAbort"));
    api.commGetAsyncError = reinterpret_cast<decltype(api.commGetAsyncError)>(dlsym(api.lib, "ncclCommGetAsyncError"));
    api.allReduce = reinterpret_cast<decltype(api.allReduce)>(dlsym(api.lib, "ncclAllReduce"));
    api.getErrorString = reinterpret_cast<decltype(api.getErrorString)>(dlsym(api.lib, "ncclGetErrorString"));
  });
  return (api.lib == nullptr || api.allReduce == nullptr) ? nullptr : &api;
}
NcclApi* nccl() {
  NcclApi* api = nccl_or_null();
  if (api == nullptr) MP_FATAL("NCCL (libnccl.so.2) could not be loaded");
  return api;
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
  NcclComm comm;          // null for a world of one: nothing to exchange
  int world, rank;
  cudaEvent_t poll_event; // created on first mpCommPoll
};
constexpr uint64_t COMM_MAGIC = 0x4d50434f4d4d3031ull;

MpComm* checked(void* comm) {
  MpComm* c = static_cast<MpComm*>(comm);
  return (c != nullptr && c->magic == COMM_MAGIC) ? c : nullptr;
}

// ---- fail points: name -> remaining hits ----------------------------------------------
std::mutex g_fail_mutex;
std::map<std::string, int> g_fail_points;
bool fail_point_hit(const char* name) {
  std::lock_guard<std::mutex> lock(g_fail_mutex);
  auto it = g_fail_points.find(name);
  if (it == g_fail_points.end() || it->second == 0) return false;
  if (it->second > 0) --it->second;
  return true;
}

}  // namespace

extern "C" void mpSetFailPoint(const char* name, int32_t count) {
  std::lock_guard<std::mutex> lock(g_fail_mutex);
  if (name == nullptr) { g_fail_points.clear(); return; }
  g_fail_points[name] = count;
}

extern "C" int32_t mpCommInitStatus(const void* unique_id128, uint32_t world_size, uint32_t rank, void** comm_out) {
  if (comm_out == nullptr || world_size == 0 || rank >= world_size) return MP_COMM_BAD_ARGUMENT;
  *comm_out = nullptr;
  if (fail_point_hit("mpCommInit")) return MP_COMM_ERROR;
  MpComm* c = new MpComm();
  c->magic = COMM_MAGIC;
  c->comm = nullptr;
  c->world = static_cast<int>(world_size);
  c->rank = static_cast<int>(rank);
  c->poll_event = nullptr;
  if (world_size > 1) {
    NcclApi* api = nccl_or_null();
    NcclId id;
    if (unique_id128 == nullptr || api == nullptr) { delete c; return MP_COMM_ERROR; }
    memcpy(&id, unique_id128, sizeof(id));
    if (api->commInitRank(&c->comm, c->world, id, c->rank) != 0) { delete c; return MP_COMM_ERROR; }
  }
  *comm_out = c;
  return MP_COMM_OK;
}

extern "C" int32_t mpAllReduceSumStatus(void* comm, void* buffer, len_t count, uint32_t dtype_key, StreamContext ctx) {
  MpComm* c = checked(comm);
  if (c == nullptr) return MP_COMM_BAD_HANDLE;
  if (dtype_key > 2) return MP_COMM_BAD_ARGUMENT;
  if (fail_point_hit("mpAllReduceSum")) return MP_COMM_ERROR;
  if (count == 0 || c->world == 1) return MP_COMM_OK;
  const int nccl_type[3] = {6 /* ncclFloat16 */, 7 /* ncclFloat32 */, 8 /* ncclFloat64 */};
  return nccl()->allReduce(buffer, buffer, count, nccl_type[dtype_key], 0 /* ncclSum */, c->comm, mp_stream(ctx)) == 0 ? MP_COMM_OK
                                                                                                                        : MP_COMM_ERROR;
}

// Host-side wait for the work queued on ctx's stream: returns MP_COMM_OK when it has finished, MP_COMM_ERROR as soon as
// NCCL reports an asynchronous error on the communicator (a peer died, a transport failed), MP_COMM_TIMEOUT after
// timeout_ms.  The stream is never synchronised without a limit; after ERROR or TIMEOUT the caller aborts the
// communicator (mpCommAbort) and rebuilds it.
extern "C" int32_t mpCommPoll(void* comm, StreamContext ctx, uint32_t timeout_ms) {
  MpComm* c = checked(comm);
  if (c == nullptr) return MP_COMM_BAD_HANDLE;
  if (fail_point_hit("mpCommPoll")) return MP_COMM_ERROR;
  if (c->poll_event == nullptr) MP_CUDA_CHECK(cudaEventCreateWithFlags(&c->poll_event, cudaEventDisableTiming));
  MP_CUDA_CHECK(cudaEventRecord(c->poll_event, mp_stream(ctx)));
  const auto t0 = std::chrono::steady_clock::now();
  while (true) {
    const cudaError_t q = cudaEventQuery(c->poll_event);
    if (q == cudaSuccess) return MP_COMM_OK;
    if (q != cudaErrorNotReady) return MP_COMM_ERROR;
    if (c->comm != nullptr && nccl()->commGetAsyncError != nullptr) {
      int async_err = 0;
      if (nccl()->commGetAsyncError(c->comm, &async_err) != 0 || (async_err != 0 && async_err != 7 /* ncclInProgress */)) return MP_COMM_ERROR;
    }
    if (std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count() >= timeout_ms) return MP_COMM_TIMEOUT;
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

// Tears the communicator down without waiting for outstanding collectives (ncclCommAbort) and frees the handle.
extern "C" void mpCommAbort(void* comm) {
  MpComm* c = checked(comm);
  if (c == nullptr) return;
  if (c->comm != nullptr && nccl()->commAbort != nullptr) nccl()->commAbort(c->comm);
  if (c->poll_event != nullptr) cudaEventDestroy(c->poll_event);
  c->magic = 0;
  delete c;
}

extern "C" void mpCommGetUniqueId(void* out128) {
  NcclId id;
  MP_NCCL_CHECK(nccl()->getUniqueId(&id));
  memcpy(out128, &id, sizeof(id));
}

extern "C" void* mpCommInit(const void* unique_id128, uint32_t world_size, uint32_t rank) {
  void* comm = nullptr;
  const int32_t rc = mpCommInitStatus(unique_id128, world_size, rank, &comm);
  if (rc != MP_COMM_OK) MP_FATAL("mpCommInit failed with status %d (rank %u of %u)", rc, rank, world_size);
  return comm;
}

extern "C" void mpCommDestroy(void* comm) {
  MpComm* c = checked(comm);
  if (c == nullptr) MP_FATAL("not a handle from mpCommInit");
  if (c->comm != nullptr) MP_NCCL_CHECK(nccl()->commDestroy(c->comm));
  if (c->poll_event != nullptr) cudaEventDestroy(c->poll_event);
  c->magic = 0;
  delete c;
}

extern "C" uint32_t mpCommWorldSize(void* comm) {
  MpComm* c = checked(comm);
  if (c == nullptr) MP_FATAL("not a handle from mpCommInit");
  return static_cast<uint32_t>(c->world);
}

extern "C" void mpAllReduceSum(void* comm, void* buffer, len_t count, uint32_t dtype_key, StreamContext ctx) {
  const int32_t rc = mpAllReduceSumStatus(comm, buffer, count, dtype_key, ctx);
  if (rc == MP_COMM_BAD_HANDLE) MP_FATAL("not a handle from mpCommInit");
  if (rc != MP_COMM_OK) MP_FATAL("mpAllReduceSum failed with status %d", rc);
}
