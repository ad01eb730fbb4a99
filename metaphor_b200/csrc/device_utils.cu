// mp* device utilities: the host-visible lifecycle / memory / copy calls.
// Replaces the reference's src/cuda/device_utils.cu:4-99.  Differences that a
// caller can observe are listed beside each function.
#include "mp_async.cuh"

#include <map>
#include <mutex>
#include <vector>

namespace {

constexpr int kMaxDevices = 64;
int g_sm_count[kMaxDevices];
std::once_flag g_sm_once[kMaxDevices];

size_t workspace_bytes_from_env() {
  const char* s = getenv("MP_WORKSPACE_MB");
  size_t mb = 64;
  if (s != nullptr) {
    long v = strtol(s, nullptr, 10);
    if (v > 0) mb = static_cast<size_t>(v);
  }
  return mb << 20;
}

StreamContext make_context(cudaStream_t stream, bool owns) {
  int device = 0;
  MP_CUDA_CHECK(cudaGetDevice(&device));
  MpStreamState* st = new MpStreamState();
  st->magic = MP_STATE_MAGIC;
  st->stream = stream;
  st->device = device;
  st->sm_count = mp_sm_count_current_device();
  st->owns_stream = owns;
  st->aux_ready = false;
  st->workspace_bytes = workspace_bytes_from_env();
  MP_CUDA_CHECK(cudaMalloc(&st->workspace, st->workspace_bytes));
  MP_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&st->status_dev), 256));
  MP_CUDA_CHECK(cudaMemsetAsync(st->status_dev, 0, 256, stream));
  MP_CUDA_CHECK(cudaMallocHost(reinterpret_cast<void**>(&st->status_host), 256));
  st->status_host[0] = 0;
  if (const char* lim = getenv("MP_SPIN_LIMIT_US")) {     // wait limit of the bounded waits, bytes 8..15 of the status block
    const unsigned long long ns = strtoull(lim, nullptr, 10) * 1000ull;
    MP_CUDA_CHECK(cudaMemcpyAsync(st->status_dev + 2, &ns, sizeof(ns), cudaMemcpyHostToDevice, stream));
    MP_CUDA_CHECK(cudaStreamSynchronize(stream));
  }
  StreamContext ctx;
  ctx.cuda_stream.ptr = reinterpret_cast<void*>(stream);
  ctx.blas_handle.ptr = reinterpret_cast<void*>(st);
  return ctx;
}

}  // namespace

int mp_sm_count_current_device() {
  int device = 0;
  MP_CUDA_CHECK(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) MP_FATAL("device index %d out of range", device);
  std::call_once(g_sm_once[device], [device]() {
    int n = 0;
    MP_CUDA_CHECK(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device));
    g_sm_count[device] = n;
  });
  return g_sm_count[device];
}

// The reference creates a fresh driver context (cuCtxCreate).  This binds the
// device's primary context instead, so the library can share a process with
// other CUDA runtime users (one process per GPU: call with the local rank).
extern "C" void mpInitDevice(uint32_t device_number) {
  int count = 0;
  MP_CUDA_CHECK(cudaGetDeviceCount(&count));
  if (count <= static_cast<int>(device_number)) {
    fprintf(stderr, "Error: no devices supporting CUDA\n");
    exit(-1);
  }
  MP_CUDA_CHECK(cudaSetDevice(static_cast<int>(device_number)));
  MP_CUDA_CHECK(cudaFree(nullptr));  // force context creation
}

extern "C" void* mpMemAlloc(len_t N, StreamContext ctx) {
  void* p = nullptr;
  MP_CUDA_CHECK(cudaMallocAsync(&p, N, mp_stream(ctx)));
  return p;
}

extern "C" void mpMemcpyHtoD(void* dptr, void const* hptr, len_t N, StreamContext ctx) {
  MP_CUDA_CHECK(cudaMemcpyAsync(dptr, hptr, N, cudaMemcpyHostToDevice, mp_stream(ctx)));
}

extern "C" void mpMemcpyDtoH(void* hptr, void const* dptr, len_t N, StreamContext ctx) {
  MP_CUDA_CHECK(cudaMemcpyAsync(hptr, dptr, N, cudaMemcpyDeviceToHost, mp_stream(ctx)));
}

extern "C" void mpMemFree(void* dptr, StreamContext ctx) {
  MP_CUDA_CHECK(cudaFreeAsync(dptr, mp_stream(ctx)));
}

extern "C" void mpStreamSynchronize(StreamContext ctx) {
  MP_CUDA_CHECK(cudaStreamSynchronize(mp_stream(ctx)));
}

extern "C" void mpDeviceSynchronize(void) { MP_CUDA_CHECK(cudaDeviceSynchronize()); }

extern "C" void mpCheckLastError(void) {
  MP_CUDA_CHECK(cudaDeviceSynchronize());
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    fprintf(stderr, "Error %s: %s", cudaGetErrorName(err), cudaGetErrorString(err));
  }
}

extern "C" len_t mpDeviceTotalMemory(uint32_t device) {
  cudaDeviceProp prop;
  MP_CUDA_CHECK(cudaGetDeviceProperties(&prop, static_cast<int>(device)));
  return static_cast<len_t>(prop.totalGlobalMem);
}

extern "C" StreamContext mpInitStream(void) {
  cudaStream_t stream = nullptr;
  MP_CUDA_CHECK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  return make_context(stream, true);
}

extern "C" StreamContext mpWrapStream(void* cuda_stream) {
  return make_context(static_cast<cudaStream_t>(cuda_stream), false);
}

extern "C" void mpDeinitStream(StreamContext ctx) {
  MpStreamState* st = mp_state_or_null(ctx);
  cudaStream_t stream = mp_stream(ctx);
  MP_CUDA_CHECK(cudaStreamSynchronize(stream));
  if (st != nullptr) {
    if (st->aux_ready) {
      for (int i = 0; i < 7; ++i) {
        MP_CUDA_CHECK(cudaStreamSynchronize(st->aux_stream[i]));
        MP_CUDA_CHECK(cudaStreamDestroy(st->aux_stream[i]));
        MP_CUDA_CHECK(cudaEventDestroy(st->aux_join[i]));
      }
      for (int i = 0; i < 4; ++i) MP_CUDA_CHECK(cudaEventDestroy(st->aux_sub_fork[i]));
      MP_CUDA_CHECK(cudaEventDestroy(st->aux_fork));
    }
    MP_CUDA_CHECK(cudaFree(st->workspace));
    MP_CUDA_CHECK(cudaFree(st->status_dev));
    MP_CUDA_CHECK(cudaFreeHost(st->status_host));
    const bool owns = st->owns_stream;
    st->magic = 0;
    delete st;
    if (owns) MP_CUDA_CHECK(cudaStreamDestroy(stream));
  } else {
    MP_CUDA_CHECK(cudaStreamDestroy(stream));
  }
}

extern "C" uint32_t mpGetStatus(StreamContext ctx) {
  MpStreamState* st = mp_state(ctx);
  MP_CUDA_CHECK(cudaMemcpyAsync(st->status_host, st->status_dev, sizeof(uint32_t),
                                cudaMemcpyDeviceToHost, st->stream));
  MP_CUDA_CHECK(cudaMemsetAsync(st->status_dev, 0, sizeof(uint32_t), st->stream));
  MP_CUDA_CHECK(cudaStreamSynchronize(st->stream));
  return st->status_host[0];
}

// Limit of every bounded wait of kernels launched on this stream from now on (stream-ordered); 0 restores the default.
extern "C" void mpSetWaitLimit(StreamContext ctx, len_t microseconds) {
  MpStreamState* st = mp_state(ctx);
  unsigned long long* slot = reinterpret_cast<unsigned long long*>(st->status_host + 2);
  MP_CUDA_CHECK(cudaStreamSynchronize(st->stream));     // the pinned slot may still feed an earlier copy
  *slot = static_cast<unsigned long long>(microseconds) * 1000ull;
  MP_CUDA_CHECK(cudaMemcpyAsync(st->status_dev + 2, slot, sizeof(*slot), cudaMemcpyHostToDevice, st->stream));
}

namespace {
// One CTA waits for a phase of a shared-memory barrier that nothing completes: the bounded wait runs out, records
// MP_STATUS_WAIT_TIMEOUT in the stream's status word and the kernel returns normally.
__global__ void wait_timeout_selftest_kernel(uint32_t* status) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
    (void)mbar_wait(&bar, 0, status);
  }
}
}  // namespace

// Exercises the time-out path of the bounded waits without any fault: returns after the wait limit of the stream.
extern "C" void mpSelfTestWaitTimeout(StreamContext ctx) {
  MpStreamState* st = mp_state(ctx);
  wait_timeout_selftest_kernel<<<1, 32, 0, st->stream>>>(st->status_dev);
  MP_LAUNCH_CHECK();
}

extern "C" len_t mpWorkspaceBytes(StreamContext ctx) { return mp_state(ctx)->workspace_bytes; }

extern "C" uint32_t mpDeviceSmCount(StreamContext ctx) { return static_cast<uint32_t>(mp_sm_count(ctx)); }

extern "C" void* mpHostAlloc(len_t N) {
  void* p = nullptr;
  MP_CUDA_CHECK(cudaMallocHost(&p, N));
  return p;
}

extern "C" void mpHostFree(void* hptr) { MP_CUDA_CHECK(cudaFreeHost(hptr)); }

// Cross-stream ordering for hosts that pipeline copies and kernels over several
// streams (the reference only offers whole-stream synchronisation).
extern "C" void* mpEventCreate(void) {
  cudaEvent_t ev = nullptr;
  MP_CUDA_CHECK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  return ev;
}
extern "C" void mpEventDestroy(void* event) { MP_CUDA_CHECK(cudaEventDestroy(static_cast<cudaEvent_t>(event))); }
extern "C" void mpEventRecord(void* event, StreamContext ctx) {
  MP_CUDA_CHECK(cudaEventRecord(static_cast<cudaEvent_t>(event), mp_stream(ctx)));
}
extern "C" void mpStreamWaitEvent(StreamContext ctx, void* event) {
  MP_CUDA_CHECK(cudaStreamWaitEvent(mp_stream(ctx), static_cast<cudaEvent_t>(event), 0));
}

// Stream capture: a launch-bound sequence of launcher calls (hundreds of kernels per training step)
// is recorded once and replayed with one call.  Everything the launchers do is stream-ordered and
// allocation-free, so any sequence of them can be captured; calls that synchronise (mpGetStatus,
// mpStreamSynchronize, mpMemcpy* from pageable memory) must stay outside the captured region.
namespace {
std::mutex g_graph_mutex;
std::map<void*, size_t> g_graph_kernels;   // executable graph -> number of kernel nodes
}
extern "C" void mpGraphBeginCapture(StreamContext ctx) {
  MP_CUDA_CHECK(cudaStreamBeginCapture(mp_stream(ctx), cudaStreamCaptureModeThreadLocal));
}
extern "C" void* mpGraphEndCapture(StreamContext ctx) {
  cudaGraph_t graph = nullptr;
  MP_CUDA_CHECK(cudaStreamEndCapture(mp_stream(ctx), &graph));
  // kernel nodes of the captured work, kept for mpGraphKernelNodes
  size_t n_nodes = 0, n_kernels = 0;
  MP_CUDA_CHECK(cudaGraphGetNodes(graph, nullptr, &n_nodes));
  std::vector<cudaGraphNode_t> nodes(n_nodes);
  if (n_nodes > 0) MP_CUDA_CHECK(cudaGraphGetNodes(graph, nodes.data(), &n_nodes));
  for (size_t i = 0; i < n_nodes; ++i) {
    cudaGraphNodeType type;
    MP_CUDA_CHECK(cudaGraphNodeGetType(nodes[i], &type));
    if (type == cudaGraphNodeTypeKernel) ++n_kernels;
  }
  cudaGraphExec_t exec = nullptr;
  MP_CUDA_CHECK(cudaGraphInstantiate(&exec, graph, 0));
  MP_CUDA_CHECK(cudaGraphDestroy(graph));
  {
    std::lock_guard<std::mutex> lock(g_graph_mutex);
    g_graph_kernels[exec] = n_kernels;
  }
  return exec;
}
extern "C" len_t mpGraphKernelNodes(void* exec) {
  std::lock_guard<std::mutex> lock(g_graph_mutex);
  auto it = g_graph_kernels.find(exec);
  return it == g_graph_kernels.end() ? 0 : it->second;
}
extern "C" void mpGraphLaunch(void* exec, StreamContext ctx) {
  MP_CUDA_CHECK(cudaGraphLaunch(static_cast<cudaGraphExec_t>(exec), mp_stream(ctx)));
}
extern "C" void mpGraphDestroy(void* exec) {
  if (exec == nullptr) return;
  {
    std::lock_guard<std::mutex> lock(g_graph_mutex);
    g_graph_kernels.erase(exec);
  }
  MP_CUDA_CHECK(cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(exec)));
}
