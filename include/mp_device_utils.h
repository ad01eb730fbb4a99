/*
 * Device utilities: context / stream lifecycle, stream-ordered memory, async
 * copies.  The first eleven prototypes are the reference's
 * src/cuda/device_utils.h:12-22, unchanged; each comment cites the reference
 * definition it replaces.  The block after them is additive.
 *
 * Error convention (reference kernel_header.h:64-98): every function returns
 * void (or a value); a CUDA error prints one line and calls
 * exit(EXIT_FAILURE).
 */
#ifndef MP_B200_DEVICE_UTILS_H
#define MP_B200_DEVICE_UTILS_H

#include "mp_types.h"

/* device_utils.cu:32-51 — bind this host thread to device `device_number`
 * (primary context).  One process per GPU calls it with its local rank. */
MP_EXTERN_C void mpInitDevice(uint32_t device_number);
/* device_utils.cu:4-9 — stream-ordered allocation of N bytes. */
MP_EXTERN_C void* mpMemAlloc(len_t N, StreamContext);
/* device_utils.cu:10-14 — async host-to-device copy of N bytes. */
MP_EXTERN_C void mpMemcpyHtoD(void* dptr, void const* hptr, len_t N, StreamContext);
/* device_utils.cu:15-19 — async device-to-host copy of N bytes. */
MP_EXTERN_C void mpMemcpyDtoH(void* hptr, void const* dptr, len_t N, StreamContext);
/* device_utils.cu:20-24 — stream-ordered free. */
MP_EXTERN_C void mpMemFree(void* dptr, StreamContext);
/* device_utils.cu:29-31 */
MP_EXTERN_C void mpDeviceSynchronize(void);
/* device_utils.cu:25-28 */
MP_EXTERN_C void mpStreamSynchronize(StreamContext);
/* device_utils.cu:70-88 — new stream + per-stream state on the current device. */
MP_EXTERN_C StreamContext mpInitStream(void);
/* device_utils.cu:90-99 */
MP_EXTERN_C void mpDeinitStream(StreamContext);
/* device_utils.cu:55-62 — device sync, print the pending error if any. */
MP_EXTERN_C void mpCheckLastError(void);
/* device_utils.cu:64-68 */
MP_EXTERN_C len_t mpDeviceTotalMemory(uint32_t device);

/* ---- additive (no counterpart in the reference) ------------------------- */

/* Build a StreamContext around a stream the caller already owns (for example
 * a framework's current stream).  mpDeinitStream releases the per-stream state
 * and leaves the caller's stream alive. */
MP_EXTERN_C StreamContext mpWrapStream(void* cuda_stream);

/* Read (and clear) the per-stream device status word after synchronising the
 * stream.  0 = no kernel reported a problem.  Non-zero codes are listed in
 * mp_kernels.h (MP_STATUS_*); kernels with bounded waits set them instead of
 * spinning forever. */
MP_EXTERN_C uint32_t mpGetStatus(StreamContext);

/* Limit, in microseconds, after which a kernel's bounded wait (on a shared-memory barrier fed by an asynchronous
 * copy or by the tensor core) gives up, records MP_STATUS_WAIT_TIMEOUT and lets the kernel end; 0 = the built-in
 * 2 s.  Applies to kernels launched on the stream after the call.  The environment variable MP_SPIN_LIMIT_US sets
 * the initial value of every stream.  (The reference's kernels have no waits; its error path is print-and-exit,
 * src/cuda/kernel_header.h:64-98.) */
MP_EXTERN_C void mpSetWaitLimit(StreamContext, len_t microseconds);
/* Launches a one-CTA kernel whose wait can never be satisfied: it returns after the stream's wait limit with
 * MP_STATUS_WAIT_TIMEOUT in the status word.  A check of the time-out path that faults nothing. */
MP_EXTERN_C void mpSelfTestWaitTimeout(StreamContext);
/* The work partition of the SSD chunk walk as the kernels compute it (host-side copy of the same function, no GPU needed):
 * segment idx of CTA cta (of ncta <= nseq) for nseq sequences of nc chunks; out[5] = {sequence, first chunk position,
 * chunks, state carried in, state carried out}; returns 0 past the CTA's last segment. */
MP_EXTERN_C int mpSsdWalkPartition(int cta, int ncta, int nseq, int nc, int idx, int* out);

/* Bytes of library-owned workspace attached to the stream (split-K partials,
 * column-reduce partials, tensor-map staging).  Allocated once in
 * mpInitStream / mpWrapStream, never inside a launcher. */
MP_EXTERN_C len_t mpWorkspaceBytes(StreamContext);

/* Number of streaming multiprocessors of the stream's device. */
MP_EXTERN_C uint32_t mpDeviceSmCount(StreamContext);

/* Events: order work across streams without blocking the host (copy-in ->
 * compute -> copy-out pipelines).  mpStreamWaitEvent makes all later work on
 * ctx's stream wait for the work recorded by mpEventRecord. */
MP_EXTERN_C void* mpEventCreate(void);
MP_EXTERN_C void mpEventDestroy(void* event);
MP_EXTERN_C void mpEventRecord(void* event, StreamContext);
MP_EXTERN_C void mpStreamWaitEvent(StreamContext, void* event);

/* Stream capture into a CUDA graph (the reference launches every kernel from the
 * host each step, graph.zig:552-631; a training step here is several hundred
 * launches).  Launcher calls made on ctx's stream between Begin and End are
 * recorded, not executed; mpGraphLaunch replays them in stream order.  Calls that
 * synchronise (mpGetStatus, mpStreamSynchronize, mpDeviceSynchronize) are not
 * allowed inside the captured region. */
MP_EXTERN_C void mpGraphBeginCapture(StreamContext);
MP_EXTERN_C void* mpGraphEndCapture(StreamContext);
MP_EXTERN_C void mpGraphLaunch(void* graph, StreamContext);
MP_EXTERN_C void mpGraphDestroy(void* graph);
/* Number of kernel launches a graph returned by mpGraphEndCapture replays (0 for an unknown handle).
 * No counterpart in the reference. */
MP_EXTERN_C len_t mpGraphKernelNodes(void* graph);

/* Pinned host memory for the end-to-end copy path (the reference copies from
 * pageable memory, src/core/utils.zig:159-218; pinned buffers let
 * mpMemcpyHtoD / mpMemcpyDtoH run at link speed). */
MP_EXTERN_C void* mpHostAlloc(len_t N);
MP_EXTERN_C void mpHostFree(void* hptr);

#endif
