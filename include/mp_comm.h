/*
 * Gradient exchange for data-parallel training - additive API, no counterpart
 * in the reference (single device, single context: src/cuda/device_utils.cu:32-51).
 * One process per GPU: every process calls mpInitDevice(local_rank), rank 0
 * creates the 128-byte unique id and hands it to the others by any host channel,
 * then every rank calls mpCommInit.
 */
#ifndef MP_B200_COMM_H
#define MP_B200_COMM_H

#include "mp_types.h"

/* Writes the 128-byte NCCL unique id (call on one rank, distribute to all). */
MP_EXTERN_C void mpCommGetUniqueId(void* out128);
/* Collective over all ranks: joins the communicator described by the id. */
MP_EXTERN_C void* mpCommInit(const void* unique_id128, uint32_t world_size, uint32_t rank);
MP_EXTERN_C void mpCommDestroy(void* comm);
MP_EXTERN_C uint32_t mpCommWorldSize(void* comm);
/* In-place sum over ranks of `count` elements (dtype_key MP_R16/R32/R64) on
 * ctx.cuda_stream; asynchronous like every launcher.  The mean is taken by the
 * optimizer (grad_scale = 1/world_size in launch_adam, or rate/world_size in
 * launch_sgd). */
MP_EXTERN_C void mpAllReduceSum(void* comm, void* buffer, len_t count, uint32_t dtype_key, StreamContext ctx);

/* Failure detection (host side only).  The calls above follow the reference's convention - print and
 * exit(EXIT_FAILURE), src/cuda/kernel_header.h:64-98 - which leaves the peers of a failed rank waiting inside
 * the collective.  These variants return a status instead, so that a trainer can notice and rebuild. */
#define MP_COMM_OK 0
#define MP_COMM_ERROR 2          /* NCCL reported an error (also asynchronously), or a fail point fired */
#define MP_COMM_TIMEOUT 3        /* mpCommPoll: the stream had not finished after timeout_ms */
#define MP_COMM_BAD_HANDLE 4
#define MP_COMM_BAD_ARGUMENT 5
MP_EXTERN_C int32_t mpCommInitStatus(const void* unique_id128, uint32_t world_size, uint32_t rank, void** comm_out);
MP_EXTERN_C int32_t mpAllReduceSumStatus(void* comm, void* buffer, len_t count, uint32_t dtype_key, StreamContext ctx);
/* Waits on the host, sleeping between polls, until the work queued on ctx.cuda_stream has finished (OK), NCCL
 * reports an asynchronous error on the communicator (ERROR) or timeout_ms have passed (TIMEOUT). */
MP_EXTERN_C int32_t mpCommPoll(void* comm, StreamContext ctx, uint32_t timeout_ms);
/* ncclCommAbort: gives up the outstanding collectives and frees the handle (after ERROR / TIMEOUT). */
MP_EXTERN_C void mpCommAbort(void* comm);
/* Test hook, host only: the next `count` calls (-1 = all) of the entry point called `name` ("mpCommInit",
 * "mpAllReduceSum", "mpCommPoll") report MP_COMM_ERROR without doing anything; name NULL clears every fail point. */
MP_EXTERN_C void mpSetFailPoint(const char* name, int32_t count);

#endif
