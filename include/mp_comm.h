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

#endif
