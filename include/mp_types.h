/*
 * Value types that cross the extern "C" boundary between the Zig host layer
 * and the device layer.  Bit-compatible with the reference's
 * src/cuda/kernel_header.h:10-17 (PaddedPtr, StreamContext) and
 * src/cuda/tensor_types.h:4-33,83-98 (len_t, r16/r32/r64, SortPair_*), so a
 * Zig `@cImport` of this file yields the same layouts the reference's
 * generated glue (file_gen.zig:330-340) expects.
 *
 * Plain C: no CUDA header is needed to include this file from host code.
 */
#ifndef MP_B200_TYPES_H
#define MP_B200_TYPES_H

#include <stdint.h>

#define MAX_DIMS 6
typedef unsigned long len_t;

#if defined(__cplusplus) && defined(__CUDACC__)
  #include <cuda_fp16.h>
  typedef __half r16;
#else
/* Host code never does arithmetic on r16; only its size matters. */
typedef struct { unsigned short __x; } r16;
#endif
typedef float  r32;
typedef double r64;

/* One pointer per struct: keeps each member in its own INTEGER eightbyte under
 * the SysV ABI (reference kernel_header.h:6-13). */
typedef struct { void* ptr; } PaddedPtr;

/* Passed BY VALUE as the last argument of every launcher.
 *  cuda_stream : the CUstream every launch and copy is ordered on.
 *  blas_handle : opaque to the host.  The reference stores a cublasHandle_t
 *                here (device_utils.cu:70-88); this library stores a pointer
 *                to its own per-stream state (workspace, status word, SM
 *                count).  It is created only by mpInitStream / mpWrapStream
 *                and destroyed only by mpDeinitStream, exactly like the
 *                handle it replaces. */
typedef struct {
  PaddedPtr cuda_stream;
  PaddedPtr blas_handle;
} StreamContext;

/* Kept for layout compatibility (tensor_types.h:83-98); no kernel of the
 * op path uses them. */
typedef struct { r16 val; unsigned key; } SortPair_r16;
typedef struct { r32 val; unsigned key; } SortPair_r32;
typedef struct { r64 val; unsigned key; } SortPair_r64;

/* Dispatch key order used by the host (src/core/scalar.zig:35-40):
 * r16 = 0, r32 = 1, r64 = 2.  Launcher triples are declared in that order. */
enum { MP_R16 = 0, MP_R32 = 1, MP_R64 = 2 };

#if defined(__cplusplus)
  #define MP_EXTERN_C extern "C"
#else
  #define MP_EXTERN_C extern
#endif

#endif
