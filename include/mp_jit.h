/*
 * Run-time fused element-wise chains (forward and reverse) - additive API, no
 * counterpart in the reference: its op layer launches one kernel per op
 * (src/ops/addition.zig:41, hadamard.zig:39, ...) and links nvrtc without
 * calling it (build.zig:139).
 *
 * An expression names its tensor operands by identifier; operands are numbered
 * in order of first appearance.  Grammar: + - * over operands, unary -,
 * numeric literals, relu(x), selu(x), parentheses.  Example:
 *   "selu((a+b)*(c+d))"  ->  leaves a, b, c, d.
 */
#ifndef MP_B200_JIT_H
#define MP_B200_JIT_H

#include "mp_types.h"

/* Parse, generate CUDA C, compile with NVRTC for sm_100a, load.  dtype_key is
 * MP_R16 / MP_R32 / MP_R64.  Programs are cached by (expression, dtype); every
 * successful call must be paired with mpJitRelease.  Returns NULL (after
 * printing the reason) if the expression does not parse. */
MP_EXTERN_C void* mpJitCompile(const char* expr, uint32_t dtype_key);
MP_EXTERN_C void mpJitRelease(void* handle);
MP_EXTERN_C uint32_t mpJitNumLeaves(void* handle);
MP_EXTERN_C const char* mpJitLeafName(void* handle, uint32_t index);

/* out[i] = f(leaves[0][i], leaves[1][i], ...) in one pass. */
MP_EXTERN_C void mpJitForward(void* handle, const void* const* leaves, void* out, len_t n, StreamContext);

/* One pass producing every leaf gradient (intermediates are recomputed):
 *   g_leaves[l][i] = g_out[i] * d f / d leaf_l + alpha * g_leaves[l][i]
 * g_out == NULL stands for an upstream gradient of ones (the seed the host's
 * Tensor.reverse uses, src/core/graph.zig:111-121); a NULL entry in g_leaves
 * skips that operand; the old gradient is not read when alpha == 0. */
MP_EXTERN_C void mpJitReverse(void* handle, const void* const* leaves, const void* g_out, void* const* g_leaves,
                              double alpha, len_t n, StreamContext);

/* The generated CUDA C for an expression (no GPU needed); free with
 * mpJitFreeSource.  NULL if the expression does not parse. */
MP_EXTERN_C char* mpJitGenerateSource(const char* expr, uint32_t dtype_key);
MP_EXTERN_C void mpJitFreeSource(char* source);

#endif
