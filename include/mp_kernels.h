/*
 * Launcher prototypes of the device layer (the drop-in boundary).
 *
 * Part 1 re-declares, with unchanged names, argument order and meaning, the
 * 60 prototypes of the reference's generated header src/cuda/kernel_decls.h
 * (20 launchers x {r16,r32,r64}); each group cites the reference kernel it
 * replaces.  Part 2 is additive and follows the same conventions: void
 * return, device pointers as void*, host scalars as double, sizes as len_t,
 * StreamContext by value as the last argument, `_r16/_r32/_r64` suffix in the
 * dtype-key order of src/core/scalar.zig:35-40 so that the host's 3-entry
 * dispatch arrays (file_gen.zig:298-328, root.zig:36-43) keep working.
 *
 * Common semantics of every launcher here:
 *  - asynchronous on ctx.cuda_stream, never synchronises, never allocates,
 *    never retains a pointer;
 *  - sizes are full 64-bit (the reference narrows them to 32 bits);
 *  - "x + alpha*dst" blends do not read dst when alpha == 0, so a fresh
 *    (uninitialised) output can never inject NaN;
 *  - r16 I/O is computed in fp32 and rounded once.
 */
#ifndef MP_B200_KERNELS_H
#define MP_B200_KERNELS_H

#include "mp_types.h"

#define MP_DECL3(name, ...)                                  \
  MP_EXTERN_C void launch_##name##_r16(__VA_ARGS__);          \
  MP_EXTERN_C void launch_##name##_r32(__VA_ARGS__);          \
  MP_EXTERN_C void launch_##name##_r64(__VA_ARGS__);

/* ======================= Part 1: reference symbols ======================= */

/* reduce_ij_i.cu:35-54 — dst[i] = sum_j src[i,j] + alpha*dst[i] */
MP_DECL3(reduce_ij_i, const void* src, void* dst, double alpha, len_t m, len_t n, StreamContext stream)
/* reduce_ij_j.cu:48-66 — dst[j] = sum_i src[i,j] + alpha*dst[j] (the formula;
 * the reference kernel is only right for alpha = 0 and m >= n) */
MP_DECL3(reduce_ij_j, const void* src, void* dst, double alpha, len_t m, len_t n, StreamContext stream)
/* broadcast_i_ij.cu:41-59 — dst[i,j] = src[i] + alpha*dst[i,j] */
MP_DECL3(broadcast_i_ij, const void* src, void* dst, double alpha, len_t m, len_t n, StreamContext stream)
/* broadcast_j_ij.cu:36-55 — dst[i,j] = src[j] + alpha*dst[i,j] */
MP_DECL3(broadcast_j_ij, const void* src, void* dst, double alpha, len_t m, len_t n, StreamContext stream)
/* dilate_reverse.cu:16-29 — b[i] += a[i]*value */
MP_DECL3(dilate_reverse, const void* a, double value, void* b, len_t N, StreamContext stream)
/* subtraction.cu:16-29 — c = a - b */
MP_DECL3(subtraction, const void* a, const void* b, void* c, len_t N, StreamContext stream)
/* relu_reverse.cu:18-31 — a_grads[i] += b_grads[i] * (a_value[i] >= 0) */
MP_DECL3(relu_reverse, const void* a_value, void* a_grads, const void* b_grads, len_t N, StreamContext stream)
/* dilate.cu:16-29 — c = a*value */
MP_DECL3(dilate, const void* a, double value, void* c, len_t N, StreamContext stream)
/* translate.cu:16-29 — c = a + value */
MP_DECL3(translate, const void* a, double value, void* c, len_t N, StreamContext stream)
/* permutate_ij_ji.cu:43-67 — dst[j,i] = src[i,j] + alpha*dst[j,i]; src is
 * [row,col] row-major.  Bit-exact when alpha = 0. */
MP_DECL3(permutate_ij_ji, const void* src, void* dst, double alpha, len_t row, len_t col, StreamContext ctx)
/* negate.cu:15-26 — b = -a */
MP_DECL3(negate, const void* a, void* b, len_t N, StreamContext stream)
/* hadamard_reverse.cu:16-29 — c += a*b */
MP_DECL3(hadamard_reverse, const void* a, const void* b, void* c, len_t N, StreamContext stream)
/* inner_product_ij_jk_ik.cu:3-27 — C[m,k] = alpha*A[m,n]*B[n,k] + beta*C,
 * all row-major.  The reference forwards to cuBLAS; here a TMA-fed
 * tcgen05/TMEM kernel (r16, r32) or an FP64 SIMT tile kernel (r64). */
MP_DECL3(inner_product_ij_jk_ik, const void* a_data, const void* b_data, const double alpha, void* c_data, const double beta, len_t m, len_t n, len_t k, StreamContext stream)
/* hadamard.cu:16-29 — c = a*b */
MP_DECL3(hadamard, const void* a, const void* b, void* c, len_t N, StreamContext stream)
/* fill.cu:16-27 — a[i] = value */
MP_DECL3(fill, void* dev_a, double value, len_t N, StreamContext stream)
/* relu.cu:16-27 — b = a >= 0 ? a : 0 */
MP_DECL3(relu, const void* a, void* b, len_t n, StreamContext stream)
/* addition.cu:16-29 — c = a + b (c may alias a or b: the host's reverse pass
 * calls it as g_x = g_z + g_x, addition.zig:67-81) */
MP_DECL3(addition, const void* a, const void* b, void* c, len_t N, StreamContext stream)
/* copy.cu:33-47 — dst = src */
MP_DECL3(copy, const void* src, void* dst, len_t n, StreamContext stream)
/* sequence.cu:18-31 — a[i] = init + step*T(i), evaluated in T */
MP_DECL3(sequence, void* dev_a, double init, double step, len_t N, StreamContext stream)
/* stepwise.cu:16-27 — b = a >= 0 ? 1 : 0.  (The reference body is a copy of
 * relu; its only caller, relu.derive at relu.zig:56-58, needs the 0/1 step.) */
MP_DECL3(stepwise, const void* a, void* b, len_t n, StreamContext stream)

/* ============================ Part 2: additive =========================== */
/* No launcher below has a kernel in the reference; the README names the ops
 * (README.md:81,97) and the Zig layer sketches the optimizer call
 * (src/optm/optimizer.zig:160-179). */

/* b = selu(a) = 1.0507009873554805 * (a > 0 ? a : 1.6732632423543772*(exp(a)-1));
 * argument order of relu.cu:16-21. */
MP_DECL3(selu, const void* a, void* b, len_t n, StreamContext stream)
/* a_grads += b_grads * selu'(a_value); argument order of relu_reverse.cu:18-24 */
MP_DECL3(selu_reverse, const void* a_value, void* a_grads, const void* b_grads, len_t N, StreamContext stream)

/* dst[i,:] = softmax(src[i,:]) over the last axis of a row-major [m,n] matrix
 * ("ij|j" in the grammar of src/ops/expression_parsing.zig:319-340). */
MP_DECL3(softmax_ij_j, const void* src, void* dst, len_t m, len_t n, StreamContext stream)
/* gx = y o (gy - sum_j gy o y) + alpha*gx, y the forward output. */
MP_DECL3(softmax_ij_j_reverse, const void* y, const void* gy, void* gx, double alpha, len_t m, len_t n, StreamContext stream)

/* y[i,j] = x[i,j] * rstd_i * gain[j], rstd_i = rsqrt(mean_j x[i,j]^2 + eps).
 * rstd (m values, r32 for r16/r32 and r64 for r64) may be NULL. */
MP_DECL3(rmsnorm_ij_j, const void* x, const void* gain, double eps, void* y, void* rstd, len_t m, len_t n, StreamContext stream)
/* gx     = rstd*(gy o gain) - x*rstd^3*mean_j(gy o gain o x) + alpha*gx
 * ggain  = sum_i gy[i,:] o x[i,:]*rstd_i                    + alpha*ggain
 * rstd may be NULL (it is then recomputed from x and eps at no extra traffic).
 * scratch: caller-owned, mpRmsnormReverseScratchBytes(m,n,ctx) bytes, holds
 * the per-CTA partial sums of ggain (deterministic two-stage reduction). */
MP_DECL3(rmsnorm_ij_j_reverse, const void* x, const void* gain, const void* rstd, const void* gy, double eps, void* gx, void* ggain, double alpha, void* scratch, len_t m, len_t n, StreamContext stream)
MP_EXTERN_C len_t mpRmsnormReverseScratchBytes(len_t m, len_t n, StreamContext stream);
/* No counterpart in the reference.  RMSNorm reverse (r32) for callers that are
 * not allowed to allocate device memory (a plug-in inside a runtime that owns
 * the whole device through its own pool, a loop where an allocation would stall
 * the device): same arguments and results as launch_rmsnorm_ij_j_reverse_r32
 * without `scratch`.  The partial sums live in a fixed array inside the library
 * (MP_RMSNORM_STATIC_SCRATCH_BYTES per GPU that loads it, held until exit); the
 * call allocates nothing.  Returns 0, or MP_STATUS_BAD_ARGUMENT with a message
 * on stderr when one row of partials plus the fold rows does not fit (rows
 * longer than about 100k columns).  The first call on a device looks up the
 * array's device address and should come before any stream capture.  Calls
 * share the array: keep them stream-ordered, overlapping calls race. */
#define MP_RMSNORM_STATIC_SCRATCH_BYTES (8u << 20)
MP_EXTERN_C int launch_rmsnorm_ij_j_reverse_static_r32(const void* x, const void* gain, const void* rstd, const void* gy, double eps, void* gx, void* ggain, double alpha, len_t m, len_t n, StreamContext stream);

/* w -= rate * clip(g, clip_lo, clip_hi); argument set of optimizer.zig:170-178 */
MP_DECL3(sgd, void* w, const void* g, double rate, double clip_lo, double clip_hi, len_t n, StreamContext stream)
/* One fused Adam step over a flat buffer, g' = grad_scale*g:
 *   m = b1*m + (1-b1)*g';  v = b2*v + (1-b2)*g'^2;
 *   w -= lr * (m/(1-b1^step)) / (sqrt(v/(1-b2^step)) + eps)
 * grad_scale folds the 1/world_size of a data-parallel all-reduce. */
MP_DECL3(adam, void* w, const void* g, void* m, void* v, double lr, double beta1, double beta2, double eps, double grad_scale, len_t step, len_t n, StreamContext stream)

/* Native transposed-operand contractions (the reference transposes into
 * scratch first, inner_product.zig:305-330,364-389):
 *   ij,kj->ik : C[m,k] = alpha*A[m,n]*B[k,n]^T + beta*C
 *   ji,jk->ik : C[m,k] = alpha*A[n,m]^T*B[n,k] + beta*C */
MP_DECL3(inner_product_ij_kj_ik, const void* a_data, const void* b_data, const double alpha, void* c_data, const double beta, len_t m, len_t n, len_t k, StreamContext stream)
MP_DECL3(inner_product_ji_jk_ik, const void* a_data, const void* b_data, const double alpha, void* c_data, const double beta, len_t m, len_t n, len_t k, StreamContext stream)
/* linear (README.md:81): C[m,k] = alpha*A[m,n]*B[n,k] + bias[k] + beta*C,
 * bias added in the GEMM epilogue. */
MP_DECL3(linear_ij_jk_ik, const void* a_data, const void* b_data, const void* bias, const double alpha, void* c_data, const double beta, len_t m, len_t n, len_t k, StreamContext stream)
/* c = alpha * a b + r + beta * c with a full [m, k] term r ("ij,jk,ik->ik": the residual form of linear; r may alias c when beta = 0) */
MP_DECL3(linear_ij_jk_ik_ik, const void* a, const void* b, const void* r, double alpha, void* c, double beta, len_t m, len_t n, len_t k, StreamContext stream)

/* Mamba-2 SSD chunked scan (no reference kernel; the op is named by the
 * project's roadmap only).  Per batch b, head h (group g = h / (heads/ngroups)):
 *   S_t = exp(dt_t*A_h) S_{t-1} + dt_t * B_t (x) x_t,   y_t = C_t^T S_t,   S_{-1} = 0.
 * x, y: [batch, seqlen, heads, headdim] of T; dt: [batch, seqlen, heads] r32
 * (already positive, e.g. after softplus); A: [heads] r32 (negative);
 * B, C: [batch, seqlen, ngroups, dstate] of T.  fp32 accumulation.
 * scratch: mpSsdScanScratchBytes(..., reverse) bytes owned by the caller (the reverse holds four
 * independent sets of intermediates, its operator instances run side by side on helper streams that
 * the library forks from and joins back into the caller's stream).
 * Two implementations: a tensor-core path (r16 with dstate = 128, headdim 64 or 128, chunk 128 or 256,
 * seqlen a multiple of chunk) and a sequential-recurrence path for every other shape of r16 and for r32 /
 * r64 storage (dt, A, gdt, gA then have the storage type; `chunk` is ignored).  Scratch: r16 ->
 * mpSsdScanScratchBytes (either path), r32 / r64 -> mpSsdScanGenericScratchBytes(dtype_key, ...); the
 * forward of the sequential path needs none. */
MP_DECL3(ssd_scan, const void* x, const void* dt, const void* A, const void* B, const void* C, void* y, void* scratch, len_t batch, len_t seqlen, len_t heads, len_t headdim, len_t dstate, len_t ngroups, len_t chunk, StreamContext stream)
/* Reverse of the scan: given gy (shape of y) writes (overwrites) gx, gdt (r32),
 * gA (r32, [heads]), gB, gC.  gB and gC are summed over the heads of a group. */
MP_DECL3(ssd_scan_reverse, const void* x, const void* dt, const void* A, const void* B, const void* C, const void* gy, void* gx, void* gdt, void* gA, void* gB, void* gC, void* scratch, len_t batch, len_t seqlen, len_t heads, len_t headdim, len_t dstate, len_t ngroups, len_t chunk, StreamContext stream)
/* launch_ssd_scan from the projection's raw outputs: dt = softplus(dt_raw + dt_bias[h]) (dt_raw: T, pitched [batch*seqlen, heads];
 * dt_bias: acc [heads]) and A = -exp(A_log[h]) (acc) are formed inside the scan and left in dt_out (acc [batch, seqlen, heads])
 * and A_out (acc [heads]) for launch_ssd_scan_reverse.  Same scratch as launch_ssd_scan. */
MP_DECL3(ssd_scan_raw, const void* x, const void* dt_raw, len_t dt_pitch, const void* dt_bias, const void* A_log, const void* B, const void* C, void* y, void* dt_out, void* A_out, void* scratch, len_t batch, len_t seqlen, len_t heads, len_t headdim, len_t dstate, len_t ngroups, len_t chunk, StreamContext stream)
/* launch_ssd_scan_reverse plus the reverses of dt = softplus(dt_raw + dt_bias[h]) and A = -exp(A_log[h]):
 *   gdt_raw = gdt * sigmoid(dt_raw + dt_bias) (T, pitched), gdt_bias[h] += its sum (acc, may be NULL), gA_log[h] += gA[h] * A[h] (acc, may be NULL).
 * gdt and gA are written too.  Same scratch as launch_ssd_scan_reverse. */
MP_DECL3(ssd_scan_reverse_raw, const void* x, const void* dt, const void* A, const void* B, const void* C, const void* gy, const void* dt_raw, len_t dt_pitch, const void* dt_bias, void* gx, void* gdt, void* gA, void* gdt_raw, len_t gdt_raw_pitch, void* gdt_bias, void* gA_log, void* gB, void* gC, void* scratch, len_t batch, len_t seqlen, len_t heads, len_t headdim, len_t dstate, len_t ngroups, len_t chunk, StreamContext stream)
MP_EXTERN_C len_t mpSsdScanScratchBytes(len_t batch, len_t seqlen, len_t heads, len_t headdim, len_t dstate, len_t ngroups, len_t chunk, uint32_t reverse);
MP_EXTERN_C len_t mpSsdScanGenericScratchBytes(uint32_t dtype_key, len_t batch, len_t seqlen, len_t heads, len_t headdim, len_t dstate, len_t ngroups, uint32_t reverse);

/* ---- operators around the scan in a Mamba-2 language-model step ------------
 * No counterpart in the reference (its loss layer is a sketch,
 * src/ops/loss.zig:60-237; the model is named by the project's roadmap only).
 * "acc" below is the accumulator type of T: r32 for r16 and r32, r64 for r64.
 * Parameter gradients and per-head parameters use acc; they are ACCUMULATED
 * (+=), the caller zeroes them once per step.  Pitches are in elements. */

/* out[t,:] = table[ids[t],:]; ids: int32; ids outside [0, vocab) give a zero row */
MP_DECL3(embedding, const void* table, const void* ids, void* out, len_t n, len_t dim, len_t vocab, StreamContext stream)
/* gtable[ids[t],:] += gy[t,:]; gtable: acc [vocab, dim] */
MP_DECL3(embedding_reverse, const void* ids, const void* gy, void* gtable, len_t n, len_t dim, len_t vocab, StreamContext stream)
/* Depthwise causal convolution + SiLU over x[batch, len, channels] (row pitch
 * x_pitch): pre = bias[c] + sum_k w[c,k] x[b, l-width+1+k, c] (zero before the
 * sequence), y = pre*sigmoid(pre).  w: [channels, width] of T, width 2..4;
 * bias may be NULL. */
MP_DECL3(causal_conv1d_silu, const void* x, len_t x_pitch, const void* w, const void* bias, void* y, len_t y_pitch, len_t batch, len_t len, len_t channels, len_t width, StreamContext stream)
/* gx (overwritten), gw += (acc [channels, width]), gbias += (acc [channels], may be NULL) */
MP_DECL3(causal_conv1d_silu_reverse, const void* x, len_t x_pitch, const void* w, const void* bias, const void* gy, len_t gy_pitch, void* gx, len_t gx_pitch, void* gw, void* gbias, len_t batch, len_t len, len_t channels, len_t width, StreamContext stream)
/* The same convolution over sum(seg_channels) consecutive channels of x, cut into nseg <= 4 consecutive segments whose
 * outputs (reverse: incoming gradients) live in buffers of their own: ys[i] / gys[i] with row pitch pitches[i] hold
 * seg_channels[i] channels.  w, bias, gx, gw, gbias are indexed by the channel of x.  ys / gys / pitches / seg_channels
 * are HOST arrays, read before the call returns.  One launch for r16 with 16-byte-aligned rows (x, B and C of a Mamba-2
 * block are neighbouring column ranges of one projection), otherwise one launch per segment. */
MP_DECL3(causal_conv1d_silu_segments, const void* x, len_t x_pitch, const void* w, const void* bias, void* const* ys, const len_t* y_pitches, const len_t* seg_channels, len_t nseg, len_t batch, len_t len, len_t width, StreamContext stream)
MP_DECL3(causal_conv1d_silu_segments_reverse, const void* x, len_t x_pitch, const void* w, const void* bias, const void* const* gys, const len_t* gy_pitches, const len_t* seg_channels, len_t nseg, void* gx, len_t gx_pitch, void* gw, void* gbias, len_t batch, len_t len, len_t width, StreamContext stream)
/* The same with a second upstream term on chosen segments (host arrays of nseg entries; skips[i] NULL: none):
 *   gy_total[i] = gys[i] + skip_scales[i][channel / skip_group] * skips[i]      (skip_scales[i]: acc [seg_channels[i] / skip_group])
 * i.e. the reverse of y_total = conv(...) feeding both an operator and a per-group scaled skip around it.  The upstream
 * buffers of segments with a skip term are unspecified afterwards. */
MP_DECL3(causal_conv1d_silu_segments_reverse_skip, const void* x, len_t x_pitch, const void* w, const void* bias, const void* const* gys, const len_t* gy_pitches, const len_t* seg_channels, len_t nseg, const void* const* skips, const len_t* skip_pitches, const void* const* skip_scales, len_t skip_group, void* gx, len_t gx_pitch, void* gw, void* gbias, len_t batch, len_t len, len_t width, StreamContext stream)
/* out[r,h] = softplus(raw[r,h] + bias[h]); raw: T with row pitch; bias, out: acc */
MP_DECL3(softplus_bias, const void* raw, len_t raw_pitch, const void* bias, void* out, len_t rows, len_t heads, StreamContext stream)
/* graw[r,h] = gdt[r,h]*sigmoid(raw[r,h] + bias[h]) (T, pitched); gbias[h] += sum_r graw (acc, may be NULL) */
MP_DECL3(softplus_bias_reverse, const void* raw, len_t raw_pitch, const void* bias, const void* gdt, void* graw, len_t graw_pitch, void* gbias, len_t rows, len_t heads, StreamContext stream)
/* u = (y + D[h]*x) * silu(z); y, x, u: [rows, heads*headdim]; z pitched; D: acc [heads] or NULL */
MP_DECL3(ssd_gate, const void* y, const void* x, const void* D, const void* z, len_t z_pitch, void* u, len_t rows, len_t heads, len_t headdim, StreamContext stream)
/* gy = gu*silu(z); gz = gu*(y + D x)*silu'(z) (pitched); gD[h] += sum gy*x (acc, may be NULL).
 * The skip's share of gx is added afterwards with launch_head_scale_accumulate. */
MP_DECL3(ssd_gate_reverse, const void* y, const void* x, const void* D, const void* z, len_t z_pitch, const void* gu, void* gy, void* gz, len_t gz_pitch, void* gD, len_t rows, len_t heads, len_t headdim, StreamContext stream)
/* Gate and RMSNorm in one pass: with u = (y + D[h]*x) * silu(z) (never written),
 *   out = u * rstd * gain, rstd[r] = 1/sqrt(mean_j u[r,j]^2 + eps)   (rstd: acc [rows], may be NULL) */
MP_DECL3(ssd_gate_rmsnorm, const void* y, const void* x, const void* D, const void* z, len_t z_pitch, const void* gain, double eps, void* out, void* rstd, len_t rows, len_t heads, len_t headdim, StreamContext stream)
/* Reverse of launch_ssd_gate_rmsnorm: u is recomputed from y, x, z; gout is d loss / d out.
 *   gy = gu*silu(z); gz = gu*(y + D x)*silu'(z) (pitched) with gu the RMSNorm reverse of gout;
 *   gD[h] += sum gy*x (acc, may be NULL); ggain = alpha*ggain + sum_r gout*u*rstd (T [heads*headdim], may be NULL).
 * scratch: caller-owned, mpSsdGateRmsnormReverseScratchBytes(rows, heads, headdim, ctx) bytes. */
MP_DECL3(ssd_gate_rmsnorm_reverse, const void* y, const void* x, const void* D, const void* z, len_t z_pitch, const void* gain, const void* rstd, const void* gout, void* gy, void* gz, len_t gz_pitch, void* gD, void* ggain, double alpha, void* scratch, len_t rows, len_t heads, len_t headdim, StreamContext stream)
MP_EXTERN_C len_t mpSsdGateRmsnormReverseScratchBytes(len_t rows, len_t heads, len_t headdim, StreamContext stream);
/* gx[r,h,:] += D[h]*gy[r,h,:] */
MP_DECL3(head_scale_accumulate, const void* D, const void* gy, void* gx, len_t rows, len_t heads, len_t headdim, StreamContext stream)
/* Cross-entropy of logits [m, n] against int32 targets, loss and gradient in one pass:
 *   loss[i] = logsumexp_j(logits[i,:]) - logits[i,target_i]               (acc [m], may be NULL)
 *   glogits[i,j] = scale*(softmax(logits[i,:])_j - [j == target_i])       (T, may alias logits, may be NULL)
 * Rows whose target lies outside [0, n) contribute zero loss and zero gradient. */
MP_DECL3(cross_entropy, const void* logits, const void* targets, double scale, void* loss, void* glogits, len_t m, len_t n, StreamContext stream)
/* dst = -exp(src) (the scan's decay parameter A from its logarithm) */
MP_DECL3(neg_exp, const void* src, void* dst, len_t n, StreamContext stream)
/* Precision conversion between r16 working copies and r32 master buffers:
 * dst(r32) = src(r16) + beta*dst;  dst(r16) = round(src(r32)). */
MP_EXTERN_C void launch_convert_r16_r32(const void* src, void* dst, double beta, len_t n, StreamContext stream);
MP_EXTERN_C void launch_convert_r32_r16(const void* src, void* dst, len_t n, StreamContext stream);
/* Mixed-precision Adam over a flat parameter bucket (the reference names Adam only in NOTES.md:11; its update loop
 * over the weights is optimizer.zig:140-179).  `tick` = 16 bytes of zero-initialised device memory holding
 * {1/(1-beta1^t), 1/(1-beta2^t), t, non-finite flag}; launch_adam_tick advances t on the stream, so a step replayed
 * from a captured graph uses its own step number.  launch_adam_mixed_r32: g = (g32 + g16) * grad_scale (g16 may be
 * NULL), Adam update of w32 / m / v, and w16 = round(w32) in the same pass.  Elements whose gradient is not finite are
 * left unchanged and the flag (4th word of `tick`) is set. */
MP_EXTERN_C void launch_adam_tick(void* tick, double beta1, double beta2, StreamContext stream);
MP_EXTERN_C void launch_adam_mixed_r32(void* w32, void* w16, const void* g32, const void* g16, void* m, void* v, double lr, double beta1,
                                       double beta2, double eps, double grad_scale, void* tick, len_t n, StreamContext stream);

/* Rank-1 losses and the momentum step.  The reference calls kernels of these names (loss.zig:58-136,
 * optimizer.zig:263-273) but contains no implementation; argument order follows those call sites.
 *   mse: redux = mean (x-t)^2,                         grad = 2 (x-t)/n
 *   bce: x = probabilities (sigmoid applied by the host first, loss.zig:117-119),
 *        redux = -mean [t log p + (1-t) log(1-p)],     grad = (p-t)/n  (w.r.t. the logits)
 * scratch: n/4096 + 2 accumulator-typed slots (r32 for r16/r32, r64 for r64); redux: one accumulator-typed
 * value; grad or redux may be NULL. */
MP_DECL3(mse_loss_i_i, const void* x, void* grad, const void* trg, void* scratch, void* redux, len_t n, StreamContext stream)
MP_DECL3(bce_loss_i_i, const void* x, void* grad, const void* trg, void* scratch, void* redux, len_t n, StreamContext stream)
/* m = alpha*m + clip(g, clip_lo, clip_hi);  w -= rate*m */
MP_DECL3(momentum, void* w, const void* g, void* m, double rate, double alpha, double clip_lo, double clip_hi, len_t n, StreamContext stream)

/* Roadmap operators of the reference beyond rank 2 (NOTES.md:3-5 "General Permutation", NOTES.md:18
 * "_ij,_jk->_ik"); the reference holds the expression grammar (expression_parsing.zig:205-255, :257-317)
 * but no kernels.
 *
 * permutate: dst = permute(src) + alpha*dst for any rank <= MAX_DIMS.  `sizes` are the source sizes and
 * `perm[i]` is the position of source dimension i in the output (the `perm` array that `permutateSizes`
 * derives from "ijk->kij": lhs index i sits at rhs position perm[i]); both are HOST arrays of `rank`
 * entries, read before the call returns.  Bit-exact when alpha = 0.  permutate_ij_ji is the instance
 * sizes = {row, col}, perm = {1, 0}. */
MP_DECL3(permutate, const void* src, void* dst, double alpha, const len_t* sizes, const len_t* perm, len_t rank, StreamContext stream)
/* Batched contractions over densely packed operands, one (m,n)x(n,k) product per batch entry:
 *   bij,bjk->bik : C[b,m,k] = alpha*A[b,m,n]*B[b,n,k]   + beta*C
 *   bij,bkj->bik : C[b,m,k] = alpha*A[b,m,n]*B[b,k,n]^T + beta*C
 *   bji,bjk->bik : C[b,m,k] = alpha*A[b,n,m]^T*B[b,n,k] + beta*C
 * Same tcgen05 kernel as the rank-2 forms over 3-D tensor maps (work unit = batch entry x output tile). */
MP_DECL3(inner_product_bij_bjk_bik, const void* a_data, const void* b_data, const double alpha, void* c_data, const double beta, len_t batch, len_t m, len_t n, len_t k, StreamContext stream)
MP_DECL3(inner_product_bij_bkj_bik, const void* a_data, const void* b_data, const double alpha, void* c_data, const double beta, len_t batch, len_t m, len_t n, len_t k, StreamContext stream)
MP_DECL3(inner_product_bji_bjk_bik, const void* a_data, const void* b_data, const double alpha, void* c_data, const double beta, len_t batch, len_t m, len_t n, len_t k, StreamContext stream)

/* Status word values returned by mpGetStatus (mp_device_utils.h). */
#define MP_STATUS_OK             0u
#define MP_STATUS_WAIT_TIMEOUT   1u  /* a bounded mbarrier wait gave up    */
#define MP_STATUS_BAD_ARGUMENT   2u  /* launcher rejected sizes/alignment  */

#endif
