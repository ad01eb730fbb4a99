/*
 * CPU ORACLE - TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A scalar restatement, in plain C, of the op-kernel layer behind the
 * reference's mp.ops / mp.optm.  Only tests/, the smoke check and the
 * benchmark's CPU-baseline leg may load it; the product (the CUDA library
 * under metaphor_b200/) never links or calls it.
 *
 * Each function cites the reference kernel (src/cuda/nvcc_src/<file>:line) or
 * host routine it restates.  Ops the reference names but never implemented
 * (selu, softmax, RMSNorm, SSD scan, SGD/Adam: README.md:81,97; NOTES.md:7-13)
 * are restated from their mathematical definitions.
 *
 * PARITY PINNING.  The reference ships no golden vectors or numeric tests
 * (the programs under src/examples print, they do not assert; example_utils.zig:160-176
 * verifyResults is never called).  The oracle is pinned two ways:
 *   1. the hand-derivable values of src/examples/experimental.zig:19-69
 *      (tests/test_oracle.py), and
 *   2. outputs of the reference's own CUDA kernels, compiled unmodified from
 *      the reference checkout by oracle/build_ref.py into oracle/_ref/ and run on the
 *      GPU (tests/test_reference_kernels.py; fixtures in tests/golden/).
 * For selu, softmax, RMSNorm, SSD, SGD and Adam the reference has neither
 * code nor tests: for those ops parity is unpinned by the reference, and the
 * oracle is cross-checked against torch float64 autograd instead.
 *
 * Single-threaded by design: callers that want all host cores run disjoint
 * row ranges from several threads (every row-wise function is re-entrant).
 *
 * Build: make -C oracle   (gcc -O2 -shared -> liboracle.so)
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_SELU_LAMBDA 1.0507009873554805
#define ORC_SELU_ALPHA 1.6732632423543772

#define REAL float
#define FN(x) x##_f32
#include "oracle_body.inc"
#undef REAL
#undef FN

#define REAL double
#define FN(x) x##_f64
#include "oracle_body.inc"
#undef REAL
#undef FN

/* ---------------------------------------------------------------------------
 * Mamba-2 SSD scan, sequential recurrence, double precision (no reference
 * kernel; definition):
 *   per (batch b, head h), group g = h / (H/G):
 *     a_t = dt[b,t,h] * A[h];  alpha_t = exp(a_t)
 *     S_t = alpha_t * S_{t-1} + dt_t * B_t (x) x_t          S in R^{N x P}, S_{-1} = 0
 *     y_t[p] = sum_n C_t[n] * S_t[n,p]
 * Layouts: x,y [B,L,H,P]; dt [B,L,H]; A [H]; Bm,Cm [B,L,G,N].
 * ------------------------------------------------------------------------- */
void orc_ssd_forward_f64(const double* x, const double* dt, const double* A, const double* Bm, const double* Cm,
                         double* y, size_t nb, size_t L, size_t H, size_t P, size_t N, size_t G) {
  const size_t hpg = H / G;
  for (size_t b = 0; b < nb; ++b)
    for (size_t h = 0; h < H; ++h) {
      const size_t g = h / hpg;
      double* S = (double*)calloc(N * P, sizeof(double));
      for (size_t t = 0; t < L; ++t) {
        const double dtt = dt[(b * L + t) * H + h];
        const double al = exp(dtt * A[h]);
        const double* xt = x + ((b * L + t) * H + h) * P;
        const double* Bt = Bm + ((b * L + t) * G + g) * N;
        const double* Ct = Cm + ((b * L + t) * G + g) * N;
        double* yt = y + ((b * L + t) * H + h) * P;
        for (size_t p = 0; p < P; ++p) yt[p] = 0.0;
        for (size_t n = 0; n < N; ++n) {
          double* Sn = S + n * P;
          const double bn = dtt * Bt[n], cn = Ct[n];
          for (size_t p = 0; p < P; ++p) {
            Sn[p] = al * Sn[p] + bn * xt[p];
            yt[p] += cn * Sn[p];
          }
        }
      }
      free(S);
    }
}

/* Sequential reverse of the recurrence above.  With gy_t = dl/dy_t and
 * lam_t = C_t gy_t^T + alpha_{t+1} lam_{t+1} (lam_L = 0):
 *   gC_t += S_t gy_t;  gx_t = dt_t * lam_t^T B_t;  gB_t += dt_t * lam_t x_t
 *   gdt_t = <lam_t, B_t x_t^T> + A_h*alpha_t*<lam_t, S_{t-1}>;  gA_h += dt_t*alpha_t*<lam_t, S_{t-1}>
 * gB, gC are summed over the heads of a group.  Outputs are overwritten
 * (gradients start at zero).  States S_t of one (b,h) are stored (L*N*P doubles). */
void orc_ssd_reverse_f64(const double* x, const double* dt, const double* A, const double* Bm, const double* Cm,
                         const double* gy, double* gx, double* gdt, double* gA, double* gB, double* gC,
                         size_t nb, size_t L, size_t H, size_t P, size_t N, size_t G) {
  const size_t hpg = H / G;
  memset(gA, 0, H * sizeof(double));
  memset(gB, 0, nb * L * G * N * sizeof(double));
  memset(gC, 0, nb * L * G * N * sizeof(double));
  double* S = (double*)malloc((L + 1) * N * P * sizeof(double));
  double* lam = (double*)malloc(N * P * sizeof(double));
  for (size_t b = 0; b < nb; ++b)
    for (size_t h = 0; h < H; ++h) {
      const size_t g = h / hpg;
      memset(S, 0, N * P * sizeof(double)); /* S[0] = S_{-1} */
      for (size_t t = 0; t < L; ++t) {
        const double dtt = dt[(b * L + t) * H + h];
        const double al = exp(dtt * A[h]);
        const double* xt = x + ((b * L + t) * H + h) * P;
        const double* Bt = Bm + ((b * L + t) * G + g) * N;
        const double* Sp = S + t * N * P;
        double* Sc = S + (t + 1) * N * P;
        for (size_t n = 0; n < N; ++n)
          for (size_t p = 0; p < P; ++p) Sc[n * P + p] = al * Sp[n * P + p] + dtt * Bt[n] * xt[p];
      }
      memset(lam, 0, N * P * sizeof(double));
      double al_next = 0.0;
      for (size_t tt = L; tt-- > 0;) {
        const size_t t = tt;
        const double dtt = dt[(b * L + t) * H + h];
        const double al = exp(dtt * A[h]);
        const double* xt = x + ((b * L + t) * H + h) * P;
        const double* gyt = gy + ((b * L + t) * H + h) * P;
        const double* Bt = Bm + ((b * L + t) * G + g) * N;
        const double* Ct = Cm + ((b * L + t) * G + g) * N;
        const double* Sp = S + t * N * P;
        const double* Sc = S + (t + 1) * N * P;
        double* gxt = gx + ((b * L + t) * H + h) * P;
        double* gBt = gB + ((b * L + t) * G + g) * N;
        double* gCt = gC + ((b * L + t) * G + g) * N;
        for (size_t p = 0; p < P; ++p) gxt[p] = 0.0;
        double d_bx = 0.0, d_sp = 0.0;
        for (size_t n = 0; n < N; ++n) {
          double gc = 0.0, gb = 0.0;
          for (size_t p = 0; p < P; ++p) {
            const double l = Ct[n] * gyt[p] + al_next * lam[n * P + p];
            lam[n * P + p] = l;
            gc += Sc[n * P + p] * gyt[p];
            gb += l * xt[p];
            gxt[p] += dtt * l * Bt[n];
            d_bx += l * Bt[n] * xt[p];
            d_sp += l * Sp[n * P + p];
          }
          gCt[n] += gc;
          gBt[n] += dtt * gb;
        }
        gdt[(b * L + t) * H + h] = d_bx + A[h] * al * d_sp;
        gA[h] += dtt * al * d_sp;
        al_next = al;
      }
    }
  free(S);
  free(lam);
}

