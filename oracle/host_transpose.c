/*
 * CPU oracle for out-of-place tensor permutation.  TEST INFRASTRUCTURE ONLY:
 * nothing in the shipped library calls into this file; it is the checker that
 * the CUDA path is compared with, and the "port" CPU baseline that the
 * benchmark times on the host cores.
 *
 * The reference library (cuTT) has no CPU transpose of its own: its tests
 * define correctness through an index formula evaluated on the GPU
 * (src/TensorTester.cu:151-170 builds the constants, src/TensorTester.cu:56-70
 * evaluates them).  This file restates that formula on the host with 64-bit
 * indices:
 *
 *   dim[0] is the fastest-varying dimension; outDim[i] = dim[perm[i]];
 *   for every output linear index o,
 *       out[o] = in[ sum_j ((o / c_j) mod d_j) * ct_j ]
 *   with ct_j = prod_{m<j} dim[m]                 (input stride of rank j)
 *        c_{perm[k]} = prod_{m<k} dim[perm[m]]    (output stride of rank perm[k])
 *        d_j = dim[j].
 *
 * Two implementations are provided:
 *   cutt_oracle_formula  - the formula, literally, one output element at a time;
 *   cutt_oracle_blocked  - an OpenMP nested-loop permutation with 2-D blocking
 *                          over the input-fastest and output-fastest ranks; the
 *                          tests check it against the formula, the benchmark
 *                          uses it as the CPU baseline.
 * Elements are moved as 4- or 8-byte integers so that NaN payloads and signed
 * zeros survive bit for bit.
 *
 * Parity pinning: the reference holds no stored output vectors; its known
 * answers are closed-form (input word w holds the value w, and the checker
 * recomputes the expected source index).  tests/golden/ pins this oracle to
 * that closed form on the reference's own test shapes
 * (src/cutt_test.cpp:138-158, 245-366, 371-404; README.md:94-97).
 */
#include <stdint.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_MAX_RANK 32

/* Validation rules of cuttPlanCheckInput (src/cutt.cpp:59-82). Returns 0 when valid. */
int cutt_oracle_check_input(int rank, const int *dim, const int *perm, size_t elt) {
  if (elt != 4 && elt != 8) return 2;
  if (rank <= 1 || rank > ORACLE_MAX_RANK) return 2;
  int seen[ORACLE_MAX_RANK];
  for (int i = 0; i < rank; i++) {
    if (dim[i] <= 1) return 2;
    seen[i] = 0;
  }
  for (int i = 0; i < rank; i++) {
    if (perm[i] < 0 || perm[i] >= rank || seen[perm[i]]++) return 2;
  }
  return 0;
}

/* c, d, ct of TensorTester::calcTensorConv (src/TensorTester.cu:151-170), 64-bit. */
static void conv_constants(int rank, const int *dim, const int *perm,
                           int64_t *c, int64_t *d, int64_t *ct) {
  c[perm[0]] = 1;
  ct[0] = 1;
  d[0] = dim[0];
  for (int i = 1; i < rank; i++) {
    c[perm[i]] = c[perm[i - 1]] * dim[perm[i - 1]];
    d[i] = dim[i];
    ct[i] = ct[i - 1] * dim[i - 1];
  }
}

/* Source element index for output index o: the sum of src/TensorTester.cu:59-62. */
int64_t cutt_oracle_source_index(int rank, const int *dim, const int *perm, int64_t o) {
  int64_t c[ORACLE_MAX_RANK], d[ORACLE_MAX_RANK], ct[ORACLE_MAX_RANK];
  conv_constants(rank, dim, perm, c, d, ct);
  int64_t src = 0;
  for (int j = 0; j < rank; j++) src += ((o / c[j]) % d[j]) * ct[j];
  return src;
}

int cutt_oracle_formula(int rank, const int *dim, const int *perm, size_t elt,
                        const void *in, void *out) {
  int rc = cutt_oracle_check_input(rank, dim, perm, elt);
  if (rc) return rc;
  int64_t c[ORACLE_MAX_RANK], d[ORACLE_MAX_RANK], ct[ORACLE_MAX_RANK];
  conv_constants(rank, dim, perm, c, d, ct);
  int64_t vol = 1;
  for (int i = 0; i < rank; i++) vol *= dim[i];
#pragma omp parallel for schedule(static)
  for (int64_t o = 0; o < vol; o++) {
    int64_t src = 0;
    for (int j = 0; j < rank; j++) src += ((o / c[j]) % d[j]) * ct[j];
    if (elt == 4) ((uint32_t *)out)[o] = ((const uint32_t *)in)[src];
    else          ((uint64_t *)out)[o] = ((const uint64_t *)in)[src];
  }
  return 0;
}

/*
 * Blocked nested-loop permutation.  Work is split over "outer" positions (all
 * output ranks except the output-fastest rank and the rank that is fastest in
 * the input); inside, a BxB block over those two ranks keeps both the reads and
 * the writes inside a few cache lines.
 */
#define ORACLE_BLOCK 32

#define BLOCKED_BODY(T)                                                                  \
  do {                                                                                   \
    const T *src = (const T *)in;                                                        \
    T *dst = (T *)out;                                                                   \
    if (pa == pb) { /* leading rank unchanged: contiguous row copies */                  \
      _Pragma("omp parallel for schedule(static)")                                       \
      for (int64_t r = 0; r < nouter; r++) {                                             \
        int64_t rem = r, io = 0, oo = 0;                                                 \
        for (int k = 0; k < nod; k++) {                                                  \
          int64_t cc = rem % od[k]; rem /= od[k];                                        \
          io += cc * ois[k]; oo += cc * oos[k];                                          \
        }                                                                                \
        memcpy(dst + oo, src + io, (size_t)da * sizeof(T));                              \
      }                                                                                  \
    } else {                                                                             \
      const int64_t nba = (da + ORACLE_BLOCK - 1) / ORACLE_BLOCK;                        \
      const int64_t nbb = (db + ORACLE_BLOCK - 1) / ORACLE_BLOCK;                        \
      const int64_t nwork = nouter * nba * nbb;                                          \
      _Pragma("omp parallel for schedule(static)")                                       \
      for (int64_t w = 0; w < nwork; w++) {                                              \
        int64_t ba = w % nba, t = w / nba;                                               \
        int64_t bb = t % nbb, rem = t / nbb;                                             \
        int64_t io = 0, oo = 0;                                                          \
        for (int k = 0; k < nod; k++) {                                                  \
          int64_t cc = rem % od[k]; rem /= od[k];                                        \
          io += cc * ois[k]; oo += cc * oos[k];                                          \
        }                                                                                \
        int64_t a0 = ba * ORACLE_BLOCK, a1 = a0 + ORACLE_BLOCK < da ? a0 + ORACLE_BLOCK : da; \
        int64_t b0 = bb * ORACLE_BLOCK, b1 = b0 + ORACLE_BLOCK < db ? b0 + ORACLE_BLOCK : db; \
        for (int64_t a = a0; a < a1; a++) {                                              \
          const T *s = src + io + a * isa;                                               \
          T *q = dst + oo + a * osa;                                                     \
          for (int64_t b = b0; b < b1; b++) q[b * osb] = s[b * isb];                     \
        }                                                                                \
      }                                                                                  \
    }                                                                                    \
  } while (0)

int cutt_oracle_blocked(int rank, const int *dim, const int *perm, size_t elt,
                        const void *in, void *out) {
  int rc = cutt_oracle_check_input(rank, dim, perm, elt);
  if (rc) return rc;
  int64_t is[ORACLE_MAX_RANK], os[ORACLE_MAX_RANK]; /* strides per INPUT rank */
  is[0] = 1;
  for (int i = 1; i < rank; i++) is[i] = is[i - 1] * dim[i - 1];
  int64_t acc = 1;
  for (int k = 0; k < rank; k++) { os[perm[k]] = acc; acc *= dim[perm[k]]; }

  /* pa: rank fastest in the input (0); pb: rank fastest in the output. */
  const int pa = 0, pb = perm[0];
  const int64_t da = dim[pa], db = dim[pb];
  const int64_t isa = is[pa], osa = os[pa], isb = is[pb], osb = os[pb];
  /* the remaining ranks, in output order, enumerate the outer positions */
  int nod = 0;
  int64_t od[ORACLE_MAX_RANK], ois[ORACLE_MAX_RANK], oos[ORACLE_MAX_RANK];
  int64_t nouter = 1;
  for (int k = 0; k < rank; k++) {
    int j = perm[k];
    if (j == pa || j == pb) continue;
    od[nod] = dim[j]; ois[nod] = is[j]; oos[nod] = os[j]; nod++;
    nouter *= dim[j];
  }
  (void)isa; (void)osb;
  if (elt == 4) BLOCKED_BODY(uint32_t);
  else          BLOCKED_BODY(uint64_t);
  return 0;
}

int cutt_oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Sets the number of OpenMP threads later calls use (launchers such as torchrun export
 * OMP_NUM_THREADS=1 to their children). Returns the value now in effect. */
int cutt_oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n >= 1) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}
