/*
 * TEST INFRASTRUCTURE -- not part of the product.
 *
 * CPU restatement of the arithmetic of FeatGraph's x86 SpMM / SDDMM kernels
 * (amazon-science/FeatGraph; paths below are relative to that project).  Only
 * tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm
 * may load this library, and only as the checker or the timed CPU baseline.
 *
 * The reference generates its x86 code at run time with Apache TVM v0.7
 * (README.md:22-25), a dependency that is neither vendored nor installable
 * here.  What is restated is therefore the loop nest its tensor expressions
 * and schedules spell out:
 *   - one fp32 accumulator per output element, initialised to 0;
 *   - reduction order: nonzeros of a row in CSR order (SpMM), k ascending
 *     (SDDMM);
 *   - product and sum rounded separately (TVM's generic "llvm" target carries
 *     no FMA feature, so its backend cannot contract) and no reassociation.
 * PARITY PIN: the reference's tests hold no golden vectors for these kernels;
 * they compare against scipy `A.dot(X)` and numpy `(src[col]*dst[row]).sum(-1)`
 * at rtol = atol = 1e-4 (tests/test_module_spmm.py:29-30,
 * tests/test_module_sddmm.py:34-37).  This oracle is pinned to those same
 * checks and to committed fixtures; its bit-level summation order is the
 * documented assumption above, not something TVM itself confirmed here.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math -fopenmp -shared -fPIC
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int fg_oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void fg_oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/*
 * SpMM, CSR, x86 path: python/featgraph/op/vanilla_spmm.py:6-62 with the
 * schedule of :65-80.  Three stages, all inside the timed function:
 *   ReshapedSrcFeat[fo, n, fi] = SrcFeat[n, fo*Fp + fi]                (:43-44)
 *   ReshapedOut[fo, row, fi]   = sum_e vals[e] * Reshaped[fo, idx[e], fi]
 *                                loops (fo, row || , e, fi)         (:46-56, :73)
 *   Out[n, ff]                 = ReshapedOut[ff / Fp, n, ff % Fp]       (:58-60)
 * rows are the parallel axis of every stage (:76-78).  `work` must hold
 * (n_cols + n_rows) * feat_len floats.  Returns 0, or 1 on a bad argument.
 */
int fg_oracle_spmm_csr_f32(int64_t n_rows, int64_t n_cols, int32_t feat_len,
                           const int32_t* indptr, const int32_t* indices,
                           const float* vals, const float* x, float* y,
                           int32_t num_feat_partitions, float* work) {
  if (num_feat_partitions < 1 || feat_len < 1 || !work) return 1;
  const int64_t P = num_feat_partitions;
  const int64_t Fp = feat_len / P; /* the reference assumes feat_len % P == 0 (:41) */
  if (Fp * P != feat_len) return 1;
  float* rx = work;                               /* (P, n_cols, Fp) */
  float* ro = work + (size_t)n_cols * feat_len;   /* (P, n_rows, Fp) */

#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < n_cols; ++n)
    for (int64_t fo = 0; fo < P; ++fo)
      for (int64_t fi = 0; fi < Fp; ++fi)
        rx[(fo * n_cols + n) * Fp + fi] = x[n * feat_len + fo * Fp + fi];

  for (int64_t fo = 0; fo < P; ++fo) {
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t row = 0; row < n_rows; ++row) {
      float* acc = ro + (fo * n_rows + row) * Fp;
      for (int64_t fi = 0; fi < Fp; ++fi) acc[fi] = 0.0f;
      for (int64_t e = indptr[row]; e < indptr[row + 1]; ++e) {
        const float v = vals[e];
        const float* src = rx + (fo * n_cols + (int64_t)indices[e]) * Fp;
        for (int64_t fi = 0; fi < Fp; ++fi) acc[fi] = acc[fi] + v * src[fi];
      }
    }
  }

#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < n_rows; ++n)
    for (int64_t ff = 0; ff < feat_len; ++ff)
      y[n * feat_len + ff] = ro[((ff / Fp) * n_rows + n) * Fp + ff % Fp];
  return 0;
}

/* fp64 "truth" of the same sum (inputs fp32, accumulation and output fp64);
 * used only to attribute error, never as the parity target. */
int fg_oracle_spmm_csr_f64(int64_t n_rows, int32_t feat_len, const int32_t* indptr,
                           const int32_t* indices, const float* vals, const float* x,
                           double* y) {
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t row = 0; row < n_rows; ++row) {
    double* acc = y + row * feat_len;
    for (int64_t f = 0; f < feat_len; ++f) acc[f] = 0.0;
    for (int64_t e = indptr[row]; e < indptr[row + 1]; ++e) {
      const double v = vals[e];
      const float* src = x + (int64_t)indices[e] * feat_len;
      for (int64_t f = 0; f < feat_len; ++f) acc[f] += v * (double)src[f];
    }
  }
  return 0;
}

/*
 * SDDMM, COO: python/featgraph/op/vanilla_sddmm.py:43-47 (one partition) and
 * :48-60 (feature partitions: both inputs are first re-laid-out to
 * (P, N, F/P)), with the x86 schedule of :66-74: loops (fo, e, fi), which
 * visits k = fo*Fp + fi in ascending order for every edge.  src is indexed by
 * COL and dst by ROW (:47).  The reference's x86 schedule is serial (:11, :73);
 * `parallel` != 0 splits the edges over the OpenMP threads instead (a labelled
 * deviation used only for a second baseline figure; the values are the same).
 *
 * num_heads > 1 restates the same loop per head: out[e, h] sums d ascending
 * over src[col[e], h*D + d] * dst[row[e], h*D + d]; the reference has no
 * multi-head kernel, so this case is pinned by nothing in it.
 * With num_feat_partitions > 1 (single head only) `work` must hold
 * (n_cols + n_rows) * feat_len floats; otherwise it may be NULL.
 */
int fg_oracle_sddmm_coo_f32(int64_t nnz, int64_t n_rows, int64_t n_cols, int32_t feat_len,
                            int32_t num_heads, const int32_t* row, const int32_t* col,
                            const float* src, const float* dst, float* out,
                            int32_t num_feat_partitions, int32_t parallel, float* work) {
  if (feat_len < 1 || num_heads < 1 || feat_len % num_heads != 0) return 1;
  if (num_feat_partitions < 1) return 1;
  const int64_t D = feat_len / num_heads;
  if (num_feat_partitions > 1) {
    if (num_heads != 1 || !work) return 1;
    const int64_t P = num_feat_partitions, Fp = feat_len / P;
    if (Fp * P != feat_len) return 1;
    float* rs = work;                             /* (P, n_cols, Fp) */
    float* rd = work + (size_t)n_cols * feat_len; /* (P, n_rows, Fp) */
    for (int64_t n = 0; n < n_cols; ++n)
      for (int64_t k = 0; k < feat_len; ++k)
        rs[((k / Fp) * n_cols + n) * Fp + k % Fp] = src[n * feat_len + k];
    for (int64_t n = 0; n < n_rows; ++n)
      for (int64_t k = 0; k < feat_len; ++k)
        rd[((k / Fp) * n_rows + n) * Fp + k % Fp] = dst[n * feat_len + k];
    for (int64_t e = 0; e < nnz; ++e) out[e] = 0.0f;
    for (int64_t fo = 0; fo < P; ++fo) {
#pragma omp parallel for schedule(static) if (parallel)
      for (int64_t e = 0; e < nnz; ++e) {
        const float* a = rs + (fo * n_cols + (int64_t)col[e]) * Fp;
        const float* b = rd + (fo * n_rows + (int64_t)row[e]) * Fp;
        float acc = out[e];
        for (int64_t fi = 0; fi < Fp; ++fi) acc = acc + a[fi] * b[fi];
        out[e] = acc;
      }
    }
    return 0;
  }
#pragma omp parallel for schedule(static) if (parallel)
  for (int64_t e = 0; e < nnz; ++e) {
    const float* a = src + (int64_t)col[e] * feat_len;
    const float* b = dst + (int64_t)row[e] * feat_len;
    for (int64_t h = 0; h < num_heads; ++h) {
      float acc = 0.0f;
      for (int64_t d = 0; d < D; ++d) acc = acc + a[h * D + d] * b[h * D + d];
      out[e * num_heads + h] = acc;
    }
  }
  return 0;
}

/* fp64 truth of the SDDMM sum. */
int fg_oracle_sddmm_coo_f64(int64_t nnz, int32_t feat_len, int32_t num_heads,
                            const int32_t* row, const int32_t* col, const float* src,
                            const float* dst, double* out) {
  if (feat_len < 1 || num_heads < 1 || feat_len % num_heads != 0) return 1;
  const int64_t D = feat_len / num_heads;
#pragma omp parallel for schedule(static)
  for (int64_t e = 0; e < nnz; ++e) {
    const float* a = src + (int64_t)col[e] * feat_len;
    const float* b = dst + (int64_t)row[e] * feat_len;
    for (int64_t h = 0; h < num_heads; ++h) {
      double acc = 0.0;
      for (int64_t d = 0; d < D; ++d) acc += (double)a[h * D + d] * (double)b[h * D + d];
      out[e * num_heads + h] = acc;
    }
  }
  return 0;
}

/*
 * Generalised SpMM / SDDMM: a binary message function and a reducer in place
 * of multiply and sum.  The reference frames its kernels as "generalized"
 * (README.md:6) but ships only adj_val * feat_val under te.sum
 * (python/featgraph/op/vanilla_spmm.py:53, 121) and Src * Dst under te.sum
 * (python/featgraph/op/vanilla_sddmm.py:47); these two expressions are what is
 * generalised here, in the same loop order, so NOTHING in the reference pins
 * the other operator pairs -- they are defined by this restatement.
 *
 *   msg_op:    0 mul  lhs * rhs      3 div       lhs / rhs
 *              1 add  lhs + rhs      4 copy_lhs  lhs
 *              2 sub  lhs - rhs      5 copy_rhs  rhs
 *   reduce_op: 0 sum  acc + m                      identity 0
 *              1 max  m > acc ? m : acc            identity -FLT_MAX
 *              2 min  m < acc ? m : acc            identity +FLT_MAX
 * The identities of max / min are those of TVM's te.max / te.min reducers (the
 * lowest / highest finite value of the type).  A NaN message never replaces
 * the accumulator of max / min; ties keep the accumulator; so the result is
 * defined for every input and, walked in order, bit-reproducible.
 * SpMM: lhs = X[indices[e], f] (the source vertex's feature), rhs = vals[e] (the
 * edge's value); nonzeros of a row in CSR order.  SDDMM: lhs = src[col[e], k],
 * rhs = dst[row[e], k]; k ascending within a head.
 */
#include <float.h>

static inline float fg_msg(int op, float lhs, float rhs) {
  switch (op) {
    case 0: return lhs * rhs;
    case 1: return lhs + rhs;
    case 2: return lhs - rhs;
    case 3: return lhs / rhs;
    case 4: return lhs;
    default: return rhs;
  }
}

static inline float fg_reduce(int op, float acc, float m) {
  switch (op) {
    case 0: return acc + m;
    case 1: return m > acc ? m : acc;
    default: return m < acc ? m : acc;
  }
}

static inline float fg_identity(int op) { return op == 0 ? 0.0f : (op == 1 ? -FLT_MAX : FLT_MAX); }

int fg_oracle_gspmm_csr_f32(int64_t n_rows, int32_t feat_len, const int32_t* indptr,
                            const int32_t* indices, const float* vals, const float* x,
                            float* y, int32_t msg_op, int32_t reduce_op) {
  if (feat_len < 1 || msg_op < 0 || msg_op > 5 || reduce_op < 0 || reduce_op > 2) return 1;
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t row = 0; row < n_rows; ++row) {
    float* acc = y + row * feat_len;
    for (int64_t f = 0; f < feat_len; ++f) acc[f] = fg_identity(reduce_op);
    for (int64_t e = indptr[row]; e < indptr[row + 1]; ++e) {
      const float v = vals[e];
      const float* src = x + (int64_t)indices[e] * feat_len;
      for (int64_t f = 0; f < feat_len; ++f)
        acc[f] = fg_reduce(reduce_op, acc[f], fg_msg(msg_op, src[f], v));
    }
  }
  return 0;
}

int fg_oracle_gsddmm_coo_f32(int64_t nnz, int32_t feat_len, int32_t num_heads,
                             const int32_t* row, const int32_t* col, const float* src,
                             const float* dst, float* out, int32_t msg_op, int32_t reduce_op) {
  if (feat_len < 1 || num_heads < 1 || feat_len % num_heads != 0) return 1;
  if (msg_op < 0 || msg_op > 5 || reduce_op < 0 || reduce_op > 2) return 1;
  const int64_t D = feat_len / num_heads;
#pragma omp parallel for schedule(static)
  for (int64_t e = 0; e < nnz; ++e) {
    const float* a = src + (int64_t)col[e] * feat_len;
    const float* b = dst + (int64_t)row[e] * feat_len;
    for (int64_t h = 0; h < num_heads; ++h) {
      float acc = fg_identity(reduce_op);
      for (int64_t d = 0; d < D; ++d)
        acc = fg_reduce(reduce_op, acc, fg_msg(msg_op, a[h * D + d], b[h * D + d]));
      out[e * num_heads + h] = acc;
    }
  }
  return 0;
}

/*
 * SpMM over the dense-dense-sparse (DDS) form, the reference's 1-D source-vertex
 * partitioning: python/featgraph/op/vanilla_spmm.py:149-220 with the schedule of
 * :223-246.  The columns are cut into P blocks of width ceil(n_cols / P); block p holds
 * its own CSR (row pointers s1_pos[p * (n_rows + 1) ...], block-local column indices).
 *   Intermediate[p, row, f] = sum_e vals[e] * X[s1_idx[e] + p * width, f]   (:201-213)
 *       e ascending within the block's row, accumulator starting at 0;
 *   Out[row, f] = sum_p Intermediate[p, row, f]                             (:215-218)
 *       p ascending, accumulator starting at 0 (so the first step is 0 + Intermediate[0]).
 * The feature partitioning of the op (fo / fi) only re-lays the arrays out and is left
 * out.  The per-block partial sums make this a DIFFERENT summation order from the CSR
 * op's: the two agree to rounding (the reference's tests compare both with scipy at
 * 1e-4), not bit for bit.  Rows are the parallel axis (:240-243).
 */
int fg_oracle_spmm_dds_f32(int64_t n_rows, int64_t n_cols, int32_t feat_len,
                           int32_t num_col_partitions, const int32_t* s1_pos,
                           const int32_t* s1_idx, const float* vals, const float* x, float* y) {
  if (feat_len < 1 || num_col_partitions < 1) return 1;
  const int64_t P = num_col_partitions;
  const int64_t width = (n_cols + P - 1) / P;
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t row = 0; row < n_rows; ++row) {
    float* out = y + row * feat_len;
    for (int64_t f = 0; f < feat_len; ++f) out[f] = 0.0f;
    for (int64_t p = 0; p < P; ++p) {
      const int64_t beg = s1_pos[p * (n_rows + 1) + row], end = s1_pos[p * (n_rows + 1) + row + 1];
      for (int64_t f = 0; f < feat_len; ++f) {
        float acc = 0.0f;
        for (int64_t e = beg; e < end; ++e)
          acc = acc + vals[e] * x[((int64_t)s1_idx[e] + p * width) * feat_len + f];
        out[f] = out[f] + acc;
      }
    }
  }
  return 0;
}
