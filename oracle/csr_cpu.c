/* TEST INFRASTRUCTURE: CPU restatement in C of the destination-row (CSR) reductions, used only as a checker at
 * full graph sizes and as the timed CPU baseline of bench.py.  Never linked into or called by the product library.
 *
 * What is restated (by the reference file the semantics come from):
 *   csr_gather_sum_*    out[v,:] = sum over in-edges i of row v of x[idx[i],:]      src/ops/dgl_primitives/spmm.cu:375-389
 *                                                                                   (SpMMSrc; SpMMEdge :359-373 with edge ids)
 *   csr_u_mul_e_sum_*   out[v,:] = sum_i x[nid[i],:] * w[eid[i], head]              src/ops/dgl_primitives/spmm.cu:192-356
 *   csr_segment_softmax per destination row, per head, over the edge ids of the row src/ops/segment_softmax/segment_softmax_kernel.cu:4-49
 *                       (true softmax: the maximum starts at -inf, not at 0)
 * Positions of a row are visited in ascending order, as the reference's kernels do.  The `_f32` forms add in
 * float (the reference's arithmetic, and the timed baseline); the `_f64` forms add in double and return double
 * (numerical truth for the parity tests).  An optional per-row factor and max(.,0) reproduce the GCN epilogue.
 *
 * Rows are dealt to OpenMP threads dynamically in blocks (power-law graphs).  Build: oracle/build_oracle_c.py.
 */
#include <math.h>
#include <stdint.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ROW_BLOCK 64

int csr_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void csr_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* out (n_rows, feat) float; rows [row0, row1) only are computed and written (the others are left alone). */
void csr_gather_sum_f32(const int32_t *ptr, const int32_t *idx, int64_t row0, int64_t row1, int64_t feat, const float *x,
                        const float *dst_scale, int relu, float *out) {
#pragma omp parallel for schedule(dynamic, ROW_BLOCK)
  for (int64_t v = row0; v < row1; ++v) {
    float *o = out + v * feat;
    for (int64_t f = 0; f < feat; ++f) o[f] = 0.f;
    for (int64_t i = ptr[v]; i < ptr[v + 1]; ++i) {
      const float *r = x + (int64_t)idx[i] * feat;
      for (int64_t f = 0; f < feat; ++f) o[f] += r[f];
    }
    if (dst_scale) {
      const float s = dst_scale[v];
      for (int64_t f = 0; f < feat; ++f) o[f] *= s;
    }
    if (relu)
      for (int64_t f = 0; f < feat; ++f) o[f] = o[f] > 0.f ? o[f] : 0.f;
  }
}

/* The same sum in double; out is (row1 - row0, feat) double, row v at out + (v - row0) * feat.  The per-row factor
 * and the max are applied to the float-rounded sum, as a float implementation applies them. */
void csr_gather_sum_f64(const int32_t *ptr, const int32_t *idx, int64_t row0, int64_t row1, int64_t feat, const float *x,
                        const float *dst_scale, int relu, double *out) {
#pragma omp parallel for schedule(dynamic, ROW_BLOCK)
  for (int64_t v = row0; v < row1; ++v) {
    double *o = out + (v - row0) * feat;
    for (int64_t f = 0; f < feat; ++f) o[f] = 0.0;
    for (int64_t i = ptr[v]; i < ptr[v + 1]; ++i) {
      const float *r = x + (int64_t)idx[i] * feat;
      for (int64_t f = 0; f < feat; ++f) o[f] += (double)r[f];
    }
    if (dst_scale) {
      const double s = (double)dst_scale[v];
      for (int64_t f = 0; f < feat; ++f) o[f] *= s;
    }
    if (relu)
      for (int64_t f = 0; f < feat; ++f) o[f] = o[f] > 0.0 ? o[f] : 0.0;
  }
}

/* x (n_src, heads * dim), w (n_edges, heads): out[v, h, d] = sum_i x[nid[i], h, d] * w[eid[i], h]; eid may be NULL
 * (position == edge id).  out is (row1 - row0, heads * dim) double. */
void csr_u_mul_e_sum_f64(const int32_t *ptr, const int32_t *nid, const int32_t *eid, int64_t row0, int64_t row1,
                         int64_t heads, int64_t dim, const float *x, const float *w, double *out) {
  const int64_t feat = heads * dim;
#pragma omp parallel for schedule(dynamic, ROW_BLOCK)
  for (int64_t v = row0; v < row1; ++v) {
    double *o = out + (v - row0) * feat;
    for (int64_t f = 0; f < feat; ++f) o[f] = 0.0;
    for (int64_t i = ptr[v]; i < ptr[v + 1]; ++i) {
      const float *r = x + (int64_t)nid[i] * feat;
      const float *wr = w + (int64_t)(eid ? eid[i] : i) * heads;
      for (int64_t h = 0; h < heads; ++h) {
        const double wh = (double)wr[h];
        for (int64_t d = 0; d < dim; ++d) o[h * dim + d] += (double)r[h * dim + d] * wh;
      }
    }
  }
}

/* logits (n_edges, heads) float, indexed by edge id; out (n_edges, heads) double, same indexing.  eid may be NULL. */
void csr_segment_softmax_f64(const int32_t *ptr, const int32_t *eid, int64_t n_rows, int64_t heads, const float *logits,
                             double *out) {
#pragma omp parallel for schedule(dynamic, ROW_BLOCK)
  for (int64_t v = 0; v < n_rows; ++v) {
    for (int64_t h = 0; h < heads; ++h) {
      double m = -INFINITY, s = 0.0;
      for (int64_t i = ptr[v]; i < ptr[v + 1]; ++i) {
        const double z = (double)logits[(int64_t)(eid ? eid[i] : i) * heads + h];
        if (z > m) m = z;
      }
      for (int64_t i = ptr[v]; i < ptr[v + 1]; ++i) s += exp((double)logits[(int64_t)(eid ? eid[i] : i) * heads + h] - m);
      for (int64_t i = ptr[v]; i < ptr[v + 1]; ++i) {
        const int64_t e = (int64_t)(eid ? eid[i] : i) * heads + h;
        out[e] = exp((double)logits[e] - m) / s;
      }
    }
  }
}

/* z[e, h] = sum_d l[src[e], h, d] * r[dst[e], h, d] in double (functor.cuh:103-116 `Dot`, sddmm.cuh:80-120). */
void coo_u_dot_v_f64(const int64_t *src, const int64_t *dst, int64_t n_edges, int64_t heads, int64_t dim, const float *l,
                     const float *r, double *z) {
  const int64_t feat = heads * dim;
#pragma omp parallel for schedule(static, 4096)
  for (int64_t e = 0; e < n_edges; ++e) {
    const float *a = l + src[e] * feat, *b = r + dst[e] * feat;
    for (int64_t h = 0; h < heads; ++h) {
      double s = 0.0;
      for (int64_t d = 0; d < dim; ++d) s += (double)a[h * dim + d] * (double)b[h * dim + d];
      z[e * heads + h] = s;
    }
  }
}

/* y[i,:] = x[gather ? gather[i] : i, :] @ w[type of row i] with types given by a pointer array (segment_mm.cu:4-33),
 * products and sums in double; y is (m, n) double. */
void segment_mm_f64(const float *x, const float *w, const int32_t *type_ptr, int64_t n_types, int64_t k, int64_t n,
                    const int64_t *gather, double *y) {
  for (int64_t t = 0; t < n_types; ++t) {
    const float *wt = w + t * k * n;
#pragma omp parallel for schedule(static, 256)
    for (int64_t i = type_ptr[t]; i < type_ptr[t + 1]; ++i) {
      const float *xi = x + (gather ? gather[i] : i) * k;
      double *yi = y + i * n;
      for (int64_t c = 0; c < n; ++c) yi[c] = 0.0;
      for (int64_t j = 0; j < k; ++j) {
        const double xv = (double)xi[j];
        for (int64_t c = 0; c < n; ++c) yi[c] += xv * (double)wt[j * n + c];
      }
    }
  }
}
