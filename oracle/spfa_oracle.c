/*
 * spfa_oracle.c -- CPU restatement of the reference's six sparse FlashAttention forward operators.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker the CUDA library is compared against; it is
 * never linked into, imported by or called from the product library. Only the test-suite, the
 * smoke check and the benchmark's CPU-baseline leg may load it.
 *
 * What it restates (paths relative to the reference tree):
 *   index sets   Sparse_FlashAttention_CSR/sp_flatt_csr_kernel.cu:29-33,117
 *                Sparse_FlashAttention_COO/sp_flatt_coo_kernel.cu:47-79,152
 *                Sparse_FlashAttention_Local/sp_flatt_local_kernel.cu:24-28,101
 *                Sparse_FlashAttention_Local_1D_Dilated/sp_flatt_local_1d_dilated_kernel.cu:25-29,102
 *                Sparse_FlashAttention_Local_2D_Dilated/sp_flatt_local_2d_dilated_kernel.cu:26-39,123
 *                Sparse_FlashAttention_Global_No_Local/sp_flatt_global_no_local_kernel.cu:38-64,135-162
 *   arithmetic   sp_flatt_csr_kernel.cu:130-201 (identical in all six): s = q.k/sqrt(d), online
 *                softmax with running (m, l) and a normalised O, merged into the caller's state.
 * The arithmetic here is carried in fp64 and evaluated in one pass over the whole key list of a row,
 * which is the exact value the reference's chunked fp32 recurrence approximates.
 *
 * Parity pin: checked against fixtures produced by running the reference's own
 * verification/verify.py (mask builders and SDPA-MATH outputs) -- see tests/golden/.
 *
 * Two index modes:
 *   ref_mepi == 0  closed-form index set (what the reference documents and what verify.py builds)
 *   ref_mepi  > 0  the key list the UNPATCHED reference kernel really walks with that
 *                  maskElePerIter: last chunk dropped when the count is an exact multiple >= 2x
 *                  (sp_flatt_csr_kernel.cu:98-109) and, for the dilated kernels, the window base
 *                  advanced by maskElePerIter instead of maskElePerIter*(dil+1)
 *                  (sp_flatt_local_1d_dilated_kernel.cu:111, sp_flatt_local_2d_dilated_kernel.cu:132).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum { K_LOCAL = 0, K_L1D = 1, K_L2D = 2, K_GNL = 3 };

static inline int64_t i64max(int64_t a, int64_t b) { return a > b ? a : b; }
static inline int64_t i64min(int64_t a, int64_t b) { return a < b ? a : b; }

/* maskElePerIter as the reference computes it on a GPU with 48 KiB default shared memory, where
 * sizeof(Q.type()) is the size of a type-properties object (8), not of an element
 * (sp_flatt_csr_kernel.cu:260-261; COO :300-301 subtracts two ints; global :316-317 adds ints). */
int64_t spfa_oracle_ref_mepi(int family, int d) {
  const int64_t smem = 49152, ts = 8;
  switch (family) {
    case 0: /* csr, local, 1d, 2d */ return (smem - 2 * d * ts - 6 * ts) / (ts + 2 * d * ts);
    case 1: /* coo */ return (smem - 2 * d * ts - 6 * ts - 8) / (ts + 2 * d * ts);
    default: /* global */ return (smem - 2 * d * ts - 6 * ts - 4) / (ts + 4 + 2 * d * ts);
  }
}

/* Walks `tot` logical key slots the way the reference's chunk loop does and appends the slots it
 * really visits to `slot_out` (as slot numbers 0..tot-1 for stride-1 families). Returns the count.
 * For the dilated families the visited COLUMN is base + chunk_base + t*s with chunk_base advanced
 * by mepi (not mepi*s); it is returned directly as a column through `col_out`. */
static int64_t walk_ref_chunks(int64_t tot, int64_t mepi_cfg, int64_t base, int64_t s, int dilated_bug,
                               uint32_t* col_out) {
  if (tot <= 0) return 0;
  int64_t mepi = tot < mepi_cfg ? tot : mepi_cfg;
  int64_t iters = (int64_t)ceilf((float)tot / (float)mepi);
  int64_t last = tot % mepi;
  int64_t low = base, n = 0;
  for (int64_t b = 0; b < iters; ++b) {
    if (b == iters - 1 && b != 0) mepi = last;
    for (int64_t t = 0; t < mepi; ++t) {
      if (col_out) col_out[n] = (uint32_t)(low + t * s);
      ++n;
    }
    low += dilated_bug ? mepi : mepi * s;
  }
  return n;
}

/* Key list of row i for an implicit mask, in visiting order. out may be NULL (count only).
 * p0/p1: local(w,-), 1d(w,dil), 2d(B,dil), global(w,-). */
int64_t spfa_oracle_row_cols(int kind, int64_t i, int64_t L, int64_t p0, int64_t p1,
                             const int32_t* G, int64_t nG, int64_t ref_mepi, uint32_t* out) {
  if (kind == K_LOCAL) {
    int64_t lo = i64max(0, i - p0), hi = i64min(L, i + p0 + 1), n = hi - lo;
    if (ref_mepi > 0) return walk_ref_chunks(n, ref_mepi, lo, 1, 0, out);
    if (out) for (int64_t t = 0; t < n; ++t) out[t] = (uint32_t)(lo + t);
    return n;
  }
  if (kind == K_L1D) {
    int64_t s = p1 + 1;
    int64_t lo = i64max(i - p0 * s, i % s), hi = i64min(i + p0 * s, L - 1);
    int64_t n = (hi - lo) / s + 1;
    if (ref_mepi > 0) return walk_ref_chunks(n, ref_mepi, lo, s, 1, out);
    if (out) for (int64_t t = 0; t < n; ++t) out[t] = (uint32_t)(lo + t * s);
    return n;
  }
  if (kind == K_L2D) {
    int64_t s = p1 + 1, B = p0, start = (i / B) * B;
    if ((i - start) % s != 0) return 0;
    int64_t n = i64min(B, (B - 1) / s + 1);
    if (ref_mepi > 0) return walk_ref_chunks(n, ref_mepi, start, s, 1, out);
    if (out) for (int64_t t = 0; t < n; ++t) out[t] = (uint32_t)(start + t * s);
    return n;
  }
  /* global-no-local */
  int64_t lo = i64max(0, i - p0), hi = i64min(L, i + p0 + 1); /* window [lo, hi) */
  int is_global = 0;
  for (int64_t t = 0; t < nG; ++t) { /* membership scan, sp_flatt_global_no_local_kernel.cu:47-64 */
    if ((int64_t)G[t] == i) { is_global = 1; break; }
  }
  int64_t n = 0;
  if (is_global) {
    for (int64_t j = 0; j < L; ++j) {
      if (j >= lo && j < hi) continue;
      if (out) out[n] = (uint32_t)j;
      ++n;
    }
  } else {
    for (int64_t t = 0; t < nG; ++t) {
      int64_t g = G[t];
      if (g >= lo && g < hi) continue;
      if (out) out[n] = (uint32_t)g;
      ++n;
    }
  }
  if (ref_mepi > 0 && n >= 2 * ref_mepi && n % ref_mepi == 0) n -= ref_mepi; /* dropped last chunk */
  return n;
}

/* One row of attention over an explicit key list, fp64, merged into the (m, l, O) state.
 * Restates the update of sp_flatt_csr_kernel.cu:130-201 evaluated over the whole list at once. */
static void attend_row(const float* q, const float* K, const float* V, const uint32_t* cols, int64_t n,
                       int64_t Lk, int d, double* m, double* l, double* O, double* sbuf) {
  if (n <= 0) return;
  const double scale = 1.0 / sqrt((double)d);
  double mloc = -INFINITY;
  int64_t nv = 0;
  for (int64_t t = 0; t < n; ++t) {
    int64_t c = cols[t];
    if (c >= Lk) { sbuf[t] = -INFINITY; continue; }
    const float* k = K + c * d;
    double acc = 0.0;
    for (int e = 0; e < d; ++e) acc += (double)q[e] * (double)k[e];
    sbuf[t] = acc * scale;
    if (sbuf[t] > mloc) mloc = sbuf[t];
    ++nv;
  }
  if (nv == 0) return;
  double m_in = *m, l_in = *l;
  double m_out = m_in > mloc ? m_in : mloc;
  double a = l_in * exp(m_in - m_out);
  double lsum = 0.0;
  double* acc = (double*)calloc((size_t)d, sizeof(double));
  for (int64_t t = 0; t < n; ++t) {
    if ((int64_t)cols[t] >= Lk) continue;
    double p = exp(sbuf[t] - m_out);
    lsum += p;
    const float* v = V + (int64_t)cols[t] * d;
    for (int e = 0; e < d; ++e) acc[e] += p * (double)v[e];
  }
  double l_out = a + lsum;
  for (int e = 0; e < d; ++e) O[e] = (a * O[e] + acc[e]) / l_out; /* 0*NaN stays NaN, as in the reference */
  *m = m_out;
  *l = l_out;
  free(acc);
}

static void nan_fill(double* O, int d) {
  for (int e = 0; e < d; ++e) O[e] = NAN;
}

/* CSR forward over rows [0, n_rows): state arrays are fp64. */
void spfa_oracle_csr_forward(const float* Q, const float* K, const float* V,
                             const uint64_t* row_off, const uint32_t* col,
                             double* m, double* l, double* O,
                             int64_t n_rows, int64_t Lk, int d, int use_nan, int64_t ref_mepi) {
#pragma omp parallel
  {
    double* sbuf = NULL;
    int64_t cap = 0;
#pragma omp for schedule(dynamic, 64)
    for (int64_t r = 0; r < n_rows; ++r) {
      int64_t lo = (int64_t)row_off[r], n = (int64_t)row_off[r + 1] - lo;
      if (n <= 0) {
        if (use_nan) nan_fill(O + r * d, d);
        continue;
      }
      if (ref_mepi > 0 && n >= 2 * ref_mepi && n % ref_mepi == 0) n -= ref_mepi;
      if (n > cap) { cap = n * 2; sbuf = (double*)realloc(sbuf, (size_t)cap * sizeof(double)); }
      attend_row(Q + r * d, K, V, col + lo, n, Lk, d, m + r, l + r, O + r * d, sbuf);
    }
    free(sbuf);
  }
}

/* COO forward: rows [row_begin, row_begin+n_rows) of a row-sorted COO list.
 * Row r owns entries [first index with row==r, first index with row>r)  (sp_flatt_coo_kernel.cu:47-79). */
void spfa_oracle_coo_forward(const float* Q, const float* K, const float* V,
                             const uint64_t* row, const uint32_t* col, int64_t nnz,
                             double* m, double* l, double* O,
                             int64_t row_begin, int64_t n_rows, int64_t Lk, int d, int use_nan,
                             int64_t ref_mepi) {
  uint64_t* off = (uint64_t*)malloc((size_t)(n_rows + 1) * sizeof(uint64_t));
  int64_t k = 0;
  for (int64_t r = 0; r <= n_rows; ++r) {
    while (k < nnz && (int64_t)row[k] < row_begin + r) ++k;
    off[r] = (uint64_t)k;
  }
  spfa_oracle_csr_forward(Q, K, V, off, col, m, l, O, n_rows, Lk, d, use_nan, ref_mepi);
  free(off);
}

/* Implicit-mask forward over absolute rows [row_begin, row_end); Q/m/l/O start at row_begin. */
void spfa_oracle_implicit_forward(int kind, const float* Q, const float* K, const float* V,
                                  double* m, double* l, double* O,
                                  int64_t L, int d, int64_t p0, int64_t p1,
                                  const int32_t* G, int64_t nG, int use_nan,
                                  int64_t row_begin, int64_t row_end, int64_t ref_mepi) {
#pragma omp parallel
  {
    uint32_t* cols = NULL;
    double* sbuf = NULL;
    int64_t cap = 0;
#pragma omp for schedule(dynamic, 16)
    for (int64_t i = row_begin; i < row_end; ++i) {
      int64_t r = i - row_begin;
      int64_t n = spfa_oracle_row_cols(kind, i, L, p0, p1, G, nG, ref_mepi, NULL);
      if (n <= 0) {
        if (use_nan && kind == K_L2D) nan_fill(O + r * d, d);
        continue;
      }
      if (n > cap) {
        cap = n * 2;
        cols = (uint32_t*)realloc(cols, (size_t)cap * sizeof(uint32_t));
        sbuf = (double*)realloc(sbuf, (size_t)cap * sizeof(double));
      }
      spfa_oracle_row_cols(kind, i, L, p0, p1, G, nG, ref_mepi, cols);
      attend_row(Q + r * d, K, V, cols, n, L, d, m + r, l + r, O + r * d, sbuf);
    }
    free(cols);
    free(sbuf);
  }
}

/* Index set of an implicit mask as CSR: pass 1 with cols == NULL fills counts via row_off[r+1]-row_off[r]
 * being written as counts into row_off[1..]; the caller prefix-sums. Here done in one call:
 * row_off[n_rows+1] is written; if cols != NULL it must have row_off[n_rows] entries (call twice). */
int64_t spfa_oracle_implicit_csr(int kind, int64_t L, int64_t p0, int64_t p1,
                                 const int32_t* G, int64_t nG, int64_t row_begin, int64_t row_end,
                                 int64_t ref_mepi, uint64_t* row_off, uint32_t* cols) {
  int64_t n_rows = row_end - row_begin;
  row_off[0] = 0;
  for (int64_t r = 0; r < n_rows; ++r) {
    int64_t n = spfa_oracle_row_cols(kind, row_begin + r, L, p0, p1, G, nG, ref_mepi,
                                     cols ? cols + row_off[r] : NULL);
    row_off[r + 1] = row_off[r] + (uint64_t)n;
  }
  return (int64_t)row_off[n_rows];
}
