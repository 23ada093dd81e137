/*
 * dnpeff_oracle.c -- TEST INFRASTRUCTURE ONLY.
 *
 * A host-CPU restatement of the D-NPEFF multiplicative-update NMF path of
 * mmatena/npeff_ref (the `run_nmf_on_pefs` executable).  It is the checker the
 * CUDA engine is compared against and the timed CPU baseline; it is never
 * linked into, imported by, or called from the shipped library.
 *
 * Parity status: PARITY UNPINNED by reference tests.  The reference holds no
 * test, golden vector or fixture for cc/cuda_d_npeff.  The only pinned
 * behaviour nearby is the column-pruning known-answer test of the sibling
 * tree (cc/cuda_lrm_npeff/src/preprocess/column_pruning_test.cc:12-105), whose
 * algorithm is the same scheme as util/sparse_util.h:79-159; this oracle is
 * checked against those four cases.  Where the reference engine could be run
 * on a GPU box from the harness in this folder, its outputs are committed as
 * fixtures and this oracle is checked against them as well.
 *
 * Layouts used here (all fp32 storage):
 *   A    CSR: vals[nnz], colind[nnz] (int32), rowptr[n+1] (int64)
 *   W    n x r, row-major (one example's r coefficients contiguous)
 *   Ht   m x r, row-major (one feature's r component values contiguous).
 *        This is the reference's column-major r x m device matrix H
 *        (multi_mu_dense_factors_device_contexts1.h:413-429), byte for byte.
 *
 * Accumulation precision is selectable per call: acc64 != 0 accumulates every
 * contraction in double (the "truth" rendering), acc64 == 0 in float (what a
 * fp32 engine can be expected to match most closely).  Storage, the
 * elementwise update and its evaluation order are fp32 in both renderings.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

ORACLE_API void oracle_set_num_threads(int t) {
#ifdef _OPENMP
    if (t > 0) omp_set_num_threads(t);
#else
    (void)t;
#endif
}

/* ------------------------------------------------------------------------- */
/* Counter-based uniform generator shared (bit for bit) with the CUDA engine.
 * The reference draws cuRAND XORWOW uniforms in (0,1]
 * (multi_mu_dense_factors_device_contexts1.h:197-207); a closed library stream
 * cannot be reproduced, so both sides use this hash instead and the reference
 * range (0,1] is kept.  Index = position in the row-major factor, so a column
 * shard sees the same values as the unsharded matrix. */
static inline uint64_t mix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

static inline float uniform01(uint64_t seed, uint64_t stream, uint64_t index) {
    uint64_t h = mix64(mix64(seed ^ (stream * 0xD1B54A32D192ED03ull)) + index);
    return (float)((uint32_t)(h >> 40) + 1u) * (1.0f / 16777216.0f);
}

/* out[i] = scale * U(0,1], i in [0,count), global index = first + i.
 * stream 0 is W, stream 1 is H. */
ORACLE_API void oracle_init_uniform(float* out, int64_t first, int64_t count,
                                    uint64_t seed, uint64_t stream, float scale) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < count; i++)
        out[i] = uniform01(seed, stream, (uint64_t)(first + i)) * scale;
}

/* ------------------------------------------------------------------------- */
/* io/pef_fisher_h5.h:38-52 -- val /= (norm_row + eps), eps = 1e-9f, float. */
ORACLE_API void oracle_normalize_rows(float* vals, const int64_t* rowptr, int64_t n,
                                      const float* norms, float eps) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) {
        float d = norms[i] + eps;
        for (int64_t p = rowptr[i]; p < rowptr[i + 1]; p++) vals[p] /= d;
    }
}

/* util/sparse_util.h:79-159 -- count explicit entries per column (int
 * counters), keep columns with count >= min_count, renumber kept columns in
 * ascending order, compact the CSR in place keeping the within-row order.
 * Empty rows stay as empty rows.  new_to_og must hold n_cols entries; returns
 * the number of kept columns; *nnz_out is the new nnz. */
ORACLE_API int64_t oracle_prune_columns(float* vals, int32_t* colind, int64_t* rowptr,
                                        int64_t n, int64_t n_cols, int32_t min_count,
                                        int32_t* new_to_og, int64_t* nnz_out) {
    int64_t nnz = rowptr[n];
    int32_t* cnt = (int32_t*)calloc((size_t)(n_cols > 0 ? n_cols : 1), sizeof(int32_t));
    int32_t* og_to_new = (int32_t*)malloc(sizeof(int32_t) * (size_t)(n_cols > 0 ? n_cols : 1));
    for (int64_t p = 0; p < nnz; p++) cnt[colind[p]] += 1;
    int64_t kept = 0;
    for (int64_t c = 0; c < n_cols; c++) {
        if (cnt[c] >= min_count) {
            og_to_new[c] = (int32_t)kept;
            new_to_og[kept++] = (int32_t)c;
        } else {
            og_to_new[c] = -1;
        }
    }
    int64_t q = 0;
    for (int64_t i = 0; i < n; i++) {
        int64_t b = rowptr[i], e = rowptr[i + 1];
        rowptr[i] = q;
        for (int64_t p = b; p < e; p++) {
            int32_t c = og_to_new[colind[p]];
            if (c != -1) {
                colind[q] = c;
                vals[q] = vals[p];
                q++;
            }
        }
        /* rowptr[i+1] still holds the old end; the next iteration reads it as
         * its begin before overwriting it. */
    }
    rowptr[n] = q;
    *nnz_out = q;
    free(cnt);
    free(og_to_new);
    return kept;
}

/* util/matrix_util.h:10-20 -- equal-width contiguous ranges, the last one
 * takes the remainder. */
ORACLE_API void oracle_split_range(int64_t total, int64_t n_splits, int64_t idx,
                                   int64_t* start, int64_t* size) {
    int64_t base = total / n_splits;
    *start = base * idx;
    *size = (idx == n_splits - 1) ? base + (total % n_splits) : base;
}

/* util/matrix_util.h:24-69 -- extract columns [c0, c0+w) of a CSR, rebasing
 * the column ids to the range start and keeping the within-row order.
 * Pass out arrays == NULL to only count; returns the shard nnz. */
ORACLE_API int64_t oracle_split_columns(const float* vals, const int32_t* colind,
                                        const int64_t* rowptr, int64_t n, int64_t c0, int64_t w,
                                        float* ovals, int32_t* ocolind, int64_t* orowptr) {
    int64_t q = 0;
    for (int64_t i = 0; i < n; i++) {
        if (orowptr) orowptr[i] = q;
        for (int64_t p = rowptr[i]; p < rowptr[i + 1]; p++) {
            int64_t c = colind[p];
            if (c >= c0 && c < c0 + w) {
                if (ovals) {
                    ovals[q] = vals[p];
                    ocolind[q] = (int32_t)(c - c0);
                }
                q++;
            }
        }
    }
    if (orowptr) orowptr[n] = q;
    return q;
}

/* Stable counting-sort transpose: CSR (n x m) -> CSC, rows ascending within a
 * column.  (The reference lets cuSPARSE apply op(A)=A^T to the CSR; a CPU
 * rendering needs the explicit transpose.) */
ORACLE_API void oracle_csr_to_csc(const float* vals, const int32_t* colind, const int64_t* rowptr,
                                  int64_t n, int64_t m, float* cvals, int32_t* crow,
                                  int64_t* colptr) {
    memset(colptr, 0, sizeof(int64_t) * (size_t)(m + 1));
    int64_t nnz = rowptr[n];
    for (int64_t p = 0; p < nnz; p++) colptr[colind[p] + 1]++;
    for (int64_t c = 0; c < m; c++) colptr[c + 1] += colptr[c];
    int64_t* cur = (int64_t*)malloc(sizeof(int64_t) * (size_t)(m > 0 ? m : 1));
    memcpy(cur, colptr, sizeof(int64_t) * (size_t)m);
    for (int64_t i = 0; i < n; i++)
        for (int64_t p = rowptr[i]; p < rowptr[i + 1]; p++) {
            int64_t q = cur[colind[p]]++;
            cvals[q] = vals[p];
            crow[q] = (int32_t)i;
        }
    free(cur);
}

/* ------------------------------------------------------------------------- */
/* Contractions.  Each has a float-accumulate and a double-accumulate body.   */

/* out[i,:] = sum_p vals[p] * D[ind[p],:]   (S is rows x ?, D is ? x r).
 * Used for A*H^T (S = CSR(A), D = Ht) and for A^T*W (S = CSC(A), D = W):
 * the two cusparseSpMM calls at
 * multi_mu_dense_factors_device_contexts1.h:255-265. */
ORACLE_API void oracle_spmm(const float* vals, const int32_t* ind, const int64_t* ptr,
                            int64_t rows, const float* D, int64_t r, float* out, int acc64) {
#pragma omp parallel
    {
        double* accd = (double*)malloc(sizeof(double) * (size_t)r);
        float* accf = (float*)malloc(sizeof(float) * (size_t)r);
#pragma omp for schedule(dynamic, 16)
        for (int64_t i = 0; i < rows; i++) {
            if (acc64) {
                for (int64_t c = 0; c < r; c++) accd[c] = 0.0;
                for (int64_t p = ptr[i]; p < ptr[i + 1]; p++) {
                    const float* d = D + (int64_t)ind[p] * r;
                    double v = vals[p];
                    for (int64_t c = 0; c < r; c++) accd[c] += v * (double)d[c];
                }
                for (int64_t c = 0; c < r; c++) out[i * r + c] = (float)accd[c];
            } else {
                for (int64_t c = 0; c < r; c++) accf[c] = 0.0f;
                const int64_t pe = ptr[i + 1];
                for (int64_t p = ptr[i]; p < pe; p++) {
                    /* the gathered rows of D miss every cache level when D is large:
                     * ask for the row of the entry eight places ahead now */
                    if (p + 8 < pe) {
                        const char* nx = (const char*)(D + (int64_t)ind[p + 8] * r);
                        for (int64_t b = 0; b < r * 4; b += 64) __builtin_prefetch(nx + b, 0, 1);
                    }
                    const float* d = D + (int64_t)ind[p] * r;
                    float v = vals[p];
                    for (int64_t c = 0; c < r; c++) accf[c] += v * d[c];
                }
                for (int64_t c = 0; c < r; c++) out[i * r + c] = accf[c];
            }
        }
        free(accd);
        free(accf);
    }
}

/* G = X^T X for X rows x r row-major; G is r x r.  H*H^T and W^T*W of
 * multi_mu_dense_factors_device_contexts1.h:303,322. */
ORACLE_API void oracle_gram(const float* X, int64_t rows, int64_t r, float* G, int acc64) {
    int nt = oracle_num_threads();
    double* part = (double*)calloc((size_t)nt * (size_t)(r * r), sizeof(double));
#pragma omp parallel
    {
#ifdef _OPENMP
        int t = omp_get_thread_num();
#else
        int t = 0;
#endif
        double* pd = part + (size_t)t * (size_t)(r * r);
        float* pf = (float*)calloc((size_t)(r * r), sizeof(float));
#pragma omp for schedule(static)
        for (int64_t i = 0; i < rows; i++) {
            const float* x = X + i * r;
            if (acc64) {
                for (int64_t a = 0; a < r; a++) {
                    double xa = x[a];
                    for (int64_t b = 0; b < r; b++) pd[a * r + b] += xa * (double)x[b];
                }
            }
        }
        if (!acc64) {
            /* float rendering: the same sums, rows added in the same order, but eight
             * rows per pass over the r x r partial so that it is not re-read per row */
            int64_t lo, hi;
            {
#ifdef _OPENMP
                int nth = omp_get_num_threads();
#else
                int nth = 1;
#endif
                lo = rows * t / nth;
                hi = rows * (t + 1) / nth;
            }
            for (int64_t i0 = lo; i0 < hi; i0 += 8) {
                const int nb = (int)(hi - i0 < 8 ? hi - i0 : 8);
                for (int64_t a = 0; a < r; a++) {
                    float xa[8];
                    for (int j = 0; j < nb; j++) xa[j] = X[(i0 + j) * r + a];
                    float* pr = pf + a * r;
                    for (int j = 0; j < nb; j++) {
                        const float* xj = X + (i0 + j) * r;
                        const float v = xa[j];
                        for (int64_t b = 0; b < r; b++) pr[b] += v * xj[b];
                    }
                }
            }
        }
        if (!acc64)
            for (int64_t e = 0; e < r * r; e++) pd[e] = pf[e];
        free(pf);
    }
    for (int64_t e = 0; e < r * r; e++) {
        if (acc64) {
            double s = 0.0;
            for (int t = 0; t < nt; t++) s += part[(size_t)t * (size_t)(r * r) + e];
            G[e] = (float)s;
        } else {
            float s = 0.0f;
            for (int t = 0; t < nt; t++) s += (float)part[(size_t)t * (size_t)(r * r) + e];
            G[e] = s;
        }
    }
    free(part);
}

/* X[i,c] *= Num[i,c] / (sum_t X[i,t]*G[t,c] + eps), the dense product of
 * multi_mu_dense_factors_device_contexts1.h:306,329 followed by
 * kernelNmfMuUpdate (nmf/sparse/kernels.h:31-33): add eps, divide, multiply,
 * all in float. */
ORACLE_API void oracle_mu_update(float* X, const float* Num, const float* G, int64_t rows,
                                 int64_t r, float eps, int acc64) {
#pragma omp parallel
    {
        float* den = (float*)malloc(sizeof(float) * (size_t)r);
        double* dd = (double*)malloc(sizeof(double) * (size_t)r);
        /* float rendering, four rows at a time: the same sums over t in the same order,
         * with a 4 x 32 block of denominators held in registers while G streams by */
        if (!acc64) {
            float* den4 = (float*)malloc(sizeof(float) * 4 * (size_t)r);
#pragma omp for schedule(static)
            for (int64_t i0 = 0; i0 < rows; i0 += 4) {
                const int nb = (int)(rows - i0 < 4 ? rows - i0 : 4);
                const float* x0 = X + i0 * r;
                const float* x1 = X + (i0 + (nb > 1 ? 1 : 0)) * r;
                const float* x2 = X + (i0 + (nb > 2 ? 2 : 0)) * r;
                const float* x3 = X + (i0 + (nb > 3 ? 3 : 0)) * r;
                for (int64_t c0 = 0; c0 < r; c0 += 32) {
                    const int cw = (int)(r - c0 < 32 ? r - c0 : 32);
                    float a0[32], a1[32], a2[32], a3[32];
                    for (int c = 0; c < 32; c++) a0[c] = a1[c] = a2[c] = a3[c] = 0.0f;
                    if (cw == 32) {
                        for (int64_t t = 0; t < r; t++) {
                            const float* g = G + t * r + c0;
                            const float v0 = x0[t], v1 = x1[t], v2 = x2[t], v3 = x3[t];
                            for (int c = 0; c < 32; c++) {
                                a0[c] += v0 * g[c];
                                a1[c] += v1 * g[c];
                                a2[c] += v2 * g[c];
                                a3[c] += v3 * g[c];
                            }
                        }
                    } else {
                        for (int64_t t = 0; t < r; t++) {
                            const float* g = G + t * r + c0;
                            const float v0 = x0[t], v1 = x1[t], v2 = x2[t], v3 = x3[t];
                            for (int c = 0; c < cw; c++) {
                                a0[c] += v0 * g[c];
                                a1[c] += v1 * g[c];
                                a2[c] += v2 * g[c];
                                a3[c] += v3 * g[c];
                            }
                        }
                    }
                    for (int c = 0; c < cw; c++) {
                        den4[0 * r + c0 + c] = a0[c];
                        den4[1 * r + c0 + c] = a1[c];
                        den4[2 * r + c0 + c] = a2[c];
                        den4[3 * r + c0 + c] = a3[c];
                    }
                }
                for (int j = 0; j < nb; j++) {
                    float* x = X + (i0 + j) * r;
                    const float* nu = Num + (i0 + j) * r;
                    const float* dj = den4 + (size_t)j * (size_t)r;
                    for (int64_t c = 0; c < r; c++) {
                        volatile float q = nu[c] / (dj[c] + eps); /* no fused reassociation */
                        x[c] = x[c] * q;
                    }
                }
            }
            free(den4);
        }
#pragma omp for schedule(static)
        for (int64_t i = 0; i < (acc64 ? rows : 0); i++) {
            float* x = X + i * r;
            if (acc64) {
                for (int64_t c = 0; c < r; c++) dd[c] = 0.0;
                for (int64_t t = 0; t < r; t++) {
                    double xt = x[t];
                    const float* g = G + t * r;
                    for (int64_t c = 0; c < r; c++) dd[c] += xt * (double)g[c];
                }
                for (int64_t c = 0; c < r; c++) den[c] = (float)dd[c];
            } else {
                for (int64_t c = 0; c < r; c++) den[c] = 0.0f;
                for (int64_t t = 0; t < r; t++) {
                    float xt = x[t];
                    const float* g = G + t * r;
                    for (int64_t c = 0; c < r; c++) den[c] += xt * g[c];
                }
            }
            const float* nu = Num + i * r;
            for (int64_t c = 0; c < r; c++) {
                volatile float q = nu[c] / (den[c] + eps); /* no fused reassociation */
                x[c] = x[c] * q;
            }
        }
        free(den);
        free(dd);
    }
}

ORACLE_API double oracle_dot(const float* a, const float* b, int64_t count) {
    double s = 0.0;
#pragma omp parallel for reduction(+ : s) schedule(static)
    for (int64_t i = 0; i < count; i++) s += (double)a[i] * (double)b[i];
    return s;
}

ORACLE_API double oracle_sq_norm(const float* a, int64_t count) { return oracle_dot(a, a, count); }

/* ------------------------------------------------------------------------- */
/* The engine, one shard (single device) rendering.                           */

typedef struct {
    int64_t n, m, r;
    const float* vals;
    const int32_t* colind;
    const int64_t* rowptr; /* CSR */
    float* cvals;
    int32_t* crow;
    int64_t* colptr; /* CSC, owned */
    float* AH;       /* n x r */
    float* WA;       /* m x r */
    float* G;        /* r x r */
} oracle_ws;

static void ws_init(oracle_ws* w, const float* vals, const int32_t* colind, const int64_t* rowptr,
                    int64_t n, int64_t m, int64_t r, int need_csc) {
    memset(w, 0, sizeof(*w));
    w->n = n; w->m = m; w->r = r;
    w->vals = vals; w->colind = colind; w->rowptr = rowptr;
    int64_t nnz = rowptr[n];
    if (need_csc) {
        w->cvals = (float*)malloc(sizeof(float) * (size_t)(nnz > 0 ? nnz : 1));
        w->crow = (int32_t*)malloc(sizeof(int32_t) * (size_t)(nnz > 0 ? nnz : 1));
        w->colptr = (int64_t*)malloc(sizeof(int64_t) * (size_t)(m + 1));
        oracle_csr_to_csc(vals, colind, rowptr, n, m, w->cvals, w->crow, w->colptr);
        w->WA = (float*)malloc(sizeof(float) * (size_t)(m * r > 0 ? m * r : 1));
    }
    w->AH = (float*)malloc(sizeof(float) * (size_t)(n * r > 0 ? n * r : 1));
    w->G = (float*)malloc(sizeof(float) * (size_t)(r * r));
}

static void ws_free(oracle_ws* w) {
    free(w->cvals); free(w->crow); free(w->colptr); free(w->AH); free(w->WA); free(w->G);
}

/* One W update (multi_mu_dense_factors_nmf1.h:293-305,
 * ..._device_contexts1.h:315-333): uses the OLD H. */
static void step_w(oracle_ws* w, float* W, const float* Ht, float eps, int acc64) {
    oracle_spmm(w->vals, w->colind, w->rowptr, w->n, Ht, w->r, w->AH, acc64);
    oracle_gram(Ht, w->m, w->r, w->G, acc64);
    oracle_mu_update(W, w->AH, w->G, w->n, w->r, eps, acc64);
}

/* One H update (..._device_contexts1.h:296-309): uses the NEW W. */
static void step_h(oracle_ws* w, const float* W, float* Ht, float eps, int acc64) {
    oracle_spmm(w->cvals, w->crow, w->colptr, w->m, W, w->r, w->WA, acc64);
    oracle_gram(W, w->n, w->r, w->G, acc64);
    oracle_mu_update(Ht, w->WA, w->G, w->m, w->r, eps, acc64);
}

/* multi_mu_dense_factors_nmf1.h:242-274 + ..._device_contexts1.h:337-354:
 * sqrt(|A|^2 + <H,(W^T W)H> - 2<W^T A, H>).  The reference sums the three
 * terms in float; here they are summed in double in both renderings because
 * the float sum loses the 1e-5 the parity target asks for. */
static double loss_of(oracle_ws* w, const float* W, const float* Ht, int acc64) {
    int64_t r = w->r, m = w->m, n = w->n;
    double a2 = oracle_sq_norm(w->vals, w->rowptr[n]);
    oracle_gram(W, n, r, w->G, acc64);
    double pos = 0.0;
#pragma omp parallel for reduction(+ : pos) schedule(static)
    for (int64_t j = 0; j < m; j++) {
        const float* h = Ht + j * r;
        double s = 0.0;
        for (int64_t a = 0; a < r; a++) {
            double t = 0.0;
            for (int64_t b = 0; b < r; b++) t += (double)w->G[a * r + b] * (double)h[b];
            s += t * (double)h[a];
        }
        pos += s;
    }
    /* <W^T A, H> = sum over stored entries a_ij * <W[i,:], H[:,j]> */
    double neg = 0.0;
#pragma omp parallel for reduction(+ : neg) schedule(dynamic, 16)
    for (int64_t i = 0; i < n; i++) {
        const float* wi = W + i * r;
        double s = 0.0;
        for (int64_t p = w->rowptr[i]; p < w->rowptr[i + 1]; p++) {
            const float* h = Ht + (int64_t)w->colind[p] * r;
            double d = 0.0;
            for (int64_t c = 0; c < r; c++) d += (double)wi[c] * (double)h[c];
            s += (double)w->vals[p] * d;
        }
        neg += s;
    }
    double sq = a2 + pos - 2.0 * neg;
    return sq > 0.0 ? sqrt(sq) : 0.0;
}

ORACLE_API double oracle_loss(const float* vals, const int32_t* colind, const int64_t* rowptr,
                              int64_t n, int64_t m, int64_t r, const float* W, const float* Ht,
                              int acc64) {
    oracle_ws w;
    ws_init(&w, vals, colind, rowptr, n, m, r, 0);
    double l = loss_of(&w, W, Ht, acc64);
    ws_free(&w);
    return l;
}

/* multi_mu_dense_factors_nmf1.h:175-182: `iters` iterations of (update W,
 * then update H).  W and Ht are updated in place.  If losses != NULL it
 * receives the loss after every iteration (iters doubles). */
ORACLE_API void oracle_run(const float* vals, const int32_t* colind, const int64_t* rowptr,
                           int64_t n, int64_t m, int64_t r, float* W, float* Ht, int32_t iters,
                           float eps, int acc64, double* losses) {
    oracle_ws w;
    ws_init(&w, vals, colind, rowptr, n, m, r, 1);
    for (int32_t it = 0; it < iters; it++) {
        step_w(&w, W, Ht, eps, acc64);
        step_h(&w, W, Ht, eps, acc64);
        if (losses) losses[it] = loss_of(&w, W, Ht, acc64);
    }
    ws_free(&w);
}

/* Single half-steps, for kernel-level parity tests. */
ORACLE_API void oracle_step_w(const float* vals, const int32_t* colind, const int64_t* rowptr,
                              int64_t n, int64_t m, int64_t r, float* W, const float* Ht,
                              float eps, int acc64) {
    oracle_ws w;
    ws_init(&w, vals, colind, rowptr, n, m, r, 0);
    step_w(&w, W, Ht, eps, acc64);
    ws_free(&w);
}

ORACLE_API void oracle_step_h(const float* vals, const int32_t* colind, const int64_t* rowptr,
                              int64_t n, int64_t m, int64_t r, const float* W, float* Ht,
                              float eps, int acc64) {
    oracle_ws w;
    ws_init(&w, vals, colind, rowptr, n, m, r, 1);
    step_h(&w, W, Ht, eps, acc64);
    ws_free(&w);
}

/* W-only fit with H fixed: nmf/sparse2/nmf_sparse_H.h:116-127,157-211,298-345.
 * Stage 1 computes AH = A*H^T and HH = H*H^T once; stage 2 repeats
 * W *= AH / (W*HH + eps).  Returns the final loss
 * sqrt(|A|^2 + <W*HH, W> - 2<AH, W>). */
ORACLE_API double oracle_fit_w_only(const float* vals, const int32_t* colind,
                                    const int64_t* rowptr, int64_t n, int64_t m, int64_t r,
                                    float* W, const float* Ht, int32_t iters, float eps,
                                    int acc64) {
    oracle_ws w;
    ws_init(&w, vals, colind, rowptr, n, m, r, 0);
    oracle_spmm(vals, colind, rowptr, n, Ht, r, w.AH, acc64);
    oracle_gram(Ht, m, r, w.G, acc64);
    for (int32_t it = 0; it < iters; it++) oracle_mu_update(W, w.AH, w.G, n, r, eps, acc64);
    double a2 = oracle_sq_norm(vals, rowptr[n]);
    double pos = 0.0, neg = oracle_dot(w.AH, W, n * r);
#pragma omp parallel for reduction(+ : pos) schedule(static)
    for (int64_t i = 0; i < n; i++) {
        const float* x = W + i * r;
        double s = 0.0;
        for (int64_t a = 0; a < r; a++) {
            double t = 0.0;
            for (int64_t b = 0; b < r; b++) t += (double)x[b] * (double)w.G[b * r + a];
            s += t * (double)x[a];
        }
        pos += s;
    }
    ws_free(&w);
    double sq = a2 + pos - 2.0 * neg;
    return sq > 0.0 ? sqrt(sq) : 0.0;
}

/* ------------------------------------------------------------------------- */
/* Synthetic D-PEF generator, the host twin of the device generator the        */
/* benchmark uses (same counter-based hashes, same draw order), so that the    */
/* timed CPU arm works on the matrix the GPU arm works on.  Column indices are */
/* identical bit for bit (integer hashes and a search in the same cumulative   */
/* table); values agree to a few ulp (log / exp / inverse erfc come from       */
/* different maths libraries).  No reference counterpart: the reference reads  */
/* real D-PEF files (npeff/fishers/d_pefs_computer.py:217-287).                */

#define SYNTH_THREADS 1024
#define SYNTH_MAX_ROUNDS (1ull << 15)

static inline uint64_t stream_key(uint64_t seed, uint64_t stream) {
    return mix64(seed ^ (stream * 0xD1B54A32D192ED03ull));
}

static inline double u01_open(uint64_t h) { /* (0,1] */
    return (double)((h >> 11) + 1ull) * (1.0 / 9007199254740992.0);
}

static inline uint32_t perm_bits(uint32_t x, int bits, uint32_t key) {
    uint32_t mask = (bits >= 32) ? 0xffffffffu : ((1u << bits) - 1u);
    int half = bits > 1 ? bits / 2 : 1;
    x = (x * 0x9E3779B1u + key) & mask;
    x ^= x >> half;
    x = (x * 0x85EBCA6Bu + (key >> 7) * 2u + 1u) & mask;
    x ^= x >> half;
    return x & mask;
}

/* q with erfc(q) = s, 0 < s <= 1, by Newton steps on the convex function
 * erfc(q) - s from the start value q0 (any non-negative number). */
static double erfcinv_from(double s, double q0) {
    if (s >= 1.0) return 0.0;
    double q = q0;
    for (int it = 0; it < 40; it++) {
        double f = erfc(q) - s;
        double d = -1.1283791670955126 * exp(-q * q); /* d/dq erfc(q) = -2/sqrt(pi) exp(-q^2) */
        double step = f / d;
        double qn = q - step;
        if (qn < 0.0) qn = 0.5 * q;
        if (fabs(qn - q) <= 4e-16 * qn) { q = qn; break; }
        q = qn;
    }
    return q;
}

typedef struct {
    uint64_t hash;
    int32_t col;
} synth_cand;

static int synth_cand_cmp(const void* a, const void* b) {
    const synth_cand* x = (const synth_cand*)a;
    const synth_cand* y = (const synth_cand*)b;
    if (x->hash != y->hash) return x->hash < y->hash ? -1 : 1;
    return x->col < y->col ? -1 : (x->col > y->col ? 1 : 0);
}

/* vals, idx: [n, k]; norms: [n].  Returns 0, or -1 on a bad shape. */
ORACLE_API int oracle_synth_pef(int64_t n, int64_t m, int64_t k, double alpha, double sigma, uint64_t seed,
                                float* vals, int32_t* idx, float* norms) {
    if (n < 0 || m <= 0 || k <= 0 || k > m || m >= INT32_MAX) return -1;
    double* cdf = (double*)malloc(sizeof(double) * (size_t)m);
    double acc = 0.0;
    for (int64_t c = 0; c < m; c++) {
        acc += pow((double)(c + 1), -alpha);
        cdf[c] = acc;
    }
    const double total = cdf[m - 1];
    /* guide table: for bucket b of [0,total), the first column whose cumulative
     * weight reaches the bucket's lower edge; the search for u starts there */
    const int64_t G = 1 << 20;
    int32_t* guide = (int32_t*)malloc(sizeof(int32_t) * (size_t)(G + 1));
    {
        int64_t c = 0;
        for (int64_t b = 0; b <= G; b++) {
            double edge = total * (double)b / (double)G;
            while (c < m - 1 && cdf[c] < edge) c++;
            guide[b] = (int32_t)c;
        }
    }
    int bits = 1;
    while ((1ll << bits) < k) bits++;
    const int64_t words = (m + 31) / 32;
#pragma omp parallel
    {
        uint32_t* bitmap = (uint32_t*)calloc((size_t)words, sizeof(uint32_t));
        int32_t* claimed = (int32_t*)malloc(sizeof(int32_t) * (size_t)k);
        synth_cand* cand = (synth_cand*)malloc(sizeof(synth_cand) * SYNTH_THREADS);
#pragma omp for schedule(dynamic, 4)
        for (int64_t row = 0; row < n; row++) {
            const uint64_t rkey = mix64(stream_key(seed, 2) + (uint64_t)row);
            int64_t count = 0;
            for (uint64_t round = 0; count < k; round++) {
                if (round >= SYNTH_MAX_ROUNDS) {
                    for (int64_t c = 0; c < m && count < k; c++) {
                        uint32_t b = 1u << (c & 31);
                        if (!(bitmap[c >> 5] & b)) {
                            bitmap[c >> 5] |= b;
                            count++;
                        }
                    }
                    break;
                }
                int n_new = 0;
                for (int tid = 0; tid < SYNTH_THREADS; tid++) {
                    uint64_t h = mix64(rkey + round * SYNTH_THREADS + (uint64_t)tid + 0x1234567ull);
                    double u = u01_open(h) * total;
                    /* first c with cdf[c] >= u */
                    int64_t b = (int64_t)(u / total * (double)G);
                    if (b > G - 1) b = G - 1;
                    if (b < 0) b = 0;
                    int64_t lo = guide[b], hi = guide[b + 1];
                    while (lo > 0 && cdf[lo - 1] >= u) lo--;      /* rounding of the bucket index */
                    while (hi < m - 1 && cdf[hi] < u) hi++;
                    while (lo < hi) {
                        int64_t mid = (lo + hi) >> 1;
                        if (cdf[mid] >= u) hi = mid; else lo = mid + 1;
                    }
                    int32_t c = (int32_t)lo;
                    uint32_t bit = 1u << (c & 31);
                    if (!(bitmap[c >> 5] & bit)) {
                        bitmap[c >> 5] |= bit;
                        cand[n_new].col = c;
                        cand[n_new].hash = mix64(rkey ^ (uint64_t)c);
                        n_new++;
                    }
                }
                if (count + n_new > k) {
                    /* the last round overshoots: keep the (k - count) new columns with
                     * the smallest keyed hash */
                    qsort(cand, (size_t)n_new, sizeof(synth_cand), synth_cand_cmp);
                    for (int i = (int)(k - count); i < n_new; i++) {
                        int32_t c = cand[i].col;
                        bitmap[c >> 5] &= ~(1u << (c & 31));
                    }
                    n_new = (int)(k - count);
                }
                count += n_new;
            }
            /* the claimed set in ascending order; the bitmap is cleared on the way */
            {
                int64_t q = 0;
                for (int64_t w = 0; w < words; w++) {
                    uint32_t bw = bitmap[w];
                    if (!bw) continue;
                    bitmap[w] = 0u;
                    while (bw) {
                        int b = __builtin_ctz(bw);
                        claimed[q++] = (int32_t)(w * 32 + b);
                        bw &= bw - 1u;
                    }
                }
            }
            /* values: descending order statistics of k chi-square(1) draws */
            double zu1 = u01_open(mix64(rkey + 0xABCDEFull)), zu2 = u01_open(mix64(rkey + 0xFEDCBAull));
            double z = sqrt(-2.0 * log(zu1)) * cos(6.283185307179586 * zu2);
            double srow = exp(sigma * z);
            double run = 0.0, sq = 0.0, qprev = -1.0;
            for (int64_t j = 0; j < k; j++) {
                double e = -log(u01_open(mix64(rkey ^ (0x5555ull << 32) ^ (uint64_t)(j + 1) * 0x9E3779B97F4A7C15ull)));
                run += e / (double)(k - j);
                double surv = -expm1(-run);
                double q0 = qprev >= 0.0 ? qprev : sqrt(-log(surv > 1e-300 ? surv : 1e-300));
                double q = erfcinv_from(surv, q0);
                qprev = q;
                double x = 2.0 * q * q * srow;
                float xf = (float)x;
                uint32_t pj = (uint32_t)j;
                do { pj = perm_bits(pj, bits, (uint32_t)(rkey >> 17)); } while (pj >= (uint32_t)k);
                vals[row * k + j] = xf;
                idx[row * k + j] = claimed[pj];
                sq += (double)xf * (double)xf;
            }
            norms[row] = (float)sqrt(sq);
        }
        free(bitmap);
        free(claimed);
        free(cand);
    }
    free(cdf);
    free(guide);
    return 0;
}

/* ------------------------------------------------------------------------- */
/* A loaded problem kept between calls, for the timed CPU arm of the           */
/* benchmark: normalise, prune, transpose once; then one iteration per call.   */

typedef struct {
    oracle_ws w;
    float* vals;
    int32_t* colind;
    int64_t* rowptr;
    float* W;
    float* Ht;
    float eps;
    double a_sum;
} oracle_problem;

/* CSR -> CSC with every thread transposing a block of rows: per-thread column
 * histograms, one prefix pass over (column, thread), then disjoint scatters.
 * Rows stay ascending inside a column (thread t owns rows before thread t+1's). */
static void csr_to_csc_threads(const float* vals, const int32_t* colind, const int64_t* rowptr, int64_t n,
                               int64_t m, float* cvals, int32_t* crow, int64_t* colptr) {
    int T = oracle_num_threads();
    if (T < 1) T = 1;
    int64_t* hist = (int64_t*)calloc((size_t)T * (size_t)(m + 1), sizeof(int64_t));
#pragma omp parallel num_threads(T)
    {
#ifdef _OPENMP
        int t = omp_get_thread_num();
#else
        int t = 0;
#endif
        int64_t r0 = n * t / T, r1 = n * (t + 1) / T;
        int64_t* h = hist + (size_t)t * (size_t)(m + 1);
        for (int64_t p = rowptr[r0]; p < rowptr[r1]; p++) h[colind[p]]++;
    }
    int64_t q = 0;
    for (int64_t c = 0; c < m; c++) {
        colptr[c] = q;
        for (int t = 0; t < T; t++) {
            int64_t* h = hist + (size_t)t * (size_t)(m + 1);
            int64_t cnt = h[c];
            h[c] = q;
            q += cnt;
        }
    }
    colptr[m] = q;
#pragma omp parallel num_threads(T)
    {
#ifdef _OPENMP
        int t = omp_get_thread_num();
#else
        int t = 0;
#endif
        int64_t r0 = n * t / T, r1 = n * (t + 1) / T;
        int64_t* h = hist + (size_t)t * (size_t)(m + 1);
        for (int64_t i = r0; i < r1; i++)
            for (int64_t p = rowptr[i]; p < rowptr[i + 1]; p++) {
                int64_t s = h[colind[p]]++;
                cvals[s] = vals[p];
                crow[s] = (int32_t)i;
            }
    }
    free(hist);
}

/* Takes ownership of nothing: vals/idx/norms ([n,k], [n,k], [n]) are copied.
 * Normalises the rows (norms may be NULL), prunes with min_count, builds the
 * CSC and initial factors scale * U(0,1] from the shared hash; init_scale <= 0
 * means sqrt(mean(A) / r) with the mean over all n x m_kept entries.
 * Returns NULL when memory runs out. */
ORACLE_API void* oracle_problem_create(int64_t n, int64_t m, int64_t k, int64_t r, const float* vals,
                                       const int32_t* idx, const float* norms, int32_t min_count, float eps,
                                       uint64_t seed, float init_scale, int64_t* m_kept_out) {
    oracle_problem* P = (oracle_problem*)calloc(1, sizeof(oracle_problem));
    if (!P) return NULL;
    int64_t nnz = n * k;
    P->vals = (float*)malloc(sizeof(float) * (size_t)(nnz > 0 ? nnz : 1));
    P->colind = (int32_t*)malloc(sizeof(int32_t) * (size_t)(nnz > 0 ? nnz : 1));
    P->rowptr = (int64_t*)malloc(sizeof(int64_t) * (size_t)(n + 1));
    int32_t* n2o = (int32_t*)malloc(sizeof(int32_t) * (size_t)(m > 0 ? m : 1));
    if (!P->vals || !P->colind || !P->rowptr || !n2o) return NULL;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) {
        P->rowptr[i] = i * k;
        memcpy(P->vals + i * k, vals + i * k, sizeof(float) * (size_t)k);
        memcpy(P->colind + i * k, idx + i * k, sizeof(int32_t) * (size_t)k);
    }
    P->rowptr[n] = nnz;
    if (norms) oracle_normalize_rows(P->vals, P->rowptr, n, norms, 1e-9f);
    int64_t nnz2 = 0;
    int64_t mk = oracle_prune_columns(P->vals, P->colind, P->rowptr, n, m, min_count, n2o, &nnz2);
    free(n2o);
    if (m_kept_out) *m_kept_out = mk;
    oracle_ws* w = &P->w;
    memset(w, 0, sizeof(*w));
    w->n = n; w->m = mk; w->r = r;
    w->vals = P->vals; w->colind = P->colind; w->rowptr = P->rowptr;
    w->cvals = (float*)malloc(sizeof(float) * (size_t)(nnz2 > 0 ? nnz2 : 1));
    w->crow = (int32_t*)malloc(sizeof(int32_t) * (size_t)(nnz2 > 0 ? nnz2 : 1));
    w->colptr = (int64_t*)malloc(sizeof(int64_t) * (size_t)(mk + 1));
    w->WA = (float*)malloc(sizeof(float) * (size_t)(mk * r > 0 ? mk * r : 1));
    w->AH = (float*)malloc(sizeof(float) * (size_t)(n * r > 0 ? n * r : 1));
    w->G = (float*)malloc(sizeof(float) * (size_t)(r * r));
    P->W = (float*)malloc(sizeof(float) * (size_t)(n * r > 0 ? n * r : 1));
    P->Ht = (float*)malloc(sizeof(float) * (size_t)(mk * r > 0 ? mk * r : 1));
    if (!w->cvals || !w->crow || !w->colptr || !w->WA || !w->AH || !w->G || !P->W || !P->Ht) return NULL;
    csr_to_csc_threads(P->vals, P->colind, P->rowptr, n, mk, w->cvals, w->crow, w->colptr);
    double s = 0.0;
#pragma omp parallel for reduction(+ : s) schedule(static)
    for (int64_t p = 0; p < nnz2; p++) s += (double)P->vals[p];
    P->a_sum = s;
    float scale = init_scale > 0.f ? init_scale : (float)sqrt(s / ((double)n * (double)mk) / (double)r);
    oracle_init_uniform(P->W, 0, n * r, seed, 0, scale);
    oracle_init_uniform(P->Ht, 0, mk * r, seed, 1, scale);
    P->eps = eps;
    return P;
}

/* One iteration (W update, then H update) in the given accumulation precision. */
ORACLE_API void oracle_problem_step(void* handle, int acc64) {
    oracle_problem* P = (oracle_problem*)handle;
    step_w(&P->w, P->W, P->Ht, P->eps, acc64);
    step_h(&P->w, P->W, P->Ht, P->eps, acc64);
}

ORACLE_API double oracle_problem_loss(void* handle) {
    oracle_problem* P = (oracle_problem*)handle;
    return loss_of(&P->w, P->W, P->Ht, 1);
}

ORACLE_API void oracle_problem_free(void* handle) {
    oracle_problem* P = (oracle_problem*)handle;
    if (!P) return;
    ws_free(&P->w);
    free(P->vals); free(P->colind); free(P->rowptr); free(P->W); free(P->Ht);
    free(P);
}
