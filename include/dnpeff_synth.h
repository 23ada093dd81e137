/*
 * dnpeff_synth.h -- synthetic D-PEF generator (benchmark and test support).
 *
 * No counterpart in the reference: its inputs are real D-PEF files written by
 * npeff/fishers/d_pefs_computer.py:217-287.  This entry point fills, directly
 * in device memory, the three arrays such a file holds:
 *   d_vals  [n_rows, k_per_row] float32   data/fisher/values   (descending per row)
 *   d_idx   [n_rows, k_per_row] int32     data/fisher/indices  (distinct per row)
 *   d_norms [n_rows]            float32   data/dense_fisher_norms (L2 norm of the row)
 * Columns follow a Zipf(alpha) popularity over n_cols; values are
 * g^2 * LogNormal(0, sigma) with g ~ N(0,1).  Deterministic in `seed`.
 * The call synchronises `stream` before returning.
 */
#ifndef DNPEFF_SYNTH_H_
#define DNPEFF_SYNTH_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

int dnpeff_synth_pef_device(int64_t n_rows, int64_t n_cols, int64_t k_per_row, double alpha,
                            double sigma, uint64_t seed, float* d_vals, int32_t* d_idx,
                            float* d_norms, void* stream);

/* Rows [row_first, row_first + n_rows) of the same matrix (a row's content depends on
 * its index and the seed only): what one rank of a row-split job generates. */
int dnpeff_synth_pef_device_rows(int64_t row_first, int64_t n_rows, int64_t n_cols, int64_t k_per_row,
                                 double alpha, double sigma, uint64_t seed, float* d_vals, int32_t* d_idx,
                                 float* d_norms, void* stream);

/* Writes host arrays as a D-PEF file in the layout of
 * npeff/fishers/d_pefs_computer.py:235-251 (what dnpeff_load_pef_hdf5 and the
 * reference's PefSparseFishers::read consume).  The reference has no C++ writer
 * for this file: it is produced by its TensorFlow pipeline. */
int dnpeff_write_pef_hdf5(const char* path, int64_t n_examples, int64_t n_values_per_example,
                          const float* vals, const int32_t* indices, const float* norms,
                          int64_t dense_fisher_size);

#ifdef __cplusplus
}
#endif
#endif /* DNPEFF_SYNTH_H_ */
