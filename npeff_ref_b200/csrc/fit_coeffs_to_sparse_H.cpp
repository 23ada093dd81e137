// fit_coeffs_to_sparse_H -- drop-in for the reference executable of the same name
// (cc/cuda_d_npeff/mains/fit_coeffs_to_sparse_H.cu): learns W for a new set of
// D-PEFs with the sparse H of an existing decomposition held fixed.
//
//   read the sparse decomposition (--H_path)           fit.cu:118-122
//   read + normalise the D-PEFs (--pef_path)           fit.cu:124-130
//   keep the decomposition's columns of A only         fit.cu:134-135 (RetainColumns_InPlace)
//   split A by rows (--n_row_splits_pefs)              fit.cu:153, sparse_matrix.h:219-245
//   A*H^T and H*H^T once, then nmf_max_iter x
//     W *= AH / (W*HH + 1e-7) from a uniform W         nmf_sparse_H.h:116-127,298-345; fit.cu:189
//   write W + the same sparse H                        fit.cu:196-211
//
// Flags (fit.cu:45-69): --output_path --pef_path --H_path --n_splits_sparse_matmul
// --n_row_splits_pefs --nmf_max_iter (required); --n_examples --n_fisher_values
// --main_device --DEV_n_cols.  As there, any argument that is not one of the
// flags read ends the program with "Unrecognized flags.".
// --n_splits_sparse_matmul partitions the reference's sparse-sparse products to
// bound their scratch memory; this engine keeps H dense in HBM and has no such
// scratch, so the value is read and not used.  Rows are independent given H, so
// every row chunk is loaded, fitted and read back on its own: device memory is
// bounded by the largest chunk.
// Extra, optional: --seed (43190432042) --init_scale (1).
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <set>
#include <string>
#include <vector>

#include "../../include/dnpeff.h"

namespace {

int g_argc;
char** g_argv;
std::set<std::string> g_read;

// util/flag_util.h:23-41: first argv that starts with --name= wins.
bool flag_str(const std::string& name, std::string* out, bool required) {
    std::string prefix = "--" + name + "=";
    for (int i = 0; i < g_argc; i++) {
        if (strncmp(g_argv[i], prefix.c_str(), prefix.size()) == 0) {
            *out = std::string(g_argv[i] + prefix.size());
            g_read.insert(name);
            return true;
        }
    }
    if (required) {
        printf("Missing flag: %s\n", name.c_str());
        fflush(stdout);
        std::abort();  // the reference terminates here (flag_util.h:37-40)
    }
    return false;
}

void flag_i64(const std::string& name, long long* out, bool required) {
    std::string s;
    if (flag_str(name, &s, required)) *out = atoll(s.c_str());
}

void flag_f64(const std::string& name, double* out, bool required) {
    std::string s;
    if (flag_str(name, &s, required)) *out = atof(s.c_str());
}

[[noreturn]] void die(const char* what) {
    fprintf(stderr, "fit_coeffs_to_sparse_H: %s: %s\n", what, dnpeff_last_error());
    fflush(stderr);
    std::exit(1);
}

// GetSizeOfSplit: equal sizes, the remainder to the last one.
void split_rows(long long n, int n_splits, int i, long long* start, long long* size) {
    long long base = n / n_splits;
    *start = base * i;
    *size = (i == n_splits - 1) ? base + n % n_splits : base;
}

}  // namespace

int main(int argc, char** argv) {
    g_argc = argc;
    g_argv = argv;
    std::string out_path, pef_path, h_path;
    long long n_splits_mm = 0, n_row_splits = 1, max_iters = 0, n_examples = -1, n_values = -1, main_device = 0;
    long long dev_n_cols = -1, seed = 43190432042LL;
    double init_scale = 1.0;
    flag_str("output_path", &out_path, true);
    flag_str("pef_path", &pef_path, true);
    flag_str("H_path", &h_path, true);
    flag_i64("n_splits_sparse_matmul", &n_splits_mm, true);
    flag_i64("n_row_splits_pefs", &n_row_splits, true);
    flag_i64("nmf_max_iter", &max_iters, true);
    flag_i64("n_examples", &n_examples, false);
    flag_i64("n_fisher_values", &n_values, false);
    flag_i64("main_device", &main_device, false);
    flag_i64("DEV_n_cols", &dev_n_cols, false);
    flag_i64("seed", &seed, false);
    flag_f64("init_scale", &init_scale, false);
    if ((int)g_read.size() != argc - 1) {  // flag_util.h:43-56
        printf("Unrecognized flags.\n");
        fflush(stdout);
        std::abort();
    }
    if (n_row_splits < 1) n_row_splits = 1;

    int n_dev = 0;
    if (dnpeff_device_count(&n_dev) != DNPEFF_OK || n_dev < 1) die("no CUDA device");
    if (main_device < 0 || main_device >= n_dev) {
        fprintf(stderr, "fit_coeffs_to_sparse_H: --main_device=%lld but %d device(s) are visible\n", main_device, n_dev);
        return 1;
    }

    // ---- the decomposition whose H is kept
    printf("Starting to read in H.\n");
    int64_t n_old = 0, m_kept = 0, h_nnz = 0, full_dense = 0;
    int32_t rank = 0;
    if (dnpeff_sparse_decomposition_hdf5_info(h_path.c_str(), &n_old, &rank, &m_kept, &h_nnz, &full_dense) != DNPEFF_OK)
        die("reading the decomposition");
    std::vector<int64_t> h_rowptr((size_t)rank + 1);
    std::vector<int32_t> h_col((size_t)std::max<int64_t>(h_nnz, 1)), kept((size_t)std::max<int64_t>(m_kept, 1));
    std::vector<float> h_val((size_t)std::max<int64_t>(h_nnz, 1));
    if (dnpeff_read_sparse_decomposition_hdf5(h_path.c_str(), nullptr, h_rowptr.data(), h_col.data(), h_val.data(),
                                              kept.data()) != DNPEFF_OK)
        die("reading the decomposition");
    printf("H read in.\n");

    if (dev_n_cols >= 0) {
        // development flag of the reference (fit.cu:139-149): the first DEV_n_cols kept columns only
        printf("NOTE: Using flag intended only for development purposes.\n");
        if (dev_n_cols > m_kept) dev_n_cols = m_kept;
        std::vector<int64_t> rp((size_t)rank + 1, 0);
        int64_t w = 0;
        for (int t = 0; t < rank; t++) {
            for (int64_t p = h_rowptr[(size_t)t]; p < h_rowptr[(size_t)t + 1]; p++) {
                if (h_col[(size_t)p] < dev_n_cols) {
                    h_col[(size_t)w] = h_col[(size_t)p];
                    h_val[(size_t)w] = h_val[(size_t)p];
                    w++;
                }
            }
            rp[(size_t)t + 1] = w;
        }
        h_rowptr = rp;
        h_nnz = w;
        m_kept = dev_n_cols;
    }

    // ---- the D-PEFs
    printf("Starting to read in PEFs.\n");
    int64_t n_file = 0, k_file = 0, dense = 0;
    if (dnpeff_pef_hdf5_info(pef_path.c_str(), &n_file, &k_file, &dense) != DNPEFF_OK) die("reading the D-PEF file");
    int64_t n = (n_examples >= 0 && n_examples < n_file) ? n_examples : n_file;
    int64_t k = (n_values >= 0 && n_values < k_file) ? n_values : k_file;
    std::vector<float> vals((size_t)std::max<int64_t>(n * k, 1)), norms((size_t)std::max<int64_t>(n, 1));
    std::vector<int32_t> idx((size_t)std::max<int64_t>(n * k, 1));
    if (dnpeff_read_pef_hdf5(pef_path.c_str(), n, k, vals.data(), idx.data(), norms.data()) != DNPEFF_OK)
        die("reading the D-PEF file");
    printf("PEFS read in.\n");
    if (n_row_splits > n && n > 0) n_row_splits = n;

    dnpeff_params p;
    memset(&p, 0, sizeof(p));
    p.rank = rank;
    p.eps = 1e-7f;  // fit.cu:189
    p.seed = (uint64_t)seed;
    p.init_scale = (float)init_scale;
    p.shard_index = 0;
    p.n_shards = 1;
    p.shard_mode = DNPEFF_SHARD_CONTIGUOUS;
    dnpeff_engine* eng = nullptr;
    if (dnpeff_create(&p, (int)main_device, nullptr, &eng) != DNPEFF_OK) die("creating the engine");

    std::vector<float> W((size_t)std::max<int64_t>(n * rank, 1));
    double loss_sq = 0.0;
    auto t0 = std::chrono::high_resolution_clock::now();
    for (int c = 0; c < (int)n_row_splits; c++) {
        long long r0 = 0, rows = 0;
        split_rows(n, (int)n_row_splits, c, &r0, &rows);
        if (rows <= 0) continue;
        if (dnpeff_set_csr_retain(eng, rows, dense, k, nullptr, vals.data() + r0 * k, idx.data() + r0 * k,
                                  norms.data() + r0, kept.data(), m_kept) != DNPEFF_OK)
            die("loading a row chunk");
        if (dnpeff_set_w_row_offset(eng, r0) != DNPEFF_OK) die("row offset");
        if (dnpeff_init_factors(eng, nullptr, nullptr) != DNPEFF_OK) die("initialising W");
        if (dnpeff_set_h_csr(eng, h_rowptr.data(), h_col.data(), h_val.data()) != DNPEFF_OK) die("setting H");
        double loss = 0.0;
        if (dnpeff_fit_w_only(eng, (int32_t)max_iters, &loss) != DNPEFF_OK) die("fitting W");
        if (dnpeff_get_w(eng, W.data() + r0 * rank) != DNPEFF_OK) die("reading W back");
        if (dnpeff_synchronize(eng) != DNPEFF_OK) die("synchronising");
        loss_sq += loss * loss;
    }
    auto t1 = std::chrono::high_resolution_clock::now();
    double ms = std::chrono::duration<double, std::milli>(t1 - t0).count();
    // the reference's progress line (nmf_sparse_H.h:329-331), once, for the whole fit
    printf("step %lld: %g [%g ms/step]\n", max_iters, std::sqrt(loss_sq), max_iters > 0 ? ms / (double)max_iters : ms);
    printf("Finished running second stage.\n");
    dnpeff_destroy(eng);

    if (dnpeff_save_sparse_decomposition_hdf5(out_path.c_str(), W.data(), n, rank, h_rowptr.data(), h_col.data(),
                                              h_val.data(), kept.data(), m_kept, full_dense) != DNPEFF_OK)
        die("writing the output");
    fflush(stdout);
    return 0;
}
