// TEST INFRASTRUCTURE ONLY: drives the UNMODIFIED reference engine
// (cc/cuda_d_npeff/src, included from where the reference tree is mounted; no
// reference source lives in this repository) on a matrix read from a flat
// binary file, and writes what it computed to another flat file.  It exists to
// pin the CPU oracle -- and through it the CUDA engine -- to outputs of the
// reference itself, since the reference ships no tests for this path.
//
// The reference executable cannot be built here (it needs libhdf5); this
// harness reaches the same engine without the HDF5 headers:
//   removeSmallestL0NormColumns_inPlace  util/sparse_util.h:79
//   splitColumnWise                      util/matrix_util.h:24
//   MuNmf<int32_t>                       nmf/sparse/multi_mu_dense_factors_nmf1.h:40
// Row normalisation (io/pef_fisher_h5.h:38-52) lives in an HDF5-dependent
// header, so the input file carries already-normalised values.
//
// Identical initial factors: the engine seeds cuRAND per instance, so one
// instance run with max_iters = 0 yields the initial W and H, and a second one
// with the same seed reproduces them before iterating.
//
// usage: ref_engine <in.bin> <out.bin> <rank> <iters> <eps> <seed> <min_count> [timing]
// With the word `timing` as the last argument only the iterating instance runs and
// nothing is written: the engine's own "step N: loss [ms/step]" lines on stdout
// (multi_mu_dense_factors_nmf1.h:186-201) are the result.
// in.bin : int64 n, m, nnz; int32 rowptr[n+1]; int32 colind[nnz]; float vals[nnz]
// out.bin: int64 n, m_kept, nnz_kept, rank, n_devices;
//          int32 new_to_og[m_kept]; int32 rowptr[n+1]; int32 colind[nnz_kept]; float vals[nnz_kept];
//          float W0[n*rank] (col-major n x rank); float H0[rank*m_kept] (col-major rank x m_kept);
//          float W[n*rank]; float H[rank*m_kept]; float loss0; float loss; double ms_per_step
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include <util/cuda_system.h>
#include <util/matrices.h>
#include <util/sparse_util.h>
#include <nmf/sparse/multi_mu_dense_factors_nmf1.h>

template <typename T>
static void rd(FILE* f, T* p, size_t n) {
    if (fread(p, sizeof(T), n, f) != n) { fprintf(stderr, "short read\n"); exit(2); }
}
template <typename T>
static void wr(FILE* f, const T* p, size_t n) {
    if (fwrite(p, sizeof(T), n, f) != n) { fprintf(stderr, "short write\n"); exit(2); }
}

int main(int argc, char** argv) {
    if (argc < 8) { fprintf(stderr, "usage: %s in out rank iters eps seed min_count\n", argv[0]); return 1; }
    int rank = atoi(argv[3]), iters = atoi(argv[4]);
    float eps = (float)atof(argv[5]);
    long seed = atol(argv[6]);
    int min_count = atoi(argv[7]);
    const bool timing_only = argc >= 9 && strcmp(argv[8], "timing") == 0;

    FILE* f = fopen(argv[1], "rb");
    if (!f) { perror("open in"); return 1; }
    int64_t hdr[3];
    rd(f, hdr, 3);
    long n = hdr[0], m = hdr[1], nnz = hdr[2];
    ElCsrMatrix<int32_t> A((int)n, (int)m, nnz);
    rd(f, A.csrRowPtrA, n + 1);
    rd(f, A.csrColIndA, nnz);
    rd(f, A.csrValA, nnz);
    fclose(f);

    int32_t* newToOg = nullptr;
    removeSmallestL0NormColumns_inPlace<int32_t>(&A, &newToOg, min_count);
    long m_kept = A.n_cols, nnz_kept = A.nnz;

    int nDevices = 0;
    cudaGetDeviceCount(&nDevices);
    ElCsrMatrix<int32_t>* parts = splitColumnWise<int32_t>(A, nDevices);

    MuNmfParams p;
    p.rank = rank;
    p.eps = eps;
    p.seed = seed;

    if (timing_only) {
        p.max_iters = iters;
        MuNmf<int32_t> nmf(parts, p);
        nmf.run();
        fflush(stdout);
        return 0;
    }

    p.max_iters = 0;
    MuNmf<int32_t> nmf0(parts, p);
    nmf0.run();
    MeMatrix W0 = nmf0.loadWToHostSync();
    MeMatrix H0 = nmf0.loadHToHostSync();
    float loss0 = nmf0.computeUncachedLoss();

    p.max_iters = iters;
    MuNmf<int32_t> nmf1(parts, p);
    auto t0 = std::chrono::high_resolution_clock::now();
    nmf1.run();
    auto t1 = std::chrono::high_resolution_clock::now();
    double ms = std::chrono::duration<double, std::milli>(t1 - t0).count() / (iters > 0 ? iters : 1);
    MeMatrix W = nmf1.loadWToHostSync();
    MeMatrix H = nmf1.loadHToHostSync();
    float loss = nmf1.computeUncachedLoss();

    FILE* o = fopen(argv[2], "wb");
    if (!o) { perror("open out"); return 1; }
    int64_t oh[5] = {n, m_kept, nnz_kept, rank, nDevices};
    wr(o, oh, 5);
    wr(o, newToOg, m_kept);
    wr(o, A.csrRowPtrA, n + 1);
    wr(o, A.csrColIndA, nnz_kept);
    wr(o, A.csrValA, nnz_kept);
    wr(o, W0.data, (size_t)n * rank);
    wr(o, H0.data, (size_t)rank * m_kept);
    wr(o, W.data, (size_t)n * rank);
    wr(o, H.data, (size_t)rank * m_kept);
    wr(o, &loss0, 1);
    wr(o, &loss, 1);
    wr(o, &ms, 1);
    fclose(o);
    printf("ref_engine: n=%ld m_kept=%ld nnz=%ld rank=%d iters=%d devices=%d loss0=%g loss=%g ms/step(incl. init)=%g\n",
           n, m_kept, nnz_kept, rank, iters, nDevices, loss0, loss, ms);
    return 0;
}
