// run_nmf_on_pefs -- drop-in for the reference executable of the same name
// (cc/cuda_d_npeff/mains/run_nmf_on_pefs.cu): same flags in --name=value form,
// same D-PEF input file, same decomposition output file, same
// "step N: <loss> [<ms> ms/step]" progress line every 10 steps.  One host thread
// per visible GPU drives one engine (one column shard) through the C ABI.
//
// Flags (run_nmf_on_pefs.cu:49-70): --output_path --per_example_fishers
// --nmf_n_components --nmf_max_iter (required); --n_examples --n_fisher_values
// --min_values_per_parameter --sparsity_W --initial_H_path --initial_W_path.
// Unknown flags are ignored, as in the reference (it never calls
// VerifyNoUnreadFlags).  --sparsity_W alone changes nothing, as in the reference:
// there it only builds the Hoyer projection context for W (l1 = the flag's value,
// l2 = 1) and the one call that would use it, on the initial W before the first
// step, is commented out (multi_mu_dense_factors_nmf1.h:162).
// Extra, optional: --eps (1e-8) --seed (43190432042) --init_scale (1 = unscaled
// uniform) --n_devices (all) --log_every (10) --shard_mode (cyclic|contiguous)
// --sparsify_initial_W (0; 1 makes that call: with --sparsity_W > 0 the columns of
// the initial W are projected onto L1 = sparsity_W, L2 = 1 before the first step)
// --checkpoint_every (0 = never; K > 0: after every K-th step the factors are written
// to <output_path>.checkpoint -- a decomposition file like the output, written under
// a temporary name and renamed, so a reader never sees half a file; a run continues
// from it with --initial_W_path / --initial_H_path set to that file and
// --nmf_max_iter set to the steps that remain, and ends bit for bit where the
// uninterrupted run ends).
//
// Every engine reads only its own slice of the file's rows, in chunks through
// page-locked staging buffers (dnpeff_load_pef_hdf5); the reference reads the whole
// file into one host array first (src/io/pef_fisher_h5.h:175-220).
#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../include/dnpeff.h"

namespace {

int g_argc;
char** g_argv;

// util/flag_util.h:30-47: first argv that starts with --name= wins.
bool flag_str(const std::string& name, std::string* out, bool required) {
    std::string prefix = "--" + name + "=";
    for (int i = 0; i < g_argc; i++) {
        if (strncmp(g_argv[i], prefix.c_str(), prefix.size()) == 0) {
            *out = std::string(g_argv[i] + prefix.size());
            return true;
        }
    }
    if (required) {
        printf("Missing flag: %s\n", name.c_str());
        fflush(stdout);
        std::abort();  // the reference terminates here (flag_util.h:41-44)
    }
    return false;
}

template <typename T>
void flag_num(const std::string& name, T* out, bool required) {
    std::string s;
    if (flag_str(name, &s, required)) *out = (T)atof(s.c_str());
}

void flag_i64(const std::string& name, long long* out, bool required) {
    std::string s;
    if (flag_str(name, &s, required)) *out = atoll(s.c_str());
}

[[noreturn]] void die(const char* what) {
    fprintf(stderr, "run_nmf_on_pefs: %s: %s\n", what, dnpeff_last_error());
    fflush(stderr);
    std::exit(1);
}

struct Barrier {
    std::mutex mu;
    std::condition_variable cv;
    int n, waiting = 0, gen = 0;
    explicit Barrier(int n_) : n(n_) {}
    void wait() {
        std::unique_lock<std::mutex> lk(mu);
        int g = gen;
        if (++waiting == n) { waiting = 0; gen++; cv.notify_all(); }
        else cv.wait(lk, [&] { return gen != g; });
    }
};

}  // namespace

int main(int argc, char** argv) {
    g_argc = argc;
    g_argv = argv;
    std::string output_path, pef_path, init_h_path, init_w_path, shard_mode_s = "cyclic";
    int n_components = 0, max_iters = 0, min_values = 1, n_devices_flag = 0, log_every = 10, sparsify_initial_w = 0;
    int checkpoint_every = 0;
    long long n_examples = -1, n_fisher_values = -1, seed = 43190432042ll;
    float sparsity_w = -1.f, eps = 1e-8f, init_scale = 0.f;
    flag_str("output_path", &output_path, true);
    flag_str("per_example_fishers", &pef_path, true);
    flag_num("nmf_n_components", &n_components, true);
    flag_num("nmf_max_iter", &max_iters, true);
    flag_i64("n_examples", &n_examples, false);
    flag_i64("n_fisher_values", &n_fisher_values, false);
    flag_num("min_values_per_parameter", &min_values, false);
    flag_num("sparsity_W", &sparsity_w, false);
    bool has_init_h = flag_str("initial_H_path", &init_h_path, false);
    bool has_init_w = flag_str("initial_W_path", &init_w_path, false);
    flag_num("eps", &eps, false);
    flag_i64("seed", &seed, false);
    flag_num("init_scale", &init_scale, false);
    flag_num("n_devices", &n_devices_flag, false);
    flag_num("log_every", &log_every, false);
    flag_str("shard_mode", &shard_mode_s, false);
    flag_num("sparsify_initial_W", &sparsify_initial_w, false);
    flag_num("checkpoint_every", &checkpoint_every, false);
    const int shard_mode = shard_mode_s == "contiguous" ? DNPEFF_SHARD_CONTIGUOUS : DNPEFF_SHARD_CYCLIC;

    int64_t n = 0, k = 0, dense = 0;
    if (dnpeff_pef_hdf5_info(pef_path.c_str(), &n, &k, &dense)) die("reading the D-PEF file");
    if (n_examples > 0) {
        if (n_examples > n) { fprintf(stderr, "--n_examples exceeds the file's rows\n"); return 1; }
        n = n_examples;
    }
    if (n_fisher_values > 0) {
        if (n_fisher_values > k) { fprintf(stderr, "--n_fisher_values exceeds the file's values per row\n"); return 1; }
        k = n_fisher_values;
    }
    // Pef::pefRequiresInt64Indices (pef_fisher_h5.h:57-90).  Offsets are 64-bit
    // and column ids 32-bit here in every case; the line is kept for log scrapers.
    if ((long double)n * (long double)k > 2147483647.0L) printf("Reading in PEFs using 64 bit indices.\n");
    else printf("Using 32 bit indices.\n");

    int n_dev = 0;
    if (dnpeff_device_count(&n_dev)) die("counting devices");
    if (n_dev < 1) { fprintf(stderr, "run_nmf_on_pefs: no CUDA device (there is no CPU fallback)\n"); return 1; }
    if (n_devices_flag > 0 && n_devices_flag < n_dev) n_dev = n_devices_flag;

    printf("Reading in PEFs.\n");
    fflush(stdout);

    // optional initial factors from an earlier decomposition file
    std::vector<float> W_init, H_init;
    std::vector<int32_t> kept_init;
    int64_t in_n = 0, in_m = 0, in_dense = 0;
    int32_t in_r = 0;
    for (int which = 0; which < 2; which++) {
        const bool has = which ? has_init_h : has_init_w;
        const std::string& p = which ? init_h_path : init_w_path;
        if (!has) continue;
        if (dnpeff_decomposition_hdf5_info(p.c_str(), &in_n, &in_r, &in_m, &in_dense)) die("reading the initial factors");
        if (in_r != n_components) { fprintf(stderr, "initial factors have rank %d, not %d\n", in_r, n_components); return 1; }
        if (which == 0) {
            if (in_n != n) { fprintf(stderr, "initial W has %ld rows, not %ld\n", (long)in_n, (long)n); return 1; }
            W_init.resize((size_t)in_n * in_r);
            if (dnpeff_read_decomposition_hdf5(p.c_str(), W_init.data(), nullptr, nullptr)) die("reading the initial W");
        } else {
            H_init.resize((size_t)in_r * in_m);
            kept_init.resize((size_t)in_m);
            if (dnpeff_read_decomposition_hdf5(p.c_str(), nullptr, H_init.data(), kept_init.data())) die("reading the initial H");
        }
    }

    printf("Initializing NMF.\n");
    fflush(stdout);
    uint8_t nccl_id[128];
    if (n_dev > 1 && dnpeff_nccl_unique_id(nccl_id)) die("making the NCCL id");

    struct Shard {
        std::vector<float> H;
        std::vector<int32_t> kept_ids;
        int64_t ms = 0;
    };
    std::vector<Shard> shards(n_dev);
    std::vector<float> W((size_t)n * n_components);
    std::vector<int32_t> new_to_og;
    int64_t m_kept = 0;
    std::atomic<int> failed{0};
    std::mutex err_mu;
    std::string first_error;
    Barrier bar(n_dev);

    // loadHToHostSync: the shards side by side in kept-column order, then the file
    auto save_decomposition = [&](const std::string& path) -> bool {
        std::vector<float> H((size_t)n_components * m_kept);
        for (int d = 0; d < n_dev; d++)
            for (int t = 0; t < n_components; t++)
                for (int64_t j = 0; j < shards[d].ms; j++)
                    H[(size_t)t * m_kept + shards[d].kept_ids[(size_t)j]] = shards[d].H[(size_t)t * shards[d].ms + j];
        return dnpeff_save_decomposition_hdf5(path.c_str(), W.data(), H.data(), new_to_og.data(), n, n_components,
                                              m_kept, dense) == DNPEFF_OK;
    };
    auto write_checkpoint = [&](int step) {
        const std::string final_name = output_path + ".checkpoint", tmp_name = final_name + ".tmp";
        if (!save_decomposition(tmp_name) || std::rename(tmp_name.c_str(), final_name.c_str()) != 0) {
            fprintf(stderr, "run_nmf_on_pefs: checkpoint at step %d could not be written: %s\n", step, dnpeff_last_error());
            return;  // the run itself goes on
        }
        printf("Checkpoint after step %d written to %s\n", step, final_name.c_str());
        fflush(stdout);
    };

    auto worker = [&](int d) {
        auto fail_here = [&](const char* what) {
            std::lock_guard<std::mutex> lk(err_mu);
            if (first_error.empty()) first_error = std::string(what) + ": " + dnpeff_last_error();
            failed = 1;
        };
        dnpeff_params p = {n_components, eps, (uint64_t)seed, init_scale, d, n_dev, shard_mode};
        dnpeff_engine* eng = nullptr;
        bool ok = dnpeff_create(&p, d, nullptr, &eng) == DNPEFF_OK;
        if (!ok) fail_here("creating the engine");
        bar.wait();  // nobody joins the communicator if an engine could not be made
        if (failed) { if (eng) dnpeff_destroy(eng); return; }
        if (n_dev > 1 && dnpeff_comm_init(eng, nccl_id, d, n_dev)) { fail_here("joining the communicator"); std::exit(1); }
        // every engine streams its own slice of the rows from the file; the engines
        // agree on the outcome of the reads before the collective part of the load
        if (dnpeff_load_pef_hdf5(eng, pef_path.c_str(), n, k, min_values)) {
            ok = false;
            fail_here("loading the matrix");
        }
        int64_t nn = 0, mk = 0, c0 = 0, ms = 0, nnz = 0;
        if (ok) dnpeff_get_shape(eng, &nn, &mk, &c0, &ms, &nnz);
        if (ok) {
            shards[d].ms = ms;
            shards[d].kept_ids.resize((size_t)ms);
            if (dnpeff_get_shard_columns(eng, shards[d].kept_ids.data(), nullptr)) { ok = false; fail_here("shard columns"); }
        }
        if (ok && d == 0) {
            m_kept = mk;
            new_to_og.resize((size_t)mk);
            if (dnpeff_get_new_to_og(eng, new_to_og.data())) { ok = false; fail_here("pruning map"); }
            printf("Examples: %ld, kept parameters: %ld of %ld, devices: %d\n", (long)nn, (long)mk, (long)dense, n_dev);
            fflush(stdout);
        }
        bar.wait();  // nobody enters a collective if anybody failed so far
        if (failed) { if (eng) dnpeff_destroy(eng); return; }
        // initial factors: generated, or taken from the files
        std::vector<float> Hs;
        if (!H_init.empty()) {
            bool same = (int64_t)kept_init.size() == mk;
            bar.wait();  // new_to_og is complete
            for (int64_t j = 0; same && j < mk; j++) same = kept_init[(size_t)j] == new_to_og[(size_t)j];
            if (!same) { fail_here("initial H was computed for a different set of kept parameters"); std::exit(1); }
            Hs.resize((size_t)n_components * ms);
            for (int t = 0; t < n_components; t++)
                for (int64_t j = 0; j < ms; j++)
                    Hs[(size_t)t * ms + j] = H_init[(size_t)t * mk + shards[d].kept_ids[(size_t)j]];
        }
        if (dnpeff_init_factors(eng, W_init.empty() ? nullptr : W_init.data(), Hs.empty() ? nullptr : Hs.data())) {
            fail_here("initialising the factors");
            std::exit(1);
        }
        if (sparsify_initial_w && sparsity_w > 0.f) {
            int32_t passes = 0, conv = 0;
            if (dnpeff_sparsify_w(eng, sparsity_w, 1.0f, 0, &passes, &conv)) {
                fail_here("projecting the initial W");
                std::exit(1);
            }
            if (d == 0) {
                printf("Projected the initial W onto L1 = %g, L2 = 1: %d passes%s.\n", (double)sparsity_w, (int)passes,
                       conv ? "" : " (not converged)");
                fflush(stdout);
            }
        }
        if (d == 0) { printf("Running NMF.\n"); fflush(stdout); }
        shards[d].H.resize((size_t)n_components * ms);
        auto read_factors = [&]() {
            if (d == 0 && dnpeff_get_w(eng, W.data())) { fail_here("reading W"); std::exit(1); }
            if (dnpeff_get_h(eng, shards[d].H.data())) { fail_here("reading H"); std::exit(1); }
        };
        // the run, in stretches of --checkpoint_every steps when that is set
        for (int done = 0; done < max_iters;) {
            const int stretch = checkpoint_every > 0 ? std::min(checkpoint_every, max_iters - done) : max_iters - done;
            if (dnpeff_run_steps(eng, done, stretch, log_every)) {
                fail_here("running the NMF");
                fprintf(stderr, "%s\n", first_error.c_str());
                std::exit(1);
            }
            done += stretch;
            if (checkpoint_every > 0 && done < max_iters) {
                read_factors();
                bar.wait();  // every shard of H is on the host
                if (d == 0) write_checkpoint(done);
                bar.wait();  // the host buffers may be overwritten again
            }
        }
        read_factors();
        dnpeff_destroy(eng);
    };

    std::vector<std::thread> threads;
    for (int d = 0; d < n_dev; d++) threads.emplace_back(worker, d);
    for (auto& t : threads) t.join();
    if (failed) {
        fprintf(stderr, "run_nmf_on_pefs: %s\n", first_error.c_str());
        return 1;
    }

    printf("Saving decomposition to file.\n");
    fflush(stdout);
    if (!save_decomposition(output_path)) die("saving the decomposition");
    return 0;
}
