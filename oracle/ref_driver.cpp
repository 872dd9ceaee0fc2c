// ref_driver.cpp - C entry points around the UNMODIFIED reference sampler.  TEST INFRASTRUCTURE ONLY.
//
// Compiled together with the reference's own src/sampler.cpp (from where it lies in the reference
// checkout, never copied) with the reference's flags (Makefile:2: -O3 -std=c++17 -fno-math-errno -fPIC)
// into oracle/_ref/libferro_ref.so.  It is used to (a) pin the C restatement in sampler_oracle.c,
// (b) generate the golden vectors under tests/golden/, and (c) time the reference's CPU path beside
// the GPU path.  Nothing in the product library links or loads it.
//
// The wrappers mirror the reference's call sites:
//   ref_sampler_sample      one call of Sampler::sample              (src/sampler.cpp:10)
//   ref_sample_rows         the per-slot loop of a decode step       (src/server.cpp:603-608)
//   ref_verify_window       the accept loop of a verification window (src/server.cpp:626-636)
//   ref_time_rows           the per-slot loop, timed, rows spread over host threads
#include <chrono>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "sampler.h"   // the reference's header, found through -I<reference>/src

using ferro::Sampler;
using ferro::SamplerParams;

static_assert(sizeof(SamplerParams) == 40, "reference parameter struct layout changed");

extern "C" {

int ref_sizeof_params() { return (int)sizeof(SamplerParams); }
int ref_sizeof_sampler() { return (int)sizeof(Sampler); }

void* ref_sampler_new(const SamplerParams* p) { return new Sampler(*p); }
void ref_sampler_free(void* s) { delete static_cast<Sampler*>(s); }

int ref_sampler_sample(void* s, float* logits, int n, const int* hist, int64_t hist_len) {
    std::vector<int> h(hist, hist + hist_len);
    return static_cast<Sampler*>(s)->sample(logits, n, h);
}

// Independent rows, one fresh Sampler per row (seeded from params[i].seed), one call each.
void ref_sample_rows(int n_rows, const SamplerParams* params, float* logits, int64_t ld, int n,
                     const int* hist_flat, const int64_t* hist_off, int* tokens) {
    for (int i = 0; i < n_rows; ++i) {
        Sampler s(params[i]);
        std::vector<int> h(hist_flat + hist_off[i], hist_flat + hist_off[i + 1]);
        tokens[i] = s.sample(logits + (int64_t)i * ld, n, h);
    }
}

// n_draws successive calls on ONE sampler (one engine stream); every call starts from a fresh copy
// of the same logits row because sample() modifies its input.
void ref_sample_repeat(const SamplerParams* p, const float* logits, int n, const int* hist, int64_t hist_len,
                       int n_draws, int* tokens) {
    Sampler s(*p);
    std::vector<int> h(hist, hist + hist_len);
    std::vector<float> row((size_t)n);
    for (int d = 0; d < n_draws; ++d) {
        std::memcpy(row.data(), logits, sizeof(float) * (size_t)n);
        tokens[d] = s.sample(row.data(), n, h);
    }
}

// Verification window of one stream, as the scheduler runs it (without gen_token's end-of-sequence
// bookkeeping): sample row r, append the token to the history, go on only while it equals the next draft.
int ref_verify_window(void* sampler, float* logits, int64_t ld, int n, int m, const int* rows,
                      const int* hist, int64_t hist_len, int* tokens, int* confirmed) {
    Sampler* s = static_cast<Sampler*>(sampler);
    std::vector<int> h(hist, hist + hist_len);
    int acc = 0, conf = 0;
    for (int r = 0; r < m; ++r) {
        const int tok = s->sample(logits + (int64_t)r * ld, n, h);
        tokens[r] = tok;
        h.push_back(tok);
        acc = r + 1;
        if (r + 1 < m && tok == rows[r + 1]) { ++conf; continue; }
        break;
    }
    if (confirmed) *confirmed = conf;
    return acc;
}

// The decode-step loop timed on the host: rows are dealt to n_threads std::threads in contiguous
// blocks, one Sampler per row (built outside the timed region), steady_clock around the sample()
// calls only.  logits must be a fresh copy (it is modified).  Returns seconds (max over threads).
double ref_time_rows(int n_rows, const SamplerParams* params, float* logits, int64_t ld, int n,
                     const int* hist_flat, const int64_t* hist_off, int* tokens, int n_threads) {
    if (n_threads < 1) n_threads = 1;
    if (n_threads > n_rows) n_threads = n_rows;
    std::vector<Sampler> samplers;
    samplers.reserve((size_t)n_rows);
    std::vector<std::vector<int>> hs((size_t)n_rows);
    for (int i = 0; i < n_rows; ++i) {
        samplers.emplace_back(params[i]);
        hs[(size_t)i].assign(hist_flat + hist_off[i], hist_flat + hist_off[i + 1]);
    }
    std::vector<double> secs((size_t)n_threads, 0.0);
    auto work = [&](int t) {
        const int lo = (int)((int64_t)n_rows * t / n_threads), hi = (int)((int64_t)n_rows * (t + 1) / n_threads);
        const auto t0 = std::chrono::steady_clock::now();
        for (int i = lo; i < hi; ++i) tokens[i] = samplers[(size_t)i].sample(logits + (int64_t)i * ld, n, hs[(size_t)i]);
        secs[(size_t)t] = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    };
    if (n_threads == 1) {
        work(0);
    } else {
        std::vector<std::thread> th;
        const auto t0 = std::chrono::steady_clock::now();
        for (int t = 0; t < n_threads; ++t) th.emplace_back(work, t);
        for (auto& x : th) x.join();
        const double wall = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        return wall;   // includes thread start/join: what a multi-threaded caller would pay
    }
    return secs[0];
}

int ref_hardware_threads() { return (int)std::thread::hardware_concurrency(); }

}  // extern "C"
