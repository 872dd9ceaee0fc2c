// call_latency.cpp - wall-clock cost of the public calls of the C ABI, measured from C++ (no Python in the loop).
// Usage: call_latency [rows vocab hist iters]; prints one JSON object.  Built by bench.py and by the tests with
//   g++ -std=c++17 -O2 -I include -I $CUDA/include tests/call_latency.cpp -L ferro_b200/lib -lferro_sampler_b200 -L $CUDA/lib64 -lcudart
// The CUDA runtime is used only to put synthetic logits into device memory.
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#include "ferro_sampler_b200.h"

namespace {

double median_us(std::vector<double>& v) {
    std::sort(v.begin(), v.end());
    return v[v.size() / 2];
}

template <class F>
double time_calls(int iters, F&& call) {
    for (int i = 0; i < 5; ++i) call(i);
    std::vector<double> us;
    for (int i = 0; i < iters; ++i) {
        const auto t0 = std::chrono::steady_clock::now();
        call(i);
        us.push_back(std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count());
    }
    return median_us(us);
}

#define CHECK(x)                                                                          \
    do {                                                                                  \
        const int rc_ = (x);                                                              \
        if (rc_ != 0) {                                                                   \
            std::fprintf(stderr, "%s failed: %d (%s)\n", #x, rc_, fsb_last_error(h));     \
            return 1;                                                                     \
        }                                                                                 \
    } while (0)

}  // namespace

int main(int argc, char** argv) {
    const int rows = argc > 1 ? std::atoi(argv[1]) : 64;
    const int vocab = argc > 2 ? std::atoi(argv[2]) : 262144;
    const int hist = argc > 3 ? std::atoi(argv[3]) : 512;
    const int iters = argc > 4 ? std::atoi(argv[4]) : 200;
    fsb_handle* h = nullptr;
    if (fsb_create(0, rows, vocab, (int64_t)rows * (hist + 4096) * 2 + 64, &h) != 0) {
        std::fprintf(stderr, "fsb_create failed (no B200?)\n");
        return 2;
    }
    // synthetic logits: several matrices so that consecutive calls stream from HBM, not from L2
    const size_t elems = (size_t)rows * vocab;
    const int n_buf = (int)std::max<size_t>(2, (size_t)600e6 / (elems * 4));
    std::vector<float*> bufs((size_t)n_buf, nullptr);
    {
        std::mt19937 g(7);
        std::normal_distribution<float> nd(0.f, 3.f);
        std::vector<float> host(elems);
        for (auto& b : bufs) {
            for (size_t i = 0; i < elems; i += 97) host[i] = nd(g);   // sparse refresh keeps set-up short; values differ per buffer
            if (&b == &bufs[0])
                for (auto& x : host) x = nd(g);
            if (cudaMalloc(reinterpret_cast<void**>(&b), elems * 4) != cudaSuccess) return 3;
            cudaMemcpy(b, host.data(), elems * 4, cudaMemcpyHostToDevice);
        }
    }
    std::vector<int> sids((size_t)rows);
    std::vector<int32_t> hist_flat((size_t)rows * hist);
    std::vector<int64_t> hist_off((size_t)rows + 1, 0);
    std::mt19937 g(11);
    for (int r = 0; r < rows; ++r) {
        ferro_sampler_params p;
        fsb_params_default(&p);
        p.temperature = 1.0f;
        p.top_k = 64;
        p.top_p = 0.95f;
        p.repetition_penalty = (r & 1) ? 1.1f : 1.0f;
        p.seed = 7 + (uint64_t)r;
        CHECK(fsb_stream_open(h, &p, &sids[(size_t)r]));
        for (int i = 0; i < hist; ++i) hist_flat[(size_t)r * hist + i] = (int32_t)(g() % (unsigned)vocab);
        hist_off[(size_t)r + 1] = (int64_t)(r + 1) * hist;
        CHECK(fsb_stream_history_set(h, sids[(size_t)r], hist_flat.data() + (size_t)r * hist, hist));
    }
    std::vector<int32_t> tok((size_t)rows);
    const double explicit_us = time_calls(iters, [&](int i) {
        fsb_sample_batch(h, rows, sids.data(), bufs[(size_t)(i % n_buf)], vocab, vocab, hist_flat.data(), hist_off.data(), tok.data(), 0);
    });
    const double resident_us = time_calls(iters, [&](int i) {
        fsb_sample_batch_resident(h, rows, sids.data(), bufs[(size_t)(i % n_buf)], vocab, vocab, tok.data(), 0);
    });
    const double append_us = time_calls(iters, [&](int i) {
        fsb_sample_batch_resident(h, rows, sids.data(), bufs[(size_t)(i % n_buf)], vocab, vocab, tok.data(), FSB_APPEND_SAMPLED);
    });
    // speculative windows: the rows as streams x m windows, greedy
    const int m = 17, streams = std::max(1, std::min(rows / m, 8));
    double windows_us = 0.0, drafts_us = 0.0;
    if (rows >= m) {
        std::vector<int> row_off((size_t)streams + 1), acc((size_t)streams), conf((size_t)streams);
        std::vector<int32_t> rows_flat((size_t)streams * m), wt((size_t)streams * m);
        for (int s = 0; s <= streams; ++s) row_off[(size_t)s] = s * m;
        for (auto& x : rows_flat) x = (int32_t)(g() % (unsigned)vocab);
        windows_us = time_calls(iters, [&](int i) {
            fsb_verify_windows_resident(h, streams, sids.data(), row_off.data(), rows_flat.data(), bufs[(size_t)(i % n_buf)], vocab, vocab, nullptr,
                                        wt.data(), acc.data(), conf.data(), 0);
        });
        std::vector<int> kmax((size_t)streams, 7), min_n((size_t)streams, 2), n_out((size_t)streams);
        std::vector<int32_t> drafts((size_t)streams * 8);
        drafts_us = time_calls(iters, [&](int) {
            fsb_lookup_drafts_resident(h, streams, sids.data(), kmax.data(), min_n.data(), 1, drafts.data(), 8, n_out.data());
        });
    }
    std::printf("{\"rows\": %d, \"vocab\": %d, \"history_ids\": %d, \"iters\": %d, \"sample_batch_device_logits_us\": %.2f, "
                "\"sample_batch_resident_us\": %.2f, \"sample_batch_resident_append_us\": %.2f, \"verify_windows_resident_%dx%d_us\": %.2f, "
                "\"lookup_drafts_resident_us\": %.2f}\n",
                rows, vocab, hist, iters, explicit_us, resident_us, append_us, streams, m, windows_us, drafts_us);
    for (auto b : bufs) cudaFree(b);
    fsb_destroy(h);
    return 0;
}
