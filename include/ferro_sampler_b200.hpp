// ferro_sampler_b200.hpp - header-only C++ adapter with the reference's own class shape.
//
// `ferro::SamplerParams` and `ferro::Sampler` below have the field layout, constructor and member signatures of
// the reference (src/sampler.h:12-34 of paragontasx/ferro), so the reference's call sites compile unchanged against
// this header:
//     src/server.cpp:545   j.sampler.reset(new Sampler(j.sp));
//     src/server.cpp:546   const int tok = j.sampler->sample(S.lg.data(), V, j.hist);
//     src/lm_cli.cpp:124   Sampler smp(a.sp);          src/lm_cli.cpp:129   smp.sample(logits, m.n_vocab, hist)
//     tests/test_kernels.cpp:351-353   Sampler s(p); s.sample(lg.data(), (int)lg.size(), std::vector<int>{1, 2, 3})
// One call samples one row through the C ABI (host logits are staged to the device; the penalised entries are
// written back into the caller's row, as the reference modifies it in place).  Schedulers that want the batched
// path call fsb_sample_batch / fsb_verify_windows directly, or ferro::sample_rows below.
//
// Unlike the reference class this one can fail (no device, CUDA error): failures throw std::runtime_error.
#pragma once
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "ferro_sampler_b200.h"

namespace ferro {

struct SamplerParams {
    float temperature = 0.05f;
    int top_k = 50;                  // 0 = off
    float top_p = 1.0f;              // 1 = off
    float min_p = 0.0f;              // 0 = off
    float repetition_penalty = 1.05f;
    int repeat_last_n = -1;          // last N tokens of the history; -1 = the whole context, 0 = no penalty
    int penalty_from = 0;            // history positions before this are never penalized
    uint64_t seed = 0;               // 0 = random
};
static_assert(sizeof(SamplerParams) == sizeof(ferro_sampler_params), "SamplerParams must mirror the C struct byte for byte");

// One engine per device, shared by all samplers of the process (the reference's samplers are only ever touched by
// the single inference worker thread, src/server.cpp:3-4; this engine is not thread-safe either).
class SamplerEngine {
public:
    static SamplerEngine& instance(int device = 0, int max_rows = 64, int max_vocab = 262144, int64_t max_hist_ids = 1 << 20) {
        static SamplerEngine e(device, max_rows, max_vocab, max_hist_ids);
        return e;
    }
    fsb_handle* handle() const { return h_; }
    void check(int rc) const {
        if (rc != FSB_OK) throw std::runtime_error(std::string("ferro sampler: ") + fsb_last_error(h_) + " (status " + std::to_string(rc) + ")");
    }
    ~SamplerEngine() {
        if (h_) fsb_destroy(h_);
    }

private:
    SamplerEngine(int device, int max_rows, int max_vocab, int64_t max_hist_ids) {
        const int rc = fsb_create(device, max_rows, max_vocab, max_hist_ids, &h_);
        if (rc != FSB_OK) throw std::runtime_error("ferro sampler: no usable CUDA device (status " + std::to_string(rc) + "); there is no CPU path");
    }
    fsb_handle* h_ = nullptr;
};

class Sampler {
public:
    explicit Sampler(const SamplerParams& p) : p_(p), eng_(&SamplerEngine::instance()) {
        eng_->check(fsb_stream_open(eng_->handle(), reinterpret_cast<const ferro_sampler_params*>(&p_), &sid_));
    }
    ~Sampler() {
        if (sid_ >= 0) fsb_stream_close(eng_->handle(), sid_);
    }
    Sampler(const Sampler&) = delete;
    Sampler& operator=(const Sampler&) = delete;

    // logits: [n_vocab], modified in place. history: all tokens of the context so far.
    int sample(float* logits, int n_vocab, const std::vector<int>& history) {
        const int64_t off[2] = {0, (int64_t)history.size()};
        int32_t tok = -1;
        static_assert(sizeof(int) == sizeof(int32_t), "history ids are 32-bit");
        eng_->check(fsb_sample_batch(eng_->handle(), 1, &sid_, logits, n_vocab, n_vocab, reinterpret_cast<const int32_t*>(history.data()), off,
                                     &tok, FSB_LOGITS_ON_HOST | FSB_WRITE_BACK));
        return tok;
    }
    const SamplerParams& params() const { return p_; }
    int stream_id() const { return sid_; }

private:
    SamplerParams p_;
    SamplerEngine* eng_;
    int sid_ = -1;
};

// The per-slot loop of a decode step (src/server.cpp:603-608) as one call: row i of `logits` is sampled by
// samplers[i] with histories[i].  Logits may live on the device (the natural place on a GPU server).
inline std::vector<int> sample_rows(const std::vector<Sampler*>& samplers, const float* logits, int64_t ld, int n_vocab,
                                    const std::vector<const std::vector<int>*>& histories, bool logits_on_host) {
    SamplerEngine& e = SamplerEngine::instance();
    const int n = (int)samplers.size();
    std::vector<int> sid((size_t)n), tok((size_t)n);
    std::vector<int64_t> off((size_t)n + 1, 0);
    std::vector<int32_t> flat;
    for (int i = 0; i < n; ++i) {
        sid[(size_t)i] = samplers[(size_t)i]->stream_id();
        flat.insert(flat.end(), histories[(size_t)i]->begin(), histories[(size_t)i]->end());
        off[(size_t)i + 1] = (int64_t)flat.size();
    }
    e.check(fsb_sample_batch(e.handle(), n, sid.data(), logits, ld, n_vocab, flat.data(), off.data(), tok.data(),
                             logits_on_host ? FSB_LOGITS_ON_HOST : 0u));
    return tok;
}

}  // namespace ferro
