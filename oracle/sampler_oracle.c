/*
 * sampler_oracle.c - CPU restatement of the reference token sampler.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker for the CUDA sampler.  It is never linked into, imported by or
 * called from the product library; only the test-suite, the smoke check and the CPU-baseline
 * leg of the benchmark load it.
 *
 * What it restates (reference paths are relative to the reference project's root):
 *   - struct SamplerParams                                   src/sampler.h:12-21
 *   - Sampler::Sampler (seeding of the 64-bit Mersenne twister) src/sampler.h:25
 *   - Sampler::sample                                        src/sampler.cpp:10-50
 *   - the speculative-window accept loop of the scheduler    src/server.cpp:626-645
 *   - the final-logit softcap applied by the Gemma-4 forward src/model_gemma4.cpp:520-521
 * and one piece of the C++ standard library that the reference relies on:
 *   - std::mt19937_64 (MT19937-64, Matsumoto & Nishimura) and the mapping that
 *     std::uniform_real_distribution<double>(0, tot) applies to ONE 64-bit output x:
 *         u = min(double(x) * 2^-64, nextafter(1, 0));   r = u * tot + 0.0
 *     (libstdc++ 13, bits/random.tcc generate_canonical with k = 1).
 *
 * Parity pin: the restatement is checked token-for-token against (a) the reference's own
 * known-answer test tests/test_kernels.cpp:348-359 (tokens 4 2 1 2 2) and (b) the reference
 * sampler itself, compiled unmodified from its own sources (see ref_driver.cpp), on seeded
 * random cases covering every branch.  Unlike the reference class it also reports the kept
 * set (ids and fp64 probabilities), which the reference computes but never exposes.
 *
 * The candidate order is a strict total order (value descending, index ascending), so any
 * correct selection + sort gives the same sequence as std::partial_sort / std::sort.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    float temperature;
    int top_k;
    float top_p;
    float min_p;
    float repetition_penalty;
    int repeat_last_n;
    int penalty_from;
    /* 4 bytes of padding here, as in the reference struct on x86-64 */
    uint64_t seed;
} oracle_params;

/* ------------------------------------------------------------------ MT19937-64 */
#define MT_NN 312
#define MT_MM 156
typedef struct {
    uint64_t mt[MT_NN];
    int idx;
} oracle_mt64;

void oracle_mt64_seed(oracle_mt64* g, uint64_t seed) {
    g->mt[0] = seed;
    for (int i = 1; i < MT_NN; ++i)
        g->mt[i] = 6364136223846793005ULL * (g->mt[i - 1] ^ (g->mt[i - 1] >> 62)) + (uint64_t)i;
    g->idx = MT_NN;
}

uint64_t oracle_mt64_next(oracle_mt64* g) {
    static const uint64_t MATRIX_A = 0xB5026F5AA96619E9ULL, UM = 0xFFFFFFFF80000000ULL, LM = 0x7FFFFFFFULL;
    if (g->idx >= MT_NN) {
        for (int i = 0; i < MT_NN; ++i) {
            uint64_t x = (g->mt[i] & UM) | (g->mt[(i + 1) % MT_NN] & LM);
            g->mt[i] = g->mt[(i + MT_MM) % MT_NN] ^ (x >> 1) ^ ((x & 1ULL) ? MATRIX_A : 0ULL);
        }
        g->idx = 0;
    }
    uint64_t x = g->mt[g->idx++];
    x ^= (x >> 29) & 0x5555555555555555ULL;
    x ^= (x << 17) & 0x71D67FFFEDA60000ULL;
    x ^= (x << 37) & 0xFFF7EEE000000000ULL;
    x ^= (x >> 43);
    return x;
}

/* uniform in [0, 1) from one engine output, as libstdc++ maps it */
double oracle_canonical(uint64_t x) {
    double u = (double)x / 18446744073709551616.0;
    if (u >= 1.0) u = nextafter(1.0, 0.0);
    return u;
}

/* ------------------------------------------------------------------ softcap (producer side) */
void oracle_softcap(float* logits, int64_t n, float cap) {
    for (int64_t i = 0; i < n; ++i) logits[i] = cap * tanhf(logits[i] / cap);
}

/* ------------------------------------------------------------------ sample() */
typedef struct {
    float v;
    int id;
} cand_t;

/* "a comes before b": value descending, index ascending on equal values (-0.0f == +0.0f) */
static inline int before(cand_t a, cand_t b) { return a.v > b.v || (a.v == b.v && a.id < b.id); }

static int cmp_qsort(const void* pa, const void* pb) {
    cand_t a = *(const cand_t*)pa, b = *(const cand_t*)pb;
    if (before(a, b)) return -1;
    if (before(b, a)) return 1;
    return 0;
}

/* min-heap on the "before" order: the root is the candidate that comes LAST among the kept */
static void sift_down(cand_t* h, int n, int i) {
    for (;;) {
        int l = 2 * i + 1, r = l + 1, m = i;
        if (l < n && before(h[m], h[l])) m = l;
        if (r < n && before(h[m], h[r])) m = r;
        if (m == i) return;
        cand_t t = h[i]; h[i] = h[m]; h[m] = t;
        i = m;
    }
}

/* penalty window of src/sampler.cpp:13-14: ids hist[b .. hist_len) */
int64_t oracle_window_begin(const oracle_params* p, int64_t hist_len) {
    int64_t b = (p->repeat_last_n > 0 && (int64_t)p->repeat_last_n < hist_len) ? hist_len - (int64_t)p->repeat_last_n : 0;
    if (p->penalty_from > 0 && (int64_t)p->penalty_from > b) b = (int64_t)p->penalty_from;
    return b;
}

/*
 * One sampler call.  logits[n] is modified in place exactly as the reference does.
 * rng may be NULL for greedy calls.  Optional outputs (each may be NULL):
 *   kept_ids[cap], kept_pr[cap]  the first min(keep, cap) kept candidates in order, with their
 *                                normalised probabilities (pr = exp(..)/sum over the k candidates)
 *   n_keep                       size of the kept set after min-p / top-p
 *   n_cand                       k, the number of candidates that entered the softmax
 *   rng_word                     the raw 64-bit engine output consumed (0 for greedy)
 *   r_tot[3]                     {r, tot} of the draw, and the probability of the last kept candidate (tot minus it is
 *                                the cumulative probability the top-p cut saw just before its last step)
 * Returns the token id, or -1 on allocation failure.
 */
int oracle_sample(const oracle_params* p, oracle_mt64* rng, float* logits, int n, const int* hist, int64_t hist_len,
                  int* kept_ids, double* kept_pr, int cap, int* n_keep, int* n_cand, uint64_t* rng_word, double* r_tot) {
    if (n_keep) *n_keep = 0;
    if (n_cand) *n_cand = 0;
    if (rng_word) *rng_word = 0;
    /* repetition penalty, once per distinct id in the window (src/sampler.cpp:11-18) */
    if (p->repetition_penalty != 1.0f && p->repeat_last_n != 0 && hist_len > 0) {
        int64_t b = oracle_window_begin(p, hist_len);
        uint8_t* seen = (uint8_t*)calloc((size_t)n + 1, 1);
        if (!seen) return -1;
        for (int64_t i = b; i < hist_len; ++i) {
            int id = hist[i];
            if (id >= 0 && id < n && !seen[id]) {
                seen[id] = 1;
                logits[id] = logits[id] > 0 ? logits[id] / p->repetition_penalty : logits[id] * p->repetition_penalty;
            }
        }
        free(seen);
    }
    /* greedy: first index of the maximum, no engine output consumed (src/sampler.cpp:19-23) */
    if (p->temperature <= 0.0f || p->top_k == 1) {
        int best = 0;
        for (int i = 1; i < n; ++i)
            if (logits[i] > logits[best]) best = i;
        return best;
    }
    /* candidates (src/sampler.cpp:25-35) */
    const int k = (p->top_k > 0 && p->top_k < n) ? p->top_k : n;
    cand_t* c = (cand_t*)malloc(sizeof(cand_t) * (size_t)k);
    double* pr = (double*)malloc(sizeof(double) * (size_t)k);
    if (!c || !pr) { free(c); free(pr); return -1; }
    if (k < n) {
        for (int i = 0; i < k; ++i) { c[i].v = logits[i]; c[i].id = i; }
        for (int i = k / 2 - 1; i >= 0; --i) sift_down(c, k, i);
        for (int i = k; i < n; ++i) {
            cand_t x = { logits[i], i };
            if (before(x, c[0])) { c[0] = x; sift_down(c, k, 0); }
        }
    } else {
        for (int i = 0; i < n; ++i) { c[i].v = logits[i]; c[i].id = i; }
    }
    qsort(c, (size_t)k, sizeof(cand_t), cmp_qsort);
    /* softmax over the candidates in fp64, sequential sum in sorted order (src/sampler.cpp:37-41) */
    const float mx = c[0].v;
    double sum = 0;
    for (int i = 0; i < k; ++i) { pr[i] = exp((double)(c[i].v - mx) / p->temperature); sum += pr[i]; }
    for (int i = 0; i < k; ++i) pr[i] /= sum;
    size_t keep = (size_t)k;
    /* min-p then top-p, no renormalisation (src/sampler.cpp:43-44) */
    if (p->min_p > 0.0f) { const double thr = pr[0] * p->min_p; while (keep > 1 && pr[keep - 1] < thr) --keep; }
    if (p->top_p < 1.0f) {
        double cum = 0; size_t i = 0;
        for (; i < keep; ++i) { cum += pr[i]; if (cum >= p->top_p) { ++i; break; } }
        size_t m = keep < i ? keep : i;
        keep = m > 1 ? m : 1;
    }
    /* draw (src/sampler.cpp:45-49) */
    double tot = 0;
    for (size_t i = 0; i < keep; ++i) tot += pr[i];
    const uint64_t w = oracle_mt64_next(rng);
    const double r = oracle_canonical(w) * tot + 0.0;
    int tok = c[keep - 1].id;
    double cum = 0;
    for (size_t i = 0; i < keep; ++i) { cum += pr[i]; if (r <= cum) { tok = c[i].id; break; } }
    if (n_keep) *n_keep = (int)keep;
    if (n_cand) *n_cand = k;
    if (rng_word) *rng_word = w;
    if (r_tot) { r_tot[0] = r; r_tot[1] = tot; r_tot[2] = pr[keep - 1]; }
    for (size_t i = 0; i < keep && (int)i < cap; ++i) {
        if (kept_ids) kept_ids[i] = c[i].id;
        if (kept_pr) kept_pr[i] = pr[i];
    }
    free(c); free(pr);
    return tok;
}

/*
 * A batch of independent rows, each with its own parameters, engine and history
 * ("for every active slot: sampler->sample(row)" of src/server.cpp:603-608).
 * hist_off has n_rows + 1 entries into hist_flat.  rngs[i] is advanced in place.
 * kept outputs are [n_rows][cap] or NULL.
 */
int oracle_sample_rows(int n_rows, const oracle_params* params, oracle_mt64* rngs, float* logits, int64_t ld, int n,
                       const int* hist_flat, const int64_t* hist_off, int* tokens,
                       int* kept_ids, double* kept_pr, int cap, int* n_keep, uint64_t* rng_words, double* r_tot) {
    for (int i = 0; i < n_rows; ++i) {
        int t = oracle_sample(&params[i], rngs ? &rngs[i] : NULL, logits + (int64_t)i * ld, n,
                              hist_flat + hist_off[i], hist_off[i + 1] - hist_off[i],
                              kept_ids ? kept_ids + (int64_t)i * cap : NULL, kept_pr ? kept_pr + (int64_t)i * cap : NULL, cap,
                              n_keep ? n_keep + i : NULL, NULL, rng_words ? rng_words + i : NULL, r_tot ? r_tot + 3 * i : NULL);
        if (t < 0) return -1;
        tokens[i] = t;
    }
    return 0;
}

/*
 * Speculative verification window of one stream (src/server.cpp:626-636, without the
 * end-of-sequence bookkeeping of gen_token): rows[0] is the stream's last token, rows[1..m-1]
 * the drafts; logits is [m][ld].  Rows are sampled in order with the history growing by each
 * sampled token; row r+1 is sampled only if the token sampled from row r equals rows[r+1].
 * hist must have room for hist_len + m ids; on return it holds the accepted tokens appended.
 * tokens[r] is written for the rows that were sampled.  Returns acc (rows sampled);
 * *confirmed = number of drafts that were confirmed.
 */
int oracle_verify_window(const oracle_params* p, oracle_mt64* rng, float* logits, int64_t ld, int n, int m, const int* rows,
                         int* hist, int64_t hist_len, int* tokens, int* confirmed) {
    int acc = 0, conf = 0;
    for (int r = 0; r < m; ++r) {
        int tok = oracle_sample(p, rng, logits + (int64_t)r * ld, n, hist, hist_len, NULL, NULL, 0, NULL, NULL, NULL, NULL);
        if (tok < 0) return -1;
        tokens[r] = tok;
        hist[hist_len++] = tok;
        acc = r + 1;
        if (r + 1 < m && tok == rows[r + 1]) { ++conf; continue; }
        break;
    }
    if (confirmed) *confirmed = conf;
    return acc;
}

/*
 * Prompt-lookup drafting (lookup_draft, src/server.cpp:552-564): for n = min(4, len - 1) down to min_n, the start
 * positions p = len - n - 1 .. 0 are tried from the most recent one; at the first p where h[p .. p+n) equals the
 * last n tokens, the tokens after the occurrence are copied - at most kmax, stopping before `eos` - and returned if
 * there is at least one; otherwise the search goes on (earlier p, then shorter n).  Returns the number of drafts.
 * Parity unpinned: the reference holds no vectors for this function (its test needs a running server); the
 * restatement follows the source line by line and tests/ compare it with an independent brute-force search.
 */
int oracle_lookup_draft(const int* h, int len, int kmax, int eos, int min_n, int* drafts) {
    for (int n = (len - 1 < 4 ? len - 1 : 4); n >= min_n; --n) {
        for (int p = len - n - 1; p >= 0; --p) {
            int eq = 1;
            for (int k = 0; k < n; ++k)
                if (h[p + k] != h[len - n + k]) { eq = 0; break; }
            if (!eq) continue;
            int cnt = 0;
            for (int k = p + n; k < len && cnt < kmax; ++k) {
                if (h[k] == eos) break;
                drafts[cnt++] = h[k];
            }
            if (cnt > 0) return cnt;
        }
    }
    return 0;
}
