// fsb_fullrow.cu - the multi-pass full-row kernel of the B200 batched token sampler (sm_100a).
//
// Rows whose effective candidate count k exceeds kMaxK - above all `top_k == 0`, where the reference sorts the
// whole vocabulary (src/sampler.cpp:32-35 of paragontasx/ferro) - cannot keep their candidates on chip.  One CTA
// works on one such row in several passes over the row (which stays in L2 after the first):
//   1. penalty bitmap of the row, row maximum                                      (src/sampler.cpp:11-18, :38)
//   2. if k < n: the k-th candidate by a counting radix descent over the candidate keys      (:27-31)
//   3. weights e_i = exp((double)(x_i - max) / T) of the candidates, kept as 2^-62 fixed point      (:40)
//   4. min-p bound, top-p crossing and the draw by radix descents over accumulated weight     (:43-49)
// Before the descents of step 4 the kernel tries a shortcut: the elements that weigh at least 2^-10 of the row's
// total are, in candidate order, a prefix of the sorted row; at most kHeavyCap of them are gathered, sorted and
// summed exactly, and the top-p crossing, the kept set and the draw are looked up in that prefix.  A descent over
// the whole row is only run when a target lies beyond the prefix (flat rows).  Both ways give the same answer.
// Sums of weights are accumulated as integers, so they do not depend on the order in which threads add: the
// result is deterministic and differs from the reference's sequential fp64 sums by rounding only (~1e-13).
#include <cuda_runtime.h>

#include "fsb_device.cuh"

namespace fsb {
namespace {

constexpr int kFullThreads = 1024;
constexpr int kFullWarps = kFullThreads / 32;

struct U128 {
    u64 hi, lo;
};
__device__ __forceinline__ U128 u128_add(U128 a, U128 b) {
    U128 r;
    r.lo = a.lo + b.lo;
    r.hi = a.hi + b.hi + (r.lo < a.lo ? 1ull : 0ull);
    return r;
}
__device__ __forceinline__ bool u128_ge(U128 a, U128 b) { return a.hi > b.hi || (a.hi == b.hi && a.lo >= b.lo); }
__device__ __forceinline__ double u128_to_double(U128 a) {
    return __dadd_rn(__dmul_rn(__ull2double_rn(a.hi), 18446744073709551616.0), __ull2double_rn(a.lo));
}
// smallest U128 that is >= d (d >= 0, finite, below 2^127)
__device__ __forceinline__ U128 double_to_u128_ceil(double d) {
    U128 r{0ull, 0ull};
    if (!(d > 0.0)) return r;
    const double hi_d = floor(d * (1.0 / 18446744073709551616.0));
    r.hi = __double2ull_rz(hi_d);
    const double rest = d - hi_d * 18446744073709551616.0;   // exact: both are multiples of ulp(d)
    r.lo = __double2ull_ru(rest);
    if (rest >= 18446744073709551616.0) { r.hi += 1ull; r.lo = 0ull; }
    return r;
}

constexpr int kHistCopies = 16;  // the level histogram is kept in several copies (one per lane group): fewer threads
                                 // hit the same shared-memory word at once; the copies are added up before the walk
struct FullShared {
    u64 h_lo[kHistCopies * 256];        // weight histogram of one radix level, low words (copy c at [c * 256])
    u64 h_hi[kHistCopies * 256];        // high words
    unsigned h_cnt[kHistCopies * 256];  // element counts per digit
    u64 red[2 * kFullWarps];
    float redf[kFullWarps];
    u64 res_pfx;
    U128 res_above;
    int res_found;
    int heavy_cnt;        // elements gathered into the heavy prefix
    int hit[2];           // results of look-ups in the prefix
};

constexpr int kHeavyCap = 1024;   // one element per thread
// Heavy prefix of a row in shared memory: gathered composites, the same in order, and their cumulative weights.
struct Heavy {
    u64* raw;      // [kHeavyCap] as gathered; reused for the sorted runs
    u64* sorted;   // [kHeavyCap] descending
    u64* cum_lo;   // [kHeavyCap] inclusive cumulative weight, low and high words
    u64* cum_hi;
};

struct FullArgs {
    const float* logits;
    const RowDesc* rows;      // the rows of this kernel
    const int32_t* hist;
    u64* weights;             // [n_rows][n_vocab] fixed-point weights (scratch)
    int32_t* tokens;
    int32_t* kept_ids;        // [rows][kMaxK]: entry 0 = id of the last kept candidate
    double* kept_pr;          // [rows][kMaxK]: entry 0 = total probability of the kept set
    int32_t* kept_n;
    unsigned* status;
    int32_t n_vocab;
    int32_t vocab_offset;
    int32_t write_back;
    float softcap;
};

// The row as the sampler sees it: softcap, then penalty on the columns flagged in the bitmap.
struct RowView {
    const float* row;
    const unsigned* bitmap;   // null: no penalty
    float pen, cap;
    __device__ __forceinline__ float fix(float x, int i) const {   // a loaded logit as the sampler sees it
        if (cap != 0.0f) x = __fmul_rn(cap, tanhf(__fdiv_rn(x, cap)));
        if (bitmap && ((bitmap[i >> 5] >> (i & 31)) & 1u)) x = x > 0.0f ? __fdiv_rn(x, pen) : __fmul_rn(x, pen);
        return x;
    }
    __device__ __forceinline__ float at(int i) const { return fix(row[i], i); }
};

__device__ __forceinline__ u64 block_max_u64(u64 v, FullShared* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (lane == 0) sh->red[warp] = v;
    __syncthreads();
    u64 r = sh->red[0];
    for (int w = 1; w < kFullWarps; ++w) r = max(r, sh->red[w]);
    __syncthreads();
    return r;
}
__device__ __forceinline__ u64 block_min_u64(u64 v, FullShared* sh) { return ~block_max_u64(~v, sh); }

// Adds (digit, weight, 1) to the level histogram; a thread collects runs of equal digits before touching shared memory.
struct HistAcc {
    int d;
    U128 w;
    unsigned c;
    __device__ __forceinline__ void flush(FullShared* sh) {
        if (d < 0 || c == 0u) return;
        const int b = (int)(threadIdx.x & (kHistCopies - 1)) * 256 + d;
        atomicAdd(&sh->h_cnt[b], c);
        if (w.lo) {
            const u64 old = atomicAdd(&sh->h_lo[b], w.lo);
            if (old + w.lo < old) atomicAdd(&sh->h_hi[b], 1ull);
        }
        if (w.hi) atomicAdd(&sh->h_hi[b], w.hi);
        c = 0u;
        w = U128{0ull, 0ull};
    }
    __device__ __forceinline__ void add(int digit, u64 weight, FullShared* sh) {
        if (digit != d) {
            flush(sh);
            d = digit;
        }
        const u64 lo = w.lo + weight;
        if (lo < w.lo) w.hi += 1ull;
        w.lo = lo;
        ++c;
    }
};

// Radix descent over accumulated weight.  Candidates are the elements with composite >= floor_c; element j has
// weight W_j (from `weights`, or 1 when weights is null).  With P(c) = sum of W_j over candidates with composite
// >= c, finds c* = the largest candidate composite with P(c*) >= target.  Returns false if even the whole
// candidate set weighs less than target.  *above_out = P(c*) - W(c*) ... i.e. the weight strictly before c*.
__device__ bool weight_descent(const RowView& rv, int n, int id_base, const u64* weights, u64 floor_c, U128 target, u64 hi_c, u64 lo_c,
                               FullShared* sh, u64* c_out, U128* above_out) {
    const int tid = threadIdx.x;
    u64 mask = 0ull, pfx = 0ull;
    U128 above{0ull, 0ull};
    if (hi_c != lo_c) {
        const int hb0 = 63 - __clzll((long long)(hi_c ^ lo_c));
        mask = (hb0 == 63) ? 0ull : (~0ull << (hb0 + 1));
        pfx = hi_c & mask;
    } else {
        mask = ~0ull;
        pfx = hi_c;
    }
    int hb = (mask == ~0ull) ? -1 : 63 - __clzll((long long)(~mask));
    bool found = true;
    if (hb < 0) {   // a single distinct composite: check that it weighs enough
        U128 tot{0ull, 0ull};
        for (int i = tid; i < n; i += kFullThreads) {
            const float x = rv.at(i);
            if (!(x == x)) continue;
            const u64 c = make_comp(x, i + id_base);
            if (c == pfx && c >= floor_c) tot.lo += weights ? weights[i] : 1ull;
        }
        const u64 t = block_max_u64(tot.lo, sh);
        found = u128_ge(U128{0ull, t}, target);
    }
    while (hb >= 0 && found) {
        const int w = hb + 1 < 8 ? hb + 1 : 8, lo = hb + 1 - w;
        const unsigned dmask = (1u << w) - 1u;
        for (int i = tid; i < kHistCopies * 256; i += kFullThreads) {
            sh->h_lo[i] = 0ull;
            sh->h_hi[i] = 0ull;
            sh->h_cnt[i] = 0u;
        }
        __syncthreads();
        HistAcc acc{-1, U128{0ull, 0ull}, 0u};
        for (int i = tid; i < n; i += kFullThreads) {
            const float x = rv.at(i);
            if (!(x == x)) continue;
            const u64 c = make_comp(x, i + id_base);
            if (c >= floor_c && (c & mask) == pfx) acc.add((int)((unsigned)(c >> lo) & dmask), weights ? weights[i] : 1ull, sh);
        }
        acc.flush(sh);
        __syncthreads();
        if (tid < 256) {   // add the copies up into copy 0
            U128 t{sh->h_hi[tid], sh->h_lo[tid]};
            unsigned cn = sh->h_cnt[tid];
#pragma unroll
            for (int c = 1; c < kHistCopies; ++c) {
                t = u128_add(t, U128{sh->h_hi[c * 256 + tid], sh->h_lo[c * 256 + tid]});
                cn += sh->h_cnt[c * 256 + tid];
            }
            sh->h_lo[tid] = t.lo;
            sh->h_hi[tid] = t.hi;
            sh->h_cnt[tid] = cn;
        }
        __syncthreads();
        if (tid == 0) {   // walk the digits from the top until the accumulated weight reaches the target
            U128 run = above;
            int d = (int)dmask;
            int hit = -1;
            for (; d >= 0; --d) {
                const U128 with = u128_add(run, U128{sh->h_hi[d], sh->h_lo[d]});
                if (sh->h_cnt[d] != 0u && u128_ge(with, target)) {
                    hit = d;
                    break;
                }
                run = with;
            }
            sh->res_found = hit >= 0 ? 1 : 0;
            sh->res_pfx = hit >= 0 ? (u64)(unsigned)hit << lo : 0ull;
            sh->res_above = run;
        }
        __syncthreads();
        found = sh->res_found != 0;
        pfx |= sh->res_pfx;
        above = sh->res_above;
        mask |= (u64)dmask << lo;
        hb = lo - 1;
        __syncthreads();
    }
    if (found) {
        *c_out = pfx;
        *above_out = above;
    }
    return found;
}


// Index of the first entry of the heavy prefix whose cumulative weight reaches `target`, or -1 if even the whole
// prefix weighs less.  All threads of the CTA must call; `slot` is 0 or 1.
__device__ int heavy_first_reaching(const Heavy& hv, int m, U128 target, FullShared* sh, int slot) {
    const int t = threadIdx.x;
    if (t == 0) sh->hit[slot] = -1;
    __syncthreads();
    if (t < m) {
        const bool here = u128_ge(U128{hv.cum_hi[t], hv.cum_lo[t]}, target);
        const bool before = t > 0 && u128_ge(U128{hv.cum_hi[t - 1], hv.cum_lo[t - 1]}, target);
        if (here && !before) sh->hit[slot] = t;
    }
    __syncthreads();
    const int r = sh->hit[slot];
    __syncthreads();
    return r;
}

__global__ void __launch_bounds__(kFullThreads, 1) full_row_kernel(const FullArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    FullShared* sh = reinterpret_cast<FullShared*>(smem_raw);
    unsigned* bitmap = reinterpret_cast<unsigned*>(smem_raw + sizeof(FullShared));
    const int tid = threadIdx.x;
    const RowDesc d = a.rows[blockIdx.x];
    const int n = a.n_vocab;
    Heavy hv;
    hv.raw = reinterpret_cast<u64*>(smem_raw + sizeof(FullShared) + ((sizeof(unsigned) * (size_t)((n + 31) / 32) + 15) & ~(size_t)15));
    hv.sorted = hv.raw + kHeavyCap;
    hv.cum_lo = hv.sorted + kHeavyCap;
    hv.cum_hi = hv.cum_lo + kHeavyCap;
    const int id_base = a.vocab_offset;
    const float* row = a.logits + d.logits_off;

    // ---- 1. penalty bitmap, optional write-back, row extremes
    const bool has_pen = (d.flags & kRowPenalty) != 0;
    if (has_pen) {
        const int words = (n + 31) >> 5;
        for (int i = tid; i < words; i += kFullThreads) bitmap[i] = 0u;
        __syncthreads();
        const int32_t* h = a.hist + d.hist_begin;
        for (int i = tid; i < d.hist_len; i += kFullThreads) {
            const int c = h[i] - id_base;
            if (c >= 0 && c < n) atomicOr(&bitmap[c >> 5], 1u << (c & 31));
        }
        __syncthreads();
    }
    const RowView rv{row, has_pen ? bitmap : nullptr, d.penalty, a.softcap};
    u64 cmax = 0ull, cmin = ~0ull;
    for (int i = tid; i < n; i += kFullThreads) {
        const float x = rv.at(i);
        if (x == x) {   // NaNs take no part
            const u64 c = make_comp(x, i + id_base);
            cmax = max(cmax, c);
            cmin = min(cmin, c);
        }
        if (a.write_back && (a.softcap != 0.0f || (has_pen && ((bitmap[i >> 5] >> (i & 31)) & 1u)))) const_cast<float*>(row)[i] = x;
    }
    cmax = block_max_u64(cmax, sh);
    cmin = block_min_u64(cmin, sh);
    const int out = d.out_index;
    if (cmax == 0ull) {   // nothing but NaNs
        if (tid == 0) {
            atomicOr(a.status, kStatusEmptyRow);
            a.tokens[out] = 0;
            if (a.kept_n) a.kept_n[out] = 0;
        }
        return;
    }
    const float mx = comp_value(cmax);
    // write-back changed the row under our feet: from here on read it as final
    const RowView rf = a.write_back ? RowView{row, nullptr, 1.0f, 0.0f} : rv;

    // ---- 2. the k-th candidate (k < n only)
    u64 c_k = cmin;
    U128 dummy;
    if (d.k < n) {
        if (!weight_descent(rf, n, id_base, nullptr, 0ull, U128{0ull, (u64)d.k}, cmax, cmin, sh, &c_k, &dummy)) c_k = cmin;
    }

    // ---- 3. weights of the candidates, their sum
    u64* wts = a.weights + (size_t)blockIdx.x * (size_t)n;
    U128 part{0ull, 0ull};
    unsigned cand_part = 0u;
    const double inv_t = (double)d.temperature;
    for (int i = tid; i < n; i += kFullThreads) {
        const float x = rf.at(i);
        u64 wgt = 0ull;
        if (x == x && make_comp(x, i + id_base) >= c_k) {
            const double e = exp(__ddiv_rn((double)__fsub_rn(x, mx), inv_t));
            wgt = __double2ull_rn(__dmul_rn(e, 4611686018427387904.0));   // 2^62
            ++cand_part;
        }
        wts[i] = wgt;
        const u64 lo = part.lo + wgt;
        if (lo < part.lo) part.hi += 1ull;
        part.lo = lo;
    }
    // exact 128-bit block sum: low words first (with carries), then high words
    __syncthreads();
    if (tid < 256) {
        sh->h_lo[tid] = 0ull;
        sh->h_hi[tid] = 0ull;
        sh->h_cnt[tid] = 0u;
    }
    if (tid == 0) sh->heavy_cnt = 0;
    __syncthreads();
    {
        const u64 old = atomicAdd(&sh->h_lo[0], part.lo);
        if (old + part.lo < old) atomicAdd(&sh->h_hi[0], 1ull);
        if (part.hi) atomicAdd(&sh->h_hi[0], part.hi);
        if (cand_part) atomicAdd(&sh->h_cnt[0], cand_part);
    }
    __syncthreads();
    const U128 S{sh->h_hi[0], sh->h_lo[0]};
    const int n_cand = (int)sh->h_cnt[0];
    __syncthreads();
    const double sum = __dmul_rn(u128_to_double(S), 2.168404344971008868014905601739883422851562500e-19);   // * 2^-62

    // ---- 3b. the heavy prefix: every candidate that weighs at least 2^-10 of the total (there are at most 1024 of
    // them, and in candidate order they come before every lighter one), in order, with exact cumulative weights
    int m = 0;   // length of the prefix; 0 = no shortcut (too many heavy elements cannot happen, none can: flat rows)
    if ((S.hi >> 10) == 0ull) {
        u64 thr_w = (S.hi << 54) | (S.lo >> 10);
        if (thr_w == 0ull) thr_w = 1ull;
        for (int i = tid; i < n; i += kFullThreads) {
            const u64 wgt = wts[i];
            if (wgt >= thr_w) {
                const int pos = atomicAdd(&sh->heavy_cnt, 1);
                if (pos < kHeavyCap) hv.raw[pos] = make_comp(rf.at(i), i + id_base);
            }
        }
        __syncthreads();
        m = sh->heavy_cnt <= kHeavyCap ? sh->heavy_cnt : 0;
        __syncthreads();
    }
    if (m > 0) {
        // order them: every warp sorts a run of 32 in registers, then each entry counts, by binary search, the
        // entries of the other runs above it
        const int lane = tid & 31, warp = tid >> 5, runs = (m + 31) >> 5;
        u64 c = 0ull;
        if (warp < runs) {
            c = warp_sort32_desc(tid < m ? hv.raw[tid] : 0ull);
            hv.raw[tid] = c;
        }
        __syncthreads();
        if (c != 0ull) {
            int rank = lane;
            for (int r2 = 0; r2 < runs; ++r2) {
                if (r2 == warp) continue;
                const u64* run = hv.raw + 32 * r2;
                int lo = 0;
#pragma unroll
                for (int step = 16; step > 0; step >>= 1)
                    if (run[lo + step - 1] > c) lo += step;
                if (run[lo] > c) ++lo;
                rank += lo;
            }
            hv.sorted[rank] = c;
        }
        __syncthreads();
        // weights from the values (the same formula as above), then one thread adds them up exactly
        if (tid < m) {
            const double e = exp(__ddiv_rn((double)__fsub_rn(comp_value(hv.sorted[tid]), mx), inv_t));
            hv.cum_lo[tid] = __double2ull_rn(__dmul_rn(e, 4611686018427387904.0));
        }
        __syncthreads();
        if (tid == 0) {
            U128 run{0ull, 0ull};
            for (int i = 0; i < m; ++i) {
                run = u128_add(run, U128{0ull, hv.cum_lo[i]});
                hv.cum_lo[i] = run.lo;
                hv.cum_hi[i] = run.hi;
            }
        }
        __syncthreads();
    }

    // ---- 4a. min-p: the last candidate whose probability is not below pr[0] * min_p   (pr[0] = 1 / sum)
    u64 c_keep = c_k;
    if (d.min_p > 0.0f) {
        const double thr = __dmul_rn(__ddiv_rn(1.0, sum), (double)d.min_p);
        u64 lowest = ~0ull;
        for (int i = tid; i < n; i += kFullThreads) {
            const float x = rf.at(i);
            if (!(x == x)) continue;
            const u64 c = make_comp(x, i + id_base);
            if (c < c_k) continue;
            const double e = exp(__ddiv_rn((double)__fsub_rn(x, mx), inv_t));
            if (!(__ddiv_rn(e, sum) < thr)) lowest = min(lowest, c);
        }
        lowest = block_min_u64(lowest, sh);
        if (lowest == ~0ull) lowest = cmax;   // keep at least the best
        c_keep = max(c_keep, lowest);
    }
    // ---- 4b. top-p: the first candidate at which the cumulative probability reaches top_p, included
    if (d.top_p < 1.0f) {
        const U128 target = double_to_u128_ceil(__dmul_rn(__dmul_rn((double)d.top_p, sum), 4611686018427387904.0));
        u64 c_p;
        const int ip = m > 0 ? heavy_first_reaching(hv, m, target, sh, 0) : -1;
        if (ip >= 0) c_keep = max(c_keep, hv.sorted[ip]);
        else if (weight_descent(rf, n, id_base, wts, c_k, target, cmax, cmin, sh, &c_p, &dummy)) c_keep = max(c_keep, c_p);
    }
    // ---- 4c. total weight and size of the kept set
    // (known without a pass when the kept set is the whole candidate set, or ends inside the heavy prefix)
    int keep_idx = -1;   // index of c_keep in the prefix, if it lies there
    if (m > 0 && c_keep >= hv.sorted[m - 1]) {
        if (tid == 0) sh->hit[1] = -1;
        __syncthreads();
        if (tid < m && hv.sorted[tid] == c_keep) sh->hit[1] = tid;
        __syncthreads();
        keep_idx = sh->hit[1];
        __syncthreads();
    }
    const bool keep_all = c_keep == c_k;
    U128 kept_w{0ull, 0ull};
    unsigned kept_cnt = 0u;
    for (int i = tid; i < ((keep_all || keep_idx >= 0) ? 0 : n); i += kFullThreads) {
        const float x = rf.at(i);
        if (x == x && make_comp(x, i + id_base) >= c_keep) {
            const u64 lo = kept_w.lo + wts[i];
            if (lo < kept_w.lo) kept_w.hi += 1ull;
            kept_w.lo = lo;
            ++kept_cnt;
        }
    }
    if (tid < 256) {
        sh->h_lo[tid] = 0ull;
        sh->h_hi[tid] = 0ull;
        sh->h_cnt[tid] = 0u;
    }
    __syncthreads();
    {
        const u64 old = atomicAdd(&sh->h_lo[0], kept_w.lo);
        if (old + kept_w.lo < old) atomicAdd(&sh->h_hi[0], 1ull);
        if (kept_w.hi) atomicAdd(&sh->h_hi[0], kept_w.hi);
        atomicAdd(&sh->h_cnt[0], kept_cnt);
    }
    __syncthreads();
    const U128 KW = keep_idx >= 0 ? U128{hv.cum_hi[keep_idx], hv.cum_lo[keep_idx]} : keep_all ? S : U128{sh->h_hi[0], sh->h_lo[0]};
    const int n_keep = keep_idx >= 0 ? keep_idx + 1 : keep_all ? n_cand : (int)sh->h_cnt[0];
    __syncthreads();
    // ---- 4d. the draw: first kept candidate whose cumulative weight reaches u * (kept weight)
    double u = __dmul_rn(__ull2double_rn(d.rng_word), 5.42101086242752217003726400434970855712890625e-20);   // 2^-64
    if (u >= 1.0) u = __longlong_as_double(0x3FEFFFFFFFFFFFFFll);
    const U128 target = double_to_u128_ceil(__dmul_rn(u, u128_to_double(KW)));
    u64 c_tok;
    const int it = m > 0 ? heavy_first_reaching(hv, m, target, sh, 0) : -1;
    if (it >= 0) c_tok = max(hv.sorted[it], c_keep);
    else if (!weight_descent(rf, n, id_base, wts, c_keep, target, cmax, cmin, sh, &c_tok, &dummy) || c_tok < c_keep) c_tok = c_keep;
    if (tid == 0) {
        a.tokens[out] = comp_id(c_tok);
        if (a.kept_n) {
            a.kept_n[out] = n_keep;
            a.kept_ids[(size_t)out * kMaxK] = comp_id(c_keep);
            a.kept_pr[(size_t)out * kMaxK] = __ddiv_rn(u128_to_double(KW), u128_to_double(S));
        }
    }
}

}  // namespace

size_t full_row_smem_bytes(int n_vocab) {
    const size_t bitmap = (sizeof(unsigned) * (size_t)((n_vocab + 31) / 32) + 15) & ~(size_t)15;
    return sizeof(FullShared) + bitmap + 4 * sizeof(u64) * (size_t)kHeavyCap;
}

int prepare_full_row_kernel(int max_vocab) {
    return (int)cudaFuncSetAttribute(full_row_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)full_row_smem_bytes(max_vocab));
}

int launch_full_row_kernel(const float* logits, const RowDesc* rows, int n_rows, const int32_t* hist, uint64_t* weights, int32_t* tokens,
                           int32_t* kept_ids, double* kept_pr, int32_t* kept_n, uint32_t* status, int n_vocab, int vocab_offset,
                           int write_back, float softcap, void* stream) {
    FullArgs a{};
    a.logits = logits;
    a.rows = rows;
    a.hist = hist;
    a.weights = reinterpret_cast<u64*>(weights);
    a.tokens = tokens;
    a.kept_ids = kept_ids;
    a.kept_pr = kept_pr;
    a.kept_n = kept_n;
    a.status = status;
    a.n_vocab = n_vocab;
    a.vocab_offset = vocab_offset;
    a.write_back = write_back;
    a.softcap = softcap;
    full_row_kernel<<<n_rows, kFullThreads, full_row_smem_bytes(n_vocab), static_cast<cudaStream_t>(stream)>>>(a);
    return (int)cudaGetLastError();
}

}  // namespace fsb
