// fsb_fullrow.cu - the full-vocabulary kernel of the B200 batched token sampler (sm_100a).
//
// Rows whose effective candidate count k exceeds kMaxK - above all `top_k == 0`, where the reference sorts the
// whole vocabulary (src/sampler.cpp:32-35 of paragontasx/ferro) - cannot keep their candidates in one CTA.  A
// cluster of kFullCluster CTAs works on one such row.  Every CTA keeps its slice of the row in shared memory
// (softcap and penalty applied once, src/model_gemma4.cpp:521 and src/sampler.cpp:11-18), so the row is read from
// HBM exactly once; everything after that reads shared memory:
//   1. the row's largest and smallest candidate key                                            (src/sampler.cpp:38)
//   2. if k < n: the k-th candidate, by a radix descent over the keys that counts                      (:27-31)
//   3. the weights e_i = exp((double)(x_i - max) / T) of the candidates as 2^-62 fixed point, histogrammed by the
//      leading digit of their keys; the sum of the histogram is the softmax denominator                    (:40-41)
//   4. min-p bound (:43), top-p crossing (:44) and the draw (:45-49) by radix descents over accumulated weight.
// A descent is MSB-first over 8-bit digits of the 64-bit candidate key.  At every level each CTA histograms the
// candidates of its slice that match the prefix found so far (count and weight per digit), all CTAs of the
// cluster read all histograms through distributed shared memory and walk the digits - each CTA does the same
// integer arithmetic, so all arrive at the same digit without a broadcast - and the descent stops as soon as the
// digit it lands on holds a single candidate.  Weights are recomputed from the values where they are needed
// (the function is pure), never stored.  Sums of weights are integers, so they do not depend on the order in
// which threads add: the result is deterministic and differs from the reference's sequential fp64 sums by
// rounding only (~1e-13).
#include <cuda_runtime.h>

#include <algorithm>

#include "fsb_device.cuh"

namespace fsb {
namespace {

constexpr int kFullThreads = 1024;
constexpr int kFullWarps = kFullThreads / 32;
static_assert(kFullWarps == 32, "the block reductions read one partial per lane");
constexpr int kFullCluster = 8;                 // CTAs per row
constexpr int kSliceCache = 32768;              // logits of a slice that are kept in shared memory (rows up to 8 x this)
constexpr int kStripes = 8;                     // copies of the level histogram (by warp): fewer warps hit one word at once
constexpr int kLimbs = 4;                       // a weight is added to a histogram as four 16-bit limbs (32-bit native atomics)

struct U128 {
    u64 hi, lo;
};
__device__ __forceinline__ U128 u128_add(U128 a, U128 b) {
    U128 r;
    r.lo = a.lo + b.lo;
    r.hi = a.hi + b.hi + (r.lo < a.lo ? 1ull : 0ull);
    return r;
}
__device__ __forceinline__ U128 u128_sub(U128 a, U128 b) {
    U128 r;
    r.lo = a.lo - b.lo;
    r.hi = a.hi - b.hi - (a.lo < b.lo ? 1ull : 0ull);
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

// ---- the cluster ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The cluster's barrier: arrive releases this thread's shared-memory writes to the cluster, wait acquires the others'.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of a shared-memory location of CTA `rank` of the cluster, and loads from there.
__device__ __forceinline__ unsigned map_to_rank(const void* p, unsigned rank) {
    unsigned a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_u32(p)), "r"(rank));
    return a;
}
__device__ __forceinline__ u64 ld_cluster_u64(unsigned addr) {
    u64 v;
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ unsigned ld_cluster_u32(unsigned addr) {
    unsigned v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}

// ---- shared memory of a CTA -------------------------------------------------------------------------------------------
struct FullShared {
    // the level histogram being built (kStripes copies), then this CTA's sum of them, which the other CTAs read
    // [stripe][limb 0..3, then the candidate count][digit], four words of padding between stripes: a limb sum stays
    // below 2^32 while a stripe sees fewer than 65537 candidates, i.e. for rows of up to 4 M logits
    alignas(16) unsigned h[kStripes][(kLimbs + 1) * 256 + 4];
    u64 x_lo[2][256];          // double buffered by level: a CTA may build the next level while others still read this one
    u64 x_hi[2][256];
    unsigned x_cnt[2][256];
    u64 x_small[2][4];         // small values exchanged across the cluster (extremes, sums), double buffered by use
    u64 x_all[2][kFullCluster * 4];   // ... and every CTA's copy of all of them
    // the cluster-wide histogram of the first weighted level: the descents of step 4 all start from it
    u64 l1_lo[256];
    u64 l1_hi[256];
    unsigned l1_cnt[256];
    // suffix sums of the walk
    u64 w_lo[8], w_hi[8];
    unsigned w_cnt[8];
    int res_digit;
    unsigned res_cnt;          // candidates in the chosen digit
    unsigned res_above_cnt;    // candidates before it
    u64 res_above_lo, res_above_hi;
    u64 tot_lo, tot_hi;        // weight and number of all candidates of the level just walked (before-weight included)
    unsigned tot_cnt;
    u64 red[kFullWarps];
    u64 red_hi[kFullWarps];
    unsigned red_cnt[kFullWarps];
    int pick;                  // index of the drawn candidate in the ordered kept set
};

struct FullArgs {
    const float* logits;
    const RowDesc* rows;      // the rows of this kernel
    const int32_t* hist;
    int32_t* tokens;
    int32_t* tokens_host;     // mirror of the tokens in mapped host memory, or null
    unsigned* status_host;    // takes a non-zero word whenever a status bit is set, or null
    int32_t* kept_ids;        // [rows][kMaxK]
    double* kept_pr;          // [rows][kMaxK]; also the staging of the kept set's first candidates while they are gathered
    int32_t* kept_n;
    unsigned* status;
    int32_t n_vocab;
    int32_t vocab_offset;
    int32_t write_back;
    int32_t record;           // the caller wants the kept sets (their memory is used as a staging area either way)
    float softcap;
    u64* trace;               // diagnostics: time stamps of the last row's phases, or null
};

// What the passes of a row share.
struct RowCtx {
    const float* vals;        // the slice in shared memory (as the sampler sees it), or null: read and transform the row
    const float* row;         // the row in global memory
    const unsigned* bitmap;   // penalised columns of the slice (bit i = column lo + i), or null
    float pen, cap;
    int lo, n;                // first column and number of columns of this CTA's slice
    int id_base;              // token id of column 0
    float mx;                 // the row's maximum
    double temp;
    u64* dbg;                 // diagnostics
    __device__ __forceinline__ float at(int i) const {   // logit i of the slice as the sampler sees it
        if (vals) return vals[i];
        float x = row[lo + i];
        if (cap != 0.0f) x = __fmul_rn(cap, tanhf(__fdiv_rn(x, cap)));
        if (bitmap && ((bitmap[i >> 5] >> (i & 31)) & 1u)) x = x > 0.0f ? __fdiv_rn(x, pen) : __fmul_rn(x, pen);
        return x;
    }
    __device__ __forceinline__ u64 comp(float x, int i) const { return make_comp(x, lo + i + id_base); }
    __device__ __forceinline__ u64 weight(float x) const {   // src/sampler.cpp:40, as 2^-62 fixed point
        const double e = exp(__ddiv_rn((double)__fsub_rn(x, mx), temp));
        return __double2ull_rn(__dmul_rn(e, 4611686018427387904.0));
    }
};

__device__ __forceinline__ u64 block_max_u64(u64 v, FullShared* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (lane == 0) sh->red[warp] = v;
    __syncthreads();
    u64 r = sh->red[lane];   // kFullWarps == 32: one partial per lane
#pragma unroll
    for (int o = 16; o; o >>= 1) r = max(r, __shfl_xor_sync(0xffffffffu, r, o));
    __syncthreads();
    return r;
}

// Largest `hi` and smallest `lo` over the CTA in one go.
__device__ __forceinline__ void block_max2_u64(u64& hi, u64& lo, FullShared* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    u64 a = hi, b = ~lo;
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        a = max(a, __shfl_xor_sync(0xffffffffu, a, o));
        b = max(b, __shfl_xor_sync(0xffffffffu, b, o));
    }
    if (lane == 0) {
        sh->red[warp] = a;
        sh->red_hi[warp] = b;
    }
    __syncthreads();
    a = sh->red[lane];
    b = sh->red_hi[lane];
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        a = max(a, __shfl_xor_sync(0xffffffffu, a, o));
        b = max(b, __shfl_xor_sync(0xffffffffu, b, o));
    }
    __syncthreads();
    hi = a;
    lo = ~b;
}

// Exchanges up to four 64-bit values per CTA across the cluster: every CTA gets all kFullCluster x 4 values.
// `use` alternates 0/1 between consecutive exchanges.  Contains one cluster barrier.
__device__ __forceinline__ void cluster_exchange(FullShared* sh, int use, const u64 (&mine)[4], u64 (&all)[kFullCluster][4]) {
    if (threadIdx.x < 4) sh->x_small[use][threadIdx.x] = mine[threadIdx.x];
    cluster_sync_all();
    // one warp fetches the remote words; everybody else reads the local copy
    if (threadIdx.x < kFullCluster * 4)
        sh->x_all[use][threadIdx.x] = ld_cluster_u64(map_to_rank(&sh->x_small[use][threadIdx.x & 3], threadIdx.x >> 2));
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kFullCluster; ++r)
#pragma unroll
        for (int j = 0; j < 4; ++j) all[r][j] = sh->x_all[use][r * 4 + j];
}

// Exact sum of one 128-bit value and one count per thread over the CTA.
__device__ __forceinline__ void block_sum_u128(U128& v, unsigned& cnt, FullShared* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const u64 l = __shfl_xor_sync(0xffffffffu, v.lo, o);
        const u64 h = __shfl_xor_sync(0xffffffffu, v.hi, o);
        cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
        v = u128_add(v, U128{h, l});
    }
    if (lane == 0) {
        sh->red[warp] = v.lo;
        sh->red_hi[warp] = v.hi;
        sh->red_cnt[warp] = cnt;
    }
    __syncthreads();
    v = U128{0ull, 0ull};
    cnt = 0u;
    for (int w = 0; w < kFullWarps; ++w) {
        v = u128_add(v, U128{sh->red_hi[w], sh->red[w]});
        cnt += sh->red_cnt[w];
    }
    __syncthreads();
}

// Adds (digit, weight, one candidate) to the level histogram: native 32-bit shared-memory atomics on the count and on
// the weight's non-zero 16-bit limbs.  The lanes of a warp spread over the stripes, and the stripes start in
// different banks, so that lanes with the same digit seldom meet in one word.
__device__ __forceinline__ void hist_add(FullShared* sh, bool active, int digit, u64 weight, bool weighted, unsigned stripe_mask) {
    if (!active) return;
    unsigned* h = &sh->h[threadIdx.x & stripe_mask][digit];
    atomicAdd(h + kLimbs * 256, 1u);
    if (weighted) {
        const unsigned l0 = (unsigned)(weight & 0xFFFFull), l1 = (unsigned)((weight >> 16) & 0xFFFFull);
        const unsigned l2 = (unsigned)((weight >> 32) & 0xFFFFull), l3 = (unsigned)(weight >> 48);
        if (l0) atomicAdd(h, l0);
        if (l1) atomicAdd(h + 256, l1);
        if (l2) atomicAdd(h + 512, l2);
        if (l3) atomicAdd(h + 768, l3);
    }
}

// What a descent found: the candidate at which the accumulated weight (or count) reaches the target, the weight and
// the number of candidates strictly before it, and whether there was such a candidate at all.
struct Crossing {
    u64 c;
    U128 above;
    unsigned above_cnt;
    bool found;
};

// One level's histogram of this CTA (the stripes added up) goes to the exchange buffer `par`; after the cluster's
// barrier every CTA adds up all CTAs' histograms (thread d < 256 owns digit d) and walks the digits from the top:
// the crossing digit is the highest digit d that holds a candidate and whose suffix sum (the weight of all higher
// digits and its own, plus `above`) reaches the target.  Leaves digit, its candidate count and the weight and count
// before it in shared memory; digit -1 if the target is beyond all candidates.  If `keep_l1`, the cluster-wide
// histogram is also stored for later descents.  All threads of all CTAs of the cluster must call.
__device__ __forceinline__ void level_reduce_and_walk(FullShared* sh, int par, U128 target, U128 above, unsigned above_cnt, bool by_count,
                                                      bool keep_l1, bool from_l1, unsigned stripe_mask) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    u64 lo = 0ull, hi = 0ull;
    unsigned cnt = 0u;
    if (from_l1) {
        if (tid < 256) {
            lo = sh->l1_lo[tid];
            hi = sh->l1_hi[tid];
            cnt = sh->l1_cnt[tid];
        }
    } else {
        if (tid < 256) {
            u64 l0 = 0ull, l1 = 0ull, l2 = 0ull, l3 = 0ull;   // limb sums over the stripes: below 2^35 each
            unsigned c = 0u;
#pragma unroll
            for (int s = 0; s <= (int)stripe_mask; ++s) {
                l0 += sh->h[s][tid];
                l1 += sh->h[s][256 + tid];
                l2 += sh->h[s][512 + tid];
                l3 += sh->h[s][768 + tid];
                c += sh->h[s][kLimbs * 256 + tid];
            }
            U128 acc{0ull, l0};
            acc = u128_add(acc, U128{l1 >> 48, l1 << 16});
            acc = u128_add(acc, U128{l2 >> 32, l2 << 32});
            acc = u128_add(acc, U128{l3 >> 16, l3 << 48});
            sh->x_lo[par][tid] = acc.lo;
            sh->x_hi[par][tid] = acc.hi;
            sh->x_cnt[par][tid] = c;
        }
        cluster_sync_all();
        if (tid < 256) {
#pragma unroll
            for (unsigned r = 0; r < (unsigned)kFullCluster; ++r) {
                const u64 l = ld_cluster_u64(map_to_rank(&sh->x_lo[par][tid], r));
                const u64 h = ld_cluster_u64(map_to_rank(&sh->x_hi[par][tid], r));
                const unsigned c = ld_cluster_u32(map_to_rank(&sh->x_cnt[par][tid], r));
                lo += l;
                hi += h + (lo < l ? 1ull : 0ull);
                cnt += c;
            }
            if (keep_l1) {
                sh->l1_lo[tid] = lo;
                sh->l1_hi[tid] = hi;
                sh->l1_cnt[tid] = cnt;
            }
        }
    }
    if (by_count) {   // the "weight" of a digit is its number of candidates
        lo = cnt;
        hi = 0ull;
    }
    // suffix sums over the digits: within a warp (digits warp * 32 .. + 31), then the warps above
    U128 suf{hi, lo};
    unsigned sufc = cnt;
    if (tid < 256) {
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const u64 l = __shfl_down_sync(0xffffffffu, suf.lo, o);
            const u64 h = __shfl_down_sync(0xffffffffu, suf.hi, o);
            const unsigned c = __shfl_down_sync(0xffffffffu, sufc, o);
            if (lane + o < 32) {
                suf = u128_add(suf, U128{h, l});
                sufc += c;
            }
        }
        if (lane == 0) {
            sh->w_lo[warp] = suf.lo;
            sh->w_hi[warp] = suf.hi;
            sh->w_cnt[warp] = sufc;
        }
    }
    if (tid == 0) sh->res_digit = -1;
    __syncthreads();
    U128 with{0ull, 0ull};
    unsigned with_c = 0u;
    if (tid < 256) {
        U128 higher = above;
        unsigned higher_c = above_cnt;
        for (int w = warp + 1; w < 8; ++w) {
            higher = u128_add(higher, U128{sh->w_hi[w], sh->w_lo[w]});
            higher_c += sh->w_cnt[w];
        }
        with = u128_add(suf, higher);        // everything from this digit up, and what came before the level
        with_c = sufc + higher_c;
        if (cnt != 0u && u128_ge(with, target)) atomicMax(&sh->res_digit, tid);   // the highest digit that reaches wins
        if (tid == 0) {   // digit 0's suffix is everything
            sh->tot_lo = with.lo;
            sh->tot_hi = with.hi;
            sh->tot_cnt = with_c;
        }
    }
    __syncthreads();
    if (tid < 256 && tid == sh->res_digit) {
        const U128 before = u128_sub(with, U128{hi, lo});
        sh->res_above_lo = before.lo;
        sh->res_above_hi = before.hi;
        sh->res_above_cnt = with_c - cnt;
        sh->res_cnt = cnt;
    }
    __syncthreads();
}

// Radix descent over the candidates with composite in [floor_c, top_c] (the extremes of the candidate set): finds
// the candidate at which the accumulated weight - or, with by_count, the number of candidates - counted from the
// largest candidate down reaches `target`.  With use_l1 the first level is the stored histogram (the caller
// guarantees it was built over the same candidate set with the same extremes).  All threads of the cluster call.
__device__ Crossing cluster_descent(const RowCtx& rc, FullShared* sh, u64 floor_c, u64 top_c, U128 target, bool by_count, bool use_l1,
                                    bool build_l1, int& par) {
    const int tid = threadIdx.x;
    Crossing out{0ull, U128{0ull, 0ull}, 0u, false};
    u64 mask, pfx;
    int hb;
    if (top_c != floor_c) {
        const int hb0 = 63 - __clzll((long long)(top_c ^ floor_c));
        mask = (hb0 == 63) ? 0ull : (~0ull << (hb0 + 1));
        pfx = top_c & mask;
        hb = hb0;
    } else {
        mask = ~0ull;
        pfx = top_c;
        hb = -1;
    }
    U128 above{0ull, 0ull};
    unsigned above_cnt = 0u;
    bool first = true;
    while (hb >= 0) {
        const int w = hb + 1 < 8 ? hb + 1 : 8, lo = hb + 1 - w;
        const unsigned dmask = (1u << w) - 1u;
        const bool from_l1 = first && use_l1;
        // the first level sees every candidate, a few digits take most of them: eight stripes keep the lanes of a warp
        // apart.  Deeper levels see the few candidates that match the prefix: one stripe, an eighth of the clearing
        // and adding up.
        // (a 16-bit limb summed over one stripe stays below 2^32 for slices of up to 65536 logits)
        const unsigned stripe_mask = (first || rc.n > 65536) ? (unsigned)(kStripes - 1) : 0u;
        const bool dbg = rc.dbg && build_l1;
        if (dbg) rc.dbg[16] = global_timer_ns();
        if (!from_l1) {
            for (int i = tid; i < (int)((stripe_mask + 1u) * sizeof(sh->h[0]) / sizeof(uint4)); i += kFullThreads)
                reinterpret_cast<uint4*>(&sh->h[0][0])[i] = make_uint4(0u, 0u, 0u, 0u);
            __syncthreads();
            if (dbg) rc.dbg[17] = global_timer_ns();
            const int n_iter = (rc.n + kFullThreads - 1) / kFullThreads;
            for (int it = 0; it < n_iter; ++it) {
                const int i = it * kFullThreads + tid;
                bool active = false;
                int digit = 0;
                u64 wgt = 0ull;
                if (i < rc.n) {
                    const float x = rc.at(i);
                    if (x == x) {   // NaNs take no part
                        const u64 c = rc.comp(x, i);
                        if (c >= floor_c && (c & mask) == pfx) {
                            active = true;
                            digit = (int)((unsigned)(c >> lo) & dmask);
                            if (!by_count) wgt = rc.weight(x);
                        }
                    }
                }
                hist_add(sh, active, digit, wgt, !by_count, stripe_mask);
            }
            __syncthreads();
            if (dbg) rc.dbg[18] = global_timer_ns();
        }
        level_reduce_and_walk(sh, par, target, above, above_cnt, by_count, first && build_l1, from_l1, stripe_mask);
        if (dbg) rc.dbg[19] = global_timer_ns();
        if (!from_l1) par ^= 1;
        first = false;
        const int d = sh->res_digit;
        const unsigned in_digit = sh->res_cnt;
        const U128 nabove{sh->res_above_hi, sh->res_above_lo};
        const unsigned nabove_cnt = sh->res_above_cnt;
        __syncthreads();   // the results may be overwritten
        if (d < 0) return out;   // the target lies beyond the candidates
        pfx |= (u64)(unsigned)d << lo;
        mask |= (u64)dmask << lo;
        above = nabove;
        above_cnt = nabove_cnt;
        hb = lo - 1;
        if (in_digit == 1u && hb >= 0) break;   // a single candidate matches the prefix: no need to resolve its other bits
    }
    if (hb >= 0) {
        // the single candidate that matches the prefix, wherever it lies: its owner finds it, the cluster takes the maximum
        u64 mine = 0ull;
        for (int i = tid; i < rc.n; i += kFullThreads) {
            const float x = rc.at(i);
            if (x == x) {
                const u64 c = rc.comp(x, i);
                if (c >= floor_c && (c & mask) == pfx) mine = c;
            }
        }
        // exactly one thread of the cluster holds it: that thread tells every CTA, one barrier makes it visible
        if (mine != 0ull) {
#pragma unroll
            for (unsigned r = 0; r < (unsigned)kFullCluster; ++r) cluster_store_u64(map_to_rank(&sh->x_small[par][0], r), mine);
        }
        cluster_sync_all();
        pfx = sh->x_small[par][0];
        par ^= 1;
    }
    out.c = pfx;
    out.above = above;
    out.above_cnt = above_cnt;
    out.found = true;
    return out;
}

__global__ void __launch_bounds__(kFullThreads, 1) full_row_kernel(const FullArgs a, int cache_slice) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    FullShared* sh = reinterpret_cast<FullShared*>(smem_raw);
    const int tid = threadIdx.x;
    const unsigned rank = cluster_rank();
    const RowDesc d = a.rows[blockIdx.x / kFullCluster];
    const int V = a.n_vocab;
    // the slices: equal runs of columns, a multiple of four each
    const int per = (((V + kFullCluster - 1) / kFullCluster) + 3) & ~3;
    const int lo = min(V, (int)rank * per), n = min(V, lo + per) - lo;
    unsigned* bitmap = reinterpret_cast<unsigned*>(smem_raw + sizeof(FullShared));
    float* vals = reinterpret_cast<float*>(smem_raw + sizeof(FullShared) + (size_t)((per + 31) / 32) * sizeof(unsigned));
    vals = reinterpret_cast<float*>(((uintptr_t)vals + 15) & ~(uintptr_t)15);
    const float* row = a.logits + d.logits_off;
    const int id_base = a.vocab_offset;
    int par = 0;
#define FTR(n)                                                                                                      \
    do {                                                                                                            \
        if (a.trace && blockIdx.x == gridDim.x - kFullCluster && tid == 0) a.trace[(n)] = global_timer_ns();        \
    } while (0)
    FTR(0);

    // ---- 0. the slice as the sampler sees it: penalty bitmap, softcap, penalty, optional write-back
    const bool has_pen = (d.flags & kRowPenalty) != 0;
    if (has_pen) {
        const int words = (n + 31) >> 5;
        for (int i = tid; i < words; i += kFullThreads) bitmap[i] = 0u;
        __syncthreads();
        const int32_t* h = a.hist + d.hist_begin;
        for (int i = tid; i < d.hist_len; i += kFullThreads) {
            const int c = h[i] - id_base - lo;
            if (c >= 0 && c < n) atomicOr(&bitmap[c >> 5], 1u << (c & 31));
        }
        __syncthreads();
    }
    RowCtx rc{nullptr, row, has_pen ? bitmap : nullptr, d.penalty, a.softcap, lo, n, id_base, 0.0f, (double)d.temperature,
              (a.trace && blockIdx.x == gridDim.x - kFullCluster && tid == 0) ? a.trace : nullptr};
    u64 cmax = 0ull, cmin = ~0ull;
    auto take = [&](float x, int i) {   // logit i of the slice as loaded: transform, keep, note the extremes, write back
        const bool hit = has_pen && ((bitmap[i >> 5] >> (i & 31)) & 1u);
        if (a.softcap != 0.0f) x = __fmul_rn(a.softcap, tanhf(__fdiv_rn(x, a.softcap)));
        if (hit) x = x > 0.0f ? __fdiv_rn(x, d.penalty) : __fmul_rn(x, d.penalty);
        if (cache_slice) vals[i] = x;
        if (x == x) {   // NaNs take no part
            const u64 c = rc.comp(x, i);
            cmax = max(cmax, c);
            cmin = min(cmin, c);
        }
        if (a.write_back && (a.softcap != 0.0f || hit)) const_cast<float*>(row)[lo + i] = x;
    };
    if (((reinterpret_cast<uintptr_t>(row + lo) & 15u) == 0) && (n & 3) == 0) {
        // 16-byte loads, four of them in flight per thread (the stores of a write-back come after the loads of a round)
        const float4* src = reinterpret_cast<const float4*>(row + lo);
        const int n4 = n >> 2;
        for (int i0 = 0; i0 < n4; i0 += 4 * kFullThreads) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * kFullThreads + tid;
                v[u] = i < n4 ? __ldcs(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * kFullThreads + tid;
                if (i < n4) {
                    take(v[u].x, 4 * i);
                    take(v[u].y, 4 * i + 1);
                    take(v[u].z, 4 * i + 2);
                    take(v[u].w, 4 * i + 3);
                }
            }
        }
    } else {
        for (int i = tid; i < n; i += kFullThreads) take(row[lo + i], i);
    }
    __syncthreads();
    if (cache_slice) {
        rc.vals = vals;
    } else if (a.write_back) {   // the row in memory now holds the transformed values: read it as final
        rc.bitmap = nullptr;
        rc.cap = 0.0f;
    }
    FTR(1);
    // ---- 1. the row's extremes
    block_max2_u64(cmax, cmin, sh);
    {
        u64 v[4] = {cmax, ~cmin, 0ull, 0ull}, all[kFullCluster][4];
        cluster_exchange(sh, par, v, all);
        par ^= 1;
        for (int r = 0; r < kFullCluster; ++r) {
            cmax = max(cmax, all[r][0]);
            cmin = min(cmin, ~all[r][1]);
        }
    }
    const int out = d.out_index;
    if (cmax == 0ull) {   // nothing but NaNs
        if (rank == 0 && tid == 0) {
            report_status(a.status, a.status_host, kStatusEmptyRow);
            put_token(a.tokens, a.tokens_host, out, 0);
            a.kept_n[out] = 0;
        }
        cluster_sync_all();   // no CTA leaves while another may still read its shared memory
        return;
    }
    rc.mx = comp_value(cmax);
    FTR(2);

    // ---- 2. the k-th candidate (k < n only)
    u64 c_k = cmin;
    if (d.k < V) {
        const Crossing ck = cluster_descent(rc, sh, 0ull, cmax, U128{0ull, (u64)d.k}, true, false, false, par);
        if (ck.found) c_k = max(cmin, ck.c);
    }

    FTR(3);
    // ---- 3. the weights' histogram by leading digit (kept for the descents), their sum and the number of candidates
    // (a descent towards an unreachable target builds the first level and stops there)
    cluster_descent(rc, sh, c_k, cmax, U128{~0ull, ~0ull}, false, false, true, par);
    U128 S{0ull, 0ull};
    unsigned n_cand = 0u;
    const bool have_l1 = cmax != c_k;
    if (have_l1) {   // the walk left the level's totals behind
        S = U128{sh->tot_hi, sh->tot_lo};
        n_cand = sh->tot_cnt;
        __syncthreads();
    } else {   // a single candidate: there was no level to build
        S = U128{0ull, rc.weight(rc.mx)};
        n_cand = 1u;
    }
    const double sum = __dmul_rn(u128_to_double(S), 2.168404344971008868014905601739883422851562500e-19);   // * 2^-62

    FTR(4);
    // ---- 4a. min-p: the last candidate whose probability is not below pr[0] * min_p   (pr[0] = 1 / sum)
    u64 c_keep = c_k;
    if (d.min_p > 0.0f) {
        const double thr = __dmul_rn(__ddiv_rn(1.0, sum), (double)d.min_p);
        // the test below is monotone in the logit and flips near mx + T * ln(min_p): only logits within a band around
        // that value need the exact arithmetic, those above it are kept, those below it are not
        const double x_flip = (double)rc.mx + rc.temp * log((double)d.min_p);
        const double band = 1e-3 * (fabs(x_flip) + rc.temp + 1.0);
        const float x_sure = (float)(x_flip + band), x_never = (float)(x_flip - band);
        u64 lowest = ~0ull;
        for (int i = tid; i < n; i += kFullThreads) {
            const float x = rc.at(i);
            if (!(x == x) || x < x_never) continue;
            const u64 c = rc.comp(x, i);
            if (c < c_k) continue;
            if (x > x_sure) {
                lowest = min(lowest, c);
                continue;
            }
            const double e = exp(__ddiv_rn((double)__fsub_rn(x, rc.mx), rc.temp));
            if (!(__ddiv_rn(e, sum) < thr)) lowest = min(lowest, c);
        }
        lowest = ~block_max_u64(~lowest, sh);
        u64 v[4] = {~lowest, 0ull, 0ull, 0ull}, all[kFullCluster][4];
        cluster_exchange(sh, par, v, all);
        par ^= 1;
        for (int r = 0; r < kFullCluster; ++r) lowest = min(lowest, ~all[r][0]);
        if (lowest == ~0ull) lowest = cmax;   // keep at least the best
        c_keep = max(c_keep, lowest);
    }
    FTR(5);
    // ---- 4b. top-p: the first candidate at which the cumulative probability reaches top_p, included
    bool keep_from_top_p = false;
    Crossing cp{0ull, U128{0ull, 0ull}, 0u, false};
    if (d.top_p < 1.0f) {
        const U128 target = double_to_u128_ceil(__dmul_rn(__dmul_rn((double)d.top_p, sum), 4611686018427387904.0));
        cp = cluster_descent(rc, sh, c_k, cmax, target, false, have_l1, false, par);
        if (cp.found && cp.c >= c_keep) {
            c_keep = cp.c;
            keep_from_top_p = true;
        }
    }
    FTR(6);
    // ---- 4c. total weight and size of the kept set: known from the descent when top-p made the cut, the whole
    // candidate set when nothing cut, otherwise one pass
    U128 KW = S;
    unsigned n_keep = n_cand;
    if (keep_from_top_p) {
        KW = u128_add(cp.above, U128{0ull, rc.weight(comp_value(cp.c))});
        n_keep = cp.above_cnt + 1u;
    } else if (c_keep != c_k) {
        U128 part{0ull, 0ull};
        unsigned pc = 0u;
        for (int i = tid; i < n; i += kFullThreads) {
            const float x = rc.at(i);
            if (x == x && rc.comp(x, i) >= c_keep) {
                const u64 w = rc.weight(x);
                const u64 l = part.lo + w;
                if (l < part.lo) part.hi += 1ull;
                part.lo = l;
                ++pc;
            }
        }
        block_sum_u128(part, pc, sh);
        u64 v[4] = {part.lo, part.hi, (u64)pc, 0ull}, all[kFullCluster][4];
        cluster_exchange(sh, par, v, all);
        par ^= 1;
        KW = U128{0ull, 0ull};
        n_keep = 0u;
        for (int r = 0; r < kFullCluster; ++r) {
            KW = u128_add(KW, U128{all[r][1], all[r][0]});
            n_keep += (unsigned)all[r][2];
        }
    }
    FTR(7);
    // ---- 4d. the draw: first kept candidate whose cumulative weight reaches u * (kept weight).  A kept set that fits
    // the record is gathered for it anyway, and the first CTA then draws from the ordered list; otherwise a descent.
    double u = __dmul_rn(__ull2double_rn(d.rng_word), 5.42101086242752217003726400434970855712890625e-20);   // 2^-64
    if (u >= 1.0) u = __longlong_as_double(0x3FEFFFFFFFFFFFFFll);
    const U128 target = double_to_u128_ceil(__dmul_rn(u, u128_to_double(KW)));
    const bool draw_from_list = n_keep <= (unsigned)kMaxK;
    if (!draw_from_list) {
        const Crossing ct = cluster_descent(rc, sh, c_k, cmax, target, false, have_l1, false, par);
        const u64 c_tok = (ct.found && ct.c >= c_keep) ? ct.c : c_keep;
        if (rank == 0 && tid == 0) put_token(a.tokens, a.tokens_host, out, comp_id(c_tok));
    }
    FTR(8);

    // ---- 5. the kept set's record: its size, and its first kMaxK candidates in order with their probabilities
    if (a.record || draw_from_list) {
        const int want = (int)min(n_keep, (unsigned)kMaxK);
        u64 c_first = c_keep;   // the last of the first `want` kept candidates
        if ((unsigned)want < n_keep) {
            const Crossing cf = cluster_descent(rc, sh, c_k, cmax, U128{0ull, (u64)want}, true, false, false, par);
            if (cf.found) c_first = max(c_keep, cf.c);
        }
        // every CTA appends its candidates >= c_first to the row's staging area (the probabilities' memory, as keys);
        // the kept-set size doubles as the fill counter until the first CTA has ordered them
        u64* stage = reinterpret_cast<u64*>(a.kept_pr + (size_t)out * kMaxK);
        if (rank == 0 && tid == 0) a.kept_n[out] = 0;
        __threadfence();
        cluster_sync_all();
        for (int i = tid; i < n; i += kFullThreads) {
            const float x = rc.at(i);
            if (x == x) {
                const u64 c = rc.comp(x, i);
                if (c >= c_first) {
                    const int p = atomicAdd(&a.kept_n[out], 1);
                    if (p < kMaxK) stage[p] = c;
                }
            }
        }
        __threadfence();
        cluster_sync_all();
        if (rank == 0) {
            // the first CTA's slice is no longer needed: the candidates, then (by rank) their ids' composites and weights
            u64* srt = reinterpret_cast<u64*>(vals);
            u64* by_rank_c = srt + kMaxK;
            u64* by_rank_w = srt + 2 * kMaxK;
            u64 c = 0ull;
            if (tid < want) c = __ldcg(stage + tid);
            __syncthreads();
            if (tid < want) srt[tid] = c;
            if (tid == 0) sh->pick = want - 1;   // a target beyond the list (rounding) takes the last kept candidate
            __syncthreads();
            if (tid < want) {
                int rank_in = 0;
                for (int j = 0; j < want; ++j) rank_in += srt[j] > c ? 1 : 0;
                const float x = comp_value(c);
                const double e = exp(__ddiv_rn((double)__fsub_rn(x, rc.mx), rc.temp));
                a.kept_ids[(size_t)out * kMaxK + rank_in] = comp_id(c);
                a.kept_pr[(size_t)out * kMaxK + rank_in] = __ddiv_rn(e, sum);
                by_rank_c[rank_in] = c;
                by_rank_w[rank_in] = rc.weight(x);
            }
            __syncthreads();
            if (draw_from_list && tid < want) {   // thread r: the weight of candidates 0 .. r
                U128 cum{0ull, 0ull};
                for (int j = 0; j <= tid; ++j) cum = u128_add(cum, U128{0ull, by_rank_w[j]});
                const U128 before = u128_sub(cum, U128{0ull, by_rank_w[tid]});
                if (u128_ge(cum, target) && (tid == 0 || !u128_ge(before, target))) sh->pick = tid;
            }
            __syncthreads();
            if (tid == 0) {
                if (draw_from_list) put_token(a.tokens, a.tokens_host, out, comp_id(by_rank_c[sh->pick]));
                a.kept_n[out] = (int)n_keep;
            }
        }
    }
    cluster_sync_all();   // no CTA leaves while another may still read its shared memory
}

}  // namespace

size_t full_row_smem_bytes(int n_vocab) {
    const int per = (((n_vocab + kFullCluster - 1) / kFullCluster) + 3) & ~3;
    const size_t bitmap = sizeof(unsigned) * (size_t)((per + 31) / 32);
    // (the kept set is ordered in the slice's memory: three arrays of kMaxK 64-bit words)
    const size_t slice = per <= kSliceCache ? sizeof(float) * (size_t)std::max(per, 6 * kMaxK) : 3 * sizeof(u64) * (size_t)kMaxK;
    return sizeof(FullShared) + bitmap + 16 + slice;
}

int prepare_full_row_kernel(int max_vocab) {
    // the largest request of any row length up to max_vocab: rows that still fit the slice cache need the most
    const size_t most = std::max(full_row_smem_bytes(max_vocab), full_row_smem_bytes(std::min(max_vocab, kFullCluster * kSliceCache)));
    cudaError_t e = cudaFuncSetAttribute(full_row_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most);
    return (int)e;
}

int launch_full_row_kernel(const float* logits, const RowDesc* rows, int n_rows, const int32_t* hist, int32_t* tokens, int32_t* tokens_host,
                           int32_t* kept_ids, double* kept_pr, int32_t* kept_n, int record, uint32_t* status, uint32_t* status_host, int n_vocab,
                           int vocab_offset, int write_back, float softcap, uint64_t* trace, void* stream) {
    if (n_vocab > (1 << 22)) return (int)cudaErrorInvalidValue;   // the histogram's limb sums are sized for 4 M logits
    FullArgs a{};
    a.logits = logits;
    a.rows = rows;
    a.hist = hist;
    a.tokens = tokens;
    a.tokens_host = tokens_host;
    a.status_host = status_host;
    a.kept_ids = kept_ids;
    a.kept_pr = kept_pr;
    a.kept_n = kept_n;
    a.status = status;
    a.n_vocab = n_vocab;
    a.vocab_offset = vocab_offset;
    a.write_back = write_back;
    a.record = record;
    a.softcap = softcap;
    a.trace = reinterpret_cast<u64*>(trace);
    const int per = (((n_vocab + kFullCluster - 1) / kFullCluster) + 3) & ~3;
    const int cache_slice = per <= kSliceCache ? 1 : 0;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kFullCluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)(n_rows * kFullCluster));
    cfg.blockDim = dim3(kFullThreads);
    cfg.dynamicSmemBytes = full_row_smem_bytes(n_vocab);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, full_row_kernel, a, cache_slice);
}

}  // namespace fsb
