// fsb_device.cuh - device-side building blocks shared by the sampler kernels (sm_100a).
//
//  * order-preserving 64-bit candidate keys ("composites"): (logit descending, token id ascending) becomes plain
//    unsigned descending order, with -0.0f and +0.0f mapped to the same key - the order of the reference's
//    comparator `a.first > b.first || (a.first == b.first && a.second < b.second)` (src/sampler.cpp:31,34);
//  * mbarrier + 1-D bulk asynchronous copy (global -> this CTA's shared memory) wrappers with bounded waits;
//  * a CTA-wide radix selection of the k largest composites held in shared memory;
//  * the per-row epilogue: softmax in fp64 with the reference's sequential sums, min-p, top-p and the draw
//    (src/sampler.cpp:37-49).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "fsb_internal.h"

namespace fsb {

using u64 = unsigned long long;

// ---------------------------------------------------------------------------------------------- composites
__device__ __forceinline__ u64 make_comp(float x, int id) {
    unsigned u = __float_as_uint(x);
    if (u == 0x80000000u) u = 0u;                                     // -0.0f ties with +0.0f
    const unsigned key = (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // monotone: larger float -> larger key
    return ((u64)key << 32) | (u64)(0xFFFFFFFFu - (unsigned)id);      // lower id -> larger composite
}
__device__ __forceinline__ float comp_value(u64 c) {
    const unsigned key = (unsigned)(c >> 32);
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7FFFFFFFu) : ~key);
}
__device__ __forceinline__ int comp_id(u64 c) { return (int)(0xFFFFFFFFu - (unsigned)(c & 0xFFFFFFFFull)); }

// Order-preserving 32-bit key of a float (the upper half of a composite) and its inverse.
__device__ __forceinline__ unsigned float_key(float x) {
    unsigned u = __float_as_uint(x);
    if (u == 0x80000000u) u = 0u;
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_float(unsigned key) { return __uint_as_float((key & 0x80000000u) ? (key & 0x7FFFFFFFu) : ~key); }

// max of three floats in one instruction (sm_100)
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// A float t with: key(x) >= (L >> 32)  =>  x >= t.  L may have its low bits cleared, which can name a NaN pattern.
__device__ __forceinline__ float comp_floor_value(u64 L) {
    const float t = comp_value(L);
    return (t != t) ? -__int_as_float(0x7f800000) : t;
}

// ---------------------------------------------------------------------------------------------- mbarrier / bulk copy
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(u64* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(u64* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// 1-D bulk copy global -> shared memory of this CTA; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, unsigned bytes, u64* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// One poll of a barrier phase.  The suspend-time hint lets the hardware park the thread until the phase completes
// (or the hint runs out) instead of re-polling: idle warps then stay out of the shared-memory pipeline that the
// working warps need.
__device__ __forceinline__ bool mbar_try_wait(u64* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(20000u)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void mbar_arrive(u64* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Non-blocking look at a barrier phase.
__device__ __forceinline__ bool mbar_test_wait(u64* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(smem_u32(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}
__device__ __forceinline__ u64 global_timer_ns() {
    u64 t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: gives up after limit_cycles SM clocks and reports false; the caller records the failure and
// carries on.  (The SM cycle counter is read, not %globaltimer: a read of the global timer costs about a
// microsecond, which would be paid on every tile.)
__device__ __forceinline__ bool mbar_wait_bounded(u64* bar, unsigned parity, long long limit_cycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 16; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > limit_cycles) return false;
    }
}

// ---------------------------------------------------------------------------------------------- shared control block
constexpr int kNumWarps = kThreads / 32;   // consumer warps of a CTA

// Barrier of the kThreads consumer threads of a CTA (named barrier 1).  The streaming kernel has one more warp,
// the copy producer, which never takes part in it; kernels with only kThreads threads use it like __syncthreads().
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory"); }

struct SharedCtl {
    u64 full[kStages];                // "tile landed": completed by the copy (or by the producer for tiny tails)
    u64 empty[kStages];               // "tile consumed": every consumer warp hands the ring slot back
    u64 red[16];                      // cross-warp reduction scratch
    double dsum;
    unsigned hist[256];
    float wbound[kNumWarps];          // per-warp admission bounds (see the streaming kernel)
    int out_cnt;
    int sel_digit, sel_above, sel_count;
    int base, last;
    int imax, imin1, imin2;
    int abort;
    int need_compact;                 // a lane found its candidate queue full
};

// The candidates a selection looks at: this thread's own queue (entries myq[s * 32], s < mycnt) plus a list of
// composites shared by the CTA (list[i], i < list_n, dealt to the threads).  Calls f(c) for every candidate once.
template <class F>
__device__ __forceinline__ void for_each_candidate(const u64* myq, int mycnt, const u64* list, int list_n, F f) {
#pragma unroll 1
    for (int s = 0; s < mycnt; ++s) f(myq[s * 32]);
#pragma unroll 1
    for (int i = threadIdx.x; i < list_n; i += kThreads) f(list[i]);
}

// ---------------------------------------------------------------------------------------------- top-k selection
// Writes the k largest candidates (all of them when there are no more than k) to dst, unordered, and returns how
// many.  *L_out receives a bound L with: chosen == { c : c >= L } (0 when everything was taken), so L is also a
// valid admission bound for later candidates.  `out` is kMaxK entries of scratch; dst may be the shared list
// itself.  All kThreads consumer threads must call.  MSB-first radix descent, starting at the highest bit in
// which the candidates differ and stopping as soon as a digit bucket is taken whole.
static __device__ __noinline__ int select_topk(const u64* myq, int mycnt, const u64* list, int list_n, int k, u64* out, u64* dst,
                                        SharedCtl* ctl, unsigned* status, u64* L_out) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    u64 mn = ~0ull, mx = 0ull;
    for_each_candidate(myq, mycnt, list, list_n, [&](u64 c) {
        mn = min(mn, c);
        mx = max(mx, c);
    });
    int cnt = __reduce_add_sync(0xffffffffu, mycnt);
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if (lane == 0) {
        ctl->red[warp] = mn;
        ctl->red[8 + warp] = mx;
        ctl->hist[warp] = (unsigned)cnt;
    }
    consumer_sync();
    mn = ctl->red[0];
    mx = ctl->red[8];
    cnt = list_n + (int)ctl->hist[0];
#pragma unroll
    for (int w = 1; w < kNumWarps; ++w) {
        mn = min(mn, ctl->red[w]);
        mx = max(mx, ctl->red[8 + w]);
        cnt += (int)ctl->hist[w];
    }
    consumer_sync();   // hist is reused below
    u64 mask = 0ull, pfx = 0ull;
    if (cnt > k) {
        int need = k;
        if (mx != mn) {
            int hb = 63 - __clzll((long long)(mx ^ mn));
            mask = (hb == 63) ? 0ull : (~0ull << (hb + 1));
            pfx = mx & mask;
            for (;;) {
                const int w = hb + 1 < 8 ? hb + 1 : 8, lo = hb + 1 - w;
                const unsigned dmask = (1u << w) - 1u;
                ctl->hist[tid] = 0u;
                consumer_sync();
                for_each_candidate(myq, mycnt, list, list_n, [&](u64 c) {
                    if ((c & mask) == pfx) atomicAdd(&ctl->hist[(unsigned)(c >> lo) & dmask], 1u);
                });
                consumer_sync();
                if (warp == 0) {
                    unsigned h[8], s = 0u;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        h[j] = ctl->hist[lane * 8 + j];
                        s += h[j];
                    }
                    unsigned suf = s;   // inclusive suffix sum: this lane's bins and all higher ones
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const unsigned t = __shfl_down_sync(0xffffffffu, suf, o);
                        if (lane + o < 32) suf += t;
                    }
                    const unsigned above = suf - s;
                    if (above < (unsigned)need && suf >= (unsigned)need) {
                        unsigned acc = above;
                        int d = 7;
                        for (; d > 0; --d) {
                            if (acc + h[d] >= (unsigned)need) break;
                            acc += h[d];
                        }
                        ctl->sel_digit = lane * 8 + d;
                        ctl->sel_above = (int)acc;
                        ctl->sel_count = (int)h[d];
                    }
                }
                consumer_sync();
                const int d = ctl->sel_digit, sc = ctl->sel_count;
                need -= ctl->sel_above;
                pfx |= (u64)(unsigned)d << lo;
                mask |= (u64)dmask << lo;
                if (sc == need) break;
                if (lo == 0) {   // equal composites: cannot happen for distinct token ids
                    if (tid == 0) atomicOr(status, kStatusBadTie);
                    break;
                }
                hb = lo - 1;
            }
        } else if (tid == 0) {
            atomicOr(status, kStatusBadTie);
        }
    }
    const int kk = cnt < k ? cnt : k;
    if (tid == 0) ctl->out_cnt = 0;
    consumer_sync();
    for_each_candidate(myq, mycnt, list, list_n, [&](u64 c) {
        if ((c & mask) >= pfx) {
            const int p = atomicAdd(&ctl->out_cnt, 1);
            if (p < kk) out[p] = c;
        }
    });
    consumer_sync();
    if (dst != out) {
#pragma unroll 1
        for (int i = tid; i < kk; i += kThreads) dst[i] = out[i];
        consumer_sync();
    }
    if (L_out) *L_out = pfx;
    return kk;
}

// ---------------------------------------------------------------------------------------------- row epilogue
// What the epilogue needs to know about a row.
struct RowTail {
    u64 rng_word;
    float temperature, top_p, min_p;
    int k;
    int flags;
    int out_index;
};

struct TailOut {
    int32_t* tokens;
    int32_t* kept_ids;
    double* kept_pr;
    int32_t* kept_n;
    u64* shard_out;
    int32_t* shard_n;
    unsigned* status;
};

// buf[0..total) holds a superset of the row's top-k composites (total <= kMergeCap, buf has kCap entries).
// Selects the k best, orders them, and either hands them out (vocabulary-sharded mode) or finishes the row:
// softmax over the candidates in fp64, sequential sums in candidate order, min-p, top-p, draw.
// All threads of the CTA must call it with the same arguments.
static __device__ __noinline__ void finish_row(u64* buf, int total, const RowTail r, u64* out, SharedCtl* ctl, const TailOut o) {
    const int tid = threadIdx.x;
    if (total > r.k) total = select_topk(nullptr, 0, buf, total, r.k, out, buf, ctl, o.status, nullptr);
    const int kk = total;
    u64* srt = buf + kMaxK;
    double* e = reinterpret_cast<double*>(buf + 2 * kMaxK);
    double* P = reinterpret_cast<double*>(buf + 3 * kMaxK);
    if (kk <= 0) {   // nothing but NaNs in the row
        if (tid == 0) {
            atomicOr(o.status, kStatusEmptyRow);
            if (o.shard_out) o.shard_n[r.out_index] = 0;
            else o.tokens[r.out_index] = 0;
            if (o.kept_n) o.kept_n[r.out_index] = 0;
        }
        return;
    }
    // order by rank counting: composites are distinct, so ranks are a permutation of 0..kk-1
    if (tid < kk) {
        const u64 c = buf[tid];
        int rank = 0;
#pragma unroll 4
        for (int j = 0; j < kk; ++j) rank += (buf[j] > c) ? 1 : 0;
        srt[rank] = c;
    }
    consumer_sync();
    if (o.shard_out) {
        if (tid < kk) o.shard_out[(size_t)r.out_index * kMaxK + tid] = srt[tid];
        if (tid == 0) o.shard_n[r.out_index] = kk;
        consumer_sync();
        return;
    }
    if (r.flags & kRowGreedy) {   // first index of the maximum (src/sampler.cpp:19-23)
        if (tid == 0) {
            o.tokens[r.out_index] = comp_id(srt[0]);
            if (o.kept_n) o.kept_n[r.out_index] = 0;
        }
        consumer_sync();
        return;
    }
    // pr[i] = exp((double)(x_i - x_0) / T)   (fp32 subtraction, fp64 division, src/sampler.cpp:40)
    const float mx = comp_value(srt[0]);
    if (tid < kk) e[tid] = exp(__ddiv_rn((double)__fsub_rn(comp_value(srt[tid]), mx), (double)r.temperature));
    consumer_sync();
    if (tid == 0) {
        double s = 0.0;
#pragma unroll 4
        for (int i = 0; i < kk; ++i) s = __dadd_rn(s, e[i]);   // sequential, candidate order
        ctl->dsum = s;
        ctl->imax = 0;
        ctl->imin1 = 0x7fffffff;
        ctl->imin2 = 0x7fffffff;
    }
    consumer_sync();
    const double sum = ctl->dsum;
    double pr = 0.0;
    if (tid < kk) {
        pr = __ddiv_rn(e[tid], sum);
        e[tid] = pr;
    }
    consumer_sync();
    // cumulative sums P[i] = pr[0] + ... + pr[i], sequential: the top-p walk, `tot` and the draw walk of the
    // reference all add the same numbers in the same order, so one array serves the three of them
    if (tid == 0) {
        double c = 0.0;
#pragma unroll 4
        for (int i = 0; i < kk; ++i) {
            c = __dadd_rn(c, e[i]);
            P[i] = c;
        }
    }
    if (r.min_p > 0.0f && tid < kk) {   // keep = 1 + last index whose probability is not below pr[0] * min_p
        const double thr = __dmul_rn(e[0], (double)r.min_p);
        if (!(pr < thr)) atomicMax(&ctl->imax, tid);
    }
    consumer_sync();
    int keep = kk;
    if (r.min_p > 0.0f) keep = ctl->imax + 1;
    if (r.top_p < 1.0f) {   // shortest prefix whose cumulative probability reaches top_p, crossing element included
        if (tid < keep && P[tid] >= (double)r.top_p) atomicMin(&ctl->imin1, tid);
        consumer_sync();
        const int i1 = ctl->imin1;
        if (i1 != 0x7fffffff && i1 + 1 < keep) keep = i1 + 1;
    }
    const double tot = P[keep - 1];
    // one engine output -> U[0,1) as libstdc++ does it, then r = u * tot + 0.0
    double u = __dmul_rn(__ull2double_rn(r.rng_word), 5.42101086242752217003726400434970855712890625e-20);   // 2^-64
    if (u >= 1.0) u = __longlong_as_double(0x3FEFFFFFFFFFFFFFll);
    const double rr = __dadd_rn(__dmul_rn(u, tot), 0.0);
    if (tid < keep && rr <= P[tid]) atomicMin(&ctl->imin2, tid);
    consumer_sync();
    const int i2 = ctl->imin2;
    const int pick = (i2 != 0x7fffffff) ? i2 : keep - 1;
    if (tid == 0) o.tokens[r.out_index] = comp_id(srt[pick]);
    if (o.kept_n) {
        if (tid < keep) {
            o.kept_ids[(size_t)r.out_index * kMaxK + tid] = comp_id(srt[tid]);
            o.kept_pr[(size_t)r.out_index * kMaxK + tid] = e[tid];
        }
        if (tid == 0) o.kept_n[r.out_index] = keep;
    }
    consumer_sync();
}

}  // namespace fsb
