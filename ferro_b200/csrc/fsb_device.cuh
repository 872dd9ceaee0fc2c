// fsb_device.cuh - device-side building blocks shared by the sampler kernels (sm_100a).
//
//  * order-preserving 64-bit candidate keys ("composites"): (logit descending, token id ascending) becomes plain
//    unsigned descending order, with -0.0f and +0.0f mapped to the same key - the order of the reference's
//    comparator `a.first > b.first || (a.first == b.first && a.second < b.second)` (src/sampler.cpp:31,34);
//  * mbarrier + 1-D bulk asynchronous copy (global -> this CTA's shared memory) wrappers and the
//    programmatic-dependent-launch controls;
//  * CTA-wide selection and ordering of the k largest composites of a list in shared memory;
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
// The smallest composite a logit >= t can have (t is not NaN): its key with every token id allowed.
__device__ __forceinline__ u64 comp_floor_of(float t) { return (u64)float_key(t) << 32; }

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
// One poll of a barrier phase, with a suspend-time hint (the hardware may park the thread until the phase completes).
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
// ---------------------------------------------------------------------------------------------- launch order
// Programmatic dependent launch: let the next launch in the stream begin as resources free up, and wait for the
// previous launch to be complete (and its memory visible) before touching anything it wrote.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_prior() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Ticket counter shared by the CTAs that work on one row: the add releases this thread's earlier writes - and those
// of the CTA's other threads that a barrier ordered before it - to the whole device, and acquires what earlier
// ticket holders released.
__device__ __forceinline__ unsigned ticket_add_acq_rel(unsigned* p, unsigned v) {
    unsigned old;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}

__device__ __forceinline__ u64 global_timer_ns() {
    u64 t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// ---------------------------------------------------------------------------------------------- shared control block
constexpr int kNumWarps = kThreads / 32;

// Barrier of the kThreads consumer threads of a CTA (named barrier 1).  The streaming kernel has two more warps
// (copies, set-up), which never take part in it; kernels with only kThreads threads use it like __syncthreads().
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory"); }

// One work item of the streaming kernel as its set-up warp hands it to the copy warp and the consumers.
struct alignas(16) ItemCtx {
    alignas(16) RowDesc d;  // the row's descriptor (written with 16-byte stores)
    const float* row_ptr;   // the row's logits
    int done;               // 1: there is no more work (the other fields are not set)
    int row;                // index of the row's descriptor
    int chunk;              // chunk of the row
    int tile0, ntiles;      // tiles of the row that make up the chunk
    float thr0;             // a value that k logits of the row are already known to reach (-inf: none)
};

struct alignas(16) SharedCtl {
    u64 full[kStages];                // "tile landed": completed by the copy (or by the copy warp for tiny tails)
    u64 empty[kStages];               // "tile consumed": every consumer warp hands the ring slot back
    u64 item_posted[2];               // "the item's place in the matrix is known": the copies may start
    u64 item_ready[2];                // "the item's descriptor and penalty bitmap are complete": the consumers may start
    u64 item_free[2];                 // "the consumers are done with the item's descriptor and bitmap"
    u64 red[2 * kNumWarps];           // cross-warp reduction scratch
    double dsum;
    alignas(16) u64 wbound[kNumWarps];     // per-warp admission bounds (see the streaming kernel): item tag << 32 | float bits
    int wcount[kMaxChunks];           // lengths of a row's ordered candidate lists while they are merged
    int sum[3];                       // rotating counters of the selection steps
    int out_cnt;
    int n_el;                         // candidates of the current item written so far
    int last;
    int bsel, nsel;                   // histogram selection: the bucket the k-th candidate lies in, candidates from there up
    int imax, imin1, imin2;
    int abort;                        // a wait ran out of time: every later wait is cut short, the kernel winds down
    RowDesc cur;                      // descriptor of the item whose end-of-item work is running
    RowDesc prev;                     // descriptor of the row whose ticket is still on its way (see the streaming kernel)
    alignas(16) ItemCtx item[2];
};

// ---------------------------------------------------------------------------------------------- top-k selection
// Smallest and largest of the composites the threads hold (each thread passes the extremes of its own; threads
// with nothing pass ~0 and 0).  All threads of the CTA must call.
__device__ __forceinline__ void cta_minmax(u64& mn, u64& mx, SharedCtl* ctl) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if (lane == 0) {
        ctl->red[warp] = mn;
        ctl->red[kNumWarps + warp] = mx;
    }
    consumer_sync();
    mn = ctl->red[0];
    mx = ctl->red[kNumWarps];
#pragma unroll
    for (int w = 1; w < kNumWarps; ++w) {
        mn = min(mn, ctl->red[w]);
        mx = max(mx, ctl->red[kNumWarps + w]);
    }
    consumer_sync();   // the scratch may be written again
}

// Bound L of the k largest among n > k distinct composites held by the threads of the CTA: exactly k composites
// are >= L.  count_ge(t) = how many of this thread's composites are >= t.  MSB-first bisection from the highest bit
// in which the composites differ: every step is one warp reduction, one shared-memory add per warp and one
// barrier, and the search stops as soon as a trial bound is passed by exactly k composites.
template <class Count>
__device__ __forceinline__ u64 bisect_bound(int k, u64 mn, u64 mx, SharedCtl* ctl, Count count_ge) {
    if (mx == mn) return mn;
    const int tid = threadIdx.x;
    const int hb = 63 - __clzll((long long)(mx ^ mn));
    u64 pfx = (hb == 63) ? 0ull : (mx & (~0ull << (hb + 1)));
    if (tid == 0) ctl->sum[0] = 0;
    consumer_sync();
    int step = 0;
#pragma unroll 1
    for (int b = hb; b >= 0; --b, ++step) {
        const u64 trial = pfx | (1ull << b);
        const int wsum = __reduce_add_sync(0xffffffffu, count_ge(trial));
        if ((tid & 31) == 0 && wsum) atomicAdd(&ctl->sum[step % 3], wsum);
        if (tid == 0) ctl->sum[(step + 1) % 3] = 0;   // last read two barriers ago
        consumer_sync();
        const int total = ctl->sum[step % 3];
        if (total >= k) pfx = trial;
        if (total == k) break;
    }
    return pfx;
}

// Keeps the k largest of list[0..n) (distinct composites in shared memory) in list[0..k), unordered, and returns
// min(n, k).  `tmp` is scratch for k composites outside the list.  All threads of the CTA must call.
static __device__ __noinline__ int select_list_topk(u64* list, int n, int k, u64* tmp, SharedCtl* ctl) {
    if (n <= k) return n;
    const int tid = threadIdx.x;
    u64 mn = ~0ull, mx = 0ull;
#pragma unroll 1
    for (int i = tid; i < n; i += kThreads) {
        const u64 c = list[i];
        mn = min(mn, c);
        mx = max(mx, c);
    }
    cta_minmax(mn, mx, ctl);
    const u64 L = bisect_bound(k, mn, mx, ctl, [&](u64 t) {
        int c = 0;
#pragma unroll 1
        for (int i = tid; i < n; i += kThreads) c += list[i] >= t ? 1 : 0;
        return c;
    });
    if (tid == 0) ctl->out_cnt = 0;
    consumer_sync();
#pragma unroll 1
    for (int i = tid; i < n; i += kThreads) {
        const u64 c = list[i];
        if (c >= L) {
            const int p = atomicAdd(&ctl->out_cnt, 1);
            if (p < k) tmp[p] = c;
        }
    }
    consumer_sync();
#pragma unroll 1
    for (int i = tid; i < k; i += kThreads) list[i] = tmp[i];
    consumer_sync();
    return k;
}

// ---------------------------------------------------------------------------------------------- row epilogue
// What the epilogue needs to know about a row.
struct RowTail {
    u64 rng_word;
    float temperature, top_p, min_p;
    int k;
    int flags;
    int out_index;
    int scan_sums;
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

// Bitonic sort, descending, of the 32 values held by the lanes of one warp.
__device__ __forceinline__ u64 warp_sort32_desc(u64 v) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int k2 = 2; k2 <= 32; k2 <<= 1) {
#pragma unroll
        for (int j = k2 >> 1; j > 0; j >>= 1) {
            const u64 o = __shfl_xor_sync(0xffffffffu, v, j);
            const bool up = (lane & k2) == 0;
            const bool lower = (lane & j) == 0;
            v = (up == lower) ? max(v, o) : min(v, o);
        }
    }
    return v;
}

// Orders the k largest of buf[0..n) (distinct composites in shared memory; fewer if n < k) into out[0..kk),
// descending, and returns kk = min(n, k).  Lists longer than kThreads entries are first cut down to k by bisection.
// The rank of an entry is the number of entries above it: entry i is counted by kThreads / n' neighbouring threads
// (n' = n rounded up to a power of two), each over its share of the list (every load is a broadcast), and their
// counts are added with shuffles.  buf is overwritten only by the cut; `out` has room for kMaxK composites and must
// not overlap buf.  All consumer threads must call, after a barrier that made buf visible; out is visible on return.
static __device__ __forceinline__ int topk_sorted(u64* buf, int n, int k, u64* out, SharedCtl* ctl) {
    const int tid = threadIdx.x;
    if (n > kThreads) n = select_list_topk(buf, n, k, out, ctl);
    int shift = 0;   // log2 of the threads per entry
    while ((n << (shift + 1)) <= kThreads && shift < 5) ++shift;
    const int P = 1 << shift;
    const int i = tid >> shift, part = tid & (P - 1);
    const int len = (n + P - 1) >> shift;
    const int j0 = part * len, j1 = min(n, j0 + len);
    const u64 c = i < n ? buf[i] : ~0ull;
    int cnt = 0;
#pragma unroll 4
    for (int j = j0; j < j1; ++j) cnt += buf[j] > c ? 1 : 0;
    for (int o = 1; o < P; o <<= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    if (i < n && part == 0 && cnt < k) out[cnt] = c;
    consumer_sync();
    return n < k ? n : k;
}

// srt[0..kk) holds the row's candidates in order (largest first).  Either hands them out (vocabulary-sharded mode)
// or finishes the row: softmax over the candidates in fp64, sums in candidate order, min-p, top-p, draw.  `work` is
// scratch for 2 * kMaxK doubles that does not overlap srt.  All consumer threads must call it with the same
// arguments; only the first warp works, so the call contains no CTA barrier.  srt and work must be visible to the
// first warp (a barrier before the call), and must not be rewritten before the next CTA barrier after it.
static __device__ __forceinline__ void row_epilogue(const u64* srt, int kk, const RowTail r, double* work, const TailOut o) {
    const int tid = threadIdx.x;
    if (tid >= 32) return;
    const int lane = tid;
    double* e = work;
    double* P = work + kMaxK;
    if (kk <= 0) {   // nothing but NaNs in the row
        if (lane == 0) {
            atomicOr(o.status, kStatusEmptyRow);
            if (o.shard_out) o.shard_n[r.out_index] = 0;
            else o.tokens[r.out_index] = 0;
            if (o.kept_n) o.kept_n[r.out_index] = 0;
        }
        return;
    }
    if (o.shard_out) {
        for (int i = lane; i < kk; i += 32) o.shard_out[(size_t)r.out_index * kMaxK + i] = srt[i];
        if (lane == 0) o.shard_n[r.out_index] = kk;
        return;
    }
    if (r.flags & kRowGreedy) {   // first index of the maximum (src/sampler.cpp:19-23)
        if (lane == 0) {
            o.tokens[r.out_index] = comp_id(srt[0]);
            if (o.kept_n) o.kept_n[r.out_index] = 0;
        }
        return;
    }
    // pr[i] = exp((double)(x_i - x_0) / T)   (fp32 subtraction, fp64 division, src/sampler.cpp:40)
    const float mx = comp_value(srt[0]);
    const double temp = (double)r.temperature;
    for (int i = lane; i < kk; i += 32) e[i] = exp(__ddiv_rn((double)__fsub_rn(comp_value(srt[i]), mx), temp));
    __syncwarp();
    // The reference adds in candidate order, one after the other (src/sampler.cpp:41,44,46): one lane runs the chain
    // (the loads do not depend on it, so they run ahead).  The cumulative sums P[i] = pr[0] + ... + pr[i] serve the
    // top-p walk, `tot` and the draw walk alike: the reference adds the same numbers in the same order in all three.
    // With scan_sums the two chains are warp prefix scans instead: the sums then differ from the reference's in the
    // last bits (far inside the 1e-6 the parity contract allows), and a row costs two short scans.
    double s = 0.0;
    if (!r.scan_sums) {
        if (lane == 0) {
#pragma unroll 8
            for (int i = 0; i < kk; ++i) s = __dadd_rn(s, e[i]);
        }
        s = __shfl_sync(0xffffffffu, s, 0);
        for (int i = lane; i < kk; i += 32) e[i] = __ddiv_rn(e[i], s);
        __syncwarp();
        if (lane == 0) {
            double c = 0.0;
#pragma unroll 8
            for (int i = 0; i < kk; ++i) {
                c = __dadd_rn(c, e[i]);
                P[i] = c;
            }
        }
    } else {
        // lane l owns the contiguous block [l * per, l * per + per) of the candidates
        const int per = (kk + 31) >> 5;
        const int b0 = lane * per, b1 = min(kk, b0 + per);
        double part = 0.0;
        for (int i = b0; i < b1; ++i) part += e[i];
        double inc = part;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const double t = __shfl_up_sync(0xffffffffu, inc, d);
            if (lane >= d) inc += t;
        }
        s = __shfl_sync(0xffffffffu, inc, 31);
        part = 0.0;
        for (int i = b0; i < b1; ++i) {
            e[i] = __ddiv_rn(e[i], s);
            part += e[i];
        }
        inc = part;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const double t = __shfl_up_sync(0xffffffffu, inc, d);
            if (lane >= d) inc += t;
        }
        double c = inc - part;
        for (int i = b0; i < b1; ++i) {
            c += e[i];
            P[i] = c;
        }
    }
    __syncwarp();
    // keep = 1 + last index whose probability is not below pr[0] * min_p   (src/sampler.cpp:43)
    int keep = kk;
    if (r.min_p > 0.0f) {
        const double thr = __dmul_rn(e[0], (double)r.min_p);
        int last = 0;
        for (int i = lane; i < kk; i += 32)
            if (!(e[i] < thr)) last = i;
        keep = __reduce_max_sync(0xffffffffu, last) + 1;
    }
    if (r.top_p < 1.0f) {   // shortest prefix whose cumulative probability reaches top_p, crossing element included (:44)
        int first = 0x7fffffff;
        for (int i = lane; i < keep; i += 32)
            if (P[i] >= (double)r.top_p) {
                first = i;
                break;
            }
        first = __reduce_min_sync(0xffffffffu, first);
        if (first != 0x7fffffff && first + 1 < keep) keep = first + 1;
    }
    const double tot = P[keep - 1];
    // one engine output -> U[0,1) as libstdc++ does it, then r = u * tot + 0.0   (:45-47)
    double u = __dmul_rn(__ull2double_rn(r.rng_word), 5.42101086242752217003726400434970855712890625e-20);   // 2^-64
    if (u >= 1.0) u = __longlong_as_double(0x3FEFFFFFFFFFFFFFll);
    const double rr = __dadd_rn(__dmul_rn(u, tot), 0.0);
    int pick = 0x7fffffff;
    for (int i = lane; i < keep; i += 32)
        if (rr <= P[i]) {
            pick = i;
            break;
        }
    pick = __reduce_min_sync(0xffffffffu, pick);
    if (pick == 0x7fffffff) pick = keep - 1;
    if (lane == 0) o.tokens[r.out_index] = comp_id(srt[pick]);
    if (o.kept_n) {
        for (int i = lane; i < keep; i += 32) {
            o.kept_ids[(size_t)r.out_index * kMaxK + i] = comp_id(srt[i]);
            o.kept_pr[(size_t)r.out_index * kMaxK + i] = e[i];
        }
        if (lane == 0) o.kept_n[r.out_index] = keep;
    }
}

}  // namespace fsb
