// fsb_device.cuh - device-side building blocks of the static-plan streaming kernel (sm_100a).
//
//  * order-preserving 64-bit candidate keys ("composites"): (logit descending, token id ascending) becomes plain
//    unsigned descending order, with -0.0f and +0.0f mapped to the same key - the order of the reference's
//    comparator `a.first > b.first || (a.first == b.first && a.second < b.second)` (src/sampler.cpp:31,34);
//  * mbarrier + 1-D bulk asynchronous copy (global -> this CTA's shared memory) wrappers; streaming 16-byte
//    loads and the programmatic-dependent-launch controls;
//  * a CTA-wide selection of the k largest composites by bisection with counting barriers;
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

// Thread-block clusters (pairs of CTAs that share a row): rank in the cluster, the address of a shared-memory
// location in another CTA of the cluster, stores to it, and the cluster's barrier (arrive releases this thread's
// stores to the cluster, wait acquires the others').
__device__ __forceinline__ unsigned cluster_cta_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ unsigned cluster_map_shared(unsigned local_addr, unsigned rank) {
    unsigned a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local_addr), "r"(rank));
    return a;
}
__device__ __forceinline__ void cluster_store_u64(unsigned addr, u64 v) { asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(addr), "l"(v) : "memory"); }
__device__ __forceinline__ void cluster_store_u32(unsigned addr, unsigned v) { asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// Ticket counter shared by the CTAs of a row: the add releases this thread's earlier writes - and those of the
// CTA's other threads that a barrier ordered before it - to the whole device, and acquires what earlier ticket
// holders released.
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

// Barrier of the kThreads consumer threads of a CTA (named barrier 1).  The streaming kernel has one more warp,
// the copy producer, which never takes part in it; kernels with only kThreads threads use it like __syncthreads().
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory"); }

// What the streaming kernel knows about the segment it is working on (written once per segment by one thread).
struct SegCtx {
    const float* row;   // the row's logits
    float pen;          // repetition penalty of the row
    float cap;          // softcap, 0 = off
    int has_pen;
    int id_base;        // token id of column 0
    int seg_lo;         // first column of the segment (= column of bit 0 of the bitmap)
    int seg_hi;         // one past its last column
    int n_vocab;
    int vec_ok;         // rows start on 16-byte boundaries
    int k;              // the row's candidate count
    int final_in_mem;   // write-back mode: the row in global memory already holds the transformed logits
};

struct SharedCtl {
    u64 full[kStages];                // "tile landed": completed by the copy (or by the producer for tiny tails)
    u64 empty[kStages];               // "tile consumed": every consumer warp hands the ring slot back
    u64 red[2 * kNumWarps];           // cross-warp reduction scratch
    double dsum;
    alignas(16) float wbound[kNumWarps];   // per-warp admission bounds (see the streaming kernel); read with 16-byte loads
    int wcount[kNumWarps];            // lengths of a row's ordered candidate lists while they are merged
    int sum[3];                       // rotating counters of the selection steps
    int out_cnt;
    int base, last;
    int imax, imin1, imin2;
    int need_compact;                 // a lane's queue is nearly full: the CTA must re-select
    int abort;                        // a copy did not land in time
    u64 ev_bound;                     // composite bound of the latest re-selection (0: nothing was dropped)
    int rank[kMaxK];                  // ranks of the entries while a list is ordered
    int recv_n[8];                    // clustered CTAs: candidates CTA r of the row's cluster has put into part r - 1 of the receive buffer (entry r)
    SegCtx seg;
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
};

struct TailOut {
    int32_t* tokens;
    int32_t* tokens_host;   // mirror of the tokens in mapped host memory, or null
    unsigned* status_host;  // takes a non-zero word whenever a status bit is set, or null
    int32_t* kept_ids;
    double* kept_pr;
    int32_t* kept_n;
    u64* shard_out;
    int32_t* shard_n;       // null: the count goes to the header word of the row's list
    int shard_stride;
    unsigned* status;
};

// Orders the k largest of buf[0..n) (distinct composites in shared memory; fewer if n < k) into out[0..kk),
// descending, and returns kk = min(n, k).  Long lists are first cut down to k by bisection.  What is left (at most
// kMaxK entries) is ranked by counting: entry e is looked after by kThreads / n threads, each of which counts the
// larger entries in its part of the list - two per 16-byte broadcast read, no dependency between the reads - and
// the parts are added up with one shared-memory atomic each.  buf (16-byte aligned, room for one entry of padding)
// is overwritten; `out` has room for kMaxK composites and must not overlap buf; the ranks live in ctl->rank.  All
// consumer threads must call, after a barrier that made buf visible; out is visible to all on return.
static __device__ __forceinline__ int topk_sorted(u64* buf, int n, int k, u64* out, SharedCtl* ctl) {
    const int tid = threadIdx.x;
    if (n > kMaxK) n = select_list_topk(buf, n, k, out, ctl);
    if (n <= 0) return 0;
    const int parts = kThreads / n;                    // >= 2 threads per entry
    const int part = tid / n, e = tid - part * n;
    if (tid < kMaxK) ctl->rank[tid] = 0;
    if (tid == 0 && (n & 1)) buf[n] = 0ull;            // padding: 0 is below every composite
    consumer_sync();
    if (part < parts) {
        const u64 c = buf[e];
        const int per = (((n + parts - 1) / parts) + 1) & ~1;   // entries per part, even: parts start on 16-byte boundaries
        const int j0 = part * per, j1 = min(n, j0 + per);
        int larger = 0;
#pragma unroll 4
        for (int j = j0; j < j1; j += 2) {
            const ulonglong2 v = *reinterpret_cast<const ulonglong2*>(buf + j);
            larger += (v.x > c ? 1 : 0) + (v.y > c ? 1 : 0);
        }
        if (larger) atomicAdd(&ctl->rank[e], larger);
    }
    consumer_sync();
    if (tid < n) {
        const int r = ctl->rank[tid];
        if (r < k) out[r] = buf[tid];
    }
    consumer_sync();
    return n < k ? n : k;
}

// A status bit for the host: the device word collects the bits, the host mirror (if any) just becomes non-zero.
__device__ __forceinline__ void report_status(unsigned* status, unsigned* status_host, unsigned bit) {
    atomicOr(status, bit);
    if (status_host) *reinterpret_cast<volatile unsigned*>(status_host) = bit;
}
// A row's token: to the device array and, if the caller reads its own memory, to the host mirror.
__device__ __forceinline__ void put_token(int32_t* tokens, int32_t* tokens_host, int index, int token) {
    tokens[index] = token;
    if (tokens_host) tokens_host[index] = token;
}

// srt[0..kk) holds the row's candidates in order (largest first).  Either hands them out (vocabulary-sharded mode)
// or finishes the row: softmax over the candidates in fp64, sequential sums in candidate order, min-p, top-p,
// draw.  `work` is scratch for 2 * kMaxK doubles that does not overlap srt.  All consumer threads must call it with
// the same arguments.
static __device__ __forceinline__ void row_epilogue(const u64* srt, int kk, const RowTail r, double* work, SharedCtl* ctl, const TailOut o) {
    const int tid = threadIdx.x;
    double* e = work;
    double* P = work + kMaxK;
    if (kk <= 0) {   // nothing but NaNs in the row
        if (tid == 0) {
            report_status(o.status, o.status_host, kStatusEmptyRow);
            if (o.shard_out && o.shard_n) o.shard_n[r.out_index] = 0;
            else if (o.shard_out) o.shard_out[(size_t)r.out_index * o.shard_stride] = 0ull;
            else put_token(o.tokens, o.tokens_host, r.out_index, 0);
            if (o.kept_n) o.kept_n[r.out_index] = 0;
        }
        return;
    }
    if (o.shard_out) {
        u64* list = o.shard_out + (size_t)r.out_index * o.shard_stride;
        if (o.shard_n) {
            if (tid < kk) list[tid] = srt[tid];
            if (tid == 0) o.shard_n[r.out_index] = kk;
        } else {
            if (tid < kk) list[1 + tid] = srt[tid];
            if (tid == 0) list[0] = (u64)kk;
        }
        return;
    }
    if (r.flags & kRowGreedy) {   // first index of the maximum (src/sampler.cpp:19-23)
        if (tid == 0) {
            put_token(o.tokens, o.tokens_host, r.out_index, comp_id(srt[0]));
            if (o.kept_n) o.kept_n[r.out_index] = 0;
        }
        return;
    }
    // pr[i] = exp((double)(x_i - x_0) / T)   (fp32 subtraction, fp64 division, src/sampler.cpp:40)
    const float mx = comp_value(srt[0]);
    if (tid < kk) e[tid] = exp(__ddiv_rn((double)__fsub_rn(comp_value(srt[tid]), mx), (double)r.temperature));
    consumer_sync();
    // The reference adds in candidate order, one after the other: one thread runs the chain (the loads do not depend
    // on it, so they run ahead).  (Letting that thread also find the min-p and top-p cuts and the draw while it walks
    // the sums - no atomics, two barriers fewer - was measured 0.3 us slower: the compares lengthen the chain.)  The cumulative sums P[i] = pr[0] + ... + pr[i] serve the top-p walk, `tot` and the
    // draw walk alike: the reference adds the same numbers in the same order in all three.
    if (tid == 0) {
        double s = 0.0;
#pragma unroll 8
        for (int i = 0; i < kk; ++i) s = __dadd_rn(s, e[i]);
        ctl->dsum = s;
        ctl->imax = 0;
        ctl->imin1 = 0x7fffffff;
        ctl->imin2 = 0x7fffffff;
    }
    consumer_sync();
    if (tid < kk) e[tid] = __ddiv_rn(e[tid], ctl->dsum);
    consumer_sync();
    if (tid == 0) {
        double c = 0.0;
#pragma unroll 8
        for (int i = 0; i < kk; ++i) {
            c = __dadd_rn(c, e[i]);
            P[i] = c;
        }
    }
    consumer_sync();
    const double pr = tid < kk ? e[tid] : 0.0;
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
    if (tid == 0) put_token(o.tokens, o.tokens_host, r.out_index, comp_id(srt[pick]));
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
