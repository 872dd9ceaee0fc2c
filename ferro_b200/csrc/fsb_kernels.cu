// fsb_kernels.cu - the streaming candidate kernel of the B200 batched token sampler (sm_100a).
//
// One launch samples every row of a batch whose effective k is at most kMaxK (greedy rows are k = 1):
//   repetition penalty (src/sampler.cpp:11-18) -> greedy argmax (:19-23) or top-k candidates (:25-35)
//   -> fp64 softmax (:37-41) -> min-p (:43) -> top-p (:44) -> seeded draw (:45-49).
// (reference paths are relative to the paragontasx/ferro project root)
// How it works is described above the kernel below.
#include <cuda_runtime.h>

#include <cstddef>

#include "../../include/ferro_sampler_b200.h"
#include "fsb_device.cuh"

namespace fsb {
namespace {

constexpr int kWarps = kThreads / 32;
constexpr int kWTile = kTile / kWarps;          // 512 logits: a warp's part of a CTA tile
constexpr int kCopyWarp = kWarps;               // fetches work items, issues the bulk copies
constexpr int kSetupWarp0 = kWarps + 1;         // two set-up warps (one per hand-over slot): descriptors, penalty bitmaps
constexpr int kBlockThreads = kThreads + 96;

constexpr size_t kSmemStage = (size_t)kStages * kTile * sizeof(float);
constexpr size_t kSmemQv = (size_t)kLaneQueue * kThreads * sizeof(float4);     // the lanes' queues of noted cells: the four logits ...
constexpr size_t kSmemQc = (size_t)kLaneQueue * kThreads * sizeof(int);        // ... and the token id of the first
constexpr size_t kSmemBitmap = 2 * (size_t)kItemBitmapWords * sizeof(unsigned);   // penalty bitmaps of two work items
constexpr size_t kSmemList = (size_t)kListCap * sizeof(u64);                    // candidates about to be ordered
constexpr size_t kSmemSorted = (size_t)kMaxK * sizeof(u64);                     // ordered candidates
constexpr size_t kSmemWork = 2 * (size_t)kMaxK * sizeof(double);                // the epilogue's doubles
constexpr size_t kSmemHist = 256 * sizeof(unsigned);                            // histogram of the selection
constexpr size_t kSmemTotal = kSmemStage + kSmemQv + kSmemQc + kSmemBitmap + kSmemList + kSmemSorted + kSmemWork + kSmemHist + sizeof(SharedCtl);
static_assert(kSmemTotal <= 227 * 1024, "one CTA per SM");
static_assert((kSmemStage + kSmemQv + kSmemQc + kSmemBitmap + kSmemList + kSmemSorted + kSmemWork + kSmemHist) % 16 == 0, "the control block starts on a 16-byte boundary");
static_assert(offsetof(SharedCtl, item) % 16 == 0 && offsetof(ItemCtx, d) % 16 == 0 && sizeof(ItemCtx) % 16 == 0, "descriptors are written with 16-byte stores");
static_assert(offsetof(SharedCtl, wbound) % 16 == 0, "the warps' bounds are read with 16-byte loads");
static_assert(kSmemStage % 16 == 0 && (kSmemStage + kSmemQv + kSmemQc) % 16 == 0, "queue entries and bitmaps are written with 16-byte stores");
static_assert(kSmemQv >= (size_t)kGatherCap * sizeof(u64), "a row's published candidates fit into the queues' memory");
static_assert(kWTile == 512, "a lane owns four float4 of a warp tile");
static_assert(kLaneQueue > 4, "a lane may note four cells per tile");
static_assert(kPoolCap >= kMaxK + 128, "a warp keeps its k best and still has room for the candidates of 32 cells");
static_assert(kPoolCap % 32 == 0 && kPoolCap / 32 <= 12, "a warp holds its pool in twelve registers per lane when it selects");

constexpr long long kWaitCycles = 2000000000ll;   // about 1 s: a wait that has not ended by then is reported, not continued

// How the streaming kernel works.
// The [rows][n_vocab] matrix is cut into CTA tiles of kTile logits, and every row into the same few chunks of up
// to kItemTilesMax tiles.  A work item is one chunk of one row.  The grid is one CTA per SM (or fewer, for small
// batches); CTA b starts with item b and draws further items from a counter in global memory, so that the CTAs
// finish together however unevenly the SMs are served.  Items are numbered chunk by chunk (the first chunk of
// every row, then the second, ...).
//
// The SM's instruction issue rate, not its memory bandwidth, is what the consumers have to respect: a tile is
// 32 KiB every ~0.75 us per SM at full HBM rate, which leaves sixteen warps a few hundred instructions each.  So the
// per-tile work is a handful of instructions per cell, and whatever is rare or happens once per item is kept out
// of the tile loop.
//
// A CTA has three kinds of warps, which meet only at mbarriers:
//   * the copy warp draws the items and brings their tiles into a ring of kStages shared-memory slots, one 1-D
//     bulk copy per tile, so every logit is read from HBM exactly once; it runs ahead of the consumers across item
//     borders;
//   * two set-up warps, one per hand-over slot, read the item's row descriptor and build the bitmap of the item's
//     penalised columns from the row's window ids - while the consumers work on the items before;
//   * sixteen consumer warps each own one sixteenth (512 logits) of every tile.  A lane owns four cells (float4)
//     per tile.  It takes each cell's maximum and, where that reaches the admission bound, notes the cell - its four
//     logits and its first token id - in a queue only this lane writes: a compare, two predicated stores and a
//     predicated increment, no branch.  The bound is the smallest, over the warps, of the r-th largest of a warp's
//     32 lane maxima (r = ceil(k / 16)): at least k logits of the item reach it.  It is set at the item's first
//     tile and refreshed at tiles 1, 2, 4 without a barrier; a later chunk of a row starts from the bound the row's
//     earlier chunks have left in global memory.  A warp with a nearly full queue drops the cells the bound has
//     overtaken, evens the rest out over its lanes, and only if that is not enough (rows of equal values, masked
//     stretches) moves their logits to an overflow pool in global memory, of which it keeps exactly its k best -
//     ties by token id.
// At the end of an item the logits of the noted cells that reach the final bound are written, unordered, into
// the item's slot of the row's scratch, and a ticket is drawn for the row.  The ticket's value is looked at one
// item later (its round trip to L2 overlaps the next item): the CTA that drew the row's last ticket gathers the
// row's candidates, selects the k best (a histogram over the candidates' keys, then ranks by counting), and runs
// the epilogue.  No CTA ever waits for another CTA; waits for this CTA's own copies and hand-overs are bounded.

// The shared memory of a CTA.
struct Smem {
    float* stage;       // [kStages][kTile] ring of CTA tiles
    float4* qv;         // [kLaneQueue][kThreads] noted cells; the gathered candidates of a row while it is finished
    int* qc;            // [kLaneQueue][kThreads] token id of a noted cell's first logit
    unsigned* bitmap;   // [2][kItemBitmapWords]
    u64* list;          // [kListCap] candidates about to be ordered
    u64* sorted;        // [kMaxK] the k best, in order
    double* work;       // [2 * kMaxK] the epilogue's arrays
    unsigned* hist;     // [256]
    SharedCtl* ctl;
};
__device__ __forceinline__ Smem smem_view() {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Smem m;
    unsigned char* p = smem_raw;
    m.stage = reinterpret_cast<float*>(p);
    p += kSmemStage;
    m.qv = reinterpret_cast<float4*>(p);
    p += kSmemQv;
    m.qc = reinterpret_cast<int*>(p);
    p += kSmemQc;
    m.bitmap = reinterpret_cast<unsigned*>(p);
    p += kSmemBitmap;
    m.list = reinterpret_cast<u64*>(p);
    p += kSmemList;
    m.sorted = reinterpret_cast<u64*>(p);
    p += kSmemSorted;
    m.work = reinterpret_cast<double*>(p);
    p += kSmemWork;
    m.hist = reinterpret_cast<unsigned*>(p);
    p += kSmemHist;
    m.ctl = reinterpret_cast<SharedCtl*>(p);
    return m;
}

// Waits for a barrier phase, for about a second at most (much less once some wait of this CTA has run out).
__device__ __forceinline__ bool mbar_wait_bounded(u64* bar, unsigned parity, SharedCtl* ctl) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long lim = *reinterpret_cast<volatile int*>(&ctl->abort) ? 2000ll : kWaitCycles;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity))
        if (clock64() - t0 > lim) return false;
    return true;
}
__device__ __forceinline__ void report_timeout(SharedCtl* ctl, unsigned* status) {
    *reinterpret_cast<volatile int*>(&ctl->abort) = 1;
    atomicOr(status, kStatusCopyTimeout);
}

// Final-logit softcap over a warp tile, in place (src/model_gemma4.cpp:521).  Only the softcap build calls it.
__device__ __noinline__ void softcap_tile(float* st, int len, float cap, float* wb) {
    for (int e = threadIdx.x & 31; e < len; e += 32) {
        const float y = __fmul_rn(cap, tanhf(__fdiv_rn(st[e], cap)));
        st[e] = y;
        if (wb) wb[e] = y;
    }
    __syncwarp();
}

// Repetition penalty on the penalised columns of a warp tile, in place in shared memory (src/sampler.cpp:17).
// The tile's bits of the item's bitmap are one word per 32 columns; each of the first lanes owns one word and
// patches the columns whose bits are set.  A bit is set once however often an id occurs in the window.
__device__ __forceinline__ void patch_tile(float* st, int len, int col0, int item_lo, float pen, const unsigned* bitmap, float* wb_row) {
    const int lane = threadIdx.x & 31;
    const int nw = (len + 31) >> 5;
    unsigned w = (lane < nw) ? bitmap[((col0 - item_lo) >> 5) + lane] : 0u;
    if (__ballot_sync(0xffffffffu, w != 0u) == 0u) return;
    while (w) {
        const int off = 32 * lane + __ffs(w) - 1;
        w &= w - 1u;
        const float x = st[off];
        const float y = x > 0.0f ? __fdiv_rn(x, pen) : __fmul_rn(x, pen);
        st[off] = y;
        if (wb_row) wb_row[col0 + off] = y;
    }
    __syncwarp();
}

// A bound that at least r = min(32, ceil(k / warps)) logits of this warp's stream reach: the r-th largest of the
// lanes' running maxima (each is a logit of its own) - r rounds of a warp-wide maximum, the holder drops out.
__device__ __forceinline__ float warp_bound(float run_max, int k) {
    const int r = min(32, (k + kWarps - 1) / kWarps);
    const unsigned lane = threadIdx.x & 31;
    unsigned key = float_key(run_max), m = 0u;
#pragma unroll 1
    for (int j = 0; j < r; ++j) {
        m = __reduce_max_sync(0xffffffffu, key);
        const unsigned holders = __ballot_sync(0xffffffffu, key == m);
        if (lane == (unsigned)__ffs(holders) - 1u) key = 0u;   // below the key of every float
    }
    return key_float(m);
}

// Admission bound of the CTA: at least k logits of the item reach the smallest of the warps' bounds (sixteen
// warps, at least ceil(k / 16) logits each, or 32 * 16 >= kMaxK), so no logit below it is among the item's k
// best.  Each warp posts its value with the item's tag; within an item values only grow, so a reader may use
// another warp's older value without a barrier - but only values of the same item: until every warp has posted
// for this item there is no bound (-inf).
__device__ __forceinline__ void post_warp_bound(SharedCtl* ctl, unsigned tag, float wb) {
    if ((threadIdx.x & 31) == 0) *reinterpret_cast<volatile u64*>(&ctl->wbound[threadIdx.x >> 5]) = ((u64)tag << 32) | (u64)__float_as_uint(wb);
}
__device__ __forceinline__ float min_warp_bounds(SharedCtl* ctl, unsigned tag) {
    float m = __int_as_float(0x7f800000);
    bool all = true;
#pragma unroll
    for (int w = 0; w < kWarps; w += 2) {
        u64 a, b;   // volatile: re-read on every call
        asm volatile("ld.volatile.shared.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "r"(smem_u32(&ctl->wbound[w])));
        all = all && (unsigned)(a >> 32) == tag && (unsigned)(b >> 32) == tag;
        m = fminf(m, fminf(__uint_as_float((unsigned)a), __uint_as_float((unsigned)b)));
    }
    return all ? m : -__int_as_float(0x7f800000);
}

// Diagnostics: time stamps of CTA phases (see fsb_set_trace_buffer).
__device__ __forceinline__ void trace_mark(const StreamArgs& a, int slot) {
    if (a.trace && threadIdx.x == 0) a.trace[(size_t)blockIdx.x * 16 + slot] = global_timer_ns();
}
#define TR(n)                                                                                              \
    do {                                                                                               \
        if (a.trace && blockIdx.x == 0 && threadIdx.x == 0) a.trace[148 * 16 + (n)] = (u64)clock64();   \
    } while (0)
__device__ __forceinline__ void trace_add(const StreamArgs& a, int slot, u64 v) {
    if (a.trace && threadIdx.x == 0) a.trace[(size_t)blockIdx.x * 16 + slot] += v;
}

// ---- noting a cell -----------------------------------------------------------------------------------------------
// Notes a cell in this lane's queue if its maximum reaches the bound: a compare, two address computations, two
// predicated stores and a predicated increment - no branch.  `qv_base` / `qc_base` are the shared-memory addresses
// of the lane's entry 0; entries of one lane are kThreads entries apart.
__device__ __forceinline__ void note_cell_if(const float4 x, float mx, float thr, int id0, unsigned qv_base, unsigned qc_base, int& qn) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .u32 av, ac;\n\t"
        "setp.ge.f32 p, %1, %2;\n\t"
        "mad.lo.u32 av, %0, %10, %3;\n\t"
        "mad.lo.u32 ac, %0, %11, %4;\n\t"
        "@p st.shared.v4.f32 [av], {%5, %6, %7, %8};\n\t"
        "@p st.shared.u32 [ac], %9;\n\t"
        "@p add.s32 %0, %0, 1;\n\t}"
        : "+r"(qn)
        : "f"(mx), "f"(thr), "r"(qv_base), "r"(qc_base), "f"(x.x), "f"(x.y), "f"(x.z), "f"(x.w), "r"(id0), "n"(kThreads * 16), "n"(kThreads * 4)
        : "memory");
}

// ---- a warp's overflow pool (global memory; hostile data only) ------------------------------------------------------
// Keeps the entries of the warp's pool that are >= floor_c, in place and in order; returns their number.
__device__ __forceinline__ int filter_pool(u64* pool, int n, u64 floor_c) {
    const int lane = threadIdx.x & 31;
    const unsigned lt = (1u << lane) - 1u;
    int w = 0;
    for (int i0 = 0; i0 < n; i0 += 32) {
        const int i = i0 + lane;
        const u64 c = i < n ? pool[i] : 0ull;
        const bool keep = i < n && c >= floor_c;
        const unsigned bm = __ballot_sync(0xffffffffu, keep);   // every lane has read its entry by now
        if (keep) pool[w + __popc(bm & lt)] = c;
        w += __popc(bm);
    }
    __syncwarp();
    return w;
}

// The k-th largest of the n > k distinct composites of the warp's pool: exactly k entries are >= the result.
__device__ __forceinline__ u64 warp_kth_largest(const u64* pool, int n, int k) {
    const int lane = threadIdx.x & 31;
    u64 v[kPoolCap / 32];
    u64 mn = ~0ull, mx = 0ull;
#pragma unroll
    for (int j = 0; j < kPoolCap / 32; ++j) {
        const int i = lane + 32 * j;
        v[j] = i < n ? pool[i] : 0ull;
        if (i < n) {
            mn = min(mn, v[j]);
            mx = max(mx, v[j]);
        }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if (mx == mn) return mn;
    const int hb = 63 - __clzll((long long)(mx ^ mn));
    u64 pfx = (hb == 63) ? 0ull : (mx & (~0ull << (hb + 1)));
#pragma unroll 1
    for (int b = hb; b >= 0; --b) {
        const u64 trial = pfx | (1ull << b);
        int c = 0;
#pragma unroll
        for (int j = 0; j < kPoolCap / 32; ++j) c += v[j] >= trial ? 1 : 0;   // empty slots hold 0, trial is never 0
        const int total = __reduce_add_sync(0xffffffffu, c);
        if (total >= k) pfx = trial;
        if (total == k) break;
    }
    return pfx;
}

// What a warp carries through an item: cells in this lane's queue; and, the same in every lane, the value bound, the
// composite bound its pool's entries passed (0: none) and the number of pool entries.
struct WarpState {
    int qn;
    float thr;
    u64 wcomp;
    int pn;
};

// Makes room in a pool that is nearly full: drop what the bound has overtaken; if the pool is still too full, keep
// exactly the warp's k best - no logit of this warp's stream below the k-th of them can be among the item's k best.
__device__ __forceinline__ void compact_pool(u64* pool, WarpState& st, int k, int pool_cap) {
    st.pn = filter_pool(pool, st.pn, max(comp_floor_of(st.thr), st.wcomp));
    if (st.pn > pool_cap - 128) {
        const u64 L = warp_kth_largest(pool, st.pn, k);
        st.pn = filter_pool(pool, st.pn, L);
        st.wcomp = max(st.wcomp, L);
        st.thr = fmaxf(st.thr, comp_floor_value(L));
    }
}

// Moves the logits of this warp's noted cells that reach the bounds into the warp's pool; the queues are empty after.
__device__ __forceinline__ void flush_queues_to_pool(const Smem& m, u64* pool, WarpState& st, int k, int pool_cap) {
    const int tid = threadIdx.x, lane = tid & 31;
    const unsigned lt = (1u << lane) - 1u;
    pdl_wait_prior();   // the pools are the engine's: the previous launch in the stream may still be using them
    const int rounds = __reduce_max_sync(0xffffffffu, st.qn);
    for (int j = 0; j < rounds; ++j) {
        if (st.pn > pool_cap - 128) compact_pool(pool, st, k, pool_cap);
        const bool have = j < st.qn;
        const float4 v = have ? m.qv[j * kThreads + tid] : make_float4(0.f, 0.f, 0.f, 0.f);
        const int id0 = have ? m.qc[j * kThreads + tid] : 0;
        const float xs[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const u64 c = make_comp(xs[e], id0 + e);
            const bool ok = have && xs[e] >= st.thr && c >= st.wcomp;
            const unsigned be = __ballot_sync(0xffffffffu, ok);
            if (ok) pool[st.pn + __popc(be & lt)] = c;
            st.pn += __popc(be);
        }
    }
    __syncwarp();
    st.qn = 0;
}

// A lane's queue is nearly full.  The warp refreshes its bound and drops the noted cells it has overtaken; if a lane
// is still short of room, the cells are evened out over the warp's lanes (a cell carries its token id, so any lane
// may hold it); and if the warp holds more live cells than that leaves room for, their logits move to the pool.
__device__ __noinline__ WarpState make_room(WarpState st, int k, unsigned tag, u64* pool, int pool_cap) {
    const Smem m = smem_view();
    const int tid = threadIdx.x, lane = tid & 31;
    const unsigned lt = (1u << lane) - 1u;
    st.thr = fmaxf(st.thr, min_warp_bounds(m.ctl, tag));
    int w = 0;
    for (int i = 0; i < st.qn; ++i) {
        const float4 v = m.qv[i * kThreads + tid];
        if (fmaxf(max3(v.x, v.y, v.z), v.w) >= st.thr) {
            if (w != i) {
                m.qv[w * kThreads + tid] = v;
                m.qc[w * kThreads + tid] = m.qc[i * kThreads + tid];
            }
            ++w;
        }
    }
    st.qn = w;
    if (!__any_sync(0xffffffffu, st.qn > kLaneQueue - 4)) return st;
    const int wbase = tid & ~31;
    int total = 0;
    for (int j = 0; j < kLaneQueue; ++j) {
        const bool have = j < st.qn;
        const float4 v = have ? m.qv[j * kThreads + tid] : make_float4(0.f, 0.f, 0.f, 0.f);
        const int c = have ? m.qc[j * kThreads + tid] : 0;
        const unsigned bm = __ballot_sync(0xffffffffu, have);   // every lane has read its entry j by now
        if (have) {
            const int p = total + __popc(bm & lt);   // p < 32 * (j + 1): the target row is at most j
            m.qv[(p >> 5) * kThreads + wbase + (p & 31)] = v;
            m.qc[(p >> 5) * kThreads + wbase + (p & 31)] = c;
        }
        total += __popc(bm);
        __syncwarp();
    }
    st.qn = total > lane ? (total - lane + 31) >> 5 : 0;
    if (total > 32 * (kLaneQueue - 4)) flush_queues_to_pool(m, pool, st, k, pool_cap);
    return st;
}

// ---- selection and order of a row's candidates ----------------------------------------------------------------------
// The candidates lie in `buf` (shared memory) in n_parts parts, part c at buf + c * stride with ctl->wcount[c]
// entries, unordered, `total` in all.  Orders the k best into m.sorted and returns their number.  Few candidates are
// ranked by counting right away; otherwise a 256-bucket histogram over the range of their value keys finds the
// bucket the k-th lies in, and only the candidates from that bucket up (k and a few more, as a rule) are ranked.
// All consumer threads must call, after a barrier that made buf and the counts visible.
__device__ __forceinline__ int select_and_order(const StreamArgs& a, const Smem& m, const u64* buf, int n_parts, int stride, int total, int k) {
    SharedCtl* ctl = m.ctl;
    const int tid = threadIdx.x, lane = tid & 31;
    if (total <= 0) return 0;
    int n = total;
    // where the candidates that are ranked go: the list - or, when they come from the list, the epilogue's arrays
    u64* rk = buf == m.list ? reinterpret_cast<u64*>(m.work) : m.list;
    static_assert(kSmemWork >= kSmemList, "the epilogue's arrays can hold a list");
    if (buf == m.list && total <= 160) {
        rk = m.list;   // ranked where they lie
    } else if (total <= 160) {
        // (the parts are copied into the list one after the other)
        int at = 0;
        for (int c = 0; c < n_parts; ++c) {
            const int cnt = ctl->wcount[c];
            for (int i = tid; i < cnt; i += kThreads) rk[at + i] = buf[(size_t)c * stride + i];
            at += cnt;
        }
        consumer_sync();
    } else {
        unsigned kmn = 0xFFFFFFFFu, kmx = 0u;
        for (int c = 0; c < n_parts; ++c) {
            const int cnt = ctl->wcount[c];
            for (int i = tid; i < cnt; i += kThreads) {
                const unsigned key = (unsigned)(buf[(size_t)c * stride + i] >> 32);
                kmn = min(kmn, key);
                kmx = max(kmx, key);
            }
        }
        u64 mn = kmn, mx = kmx;
        if (tid < 256) m.hist[tid] = 0u;
        if (tid == 0) ctl->n_el = 0;
        TR(13);
        cta_minmax(mn, mx, ctl);   // two barriers
        TR(14);
        kmn = (unsigned)mn;
        kmx = (unsigned)mx;
        const unsigned range = kmx - kmn;
        const int sh = range >= 256u ? (32 - __clz(range)) - 8 : 0;
        for (int c = 0; c < n_parts; ++c) {
            const int cnt = ctl->wcount[c];
            for (int i = tid; i < cnt; i += kThreads) atomicAdd(&m.hist[((unsigned)(buf[(size_t)c * stride + i] >> 32) - kmn) >> sh], 1u);
        }
        consumer_sync();
        TR(15);
        if (tid < 32) {   // the highest bucket b with at least min(k, total) candidates in buckets >= b
            unsigned mine = 0u, h[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                h[j] = m.hist[8 * lane + j];
                mine += h[j];
            }
            unsigned above = mine;   // candidates in this lane's buckets and all higher ones
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned t = __shfl_down_sync(0xffffffffu, above, o);
                if (lane + o < 32) above += t;
            }
            const unsigned want = (unsigned)min(k, total);
            const unsigned ok = __ballot_sync(0xffffffffu, above >= want);
            const int sel = 31 - __clz(ok);   // lane 0 always qualifies
            if (lane == sel) {
                unsigned run = above - mine;
                int b = 8 * lane + 7;
                for (; b > 8 * lane; --b) {
                    if (run + h[b - 8 * lane] >= want) break;
                    run += h[b - 8 * lane];
                }
                ctl->bsel = b;
                ctl->nsel = (int)(run + h[b - 8 * lane]);
            }
        }
        consumer_sync();
        TR(16);
        const unsigned bsel = (unsigned)ctl->bsel;
        n = ctl->nsel;
        if (n > kListCap) {
            // many equal values around the k-th: the exact selection by bisection, over a flat copy of the candidates
            // (the parts are moved together first; a part never moves past its own start)
            u64* flat = const_cast<u64*>(buf);
            int at = 0;
            for (int c = 0; c < n_parts; ++c) {
                const int cnt = ctl->wcount[c];
                for (int i0 = 0; i0 < cnt; i0 += kThreads) {
                    const int i = i0 + tid;
                    const u64 v = i < cnt ? buf[(size_t)c * stride + i] : 0ull;
                    consumer_sync();
                    if (i < cnt) flat[at + i] = v;
                    consumer_sync();
                }
                at += cnt;
            }
            n = select_list_topk(flat, total, k, m.sorted, ctl);
            rk = flat;
        } else {
            for (int c = 0; c < n_parts; ++c) {
                const int cnt = ctl->wcount[c];
                for (int i0 = 0; i0 < cnt; i0 += kThreads) {
                    const int i = i0 + tid;
                    u64 v = 0ull;
                    bool take = false;
                    if (i < cnt) {
                        v = buf[(size_t)c * stride + i];
                        take = (((unsigned)(v >> 32) - kmn) >> sh) >= bsel;
                    }
                    const unsigned bm = __ballot_sync(0xffffffffu, take);
                    int base = 0;
                    if (lane == 0 && bm) base = atomicAdd(&ctl->n_el, __popc(bm));
                    base = __shfl_sync(0xffffffffu, base, 0);
                    if (take) rk[base + __popc(bm & ((1u << lane) - 1u))] = v;
                }
            }
            consumer_sync();
        }
        if (tid == 0) ctl->n_el = 0;
        TR(17);
        if (a.trace && blockIdx.x == 0 && threadIdx.x == 0) a.trace[148 * 16 + 41] = (u64)n | ((u64)total << 32);
    }
    return topk_sorted(rk, n, k, m.sorted, ctl);
}

// ---- the copy warp --------------------------------------------------------------------------------------------
// One lane draws the work items (the first is the CTA's own number, the others come from the counter in global
// memory, fetched one item ahead), posts each item's place in the matrix to the set-up warp of its slot, and brings
// the item's tiles in, one 1-D bulk copy per tile (large copies: the copy engine's cost is per request), into a
// ring of kStages slots.  A slot is refilled once all consumer warps have handed it back.
__device__ __forceinline__ void copy_loop(const StreamArgs& a, const Smem& m) {
    if ((threadIdx.x & 31) != 0) return;
    SharedCtl* ctl = m.ctl;
    const int V = a.n_vocab;
    int next_idx = (int)blockIdx.x;
    bool waited = !a.overlap;   // without launch overlap there is nothing to wait for
    int it = 0, seq = 0;
    bool ok = true;
    for (;; ++seq) {
        const int b = seq & 1;
        ItemCtx* ic = &ctl->item[b];
        // the slot is free once the consumers have looked at the last tile of the item two before
        if (seq >= 2 && !mbar_wait_bounded(&ctl->item_free[b], (unsigned)(((seq >> 1) - 1) & 1), ctl)) ok = false;
        const int idx = next_idx;
        if (!ok || idx >= a.n_items || *reinterpret_cast<volatile int*>(&ctl->abort)) break;
        const int chunk = idx / a.n_rows, row = idx - chunk * a.n_rows;
        int tile0 = 0;
        for (int c = 0; c < chunk; ++c) tile0 += a.chunk_len[c];
        const int nt = a.chunk_len[chunk];
        const float* row_ptr = a.logits + (a.row_ld >= 0 ? (int64_t)row * a.row_ld : a.rows[row].logits_off);
        ic->done = 0;
        ic->row = row;
        ic->chunk = chunk;
        ic->tile0 = tile0;
        ic->ntiles = nt;
        ic->row_ptr = row_ptr;
        mbar_arrive(&ctl->item_posted[b]);   // the slot's set-up warp may start
        // the next item's number: the round trip to the counter overlaps this item's copies
        if (!waited) {
            pdl_wait_prior();   // the counter belongs to the previous launch until that is complete
            waited = true;
        }
        next_idx = (int)gridDim.x + (int)atomicAdd(a.work, 1u);
        if (!a.bulk_ok) continue;   // rows not on 16-byte boundaries: the consumers load their tiles themselves
        for (int j = 0; j < nt && ok; ++j, ++it) {
            const int slot = it % kStages;
            // the first kStages tiles find their slots free; later ones wait for the consumers' hand-back
            if (it >= kStages && !mbar_wait_bounded(&ctl->empty[slot], (unsigned)((it / kStages - 1) & 1), ctl)) {
                ok = false;
                break;
            }
            const int col0 = (tile0 + j) * kTile;
            const int len = min(kTile, V - col0);   // >= 1
            const float* src = row_ptr + col0;
            float* dst = m.stage + (size_t)slot * kTile;
            const unsigned bytes = (unsigned)(len & ~3) * 4u;
            for (int e = len & ~3; e < len; ++e) dst[e] = src[e];   // ragged tail by plain loads
            if (bytes) {
                fence_proxy_async_smem();   // generic-proxy accesses to this slot (the consumers' patches) precede the async write
                mbar_expect_tx(&ctl->full[slot], bytes);
                bulk_g2s(dst, src, bytes, &ctl->full[slot]);
            } else {
                mbar_arrive(&ctl->full[slot]);
            }
        }
        if (!ok) {
            ++seq;
            break;
        }
    }
    if (!ok) report_timeout(ctl, a.status);
    // no more work: both slots say so (the consumers stop at the first, the other releases its set-up warp)
    for (int e = 0; e < 2; ++e, ++seq) {
        const int b = seq & 1;
        if (e == 1 && seq >= 2) mbar_wait_bounded(&ctl->item_free[b], (unsigned)(((seq >> 1) - 1) & 1), ctl);
        ctl->item[b].done = 1;
        mbar_arrive(&ctl->item_posted[b]);
    }
    // the CTA that leaves last puts the counters back for the next launch (every CTA has drawn its last number)
    if (!waited) pdl_wait_prior();
    if (ticket_add_acq_rel(a.work + 1, 1u) == gridDim.x - 1u) {
        a.work[0] = 0u;
        a.work[1] = 0u;
    }
}

// ---- the set-up warps -----------------------------------------------------------------------------------------
// Warp `b` serves hand-over slot b (items 0, 2, 4, ... or 1, 3, 5, ... of the CTA): once the copy warp has posted
// the item, it reads the row's descriptor and the bound the row's earlier chunks have left, builds the bitmap of
// the item's penalised columns, and hands the item to the consumers.
__device__ __forceinline__ void setup_loop(const StreamArgs& a, const Smem& m, int b) {
    SharedCtl* ctl = m.ctl;
    const int lane = threadIdx.x & 31;
    ItemCtx* ic = &ctl->item[b];
    unsigned* bm = m.bitmap + (size_t)b * kItemBitmapWords;
    for (int n = 0;; ++n) {
        const bool ok = mbar_wait_bounded(&ctl->item_posted[b], (unsigned)(n & 1), ctl);
        if (!ok && lane == 0) report_timeout(ctl, a.status);
        if (!ok || ic->done) {
            if (lane == 0) {
                ic->done = 1;
                mbar_arrive(&ctl->item_ready[b]);
            }
            return;
        }
        const int row = ic->row, tile0 = ic->tile0, nt = ic->ntiles;
        // the row's descriptor (four lanes, 16 bytes each) and the row's bound, all loads in flight together.  The bound
        // is not read by the first item of a launch that overlaps its predecessor (which resets it when it completes).
        uint4 dq = make_uint4(0u, 0u, 0u, 0u);
        unsigned key = 0u;
        if (lane < 4) dq = __ldg(reinterpret_cast<const uint4*>(a.rows + row) + lane);
        if (lane == 4 && a.n_chunks > 1 && (!a.overlap || n > 0 || b > 0)) key = __ldcg(a.row_bound + row);
        if (lane < 4) reinterpret_cast<uint4*>(&ic->d)[lane] = dq;
        if (lane == 4) ic->thr0 = key ? key_float(key) : -__int_as_float(0x7f800000);
        __syncwarp();
        const RowDesc& d = ic->d;
        if (d.flags & kRowPenalty) {
            const int lo = tile0 * kTile, hi = min(a.n_vocab, (tile0 + nt) * kTile);
            const int32_t* h = a.hist + d.hist_begin;
            const int nh = d.hist_len;
            int c[16];   // the first 512 window ids: loads issued before the bitmap is cleared
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const int i = 32 * u + lane;
                c[u] = i < nh ? __ldg(h + i) - a.vocab_offset : -1;
            }
            const int words4 = ((hi - lo + 31) / 32 + 3) / 4;
            for (int i = lane; i < words4; i += 32) reinterpret_cast<uint4*>(bm)[i] = make_uint4(0u, 0u, 0u, 0u);
            __syncwarp();
#pragma unroll
            for (int u = 0; u < 16; ++u)
                if (c[u] >= lo && c[u] < hi) atomicOr(&bm[(c[u] - lo) >> 5], 1u << ((c[u] - lo) & 31));
            for (int i0 = 512; i0 < nh; i0 += 512) {
#pragma unroll
                for (int u = 0; u < 16; ++u) {
                    const int i = i0 + 32 * u + lane;
                    c[u] = i < nh ? __ldg(h + i) - a.vocab_offset : -1;
                }
#pragma unroll
                for (int u = 0; u < 16; ++u)
                    if (c[u] >= lo && c[u] < hi) atomicOr(&bm[(c[u] - lo) >> 5], 1u << ((c[u] - lo) & 31));
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->item_ready[b]);   // releases the warp's writes to the waiting consumers
    }
}

// ---- the end of a row -----------------------------------------------------------------------------------------
// What the consumers carry from one item's end to the next: the row whose ticket is on its way (-1: none) and,
// in thread 0 only, the ticket.
struct Pending {
    int row;
    unsigned ticket;
};

// Orders the row's candidates (see select_and_order) and runs the epilogue.  All consumer threads call.
__device__ __forceinline__ void finish_row(const StreamArgs& a, const Smem& m, const u64* buf, int n_parts, int stride, int total, const RowDesc& d) {
    const int kk = select_and_order(a, m, buf, n_parts, stride, total, d.k);
    TR(20);
    trace_mark(a, 8);
    const TailOut tout{a.tokens, a.kept_ids, a.kept_pr, a.kept_n, reinterpret_cast<u64*>(a.shard_out), a.shard_n, a.status};
    const RowTail rt{d.rng_word, d.temperature, d.top_p, d.min_p, d.k, d.flags, d.out_index, a.scan_sums};
    row_epilogue(m.sorted, kk, rt, m.work, tout);
    TR(21);
    trace_mark(a, 9);
    consumer_sync();   // the list, the ordered candidates and the gathered candidates may be written again
    TR(22);
}

// The ticket of the row in `pend` has had an item's time to arrive: if it was the row's last, all chunks of the row
// have published, and this CTA gathers their candidates and finishes the row.  All consumer threads call, between
// items (the lanes' queues are empty then: the gathered candidates take their memory).
__device__ __forceinline__ void resolve_pending(const StreamArgs& a, const Smem& m, Pending& pend, const RowDesc* desc) {
    SharedCtl* ctl = m.ctl;
    const int tid = threadIdx.x;
    const int row = pend.row;
    if (row < 0) return;
    if (tid == 0) ctl->last = (pend.ticket == (unsigned)(a.n_chunks - 1)) ? 1 : 0;
    pend.row = -1;
    consumer_sync();
    if (!ctl->last) return;
    TR(10);
    trace_mark(a, 7);
    const RowDesc d = *desc;
    const int nl = a.n_chunks, cap = a.slot_cap;
    const u64* src = reinterpret_cast<const u64*>(a.scratch) + (size_t)row * (size_t)a.scratch_stride;
    if (tid == 0) {
        a.ticket[row] = 0u;   // ready for the next launch
        a.row_bound[row] = 0u;
    }
    // Slots and counts are read in one go (L2 reads, never L1): what lies past a slot's count is stale and never looked at.
    u64* gathered = reinterpret_cast<u64*>(m.qv);
    const int span = nl * cap;
    for (int e = tid; e < span; e += kThreads) gathered[e] = __ldcg(src + e);
    if (tid < nl) ctl->wcount[tid] = min((int)__ldcg(src + a.scratch_stride - 1 - tid), cap);
    TR(11);
    consumer_sync();
    TR(12);
    int total = 0;
    for (int c = 0; c < nl; ++c) total += ctl->wcount[c];
    finish_row(a, m, gathered, nl, cap, total, d);
}

// ---- the end of an item ---------------------------------------------------------------------------------------
// More candidates than the item's slot holds have reached the final bound (many equal values): every warp moves its
// noted cells' logits to its pool and keeps its k best, the CTA finds the k-th largest over all pools by bisection,
// and exactly the k best are written.  All consumer threads call; returns the number written.
__device__ __noinline__ int overflow_exact(WarpState st, u64* pool, int pool_cap, int k, u64* dst) {
    const Smem m = smem_view();
    SharedCtl* ctl = m.ctl;
    const int tid = threadIdx.x, lane = tid & 31;
    flush_queues_to_pool(m, pool, st, k, pool_cap);
    compact_pool(pool, st, k, pool_cap);
    if (st.pn > k) {   // the warp's k best are all the item can need from it
        const u64 L = warp_kth_largest(pool, st.pn, k);
        st.pn = filter_pool(pool, st.pn, L);
    }
    u64 v[kPoolCap / 32];
    u64 mn = ~0ull, mx = 0ull;
    int mine = 0;
#pragma unroll
    for (int j = 0; j < kPoolCap / 32; ++j) {
        const int i = lane + 32 * j;
        v[j] = i < st.pn ? pool[i] : 0ull;
        if (i < st.pn) {
            mn = min(mn, v[j]);
            mx = max(mx, v[j]);
            ++mine;
        }
    }
    if (tid == 0) ctl->sum[0] = 0;
    cta_minmax(mn, mx, ctl);
    const int wsum = __reduce_add_sync(0xffffffffu, mine);
    if (lane == 0 && wsum) atomicAdd(&ctl->sum[0], wsum);
    consumer_sync();
    const int total = ctl->sum[0];
    consumer_sync();
    u64 L = 0ull;
    if (total > k)
        L = bisect_bound(k, mn, mx, ctl, [&](u64 t) {
            int c = 0;
#pragma unroll
            for (int j = 0; j < kPoolCap / 32; ++j) c += v[j] >= t ? 1 : 0;
            return c;
        });
    if (tid == 0) ctl->n_el = 0;
    consumer_sync();
    st.pn = filter_pool(pool, st.pn, L);
    int base = 0;
    if (lane == 0 && st.pn) base = atomicAdd(&ctl->n_el, st.pn);
    base = __shfl_sync(0xffffffffu, base, 0);
    for (int i = lane; i < st.pn; i += 32) dst[base + i] = pool[i];   // k entries at most in all: they fit every slot
    consumer_sync();
    return ctl->n_el;
}

// All consumer threads call it once they have looked at the item's last tile: the final bound; the logits of the
// noted cells (and of the overflow pool, if it was used) that reach it are written - unordered - to the item's slot
// of the row's scratch and a ticket is drawn, whose value the next call looks at; a row that is a single chunk is
// finished right away.
__device__ __forceinline__ void item_end(const StreamArgs& a, const Smem& m, u64* pool, WarpState st, float run_max, int row, int chunk,
                                         unsigned tag, Pending& pend) {
    SharedCtl* ctl = m.ctl;
    const int tid = threadIdx.x, lane = tid & 31;
    const int k = ctl->cur.k;
    const bool single = a.n_chunks == 1;
    TR(0);
    post_warp_bound(ctl, tag, warp_bound(run_max, k));
    TR(1);
    consumer_sync();
    TR(2);
    st.thr = fmaxf(st.thr, min_warp_bounds(ctl, tag));
    TR(3);
    pdl_wait_prior();   // from here on this launch writes what the previous launch in the stream may still be using
    u64* dst = single ? m.list : reinterpret_cast<u64*>(a.scratch) + (size_t)row * (size_t)a.scratch_stride + (size_t)chunk * a.slot_cap;
    const int cap = single ? kListCap : a.slot_cap;
    // one noted cell per lane and round: the logits that reach the bounds are counted, the warp reserves room for them
    // with one shared-memory atomic, and every lane writes its own
    const int rounds = __reduce_max_sync(0xffffffffu, st.qn);
    for (int j = 0; j < rounds; ++j) {
        unsigned mask = 0u;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        int id0 = 0;
        if (j < st.qn) {
            v = m.qv[j * kThreads + tid];
            id0 = m.qc[j * kThreads + tid];
            const float xs[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (xs[e] >= st.thr && (st.wcomp == 0ull || make_comp(xs[e], id0 + e) >= st.wcomp)) mask |= 1u << e;
        }
        const int cnt = __popc(mask);
        int inc = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += t;
        }
        const int wtotal = __shfl_sync(0xffffffffu, inc, 31);
        if (wtotal == 0) continue;
        int base = 0;
        if (lane == 31) base = atomicAdd(&ctl->n_el, wtotal);
        base = __shfl_sync(0xffffffffu, base, 31);
        int p = base + inc - cnt;
        const float xs[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
            if (mask & (1u << e)) {
                if (p < cap) dst[p] = make_comp(xs[e], id0 + e);
                ++p;
            }
    }
    TR(4);
    if (st.pn > 0) {
        st.pn = filter_pool(pool, st.pn, max(comp_floor_of(st.thr), st.wcomp));
        int base = 0;
        if (lane == 0 && st.pn) base = atomicAdd(&ctl->n_el, st.pn);
        base = __shfl_sync(0xffffffffu, base, 0);
        for (int i = lane; i < st.pn; i += 32)
            if (base + i < cap) dst[base + i] = pool[i];
    }
    consumer_sync();
    TR(5);
    int n_el = ctl->n_el;
    if (n_el > cap) n_el = overflow_exact(st, pool, a.pool_cap, k, dst);
    trace_mark(a, 5);
    if (a.trace && blockIdx.x == 0 && threadIdx.x == 0) a.trace[148 * 16 + 40] = (u64)n_el | ((u64)rounds << 32);
    if (!single) {
        if (tid == 0) {
            ctl->n_el = 0;   // for the next item (barriers follow)
            u64* rowp = reinterpret_cast<u64*>(a.scratch) + (size_t)row * (size_t)a.scratch_stride;
            rowp[a.scratch_stride - 1 - chunk] = (u64)n_el;
            atomicMax(a.row_bound + row, float_key(st.thr));   // at least k logits of the row reach this item's final bound
        }
        consumer_sync();   // orders the CTA's stores before the ticket, whose release publishes them to the device
        TR(6);
        // the ticket drawn at the end of the item before has had this item's time to arrive
        Pending prev = pend;
        if (tid == 0) pend.ticket = ticket_add_acq_rel(a.ticket + row, 1u);   // not looked at before the next item's end
        pend.row = row;
        TR(7);
        resolve_pending(a, m, prev, &ctl->prev);
        if (tid == 0) ctl->prev = ctl->cur;
        TR(8);
        trace_mark(a, 6);
    } else {
        if (tid == 0) {
            ctl->n_el = 0;
            ctl->wcount[0] = n_el;
        }
        consumer_sync();
        finish_row(a, m, m.list, 1, 0, n_el, ctl->cur);
    }
}

template <bool SOFTCAP>
__global__ void __launch_bounds__(kBlockThreads, 1) stream_select_kernel(const __grid_constant__ StreamArgs a) {
    const Smem m = smem_view();
    SharedCtl* ctl = m.ctl;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int V = a.n_vocab;
    // With launch overlap on, the next launch in the stream may start as soon as this one leaves room; like this one
    // it waits for its predecessor before it writes anything or draws from the work counter, so only the reading of
    // a CTA's first item overlaps.
    pdl_launch_dependents();
    if (tid == 0) {   // one thread initialises every barrier, then makes the initialisation visible to the copy engine
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&ctl->full[s], 1u);                  // the copy warp's arrive (+ the copy's bytes)
            mbar_init(&ctl->empty[s], (unsigned)kWarps);   // one arrive per consumer warp
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&ctl->item_posted[b], 1u);
            mbar_init(&ctl->item_ready[b], 1u);
            mbar_init(&ctl->item_free[b], (unsigned)kWarps);
        }
        for (int w = 0; w < kWarps; ++w) ctl->wbound[w] = 0ull;
        ctl->abort = 0;
        ctl->n_el = 0;
        fence_mbar_init();
        if (a.trace) {
            for (int s = 0; s < 16; ++s) a.trace[(size_t)blockIdx.x * 16 + s] = 0ull;
            a.trace[(size_t)blockIdx.x * 16 + 0] = global_timer_ns();
        }
    }
    __syncthreads();   // the only barrier all warps take part in
    if (warp == kCopyWarp) {
        copy_loop(a, m);
        return;
    }
    if (warp > kCopyWarp) {
        setup_loop(a, m, warp - kSetupWarp0);
        return;
    }
    if (a.write_back) pdl_wait_prior();   // this launch stores into the logits while it streams

    // ------------------------------------------------------------------------------------------ consumers
    const float ninf = -__int_as_float(0x7f800000);
    u64* const pool = reinterpret_cast<u64*>(a.pools) + ((size_t)blockIdx.x * kWarps + warp) * (size_t)a.pool_cap;
    float* const st_warp = m.stage + warp * kWTile;
    const unsigned qv_base = smem_u32(m.qv + tid), qc_base = smem_u32(m.qc + tid);
    int it = 0;        // tiles of this CTA looked at so far (the position in the ring)
    int n_items = 0;
    Pending pend{-1, 0u};
    long long t_ready = 0;
    for (int seq = 0;; ++seq) {
        const int b = seq & 1;
        const unsigned tag = (unsigned)seq + 1u;
        const ItemCtx* ic = &ctl->item[b];
        const long long tr0 = a.trace ? clock64() : 0;
        if (!mbar_wait_bounded(&ctl->item_ready[b], (unsigned)((seq >> 1) & 1), ctl) && lane == 0) report_timeout(ctl, a.status);
        if (a.trace) t_ready += clock64() - tr0;
        if (tid == 0 && !ctl->abort && !ic->done) ctl->cur = ic->d;   // the end-of-item work outlives the hand-over slot
        consumer_sync();   // every warp takes the same way out
        if (*reinterpret_cast<volatile int*>(&ctl->abort) || ic->done) break;
        const int row = ic->row, chunk = ic->chunk, tile0 = ic->tile0, nt = ic->ntiles;
        const float* row_ptr = ic->row_ptr;
        float* wb_row = a.write_back ? const_cast<float*>(row_ptr) : nullptr;
        const float pen = ic->d.penalty;
        const int k = ic->d.k;
        const bool has_pen = (ic->d.flags & kRowPenalty) != 0;
        const unsigned* bitmap = m.bitmap + (size_t)b * kItemBitmapWords;
        const int item_lo = tile0 * kTile;
        const float thr0 = ic->thr0;
        WarpState st{0, thr0, 0ull, 0};
        float run_max = ninf;
        int col0 = item_lo + warp * kWTile;   // first column of this warp's part of the tile
        if (seq == 0) trace_mark(a, 1);

        for (int s = 0; s < nt; ++s, ++it, col0 += kTile) {
            const unsigned slot = (unsigned)it % kStages, par = ((unsigned)it / kStages) & 1u;
            float* stg = st_warp + slot * kTile;              // this warp's part of the CTA tile
            const int len = min(kWTile, V - col0);            // may be <= 0 in a row's last tile
            if (a.bulk_ok) {
                if (!mbar_wait_bounded(&ctl->full[slot], par, ctl) && lane == 0) report_timeout(ctl, a.status);   // carry on with what is there
            } else if (len > 0) {   // rows not on 16-byte boundaries: the warp loads its part of the tile itself
                const float* src = row_ptr + col0;
                for (int e = lane; e < len; e += 32) stg[e] = src[e];
                __syncwarp();
            }
            if (seq == 0 && s == 0) trace_mark(a, 2);
            if (SOFTCAP) {
                if (len > 0) softcap_tile(stg, len, a.softcap, wb_row ? wb_row + col0 : nullptr);
            }
            if (has_pen && len > 0 && !(a.debug & 4)) patch_tile(stg, len, col0, item_lo, pen, bitmap, wb_row);
            if (len < kWTile) {   // what lies past the end of a ragged row is made NaN: never a maximum, never reaches a bound
                for (int e = max(len, 0) + lane; e < kWTile; e += 32) stg[e] = __int_as_float(0x7fc00000);
                __syncwarp();
            }
            // ---- look: the lane's four cells go to registers (four independent 16-byte loads)
            const float4* st4 = reinterpret_cast<const float4*>(stg);
            const float4 x0 = st4[lane], x1 = st4[lane + 32], x2 = st4[lane + 64], x3 = st4[lane + 96];
            const float m0 = fmaxf(max3(x0.x, x0.y, x0.z), x0.w);
            const float m1 = fmaxf(max3(x1.x, x1.y, x1.z), x1.w);
            const float m2 = fmaxf(max3(x2.x, x2.y, x2.z), x2.w);
            const float m3 = fmaxf(max3(x3.x, x3.y, x3.z), x3.w);
            run_max = fmaxf(max3(run_max, m0, m1), fmaxf(m2, m3));
            __syncwarp();
            if (lane == 0 && a.bulk_ok) mbar_arrive(&ctl->empty[slot]);   // the slot goes back to the copy warp

            // ---- the admission bound: posted at the item's first tile - with a barrier when the row has left no bound
            // yet, so that the first tile is not admitted wholesale - and refreshed without one at tiles 1, 2, 4
            if ((s & (s - 1)) == 0) {   // s = 0, 1, 2, 4, 8, ...
                post_warp_bound(ctl, tag, warp_bound(run_max, k));
                if (s == 0 && thr0 == ninf) consumer_sync();
                else __syncwarp();
                st.thr = fmaxf(st.thr, min_warp_bounds(ctl, tag));
            }
            // ---- note the cells whose maximum reaches the bound (padding past the end of a row never does)
            if (__any_sync(0xffffffffu, st.qn > kLaneQueue - 4)) st = make_room(st, k, tag, pool, a.pool_cap);
            if (!(a.debug & 1)) {
                const int id_lane = col0 + 4 * lane + a.vocab_offset;
                note_cell_if(x0, m0, st.thr, id_lane, qv_base, qc_base, st.qn);
                note_cell_if(x1, m1, st.thr, id_lane + 128, qv_base, qc_base, st.qn);
                note_cell_if(x2, m2, st.thr, id_lane + 256, qv_base, qc_base, st.qn);
                note_cell_if(x3, m3, st.thr, id_lane + 384, qv_base, qc_base, st.qn);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->item_free[b]);   // descriptor slot and bitmap go back
        ++n_items;
        trace_mark(a, 4);
        const long long te0 = a.trace ? clock64() : 0;
        if (a.debug & 2) {
            consumer_sync();
            continue;
        }
        item_end(a, m, pool, st, run_max, row, chunk, tag, pend);
        if (a.trace) trace_add(a, 13, (u64)(clock64() - te0));
    }
    // the last ticket this CTA drew may have been its row's last
    resolve_pending(a, m, pend, &ctl->prev);
    if (a.trace && tid == 0) {
        a.trace[(size_t)blockIdx.x * 16 + 3] = (u64)n_items;
        a.trace[(size_t)blockIdx.x * 16 + 12] = (u64)t_ready;
    }
    trace_mark(a, 10);
}

// Merge of per-shard candidate lists (vocabulary-sharded mode): one CTA per row gathers n_lists sorted lists of
// up to kMaxK composites each (already in this device's memory, list g of row r at lists + (g * n_rows + r) * list_stride)
// and runs the row epilogue.
__global__ void __launch_bounds__(kThreads, 1) merge_lists_kernel(const u64* lists, const int32_t* list_n, int n_lists, int list_stride, int n_rows,
                                                                 const RowDesc* rows, int32_t* tokens, int32_t* kept_ids, double* kept_pr,
                                                                 int32_t* kept_n, unsigned* status, int scan_sums) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    u64* buf = reinterpret_cast<u64*>(smem_raw);
    u64* out = buf + kMergeCap;
    double* work = reinterpret_cast<double*>(out + kMaxK);
    SharedCtl* ctl = reinterpret_cast<SharedCtl*>(work + 2 * kMaxK);
    const int row = blockIdx.x, tid = threadIdx.x;
    if (row >= n_rows) return;
    const RowDesc d = rows[row];
    int total = 0;   // the same in every thread
    for (int g = 0; g < n_lists; ++g) {
        const int n = min(min(list_n[(size_t)g * n_rows + row], kMaxK), list_stride);
        const u64* src = lists + ((size_t)g * n_rows + row) * (size_t)list_stride;
        if (total + n <= kMergeCap) {
            for (int i = tid; i < n; i += kThreads) buf[total + i] = src[i];
            total += n;
        } else if (tid == 0) {
            atomicOr(status, kStatusMergeOverflow);
        }
    }
    consumer_sync();
    const TailOut tout{tokens, kept_ids, kept_pr, kept_n, nullptr, nullptr, status};
    const RowTail rt{d.rng_word, d.temperature, d.top_p, d.min_p, d.k_global, d.flags, d.out_index, scan_sums};
    const int kk = topk_sorted(buf, total, d.k_global, out, ctl);
    row_epilogue(out, kk, rt, work, tout);
}

// Write-back for callers whose logits live in host memory: after a launch with write-back on the device copy, the
// values at the rows' window ids (the only entries the penalty touches) are gathered, one float per window id in
// window order, so that the host can store them into the caller's rows without redoing any arithmetic.
__global__ void gather_patched_kernel(const float* logits, const RowDesc* rows, int n_rows, const int32_t* hist, int n_vocab, int vocab_offset,
                                      float* out) {
    const int row = blockIdx.x;
    if (row >= n_rows) return;
    const RowDesc d = rows[row];
    for (int i = threadIdx.x; i < d.hist_len; i += blockDim.x) {
        const int c = hist[d.hist_begin + i] - vocab_offset;
        out[d.gather_off + i] = (c >= 0 && c < n_vocab) ? logits[d.logits_off + c] : 0.0f;
    }
}

}  // namespace

size_t stream_kernel_smem_bytes() { return kSmemTotal; }

constexpr size_t kSmemMerge = (size_t)(kMergeCap + kMaxK) * sizeof(u64) + 2 * (size_t)kMaxK * sizeof(double) + sizeof(SharedCtl);

// Per-device set-up (the current device): opt in to the large dynamic shared memory; report resident CTAs per SM.
int prepare_device_kernels(int* ctas_per_sm) {
    cudaError_t e = cudaFuncSetAttribute(stream_select_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTotal);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(stream_select_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTotal);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(merge_lists_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemMerge);
    if (e != cudaSuccess) return (int)e;
    int n = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, stream_select_kernel<false>, kBlockThreads, kSmemTotal);
    if (e != cudaSuccess) return (int)e;
    if (ctas_per_sm) *ctas_per_sm = n;
    return 0;
}

int launch_stream_kernel(const StreamArgs& a, int grid, void* stream) {
    cudaLaunchAttribute attr[1];
    int n = 0;
    if (a.overlap) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kBlockThreads);
    cfg.dynamicSmemBytes = kSmemTotal;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cfg.attrs = attr;
    cfg.numAttrs = n;
    if (a.softcap != 0.0f) return (int)cudaLaunchKernelEx(&cfg, stream_select_kernel<true>, a);
    return (int)cudaLaunchKernelEx(&cfg, stream_select_kernel<false>, a);
}

// Resident histories: appends every row's new token to its stream's history on the device.  A row's window always
// ends where its history ends, so the token goes to entry hist_begin + hist_len of the id pool.
namespace {
__global__ void append_tokens_kernel(const RowDesc* rows, int n_rows, const int32_t* tokens, int32_t* pool) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_rows) return;
    if (rows[r].flags & kRowAppend) pool[rows[r].hist_begin + rows[r].hist_len] = tokens[rows[r].out_index];
}
}  // namespace

// Resident verification windows.  Before the launch: draft r of a stream is the last id of row r's window, and goes
// to that place of the id pool.  After it: per stream the accept loop of src/server.cpp:630-636 over the sampled
// tokens (accept while the token equals the next draft, at most `lim` rows), and the last accepted token is stored
// where the history will end - the confirmed drafts before it are in place already.  Table entry of a stream:
// first row, rows m, limit, unused, end of the history in the pool (two words), then the m - 1 drafts.
namespace {
__global__ void write_drafts_kernel(const RowDesc* rows, int n_rows, int32_t* pool) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_rows) return;
    if (rows[r].flags & kRowDraft) pool[rows[r].hist_begin + rows[r].hist_len - 1] = rows[r].gather_off;
}
__global__ void accept_windows_kernel(const int32_t* table, int n_streams, const int32_t* tokens, int32_t* pool) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_streams) return;
    const int32_t* t = table + (size_t)i * kWindowTableInts;
    const int r0 = t[0], m = t[1], lim = t[2];
    const int64_t end = ((int64_t)t[5] << 32) | (uint32_t)t[4];
    int acc = 0;
    for (int r = 0; r < lim; ++r) {
        acc = r + 1;
        if (r + 1 < m && tokens[r0 + r] == t[6 + r]) continue;
        break;
    }
    if (acc > 0) pool[end + acc - 1] = tokens[r0 + acc - 1];
}
}  // namespace

int launch_write_drafts(const RowDesc* rows, int n_rows, int32_t* pool, void* stream) {
    write_drafts_kernel<<<(n_rows + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(rows, n_rows, pool);
    return (int)cudaGetLastError();
}
int launch_accept_windows(const int32_t* table, int n_streams, const int32_t* tokens, int32_t* pool, void* stream) {
    accept_windows_kernel<<<(n_streams + 63) / 64, 64, 0, static_cast<cudaStream_t>(stream)>>>(table, n_streams, tokens, pool);
    return (int)cudaGetLastError();
}

int launch_append_tokens(const RowDesc* rows, int n_rows, const int32_t* tokens, int32_t* pool, void* stream) {
    append_tokens_kernel<<<(n_rows + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(rows, n_rows, tokens, pool);
    return (int)cudaGetLastError();
}

int launch_merge_lists(const void* lists, const int32_t* list_n, int n_lists, int list_stride, int n_rows, const RowDesc* rows, int32_t* tokens,
                       int32_t* kept_ids, double* kept_pr, int32_t* kept_n, uint32_t* status, int scan_sums, void* stream) {
    merge_lists_kernel<<<n_rows, kThreads, kSmemMerge, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const u64*>(lists), list_n, n_lists, list_stride, n_rows, rows, tokens, kept_ids, kept_pr, kept_n, status, scan_sums);
    return (int)cudaGetLastError();
}

int launch_gather_patched(const float* logits, const RowDesc* rows, int n_rows, const int32_t* hist, int n_vocab, int vocab_offset,
                          float* out, void* stream) {
    gather_patched_kernel<<<n_rows, 128, 0, static_cast<cudaStream_t>(stream)>>>(logits, rows, n_rows, hist, n_vocab, vocab_offset, out);
    return (int)cudaGetLastError();
}

// The chunk schedule of a launch: how every row is cut into work items.  `slots` = CTAs that run at once; a row may
// have at most max_chunks chunks, and every chunk gets a slot of gather_cap / chunks entries (at least 3 k where
// possible: about 2.3 k candidates reach an item's final bound, as a rule; never fewer than k).  Returns the number
// of chunks (0: the rows cannot be scheduled) and the slot size.
int plan_chunks(int n_rows, int n_vocab, int kmax, int slots, int gather_cap, int max_chunks, uint8_t* chunk_len, int* slot_cap) {
    const int T = (n_vocab + kTile - 1) / kTile;
    kmax = kmax > 1 ? kmax : 1;
    max_chunks = max_chunks < kMaxChunks ? max_chunks : kMaxChunks;
    const int want = 3 * kmax > 96 ? 3 * kmax : 96;             // the slot size aimed at
    int by_slot = gather_cap / want;
    const int hard = gather_cap / kmax;                          // more chunks than this and a slot could not hold k
    const int min_chunks = (T + kItemTilesMax - 1) / kItemTilesMax;
    if (by_slot < min_chunks) by_slot = min_chunks;              // long rows: smaller slots rather than no plan
    if (by_slot < max_chunks) max_chunks = by_slot;
    if (hard < max_chunks) max_chunks = hard;
    if (max_chunks < 1 || min_chunks > max_chunks) return 0;
    const double per_cta = (double)n_rows * T / (slots > 1 ? slots : 1);   // tiles a CTA streams on average
    // Two to three items per CTA keep the dynamic hand-out balanced at little end-of-item work; an item never spans
    // more than kItemTilesMax tiles.
    int q = (int)(per_cta / 2.5 + 0.5);
    q = q < 1 ? 1 : (q > kItemTilesMax ? kItemTilesMax : q);
    while ((T + q - 1) / q > max_chunks && q < kItemTilesMax) ++q;
    // The last tiles of a row are cut into pieces that halve down to single tiles: the items the CTAs draw last are
    // short, so the CTAs finish together (pointless when a CTA works on one item only).
    int taper = (per_cta > q && q > 1) ? (q < T / 4 ? q : T / 4) : 0;
    for (;;) {
        int n = 0;
        const int main_tiles = T - taper;
        const int n_main = (main_tiles + q - 1) / q;
        for (int i = 0; i < n_main && n < kMaxChunks; ++i) chunk_len[n++] = (uint8_t)(main_tiles / n_main + (i < main_tiles % n_main ? 1 : 0));
        bool fits = n_main <= kMaxChunks;
        for (int t = taper; t > 0;) {
            const int h = t > 1 ? (t + 1) / 2 : 1;
            if (n == kMaxChunks) {
                fits = false;
                break;
            }
            chunk_len[n++] = (uint8_t)h;
            t -= h;
        }
        if (fits && n <= max_chunks) {
            *slot_cap = gather_cap / n;
            return n;
        }
        if (taper == 0) return 0;
        taper = 0;   // no room for the short pieces
    }
}

}  // namespace fsb
