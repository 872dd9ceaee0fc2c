// fsb_stream.cu - the static-plan streaming candidate kernel of the B200 batched token sampler (sm_100a).
//
// One launch samples every row of a batch whose effective k is at most kMaxK (greedy rows are k = 1):
//   repetition penalty (src/sampler.cpp:11-18) -> greedy argmax (:19-23) or top-k candidates (:25-35)
//   -> fp64 softmax (:37-41) -> min-p (:43) -> top-p (:44) -> seeded draw (:45-49).
// (reference paths are relative to the paragontasx/ferro project root)
// How it works is described above SegCtx below.
#include <cuda_runtime.h>

#include "../../include/ferro_sampler_b200.h"
#include <algorithm>

#include "fsb_device.cuh"

namespace fsb {
namespace {

constexpr int kWarps = kThreads / 32;
constexpr int kWTile = kTile / kWarps;          // 512 logits: a warp's part of a CTA tile
constexpr int kBlockThreads = kThreads + 32;    // consumers + the producer warp
constexpr int kMaxJ = (kFlatCells + kMaxK + kThreads - 1) / kThreads;   // cells one thread may hold in a re-selection

constexpr size_t kSmemStage = (size_t)kStages * kTile * sizeof(float);
constexpr size_t kSmemQueue = (size_t)kLaneQueue * kThreads * sizeof(unsigned);   // the lanes' queues of noted cells
constexpr size_t kSmemCells = (size_t)kFlatCells * kCellBytes;                     // gathered cells; a list of composites otherwise
constexpr size_t kSmemKept = (size_t)kMaxK * kCellBytes;                           // cells that survived a re-selection; selection scratch
constexpr size_t kSmemBitmap = (size_t)kBitmapWords * sizeof(unsigned);
constexpr int kRecvCap = 512;                                // clustered CTAs: the other CTAs' ordered candidates arrive here,
constexpr size_t kSmemRecv = (size_t)kRecvCap * sizeof(u64);   // (cluster size - 1) parts of k entries
static_assert(kRecvCap >= kMaxK, "a pair can always exchange");
constexpr size_t kSmemTotal = kSmemStage + kSmemQueue + kSmemCells + kSmemKept + kSmemBitmap + kSmemRecv + sizeof(SharedCtl);
static_assert(kSmemTotal <= 227 * 1024, "one CTA per SM");
static_assert(kSmemCells >= (size_t)kMergeCap * sizeof(u64), "the element list lives in the gathered cells' memory");
static_assert(kMergeCap >= 4 * kMaxK, "the logits of kMaxK surviving cells must fit into the element list");
static_assert(kMergeCap >= 2 * kMaxK, "the epilogue's arrays live in the list's memory");
static_assert(kSmemKept >= (size_t)kMaxK * sizeof(u64), "the ordered candidates live in the survivors' memory");
static_assert(kWTile == 512, "a lane owns four float4 of a warp tile");
static_assert(kMaxTilesPerCta <= 32, "a location is seven bits: the tile number above two bits (bit 7 is free)");
static_assert(kFlatCells >= kThreads, "a capped gather round takes at least one cell per thread");
static_assert(kLaneQueue % 4 == 0 && kLaneQueue >= 8, "lanes look at four cells per tile");

constexpr long long kCopyWaitCycles = 2000000000ll;   // about 1 s: a bulk copy that has not landed by then is reported, not awaited

// How the streaming kernel works.
// The [rows][n_vocab] matrix is cut into CTA tiles of kTile logits; the flat list of tiles is dealt to the CTAs in
// equal contiguous ranges, and the part of a row that one CTA owns is a "segment".  One extra warp, the producer,
// brings the CTA tiles into a ring of kStages shared-memory slots, one 1-D bulk copy per tile, so every logit is
// read from HBM exactly once; the sixteen consumer warps each own one sixteenth (a warp tile of kWTile logits) of
// every tile, wait for it to land, look at it and hand the slot back - they meet at the ring, never at a barrier.
// Lane l owns float4 number l + 32 * q (q = 0..3) of a warp tile: a "cell" of four consecutive logits.  While
// streaming a lane does not look at single logits: it takes the maximum of each cell, and where that reaches the
// admission bound it notes the cell (one predicated 4-byte store of its truncated maximum and its location into a
// queue only this lane writes).  At the end of a segment the noted cells the bound has not overtaken are read again
// (from L2, as a rule), their logits that reach the final bound are ordered, and the segment's k best are the row's
// candidates - or, when a row has several segments, go to the first CTA of the row's cluster through shared memory,
// or to the row's scratch area, where the CTA that draws the row's last ticket merges them.  Nobody spins on
// another CTA; waits for this CTA's own copies are bounded.

// The shared memory of a CTA.  The gathered cells' memory doubles as a list of composites (elements, merging),
// the survivors' memory as the ordered candidates of the epilogue.
struct Smem {
    float* stage;       // [kStages][kTile] ring of CTA tiles
    unsigned* queue;    // [kLaneQueue][kThreads] cells noted by each lane: truncated maximum | location
    float4* cells;      // [kFlatCells] gathered cells ...
    int* ids;           // [kFlatCells] ... and their first token ids
    float4* kcells;     // [kMaxK] survivors of re-selections
    int* kids;          // [kMaxK]
    u64* list;          // = cells
    u64* sorted;        // = kcells
    unsigned* bitmap;
    u64* recv;          // [kRecvCap] receive buffer of the first CTA of a cluster
    SharedCtl* ctl;
};
__device__ __forceinline__ Smem smem_view() {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Smem m;
    unsigned char* p = smem_raw;
    m.stage = reinterpret_cast<float*>(p);
    p += kSmemStage;
    m.queue = reinterpret_cast<unsigned*>(p);
    p += kSmemQueue;
    m.cells = reinterpret_cast<float4*>(p);
    m.ids = reinterpret_cast<int*>(p + (size_t)kFlatCells * sizeof(float4));
    m.list = reinterpret_cast<u64*>(p);
    p += kSmemCells;
    m.kcells = reinterpret_cast<float4*>(p);
    m.kids = reinterpret_cast<int*>(p + (size_t)kMaxK * sizeof(float4));
    m.sorted = reinterpret_cast<u64*>(p);
    p += kSmemKept;
    m.bitmap = reinterpret_cast<unsigned*>(p);
    p += kSmemBitmap;
    m.recv = reinterpret_cast<u64*>(p);
    m.ctl = reinterpret_cast<SharedCtl*>(p + kSmemRecv);
    return m;
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
// The tile's bits of the segment bitmap are one word per 32 columns; each of the first lanes owns one word and
// patches the columns whose bits are set.  A bit is set once however often an id occurs in the window.
// (Patching the lanes' registers after the look's loads instead - four bitmap reads per lane and tile - was measured
// slower: the loop is bound by instruction issue, and this way most lanes do nothing.)
__device__ __forceinline__ void patch_tile(float* st, int len, int col0, int seg_lo, float pen, const unsigned* bitmap, float* wb_row) {
    const int lane = threadIdx.x & 31;
    const int nw = (len + 31) >> 5;
    unsigned w = (lane < nw) ? bitmap[((col0 - seg_lo) >> 5) + lane] : 0u;
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

// The r-th largest (r = 1..32) of the 32 lane values of a warp: a bitonic sort across the lanes.
__device__ __forceinline__ unsigned warp_rth_largest(unsigned v, int r) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
        for (int j = k >> 1; j > 0; j >>= 1) {
            const unsigned o = __shfl_xor_sync(0xffffffffu, v, j);
            const bool up = (lane & k) == 0;   // k == 32: every lane, the final order is ascending
            const bool low = (lane & j) == 0;
            v = (up == low) ? min(v, o) : max(v, o);
        }
    }
    return __shfl_sync(0xffffffffu, v, 32 - r);
}

// A bound that at least r = min(32, ceil(k / warps)) logits of this warp's stream reach: the r-th largest of the
// lanes' running maxima (each is a logit of its own).
__device__ __forceinline__ float warp_bound(float run_max, int k) {
    const int r = min(32, (k + kWarps - 1) / kWarps);
    const unsigned key = warp_rth_largest(float_key(run_max), r);
    return key_float(key);
}

// Admission bound of the CTA: at least k logits of the segment reach the smallest of the warps' bounds (eight
// warps, at least ceil(k / 8) logits each, or 32 * 8 >= kMaxK), so no logit below it is among the segment's k
// best.  Each warp posts its value; values only grow, so a reader may use another warp's older value without a
// barrier.
__device__ __forceinline__ float min_warp_bounds(SharedCtl* ctl) {
    float m = __int_as_float(0x7f800000);
#pragma unroll
    for (int w = 0; w < kWarps; w += 4) {
        float4 v;   // volatile: re-read on every call
        asm volatile("ld.volatile.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(smem_u32(&ctl->wbound[w])));
        m = fminf(m, fminf(fminf(v.x, v.y), fminf(v.z, v.w)));
    }
    return m;
}
// Diagnostics: slot 0 takes the global timer (ns) once, the others the SM cycle counter (cheap to read).
__device__ __forceinline__ void trace_mark(const StreamArgs& a, int slot) {
    if (a.trace && threadIdx.x == 0) {
        a.trace[(size_t)blockIdx.x * 8 + slot] = slot == 0 ? global_timer_ns() : (u64)clock64();
        if (slot == 0) a.trace[(size_t)blockIdx.x * 8 + 7] = (u64)clock64();
    }
}

// Composite of a cell: (largest of its four logits, first token id).  A logit of the k best of a set of cells
// always lies in one of the k cells with the largest composites.
__device__ __forceinline__ u64 cell_comp(float4 x, int id0) { return make_comp(fmaxf(max3(x.x, x.y, x.z), x.w), id0); }

// A queue entry: the cell's maximum with its low eight bits cleared (rounded toward zero) | the cell's location,
// (tile of the segment << 2) | q.  For any a >= b, entry_value of a's entry >= truncated(b): testing entries
// against a truncated bound never drops a cell whose maximum reaches the bound.
__device__ __forceinline__ unsigned make_entry(float mx, unsigned loc) { return (__float_as_uint(mx) & 0xFFFFFF00u) | loc; }
__device__ __forceinline__ float entry_value(unsigned e) { return __uint_as_float(e & 0xFFFFFF00u); }
__device__ __forceinline__ float truncated(float x) { return __uint_as_float(__float_as_uint(x) & 0xFFFFFF00u); }

// Notes a cell in this lane's queue if its maximum reaches the bound: a compare, the entry, one predicated store and
// one predicated increment - no branch.  `q_base` is the shared-memory address of the lane's entry 0; entries of
// one lane are kThreads * 4 bytes apart.
__device__ __forceinline__ void note_cell_if(float mx, float thr, unsigned loc, unsigned q_base, int& qn) {
    const unsigned entry = make_entry(mx, loc);
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .u32 a;\n\t"
        "setp.ge.f32 p, %2, %3;\n\t"
        "mad.lo.u32 a, %0, %5, %1;\n\t"
        "@p st.shared.u32 [a], %4;\n\t"
        "@p add.s32 %0, %0, 1;\n\t}"
        : "+r"(qn)
        : "r"(q_base), "f"(mx), "f"(thr), "r"(entry), "n"(kThreads * 4)
        : "memory");
}

// Drops the entries of this lane's queue whose cell maximum cannot reach `thr` any more; returns the new length.
__device__ __forceinline__ int drop_stale(unsigned* myq, int qn, float thr) {
    const float t = truncated(thr);
    int w = 0;
    for (int i = 0; i < qn; ++i) {
        const unsigned e = myq[i * kThreads];
        if (entry_value(e) >= t) myq[(w++) * kThreads] = e;
    }
    return w;
}

// Column of the cell a queue entry of this thread names.
__device__ __forceinline__ int loc_column(unsigned loc, const SegCtx& sc) {
    loc &= 0xFFu;
    return sc.seg_lo + (int)(loc >> 2) * kTile + (int)(threadIdx.x >> 5) * kWTile + 4 * ((int)(threadIdx.x & 31) + 32 * (int)(loc & 3u));
}

// The cell at column `col` of the row, as loaded (no transformation).  Columns past the end of the row are NaN.
__device__ __forceinline__ float4 load_cell(const SegCtx& sc, int col) {
    if (sc.vec_ok && col + 4 <= sc.n_vocab) return __ldcg(reinterpret_cast<const float4*>(sc.row + col));
    const float qnan = __int_as_float(0x7fc00000);
    float4 t;
    t.x = (col < sc.n_vocab) ? __ldcg(sc.row + col) : qnan;
    t.y = (col + 1 < sc.n_vocab) ? __ldcg(sc.row + col + 1) : qnan;
    t.z = (col + 2 < sc.n_vocab) ? __ldcg(sc.row + col + 2) : qnan;
    t.w = (col + 3 < sc.n_vocab) ? __ldcg(sc.row + col + 3) : qnan;
    return t;
}

// Softcap, then penalty, as the streaming pass applied them to the cell at column `col`.
template <bool SOFTCAP>
__device__ __forceinline__ float4 transform_cell(float4 t, const SegCtx& sc, const unsigned* bitmap, int col) {
    if (sc.final_in_mem) return t;
    if (SOFTCAP) {
        t.x = __fmul_rn(sc.cap, tanhf(__fdiv_rn(t.x, sc.cap)));
        t.y = __fmul_rn(sc.cap, tanhf(__fdiv_rn(t.y, sc.cap)));
        t.z = __fmul_rn(sc.cap, tanhf(__fdiv_rn(t.z, sc.cap)));
        t.w = __fmul_rn(sc.cap, tanhf(__fdiv_rn(t.w, sc.cap)));
    }
    if (sc.has_pen) {
        const int b = col - sc.seg_lo;   // a multiple of four: the four bits lie in one word
        const unsigned bits = (bitmap[b >> 5] >> (b & 31)) & 0xFu;
        if (bits) {
            if (bits & 1u) t.x = t.x > 0.0f ? __fdiv_rn(t.x, sc.pen) : __fmul_rn(t.x, sc.pen);
            if (bits & 2u) t.y = t.y > 0.0f ? __fdiv_rn(t.y, sc.pen) : __fmul_rn(t.y, sc.pen);
            if (bits & 4u) t.z = t.z > 0.0f ? __fdiv_rn(t.z, sc.pen) : __fmul_rn(t.z, sc.pen);
            if (bits & 8u) t.w = t.w > 0.0f ? __fdiv_rn(t.w, sc.pen) : __fmul_rn(t.w, sc.pen);
        }
    }
    return t;
}

// Exclusive prefix sum of one int per consumer thread over the CTA (thread order) and the total.  Contains two
// barriers; uses ctl->red.
struct ScanResult {
    int before;
    int total;
};
__device__ __forceinline__ ScanResult cta_scan(int v, SharedCtl* ctl) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) reinterpret_cast<int*>(ctl->red)[warp] = inc;
    consumer_sync();
    int before = inc - v, total = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
        const int s = reinterpret_cast<int*>(ctl->red)[w];
        if (w < warp) before += s;
        total += s;
    }
    consumer_sync();   // the scratch may be written again
    return ScanResult{before, total};
}

// Re-selection over the nq gathered cells (flat arrays) and the nkept survivors: the k cells with the largest
// composites become the survivors' list.  Returns their number and the composite bound they passed (0: nothing was
// dropped).  All consumer threads must call, after a barrier that made the gathered cells visible.
struct SelectResult {
    int count;
    u64 bound;
};
__device__ __noinline__ SelectResult select_cells(int nq, int nkept, int k) {
    const Smem cs = smem_view();
    SharedCtl* ctl = cs.ctl;
    const int tid = threadIdx.x;
    const int n = nq + nkept;
    float4 cx[kMaxJ];
    int cid[kMaxJ];
    u64 cc[kMaxJ];
#pragma unroll
    for (int j = 0; j < kMaxJ; ++j) {
        const int f = tid + j * kThreads;
        cc[j] = 0ull;
        cid[j] = 0;
        cx[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (f < n) {
            cx[j] = f < nq ? cs.cells[f] : cs.kcells[f - nq];
            cid[j] = f < nq ? cs.ids[f] : cs.kids[f - nq];
            cc[j] = cell_comp(cx[j], cid[j]);
        }
    }
    consumer_sync();   // every cell is in registers: the survivors' memory may be rewritten
    u64 L = 0ull;
    if (n > k) {
        u64 mn = ~0ull, mx = 0ull;
#pragma unroll
        for (int j = 0; j < kMaxJ; ++j) {
            if (cc[j] != 0ull) {
                mn = min(mn, cc[j]);
                mx = max(mx, cc[j]);
            }
        }
        cta_minmax(mn, mx, ctl);
        L = bisect_bound(k, mn, mx, ctl, [&](u64 t) {
            int c = 0;
#pragma unroll
            for (int j = 0; j < kMaxJ; ++j) c += cc[j] >= t ? 1 : 0;   // empty slots hold 0, t is never 0
            return c;
        });
    }
    if (tid == 0) ctl->out_cnt = 0;
    consumer_sync();
#pragma unroll
    for (int j = 0; j < kMaxJ; ++j) {
        if (cc[j] != 0ull && cc[j] >= L) {
            const int p = atomicAdd(&ctl->out_cnt, 1);
            if (p < kMaxK) {
                cs.kcells[p] = cx[j];
                cs.kids[p] = cid[j];
            }
        }
    }
    consumer_sync();
    return SelectResult{min(ctl->out_cnt, kMaxK), L};
}

// The re-selection proper (rare): every lane drops the noted cells the bound has overtaken, the rest are read again
// and the CTA keeps the k best cells.  All consumer threads call it, after the barrier of the rendez-vous.
template <bool SOFTCAP>
__device__ __noinline__ int compact_cells(int qn, int nkept, float thr_f) {
    const Smem m = smem_view();
    SharedCtl* ctl = m.ctl;
    const SegCtx& sc = ctl->seg;
    const int k = sc.k;
    const int tid = threadIdx.x;
    u64 bound = 0ull;
    // every lane first drops what the bound has overtaken; then gather rounds: everything at once if it fits, else
    // three cells per thread and round
    qn = drop_stale(m.queue + tid, qn, fmaxf(thr_f, min_warp_bounds(ctl)));
    int cap = kLaneQueue;
    if (cta_scan(qn, ctl).total > kFlatCells) cap = kFlatCells / kThreads;
    for (;;) {
        const int cnt = min(qn, cap);
        const ScanResult sr = cta_scan(cnt, ctl);
        if (sr.total == 0) break;
        for (int i0 = 0; i0 < cnt; i0 += 4) {   // four loads in flight
            float4 c[4];
            int col[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                col[u] = -1;
                if (i0 + u < cnt) {
                    col[u] = loc_column(m.queue[(size_t)(qn - 1 - i0 - u) * kThreads + tid], sc);
                    c[u] = load_cell(sc, col[u]);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (col[u] >= 0) {
                    m.cells[sr.before + i0 + u] = transform_cell<SOFTCAP>(c[u], sc, m.bitmap, col[u]);
                    m.ids[sr.before + i0 + u] = col[u] + sc.id_base;
                }
            }
        }
        qn -= cnt;
        consumer_sync();
        const SelectResult r = select_cells(sr.total, nkept, k);
        nkept = r.count;
        bound = max(bound, r.bound);
    }
    if (tid == 0) {
        ctl->need_compact = 0;
        ctl->ev_bound = bound;
    }
    consumer_sync();
    return 1 | (nkept << 1);
}

// One rendez-vous of all consumer warps of the CTA.  A warp comes here because it saw a request for a re-selection
// (a lane's queue is nearly full), or because it has finished its part of the segment.  Every warp posts its
// bound and the number of cells its lanes hold.  If a re-selection was asked for, the queued cells are read again
// and the CTA keeps the k best cells (they become the survivors' list, all queues become empty), and `happened`
// is set; otherwise every warp had finished and the posted values describe the whole segment.  Warps depend on
// nothing but their own copies while streaming and look out for requests at every tile and in every wait, so
// every warp gets here in bounded time.
// Returns (happened) | (survivors << 1); the composite bound of a re-selection is left in ctl->ev_bound and the
// warps' bounds in ctl->wbound.
__device__ __forceinline__ int event_happened(int ev) { return ev & 1; }
__device__ __forceinline__ int event_nkept(int ev) { return (ev >> 1) & 1023; }
template <bool SOFTCAP>
__device__ __forceinline__ int cta_event(int qn, int nkept, float run_max, float thr_f) {
    const Smem m = smem_view();
    SharedCtl* ctl = m.ctl;
    const SegCtx& sc = ctl->seg;
    const int k = sc.k;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float wb = warp_bound(run_max, k);
    if (lane == 0) *reinterpret_cast<volatile float*>(&ctl->wbound[warp]) = wb;
    if (tid == 0) ctl->out_cnt = 0;
    consumer_sync();
    if (*reinterpret_cast<volatile int*>(&ctl->need_compact) == 0) return nkept << 1;
    return compact_cells<SOFTCAP>(qn, nkept, thr_f);
}

// Appends to the element list the logits of up to N cells of this thread that reach `thr` (NaNs and columns past
// the end of the row take no part).  A warp reserves its part of the list with one atomic.  All lanes of the warp
// must call; ncell = 0 contributes nothing.  Entries past the list's capacity are counted but not written.
template <int N>
__device__ __forceinline__ void append_elements(const float4 (&c)[N], const int (&id0)[N], int ncell, float thr, int id_end, u64* list,
                                                SharedCtl* ctl) {
    static_assert(N <= 8, "one mask bit per logit");
    const int lane = threadIdx.x & 31;
    unsigned mask = 0u;
#pragma unroll
    for (int u = 0; u < N; ++u) {
        if (u < ncell) {
            const float xs[4] = {c[u].x, c[u].y, c[u].z, c[u].w};
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (xs[e] >= thr && id0[u] + e < id_end) mask |= 1u << (4 * u + e);
        }
    }
    const int mine = __popc(mask);
    int inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    const int wtotal = __shfl_sync(0xffffffffu, inc, 31);
    if (wtotal == 0) return;
    int base = 0;
    if (lane == 31) base = atomicAdd(&ctl->out_cnt, wtotal);
    base = __shfl_sync(0xffffffffu, base, 31);
    int p = base + inc - mine;
#pragma unroll
    for (int u = 0; u < N; ++u) {
        const float xs[4] = {c[u].x, c[u].y, c[u].z, c[u].w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
            if (mask & (1u << (4 * u + e))) {
                if (p < kMergeCap) list[p] = make_comp(xs[e], id0[u] + e);
                ++p;
            }
    }
}

// The producer: one lane brings the CTA tiles in, one 1-D bulk copy per tile (large copies: the copy engine's cost
// is per request), into a ring of kStages slots.  A slot is refilled once all consumer warps have handed it back.
__device__ __forceinline__ void producer_loop(const StreamArgs& a, float* stage, SharedCtl* ctl, int t_begin, int nt) {
    if ((threadIdx.x & 31) != 0) return;
    const int T = a.tiles_per_row, V = a.n_vocab;
    int irow = t_begin / T, ij = t_begin - irow * T;
    long long t_last = clock64();
    int i = 0;
    while (i < nt) {
        const int slot = i % kStages;
        // the first kStages tiles find their slots free; later ones wait for the consumers' hand-back
        if (i >= kStages && !mbar_try_wait(&ctl->empty[slot], (unsigned)((i / kStages - 1) & 1))) {
            if (clock64() - t_last > kCopyWaitCycles) {   // the consumers never came back: report and stop
                report_status(a.status, a.status_host, kStatusCopyTimeout);
                return;
            }
            continue;
        }
        const int col0 = ij * kTile;
        const int len = min(kTile, V - col0);   // >= 1
        const float* src = a.logits + (a.row_ld >= 0 ? (int64_t)irow * a.row_ld : a.rows[irow].logits_off) + col0;
        float* dst = stage + (size_t)slot * kTile;
        const unsigned bytes = (unsigned)(len & ~3) * 4u;
        for (int e = len & ~3; e < len; ++e) dst[e] = src[e];   // ragged tail by plain loads
        if (bytes) {
            fence_proxy_async_smem();   // generic-proxy accesses to this slot (the consumers' patches) precede the async write
            mbar_expect_tx(&ctl->full[slot], bytes);
            bulk_g2s(dst, src, bytes, &ctl->full[slot]);
        } else {
            mbar_arrive(&ctl->full[slot]);
        }
        t_last = clock64();
        ++i;
        if (++ij == T) {
            ij = 0;
            ++irow;
        }
    }
}

// The end of a segment.  All consumer threads call it once they have looked at their last tile of the segment:
// re-selections that were still asked for, the rendez-vous of the finished warps, the element list, the segment's
// k best logits in order, and - in the CTA that draws the row's last ticket - the merge and the row's epilogue.
// With GREEDY (a launch whose rows are all greedy: a verification step, the static entry point) the streaming loop has
// kept no queues: every lane brings the best logit it saw as a composite (`lane_best`, 0 = none), the CTA takes the
// largest, and that one candidate goes through the same merge and epilogue as an ordered list of length one.
template <bool SOFTCAP, bool GREEDY>
__device__ __forceinline__ void segment_end(const StreamArgs& a, int row, int qn, int nkept, float thr_f, float run_max, bool mark, u64 lane_best) {
    const Smem m = smem_view();
    SharedCtl* ctl = m.ctl;
    const SegCtx& sc = ctl->seg;
    const int tid = threadIdx.x;
    const int T = a.tiles_per_row, V = a.n_vocab, Q = a.tiles_per_cta;
    const RowDesc d = a.rows[row];
    unsigned* myq = m.queue + tid;
    const TailOut tout{a.tokens, a.tokens_host, a.status_host, a.kept_ids, a.kept_pr, a.kept_n, reinterpret_cast<u64*>(a.shard_out), a.shard_n, a.shard_stride, a.status};
    float thr_final;
    int n_el = 0;
    int kk = 0;
    if (GREEDY) {
        u64 mn = lane_best ? lane_best : ~0ull, mx = lane_best;
        cta_minmax(mn, mx, ctl);
        if (mx == 0ull && !SOFTCAP) {
            // No lane saw anything above minus infinity.  A segment of nothing but -inf (and NaN) still has an argmax in
            // the reference - its first -inf - so look for one in memory (the penalty leaves -inf as it is).
            u64 mine = 0ull;
            for (int c = sc.seg_lo + tid; c < sc.seg_hi; c += kThreads) {
                const float x = __ldcg(sc.row + c);
                if (x == -__int_as_float(0x7f800000)) mine = max(mine, make_comp(x, c + sc.id_base));
            }
            mn = mine ? mine : ~0ull;
            mx = mine;
            cta_minmax(mn, mx, ctl);
        }
        if (mark) trace_mark(a, 4);
        if (tid == 0) m.sorted[0] = mx;
        consumer_sync();
        kk = mx != 0ull ? 1 : 0;
        n_el = kk;
    }
    for (; !GREEDY;) {
        for (;;) {   // re-selections that were still asked for, then the rendez-vous of the finished warps
            const int ev = cta_event<SOFTCAP>(qn, nkept, run_max, thr_f);
            if (!event_happened(ev)) break;
            qn = 0;
            nkept = event_nkept(ev);
        }
        thr_final = fmaxf(thr_f, min_warp_bounds(ctl));
        if (mark) trace_mark(a, 4);
        // ---- the logits of the noted cells that reach the final bound become the element list
        const int id_end = V + sc.id_base;
        if (nkept > 0) {
            float4 c[1];
            int id0[1];
            c[0] = m.kcells[min(tid, nkept - 1)];
            id0[0] = m.kids[min(tid, nkept - 1)];
            append_elements<1>(c, id0, tid < nkept ? 1 : 0, thr_final, id_end, m.list, ctl);
        }
        qn = drop_stale(myq, qn, thr_final);   // most noted cells have been overtaken by the bound
        // a thread reads up to four of its cells per round (lanes rarely hold more that the bound has not overtaken)
        const int rounds = (__reduce_max_sync(0xffffffffu, qn) + 3) >> 2;
#pragma unroll 1
        for (int rd = 0; rd < rounds; ++rd) {
            float4 c[4];
            int id0[4];
            const int n = max(0, min(4, qn - 4 * rd));
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                id0[u] = 0;
                c[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (u < n) {
                    id0[u] = loc_column(myq[(4 * rd + u) * kThreads], sc);
                    c[u] = load_cell(sc, id0[u]);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (u < n) {
                    c[u] = transform_cell<SOFTCAP>(c[u], sc, m.bitmap, id0[u]);
                    id0[u] += sc.id_base;
                }
            }
            append_elements<4>(c, id0, n, thr_final, id_end, m.list, ctl);
        }
        consumer_sync();
        n_el = ctl->out_cnt;
        if (n_el <= kMergeCap) break;
        // more logits reach the bound than the list can take (many equal values): keep the k best cells first
        consumer_sync();
        *reinterpret_cast<volatile int*>(&ctl->need_compact) = 1;
    }
    if (mark) trace_mark(a, 2);
    if (mark && a.trace && tid == 0) a.trace[(size_t)blockIdx.x * 8 + 3] = (u64)n_el;
    if (a.overlap == 1) pdl_wait_prior();   // from here on this launch writes what the previous launch in the stream may still be using
    // the segment's k best logits (or all, if fewer), in order
    const int first_cta = (row * T) / Q, last_cta = (row * T + T - 1) / Q;
    const int nseg = last_cta - first_cta + 1;
    bool merge_here = true;
    if (!GREEDY) kk = topk_sorted(m.list, n_el, d.k, m.sorted, ctl);
    if (a.pair) {
        // The row's CTAs are a cluster: CTA r > 0 puts its ordered candidates into part r - 1 of CTA 0's receive
        // buffer, all arrive at the cluster's barrier (the only phase of it in this kernel: the producer warps arrived
        // when they finished), and CTA 0 merges.  No global memory, no ticket.
        const unsigned rank = cluster_cta_rank();
        if (rank != 0u) {
            const unsigned remote = cluster_map_shared(smem_u32(m.recv + (rank - 1u) * (unsigned)d.k), 0u);
            for (int i = tid; i < kk; i += kThreads) cluster_store_u64(remote + 8u * (unsigned)i, m.sorted[i]);
            if (tid == 0) cluster_store_u32(cluster_map_shared(smem_u32(&ctl->recv_n[rank]), 0u), (unsigned)kk);
        }
        __syncwarp();
        cluster_arrive_release();
        merge_here = rank == 0u;
        if (merge_here) {
            cluster_wait_acquire();
            if (a.pair == 2) {
                // two lists: the rank of an entry is its place in its own list plus the number of entries of the other above it
                const int n1 = min(*reinterpret_cast<volatile int*>(&ctl->recv_n[1]), d.k);
                for (int e = tid; e < kk + n1; e += kThreads) {
                    const bool mine = e < kk;
                    const int i1 = mine ? e : e - kk;
                    const u64 c = mine ? m.sorted[i1] : m.recv[i1];
                    const u64* run = mine ? m.recv : m.sorted;
                    int lo = 0, hi = mine ? n1 : kk;
                    while (lo < hi) {
                        const int mid = (lo + hi) >> 1;
                        if (run[mid] > c) lo = mid + 1;
                        else hi = mid;
                    }
                    if (i1 + lo < d.k) m.list[i1 + lo] = c;
                }
                consumer_sync();
                kk = min(kk + n1, d.k);
            } else {
                // several lists: the same, summed over all the other lists
                const int nl = a.pair;
                if (tid == 0) ctl->recv_n[0] = kk;
                consumer_sync();
                int total = 0;
                for (int s2 = 0; s2 < nl; ++s2) total += min(*reinterpret_cast<volatile int*>(&ctl->recv_n[s2]), d.k);
                for (int e = tid; e < nl * d.k; e += kThreads) {
                    const int s1 = e / d.k, i1 = e - s1 * d.k;
                    if (i1 >= min(ctl->recv_n[s1], d.k)) continue;
                    const u64 c = s1 == 0 ? m.sorted[i1] : m.recv[(s1 - 1) * d.k + i1];
                    int rk = i1;
                    for (int s2 = 0; s2 < nl; ++s2) {
                        if (s2 == s1) continue;
                        const u64* run = s2 == 0 ? m.sorted : m.recv + (s2 - 1) * d.k;   // descending: count its entries above c
                        int lo = 0, hi = min(ctl->recv_n[s2], d.k);
                        while (lo < hi) {
                            const int mid = (lo + hi) >> 1;
                            if (run[mid] > c) lo = mid + 1;
                            else hi = mid;
                        }
                        rk += lo;
                    }
                    if (rk < d.k) m.list[rk] = c;
                }
                consumer_sync();
                kk = min(total, d.k);
            }
            for (int i = tid; i < kk; i += kThreads) m.sorted[i] = m.list[i];
            consumer_sync();
        }
    } else if (nseg > 1) {
        // A row with several segments: segment s publishes its ordered candidates in its own part of the row's
        // scratch (entries [s * k, s * k + count), the count in entry kMergeCap - 1 - s), then draws a ticket; the
        // CTA that draws the row's last ticket merges.  The planner keeps nseg * (k + 1) within kMergeCap.
        const int seg = (int)blockIdx.x - first_cta;
        u64* dst = reinterpret_cast<u64*>(a.scratch) + (size_t)row * kMergeCap;
        if ((seg + 1) * d.k + nseg <= kMergeCap) {
            for (int i = tid; i < kk; i += kThreads) dst[seg * d.k + i] = m.sorted[i];
            if (tid == 0) dst[kMergeCap - 1 - seg] = (u64)kk;
        } else if (tid == 0) {
            report_status(a.status, a.status_host, kStatusMergeOverflow);
        }
        consumer_sync();   // orders the CTA's stores before the ticket, whose release publishes them to the device
        if (tid == 0) ctl->last = (ticket_add_acq_rel(&a.ticket[row], 1u) == (unsigned)(nseg - 1)) ? 1 : 0;
        consumer_sync();
        merge_here = ctl->last != 0;
        if (merge_here) {   // all segments of the row have published (L2 reads, never L1)
            if (tid == 0) a.ticket[row] = 0u;   // ready for the next launch
            if (nseg <= kNumWarps) {
                // few ordered lists: the rank of an entry is its place in its own list plus, for every other list,
                // the number of entries above it (binary search); the lists keep their places in shared memory
                // (counts and entries are read in one go; entries past a list's count are stale and ignored below)
                const int span = nseg * d.k;
                if (tid < nseg) ctl->wcount[tid] = min((int)__ldcg(dst + kMergeCap - 1 - tid), d.k);
                for (int e = tid; e < span; e += kThreads) m.list[e] = __ldcg(dst + e);
                consumer_sync();
                int total = 0;
                for (int s2 = 0; s2 < nseg; ++s2) total += ctl->wcount[s2];
                for (int e = tid; e < span; e += kThreads) {
                    const int s1 = e / d.k, i1 = e - s1 * d.k;
                    if (i1 >= ctl->wcount[s1]) continue;
                    const u64 c = m.list[e];
                    int rank = i1;
                    for (int s2 = 0; s2 < nseg; ++s2) {
                        if (s2 == s1) continue;
                        const u64* run = m.list + s2 * d.k;   // descending: count its entries above c
                        int lo = 0, hi = ctl->wcount[s2];
                        while (lo < hi) {
                            const int mid = (lo + hi) >> 1;
                            if (run[mid] > c) lo = mid + 1;
                            else hi = mid;
                        }
                        rank += lo;
                    }
                    if (rank < d.k) m.sorted[rank] = c;
                }
                kk = min(total, d.k);
                consumer_sync();
            } else {   // many short lists: gather them into one list and order that
                int total = 0;
                for (int s2 = 0; s2 < nseg; ++s2) {
                    const int n2 = min((int)__ldcg(dst + kMergeCap - 1 - s2), d.k);
                    for (int i = tid; i < n2; i += kThreads) m.list[total + i] = __ldcg(dst + s2 * d.k + i);
                    total += n2;
                }
                consumer_sync();
                kk = topk_sorted(m.list, total, d.k, m.sorted, ctl);
            }
        }
    }
    if (mark) trace_mark(a, 5);
    if (merge_here) {
        const RowTail rt{d.rng_word, d.temperature, d.top_p, d.min_p, d.k, d.flags, d.out_index};
        row_epilogue(m.sorted, kk, rt, reinterpret_cast<double*>(m.list), ctl, tout);
    }
    consumer_sync();
    if (mark) trace_mark(a, 6);
}

template <bool SOFTCAP, bool GREEDY>
__global__ void __launch_bounds__(kBlockThreads, 1) stream_select_kernel(const __grid_constant__ StreamArgs a) {
    const Smem m = smem_view();
    SharedCtl* ctl = m.ctl;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int T = a.tiles_per_row, V = a.n_vocab;
    const int t_begin = blockIdx.x * a.tiles_per_cta;
    const int t_end = min(t_begin + a.tiles_per_cta, a.total_tiles);
    const int nt = t_end - t_begin;
    // With launch overlap on, the next launch in the stream may start as soon as this one leaves room; like this one
    // it waits for its predecessor before it writes anything (segment_end), so only the reading of logits overlaps -
    // or, in mode 2, before it does anything at all, so only its placement on the SMs does.
    pdl_launch_dependents();
    if (nt <= 0) return;
    trace_mark(a, 0);
    if (a.write_back || a.overlap == 2) pdl_wait_prior();   // this launch stores into the logits while it streams, or was asked to wait

    if (tid == 0) {   // one thread initialises every barrier, then makes the initialisation visible to the copy engine
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&ctl->full[s], 1u);                  // the producer's arrive (+ the copy's bytes)
            mbar_init(&ctl->empty[s], (unsigned)kWarps);   // one arrive per consumer warp
        }
        ctl->abort = 0;
        ctl->need_compact = 0;
        fence_mbar_init();
    }
    __syncthreads();   // the only barrier the producer warp takes part in
    if (warp == kWarps) {
        if (a.bulk_ok) producer_loop(a, m.stage, ctl, t_begin, nt);
        __syncwarp();
        if (a.pair) cluster_arrive_release();   // every thread of the cluster arrives exactly once (see segment_end)
        return;
    }
    trace_mark(a, 1);

    // ------------------------------------------------------------------------------------------ consumers
    // The loop over a segment's tiles contains no call: everything rare (re-selections, the end of the segment)
    // happens outside it, so that the loop's state stays in registers.
    const float ninf = -__int_as_float(0x7f800000);
    unsigned* myq = m.queue + tid;   // entry i of this lane's queue is myq[i * kThreads]
    const unsigned q_base = smem_u32(myq);
    float* const st_warp = m.stage + warp * kWTile;
    int it = 0;                            // tiles of this CTA looked at so far (the position in the ring)
    for (int tile = t_begin; tile < t_end;) {
        // ---- a new segment starts (all consumer warps are here together: kernel start or after a segment end)
        const int row = tile / T, j0 = tile - row * T;
        const int seg_nt = min(t_end - tile, T - j0);
        const int seg_lo = j0 * kTile;
        const int seg_hi = min(V, (j0 + seg_nt) * kTile);
        const RowDesc d = a.rows[row];
        const float* row_ptr = a.logits + d.logits_off;
        float* wb_row = a.write_back ? const_cast<float*>(row_ptr) : nullptr;
        const float pen = d.penalty;
        const int row_k = d.k;
        const bool has_pen = (d.flags & kRowPenalty) != 0;
        if (tid == 0) {   // what the rendez-vous code needs to know about the segment
            SegCtx& sc = ctl->seg;
            sc.row = row_ptr;
            sc.pen = pen;
            sc.cap = a.softcap;
            sc.has_pen = has_pen ? 1 : 0;
            sc.id_base = a.vocab_offset;
            sc.seg_lo = seg_lo;
            sc.seg_hi = seg_hi;
            sc.n_vocab = V;
            sc.vec_ok = a.bulk_ok;
            sc.k = row_k;
            sc.final_in_mem = a.write_back;
        }
        if (has_pen) {   // bitmap of the penalised columns of this segment
            const int words = (seg_hi - seg_lo + 31) >> 5;
            for (int i = tid; i < words; i += kThreads) m.bitmap[i] = 0u;
            consumer_sync();
            const int32_t* h = a.hist + d.hist_begin;
            for (int i = tid; i < d.hist_len; i += kThreads) {
                const int c = h[i] - a.vocab_offset;
                if (c >= seg_lo && c < seg_hi) atomicOr(&m.bitmap[(c - seg_lo) >> 5], 1u << ((c - seg_lo) & 31));
            }
        }
        consumer_sync();

        float thr_f = ninf, run_max = ninf;
        // GREEDY: the lane's best logit so far - the cell it sits in, that cell's first column, the cell's maximum
        float4 best_cell = make_float4(0.f, 0.f, 0.f, 0.f);
        float best = ninf;
        int best_col = -1;
        u64 thr_comp = 0ull;
        int qn = 0;       // cells in this lane's queue
        int nkept = 0;    // cells in the survivors' list (the same value in every thread)
        int s = 0;        // tiles of the segment this warp has looked at
        int col0 = seg_lo + warp * kWTile;   // first column of this warp's part of tile s

        for (;;) {
            int reason = 0;   // why the loop over the tiles was left: 0 = segment done, 1 = a queue of this warp is nearly full,
                              // 2 = another warp asked for a re-selection while this one was waiting for a copy
            unsigned slot = (unsigned)it % kStages, par = ((unsigned)it / kStages) & 1u;   // ring slot of tile `it` and its phase
            for (; s < seg_nt; ++s, ++it, col0 += kTile, slot = (slot + 1u) % kStages, par ^= (slot == 0u ? 1u : 0u)) {
                if (!GREEDY && __any_sync(0xffffffffu, qn > kLaneQueue - 4)) {
                    reason = 1;
                    break;
                }
                float* st = st_warp + slot * kTile;              // this warp's part of the CTA tile
                const int len = min(kWTile, V - col0);            // may be <= 0 in a row's last tile
                if (a.bulk_ok) {
                    // ---- wait for the CTA tile's copy.  A warp that has to wait also answers re-selection requests of
                    // other warps: a requester sits at the barrier of cta_event, and the ring only moves when every warp does.
                    bool landed = mbar_try_wait(&ctl->full[slot], par);
                    if (!landed) {
                        const long long lim = ctl->abort ? 2000ll : kCopyWaitCycles;
                        const long long t0 = clock64();
                        for (;;) {
                            if (mbar_try_wait(&ctl->full[slot], par)) {
                                landed = true;
                                break;
                            }
                            if (__any_sync(0xffffffffu, *reinterpret_cast<volatile int*>(&ctl->need_compact) != 0)) break;
                            if (clock64() - t0 > lim) {   // the copy never landed: report, carry on with what is there
                                ctl->abort = 1;
                                report_status(a.status, a.status_host, kStatusCopyTimeout);
                                landed = true;
                                break;
                            }
                        }
                        if (!landed) {
                            reason = 2;
                            break;
                        }
                    }
                } else if (len > 0) {   // rows not on 16-byte boundaries: the warp loads its tile itself
                    const float* src = row_ptr + col0;
                    for (int e = lane; e < len; e += 32) st[e] = src[e];
                    __syncwarp();
                }
                if (SOFTCAP) {
                    if (len > 0) softcap_tile(st, len, a.softcap, wb_row ? wb_row + col0 : nullptr);
                }
                if (has_pen && len > 0) patch_tile(st, len, col0, seg_lo, pen, m.bitmap, wb_row);
                if (len < kWTile) {   // what lies past the end of a ragged row is made NaN: never a maximum, never reaches a bound
                    for (int e = max(len, 0) + lane; e < kWTile; e += 32) st[e] = __int_as_float(0x7fc00000);
                    __syncwarp();
                }
                // ---- look: the lane's four cells go to registers (four independent 16-byte loads)
                const float4* st4 = reinterpret_cast<const float4*>(st);
                const float4 x0 = st4[lane], x1 = st4[lane + 32], x2 = st4[lane + 64], x3 = st4[lane + 96];
                const float m0 = fmaxf(max3(x0.x, x0.y, x0.z), x0.w);
                const float m1 = fmaxf(max3(x1.x, x1.y, x1.z), x1.w);
                const float m2 = fmaxf(max3(x2.x, x2.y, x2.z), x2.w);
                const float m3 = fmaxf(max3(x3.x, x3.y, x3.z), x3.w);
                run_max = fmaxf(max3(run_max, m0, m1), fmaxf(m2, m3));
                __syncwarp();
                if (lane == 0 && a.bulk_ok) mbar_arrive(&ctl->empty[slot]);   // the slot goes back to the producer
                if (GREEDY) {
                    // the lane meets its cells in ascending column order, so "strictly larger" keeps the first of equals
                    const int c0 = col0 + 4 * lane;
                    if (m0 > best) { best = m0; best_cell = x0; best_col = c0; }
                    if (m1 > best) { best = m1; best_cell = x1; best_col = c0 + 128; }
                    if (m2 > best) { best = m2; best_cell = x2; best_col = c0 + 256; }
                    if (m3 > best) { best = m3; best_cell = x3; best_col = c0 + 384; }
                    continue;
                }

                // ---- the admission bound: set at the segment's first tile (all warps must have posted: one barrier per
                // segment), then refreshed without a barrier at tiles 1, 2, 4, 8, ... of the segment
                if ((s & (s - 1)) == 0) {   // s = 0, 1, 2, 4, 8, ...
                    const float wb = warp_bound(run_max, row_k);
                    if (lane == 0) *reinterpret_cast<volatile float*>(&ctl->wbound[warp]) = wb;
                    if (s == 0) consumer_sync();
                    else __syncwarp();
                    thr_f = fmaxf(thr_f, min_warp_bounds(ctl));
                }

                // ---- note the cells whose maximum reaches the bound (padding past the end of a row never does)
                const unsigned loc = (unsigned)s << 2;
                if (thr_comp == 0ull) {
                    note_cell_if(m0, thr_f, loc, q_base, qn);
                    note_cell_if(m1, thr_f, loc | 1u, q_base, qn);
                    note_cell_if(m2, thr_f, loc | 2u, q_base, qn);
                    note_cell_if(m3, thr_f, loc | 3u, q_base, qn);
                } else {   // after a re-selection: ties at the bound are settled by token id
                    const int id_lane = col0 + 4 * lane + a.vocab_offset;
                    if (m0 >= thr_f && make_comp(m0, id_lane) >= thr_comp) myq[(qn++) * kThreads] = make_entry(m0, loc);
                    if (m1 >= thr_f && make_comp(m1, id_lane + 128) >= thr_comp) myq[(qn++) * kThreads] = make_entry(m1, loc | 1u);
                    if (m2 >= thr_f && make_comp(m2, id_lane + 256) >= thr_comp) myq[(qn++) * kThreads] = make_entry(m2, loc | 2u);
                    if (m3 >= thr_f && make_comp(m3, id_lane + 384) >= thr_comp) myq[(qn++) * kThreads] = make_entry(m3, loc | 3u);
                }
            }
            if (reason == 0) break;
            // ---- a re-selection: the CTA keeps the k best of the cells noted so far, every queue becomes empty
            if (reason == 1) {   // first drop what the bound has overtaken: that alone makes room, as a rule
                qn = drop_stale(myq, qn, thr_f);
                if (!__any_sync(0xffffffffu, qn > kLaneQueue - 4)) continue;
                *reinterpret_cast<volatile int*>(&ctl->need_compact) = 1;
            }
            const int ev = cta_event<SOFTCAP>(qn, nkept, run_max, thr_f);
            if (event_happened(ev)) {
                qn = 0;
                nkept = event_nkept(ev);
                const u64 eb = ctl->ev_bound;
                if (eb) {
                    thr_comp = max(thr_comp, eb);
                    thr_f = fmaxf(thr_f, comp_floor_value(eb));
                }
            }
        }
        u64 lane_best = 0ull;
        if (GREEDY && best_col >= 0) {   // the first logit of the cell that equals its maximum (-0 and +0 are equal here and in a composite)
            const int e = best_cell.x == best ? 0 : best_cell.y == best ? 1 : best_cell.z == best ? 2 : 3;
            lane_best = make_comp(best, best_col + e + a.vocab_offset);
        }
        segment_end<SOFTCAP, GREEDY>(a, row, qn, nkept, thr_f, run_max, tile + seg_nt >= t_end, lane_best);
        tile += seg_nt;
    }
}

}  // namespace

size_t stream_kernel_smem_bytes() { return kSmemTotal; }

// Per-device set-up (the current device): opt in to the large dynamic shared memory; report resident CTAs per SM.
int prepare_device_kernels(int* ctas_per_sm) {
    cudaError_t e = cudaFuncSetAttribute(stream_select_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTotal);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(stream_select_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTotal);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(stream_select_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTotal);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(stream_select_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTotal);
    if (e != cudaSuccess) return (int)e;
    int n = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, stream_select_kernel<false, false>, kBlockThreads, kSmemTotal);
    if (e != cudaSuccess) return (int)e;
    if (ctas_per_sm) *ctas_per_sm = n;
    return 0;
}

int launch_stream_kernel(const StreamArgs& a, int grid, void* stream) {
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (a.overlap) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (a.pair) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)a.pair;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kBlockThreads);
    cfg.dynamicSmemBytes = kSmemTotal;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cfg.attrs = attr;
    cfg.numAttrs = n;
    if (a.all_greedy) {
        if (a.softcap != 0.0f) return (int)cudaLaunchKernelEx(&cfg, stream_select_kernel<true, true>, a);
        return (int)cudaLaunchKernelEx(&cfg, stream_select_kernel<false, true>, a);
    }
    if (a.softcap != 0.0f) return (int)cudaLaunchKernelEx(&cfg, stream_select_kernel<true, false>, a);
    return (int)cudaLaunchKernelEx(&cfg, stream_select_kernel<false, false>, a);
}

// The launch plan (host).  A row's scratch holds kMergeCap entries: k candidates and a count per segment.
Plan make_plan(int n_rows, int n_vocab, int kmax, int slots) {
    Plan pl;
    const int T = (n_vocab + kTile - 1) / kTile;
    pl.tiles_per_row = T;
    pl.total_tiles = n_rows * T;
    slots = std::max(1, slots);
    const int max_seg = std::max(2, kMergeCap / (std::max(1, kmax) + 1));
    const int q_min = (T + (max_seg - 1) - 1) / (max_seg - 1);
    const int q_fill = (pl.total_tiles + slots - 1) / slots;   // fewest tiles per CTA that still give a single wave
    int q = std::max(1, std::min(std::max(q_fill, q_min), kMaxTilesPerCta));
    if (T <= kMaxTilesPerCta && n_rows >= 2 * slots) {
        // Plenty of rows: one CTA per row, in waves.  Every CTA pays its start and its end-of-segment work once per row
        // and no row has to be merged.  The exception is a last wave that would be nearly empty (300 rows on 148 SMs:
        // two full waves and four CTAs): then one wave of CTAs each takes the same number of consecutive tiles, a little
        // more than two rows' worth, and a row that straddles two CTAs is merged through its scratch.  Measured on B200:
        // 300 x 262144 takes 101 us by rows and 87 us this way; with a last wave that is a third full or more the waves
        // win (512 rows: 138 against 141 us), because a thin last wave streams faster than a full one.
        const int rest = n_rows % slots;
        q = (rest > 0 && rest * 8 < slots) ? (pl.total_tiles + slots - 1) / slots : T;
    } else {
        // Otherwise a row is cut into nseg = T / q aligned pieces.  Fewer tiles per CTA shorten the streaming (per 32 KiB
        // tile about 0.4 us on a lone SM, 0.6 us when every SM streams), more pieces lengthen the merge: nothing for one
        // piece, the on-chip exchange inside a cluster of 2, 4 or 8 CTAs, ordered lists merged through scratch up to 16, a
        // gather-and-select beyond (measured on B200, in us).  Pick the cheapest q that divides the row and keeps
        // the grid within one wave.
        double best = 1e30;
        for (int c = q; c <= std::min(T, kMaxTilesPerCta); ++c) {
            if (T % c != 0) continue;
            const int nseg = T / c;
            const double busy = std::min(1.0, (double)n_rows * nseg / slots);
            const bool on_chip = (nseg == 2 || nseg == 4 || nseg == 8) && (nseg - 1) * std::max(1, kmax) <= 512;   // a cluster per row
            const double merge = nseg == 1 ? 0.0 : on_chip ? (nseg == 2 ? 1.4 : nseg == 4 ? 2.8 : 4.3)
                                 : nseg <= 8 ? 2.4 + 0.25 * nseg : nseg <= 16 ? 4.4 + 0.5 * nseg : 10.0 + 0.3 * nseg;
            const double cost = (0.4 + 0.2 * busy) * c + merge;
            if (cost < best) {
                best = cost;
                q = c;
            }
        }
    }
    pl.tiles_per_cta = q;
    pl.grid = (pl.total_tiles + q - 1) / q;
    return pl;
}

}  // namespace fsb

// ---------------------------------------------------------------------------------------------- fsb_argmax_rows_static
// Greedy tokens of device-resident rows with no allocation at all: the streaming kernel above, run with every piece
// of device memory it needs taken from one array that is part of this library's image.
namespace fsb {
namespace {

constexpr int kStaticMaxRows = FSB_STATIC_MAX_ROWS;
constexpr size_t kStaticRowsOff = 0;                                                       // RowDesc[kStaticMaxRows]
constexpr size_t kStaticFillOff = kStaticRowsOff + sizeof(RowDesc) * kStaticMaxRows;       // fill[], ticket[]: zero between calls
constexpr size_t kStaticStatusOff = kStaticFillOff + 2 * sizeof(uint32_t) * kStaticMaxRows;   // status word: zero between calls
constexpr size_t kStaticScratchOff = 8192;                                                 // [kStaticMaxRows][kMergeCap] candidates
constexpr size_t kStaticBytes = kStaticScratchOff + sizeof(u64) * (size_t)kMergeCap * kStaticMaxRows;
static_assert(kStaticStatusOff + sizeof(uint32_t) <= kStaticScratchOff, "descriptors, counters and status fit below the candidates");

// Zero when the library is loaded (static storage); every call starts by putting counters and status back to zero.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

constexpr int kStaticMaxDevices = 64;
struct StaticDevice {
    void* base = nullptr;   // device address of g_static_scratch on this device
    int slots = 0;          // CTAs of the streaming kernel that fit on the device at once
};
StaticDevice g_static_dev[kStaticMaxDevices];

// Row descriptors of plain greedy rows (no penalty window): row r starts at r * ld, its token goes to tokens[r].
// The kernel also clears the counters and the status word a previous call may have left set (a call that was not
// waited for and whose kernel reported an error): stream order puts this before the streaming kernel.
__global__ void static_greedy_rows_kernel(RowDesc* rows, int n_rows, int64_t ld, uint32_t* counters, int n_counter_words) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < n_counter_words) counters[r] = 0u;
    if (r >= n_rows) return;
    RowDesc d{};
    d.logits_off = (int64_t)r * ld;
    d.k = 1;
    d.temperature = 0.0f;
    d.top_p = 1.0f;
    d.penalty = 1.0f;
    d.flags = kRowGreedy;
    d.out_index = r;
    rows[r] = d;
}

}  // namespace
}  // namespace fsb

extern "C" int fsb_argmax_rows_static(int device, const float* logits_dev, int64_t ld, int n_rows, int n_vocab, int32_t* tokens_dev,
                                      void* cuda_stream, unsigned flags) {
    using namespace fsb;
    if (!logits_dev || !tokens_dev || n_rows < 0 || n_vocab <= 0 || ld < n_vocab || (flags & ~FSB_STATIC_WAIT)) return FSB_ERR_INVALID;
    if (n_rows > kStaticMaxRows) return FSB_ERR_CAPACITY;   // the static array holds FSB_STATIC_MAX_ROWS rows of scratch, no more
    if (device < 0 || device >= kStaticMaxDevices) return FSB_ERR_NO_DEVICE;
    if (n_rows == 0) return FSB_OK;
    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess) return FSB_ERR_NO_DEVICE;
    if (cudaSetDevice(device) != cudaSuccess) return FSB_ERR_NO_DEVICE;
    int rc = FSB_OK;
    StaticDevice& sd = g_static_dev[device];
    if (!sd.base) {   // first call on this device (it is current): where the array lives, how many CTAs fit
        void* p = nullptr;
        int per_sm = 0, sms = 0;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) rc = FSB_ERR_CUDA;
        if (rc == FSB_OK && prepare_device_kernels(&per_sm) != 0) rc = FSB_ERR_CUDA;
        if (rc == FSB_OK && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) rc = FSB_ERR_CUDA;
        if (rc == FSB_OK) {
            sd.slots = (sms > 0 ? sms : 1) * (per_sm > 0 ? per_sm : 1);
            sd.base = p;
        }
    }
    if (rc == FSB_OK) {
        unsigned char* base = static_cast<unsigned char*>(sd.base);
        cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
        RowDesc* rows = reinterpret_cast<RowDesc*>(base + kStaticRowsOff);
        const int n_counter_words = (int)((kStaticScratchOff - kStaticFillOff) / sizeof(uint32_t));   // fill[], ticket[], status
        static_greedy_rows_kernel<<<(n_counter_words + 63) / 64, 64, 0, st>>>(rows, n_rows, ld, reinterpret_cast<uint32_t*>(base + kStaticFillOff), n_counter_words);
        if (cudaGetLastError() != cudaSuccess) rc = FSB_ERR_CUDA;
        StreamArgs a{};
        a.logits = logits_dev;
        a.rows = rows;
        a.hist = nullptr;
        a.scratch = reinterpret_cast<uint64_t*>(base + kStaticScratchOff);
        a.ticket = reinterpret_cast<uint32_t*>(base + kStaticFillOff) + kStaticMaxRows;
        a.tokens = tokens_dev;
        a.status = reinterpret_cast<uint32_t*>(base + kStaticStatusOff);
        a.row_ld = ld;
        a.n_rows = n_rows;
        a.n_vocab = n_vocab;
        a.tiles_per_row = (n_vocab + kTile - 1) / kTile;
        a.total_tiles = n_rows * a.tiles_per_row;
        int q = (a.total_tiles + sd.slots - 1) / sd.slots;   // equal contiguous ranges of tiles, one per resident CTA
        q = q < 1 ? 1 : (q > kMaxTilesPerCta ? kMaxTilesPerCta : q);
        a.tiles_per_cta = q;
        a.all_greedy = 1;
        a.bulk_ok = ((reinterpret_cast<uintptr_t>(logits_dev) & 15u) == 0 && (ld & 3) == 0) ? 1 : 0;
        if (rc != FSB_OK) {
        } else if (2 * ((a.tiles_per_row + q - 1) / q + 1) > kMergeCap) {   // one candidate and one count per segment
            rc = FSB_ERR_CAPACITY;   // more segments per row than a row's scratch has entries (one candidate per segment)
        } else if (launch_stream_kernel(a, (a.total_tiles + q - 1) / q, st) != 0) {
            rc = FSB_ERR_CUDA;
        } else if (flags & FSB_STATIC_WAIT) {
            uint32_t status = 0;
            if (cudaMemcpyAsync(&status, a.status, sizeof status, cudaMemcpyDeviceToHost, st) != cudaSuccess ||
                cudaStreamSynchronize(st) != cudaSuccess) {
                rc = FSB_ERR_CUDA;
            } else if (status != 0u) {
                rc = FSB_ERR_DEVICE;
            }
        }
    }
    if (prev >= 0 && prev != device) cudaSetDevice(prev);
    return rc;
}
