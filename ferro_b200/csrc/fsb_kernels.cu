// fsb_kernels.cu - the streaming candidate kernel of the B200 batched token sampler (sm_100a).
//
// One launch samples every row of a batch whose effective k is at most kMaxK (greedy rows are k = 1):
//   repetition penalty (src/sampler.cpp:11-18) -> greedy argmax (:19-23) or top-k candidates (:25-35)
//   -> fp64 softmax (:37-41) -> min-p (:43) -> top-p (:44) -> seeded draw (:45-49).
// (reference paths are relative to the paragontasx/ferro project root)
//
// Work decomposition.  The [rows][n_vocab] matrix is cut into tiles of kTile logits; the flat list of tiles is
// dealt to CTAs in equal contiguous ranges, so every CTA streams the same number of bytes whatever the row
// count.  The part of a row that one CTA owns is a "segment".  Each logit is read from HBM exactly once, by a
// 1-D bulk asynchronous copy into a ring of kStages shared-memory tiles.  A segment keeps only the logits that
// can still belong to the row's top-k: a running admission bound (first taken from the per-thread maxima of the
// segment's first tile, later tightened by an exact radix selection whenever the candidate buffer fills) filters
// the stream with one float compare per logit.  When a segment ends it emits its k best candidates to a per-row
// scratch area and draws a ticket; the CTA that draws the row's last ticket merges the candidates and runs the
// row epilogue.  Nobody spins on another CTA: the only device-side wait is for this CTA's own bulk copies, and
// it is bounded.
#include <cuda_runtime.h>

#include "fsb_device.cuh"

namespace fsb {
namespace {

constexpr size_t kSmemStage = (size_t)kStages * kTile * sizeof(float);
constexpr size_t kSmemBuf = (size_t)kCap * sizeof(u64);
constexpr size_t kSmemKept = (size_t)kMaxK * sizeof(u64);
constexpr size_t kSmemOut = (size_t)kMaxK * sizeof(u64);
constexpr size_t kSmemBitmap = (size_t)kBitmapWords * sizeof(unsigned);
constexpr size_t kSmemTotal = kSmemStage + kSmemBuf + kSmemKept + kSmemOut + kSmemBitmap + sizeof(SharedCtl);
static_assert(kSmemTotal <= 115 * 1024, "two CTAs must fit into one SM's shared memory");
static_assert(kCap >= 4 * kMaxK, "the epilogue arrays alias the candidate buffer");
static_assert(kThreads == 256, "selection histogram assumes 256 threads");

constexpr long long kCopyWaitCycles = 2000000000ll;   // about 1 s: a bulk copy that has not landed by then is reported, not awaited

// A CTA tile of kTile logits is cut into one warp tile of kWTile logits per consumer warp; warp w owns the w-th
// of every CTA tile of its CTA.  One extra warp, the producer, brings the CTA tiles into a ring of kStages
// shared-memory slots, one bulk copy per tile; a consumer warp waits for a tile to land, works on its part on its
// own and hands the slot back.  Consumer warps therefore only meet at the ring (at most kStages tiles apart),
// never at a barrier while streaming, and never issue a copy themselves.
// Lane l of a consumer warp owns float4 number l + 32 * q (q = 0..3) of a warp tile; the candidates it admits go
// to a queue of kLaneQueue entries that only this lane writes, so admitting needs no atomics and no warp-wide step.
constexpr int kWarps = kThreads / 32;
constexpr int kWTile = kTile / kWarps;          // 512 logits = 2 KiB per bulk copy
constexpr int kBlockThreads = kThreads + 32;    // consumers + the producer warp
static_assert(kWTile == 512, "a lane owns four float4 of a warp tile");
static_assert(kLaneQueue >= 4, "a lane must be able to queue one float4 after a re-selection");
static_assert(kWarps <= 32, "one producer lane per consumer warp");

struct SegCtx {
    float pen;        // repetition penalty of the row
    float cap;        // softcap, 0 = off
    int has_pen;
    int id_base;      // token id of column 0
    float* wb_row;    // row base for write-back, or null
};

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
__device__ __forceinline__ void patch_tile(float* st, int len, int col0, const SegCtx& sc, const unsigned* bitmap, int bm_lo) {
    const int lane = threadIdx.x & 31;
    const int nw = (len + 31) >> 5;
    unsigned w = (lane < nw) ? bitmap[((col0 - bm_lo) >> 5) + lane] : 0u;
    if (__ballot_sync(0xffffffffu, w != 0u) == 0u) return;
    while (w) {
        const int off = 32 * lane + __ffs(w) - 1;
        w &= w - 1u;
        const float x = st[off];
        const float y = x > 0.0f ? __fdiv_rn(x, sc.pen) : __fmul_rn(x, sc.pen);
        st[off] = y;
        if (sc.wb_row) sc.wb_row[col0 + off] = y;
    }
    __syncwarp();
}

// Admission test of one logit: at or above the float bound and, once a re-selection has set a composite bound,
// not a tie at the bound that loses on token id.
__device__ __forceinline__ bool admitted(float x, int id, float thr_f, u64 thr_comp) {
    return x >= thr_f && (thr_comp == 0ull || make_comp(x, id) >= thr_comp);
}

// r-th largest of the 32 lane values of a warp (r in 1..32): r rounds of "warp maximum, strike one holder".
// -inf when fewer than r lanes hold a value above the filler.
__device__ __forceinline__ float warp_rth_largest(float v, int r) {
    const int lane = threadIdx.x & 31;
    unsigned cur = (v == v) ? float_key(v) : 0u;   // 0 ranks below every real logit
    unsigned top = 0u;
#pragma unroll 1
    for (int i = 0; i < r; ++i) {
        top = __reduce_max_sync(0xffffffffu, cur);
        const unsigned who = __ballot_sync(0xffffffffu, cur == top);
        if (lane == __ffs(who) - 1) cur = 0u;
    }
    return top == 0u ? -__int_as_float(0x7f800000) : key_float(top);
}

// Admission bound of the CTA from the per-lane running maxima: with r = ceil(k / warps), at least r logits of a
// warp's stream reach the r-th largest of its lanes' running maxima, so at least k logits of the segment reach
// the smallest of those values over the warps: no logit below it can be among the segment's k best.  Each warp
// posts its value; values only grow, so a reader may use another warp's older value without a barrier.
__device__ __forceinline__ float refresh_bound(float run_max, int k, SharedCtl* ctl) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float wb = warp_rth_largest(run_max, (k + kWarps - 1) / kWarps);
    volatile float* vb = ctl->wbound;
    if (lane == 0) vb[warp] = wb;
    __syncwarp();
    float t = vb[0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) t = fminf(t, vb[w]);
    return t;
}

// Diagnostics: slot 0 takes the global timer (ns) once, the others the SM cycle counter (cheap to read).
__device__ __forceinline__ void trace_mark(const StreamArgs& a, int slot) {
    if (a.trace && threadIdx.x == 0) {
        a.trace[(size_t)blockIdx.x * 8 + slot] = slot == 0 ? global_timer_ns() : (u64)clock64();
        if (slot == 0) a.trace[(size_t)blockIdx.x * 8 + 7] = (u64)clock64();
    }
}

// One rendez-vous of all consumer warps of the CTA.  A warp comes here either because one of its lanes had no room
// left in its queue (overflowed) or because it has finished its part of the segment.  If any warp overflowed, the
// CTA keeps the k best candidates (they move to the shared survivors' list, the queues become empty), tightens
// the admission bound, and the function returns true; it returns false when every warp had finished.  Every warp
// reaches one of the two call sites in bounded time on its own (while streaming, a consumer depends on nothing
// but its own copies), so the barrier cannot deadlock.
__device__ __noinline__ bool cta_event(bool overflowed, int k, const u64* myq, int* mycnt, u64* kept, int* nkept, u64* out,
                                       SharedCtl* ctl, unsigned* status, float* thr_f, u64* thr_comp) {
    if (overflowed) *reinterpret_cast<volatile int*>(&ctl->need_compact) = 1;
    consumer_sync();
    if (*reinterpret_cast<volatile int*>(&ctl->need_compact) == 0) return false;
    u64 L = 0ull;
    *nkept = select_topk(myq, *mycnt, kept, *nkept, k, out, kept, ctl, status, &L);
    *mycnt = 0;
    if (L != 0ull) {
        *thr_comp = L;
        *thr_f = fmaxf(*thr_f, comp_floor_value(L));
    }
    if (threadIdx.x == 0) ctl->need_compact = 0;
    consumer_sync();
    return true;
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
        if (i >= kStages && !mbar_test_wait(&ctl->empty[slot], (unsigned)((i / kStages - 1) & 1))) {
            if (clock64() - t_last > kCopyWaitCycles) {   // the consumers never came back: report and stop
                atomicOr(a.status, kStatusCopyTimeout);
                return;
            }
            __nanosleep(32);
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

template <bool SOFTCAP>
__global__ void __launch_bounds__(kBlockThreads, 2) stream_select_kernel(const StreamArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float* stage = reinterpret_cast<float*>(smem_raw);
    u64* buf = reinterpret_cast<u64*>(smem_raw + kSmemStage);   // kCap entries: the lanes' queues; contiguous list when merging
    u64* kept = buf + kCap;                                     // kMaxK entries: survivors of re-selections
    u64* out = kept + kMaxK;                                    // kMaxK entries: selection scratch
    unsigned* bitmap = reinterpret_cast<unsigned*>(out + kMaxK);
    SharedCtl* ctl = reinterpret_cast<SharedCtl*>(bitmap + kBitmapWords);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int T = a.tiles_per_row, V = a.n_vocab, Q = a.tiles_per_cta;
    const int t_begin = blockIdx.x * Q;
    const int t_end = min(t_begin + Q, a.total_tiles);
    const int nt = t_end - t_begin;
    if (nt <= 0) return;
    trace_mark(a, 0);

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
        if (a.bulk_ok) producer_loop(a, stage, ctl, t_begin, nt);
        return;
    }
    trace_mark(a, 1);

    // ------------------------------------------------------------------------------------------ consumers
    int row = t_begin / T, j = t_begin - row * T;
    u64* myq = buf + (size_t)warp * (32 * kLaneQueue) + lane;   // this lane's queue: entry s at myq[s * 32]

    const TailOut tout{a.tokens, a.kept_ids, a.kept_pr, a.kept_n, reinterpret_cast<u64*>(a.shard_out), a.shard_n, a.status};
    unsigned phase_bits = 0u;
    int cur_row = -1;
    RowDesc d;
    SegCtx sc;
    float thr_f = 0.0f, run_max = 0.0f;
    u64 thr_comp = 0ull;
    int bm_lo = 0, seg_it = 0;
    int mycnt = 0;    // entries in this lane's queue
    int nkept = 0;    // entries in the survivors' list (the same value in every thread)
    int dbg_events = 0;
    long long acc[6] = {0, 0, 0, 0, 0, 0}, tq, tn;

    for (int it = 0; it < nt; ++it) {
        const int col0 = j * kTile + warp * kWTile;          // first column of this warp's part
        const int len = max(0, min(kWTile, V - col0));
        const int slot = it % kStages;
        float* st = stage + (size_t)slot * kTile + warp * kWTile;   // this warp's part of the CTA tile
        const bool new_seg = (row != cur_row);

        if (new_seg) {   // ---- a new segment starts (all consumer warps are here together: kernel start or after a segment end)
            cur_row = row;
            d = a.rows[row];
            const int seg_lo_col = j * kTile;
            const int f_last = min(t_end, (row + 1) * T) - 1;
            const int seg_hi_col = min(V, (f_last - row * T + 1) * kTile);
            sc.pen = d.penalty;
            sc.cap = a.softcap;
            sc.has_pen = (d.flags & kRowPenalty) ? 1 : 0;
            sc.id_base = a.vocab_offset;
            sc.wb_row = a.write_back ? const_cast<float*>(a.logits) + d.logits_off : nullptr;
            bm_lo = seg_lo_col;
            if (sc.has_pen) {   // bitmap of the penalised columns of this segment
                const int words = (seg_hi_col - seg_lo_col + 31) >> 5;
                for (int i = tid; i < words; i += kThreads) bitmap[i] = 0u;
                consumer_sync();
                const int32_t* h = a.hist + d.hist_begin;
                for (int i = tid; i < d.hist_len; i += kThreads) {
                    const int c = h[i] - a.vocab_offset;
                    if (c >= seg_lo_col && c < seg_hi_col) atomicOr(&bitmap[(c - seg_lo_col) >> 5], 1u << ((c - seg_lo_col) & 31));
                }
            }
            mycnt = 0;
            nkept = 0;
            thr_comp = 0ull;
            thr_f = -__int_as_float(0x7f800000);
            run_max = -__int_as_float(0x7f800000);
            seg_it = 0;
            consumer_sync();
        }

        // ---- wait for the CTA tile's copy.  A warp that is waiting (or about to) also answers re-selection requests
        // of other warps: a requester sits at the barrier of cta_event, and the ring only moves when every warp does.
        tq = clock64();
        if (__any_sync(0xffffffffu, *reinterpret_cast<volatile int*>(&ctl->need_compact) != 0))
            cta_event(false, d.k, myq, &mycnt, kept, &nkept, out, ctl, a.status, &thr_f, &thr_comp);
        if (a.bulk_ok) {
            const unsigned par = (phase_bits >> slot) & 1u;
            const long long lim = ctl->abort ? 2000ll : kCopyWaitCycles;
            const long long t0 = clock64();
            while (!mbar_try_wait(&ctl->full[slot], par)) {
                if (__any_sync(0xffffffffu, *reinterpret_cast<volatile int*>(&ctl->need_compact) != 0)) {
                    cta_event(false, d.k, myq, &mycnt, kept, &nkept, out, ctl, a.status, &thr_f, &thr_comp);
                } else if (clock64() - t0 > lim) {   // the copy never landed: report, carry on with what is there
                    ctl->abort = 1;
                    atomicOr(a.status, kStatusCopyTimeout);
                    break;
                }
            }
            phase_bits ^= 1u << slot;
        } else if (len > 0) {   // rows not on 16-byte boundaries: the warp loads its tile itself
            const float* src = a.logits + d.logits_off + col0;
            for (int e = lane; e < len; e += 32) st[e] = src[e];
            __syncwarp();
        }
        if (len > 0) {
            if (SOFTCAP) softcap_tile(st, len, sc.cap, sc.wb_row ? sc.wb_row + col0 : nullptr);
            if (sc.has_pen && !(a.dbg & 8)) patch_tile(st, len, col0, sc, bitmap, bm_lo);
        }
        tn = clock64(); acc[0] += tn - tq; tq = tn;
        if (it == 0) trace_mark(a, 2);

        // ---- look: the lane's 16 logits go to registers (four independent 16-byte loads); what lies past the end of
        // a ragged row is made -inf first
        float4* st4 = reinterpret_cast<float4*>(st);
        if (len < kWTile) {
            for (int e = len + lane; e < kWTile; e += 32) st[e] = -__int_as_float(0x7f800000);
            __syncwarp();
        }
        float4 x0 = st4[lane], x1 = st4[lane + 32], x2 = st4[lane + 64], x3 = st4[lane + 96];
        const float m0 = fmaxf(max3(x0.x, x0.y, x0.z), x0.w);
        const float m1 = fmaxf(max3(x1.x, x1.y, x1.z), x1.w);
        const float m2 = fmaxf(max3(x2.x, x2.y, x2.z), x2.w);
        const float m3 = fmaxf(max3(x3.x, x3.y, x3.z), x3.w);
        run_max = fmaxf(max3(run_max, m0, m1), fmaxf(m2, m3));

        tn = clock64(); acc[1] += tn - tq; tq = tn;
        // ---- the admission bound: set at the segment's first tile (all warps must have posted: one barrier per
        // segment), then refreshed without a barrier at tiles 1, 2, 4, 8, ... of the segment
        if (new_seg) {
            const float wb = warp_rth_largest(run_max, (d.k + kWarps - 1) / kWarps);
            if (lane == 0) ctl->wbound[warp] = wb;
            consumer_sync();
            float t = ctl->wbound[0];
#pragma unroll
            for (int w = 1; w < kWarps; ++w) t = fminf(t, ctl->wbound[w]);
            thr_f = t;
            if (it == 0) trace_mark(a, 3);
        } else if ((seg_it & (seg_it - 1)) == 0 && !(a.dbg & 2)) {
            thr_f = fmaxf(thr_f, refresh_bound(run_max, d.k, ctl));
        }
        ++seg_it;

        tn = clock64(); acc[2] += tn - tq; tq = tn;
        // ---- admit: a lane looks closer only at those of its four float4 that hold a logit at or above the bound
        unsigned pend = (m0 >= thr_f ? 1u : 0u) | (m1 >= thr_f ? 2u : 0u) | (m2 >= thr_f ? 4u : 0u) | (m3 >= thr_f ? 8u : 0u);
        if (!(a.dbg & 1) && __any_sync(0xffffffffu, pend != 0u)) {
            acc[5] += 1;
            const int id_lane = col0 + 4 * lane + sc.id_base;   // token id of this lane's first logit
            const int lim = len - 4 * lane;                      // logits of the row from there on (ragged tiles)
            // queue the admitted logits of float4 number Q (X), unless the queue may not take four more
#define FSB_ADMIT_BLOCK(Q, X)                                                                      \
    if ((pend >> (Q)) & 1u) {                                                                      \
        if (mycnt + 4 <= kLaneQueue) {                                                             \
            pend &= ~(1u << (Q));                                                                  \
            if (0 + 128 * (Q) < lim && admitted((X).x, id_lane + 128 * (Q) + 0, thr_f, thr_comp)) myq[32 * mycnt++] = make_comp((X).x, id_lane + 128 * (Q) + 0); \
            if (1 + 128 * (Q) < lim && admitted((X).y, id_lane + 128 * (Q) + 1, thr_f, thr_comp)) myq[32 * mycnt++] = make_comp((X).y, id_lane + 128 * (Q) + 1); \
            if (2 + 128 * (Q) < lim && admitted((X).z, id_lane + 128 * (Q) + 2, thr_f, thr_comp)) myq[32 * mycnt++] = make_comp((X).z, id_lane + 128 * (Q) + 2); \
            if (3 + 128 * (Q) < lim && admitted((X).w, id_lane + 128 * (Q) + 3, thr_f, thr_comp)) myq[32 * mycnt++] = make_comp((X).w, id_lane + 128 * (Q) + 3); \
        }                                                                                          \
    }
            for (;;) {
                FSB_ADMIT_BLOCK(0, x0)
                FSB_ADMIT_BLOCK(1, x1)
                FSB_ADMIT_BLOCK(2, x2)
                FSB_ADMIT_BLOCK(3, x3)
                if (!__any_sync(0xffffffffu, pend != 0u)) break;
                // a lane's queue is full: the CTA re-selects, then the float4 still pending are looked at again
                cta_event(true, d.k, myq, &mycnt, kept, &nkept, out, ctl, a.status, &thr_f, &thr_comp);
                ++dbg_events;
                x0 = st4[lane];   // reloaded rather than kept alive across the call
                x1 = st4[lane + 32];
                x2 = st4[lane + 64];
                x3 = st4[lane + 96];
                pend &= (m0 >= thr_f ? 1u : 0u) | (m1 >= thr_f ? 2u : 0u) | (m2 >= thr_f ? 4u : 0u) | (m3 >= thr_f ? 8u : 0u);
            }
#undef FSB_ADMIT_BLOCK
        }
        __syncwarp();
        if (lane == 0 && a.bulk_ok) mbar_arrive(&ctl->empty[slot]);   // hand the slot back to the producer
        tn = clock64(); acc[3] += tn - tq;

        const bool seg_end = (it == nt - 1) || (j == T - 1);
        if (seg_end) {
            while (cta_event(false, d.k, myq, &mycnt, kept, &nkept, out, ctl, a.status, &thr_f, &thr_comp)) {
            }
            if (it == nt - 1) trace_mark(a, 4);
            if (it == nt - 1 && a.trace) { const int tot = __reduce_add_sync(0xffffffffu, mycnt); if (lane == 0) { atomicAdd((unsigned long long*)(a.trace + 4096 * 8 + (size_t)blockIdx.x * 8), (unsigned long long)tot); atomicAdd((unsigned long long*)(a.trace + 4096 * 8 + (size_t)blockIdx.x * 8 + 1), (unsigned long long)dbg_events); if (warp == 0) { uint64_t* t3 = a.trace + 4096 * 16 + (size_t)blockIdx.x * 8; for (int q = 0; q < 6; ++q) t3[q] = (uint64_t)acc[q]; a.trace[4096 * 8 + (size_t)blockIdx.x * 8 + 2] = (uint64_t)nkept; a.trace[4096 * 8 + (size_t)blockIdx.x * 8 + 3] = (uint64_t)__float_as_uint(thr_f); } } }
            // the segment's k best (or all, if fewer) go to the survivors' list, contiguous
            const int c = select_topk(myq, mycnt, kept, nkept, d.k, out, kept, ctl, a.status, nullptr);
            const int first_cta = (row * T) / Q, last_cta = (row * T + T - 1) / Q;
            const int nseg = last_cta - first_cta + 1;
            int total = c;
            bool merge_here = true;
            if (nseg > 1) {
                if (tid == 0) ctl->base = (int)atomicAdd(&a.fill[row], (unsigned)c);
                consumer_sync();
                const int base = ctl->base;
                u64* dst = reinterpret_cast<u64*>(a.scratch) + (size_t)row * kMergeCap;
                if (base + c <= kMergeCap) {
                    for (int i = tid; i < c; i += kThreads) dst[base + i] = kept[i];
                } else if (tid == 0) {
                    atomicOr(a.status, kStatusMergeOverflow);
                }
                __threadfence();
                consumer_sync();
                if (tid == 0) ctl->last = (atomicAdd(&a.ticket[row], 1u) == (unsigned)(nseg - 1)) ? 1 : 0;
                consumer_sync();
                merge_here = ctl->last != 0;
                if (merge_here) {   // all segments of the row have published: gather them (L2 reads, never L1)
                    __threadfence();
                    total = min((int)__ldcg(&a.fill[row]), kMergeCap);
                    for (int i = tid; i < total; i += kThreads) buf[i] = __ldcg(dst + i);
                    consumer_sync();
                    if (tid == 0) {   // leave the counters ready for the next launch
                        a.fill[row] = 0u;
                        a.ticket[row] = 0u;
                    }
                }
            } else {
                for (int i = tid; i < c; i += kThreads) buf[i] = kept[i];
                consumer_sync();
            }
            if (it == nt - 1) trace_mark(a, 5);
            if (merge_here) {
                const RowTail rt{d.rng_word, d.temperature, d.top_p, d.min_p, d.k, d.flags, d.out_index};
                finish_row(buf, total, rt, out, ctl, tout);
            }
            consumer_sync();
            if (it == nt - 1) trace_mark(a, 6);
        }
        if (++j == T) {
            j = 0;
            ++row;
        }
    }
}

// Merge of per-shard candidate lists (vocabulary-sharded mode): one CTA per row gathers n_lists sorted lists of
// up to kMaxK composites each (already in this device's memory) and runs the row epilogue.
__global__ void __launch_bounds__(kThreads, 2) merge_lists_kernel(const u64* lists, const int32_t* list_n, int n_lists, int n_rows,
                                                                 const RowDesc* rows, int32_t* tokens, int32_t* kept_ids,
                                                                 double* kept_pr, int32_t* kept_n, unsigned* status) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    u64* buf = reinterpret_cast<u64*>(smem_raw);
    u64* out = buf + kCap;
    SharedCtl* ctl = reinterpret_cast<SharedCtl*>(out + kMaxK);
    const int row = blockIdx.x, tid = threadIdx.x;
    if (row >= n_rows) return;
    const RowDesc d = rows[row];
    int total = 0;   // the same in every thread
    for (int g = 0; g < n_lists; ++g) {
        const int n = min(list_n[(size_t)g * n_rows + row], kMaxK);
        const u64* src = lists + ((size_t)g * n_rows + row) * kMaxK;
        if (total + n <= kCap) {
            for (int i = tid; i < n; i += kThreads) buf[total + i] = src[i];
            total += n;
        } else if (tid == 0) {
            atomicOr(status, kStatusMergeOverflow);
        }
    }
    consumer_sync();
    const TailOut tout{tokens, kept_ids, kept_pr, kept_n, nullptr, nullptr, status};
    const RowTail rt{d.rng_word, d.temperature, d.top_p, d.min_p, d.k, d.flags, d.out_index};
    finish_row(buf, total, rt, out, ctl, tout);
}

}  // namespace

size_t stream_kernel_smem_bytes() { return kSmemTotal; }

constexpr size_t kSmemMerge = kSmemBuf + kSmemOut + sizeof(SharedCtl);   // candidate list, selection scratch, control

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
    if (a.softcap != 0.0f) stream_select_kernel<true><<<grid, kBlockThreads, kSmemTotal, static_cast<cudaStream_t>(stream)>>>(a);
    else stream_select_kernel<false><<<grid, kBlockThreads, kSmemTotal, static_cast<cudaStream_t>(stream)>>>(a);
    return (int)cudaGetLastError();
}

int launch_merge_lists(const void* lists, const int32_t* list_n, int n_lists, int n_rows, const RowDesc* rows, int32_t* tokens,
                       int32_t* kept_ids, double* kept_pr, int32_t* kept_n, uint32_t* status, void* stream) {
    merge_lists_kernel<<<n_rows, kThreads, kSmemMerge, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const u64*>(lists), list_n, n_lists, n_rows, rows, tokens, kept_ids, kept_pr, kept_n, status);
    return (int)cudaGetLastError();
}

}  // namespace fsb
