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
constexpr size_t kSmemOut = (size_t)kMaxK * sizeof(u64);
constexpr size_t kSmemBitmap = (size_t)kBitmapWords * sizeof(unsigned);
constexpr size_t kSmemTotal = kSmemStage + kSmemBuf + kSmemOut + kSmemBitmap + sizeof(SharedCtl);
static_assert(kCap >= 4 * kMaxK, "the epilogue arrays alias the candidate buffer");
static_assert(kThreads == 256, "selection histogram assumes 256 threads");
static_assert(kTrigger > kMaxK, "a re-selection must always shrink the buffer");

constexpr u64 kCopyWaitNs = 1000000000ull;   // 1 s: a bulk copy that has not landed by then is reported, not awaited

struct SegCtx {
    float pen;        // repetition penalty of the row
    float cap;        // softcap, 0 = off
    int has_pen;
    int bm_lo;        // column of bit 0 of the bitmap
    int id_base;      // token id of column 0
    float* wb_row;    // row base for write-back, or null
};

__device__ __forceinline__ float xform(float x, unsigned bit, const SegCtx& c, int col) {
    if (c.cap != 0.0f) x = __fmul_rn(c.cap, tanhf(__fdiv_rn(x, c.cap)));                  // src/model_gemma4.cpp:521
    if (bit) x = x > 0.0f ? __fdiv_rn(x, c.pen) : __fmul_rn(x, c.pen);                    // src/sampler.cpp:17
    if (c.wb_row && (bit || c.cap != 0.0f)) c.wb_row[col] = x;
    return x;
}

__device__ __forceinline__ void admit(float x, int col, float thr_f, u64 thr_comp, u64* buf, SharedCtl* ctl, int id_base,
                                      unsigned* status) {
    if (x >= thr_f) {
        const u64 c = make_comp(x, col + id_base);
        if (c >= thr_comp) {
            const int p = atomicAdd(&ctl->cnt, 1);
            if (p < kCap) buf[p] = c;
            else atomicOr(status, kStatusCandOverflow);
        }
    }
}

__device__ __forceinline__ unsigned pen_bits(const unsigned* bitmap, const SegCtx& c, int col) {
    const int b = col - c.bm_lo;
    return c.has_pen ? (bitmap[b >> 5] >> (b & 31)) : 0u;
}

// Streaming pass over one tile in shared memory: transform (softcap, penalty) in registers, admit candidates.
template <bool XFORM>
__device__ __forceinline__ void scan_tile(const float* st, int len, int col0, const SegCtx& c, const unsigned* bitmap, float thr_f,
                                          u64 thr_comp, u64* buf, SharedCtl* ctl, unsigned* status) {
    const int tid = threadIdx.x;
    const int nvec = len >> 2;
    const float4* st4 = reinterpret_cast<const float4*>(st);
    const bool any_x = XFORM && (c.has_pen || c.cap != 0.0f);
#pragma unroll 4
    for (int v = tid; v < nvec; v += kThreads) {
        float4 x = st4[v];
        const int col = col0 + 4 * v;
        if (any_x) {
            const unsigned bits = pen_bits(bitmap, c, col) & 0xFu;
            if (bits || c.cap != 0.0f) {
                x.x = xform(x.x, bits & 1u, c, col);
                x.y = xform(x.y, bits & 2u, c, col + 1);
                x.z = xform(x.z, bits & 4u, c, col + 2);
                x.w = xform(x.w, bits & 8u, c, col + 3);
            }
        }
        const float m = fmaxf(fmaxf(x.x, x.y), fmaxf(x.z, x.w));
        if (m >= thr_f) {
            admit(x.x, col, thr_f, thr_comp, buf, ctl, c.id_base, status);
            admit(x.y, col + 1, thr_f, thr_comp, buf, ctl, c.id_base, status);
            admit(x.z, col + 2, thr_f, thr_comp, buf, ctl, c.id_base, status);
            admit(x.w, col + 3, thr_f, thr_comp, buf, ctl, c.id_base, status);
        }
    }
    if (tid < (len & 3)) {
        const int e = (len & ~3) + tid, col = col0 + e;
        float x = st[e];
        if (any_x) x = xform(x, pen_bits(bitmap, c, col) & 1u, c, col);
        admit(x, col, thr_f, thr_comp, buf, ctl, c.id_base, status);
    }
}

// First tile of a segment: transform in place in shared memory and return this thread's maximum as a composite
// (0 when the thread saw no element).  Elements are visited in ascending column order and replaced only by a
// strictly larger value, so the lowest column wins ties.
__device__ __forceinline__ u64 first_tile_max(float* st, int len, int col0, const SegCtx& c, const unsigned* bitmap) {
    const int tid = threadIdx.x;
    const int nvec = len >> 2;
    float4* st4 = reinterpret_cast<float4*>(st);
    const bool any_x = c.has_pen || c.cap != 0.0f;
    float m = 0.0f;
    int mcol = -1;
    for (int v = tid; v < nvec; v += kThreads) {
        float4 x = st4[v];
        const int col = col0 + 4 * v;
        if (any_x) {
            const unsigned bits = pen_bits(bitmap, c, col) & 0xFu;
            if (bits || c.cap != 0.0f) {
                x.x = xform(x.x, bits & 1u, c, col);
                x.y = xform(x.y, bits & 2u, c, col + 1);
                x.z = xform(x.z, bits & 4u, c, col + 2);
                x.w = xform(x.w, bits & 8u, c, col + 3);
                st4[v] = x;
            }
        }
        if (mcol < 0 || x.x > m) { m = x.x; mcol = col; }
        if (x.y > m) { m = x.y; mcol = col + 1; }
        if (x.z > m) { m = x.z; mcol = col + 2; }
        if (x.w > m) { m = x.w; mcol = col + 3; }
    }
    if (tid < (len & 3)) {
        const int e = (len & ~3) + tid, col = col0 + e;
        float x = st[e];
        if (any_x) {
            x = xform(x, pen_bits(bitmap, c, col) & 1u, c, col);
            st[e] = x;
        }
        if (mcol < 0 || x > m) { m = x; mcol = col; }
    }
    // threads without a usable maximum hand in distinct fillers that rank below every real logit
    return (mcol >= 0 && m == m) ? make_comp(m, mcol + c.id_base) : (u64)(kThreads - 1 - tid);
}

__global__ void __launch_bounds__(kThreads, 2) stream_select_kernel(const StreamArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float* stage = reinterpret_cast<float*>(smem_raw);
    u64* buf = reinterpret_cast<u64*>(smem_raw + kSmemStage);
    u64* out = buf + kCap;
    unsigned* bitmap = reinterpret_cast<unsigned*>(out + kMaxK);
    SharedCtl* ctl = reinterpret_cast<SharedCtl*>(bitmap + kBitmapWords);

    const int tid = threadIdx.x;
    const int T = a.tiles_per_row, V = a.n_vocab, Q = a.tiles_per_cta;
    const int t_begin = blockIdx.x * Q;
    const int t_end = min(t_begin + Q, a.total_tiles);
    const int nt = t_end - t_begin;
    if (nt <= 0) return;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&ctl->full[s], 1u);
        ctl->cnt = 0;
        ctl->abort = 0;
        fence_mbar_init();
    }
    __syncthreads();

    // Bring tile `it` of this CTA into its ring slot.  Called by all threads (uniform).
    auto issue = [&](int it) {
        const int f = t_begin + it;
        const int row = f / T, j = f - row * T;
        const int col0 = j * kTile;
        const int len = min(kTile, V - col0);
        const float* src = a.logits + a.rows[row].logits_off + col0;
        float* dst = stage + (size_t)(it % kStages) * kTile;
        if (a.bulk_ok) {
            if (tid == 0) {
                const unsigned bytes = (unsigned)(len & ~3) * 4u;
                if (bytes) {
                    fence_proxy_async_smem();   // earlier generic-proxy accesses to this slot precede the async write
                    mbar_expect_tx(&ctl->full[it % kStages], bytes);
                    bulk_g2s(dst, src, bytes, &ctl->full[it % kStages]);
                }
                for (int e = len & ~3; e < len; ++e) dst[e] = src[e];
            }
        } else {
            for (int e = tid; e < len; e += kThreads) dst[e] = src[e];
        }
    };

    const int pro = nt < kStages ? nt : kStages;
    for (int it = 0; it < pro; ++it) issue(it);
    __syncthreads();

    const TailOut tout{a.tokens, a.kept_ids, a.kept_pr, a.kept_n, reinterpret_cast<u64*>(a.shard_out), a.shard_n, a.status};
    unsigned phase_bits = 0u;
    int cur_row = -1;
    RowDesc d;
    SegCtx sc;
    float thr_f = 0.0f;
    u64 thr_comp = 0ull;
    bool first_tile = true;
    int seg_hi_col = 0;

    for (int it = 0; it < nt; ++it) {
        const int f = t_begin + it;
        const int row = f / T, j = f - row * T;
        const int col0 = j * kTile;
        const int len = min(kTile, V - col0);
        const int slot = it % kStages;

        if (row != cur_row) {   // ---- a new segment starts
            cur_row = row;
            d = a.rows[row];
            const int f_last = min(t_end, (row + 1) * T) - 1;
            seg_hi_col = min(V, (f_last - row * T + 1) * kTile);
            sc.pen = d.penalty;
            sc.cap = a.softcap;
            sc.has_pen = (d.flags & kRowPenalty) ? 1 : 0;
            sc.bm_lo = col0;
            sc.id_base = a.vocab_offset;
            sc.wb_row = a.write_back ? const_cast<float*>(a.logits) + d.logits_off : nullptr;
            if (sc.has_pen) {   // bitmap of the penalised columns of this segment; a bit is set once however often an id occurs
                const int words = (seg_hi_col - col0 + 31) >> 5;
                for (int i = tid; i < words; i += kThreads) bitmap[i] = 0u;
                __syncthreads();
                const int32_t* h = a.hist + d.hist_begin;
                for (int i = tid; i < d.hist_len; i += kThreads) {
                    const int c = h[i] - a.vocab_offset;
                    if (c >= col0 && c < seg_hi_col) atomicOr(&bitmap[(c - col0) >> 5], 1u << ((c - col0) & 31));
                }
            }
            if (tid == 0) ctl->cnt = 0;
            thr_f = -__int_as_float(0x7f800000);
            thr_comp = 0ull;
            first_tile = true;
            __syncthreads();
        }

        if (a.bulk_ok && (len & ~3)) {
            const u64 lim = ctl->abort ? 1000ull : kCopyWaitNs;
            if (!mbar_wait_bounded(&ctl->full[slot], (phase_bits >> slot) & 1u, lim)) {
                ctl->abort = 1;
                atomicOr(a.status, kStatusCopyTimeout);
            }
            phase_bits ^= 1u << slot;
        }
        float* st = stage + (size_t)slot * kTile;

        if (first_tile) {
            first_tile = false;
            buf[tid] = first_tile_max(st, len, col0, sc, bitmap);
            __syncthreads();
            if (d.k < kThreads) {
                thr_comp = select_topk(buf, kThreads, d.k, out, ctl, a.status);
                thr_f = comp_floor_value(thr_comp);
            } else {
                __syncthreads();
            }
            scan_tile<false>(st, len, col0, sc, bitmap, thr_f, thr_comp, buf, ctl, a.status);
        } else {
            scan_tile<true>(st, len, col0, sc, bitmap, thr_f, thr_comp, buf, ctl, a.status);
        }

        // every thread is done with the slot and with its admissions; the last arriver sees the final count
        const int need_sel = __syncthreads_or(*reinterpret_cast<volatile int*>(&ctl->cnt) > kTrigger);
        if (it + kStages < nt) issue(it + kStages);

        if (need_sel) {
            const int c = min(*reinterpret_cast<volatile int*>(&ctl->cnt), kCap);
            thr_comp = select_topk(buf, c, d.k, out, ctl, a.status);
            thr_f = comp_floor_value(thr_comp);
            if (tid == 0) ctl->cnt = d.k;
            __syncthreads();
        }

        const bool seg_end = (it == nt - 1) || ((f + 1) / T != row);
        if (seg_end) {
            int c = min(*reinterpret_cast<volatile int*>(&ctl->cnt), kCap);
            if (c > d.k) {
                select_topk(buf, c, d.k, out, ctl, a.status);
                c = d.k;
            }
            const int first_cta = (row * T) / Q, last_cta = (row * T + T - 1) / Q;
            const int nseg = last_cta - first_cta + 1;
            int total = c;
            bool merge_here = true;
            if (nseg > 1) {
                if (tid == 0) ctl->base = (int)atomicAdd(&a.fill[row], (unsigned)c);
                __syncthreads();
                const int base = ctl->base;
                u64* dst = reinterpret_cast<u64*>(a.scratch) + (size_t)row * kMergeCap;
                if (base + c <= kMergeCap) {
                    for (int i = tid; i < c; i += kThreads) dst[base + i] = buf[i];
                } else if (tid == 0) {
                    atomicOr(a.status, kStatusMergeOverflow);
                }
                __threadfence();
                __syncthreads();
                if (tid == 0) ctl->last = (atomicAdd(&a.ticket[row], 1u) == (unsigned)(nseg - 1)) ? 1 : 0;
                __syncthreads();
                merge_here = ctl->last != 0;
                if (merge_here) {   // all segments of the row have published: gather them (L2 reads, never L1)
                    __threadfence();
                    total = min((int)__ldcg(&a.fill[row]), kMergeCap);
                    for (int i = tid; i < total; i += kThreads) buf[i] = __ldcg(dst + i);
                    __syncthreads();
                    if (tid == 0) {   // leave the counters ready for the next launch
                        a.fill[row] = 0u;
                        a.ticket[row] = 0u;
                    }
                }
            }
            if (merge_here) {
                const RowTail rt{d.rng_word, d.temperature, d.top_p, d.min_p, d.k, d.flags, d.out_index};
                finish_row(buf, total, rt, out, ctl, tout);
            }
            __syncthreads();
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
    if (tid == 0) ctl->cnt = 0;
    __syncthreads();
    for (int g = 0; g < n_lists; ++g) {
        const int n = min(list_n[(size_t)g * n_rows + row], kMaxK);
        const u64* src = lists + ((size_t)g * n_rows + row) * kMaxK;
        const int base = ctl->cnt;
        __syncthreads();
        if (base + n <= kCap) {
            for (int i = tid; i < n; i += kThreads) buf[base + i] = src[i];
            if (tid == 0) ctl->cnt = base + n;
        } else if (tid == 0) {
            atomicOr(status, kStatusMergeOverflow);
        }
        __syncthreads();
    }
    const int total = ctl->cnt;
    __syncthreads();
    const TailOut tout{tokens, kept_ids, kept_pr, kept_n, nullptr, nullptr, status};
    const RowTail rt{d.rng_word, d.temperature, d.top_p, d.min_p, d.k, d.flags, d.out_index};
    finish_row(buf, total, rt, out, ctl, tout);
}

}  // namespace

size_t stream_kernel_smem_bytes() { return kSmemTotal; }

constexpr size_t kSmemMerge = kSmemBuf + kSmemOut + sizeof(SharedCtl);

// Per-device set-up (the current device): opt in to the large dynamic shared memory; report resident CTAs per SM.
int prepare_device_kernels(int* ctas_per_sm) {
    cudaError_t e = cudaFuncSetAttribute(stream_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTotal);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(merge_lists_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemMerge);
    if (e != cudaSuccess) return (int)e;
    int n = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, stream_select_kernel, kThreads, kSmemTotal);
    if (e != cudaSuccess) return (int)e;
    if (ctas_per_sm) *ctas_per_sm = n;
    return 0;
}

int launch_stream_kernel(const StreamArgs& a, int grid, void* stream) {
    stream_select_kernel<<<grid, kThreads, kSmemTotal, static_cast<cudaStream_t>(stream)>>>(a);
    return (int)cudaGetLastError();
}

int launch_merge_lists(const void* lists, const int32_t* list_n, int n_lists, int n_rows, const RowDesc* rows, int32_t* tokens,
                       int32_t* kept_ids, double* kept_pr, int32_t* kept_n, uint32_t* status, void* stream) {
    merge_lists_kernel<<<n_rows, kThreads, kSmemMerge, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const u64*>(lists), list_n, n_lists, n_rows, rows, tokens, kept_ids, kept_pr, kept_n, status);
    return (int)cudaGetLastError();
}

}  // namespace fsb
