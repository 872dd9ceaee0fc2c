// fsb_shim.cpp - host side of the C ABI declared in include/ferro_sampler_b200.h.
//
// Keeps what the reference keeps on the host, per stream: the parameter struct and the std::mt19937_64 engine
// (src/sampler.h:30-32 of paragontasx/ferro), so the draws come from the reference's own random stream by
// construction.  Everything that touches logits runs in the CUDA kernels; there is no host implementation of
// the sampling path in this file.
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <random>
#include <string>
#include <vector>

#include "../../include/ferro_sampler_b200.h"
#include "fsb_internal.h"

static_assert(sizeof(ferro_sampler_params) == 40, "parameter struct must match the reference's 40-byte SamplerParams");
static_assert(offsetof(ferro_sampler_params, seed) == 32, "seed sits at offset 32 in the reference struct");
static_assert(FSB_MAX_CANDIDATE_K == fsb::kMaxK, "header constant out of step with the kernel geometry");

namespace {

struct Stream {
    ferro_sampler_params p{};
    std::mt19937_64 rng;
    uint64_t seed_used = 0;
    uint64_t draws = 0;
    bool open = false;
    // device-resident history (optional): a host mirror, and a region [pool_off, pool_off + 2^pool_class) of the
    // engine's id pool that holds its first dev_len ids
    std::vector<int32_t> hist;
    int64_t pool_off = -1;
    int pool_class = -1;
    int64_t dev_len = 0;
    uint64_t seen = 0;   // number of the last call that listed this stream (a stream may appear once per call)
};

}  // namespace

struct fsb_batch {
    int n_rows = 0, n_vocab = 0;
    int64_t ld = 0;
    unsigned flags = 0;
    int cap_rows = 0;
    int64_t cap_hist = 0;
    int n_cand = 0, n_full = 0;   // rows of the candidate kernel / of the full-row kernel
    int kmax = 1;
    bool all_greedy = false;      // every row of the streaming kernel is greedy
    fsb::Plan plan;               // how the candidate rows are dealt to the CTAs of the streaming kernel
    int64_t hist_ids = 0;         // window ids staged with the batch
    int64_t gather_ids = 0;       // window values a write-back for a host caller brings back
    int64_t table_ints = 0;       // int32 words of the per-stream table of a resident verification call, staged behind the window ids
    // pinned host staging: [RowDesc x cap_rows][int32 x cap_hist], tokens, gathered window values
    unsigned char* h_in = nullptr;
    int32_t* h_tokens = nullptr;
    int32_t* h_tokens_dev = nullptr;   // the device's address of h_tokens (pinned memory is mapped): kernels mirror tokens and a status flag there
    bool mirrored = false;            // the last launch wrote the mirror: tokens need no copy back
    float* h_patched = nullptr;
    // device
    unsigned char* d_in = nullptr;
    int32_t* d_tokens = nullptr;
    float* d_patched = nullptr;
    std::vector<int> sid;
    std::vector<unsigned char> stochastic;
    std::vector<fsb::RowDesc> descs;   // descriptors in row order while a batch is staged (capacity kept between calls)
    bool launched = false;
    const int32_t* hist_dev = nullptr;   // where the rows' penalty windows live: the batch's staged copy, or the engine's id pool

    fsb::RowDesc* h_rows() const { return reinterpret_cast<fsb::RowDesc*>(h_in); }
    int32_t* h_hist() const { return reinterpret_cast<int32_t*>(h_in + sizeof(fsb::RowDesc) * (size_t)cap_rows); }
    // where the kernels read the descriptors: the device copy, or the pinned host block itself through its device address
    // (see upload_batch)
    fsb::RowDesc* d_rows() const { return rows_from_host ? reinterpret_cast<fsb::RowDesc*>(h_in_dev) : reinterpret_cast<fsb::RowDesc*>(d_in); }
    unsigned char* h_in_dev = nullptr;
    bool rows_from_host = false;
    int32_t* d_hist() const { return reinterpret_cast<int32_t*>(d_in + sizeof(fsb::RowDesc) * (size_t)cap_rows); }
    // the kernels' status word sits right behind the tokens, so that one copy brings both back
    uint32_t* d_status() const { return reinterpret_cast<uint32_t*>(d_tokens + cap_rows); }
    size_t in_bytes_used() const { return sizeof(fsb::RowDesc) * (size_t)cap_rows + sizeof(int32_t) * (size_t)(hist_ids + table_ints); }
};

struct fsb_handle {
    int device = 0;
    int max_rows = 0, max_vocab = 0;
    int64_t max_hist = 0;
    int sm_count = 0, ctas_per_sm = 0;
    int pair_ok = 1;                   // clusters of CTAs can be launched on this device
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    cudaStream_t side = nullptr;       // the full-vocabulary kernel of a mixed batch runs here, beside the streaming kernel
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    float softcap = 0.0f;
    int32_t vocab_offset = 0;
    int32_t global_vocab = 0;          // vocabulary sharding: columns of the whole row (0: this engine holds whole rows)
    int launch_overlap = 0;
    uint64_t call_no = 0;              // counts the calls that check their streams for duplicates
    std::vector<Stream> streams;
    std::vector<int> free_ids;
    // device scratch shared by all batches of this handle
    uint64_t* d_scratch = nullptr;     // [max_rows][kMergeCap] candidates the segments of a row publish
    uint32_t* d_counters = nullptr;    // [max_rows] tickets: all zero between launches
    int32_t* d_kept_ids = nullptr;
    double* d_kept_pr = nullptr;
    int32_t* d_kept_n = nullptr;
    bool kept_valid = false;
    // prompt-lookup drafting: descriptors up, drafts down (pinned host copies beside the device arrays)
    fsb::LookupDesc* h_lookup = nullptr;
    fsb::LookupDesc* d_lookup = nullptr;
    int32_t* h_drafts = nullptr;
    int32_t* d_drafts = nullptr;
    float* d_logits_stage = nullptr;   // device copy of host logits: max_rows x max_vocab, allocated with the engine
    size_t logits_stage_elems = 0;
    uint64_t* d_trace = nullptr;       // caller-owned diagnostics buffer, or null
    fsb_batch* own = nullptr;          // the batch behind fsb_sample_batch / fsb_verify_windows
    int32_t* d_pool = nullptr;         // resident histories: max_hist ids, carved into power-of-two regions
    int64_t pool_top = 0;              // ids handed out so far (bump pointer)
    std::vector<std::vector<int64_t>> pool_free;   // freed regions by size class
    fsb_counters_t counters{};
    std::string err;

    size_t counter_words() const { return (size_t)max_rows; }
};

namespace {

int fail(fsb_handle* h, int code, const char* fmt, ...) {
    if (h) {
        char tmp[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(tmp, sizeof tmp, fmt, ap);
        va_end(ap);
        h->err = tmp;
    }
    return code;
}

#define FSB_CUDA(h, call)                                                                                  \
    do {                                                                                                   \
        cudaError_t e_ = (call);                                                                           \
        if (e_ != cudaSuccess) return fail(h, FSB_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_));      \
    } while (0)

bool is_greedy(const ferro_sampler_params& p) { return p.temperature <= 0.0f || p.top_k == 1; }   // src/sampler.cpp:19

// penalty window [b, len) of src/sampler.cpp:11-14; returns len when the window is empty or the penalty is off
int64_t window_begin(const ferro_sampler_params& p, int64_t len) {
    if (p.repetition_penalty == 1.0f || p.repeat_last_n == 0 || len <= 0) return len;
    int64_t b = (p.repeat_last_n > 0 && (int64_t)p.repeat_last_n < len) ? len - (int64_t)p.repeat_last_n : 0;
    if (p.penalty_from > 0) b = std::max<int64_t>(b, (int64_t)p.penalty_from);
    return std::min(b, len);
}

void free_batch_buffers(fsb_batch* b) {
    if (!b) return;
    if (b->h_in) cudaFreeHost(b->h_in);
    if (b->h_tokens) cudaFreeHost(b->h_tokens);
    if (b->h_patched) cudaFreeHost(b->h_patched);
    if (b->d_in) cudaFree(b->d_in);
    if (b->d_tokens) cudaFree(b->d_tokens);
    if (b->d_patched) cudaFree(b->d_patched);
    b->h_in = nullptr; b->h_tokens = nullptr; b->h_patched = nullptr; b->d_in = nullptr; b->d_tokens = nullptr; b->d_patched = nullptr;
}

// `patched` > 0: also buffers for that many gathered window values (write-back for host callers).
int alloc_batch(fsb_handle* h, int cap_rows, int64_t cap_hist, int64_t patched, fsb_batch** out) {
    fsb_batch* b = new (std::nothrow) fsb_batch();
    if (!b) return fail(h, FSB_ERR_INVALID, "out of host memory");
    b->cap_rows = cap_rows;
    b->cap_hist = std::max<int64_t>(cap_hist, 1);
    cap_hist = b->cap_hist + (int64_t)fsb::kWindowTableInts * cap_rows;   // room for the table of a resident verification call
    b->descs.reserve((size_t)cap_rows);
    b->sid.reserve((size_t)cap_rows);
    b->stochastic.reserve((size_t)cap_rows);
    const size_t in_bytes = sizeof(fsb::RowDesc) * (size_t)cap_rows + sizeof(int32_t) * (size_t)cap_hist;
    cudaError_t e = cudaMallocHost(reinterpret_cast<void**>(&b->h_in), in_bytes);
    if (e == cudaSuccess) e = cudaMallocHost(reinterpret_cast<void**>(&b->h_tokens), sizeof(int32_t) * ((size_t)cap_rows + 1));
    if (e == cudaSuccess && cudaHostGetDevicePointer(reinterpret_cast<void**>(&b->h_in_dev), b->h_in, 0) != cudaSuccess) {
        b->h_in_dev = nullptr;
        cudaGetLastError();
    }
    if (e == cudaSuccess && cudaHostGetDevicePointer(reinterpret_cast<void**>(&b->h_tokens_dev), b->h_tokens, 0) != cudaSuccess) {
        b->h_tokens_dev = nullptr;   // no mapping on this system: tokens come back by copy
        cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&b->d_in), in_bytes);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&b->d_tokens), sizeof(int32_t) * ((size_t)cap_rows + 1));
    if (e == cudaSuccess) e = cudaMemset(b->d_tokens, 0, sizeof(int32_t) * ((size_t)cap_rows + 1));
    if (e == cudaSuccess && patched > 0) e = cudaMallocHost(reinterpret_cast<void**>(&b->h_patched), sizeof(float) * (size_t)patched);
    if (e == cudaSuccess && patched > 0) e = cudaMalloc(reinterpret_cast<void**>(&b->d_patched), sizeof(float) * (size_t)patched);
    if (e != cudaSuccess) {
        free_batch_buffers(b);
        delete b;
        return fail(h, FSB_ERR_CUDA, "batch allocation: %s", cudaGetErrorString(e));
    }
    *out = b;
    return FSB_OK;
}

Stream* get_stream(fsb_handle* h, int sid) {
    if (sid < 0 || sid >= (int)h->streams.size() || !h->streams[(size_t)sid].open) return nullptr;
    return &h->streams[(size_t)sid];
}

// `n_vocab` = the columns this engine holds; with vocabulary sharding the row's candidate count follows the whole
// row's width (src/sampler.cpp:27 with n = the global vocabulary), the shard's its own.
void fill_desc(const fsb_handle* h, fsb::RowDesc& d, const ferro_sampler_params& p, int n_vocab, int64_t logits_off, int64_t hist_begin,
               int64_t hist_len, uint64_t word, int out_index) {
    std::memset(&d, 0, sizeof d);
    d.rng_word = word;
    d.logits_off = logits_off;
    d.hist_begin = hist_begin;
    d.hist_len = (int32_t)hist_len;
    const bool greedy = is_greedy(p);
    const int n_global = h->global_vocab > 0 ? h->global_vocab : n_vocab;
    d.k = greedy ? 1 : ((p.top_k > 0 && p.top_k < n_vocab) ? p.top_k : n_vocab);   // src/sampler.cpp:27
    d.k_global = greedy ? 1 : ((p.top_k > 0 && p.top_k < n_global) ? p.top_k : n_global);
    d.temperature = p.temperature;
    d.top_p = p.top_p;
    d.min_p = p.min_p;
    d.penalty = p.repetition_penalty;
    d.flags = (greedy ? fsb::kRowGreedy : 0) | (hist_len > 0 ? fsb::kRowPenalty : 0);
    d.out_index = out_index;
    d.gather_off = 0;
}

// Orders the staged descriptors: candidate-path rows first, full-row-path rows after; fixes the launch plan.
int finalize_batch(fsb_handle* h, fsb_batch* b) {
    int n_cand = 0, kmax = 1;
    fsb::RowDesc* dst = b->h_rows();
    auto on_chip = [](const fsb::RowDesc& d) { return d.k <= fsb::kMaxK && d.k_global <= fsb::kMaxK; };
    bool all_greedy = true;
    for (const auto& d : b->descs)
        if (on_chip(d)) {
            dst[n_cand++] = d;
            kmax = std::max(kmax, d.k);
            all_greedy = all_greedy && (d.flags & fsb::kRowGreedy) != 0;
        }
    b->all_greedy = all_greedy && n_cand > 0;
    int n_full = 0;
    for (const auto& d : b->descs)
        if (!on_chip(d)) dst[n_cand + n_full++] = d;
    b->n_cand = n_cand;
    b->n_full = n_full;
    b->kmax = kmax;
    b->plan = fsb::make_plan(std::max(n_cand, 1), b->n_vocab, kmax, std::max(1, h->sm_count * std::max(1, h->ctas_per_sm)));
    return FSB_OK;
}

// Sends what the kernels need to know about the batch.  `lone_launch`: the sampling kernels are the only readers of the
// descriptors (nothing is appended, gathered or drafted on the device afterwards).  Then, if only descriptors are to be
// sent, the batch is one wave of CTAs and long enough to hide a read across PCIe behind its first tiles (measured on
// B200: 64 x 262144 gains 6 us per call, 8 x 65536 nothing, one row loses 2 us), nothing is copied at all: the kernels
// read the descriptors from the pinned host block.
int upload_batch(fsb_handle* h, fsb_batch* b, bool lone_launch = false) {
    // descriptors, then (behind room for cap_rows of them) window ids and tables: one copy, cut short when only descriptors go up
    b->rows_from_host = false;
    if (lone_launch && b->hist_ids + b->table_ints == 0 && b->h_in_dev && b->n_rows <= h->sm_count &&
        (int64_t)b->n_rows * b->n_vocab >= ((int64_t)4 << 20)) {
        b->rows_from_host = true;
        return FSB_OK;
    }
    const size_t bytes = (b->hist_ids + b->table_ints == 0) ? sizeof(fsb::RowDesc) * (size_t)b->n_rows : b->in_bytes_used();
    FSB_CUDA(h, cudaMemcpyAsync(b->d_in, b->h_in, bytes, cudaMemcpyHostToDevice, h->stream));
    return FSB_OK;
}

int launch_batch(fsb_handle* h, fsb_batch* b, const float* logits_dev, bool keep_kept, uint64_t* shard_out = nullptr,
                 int32_t* shard_n = nullptr, int shard_stride = fsb::kMaxK, bool mirror = false) {
    // `mirror`: the caller is about to wait for the tokens - the kernels store them (and a flag for any status bit) into
    // the batch's pinned host words as well, and fetch_tokens only waits for the stream
    int32_t* tokens_host = (mirror && b->h_tokens_dev) ? b->h_tokens_dev : nullptr;
    uint32_t* status_host = tokens_host ? reinterpret_cast<uint32_t*>(tokens_host + b->cap_rows) : nullptr;
    if (tokens_host) b->h_tokens[b->cap_rows] = 0;
    b->mirrored = tokens_host != nullptr;
    if (shard_out && b->n_full > 0)
        return fail(h, FSB_ERR_RANGE, "rows whose candidate count exceeds %d (top_k = 0 or large) cannot be sharded by vocabulary", fsb::kMaxK);
    const int32_t* hist = b->hist_dev ? b->hist_dev : b->d_hist();
    // A mixed batch runs its two kernels side by side (they touch different rows): the full-vocabulary kernel, the
    // longer of the two, goes first, on the side stream, behind everything already queued on the engine's stream.
    const bool side_by_side = b->n_full > 0 && b->n_cand > 0;
    if (b->n_full > 0) {
        cudaStream_t where = h->stream;
        if (side_by_side) {
            FSB_CUDA(h, cudaEventRecord(h->ev_fork, h->stream));
            FSB_CUDA(h, cudaStreamWaitEvent(h->side, h->ev_fork, 0));
            where = h->side;
        }
        const int e = fsb::launch_full_row_kernel(logits_dev, b->d_rows() + b->n_cand, b->n_full, hist, b->d_tokens, tokens_host,
                                                  h->d_kept_ids, h->d_kept_pr, h->d_kept_n, keep_kept ? 1 : 0, b->d_status(), status_host, b->n_vocab, h->vocab_offset,
                                                  (b->flags & FSB_WRITE_BACK) ? 1 : 0, h->softcap, h->d_trace ? h->d_trace + 4096 * 8 : nullptr, where);
        if (e != 0) return fail(h, FSB_ERR_CUDA, "full-row kernel launch: %s", cudaGetErrorString((cudaError_t)e));
        h->counters.kernel_launches++;
        if (side_by_side) FSB_CUDA(h, cudaEventRecord(h->ev_join, h->side));
    }
    if (b->n_cand > 0) {
        fsb::StreamArgs a{};
        a.logits = logits_dev;
        a.rows = b->d_rows();
        a.hist = hist;
        a.scratch = h->d_scratch;
        a.ticket = h->d_counters;
        a.tokens = b->d_tokens;
        a.status = b->d_status();
        a.tokens_host = tokens_host;
        a.status_host = status_host;
        a.kept_ids = keep_kept ? h->d_kept_ids : nullptr;
        a.kept_pr = keep_kept ? h->d_kept_pr : nullptr;
        a.kept_n = keep_kept ? h->d_kept_n : nullptr;
        a.shard_out = shard_out;
        a.shard_n = shard_n;
        a.shard_stride = shard_stride;
        a.trace = h->d_trace;
        a.row_ld = (b->n_full == 0) ? b->ld : -1;   // descriptors are in row order when every row takes this kernel
        a.n_rows = b->n_cand;
        a.n_vocab = b->n_vocab;
        a.tiles_per_row = b->plan.tiles_per_row;
        a.tiles_per_cta = b->plan.tiles_per_cta;
        a.total_tiles = b->n_cand * b->plan.tiles_per_row;
        a.bulk_ok = ((reinterpret_cast<uintptr_t>(logits_dev) & 15u) == 0 && (b->ld & 3) == 0) ? 1 : 0;
        a.write_back = (b->flags & FSB_WRITE_BACK) ? 1 : 0;
        a.vocab_offset = h->vocab_offset;
        a.softcap = h->softcap;
        a.overlap = h->launch_overlap;
        a.all_greedy = b->all_greedy ? 1 : 0;
        const int grid = (a.total_tiles + a.tiles_per_cta - 1) / a.tiles_per_cta;
        // rows of exactly 2, 4 or 8 aligned segments: the CTAs of a row run as a cluster and exchange candidates on chip
        a.pair = 0;
        for (int c = 2; c <= 8; c *= 2)   // receive buffer: (c - 1) lists of kmax entries in 512
            if (h->pair_ok && a.tiles_per_row == c * a.tiles_per_cta && grid == c * a.n_rows && (c - 1) * b->kmax <= 512) a.pair = c;
        const int e = fsb::launch_stream_kernel(a, grid, h->stream);
        if (e != 0) return fail(h, FSB_ERR_CUDA, "stream kernel launch: %s", cudaGetErrorString((cudaError_t)e));
        h->counters.kernel_launches++;
    }
    if (side_by_side) FSB_CUDA(h, cudaStreamWaitEvent(h->stream, h->ev_join, 0));
    b->launched = true;
    h->kept_valid = keep_kept;
    return FSB_OK;
}

// Tokens and the status word behind them in one copy; `extra` floats of gathered window values in a second one.
int fetch_tokens(fsb_handle* h, fsb_batch* b, int32_t* tokens_out, int64_t patched = 0) {
    if (!b->mirrored)
        FSB_CUDA(h, cudaMemcpyAsync(b->h_tokens, b->d_tokens, sizeof(int32_t) * ((size_t)b->cap_rows + 1), cudaMemcpyDeviceToHost, h->stream));
    if (patched > 0) FSB_CUDA(h, cudaMemcpyAsync(b->h_patched, b->d_patched, sizeof(float) * (size_t)patched, cudaMemcpyDeviceToHost, h->stream));
    FSB_CUDA(h, cudaStreamSynchronize(h->stream));
    unsigned st = (unsigned)b->h_tokens[b->cap_rows];
    if (st != 0u && b->mirrored) {   // the mirror only says "something": the device word has the bits
        uint32_t word = 0;
        if (cudaMemcpy(&word, b->d_status(), sizeof word, cudaMemcpyDeviceToHost) == cudaSuccess && word != 0u) st = word;
    }
    if (st != 0u) {
        // put the self-resetting counters and the status word back into their idle state
        cudaMemsetAsync(h->d_counters, 0, sizeof(uint32_t) * h->counter_words(), h->stream);
        cudaMemsetAsync(b->d_status(), 0, sizeof(uint32_t), h->stream);
        cudaStreamSynchronize(h->stream);
        return fail(h, FSB_ERR_DEVICE, "kernel status 0x%x (1 wait timeout, 4 merge overflow, 8 row without a finite logit)", st);
    }
    if (tokens_out) std::memcpy(tokens_out, b->h_tokens, sizeof(int32_t) * (size_t)b->n_rows);
    return FSB_OK;
}

int check_common(fsb_handle* h, int n_rows, int64_t ld, int n_vocab, const fsb_batch* b) {
    if (n_rows <= 0) return fail(h, FSB_ERR_INVALID, "n_rows must be positive");
    if (n_vocab <= 0) return fail(h, FSB_ERR_INVALID, "n_vocab must be positive");
    if (ld < n_vocab) return fail(h, FSB_ERR_INVALID, "row stride ld is smaller than n_vocab");
    if (n_rows > b->cap_rows) return fail(h, FSB_ERR_CAPACITY, "%d rows exceed the capacity of %d", n_rows, b->cap_rows);
    if (n_rows > h->max_rows) return fail(h, FSB_ERR_CAPACITY, "%d rows exceed the engine's %d", n_rows, h->max_rows);
    if (n_vocab > h->max_vocab) return fail(h, FSB_ERR_CAPACITY, "n_vocab %d exceeds the engine's %d", n_vocab, h->max_vocab);
    return FSB_OK;
}

// ---- resident histories: regions of the engine's id pool, sizes 2^class ids (class >= 8) ----------------------
void release_region(fsb_handle* h, Stream* s) {
    if (s->pool_off >= 0) {
        if ((size_t)s->pool_class >= h->pool_free.size()) h->pool_free.resize((size_t)s->pool_class + 1);
        h->pool_free[(size_t)s->pool_class].push_back(s->pool_off);
    }
    s->pool_off = -1;
    s->pool_class = -1;
    s->dev_len = 0;
}

// Makes sure the stream's region holds at least `need` ids; moves what is already on the device if it must grow.
int ensure_region(fsb_handle* h, Stream* s, int64_t need) {
    if (s->pool_off >= 0 && need <= ((int64_t)1 << s->pool_class)) return FSB_OK;
    int c = 8;
    while (((int64_t)1 << c) < need) ++c;
    int64_t off = -1;
    if ((size_t)c < h->pool_free.size() && !h->pool_free[(size_t)c].empty()) {
        off = h->pool_free[(size_t)c].back();
        h->pool_free[(size_t)c].pop_back();
    } else if (h->pool_top + ((int64_t)1 << c) <= h->max_hist) {
        off = h->pool_top;
        h->pool_top += (int64_t)1 << c;
    } else {
        return fail(h, FSB_ERR_CAPACITY, "resident histories need %lld more ids than the engine's pool of %lld holds", (long long)((int64_t)1 << c),
                    (long long)h->max_hist);
    }
    if (s->pool_off >= 0 && s->dev_len > 0)
        FSB_CUDA(h, cudaMemcpyAsync(h->d_pool + off, h->d_pool + s->pool_off, sizeof(int32_t) * (size_t)s->dev_len, cudaMemcpyDeviceToDevice, h->stream));
    const int64_t kept = s->dev_len;
    release_region(h, s);
    s->pool_off = off;
    s->pool_class = c;
    s->dev_len = kept;
    return FSB_OK;
}

// Brings the device copy of the stream's history up to date with its host mirror.
int sync_history(fsb_handle* h, Stream* s) {
    const int64_t n = (int64_t)s->hist.size();
    if (n <= s->dev_len) return FSB_OK;
    const int rc = ensure_region(h, s, n);
    if (rc) return rc;
    FSB_CUDA(h, cudaMemcpyAsync(h->d_pool + s->pool_off + s->dev_len, s->hist.data() + s->dev_len, sizeof(int32_t) * (size_t)(n - s->dev_len),
                                cudaMemcpyHostToDevice, h->stream));
    FSB_CUDA(h, cudaStreamSynchronize(h->stream));   // the source is pageable host memory that may change after return
    s->dev_len = n;
    return FSB_OK;
}

// A call that fails after its rows were staged has consumed engine outputs without returning tokens: the engines of
// its stochastic rows are put back, so that the streams stay in step with the reference's.
void rollback_draws(fsb_handle* h, const fsb_batch* b) {
    for (int i = 0; i < b->n_rows && i < (int)b->sid.size(); ++i) {
        if (!b->stochastic[(size_t)i]) continue;
        Stream* s = get_stream(h, b->sid[(size_t)i]);
        if (!s || s->draws == 0) continue;
        s->draws--;
        s->rng.seed(s->seed_used);
        s->rng.discard(s->draws);
    }
}

// Stages rows "stream_ids[i] samples row i with history i" into batch b.  Consumes engine outputs.
int stage_rows(fsb_handle* h, fsb_batch* b, int n_rows, const int* stream_ids, int64_t ld, int n_vocab, const int32_t* hist_flat,
               const int64_t* hist_off, unsigned flags) {
    int rc = check_common(h, n_rows, ld, n_vocab, b);
    if (rc) return rc;
    if (!stream_ids) return fail(h, FSB_ERR_INVALID, "stream_ids is null");
    if (!hist_off) return fail(h, FSB_ERR_INVALID, "hist_off is null");
    // first pass: validate and size the staged windows, without touching any engine
    int64_t need = 0;
    for (int i = 0; i < n_rows; ++i) {
        Stream* s = get_stream(h, stream_ids[i]);
        if (!s) return fail(h, FSB_ERR_STREAM_ID, "row %d: unknown stream id %d", i, stream_ids[i]);
        const int64_t len = hist_off[i + 1] - hist_off[i];
        if (len < 0) return fail(h, FSB_ERR_INVALID, "row %d: hist_off is not ascending", i);
        if (len > 0 && !hist_flat) return fail(h, FSB_ERR_INVALID, "hist_flat is null");
        need += len - window_begin(s->p, len);
    }
    if (need > b->cap_hist) return fail(h, FSB_ERR_CAPACITY, "%lld penalty-window ids exceed the capacity of %lld", (long long)need,
                                        (long long)b->cap_hist);
    b->n_rows = n_rows;
    b->n_vocab = n_vocab;
    b->ld = ld;
    b->flags = flags;
    b->hist_dev = nullptr;
    b->sid.assign(stream_ids, stream_ids + n_rows);
    b->stochastic.assign((size_t)n_rows, 0);
    b->descs.resize((size_t)n_rows);
    int32_t* hs = b->h_hist();
    int64_t pos = 0;
    for (int i = 0; i < n_rows; ++i) {
        Stream* s = get_stream(h, stream_ids[i]);
        const int64_t len = hist_off[i + 1] - hist_off[i];
        const int64_t wb = window_begin(s->p, len), wl = len - wb;
        if (wl > 0) std::memcpy(hs + pos, hist_flat + hist_off[i] + wb, sizeof(int32_t) * (size_t)wl);
        uint64_t word = 0;
        if (!is_greedy(s->p)) {   // exactly one engine output per stochastic call, none per greedy call
            word = s->rng();
            s->draws++;
            b->stochastic[(size_t)i] = 1;
        }
        fill_desc(h, b->descs[(size_t)i], s->p, n_vocab, (int64_t)i * ld, pos, wl, word, i);
        b->descs[(size_t)i].gather_off = (int32_t)pos;
        pos += wl;
    }
    b->hist_ids = pos;
    b->gather_ids = pos;
    b->table_ints = 0;
    rc = finalize_batch(h, b);
    if (rc) rollback_draws(h, b);
    return rc;
}

void count_rows(fsb_handle* h, const fsb_batch* b) {
    for (int i = 0; i < b->n_rows; ++i) {
        h->counters.rows_sampled++;
        if (b->stochastic[(size_t)i]) h->counters.rows_stochastic++;
        else h->counters.rows_greedy++;
    }
    h->counters.rows_full_vocab += (uint64_t)b->n_full;
}

int stage_host_logits(fsb_handle* h, const float* logits, int n_rows, int64_t ld, int n_vocab, const float** dev) {
    const size_t elems = (size_t)(n_rows - 1) * (size_t)ld + (size_t)n_vocab;
    if (elems > h->logits_stage_elems)
        return fail(h, FSB_ERR_CAPACITY, "host logits of %zu values (row stride %lld) exceed the engine's staging area of %zu", elems, (long long)ld,
                    h->logits_stage_elems);
    FSB_CUDA(h, cudaMemcpyAsync(h->d_logits_stage, logits, elems * sizeof(float), cudaMemcpyHostToDevice, h->stream));
    *dev = h->d_logits_stage;
    return FSB_OK;
}

// The reference modifies the caller's host row in place (src/sampler.cpp:17).  With host logits the kernels work on
// a device copy; the penalised values they leave there are gathered on the device (one per window id) and stored
// into the caller's rows here: the host moves values, it computes nothing.
int launch_gather(fsb_handle* h, fsb_batch* b, const float* logits_dev) {
    if (b->gather_ids <= 0) return FSB_OK;
    const int e = fsb::launch_gather_patched(logits_dev, b->d_rows(), b->n_rows, b->hist_dev ? b->hist_dev : b->d_hist(), b->n_vocab, h->vocab_offset,
                                             b->d_patched, h->stream);
    if (e != 0) return fail(h, FSB_ERR_CUDA, "gather kernel launch: %s", cudaGetErrorString((cudaError_t)e));
    h->counters.kernel_launches++;
    return FSB_OK;
}
void scatter_patched(const fsb_handle* h, const fsb_batch* b, float* logits_host, const int32_t* ids, int64_t n, int row, int gather_off) {
    float* rowp = logits_host + (int64_t)row * b->ld;
    for (int64_t i = 0; i < n; ++i) {
        const int64_t c = (int64_t)ids[i] - h->vocab_offset;
        if (c >= 0 && c < b->n_vocab) rowp[c] = b->h_patched[gather_off + i];
    }
}

// The common tail of the synchronous calls: upload, (stage host logits), launch, (append), fetch, (write back to host).
// `window_streams` > 0: a resident verification call - the drafts go into the id pool before the launch, and the last
// accepted token of every stream after it (see verify_windows_impl).
int run_staged(fsb_handle* h, fsb_batch* b, const float* logits, unsigned flags, bool append, int32_t* tokens_out, int window_streams = 0,
               bool window_append = false) {
    const bool on_host = (flags & FSB_LOGITS_ON_HOST) != 0;
    const bool host_wb = on_host && (flags & FSB_WRITE_BACK) && b->gather_ids > 0;
    int rc = upload_batch(h, b, !append && window_streams == 0 && !host_wb);
    const float* dev = logits;
    if (rc == FSB_OK && on_host) rc = stage_host_logits(h, logits, b->n_rows, b->ld, b->n_vocab, &dev);
    if (rc == FSB_OK && window_streams > 0) {
        const int e = fsb::launch_write_drafts(b->d_rows(), b->n_rows, h->d_pool, h->stream);
        if (e != 0) rc = fail(h, FSB_ERR_CUDA, "draft kernel launch: %s", cudaGetErrorString((cudaError_t)e));
        else h->counters.kernel_launches++;
    }
    if (rc == FSB_OK) rc = launch_batch(h, b, dev, (flags & FSB_KEEP_KEPT_SET) != 0, nullptr, nullptr, fsb::kMaxK, true);
    if (rc == FSB_OK && window_streams > 0 && window_append) {
        const int e = fsb::launch_accept_windows(b->d_hist() + b->hist_ids, window_streams, b->d_tokens, h->d_pool, h->stream);
        if (e != 0) rc = fail(h, FSB_ERR_CUDA, "accept kernel launch: %s", cudaGetErrorString((cudaError_t)e));
        else h->counters.kernel_launches++;
    }
    if (rc == FSB_OK && host_wb) rc = launch_gather(h, b, dev);
    if (rc == FSB_OK && append) {
        const int e = fsb::launch_append_tokens(b->d_rows(), b->n_rows, b->d_tokens, h->d_pool, h->stream);
        if (e != 0) rc = fail(h, FSB_ERR_CUDA, "append kernel launch: %s", cudaGetErrorString((cudaError_t)e));
        else h->counters.kernel_launches++;
    }
    if (rc == FSB_OK) rc = fetch_tokens(h, b, tokens_out, host_wb ? b->gather_ids : 0);
    if (rc) rollback_draws(h, b);
    return rc;
}

}  // namespace

// ================================================================================================ C ABI
extern "C" {

void fsb_params_default(ferro_sampler_params* p) {
    if (!p) return;
    std::memset(p, 0, sizeof *p);
    p->temperature = 0.05f;
    p->top_k = 50;
    p->top_p = 1.0f;
    p->min_p = 0.0f;
    p->repetition_penalty = 1.05f;
    p->repeat_last_n = -1;
    p->penalty_from = 0;
    p->seed = 0;
}

int fsb_params_validate(const ferro_sampler_params* p) {
    if (!p) return FSB_ERR_INVALID;
    // src/server.cpp:1071, negated; written so that NaNs fail
    if (!(p->temperature >= 0.0f)) return FSB_ERR_RANGE;
    if (!(p->top_p > 0.0f && p->top_p <= 1.0f)) return FSB_ERR_RANGE;
    if (p->top_k < 0) return FSB_ERR_RANGE;
    if (!(p->repetition_penalty > 0.0f) || std::isinf(p->repetition_penalty)) return FSB_ERR_RANGE;
    if (p->repeat_last_n < -1) return FSB_ERR_RANGE;
    if (!(p->min_p >= 0.0f && p->min_p <= 1.0f)) return FSB_ERR_RANGE;
    if (p->penalty_from < 0) return FSB_ERR_RANGE;
    if (std::isinf(p->temperature)) return FSB_ERR_RANGE;
    return FSB_OK;
}

int fsb_create(int device, int max_rows, int max_vocab, int64_t max_hist_ids, fsb_handle** out) {
    if (!out) return FSB_ERR_INVALID;
    *out = nullptr;
    if (max_rows <= 0 || max_vocab <= 0 || max_hist_ids < 0) return FSB_ERR_INVALID;
    if (max_vocab > (1 << 20)) return FSB_ERR_CAPACITY;
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev <= 0 || device < 0 || device >= n_dev) {
        cudaGetLastError();
        return FSB_ERR_NO_DEVICE;
    }
    fsb_handle* h = new (std::nothrow) fsb_handle();
    if (!h) return FSB_ERR_INVALID;
    h->device = device;
    h->max_rows = max_rows;
    h->max_vocab = max_vocab;
    h->max_hist = max_hist_ids;
    auto bail = [&](int code) {
        fsb_destroy(h);
        return code;
    };
    if (cudaSetDevice(device) != cudaSuccess) return bail(FSB_ERR_NO_DEVICE);
    cudaDeviceProp prop{};
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return bail(FSB_ERR_CUDA);
    if (prop.major < 10) return bail(FSB_ERR_NO_DEVICE);   // kernels are built for sm_100a only
    h->sm_count = prop.multiProcessorCount;
    if (fsb::prepare_device_kernels(&h->ctas_per_sm) != 0 || h->ctas_per_sm <= 0) return bail(FSB_ERR_CUDA);
    if (fsb::prepare_support_kernels() != 0) return bail(FSB_ERR_CUDA);
    if (fsb::prepare_full_row_kernel(max_vocab) != 0) return bail(FSB_ERR_CUDA);
    if (cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking) != cudaSuccess) return bail(FSB_ERR_CUDA);
    h->own_stream = true;
    if (cudaStreamCreateWithFlags(&h->side, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&h->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&h->ev_join, cudaEventDisableTiming) != cudaSuccess)
        return bail(FSB_ERR_CUDA);
    // Everything a call may need is allocated here, so that no call allocates: the rows' scratch, the counters, the
    // kept-set record, the id pool and the staging area of host logits.
    h->logits_stage_elems = (size_t)max_rows * (size_t)max_vocab;
    if (cudaMalloc(reinterpret_cast<void**>(&h->d_scratch), sizeof(uint64_t) * (size_t)max_rows * fsb::kMergeCap) != cudaSuccess ||
        cudaMalloc(reinterpret_cast<void**>(&h->d_counters), sizeof(uint32_t) * h->counter_words()) != cudaSuccess ||
        cudaMemset(h->d_counters, 0, sizeof(uint32_t) * h->counter_words()) != cudaSuccess ||
        cudaMalloc(reinterpret_cast<void**>(&h->d_kept_ids), sizeof(int32_t) * (size_t)max_rows * fsb::kMaxK) != cudaSuccess ||
        cudaMalloc(reinterpret_cast<void**>(&h->d_kept_pr), sizeof(double) * (size_t)max_rows * fsb::kMaxK) != cudaSuccess ||
        cudaMalloc(reinterpret_cast<void**>(&h->d_kept_n), sizeof(int32_t) * (size_t)max_rows) != cudaSuccess ||
        cudaMalloc(reinterpret_cast<void**>(&h->d_pool), sizeof(int32_t) * (size_t)std::max<int64_t>(max_hist_ids, 1)) != cudaSuccess ||
        cudaMalloc(reinterpret_cast<void**>(&h->d_logits_stage), sizeof(float) * h->logits_stage_elems) != cudaSuccess ||
        cudaMalloc(reinterpret_cast<void**>(&h->d_lookup), sizeof(fsb::LookupDesc) * (size_t)max_rows) != cudaSuccess ||
        cudaMalloc(reinterpret_cast<void**>(&h->d_drafts), sizeof(int32_t) * (size_t)max_rows * fsb::kDraftStride) != cudaSuccess ||
        cudaMallocHost(reinterpret_cast<void**>(&h->h_lookup), sizeof(fsb::LookupDesc) * (size_t)max_rows) != cudaSuccess ||
        cudaMallocHost(reinterpret_cast<void**>(&h->h_drafts), sizeof(int32_t) * (size_t)max_rows * fsb::kDraftStride) != cudaSuccess)
        return bail(FSB_ERR_CUDA);
    if (alloc_batch(h, max_rows, max_hist_ids, std::max<int64_t>(max_hist_ids, 1), &h->own) != FSB_OK) return bail(FSB_ERR_CUDA);
    *out = h;
    return FSB_OK;
}

int fsb_destroy(fsb_handle* h) {
    if (!h) return FSB_ERR_INVALID;
    cudaSetDevice(h->device);
    if (h->stream) cudaStreamSynchronize(h->stream);
    if (h->own) {
        free_batch_buffers(h->own);
        delete h->own;
    }
    if (h->d_scratch) cudaFree(h->d_scratch);
    if (h->d_counters) cudaFree(h->d_counters);
    if (h->d_kept_ids) cudaFree(h->d_kept_ids);
    if (h->d_kept_pr) cudaFree(h->d_kept_pr);
    if (h->d_kept_n) cudaFree(h->d_kept_n);
    if (h->d_pool) cudaFree(h->d_pool);
    if (h->d_logits_stage) cudaFree(h->d_logits_stage);
    if (h->d_lookup) cudaFree(h->d_lookup);
    if (h->d_drafts) cudaFree(h->d_drafts);
    if (h->h_lookup) cudaFreeHost(h->h_lookup);
    if (h->h_drafts) cudaFreeHost(h->h_drafts);
    if (h->own_stream && h->stream) cudaStreamDestroy(h->stream);
    if (h->side) cudaStreamDestroy(h->side);
    if (h->ev_fork) cudaEventDestroy(h->ev_fork);
    if (h->ev_join) cudaEventDestroy(h->ev_join);
    delete h;
    return FSB_OK;
}

const char* fsb_last_error(const fsb_handle* h) { return h ? h->err.c_str() : "null handle"; }

int fsb_set_cuda_stream(fsb_handle* h, void* cuda_stream) {
    if (!h) return FSB_ERR_INVALID;
    cudaSetDevice(h->device);
    if (h->stream) cudaStreamSynchronize(h->stream);
    if (h->own_stream && h->stream) cudaStreamDestroy(h->stream);
    h->stream = static_cast<cudaStream_t>(cuda_stream);
    h->own_stream = false;
    return FSB_OK;
}

int fsb_set_softcap(fsb_handle* h, float cap) {
    if (!h) return FSB_ERR_INVALID;
    if (!(cap >= 0.0f) || std::isinf(cap)) return fail(h, FSB_ERR_RANGE, "softcap must be finite and >= 0");
    h->softcap = cap;
    return FSB_OK;
}

int fsb_set_trace_buffer(fsb_handle* h, void* device_buffer) {
    if (!h) return FSB_ERR_INVALID;
    h->d_trace = static_cast<uint64_t*>(device_buffer);
    return FSB_OK;
}

int fsb_set_launch_overlap(fsb_handle* h, int on) {
    if (!h) return FSB_ERR_INVALID;
    if (on < 0 || on > 2) return fail(h, FSB_ERR_RANGE, "launch overlap mode is 0, 1 or 2");
    h->launch_overlap = on;
    return FSB_OK;
}

int fsb_set_vocab_offset(fsb_handle* h, int32_t offset) {
    if (!h) return FSB_ERR_INVALID;
    if (offset < 0) return fail(h, FSB_ERR_RANGE, "vocab offset must be >= 0");
    h->vocab_offset = offset;
    return FSB_OK;
}

int fsb_set_vocab_shard(fsb_handle* h, int32_t offset, int32_t global_vocab) {
    if (!h) return FSB_ERR_INVALID;
    if (offset < 0 || global_vocab < 0 || (global_vocab > 0 && offset >= global_vocab)) return fail(h, FSB_ERR_RANGE, "bad shard: offset %d of %d columns", offset, global_vocab);
    h->vocab_offset = offset;
    h->global_vocab = global_vocab;
    return FSB_OK;
}

int fsb_stream_open(fsb_handle* h, const ferro_sampler_params* p, int* stream_id) {
    if (!h || !p || !stream_id) return fail(h, FSB_ERR_INVALID, "null argument");
    const int v = fsb_params_validate(p);
    if (v != FSB_OK) return fail(h, v, "sampling parameter out of range");
    int id;
    if (!h->free_ids.empty()) {
        id = h->free_ids.back();
        h->free_ids.pop_back();
    } else {
        id = (int)h->streams.size();
        h->streams.emplace_back();
    }
    Stream& s = h->streams[(size_t)id];
    s.p = *p;
    s.seed_used = p->seed ? p->seed : (uint64_t)std::random_device{}();   // src/sampler.h:25
    s.rng.seed(s.seed_used);
    s.draws = 0;
    s.open = true;
    *stream_id = id;
    return FSB_OK;
}

int fsb_stream_close(fsb_handle* h, int stream_id) {
    if (!h) return FSB_ERR_INVALID;
    Stream* s = get_stream(h, stream_id);
    if (!s) return fail(h, FSB_ERR_STREAM_ID, "unknown stream id %d", stream_id);
    release_region(h, s);
    s->hist.clear();
    s->hist.shrink_to_fit();
    s->open = false;
    h->free_ids.push_back(stream_id);
    return FSB_OK;
}

int fsb_stream_params(const fsb_handle* h, int stream_id, ferro_sampler_params* out) {
    if (!h || !out) return FSB_ERR_INVALID;
    Stream* s = get_stream(const_cast<fsb_handle*>(h), stream_id);
    if (!s) return FSB_ERR_STREAM_ID;
    *out = s->p;
    return FSB_OK;
}

int fsb_stream_state_get(const fsb_handle* h, int stream_id, uint64_t* seed, uint64_t* draws) {
    if (!h) return FSB_ERR_INVALID;
    Stream* s = get_stream(const_cast<fsb_handle*>(h), stream_id);
    if (!s) return FSB_ERR_STREAM_ID;
    if (seed) *seed = s->seed_used;
    if (draws) *draws = s->draws;
    return FSB_OK;
}

int fsb_stream_state_set(fsb_handle* h, int stream_id, uint64_t seed, uint64_t draws) {
    if (!h) return FSB_ERR_INVALID;
    Stream* s = get_stream(h, stream_id);
    if (!s) return fail(h, FSB_ERR_STREAM_ID, "unknown stream id %d", stream_id);
    s->seed_used = seed;
    s->rng.seed(seed);
    s->rng.discard(draws);
    s->draws = draws;
    return FSB_OK;
}

int fsb_sample_batch(fsb_handle* h, int n_rows, const int* stream_ids, const float* logits, int64_t ld, int n_vocab,
                     const int32_t* hist_flat, const int64_t* hist_off, int32_t* tokens_out, unsigned flags) {
    if (!h) return FSB_ERR_INVALID;
    if (!logits || !tokens_out) return fail(h, FSB_ERR_INVALID, "null logits or tokens_out");
    cudaSetDevice(h->device);
    fsb_batch* b = h->own;
    int rc = stage_rows(h, b, n_rows, stream_ids, ld, n_vocab, hist_flat, hist_off, flags);
    if (rc) return rc;
    rc = run_staged(h, b, logits, flags, false, tokens_out);
    if (rc) return rc;
    if ((flags & FSB_LOGITS_ON_HOST) && (flags & FSB_WRITE_BACK)) {
        for (int i = 0; i < n_rows; ++i) {
            const fsb::RowDesc& d = b->descs[(size_t)i];
            scatter_patched(h, b, const_cast<float*>(logits), b->h_hist() + d.hist_begin, d.hist_len, i, d.gather_off);
        }
    }
    count_rows(h, b);
    return FSB_OK;
}

int fsb_stream_history_set(fsb_handle* h, int stream_id, const int32_t* ids, int64_t n) {
    if (!h || n < 0 || (n > 0 && !ids)) return FSB_ERR_INVALID;
    Stream* s = get_stream(h, stream_id);
    if (!s) return fail(h, FSB_ERR_STREAM_ID, "unknown stream id %d", stream_id);
    cudaSetDevice(h->device);
    s->hist.assign(ids, ids + n);
    s->dev_len = 0;
    return sync_history(h, s);
}

int fsb_stream_history_append(fsb_handle* h, int stream_id, const int32_t* ids, int n) {
    if (!h || n < 0 || (n > 0 && !ids)) return FSB_ERR_INVALID;
    Stream* s = get_stream(h, stream_id);
    if (!s) return fail(h, FSB_ERR_STREAM_ID, "unknown stream id %d", stream_id);
    cudaSetDevice(h->device);
    s->hist.insert(s->hist.end(), ids, ids + n);
    return sync_history(h, s);
}

int fsb_lookup_drafts_resident(fsb_handle* h, int n_streams, const int* stream_ids, const int* kmax, const int* min_n, int32_t eos,
                               int32_t* drafts_out, int stride, int* n_out) {
    if (!h || !stream_ids || !kmax || !min_n || !drafts_out || !n_out) return FSB_ERR_INVALID;
    if (n_streams <= 0 || n_streams > h->max_rows) return fail(h, FSB_ERR_CAPACITY, "%d streams, the engine holds %d rows", n_streams, h->max_rows);
    if (stride < 1) return fail(h, FSB_ERR_INVALID, "stride must be positive");
    cudaSetDevice(h->device);
    for (int i = 0; i < n_streams; ++i) {
        Stream* s = get_stream(h, stream_ids[i]);
        if (!s) return fail(h, FSB_ERR_STREAM_ID, "unknown stream id %d", stream_ids[i]);
        if (min_n[i] < 1) return fail(h, FSB_ERR_RANGE, "stream %d: the shortest match is one token, got %d", i, min_n[i]);
        if (kmax[i] > stride || kmax[i] > fsb::kDraftStride - 1)
            return fail(h, FSB_ERR_CAPACITY, "stream %d: %d drafts do not fit (stride %d, at most %d per call)", i, kmax[i], stride, fsb::kDraftStride - 1);
        const int rc = sync_history(h, s);
        if (rc != FSB_OK) return rc;
        fsb::LookupDesc& d = h->h_lookup[i];
        d.begin = s->pool_off >= 0 ? s->pool_off : 0;
        d.len = (int32_t)s->hist.size();
        d.kmax = std::max(0, kmax[i]);
        d.min_n = min_n[i];
        d.eos = eos;
    }
    FSB_CUDA(h, cudaMemcpyAsync(h->d_lookup, h->h_lookup, sizeof(fsb::LookupDesc) * (size_t)n_streams, cudaMemcpyHostToDevice, h->stream));
    const int e = fsb::launch_lookup_drafts(h->d_pool, h->d_lookup, n_streams, h->d_drafts, fsb::kDraftStride, h->stream);
    if (e != 0) return fail(h, FSB_ERR_CUDA, "draft kernel launch: %s", cudaGetErrorString((cudaError_t)e));
    h->counters.kernel_launches++;
    FSB_CUDA(h, cudaMemcpyAsync(h->h_drafts, h->d_drafts, sizeof(int32_t) * (size_t)n_streams * fsb::kDraftStride, cudaMemcpyDeviceToHost, h->stream));
    FSB_CUDA(h, cudaStreamSynchronize(h->stream));
    for (int i = 0; i < n_streams; ++i) {
        const int32_t* src = h->h_drafts + (size_t)i * fsb::kDraftStride;
        n_out[i] = src[0];
        for (int k = 0; k < src[0]; ++k) drafts_out[(size_t)i * stride + k] = src[1 + k];
    }
    return FSB_OK;
}

int fsb_stream_history_len(const fsb_handle* h, int stream_id, int64_t* n) {
    if (!h || !n) return FSB_ERR_INVALID;
    Stream* s = get_stream(const_cast<fsb_handle*>(h), stream_id);
    if (!s) return FSB_ERR_STREAM_ID;
    *n = (int64_t)s->hist.size();
    return FSB_OK;
}

int fsb_sample_batch_resident(fsb_handle* h, int n_rows, const int* stream_ids, const float* logits, int64_t ld, int n_vocab,
                              int32_t* tokens_out, unsigned flags) {
    if (!h) return FSB_ERR_INVALID;
    if (!logits || !tokens_out || !stream_ids) return fail(h, FSB_ERR_INVALID, "null logits, stream_ids or tokens_out");
    cudaSetDevice(h->device);
    fsb_batch* b = h->own;
    int rc = check_common(h, n_rows, ld, n_vocab, b);
    if (rc) return rc;
    const bool append = (flags & FSB_APPEND_SAMPLED) != 0;
    // validate first, without touching any engine: known streams, each at most once, room for the new ids
    ++h->call_no;
    for (int i = 0; i < n_rows; ++i) {
        Stream* s = get_stream(h, stream_ids[i]);
        if (!s) return fail(h, FSB_ERR_STREAM_ID, "row %d: unknown stream id %d", i, stream_ids[i]);
        if (s->seen == h->call_no) return fail(h, FSB_ERR_INVALID, "stream %d appears twice in one resident batch", stream_ids[i]);
        s->seen = h->call_no;
    }
    int64_t gather = 0;
    for (int i = 0; i < n_rows; ++i) {
        Stream* s = get_stream(h, stream_ids[i]);
        rc = sync_history(h, s);
        if (rc == FSB_OK && append) rc = ensure_region(h, s, (int64_t)s->hist.size() + 1);
        if (rc) return rc;
        const int64_t len = (int64_t)s->hist.size();
        gather += len - window_begin(s->p, len);
    }
    const bool host_wb = (flags & FSB_LOGITS_ON_HOST) && (flags & FSB_WRITE_BACK);
    if (host_wb && gather > b->cap_hist) return fail(h, FSB_ERR_CAPACITY, "%lld penalty-window ids exceed the capacity of %lld", (long long)gather, (long long)b->cap_hist);
    b->n_rows = n_rows;
    b->n_vocab = n_vocab;
    b->ld = ld;
    b->flags = flags & ~FSB_APPEND_SAMPLED;
    b->hist_dev = h->d_pool;
    b->hist_ids = 0;
    b->sid.assign(stream_ids, stream_ids + n_rows);
    b->stochastic.assign((size_t)n_rows, 0);
    b->descs.resize((size_t)n_rows);
    int64_t goff = 0;
    for (int i = 0; i < n_rows; ++i) {
        Stream* s = get_stream(h, stream_ids[i]);
        const int64_t len = (int64_t)s->hist.size();
        const int64_t wb = window_begin(s->p, len), wl = len - wb;
        uint64_t word = 0;
        if (!is_greedy(s->p)) {
            word = s->rng();
            s->draws++;
            b->stochastic[(size_t)i] = 1;
        }
        // the window ends where the history ends: hist_begin + hist_len is where an appended token goes
        fsb::RowDesc& d = b->descs[(size_t)i];
        fill_desc(h, d, s->p, n_vocab, (int64_t)i * ld, (s->pool_off >= 0 ? s->pool_off : 0) + wb, wl, word, i);
        if (append) d.flags |= fsb::kRowAppend;
        d.gather_off = (int32_t)goff;
        goff += wl;
    }
    b->gather_ids = host_wb ? goff : 0;
    rc = finalize_batch(h, b);
    if (rc) {
        rollback_draws(h, b);
        return rc;
    }
    rc = run_staged(h, b, logits, flags & ~FSB_APPEND_SAMPLED, append, tokens_out);
    if (rc) return rc;
    for (int i = 0; i < n_rows; ++i) {
        Stream* s = get_stream(h, stream_ids[i]);
        if (host_wb) {
            const fsb::RowDesc& d = b->descs[(size_t)i];
            scatter_patched(h, b, const_cast<float*>(logits), s->hist.data() + (s->hist.size() - (size_t)d.hist_len), d.hist_len, i, d.gather_off);
        }
        if (append) {   // the device copy already holds the token
            s->hist.push_back(tokens_out[i]);
            s->dev_len = (int64_t)s->hist.size();
        }
    }
    count_rows(h, b);
    return FSB_OK;
}

// The two window calls share everything but where a stream's history comes from: `hist_flat` / `hist_off` (host
// memory, staged with the call) or, when hist_off is null, the streams' resident histories.
static int verify_windows_impl(fsb_handle* h, int n_streams, const int* stream_ids, const int* row_off, const int32_t* rows_flat,
                               const float* logits, int64_t ld, int n_vocab, const int32_t* hist_flat, const int64_t* hist_off,
                               const int* max_accept, int32_t* tokens_out, int* acc_out, int* confirmed_out, unsigned flags) {
    const bool resident = hist_off == nullptr;
    if (!stream_ids || !row_off || !rows_flat || !logits || !tokens_out || !acc_out) return fail(h, FSB_ERR_INVALID, "null argument");
    if (n_streams <= 0) return fail(h, FSB_ERR_INVALID, "n_streams must be positive");
    if (flags & FSB_WRITE_BACK) return fail(h, FSB_ERR_INVALID, "write-back is not defined for verification windows");
    if (!resident && (flags & FSB_APPEND_SAMPLED)) return fail(h, FSB_ERR_INVALID, "FSB_APPEND_SAMPLED needs resident histories");
    cudaSetDevice(h->device);
    fsb_batch* b = h->own;
    const int n_rows = row_off[n_streams] - row_off[0];
    if (row_off[0] != 0) return fail(h, FSB_ERR_INVALID, "row_off[0] must be 0");
    int rc = check_common(h, n_rows, ld, n_vocab, b);
    if (rc) return rc;
    // validate, size the staging
    int64_t need = 0;
    ++h->call_no;
    for (int i = 0; i < n_streams; ++i) {
        Stream* s = get_stream(h, stream_ids[i]);
        if (!s) return fail(h, FSB_ERR_STREAM_ID, "stream %d: unknown stream id %d", i, stream_ids[i]);
        if (s->seen == h->call_no) return fail(h, FSB_ERR_INVALID, "stream id %d appears twice", stream_ids[i]);
        s->seen = h->call_no;
        const int m = row_off[i + 1] - row_off[i];
        const int64_t len = resident ? (int64_t)s->hist.size() : hist_off[i + 1] - hist_off[i];
        if (m <= 0 || len < 0) return fail(h, FSB_ERR_INVALID, "stream %d: empty window or bad history offsets", i);
        if (resident && (flags & FSB_APPEND_SAMPLED) && m - 1 > fsb::kWindowTableInts - 6)
            return fail(h, FSB_ERR_CAPACITY, "stream %d: a resident window with FSB_APPEND_SAMPLED holds at most %d drafts", i, fsb::kWindowTableInts - 6);
        if (!resident && len > 0 && !hist_flat) return fail(h, FSB_ERR_INVALID, "hist_flat is null");
        need += resident ? 0 : (len - window_begin(s->p, len)) + (m - 1);
    }
    if (need > b->cap_hist) return fail(h, FSB_ERR_CAPACITY, "%lld penalty-window ids exceed the capacity of %lld", (long long)need,
                                        (long long)b->cap_hist);
    if (resident) {
        // The drafts of a window go behind the stream's history in its region of the id pool (they are what the history
        // will hold if they are accepted), so that row r's window is a range of the pool like any other: make room.
        for (int i = 0; i < n_streams; ++i) {
            Stream* s = get_stream(h, stream_ids[i]);
            rc = sync_history(h, s);
            if (rc == FSB_OK) rc = ensure_region(h, s, (int64_t)s->hist.size() + (row_off[i + 1] - row_off[i]));
            if (rc) return rc;
        }
    }
    b->n_rows = n_rows;
    b->n_vocab = n_vocab;
    b->ld = ld;
    b->flags = flags & ~FSB_APPEND_SAMPLED;
    b->hist_dev = resident ? h->d_pool : nullptr;
    b->gather_ids = 0;
    b->sid.assign((size_t)n_rows, 0);
    b->stochastic.assign((size_t)n_rows, 0);
    b->descs.resize((size_t)n_rows);
    int32_t* hs = b->h_hist();
    int64_t pos = 0;
    for (int i = 0; i < n_streams; ++i) {
        Stream* s = get_stream(h, stream_ids[i]);
        const int r0 = row_off[i], m = row_off[i + 1] - r0;
        const int64_t len = resident ? (int64_t)s->hist.size() : hist_off[i + 1] - hist_off[i];
        const bool pen_on = !(s->p.repetition_penalty == 1.0f || s->p.repeat_last_n == 0);
        // row r samples with history_i followed by draft_1..draft_r; the windows of successive rows only move
        // forward, so one copy [b_0 .. len + m - 1) serves the whole stream: staged here, or the stream's pool region
        const int64_t b0 = pen_on ? window_begin(s->p, len) : len;
        int64_t base = pos;
        if (resident) {
            base = s->pool_off + b0;
        } else if (pen_on) {
            if (len > b0) std::memcpy(hs + pos, hist_flat + hist_off[i] + b0, sizeof(int32_t) * (size_t)(len - b0));
            pos += len - b0;
            for (int r = 1; r < m; ++r) hs[pos++] = rows_flat[r0 + r];
        }
        std::mt19937_64 look = s->rng;   // draws are taken from a copy; the real engine advances by acc afterwards
        const bool greedy = is_greedy(s->p);
        for (int r = 0; r < m; ++r) {
            int64_t hb = 0, hl = 0;
            if (pen_on) {
                const int64_t len_r = len + r;
                const int64_t br = window_begin(s->p, len_r);
                hb = base + (br - b0);
                hl = len_r - br;
            }
            const uint64_t word = greedy ? 0ull : look();
            b->sid[(size_t)(r0 + r)] = stream_ids[i];
            fsb::RowDesc& d = b->descs[(size_t)(r0 + r)];
            fill_desc(h, d, s->p, n_vocab, (int64_t)(r0 + r) * ld, hb, hl, word, r0 + r);
            if (resident && r >= 1 && hl >= 1) {   // draft_r is the last id of row r's window: a kernel puts it there before the launch
                d.flags |= fsb::kRowDraft;
                d.gather_off = rows_flat[r0 + r];
            }
        }
    }
    b->hist_ids = pos;
    b->table_ints = 0;
    const bool win_append = resident && (flags & FSB_APPEND_SAMPLED);
    if (win_append) {
        // per stream: first row, rows, accept limit, and where the stream's history ends in the id pool; the device walks
        // the same accept loop as the host below and stores the last accepted token there (the confirmed drafts before
        // it are in place already)
        int32_t* tab = hs + pos;
        for (int i = 0; i < n_streams; ++i) {
            Stream* s = get_stream(h, stream_ids[i]);
            const int r0 = row_off[i], m = row_off[i + 1] - r0;
            const int64_t end = s->pool_off + (int64_t)s->hist.size();
            int32_t* t = tab + (size_t)i * fsb::kWindowTableInts;
            t[0] = r0;
            t[1] = m;
            t[2] = (max_accept && max_accept[i] > 0 && max_accept[i] < m) ? max_accept[i] : m;
            t[3] = 0;
            t[4] = (int32_t)(uint32_t)(end & 0xFFFFFFFFll);
            t[5] = (int32_t)(end >> 32);
            for (int r = 1; r < m; ++r) t[5 + r] = rows_flat[r0 + r];   // the drafts, for the comparison (at most kWindowTableInts - 6)
        }
        b->table_ints = (int64_t)n_streams * fsb::kWindowTableInts;
    }
    rc = finalize_batch(h, b);
    if (rc) return rc;
    rc = run_staged(h, b, logits, flags & ~FSB_APPEND_SAMPLED, false, nullptr, resident ? n_streams : 0, win_append);   // no engine was advanced: nothing to roll back
    if (rc) return rc;
    // accept loop of src/server.cpp:626-636 on the sampled tokens
    for (int i = 0; i < n_streams; ++i) {
        Stream* s = get_stream(h, stream_ids[i]);
        const int r0 = row_off[i], m = row_off[i + 1] - r0;
        const int lim = (max_accept && max_accept[i] > 0 && max_accept[i] < m) ? max_accept[i] : m;
        int acc = 0, conf = 0;
        for (int r = 0; r < lim; ++r) {
            const int tok = b->h_tokens[r0 + r];
            tokens_out[r0 + r] = tok;
            acc = r + 1;
            if (r + 1 < m && tok == rows_flat[r0 + r + 1]) {
                if (r + 1 < lim) ++conf;
                continue;
            }
            break;
        }
        for (int r = acc; r < m; ++r) tokens_out[r0 + r] = -1;
        acc_out[i] = acc;
        if (confirmed_out) confirmed_out[i] = conf;
        if (!is_greedy(s->p)) {
            s->rng.discard((unsigned long long)acc);
            s->draws += (uint64_t)acc;
            h->counters.rows_stochastic += (uint64_t)acc;
        } else {
            h->counters.rows_greedy += (uint64_t)acc;
        }
        h->counters.rows_sampled += (uint64_t)acc;
        h->counters.drafted += (uint64_t)(m - 1);
        h->counters.accepted += (uint64_t)conf;
        if (resident && (flags & FSB_APPEND_SAMPLED)) {
            // what gen_token appends (src/server.cpp:342): the sampled tokens of the accepted rows
            for (int r = 0; r < acc; ++r) s->hist.push_back(tokens_out[r0 + r]);
            s->dev_len = (int64_t)s->hist.size();   // the device copy holds them: confirmed drafts, and the last token stored by the accept kernel
        }
    }
    return FSB_OK;
}

int fsb_verify_windows(fsb_handle* h, int n_streams, const int* stream_ids, const int* row_off, const int32_t* rows_flat,
                       const float* logits, int64_t ld, int n_vocab, const int32_t* hist_flat, const int64_t* hist_off,
                       const int* max_accept, int32_t* tokens_out, int* acc_out, int* confirmed_out, unsigned flags) {
    if (!h) return FSB_ERR_INVALID;
    if (!hist_off) return fail(h, FSB_ERR_INVALID, "null argument");
    return verify_windows_impl(h, n_streams, stream_ids, row_off, rows_flat, logits, ld, n_vocab, hist_flat, hist_off, max_accept, tokens_out, acc_out,
                               confirmed_out, flags);
}

int fsb_verify_windows_resident(fsb_handle* h, int n_streams, const int* stream_ids, const int* row_off, const int32_t* rows_flat,
                                const float* logits, int64_t ld, int n_vocab, const int* max_accept, int32_t* tokens_out, int* acc_out,
                                int* confirmed_out, unsigned flags) {
    if (!h) return FSB_ERR_INVALID;
    return verify_windows_impl(h, n_streams, stream_ids, row_off, rows_flat, logits, ld, n_vocab, nullptr, nullptr, max_accept, tokens_out, acc_out,
                               confirmed_out, flags);
}

int fsb_last_kept(fsb_handle* h, int row, int cap, int32_t* ids, double* probs, int* n_keep) {
    if (!h || !n_keep) return FSB_ERR_INVALID;
    if (!h->kept_valid) return fail(h, FSB_ERR_INVALID, "the last call did not record kept sets (FSB_KEEP_KEPT_SET)");
    if (row < 0 || row >= h->max_rows) return fail(h, FSB_ERR_INVALID, "row out of range");
    cudaSetDevice(h->device);
    int32_t n = 0;
    FSB_CUDA(h, cudaMemcpy(&n, h->d_kept_n + row, sizeof n, cudaMemcpyDeviceToHost));
    *n_keep = n;
    const int c = std::min(std::min(cap, (int)n), fsb::kMaxK);
    if (c > 0 && ids) FSB_CUDA(h, cudaMemcpy(ids, h->d_kept_ids + (size_t)row * fsb::kMaxK, sizeof(int32_t) * (size_t)c, cudaMemcpyDeviceToHost));
    if (c > 0 && probs) FSB_CUDA(h, cudaMemcpy(probs, h->d_kept_pr + (size_t)row * fsb::kMaxK, sizeof(double) * (size_t)c, cudaMemcpyDeviceToHost));
    return FSB_OK;
}

int fsb_batch_prepare(fsb_handle* h, int n_rows, const int* stream_ids, int64_t ld, int n_vocab, const int32_t* hist_flat,
                      const int64_t* hist_off, unsigned flags, fsb_batch** out) {
    if (!h || !out) return FSB_ERR_INVALID;
    *out = nullptr;
    if (flags & FSB_LOGITS_ON_HOST) return fail(h, FSB_ERR_INVALID, "prepared batches take device logits");
    if (n_rows <= 0 || !hist_off) return fail(h, FSB_ERR_INVALID, "bad arguments");
    cudaSetDevice(h->device);
    fsb_batch* b = nullptr;
    int rc = alloc_batch(h, n_rows, hist_off[n_rows] - hist_off[0], 0, &b);
    if (rc) return rc;
    rc = stage_rows(h, b, n_rows, stream_ids, ld, n_vocab, hist_flat, hist_off, flags);
    if (rc == FSB_OK) {
        rc = upload_batch(h, b);
        if (rc == FSB_OK && cudaStreamSynchronize(h->stream) != cudaSuccess) rc = fail(h, FSB_ERR_CUDA, "upload failed");
        if (rc) rollback_draws(h, b);
    }
    if (rc) {
        free_batch_buffers(b);
        delete b;
        return rc;
    }
    *out = b;
    return FSB_OK;
}

int fsb_batch_redraw(fsb_handle* h, fsb_batch* b) {
    if (!h || !b) return FSB_ERR_INVALID;
    cudaSetDevice(h->device);
    fsb::RowDesc* rows = b->h_rows();
    for (int j = 0; j < b->n_rows; ++j) {
        const int i = rows[j].out_index;
        if (!b->stochastic[(size_t)i]) continue;
        Stream* s = get_stream(h, b->sid[(size_t)i]);
        if (!s) return fail(h, FSB_ERR_STREAM_ID, "stream id %d was closed", b->sid[(size_t)i]);
    }
    // rows draw in row order, as a per-slot loop would
    std::vector<int> order((size_t)b->n_rows);
    for (int j = 0; j < b->n_rows; ++j) order[(size_t)rows[j].out_index] = j;
    for (int i = 0; i < b->n_rows; ++i) {
        if (!b->stochastic[(size_t)i]) continue;
        Stream* s = get_stream(h, b->sid[(size_t)i]);
        rows[order[(size_t)i]].rng_word = s->rng();
        s->draws++;
    }
    FSB_CUDA(h, cudaMemcpyAsync(b->d_in, b->h_in, sizeof(fsb::RowDesc) * (size_t)b->n_rows, cudaMemcpyHostToDevice, h->stream));
    return FSB_OK;
}

int fsb_batch_launch(fsb_handle* h, fsb_batch* b, const float* logits_dev) {
    if (!h || !b || !logits_dev) return FSB_ERR_INVALID;
    cudaSetDevice(h->device);
    return launch_batch(h, b, logits_dev, (b->flags & FSB_KEEP_KEPT_SET) != 0);
}

int fsb_batch_shard_launch(fsb_handle* h, fsb_batch* b, const float* logits_shard_dev, uint64_t* lists_out_dev, int32_t* counts_out_dev) {
    if (!h || !b || !logits_shard_dev || !lists_out_dev || !counts_out_dev) return FSB_ERR_INVALID;
    cudaSetDevice(h->device);
    return launch_batch(h, b, logits_shard_dev, false, lists_out_dev, counts_out_dev);
}
int fsb_batch_merge_launch(fsb_handle* h, fsb_batch* b, const uint64_t* lists_dev, const int32_t* counts_dev, int n_lists) {
    if (!h || !b || !lists_dev || !counts_dev) return FSB_ERR_INVALID;
    if (n_lists < 1 || (int64_t)n_lists * fsb::kMaxK > fsb::kMergeCap)
        return fail(h, FSB_ERR_RANGE, "between 1 and %d candidate lists can be merged", fsb::kMergeCap / fsb::kMaxK);
    if (b->n_full > 0) return fail(h, FSB_ERR_RANGE, "the batch has rows that cannot be sharded by vocabulary");
    cudaSetDevice(h->device);
    const bool keep_kept = (b->flags & FSB_KEEP_KEPT_SET) != 0;
    const int e = fsb::launch_merge_lists(lists_dev, counts_dev, n_lists, fsb::kMaxK, b->n_cand, b->d_rows(), b->d_tokens, keep_kept ? h->d_kept_ids : nullptr,
                                          keep_kept ? h->d_kept_pr : nullptr, keep_kept ? h->d_kept_n : nullptr, b->d_status(), h->stream);
    if (e != 0) return fail(h, FSB_ERR_CUDA, "merge kernel launch: %s", cudaGetErrorString((cudaError_t)e));
    h->counters.kernel_launches++;
    b->launched = true;
    h->kept_valid = keep_kept;
    return FSB_OK;
}
int fsb_batch_max_k(const fsb_batch* b) { return b ? b->kmax : 0; }
int fsb_batch_shard_launch_packed(fsb_handle* h, fsb_batch* b, const float* logits_shard_dev, uint64_t* packed_out_dev, int32_t stride_words) {
    if (!h || !b || !logits_shard_dev || !packed_out_dev) return FSB_ERR_INVALID;
    if (stride_words < b->kmax + 1) return fail(h, FSB_ERR_RANGE, "a packed list needs %d words (1 + the batch's largest k), got %d", b->kmax + 1, stride_words);
    cudaSetDevice(h->device);
    return launch_batch(h, b, logits_shard_dev, false, packed_out_dev, nullptr, stride_words);
}
int fsb_batch_merge_launch_packed(fsb_handle* h, fsb_batch* b, const uint64_t* packed_dev, int32_t stride_words, int n_lists, int32_t row_begin,
                                  int32_t n_rows) {
    if (!h || !b || (!packed_dev && n_rows > 0)) return FSB_ERR_INVALID;   // a rank whose block of rows is empty has nothing to pass
    if (b->n_full > 0) return fail(h, FSB_ERR_RANGE, "the batch has rows that cannot be sharded by vocabulary");
    if (stride_words < 2 || n_lists < 1 || (int64_t)n_lists * std::min(fsb::kMaxK, stride_words - 1) > fsb::kMergeCap)
        return fail(h, FSB_ERR_RANGE, "%d lists of %d words exceed the %d candidates a row can merge", n_lists, stride_words, fsb::kMergeCap);
    if (row_begin < 0 || n_rows < 0 || row_begin + n_rows > b->n_cand) return fail(h, FSB_ERR_RANGE, "rows %d..%d are not rows of the batch", row_begin, row_begin + n_rows);
    cudaSetDevice(h->device);
    const bool keep_kept = (b->flags & FSB_KEEP_KEPT_SET) != 0;
    if (n_rows > 0) {
        const int e = fsb::launch_merge_lists(packed_dev, nullptr, n_lists, stride_words, n_rows, b->d_rows() + row_begin, b->d_tokens,
                                              keep_kept ? h->d_kept_ids : nullptr, keep_kept ? h->d_kept_pr : nullptr, keep_kept ? h->d_kept_n : nullptr,
                                              b->d_status(), h->stream);
        if (e != 0) return fail(h, FSB_ERR_CUDA, "merge kernel launch: %s", cudaGetErrorString((cudaError_t)e));
        h->counters.kernel_launches++;
    }
    b->launched = true;
    h->kept_valid = keep_kept && row_begin == 0 && n_rows == b->n_cand;
    return FSB_OK;
}
int32_t* fsb_batch_tokens_device(fsb_batch* b) { return b ? b->d_tokens : nullptr; }
int fsb_batch_check(fsb_handle* h, fsb_batch* b) {
    if (!h || !b) return FSB_ERR_INVALID;
    if (!b->launched) return fail(h, FSB_ERR_INVALID, "the batch has not been launched");
    cudaSetDevice(h->device);
    return fetch_tokens(h, b, nullptr);
}
int fsb_batch_tokens(fsb_handle* h, fsb_batch* b, int32_t* tokens_out) {
    if (!h || !b || !tokens_out) return FSB_ERR_INVALID;
    if (!b->launched) return fail(h, FSB_ERR_INVALID, "the batch has not been launched");
    cudaSetDevice(h->device);
    const int rc = fetch_tokens(h, b, tokens_out);
    if (rc == FSB_OK) count_rows(h, b);
    return rc;
}

int fsb_batch_kernel_count(const fsb_batch* b) {
    if (!b) return 0;
    return (b->n_cand > 0 ? 1 : 0) + (b->n_full > 0 ? 1 : 0);
}

int fsb_batch_free(fsb_handle* h, fsb_batch* b) {
    if (!h || !b) return FSB_ERR_INVALID;
    cudaSetDevice(h->device);
    cudaStreamSynchronize(h->stream);
    free_batch_buffers(b);
    delete b;
    return FSB_OK;
}

int fsb_counters(const fsb_handle* h, fsb_counters_t* out) {
    if (!h || !out) return FSB_ERR_INVALID;
    *out = h->counters;
    return FSB_OK;
}

}  // extern "C"
