// fsb_internal.h - structures shared by the host shim (fsb_shim.cpp) and the CUDA kernels.
#pragma once
#include <stddef.h>
#include <stdint.h>

namespace fsb {

// ---- compile-time geometry of the streaming kernel ---------------------------------------------------------
constexpr int kThreads = 512;                 // consumer threads per CTA (16 warps); the streaming kernel adds one producer warp
constexpr int kTile = 8192;                   // fp32 logits per CTA tile (32 KiB, one bulk copy; 512 logits per warp)
constexpr int kStages = 4;                    // tiles in flight per CTA
constexpr int kMaxK = 256;                    // largest k of the candidate path (== FSB_MAX_CANDIDATE_K)
constexpr int kLaneQueue = 16;                // cells (4-byte entries) a lane can note before it must drop stale ones
constexpr int kFlatCells = 960;               // cells (float4 + token id) gathered for one selection round
constexpr int kCellBytes = 20;
constexpr int kMergeCap = kFlatCells * kCellBytes / 8;   // 2400: candidates one row may gather from all its segments
                                                          // (the gathered cells' memory seen as a list of composites)
constexpr int kBitmapSpan = 262144;           // columns one penalty bitmap covers (one segment never spans more)
constexpr int kBitmapWords = kBitmapSpan / 32;
constexpr int kMaxTilesPerCta = kBitmapSpan / kTile;

// status word bits written by kernels (0 = fine)
enum : uint32_t {
    kStatusCopyTimeout = 1u,     // a bulk copy did not land within the wait limit
    kStatusMergeOverflow = 4u,   // a row has more segments than its scratch has room for (the planner prevents it)
    kStatusEmptyRow = 8u         // a row produced no candidate (all logits NaN)
};

// row flags
enum : int32_t {
    kRowGreedy = 1,       // temperature <= 0 or top_k == 1: argmax, no draw
    kRowPenalty = 2,      // the row has a non-empty penalty window and penalty != 1
    kRowAppend = 4,       // resident histories: the row's token is appended at hist_begin + hist_len of the id pool
    kRowDraft = 8         // resident verification windows: gather_off holds the draft id that is the last id of the row's window
};

constexpr int kWindowTableInts = 72;          // int32 words per stream of a resident verification call: 6 + up to 66 drafts

// One row of a batch, as the kernels see it (64 bytes).
struct RowDesc {
    uint64_t rng_word;     // raw 64-bit engine output of this row's draw (unused for greedy rows)
    int64_t logits_off;    // element offset of the row from the logits base pointer
    int64_t hist_begin;    // first id of the penalty window in the device history array
    int32_t hist_len;      // ids in the window (0: no penalty)
    int32_t k;             // effective candidate count: 1 for greedy, else (0 < top_k < n) ? top_k : n
    float temperature;
    float top_p;
    float min_p;
    float penalty;
    int32_t flags;
    int32_t out_index;     // position of the row's token in the output array
    int32_t k_global;      // vocabulary sharding: candidate count of the whole row (k is the shard's); otherwise == k
    int32_t gather_off;    // where the row's window values go when patched entries are gathered for a host caller
};
static_assert(sizeof(RowDesc) == 64, "RowDesc layout");

// Arguments of the streaming candidate kernel.
struct StreamArgs {
    const float* logits;       // base of the [rows][ld] matrix
    const RowDesc* rows;       // n_rows descriptors (only rows of the candidate path)
    const int32_t* hist;       // packed penalty-window ids
    uint64_t* scratch;         // [n_rows][kMergeCap]: per segment of a row k ordered candidates, the counts at the end
    uint32_t* ticket;          // [n_rows] segments that have finished (self-resetting)
    int32_t* tokens;           // output tokens, indexed by RowDesc::out_index
    uint32_t* status;          // one word, OR of kStatus* bits
    // optional mirror in mapped host memory (device addresses of pinned host words; null = off): tokens are stored
    // there as well, and a non-zero word is stored to status_host whenever a status bit is set, so that a synchronous
    // caller needs no copy back - it waits for the stream and reads its own memory
    int32_t* tokens_host;
    uint32_t* status_host;
    // optional kept-set record, indexed by out_index (null = off)
    int32_t* kept_ids;         // [rows][kMaxK]
    double* kept_pr;           // [rows][kMaxK]
    int32_t* kept_n;           // [rows]
    // optional per-row sorted candidates for the vocabulary-sharded mode (null = run the epilogue here)
    uint64_t* shard_out;       // [rows][shard_stride] composites, descending
    int32_t* shard_n;          // [rows] their number; null: a list starts with a header word that holds it
    int32_t shard_stride;      // 64-bit words per row of shard_out
    uint64_t* trace;           // optional [grid][8] timestamps (diagnostics), null = off
    int64_t row_ld;            // >= 0: row r starts at r * row_ld (no descriptor read before the first copy)
    int32_t n_rows;
    int32_t n_vocab;
    int32_t tiles_per_row;
    int32_t tiles_per_cta;
    int32_t total_tiles;
    int32_t bulk_ok;           // rows start on 16-byte boundaries: tiles can come by bulk async copy
    int32_t write_back;        // store penalised values into the caller's rows
    int32_t vocab_offset;      // token id of column 0
    float softcap;             // 0 = off
    int32_t overlap;           // launch with programmatic stream serialization (see fsb_set_launch_overlap)
    int32_t all_greedy;        // every row of the launch is greedy: the variant of the kernel that keeps one best logit per lane
                               // instead of queues of candidates
    int32_t pair;              // 0, or c = 2, 4, 8: every row is exactly c aligned CTAs (c r .. c r + c - 1), launched as a cluster
                               // whose CTAs hand their candidates to the first one through shared memory instead of the row's scratch
};

// The launch plan: the flat list of tiles is dealt to the CTAs in equal contiguous ranges of tiles_per_cta tiles.
struct Plan {
    int tiles_per_row = 0, tiles_per_cta = 0, total_tiles = 0, grid = 0;
};
// `slots` = CTAs that run at once.
Plan make_plan(int n_rows, int n_vocab, int kmax, int slots);

size_t stream_kernel_smem_bytes();
// All return a cudaError_t as int (0 = success).
int prepare_device_kernels(int* ctas_per_sm);
int launch_stream_kernel(const StreamArgs& a, int grid, void* stream);

// One stream of a prompt-lookup drafting call: where its history lies in the id pool and what to look for.
struct LookupDesc {
    int64_t begin;         // first id of the history in the id pool
    int32_t len;           // ids in the history
    int32_t kmax;          // most drafts wanted
    int32_t min_n;         // shortest suffix that may be matched (>= 1)
    int32_t eos;           // end-of-sequence id: a draft stops before it
};
static_assert(sizeof(LookupDesc) == 24, "LookupDesc layout");
constexpr int kDraftStride = 68;              // int32 words per stream of a drafting call: the count, then up to 67 drafts

// Defined in fsb_support.cu.
int prepare_support_kernels();
int launch_lookup_drafts(const int32_t* pool, const LookupDesc* desc, int n_streams, int32_t* out, int stride, void* stream);
int launch_append_tokens(const RowDesc* rows, int n_rows, const int32_t* tokens, int32_t* pool, void* stream);
int launch_merge_lists(const void* lists, const int32_t* list_n, int n_lists, int list_stride, int n_rows, const RowDesc* rows, int32_t* tokens,
                       int32_t* kept_ids, double* kept_pr, int32_t* kept_n, uint32_t* status, void* stream);
int launch_write_drafts(const RowDesc* rows, int n_rows, int32_t* pool, void* stream);
int launch_accept_windows(const int32_t* table, int n_streams, const int32_t* tokens, int32_t* pool, void* stream);
int launch_gather_patched(const float* logits, const RowDesc* rows, int n_rows, const int32_t* hist, int n_vocab, int vocab_offset,
                          float* out, void* stream);

// Defined in fsb_fullrow.cu.
size_t full_row_smem_bytes(int n_vocab);
int prepare_full_row_kernel(int max_vocab);
int launch_full_row_kernel(const float* logits, const RowDesc* rows, int n_rows, const int32_t* hist, int32_t* tokens, int32_t* tokens_host,
                           int32_t* kept_ids, double* kept_pr, int32_t* kept_n, int record, uint32_t* status, uint32_t* status_host, int n_vocab,
                           int vocab_offset, int write_back, float softcap, uint64_t* trace, void* stream);

}  // namespace fsb
