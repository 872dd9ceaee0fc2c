// fsb_internal.h - structures shared by the host shim (fsb_shim.cpp) and the CUDA kernels.
#pragma once
#include <stddef.h>
#include <stdint.h>

namespace fsb {

// ---- compile-time geometry of the streaming kernel ---------------------------------------------------------
constexpr int kThreads = 512;                 // consumer threads per CTA (16 warps); the streaming kernel adds a copy warp and a set-up warp
constexpr int kTile = 8192;                   // fp32 logits per CTA tile (32 KiB, one bulk copy; 512 logits per warp)
constexpr int kStages = 4;                    // tiles in flight per CTA
constexpr int kMaxK = 256;                    // largest k of the candidate path (== FSB_MAX_CANDIDATE_K)
constexpr int kLaneQueue = 6;                 // cells (four logits and their first token id) a lane can note before room must be made
constexpr int kPoolCap = 384;                 // candidates of a warp's overflow pool in global memory (>= kMaxK + 128)
constexpr int kItemTilesMax = 8;              // tiles of the largest work item (a chunk of one row)
constexpr int kItemBitmapWords = kItemTilesMax * kTile / 32;   // penalty bitmap of one work item
constexpr int kMaxChunks = 32;                // chunks a row may be cut into
constexpr int kListCap = 512;                 // candidates that are ordered by counting ranks (one thread per entry at most)
constexpr int kGatherCap = kLaneQueue * kThreads * 2;   // 6144: candidates of all chunks of a row that the merging CTA gathers
                                                        // (they land in the lanes' queue memory, 16 bytes per queue entry)
constexpr int kRowScratch = kGatherCap + kMaxChunks;    // entries of a row's scratch in an engine: the chunks' slots, then their counts
constexpr int kMergeCap = 2400;               // candidates the list-merge kernel (vocabulary sharding) gathers per row
constexpr int kWindowTableInts = 72;          // int32 words per stream of a resident verification call: 6 + up to 66 drafts
constexpr int kCounterWords = 4;              // work counters of a launch: [0] items handed out, [1] CTAs that have left

// status word bits written by kernels (0 = fine)
enum : uint32_t {
    kStatusCopyTimeout = 1u,     // a wait on this CTA's own copies or hand-overs did not end within the limit
    kStatusMergeOverflow = 4u,   // a row has more candidates to merge than its scratch has room for (the planner prevents it)
    kStatusEmptyRow = 8u         // a row produced no candidate (all logits NaN)
};

// row flags
enum : int32_t {
    kRowGreedy = 1,       // temperature <= 0 or top_k == 1: argmax, no draw
    kRowPenalty = 2,      // the row has a non-empty penalty window and penalty != 1
    kRowAppend = 4,       // resident histories: the row's token is appended at hist_begin + hist_len of the id pool
    kRowDraft = 8         // resident verification windows: gather_off holds the draft id that is the last id of the row's window
};

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

// Arguments of the streaming candidate kernel.  A row is cut into n_chunks chunks of chunk_len[c] tiles; the work items
// (row, chunk) are numbered chunk-major (item = chunk * n_rows + row) and handed to the CTAs in that order.
struct StreamArgs {
    const float* logits;       // base of the [rows][ld] matrix
    const RowDesc* rows;       // n_rows descriptors (only rows of the candidate path)
    const int32_t* hist;       // packed penalty-window ids
    uint64_t* scratch;         // [n_rows][scratch_stride]: chunk c of a row publishes its candidates in slot c (slot_cap entries),
                               // their number in entry scratch_stride - 1 - c
    uint64_t* pools;           // [grid][16][pool_cap] overflow pools of the consumer warps (touched on hostile data only)
    uint32_t* ticket;          // [n_rows] chunks of the row that have finished (self-resetting)
    uint32_t* row_bound;       // [n_rows] order-preserving key of a value that k logits of the row are known to reach (self-resetting)
    uint32_t* work;            // [kCounterWords] dynamic work counter and exit counter (self-resetting)
    int32_t* tokens;           // output tokens, indexed by RowDesc::out_index
    uint32_t* status;          // one word, OR of kStatus* bits
    // optional kept-set record, indexed by out_index (null = off)
    int32_t* kept_ids;         // [rows][kMaxK]
    double* kept_pr;           // [rows][kMaxK]
    int32_t* kept_n;           // [rows]
    // optional per-row sorted candidates for the vocabulary-sharded mode (null = run the epilogue here)
    uint64_t* shard_out;       // [rows][kMaxK] composites, descending
    int32_t* shard_n;          // [rows]
    uint64_t* trace;           // optional [grid][16] timestamps (diagnostics), null = off
    int64_t row_ld;            // >= 0: row r starts at r * row_ld (no descriptor read before the first copy)
    int64_t scratch_stride;    // entries per row of `scratch`
    int32_t n_rows;
    int32_t n_vocab;
    int32_t tiles_per_row;
    int32_t n_chunks;
    int32_t n_items;           // n_rows * n_chunks
    int32_t slot_cap;          // entries of a chunk's slot in the row's scratch (>= the largest k of the launch)
    int32_t pool_cap;          // entries of a warp's overflow pool (>= the largest k of the launch + 128)
    int32_t bulk_ok;           // rows start on 16-byte boundaries: tiles can come by bulk async copy
    int32_t write_back;        // store penalised values into the caller's rows
    int32_t vocab_offset;      // token id of column 0
    float softcap;             // 0 = off
    int32_t overlap;           // launch with programmatic stream serialization (see fsb_set_launch_overlap)
    int32_t scan_sums;         // epilogue: 0 = sums in candidate order by one thread (the reference's order), 1 = warp prefix scan
    int32_t debug;             // development switches (wrong results): 1 admit nothing, 2 skip the end-of-item work, 4 skip the penalty
    uint8_t chunk_len[kMaxChunks];
};

size_t stream_kernel_smem_bytes();
// Defined in fsb_kernels.cu.  All return a cudaError_t as int (0 = success).
int prepare_device_kernels(int* ctas_per_sm);
int launch_stream_kernel(const StreamArgs& a, int grid, void* stream);
// How every row of a launch is cut into work items (chunk_len[c] tiles each); returns the number of chunks, 0 if
// the rows cannot be scheduled: at most max_chunks chunks, each with a slot of at least kmax of the gather_cap
// entries the merging CTA can take.  `slots` = CTAs that run at once.  *slot_cap = entries per chunk slot.
int plan_chunks(int n_rows, int n_vocab, int kmax, int slots, int gather_cap, int max_chunks, uint8_t* chunk_len, int* slot_cap);
int launch_append_tokens(const RowDesc* rows, int n_rows, const int32_t* tokens, int32_t* pool, void* stream);
int launch_merge_lists(const void* lists, const int32_t* list_n, int n_lists, int list_stride, int n_rows, const RowDesc* rows, int32_t* tokens,
                       int32_t* kept_ids, double* kept_pr, int32_t* kept_n, uint32_t* status, int scan_sums, void* stream);
int launch_write_drafts(const RowDesc* rows, int n_rows, int32_t* pool, void* stream);
int launch_accept_windows(const int32_t* table, int n_streams, const int32_t* tokens, int32_t* pool, void* stream);
int launch_gather_patched(const float* logits, const RowDesc* rows, int n_rows, const int32_t* hist, int n_vocab, int vocab_offset,
                          float* out, void* stream);

// Defined in fsb_fullrow.cu.
size_t full_row_smem_bytes(int n_vocab);
int prepare_full_row_kernel(int max_vocab);
int launch_full_row_kernel(const float* logits, const RowDesc* rows, int n_rows, const int32_t* hist, int32_t* tokens, int32_t* kept_ids,
                           double* kept_pr, int32_t* kept_n, int record, uint32_t* status, int n_vocab, int vocab_offset, int write_back,
                           float softcap, uint64_t* trace, void* stream);

}  // namespace fsb
