/*
 * ferro_sampler_b200.h - C ABI of the B200 batched token sampler.
 *
 * Drop-in boundary for the token sampler of paragontasx/ferro (reference paths below are relative
 * to that project's root).  The reference has no FFI layer for this path: it is a C++ class,
 * ferro::Sampler (src/sampler.h:23-34), called once per produced token per stream by the decode
 * loops.  This header exports the same operation as a plain-C interface over hand-written sm_100a
 * CUDA kernels: one call samples a whole batch of rows (one row per stream / verification-window
 * position).  A header-only C++ adapter with the reference's own class signature lives in
 * ferro_sampler_b200.hpp.
 *
 * Conventions
 *   - every function returns 0 (FSB_OK) or a negative fsb_status; nothing throws, nothing aborts;
 *   - fsb_last_error() gives the text of the most recent failure on a handle;
 *   - a handle is single-threaded (like the reference sampler, which only the one inference worker
 *     thread touches, src/server.cpp:3-4); distinct handles are independent;
 *   - there is no CPU fallback: without a CUDA device fsb_create fails with FSB_ERR_NO_DEVICE.
 */
#ifndef FERRO_SAMPLER_B200_H
#define FERRO_SAMPLER_B200_H

#include <stdint.h>

#if defined(__GNUC__)
#define FSB_API __attribute__((visibility("default")))
#else
#define FSB_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Field-for-field the reference's `struct SamplerParams` (src/sampler.h:12-21): 40 bytes, seed at offset 32. */
typedef struct ferro_sampler_params {
    float temperature;        /* <= 0 (or top_k == 1): greedy argmax after the penalty; default 0.05 */
    int32_t top_k;            /* 0 = off (all tokens are candidates); default 50 */
    float top_p;              /* 1 = off; default 1 */
    float min_p;              /* 0 = off; default 0 */
    float repetition_penalty; /* 1 = off; default 1.05 */
    int32_t repeat_last_n;    /* penalty window: last N history ids; -1 = whole history; 0 = no penalty */
    int32_t penalty_from;     /* history positions before this are never penalised */
    uint64_t seed;            /* 0 = nondeterministic (std::random_device), as in the reference */
} ferro_sampler_params;

typedef struct fsb_handle fsb_handle; /* one sampler engine bound to one CUDA device */
typedef struct fsb_batch fsb_batch;   /* a prepared, device-resident batch (see fsb_batch_prepare) */

typedef enum fsb_status {
    FSB_OK = 0,
    FSB_ERR_INVALID = -1,   /* null pointer, negative size, bad flag combination */
    FSB_ERR_RANGE = -2,     /* a sampling parameter outside the ranges the reference's server accepts */
    FSB_ERR_CAPACITY = -3,  /* rows / vocabulary / history beyond what the handle was created for */
    FSB_ERR_CUDA = -4,      /* a CUDA runtime call failed; text in fsb_last_error */
    FSB_ERR_STREAM_ID = -5, /* unknown or closed stream id */
    FSB_ERR_NO_DEVICE = -6, /* no usable CUDA device */
    FSB_ERR_DEVICE = -7     /* a kernel reported an internal error through its status word */
} fsb_status;

/* flags of fsb_sample_batch / fsb_verify_windows / fsb_batch_prepare */
enum {
    FSB_LOGITS_ON_HOST = 1u, /* `logits` is a host pointer (staged to the device inside the call); default: device pointer */
    FSB_WRITE_BACK = 2u,     /* store the penalised logits back into the caller's rows, the reference's in-place side
                                effect ("logits: [n_vocab], modified in place", src/sampler.h:26) */
    FSB_KEEP_KEPT_SET = 4u,  /* record every row's kept set (ids + probabilities) for fsb_last_kept */
    FSB_APPEND_SAMPLED = 8u  /* resident calls only: append the sampled tokens to their streams' resident histories */
};

/* Largest effective k (after the reference's clamp k = (0 < top_k < n_vocab) ? top_k : n_vocab) that
 * the single-pass candidate kernel handles; rows with a larger k take the multi-pass full-row kernel. */
#define FSB_MAX_CANDIDATE_K 256

/* ---- engine ------------------------------------------------------------------------------------------- */

/* Create an engine on CUDA device `device` able to take batches of up to max_rows rows of up to max_vocab
 * logits with up to max_hist_ids penalty-window ids per batch in total.  All scratch is allocated here.
 * Replaces: construction of the per-request samplers' shared resources; no reference counterpart
 * (the reference keeps a scratch vector inside each Sampler, src/sampler.h:33). */
FSB_API int fsb_create(int device, int max_rows, int max_vocab, int64_t max_hist_ids, fsb_handle** out);
FSB_API int fsb_destroy(fsb_handle* h);
FSB_API const char* fsb_last_error(const fsb_handle* h);

/* Launch on the caller's CUDA stream (a cudaStream_t passed as void*) instead of the handle's own. */
FSB_API int fsb_set_cuda_stream(fsb_handle* h, void* cuda_stream);

/* Fuse the final-logit softcap x = cap * tanhf(x / cap) in front of the penalty (the producer-side step
 * of src/model_gemma4.cpp:520-521).  cap = 0 turns it off (the default: the caller's logits are final). */
FSB_API int fsb_set_softcap(fsb_handle* h, float cap);

/* Diagnostics: when set to a device buffer of 8 uint64 per CTA of the streaming kernel (and 64 more words after
 * the first 4096 x 8 for the full-vocabulary kernel), the kernels write time stamps of their phases there.  The
 * streaming kernel: word 0 %globaltimer (ns) at the CTA's start and word 7 the SM's cycle counter at the same
 * moment; words 1, 4, 2, 5, 6 the cycle counter after set-up, after the CTA's last tile, after the candidate list of
 * its last segment, after ordering / merging, and at the end; word 3 the length of that candidate list.  NULL (the
 * default) turns it off.  No reference
 * counterpart. */
FSB_API int fsb_set_trace_buffer(fsb_handle* h, void* device_buffer);

/* How consecutive launches follow one another (0, the default: plain stream order).
 * 1: fsb_batch_launch starts the streaming kernel with programmatic stream serialization and its CTAs may begin to
 *    read logits while the previous kernel in the stream is still finishing; every write of the launch (tokens, kept
 *    sets, scratch) waits for that kernel to be complete.  Use it only if the logits of a launch are complete before
 *    the previous kernel in the stream starts (for instance logits that alternate between buffers filled well ahead);
 *    batches with FSB_WRITE_BACK wait before they read anything, so they gain nothing.
 * 2: the same launch attribute, but every CTA waits for the previous kernel to be complete before it reads or writes
 *    anything.  Results and ordering are those of plain stream order - the logits may be produced by the kernel just
 *    before - and only the launch latency (CTA placement, barrier set-up) is hidden behind that kernel's end.
 * No reference counterpart. */
FSB_API int fsb_set_launch_overlap(fsb_handle* h, int on);

/* Column offset of this device's vocabulary shard: local column c is token id c + offset (vocab sharding).
 * fsb_set_vocab_shard also tells the engine how many columns the whole row has, so that a row's candidate count
 * follows the whole row (k = (0 < top_k < global_vocab) ? top_k : global_vocab, src/sampler.cpp:27) even when top_k
 * exceeds the shard's width; global_vocab = 0 means "this engine holds whole rows". */
FSB_API int fsb_set_vocab_offset(fsb_handle* h, int32_t offset);
FSB_API int fsb_set_vocab_shard(fsb_handle* h, int32_t offset, int32_t global_vocab);

/* Reference defaults (src/sampler.h:13-20) and the range check of the reference's request parser
 * (src/server.cpp:1071: temperature >= 0, 0 < top_p <= 1, top_k >= 0, repetition_penalty > 0, repeat_last_n >= -1)
 * extended by 0 <= min_p <= 1 and penalty_from >= 0. */
FSB_API void fsb_params_default(ferro_sampler_params* p);
FSB_API int fsb_params_validate(const ferro_sampler_params* p);

/* ---- request front end --------------------------------------------------------------------------------- */

/* The request fields the reference's chat-completion handler reads before it constructs a sampler
 * (src/server.cpp:1060-1072).  The reference takes a field only when it is a JSON number (its jnum falls back to the
 * default for strings, booleans and null; penalize_prompt only when it is a JSON boolean): the caller sets the
 * field's bit in `present` in exactly those cases.  Numbers are doubles, as jnum returns them. */
enum {
    FSB_REQ_TEMPERATURE = 1u << 0, FSB_REQ_TOP_P = 1u << 1, FSB_REQ_TOP_K = 1u << 2, FSB_REQ_MIN_P = 1u << 3,
    FSB_REQ_REPETITION_PENALTY = 1u << 4, FSB_REQ_REPEAT_PENALTY = 1u << 5, /* alias, used when the first is absent */
    FSB_REQ_REPEAT_LAST_N = 1u << 6, FSB_REQ_PENALTY_LAST_N = 1u << 7,       /* alias, used when the first is absent */
    FSB_REQ_PENALIZE_PROMPT = 1u << 8, FSB_REQ_SEED = 1u << 9
};
typedef struct fsb_request_fields {
    uint32_t present;
    int32_t penalize_prompt;
    double temperature, top_p, top_k, min_p, repetition_penalty, repeat_penalty, repeat_last_n, penalty_last_n, seed;
} fsb_request_fields;
/* The server options that act as per-request defaults (src/server.h:35-37; flags --repeat-penalty, --repeat-last-n,
 * --penalty-scope, src/main.cpp:250-252). */
typedef struct fsb_server_defaults {
    float repeat_penalty;    /* <= 0: the sampler's own default 1.05 */
    int32_t repeat_last_n;   /* -1 whole context, 0 off, N last tokens */
    int32_t penalize_prompt; /* 1 = "--penalty-scope all" (default), 0 = "generated" */
} fsb_server_defaults;
FSB_API void fsb_server_defaults_init(fsb_server_defaults* d);
/* src/server.cpp:1060-1072: struct defaults, overridden by the request; repetition_penalty falls back to repeat_penalty,
 * then to the server default, then to 1.05; repeat_last_n to penalty_last_n, then to the server default; with
 * penalize_prompt false penalty_from = prompt_tokens; seed defaults to 0.  FSB_ERR_RANGE where the reference answers
 * 400 "sampling parameter out of range" (temperature < 0, top_p outside (0, 1], top_k < 0, repetition_penalty <= 0,
 * repeat_last_n < -1).  `d` may be NULL (the defaults of fsb_server_defaults_init). */
FSB_API int fsb_params_from_request(const fsb_request_fields* f, const fsb_server_defaults* d, int32_t prompt_tokens, ferro_sampler_params* out);
/* One command-line flag of the reference's binary (src/main.cpp:250-262): --temp --top-k --top-p --min-p --rep-penalty
 * --seed set the generate command's parameters `p`; --repeat-penalty --repeat-last-n --penalty-scope set the server
 * defaults `d` (--repeat-last-n both).  Returns 1 if the flag was one of these, 0 if it is not a sampling flag,
 * FSB_ERR_RANGE for a bad --penalty-scope value, FSB_ERR_INVALID for a missing value. */
FSB_API int fsb_params_apply_cli_flag(ferro_sampler_params* p, fsb_server_defaults* d, const char* flag, const char* value);

/* ---- streams: one per request, like `new Sampler(j.sp)` at src/server.cpp:545 ---------------------------- */

/* Opens a stream: copies the parameters and seeds a std::mt19937_64 exactly as src/sampler.h:25 does. */
FSB_API int fsb_stream_open(fsb_handle* h, const ferro_sampler_params* p, int* stream_id);
FSB_API int fsb_stream_close(fsb_handle* h, int stream_id);
/* Sampler::params() (src/sampler.h:29) */
FSB_API int fsb_stream_params(const fsb_handle* h, int stream_id, ferro_sampler_params* out);
/* The engine position as (seed actually used, number of 64-bit outputs consumed); set re-creates it. */
FSB_API int fsb_stream_state_get(const fsb_handle* h, int stream_id, uint64_t* seed, uint64_t* draws);
FSB_API int fsb_stream_state_set(fsb_handle* h, int stream_id, uint64_t seed, uint64_t draws);

/* ---- sampling ------------------------------------------------------------------------------------------- */

/* Equivalent to, for i in 0..n_rows-1 in order:
 *     tokens_out[i] = stream[stream_ids[i]].sample(logits + i*ld, n_vocab, history_i)      (src/sampler.cpp:10-50)
 * i.e. the per-slot loop of a decode step (src/server.cpp:603-608) as one device call.
 * history_i = hist_flat[hist_off[i] .. hist_off[i+1]) (host memory; all tokens of the context so far).
 * One 64-bit engine output is consumed per stochastic row, none per greedy row.  Synchronous: tokens are
 * in tokens_out (host) on return.  The history is not modified (the caller appends, src/server.cpp:342). */
FSB_API int fsb_sample_batch(fsb_handle* h, int n_rows, const int* stream_ids, const float* logits, int64_t ld, int n_vocab,
                     const int32_t* hist_flat, const int64_t* hist_off, int32_t* tokens_out, unsigned flags);

/* Device-resident histories.  The reference's scheduler keeps one growing token history per request and hands the
 * whole of it to every sample() call (src/server.cpp:605 with g.hist, appended by gen_token at :342).  With these
 * calls a stream keeps its history in the engine (a host mirror and a device copy in a pool of max_hist_ids ids,
 * regions of power-of-two size), so that a decode step moves one token id per stream instead of the whole window.
 *   fsb_stream_history_set     replaces the stream's history (the prompt, at request start);
 *   fsb_stream_history_append  adds ids (tokens produced elsewhere: accepted drafts, a forced token);
 *   fsb_sample_batch_resident  is fsb_sample_batch with history_i = the resident history of stream_ids[i]; with
 *                              FSB_APPEND_SAMPLED every sampled token is appended to its stream's history (on the
 *                              device by a small kernel, in the mirror after the read-back), which is what
 *                              gen_token does next anyway.  A stream may appear once per call.
 * Closing a stream frees its region.  FSB_ERR_CAPACITY when the pool cannot hold a region. */
FSB_API int fsb_stream_history_set(fsb_handle* h, int stream_id, const int32_t* ids, int64_t n);
FSB_API int fsb_stream_history_append(fsb_handle* h, int stream_id, const int32_t* ids, int n);
FSB_API int fsb_stream_history_len(const fsb_handle* h, int stream_id, int64_t* n);
FSB_API int fsb_sample_batch_resident(fsb_handle* h, int n_rows, const int* stream_ids, const float* logits, int64_t ld, int n_vocab,
                                      int32_t* tokens_out, unsigned flags);

/* Prompt-lookup drafting (lookup_draft, src/server.cpp:552-564) over resident histories: for stream i the tokens that
 * followed the most recent earlier occurrence of the last n tokens of its history, n = 4, 3, ... min_n[i] - at most
 * kmax[i] of them (and at most 67), never the end-of-sequence id `eos` or anything after it; an occurrence with an empty
 * continuation is passed over, as in the reference.  One small kernel over the id pool, one CTA per stream; the drafts
 * of stream i are written to drafts_out[i * stride ..] and their number to n_out[i].  min_n[i] >= 1 (the reference
 * passes 2 or 3).  The caller builds the rows [last token, drafts ...] of fsb_verify_windows_resident from them. */
FSB_API int fsb_lookup_drafts_resident(fsb_handle* h, int n_streams, const int* stream_ids, const int* kmax, const int* min_n, int32_t eos,
                                       int32_t* drafts_out, int stride, int* n_out);

/* Speculative verification windows (the accept loop of src/server.cpp:626-645) for n_streams streams.
 * Stream i owns rows row_off[i] .. row_off[i+1]) of `logits`; rows_flat holds, per stream, [last token, draft_1 ..
 * draft_{m-1}] as the scheduler builds them (src/server.cpp:617).  Row r is sampled with history_i followed by
 * draft_1..draft_r, and is accepted while every earlier sampled token equalled the next draft.  On return
 * tokens_out[row] holds the sampled token of every accepted row (-1 for rows the reference would not have
 * sampled), acc_out[i] the number of rows sampled, confirmed_out[i] the number of confirmed drafts, and each
 * stream's engine has advanced by exactly the draws of its sampled rows.  max_accept (may be NULL) caps acc per
 * stream (e.g. the remaining token budget). */
FSB_API int fsb_verify_windows(fsb_handle* h, int n_streams, const int* stream_ids, const int* row_off, const int32_t* rows_flat,
                       const float* logits, int64_t ld, int n_vocab, const int32_t* hist_flat, const int64_t* hist_off,
                       const int* max_accept, int32_t* tokens_out, int* acc_out, int* confirmed_out, unsigned flags);

/* fsb_verify_windows with every stream's history taken from its resident history (fsb_stream_history_*): a
 * speculative step then uploads the drafts only.  The drafts are written behind the stream's history in the id pool
 * before the launch (the pool must have room for history + window rows per stream).  With FSB_APPEND_SAMPLED the
 * sampled tokens of the accepted rows are appended to the stream's history (what gen_token does next,
 * src/server.cpp:342): on the device by a small kernel that walks the same accept loop, in the mirror after the
 * read-back; a window may then hold at most 66 drafts.  Without the flag the histories are left as they were. */
FSB_API int fsb_verify_windows_resident(fsb_handle* h, int n_streams, const int* stream_ids, const int* row_off, const int32_t* rows_flat,
                                        const float* logits, int64_t ld, int n_vocab, const int* max_accept, int32_t* tokens_out,
                                        int* acc_out, int* confirmed_out, unsigned flags);

/* Kept set of row `row` of the most recent call made with FSB_KEEP_KEPT_SET: the candidates that survived
 * min-p / top-p in (logit descending, id ascending) order with their probabilities (normalised over the k
 * candidates, as src/sampler.cpp:41 leaves them).  At most `cap` entries are copied; *n_keep is the full size. */
FSB_API int fsb_last_kept(fsb_handle* h, int row, int cap, int32_t* ids, double* probs, int* n_keep);

/* ---- device-resident batches (serving loops that keep everything on the device; the benchmark) -------------- */

/* Validates and uploads everything a batch needs except the logits: row descriptors (parameters, penalty
 * windows, one engine output per stochastic row) and the window ids.  The same batch can then be launched many
 * times on different logits buffers. */
FSB_API int fsb_batch_prepare(fsb_handle* h, int n_rows, const int* stream_ids, int64_t ld, int n_vocab,
                      const int32_t* hist_flat, const int64_t* hist_off, unsigned flags, fsb_batch** out);
/* Draw fresh engine outputs for the batch's stochastic rows and upload them (8 bytes per row). */
FSB_API int fsb_batch_redraw(fsb_handle* h, fsb_batch* b);
/* Enqueue the kernels for one step on `logits_dev` ([n_rows][ld] fp32 in device memory); asynchronous. */
FSB_API int fsb_batch_launch(fsb_handle* h, fsb_batch* b, const float* logits_dev);
/* Wait for the last launch of `b` and copy its tokens (n_rows int32) to host memory. */
FSB_API int fsb_batch_tokens(fsb_handle* h, fsb_batch* b, int32_t* tokens_out);
/* Vocabulary sharding: this device holds columns [offset, offset + n_vocab) of every row (fsb_set_vocab_shard gives
 * the offset and the width of the whole row; history ids stay global).  fsb_batch_shard_launch runs the streaming kernel on the shard and leaves,
 * per row, the shard's best k candidates in descending order: `lists_out_dev` is [n_rows][FSB_MAX_CANDIDATE_K]
 * 64-bit keys (order-preserving value key << 32 | 0xFFFFFFFF - global token id), `counts_out_dev` [n_rows] how many
 * are valid.  The caller brings the lists of all shards into this device's memory (an all-gather: [n_lists][n_rows]
 * [FSB_MAX_CANDIDATE_K] and [n_lists][n_rows]) and calls fsb_batch_merge_launch, which finishes every row exactly
 * as the unsharded launch would (the best k of the whole row are among the shards' best k); fsb_batch_tokens then
 * returns the tokens.  Every rank must have opened the same streams in the same state, so that all ranks draw the
 * same engine outputs.  Rows with top_k = 0 or k > FSB_MAX_CANDIDATE_K are refused (FSB_ERR_RANGE): shard those by
 * rows.  At most 9 lists.  Both calls are asynchronous on the engine's stream.  No reference counterpart. */
FSB_API int fsb_batch_shard_launch(fsb_handle* h, fsb_batch* b, const float* logits_shard_dev, uint64_t* lists_out_dev,
                                   int32_t* counts_out_dev);
FSB_API int fsb_batch_merge_launch(fsb_handle* h, fsb_batch* b, const uint64_t* lists_dev, const int32_t* counts_dev, int n_lists);
/* The same two steps with packed lists, for exchanges that should move no more than they must: a row's list is
 * `stride_words` 64-bit words - word 0 its length, words 1 .. length its candidates in descending order - with
 * stride_words >= 1 + fsb_batch_max_k(b) (the largest candidate count of the staged rows on this shard), so a rank
 * sends rows x stride_words x 8 bytes in one piece, counts included.  fsb_batch_merge_launch_packed finishes rows
 * [row_begin, row_begin + n_rows) of the batch from `packed_dev` = [n_lists][n_rows][stride_words]: with an
 * all-to-all that brings every rank the lists of its own block of rows, each rank merges only that block and the
 * tokens are exchanged afterwards (fsb_batch_tokens_device gives the device array, [rows] int32 indexed by row;
 * fsb_batch_check waits for the launches and reports the device status without copying tokens to the caller). */
FSB_API int fsb_batch_max_k(const fsb_batch* b);
FSB_API int fsb_batch_shard_launch_packed(fsb_handle* h, fsb_batch* b, const float* logits_shard_dev, uint64_t* packed_out_dev, int32_t stride_words);
FSB_API int fsb_batch_merge_launch_packed(fsb_handle* h, fsb_batch* b, const uint64_t* packed_dev, int32_t stride_words, int n_lists,
                                          int32_t row_begin, int32_t n_rows);
FSB_API int32_t* fsb_batch_tokens_device(fsb_batch* b);
FSB_API int fsb_batch_check(fsb_handle* h, fsb_batch* b);
/* Number of kernels one fsb_batch_launch enqueues (for launch accounting). */
FSB_API int fsb_batch_kernel_count(const fsb_batch* b);
FSB_API int fsb_batch_free(fsb_handle* h, fsb_batch* b);

/* ---- counters --------------------------------------------------------------------------------------------- */
typedef struct fsb_counters_t {
    uint64_t rows_sampled;    /* rows that produced a token */
    uint64_t rows_greedy;     /* of those, greedy rows (no engine output) */
    uint64_t rows_stochastic; /* of those, rows that consumed one engine output */
    uint64_t rows_full_vocab; /* rows that took the multi-pass full-row kernel */
    uint64_t drafted;         /* drafts offered to fsb_verify_windows (src/server.cpp:639 spec_drafted) */
    uint64_t accepted;        /* drafts confirmed (spec_accepted) */
    uint64_t kernel_launches; /* kernels enqueued by this handle */
} fsb_counters_t;
FSB_API int fsb_counters(const fsb_handle* h, fsb_counters_t* out);

/* Greedy tokens (temperature 0: lowest index of the row maximum, src/sampler.cpp:19-23) of up to FSB_STATIC_MAX_ROWS
 * device-resident rows, for callers that must not allocate: no handle, no cudaMalloc / cudaFree / pinned host memory,
 * in this call or any earlier one.  That is the situation of a decode loop whose device memory is owned entirely by
 * the serving engine's own pool, and of code that runs where an allocation would stall the device (a cudaMalloc
 * waits for running kernels).  All device memory the streaming kernel needs besides the caller's buffers (row
 * descriptors, the rows' candidate scratch, its counters and status word: about 1.2 MB) is one array inside the
 * library's own image.  No penalty window, no softcap, no random draw: exactly the rows of a verification window
 * with repetition_penalty 1 (src/server.cpp:630-636).
 *   logits_dev [n_rows][ld] fp32 and tokens_dev [n_rows] int32 are device memory of `device`; the kernels are
 *   enqueued on `cuda_stream` (0 = the default stream).  With FSB_STATIC_WAIT the call waits for them and reports a
 *   kernel error as FSB_ERR_DEVICE; without it the call returns as soon as the work is enqueued.
 *   n_rows > FSB_STATIC_MAX_ROWS is refused with FSB_ERR_CAPACITY (the array has room for that many rows).
 * The first call on a device looks up the array's address and sets the kernel's attributes (with that device
 * current); make that first call before any stream capture begins.  All calls on a device share the one array: every
 * call begins, in stream order, by clearing its counters and its status word, so a kernel error of an earlier call
 * that nobody waited for does not leak into the next one - and is lost: a caller that does not pass FSB_STATIC_WAIT
 * learns of kernel errors only by making a later call with it on the same input.  Two calls whose kernels can run at
 * the same time - different streams, different threads - race on the array.  Not thread-safe.  No reference
 * counterpart. */
#define FSB_STATIC_MAX_ROWS 64
#define FSB_STATIC_WAIT 1u
FSB_API int fsb_argmax_rows_static(int device, const float* logits_dev, int64_t ld, int n_rows, int n_vocab, int32_t* tokens_dev,
                                   void* cuda_stream, unsigned flags);

#ifdef __cplusplus
}
#endif
#endif /* FERRO_SAMPLER_B200_H */
