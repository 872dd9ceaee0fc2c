// fsb_support.cu - the small kernels around the two sampling kernels of the B200 batched token sampler (sm_100a):
// the merge of per-shard candidate lists (vocabulary sharding), the device side of resident histories and resident
// verification windows (src/server.cpp:598-636 of paragontasx/ferro is the host loop they replace), and the gather
// that lets a host caller see the penalised values without any host arithmetic.
#include <cuda_runtime.h>

#include "fsb_device.cuh"

namespace fsb {
namespace {

constexpr size_t kSmemMerge = (size_t)(kMergeCap + kMaxK) * sizeof(u64) + sizeof(SharedCtl);   // gathered lists, ordered candidates, control

// Merge of per-shard candidate lists: one CTA per row gathers the row's n_lists ordered lists (already in this
// device's memory, list g of row r at lists + (g * n_rows + r) * list_stride) and finishes the row exactly as the
// streaming kernel does after its own selection - the k best of the whole row are among the shards' k best, and
// the order (value descending, id ascending) does not depend on the split.  With list_n the lists are bare and
// list_n[g * n_rows + r] gives their lengths; without it a list starts with a header word that holds its length.
__global__ void __launch_bounds__(kThreads, 1) merge_lists_kernel(const u64* lists, const int32_t* list_n, int n_lists, int list_stride, int n_rows,
                                                                 const RowDesc* rows, int32_t* tokens, int32_t* kept_ids, double* kept_pr,
                                                                 int32_t* kept_n, unsigned* status) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    u64* buf = reinterpret_cast<u64*>(smem_raw);
    u64* out = buf + kMergeCap;
    SharedCtl* ctl = reinterpret_cast<SharedCtl*>(out + kMaxK);
    const int row = blockIdx.x, tid = threadIdx.x;
    if (row >= n_rows) return;
    const RowDesc d = rows[row];
    const int hdr = list_n ? 0 : 1;
    int total = 0;   // the same in every thread
    for (int g = 0; g < n_lists; ++g) {
        const u64* src = lists + ((size_t)g * n_rows + row) * (size_t)list_stride;
        const long long stated = list_n ? (long long)list_n[(size_t)g * n_rows + row] : (long long)src[0];
        const int n = (int)max(0ll, min(stated, (long long)min(kMaxK, list_stride - hdr)));
        if (total + n <= kMergeCap) {
            for (int i = tid; i < n; i += kThreads) buf[total + i] = src[hdr + i];
            total += n;
        } else if (tid == 0) {
            atomicOr(status, kStatusMergeOverflow);
        }
    }
    consumer_sync();
    const TailOut tout{tokens, nullptr, nullptr, kept_ids, kept_pr, kept_n, nullptr, nullptr, 0, status};
    const RowTail rt{d.rng_word, d.temperature, d.top_p, d.min_p, d.k_global, d.flags, d.out_index};
    const int kk = topk_sorted(buf, total, d.k_global, out, ctl);
    row_epilogue(out, kk, rt, reinterpret_cast<double*>(buf), ctl, tout);
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

// Resident histories: appends every row's new token to its stream's history on the device.  A row's window always
// ends where its history ends, so the token goes to entry hist_begin + hist_len of the id pool.
__global__ void append_tokens_kernel(const RowDesc* rows, int n_rows, const int32_t* tokens, int32_t* pool) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_rows) return;
    if (rows[r].flags & kRowAppend) pool[rows[r].hist_begin + rows[r].hist_len] = tokens[rows[r].out_index];
}

// Resident verification windows.  Before the launch: draft r of a stream is the last id of row r's window, and goes
// to that place of the id pool.  After it: per stream the accept loop of src/server.cpp:630-636 over the sampled
// tokens (accept while the token equals the next draft, at most `lim` rows), and the accepted tokens are stored
// behind the history.  Table entry of a stream:
// first row, rows m, limit, unused, end of the history in the pool (two words), then the m - 1 drafts.
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
    // every accepted token, not only the last: a row whose penalty window is empty (penalty off) never had its draft
    // written into the pool before the launch
    for (int r = 0; r < acc; ++r) pool[end + r] = tokens[r0 + r];
}

// Prompt-lookup drafting over resident histories (lookup_draft, src/server.cpp:552-564): the tokens that followed
// the most recent earlier occurrence of the history's last n tokens, n = 4, 3, ... min_n - at most kmax of them, cut
// at the end-of-sequence id; an occurrence whose continuation is empty is passed over.  One CTA per stream: every
// thread tests some start positions of an n, the largest matching position wins, one thread copies the draft.
// out[i * stride] = number of drafts of stream i, then the drafts.
__global__ void lookup_drafts_kernel(const int32_t* pool, const LookupDesc* desc, int n_streams, int32_t* out, int stride) {
    __shared__ int best;
    const int i = blockIdx.x;
    if (i >= n_streams) return;
    const LookupDesc d = desc[i];
    const int32_t* h = pool + d.begin;
    const int L = d.len;
    int found_n = 0;
    for (int n = min(4, L - 1); n >= d.min_n && d.kmax > 0; --n) {
        if (threadIdx.x == 0) best = -1;
        __syncthreads();
        for (int p = L - n - 1 - (int)threadIdx.x; p >= 0; p -= (int)blockDim.x) {
            bool eq = h[p + n] != d.eos;            // an occurrence followed by the end-of-sequence id drafts nothing
            for (int k = 0; k < n && eq; ++k) eq = h[p + k] == h[L - n + k];
            if (eq) atomicMax(&best, p);
        }
        __syncthreads();
        if (best >= 0) {
            found_n = n;
            break;
        }
        __syncthreads();   // `best` is reset by thread 0 at the top of the next round
    }
    if (threadIdx.x == 0) {
        int cnt = 0;
        if (found_n > 0)
            for (int k = best + found_n; k < L && cnt < d.kmax && cnt < stride - 1; ++k) {
                if (h[k] == d.eos) break;
                out[(size_t)i * stride + 1 + cnt++] = h[k];
            }
        out[(size_t)i * stride] = cnt;
    }
}

}  // namespace

int launch_lookup_drafts(const int32_t* pool, const LookupDesc* desc, int n_streams, int32_t* out, int stride, void* stream) {
    lookup_drafts_kernel<<<n_streams, 256, 0, static_cast<cudaStream_t>(stream)>>>(pool, desc, n_streams, out, stride);
    return (int)cudaGetLastError();
}

int prepare_support_kernels() {
    return (int)cudaFuncSetAttribute(merge_lists_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemMerge);
}

int launch_merge_lists(const void* lists, const int32_t* list_n, int n_lists, int list_stride, int n_rows, const RowDesc* rows, int32_t* tokens,
                       int32_t* kept_ids, double* kept_pr, int32_t* kept_n, uint32_t* status, void* stream) {
    merge_lists_kernel<<<n_rows, kThreads, kSmemMerge, static_cast<cudaStream_t>(stream)>>>(static_cast<const u64*>(lists), list_n, n_lists, list_stride,
                                                                                           n_rows, rows, tokens, kept_ids, kept_pr, kept_n, status);
    return (int)cudaGetLastError();
}

int launch_gather_patched(const float* logits, const RowDesc* rows, int n_rows, const int32_t* hist, int n_vocab, int vocab_offset, float* out,
                          void* stream) {
    gather_patched_kernel<<<n_rows, 128, 0, static_cast<cudaStream_t>(stream)>>>(logits, rows, n_rows, hist, n_vocab, vocab_offset, out);
    return (int)cudaGetLastError();
}

int launch_append_tokens(const RowDesc* rows, int n_rows, const int32_t* tokens, int32_t* pool, void* stream) {
    append_tokens_kernel<<<(n_rows + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(rows, n_rows, tokens, pool);
    return (int)cudaGetLastError();
}

int launch_write_drafts(const RowDesc* rows, int n_rows, int32_t* pool, void* stream) {
    write_drafts_kernel<<<(n_rows + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(rows, n_rows, pool);
    return (int)cudaGetLastError();
}

int launch_accept_windows(const int32_t* table, int n_streams, const int32_t* tokens, int32_t* pool, void* stream) {
    accept_windows_kernel<<<(n_streams + 63) / 64, 64, 0, static_cast<cudaStream_t>(stream)>>>(table, n_streams, tokens, pool);
    return (int)cudaGetLastError();
}

}  // namespace fsb
