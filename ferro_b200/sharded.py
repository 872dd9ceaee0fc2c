"""Multi-GPU use of the sampler: one process per GPU, ``torch.distributed`` for the plumbing.

Row sharding is the primary mode: rows are independent streams (the reference's decode loop,
src/server.cpp:603-608, is a loop over slots), so rank g samples a contiguous block of rows with no data-path
collective at all; ``row_partition`` gives the blocks and ``gather_tokens`` an optional all-gather of the ids.

Vocabulary sharding is for a logits matrix that is split by columns (a tensor-parallel LM head leaves columns
[g V/G, (g+1) V/G) of every row on GPU g).  Every rank selects the best k candidates of its columns and writes
them as packed lists - per row one count word and k candidates, (k + 1) x 8 bytes, 168 KB for 512 rows at k = 40.
Then either one all-to-all hands every rank the G lists of its own block of rows (row_partition), the merge
kernel finishes that block, and one all-gather of 4 bytes per row leaves all tokens on all ranks; or
(``exchange="all_gather"``) all lists are gathered everywhere and every rank merges every row - one collective instead
of two, G times the bytes and G times the merge work, the faster route up to four ranks and the default there.  The global top-k is a subset of the union of the shards'
top-k lists and the (value descending, id ascending) order does not depend on the split, so the result is the
unsharded one.  Rows with top_k = 0 (the whole vocabulary is the candidate set) cannot be done this way: shard
those by rows.

Nothing here touches another GPU's memory directly: the exchanges are NCCL (or, in CPU tests, gloo) collectives
into local buffers.
"""
from __future__ import annotations

import numpy as np

MAX_K = 256   # FSB_MAX_CANDIDATE_K: entries per candidate list


def row_partition(n_rows: int, world: int) -> list[tuple[int, int]]:
    """Contiguous row blocks [lo, hi) per rank; the first n_rows % world ranks get one row more."""
    if world < 1 or n_rows < 0:
        raise ValueError("world >= 1 and n_rows >= 0")
    base, extra = divmod(n_rows, world)
    out, lo = [], 0
    for g in range(world):
        hi = lo + base + (1 if g < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out


def vocab_partition(n_vocab: int, world: int, align: int = 4) -> list[tuple[int, int]]:
    """Column ranges [lo, hi) per rank, boundaries on multiples of `align` columns (16 bytes of fp32: shards stay on
    the bulk-copy path).  Later ranks may get an empty range when the vocabulary is tiny."""
    if world < 1 or n_vocab < 1 or align < 1:
        raise ValueError("world >= 1, n_vocab >= 1, align >= 1")
    per = -(-n_vocab // world)
    per = -(-per // align) * align
    return [(min(n_vocab, g * per), min(n_vocab, (g + 1) * per)) for g in range(world)]


def pack_candidates(values: np.ndarray, ids: np.ndarray) -> np.ndarray:
    """Host-side twin of the device's 64-bit candidate keys: larger key = earlier in the reference's order
    (value descending, id ascending; -0.0 ties with +0.0, src/sampler.cpp:31,34)."""
    u = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32).copy()
    u[u == np.uint32(0x80000000)] = 0
    neg = (u & np.uint32(0x80000000)) != 0
    key = np.where(neg, ~u, u | np.uint32(0x80000000)).astype(np.uint64)
    return (key << np.uint64(32)) | (np.uint64(0xFFFFFFFF) - np.asarray(ids, dtype=np.uint64))


def unpack_candidates(keys: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """(values float32, token ids int64) of candidate keys."""
    keys = np.asarray(keys, dtype=np.uint64)
    k = (keys >> np.uint64(32)).astype(np.uint32)
    u = np.where((k & np.uint32(0x80000000)) != 0, k & np.uint32(0x7FFFFFFF), ~k).astype(np.uint32)
    return u.view(np.float32), (np.uint64(0xFFFFFFFF) - (keys & np.uint64(0xFFFFFFFF))).astype(np.int64)


def gather_candidate_lists(lists, counts, group=None):
    """All-gather of every rank's [rows][MAX_K] int64 key lists and [rows] int32 counts into local
    [world][rows][MAX_K] and [world][rows] tensors (on the tensors' own device: NCCL for CUDA, gloo for CPU)."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    rows = lists.shape[0]
    flat_lists = torch.empty((world * rows,) + tuple(lists.shape[1:]), dtype=lists.dtype, device=lists.device)
    flat_counts = torch.empty((world * rows,), dtype=counts.dtype, device=counts.device)
    dist.all_gather_into_tensor(flat_lists, lists.contiguous(), group=group)     # rank-major: rank g's rows at g * rows
    dist.all_gather_into_tensor(flat_counts, counts.contiguous(), group=group)
    all_lists = flat_lists.view((world,) + tuple(lists.shape))
    all_counts = flat_counts.view(world, rows)
    return all_lists, all_counts


def exchange_packed_lists(packed, rank: int, world: int, mode: str = "all_to_all", group=None, out=None):
    """Brings the shards' packed candidate lists to where they are merged.  `packed` is this rank's [rows][stride]
    int64 tensor (CUDA for NCCL, CPU for gloo).  Returns (lists, row_begin, n_rows): `lists` is
    [world][n_rows][stride], the lists of rows [row_begin, row_begin + n_rows) from every rank in rank order - this
    rank's block of rows after an all-to-all, all rows after an all-gather.  `out`: a preallocated result."""
    import torch
    import torch.distributed as dist
    rows, stride = packed.shape
    if mode == "all_gather":
        if out is None:
            out = torch.empty((world * rows, stride), dtype=packed.dtype, device=packed.device)
        dist.all_gather_into_tensor(out.view(world * rows, stride), packed, group=group)
        return out.view(world, rows, stride), 0, rows
    if mode != "all_to_all":
        raise ValueError("mode is 'all_to_all' or 'all_gather'")
    blocks = row_partition(rows, world)
    lo, hi = blocks[rank]
    mine = hi - lo
    if out is None:
        out = torch.empty((world * mine, stride), dtype=packed.dtype, device=packed.device)
    dist.all_to_all_single(out.view(world * mine, stride), packed, output_split_sizes=[mine] * world,
                           input_split_sizes=[b - a for a, b in blocks], group=group)
    return out.view(world, mine, stride), lo, mine


def exchange_block_tokens(tokens, rank: int, world: int, group=None, pad=None, out=None):
    """After an all-to-all exchange every rank has finished its block of rows: `tokens` is the [rows] int32 tensor
    whose entries [row_partition(rows, world)[rank]] are valid.  One all-gather leaves all rows' tokens on every
    rank; returns the [rows] tensor.  Blocks are padded to the largest block (they differ by at most one row)."""
    import torch
    import torch.distributed as dist
    rows = tokens.shape[0]
    blocks = row_partition(rows, world)
    width = blocks[0][1] - blocks[0][0]
    lo, hi = blocks[rank]
    if out is None:
        out = torch.empty((world * width,), dtype=tokens.dtype, device=tokens.device)
    if hi - lo == width:
        src = tokens[lo:hi]
    else:
        src = pad if pad is not None else torch.zeros((width,), dtype=tokens.dtype, device=tokens.device)
        src[: hi - lo].copy_(tokens[lo:hi])
    dist.all_gather_into_tensor(out, src.contiguous(), group=group)
    if rows % world == 0:
        return out
    return torch.cat([out[g * width: g * width + (b - a)] for g, (a, b) in enumerate(blocks)])


def gather_tokens(tokens, group=None):
    """Row sharding: every rank's token ids, concatenated in rank order (ranks may hold different numbers of rows)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    parts = [None] * world
    dist.all_gather_object(parts, np.asarray(tokens, dtype=np.int32), group=group)
    return np.concatenate(parts)


class _DeviceInts:
    """A device array of int32 owned by the engine, as PyTorch's tensor constructor can take it."""

    def __init__(self, ptr: int, n: int):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<i4", "data": (int(ptr), False), "version": 2}


class VocabShardedSampler:
    """One rank of a vocabulary-sharded sampler.  Every rank opens the same streams (same parameters and seeds), so
    all ranks draw the same engine outputs; after a step every rank holds all tokens.

    ``prepare`` stages a batch once (streams, histories, buffers), ``step`` samples one matrix of logits with it -
    shard launch, exchange, merge, token exchange, all queued on the current CUDA stream - and ``tokens`` waits and
    returns the ids; ``sample`` does all three for one-off use."""

    def __init__(self, engine, n_vocab: int, rank: int, world: int, group=None, exchange: str = "auto"):
        if exchange == "auto":   # measured on B200: one all-gather is the faster route at two and four ranks
            exchange = "all_gather" if world <= 4 else "all_to_all"
        if exchange not in ("all_to_all", "all_gather"):
            raise ValueError("exchange is 'auto', 'all_to_all' or 'all_gather'")
        self.engine, self.rank, self.world, self.group, self.exchange = engine, rank, world, group, exchange
        self.n_vocab = n_vocab
        self.lo, self.hi = vocab_partition(n_vocab, world)[rank]
        engine.set_vocab_shard(self.lo, n_vocab)
        self.batch = None

    @property
    def columns(self) -> tuple[int, int]:
        return self.lo, self.hi

    def prepare(self, stream_ids, histories, rows: int, ld: int | None = None, device=None):
        """Stages `rows` rows (one per stream id) and allocates the exchange buffers."""
        import torch
        self.release()
        width = self.hi - self.lo
        self.engine.set_cuda_stream(torch.cuda.current_stream().cuda_stream)
        self.batch = self.engine.prepare_batch(stream_ids, histories, width, ld=width if ld is None else ld)
        self.rows, self.width, self._fresh = rows, width, True
        # every rank uses the same stride: the largest k any shard can see is the rows' k clamped by the widest shard
        self.stride = self.batch.max_k + 1
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        t = torch.tensor([self.stride], dtype=torch.int64, device=device)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        self.stride = int(t.item())
        self._packed = torch.zeros((rows, self.stride), dtype=torch.int64, device=device)
        lo, hi = row_partition(rows, self.world)[self.rank]
        n_recv = rows if self.exchange == "all_gather" else hi - lo
        self._lists = torch.zeros((self.world * n_recv, self.stride), dtype=torch.int64, device=device)
        self._tok = torch.as_tensor(_DeviceInts(self.batch.tokens_device_ptr, rows), device=device)
        width_b = -(-rows // self.world)
        self._tok_all = torch.zeros((self.world * width_b,), dtype=torch.int32, device=device)
        self._tok_pad = torch.zeros((width_b,), dtype=torch.int32, device=device)
        self._result = None

    def step(self, logits_shard):
        """One sampling step over this rank's columns of the logits ([rows][hi - lo], CUDA float32).  Asynchronous."""
        if self.batch is None:
            raise RuntimeError("prepare() first")
        if tuple(logits_shard.shape) != (self.rows, self.width):
            raise ValueError(f"this rank holds {self.rows} rows of columns {self.lo}..{self.hi}, got {tuple(logits_shard.shape)}")
        if not self._fresh:
            self.batch.redraw()                      # the next engine output of every stream
        self._fresh = False
        self.batch.shard_launch_packed(logits_shard.data_ptr(), self._packed.data_ptr(), self.stride)
        if self.world == 1:
            self.batch.merge_launch_packed(self._packed.data_ptr(), self.stride, 1, 0, self.rows)
            self._result = self._tok
            return
        lists, row_begin, n_rows = exchange_packed_lists(self._packed, self.rank, self.world, self.exchange, self.group, out=self._lists)
        self.batch.merge_launch_packed(lists.data_ptr(), self.stride, self.world, row_begin, n_rows)
        if self.exchange == "all_gather":
            self._result = self._tok
        else:
            self._result = exchange_block_tokens(self._tok, self.rank, self.world, self.group, pad=self._tok_pad, out=self._tok_all)

    def tokens(self) -> np.ndarray:
        """Waits for the last step; raises if the device reported an error; returns all rows' token ids."""
        self.batch.check()
        return self._result[: self.rows].cpu().numpy().astype(np.int32)

    def exchange_description(self) -> str:
        per_rank = self.rows * self.stride * 8
        if self.world == 1:
            return "single rank: no exchange"
        if self.exchange == "all_gather":
            return f"one all-gather of packed lists ({per_rank} bytes from each rank), every rank merges all {self.rows} rows"
        return (f"all-to-all of packed lists ({per_rank} bytes sent per rank, {self.stride} words per row), each rank merges its block of "
                f"{-(-self.rows // self.world)} rows, all-gather of the tokens ({4 * self.rows} bytes)")

    def release(self):
        if getattr(self, "batch", None) is not None:
            self.batch.free()
            self.batch = None

    def sample(self, stream_ids, logits_shard, histories):
        """logits_shard: CUDA float32 tensor [rows][hi - lo] (this rank's columns).  Returns the token ids."""
        rows, width = logits_shard.shape
        if width != self.hi - self.lo:
            raise ValueError(f"this rank holds columns {self.lo}..{self.hi}, got {width}")
        self.prepare(stream_ids, histories, rows, ld=logits_shard.stride(0), device=logits_shard.device)
        try:
            self.step(logits_shard)
            return self.tokens()
        finally:
            self.release()
