"""Multi-GPU use of the sampler: one process per GPU, ``torch.distributed`` for the plumbing.

Row sharding is the primary mode: rows are independent streams (the reference's decode loop,
src/server.cpp:603-608, is a loop over slots), so rank g samples a contiguous block of rows with no data-path
collective at all; ``row_partition`` gives the blocks and ``gather_tokens`` an optional all-gather of the ids.

Vocabulary sharding is for a logits matrix that is split by columns (a tensor-parallel LM head leaves columns
[g V/G, (g+1) V/G) of every row on GPU g): every rank selects the best k candidates of its columns, one all-gather
brings the G lists of every row into local memory (B x k x 8 bytes per rank: 164 KB at B = 512, k = 40), and the
merge kernel finishes the rows.  The global top-k is a subset of the union of the shards' top-k lists and the
(value descending, id ascending) order does not depend on the split, so the result is the unsharded one.  Rows with
top_k = 0 (the whole vocabulary is the candidate set) cannot be done this way: shard those by rows.

Nothing here touches another GPU's memory directly: the exchange is a NCCL (or, in CPU tests, gloo) all-gather
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


def gather_tokens(tokens, group=None):
    """Row sharding: every rank's token ids, concatenated in rank order (ranks may hold different numbers of rows)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    parts = [None] * world
    dist.all_gather_object(parts, np.asarray(tokens, dtype=np.int32), group=group)
    return np.concatenate(parts)


class VocabShardedSampler:
    """One rank of a vocabulary-sharded sampler.  Every rank opens the same streams (same parameters and seeds), so
    all ranks draw the same engine outputs; after `sample` every rank holds all tokens."""

    def __init__(self, engine, n_vocab: int, rank: int, world: int, group=None):
        self.engine, self.rank, self.world, self.group = engine, rank, world, group
        self.lo, self.hi = vocab_partition(n_vocab, world)[rank]
        engine.set_vocab_shard(self.lo, n_vocab)

    @property
    def columns(self) -> tuple[int, int]:
        return self.lo, self.hi

    def sample(self, stream_ids, logits_shard, histories):
        """logits_shard: CUDA float32 tensor [rows][hi - lo] (this rank's columns).  Returns the token ids."""
        import torch
        rows, width = logits_shard.shape
        if width != self.hi - self.lo:
            raise ValueError(f"this rank holds columns {self.lo}..{self.hi}, got {width}")
        self.engine.set_cuda_stream(torch.cuda.current_stream().cuda_stream)
        batch = self.engine.prepare_batch(stream_ids, histories, width, ld=logits_shard.stride(0))
        try:
            lists = torch.zeros((rows, MAX_K), dtype=torch.int64, device=logits_shard.device)
            counts = torch.zeros((rows,), dtype=torch.int32, device=logits_shard.device)
            batch.shard_launch(logits_shard.data_ptr(), lists.data_ptr(), counts.data_ptr())
            all_lists, all_counts = gather_candidate_lists(lists, counts, self.group)
            batch.merge_launch(all_lists.data_ptr(), all_counts.data_ptr(), self.world)
            return batch.tokens()
        finally:
            batch.free()
