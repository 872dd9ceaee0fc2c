"""Host logic of the multi-GPU modes, on CPU: partitions, candidate keys, and the N > 1 exchange path run as two
gloo ranks.  The ranks stand in for GPUs: each takes the best k candidates of its columns with numpy (the job of the
streaming kernel), the lists travel through the package's own all-gather, and the merged result must be the
oracle's kept set for the whole row."""
import os
import socket

import numpy as np
import pytest

from ferro_b200 import sharded


def test_row_partition_covers_rows_in_order():
    for n, w in [(64, 8), (512, 8), (7, 3), (2, 4), (0, 2), (136, 1)]:
        parts = sharded.row_partition(n, w)
        assert len(parts) == w and parts[0][0] == 0 and parts[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(parts[:-1], parts[1:]))
        sizes = [hi - lo for lo, hi in parts]
        assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    with pytest.raises(ValueError):
        sharded.row_partition(4, 0)


def test_vocab_partition_is_aligned_and_covers_the_vocabulary():
    for v, w in [(262144, 8), (65536, 2), (70001, 3), (10, 4), (3, 2)]:
        parts = sharded.vocab_partition(v, w)
        assert parts[0][0] == 0 and max(hi for _, hi in parts) == v
        assert all(a[1] == b[0] or b[0] == b[1] == v for a, b in zip(parts[:-1], parts[1:]))
        assert all(lo % 4 == 0 for lo, hi in parts if hi > lo)


def test_candidate_keys_order_like_the_reference_comparator():
    vals = np.array([1.5, -2.0, 0.0, -0.0, np.inf, -np.inf, 1.5, 3e-39, -3e-39], dtype=np.float32)
    ids = np.arange(len(vals))
    keys = sharded.pack_candidates(vals, ids)
    order = np.argsort(keys)[::-1]                       # larger key first
    want = sorted(range(len(vals)), key=lambda i: (-float(vals[i]), i))   # value descending, id ascending; -0 == +0
    assert order.tolist() == want
    v2, i2 = sharded.unpack_candidates(keys)
    assert np.array_equal(i2, ids) and np.array_equal(v2 == vals, np.ones(len(vals), bool))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, B, V, k, out_dir):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(5)                   # the same matrix on every rank; each uses its own columns
        lg = (np.round(rng.standard_normal((B, V)) * 4) / 2).astype(np.float32)   # many ties across shards
        lo, hi = sharded.vocab_partition(V, world)[rank]
        # the bare lists with separate counts (all-gather of both) ...
        lists = np.zeros((B, sharded.MAX_K), dtype=np.uint64)
        counts = np.zeros(B, dtype=np.int32)
        # ... and the packed ones: [count, candidates ...] in k + 1 words per row
        packed = np.zeros((B, k + 1), dtype=np.uint64)
        for r in range(B):
            keys = np.sort(sharded.pack_candidates(lg[r, lo:hi], np.arange(lo, hi)))[::-1][:k]
            lists[r, : len(keys)], counts[r] = keys, len(keys)
            packed[r, 0], packed[r, 1: 1 + len(keys)] = len(keys), keys
        al, ac = sharded.gather_candidate_lists(torch.from_numpy(lists.view(np.int64)), torch.from_numpy(counts))
        al, ac = al.numpy().view(np.uint64), ac.numpy()
        assert al.shape == (world, B, sharded.MAX_K) and ac.shape == (world, B)
        merged = np.zeros((B, k), dtype=np.int64)
        for r in range(B):
            keys = np.concatenate([al[g, r, : ac[g, r]] for g in range(world)])
            merged[r] = sharded.unpack_candidates(np.sort(keys)[::-1][:k])[1]
        toks = sharded.gather_tokens(merged[sharded.row_partition(B, world)[rank][0]: sharded.row_partition(B, world)[rank][1], 0])
        np.save(os.path.join(out_dir, f"merged{rank}.npy"), merged)
        np.save(os.path.join(out_dir, f"tokens{rank}.npy"), toks)

        def merge(lists3, n_rows):   # what the merge kernel does with [world][n_rows][k + 1]
            out = np.zeros((n_rows, k), dtype=np.int64)
            for r in range(n_rows):
                keys = np.concatenate([lists3[g, r, 1: 1 + int(lists3[g, r, 0])] for g in range(world)])
                out[r] = sharded.unpack_candidates(np.sort(keys)[::-1][:k])[1]
            return out

        tp = torch.from_numpy(packed.view(np.int64))
        l3, b0, n = sharded.exchange_packed_lists(tp, rank, world, "all_gather")
        assert (b0, n) == (0, B) and np.array_equal(merge(l3.numpy().view(np.uint64), n), merged)
        l3, b0, n = sharded.exchange_packed_lists(tp, rank, world, "all_to_all")
        assert (b0, b0 + n) == sharded.row_partition(B, world)[rank] and tuple(l3.shape) == (world, n, k + 1)
        mine = merge(l3.numpy().view(np.uint64), n)
        assert np.array_equal(mine, merged[b0: b0 + n])
        tok = torch.zeros(B, dtype=torch.int32)
        tok[b0: b0 + n] = torch.from_numpy(mine[:, 0].astype(np.int32))
        np.save(os.path.join(out_dir, f"blocktokens{rank}.npy"), sharded.exchange_block_tokens(tok, rank, world).numpy())
    finally:
        dist.destroy_process_group()


def test_two_ranks_exchange_candidates_and_agree_with_the_oracle(oracle, tmp_path):
    import torch.multiprocessing as mp
    from oracle import make_params
    B, V, k, world = 7, 4099, 40, 2                                   # an odd number of rows: unequal blocks
    mp.spawn(_rank_main, args=(world, _free_port(), B, V, k, str(tmp_path)), nprocs=world, join=True)
    rng = np.random.default_rng(5)
    lg = (np.round(rng.standard_normal((B, V)) * 4) / 2).astype(np.float32)
    p = make_params(B, temperature=1.0, top_k=k, top_p=1.0, min_p=0.0, repetition_penalty=1.0)
    p["seed"] = 1 + np.arange(B)
    ref = oracle.sample_rows(p, oracle.new_rngs(p["seed"]), lg.copy(), [np.zeros(0, np.int32)] * B, cap=k)
    m0, m1 = np.load(tmp_path / "merged0.npy"), np.load(tmp_path / "merged1.npy")
    assert np.array_equal(m0, m1)                                     # every rank ends with the same candidates
    assert np.array_equal(m0, ref["kept_ids"][:, :k].astype(np.int64))  # and they are the reference's, in its order
    t0 = np.load(tmp_path / "tokens0.npy")
    assert np.array_equal(t0, np.load(tmp_path / "tokens1.npy")) and np.array_equal(t0, m0[:, 0].astype(np.int32))
    for r in range(world):                                             # the all-to-all route ends with the same tokens on every rank
        assert np.array_equal(np.load(tmp_path / f"blocktokens{r}.npy"), t0)
