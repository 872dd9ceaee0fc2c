"""Vocabulary sharding on one GPU: G engines stand in for G ranks (same streams, same seeds, different column
offsets); their candidate lists are stacked as an all-gather would leave them and merged.  The tokens must be those
of the oracle and of the unsharded launch."""
import numpy as np
import pytest

import ferro_b200 as fb
from ferro_b200 import sharded

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(16, 262144, 4), (9, 70001, 3), (4, 65536, 8)])
def test_sharded_candidates_merge_to_the_unsharded_result(engine, oracle, shape):
    import torch
    B, V, G = shape
    rng = np.random.default_rng(31 + G)
    lg = (rng.standard_normal((B, V)) * 3).astype(np.float32)
    lg[:, ::7] = np.round(lg[:, ::7])                      # ties that straddle shard boundaries
    p = fb.make_params(B, temperature=0.8, top_k=40, top_p=0.9, min_p=0.02, repetition_penalty=1.3)
    p["temperature"][::4] = 0.0
    p["top_k"][1::3] = 256
    p["seed"] = 500 + np.arange(B)
    hists = [rng.integers(0, V, size=200).astype(np.int32) for _ in range(B)]
    ref = oracle.sample_rows(p, oracle.new_rngs(p["seed"]), lg.copy(), hists, cap=fb.MAX_CANDIDATE_K)
    dev = torch.from_numpy(lg).cuda()
    parts = sharded.vocab_partition(V, G)
    lists = torch.zeros((G, B, sharded.MAX_K), dtype=torch.int64, device="cuda")
    counts = torch.zeros((G, B), dtype=torch.int32, device="cuda")
    engines, batches = [], []
    try:
        for g, (lo, hi) in enumerate(parts):
            eng = fb.Engine(device=0, max_rows=B, max_vocab=hi - lo, max_hist_ids=B * 200 + 16)
            engines.append(eng)
            eng.set_vocab_offset(lo)
            sids = eng.open_streams(p)
            b = eng.prepare_batch(sids, hists, hi - lo, ld=V, flags=fb.KEEP_KEPT_SET)
            batches.append(b)
            b.shard_launch(dev.data_ptr() + 4 * lo, lists[g].data_ptr(), counts[g].data_ptr())
        torch.cuda.synchronize()
        batches[0].merge_launch(lists.data_ptr(), counts.data_ptr(), G)
        tok = batches[0].tokens()
        assert np.array_equal(tok, ref["tokens"])
        for i in range(B):
            if p["temperature"][i] > 0:
                ids, pr, n = engines[0].last_kept(i)
                assert n == ref["n_keep"][i] and np.array_equal(ids, ref["kept_ids"][i, :n])
                assert np.abs(pr - ref["kept_pr"][i, :n]).max() <= 1e-6
    finally:
        for b in batches:
            b.free()
        for eng in engines:
            eng.close()
    # the unsharded launch on the same inputs
    sids = engine.open_streams(p)
    try:
        assert np.array_equal(engine.sample_batch(sids, lg.copy(), hists), tok)
    finally:
        for s in sids:
            engine.close_stream(int(s))


@pytest.mark.parametrize("shape", [(16, 262144, 8, 40), (9, 70001, 3, 64), (5, 1000, 8, 200), (7, 4096, 2, 256)])
def test_packed_lists_merged_block_by_block_match_the_oracle(oracle, shape):
    """The all-to-all route on one GPU: G engines write packed lists; "rank" q merges only its block of rows from
    the G lists of that block.  (5, 1000, 8, 200): top_k exceeds a shard's 125 columns, so a shard's list is its
    whole slice and the merged row still keeps the row-wide 200."""
    import torch
    B, V, G, k = shape
    rng = np.random.default_rng(77 + G)
    lg = (rng.standard_normal((B, V)) * 3).astype(np.float32)
    lg[:, ::5] = np.round(lg[:, ::5])
    p = fb.make_params(B, temperature=0.9, top_k=k, top_p=0.95, min_p=0.01, repetition_penalty=1.2)
    p["temperature"][::3] = 0.0
    p["seed"] = 800 + np.arange(B)
    hists = [rng.integers(0, V, size=100).astype(np.int32) for _ in range(B)]
    ref = oracle.sample_rows(p, oracle.new_rngs(p["seed"]), lg.copy(), hists, cap=fb.MAX_CANDIDATE_K)
    dev = torch.from_numpy(lg).cuda()
    parts = sharded.vocab_partition(V, G)
    engines, batches = [], []
    try:
        for g, (lo, hi) in enumerate(parts):
            eng = fb.Engine(device=0, max_rows=B, max_vocab=max(hi - lo, 1), max_hist_ids=B * 100 + 16)
            engines.append(eng)
            eng.set_vocab_shard(lo, V)
            batches.append(eng.prepare_batch(eng.open_streams(p), hists, hi - lo, ld=V, flags=fb.KEEP_KEPT_SET))
        stride = max(b.max_k for b in batches) + 1
        assert stride == min(k, max(hi - lo for lo, hi in parts)) + 1
        packed = torch.zeros((G, B, stride), dtype=torch.int64, device="cuda")
        for g, (lo, hi) in enumerate(parts):
            batches[g].shard_launch_packed(dev.data_ptr() + 4 * lo, packed[g].data_ptr(), stride)
        torch.cuda.synchronize()
        counts = packed[:, :, 0].cpu().numpy()
        assert (counts == np.array([[min(k if p["temperature"][r] > 0 else 1, hi - lo) for r in range(B)] for lo, hi in parts])).all()
        tok = np.zeros(B, dtype=np.int32)
        for q, (r0, r1) in enumerate(sharded.row_partition(B, G)):
            lists = packed[:, r0:r1, :].contiguous()
            batches[q].merge_launch_packed(lists.data_ptr(), stride, G, r0, r1 - r0)
            batches[q].check()
            mine = torch.as_tensor(sharded._DeviceInts(batches[q].tokens_device_ptr, B), device="cuda")
            tok[r0:r1] = mine[r0:r1].cpu().numpy()
        assert np.array_equal(tok, ref["tokens"])
        # all rows on one rank (the all-gather route), with the kept sets
        batches[0].merge_launch_packed(packed.data_ptr(), stride, G, 0, B)
        assert np.array_equal(batches[0].tokens(), ref["tokens"])
        for i in range(B):
            if p["temperature"][i] > 0:
                ids, pr, n = engines[0].last_kept(i)
                assert n == ref["n_keep"][i] and np.array_equal(ids, ref["kept_ids"][i, :n])
                assert np.abs(pr - ref["kept_pr"][i, :n]).max() <= 1e-6
        with pytest.raises(fb.SamplerError):                       # a list cannot be shorter than the batch's largest k + 1
            batches[0].shard_launch_packed(dev.data_ptr(), packed[0].data_ptr(), stride - 1)
    finally:
        for b in batches:
            b.free()
        for eng in engines:
            eng.close()


def test_full_vocabulary_rows_are_refused_by_the_sharded_launch(engine):
    import torch
    p = fb.make_params(2, temperature=1.0, top_k=0)
    p["seed"] = [3, 4]
    sids = engine.open_streams(p)
    try:
        b = engine.prepare_batch(sids, [np.zeros(0, np.int32)] * 2, 4096)
        lists = torch.zeros((2, sharded.MAX_K), dtype=torch.int64, device="cuda")
        counts = torch.zeros(2, dtype=torch.int32, device="cuda")
        with pytest.raises(fb.SamplerError):
            b.shard_launch(torch.zeros(2, 4096, device="cuda").data_ptr(), lists.data_ptr(), counts.data_ptr())
        b.free()
    finally:
        for s in sids:
            engine.close_stream(int(s))


def _nccl_rank(rank, world, port, B, V, out_dir):
    import os
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        rng = np.random.default_rng(77)
        lg = (rng.standard_normal((B, V)) * 3).astype(np.float32)
        p = fb.make_params(B, temperature=0.9, top_k=50, top_p=0.95, repetition_penalty=1.1)
        p["temperature"][::3] = 0.0
        p["seed"] = 900 + np.arange(B)
        hists = [rng.integers(0, V, size=64).astype(np.int32) for _ in range(B)]
        eng = fb.Engine(device=rank, max_rows=B, max_vocab=V, max_hist_ids=B * 64 + 16)
        vs = sharded.VocabShardedSampler(eng, V, rank, world)
        lo, hi = vs.columns
        shard = torch.from_numpy(np.ascontiguousarray(lg[:, lo:hi])).cuda()
        sids = eng.open_streams(p)
        tok = vs.sample(sids, shard, hists)
        np.save(os.path.join(out_dir, f"tok{rank}.npy"), tok)
        eng.close()
    finally:
        dist.destroy_process_group()


def test_two_gpus_vocabulary_sharded_over_nccl(oracle, tmp_path):
    import socket
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    B, V, world = 32, 262144, 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_nccl_rank, args=(world, port, B, V, str(tmp_path)), nprocs=world, join=True)
    rng = np.random.default_rng(77)
    lg = (rng.standard_normal((B, V)) * 3).astype(np.float32)
    p = fb.make_params(B, temperature=0.9, top_k=50, top_p=0.95, repetition_penalty=1.1)
    p["temperature"][::3] = 0.0
    p["seed"] = 900 + np.arange(B)
    hists = [rng.integers(0, V, size=64).astype(np.int32) for _ in range(B)]
    ref = oracle.sample_rows(p, oracle.new_rngs(p["seed"]), lg, hists)
    t0, t1 = np.load(tmp_path / "tok0.npy"), np.load(tmp_path / "tok1.npy")
    assert np.array_equal(t0, t1) and np.array_equal(t0, ref["tokens"])
