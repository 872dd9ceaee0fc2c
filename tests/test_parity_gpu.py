"""GPU parity tests: the CUDA library, called through its C ABI, against the CPU oracle on the same inputs.

Bar: token ids bit-exact at temperature 0; stochastic draws identical except where the uniform lands within 1e-6
of a boundary of the cumulative distribution (counted and bounded); kept-set probabilities within 1e-6 absolute.
"""
import numpy as np
import pytest

import ferro_b200 as fb
from ferro_b200 import synth
from helpers import CDF_TOL, PROB_TOL, compare_with_oracle, golden_case_inputs, load_golden, random_case

pytestmark = pytest.mark.gpu


def run_batch(engine, oracle, lg, p, hists, check_kept=True, flags=0, logits_for_engine=None):
    ref = oracle.sample_rows(p, oracle.new_rngs(p["seed"]), lg.copy(), hists, cap=lg.shape[1] if lg.shape[1] <= 70001 else fb.MAX_CANDIDATE_K)
    sids = engine.open_streams(p)
    try:
        x = lg.copy() if logits_for_engine is None else logits_for_engine
        tok = engine.sample_batch(sids, x, hists, n_vocab=lg.shape[1], flags=flags | (fb.KEEP_KEPT_SET if check_kept else 0))
        hard, near, kept_bad = compare_with_oracle(engine, tok, ref, p, lg.shape[1], check_kept)
    finally:
        for s in sids:
            engine.close_stream(int(s))
    return tok, ref, hard, near, kept_bad


def test_reference_known_answer_vector_through_the_sampler_class(engine):
    # the reference's own sampler test (tests/test_kernels.cpp:348-359), written against the same class shape
    def pick(last_n, frm):
        p = fb.make_params(1, temperature=0.0, repetition_penalty=2.0, repeat_last_n=last_n, penalty_from=frm)
        s = fb.Sampler(p, engine)
        lg = np.array([0.0, 9.0, 10.0, 9.5, 6.0, 0.0], dtype=np.float32)
        t = s.sample(lg, len(lg), [1, 2, 3])      # prompt {1, 2}, generated {3}
        s.close()
        return t
    assert [pick(-1, 0), pick(-1, 2), pick(2, 0), pick(0, 0), pick(2, 2)] == [4, 2, 1, 2, 2]


@pytest.mark.parametrize("idx", range(5))
def test_golden_vectors_of_the_reference(engine, idx):
    case = load_golden()["cases"][idx]
    lg, p, hists = golden_case_inputs(case)
    sids = engine.open_streams(p)
    got = [[] for _ in range(case["rows"])]
    for _ in range(case["n_draws"]):
        tok = engine.sample_batch(sids, lg.copy(), hists)
        for r in range(case["rows"]):
            got[r].append(int(tok[r]))
    for s in sids:
        engine.close_stream(int(s))
    assert got == case["tokens"], case["name"]


@pytest.mark.parametrize("shape", [(1, 1), (1, 6), (3, 33), (4, 1000), (2, 4096), (5, 4097), (8, 65536), (3, 70001), (2, 262144), (64, 8192), (300, 5000)])
def test_random_batches_candidate_kernel(engine, oracle, shape):
    B, V = shape
    rng = np.random.default_rng(1000 + B * 7 + V)
    near_total = 0
    for trial in range(6):
        lg, p, hists = random_case(rng, B, V, trial, allow_full=False)
        _, _, hard, near, kept_bad = run_batch(engine, oracle, lg, p, hists)
        assert not hard, (shape, trial, hard[:3])
        assert not kept_bad, (shape, trial, kept_bad[:3])
        near_total += near
    assert near_total <= 1


@pytest.mark.parametrize("shape", [(2, 6), (3, 33), (4, 1000), (2, 4097), (4, 65536), (2, 70001), (2, 262144)])
def test_random_batches_with_full_vocabulary_rows(engine, oracle, shape):
    B, V = shape
    rng = np.random.default_rng(2000 + B * 7 + V)
    for trial in range(6):
        lg, p, hists = random_case(rng, B, V, trial, allow_full=True)
        _, _, hard, near, kept_bad = run_batch(engine, oracle, lg, p, hists)
        assert not hard, (shape, trial, hard[:3])
        assert not kept_bad, (shape, trial, kept_bad[:3])
        assert near <= 1


def test_full_vocabulary_rows_too_long_for_shared_memory(oracle):
    """Rows of more than 8 x 32768 logits: a CTA's slice no longer fits its shared memory, so the passes of the
    full-vocabulary kernel read the row from global memory and transform it again each time."""
    B, V = 3, 300001
    eng = fb.Engine(device=0, max_rows=B, max_vocab=V, max_hist_ids=B * 2100 + 16)
    try:
        rng = np.random.default_rng(8128)
        # the same engine must also take shorter rows, whose slices do fit (and need more shared memory than the long ones)
        for v2 in (262144, 5000):
            lg, p, hists = random_case(rng, B, v2, 1, allow_full=True)
            p["top_k"][0] = 0
            p["temperature"][0] = 1.0
            _, _, hard, near, kept_bad = run_batch(eng, oracle, lg, p, hists)
            assert not hard and not kept_bad and near <= 1, (v2, hard[:3], kept_bad[:3])
        for trial in range(3):
            lg, p, hists = random_case(rng, B, V, trial, allow_full=True)
            p["top_k"][0] = 0                                   # at least one row takes the full-vocabulary kernel
            p["temperature"][0] = max(float(p["temperature"][0]), 0.5)
            _, _, hard, near, kept_bad = run_batch(eng, oracle, lg, p, hists)
            assert not hard and not kept_bad and near <= 1, (trial, hard[:3], kept_bad[:3])
    finally:
        eng.close()


def test_many_rows_dealt_as_equal_runs_of_tiles(engine, oracle):
    """300 rows of 262144 logits on 148 SMs would be three waves of whole-row CTAs; the planner deals the 9600 tiles
    in equal runs instead, so a CTA works through two rows and a bit, and most rows straddle two CTAs."""
    B, V = 300, 262144
    rng = np.random.default_rng(300)
    lg = (rng.standard_normal((B, V), dtype=np.float32) * 3).astype(np.float32)
    lg[:, ::9] = np.round(lg[:, ::9])
    p = fb.make_params(B, temperature=0.8, top_k=40, top_p=0.9, min_p=0.01, repetition_penalty=1.1)
    p["temperature"][::5] = 0.0
    p["top_k"][1::7] = 200
    p["seed"] = 3000 + np.arange(B)
    hists = [rng.integers(0, V, size=300).astype(np.int32) for _ in range(B)]
    _, _, hard, near, kept_bad = run_batch(engine, oracle, lg, p, hists)
    assert not hard and not kept_bad and near <= 1, (hard[:3], near, kept_bad[:3])


def test_unaligned_rows_take_the_plain_load_path(engine, oracle):
    import torch
    rng = np.random.default_rng(7)
    B, V = 5, 4099
    lg, p, hists = random_case(rng, B, V, 1, allow_full=True)
    wide = np.zeros((B, V + 1), dtype=np.float32)          # row stride V + 1: rows are not on 16-byte boundaries
    wide[:, :V] = lg
    dev = torch.from_numpy(wide).cuda()[:, :V]
    _, _, hard, near, kept_bad = run_batch(engine, oracle, lg, p, hists, logits_for_engine=dev)
    assert not hard and not kept_bad and near <= 1


def test_write_back_reproduces_the_in_place_penalty(engine, oracle):
    import torch
    rng = np.random.default_rng(9)
    B, V = 6, 9000
    lg, p, hists = random_case(rng, B, V, 2, allow_full=True)
    p["repetition_penalty"] = 1.25
    p["repeat_last_n"] = -1
    p["penalty_from"] = 0
    want = lg.copy()
    oracle.sample_rows(p, oracle.new_rngs(p["seed"]), want, hists)
    for where in ("device", "host"):
        sids = engine.open_streams(p)
        x = torch.from_numpy(lg.copy()).cuda() if where == "device" else lg.copy()
        engine.sample_batch(sids, x, hists, flags=fb.WRITE_BACK)
        got = x.cpu().numpy() if where == "device" else x
        for s in sids:
            engine.close_stream(int(s))
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), where


def test_results_are_bit_identical_from_run_to_run(engine):
    rng = np.random.default_rng(11)
    lg, p, hists = random_case(rng, 32, 65536, 1, allow_full=False)
    outs = []
    for _ in range(3):
        sids = engine.open_streams(p)
        outs.append(engine.sample_batch(sids, lg.copy(), hists, flags=fb.KEEP_KEPT_SET).copy())
        kept = [engine.last_kept(i) for i in range(4)]
        outs.append(np.concatenate([k[1] for k in kept]).view(np.uint64).copy())
        for s in sids:
            engine.close_stream(int(s))
    assert np.array_equal(outs[0], outs[2]) and np.array_equal(outs[2], outs[4])
    assert np.array_equal(outs[1], outs[3]) and np.array_equal(outs[3], outs[5])


def test_stream_state_and_draw_accounting(engine, oracle):
    rng = np.random.default_rng(13)
    V = 3000
    lg = (rng.standard_normal((1, V)) * 3).astype(np.float32)
    p = fb.make_params(1, temperature=0.9, top_k=30, repetition_penalty=1.0, seed=4242)
    sid = engine.open_stream(p)
    toks = [int(engine.sample_batch([sid], lg.copy(), [[]])[0]) for _ in range(7)]
    seed, draws = engine.stream_state(sid)
    assert (seed, draws) == (4242, 7)            # one engine output per stochastic call
    engine.set_stream_state(sid, 4242, 3)        # rewind: the same draws come again
    again = [int(engine.sample_batch([sid], lg.copy(), [[]])[0]) for _ in range(4)]
    assert again == toks[3:]
    g = fb.make_params(1, temperature=0.0, seed=5)
    gs = engine.open_stream(g)
    engine.sample_batch([gs], lg.copy(), [[]])
    assert engine.stream_state(gs)[1] == 0        # greedy calls consume nothing
    orng = oracle.new_rngs([4242])
    want = [int(oracle.sample_rows(p, orng, lg.copy(), [[]])["tokens"][0]) for _ in range(7)]
    assert toks == want
    engine.close_stream(sid)
    engine.close_stream(gs)


def test_errors_are_reported_not_fatal(engine):
    lg = np.zeros((2, 100), dtype=np.float32)
    p = fb.make_params(1, temperature=0.0)
    sid = engine.open_stream(p)
    with pytest.raises(fb.SamplerError) as e:
        engine.sample_batch([sid, 9999], lg, [[], []])
    assert e.value.code == -5
    with pytest.raises(fb.SamplerError) as e:
        engine.sample_batch([sid] * 600, np.zeros((600, 100), dtype=np.float32), [[]] * 600)
    assert e.value.code == -3
    bad = fb.make_params(1, top_p=0.0)
    with pytest.raises(fb.SamplerError) as e:
        engine.open_stream(bad)
    assert e.value.code == -2
    assert int(engine.sample_batch([sid], lg[:1], [[]])[0]) == 0     # the engine still works; all-equal row: lowest id
    engine.close_stream(sid)


@pytest.mark.parametrize("shape", [(24, 65536), (8, 262144), (40, 20000)])
def test_overlapping_launches_give_the_same_tokens(engine, oracle, shape):
    """Launch overlap (programmatic stream serialization) changes when a launch may start, never what it writes:
    a train of launches over rotating device buffers ends with the tokens of the oracle, and with the tokens the
    same train gives without overlap.  (24, 65536) and (40, 20000) split rows over several CTAs, so the rows'
    scratch counters are reused from launch to launch."""
    import torch
    B, V = shape
    rng = np.random.default_rng(101)
    lgs = [(rng.standard_normal((B, V)) * 3).astype(np.float32) for _ in range(3)]
    devs = [torch.from_numpy(x).cuda() for x in lgs]
    p = fb.make_params(B, temperature=0.9, top_k=50, top_p=0.9, repetition_penalty=1.2)
    p["temperature"][::5] = 0.0
    p["seed"] = 1000 + np.arange(B)
    hists = [rng.integers(0, V, size=100).astype(np.int32) for _ in range(B)]
    ref = oracle.sample_rows(p, oracle.new_rngs(p["seed"]), lgs[10 % 3].copy(), hists, cap=fb.MAX_CANDIDATE_K)
    outs = []
    for overlap in (False, True):
        sids = engine.open_streams(p)
        engine.set_launch_overlap(overlap)
        try:
            batch = engine.prepare_batch(sids, hists, V)
            for i in range(11):
                batch.launch(devs[i % 3].data_ptr())
            outs.append(batch.tokens().copy())
            batch.free()
        finally:
            engine.set_launch_overlap(False)
            for s in sids:
                engine.close_stream(int(s))
    assert np.array_equal(outs[0], outs[1])
    assert np.array_equal(outs[1], ref["tokens"])


@pytest.mark.parametrize("case", [(2, 262144, 40), (1, 200000, 1), (3, 150001, 64)])
def test_rows_cut_into_many_short_segments(engine, oracle, case):
    """Small batches of long rows, where the planner cuts a row into pieces: (2, 262144) eight pieces per row that run
    as a cluster and exchange candidates on chip; (1, 200000) five pieces whose ordered lists meet in the row's scratch
    behind a ticket; (3, 150001) a prime number of tiles, one CTA per row.  (Rows of more than 16 pieces, which are
    merged by gathering and re-ordering, only arise in the static-scratch entry point: tests/test_zz_no_alloc.py.)"""
    B, V, k = case
    rng = np.random.default_rng(4242 + V)
    lg = (rng.standard_normal((B, V)) * 3).astype(np.float32)
    lg[:, ::11] = np.round(lg[:, ::11])
    p = fb.make_params(B, temperature=0.0 if k == 1 else 0.9, top_k=k, top_p=0.95, repetition_penalty=1.2)
    p["seed"] = 77 + np.arange(B)
    hists = [rng.integers(0, V, size=300).astype(np.int32) for _ in range(B)]
    tok, ref, hard, near, kept_bad = run_batch(engine, oracle, lg, p, hists)
    assert not hard and not kept_bad, (hard, near, kept_bad)
