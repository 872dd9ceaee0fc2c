"""Device-resident histories: a decode loop that moves one token per stream and step must produce the tokens of the
reference loop, which hands the whole growing history to every call (src/server.cpp:603-608 with gen_token's
push_back at :342)."""
import numpy as np
import pytest

import ferro_b200 as fb

pytestmark = pytest.mark.gpu


def test_decode_loop_with_resident_histories_matches_the_reference_loop(engine, oracle):
    import torch
    B, V, steps = 8, 65536, 40
    rng = np.random.default_rng(314)
    p = fb.make_params(B, temperature=0.8, top_k=40, top_p=0.95, repetition_penalty=1.3, repeat_last_n=-1)
    p["temperature"][:2] = 0.0
    p["repeat_last_n"][2:4] = 16                      # a sliding window
    p["penalty_from"][4:6] = 250                      # prompt tokens are never penalised
    p["seed"] = 4000 + np.arange(B)
    prompts = [rng.integers(0, V, size=int(n)).astype(np.int32) for n in rng.integers(200, 300, size=B)]   # crosses 256: regions grow
    sids = engine.open_streams(p)
    rngs = oracle.new_rngs(p["seed"])
    hists = [x.copy() for x in prompts]
    try:
        for i, s in enumerate(sids):
            engine.history_set(int(s), prompts[i])
        for step in range(steps):
            lg = (rng.standard_normal((B, V)) * 3).astype(np.float32)
            ref = oracle.sample_rows(p, rngs, lg.copy(), hists)          # advances rngs
            if step % 2 == 0:
                tok = engine.sample_batch_resident(sids, lg.copy(), flags=fb.APPEND_SAMPLED)
            else:                                                          # device logits, host-side append
                dev = torch.from_numpy(lg).cuda()
                tok = engine.sample_batch_resident(sids, dev.data_ptr(), n_vocab=V)
                for i, s in enumerate(sids):
                    engine.history_append(int(s), tok[i])
            assert np.array_equal(tok, ref["tokens"]), step
            hists = [np.append(hh, t).astype(np.int32) for hh, t in zip(hists, ref["tokens"])]
        assert [engine.history_len(int(s)) for s in sids] == [len(x) for x in hists]
    finally:
        for s in sids:
            engine.close_stream(int(s))


def test_resident_history_errors_and_region_reuse(engine):
    p = fb.make_params(2, temperature=0.0, repetition_penalty=1.1)
    p["seed"] = [1, 2]
    sids = engine.open_streams(p)
    lg = np.zeros((2, 4096), dtype=np.float32)
    lg[:, 7], lg[:, 9] = 1.0, 0.95
    try:
        with pytest.raises(fb.SamplerError):                               # a stream twice in one call
            engine.sample_batch_resident([sids[0], sids[0]], lg)
        engine.history_set(int(sids[0]), np.arange(1000, 2000, dtype=np.int32))
        engine.history_set(int(sids[0]), np.array([7], dtype=np.int32))   # replaced: only token 7 is penalised now
        engine.history_set(int(sids[1]), np.zeros(0, dtype=np.int32))
        assert engine.history_len(int(sids[0])) == 1 and engine.history_len(int(sids[1])) == 0
        tok = engine.sample_batch_resident(sids, lg.copy())
        assert tok.tolist() == [9, 7]                                      # 1.0 / 1.1 < 0.95 in row 0; row 1 has no history
        engine.history_append(int(sids[1]), [7, 9])
        assert engine.sample_batch_resident(sids, lg.copy()).tolist() == [9, 7]   # row 1: 0.909 vs 0.864
    finally:
        for s in sids:
            engine.close_stream(int(s))
    with pytest.raises(fb.SamplerError):
        engine.history_len(int(sids[0]))                                   # closed
