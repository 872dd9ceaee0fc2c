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


def test_calls_with_explicit_histories_after_a_resident_call_use_their_own_histories(engine, oracle):
    """The engine's one internal batch serves every public call.  A resident call points it at the id pool; the next
    call that brings its histories along (fsb_sample_batch, fsb_verify_windows) must read those, not the pool."""
    B, V = 4, 8192
    rng = np.random.default_rng(2718)
    p = fb.make_params(B, temperature=0.7, top_k=30, top_p=0.9, repetition_penalty=1.5)
    p["seed"] = 60 + np.arange(B)
    sids = engine.open_streams(p)
    rngs = oracle.new_rngs(p["seed"])
    resident = [rng.integers(0, V, size=50).astype(np.int32) for _ in range(B)]
    try:
        for i, s in enumerate(sids):
            engine.history_set(int(s), resident[i])
        lg = (rng.standard_normal((B, V)) * 3).astype(np.float32)
        ref = oracle.sample_rows(p, rngs, lg.copy(), resident)
        assert np.array_equal(engine.sample_batch_resident(sids, lg.copy()), ref["tokens"])
        # explicit histories that penalise other ids than the resident ones
        other = [rng.integers(0, V, size=70).astype(np.int32) for _ in range(B)]
        lg = (rng.standard_normal((B, V)) * 3).astype(np.float32)
        for i in range(B):
            lg[i, other[i][:5]] += 9.0                     # the penalty decides among these
        ref = oracle.sample_rows(p, rngs, lg.copy(), other)
        assert np.array_equal(engine.sample_batch(sids, lg.copy(), other), ref["tokens"])
        # ... and the same for verification windows right after another resident call
        lg = (rng.standard_normal((B, V)) * 3).astype(np.float32)
        ref = oracle.sample_rows(p, rngs, lg.copy(), resident)
        assert np.array_equal(engine.sample_batch_resident(sids, lg.copy()), ref["tokens"])
        m = 4
        lgw = (rng.standard_normal((B * m, V)) * 3).astype(np.float32)
        rows = []
        for i in range(B):
            lgw[i * m:(i + 1) * m, other[i][:5]] += 9.0
            rows.append(np.concatenate([[int(other[i][-1])], rng.integers(0, V, size=m - 1)]).astype(np.int32))
        want = [oracle.verify_window(p[i:i + 1], rngs[i], lgw[i * m:(i + 1) * m].copy(), rows[i], other[i]) for i in range(B)]
        toks, acc, conf = engine.verify_windows(sids, rows, lgw.copy(), other)
        for i in range(B):
            t, a, c, _ = want[i]
            assert acc[i] == a and conf[i] == c and list(toks[i][:a]) == list(t[:a]), i
    finally:
        for s in sids:
            engine.close_stream(int(s))


@pytest.mark.parametrize("append", [False, True])
def test_resident_verification_windows_match_the_reference_accept_loop(engine, oracle, append):
    """Speculative steps on resident histories (src/server.cpp:598-645): only the drafts go up.  With APPEND_SAMPLED
    the accepted tokens join the history on the device, so the next step - resident as well - sees them."""
    import torch
    S, V, m, steps = 6, 32768, 5, 6
    rng = np.random.default_rng(1618)
    p = fb.make_params(S, temperature=0.8, top_k=40, top_p=0.95, repetition_penalty=1.4)
    p["temperature"][:3] = 0.0
    p["repeat_last_n"][1] = 8
    p["seed"] = 300 + np.arange(S)
    sids = engine.open_streams(p)
    rngs = oracle.new_rngs(p["seed"])
    hists = [rng.integers(0, V, size=int(n)).astype(np.int32) for n in rng.integers(20, 40, size=S)]
    try:
        for i, s in enumerate(sids):
            engine.history_set(int(s), hists[i])
        for step in range(steps):
            lg = (rng.standard_normal((S * m, V)) * 2).astype(np.float32)
            rows, want = [], []
            for i in range(S):
                drafts = rng.integers(0, V, size=m - 1).astype(np.int32)
                # make the first drafts right: what the oracle samples for rows 0 .. good-1 with the growing history
                good = int(rng.integers(0, m))
                h = list(hists[i])
                probe = rngs[i:i + 1].copy()                 # a copy of the stream's engine: the real one must not advance
                for r in range(good):
                    t = int(oracle.sample_rows(p[i:i + 1], probe, lg[i * m + r:i * m + r + 1].copy(), [np.array(h, dtype=np.int32)])["tokens"][0])
                    if r < m - 1:
                        drafts[r] = t
                    h.append(t)
                rows.append(np.concatenate([[int(hists[i][-1])], drafts]).astype(np.int32))
                want.append(oracle.verify_window(p[i:i + 1], rngs[i], lg[i * m:(i + 1) * m].copy(), rows[i], hists[i]))
            src = torch.from_numpy(lg).cuda() if step % 2 else lg.copy()
            toks, acc, conf = engine.verify_windows_resident(sids, rows, src, n_vocab=V,
                                                             flags=fb.APPEND_SAMPLED if append else 0)
            for i in range(S):
                t, a, c, _ = want[i]
                assert acc[i] == a and conf[i] == c and list(toks[i][:a]) == list(t[:a]), (step, i)
                new = np.asarray(t[:a], dtype=np.int32)
                if append:
                    hists[i] = np.concatenate([hists[i], new]).astype(np.int32)
                else:                                          # the caller appends what it accepted
                    engine.history_append(int(sids[i]), new)
                    hists[i] = np.concatenate([hists[i], new]).astype(np.int32)
            assert [engine.history_len(int(s)) for s in sids] == [len(x) for x in hists]
        # a plain resident step afterwards reads the histories the windows left behind
        lg = (rng.standard_normal((S, V)) * 2).astype(np.float32)
        for i in range(S):
            lg[i, hists[i][-3:]] += 8.0
        ref = oracle.sample_rows(p, rngs, lg.copy(), hists)
        assert np.array_equal(engine.sample_batch_resident(sids, lg.copy()), ref["tokens"])
    finally:
        for s in sids:
            engine.close_stream(int(s))


def test_prompt_lookup_drafts_of_resident_histories_match_the_oracle(engine, oracle):
    """lookup_draft (src/server.cpp:552-564) run on the device over the id pool, 40 streams at a time."""
    rng = np.random.default_rng(99)
    S = 40
    p = fb.make_params(S)
    p["seed"] = np.arange(S)
    sids = engine.open_streams(p)
    try:
        for trial in range(4):
            hists = []
            for i in range(S):
                L = int(rng.integers(0, 30)) if i % 4 == 0 else int(rng.integers(200, 3000))
                alphabet = 3 if i % 3 == 0 else 200                # dense repeats / natural-looking text
                h = rng.integers(0, alphabet, size=L).astype(np.int32)
                if L > 100 and i % 2:                              # a copied run: the end repeats an earlier stretch
                    a = int(rng.integers(0, L // 2))
                    h[-12:] = h[a:a + 12]
                hists.append(h)
                engine.history_set(int(sids[i]), h)
            kmax = rng.integers(1, 9, size=S).astype(np.int32)
            min_n = rng.integers(1, 4, size=S).astype(np.int32)
            eos = int(rng.integers(0, 3))
            got = engine.lookup_drafts(sids, kmax, min_n, eos)
            for i in range(S):
                assert list(got[i]) == list(oracle.lookup_draft(hists[i], int(kmax[i]), eos, int(min_n[i]))), (trial, i)
        with pytest.raises(fb.SamplerError):
            engine.lookup_drafts(sids[:1], 4, 0, 0)                # a match of zero tokens is not a match
    finally:
        for s in sids:
            engine.close_stream(int(s))


def test_resident_windows_of_streams_without_a_penalty_keep_their_device_history(engine, oracle):
    """A stream whose penalty is off has empty penalty windows, so its drafts are never written into the id pool before
    the launch; the accepted tokens must still reach the device copy of its history (the drafting kernel reads it)."""
    S, V, m = 4, 33, 5                                     # a tiny vocabulary: n-grams repeat, the lookup finds matches
    rng = np.random.default_rng(4711)
    p = fb.make_params(S, temperature=0.8, top_k=10, top_p=0.9, repetition_penalty=1.2)
    p["repetition_penalty"][:2] = 1.0                      # penalty off
    p["repeat_last_n"][2] = 0                              # window off
    p["temperature"][1] = 0.0
    p["seed"] = 900 + np.arange(S)
    sids = engine.open_streams(p)
    rngs = oracle.new_rngs(p["seed"])
    hists = [rng.integers(0, V, size=int(n)).astype(np.int32) for n in rng.integers(5, 30, size=S)]
    try:
        for i, s in enumerate(sids):
            engine.history_set(int(s), hists[i])
        for step in range(5):
            lg = (rng.standard_normal((S * m, V)) * 2).astype(np.float32)
            rows = []
            for i in range(S):
                drafts = rng.integers(0, V, size=m - 1).astype(np.int32)
                h, probe = list(hists[i]), rngs[i:i + 1].copy()
                for r in range(int(rng.integers(0, m))):           # a prefix of right drafts
                    t = int(oracle.sample_rows(p[i:i + 1], probe, lg[i * m + r:i * m + r + 1].copy(), [np.array(h, dtype=np.int32)])["tokens"][0])
                    if r < m - 1:
                        drafts[r] = t
                    h.append(t)
                rows.append(np.concatenate([[int(hists[i][-1])], drafts]).astype(np.int32))
            want = [oracle.verify_window(p[i:i + 1], rngs[i], lg[i * m:(i + 1) * m].copy(), rows[i], hists[i]) for i in range(S)]
            toks, acc, conf = engine.verify_windows_resident(sids, rows, lg.copy(), n_vocab=V, flags=fb.APPEND_SAMPLED)
            for i in range(S):
                t, a, c, _ = want[i]
                assert acc[i] == a and conf[i] == c and list(toks[i][:a]) == list(t[:a]), (step, i)
                hists[i] = np.concatenate([hists[i], np.asarray(t[:a], dtype=np.int32)]).astype(np.int32)
            got = engine.lookup_drafts(sids, 6, 1, V)               # eos outside the vocabulary: never cuts
            for i in range(S):
                assert list(got[i]) == list(oracle.lookup_draft(hists[i], 6, V, 1)), (step, i)
    finally:
        for s in sids:
            engine.close_stream(int(s))
