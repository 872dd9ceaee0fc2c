"""A seeded walk over shapes, parameter mixes and call flags against the oracle: every third batch without
full-vocabulary rows, every fifth all greedy (the lane-best variant of the streaming kernel), every fourth with
write-back.  One engine sized for the longest rows serves all shapes, as a server's would."""
import numpy as np
import pytest

import ferro_b200 as fb
from helpers import compare_with_oracle, random_case

pytestmark = pytest.mark.gpu

SHAPES = [(1, 7), (2, 129), (3, 4096), (5, 8193), (4, 50000), (8, 65536), (2, 131072), (3, 262144), (17, 32768), (2, 299999), (33, 16384), (64, 9000)]


def test_seeded_walk_over_shapes_and_flags(oracle):
    eng = fb.Engine(device=0, max_rows=64, max_vocab=300000, max_hist_ids=1 << 20)
    rng = np.random.default_rng(2025)
    near_total = 0
    try:
        for n in range(360):
            B, V = SHAPES[n % len(SHAPES)]
            trial = int(rng.integers(0, 1000))
            lg, p, hists = random_case(rng, B, V, trial, allow_full=(n % 3 != 0))
            if n % 5 == 0:
                p["temperature"] = 0.0
            flags = fb.KEEP_KEPT_SET | (fb.WRITE_BACK if n % 4 == 1 else 0)
            ref_lg = lg.copy()
            ref = oracle.sample_rows(p, oracle.new_rngs(p["seed"]), ref_lg, hists, cap=fb.MAX_CANDIDATE_K)
            sids = eng.open_streams(p)
            work = lg.copy()
            tok = eng.sample_batch(sids, work, hists, flags=flags)
            hard, near, kept_bad = compare_with_oracle(eng, tok, ref, p, V)
            for s in sids:
                eng.close_stream(int(s))
            assert not hard and not kept_bad, (n, (B, V), trial, hard[:2], kept_bad[:2])
            if flags & fb.WRITE_BACK:
                assert np.array_equal(work, ref_lg, equal_nan=True), (n, (B, V), trial)
            near_total += near
        assert near_total <= 2
    finally:
        eng.close()
