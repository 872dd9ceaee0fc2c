"""CPU tests: the C restatement of the reference sampler against the reference's own known-answer test, the
committed golden vectors (made by the unmodified reference) and, where it is built, the reference itself."""
import numpy as np
import pytest

from helpers import golden_case_inputs, load_golden, random_case


def test_known_answer_vector_of_the_reference(oracle):
    # tests/test_kernels.cpp:348-359 of the reference: whole=4 generated=2 last2=1 off=2 generated+last2=2
    from oracle import make_params
    kat = load_golden()["kat"]
    got = []
    for last_n, frm in kat["window_scope"]:
        p = make_params(1, temperature=kat["temperature"], repetition_penalty=kat["repetition_penalty"], repeat_last_n=last_n, penalty_from=frm)
        lg = np.array([kat["logits"]], dtype=np.float32)
        got.append(int(oracle.sample_rows(p, oracle.new_rngs([1]), lg, [kat["history"]])["tokens"][0]))
    assert got == kat["tokens"] == [4, 2, 1, 2, 2]


def test_mt19937_64_check_value(oracle):
    # the C++ standard fixes the 10000th output of a default-seeded (5489) mt19937_64
    st = oracle.new_rngs([5489])
    x = 0
    for _ in range(10000):
        x = oracle.next_word(st[0])
    assert x == 9981545732273789042


def test_uniform_mapping(oracle):
    assert oracle.canonical(0) == 0.0
    assert oracle.canonical((1 << 64) - 1) == np.nextafter(1.0, 0.0)      # rounds to 1.0, then clamped
    assert oracle.canonical(1 << 63) == 0.5


@pytest.mark.parametrize("idx", range(5))
def test_oracle_reproduces_golden_vectors(oracle, idx):
    case = load_golden()["cases"][idx]
    lg, p, hists = golden_case_inputs(case)
    for r in range(case["rows"]):
        rng = oracle.new_rngs([p["seed"][r]])
        toks = []
        for _ in range(case["n_draws"]):
            row = lg[r:r + 1].copy()
            toks.append(int(oracle.sample_rows(p[r:r + 1], rng, row, [hists[r]])["tokens"][0]))
        assert toks == case["tokens"][r], (case["name"], r)


def test_oracle_matches_reference_on_random_cases(oracle, reflib):
    rng = np.random.default_rng(0)
    shapes = [(4, 6), (4, 33), (4, 1000), (4, 4096), (3, 65536)]
    bad = 0
    for trial in range(120):
        B, V = shapes[trial % len(shapes)]
        lg, p, hists = random_case(rng, B, V, trial)
        a = oracle.sample_rows(p, oracle.new_rngs(p["seed"]), lg.copy(), hists)["tokens"]
        b = reflib.sample_rows(p, lg.copy(), hists)
        bad += int((a != b).sum())
    assert bad == 0


def test_oracle_in_place_penalty_matches_reference(oracle, reflib):
    rng = np.random.default_rng(3)
    lg, p, hists = random_case(rng, 4, 1000, 1)
    p["repetition_penalty"] = 1.3
    p["repeat_last_n"] = -1
    p["penalty_from"] = 0
    a, b = lg.copy(), lg.copy()
    oracle.sample_rows(p, oracle.new_rngs(p["seed"]), a, hists)
    reflib.sample_rows(p, b, hists)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_oracle_window_matches_reference(oracle, reflib):
    from oracle import make_params
    rng = np.random.default_rng(5)
    V, m = 2000, 9
    for trial in range(20):
        lg = (rng.standard_normal((m, V)) * 2).astype(np.float32)
        greedy = trial % 2 == 0
        p = make_params(1, temperature=0.0 if greedy else 0.8, top_k=50, repetition_penalty=1.2, repeat_last_n=int(rng.choice([-1, 4])), seed=77 + trial)
        hist = rng.integers(0, V, size=30).astype(np.int32)
        rows = rng.integers(0, V, size=m).astype(np.int32)
        # make a prefix of the drafts right (greedy rows only: the argmax of the row before, with the growing history)
        L = int(rng.integers(0, m))
        if greedy:
            h = list(hist)
            for r in range(min(L, m - 1)):
                t = int(oracle.sample_rows(p, oracle.new_rngs([1]), lg[r:r + 1].copy(), [np.array(h, dtype=np.int32)])["tokens"][0])
                rows[r + 1] = t
                h.append(t)
        ta, acc_a, conf_a, _ = oracle.verify_window(p, oracle.new_rngs(p["seed"])[0], lg.copy(), rows, hist)
        tb, acc_b, conf_b = reflib.verify_window(p, lg.copy(), rows, hist)
        assert acc_a == acc_b and conf_a == conf_b and list(ta[:acc_a]) == list(tb[:acc_b])


def _lookup_by_definition(h, kmax, eos, min_n):
    """The drafting rule written as a search over all candidates, independent of the restatement's loop order."""
    L = len(h)
    for n in range(min(4, L - 1), min_n - 1, -1):
        hits = [p for p in range(0, L - n) if list(h[p:p + n]) == list(h[L - n:])]
        for p in sorted(hits, reverse=True):
            d = []
            for t in h[p + n:]:
                if t == eos or len(d) >= kmax:
                    break
                d.append(int(t))
            if d:
                return d
    return []


def test_prompt_lookup_drafting_follows_its_definition(oracle):
    rng = np.random.default_rng(12)
    assert list(oracle.lookup_draft([5, 6, 7, 8, 9, 1, 5, 6, 7, 8], 3, 0, 2)) == [9, 1, 5]          # the 4-gram, three drafts
    assert list(oracle.lookup_draft([5, 6, 7, 0, 9, 5, 6, 7], 4, 0, 2)) == []                        # only continuation starts with eos
    assert list(oracle.lookup_draft([1, 2, 9, 3, 1, 2, 0, 4, 1, 2], 4, 0, 2)) == [9, 3, 1, 2]        # the recent hit drafts nothing: the earlier one
    assert list(oracle.lookup_draft([7], 4, 0, 2)) == [] and list(oracle.lookup_draft([], 4, 0, 2)) == []
    assert list(oracle.lookup_draft([3, 4, 3], 2, 0, 1)) == [4, 3] and list(oracle.lookup_draft([3, 4, 3], 2, 0, 2)) == []
    for trial in range(300):
        L = int(rng.integers(0, 60))
        h = rng.integers(0, 4, size=L).astype(np.int32)            # a tiny alphabet: repeats everywhere
        kmax, eos, min_n = int(rng.integers(1, 9)), int(rng.integers(0, 5)), int(rng.integers(1, 5))
        assert list(oracle.lookup_draft(h, kmax, eos, min_n)) == _lookup_by_definition(h, kmax, eos, min_n), (h, kmax, eos, min_n)
