"""Shared helpers of the test-suite: golden cases, random cases, comparison of a device result with the oracle."""
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden", "sampler_golden.json")

# Tolerances of the parity contract: kept-set probabilities within 1e-6 absolute; a stochastic draw may differ
# from the reference only where the uniform lands within 1e-6 of a boundary of the cumulative distribution.
PROB_TOL = 1e-6
CDF_TOL = 1e-6


def load_golden():
    with open(GOLDEN) as f:
        return json.load(f)


def golden_case_inputs(case):
    """Rebuilds the inputs of a golden case exactly as tests/golden/make_golden.py did."""
    from ferro_b200 import synth
    from oracle import make_params
    lg = synth.exact_logits(case["lseed"], case["rows"], case["vocab"], ties=case["ties"])
    assert int(lg.view(np.uint32).astype(np.uint64).sum() % (1 << 61)) == case["logits_checksum"], "input generator drifted"
    p = make_params(case["rows"])
    for r, kw in enumerate(case["params"]):
        for k, v in kw.items():
            p[k][r] = v
        p["seed"][r] = 1000 * case["lseed"] + r + 1
    hists = [synth.randint(case["lseed"], 50 + r, n, case["vocab"] + 4).astype(np.int32) - 2 for r, n in enumerate(case["hist_len"])]
    return lg, p, hists


def random_case(rng, B, V, trial, allow_full=True, max_hist=300):
    """A seeded random batch that walks through the branches of the reference sampler."""
    from oracle import make_params
    lg = (rng.standard_normal((B, V)) * 3).astype(np.float32)
    if trial % 4 == 0:
        lg = (np.round(lg * 2) / 2).astype(np.float32)      # many equal logits
    if trial % 7 == 0:
        lg[:, : V // 2] = -np.inf                          # masked half
    if trial % 9 == 0:
        lg[:] = 1.5                                        # all equal
    if trial % 5 == 0:
        lg[:, ::3] = np.where(lg[:, ::3] == 0, -0.0, lg[:, ::3])
        lg[0, : min(V, 4)] = [0.0, -0.0, 0.0, -0.0][: min(V, 4)]
    p = make_params(B)
    p["temperature"] = rng.choice([0, 0.7, 1.0, 0.05], size=B)
    ks = [1, 2, 40, 50, 64, 200, 256] + ([0, V, V + 5, 300, 1000] if allow_full else [])
    p["top_k"] = rng.choice(ks, size=B)
    if not allow_full:
        for i in range(B):
            if not (0 < p["top_k"][i] < V) and V > 256 and p["temperature"][i] > 0:
                p["top_k"][i] = 40
    p["top_p"] = rng.choice([1.0, 0.9, 0.5, 0.95], size=B)
    p["min_p"] = rng.choice([0, 0.05, 0.3], size=B)
    p["repetition_penalty"] = rng.choice([1.0, 1.1, 2.0, 0.8], size=B)
    p["repeat_last_n"] = rng.choice([-1, 0, 3, 64], size=B)
    p["penalty_from"] = rng.choice([0, 2, 10], size=B)
    p["seed"] = rng.integers(1, 1 << 62, size=B)
    hists = [rng.integers(-2, V + 2, size=int(rng.integers(0, max_hist))).astype(np.int32) for _ in range(B)]
    return lg, p, hists


def effective_k(p_row, V):
    if p_row["temperature"] <= 0 or p_row["top_k"] == 1:
        return 1
    return int(p_row["top_k"]) if 0 < p_row["top_k"] < V else V


def compare_with_oracle(engine, tokens, ref, params, V, check_kept=True):
    """Returns (exact token mismatches that are NOT within CDF_TOL of a boundary, near-boundary mismatches, kept-set errors)."""
    import ferro_b200 as fb
    hard, near, kept_bad = [], 0, []
    B = len(tokens)
    for i in range(B):
        k = effective_k(params[i], V)
        if tokens[i] != ref["tokens"][i]:
            if k == 1:
                hard.append((i, int(tokens[i]), int(ref["tokens"][i]), "greedy"))
            else:
                nk = int(ref["n_keep"][i])
                cdf = np.cumsum(ref["kept_pr"][i, :nk])
                if np.abs(cdf - ref["r_tot"][i, 0]).min() < CDF_TOL:
                    near += 1
                else:
                    hard.append((i, int(tokens[i]), int(ref["tokens"][i]), "draw"))
        if check_kept and k > 1:
            ids, pr, n = engine.last_kept(i)
            nk = int(ref["n_keep"][i])
            if n != nk and abs(n - nk) == 1 and params[i]["top_p"] < 1.0:
                # The top-p cut sits on a boundary of the cumulative distribution: the reference's sequential sum
                # reached top_p (or missed it) by rounding alone, e.g. equal probabilities that add up to exactly top_p.
                # Counted like a draw that lands on a boundary; what both kept is still compared.
                tot, last = ref["r_tot"][i, 1], ref["r_tot"][i, 2]
                if min(abs(tot - params[i]["top_p"]), abs(tot - last - params[i]["top_p"])) < CDF_TOL:
                    near += 1
                    nk = n = min(n, nk)
                    ids, pr = ids[:n], pr[:n]
            if k <= fb.MAX_CANDIDATE_K:
                if n != nk or (ids != ref["kept_ids"][i, :nk]).any() or np.abs(pr - ref["kept_pr"][i, :nk]).max() > PROB_TOL:
                    kept_bad.append(i)
            else:   # full-vocabulary kernel: the kept set's size, and its first MAX_CANDIDATE_K candidates one by one
                m = min(nk, fb.MAX_CANDIDATE_K, ref["kept_ids"].shape[1])
                if n != nk or len(ids) < m or (ids[:m] != ref["kept_ids"][i, :m]).any() or np.abs(pr[:m] - ref["kept_pr"][i, :m]).max() > PROB_TOL:
                    kept_bad.append(i)
    return hard, near, kept_bad
