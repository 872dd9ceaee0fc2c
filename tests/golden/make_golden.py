"""Generates tests/golden/sampler_golden.json from the UNMODIFIED reference sampler.

Run in a checkout that has the reference sources (oracle/_ref is built from them):
    python tests/golden/make_golden.py
Inputs come from the integer-only generator `ferro_b200.synth.exact_logits` (exact in binary floating point, so
they are the same on every machine); the file stores the parameters, the histories and the tokens the reference
produced.  The tests replay the cases through the C oracle (CPU) and through the CUDA library (GPU).
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from ferro_b200 import synth  # noqa: E402
from oracle import RefLib, make_params  # noqa: E402

FIELDS = ["temperature", "top_k", "top_p", "min_p", "repetition_penalty", "repeat_last_n", "penalty_from", "seed"]


def cases():
    """(name, rows, vocab, logits seed, ties, per-row parameter overrides, history lengths, n_draws)"""
    out = []
    out.append(dict(name="greedy_ties", rows=4, vocab=1000, lseed=11, ties=True, n_draws=1,
                    params=[dict(temperature=0.0, repetition_penalty=1.0), dict(temperature=0.0, repetition_penalty=2.0),
                            dict(temperature=0.5, top_k=1, repetition_penalty=1.3), dict(temperature=0.0, repetition_penalty=0.7, repeat_last_n=5)],
                    hist_len=[0, 40, 17, 33]))
    out.append(dict(name="topk_small_vocab", rows=6, vocab=33, lseed=12, ties=False, n_draws=4,
                    params=[dict(temperature=0.7, top_k=5), dict(temperature=1.0, top_k=40, top_p=0.9), dict(temperature=1.3, top_k=0, min_p=0.1),
                            dict(temperature=0.2, top_k=2, top_p=0.5), dict(temperature=1.0, top_k=33), dict(temperature=0.05, top_k=50)],
                    hist_len=[3, 0, 10, 64, 5, 2]))
    out.append(dict(name="topk_65536", rows=4, vocab=65536, lseed=13, ties=False, n_draws=3,
                    params=[dict(temperature=0.7, top_k=40, top_p=0.95, repetition_penalty=1.1), dict(temperature=0.8, top_k=50),
                            dict(temperature=1.0, top_k=64, top_p=0.9, min_p=0.02), dict(temperature=1.0, top_k=256, repetition_penalty=1.15, penalty_from=100)],
                    hist_len=[64, 256, 512, 300]))
    out.append(dict(name="full_vocab_4097", rows=4, vocab=4097, lseed=14, ties=False, n_draws=3,
                    params=[dict(temperature=1.0, top_k=0), dict(temperature=1.0, top_k=0, top_p=0.9, min_p=0.05),
                            dict(temperature=0.6, top_k=1000, top_p=0.8), dict(temperature=1.5, top_k=5000, min_p=0.001, repetition_penalty=1.2)],
                    hist_len=[0, 100, 50, 200]))
    out.append(dict(name="ties_topk", rows=3, vocab=5000, lseed=15, ties=True, n_draws=3,
                    params=[dict(temperature=1.0, top_k=40), dict(temperature=0.9, top_k=0, top_p=0.7), dict(temperature=1.0, top_k=300, min_p=0.05)],
                    hist_len=[20, 20, 20]))
    return out


def build(case):
    lg = synth.exact_logits(case["lseed"], case["rows"], case["vocab"], ties=case["ties"])
    p = make_params(case["rows"])
    for r, kw in enumerate(case["params"]):
        for k, v in kw.items():
            p[k][r] = v
        p["seed"][r] = 1000 * case["lseed"] + r + 1
    hists = [synth.randint(case["lseed"], 50 + r, n, case["vocab"] + 4).astype(np.int32) - 2 for r, n in enumerate(case["hist_len"])]
    return lg, p, hists


def main():
    ref = RefLib()
    doc = {"generator": "tests/golden/make_golden.py", "source": "reference sampler compiled unmodified (src/sampler.cpp)", "cases": []}
    for case in cases():
        lg, p, hists = build(case)
        tokens = [ref.sample_repeat(p[r:r + 1], lg[r], hists[r], case["n_draws"]).tolist() for r in range(case["rows"])]
        rec = {k: case[k] for k in ("name", "rows", "vocab", "lseed", "ties", "n_draws", "params", "hist_len")}
        rec["tokens"] = tokens
        rec["logits_checksum"] = int(lg.view(np.uint32).astype(np.uint64).sum() % (1 << 61))
        doc["cases"].append(rec)
    # the reference's own known-answer test (tests/test_kernels.cpp:348-359)
    doc["kat"] = {"logits": [0, 9, 10, 9.5, 6, 0], "history": [1, 2, 3], "temperature": 0.0, "repetition_penalty": 2.0,
                  "window_scope": [[-1, 0], [-1, 2], [2, 0], [0, 0], [2, 2]], "tokens": [4, 2, 1, 2, 2]}
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "sampler_golden.json"), "w") as f:
        json.dump(doc, f, indent=1)
    print("wrote", len(doc["cases"]), "cases")


if __name__ == "__main__":
    main()
