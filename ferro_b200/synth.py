"""Seeded synthetic workloads with the shapes and value distributions of the sampler's benchmark configurations.

No public dataset or model is involved: the five configurations *are* the workload (logits drawn from the stated
distributions, histories from uniform / Zipf draws).  Everything is generated from a counter-based generator
(splitmix64 over (seed, stream, counter)), so the same arrays can be produced on any machine; normals come from
Box-Muller, Student-t(3) from a normal over the root of a mean of three squared normals, Zipf(s) by inverse CDF
over ranks with a seeded rank -> id permutation.  Logits are computed in float64 and rounded once to float32.

``exact_logits`` is a second, integer-only generator used for the committed golden vectors: its values are exact
in binary floating point, so they do not depend on any libm.
"""
from __future__ import annotations

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def splitmix64(x: np.ndarray) -> np.ndarray:
    """One splitmix64 output per input word (uint64 array)."""
    with np.errstate(over="ignore"):
        z = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return z ^ (z >> np.uint64(31))


def words(seed: int, stream: int, n: int, offset: int = 0) -> np.ndarray:
    """n 64-bit words of stream `stream` of generator `seed`, counters offset .. offset + n - 1."""
    with np.errstate(over="ignore"):
        base = splitmix64(np.array([np.uint64(seed) * np.uint64(0x100000001B3) + np.uint64(stream)], dtype=np.uint64))[0]
        ctr = np.arange(offset, offset + n, dtype=np.uint64)
        return splitmix64(ctr * np.uint64(0xD6E8FEB86659FD93) + base)


def uniforms(seed: int, stream: int, n: int, offset: int = 0) -> np.ndarray:
    """n doubles in (0, 1)."""
    return ((words(seed, stream, n, offset) >> np.uint64(11)).astype(np.float64) + 0.5) * (1.0 / 9007199254740992.0)


def normals(seed: int, stream: int, n: int) -> np.ndarray:
    m = (n + 1) // 2
    u1 = uniforms(seed, stream, m)
    u2 = uniforms(seed, stream + 1, m)
    r = np.sqrt(-2.0 * np.log(u1))
    z = np.concatenate([r * np.cos(2.0 * np.pi * u2), r * np.sin(2.0 * np.pi * u2)])
    return z[:n]


def student_t3(seed: int, stream: int, n: int) -> np.ndarray:
    z = normals(seed, stream, n)
    a, b, c = normals(seed, stream + 2, n), normals(seed, stream + 4, n), normals(seed, stream + 6, n)
    return z / np.sqrt((a * a + b * b + c * c) / 3.0)


def randint(seed: int, stream: int, n: int, hi: int) -> np.ndarray:
    return (words(seed, stream, n) % np.uint64(hi)).astype(np.int64)


def permutation(seed: int, stream: int, n: int) -> np.ndarray:
    """Seeded permutation of 0..n-1 (argsort of random words: deterministic, ties impossible in practice)."""
    return np.argsort(words(seed, stream, n), kind="stable").astype(np.int64)


def zipf_ids(seed: int, stream: int, n: int, vocab: int, s: float = 1.1) -> np.ndarray:
    """n token ids, Zipf(s) over ranks 1..vocab, rank -> id through a seeded permutation."""
    w = 1.0 / np.power(np.arange(1, vocab + 1, dtype=np.float64), s)
    cdf = np.cumsum(w)
    cdf /= cdf[-1]
    ranks = np.searchsorted(cdf, uniforms(seed, stream, n), side="left")
    return permutation(seed, stream + 1, vocab)[np.minimum(ranks, vocab - 1)].astype(np.int32)


def softcap_host(x: np.ndarray, cap: float, tanhf=None) -> np.ndarray:
    """cap * tanh(x / cap) in float32: the final-logit softcap the Gemma-4 forward applies (src/model_gemma4.cpp:521
    of the reference).  `tanhf(array, cap)` - an in-place float32 softcap built on the C library's tanhf, which is what
    the reference calls - is used when given; otherwise numpy's float32 tanh, which may differ from it in the last bit.
    Callers that compare with the reference pass the C function; either way every consumer of one generated array
    sees the same values."""
    x = np.ascontiguousarray(x, dtype=np.float32).copy()
    if tanhf is not None:
        tanhf(x, cap)
        return x
    c = np.float32(cap)
    return (c * np.tanh(x / c, dtype=np.float32)).astype(np.float32)


def exact_logits(seed: int, rows: int, vocab: int, scale_pow2: int = -13, ties: bool = False) -> np.ndarray:
    """Bell-shaped logits that are exact in binary: (sum of four 16-bit uniforms - 2 * 65535) * 2**scale_pow2.
    With ties=True the values are quantised to multiples of 0.5 so that many logits are equal."""
    w = words(seed, 11, rows * vocab)
    s = ((w & np.uint64(0xFFFF)) + ((w >> np.uint64(16)) & np.uint64(0xFFFF)) + ((w >> np.uint64(32)) & np.uint64(0xFFFF)) +
         ((w >> np.uint64(48)) & np.uint64(0xFFFF))).astype(np.int64) - 2 * 65535
    x = s.astype(np.float64) * (2.0 ** scale_pow2)
    if ties:
        x = np.round(x * 2.0) / 2.0
    return x.astype(np.float32).reshape(rows, vocab)


# ------------------------------------------------------------------------------------------------ the five configurations
def _params(n, **kw):
    """n parameter records with the reference's defaults (src/sampler.h:13-20); built without loading the CUDA library."""
    from . import PARAMS_DTYPE
    p = np.zeros(n, dtype=PARAMS_DTYPE)
    p["temperature"], p["top_k"], p["top_p"], p["min_p"] = 0.05, 50, 1.0, 0.0
    p["repetition_penalty"], p["repeat_last_n"], p["penalty_from"], p["seed"] = 1.05, -1, 0, 0
    for k, v in kw.items():
        p[k] = v
    return p


def config1(vocab: int = 65536):
    """Single stream, V = 65536: N(0, 3^2) logits with 8 ids boosted by +12, T 0.7, top-k 40, top-p 0.95,
    penalty 1.1 over a 64-id uniform history, sampler seed 1234.  The caller draws repeatedly from the one stream."""
    lg = normals(1, 100, vocab) * 3.0
    lg[randint(1, 110, 8, vocab)] += 12.0
    hist = randint(1, 120, 64, vocab).astype(np.int32)
    p = _params(1, temperature=0.7, top_k=40, top_p=0.95, min_p=0.0, repetition_penalty=1.1, repeat_last_n=-1, penalty_from=0, seed=1234)
    return dict(logits=lg.astype(np.float32).reshape(1, vocab), params=p, hists=[hist])


def config2(vocab: int = 65536):
    """Multi-slot decode batch: 8 rows, mixed parameters, 256-id Zipf histories, penalty 1.15, seeds 42 + row."""
    B = 8
    lg = (normals(42, 100, B * vocab) * 3.0).reshape(B, vocab)
    for r in range(B):
        ids = randint(42, 200 + r, 16, vocab)
        lg[r, ids] += 8.0 + 6.0 * uniforms(42, 300 + r, 16)
    p = _params(B, repetition_penalty=1.15, repeat_last_n=-1, penalty_from=0, top_p=1.0, min_p=0.0)
    p["temperature"] = [0, 0, 1.0, 1.0, 0.8, 0.8, 1.0, 1.0]
    p["top_k"] = [50, 50, 0, 0, 50, 50, 0, 0]
    p["top_p"][6:] = 0.9
    p["min_p"][6:] = 0.05
    p["seed"] = 42 + np.arange(B)
    hists = [zipf_ids(42, 400 + 2 * r, 256, vocab) for r in range(B)]
    return dict(logits=lg.astype(np.float32), params=p, hists=hists)


def config3(rows: int = 64, vocab: int = 262144, tanhf=None):
    """Gemma-4-style large vocabulary: Student-t(3) * 4 softcapped at 30 on the host, T 1, top-k 64, top-p 0.95,
    penalty 1.0 / 1.1 on alternating rows over 512-id uniform histories, seeds 7 + row.  `tanhf`: see softcap_host."""
    raw = (student_t3(7, 100, rows * vocab) * 4.0).astype(np.float32).reshape(rows, vocab)
    p = _params(rows, temperature=1.0, top_k=64, top_p=0.95, min_p=0.0, repetition_penalty=1.0, repeat_last_n=-1, penalty_from=0)
    p["repetition_penalty"][1::2] = 1.1
    p["seed"] = 7 + np.arange(rows)
    hists = [randint(7, 500 + r, 512, vocab).astype(np.int32) for r in range(rows)]
    return dict(logits=softcap_host(raw, 30.0, tanhf), raw_logits=raw, params=p, hists=hists)


def config4(streams: int = 8, window: int = 17, vocab: int = 65536, penalty: float = 1.0, hist_len: int = 0):
    """Speculative verification: `streams` windows of `window` rows, N(0, 2^2) logits, greedy.  For each stream the
    draft ids equal the argmax of the row they are compared with for a geometric(0.3) prefix, then random ids."""
    R = streams * window
    lg = (normals(4, 100, R * vocab) * 2.0).astype(np.float32).reshape(R, vocab)
    p = _params(streams, temperature=0.0, top_k=50, top_p=1.0, min_p=0.0, repetition_penalty=penalty, repeat_last_n=-1, penalty_from=0)
    p["seed"] = 4 + np.arange(streams)
    hists = [randint(4, 700 + s, hist_len, vocab).astype(np.int32) for s in range(streams)]
    u = uniforms(4, 800, streams)
    rows = []
    for s in range(streams):
        L = int(min(window, np.floor(np.log(u[s]) / np.log(0.7))))
        last = int(randint(4, 900 + s, 1, vocab)[0])
        drafts = randint(4, 1000 + s, window - 1, vocab)
        for r in range(1, window):
            if r <= L:
                drafts[r - 1] = int(np.argmax(lg[s * window + r - 1]))   # the token row r-1 will produce
        rows.append(np.concatenate([[last], drafts]).astype(np.int32))
    return dict(logits=lg, params=p, hists=hists, rows=rows)


def config5(rows: int = 512, vocab: int = 262144, tanhf=None):
    """Box-scale serving batch: Student-t(3) * 4 softcapped at 30, top-k 40, top-p 0.9, T 0.8, penalty 1.1 over
    1024-id Zipf histories, seeds 99 + row.  `tanhf`: see softcap_host."""
    raw = (student_t3(99, 100, rows * vocab) * 4.0).astype(np.float32).reshape(rows, vocab)
    p = _params(rows, temperature=0.8, top_k=40, top_p=0.9, min_p=0.0, repetition_penalty=1.1, repeat_last_n=-1, penalty_from=0)
    p["seed"] = 99 + np.arange(rows)
    perm = permutation(99, 601, vocab)
    w = 1.0 / np.power(np.arange(1, vocab + 1, dtype=np.float64), 1.1)
    cdf = np.cumsum(w)
    cdf /= cdf[-1]
    hists = []
    for r in range(rows):
        ranks = np.searchsorted(cdf, uniforms(99, 1000 + r, 1024), side="left")
        hists.append(perm[np.minimum(ranks, vocab - 1)].astype(np.int32))
    return dict(logits=softcap_host(raw, 30.0, tanhf), raw_logits=raw, params=p, hists=hists)
