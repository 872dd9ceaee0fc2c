"""ctypes loader for the CPU oracle.  TEST INFRASTRUCTURE ONLY.

``Oracle``  wraps the plain-C restatement of the reference sampler (``sampler_oracle.c``).
``RefLib``  wraps the unmodified reference sampler compiled from the reference checkout
            (``ref_driver.cpp`` + the reference's ``src/sampler.cpp``), when it has been built.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark may import this
package; the product library (``ferro_b200``) never does.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

PARAMS_DTYPE = np.dtype(
    {
        "names": ["temperature", "top_k", "top_p", "min_p", "repetition_penalty", "repeat_last_n", "penalty_from", "seed"],
        "formats": [np.float32, np.int32, np.float32, np.float32, np.float32, np.int32, np.int32, np.uint64],
        "offsets": [0, 4, 8, 12, 16, 20, 24, 32],
        "itemsize": 40,
    }
)

_MT_BYTES = 312 * 8 + 8  # uint64 mt[312]; int idx; padding


def make_params(n: int, **kw) -> np.ndarray:
    """n parameter records with the reference's defaults (src/sampler.h:12-21), overridden by kw."""
    p = np.zeros(n, dtype=PARAMS_DTYPE)
    p["temperature"] = 0.05
    p["top_k"] = 50
    p["top_p"] = 1.0
    p["min_p"] = 0.0
    p["repetition_penalty"] = 1.05
    p["repeat_last_n"] = -1
    p["penalty_from"] = 0
    p["seed"] = 0
    for k, v in kw.items():
        p[k] = v
    return p


def _ptr(a, typ):
    return a.ctypes.data_as(C.POINTER(typ)) if a is not None else None


def flatten_hist(hists):
    """list of 1-D int arrays -> (flat int32, offsets int64[n+1])"""
    off = np.zeros(len(hists) + 1, dtype=np.int64)
    for i, h in enumerate(hists):
        off[i + 1] = off[i] + len(h)
    flat = np.zeros(max(int(off[-1]), 1), dtype=np.int32)
    for i, h in enumerate(hists):
        flat[off[i]:off[i + 1]] = np.asarray(h, dtype=np.int32)
    return flat, off


class Oracle:
    """The C restatement.  Stateless apart from the engines the caller holds (``new_rngs``)."""

    def __init__(self):
        self.lib = C.CDLL(_build.build_oracle())
        L = self.lib
        L.oracle_mt64_seed.argtypes = [C.c_void_p, C.c_uint64]
        L.oracle_mt64_next.argtypes = [C.c_void_p]
        L.oracle_mt64_next.restype = C.c_uint64
        L.oracle_canonical.argtypes = [C.c_uint64]
        L.oracle_canonical.restype = C.c_double
        L.oracle_softcap.argtypes = [C.c_void_p, C.c_int64, C.c_float]
        L.oracle_window_begin.argtypes = [C.c_void_p, C.c_int64]
        L.oracle_window_begin.restype = C.c_int64
        L.oracle_sample.restype = C.c_int
        L.oracle_sample.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int64,
                                    C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        L.oracle_sample_rows.restype = C.c_int
        L.oracle_sample_rows.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int,
                                         C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        L.oracle_verify_window.restype = C.c_int
        L.oracle_verify_window.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p,
                                           C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]

        L.oracle_lookup_draft.restype = C.c_int
        L.oracle_lookup_draft.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]

    def lookup_draft(self, hist, kmax: int, eos: int, min_n: int) -> np.ndarray:
        """Prompt-lookup drafts of one history (lookup_draft, src/server.cpp:552-564)."""
        h = np.ascontiguousarray(hist, dtype=np.int32)
        out = np.zeros(max(kmax, 1), dtype=np.int32)
        n = self.lib.oracle_lookup_draft(h.ctypes.data, len(h), int(kmax), int(eos), int(min_n), out.ctypes.data)
        return out[:n].copy()

    # --- engines
    def new_rngs(self, seeds) -> np.ndarray:
        seeds = np.asarray(seeds, dtype=np.uint64).reshape(-1)
        st = np.zeros((len(seeds), _MT_BYTES), dtype=np.uint8)
        for i, s in enumerate(seeds):
            self.lib.oracle_mt64_seed(st[i].ctypes.data, int(s))
        return st

    def next_word(self, rng_state_row: np.ndarray) -> int:
        return int(self.lib.oracle_mt64_next(rng_state_row.ctypes.data))

    def canonical(self, word: int) -> float:
        return float(self.lib.oracle_canonical(int(word)))

    def softcap(self, logits: np.ndarray, cap: float) -> None:
        assert logits.dtype == np.float32 and logits.flags.c_contiguous
        self.lib.oracle_softcap(logits.ctypes.data, logits.size, float(cap))

    # --- batches
    def sample_rows(self, params: np.ndarray, rngs: np.ndarray, logits: np.ndarray, hists, cap: int = 0):
        """Independent rows.  logits [B][V] float32 is MODIFIED in place (as the reference does).
        Returns dict(tokens, n_keep, kept_ids, kept_pr, rng_words, r_tot)."""
        assert logits.dtype == np.float32 and logits.ndim == 2 and logits.flags.c_contiguous
        B, V = logits.shape
        assert params.dtype == PARAMS_DTYPE and len(params) == B
        flat, off = flatten_hist(hists)
        tokens = np.zeros(B, dtype=np.int32)
        n_keep = np.zeros(B, dtype=np.int32)
        words = np.zeros(B, dtype=np.uint64)
        r_tot = np.zeros((B, 3), dtype=np.float64)   # r, tot, probability of the last kept candidate
        kept_ids = np.full((B, max(cap, 1)), -1, dtype=np.int32)
        kept_pr = np.zeros((B, max(cap, 1)), dtype=np.float64)
        rc = self.lib.oracle_sample_rows(B, params.ctypes.data, rngs.ctypes.data, logits.ctypes.data, V, V,
                                         flat.ctypes.data, off.ctypes.data, tokens.ctypes.data,
                                         kept_ids.ctypes.data if cap else None, kept_pr.ctypes.data if cap else None, cap,
                                         n_keep.ctypes.data, words.ctypes.data, r_tot.ctypes.data)
        if rc != 0:
            raise MemoryError("oracle_sample_rows")
        return dict(tokens=tokens, n_keep=n_keep, kept_ids=kept_ids, kept_pr=kept_pr, rng_words=words, r_tot=r_tot)

    def verify_window(self, params_row: np.ndarray, rng_row: np.ndarray, logits: np.ndarray, rows, hist):
        """One stream's verification window.  logits [m][V] modified in place.
        Returns (tokens[m] with -1 for rows not sampled, acc, confirmed, new_history)."""
        m, V = logits.shape
        rows = np.asarray(rows, dtype=np.int32)
        h = np.zeros(len(hist) + m + 1, dtype=np.int32)
        h[:len(hist)] = hist
        tokens = np.full(m, -1, dtype=np.int32)
        conf = C.c_int(0)
        acc = self.lib.oracle_verify_window(params_row.ctypes.data, rng_row.ctypes.data, logits.ctypes.data, V, V, m,
                                            rows.ctypes.data, h.ctypes.data, len(hist), tokens.ctypes.data, C.byref(conf))
        if acc < 0:
            raise MemoryError("oracle_verify_window")
        return tokens, acc, conf.value, h[:len(hist) + acc].copy()


class RefLib:
    """The unmodified reference sampler.  ``RefLib.available()`` tells whether it was built."""

    @staticmethod
    def path():
        return _build.build_ref()

    @staticmethod
    def available() -> bool:
        p = RefLib.path()
        return p is not None and os.path.exists(p)

    def __init__(self):
        p = self.path()
        if p is None:
            raise FileNotFoundError("reference sampler library was not built (no reference checkout on this machine)")
        self.lib = C.CDLL(p)
        L = self.lib
        L.ref_sampler_new.restype = C.c_void_p
        L.ref_sampler_new.argtypes = [C.c_void_p]
        L.ref_sampler_free.argtypes = [C.c_void_p]
        L.ref_sampler_sample.restype = C.c_int
        L.ref_sampler_sample.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int64]
        L.ref_sample_rows.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        L.ref_sample_repeat.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int64, C.c_int, C.c_void_p]
        L.ref_verify_window.restype = C.c_int
        L.ref_verify_window.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int64,
                                        C.c_void_p, C.c_void_p]
        L.ref_time_rows.restype = C.c_double
        L.ref_time_rows.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        assert L.ref_sizeof_params() == 40

    def sample_rows(self, params, logits, hists):
        B, V = logits.shape
        flat, off = flatten_hist(hists)
        tokens = np.zeros(B, dtype=np.int32)
        self.lib.ref_sample_rows(B, params.ctypes.data, logits.ctypes.data, V, V, flat.ctypes.data, off.ctypes.data,
                                 tokens.ctypes.data)
        return tokens

    def sample_repeat(self, params_row, logits_row, hist, n_draws):
        hist = np.ascontiguousarray(hist, dtype=np.int32)
        tokens = np.zeros(n_draws, dtype=np.int32)
        self.lib.ref_sample_repeat(params_row.ctypes.data, logits_row.ctypes.data, logits_row.shape[-1],
                                   hist.ctypes.data, len(hist), n_draws, tokens.ctypes.data)
        return tokens

    def verify_window(self, params_row, logits, rows, hist):
        m, V = logits.shape
        rows = np.asarray(rows, dtype=np.int32)
        hist = np.ascontiguousarray(hist, dtype=np.int32)
        tokens = np.full(m, -1, dtype=np.int32)
        conf = C.c_int(0)
        s = self.lib.ref_sampler_new(params_row.ctypes.data)
        try:
            acc = self.lib.ref_verify_window(s, logits.ctypes.data, V, V, m, rows.ctypes.data, hist.ctypes.data, len(hist),
                                             tokens.ctypes.data, C.byref(conf))
        finally:
            self.lib.ref_sampler_free(s)
        return tokens, acc, conf.value

    def time_rows(self, params, logits, hists, n_threads):
        B, V = logits.shape
        flat, off = flatten_hist(hists)
        tokens = np.zeros(B, dtype=np.int32)
        secs = self.lib.ref_time_rows(B, params.ctypes.data, logits.ctypes.data, V, V, flat.ctypes.data, off.ctypes.data,
                                      tokens.ctypes.data, int(n_threads))
        return float(secs), tokens

    def hardware_threads(self) -> int:
        return int(self.lib.ref_hardware_threads())
