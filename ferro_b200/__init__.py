"""ferro_b200 - B200-native batched token sampler behind the interface of ferro's ``Sampler``.

The product is the C-ABI shared library built from ``ferro_b200/csrc`` (hand-written sm_100a CUDA kernels plus
a C++ host shim; no PyTorch inside).  This module is a thin ctypes binding used by the tests and the benchmark:

* :class:`Engine`   - one sampler engine on one CUDA device (``fsb_create``), batched calls;
* :class:`Sampler`  - the reference's class shape: ``Sampler(params).sample(logits, n_vocab, history)``
  (``src/sampler.h:23-29`` of paragontasx/ferro), one row per call, for tests that read like the reference's;
* :func:`make_params` - numpy records laid out as the reference's 40-byte ``SamplerParams``.

There is no CPU fallback: if the library is missing it is built with nvcc, and without a CUDA device
``Engine()`` raises.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import _build

__all__ = ["Engine", "Sampler", "Batch", "SamplerError", "make_params", "PARAMS_DTYPE", "load_library", "library_path",
           "LOGITS_ON_HOST", "WRITE_BACK", "KEEP_KEPT_SET", "MAX_CANDIDATE_K", "API_SYMBOLS"]

LOGITS_ON_HOST = 1
WRITE_BACK = 2
KEEP_KEPT_SET = 4
APPEND_SAMPLED = 8
MAX_CANDIDATE_K = 256
STATIC_MAX_ROWS = 64   # FSB_STATIC_MAX_ROWS
STATIC_WAIT = 1        # FSB_STATIC_WAIT

PARAMS_DTYPE = np.dtype(
    {
        "names": ["temperature", "top_k", "top_p", "min_p", "repetition_penalty", "repeat_last_n", "penalty_from", "seed"],
        "formats": [np.float32, np.int32, np.float32, np.float32, np.float32, np.int32, np.int32, np.uint64],
        "offsets": [0, 4, 8, 12, 16, 20, 24, 32],
        "itemsize": 40,
    }
)

API_SYMBOLS = [
    "fsb_create", "fsb_destroy", "fsb_last_error", "fsb_set_cuda_stream", "fsb_set_softcap", "fsb_set_vocab_offset", "fsb_set_launch_overlap", "fsb_batch_shard_launch", "fsb_batch_merge_launch", "fsb_argmax_rows_static", "fsb_stream_history_set", "fsb_stream_history_append", "fsb_stream_history_len",
    "fsb_sample_batch_resident",
    "fsb_set_trace_buffer", "fsb_set_vocab_shard", "fsb_batch_max_k", "fsb_batch_shard_launch_packed", "fsb_batch_merge_launch_packed",
    "fsb_batch_tokens_device", "fsb_batch_check", "fsb_lookup_drafts_resident", "fsb_verify_windows_resident",
    "fsb_server_defaults_init", "fsb_params_from_request", "fsb_params_apply_cli_flag",
    "fsb_params_default", "fsb_params_validate", "fsb_stream_open", "fsb_stream_close", "fsb_stream_params",
    "fsb_stream_state_get", "fsb_stream_state_set", "fsb_sample_batch", "fsb_verify_windows", "fsb_last_kept",
    "fsb_batch_prepare", "fsb_batch_redraw", "fsb_batch_launch", "fsb_batch_tokens", "fsb_batch_kernel_count",
    "fsb_batch_free", "fsb_counters",
]

STATUS_NAMES = {0: "FSB_OK", -1: "FSB_ERR_INVALID", -2: "FSB_ERR_RANGE", -3: "FSB_ERR_CAPACITY", -4: "FSB_ERR_CUDA",
                -5: "FSB_ERR_STREAM_ID", -6: "FSB_ERR_NO_DEVICE", -7: "FSB_ERR_DEVICE"}


class SamplerError(RuntimeError):
    def __init__(self, code: int, text: str = ""):
        self.code = code
        super().__init__(f"{STATUS_NAMES.get(code, code)}: {text}")


class _Counters(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("rows_sampled", "rows_greedy", "rows_stochastic", "rows_full_vocab", "drafted",
                                           "accepted", "kernel_launches")]


_lib = None


def library_path() -> str:
    return _build.LIB_PATH


def load_library(build_if_missing: bool = True):
    """Load (building first if needed) the C-ABI library.  Never falls back to anything else."""
    global _lib
    if _lib is not None:
        return _lib
    if build_if_missing:
        _build.build()
    if not os.path.exists(_build.LIB_PATH):
        raise FileNotFoundError(f"{_build.LIB_PATH} is missing: build it with `python -m ferro_b200._build`")
    L = C.CDLL(_build.LIB_PATH)
    vp, i32, i64, u32, u64 = C.c_void_p, C.c_int, C.c_int64, C.c_uint, C.c_uint64
    L.fsb_create.argtypes = [i32, i32, i32, i64, C.POINTER(vp)]
    L.fsb_destroy.argtypes = [vp]
    L.fsb_last_error.argtypes = [vp]
    L.fsb_last_error.restype = C.c_char_p
    L.fsb_set_cuda_stream.argtypes = [vp, vp]
    L.fsb_set_softcap.argtypes = [vp, C.c_float]
    L.fsb_set_vocab_offset.argtypes = [vp, C.c_int32]
    L.fsb_set_launch_overlap.argtypes = [vp, C.c_int]
    L.fsb_set_trace_buffer.argtypes = [vp, vp]
    L.fsb_set_vocab_shard.argtypes = [vp, C.c_int32, C.c_int32]
    L.fsb_verify_windows_resident.argtypes = [vp, i32, vp, vp, vp, vp, i64, i32, vp, vp, vp, vp, u32]
    L.fsb_params_default.argtypes = [vp]
    L.fsb_params_default.restype = None
    L.fsb_server_defaults_init.argtypes = [vp]
    L.fsb_server_defaults_init.restype = None
    L.fsb_params_from_request.argtypes = [vp, vp, C.c_int32, vp]
    L.fsb_params_apply_cli_flag.argtypes = [vp, vp, C.c_char_p, C.c_char_p]
    L.fsb_params_validate.argtypes = [vp]
    L.fsb_stream_open.argtypes = [vp, vp, C.POINTER(i32)]
    L.fsb_stream_close.argtypes = [vp, i32]
    L.fsb_stream_params.argtypes = [vp, i32, vp]
    L.fsb_stream_state_get.argtypes = [vp, i32, C.POINTER(u64), C.POINTER(u64)]
    L.fsb_stream_state_set.argtypes = [vp, i32, u64, u64]
    L.fsb_sample_batch.argtypes = [vp, i32, vp, vp, i64, i32, vp, vp, vp, u32]
    L.fsb_verify_windows.argtypes = [vp, i32, vp, vp, vp, vp, i64, i32, vp, vp, vp, vp, vp, vp, u32]
    L.fsb_last_kept.argtypes = [vp, i32, i32, vp, vp, C.POINTER(i32)]
    L.fsb_batch_prepare.argtypes = [vp, i32, vp, i64, i32, vp, vp, u32, C.POINTER(vp)]
    L.fsb_batch_redraw.argtypes = [vp, vp]
    L.fsb_batch_launch.argtypes = [vp, vp, vp]
    L.fsb_batch_tokens.argtypes = [vp, vp, vp]
    L.fsb_batch_shard_launch.argtypes = [vp, vp, vp, vp, vp]
    L.fsb_batch_merge_launch.argtypes = [vp, vp, vp, vp, i32]
    L.fsb_batch_max_k.argtypes = [vp]
    L.fsb_batch_shard_launch_packed.argtypes = [vp, vp, vp, vp, i32]
    L.fsb_batch_merge_launch_packed.argtypes = [vp, vp, vp, i32, i32, i32, i32]
    L.fsb_batch_tokens_device.argtypes = [vp]
    L.fsb_batch_tokens_device.restype = vp
    L.fsb_batch_check.argtypes = [vp, vp]
    L.fsb_lookup_drafts_resident.argtypes = [vp, i32, vp, vp, vp, i32, vp, i32, vp]
    L.fsb_batch_kernel_count.argtypes = [vp]
    L.fsb_batch_free.argtypes = [vp, vp]
    L.fsb_counters.argtypes = [vp, C.POINTER(_Counters)]
    L.fsb_stream_history_set.argtypes = [vp, i32, vp, i64]
    L.fsb_stream_history_append.argtypes = [vp, i32, vp, i32]
    L.fsb_stream_history_len.argtypes = [vp, i32, C.POINTER(i64)]
    L.fsb_sample_batch_resident.argtypes = [vp, i32, vp, vp, i64, i32, vp, u32]
    L.fsb_argmax_rows_static.argtypes = [C.c_int, vp, i64, i32, i32, vp, vp, u32]
    for name in API_SYMBOLS:
        if name not in ("fsb_last_error", "fsb_params_default", "fsb_server_defaults_init", "fsb_batch_tokens_device"):
            getattr(L, name).restype = i32
    _lib = L
    return L


def make_params(n: int = 1, **kw) -> np.ndarray:
    """n parameter records with the reference's defaults (src/sampler.h:13-20), overridden by keyword."""
    p = np.zeros(n, dtype=PARAMS_DTYPE)
    L = load_library()
    for i in range(n):
        L.fsb_params_default(p[i:i + 1].ctypes.data)
    for k, v in kw.items():
        p[k] = v
    return p


def _flatten_hist(hists):
    off = np.zeros(len(hists) + 1, dtype=np.int64)
    for i, h in enumerate(hists):
        off[i + 1] = off[i] + len(h)
    flat = np.zeros(max(int(off[-1]), 1), dtype=np.int32)
    for i, h in enumerate(hists):
        if len(h):
            flat[off[i]:off[i + 1]] = np.asarray(h, dtype=np.int32)
    return flat, off


def _logits_pointer(logits, n_rows, n_vocab, flags):
    """Accepts a numpy array (host), an int device pointer, or any object with ``data_ptr()`` (device tensor)."""
    if isinstance(logits, np.ndarray):
        if logits.dtype != np.float32:
            raise TypeError("logits must be float32")
        if logits.ndim == 1:
            logits = logits.reshape(1, -1)
        if logits.strides[-1] != 4 or logits.strides[0] % 4:
            raise ValueError("logits rows must be contiguous")
        return logits.ctypes.data, logits.strides[0] // 4, flags | LOGITS_ON_HOST, logits
    if hasattr(logits, "data_ptr"):
        ld = logits.stride(0) if logits.dim() == 2 else n_vocab
        return int(logits.data_ptr()), int(ld), flags & ~LOGITS_ON_HOST, logits
    raise TypeError("logits: numpy array or device tensor expected")


class Batch:
    """A prepared device-resident batch (``fsb_batch_prepare``): launch it on any device logits buffer."""

    def __init__(self, engine: "Engine", ptr, n_rows: int):
        self.engine, self._ptr, self.n_rows = engine, ptr, n_rows

    def redraw(self):
        self.engine._check(self.engine.lib.fsb_batch_redraw(self.engine._h, self._ptr))

    def launch(self, logits_dev_ptr: int):
        self.engine._check(self.engine.lib.fsb_batch_launch(self.engine._h, self._ptr, C.c_void_p(int(logits_dev_ptr))))

    def shard_launch(self, logits_shard_dev_ptr: int, lists_out_dev_ptr: int, counts_out_dev_ptr: int):
        """Vocabulary-sharded first half: this device's best k candidates per row (``fsb_batch_shard_launch``)."""
        self.engine._check(self.engine.lib.fsb_batch_shard_launch(self.engine._h, self._ptr, C.c_void_p(int(logits_shard_dev_ptr)),
                                                                  C.c_void_p(int(lists_out_dev_ptr)), C.c_void_p(int(counts_out_dev_ptr))))

    def merge_launch(self, lists_dev_ptr: int, counts_dev_ptr: int, n_lists: int):
        """Vocabulary-sharded second half: merge the gathered lists of all shards and finish the rows."""
        self.engine._check(self.engine.lib.fsb_batch_merge_launch(self.engine._h, self._ptr, C.c_void_p(int(lists_dev_ptr)),
                                                                  C.c_void_p(int(counts_dev_ptr)), int(n_lists)))

    @property
    def max_k(self) -> int:
        """Largest candidate count of the staged rows (on this shard): a packed list needs max_k + 1 words."""
        return int(self.engine.lib.fsb_batch_max_k(self._ptr))

    def shard_launch_packed(self, logits_shard_dev_ptr: int, packed_out_dev_ptr: int, stride_words: int):
        """``fsb_batch_shard_launch_packed``: per row [count, candidates ...] in `stride_words` 64-bit words."""
        self.engine._check(self.engine.lib.fsb_batch_shard_launch_packed(self.engine._h, self._ptr, C.c_void_p(int(logits_shard_dev_ptr)),
                                                                         C.c_void_p(int(packed_out_dev_ptr)), int(stride_words)))

    def merge_launch_packed(self, packed_dev_ptr: int, stride_words: int, n_lists: int, row_begin: int, n_rows: int):
        """``fsb_batch_merge_launch_packed``: finish rows [row_begin, row_begin + n_rows) from [n_lists][n_rows][stride_words]."""
        self.engine._check(self.engine.lib.fsb_batch_merge_launch_packed(self.engine._h, self._ptr, C.c_void_p(int(packed_dev_ptr)), int(stride_words),
                                                                         int(n_lists), int(row_begin), int(n_rows)))

    @property
    def tokens_device_ptr(self) -> int:
        """Device address of the batch's token array ([rows] int32, indexed by row)."""
        return int(self.engine.lib.fsb_batch_tokens_device(self._ptr))

    def check(self):
        """Waits for the batch's launches and raises if the device reported an error."""
        self.engine._check(self.engine.lib.fsb_batch_check(self.engine._h, self._ptr))

    def tokens(self) -> np.ndarray:
        out = np.zeros(self.n_rows, dtype=np.int32)
        self.engine._check(self.engine.lib.fsb_batch_tokens(self.engine._h, self._ptr, out.ctypes.data))
        return out

    @property
    def kernels_per_launch(self) -> int:
        return int(self.engine.lib.fsb_batch_kernel_count(self._ptr))

    def free(self):
        if self._ptr:
            self.engine.lib.fsb_batch_free(self.engine._h, self._ptr)
            self._ptr = None


class Engine:
    """One sampler engine on one CUDA device."""

    def __init__(self, device: int = 0, max_rows: int = 512, max_vocab: int = 262144, max_hist_ids: int = 1 << 20):
        self.lib = load_library()
        h = C.c_void_p()
        rc = self.lib.fsb_create(device, max_rows, max_vocab, max_hist_ids, C.byref(h))
        if rc != 0:
            raise SamplerError(rc, "fsb_create failed (a CUDA device of compute capability 10.x is required; there is no CPU path)")
        self._h = h
        self.max_rows, self.max_vocab = max_rows, max_vocab

    # -- plumbing
    def _check(self, rc: int):
        if rc != 0:
            raise SamplerError(rc, (self.lib.fsb_last_error(self._h) or b"").decode())

    def close(self):
        if getattr(self, "_h", None):
            self.lib.fsb_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_cuda_stream(self, stream_ptr: int):
        self._check(self.lib.fsb_set_cuda_stream(self._h, C.c_void_p(int(stream_ptr))))

    def set_softcap(self, cap: float):
        self._check(self.lib.fsb_set_softcap(self._h, float(cap)))

    def set_trace_buffer(self, device_ptr: int):
        self._check(self.lib.fsb_set_trace_buffer(self._h, C.c_void_p(int(device_ptr)) if device_ptr else None))

    def set_launch_overlap(self, mode):
        """0 / False: plain stream order; 1 / True: consecutive launches overlap their reads; 2: launch latency hidden,
        plain-order semantics (see fsb_set_launch_overlap in the C header)."""
        self._check(self.lib.fsb_set_launch_overlap(self._h, int(mode)))

    def set_vocab_offset(self, offset: int):
        self._check(self.lib.fsb_set_vocab_offset(self._h, int(offset)))

    def set_vocab_shard(self, offset: int, global_vocab: int):
        """This engine holds columns [offset, offset + n_vocab) of rows that are `global_vocab` columns wide."""
        self._check(self.lib.fsb_set_vocab_shard(self._h, int(offset), int(global_vocab)))

    # -- streams
    def open_stream(self, params) -> int:
        p = np.ascontiguousarray(np.asarray(params, dtype=PARAMS_DTYPE).reshape(-1)[:1])
        sid = C.c_int(-1)
        self._check(self.lib.fsb_stream_open(self._h, p.ctypes.data, C.byref(sid)))
        return sid.value

    def open_streams(self, params) -> np.ndarray:
        return np.array([self.open_stream(params[i:i + 1]) for i in range(len(params))], dtype=np.int32)

    def close_stream(self, sid: int):
        self._check(self.lib.fsb_stream_close(self._h, int(sid)))

    def stream_params(self, sid: int) -> np.ndarray:
        p = np.zeros(1, dtype=PARAMS_DTYPE)
        self._check(self.lib.fsb_stream_params(self._h, int(sid), p.ctypes.data))
        return p

    def stream_state(self, sid: int):
        seed, draws = C.c_uint64(0), C.c_uint64(0)
        self._check(self.lib.fsb_stream_state_get(self._h, int(sid), C.byref(seed), C.byref(draws)))
        return seed.value, draws.value

    def set_stream_state(self, sid: int, seed: int, draws: int):
        self._check(self.lib.fsb_stream_state_set(self._h, int(sid), int(seed), int(draws)))

    # -- sampling
    def sample_batch(self, stream_ids, logits, histories, n_vocab: int | None = None, flags: int = 0) -> np.ndarray:
        sids = np.ascontiguousarray(stream_ids, dtype=np.int32)
        n_rows = len(sids)
        if n_vocab is None:
            n_vocab = int(logits.shape[-1])
        ptr, ld, flags, keep = _logits_pointer(logits, n_rows, n_vocab, flags)
        flat, off = _flatten_hist(histories)
        tokens = np.zeros(n_rows, dtype=np.int32)
        self._check(self.lib.fsb_sample_batch(self._h, n_rows, sids.ctypes.data, C.c_void_p(ptr), ld, n_vocab, flat.ctypes.data,
                                              off.ctypes.data, tokens.ctypes.data, flags))
        return tokens

    def verify_windows(self, stream_ids, rows, logits, histories, n_vocab: int | None = None, max_accept=None, flags: int = 0):
        """rows: per stream [last token, draft_1, ...].  Returns (tokens[list of arrays], acc, confirmed)."""
        sids = np.ascontiguousarray(stream_ids, dtype=np.int32)
        n_streams = len(sids)
        row_off = np.zeros(n_streams + 1, dtype=np.int32)
        for i, r in enumerate(rows):
            row_off[i + 1] = row_off[i] + len(r)
        rows_flat = np.concatenate([np.asarray(r, dtype=np.int32) for r in rows]).astype(np.int32)
        n_rows = int(row_off[-1])
        if n_vocab is None:
            n_vocab = int(logits.shape[-1])
        ptr, ld, flags, keep = _logits_pointer(logits, n_rows, n_vocab, flags)
        flat, off = _flatten_hist(histories)
        tokens = np.zeros(n_rows, dtype=np.int32)
        acc = np.zeros(n_streams, dtype=np.int32)
        conf = np.zeros(n_streams, dtype=np.int32)
        ma = np.ascontiguousarray(max_accept, dtype=np.int32) if max_accept is not None else None
        self._check(self.lib.fsb_verify_windows(self._h, n_streams, sids.ctypes.data, row_off.ctypes.data, rows_flat.ctypes.data,
                                                C.c_void_p(ptr), ld, n_vocab, flat.ctypes.data, off.ctypes.data,
                                                ma.ctypes.data if ma is not None else None, tokens.ctypes.data, acc.ctypes.data,
                                                conf.ctypes.data, flags))
        return [tokens[row_off[i]:row_off[i + 1]] for i in range(n_streams)], acc, conf

    def verify_windows_resident(self, stream_ids, rows, logits, n_vocab: int | None = None, max_accept=None, flags: int = 0):
        """``verify_windows`` with the streams' resident histories; with APPEND_SAMPLED the accepted tokens are appended."""
        sids = np.ascontiguousarray(stream_ids, dtype=np.int32)
        n_streams = len(sids)
        row_off = np.zeros(n_streams + 1, dtype=np.int32)
        for i, r in enumerate(rows):
            row_off[i + 1] = row_off[i] + len(r)
        rows_flat = np.concatenate([np.asarray(r, dtype=np.int32) for r in rows]).astype(np.int32)
        n_rows = int(row_off[-1])
        if n_vocab is None:
            n_vocab = int(logits.shape[-1])
        ptr, ld, flags, keep = _logits_pointer(logits, n_rows, n_vocab, flags)
        tokens = np.zeros(n_rows, dtype=np.int32)
        acc = np.zeros(n_streams, dtype=np.int32)
        conf = np.zeros(n_streams, dtype=np.int32)
        ma = np.ascontiguousarray(max_accept, dtype=np.int32) if max_accept is not None else None
        self._check(self.lib.fsb_verify_windows_resident(self._h, n_streams, sids.ctypes.data, row_off.ctypes.data, rows_flat.ctypes.data,
                                                         C.c_void_p(ptr), ld, n_vocab, ma.ctypes.data if ma is not None else None,
                                                         tokens.ctypes.data, acc.ctypes.data, conf.ctypes.data, flags))
        return [tokens[row_off[i]:row_off[i + 1]] for i in range(n_streams)], acc, conf

    def last_kept(self, row: int, cap: int = MAX_CANDIDATE_K):
        ids = np.zeros(cap, dtype=np.int32)
        pr = np.zeros(cap, dtype=np.float64)
        n = C.c_int(0)
        self._check(self.lib.fsb_last_kept(self._h, int(row), cap, ids.ctypes.data, pr.ctypes.data, C.byref(n)))
        m = min(n.value, cap)
        return ids[:m], pr[:m], n.value

    # ---- device-resident histories (fsb_stream_history_*, fsb_sample_batch_resident)
    def history_set(self, stream_id: int, ids):
        a = np.ascontiguousarray(ids, dtype=np.int32)
        self._check(self.lib.fsb_stream_history_set(self._h, int(stream_id), a.ctypes.data, len(a)))

    def history_append(self, stream_id: int, ids):
        a = np.ascontiguousarray(np.atleast_1d(ids), dtype=np.int32)
        self._check(self.lib.fsb_stream_history_append(self._h, int(stream_id), a.ctypes.data, len(a)))

    def lookup_drafts(self, stream_ids, kmax, min_n, eos: int):
        """Prompt-lookup drafts of resident histories (``fsb_lookup_drafts_resident``): a list of int32 arrays."""
        sids = np.ascontiguousarray(stream_ids, dtype=np.int32)
        n = len(sids)
        km = np.ascontiguousarray(np.broadcast_to(np.asarray(kmax, dtype=np.int32), (n,)))
        mn = np.ascontiguousarray(np.broadcast_to(np.asarray(min_n, dtype=np.int32), (n,)))
        stride = max(int(km.max()) if n else 1, 1)
        out = np.zeros((n, stride), dtype=np.int32)
        cnt = np.zeros(n, dtype=np.int32)
        self._check(self.lib.fsb_lookup_drafts_resident(self._h, n, sids.ctypes.data, km.ctypes.data, mn.ctypes.data, int(eos), out.ctypes.data,
                                                        stride, cnt.ctypes.data))
        return [out[i, : cnt[i]].copy() for i in range(n)]

    def history_len(self, stream_id: int) -> int:
        n = C.c_int64(0)
        self._check(self.lib.fsb_stream_history_len(self._h, int(stream_id), C.byref(n)))
        return int(n.value)

    def sample_batch_resident(self, stream_ids, logits, n_vocab: int | None = None, ld: int | None = None, flags: int = 0) -> np.ndarray:
        """``fsb_sample_batch`` with every row's history taken from its stream's resident history.  `logits` is a
        host float32 array (FSB_LOGITS_ON_HOST is added) or an int device pointer (then n_vocab is required)."""
        sids = np.ascontiguousarray(stream_ids, dtype=np.int32)
        if isinstance(logits, np.ndarray):
            assert logits.dtype == np.float32 and logits.ndim == 2 and logits.flags.c_contiguous
            n_vocab = logits.shape[1] if n_vocab is None else n_vocab
            ld = logits.shape[1] if ld is None else ld
            ptr, flags = logits.ctypes.data, flags | LOGITS_ON_HOST
        else:
            ptr, ld = int(logits), (n_vocab if ld is None else ld)
        out = np.zeros(len(sids), dtype=np.int32)
        self._check(self.lib.fsb_sample_batch_resident(self._h, len(sids), sids.ctypes.data, C.c_void_p(ptr), ld, n_vocab, out.ctypes.data, flags))
        return out

    def prepare_batch(self, stream_ids, histories, n_vocab: int, ld: int | None = None, flags: int = 0) -> Batch:
        sids = np.ascontiguousarray(stream_ids, dtype=np.int32)
        flat, off = _flatten_hist(histories)
        b = C.c_void_p()
        self._check(self.lib.fsb_batch_prepare(self._h, len(sids), sids.ctypes.data, ld if ld is not None else n_vocab, n_vocab,
                                               flat.ctypes.data, off.ctypes.data, flags, C.byref(b)))
        return Batch(self, b, len(sids))

    def counters(self) -> dict:
        c = _Counters()
        self._check(self.lib.fsb_counters(self._h, C.byref(c)))
        return {n: int(getattr(c, n)) for n, _ in _Counters._fields_}


_default_engines: dict = {}


def argmax_rows_static(logits_dev_ptr: int, ld: int, n_rows: int, n_vocab: int, tokens_dev_ptr: int, device: int = 0,
                       cuda_stream: int = 0, wait: bool = True) -> None:
    """Greedy tokens of device rows through ``fsb_argmax_rows_static``: no handle and no allocation; at most
    ``STATIC_MAX_ROWS`` rows; all calls on a device share one scratch array (see the C header)."""
    rc = load_library().fsb_argmax_rows_static(int(device), C.c_void_p(int(logits_dev_ptr)), int(ld), int(n_rows), int(n_vocab),
                                               C.c_void_p(int(tokens_dev_ptr)), C.c_void_p(int(cuda_stream)), STATIC_WAIT if wait else 0)
    if rc != 0:
        raise SamplerError(rc, f"fsb_argmax_rows_static: {STATUS_NAMES.get(rc, rc)}")


def default_engine(device: int = 0) -> Engine:
    if device not in _default_engines:
        _default_engines[device] = Engine(device=device)
    return _default_engines[device]


class Sampler:
    """The reference's class shape (src/sampler.h:23-29): one stream, one row per call.

    ``sample(logits, n_vocab, history)`` takes a host float32 row, modifies it in place as the reference does
    (the penalised entries), and returns the token id.
    """

    def __init__(self, params, engine: Engine | None = None):
        self.engine = engine or default_engine()
        self._sid = self.engine.open_stream(params)

    def sample(self, logits: np.ndarray, n_vocab: int, history) -> int:
        row = logits.reshape(1, -1)[:, :n_vocab] if logits.shape[-1] != n_vocab else logits.reshape(1, -1)
        tok = self.engine.sample_batch([self._sid], row, [np.asarray(history, dtype=np.int32)], n_vocab=n_vocab, flags=WRITE_BACK)
        return int(tok[0])

    def params(self) -> np.ndarray:
        return self.engine.stream_params(self._sid)

    def close(self):
        if self._sid is not None:
            self.engine.close_stream(self._sid)
            self._sid = None
