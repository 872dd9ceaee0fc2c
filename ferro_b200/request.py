"""Request fields and command-line flags -> sampling parameters: a binding of the C ABI's front end.

``fsb_params_from_request`` and ``fsb_params_apply_cli_flag`` (ferro_b200/csrc/fsb_request.cpp) restate what
paragontasx/ferro's chat-completion handler does before it constructs a sampler (src/server.cpp:1060-1072), the
server options that feed it (src/server.h:35-37) and the flags of the binary (src/main.cpp:250-262); a C++ server
calls them directly.  This module only marshals a decoded JSON body into ``fsb_request_fields``:

* a field is used only if it is a JSON number (an integer or a float; strings, booleans and null fall back to the
  default, as the reference's ``jnum`` does); ``penalize_prompt`` only if it is a JSON boolean;
* everything else - aliases, server defaults, ``penalty_from``, the range errors - happens in the C function.

``min_p`` is not range-checked by the reference; the C ABI additionally wants 0 <= min_p <= 1 (fsb_params_validate)
and reports that when the stream is opened.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

_FIELDS = ["temperature", "top_p", "top_k", "min_p", "repetition_penalty", "repeat_penalty", "repeat_last_n", "penalty_last_n"]
_BITS = {name: 1 << i for i, name in enumerate(_FIELDS)}
_BITS["penalize_prompt"] = 1 << 8
_BITS["seed"] = 1 << 9


class _RequestFields(C.Structure):      # fsb_request_fields
    _fields_ = [("present", C.c_uint32), ("penalize_prompt", C.c_int32)] + [(n, C.c_double) for n in _FIELDS + ["seed"]]


class _ServerDefaults(C.Structure):     # fsb_server_defaults
    _fields_ = [("repeat_penalty", C.c_float), ("repeat_last_n", C.c_int32), ("penalize_prompt", C.c_int32)]


class BadRequest(ValueError):
    """The reference answers HTTP 400 with this text."""


@dataclass
class ServerDefaults:
    """The server options that act as per-request defaults (src/server.h:35-37)."""
    repeat_penalty: float = 0.0       # <= 0: the sampler's own default, 1.05
    repeat_last_n: int = -1
    penalize_prompt: bool = True

    def _c(self) -> _ServerDefaults:
        return _ServerDefaults(self.repeat_penalty, self.repeat_last_n, 1 if self.penalize_prompt else 0)


def params_from_request(body: dict, prompt_tokens: int = 0, defaults: ServerDefaults | None = None) -> np.ndarray:
    """One-row parameter record (``ferro_b200.PARAMS_DTYPE`` layout = ``ferro_sampler_params``) for a request body."""
    from . import PARAMS_DTYPE, load_library
    f = _RequestFields()
    for name in _FIELDS + ["seed"]:
        v = body.get(name)
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            continue
        f.present |= _BITS[name]
        setattr(f, name, float(v))
    if isinstance(body.get("penalize_prompt"), bool):
        f.present |= _BITS["penalize_prompt"]
        f.penalize_prompt = 1 if body["penalize_prompt"] else 0
    d = (defaults or ServerDefaults())._c()
    p = np.zeros(1, dtype=PARAMS_DTYPE)
    rc = load_library().fsb_params_from_request(C.byref(f), C.byref(d), int(prompt_tokens), p.ctypes.data)
    if rc == -2:
        raise BadRequest("sampling parameter out of range")
    if rc != 0:
        raise ValueError(f"fsb_params_from_request failed with {rc}")
    return p


def apply_cli_flags(argv, params: np.ndarray | None = None, defaults: ServerDefaults | None = None):
    """Walks `argv` as the reference's binary does (src/main.cpp:250-262) and applies the sampling flags.
    Returns (params record, ServerDefaults, the arguments that are not sampling flags)."""
    from . import make_params, load_library
    lib = load_library()
    p = make_params(1) if params is None else params.copy()
    d = (defaults or ServerDefaults())._c()
    rest, i = [], 0
    while i < len(argv):
        value = argv[i + 1] if i + 1 < len(argv) else None
        rc = lib.fsb_params_apply_cli_flag(p.ctypes.data, C.byref(d), argv[i].encode(), value.encode() if value is not None else None)
        if rc == 1:
            i += 2
        elif rc == 0:
            rest.append(argv[i])
            i += 1
        else:
            raise BadRequest(f"bad value for {argv[i]}")
    return p, ServerDefaults(float(d.repeat_penalty), int(d.repeat_last_n), bool(d.penalize_prompt)), rest
