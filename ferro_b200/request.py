"""Request fields -> sampling parameters, with the reference server's defaults, aliases and range errors.

Mirrors what paragontasx/ferro's chat-completion handler does before it constructs a sampler
(src/server.cpp:1060-1072) and the server options that feed it (src/server.h:35-37, flags in src/main.cpp:249-251):

* a field is used only if it is a JSON number (an integer or a float; strings, booleans and null fall back to the
  default, as the reference's ``jnum`` does);
* ``repetition_penalty`` falls back to ``repeat_penalty``, then to the server default (``--repeat-penalty`` if
  positive), then to the struct default 1.05; ``repeat_last_n`` falls back to ``penalty_last_n``, then to the server
  default (``--repeat-last-n``, -1);
* ``penalize_prompt`` (a JSON boolean; server default ``--penalty-scope all``) = false sets ``penalty_from`` to the
  prompt length, so the penalty window never reaches into the prompt;
* ``seed`` defaults to 0 (= nondeterministic);
* temperature < 0, top_p outside (0, 1], top_k < 0, repetition_penalty <= 0 or repeat_last_n < -1 is a bad request.

``min_p`` is not range-checked by the reference; the C ABI additionally wants 0 <= min_p <= 1 (fsb_params_validate)
and reports that when the stream is opened.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


class BadRequest(ValueError):
    """The reference answers HTTP 400 with this text."""


@dataclass
class ServerDefaults:
    """The server options that act as per-request defaults (src/server.h:35-37)."""
    repeat_penalty: float = 0.0       # <= 0: the sampler's own default, 1.05
    repeat_last_n: int = -1
    penalize_prompt: bool = True


def _num(body: dict, key: str, default):
    v = body.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        return default
    return v


def params_from_request(body: dict, prompt_tokens: int = 0, defaults: ServerDefaults | None = None) -> np.ndarray:
    """One-row parameter record (``ferro_b200.PARAMS_DTYPE`` layout = ``ferro_sampler_params``) for a request body."""
    from . import make_params
    d = defaults or ServerDefaults()
    p = make_params(1)                                    # the struct defaults (src/sampler.h:13-20)
    f32 = np.float32
    temperature = f32(_num(body, "temperature", float(p["temperature"][0])))
    top_p = f32(_num(body, "top_p", float(p["top_p"][0])))
    top_k = int(_num(body, "top_k", int(p["top_k"][0])))
    min_p = f32(_num(body, "min_p", float(p["min_p"][0])))
    server_pen = d.repeat_penalty if d.repeat_penalty > 0 else float(p["repetition_penalty"][0])
    penalty = f32(_num(body, "repetition_penalty", _num(body, "repeat_penalty", server_pen)))
    last_n = int(_num(body, "repeat_last_n", _num(body, "penalty_last_n", d.repeat_last_n)))
    pen_prompt = d.penalize_prompt
    if isinstance(body.get("penalize_prompt"), bool):
        pen_prompt = body["penalize_prompt"]
    seed = _num(body, "seed", 0)
    if temperature < 0 or top_p <= 0 or top_p > 1 or top_k < 0 or penalty <= 0 or last_n < -1:
        raise BadRequest("sampling parameter out of range")
    p["temperature"], p["top_p"], p["top_k"], p["min_p"] = temperature, top_p, top_k, min_p
    p["repetition_penalty"], p["repeat_last_n"] = penalty, last_n
    p["penalty_from"] = 0 if pen_prompt else int(prompt_tokens)
    p["seed"] = np.uint64(int(seed) & 0xFFFFFFFFFFFFFFFF)
    return p
