"""Request-parameter front end against the behaviour of the reference's handler (src/server.cpp:1060-1072)."""
import numpy as np
import pytest

import ferro_b200 as fb
from ferro_b200.request import BadRequest, ServerDefaults, params_from_request


def test_empty_request_gives_the_struct_defaults():
    p = params_from_request({})
    d = fb.make_params(1)
    for f in ("temperature", "top_k", "top_p", "min_p", "repetition_penalty", "repeat_last_n", "penalty_from", "seed"):
        assert p[f][0] == d[f][0], f
    assert p["temperature"][0] == np.float32(0.05) and p["top_k"][0] == 50 and p["repetition_penalty"][0] == np.float32(1.05)


def test_aliases_and_server_defaults():
    assert params_from_request({"repeat_penalty": 1.3})["repetition_penalty"][0] == np.float32(1.3)
    assert params_from_request({"repeat_penalty": 1.3, "repetition_penalty": 1.2})["repetition_penalty"][0] == np.float32(1.2)
    assert params_from_request({}, defaults=ServerDefaults(repeat_penalty=1.15))["repetition_penalty"][0] == np.float32(1.15)
    assert params_from_request({"penalty_last_n": 64})["repeat_last_n"][0] == 64
    assert params_from_request({"penalty_last_n": 64, "repeat_last_n": 8})["repeat_last_n"][0] == 8
    assert params_from_request({}, defaults=ServerDefaults(repeat_last_n=128))["repeat_last_n"][0] == 128


def test_penalty_scope_and_seed():
    assert params_from_request({}, prompt_tokens=37)["penalty_from"][0] == 0
    assert params_from_request({"penalize_prompt": False}, prompt_tokens=37)["penalty_from"][0] == 37
    assert params_from_request({}, prompt_tokens=37, defaults=ServerDefaults(penalize_prompt=False))["penalty_from"][0] == 37
    assert params_from_request({"penalize_prompt": "no"}, prompt_tokens=37)["penalty_from"][0] == 0   # not a boolean: ignored
    assert params_from_request({"seed": 1234})["seed"][0] == 1234 and params_from_request({})["seed"][0] == 0


def test_non_numeric_fields_fall_back_like_jnum():
    p = params_from_request({"temperature": "0.7", "top_k": None, "top_p": True})
    assert p["temperature"][0] == np.float32(0.05) and p["top_k"][0] == 50 and p["top_p"][0] == np.float32(1.0)
    assert params_from_request({"temperature": 0})["temperature"][0] == 0.0


@pytest.mark.parametrize("body", [{"temperature": -0.1}, {"top_p": 0}, {"top_p": 1.01}, {"top_k": -1}, {"repetition_penalty": 0},
                                  {"repeat_last_n": -2}])
def test_out_of_range_is_a_bad_request(body):
    with pytest.raises(BadRequest):
        params_from_request(body)


def test_result_passes_the_c_abi_validation():
    lib = fb.load_library()
    p = params_from_request({"temperature": 0.7, "top_k": 40, "top_p": 0.95, "min_p": 0.05, "repeat_penalty": 1.1, "seed": 7}, prompt_tokens=5)
    assert lib.fsb_params_validate(p.ctypes.data) == 0


def test_command_line_flags_of_the_reference_binary():
    # src/main.cpp:250-262: --temp --top-k --top-p --min-p --rep-penalty --seed go to the generate parameters,
    # --repeat-penalty --repeat-last-n --penalty-scope to the server defaults (--repeat-last-n to both)
    from ferro_b200.request import apply_cli_flags
    argv = ["--temp", "0.7", "--top-k", "40", "--port", "8080", "--top-p", "0.9", "--min-p", "0.05", "--rep-penalty", "1.2", "--seed", "99",
            "--repeat-penalty", "1.15", "--repeat-last-n", "256", "--penalty-scope", "generated", "--quiet"]
    p, d, rest = apply_cli_flags(argv)
    assert p["temperature"][0] == np.float32(0.7) and p["top_k"][0] == 40 and p["top_p"][0] == np.float32(0.9)
    assert p["min_p"][0] == np.float32(0.05) and p["repetition_penalty"][0] == np.float32(1.2) and p["seed"][0] == 99
    assert p["repeat_last_n"][0] == 256
    assert d == ServerDefaults(repeat_penalty=np.float32(1.15), repeat_last_n=256, penalize_prompt=False)
    assert rest == ["--port", "8080", "--quiet"]
    # the server defaults then shape a request that names none of them
    q = params_from_request({}, prompt_tokens=11, defaults=d)
    assert q["repetition_penalty"][0] == np.float32(1.15) and q["repeat_last_n"][0] == 256 and q["penalty_from"][0] == 11
    with pytest.raises(BadRequest):
        apply_cli_flags(["--penalty-scope", "some"])
    with pytest.raises(BadRequest):
        apply_cli_flags(["--temp"])


def test_front_end_is_callable_from_c_without_an_engine():
    import ctypes as C
    lib = fb.load_library()
    from ferro_b200.request import _RequestFields, _ServerDefaults
    d = _ServerDefaults()
    lib.fsb_server_defaults_init(C.byref(d))
    assert (d.repeat_penalty, d.repeat_last_n, d.penalize_prompt) == (0.0, -1, 1)
    f = _RequestFields()
    f.present = (1 << 5) | (1 << 9)          # repeat_penalty (the alias) and seed
    f.repeat_penalty, f.seed = 1.3, 4242.0
    p = fb.make_params(1)
    assert lib.fsb_params_from_request(C.byref(f), None, 0, p.ctypes.data) == 0
    assert p["repetition_penalty"][0] == np.float32(1.3) and p["seed"][0] == 4242 and p["top_k"][0] == 50
    assert lib.fsb_params_from_request(None, None, 0, p.ctypes.data) == -1
