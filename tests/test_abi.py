"""CPU tests of the drop-in boundary: the library builds, loads and exports exactly what include/*.h declares;
the parameter struct has the reference's layout; range checks follow the reference's request parser; and without
a GPU the engine fails loudly instead of falling back to anything."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import ferro_b200 as fb

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            names += re.findall(r"FSB_API\s+[\w\s\*]+?\b(fsb_\w+)\s*\(", text)
    return sorted(set(names))


def test_library_builds_and_exports_every_declared_symbol():
    lib = fb.load_library()
    decl = declared_symbols()
    assert len(decl) >= 20
    for name in decl:
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"
    assert sorted(fb.API_SYMBOLS) == decl, "the Python binding and the header disagree on the API"


def test_library_does_not_link_torch_or_the_oracle():
    import subprocess
    out = subprocess.run(["ldd", fb.library_path()], capture_output=True, text=True).stdout
    assert "torch" not in out and "oracle" not in out and "libferro_ref" not in out


def test_params_struct_layout_matches_reference():
    assert fb.PARAMS_DTYPE.itemsize == 40
    assert fb.PARAMS_DTYPE.fields["seed"][1] == 32
    p = fb.make_params(1)
    # defaults of src/sampler.h:13-20
    assert p["temperature"][0] == np.float32(0.05) and p["top_k"][0] == 50 and p["top_p"][0] == 1.0 and p["min_p"][0] == 0.0
    assert p["repetition_penalty"][0] == np.float32(1.05) and p["repeat_last_n"][0] == -1 and p["penalty_from"][0] == 0 and p["seed"][0] == 0


@pytest.mark.parametrize("field,value,ok", [
    ("temperature", -1.0, False), ("temperature", 0.0, True), ("top_p", 0.0, False), ("top_p", 1.0, True), ("top_p", 1.5, False),
    ("top_k", -1, False), ("top_k", 0, True), ("repetition_penalty", 0.0, False), ("repetition_penalty", 0.5, True),
    ("repeat_last_n", -2, False), ("repeat_last_n", -1, True), ("min_p", -0.1, False), ("min_p", 1.0, True), ("penalty_from", -1, False),
    ("temperature", float("nan"), False),
])
def test_params_validate_follows_the_reference_request_parser(field, value, ok):
    # src/server.cpp:1071: temperature >= 0, 0 < top_p <= 1, top_k >= 0, repetition_penalty > 0, repeat_last_n >= -1
    lib = fb.load_library()
    p = fb.make_params(1)
    p[field] = value
    rc = lib.fsb_params_validate(p.ctypes.data)
    assert (rc == 0) == ok


def test_null_arguments_are_errors_not_crashes():
    lib = fb.load_library()
    assert lib.fsb_params_validate(None) < 0
    assert lib.fsb_create(0, 0, 10, 10, C.byref(C.c_void_p())) < 0
    assert lib.fsb_destroy(None) < 0
    assert lib.fsb_sample_batch(None, 1, None, None, 1, 1, None, None, None, 0) < 0
    assert lib.fsb_counters(None, None) < 0


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(fb.SamplerError) as e:
        fb.Engine(device=0)
    assert e.value.code == -6    # FSB_ERR_NO_DEVICE


def test_product_sources_never_reference_the_oracle():
    for base, _, files in os.walk(os.path.join(ROOT, "ferro_b200")):
        for fn in files:
            if fn.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(base, fn)).read()
                assert "import oracle" not in text and "from oracle" not in text and "liboracle" not in text and "libferro_ref" not in text, fn
