"""The header-only C++ adapter: it must compile against the C ABI as the reference's call sites are written
(CPU: compile and link only), and reproduce the reference's known-answer vector on a GPU."""
import os
import shutil
import subprocess

import pytest

import ferro_b200 as fb

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build(tmp_path):
    gxx = shutil.which("g++")
    if not gxx:
        pytest.skip("no g++ on this machine")
    lib = fb.library_path()
    fb.load_library()                                   # builds the library if it is missing
    exe = str(tmp_path / "adapter_kat")
    cmd = [gxx, "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "adapter_kat.cpp"),
           "-L", os.path.dirname(lib), "-lferro_sampler_b200", "-Wl,-rpath," + os.path.dirname(lib), "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_adapter_compiles_and_links_like_a_reference_call_site(tmp_path):
    _build(tmp_path)


@pytest.mark.gpu
def test_adapter_reproduces_the_reference_known_answer_vector(tmp_path):
    r = subprocess.run([_build(tmp_path)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.split() == ["4", "2", "1", "2", "2"]
