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


def _build_call_latency(tmp_path):
    gxx = shutil.which("g++")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    if not gxx or not os.path.exists(os.path.join(cuda, "include", "cuda_runtime.h")):
        pytest.skip("no g++ or no CUDA toolkit on this machine")
    lib = fb.library_path()
    fb.load_library()
    exe = str(tmp_path / "call_latency")
    cmd = [gxx, "-std=c++17", "-O2", "-Wall", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"),
           os.path.join(ROOT, "tests", "call_latency.cpp"), "-L", os.path.dirname(lib), "-lferro_sampler_b200", "-Wl,-rpath," + os.path.dirname(lib),
           "-L", os.path.join(cuda, "lib64"), "-lcudart", "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_call_latency_driver_compiles(tmp_path):
    _build_call_latency(tmp_path)


@pytest.mark.gpu
def test_call_latency_driver_runs_every_public_call(tmp_path):
    import json
    r = subprocess.run([_build_call_latency(tmp_path), "34", "8192", "64", "5"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["rows"] == 34 and all(v > 0 for k, v in out.items() if k.endswith("_us"))
