"""Build recipe for the CPU oracle.  TEST INFRASTRUCTURE ONLY - the product never imports this.

Two shared objects:

* ``oracle/_build/liboracle.so``  - the plain-C restatement (``sampler_oracle.c``), built with gcc.
* ``oracle/_ref/libferro_ref.so`` - the UNMODIFIED reference sampler (``src/sampler.cpp`` of the
  reference checkout, compiled from where it lies, never copied) plus ``ref_driver.cpp``, built
  with the reference's own flags (its Makefile line 2: ``-O3 -std=c++17 -fno-math-errno -fPIC``).
  Only possible where the reference checkout is present; elsewhere a previously built file is used.

Run ``python oracle/build.py`` or call :func:`build_all`.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD_DIR = os.path.join(HERE, "_build")
REF_DIR = os.path.join(HERE, "_ref")
ORACLE_SO = os.path.join(BUILD_DIR, "liboracle.so")
REF_SO = os.path.join(REF_DIR, "libferro_ref.so")


def reference_root() -> str | None:
    """Directory of the reference checkout, or None when it is not on this machine."""
    root = os.environ.get("FERRO_REFERENCE_ROOT", "/root/reference")
    return root if os.path.isfile(os.path.join(root, "src", "sampler.cpp")) else None


def _newer(target: str, *sources: str) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources if os.path.exists(s))


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "sampler_oracle.c")
    if not force and _newer(ORACLE_SO, src):
        return ORACLE_SO
    os.makedirs(BUILD_DIR, exist_ok=True)
    # no FMA contraction, no re-association: the sums must run in the reference's order
    cmd = ["gcc", "-O2", "-std=c11", "-fno-math-errno", "-ffp-contract=off", "-fPIC", "-shared",
           "-o", ORACLE_SO, src, "-lm"]
    subprocess.run(cmd, check=True)
    return ORACLE_SO


def build_ref(force: bool = False) -> str | None:
    """Compile the reference sampler where its sources are available; return the .so path or None."""
    root = reference_root()
    drv = os.path.join(HERE, "ref_driver.cpp")
    if root is None:
        return REF_SO if os.path.exists(REF_SO) else None
    ref_src = os.path.join(root, "src", "sampler.cpp")
    if not force and _newer(REF_SO, drv, ref_src, os.path.join(root, "src", "sampler.h")):
        return REF_SO
    os.makedirs(REF_DIR, exist_ok=True)
    cmd = ["g++", "-O3", "-std=c++17", "-fno-math-errno", "-fPIC", "-shared", "-pthread",
           "-I" + os.path.join(root, "src"), "-o", REF_SO, drv, ref_src]
    subprocess.run(cmd, check=True)
    return REF_SO


def build_all(force: bool = False) -> dict:
    return {"oracle": build_oracle(force), "ref": build_ref(force)}


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv))
