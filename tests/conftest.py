"""Test configuration.  GPU tests carry the `gpu` marker; everything else runs on a machine without a GPU."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); deselect with -m 'not gpu'")


@pytest.fixture(scope="session")
def oracle():
    from oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reflib():
    from oracle import RefLib
    if not RefLib.available():
        pytest.skip("the reference sampler library is not built on this machine")
    return RefLib()


@pytest.fixture(scope="session")
def engine():
    import ferro_b200 as fb
    eng = fb.Engine(device=0, max_rows=512, max_vocab=262144, max_hist_ids=1 << 20)
    yield eng
    eng.close()
