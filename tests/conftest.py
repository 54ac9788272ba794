import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden", "golden.npz")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    return np.load(GOLDEN)


@pytest.fixture(scope="session")
def port():
    from oracle import oracle as O
    return O.Port.get()


@pytest.fixture(scope="session")
def tiny_model():
    from mynah_tts_b200 import synth
    return synth.make_model(synth.TINY, seed=3)


@pytest.fixture(scope="session")
def tiny_memory():
    from mynah_tts_b200 import synth
    return synth.make_memory(synth.TINY, seed=5)


def rel_err(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / (np.abs(b).max() + 1e-30))
