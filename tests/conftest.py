import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """The C-ABI library must exist for every test; build it in-tree if it is not there yet."""
    from kernels_b200 import _lib, build

    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    return _lib.load()


@pytest.fixture(scope="module", autouse=True)
def _fresh_dynamo_cache():
    """The public entry point is a ``torch.compile(fullgraph=True)`` function, as the reference's is
    (src/streaming_attention/kernel.py:1566); a long run over many distinct shapes would meet dynamo's
    recompile limit, so every test module starts from an empty cache, whatever order the modules run in
    (the reference's tests reset it per test, tests/test_streaming_attention.py:50)."""
    import torch

    torch._dynamo.reset()
    yield


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    def load(name):
        z = np.load(os.path.join(ROOT, "tests", "golden", name + ".npz"))
        cases = {}
        for key in z.files:
            case, field = key.split("/")
            cases.setdefault(case, {})[field] = z[key]
        return cases

    return load
