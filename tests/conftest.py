import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def port():
    from oracle.oracle import Oracle, build
    build()
    return Oracle("port")


@pytest.fixture(scope="session")
def ref():
    """The reference's own sampler when its build is present, else the restatement."""
    from oracle.oracle import Oracle, build
    build()
    return Oracle("best")


@pytest.fixture(scope="session")
def gpu_sampler_factory():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from mako_b200 import BatchSampler
    cache = {}

    def make(n_vocab, max_batch, cand_cap=0):
        key = (n_vocab, max_batch, cand_cap)
        if key not in cache:
            cache[key] = BatchSampler(n_vocab, max_batch, 0, cand_cap)
        return cache[key]

    return make
