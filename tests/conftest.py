import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def reference_dir():
    """The reference source tree when one is at hand ($CN_REFERENCE_DIR, else `reference` beside the repository)."""
    for cand in (os.environ.get("CN_REFERENCE_DIR"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "source")):
            return cand
    return None


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


@pytest.fixture(scope="session")
def codebook():
    import numpy as np
    return np.fromfile(os.path.join(ROOT, "tests", "golden", "codebook_126.f32"), dtype="<f4")


@pytest.fixture(scope="session")
def built_lib():
    from clusternet_b200 import build as cn_build
    cn_build.build()
    import clusternet_b200
    return clusternet_b200.load()


@pytest.fixture(scope="session")
def ctx(built_lib):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import clusternet_b200
    c = clusternet_b200.Context(0)
    yield c
    c.close()
