import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def fta_lib():
    """libfta.so, built on demand (nvcc cross-compiles without a GPU)."""
    from flash_tree_attn_b200 import _lib, build

    if not os.path.exists(_lib.LIB_PATH):
        build.build(verbose=False)
    return _lib.load()


def load_golden(name):
    import numpy as np
    import torch

    z = np.load(os.path.join(ROOT, "tests", "golden", name + ".npz"))
    d = {}
    for k in z.files:
        a = z[k]
        d[k] = torch.from_numpy(a) if a.ndim > 0 else int(a)
    return d


GOLDEN = ["cfg1", "gqa_ragged", "mask_one"]
