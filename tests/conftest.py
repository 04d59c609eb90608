import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with `-m gpu` on the GPU box)")


@pytest.fixture(scope="session")
def model_dir(tmp_path_factory):
    return str(tmp_path_factory.mktemp("models"))


@pytest.fixture(scope="session")
def tiny_paths(model_dir):
    """Config 1 of the benchmark: tiny RWKV-7, seed 0, as fp16, int8 symmetric-per-row, int8 per-group."""
    import rwkv_rsv_b200 as rsv
    out = {}
    for name, q in (("fp16", 0), ("int8", 1), ("int8g", 2)):
        out[name] = rsv.write_synthetic(os.path.join(model_dir, f"tiny_{name}.st"), "tiny", seed=0, quant=q)
    return out


def config1_tokens():
    """128 prompt tokens drawn uniformly over the tiny vocabulary (seed 0)."""
    return np.random.default_rng(0).integers(0, 4096, size=128).astype(np.uint32)
