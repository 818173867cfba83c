"""Shared test configuration: markers, import path, fixture loading."""

import glob
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu)")


def golden_names(prefix):
    return sorted(
        os.path.basename(p)[: -len(".npz")]
        for p in glob.glob(os.path.join(GOLDEN_DIR, prefix + "*.npz"))
    )


def load_golden(name):
    with np.load(os.path.join(GOLDEN_DIR, name + ".npz")) as f:
        return {k: f[k] for k in f.files}


def update_cfg(g):
    """Keyword arguments of one `update_*` fixture."""
    return dict(groups=int(g["groups"]), m=int(g["m"]), sc=int(g["sc"]), eps=float(g["eps"]),
                relu_input=bool(int(g["relu_input"])))


def max_norm_error(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


@pytest.fixture(scope="session")
def c_oracle():
    from oracle import c_oracle as mod

    mod.build()
    return mod
