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
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs the sm_100a kernels through the C ABI)")


@pytest.fixture(scope="session")
def port():
    """The plain-C oracle (built on demand)."""
    import oracle
    return oracle.port()


@pytest.fixture(scope="session")
def ref():
    """The reference's own C++ build; only where oracle/_ref/libnsos_ref.so exists."""
    import oracle
    if not oracle.ref_available():
        pytest.skip("oracle/_ref/libnsos_ref.so not built (needs the reference checkout)")
    return oracle.ref()


@pytest.fixture(scope="session")
def tbl():
    """The product library through ctypes; built on demand, never replaced by a fallback."""
    from reimagined_b200 import build
    build.build()
    from reimagined_b200 import capi
    return capi.lib()


@pytest.fixture(scope="session")
def cuda():
    """torch with a live CUDA device.  A GPU test without a device fails (no silent skip on the GPU box)."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    torch.cuda.set_device(0)
    return torch


def golden_cases(prefix=""):
    """Fixture paths; without a prefix, the linear / MoE fixtures only (row-norm, decode and router fixtures are
    asked for by name)."""
    paths = sorted(p for p in glob.glob(os.path.join(GOLDEN_DIR, prefix + "*.npz")))
    if not prefix:
        paths = [p for p in paths if not os.path.basename(p).startswith(("rownorm_", "decode_", "router_"))]
    return paths


def load_golden(path):
    """Loads a fixture; regenerates inputs from the seed when they were not stored."""
    import hashlib
    g = dict(np.load(path))
    if "x" in g and "up" in g:
        return g  # MoE fixture
    if "w" not in g:
        rng = np.random.default_rng(int(g["seed"]))
        N, K, M = int(g["N"]), int(g["K"]), int(g["M"])
        g["w"] = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
        g["x"] = rng.standard_normal((M, K)).astype(np.float32)
        h = hashlib.sha256()
        h.update(g["w"].tobytes())
        h.update(g["x"].tobytes())
        assert h.hexdigest() == str(g["input_sha"]), "numpy generator drifted: regenerate fixtures"
    return g
