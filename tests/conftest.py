import glob
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU")


@pytest.fixture(scope="session", autouse=True)
def _built():
    """Make sure the oracle and the CUDA library exist (both build without a GPU)."""
    from oracle import build as obuild
    obuild.build_oracle()
    from int4linear_b200 import build as lbuild
    if lbuild.needs_build():
        lbuild.build()
    lbuild.build_compat_check()


def golden_files():
    return sorted(glob.glob(os.path.join(ROOT, "tests", "golden", "*.npz")))


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    return torch.device("cuda:0")


def make_case(m, n, k, seed=1):
    """Seeded uniform [-8,7] operands: (x int8 [m,k], w int8 [n,k], x_packed u8, w_packed u8)."""
    from int4linear_b200 import uniform_s4, pack_bytes
    x = uniform_s4(0xA000 + seed, m, k)
    w = uniform_s4(0xB000 + seed, n, k)
    return x, w, pack_bytes(x), pack_bytes(w)
