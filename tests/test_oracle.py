"""CPU: the oracle against the fixtures made by the reference's own code, and
against the reference shim itself where it is built."""
import numpy as np
import pytest

from conftest import golden_files
from oracle import oracle as O


@pytest.mark.parametrize("path", golden_files(), ids=lambda p: p.split("/")[-1][:-4])
def test_oracle_matches_golden(path):
    g = np.load(path)
    x, w = g["x"].astype(np.int32), g["w"].astype(np.int32)
    k = x.shape[1]
    assert O.is_same(O.pack(x), g["x_packed"])
    assert O.is_same(O.pack(w), g["w_packed"])
    assert O.is_same(O.unpack(g["x_packed"], k), x)
    y = O.linear_ref(x, w)
    assert O.is_same(y, g["y"])
    assert O.is_same(O.linear_ref(x, w, single_thread=True), g["y"])
    assert O.is_same(O.linear_packed(g["x_packed"], g["w_packed"], k), g["y"])
    rows = np.array([0, x.shape[0] - 1, x.shape[0] // 2], dtype=np.int32)
    assert O.is_same(O.linear_ref_rows(x, w, rows), g["y"][rows])


def test_golden_fixtures_exist():
    assert len(golden_files()) >= 10


def test_closed_form_patterns():
    g = np.load([p for p in golden_files() if p.endswith("pattern_all_min.npz")][0])
    assert (g["y"] == 64 * 128).all()
    g = np.load([p for p in golden_files() if p.endswith("pattern_min_times_max.npz")][0])
    assert (g["y"] == -56 * 128).all()


@pytest.mark.skipif(O.ref_lib() is None, reason="reference shim not built on this machine")
def test_oracle_matches_reference_code():
    rng = np.random.default_rng(3)
    for m, n, k in [(3, 5, 8), (9, 4, 19), (64, 48, 256), (2, 2, 1)]:
        x = rng.integers(-8, 8, size=(m, k), dtype=np.int32)
        w = rng.integers(-8, 8, size=(n, k), dtype=np.int32)
        assert O.is_same(O.pack(x), O.ref_pack(x))
        assert O.is_same(O.unpack(O.pack(x), k), O.ref_unpack(O.ref_pack(x), k))
        assert O.is_same(O.linear_ref(x, w), O.ref_linear_ref(x, w))


def test_sgemm_checker_is_exact():
    """The float32-BLAS checker used at full size must agree with linear_ref bit for bit,
    including at the extreme sums."""
    rng = np.random.default_rng(5)
    x = rng.integers(-8, 8, size=(37, 4096), dtype=np.int32)
    w = rng.integers(-8, 8, size=(29, 4096), dtype=np.int32)
    x[0, :] = -8
    w[0, :] = -8
    w[1, :] = 7
    assert O.is_same(O.linear_ref_sgemm(x, w), O.linear_ref(x, w))


def test_is_same_detects_difference():
    a = np.arange(10, dtype=np.int32)
    b = a.copy()
    assert O.is_same(a, b)
    b[7] += 1
    assert not O.is_same(a, b)
