"""GPU: the few-rows kernel (int4linear_b200/csrc/gemm_fewrows.cu; M <= 128, operands swapped, W
through tensor memory, Y written back transposed; one form for up to 64 rows, one for 65 to 128).  Every shape is compared with the oracle, in the
kernel's three tail forms, with and without bias, through the bulk-store epilogue and the
per-thread one (N % 4 != 0), with K tails, and against the main kernel on the same inputs.
"""
import numpy as np
import pytest

import int4linear_b200 as L
from conftest import make_case
from oracle import oracle as O

pytestmark = pytest.mark.gpu

SHAPES = [
    (1, 8, 32), (5, 7, 32), (16, 264, 1024), (17, 520, 256), (32, 1000, 2048), (33, 264, 4096), (40, 129, 160),
    (48, 4099, 1024), (57, 2050, 1056), (64, 1024, 8192), (64, 130, 288), (64, 14336, 1024),
    (24, 18944, 512),      # 148 tiles: exactly one per SM
    (64, 19200, 2048),     # 150 tiles: one whole wave, then two tiles cut along K
    # 65 .. 128 rows: both halves of X against every stage of W
    (65, 264, 1024), (80, 1000, 2048), (96, 4099, 1056), (100, 14336, 1024), (128, 129, 160), (128, 512, 256),
    (111, 2050, 4096), (128, 19200, 1024), (72, 8, 32),
]


def _reference(x, w):
    if x.shape[0] * w.shape[0] * x.shape[1] > 2e8:
        return O.linear_ref_sgemm(x, w)
    return O.linear_ref(x.astype(np.int32), w.astype(np.int32))


@pytest.fixture
def fewrows_on():
    L.set_fewrows(1)
    try:
        yield
    finally:
        L.set_fewrows(-1)
        L.set_tail(-1)
        L.set_tuning(0, False, -1)


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_fewrows_kernel_is_exact(cuda, fewrows_on, shape):
    import torch
    m, n, k = shape
    x, w, xp, wp = make_case(m, n, k, seed=31)
    ref = _reference(x, w)
    xd, wd = torch.from_numpy(xp).to(cuda), torch.from_numpy(wp).to(cuda)
    bias_h = ((np.arange(n) * 31) % 2003 - 1001).astype(np.int32)
    bias = torch.from_numpy(bias_h).to(cuda)
    before = L.launch_count()
    for direct in (False, True):
        L.set_tuning(0, direct, -1)
        for mode in (-1, 0, 2):
            L.set_tail(mode)
            for rep in range(2):
                yd = torch.full((m, n), -777, dtype=torch.int32, device=cuda)
                L.linear(xd, wd, out=yd)
                torch.cuda.synchronize()
                assert L.last_status() == 0
                assert O.is_same(yd.cpu().numpy(), ref), f"tail {mode}, direct {direct}, launch {rep}"
            yb = torch.full((m, n), -777, dtype=torch.int32, device=cuda)
            L.linear(xd, wd, out=yb, bias=bias)
            torch.cuda.synchronize()
            assert O.is_same(yb.cpu().numpy(), ref + bias_h[None, :]), f"bias, tail {mode}, direct {direct}"
    assert L.launch_count() > before


def test_fewrows_agrees_with_the_main_kernel_at_full_size(cuda, fewrows_on):
    """64 x 14336 x 4096 and 32 x 28672 x 8192: the few-rows kernel, whole tiles and cut, against the
    main kernel's 128-row tiles on the same device buffers (the oracle covers the smaller shapes)."""
    import torch
    for (m, n, k) in [(64, 14336, 4096), (32, 28672, 8192), (17, 8192, 8192), (128, 14336, 4096), (96, 28672, 8192)]:
        g = torch.Generator(device=cuda)
        g.manual_seed(m + n)
        xd = torch.randint(0, 256, (m, k // 2), dtype=torch.uint8, device=cuda, generator=g)
        wd = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=cuda, generator=g)
        L.set_fewrows(0)
        prev = L.set_path(L.PATH_TCGEN05)
        try:
            want = L.linear(xd, wd)
            L.set_fewrows(1)
            for mode in (-1, 0, 2):
                L.set_tail(mode)
                got = L.linear(xd, wd)
                torch.cuda.synchronize()
                assert L.last_status() == 0
                assert bool((got == want).all()), f"{m}x{n}x{k}, tail {mode}"
        finally:
            L.set_path(prev)


def test_default_dispatch_by_shape(cuda):
    """By shape: the register kernels up to 16 rows (up to 32 while the weights are small), the few-rows
    kernel up to 64, the 128-row tiles above."""
    import torch
    assert L.path_for(16, 14336, 4096) == L.PATH_SKINNY
    assert L.path_for(17, 4096, 4096) == L.PATH_SKINNY      # small weights: the register kernels up to 32 rows
    assert L.path_for(17, 14336, 4096) == L.PATH_TCGEN05
    assert L.path_for(33, 1024, 1024) == L.PATH_TCGEN05
    assert L.path_for(64, 4096, 4096) == L.PATH_TCGEN05
    assert L.path_for(128, 4096, 4096) == L.PATH_TCGEN05
    m, n, k = 40, 1024, 2048
    x, w, xp, wp = make_case(m, n, k, seed=5)
    ref = O.linear_ref(x.astype(np.int32), w.astype(np.int32))
    xd, wd = torch.from_numpy(xp).to(cuda), torch.from_numpy(wp).to(cuda)
    for fewrows in (-1, 0, 1):
        L.set_fewrows(fewrows)
        try:
            y = L.linear(xd, wd)
            torch.cuda.synchronize()
        finally:
            L.set_fewrows(-1)
        assert O.is_same(y.cpu().numpy(), ref), f"fewrows mode {fewrows}"
    with pytest.raises(L.Int4LinearError):
        L.set_fewrows(2)


def test_fewrows_in_replayed_graphs_and_on_several_streams(cuda, fewrows_on):
    """Back-to-back launches from a CUDA graph (every launch must leave the SMs' tensor memory and
    barriers as it found them) and three streams at once, whole tiles and cut, both forms of the
    kernel (48 and 112 rows; 74 tiles of 16 steps are cut into 148 shares in the automatic mode)."""
    import torch
    for m, n, k in ((48, 9472, 4096), (112, 9472, 4096)):
        x, w, xp, wp = make_case(m, n, k, seed=77)
        ref = torch.from_numpy(O.linear_ref_sgemm(x, w)).to(cuda)
        xd, wd = torch.from_numpy(xp).to(cuda), torch.from_numpy(wp).to(cuda)
        for mode in (-1, 0):
            L.set_tail(mode)
            ys = [torch.full((m, n), -1, dtype=torch.int32, device=cuda) for _ in range(4)]
            L.linear(xd, wd, out=ys[0])
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    for i in range(40):
                        L.linear(xd, wd, out=ys[i % 4])
            torch.cuda.current_stream().wait_stream(side)
            for _ in range(25):
                graph.replay()
            torch.cuda.synchronize()
            assert L.last_status() == 0
            assert all(bool((y == ref).all()) for y in ys), f"graph, {m} rows, tail {mode}"
            streams = [torch.cuda.Stream() for _ in range(3)]
            outs = [torch.full((m, n), -1, dtype=torch.int32, device=cuda) for _ in range(3)]
            for _ in range(10):
                for s_, y in zip(streams, outs):
                    with torch.cuda.stream(s_):
                        L.linear(xd, wd, out=y)
            torch.cuda.synchronize()
            assert L.last_status() == 0
            assert all(bool((y == ref).all()) for y in outs), f"streams, {m} rows, tail {mode}"


def test_fewrows_random_shapes(cuda, fewrows_on):
    """Seeded random shapes with up to 128 rows through the few-rows kernel (forced on, so that it also
    takes the shapes the dispatcher would leave to the decode kernels or the 128-row tiles): ragged M, N
    and K tails, N % 4 != 0 (per-thread stores, atomic adds), all three tail forms, with bias."""
    import torch
    rng = np.random.default_rng(20241125)
    shapes = []
    for _ in range(40):
        m = int(rng.choice([rng.integers(1, 17), rng.integers(17, 65), rng.integers(65, 129)]))
        n = int(rng.choice([rng.integers(1, 130), rng.integers(130, 1500), rng.integers(1500, 6000), 4 * rng.integers(1000, 5000)]))
        k = 32 * int(rng.choice([rng.integers(1, 9), rng.integers(9, 80)]))
        shapes.append((m, n, k))
    for i, (m, n, k) in enumerate(shapes):
        x, w, xp, wp = make_case(m, n, k, seed=400 + i)
        ref = _reference(x, w)
        xd, wd = torch.from_numpy(xp).to(cuda), torch.from_numpy(wp).to(cuda)
        bias_h = ((np.arange(n) * 17) % 1999 - 999).astype(np.int32)
        bias = torch.from_numpy(bias_h).to(cuda)
        for mode in (-1, 0, 2):
            L.set_tail(mode)
            yd = torch.full((m, n), -5, dtype=torch.int32, device=cuda)
            L.linear(xd, wd, out=yd)
            yb = L.linear(xd, wd, bias=bias)
            torch.cuda.synchronize()
            assert O.is_same(yd.cpu().numpy(), ref), (m, n, k, mode)
            assert O.is_same(yb.cpu().numpy(), ref + bias_h[None, :]), (m, n, k, mode, "bias")
    assert L.last_status() == 0
