"""GPU: a last, partial wave of output tiles run as half-width items (int4_linear_set_tail) must
give the same bits as whole tiles and as the oracle.

Shapes are chosen so that the schedule of int4linear_b200/csrc/schedule.cuh really halves tiles
on a 148-SM device: fewer pair tiles than half the CTA pairs, and more tiles than pairs with a
short remainder; ragged M and N included.  Each launch is repeated, and replayed from a CUDA graph.
"""
import numpy as np
import pytest

import int4linear_b200 as L
from conftest import make_case
from oracle import oracle as O

pytestmark = pytest.mark.gpu

SHAPES = [
    (512, 512, 2048),     # 4 pair tiles on 74 pairs: eight half-width items
    (300, 520, 1024),     # ragged M and N
    (2560, 2304, 512),    # 90 pair tiles: a whole wave of 74, then 16 halved tiles
    (257, 1000, 4096),    # second row block with one row
]


def _reference(x, w):
    if x.shape[0] * w.shape[0] * x.shape[1] > 2e8:
        return O.linear_ref_sgemm(x, w)
    return O.linear_ref(x.astype(np.int32), w.astype(np.int32))


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_half_width_tail_is_exact(cuda, shape):
    import torch
    m, n, k = shape
    x, w, xp, wp = make_case(m, n, k, seed=21)
    ref = _reference(x, w)
    xd, wd = torch.from_numpy(xp).to(cuda), torch.from_numpy(wp).to(cuda)
    bias = torch.from_numpy(((np.arange(n) * 29) % 2001 - 1000).astype(np.int32)).to(cuda)
    prev = L.set_path(L.PATH_TCGEN05)
    L.set_tuning(0, False, 1)
    try:
        results = {}
        for mode in (1, 0, -1):
            L.set_tail(mode)
            for rep in range(2):
                yd = torch.full((m, n), -777, dtype=torch.int32, device=cuda)
                L.linear(xd, wd, out=yd)
                torch.cuda.synchronize()
                assert L.last_status() == 0
                got = yd.cpu().numpy()
                assert O.is_same(got, ref), f"tail mode {mode}, launch {rep}"
            results[mode] = got
            yb = torch.full((m, n), -777, dtype=torch.int32, device=cuda)
            L.linear(xd, wd, out=yb, bias=bias)
            torch.cuda.synchronize()
            assert O.is_same(yb.cpu().numpy(), ref + bias.cpu().numpy()[None, :]), f"tail mode {mode}, bias"
        assert O.is_same(results[1], results[0])
    finally:
        L.set_tail(-1)
        L.set_tuning(0, False, -1)
        L.set_path(prev)


def test_half_width_tail_in_a_replayed_graph(cuda):
    import torch
    m, n, k = 512, 768, 2048
    x, w, xp, wp = make_case(m, n, k, seed=22)
    ref = _reference(x, w)
    xd, wd = torch.from_numpy(xp).to(cuda), torch.from_numpy(wp).to(cuda)
    yd = torch.zeros((m, n), dtype=torch.int32, device=cuda)
    prev = L.set_path(L.PATH_TCGEN05)
    L.set_tail(1)
    try:
        L.linear(xd, wd, out=yd)  # first call outside the capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                L.linear(xd, wd, out=yd)
                L.linear(xd, wd, out=yd)
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(3):
            yd.fill_(-5)
            graph.replay()
            torch.cuda.synchronize()
            assert O.is_same(yd.cpu().numpy(), ref)
        assert L.last_status() == 0
    finally:
        L.set_tail(-1)
        L.set_path(prev)


def test_tail_mode_argument_check():
    from int4linear_b200 import _lib
    lib = _lib.load()
    assert lib.int4_linear_set_tail(2) == 1 and lib.int4_linear_set_tail(-2) == 1
    assert lib.int4_linear_set_tail(-1) == 0
