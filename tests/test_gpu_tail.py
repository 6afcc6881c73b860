"""GPU: the last, partial wave of output tiles in its three forms (int4_linear_set_tail): whole
tiles, half-width items, and cut along K with the shares added into Y.  All must give the same bits
as the oracle.

Shapes are chosen so that the schedule of int4linear_b200/csrc/schedule.cuh really cuts or halves
tiles on a 148-SM device: a handful of tiles with many K blocks (every tile gets several shares),
more tiles than workers (whole tiles first, then the cut ones), ragged M and N, and an N that forces
the per-thread epilogue (atomic adds instead of bulk reductions).  Each launch is repeated, replayed
from a CUDA graph, and issued on several streams at once.
"""
import numpy as np
import pytest

import int4linear_b200 as L
from conftest import make_case
from oracle import oracle as O

pytestmark = pytest.mark.gpu

SHAPES = [
    # (m, n, k, tile_n, pairs)
    (512, 512, 4096, 0, 1),      # 4 pair tiles x 32 K blocks on 74 pairs: eight shares per tile
    (512, 512, 8192, 0, 1),      # 64 K blocks
    (300, 333, 4096, 128, 0),    # single-CTA 128 x 128 tiles, n % 4 != 0: per-thread stores and atomic adds
    (1000, 520, 4096, 256, 0),   # single-CTA 128 x 256 tiles, ragged M and N
    (2560, 2304, 4096, 0, 1),    # 90 pair tiles: one whole wave of 74, then 16 cut tiles
    (130, 1000, 2048, 64, 0),    # 128 x 64 tiles
]


def _reference(x, w):
    if x.shape[0] * w.shape[0] * x.shape[1] > 2e8:
        return O.linear_ref_sgemm(x, w)
    return O.linear_ref(x.astype(np.int32), w.astype(np.int32))


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_tail_forms_are_exact(cuda, shape):
    import torch
    m, n, k, tile_n, pairs = shape
    x, w, xp, wp = make_case(m, n, k, seed=21)
    ref = _reference(x, w)
    xd, wd = torch.from_numpy(xp).to(cuda), torch.from_numpy(wp).to(cuda)
    bias = torch.from_numpy(((np.arange(n) * 29) % 2001 - 1000).astype(np.int32)).to(cuda)
    prev = L.set_path(L.PATH_TCGEN05)
    L.set_tuning(tile_n, False, pairs)
    try:
        results = {}
        for mode in (2, 1, 0, -1):
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
        assert O.is_same(results[2], results[1]) and O.is_same(results[2], results[0])
    finally:
        L.set_tail(-1)
        L.set_tuning(0, False, -1)
        L.set_path(prev)


def test_k_cut_really_launches_the_clearing_kernel(cuda):
    """Mode 2 on a shape whose tiles it cuts is two launches (clear, GEMM); mode 0 is one."""
    import torch
    m, n, k = 512, 512, 8192
    x, w, xp, wp = make_case(m, n, k, seed=24)
    xd, wd = torch.from_numpy(xp).to(cuda), torch.from_numpy(wp).to(cuda)
    prev = L.set_path(L.PATH_TCGEN05)
    try:
        counts = {}
        for mode in (2, 0):
            L.set_tail(mode)
            before = L.launch_count()
            L.linear(xd, wd)
            torch.cuda.synchronize()
            counts[mode] = L.launch_count() - before
        assert counts == {2: 2, 0: 1}
    finally:
        L.set_tail(-1)
        L.set_path(prev)


def test_tail_forms_in_a_replayed_graph(cuda):
    import torch
    m, n, k = 512, 768, 4096
    x, w, xp, wp = make_case(m, n, k, seed=22)
    ref = _reference(x, w)
    xd, wd = torch.from_numpy(xp).to(cuda), torch.from_numpy(wp).to(cuda)
    yd = torch.zeros((m, n), dtype=torch.int32, device=cuda)
    prev = L.set_path(L.PATH_TCGEN05)
    try:
        for mode in (2, 1):
            L.set_tail(mode)
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
                assert O.is_same(yd.cpu().numpy(), ref), f"tail mode {mode}"
        assert L.last_status() == 0
    finally:
        L.set_tail(-1)
        L.set_path(prev)


def test_k_cut_on_several_streams_at_once(cuda):
    """The cut needs no state shared between launches: launches that overlap in time are independent."""
    import torch
    m, n, k = 512, 512, 4096
    x, w, xp, wp = make_case(m, n, k, seed=23)
    ref = _reference(x, w)
    xd, wd = torch.from_numpy(xp).to(cuda), torch.from_numpy(wp).to(cuda)
    streams = [torch.cuda.Stream() for _ in range(3)]
    outs = [torch.zeros((m, n), dtype=torch.int32, device=cuda) for _ in streams]
    prev = L.set_path(L.PATH_TCGEN05)
    L.set_tail(2)
    try:
        torch.cuda.synchronize()
        for rep in range(4):
            for s, y in zip(streams, outs):
                with torch.cuda.stream(s):
                    L.linear(xd, wd, out=y)
        torch.cuda.synchronize()
        assert L.last_status() == 0
        for y in outs:
            assert O.is_same(y.cpu().numpy(), ref)
    finally:
        L.set_tail(-1)
        L.set_path(prev)


def test_tail_mode_argument_check():
    from int4linear_b200 import _lib
    lib = _lib.load()
    assert lib.int4_linear_set_tail(3) == 1 and lib.int4_linear_set_tail(-2) == 1
    assert lib.int4_linear_set_tail(-1) == 0
