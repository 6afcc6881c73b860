"""GPU: the five benchmark configurations and the headline shape at full size.

The CPU oracle's triple loop cannot cover these in seconds, so each shape is
checked (a) exactly on a sample of rows computed by the oracle, (b) exactly
everywhere against the float32-BLAS restatement (exact for these magnitudes,
see oracle.linear_ref_sgemm and its test), and (c) through properties that do
not need a reference at all: N-shards computed separately reproduce the
columns of the full product, and negating X negates Y.
"""
import numpy as np
import pytest

import int4linear_b200 as L
from oracle import oracle as O

pytestmark = pytest.mark.gpu

CONFIGS = {
    "c1": (1024, 1024, 1024),
    "c2": (4096, 4096, 4096),
    "c3": (4096, 4096, 8192),
    "c4": (16, 14336, 4096),
}


def operands(name, m, n, k):
    seed = int(name[1:]) if name[1:].isdigit() else 8
    xp = L.uniform_s4_packed(0xA000 + seed, m, k)
    wp = L.uniform_s4_packed(0xB000 + seed, n, k)
    return xp, wp


@pytest.mark.parametrize("name", list(CONFIGS))
def test_config_bit_exact(cuda, name):
    import torch
    m, n, k = CONFIGS[name]
    xp, wp = operands(name, m, n, k)
    xd, wd = torch.from_numpy(xp).to(cuda), torch.from_numpy(wp).to(cuda)
    yd = L.linear(xd, wd)
    torch.cuda.synchronize()
    assert L.last_status() == 0
    y = yd.cpu().numpy()

    x, w = L.unpack_bytes(xp), L.unpack_bytes(wp)
    rows = np.unique(np.concatenate([[0, m - 1], np.random.default_rng(0).integers(0, m, 6)])).astype(np.int32)
    assert O.is_same(y[rows], O.linear_ref_rows(x.astype(np.int32), w.astype(np.int32), rows))
    assert O.is_same(y, O.linear_ref_sgemm(x, w))

    # shard property: columns [n/2, n) computed alone
    y_half = L.linear(xd, wd[n // 2:].contiguous())
    # negation property: (-X) W^T = -(X W^T); -x needs x != -8, so clamp a copy
    xc = np.maximum(x, -7)
    y_pos = L.linear(torch.from_numpy(L.pack_bytes(xc)).to(cuda), wd)
    y_neg = L.linear(torch.from_numpy(L.pack_bytes(-xc)).to(cuda), wd)
    torch.cuda.synchronize()
    assert L.last_status() == 0
    assert O.is_same(y_half.cpu().numpy(), np.ascontiguousarray(y[:, n // 2:]))
    assert bool((y_pos == -y_neg).all())


def test_headline_shape_rows_and_shards(cuda):
    """M=N=K=8192 (the metric's shape) and the large config's N extent are checked on
    sampled rows and on the shard property, which together touch every tile column."""
    import torch
    m, n, k = 8192, 8192, 8192
    xp = L.uniform_s4_packed(0xA008, m, k)
    wp = L.uniform_s4_packed(0xB008, n, k)
    xd, wd = torch.from_numpy(xp).to(cuda), torch.from_numpy(wp).to(cuda)
    yd = L.linear(xd, wd)
    shards = [L.linear(xd, wd[i * (n // 8):(i + 1) * (n // 8)].contiguous()) for i in range(8)]
    torch.cuda.synchronize()
    assert L.last_status() == 0
    assert bool((torch.cat(shards, dim=1) == yd).all())
    rows = np.array([0, 127, 128, 4097, 8191], dtype=np.int32)
    x = L.unpack_bytes(xp[rows]).astype(np.int32)
    w = L.unpack_bytes(wp).astype(np.int32)
    ref = O.linear_ref(x, w)
    assert O.is_same(yd[torch.from_numpy(rows).long().to(cuda)].cpu().numpy(), ref)


def test_large_config_c5_bit_exact(cuda):
    """c5 = 8192 x 28672 x 8192, the N-sharded config: the whole 896 MiB result is compared with the
    float32-BLAS restatement (exact at these magnitudes) in row blocks, sampled rows with the
    oracle's integer loop, and the 8-way N-shard results with the matching columns."""
    import torch
    m, n, k = 8192, 28672, 8192
    xp = L.uniform_s4_packed(0xA005, m, k)
    wp = L.uniform_s4_packed(0xB005, n, k)
    xd, wd = torch.from_numpy(xp).to(cuda), torch.from_numpy(wp).to(cuda)
    yd = L.linear(xd, wd)
    torch.cuda.synchronize()
    assert L.last_status() == 0
    for s in range(8):  # what each of 8 GPUs would compute
        lo, hi = s * (n // 8), (s + 1) * (n // 8)
        ys = L.linear(xd, wd[lo:hi].contiguous())
        assert bool((ys == yd[:, lo:hi]).all())
    torch.cuda.synchronize()
    assert L.last_status() == 0
    y = yd.cpu().numpy()
    w = L.unpack_bytes(wp)
    rows = np.array([0, 255, 256, 4099, 8191], dtype=np.int32)
    x_rows = L.unpack_bytes(xp[rows]).astype(np.int32)
    assert O.is_same(y[rows], O.linear_ref(x_rows, w.astype(np.int32)))
    wf = w.astype(np.float32)
    for r0 in range(0, m, 1024):
        xf = L.unpack_bytes(xp[r0:r0 + 1024]).astype(np.float32)
        assert O.is_same(y[r0:r0 + 1024], (xf @ wf.T).astype(np.int32)), f"rows {r0}..{r0 + 1023}"
