"""The gathering GEMM: each rank's column block stored into every rank's full-width Y.

On one GPU the ranks are emulated one after the other: every "rank" launches with its own
weight shard and column offset, and the destination list holds two different buffers of the
same device, so both the multi-destination epilogue and the column shift are exercised.  With
two or more GPUs the real thing runs as one process per GPU over symmetric memory.
"""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from conftest import make_case  # noqa: E402
from oracle import oracle as O  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ref(x, w):
    return O.linear_ref_sgemm(x, w) if x.shape[0] * w.shape[0] * x.shape[1] > 2e8 else \
        O.linear_ref(x.astype(np.int32), w.astype(np.int32))


@pytest.mark.parametrize("m,n_total,k,world", [
    (256, 512, 256, 2),      # CTA-pair tiles, both ranks one tile wide
    (200, 1024, 512, 4),     # ragged M
    (64, 768, 1024, 3),      # m <= 128: single-CTA 128-wide tiles
    (384, 2 * 288, 128, 2),  # shard width 288: a tile tail inside every shard
    (1024, 4096, 2048, 8),   # eight destinations
])
def test_gather_emulated_ranks(m, n_total, k, world):
    import torch
    import int4linear_b200 as L
    from int4linear_b200.linear import linear_gather
    dev = torch.device("cuda", 0)
    x, w, xp, wp = make_case(m, n_total, k, seed=61)
    expect = _ref(x, w)
    xd = torch.from_numpy(xp).to(dev)
    wd = torch.from_numpy(wp).to(dev)
    # one full-width result per emulated rank, poisoned so that unwritten cells show
    fulls = [torch.full((m, n_total), -7, dtype=torch.int32, device=dev) for _ in range(world)]
    ptrs = [f.data_ptr() for f in fulls]
    n_local = n_total // world
    assert n_local % 32 == 0
    for r in range(world):
        linear_gather(xd, wd[r * n_local:(r + 1) * n_local], ptrs, r * n_local, n_total, k=k)
    torch.cuda.synchronize()
    assert L.last_status() == 0
    for f in fulls:
        assert np.array_equal(f.cpu().numpy(), expect)


def test_gather_bias_and_partial_fill():
    """One rank alone writes only its own columns of every destination; bias is per local column."""
    import torch
    import int4linear_b200 as L
    from int4linear_b200.linear import linear_gather
    dev = torch.device("cuda", 0)
    m, n_total, k, n_local, off = 300, 640, 256, 256, 320
    x, w, xp, wp = make_case(m, n_local, k, seed=62)
    bias = np.arange(n_local, dtype=np.int32) * 3 - 100
    expect = _ref(x, w) + bias[None, :]
    fulls = [torch.full((m, n_total), -7, dtype=torch.int32, device=dev) for _ in range(2)]
    linear_gather(torch.from_numpy(xp).to(dev), torch.from_numpy(wp).to(dev), [f.data_ptr() for f in fulls],
                  off, n_total, k=k, bias=torch.from_numpy(bias).to(dev))
    torch.cuda.synchronize()
    for f in fulls:
        got = f.cpu().numpy()
        assert np.array_equal(got[:, off:off + n_local], expect)
        assert (got[:, :off] == -7).all() and (got[:, off + n_local:] == -7).all()


@pytest.mark.parametrize("n_local,off,n_total", [(100, 0, 400), (128, 16, 512), (128, 0, 130), (128, 448, 512 - 32)])
def test_gather_rejects_unsupported_geometry(n_local, off, n_total):
    import torch
    import int4linear_b200 as L
    from int4linear_b200.linear import linear_gather, Int4LinearError
    dev = torch.device("cuda", 0)
    m, k = 64, 128
    xd = torch.zeros((m, k // 2), dtype=torch.uint8, device=dev)
    wd = torch.zeros((n_local, k // 2), dtype=torch.uint8, device=dev)
    y = torch.zeros((m, max(n_total, 1)), dtype=torch.int32, device=dev)
    with pytest.raises(Int4LinearError):
        linear_gather(xd, wd, [y.data_ptr()], off, n_total, k=k)


def test_gather_two_gpus():
    """One process per GPU, symmetric-memory result buffers, stores over NVLink."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29731",
           os.path.join(ROOT, "tests", "gather_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "GATHER_OK" in out.stdout


def test_sharded_layer_with_and_without_expanded_weights(cuda):
    """One rank: the layer with its weights also kept expanded (used for more than 128 rows of X)
    and the packed-only default give the same bits as the oracle, for a prefill and a decode call."""
    import numpy as np
    import torch
    import int4linear_b200 as L
    from int4linear_b200.sharding import ShardedInt4Linear
    from oracle import oracle as O
    n, k = 520, 512
    w = L.uniform_s4(0x7B02, n, k)
    wd = torch.from_numpy(L.pack_bytes(w)).to(cuda)
    for m in (300, 16):
        x = L.uniform_s4(0x7B01 + m, m, k)
        xd = torch.from_numpy(L.pack_bytes(x)).to(cuda)
        want = O.linear_ref(x.astype(np.int32), w.astype(np.int32))
        for expand in (True, False):
            layer = ShardedInt4Linear(wd, n, k, expand_weights=expand)
            y = layer.forward(xd)
            torch.cuda.synchronize()
            assert O.is_same(y.cpu().numpy(), want), (m, expand)
            assert (layer._w_expanded is not None) == (expand and m > 128)
    assert L.last_status() == 0
