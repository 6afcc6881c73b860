"""CPU: the N-sharding driver's host logic, including a world_size-2 gloo run in which each
rank's shard result comes from the CPU oracle (test infrastructure) and the gathered matrix
must equal the oracle's full product."""
import os
import socket

import numpy as np
import pytest

from int4linear_b200 import sharding as S


def test_bounds_cover_n_exactly():
    for n in (8192, 28672, 14336, 1000, 256, 100, 3584 * 8 + 8):
        for world in (1, 2, 4, 8):
            sh = S.all_shards(n, world)
            assert sh[0].row_start == 0
            assert sum(s.rows for s in sh) == n
            for a, b in zip(sh, sh[1:]):
                assert a.row_start + a.rows == b.row_start
            # balanced to within one tile
            assert max(s.rows for s in sh) - min(s.rows for s in sh) < 512  # one tile, plus a ragged last tile


def test_baseline_shards_are_tile_aligned():
    for n, world, want in [(28672, 8, 3584), (28672, 2, 14336), (8192, 8, 1024), (8192, 4, 2048)]:
        sh = S.all_shards(n, world)
        assert all(s.rows == want for s in sh)
        assert all(s.row_start % 256 == 0 for s in sh)


def test_shard_is_contiguous_view():
    w = np.arange(40 * 4, dtype=np.uint8).reshape(40, 4)
    s = S.shard_bounds(40, 2, 1, align=8)
    v = S.shard_rows(w, s)
    assert np.shares_memory(v, w) and v.flags['C_CONTIGUOUS']
    assert v.shape[0] == s.rows and v[0, 0] == w[s.row_start, 0]


def test_fused_gather_geometry_rule():
    """The fused gather is used only when every shard starts and ends on a 32-column boundary;
    the decision depends on the global split alone, so all ranks agree."""
    class _Probe(S.ShardedInt4Linear):
        def __init__(self, n_total, world, align=256):
            self.n_total, self.world, self.align = n_total, world, align
    assert _Probe(28672, 8)._fused_ok()
    assert _Probe(8192, 2)._fused_ok()
    assert _Probe(1536, 2)._fused_ok()
    assert not _Probe(1000, 2)._fused_ok()     # last shard ends off a 32-column boundary
    assert not _Probe(28672 + 2, 4)._fused_ok()  # row pitch of Y not a 16-byte multiple


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n, q):
    import torch
    import torch.distributed as dist
    from int4linear_b200 import uniform_s4
    from oracle import oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, k = 12, 64
        x = uniform_s4(5, m, k).astype(np.int32)
        shard = S.shard_bounds(n, world, rank, align=8)
        # this rank only ever sees its own rows of W (generated independently of the others)
        w_local = uniform_s4(6, shard.rows, k, row_start=shard.row_start).astype(np.int32)
        y_local = O.linear_ref(x, w_local) if shard.rows else np.zeros((m, 0), np.int32)
        full = S.gather_columns(torch.from_numpy(y_local), n, align=8)
        w_full = uniform_s4(6, n, k).astype(np.int32)
        ok = bool(O.is_same(full.numpy(), O.linear_ref(x, w_full)))
        q.put((rank, ok))
    except Exception as e:  # report instead of leaving the parent to time out
        q.put((rank, repr(e)))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n", [48, 40, 8])  # even split, uneven split, an empty shard
def test_gather_over_gloo_world2(n):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, n, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, True), (1, True)]
    assert all(p.exitcode == 0 for p in procs)
