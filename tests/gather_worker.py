"""Worker of the multi-GPU gather test (run under torch.distributed.run, one rank per GPU):
N-sharded layer with gather="fused" against the NCCL all-gather path and the CPU oracle."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import int4linear_b200 as L  # noqa: E402
from int4linear_b200.sharding import ShardedInt4Linear, shard_bounds  # noqa: E402
from oracle import oracle  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    for (m, n, k) in [(512, 1024, 512), (96, 2048, 1024), (1000, 1536, 256), (300, 1000, 256),  # ragged N: NCCL fallback
                      (64, 256, 128)]:  # fewer 256-row units than ranks: the last rank owns nothing
        sh = shard_bounds(n, world, rank)
        x, w = L.uniform_s4(0x7A01, m, k), L.uniform_s4(0x7A02, n, k)
        xp, wp = L.pack_bytes(x), L.pack_bytes(w)
        layer = ShardedInt4Linear(torch.from_numpy(wp[sh.row_start:sh.row_start + sh.rows]).to(dev), n, k)
        xd = torch.from_numpy(xp).to(dev)
        for rep in range(3):  # buffer reuse across calls
            fused = layer.forward(xd, gather="fused")
            torch.cuda.synchronize()
            ref = layer.forward(xd, gather=True)
            assert torch.equal(fused, ref), (rank, m, n, k, rep)
        if rank == 0:
            assert np.array_equal(fused.cpu().numpy(), oracle.linear_ref(x.astype(np.int32), w.astype(np.int32)))
    assert L.last_status() == 0
    dist.barrier()
    if rank == 0:
        print("GATHER_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
