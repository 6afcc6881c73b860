"""N-sharding of the linear layer across the GPUs of one node.

Y[:, j0:j1] = X @ W[j0:j1, :]^T, and W is stored N x K row-major, so an N-shard of W
is one contiguous byte range.  Every rank keeps the full X (replicated into its own
HBM) and its own rows of W, runs the single-GPU operator on (M, N/g, K) and owns the
matching columns of Y.  The GEMM needs no exchange at all; the only collective is the
OPTIONAL all-gather of Y for callers that want the full result everywhere.  The
reference has no multi-GPU code, so this module has no counterpart there; the
single-GPU operator it drives is the launcher of kernels/linear_v21.cu:9-49.

One process per GPU; `torch.distributed` (NCCL on GPUs, gloo in CPU tests) is the
plumbing.  Nothing here computes the operator on the CPU.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Shard:
    rank: int
    world: int
    row_start: int  # first row of W (= first column of Y) this rank owns
    rows: int       # number of rows of W (= columns of Y)


def shard_bounds(n: int, world: int, rank: int, align: int = 256) -> Shard:
    """Contiguous, balanced split of N in units of `align` rows (the widest output tile),
    so that no rank gets a ragged tile unless N itself is ragged.  Earlier ranks take the
    remainder units; the last non-empty rank absorbs the tail of N."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    if n <= 0:
        raise ValueError("n must be positive")
    units = (n + align - 1) // align
    base, extra = divmod(units, world)
    u0 = rank * base + min(rank, extra)
    u1 = u0 + base + (1 if rank < extra else 0)
    r0, r1 = min(u0 * align, n), min(u1 * align, n)
    return Shard(rank, world, r0, r1 - r0)


def all_shards(n: int, world: int, align: int = 256) -> list[Shard]:
    return [shard_bounds(n, world, r, align) for r in range(world)]


def shard_rows(w_packed, shard: Shard):
    """The rows of a full packed W (tensor or ndarray, [N, K/2]) that `shard` owns -- a view."""
    return w_packed[shard.row_start:shard.row_start + shard.rows]


def forward_local(x_packed, w_shard_packed, k: int | None = None, out=None, w_expanded=None):
    """This rank's columns of Y: the single-GPU operator on its shard (asynchronous).  With
    `w_expanded` (the shard expanded once by prepare_weights) and more than 128 rows of X the
    weights skip the in-kernel unpack."""
    from .linear import linear, linear_prepared
    if w_expanded is not None and x_packed.shape[0] > 128 and w_shard_packed.shape[0] > 0:
        return linear_prepared(x_packed, w_expanded, out=out)
    return linear(x_packed, w_shard_packed, k=k, out=out)


def gather_columns(y_local, n: int, group=None, align: int = 256):
    """All-gather of the column shards into the full [M, N] result on every rank.

    A row-major Y split by columns is not a contiguous concatenation, so the shards are
    gathered as [world][M][n_r] blocks and then copied into place.  Handles uneven shards
    (ranks may own different column counts, including zero)."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    shards = all_shards(n, world, align)
    m = y_local.shape[0]
    rank = dist.get_rank(group)
    if y_local.shape[1] != shards[rank].rows:
        raise ValueError("local result does not match this rank's shard")
    full = torch.empty((m, n), dtype=y_local.dtype, device=y_local.device)
    if all(s.rows == shards[0].rows for s in shards):
        stacked = torch.empty((world * m, shards[0].rows), dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(stacked, y_local.contiguous(), group=group)
        full.view(m, world, shards[0].rows).copy_(stacked.view(world, m, shards[0].rows).permute(1, 0, 2))
    else:
        # pad every shard to the widest one so a single collective moves everything
        widest = max(s.rows for s in shards)
        mine = torch.zeros((m, widest), dtype=y_local.dtype, device=y_local.device)
        mine[:, :y_local.shape[1]] = y_local
        stacked = torch.empty((world * m, widest), dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(stacked, mine, group=group)
        stacked = stacked.view(world, m, widest)
        for s in shards:
            if s.rows:
                full[:, s.row_start:s.row_start + s.rows] = stacked[s.rank, :, :s.rows]
    return full


class ShardedInt4Linear:
    """A weight-stationary N-sharded layer: holds this rank's rows of W on its GPU.

    expand_weights (default off): the shard is also kept expanded to bytes (twice the packed size,
    made on the first compute-bound call), and calls with more than 128 rows of X run with it:
    the weights then skip the in-kernel unpack.  Measured on one B200 in one run: +3 % at
    8192 x 8192 x 8192, -2.5 % at 8192 x 28672 x 8192, -3 to -6 % at 4096^3 (the expanded weights
    double the bytes TMA moves), so it is a per-layer choice.  Calls with few rows (decode) always
    use the packed weights, which is what they are bound by."""

    def __init__(self, w_shard_packed, n_total: int, k: int, group=None, align: int = 256, expand_weights: bool = False):
        import torch.distributed as dist
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.shard = shard_bounds(n_total, self.world, self.rank, align)
        if w_shard_packed.shape[0] != self.shard.rows:
            raise ValueError("weight shard has the wrong number of rows for this rank")
        self.w = w_shard_packed
        self.n_total, self.k, self.align = n_total, k, align
        self.expand_weights = expand_weights
        self._w_expanded = None

        self._fused = {}  # m -> FusedGatherBuffer

    def forward(self, x_packed, gather: bool | str = False):
        """gather=False: this rank's columns.  gather=True: full Y through an NCCL all-gather
        after the GEMM.  gather="fused": full Y written by the GEMM's own epilogue into every
        rank's symmetric result buffer (one kernel, no collective); the returned tensor is
        that buffer, reused by the next call with the same m."""
        if gather == "fused" and self.world > 1 and not self._fused_ok():
            gather = True  # every rank takes the same decision: it depends on the global split only
        if gather == "fused" and self.world > 1:
            m = x_packed.shape[0]
            buf = self._fused.get(m)
            if buf is None:
                buf = self._fused[m] = FusedGatherBuffer(m, self.n_total, x_packed.device, self.group)
            return buf.run(x_packed, self.w, self.shard, self.k)
        if self.expand_weights and self._w_expanded is None and x_packed.shape[0] > 128 and self.shard.rows > 0:
            from .linear import prepare_weights
            self._w_expanded = prepare_weights(self.w, self.k)
        y = forward_local(x_packed, self.w, self.k, w_expanded=self._w_expanded)
        if gather and self.world > 1:
            return gather_columns(y, self.n_total, self.group, self.align)
        return y


    def _fused_ok(self) -> bool:
        """The gathering kernel stores 32-column chunks: every shard must start and end on a
        32-column boundary and rows of Y must be 16-byte multiples."""
        return self.n_total % 4 == 0 and all(
            s.rows % 32 == 0 and s.row_start % 32 == 0 for s in all_shards(self.n_total, self.world, self.align))


class FusedGatherBuffer:
    """The full [m, n_total] int32 result of every rank, allocated as symmetric memory so that
    each rank holds an address for every peer's copy.  `run` launches the gathering GEMM
    (this rank's column block stored into all copies by the kernel's epilogue over NVLink) and
    then synchronises the ranks on the device, after which the local copy is complete.

    The exchange is plain stores to peer memory: no multicast, no loads from peers, no waits
    inside the GEMM kernel; the rank synchronisation is the symmetric-memory barrier, which runs
    as its own kernel after the GEMM on the same stream."""

    def __init__(self, m: int, n_total: int, device, group=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.m, self.n_total = m, n_total
        self.y = symm.empty((m, n_total), dtype=torch.int32, device=device)
        self.handle = symm.rendezvous(self.y, self.group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.world = self.handle.world_size

    def run(self, x_packed, w_shard_packed, shard: Shard, k: int | None = None, bias=None):
        from .linear import linear_gather
        # Nobody may still be reading the previous result when peers start overwriting it.
        self.handle.barrier(channel=0)
        if shard.rows:
            linear_gather(x_packed, w_shard_packed, self.ptrs, shard.row_start, self.n_total, k=k, bias=bias)
        self.handle.barrier(channel=1)
        return self.y
