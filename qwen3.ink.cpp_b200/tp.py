"""Tensor-parallel plumbing for the quantized linear layer: column (N) sharding + all-gather.

Every output column depends on one weight row only (the reference already parallelises over
8-column groups, qwen3/src/qwen/quantized_gemx_kernels.cc:364-365), so rank r of P owns the
weight rows [r*N/P, (r+1)*N/P), every rank quantizes the full activations itself, and one
all-gather of the fp32 [M][N/P] shards assembles the output on every rank.  Per-column
arithmetic is identical at every rank count, so the gathered result equals the 1-GPU result
bit for bit.  Works with any torch.distributed backend (NCCL on GPUs, gloo in the CPU tests).

Two ways to do the exchange:
  ColumnGather  kernel writes its shard locally, then one all-gather (the library collective) and a
                re-layout copy;
  PeerScatter   the matmul's epilogue stores each finished element into every rank's [M][N] buffer
                through peer-mapped pointers (csrc/peer.cu), followed by a small barrier kernel; no
                collective call and no re-layout.  torch.distributed only carries the 80-byte buffer
                handles at set-up.
"""
from __future__ import annotations


def shard_range(N: int, world: int, rank: int, multiple: int = 8):
    """Rows [n_begin, n_end) of rank `rank`: equal shards whose size is a multiple of `multiple`
    (the layer needs N % 8 == 0 per shard)."""
    if N % (world * multiple) != 0:
        raise ValueError(f"N={N} does not split into {world} shards of a multiple of {multiple} rows")
    n_loc = N // world
    return rank * n_loc, (rank + 1) * n_loc


class ColumnGather:
    """Pre-allocated buffers for gathering [M][N/P] shards into [M][N].

    `local` is the view each rank's kernel writes its shard into (slot `rank` of the rank-major
    gather buffer, so the all-gather runs in place); `gather()` returns the [M][N] matrix."""

    def __init__(self, dist, M: int, N: int, world: int, rank: int, device, dtype):
        import torch
        self.dist, self.M, self.N, self.world, self.rank = dist, M, N, world, rank
        self.n_loc = N // world
        self.stacked = torch.empty((world, M, self.n_loc), device=device, dtype=dtype)   # [P][M][N/P]
        self.full = torch.empty((M, N), device=device, dtype=dtype)
        self.local = self.stacked[rank]

    def gather(self):
        if self.world == 1:
            return self.local
        self.dist.all_gather_into_tensor(self.stacked.view(-1), self.local.reshape(-1))
        # [P][M][N/P] -> [M][P][N/P] = [M][N]
        self.full.view(self.M, self.world, self.n_loc).copy_(self.stacked.permute(1, 0, 2))
        return self.full


def scatter_offset(slot: int, M: int, N: int, n_begin: int, reserved: int = 256) -> int:
    """Byte offset, inside every rank's peer buffer, of element [0][n_begin] of output slot `slot`
    ([slots][M][N] fp32 after the reserved head)."""
    return reserved + 4 * (slot * M * N + n_begin)


class PeerScatter:
    """[slots][M][N] fp32 output buffers, one per rank, each mapped into every rank's process.

    `linear(w_shard, x, slot)` runs quantize + QGEMM/QGEMV on the rank's weight rows and stores the
    columns [n_begin, n_end) of slot `slot` on every rank; `barrier()` completes the exchange;
    `result(slot)` is then the full [M][N] matrix.  Alternate two slots between consecutive steps."""

    def __init__(self, pkg, ctx, dist, M: int, N: int, world: int, rank: int, slots: int = 2):
        import torch
        self.pkg, self.ctx, self.dist, self.M, self.N, self.world, self.rank, self.slots = pkg, ctx, dist, M, N, world, rank, slots
        self.n_begin, self.n_end = shard_range(N, world, rank)
        nbytes = pkg.PEER_RESERVED_BYTES + 4 * slots * M * N
        self.buf = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")      # zero head: the barrier counters start at 0
        torch.cuda.synchronize()
        # Set-up is collective: every rank takes part in both exchanges whatever happened locally, and all
        # ranks raise together, so that a caller can fall back to ColumnGather without a rank left behind.
        err = None
        try:
            blob = ctx.peer_export(self.buf)
        except Exception as e:           # e.g. an allocator whose memory CUDA IPC cannot export
            err, blob = e, b""
        blobs = self._all_gather(blob)
        self.ps = None
        if all(len(b) == pkg.PEER_HANDLE_BYTES for b in blobs):
            try:
                self.ps = ctx.peerset_open(world, rank, self.buf, blobs)
            except Exception as e:
                err = e
        oks = self._all_gather(self.ps is not None)
        if not all(oks):
            if self.ps is not None:
                self.ps.close()
            raise RuntimeError(f"peer buffers could not be mapped on every rank (this rank: {err!r})")
        self.out = self.buf[pkg.PEER_RESERVED_BYTES:].view(torch.float32).view(slots, M, N)

    def _all_gather(self, obj):
        if self.world == 1:
            return [obj]
        out = [None] * self.world
        self.dist.all_gather_object(out, obj)
        return out

    def linear(self, w, x, slot: int):
        self.ctx.linear_scatter(w, x, self.M, self.ps, scatter_offset(slot, self.M, self.N, self.n_begin, self.pkg.PEER_RESERVED_BYTES), self.N)

    def barrier(self, timeout_ms: int = 2000):
        if self.world > 1:
            self.ctx.peer_barrier(self.ps, timeout_ms)

    def result(self, slot: int):
        return self.out[slot]

    def close(self):
        if self.world > 1:
            self.ctx.synchronize()
            self.dist.barrier()   # nobody unmaps while a peer may still store
        self.ps.close()


class PeerArena:
    """One peer-mapped byte buffer per rank holding several named fp32 [rows][cols] regions (the outputs of a model's
    column-sharded linears).  `linear(name, w_shard, x, M, n_begin)` runs the sharded forward and stores the shard's
    columns of region `name` on every rank; `f16w(name, ...)` does the same for an fp16 matrix; `barrier()` completes
    the exchange.  A region may be rewritten only after every rank has passed a barrier that follows its last reader,
    which holds whenever consecutive linears use different regions and each is followed by a barrier."""

    def __init__(self, pkg, ctx, dist, world: int, rank: int, regions: dict):
        import torch
        self.pkg, self.ctx, self.dist, self.world, self.rank = pkg, ctx, dist, world, rank
        self.off, self.shape = {}, {}
        pos = pkg.PEER_RESERVED_BYTES
        for name, (rows, cols) in regions.items():
            self.off[name], self.shape[name] = pos, (rows, cols)
            pos += (4 * rows * cols + 255) // 256 * 256
        self.buf = torch.zeros(pos, dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()
        err = None
        try:
            blob = ctx.peer_export(self.buf)
        except Exception as e:
            err, blob = e, b""
        blobs = [None] * world
        dist.all_gather_object(blobs, blob)
        self.ps = None
        if all(len(b) == pkg.PEER_HANDLE_BYTES for b in blobs):
            try:
                self.ps = ctx.peerset_open(world, rank, self.buf, blobs)
            except Exception as e:
                err = e
        oks = [None] * world
        dist.all_gather_object(oks, self.ps is not None)
        if not all(oks):
            if self.ps is not None:
                self.ps.close()
            raise RuntimeError(f"peer buffers could not be mapped on every rank (this rank: {err!r})")

    def view(self, name, rows=None):
        import torch
        r, c = self.shape[name]
        rows = r if rows is None else rows
        return self.buf[self.off[name]:self.off[name] + 4 * rows * c].view(torch.float32).view(rows, c)

    def linear(self, name, w, x, M: int, n_begin: int):
        cols = self.shape[name][1]
        self.ctx.linear_scatter(w, x, M, self.ps, self.off[name] + 4 * n_begin, cols)

    def gemm(self, name, w, act, n_begin: int):
        """The same for rows that are already quantized into the activation handle `act`."""
        cols = self.shape[name][1]
        self.ctx.gemm_scatter(act, w, self.ps, self.off[name] + 4 * n_begin, cols)

    def f16w(self, name, w, x, M: int, n_begin: int, precision: int = 0):
        cols = self.shape[name][1]
        self.ctx.f16w_matmul_scatter(w, x, M, self.ps, self.off[name] + 4 * n_begin, cols, precision)

    def barrier(self, timeout_ms: int = 2000):
        self.ctx.peer_barrier(self.ps, timeout_ms)

    def close(self):
        self.ctx.synchronize()
        self.dist.barrier()   # nobody unmaps while a peer may still store
        self.ps.close()
