"""Tensor-parallel plumbing for the quantized linear layer: column (N) sharding + all-gather.

Every output column depends on one weight row only (the reference already parallelises over
8-column groups, qwen3/src/qwen/quantized_gemx_kernels.cc:364-365), so rank r of P owns the
weight rows [r*N/P, (r+1)*N/P), every rank quantizes the full activations itself, and one
all-gather of the fp32 [M][N/P] shards assembles the output on every rank.  Per-column
arithmetic is identical at every rank count, so the gathered result equals the 1-GPU result
bit for bit.  Works with any torch.distributed backend (NCCL on GPUs, gloo in the CPU tests).
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
