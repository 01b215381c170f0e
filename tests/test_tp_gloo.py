"""CPU, world_size 2 over gloo: the tensor-parallel host logic (row-range sharding of the
weights, in-place all-gather of the column shards, re-layout to [M][N]).  Each rank computes its
shard with the oracle's A81W41 arithmetic; the gathered result must equal the unsharded
result bit for bit, which is the property the GPU path relies on."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from conftest import ROOT


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    from __graft_entry__ import load_package
    from oracle.inkq_oracle import Oracle
    pkg = load_package()
    dist.init_process_group("gloo", rank=rank, world_size=world)
    M, N, K = 5, 64, 128
    x = pkg.synth.activations(M, K, 3)
    w = pkg.synth.weights(N, K, 3)
    orc = Oracle()
    q, d, s = orc.quantize(x, 2)                       # every rank quantizes the full activations
    n0, n1 = pkg.tp.shard_range(N, world, rank)
    cg = pkg.tp.ColumnGather(dist, M, N, world, rank, "cpu", torch.float32)
    shard = orc.gemm(0, q, d, s, w["nib"][n0:n1], w["d"][n0:n1], w["m"][n0:n1])
    cg.local.copy_(torch.from_numpy(shard))
    full = cg.gather().numpy()
    ref = orc.gemm(0, q, d, s, w["nib"], w["d"], w["m"])
    ok = np.array_equal(full.view(np.uint32), ref.view(np.uint32))
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write("ok" if ok else "mismatch")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_sharded_result_equals_unsharded(tmp_path, world):
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"rank{r}.txt").read() == "ok"


def test_shard_ranges(pkg):
    assert pkg.tp.shard_range(12288, 8, 3) == (4608, 6144)
    assert pkg.tp.shard_range(151936, 8, 7) == (132944, 151936)
    with pytest.raises(ValueError):
        pkg.tp.shard_range(12288 + 8, 8, 0)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_scatter_offsets_tile_every_slot_exactly_once(pkg, world):
    """The byte ranges the ranks' epilogues store to (row m of slot s: scatter_offset + 4*m*N .. + 4*n_loc)
    cover [slots][M][N] after the reserved head exactly once."""
    M, N, slots = 5, 64 * world, 2
    hit = np.zeros(pkg.PEER_RESERVED_BYTES + 4 * slots * M * N, np.int32)
    for s in range(slots):
        for r in range(world):
            n0, n1 = pkg.tp.shard_range(N, world, r)
            off = pkg.tp.scatter_offset(s, M, N, n0, pkg.PEER_RESERVED_BYTES)
            for m in range(M):
                hit[off + 4 * m * N: off + 4 * (m * N + n1 - n0)] += 1
    assert (hit[:pkg.PEER_RESERVED_BYTES] == 0).all() and (hit[pkg.PEER_RESERVED_BYTES:] == 1).all()
