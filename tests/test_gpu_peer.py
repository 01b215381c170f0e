"""GPU (one device): the multi-destination epilogue and the bounded barrier of the column-sharded
layer (csrc/peer.cu), with the peers' buffers standing in as further buffers on the same GPU.
 - two emulated ranks, run one after the other, each store their columns into both buffers: both
   buffers then hold the unsharded result bit for bit (prefill QGEMM and decode QGEMV epilogues)
 - a barrier whose peer never arrives gives up after its time limit, the host reads
   INKQ_ERR_TIMEOUT, the arrival was still delivered, and the context keeps working
 - argument checks
The two-process version over NVLink is in test_gpu_tp.py.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _buffers(torch, pkg, n, nbytes):
    return [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(n)]


@pytest.mark.parametrize("M", [1, 37, 322])
@pytest.mark.parametrize("scheme_name", ["A81W41", "A80W40"])
def test_emulated_ranks_fill_every_buffer(pkg, gpu, M, scheme_name):
    import torch
    scheme = getattr(pkg, scheme_name)
    N, K, world = 512, 256, 2
    x = torch.from_numpy(pkg.synth.activations(M, K, 21)).cuda()
    w = pkg.synth.weights(N, K, 21)
    m_or_none = w["m"] if scheme == pkg.A81W41 else None
    whole = gpu.weight(scheme, pkg.SCALES_F16, w["nib"], w["d"], m_or_none)
    ref = torch.empty((M, N), device="cuda")
    gpu.linear(whole, x, M, ref, N)
    bufs = _buffers(torch, pkg, world, pkg.PEER_RESERVED_BYTES + 4 * M * N)
    for rank in range(world):
        n0, n1 = pkg.tp.shard_range(N, world, rank)
        shard = gpu.weight(scheme, pkg.SCALES_F16, w["nib"], w["d"], m_or_none, None, n0, n1)
        ps = gpu.peerset_from_tensors(rank, bufs)
        gpu.linear_scatter(shard, x, M, ps, pkg.tp.scatter_offset(0, M, N, n0), N)
        gpu.synchronize()
        ps.close()
    for b in bufs:
        got = b[pkg.PEER_RESERVED_BYTES:].view(torch.float32).view(M, N)
        assert torch.equal(got, ref)
        assert int(b[:pkg.PEER_RESERVED_BYTES].view(torch.int32).abs().sum().item()) == 0   # the head is the barrier's alone


def test_barrier_gives_up_when_the_peer_never_arrives(pkg, gpu):
    import torch
    bufs = _buffers(torch, pkg, 2, pkg.PEER_RESERVED_BYTES + 4096)
    ps = gpu.peerset_from_tensors(0, bufs)
    gpu.peer_barrier(ps, timeout_ms=50)
    with pytest.raises(pkg.InkqError) as e:
        gpu.synchronize()
    assert e.value.code == 5                                     # INKQ_ERR_TIMEOUT
    heads = [b[:pkg.PEER_RESERVED_BYTES].view(torch.int32).cpu().numpy() for b in bufs]
    assert heads[1][0] == 1                                      # rank 0's arrival reached rank 1's buffer
    assert heads[0][16] == 1                                     # rank 0 counted its barrier
    gpu.synchronize()                                            # the flag was cleared, the context works on
    ps.close()
    # a set of one rank has nobody to wait for
    ps1 = gpu.peerset_from_tensors(0, bufs[:1])
    gpu.peer_barrier(ps1, timeout_ms=50)
    gpu.synchronize()
    ps1.close()


def test_emulated_barrier_pair_completes(pkg, gpu):
    """Rank 1's arrival is already in rank 0's buffer when rank 0 runs its barrier (and the other way round):
    neither kernel has to wait for a kernel that has not run yet."""
    import torch
    bufs = _buffers(torch, pkg, 2, pkg.PEER_RESERVED_BYTES + 4096)
    bufs[0][:pkg.PEER_RESERVED_BYTES].view(torch.int32)[1] = 1   # as if rank 1 had arrived at rank 0
    torch.cuda.synchronize()
    ps0, ps1 = gpu.peerset_from_tensors(0, bufs), gpu.peerset_from_tensors(1, bufs)
    gpu.peer_barrier(ps0, timeout_ms=200)                       # finds rank 1's arrival, delivers its own
    gpu.synchronize()
    gpu.peer_barrier(ps1, timeout_ms=200)                       # finds rank 0's arrival
    gpu.synchronize()
    ps0.close()
    ps1.close()


def test_scatter_argument_checks(pkg, gpu):
    import torch
    N, K = 256, 128
    w = pkg.synth.weights(N, K, 22)
    wh = gpu.weight(pkg.A81W41, pkg.SCALES_F16, w["nib"], w["d"], w["m"])
    x = torch.zeros((4, K), device="cuda")
    bufs = _buffers(torch, pkg, 2, pkg.PEER_RESERVED_BYTES + 4 * 4 * N)
    ps = gpu.peerset_from_tensors(0, bufs)
    with pytest.raises(pkg.InkqError):
        gpu.linear_scatter(wh, x, 4, ps, 0, N)                   # inside the reserved head
    with pytest.raises(pkg.InkqError):
        gpu.linear_scatter(wh, x, 5, ps, pkg.PEER_RESERVED_BYTES, N)   # does not fit
    with pytest.raises(pkg.InkqError):
        gpu.peer_barrier(ps, timeout_ms=0)
    ps.close()
    with pytest.raises(pkg.InkqError):
        gpu.peerset_from_tensors(3, bufs)                        # rank outside the world


@pytest.mark.parametrize("M", [1, 322])
def test_one_process_driving_two_devices(pkg, gpu, M):
    """The mode inkq_peerset_from_pointers documents for a single process that owns every GPU: one context per device,
    every rank's buffer addressed directly (peer access enabled), the two barrier kernels meeting across NVLink.  Also
    the first launch of the tensor-core kernels on a second device of the process (their shared-memory opt-in is per
    device).  Needs two visible GPUs."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible GPUs")
    if not (torch.cuda.can_device_access_peer(0, 1) and torch.cuda.can_device_access_peer(1, 0)):
        pytest.skip("the two GPUs cannot address each other")
    N, K, world = 1024, 512, 2
    x_host = pkg.synth.activations(M, K, 23)
    w = pkg.synth.weights(N, K, 23)
    whole = gpu.weight(pkg.A81W41, pkg.SCALES_F16, w["nib"], w["d"], w["m"])
    x0 = torch.from_numpy(x_host).cuda(0)
    ref = torch.empty((M, N), device="cuda:0")
    gpu.linear(whole, x0, M, ref, N)
    gpu.synchronize()
    nbytes = pkg.PEER_RESERVED_BYTES + 4 * M * N
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=f"cuda:{d}") for d in range(world)]
    # a copy in each direction makes torch enable peer access between the two devices
    bufs[0][:16].to("cuda:1")
    bufs[1][:16].to("cuda:0")
    torch.cuda.synchronize(0)
    torch.cuda.synchronize(1)
    ctxs, sets, keep = [], [], []
    try:
        for rank in range(world):
            with torch.cuda.device(rank):
                ctx = gpu if rank == 0 else pkg.Context(rank, torch.cuda.current_stream(rank).cuda_stream)
                ctxs.append(ctx)
                n0, n1 = pkg.tp.shard_range(N, world, rank)
                shard = ctx.weight(pkg.A81W41, pkg.SCALES_F16, w["nib"], w["d"], w["m"], None, n0, n1)
                xr = x0 if rank == 0 else torch.from_numpy(x_host).cuda(rank)
                ps = ctx.peerset_from_tensors(rank, bufs)
                sets.append(ps)
                keep += [shard, xr]
                ctx.linear_scatter(shard, xr, M, ps, pkg.tp.scatter_offset(0, M, N, n0), N)
        for rank in range(world):                         # asynchronous launches: rank 0's barrier kernel waits on its GPU
            with torch.cuda.device(rank):                 # for the arrival that rank 1's kernel sends from the other one
                ctxs[rank].peer_barrier(sets[rank], timeout_ms=5000)
        for ctx in ctxs:
            ctx.synchronize()
        for d, b in enumerate(bufs):
            got = b[pkg.PEER_RESERVED_BYTES:].view(torch.float32).view(M, N)
            assert torch.equal(got.to("cuda:0"), ref), f"buffer of device {d}"
    finally:
        for ps in sets:
            ps.close()
        for ctx in ctxs[1:]:
            ctx.close()
        torch.cuda.set_device(0)
