"""GPU: the allocation-free decode entry point (inkq_linear_m1_static) against the regular
forward (inkq_linear, M == 1), through the C ABI.

Some hosts cannot allocate device memory while they serve - a decode loop with a hard
latency budget, a process whose device heap is owned by another allocator - so this entry
point keeps its scratch (one quantized activation row) in a fixed device array inside the
library.  The array is shared by every call and keeps the previous call's contents; the test
therefore runs two calls in a row with different inputs, shapes and schemes and checks each
against the regular path.  Collected last on purpose (file name), passes alone as well.
"""
import numpy as np
import pytest

from conftest import rel_err
from test_gpu_matmul import GEMV_TOL

pytestmark = pytest.mark.gpu


def test_two_calls_in_a_row_match_the_regular_forward(pkg, gpu):
    import torch
    cases = [(pkg.A81W41, 4096, 4096, 11), (pkg.A80W4Z, 1024, 512, 12), (pkg.A81W41, 136, 12288, 13)]
    for scheme, N, K, seed in cases:              # back to back: each call finds the previous call's bytes in the scratch
        w = pkg.synth.weights(N, K, seed)
        wh = gpu.weight(scheme, pkg.SCALES_F16, w["nib"], w["d"], w["m"], w["zp"])
        x = torch.from_numpy(pkg.synth.activations(1, K, seed)).cuda()
        want = torch.empty((1, N), device="cuda")
        got = torch.full((1, N + 4), -5.0, device="cuda")
        gpu.linear(wh, x, 1, want, N)
        gpu.linear_m1_static(wh, x, got)
        gpu.synchronize()
        g, r = got.cpu().numpy(), want.cpu().numpy()
        assert np.all(g[0, N:] == -5.0)
        assert rel_err(g[:, :N], r) < GEMV_TOL
        assert np.array_equal(g[:, :N], r)        # same kernels on the same data: in fact identical


def test_calls_leave_the_free_device_memory_unchanged(pkg, gpu):
    """The property in the entry point's name: around calls of it, cudaMemGetInfo reports the same free figure.
    Everything the test itself needs is allocated first, and one call is made before the measurement because the
    first use of a kernel makes the driver load its code."""
    import torch
    N, K = 4096, 4096
    w = pkg.synth.weights(N, K, 21)
    wh = gpu.weight(pkg.A81W41, pkg.SCALES_F16, w["nib"], w["d"], w["m"])
    x = torch.from_numpy(pkg.synth.activations(1, K, 21)).cuda()
    out = torch.empty((1, N), device="cuda")
    gpu.linear_m1_static(wh, x, out)
    gpu.synchronize()
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(5):
        gpu.linear_m1_static(wh, x, out)
    gpu.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, f"free device memory changed by {free_before - free_after} bytes across the calls"


def test_sizes_beyond_the_static_scratch_are_rejected(pkg, gpu):
    import torch
    K = 16384 + 64
    w = pkg.synth.weights(8, K, 1)
    wh = gpu.weight(pkg.A81W41, pkg.SCALES_F16, w["nib"], w["d"], w["m"])
    x = torch.zeros((1, K), device="cuda")
    out = torch.zeros((1, 8), device="cuda")
    with pytest.raises(pkg.InkqError) as e:
        gpu.linear_m1_static(wh, x, out)
    assert e.value.code == pkg.ERR_UNSUPPORTED and "16384" in str(e.value)
