"""GPU: QGEMV, tensor-core QGEMM and the CUDA-core cross-check, through the C ABI,
against the oracle and the reference's golden outputs.
 - every int32 block dot: exact
 - QGEMM fp32 output: bit-identical to the reference order
 - QGEMV fp32 output: within 5e-4 of the oracle in the measure of conftest.rel_err
   (8 K-slices summed in ascending order; documented in csrc/qgemv.cu); the project
   tolerance is 1e-3
 - fp16 lm_head: within 1e-3 of the exact (double-accumulated) value
"""
import numpy as np
import pytest

from conftest import f16, rel_err

pytestmark = pytest.mark.gpu

GEMV_TOL = 5e-4
SCHEMES = {0: ("A81W41", 2, 1), 1: ("A80W40", 0, 0), 2: ("A80W4Z", 0, 0)}  # scheme -> (name, gemm qmode, gemv qmode)


def setup(pkg, gpu, oracle, scheme, M, N, K, scale_mode, seed=0, qmode=None):
    import torch
    x = pkg.synth.activations(M, K, 50 + seed)
    w = pkg.synth.weights(N, K, seed)
    if scale_mode == 0:
        w["d"] = (w["d"] * np.float32(1.0003)).astype(np.float32)
        w["m"] = (w["m"] * np.float32(0.9997)).astype(np.float32)
    wh = gpu.weight(scheme, scale_mode, w["nib"], w["d"], w["m"], w["zp"])
    act = gpu.act(M, K)
    xd = torch.from_numpy(x).cuda()
    gpu.quantize(act, xd, M, qmode)
    q, d, s = oracle.quantize(x, qmode)
    return x, w, wh, act, (q, d, s)


def oracle_out(oracle, scheme, qds, w, scale_mode, want_dots=False):
    q, d, s = qds
    dw = w["d"] if scale_mode == 0 else f16(w["d"])
    mw = w["m"] if scale_mode == 0 else f16(w["m"])
    return oracle.gemm(scheme, q, d, s if scheme == 0 else None, w["nib"], dw, mw if scheme == 0 else None,
                       w["zp"] if scheme == 2 else None, want_dots=want_dots)


# ------------------------------------------------------------------ QGEMV
@pytest.mark.parametrize("N,K", [(8, 64), (136, 512), (1024, 4096), (4096, 4096), (4096, 12288)])
@pytest.mark.parametrize("scheme", [0, 1, 2])
def test_gemv_matches_oracle(pkg, gpu, oracle, scheme, N, K):
    import torch
    qmode = SCHEMES[scheme][2] if scheme else 1
    x, w, wh, act, qds = setup(pkg, gpu, oracle, scheme, 1, N, K, 1, seed=scheme, qmode=qmode)
    C = torch.full((1, N + 8), -777.0, device="cuda")
    gpu.gemv(act, wh, C)
    gpu.synchronize()
    ref = oracle_out(oracle, scheme, qds, w, 1)
    got = C.cpu().numpy()
    assert np.all(got[0, N:] == -777.0)                      # nothing written past the output
    assert rel_err(got[:, :N], ref) < GEMV_TOL


def test_gemv_matches_reference_golden(pkg, gpu, golden):
    import torch
    g = golden("ref_gemv_a81w41_fp16.npz")
    N, K = g["nib"].shape[0], g["nib"].shape[1] * 2
    wh = gpu.weight(0, 1, g["nib"], g["d"], g["m"])
    act = gpu.act(1, K)
    gpu.quantize(act, torch.from_numpy(g["x"]).cuda(), 1, 1)
    C = torch.empty((1, N), device="cuda")
    gpu.gemv(act, wh, C)
    gpu.synchronize()
    assert rel_err(C.cpu().numpy(), g["C"]) < GEMV_TOL


# ------------------------------------------------------------------ int32 block dots
@pytest.mark.parametrize("tensor_core", [False, True])
@pytest.mark.parametrize("scheme,M,N,K", [(0, 1, 8, 64), (0, 5, 136, 256), (1, 13, 264, 192), (2, 37, 128, 512), (0, 130, 256, 128)])
def test_block_dots_exact(pkg, gpu, oracle, tensor_core, scheme, M, N, K):
    import torch
    qmode = 2 if scheme == 0 else 0
    x, w, wh, act, qds = setup(pkg, gpu, oracle, scheme, M, N, K, 1, seed=3, qmode=qmode)
    dots = torch.full((M, N, K // 32), 123456789, dtype=torch.int32, device="cuda")
    gpu.block_dots(act, wh, dots, tensor_core=tensor_core)
    gpu.synchronize()
    _, ref = oracle_out(oracle, scheme, qds, w, 1, want_dots=True)
    assert np.array_equal(dots.cpu().numpy(), ref)


# ------------------------------------------------------------------ QGEMM
@pytest.mark.parametrize("impl", ["simt", "tc"])
@pytest.mark.parametrize("scheme,scale_mode,M,N,K", [
    (0, 0, 2, 8, 64), (0, 0, 5, 136, 256), (0, 0, 6, 24, 128), (0, 0, 7, 16, 4096), (0, 0, 13, 136, 192),
    (0, 1, 16, 128, 256), (0, 0, 17, 264, 320), (0, 0, 129, 128, 128), (0, 0, 322, 384, 512),
    (1, 1, 6, 32, 256), (1, 1, 150, 200, 448), (2, 1, 5, 16, 64), (2, 1, 257, 136, 256)])
def test_gemm_bit_identical_to_oracle(pkg, gpu, oracle, impl, scheme, scale_mode, M, N, K):
    import torch
    qmode = 2 if scheme == 0 else 0
    x, w, wh, act, qds = setup(pkg, gpu, oracle, scheme, M, N, K, scale_mode, seed=M, qmode=qmode)
    ldc = N + 8
    C = torch.full((M + 1, ldc), -777.0, device="cuda")
    (gpu.gemm if impl == "tc" else gpu.gemm_simt)(act, wh, C, ldc)
    gpu.synchronize()
    got = C.cpu().numpy()
    ref = oracle_out(oracle, scheme, qds, w, scale_mode)
    assert np.all(got[:M, N:] == -777.0) and np.all(got[M] == -777.0)   # guard band untouched
    assert np.array_equal(got[:M, :N].view(np.uint32), ref.view(np.uint32)), f"max abs diff {np.abs(got[:M, :N] - ref).max()}"


@pytest.mark.parametrize("M", [2, 5, 6, 7, 13])
def test_gemm_matches_reference_golden(pkg, gpu, golden, M):
    import torch
    g = golden("ref_gemm_a81w41_fp32.npz")
    N, K = g["nib"].shape[0], g["nib"].shape[1] * 2
    wh = gpu.weight(0, 0, g["nib"], g["d"], g["m"])
    C = torch.empty((M, N), device="cuda")
    gpu.linear(wh, torch.from_numpy(g[f"x_M{M}"]).cuda(), M, C, N)      # the layer's forward(): quantize + QGEMM
    gpu.synchronize()
    assert np.array_equal(C.cpu().numpy().view(np.uint32), g[f"C_M{M}"].view(np.uint32))


def test_reference_throughput_recipe(pkg, gpu, golden):
    import torch
    g = golden("ref_testlinear_recipe.npz")
    N, K, M = g["nib"].shape[0], g["nib"].shape[1] * 2, g["x"].shape[0]
    wh = gpu.weight(0, 0, g["nib"], g["d"], g["m"])
    C = torch.empty((M, N), device="cuda")
    gpu.linear(wh, torch.from_numpy(g["x"]).cuda(), M, C, N)
    gpu.synchronize()
    assert np.array_equal(C.cpu().numpy().view(np.uint32), g["C"].view(np.uint32))


def test_a80w40_matches_reference_golden(pkg, gpu, golden):
    import torch
    g = golden("ref_a80w40.npz")
    N, K, M = g["nib"].shape[0], g["nib"].shape[1] * 2, g["x"].shape[0]
    wh = gpu.weight(1, 1, g["nib"], g["d"])
    C = torch.empty((M, N), device="cuda")
    gpu.linear(wh, torch.from_numpy(g["x"]).cuda(), M, C, N)
    gpu.synchronize()
    assert np.array_equal(C.cpu().numpy().view(np.uint32), g["C_gemm"].view(np.uint32))
    C1 = torch.empty((1, N), device="cuda")
    gpu.linear(wh, torch.from_numpy(g["x"][:1]).cuda(), 1, C1, N)
    gpu.synchronize()
    assert rel_err(C1.cpu().numpy(), g["C_gemv"]) < GEMV_TOL


# ------------------------------------------------------------------ full benchmark shape, properties + samples
def test_full_prefill_shape(pkg, gpu, oracle):
    """M=322, K=4096, N=12288 (the pp322 gate_proj shape): tensor-core result equals the
    CUDA-core cross-check everywhere and the oracle on sampled outputs; linear_host equals
    the device path; doubling the activations doubles the result exactly (power-of-two linearity)."""
    import torch
    M, N, K = 322, 12288, 4096
    x = pkg.synth.activations(M, K)
    w = pkg.synth.weights(N, K)
    wh = gpu.weight(0, 0, w["nib"], w["d"], w["m"])
    xd = torch.from_numpy(x).cuda()
    C = torch.empty((M, N), device="cuda")
    gpu.linear(wh, xd, M, C, N)
    act = gpu.act(M, K)
    gpu.quantize(act, xd, M, 2)
    C2 = torch.empty((M, N), device="cuda")
    gpu.gemm_simt(act, wh, C2, N)
    gpu.synchronize()
    assert torch.equal(C, C2)
    rng = np.random.default_rng(0)
    rows, cols = rng.integers(0, M, 4000), rng.integers(0, N, 4000)
    rows[:4], cols[:4] = [0, M - 1, 0, M - 1], [0, 0, N - 1, N - 1]
    q, d, s = oracle.quantize(x, 2)
    ref = oracle.gemm_samples(0, q, d, s, w["nib"], w["d"], w["m"], None, rows, cols)
    got = C.cpu().numpy()
    assert np.array_equal(got[rows, cols].view(np.uint32), ref.view(np.uint32))
    Ch = np.empty((M, N), np.float32)
    gpu.linear_host(wh, x, M, Ch, N)
    assert np.array_equal(Ch, got)
    C3 = torch.empty((M, N), device="cuda")
    gpu.linear(wh, xd * 2.0, M, C3, N)
    gpu.synchronize()
    assert torch.equal(C3, C * 2.0)


@pytest.mark.parametrize("scheme", [0, 1])
@pytest.mark.parametrize("M", [37, 97, 130, 322, 1100])
def test_linear_host_row_windows(pkg, gpu, scheme, M):
    """inkq_linear_host works on windows of rows from M = 96 on (activations in, quantizer + QGEMM, finished rows out, on
    three streams): ragged last window and last weight tile, padded host rows (ldc > N); equals the device path bit for
    bit, leaves the padding untouched, and a second call right behind the first does not disturb it."""
    import torch
    N, K, ldc = 1064, 128, 1072           # 9 weight tiles, the last one 40 rows
    w = pkg.synth.weights(N, K, 41)
    wh = gpu.weight(scheme, pkg.SCALES_F16, w["nib"], w["d"], w["m"] if scheme == 0 else None)
    x = pkg.synth.activations(M, K, 41)
    C = torch.empty((M, N), device="cuda")
    gpu.linear(wh, torch.from_numpy(x).cuda(), M, C, N)
    gpu.synchronize()
    Ch = np.full((M, ldc), -7.0, np.float32)
    gpu.linear_host(wh, x, M, Ch, ldc)
    assert np.array_equal(Ch[:, :N], C.cpu().numpy()) and (Ch[:, N:] == -7.0).all()
    x2 = pkg.synth.activations(M, K, 43)
    C2 = torch.empty((M, N), device="cuda")
    Ch2 = np.empty((M, N), np.float32)
    gpu.linear_host(wh, x2, M, Ch2, N)
    gpu.linear(wh, torch.from_numpy(x2).cuda(), M, C2, N)
    gpu.synchronize()
    assert np.array_equal(Ch2, C2.cpu().numpy())


def test_mismatched_quantizer_mode_is_rejected(pkg, gpu, oracle):
    import torch
    x, w, wh, act, _ = setup(pkg, gpu, oracle, 0, 4, 16, 64, 0, qmode=0)   # Q8_0 activations, A81W41 weights
    C = torch.empty((4, 16), device="cuda")
    with pytest.raises(pkg.InkqError) as e:
        gpu.gemm(act, wh, C, 16)
    assert e.value.code == pkg.ERR_INVALID
    with pytest.raises(pkg.InkqError):
        gpu.gemm(act, wh, C, 8)    # ldc < rows


# ------------------------------------------------------------------ weight-only W41 and fp16 lm_head
@pytest.mark.parametrize("M,N,K", [(9, 72, 256), (1, 256, 128), (1, 1064, 512), (1, 4096, 4096), (1, 512, 12288),   # M == 1: the streaming kernel
                                   (16, 128, 64), (322, 384, 512), (200, 136, 1024), (400, 264, 192),
                                   # enough work items for the two-weight-tiles-per-CTA variant: an odd tile count (the last
                                   # group holds one tile), and two activation tiles of 160 rows
                                   (16, 297 * 128, 64), (300, 74 * 256, 128)])
def test_weight_only_w41(pkg, gpu, oracle, M, N, K):
    """Tensor-core kernel (kind::f16, fp32 accumulation inside tensor memory) and its CUDA-core cross-check against
    the oracle.  The dequantised fp16 weights are identical in all three (one rounding of q*d + m); only the fp32
    summation order differs: k ascending in the oracle and the cross-check, the hardware's in the tensor-core kernel."""
    import torch
    w = pkg.synth.weights(N, K, 4)
    a16 = pkg.synth.activations(M, K, 4).astype(np.float16)
    wh = gpu.weight(3, 1, w["nib"], w["d"], w["m"])
    a_dev = torch.from_numpy(a16).cuda()
    C = torch.full((M + 1, N), 7.0, device="cuda")
    gpu.gemm_w41_f16act(a_dev, M, wh, C, N)
    Cs = torch.empty((M, N), device="cuda")
    gpu.gemm_w41_f16act_simt(a_dev, M, wh, Cs, N)
    gpu.synchronize()
    ref = oracle.gemm_w41_f16act(a16, w["nib"], w["d"], w["m"])
    assert rel_err(Cs.cpu().numpy(), ref) < 1e-5
    # Another summation order moves an fp32 sum of K terms by a few ulps of the terms' magnitude, whatever the size
    # of the result, so the bound is relative to the output's rms (observed 2e-6), not to each element.
    got = C[:M].cpu().numpy()
    assert np.abs(got - ref).max() / np.sqrt(np.mean(ref.astype(np.float64) ** 2)) < 1e-4
    assert bool((C[M] == 7.0).all())                          # nothing stored past row M


def test_weight_only_w41_dequantisation_bits(pkg, gpu, oracle):
    """One-hot fp16 activations read the dequantised weights back out of both GPU kernels: they must be the oracle's
    single rounding of q*d + m bit for bit, also for scales of very different exponents."""
    import torch
    rng = np.random.default_rng(78)
    N, K = 256, 128
    q = rng.integers(0, 16, size=(N, K), dtype=np.uint8)
    d = (rng.uniform(0.5, 2.0, size=(N, K // 32)) * 2.0 ** rng.integers(-12, 4, size=(N, K // 32))).astype(np.float16).astype(np.float32)
    m = (rng.uniform(-2.0, 2.0, size=(N, K // 32)) * 2.0 ** rng.integers(-12, 4, size=(N, K // 32))).astype(np.float16).astype(np.float32)
    nib = pkg.synth.pack_nibbles(q)
    a16 = np.eye(K, dtype=np.float16)
    wh = gpu.weight(3, 1, nib, d, m)
    a_dev = torch.from_numpy(a16).cuda()
    C, Cs = torch.empty((K, N), device="cuda"), torch.empty((K, N), device="cuda")
    gpu.gemm_w41_f16act(a_dev, K, wh, C, N)
    gpu.gemm_w41_f16act_simt(a_dev, K, wh, Cs, N)
    gpu.synchronize()
    ref = oracle.gemm_w41_f16act(a16, nib, d, m)
    assert np.array_equal(C.cpu().numpy(), ref) and np.array_equal(Cs.cpu().numpy(), ref)


@pytest.mark.parametrize("M,N,K", [(1, 1000, 4096), (1, 16, 64), (5, 264, 512)])
def test_lm_head_f16(pkg, gpu, oracle, M, N, K):
    import torch
    w16 = pkg.synth.lm_head(N, K, 6)
    x = pkg.synth.activations(M, K, 6)
    wh = gpu.f16w(w16)
    C = torch.empty((M, N), device="cuda")
    gpu.f16w_matmul(wh, torch.from_numpy(x).cuda(), M, C, N)
    gpu.synchronize()
    assert rel_err(C.cpu().numpy(), oracle.lmhead_f16w(x, w16)) < 1e-3
