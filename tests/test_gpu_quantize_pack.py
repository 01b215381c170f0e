"""GPU: the CUDA quantizer and the load-time re-tiler, through the C ABI, against the
oracle and the reference's golden outputs.  Integer blocks, scales and sums: bit-exact."""
import numpy as np
import pytest

from oracle.inkq_oracle import Q8_FP16, Q8_FP32
from test_oracle_golden import planar_from_struct

pytestmark = pytest.mark.gpu


def run_quantizer(pkg, gpu, x, mode):
    import torch
    M, K = x.shape
    act = gpu.act(M, K)
    xd = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    gpu.quantize(act, xd, M, mode)
    gpu.synchronize()
    return act.export(M)


@pytest.mark.parametrize("mode,key", [(0, "q8_0"), (1, "q8_1_fp16"), (2, "q8_1_fp32")])
def test_quantizer_matches_reference_golden(pkg, gpu, golden, mode, key):
    g = golden("ref_quantize.npz")
    q, d, s, isum = run_quantizer(pkg, gpu, g["x"], mode)
    q_ref, d_ref, s_ref = planar_from_struct(g[key].view(Q8_FP32 if mode == 2 else Q8_FP16), mode)
    assert np.array_equal(q.reshape(-1, 32), q_ref)
    assert np.array_equal(d.reshape(-1).view(np.uint32), d_ref.view(np.uint32))
    if mode != 0:
        assert np.array_equal(s.reshape(-1).view(np.uint32), s_ref.view(np.uint32))
    assert np.array_equal(isum.reshape(-1), q_ref.astype(np.int32).sum(1))


@pytest.mark.parametrize("M,K", [(1, 64), (1, 4096), (3, 192), (7, 512), (322, 4096), (5, 12288)])
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_quantizer_matches_oracle(pkg, gpu, oracle, M, K, mode):
    x = pkg.synth.activations(M, K, 7 + M)
    x[0, :32] = 0.0
    if M > 2:
        x[2] *= 1e-20
    q, d, s, isum = run_quantizer(pkg, gpu, x, mode)
    qo, do, so = oracle.quantize(x, mode)
    assert np.array_equal(q, qo)
    assert np.array_equal(d.view(np.uint32), do.view(np.uint32))
    assert np.array_equal(s.view(np.uint32), so.view(np.uint32))


def test_quantizer_rejects_bad_arguments(pkg, gpu):
    import torch
    act = gpu.act(4, 128)
    xd = torch.zeros((8, 128), device="cuda")
    with pytest.raises(pkg.InkqError) as e:
        gpu.quantize(act, xd, 8, 2)          # more rows than the handle holds
    assert e.value.code == pkg.ERR_INVALID
    with pytest.raises(pkg.InkqError):
        gpu.quantize(act, xd, 2, 9)          # unknown mode
    with pytest.raises(pkg.InkqError):
        gpu.act(4, 96)                        # K not a multiple of 64


@pytest.mark.parametrize("N,K", [(8, 64), (136, 512), (256, 4096), (1000, 192)])
@pytest.mark.parametrize("scheme,scale_mode", [(0, 0), (0, 1), (1, 1), (2, 1)])
def test_retile_round_trip(pkg, gpu, N, K, scheme, scale_mode):
    """disk layout -> sm_100a tile layout -> disk layout returns the same nibbles, scales, zero points."""
    w = pkg.synth.weights(N, K, 3)
    d_any = (w["d"] * np.float32(1.0003)).astype(np.float32)
    wh = gpu.weight(scheme, scale_mode, w["nib"], d_any, w["m"], w["zp"])
    nib, d, m, zp = wh.export()
    assert np.array_equal(nib, w["nib"])
    f16 = lambda a: a.astype(np.float16).astype(np.float32)
    assert np.array_equal(d, d_any if scale_mode == 0 else f16(d_any))
    if scheme == 0:
        assert np.array_equal(m, w["m"] if scale_mode == 0 else f16(w["m"]))
    expect_zp = {0: np.zeros_like(w["zp"]), 1: np.full_like(w["zp"], 8), 2: w["zp"]}[scheme]
    assert np.array_equal(zp, expect_zp)


def test_retile_shard_equals_slice(pkg, gpu):
    """A tensor-parallel column shard [n_begin, n_end) holds exactly those rows."""
    N, K = 512, 256
    w = pkg.synth.weights(N, K, 9)
    wh = gpu.weight(0, 0, w["nib"], w["d"], w["m"], None, 128 + 8, 400)
    nib, d, m, _ = wh.export()
    assert wh.rows == 400 - 136
    assert np.array_equal(nib, w["nib"][136:400]) and np.array_equal(d, w["d"][136:400]) and np.array_equal(m, w["m"][136:400])


def test_weight_create_rejects_bad_shapes(pkg, gpu):
    w = pkg.synth.weights(16, 128, 1)
    with pytest.raises(pkg.InkqError):
        gpu.weight(0, 0, w["nib"][:12], w["d"][:12], w["m"][:12])      # N % 8 != 0
    with pytest.raises(pkg.InkqError):
        gpu.weight(0, 0, w["nib"], w["d"], None)                        # Q4_1 needs mins
    with pytest.raises(pkg.InkqError):
        gpu.weight(2, 1, w["nib"], w["d"], None, None)                  # w4z needs zero points
    with pytest.raises(pkg.InkqError):
        gpu.weight(0, 0, w["nib"], w["d"], w["m"], None, 8, 8)          # empty shard
