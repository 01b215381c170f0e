"""CPU: the oracle (oracle/inkq_oracle.c) against the committed outputs of the
reference's own kernels (tests/golden/ref_*.npz, made by tests/golden/make_golden.py)
and, where oracle/_ref is present, against the reference kernels run live."""
import numpy as np
import pytest

from conftest import f16, rel_err
from oracle.inkq_oracle import Q4_FP16, Q4_FP32, Q8_FP16, Q8_FP32


def planar_from_struct(st, mode):
    """Reference activation structs -> (q [nb][32], d [nb], s [nb]) as fp32 numbers."""
    n = st.shape[0]
    q = np.empty((n, 2, 32), np.int8)
    q[:, 0], q[:, 1] = st["q_low"], st["q_high"]
    if mode == 2:
        d = np.stack([st["s_low"], st["s_high"]], 1)
        s = np.stack([st["ss_low"], st["ss_high"]], 1)
    else:
        d = np.stack([st["s_low"], st["s_high"]], 1).view(np.float16).astype(np.float32)
        s = np.stack([st["ss_low"], st["ss_high"]], 1).view(np.float16).astype(np.float32)
    return q.reshape(-1, 32), d.reshape(-1), s.reshape(-1)


@pytest.mark.parametrize("mode,key", [(0, "q8_0"), (1, "q8_1_fp16"), (2, "q8_1_fp32")])
def test_quantizer_matches_reference_bytes(oracle, golden, mode, key):
    g = golden("ref_quantize.npz")
    prefill = 0 if mode == 0 else 0xCD   # the Q8_0 entry point leaves the sum fields unwritten
    mine = oracle.quantize_struct(g["x"], mode, prefill=prefill).view(np.uint8)
    assert mine.tobytes() == g[key].tobytes()


def test_quantizer_planar_equals_struct(oracle, golden):
    g = golden("ref_quantize.npz")
    for mode, key in ((0, "q8_0"), (1, "q8_1_fp16"), (2, "q8_1_fp32")):
        st = g[key].view(Q8_FP32 if mode == 2 else Q8_FP16)
        q_ref, d_ref, s_ref = planar_from_struct(st, mode)
        q, d, s = oracle.quantize(g["x"], mode)
        assert np.array_equal(q.reshape(-1, 32), q_ref)
        assert np.array_equal(d.reshape(-1).view(np.uint32), d_ref.view(np.uint32))
        if mode != 0:
            assert np.array_equal(s.reshape(-1).view(np.uint32), s_ref.view(np.uint32))


@pytest.mark.parametrize("variant,key", [(0, "w80"), (1, "w81_fp16"), (2, "w81_fp32")])
def test_retiler_matches_reference_bytes(oracle, golden, variant, key):
    g = golden("ref_repack.npz")
    prefill = 0 if variant == 0 else 0xCD
    mine = oracle.repack(g["nib"], g["d"], g["m"], variant, prefill=prefill).view(np.uint8)
    assert mine.tobytes() == g[key].tobytes()


@pytest.mark.parametrize("M", [2, 5, 6, 7, 13])
def test_gemm_a81w41_fp32_bit_exact(oracle, golden, M):
    g = golden("ref_gemm_a81w41_fp32.npz")
    q, d, s = oracle.quantize(g[f"x_M{M}"], 2)
    C = oracle.gemm(0, q, d, s, g["nib"], g["d"], g["m"])
    assert np.array_equal(C.view(np.uint32), g[f"C_M{M}"].view(np.uint32))


def test_gemv_a81w41_fp16_bit_exact(oracle, golden):
    g = golden("ref_gemv_a81w41_fp16.npz")
    q, d, s = oracle.quantize(g["x"], 1)
    C = oracle.gemm(0, q, d, s, g["nib"], f16(g["d"]), f16(g["m"]))
    assert np.array_equal(C.view(np.uint32), g["C"].view(np.uint32))


def test_a80w40_bit_exact(oracle, golden):
    g = golden("ref_a80w40.npz")
    q, d, _ = oracle.quantize(g["x"], 0)
    C = oracle.gemm(1, q, d, None, g["nib"], f16(g["d"]))
    assert np.array_equal(C.view(np.uint32), g["C_gemm"].view(np.uint32))
    assert np.array_equal(C[:1].view(np.uint32), g["C_gemv"].view(np.uint32))


def test_reference_throughput_recipe(oracle, golden):
    """Inputs drawn as the reference's own test does (qwen3/tests/test_linear.cc:137-158)."""
    g = golden("ref_testlinear_recipe.npz")
    q, d, s = oracle.quantize(g["x"], 2)
    C = oracle.gemm(0, q, d, s, g["nib"], g["d"], g["m"])
    assert np.array_equal(C.view(np.uint32), g["C"].view(np.uint32))


def test_block_dots_are_plain_integer_sums(oracle, pkg):
    M, N, K = 3, 16, 128
    x = pkg.synth.activations(M, K, 5)
    w = pkg.synth.weights(N, K, 5)
    q, d, s = oracle.quantize(x, 2)
    _, dots = oracle.gemm(0, q, d, s, w["nib"], w["d"], w["m"], want_dots=True)
    qw = pkg.synth.unpack_nibbles(w["nib"]).astype(np.int32)
    ref = np.einsum("mbe,nbe->mnb", q.astype(np.int32).reshape(M, K // 32, 32), qw.reshape(N, K // 32, 32))
    assert np.array_equal(dots, ref)
    _, dz = oracle.gemm(2, q, d, None, w["nib"], w["d"], None, w["zp"], want_dots=True)
    refz = np.einsum("mbe,nbe->mnb", q.astype(np.int32).reshape(M, K // 32, 32),
                     qw.reshape(N, K // 32, 32) - w["zp"].astype(np.int32)[:, :, None])
    assert np.array_equal(dz, refz)


def test_fp16_conversion_is_ieee_rne(oracle):
    rng = np.random.default_rng(0)
    vals = (rng.standard_normal(5000) * 10.0 ** rng.integers(-9, 5, 5000)).astype(np.float32)
    vals = np.concatenate([vals, np.array([0, -0.0, 65504, 65519.9, 65520, 1e-8, 5.96e-8, 2.98e-8, 6.1e-5, 6.0975e-5], np.float32)])
    mine = np.array([oracle.lib.ink_f32_to_f16(float(v)) for v in vals], np.uint16)
    with np.errstate(over="ignore"):
        assert np.array_equal(mine, vals.astype(np.float16).view(np.uint16))
    back = np.array([oracle.lib.ink_f16_to_f32(int(h)) for h in range(0, 0x7C00, 7)], np.float32)
    assert np.array_equal(back, np.arange(0, 0x7C00, 7, dtype=np.uint16).view(np.float16).astype(np.float32))


def test_w41_dequantised_weight_is_one_rounding_of_the_exact_value(oracle, pkg):
    """Weight-only W41: w16 = fp16(q*d + m) rounded once from the exact value (what a half-precision fused
    multiply-add returns).  One-hot fp16 activations read the dequantised weights back out of the matmul; NumPy's
    float64 -> float16 conversion is the independent single rounding.  Scales cover a wide exponent range so that
    double rounding through fp32 would show."""
    rng = np.random.default_rng(77)
    N, K = 64, 128
    q = rng.integers(0, 16, size=(N, K), dtype=np.uint8)
    d = (rng.uniform(0.5, 2.0, size=(N, K // 32)) * 2.0 ** rng.integers(-12, 4, size=(N, K // 32))).astype(np.float16)
    m = (rng.uniform(-2.0, 2.0, size=(N, K // 32)) * 2.0 ** rng.integers(-12, 4, size=(N, K // 32))).astype(np.float16)
    a16 = np.eye(K, dtype=np.float16)
    got = oracle.gemm_w41_f16act(a16, pkg.synth.pack_nibbles(q), d.astype(np.float32), m.astype(np.float32))      # [K][N] = w16[n][k]
    exact = q.astype(np.float64) * np.repeat(d.astype(np.float64), 32, axis=1) + np.repeat(m.astype(np.float64), 32, axis=1)
    want = exact.astype(np.float16).astype(np.float32)
    assert np.array_equal(got.T, want)


@pytest.mark.parametrize("which,name", [(0, "q40"), (1, "q41")])
def test_weight_quantizers_match_the_python_reference(oracle, golden, which, name):
    """Fixture made by importing notebooks/quantize_methods.py of the reference (tests/golden/make_golden_weightquant.py):
    packed nibbles, scales and minima of the restatement equal the reference's bit for bit, including zero, constant,
    tie and extreme-magnitude blocks."""
    g = golden("ref_weightquant.npz")
    nib, d, m = oracle.quantize_weight(which, g["w"])
    assert np.array_equal(nib, g[name + "_nib"])
    assert np.array_equal(d.view(np.uint32), g[name + "_d"].view(np.uint32))
    assert np.array_equal(m.view(np.uint32), g[name + "_m"].view(np.uint32))
    assert (g[name + "_zp"] == (8 if which == 0 else 0)).all()


def test_weight_quantizers_round_trip(oracle, pkg):
    """Q4_1 / Q4_0 format definitions (notebooks/quantize_methods.py:13-125)."""
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((8, 128)) * 0.05).astype(np.float32)
    nib, d, m = oracle.quantize_weight(1, w)
    q = pkg.synth.unpack_nibbles(nib).astype(np.float32).reshape(8, 4, 32)
    deq = q * d[:, :, None] + m[:, :, None]
    assert np.abs(deq.reshape(8, 128) - w).max() <= d.max() * 0.5 + 1e-6
    x = w.reshape(-1, 32)
    assert np.allclose(m.reshape(-1), x.min(1)) and np.allclose(d.reshape(-1), (x.max(1) - x.min(1)) / 15)
    nib0, d0, m0 = oracle.quantize_weight(0, w)
    q0 = pkg.synth.unpack_nibbles(nib0).astype(np.float32).reshape(8, 4, 32) - 8
    assert np.abs((q0 * d0[:, :, None]).reshape(8, 128) - w).max() <= np.abs(d0).max() * 1.0 + 1e-6
    assert np.all(m0 == 0)


# ---- live comparison with the reference kernels (skipped where oracle/_ref is absent) ----
@pytest.mark.parametrize("M,N,K", [(1, 16, 64), (6, 8, 128), (11, 136, 512), (33, 64, 4096)])
def test_live_reference_a81w41(oracle, reference, pkg, M, N, K):
    x = pkg.synth.activations(M, K, 100 + M)
    w = pkg.synth.weights(N, K, M)
    d_any = (w["d"] * np.float32(1.0007)).astype(np.float32)
    A = reference.quantize_struct(x, 2, pad_rows=6 * K // 64, prefill=0)
    assert oracle.quantize_struct(x, 2).tobytes() == A[: M * K // 64].tobytes()
    B = reference.repack(w["nib"], d_any, w["m"], 2)
    q, d, s = oracle.quantize(x, 2)
    assert np.array_equal(oracle.gemm(0, q, d, s, w["nib"], d_any, w["m"]).view(np.uint32),
                          reference.matmul("gemm_repack_A81W41_fp32", A, B, M, N, K).view(np.uint32))
    A1 = reference.quantize_struct(x[:1], 1)
    B1 = reference.repack(w["nib"], d_any, w["m"], 1)
    q1, d1, s1 = oracle.quantize(x[:1], 1)
    assert np.array_equal(oracle.gemm(0, q1, d1, s1, w["nib"], f16(d_any), f16(w["m"])).view(np.uint32),
                          reference.matmul("gemv_repack_A81W41_fp16", A1, B1, 1, N, K).view(np.uint32))


# ------------------------------------------------------------------ schemes that exist only in the reference's notebooks
def rms_err(got, ref):
    ref = np.asarray(ref, np.float64)
    return float(np.abs(np.asarray(got, np.float64) - ref).max() / np.sqrt(np.mean(ref * ref)))


def test_a80w4z_matches_the_notebook(oracle, golden):
    """Fixture: outputs of the reference's own notebook cell (QuantizedLinear + pseudo_quantize_tensor_q4_zero_point,
    evaluate-qwen3_8b_A8W4.ipynb) run by tests/golden/make_golden_notebook.py.  With the notebook's own activation
    codes and fp32 scales the oracle's integer form sum_b d_a*d_w*(I - zp*sum(q_a)) equals the notebook's
    dequantise-then-linear to summation-order accuracy: this pins the scheme's math.  Through the real path (the
    reference's Q8_0 quantizer stores the activation scale as fp16, the packed weights carry fp16 scales; the notebook
    keeps both in fp32) the two fp16 roundings of the scales show: a few 1e-3 of the output's rms."""
    g = golden("ref_notebook_schemes.npz")
    y = oracle.gemm(2, g["w4z_xq"], g["w4z_xd"], None, g["w4z_nib"], g["w4z_d"], None, g["w4z_zp"])
    assert rel_err(y, g["w4z_y"]) < 1e-3
    q, d, _ = oracle.quantize(g["w4z_x"], 0)
    assert np.array_equal(q, g["w4z_xq"])                     # same integer codes as the notebook's fake quantizer
    y16 = oracle.gemm(2, q, d, None, g["w4z_nib"], f16(g["w4z_d"]), None, g["w4z_zp"])
    assert rms_err(y16, g["w4z_y"]) < 3e-3


def test_w41_matches_the_notebook(oracle, golden):
    """Fixture: the reference's weight-only notebook (evaluate-qwen3_8b_W4.ipynb: fp16 model, weights overwritten with
    pseudo_quantize_tensor_q41's output, stock fp16 F.linear).  The notebook rounds q*s to fp16 and then adds the
    minimum (two roundings); this library rounds q*d + m once: the dequantised weights differ by at most one fp16 ulp
    of the intermediate product q*s (half of them are identical).
    Its output is fp16 (this library's is fp32): agreement to the fp16 rounding of the output, a few 1e-3 of its rms."""
    g = golden("ref_notebook_schemes.npz")
    K = g["w41_x"].shape[1]
    ours = oracle.gemm_w41_f16act(np.eye(K, dtype=np.float16), g["w41_nib"], g["w41_d"], g["w41_m"]).T    # one-hot rows read the weights back
    theirs = g["w41_wf"].astype(np.float32)
    nib = g["w41_nib"].reshape(g["w41_nib"].shape[0], -1, 32)
    q = np.stack([nib & 15, nib >> 4], axis=2).reshape(theirs.shape).astype(np.float32)      # undo the AWQ interleave
    prod = q * np.repeat(g["w41_d"], 32, axis=1)
    ulp = np.spacing(np.maximum(np.abs(prod), np.abs(theirs)).astype(np.float16)).astype(np.float32)
    assert np.all(np.abs(ours - theirs) <= ulp)
    assert np.mean(ours == theirs) > 0.5
    y = oracle.gemm_w41_f16act(g["w41_x"], g["w41_nib"], g["w41_d"], g["w41_m"])
    assert rms_err(y, g["w41_y"].astype(np.float32)) < 4e-3
