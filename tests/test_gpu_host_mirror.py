"""GPU: the host-side drop-in layer.
 - the reference's kernel-level functions by their own names (host/ref_names.cc ->
   libinkq_refshim.so), driven exactly like the compiled reference and compared with the
   reference's golden bytes
 - the C++ mirror of Qwen_Linear_with_bias_Int4 (host/ink_linear.h), driven by a small C++
   program the way qwen3/tests/test_linear.cc drives the original
"""
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT, f16, rel_err
from oracle.inkq_oracle import Reference
from test_gpu_matmul import GEMV_TOL

pytestmark = pytest.mark.gpu
PKG = os.path.join(ROOT, "qwen3.ink.cpp_b200")


@pytest.fixture(scope="module")
def shim(pkg, gpu):
    pkg.build()
    return Reference(os.path.join(PKG, "libinkq_refshim.so"))


@pytest.mark.parametrize("mode,key", [(0, "q8_0"), (1, "q8_1_fp16"), (2, "q8_1_fp32")])
def test_named_quantizers_write_the_reference_bytes(shim, golden, mode, key):
    g = golden("ref_quantize.npz")
    got = shim.quantize_struct(g["x"], mode, prefill=0 if mode == 0 else 0xCD).view(np.uint8)
    assert got.tobytes() == g[key].tobytes()


@pytest.mark.parametrize("variant,key", [(0, "w80"), (1, "w81_fp16"), (2, "w81_fp32")])
def test_named_retilers_write_the_reference_bytes(shim, golden, variant, key):
    g = golden("ref_repack.npz")
    got = shim.repack(g["nib"], g["d"], g["m"], variant, prefill=0 if variant == 0 else 0xCD).view(np.uint8)
    assert got.tobytes() == g[key].tobytes()


@pytest.mark.parametrize("M", [2, 6, 13])
def test_named_gemm_matches_reference_golden(shim, golden, M):
    g = golden("ref_gemm_a81w41_fp32.npz")
    N, K = g["nib"].shape[0], g["nib"].shape[1] * 2
    A = shim.quantize_struct(g[f"x_M{M}"], 2)
    B = shim.repack(g["nib"], g["d"], g["m"], 2)
    C = shim.matmul("gemm_repack_A81W41_fp32", A, B, M, N, K)
    assert np.array_equal(C.view(np.uint32), g[f"C_M{M}"].view(np.uint32))
    B2 = B.copy()                                     # a copied weight buffer (the reference deep-copies layers) still works
    C2 = shim.matmul("gemm_repack_A81W41_fp32", A, B2, M, N, K)
    assert np.array_equal(C2, C)


def test_named_gemv_and_a80w40(shim, golden):
    g = golden("ref_gemv_a81w41_fp16.npz")
    N, K = g["nib"].shape[0], g["nib"].shape[1] * 2
    A = shim.quantize_struct(g["x"], 1)
    B = shim.repack(g["nib"], g["d"], g["m"], 1)
    assert rel_err(shim.matmul("gemv_repack_A81W41_fp16", A, B, 1, N, K), g["C"]) < GEMV_TOL
    g = golden("ref_a80w40.npz")
    N, K, M = g["nib"].shape[0], g["nib"].shape[1] * 2, g["x"].shape[0]
    A = shim.quantize_struct(g["x"], 0, prefill=0)
    B = shim.repack(g["nib"], g["d"], None, 0, prefill=0)
    assert np.array_equal(shim.matmul("gemm_repack_A80W40", A, B, M, N, K).view(np.uint32), g["C_gemm"].view(np.uint32))
    assert rel_err(shim.matmul("gemv_repack_A80W40", A, B, 1, N, K), g["C_gemv"]) < GEMV_TOL


def test_cpp_linear_class_mirror(pkg, gpu, oracle, tmp_path):
    pkg.build()
    exe = tmp_path / "test_linear_mirror"
    env = {k: v for k, v in os.environ.items() if k not in ("CC", "CXX")}
    subprocess.run(["g++", "-O1", "-std=c++17", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(PKG, "host"),
                    os.path.join(ROOT, "tests", "cpp", "test_linear_mirror.cc"), "-o", str(exe), "-L", PKG, "-linkq",
                    f"-Wl,-rpath,{PKG}"], check=True, env=env)
    N, K, M = 264, 512, 37
    w = pkg.synth.weights(N, K, 21)
    d_any = (w["d"] * np.float32(1.0003)).astype(np.float32)
    x = pkg.synth.activations(M, K, 21)
    d = str(tmp_path) + "/"
    w["nib"].tofile(d + "weight_int4.bin")                 # the four files of one exported linear (QwenOperator.h:137-140)
    d_any.tofile(d + "scaling_factor_int4.bin")
    w["m"].tofile(d + "offset_int4.bin")
    np.zeros((N, K // 32), np.int8).tofile(d + "zero_point_int4.bin")
    x.tofile(d + "input.bin")
    r = subprocess.run([str(exe), d, str(N), str(K), str(M), d + "input.bin", d + "output.bin"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    out = np.fromfile(d + "output.bin", np.float32)
    y, y1 = out[: M * N].reshape(M, N), out[M * N:].reshape(1, N)
    q, dd, s = oracle.quantize(x, 2)
    assert np.array_equal(y.view(np.uint32), oracle.gemm(0, q, dd, s, w["nib"], d_any, w["m"]).view(np.uint32))
    q1, d1, s1 = oracle.quantize(x[:1], 1)
    assert rel_err(y1, oracle.gemm(0, q1, d1, s1, w["nib"], f16(d_any), f16(w["m"]))) < GEMV_TOL
