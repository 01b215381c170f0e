"""GPU: the REFERENCE's own linear-layer class running on this library.

oracle/_ref/ref_linear_on_gpu is the reference's `Qwen_Linear_with_bias_Int4` and `ModelContext`
(qwen3/include/qwen/QwenOperator.h:34-231, qwen3/src/qwen/QwenOperator.cc:80-124, compiled unmodified by
`make -C oracle dropin`) linked WITHOUT the reference's kernel file against libinkq_refshim.so, i.e. with
quantize_row_q8_1_repack_*, gemm_repack_A81W41_fp32 and gemv_repack_A81W41_fp16 served by the GPU.
oracle/_ref/ref_linear_cpu is the same program with the reference's CPU kernels.  Both construct the class from the
four .bin files of a layer directory and call forward(); the outputs must agree: bit for bit for a prompt (M > 1,
QGEMM), within the QGEMV tolerance for one token.
"""
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT, rel_err
from test_gpu_matmul import GEMV_TOL

REF_DIR = os.path.join(ROOT, "oracle", "_ref")


def write_layer(pkg, d, N, K, seed):
    w = pkg.synth.weights(N, K, seed)
    w["nib"].tofile(os.path.join(d, "weight_int4.bin"))
    w["d"].astype(np.float32).tofile(os.path.join(d, "scaling_factor_int4.bin"))
    w["m"].astype(np.float32).tofile(os.path.join(d, "offset_int4.bin"))
    np.zeros((N, K // 32), np.int8).tofile(os.path.join(d, "zero_point_int4.bin"))   # loaded by the class, used by no kernel
    return w


def run(binary, d, N, K, M, x, tag):
    xp, op = os.path.join(d, f"x_{tag}.bin"), os.path.join(d, f"out_{tag}.bin")
    x.astype(np.float32).tofile(xp)
    res = subprocess.run([os.path.join(REF_DIR, binary), d + os.sep, str(N), str(K), str(M), xp, op], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, f"{binary} failed: {res.stderr[-500:]}"
    return np.fromfile(op, np.float32).reshape(M, N)


def have(binary):
    return os.path.exists(os.path.join(REF_DIR, binary))


def test_reference_class_on_cpu_equals_the_oracle(pkg, oracle, tmp_path):
    """The harness itself: the reference's class with the reference's kernels against the oracle (no GPU involved)."""
    if not have("ref_linear_cpu"):
        pytest.skip("oracle/_ref/ref_linear_cpu not built (make -C oracle dropin, where the reference checkout is present)")
    N, K, M = 64, 256, 7
    d = str(tmp_path)
    w = write_layer(pkg, d, N, K, 5)
    x = pkg.synth.activations(M, K, 5)
    got = run("ref_linear_cpu", d, N, K, M, x, "cpu")
    q, dd, s = oracle.quantize(x, 2)
    ref = oracle.gemm(0, q, dd, s, w["nib"], w["d"], w["m"])
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))


@pytest.mark.gpu
@pytest.mark.parametrize("N,K,M", [(256, 512, 37), (256, 512, 1), (4096, 4096, 322)])
def test_reference_class_runs_on_the_gpu_library(pkg, gpu, tmp_path, N, K, M):
    assert have("ref_linear_on_gpu") and have("ref_linear_cpu"), "oracle/_ref/ref_linear_* missing: run make -C oracle dropin where the reference is present"
    d = str(tmp_path)
    write_layer(pkg, d, N, K, 6)
    x = pkg.synth.activations(M, K, 6)
    on_gpu = run("ref_linear_on_gpu", d, N, K, M, x, "gpu")
    on_cpu = run("ref_linear_cpu", d, N, K, M, x, "cpu")
    if M > 1:
        assert np.array_equal(on_gpu.view(np.uint32), on_cpu.view(np.uint32)), f"max abs diff {np.abs(on_gpu - on_cpu).max()}"
    else:
        assert rel_err(on_gpu, on_cpu) < GEMV_TOL
