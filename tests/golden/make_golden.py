"""Generate tests/golden/ref_*.npz by running the REFERENCE's own compiled kernels.

Run once where the reference checkout is mounted (after `make -C oracle ref`):

    python tests/golden/make_golden.py

Each fixture stores the seeded inputs together with the bytes the reference's
functions produced for them, so the oracle and the CUDA path can be pinned to the
reference on machines where the reference is not available.  Functions exercised
(paths relative to the reference root): the three quantizers and four matmuls of
qwen3/src/qwen/quantized_gemx_kernels.cc and the three re-tilers of
qwen3/src/qwen/QwenOperator.cc:757-892.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from __graft_entry__ import load_package  # noqa: E402
from oracle.inkq_oracle import Reference  # noqa: E402

synth = load_package().synth
OUT = os.path.dirname(os.path.abspath(__file__))


def f16(a):
    return a.astype(np.float16).astype(np.float32)


def edge_activations(M, K, seed):
    """N(0,1) rows plus the edge cases the quantizer must get right: an all-zero
    pair, an all-zero single block, +max/-max ties, exact .5 rounding ties, tiny
    and huge magnitudes."""
    x = synth.activations(M, K, seed)
    x[1, 0:64] = 0.0
    x[2, 32:64] = 0.0
    x[3, 64:96] = np.linspace(-127, 127, 32, dtype=np.float32)       # id == 1 exactly
    x[3, 96:128] = np.linspace(-63.5, 63.5, 32, dtype=np.float32)    # .5 ties after scaling by 2
    x[3, 127] = 63.5
    x[4, 0:32] = np.float32(1e-30) * np.arange(32, dtype=np.float32)
    x[4, 32:64] = np.float32(3e30) * np.cos(np.arange(32, dtype=np.float32))
    x[5, 128:160] = -7.25
    x[5, 160:192] = 7.25
    return x


def main():
    r = Reference()
    print("reference ISA variant:", r.isa)

    # ---- quantizers --------------------------------------------------------
    x = edge_activations(7, 512, 11)
    np.savez_compressed(os.path.join(OUT, "ref_quantize.npz"), x=x,
                        q8_0=r.quantize_struct(x, 0, prefill=0).view(np.uint8),
                        q8_1_fp16=r.quantize_struct(x, 1).view(np.uint8),
                        q8_1_fp32=r.quantize_struct(x, 2).view(np.uint8))

    # ---- re-tilers -----------------------------------------------------------
    w = synth.weights(16, 256, seed_offset=1)
    d_any = (w["d"] * np.float32(1.000123)).astype(np.float32)   # not fp16-representable
    m_any = (w["m"] * np.float32(0.999877)).astype(np.float32)
    np.savez_compressed(os.path.join(OUT, "ref_repack.npz"), nib=w["nib"], d=d_any, m=m_any,
                        w80=r.repack(w["nib"], d_any, None, 0, prefill=0).view(np.uint8),
                        w81_fp16=r.repack(w["nib"], d_any, m_any, 1).view(np.uint8),
                        w81_fp32=r.repack(w["nib"], d_any, m_any, 2).view(np.uint8))

    # ---- A81W41 GEMM (fp32 scales) at ragged M ------------------------------
    K, N = 256, 24
    w = synth.weights(N, K, seed_offset=2)
    d_any = (w["d"] * np.float32(1.000123)).astype(np.float32)
    m_any = (w["m"] * np.float32(0.999877)).astype(np.float32)
    B = r.repack(w["nib"], d_any, m_any, 2)
    out = {"nib": w["nib"], "d": d_any, "m": m_any}
    for M in (2, 5, 6, 7, 13):
        xa = edge_activations(max(M, 6), K, 20 + M)[:M] if M >= 6 else synth.activations(M, K, 20 + M)
        A = r.quantize_struct(xa, 2, pad_rows=6 * K // 64, prefill=0)
        out[f"x_M{M}"] = xa
        out[f"C_M{M}"] = r.matmul("gemm_repack_A81W41_fp32", A, B, M, N, K)
    np.savez_compressed(os.path.join(OUT, "ref_gemm_a81w41_fp32.npz"), **out)

    # ---- A81W41 GEMV (fp16 scales) --------------------------------------------
    K, N = 4096, 40
    w = synth.weights(N, K, seed_offset=3)
    x1 = synth.activations(1, K, 31)
    A = r.quantize_struct(x1, 1)
    B = r.repack(w["nib"], w["d"], w["m"], 1)
    np.savez_compressed(os.path.join(OUT, "ref_gemv_a81w41_fp16.npz"), nib=w["nib"], d=w["d"], m=w["m"], x=x1,
                        C=r.matmul("gemv_repack_A81W41_fp16", A, B, 1, N, K))

    # ---- A80W40 GEMM + GEMV (N/8 and M must be even for the reference GEMM) --
    K, N, M = 256, 32, 6
    w = synth.weights(N, K, seed_offset=4)
    xa = edge_activations(M, K, 41)
    A = r.quantize_struct(xa, 0, pad_rows=2 * K // 64, prefill=0)
    B = r.repack(w["nib"], w["d"], None, 0, prefill=0)
    np.savez_compressed(os.path.join(OUT, "ref_a80w40.npz"), nib=w["nib"], d=w["d"], x=xa,
                        C_gemm=r.matmul("gemm_repack_A80W40", A, B, M, N, K),
                        C_gemv=r.matmul("gemv_repack_A80W40", A, B, 1, N, K))

    # ---- the reference throughput test's own synthetic recipe, scaled down ---
    # qwen3/tests/test_linear.cc:137-158: scale == 1, min == 2, nibble bytes rand()%256,
    # activations uniform in [0,1).
    K, N, M = 512, 16, 8
    rng = np.random.default_rng(51)
    nib = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
    d1 = np.ones((N, K // 32), np.float32)
    m2 = np.full((N, K // 32), 2.0, np.float32)
    xa = rng.random((M, K), dtype=np.float32)
    A = r.quantize_struct(xa, 2, pad_rows=6 * K // 64, prefill=0)
    B = r.repack(nib, d1, m2, 2)
    np.savez_compressed(os.path.join(OUT, "ref_testlinear_recipe.npz"), nib=nib, d=d1, m=m2, x=xa,
                        C=r.matmul("gemm_repack_A81W41_fp32", A, B, M, N, K))
    for f in sorted(os.listdir(OUT)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(OUT, f)), "bytes")


if __name__ == "__main__":
    main()
