"""Generates tests/golden/ref_weightquant.npz by IMPORTING the reference's offline weight quantizers
(notebooks/quantize_methods.py: quantize_row_q40_tinyml, quantize_row_q41_tinyml) from a checkout of the reference
project.  Run it where that checkout exists:

    python tests/golden/make_golden_weightquant.py /path/to/Qwen3.Ink.Cpp

The fixture holds the fp32 input matrices and, for both formats, the packed nibbles, scales, minima and zero points the
reference returns.  Inputs: Gaussian weights, a block of zeros, a constant block, blocks with ties at .5 steps, large
and tiny magnitudes.
"""
import contextlib
import io
import os
import sys

import numpy as np
import torch


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden_weightquant.py /path/to/Qwen3.Ink.Cpp")
    ref = sys.argv[1]
    sys.path.insert(0, os.path.join(ref, "notebooks"))
    import quantize_methods as qm   # the reference's own code

    rng = np.random.default_rng(2024)
    N, K = 12, 256
    w = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    w[0, :32] = 0.0                                   # all-zero block: d == 0
    w[1, 32:64] = 0.125                               # constant block: max == min
    w[2, :32] = np.linspace(-1.0, 1.0, 32, dtype=np.float32)           # exact .5 steps after scaling
    w[3, 64:96] = (np.arange(32) - 16).astype(np.float32) * 0.5
    w[4] *= 1e4
    w[5] *= 1e-6
    w[6, :32] = -np.abs(w[6, :32])                    # all negative
    w[7, :32] = np.abs(w[7, :32])                     # all positive
    w[8, 5] = -w[8, :32].__abs__().max()              # tie for the largest magnitude with opposite sign
    out = {"w": w}
    for name, fn in (("q40", qm.quantize_row_q40_tinyml), ("q41", qm.quantize_row_q41_tinyml)):
        with contextlib.redirect_stdout(io.StringIO()):          # the reference prints error statistics
            qs, d, m, zp = fn(torch.from_numpy(w.copy()), False)
        out[name + "_nib"] = np.ascontiguousarray(qs).reshape(N, K // 2)
        out[name + "_d"] = np.asarray(d, np.float32).reshape(N, K // 32)
        out[name + "_m"] = np.asarray(m, np.float32).reshape(N, K // 32)
        out[name + "_zp"] = np.asarray(zp, np.int8).reshape(N, K // 32)
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_weightquant.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
