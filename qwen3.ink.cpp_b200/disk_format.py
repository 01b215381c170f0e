"""The reference's on-disk format of one quantized linear layer: a directory with four raw binary files
(qwen3/include/qwen/QwenOperator.h:128-140 reads them; notebooks/save_A81W41_quantized_weight-qwen3_8b.ipynb
cells 7 and 26 write them):

    weight_int4.bin          u8  [N][K/2]   packed nibbles, byte[32g+e] = q[64g+e] | q[64g+32+e] << 4
    scaling_factor_int4.bin  f32 [N][K/32]  block scales d
    offset_int4.bin          f32 [N][K/32]  block minima m (zeros for Q4_0)
    zero_point_int4.bin      i8  [N][K/32]  8 for Q4_0, 0 for Q4_1 (the C++ code never uses it)

`path` is used as a prefix exactly as the reference does (`path + "weight_int4.bin"`), so it normally ends with '/'.
"""
from __future__ import annotations

import os

import numpy as np

FILES = (("nib", "weight_int4.bin", np.uint8), ("d", "scaling_factor_int4.bin", np.float32), ("m", "offset_int4.bin", np.float32),
         ("zp", "zero_point_int4.bin", np.int8))


def save_linear(path: str, nib, d, m, zp) -> None:
    """Writes the four files of one layer (arrays in the logical shapes above)."""
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    arrays = {"nib": nib, "d": d, "m": m, "zp": zp}
    for key, fname, dt in FILES:
        np.ascontiguousarray(arrays[key], dtype=dt).tofile(path + fname)


def load_linear(path: str, N: int, K: int) -> dict:
    """Reads one layer; raises FileNotFoundError / ValueError like the reference's loader throws on a missing or short file."""
    shapes = {"nib": (N, K // 2), "d": (N, K // 32), "m": (N, K // 32), "zp": (N, K // 32)}
    out = {}
    for key, fname, dt in FILES:
        a = np.fromfile(path + fname, dtype=dt)
        want = int(np.prod(shapes[key]))
        if a.size < want:
            raise ValueError(f"{path + fname}: {a.size} elements on disk, {want} expected for N={N}, K={K}")
        out[key] = a[:want].reshape(shapes[key])
    return out


def weight_from_disk(ctx, pkg, path: str, N: int, K: int, scheme=None, scale_mode=None, n_begin: int = 0, n_end=None):
    """What the reference's constructor does (read the four files, re-tile): a device-resident weight handle.
    The scheme defaults to A81W41, or A80W40 when the zero points on disk are 8."""
    t = load_linear(path, N, K)
    if scheme is None:
        scheme = pkg.A80W40 if (t["zp"] == 8).all() else pkg.A81W41
    if scale_mode is None:
        scale_mode = pkg.SCALES_F32
    m = t["m"] if scheme in (pkg.A81W41, pkg.W41) else None
    return ctx.weight(scheme, scale_mode, t["nib"], t["d"], m, None, n_begin, N if n_end is None else n_end)
