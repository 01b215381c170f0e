"""Seeded synthetic inputs for the A8W4 path.

They stand in for the reference's exported Qwen3-8B weights and its chat prompt:
same shapes, same formats, value distributions as the benchmark configs state.
All arrays are host NumPy arrays in the reference's *on-disk* (logical) formats,
which is what the reference's linear layer reads from its four .bin files
(qwen3/include/qwen/QwenOperator.h:128-140):

  nib  u8  [N][K/2]   AWQ-interleaved nibbles: byte[32g+e] = q[64g+e] | q[64g+32+e] << 4
                      (notebooks/quantize_methods.py:61-64,120-123)
  d    f32 [N][K/32]  per-block scale (values are fp16-representable)
  m    f32 [N][K/32]  per-block min   (values are fp16-representable)
  zp   u8  [N][K/32]  per-block zero point (A80W4z only)
"""
from __future__ import annotations

import numpy as np

SEED_ACT, SEED_NIB, SEED_D, SEED_M, SEED_ZP, SEED_LMHEAD, SEED_TOK = 1001, 1002, 1003, 1004, 1005, 1006, 1007
QK = 32


def activations(M: int, K: int, seed: int = SEED_ACT) -> np.ndarray:
    """fp32 [M][K] ~ N(0, 1)."""
    return np.random.default_rng(seed).standard_normal((M, K), dtype=np.float32)


def pack_nibbles(q: np.ndarray) -> np.ndarray:
    """Logical nibbles u8 [N][K] (values 0..15) -> on-disk interleaved bytes u8 [N][K/2]."""
    N, K = q.shape
    assert K % 64 == 0
    g = q.reshape(N, K // 64, 2, 32)
    return (g[:, :, 0, :] | (g[:, :, 1, :] << 4)).astype(np.uint8).reshape(N, K // 2)


def unpack_nibbles(nib: np.ndarray) -> np.ndarray:
    """Inverse of pack_nibbles."""
    N, K2 = nib.shape
    g = nib.reshape(N, K2 // 32, 32)
    out = np.empty((N, K2 // 32, 2, 32), dtype=np.uint8)
    out[:, :, 0, :] = g & 0x0F
    out[:, :, 1, :] = g >> 4
    return out.reshape(N, K2 * 2)


def weights(N: int, K: int, seed_offset: int = 0) -> dict:
    """Random 4-bit weight blocks: nibbles uniform in [0,15], d ~ U(0.002,0.02) and
    m ~ U(-0.1,0) rounded to fp16, zp uniform in [0,15].  The same nibbles serve all
    schemes (A80W40 reads them as q-8, A80W4z as q-zp, A81W41/W41 as q*d+m)."""
    nbk = K // QK
    q = np.random.default_rng(SEED_NIB + 100 * seed_offset).integers(0, 16, size=(N, K), dtype=np.uint8)
    d = np.random.default_rng(SEED_D + 100 * seed_offset).uniform(0.002, 0.02, size=(N, nbk))
    m = np.random.default_rng(SEED_M + 100 * seed_offset).uniform(-0.1, 0.0, size=(N, nbk))
    zp = np.random.default_rng(SEED_ZP + 100 * seed_offset).integers(0, 16, size=(N, nbk), dtype=np.uint8)
    return {
        "nib": pack_nibbles(q),
        "d": d.astype(np.float16).astype(np.float32),
        "m": m.astype(np.float16).astype(np.float32),
        "zp": zp,
    }


def lm_head(N: int, K: int, seed: int = SEED_LMHEAD) -> np.ndarray:
    """fp16 [N][K] ~ N(0, 0.02)."""
    rng = np.random.default_rng(seed)
    out = np.empty((N, K), dtype=np.float16)
    step = 8192
    for r in range(0, N, step):
        out[r:r + step] = (rng.standard_normal((min(step, N - r), K), dtype=np.float32) * 0.02).astype(np.float16)
    return out


def tokens(n: int, vocab: int = 151936, seed: int = SEED_TOK) -> np.ndarray:
    return np.random.default_rng(seed).integers(0, vocab, size=(n,), dtype=np.int32)
