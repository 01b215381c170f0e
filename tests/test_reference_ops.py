"""CPU: the C entry points of oracle/ref_ops_driver.cc (the reference's own operators compiled into oracle/_ref) give
what the operators' definitions say, computed in double with NumPy - a check of the driver's argument plumbing
(layouts, strides, the causal mask), so that the GPU comparisons in test_gpu_ops_vs_reference.py rest on it."""
import numpy as np


def test_reference_operator_driver_against_numpy(reference):
    rng = np.random.default_rng(0)
    hd, L, mx, past = 128, 7, 32, 5
    x = rng.standard_normal((5, 3, hd)).astype(np.float32)
    w = (rng.random(hd) + 0.5).astype(np.float32)
    ref = x / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-6) * w
    assert np.abs(reference.rmsnorm(x, w) - ref).max() < 5e-6
    a = (rng.standard_normal((4, 64)) * 4).astype(np.float32)
    b = rng.standard_normal((4, 64)).astype(np.float32)
    assert np.abs(reference.silu_mul(a, b) - a / (1 + np.exp(-a.astype(np.float64))) * b).max() < 2e-6
    assert np.array_equal(reference.add(a, b), a + b)
    inv = 1.0 / (1e6 ** (np.arange(0, hd, 2) / hd))
    ang = np.outer(np.arange(mx), inv)
    ang = np.concatenate([ang, ang], 1)
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    q = rng.standard_normal((4, L, hd)).astype(np.float32)
    k = rng.standard_normal((2, L, hd)).astype(np.float32)

    def rope(v, st):
        rot = np.concatenate([-v[..., hd // 2:], v[..., :hd // 2]], -1)
        return v * cos[st:st + L][None] + rot * sin[st:st + L][None]

    q2, k2 = reference.rope(q, k, 3, cos, sin)
    assert np.abs(q2 - rope(q, 3)).max() < 1e-6 and np.abs(k2 - rope(k, 3)).max() < 1e-6
    kc = np.zeros((2, mx, hd), np.float32)
    vc = np.zeros((2, mx, hd), np.float32)
    kc[:, :past + L] = rng.standard_normal((2, past + L, hd))
    vc[:, :past + L] = rng.standard_normal((2, past + L, hd))
    got = reference.attention(q, kc, vc, past, 1 / np.sqrt(hd))
    want = np.zeros((L, 4 * hd))
    for h in range(4):
        kk, vv = kc[h // 2, :past + L].astype(np.float64), vc[h // 2, :past + L].astype(np.float64)
        s = q[h].astype(np.float64) @ kk.T / np.sqrt(hd)
        for i in range(L):
            s[i, past + i + 1:] = -np.inf
        p = np.exp(s - s.max(-1, keepdims=True))
        want[:, h * hd:(h + 1) * hd] = (p / p.sum(-1, keepdims=True)) @ vv
    assert np.abs(got - want).max() < 5e-6
