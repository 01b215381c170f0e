"""GPU: the glue kernels around the quantized linears (csrc/glue_ops.cu) against the REFERENCE's own operators,
operator by operator.  The reference side is its unmodified code compiled into oracle/_ref (oracle/Makefile) and
driven through oracle/ref_ops_driver.cc: Qwen3RMSNorm::forward (qwen3/src/qwen/QwenOperator.cc:24-53), Qwen3SiLuMul
(:697-712), add (:714-721), RotaryPosEmb::apply (qwen3/src/ops/RotaryPosEmb.cc:6-79) and the attention core of
Qwen3Attention::forward (qwen3/src/qwen/QwenAttention.cc:122-190: bgemxGQA qk, causal mask, softmax, bgemxGQA pv).

Tolerances (fp32 against fp32; the two sides differ in summation order, in exp / rsqrt implementation, and the GPU
keeps K and V in fp16): stated per test, as a fraction of the largest reference magnitude unless said otherwise."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

HD = 128


def P(t):
    return C.c_void_p(t.data_ptr())


def rope_tables(max_pos, theta=1e6):
    inv = 1.0 / (theta ** (np.arange(0, HD, 2, dtype=np.float64) / HD))
    ang = np.outer(np.arange(max_pos, dtype=np.float64), inv)
    ang = np.concatenate([ang, ang], axis=1)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


@pytest.mark.parametrize("rows,dim", [(1, 4096), (37, 4096), (5, 128)])
def test_rmsnorm(pkg, gpu, reference, rows, dim):
    import torch
    rng = np.random.default_rng(rows + dim)
    x = (rng.standard_normal((rows, dim)) * 2.5).astype(np.float32)
    w = (rng.random(dim) + 0.5).astype(np.float32)
    ref = reference.rmsnorm(x, w, 1e-6)
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    y = torch.empty_like(xd)
    gpu.check(gpu.L.inkq_glue_rmsnorm(gpu.h, P(xd), P(wd), rows, dim, C.c_float(1e-6), P(y)))
    gpu.synchronize()
    # the reference sums the squares sequentially in fp32, the kernel as a tree: 4e-6 of the row's magnitude
    assert np.abs(y.cpu().numpy() - ref).max() <= 4e-6 * np.abs(ref).max()


def test_silu_mul_and_residual_add(pkg, gpu, reference):
    import torch
    rng = np.random.default_rng(3)
    T, F = 19, 1024
    gate = (rng.standard_normal((T, F)) * 4).astype(np.float32)
    up = rng.standard_normal((T, F)).astype(np.float32)
    ref = reference.silu_mul(gate, up)
    g, u = torch.from_numpy(gate).cuda(), torch.from_numpy(up).cuda()
    out = torch.empty_like(g)
    gpu.check(gpu.L.inkq_glue_silu_mul(gpu.h, P(g), P(u), C.c_longlong(T * F), P(out)))
    # the same on a fused gate_up output in (32 gate, 32 up) column groups
    gu = torch.stack((g.view(T, F // 32, 32), u.view(T, F // 32, 32)), dim=2).reshape(T, 2 * F).contiguous()
    out2 = torch.empty_like(g)
    gpu.check(gpu.L.inkq_glue_silu_mul_rows(gpu.h, P(gu), T, F, P(out2)))
    gpu.synchronize()
    # the reference evaluates exp in double, the kernel with the fast fp32 exponential: 2e-6 relative per element
    for got in (out, out2):
        err = np.abs(got.cpu().numpy() - ref)
        assert (err <= 2e-6 * np.abs(ref) + 1e-9).all(), err.max()
    a = torch.from_numpy(gate).cuda()
    gpu.check(gpu.L.inkq_glue_add_inplace(gpu.h, P(a), P(u), C.c_longlong(T * F)))
    gpu.synchronize()
    assert np.array_equal(a.cpu().numpy(), reference.add(gate, up))


@pytest.mark.parametrize("T,past", [(45, 0), (70, 50), (200, 141), (9, 20), (1, 329), (1, 0), (1, 2), (1, 130)])
def test_qk_norm_rope_cache_and_attention(pkg, gpu, reference, T, past):
    """Per-head q/k RMSNorm + RoPE + KV-cache append (QwenAttention.cc:78-121) and causal GQA attention
    (:122-190), the reference's operators chained as its forward chains them."""
    import torch
    rng = np.random.default_rng(T * 7 + past)
    nq, nkv, max_pos = 8, 2, 512
    cos, sin = rope_tables(max_pos)
    qn = (rng.random(HD) + 0.5).astype(np.float32)
    kn = (rng.random(HD) + 0.5).astype(np.float32)
    total = past + T
    # cache content of the past positions: fp16-representable values, so both sides hold the same numbers
    k_past = rng.standard_normal((nkv, past, HD)).astype(np.float16)
    v_past = rng.standard_normal((nkv, past, HD)).astype(np.float16)
    qkv = rng.standard_normal((T, (nq + 2 * nkv) * HD)).astype(np.float32)

    # ---- reference chain
    q3 = qkv[:, :nq * HD].reshape(T, nq, HD)
    k3 = qkv[:, nq * HD:(nq + nkv) * HD].reshape(T, nkv, HD)
    v3 = qkv[:, (nq + nkv) * HD:].reshape(T, nkv, HD)
    qr = reference.rmsnorm(q3, qn, 1e-6).transpose(1, 0, 2)          # permute01: [heads][T][hd]
    kr = reference.rmsnorm(k3, kn, 1e-6).transpose(1, 0, 2)
    qr, kr = reference.rope(qr, kr, past, cos, sin)
    kc = np.zeros((nkv, max_pos, HD), np.float32)
    vc = np.zeros((nkv, max_pos, HD), np.float32)
    kc[:, :past], vc[:, :past] = k_past, v_past
    kc[:, past:total], vc[:, past:total] = kr, v3.transpose(1, 0, 2)

    # ---- GPU
    kcd = torch.zeros((nkv, max_pos, HD), dtype=torch.float16, device="cuda")
    vcd = torch.zeros((nkv, max_pos, HD), dtype=torch.float16, device="cuda")
    kcd[:, :past], vcd[:, :past] = torch.from_numpy(k_past).cuda(), torch.from_numpy(v_past).cuda()
    qkvd = torch.from_numpy(qkv).cuda()
    qd = torch.empty((T, nq * HD), device="cuda")
    pos = torch.tensor([past], dtype=torch.int32, device="cuda")
    cosd, sind = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
    qnd, knd = torch.from_numpy(qn).cuda(), torch.from_numpy(kn).cuda()
    gpu.check(gpu.L.inkq_glue_qknorm_rope_cache(gpu.h, P(qkvd), P(qnd), P(knd), P(cosd), P(sind), P(pos), T, nq, nkv, max_pos, C.c_float(1e-6),
                                                P(qd), P(kcd), P(vcd)))
    gpu.synchronize()
    q_got = qd.cpu().numpy().reshape(T, nq, HD).transpose(1, 0, 2)
    assert np.abs(q_got - qr).max() <= 4e-6 * np.abs(qr).max()
    k_got = kcd[:, past:total].float().cpu().numpy()
    # the cache is fp16: the reference's fp32 key rounded to fp16, give or take one fp16 ulp where the two fp32 values straddle a tie
    assert (np.abs(k_got - kr) <= np.abs(kr) * 2.0 ** -10 + 1e-7).all()
    assert np.array_equal(vcd[:, past:total].cpu().numpy(), v3.transpose(1, 0, 2).astype(np.float16))

    # attention on identical inputs: the reference reads the GPU's cache content (fp16 values as fp32) and the GPU's q
    kc[:, past:total], vc[:, past:total] = k_got, vcd[:, past:total].float().cpu().numpy()
    ref = reference.attention(np.ascontiguousarray(q_got), kc, vc, past, 1.0 / np.sqrt(HD))
    out = torch.empty((T, nq * HD), device="cuda")
    gpu.check(gpu.L.inkq_glue_attention(gpu.h, P(qd), P(kcd), P(vcd), P(pos), T, nq, nkv, max_pos, C.c_float(1.0 / np.sqrt(HD)), P(out)))
    gpu.synchronize()
    # fast exponential and another summation order: 1e-5 of the largest output
    assert np.abs(out.cpu().numpy() - ref).max() <= 1e-5 * np.abs(ref).max()
    if T == 1:   # the decode step's variant that also quantizes the head outputs
        a = gpu.act(1, nq * HD)
        gpu.check(gpu.L.inkq_glue_attention_quant(gpu.h, P(qd), P(kcd), P(vcd), P(pos), nq, nkv, max_pos, C.c_float(1.0 / np.sqrt(HD)), a.h,
                                                  pkg.Q8_1_F16))
        gpu.synchronize()
        qv, d, _, _ = a.export(1)
        deq = qv.reshape(1, -1, 32).astype(np.float32) * d[:, :, None]
        assert np.abs(deq.reshape(1, -1) - ref).max() <= np.abs(ref).max() / 127 * 0.51 + 1e-5 * np.abs(ref).max()
