"""GPU: the thin device-resident glue around the quantized linears (csrc/glue_ops.cu) and the
synthetic Qwen3 forward built from it, on a small configuration.
 - the whole forward against the same graph written with plain PyTorch fp32 ops (the quantized
   linears are the library's own in both, they are checked elsewhere)
 - the decode path (one token, KV cache, captured CUDA graph) against the prefill path
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def small_cfg(pkg, **kw):
    return pkg.qwen3_forward.Qwen3Config(layers=2, hidden=256, nq=4, nkv=2, head_dim=128, ffn=512, vocab=1024, max_pos=64, lm_head_fp16=True, **kw)


def torch_forward(torch, model, tokens):
    """Same graph with PyTorch ops (fp32), K/V rounded to fp16 as the cache holds them."""
    cfg, ctx = model.cfg, model.ctx
    T = tokens.numel()
    x = model.embed[tokens.long()].float()

    def rms(v, w):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.eps) * w

    def lin(w, inp, N):
        out = torch.empty((inp.shape[0], N), device="cuda")
        ctx.linear(w, inp.contiguous(), inp.shape[0], out, N)
        return out

    def rope(v):    # v [T][heads][128]
        cos, sin = model.cos[:T, None, :], model.sin[:T, None, :]
        rot = torch.cat((-v[..., 64:], v[..., :64]), dim=-1)
        return v * cos + rot * sin

    for ly in model.layers:
        h = rms(x, ly["ln1"])
        qkv = lin(ly["qkv"], h, (cfg.nq + 2 * cfg.nkv) * 128).view(T, cfg.nq + 2 * cfg.nkv, 128)
        q = rope(rms(qkv[:, :cfg.nq], ly["qn"]))
        k = rope(rms(qkv[:, cfg.nq:cfg.nq + cfg.nkv], ly["kn"])).half().float()
        v = qkv[:, cfg.nq + cfg.nkv:].half().float()
        rep = cfg.nq // cfg.nkv
        k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
        s = torch.einsum("thd,shd->hts", q, k) / np.sqrt(128.0)
        s = s.masked_fill(torch.triu(torch.ones(T, T, device="cuda", dtype=torch.bool), 1), float("-inf"))
        a = torch.einsum("hts,shd->thd", torch.softmax(s, dim=-1), v).reshape(T, cfg.nq * 128)
        x = x + lin(ly["o"], a, cfg.hidden)
        h = rms(x, ly["ln2"])
        gu = lin(ly["gate_up"], h, 2 * cfg.ffn)
        gu = gu.view(T, cfg.ffn // 32, 2, 32)                     # (32 gate, 32 up) column groups
        act = (torch.nn.functional.silu(gu[:, :, 0, :]) * gu[:, :, 1, :]).reshape(T, cfg.ffn)
        x = x + lin(ly["down"], act, cfg.hidden)
    last = rms(x[T - 1:T], model.final_norm)
    return last


@pytest.mark.parametrize("T", [13, 45])     # per-(token, head) attention kernel / tiled prompt kernel (two key tiles)
def test_forward_matches_pytorch_graph(pkg, gpu, T):
    import torch
    model = pkg.qwen3_forward.Qwen3Synthetic(pkg, gpu, small_cfg(pkg), seed=1)
    tokens = torch.from_numpy(pkg.synth.tokens(T, 1024, 5)).cuda()
    model.reset()
    logits = model.prefill(tokens).clone()
    gpu.synchronize()
    last = torch_forward(torch, model, tokens)                       # final-normed hidden state of the last token
    ref = torch.empty((1, 1024), device="cuda")
    gpu.f16w_matmul(model.lm_head, last.contiguous(), 1, ref, 1024)
    gpu.synchronize()
    # The two graphs differ in the last bits of the glue (exp, rsqrt, summation order); an int8 rounding of a
    # quantizer input that sits on a tie then flips, which moves single outputs of the next linear by ~1e-3 of
    # their scale.  The bound is on the logits as a whole.
    scale = ref.abs().max().item()
    err = (logits - ref).abs().max().item() / scale
    assert err < 2e-2, err
    top2 = torch.topk(ref.flatten(), 2).values
    if (top2[0] - top2[1]).item() > 2 * err * scale:              # an unambiguous winner must be found by both
        assert int(model.token.item()) == int(ref.argmax().item())
    else:
        assert int(model.token.item()) in torch.topk(ref.flatten(), 8).indices.tolist()
    assert int(model.pos.item()) == T


def test_decode_path_and_graph_agree_with_prefill(pkg, gpu):
    import torch
    model = pkg.qwen3_forward.Qwen3Synthetic(pkg, gpu, small_cfg(pkg), seed=2)
    toks = torch.from_numpy(pkg.synth.tokens(9, 1024, 6)).cuda()
    # prefill all 9 tokens
    model.reset()
    full = model.prefill(toks).clone()
    # prefill 8, then feed the 9th through the decode path (M == 1 linears, cache append at position 8)
    model.reset()
    model.prefill(toks[:8])
    model.token.copy_(toks[8:9])
    step = model.decode_step().clone()
    gpu.synchronize()
    rel = (step - full).abs().max().item() / full.abs().max().item()
    assert rel < 6e-2, rel            # the single-token path quantizes with fp16 activation scales and uses the QGEMV order
    assert int(model.pos.item()) == 9
    # greedy generation: eager steps and replays of the captured graph give the same tokens
    model.reset()
    model.prefill(toks)
    for _ in range(5):
        model.decode_step()
    gpu.synchronize()
    eager = model.generated_tokens().copy()
    model.reset()
    model.prefill(toks)
    model.decode_step()
    model.capture_decode()
    for _ in range(4):
        model.graph.replay()
    torch.cuda.synchronize()
    assert np.array_equal(model.generated_tokens(), eager) and len(eager) == 6


def test_fused_decode_layer_equals_separate_kernels(pkg, gpu):
    """inkq_glue_linear_m1 (norm / SiLU*up + quantizer in the QGEMV prologue, residual in the epilogue) against the
    separate kernels.  Plain and SiLU*up prologues quantize the very same fp32 values, so the results are
    bit-identical; the RMSNorm prologue sums the squares in another order, so its input to the quantizer may
    differ in the last bit and the outputs agree to the tolerance of a flipped rounding."""
    import ctypes as C
    import torch
    L = gpu.L
    K, N = 512, 384
    w = pkg.synth.weights(N, K, 31)
    for scheme, m in ((pkg.A81W41, w["m"]), (pkg.A80W40, None)):
        wh = gpu.weight(scheme, pkg.SCALES_F16, w["nib"], w["d"], m)
        x = torch.randn((1, K), device="cuda")
        g = torch.rand(K, device="cuda") + 0.5
        ref = torch.empty((1, N), device="cuda")
        out = torch.empty((1, N), device="cuda")
        # plain
        gpu.linear(wh, x, 1, ref, N)
        gpu.check(L.inkq_glue_linear_m1(gpu.h, wh.h, C.c_void_p(x.data_ptr()), 0, None, C.c_float(0.0), C.c_void_p(out.data_ptr()), 0))
        gpu.synchronize()
        assert torch.equal(out, ref)
        # residual accumulate
        base = torch.randn((1, N), device="cuda")
        acc = base.clone()
        gpu.check(L.inkq_glue_linear_m1(gpu.h, wh.h, C.c_void_p(x.data_ptr()), 0, None, C.c_float(0.0), C.c_void_p(acc.data_ptr()), 1))
        gpu.synchronize()
        assert torch.equal(acc, base + ref)
        # RMSNorm prologue
        xn = torch.empty_like(x)
        gpu.check(L.inkq_glue_rmsnorm(gpu.h, C.c_void_p(x.data_ptr()), C.c_void_p(g.data_ptr()), 1, K, C.c_float(1e-6), C.c_void_p(xn.data_ptr())))
        gpu.linear(wh, xn, 1, ref, N)
        gpu.check(L.inkq_glue_linear_m1(gpu.h, wh.h, C.c_void_p(x.data_ptr()), 1, C.c_void_p(g.data_ptr()), C.c_float(1e-6), C.c_void_p(out.data_ptr()), 0))
        gpu.synchronize()
        assert (out - ref).abs().max().item() <= 5e-3 * ref.abs().max().item()
        # SiLU(gate) * up prologue: input [2K]
        gu = torch.randn((1, 2 * K), device="cuda")
        act = torch.empty((1, K), device="cuda")
        gpu.check(L.inkq_glue_silu_mul_rows(gpu.h, C.c_void_p(gu.data_ptr()), 1, K, C.c_void_p(act.data_ptr())))
        gpu.linear(wh, act, 1, ref, N)
        gpu.check(L.inkq_glue_linear_m1(gpu.h, wh.h, C.c_void_p(gu.data_ptr()), 2, None, C.c_float(0.0), C.c_void_p(out.data_ptr()), 0))
        gpu.synchronize()
        assert torch.equal(out, ref)


def test_fused_and_unfused_decode_agree(pkg, gpu):
    import torch
    toks = torch.from_numpy(pkg.synth.tokens(9, 1024, 6)).cuda()
    logits = []
    for mode in ("separate", "prologue", "epilogue"):
        model = pkg.qwen3_forward.Qwen3Synthetic(pkg, gpu, small_cfg(pkg, decode_mode=mode), seed=2)
        model.reset()
        model.prefill(toks[:8])
        model.token.copy_(toks[8:9])
        logits.append(model.decode_step().clone())
        gpu.synchronize()
    for other in logits[1:]:
        rel = (logits[0] - other).abs().max().item() / logits[0].abs().max().item()
        assert rel < 2e-2, rel


def test_decode_gemv_epilogues_equal_separate_kernels(pkg, gpu):
    """inkq_glue_decode_gemv / _rmsnorm_quant / _attention_quant against the separate operators: accumulate and the
    gate/up pair epilogue reproduce them bit for bit (same quantizer arithmetic on the same fp32 values); the
    RMSNorm epilogue sums the squares in another order, so its quantized row may differ by a flipped rounding."""
    import ctypes as C
    import torch
    L, h = gpu.L, gpu.h
    P = lambda t: C.c_void_p(t.data_ptr())
    K, N = 512, 384
    w = pkg.synth.weights(N, K, 33)
    wh = gpu.weight(pkg.A81W41, pkg.SCALES_F16, w["nib"], w["d"], w["m"])
    x = torch.randn((1, K), device="cuda")
    a_in = gpu.act(1, K)
    gpu.quantize(a_in, x, 1, pkg.Q8_1_F16)
    ref = torch.empty((1, N), device="cuda")
    gpu.linear(wh, x, 1, ref, N)
    # 0: store, 1: accumulate
    out = torch.zeros((1, N), device="cuda")
    gpu.check(L.inkq_glue_decode_gemv(h, wh.h, a_in.h, P(out), 0, None, C.c_float(0), None, pkg.Q8_1_F16, None))
    gpu.synchronize()
    assert torch.equal(out, ref)
    base = torch.randn((1, N), device="cuda")
    acc = base.clone()
    gpu.check(L.inkq_glue_decode_gemv(h, wh.h, a_in.h, P(acc), 1, None, C.c_float(0), None, pkg.Q8_1_F16, None))
    gpu.synchronize()
    assert torch.equal(acc, base + ref)
    # 2: accumulate, then RMSNorm + quantizer by the last CTA (twice in a row: the ticket counter must come back to zero)
    g = torch.rand(N, device="cuda") + 0.5
    a_out = gpu.act(1, N)
    xn = torch.empty((1, N), device="cuda")
    for _ in range(2):
        acc = base.clone()
        gpu.check(L.inkq_glue_decode_gemv(h, wh.h, a_in.h, P(acc), 2, P(g), C.c_float(1e-6), a_out.h, pkg.Q8_1_F16, P(xn)))
        gpu.synchronize()
        want = base + ref
        assert torch.equal(acc, want)
        xn_ref = torch.empty_like(want)
        gpu.check(L.inkq_glue_rmsnorm(h, P(want), P(g), 1, N, C.c_float(1e-6), P(xn_ref)))
        a_ref = gpu.act(1, N)
        gpu.quantize(a_ref, xn_ref, 1, pkg.Q8_1_F16)
        gpu.synchronize()
        assert (xn - xn_ref).abs().max().item() <= 1e-5 * xn_ref.abs().max().item()
        q1, d1, s1, _ = a_out.export(1)
        q2, d2, s2, _ = a_ref.export(1)
        assert np.abs(q1.astype(np.int32) - q2.astype(np.int32)).max() <= 1 and (q1 != q2).mean() < 0.01
        assert np.allclose(d1, d2, rtol=2e-3) and np.allclose(s1, s2, rtol=0, atol=2e-3 * np.abs(s2).max())
        # stand-alone rmsnorm_quant: same routine
        a_sa = gpu.act(1, N)
        gpu.check(L.inkq_glue_rmsnorm_quant(h, P(want), P(g), C.c_float(1e-6), N, a_sa.h, pkg.Q8_1_F16, None))
        gpu.synchronize()
        q3, d3, s3, _ = a_sa.export(1)
        assert np.array_equal(q1, q3) and np.array_equal(d1, d3) and np.array_equal(s1, s3)
    # 3: gate/up pairs -> SiLU * up -> quantized row of N/2
    a_pair = gpu.act(1, N // 2)
    gpu.check(L.inkq_glue_decode_gemv(h, wh.h, a_in.h, None, 3, None, C.c_float(0), a_pair.h, pkg.Q8_1_F16, None))
    act = torch.empty((1, N // 2), device="cuda")
    gpu.check(L.inkq_glue_silu_mul_rows(h, P(ref), 1, N // 2, P(act)))
    a_ref = gpu.act(1, N // 2)
    gpu.quantize(a_ref, act, 1, pkg.Q8_1_F16)
    gpu.synchronize()
    for got, want_ in zip(a_pair.export(1), a_ref.export(1)):
        assert np.array_equal(got, want_)
    # attention with quantized output against attention + quantizer
    nq, nkv, max_pos, pos = 4, 2, 64, 37
    qv = torch.randn((1, nq * 128), device="cuda")
    kc = torch.randn((nkv, max_pos, 128), device="cuda").half()
    vc = torch.randn((nkv, max_pos, 128), device="cuda").half()
    posd = torch.tensor([pos], dtype=torch.int32, device="cuda")
    o = torch.empty((1, nq * 128), device="cuda")
    gpu.check(L.inkq_glue_attention(h, P(qv), P(kc), P(vc), P(posd), 1, nq, nkv, max_pos, C.c_float(0.088), P(o)))
    a_ref = gpu.act(1, nq * 128)
    gpu.quantize(a_ref, o, 1, pkg.Q8_1_F16)
    a_att = gpu.act(1, nq * 128)
    gpu.check(L.inkq_glue_attention_quant(h, P(qv), P(kc), P(vc), P(posd), nq, nkv, max_pos, C.c_float(0.088), a_att.h, pkg.Q8_1_F16))
    gpu.synchronize()
    for got, want_ in zip(a_att.export(1), a_ref.export(1)):
        assert np.array_equal(got, want_)


def test_batched_prefill_equals_separate_prefills(pkg, gpu):
    """Several prompts as one batch through the linears (M = prompts x tokens, per-prompt KV caches): each prompt's
    last-token logits equal those of its own prefill bit for bit (rows of a QGEMM are independent)."""
    import torch
    B, T = 3, 21
    model = pkg.qwen3_forward.Qwen3Synthetic(pkg, gpu, small_cfg(pkg), seed=2, batch=B)
    prompts = torch.from_numpy(np.stack([pkg.synth.tokens(T, 1024, 30 + i) for i in range(B)])).cuda()
    model.reset()
    batched = model.prefill_batch(prompts).clone()
    gpu.synchronize()
    assert int(model.pos.item()) == T
    for i in range(B):
        model.reset()
        one = model.prefill(prompts[i].contiguous()).clone()
        gpu.synchronize()
        assert torch.equal(batched[i:i + 1], one)


@pytest.mark.parametrize("M,K", [(5, 256), (37, 4096), (3, 12288), (2, 16384)])
def test_prompt_add_rmsnorm_quantizer_in_one_kernel_equals_separate_operators(pkg, gpu, M, K):
    """inkq_glue_add_rmsnorm_quant_rows against k_add_inplace + k_rmsnorm + the stand-alone quantizer: the same
    element arithmetic in the same order, so x, the normalized rows and every quantized byte / scale / sum are equal."""
    import ctypes as C
    import torch
    L, h = gpu.L, gpu.h
    P = lambda t: C.c_void_p(t.data_ptr())
    g = torch.Generator(device="cuda")
    g.manual_seed(M * 131 + K)
    x0 = torch.randn((M, K), device="cuda", generator=g) * 3.0
    x0[0, 32:64] = 0.0                                          # a zero block
    delta = torch.randn((M, K), device="cuda", generator=g)
    w = torch.rand(K, device="cuda", generator=g) + 0.5
    for qmode in (pkg.Q8_1_F32, pkg.Q8_1_F16, pkg.Q8_0_F16):
        for with_delta in (True, False):
            # separate operators
            xs = x0.clone()
            if with_delta:
                gpu.check(L.inkq_glue_add_inplace(h, P(xs), P(delta), C.c_longlong(M * K)))
            xn = torch.empty_like(xs)
            gpu.check(L.inkq_glue_rmsnorm(h, P(xs), P(w), M, K, C.c_float(1e-6), P(xn)))
            a_ref = gpu.act(M, K)
            gpu.quantize(a_ref, xn, M, qmode)
            # one kernel
            xf = x0.clone()
            xn_f = torch.empty_like(xf)
            a_got = gpu.act(M + 3, K)
            gpu.check(L.inkq_glue_add_rmsnorm_quant_rows(h, P(xf), P(delta) if with_delta else None, P(w), C.c_float(1e-6), M, K, a_got.h, qmode,
                                                         P(xn_f)))
            gpu.synchronize()
            assert torch.equal(xf, xs) and torch.equal(xn_f, xn)
            for got, ref in zip(a_got.export(M), a_ref.export(M)):
                assert np.array_equal(got, ref)


@pytest.mark.parametrize("M,F", [(1, 64), (37, 1024), (322, 12288)])
def test_prompt_silu_mul_inside_the_quantizer_equals_separate_operators(pkg, gpu, M, F):
    import ctypes as C
    import torch
    L, h = gpu.L, gpu.h
    P = lambda t: C.c_void_p(t.data_ptr())
    g = torch.Generator(device="cuda")
    g.manual_seed(M + F)
    gu = torch.randn((M, 2 * F), device="cuda", generator=g) * 4.0
    act = torch.empty((M, F), device="cuda")
    gpu.check(L.inkq_glue_silu_mul_rows(h, P(gu), M, F, P(act)))
    for qmode in (pkg.Q8_1_F32, pkg.Q8_0_F16):
        a_ref, a_got = gpu.act(M, F), gpu.act(M, F)
        gpu.quantize(a_ref, act, M, qmode)
        gpu.check(L.inkq_glue_silu_mul_quant_rows(h, P(gu), M, F, a_got.h, qmode))
        gpu.synchronize()
        for got, ref in zip(a_got.export(M), a_ref.export(M)):
            assert np.array_equal(got, ref)


def test_fused_prompt_path_equals_separate_operators(pkg, gpu):
    """The whole prompt forward with the fused kernels (9 launches per layer) gives the logits of the one-kernel-per-operator
    path bit for bit, for one prompt and for a batch of prompts."""
    import torch
    toks = torch.from_numpy(pkg.synth.tokens(48, 1024, 8)).cuda()
    out = {}
    for mode in ("separate", "fused"):
        model = pkg.qwen3_forward.Qwen3Synthetic(pkg, gpu, small_cfg(pkg, prefill_mode=mode), seed=4, batch=3)
        model.reset()
        one = model.prefill(toks[:45]).clone()
        model.reset()
        # (prompts of at least 16 tokens: below that the stand-alone attention call takes its per-(token, head) kernel,
        # whose summation order differs from the prompt kernel's)
        many = model.prefill_batch(toks.reshape(3, 16).contiguous()).clone()
        gpu.synchronize()
        out[mode] = (one, many)
    assert torch.equal(out["fused"][0], out["separate"][0])
    assert torch.equal(out["fused"][1], out["separate"][1])


@pytest.mark.parametrize("T,prompts", [(45, 1), (14, 3), (2, 1)])
def test_prompt_attention_quantizing_its_output_equals_attention_then_quantizer(pkg, gpu, T, prompts):
    import ctypes as C
    import torch
    L, h = gpu.L, gpu.h
    P = lambda t: C.c_void_p(t.data_ptr())
    nq, nkv, max_pos, hd = 8, 2, 64, 128
    g = torch.Generator(device="cuda")
    g.manual_seed(T)
    rows = T * prompts
    q = torch.randn((rows, nq * hd), device="cuda", generator=g)
    kc = torch.randn((prompts, nkv, max_pos, hd), device="cuda", generator=g).half()
    vc = torch.randn((prompts, nkv, max_pos, hd), device="cuda", generator=g).half()
    pos = torch.tensor([3], dtype=torch.int32, device="cuda")
    scale = C.c_float(1.0 / np.sqrt(hd))
    for qmode in (pkg.Q8_1_F32, pkg.Q8_0_F16):
        out = torch.empty((rows, nq * hd), device="cuda")
        a_ref, a_got = gpu.act(rows, nq * hd), gpu.act(rows + 2, nq * hd)
        for p in range(prompts):
            r = slice(p * T, (p + 1) * T)
            gpu.check(L.inkq_glue_attention(h, P(q[r]), P(kc[p]), P(vc[p]), P(pos), T, nq, nkv, max_pos, scale, P(out[r])))
            gpu.check(L.inkq_glue_attention_quant_rows(h, P(q[r]), P(kc[p]), P(vc[p]), P(pos), T, nq, nkv, max_pos, scale, a_got.h, qmode, p * T, rows))
        gpu.quantize(a_ref, out, rows, qmode)
        gpu.synchronize()
        if T < 16:   # the stand-alone call takes the per-(token, head) kernel there: other summation order, compare the values
            qv, d, _, _ = a_got.export(rows)
            deq = (qv.reshape(rows, -1, 32).astype(np.float32) * d[:, :, None]).reshape(rows, -1)
            ref = out.cpu().numpy()
            assert np.abs(deq - ref).max() <= np.abs(ref).max() / 127 * 0.51 + 1e-5
        else:
            for got, ref in zip(a_got.export(rows), a_ref.export(rows)):
                assert np.array_equal(got, ref)


def test_decode_gemv_pending_norm_epilogue(pkg, gpu):
    """Epilogue 4 of inkq_glue_decode_gemv (each CTA quantizes its own 32 results times the norm weights, the row's RMS factor
    is left to the consumer) against epilogue 2 (RMSNorm + quantizer over the whole row by the last CTA): the residual row is
    the same bit for bit, the raw quantized row is x * g within half a quantization step, and the product that consumes it
    agrees with the one consuming the normalized row to 2e-3 of its largest value (two int8 roundings of slightly different
    fp32 values, and fp32 instead of fp16 block scales)."""
    import ctypes as C
    import torch
    L, h = gpu.L, gpu.h
    P = lambda t: C.c_void_p(t.data_ptr())
    K, N, N2 = 512, 384, 256
    for scheme, qm in ((pkg.A81W41, pkg.Q8_1_F16), (pkg.A80W40, pkg.Q8_0_F16)):
        w = pkg.synth.weights(N, K, 41)
        w2 = pkg.synth.weights(N2, N, 42)
        mm = lambda ww: ww["m"] if scheme == pkg.A81W41 else None
        wh = gpu.weight(scheme, pkg.SCALES_F16, w["nib"], w["d"], mm(w))
        wh2 = gpu.weight(scheme, pkg.SCALES_F16, w2["nib"], w2["d"], mm(w2))
        x = torch.randn((1, K), device="cuda")
        a_in = gpu.act(1, K)
        gpu.quantize(a_in, x, 1, qm)
        g = torch.rand(N, device="cuda") + 0.5
        base = torch.randn((1, N), device="cuda") * 30.0            # an un-normalized residual row
        res_a, res_b = base.clone(), base.clone()
        out_a, out_b = gpu.act(1, N), gpu.act(1, N)
        gpu.check(L.inkq_glue_decode_gemv(h, wh.h, a_in.h, P(res_a), 2, P(g), C.c_float(1e-6), out_a.h, qm, None))
        gpu.check(L.inkq_glue_decode_gemv(h, wh.h, a_in.h, P(res_b), 4, P(g), C.c_float(1e-6), out_b.h, qm, None))
        y_a, y_b = torch.empty((1, N2), device="cuda"), torch.empty((1, N2), device="cuda")
        gpu.check(L.inkq_glue_decode_gemv(h, wh2.h, out_a.h, P(y_a), 0, None, C.c_float(0), None, qm, None))
        gpu.check(L.inkq_glue_decode_gemv(h, wh2.h, out_b.h, P(y_b), 0, None, C.c_float(0), None, qm, None))
        gpu.synchronize()
        assert torch.equal(res_a, res_b)
        qv, d, _, _ = out_b.export(1)
        raw = (qv.reshape(1, -1, 32).astype(np.float32) * d[:, :, None]).reshape(1, -1)
        want = (res_b * g).cpu().numpy()
        assert (np.abs(raw - want) <= 0.51 * np.repeat(d, 32, axis=1) + 1e-6).all()
        assert (y_a - y_b).abs().max().item() <= 2e-3 * y_a.abs().max().item()
        # a pending row is not an input of the plain matmuls
        with pytest.raises(pkg.InkqError):
            gpu.gemv(out_b, wh2, y_b)


def test_decode_with_pending_norm_agrees_with_last_cta_norm(pkg, gpu):
    import torch
    toks = torch.from_numpy(pkg.synth.tokens(9, 1024, 6)).cuda()
    logits = []
    for norm in ("last_cta", "pending"):
        model = pkg.qwen3_forward.Qwen3Synthetic(pkg, gpu, small_cfg(pkg, decode_norm=norm), seed=2)
        model.reset()
        model.prefill(toks[:8])
        model.token.copy_(toks[8:9])
        logits.append(model.decode_step().clone())
        gpu.synchronize()
    rel = (logits[0] - logits[1]).abs().max().item() / logits[0].abs().max().item()
    assert rel < 2e-2, rel


@pytest.mark.parametrize("pos", [0, 2, 5, 130, 331])
def test_decode_attention_starting_from_the_qkv_row_equals_the_two_kernels(pkg, gpu, pos):
    """inkq_glue_qkv_attention_quant (q/k-norm, RoPE, cache append and attention in one kernel) against
    inkq_glue_qknorm_rope_cache followed by inkq_glue_attention_quant: the same arithmetic, so the appended cache rows and
    the quantized attention output are equal bit for bit; positions where a share is empty, holds only the new key, or
    the new key is its last of many."""
    import ctypes as C
    import torch
    L, h = gpu.L, gpu.h
    P = lambda t: C.c_void_p(t.data_ptr())
    nq, nkv, max_pos, hd = 8, 2, 512, 128
    g = torch.Generator(device="cuda")
    g.manual_seed(pos + 1)
    qkv = torch.randn((1, (nq + 2 * nkv) * hd), device="cuda", generator=g)
    qn = torch.rand(hd, device="cuda", generator=g) + 0.5
    kn = torch.rand(hd, device="cuda", generator=g) + 0.5
    ang = torch.rand((max_pos, hd), device="cuda", generator=g) * 6.28
    cos, sin = torch.cos(ang), torch.sin(ang)
    kc0 = torch.randn((nkv, max_pos, hd), device="cuda", generator=g).half()
    vc0 = torch.randn((nkv, max_pos, hd), device="cuda", generator=g).half()
    posd = torch.tensor([pos], dtype=torch.int32, device="cuda")
    eps, scale = C.c_float(1e-6), C.c_float(1.0 / np.sqrt(hd))
    # two kernels
    kc_a, vc_a = kc0.clone(), vc0.clone()
    q = torch.empty((1, nq * hd), device="cuda")
    a_ref = gpu.act(1, nq * hd)
    gpu.check(L.inkq_glue_qknorm_rope_cache(h, P(qkv), P(qn), P(kn), P(cos), P(sin), P(posd), 1, nq, nkv, max_pos, eps, P(q), P(kc_a), P(vc_a)))
    gpu.check(L.inkq_glue_attention_quant(h, P(q), P(kc_a), P(vc_a), P(posd), nq, nkv, max_pos, scale, a_ref.h, pkg.Q8_1_F16))
    # one kernel
    kc_b, vc_b = kc0.clone(), vc0.clone()
    a_got = gpu.act(1, nq * hd)
    gpu.check(L.inkq_glue_qkv_attention_quant(h, P(qkv), P(qn), P(kn), P(cos), P(sin), P(posd), nq, nkv, max_pos, eps, scale, P(kc_b), P(vc_b),
                                              a_got.h, pkg.Q8_1_F16))
    gpu.synchronize()
    assert torch.equal(kc_a, kc_b) and torch.equal(vc_a, vc_b)
    assert not torch.equal(kc_b[:, pos], kc0[:, pos])            # the row was really appended
    for got, ref in zip(a_got.export(1), a_ref.export(1)):
        assert np.array_equal(got, ref)
