"""Synthetic Qwen3 decoder forward on one GPU: the caller of the quantized linear layers.

It exists to *report* prompt-prefill and decode throughput of the A8W4 path inside the model
it was written for (Qwen3-8B: 36 layers, hidden 4096, 32 query / 8 KV heads of 128, SwiGLU
12288, vocabulary 151936, RoPE theta 1e6, per-head q/k RMSNorm), with random-init weights
generated directly on the device.  Structure follows the reference's model code
(qwen3/src/qwen/QwenForCausalLM.cc:11-122, QwenDecoder.cc:53-142, QwenDecoderLayer.cc:39-119,
QwenAttention.cc:52-207): fused qkv projection, fused gate_up projection (the reference's export writes
one, notebooks/save_A81W41_quantized_weight-qwen3_8b.ipynb cell 26), last-token lm_head, greedy argmax.  Every
linear goes through Context.linear (Qwen_Linear_with_bias_Int4::forward: quantize + QGEMM for
a prompt, + QGEMV for a single token); everything between them is the thin glue of
csrc/glue_ops.cu.  In a decode step (one token) the norms, SiLU*up, the activation quantizer and the residual
additions run in the epilogues of the kernels that produce each row (inkq_glue_decode_gemv,
inkq_glue_qkv_attention_quant): 5 launches per layer instead of 11.  One decode step is captured once as a CUDA
graph and replayed.

Column-sharded form (world > 1, one process per GPU): every linear holds the weight rows [rank*N/P, (rank+1)*N/P) of the
same seeded matrix, its epilogue stores the shard's output columns into every rank's copy of the output buffer over
peer-mapped memory (tp.PeerArena) and a barrier kernel follows; norms, attention, SiLU*up and the residual additions
run replicated on every rank on the assembled rows, as do the KV caches.  Per-column arithmetic is the one-GPU
arithmetic, so logits are bit-identical at every rank count.  The sharded decode step uses the separate operators
(the fused epilogues need a whole row inside one kernel).  `prefill_batch` runs several prompts of equal length as
one batch through the linears (M = prompts x tokens) with per-prompt KV caches.
"""
from __future__ import annotations

import ctypes as C
import dataclasses

import numpy as np


@dataclasses.dataclass
class Qwen3Config:
    layers: int = 36
    hidden: int = 4096
    nq: int = 32
    nkv: int = 8
    head_dim: int = 128
    ffn: int = 12288
    vocab: int = 151936
    rope_theta: float = 1e6
    eps: float = 1e-6
    max_pos: int = 512
    lm_head_fp16: bool = True     # fp16 lm_head (benchmark config); False: A81W41 like the reference
    decode_mode: str = "epilogue"  # decode step: "epilogue" (norm / SiLU*up / quantizer in the producers' epilogues, 5 launches per
                                   # layer), "prologue" (in the QGEMV prologues, 6 launches) or "separate" (one per operator: 11)
    decode_norm: str = "pending"   # "epilogue" decode mode: "pending" (each CTA quantizes its own 32 results, the row's RMS factor is applied
                                   # by the consumer: no whole-row pass) or "last_cta" (RMSNorm + quantizer by the CTA that finishes last)
    decode_qkv_attention: bool = True   # "epilogue" decode mode: q/k-norm, RoPE and the cache append inside the attention kernel
    prefill_mode: str = "fused"    # prompt: "fused" (residual add + RMSNorm + quantizer in one kernel, SiLU*up inside the quantizer,
                                   # attention quantizes its own output: 9 launches per layer) or "separate" (one kernel per
                                   # operator, 15 launches); same bits


def _p(t):
    return C.c_void_p(t.data_ptr())


class Qwen3Synthetic:
    def __init__(self, pkg, ctx, cfg: Qwen3Config, seed: int = 0, world: int = 1, rank: int = 0, dist=None, batch: int = 1, max_rows: int = 0):
        """world / rank / dist: column-sharded over `world` processes (dist = torch.distributed, initialised).  batch: number
        of per-prompt KV caches (prefill_batch).  max_rows: the largest number of rows (prompts x tokens) any call will pass;
        needed up front only when sharded (the peer-mapped output buffers are sized once)."""
        import torch
        assert cfg.head_dim == 128, "the glue kernels are written for head_dim 128"
        self.pkg, self.ctx, self.cfg, self.torch = pkg, ctx, cfg, torch
        self.world, self.rank, self.dist, self.batch = world, rank, dist, batch
        if world > 1:
            cfg.decode_mode = "separate"
        self.L = pkg.lib()
        g = torch.Generator(device="cuda")
        g.manual_seed(seed)
        H, F, V = cfg.hidden, cfg.ffn, cfg.vocab
        qkv_n = (cfg.nq + 2 * cfg.nkv) * cfg.head_dim

        def qlinear(N, K, row_perm=None):
            # nibbles uniform, d ~ U(0.002, 0.02) rounded to fp16, as the benchmark configs state.  The block
            # minimum is drawn around -7.5 d (the centre of the nibble range) instead of U(-0.1, 0): with a
            # non-zero weight mean every linear amplifies the common-mode part of its input by ~mean * K, a
            # random 36-layer stack then reaches 1e8-sized activations and the reference's fp16 scaled sums
            # (s = d * sum q, quantize_row_q8_1_repack_fp16) overflow in the decode path.  Timing does not
            # depend on the values.
            nib = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device="cuda", generator=g)
            d = (torch.rand((N, K // 32), device="cuda", generator=g) * 0.018 + 0.002).half().float()
            m = (-7.5 * d * (1.0 + 0.02 * torch.randn((N, K // 32), device="cuda", generator=g))).half().float()
            if row_perm is not None:
                nib, d, m = nib[row_perm].contiguous(), d[row_perm].contiguous(), m[row_perm].contiguous()
            n0, n1 = pkg.tp.shard_range(N, world, rank)      # every rank draws the same matrix and keeps its rows
            w = ctx.weight_dev(pkg.A81W41, pkg.SCALES_F16, N, K, nib, d, m, None, n0, n1)
            w.n_begin = n0
            return w

        # fused gate_up projection stored in (32 gate rows, 32 up rows) groups: stored row 64b + e is gate row 32b + e,
        # stored row 64b + 32 + e is up row 32b + e, so that one 64-row slice yields one quantization block of
        # SiLU(gate) * up (the decode GEMV's pair epilogue); the prompt path reads the same layout
        e = torch.arange(2 * F, device="cuda")
        gu_perm = torch.where((e % 64) < 32, (e // 64) * 32 + e % 32, F + (e // 64) * 32 + e % 32 - 32)

        self.layers = []
        for _ in range(cfg.layers):
            self.layers.append(dict(
                ln1=torch.ones(H, device="cuda"), ln2=torch.ones(H, device="cuda"),
                qn=torch.ones(cfg.head_dim, device="cuda"), kn=torch.ones(cfg.head_dim, device="cuda"),
                qkv=qlinear(qkv_n, H), o=qlinear(H, cfg.nq * cfg.head_dim), gate_up=qlinear(2 * F, H, gu_perm), down=qlinear(H, F),
                k_cache=torch.zeros((batch, cfg.nkv, cfg.max_pos, cfg.head_dim), dtype=torch.float16, device="cuda"),
                v_cache=torch.zeros((batch, cfg.nkv, cfg.max_pos, cfg.head_dim), dtype=torch.float16, device="cuda")))
        self.final_norm = torch.ones(H, device="cuda")
        self.embed = (torch.randn((V, H), device="cuda", generator=g) * 0.02).half()
        if cfg.lm_head_fp16:
            head = (torch.randn((V, H), device="cuda", generator=g) * 0.02).half()
            v0, v1 = pkg.tp.shard_range(V, world, rank)
            self.lm_head = ctx.f16w_dev(head, V, H, v0, v1)
            self.lm_head.n_begin = v0
            del head
        else:
            self.lm_head = qlinear(V, H)
        inv = 1.0 / (cfg.rope_theta ** (np.arange(0, cfg.head_dim, 2, dtype=np.float64) / cfg.head_dim))
        ang = np.outer(np.arange(cfg.max_pos, dtype=np.float64), inv)
        ang = np.concatenate([ang, ang], axis=1)                       # [max_pos][head_dim], both halves equal (HF layout)
        self.cos = torch.from_numpy(np.cos(ang).astype(np.float32)).cuda()
        self.sin = torch.from_numpy(np.sin(ang).astype(np.float32)).cuda()
        self.pos = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.token = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.generated = torch.zeros(4096, dtype=torch.int32, device="cuda")
        self.bufs = {}
        self.graph = None
        # quantized rows handed from kernel to kernel in the "epilogue" decode mode
        self.act_h = ctx.act(1, H)                        # input of qkv / gate_up
        self.act_attn = ctx.act(1, cfg.nq * cfg.head_dim)  # input of o_proj
        self.act_f = ctx.act(1, F)                        # input of down_proj
        self.arena = None
        if world > 1:
            rows = max(max_rows, 1)
            self.arena = pkg.tp.PeerArena(pkg, ctx, dist, world, rank, dict(qkv=(rows, qkv_n), proj=(rows, H), gu=(rows, 2 * F),
                                                                             logits=(max(batch, 1), V)))

    def close(self):
        if self.arena is not None:
            self.arena.close()
            self.arena = None

    def _gemm(self, name, w, act, T, out):
        """The same for T > 1 rows that a fused producer has already quantized into the activation handle `act`."""
        if self.arena is None:
            self.ctx.gemm(act, w, out, out.shape[1])
            return out
        self.arena.gemm(name, w, act, w.n_begin)
        self.arena.barrier()
        return self.arena.view(name, T)

    def _linear(self, name, w, x, T, out):
        """One quantized linear over T rows: on one GPU into `out`; sharded, into region `name` of every rank's arena
        (the returned tensor is then the assembled [T][N] matrix)."""
        if self.arena is None:
            self.ctx.linear(w, x, T, out, out.shape[1])
            return out
        self.arena.linear(name, w, x, T, w.n_begin)
        self.arena.barrier()
        return self.arena.view(name, T)

    # ------------------------------------------------------------------ buffers
    def _buffers(self, T):
        torch, cfg = self.torch, self.cfg
        if T not in self.bufs:
            qkv_n = (cfg.nq + 2 * cfg.nkv) * cfg.head_dim
            z = lambda *s: torch.empty(s, device="cuda", dtype=torch.float32)
            self.bufs[T] = dict(x=z(T, cfg.hidden), xn=z(T, cfg.hidden), qkv=z(T, qkv_n), q=z(T, cfg.nq * cfg.head_dim),
                                attn=z(T, cfg.nq * cfg.head_dim), proj=z(T, cfg.hidden), gu=z(T, 2 * cfg.ffn),
                                act=z(T, cfg.ffn), logits=z(1, cfg.vocab))
            if T > 1:   # quantized rows handed from the fused prompt kernels to the QGEMMs
                self.bufs[T]["qh"] = self.ctx.act(T, cfg.hidden)
                self.bufs[T]["qf"] = self.ctx.act(T, cfg.ffn)
                self.bufs[T]["qa"] = self.ctx.act(T, cfg.nq * cfg.head_dim)
        return self.bufs[T]

    def _chk(self, rc):
        self.ctx.check(rc)

    # ------------------------------------------------------------------ one forward over T tokens (tokens_dev int32 [T])
    def forward(self, tokens_dev, T, advance, nseq: int = 1):
        """Runs the T tokens (nseq prompts of T / nseq tokens each, every prompt at positions pos .. pos + T/nseq - 1 of its
        own cache) through the model, takes the last token's logits of each prompt, stores the argmax of the first
        prompt's in self.token (and the generated list) and advances pos by `advance`."""
        cfg, L, h, b = self.cfg, self.L, self.ctx.h, self._buffers(T)
        Ts = T // nseq
        assert nseq * Ts == T and nseq <= self.batch
        H, F = cfg.hidden, cfg.ffn
        scale = 1.0 / float(np.sqrt(cfg.head_dim))
        self._chk(L.inkq_glue_embedding(h, _p(self.embed), _p(tokens_dev), T, H, cfg.vocab, _p(b["x"])))
        mode = cfg.decode_mode if T == 1 else cfg.prefill_mode
        eps = C.c_float(cfg.eps)
        Q = self.pkg.Q8_1_F16
        if mode == "epilogue":
            # every product reads a ready quantized row; the producer of a row quantizes it in its epilogue
            nl = len(self.layers)
            self._chk(L.inkq_glue_rmsnorm_quant(h, _p(b["x"]), _p(self.layers[0]["ln1"]), eps, H, self.act_h.h, Q, None))
            for i, ly in enumerate(self.layers):
                self._chk(L.inkq_glue_decode_gemv(h, ly["qkv"].h, self.act_h.h, _p(b["qkv"]), 0, None, eps, None, Q, None))
                if cfg.decode_qkv_attention:
                    self._chk(L.inkq_glue_qkv_attention_quant(h, _p(b["qkv"]), _p(ly["qn"]), _p(ly["kn"]), _p(self.cos), _p(self.sin), _p(self.pos),
                                                              cfg.nq, cfg.nkv, cfg.max_pos, eps, C.c_float(scale), _p(ly["k_cache"][0]),
                                                              _p(ly["v_cache"][0]), self.act_attn.h, Q))
                else:
                    self._chk(L.inkq_glue_qknorm_rope_cache(h, _p(b["qkv"]), _p(ly["qn"]), _p(ly["kn"]), _p(self.cos), _p(self.sin), _p(self.pos), T,
                                                            cfg.nq, cfg.nkv, cfg.max_pos, eps, _p(b["q"]), _p(ly["k_cache"][0]), _p(ly["v_cache"][0])))
                    self._chk(L.inkq_glue_attention_quant(h, _p(b["q"]), _p(ly["k_cache"][0]), _p(ly["v_cache"][0]), _p(self.pos), cfg.nq, cfg.nkv,
                                                          cfg.max_pos, C.c_float(scale), self.act_attn.h, Q))
                tail = 4 if cfg.decode_norm == "pending" else 2
                self._chk(L.inkq_glue_decode_gemv(h, ly["o"].h, self.act_attn.h, _p(b["x"]), tail, _p(ly["ln2"]), eps, self.act_h.h, Q, None))
                self._chk(L.inkq_glue_decode_gemv(h, ly["gate_up"].h, self.act_h.h, None, 3, None, eps, self.act_f.h, Q, None))
                last = (i == nl - 1)    # the last layer's row goes to the lm_head as fp32: normalized by the last CTA
                nxt = self.final_norm if last else self.layers[i + 1]["ln1"]
                self._chk(L.inkq_glue_decode_gemv(h, ly["down"].h, self.act_f.h, _p(b["x"]), 2 if last else tail, _p(nxt), eps, self.act_h.h, Q,
                                                  _p(b["xn"]) if last else None))
        for ly in (self.layers if mode == "prologue" else []):
            # one launch per linear: norm / SiLU*up and the activation quantizer run in the QGEMV's prologue,
            # the residual connection in its epilogue (x += ...)
            self._chk(L.inkq_glue_linear_m1(h, ly["qkv"].h, _p(b["x"]), 1, _p(ly["ln1"]), eps, _p(b["qkv"]), 0))
            self._chk(L.inkq_glue_qknorm_rope_cache(h, _p(b["qkv"]), _p(ly["qn"]), _p(ly["kn"]), _p(self.cos), _p(self.sin), _p(self.pos), T,
                                                    cfg.nq, cfg.nkv, cfg.max_pos, eps, _p(b["q"]), _p(ly["k_cache"][0]), _p(ly["v_cache"][0])))
            self._chk(L.inkq_glue_attention(h, _p(b["q"]), _p(ly["k_cache"][0]), _p(ly["v_cache"][0]), _p(self.pos), T, cfg.nq, cfg.nkv, cfg.max_pos,
                                            C.c_float(scale), _p(b["attn"])))
            self._chk(L.inkq_glue_linear_m1(h, ly["o"].h, _p(b["attn"]), 0, None, eps, _p(b["x"]), 1))
            self._chk(L.inkq_glue_linear_m1(h, ly["gate_up"].h, _p(b["x"]), 1, _p(ly["ln2"]), eps, _p(b["gu"]), 0))
            self._chk(L.inkq_glue_linear_m1(h, ly["down"].h, _p(b["gu"]), 2, None, eps, _p(b["x"]), 1))
        pending = None     # fused prompt path: the down projection's output, added to x by the next norm kernel
        QM = self.pkg.Q8_1_F32    # what inkq_linear uses for an A81W41 layer with M > 1
        for ly in (self.layers if mode == "fused" else []):
            self._chk(L.inkq_glue_add_rmsnorm_quant_rows(h, _p(b["x"]), None if pending is None else _p(pending), _p(ly["ln1"]), eps, T, H,
                                                         b["qh"].h, QM, None))
            qkv = self._gemm("qkv", ly["qkv"], b["qh"], T, b["qkv"])
            for sq in range(nseq):
                rows = slice(sq * Ts, (sq + 1) * Ts)
                self._chk(L.inkq_glue_qknorm_rope_cache(h, _p(qkv[rows]), _p(ly["qn"]), _p(ly["kn"]), _p(self.cos), _p(self.sin), _p(self.pos), Ts,
                                                        cfg.nq, cfg.nkv, cfg.max_pos, eps, _p(b["q"][rows]), _p(ly["k_cache"][sq]),
                                                        _p(ly["v_cache"][sq])))
                self._chk(L.inkq_glue_attention_quant_rows(h, _p(b["q"][rows]), _p(ly["k_cache"][sq]), _p(ly["v_cache"][sq]), _p(self.pos), Ts, cfg.nq,
                                                           cfg.nkv, cfg.max_pos, C.c_float(scale), b["qa"].h, QM, sq * Ts, T))
            proj = self._gemm("proj", ly["o"], b["qa"], T, b["proj"])
            self._chk(L.inkq_glue_add_rmsnorm_quant_rows(h, _p(b["x"]), _p(proj), _p(ly["ln2"]), eps, T, H, b["qh"].h, QM, None))
            gu = self._gemm("gu", ly["gate_up"], b["qh"], T, b["gu"])       # fused gate_up projection, (32 gate, 32 up) column groups
            self._chk(L.inkq_glue_silu_mul_quant_rows(h, _p(gu), T, F, b["qf"].h, QM))
            pending = self._gemm("proj", ly["down"], b["qf"], T, b["proj"])
        if pending is not None:
            self._chk(L.inkq_glue_add_inplace(h, _p(b["x"]), _p(pending), C.c_longlong(T * H)))
        for ly in (self.layers if mode == "separate" else []):
            self._chk(L.inkq_glue_rmsnorm(h, _p(b["x"]), _p(ly["ln1"]), T, H, C.c_float(cfg.eps), _p(b["xn"])))
            qkv = self._linear("qkv", ly["qkv"], b["xn"], T, b["qkv"])
            for sq in range(nseq):            # per prompt: its own positions and KV cache
                rows = slice(sq * Ts, (sq + 1) * Ts)
                self._chk(L.inkq_glue_qknorm_rope_cache(h, _p(qkv[rows]), _p(ly["qn"]), _p(ly["kn"]), _p(self.cos), _p(self.sin), _p(self.pos), Ts,
                                                        cfg.nq, cfg.nkv, cfg.max_pos, C.c_float(cfg.eps), _p(b["q"][rows]), _p(ly["k_cache"][sq]),
                                                        _p(ly["v_cache"][sq])))
                self._chk(L.inkq_glue_attention(h, _p(b["q"][rows]), _p(ly["k_cache"][sq]), _p(ly["v_cache"][sq]), _p(self.pos), Ts, cfg.nq, cfg.nkv,
                                                cfg.max_pos, C.c_float(scale), _p(b["attn"][rows])))
            proj = self._linear("proj", ly["o"], b["attn"], T, b["proj"])
            self._chk(L.inkq_glue_add_inplace(h, _p(b["x"]), _p(proj), C.c_longlong(T * H)))
            self._chk(L.inkq_glue_rmsnorm(h, _p(b["x"]), _p(ly["ln2"]), T, H, C.c_float(cfg.eps), _p(b["xn"])))
            gu = self._linear("gu", ly["gate_up"], b["xn"], T, b["gu"])       # fused gate_up projection, (32 gate, 32 up) column groups
            self._chk(L.inkq_glue_silu_mul_rows(h, _p(gu), T, F, _p(b["act"])))
            proj = self._linear("proj", ly["down"], b["act"], T, b["proj"])
            self._chk(L.inkq_glue_add_inplace(h, _p(b["x"]), _p(proj), C.c_longlong(T * H)))
        if mode != "epilogue":      # (in that mode the last down_proj's epilogue has written the normalized row)
            if nseq == 1:
                last = b["x"][T - 1:T]
            else:
                last = b["x"][Ts - 1::Ts].contiguous()       # the last token of every prompt
            self._chk(L.inkq_glue_rmsnorm(h, _p(last), _p(self.final_norm), nseq, H, C.c_float(cfg.eps), _p(b["xn"])))
        logits = b["logits"] if nseq == 1 else self._batch_logits(nseq)
        if self.arena is not None:
            if cfg.lm_head_fp16:
                self.arena.f16w("logits", self.lm_head, b["xn"], nseq, self.lm_head.n_begin)
            else:
                self.arena.linear("logits", self.lm_head, b["xn"], nseq, self.lm_head.n_begin)
            self.arena.barrier()
            logits = self.arena.view("logits", nseq)
        elif cfg.lm_head_fp16:
            self.ctx.f16w_matmul(self.lm_head, b["xn"], nseq, logits, cfg.vocab)
        else:
            self.ctx.linear(self.lm_head, b["xn"], nseq, logits, cfg.vocab)
        self._chk(L.inkq_glue_argmax_advance(h, _p(logits), cfg.vocab, _p(self.token), _p(self.pos), advance, _p(self.generated),
                                             self.generated.numel()))
        return logits

    def _batch_logits(self, nseq):
        key = ("logits", nseq)
        if key not in self.bufs:
            self.bufs[key] = self.torch.empty((nseq, self.cfg.vocab), device="cuda", dtype=self.torch.float32)
        return self.bufs[key]

    def prefill_batch(self, prompts_dev):
        """prompts_dev int32 [B][T]: B prompts of equal length as one batch (B <= the `batch` the model was built with).
        Returns the logits [B][vocab] of each prompt's last token; pos advances by T."""
        B, T = int(prompts_dev.shape[0]), int(prompts_dev.shape[1])
        return self.forward(prompts_dev.reshape(-1), B * T, T, nseq=B)

    def reset(self):
        self.pos.zero_()
        self.generated.zero_()

    def prefill(self, prompt_dev):
        return self.forward(prompt_dev, int(prompt_dev.numel()), int(prompt_dev.numel()))

    def decode_step(self):
        return self.forward(self.token, 1, 1)

    def capture_decode(self):
        """Captures one decode step as a CUDA graph on a side stream (call after a prefill and one eager
        decode step, so that every scratch buffer already exists)."""
        torch = self.torch
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(s):
            self.ctx.set_stream(s.cuda_stream)
            with torch.cuda.graph(self.graph, stream=s):
                self.decode_step()
        self.ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        torch.cuda.current_stream().wait_stream(s)

    def generated_tokens(self):
        g = self.generated.cpu().numpy()
        return g[1:1 + int(g[0])]
