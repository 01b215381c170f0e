#!/usr/bin/env python
"""Benchmark of the A8W4 quantized-matmul path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One JSON line on stdout (rank 0).  A "step" is one forward of the quantized linear
layer (activation quantizer + QGEMM) on synthetic inputs of the prefill gate_proj
shape: M=322 activations x K=4096, N=12288 A81W41 weights (fp32 block scales).
  value   whole-job int8 TOPS (2*M*N*K per step) with inputs resident in HBM
  e2e     the same metric through the host-buffer entry point (inkq_linear_host):
          pinned host activations in, host result out, copies inside the timed region
          (N > 1: every rank calls it on its weight rows and delivers its columns of the
          result into one page-locked host matrix that all ranks map)
  N > 1   the weight rows (output columns) are sharded across the ranks, every rank
          quantizes the full activations and runs its shard; the QGEMM's epilogue stores
          each finished element into every rank's [M][N] buffer over peer-mapped memory
          and a barrier kernel completes the step (strong scaling; the same step with an
          NCCL all-gather is timed beside it, and is the fallback when peer mapping fails)
  --impl reference   the reference project's own AVX kernels (oracle/_ref, compiled
          unmodified) on this box's host cores, same shape, all host threads
The line also carries the roofline of the dominant kernel, the reference's CPU kernels timed on
this box, the decode QGEMV sweep, the scheme matrix and pp322 / tg128 of a synthetic Qwen3-8B
(--no-gemv / --no-model skip the last three).  Other workloads (--workload): qgemv_sweep,
qgemm_m2048, qgemm_m8192, lmhead_m8192 (fp16 lm_head 151936 x 4096 for 8192 rows on the tensor cores).
The K timed steps are repeated back to back until the timed region lasts --min-seconds (default 1 s), so
that the clock samples fall inside it; "repeats" says how often.
  --case NAME [ARGS]   runs one small fixed case of one kernel a few times and exits: what the profiler
          captures summarised under profiles/ run (qgemm [M], qgemv [N K], quantize [M], model [layers],
          w41 [M], lmhead [M])
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from __graft_entry__ import load_package  # noqa: E402

M_PP, K_PP, N_PP = 322, 4096, 12288
GEMV_SHAPES = [("q_proj/o_proj", 4096, 4096), ("k_proj/v_proj", 1024, 4096), ("gate/up_proj", 12288, 4096),
               ("down_proj", 4096, 12288), ("qkv_fused", 6144, 4096), ("gate_up_fused", 24576, 4096)]
L2_BYTES = 126e6


def peaks():
    p = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        p = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
             "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    except Exception:
        pass
    return p


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows = []
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=3)
        except Exception:
            pass
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
                for nme, v in zip(names, r[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(nme)
            except Exception:
                continue
        busy = [v for v in sm if mx and v > 0.5 * mx] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def base_config(wl, M, N, K):
    """The workload description both arms print (identical keys and values)."""
    if wl == "lmhead_m8192":
        return {"workload": wl, "M": M, "N": N, "K": K, "weights": "fp16", "activations": "fp32"}
    return {"workload": wl, "M": M, "N": N, "K": K, "scheme": "A81W41", "weight_scales": "fp32"}


def host_threads():
    """Pins the OpenMP team of the CPU checkers to every core this process may use (torchrun exports
    OMP_NUM_THREADS=1) and returns the team size OpenMP then reports."""
    try:
        want = len(os.sched_getaffinity(0))
    except AttributeError:
        want = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(want)
    try:
        gomp = ctypes.CDLL("libgomp.so.1", mode=ctypes.RTLD_GLOBAL)
        gomp.omp_set_num_threads(want)
        return int(gomp.omp_get_max_threads())
    except OSError:
        return want


def cuda_time_ms(torch, fn, iters):
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(iters):
        fn(i)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b)


# --------------------------------------------------------------------------- reference arm
def run_reference(args, rank, world):
    if rank != 0:
        return
    from oracle.inkq_oracle import Oracle, Reference
    pkg = load_package()
    M, K, N = M_PP, K_PP, N_PP
    x = pkg.synth.activations(M, K)
    w = pkg.synth.weights(N, K)
    cores = host_threads()
    kind = "reference" if Reference.available_path()[0] else "port"
    isa = "scalar"
    if kind == "reference":
        ref = Reference()
        isa = ref.isa
        B = ref.repack(w["nib"], w["d"], w["m"], 2)

        def step():
            A = ref.quantize_struct(x, 2, pad_rows=6 * K // 64, prefill=0)     # quantize_row_q8_1_repack_fp32
            return ref.matmul("gemm_repack_A81W41_fp32", A, B, M, N, K)       # gemm_repack_A81W41_fp32
        sample = (f"full workload: quantize_row_q8_1_repack_fp32 (1 thread, as the reference) + gemm_repack_A81W41_fp32 at {M}x{N}x{K} "
                  f"with an OpenMP team of {cores} threads (omp_get_max_threads after omp_set_num_threads)")
        ops = 2.0 * M * N * K
    else:
        orc = Oracle()
        ncols = 1536

        def step():
            q, d, s = orc.quantize(x, 2)
            return orc.gemm(0, q, d, s, w["nib"][:ncols], w["d"][:ncols], w["m"][:ncols])
        sample = f"first {ncols} of {N} output columns (oracle port, OpenMP over columns)"
        ops = 2.0 * M * ncols * K
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    step()
    est = time.perf_counter() - t0
    repeats = max(1, min(50, int(math.ceil(args.min_seconds / max(est * args.steps, 1e-6)))))
    t0 = time.perf_counter()
    for _ in range(args.steps * repeats):
        step()
    total = time.perf_counter() - t0
    dt = total / (args.steps * repeats)
    tops = ops / dt / 1e12
    line = {"impl": "reference", "metric": "qgemm_int8_tops_pp322", "value": tops, "unit": "TOPS", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "repeats": repeats, "timed_region_s": total,
            "ms_per_step": dt * 1e3 * (2.0 * M * N * K / ops), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "s8 x u4 -> s32, fp32 scale/accumulate", "data": "synthetic",
            "config": base_config("qgemm_pp322", M, N, K), "host": {"isa": isa, "omp_threads": cores},
            "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- CPU baseline leg of our arm
def cpu_baseline_pp322(pkg, x, w):
    from oracle.inkq_oracle import Oracle, Reference
    M, K, N = M_PP, K_PP, N_PP
    cores = host_threads()
    if Reference.available_path()[0]:
        ref = Reference()
        B = ref.repack(w["nib"], w["d"], w["m"], 2)
        iters, t_q, t_g = 0, 0.0, 0.0
        t_end = time.perf_counter() + 12.0
        ref.matmul("gemm_repack_A81W41_fp32", ref.quantize_struct(x, 2, pad_rows=6 * K // 64, prefill=0), B, M, N, K)
        while time.perf_counter() < t_end and iters < 200:
            t0 = time.perf_counter()
            A = ref.quantize_struct(x, 2, pad_rows=6 * K // 64, prefill=0)
            t1 = time.perf_counter()
            ref.matmul("gemm_repack_A81W41_fp32", A, B, M, N, K)
            t2 = time.perf_counter()
            t_q, t_g, iters = t_q + (t1 - t0), t_g + (t2 - t1), iters + 1
        per = (t_q + t_g) / iters
        return {"value": 2.0 * M * N * K / per / 1e12, "unit": "TOPS", "cores": cores, "kind": "reference",
                "sample": f"{iters} iterations of the full workload in ~12 s; quantizer {t_q / iters * 1e3:.2f} ms (1 thread, as the reference), "
                          f"GEMM {t_g / iters * 1e3:.2f} ms ({cores} threads), isa {ref.isa}"}
    orc = Oracle()
    ncols = 768
    t0 = time.perf_counter()
    q, d, s = orc.quantize(x, 2)
    orc.gemm(0, q, d, s, w["nib"][:ncols], w["d"][:ncols], w["m"][:ncols])
    dt = time.perf_counter() - t0
    return {"value": 2.0 * M * ncols * K / dt / 1e12, "unit": "TOPS", "cores": cores, "kind": "port",
            "sample": f"one pass over the first {ncols} of {N} columns with the scalar oracle"}


# --------------------------------------------------------------------------- GEMV sweep (extra figures)
def gemv_sweep(pkg, torch, ctx, peak_gbs, iters=200):
    out = []
    for name, n, k in GEMV_SHAPES:
        wt = pkg.synth.weights(n, k)
        per = n * k * 0.625
        copies = int(min(48, max(3, 2.2 * L2_BYTES // per + 1)))     # distinct weight sets: > L2 in total
        ws = [ctx.weight(pkg.A81W41, pkg.SCALES_F16, wt["nib"], wt["d"], wt["m"]) for _ in range(copies)]
        x = torch.randn((1, k), device="cuda")
        C = torch.empty((copies, n), device="cuda")
        act = ctx.act(1, k)
        ctx.quantize(act, x, 1, pkg.Q8_1_F16)
        torch.cuda.synchronize()
        # one CUDA graph that walks every copy once: launch gaps do not enter the figure
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            ctx.set_stream(s.cuda_stream)
            for i in range(copies):
                ctx.gemv(act, ws[i], C[i])
            torch.cuda.synchronize()
            with torch.cuda.graph(g, stream=s):
                for i in range(copies):
                    ctx.gemv(act, ws[i], C[i])
        ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        reps = max(3, iters // copies)
        for _ in range(2):
            g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1e3 / (reps * copies)
        nbytes = per + k + (k // 32) * 8 + n * 4
        gbs = nbytes / us / 1e3
        out.append({"shape": name, "N": n, "K": k, "us": round(us, 3), "GBs": round(gbs, 1), "frac_of_hbm": round(gbs / peak_gbs, 4),
                    "weight_sets": copies})
        for h in ws:
            h.close()
        act.close()
    return out


# --------------------------------------------------------------------------- scheme matrix and fp16 lm_head (extra figures)
def graph_time_us(torch, ctx, calls, reps=5):
    """Average device time of one call when the list of calls runs as one CUDA graph (launch gaps excluded)."""
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        ctx.set_stream(s.cuda_stream)
        for c in calls:
            c()
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=s):
            for c in calls:
                c()
    ctx.set_stream(torch.cuda.current_stream().cuda_stream)
    g.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / (reps * len(calls))


def scheme_matrix(pkg, torch, ctx, pk):
    """The layer's forward (quantizer + matmul, one call of inkq_linear; weight-only W41: fp16 activations into the
    tensor-core matmul) for every scheme at M in {1, 322, 2048}, K=4096, N=12288, rotating 6 weight sets (> L2)."""
    K, N, sets = K_PP, N_PP, 6
    wt = pkg.synth.weights(N, K)
    zp = wt["zp"]
    out = []
    for name, scheme in (("A81W41", pkg.A81W41), ("A80W40", pkg.A80W40), ("A80W4Z", pkg.A80W4Z), ("W41", pkg.W41)):
        m = wt["m"] if scheme in (pkg.A81W41, pkg.W41) else None
        z = zp if scheme == pkg.A80W4Z else None
        ws = [ctx.weight(scheme, pkg.SCALES_F16, wt["nib"], wt["d"], m, z) for _ in range(sets)]
        for M in (1, 322, 2048):
            x = torch.randn((M, K), device="cuda")
            x16 = x.half()
            C = torch.empty((M, N), device="cuda")
            if scheme == pkg.W41:
                calls = [(lambda w=w: ctx.gemm_w41_f16act(x16, M, w, C, N)) for w in ws]
            else:
                calls = [(lambda w=w: ctx.linear(w, x, M, C, N)) for w in ws]
            us = graph_time_us(torch, ctx, calls)
            row = {"scheme": name, "M": M, "us": round(us, 2), "TOPS": round(2.0 * M * N * K / us / 1e6, 2)}
            if M == 1:
                bpw = {"A81W41": 0.625, "A80W40": 0.5625 + 1 / 32, "A80W4Z": 0.5625 + 1 / 32, "W41": 0.625}[name]   # zero-point byte per block
                row["GBs"] = round(N * K * bpw / us / 1e3, 1)
                row["frac_of_hbm"] = round(row["GBs"] / pk["hbm_gbs"], 4)
            else:
                peak = pk["bf16_tflops"] * (1.0 if scheme == pkg.W41 else 2.0)
                row["frac_of_tensor_peak"] = round(row["TOPS"] / peak, 4)
            out.append(row)
        for h in ws:
            h.close()
    return out


def lm_head_gemv(pkg, torch, ctx, pk, vocab=151936, K=4096):
    """fp16 lm_head for one token (1.245 GB of weights per launch: far larger than L2)."""
    w16 = (torch.randn((vocab, K), device="cuda") * 0.02).half()
    wh = ctx.f16w_dev(w16, vocab, K)
    del w16
    x = torch.randn((1, K), device="cuda")
    C = torch.empty((1, vocab), device="cuda")
    us = graph_time_us(torch, ctx, [lambda: ctx.f16w_matmul(wh, x, 1, C, vocab)] * 4)
    wh.close()
    nbytes = vocab * K * 2 + K * 4 + vocab * 4
    return {"shape": "lm_head fp16", "N": vocab, "K": K, "us": round(us, 2), "GBs": round(nbytes / us / 1e3, 1),
            "frac_of_hbm": round(nbytes / us / 1e3 / pk["hbm_gbs"], 4)}


# --------------------------------------------------------------------------- synthetic Qwen3-8B forward (pp322 / tg128)
def model_pp_tg(pkg, torch, ctx, prompt_len=322, new_tokens=128, reps=3):
    """Prompt prefill and greedy decode of the synthetic Qwen3-8B (random-init A81W41 weights with fp16 block
    scales, fp16 lm_head, fp16 KV cache), activations resident on the GPU.  pp = prompt tokens / prefill time,
    tg = generated tokens / time of the decode steps (one captured CUDA graph replayed per token)."""
    cfg = pkg.qwen3_forward.Qwen3Config(max_pos=prompt_len + new_tokens + 32)
    model = pkg.qwen3_forward.Qwen3Synthetic(pkg, ctx, cfg, seed=7)
    prompt = torch.from_numpy(pkg.synth.tokens(prompt_len, cfg.vocab)).cuda()
    model.reset()
    model.prefill(prompt)
    n0 = ctx.launches
    model.decode_step()
    launches_per_token = ctx.launches - n0      # counted by the library: one eager decode step
    model.capture_decode()
    torch.cuda.synchronize()
    pp_ms, tg_ms = [], []
    for _ in range(reps):
        model.reset()
        a, b, c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        a.record()
        model.prefill(prompt)
        b.record()
        for _ in range(new_tokens):
            model.graph.replay()
        c.record()
        torch.cuda.synchronize()
        pp_ms.append(a.elapsed_time(b))
        tg_ms.append(b.elapsed_time(c))
    n_gen = len(model.generated_tokens())
    # the same decode step with every operator as its own launch, for comparison
    unfused_ms = None
    if cfg.decode_mode != "separate":
        model.cfg.decode_mode = "separate"
        model.reset()
        model.prefill(prompt)
        model.decode_step()
        model.capture_decode()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(new_tokens):
            model.graph.replay()
        b.record()
        torch.cuda.synchronize()
        unfused_ms = a.elapsed_time(b) / new_tokens
    pp, tg = prompt_len / (min(pp_ms) * 1e-3), new_tokens / (min(tg_ms) * 1e-3)
    w_bytes = cfg.layers * ((cfg.nq + 2 * cfg.nkv) * 128 * cfg.hidden + cfg.hidden * cfg.nq * 128 + 3 * cfg.hidden * cfg.ffn) * 0.625 \
        + cfg.vocab * cfg.hidden * 2
    out = {"pp322_tok_s": pp, "tg128_tok_s": tg, "prefill_ms": min(pp_ms), "decode_ms_per_token": min(tg_ms) / new_tokens,
           "tokens_generated_last_rep": int(n_gen), "decode_weight_bytes_per_token": w_bytes,
           "decode_GBs": w_bytes / (min(tg_ms) / new_tokens * 1e-3) / 1e9,
           "decode_launches_per_token": launches_per_token,
           "decode_ms_per_token_unfused_kernels": unfused_ms,
           "published_reference_cpu": {"pp322_tok_s": 134.35, "tg128_tok_s": 9.26, "hardware": "Intel i5-13600KF, 16 threads (reference README)"},
           "vs_published": {"pp322": pp / 134.35, "tg128": tg / 9.26},
           "config": "Qwen3-8B shape: 36 layers, hidden 4096, 32q/8kv heads x128, ffn 12288, vocab 151936; A81W41 fp16 scales, fp16 lm_head and KV cache; "
                     "synthetic weights and tokens"}
    del model
    torch.cuda.empty_cache()
    return out


def model_tp(pkg, torch, dist, ctx, world, rank, prompt_len=322, new_tokens=128, batch=8):
    """The synthetic Qwen3-8B with every linear column-sharded over `world` GPUs (outputs exchanged by the kernels' own
    peer stores + a barrier kernel per linear; norms, attention and caches replicated): pp322, tg128 (separate operators
    per decode step, captured as one CUDA graph) and the prefill of `batch` prompts of 322 tokens as one batch.
    Times are the maximum over ranks."""
    cfg = pkg.qwen3_forward.Qwen3Config(max_pos=prompt_len + new_tokens + 32, decode_mode="separate")
    model = pkg.qwen3_forward.Qwen3Synthetic(pkg, ctx, cfg, seed=7, world=world, rank=rank, dist=dist if world > 1 else None,
                                             batch=batch, max_rows=batch * prompt_len)
    prompt = torch.from_numpy(pkg.synth.tokens(prompt_len, cfg.vocab)).cuda()
    prompts = torch.from_numpy(np.stack([pkg.synth.tokens(prompt_len, cfg.vocab, 1007 + i) for i in range(batch)])).cuda()

    def mx(v):
        if world == 1:
            return v
        t = torch.tensor([v], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    model.reset()
    model.prefill(prompt)
    n0 = ctx.launches
    model.decode_step()
    step_launches = ctx.launches - n0      # counted by the library (barrier kernels included)
    model.capture_decode()
    torch.cuda.synchronize()
    pp_ms, tg_ms, pb_ms = [], [], []
    for _ in range(2):
        model.reset()
        if world > 1:
            dist.barrier()
        a, b, c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        a.record()
        model.prefill(prompt)
        b.record()
        for _ in range(new_tokens):
            model.graph.replay()
        c.record()
        torch.cuda.synchronize()
        pp_ms.append(mx(a.elapsed_time(b)))
        tg_ms.append(mx(b.elapsed_time(c)))
        model.reset()
        if world > 1:
            dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        model.prefill_batch(prompts)
        b.record()
        torch.cuda.synchronize()
        pb_ms.append(mx(a.elapsed_time(b)))
    out = {"n_gpus": world, "pp322_tok_s": prompt_len / (min(pp_ms) * 1e-3), "tg128_tok_s": new_tokens / (min(tg_ms) * 1e-3),
           "prefill_ms": min(pp_ms), "decode_ms_per_token": min(tg_ms) / new_tokens,
           "batch_prefill": {"prompts": batch, "tokens_each": prompt_len, "ms": min(pb_ms), "tok_s": batch * prompt_len / (min(pb_ms) * 1e-3)},
           "decode_mode": "one kernel per operator" + (" + a barrier kernel per sharded linear" if world > 1 else "") + ", one CUDA graph per step",
           "decode_launches_per_token": step_launches,
           "sharding": "every linear column-sharded, outputs exchanged by peer stores from the kernels' epilogues" if world > 1 else "none"}
    model.close()
    del model
    torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------- helpers of our arm
def timed_region(torch, dist, world, run_k_steps, est_ms_per_k, min_seconds):
    """Runs `run_k_steps()` (K steps) R times back to back between two CUDA events, R chosen so that the region lasts
    about min_seconds; returns (total ms = max over ranks, R)."""
    repeats = max(1, min(20000, int(math.ceil(min_seconds * 1e3 / max(est_ms_per_k, 1e-3)))))
    if world > 1:
        t = torch.tensor([repeats], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)      # every rank runs the same number of steps
        repeats = int(t.item())
        dist.barrier()
    torch.cuda.synchronize()
    ms = cuda_time_ms(torch, lambda i: run_k_steps(), repeats)
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    return ms, repeats


def capture_steps(torch, ctx, step, k):
    """K steps as one CUDA graph (a sharded step is tens of microseconds of GPU work; one Python process per GPU
    cannot enqueue its launches that fast).  Returns the graph, or None when capture is not possible."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    try:
        with torch.cuda.stream(side):
            ctx.set_stream(side.cuda_stream)
            with torch.cuda.graph(graph, stream=side):
                for i in range(k):
                    step(i)
    except Exception:
        graph = None
    finally:
        ctx.set_stream(torch.cuda.current_stream().cuda_stream)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    return graph


def tp_check(pkg, torch, dist, ctx, scatter, w_shard, wt, x, M, N, rank):
    """The exchange under test against one GPU: rank 0 computes the unsharded [M][N] once and broadcasts it, every
    rank runs one sharded step and compares its assembled matrix bit for bit."""
    full = torch.empty((M, N), device="cuda")
    if rank == 0:
        w_full = ctx.weight(pkg.A81W41, pkg.SCALES_F32, wt["nib"], wt["d"], wt["m"])
        ctx.linear(w_full, x, M, full, N)
        ctx.synchronize()
        w_full.close()
    dist.broadcast(full, 0)
    scatter.linear(w_shard, x, 0)
    scatter.barrier()
    ctx.synchronize()
    ok = torch.tensor([1 if torch.equal(scatter.result(0), full) else 0], device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    return bool(ok.item())


def scaling_m8192(pkg, torch, dist, ctx, world, rank, pk, min_seconds=0.3):
    """The column-sharded large-M workloads of the scaling configuration, timed like the headline step (K steps in a
    graph when sharded, max over ranks): the M=8192 prefill QGEMM (12288 x 4096) and the fp16 lm_head GEMM
    (151936 x 4096 for 8192 rows, activations rounded to fp16: one pass over the weights)."""
    out = {}
    M, K = 8192, K_PP
    x = torch.randn((M, K), device="cuda", generator=torch.Generator(device="cuda").manual_seed(5))
    # ---- QGEMM
    N = N_PP
    n0, n1 = pkg.tp.shard_range(N, world, rank)
    wt = pkg.synth.weights(N, K)
    sets = 3
    ws = [ctx.weight(pkg.A81W41, pkg.SCALES_F32, wt["nib"], wt["d"], wt["m"], None, n0, n1) for _ in range(sets)]
    sc = pkg.tp.PeerScatter(pkg, ctx, dist, M, N, world, rank, slots=2) if world > 1 else None
    Cl = torch.empty((M, n1 - n0), device="cuda") if world == 1 else None

    def step(i):
        if sc is None:
            ctx.linear(ws[i % sets], x, M, Cl, n1 - n0)
        else:
            sc.linear(ws[i % sets], x, i % 2)
            sc.barrier()
    k = 6
    for i in range(3):
        step(i)
    torch.cuda.synchronize()
    g = capture_steps(torch, ctx, step, k) if world > 1 else None
    run = (lambda: g.replay()) if g is not None else (lambda: [step(i) for i in range(k)])
    run()
    torch.cuda.synchronize()
    est = cuda_time_ms(torch, lambda i: run(), 1)
    ms, reps = timed_region(torch, dist, world, run, est, min_seconds)
    per = ms / (reps * k)
    out["qgemm"] = {"M": M, "N": N, "K": K, "ms_per_step": per, "TOPS": 2.0 * M * N * K / (per * 1e-3) / 1e12,
                    "timing": "graph" if g is not None else "eager", "exchange": "peer stores from the epilogue + barrier kernel" if sc else "none"}
    for h in ws:
        h.close()
    if sc is not None:
        sc.close()
    del sc, Cl, g
    torch.cuda.empty_cache()
    # ---- fp16 lm_head
    vocab = 151936
    v0, v1 = pkg.tp.shard_range(vocab, world, rank)
    gen = torch.Generator(device="cuda").manual_seed(1006)
    w16 = (torch.randn((v1 - v0, K), device="cuda", generator=gen) * 0.02).half()
    wh = ctx.f16w_dev(w16, v1 - v0, K)
    del w16
    # (a) every rank keeps the logits of its own vocabulary columns (what a sharded sampler consumes: per-row maxima meet
    #     in a few bytes); (b) every rank receives the whole [M][vocab] fp32 matrix through the epilogue's peer stores:
    #     (P-1)/P of 5 GB leave every rank, so that arm is bound by NVLink, not by the tensor cores
    Cl = torch.empty((M, v1 - v0), device="cuda")

    def lstep(i):
        ctx.f16w_matmul_prec(wh, x, M, Cl, v1 - v0, 1)
    for i in range(2):
        lstep(i)
    torch.cuda.synchronize()
    est = cuda_time_ms(torch, lambda i: lstep(i), 1)
    ms, reps = timed_region(torch, dist, world, lambda: lstep(0), est, min_seconds)
    per = ms / reps
    flop = 2.0 * M * vocab * K
    out["lm_head"] = {"M": M, "N": vocab, "K": K, "ms_per_step": per, "TFLOPS": flop / (per * 1e-3) / 1e12,
                      "frac_of_bf16_burst_per_gpu": flop / (per * 1e-3) / 1e12 / pk["bf16_tflops"] / world, "activations": "fp16 (one pass)",
                      "timing": "eager", "exchange": "none: every rank keeps the logits of its vocabulary columns"}
    del Cl
    torch.cuda.empty_cache()
    sc = pkg.tp.PeerScatter(pkg, ctx, dist, M, vocab, world, rank, slots=1) if world > 1 else None
    if sc is not None:
        def gstep(i):
            ctx.f16w_matmul_scatter(wh, x, M, sc.ps, pkg.tp.scatter_offset(0, M, vocab, v0, pkg.PEER_RESERVED_BYTES), vocab, 1)
            sc.barrier()
        for i in range(2):
            gstep(i)
        torch.cuda.synchronize()
        est = cuda_time_ms(torch, lambda i: gstep(i), 1)
        ms, reps = timed_region(torch, dist, world, lambda: gstep(0), est, min_seconds)
        per = ms / reps
        sent = 4.0 * M * (v1 - v0) * (world - 1)
        out["lm_head_gathered"] = {"ms_per_step": per, "TFLOPS": flop / (per * 1e-3) / 1e12, "nvlink_bytes_sent_per_rank": sent,
                                   "nvlink_GBs_per_rank": sent / (per * 1e-3) / 1e9,
                                   "exchange": "peer stores from the epilogue + barrier kernel: every rank ends with the whole [M][vocab] matrix"}
    wh.close()
    if sc is not None:
        sc.close()
    return out


# --------------------------------------------------------------------------- the lm_head workload (one GPU)
def run_lmhead(args, pkg, torch, ctx, pk, local_rank):
    M, K, N = 8192, K_PP, 151936
    gen = torch.Generator(device="cuda").manual_seed(1006)
    w16 = (torch.randn((N, K), device="cuda", generator=gen) * 0.02).half()
    wh = ctx.f16w_dev(w16, N, K)
    del w16
    x_host = pkg.synth.activations(M, K)
    x = torch.from_numpy(x_host).cuda()
    C = torch.empty((M, N), device="cuda")
    sampler = ClockSampler(local_rank)
    sampler.start()
    res = {}
    for name, prec in (("fp16_activations_one_pass", 1), ("fp32_grade_two_passes", 0)):
        for _ in range(max(1, args.warmup // 2)):
            ctx.f16w_matmul_prec(wh, x, M, C, N, prec)
        torch.cuda.synchronize()
        l0 = ctx.launches
        est = cuda_time_ms(torch, lambda i: ctx.f16w_matmul_prec(wh, x, M, C, N, prec), 1)
        k = max(1, min(args.steps, 10))
        ms, reps = timed_region(torch, None, 1, lambda: [ctx.f16w_matmul_prec(wh, x, M, C, N, prec) for _ in range(k)], est * k, args.min_seconds)
        res[name] = {"ms_per_step": ms / (reps * k), "steps": k, "repeats": reps, "launches": ctx.launches - l0}
    clocks = sampler.stop()
    flop = 2.0 * M * N * K
    one = res["fp16_activations_one_pass"]
    tf = flop / (one["ms_per_step"] * 1e-3) / 1e12
    line = {"metric": "lmhead_fp16w_tflops_m8192", "value": tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": one["steps"], "warmup": args.warmup,
            "repeats": one["repeats"], "ms_per_step": one["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp16 x fp16 -> fp32 (tcgen05 kind::f16), activations rounded from fp32", "data": "synthetic",
            "config": base_config("lmhead_m8192", M, N, K), "clocks": clocks, "gpu_launches": int(one["launches"]),
            "roofline": {"bound": "tensor", "achieved": tf, "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": tf / pk["bf16_tflops"],
                         "traffic": None, "kernel": "k_gemm_f16w_tc", "peak_note": f"{pk['source']} dense bf16 burst figure"},
            "fp32_grade_two_passes": {"ms_per_step": res["fp32_grade_two_passes"]["ms_per_step"],
                                      "TFLOPS_nominal": flop / (res["fp32_grade_two_passes"]["ms_per_step"] * 1e-3) / 1e12,
                                      "note": "inkq_f16w_matmul's default: the activations enter as fp16 hi + lo, two passes over the weights"},
            "e2e": None, "cpu_baseline": None}
    print(json.dumps(line), flush=True)
    wh.close()


# --------------------------------------------------------------------------- small fixed cases for profiler captures
def run_case(args):
    import torch
    pkg = load_package()
    what, nums = args.case[0], [int(a) for a in args.case[1:]]
    torch.cuda.set_device(0)
    ctx = pkg.Context(0, torch.cuda.current_stream().cuda_stream)
    if what == "qgemm":
        M, N, K = (nums + [M_PP])[0], N_PP, K_PP
        w = pkg.synth.weights(N, K)
        wh = ctx.weight(pkg.A81W41, pkg.SCALES_F32, w["nib"], w["d"], w["m"])
        x = torch.from_numpy(pkg.synth.activations(M, K)).cuda()
        C = torch.empty((M, N), device="cuda")
        act = ctx.act(M, K)
        for _ in range(3):
            ctx.quantize(act, x, M, pkg.Q8_1_F32)
            ctx.gemm(act, wh, C, N)
        ctx.synchronize()
        print("qgemm ok", M, N, K, float(C.abs().mean()))
    elif what == "qgemv":
        N, K = (nums + [12288, 4096])[:2]
        w = pkg.synth.weights(N, K)
        whs = [ctx.weight(pkg.A81W41, pkg.SCALES_F16, w["nib"], w["d"], w["m"]) for _ in range(12)]   # distinct sets: > L2 in total
        x = torch.from_numpy(pkg.synth.activations(1, K)).cuda()
        C = torch.empty((1, N), device="cuda")
        act = ctx.act(1, K)
        ctx.quantize(act, x, 1, pkg.Q8_1_F16)
        for wh in whs:
            ctx.gemv(act, wh, C)
        ctx.synchronize()
        print("qgemv ok", N, K, float(C.abs().mean()))
    elif what == "quantize":
        M, K = (nums + [8192])[0], K_PP
        x = torch.randn((M, K), device="cuda")
        act = ctx.act(M, K)
        for _ in range(3):
            ctx.quantize(act, x, M, pkg.Q8_1_F32)
        ctx.synchronize()
        print("quantize ok", M, K)
    elif what == "model":
        layers = (nums + [2])[0]
        cfg = pkg.qwen3_forward.Qwen3Config(layers=layers, max_pos=512)
        model = pkg.qwen3_forward.Qwen3Synthetic(pkg, ctx, cfg, seed=7)
        prompt = torch.from_numpy(pkg.synth.tokens(322, cfg.vocab)).cuda()
        model.reset()
        model.prefill(prompt)
        for _ in range(3):
            model.decode_step()
        ctx.synchronize()
        print("model ok", layers, model.generated_tokens())
    elif what == "w41":
        M, N, K = (nums + [2048])[0], N_PP, K_PP
        w = pkg.synth.weights(N, K)
        wh = ctx.weight(pkg.W41, pkg.SCALES_F16, w["nib"], w["d"], w["m"])
        a16 = torch.from_numpy(pkg.synth.activations(M, K)).cuda().half()
        C = torch.empty((M, N), device="cuda")
        for _ in range(3):
            ctx.gemm_w41_f16act(a16, M, wh, C, N)
        ctx.synchronize()
        print("w41 ok", M, N, K, float(C.abs().mean()))
    elif what == "lmhead":
        M, N, K = (nums + [2048])[0], 32768, K_PP            # a slice of the vocabulary: > L2, a few hundred MB on the device
        w16 = (torch.randn((N, K), device="cuda") * 0.02).half()
        wh = ctx.f16w_dev(w16, N, K)
        x = torch.randn((M, K), device="cuda")
        C = torch.empty((M, N), device="cuda")
        for _ in range(3):
            ctx.f16w_matmul_prec(wh, x, M, C, N, 1)
        ctx.synchronize()
        print("lmhead ok", M, N, K, float(C.abs().mean()))
    else:
        raise SystemExit("unknown case " + what)


# --------------------------------------------------------------------------- our arm
def run_ours(args, rank, world, local_rank):
    import torch
    pkg = load_package()
    pk = peaks()
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":    # its banner would share stdout with the JSON line
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = pkg.Context(local_rank, torch.cuda.current_stream().cuda_stream)

    wl = args.workload
    if wl == "lmhead_m8192":
        if world > 1:
            raise SystemExit("the lm_head workload is a one-GPU line; its sharded form is part of `scaling_m8192` of the N > 1 headline run")
        return run_lmhead(args, pkg, torch, ctx, pk, local_rank)
    M = {"qgemm_pp322": M_PP, "qgemm_m2048": 2048, "qgemm_m8192": 8192, "qgemv_sweep": M_PP}[wl]
    K, N = K_PP, N_PP
    n0, n1 = pkg.tp.shard_range(N, world, rank)
    n_loc = n1 - n0
    x_host = pkg.synth.activations(M, K)
    wt = pkg.synth.weights(N, K)

    # distinct weight sets so that consecutive steps never find their weights in L2
    w_bytes_one = n_loc * K * (0.5 + 0.125 * 3) + n_loc * (K // 64) * 2
    sets = int(max(3, min(16, 1.5 * L2_BYTES // w_bytes_one + 2)))
    ws = [ctx.weight(pkg.A81W41, pkg.SCALES_F32, wt["nib"], wt["d"], wt["m"], None, n0, n1) for _ in range(sets)]
    xs = [torch.from_numpy(x_host).cuda() for _ in range(sets)]
    scatter, exchange, tp_equal = None, "single GPU", None
    if world > 1:
        cg = pkg.tp.ColumnGather(dist, M, N, world, rank, "cuda", torch.float32)   # in-place all-gather target
        Cs = [cg.local]
        try:
            scatter = pkg.tp.PeerScatter(pkg, ctx, dist, M, N, world, rank, slots=2)
            exchange = f"tp{world}: N-sharded, QGEMM epilogue stores into every rank's [M][N] over NVLink + barrier kernel"
        except RuntimeError as e:
            exchange = f"tp{world}: N-sharded, NCCL all-gather (peer mapping unavailable: {str(e)[:120]})"
    else:
        Cs = [torch.empty((M, n_loc), device="cuda") for _ in range(2)]

    def step_gather(i):
        ctx.linear(ws[i % sets], xs[i % sets], M, Cs[i % len(Cs)], n_loc)   # quantizer + QGEMM (Qwen_Linear_with_bias_Int4::forward)
        if world > 1:
            cg.gather()                                                 # NCCL all-gather + [P][M][N/P] -> [M][N]

    def step_scatter(i):
        scatter.linear(ws[i % sets], xs[i % sets], i % 2)               # quantizer + QGEMM, C stored on every rank
        scatter.barrier()

    step = step_scatter if scatter is not None else step_gather
    if scatter is not None:
        tp_equal = tp_check(pkg, torch, dist, ctx, scatter, ws[0], wt, xs[0], M, N, rank)

    sampler = ClockSampler(local_rank)
    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    # a sharded step is replayed from a CUDA graph of the K steps; the barrier kernel keeps its count in device memory,
    # so a replay is a valid sequence of K more barriers
    graph = capture_steps(torch, ctx, step, args.steps) if scatter is not None else None
    run_k = (lambda: graph.replay()) if graph is not None else (lambda: [step(i) for i in range(args.steps)])
    run_k()                                  # untimed: every rank runs the same K steps
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    est = cuda_time_ms(torch, lambda i: run_k(), 1)
    l0 = ctx.launches
    sampler.start()                          # clocks are sampled over the timed region
    ms, repeats = timed_region(torch, dist, world, run_k, est, args.min_seconds)
    clocks = sampler.stop()
    launches = (3 * args.steps * repeats) if graph is not None else (ctx.launches - l0)   # quantizer, QGEMM (+ barrier kernel) per step
    ctx.synchronize()
    ops = 2.0 * M * N * K
    n_steps = args.steps * repeats
    tops = ops * n_steps / (ms * 1e-3) / 1e12

    roof, quant = None, None
    if rank == 0:
        # ---- kernel-only figures for the roofline (dominant kernel: the tensor-core QGEMM), taken right after the timed
        # region: the heavier extras further down push the GPU into its power cap
        act = ctx.act(M, K)
        ctx.quantize(act, xs[0], M, pkg.Q8_1_F32)
        Ck = torch.empty((M, n_loc), device="cuda")
        for i in range(3):
            ctx.gemm(act, ws[i % sets], Ck, n_loc)
        torch.cuda.synchronize()
        it = max(10, args.steps)
        ms_g = cuda_time_ms(torch, lambda i: ctx.gemm(act, ws[i % sets], Ck, n_loc), it) / it
        ms_q = cuda_time_ms(torch, lambda i: ctx.quantize(act, xs[i % sets], M, pkg.Q8_1_F32), it) / it
        ach = 2.0 * M * n_loc * K / (ms_g * 1e-3) / 1e12
        int8_peak = 2.0 * pk["bf16_tflops"]
        full_shape = wl in ("qgemm_pp322", "qgemv_sweep") and world == 1
        roof = {"bound": "tensor", "achieved": ach, "peak": int8_peak, "unit": "TOP/s", "frac": ach / int8_peak,
                            "traffic": 41.12e6 if full_shape else None,
                            "traffic_source": "profiles/qgemm_tc_pp322.md: dram__bytes_read.sum + dram__bytes_write.sum of one launch at this shape "
                                              "(not measured by this run)" if full_shape else None,
                            "kernel": "k_qgemm_tc", "us_per_launch": ms_g * 1e3,
                            "peak_note": f"2 x the {pk['source']} dense bf16 figure ({pk['bf16_tflops']} TFLOP/s); int8 itself is not in MEASURED_PEAKS.json",
                            "cuda_core_note": "every K=32 MMA is followed by an fp32 scale+accumulate of its whole tile on the CUDA cores "
                                              "(M*N*K/32 block dots per launch); that, not the tensor pipe, bounds this kernel"}
        # the second roof of this kernel: the per-block fp32 epilogue on the CUDA cores.  The exact operation order needs, per
        # block dot, three fp32 operations on the FMA pipe (scale product, main term, min term); the packed f32x2 forms occupy
        # the pipe for two cycles, so the floor is 3 FMA-pipe lane-cycles per block dot at 128 lanes per SM.
        tiles_m = -(-M // 128)
        bm = -(-(-(-M // tiles_m)) // 16) * 16
        dots = float(tiles_m * bm) * n_loc * (K // 32)
        sm_clock = (clocks.get("sm_mhz") or 1965.0) * 1e6
        n_sms = torch.cuda.get_device_properties(local_rank).multi_processor_count
        t_min = dots * 3.0 / 128.0 / n_sms / sm_clock
        roof["cuda_core_roof"] = {"block_dots_per_launch": dots, "fma_pipe_ops_per_block_dot": 3.0,
                                              "min_us": t_min * 1e6, "frac": t_min / (ms_g * 1e-3)}
        quant = {"us_per_launch": ms_q * 1e3, "GBs": M * K * 5.375 / (ms_q * 1e-3) / 1e9, "frac_of_hbm": M * K * 5.375 / (ms_q * 1e-3) / 1e9 / pk["hbm_gbs"]}
        act.close()

    gather_cmp = None
    if scatter is not None:
        # The library-collective variant of the same step.  Both arms are timed the same way here - eager launches from
        # Python, which for a step this short includes the host's enqueue cost - so that the pair of numbers compares the
        # exchange methods; the headline above replays the peer-store step from a CUDA graph.  (The NCCL arm is not
        # captured: a collective inside a capture is at the mercy of the process group's watchdog.)
        def eager_tops(fn):
            for i in range(args.warmup):
                fn(i)
            torch.cuda.synchronize()
            dist.barrier()
            est_e = cuda_time_ms(torch, lambda i: [fn(j) for j in range(args.steps)], 1)
            ms_e, rep_e = timed_region(torch, dist, world, lambda: [fn(j) for j in range(args.steps)], est_e, min(args.min_seconds, 0.3))
            return ops * args.steps * rep_e / (ms_e * 1e-3) / 1e12
        gather_cmp = {"nccl_all_gather_TOPS": eager_tops(step_gather), "peer_stores_TOPS": eager_tops(step_scatter), "timing": "eager launches, both"}
        ctx.synchronize()

    line = {"metric": "qgemm_int8_tops_pp322" if wl in ("qgemm_pp322", "qgemv_sweep") else f"qgemm_int8_tops_{wl.split('_')[1]}",
            "value": tops, "unit": "TOPS", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "repeats": repeats,
            "timed_region_s": ms * 1e-3, "ms_per_step": ms / n_steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "s8 x u4 -> s32 block dots (tcgen05 kind::i8), fp32 scale/accumulate", "data": "synthetic",
            "config": base_config(wl if wl != "qgemv_sweep" else "qgemm_pp322", M, N, K),
            "run": {"parallelism": exchange, "timing": "CUDA graph of the K steps, replayed" if graph is not None else "eager launches",
                    "l2": f"{sets} distinct weight sets ({sets * w_bytes_one / 1e6:.0f} MB per rank) rotated between steps, > 126 MB L2"},
            "clocks": clocks, "gpu_launches": int(launches)}
    if clocks.get("sm_mhz"):
        line["clocks"]["ms_per_step_x_sm_mhz"] = ms / n_steps * clocks["sm_mhz"]
    if roof is not None:
        line["roofline"], line["quantizer"] = roof, quant
    if tp_equal is not None:
        line["tp_equals_1gpu"] = tp_equal
    if gather_cmp is not None:
        line["run"]["exchange_methods_eager"] = gather_cmp

    # ---- end to end through host buffers, every N: pinned host activations in, the [M][N] result out to the host
    it = max(10, args.steps)
    if world == 1:
        xh = torch.from_numpy(x_host).pin_memory()
        ch = torch.empty((M, N), dtype=torch.float32).pin_memory()
        for i in range(3):
            ctx.linear_host(ws[i % sets], xh, M, ch, N)
        t0 = time.perf_counter()
        for i in range(it):
            ctx.linear_host(ws[i % sets], xh, M, ch, N)
        dt = (time.perf_counter() - t0) / it
        e2e = {"value": ops / dt / 1e12, "unit": "TOPS", "h2d_bytes_per_step": M * K * 4, "d2h_bytes_per_step": M * N * 4, "ms_per_step": dt * 1e3,
               "path": "inkq_linear_host (windows of rows: activations in, quantizer + QGEMM, finished rows out, on three streams)"}
    elif scatter is not None:
        # Sharded: every rank calls the host-buffer entry point on its own weight rows and delivers its own columns of the
        # result straight into one host matrix that all ranks map (a file in /dev/shm, page-locked by every process): the
        # activations go up every rank's own PCIe link in parallel, the result comes down P links at once, and no GPU-to-GPU
        # exchange is needed at all.
        xh = torch.from_numpy(x_host).pin_memory()
        shm_path = f"/dev/shm/inkq_e2e_{os.environ.get('MASTER_PORT', '0')}_{os.getuid()}.bin"
        if rank == 0:
            with open(shm_path, "wb") as f:
                f.truncate(M * N * 4)
        dist.barrier()
        mm = np.memmap(shm_path, dtype=np.float32, mode="r+", shape=(M, N))
        ch = torch.from_numpy(mm)
        pinned = torch.cuda.cudart().cudaHostRegister(ch.data_ptr(), M * N * 4, 0)
        pinned_ok = int(pinned) == 0 if not isinstance(pinned, tuple) else int(pinned[0]) == 0
        n0, n1 = pkg.tp.shard_range(N, world, rank)
        mine = ch[:, n0:n1]                                            # this rank's columns: row pitch N, as ldc

        def e2e_step(i):
            ctx.linear_host(ws[i % sets], xh, M, mine, N)
        for i in range(3):
            e2e_step(i)
        dist.barrier()
        # the host matrix now holds every rank's columns of step 2: the same bits as the result assembled on the device
        step_scatter(2)
        ctx.synchronize()
        same = bool(torch.equal(torch.from_numpy(np.array(mm)), scatter.result(0).cpu())) if rank == 0 else True
        dist.barrier()
        t0 = time.perf_counter()
        for i in range(it):
            e2e_step(i)
        dist.barrier()
        t = torch.tensor([(time.perf_counter() - t0) / it], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
        e2e = {"value": ops / dt / 1e12, "unit": "TOPS", "h2d_bytes_per_step": M * K * 4 * world, "d2h_bytes_per_step": M * N * 4,
               "ms_per_step": dt * 1e3, "host_result_equals_device_result": same, "host_buffer_page_locked": pinned_ok,
               "path": "every rank: inkq_linear_host on its weight rows (activations up its own PCIe link, its columns of the result down "
                       "into one host matrix shared by all ranks); host clock, max over ranks"}
        if pinned_ok:
            torch.cuda.cudart().cudaHostUnregister(ch.data_ptr())
        del mine, ch, mm
        dist.barrier()
        if rank == 0:
            try:
                os.unlink(shm_path)
            except OSError:
                pass
    else:
        e2e = None
    line["e2e"] = e2e

    scal = None
    if world > 1 and scatter is not None and args.scaling:
        for h in ws:
            h.close()
        ws = []
        scatter.close()
        scatter = None
        del cg, Cs
        torch.cuda.empty_cache()
        try:
            scal = scaling_m8192(pkg, torch, dist, ctx, world, rank, pk)
        except Exception as e:
            scal = {"error": repr(e)[:300]}
    elif world == 1 and args.scaling and wl == "qgemm_pp322":
        try:
            scal = scaling_m8192(pkg, torch, None, ctx, 1, 0, pk)
        except Exception as e:
            scal = {"error": repr(e)[:300]}
    if scal is not None:
        line["scaling_m8192"] = scal
    if world > 1 and args.model:
        if scatter is not None:
            scatter.close()
            scatter = None
        for h in ws:
            h.close()
        ws = []
        torch.cuda.empty_cache()
        try:
            line["model"] = model_tp(pkg, torch, dist, ctx, world, rank)
        except Exception as e:
            line["model"] = {"error": repr(e)[:300]}

    if rank == 0:
        if world == 1 and wl in ("qgemm_pp322", "qgemv_sweep"):
            line["cpu_baseline"] = cpu_baseline_pp322(pkg, x_host, wt)
        if world == 1 and (wl == "qgemv_sweep" or args.gemv):
            for h in ws:
                h.close()
            ws = []
            line["gemv"] = gemv_sweep(pkg, torch, ctx, pk["hbm_gbs"])
            line["gemv"].append(lm_head_gemv(pkg, torch, ctx, pk))
            line["scheme_matrix"] = scheme_matrix(pkg, torch, ctx, pk)
        if world == 1 and args.model:
            try:
                line["model"] = model_pp_tg(pkg, torch, ctx)
                line["model"]["same_operators_as_the_sharded_runs"] = model_tp(pkg, torch, None, ctx, 1, 0)
            except Exception as e:   # the headline metric above stands on its own
                line["model"] = {"error": repr(e)[:300]}
        print(json.dumps(line), flush=True)
    if scatter is not None:
        scatter.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="qgemm_pp322", choices=["qgemm_pp322", "qgemv_sweep", "qgemm_m2048", "qgemm_m8192", "lmhead_m8192"])
    ap.add_argument("--min-seconds", type=float, default=1.0, help="repeat the K timed steps until the timed region lasts this long")
    ap.add_argument("--no-gemv", dest="gemv", action="store_false", help="skip the decode QGEMV sweep figures")
    ap.add_argument("--no-model", dest="model", action="store_false", help="skip the synthetic Qwen3-8B pp322/tg128 figures")
    ap.add_argument("--no-scaling", dest="scaling", action="store_false", help="skip the M=8192 QGEMM / lm_head figures of the scaling configuration")
    ap.add_argument("--case", nargs="+", default=None, help="run one small fixed case for a profiler capture and exit")
    args = ap.parse_args()
    if args.case:
        return run_case(args)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 1)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
