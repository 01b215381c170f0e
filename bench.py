#!/usr/bin/env python
"""Benchmark of the A8W4 quantized-matmul path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One JSON line on stdout (rank 0).  A "step" is one forward of the quantized linear
layer (activation quantizer + QGEMM) on synthetic inputs of the prefill gate_proj
shape: M=322 activations x K=4096, N=12288 A81W41 weights (fp32 block scales).
  value   whole-job int8 TOPS (2*M*N*K per step) with inputs resident in HBM
  e2e     the same metric through the host-buffer entry point (inkq_linear_host):
          pinned host activations in, host result out, copies inside the timed region
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
qgemm_m2048, qgemm_m8192.
"""
from __future__ import annotations

import argparse
import json
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
    cores = os.cpu_count() or 1
    kind = "reference" if Reference.available_path()[0] else "port"
    isa = "scalar"
    if kind == "reference":
        ref = Reference()
        isa = ref.isa
        B = ref.repack(w["nib"], w["d"], w["m"], 2)

        def step():
            A = ref.quantize_struct(x, 2, pad_rows=6 * K // 64, prefill=0)     # quantize_row_q8_1_repack_fp32
            return ref.matmul("gemm_repack_A81W41_fp32", A, B, M, N, K)       # gemm_repack_A81W41_fp32
        sample = f"full workload: quantize_row_q8_1_repack_fp32 + gemm_repack_A81W41_fp32 at {M}x{N}x{K}, all {cores} host threads"
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
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    tops = ops / dt / 1e12
    line = {"impl": "reference", "metric": "qgemm_int8_tops_pp322", "value": tops, "unit": "TOPS", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3 * (2.0 * M * N * K / ops), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "s8 x u4 -> s32, fp32 scale/accumulate", "data": "synthetic",
            "config": {"workload": "qgemm_pp322", "M": M, "N": N, "K": K, "scheme": "A81W41", "isa": isa},
            "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- CPU baseline leg of our arm
def cpu_baseline_pp322(pkg, x, w):
    from oracle.inkq_oracle import Oracle, Reference
    M, K, N = M_PP, K_PP, N_PP
    cores = os.cpu_count() or 1
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
    model.decode_step()
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
    # the same decode step with every operator as its own launch (17 per layer), for comparison
    unfused_ms = None
    launches_per_token = {"epilogue": 5 * cfg.layers + 4, "prologue": 6 * cfg.layers + 4, "separate": 17 * cfg.layers + 4}[cfg.decode_mode]
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
    scatter, exchange = None, "single GPU"
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

    # clocks are sampled from the warm-up on: the timed region itself lasts only a few milliseconds, less than the
    # sampling period of nvidia-smi, and the warm-up steps put the same load on the GPU
    sampler = ClockSampler(local_rank)
    sampler.start()
    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    graph = None
    if scatter is not None:
        # A sharded step is short (tens of microseconds of GPU work) and one Python process per GPU cannot enqueue
        # its three launches that fast: the K timed steps are captured once as a CUDA graph and replayed.  The
        # barrier kernel keeps its count in device memory, so a replay is a valid sequence of K more barriers.
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            ctx.set_stream(side.cuda_stream)
            with torch.cuda.graph(graph, stream=side):
                for i in range(args.steps):
                    step(i)
        ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        torch.cuda.current_stream().wait_stream(side)
        graph.replay()                       # untimed: every rank runs the same K steps
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    l0 = ctx.launches
    torch.cuda.synchronize()
    if graph is not None:
        ms = cuda_time_ms(torch, lambda i: graph.replay(), 1)
        launches = 3 * args.steps            # quantizer, QGEMM, barrier kernel per step, replayed from the graph
    else:
        ms = cuda_time_ms(torch, step, args.steps)
        launches = ctx.launches - l0
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    ctx.synchronize()
    clocks = sampler.stop()
    ops = 2.0 * M * N * K
    tops = ops * args.steps / (ms * 1e-3) / 1e12
    gather_tops = None
    if scatter is not None:          # the library-collective variant of the same step, for comparison
        for i in range(args.warmup):
            step_gather(i)
        torch.cuda.synchronize()
        dist.barrier()
        ms2 = cuda_time_ms(torch, step_gather, args.steps)
        t = torch.tensor([ms2], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        gather_tops = ops * args.steps / (float(t.item()) * 1e-3) / 1e12
        dist.barrier()
        ctx.synchronize()

    line = {"metric": "qgemm_int8_tops_pp322" if wl in ("qgemm_pp322", "qgemv_sweep") else f"qgemm_int8_tops_{wl.split('_')[1]}",
            "value": tops, "unit": "TOPS", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "s8 x u4 -> s32 block dots (tcgen05 kind::i8), fp32 scale/accumulate", "data": "synthetic",
            "config": {"workload": wl if wl != "qgemv_sweep" else "qgemm_pp322", "M": M, "N": N, "K": K, "scheme": "A81W41",
                       "weight_scales": "fp32", "parallelism": exchange,
                       "l2": f"{sets} distinct weight sets ({sets * w_bytes_one / 1e6:.0f} MB per rank) rotated between steps, > 126 MB L2"},
            "clocks": clocks, "gpu_launches": int(launches)}
    if gather_tops is not None:
        line["config"]["same_step_with_nccl_all_gather_tops"] = gather_tops

    if rank == 0:
        # ---- kernel-only figures for the roofline (dominant kernel: the tensor-core QGEMM) ----
        act = ctx.act(M, K)
        ctx.quantize(act, xs[0], M, pkg.Q8_1_F32)
        Ck = Cs[0]
        for i in range(3):
            ctx.gemm(act, ws[i % sets], Ck, n_loc)
        torch.cuda.synchronize()
        it = max(10, args.steps)
        ms_g = cuda_time_ms(torch, lambda i: ctx.gemm(act, ws[i % sets], Ck, n_loc), it) / it
        ms_q = cuda_time_ms(torch, lambda i: ctx.quantize(act, xs[i % sets], M, pkg.Q8_1_F32), it) / it
        ach = 2.0 * M * n_loc * K / (ms_g * 1e-3) / 1e12
        int8_peak = 2.0 * pk["bf16_tflops"]
        line["roofline"] = {"bound": "tensor", "achieved": ach, "peak": int8_peak, "unit": "TOP/s", "frac": ach / int8_peak,
                            "traffic": 41.12e6 if (wl in ("qgemm_pp322", "qgemv_sweep") and world == 1) else None,
                            "traffic_note": "dram__bytes_read.sum + dram__bytes_write.sum of one launch at this shape (ncu capture summarised under "
                                            "profiles/): 41.01 MB read = the compulsory operand bytes, 0.11 MB written (the 15.8 MB result stays in L2)",
                            "kernel": "k_qgemm_tc", "us_per_launch": ms_g * 1e3,
                            "peak_note": f"2 x the {pk['source']} dense bf16 figure ({pk['bf16_tflops']} TFLOP/s); int8 itself is not in MEASURED_PEAKS.json",
                            "cuda_core_note": "every K=32 MMA is followed by an fp32 scale+accumulate of its whole tile on the CUDA cores "
                                              "(M*N*K/32 block dots per launch); that, not the tensor pipe, bounds this kernel"}
        # the second roof of this kernel: the per-block fp32 epilogue on the CUDA cores.  Per block dot and lane the exact
        # arithmetic needs one int->float conversion, half a packed multiply (d_a*d_w), one packed fma pair (main and min
        # terms) and half a shared load: 3 issue slots per warp-level block dot.
        tiles_m = -(-M // 128)
        bm = -(-(-(-M // tiles_m)) // 16) * 16
        dots = float(tiles_m * bm) * n_loc * (K // 32)
        sm_clock = (clocks.get("sm_mhz") or 1965.0) * 1e6
        n_sms = torch.cuda.get_device_properties(local_rank).multi_processor_count
        t_min = dots * 3.0 / 32.0 / (n_sms * 4) / sm_clock
        line["roofline"]["cuda_core_roof"] = {"block_dots_per_launch": dots, "issue_slots_per_warp_block_dot": 3.0,
                                              "min_us": t_min * 1e6, "frac": t_min / (ms_g * 1e-3)}
        line["quantizer"] = {"us_per_launch": ms_q * 1e3, "GBs": M * K * 5.375 / (ms_q * 1e-3) / 1e9, "frac_of_hbm": M * K * 5.375 / (ms_q * 1e-3) / 1e9 / pk["hbm_gbs"]}
        act.close()

        # ---- end to end through the host-buffer entry point ----
        if world == 1:
            xh = torch.from_numpy(x_host).pin_memory()
            ch = torch.empty((M, N), dtype=torch.float32).pin_memory()
            for i in range(3):
                ctx.linear_host(ws[i % sets], xh, M, ch, N)
            it = max(10, args.steps)
            t0 = time.perf_counter()
            for i in range(it):
                ctx.linear_host(ws[i % sets], xh, M, ch, N)
            dt = (time.perf_counter() - t0) / it
            line["e2e"] = {"value": ops / dt / 1e12, "unit": "TOPS", "h2d_bytes_per_step": M * K * 4, "d2h_bytes_per_step": M * N * 4,
                           "ms_per_step": dt * 1e3}
        else:
            line["e2e"] = {"value": None, "unit": "TOPS", "h2d_bytes_per_step": M * K * 4, "d2h_bytes_per_step": M * N * 4,
                           "note": "measured at N=1 only"}
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
    ap.add_argument("--workload", default="qgemm_pp322", choices=["qgemm_pp322", "qgemv_sweep", "qgemm_m2048", "qgemm_m8192"])
    ap.add_argument("--no-gemv", dest="gemv", action="store_false", help="skip the decode QGEMV sweep figures")
    ap.add_argument("--no-model", dest="model", action="store_false", help="skip the synthetic Qwen3-8B pp322/tg128 figures")
    args = ap.parse_args()
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
