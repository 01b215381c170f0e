"""Runs one small, fixed case of a kernel a few times so that it can be captured under ncu.

    python qwen3.ink.cpp_b200/profile_case.py qgemm [M]       # k_qgemm_tc, N=12288, K=4096 (default M=322)
    python qwen3.ink.cpp_b200/profile_case.py qgemv [N] [K]   # k_qgemv_a8w4 (default 12288 x 4096), 12 distinct weight sets
    python qwen3.ink.cpp_b200/profile_case.py quantize [M]    # k_quantize_q8, K=4096 (default M=8192)
    python qwen3.ink.cpp_b200/profile_case.py model [layers]  # synthetic Qwen3-8B-shaped forward with few layers (default 2): prefill of 322
                                                              # tokens, then 3 decode steps (launch list of the glue around the linears)
    python qwen3.ink.cpp_b200/profile_case.py w41 [M]         # k_gemm_w41_tc, N=12288, K=4096 (default M=2048); prints its time

Typical capture (one kernel, one launch, after the same command has exited 0 without ncu):
    ncu --set full --clock-control none -k regex:k_qgemm_tc -s 1 -c 1 -o prof python qwen3.ink.cpp_b200/profile_case.py qgemm
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from __graft_entry__ import load_package  # noqa: E402


def main():
    pkg = load_package()
    what = sys.argv[1] if len(sys.argv) > 1 else "qgemm"
    args = [int(a) for a in sys.argv[2:]]
    torch.cuda.set_device(0)
    ctx = pkg.Context(0, torch.cuda.current_stream().cuda_stream)
    if what == "qgemm":
        M, N, K = (args + [322])[0], 12288, 4096
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
        N, K = (args + [12288, 4096])[:2]
        w = pkg.synth.weights(N, K)
        whs = [ctx.weight(pkg.A81W41, pkg.SCALES_F16, w["nib"], w["d"], w["m"]) for _ in range(12)]
        x = torch.from_numpy(pkg.synth.activations(1, K)).cuda()
        C = torch.empty((1, N), device="cuda")
        act = ctx.act(1, K)
        ctx.quantize(act, x, 1, pkg.Q8_1_F16)
        for wh in whs:
            ctx.gemv(act, wh, C)
        ctx.synchronize()
        print("qgemv ok", N, K, float(C.abs().mean()))
    elif what == "quantize":
        M, K = (args + [8192])[0], 4096
        x = torch.randn((M, K), device="cuda")
        act = ctx.act(M, K)
        for _ in range(3):
            ctx.quantize(act, x, M, pkg.Q8_1_F32)
        ctx.synchronize()
        print("quantize ok", M, K)
    elif what == "model":
        layers = (args + [2])[0]
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
        M, N, K = (args + [2048])[0], 12288, 4096
        w = pkg.synth.weights(N, K)
        wh = ctx.weight(pkg.W41, pkg.SCALES_F16, w["nib"], w["d"], w["m"])
        a16 = torch.from_numpy(pkg.synth.activations(M, K)).cuda().half()
        C = torch.empty((M, N), device="cuda")
        for _ in range(3):
            ctx.gemm_w41_f16act(a16, M, wh, C, N)
        ctx.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(10):
            ctx.gemm_w41_f16act(a16, M, wh, C, N)
        b.record()
        ctx.synchronize()
        us = a.elapsed_time(b) * 100
        print(f"w41 ok {M} {N} {K} mean|C| {float(C.abs().mean()):.4f}  {us:.1f} us per launch, {2.0 * M * N * K / us / 1e6:.1f} TFLOP/s")
    else:
        raise SystemExit("unknown case " + what)


if __name__ == "__main__":
    main()
