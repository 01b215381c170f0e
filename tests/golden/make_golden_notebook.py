"""Generates tests/golden/ref_notebook_schemes.npz by RUNNING the reference's own notebook code for the two
schemes that have no C++ kernel in the reference:

  A80W4Z  notebooks/evaluate-qwen3_8b_A8W4.ipynb, the cell that defines `QuantizedLinear` and
          `pseudo_quantize_tensor_q4_zero_point` (Q8_0 fake-quantized activations x zero-point int4 weights)
  W41     notebooks/evaluate-qwen3_8b_W4.ipynb, the cell that defines `pseudo_quantize_tensor_q41` and overwrites
          `m.weight.data` of an fp16 model with the dequantised tensor (stock fp16 F.linear follows)

The cells' source is taken out of the .ipynb JSON and exec'd unchanged; nothing of it is copied into this
repository.  Run where a checkout of the reference exists:

    python tests/golden/make_golden_notebook.py /path/to/Qwen3.Ink.Cpp

The notebook functions return only the dequantised weights.  The integer codes, scales and zero points that this
library's entry points take are recovered beside them with the same one-line formulas and then VERIFIED against
the notebook's output bits (`(q - zp) * s == w_f`, `q * s + min == w_f`) before anything is stored, so the
fixture's packed weights are exactly what the notebook's tensors encode.
"""
import json
import os
import sys

import numpy as np
import torch
import torch.nn as nn


def cell_defining(nb_path, *names):
    nb = json.load(open(nb_path))
    for c in nb["cells"]:
        if c["cell_type"] != "code":
            continue
        src = "".join(c["source"])
        if all(("def " + n in src) or ("class " + n in src) for n in names):
            return src
    raise SystemExit(f"no cell of {nb_path} defines {names}")


def pack_nibbles(q):
    """AWQ interleave of the on-disk format: byte[32g+e] = q[64g+e] | q[64g+32+e] << 4."""
    N, K = q.shape
    g = q.reshape(N, K // 64, 2, 32)
    return (g[:, :, 0, :] | (g[:, :, 1, :] << 4)).reshape(N, K // 2).astype(np.uint8)


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden_notebook.py /path/to/Qwen3.Ink.Cpp")
    ref = sys.argv[1]
    torch.manual_seed(0)
    rng = np.random.default_rng(4242)
    N, K, M = 72, 256, 9
    out = {}

    # ---------------- A80W4Z: the A8W4 notebook ----------------
    ns = {"torch": torch, "nn": nn}
    exec(cell_defining(os.path.join(ref, "notebooks", "evaluate-qwen3_8b_A8W4.ipynb"), "QuantizedLinear",
                       "pseudo_quantize_tensor_q4_zero_point"), ns)
    w = (rng.standard_normal((N, K)) * 0.04 + 0.01).astype(np.float32)
    w[0, :32] = 0.0                       # constant block: the scale is clamped to 1e-5 / 15
    w[1, 32:64] = np.abs(w[1, 32:64])     # all positive: zero point 0
    w[2, 64:96] = -np.abs(w[2, 64:96])    # all negative: zero point 15
    x = rng.standard_normal((M, K)).astype(np.float32)
    x[3, :32] = 0.0                       # an all-zero activation block
    wt, xt = torch.from_numpy(w), torch.from_numpy(x)
    w_f = ns["pseudo_quantize_tensor_q4_zero_point"](wt.clone(), 4, 32)
    layer = ns["QuantizedLinear"](w_f, None, 8, 4)
    y = layer.forward(xt.clone())
    # recover (q, zp, s) and verify them against the notebook's dequantised weights, bit for bit
    wb = wt.reshape(-1, 32)
    s = (wb.amax(-1, keepdim=True) - wb.amin(-1, keepdim=True)).clamp(min=1e-5) / 15
    zp = (-torch.round(wb.amin(-1, keepdim=True) / s)).clamp(0, 15)
    q = (torch.round(wb / s) + zp).clamp(0, 15)
    assert torch.equal(((q - zp) * s).reshape(N, K), w_f), "recovered codes do not reproduce the notebook's weights"
    # recover the activation codes and verify them through the notebook's own output
    xb = xt.reshape(-1, 32)
    xs = xb.abs().amax(-1, keepdim=True) / 127
    xr = 1 / xs
    xr[xs == 0] = 0
    xq = (xb * xr).round()
    assert torch.equal(torch.nn.functional.linear((xq * xs).reshape(M, K), w_f), y), "recovered activation codes do not reproduce the notebook's output"
    out.update(w4z_w=w, w4z_x=x, w4z_y=y.numpy(), w4z_wf=w_f.numpy(),
               w4z_nib=pack_nibbles(q.reshape(N, K).numpy().astype(np.uint8)), w4z_d=s.reshape(N, K // 32).numpy(),
               w4z_zp=zp.reshape(N, K // 32).numpy().astype(np.uint8),
               w4z_xq=xq.reshape(M, K).numpy().astype(np.int8), w4z_xd=xs.reshape(M, K // 32).numpy())

    # ---------------- W41: the weight-only notebook (fp16 model) ----------------
    ns2 = {"torch": torch, "nn": nn}
    exec(cell_defining(os.path.join(ref, "notebooks", "evaluate-qwen3_8b_W4.ipynb"), "pseudo_quantize_tensor_q41",
                       "pseudo_quantize_model_weight"), ns2)
    w16 = torch.from_numpy((rng.standard_normal((N, K)) * 0.04 + 0.01).astype(np.float16))
    x16 = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float16))
    lin = nn.Linear(K, N, bias=False).half()
    lin.weight.data = w16.clone()
    ns2["pseudo_quantize_model_weight"](lin, 4, 32, "q41")        # the notebook's own loop over nn.Linear modules
    wf16 = lin.weight.data
    y16 = lin(x16)                                                # stock fp16 F.linear
    wb = w16.reshape(-1, 32)
    mn = wb.amin(-1, keepdim=True)
    s16 = (wb.amax(-1, keepdim=True) - mn).clamp(min=1e-5) / 15
    q16 = torch.round((wb - mn) / s16).clamp(0, 15)
    assert torch.equal((q16 * s16 + mn).reshape(N, K), wf16), "recovered codes do not reproduce the notebook's fp16 weights"
    out.update(w41_x=x16.numpy(), w41_y=y16.detach().numpy(), w41_wf=wf16.numpy(),
               w41_nib=pack_nibbles(q16.reshape(N, K).numpy().astype(np.uint8)),
               w41_d=s16.reshape(N, K // 32).float().numpy(), w41_m=mn.reshape(N, K // 32).float().numpy())

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_notebook_schemes.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
