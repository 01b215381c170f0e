"""GPU: the offline weight quantizers (csrc/weight_quant.cu) against the fixture made from the reference's Python code
and against the oracle, and the on-disk format round trip: quantize on the GPU -> four files -> load -> re-tile ->
the layer computes what the oracle computes from the same files."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt,name", [(0, "q40"), (1, "q41")])
def test_gpu_weight_quantizer_equals_python_reference(pkg, gpu, golden, fmt, name):
    import torch
    g = golden("ref_weightquant.npz")
    nib, d, m, zp = gpu.quantize_weights(fmt, torch.from_numpy(g["w"]).cuda())
    gpu.synchronize()
    assert np.array_equal(nib.cpu().numpy(), g[name + "_nib"])
    assert np.array_equal(d.cpu().numpy().view(np.uint32), g[name + "_d"].view(np.uint32))
    assert np.array_equal(m.cpu().numpy().view(np.uint32), g[name + "_m"].view(np.uint32))
    assert np.array_equal(zp.cpu().numpy(), g[name + "_zp"])


@pytest.mark.parametrize("fmt", [0, 1])
def test_gpu_weight_quantizer_equals_oracle_on_a_layer(pkg, gpu, oracle, fmt):
    import torch
    w = (np.random.default_rng(5).standard_normal((264, 1024)) * 0.03).astype(np.float32)
    nib, d, m, _ = gpu.quantize_weights(fmt, torch.from_numpy(w).cuda())
    gpu.synchronize()
    rn, rd, rm = oracle.quantize_weight(fmt, w)
    assert np.array_equal(nib.cpu().numpy(), rn) and np.array_equal(d.cpu().numpy(), rd) and np.array_equal(m.cpu().numpy(), rm)


def test_disk_format_round_trip(pkg, gpu, oracle, tmp_path):
    import torch
    N, K, M = 136, 512, 9
    w = (np.random.default_rng(6).standard_normal((N, K)) * 0.03).astype(np.float32)
    nib, d, m, zp = (t.cpu().numpy() for t in gpu.quantize_weights(1, torch.from_numpy(w).cuda()))
    prefix = str(tmp_path / "layers" / "0" / "q_proj") + "/"
    pkg.disk_format.save_linear(prefix, nib, d, m, zp)
    back = pkg.disk_format.load_linear(prefix, N, K)
    assert all(np.array_equal(back[k], v) for k, v in (("nib", nib), ("d", d), ("m", m), ("zp", zp)))
    wh = pkg.disk_format.weight_from_disk(gpu, pkg, prefix, N, K)
    assert wh.scheme == pkg.A81W41
    x = pkg.synth.activations(M, K, 9)
    C = torch.empty((M, N), device="cuda")
    gpu.linear(wh, torch.from_numpy(x).cuda(), M, C, N)
    gpu.synchronize()
    q, da, sa = oracle.quantize(x, 2)
    ref = oracle.gemm(0, q, da, sa, nib, d, m)
    assert np.array_equal(C.cpu().numpy().view(np.uint32), ref.view(np.uint32))
    with pytest.raises(ValueError):
        pkg.disk_format.load_linear(prefix, N + 1, K)       # short files
    with pytest.raises(FileNotFoundError):
        pkg.disk_format.load_linear(prefix + "missing/", N, K)
