"""CPU: the C-ABI library loads and exports every entry point include/inkq.h declares;
argument validation that needs no device."""
import ctypes
import os
import re

from conftest import ROOT


def declared_symbols(header="inkq.h"):
    src = open(os.path.join(ROOT, "include", header)).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(inkq_[a-z0-9_]+)\s*\(", src)))


def test_header_and_binding_agree(pkg):
    assert declared_symbols() == sorted(pkg.SYMBOLS)
    assert declared_symbols("inkq_glue.h") == sorted(pkg.GLUE_SYMBOLS)


def test_library_exports_every_declared_symbol(pkg):
    pkg.build()
    L = pkg.lib()
    for name in declared_symbols() + declared_symbols("inkq_glue.h"):
        assert hasattr(L, name), name


def test_context_creation_fails_loudly_without_a_device(pkg):
    import torch
    if torch.cuda.is_available():
        return
    pkg.build()
    L = pkg.lib()
    h = ctypes.c_void_p()
    rc = L.inkq_ctx_create(0, None, ctypes.byref(h))
    assert rc != 0 and not h.value
    assert b"CUDA" in L.inkq_last_error(None) or b"device" in L.inkq_last_error(None)


def test_null_handles_are_rejected(pkg):
    pkg.build()
    L = pkg.lib()
    assert L.inkq_ctx_create(0, None, None) == pkg.ERR_INVALID
    assert L.inkq_weight_info(None, None, None, None, None) == pkg.ERR_INVALID
    assert L.inkq_ctx_synchronize(None) == pkg.ERR_INVALID
    assert L.inkq_ctx_destroy(None) == pkg.OK
    assert L.inkq_launch_count(None) == 0


def test_synth_nibble_packing_round_trip(pkg):
    import numpy as np
    q = np.random.default_rng(1).integers(0, 16, (8, 256), dtype=np.uint8)
    nib = pkg.synth.pack_nibbles(q)
    assert nib.shape == (8, 128)
    # byte[32g+e] = q[64g+e] | q[64g+32+e] << 4  (notebooks/quantize_methods.py:120-123)
    assert nib[3, 32 + 5] == (q[3, 64 + 5] | (q[3, 64 + 32 + 5] << 4))
    assert np.array_equal(pkg.synth.unpack_nibbles(nib), q)


def test_reference_named_shim_exports_the_reference_symbols(pkg):
    """The GPU-backed drop-in exports the same (C++-mangled) names as the compiled reference."""
    import ctypes
    from oracle.inkq_oracle import Reference
    pkg.build()
    path = os.path.join(ROOT, "qwen3.ink.cpp_b200", "libinkq_refshim.so")
    assert os.path.exists(path)
    L = ctypes.CDLL(path)
    for mangled in Reference.SYMS.values():
        assert hasattr(L, mangled), mangled
