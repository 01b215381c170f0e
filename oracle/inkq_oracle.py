"""ctypes front-ends for the two CPU checkers.

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by
bench.py's CPU-baseline legs; never by the product package.

  Oracle     our scalar C restatement (oracle/inkq_oracle.c -> _build/libinkq_oracle.so)
  Reference  the reference project's own kernels compiled unmodified by
             oracle/Makefile (-> _ref/libinkref_<isa>.so); None when not built.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
QK = 32

# Reference tile structs (qwen3/include/qwen/QwenOperator.h:46-80) as NumPy dtypes.
Q8_FP16 = np.dtype([("s_low", "<u2"), ("s_high", "<u2"), ("ss_low", "<u2"), ("ss_high", "<u2"),
                    ("q_low", "i1", 32), ("q_high", "i1", 32)])
Q8_FP32 = np.dtype([("s_low", "<f4"), ("s_high", "<f4"), ("ss_low", "<f4"), ("ss_high", "<f4"),
                    ("q_low", "i1", 32), ("q_high", "i1", 32)])
Q4_FP16 = np.dtype([("s_low", "<u2", 8), ("s_high", "<u2", 8), ("min_low", "<u2", 8), ("min_high", "<u2", 8),
                    ("q_coupled", "u1", 256)])
Q4_FP32 = np.dtype([("s_low", "<f4", 8), ("s_high", "<f4", 8), ("min_low", "<f4", 8), ("min_high", "<f4", 8),
                    ("q_coupled", "u1", 256)])
assert (Q8_FP16.itemsize, Q8_FP32.itemsize, Q4_FP16.itemsize, Q4_FP32.itemsize) == (72, 80, 320, 384)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dtype):
    a = np.ascontiguousarray(a, dtype=dtype)
    return a


def build(which: str = "oracle") -> None:
    subprocess.run(["make", "-C", HERE, which], check=True, stdout=subprocess.DEVNULL)


class Oracle:
    """Scalar restatement.  Scheme ids: 0 A81W41, 1 A80W40, 2 A80W4z."""

    def __init__(self):
        so = os.path.join(HERE, "_build", "libinkq_oracle.so")
        src = os.path.join(HERE, "inkq_oracle.c")
        if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
            build("oracle")
        self.lib = C.CDLL(so)
        self.lib.ink_f32_to_f16.restype = C.c_uint16
        self.lib.ink_f32_to_f16.argtypes = [C.c_float]
        self.lib.ink_f16_to_f32.restype = C.c_float
        self.lib.ink_f16_to_f32.argtypes = [C.c_uint16]

    # --- quantizer -------------------------------------------------------
    def quantize(self, x: np.ndarray, mode: int):
        """mode 0 Q8_0/fp16, 1 Q8_1/fp16, 2 Q8_1/fp32 -> (q s8 [M][K], d f32 [M][K/32], s f32 [M][K/32])."""
        x = _c(x, np.float32)
        M, K = x.shape
        q = np.empty((M, K), np.int8)
        d = np.empty((M, K // QK), np.float32)
        s = np.empty((M, K // QK), np.float32)
        self.lib.ink_quantize_q8(_ptr(x), C.c_int64(M * K), C.c_int(mode), _ptr(q), _ptr(d), _ptr(s))
        return q, d, s

    def quantize_struct(self, x: np.ndarray, mode: int, prefill: int = 0xCD) -> np.ndarray:
        """The reference's entry points, reference byte layout (one flat struct array)."""
        x = _c(x, np.float32).reshape(-1)
        dt = Q8_FP32 if mode == 2 else Q8_FP16
        out = np.full(x.size // 64 * dt.itemsize, prefill, np.uint8)
        fn = [self.lib.ink_quantize_row_q8_0_repack, self.lib.ink_quantize_row_q8_1_repack_fp16,
              self.lib.ink_quantize_row_q8_1_repack_fp32][mode]
        fn(_ptr(x), _ptr(out), C.c_int64(x.size))
        return out.view(dt)

    # --- re-tilers ---------------------------------------------------------
    def repack(self, nib, d, m, variant: int, prefill: int = 0xCD) -> np.ndarray:
        """variant 0 w80, 1 w81_fp16, 2 w81_fp32 -> reference superblock array."""
        nib, d = _c(nib, np.uint8), _c(d, np.float32)
        N, K = nib.shape[0], nib.shape[1] * 2
        dt = Q4_FP32 if variant == 2 else Q4_FP16
        out = np.full((N // 8) * (K // 64) * dt.itemsize, prefill, np.uint8)
        if variant == 0:
            self.lib.ink_repack_w80_weight(K, N, _ptr(out), _ptr(d), _ptr(nib))
        else:
            m = _c(m, np.float32)
            fn = self.lib.ink_repack_w81_weight_fp16 if variant == 1 else self.lib.ink_repack_w81_weight_fp32
            fn(K, N, _ptr(out), _ptr(d), _ptr(m), _ptr(nib))
        return out.view(dt)

    # --- matmuls -----------------------------------------------------------
    def gemm(self, scheme, q_a, d_a, s_a, nib, d_w, m_w=None, zp=None, want_dots=False, n0=0, n1=None):
        q_a, d_a = _c(q_a, np.int8), _c(d_a, np.float32)
        s_a = None if s_a is None else _c(s_a, np.float32)
        nib, d_w = _c(nib, np.uint8), _c(d_w, np.float32)
        m_w = None if m_w is None else _c(m_w, np.float32)
        zp = None if zp is None else _c(zp, np.uint8)
        M, K = q_a.shape
        N = nib.shape[0]
        n1 = N if n1 is None else n1
        Cm = np.zeros((M, N), np.float32)
        dots = np.zeros((M, N, K // QK), np.int32) if want_dots else None
        self.lib.ink_gemm_a8w4(scheme, M, N, K, _ptr(q_a), _ptr(d_a), _ptr(s_a), _ptr(nib), _ptr(d_w),
                               _ptr(m_w), _ptr(zp), _ptr(Cm), N, _ptr(dots), n0, n1)
        return (Cm, dots) if want_dots else Cm

    def gemm_samples(self, scheme, q_a, d_a, s_a, nib, d_w, m_w, zp, rows, cols):
        q_a, d_a = _c(q_a, np.int8), _c(d_a, np.float32)
        s_a = None if s_a is None else _c(s_a, np.float32)
        nib, d_w = _c(nib, np.uint8), _c(d_w, np.float32)
        m_w = None if m_w is None else _c(m_w, np.float32)
        zp = None if zp is None else _c(zp, np.uint8)
        rows, cols = _c(rows, np.int32), _c(cols, np.int32)
        K = q_a.shape[1]
        out = np.zeros(rows.size, np.float32)
        self.lib.ink_gemm_a8w4_samples(scheme, nib.shape[0], K, _ptr(q_a), _ptr(d_a), _ptr(s_a), _ptr(nib),
                                       _ptr(d_w), _ptr(m_w), _ptr(zp), _ptr(rows), _ptr(cols),
                                       int(rows.size), _ptr(out))
        return out

    def gemm_w41_f16act(self, a16, nib, d_w, m_w):
        a16 = _c(a16, np.float16)
        nib, d_w, m_w = _c(nib, np.uint8), _c(d_w, np.float32), _c(m_w, np.float32)
        M, K = a16.shape
        N = nib.shape[0]
        Cm = np.zeros((M, N), np.float32)
        self.lib.ink_gemm_w41_f16act(M, N, K, _ptr(a16), _ptr(nib), _ptr(d_w), _ptr(m_w), _ptr(Cm), N)
        return Cm

    def lmhead_f16w(self, x, w16, n0=0, n1=None):
        x, w16 = _c(x, np.float32), _c(w16, np.float16)
        M, K = x.shape
        N = w16.shape[0]
        n1 = N if n1 is None else n1
        Cm = np.zeros((M, N), np.float32)
        self.lib.ink_lmhead_f16w(M, N, K, _ptr(x), _ptr(w16), _ptr(Cm), N, n0, n1)
        return Cm

    def quantize_weight(self, which: int, w: np.ndarray):
        """which 0: Q4_0, 1: Q4_1 -> (nib, d, m) in the disk layout."""
        w = _c(w, np.float32)
        N, K = w.shape
        nib = np.zeros((N, K // 2), np.uint8)
        d = np.empty((N, K // QK), np.float32)
        m = np.empty((N, K // QK), np.float32)
        self.lib.ink_quantize_weight_q4(which, N, K, _ptr(w), _ptr(nib), _ptr(d), _ptr(m))
        return nib, d, m

    def f16_round(self, a: np.ndarray) -> np.ndarray:
        flat = np.ascontiguousarray(a, np.float32).reshape(-1)
        out = np.array([self.lib.ink_f16_to_f32(self.lib.ink_f32_to_f16(float(v))) for v in flat], np.float32)
        return out.reshape(np.shape(a))


def _cpu_flags() -> set:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


class Reference:
    """The reference's own compiled kernels (C++ symbols, called by mangled name)."""

    SYMS = {
        "quantize_row_q8_0_repack": "_Z24quantize_row_q8_0_repackPKfPvl",
        "quantize_row_q8_1_repack_fp16": "_Z29quantize_row_q8_1_repack_fp16PKfPvl",
        "quantize_row_q8_1_repack_fp32": "_Z29quantize_row_q8_1_repack_fp32PKfPvl",
        "repack_w80_weight": "_Z17repack_w80_weightiiiPvPKfPKh",
        "repack_w81_weight_fp16": "_Z22repack_w81_weight_fp16iiiPvPKfS1_PKh",
        "repack_w81_weight_fp32": "_Z22repack_w81_weight_fp32iiiPvPKfS1_PKh",
        "gemm_repack_A80W40": "_Z18gemm_repack_A80W40PvS_Pfiii",
        "gemv_repack_A80W40": "_Z18gemv_repack_A80W40PvS_Pfiii",
        "gemm_repack_A81W41_fp32": "_Z23gemm_repack_A81W41_fp32PvS_Pfiii",
        "gemv_repack_A81W41_fp16": "_Z23gemv_repack_A81W41_fp16PvS_Pfiii",
    }
    NEED_VNNI = {"avx512f", "avx512vl", "avx512bw", "avx512dq", "avx512_vnni", "avx2", "fma", "f16c", "bmi2"}
    NEED_AVX2 = {"avx2", "fma", "f16c", "bmi2"}

    @staticmethod
    def available_path():
        flags = _cpu_flags()
        for isa, need in (("vnni", Reference.NEED_VNNI), ("avx2", Reference.NEED_AVX2)):
            p = os.path.join(HERE, "_ref", f"libinkref_{isa}.so")
            if os.path.exists(p) and need <= flags:
                return p, isa
        return None, None

    def __init__(self, path=None):
        """path: any shared library exporting the reference's function names (e.g. the
        GPU-backed drop-in built from qwen3.ink.cpp_b200/host/ref_names.cc); default: oracle/_ref."""
        if path is not None:
            p, isa = path, "custom"
        else:
            p, isa = self.available_path()
        if p is None:
            raise FileNotFoundError("oracle/_ref/libinkref_*.so not built (run `make -C oracle ref` where the "
                                    "reference checkout is present) or host ISA unsupported")
        self.isa = isa
        self.lib = C.CDLL(p)
        self.fn = {k: getattr(self.lib, v) for k, v in self.SYMS.items()}
        for f in self.fn.values():
            f.restype = None

    def quantize_struct(self, x, mode: int, prefill: int = 0xCD, pad_rows: int = 0) -> np.ndarray:
        x = _c(x, np.float32).reshape(-1)
        dt = Q8_FP32 if mode == 2 else Q8_FP16
        out = np.full((x.size // 64 + pad_rows) * dt.itemsize, prefill, np.uint8)
        name = ["quantize_row_q8_0_repack", "quantize_row_q8_1_repack_fp16", "quantize_row_q8_1_repack_fp32"][mode]
        self.fn[name](_ptr(x), _ptr(out), C.c_int64(x.size))
        return out.view(dt)

    def repack(self, nib, d, m, variant: int, prefill: int = 0xCD) -> np.ndarray:
        nib, d = _c(nib, np.uint8), _c(d, np.float32)
        N, K = nib.shape[0], nib.shape[1] * 2
        dt = Q4_FP32 if variant == 2 else Q4_FP16
        out = np.full((N // 8) * (K // 64) * dt.itemsize, prefill, np.uint8)
        if variant == 0:
            self.fn["repack_w80_weight"](K, N, 32, _ptr(out), _ptr(d), _ptr(nib))
        else:
            m = _c(m, np.float32)
            name = "repack_w81_weight_fp16" if variant == 1 else "repack_w81_weight_fp32"
            self.fn[name](K, N, 32, _ptr(out), _ptr(d), _ptr(m), _ptr(nib))
        return out.view(dt)

    # ---- the reference's operators around the linear layer (oracle/ref_ops_driver.cc)
    def _op(self, name):
        fn = getattr(self.lib, name)
        fn.restype = None
        return fn

    def rmsnorm(self, x, w, eps: float = 1e-6) -> np.ndarray:
        """Qwen3RMSNorm::forward over the last axis of x [rows][heads][dim] (or [rows][dim])."""
        x, w = _c(x, np.float32), _c(w, np.float32)
        shape = x.shape
        x3 = x.reshape(shape[0], -1, shape[-1])
        out = np.empty_like(x3)
        self._op("refop_rmsnorm")(_ptr(x3), _ptr(w), x3.shape[0], x3.shape[1], x3.shape[2], C.c_float(eps), _ptr(out))
        return out.reshape(shape)

    def silu_mul(self, a, b) -> np.ndarray:
        a, b = _c(a, np.float32), _c(b, np.float32)
        out = np.empty_like(a)
        self._op("refop_silu_mul")(_ptr(a), _ptr(b), a.shape[0], a.shape[1], _ptr(out))
        return out

    def add(self, a, b) -> np.ndarray:
        a, b = _c(a, np.float32), _c(b, np.float32)
        out = np.empty_like(a)
        self._op("refop_add")(_ptr(a), _ptr(b), a.shape[0], a.shape[1], _ptr(out))
        return out

    def rope(self, q, k, start: int, cos, sin):
        """RotaryPosEmb::apply on q [nq][len][hd], k [nk][len][hd]; returns the rotated copies."""
        q, k = _c(q, np.float32).copy(), _c(k, np.float32).copy()
        cos, sin = _c(cos, np.float32), _c(sin, np.float32)
        self._op("refop_rope")(_ptr(q), _ptr(k), q.shape[0], k.shape[0], q.shape[1], q.shape[2], start, _ptr(cos), _ptr(sin), cos.shape[0])
        return q, k

    def attention(self, q, k_cache, v_cache, past: int, alpha: float) -> np.ndarray:
        """The attention core of Qwen3Attention::forward: q [nq][sq][hd], caches [nkv][max_len][hd] (fp32) holding
        past + sq positions; returns [sq][nq * hd]."""
        q, k_cache, v_cache = _c(q, np.float32), _c(k_cache, np.float32), _c(v_cache, np.float32)
        nq, sq, hd = q.shape
        out = np.empty((sq, nq * hd), np.float32)
        self._op("refop_attention")(_ptr(q), _ptr(k_cache), _ptr(v_cache), nq, k_cache.shape[0], sq, past, hd, k_cache.shape[1], C.c_float(alpha),
                                    _ptr(out))
        return out

    def matmul(self, name: str, A: np.ndarray, B: np.ndarray, M: int, N: int, K: int) -> np.ndarray:
        """name in {gemm,gemv}_repack_*.  A must carry readable padding rows: the
        reference GEMMs read up to 5 (A81W41) or 1 (A80W40) activation rows past M
        (quantized_gemx_kernels.cc:371-375, :215-221)."""
        Cm = np.zeros((M, N), np.float32)
        self.fn[name](_ptr(A), _ptr(B), _ptr(Cm), M, N, K)
        return Cm
