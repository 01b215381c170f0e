"""B200-native A8W4 quantized-matmul path of Qwen3.Ink.Cpp: Python driver side.

The product is the CUDA library (csrc/ -> libinkq.so) behind the C ABI declared in
include/inkq.h, plus the C++ host mirror of the reference's linear layer in host/.
This package is the thin ctypes binding tests and benchmarks drive it with.  It
never computes anything itself: if libinkq.so is missing or no B200 is present the
calls raise, there is no CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build
from . import synth  # noqa: F401  (re-exported)
from . import tp  # noqa: F401
from . import qwen3_forward  # noqa: F401
from . import disk_format  # noqa: F401

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libinkq.so")

# enums of include/inkq.h
A81W41, A80W40, A80W4Z, W41 = 0, 1, 2, 3
Q8_0_F16, Q8_1_F16, Q8_1_F32 = 0, 1, 2
SCALES_F32, SCALES_F16 = 0, 1
OK, ERR_INVALID, ERR_CUDA, ERR_ALLOC, ERR_UNSUPPORTED, ERR_TIMEOUT = range(6)

# every symbol include/inkq.h declares
SYMBOLS = [
    "inkq_ctx_create", "inkq_ctx_destroy", "inkq_ctx_set_stream", "inkq_ctx_synchronize", "inkq_last_error",
    "inkq_launch_count", "inkq_weight_create", "inkq_weight_create_dev", "inkq_weight_destroy", "inkq_weight_info",
    "inkq_weight_export", "inkq_act_create", "inkq_act_destroy", "inkq_quantize", "inkq_act_export", "inkq_act_import", "inkq_quantize_host", "inkq_gemm_host", "inkq_gemv_host", "inkq_gemm",
    "inkq_gemv", "inkq_gemm_simt", "inkq_debug_block_dots", "inkq_debug_block_dots_tc", "inkq_linear",
    "inkq_linear_host", "inkq_linear_m1_static", "inkq_gemm_w41_f16act", "inkq_gemm_w41_f16act_simt", "inkq_f16w_create", "inkq_f16w_create_dev", "inkq_f16w_destroy", "inkq_f16w_matmul_prec",
    "inkq_f16w_matmul", "inkq_peer_export", "inkq_peerset_open", "inkq_peerset_from_pointers", "inkq_peerset_destroy",
    "inkq_linear_scatter", "inkq_gemm_scatter", "inkq_peer_barrier", "inkq_f16w_matmul_scatter", "inkq_weight_quantize_dev",
]


# every symbol include/inkq_glue.h declares
GLUE_SYMBOLS = ["inkq_glue_embedding", "inkq_glue_rmsnorm", "inkq_glue_qknorm_rope_cache", "inkq_glue_attention", "inkq_glue_silu_mul",
                "inkq_glue_add_inplace", "inkq_glue_argmax_advance", "inkq_glue_silu_mul_rows", "inkq_glue_linear_m1", "inkq_glue_decode_gemv", "inkq_glue_rmsnorm_quant",
                "inkq_glue_attention_quant", "inkq_glue_add_rmsnorm_quant_rows", "inkq_glue_silu_mul_quant_rows", "inkq_glue_attention_quant_rows", "inkq_glue_qkv_attention_quant"]


PEER_RESERVED_BYTES = 256   # INKQ_PEER_RESERVED_BYTES
PEER_HANDLE_BYTES = 80      # INKQ_PEER_HANDLE_BYTES


class InkqError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"inkq status {code}: {msg}")
        self.code = code


_lib = None


def lib() -> C.CDLL:
    """Loads libinkq.so (must have been built: `__graft_entry__.build()`)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'`")
        L = C.CDLL(LIB_PATH)
        L.inkq_last_error.restype = C.c_char_p
        L.inkq_last_error.argtypes = [C.c_void_p]
        L.inkq_launch_count.restype = C.c_uint64
        L.inkq_launch_count.argtypes = [C.c_void_p]
        for name in SYMBOLS + GLUE_SYMBOLS:
            fn = getattr(L, name)
            if name not in ("inkq_last_error", "inkq_launch_count"):
                fn.restype = C.c_int
        _lib = L
    return _lib


def _dp(t):
    """Device pointer of a torch tensor (or an int address, or None)."""
    if t is None:
        return None
    if isinstance(t, int):
        return C.c_void_p(t)
    return C.c_void_p(t.data_ptr())


def _hp(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class PeerSet:
    """Handle of a peer set (keeps the local buffers alive)."""

    def __init__(self, ctx, h, world, rank, keep):
        self.ctx, self.h, self.world, self.rank, self.keep = ctx, h, world, rank, keep

    def close(self):
        if self.h:
            self.ctx.L.inkq_peerset_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Context:
    """One device + stream.  Mirrors the role of the reference's ModelContext
    (qwen3/include/qwen/QwenOperator.h:34-43): it owns the activation scratch."""

    def __init__(self, device: int = 0, stream: int | None = None):
        self.L = lib()
        h = C.c_void_p()
        rc = self.L.inkq_ctx_create(int(device), C.c_void_p(stream or 0), C.byref(h))
        if rc != OK:
            raise InkqError(rc, self.L.inkq_last_error(None).decode())
        self.h = h
        self.device = device

    def check(self, rc: int):
        if rc != OK:
            raise InkqError(rc, self.L.inkq_last_error(self.h).decode())

    def close(self):
        if getattr(self, "h", None):
            self.L.inkq_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_stream(self, stream: int):
        self.check(self.L.inkq_ctx_set_stream(self.h, C.c_void_p(stream)))

    def synchronize(self):
        self.check(self.L.inkq_ctx_synchronize(self.h))

    @property
    def launches(self) -> int:
        return int(self.L.inkq_launch_count(self.h))

    # ---- weights ----------------------------------------------------------------
    def weight(self, scheme: int, scale_mode: int, nib, d, m=None, zp=None, n_begin: int = 0, n_end: int | None = None):
        """Host NumPy arrays in the logical disk format -> device-resident re-tiled weight."""
        nib = np.ascontiguousarray(nib, np.uint8)
        d = np.ascontiguousarray(d, np.float32)
        m = None if m is None else np.ascontiguousarray(m, np.float32)
        zp = None if zp is None else np.ascontiguousarray(zp, np.uint8)
        N, K = nib.shape[0], nib.shape[1] * 2
        h = C.c_void_p()
        self.check(self.L.inkq_weight_create(self.h, scheme, scale_mode, N, K, _hp(nib), _hp(d), _hp(m), _hp(zp),
                                             n_begin, N if n_end is None else n_end, C.byref(h)))
        return Weight(self, h, scheme)

    def weight_dev(self, scheme: int, scale_mode: int, N: int, K: int, nib, d, m=None, zp=None, n_begin: int = 0,
                   n_end: int | None = None):
        """Same from device tensors (torch) holding the logical format."""
        h = C.c_void_p()
        self.check(self.L.inkq_weight_create_dev(self.h, scheme, scale_mode, N, K, _dp(nib), _dp(d), _dp(m), _dp(zp),
                                                 n_begin, N if n_end is None else n_end, C.byref(h)))
        return Weight(self, h, scheme)

    def quantize_weights(self, fmt: int, w):
        """fp32 weights [N][K] (torch, on the device) -> (nib, d, m, zp) device tensors in the on-disk format.
        fmt 0: Q4_0 (quantize_row_q40_tinyml), 1: Q4_1 (quantize_row_q41_tinyml)."""
        import torch
        N, K = w.shape
        nib = torch.empty((N, K // 2), dtype=torch.uint8, device=w.device)
        d = torch.empty((N, K // 32), dtype=torch.float32, device=w.device)
        m = torch.empty_like(d)
        zp = torch.empty((N, K // 32), dtype=torch.int8, device=w.device)
        self.check(self.L.inkq_weight_quantize_dev(self.h, fmt, N, K, _dp(w.contiguous()), _dp(nib), _dp(d), _dp(m), _dp(zp)))
        return nib, d, m, zp

    def act(self, max_rows: int, K: int):
        h = C.c_void_p()
        self.check(self.L.inkq_act_create(self.h, max_rows, K, C.byref(h)))
        return Act(self, h, K)

    def f16w(self, w16: np.ndarray, n_begin: int = 0, n_end: int | None = None):
        w16 = np.ascontiguousarray(w16, np.float16)
        N, K = w16.shape
        h = C.c_void_p()
        self.check(self.L.inkq_f16w_create(self.h, N, K, _hp(w16), n_begin, N if n_end is None else n_end, C.byref(h)))
        return F16W(self, h, (N if n_end is None else n_end) - n_begin, K)

    def f16w_dev(self, w16, N: int, K: int, n_begin: int = 0, n_end: int | None = None):
        h = C.c_void_p()
        self.check(self.L.inkq_f16w_create_dev(self.h, N, K, _dp(w16), n_begin, N if n_end is None else n_end, C.byref(h)))
        return F16W(self, h, (N if n_end is None else n_end) - n_begin, K)

    # ---- kernels ------------------------------------------------------------------
    def quantize(self, act: "Act", x, M: int, qmode: int):
        self.check(self.L.inkq_quantize(self.h, qmode, _dp(x), M, act.K, act.h))

    def act_import(self, act: "Act", qmode: int, q, d, s=None):
        q = np.ascontiguousarray(q, np.int8)
        d = np.ascontiguousarray(d, np.float32)
        s = None if s is None else np.ascontiguousarray(s, np.float32)
        self.check(self.L.inkq_act_import(self.h, act.h, qmode, q.shape[0], _hp(q), _hp(d), _hp(s)))

    def gemm(self, act, w, Cdev, ldc: int):
        self.check(self.L.inkq_gemm(self.h, act.h, w.h, _dp(Cdev), ldc))

    def gemm_simt(self, act, w, Cdev, ldc: int):
        self.check(self.L.inkq_gemm_simt(self.h, act.h, w.h, _dp(Cdev), ldc))

    def gemv(self, act, w, Cdev):
        self.check(self.L.inkq_gemv(self.h, act.h, w.h, _dp(Cdev)))

    def block_dots(self, act, w, dots_dev, tensor_core: bool = False):
        fn = self.L.inkq_debug_block_dots_tc if tensor_core else self.L.inkq_debug_block_dots
        self.check(fn(self.h, act.h, w.h, _dp(dots_dev)))

    def linear(self, w, x, M: int, Cdev, ldc: int):
        """Qwen_Linear_with_bias_Int4::forward on device buffers."""
        self.check(self.L.inkq_linear(self.h, w.h, _dp(x), M, _dp(Cdev), ldc))

    def linear_host(self, w, x_host, M: int, C_host, ldc: int):
        """Same with host buffers (NumPy arrays, or torch CPU tensors, ideally pinned)."""
        xp = x_host.ctypes.data_as(C.c_void_p) if isinstance(x_host, np.ndarray) else C.c_void_p(x_host.data_ptr())
        cp = C_host.ctypes.data_as(C.c_void_p) if isinstance(C_host, np.ndarray) else C.c_void_p(C_host.data_ptr())
        self.check(self.L.inkq_linear_host(self.h, w.h, xp, M, cp, ldc))

    # ---- column-sharded layer with in-kernel exchange (csrc/peer.cu)
    def peer_export(self, buf) -> bytes:
        """80-byte blob naming the device buffer `buf` (a torch uint8/float tensor) for other processes."""
        blob = C.create_string_buffer(PEER_HANDLE_BYTES)
        self.check(self.L.inkq_peer_export(self.h, _dp(buf), C.c_size_t(buf.numel() * buf.element_size()), blob))
        return blob.raw

    def peerset_open(self, world: int, rank: int, local_buf, blobs):
        h = C.c_void_p()
        raw = b"".join(blobs)
        assert len(raw) == world * PEER_HANDLE_BYTES
        self.check(self.L.inkq_peerset_open(self.h, world, rank, _dp(local_buf), raw, C.byref(h)))
        return PeerSet(self, h, world, rank, [local_buf])

    def peerset_from_tensors(self, rank: int, bufs):
        """Peer set over buffers this process can address itself (same GPU, or peer access enabled)."""
        h = C.c_void_p()
        arr = (C.c_void_p * len(bufs))(*[b.data_ptr() for b in bufs])
        nbytes = bufs[0].numel() * bufs[0].element_size()
        self.check(self.L.inkq_peerset_from_pointers(self.h, len(bufs), rank, arr, C.c_size_t(nbytes), C.byref(h)))
        return PeerSet(self, h, len(bufs), rank, list(bufs))

    def linear_scatter(self, w, x, M: int, ps, byte_offset: int, ldc: int):
        """inkq_linear whose epilogue stores the shard's columns into every rank's buffer of the peer set."""
        self.check(self.L.inkq_linear_scatter(self.h, w.h, _dp(x), M, ps.h, C.c_size_t(byte_offset), ldc))

    def gemm_scatter(self, act, w, ps, byte_offset: int, ldc: int):
        """inkq_gemm on rows already quantized into `act`, same multi-destination epilogue."""
        self.check(self.L.inkq_gemm_scatter(self.h, act.h, w.h, ps.h, C.c_size_t(byte_offset), ldc))

    def f16w_matmul_scatter(self, w, x, M: int, ps, byte_offset: int, ldc: int, precision: int = 0):
        self.check(self.L.inkq_f16w_matmul_scatter(self.h, w.h, _dp(x), M, ps.h, C.c_size_t(byte_offset), ldc, precision))

    def peer_barrier(self, ps, timeout_ms: int = 2000):
        self.check(self.L.inkq_peer_barrier(self.h, ps.h, timeout_ms))

    def linear_m1_static(self, w, x, Cdev):
        """M == 1 forward that never allocates: scratch in the library's fixed device array (K <= 16384)."""
        self.check(self.L.inkq_linear_m1_static(self.h, w.h, _dp(x), _dp(Cdev)))

    def gemm_w41_f16act(self, a16, M: int, w, Cdev, ldc: int):
        self.check(self.L.inkq_gemm_w41_f16act(self.h, _dp(a16), M, w.h, _dp(Cdev), ldc))

    def gemm_w41_f16act_simt(self, a16, M: int, w, Cdev, ldc: int):
        """CUDA-core cross-check of gemm_w41_f16act (slow)."""
        self.check(self.L.inkq_gemm_w41_f16act_simt(self.h, _dp(a16), M, w.h, _dp(Cdev), ldc))

    def f16w_matmul_prec(self, w, x, M: int, Cdev, ldc: int, precision: int):
        """precision 0: fp32-grade activations (fp16 hi + lo, two passes), 1: activations rounded to fp16 (one pass)."""
        self.check(self.L.inkq_f16w_matmul_prec(self.h, w.h, _dp(x), M, _dp(Cdev), ldc, precision))

    def f16w_matmul(self, w, x, M: int, Cdev, ldc: int):
        self.check(self.L.inkq_f16w_matmul(self.h, w.h, _dp(x), M, _dp(Cdev), ldc))


class Weight:
    def __init__(self, ctx: Context, h, scheme: int):
        self.ctx, self.h, self.scheme = ctx, h, scheme
        rows, K, sch, nbytes = C.c_int(), C.c_int(), C.c_int(), C.c_size_t()
        ctx.check(ctx.L.inkq_weight_info(h, C.byref(rows), C.byref(K), C.byref(sch), C.byref(nbytes)))
        self.rows, self.K, self.device_bytes = rows.value, K.value, nbytes.value

    def export(self):
        """Inverse re-tiling -> (nib, d, m, zp) host arrays of the held rows."""
        nb = self.K // 32
        nib = np.empty((self.rows, self.K // 2), np.uint8)
        d = np.empty((self.rows, nb), np.float32)
        m = np.empty((self.rows, nb), np.float32)
        zp = np.empty((self.rows, nb), np.uint8)
        self.ctx.check(self.ctx.L.inkq_weight_export(self.ctx.h, self.h, _hp(nib), _hp(d), _hp(m), _hp(zp)))
        return nib, d, m, zp

    def close(self):
        if self.h:
            self.ctx.L.inkq_weight_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            if self.ctx.h:
                self.close()
        except Exception:
            pass


class Act:
    def __init__(self, ctx: Context, h, K: int):
        self.ctx, self.h, self.K = ctx, h, K

    def export(self, M: int):
        nb = self.K // 32
        q = np.empty((M, self.K), np.int8)
        d = np.empty((M, nb), np.float32)
        s = np.empty((M, nb), np.float32)
        isum = np.empty((M, nb), np.int32)
        self.ctx.check(self.ctx.L.inkq_act_export(self.ctx.h, self.h, _hp(q), _hp(d), _hp(s), _hp(isum)))
        return q, d, s, isum

    def close(self):
        if self.h:
            self.ctx.L.inkq_act_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            if self.ctx.h:
                self.close()
        except Exception:
            pass


class F16W:
    def __init__(self, ctx: Context, h, rows: int, K: int):
        self.ctx, self.h, self.rows, self.K = ctx, h, rows, K

    def close(self):
        if self.h:
            self.ctx.L.inkq_f16w_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            if self.ctx.h:
                self.close()
        except Exception:
            pass


def build(force: bool = False) -> None:
    _build.build_all(force)
