"""ctypes front end of the CPU oracle (oracle/muser_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg.  The product package never imports this module.

Every function takes and returns numpy arrays; the C symbol it wraps cites the
reference function it restates.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libmuser_oracle.so"

F32, F16, Q4_K, Q5_K, Q6_K, BF16, NVFP4 = 0, 1, 12, 13, 14, 30, 1000
BLOCK_BYTES = {Q4_K: 144, Q5_K: 176, Q6_K: 210}


def build(force: bool = False) -> Path:
    """Compile the oracle with gcc if the shared object is missing or stale."""
    src = _HERE / "muser_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B", "-s"], check=True, capture_output=True)
    return _LIB_PATH


class _TensorView(C.Structure):
    _fields_ = [
        ("raw", C.c_void_p),
        ("dtype", C.c_uint32),
        ("n_in", C.c_size_t),
        ("n_out", C.c_size_t),
        ("block_scales", C.c_void_p),
        ("scale2", C.c_float),
        ("has_input_scale_inv", C.c_int),
        ("input_scale_inv", C.c_float),
    ]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(build()))
        L = _lib
        u8p, f32p, i8p = C.c_void_p, C.c_void_p, C.c_void_p
        L.oracle_f16_to_f32.restype = C.c_float
        L.oracle_f16_to_f32.argtypes = [C.c_uint16]
        L.oracle_f32_to_f16_trunc.restype = C.c_uint16
        L.oracle_f32_to_f16_trunc.argtypes = [C.c_float]
        L.oracle_f32_to_f16_rne.restype = C.c_uint16
        L.oracle_f32_to_f16_rne.argtypes = [C.c_float]
        L.oracle_silu_fast.restype = C.c_float
        L.oracle_silu_fast.argtypes = [C.c_float]
        for name in ("q4_k", "q5_k", "q6_k"):
            f = getattr(L, f"oracle_dequant_{name}")
            f.restype = None
            f.argtypes = [u8p, f32p]
        for name in ("q4_k_f32", "q4_k_f32_llama", "q5_k_f32", "q6_k_f32"):
            f = getattr(L, f"oracle_dot_{name}")
            f.restype = C.c_float
            f.argtypes = [u8p, f32p, C.c_size_t]
        L.oracle_e2m1_q1.restype = C.c_int32
        L.oracle_e2m1_q1.argtypes = [C.c_uint8]
        L.oracle_e4m3fn_q9.restype = C.c_int32
        L.oracle_e4m3fn_q9.argtypes = [C.c_uint8]
        L.oracle_e2m1_to_f32.restype = C.c_float
        L.oracle_e2m1_to_f32.argtypes = [C.c_uint8]
        L.oracle_e4m3fn_to_f32.restype = C.c_float
        L.oracle_e4m3fn_to_f32.argtypes = [C.c_uint8]
        L.oracle_e4m3fn_from_f32.restype = C.c_uint8
        L.oracle_e4m3fn_from_f32.argtypes = [C.c_float]
        L.oracle_e2m1_from_f32.restype = C.c_uint8
        L.oracle_e2m1_from_f32.argtypes = [C.c_float]
        L.oracle_quantize_nvfp4_activation.restype = None
        L.oracle_quantize_nvfp4_activation.argtypes = [f32p, C.c_size_t, C.c_float, u8p, u8p]
        L.oracle_dequant_nvfp4_row.restype = None
        L.oracle_dequant_nvfp4_row.argtypes = [u8p, u8p, C.c_float, f32p, C.c_size_t]
        for name in ("oracle_dot_nvfp4_f32", "oracle_dot_nvfp4_block_fused_f32", "oracle_dot_nvfp4_a16_q8_f32"):
            f = getattr(L, name)
            f.restype = C.c_float
            f.argtypes = [u8p, u8p, C.c_float, f32p, C.c_size_t]
        L.oracle_dot_nvfp4_w4a4_f32.restype = C.c_float
        L.oracle_dot_nvfp4_w4a4_f32.argtypes = [u8p, u8p, C.c_float, C.c_float, f32p, C.c_size_t]
        L.oracle_quantize_nvfp4_q8_block.restype = C.c_float
        L.oracle_quantize_nvfp4_q8_block.argtypes = [f32p, i8p]
        L.oracle_row_bytes.restype = C.c_size_t
        L.oracle_row_bytes.argtypes = [C.c_uint32, C.c_size_t]
        L.oracle_dequant_row.restype = C.c_int
        L.oracle_dequant_row.argtypes = [C.POINTER(_TensorView), C.c_size_t, f32p]
        L.oracle_matmul.restype = C.c_int
        L.oracle_matmul.argtypes = [C.POINTER(_TensorView), f32p, C.c_size_t, f32p, f32p, C.c_int, C.c_int]
        L.oracle_rms_norm_mul.restype = None
        L.oracle_rms_norm_mul.argtypes = [f32p, C.c_size_t, C.c_size_t, C.c_float, f32p]
        L.oracle_silu_mul.restype = None
        L.oracle_silu_mul.argtypes = [f32p, f32p, f32p, C.c_size_t]
        L.oracle_sigmoid_gate.restype = None
        L.oracle_sigmoid_gate.argtypes = [f32p, f32p, C.c_size_t]
        L.oracle_logit_tail.restype = None
        L.oracle_logit_tail.argtypes = [f32p, C.c_size_t, C.c_float, C.c_float]
        L.oracle_matmul_rows.restype = C.c_int
        L.oracle_matmul_rows.argtypes = [C.POINTER(_TensorView), f32p, C.c_size_t, C.c_void_p, C.c_size_t, f32p]
    return _lib


def _p(a: np.ndarray) -> int:
    return a.ctypes.data


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.uint8))


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def host_threads() -> int:
    return len(os.sched_getaffinity(0))


# ---------------------------------------------------------------- scalars

def f16_to_f32(h: int) -> float:
    return lib().oracle_f16_to_f32(h)


def f32_to_f16_rne(x: float) -> int:
    return lib().oracle_f32_to_f16_rne(x)


def f32_to_f16_trunc(x: float) -> int:
    return lib().oracle_f32_to_f16_trunc(x)


def e2m1_to_f32(code: int) -> float:
    return lib().oracle_e2m1_to_f32(code)


def e4m3fn_to_f32(code: int) -> float:
    return lib().oracle_e4m3fn_to_f32(code)


def e4m3fn_from_f32(v: float) -> int:
    return lib().oracle_e4m3fn_from_f32(v)


def e2m1_from_f32(v: float) -> int:
    return lib().oracle_e2m1_from_f32(v)


def e2m1_q1(code: int) -> int:
    return lib().oracle_e2m1_q1(code)


def e4m3fn_q9(code: int) -> int:
    return lib().oracle_e4m3fn_q9(code)


def silu_fast(x: float) -> float:
    return lib().oracle_silu_fast(x)


# ---------------------------------------------------------------- K-quants

def dequant_blocks(dtype: int, blocks) -> np.ndarray:
    """Dequantise a byte string of whole K-quant blocks to f32."""
    blocks = _u8(blocks).reshape(-1)
    bs = BLOCK_BYTES[dtype]
    n = blocks.size // bs
    out = np.empty(n * 256, dtype=np.float32)
    fn = {Q4_K: lib().oracle_dequant_q4_k, Q5_K: lib().oracle_dequant_q5_k, Q6_K: lib().oracle_dequant_q6_k}[dtype]
    for b in range(n):
        fn(_p(blocks) + b * bs, _p(out) + b * 1024)
    return out


def dot_kquant(dtype: int, row, x, llama_order: bool = False) -> float:
    row, x = _u8(row), _f32(x)
    L = lib()
    if dtype == Q4_K:
        fn = L.oracle_dot_q4_k_f32_llama if llama_order else L.oracle_dot_q4_k_f32
    else:
        fn = {Q5_K: L.oracle_dot_q5_k_f32, Q6_K: L.oracle_dot_q6_k_f32}[dtype]
    return fn(_p(row), _p(x), x.size)


# ------------------------------------------------------------------- NVFP4

def quantize_nvfp4_activation(x, input_scale_inv: float):
    """x: [..., K] f32 -> (packed [..., K/2] u8, scales [..., K/16] u8), row-major (unswizzled)."""
    x = _f32(x)
    packed = np.empty(x.shape[:-1] + (x.shape[-1] // 2,), dtype=np.uint8)
    scales = np.empty(x.shape[:-1] + (x.shape[-1] // 16,), dtype=np.uint8)
    lib().oracle_quantize_nvfp4_activation(_p(x), x.size, input_scale_inv, _p(packed), _p(scales))
    return packed, scales


def dequant_nvfp4(packed, scales, scale2: float) -> np.ndarray:
    packed, scales = _u8(packed), _u8(scales)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.float32)
    lib().oracle_dequant_nvfp4_row(_p(packed), _p(scales), scale2, _p(out), out.size)
    return out


def dot_nvfp4_f32(packed, scales, scale2, x) -> float:
    packed, scales, x = _u8(packed), _u8(scales), _f32(x)
    return lib().oracle_dot_nvfp4_f32(_p(packed), _p(scales), scale2, _p(x), x.size)


def dot_nvfp4_block_fused_f32(packed, scales, scale2, x) -> float:
    packed, scales, x = _u8(packed), _u8(scales), _f32(x)
    return lib().oracle_dot_nvfp4_block_fused_f32(_p(packed), _p(scales), scale2, _p(x), x.size)


def dot_nvfp4_w4a4_f32(packed, scales, scale2, input_scale_inv, x) -> float:
    packed, scales, x = _u8(packed), _u8(scales), _f32(x)
    return lib().oracle_dot_nvfp4_w4a4_f32(_p(packed), _p(scales), scale2, input_scale_inv, _p(x), x.size)


def dot_nvfp4_a16_q8_f32(packed, scales, scale2, x) -> float:
    packed, scales, x = _u8(packed), _u8(scales), _f32(x)
    return lib().oracle_dot_nvfp4_a16_q8_f32(_p(packed), _p(scales), scale2, _p(x), x.size)


def quantize_nvfp4_q8_block(x):
    x = _f32(x)
    assert x.size == 256
    qs = np.empty(256, dtype=np.int8)
    d = lib().oracle_quantize_nvfp4_q8_block(_p(x), _p(qs))
    return d, qs


# ---------------------------------------------------------------- operator

class TensorView:
    """Mirror of weights.rs `TensorView` + `Nvfp4AuxView` over numpy byte arrays."""

    def __init__(self, raw, dtype: int, n_in: int, n_out: int, block_scales=None, scale2: float = 1.0,
                 input_scale_inv: float | None = None):
        self.raw = _u8(raw).reshape(-1)
        self.dtype, self.n_in, self.n_out = dtype, n_in, n_out
        self.block_scales = None if block_scales is None else _u8(block_scales).reshape(-1)
        self.scale2 = float(scale2)
        self.input_scale_inv = input_scale_inv
        assert self.raw.size == n_out * row_bytes(dtype, n_in), "weight bytes do not match the geometry"
        if dtype == NVFP4:
            assert self.block_scales is not None and self.block_scales.size == n_out * n_in // 16

    def _c(self) -> _TensorView:
        return _TensorView(
            _p(self.raw), self.dtype, self.n_in, self.n_out,
            0 if self.block_scales is None else _p(self.block_scales), self.scale2,
            0 if self.input_scale_inv is None else 1,
            0.0 if self.input_scale_inv is None else float(self.input_scale_inv),
        )


def row_bytes(dtype: int, n_in: int) -> int:
    return lib().oracle_row_bytes(dtype, n_in)


def dequant_tensor(w: TensorView) -> np.ndarray:
    out = np.empty((w.n_out, w.n_in), dtype=np.float32)
    v = w._c()
    for r in range(w.n_out):
        rc = lib().oracle_dequant_row(C.byref(v), r, _p(out) + r * w.n_in * 4)
        assert rc == 0
    return out


def matmul(w: TensorView, x, threads: int = 1, hoist_activation: bool = True, return_pre_round: bool = False):
    """weights.rs `matmul`: x [T][n_in] f32 -> out [T][n_out] f32."""
    x = _f32(x).reshape(-1, w.n_in)
    t = x.shape[0]
    out = np.empty((t, w.n_out), dtype=np.float32)
    pre = np.empty((t, w.n_out), dtype=np.float32) if return_pre_round else None
    v = w._c()
    rc = lib().oracle_matmul(C.byref(v), _p(x), t, _p(out), 0 if pre is None else _p(pre), threads,
                             1 if hoist_activation else 0)
    if rc != 0:
        raise ValueError("oracle_matmul rejected the shapes / dtype")
    return (out, pre) if return_pre_round else out


def rms_norm_mul(x, eps: float, w=None) -> np.ndarray:
    x = _f32(x).copy()
    rows, dim = x.reshape(-1, x.shape[-1]).shape
    wv = None if w is None else _f32(w)
    lib().oracle_rms_norm_mul(_p(x), rows, dim, eps, 0 if wv is None else _p(wv))
    return x


def logit_tail(logits, logit_scale: float, softcap: float) -> np.ndarray:
    """reference.rs:559-570: logits * logit_scale, then softcap * tanh(. / softcap) when softcap > 0."""
    out = _f32(logits).copy()
    lib().oracle_logit_tail(_p(out), out.size, logit_scale, softcap)
    return out


def matmul_rows(w: "TensorView", x, rows) -> np.ndarray:
    """weights.rs `matmul_rows`: out [T][len(rows)]."""
    x = _f32(x).reshape(-1, w.n_in)
    idx = np.ascontiguousarray(rows, dtype=np.uint64)
    out = np.empty((x.shape[0], idx.size), dtype=np.float32)
    v = w._c()
    if lib().oracle_matmul_rows(C.byref(v), _p(x), x.shape[0], idx.ctypes.data, idx.size, _p(out)) != 0:
        raise ValueError("oracle_matmul_rows rejected a row index, the shapes or the dtype")
    return out


def sigmoid_gate(x, gate) -> np.ndarray:
    """reference.rs:447-455: x * sigmoid(gate)."""
    out, g = _f32(x).copy(), _f32(gate)
    lib().oracle_sigmoid_gate(_p(out), _p(g), out.size)
    return out


def norm_residual_norm(hidden, src, w1, eps1, w2=None, eps2=0.0):
    """reference.rs:466-490: hidden + rms_norm_mul(src, eps1, w1), and rms_norm_mul of that with (eps2, w2)."""
    h = _f32(hidden) + rms_norm_mul(src, eps1, w1)
    return h, (rms_norm_mul(h, eps2, w2) if w2 is not None else None)


def silu_mul(gate, up) -> np.ndarray:
    gate, up = _f32(gate), _f32(up)
    out = np.empty_like(gate)
    lib().oracle_silu_mul(_p(gate), _p(up), _p(out), gate.size)
    return out
