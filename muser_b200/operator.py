"""Host-side mirror of the reference's quantized-matmul operator interface, over the C ABI.

Names, argument meaning and error behaviour follow the reference so that a test written against
`MetalKernels` / `weights::matmul` reads the same here:

    crates/muser-engine/src/weights.rs:29-48     TensorView / Nvfp4AuxView   -> TensorView
    src/weights.rs:398-421                       matmul(w, x, n_tokens, out) -> matmul
    src/metal/encode.rs:370-385                  supports_projection         -> CudaKernels.supports_projection
    src/metal/encode/qkv.rs:414-424              encode_quantized_matmul     -> CudaKernels.encode_quantized_matmul
    src/metal/encode/qkv.rs:128-140              encode_nvfp4_matmul         -> CudaKernels.encode_nvfp4_matmul
    src/metal/encode/qkv.rs:13-26                encode_nvfp4_w4a4_prequant_m16 -> CudaKernels.encode_nvfp4_prequant
    src/metal/encode/ffn.rs:10-19                encode_ffn_q4k_gate_up_silu_4r2s -> CudaKernels.encode_ffn_gate_up_silu

torch supplies device memory and streams only; every computation goes through libmuser_cuda.so.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib
from ._lib import (BF16, F16, F32, NVFP4, Q4_K, Q6_K, SHARD_K, SHARD_NONE, SHARD_ROWS, TUNE_DECODE_KSPLIT, TUNE_DECODE_RING,
                   TUNE_DECODE_WARPS, TUNE_DECODE_WSPLIT, TUNE_TC_MIN_ROWS, TUNE_TC_MIN_TOKENS_Q4_K, TUNE_TC_MIN_TOKENS_Q6_K, MuserCudaError)

_L = _lib.lib
_TORCH_DTYPE = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


@dataclass
class TensorView:
    """The stored tensor, exactly as the reference's weight loader sees it (weights.rs:29-48).

    raw: K-quant rows of blocks, or NVFP4 packed E2M1 bytes [n_out][n_in/2]; a host numpy array or a
    torch uint8 tensor (host or device).  block_scales / scale2 / input_scale_inv are the NVFP4 companions.
    """
    raw: object
    dtype: int
    n_in: int
    n_out: int
    block_scales: object = None
    scale2: float = 1.0
    input_scale_inv: float | None = None


class Context:
    """One per device: owns the workspace that the NVFP4 lane quantizes activations into."""

    def __init__(self, device: int = 0, workspace_bytes: int = 64 << 20):
        self.device = device
        h = C.c_void_p()
        st = _L.muser_cuda_ctx_create(device, workspace_bytes, C.byref(h))
        if st != 0:
            raise MuserCudaError(st, (_L.muser_cuda_last_error(None) or b"").decode())
        self._h = h

    def check(self, st: int) -> None:
        if st != 0:
            raise MuserCudaError(st, (_L.muser_cuda_last_error(self._h) or b"").decode())

    def sync_status(self) -> None:
        self.check(_L.muser_cuda_sync_status(self._h, _stream_ptr(self.device)))

    def tuning_set(self, key: int, value: int) -> None:
        """muser_cuda_tuning_set: move a kernel-choice threshold (the TUNE_* keys)."""
        self.check(_L.muser_cuda_tuning_set(self._h, key, value))

    def close(self) -> None:
        if self._h:
            _L.muser_cuda_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Weight:
    """A repacked device image of one projection (or of one tensor-parallel shard of it)."""

    def __init__(self, ctx: Context, view: TensorView, shard: tuple[int, int, int] | None = None):
        self.ctx = ctx
        h = C.c_void_p()
        sh = _lib.Shard(*shard) if shard else None
        raw, scales = view.raw, view.block_scales
        on_device = isinstance(raw, torch.Tensor) and raw.is_cuda
        has_isi = 0 if view.input_scale_inv is None else 1
        isi = 0.0 if view.input_scale_inv is None else float(view.input_scale_inv)
        if on_device:
            raw = raw.contiguous()
            sp = None
            if scales is not None:
                scales = scales.contiguous()
                sp = scales.data_ptr()
            st = _L.muser_cuda_weight_repack_device(ctx._h, view.dtype, raw.data_ptr(), sp, view.scale2, has_isi, isi,
                                                    view.n_in, view.n_out, C.byref(sh) if sh else None,
                                                    _stream_ptr(ctx.device), C.byref(h))
        else:
            raw = np.ascontiguousarray(raw.numpy() if isinstance(raw, torch.Tensor) else raw, dtype=np.uint8)
            sp = None
            if scales is not None:
                scales = np.ascontiguousarray(scales.numpy() if isinstance(scales, torch.Tensor) else scales, dtype=np.uint8)
                sp = scales.ctypes.data
            expect = view.n_out * _row_bytes(view.dtype, view.n_in)
            if raw.size != expect:
                raise MuserCudaError(2, f"weight bytes {raw.size} do not match the geometry ({expect})")
            st = _L.muser_cuda_weight_repack(ctx._h, view.dtype, raw.ctypes.data, sp, view.scale2, has_isi, isi,
                                             view.n_in, view.n_out, C.byref(sh) if sh else None, C.byref(h))
        ctx.check(st)
        self._h = h
        info = _lib.WeightInfo()
        self.dtype, self.view_dtype = view.dtype, view.dtype
        self._info = None
        self.n_in_full, self.n_out_full = view.n_in, view.n_out
        world = shard[1] if shard else 1
        axis = shard[2] if shard else SHARD_NONE
        self.n_in = view.n_in // world if axis == SHARD_K else view.n_in
        self.n_out = view.n_out // world if axis == SHARD_ROWS else view.n_out
        self.scale2, self.input_scale_inv = view.scale2, view.input_scale_inv
        del info

    def info(self) -> _lib.WeightInfo:
        out = _lib.WeightInfo()
        st = _L.muser_cuda_weight_info_get(self._h, C.byref(out))
        self.ctx.check(st)
        return out

    def free(self) -> None:
        if self._h:
            _L.muser_cuda_weight_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _row_bytes(dtype: int, n_in: int) -> int:
    if dtype == Q4_K:
        return n_in // 256 * 144
    if dtype == _lib.Q5_K:
        return n_in // 256 * 176
    if dtype == Q6_K:
        return n_in // 256 * 210
    if dtype == NVFP4:
        return n_in // 2
    raise MuserCudaError(4, f"dtype {dtype} has no CUDA projection kernel")


def _epilogue(row_scale=None, residual=None, norm_weight=None, norm_eps=0.0, out_scale=1.0, softcap=0.0, all_reduce=False):
    """muser_cuda_epilogue; `norm_weight` (f32 [n_in], device) fuses rms_norm_mul(x, eps, norm_weight) in front,
    `out_scale` / `softcap` the LM-head tail y <- softcap * tanh(y * out_scale / softcap) behind."""
    if row_scale is None and residual is None and norm_weight is None and out_scale == 1.0 and softcap == 0.0 and not all_reduce:
        return None
    if norm_weight is not None and norm_weight.dtype != torch.float32:
        raise MuserCudaError(1, "norm_weight must be f32")
    return _lib.Epilogue(row_scale.data_ptr() if row_scale is not None else None,
                         residual.data_ptr() if residual is not None else None, 0, float(norm_eps),
                         norm_weight.data_ptr() if norm_weight is not None else None, float(out_scale), float(softcap), int(bool(all_reduce)))


class CudaKernels:
    """Counterpart of the reference's `MetalKernels` for the projections of one device."""

    def __init__(self, ctx: Context):
        self.ctx = ctx
        self.launches = 0  # kernels this object has enqueued

    @staticmethod
    def supports_projection(dtype: int) -> bool:
        return bool(_L.muser_cuda_supports_projection(dtype))

    def dequant(self, w: Weight) -> torch.Tensor:
        out = torch.empty((w.n_out, w.n_in), dtype=torch.float32, device=f"cuda:{self.ctx.device}")
        self.ctx.check(_L.muser_cuda_dequant(self.ctx._h, w._h, out.data_ptr(), _stream_ptr(self.ctx.device)))
        self.launches += 1
        return out

    def encode_quantized_matmul(self, weights: Weight, input: torch.Tensor, output: torch.Tensor, tokens: int,
                                row_scale=None, residual=None, norm_weight=None, norm_eps=0.0, out_scale=1.0,
                                softcap=0.0, all_reduce=False) -> None:
        """y[t][r] = dot(W_r, x_t) for K-quant weights; input [tokens][n_in] f32|bf16, output [tokens][n_out] f32|bf16.
        all_reduce: the weight is a K shard; the call also sums the output over the context's communicator."""
        ep = _epilogue(row_scale, residual, norm_weight, norm_eps, out_scale, softcap, all_reduce)
        self.ctx.check(_L.muser_cuda_quantized_matmul(
            self.ctx._h, weights._h, input.data_ptr(), _TORCH_DTYPE[input.dtype], output.data_ptr(),
            _TORCH_DTYPE[output.dtype], tokens, C.byref(ep) if ep else None, _stream_ptr(self.ctx.device)))
        self.launches += 2 if all_reduce else 1

    def encode_quantized_matmul_group(self, weights, input: torch.Tensor, outputs, tokens: int, epilogues=None) -> None:
        """Up to four K-quant projections of the same `input` in one launch (q | k | v, or gate | up), the counterpart
        of the reference's one-barrier-interval dispatch (decode.rs:5569-5598).  `epilogues`: per projection a dict of
        encode_quantized_matmul's keyword arguments, or None."""
        n = len(weights)
        items = (_lib.GroupItem * n)()
        keep = []
        for i, (w, y) in enumerate(zip(weights, outputs)):
            ep = _epilogue(**(epilogues[i] or {})) if epilogues else None
            keep.append(ep)
            items[i].w, items[i].y, items[i].y_dtype, items[i].reserved = w._h.value, y.data_ptr(), _TORCH_DTYPE[y.dtype], 0
            items[i].epilogue = C.pointer(ep) if ep is not None else None
        self.ctx.check(_L.muser_cuda_quantized_matmul_group(
            self.ctx._h, items, n, input.data_ptr(), _TORCH_DTYPE[input.dtype], tokens, _stream_ptr(self.ctx.device)))
        self.launches += 1

    def last_decode_plan(self) -> tuple:
        """(warps per CTA, K slices between CTAs, K parts between a CTA's warps, ring depth) of the latest decode launch."""
        out = (C.c_uint32 * 4)()
        _L.muser_cuda_decode_last_plan(self.ctx._h, C.byref(out))
        return tuple(out)

    def autotune(self, weights, up: Weight | None = None, max_tokens: int = 16) -> None:
        """muser_cuda_decode_autotune: measure the decode kernel's launch plans for one projection or one group of
        projections (and `up` for the fused gate/up form) and keep the fastest per token count.  Load-time work."""
        arr = (C.c_void_p * len(weights))(*[w._h.value for w in weights])
        self.ctx.check(_L.muser_cuda_decode_autotune(self.ctx._h, arr, len(weights), up._h if up is not None else None, max_tokens,
                                                     _stream_ptr(self.ctx.device)))

    def encode_quantized_matmul_rows(self, weights: Weight, rows: torch.Tensor, input: torch.Tensor, output: torch.Tensor,
                                     tokens: int) -> None:
        """weights::matmul_rows: output[t][i] = dot(W_rows[i], x_t); rows int32/uint32 on the device, output f32."""
        self.ctx.check(_L.muser_cuda_quantized_matmul_rows(
            self.ctx._h, weights._h, rows.data_ptr(), rows.numel(), input.data_ptr(), _TORCH_DTYPE[input.dtype],
            output.data_ptr(), tokens, _stream_ptr(self.ctx.device)))
        self.launches += 1

    def encode_lm_head_argmax(self, weights: Weight, input: torch.Tensor, tokens: int, logits: torch.Tensor | None = None,
                              norm_weight=None, norm_eps=0.0, out_scale=1.0, softcap=0.0):
        """muser_cuda_lm_head_argmax: the LM head (logit scale and softcap of reference.rs:559-570) with the greedy pick
        fused into the projection kernel.  Returns (index u32 [tokens], value f32 [tokens], nonfinite u32 [tokens]) on
        the device; `logits` ([tokens][n_out], f32 or bf16) also receives the full logits when given."""
        dev = input.device
        index = torch.empty(tokens, dtype=torch.int32, device=dev)
        value = torch.empty(tokens, dtype=torch.float32, device=dev)
        nonfinite = torch.empty(tokens, dtype=torch.int32, device=dev)
        ep = _epilogue(None, None, norm_weight, norm_eps, out_scale, softcap)
        self.ctx.check(_L.muser_cuda_lm_head_argmax(
            self.ctx._h, weights._h, input.data_ptr(), _TORCH_DTYPE[input.dtype], tokens, C.byref(ep) if ep else None,
            logits.data_ptr() if logits is not None else None, _TORCH_DTYPE[logits.dtype] if logits is not None else F32,
            index.data_ptr(), value.data_ptr(), nonfinite.data_ptr(), _stream_ptr(self.ctx.device)))
        self.launches += 2
        return index, value, nonfinite

    def encode_fused_norm_residual_rms_norm(self, hidden: torch.Tensor, src: torch.Tensor, weight1: torch.Tensor, eps1: float,
                                            output: torch.Tensor | None = None, weight2: torch.Tensor | None = None, eps2: float = 0.0) -> None:
        """hidden += rms_norm(src, eps1) * weight1 in place; output = rms_norm(hidden, eps2) * weight2 when given
        (rmsnorm_batch_tail.metal:147-200; reference.rs:466-490).  f32 [tokens][n]."""
        tokens, n = src.shape
        self.ctx.check(_L.muser_cuda_fused_norm_residual_rms_norm(
            self.ctx._h, hidden.data_ptr(), src.data_ptr(), output.data_ptr() if output is not None else None, weight1.data_ptr(),
            weight2.data_ptr() if weight2 is not None else None, tokens, n, C.c_float(eps1), C.c_float(eps2), _stream_ptr(self.ctx.device)))
        self.launches += 1

    def encode_sigmoid_gate(self, x: torch.Tensor, gate: torch.Tensor) -> None:
        """x *= sigmoid(gate) in place (reference.rs:447-455)."""
        self.ctx.check(_L.muser_cuda_sigmoid_gate(self.ctx._h, x.data_ptr(), gate.data_ptr(), x.numel(), _stream_ptr(self.ctx.device)))
        self.launches += 1

    def encode_head_rms_norm(self, x: torch.Tensor, weight: torch.Tensor, eps: float, heads: int) -> None:
        """Per-head rms_norm_mul of x [tokens][heads * head_dim] in place (reference.rs:384-393)."""
        tokens = x.shape[0]
        self.ctx.check(_L.muser_cuda_head_rms_norm(self.ctx._h, x.data_ptr(), weight.data_ptr(), C.c_float(eps), tokens, heads,
                                                   x.shape[1] // heads, _stream_ptr(self.ctx.device)))
        self.launches += 1

    def encode_ffn_gate_up_silu(self, gate_w: Weight, up_w: Weight, input: torch.Tensor, output: torch.Tensor,
                                tokens: int, norm_weight=None, norm_eps=0.0) -> None:
        """output[t][j] = silu(gate_j . x_t) * (up_j . x_t); K-quant (tokens <= 16) or NVFP4 weights."""
        ep = _epilogue(None, None, norm_weight, norm_eps)
        self.ctx.check(_L.muser_cuda_ffn_gate_up_silu(
            self.ctx._h, gate_w._h, up_w._h, input.data_ptr(), _TORCH_DTYPE[input.dtype], output.data_ptr(),
            _TORCH_DTYPE[output.dtype], tokens, C.byref(ep) if ep else None, _stream_ptr(self.ctx.device)))
        self.launches += 2 if gate_w.dtype == NVFP4 else 1

    def encode_nvfp4_ffn_gate_up_silu_requant(self, gate_w: Weight, up_w: Weight, packed: torch.Tensor, scales: torch.Tensor,
                                              tokens: int, out_input_scale_inv: float, out_packed: torch.Tensor | None = None,
                                              out_scales: torch.Tensor | None = None):
        """muser_cuda_nvfp4_ffn_gate_up_silu_requant: silu(gate) * up leaves the GEMM as NVFP4 activations for the down
        projection (codes [tokens][n_out / 2] + swizzled scales), never as numbers."""
        n_out = gate_w.n_out
        if out_packed is None:
            out_packed = torch.empty((tokens, n_out // 2), dtype=torch.uint8, device=packed.device)
        if out_scales is None:
            out_scales = torch.empty(_L.muser_cuda_nvfp4_swizzled_scale_bytes(tokens, n_out), dtype=torch.uint8, device=packed.device)
        self.ctx.check(_L.muser_cuda_nvfp4_ffn_gate_up_silu_requant(
            self.ctx._h, gate_w._h, up_w._h, packed.data_ptr(), scales.data_ptr(), tokens, C.c_float(out_input_scale_inv),
            out_packed.data_ptr(), out_scales.data_ptr(), _stream_ptr(self.ctx.device)))
        self.launches += 1
        return out_packed, out_scales

    def encode_nvfp4_ffn_gate_up_silu_prequant(self, gate_w: Weight, up_w: Weight, packed: torch.Tensor,
                                               scales: torch.Tensor, output: torch.Tensor, columns: int) -> None:
        self.ctx.check(_L.muser_cuda_nvfp4_ffn_gate_up_silu_prequant(
            self.ctx._h, gate_w._h, up_w._h, packed.data_ptr(), scales.data_ptr(), output.data_ptr(),
            _TORCH_DTYPE[output.dtype], columns, _stream_ptr(self.ctx.device)))
        self.launches += 1

    def quantize_nvfp4_activation(self, input: torch.Tensor, input_scale_inv: float, norm_weight=None, norm_eps=0.0,
                                  out=None):
        """(packed codes, swizzled scales) of `input`; with norm_weight, of rms_norm_mul(input, norm_eps, norm_weight).
        `out` = (packed, scales) reuses earlier buffers."""
        tokens, n_in = input.shape
        dev = input.device
        if out is None:
            packed = torch.empty((tokens, n_in // 2), dtype=torch.uint8, device=dev)
            scales = torch.empty((_L.muser_cuda_nvfp4_swizzled_scale_bytes(tokens, n_in),), dtype=torch.uint8, device=dev)
        else:
            packed, scales = out
        if norm_weight is not None:
            self.ctx.check(_L.muser_cuda_rmsnorm_quantize_nvfp4_activation(
                self.ctx._h, input.data_ptr(), _TORCH_DTYPE[input.dtype], tokens, n_in, norm_weight.data_ptr(),
                float(norm_eps), input_scale_inv, packed.data_ptr(), scales.data_ptr(), _stream_ptr(self.ctx.device)))
        else:
            self.ctx.check(_L.muser_cuda_quantize_nvfp4_activation(
                self.ctx._h, input.data_ptr(), _TORCH_DTYPE[input.dtype], tokens, n_in, input_scale_inv, packed.data_ptr(),
                scales.data_ptr(), _stream_ptr(self.ctx.device)))
        self.launches += 1
        return packed, scales

    def encode_nvfp4_matmul(self, weights: Weight, input: torch.Tensor, output: torch.Tensor, columns: int,
                            row_scale=None, residual=None, norm_weight=None, norm_eps=0.0, out_scale=1.0,
                            softcap=0.0) -> None:
        """W4A4 lane: quantizes `input` with the weight's input_scale_inv, then the block-scaled GEMM."""
        ep = _epilogue(row_scale, residual, norm_weight, norm_eps, out_scale, softcap)
        self.ctx.check(_L.muser_cuda_nvfp4_matmul(
            self.ctx._h, weights._h, input.data_ptr(), _TORCH_DTYPE[input.dtype], output.data_ptr(),
            _TORCH_DTYPE[output.dtype], columns, C.byref(ep) if ep else None, _stream_ptr(self.ctx.device)))
        self.launches += 2

    def encode_nvfp4_prequant(self, weights: Weight, packed: torch.Tensor, scales: torch.Tensor, output: torch.Tensor,
                              columns: int, row_scale=None, residual=None) -> None:
        ep = _epilogue(row_scale, residual)
        self.ctx.check(_L.muser_cuda_nvfp4_matmul_prequant(
            self.ctx._h, weights._h, packed.data_ptr(), scales.data_ptr(), output.data_ptr(),
            _TORCH_DTYPE[output.dtype], columns, C.byref(ep) if ep else None, _stream_ptr(self.ctx.device)))
        self.launches += 1

    def encode_nvfp4_group_prequant(self, weights, packed: torch.Tensor, scales: torch.Tensor, outputs, columns: int) -> None:
        """muser_cuda_nvfp4_matmul_group_prequant: 2..4 NVFP4 projections of the same quantized activations (q | k | v)
        in one launch; every output carries the bits encode_nvfp4_prequant gives for its weight."""
        n = len(weights)
        ws = (C.c_void_p * n)(*[w._h.value for w in weights])
        ys = (C.c_void_p * n)(*[y.data_ptr() for y in outputs])
        self.ctx.check(_L.muser_cuda_nvfp4_matmul_group_prequant(
            self.ctx._h, ws, n, packed.data_ptr(), scales.data_ptr(), ys, _TORCH_DTYPE[outputs[0].dtype], columns,
            _stream_ptr(self.ctx.device)))
        self.launches += 1


def fp4_peak_tflops(ctx: Context, iters: int = 20000, reps: int = 3) -> float:
    """Dense block-scaled FP4 tensor throughput of this GPU (TFLOP/s), from muser_cuda_fp4_peak_probe."""
    flops = C.c_double()
    best = 0.0
    for _ in range(reps + 1):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ctx.check(_L.muser_cuda_fp4_peak_probe(ctx._h, iters, C.byref(flops), _stream_ptr(ctx.device)))
        e1.record()
        torch.cuda.synchronize()
        best = max(best, flops.value / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    ctx.sync_status()
    return best


def fp4_pipe_probe_us(ctx: Context, mode: int, iters: int = 20000, load_kib: int = 0, random_data: bool = False) -> float:
    """Microseconds of one muser_cuda_fp4_pipe_probe kernel (second of two runs); divide by `iters` for one slab."""
    for _ in range(2):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ctx.check(_L.muser_cuda_fp4_pipe_probe(ctx._h, mode, iters, load_kib, int(random_data), _stream_ptr(ctx.device)))
        e1.record()
        torch.cuda.synchronize()
    ctx.sync_status()
    return e0.elapsed_time(e1) * 1e3


def f16_mma_cycles(ctx: Context, n_cols: int, iters: int = 2000) -> float:
    """SM cycles per tcgen05.mma kind::f16 (128 x n_cols x 16) issued back to back (muser_cuda_f16_mma_probe)."""
    out = C.c_double()
    ctx.check(_L.muser_cuda_f16_mma_probe(ctx._h, n_cols, iters, C.byref(out)))
    ctx.check(_L.muser_cuda_f16_mma_probe(ctx._h, n_cols, iters, C.byref(out)))  # second run: warm
    ctx.sync_status()
    return out.value


def nvfp4_matmul_static(weights: Weight, input: torch.Tensor, output: torch.Tensor, columns: int) -> None:
    """muser_cuda_nvfp4_matmul_static: the W4A4 projection without a context and without any allocation
    (tokens <= 128, n_in <= 32768); scratch lives in the library image.  Enqueued on torch's current stream."""
    st = _L.muser_cuda_nvfp4_matmul_static(weights._h, input.data_ptr(), _TORCH_DTYPE[input.dtype], output.data_ptr(),
                                           _TORCH_DTYPE[output.dtype], columns, _stream_ptr(input.device.index or 0))
    if st != 0:
        raise MuserCudaError(st, (_L.muser_cuda_last_error(None) or b"").decode())


def static_sync_status(device: int = 0) -> None:
    """muser_cuda_static_sync_status: the bounded-wait report of the context-free entry point above."""
    st = _L.muser_cuda_static_sync_status(device, _stream_ptr(device))
    if st != 0:
        raise MuserCudaError(st, (_L.muser_cuda_last_error(None) or b"").decode())


def matmul(ctx: Context, w: Weight, x: np.ndarray, n_tokens: int, out: np.ndarray | None = None) -> np.ndarray:
    """weights::matmul (weights.rs:398): host f32 slices in and out, the device path in between."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(n_tokens, w.n_in)
    if out is None:
        out = np.empty((n_tokens, w.n_out), dtype=np.float32)
    ctx.check(_L.muser_cuda_matmul_host(ctx._h, w._h, x.ctypes.data, n_tokens, out.ctypes.data))
    return out


def matmul_enqueue(ctx: Context, w: Weight, x_ptr: int, n_tokens: int, out_ptr: int, stream: int) -> None:
    """muser_cuda_matmul_host_enqueue: weights::matmul on host f32 buffers (given as addresses, ideally of pinned memory)
    without the wait; ctx.sync_status() on the same stream completes the step."""
    ctx.check(_L.muser_cuda_matmul_host_enqueue(ctx._h, w._h, x_ptr, n_tokens, out_ptr, stream))


def host_groups(groups):
    """A decode step's call list for matmul_groups_enqueue, built once: `groups` is a sequence of
    (weights, x_host_address, tokens, [y_host_addresses]) with 1..4 weights that read the same x."""
    arr = (_lib.HostGroup * len(groups))()
    for g, (weights, x_ptr, tokens, y_ptrs) in zip(arr, groups):
        for i, (w, y) in enumerate(zip(weights, y_ptrs)):
            g.w[i], g.y_host[i] = w._h.value, y
        g.x_host, g.n_items, g.tokens = x_ptr, len(weights), tokens
    return arr


def matmul_groups_enqueue(ctx: Context, groups, stream: int) -> None:
    """muser_cuda_matmul_host_groups_enqueue: a whole step's grouped projections through host f32 buffers in one call;
    `groups` from host_groups().  ctx.sync_status() on the same stream completes the step."""
    ctx.check(_L.muser_cuda_matmul_host_groups_enqueue(ctx._h, groups, len(groups), stream))


def unswizzle_scales(swizzled: torch.Tensor, rows: int, n_in: int) -> torch.Tensor:
    """Logical [rows][n_in/16] view of the [rows/128][n_in/64][32][4][4] scale plane (test helper)."""
    groups = n_in // 16
    kt = (n_in + 63) // 64
    r = torch.arange(rows, device=swizzled.device)[:, None]
    g = torch.arange(groups, device=swizzled.device)[None, :]
    off = (r // 128) * (kt * 512) + (g // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + g % 4
    return swizzled.reshape(-1)[off]
