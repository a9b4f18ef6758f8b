"""ctypes binding of libmuser_cuda.so (include/muser_cuda.h), one Python function per C entry point.

The library is the product; there is no fallback.  Importing this module fails loudly when the
shared object has not been built (run `python -m muser_b200.build` or `__graft_entry__.build()`).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libmuser_cuda.so"

F32, F16, Q4_K, Q5_K, Q6_K, BF16, NVFP4 = 0, 1, 12, 13, 14, 30, 1000
SHARD_NONE, SHARD_ROWS, SHARD_K = 0, 1, 2
TUNE_TC_MIN_TOKENS_Q4_K, TUNE_TC_MIN_TOKENS_Q6_K, TUNE_TC_MIN_ROWS = 1, 2, 3
TUNE_DECODE_WARPS, TUNE_DECODE_KSPLIT, TUNE_DECODE_RING, TUNE_ONESHOT_MAX_BYTES, TUNE_DECODE_WSPLIT = 8, 9, 10, 11, 12
TUNE_NVFP4_PAIR = 13
TUNE_HOST_DIRECT_OUTPUT = 14
TUNE_NVFP4_GROUP_M = 15
STATUS_NAMES = ["OK", "BAD_ARG", "BAD_SHAPE", "BAD_ALIGN", "UNSUPPORTED_DTYPE", "NAN_SCALE", "CUDA_ERROR", "NCCL_ERROR",
                "TIMEOUT", "WORKSPACE_TOO_SMALL"]

# every symbol include/muser_cuda.h declares
EXPORTS = [
    "muser_cuda_abi_version", "muser_cuda_supports_projection", "muser_cuda_ctx_create", "muser_cuda_ctx_destroy",
    "muser_cuda_last_error", "muser_cuda_sync_status", "muser_cuda_weight_repack", "muser_cuda_weight_repack_device",
    "muser_cuda_weight_free", "muser_cuda_weight_info_get", "muser_cuda_dequant", "muser_cuda_quantized_matmul",
    "muser_cuda_ffn_gate_up_silu", "muser_cuda_quantize_nvfp4_activation", "muser_cuda_nvfp4_swizzled_scale_bytes",
    "muser_cuda_nvfp4_matmul", "muser_cuda_nvfp4_matmul_prequant", "muser_cuda_nvfp4_matmul_group_prequant", "muser_cuda_matmul_host",
    "muser_cuda_nvfp4_matmul_static", "muser_cuda_fp4_peak_probe", "muser_cuda_fp4_pipe_probe", "muser_cuda_lm_head_argmax", "muser_cuda_matmul_host_groups_enqueue", "muser_cuda_fused_norm_residual_rms_norm",
    "muser_cuda_sigmoid_gate", "muser_cuda_head_rms_norm", "muser_cuda_nvfp4_ffn_gate_up_silu_requant", "muser_cuda_nvfp4_ffn_gate_up_silu_prequant",
    "muser_cuda_rmsnorm_quantize_nvfp4_activation", "muser_cuda_tuning_set", "muser_cuda_f16_mma_probe", "muser_cuda_quantized_matmul_rows",
    "muser_cuda_static_sync_status", "muser_cuda_wait_probe", "muser_cuda_quantized_matmul_group",
    "muser_cuda_matmul_host_enqueue", "muser_cuda_comm_unique_id", "muser_cuda_ctx_comm_init", "muser_cuda_ctx_comm_attach",
    "muser_cuda_ctx_comm_has_oneshot", "muser_cuda_all_reduce", "muser_cuda_decode_autotune", "muser_cuda_decode_last_plan",
]


class Shard(C.Structure):
    _fields_ = [("rank", C.c_uint32), ("world", C.c_uint32), ("axis", C.c_uint32)]


class Epilogue(C.Structure):
    _fields_ = [("row_scale", C.c_void_p), ("residual", C.c_void_p), ("swiglu", C.c_uint32), ("norm_eps", C.c_float),
                ("norm_weight", C.c_void_p), ("out_scale", C.c_float), ("softcap", C.c_float), ("all_reduce", C.c_uint32)]


class GroupItem(C.Structure):
    _fields_ = [("w", C.c_void_p), ("y", C.c_void_p), ("y_dtype", C.c_uint32), ("reserved", C.c_uint32),
                ("epilogue", C.POINTER(Epilogue))]


class HostGroup(C.Structure):
    _fields_ = [("w", C.c_void_p * 4), ("y_host", C.c_void_p * 4), ("x_host", C.c_void_p), ("n_items", C.c_uint32), ("tokens", C.c_uint32)]


class WeightInfo(C.Structure):
    _fields_ = [
        ("dtype", C.c_uint32), ("shard_axis", C.c_uint32), ("shard_rank", C.c_uint32), ("shard_world", C.c_uint32),
        ("n_in", C.c_uint64), ("n_out", C.c_uint64), ("n_in_full", C.c_uint64), ("n_out_full", C.c_uint64),
        ("image_bytes", C.c_uint64), ("image_hash", C.c_uint64), ("scale2", C.c_float), ("input_scale_inv", C.c_float),
        ("has_input_scale_inv", C.c_uint32), ("reserved", C.c_uint32),
    ]


class MuserCudaError(RuntimeError):
    def __init__(self, status: int, message: str):
        name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)
        super().__init__(f"muser-cuda {name}: {message}")
        self.status = status
        self.status_name = name


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA library has not been built and there is no CPU fallback. "
            "Run `python -m muser_b200.build`.")
    lib = C.CDLL(str(LIB_PATH))
    vp, u32, u64, f32, i32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_float, C.c_int
    sig = {
        "muser_cuda_abi_version": (u32, []),
        "muser_cuda_supports_projection": (i32, [u32]),
        "muser_cuda_ctx_create": (i32, [i32, C.c_size_t, C.POINTER(vp)]),
        "muser_cuda_ctx_destroy": (None, [vp]),
        "muser_cuda_last_error": (C.c_char_p, [vp]),
        "muser_cuda_sync_status": (i32, [vp, vp]),
        "muser_cuda_weight_repack": (i32, [vp, u32, vp, vp, f32, i32, f32, u64, u64, C.POINTER(Shard), C.POINTER(vp)]),
        "muser_cuda_weight_repack_device": (i32, [vp, u32, vp, vp, f32, i32, f32, u64, u64, C.POINTER(Shard), vp, C.POINTER(vp)]),
        "muser_cuda_weight_free": (None, [vp]),
        "muser_cuda_weight_info_get": (i32, [vp, C.POINTER(WeightInfo)]),
        "muser_cuda_dequant": (i32, [vp, vp, vp, vp]),
        "muser_cuda_quantized_matmul": (i32, [vp, vp, vp, u32, vp, u32, u32, C.POINTER(Epilogue), vp]),
        "muser_cuda_ffn_gate_up_silu": (i32, [vp, vp, vp, vp, u32, vp, u32, u32, C.POINTER(Epilogue), vp]),
        "muser_cuda_quantize_nvfp4_activation": (i32, [vp, vp, u32, u32, u64, f32, vp, vp, vp]),
        "muser_cuda_nvfp4_swizzled_scale_bytes": (C.c_size_t, [u64, u64]),
        "muser_cuda_nvfp4_matmul": (i32, [vp, vp, vp, u32, vp, u32, u32, C.POINTER(Epilogue), vp]),
        "muser_cuda_nvfp4_matmul_prequant": (i32, [vp, vp, vp, vp, vp, u32, u32, C.POINTER(Epilogue), vp]),
        "muser_cuda_nvfp4_matmul_group_prequant": (i32, [vp, C.POINTER(vp), u32, vp, vp, C.POINTER(vp), u32, u32, vp]),
        "muser_cuda_matmul_host": (i32, [vp, vp, vp, u32, vp]),
        "muser_cuda_matmul_host_enqueue": (i32, [vp, vp, vp, u32, vp, vp]),
        "muser_cuda_comm_unique_id": (i32, [vp, C.c_size_t]),
        "muser_cuda_ctx_comm_init": (i32, [vp, vp, u32, u32, vp]),
        "muser_cuda_ctx_comm_attach": (i32, [vp, vp, u32, u32, vp]),
        "muser_cuda_ctx_comm_has_oneshot": (i32, [vp]),
        "muser_cuda_all_reduce": (i32, [vp, vp, u64, u32, vp]),
        "muser_cuda_decode_autotune": (i32, [vp, C.POINTER(vp), u32, vp, u32, vp]),
        "muser_cuda_decode_last_plan": (i32, [vp, C.POINTER(u32 * 4)]),
        "muser_cuda_nvfp4_matmul_static": (i32, [vp, vp, u32, vp, u32, u32, vp]),
        "muser_cuda_fp4_peak_probe": (i32, [vp, u32, C.POINTER(C.c_double), vp]),
        "muser_cuda_fp4_pipe_probe": (i32, [vp, u32, u32, u32, u32, vp]),
        "muser_cuda_nvfp4_ffn_gate_up_silu_requant": (i32, [vp, vp, vp, vp, vp, u32, C.c_float, vp, vp, vp]),
        "muser_cuda_matmul_host_groups_enqueue": (i32, [vp, vp, u32, vp]),
        "muser_cuda_fused_norm_residual_rms_norm": (i32, [vp, vp, vp, vp, vp, vp, u32, u32, C.c_float, C.c_float, vp]),
        "muser_cuda_sigmoid_gate": (i32, [vp, vp, vp, C.c_uint64, vp]),
        "muser_cuda_head_rms_norm": (i32, [vp, vp, vp, C.c_float, u32, u32, u32, vp]),
        "muser_cuda_lm_head_argmax": (i32, [vp, vp, vp, u32, u32, vp, vp, u32, vp, vp, vp, vp]),
        "muser_cuda_nvfp4_ffn_gate_up_silu_prequant": (i32, [vp, vp, vp, vp, vp, vp, u32, u32, vp]),
        "muser_cuda_tuning_set": (i32, [vp, u32, u32]),
        "muser_cuda_quantized_matmul_rows": (i32, [vp, vp, vp, u32, vp, u32, vp, u32, vp]),
        "muser_cuda_f16_mma_probe": (i32, [vp, u32, u32, C.POINTER(C.c_double)]),
        "muser_cuda_static_sync_status": (i32, [i32, vp]),
        "muser_cuda_wait_probe": (i32, [vp, u32, vp]),
        "muser_cuda_quantized_matmul_group": (i32, [vp, C.POINTER(GroupItem), u32, vp, u32, u32, vp]),
        "muser_cuda_rmsnorm_quantize_nvfp4_activation": (i32, [vp, vp, u32, u32, u64, vp, f32, f32, vp, vp, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)  # AttributeError here means the library does not export what the header declares
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()
