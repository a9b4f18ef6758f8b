//! Raw declarations of `include/muser_cuda.h`, one per entry point, in the header's order.
//! Not compiled in this repository's environment; kept in step with the header by a test that compares names and
//! argument counts.
#![allow(non_camel_case_types)]

use std::os::raw::{c_char, c_int, c_void};

pub const MUSER_CUDA_ABI_VERSION: u32 = 3;

pub const MUSER_DTYPE_F32: u32 = 0;
pub const MUSER_DTYPE_F16: u32 = 1;
pub const MUSER_DTYPE_Q4_K: u32 = 12;
pub const MUSER_DTYPE_Q5_K: u32 = 13;
pub const MUSER_DTYPE_Q6_K: u32 = 14;
pub const MUSER_DTYPE_BF16: u32 = 30;
pub const MUSER_DTYPE_NVFP4_E2M1: u32 = 1000;
pub const MUSER_DTYPE_F8_E4M3FN: u32 = 1001;

pub const MUSER_SHARD_NONE: u32 = 0;
pub const MUSER_SHARD_ROWS: u32 = 1;
pub const MUSER_SHARD_K: u32 = 2;

pub const MUSER_TUNE_TC_MIN_TOKENS_Q4_K: u32 = 1;
pub const MUSER_TUNE_TC_MIN_TOKENS_Q6_K: u32 = 2;
pub const MUSER_TUNE_TC_MIN_ROWS: u32 = 3;
pub const MUSER_TUNE_DECODE_WARPS: u32 = 8;
pub const MUSER_TUNE_DECODE_KSPLIT: u32 = 9;
pub const MUSER_TUNE_DECODE_RING: u32 = 10;
pub const MUSER_TUNE_ONESHOT_MAX_BYTES: u32 = 11;
pub const MUSER_TUNE_DECODE_WSPLIT: u32 = 12;
pub const MUSER_TUNE_NVFP4_PAIR: u32 = 13;
pub const MUSER_TUNE_HOST_DIRECT_OUTPUT: u32 = 14;
pub const MUSER_TUNE_NVFP4_GROUP_M: u32 = 15;

pub const MUSER_CUDA_COMM_ID_BYTES: usize = 128;

#[repr(C)]
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum muser_cuda_status {
    MUSER_CUDA_OK = 0,
    MUSER_CUDA_BAD_ARG = 1,
    MUSER_CUDA_BAD_SHAPE = 2,
    MUSER_CUDA_BAD_ALIGN = 3,
    MUSER_CUDA_UNSUPPORTED_DTYPE = 4,
    MUSER_CUDA_NAN_SCALE = 5,
    MUSER_CUDA_ERROR = 6,
    MUSER_CUDA_NCCL_ERROR = 7,
    MUSER_CUDA_TIMEOUT = 8,
    MUSER_CUDA_WORKSPACE_TOO_SMALL = 9,
}

#[repr(C)]
pub struct muser_cuda_ctx {
    _opaque: [u8; 0],
}
#[repr(C)]
pub struct muser_cuda_weight {
    _opaque: [u8; 0],
}

#[repr(C)]
#[derive(Debug, Clone, Copy, Default)]
pub struct muser_cuda_shard {
    pub rank: u32,
    pub world: u32,
    pub axis: u32,
}

#[repr(C)]
#[derive(Debug, Clone, Copy)]
pub struct muser_cuda_epilogue {
    pub row_scale: *const f32,
    pub residual: *const c_void,
    pub swiglu: u32,
    pub norm_eps: f32,
    pub norm_weight: *const f32,
    pub out_scale: f32,
    pub softcap: f32,
    pub all_reduce: u32,
}

#[repr(C)]
#[derive(Debug, Clone, Copy, Default)]
pub struct muser_cuda_weight_info {
    pub dtype: u32,
    pub shard_axis: u32,
    pub shard_rank: u32,
    pub shard_world: u32,
    pub n_in: u64,
    pub n_out: u64,
    pub n_in_full: u64,
    pub n_out_full: u64,
    pub image_bytes: u64,
    pub image_hash: u64,
    pub scale2: f32,
    pub input_scale_inv: f32,
    pub has_input_scale_inv: u32,
    pub reserved: u32,
}

#[repr(C)]
#[derive(Debug, Clone, Copy)]
pub struct muser_cuda_group_item {
    pub w: *const muser_cuda_weight,
    pub y: *mut c_void,
    pub y_dtype: u32,
    pub reserved: u32,
    pub epilogue: *const muser_cuda_epilogue,
}

#[repr(C)]
#[derive(Debug, Clone, Copy)]
pub struct muser_cuda_host_group {
    pub w: [*const muser_cuda_weight; 4],
    pub y_host: [*mut f32; 4],
    pub x_host: *const f32,
    pub n_items: u32,
    pub tokens: u32,
}

extern "C" {
    pub fn muser_cuda_abi_version() -> u32;
    pub fn muser_cuda_supports_projection(ggml_type: u32) -> c_int;
    pub fn muser_cuda_ctx_create(device: c_int, workspace_bytes: usize, out: *mut *mut muser_cuda_ctx) -> muser_cuda_status;
    pub fn muser_cuda_ctx_destroy(ctx: *mut muser_cuda_ctx);
    pub fn muser_cuda_last_error(ctx: *const muser_cuda_ctx) -> *const c_char;
    pub fn muser_cuda_sync_status(ctx: *mut muser_cuda_ctx, stream: *mut c_void) -> muser_cuda_status;
    pub fn muser_cuda_tuning_set(ctx: *mut muser_cuda_ctx, key: u32, value: u32) -> muser_cuda_status;
    pub fn muser_cuda_weight_repack(
        ctx: *mut muser_cuda_ctx,
        ggml_type: u32,
        host_blocks: *const u8,
        host_block_scales: *const u8,
        scale2: f32,
        has_input_scale_inv: c_int,
        input_scale_inv: f32,
        n_in: u64,
        n_out: u64,
        shard: *const muser_cuda_shard,
        out: *mut *mut muser_cuda_weight,
    ) -> muser_cuda_status;
    pub fn muser_cuda_weight_repack_device(
        ctx: *mut muser_cuda_ctx,
        ggml_type: u32,
        dev_blocks: *const u8,
        dev_block_scales: *const u8,
        scale2: f32,
        has_input_scale_inv: c_int,
        input_scale_inv: f32,
        n_in: u64,
        n_out: u64,
        shard: *const muser_cuda_shard,
        stream: *mut c_void,
        out: *mut *mut muser_cuda_weight,
    ) -> muser_cuda_status;
    pub fn muser_cuda_weight_free(w: *mut muser_cuda_weight);
    pub fn muser_cuda_weight_info_get(w: *const muser_cuda_weight, out: *mut muser_cuda_weight_info) -> muser_cuda_status;
    pub fn muser_cuda_dequant(ctx: *mut muser_cuda_ctx, w: *const muser_cuda_weight, out: *mut f32, stream: *mut c_void) -> muser_cuda_status;
    pub fn muser_cuda_quantized_matmul(
        ctx: *mut muser_cuda_ctx,
        w: *const muser_cuda_weight,
        x: *const c_void,
        x_dtype: u32,
        y: *mut c_void,
        y_dtype: u32,
        tokens: u32,
        epilogue: *const muser_cuda_epilogue,
        stream: *mut c_void,
    ) -> muser_cuda_status;
    pub fn muser_cuda_quantized_matmul_group(
        ctx: *mut muser_cuda_ctx,
        items: *const muser_cuda_group_item,
        n_items: u32,
        x: *const c_void,
        x_dtype: u32,
        tokens: u32,
        stream: *mut c_void,
    ) -> muser_cuda_status;
    pub fn muser_cuda_decode_autotune(
        ctx: *mut muser_cuda_ctx,
        weights: *const *const muser_cuda_weight,
        n_weights: u32,
        w_up: *const muser_cuda_weight,
        max_tokens: u32,
        stream: *mut c_void,
    ) -> muser_cuda_status;
    pub fn muser_cuda_decode_last_plan(ctx: *const muser_cuda_ctx, out: *mut u32) -> muser_cuda_status;
    pub fn muser_cuda_quantized_matmul_rows(
        ctx: *mut muser_cuda_ctx,
        w: *const muser_cuda_weight,
        rows: *const u32,
        n_rows: u32,
        x: *const c_void,
        x_dtype: u32,
        y: *mut f32,
        tokens: u32,
        stream: *mut c_void,
    ) -> muser_cuda_status;
    pub fn muser_cuda_lm_head_argmax(
        ctx: *mut muser_cuda_ctx,
        w: *const muser_cuda_weight,
        x: *const c_void,
        x_dtype: u32,
        tokens: u32,
        epilogue: *const muser_cuda_epilogue,
        logits: *mut c_void,
        logits_dtype: u32,
        out_index: *mut u32,
        out_value: *mut f32,
        out_nonfinite: *mut u32,
        stream: *mut c_void,
    ) -> muser_cuda_status;
    pub fn muser_cuda_ffn_gate_up_silu(
        ctx: *mut muser_cuda_ctx,
        w_gate: *const muser_cuda_weight,
        w_up: *const muser_cuda_weight,
        x: *const c_void,
        x_dtype: u32,
        y: *mut c_void,
        y_dtype: u32,
        tokens: u32,
        epilogue: *const muser_cuda_epilogue,
        stream: *mut c_void,
    ) -> muser_cuda_status;
    pub fn muser_cuda_quantize_nvfp4_activation(
        ctx: *mut muser_cuda_ctx,
        x: *const c_void,
        x_dtype: u32,
        tokens: u32,
        n_in: u64,
        input_scale_inv: f32,
        packed: *mut u8,
        scales_swizzled: *mut u8,
        stream: *mut c_void,
    ) -> muser_cuda_status;
    pub fn muser_cuda_nvfp4_swizzled_scale_bytes(rows: u64, n_in: u64) -> usize;
    pub fn muser_cuda_rmsnorm_quantize_nvfp4_activation(
        ctx: *mut muser_cuda_ctx,
        x: *const c_void,
        x_dtype: u32,
        tokens: u32,
        n_in: u64,
        norm_weight: *const f32,
        norm_eps: f32,
        input_scale_inv: f32,
        packed: *mut u8,
        scales_swizzled: *mut u8,
        stream: *mut c_void,
    ) -> muser_cuda_status;
    pub fn muser_cuda_nvfp4_matmul(
        ctx: *mut muser_cuda_ctx,
        w: *const muser_cuda_weight,
        x: *const c_void,
        x_dtype: u32,
        y: *mut c_void,
        y_dtype: u32,
        tokens: u32,
        epilogue: *const muser_cuda_epilogue,
        stream: *mut c_void,
    ) -> muser_cuda_status;
    pub fn muser_cuda_nvfp4_matmul_prequant(
        ctx: *mut muser_cuda_ctx,
        w: *const muser_cuda_weight,
        x_packed: *const u8,
        x_scales_swizzled: *const u8,
        y: *mut c_void,
        y_dtype: u32,
        tokens: u32,
        epilogue: *const muser_cuda_epilogue,
        stream: *mut c_void,
    ) -> muser_cuda_status;
    pub fn muser_cuda_nvfp4_matmul_group_prequant(
        ctx: *mut muser_cuda_ctx,
        weights: *const *const muser_cuda_weight,
        n_weights: u32,
        x_packed: *const u8,
        x_scales_swizzled: *const u8,
        outputs: *const *mut c_void,
        y_dtype: u32,
        tokens: u32,
        stream: *mut c_void,
    ) -> muser_cuda_status;
    pub fn muser_cuda_nvfp4_ffn_gate_up_silu_prequant(
        ctx: *mut muser_cuda_ctx,
        w_gate: *const muser_cuda_weight,
        w_up: *const muser_cuda_weight,
        x_packed: *const u8,
        x_scales_swizzled: *const u8,
        y: *mut c_void,
        y_dtype: u32,
        tokens: u32,
        stream: *mut c_void,
    ) -> muser_cuda_status;
    pub fn muser_cuda_nvfp4_ffn_gate_up_silu_requant(
        ctx: *mut muser_cuda_ctx,
        w_gate: *const muser_cuda_weight,
        w_up: *const muser_cuda_weight,
        x_packed: *const u8,
        x_scales_swizzled: *const u8,
        tokens: u32,
        out_input_scale_inv: f32,
        out_packed: *mut u8,
        out_scales_swizzled: *mut u8,
        stream: *mut c_void,
    ) -> muser_cuda_status;
    pub fn muser_cuda_nvfp4_matmul_static(
        w: *const muser_cuda_weight,
        x: *const c_void,
        x_dtype: u32,
        y: *mut c_void,
        y_dtype: u32,
        tokens: u32,
        stream: *mut c_void,
    ) -> muser_cuda_status;
    pub fn muser_cuda_static_sync_status(device: c_int, stream: *mut c_void) -> muser_cuda_status;
    pub fn muser_cuda_fp4_peak_probe(ctx: *mut muser_cuda_ctx, iters: u32, flops: *mut f64, stream: *mut c_void) -> muser_cuda_status;
    pub fn muser_cuda_fp4_pipe_probe(ctx: *mut muser_cuda_ctx, mode: u32, iters: u32, load_kib: u32, random_data: u32, stream: *mut c_void) -> muser_cuda_status;
    pub fn muser_cuda_f16_mma_probe(ctx: *mut muser_cuda_ctx, n_cols: u32, iters: u32, cycles_per_mma: *mut f64) -> muser_cuda_status;
    pub fn muser_cuda_wait_probe(ctx: *mut muser_cuda_ctx, polls: u32, stream: *mut c_void) -> muser_cuda_status;
    pub fn muser_cuda_comm_unique_id(out: *mut u8, out_bytes: usize) -> muser_cuda_status;
    pub fn muser_cuda_ctx_comm_init(ctx: *mut muser_cuda_ctx, id: *const u8, rank: u32, world: u32, stream: *mut c_void) -> muser_cuda_status;
    pub fn muser_cuda_ctx_comm_attach(ctx: *mut muser_cuda_ctx, nccl_comm: *mut c_void, rank: u32, world: u32, stream: *mut c_void) -> muser_cuda_status;
    pub fn muser_cuda_ctx_comm_has_oneshot(ctx: *const muser_cuda_ctx) -> c_int;
    pub fn muser_cuda_all_reduce(ctx: *mut muser_cuda_ctx, buf: *mut c_void, count: u64, dtype: u32, stream: *mut c_void) -> muser_cuda_status;
    pub fn muser_cuda_matmul_host(ctx: *mut muser_cuda_ctx, w: *const muser_cuda_weight, x_host: *const f32, tokens: u32, y_host: *mut f32) -> muser_cuda_status;
    pub fn muser_cuda_matmul_host_enqueue(
        ctx: *mut muser_cuda_ctx,
        w: *const muser_cuda_weight,
        x_host: *const f32,
        tokens: u32,
        y_host: *mut f32,
        stream: *mut c_void,
    ) -> muser_cuda_status;
    pub fn muser_cuda_fused_norm_residual_rms_norm(
        ctx: *mut muser_cuda_ctx,
        hidden: *mut f32,
        src: *const f32,
        output: *mut f32,
        weight1: *const f32,
        weight2: *const f32,
        tokens: u32,
        n: u32,
        eps1: f32,
        eps2: f32,
        stream: *mut c_void,
    ) -> muser_cuda_status;
    pub fn muser_cuda_sigmoid_gate(ctx: *mut muser_cuda_ctx, x: *mut f32, gate: *const f32, count: u64, stream: *mut c_void) -> muser_cuda_status;
    pub fn muser_cuda_head_rms_norm(ctx: *mut muser_cuda_ctx, x: *mut f32, weight: *const f32, eps: f32, tokens: u32, heads: u32, head_dim: u32, stream: *mut c_void) -> muser_cuda_status;
    pub fn muser_cuda_matmul_host_groups_enqueue(ctx: *mut muser_cuda_ctx, groups: *const muser_cuda_host_group, n_groups: u32, stream: *mut c_void) -> muser_cuda_status;
}
