//! Safe wrappers over `libmuser_cuda`'s C ABI, shaped like the engine's Metal backend so that a forward-graph
//! driver can select this backend the way it selects Metal (`SessionBackend`, crates/muser-engine/src/api.rs:626-631).
//!
//! NOT COMPILED in this repository's environment (no Rust toolchain there).  The raw declarations live in
//! [`ffi`]; this file gives them the reference's names and argument meaning:
//!
//! | here                                         | reference                                                              |
//! |----------------------------------------------|------------------------------------------------------------------------|
//! | `CudaContext::new`, `wait_for_completion`    | `MetalContext::new`, `wait_for_completion` (src/metal/context.rs)        |
//! | `CudaKernels::supports_projection`           | `MetalKernels::supports_projection` (src/metal/encode.rs:370-385)        |
//! | `CudaWeight::from_view`                      | the loader's tensor binding (src/weights.rs:171-373)                     |
//! | `CudaKernels::encode_quantized_matmul`       | `MetalKernels::encode_quantized_matmul` (src/metal/encode/qkv.rs:414)    |
//! | `CudaKernels::encode_quantized_decode_group` | `encode_quantized_decode_group` (src/metal/encode/qkv.rs:234-281)        |
//! | `CudaKernels::encode_ffn_gate_up_silu`       | `encode_ffn_q4k_gate_up_silu_4r2s` (src/metal/encode/ffn.rs:10-19)       |
//! | `CudaKernels::encode_nvfp4_matmul`           | `MetalKernels::encode_nvfp4_matmul` (src/metal/encode/qkv.rs:128-227)    |
//! | `matmul`                                     | `weights::matmul` (src/weights.rs:398-421)                               |
//!
//! Where the reference's encoders `debug_assert!` and return `()`, these return `Result`: the library validates
//! every call on the host and reports a status instead of aborting.

pub mod ffi;

use std::ffi::{c_void, CStr};
use std::marker::PhantomData;
use std::ptr;

/// `GgmlType` discriminants the backend understands (src/gguf/types.rs:9-39).
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
#[repr(u32)]
pub enum Dtype {
    F32 = ffi::MUSER_DTYPE_F32,
    F16 = ffi::MUSER_DTYPE_F16,
    Q4K = ffi::MUSER_DTYPE_Q4_K,
    Q5K = ffi::MUSER_DTYPE_Q5_K,
    Q6K = ffi::MUSER_DTYPE_Q6_K,
    Bf16 = ffi::MUSER_DTYPE_BF16,
    Nvfp4E2m1 = ffi::MUSER_DTYPE_NVFP4_E2M1,
}

#[derive(Debug, thiserror::Error)]
pub enum CudaError {
    #[error("bad argument: {0}")]
    BadArg(String),
    #[error("unsupported shape: {0}")]
    BadShape(String),
    #[error("misaligned device pointer: {0}")]
    BadAlign(String),
    #[error("unsupported dtype: {0}")]
    UnsupportedDtype(String),
    #[error("NaN scale: {0}")]
    NanScale(String),
    #[error("CUDA: {0}")]
    Command(String),
    #[error("NCCL: {0}")]
    Nccl(String),
    /// A bounded device-side wait gave up: the counterpart of `MetalError::Deadline` (src/metal/context.rs:8-30).
    #[error("deadline: {0}")]
    Deadline(String),
    #[error("workspace too small: {0}")]
    WorkspaceTooSmall(String),
}

pub type Result<T> = std::result::Result<T, CudaError>;

fn check(status: ffi::muser_cuda_status, ctx: *const ffi::muser_cuda_ctx) -> Result<()> {
    use ffi::muser_cuda_status::*;
    if status == MUSER_CUDA_OK {
        return Ok(());
    }
    // SAFETY: last_error returns a NUL-terminated string owned by the library (or by the context).
    let text = unsafe { CStr::from_ptr(ffi::muser_cuda_last_error(ctx)) }.to_string_lossy().into_owned();
    Err(match status {
        MUSER_CUDA_OK => unreachable!(),
        MUSER_CUDA_BAD_ARG => CudaError::BadArg(text),
        MUSER_CUDA_BAD_SHAPE => CudaError::BadShape(text),
        MUSER_CUDA_BAD_ALIGN => CudaError::BadAlign(text),
        MUSER_CUDA_UNSUPPORTED_DTYPE => CudaError::UnsupportedDtype(text),
        MUSER_CUDA_NAN_SCALE => CudaError::NanScale(text),
        MUSER_CUDA_ERROR => CudaError::Command(text),
        MUSER_CUDA_NCCL_ERROR => CudaError::Nccl(text),
        MUSER_CUDA_TIMEOUT => CudaError::Deadline(text),
        MUSER_CUDA_WORKSPACE_TOO_SMALL => CudaError::WorkspaceTooSmall(text),
    })
}

/// A `cudaStream_t`; null is the default stream.
#[derive(Debug, Clone, Copy)]
pub struct Stream(pub *mut c_void);

impl Default for Stream {
    fn default() -> Self {
        Stream(ptr::null_mut())
    }
}

/// A device allocation the caller owns (the counterpart of `GpuBuffer`): pointer, element type, element count.
#[derive(Debug, Clone, Copy)]
pub struct DeviceSlice<'a> {
    pub ptr: *mut c_void,
    pub dtype: Dtype,
    pub len: usize,
    pub _life: PhantomData<&'a ()>,
}

/// One context per device; not `Sync` (calls on one context come from one thread at a time).
pub struct CudaContext {
    raw: *mut ffi::muser_cuda_ctx,
    pub device: i32,
}

unsafe impl Send for CudaContext {}

impl CudaContext {
    pub fn new(device: i32, workspace_bytes: usize) -> Result<Self> {
        let mut raw = ptr::null_mut();
        // SAFETY: `raw` is a valid out pointer.
        check(unsafe { ffi::muser_cuda_ctx_create(device, workspace_bytes, &mut raw) }, ptr::null())?;
        Ok(Self { raw, device })
    }

    /// Synchronizes `stream` and folds asynchronous faults and device-side give-ups into an error.
    pub fn wait_for_completion(&self, stream: Stream) -> Result<()> {
        check(unsafe { ffi::muser_cuda_sync_status(self.raw, stream.0) }, self.raw)
    }

    pub fn tuning_set(&self, key: u32, value: u32) -> Result<()> {
        check(unsafe { ffi::muser_cuda_tuning_set(self.raw, key, value) }, self.raw)
    }

    /// Joins this context to a tensor-parallel group; `id` comes from [`comm_unique_id`] on rank 0.
    pub fn comm_init(&self, id: &[u8; ffi::MUSER_CUDA_COMM_ID_BYTES], rank: u32, world: u32, stream: Stream) -> Result<()> {
        check(unsafe { ffi::muser_cuda_ctx_comm_init(self.raw, id.as_ptr(), rank, world, stream.0) }, self.raw)
    }

    /// In-place sum over the ranks after a row-parallel projection.
    pub fn all_reduce(&self, buf: DeviceSlice<'_>, stream: Stream) -> Result<()> {
        check(unsafe { ffi::muser_cuda_all_reduce(self.raw, buf.ptr, buf.len as u64, buf.dtype as u32, stream.0) }, self.raw)
    }
}

impl Drop for CudaContext {
    fn drop(&mut self) {
        // SAFETY: created by ctx_create, destroyed once.
        unsafe { ffi::muser_cuda_ctx_destroy(self.raw) }
    }
}

pub fn comm_unique_id() -> Result<[u8; ffi::MUSER_CUDA_COMM_ID_BYTES]> {
    let mut id = [0u8; ffi::MUSER_CUDA_COMM_ID_BYTES];
    check(unsafe { ffi::muser_cuda_comm_unique_id(id.as_mut_ptr(), id.len()) }, ptr::null())?;
    Ok(id)
}

/// The stored tensor as the engine's loader hands it over: the fields of `weights::TensorView`
/// (src/weights.rs:40-48) with the NVFP4 companions of `Nvfp4AuxView` inlined.
pub struct TensorView<'a> {
    pub raw: &'a [u8],
    pub dtype: Dtype,
    pub n_in: usize,
    pub n_out: usize,
    pub block_scales: Option<&'a [u8]>,
    pub scale2: f32,
    pub input_scale_inv: Option<f32>,
}

#[derive(Debug, Clone, Copy, Default)]
pub struct Shard {
    pub rank: u32,
    pub world: u32,
    /// `ffi::MUSER_SHARD_ROWS` (column-parallel) or `ffi::MUSER_SHARD_K` (row-parallel).
    pub axis: u32,
}

/// The repacked device image of one tensor (or of this rank's shard of it).
pub struct CudaWeight {
    raw: *mut ffi::muser_cuda_weight,
}

unsafe impl Send for CudaWeight {}
unsafe impl Sync for CudaWeight {}

impl CudaWeight {
    pub fn from_view(ctx: &CudaContext, view: &TensorView<'_>, shard: Option<Shard>) -> Result<Self> {
        let sh = shard.map(|s| ffi::muser_cuda_shard { rank: s.rank, world: s.world, axis: s.axis });
        let mut raw = ptr::null_mut();
        let status = unsafe {
            ffi::muser_cuda_weight_repack(
                ctx.raw,
                view.dtype as u32,
                view.raw.as_ptr(),
                view.block_scales.map_or(ptr::null(), |s| s.as_ptr()),
                view.scale2,
                view.input_scale_inv.is_some() as i32,
                view.input_scale_inv.unwrap_or(0.0),
                view.n_in as u64,
                view.n_out as u64,
                sh.as_ref().map_or(ptr::null(), |s| s as *const _),
                &mut raw,
            )
        };
        check(status, ctx.raw)?;
        Ok(Self { raw })
    }

    pub fn info(&self) -> ffi::muser_cuda_weight_info {
        let mut info = ffi::muser_cuda_weight_info::default();
        // SAFETY: `self.raw` is a live handle; `info` is a valid out pointer.
        unsafe { ffi::muser_cuda_weight_info_get(self.raw, &mut info) };
        info
    }
}

impl Drop for CudaWeight {
    fn drop(&mut self) {
        unsafe { ffi::muser_cuda_weight_free(self.raw) }
    }
}

/// Work fused around a projection (rms_norm_mul on the input rows, residual add, LM-head scale and softcap).
#[derive(Debug, Clone, Copy, Default)]
pub struct Epilogue<'a> {
    pub row_scale: Option<DeviceSlice<'a>>,
    pub residual: Option<DeviceSlice<'a>>,
    pub norm: Option<(DeviceSlice<'a>, f32)>,
    pub out_scale: f32,
    pub softcap: f32,
    /// Row-parallel projection: also sum the output over the context's communicator.
    pub all_reduce: bool,
}

impl Default for DeviceSlice<'_> {
    fn default() -> Self {
        DeviceSlice { ptr: ptr::null_mut(), dtype: Dtype::F32, len: 0, _life: PhantomData }
    }
}

impl Epilogue<'_> {
    fn raw(&self) -> ffi::muser_cuda_epilogue {
        ffi::muser_cuda_epilogue {
            row_scale: self.row_scale.map_or(ptr::null(), |s| s.ptr as *const f32),
            residual: self.residual.map_or(ptr::null(), |s| s.ptr as *const c_void),
            swiglu: 0,
            norm_eps: self.norm.map_or(0.0, |n| n.1),
            norm_weight: self.norm.map_or(ptr::null(), |n| n.0.ptr as *const f32),
            out_scale: self.out_scale,
            softcap: self.softcap,
            all_reduce: self.all_reduce as u32,
        }
    }
}

/// The encoders.  Every call enqueues on `stream` and returns; `CudaContext::wait_for_completion` is the one wait.
pub struct CudaKernels<'c> {
    ctx: &'c CudaContext,
}

impl<'c> CudaKernels<'c> {
    pub fn new(ctx: &'c CudaContext) -> Self {
        Self { ctx }
    }

    pub fn supports_projection(dtype: Dtype) -> bool {
        unsafe { ffi::muser_cuda_supports_projection(dtype as u32) != 0 }
    }

    /// y[t][r] = dot(W_r, x_t) for a K-quant weight, 1..=64 tokens.
    pub fn encode_quantized_matmul(
        &self,
        stream: Stream,
        weights: &CudaWeight,
        input: DeviceSlice<'_>,
        output: DeviceSlice<'_>,
        tokens: usize,
        epilogue: Option<&Epilogue<'_>>,
    ) -> Result<()> {
        let ep = epilogue.map(Epilogue::raw);
        check(
            unsafe {
                ffi::muser_cuda_quantized_matmul(
                    self.ctx.raw,
                    weights.raw,
                    input.ptr,
                    input.dtype as u32,
                    output.ptr,
                    output.dtype as u32,
                    tokens as u32,
                    ep.as_ref().map_or(ptr::null(), |e| e as *const _),
                    stream.0,
                )
            },
            self.ctx.raw,
        )
    }

    /// Up to four projections of the same activations (q | k | v, gate | up) in one launch, 1..=16 tokens.
    pub fn encode_quantized_decode_group(
        &self,
        stream: Stream,
        items: &[(&CudaWeight, DeviceSlice<'_>, Option<&Epilogue<'_>>)],
        input: DeviceSlice<'_>,
        tokens: usize,
    ) -> Result<()> {
        let eps: Vec<Option<ffi::muser_cuda_epilogue>> = items.iter().map(|i| i.2.map(Epilogue::raw)).collect();
        let raw: Vec<ffi::muser_cuda_group_item> = items
            .iter()
            .zip(&eps)
            .map(|(i, e)| ffi::muser_cuda_group_item {
                w: i.0.raw,
                y: i.1.ptr,
                y_dtype: i.1.dtype as u32,
                reserved: 0,
                epilogue: e.as_ref().map_or(ptr::null(), |e| e as *const _),
            })
            .collect();
        check(
            unsafe {
                ffi::muser_cuda_quantized_matmul_group(self.ctx.raw, raw.as_ptr(), raw.len() as u32, input.ptr, input.dtype as u32, tokens as u32, stream.0)
            },
            self.ctx.raw,
        )
    }

    /// y[t][j] = silu(Wgate_j . x_t) * (Wup_j . x_t); the two projections are never written out.
    pub fn encode_ffn_gate_up_silu(
        &self,
        stream: Stream,
        gate: &CudaWeight,
        up: &CudaWeight,
        input: DeviceSlice<'_>,
        output: DeviceSlice<'_>,
        tokens: usize,
        epilogue: Option<&Epilogue<'_>>,
    ) -> Result<()> {
        let ep = epilogue.map(Epilogue::raw);
        check(
            unsafe {
                ffi::muser_cuda_ffn_gate_up_silu(
                    self.ctx.raw,
                    gate.raw,
                    up.raw,
                    input.ptr,
                    input.dtype as u32,
                    output.ptr,
                    output.dtype as u32,
                    tokens as u32,
                    ep.as_ref().map_or(ptr::null(), |e| e as *const _),
                    stream.0,
                )
            },
            self.ctx.raw,
        )
    }

    /// The NVFP4 projection: W4A4 when the weight carries `input_scale_inv`, the weight-only lane otherwise.
    pub fn encode_nvfp4_matmul(
        &self,
        stream: Stream,
        weights: &CudaWeight,
        input: DeviceSlice<'_>,
        output: DeviceSlice<'_>,
        columns: usize,
        epilogue: Option<&Epilogue<'_>>,
    ) -> Result<()> {
        let ep = epilogue.map(Epilogue::raw);
        check(
            unsafe {
                ffi::muser_cuda_nvfp4_matmul(
                    self.ctx.raw,
                    weights.raw,
                    input.ptr,
                    input.dtype as u32,
                    output.ptr,
                    output.dtype as u32,
                    columns as u32,
                    ep.as_ref().map_or(ptr::null(), |e| e as *const _),
                    stream.0,
                )
            },
            self.ctx.raw,
        )
    }

    /// q | k | v (2..4 NVFP4 weights with the same inputs and `input_scale_inv`) on activations quantized earlier, one
    /// launch over the output tiles of all of them; every output equals the single call's, bit for bit.
    pub fn encode_nvfp4_group_prequant(
        &self,
        stream: Stream,
        weights: &[&CudaWeight],
        packed: DeviceSlice<'_>,
        scales_swizzled: DeviceSlice<'_>,
        outputs: &[DeviceSlice<'_>],
        columns: usize,
    ) -> Result<()> {
        let ws: Vec<*const ffi::muser_cuda_weight> = weights.iter().map(|w| w.raw as *const _).collect();
        let ys: Vec<*mut std::ffi::c_void> = outputs.iter().map(|o| o.ptr).collect();
        let y_dtype = outputs.first().map_or(0, |o| o.dtype as u32);
        check(
            unsafe {
                ffi::muser_cuda_nvfp4_matmul_group_prequant(
                    self.ctx.raw,
                    ws.as_ptr(),
                    ws.len() as u32,
                    packed.ptr as *const u8,
                    scales_swizzled.ptr as *const u8,
                    ys.as_ptr(),
                    y_dtype,
                    columns as u32,
                    stream.0,
                )
            },
            self.ctx.raw,
        )
    }

    /// Measures the decode kernel's launch plans for one projection or group once, at load time.
    pub fn autotune(&self, stream: Stream, weights: &[&CudaWeight], up: Option<&CudaWeight>, max_tokens: usize) -> Result<()> {
        let raw: Vec<*const ffi::muser_cuda_weight> = weights.iter().map(|w| w.raw as *const _).collect();
        check(
            unsafe {
                ffi::muser_cuda_decode_autotune(self.ctx.raw, raw.as_ptr(), raw.len() as u32, up.map_or(ptr::null(), |w| w.raw as *const _), max_tokens as u32, stream.0)
            },
            self.ctx.raw,
        )
    }
}

/// `weights::matmul` with the weight resident on the GPU: host slices in, host slices out, f32 both ways.
pub fn matmul(ctx: &CudaContext, w: &CudaWeight, x: &[f32], n_tokens: usize, out: &mut [f32]) -> Result<()> {
    let info = w.info();
    if x.len() != n_tokens * info.n_in as usize || out.len() != n_tokens * info.n_out as usize {
        return Err(CudaError::BadShape(format!("x has {} values, out {}, for {} tokens of {} -> {}", x.len(), out.len(), n_tokens, info.n_in, info.n_out)));
    }
    check(unsafe { ffi::muser_cuda_matmul_host(ctx.raw, w.raw, x.as_ptr(), n_tokens as u32, out.as_mut_ptr()) }, ctx.raw)
}
