// C ABI of the library: argument validation, handle lifetime, dispatch.  See include/muser_cuda.h.
#include <cmath>
#include <cstring>
#include <map>
#include <new>

#include "common.cuh"
#include "kquant_layout.cuh"
#include "tcgen05.cuh"

namespace muser {
thread_local std::string g_create_error;

cudaError_t ensure_dynamic_smem(const void *kernel, int device, size_t bytes) {
    static std::mutex mu;
    static std::map<std::pair<const void *, int>, size_t> set;
    std::lock_guard<std::mutex> lock(mu);
    size_t &have = set[{kernel, device}];
    if (bytes <= have) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess) have = bytes;
    return e;
}

// The give-up path of the kernels' bounded waits, run on its own: one thread waits on a barrier that nobody will
// ever arrive at, for `polls` polls, then records code 901 the way the kernels record theirs and returns.  Nothing
// hangs and nothing faults; muser_cuda_sync_status must then report MUSER_CUDA_TIMEOUT once.
__global__ void wait_probe_kernel(uint32_t polls, int *status) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (!mbar_wait(smem_u32(&bar), 0, &abort_flag, polls)) atomicExch(status + 1, 901);
}

static bool is_kquant(uint32_t t) { return t == MUSER_DTYPE_Q4_K || t == MUSER_DTYPE_Q5_K || t == MUSER_DTYPE_Q6_K; }

// 64-bit digest of a device buffer, independent of thread scheduling: sum over 8-byte words of a
// position-keyed multiplicative mix.
__global__ void image_hash_kernel(const uint64_t *__restrict__ p, uint64_t n, unsigned long long *out) {
    uint64_t h = 0;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t v = (p[i] + 0x9E3779B97F4A7C15ull * (i + 1)) * 0xBF58476D1CE4E5B9ull;
        v ^= v >> 29;
        h += v * 0x94D049BB133111EBull;
    }
    for (int o = 16; o > 0; o >>= 1) h += __shfl_xor_sync(0xffffffffu, h, o);
    if ((threadIdx.x & 31) == 0) atomicAdd(out, (unsigned long long)h);
}

static muser_cuda_status validate_shard(Ctx *ctx, uint32_t dtype, uint64_t n_in, uint64_t n_out,
                                        const muser_cuda_shard *shard, Weight *w) {
    w->n_in_full = n_in;
    w->n_out_full = n_out;
    w->n_in = n_in;
    w->n_out = n_out;
    w->shard = muser_cuda_shard{0, 1, MUSER_SHARD_NONE};
    if (!shard || shard->axis == MUSER_SHARD_NONE || shard->world <= 1) return MUSER_CUDA_OK;
    if (shard->rank >= shard->world || shard->axis > MUSER_SHARD_K) return fail(ctx, MUSER_CUDA_BAD_ARG, "bad shard descriptor");
    w->shard = *shard;
    if (shard->axis == MUSER_SHARD_ROWS) {
        // whole 16-row groups per rank keep K-quant tiles unshared; NVFP4 needs nothing beyond divisibility
        if (n_out % shard->world) return fail(ctx, MUSER_CUDA_BAD_SHAPE, "n_out is not divisible by the shard count");
        w->n_out = n_out / shard->world;
    } else {
        const uint64_t gran = (dtype == MUSER_DTYPE_Q4_K || dtype == MUSER_DTYPE_Q5_K) ? 32 : dtype == MUSER_DTYPE_Q6_K ? 16 : 64;
        if (n_in % shard->world || (n_in / shard->world) % gran)
            return fail(ctx, MUSER_CUDA_BAD_SHAPE, "the K shard is not a whole number of sub-blocks");
        w->n_in = n_in / shard->world;
    }
    return MUSER_CUDA_OK;
}

static muser_cuda_status repack_common(Ctx *ctx, uint32_t dtype, const uint8_t *blocks, const uint8_t *scales,
                                       bool on_host, float scale2, int has_isi, float isi, uint64_t n_in,
                                       uint64_t n_out, const muser_cuda_shard *shard, cudaStream_t stream,
                                       muser_cuda_weight **out) {
    if (!ctx || !out) return MUSER_CUDA_BAD_ARG;
    *out = nullptr;
    if (!muser_cuda_supports_projection(dtype)) return fail(ctx, MUSER_CUDA_UNSUPPORTED_DTYPE, "dtype has no CUDA projection kernel");
    if (!blocks || n_in == 0 || n_out == 0) return fail(ctx, MUSER_CUDA_BAD_ARG, "null weight bytes or empty geometry");
    if (n_in > (1ull << 30) || n_out > (1ull << 30)) return fail(ctx, MUSER_CUDA_BAD_SHAPE, "dimension too large");
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    Weight *w = new (std::nothrow) Weight();
    if (!w) return fail(ctx, MUSER_CUDA_ERROR, "out of host memory");
    w->dtype = dtype;
    w->device = ctx->device;
    muser_cuda_status st = validate_shard(ctx, dtype, n_in, n_out, shard, w);
    auto bail = [&](muser_cuda_status s) {
        muser_cuda_weight_free(reinterpret_cast<muser_cuda_weight *>(w));
        return s;
    };
    if (st != MUSER_CUDA_OK) return bail(st);
    size_t raw_bytes = 0, raw_scale_bytes = 0;
    if (is_kquant(dtype)) {
        if (n_in % 256) return bail(fail(ctx, MUSER_CUDA_BAD_SHAPE, "K-quant rows need n_in % 256 == 0"));
        raw_bytes = n_out * (n_in / 256) * (dtype == MUSER_DTYPE_Q4_K ? 144 : dtype == MUSER_DTYPE_Q5_K ? 176 : 210);
        const uint64_t k0 = w->shard.axis == MUSER_SHARD_K ? w->shard.rank * w->n_in : 0;
        w->k_off = (uint32_t)(k0 % 256);
        w->nsb = (uint32_t)((w->k_off + w->n_in + 255) / 256);
        w->row_tiles = (uint32_t)((w->n_out + 15) / 16);
        w->image_bytes = (uint64_t)w->row_tiles * w->nsb * kquant_tile_bytes(dtype);
        cudaError_t e = cudaMalloc(&w->image, w->image_bytes);
        if (e != cudaSuccess) return bail(fail(ctx, MUSER_CUDA_ERROR, std::string("cudaMalloc(image): ") + cudaGetErrorString(e)));
    } else {
        if (!scales) return bail(fail(ctx, MUSER_CUDA_BAD_ARG, "NVFP4 weights need their block scales"));
        if (n_in % 64) return bail(fail(ctx, MUSER_CUDA_BAD_SHAPE, "NVFP4 rows need n_in % 64 == 0"));
        if (!std::isfinite(scale2) || (has_isi && !(std::isfinite(isi) && isi > 0.0f)))
            return bail(fail(ctx, MUSER_CUDA_NAN_SCALE, "non-finite NVFP4 tensor scale"));
        raw_bytes = n_out * (n_in / 2);
        raw_scale_bytes = n_out * (n_in / 16);
        w->scale2 = scale2;
        w->has_input_scale_inv = has_isi != 0;
        w->input_scale_inv = has_isi ? isi : 0.0f;
        w->n_out_pad = (w->n_out + 255) / 256 * 256; // whole 256-row GEMM tiles
        const size_t packed_bytes = w->n_out_pad * (w->n_in / 2);
        const size_t scale_bytes = (w->n_out_pad / 128) * ((w->n_in + 63) / 64) * 512;
        w->image_bytes = packed_bytes + scale_bytes;
        cudaError_t e = cudaMalloc(&w->packed, packed_bytes);
        if (e == cudaSuccess) e = cudaMalloc(&w->scales, scale_bytes);
        if (e != cudaSuccess) return bail(fail(ctx, MUSER_CUDA_ERROR, std::string("cudaMalloc(nvfp4): ") + cudaGetErrorString(e)));
    }
    const uint8_t *dev_blocks = blocks, *dev_scales = scales;
    uint8_t *tmp = nullptr, *tmp_s = nullptr;
    if (on_host) {
        cudaError_t e = cudaMalloc(&tmp, raw_bytes);
        if (e == cudaSuccess && raw_scale_bytes) e = cudaMalloc(&tmp_s, raw_scale_bytes);
        if (e == cudaSuccess) e = cudaMemcpyAsync(tmp, blocks, raw_bytes, cudaMemcpyHostToDevice, stream);
        if (e == cudaSuccess && raw_scale_bytes) e = cudaMemcpyAsync(tmp_s, scales, raw_scale_bytes, cudaMemcpyHostToDevice, stream);
        if (e != cudaSuccess) {
            cudaFree(tmp);
            cudaFree(tmp_s);
            return bail(fail(ctx, MUSER_CUDA_ERROR, std::string("staging the stored tensor: ") + cudaGetErrorString(e)));
        }
        dev_blocks = tmp;
        dev_scales = tmp_s;
    }
    st = is_kquant(dtype) ? launch_repack_kquant(ctx, w, dev_blocks, stream)
                          : launch_repack_nvfp4(ctx, w, dev_blocks, dev_scales, stream);
    cudaError_t e = cudaStreamSynchronize(stream);
    cudaFree(tmp);
    cudaFree(tmp_s);
    if (st != MUSER_CUDA_OK) return bail(st);
    if (e != cudaSuccess) return bail(fail(ctx, MUSER_CUDA_ERROR, std::string("repack: ") + cudaGetErrorString(e)));
    if (dtype == MUSER_DTYPE_NVFP4_E2M1) {
        st = nvfp4_build_tensor_map(ctx, w);
        if (st != MUSER_CUDA_OK) return bail(st);
    }
    *out = reinterpret_cast<muser_cuda_weight *>(w);
    return MUSER_CUDA_OK;
}

static muser_cuda_status check_io(Ctx *ctx, const Weight *w, const void *x, uint32_t x_dtype, const void *y,
                                  uint32_t y_dtype, uint32_t tokens, bool y_f16_ok) {
    if (!ctx || !w || !x || !y) return fail(ctx, MUSER_CUDA_BAD_ARG, "null argument");
    if (w->device != ctx->device) return fail(ctx, MUSER_CUDA_BAD_ARG, "weight lives on another device");
    if (tokens == 0) return fail(ctx, MUSER_CUDA_BAD_SHAPE, "tokens must be positive");
    if (x_dtype != MUSER_DTYPE_F32 && x_dtype != MUSER_DTYPE_BF16) return fail(ctx, MUSER_CUDA_UNSUPPORTED_DTYPE, "activations must be f32 or bf16");
    if (y_dtype != MUSER_DTYPE_F32 && y_dtype != MUSER_DTYPE_BF16 && !(y_f16_ok && y_dtype == MUSER_DTYPE_F16))
        return fail(ctx, MUSER_CUDA_UNSUPPORTED_DTYPE, "unsupported output dtype");
    if (!aligned16(x) || !aligned16(y)) return fail(ctx, MUSER_CUDA_BAD_ALIGN, "x and y must be 16-byte aligned");
    return MUSER_CUDA_OK;
}

// Public epilogue -> the launchers' form.  The fused input norm needs the whole input row, so it is refused on
// K shards, and its weight vector must be readable with 16-byte loads.
static muser_cuda_status take_epilogue(Ctx *ctx, const Weight *w, const muser_cuda_epilogue *ep, Epilogue *e, bool may_all_reduce = false) {
    if (!ep) return MUSER_CUDA_OK;
    if (ep->all_reduce) {
        if (!may_all_reduce) return fail(ctx, MUSER_CUDA_BAD_ARG, "all_reduce is honoured by muser_cuda_quantized_matmul only; elsewhere call muser_cuda_all_reduce after the projection");
        if (!ctx->comm) return fail(ctx, MUSER_CUDA_BAD_ARG, "all_reduce needs a communicator on this context (muser_cuda_ctx_comm_init / _attach)");
        e->all_reduce = true;
    }
    e->row_scale = ep->row_scale;
    e->residual = ep->residual;
    if (!(ep->out_scale == ep->out_scale) || !(ep->softcap >= 0.0f)) return fail(ctx, MUSER_CUDA_BAD_ARG, "out_scale / softcap must be numbers, softcap non-negative");
    e->out_scale = ep->out_scale == 0.0f ? 1.0f : ep->out_scale;
    e->softcap = ep->softcap;
    if (ep->softcap > 0.0f && w->shard.axis == MUSER_SHARD_K && w->shard.world > 1)
        return fail(ctx, MUSER_CUDA_BAD_SHAPE, "softcap is not linear: it cannot be applied to a K shard's partial sums");
    if (ep->norm_weight) {
        if (w->shard.axis == MUSER_SHARD_K && w->shard.world > 1)
            return fail(ctx, MUSER_CUDA_BAD_SHAPE, "the fused input norm needs whole input rows; this weight is a K shard");
        if (!aligned16(ep->norm_weight)) return fail(ctx, MUSER_CUDA_BAD_ALIGN, "norm_weight must be 16-byte aligned");
        if (!(ep->norm_eps >= 0.0f)) return fail(ctx, MUSER_CUDA_BAD_ARG, "norm_eps must be non-negative");
        e->norm_weight = ep->norm_weight;
        e->norm_eps = ep->norm_eps;
    }
    return MUSER_CUDA_OK;
}

} // namespace muser

using namespace muser;

extern "C" {

uint32_t muser_cuda_abi_version(void) { return MUSER_CUDA_ABI_VERSION; }

int muser_cuda_supports_projection(uint32_t t) {
    return t == MUSER_DTYPE_Q4_K || t == MUSER_DTYPE_Q5_K || t == MUSER_DTYPE_Q6_K || t == MUSER_DTYPE_NVFP4_E2M1;
}

muser_cuda_status muser_cuda_ctx_create(int device, size_t workspace_bytes, muser_cuda_ctx **out) {
    if (!out) return MUSER_CUDA_BAD_ARG;
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || device < 0 || device >= count) {
        g_create_error = e != cudaSuccess ? std::string("cudaGetDeviceCount: ") + cudaGetErrorString(e)
                                          : "no such CUDA device";
        return e != cudaSuccess ? MUSER_CUDA_ERROR : MUSER_CUDA_BAD_ARG;
    }
    cudaDeviceProp prop;
    e = cudaSetDevice(device);
    if (e == cudaSuccess) e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) {
        g_create_error = std::string("cudaSetDevice: ") + cudaGetErrorString(e);
        return MUSER_CUDA_ERROR;
    }
    if (prop.major != 10) {
        g_create_error = "this library is built for sm_100a only (found sm_" + std::to_string(prop.major) + std::to_string(prop.minor) + ")";
        return MUSER_CUDA_ERROR;
    }
    Ctx *ctx = new (std::nothrow) Ctx();
    if (!ctx) return MUSER_CUDA_ERROR;
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->workspace_bytes = workspace_bytes;
    e = cudaMalloc(&ctx->dev_status, 4 * sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(ctx->dev_status, 0, 4 * sizeof(int));
    ctx->gemv_partial_bytes = 16u << 20;
    ctx->gemv_counter_slots = 1u << 16;
    if (e == cudaSuccess) e = cudaMalloc(&ctx->gemv_partial, ctx->gemv_partial_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&ctx->gemv_counters, ctx->gemv_counter_slots * sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMemset(ctx->gemv_counters, 0, ctx->gemv_counter_slots * sizeof(unsigned int));
    ctx->tc_scratch_bytes = (size_t)64 * 32768 * 2 + (size_t)64 * 2048 * 2 + 4096; // f16 rows + sub-block sums, 64 tokens
    if (e == cudaSuccess) e = cudaMalloc(&ctx->tc_scratch, ctx->tc_scratch_bytes);
    ctx->norm_scratch_bytes = (size_t)64 * 32768 * sizeof(float); // 64 tokens x the widest row
    if (e == cudaSuccess) e = cudaMalloc(&ctx->norm_scratch, ctx->norm_scratch_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&ctx->amax_keys, 16 * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMemset(ctx->amax_keys, 0, 16 * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMalloc(&ctx->amax_flags, 16 * sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMemset(ctx->amax_flags, 0, 16 * sizeof(unsigned int));
    ctx->inv_rms_rows = 1u << 20; // token rows per call of a fused input norm
    if (e == cudaSuccess) e = cudaMalloc(&ctx->inv_rms, (size_t)ctx->inv_rms_rows * sizeof(float));
    if (e == cudaSuccess && workspace_bytes) e = cudaMalloc(&ctx->workspace, workspace_bytes);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        g_create_error = std::string("context allocation: ") + cudaGetErrorString(e);
        muser_cuda_ctx_destroy(reinterpret_cast<muser_cuda_ctx *>(ctx));
        return MUSER_CUDA_ERROR;
    }
    *out = reinterpret_cast<muser_cuda_ctx *>(ctx);
    return MUSER_CUDA_OK;
}

void muser_cuda_ctx_destroy(muser_cuda_ctx *c) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    comm_destroy(ctx);
    cudaFree(ctx->workspace);
    cudaFree(ctx->dev_status);
    cudaFree(ctx->gemv_partial);
    cudaFree(ctx->gemv_counters);
    cudaFree(ctx->norm_scratch);
    cudaFree(ctx->inv_rms);
    cudaFree(ctx->amax_keys);
    cudaFree(ctx->amax_flags);
    cudaFree(ctx->tc_scratch);
    cudaFree(ctx->dev_stage);
    cudaFree(ctx->arena);
    if (ctx->host_stage) cudaFreeHost(ctx->host_stage);
    for (cudaEvent_t ev : ctx->copy_events)
        if (ev) cudaEventDestroy(ev);
    if (ctx->copy_stream) cudaStreamDestroy(ctx->copy_stream);
    delete ctx;
}

const char *muser_cuda_last_error(const muser_cuda_ctx *c) {
    const Ctx *ctx = reinterpret_cast<const Ctx *>(c);
    return ctx ? ctx->last_error.c_str() : g_create_error.c_str();
}

muser_cuda_status muser_cuda_sync_status(muser_cuda_ctx *c, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (!ctx) return MUSER_CUDA_BAD_ARG;
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    int flags[4] = {0, 0, 0, 0};
    MUSER_CUDA_TRY(ctx, cudaMemcpyAsync(flags, ctx->dev_status, sizeof(flags), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    MUSER_CUDA_TRY(ctx, cudaStreamSynchronize((cudaStream_t)stream));
    ctx->arena_used = 0; // everything enqueued through matmul_host_enqueue on this stream has finished
    if (flags[1]) {
        cudaMemsetAsync(ctx->dev_status, 0, sizeof(flags), (cudaStream_t)stream);
        return fail(ctx, MUSER_CUDA_TIMEOUT, "a device-side bounded wait gave up (code " + std::to_string(flags[1]) + ")");
    }
    return MUSER_CUDA_OK;
}

muser_cuda_status muser_cuda_tuning_set(muser_cuda_ctx *c, uint32_t key, uint32_t value) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (!ctx) return MUSER_CUDA_BAD_ARG;
    switch (key) {
    case MUSER_TUNE_TC_MIN_TOKENS_Q4_K: ctx->tc_min_tokens[0] = value; return MUSER_CUDA_OK;
    case MUSER_TUNE_TC_MIN_TOKENS_Q6_K: ctx->tc_min_tokens[1] = value; return MUSER_CUDA_OK;
    case MUSER_TUNE_TC_MIN_ROWS: ctx->tc_min_rows = value; return MUSER_CUDA_OK;
    case MUSER_TUNE_DECODE_WARPS: ctx->dec_warps = value & ~1u; return MUSER_CUDA_OK;
    case MUSER_TUNE_DECODE_KSPLIT: ctx->dec_ksplit = value; return MUSER_CUDA_OK;
    case MUSER_TUNE_DECODE_RING: ctx->dec_ring = value; return MUSER_CUDA_OK;
    case MUSER_TUNE_DECODE_WSPLIT: ctx->dec_wsplit = value; return MUSER_CUDA_OK;
    case MUSER_TUNE_NVFP4_PAIR:
        if (value > 1) return fail(ctx, MUSER_CUDA_BAD_ARG, "MUSER_TUNE_NVFP4_PAIR takes 0 (one CTA per tile) or 1 (pairs of SMs)");
        ctx->nvfp4_pair = value;
        return MUSER_CUDA_OK;
    case MUSER_TUNE_ONESHOT_MAX_BYTES: ctx->oneshot_max_bytes = value; return MUSER_CUDA_OK;
    case MUSER_TUNE_HOST_DIRECT_OUTPUT:
        if (value > 2) return fail(ctx, MUSER_CUDA_BAD_ARG, "MUSER_TUNE_HOST_DIRECT_OUTPUT takes 0, 1 or 2");
        ctx->host_direct_output = value;
        return MUSER_CUDA_OK;
    case MUSER_TUNE_NVFP4_GROUP_M: ctx->nvfp4_group_m = value; return MUSER_CUDA_OK;
    default: return fail(ctx, MUSER_CUDA_BAD_ARG, "unknown tuning key");
    }
}

muser_cuda_status muser_cuda_weight_repack(muser_cuda_ctx *c, uint32_t t, const uint8_t *blocks, const uint8_t *scales,
                                           float scale2, int has_isi, float isi, uint64_t n_in, uint64_t n_out,
                                           const muser_cuda_shard *shard, muser_cuda_weight **out) {
    return repack_common(reinterpret_cast<Ctx *>(c), t, blocks, scales, true, scale2, has_isi, isi, n_in, n_out, shard, nullptr, out);
}

muser_cuda_status muser_cuda_weight_repack_device(muser_cuda_ctx *c, uint32_t t, const uint8_t *blocks,
                                                  const uint8_t *scales, float scale2, int has_isi, float isi,
                                                  uint64_t n_in, uint64_t n_out, const muser_cuda_shard *shard,
                                                  void *stream, muser_cuda_weight **out) {
    return repack_common(reinterpret_cast<Ctx *>(c), t, blocks, scales, false, scale2, has_isi, isi, n_in, n_out, shard,
                         (cudaStream_t)stream, out);
}

void muser_cuda_weight_free(muser_cuda_weight *wp) {
    Weight *w = reinterpret_cast<Weight *>(wp);
    if (!w) return;
    cudaSetDevice(w->device);
    cudaFree(w->image);
    cudaFree(w->packed);
    cudaFree(w->scales);
    nvfp4_free_tensor_map(w);
    delete w;
}

muser_cuda_status muser_cuda_weight_info_get(const muser_cuda_weight *wp, muser_cuda_weight_info *out) {
    const Weight *w = reinterpret_cast<const Weight *>(wp);
    if (!w || !out) return MUSER_CUDA_BAD_ARG;
    std::memset(out, 0, sizeof(*out));
    out->dtype = w->dtype;
    out->shard_axis = w->shard.axis;
    out->shard_rank = w->shard.rank;
    out->shard_world = w->shard.world;
    out->n_in = w->n_in;
    out->n_out = w->n_out;
    out->n_in_full = w->n_in_full;
    out->n_out_full = w->n_out_full;
    out->image_bytes = w->image_bytes;
    out->scale2 = w->scale2;
    out->input_scale_inv = w->input_scale_inv;
    out->has_input_scale_inv = w->has_input_scale_inv;
    // digest computed on request (load-time diagnostics, synchronizes the device)
    if (cudaSetDevice(w->device) != cudaSuccess) return MUSER_CUDA_ERROR;
    unsigned long long *acc = nullptr;
    if (cudaMalloc(&acc, 8) != cudaSuccess) return MUSER_CUDA_ERROR;
    cudaMemset(acc, 0, 8);
    if (w->image) {
        image_hash_kernel<<<592, 256>>>(reinterpret_cast<const uint64_t *>(w->image), w->image_bytes / 8, acc);
    } else {
        const uint64_t pb = w->n_out_pad * (w->n_in / 2);
        image_hash_kernel<<<592, 256>>>(reinterpret_cast<const uint64_t *>(w->packed), pb / 8, acc);
        image_hash_kernel<<<592, 256>>>(reinterpret_cast<const uint64_t *>(w->scales), (w->image_bytes - pb) / 8, acc);
    }
    unsigned long long h = 0;
    cudaError_t e = cudaMemcpy(&h, acc, 8, cudaMemcpyDeviceToHost);
    cudaFree(acc);
    if (e != cudaSuccess) return MUSER_CUDA_ERROR;
    out->image_hash = h;
    return MUSER_CUDA_OK;
}

muser_cuda_status muser_cuda_dequant(muser_cuda_ctx *c, const muser_cuda_weight *wp, float *out, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    const Weight *w = reinterpret_cast<const Weight *>(wp);
    if (!ctx || !w || !out) return fail(ctx, MUSER_CUDA_BAD_ARG, "null argument");
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_dequant(ctx, w, out, (cudaStream_t)stream);
}

muser_cuda_status muser_cuda_quantized_matmul(muser_cuda_ctx *c, const muser_cuda_weight *wp, const void *x,
                                              uint32_t x_dtype, void *y, uint32_t y_dtype, uint32_t tokens,
                                              const muser_cuda_epilogue *ep, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    const Weight *w = reinterpret_cast<const Weight *>(wp);
    muser_cuda_status st = check_io(ctx, w, x, x_dtype, y, y_dtype, tokens, false);
    if (st != MUSER_CUDA_OK) return st;
    if (!is_kquant(w->dtype)) return fail(ctx, MUSER_CUDA_UNSUPPORTED_DTYPE, "quantized_matmul takes K-quant weights; use nvfp4_matmul");
    if (tokens > 64) return fail(ctx, MUSER_CUDA_BAD_SHAPE, "quantized_matmul serves 1..64 tokens per call");
    if (ep && ep->swiglu) return fail(ctx, MUSER_CUDA_BAD_ARG, "use muser_cuda_ffn_gate_up_silu for the fused K-quant gate/up");
    Epilogue e;
    st = take_epilogue(ctx, w, ep, &e, true);
    if (st != MUSER_CUDA_OK) return st;
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_kquant_matmul(ctx, w, nullptr, x, x_dtype, y, y_dtype, tokens, e, (cudaStream_t)stream);
}

muser_cuda_status muser_cuda_quantized_matmul_group(muser_cuda_ctx *c, const muser_cuda_group_item *items, uint32_t n_items,
                                                    const void *x, uint32_t x_dtype, uint32_t tokens, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (!ctx || !items || n_items == 0 || n_items > 4) return fail(ctx, MUSER_CUDA_BAD_ARG, "a group holds 1..4 projections");
    if (tokens > 16) return fail(ctx, MUSER_CUDA_BAD_SHAPE, "a grouped launch serves 1..16 tokens");
    const Weight *w[4];
    void *y[4];
    uint32_t yd[4];
    Epilogue e[4];
    for (uint32_t i = 0; i < n_items; ++i) {
        w[i] = reinterpret_cast<const Weight *>(items[i].w);
        y[i] = items[i].y;
        yd[i] = items[i].y_dtype;
        muser_cuda_status st = check_io(ctx, w[i], x, x_dtype, y[i], yd[i], tokens, false);
        if (st != MUSER_CUDA_OK) return st;
        if (!is_kquant(w[i]->dtype)) return fail(ctx, MUSER_CUDA_UNSUPPORTED_DTYPE, "grouped launches take K-quant weights");
        if (items[i].epilogue && items[i].epilogue->swiglu) return fail(ctx, MUSER_CUDA_BAD_ARG, "use muser_cuda_ffn_gate_up_silu for the fused gate/up");
        st = take_epilogue(ctx, w[i], items[i].epilogue, &e[i]);
        if (st != MUSER_CUDA_OK) return st;
        if (w[i]->n_in != w[0]->n_in || w[i]->nsb != w[0]->nsb || w[i]->k_off != w[0]->k_off)
            return fail(ctx, MUSER_CUDA_BAD_SHAPE, "the projections of a group must share n_in and the K shard geometry");
        if (e[i].norm_weight != e[0].norm_weight || e[i].norm_eps != e[0].norm_eps)
            return fail(ctx, MUSER_CUDA_BAD_ARG, "the projections of a group share one input, so they must share the fused input norm");
    }
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const cudaError_t de = launch_kquant_decode(ctx, w, nullptr, n_items, x, x_dtype, y, yd, tokens, e, (cudaStream_t)stream);
    if (de != cudaErrorNotSupported) {
        MUSER_CUDA_TRY(ctx, de);
        return MUSER_CUDA_OK;
    }
    for (uint32_t i = 0; i < n_items; ++i) { // shapes the grouped kernel does not take: one launch each
        const muser_cuda_status st = launch_kquant_matmul(ctx, w[i], nullptr, x, x_dtype, y[i], yd[i], tokens, e[i], (cudaStream_t)stream);
        if (st != MUSER_CUDA_OK) return st;
    }
    return MUSER_CUDA_OK;
}

muser_cuda_status muser_cuda_decode_last_plan(const muser_cuda_ctx *c, uint32_t out[4]) {
    const Ctx *ctx = reinterpret_cast<const Ctx *>(c);
    if (!ctx || !out) return MUSER_CUDA_BAD_ARG;
    for (int i = 0; i < 4; ++i) out[i] = ctx->dec_last_plan[i];
    return MUSER_CUDA_OK;
}

muser_cuda_status muser_cuda_decode_autotune(muser_cuda_ctx *c, const muser_cuda_weight *const *weights, uint32_t n_weights,
                                             const muser_cuda_weight *w_up, uint32_t max_tokens, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (!ctx || !weights) return fail(ctx, MUSER_CUDA_BAD_ARG, "null argument");
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return decode_autotune(ctx, reinterpret_cast<const Weight *const *>(weights), reinterpret_cast<const Weight *>(w_up), n_weights, max_tokens,
                           (cudaStream_t)stream);
}

muser_cuda_status muser_cuda_quantized_matmul_rows(muser_cuda_ctx *c, const muser_cuda_weight *wp, const uint32_t *rows,
                                                   uint32_t n_rows, const void *x, uint32_t x_dtype, float *y,
                                                   uint32_t tokens, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    const Weight *w = reinterpret_cast<const Weight *>(wp);
    muser_cuda_status st = check_io(ctx, w, x, x_dtype, y, MUSER_DTYPE_F32, tokens, false);
    if (st != MUSER_CUDA_OK) return st;
    if (!rows || n_rows == 0) return fail(ctx, MUSER_CUDA_BAD_ARG, "empty row list");
    if (!is_kquant(w->dtype)) return fail(ctx, MUSER_CUDA_UNSUPPORTED_DTYPE, "matmul_rows takes K-quant weights");
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_kquant_rows(ctx, w, rows, n_rows, x, x_dtype, y, tokens, (cudaStream_t)stream);
}

muser_cuda_status muser_cuda_lm_head_argmax(muser_cuda_ctx *c, const muser_cuda_weight *wp, const void *x, uint32_t x_dtype,
                                            uint32_t tokens, const muser_cuda_epilogue *ep, void *logits, uint32_t logits_dtype,
                                            uint32_t *out_index, float *out_value, uint32_t *out_nonfinite, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    const Weight *w = reinterpret_cast<const Weight *>(wp);
    if (!out_index) return fail(ctx, MUSER_CUDA_BAD_ARG, "null argument");
    muser_cuda_status st = check_io(ctx, w, x, x_dtype, logits ? logits : x, logits ? logits_dtype : MUSER_DTYPE_F32, tokens, false);
    if (st != MUSER_CUDA_OK) return st;
    if (!is_kquant(w->dtype)) return fail(ctx, MUSER_CUDA_UNSUPPORTED_DTYPE, "lm_head_argmax takes K-quant weights");
    if (tokens > 16) return fail(ctx, MUSER_CUDA_BAD_SHAPE, "lm_head_argmax serves 1..16 tokens per call");
    if (w->shard.world > 1) return fail(ctx, MUSER_CUDA_BAD_SHAPE, "the greedy pick needs the whole vocabulary: unsharded weights only");
    if (ep && (ep->swiglu || ep->residual)) return fail(ctx, MUSER_CUDA_BAD_ARG, "lm_head_argmax takes the input norm, row scale, logit scale and softcap only");
    Epilogue e;
    st = take_epilogue(ctx, w, ep, &e);
    if (st != MUSER_CUDA_OK) return st;
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const cudaError_t de = launch_lm_head_argmax(ctx, w, x, x_dtype, logits, logits_dtype, tokens, e, out_index, out_value, out_nonfinite, (cudaStream_t)stream);
    if (de == cudaErrorNotSupported) return fail(ctx, MUSER_CUDA_BAD_SHAPE, "this weight's geometry does not fit the decode kernel");
    MUSER_CUDA_TRY(ctx, de);
    return MUSER_CUDA_OK;
}

muser_cuda_status muser_cuda_fused_norm_residual_rms_norm(muser_cuda_ctx *c, float *hidden, const float *src, float *output,
                                                          const float *weight1, const float *weight2, uint32_t tokens, uint32_t n,
                                                          float eps1, float eps2, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (!ctx || !hidden || !src || !weight1 || (output && !weight2)) return fail(ctx, MUSER_CUDA_BAD_ARG, "null argument");
    if (tokens == 0 || n == 0 || n % 4) return fail(ctx, MUSER_CUDA_BAD_SHAPE, "rows of a multiple of 4 values");
    if (!aligned16(hidden) || !aligned16(src) || !aligned16(weight1) || (output && (!aligned16(output) || !aligned16(weight2))))
        return fail(ctx, MUSER_CUDA_BAD_ALIGN, "rows and weights must be 16-byte aligned");
    if (!(eps1 >= 0.0f) || !(eps2 >= 0.0f)) return fail(ctx, MUSER_CUDA_BAD_ARG, "epsilons must be non-negative numbers");
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_norm_residual_norm(ctx, hidden, src, output, weight1, weight2, tokens, n, eps1, eps2, (cudaStream_t)stream);
}

muser_cuda_status muser_cuda_sigmoid_gate(muser_cuda_ctx *c, float *x, const float *gate, uint64_t count, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (!ctx || !x || !gate) return fail(ctx, MUSER_CUDA_BAD_ARG, "null argument");
    if (count == 0 || count % 4) return fail(ctx, MUSER_CUDA_BAD_SHAPE, "a multiple of 4 values");
    if (!aligned16(x) || !aligned16(gate)) return fail(ctx, MUSER_CUDA_BAD_ALIGN, "x and gate must be 16-byte aligned");
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_sigmoid_gate(ctx, x, gate, (size_t)count, (cudaStream_t)stream);
}

muser_cuda_status muser_cuda_head_rms_norm(muser_cuda_ctx *c, float *x, const float *weight, float eps, uint32_t tokens, uint32_t heads,
                                           uint32_t head_dim, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (!ctx || !x || !weight) return fail(ctx, MUSER_CUDA_BAD_ARG, "null argument");
    if (tokens == 0 || heads == 0 || head_dim == 0 || head_dim % 4 || (uint64_t)tokens * heads > (1u << 30))
        return fail(ctx, MUSER_CUDA_BAD_SHAPE, "heads of a multiple of 4 values");
    if (!aligned16(x) || !aligned16(weight)) return fail(ctx, MUSER_CUDA_BAD_ALIGN, "x and weight must be 16-byte aligned");
    if (!(eps >= 0.0f)) return fail(ctx, MUSER_CUDA_BAD_ARG, "epsilon must be a non-negative number");
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_head_rms_norm(ctx, x, weight, eps, tokens, heads, head_dim, (cudaStream_t)stream);
}

// The NVFP4 side of the fused gate/up call: both weights must quantize their input alike, because one set of
// activation codes feeds both.
static muser_cuda_status nvfp4_pair_checks(Ctx *ctx, const Weight *g, const Weight *u) {
    if (!u) return fail(ctx, MUSER_CUDA_BAD_ARG, "null up weight");
    if (g->dtype != MUSER_DTYPE_NVFP4_E2M1 || u->dtype != MUSER_DTYPE_NVFP4_E2M1)
        return fail(ctx, MUSER_CUDA_UNSUPPORTED_DTYPE, "gate and up must both be NVFP4");
    if (g->n_in != u->n_in || g->n_out != u->n_out) return fail(ctx, MUSER_CUDA_BAD_SHAPE, "gate and up geometry differ");
    if (g->shard.axis == MUSER_SHARD_K || u->shard.axis == MUSER_SHARD_K)
        return fail(ctx, MUSER_CUDA_BAD_SHAPE, "silu cannot be applied to K-sharded partial sums");
    if (!g->has_input_scale_inv || !u->has_input_scale_inv)
        return fail(ctx, MUSER_CUDA_UNSUPPORTED_DTYPE, "the W4A4 lane needs input_scale_inv on both weights");
    if (g->input_scale_inv != u->input_scale_inv)
        return fail(ctx, MUSER_CUDA_BAD_ARG, "gate and up must share one input_scale_inv: they read the same quantized activations");
    return MUSER_CUDA_OK;
}

muser_cuda_status muser_cuda_ffn_gate_up_silu(muser_cuda_ctx *c, const muser_cuda_weight *gp, const muser_cuda_weight *up,
                                              const void *x, uint32_t x_dtype, void *y, uint32_t y_dtype,
                                              uint32_t tokens, const muser_cuda_epilogue *ep, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    const Weight *g = reinterpret_cast<const Weight *>(gp), *u = reinterpret_cast<const Weight *>(up);
    const bool fp4 = g && g->dtype == MUSER_DTYPE_NVFP4_E2M1;
    muser_cuda_status st = check_io(ctx, g, x, x_dtype, y, y_dtype, tokens, fp4);
    if (st != MUSER_CUDA_OK) return st;
    if (ep && (ep->row_scale || ep->residual || ep->swiglu))
        return fail(ctx, MUSER_CUDA_BAD_ARG, "the fused gate/up call takes only the input-norm fields of the epilogue");
    Epilogue e;
    st = take_epilogue(ctx, g, ep, &e);
    if (st != MUSER_CUDA_OK) return st;
    if (fp4) {
        st = nvfp4_pair_checks(ctx, g, u);
        if (st != MUSER_CUDA_OK) return st;
        const size_t tok_pad = ((size_t)tokens + 127) / 128 * 128;
        const size_t packed_bytes = tok_pad * (g->n_in / 2);
        const size_t scale_bytes = muser_cuda_nvfp4_swizzled_scale_bytes(tokens, g->n_in);
        if (packed_bytes + scale_bytes > ctx->workspace_bytes)
            return fail(ctx, MUSER_CUDA_WORKSPACE_TOO_SMALL,
                        "context workspace holds " + std::to_string(ctx->workspace_bytes) + " bytes, this call needs " +
                            std::to_string(packed_bytes + scale_bytes));
        uint8_t *xp = reinterpret_cast<uint8_t *>(ctx->workspace), *xs = xp + packed_bytes;
        MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        st = launch_nvfp4_quantize(ctx, x, x_dtype, tokens, g->n_in, g->input_scale_inv, xp, xs, (cudaStream_t)stream,
                                   e.norm_weight, e.norm_eps);
        if (st != MUSER_CUDA_OK) return st;
        return launch_nvfp4_gemm(ctx, g, xp, xs, y, y_dtype, tokens, Epilogue{}, (cudaStream_t)stream, u);
    }
    if (!u) return fail(ctx, MUSER_CUDA_BAD_ARG, "null up weight");
    if (!is_kquant(g->dtype) || g->dtype != u->dtype) return fail(ctx, MUSER_CUDA_UNSUPPORTED_DTYPE, "gate and up must share one dtype (K-quant or NVFP4)");
    if (g->n_in != u->n_in || g->n_out != u->n_out || g->k_off != u->k_off || g->nsb != u->nsb)
        return fail(ctx, MUSER_CUDA_BAD_SHAPE, "gate and up geometry differ");
    if (g->shard.axis == MUSER_SHARD_K) return fail(ctx, MUSER_CUDA_BAD_SHAPE, "silu cannot be applied to K-sharded partial sums");
    if (tokens > 16) return fail(ctx, MUSER_CUDA_BAD_SHAPE, "the fused K-quant gate/up call serves 1..16 tokens");
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_kquant_matmul(ctx, g, u, x, x_dtype, y, y_dtype, tokens, e, (cudaStream_t)stream);
}

muser_cuda_status muser_cuda_nvfp4_ffn_gate_up_silu_prequant(muser_cuda_ctx *c, const muser_cuda_weight *gp,
                                                             const muser_cuda_weight *up, const uint8_t *xp,
                                                             const uint8_t *xs, void *y, uint32_t y_dtype,
                                                             uint32_t tokens, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    const Weight *g = reinterpret_cast<const Weight *>(gp), *u = reinterpret_cast<const Weight *>(up);
    muser_cuda_status st = check_io(ctx, g, xp, MUSER_DTYPE_BF16, y, y_dtype, tokens, true);
    if (st != MUSER_CUDA_OK) return st;
    if (!xs || !aligned16(xs)) return fail(ctx, MUSER_CUDA_BAD_ALIGN, "activation scales must be 16-byte aligned");
    st = nvfp4_pair_checks(ctx, g, u);
    if (st != MUSER_CUDA_OK) return st;
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_nvfp4_gemm(ctx, g, xp, xs, y, y_dtype, tokens, Epilogue{}, (cudaStream_t)stream, u);
}

muser_cuda_status muser_cuda_nvfp4_ffn_gate_up_silu_requant(muser_cuda_ctx *c, const muser_cuda_weight *gp,
                                                            const muser_cuda_weight *up, const uint8_t *xp, const uint8_t *xs,
                                                            uint32_t tokens, float out_input_scale_inv, uint8_t *out_packed,
                                                            uint8_t *out_scales, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    const Weight *g = reinterpret_cast<const Weight *>(gp), *u = reinterpret_cast<const Weight *>(up);
    muser_cuda_status st = check_io(ctx, g, xp, MUSER_DTYPE_BF16, out_packed, MUSER_DTYPE_BF16, tokens, false);
    if (st != MUSER_CUDA_OK) return st;
    if (!xs || !aligned16(xs) || !out_scales || !aligned16(out_scales)) return fail(ctx, MUSER_CUDA_BAD_ALIGN, "scale planes must be 16-byte aligned");
    if (!(std::isfinite(out_input_scale_inv) && out_input_scale_inv > 0.0f)) return fail(ctx, MUSER_CUDA_NAN_SCALE, "input_scale_inv must be finite and positive");
    st = nvfp4_pair_checks(ctx, g, u);
    if (st != MUSER_CUDA_OK) return st;
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const NvFp4Out q{out_packed, out_scales, out_input_scale_inv};
    return launch_nvfp4_gemm(ctx, g, xp, xs, nullptr, MUSER_DTYPE_BF16, tokens, Epilogue{}, (cudaStream_t)stream, u, &q);
}

size_t muser_cuda_nvfp4_swizzled_scale_bytes(uint64_t rows, uint64_t n_in) {
    return (size_t)((rows + 127) / 128 * ((n_in + 63) / 64) * 512);
}

muser_cuda_status muser_cuda_quantize_nvfp4_activation(muser_cuda_ctx *c, const void *x, uint32_t x_dtype,
                                                       uint32_t tokens, uint64_t n_in, float isi, uint8_t *packed,
                                                       uint8_t *scales, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (!ctx || !x || !packed || !scales) return fail(ctx, MUSER_CUDA_BAD_ARG, "null argument");
    if (tokens == 0 || n_in == 0 || n_in % 16) return fail(ctx, MUSER_CUDA_BAD_SHAPE, "NVFP4 rows are grouped by 16");
    if (x_dtype != MUSER_DTYPE_F32 && x_dtype != MUSER_DTYPE_BF16) return fail(ctx, MUSER_CUDA_UNSUPPORTED_DTYPE, "activations must be f32 or bf16");
    if (!(std::isfinite(isi) && isi > 0.0f)) return fail(ctx, MUSER_CUDA_NAN_SCALE, "input_scale_inv must be finite and positive");
    if (!aligned16(x) || !aligned16(packed) || !aligned16(scales)) return fail(ctx, MUSER_CUDA_BAD_ALIGN, "buffers must be 16-byte aligned");
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_nvfp4_quantize(ctx, x, x_dtype, tokens, n_in, isi, packed, scales, (cudaStream_t)stream);
}

muser_cuda_status muser_cuda_rmsnorm_quantize_nvfp4_activation(muser_cuda_ctx *c, const void *x, uint32_t x_dtype,
                                                               uint32_t tokens, uint64_t n_in, const float *norm_weight,
                                                               float norm_eps, float isi, uint8_t *packed,
                                                               uint8_t *scales, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (!ctx || !x || !packed || !scales || !norm_weight) return fail(ctx, MUSER_CUDA_BAD_ARG, "null argument");
    if (tokens == 0 || n_in == 0 || n_in % 16) return fail(ctx, MUSER_CUDA_BAD_SHAPE, "NVFP4 rows are grouped by 16");
    if (x_dtype != MUSER_DTYPE_F32 && x_dtype != MUSER_DTYPE_BF16) return fail(ctx, MUSER_CUDA_UNSUPPORTED_DTYPE, "activations must be f32 or bf16");
    if (!(std::isfinite(isi) && isi > 0.0f)) return fail(ctx, MUSER_CUDA_NAN_SCALE, "input_scale_inv must be finite and positive");
    if (!(norm_eps >= 0.0f)) return fail(ctx, MUSER_CUDA_BAD_ARG, "norm_eps must be non-negative");
    if (!aligned16(x) || !aligned16(packed) || !aligned16(scales) || !aligned16(norm_weight))
        return fail(ctx, MUSER_CUDA_BAD_ALIGN, "buffers must be 16-byte aligned");
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_nvfp4_quantize(ctx, x, x_dtype, tokens, n_in, isi, packed, scales, (cudaStream_t)stream, norm_weight, norm_eps);
}

static muser_cuda_status nvfp4_checks(Ctx *ctx, const Weight *w, const muser_cuda_epilogue *ep, Epilogue *e, bool a16_ok = false) {
    if (w->dtype != MUSER_DTYPE_NVFP4_E2M1) return fail(ctx, MUSER_CUDA_UNSUPPORTED_DTYPE, "nvfp4_matmul takes NVFP4 weights");
    if (!w->has_input_scale_inv && !a16_ok)
        return fail(ctx, MUSER_CUDA_UNSUPPORTED_DTYPE, "this entry point is the W4A4 lane: the weight has no input_scale_inv (muser_cuda_nvfp4_matmul serves the weight-only lane)");
    return take_epilogue(ctx, w, ep, e);
}

muser_cuda_status muser_cuda_nvfp4_matmul_prequant(muser_cuda_ctx *c, const muser_cuda_weight *wp, const uint8_t *xp,
                                                   const uint8_t *xs, void *y, uint32_t y_dtype, uint32_t tokens,
                                                   const muser_cuda_epilogue *ep, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    const Weight *w = reinterpret_cast<const Weight *>(wp);
    muser_cuda_status st = check_io(ctx, w, xp, MUSER_DTYPE_BF16, y, y_dtype, tokens, true);
    if (st != MUSER_CUDA_OK) return st;
    if (!xs || !aligned16(xs)) return fail(ctx, MUSER_CUDA_BAD_ALIGN, "activation scales must be 16-byte aligned");
    Epilogue e;
    st = nvfp4_checks(ctx, w, ep, &e);
    if (st != MUSER_CUDA_OK) return st;
    if (ep && ep->swiglu) return fail(ctx, MUSER_CUDA_BAD_ARG, "gate and up are two weights: use muser_cuda_ffn_gate_up_silu for the fused SwiGLU form");
    if (e.norm_weight) return fail(ctx, MUSER_CUDA_BAD_ARG, "activations that are already quantized cannot be normalized: pass norm_weight to the quantizer");
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_nvfp4_gemm(ctx, w, xp, xs, y, y_dtype, tokens, e, (cudaStream_t)stream);
}

muser_cuda_status muser_cuda_nvfp4_matmul_group_prequant(muser_cuda_ctx *c, const muser_cuda_weight *const *wps, uint32_t n,
                                                         const uint8_t *xp, const uint8_t *xs, void *const *ys,
                                                         uint32_t y_dtype, uint32_t tokens, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (!ctx) return MUSER_CUDA_BAD_ARG;
    if (!wps || !ys || n < 2 || n > 4) return fail(ctx, MUSER_CUDA_BAD_ARG, "a group holds 2 to 4 weights");
    const Weight *ws[4];
    for (uint32_t i = 0; i < n; ++i) {
        ws[i] = reinterpret_cast<const Weight *>(wps[i]);
        if (!ws[i]) return fail(ctx, MUSER_CUDA_BAD_ARG, "null weight in the group");
        muser_cuda_status st = check_io(ctx, ws[i], xp, MUSER_DTYPE_BF16, ys[i], y_dtype, tokens, true);
        if (st != MUSER_CUDA_OK) return st;
        Epilogue e;
        st = nvfp4_checks(ctx, ws[i], nullptr, &e);
        if (st != MUSER_CUDA_OK) return st;
        if (ws[i]->n_in != ws[0]->n_in || ws[i]->input_scale_inv != ws[0]->input_scale_inv)
            return fail(ctx, MUSER_CUDA_BAD_SHAPE, "the weights of a group read the same quantized activations: same n_in, same input_scale_inv");
    }
    if (!xs || !aligned16(xs)) return fail(ctx, MUSER_CUDA_BAD_ALIGN, "activation scales must be 16-byte aligned");
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_nvfp4_gemm_group(ctx, ws, n, xp, xs, ys, y_dtype, tokens, (cudaStream_t)stream);
}

muser_cuda_status muser_cuda_nvfp4_matmul(muser_cuda_ctx *c, const muser_cuda_weight *wp, const void *x, uint32_t x_dtype,
                                          void *y, uint32_t y_dtype, uint32_t tokens, const muser_cuda_epilogue *ep,
                                          void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    const Weight *w = reinterpret_cast<const Weight *>(wp);
    muser_cuda_status st = check_io(ctx, w, x, x_dtype, y, y_dtype, tokens, true);
    if (st != MUSER_CUDA_OK) return st;
    Epilogue e;
    st = nvfp4_checks(ctx, w, ep, &e, true);
    if (st != MUSER_CUDA_OK) return st;
    if (ep && ep->swiglu) return fail(ctx, MUSER_CUDA_BAD_ARG, "gate and up are two weights: use muser_cuda_ffn_gate_up_silu for the fused SwiGLU form");
    if (!w->has_input_scale_inv) {
        // the weight-only lane (weights.rs:117-121): its result is the reference's f16-rounded dot, nothing is fused around it
        if (ep && (ep->row_scale || ep->residual || ep->norm_weight || e.out_scale != 1.0f || e.softcap > 0.0f))
            return fail(ctx, MUSER_CUDA_BAD_ARG, "the weight-only NVFP4 lane takes no epilogue");
        MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        return launch_nvfp4_a16(ctx, w, x, x_dtype, y, y_dtype, tokens, ctx->workspace, ctx->workspace_bytes, (cudaStream_t)stream);
    }
    const size_t tok_pad = ((size_t)tokens + 127) / 128 * 128;
    const size_t packed_bytes = tok_pad * (w->n_in / 2);
    const size_t scale_bytes = muser_cuda_nvfp4_swizzled_scale_bytes(tokens, w->n_in);
    if (packed_bytes + scale_bytes > ctx->workspace_bytes)
        return fail(ctx, MUSER_CUDA_WORKSPACE_TOO_SMALL,
                    "context workspace holds " + std::to_string(ctx->workspace_bytes) + " bytes, this call needs " +
                        std::to_string(packed_bytes + scale_bytes));
    uint8_t *xp = reinterpret_cast<uint8_t *>(ctx->workspace), *xs = xp + packed_bytes;
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    st = launch_nvfp4_quantize(ctx, x, x_dtype, tokens, w->n_in, w->input_scale_inv, xp, xs, (cudaStream_t)stream,
                               e.norm_weight, e.norm_eps);
    if (st != MUSER_CUDA_OK) return st;
    return launch_nvfp4_gemm(ctx, w, xp, xs, y, y_dtype, tokens, e, (cudaStream_t)stream);
}

muser_cuda_status muser_cuda_fp4_peak_probe(muser_cuda_ctx *c, uint32_t iters, double *flops, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (!ctx || !flops || iters == 0 || iters > (1u << 20)) return fail(ctx, MUSER_CUDA_BAD_ARG, "bad probe arguments");
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_nvfp4_peak(ctx, iters, flops, (cudaStream_t)stream);
}

muser_cuda_status muser_cuda_fp4_pipe_probe(muser_cuda_ctx *c, uint32_t mode, uint32_t iters, uint32_t load_kib, uint32_t random_data, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (!ctx || iters == 0 || iters > (1u << 20)) return fail(ctx, MUSER_CUDA_BAD_ARG, "bad probe arguments");
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_nvfp4_pipe_probe(ctx, mode, iters, load_kib, random_data, (cudaStream_t)stream);
}

muser_cuda_status muser_cuda_wait_probe(muser_cuda_ctx *c, uint32_t polls, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (!ctx || polls == 0 || polls > (1u << 16)) return fail(ctx, MUSER_CUDA_BAD_ARG, "polls must be 1..65536");
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    wait_probe_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(polls, ctx->dev_status);
    MUSER_CUDA_TRY(ctx, cudaGetLastError());
    return MUSER_CUDA_OK;
}

muser_cuda_status muser_cuda_f16_mma_probe(muser_cuda_ctx *c, uint32_t n_cols, uint32_t iters, double *cycles_per_mma) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (!ctx || !cycles_per_mma || iters == 0) return fail(ctx, MUSER_CUDA_BAD_ARG, "null argument");
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    MUSER_CUDA_TRY(ctx, cudaDeviceSynchronize()); // the probe borrows the split-K scratch
    return launch_f16_mma_probe(ctx, n_cols, iters, cycles_per_mma);
}

muser_cuda_status muser_cuda_matmul_host_enqueue(muser_cuda_ctx *c, const muser_cuda_weight *wp, const float *x_host,
                                                 uint32_t tokens, float *y_host, void *stream_) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    const Weight *w = reinterpret_cast<const Weight *>(wp);
    cudaStream_t s = (cudaStream_t)stream_;
    if (!ctx || !w || !x_host || !y_host || tokens == 0) return fail(ctx, MUSER_CUDA_BAD_ARG, "null argument");
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const size_t xb = (size_t)tokens * w->n_in * 4, yb = (size_t)tokens * w->n_out * 4;
    const size_t need = (xb + 255) / 256 * 256 + (yb + 255) / 256 * 256;
    if (ctx->arena_used + need > ctx->arena_bytes) {
        // out of staging: wait for what is in flight, then start over (and grow, for a call larger than the arena)
        MUSER_CUDA_TRY(ctx, cudaStreamSynchronize(s));
        ctx->arena_used = 0;
        if (need > ctx->arena_bytes) {
            cudaFree(ctx->arena);
            ctx->arena = nullptr;
            ctx->arena_bytes = 0;
            const size_t want = need > ((size_t)64 << 20) ? need : ((size_t)64 << 20);
            MUSER_CUDA_TRY(ctx, cudaMalloc(&ctx->arena, want));
            ctx->arena_bytes = want;
        }
    }
    uint8_t *dx = reinterpret_cast<uint8_t *>(ctx->arena) + ctx->arena_used, *dy = dx + (xb + 255) / 256 * 256;
    ctx->arena_used += need;
    MUSER_CUDA_TRY(ctx, cudaMemcpyAsync(dx, x_host, xb, cudaMemcpyHostToDevice, s));
    muser_cuda_status st = MUSER_CUDA_OK;
    if (w->dtype == MUSER_DTYPE_NVFP4_E2M1) {
        st = muser_cuda_nvfp4_matmul(c, wp, dx, MUSER_DTYPE_F32, dy, MUSER_DTYPE_F32, tokens, nullptr, s);
    } else {
        for (uint32_t t0 = 0; t0 < tokens && st == MUSER_CUDA_OK; t0 += 64) {
            const uint32_t n = tokens - t0 < 64 ? tokens - t0 : 64;
            st = muser_cuda_quantized_matmul(c, wp, dx + (size_t)t0 * w->n_in * 4, MUSER_DTYPE_F32,
                                             dy + (size_t)t0 * w->n_out * 4, MUSER_DTYPE_F32, n, nullptr, s);
        }
    }
    if (st != MUSER_CUDA_OK) return st;
    MUSER_CUDA_TRY(ctx, cudaMemcpyAsync(y_host, dy, yb, cudaMemcpyDeviceToHost, s));
    return MUSER_CUDA_OK;
}

// Staged outputs -> the caller's pinned host buffers, 16 bytes a lane, every warp a contiguous 512 bytes.
struct HostScatter {
    static constexpr uint32_t kMax = 12;
    const uint4 *src[kMax];
    uint4 *dst[kMax];
    uint32_t n16[kMax];
    uint32_t n;
};
static __global__ void __launch_bounds__(256) host_scatter_kernel(const HostScatter t) {
    for (uint32_t e = 0; e < t.n; ++e)
        for (uint32_t i = blockIdx.x * 256 + threadIdx.x; i < t.n16[e]; i += gridDim.x * 256) t.dst[e][i] = t.src[e][i];
}

muser_cuda_status muser_cuda_matmul_host_groups_enqueue(muser_cuda_ctx *c, const muser_cuda_host_group *groups, uint32_t n_groups,
                                                        void *stream_) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    cudaStream_t s = (cudaStream_t)stream_;
    if (!ctx || !groups || n_groups == 0) return fail(ctx, MUSER_CUDA_BAD_ARG, "null argument");
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    size_t need = 0;
    for (uint32_t gi = 0; gi < n_groups; ++gi) {
        const muser_cuda_host_group &g = groups[gi];
        if (g.n_items == 0 || g.n_items > 4 || !g.x_host || g.tokens == 0 || g.tokens > 16)
            return fail(ctx, MUSER_CUDA_BAD_SHAPE, "a host group holds 1..4 projections of 1..16 tokens");
        for (uint32_t i = 0; i < g.n_items; ++i)
            if (!g.w[i] || !g.y_host[i]) return fail(ctx, MUSER_CUDA_BAD_ARG, "null argument");
        need += ((size_t)g.tokens * reinterpret_cast<const Weight *>(g.w[0])->n_in * 4 + 255) / 256 * 256;
        for (uint32_t i = 0; i < g.n_items; ++i) need += ((size_t)g.tokens * reinterpret_cast<const Weight *>(g.w[i])->n_out * 4 + 255) / 256 * 256;
    }
    if (ctx->arena_used + need > ctx->arena_bytes) {
        cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
        MUSER_CUDA_TRY(ctx, cudaStreamIsCapturing(s, &capturing));
        if (capturing != cudaStreamCaptureStatusNone)
            return fail(ctx, MUSER_CUDA_WORKSPACE_TOO_SMALL, "the staging arena is full and cannot be rewound during a stream capture: call muser_cuda_sync_status first");
        MUSER_CUDA_TRY(ctx, cudaStreamSynchronize(s));
        ctx->arena_used = 0;
        if (need > ctx->arena_bytes) {
            cudaFree(ctx->arena);
            ctx->arena = nullptr;
            ctx->arena_bytes = 0;
            const size_t want = need > ((size_t)64 << 20) ? need : ((size_t)64 << 20);
            MUSER_CUDA_TRY(ctx, cudaMalloc(&ctx->arena, want));
            ctx->arena_bytes = want;
        }
    }
    uint8_t *const first = reinterpret_cast<uint8_t *>(ctx->arena) + ctx->arena_used;
    ctx->arena_used += need;
    // The inputs travel on the context's copy stream, each followed by an event that its launch waits for: a small
    // host-to-device copy takes several microseconds to land, and on the launches' own stream every kernel would
    // wait for all the copies issued before it.
    constexpr uint32_t kEvents = 32;
    if (n_groups > kEvents - 4) return fail(ctx, MUSER_CUDA_BAD_SHAPE, "at most 28 groups per call");
    if (!ctx->copy_events[0])
        for (uint32_t i = 0; i < kEvents; ++i) MUSER_CUDA_TRY(ctx, cudaEventCreateWithFlags(&ctx->copy_events[i], cudaEventDisableTiming));
    // the copy stream's work hangs off `stream` at both ends, so the call can be captured into a CUDA graph from there
    MUSER_CUDA_TRY(ctx, cudaEventRecord(ctx->copy_events[kEvents - 3], s));
    MUSER_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->copy_stream, ctx->copy_events[kEvents - 3], 0));
    uint8_t *at = first;
    for (uint32_t gi = 0; gi < n_groups; ++gi) { // pass 1: inputs
        const muser_cuda_host_group &g = groups[gi];
        const size_t xb = (size_t)g.tokens * reinterpret_cast<const Weight *>(g.w[0])->n_in * 4;
        MUSER_CUDA_TRY(ctx, cudaMemcpyAsync(at, g.x_host, xb, cudaMemcpyHostToDevice, ctx->copy_stream));
        MUSER_CUDA_TRY(ctx, cudaEventRecord(ctx->copy_events[gi], ctx->copy_stream));
        at += (xb + 255) / 256 * 256;
        for (uint32_t i = 0; i < g.n_items; ++i) at += ((size_t)g.tokens * reinterpret_cast<const Weight *>(g.w[i])->n_out * 4 + 255) / 256 * 256;
    }
    // Pass 2: the launches, back to back.  Outputs are written to the arena and leave in batches: after every four
    // groups one small kernel on the copy stream stores them into the caller's pinned buffers with full-width,
    // contiguous stores (the bus takes those at several times the rate of the projection kernel's own 32-byte
    // pieces), beside the next groups' projections.  Buffers the device cannot address get a plain copy instead.
    HostScatter batch;
    batch.n = 0;
    bool copies_pending = false;
    // mode 2: the copy engine takes the outputs (one copy each) on the copy stream, behind an event of the launch that
    // produced them; it needs no SM, so it runs beside the next launches, which fill every SM's registers
    struct PendingCopy { void *dst; const void *src; size_t bytes; };
    PendingCopy pending[4];
    uint32_t n_pending = 0;
    auto flush = [&]() -> cudaError_t {
        if (batch.n == 0 && n_pending == 0) return cudaSuccess;
        cudaError_t e = cudaEventRecord(ctx->copy_events[kEvents - 1], s);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->copy_stream, ctx->copy_events[kEvents - 1], 0);
        if (e != cudaSuccess) return e;
        for (uint32_t i = 0; i < n_pending && e == cudaSuccess; ++i)
            e = cudaMemcpyAsync(pending[i].dst, pending[i].src, pending[i].bytes, cudaMemcpyDeviceToHost, ctx->copy_stream);
        n_pending = 0;
        if (e != cudaSuccess) return e;
        copies_pending = true;
        if (batch.n == 0) return cudaSuccess;
        host_scatter_kernel<<<32, 256, 0, ctx->copy_stream>>>(batch);
        batch.n = 0;
        return cudaGetLastError();
    };
    at = first;
    for (uint32_t gi = 0; gi < n_groups; ++gi) {
        const muser_cuda_host_group &g = groups[gi];
        MUSER_CUDA_TRY(ctx, cudaStreamWaitEvent(s, ctx->copy_events[gi], 0));
        uint8_t *dx = at;
        at += ((size_t)g.tokens * reinterpret_cast<const Weight *>(g.w[0])->n_in * 4 + 255) / 256 * 256;
        muser_cuda_group_item items[4];
        uint8_t *staged[4];
        for (uint32_t i = 0; i < g.n_items; ++i) {
            staged[i] = at;
            items[i].w = g.w[i], items[i].y = at, items[i].y_dtype = MUSER_DTYPE_F32, items[i].reserved = 0, items[i].epilogue = nullptr;
            at += ((size_t)g.tokens * reinterpret_cast<const Weight *>(g.w[i])->n_out * 4 + 255) / 256 * 256;
        }
        const muser_cuda_status st = muser_cuda_quantized_matmul_group(c, items, g.n_items, dx, MUSER_DTYPE_F32, g.tokens, s);
        if (st != MUSER_CUDA_OK) return st;
        for (uint32_t i = 0; i < g.n_items; ++i) {
            const size_t yb = (size_t)g.tokens * reinterpret_cast<const Weight *>(g.w[i])->n_out * 4;
            void *mapped = nullptr;
            if (ctx->host_direct_output == 2) {
                pending[n_pending++] = PendingCopy{g.y_host[i], staged[i], yb};
            } else if (ctx->host_direct_output == 1 && cudaHostGetDevicePointer(&mapped, g.y_host[i], 0) == cudaSuccess && ((uintptr_t)mapped & 15u) == 0 && yb % 16 == 0) {
                batch.src[batch.n] = reinterpret_cast<const uint4 *>(staged[i]);
                batch.dst[batch.n] = reinterpret_cast<uint4 *>(mapped);
                batch.n16[batch.n] = (uint32_t)(yb / 16);
                if (++batch.n == HostScatter::kMax) MUSER_CUDA_TRY(ctx, flush());
            } else {
                (void)cudaGetLastError();
                MUSER_CUDA_TRY(ctx, cudaMemcpyAsync(g.y_host[i], staged[i], yb, cudaMemcpyDeviceToHost, s));
            }
        }
        if ((gi & 3) == 3 || n_pending) MUSER_CUDA_TRY(ctx, flush()); // (a store kernel per group measured slower than one per four; copies leave per group)
    }
    MUSER_CUDA_TRY(ctx, flush());
    (void)copies_pending; // the caller's wait on `stream` covers the copy stream's stores
    MUSER_CUDA_TRY(ctx, cudaEventRecord(ctx->copy_events[kEvents - 2], ctx->copy_stream));
    MUSER_CUDA_TRY(ctx, cudaStreamWaitEvent(s, ctx->copy_events[kEvents - 2], 0));
    return MUSER_CUDA_OK;
}

muser_cuda_status muser_cuda_matmul_host(muser_cuda_ctx *c, const muser_cuda_weight *wp, const float *x_host,
                                         uint32_t tokens, float *y_host) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    const Weight *w = reinterpret_cast<const Weight *>(wp);
    if (!ctx || !w || !x_host || !y_host || tokens == 0) return fail(ctx, MUSER_CUDA_BAD_ARG, "null argument");
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const size_t xb = (size_t)tokens * w->n_in * 4, yb = (size_t)tokens * w->n_out * 4;
    const size_t need = (xb + 255) / 256 * 256 + yb;
    if (need > ctx->dev_stage_bytes) { // grows on first use / larger shapes only
        cudaFree(ctx->dev_stage);
        if (ctx->host_stage) cudaFreeHost(ctx->host_stage);
        ctx->dev_stage = ctx->host_stage = nullptr;
        ctx->dev_stage_bytes = 0;
        MUSER_CUDA_TRY(ctx, cudaMalloc(&ctx->dev_stage, need));
        MUSER_CUDA_TRY(ctx, cudaMallocHost(&ctx->host_stage, need));
        ctx->dev_stage_bytes = ctx->host_stage_bytes = need;
    }
    uint8_t *dx = reinterpret_cast<uint8_t *>(ctx->dev_stage), *dy = dx + (xb + 255) / 256 * 256;
    uint8_t *hx = reinterpret_cast<uint8_t *>(ctx->host_stage), *hy = hx + (xb + 255) / 256 * 256;
    std::memcpy(hx, x_host, xb);
    cudaStream_t s = ctx->copy_stream;
    MUSER_CUDA_TRY(ctx, cudaMemcpyAsync(dx, hx, xb, cudaMemcpyHostToDevice, s));
    muser_cuda_status st;
    if (w->dtype == MUSER_DTYPE_NVFP4_E2M1) {
        st = muser_cuda_nvfp4_matmul(c, wp, dx, MUSER_DTYPE_F32, dy, MUSER_DTYPE_F32, tokens, nullptr, s);
    } else {
        st = MUSER_CUDA_OK;
        for (uint32_t t0 = 0; t0 < tokens && st == MUSER_CUDA_OK; t0 += 64) {
            const uint32_t n = tokens - t0 < 64 ? tokens - t0 : 64;
            st = muser_cuda_quantized_matmul(c, wp, dx + (size_t)t0 * w->n_in * 4, MUSER_DTYPE_F32,
                                             dy + (size_t)t0 * w->n_out * 4, MUSER_DTYPE_F32, n, nullptr, s);
        }
    }
    if (st != MUSER_CUDA_OK) return st;
    MUSER_CUDA_TRY(ctx, cudaMemcpyAsync(hy, dy, yb, cudaMemcpyDeviceToHost, s));
    MUSER_CUDA_TRY(ctx, cudaStreamSynchronize(s));
    std::memcpy(y_host, hy, yb);
    return MUSER_CUDA_OK;
}

} // extern "C"
