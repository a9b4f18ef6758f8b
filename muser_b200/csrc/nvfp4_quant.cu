// NVFP4 activation quantizer: f32/bf16 rows -> packed E2M1 codes + one E4M3FN scale per 16 values.
//
// Reproduces quant::activation_group_codes / quantize_nvfp4_activation bit for bit
// (crates/muser-engine/src/quant/nvfp4.rs:173-238): round to f16, amax/6 * input_scale_inv saturated at 448
// and rounded to E4M3 (nearest, ties to even), then threshold compares of |x| * input_scale_inv against
// scale * {0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5} with the reference's <= / < pattern.  Scales are written in
// the 128-row x 4-group swizzle of scripts/gx10/vllm/muser_vllm/exact_fp4_quant.py:149-162, which is also
// the order the block-scaled MMA wants them in tensor memory.
#include "common.cuh"
#include "nvfp4_codec.cuh"
#include "rmsnorm.cuh"

namespace muser {

// Four neighbouring threads (groups 4q .. 4q+3 of one row) merge their scale bytes into one aligned 32-bit store.
// Every lane of the warp calls this; lanes past the row's last group slot pass live = false.
__device__ __forceinline__ void store_scale_quad(uint32_t scale_code, uint32_t row, uint32_t grp, uint32_t kt, uint8_t *scales,
                                                 bool live = true) {
    uint32_t word = scale_code;
    word |= __shfl_down_sync(0xffffffffu, scale_code, 1) << 8;
    word |= __shfl_down_sync(0xffffffffu, scale_code, 2) << 16;
    word |= __shfl_down_sync(0xffffffffu, scale_code, 3) << 24;
    if (live && (grp & 3) == 0) {
        const size_t off = (size_t)(row / 128) * ((size_t)kt * 512) + (size_t)(grp / 4) * 512 + (row % 32) * 16 + ((row % 128) / 32) * 4;
        *reinterpret_cast<uint32_t *>(scales + off) = word;
    }
}

// One thread per 16-value group; the four threads of a 64-value span merge their scale bytes into one
// aligned 32-bit store.  Rows tokens..tokens_pad-1 only clear their scale slots.
template <bool XF32>
__global__ void nvfp4_quantize_kernel(const void *__restrict__ x, uint32_t tokens, uint32_t tokens_pad, uint32_t n_in,
                                      uint32_t kt, float isi, uint8_t *__restrict__ packed,
                                      uint8_t *__restrict__ scales) {
    const uint32_t groups_pad = kt * 4; // group slots per row in the swizzled plane
    const uint64_t idx = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
    if (idx >= (uint64_t)tokens_pad * groups_pad) return; // groups_pad % 4 == 0: quads never straddle the edge
    const uint32_t row = (uint32_t)(idx / groups_pad), grp = (uint32_t)(idx % groups_pad);
    uint32_t scale_code = 0;
    if (row < tokens && grp * 16 < n_in) {
        float r[16];
        if constexpr (XF32) {
            const float4 *p = reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(x) + (size_t)row * n_in + grp * 16);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 v = __ldg(p + i);
                r[4 * i] = v.x, r[4 * i + 1] = v.y, r[4 * i + 2] = v.z, r[4 * i + 3] = v.w;
            }
        } else {
            const uint4 *p = reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(x) + (size_t)row * n_in + grp * 16);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint4 v = __ldg(p + i);
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    r[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
                    r[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
                }
            }
        }
        scale_code = quantize_group(r, isi, packed + (size_t)row * (n_in / 2) + grp * 8);
    }
    store_scale_quad(scale_code, row, grp, kt, scales);
}

// 1 / sqrt(mean(x^2) + eps) per row with the squares added FRONT TO BACK in f32, one rounding per step, exactly as
// rms_norm does on the CPU lane (crates/muser-engine/src/reference.rs:59-72).  The order matters here more than
// anywhere else on the path: the NVFP4 quantizer that consumes the normalized row is a chain of threshold compares,
// so a factor that differs in its last bits flips a 4-bit code now and then, and one flipped code moves that
// token's outputs by a few 1e-3 of their norm.  One thread owns one row's chain; its warp stages 256 inputs of its 32
// rows at a time through shared memory (asynchronous copies, two buffers), so that global loads stay coalesced
// (consecutive threads read consecutive 16 bytes of one row) while the sums stay sequential.
template <bool XF32>
__global__ void __launch_bounds__(32) rms_rows_sequential_kernel(const void *__restrict__ x, uint32_t tokens, uint32_t n_in, float eps,
                                                                 float *__restrict__ inv_rms) {
    constexpr int kRows = 32, kChunk = 256;                       // rows per block (one warp), inputs per row and step
    constexpr int kParts = kChunk * (XF32 ? 4 : 2) / 16;          // 16-byte pieces per row and step
    constexpr int kStride = kParts + 1;                           // row stride in pieces: conflict-free 16-byte reads down a column
    extern __shared__ uint4 rms_tile[];                           // two buffers of kRows x kStride pieces
    const uint32_t row0 = blockIdx.x * kRows, lane = threadIdx.x, my_row = row0 + lane;
    const size_t row_bytes = (size_t)n_in * (XF32 ? 4 : 2);
    const uint8_t *base = reinterpret_cast<const uint8_t *>(x);
    const uint32_t steps = (n_in + kChunk - 1) / kChunk;
    // the next step's pieces travel global -> shared asynchronously while this step's chain runs
    auto stage = [&](uint32_t step, uint4 *buf) {
        const uint32_t k0 = step * kChunk;
        const uint32_t parts_here = min((uint32_t)kParts, (n_in - k0) * (XF32 ? 4u : 2u) / 16u);
        for (uint32_t i = lane; i < kRows * kParts; i += 32) {
            const uint32_t r = i / kParts, part = i % kParts;
            uint4 *dst = buf + r * kStride + part;
            if (row0 + r < tokens && part < parts_here) {
                const void *src = base + (size_t)(row0 + r) * row_bytes + (size_t)k0 * (XF32 ? 4 : 2) + (size_t)part * 16;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
            } else {
                *dst = make_uint4(0, 0, 0, 0); // zeros add nothing to the chain
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float ss = 0.0f;
    stage(0, rms_tile);
    for (uint32_t step = 0; step < steps; ++step) {
        uint4 *cur = rms_tile + (step & 1) * (kRows * kStride);
        if (step + 1 < steps) {
            stage(step + 1, rms_tile + ((step + 1) & 1) * (kRows * kStride));
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncwarp();
#pragma unroll 4
        for (int part = 0; part < kParts; ++part) {
            const uint4 v = cur[lane * kStride + part];
            if constexpr (XF32) {
                const float f[4] = {__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w)};
#pragma unroll
                for (int i = 0; i < 4; ++i) ss = __fadd_rn(ss, __fmul_rn(f[i], f[i]));
            } else {
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float lo = __uint_as_float(w[i] << 16), hi = __uint_as_float(w[i] & 0xFFFF0000u);
                    ss = __fadd_rn(ss, __fmul_rn(lo, lo));
                    ss = __fadd_rn(ss, __fmul_rn(hi, hi));
                }
            }
        }
        __syncwarp(); // this buffer is refilled by the step after next
    }
    if (my_row < tokens) inv_rms[my_row] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)n_in), eps)));
}

static cudaError_t launch_rms_rows_sequential(Ctx *ctx, const void *x, uint32_t x_dtype, uint32_t tokens, uint32_t n_in, float eps,
                                              float *inv_rms, cudaStream_t stream) {
    const unsigned blocks = (tokens + 31) / 32;
    const bool f32 = x_dtype == MUSER_DTYPE_F32;
    const size_t smem = (size_t)2 * 32 * ((f32 ? 64 : 32) + 1) * sizeof(uint4);
    const void *fn = f32 ? reinterpret_cast<const void *>(rms_rows_sequential_kernel<true>) : reinterpret_cast<const void *>(rms_rows_sequential_kernel<false>);
    const cudaError_t e = ensure_dynamic_smem(fn, ctx->device, smem);
    if (e != cudaSuccess) return e;
    if (f32) rms_rows_sequential_kernel<true><<<blocks, 32, smem, stream>>>(x, tokens, n_in, eps, inv_rms);
    else rms_rows_sequential_kernel<false><<<blocks, 32, smem, stream>>>(x, tokens, n_in, eps, inv_rms);
    return cudaGetLastError();
}

// The same quantizer behind a fused input RMSNorm (reference.rs:73-80): one block per token row quantizes
// (x * inv_rms) * w group by group, inv_rms from the pass above.  Blocks of the padding rows only clear scales.
template <bool XF32>
__global__ void __launch_bounds__(256) nvfp4_norm_quantize_kernel(const void *__restrict__ x, uint32_t tokens, uint32_t n_in,
                                                                  uint32_t kt, float isi, const float *__restrict__ norm_w,
                                                                  const float *__restrict__ inv_rms, uint8_t *__restrict__ packed,
                                                                  uint8_t *__restrict__ scales) {
    const uint32_t row = blockIdx.x, groups_pad = kt * 4;
    const void *xr = XF32 ? (const void *)(reinterpret_cast<const float *>(x) + (size_t)row * n_in)
                          : (const void *)(reinterpret_cast<const __nv_bfloat16 *>(x) + (size_t)row * n_in);
    const float inv = row < tokens ? inv_rms[row] : 0.0f;
    for (uint32_t g0 = 0; g0 < groups_pad; g0 += blockDim.x) { // blockDim % 4 == 0: quads stay together
        const uint32_t grp = g0 + threadIdx.x;
        uint32_t scale_code = 0;
        if (row < tokens && grp * 16 < n_in) {
            float r[16], a[8], b[8];
            load8<XF32>(xr, 2 * grp, a);
            load8<XF32>(xr, 2 * grp + 1, b);
            const float4 *wp = reinterpret_cast<const float4 *>(norm_w + grp * 16);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 w = __ldg(wp + i);
                const float *src = i < 2 ? a + 4 * i : b + 4 * (i - 2);
                r[4 * i] = __fmul_rn(__fmul_rn(src[0], inv), w.x);
                r[4 * i + 1] = __fmul_rn(__fmul_rn(src[1], inv), w.y);
                r[4 * i + 2] = __fmul_rn(__fmul_rn(src[2], inv), w.z);
                r[4 * i + 3] = __fmul_rn(__fmul_rn(src[3], inv), w.w);
            }
            scale_code = quantize_group(r, isi, packed + (size_t)row * (n_in / 2) + grp * 8);
        }
        store_scale_quad(scale_code, row, grp, kt, scales, grp < groups_pad);
    }
}

// Plain rows: out[t][k] = (x[t][k] * inv_rms_t) * w[k] in f32, for the kernels that read their activations as they go.
template <bool XF32>
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const void *__restrict__ x, uint32_t n_in, const float *__restrict__ norm_w,
                                                           const float *__restrict__ inv_rms, float *__restrict__ out) {
    const uint32_t row = blockIdx.x;
    const void *xr = XF32 ? (const void *)(reinterpret_cast<const float *>(x) + (size_t)row * n_in)
                          : (const void *)(reinterpret_cast<const __nv_bfloat16 *>(x) + (size_t)row * n_in);
    const float inv = inv_rms[row];
    for (uint32_t i = threadIdx.x; i < n_in / 8; i += blockDim.x) {
        float v[8];
        load8<XF32>(xr, i, v);
        const float4 w0 = __ldg(reinterpret_cast<const float4 *>(norm_w) + 2 * i), w1 = __ldg(reinterpret_cast<const float4 *>(norm_w) + 2 * i + 1);
        float4 *o = reinterpret_cast<float4 *>(out + (size_t)row * n_in) + 2 * i;
        o[0] = make_float4(__fmul_rn(__fmul_rn(v[0], inv), w0.x), __fmul_rn(__fmul_rn(v[1], inv), w0.y),
                           __fmul_rn(__fmul_rn(v[2], inv), w0.z), __fmul_rn(__fmul_rn(v[3], inv), w0.w));
        o[1] = make_float4(__fmul_rn(__fmul_rn(v[4], inv), w1.x), __fmul_rn(__fmul_rn(v[5], inv), w1.y),
                           __fmul_rn(__fmul_rn(v[6], inv), w1.z), __fmul_rn(__fmul_rn(v[7], inv), w1.w));
    }
}

muser_cuda_status launch_rmsnorm_rows(Ctx *ctx, const void *x, uint32_t x_dtype, uint32_t tokens, uint64_t n_in,
                                      const float *norm_weight, float norm_eps, float *out, cudaStream_t stream) {
    // the factors sit behind the rows in the same scratch (the caller sized it for tokens x n_in floats and more)
    float *inv = ctx->inv_rms;
    if (tokens > ctx->inv_rms_rows) return fail(ctx, MUSER_CUDA_WORKSPACE_TOO_SMALL, "fused input norm: more rows than the context's per-row scratch holds");
    MUSER_CUDA_TRY(ctx, launch_rms_rows_sequential(ctx, x, x_dtype, tokens, (uint32_t)n_in, norm_eps, inv, stream));
    if (x_dtype == MUSER_DTYPE_F32)
        rmsnorm_rows_kernel<true><<<tokens, 256, 0, stream>>>(x, (uint32_t)n_in, norm_weight, inv, out);
    else
        rmsnorm_rows_kernel<false><<<tokens, 256, 0, stream>>>(x, (uint32_t)n_in, norm_weight, inv, out);
    MUSER_CUDA_TRY(ctx, cudaGetLastError());
    return MUSER_CUDA_OK;
}

muser_cuda_status launch_nvfp4_quantize(Ctx *ctx, const void *x, uint32_t x_dtype, uint32_t tokens, uint64_t n_in,
                                        float isi, uint8_t *packed, uint8_t *scales, cudaStream_t stream,
                                        const float *norm_weight, float norm_eps) {
    const uint32_t kt = (uint32_t)((n_in + 63) / 64);
    const uint32_t tokens_pad = (tokens + 127) / 128 * 128;
    if (norm_weight) {
        float *inv = ctx->inv_rms;
        if (!inv || tokens > ctx->inv_rms_rows) return fail(ctx, MUSER_CUDA_WORKSPACE_TOO_SMALL, "fused input norm: more rows than the context's per-row scratch holds");
        MUSER_CUDA_TRY(ctx, launch_rms_rows_sequential(ctx, x, x_dtype, tokens, (uint32_t)n_in, norm_eps, inv, stream));
        if (x_dtype == MUSER_DTYPE_F32)
            nvfp4_norm_quantize_kernel<true><<<tokens_pad, 256, 0, stream>>>(x, tokens, (uint32_t)n_in, kt, isi, norm_weight, inv, packed, scales);
        else
            nvfp4_norm_quantize_kernel<false><<<tokens_pad, 256, 0, stream>>>(x, tokens, (uint32_t)n_in, kt, isi, norm_weight, inv, packed, scales);
        MUSER_CUDA_TRY(ctx, cudaGetLastError());
        return MUSER_CUDA_OK;
    }
    const uint64_t total = (uint64_t)tokens_pad * kt * 4;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (x_dtype == MUSER_DTYPE_F32)
        nvfp4_quantize_kernel<true><<<blocks, 256, 0, stream>>>(x, tokens, tokens_pad, (uint32_t)n_in, kt, isi, packed, scales);
    else
        nvfp4_quantize_kernel<false><<<blocks, 256, 0, stream>>>(x, tokens, tokens_pad, (uint32_t)n_in, kt, isi, packed, scales);
    MUSER_CUDA_TRY(ctx, cudaGetLastError());
    return MUSER_CUDA_OK;
}

} // namespace muser
