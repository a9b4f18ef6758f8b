// The step either side of the projections, so that a layer's non-attention work can stay on the device between two
// projection calls: the sandwich-norm tail, the attention output gate, and the per-head QK norm.
//
// Reference semantics (CPU lane, f32): crates/muser-engine/src/reference.rs:59-80 (rms_norm, rms_norm_mul),
// :384-393 (per-head norm of q and k), :447-455 (sigmoid gate in front of o_proj), :466-480 and :530-542 (post-norm
// with its own epsilon, then the residual), :484-490 (the next pre-norm).  On the reference's GPU path the tail is one
// kernel, muser_fused_norm_residual_rms_norm_32sg (src/shaders/ferrite/rmsnorm_batch_tail.metal:147-200):
//     hidden += rms_norm(src, eps1) * weight1;  output = rms_norm(hidden, eps2) * weight2
// Sums of squares are block-wide trees here (the CPU lane adds front to back, the shader in simdgroups): results
// agree to rounding, not bit for bit, and are compared by relative error.
#include "common.cuh"

namespace muser {

// Sum over the block of one value per thread; `red` holds 33 floats; every thread gets the total.
__device__ __forceinline__ float block_sum(float v, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = (blockDim.x + 31) >> 5;
    __syncthreads(); // `red` may still be read from an earlier call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < warps ? red[lane] : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// One block per token row.  n % 4 == 0; rows 16-byte aligned.
__global__ void __launch_bounds__(512) norm_residual_norm_kernel(float *__restrict__ hidden, const float *__restrict__ src, float *__restrict__ output,
                                                                 const float *__restrict__ w1, const float *__restrict__ w2, uint32_t n, float eps1,
                                                                 float eps2) {
    __shared__ float red[33];
    pdl_wait();
    const uint32_t n4 = n / 4;
    float4 *h4 = reinterpret_cast<float4 *>(hidden + (size_t)blockIdx.x * n);
    const float4 *s4 = reinterpret_cast<const float4 *>(src + (size_t)blockIdx.x * n);
    const float4 *w14 = reinterpret_cast<const float4 *>(w1), *w24 = reinterpret_cast<const float4 *>(w2);
    float ss = 0.0f;
    for (uint32_t i = threadIdx.x; i < n4; i += blockDim.x) {
        const float4 v = s4[i];
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    const float inv_src = __fdiv_rn(1.0f, __fsqrt_rn(__fdiv_rn(block_sum(ss, red), (float)n) + eps1));
    float sh = 0.0f;
    for (uint32_t i = threadIdx.x; i < n4; i += blockDim.x) {
        const float4 s = s4[i], w = w14[i];
        float4 h = h4[i];
        h.x += s.x * inv_src * w.x, h.y += s.y * inv_src * w.y, h.z += s.z * inv_src * w.z, h.w += s.w * inv_src * w.w;
        h4[i] = h;
        sh += h.x * h.x + h.y * h.y + h.z * h.z + h.w * h.w;
    }
    if (!output) return;
    const float inv_h = __fdiv_rn(1.0f, __fsqrt_rn(__fdiv_rn(block_sum(sh, red), (float)n) + eps2));
    float4 *o4 = reinterpret_cast<float4 *>(output + (size_t)blockIdx.x * n);
    for (uint32_t i = threadIdx.x; i < n4; i += blockDim.x) { // this thread re-reads what it wrote itself
        const float4 h = h4[i], w = w24[i];
        o4[i] = make_float4(h.x * inv_h * w.x, h.y * inv_h * w.y, h.z * inv_h * w.z, h.w * inv_h * w.w);
    }
}

// x[i] *= 1 / (1 + exp(-gate[i])), four at a time.
__global__ void __launch_bounds__(256) sigmoid_gate_kernel(float *__restrict__ x, const float *__restrict__ gate, size_t n4) {
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n4; i += (size_t)gridDim.x * 256) {
        float4 v = reinterpret_cast<float4 *>(x)[i];
        const float4 g = reinterpret_cast<const float4 *>(gate)[i];
        v.x *= __fdiv_rn(1.0f, 1.0f + expf(-g.x)), v.y *= __fdiv_rn(1.0f, 1.0f + expf(-g.y));
        v.z *= __fdiv_rn(1.0f, 1.0f + expf(-g.z)), v.w *= __fdiv_rn(1.0f, 1.0f + expf(-g.w));
        reinterpret_cast<float4 *>(x)[i] = v;
    }
}

// One warp per (token, head): x <- x * 1/sqrt(mean(x^2) + eps) * w, head_dim % 4 == 0, head_dim <= 1024.
__global__ void __launch_bounds__(256) head_rms_norm_kernel(float *__restrict__ x, const float *__restrict__ w, float eps, uint32_t heads_total,
                                                            uint32_t head_dim) {
    pdl_wait();
    const uint32_t head = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (head >= heads_total) return;
    float4 *row = reinterpret_cast<float4 *>(x + (size_t)head * head_dim);
    const float4 *w4 = reinterpret_cast<const float4 *>(w);
    const uint32_t n4 = head_dim / 4;
    float ss = 0.0f;
    for (uint32_t i = lane; i < n4; i += 32) {
        const float4 v = row[i];
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fdiv_rn(ss, (float)head_dim) + eps));
    for (uint32_t i = lane; i < n4; i += 32) {
        const float4 v = row[i], ww = w4[i];
        row[i] = make_float4(v.x * inv * ww.x, v.y * inv * ww.y, v.z * inv * ww.z, v.w * inv * ww.w);
    }
}

muser_cuda_status launch_norm_residual_norm(Ctx *ctx, float *hidden, const float *src, float *output, const float *w1, const float *w2,
                                            uint32_t tokens, uint32_t n, float eps1, float eps2, cudaStream_t stream) {
    const unsigned threads = n / 4 >= 512 ? 512 : n / 4 >= 256 ? 256 : 128;
    MUSER_CUDA_TRY(ctx, launch_pdl(norm_residual_norm_kernel, dim3(tokens), dim3(threads), 0, stream, hidden, src, output, w1, w2, n, eps1, eps2));
    return MUSER_CUDA_OK;
}

muser_cuda_status launch_sigmoid_gate(Ctx *ctx, float *x, const float *gate, size_t count, cudaStream_t stream) {
    const size_t n4 = count / 4;
    const unsigned blocks = (unsigned)std::min<size_t>((n4 + 255) / 256, (size_t)ctx->sm_count * 8);
    MUSER_CUDA_TRY(ctx, launch_pdl(sigmoid_gate_kernel, dim3(blocks), dim3(256), 0, stream, x, gate, n4));
    return MUSER_CUDA_OK;
}

muser_cuda_status launch_head_rms_norm(Ctx *ctx, float *x, const float *w, float eps, uint32_t tokens, uint32_t heads, uint32_t head_dim,
                                       cudaStream_t stream) {
    const uint32_t total = tokens * heads;
    MUSER_CUDA_TRY(ctx, launch_pdl(head_rms_norm_kernel, dim3((total + 7) / 8), dim3(256), 0, stream, x, w, eps, total, head_dim));
    return MUSER_CUDA_OK;
}

} // namespace muser
