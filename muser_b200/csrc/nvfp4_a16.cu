// The weight-only NVFP4 lane: y[t][r] = dot_nvfp4_a16_q8_f32(W_r, x_t), taken when a weight carries no
// input_scale_inv (crates/muser-engine/src/weights.rs:117-121).
//
// Reproduces quant::quantize_nvfp4_q8_block and dot_nvfp4_a16_q8_f32 bit for bit (src/quant/nvfp4.rs:62-99,348-379;
// the GB10 twin is scripts/gx10/vllm/muser_vllm/exact_fp4_a16_mm.py): every 256 activations are rounded to f16 and
// quantized to int8 against the FIRST element of largest magnitude (inverse scale -127 / that element, nearest
// through the 12582912 magic-number FMA, capped at 127); a block's contraction is an exact integer: E2M1 codes in
// halves times int8, the sum of a 16-group times its E4M3 scale in units of 2^-9, sixteen groups added in 64 bits;
// then four FMAs in a fixed order turn it into f32, the blocks are added front to back, and the result is rounded
// to f16.  Nothing here is approximate, so outputs are compared for equal bits.
//
// This is the lane for checkpoints without activation scales, not the prefill hot path: one warp per output row,
// the row's codes read once per group of eight tokens, every weight byte read with 4-byte loads.  The activations
// of a call are quantized once into the context workspace by a kernel of their own.
#include "common.cuh"

namespace muser {

// int8 codes [tokens][n_in] followed by one f32 d per (token, 256-block)
__global__ void __launch_bounds__(256) nvfp4_q8_quantize_kernel(const void *__restrict__ x, uint32_t x_f32, uint32_t n_in,
                                                                int8_t *__restrict__ qs, float *__restrict__ ds) {
    __shared__ float s_mag[8];
    __shared__ uint32_t s_idx[8];
    __shared__ float s_val[8];
    const uint32_t block = blockIdx.x, tok = blockIdx.y, i = threadIdx.x, blocks = n_in / 256;
    const size_t at = (size_t)tok * n_in + (size_t)block * 256 + i;
    const float raw = x_f32 ? reinterpret_cast<const float *>(x)[at] : __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(x)[at]);
    const float v = __half2float(__float2half_rn(raw));
    // first element of largest magnitude: larger magnitude wins, the lower index wins a tie
    float mag = v == v ? fabsf(v) : -1.0f, val = v; // a NaN never wins the reference's `>` scan
    uint32_t idx = i;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, mag, o), v2 = __shfl_xor_sync(0xffffffffu, val, o);
        const uint32_t i2 = __shfl_xor_sync(0xffffffffu, idx, o);
        if (m2 > mag || (m2 == mag && i2 < idx)) mag = m2, val = v2, idx = i2;
    }
    if ((i & 31) == 0) s_mag[i >> 5] = mag, s_idx[i >> 5] = idx, s_val[i >> 5] = val;
    __syncthreads();
    mag = s_mag[0], val = s_val[0], idx = s_idx[0];
#pragma unroll
    for (int w = 1; w < 8; ++w)
        if (s_mag[w] > mag || (s_mag[w] == mag && s_idx[w] < idx)) mag = s_mag[w], val = s_val[w], idx = s_idx[w];
    int q = 0;
    float d = 0.0f;
    if (mag > 0.0f) {
        const float inverse_scale = __fdiv_rn(-127.0f, val);
        const float rounded = __fmaf_rn(inverse_scale, v, 12582912.0f);
        q = (int)(__float_as_uint(rounded) & 0x007fffffu) - 0x00400000;
        q = q < 127 ? q : 127;
        d = __fdiv_rn(1.0f, inverse_scale);
    }
    qs[at] = (int8_t)q;
    if (i == 0) ds[(size_t)tok * blocks + block] = d;
}

__device__ __forceinline__ int e2m1_q1(uint32_t nibble) { // the code's value in halves (quant/nvfp4.rs:16-30)
    const int m = (int)((0xC8643210u >> (4 * (nibble & 7))) & 15u); // 0, 1, 2, 3, 4, 6, 8, 12
    return (nibble & 8) ? -m : m;
}
__device__ __forceinline__ int e4m3_q9(uint32_t code) { // a finite, non-negative scale code in units of 2^-9 (nvfp4.rs:33-51)
    const uint32_t ex = (code >> 3) & 15u, man = code & 7u;
    return ex == 0 ? (int)man : (int)((8u + man) << (ex - 1));
}

struct A16Args {
    const uint8_t *packed, *scales; // the repacked image: codes [n_out_pad][n_in/2], swizzled unsigned scales
    const int8_t *qs;
    const float *ds;
    void *y;
    float scale2;
    uint32_t n_out, n_in, kt, tokens, y_dtype;
};

// One warp per output row, eight tokens at a time.  Lane l takes bytes 4l .. 4l+3 of every 128-byte (256-value) block
// of the row, i.e. half of 16-group l / 2.
__global__ void __launch_bounds__(256) nvfp4_a16_kernel(const A16Args a) {
    const uint32_t row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= a.n_out) return;
    const uint32_t blocks = a.n_in / 256;
    const uint8_t *codes = a.packed + (size_t)row * (a.n_in / 2);
    for (uint32_t t0 = 0; t0 < a.tokens; t0 += 8) {
        float total[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) total[t] = 0.0f;
        for (uint32_t b = 0; b < blocks; ++b) {
            const uint32_t w = *reinterpret_cast<const uint32_t *>(codes + (size_t)b * 128 + 4 * lane);
            const uint32_t grp = b * 16 + lane / 2;
            const size_t soff = (size_t)(row / 128) * ((size_t)a.kt * 512) + (size_t)(grp / 4) * 512 + (row % 32) * 16 + ((row % 128) / 32) * 4 + grp % 4;
            const long long q9 = e4m3_q9(a.scales[soff]);
            int wq[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) wq[i] = e2m1_q1((w >> (4 * i)) & 15u); // low nibble = even element
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                if (t0 + t >= a.tokens) break; // warp-uniform
                const float d = a.ds[(size_t)(t0 + t) * blocks + b];
                const int2 q = *reinterpret_cast<const int2 *>(a.qs + (size_t)(t0 + t) * a.n_in + (size_t)b * 256 + 8 * lane);
                int dot = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) dot += wq[i] * (int)(int8_t)(((i < 4 ? q.x : q.y) >> (8 * (i & 3))) & 0xFF);
                dot += __shfl_xor_sync(0xffffffffu, dot, 1); // the two halves of a 16-group
                long long part = (lane & 1) ? 0ll : (long long)dot * q9;
#pragma unroll
                for (int o = 2; o < 32; o <<= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
                if (d != 0.0f) { // a block of zeros is skipped (nvfp4.rs:356-358)
                    float c = __fmaf_rn(__ll2float_rn(part), 1.0f / 1024.0f, 0.0f);
                    c = __fmaf_rn(c, d, 0.0f);
                    c = __fmaf_rn(c, a.scale2, 0.0f);
                    total[t] = __fmaf_rn(1.0f, c, total[t]);
                }
            }
        }
        if (lane == 0) {
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                if (t0 + t >= a.tokens) break;
                const __half h = __float2half_rn(total[t]); // the lane's output boundary (nvfp4.rs:378)
                const size_t o = (size_t)(t0 + t) * a.n_out + row;
                if (a.y_dtype == MUSER_DTYPE_F16) reinterpret_cast<__half *>(a.y)[o] = h;
                else if (a.y_dtype == MUSER_DTYPE_BF16) reinterpret_cast<__nv_bfloat16 *>(a.y)[o] = __float2bfloat16_rn(__half2float(h));
                else reinterpret_cast<float *>(a.y)[o] = __half2float(h);
            }
        }
    }
}

// x: [tokens][n_in] f32 or bf16; the int8 codes and block scales pass through `workspace`.
muser_cuda_status launch_nvfp4_a16(Ctx *ctx, const Weight *w, const void *x, uint32_t x_dtype, void *y, uint32_t y_dtype,
                                   uint32_t tokens, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
    if (w->n_in % 256) return fail(ctx, MUSER_CUDA_BAD_SHAPE, "the weight-only NVFP4 lane quantizes activations per 256: n_in % 256 != 0");
    if (w->shard.axis == MUSER_SHARD_K && w->shard.world > 1)
        return fail(ctx, MUSER_CUDA_BAD_SHAPE, "the weight-only NVFP4 lane rounds its result to f16: it cannot produce a K shard's partial sums");
    const size_t q_bytes = ((size_t)tokens * w->n_in + 15) / 16 * 16, d_bytes = (size_t)tokens * (w->n_in / 256) * sizeof(float);
    if (q_bytes + d_bytes > workspace_bytes)
        return fail(ctx, MUSER_CUDA_WORKSPACE_TOO_SMALL, "context workspace holds " + std::to_string(workspace_bytes) + " bytes, this call needs " + std::to_string(q_bytes + d_bytes));
    int8_t *qs = reinterpret_cast<int8_t *>(workspace);
    float *ds = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(workspace) + q_bytes);
    nvfp4_q8_quantize_kernel<<<dim3((unsigned)(w->n_in / 256), tokens), 256, 0, stream>>>(x, x_dtype == MUSER_DTYPE_F32, (uint32_t)w->n_in, qs, ds);
    MUSER_CUDA_TRY(ctx, cudaGetLastError());
    A16Args a;
    a.packed = w->packed, a.scales = w->scales, a.qs = qs, a.ds = ds, a.y = y;
    a.scale2 = w->scale2;
    a.n_out = (uint32_t)w->n_out, a.n_in = (uint32_t)w->n_in, a.kt = (uint32_t)((w->n_in + 63) / 64), a.tokens = tokens, a.y_dtype = y_dtype;
    nvfp4_a16_kernel<<<(unsigned)((w->n_out + 7) / 8), 256, 0, stream>>>(a);
    MUSER_CUDA_TRY(ctx, cudaGetLastError());
    return MUSER_CUDA_OK;
}

} // namespace muser
