// Input RMSNorm pieces shared by the kernels that fuse it: rms_norm / rms_norm_mul of
// crates/muser-engine/src/reference.rs:59-80, y = (x * 1/sqrt(sum(x^2)/n + eps)) * w, all in f32.
// The reference adds the squares front to back; here a block adds them as a tree, so the factor can differ from
// the CPU lane's in its last bits (outputs are compared by relative L2, not bit for bit).
#pragma once
#include "common.cuh"

namespace muser {

// Eight consecutive activations of one row as f32 (the row starts 16-byte aligned and i8 counts groups of eight).
template <bool XF32>
__device__ __forceinline__ void load8(const void *row, uint32_t i8, float (&v)[8]) {
    if constexpr (XF32) {
        const float4 *p = reinterpret_cast<const float4 *>(row) + 2 * (size_t)i8;
        const float4 a = __ldg(p), b = __ldg(p + 1);
        v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
    } else {
        const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(row) + i8);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
}

// 1/sqrt(mean(x^2) + eps) of one row of n values (n % 8 == 0), computed by the whole block; `red` holds 33 floats
// of shared memory.  Every thread of the block must call it, and all get the result.
template <bool XF32>
__device__ __forceinline__ float block_inv_rms(const void *row, uint32_t n, float eps, float *red) {
    float ss = 0.0f;
    for (uint32_t i = threadIdx.x; i < n / 8; i += blockDim.x) {
        float v[8];
        load8<XF32>(row, i, v);
#pragma unroll
        for (int k = 0; k < 8; ++k) ss = fmaf(v[k], v[k], ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = (blockDim.x + 31) >> 5;
    __syncthreads(); // `red` may still be read from an earlier call
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (warp == 0) {
        float t = lane < warps ? red[lane] : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) red[32] = __fdiv_rn(1.0f, __fsqrt_rn(__fdiv_rn(t, (float)n) + eps));
    }
    __syncthreads();
    return red[32];
}

} // namespace muser
