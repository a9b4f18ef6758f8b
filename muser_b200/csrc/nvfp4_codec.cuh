// The NVFP4 activation codec shared by the quantizer kernels and by the GEMM epilogue that emits quantized outputs:
// quant::activation_group_codes (crates/muser-engine/src/quant/nvfp4.rs:173-217), bit for bit.
#pragma once
#include <cuda_fp8.h>

#include "common.cuh"

namespace muser {

__device__ __forceinline__ float e4m3_to_f32(uint32_t code) { // finite, non-negative codes only
    const uint32_t ex = (code >> 3) & 15u, man = code & 7u;
    if (ex == 0) return (float)man * (1.0f / 512.0f);
    return __fmul_rn(1.0f + (float)man * 0.125f, __uint_as_float((ex + 120u) << 23));
}

__device__ __forceinline__ uint32_t e2m1_code(float r, float isi, float scale) {
    const uint32_t sign = (__float_as_uint(r) >> 31) << 3;
    if (scale == 0.0f) return sign;
    const float m = __fmul_rn(fabsf(r), isi);
    uint32_t code = 0;
    code += m > __fmul_rn(scale, 0.25f);
    code += m >= __fmul_rn(scale, 0.75f);
    code += m > __fmul_rn(scale, 1.25f);
    code += m >= __fmul_rn(scale, 1.75f);
    code += m > __fmul_rn(scale, 2.5f);
    code += m >= __fmul_rn(scale, 3.5f);
    code += m > __fmul_rn(scale, 5.0f);
    return sign | code;
}

// Quantizes one group of 16 values: writes its 8 code bytes and returns its E4M3 scale code.
__device__ __forceinline__ uint32_t quantize_group(float (&r)[16], float isi, uint8_t *codes) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        r[i] = __half2float(__float2half_rn(r[i]));
        amax = fmaxf(amax, fabsf(r[i]));
    }
    const float target = fminf(__fmul_rn(__fmul_rn(amax, 1.0f / 6.0f), isi), 448.0f);
    const uint32_t scale_code = __nv_cvt_float_to_fp8(target, __NV_SATFINITE, __NV_E4M3) & 0x7Fu;
    const float scale = e4m3_to_f32(scale_code);
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        lo |= e2m1_code(r[i], isi, scale) << (4 * i);
        hi |= e2m1_code(r[8 + i], isi, scale) << (4 * i);
    }
    *reinterpret_cast<uint2 *>(codes) = make_uint2(lo, hi);
    return scale_code;
}

// Where the scale byte of (row, 16-value group grp) lives in the swizzled plane of a tensor with kt 64-value chunks
// per row (scripts/gx10/vllm/muser_vllm/exact_fp4_quant.py:149-162); the four groups of a chunk are consecutive bytes.
__device__ __forceinline__ size_t swizzled_scale_offset(uint32_t row, uint32_t grp, uint32_t kt) {
    return (size_t)(row / 128) * ((size_t)kt * 512) + (size_t)(grp / 4) * 512 + (row % 32) * 16 + ((row % 128) / 32) * 4 + grp % 4;
}

} // namespace muser
