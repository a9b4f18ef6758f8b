/*
 * CPU oracle for muser's quantized linear-layer path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference's CPU
 * reference lane (crates/muser-engine/src/quant/ and weights.rs).  It is the
 * checker that the CUDA path is compared against and the CPU baseline that the
 * benchmark times.  Nothing in the shipped library links, loads or calls it.
 *
 * Parity status: the NVFP4 functions are pinned against the known-answer
 * tests the reference holds (quant/nvfp4.rs:381-543) and against the
 * reference's own Python decoder (scripts/nvfp4_codec.py) and the numpy halves
 * of its GB10 fixtures.  The K-quant dot products have no CPU-only
 * known-answer test in the reference; for them parity is "unpinned by the
 * reference's tests": they are pinned here by construction (dequantisation is
 * integer/f16 layout work, checked against an independent numpy decoder) and
 * by an f64 cross-check of the documented summation order.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math (fmaf appears only where the
 * Rust source calls mul_add).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

/* dtype ids: crates/muser-engine/src/gguf/types.rs:9-39 */
enum {
    GGML_F32 = 0,
    GGML_F16 = 1,
    GGML_Q4_K = 12,
    GGML_Q5_K = 13,
    GGML_Q6_K = 14,
    GGML_BF16 = 30,
    GGML_NVFP4_E2M1 = 1000,
};

static inline float bits_f32(uint32_t b) {
    float f;
    memcpy(&f, &b, 4);
    return f;
}
static inline uint32_t f32_bits(float f) {
    uint32_t b;
    memcpy(&b, &f, 4);
    return b;
}

/* quant/helpers.rs:4-38 */
ORACLE_API float oracle_f16_to_f32(uint16_t h) {
    uint32_t sign = (h >> 15) & 1u;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t mant = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (mant == 0) {
            bits = sign << 31;
        } else {
            uint32_t e = 0, m = mant;
            while ((m & 0x400u) == 0) {
                m <<= 1;
                e += 1;
            }
            e = 127 - 14 - e;
            m = (m & 0x3ffu) << 13;
            bits = (sign << 31) | (e << 23) | m;
        }
    } else if (exp == 31) {
        bits = (sign << 31) | (0xffu << 23) | (mant << 13);
    } else {
        bits = (sign << 31) | ((exp + 127 - 15) << 23) | (mant << 13);
    }
    return bits_f32(bits);
}

/* quant/helpers.rs:43-68 -- the TRUNCATING converter used only by the
 * reference's test-data generators (metal/encode/multicol.rs:310-314). */
ORACLE_API uint16_t oracle_f32_to_f16_trunc(float x) {
    uint32_t b = f32_bits(x);
    uint16_t sign = (uint16_t)((b >> 16) & 0x8000u);
    int32_t exp = (int32_t)((b >> 23) & 0xffu);
    uint32_t mant = b & 0x7fffffu;
    if (exp == 0) return sign;
    if (exp >= 143) return sign | 0x7c00u;
    if (exp > 112) return sign | (uint16_t)((exp - 112) << 10) | (uint16_t)(mant >> 13);
    int32_t shift = 126 - exp;
    if (shift > 23) return sign;
    uint32_t full = (1u << 23) | mant;
    return sign | (uint16_t)(full >> shift);
}

/* IEEE round-to-nearest-even f32 -> f16, the behaviour of half::f16::from_f32
 * (crate `half` 2.x, pinned in crates/muser-engine/Cargo.toml:34), used at
 * quant/nvfp4.rs:77,181,337. */
ORACLE_API uint16_t oracle_f32_to_f16_rne(float x) {
    uint32_t b = f32_bits(x);
    uint16_t sign = (uint16_t)((b >> 16) & 0x8000u);
    uint32_t exp = (b >> 23) & 0xffu;
    uint32_t mant = b & 0x7fffffu;
    if (exp == 0xff) {
        if (mant == 0) return sign | 0x7c00u;
        return sign | 0x7c00u | 0x0200u | (uint16_t)(mant >> 13); /* quiet NaN */
    }
    int32_t e = (int32_t)exp - 127 + 15;
    if (e >= 31) return sign | 0x7c00u;
    if (e <= 0) {
        if (e < -10) return sign; /* below half of the smallest subnormal */
        uint32_t full = mant | 0x800000u;
        uint32_t shift = (uint32_t)(14 - e); /* 14..24 */
        uint32_t half_mant = full >> shift;
        uint32_t rem = full & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_mant & 1u))) half_mant += 1;
        return sign | (uint16_t)half_mant;
    }
    uint32_t half_bits = ((uint32_t)e << 10) | (mant >> 13);
    uint32_t rem = mant & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (half_bits & 1u))) half_bits += 1;
    return sign | (uint16_t)half_bits; /* a carry into the exponent is correct, inf included */
}

static inline float round_f16(float x) { return oracle_f16_to_f32(oracle_f32_to_f16_rne(x)); }

ORACLE_API float oracle_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* quant/helpers.rs:72 */
ORACLE_API float oracle_silu_fast(float x) { return x / (1.0f + expf(-x)); }

/* ---------------------------------------------------------------- K-quants */

static inline uint16_t le16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* 6-bit (sc, m) unpack shared by Q4_K and Q5_K: quant/k_block.rs:22-31 */
static inline void k4_scale_min(const uint8_t *scales, int j, uint8_t *sc, uint8_t *m) {
    if (j < 4) {
        *sc = scales[j] & 0x3f;
        *m = scales[j + 4] & 0x3f;
    } else {
        *sc = (uint8_t)((scales[j + 4] & 0x0f) | ((scales[j - 4] >> 6) << 4));
        *m = (uint8_t)((scales[j + 4] >> 4) | ((scales[j] >> 6) << 4));
    }
}

/* quant/k_block.rs:12-49 */
ORACLE_API void oracle_dequant_q4_k(const uint8_t *block, float *out) {
    float d = oracle_f16_to_f32(le16(block));
    float dmin = oracle_f16_to_f32(le16(block + 2));
    const uint8_t *scales = block + 4;
    const uint8_t *qs = block + 16;
    int is = 0;
    for (int base = 0, q_off = 0; base < 256; base += 64, q_off += 32, is += 2) {
        uint8_t sc, m;
        k4_scale_min(scales, is, &sc, &m);
        float d1 = d * (float)sc, m1 = dmin * (float)m;
        k4_scale_min(scales, is + 1, &sc, &m);
        float d2 = d * (float)sc, m2 = dmin * (float)m;
        for (int l = 0; l < 32; ++l) {
            uint8_t q = qs[q_off + l];
            out[base + l] = d1 * (float)(q & 0x0f) - m1;
            out[base + l + 32] = d2 * (float)(q >> 4) - m2;
        }
    }
}

/* quant/k_block.rs:61-105 */
ORACLE_API void oracle_dequant_q5_k(const uint8_t *block, float *out) {
    float d = oracle_f16_to_f32(le16(block));
    float dmin = oracle_f16_to_f32(le16(block + 2));
    const uint8_t *scales = block + 4;
    const uint8_t *qh = block + 16;
    const uint8_t *qs = block + 48;
    int is = 0;
    uint8_t u1 = 1, u2 = 2;
    for (int base = 0, q_off = 0; base < 256; base += 64, q_off += 32, is += 2) {
        uint8_t sc, m;
        k4_scale_min(scales, is, &sc, &m);
        float d1 = d * (float)sc, m1 = dmin * (float)m;
        k4_scale_min(scales, is + 1, &sc, &m);
        float d2 = d * (float)sc, m2 = dmin * (float)m;
        for (int l = 0; l < 32; ++l) {
            uint8_t q = qs[q_off + l];
            uint32_t lo = (q & 0x0f) + ((qh[l] & u1) ? 16u : 0u);
            uint32_t hi = (q >> 4) + ((qh[l] & u2) ? 16u : 0u);
            out[base + l] = d1 * (float)lo - m1;
            out[base + l + 32] = d2 * (float)hi - m2;
        }
        u1 = (uint8_t)(u1 << 2);
        u2 = (uint8_t)(u2 << 2);
    }
}

/* quant/k_block/q6.rs:283-325 */
ORACLE_API void oracle_dequant_q6_k(const uint8_t *block, float *out) {
    float d = oracle_f16_to_f32(le16(block + 208));
    const uint8_t *ql = block;
    const uint8_t *qh = block + 128;
    const int8_t *sc = (const int8_t *)(block + 192);
    for (int g = 0; g < 2; ++g) {
        for (int l = 0; l < 32; ++l) {
            int is = l / 16;
            uint32_t ql0 = ql[l], ql32 = ql[l + 32], qhl = qh[l];
            int q1 = (int)((ql0 & 0xf) | ((qhl & 3) << 4)) - 32;
            int q2 = (int)((ql32 & 0xf) | (((qhl >> 2) & 3) << 4)) - 32;
            int q3 = (int)((ql0 >> 4) | (((qhl >> 4) & 3) << 4)) - 32;
            int q4 = (int)((ql32 >> 4) | (((qhl >> 6) & 3) << 4)) - 32;
            float s1 = d * (float)sc[is];
            float s2 = d * (float)sc[is + 2];
            float s3 = d * (float)sc[is + 4];
            float s4 = d * (float)sc[is + 6];
            out[l] = s1 * (float)q1;
            out[l + 32] = s2 * (float)q2;
            out[l + 64] = s3 * (float)q3;
            out[l + 96] = s4 * (float)q4;
        }
        out += 128;
        ql += 64;
        qh += 32;
        sc += 8;
    }
}

/* quant/k_block.rs:242-286 (the x86 path of dot_q4_k_f32, k_block.rs:160-167):
 * one fused multiply-add per weight, sequential f32 accumulation. */
ORACLE_API float oracle_dot_q4_k_f32(const uint8_t *blocks, const float *x, size_t n) {
    size_t n_blocks = n / 256;
    float acc = 0.0f;
    for (size_t b = 0; b < n_blocks; ++b) {
        const uint8_t *block = blocks + b * 144;
        float d = oracle_f16_to_f32(le16(block));
        float dmin = oracle_f16_to_f32(le16(block + 2));
        const uint8_t *scales = block + 4;
        const uint8_t *qs = block + 16;
        const float *xb = x + b * 256;
        int is = 0;
        for (int base = 0, q_off = 0; base < 256; base += 64, q_off += 32, is += 2) {
            uint8_t sc, m;
            k4_scale_min(scales, is, &sc, &m);
            float d1 = d * (float)sc, m1 = dmin * (float)m;
            k4_scale_min(scales, is + 1, &sc, &m);
            float d2 = d * (float)sc, m2 = dmin * (float)m;
            for (int l = 0; l < 32; ++l) {
                uint8_t q = qs[q_off + l];
                acc += fmaf(d1, (float)(q & 0x0f), -m1) * xb[base + l];
                acc += fmaf(d2, (float)(q >> 4), -m2) * xb[base + l + 32];
            }
        }
    }
    return acc;
}

/* quant/k_block.rs:178-240: deferred-scaling order (per sub-block sum of q*x
 * and of x, scaled once). */
ORACLE_API float oracle_dot_q4_k_f32_llama(const uint8_t *blocks, const float *x, size_t n) {
    size_t n_blocks = n / 256;
    float sumf = 0.0f;
    for (size_t b = 0; b < n_blocks; ++b) {
        const uint8_t *block = blocks + b * 144;
        float d = oracle_f16_to_f32(le16(block));
        float dmin = oracle_f16_to_f32(le16(block + 2));
        const uint8_t *scales = block + 4;
        const uint8_t *qs = block + 16;
        const float *xb = x + b * 256;
        int is = 0;
        for (int base = 0, q_off = 0; base < 256; base += 64, q_off += 32, is += 2) {
            uint8_t sc_lo, m_lo, sc_hi, m_hi;
            k4_scale_min(scales, is, &sc_lo, &m_lo);
            k4_scale_min(scales, is + 1, &sc_hi, &m_hi);
            float acc_lo = 0.0f, acc_hi = 0.0f, xs_lo = 0.0f, xs_hi = 0.0f;
            for (int l = 0; l < 32; ++l) {
                uint8_t q = qs[q_off + l];
                float x_lo = xb[base + l], x_hi = xb[base + l + 32];
                acc_lo += (float)(q & 0x0f) * x_lo;
                acc_hi += (float)(q >> 4) * x_hi;
                xs_lo += x_lo;
                xs_hi += x_hi;
            }
            sumf += d * ((float)sc_lo * acc_lo + (float)sc_hi * acc_hi) -
                    dmin * ((float)m_lo * xs_lo + (float)m_hi * xs_hi);
        }
    }
    return sumf;
}

/* quant/k_block.rs:300-351 */
ORACLE_API float oracle_dot_q5_k_f32(const uint8_t *blocks, const float *x, size_t n) {
    size_t n_blocks = n / 256;
    float acc = 0.0f;
    for (size_t b = 0; b < n_blocks; ++b) {
        const uint8_t *block = blocks + b * 176;
        float d = oracle_f16_to_f32(le16(block));
        float dmin = oracle_f16_to_f32(le16(block + 2));
        const uint8_t *scales = block + 4;
        const uint8_t *qh = block + 16;
        const uint8_t *qs = block + 48;
        const float *xb = x + b * 256;
        int is = 0;
        uint8_t u1 = 1, u2 = 2;
        for (int base = 0, q_off = 0; base < 256; base += 64, q_off += 32, is += 2) {
            uint8_t sc, m;
            k4_scale_min(scales, is, &sc, &m);
            float d1 = d * (float)sc, m1 = dmin * (float)m;
            k4_scale_min(scales, is + 1, &sc, &m);
            float d2 = d * (float)sc, m2 = dmin * (float)m;
            for (int l = 0; l < 32; ++l) {
                uint8_t q = qs[q_off + l];
                uint32_t lo = (q & 0x0f) + ((qh[l] & u1) ? 16u : 0u);
                uint32_t hi = (q >> 4) + ((qh[l] & u2) ? 16u : 0u);
                acc += (d1 * (float)lo - m1) * xb[base + l];
                acc += (d2 * (float)hi - m2) * xb[base + l + 32];
            }
            u1 = (uint8_t)(u1 << 2);
            u2 = (uint8_t)(u2 << 2);
        }
    }
    return acc;
}

/* quant/k_block/q6.rs:90-141 (x86 path of dot_q6_k_f32, q6.rs:81-88) */
ORACLE_API float oracle_dot_q6_k_f32(const uint8_t *blocks, const float *x, size_t n) {
    size_t n_blocks = n / 256;
    float sumf = 0.0f;
    for (size_t b = 0; b < n_blocks; ++b) {
        const uint8_t *block = blocks + b * 210;
        float d = oracle_f16_to_f32(le16(block + 208));
        const uint8_t *ql = block;
        const uint8_t *qh = block + 128;
        const int8_t *sc = (const int8_t *)(block + 192);
        const float *xb = x + b * 256;
        for (int g = 0; g < 2; ++g) {
            for (int l_base = 0; l_base < 32; l_base += 16) {
                int is = l_base / 16;
                float sums[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                for (int l = l_base; l < l_base + 16; ++l) {
                    uint32_t ql0 = ql[l], ql32 = ql[l + 32], qhl = qh[l];
                    int q1 = (int)((ql0 & 0xf) | ((qhl & 3) << 4)) - 32;
                    int q2 = (int)((ql32 & 0xf) | (((qhl >> 2) & 3) << 4)) - 32;
                    int q3 = (int)((ql0 >> 4) | (((qhl >> 4) & 3) << 4)) - 32;
                    int q4 = (int)((ql32 >> 4) | (((qhl >> 6) & 3) << 4)) - 32;
                    sums[0] += (float)q1 * xb[l];
                    sums[1] += (float)q2 * xb[l + 32];
                    sums[2] += (float)q3 * xb[l + 64];
                    sums[3] += (float)q4 * xb[l + 96];
                }
                float s0 = (float)sc[is], s1 = (float)sc[is + 2];
                float s2 = (float)sc[is + 4], s3 = (float)sc[is + 6];
                sumf += d * (sums[0] * s0 + sums[1] * s1 + sums[2] * s2 + sums[3] * s3);
            }
            ql += 64;
            qh += 32;
            sc += 8;
            xb += 128;
        }
    }
    return sumf;
}

/* ------------------------------------------------------------------- NVFP4 */

static const float E2M1_LUT[16] = {0.0f,  0.5f,  1.0f,  1.5f,  2.0f,  3.0f,  4.0f,  6.0f,
                                   -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

/* quant/nvfp4.rs:16-30 */
ORACLE_API int32_t oracle_e2m1_q1(uint8_t nibble) {
    static const int32_t mag[8] = {0, 1, 2, 3, 4, 6, 8, 12};
    int32_t m = mag[nibble & 7];
    return (nibble & 8) ? -m : m;
}

/* quant/nvfp4.rs:33-51; returns INT32_MIN for the two NaN codes where the
 * reference asserts. */
ORACLE_API int32_t oracle_e4m3fn_q9(uint8_t byte) {
    uint32_t exponent = (byte >> 3) & 0x0f;
    uint32_t mantissa = byte & 7;
    if (exponent == 0x0f && mantissa == 7) return INT32_MIN;
    int32_t magnitude = exponent == 0 ? (int32_t)mantissa : (int32_t)((8 + mantissa) << (exponent - 1));
    return (byte & 0x80) ? -magnitude : magnitude;
}

/* quant/nvfp4.rs:101-103 */
ORACLE_API float oracle_e2m1_to_f32(uint8_t nibble) { return E2M1_LUT[nibble & 0x0f]; }

/* quant/nvfp4.rs:108-120 */
ORACLE_API float oracle_e4m3fn_to_f32(uint8_t byte) {
    float sign = (byte & 0x80) ? -1.0f : 1.0f;
    int exponent = (byte >> 3) & 0x0f;
    int mantissa = byte & 0x07;
    float magnitude;
    if (exponent == 0) {
        magnitude = (float)mantissa * (1.0f / 512.0f);
    } else if (exponent == 0x0f && mantissa == 0x07) {
        return NAN;
    } else {
        magnitude = (1.0f + (float)mantissa * 0.125f) * ldexpf(1.0f, exponent - 7);
    }
    return sign * magnitude;
}

/* quant/nvfp4.rs:127-144: exhaustive nearest search, ties to the even code,
 * saturating at 448. */
ORACLE_API uint8_t oracle_e4m3fn_from_f32(float value) {
    if (isnan(value)) return 0x7f;
    uint8_t sign = signbit(value) ? 0x80 : 0;
    float magnitude = fminf(fabsf(value), 448.0f);
    uint8_t best = 0;
    float best_distance = INFINITY;
    for (unsigned code = 0; code <= 0x7e; ++code) {
        float distance = fabsf(oracle_e4m3fn_to_f32((uint8_t)code) - magnitude);
        if (distance < best_distance ||
            (distance == best_distance && (code & 1) == 0 && (best & 1) != 0)) {
            best = (uint8_t)code;
            best_distance = distance;
        }
    }
    return sign | best;
}

static inline uint8_t e2m1_magnitude_code(float magnitude, float scale) {
    if (magnitude <= scale * 0.25f) return 0;
    if (magnitude < scale * 0.75f) return 1;
    if (magnitude <= scale * 1.25f) return 2;
    if (magnitude < scale * 1.75f) return 3;
    if (magnitude <= scale * 2.5f) return 4;
    if (magnitude < scale * 3.5f) return 5;
    if (magnitude <= scale * 5.0f) return 6;
    return 7;
}

/* quant/nvfp4.rs:149-170 */
ORACLE_API uint8_t oracle_e2m1_from_f32(float value) {
    uint8_t sign = signbit(value) ? 8 : 0;
    return sign | e2m1_magnitude_code(fabsf(value), 1.0f);
}

/* quant/nvfp4.rs:173-217 */
static uint8_t activation_group_codes(const float *input, float input_scale_inv, uint8_t codes[16]) {
    float rounded[16];
    float abs_max = 0.0f;
    for (int i = 0; i < 16; ++i) {
        rounded[i] = round_f16(input[i]);
        float a = fabsf(rounded[i]);
        if (a > abs_max) abs_max = a; /* f32::max: a NaN operand is ignored */
    }
    float normalized_max = abs_max * (1.0f / 6.0f);
    uint8_t scale_code = oracle_e4m3fn_from_f32(fminf(normalized_max * input_scale_inv, 448.0f));
    float scale = oracle_e4m3fn_to_f32(scale_code);
    if (scale == 0.0f) {
        for (int i = 0; i < 16; ++i) codes[i] = signbit(rounded[i]) ? 8 : 0;
    } else {
        for (int i = 0; i < 16; ++i) {
            uint8_t sign = signbit(rounded[i]) ? 8 : 0;
            float magnitude = fabsf(rounded[i]) * input_scale_inv;
            codes[i] = sign | e2m1_magnitude_code(magnitude, scale);
        }
    }
    return scale_code;
}

/* quant/nvfp4.rs:221-238; `n` values, packed n/2 bytes, scales n/16 bytes */
ORACLE_API void oracle_quantize_nvfp4_activation(const float *input, size_t n, float input_scale_inv,
                                                 uint8_t *packed, uint8_t *scales) {
    for (size_t group = 0; group < n / 16; ++group) {
        uint8_t codes[16];
        scales[group] = activation_group_codes(input + group * 16, input_scale_inv, codes);
        for (int pair = 0; pair < 8; ++pair)
            packed[group * 8 + pair] = (uint8_t)(codes[pair * 2] | (codes[pair * 2 + 1] << 4));
    }
}

/* quant/nvfp4.rs:240-255; order (e2m1 * e4m3) * scale2 */
ORACLE_API void oracle_dequant_nvfp4_row(const uint8_t *packed, const uint8_t *scales, float scale2,
                                         float *out, size_t n) {
    for (size_t group = 0; group < n / 16; ++group) {
        float scale = oracle_e4m3fn_to_f32(scales[group]);
        for (int pair = 0; pair < 8; ++pair) {
            uint8_t byte = packed[group * 8 + pair];
            out[group * 16 + pair * 2] = E2M1_LUT[byte & 0x0f] * scale * scale2;
            out[group * 16 + pair * 2 + 1] = E2M1_LUT[byte >> 4] * scale * scale2;
        }
    }
}

/* quant/nvfp4.rs:258-276 */
ORACLE_API float oracle_dot_nvfp4_f32(const uint8_t *packed, const uint8_t *scales, float scale2,
                                      const float *x, size_t n) {
    float sum = 0.0f;
    for (size_t group = 0; group < n / 16; ++group) {
        float scale = oracle_e4m3fn_to_f32(scales[group]);
        for (int pair = 0; pair < 8; ++pair) {
            uint8_t byte = packed[group * 8 + pair];
            float w0 = E2M1_LUT[byte & 0x0f] * scale * scale2;
            float w1 = E2M1_LUT[byte >> 4] * scale * scale2;
            sum += w0 * x[group * 16 + pair * 2];
            sum += w1 * x[group * 16 + pair * 2 + 1];
        }
    }
    return sum;
}

/* quant/nvfp4.rs:281-298 */
ORACLE_API float oracle_dot_nvfp4_block_fused_f32(const uint8_t *packed, const uint8_t *scales,
                                                  float scale2, const float *x, size_t n) {
    float sum = 0.0f;
    for (size_t group = 0; group < n / 16; ++group) {
        float block_sum = 0.0f;
        for (int pair = 0; pair < 8; ++pair) {
            uint8_t byte = packed[group * 8 + pair];
            block_sum += E2M1_LUT[byte & 0x0f] * x[group * 16 + pair * 2];
            block_sum += E2M1_LUT[byte >> 4] * x[group * 16 + pair * 2 + 1];
        }
        sum += block_sum * oracle_e4m3fn_to_f32(scales[group]);
    }
    return sum * scale2;
}

/* The integer contraction of quant/nvfp4.rs:304-338 on already quantised
 * activation codes.  The reference re-derives the activation codes inside
 * every row's dot (nvfp4.rs:319-320); they depend on x only, so hoisting the
 * quantisation out of the row loop is bit-identical. */
static int64_t w4a4_integer_sum(const uint8_t *w_packed, const uint8_t *w_scales, const uint8_t *a_packed,
                                const uint8_t *a_scales, size_t n) {
    int64_t sum = 0;
    for (size_t group = 0; group < n / 16; ++group) {
        int32_t block_sum = 0;
        for (int pair = 0; pair < 8; ++pair) {
            uint8_t wb = w_packed[group * 8 + pair], ab = a_packed[group * 8 + pair];
            block_sum += oracle_e2m1_q1(wb & 0x0f) * oracle_e2m1_q1(ab & 0x0f);
            block_sum += oracle_e2m1_q1(wb >> 4) * oracle_e2m1_q1(ab >> 4);
        }
        sum += (int64_t)block_sum * (int64_t)oracle_e4m3fn_q9(w_scales[group]) *
               (int64_t)oracle_e4m3fn_q9(a_scales[group]);
    }
    return sum;
}

/* Epilogue of quant/nvfp4.rs:331-337.  *pre_round receives the f32 value
 * before the final f16 rounding; the return value is what the reference
 * emits. */
static float w4a4_epilogue(int64_t sum, float weight_scale2, float input_scale_inv, float *pre_round) {
    float scaled = (float)sum * (1.0f / 1048576.0f);
    scaled = scaled * weight_scale2;
    scaled = scaled * (1.0f / input_scale_inv);
    if (pre_round) *pre_round = scaled;
    return round_f16(scaled);
}

/* quant/nvfp4.rs:304-338, faithful form (quantises x inside the call) */
ORACLE_API float oracle_dot_nvfp4_w4a4_f32(const uint8_t *packed, const uint8_t *scales, float weight_scale2,
                                           float input_scale_inv, const float *x, size_t n) {
    uint8_t *a_packed = (uint8_t *)malloc(n / 2 + n / 16);
    uint8_t *a_scales = a_packed + n / 2;
    oracle_quantize_nvfp4_activation(x, n, input_scale_inv, a_packed, a_scales);
    int64_t sum = w4a4_integer_sum(packed, scales, a_packed, a_scales, n);
    free(a_packed);
    return w4a4_epilogue(sum, weight_scale2, input_scale_inv, NULL);
}

/* quant/nvfp4.rs:62-66 */
static inline int32_t q8_nearest(float scale, float value) {
    float rounded = fmaf(scale, value, 12582912.0f);
    return ((int32_t)f32_bits(rounded) & 0x007fffff) - 0x00400000;
}

/* quant/nvfp4.rs:71-99; returns d */
ORACLE_API float oracle_quantize_nvfp4_q8_block(const float *input, int8_t *qs) {
    float rounded[256];
    float signed_max = 0.0f, abs_max = 0.0f;
    for (int i = 0; i < 256; ++i) {
        rounded[i] = round_f16(input[i]);
        float magnitude = fabsf(rounded[i]);
        if (magnitude > abs_max) {
            abs_max = magnitude;
            signed_max = rounded[i];
        }
    }
    if (abs_max == 0.0f) {
        memset(qs, 0, 256);
        return 0.0f;
    }
    float inverse_scale = -127.0f / signed_max;
    for (int i = 0; i < 256; ++i) {
        int32_t q = q8_nearest(inverse_scale, rounded[i]);
        qs[i] = (int8_t)(q < 127 ? q : 127);
    }
    return 1.0f / inverse_scale;
}

/* quant/nvfp4.rs:348-379 */
ORACLE_API float oracle_dot_nvfp4_a16_q8_f32(const uint8_t *packed, const uint8_t *scales, float weight_scale2,
                                             const float *x, size_t n) {
    float total = 0.0f;
    for (size_t block = 0; block < n / 256; ++block) {
        int8_t qs[256];
        float d = oracle_quantize_nvfp4_q8_block(x + block * 256, qs);
        if (d == 0.0f) continue;
        int64_t integer_total = 0;
        for (int gb = 0; gb < 16; ++gb) {
            size_t group = block * 16 + (size_t)gb;
            int32_t dot = 0;
            for (int pair = 0; pair < 8; ++pair) {
                uint8_t byte = packed[group * 8 + pair];
                dot += oracle_e2m1_q1(byte & 0x0f) * (int32_t)qs[gb * 16 + pair * 2];
                dot += oracle_e2m1_q1(byte >> 4) * (int32_t)qs[gb * 16 + pair * 2 + 1];
            }
            integer_total += (int64_t)dot * (int64_t)oracle_e4m3fn_q9(scales[group]);
        }
        float contribution = fmaf((float)integer_total, 1.0f / 1024.0f, 0.0f);
        contribution = fmaf(contribution, d, 0.0f);
        contribution = fmaf(contribution, weight_scale2, 0.0f);
        total = fmaf(1.0f, contribution, total);
    }
    return round_f16(total);
}

/* ------------------------------------------------- weights.rs: the operator */

typedef struct {
    const uint8_t *raw;          /* K-quant blocks, or packed E2M1 bytes [n_out][n_in/2] */
    uint32_t dtype;              /* GGML_* */
    size_t n_in, n_out;
    const uint8_t *block_scales; /* NVFP4: [n_out][n_in/16] E4M3FN bytes */
    float scale2;                /* NVFP4 per-tensor scale */
    int has_input_scale_inv;     /* NVFP4: W4A4 lane when set, a16_q8 lane otherwise */
    float input_scale_inv;
} oracle_tensor_view; /* weights.rs:29-48 */

/* weights.rs:63-67 */
ORACLE_API size_t oracle_row_bytes(uint32_t dtype, size_t n_in) {
    switch (dtype) {
        case GGML_Q4_K: return (n_in + 255) / 256 * 144;
        case GGML_Q5_K: return (n_in + 255) / 256 * 176;
        case GGML_Q6_K: return (n_in + 255) / 256 * 210;
        case GGML_F32: return n_in * 4;
        case GGML_F16:
        case GGML_BF16: return n_in * 2;
        case GGML_NVFP4_E2M1: return (n_in + 1) / 2;
        default: return 0;
    }
}

/* weights.rs:82-108 */
ORACLE_API int oracle_dequant_row(const oracle_tensor_view *t, size_t r, float *out) {
    if (t->dtype == GGML_NVFP4_E2M1) {
        oracle_dequant_nvfp4_row(t->raw + r * (t->n_in / 2), t->block_scales + r * (t->n_in / 16), t->scale2,
                                 out, t->n_in);
        return 0;
    }
    size_t rb = oracle_row_bytes(t->dtype, t->n_in);
    const uint8_t *row = t->raw + r * rb;
    size_t n_blocks = t->n_in / 256;
    for (size_t b = 0; b < n_blocks; ++b) {
        switch (t->dtype) {
            case GGML_Q4_K: oracle_dequant_q4_k(row + b * 144, out + b * 256); break;
            case GGML_Q5_K: oracle_dequant_q5_k(row + b * 176, out + b * 256); break;
            case GGML_Q6_K: oracle_dequant_q6_k(row + b * 210, out + b * 256); break;
            default: return -1;
        }
    }
    return 0;
}

typedef struct {
    const oracle_tensor_view *w;
    const float *x;
    size_t n_tokens;
    float *rt;        /* [n_out][n_tokens] scratch, weights.rs:405 */
    float *rt_f32;    /* optional: W4A4 value before the f16 rounding */
    const uint8_t *a_packed, *a_scales; /* hoisted W4A4 activation codes, or NULL */
    size_t r0, r1;
} matmul_job;

/* weights.rs:111-161 for the dtypes of this path */
static float dot_row(const matmul_job *j, size_t r, size_t t, float *pre_round) {
    const oracle_tensor_view *w = j->w;
    size_t n = w->n_in;
    const uint8_t *row = w->raw + r * oracle_row_bytes(w->dtype, n);
    const float *x = j->x + t * n;
    if (pre_round) *pre_round = NAN;
    switch (w->dtype) {
        case GGML_Q4_K: return oracle_dot_q4_k_f32(row, x, n);
        case GGML_Q5_K: return oracle_dot_q5_k_f32(row, x, n);
        case GGML_Q6_K: return oracle_dot_q6_k_f32(row, x, n);
        case GGML_NVFP4_E2M1: {
            const uint8_t *scales = w->block_scales + r * (n / 16);
            if (w->has_input_scale_inv) {
                if (j->a_packed) {
                    int64_t s = w4a4_integer_sum(row, scales, j->a_packed + t * (n / 2), j->a_scales + t * (n / 16), n);
                    return w4a4_epilogue(s, w->scale2, w->input_scale_inv, pre_round);
                }
                return oracle_dot_nvfp4_w4a4_f32(row, scales, w->scale2, w->input_scale_inv, x, n);
            }
            return oracle_dot_nvfp4_a16_q8_f32(row, scales, w->scale2, x, n);
        }
        default: return NAN;
    }
}

static void *matmul_worker(void *arg) {
    matmul_job *j = (matmul_job *)arg;
    for (size_t r = j->r0; r < j->r1; ++r)
        for (size_t t = 0; t < j->n_tokens; ++t) {
            float pre;
            j->rt[r * j->n_tokens + t] = dot_row(j, r, t, &pre);
            if (j->rt_f32) j->rt_f32[r * j->n_tokens + t] = pre;
        }
    return NULL;
}

/*
 * weights.rs:398-421: out[t][r] = dot(W_r, x_t); one task per output row over
 * all tokens (rayon par_chunks_mut there, `threads` pthreads over contiguous
 * row ranges here), a row-major [n_out][n_tokens] scratch, then the transpose
 * to token-major.
 *
 * hoist_activation != 0 quantises each W4A4 token once before the row loop
 * (same bits, feasible cost); 0 keeps the reference's per-row requantisation.
 * out_pre_round (optional, W4A4 only) receives the f32 values before the final
 * f16 rounding of nvfp4.rs:337.
 */
ORACLE_API int oracle_matmul(const oracle_tensor_view *w, const float *x, size_t n_tokens, float *out,
                             float *out_pre_round, int threads, int hoist_activation) {
    size_t n_in = w->n_in, n_out = w->n_out;
    if (oracle_row_bytes(w->dtype, n_in) == 0) return -1;
    if (w->dtype != GGML_NVFP4_E2M1 && n_in % 256) return -1;
    if (w->dtype == GGML_NVFP4_E2M1 && n_in % 16) return -1;
    if (threads < 1) threads = 1;
    if ((size_t)threads > n_out) threads = (int)(n_out ? n_out : 1);
    float *rt = (float *)malloc(sizeof(float) * n_out * n_tokens + 4);
    int w4a4 = w->dtype == GGML_NVFP4_E2M1 && w->has_input_scale_inv;
    float *rt_f32 = (out_pre_round && w4a4) ? (float *)malloc(sizeof(float) * n_out * n_tokens + 4) : NULL;
    uint8_t *a_packed = NULL, *a_scales = NULL;
    if (w4a4 && hoist_activation) {
        a_packed = (uint8_t *)malloc(n_tokens * (n_in / 2) + 1);
        a_scales = (uint8_t *)malloc(n_tokens * (n_in / 16) + 1);
        oracle_quantize_nvfp4_activation(x, n_tokens * n_in, w->input_scale_inv, a_packed, a_scales);
    }
    matmul_job *jobs = (matmul_job *)calloc((size_t)threads, sizeof(matmul_job));
    pthread_t *tids = (pthread_t *)calloc((size_t)threads, sizeof(pthread_t));
    for (int i = 0; i < threads; ++i) {
        jobs[i] = (matmul_job){w, x, n_tokens, rt, rt_f32, a_packed, a_scales,
                               n_out * (size_t)i / (size_t)threads, n_out * (size_t)(i + 1) / (size_t)threads};
        if (threads == 1)
            matmul_worker(&jobs[i]);
        else
            pthread_create(&tids[i], NULL, matmul_worker, &jobs[i]);
    }
    if (threads > 1)
        for (int i = 0; i < threads; ++i) pthread_join(tids[i], NULL);
    for (size_t r = 0; r < n_out; ++r)
        for (size_t t = 0; t < n_tokens; ++t) {
            out[t * n_out + r] = rt[r * n_tokens + t];
            if (rt_f32) out_pre_round[t * n_out + r] = rt_f32[r * n_tokens + t];
        }
    free(rt);
    free(rt_f32);
    free(a_packed);
    free(a_scales);
    free(jobs);
    free(tids);
    return 0;
}

/* reference.rs:59-80: x * 1/sqrt(mean(x^2)+eps), then the weight multiply */
ORACLE_API void oracle_rms_norm_mul(float *x, size_t rows, size_t dim, float eps, const float *w) {
    for (size_t r = 0; r < rows; ++r) {
        float *row = x + r * dim;
        float ss = 0.0f;
        for (size_t i = 0; i < dim; ++i) ss += row[i] * row[i];
        float scale = 1.0f / sqrtf(ss / (float)dim + eps);
        for (size_t i = 0; i < dim; ++i) row[i] *= scale;
        if (w)
            for (size_t i = 0; i < dim; ++i) row[i] *= w[i];
    }
}

/* reference.rs:559-570: logits *= logit_scale; then, if the cap is positive, cap * tanh(logit / cap) */
ORACLE_API void oracle_logit_tail(float *logits, size_t n, float logit_scale, float softcap) {
    for (size_t i = 0; i < n; ++i) logits[i] *= logit_scale;
    if (softcap > 0.0f) {
        float inv = 1.0f / softcap;
        for (size_t i = 0; i < n; ++i) logits[i] = softcap * tanhf(logits[i] * inv);
    }
}

/* weights.rs:425-449 matmul_rows: the same dot_row as matmul, over the listed rows only; out is [n_tokens][n_rows] */
ORACLE_API int oracle_matmul_rows(const oracle_tensor_view *w, const float *x, size_t n_tokens, const size_t *rows,
                                  size_t n_rows, float *out) {
    size_t rb = oracle_row_bytes(w->dtype, w->n_in);
    for (size_t i = 0; i < n_rows; ++i) {
        if (rows[i] >= w->n_out) return 1;
        oracle_tensor_view one = *w;
        one.raw = w->raw + rows[i] * rb;
        one.n_out = 1;
        if (w->block_scales) one.block_scales = w->block_scales + rows[i] * (w->n_in / 16);
        for (size_t t = 0; t < n_tokens; ++t) {
            float v;
            int rc = oracle_matmul(&one, x + t * w->n_in, 1, &v, NULL, 1, 1);
            if (rc) return rc;
            out[t * n_rows + i] = v;
        }
    }
    return 0;
}

/* reference.rs:511-513: silu_fast(gate) * up */
/* reference.rs:447-455: gate <- 1 / (1 + exp(-gate)); attn_out *= gate */
ORACLE_API void oracle_sigmoid_gate(float *x, const float *gate, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        float g = 1.0f / (1.0f + expf(-gate[i]));
        x[i] *= g;
    }
}

ORACLE_API void oracle_silu_mul(const float *gate, const float *up, float *out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = oracle_silu_fast(gate[i]) * up[i];
}
