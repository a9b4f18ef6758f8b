// Dequant-fused skinny GEMM for Q4_K and Q6_K weights: y[t][r] = dot(W_r, x_t), 1 <= tokens <= 64.
// (bf16 activations of up to 2 tokens, 8 for Q6_K, take the decode kernel in kquant_gemv.cu instead.)
//
// Stands in for MetalKernels::encode_quantized_matmul (crates/muser-engine/src/metal/encode/qkv.rs:414-641),
// encode_ffn_q4k_gate_up_silu_4r2s (src/metal/encode/ffn.rs:10-36) and, on the CPU lane, weights::matmul
// (src/weights.rs:398-421) with quant::dot_q4_k_f32 / dot_q6_k_f32.
//
// The kernel is HBM-bound: every weight byte is read exactly once with 16-byte, fully coalesced loads in the
// order the repacked tile stores them.  One warp owns a tile of 16 rows x 256 inputs at a time and walks along
// K.  The raw integer quants go straight from registers into bf16 m16n8k16 tensor-core fragments (0x4300 | q
// is the bf16 number 128 + q, so unpacking is one AND-OR per two weights); activations are the B operand.
// Products of an integer quant and a bf16 activation are exact, sums are f32.  The +128 (Q4_K) or +160 (Q6_K:
// 128 + the format's own 32) offset is cancelled by a second MMA whose A operand is the constant -128 / -160;
// for Q4_K that MMA also delivers -128 * sum(x), which is what the block's `- dmin * m` term multiplies.
// Scales are applied in f32 per sub-block, in the deferred order of quant/k_block.rs:178-240 and
// quant/k_block/q6.rs:90-141.
//
// With MT = 4 tokens a fragment column stands for a (token, sub-block slot) pair: while sub-block j is
// multiplied only the lanes that own column j % 2 feed activations, so one accumulator collects two sub-blocks
// and the scale epilogue runs half as often.  Each warp first passes its tile through shared memory to regroup
// the stored words (every lane owns whole sub-blocks, kquant_layout.cuh) so that every lane holds a quarter of
// every sub-block, the operand order of a sub-block-at-a-time MMA.
#include <algorithm>

#include "common.cuh"
#include "kquant_layout.cuh"

namespace muser {

struct KqArgs {
    const uint8_t *image;
    const uint8_t *image_up; // second weight of the fused gate/up call, else null
    const void *x;
    void *y;
    const float *row_scale;
    float out_scale, softcap; // LM-head tail
    const void *residual;
    uint32_t n_out, n_in, nsb, k_off, tokens, y_bf16, row_tiles;
};

__device__ __forceinline__ uint4 ldg_stream(const void *p) {
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1, const float (&c)[4]) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

// float(byte `idx` of w) + 2^23, as raw bits: the byte lands in the low mantissa bits of 0x4B000000.
__device__ __forceinline__ float byte_plus_2p23(uint32_t w, int idx) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u + idx));
}

// Eight (Q4_K) or four (Q6_K) consecutive activations of one token as bf16 pairs.  f32 activations are split
// into a bf16 head and a bf16 remainder (16 mantissa bits together) and multiplied in two passes.
template <bool XF32, int N>
struct XFrag {
    uint32_t hi[N / 2];
    uint32_t lo[XF32 ? N / 2 : 1];
};

__device__ __forceinline__ void split_bf16(float a, float b, uint32_t &hi, uint32_t &lo) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    float2 hf = __bfloat1622float2(h);
    __nv_bfloat162 l = __floats2bfloat162_rn(a - hf.x, b - hf.y);
    hi = *reinterpret_cast<uint32_t *>(&h);
    lo = *reinterpret_cast<uint32_t *>(&l);
}

template <bool XF32, int N>
__device__ __forceinline__ XFrag<XF32, N> load_x(const void *x_row, int64_t k, uint32_t n_in) {
    XFrag<XF32, N> f;
#pragma unroll
    for (int i = 0; i < N / 2; ++i) f.hi[i] = 0;
#pragma unroll
    for (int i = 0; i < (XF32 ? N / 2 : 1); ++i) f.lo[i] = 0;
    if (x_row == nullptr || (uint64_t)k >= n_in) return f; // a negative k wraps to a huge value
    if constexpr (XF32) {
        const float *p = reinterpret_cast<const float *>(x_row) + k;
#pragma unroll
        for (int i = 0; i < N / 4; ++i) {
            float4 v = __ldg(reinterpret_cast<const float4 *>(p) + i);
            split_bf16(v.x, v.y, f.hi[2 * i], f.lo[2 * i]);
            split_bf16(v.z, v.w, f.hi[2 * i + 1], f.lo[2 * i + 1]);
        }
    } else {
        const __nv_bfloat16 *p = reinterpret_cast<const __nv_bfloat16 *>(x_row) + k;
        if constexpr (N == 8) {
            uint4 v = __ldg(reinterpret_cast<const uint4 *>(p));
            f.hi[0] = v.x, f.hi[1] = v.y, f.hi[2] = v.z, f.hi[3] = v.w;
        } else {
            uint2 v = __ldg(reinterpret_cast<const uint2 *>(p));
            f.hi[0] = v.x, f.hi[1] = v.y;
        }
    }
    return f;
}

__device__ __forceinline__ uint32_t pick2(uint32_t a, uint32_t b, int i) { return i ? b : a; }
__device__ __forceinline__ uint32_t w4(const uint4 &v, int i) { return (&v.x)[i]; } // compile-time i only

constexpr uint32_t kNibMask = 0x000F000Fu, kBias128 = 0x43004300u; // 0x4300 | q == bf16(128 + q)
constexpr uint32_t kNeg128 = 0xC300C300u, kNeg160 = 0xC320C320u;   // bf16 pairs of -128 and -160
__device__ __forceinline__ uint32_t nib_pair(uint32_t w, int p) { return ((w >> (4 * p)) & kNibMask) | kBias128; }

// ---------------------------------------------------------------------------------------- tiles in registers
struct Q4Tile {
    uint4 q[4]; // [2*rowsel + hi]: row g + 8*rowsel, sub-block t + 4*hi
    uint4 ha, hb;
};
struct Q6Tile {
    uint4 lo[4]; // [2*rowsel + half]
    uint4 hi[2]; // [rowsel]
    uint4 sa, sb;
    float da, db;
};

__device__ __forceinline__ Q4Tile q4_load(const uint8_t *tile, int lane) {
    Q4Tile t;
    const uint4 *q = reinterpret_cast<const uint4 *>(tile);
#pragma unroll
    for (int i = 0; i < 4; ++i) t.q[i] = ldg_stream(q + 32 * i + lane);
    const uint4 *h = reinterpret_cast<const uint4 *>(tile + 2048);
    t.ha = ldg_stream(h + (lane >> 2));
    t.hb = ldg_stream(h + (lane >> 2) + 8);
    return t;
}
__device__ __forceinline__ Q6Tile q6_load(const uint8_t *tile, int lane) {
    Q6Tile t;
    const uint4 *q = reinterpret_cast<const uint4 *>(tile);
#pragma unroll
    for (int i = 0; i < 4; ++i) t.lo[i] = ldg_stream(q + 32 * i + lane);
    const uint4 *h = reinterpret_cast<const uint4 *>(tile + kQ6OffHi);
    t.hi[0] = ldg_stream(h + lane);
    t.hi[1] = ldg_stream(h + 32 + lane);
    const uint4 *s = reinterpret_cast<const uint4 *>(tile + kQ6OffSc);
    t.sa = ldg_stream(s + (lane >> 2));
    t.sb = ldg_stream(s + (lane >> 2) + 8);
    const __half *d = reinterpret_cast<const __half *>(tile + kQ6OffD);
    t.da = __half2float(__ldg(d + (lane >> 2)));
    t.db = __half2float(__ldg(d + (lane >> 2) + 8));
    return t;
}

struct Q4Scales {
    float d, c_d;   // d and -d * 2^23
    float dm, c_dm; // dmin / 128 and its -2^23 multiple
    uint32_t sc[2], mn[2];
    // d * sc_j and (dmin / 128) * m_j are exact in f32; fma(d, 2^23 + sc, -d * 2^23) returns them unrounded
    __device__ __forceinline__ float scale(int j) const { return fmaf(d, byte_plus_2p23(pick2(sc[0], sc[1], j >> 2), j & 3), c_d); }
    __device__ __forceinline__ float min128(int j) const { return fmaf(dm, byte_plus_2p23(pick2(mn[0], mn[1], j >> 2), j & 3), c_dm); }
};
__device__ __forceinline__ Q4Scales q4_scales(uint4 h) {
    Q4Scales s;
    __half2 dd = *reinterpret_cast<__half2 *>(&h.x);
    s.d = __low2float(dd);
    s.dm = __high2float(dd) * (1.0f / 128.0f);
    s.c_d = -s.d * 8388608.0f;
    s.c_dm = -s.dm * 8388608.0f;
    s.sc[0] = h.y & 0x3F3F3F3Fu;
    s.mn[0] = h.z & 0x3F3F3F3Fu;
    s.sc[1] = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
    s.mn[1] = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
    return s;
}
// int8 scale j of a row as f32: flip the sign bit, read the byte as 2^23 + (sc + 128), subtract both offsets
__device__ __forceinline__ float q6_scale(const uint4 &sc, int j) {
    const int w = j >> 2;
    const uint32_t word = pick2(pick2(sc.x, sc.y, w & 1), pick2(sc.z, sc.w, w & 1), w >> 1);
    return byte_plus_2p23(word ^ 0x80808080u, j & 3) - 8388736.0f;
}
// four 6-bit quants as bytes: low nibbles (even or odd nibble of each byte of `lo`) + 2 high bits of group x
__device__ __forceinline__ uint32_t q6_bytes(uint32_t lo, uint32_t hi, int x) {
    const uint32_t n = ((x & 1) ? lo >> 4 : lo) & 0x0F0F0F0Fu;
    const uint32_t h = x == 0 ? hi << 4 : x == 1 ? hi << 2 : x == 2 ? hi : hi >> 2;
    return n | (h & 0x30303030u);
}
// bytes (q0, q1, q2, q3) -> bf16 pair (128 + q0, 128 + q1) for pr = 0, (128 + q2, 128 + q3) for pr = 1
__device__ __forceinline__ uint32_t q6_pair(uint32_t q, int pr) { return __byte_perm(q, 0x43434343u, pr ? 0x4342 : 0x4140); }

// ---------------------------------------------------------------------------------------- tile compute
// Column c of a fragment stands for token c % MT and sub-block slot c / MT (MT = 4 or 8).
template <int MT> struct Cols {
    static constexpr int S = 8 / MT; // sub-blocks that share one accumulator
};

// `sm` is this warp's copy of the tile's quant planes in shared memory, in the stored (owned sub-block) order;
// word (row g + 8*rowsel, sub-block j, 8-element group wi) of a Q4_K tile sits at:
__device__ __forceinline__ uint32_t q4_nat_word(const uint32_t *sm, int rowsel, int j, int g, int wi) {
    return sm[((2 * rowsel + (j >> 2)) * 32 + g * 4 + (j & 3)) * 4 + wi];
}

template <int MT, int NT, bool XF32>
__device__ __forceinline__ void q4_nat_compute(const Q4Tile &tl, const uint32_t *sm, int64_t k_tile,
                                               const void *const (&x_rows)[NT], uint32_t n_in, int g, int t,
                                               float (&out)[NT][4]) {
    constexpr int S = Cols<MT>::S;
    const Q4Scales sa = q4_scales(tl.ha), sb = q4_scales(tl.hb);
    const int my_slot = g / MT;
#pragma unroll
    for (int a = 0; a < 8 / S; ++a) {
        XFrag<XF32, 8> xf[NT];
        float d[NT][4], dx[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            xf[nt] = load_x<XF32, 8>(x_rows[nt], k_tile + 32 * (S * a + my_slot) + 8 * t, n_in);
            d[nt][0] = d[nt][1] = d[nt][2] = d[nt][3] = 0.f;
            dx[nt][0] = dx[nt][1] = dx[nt][2] = dx[nt][3] = 0.f;
        }
#pragma unroll
        for (int s = 0; s < S; ++s) {
            const int j = S * a + s;
            const uint32_t wa = q4_nat_word(sm, 0, j, g, t), wb = q4_nat_word(sm, 1, j, g, t);
            const bool on = S == 1 || my_slot == s;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint32_t b0 = on ? xf[nt].hi[0] : 0u, b1 = on ? xf[nt].hi[1] : 0u;
                const uint32_t b2 = on ? xf[nt].hi[2] : 0u, b3 = on ? xf[nt].hi[3] : 0u;
                mma_bf16(dx[nt], kNeg128, kNeg128, kNeg128, kNeg128, b0, b1, dx[nt]);
                mma_bf16(dx[nt], kNeg128, kNeg128, kNeg128, kNeg128, b2, b3, dx[nt]);
                mma_bf16(d[nt], nib_pair(wa, 0), nib_pair(wb, 0), nib_pair(wa, 1), nib_pair(wb, 1), b0, b1, d[nt]);
                mma_bf16(d[nt], nib_pair(wa, 2), nib_pair(wb, 2), nib_pair(wa, 3), nib_pair(wb, 3), b2, b3, d[nt]);
                if constexpr (XF32) {
                    const uint32_t l0 = on ? xf[nt].lo[0] : 0u, l1 = on ? xf[nt].lo[1] : 0u;
                    const uint32_t l2 = on ? xf[nt].lo[2] : 0u, l3 = on ? xf[nt].lo[3] : 0u;
                    mma_bf16(dx[nt], kNeg128, kNeg128, kNeg128, kNeg128, l0, l1, dx[nt]);
                    mma_bf16(dx[nt], kNeg128, kNeg128, kNeg128, kNeg128, l2, l3, dx[nt]);
                    mma_bf16(d[nt], nib_pair(wa, 0), nib_pair(wb, 0), nib_pair(wa, 1), nib_pair(wb, 1), l0, l1, d[nt]);
                    mma_bf16(d[nt], nib_pair(wa, 2), nib_pair(wb, 2), nib_pair(wa, 3), nib_pair(wb, 3), l2, l3, d[nt]);
                }
            }
        }
        // d = sum (128 + q) x and dx = -128 sum x over the sub-block that this column stands for
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int j = S * a + (2 * t + e) / MT;
            const float s_a = sa.scale(j), m_a = sa.min128(j), s_b = sb.scale(j), m_b = sb.min128(j);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                out[nt][e] = fmaf(s_a, d[nt][e] + dx[nt][e], fmaf(m_a, dx[nt][e], out[nt][e]));
                out[nt][2 + e] = fmaf(s_b, d[nt][2 + e] + dx[nt][2 + e], fmaf(m_b, dx[nt][2 + e], out[nt][2 + e]));
            }
        }
    }
}

template <int MT, int NT, bool XF32>
__device__ __forceinline__ void q6_nat_compute(const Q6Tile &tl, const uint32_t *sm, int64_t k_tile,
                                               const void *const (&x_rows)[NT], uint32_t n_in, int g, int t,
                                               float (&out)[NT][4]) {
    constexpr int S = Cols<MT>::S;
    const int my_slot = g / MT;
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll
    for (int a = 0; a < 16 / S; ++a) {
        XFrag<XF32, 4> xf[NT];
        float d[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            xf[nt] = load_x<XF32, 4>(x_rows[nt], k_tile + 16 * (S * a + my_slot) + 4 * t, n_in);
            d[nt][0] = d[nt][1] = d[nt][2] = d[nt][3] = 0.f;
        }
#pragma unroll
        for (int s = 0; s < S; ++s) {
            const int j = S * a + s, o = j >> 2, owner = g * 4 + (j & 3);
            // this lane takes elements 4t .. 4t+3 of sub-block j: nibble parity t & 1 of word t / 2, high-bit group t
            const uint32_t la = sm[((o >> 1) * 32 + owner) * 4 + (o & 1) * 2 + (t >> 1)];
            const uint32_t lb = sm[((2 + (o >> 1)) * 32 + owner) * 4 + (o & 1) * 2 + (t >> 1)];
            const uint32_t ha = sm[kQ6OffHi / 4 + owner * 4 + o], hb = sm[kQ6OffHi / 4 + (32 + owner) * 4 + o];
            const uint32_t qa = (((t & 1) ? la >> 4 : la) & 0x0F0F0F0Fu) | (((ha >> (2 * t)) << 4) & 0x30303030u);
            const uint32_t qb = (((t & 1) ? lb >> 4 : lb) & 0x0F0F0F0Fu) | (((hb >> (2 * t)) << 4) & 0x30303030u);
            const bool on = S == 1 || my_slot == s;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint32_t b0 = on ? xf[nt].hi[0] : 0u, b1 = on ? xf[nt].hi[1] : 0u;
                mma_bf16(d[nt], kNeg160, kNeg160, kNeg160, kNeg160, b0, b1, d[nt]);
                mma_bf16(d[nt], q6_pair(qa, 0), q6_pair(qb, 0), q6_pair(qa, 1), q6_pair(qb, 1), b0, b1, d[nt]);
                if constexpr (XF32) {
                    const uint32_t l0 = on ? xf[nt].lo[0] : 0u, l1 = on ? xf[nt].lo[1] : 0u;
                    mma_bf16(d[nt], kNeg160, kNeg160, kNeg160, kNeg160, l0, l1, d[nt]);
                    mma_bf16(d[nt], q6_pair(qa, 0), q6_pair(qb, 0), q6_pair(qa, 1), q6_pair(qb, 1), l0, l1, d[nt]);
                }
            }
        }
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int j = S * a + (2 * t + e) / MT;
            const float f_a = q6_scale(tl.sa, j), f_b = q6_scale(tl.sb, j);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                acc[nt][e] = fmaf(f_a, d[nt][e], acc[nt][e]);
                acc[nt][2 + e] = fmaf(f_b, d[nt][2 + e], acc[nt][2 + e]);
            }
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        out[nt][0] = fmaf(tl.da, acc[nt][0], out[nt][0]);
        out[nt][1] = fmaf(tl.da, acc[nt][1], out[nt][1]);
        out[nt][2] = fmaf(tl.db, acc[nt][2], out[nt][2]);
        out[nt][3] = fmaf(tl.db, acc[nt][3], out[nt][3]);
    }
}

// ---------------------------------------------------------------------------------------- kernel
constexpr int kMaxWarps = 8;

template <int DT> struct TileOf;
template <> struct TileOf<MUSER_DTYPE_Q4_K> {
    using type = Q4Tile;
    static constexpr int bytes = kQ4TileBytes, plane_words = 2048 / 4;
};
template <> struct TileOf<MUSER_DTYPE_Q6_K> {
    using type = Q6Tile;
    static constexpr int bytes = kQ6TileBytes, plane_words = 3072 / 4;
};
template <int DT>
__device__ __forceinline__ typename TileOf<DT>::type load_tile(const uint8_t *p, int lane) {
    if constexpr (DT == MUSER_DTYPE_Q4_K) return q4_load(p, lane); else return q6_load(p, lane);
}
__device__ __forceinline__ void stage_tile(const Q4Tile &t, uint32_t *sm, int lane) {
#pragma unroll
    for (int i = 0; i < 4; ++i) reinterpret_cast<uint4 *>(sm)[32 * i + lane] = t.q[i];
}
__device__ __forceinline__ void stage_tile(const Q6Tile &t, uint32_t *sm, int lane) {
#pragma unroll
    for (int i = 0; i < 4; ++i) reinterpret_cast<uint4 *>(sm)[32 * i + lane] = t.lo[i];
    reinterpret_cast<uint4 *>(sm)[128 + lane] = t.hi[0];
    reinterpret_cast<uint4 *>(sm)[160 + lane] = t.hi[1];
}

// Grid: min(row tiles, resident CTAs); each CTA walks row tiles blockIdx.x, blockIdx.x + gridDim.x, ...  The
// CTA's warps split K evenly and add their partial sums through shared memory in a fixed order, so results
// do not depend on scheduling.
template <int DT, int MT, int NT, bool XF32, bool DUAL>
__global__ void __launch_bounds__(kMaxWarps * 32) kquant_matmul_kernel(const KqArgs a) {
    using Tile = typename TileOf<DT>::type;
    constexpr int kBytes = TileOf<DT>::bytes, kImages = DUAL ? 2 : 1;
    __shared__ float red[kImages][kMaxWarps][4][32];
    __shared__ __align__(16) uint32_t stage[kMaxWarps][TileOf<DT>::plane_words];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t sb0 = a.nsb * warp / warps, sb1 = a.nsb * (warp + 1) / warps;
    // which token's activations this lane's fragment column stands for
    const void *x_rows[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const uint32_t tok = nt * 8 + g % MT;
        x_rows[nt] = tok < a.tokens ? reinterpret_cast<const uint8_t *>(a.x) + (size_t)tok * a.n_in * (XF32 ? 4 : 2) : nullptr;
    }
    const uint8_t *images[kImages];
    images[0] = a.image;
    if constexpr (DUAL) images[1] = a.image_up;

    for (uint32_t rt = blockIdx.x; rt < a.row_tiles; rt += gridDim.x) {
        float out[kImages][NT][4];
#pragma unroll
        for (int im = 0; im < kImages; ++im) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) out[im][nt][0] = out[im][nt][1] = out[im][nt][2] = out[im][nt][3] = 0.f;
            if (sb0 < sb1) {
                const uint8_t *tp = images[im] + ((uint64_t)rt * a.nsb + sb0) * kBytes;
                Tile cur = load_tile<DT>(tp, lane), nxt;
                for (uint32_t sb = sb0; sb < sb1; ++sb) {
                    nxt = cur;
                    if (sb + 1 < sb1) nxt = load_tile<DT>(tp + kBytes, lane);
                    const int64_t k_tile = (int64_t)sb * 256 - (int64_t)a.k_off;
                    __syncwarp();
                    stage_tile(cur, stage[warp], lane);
                    __syncwarp();
                    if constexpr (DT == MUSER_DTYPE_Q4_K)
                        q4_nat_compute<MT, NT, XF32>(cur, stage[warp], k_tile, x_rows, a.n_in, g, t, out[im]);
                    else
                        q6_nat_compute<MT, NT, XF32>(cur, stage[warp], k_tile, x_rows, a.n_in, g, t, out[im]);
                    cur = nxt;
                    tp += kBytes;
                }
            }
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                red[0][warp][c][lane] = out[0][nt][c];
                if constexpr (DUAL) red[1][warp][c][lane] = out[1][nt][c];
            }
            __syncthreads();
            if (warp == 0) {
                float v[kImages][4];
#pragma unroll
                for (int im = 0; im < kImages; ++im) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        float s = red[im][0][c][lane];
                        for (int w = 1; w < warps; ++w) s += red[im][w][c][lane];
                        v[im][c] = s;
                    }
                    // lanes whose columns stand for the same token hold partial sums of the same output
                    if constexpr (MT <= 4) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) v[im][c] += __shfl_xor_sync(0xffffffffu, v[im][c], 2);
                    }
                }
                const bool writer = MT == 8 ? true : t < MT / 2;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    if (!writer) continue;
                    float r = v[0][c];
                    if constexpr (DUAL) r = __fdiv_rn(r, 1.0f + expf(-r)) * v[1][c]; // silu_fast(gate) * up, quant/helpers.rs:72
                    const uint32_t row = rt * 16 + g + 8 * (c >> 1);
                    const uint32_t tok = nt * 8 + (2 * t + (c & 1)) % MT;
                    if (row < a.n_out && tok < a.tokens) {
                        const size_t o = (size_t)tok * a.n_out + row;
                        if (a.row_scale) r *= a.row_scale[tok];
                        r = logit_tail(r, a.out_scale, a.softcap);
                        if (a.y_bf16) {
                            if (a.residual) r += __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(a.residual)[o]);
                            reinterpret_cast<__nv_bfloat16 *>(a.y)[o] = __float2bfloat16_rn(r);
                        } else {
                            if (a.residual) r += reinterpret_cast<const float *>(a.residual)[o];
                            reinterpret_cast<float *>(a.y)[o] = r;
                        }
                    }
                }
            }
            __syncthreads();
        }
    }
}

template <int DT, int MT, int NT, bool XF32, bool DUAL>
static cudaError_t launch_one(const KqArgs &a, int warps, int device, int sm_count, cudaStream_t stream) {
    struct Occ {
        int ctas_per_sm[kMaxWarps + 1] = {}; // occupancy of this instantiation per CTA width, queried once each
    };
    static PerDevice<Occ> occ;
    int per_sm;
    {
        std::lock_guard<std::mutex> lock(occ.mu);
        int &slot = occ.slot[device].ctas_per_sm[warps];
        if (slot == 0) {
            int n = 0;
            cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(
                &n, kquant_matmul_kernel<DT, MT, NT, XF32, DUAL>, warps * 32, 0);
            if (e != cudaSuccess) return e;
            slot = n > 0 ? n : 1;
        }
        per_sm = slot;
    }
    const uint32_t resident = (uint32_t)(per_sm * sm_count);
    dim3 grid(a.row_tiles < resident ? a.row_tiles : resident), block(warps * 32);
    kquant_matmul_kernel<DT, MT, NT, XF32, DUAL><<<grid, block, 0, stream>>>(a);
    return cudaGetLastError();
}

template <int DT, bool XF32, bool DUAL>
static cudaError_t launch_tokens(const KqArgs &a, int warps, int device, int sm_count, cudaStream_t stream) {
    const uint32_t m = a.tokens;
    if (m <= 4) return launch_one<DT, 4, 1, XF32, DUAL>(a, warps, device, sm_count, stream);
    if (m <= 8) return launch_one<DT, 8, 1, XF32, DUAL>(a, warps, device, sm_count, stream);
    if (m <= 16) return launch_one<DT, 8, 2, XF32, DUAL>(a, warps, device, sm_count, stream);
    if constexpr (!DUAL) {
        if (m <= 32) return launch_one<DT, 8, 4, XF32, false>(a, warps, device, sm_count, stream);
        return launch_one<DT, 8, 8, XF32, false>(a, warps, device, sm_count, stream);
    }
    return cudaErrorInvalidValue;
}

muser_cuda_status launch_kquant_matmul(Ctx *ctx, const Weight *w, const Weight *w_up, const void *x, uint32_t x_dtype,
                                       void *y, uint32_t y_dtype, uint32_t tokens, const Epilogue &ep,
                                       cudaStream_t stream) {
    // Measured crossovers on B200 (bf16 activations): the decode kernel (kquant_gemv.cu) up to 2 tokens for Q4_K and 4
    // for Q6_K; the tcgen05 kernel (kquant_tc.cu) from 12 / 5 tokens when the weight has enough 128-row blocks to
    // fill the GPU; this file's kernel in between, for f32 activations and for small weights.
    if (w->layout == 1) {
        // column-layout images are read by the decode kernel: up to 16 tokens a launch, more in chunks of 16
        if (w_up && w_up->layout != 1) return fail(ctx, MUSER_CUDA_BAD_ARG, "gate and up images differ in layout");
        const size_t xb = x_dtype == MUSER_DTYPE_F32 ? 4 : 2, yb = y_dtype == MUSER_DTYPE_BF16 ? 2 : 4;
        for (uint32_t t0 = 0; t0 < tokens; t0 += 16) {
            const uint32_t n = std::min(16u, tokens - t0);
            Epilogue e = ep;
            if (e.row_scale) e.row_scale += t0;
            if (e.residual) e.residual = reinterpret_cast<const uint8_t *>(e.residual) + (size_t)t0 * w->n_out * yb;
            void *yc = reinterpret_cast<uint8_t *>(y) + (size_t)t0 * w->n_out * yb;
            const cudaError_t de = launch_kquant_decode(ctx, &w, w_up, 1, reinterpret_cast<const uint8_t *>(x) + (size_t)t0 * w->n_in * xb,
                                                        x_dtype, &yc, &y_dtype, n, &e, stream);
            if (de == cudaErrorNotSupported) return fail(ctx, MUSER_CUDA_BAD_SHAPE, "this shape does not fit the decode kernel");
            MUSER_CUDA_TRY(ctx, de);
        }
        return MUSER_CUDA_OK;
    }
    const bool q6 = w->dtype == MUSER_DTYPE_Q6_K;
    // (f32 activations cost the legacy kernel a second MMA pass, so the tensor-core kernel takes over earlier;
    //  it carries them as f16 head + remainder column pairs, hence at most 32 tokens)
    const bool xf32_in = x_dtype == MUSER_DTYPE_F32;
    const uint32_t tc_set = ctx->tc_min_tokens[q6 ? 1 : 0]; // above 64: switched off
    uint32_t tc_from = (xf32_in && tc_set <= 64) ? std::min(tc_set, 5u) : tc_set;
    // (a Q4_K weight with fewer than 8 row tiles per SM gives the tcgen05 kernel too few 128-row blocks: on attn_q,
    //  5120 rows, the general kernel takes 17.7 us up to 16 tokens of bf16 against 21.8; a threshold set below the
    //  default is a caller's explicit choice and stands)
    if (!q6 && !xf32_in && tc_from >= 12 && tc_from <= 16 && w->row_tiles < 8u * (uint32_t)ctx->sm_count) tc_from = 17;
    const bool tc_fits = !w_up && tokens >= tc_from && tokens <= (xf32_in ? 32u : 64u) && w->n_out >= ctx->tc_min_rows;
    // (a weight of few row tiles cannot fill the GEMV's rings: attn_k / attn_v of 1024 rows take 7.3 / 9.9 us in the
    //  general kernel at 2 / 4 tokens of bf16, 9.3 / 14.9 us in the GEMV)
    uint32_t gemv_max = ctx->gemv_max_tokens[q6 ? 1 : 0];
    if (!xf32_in && w->row_tiles < (uint32_t)ctx->sm_count) gemv_max = std::min(gemv_max, q6 ? 2u : 1u);
    if (!tc_fits && tokens <= gemv_max) { // bf16 or f32 activations: either becomes 15-bit fixed point per sub-block
        const cudaError_t ge = launch_kquant_gemv(ctx, w, w_up, x, x_dtype, y, y_dtype, tokens, ep, stream);
        if (ge != cudaErrorNotSupported) {
            MUSER_CUDA_TRY(ctx, ge);
            return MUSER_CUDA_OK;
        }
    }
    if (ep.norm_weight) {
        // the kernels below read their activations as they go, so the fused input norm runs as a pass of its own
        // into the context's scratch rows (f32), which the projection then reads instead of x
        const size_t need = (size_t)tokens * w->n_in * sizeof(float);
        if (need > ctx->norm_scratch_bytes) return fail(ctx, MUSER_CUDA_WORKSPACE_TOO_SMALL, "fused input norm: tokens x n_in exceeds the context's norm scratch");
        muser_cuda_status st = launch_rmsnorm_rows(ctx, x, x_dtype, tokens, w->n_in, ep.norm_weight, ep.norm_eps, ctx->norm_scratch, stream);
        if (st != MUSER_CUDA_OK) return st;
        x = ctx->norm_scratch;
        x_dtype = MUSER_DTYPE_F32;
    }
    if (tc_fits) {
        Epilogue tail = ep;
        tail.norm_weight = nullptr;
        const cudaError_t te = launch_kquant_tc(ctx, w, x, x_dtype, y, y_dtype, tokens, tail, stream);
        if (te != cudaErrorNotSupported) {
            MUSER_CUDA_TRY(ctx, te);
            return MUSER_CUDA_OK;
        }
    }
    KqArgs a;
    a.image = w->image;
    a.image_up = w_up ? w_up->image : nullptr;
    a.x = x;
    a.y = y;
    a.row_scale = ep.row_scale;
    a.out_scale = ep.out_scale;
    a.softcap = ep.softcap;
    a.residual = ep.residual;
    a.n_out = (uint32_t)w->n_out;
    a.n_in = (uint32_t)w->n_in;
    a.nsb = w->nsb;
    a.k_off = w->k_off;
    a.tokens = tokens;
    a.y_bf16 = y_dtype == MUSER_DTYPE_BF16;
    a.row_tiles = w->row_tiles;
    const bool xf32 = x_dtype == MUSER_DTYPE_F32, dual = w_up != nullptr;
    // Warps that split K inside a CTA.  A warp pays about two tiles' worth of start-up (its first load, its share of
    // the CTA's reduction) per row tile, so with row tiles to spare the cheapest split is the one with the smallest
    // warps x (longest K run + 2): 4 warps x 5 tiles for K = 5120 took 35 us where 8 warps x 3 took 42 (ffn_gate,
    // 4 tokens).  A weight with few row tiles needs all 8 warps to keep the SMs' load queues full.
    int warps = w->nsb >= 8 ? 8 : (w->nsb >= 4 ? 4 : (w->nsb >= 2 ? 2 : 1));
    if (w->nsb >= 8 && w->row_tiles >= 2u * (uint32_t)ctx->sm_count) {
        uint32_t best = ~0u;
        for (int c = 4; c <= kMaxWarps; ++c) {
            const uint32_t cost = (uint32_t)c * ((w->nsb + c - 1) / c + 2);
            if (cost < best) best = cost, warps = c;
        }
    }
    if (ctx->matmul_warps) warps = (int)std::min(ctx->matmul_warps, w->nsb);
    const int sms = ctx->sm_count;
    cudaError_t e;
    if (w->dtype == MUSER_DTYPE_Q4_K) {
        if (dual) e = xf32 ? launch_tokens<MUSER_DTYPE_Q4_K, true, true>(a, warps, ctx->device, sms, stream)
                           : launch_tokens<MUSER_DTYPE_Q4_K, false, true>(a, warps, ctx->device, sms, stream);
        else e = xf32 ? launch_tokens<MUSER_DTYPE_Q4_K, true, false>(a, warps, ctx->device, sms, stream)
                      : launch_tokens<MUSER_DTYPE_Q4_K, false, false>(a, warps, ctx->device, sms, stream);
    } else {
        if (dual) e = xf32 ? launch_tokens<MUSER_DTYPE_Q6_K, true, true>(a, warps, ctx->device, sms, stream)
                           : launch_tokens<MUSER_DTYPE_Q6_K, false, true>(a, warps, ctx->device, sms, stream);
        else e = xf32 ? launch_tokens<MUSER_DTYPE_Q6_K, true, false>(a, warps, ctx->device, sms, stream)
                      : launch_tokens<MUSER_DTYPE_Q6_K, false, false>(a, warps, ctx->device, sms, stream);
    }
    MUSER_CUDA_TRY(ctx, e);
    return MUSER_CUDA_OK;
}

} // namespace muser
