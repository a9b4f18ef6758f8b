// Dequant-fused GEMV / skinny GEMM for Q4_K and Q6_K weights: y[t][r] = dot(W_r, x_t), 1 <= tokens <= 64.
//
// Stands in for MetalKernels::encode_quantized_matmul (crates/muser-engine/src/metal/encode/qkv.rs:414-641),
// encode_ffn_q4k_gate_up_silu_4r2s (src/metal/encode/ffn.rs:10-36) and, on the CPU lane, weights::matmul
// (src/weights.rs:398-421) with quant::dot_q4_k_f32 / dot_q6_k_f32.
//
// The kernel is HBM-bound: every weight byte is read exactly once with 16-byte, fully coalesced loads in the
// order the repacked tile stores them.  One warp owns a tile of 16 rows and walks along K.  The raw integer
// quants go straight from registers into bf16 m16n8k16 tensor-core fragments (0x4300 | q is the bf16 number
// 128 + q, so unpacking is one AND-OR per two weights); activations are the B operand, eight tokens per
// fragment.  Products of an integer quant and a bf16 activation are exact, sums are f32.  The +128 (Q4_K) or
// +160 (Q6_K: 128 + the format's own 32) offset is cancelled by chaining the accumulator through a second MMA
// whose A operand is the constant -128 / -160; for Q4_K that same MMA delivers -128 * sum(x), which is what
// the block's `- dmin * m` term multiplies.  Scales are applied in f32 per sub-block, in the deferred order of
// quant/k_block.rs:178-240 and quant/k_block/q6.rs:90-141.
#include "common.cuh"
#include "kquant_layout.cuh"

namespace muser {

struct KqArgs {
    const uint8_t *image;
    const uint8_t *image_up; // second weight of the fused gate/up call, else null
    const void *x;
    void *y;
    const float *row_scale;
    const void *residual;
    uint32_t n_out, n_in, nsb, k_off, tokens, y_bf16;
};

__device__ __forceinline__ uint4 ldg_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1, const float (&c)[4]) {
    asm volatile(
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

// ---------------------------------------------------------------------------------------- Q4_K
struct Q4Tile {
    uint4 qa[2], qb[2]; // nibble words of row g / row g+8, sub-blocks 0..3 and 4..7
    uint4 ha, hb;       // their headers
};

__device__ __forceinline__ Q4Tile q4_load(const uint8_t *tile, int lane) {
    Q4Tile t;
    const uint4 *q = reinterpret_cast<const uint4 *>(tile);
    t.qa[0] = ldg_stream(q + lane);
    t.qa[1] = ldg_stream(q + 32 + lane);
    t.qb[0] = ldg_stream(q + 64 + lane);
    t.qb[1] = ldg_stream(q + 96 + lane);
    const uint4 *h = reinterpret_cast<const uint4 *>(tile + 2048);
    t.ha = ldg_stream(h + (lane >> 2));
    t.hb = ldg_stream(h + (lane >> 2) + 8);
    return t;
}

struct Q4Scales {
    float d, c_d;   // d and -d * 2^23
    float dm, c_dm; // dmin / 128 and its -2^23 multiple
    uint32_t sc[2], mn[2];
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

template <int NT, bool XF32>
__device__ __forceinline__ void q4_tile_compute(const Q4Tile &tl, int64_t k_tile, const void *const (&x_rows)[NT],
                                                uint32_t n_in, int t, float (&out)[NT][4]) {
    const Q4Scales sa = q4_scales(tl.ha), sb = q4_scales(tl.hb);
    constexpr uint32_t kMask = 0x000F000Fu, kBias = 0x43004300u, kNeg = 0xC300C300u; // 128.0 and -128.0 in bf16
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t wa = (&tl.qa[j >> 2].x)[j & 3], wb = (&tl.qb[j >> 2].x)[j & 3];
        // d * sc and (dmin / 128) * m are exact in f32; fma(d, 2^23 + sc, -d * 2^23) returns them unrounded
        const float s_a = fmaf(sa.d, byte_plus_2p23(sa.sc[j >> 2], j & 3), sa.c_d);
        const float m_a = fmaf(sa.dm, byte_plus_2p23(sa.mn[j >> 2], j & 3), sa.c_dm);
        const float s_b = fmaf(sb.d, byte_plus_2p23(sb.sc[j >> 2], j & 3), sb.c_d);
        const float m_b = fmaf(sb.dm, byte_plus_2p23(sb.mn[j >> 2], j & 3), sb.c_dm);
        const uint32_t a0 = (wa & kMask) | kBias, a1 = (wb & kMask) | kBias;
        const uint32_t a2 = ((wa >> 4) & kMask) | kBias, a3 = ((wb >> 4) & kMask) | kBias;
        const uint32_t e0 = ((wa >> 8) & kMask) | kBias, e1 = ((wb >> 8) & kMask) | kBias;
        const uint32_t e2 = ((wa >> 12) & kMask) | kBias, e3 = ((wb >> 12) & kMask) | kBias;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const XFrag<XF32, 8> xf = load_x<XF32, 8>(x_rows[nt], k_tile + 32 * j + 8 * t, n_in);
            float dx[4] = {0.f, 0.f, 0.f, 0.f}, d[4];
            mma_bf16(dx, kNeg, kNeg, kNeg, kNeg, xf.hi[0], xf.hi[1], dx);
            mma_bf16(dx, kNeg, kNeg, kNeg, kNeg, xf.hi[2], xf.hi[3], dx);
            if constexpr (XF32) {
                mma_bf16(dx, kNeg, kNeg, kNeg, kNeg, xf.lo[0], xf.lo[1], dx);
                mma_bf16(dx, kNeg, kNeg, kNeg, kNeg, xf.lo[2], xf.lo[3], dx);
            }
            mma_bf16(d, a0, a1, a2, a3, xf.hi[0], xf.hi[1], dx);
            mma_bf16(d, e0, e1, e2, e3, xf.hi[2], xf.hi[3], d);
            if constexpr (XF32) {
                mma_bf16(d, a0, a1, a2, a3, xf.lo[0], xf.lo[1], d);
                mma_bf16(d, e0, e1, e2, e3, xf.lo[2], xf.lo[3], d);
            }
            // d = sum q x over the sub-block, dx = -128 sum x
            out[nt][0] = fmaf(s_a, d[0], fmaf(m_a, dx[0], out[nt][0]));
            out[nt][1] = fmaf(s_a, d[1], fmaf(m_a, dx[1], out[nt][1]));
            out[nt][2] = fmaf(s_b, d[2], fmaf(m_b, dx[2], out[nt][2]));
            out[nt][3] = fmaf(s_b, d[3], fmaf(m_b, dx[3], out[nt][3]));
        }
    }
}

// ---------------------------------------------------------------------------------------- Q6_K
struct Q6Tile {
    uint4 la[2], lb[2]; // low nibbles of row g / g+8, sub-blocks 0..7 and 8..15
    uint4 ha, hb;       // high bits
    uint4 sa, sb;       // int8 scales
    float da, db;
};

__device__ __forceinline__ Q6Tile q6_load(const uint8_t *tile, int lane) {
    Q6Tile t;
    const uint4 *q = reinterpret_cast<const uint4 *>(tile);
    t.la[0] = ldg_stream(q + lane);
    t.la[1] = ldg_stream(q + 32 + lane);
    t.lb[0] = ldg_stream(q + 64 + lane);
    t.lb[1] = ldg_stream(q + 96 + lane);
    const uint4 *h = reinterpret_cast<const uint4 *>(tile + kQ6OffHi);
    t.ha = ldg_stream(h + lane);
    t.hb = ldg_stream(h + 32 + lane);
    const uint4 *s = reinterpret_cast<const uint4 *>(tile + kQ6OffSc);
    t.sa = ldg_stream(s + (lane >> 2));
    t.sb = ldg_stream(s + (lane >> 2) + 8);
    const __half *d = reinterpret_cast<const __half *>(tile + kQ6OffD);
    t.da = __half2float(__ldg(d + (lane >> 2)));
    t.db = __half2float(__ldg(d + (lane >> 2) + 8));
    return t;
}

template <int NT, bool XF32>
__device__ __forceinline__ void q6_tile_compute(const Q6Tile &tl, int64_t k_tile, const void *const (&x_rows)[NT],
                                                uint32_t n_in, int t, float (&out)[NT][4]) {
    constexpr uint32_t kNeg = 0xC320C320u; // -160.0 in bf16: cancels 128 (fragment bias) + 32 (format offset)
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll
    for (int s = 0; s < 16; ++s) {
        const uint32_t la = (&tl.la[s >> 3].x)[(s & 7) >> 1], lb = (&tl.lb[s >> 3].x)[(s & 7) >> 1];
        const uint32_t ha = (&tl.ha.x)[s >> 2], hb = (&tl.hb.x)[s >> 2];
        const int u = s & 3;
        const uint32_t ha_s = u == 0 ? ha << 4 : u == 1 ? ha << 2 : u == 2 ? ha : ha >> 2;
        const uint32_t hb_s = u == 0 ? hb << 4 : u == 1 ? hb << 2 : u == 2 ? hb : hb >> 2;
        const uint32_t qa = (((s & 1) ? la >> 4 : la) & 0x0F0F0F0Fu) | (ha_s & 0x30303030u);
        const uint32_t qb = (((s & 1) ? lb >> 4 : lb) & 0x0F0F0F0Fu) | (hb_s & 0x30303030u);
        // bytes (q0, q1, q2, q3) -> bf16 pairs (128 + q0, 128 + q1) and (128 + q2, 128 + q3)
        const uint32_t a0 = __byte_perm(qa, 0x43434343u, 0x4140), a2 = __byte_perm(qa, 0x43434343u, 0x4342);
        const uint32_t a1 = __byte_perm(qb, 0x43434343u, 0x4140), a3 = __byte_perm(qb, 0x43434343u, 0x4342);
        // int8 scale -> f32: flip the sign bit, read the byte as 2^23 + (sc + 128), subtract both offsets
        const float f_a = byte_plus_2p23((&tl.sa.x)[s >> 2] ^ 0x80808080u, s & 3) - 8388736.0f;
        const float f_b = byte_plus_2p23((&tl.sb.x)[s >> 2] ^ 0x80808080u, s & 3) - 8388736.0f;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const XFrag<XF32, 4> xf = load_x<XF32, 4>(x_rows[nt], k_tile + 16 * s + 4 * t, n_in);
            float dx[4] = {0.f, 0.f, 0.f, 0.f}, d[4];
            mma_bf16(dx, kNeg, kNeg, kNeg, kNeg, xf.hi[0], xf.hi[1], dx);
            if constexpr (XF32) mma_bf16(dx, kNeg, kNeg, kNeg, kNeg, xf.lo[0], xf.lo[1], dx);
            mma_bf16(d, a0, a1, a2, a3, xf.hi[0], xf.hi[1], dx);
            if constexpr (XF32) mma_bf16(d, a0, a1, a2, a3, xf.lo[0], xf.lo[1], d);
            acc[nt][0] = fmaf(f_a, d[0], acc[nt][0]);
            acc[nt][1] = fmaf(f_a, d[1], acc[nt][1]);
            acc[nt][2] = fmaf(f_b, d[2], acc[nt][2]);
            acc[nt][3] = fmaf(f_b, d[3], acc[nt][3]);
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
    static constexpr int bytes = kQ4TileBytes;
};
template <> struct TileOf<MUSER_DTYPE_Q6_K> {
    using type = Q6Tile;
    static constexpr int bytes = kQ6TileBytes;
};

template <int DT, int NT, bool XF32>
__device__ __forceinline__ void walk_tiles(const uint8_t *image, uint32_t rt, uint32_t nsb, uint32_t sb0, uint32_t sb1,
                                           uint32_t k_off, const void *const (&x_rows)[NT], uint32_t n_in, int lane,
                                           float (&out)[NT][4]) {
    using Tile = typename TileOf<DT>::type;
    constexpr int kBytes = TileOf<DT>::bytes;
    if (sb0 >= sb1) return;
    const uint8_t *tp = image + ((uint64_t)rt * nsb + sb0) * kBytes;
    const int t = lane & 3;
    Tile cur, nxt;
    if constexpr (DT == MUSER_DTYPE_Q4_K) cur = q4_load(tp, lane); else cur = q6_load(tp, lane);
    for (uint32_t sb = sb0; sb < sb1; ++sb) {
        nxt = cur;
        if (sb + 1 < sb1) {
            if constexpr (DT == MUSER_DTYPE_Q4_K) nxt = q4_load(tp + kBytes, lane); else nxt = q6_load(tp + kBytes, lane);
        }
        const int64_t k_tile = (int64_t)sb * 256 - (int64_t)k_off;
        if constexpr (DT == MUSER_DTYPE_Q4_K)
            q4_tile_compute<NT, XF32>(cur, k_tile, x_rows, n_in, t, out);
        else
            q6_tile_compute<NT, XF32>(cur, k_tile, x_rows, n_in, t, out);
        cur = nxt;
        tp += kBytes;
    }
}

// Grid: one CTA per 16-row tile.  The CTA's warps split K evenly and add their partial sums through shared
// memory in a fixed order, so results do not depend on scheduling.
template <int DT, int NT, bool XF32, bool DUAL>
__global__ void __launch_bounds__(kMaxWarps * 32) kquant_matmul_kernel(const KqArgs a) {
    __shared__ float red[DUAL ? 2 : 1][kMaxWarps][4][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t rt = blockIdx.x;
    const uint32_t sb0 = a.nsb * warp / warps, sb1 = a.nsb * (warp + 1) / warps;
    const size_t x_elem = XF32 ? 4 : 2;
    const void *x_rows[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const uint32_t tok = nt * 8 + g;
        x_rows[nt] = tok < a.tokens ? reinterpret_cast<const uint8_t *>(a.x) + (size_t)tok * a.n_in * x_elem : nullptr;
    }
    float out[NT][4], out_up[DUAL ? NT : 1][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) out[nt][0] = out[nt][1] = out[nt][2] = out[nt][3] = 0.f;
    walk_tiles<DT, NT, XF32>(a.image, rt, a.nsb, sb0, sb1, a.k_off, x_rows, a.n_in, lane, out);
    if constexpr (DUAL) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) out_up[nt][0] = out_up[nt][1] = out_up[nt][2] = out_up[nt][3] = 0.f;
        walk_tiles<DT, NT, XF32>(a.image_up, rt, a.nsb, sb0, sb1, a.k_off, x_rows, a.n_in, lane, out_up);
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            red[0][warp][c][lane] = out[nt][c];
            if constexpr (DUAL) red[1][warp][c][lane] = out_up[nt][c];
        }
        __syncthreads();
        if (warp == 0) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float v = red[0][0][c][lane], vu = 0.f;
                for (int w = 1; w < warps; ++w) v += red[0][w][c][lane];
                if constexpr (DUAL) {
                    vu = red[1][0][c][lane];
                    for (int w = 1; w < warps; ++w) vu += red[1][w][c][lane];
                    v = __fdiv_rn(v, 1.0f + expf(-v)) * vu; // silu_fast(gate) * up, quant/helpers.rs:72
                }
                const uint32_t row = rt * 16 + g + 8 * (c >> 1);
                const uint32_t tok = nt * 8 + 2 * t + (c & 1);
                if (row < a.n_out && tok < a.tokens) {
                    const size_t o = (size_t)tok * a.n_out + row;
                    if (a.row_scale) v *= a.row_scale[tok];
                    if (a.y_bf16) {
                        if (a.residual) v += __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(a.residual)[o]);
                        reinterpret_cast<__nv_bfloat16 *>(a.y)[o] = __float2bfloat16_rn(v);
                    } else {
                        if (a.residual) v += reinterpret_cast<const float *>(a.residual)[o];
                        reinterpret_cast<float *>(a.y)[o] = v;
                    }
                }
            }
        }
        __syncthreads();
    }
}

template <int DT, bool XF32, bool DUAL>
static cudaError_t launch_nt(const KqArgs &a, uint32_t row_tiles, int warps, cudaStream_t stream) {
    const int nt = (a.tokens + 7) / 8;
    dim3 grid(row_tiles), block(warps * 32);
    if (nt <= 1) kquant_matmul_kernel<DT, 1, XF32, DUAL><<<grid, block, 0, stream>>>(a);
    else if (nt <= 2) kquant_matmul_kernel<DT, 2, XF32, DUAL><<<grid, block, 0, stream>>>(a);
    else if constexpr (!DUAL) {
        if (nt <= 4) kquant_matmul_kernel<DT, 4, XF32, false><<<grid, block, 0, stream>>>(a);
        else kquant_matmul_kernel<DT, 8, XF32, false><<<grid, block, 0, stream>>>(a);
    }
    return cudaGetLastError();
}

muser_cuda_status launch_kquant_matmul(Ctx *ctx, const Weight *w, const Weight *w_up, const void *x, uint32_t x_dtype,
                                       void *y, uint32_t y_dtype, uint32_t tokens, const Epilogue &ep,
                                       cudaStream_t stream) {
    KqArgs a;
    a.image = w->image;
    a.image_up = w_up ? w_up->image : nullptr;
    a.x = x;
    a.y = y;
    a.row_scale = ep.row_scale;
    a.residual = ep.residual;
    a.n_out = (uint32_t)w->n_out;
    a.n_in = (uint32_t)w->n_in;
    a.nsb = w->nsb;
    a.k_off = w->k_off;
    a.tokens = tokens;
    a.y_bf16 = y_dtype == MUSER_DTYPE_BF16;
    const bool xf32 = x_dtype == MUSER_DTYPE_F32, dual = w_up != nullptr;
    const int warps = w->nsb >= 32 ? 8 : (w->nsb >= 4 ? 4 : (int)w->nsb);
    cudaError_t e;
    if (w->dtype == MUSER_DTYPE_Q4_K) {
        if (dual) e = xf32 ? launch_nt<MUSER_DTYPE_Q4_K, true, true>(a, w->row_tiles, warps, stream)
                           : launch_nt<MUSER_DTYPE_Q4_K, false, true>(a, w->row_tiles, warps, stream);
        else e = xf32 ? launch_nt<MUSER_DTYPE_Q4_K, true, false>(a, w->row_tiles, warps, stream)
                      : launch_nt<MUSER_DTYPE_Q4_K, false, false>(a, w->row_tiles, warps, stream);
    } else {
        if (dual) e = xf32 ? launch_nt<MUSER_DTYPE_Q6_K, true, true>(a, w->row_tiles, warps, stream)
                           : launch_nt<MUSER_DTYPE_Q6_K, false, true>(a, w->row_tiles, warps, stream);
        else e = xf32 ? launch_nt<MUSER_DTYPE_Q6_K, true, false>(a, w->row_tiles, warps, stream)
                      : launch_nt<MUSER_DTYPE_Q6_K, false, false>(a, w->row_tiles, warps, stream);
    }
    MUSER_CUDA_TRY(ctx, e);
    return MUSER_CUDA_OK;
}

} // namespace muser
