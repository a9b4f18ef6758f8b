// Decode GEMV for Q4_K / Q6_K weights, 1 to 8 tokens: y[t][r] = dot(W_r, x_t).
//
// Stands in for the single-token routes of MetalKernels::encode_quantized_matmul
// (crates/muser-engine/src/metal/encode/qkv.rs:425-449), encode_quantized_decode_group (qkv.rs:234-281) and
// encode_ffn_q4k_gate_up_silu_4r2s (src/metal/encode/ffn.rs:10-36); on the CPU lane, weights::matmul with
// quant::dot_q4_k_f32 / dot_q6_k_f32 (src/weights.rs:398-421).
//
// HBM-bound by design: every weight byte is read once, with warp-wide 512-byte loads in the order the
// repacked tile stores it (kquant_layout.cuh).  What had to be engineered is the instruction count, because
// the integer/logic pipe of an SM retires half as many instructions per clock as the FMA pipe:
//   - the 4-bit (6-bit) quants go into int8 tensor-core fragments (mma.sync m16n8k32 u8 x s8 -> s32): four
//     weights per AND, no conversion to floating point;
//   - activations are turned, once per CTA, into 15-bit fixed point per sub-block (x ~ sx * (128 hi + lo),
//     two int8 planes, |error| <= amax(sub-block) * 2^-15) and parked in shared memory in fragment order;
//   - the fragment's eight output columns stand for eight sub-blocks (one token) or four sub-blocks x two
//     tokens, not for eight tokens: the k-slots of lane t always carry the sub-blocks lane t owns, and only the
//     lanes whose column is that sub-block feed activations (the others read a zero block), so the B operand
//     is block diagonal and one accumulator collects the exact integer dot products of a whole tile side by
//     side.  The scale / min arithmetic of quant/k_block.rs:178-240 and quant/k_block/q6.rs:90-141 then runs
//     once per tile in f32, including the per-sub-block activation scale.
// Weight tiles travel global -> shared memory as single bulk copies (one 2304- or 3360-byte cp.async.bulk per tile,
// issued by one lane, completion on an mbarrier), two tiles ahead per warp: the bytes in flight that a
// 6.5 TB/s stream needs no longer cost registers.  Every wait on those barriers is bounded.
// Work is cut into (row tile, K slice) items so that every SM stays busy to the end; the K slices of a row
// tile meet in a scratch buffer and the last CTA to arrive adds them in slice order (deterministic).
#include <algorithm>
#include <cmath>

#include "common.cuh"
#include "kquant_layout.cuh"
#include "rmsnorm.cuh"

namespace muser {

struct GemvArgs {
    const uint8_t *image;
    const uint8_t *image_up; // second weight of the fused gate/up call, else null
    const void *x;           // [tokens][n_in], bf16 or (x_f32) f32
    void *y;
    const float *row_scale;
    float out_scale, softcap; // LM-head tail
    const void *residual;
    const float *norm_weight; // fused input RMSNorm (reference.rs:73-80), or null
    float norm_eps;
    float *partial;          // [ksplit][images][tokens][n_out] partial sums (ksplit > 1)
    unsigned int *counters;  // [row_tiles] arrival counters, zero between launches
    int *status;             // context status words; [1] records a wait that gave up
    uint32_t n_out, n_in, nsb, k_off, tokens, y_bf16, x_f32, row_tiles, ksplit, groups, max_tiles;
};

constexpr int kRing = 2;                 // weight tiles in flight per warp
constexpr uint32_t kWaitLimit = 1u << 22; // polls before a wait gives up

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tile_fetch(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ bool tile_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kWaitLimit; ++i) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void imma(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                     uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t gw(const uint4 &v, int i) { return (&v.x)[i]; } // compile-time i only
__device__ __forceinline__ uint32_t sel2(uint32_t a, uint32_t b, int i) { return i ? b : a; }
__device__ __forceinline__ float byte_f32(uint32_t w, int idx) { // float(byte idx of w), idx may be a run-time value
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u + idx)) - 8388608.0f;
}

template <int DT> struct Fmt;
template <> struct Fmt<MUSER_DTYPE_Q4_K> {
    static constexpr int kBlock = 32, kSubs = 8, kTileBytes = kQ4TileBytes;
};
template <> struct Fmt<MUSER_DTYPE_Q6_K> {
    static constexpr int kBlock = 16, kSubs = 16, kTileBytes = kQ6TileBytes;
};

// ------------------------------------------------------------------------------------ activation staging
// Shared memory, per tile of 256 inputs: 1 KiB of B fragments, 16 bytes per (MMA, feeding lane):
// (b0 of the high plane, b1 of the high plane, b0 of the low plane, b1 of the low plane).
//   one token : entry ((a * 8 + c) * V + v): column c of accumulator a (sub-block 8a + c), MMA v; columns 0-3
//               live in b0 (k-slots 4t..4t+3 of lane t = c), columns 4-7 in b1, the other half is zero.
//   two tokens: entry (((tok * SUBS) + j) * V + v): sub-block j of token tok, b0 and b1 both carry data.
// More tokens are NG groups of two, 1 KiB per group and tile.  Plus kSubs * tokens (scale, integer sum) pairs per tile.
template <int DT, int MT, int NG>
__device__ __forceinline__ void stage_activations(const GemvArgs &a, uint32_t sb_first, uint32_t n_tiles, uint4 *frag,
                                                  float2 *meta, const float *inv_rms) {
    constexpr int BW = Fmt<DT>::kBlock, SUBS = Fmt<DT>::kSubs, PARTS = BW / 8; // threads per sub-block, 8 values each
    constexpr int V = MT == 1 ? BW / 4 : BW / 8;                               // MMAs that consume one sub-block
    constexpr int TOK = MT * NG;                                               // tokens, in NG groups of MT
    const uint32_t items = n_tiles * TOK * SUBS * PARTS;
    // whole sub-blocks stay inside one warp, so the shuffles below always find their partners
    for (uint32_t base = 0; base < items; base += blockDim.x) {
        const uint32_t it = base + threadIdx.x;
        const bool live = it < items;
        const uint32_t part = it % PARTS, j = (it / PARTS) % SUBS, tok = (it / (PARTS * SUBS)) % TOK;
        const uint32_t tile = it / (PARTS * SUBS * TOK);
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
        const int64_t k = (int64_t)(sb_first + tile) * 256 - (int64_t)a.k_off + j * BW + part * 8;
        if (live && tok < a.tokens && (uint64_t)k < a.n_in) {
            if (a.x_f32) load8<true>(reinterpret_cast<const float *>(a.x) + (size_t)tok * a.n_in + k, 0, v);
            else load8<false>(reinterpret_cast<const __nv_bfloat16 *>(a.x) + (size_t)tok * a.n_in + k, 0, v);
            if (a.norm_weight) { // (x * 1/rms) * weight, in that order
                const float rs = inv_rms[tok];
                const float4 w0 = __ldg(reinterpret_cast<const float4 *>(a.norm_weight + k)), w1 = __ldg(reinterpret_cast<const float4 *>(a.norm_weight + k) + 1);
                const float nw[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(v[i], rs), nw[i]);
            }
        }
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
        for (int o = 1; o < PARTS; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const bool usable = amax > 0.f && amax < 3.0e38f; // an all-zero or non-finite sub-block contributes nothing
        const float inv = usable ? __fdiv_rn(16383.0f, amax) : 0.f;
        int xi[8], sum = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            xi[i] = __float2int_rn(v[i] * inv);
            sum += xi[i];
        }
#pragma unroll
        for (int o = 1; o < PARTS; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (!live) continue;
        if (part == 0) meta[(tile * SUBS + j) * TOK + tok] = make_float2(usable ? __fdiv_rn(amax, 16383.0f) : 0.f, (float)sum);
        // byte order inside an MMA's k-slots must match how the weights come out of their words
        auto pack = [&](int e0, int e1, int e2, int e3, uint32_t &hi, uint32_t &lo) {
            const int e[4] = {e0, e1, e2, e3};
            hi = lo = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                hi |= (uint32_t)((xi[e[b]] >> 7) & 0xFF) << (8 * b);
                lo |= (uint32_t)(xi[e[b]] & 127) << (8 * b);
            }
        };
        uint32_t h0, l0, h1, l1;
        if constexpr (DT == MUSER_DTYPE_Q4_K) { // word nibbles: even positions hold elements 0,4,1,5, odd 2,6,3,7
            pack(0, 4, 1, 5, h0, l0);
            pack(2, 6, 3, 7, h1, l1);
        } else { // byte b of a Q6_K word: element b in the low nibble, element 4 + b in the high nibble
            pack(0, 1, 2, 3, h0, l0);
            pack(4, 5, 6, 7, h1, l1);
        }
        uint4 *dst = frag + ((size_t)tile * NG + tok / MT) * 64;
        if constexpr (MT == 1) {
            const uint32_t acc = j / 8, col = j % 8;
            const bool low = col < 4;
            uint4 *e = dst + (acc * 8 + col) * V + part * 2;
            e[0] = low ? make_uint4(h0, 0, l0, 0) : make_uint4(0, h0, 0, l0);
            e[1] = low ? make_uint4(h1, 0, l1, 0) : make_uint4(0, h1, 0, l1);
        } else {
            dst[((tok % MT) * SUBS + j) * V + part] = make_uint4(h0, h1, l0, l1);
        }
    }
}

// ------------------------------------------------------------------------------------ Q4_K
struct Q4Regs {
    uint4 q[4]; // [2*rowsel + hi]: row g + 8*rowsel, sub-block t + 4*hi
    uint4 ha, hb;
};
__device__ __forceinline__ Q4Regs load_regs(const uint8_t *tile, int lane, Q4Regs *) { // tile: shared memory
    Q4Regs r;
    const uint4 *q = reinterpret_cast<const uint4 *>(tile);
#pragma unroll
    for (int i = 0; i < 4; ++i) r.q[i] = q[32 * i + lane];
    const uint4 *h = reinterpret_cast<const uint4 *>(tile + 2048);
    r.ha = h[lane >> 2];
    r.hb = h[(lane >> 2) + 8];
    return r;
}
struct Q4Hdr {
    float d, dmin;
    uint32_t sc[2], mn[2];
    __device__ __forceinline__ float scale(int j) const { return d * byte_f32(sel2(sc[0], sc[1], j >> 2), j & 3); }
    __device__ __forceinline__ float minv(int j) const { return dmin * byte_f32(sel2(mn[0], mn[1], j >> 2), j & 3); }
};
__device__ __forceinline__ Q4Hdr q4_hdr(uint4 h) { // 6-bit (scale, min) unpack of quant/k_block.rs:22-31, four at a time
    Q4Hdr s;
    const __half2 dd = *reinterpret_cast<const __half2 *>(&h.x);
    s.d = __low2float(dd);
    s.dmin = __high2float(dd);
    s.sc[0] = h.y & 0x3F3F3F3Fu;
    s.mn[0] = h.z & 0x3F3F3F3Fu;
    s.sc[1] = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
    s.mn[1] = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
    return s;
}
__device__ __forceinline__ uint32_t nib4(uint32_t w, int odd) { return (odd ? w >> 4 : w) & 0x0F0F0F0Fu; }

// out[gp][c]: c = 0, 1 -> row g, c = 2, 3 -> row g+8; with two tokens per group the low bit of c is the token.
// fb: this lane's fragment entries of group 0, `gs` entries further for each next group (0 for lanes that read zeros).
template <int MT, int NG>
__device__ __forceinline__ void tile_compute(const Q4Regs &r, const uint4 *fb, uint32_t gs, const float2 *meta, int t,
                                             float (&out)[NG][4]) {
    constexpr int TOK = MT * NG;
    const Q4Hdr ha = q4_hdr(r.ha), hb = q4_hdr(r.hb);
    if constexpr (MT == 1) {
        int dh[4] = {0, 0, 0, 0}, dl[4] = {0, 0, 0, 0};
#pragma unroll
        for (int v = 0; v < 8; ++v) { // elements 8(v/2) .. +7 of sub-blocks t (k-slots 4t..) and t + 4 (k-slots 16+4t..)
            const uint4 b = fb[v];
            const uint32_t a0 = nib4(gw(r.q[0], v >> 1), v & 1), a2 = nib4(gw(r.q[1], v >> 1), v & 1);
            const uint32_t a1 = nib4(gw(r.q[2], v >> 1), v & 1), a3 = nib4(gw(r.q[3], v >> 1), v & 1);
            imma(dh, a0, a1, a2, a3, b.x, b.y);
            imma(dl, a0, a1, a2, a3, b.z, b.w);
        }
        const float4 m = *reinterpret_cast<const float4 *>(meta + 2 * t); // (sx, sum) of sub-blocks 2t and 2t + 1
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int j = 2 * t + e;
            const float sx = e ? m.z : m.x, xs = e ? m.w : m.y;
            const float pa = (float)(dh[e] * 128 + dl[e]), pb = (float)(dh[2 + e] * 128 + dl[2 + e]);
            out[0][0] = fmaf(sx, fmaf(ha.scale(j), pa, -ha.minv(j) * xs), out[0][0]);
            out[0][2] = fmaf(sx, fmaf(hb.scale(j), pb, -hb.minv(j) * xs), out[0][2]);
        }
    } else {
#pragma unroll
        for (int a = 0; a < 2; ++a) { // this lane's k-slots carry sub-block 4a + t
            int dh[NG][4], dl[NG][4];
#pragma unroll
            for (int gp = 0; gp < NG; ++gp)
#pragma unroll
                for (int c = 0; c < 4; ++c) dh[gp][c] = dl[gp][c] = 0;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const uint32_t wg = gw(r.q[a], v), wg8 = gw(r.q[2 + a], v);
                const uint32_t a0 = nib4(wg, 0), a2 = nib4(wg, 1), a1 = nib4(wg8, 0), a3 = nib4(wg8, 1);
#pragma unroll
                for (int gp = 0; gp < NG; ++gp) {
                    const uint4 b = fb[gp * gs + a * 16 + v]; // (4a + t) * 4 + v, the lane's base already holds t * 4
                    imma(dh[gp], a0, a1, a2, a3, b.x, b.y);
                    imma(dl[gp], a0, a1, a2, a3, b.z, b.w);
                }
            }
            const int j = 4 * a + t;
            const float s_a = ha.scale(j), m_a = ha.minv(j), s_b = hb.scale(j), m_b = hb.minv(j);
#pragma unroll
            for (int gp = 0; gp < NG; ++gp) {
                const float4 m = *reinterpret_cast<const float4 *>(meta + j * TOK + 2 * gp); // both tokens of the group
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float sx = e ? m.z : m.x, xs = e ? m.w : m.y;
                    const float pa = (float)(dh[gp][e] * 128 + dl[gp][e]), pb = (float)(dh[gp][2 + e] * 128 + dl[gp][2 + e]);
                    out[gp][e] = fmaf(sx, fmaf(s_a, pa, -m_a * xs), out[gp][e]);
                    out[gp][2 + e] = fmaf(sx, fmaf(s_b, pb, -m_b * xs), out[gp][2 + e]);
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------ Q6_K
struct Q6Regs {
    uint4 lo[4]; // [2*rowsel + half]
    uint4 hi[2]; // [rowsel]
    uint4 sa, sb;
    float da, db;
};
__device__ __forceinline__ Q6Regs load_regs(const uint8_t *tile, int lane, Q6Regs *) { // tile: shared memory
    Q6Regs r;
    const uint4 *q = reinterpret_cast<const uint4 *>(tile);
#pragma unroll
    for (int i = 0; i < 4; ++i) r.lo[i] = q[32 * i + lane];
    const uint4 *h = reinterpret_cast<const uint4 *>(tile + kQ6OffHi);
    r.hi[0] = h[lane];
    r.hi[1] = h[32 + lane];
    const uint4 *s = reinterpret_cast<const uint4 *>(tile + kQ6OffSc);
    r.sa = s[lane >> 2];
    r.sb = s[(lane >> 2) + 8];
    const __half *d = reinterpret_cast<const __half *>(tile + kQ6OffD);
    r.da = __half2float(d[lane >> 2]);
    r.db = __half2float(d[(lane >> 2) + 8]);
    return r;
}
// int8 scale j as f32: flip the sign bit so the byte reads as sc + 128, then take the 128 off again
__device__ __forceinline__ float q6_scale(const uint4 &sc, int j) {
    const int w = j >> 2;
    const uint32_t word = sel2(sel2(sc.x, sc.y, w & 1), sel2(sc.z, sc.w, w & 1), w >> 1);
    return byte_f32(word ^ 0x80808080u, j & 3) - 128.0f;
}
// elements 4x .. 4x+3 of one sub-block as bytes: low nibbles from `lo`, two high bits from `hi`
__device__ __forceinline__ uint32_t q6_bytes(uint32_t lo, uint32_t hi, int x) {
    const uint32_t n = ((x & 1) ? lo >> 4 : lo) & 0x0F0F0F0Fu;
    const uint32_t h = x == 0 ? hi << 4 : x == 1 ? hi << 2 : x == 2 ? hi : hi >> 2;
    return n | (h & 0x30303030u);
}

template <int MT, int NG>
__device__ __forceinline__ void tile_compute(const Q6Regs &r, const uint4 *fb, uint32_t gs, const float2 *meta, int t,
                                             float (&out)[NG][4]) {
    constexpr int TOK = MT * NG;
    float acc[NG][4];
#pragma unroll
    for (int gp = 0; gp < NG; ++gp) acc[gp][0] = acc[gp][1] = acc[gp][2] = acc[gp][3] = 0.f;
    if constexpr (MT == 1) {
#pragma unroll
        for (int a = 0; a < 2; ++a) { // sub-blocks 8a + t (owned index 2a) and 8a + t + 4 (owned index 2a + 1)
            int dh[4] = {0, 0, 0, 0}, dl[4] = {0, 0, 0, 0};
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const uint4 b = fb[a * 32 + v]; // (a * 8 + column) * 4 + v, the lane's base already holds column * 4
                const uint32_t a0 = q6_bytes(gw(r.lo[a], v >> 1), gw(r.hi[0], 2 * a), v);
                const uint32_t a2 = q6_bytes(gw(r.lo[a], 2 + (v >> 1)), gw(r.hi[0], 2 * a + 1), v);
                const uint32_t a1 = q6_bytes(gw(r.lo[2 + a], v >> 1), gw(r.hi[1], 2 * a), v);
                const uint32_t a3 = q6_bytes(gw(r.lo[2 + a], 2 + (v >> 1)), gw(r.hi[1], 2 * a + 1), v);
                imma(dh, a0, a1, a2, a3, b.x, b.y);
                imma(dl, a0, a1, a2, a3, b.z, b.w);
            }
            const float4 m = *reinterpret_cast<const float4 *>(meta + 8 * a + 2 * t);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = 8 * a + 2 * t + e;
                const float sx = e ? m.z : m.x, xs32 = 32.0f * (e ? m.w : m.y);
                // sum (q - 32) x = sum q x - 32 sum x
                acc[0][0] = fmaf(q6_scale(r.sa, j) * sx, (float)(dh[e] * 128 + dl[e]) - xs32, acc[0][0]);
                acc[0][2] = fmaf(q6_scale(r.sb, j) * sx, (float)(dh[2 + e] * 128 + dl[2 + e]) - xs32, acc[0][2]);
            }
        }
    } else {
#pragma unroll
        for (int a = 0; a < 4; ++a) { // this lane's k-slots carry sub-block 4a + t (owned index a)
            int dh[NG][4], dl[NG][4];
#pragma unroll
            for (int gp = 0; gp < NG; ++gp)
#pragma unroll
                for (int c = 0; c < 4; ++c) dh[gp][c] = dl[gp][c] = 0;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const uint32_t lg = gw(r.lo[a >> 1], (a & 1) * 2 + u), lg8 = gw(r.lo[2 + (a >> 1)], (a & 1) * 2 + u);
                const uint32_t a0 = q6_bytes(lg, gw(r.hi[0], a), 2 * u), a2 = q6_bytes(lg, gw(r.hi[0], a), 2 * u + 1);
                const uint32_t a1 = q6_bytes(lg8, gw(r.hi[1], a), 2 * u), a3 = q6_bytes(lg8, gw(r.hi[1], a), 2 * u + 1);
#pragma unroll
                for (int gp = 0; gp < NG; ++gp) {
                    const uint4 b = fb[gp * gs + a * 8 + u]; // (4a + t) * 2 + u, the lane's base already holds t * 2
                    imma(dh[gp], a0, a1, a2, a3, b.x, b.y);
                    imma(dl[gp], a0, a1, a2, a3, b.z, b.w);
                }
            }
            const int j = 4 * a + t;
            const float f_a = q6_scale(r.sa, j), f_b = q6_scale(r.sb, j);
#pragma unroll
            for (int gp = 0; gp < NG; ++gp) {
                const float4 m = *reinterpret_cast<const float4 *>(meta + j * TOK + 2 * gp);
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float sx = e ? m.z : m.x, xs32 = 32.0f * (e ? m.w : m.y);
                    acc[gp][e] = fmaf(f_a * sx, (float)(dh[gp][e] * 128 + dl[gp][e]) - xs32, acc[gp][e]);
                    acc[gp][2 + e] = fmaf(f_b * sx, (float)(dh[gp][2 + e] * 128 + dl[gp][2 + e]) - xs32, acc[gp][2 + e]);
                }
            }
        }
    }
#pragma unroll
    for (int gp = 0; gp < NG; ++gp) {
        out[gp][0] = fmaf(r.da, acc[gp][0], out[gp][0]);
        out[gp][1] = fmaf(r.da, acc[gp][1], out[gp][1]);
        out[gp][2] = fmaf(r.db, acc[gp][2], out[gp][2]);
        out[gp][3] = fmaf(r.db, acc[gp][3], out[gp][3]);
    }
}

// ------------------------------------------------------------------------------------ kernel
// Warps per CTA at most: 14 where two CTAs share an SM (448 threads x 2 leave 72 registers a thread, which is what the
// one- and two-token loops need to stay out of local memory), 16 for the token-group variants (one CTA per SM).
constexpr int gemv_max_warps(int ng) { return ng > 1 ? 16 : 14; }

template <int DT> struct RegsOf;
template <> struct RegsOf<MUSER_DTYPE_Q4_K> { using type = Q4Regs; };
template <> struct RegsOf<MUSER_DTYPE_Q6_K> { using type = Q6Regs; };

// blockIdx.x = group * ksplit + slice.  A CTA keeps one K slice for its whole life, so it stages only that part of
// the activations.  Inside the CTA every warp works alone: warp w of group G takes row tiles G * warps + w,
// + groups * warps, ... and streams the slice's tiles of each through its own two-slot ring.  There is no CTA-wide
// synchronisation after the staging.  With more than one slice, a warp drops its 16 x MT partial sums into the
// scratch buffer and bumps the row tile's counter; the warp that finds the counter full adds the slices in order.
template <int DT, int MT, int NG, bool DUAL>
__global__ void __launch_bounds__(gemv_max_warps(NG) * 32, (NG > 1 ? 1 : 2)) kquant_gemv_kernel(const GemvArgs a) {
    using Regs = typename RegsOf<DT>::type;
    constexpr int SUBS = Fmt<DT>::kSubs, kBytes = Fmt<DT>::kTileBytes, kImages = DUAL ? 2 : 1, TOK = MT * NG;
    extern __shared__ uint4 dyn[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t slice = blockIdx.x % a.ksplit, group = blockIdx.x / a.ksplit;
    const uint32_t sb_first = a.nsb * slice / a.ksplit, sb_last = a.nsb * (slice + 1) / a.ksplit, n_tiles = sb_last - sb_first;

    uint4 *zero_block = dyn;                         // 1 KiB that lanes without a column of their own read
    uint4 *frag = dyn + 64;                          // n_tiles x NG KiB
    float2 *meta = reinterpret_cast<float2 *>(frag + (size_t)a.max_tiles * 64 * NG);
    uint8_t *ring_base = reinterpret_cast<uint8_t *>(meta + (size_t)a.max_tiles * SUBS * TOK); // warps x kRing tiles
    uint64_t *bars = reinterpret_cast<uint64_t *>(ring_base + (size_t)warps * kRing * kBytes);
    for (int i = threadIdx.x; i < 64; i += blockDim.x) zero_block[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x < (unsigned)(warps * kRing))
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(bars + threadIdx.x)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");

    // this warp's tiles, over all its row tiles, form one stream: n -> (row tile, image, tile); start it before staging
    const uint32_t first_row = group * warps + warp, row_step = a.groups * warps;
    const uint32_t my_rows = a.row_tiles > first_row ? (a.row_tiles - first_row + row_step - 1) / row_step : 0;
    const uint32_t per_row = n_tiles * kImages, total = per_row * my_rows;
    const uint8_t *images[kImages];
    images[0] = a.image;
    if constexpr (DUAL) images[1] = a.image_up;
    uint8_t *ring = ring_base + (size_t)warp * kRing * kBytes;
    const uint32_t bar0 = smem_addr(bars + warp * kRing);
    // the fetch cursor walks the stream with additions only: (tile in slice, image, row tile) -> tile index in the image
    uint32_t f_tile = first_row * a.nsb + sb_first, f_tl = 0, f_im = 0;
    auto fetch_next = [&](uint32_t slot) { // warp-uniform bookkeeping, lane 0 issues the copy
        const uint8_t *base = images[0];
        if constexpr (DUAL) base = f_im ? images[1] : images[0];
        if (lane == 0) tile_fetch(smem_addr(ring) + slot * kBytes, base + (uint64_t)f_tile * kBytes, kBytes, bar0 + 8 * slot);
        ++f_tile;
        if (++f_tl == n_tiles) {
            f_tl = 0;
            if (DUAL && f_im == 0) {
                f_im = 1;
                f_tile -= n_tiles;
            } else {
                f_im = 0;
                f_tile += row_step * a.nsb - n_tiles;
            }
        }
    };
    __syncthreads(); // barriers initialised
    for (uint32_t i = 0; i < kRing && i < total; ++i) fetch_next(i);
    // the first weight tiles are on their way; everything from here on may depend on the kernel before this one
    pdl_release();
    pdl_wait();

    __shared__ float norm_red[33], inv_rms[TOK];
    if (a.norm_weight) { // every CTA needs the whole row's mean square, whatever its K slice
        for (uint32_t tok = 0; tok < a.tokens; ++tok) {
            const float r = a.x_f32 ? block_inv_rms<true>(reinterpret_cast<const float *>(a.x) + (size_t)tok * a.n_in, a.n_in, a.norm_eps, norm_red)
                                    : block_inv_rms<false>(reinterpret_cast<const __nv_bfloat16 *>(a.x) + (size_t)tok * a.n_in, a.n_in, a.norm_eps, norm_red);
            if (threadIdx.x == 0) inv_rms[tok] = r;
        }
        __syncthreads();
    }
    stage_activations<DT, MT, NG>(a, sb_first, n_tiles, frag, meta, inv_rms);
    __syncthreads();

    // which fragment entries this lane reads, relative to a tile's 1 KiB
    constexpr int V = MT == 1 ? Fmt<DT>::kBlock / 4 : Fmt<DT>::kBlock / 8;
    const bool feeds = MT == 1 ? (g & 3) == t : (g >> 1) == t;
    const uint32_t lane_entry = MT == 1 ? g * V : ((g & 1) * SUBS + t) * V;
    uint32_t n = 0;
    bool healthy = true;

    for (uint32_t rt = first_row; rt < a.row_tiles; rt += row_step) {
        float out[kImages][NG][4];
#pragma unroll
        for (int im = 0; im < kImages; ++im) {
#pragma unroll
            for (int gp = 0; gp < NG; ++gp) out[im][gp][0] = out[im][gp][1] = out[im][gp][2] = out[im][gp][3] = 0.f;
            for (uint32_t tl = 0; tl < n_tiles; ++tl, ++n) {
                if (healthy && !tile_wait(bar0 + 8 * (n & (kRing - 1)), (n / kRing) & 1)) {
                    healthy = false;
                    atomicExch(a.status + 1, 201);
                }
                if (healthy) {
                    const Regs cur = load_regs(ring + (n & (kRing - 1)) * kBytes, lane, (Regs *)nullptr);
                    __syncwarp(); // every lane has its copy: the slot may be refilled
                    if (n + kRing < total) fetch_next(n & (kRing - 1));
                    const uint4 *fb = feeds ? frag + (size_t)tl * 64 * NG + lane_entry : zero_block;
                    tile_compute<MT, NG>(cur, fb, feeds ? 64u : 0u, meta + (size_t)tl * SUBS * TOK, t, out[im]);
                }
            }
            // columns that stand for the same token sit in the four lanes of a quad
#pragma unroll
            for (int gp = 0; gp < NG; ++gp)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    out[im][gp][c] += __shfl_xor_sync(0xffffffffu, out[im][gp][c], 1);
                    out[im][gp][c] += __shfl_xor_sync(0xffffffffu, out[im][gp][c], 2);
                }
        }
        // every lane of a quad now holds, per group gp: c = 0, 1 -> row g, token MT*gp + c; c = 2, 3 -> row g + 8
        bool finish = true;
        if (a.ksplit > 1) {
            if (t == 0) {
#pragma unroll
                for (int im = 0; im < kImages; ++im)
#pragma unroll
                    for (int gp = 0; gp < NG; ++gp)
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const uint32_t row = rt * 16 + g + 8 * (c >> 1), tok = MT * gp + (c & 1);
                            if (row < a.n_out && (c & 1) < MT)
                                a.partial[(((size_t)slice * kImages + im) * TOK + tok) * a.n_out + row] = out[im][gp][c];
                        }
            }
            // Release / acquire through the counter: the warp barrier orders every lane's stores before lane 0's
            // releasing add, and lane 0's acquire (handed on by the shuffle) before every lane's loads below.
            __syncwarp();
            unsigned int seen = 0;
            if (lane == 0) asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(seen) : "l"(a.counters + rt) : "memory");
            seen = __shfl_sync(0xffffffffu, seen, 0);
            finish = seen == a.ksplit - 1;
            if (finish) {
                if (lane == 0) a.counters[rt] = 0; // ready for the next launch
#pragma unroll
                for (int im = 0; im < kImages; ++im)
#pragma unroll
                    for (int gp = 0; gp < NG; ++gp)
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const uint32_t row = rt * 16 + g + 8 * (c >> 1), tok = MT * gp + (c & 1);
                            float sum = 0.f;
                            if (row < a.n_out && (c & 1) < MT)
                                for (uint32_t sl = 0; sl < a.ksplit; ++sl)
                                    sum += __ldcg(a.partial + (((size_t)sl * kImages + im) * TOK + tok) * a.n_out + row);
                            out[im][gp][c] = sum;
                        }
            }
        }
        if (finish && t == 0) {
#pragma unroll
            for (int gc = 0; gc < 4 * NG; ++gc) {
                const int gp = gc >> 2, c = gc & 3;
                const uint32_t row = rt * 16 + g + 8 * (c >> 1), tok = MT * gp + (c & 1);
                if (row >= a.n_out || tok >= a.tokens || (c & 1) >= MT) continue;
                float r = out[0][gp][c];
                if constexpr (DUAL) r = __fdiv_rn(r, 1.0f + expf(-r)) * out[1][gp][c]; // silu_fast(gate) * up, quant/helpers.rs:72
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
}

// ------------------------------------------------------------------------------------ host side
struct GemvPlan {
    int warps, ksplit;
};

// meta_bytes_per_tile also carries the fragment KiB count: fragments are `frag_kib` KiB per tile
static size_t gemv_smem_bytes(uint32_t nsb, int ksplit, int warps, int tile_bytes, int meta_bytes_per_tile, int frag_kib = 1) {
    const uint32_t max_tiles = (nsb + ksplit - 1) / ksplit + 1;
    return 1024 + (size_t)max_tiles * (1024 * frag_kib + meta_bytes_per_tile) + (size_t)warps * kRing * (tile_bytes + 8);
}

// K slices and warps per CTA from a small cost model fitted to profiles of this kernel: a tile costs about 300
// issue slots, a scheduler reaches about 0.12 instructions per clock per resident warp (the tile body is a chain
// of shared-memory loads, unpacking, MMAs and an epilogue), and an SM cannot take tiles faster than HBM delivers
// them (about 100 cycles each).  So: as many busy warps per SM as fit, spread evenly over the SMs, and slices only
// as far as that needs, because every slice costs a trip through the scratch buffer.
static GemvPlan plan_split(uint32_t nsb, uint32_t row_tiles, int sm_count, int tile_bytes, int meta_bytes_per_tile,
                           int frag_kib = 1) {
    GemvPlan best{2, 1};
    double best_cost = 1e300;
    for (int ks = 1; ks <= 16 && (uint32_t)ks <= nsb; ++ks)
        for (int w = 2; w <= gemv_max_warps(frag_kib); w += 2) {
            const size_t smem = gemv_smem_bytes(nsb, ks, w, tile_bytes, meta_bytes_per_tile, frag_kib);
            if (smem > 220u * 1024) continue;
            int ctas = (int)((227u * 1024) / (smem + 1024));
            ctas = std::min(ctas, std::max(1, (frag_kib > 1 ? 16 : 28) / w)); // 72 (128) registers a thread
            const double tiles = std::ceil((double)nsb / ks);
            const double cta_count = std::ceil((double)row_tiles / w) * ks;           // one row tile per warp and round
            const double ctas_on_sm = std::ceil(cta_count / sm_count);                // the busiest SM
            const double busy = std::min(ctas_on_sm, (double)ctas) * w;               // warps at work there
            const double per_tile = std::max(100.0, 77.0 / std::min(0.95, 0.03 * busy));
            const double staging = std::min(ctas_on_sm, (double)ctas) * tiles * 25.0;  // per CTA, before its first tile
            const double per_item = 350.0 + (ks > 1 ? 900.0 : 0.0);                    // epilogue, scratch round trip
            const double cost = ctas_on_sm * w * (tiles * per_tile + per_item / std::max(1.0, busy / 4)) + staging;
            if (cost < best_cost * (1.0 - 1e-9)) best_cost = cost, best = GemvPlan{w, ks};
        }
    return best;
}

template <int DT, int MT, int NG, bool DUAL>
static cudaError_t launch_gemv(GemvArgs &a, Ctx *ctx, cudaStream_t stream) {
    constexpr int kMeta = Fmt<DT>::kSubs * MT * NG * (int)sizeof(float2);
    struct Cached {
        uint32_t nsb = 0, row_tiles = 0, n_out = 0;
        GemvPlan plan{1, 1};
        size_t smem = 0;
        uint32_t groups = 0;
    };
    static PerDevice<Cached> cached; // last geometry of this instantiation, per device
    if (ctx->device < 0 || ctx->device >= kMaxDevices) return cudaErrorInvalidDevice;
    Cached cache;
    {
        std::lock_guard<std::mutex> lock(cached.mu);
        Cached &slot = cached.slot[ctx->device];
        if (slot.nsb != a.nsb || slot.row_tiles != a.row_tiles || slot.n_out != a.n_out) {
            GemvPlan p = plan_split(a.nsb, a.row_tiles, ctx->sm_count, Fmt<DT>::kTileBytes, kMeta, NG);
            const size_t images = DUAL ? 2 : 1;
            while (p.ksplit > 1 && (size_t)p.ksplit * images * MT * NG * a.n_out * sizeof(float) > ctx->gemv_partial_bytes) --p.ksplit;
            if (a.row_tiles > ctx->gemv_counter_slots) p.ksplit = 1;
            const size_t smem = gemv_smem_bytes(a.nsb, p.ksplit, p.warps, Fmt<DT>::kTileBytes, kMeta, NG);
            cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void *>(kquant_gemv_kernel<DT, MT, NG, DUAL>), ctx->device, smem);
            if (e != cudaSuccess) return e;
            int per_sm = 0;
            e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kquant_gemv_kernel<DT, MT, NG, DUAL>, p.warps * 32, smem);
            if (e != cudaSuccess) return e;
            if (per_sm < 1) return cudaErrorInvalidConfiguration;
            // CTAs per slice: all that fit at once, but no more than there are row tiles for their warps
            uint32_t groups = std::max(1u, (uint32_t)per_sm * ctx->sm_count / p.ksplit);
            const uint32_t wanted = (a.row_tiles + p.warps - 1) / p.warps;
            if (groups > wanted) groups = wanted;
            const uint32_t rounds = (wanted + groups - 1) / groups;
            groups = (wanted + rounds - 1) / rounds;
            slot.nsb = a.nsb, slot.row_tiles = a.row_tiles, slot.n_out = a.n_out;
            slot.plan = p, slot.smem = smem, slot.groups = groups;
        }
        cache = slot;
    }
    a.ksplit = cache.plan.ksplit;
    a.groups = cache.groups;
    a.max_tiles = (a.nsb + a.ksplit - 1) / a.ksplit + 1;
    return launch_pdl(kquant_gemv_kernel<DT, MT, NG, DUAL>, dim3(cache.groups * a.ksplit), dim3(cache.plan.warps * 32), cache.smem, stream, a);
}

template <int DT, bool DUAL>
static cudaError_t launch_gemv_tokens(GemvArgs &a, Ctx *ctx, cudaStream_t stream) {
    if (a.tokens == 1) return launch_gemv<DT, 1, 1, DUAL>(a, ctx, stream);
    if (a.tokens == 2) return launch_gemv<DT, 2, 1, DUAL>(a, ctx, stream);
    if (a.tokens <= 4) return launch_gemv<DT, 2, 2, DUAL>(a, ctx, stream);
    return launch_gemv<DT, 2, 4, DUAL>(a, ctx, stream);
}

// 1 to 8 tokens of bf16 activations.  Returns cudaErrorNotSupported when the shape does not fit this kernel
// (the caller then takes the general one).
cudaError_t launch_kquant_gemv(Ctx *ctx, const Weight *w, const Weight *w_up, const void *x, uint32_t x_dtype, void *y,
                               uint32_t y_dtype, uint32_t tokens, const Epilogue &ep, cudaStream_t stream) {
    if (tokens > 8 || w->nsb > 2048) return cudaErrorNotSupported;
    GemvArgs a;
    a.image = w->image;
    a.image_up = w_up ? w_up->image : nullptr;
    a.x = x;
    a.x_f32 = x_dtype == MUSER_DTYPE_F32;
    a.y = y;
    a.row_scale = ep.row_scale;
    a.out_scale = ep.out_scale;
    a.softcap = ep.softcap;
    a.residual = ep.residual;
    a.norm_weight = ep.norm_weight;
    a.norm_eps = ep.norm_eps;
    a.partial = ctx->gemv_partial;
    a.counters = ctx->gemv_counters;
    a.status = ctx->dev_status;
    a.n_out = (uint32_t)w->n_out;
    a.n_in = (uint32_t)w->n_in;
    a.nsb = w->nsb;
    a.k_off = w->k_off;
    a.tokens = tokens;
    a.y_bf16 = y_dtype == MUSER_DTYPE_BF16;
    a.row_tiles = w->row_tiles;
    a.ksplit = a.groups = 1;
    a.max_tiles = 0;
    const bool dual = w_up != nullptr;
    if (w->dtype == MUSER_DTYPE_Q4_K)
        return dual ? launch_gemv_tokens<MUSER_DTYPE_Q4_K, true>(a, ctx, stream) : launch_gemv_tokens<MUSER_DTYPE_Q4_K, false>(a, ctx, stream);
    return dual ? launch_gemv_tokens<MUSER_DTYPE_Q6_K, true>(a, ctx, stream) : launch_gemv_tokens<MUSER_DTYPE_Q6_K, false>(a, ctx, stream);
}

} // namespace muser
