// Decode / small-batch projection for Q4_K, Q5_K and Q6_K weights, 1 to 16 tokens: y[t][r] = dot(W_r, x_t), for up to
// four projections of the same input in one launch.
//
// Stands in for MetalKernels::encode_quantized_matmul at decode (crates/muser-engine/src/metal/encode/qkv.rs:425-449),
// encode_quantized_decode_group (qkv.rs:234-281: up to four sequences per dispatch), the one-barrier-interval dispatch
// of the projections that read the same hidden state (src/decode.rs:5569-5598) and encode_ffn_q4k_gate_up_silu_4r2s
// (src/metal/encode/ffn.rs:10-36); on the CPU lane, weights::matmul with quant::dot_q4_k_f32 / dot_q6_k_f32
// (src/weights.rs:398-421) in the deferred-scale order of quant/k_block.rs:178-240 and quant/k_block/q6.rs:90-141.
//
// HBM-bound by design: every weight byte is read once, as one bulk copy per 16-row x 256-input tile into a private
// ring of the warp that consumes it.  The arithmetic is integer until the last step:
//   - activations become 15-bit fixed point per token and 256-input tile (x ~ sx * (128 hi + lo), two int8 planes,
//     |error| <= amax(tile) * 2^-15), once per CTA, parked in shared memory in tensor-core fragment order;
//   - the 4-bit (6-bit) quants go straight from the tile into int8 mma.sync fragments: the image is laid out so that
//     a lane already owns its fragment's bytes (kquant_layout.cuh);
//   - one MMA multiplies a whole sub-block (32 weights of 16 rows for Q4_K / Q5_K, 16 for Q6_K) with a group of four
//     tokens: the eight fragment columns are (token, plane) pairs, so a lane ends up with the high- and low-plane
//     sums of ITS token for rows g and g + 8 and no value ever crosses lanes;
//   - the sub-block scale (6-bit, or int8 for Q6_K) is applied to the integer sums with integer multiply-adds, the
//     Q4_K min term is an integer dot product of the 6-bit mins with the tile's per-sub-block activation sums, and
//     only the per-256 factors d, dmin and sx are applied in f32, once per tile.
// Work is cut into (row tile, K slice) items; a CTA keeps one K slice (it stages only that part of the
// activations), its warps take row tiles in turn and never synchronise after the staging.  With more than one
// slice the partial sums meet in the context's scratch and the last arriver adds them in slice order
// (deterministic).  Every wait on a copy barrier is bounded.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>
#include <vector>

#include "common.cuh"
#include "kquant_layout.cuh"
#include "oneshot_exchange.h"
#include "rmsnorm.cuh"

namespace muser {

constexpr int kDecMaxJobs = 4;
constexpr uint32_t kDecWaitLimit = 1u << 22; // polls before a wait gives up

struct DecJob {
    const uint8_t *image;
    const uint8_t *image_up; // second weight of the fused gate/up call, else null
    void *y;
    const float *row_scale;
    const void *residual;
    float out_scale, softcap; // LM-head tail
    uint32_t dtype, n_out, row_tiles, y_bf16;
    uint32_t cta0;     // first CTA of this job in the grid
    uint32_t groups;   // CTAs per K slice
    uint32_t counter0; // first arrival counter of this job (one per row tile)
    uint32_t partial0; // first float of this job's partial sums in the scratch
    // fused greedy pick (AMAX kernels only): per token one 64-bit key (ordered value bits, ~row) that every finishing
    // warp raises with an atomic max, and one flag word that records a non-finite output; y may then be null
    unsigned long long *amax_keys;
    unsigned int *amax_flags;
};

struct DecArgs {
    DecJob job[kDecMaxJobs];
    uint32_t n_jobs;
    const void *x;            // [tokens][n_in], bf16 or (x_f32) f32
    const float *norm_weight; // fused input RMSNorm (reference.rs:73-80), or null
    float norm_eps;
    float *partial;
    unsigned int *counters; // zero between launches
    int *status;            // context status words; [1] records a wait that gave up
    uint32_t n_in, nsb, k_off, tokens, x_f32, ksplit, max_tiles, ring /* tiles in flight per warp: 2 or 4 */;
    uint32_t slot_bytes; // bytes of one ring slot: the largest tile among the launch's jobs
    uint32_t wsplit;     // warps of a CTA that share one row tile, each with a part of the CTA's K slice (1: none)
    OneShotPush push;    // PUSH kernels only: job 0's f32 outputs also go to every rank's all-reduce cells as they finish
};

namespace dec {

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
// Weight tiles are read once per launch: they travel with an evict-first L2 policy, so that a launch's 15 to 230 MB
// of weights do not push the kernels' own code, the activations and the split-K scratch out of the 126 MB L2 (a
// launch whose code had been evicted by its predecessor's stream started about 3 us later).
__device__ __forceinline__ uint64_t evict_first_policy() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// One weight tile global -> shared (arrive with the byte count, then the bulk copy with the L2 policy), called by the
// whole (converged) warp: one elected lane issues.  Bulk copies take their operands from the
// warp-uniform registers, and issued from inside an `if (lane == 0)` branch each one cost the warp 100+ cycles.
__device__ __forceinline__ void tile_fetch_elect(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar, uint64_t policy) {
    asm volatile(
        "{\n\t.reg .pred e;\n\telect.sync _|e, 0xffffffff;\n\t"
        "@e mbarrier.arrive.expect_tx.shared::cta.b64 _, [%3], %2;\n\t"
        "@e cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;\n\t}"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
}
__device__ __forceinline__ bool tile_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kDecWaitLimit; ++i) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
// 16 rows x 32 inputs (Q4_K sub-block): unsigned 4-bit weights as bytes times signed activation bytes
__device__ __forceinline__ void imma32(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// 16 rows x 16 inputs (Q6_K sub-block): signed bytes 4 * (q - 32) times signed activation bytes
__device__ __forceinline__ void imma16(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
__device__ __forceinline__ uint32_t gw(const uint4 &v, int i) { return (&v.x)[i]; } // compile-time i only
__device__ __forceinline__ int ubyte(uint32_t w, int i) { return (int)__byte_perm(w, 0u, 0x4440u | (uint32_t)i); }
__device__ __forceinline__ int sbyte(uint32_t w, int i) { // sign-extended byte i: a selector nibble of 8 + i replicates that byte's sign bit
    const uint32_t s = 8u | (uint32_t)i;
    int r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(0u), "r"((s << 12) | (s << 8) | (s << 4) | (uint32_t)i));
    return r;
}

template <int DT> struct Fmt;
template <> struct Fmt<MUSER_DTYPE_Q4_K> { static constexpr int kTileBytes = kQ4TileBytes; };
template <> struct Fmt<MUSER_DTYPE_Q6_K> { static constexpr int kTileBytes = kQ6TileBytes; };
template <> struct Fmt<MUSER_DTYPE_Q5_K> { static constexpr int kTileBytes = kQ5TileBytes; };

constexpr int kFragU4 = 128; // uint4 of B fragments per (tile, token group): 4 fragment quads x 32 lanes
constexpr int kMetaU4 = 2;   // uint4 per (tile, token): sx, then (Q4_K) the eight sub-block sums as three byte planes

// ------------------------------------------------------------------------------------ activation staging
// One warp turns one (tile, token) into fragment bytes: lane l holds inputs 8l .. 8l+7 of the tile.
//   Q4_K: sub-block j = l / 4, quarter tq = l % 4; the lane's eight values are exactly what fragment lane (., tq)
//         feeds for that sub-block: b0 = elements (0, 4, 1, 5) of its eight (the order in which the low nibbles of a
//         weight word come out), b1 = elements (2, 6, 3, 7).  Entry (tile, group, j / 2, column, tq) is a uint4
//         (b0_j, b1_j, b0_j+1, b1_j+1) for even j; the column is 2 * (token % 4) + plane.
//   Q6_K: sub-block s = l / 2; the lane's values are the bytes of fragment lanes 2 * (l % 2) and 2 * (l % 2) + 1.
//         Entry (tile, group, s / 4, column, t) is a uint4 over sub-blocks 4 * (s / 4) .. + 3.
template <int DT, int NG>
__device__ __forceinline__ void stage(const DecArgs &a, uint32_t sb_first, uint32_t n_tiles, uint4 *frag, uint4 *meta, const float *inv_rms) {
    constexpr int TOK = 4 * NG;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    uint32_t *fw = reinterpret_cast<uint32_t *>(frag), *mw = reinterpret_cast<uint32_t *>(meta);
    // one task = one (tile, token); a warp takes its tasks a few at a time and has all their inputs in flight before
    // it works on the first (the loads come from L2 and would otherwise be paid once per task in turn)
    auto fetch = [&](uint32_t task, float (&v)[8]) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
        if (task >= n_tiles * a.tokens) return;
        const uint32_t tile = task / a.tokens, tok = task % a.tokens;
        const int64_t k = (int64_t)(sb_first + tile) * 256 - (int64_t)a.k_off + 8 * lane;
        if ((uint64_t)k < a.n_in) { // a negative k wraps to a huge value
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
    };
    // columns of tokens that do not exist are zero; meta entries of such tokens are never used for a stored result
    if (a.tokens < (uint32_t)TOK) {
        const uint32_t per_tile = NG * kFragU4;
        for (uint32_t i = threadIdx.x; i < n_tiles * per_tile; i += blockDim.x) {
            const uint32_t col = (i % 32) >> 2, tok = 4 * ((i % per_tile) / kFragU4) + (col >> 1); // entry (quad, column, t)
            if (tok >= a.tokens) frag[i] = make_uint4(0, 0, 0, 0);
        }
        for (uint32_t i = threadIdx.x; i < n_tiles * TOK * kMetaU4; i += blockDim.x)
            if ((i / kMetaU4) % TOK >= a.tokens) meta[i] = make_uint4(0, 0, 0, 0);
    }
    const uint32_t n_tasks = n_tiles * a.tokens; // task -> (tile, token < tokens)
    constexpr int kBatch = NG >= 3 ? 4 : 2;      // tasks whose inputs are in flight together (they come from L2)
    for (uint32_t task0 = warp * kBatch; task0 < n_tasks; task0 += warps * kBatch) {
      float vb[kBatch][8];
#pragma unroll
      for (int bi = 0; bi < kBatch; ++bi) fetch(task0 + bi, vb[bi]);
#pragma unroll
      for (int bi = 0; bi < kBatch; ++bi) {
        const uint32_t task = task0 + bi;
        if (task >= n_tasks) break;
        const uint32_t tile = task / a.tokens, tok = task % a.tokens, gp = tok >> 2, t4 = tok & 3;
        float (&v)[8] = vb[bi];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        bool nan = false;
#pragma unroll
        for (int i = 0; i < 8; ++i) nan = nan || v[i] != v[i];
        // an all-zero tile contributes nothing; a tile with a NaN or an infinity makes every output of its token NaN
        // (its integers are zero and its scale is NaN), as such inputs do on the CPU lane
        const bool poisoned = __any_sync(0xffffffffu, nan) || !(amax < 3.0e38f);
        const bool usable = amax > 0.f && !poisoned;
        const float inv = usable ? __fdiv_rn(16383.0f, amax) : 0.f;
        int xi[8], sum = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            xi[i] = __float2int_rn(v[i] * inv);
            sum += xi[i];
        }
        auto pack = [&](int e0, int e1, int e2, int e3, uint32_t &hi, uint32_t &lo) {
            const int e[4] = {e0, e1, e2, e3};
            hi = lo = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                hi |= (uint32_t)((xi[e[b]] >> 7) & 0xFF) << (8 * b);
                lo |= (uint32_t)(xi[e[b]] & 127) << (8 * b);
            }
        };
        const float sx = usable ? __fdiv_rn(amax, 16383.0f) : poisoned ? __uint_as_float(0x7FC00000u) : 0.f;
        uint32_t *mrow = mw + (size_t)(tile * TOK + tok) * (kMetaU4 * 4);
        uint32_t *fbase = fw + (size_t)(tile * NG + gp) * (kFragU4 * 4);
        if constexpr (DT != MUSER_DTYPE_Q6_K) { // Q4_K and Q5_K: 32-element sub-blocks with a min term
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            const uint32_t j = lane >> 2, tq = lane & 3;
            uint32_t h0, l0, h1, l1;
            pack(0, 4, 1, 5, h0, l0);
            pack(2, 6, 3, 7, h1, l1);
            uint32_t *e = fbase + (((j >> 1) * 32 + (2 * t4) * 4 + tq) * 4 + (j & 1) * 2);
            *reinterpret_cast<uint2 *>(e) = make_uint2(h0, h1);      // column 2 * t4: high plane
            *reinterpret_cast<uint2 *>(e + 16) = make_uint2(l0, l1); // column 2 * t4 + 1: low plane
            // the sub-block's integer sum S (|S| <= 2^19) as three byte planes, S = 2^14 s2 + 2^7 s1 + s0 with s0, s1 in
            // 0..127 and s2 signed, so that four sub-blocks' worth multiply a word of 6-bit mins in one dp4a each
            if (tq == 0) {
                uint8_t *mb = reinterpret_cast<uint8_t *>(mrow + 1);
                mb[j] = (uint8_t)(sum & 127);
                mb[8 + j] = (uint8_t)((sum >> 7) & 127);
                mb[16 + j] = (uint8_t)((sum >> 14) & 0xFF);
            }
            if (lane == 0) mrow[0] = __float_as_uint(sx);
        } else {
            const uint32_t s = lane >> 1, t = 2 * (lane & 1);
            uint32_t h0, l0, h1, l1;
            pack(0, 1, 2, 3, h0, l0);
            pack(4, 5, 6, 7, h1, l1);
            uint32_t *e = fbase + (((s >> 2) * 32 + (2 * t4) * 4 + t) * 4 + (s & 3));
            e[0] = h0, e[4] = h1;   // fragment lanes t and t + 1 of the high-plane column
            e[16] = l0, e[20] = l1; // and of the low-plane column
            if (lane == 0) mrow[0] = __float_as_uint(sx * 0.25f); // the fragment bytes are 4 * (q - 32)
        }
      }
    }
}

// ------------------------------------------------------------------------------------ Q4_K tile
struct Q4Regs {
    uint4 q[4]; // [2*rowsel + half]: row g + 8*rowsel, word jj = sub-block 4*half + jj, this lane's eight elements
    uint4 ha, hb;
};
struct Q5Regs {
    uint4 q[4];
    uint4 hbits; // [2*rowsel + half]: byte jj = the fifth bits of the lane's eight elements of sub-block 4*half + jj
    uint4 ha, hb;
};
__device__ __forceinline__ Q5Regs load_regs(const uint8_t *tile, int lane, Q5Regs *) { // tile: shared memory
    Q5Regs r;
    const uint4 *q = reinterpret_cast<const uint4 *>(tile);
#pragma unroll
    for (int i = 0; i < 4; ++i) r.q[i] = q[32 * i + lane];
    r.hbits = reinterpret_cast<const uint4 *>(tile + kQ5OffHi)[lane];
    const uint4 *h = reinterpret_cast<const uint4 *>(tile + kQ5OffHdr);
    r.ha = h[lane >> 2];
    r.hb = h[(lane >> 2) + 8];
    return r;
}
// four fifth bits (x < 16) onto bit 4 of four bytes
__device__ __forceinline__ uint32_t spread_bit4(uint32_t x) { return (x * 0x02040810u) & 0x10101010u; }
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
    uint32_t sc[2], mn[2]; // 6-bit values as bytes: sub-blocks 0-3, 4-7 (quant/k_block.rs:22-31)
};
__device__ __forceinline__ Q4Hdr q4_hdr(uint4 h) {
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

// out[gp][0 / 1]: row g / g + 8, token 4 * gp + t.  fb: this lane's fragment entries of the tile; mt: the tile's meta.
// Regs is Q4Regs or Q5Regs: the same arithmetic on 4-bit or 5-bit quants.
template <int NG, typename Regs>
__device__ __forceinline__ void q45_compute(const Regs &r, const uint4 *fb, const uint4 *mt, int t, float (&out)[NG][2]) {
    constexpr bool Q5 = sizeof(Regs) == sizeof(Q5Regs);
    const Q4Hdr ha = q4_hdr(r.ha), hb = q4_hdr(r.hb);
    int acc[NG][4];
#pragma unroll
    for (int gp = 0; gp < NG; ++gp) acc[gp][0] = acc[gp][1] = acc[gp][2] = acc[gp][3] = 0;
#pragma unroll
    for (int jp = 0; jp < 4; ++jp) {
        uint4 b[NG];
#pragma unroll
        for (int gp = 0; gp < NG; ++gp) b[gp] = fb[(gp * 4 + jp) * 32];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int j = 2 * jp + e;
            const uint32_t wa = gw(r.q[j >> 2], j & 3), wb = gw(r.q[2 + (j >> 2)], j & 3);
            uint32_t a0 = wa & 0x0F0F0F0Fu, a2 = (wa >> 4) & 0x0F0F0F0Fu;
            uint32_t a1 = wb & 0x0F0F0F0Fu, a3 = (wb >> 4) & 0x0F0F0F0Fu;
            if constexpr (Q5) {
                const uint32_t ba = (uint32_t)ubyte(gw(r.hbits, j >> 2), j & 3), bb = (uint32_t)ubyte(gw(r.hbits, 2 + (j >> 2)), j & 3);
                a0 |= spread_bit4(ba & 15u), a2 |= spread_bit4(ba >> 4);
                a1 |= spread_bit4(bb & 15u), a3 |= spread_bit4(bb >> 4);
            }
            const int sa = ubyte(ha.sc[j >> 2], j & 3), sb = ubyte(hb.sc[j >> 2], j & 3);
#pragma unroll
            for (int gp = 0; gp < NG; ++gp) {
                int d[4];
                imma32(d, a0, a1, a2, a3, e ? b[gp].z : b[gp].x, e ? b[gp].w : b[gp].y);
                acc[gp][0] += sa * d[0];
                acc[gp][1] += sa * d[1];
                acc[gp][2] += sb * d[2];
                acc[gp][3] += sb * d[3];
            }
        }
    }
#pragma unroll
    for (int gp = 0; gp < NG; ++gp) {
        const uint4 *m = mt + (gp * 4 + t) * kMetaU4;
        const uint4 m0 = m[0], m1 = m[1];
        // sum_j min_j S_j with S_j = 2^14 s2 + 2^7 s1 + s0: planes (m0.y, m0.z), (m0.w, m1.x), (m1.y, m1.z)
        auto dot8 = [](const uint32_t (&mn)[2], uint32_t p0, uint32_t p1) { return __dp4a((int)mn[0], (int)p0, __dp4a((int)mn[1], (int)p1, 0)); };
        const int a0 = dot8(ha.mn, m0.y, m0.z), a1 = dot8(ha.mn, m0.w, m1.x), a2 = dot8(ha.mn, m1.y, m1.z);
        const int b0 = dot8(hb.mn, m0.y, m0.z), b1 = dot8(hb.mn, m0.w, m1.x), b2 = dot8(hb.mn, m1.y, m1.z);
        const int mina = (a2 << 14) + (a1 << 7) + a0, minb = (b2 << 14) + (b1 << 7) + b0;
        const float sx = __uint_as_float(m0.x);
        const float pa = fmaf(128.0f, (float)acc[gp][0], (float)acc[gp][1]), pb = fmaf(128.0f, (float)acc[gp][2], (float)acc[gp][3]);
        out[gp][0] = fmaf(sx, fmaf(-ha.dmin, (float)mina, ha.d * pa), out[gp][0]);
        out[gp][1] = fmaf(sx, fmaf(-hb.dmin, (float)minb, hb.d * pb), out[gp][1]);
    }
}

template <int NG>
__device__ __forceinline__ void tile_compute(const Q4Regs &r, const uint4 *fb, const uint4 *mt, int t, float (&out)[NG][2]) {
    q45_compute<NG>(r, fb, mt, t, out);
}
template <int NG>
__device__ __forceinline__ void tile_compute(const Q5Regs &r, const uint4 *fb, const uint4 *mt, int t, float (&out)[NG][2]) {
    q45_compute<NG>(r, fb, mt, t, out);
}

// ------------------------------------------------------------------------------------ Q6_K tile
struct Q6Regs {
    uint4 top[4]; // [2*rowsel + half]
    uint4 low[2]; // [rowsel]
    uint4 sa, sb;
    float da, db;
};
__device__ __forceinline__ Q6Regs load_regs(const uint8_t *tile, int lane, Q6Regs *) { // tile: shared memory
    Q6Regs r;
    const uint4 *q = reinterpret_cast<const uint4 *>(tile);
#pragma unroll
    for (int i = 0; i < 4; ++i) r.top[i] = q[32 * i + lane];
    const uint4 *h = reinterpret_cast<const uint4 *>(tile + kQ6OffHi);
    r.low[0] = h[lane];
    r.low[1] = h[32 + lane];
    const uint4 *s = reinterpret_cast<const uint4 *>(tile + kQ6OffSc);
    r.sa = s[lane >> 2];
    r.sb = s[(lane >> 2) + 8];
    const __half *d = reinterpret_cast<const __half *>(tile + kQ6OffD);
    r.da = __half2float(d[lane >> 2]);
    r.db = __half2float(d[(lane >> 2) + 8]);
    return r;
}
// the signed bytes 4 * (q - 32) of this lane's four elements of sub-block s, row selector rs
template <int S>
__device__ __forceinline__ uint32_t q6_bytes(const Q6Regs &r, int rs) {
    const uint32_t tw = gw(r.top[2 * rs + (S >> 3)], (S & 7) >> 1), lw = gw(r.low[rs], S >> 2);
    const uint32_t top = (S & 1) ? tw : tw << 4;
    constexpr int x = S & 3;
    const uint32_t low = x == 0 ? lw << 2 : x == 1 ? lw : x == 2 ? lw >> 2 : lw >> 4;
    return (top & 0xF0F0F0F0u) | (low & 0x0C0C0C0Cu);
}

template <int NG, int S>
__device__ __forceinline__ void q6_sub_block(const Q6Regs &r, const uint4 (&b)[NG], int (&acc)[NG][4]) {
    const uint32_t a0 = q6_bytes<S>(r, 0), a1 = q6_bytes<S>(r, 1);
    const int sa = sbyte(gw(r.sa, S >> 2), S & 3), sb = sbyte(gw(r.sb, S >> 2), S & 3);
#pragma unroll
    for (int gp = 0; gp < NG; ++gp) {
        int d[4];
        imma16(d, a0, a1, gw(b[gp], S & 3));
        acc[gp][0] += sa * d[0];
        acc[gp][1] += sa * d[1];
        acc[gp][2] += sb * d[2];
        acc[gp][3] += sb * d[3];
    }
}

template <int NG>
__device__ __forceinline__ void tile_compute(const Q6Regs &r, const uint4 *fb, const uint4 *mt, int t, float (&out)[NG][2]) {
    int acc[NG][4];
#pragma unroll
    for (int gp = 0; gp < NG; ++gp) acc[gp][0] = acc[gp][1] = acc[gp][2] = acc[gp][3] = 0;
#define MUSER_Q6_QUAD(Q)                                                     \
    {                                                                        \
        uint4 b[NG];                                                         \
        _Pragma("unroll") for (int gp = 0; gp < NG; ++gp) b[gp] = fb[(gp * 4 + (Q)) * 32]; \
        q6_sub_block<NG, 4 * (Q) + 0>(r, b, acc);                            \
        q6_sub_block<NG, 4 * (Q) + 1>(r, b, acc);                            \
        q6_sub_block<NG, 4 * (Q) + 2>(r, b, acc);                            \
        q6_sub_block<NG, 4 * (Q) + 3>(r, b, acc);                            \
    }
    MUSER_Q6_QUAD(0)
    MUSER_Q6_QUAD(1)
    MUSER_Q6_QUAD(2)
    MUSER_Q6_QUAD(3)
#undef MUSER_Q6_QUAD
#pragma unroll
    for (int gp = 0; gp < NG; ++gp) {
        const float sx = __uint_as_float(mt[(gp * 4 + t) * kMetaU4].x); // includes the 1/4 of the fragment bytes
        const float pa = fmaf(128.0f, (float)acc[gp][0], (float)acc[gp][1]), pb = fmaf(128.0f, (float)acc[gp][2], (float)acc[gp][3]);
        out[gp][0] = fmaf(sx * r.da, pa, out[gp][0]);
        out[gp][1] = fmaf(sx * r.db, pb, out[gp][1]);
    }
}

// Zero, but only once every shared-memory load that filled `r` has delivered: one word of each load goes into an
// instruction whose result the compiler cannot see through.  The ring slot is refilled by a bulk copy (asynchronous
// proxy) right after the warp has read it (generic proxy): the reads must be complete and a proxy fence must stand
// between them and the copy.  While one thread issued the copy from inside a divergent branch, the ~100 cycles that
// cost hid the hazard; with the copy issued 20 cycles after the loads, one call in a few hundred of the 16-token
// ffn_down projection (ring of two, 14 K slices) read a slot that was being refilled.  Adding this zero to the copy's
// byte count makes the copy wait for the loaded registers; the fence orders the two proxies.
__device__ __forceinline__ uint32_t opaque_zero(uint32_t x) {
    uint32_t z;
    asm volatile("and.b32 %0, %1, 0;" : "=r"(z) : "r"(x));
    return z;
}
__device__ __forceinline__ uint32_t regs_landed(const Q4Regs &r) {
    return opaque_zero(r.q[0].x ^ r.q[1].x ^ r.q[2].x ^ r.q[3].x ^ r.ha.x ^ r.hb.x);
}
__device__ __forceinline__ uint32_t regs_landed(const Q5Regs &r) {
    return opaque_zero(r.q[0].x ^ r.q[1].x ^ r.q[2].x ^ r.q[3].x ^ r.hbits.x ^ r.ha.x ^ r.hb.x);
}
__device__ __forceinline__ uint32_t regs_landed(const Q6Regs &r) {
    return opaque_zero(r.top[0].x ^ r.top[1].x ^ r.top[2].x ^ r.top[3].x ^ r.low[0].x ^ r.low[1].x ^ r.sa.x ^ r.sb.x ^
                       __float_as_uint(r.da) ^ __float_as_uint(r.db));
}

template <int DT> struct RegsOf;
template <> struct RegsOf<MUSER_DTYPE_Q4_K> { using type = Q4Regs; };
template <> struct RegsOf<MUSER_DTYPE_Q6_K> { using type = Q6Regs; };
template <> struct RegsOf<MUSER_DTYPE_Q5_K> { using type = Q5Regs; };

// ------------------------------------------------------------------------------------ one CTA's work
// The CTA's warps form warps / wsplit row slots of wsplit warps each.  Slot r of CTA group G takes row tiles
// G * slots + r, + groups * slots, ...; its warps cut the CTA's K slice into wsplit parts, each streams its part's
// tiles through its own ring, and the parts meet in shared memory (named barrier per slot, first warp adds them in
// part order), which costs a few hundred cycles where the exchange between CTAs through global memory costs
// microseconds.  Small weights, which need every warp of the GPU to hide HBM latency, are split this way.
// Largest first, and among equal values the lowest row first: the scalar first-maximum convention of the reference's
// greedy pick (crates/muser-engine/src/api.rs:1842-1850, shaders/ferrite/argmax_f32.metal).  A NaN yields key 0 and
// never wins.
__device__ __forceinline__ unsigned long long amax_key(float v, uint32_t row) {
    if (v != v) return 0ull;
    uint32_t u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return (unsigned long long)u << 32 | (0xFFFFFFFFu - row);
}

// The store half of the one-shot all-reduce's device memory policy (collective.cu has the whole of it).
struct PushCells {
    __device__ __forceinline__ void store(xchg::Cell *p, uint32_t bits, uint32_t seq) {
        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(bits), "r"(seq) : "memory");
    }
};

template <int DT, int NG, bool DUAL, bool AMAX = false, bool PUSH = false>
__device__ __forceinline__ void run(const DecArgs &a, const DecJob &jb, uint32_t group, uint32_t slice, uint4 *dyn, float *inv_rms) {
    using Regs = typename RegsOf<DT>::type;
    constexpr int kBytes = Fmt<DT>::kTileBytes, kImages = DUAL ? 2 : 1, TOK = 4 * NG;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t sb_first = a.nsb * slice / a.ksplit, sb_last = a.nsb * (slice + 1) / a.ksplit, n_tiles = sb_last - sb_first;
    const uint32_t ring_n = a.ring, ring_mask = a.ring - 1, ring_shift = a.ring == 4 ? 2 : 1;

    uint4 *frag = dyn;                                                  // max_tiles x NG x 2 KiB
    uint4 *meta = frag + (size_t)a.max_tiles * NG * kFragU4;            // max_tiles x TOK x 48 bytes
    uint8_t *ring_base = reinterpret_cast<uint8_t *>(meta + (size_t)a.max_tiles * TOK * kMetaU4);
    uint64_t *bars = reinterpret_cast<uint64_t *>(ring_base + (size_t)warps * ring_n * a.slot_bytes); // sized for the launch's largest tile
    constexpr int kOutWords = kImages * NG * 2;                         // partial sums per lane
    float *red = reinterpret_cast<float *>(bars + warps * ring_n);      // [2][warps][kOutWords][32], used when wsplit > 1
    if (threadIdx.x < (unsigned)(warps * ring_n))
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(bars + threadIdx.x)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");

    // this warp's tiles, over all its row tiles, form one stream: n -> (row tile, image, tile); start it before staging
    const uint32_t wsplit = a.wsplit, slots = warps / wsplit, wslot = warp / wsplit, wpart = warp % wsplit;
    const uint32_t t_first = n_tiles * wpart / wsplit, my_tiles = n_tiles * (wpart + 1) / wsplit - t_first; // this warp's part of the slice
    const uint32_t first_row = group * slots + wslot, row_step = jb.groups * slots;
    const uint32_t my_rows = jb.row_tiles > first_row ? (jb.row_tiles - first_row + row_step - 1) / row_step : 0;
    const uint32_t per_row = my_tiles * kImages, total = per_row * my_rows;
    uint8_t *ring = ring_base + (size_t)warp * ring_n * kBytes;
    const uint32_t bar0 = smem_addr(bars + warp * ring_n);
    uint32_t f_tile = first_row * a.nsb + sb_first + t_first, f_tl = 0, f_im = 0;
    const uint64_t policy = evict_first_policy();
    auto fetch_next = [&](uint32_t slot, uint32_t zero_after_reads = 0) { // warp-uniform bookkeeping, one elected lane issues the copy
        const uint8_t *base = jb.image;
        if constexpr (DUAL) base = f_im ? jb.image_up : jb.image;
        tile_fetch_elect(smem_addr(ring) + slot * kBytes, base + (uint64_t)f_tile * kBytes, kBytes + zero_after_reads, bar0 + 8 * slot, policy);
        ++f_tile;
        if (++f_tl == my_tiles) {
            f_tl = 0;
            if (DUAL && f_im == 0) {
                f_im = 1;
                f_tile -= my_tiles;
            } else {
                f_im = 0;
                f_tile += row_step * a.nsb - my_tiles;
            }
        }
    };
    __syncthreads(); // barriers initialised
    for (uint32_t i = 0; i < ring_n && i < total; ++i) fetch_next(i);
    // the first weight tiles are on their way; everything from here on may depend on the kernel before this one
    pdl_release();
    pdl_wait();

    __shared__ float norm_red[33];
    if (a.norm_weight) { // every CTA needs the whole row's mean square, whatever its K slice
        for (uint32_t tok = 0; tok < a.tokens; ++tok) {
            const float r = a.x_f32 ? block_inv_rms<true>(reinterpret_cast<const float *>(a.x) + (size_t)tok * a.n_in, a.n_in, a.norm_eps, norm_red)
                                    : block_inv_rms<false>(reinterpret_cast<const __nv_bfloat16 *>(a.x) + (size_t)tok * a.n_in, a.n_in, a.norm_eps, norm_red);
            if (threadIdx.x == 0) inv_rms[tok] = r;
        }
        __syncthreads();
    }
    stage<DT, NG>(a, sb_first, n_tiles, frag, meta, inv_rms);
    __syncthreads();

    uint32_t n = 0, iter = 0;
    bool healthy = true;
    for (uint32_t rt = first_row; rt < jb.row_tiles; rt += row_step, ++iter) {
        float out[kImages][NG][2];
#pragma unroll
        for (int im = 0; im < kImages; ++im) {
#pragma unroll
            for (int gp = 0; gp < NG; ++gp) out[im][gp][0] = out[im][gp][1] = 0.f;
            for (uint32_t tl = t_first; tl < t_first + my_tiles; ++tl, ++n) {
                const uint32_t slot = n & ring_mask;
                // (the warp agrees on the outcome: the fetch below is issued by an elected lane of the WHOLE warp)
                if (healthy && !__all_sync(0xffffffffu, tile_wait(bar0 + 8 * slot, (n >> ring_shift) & 1))) {
                    healthy = false;
                    atomicExch(a.status + 1, 211);
                }
                if (healthy) {
                    const Regs cur = load_regs(ring + slot * kBytes, lane, (Regs *)nullptr);
                    __syncwarp(); // every lane has issued its loads; regs_landed makes the refill wait for their data
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // generic-proxy reads before the async-proxy refill
                    if (n + ring_n < total) fetch_next(slot, regs_landed(cur));
                    tile_compute<NG>(cur, frag + (size_t)tl * NG * kFragU4 + lane, meta + (size_t)tl * TOK * kMetaU4, t, out[im]);
                }
            }
        }
        // this lane now holds, per group gp: [0] -> row g, [1] -> row g + 8, token 4 * gp + t
        if (wsplit > 1) {
            // the slot's warps meet: every warp leaves its sums, the first one adds them in part order.  Two buffers
            // taken in turn: a warp can be at most one row tile ahead of the slot's first warp (the next barrier needs
            // that warp too), so what it writes is never what is still being read.
            float *mine = red + ((size_t)(iter & 1) * warps + warp) * (kOutWords * 32) + lane;
#pragma unroll
            for (int im = 0; im < kImages; ++im)
#pragma unroll
                for (int gp = 0; gp < NG; ++gp) {
                    mine[((im * NG + gp) * 2 + 0) * 32] = out[im][gp][0];
                    mine[((im * NG + gp) * 2 + 1) * 32] = out[im][gp][1];
                }
            asm volatile("bar.sync %0, %1;" ::"r"(1 + wslot), "r"(wsplit * 32) : "memory");
            if (wpart != 0) continue;
#pragma unroll
            for (int im = 0; im < kImages; ++im)
#pragma unroll
                for (int gp = 0; gp < NG; ++gp)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        float sum = out[im][gp][c];
                        for (uint32_t p = 1; p < wsplit; ++p) sum += mine[(size_t)p * (kOutWords * 32) + ((im * NG + gp) * 2 + c) * 32];
                        out[im][gp][c] = sum;
                    }
        }
        bool finish = true;
        if (a.ksplit > 1) {
#pragma unroll
            for (int im = 0; im < kImages; ++im)
#pragma unroll
                for (int gp = 0; gp < NG; ++gp)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const uint32_t row = rt * 16 + g + 8 * c, tok = 4 * gp + t;
                        if (row < jb.n_out && tok < a.tokens)
                            a.partial[jb.partial0 + (((size_t)slice * kImages + im) * TOK + tok) * jb.n_out + row] = out[im][gp][c];
                    }
            // Release / acquire through the counter: the warp barrier orders every lane's stores before lane 0's
            // releasing add, and lane 0's acquire (handed on by the shuffle) before every lane's loads below.
            __syncwarp();
            unsigned int seen = 0;
            if (lane == 0) asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(seen) : "l"(a.counters + jb.counter0 + rt) : "memory");
            seen = __shfl_sync(0xffffffffu, seen, 0);
            finish = seen == a.ksplit - 1;
            if (finish) {
                if (lane == 0) a.counters[jb.counter0 + rt] = 0; // ready for the next launch
#pragma unroll
                for (int im = 0; im < kImages; ++im)
#pragma unroll
                    for (int gp = 0; gp < NG; ++gp)
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            const uint32_t row = rt * 16 + g + 8 * c, tok = 4 * gp + t;
                            float sum = 0.f;
                            if (row < jb.n_out && tok < a.tokens)
                                for (uint32_t sl = 0; sl < a.ksplit; ++sl)
                                    sum += __ldcg(a.partial + jb.partial0 + (((size_t)sl * kImages + im) * TOK + tok) * jb.n_out + row);
                            out[im][gp][c] = sum;
                        }
            }
        }
        if (finish) {
#pragma unroll
            for (int gp = 0; gp < NG; ++gp) {
                unsigned long long best = 0ull; // AMAX: this lane's rows g, g + 8 of token 4 * gp + t
                bool bad = false;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const uint32_t row = rt * 16 + g + 8 * c, tok = 4 * gp + t;
                    if (row >= jb.n_out || tok >= a.tokens) continue;
                    float r = out[0][gp][c];
                    if constexpr (DUAL) r = __fdiv_rn(r, 1.0f + expf(-r)) * out[1][gp][c]; // silu_fast(gate) * up, quant/helpers.rs:72
                    const size_t o = (size_t)tok * jb.n_out + row;
                    if (jb.row_scale) r *= jb.row_scale[tok];
                    r = logit_tail(r, jb.out_scale, jb.softcap);
                    if (jb.y_bf16) {
                        if (jb.residual) r += __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(jb.residual)[o]);
                        if (!AMAX || jb.y) reinterpret_cast<__nv_bfloat16 *>(jb.y)[o] = __float2bfloat16_rn(r);
                    } else {
                        if (jb.residual) r += reinterpret_cast<const float *>(jb.residual)[o];
                        if (!AMAX || jb.y) reinterpret_cast<float *>(jb.y)[o] = r;
                        if constexpr (PUSH) {
                            // the row-parallel projection's partial sum leaves for every rank the moment it exists:
                            // the transfer over NVLink runs beside the rest of this kernel's tiles, and the kernel
                            // that follows only gathers.  The call's sequence number is the one that kernel will
                            // take: this chunk's counter + 1.
                            PushCells cells;
                            // (read past L1: the counter was bumped by a kernel that may have run beside this one's start)
                            const uint32_t e = (uint32_t)o, seq = __ldcg(a.push.seq + e / xchg::kChunkElems) + 1;
                            xchg::push_element(cells, reinterpret_cast<xchg::Cell *const *>(a.push.peer), a.push.rank, a.push.world, seq, e, r);
                        }
                    }
                    if constexpr (AMAX) {
                        const unsigned long long key = amax_key(r, row);
                        best = key > best ? key : best;
                        bad = bad || !(fabsf(r) <= 3.402823466e38f);
                    }
                }
                if constexpr (AMAX) {
                    // the eight lanes that share a token column hold the tile's 16 rows of it: one candidate per token
                    // and row tile, and an atomic only if it would beat what is there already
#pragma unroll
                    for (int o = 4; o < 32; o <<= 1) {
                        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
                        best = other > best ? other : best;
                    }
                    const uint32_t bad_lanes = __ballot_sync(0xffffffffu, bad);
                    const uint32_t tok = 4 * gp + t;
                    if (g == 0 && tok < a.tokens) {
                        if (best != 0ull && best > *reinterpret_cast<volatile unsigned long long *>(jb.amax_keys + tok)) atomicMax(jb.amax_keys + tok, best);
                        if (bad_lanes & (0x11111111u << t)) atomicOr(jb.amax_flags + tok, 1u);
                    }
                }
            }
        }
    }
}

// One CTA per SM, so that the activations are staged once per SM: up to 28 warps for one token group (72 registers a
// thread), 24 for two (80 registers), 16 beyond.
constexpr int max_warps(int ng) { return ng == 1 ? 28 : ng == 2 ? 24 : 16; }
constexpr int ctas_per_sm(int ng) { return 1; }

} // namespace dec

// blockIdx.x -> (job, CTA group, K slice): a job's CTAs are contiguous, group-major.
// FAM 0: jobs of Q4_K and Q6_K in any mix (the layer's projections); FAM 1: Q5_K jobs only (the LM head), compiled
// apart so that the common kernels do not carry its code.  Everything else that varies between the launches of a
// decode step (warps, K slices, warp parts, jobs) is a run-time argument of ONE function per token-group count:
// measured on a B200, a launch whose function differs from its predecessor's starts ~3 us later when the predecessor
// streamed enough weights to push the code out of L2 (instruction fetches then miss all the way to HBM), which is
// more than any specialised variant saved.
template <int NG, bool DUAL, int FAM>
__global__ void __launch_bounds__(dec::max_warps(NG) * 32, dec::ctas_per_sm(NG)) kquant_decode_kernel(const __grid_constant__ DecArgs a) {
    extern __shared__ uint4 dec_dyn[];
    __shared__ float inv_rms[4 * NG];
    uint32_t ji = 0;
#pragma unroll
    for (uint32_t i = 1; i < kDecMaxJobs; ++i)
        if (i < a.n_jobs && blockIdx.x >= a.job[i].cta0) ji = i;
    const DecJob &jb = a.job[ji];
    const uint32_t local = blockIdx.x - jb.cta0, slice = local % a.ksplit, group = local / a.ksplit;
    constexpr bool AMAX = FAM == 2 || FAM == 3; // FAM 0, 1 with the fused greedy pick over the output rows (the LM head)
    constexpr bool PUSH = FAM == 4;             // FAM 0 whose f32 outputs are also pushed into the all-reduce's cells
    if constexpr ((FAM & 1) == 1) {
        dec::run<MUSER_DTYPE_Q5_K, NG, DUAL, AMAX, PUSH>(a, jb, group, slice, dec_dyn, inv_rms);
    } else {
        if (jb.dtype == MUSER_DTYPE_Q4_K) dec::run<MUSER_DTYPE_Q4_K, NG, DUAL, AMAX, PUSH>(a, jb, group, slice, dec_dyn, inv_rms);
        else dec::run<MUSER_DTYPE_Q6_K, NG, DUAL, AMAX, PUSH>(a, jb, group, slice, dec_dyn, inv_rms);
    }
}

// ------------------------------------------------------------------------------------ host side
namespace {

struct DecPlan {
    int warps, ksplit, ring, wsplit;
};

// fmt: 0 = Q4_K jobs only, 1 = Q6_K among them (the largest tile), 2 = Q5_K
constexpr int fmt_tile_bytes(int fmt) { return fmt == 0 ? kQ4TileBytes : fmt == 1 ? kQ6TileBytes : kQ5TileBytes; }

size_t dec_smem_bytes(uint32_t nsb, int ksplit, int warps, int ring, int ng, int fmt, int out_words) {
    const uint32_t max_tiles = (nsb + ksplit - 1) / ksplit + 1;
    return (size_t)max_tiles * ng * (dec::kFragU4 * 16 + 4 * dec::kMetaU4 * 16) + (size_t)warps * ring * (fmt_tile_bytes(fmt) + 8) +
           (size_t)2 * warps * out_words * 32 * sizeof(float) + 16;
}

// Warps per CTA, K slices between CTAs (`ksplit`, met through global scratch), K parts between the warps of a CTA
// (`wsplit`, met through shared memory) from a cost model in SM cycles, fitted to timings of ~1800 (shape, tokens,
// plan) combinations on a B200: a warp needs about 1300 (Q4_K) / 1750 (Q6_K) cycles per tile, 1450 / 1600 more per
// further token group, whatever the number of warps beside it up to 16 an SM and ~7 % more per warp beyond; the
// tensor cannot arrive faster than HBM delivers it; staging costs every CTA ~930 warp cycles per (tile, token) spread
// over its warps; a meeting in shared memory costs ~330 cycles, one through global memory ~5800; a launch ~5900.
// The landscape is rugged (whether the row tiles fill one wave of CTAs exactly matters more than anything smooth), so
// the model ranks the candidates and muser_cuda_decode_autotune can measure the best of them.
struct DecCandidate {
    DecPlan plan;
    double cost;
};

void dec_candidates(uint32_t nsb, uint32_t row_tiles, int sm_count, int ng, int fmt, uint32_t tokens, int out_words, std::vector<DecCandidate> &out) {
    out.clear();
    const double t_warp = (fmt == 1 ? 1750.0 : fmt == 2 ? 1800.0 : 1300.0) + (ng - 1) * (fmt == 1 ? 1600.0 : 1450.0);
    const double bytes = (double)nsb * row_tiles * fmt_tile_bytes(fmt), hbm_bytes_per_cycle = 2800.0;
    const int max_w = dec::max_warps(ng), batch = ng >= 3 ? 4 : 2, ring = 2;
    static const int kParts[] = {1, 2, 3, 4, 5, 6, 7, 8, 10, 12};
    for (int ks = 1; ks <= 16 && (uint32_t)ks <= nsb; ++ks)
        for (int ws : kParts)
            for (int w = 4; w <= max_w; w += 2) {
                if (w % ws) continue;
                const int slots = w / ws;
                if (ws > 1 && slots > 15) continue; // one named barrier per slot
                if ((uint32_t)ws > nsb / ks) continue;
                const double tiles_cta = std::ceil((double)nsb / ks), tiles_warp = std::ceil(tiles_cta / ws);
                const size_t smem = dec_smem_bytes(nsb, ks, w, ring, ng, fmt, out_words);
                if (smem > 220u * 1024) continue;
                int ctas = (int)((227u * 1024) / (smem + 1024));
                ctas = std::min(ctas, std::max(1, max_w / w)); // the register file
                const double wanted = std::ceil((double)row_tiles / slots); // CTAs per slice if every slot took one row tile
                const double groups = std::min(wanted, std::floor((double)ctas * sm_count / ks));
                if (groups < 1.0) continue;
                const double rows_per_slot = std::ceil(wanted / groups);
                const double ctas_on_sm = std::ceil(groups * ks / sm_count); // the busiest SM
                const double busy = ctas_on_sm * w;                          // warps at work there
                const double tasks = tiles_cta * tokens;
                const double staging = ctas_on_sm * (std::ceil(tasks / (w * batch)) * 100.0 + tasks * 930.0 / w);
                const double warp_time = rows_per_slot * tiles_warp * t_warp * (1.0 + 0.066 * std::max(0.0, busy - 16.0));
                const double tail = rows_per_slot * ((ws > 1 ? 330.0 : 0.0) + (ks > 1 ? 5800.0 : 0.0));
                out.push_back({DecPlan{w, ks, ring, ws}, 5900.0 + staging + std::max(warp_time, bytes / hbm_bytes_per_cycle) + tail});
            }
    std::sort(out.begin(), out.end(), [](const DecCandidate &x, const DecCandidate &y) { return x.cost < y.cost; });
}

DecPlan dec_plan(uint32_t nsb, uint32_t row_tiles, int sm_count, int ng, int fmt, uint32_t tokens, int out_words) {
    std::vector<DecCandidate> c;
    dec_candidates(nsb, row_tiles, sm_count, ng, fmt, tokens, out_words, c);
    return c.empty() ? DecPlan{2, 1, 2, 1} : c[0].plan;
}

// Plans that muser_cuda_decode_autotune measured, per device: (jobs' row tiles, dtype mix, nsb, token groups, fused
// gate/up) -> plan per token count.  Looked up before the cost model.
struct TunedKey {
    uint32_t nsb, n_jobs, rows[kDecMaxJobs], q6, dual, tokens;
    bool operator<(const TunedKey &o) const { return memcmp(this, &o, sizeof(*this)) < 0; }
};
struct TunedTable {
    std::mutex mu;
    std::map<TunedKey, DecPlan> plans[kMaxDevices];
    uint32_t generation[kMaxDevices] = {}; // bumped (under mu) when a device's plans change, so cached launch plans are looked up again
};
TunedTable &tuned_table() {
    static TunedTable t;
    return t;
}
TunedKey tuned_key(const DecArgs &a, bool dual) {
    TunedKey k;
    memset(&k, 0, sizeof(k));
    k.nsb = a.nsb, k.n_jobs = a.n_jobs, k.dual = dual, k.tokens = a.tokens;
    for (uint32_t i = 0; i < a.n_jobs; ++i) {
        k.rows[i] = a.job[i].row_tiles;
        k.q6 |= (a.job[i].dtype == MUSER_DTYPE_Q6_K ? 1u : a.job[i].dtype == MUSER_DTYPE_Q5_K ? 2u : 0u) << (2 * i);
    }
    return k;
}

template <int NG, bool DUAL, int FAM>
cudaError_t dec_launch(DecArgs &a, Ctx *ctx, const DecPlan &forced, cudaStream_t stream) {
    struct Cached {
        uint32_t nsb = 0, rows[kDecMaxJobs] = {0, 0, 0, 0}, n_jobs = 0;
        int fmt = 0;
        DecPlan plan{1, 1, 2, 1};
        size_t smem = 0;
        uint32_t groups[kDecMaxJobs] = {0, 0, 0, 0};
        uint32_t forced_w = 0, forced_k = 0, forced_r = 0, forced_s = 0, tokens = 0, generation = 0;
    };
    // The geometries this instantiation was launched with lately, per device: a decode step alternates between a
    // handful (q|k|v, o, gate|up, down, each at a few token counts), and working a plan out again (cost model,
    // occupancy query) costs tens of microseconds of host time, more than the launch itself.
    struct CacheSet {
        Cached entry[16];
        uint32_t next = 0;
    };
    static PerDevice<CacheSet> cached;
    if (ctx->device < 0 || ctx->device >= kMaxDevices) return cudaErrorInvalidDevice;
    Cached cache;
    {
        std::lock_guard<std::mutex> lock(cached.mu);
        CacheSet &set = cached.slot[ctx->device];
        constexpr int kOutWords = (DUAL ? 2 : 1) * NG * 2;
        uint32_t generation;
        {
            TunedTable &tt = tuned_table();
            std::lock_guard<std::mutex> tl(tt.mu);
            generation = tt.generation[ctx->device];
        }
        int fmt = (FAM & 1) == 1 ? 2 : 0;
        uint32_t total_tiles = 0;
        size_t out_floats = 0;
        for (uint32_t i = 0; i < a.n_jobs; ++i) {
            if (a.job[i].dtype == MUSER_DTYPE_Q6_K) fmt = 1;
            total_tiles += a.job[i].row_tiles;
            out_floats += (size_t)(DUAL ? 2 : 1) * 4 * NG * a.job[i].n_out;
        }
        Cached *hit = nullptr;
        for (Cached &c : set.entry) {
            bool same = c.nsb == a.nsb && c.n_jobs == a.n_jobs && c.tokens == a.tokens && c.forced_w == (uint32_t)forced.warps &&
                        c.forced_k == (uint32_t)forced.ksplit && c.forced_r == (uint32_t)forced.ring && c.forced_s == (uint32_t)forced.wsplit &&
                        c.generation == generation && c.fmt == fmt;
            for (uint32_t i = 0; same && i < a.n_jobs; ++i) same = c.rows[i] == a.job[i].row_tiles;
            if (same) {
                hit = &c;
                break;
            }
        }
        const bool same = hit != nullptr;
        Cached &slot = same ? *hit : set.entry[set.next];
        if (!same) {
            set.next = (set.next + 1) % 16;
            DecPlan p = dec_plan(a.nsb, total_tiles, ctx->sm_count, NG, fmt, a.tokens, kOutWords);
            {
                TunedTable &tt = tuned_table();
                std::lock_guard<std::mutex> tl(tt.mu);
                auto it = tt.plans[ctx->device].find(tuned_key(a, DUAL));
                if (it != tt.plans[ctx->device].end()) p = it->second;
            }
            if (forced.warps) p.warps = std::min(forced.warps, dec::max_warps(NG));
            if (forced.ksplit) p.ksplit = (int)std::min<uint32_t>((uint32_t)forced.ksplit, a.nsb);
            if (forced.ring) p.ring = forced.ring >= 4 ? 4 : 2;
            if (forced.wsplit) p.wsplit = forced.wsplit;
            if (forced.warps || forced.ksplit || forced.wsplit) { // a forced plan is made consistent rather than refused
                const uint32_t tiles_cta = a.nsb / p.ksplit; // the shortest slice
                while (p.wsplit > 1 && (p.warps % p.wsplit || (uint32_t)p.wsplit > std::max(1u, tiles_cta) || p.warps / p.wsplit > 15)) --p.wsplit;
            }
            while (p.ksplit > 1 && (size_t)p.ksplit * out_floats * sizeof(float) > ctx->gemv_partial_bytes) --p.ksplit;
            if (total_tiles > ctx->gemv_counter_slots) p.ksplit = 1;
            size_t smem = dec_smem_bytes(a.nsb, p.ksplit, p.warps, p.ring, NG, fmt, kOutWords);
            while (smem > 226u * 1024 && p.ring > 2) p.ring = 2, smem = dec_smem_bytes(a.nsb, p.ksplit, p.warps, p.ring, NG, fmt, kOutWords);
            while (smem > 226u * 1024 && (uint32_t)p.ksplit < a.nsb &&
                   (size_t)(p.ksplit + 1) * out_floats * sizeof(float) <= ctx->gemv_partial_bytes && total_tiles <= ctx->gemv_counter_slots)
                ++p.ksplit, smem = dec_smem_bytes(a.nsb, p.ksplit, p.warps, p.ring, NG, fmt, kOutWords);
            while (smem > 226u * 1024 && p.warps > 2) p.warps -= 2, p.wsplit = 1, smem = dec_smem_bytes(a.nsb, p.ksplit, p.warps, p.ring, NG, fmt, kOutWords);
            if (smem > 226u * 1024) return cudaErrorNotSupported;
            cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void *>(kquant_decode_kernel<NG, DUAL, FAM>), ctx->device, smem);
            if (e != cudaSuccess) return e;
            int per_sm = 0;
            e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kquant_decode_kernel<NG, DUAL, FAM>, p.warps * 32, smem);
            if (e != cudaSuccess) return e;
            if (per_sm < 1) return cudaErrorInvalidConfiguration;
            // CTAs per slice over all jobs: all that fit at once, but no more than there are row tiles for their warps
            const uint32_t slots = (uint32_t)(p.warps / p.wsplit);
            uint32_t wanted = 0;
            for (uint32_t i = 0; i < a.n_jobs; ++i) wanted += (a.job[i].row_tiles + slots - 1) / slots;
            const uint32_t resident = std::max(1u, (uint32_t)per_sm * ctx->sm_count / p.ksplit);
            const uint32_t rounds = (wanted + resident - 1) / resident;
            slot = Cached{};
            for (uint32_t i = 0; i < a.n_jobs; ++i) {
                const uint32_t w_i = (a.job[i].row_tiles + slots - 1) / slots;
                slot.groups[i] = std::max(1u, (w_i + rounds - 1) / rounds);
                slot.rows[i] = a.job[i].row_tiles;
            }
            slot.nsb = a.nsb, slot.n_jobs = a.n_jobs, slot.fmt = fmt;
            slot.plan = p, slot.smem = smem;
            slot.forced_w = forced.warps, slot.forced_k = forced.ksplit, slot.forced_r = forced.ring, slot.forced_s = forced.wsplit;
            slot.tokens = a.tokens;
            slot.generation = generation;
        }
        cache = slot;
    }
    a.slot_bytes = (uint32_t)fmt_tile_bytes(cache.fmt);
    a.ksplit = cache.plan.ksplit;
    a.ring = cache.plan.ring;
    a.wsplit = (uint32_t)cache.plan.wsplit;
    ctx->dec_last_plan[0] = (uint32_t)cache.plan.warps, ctx->dec_last_plan[1] = (uint32_t)cache.plan.ksplit;
    ctx->dec_last_plan[2] = (uint32_t)cache.plan.wsplit, ctx->dec_last_plan[3] = (uint32_t)cache.plan.ring;
    a.max_tiles = (a.nsb + a.ksplit - 1) / a.ksplit + 1;
    uint32_t cta = 0, counter = 0;
    size_t partial = 0;
    for (uint32_t i = 0; i < a.n_jobs; ++i) {
        a.job[i].cta0 = cta;
        a.job[i].groups = cache.groups[i];
        a.job[i].counter0 = counter;
        a.job[i].partial0 = (uint32_t)partial;
        cta += cache.groups[i] * a.ksplit;
        counter += a.job[i].row_tiles;
        partial += (size_t)a.ksplit * (DUAL ? 2 : 1) * 4 * NG * a.job[i].n_out;
    }
    return launch_pdl(kquant_decode_kernel<NG, DUAL, FAM>, dim3(cta), dim3(cache.plan.warps * 32), cache.smem, stream, a);
}

} // namespace

// Up to four K-quant weights of one n_in (and one K shard geometry) applied to the same 1..16 tokens.
// w_up: the fused gate/up form (one job).  Returns cudaErrorNotSupported when the shape does not fit this kernel.
cudaError_t launch_kquant_decode(Ctx *ctx, const Weight *const *w, const Weight *w_up, uint32_t n_jobs, const void *x,
                                 uint32_t x_dtype, void *const *y, const uint32_t *y_dtype, uint32_t tokens,
                                 const Epilogue *ep, cudaStream_t stream, unsigned long long *amax_keys, unsigned int *amax_flags,
                                 const OneShotPush *push) {
    if (n_jobs == 0 || n_jobs > (uint32_t)kDecMaxJobs || tokens == 0 || tokens > 16 || w[0]->nsb > 4096) return cudaErrorNotSupported;
    DecArgs a;
    a.n_jobs = n_jobs;
    for (uint32_t i = 0; i < n_jobs; ++i) {
        if (w[i]->nsb != w[0]->nsb || w[i]->k_off != w[0]->k_off || w[i]->n_in != w[0]->n_in) return cudaErrorNotSupported;
        DecJob &j = a.job[i];
        j.image = w[i]->image;
        j.image_up = w_up ? w_up->image : nullptr;
        j.y = y[i];
        j.row_scale = ep[i].row_scale;
        j.residual = ep[i].residual;
        j.out_scale = ep[i].out_scale;
        j.softcap = ep[i].softcap;
        j.dtype = w[i]->dtype;
        j.n_out = (uint32_t)w[i]->n_out;
        j.row_tiles = w[i]->row_tiles;
        j.y_bf16 = y_dtype[i] == MUSER_DTYPE_BF16;
        j.cta0 = j.groups = j.counter0 = j.partial0 = 0;
        j.amax_keys = amax_keys, j.amax_flags = amax_flags;
    }
    for (uint32_t i = n_jobs; i < (uint32_t)kDecMaxJobs; ++i) a.job[i] = a.job[0];
    a.x = x;
    a.x_f32 = x_dtype == MUSER_DTYPE_F32;
    a.norm_weight = ep[0].norm_weight;
    a.norm_eps = ep[0].norm_eps;
    a.partial = ctx->gemv_partial;
    a.counters = ctx->gemv_counters;
    a.status = ctx->dev_status;
    a.n_in = (uint32_t)w[0]->n_in;
    a.nsb = w[0]->nsb;
    a.k_off = w[0]->k_off;
    a.tokens = tokens;
    a.ksplit = 1, a.max_tiles = 0, a.ring = 2, a.slot_bytes = kQ6TileBytes, a.wsplit = 1;
    a.push = OneShotPush{};
    const DecPlan forced{(int)ctx->dec_warps, (int)ctx->dec_ksplit, (int)ctx->dec_ring, (int)ctx->dec_wsplit};
    const uint32_t ng = (tokens + 3) / 4;
    uint32_t n_q5 = 0;
    for (uint32_t i = 0; i < n_jobs; ++i) n_q5 += w[i]->dtype == MUSER_DTYPE_Q5_K;
    if (n_q5 != 0 && (n_q5 != n_jobs || w_up)) return cudaErrorNotSupported; // Q5_K jobs run in launches of their own, unfused
    if (push) { // one row-parallel projection whose f32 partial sums go straight into the all-reduce's cells
        if (n_jobs != 1 || w_up || n_q5 || amax_keys || y_dtype[0] != MUSER_DTYPE_F32) return cudaErrorNotSupported;
        a.push = *push;
        switch (ng) {
        case 1: return dec_launch<1, false, 4>(a, ctx, forced, stream);
        case 2: return dec_launch<2, false, 4>(a, ctx, forced, stream);
        case 3: return dec_launch<3, false, 4>(a, ctx, forced, stream);
        default: return dec_launch<4, false, 4>(a, ctx, forced, stream);
        }
    }
    if (amax_keys) { // the LM head with the fused greedy pick: one projection
        if (n_jobs != 1 || w_up || !amax_flags) return cudaErrorNotSupported;
        if (n_q5) {
            switch (ng) {
            case 1: return dec_launch<1, false, 3>(a, ctx, forced, stream);
            case 2: return dec_launch<2, false, 3>(a, ctx, forced, stream);
            case 3: return dec_launch<3, false, 3>(a, ctx, forced, stream);
            default: return dec_launch<4, false, 3>(a, ctx, forced, stream);
            }
        }
        switch (ng) {
        case 1: return dec_launch<1, false, 2>(a, ctx, forced, stream);
        case 2: return dec_launch<2, false, 2>(a, ctx, forced, stream);
        case 3: return dec_launch<3, false, 2>(a, ctx, forced, stream);
        default: return dec_launch<4, false, 2>(a, ctx, forced, stream);
        }
    }
    if (n_q5) {
        switch (ng) {
        case 1: return dec_launch<1, false, 1>(a, ctx, forced, stream);
        case 2: return dec_launch<2, false, 1>(a, ctx, forced, stream);
        case 3: return dec_launch<3, false, 1>(a, ctx, forced, stream);
        default: return dec_launch<4, false, 1>(a, ctx, forced, stream);
        }
    }
    if (w_up) {
        if (n_jobs != 1) return cudaErrorNotSupported;
        switch (ng) {
        case 1: return dec_launch<1, true, 0>(a, ctx, forced, stream);
        case 2: return dec_launch<2, true, 0>(a, ctx, forced, stream);
        case 3: return dec_launch<3, true, 0>(a, ctx, forced, stream);
        default: return dec_launch<4, true, 0>(a, ctx, forced, stream);
        }
    }
    switch (ng) {
    case 1: return dec_launch<1, false, 0>(a, ctx, forced, stream);
    case 2: return dec_launch<2, false, 0>(a, ctx, forced, stream);
    case 3: return dec_launch<3, false, 0>(a, ctx, forced, stream);
    default: return dec_launch<4, false, 0>(a, ctx, forced, stream);
    }
}

// Keys -> (row index, value, non-finite flag) per token, and the keys go back to zero for the next call.
__global__ void lm_head_argmax_finalize_kernel(unsigned long long *keys, unsigned int *flags, uint32_t tokens, uint32_t *out_index,
                                               float *out_value, uint32_t *out_nonfinite) {
    pdl_wait();
    const uint32_t t = threadIdx.x;
    if (t >= tokens) return;
    const unsigned long long key = keys[t];
    const unsigned int flag = flags[t];
    keys[t] = 0ull, flags[t] = 0u;
    uint32_t u = (uint32_t)(key >> 32);
    u = (u & 0x80000000u) ? (u & 0x7FFFFFFFu) : ~u;
    // no candidate at all (every output NaN): the scalar scan never leaves index 0 (api.rs:1842-1850)
    out_index[t] = key ? 0xFFFFFFFFu - (uint32_t)key : 0u;
    if (out_value) out_value[t] = key ? __uint_as_float(u) : __uint_as_float(0x7FC00000u);
    if (out_nonfinite) out_nonfinite[t] = flag | (key ? 0u : 1u);
}

cudaError_t launch_lm_head_argmax(Ctx *ctx, const Weight *w, const void *x, uint32_t x_dtype, void *logits, uint32_t logits_dtype,
                                  uint32_t tokens, const Epilogue &ep, uint32_t *out_index, float *out_value, uint32_t *out_nonfinite,
                                  cudaStream_t stream) {
    void *ys[1] = {logits};
    uint32_t yd[1] = {logits_dtype};
    const cudaError_t e = launch_kquant_decode(ctx, &w, nullptr, 1, x, x_dtype, ys, yd, tokens, &ep, stream, ctx->amax_keys, ctx->amax_flags);
    if (e != cudaSuccess) return e;
    return launch_pdl(lm_head_argmax_finalize_kernel, dim3(1), dim3(32), 0, stream, ctx->amax_keys, ctx->amax_flags, tokens, out_index, out_value, out_nonfinite);
}

// ------------------------------------------------------------------------------------ measured plans
// Times the cost model's best candidates for this group of weights at 1, 2, 4, 8, 12 and 16 tokens and remembers the
// fastest per token count for this device.  Every candidate runs the way a decode step runs it: a CUDA graph of
// back-to-back launches (so each overlaps its predecessor's tail as in the step) that rotate over temporary copies of
// the weight images, together larger than L2, so that every launch streams its weights from HBM.  A measured plan
// replaces the model's choice only if it is at least 2 % faster.  Load-time work: allocates its scratch (the image
// copies, up to ~350 MB), synchronizes, frees it.
muser_cuda_status decode_autotune(Ctx *ctx, const Weight *const *w, const Weight *w_up, uint32_t n_jobs, uint32_t max_tokens, cudaStream_t stream) {
    constexpr int kCandidates = 24, kLaunches = 12, kReplays = 3;
    if (n_jobs == 0 || n_jobs > (uint32_t)kDecMaxJobs || (w_up && n_jobs != 1)) return fail(ctx, MUSER_CUDA_BAD_ARG, "a group holds 1..4 projections");
    max_tokens = std::min(std::max(max_tokens, 1u), 16u);
    size_t y_floats = 0, image_bytes = 0;
    for (uint32_t i = 0; i < n_jobs; ++i) {
        if (!w[i] || w[i]->device != ctx->device || (w[i]->dtype != MUSER_DTYPE_Q4_K && w[i]->dtype != MUSER_DTYPE_Q5_K && w[i]->dtype != MUSER_DTYPE_Q6_K))
            return fail(ctx, MUSER_CUDA_UNSUPPORTED_DTYPE, "autotune takes K-quant weights of this context's device");
        if (w[i]->n_in != w[0]->n_in || w[i]->nsb != w[0]->nsb || w[i]->k_off != w[0]->k_off)
            return fail(ctx, MUSER_CUDA_BAD_SHAPE, "the projections of a group must share n_in and the K shard geometry");
        y_floats += (size_t)16 * w[i]->n_out;
        image_bytes += w[i]->image_bytes;
    }
    if (w_up) {
        if (w_up->dtype != w[0]->dtype || w_up->n_in != w[0]->n_in || w_up->n_out != w[0]->n_out || w_up->nsb != w[0]->nsb)
            return fail(ctx, MUSER_CUDA_BAD_SHAPE, "gate and up geometry differ");
        image_bytes += w_up->image_bytes;
    }
    const int copies = (int)std::min<size_t>(12, std::max<size_t>(2, ((size_t)256 << 20) / image_bytes + 1));
    uint8_t *x = nullptr;
    float *y = nullptr;
    std::vector<uint8_t *> images;                 // copies x (jobs + up)
    std::vector<Weight> shadow((size_t)copies * (n_jobs + 1));
    cudaEvent_t ev[2] = {nullptr, nullptr};
    cudaStream_t side = nullptr;
    auto cleanup = [&]() {
        cudaFree(x), cudaFree(y);
        for (uint8_t *p : images) cudaFree(p);
        if (ev[0]) cudaEventDestroy(ev[0]);
        if (ev[1]) cudaEventDestroy(ev[1]);
        if (side) cudaStreamDestroy(side);
        ctx->dec_warps = ctx->dec_ksplit = ctx->dec_ring = ctx->dec_wsplit = 0;
    };
    cudaError_t e = cudaStreamSynchronize(stream);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&side, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMalloc(&x, (size_t)16 * w[0]->n_in * 2);
    if (e == cudaSuccess) e = cudaMemsetAsync(x, 0x3c, (size_t)16 * w[0]->n_in * 2, side); // bf16 0x3c3c: small positive values
    if (e == cudaSuccess) e = cudaMalloc(&y, y_floats * sizeof(float));
    if (e == cudaSuccess) e = cudaEventCreate(&ev[0]);
    if (e == cudaSuccess) e = cudaEventCreate(&ev[1]);
    for (int c = 0; c < copies && e == cudaSuccess; ++c)
        for (uint32_t i = 0; i <= n_jobs && e == cudaSuccess; ++i) {
            const Weight *src = i < n_jobs ? w[i] : w_up;
            if (!src) continue;
            uint8_t *p = nullptr;
            e = cudaMalloc(&p, src->image_bytes);
            if (e != cudaSuccess) break;
            images.push_back(p);
            e = cudaMemcpyAsync(p, src->image, src->image_bytes, cudaMemcpyDeviceToDevice, side);
            shadow[(size_t)c * (n_jobs + 1) + i] = *src;
            shadow[(size_t)c * (n_jobs + 1) + i].image = p;
        }
    if (e != cudaSuccess) {
        cleanup();
        return fail(ctx, MUSER_CUDA_ERROR, std::string("autotune scratch: ") + cudaGetErrorString(e));
    }
    void *ys[kDecMaxJobs];
    uint32_t yd[kDecMaxJobs];
    Epilogue eps[kDecMaxJobs];
    uint32_t total_tiles = 0;
    int fmt = 0;
    {
        float *yp = y;
        for (uint32_t i = 0; i < n_jobs; ++i) {
            ys[i] = yp, yd[i] = MUSER_DTYPE_F32;
            yp += (size_t)16 * w[i]->n_out;
            total_tiles += w[i]->row_tiles;
            if (w[i]->dtype == MUSER_DTYPE_Q6_K) fmt = 1;
            else if (w[i]->dtype == MUSER_DTYPE_Q5_K && fmt == 0) fmt = 2;
        }
    }
    auto launch_copy = [&](int c, uint32_t tokens) {
        const Weight *wc[kDecMaxJobs];
        for (uint32_t i = 0; i < n_jobs; ++i) wc[i] = &shadow[(size_t)c * (n_jobs + 1) + i];
        return launch_kquant_decode(ctx, wc, w_up ? &shadow[(size_t)c * (n_jobs + 1) + n_jobs] : nullptr, n_jobs, x, MUSER_DTYPE_BF16, ys, yd, tokens, eps, side);
    };
    static const uint32_t kTokenSteps[] = {1, 2, 4, 8, 12, 16};
    std::vector<DecCandidate> cands;
    muser_cuda_status st = MUSER_CUDA_OK;
    for (uint32_t tokens : kTokenSteps) {
        if (tokens > max_tokens && tokens != 1 && (tokens + 3) / 4 != (max_tokens + 3) / 4) continue;
        const int ng = (int)(tokens + 3) / 4;
        dec_candidates(w[0]->nsb, total_tiles, ctx->sm_count, ng, fmt, tokens, (w_up ? 2 : 1) * ng * 2, cands);
        const int n_c = std::min<int>(kCandidates, (int)cands.size());
        int best = 0;
        float best_ms = 1e30f, model_ms = 1e30f;
        for (int c = 0; c < n_c && st == MUSER_CUDA_OK; ++c) {
            ctx->dec_warps = cands[c].plan.warps, ctx->dec_ksplit = cands[c].plan.ksplit, ctx->dec_ring = cands[c].plan.ring, ctx->dec_wsplit = cands[c].plan.wsplit;
            cudaError_t le = launch_copy(0, tokens); // outside the capture: sets the kernel's attributes for this plan
            cudaGraph_t graph = nullptr;
            cudaGraphExec_t exec = nullptr;
            if (le == cudaSuccess) le = cudaStreamBeginCapture(side, cudaStreamCaptureModeThreadLocal);
            if (le == cudaSuccess) {
                for (int l = 0; l < kLaunches && le == cudaSuccess; ++l) le = launch_copy(l % copies, tokens);
                const cudaError_t ce = cudaStreamEndCapture(side, &graph);
                if (le == cudaSuccess) le = ce;
            }
            if (le == cudaSuccess) le = cudaGraphInstantiate(&exec, graph, 0);
            if (le == cudaSuccess) le = cudaGraphLaunch(exec, side); // warm
            if (le == cudaSuccess) le = cudaEventRecord(ev[0], side);
            for (int r = 0; r < kReplays && le == cudaSuccess; ++r) le = cudaGraphLaunch(exec, side);
            if (le == cudaSuccess) le = cudaEventRecord(ev[1], side);
            if (le == cudaSuccess) le = cudaStreamSynchronize(side);
            float ms = 1e30f;
            if (le == cudaSuccess) le = cudaEventElapsedTime(&ms, ev[0], ev[1]);
            if (exec) cudaGraphExecDestroy(exec);
            if (graph) cudaGraphDestroy(graph);
            if (le != cudaSuccess) {
                st = fail(ctx, MUSER_CUDA_ERROR, std::string("autotune measurement: ") + cudaGetErrorString(le));
                break;
            }
            if (c == 0) model_ms = ms;
            if (ms < best_ms) best_ms = ms, best = c;
        }
        if (st != MUSER_CUDA_OK) break;
        if (best_ms > 0.98f * model_ms) best = 0; // not clearly better than the model's own choice: keep that
        // remember it for this token count and for the counts below it that run the same token groups
        DecArgs key_args;
        key_args.nsb = w[0]->nsb, key_args.n_jobs = n_jobs;
        for (uint32_t i = 0; i < n_jobs; ++i) key_args.job[i].row_tiles = w[i]->row_tiles, key_args.job[i].dtype = w[i]->dtype;
        TunedTable &tt = tuned_table();
        std::lock_guard<std::mutex> tl(tt.mu);
        for (uint32_t t = tokens; t >= 1 && (t + 3) / 4 == (tokens + 3) / 4; --t) {
            if (t < tokens && (t == 1 || t == 2 || t == 4 || t == 8 || t == 12)) break; // tuned on its own
            key_args.tokens = t;
            tt.plans[ctx->device][tuned_key(key_args, w_up != nullptr)] = cands[best].plan;
        }
        ++tt.generation[ctx->device];
    }
    cleanup();
    return st;
}

// ------------------------------------------------------------------------------------ dispatch
// Which kernel serves a K-quant call (bf16 or f32 activations alike): up to 16 tokens the decode kernel above; from
// 17 tokens the tcgen05 kernel (kquant_tc.cu) when the weight has enough 128-row blocks to fill the GPU and the token
// count fits its columns (64, or 32 for f32 activations, which travel as f16 head + remainder pairs); everything else
// in chunks of 16 tokens through the decode kernel.  The thresholds can be moved through muser_cuda_tuning_set.
muser_cuda_status launch_kquant_matmul(Ctx *ctx, const Weight *w, const Weight *w_up, const void *x, uint32_t x_dtype,
                                       void *y, uint32_t y_dtype, uint32_t tokens, const Epilogue &ep,
                                       cudaStream_t stream) {
    const bool q6 = w->dtype == MUSER_DTYPE_Q6_K, xf32 = x_dtype == MUSER_DTYPE_F32;
    const uint32_t tc_from = ctx->tc_min_tokens[q6 ? 1 : 0]; // above 64: switched off
    const bool tc_fits = !w_up && w->dtype != MUSER_DTYPE_Q5_K && tokens >= tc_from && tokens <= (xf32 ? 32u : 64u) && w->n_out >= ctx->tc_min_rows;
    if (tc_fits) {
        const void *xin = x;
        uint32_t xin_dtype = x_dtype;
        if (ep.norm_weight) {
            // the tensor-core kernel reads its activations through TMA, so the fused input norm runs as a pass of its
            // own into the context's scratch rows (f32), which the projection then reads instead of x
            const size_t need = (size_t)tokens * w->n_in * sizeof(float);
            if (need > ctx->norm_scratch_bytes) return fail(ctx, MUSER_CUDA_WORKSPACE_TOO_SMALL, "fused input norm: tokens x n_in exceeds the context's norm scratch");
            muser_cuda_status st = launch_rmsnorm_rows(ctx, x, x_dtype, tokens, w->n_in, ep.norm_weight, ep.norm_eps, ctx->norm_scratch, stream);
            if (st != MUSER_CUDA_OK) return st;
            xin = ctx->norm_scratch;
            xin_dtype = MUSER_DTYPE_F32;
        }
        if (xin_dtype != MUSER_DTYPE_F32 || tokens <= 32) {
            Epilogue tail = ep;
            tail.norm_weight = nullptr;
            const cudaError_t te = launch_kquant_tc(ctx, w, xin, xin_dtype, y, y_dtype, tokens, tail, stream);
            if (te != cudaErrorNotSupported) {
                MUSER_CUDA_TRY(ctx, te);
                return MUSER_CUDA_OK;
            }
        }
    }
    if (ep.all_reduce) {
        // A row-parallel projection: y is one rank's partial sum.  Up to 16 tokens of f32 the decode kernel pushes
        // every value into all ranks' exchange cells as its row tile finishes, and a second, small kernel gathers
        // and adds them: the transfer runs beside the projection's remaining tiles.  Otherwise projection, then all-reduce.
        Epilogue plain = ep;
        plain.all_reduce = false;
        OneShotPush push;
        const uint64_t count = (uint64_t)tokens * w->n_out;
        if (!tc_fits && !w_up && tokens <= 16 && y_dtype == MUSER_DTYPE_F32 && w->dtype != MUSER_DTYPE_Q5_K && oneshot_push_target(ctx, count, &push)) {
            const cudaError_t de = launch_kquant_decode(ctx, &w, nullptr, 1, x, x_dtype, &y, &y_dtype, tokens, &plain, stream, nullptr, nullptr, &push);
            if (de == cudaErrorNotSupported) return fail(ctx, MUSER_CUDA_BAD_SHAPE, "this shape does not fit the decode kernel");
            MUSER_CUDA_TRY(ctx, de);
            MUSER_CUDA_TRY(ctx, launch_oneshot_gather(ctx, reinterpret_cast<float *>(y), count, stream));
            return MUSER_CUDA_OK;
        }
        const muser_cuda_status st = launch_kquant_matmul(ctx, w, w_up, x, x_dtype, y, y_dtype, tokens, plain, stream);
        if (st != MUSER_CUDA_OK) return st;
        return muser_cuda_all_reduce(reinterpret_cast<muser_cuda_ctx *>(ctx), y, count, y_dtype, stream);
    }
    const size_t xb = xf32 ? 4 : 2, yb = y_dtype == MUSER_DTYPE_BF16 ? 2 : 4;
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

} // namespace muser
