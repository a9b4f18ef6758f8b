// Skinny GEMM for Q4_K / Q6_K weights on the 5th-generation tensor cores: y[t][r] = dot(W_r, x_t), 3..64 tokens.
//
// Stands in for the batched routes of MetalKernels::encode_quantized_matmul and the speculative-verify batches of
// encode_quantized_decode_group (crates/muser-engine/src/metal/encode/qkv.rs:234-281,414-449); on the CPU lane,
// weights::matmul with quant::dot_q4_k_f32 / dot_q6_k_f32 (src/weights.rs:398-421).
//
// The weights stay in their 4.5 / 6.56-bit form in HBM and are read once, whatever the token count.  What goes to
// the tensor cores is exact: the f16 operand built from a Q4_K weight is the INTEGER sc * q (6-bit scale times
// 4-bit quant, at most 945), from a Q6_K weight sc * (q - 32) (at most 4096 in magnitude; f16 holds every such
// product exactly up to 2048 and the even ones beyond), and the activations are the caller's bf16 values as f16.
// The per-super-block factors d and dmin, which differ per row and per 256 inputs, cannot ride in the operands, so
// the accumulator is drained once per 256 inputs: acc += d * sum(sc q x) - dmin * sum_j m_j X_j, with the second
// sum (X_j = sum of the 32 activations of sub-block j, carried as an f16 head + remainder pair) done by one more
// MMA.  This is the deferred order of quant/k_block.rs:178-240 and quant/k_block/q6.rs:90-141 with exact inner sums.
//
// One CTA per SM, persistent over (128-row block, K slice) items; every role walks the same (item, column) sequence:
//   warp 0      TMA: activation slabs (N tokens x 128 inputs, 128-byte swizzle) and the X_j pairs (32-byte swizzle)
//   warp 1 and the last warp
//               tcgen05.mma kind::f16, M = 128 rows, N = tokens (16 / 32 / 64), K = 16, the A operand read from
//               tensor memory; one warp takes the even columns of the sequence, the other the odd ones
//   warps 2-17  one weight row per thread: (column parity, half of the column, 32-row quarter) per warp; the row's
//               bytes come straight from global memory, become the f16 integers above and go to tensor memory
//               (tcgen05.st), 64 inputs = one A stage at a time (eight stages = two columns)
//   then 4 or 8 drain warps (eight from 32 token columns on, half the columns each, so that the running sums stay in
//               registers): tcgen05.ld, scale by d / dmin (f32), keep the running sums per row in registers; at the
//               end of an item add the K slices through the context scratch (last arriver sums in slice order) and
//               store
// The producer and MMA warps run their loops converged and issue through an elected lane (tcgen05.cuh).
// Every wait is bounded; a wait that gives up records a code in the context's status word and the CTA winds down.
#include <algorithm>
#include <cmath>
#include <type_traits>

#include "common.cuh"
#include "kquant_layout.cuh"
#include "tcgen05.cuh"

namespace muser {

// Development aid, compiled in only with -DMUSER_GEMM_WAIT_PROFILE: some roles of the first CTAs add up the SM cycles
// they spend in each kind of wait, and a debug entry point copies the sums out.
#ifdef MUSER_GEMM_WAIT_PROFILE
__device__ unsigned long long g_tc_wait_prof[4 * 8 * 4]; // [cta < 4][role < 8][slot < 4]
#define TPROF_DECL long long prof_t0 = 0, prof_start = clock64(); unsigned long long prof_acc[3] = {0, 0, 0};
#define TPROF_BEGIN prof_t0 = clock64();
#define TPROF_END(i) prof_acc[i] += (unsigned long long)(clock64() - prof_t0);
#define TPROF_FLUSH(role)                                                                                 \
    if (blockIdx.x < 4) {                                                                                 \
        for (int i_ = 0; i_ < 3; ++i_) g_tc_wait_prof[(blockIdx.x * 8 + (role)) * 4 + i_] = prof_acc[i_]; \
        g_tc_wait_prof[(blockIdx.x * 8 + (role)) * 4 + 3] = (unsigned long long)(clock64() - prof_start); \
    }
__device__ unsigned long long g_tc_stamps[8]; // ns: prepare first start, last end; GEMM first entry, CTA 0 set up, last loop end, last exit
__device__ __forceinline__ unsigned long long tprof_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define TPROF_STAMP_MIN(i) atomicMin(&g_tc_stamps[i], tprof_ns());
#define TPROF_STAMP_MAX(i) atomicMax(&g_tc_stamps[i], tprof_ns());
#else
#define TPROF_STAMP_MIN(i)
#define TPROF_STAMP_MAX(i)
#define TPROF_DECL
#define TPROF_BEGIN
#define TPROF_END(i)
#define TPROF_FLUSH(role)
#endif

constexpr int kTcRows = 128;             // weight rows per block = MMA M
constexpr int kTcStagesA = 8;            // A stages in tensor memory: the four 64-input quarters of two super-block columns
constexpr int kTcStageCols = 32;         // 64 inputs as f16 pairs
constexpr int kTcDequantWarps = 16;      // warp = (column parity, half of the column, 32-row quarter of the block)

struct TcArgs {
    const uint8_t *image;
    void *y;
    const float *row_scale;
    float out_scale, softcap; // LM-head tail
    const void *residual;
    float *partial;         // [ksplit][tokens][n_out] partial sums (ksplit > 1)
    unsigned int *counters; // [row_blocks * 8] arrival counters (row quarter x column half), zero between launches
    int *status;
    uint32_t n_out, nsb, row_tiles, tokens, y_bf16;
    uint32_t fold;          // f32 activations travel as f16 head + remainder in columns 2t and 2t + 1: add the pairs
    uint32_t whole, ksplit, items; // items 0..whole-1: one row block each, all of K; then the other row blocks in ksplit slices
};

// The (item, super-block column) sequence of one CTA; every role walks the same sequence.
struct TcWalk {
    uint32_t item, rb, slice, k, k_begin, len, idx;
    bool split;
    __device__ __forceinline__ void load(const TcArgs &a) {
        if (item >= a.items) return;
        uint32_t k_end;
        if (item < a.whole) {
            rb = item, slice = 0, k_begin = 0, k_end = a.nsb, split = false;
        } else {
            const uint32_t j = item - a.whole;
            rb = a.whole + j / a.ksplit;
            slice = j % a.ksplit;
            k_begin = a.nsb * slice / a.ksplit;
            k_end = a.nsb * (slice + 1) / a.ksplit;
            split = a.ksplit > 1;
        }
        // CTAs that work on the same columns at the same time would all ask L2 for the same activation lines: each
        // starts its sweep at another column (the order of the f32 sums differs per row block, but is fixed)
        len = k_end - k_begin;
        idx = 0;
        k = k_begin + blockIdx.x % len;
    }
    __device__ __forceinline__ void start(const TcArgs &a) {
        item = blockIdx.x;
        load(a);
    }
    __device__ __forceinline__ bool done(const TcArgs &a) const { return item >= a.items; }
    __device__ __forceinline__ bool last_column() const { return idx + 1 == len; }
    __device__ __forceinline__ void next(const TcArgs &a) {
        if (++idx == len) {
            item += gridDim.x;
            load(a);
        } else if (++k == k_begin + len) {
            k = k_begin;
        }
    }
};

__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The same with the A operand in tensor memory: lane = row, eight 32-bit columns = 16 f16 along K.
__device__ __forceinline__ void mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Issued by the elected lane of a converged warp (tcgen05.cuh).
__device__ __forceinline__ void mma_f16_elect(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t" MUSER_ELECT_PRED
        "setp.ne.b32 p, %4, 0;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_f16_ts_elect(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t" MUSER_ELECT_PRED
        "setp.ne.b32 p, %4, 0;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// K-major operand, 32 bytes (16 f16) per row, 32-byte swizzle, 8-row groups 256 bytes apart.
__device__ __forceinline__ uint64_t operand_desc32(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(256 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)6 << 61; // SWIZZLE_32B
    return d;
}
__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(addr));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint32_t h2u(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 u2h(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }
__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i) { return (&v.x)[i]; } // compile-time i only

// (byte `idx` of w) as an exact f16 pair (v, v): 0x6400 | v is 1024 + v
__device__ __forceinline__ __half2 byte_pair(uint32_t w, uint32_t idx, float bias) {
    const uint32_t m = __byte_perm(w, 0x64646464u, 0x4040u | idx | (idx << 8));
    return __hsub2(u2h(m), __float2half2_rn(bias));
}

// ------------------------------------------------------------------------------------ weights -> A operand
// The A operand lives in TENSOR memory, not in shared memory: TMEM lane = weight row of the 128-row block, and a
// 32-bit column of a lane holds two consecutive inputs as f16 (tcgen05.mma with A from tensor memory reads K = 16 from
// eight columns).  An unpacking thread therefore owns one ROW: it reads that row's bytes of a weight tile straight
// from global memory (streaming loads; its warp's 32 rows make whole 512-byte runs), turns them into the f16 integers
// and writes 32 columns (64 inputs = one A stage) with one tcgen05.st.  Shared memory carries only the activations:
// with the operand in shared memory the stage stores, the MMA's reads of them and the raw-tile rings together asked
// the SM's shared-memory pipe for ~200 KB per super-block column, which is what bounded that kernel.
__device__ __forceinline__ uint4 ldg_stream128(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_stream64(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ void tmem_st16(uint32_t addr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ------------------------------------------------------------------------------------ Q4_K
// One row's 128 inputs of one half of a super-block (kquant_layout.cuh: uint4 (2 * rowsel + half, lane = 4 g + t),
// word jj = sub-block 4 * half + jj, elements 8t .. 8t + 7) and the row's header.
struct TcQ4 {
    uint4 c[4]; // [t]
    uint4 h;
};
struct TcQ4Hdr {
    float d, dmin;
    uint32_t sc[2], mn[2]; // 6-bit values as bytes: sub-blocks 0-3, 4-7 (quant/k_block.rs:22-31)
};
__device__ __forceinline__ TcQ4Hdr tc_q4_hdr(uint4 h) {
    TcQ4Hdr s;
    const __half2 dd = *reinterpret_cast<const __half2 *>(&h.x);
    s.d = __low2float(dd);
    s.dmin = __high2float(dd);
    s.sc[0] = h.y & 0x3F3F3F3Fu;
    s.mn[0] = h.z & 0x3F3F3F3Fu;
    s.sc[1] = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
    s.mn[1] = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
    return s;
}
// `tile`: the 16-row tile of this thread's row; r16: the row inside it.
__device__ __forceinline__ TcQ4 tc_fetch(const uint8_t *tile, uint32_t half, uint32_t r16, TcQ4 *) {
    TcQ4 r;
    const uint8_t *p = tile + (2 * (r16 >> 3) + half) * 512 + (r16 & 7) * 64;
#pragma unroll
    for (int t = 0; t < 4; ++t) r.c[t] = ldg_stream128(p + 16 * t);
    r.h = ldg_stream128(tile + 2048 + r16 * 16);
    return r;
}
// Sub-block JJ of the half (32 inputs) -> 16 columns, sc * q as exact f16 integers.
// (word >> 4p) & 0x000F000F is the pair of elements (2p, 2p + 1); the nibbles at bits 4-7 / 20-23 are not shifted
// down: 0x6400 | (q << 4) is 1024 + 16 q, and the fused multiply-add with sc / 16 and -64 sc gives sc * q just as
// exactly (one rounding, of an integer below 2048).
template <int JJ>
__device__ __forceinline__ void tc_unpack(const TcQ4 &r, uint32_t scw, uint32_t (&o)[16]) {
    const __half2 sc = byte_pair(scw, (uint32_t)JJ, 1024.0f);
    const __half2 off = __hmul2(sc, __float2half2_rn(-1024.0f)); // exact: at most 63 * 1024
    const __half2 sc16 = __hmul2(sc, __float2half2_rn(0.0625f)), off16 = __hmul2(sc, __float2half2_rn(-64.0f));
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        const uint32_t w = word_of(r.c[t], JJ), w8 = w >> 8;
        o[4 * t + 0] = h2u(__hfma2(u2h((w & 0x000F000Fu) | 0x64006400u), sc, off));
        o[4 * t + 1] = h2u(__hfma2(u2h((w & 0x00F000F0u) | 0x64006400u), sc16, off16));
        o[4 * t + 2] = h2u(__hfma2(u2h((w8 & 0x000F000Fu) | 0x64006400u), sc, off));
        o[4 * t + 3] = h2u(__hfma2(u2h((w8 & 0x00F000F0u) | 0x64006400u), sc16, off16));
    }
}

// ------------------------------------------------------------------------------------ Q6_K
// One row's 128 inputs of one half: the top-nibble plane (uint4 per t: word wi covers sub-blocks 8 * half + 2 wi and
// + 1 in its low / high nibbles, byte b = element 4t + b), the two words of the low-two-bits plane that belong to the
// half (word v covers sub-blocks 4v .. 4v + 3, two bits each), the half's eight int8 scales, and d.
struct TcQ6 {
    uint4 lo[4]; // [t]
    uint2 hi[4]; // [t]
    uint2 sc;
    float d;
};
__device__ __forceinline__ TcQ6 tc_fetch(const uint8_t *tile, uint32_t half, uint32_t r16, TcQ6 *) {
    TcQ6 r;
    const uint32_t rowsel = r16 >> 3, g = r16 & 7;
    const uint8_t *p = tile + (2 * rowsel + half) * 512 + g * 64, *ph = tile + kQ6OffHi + rowsel * 512 + g * 64 + 8 * half;
#pragma unroll
    for (int t = 0; t < 4; ++t) r.lo[t] = ldg_stream128(p + 16 * t);
#pragma unroll
    for (int t = 0; t < 4; ++t) r.hi[t] = ldg_stream64(ph + 16 * t);
    r.sc = ldg_stream64(tile + kQ6OffSc + r16 * 16 + 8 * half);
    r.d = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short *>(tile + kQ6OffD) + r16)));
    return r;
}
// Sub-blocks 2 JJ, 2 JJ + 1 of the half (16 inputs each; JJ = 0..3) -> 16 columns of sc * (q - 32).
// (T << 4) | (L << 2) is the signed byte 4 (q - 32); with its sign bit flipped, b = 4 (q - 32) + 128, and one fused
// multiply-add gives (1024 + b) * (sc / 4) - 288 sc = sc (q - 32): every input is exact in f16 (288 |sc| <= 36864 =
// 2^5 * 9 |sc|), the result is rounded once (to even beyond 2048, as f16 must).
template <int JJ>
__device__ __forceinline__ void tc_unpack(const TcQ6 &r, uint32_t (&o)[16]) {
    const uint32_t scw = ((JJ >> 1) ? r.sc.y : r.sc.x) ^ 0x80808080u; // int8 scales + 128
#pragma unroll
    for (int ci = 0; ci < 2; ++ci) {
        const int c = 2 * (JJ & 1) + ci; // sub-block 4 (JJ / 2) + c of the half
        const __half2 sc = byte_pair(scw, (uint32_t)c, 1152.0f); // exact
        const __half2 sc4 = __hmul2(sc, __float2half2_rn(0.25f)), off = __hmul2(sc, __float2half2_rn(-288.0f));
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const uint32_t tw = word_of(r.lo[t], JJ), lw = (JJ >> 1) ? r.hi[t].y : r.hi[t].x;
            // even sub-blocks sit in the low nibbles of the plane's bytes, odd ones in the high nibbles
            const uint32_t top = (c & 1) ? ((tw ^ 0x80808080u) & 0xF0F0F0F0u) : (((tw ^ 0x08080808u) & 0x0F0F0F0Fu) << 4);
            const uint32_t low = c == 0 ? lw << 2 : c == 1 ? lw : c == 2 ? lw >> 2 : lw >> 4;
            const uint32_t b = top | (low & 0x0C0C0C0Cu);
            o[8 * ci + 2 * t + 0] = h2u(__hfma2(u2h(__byte_perm(b, 0x64646464u, 0x4140u)), sc4, off));
            o[8 * ci + 2 * t + 1] = h2u(__hfma2(u2h(__byte_perm(b, 0x64646464u, 0x4342u)), sc4, off));
        }
    }
}

// ------------------------------------------------------------------------------------ kernel
template <int DT, int N>
struct TcSmem {
    static constexpr bool kQ4 = DT == MUSER_DTYPE_Q4_K;
    static constexpr int kTile = kQ4 ? kQ4TileBytes : kQ6TileBytes;
    static constexpr int kStagesB = 4;               // activation slabs (128 inputs each) come from L2 with ~1500 cycles of latency
    static constexpr int kBBytes = N * 256;          // two atoms of N rows x 128 bytes
    static constexpr int kMinA = kTcRows * 32, kMinB = N * 32 < 1024 ? 1024 : N * 32;
    static constexpr int kOffB = 0;
    static constexpr int kOffMinA = kOffB + kStagesB * kBBytes;
    static constexpr int kOffMinB = kOffMinA + 2 * kMinA;
    static constexpr int kOffHdr = kOffMinB + 2 * kMinB;
    static constexpr int kHdrDepth = 8;              // (d, dmin) per row of the last eight super-block columns
    static constexpr int kOffBars = kOffHdr + kHdrDepth * kTcRows * 8;
    // Tensor memory: kBufs accumulator buffers (kAcc main parts + the min part each), then the A stages.
    // An MMA warp cannot start a column before the drain warps have read that buffer's previous column, so buffers
    // are worth more than a second main accumulator per buffer (back-to-back MMAs into one accumulator run at the
    // same 46 cycles as alternating ones): four buffers up to 32 columns, two at 64.
    static constexpr int kAcc = N == 16 ? 2 : 1;
    static constexpr int kBufCols = (kAcc + 1) * N;
    static constexpr int kBufs = N <= 32 ? 4 : 2;
    static constexpr uint32_t kACol = kBufs * kBufCols, kTmemCols = 512;
    static_assert(kACol + kTcStagesA * kTcStageCols <= kTmemCols, "tensor memory exceeded");
    static constexpr int kDrainWarps = N >= 32 ? 8 : 4, kDrainCols = N / (kDrainWarps / 4);
    static constexpr int kMmaWarp1 = 2 + kTcDequantWarps + kDrainWarps; // the second MMA warp comes last, so that the others keep their lane quarters
    static constexpr int kThreads = 32 * (2 + kTcDequantWarps + kDrainWarps + 1);
    static constexpr int kBars = 2 * kTcStagesA + 2 * kStagesB + 2 * kBufs;
    static constexpr int kBytes = kOffBars + kBars * 8 + 16 + 1024 /*alignment slack*/;
    static_assert(kBytes <= 227 * 1024, "shared memory of one CTA exceeded");
};

template <int DT, int N>
__global__ void __launch_bounds__((TcSmem<DT, N>::kThreads), 1)
kquant_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_xs, const TcArgs a) {
    using S = TcSmem<DT, N>;
    constexpr bool Q4 = S::kQ4;
    if (threadIdx.x == 0) { TPROF_STAMP_MIN(2) }
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *aligned = smem_raw + (base - smem_u32(smem_raw));
    uint64_t *bars = reinterpret_cast<uint64_t *>(aligned + S::kOffBars);
    constexpr int kStagesB = S::kStagesB, kStagesA = kTcStagesA;
    const uint32_t bar_full_a = smem_u32(bars), bar_empty_a = bar_full_a + 8 * kStagesA;
    const uint32_t bar_full_b = bar_empty_a + 8 * kStagesA, bar_empty_b = bar_full_b + 8 * kStagesB;
    constexpr int kBufs = S::kBufs;
    const uint32_t bar_tmem_full = bar_empty_b + 8 * kStagesB, bar_tmem_empty = bar_tmem_full + 8 * kBufs;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + S::kBars);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    float2 *hdr = reinterpret_cast<float2 *>(aligned + S::kOffHdr);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStagesA; ++s) {
            mbar_init(bar_full_a + 8 * s, 4); // the four 32-row quarters of the stage
            mbar_init(bar_empty_a + 8 * s, 1);
        }
        for (int s = 0; s < kStagesB; ++s) {
            mbar_init(bar_full_b + 8 * s, 1);
            mbar_init(bar_empty_b + 8 * s, 1);
        }
        for (int b = 0; b < kBufs; ++b) {
            mbar_init(bar_tmem_full + 8 * b, 1);
            mbar_init(bar_tmem_empty + 8 * b, S::kDrainWarps);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(S::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    if (threadIdx.x == 0 && blockIdx.x == 0) { TPROF_STAMP_MAX(3) }

    if (warp == 0) {
        // ---------------------------------------------------------------- activation producer (whole warp, one lane issues)
        {
            TcWalk w;
            w.start(a);
            uint32_t hs = 0, tc = 0, issued = 0;
            bool ok = true; TPROF_DECL
            pdl_wait(); // the activations come from the kernel before this one; everything up to here overlapped its tail
            for (; !w.done(a) && ok; w.next(a), ++tc) {
                for (uint32_t h = 0; h < 2; ++h, ++hs) {
                    const uint32_t s = hs % kStagesB, round = hs / kStagesB;
                    TPROF_BEGIN if (round > 0) ok = __all_sync(0xffffffffu, mbar_wait_relaxed(bar_empty_b + 8 * s, (round - 1) & 1, abort_flag, 32)); TPROF_END(0)
                    if (!ok) break;
                    const uint32_t full = bar_full_b + 8 * s, dst = base + S::kOffB + s * S::kBBytes;
                    const bool with_sums = Q4 && h == 1;
                    mbar_expect_tx_elect(full, S::kBBytes + (with_sums ? N * 32 : 0));
                    const int x0 = (int)((w.k * 256 + h * 128) * 2);
                    tma_load_2d_elect(dst, &map_x, x0, 0, full);
                    tma_load_2d_elect(dst + N * 128, &map_x, x0 + 128, 0, full);
                    if (with_sums) tma_load_2d_elect(base + S::kOffMinB + (tc & 1) * S::kMinB, &map_xs, (int)(w.k * 32), 0, full);
                    issued = hs + 1;
                }
            }
            if (lane == 0) { TPROF_FLUSH(0) }
            if (!ok) {
                if (lane == 0) {
                    *abort_flag = 1;
                    atomicExch(a.status + 1, 301);
                }
                // let the copies already in flight land before the CTA's shared memory goes away
                const uint32_t first = issued > (uint32_t)kStagesB ? issued - kStagesB : 0;
                for (uint32_t k = first; k < issued; ++k) mbar_wait_alone(bar_full_b + 8 * (k % kStagesB), (k / kStagesB) & 1);
            }
        }
    } else if (warp == 1 || warp == S::kMmaWarp1) {
        // ---------------------------------------------------------------- MMA issuers (whole warps, one lane issues)
        // Two warps, one for the even and one for the odd super-block columns of the CTA's sequence (their A stages,
        // activation slabs and accumulator buffers are disjoint by parity): issuing a column's 17 MMAs and 7 commits
        // takes one warp longer than the tensor pipe needs to run them.
        {
            const uint32_t par = warp == 1 ? 0u : 1u;
            // kind::f16: f32 accumulator (bit 4), A and B f16 (format 0), both K-major, N >> 3 at bit 17, M >> 4 at bit 24
            const uint32_t idesc = (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(kTcRows >> 4) << 24);
            TcWalk w;
            w.start(a);
            if (par && !w.done(a)) w.next(a);
            uint32_t tc = par;
            bool ok = true; TPROF_DECL
            auto advance2 = [&]() {
                w.next(a);
                if (!w.done(a)) w.next(a);
            };
            for (; !w.done(a) && ok; advance2(), tc += 2) {
                uint32_t hs = 2 * tc; // the column's two activation slabs
                const uint32_t buf = tc % kBufs, d_main = tmem + buf * S::kBufCols, d_min = d_main + S::kAcc * N;
                if (tc >= (uint32_t)kBufs) { // the drain warps must have read this buffer's previous contents
                    TPROF_BEGIN ok = mbar_wait_warp(bar_tmem_empty + 8 * buf, ((tc / kBufs) - 1) & 1, abort_flag); TPROF_END(0)
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                }
                const uint32_t a_col = tmem + S::kACol + (tc & 1) * 4 * kTcStageCols; // this column's four stages
                for (uint32_t h = 0; h < 2 && ok; ++h, ++hs) {
                    const uint32_t s_b = hs % kStagesB, round_b = hs / kStagesB;
                    TPROF_BEGIN ok = mbar_wait_warp(bar_full_b + 8 * s_b, round_b & 1, abort_flag); TPROF_END(1)
                    if (!ok) break;
                    const uint32_t sb = base + S::kOffB + s_b * S::kBBytes;
#pragma unroll
                    for (uint32_t atom = 0; atom < 2; ++atom) { // one A stage = 64 inputs = one atom of the activation slab
                        const uint32_t s = (tc & 1) * 4 + 2 * h + atom;
                        TPROF_BEGIN ok = mbar_wait_warp(bar_full_a + 8 * s, (tc >> 1) & 1, abort_flag); TPROF_END(1)
                        if (!ok) break;
                        TPROF_BEGIN
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t ta = a_col + (2 * h + atom) * kTcStageCols;
                        const uint64_t db = operand_desc(sb + atom * (N * 128u));
#pragma unroll
                        for (uint32_t kk = 0; kk < 4; ++kk) // 16 inputs: 8 columns of A, 32 bytes along B's swizzled 128-byte rows
                            mma_f16_ts_elect(d_main + (S::kAcc == 2 ? (kk & 1) * N : 0), ta + 8 * kk, db + 2 * kk, idesc,
                                             (h | atom | (S::kAcc == 2 ? kk >> 1 : kk)) != 0);
                        if (Q4 && h == 1 && atom == 1)
                            mma_f16_elect(d_min, operand_desc32(base + S::kOffMinA + (tc & 1) * S::kMinA),
                                          operand_desc32(base + S::kOffMinB + (tc & 1) * S::kMinB), idesc, 0);
                        mma_commit_elect(bar_empty_a + 8 * s); // the stage (and the min operand) reusable once these MMAs have read it
                        TPROF_END(2)
                    }
                    if (ok) mma_commit_elect(bar_empty_b + 8 * s_b);
                }
                if (ok) mma_commit_elect(bar_tmem_full + 8 * buf);
            }
            if (lane == 0 && warp == 1) { TPROF_FLUSH(1) }
            if (!ok && lane == 0) {
                *abort_flag = 1;
                atomicExch(a.status + 1, 302);
            }
        }
    } else if (warp < 2 + kTcDequantWarps) {
        // ---------------------------------------------------------------- weight unpackers
        // Warp = (column parity p, half of the column, 32-row quarter): thread = one weight row, every other
        // super-block column, 128 inputs of it = two A stages.  The row's bytes of the NEXT own column are requested
        // before this one is unpacked (about two column times of latency hidden; ~40 KB in flight per SM).
        using Regs = typename std::conditional<Q4, TcQ4, TcQ6>::type;
        const uint32_t kg = (uint32_t)(warp - 2) >> 2, p = kg >> 1, half = kg & 1, qd = (uint32_t)warp & 3; // (tensor-memory lanes 32 qd ..)
        const uint32_t row = qd * 32 + lane, r16 = (uint32_t)lane & 15;
        const uint32_t st_base = tmem + ((qd * 32) << 16) + S::kACol + (p * 4 + half * 2) * kTcStageCols;
        auto fetch = [&](const TcWalk &x) {
            const uint32_t rt = min(x.rb * (kTcRows / kTileRows) + 2 * qd + ((uint32_t)lane >> 4), a.row_tiles - 1); // a short last block repeats its last tile
            return tc_fetch(a.image + ((uint64_t)rt * a.nsb + x.k) * S::kTile, half, r16, (Regs *)nullptr);
        };
        auto advance2 = [&](TcWalk &x) {
            x.next(a);
            if (!x.done(a)) x.next(a);
        };
        TcWalk f;
        f.start(a);
        if (p && !f.done(a)) f.next(a);
        bool have = !f.done(a), ok = true; TPROF_DECL
        Regs nxt{};
        if (have) {
            nxt = fetch(f);
            advance2(f);
        }
        for (uint32_t n = p, own = 0; have && ok; n += 2, ++own) { // n: the column's number in this CTA's sequence
            const Regs cur = nxt;
            have = !f.done(a);
            if (have) {
                nxt = fetch(f);
                advance2(f);
            }
            TcQ4Hdr hd{};
            if constexpr (Q4) hd = tc_q4_hdr(cur.h);
            auto quarter_step = [&](auto quarter_tag) {
                constexpr int QD = decltype(quarter_tag)::value;
                const uint32_t s = p * 4 + half * 2 + QD;
                TPROF_BEGIN if (own > 0) ok = mbar_wait(bar_empty_a + 8 * s, (own - 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok); TPROF_END(1)
                if (!ok) return;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                TPROF_BEGIN
#pragma unroll
                for (int j = 0; j < 2; ++j) { // 16 columns at a time keeps the live registers down
                    uint32_t o[16];
                    if (j == 0) {
                        if constexpr (Q4) tc_unpack<2 * QD>(cur, half ? hd.sc[1] : hd.sc[0], o);
                        else tc_unpack<2 * QD>(cur, o);
                    } else {
                        if constexpr (Q4) tc_unpack<2 * QD + 1>(cur, half ? hd.sc[1] : hd.sc[0], o);
                        else tc_unpack<2 * QD + 1>(cur, o);
                    }
                    tmem_st16(st_base + QD * kTcStageCols + 16 * j, o);
                }
                TPROF_END(0)
                TPROF_BEGIN
                if (QD == 1 && half == 1) {
                    if constexpr (Q4) {
                        // min operand (shared memory): 16 f16 per row, (m_j, m_j) for j = 0..7, two 16-byte chunks, 32-byte swizzle.
                        // Its two buffers go by column parity: the wait above covered the min MMA of this parity's last column.
                        const uint32_t mrow = base + S::kOffMinA + (n & 1) * S::kMinA + (row >> 3) * 256u + (row & 7) * 32u, sw = (row >> 2) & 1;
                        sts128(mrow + (0u ^ sw) * 16u, h2u(byte_pair(hd.mn[0], 0, 1024.0f)), h2u(byte_pair(hd.mn[0], 1, 1024.0f)),
                               h2u(byte_pair(hd.mn[0], 2, 1024.0f)), h2u(byte_pair(hd.mn[0], 3, 1024.0f)));
                        sts128(mrow + (1u ^ sw) * 16u, h2u(byte_pair(hd.mn[1], 0, 1024.0f)), h2u(byte_pair(hd.mn[1], 1, 1024.0f)),
                               h2u(byte_pair(hd.mn[1], 2, 1024.0f)), h2u(byte_pair(hd.mn[1], 3, 1024.0f)));
                        hdr[(n % S::kHdrDepth) * kTcRows + row] = make_float2(hd.d, hd.dmin);
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // generic stores -> visible to the MMA's reads
                    } else {
                        hdr[(n % S::kHdrDepth) * kTcRows + row] = make_float2(cur.d, 0.0f);
                    }
                }
                tmem_st_wait();
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_full_a + 8 * s);
                TPROF_END(2)
            };
            quarter_step(std::integral_constant<int, 0>{});
            if (ok) quarter_step(std::integral_constant<int, 1>{});
        }
        if (lane == 0 && (warp == 2 || warp == 17)) { TPROF_FLUSH(warp == 2 ? 2 : 3) }
        if (!ok && lane == 0) {
            *abort_flag = 1;
            atomicCAS(a.status + 1, 0, 303);
        }
    } else if (warp < S::kMmaWarp1) {
        // ---------------------------------------------------------------- drain (4 or 8 warps)
        constexpr int C = S::kDrainCols;                                          // token columns of this warp
        const uint32_t quad = warp & 3, row_in_block = quad * 32 + lane;          // its 32 accumulator lanes = rows
        const uint32_t part = (uint32_t)(warp - 2 - kTcDequantWarps) >> 2, col0 = part * C;
        // f32 activations occupy column pairs (2t, 2t + 1): after folding, this warp holds tokens col0/2 .. col0/2 + C/2 - 1
        const uint32_t tok0 = a.fold ? col0 / 2 : col0, n_tok = a.fold ? C / 2 : C;
        float acc[C];
#pragma unroll
        for (int i = 0; i < C; ++i) acc[i] = 0.0f;
        TcWalk w;
        w.start(a);
        uint32_t tc = 0; TPROF_DECL
        while (!w.done(a)) {
            const uint32_t buf = tc % kBufs;
            TPROF_BEGIN const bool ok = __all_sync(0xffffffffu, mbar_wait_relaxed(bar_tmem_full + 8 * buf, (tc / kBufs) & 1, abort_flag, 40)); TPROF_END(0)
            if (!ok) {
                if (lane == 0) {
                    *abort_flag = 1;
                    atomicCAS(a.status + 1, 0, 304);
                }
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float2 hd = hdr[(tc % S::kHdrDepth) * kTcRows + row_in_block];
            const uint32_t taddr = tmem + ((quad * 32) << 16) + buf * S::kBufCols + col0;
#pragma unroll
            for (int c0 = 0; c0 < C; c0 += 16) {
                uint32_t p[16], p2[S::kAcc == 2 ? 16 : 1], m[16];
                tmem_ld16(taddr + c0, p);
                if constexpr (S::kAcc == 2) tmem_ld16(taddr + N + c0, p2);
                if constexpr (Q4) tmem_ld16(taddr + S::kAcc * N + c0, m);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float main = __uint_as_float(p[i]);
                    if constexpr (S::kAcc == 2) main += __uint_as_float(p2[i]);
                    acc[c0 + i] = fmaf(hd.x, main, acc[c0 + i]);
                    if constexpr (Q4) acc[c0 + i] = fmaf(-hd.y, __uint_as_float(m[i]), acc[c0 + i]);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tmem_empty + 8 * buf);
            const bool last = w.last_column();
            const uint32_t rb = w.rb, slice = w.slice;
            const bool split = w.split;
            w.next(a);
            ++tc;
            if (!last) continue;
            TPROF_BEGIN

            // ---- end of an item: meet the other K slices, then store
            if (a.fold)
#pragma unroll
                for (int i = 0; i < C / 2; ++i) acc[i] = acc[2 * i] + acc[2 * i + 1];
            const uint32_t row = rb * kTcRows + row_in_block;
            const bool live = row < a.n_out;
            bool finish = true;
            if (split) {
                if (live)
#pragma unroll
                    for (int i = 0; i < C; ++i)
                        if ((uint32_t)i < n_tok && tok0 + i < a.tokens) a.partial[((size_t)slice * a.tokens + tok0 + i) * a.n_out + row] = acc[i];
                // Release / acquire through the counter: the warp barrier orders every lane's stores before lane 0's
                // releasing add, and lane 0's acquire (handed on by the shuffle) before every lane's loads below.
                __syncwarp();
                unsigned int seen = 0;
                unsigned int *counter = a.counters + (rb * 4 + quad) * 2 + part;
                if (lane == 0) asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(seen) : "l"(counter) : "memory");
                seen = __shfl_sync(0xffffffffu, seen, 0);
                finish = seen == a.ksplit - 1;
                if (finish) {
                    if (lane == 0) *counter = 0; // ready for the next launch
                    // Slices are added in slice order (deterministic), but fetched four at a time: a step's 32 loads
                    // are in flight together, so eighteen slices cost five trips to L2 instead of eighteen.
#pragma unroll
                    for (int c0 = 0; c0 < C; c0 += 8) {
                        float v[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) v[j] = 0.0f;
                        for (uint32_t sl0 = 0; sl0 < a.ksplit; sl0 += 4) {
                            float got[4][8];
#pragma unroll
                            for (uint32_t b = 0; b < 4; ++b) {
                                const uint32_t sl = min(sl0 + b, a.ksplit - 1); // past the last slice: re-read it, and do not add it
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    const uint32_t t = min(tok0 + (uint32_t)(c0 + j), a.tokens - 1); // past `tokens`: re-read the last one
                                    got[b][j] = __ldcg(a.partial + ((size_t)sl * a.tokens + t) * a.n_out + (live ? row : 0u));
                                }
                            }
#pragma unroll
                            for (uint32_t b = 0; b < 4; ++b)
                                if (sl0 + b < a.ksplit)
#pragma unroll
                                    for (int j = 0; j < 8; ++j) v[j] += got[b][j];
                        }
#pragma unroll
                        for (int j = 0; j < 8; ++j) acc[c0 + j] = v[j];
                    }
                }
            }
            if (finish && live) {
#pragma unroll
                for (int i = 0; i < C; ++i) {
                    const uint32_t t = tok0 + i;
                    if ((uint32_t)i >= n_tok || t >= a.tokens) continue;
                    float r = acc[i];
                    const size_t o = (size_t)t * a.n_out + row;
                    if (a.row_scale) r *= a.row_scale[t];
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
#pragma unroll
            for (int i = 0; i < C; ++i) acc[i] = 0.0f;
            TPROF_END(1)
        }
        if (lane == 0 && warp == 2 + kTcDequantWarps) { TPROF_FLUSH(4) }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0) { TPROF_STAMP_MAX(4) }
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(S::kTmemCols) : "memory");
    if (threadIdx.x == 32) { TPROF_STAMP_MAX(5) }
}

#ifdef MUSER_GEMM_WAIT_PROFILE
extern "C" __attribute__((visibility("default"))) int muser_cuda_debug_tc_wait_profile(unsigned long long *out) {
    return (int)cudaMemcpyFromSymbol(out, g_tc_wait_prof, sizeof(g_tc_wait_prof));
}
extern "C" __attribute__((visibility("default"))) int muser_cuda_debug_tc_stamps(unsigned long long *out) {
    return (int)cudaMemcpyFromSymbol(out, g_tc_stamps, sizeof(g_tc_stamps));
}
#endif

// Activations into the form the kernel reads: f16, N rows (rows past `tokens` zero), columns in the weight image's
// tile coordinates (a K shard's first tile may start before the shard's first input: those columns are zero), and
// per 32-input sub-block the sum of the f16 values as an f16 head + remainder pair.
template <bool XF32>
__global__ void __launch_bounds__(256) kquant_tc_prepare_kernel(const void *__restrict__ x, uint32_t tokens, uint32_t n_in, uint32_t k_off,
                                                                uint32_t nsb, __half *__restrict__ xh, __half *__restrict__ xs) {
    // Output row = token.  bf16 activations inside f16's range (2^-14 <= |x| <= 65504, which covers normalized
    // hidden states) are exact in f16; larger magnitudes are clamped to 65504 and smaller ones lose bits: the range
    // limit of this kernel (the decode kernel, which serves up to 16 tokens, scales every tile by its own maximum
    // and has none).  f32 activations
    // are carried (to 22 bits, same range) as an f16 head in row 2t and the remainder in row 2t + 1; the kernel
    // adds the two columns at the end.
#ifdef MUSER_GEMM_WAIT_PROFILE
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) { // (the GEMM cannot start before every block of this grid has passed pdl_release)
        g_tc_stamps[0] = g_tc_stamps[2] = ~0ull;
        g_tc_stamps[1] = g_tc_stamps[3] = g_tc_stamps[4] = g_tc_stamps[5] = 0;
        __threadfence();
    }
    __syncthreads();
    if (threadIdx.x == 0) { TPROF_STAMP_MIN(0) }
#endif
    pdl_release(); // the GEMM behind this kernel may start its set-up and its weight copies now; it waits before it reads xh / xs
    const uint32_t tile = blockIdx.x, r = blockIdx.y, i = threadIdx.x;
    const uint32_t tok = XF32 ? r >> 1 : r, part = XF32 ? r & 1 : 0;
    const int64_t k = (int64_t)tile * 256 + i - (int64_t)k_off;
    float v = 0.0f;
    if (tok < tokens && k >= 0 && k < (int64_t)n_in)
        v = XF32 ? reinterpret_cast<const float *>(x)[(size_t)tok * n_in + k]
                 : __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(x)[(size_t)tok * n_in + k]);
    v = fminf(fmaxf(v, -65504.0f), 65504.0f); // f16 range; NaN passes through
    __half hv = __float2half_rn(v);
    if (part) hv = __float2half_rn(v - __half2float(hv));
    xh[(size_t)r * nsb * 256 + (size_t)tile * 256 + i] = hv;
    float s = __half2float(hv);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((i & 31) == 0) {
        const __half head = __float2half_rn(s);
        const __half rest = __float2half_rn(s - __half2float(head));
        __half *dst = xs + (size_t)r * nsb * 16 + (size_t)tile * 16 + 2 * (i >> 5);
        dst[0] = head;
        dst[1] = rest;
    }
    if (threadIdx.x == 0) { TPROF_STAMP_MAX(1) }
}

// Issue-rate probe for the instruction this kernel is built on: one thread per SM issues `iters` x 4
// tcgen05.mma kind::f16 (M = 128, K = 16, N columns) back to back on resident operands and one accumulator, and CTA 0
// reports the cycles from the first issue to the completion of the last.
template <int N>
__global__ void __launch_bounds__(128, 1) f16_mma_probe_kernel(uint32_t iters, long long *out, int *status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *aligned = smem_raw + (base - smem_u32(smem_raw));
    constexpr int kOperands = 16384 + 32768; // A: 128 rows x 128 bytes, B: up to 256 rows x 128 bytes
    uint64_t *bars = reinterpret_cast<uint64_t *>(aligned + kOperands);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    for (uint32_t i = threadIdx.x; i < kOperands / 16; i += blockDim.x) reinterpret_cast<uint4 *>(aligned)[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(bars), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    const int warp = threadIdx.x >> 5;
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    if (threadIdx.x == 32) {
        const uint32_t idesc = (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(kTcRows >> 4) << 24);
        const uint64_t da = operand_desc(base), db = operand_desc(base + 16384);
        const long long t0 = clock64();
        for (uint32_t i = 0; i < iters; ++i)
#pragma unroll
            for (uint32_t kk = 0; kk < 4; ++kk) mma_f16(tmem, da + 2 * kk, db + 2 * kk, idesc, (i | kk) != 0);
        mma_commit(smem_u32(bars));
        if (!mbar_wait(smem_u32(bars), 0, abort_flag)) atomicExch(status + 1, 305);
        if (blockIdx.x == 0) out[0] = clock64() - t0;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u) : "memory");
}

muser_cuda_status launch_f16_mma_probe(Ctx *ctx, uint32_t n_cols, uint32_t iters, double *cycles_per_mma) {
    constexpr int kSmem = 16384 + 32768 + 64 + 1024;
    long long *out = reinterpret_cast<long long *>(ctx->gemv_partial); // scratch; the call synchronizes
    auto run = [&](auto kernel) -> cudaError_t {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
        if (e != cudaSuccess) return e;
        kernel<<<ctx->sm_count, 128, kSmem>>>(iters, out, ctx->dev_status);
        return cudaGetLastError();
    };
    cudaError_t e;
    switch (n_cols) {
    case 16: e = run(f16_mma_probe_kernel<16>); break;
    case 32: e = run(f16_mma_probe_kernel<32>); break;
    case 64: e = run(f16_mma_probe_kernel<64>); break;
    case 128: e = run(f16_mma_probe_kernel<128>); break;
    case 256: e = run(f16_mma_probe_kernel<256>); break;
    default: return fail(ctx, MUSER_CUDA_BAD_ARG, "probe widths: 16, 32, 64, 128, 256");
    }
    MUSER_CUDA_TRY(ctx, e);
    long long cycles = 0;
    MUSER_CUDA_TRY(ctx, cudaMemcpy(&cycles, out, sizeof cycles, cudaMemcpyDeviceToHost));
    *cycles_per_mma = (double)cycles / (4.0 * iters);
    return MUSER_CUDA_OK;
}

// ------------------------------------------------------------------------------------------ host side
// Items: as many whole row blocks as fill complete rounds over the SMs run unsplit (no exchange at their end); the
// remaining row blocks are cut into K slices so that the last round keeps the SMs busy too.  An exchange costs about
// as much as four super-block columns.
struct TcPlan {
    uint32_t whole, ksplit;
};
static TcPlan tc_plan(uint32_t nsb, uint32_t row_blocks, int sm_count, uint32_t max_split) {
    TcPlan p{row_blocks / sm_count * sm_count, 1};
    const uint32_t tail = row_blocks - p.whole;
    if (tail == 0) return p;
    double best_cost = 1e300;
    for (uint32_t ks = 1; ks <= max_split && ks <= nsb && ks <= 32; ++ks) {
        const double rounds = std::ceil((double)tail * ks / sm_count);
        const double cost = rounds * (std::ceil((double)nsb / ks) + (ks > 1 ? 4.0 : 0.0));
        if (cost < best_cost * (1.0 - 1e-9)) best_cost = cost, p.ksplit = ks;
    }
    return p;
}

template <int DT, int N>
static cudaError_t tc_launch(const CUtensorMap &mx, const CUtensorMap &mxs, const TcArgs &a, int device, int grid, cudaStream_t stream) {
    using S = TcSmem<DT, N>;
    const cudaError_t ae = ensure_dynamic_smem(reinterpret_cast<const void *>(kquant_tc_kernel<DT, N>), device, S::kBytes);
    if (ae != cudaSuccess) return ae;
    // may begin while the kernel that prepares its activations is still running: set-up and the first weight tiles overlap it
    return launch_pdl(kquant_tc_kernel<DT, N>, dim3(grid), dim3(S::kThreads), S::kBytes, stream, mx, mxs, a);
}

// cudaErrorNotSupported: this shape is not served here (the caller falls back to the other kernels).
cudaError_t launch_kquant_tc(Ctx *ctx, const Weight *w, const void *x, uint32_t x_dtype, void *y, uint32_t y_dtype,
                             uint32_t tokens, const Epilogue &ep, cudaStream_t stream) {
    const bool xf32 = x_dtype == MUSER_DTYPE_F32;
    const uint32_t cols = xf32 ? 2 * tokens : tokens; // f32 activations take two columns each (f16 head + remainder)
    if (cols > 64 || !ctx->tc_scratch) return cudaErrorNotSupported;
    const uint32_t n = cols <= 16 ? 16 : (cols <= 32 ? 32 : 64);
    const size_t xh_bytes = (size_t)n * w->nsb * 256 * sizeof(__half), xs_bytes = (size_t)n * w->nsb * 16 * sizeof(__half);
    const size_t xs_off = (xh_bytes + 1023) & ~(size_t)1023;
    if (xs_off + xs_bytes > ctx->tc_scratch_bytes) return cudaErrorNotSupported;
    __half *xh = reinterpret_cast<__half *>(ctx->tc_scratch);
    __half *xs = reinterpret_cast<__half *>(reinterpret_cast<uint8_t *>(ctx->tc_scratch) + xs_off);
    const dim3 pgrid(w->nsb, n);
    if (xf32)
        kquant_tc_prepare_kernel<true><<<pgrid, 256, 0, stream>>>(x, tokens, (uint32_t)w->n_in, w->k_off, w->nsb, xh, xs);
    else
        kquant_tc_prepare_kernel<false><<<pgrid, 256, 0, stream>>>(x, tokens, (uint32_t)w->n_in, w->k_off, w->nsb, xh, xs);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;

    CUtensorMap mx, mxs;
    if (!tma_make_map(&mx, xh, n, (uint64_t)w->nsb * 512, n, 128) || !tma_make_map(&mxs, xs, n, (uint64_t)w->nsb * 32, n, 32))
        return cudaErrorInvalidValue;
    TcArgs a;
    a.image = w->image;
    a.y = y;
    a.row_scale = ep.row_scale;
    a.out_scale = ep.out_scale;
    a.softcap = ep.softcap;
    a.residual = ep.residual;
    a.partial = ctx->gemv_partial;
    a.counters = ctx->gemv_counters;
    a.status = ctx->dev_status;
    a.n_out = (uint32_t)w->n_out;
    a.nsb = w->nsb;
    a.row_tiles = w->row_tiles;
    a.tokens = tokens;
    a.y_bf16 = y_dtype == MUSER_DTYPE_BF16;
    a.fold = xf32 ? 1u : 0u;
    const uint32_t row_blocks = (w->row_tiles + 7) / 8;
    const size_t slice_bytes = (size_t)tokens * w->n_out * sizeof(float);
    uint32_t max_split = (uint32_t)std::max<size_t>(1, ctx->gemv_partial_bytes / std::max<size_t>(1, slice_bytes));
    if ((size_t)row_blocks * 8 > ctx->gemv_counter_slots) max_split = 1;
    const TcPlan plan = tc_plan(w->nsb, row_blocks, ctx->sm_count, max_split);
    a.whole = plan.whole;
    a.ksplit = plan.ksplit;
    a.items = plan.whole + (row_blocks - plan.whole) * plan.ksplit;
    const int grid = (int)std::min<uint32_t>(a.items, (uint32_t)ctx->sm_count);
    if (w->dtype == MUSER_DTYPE_Q4_K)
        return n == 16 ? tc_launch<MUSER_DTYPE_Q4_K, 16>(mx, mxs, a, ctx->device, grid, stream)
             : n == 32 ? tc_launch<MUSER_DTYPE_Q4_K, 32>(mx, mxs, a, ctx->device, grid, stream)
                       : tc_launch<MUSER_DTYPE_Q4_K, 64>(mx, mxs, a, ctx->device, grid, stream);
    return n == 16 ? tc_launch<MUSER_DTYPE_Q6_K, 16>(mx, mxs, a, ctx->device, grid, stream)
         : n == 32 ? tc_launch<MUSER_DTYPE_Q6_K, 32>(mx, mxs, a, ctx->device, grid, stream)
                   : tc_launch<MUSER_DTYPE_Q6_K, 64>(mx, mxs, a, ctx->device, grid, stream);
}

} // namespace muser
