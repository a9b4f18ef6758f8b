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
// One CTA per SM, persistent over (128-row block, K slice) items:
//   warp 0      TMA: activation slabs (N tokens x 128 inputs, 128-byte swizzle) and the X_j pairs (32-byte swizzle)
//   warp 1      tcgen05.mma kind::f16, M = 128 rows, N = tokens (16 / 32 / 64), K = 16; accumulators in tensor memory,
//               four buffers so that the drain of one super-block column runs under the MMAs of the next ones
//   warps 2-17  eight rows of one 16-row weight tile each: bulk copies global -> shared (three or four tiles in flight
//               per warp), unpack to the f16 integers above, store into the swizzled A stage (two stages of 128 inputs)
//   warps 18-.. drain (four warps; eight from 32 token columns on, half the columns each, so that the running sums
//               stay in registers): tcgen05.ld, scale by d / dmin (f32), keep the running sums per row in registers;
//               at the end of an item add the K slices through the context scratch (last arriver sums in slice
//               order) and store
// Every wait is bounded; a wait that gives up records a code in the context's status word and the CTA winds down.
#include <algorithm>
#include <cmath>
#include <type_traits>

#include "common.cuh"
#include "kquant_layout.cuh"
#include "tcgen05.cuh"

namespace muser {

constexpr int kTcRows = 128;             // weight rows per block = MMA M
constexpr int kTcStages = 2;             // A stages of 128 inputs each (the unpacked weights are the expensive bytes)
constexpr int kTcABytes = kTcRows * 256; // 128 rows x 128 f16: two 64-column swizzle atoms of 16 KiB
constexpr int kTcDequantWarps = 16;           // warp = (row tile of the block, upper / lower eight rows)

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

// ------------------------------------------------------------------------------------ Q4_K
// What one unpacking warp holds of a tile: rows g (+ 8 * rowsel, rowsel fixed per warp), lane (g, t).
// Its ring slot is [2 planes of 512 bytes: sub-blocks 0-3 and 4-7, this lane's eight elements of each][8 row headers].
constexpr int kTcQ4Slot = 1024 + 128, kTcQ6Slot = 1024 + 512 + 128 + 16;
struct TcQ4 {
    uint4 q[2]; // [half]: word jj = sub-block 4*half + jj, elements 8t .. 8t+7
    uint4 h;    // the row's header
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
__device__ __forceinline__ TcQ4 tc_load(const uint8_t *slot, int lane, TcQ4 *) {
    TcQ4 r;
    const uint4 *q = reinterpret_cast<const uint4 *>(slot);
    r.q[0] = q[lane];
    r.q[1] = q[32 + lane];
    r.h = reinterpret_cast<const uint4 *>(slot + 1024)[lane >> 2];
    return r;
}
// Inputs 128*HALF .. +127 of row `row` (a multiple of 8 plus g) -> the A stage: sc * q as f16.
// Column layout (kquant_layout.cuh): word jj of r.q[HALF] holds elements 8t .. 8t+7 of sub-block 4*HALF + jj, i.e.
// the 16-byte chunk 4*jj + t of the row's 128 inputs: atom jj / 2, chunk (jj % 2) * 4 + t inside it.
template <int HALF>
__device__ __forceinline__ void tc_unpack_half(const TcQ4 &r, const TcQ4Hdr &hd, uint32_t stage, uint32_t row, int g, int t) {
    const uint32_t base = stage + (row >> 3) * 1024u + (row & 7) * 128u;
    // In one store instruction the lanes of rows g and g + 1 would write the same four chunks of two rows, i.e. the
    // same banks; odd rows therefore take their words in the order 1, 0, 3, 2, which puts them in the other half of
    // the 128-byte row and makes the warp's stores conflict-free.
    const uint32_t odd = (uint32_t)g & 1u;
    uint4 qv = r.q[HALF];
    if (odd) qv = make_uint4(qv.y, qv.x, qv.w, qv.z);
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
        const uint32_t jj = (uint32_t)wi ^ odd; // sub-block 4*HALF + jj
        const __half2 sc = byte_pair(hd.sc[HALF], jj, 1024.0f);
        const __half2 off = __hmul2(sc, __float2half2_rn(-1024.0f)); // exact: at most 63 * 1024
        const uint32_t w = word_of(qv, wi);
        uint32_t o[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) { // nibbles p and p + 4 of the word are elements 2p, 2p + 1
            const uint32_t e = ((w >> (4 * p)) & 0x000F000Fu) | 0x64006400u; // (1024 + q, 1024 + q')
            o[p] = h2u(__hfma2(u2h(e), sc, off));                            // sc * q, exact
        }
        const uint32_t chunk = ((jj & 1u) * 4u + (uint32_t)t) ^ (uint32_t)g;
        sts128(base + (jj >> 1) * 16384u + chunk * 16u, o[0], o[1], o[2], o[3]);
    }
}

// ------------------------------------------------------------------------------------ Q6_K
// Ring slot: [2 top-nibble planes of 512 bytes][low-two-bits plane, 512][8 x sc[16] int8][8 x d f16].
struct TcQ6 {
    uint4 lo[2]; // [half]
    uint4 hi;
    uint4 sc;
    float d;
};
__device__ __forceinline__ TcQ6 tc_load(const uint8_t *slot, int lane, TcQ6 *) {
    TcQ6 r;
    const uint4 *q = reinterpret_cast<const uint4 *>(slot);
    r.lo[0] = q[lane];
    r.lo[1] = q[32 + lane];
    r.hi = q[64 + lane];
    r.sc = reinterpret_cast<const uint4 *>(slot + 1536)[lane >> 2];
    r.d = __half2float(reinterpret_cast<const __half *>(slot + 1664)[lane >> 2]);
    return r;
}
__device__ __forceinline__ void sts64(uint32_t addr, uint32_t a, uint32_t b) {
    asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
// Column layout: the lane holds elements 4t .. 4t+3 of every sub-block of its row, stored as (q - 32) & 63 split
// into a top-nibble plane (r.lo) and a low-two-bits plane (r.hi); (T << 4) | (L << 2) is the signed byte 4 (q - 32).
// What goes to the A stage is 4 * sc * (q - 32) as f16 (the factor 4 is a shift of the exponent, so the products are
// as exact as sc * (q - 32) itself); the drain's d carries the 1/4.
template <int HALF>
__device__ __forceinline__ void tc_unpack_half(const TcQ6 &r, uint32_t stage, uint32_t row, int g, int t) {
    const __half2 k1152 = __float2half2_rn(1152.0f);
    const uint32_t base = stage + (row >> 3) * 1024u + (row & 7) * 128u + (uint32_t)(t & 1) * 8u;
#pragma unroll
    for (int sl = 0; sl < 8; ++sl) { // sub-block 8*HALF + sl: inputs 16*sl + 4t .. + 3 of the half
        constexpr int kX[4] = {2, 0, -2, -4};
        const uint32_t tw = word_of(r.lo[HALF], sl >> 1), lw = word_of(r.hi, 2 * HALF + (sl >> 2));
        const uint32_t top = (sl & 1) ? tw : tw << 4;
        const int sh = kX[sl & 3];
        const uint32_t low = sh > 0 ? lw << sh : lw >> (-sh);
        const uint32_t b = ((top & 0xF0F0F0F0u) | (low & 0x0C0C0C0Cu)) ^ 0x80808080u; // bytes 4 (q - 32) + 128
        const __half2 sc = byte_pair(word_of(r.sc, 2 * HALF + (sl >> 2)) ^ 0x80808080u, (uint32_t)(sl & 3), 1152.0f); // int8 scale, exact
        const uint32_t p0 = __byte_perm(b, 0x64646464u, 0x4140u), p1 = __byte_perm(b, 0x64646464u, 0x4342u);
        const uint32_t o0 = h2u(__hmul2(__hsub2(u2h(p0), k1152), sc)), o1 = h2u(__hmul2(__hsub2(u2h(p1), k1152), sc));
        const uint32_t chunk = (uint32_t)(2 * (sl & 3) + (t >> 1)) ^ (uint32_t)g;
        sts64(base + (uint32_t)(sl >> 2) * 16384u + chunk * 16u, o0, o1);
    }
}

// ------------------------------------------------------------------------------------ kernel
template <int DT, int N>
struct TcSmem {
    static constexpr bool kQ4 = DT == MUSER_DTYPE_Q4_K;
    static constexpr int kTile = kQ4 ? kQ4TileBytes : kQ6TileBytes, kSlot = kQ4 ? kTcQ4Slot : kTcQ6Slot;
    // Raw tiles in flight per unpacking warp.  HBM latency times the stream's rate is ~55 KB per SM, and the warps
    // run in step, so the rings are made as deep as shared memory allows: 72-105 KB of weights in flight per SM.
    static constexpr int kRing = (!kQ4 && N == 64) ? 3 : 4;
    static constexpr int kStagesB = N == 64 ? 3 : 4; // activation slabs come from L2 with ~1500 cycles of latency
    static constexpr int kBBytes = N * 256;          // two atoms of N rows x 128 bytes
    static constexpr int kMinA = kTcRows * 32, kMinB = N * 32 < 1024 ? 1024 : N * 32;
    static constexpr int kOffB = kTcStages * kTcABytes;
    static constexpr int kOffMinA = kOffB + kStagesB * kBBytes;
    static constexpr int kOffMinB = kOffMinA + 2 * kMinA;
    static constexpr int kOffRing = kOffMinB + 2 * kMinB;
    static constexpr int kOffHdr = kOffRing + kTcDequantWarps * kRing * kSlot;
    static constexpr int kHdrDepth = 8;              // (d, dmin) per row of the last eight super-block columns
    static constexpr int kOffBars = kOffHdr + kHdrDepth * kTcRows * 8;
    static constexpr int kBufs = 4;                  // accumulator buffers in tensor memory, each kAcc main parts + the min part
    static constexpr int kAcc = N <= 32 ? 2 : 1;     // two main accumulators taken in turn where the columns allow (measured faster)
    static constexpr int kBufCols = (kAcc + 1) * N;
    static constexpr int kDrainWarps = N >= 32 ? 8 : 4, kDrainCols = N / (kDrainWarps / 4);
    static constexpr int kThreads = 32 * (2 + kTcDequantWarps + kDrainWarps);
    static constexpr int kBars = 2 * kTcStages + 2 * kStagesB + 2 * kBufs + kTcDequantWarps * kRing;
    static constexpr int kBytes = kOffBars + kBars * 8 + 16 + 1024 /*alignment slack*/;
    static_assert(kBytes <= 227 * 1024, "shared memory of one CTA exceeded");
    static constexpr uint32_t kTmemCols = N == 16 ? 256 : 512; // kBufs x kBufCols = 192 / 384 / 512, rounded up to a power of two
};

template <int DT, int N>
__global__ void __launch_bounds__((TcSmem<DT, N>::kThreads), 1)
kquant_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_xs, const TcArgs a) {
    using S = TcSmem<DT, N>;
    constexpr bool Q4 = S::kQ4;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *aligned = smem_raw + (base - smem_u32(smem_raw));
    uint64_t *bars = reinterpret_cast<uint64_t *>(aligned + S::kOffBars);
    constexpr int kRing = S::kRing, kStagesB = S::kStagesB;
    const uint32_t bar_full_a = smem_u32(bars), bar_empty_a = bar_full_a + 8 * kTcStages;
    const uint32_t bar_full_b = bar_empty_a + 8 * kTcStages, bar_empty_b = bar_full_b + 8 * kStagesB;
    constexpr int kBufs = S::kBufs;
    const uint32_t bar_tmem_full = bar_empty_b + 8 * kStagesB, bar_tmem_empty = bar_tmem_full + 8 * kBufs, bar_ring = bar_tmem_empty + 8 * kBufs;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + S::kBars);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    float2 *hdr = reinterpret_cast<float2 *>(aligned + S::kOffHdr);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kTcStages; ++s) {
            mbar_init(bar_full_a + 8 * s, kTcDequantWarps);
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
        for (int i = 0; i < kTcDequantWarps * kRing; ++i) mbar_init(bar_ring + 8 * i, 1);
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

    if (warp == 0) {
        // ---------------------------------------------------------------- activation producer
        if (lane == 0) {
            TcWalk w;
            w.start(a);
            uint32_t hs = 0, tc = 0, issued = 0;
            bool ok = true;
            for (; !w.done(a) && ok; w.next(a), ++tc) {
                for (uint32_t h = 0; h < 2; ++h, ++hs) {
                    const uint32_t s = hs % kStagesB, round = hs / kStagesB;
                    if (round > 0) ok = mbar_wait_relaxed(bar_empty_b + 8 * s, (round - 1) & 1, abort_flag, 32);
                    if (!ok) break;
                    const uint32_t full = bar_full_b + 8 * s, dst = base + S::kOffB + s * S::kBBytes;
                    const bool with_sums = Q4 && h == 1;
                    mbar_expect_tx(full, S::kBBytes + (with_sums ? N * 32 : 0));
                    const int x0 = (int)((w.k * 256 + h * 128) * 2);
                    tma_load_2d(dst, &map_x, x0, 0, full);
                    tma_load_2d(dst + N * 128, &map_x, x0 + 128, 0, full);
                    if (with_sums) tma_load_2d(base + S::kOffMinB + (tc & 1) * S::kMinB, &map_xs, (int)(w.k * 32), 0, full);
                    issued = hs + 1;
                }
            }
            if (!ok) {
                *abort_flag = 1;
                atomicExch(a.status + 1, 301);
                // let the copies already in flight land before the CTA's shared memory goes away
                const uint32_t first = issued > (uint32_t)kStagesB ? issued - kStagesB : 0;
                for (uint32_t k = first; k < issued; ++k) mbar_wait_alone(bar_full_b + 8 * (k % kStagesB), (k / kStagesB) & 1);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            // kind::f16: f32 accumulator (bit 4), A and B f16 (format 0), both K-major, N >> 3 at bit 17, M >> 4 at bit 24
            const uint32_t idesc = (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(kTcRows >> 4) << 24);
            TcWalk w;
            w.start(a);
            uint32_t hs = 0, tc = 0;
            bool ok = true;
            for (; !w.done(a) && ok; w.next(a), ++tc) {
                const uint32_t buf = tc % kBufs, d_main = tmem + buf * S::kBufCols, d_min = d_main + S::kAcc * N;
                if (tc >= (uint32_t)kBufs) { // the drain warps must have read this buffer's previous contents
                    ok = mbar_wait(bar_tmem_empty + 8 * buf, ((tc / kBufs) - 1) & 1, abort_flag);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                }
                for (uint32_t h = 0; h < 2; ++h, ++hs) {
                    const uint32_t s = hs % kTcStages, round = hs / kTcStages, s_b = hs % kStagesB, round_b = hs / kStagesB;
                    ok = mbar_wait(bar_full_b + 8 * s_b, round_b & 1, abort_flag); if (ok) ok = mbar_wait(bar_full_a + 8 * s, round & 1, abort_flag);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sa = base + s * kTcABytes, sb = base + S::kOffB + s_b * S::kBBytes;
#pragma unroll
                    for (uint32_t atom = 0; atom < 2; ++atom) {
                        const uint64_t da = operand_desc(sa + atom * 16384u), db = operand_desc(sb + atom * (N * 128u));
#pragma unroll
                        for (uint32_t kk = 0; kk < 4; ++kk) // 16 values = 32 bytes along the swizzled 128-byte rows
                            mma_f16(d_main + (S::kAcc == 2 ? (kk & 1) * N : 0), da + 2 * kk, db + 2 * kk, idesc,
                                    (h | atom | (S::kAcc == 2 ? kk >> 1 : kk)) != 0);
                    }
                    if (Q4 && h == 1)
                        mma_f16(d_min, operand_desc32(base + S::kOffMinA + (tc & 1) * S::kMinA),
                                operand_desc32(base + S::kOffMinB + (tc & 1) * S::kMinB), idesc, 0);
                    mma_commit(bar_empty_a + 8 * s); // stages (and the sum buffers) reusable once these MMAs have read them
                    mma_commit(bar_empty_b + 8 * s_b);
                }
                if (ok) mma_commit(bar_tmem_full + 8 * buf);
            }
            if (!ok) {
                *abort_flag = 1;
                atomicExch(a.status + 1, 302);
            }
        }
    } else if (warp < 2 + kTcDequantWarps) {
        // ---------------------------------------------------------------- weight unpackers
        using Regs = typename std::conditional<Q4, TcQ4, TcQ6>::type;
        const int dw = warp - 2, g = lane >> 2, t = lane & 3;
        const uint32_t rsel = (uint32_t)dw & 1, row = (uint32_t)(dw >> 1) * 16 + g + 8 * rsel; // this lane's row of the block
        uint8_t *ring = aligned + S::kOffRing + dw * kRing * S::kSlot;
        const uint32_t rbar = bar_ring + 8 * dw * kRing;
        auto fetch = [&](const TcWalk &x, uint32_t slot) { // this warp's eight rows of one tile: its planes and headers
            if (lane == 0) {
                const uint32_t rt = min(x.rb * (kTcRows / kTileRows) + (uint32_t)(dw >> 1), a.row_tiles - 1); // a short last block repeats its last tile
                const uint8_t *src = a.image + ((uint64_t)rt * a.nsb + x.k) * S::kTile;
                const uint32_t dst = smem_u32(ring) + slot * S::kSlot, bar = rbar + 8 * slot;
                mbar_expect_tx(bar, S::kSlot);
                bulk_load(dst, src + 1024 * rsel, 1024, bar);
                if constexpr (Q4) {
                    bulk_load(dst + 1024, src + 2048 + 128 * rsel, 128, bar);
                } else {
                    bulk_load(dst + 1024, src + kQ6OffHi + 512 * rsel, 512, bar);
                    bulk_load(dst + 1536, src + kQ6OffSc + 128 * rsel, 128, bar);
                    bulk_load(dst + 1664, src + kQ6OffD + 16 * rsel, 16, bar);
                }
            }
        };
        TcWalk w, f;
        w.start(a);
        f = w;
        uint32_t fetched = 0;
        for (; fetched < (uint32_t)kRing && !f.done(a); ++fetched, f.next(a)) fetch(f, fetched);
        uint32_t n = 0, hs = 0;
        bool ok = true;
        // one half (128 inputs) of the tile in `cur` into its stage, then tell the MMA warp
        auto half_step = [&](const Regs &cur, const TcQ4Hdr &hd, auto half_tag) {
            constexpr int HALF = decltype(half_tag)::value;
            const uint32_t s = hs % kTcStages, round = hs / kTcStages;
            if (round > 0) ok = mbar_wait(bar_empty_a + 8 * s, (round - 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) return;
            if constexpr (Q4) tc_unpack_half<HALF>(cur, hd, base + s * kTcABytes, row, g, t);
            else tc_unpack_half<HALF>(cur, base + s * kTcABytes, row, g, t);
            if constexpr (HALF == 1) {
                if constexpr (Q4) {
                    // min operand: 16 f16 per row, (m_j, m_j) for j = 0..7; lanes t = 0, 1 write the row's two 16-byte chunks
                    if (t < 2) {
                        const uint32_t mw = t ? hd.mn[1] : hd.mn[0];
                        const uint32_t chunk = (uint32_t)t ^ ((row >> 2) & 1);
                        sts128(base + S::kOffMinA + (n & 1) * S::kMinA + (row >> 3) * 256u + (row & 7) * 32u + chunk * 16u,
                               h2u(byte_pair(mw, 0, 1024.0f)), h2u(byte_pair(mw, 1, 1024.0f)), h2u(byte_pair(mw, 2, 1024.0f)),
                               h2u(byte_pair(mw, 3, 1024.0f)));
                    }
                    if (t == 2) hdr[(n % S::kHdrDepth) * kTcRows + row] = make_float2(hd.d, hd.dmin);
                } else {
                    if (t == 2) hdr[(n % S::kHdrDepth) * kTcRows + row] = make_float2(0.25f * cur.d, 0.0f); // the A operand is 4 sc (q - 32)
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // generic stores -> visible to the MMA's reads
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_full_a + 8 * s);
            ++hs;
        };
        for (; !w.done(a) && ok; w.next(a), ++n) {
            const uint32_t slot = n % kRing;
            ok = mbar_wait(rbar + 8 * slot, (n / kRing) & 1, abort_flag);
            if (!ok) break;
            const Regs cur = tc_load(ring + slot * S::kSlot, lane, (Regs *)nullptr);
            __syncwarp(); // every lane has its copy: the slot may be refilled
            if (!f.done(a)) {
                fetch(f, slot);
                f.next(a);
                ++fetched;
            }
            TcQ4Hdr hd{};
            if constexpr (Q4) hd = tc_q4_hdr(cur.h);
            half_step(cur, hd, std::integral_constant<int, 0>{});
            if (ok) half_step(cur, hd, std::integral_constant<int, 1>{});
        }
        if (!ok && lane == 0) {
            *abort_flag = 1;
            atomicCAS(a.status + 1, 0, 303);
        }
        // copies still in flight into this warp's ring must land before the CTA's shared memory goes away
        if (!ok)
            for (uint32_t k = n; k < fetched; ++k) mbar_wait_alone(rbar + 8 * (k % kRing), (k / kRing) & 1);
    } else {
        // ---------------------------------------------------------------- drain (the last 4 or 8 warps)
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
        uint32_t tc = 0;
        while (!w.done(a)) {
            const uint32_t buf = tc % kBufs;
            const bool ok = __all_sync(0xffffffffu, mbar_wait_relaxed(bar_tmem_full + 8 * buf, (tc / kBufs) & 1, abort_flag, 40));
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
                    // slices in order (deterministic); sixteen independent loads in flight per step, not one
#pragma unroll
                    for (int c0 = 0; c0 < C; c0 += 16) {
                        float v[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                        for (uint32_t sl = 0; sl < a.ksplit; ++sl) {
                            float got[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const uint32_t t = min(tok0 + (uint32_t)(c0 + j), a.tokens - 1); // past `tokens`: re-read the last one
                                got[j] = __ldcg(a.partial + ((size_t)sl * a.tokens + t) * a.n_out + (live ? row : 0u));
                            }
#pragma unroll
                            for (int j = 0; j < 16; ++j) v[j] += got[j];
                        }
#pragma unroll
                        for (int j = 0; j < 16; ++j) acc[c0 + j] = v[j];
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
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(S::kTmemCols) : "memory");
}

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
    kquant_tc_kernel<DT, N><<<grid, S::kThreads, S::kBytes, stream>>>(mx, mxs, a);
    return cudaGetLastError();
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
