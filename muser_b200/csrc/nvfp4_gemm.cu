// NVFP4 x NVFP4 block-scaled GEMM on the 5th-generation tensor cores: y[t][n] = sum_k x[t][k] * w[n][k].
//
// Stands in for MetalKernels::encode_nvfp4_matmul / encode_nvfp4_w4a4_prequant_m16
// (crates/muser-engine/src/metal/encode/qkv.rs:13-65,128-227) and the W4A4 lane of weights::matmul
// (src/weights.rs:111-121, quant/nvfp4.rs:304-338): E2M1 codes of activations and weights, one E4M3 scale per
// 16 values on each side, then (acc * weight_scale2) * (1 / input_scale_inv) in that order.
//
// Shape of the kernel: persistent CTAs, one per SM, each walking 128-token x 256-row output tiles.  Warp 0 streams 128-byte-swizzled
// K slabs (256 values) of both operands with TMA plus their scale factors with bulk copies through a
// 4-stage shared-memory ring; warp 1 copies each K = 64 block's scale factors into tensor memory (tcgen05.cp) and
// issues its tcgen05.mma kind::mxf4nvf4 right behind them into a 128 x 256 f32 accumulator in tensor memory (both
// warps run their loops converged and issue through an elected lane: tcgen05.cuh);
// warps 2-9 read the accumulator back (tcgen05.ld), apply the two tensor scales and the fused epilogue, and
// store.  Every mbarrier wait is bounded: on expiry the CTA records a code in the context's status word,
// stops issuing work, waits (bounded) for its own copies in flight, frees its tensor memory and returns.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "nvfp4_codec.cuh"
#include "tcgen05.cuh"

namespace muser {

// Development aid, compiled in only with -DMUSER_GEMM_WAIT_PROFILE: the single-thread roles of the first CTAs add
// up the SM cycles they spend in each kind of wait, and a debug entry point copies the sums out.
#ifdef MUSER_GEMM_WAIT_PROFILE
__device__ unsigned long long g_wait_prof[4 * 8 * 4]; // [cta < 4][role < 8][slot < 4]
#define PROF_DECL long long prof_t0 = 0, prof_start = clock64(); unsigned long long prof_acc[3] = {0, 0, 0};
#define PROF_BEGIN prof_t0 = clock64();
#define PROF_END(i) prof_acc[i] += (unsigned long long)(clock64() - prof_t0);
#define PROF_FLUSH(role)                                                                              \
    if (blockIdx.x < 4) {                                                                             \
        for (int i_ = 0; i_ < 3; ++i_) g_wait_prof[(blockIdx.x * 8 + (role)) * 4 + i_] = prof_acc[i_]; \
        g_wait_prof[(blockIdx.x * 8 + (role)) * 4 + 3] = (unsigned long long)(clock64() - prof_start); \
    }
#else
#define PROF_DECL
#define PROF_BEGIN
#define PROF_END(i)
#define PROF_FLUSH(role)
#endif

constexpr int BM = 128, BN = 256, BK = 256;      // tile: tokens x weight rows x values
constexpr int kStages = 4;
constexpr int kABytes = BM * BK / 2;             // 16 KiB
constexpr int kBBytes = BN * BK / 2;             // 32 KiB
constexpr int kSfaBytes = 4 * 512;               // 128 rows x 16 scales
constexpr int kSfbBytes = 2 * 4 * 512;           // 256 rows x 16 scales
constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
static_assert(kSmemBytes <= 227 * 1024, "stage ring exceeds the shared memory of one CTA");
constexpr uint32_t kTmemCols = 512;              // 256 accumulator + 16 SFA + 32 SFB, rounded to a power of two
constexpr uint32_t kSfCol = 256, kSfBufCols = 48, kSfBufs = 4; // scale buffers of 16 (SFA) + 32 (SFB) columns behind the accumulator

struct GemmArgs {
    const uint8_t *a_scales; // activations, swizzled
    const uint8_t *b_scales; // weights, swizzled
    const uint8_t *b2_scales; // second weight (up projection) of the fused gate/up form, else null
    void *y;
    const float *row_scale;
    float out_scale, softcap; // LM-head tail
    const void *residual;
    int *status;
    uint32_t tokens, n_out, k_tiles, kt64; // kt64: 64-value blocks per row (one MMA and one scale chunk each)
    uint32_t n_tiles;                      // 256-row tiles of the weight
    uint32_t y_dtype;
    float scale2, scale2_up, inv_input_scale;
    // QOUT form: the output leaves as NVFP4 activations for the next projection instead of as numbers
    uint8_t *q_packed;  // [tokens][n_out / 2]
    uint8_t *q_scales;  // swizzled, ceil(tokens / 128) x (n_out / 64) chunks
    float q_isi;        // the next projection's input_scale_inv
    uint32_t q_kt;      // n_out / 64
    uint32_t group_m;   // token tiles per raster group (tile_coords)
    // GROUP form: up to four projections of the same activations in one launch; weight-row tiles are numbered through
    // all of them (projection p owns tiles grp_tile0[p] .. grp_tile0[p + 1] - 1)
    uint32_t grp_tile0[5];
    const uint8_t *grp_b_scales[4];
    void *grp_y[4];
    uint32_t grp_n_out[4];
    float grp_scale2[4];
};

// Output tile number -> (token tile, weight-row tile).  Tiles are numbered group by group: a group is `group_m` token
// tiles; inside it the token tile runs fastest, then the weight-row tile.  The CTAs that run side by side thus share
// a few weight tiles (read from HBM once per group, from L2 by the others) and together touch only the group's
// activations, which stay in L2 while the group sweeps all weight rows.  With every token tile in one group
// (group_m >= m_tiles, the case up to a few thousand tokens) this is "token tile fastest"; at 32768 tokens the
// activations of ffn_down alone are 453 MB, and without groups each of its 20 weight-row tiles re-read them from HBM.
__device__ __forceinline__ void tile_coords(uint32_t tile, uint32_t m_tiles, uint32_t n_tiles, uint32_t group_m, uint32_t &tile_m, uint32_t &tile_n) {
    const uint32_t per_group = group_m * n_tiles, group = tile / per_group, r = tile - group * per_group;
    const uint32_t gm = min(group_m, m_tiles - group * group_m); // the last group may be short
    tile_n = r / gm;
    tile_m = group * group_m + (r - tile_n * gm);
}

// Scale-factor chunk: 32 rows x 16 bytes, unswizzled, 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t scale_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)(128 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

__device__ __forceinline__ void tmem_cp_scales(uint32_t tmem_addr, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(desc) : "memory");
}
__device__ __forceinline__ void mma_nvf4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}
// The same two, issued by the elected lane of a warp that runs its role converged (tcgen05.cuh).
__device__ __forceinline__ void tmem_cp_scales_elect(uint32_t tmem_addr, uint64_t desc) {
    asm volatile("{\n\t" MUSER_ELECT_PRED "@e tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;\n\t}" ::"r"(tmem_addr), "l"(desc) : "memory");
}
__device__ __forceinline__ void mma_nvf4_elect(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t" MUSER_ELECT_PRED
        "setp.ne.b32 p, %4, 0;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}
// One 32-column strip of one accumulator row: scale, fuse, convert, store (16-byte stores when the row allows).
template <typename T>
__device__ __forceinline__ void store_strip(const float (&v)[32], T *y, const T *res, uint32_t valid, bool vec_ok) {
    if constexpr (sizeof(T) == 4) {
        if (vec_ok && valid == 32) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                float4 q = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                if (res) {
                    const float4 r = *reinterpret_cast<const float4 *>(res + i);
                    q.x += r.x, q.y += r.y, q.z += r.z, q.w += r.w;
                }
                *reinterpret_cast<float4 *>(y + i) = q;
            }
            return;
        }
#pragma unroll
        for (uint32_t i = 0; i < 32; ++i) // (unrolled with a predicate: a run-time index would push v[] out of registers)
            if (i < valid) y[i] = v[i] + (res ? res[i] : 0.0f);
    } else {
        auto to_f = [](T h) { if constexpr (std::is_same<T, __half>::value) return __half2float(h); else return __bfloat162float(h); };
        auto pack = [](float a, float b) -> uint32_t {
            if constexpr (std::is_same<T, __half>::value) {
                const __half2 h = __floats2half2_rn(a, b);
                return *reinterpret_cast<const uint32_t *>(&h);
            } else {
                const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                return *reinterpret_cast<const uint32_t *>(&h);
            }
        };
        if (vec_ok && valid == 32) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
                float f[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) f[k] = v[i + k];
                if (res) {
                    const uint4 r = *reinterpret_cast<const uint4 *>(res + i);
                    const T *rt = reinterpret_cast<const T *>(&r);
#pragma unroll
                    for (int k = 0; k < 8; ++k) f[k] += to_f(rt[k]);
                }
                *reinterpret_cast<uint4 *>(y + i) = make_uint4(pack(f[0], f[1]), pack(f[2], f[3]), pack(f[4], f[5]), pack(f[6], f[7]));
            }
            return;
        }
#pragma unroll
        for (uint32_t i = 0; i < 32; ++i) {
            if (i >= valid) continue;
            const float f = v[i] + (res ? to_f(res[i]) : 0.0f);
            if constexpr (std::is_same<T, __half>::value) y[i] = __float2half_rn(f); else y[i] = __float2bfloat16_rn(f);
        }
    }
}

// Persistent: CTA b takes output tiles b, b + gridDim.x, ...; tile index -> (n tile, m tile) with m fastest, so the
// CTAs that run side by side share one weight tile (read from HBM once, from L2 afterwards).
//
// DUAL is the fused FFN front half (reference: encode_ffn_q4k_gate_up_silu_4r2s, src/metal/encode/ffn.rs:10-36, and
// reference.rs:511-513 on the CPU lane): the 256 accumulator columns of a tile are 128 rows of the gate weight next to
// the same 128 rows of the up weight (map_b, map_b2: 128-row boxes), and the epilogue writes silu_fast(gate) * up,
// each factor first rounded to f16 as the unfused W4A4 lane returns it (quant/nvfp4.rs:337).
// TAIL compiles the LM-head tail (logit scale, tanh soft cap) into the epilogue; the common instantiation has none of it.
// QOUT (with DUAL): silu(gate) * up is not stored but quantized on the spot for the down projection, exactly as
// quant::quantize_nvfp4_activation would quantize the f32 product (quant/nvfp4.rs:173-238): a thread holds 64
// consecutive outputs of its token, i.e. four 16-value groups = one chunk of the swizzled scale plane, and writes
// 32 bytes of codes and one word of scales.  The 27648-wide intermediate is never written or read as numbers.
// GROUP: several projections that read the same quantized activations (q | k | v) share one launch: their weight-row
// tiles form one tile space, so the small ones fill the SMs that a launch of their own would leave idle.  Plain
// outputs only (no fused tail, row scale or residual).
template <bool DUAL, bool TAIL, bool QOUT = false, bool GROUP = false>
__global__ void __launch_bounds__(352, 1)
nvfp4_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  const __grid_constant__ CUtensorMap map_b2, const __grid_constant__ CUtensorMap map_b3,
                  const __grid_constant__ CUtensorMap map_b4, const GemmArgs g) {
    constexpr uint32_t kTileRows = DUAL ? BN / 2 : BN; // output columns (weight rows) per tile
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u; // swizzled tiles need 1024-byte alignment
    uint8_t *aligned = smem_raw + (base - smem_u32(smem_raw));
    uint64_t *bars = reinterpret_cast<uint64_t *>(aligned + kStages * kStageBytes);
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + kStages);
    const uint32_t bar_acc_full = smem_u32(bars + 2 * kStages), bar_acc_empty = smem_u32(bars + 2 * kStages + 1);
    const uint32_t bar_sf_full = smem_u32(bars + 2 * kStages + 2), bar_sf_empty = smem_u32(bars + 2 * kStages + 2 + kSfBufs);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kStages + 2 + 2 * kSfBufs);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t m_tiles = (g.tokens + BM - 1) / BM, n_tiles_total = g.n_tiles * m_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_acc_full, 1);
        mbar_init(bar_acc_empty, 8); // one arrival per epilogue warp
        for (int b = 0; b < (int)kSfBufs; ++b) {
            mbar_init(bar_sf_full + 8 * b, 1);
            mbar_init(bar_sf_empty + 8 * b, 1);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer (whole warp; one elected lane issues)
        {
            uint32_t it = 0, issued = 0; // k slabs issued so far, over all tiles
            bool ok = true; PROF_DECL
            for (uint32_t tile = blockIdx.x; tile < n_tiles_total && ok; tile += gridDim.x) {
                uint32_t tile_m, tile_n;
                tile_coords(tile, m_tiles, g.n_tiles, g.group_m, tile_m, tile_n);
                const uint8_t *b_scales = g.b_scales;
                const CUtensorMap *mb = &map_b;
                if constexpr (GROUP) {
                    const uint32_t p = (tile_n >= g.grp_tile0[1]) + (tile_n >= g.grp_tile0[2]) + (tile_n >= g.grp_tile0[3]);
                    tile_n -= g.grp_tile0[p];
                    b_scales = g.grp_b_scales[p];
                    mb = p == 0 ? &map_b : p == 1 ? &map_b2 : p == 2 ? &map_b3 : &map_b4;
                }
                const uint8_t *sfa = g.a_scales + (size_t)tile_m * g.kt64 * 512;
                const uint8_t *sfb0 = b_scales + (size_t)(DUAL ? tile_n : 2 * tile_n) * g.kt64 * 512;
                const uint8_t *sfb1 = DUAL ? g.b2_scales + (size_t)tile_n * g.kt64 * 512 : sfb0 + (size_t)g.kt64 * 512;
                for (uint32_t kt = 0; kt < g.k_tiles; ++kt, ++it) {
                    const uint32_t s = it % kStages, round = it / kStages;
                    PROF_BEGIN if (round > 0) ok = mbar_wait_warp(bar_empty + 8 * s, (round - 1) & 1, abort_flag); PROF_END(0)
                    if (!ok) break;
                    const uint32_t st = base + s * kStageBytes;
                    const uint32_t full = bar_full + 8 * s;
                    // the last slab may hold fewer than four 64-value blocks: the operand boxes are zero-filled
                    // past the row end, and only the scale chunks that exist are fetched
                    const uint32_t nkb = min(4u, g.kt64 - 4 * kt), sf_bytes = nkb * 512;
                    mbar_expect_tx_elect(full, kABytes + kBBytes + 3 * sf_bytes);
                    tma_load_2d_elect(st, &map_a, (int)(kt * (BK / 2)), (int)(tile_m * BM), full);
                    if constexpr (DUAL) {
                        tma_load_2d_elect(st + kABytes, &map_b, (int)(kt * (BK / 2)), (int)(tile_n * kTileRows), full);
                        tma_load_2d_elect(st + kABytes + kBBytes / 2, &map_b2, (int)(kt * (BK / 2)), (int)(tile_n * kTileRows), full);
                    } else {
                        tma_load_2d_elect(st + kABytes, mb, (int)(kt * (BK / 2)), (int)(tile_n * BN), full);
                    }
                    bulk_load_elect(st + kABytes + kBBytes, sfa + (size_t)kt * kSfaBytes, sf_bytes, full);
                    bulk_load_elect(st + kABytes + kBBytes + kSfaBytes, sfb0 + (size_t)kt * 2048, sf_bytes, full);
                    bulk_load_elect(st + kABytes + kBBytes + kSfaBytes + 2048, sfb1 + (size_t)kt * 2048, sf_bytes, full);
                    issued = it + 1;
                }
            }
            if (lane == 0) { PROF_FLUSH(0) }
            if (!ok) {
                if (lane == 0) {
                    *abort_flag = 1;
                    atomicExch(g.status + 1, 101);
                }
                // let the copies already in flight land before the CTA's shared memory goes away
                const uint32_t first = issued > kStages ? issued - kStages : 0;
                for (uint32_t k = first; k < issued; ++k) {
                    uint32_t done = 0;
                    for (uint32_t i = 0; i < kSpinLimit && !done; ++i)
                        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                                     : "=r"(done) : "r"(bar_full + 8 * (k % kStages)), "r"((k / kStages) & 1) : "memory");
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (whole warp; one elected lane issues)
        {
            // kind::mxf4nvf4: A and B E2M1 (format 1), K-major, UE4M3 scales, N >> 3 at bit 17, M >> 4 at bit 24
            const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            uint32_t it = 0, local = 0;
            bool ok = true; PROF_DECL
            for (uint32_t tile = blockIdx.x; tile < n_tiles_total && ok; tile += gridDim.x, ++local) {
                // the accumulator is free again once the epilogue warps have read the previous tile out of it
                if (local > 0) {
                    PROF_BEGIN ok = mbar_wait_warp(bar_acc_empty, (local - 1) & 1, abort_flag); PROF_END(0)
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                }
                for (uint32_t kt = 0; kt < g.k_tiles; ++kt, ++it) {
                    const uint32_t s = it % kStages, round = it / kStages;
                    PROF_BEGIN ok = mbar_wait_warp(bar_full + 8 * s, round & 1, abort_flag); PROF_END(1)
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t st = base + s * kStageBytes;
                    const uint64_t da = operand_desc(st), db = operand_desc(st + kABytes);
                    const uint32_t nkb = min(4u, g.kt64 - 4 * kt);
                    const uint32_t buf = it % kSfBufs, sf = tmem + kSfCol + buf * kSfBufCols;
#ifdef MUSER_GEMM_COPIER_WARP
                    // the scale factors of this slab were copied into tensor memory by the copier warp
                    PROF_BEGIN ok = mbar_wait_warp(bar_sf_full + 8 * buf, (it / kSfBufs) & 1, abort_flag); PROF_END(2)
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    for (uint32_t kb = 0; kb < nkb; ++kb) // 64 values = 32 bytes further along the swizzled 128-byte rows: +2 in 16-byte units
                        mma_nvf4_elect(tmem, da + 2 * kb, db + 2 * kb, idesc, sf + 4 * kb, sf + 16 + 8 * kb, (kt | kb) != 0);
                    mma_commit_elect(bar_sf_empty + 8 * buf);
#else
                    // Each MMA's scale factors go to tensor memory right in front of it, from the same lane: the tensor
                    // pipe takes both in issue order, so no barrier stands between a copy and the MMA that reads it, and
                    // the copies run under the MMAs before them (691 cycles per slab in isolation against 548 for the
                    // MMAs alone).  The buffers alternate so that a copy never lands in what an earlier MMA still reads.
                    const uint32_t sfa = st + kABytes + kBBytes, sfb = sfa + kSfaBytes;
                    for (uint32_t kb = 0; kb < nkb; ++kb) { // 64 values = 32 bytes further along the swizzled 128-byte rows: +2 in 16-byte units
                        tmem_cp_scales_elect(sf + 4 * kb, scale_desc(sfa + 512 * kb));
                        tmem_cp_scales_elect(sf + 16 + 8 * kb, scale_desc(sfb + 512 * kb));
                        tmem_cp_scales_elect(sf + 16 + 8 * kb + 4, scale_desc(sfb + 2048 + 512 * kb));
                        mma_nvf4_elect(tmem, da + 2 * kb, db + 2 * kb, idesc, sf + 4 * kb, sf + 16 + 8 * kb, (kt | kb) != 0);
                    }
#endif
                    mma_commit_elect(bar_empty + 8 * s); // the stage may be overwritten once these MMAs have read it
                }
                if (ok) mma_commit_elect(bar_acc_full);
            }
            if (lane == 0) { PROF_FLUSH(1) }
            if (!ok && lane == 0) {
                *abort_flag = 1;
                atomicExch(g.status + 1, 102);
            }
        }
    } else if (warp == 10) {
#ifdef MUSER_GEMM_COPIER_WARP
        // ---------------------------------------------------------------- scale copier (development alternative)
        // tcgen05.cp of the slab's scale factors into one of the tensor-memory buffers, issued by a warp of its own.
        {
            uint32_t it = 0;
            bool ok = true; PROF_DECL
            for (uint32_t tile = blockIdx.x; tile < n_tiles_total && ok; tile += gridDim.x) {
                for (uint32_t kt = 0; kt < g.k_tiles; ++kt, ++it) {
                    const uint32_t s = it % kStages, round = it / kStages, buf = it % kSfBufs;
                    PROF_BEGIN ok = mbar_wait_warp(bar_full + 8 * s, round & 1, abort_flag); PROF_END(0)
                    PROF_BEGIN if (ok && it >= kSfBufs) ok = mbar_wait_warp(bar_sf_empty + 8 * buf, ((it / kSfBufs) - 1) & 1, abort_flag); PROF_END(1)
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t st = base + s * kStageBytes, sfa = st + kABytes + kBBytes, sfb = sfa + kSfaBytes;
                    const uint32_t sf = tmem + kSfCol + buf * kSfBufCols, nkb = min(4u, g.kt64 - 4 * kt);
                    for (uint32_t kb = 0; kb < nkb; ++kb) {
                        tmem_cp_scales_elect(sf + 4 * kb, scale_desc(sfa + 512 * kb));
                        tmem_cp_scales_elect(sf + 16 + 8 * kb, scale_desc(sfb + 512 * kb));
                        tmem_cp_scales_elect(sf + 16 + 8 * kb + 4, scale_desc(sfb + 2048 + 512 * kb));
                    }
                    mma_commit_elect(bar_sf_full + 8 * buf);
                }
            }
            if (lane == 0) { PROF_FLUSH(2) }
            if (!ok && lane == 0) {
                *abort_flag = 1;
                atomicCAS(g.status + 1, 0, 105);
            }
        }
#endif
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..9)
        // Eight warps: two per 32-lane quarter of the accumulator, one for each half of the tile's output columns.
        // There is room for one accumulator only, so the MMA warp cannot start the next tile before the last
        // tcgen05.ld of this one.
        const uint32_t quad = warp & 3;                 // the 32 accumulator lanes this warp may read
        const uint32_t part = (uint32_t)(warp - 2) >> 2; // which half of the output columns
        constexpr uint32_t kOutCols = DUAL ? BN / 2 : BN, kPartCols = kOutCols / 2;
        uint32_t local = 0;
        for (uint32_t tile = blockIdx.x; tile < n_tiles_total; tile += gridDim.x, ++local) {
            uint32_t tile_m, tile_n;
            tile_coords(tile, m_tiles, g.n_tiles, g.group_m, tile_m, tile_n);
            uint32_t n_out = g.n_out; // (of this tile's projection)
            void *y_out = g.y;
            float scale2 = g.scale2;
            if constexpr (GROUP) {
                const uint32_t p = (tile_n >= g.grp_tile0[1]) + (tile_n >= g.grp_tile0[2]) + (tile_n >= g.grp_tile0[3]);
                tile_n -= g.grp_tile0[p];
                n_out = g.grp_n_out[p], y_out = g.grp_y[p], scale2 = g.grp_scale2[p];
            }
            const bool ok = __all_sync(0xffffffffu, mbar_wait(bar_acc_full, local & 1, abort_flag));
            if (!ok) {
                if (lane == 0) {
                    *abort_flag = 1;
                    atomicCAS(g.status + 1, 0, 103);
                }
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tok = tile_m * BM + quad * 32 + lane;
            const float rs = (g.row_scale && tok < g.tokens) ? g.row_scale[tok] : 1.0f;
            const bool vec_ok = (n_out & 7) == 0;
            const uint32_t lane_base = tmem + ((quad * 32) << 16), col0 = part * kPartCols;
            // All of this warp's part of the accumulator goes to registers first (128 values a thread) and the
            // accumulator is handed back at once: the MMA warp cannot start the next tile before that, so nothing
            // that touches global memory may sit in between.
            uint32_t r[4][32];
#pragma unroll
            for (uint32_t s = 0; s < 4; ++s) // fused form: strips 0, 1 are gate columns, 2, 3 the same columns of up
                tmem_ld32(lane_base + col0 + (DUAL ? (s & 1) * 32 + (s >> 1) * kOutCols : 32 * s), r[s]);
            tmem_ld_wait();
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_acc_empty) : "memory");
            uint32_t q_word = 0; // QOUT: the four scale bytes of this thread's 64 outputs
#pragma unroll
            for (uint32_t s = 0; s < kPartCols / 32; ++s) {
                const uint32_t c0 = col0 + 32 * s;
                uint32_t(&cur)[32] = r[s];
                uint32_t(&r_up)[32] = r[DUAL ? 2 + s : s];
                const uint32_t n0 = tile_n * kOutCols + c0;
                if constexpr (QOUT) {
                    // rows of the last 128-token block that hold no token get zero scale bytes: the next GEMM reads the
                    // block's whole scale chunk (their codes come from TMA's zero fill)
                    if (n0 < n_out) {
                        float v[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float gate = __half2float(__float2half_rn(__fmul_rn(__fmul_rn(__uint_as_float(cur[i]), scale2), g.inv_input_scale)));
                            const float up = __half2float(__float2half_rn(__fmul_rn(__fmul_rn(__uint_as_float(r_up[i]), g.scale2_up), g.inv_input_scale)));
                            v[i] = __fdiv_rn(gate, 1.0f + expf(-gate)) * up;
                        }
                        if (tok < g.tokens) {
                            uint8_t *codes = g.q_packed + (size_t)tok * (n_out / 2) + n0 / 2;
                            float(&lo)[16] = *reinterpret_cast<float(*)[16]>(&v[0]);
                            float(&hi)[16] = *reinterpret_cast<float(*)[16]>(&v[16]);
                            q_word |= quantize_group(lo, g.q_isi, codes) << (16 * s);
                            q_word |= quantize_group(hi, g.q_isi, codes + 8) << (16 * s + 8);
                        }
                    }
                    if (s + 1 == kPartCols / 32 && tile_n * kOutCols + col0 < n_out)
                        *reinterpret_cast<uint32_t *>(g.q_scales + swizzled_scale_offset(tok, (tile_n * kOutCols + col0) / 16, g.q_kt)) = q_word;
                    continue;
                }
                if (tok < g.tokens && n0 < n_out) {
                    const size_t o = (size_t)tok * n_out + n0;
                    const uint32_t valid = min(32u, n_out - n0);
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) { // quant/nvfp4.rs:334-336: tensor scales applied one after the other
                        v[i] = __fmul_rn(__fmul_rn(__uint_as_float(cur[i]), scale2), g.inv_input_scale);
                        if constexpr (DUAL) {
                            const float gate = __half2float(__float2half_rn(v[i]));
                            const float up = __half2float(__float2half_rn(
                                __fmul_rn(__fmul_rn(__uint_as_float(r_up[i]), g.scale2_up), g.inv_input_scale)));
                            v[i] = __fdiv_rn(gate, 1.0f + expf(-gate)) * up; // silu_fast, quant/helpers.rs:72
                        }
                        v[i] *= rs;
                        if constexpr (TAIL) v[i] = logit_tail(v[i], g.out_scale, g.softcap);
                    }
                    if (g.y_dtype == MUSER_DTYPE_F32)
                        store_strip<float>(v, reinterpret_cast<float *>(y_out) + o,
                                           g.residual ? reinterpret_cast<const float *>(g.residual) + o : nullptr, valid, vec_ok);
                    else if (g.y_dtype == MUSER_DTYPE_BF16)
                        store_strip<__nv_bfloat16>(v, reinterpret_cast<__nv_bfloat16 *>(y_out) + o,
                                                   g.residual ? reinterpret_cast<const __nv_bfloat16 *>(g.residual) + o : nullptr, valid, vec_ok);
                    else
                        store_strip<__half>(v, reinterpret_cast<__half *>(y_out) + o,
                                            g.residual ? reinterpret_cast<const __half *>(g.residual) + o : nullptr, valid, vec_ok);
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// ------------------------------------------------------------------------------------------ paired CTAs
// The same GEMM on pairs of SMs (tcgen05 cta_group::2): a cluster of two CTAs owns a 256-token x 256-row output tile,
// each CTA holding 128 of the tokens (its own accumulator, 128 lanes x 256 columns) and HALF of the weight rows of
// every K slab; the tensor cores of the pair read both halves.  Per slab a CTA therefore fetches 16 KiB of
// activations + 16 KiB of weights (+ 6 KiB of scale factors) for the same 128 x 256 x 256 of work that costs the
// single-CTA kernel 48 + 6 KiB: the L2-to-SM traffic, which bounds that kernel, drops by 30 %.
//
// Roles as above, with the pair's hand-offs made of plain cluster instructions (no multicast of any kind):
//   - every CTA loads its own operands (TMA, own mbarrier);
//   - the follower (cluster rank 1) has one thread that waits for each of its stages to land and then arrives on the
//     leader's barrier of that stage (mbarrier.arrive on the mapped address), so one wait in the leader covers the pair;
//   - the leader (rank 0) issues the scale copies and the MMAs for both CTAs; "stage consumed" and "accumulator
//     complete" are committed twice, once to its own barrier and once to the follower's;
//   - the follower's epilogue warps hand the accumulator back by arriving on the leader's barrier.
// All waits are bounded as in the single-CTA kernel; both CTAs meet at a cluster barrier before they free tensor
// memory and leave, so no arrival can reach a CTA that is gone.
constexpr int kPStages = 5;
constexpr int kPBBytes = (BN / 2) * BK / 2; // 16 KiB: this CTA's half of the pair's 256 weight rows
constexpr int kPStageBytes = kABytes + kPBBytes + kSfaBytes + kSfbBytes;
constexpr int kPSmemBytes = kPStages * kPStageBytes + 1024 + 256;
static_assert(kPSmemBytes <= 227 * 1024, "stage ring exceeds the shared memory of one CTA");

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t cta_addr, uint32_t rank) { // shared::cta address -> that CTA's window
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(cta_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// mbar_wait for barriers that the other CTA of the pair arrives on.
__device__ __forceinline__ bool mbar_wait_pair(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    return false;
}
__device__ __forceinline__ void pair_commit(uint32_t cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void pair_cp_scales(uint32_t tmem_addr, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(desc) : "memory");
}
__device__ __forceinline__ void pair_mma_nvf4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}

__device__ __forceinline__ bool mbar_wait_pair_warp(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    return __all_sync(0xffffffffu, mbar_wait_pair(bar, parity, abort_flag));
}
__device__ __forceinline__ void mbar_arrive_cluster_elect(uint32_t cluster_addr) {
    asm volatile("{\n\t" MUSER_ELECT_PRED "@e mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n\t}" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void pair_commit_elect(uint32_t cluster_addr) {
    asm volatile("{\n\t" MUSER_ELECT_PRED "@e tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void pair_cp_scales_elect(uint32_t tmem_addr, uint64_t desc) {
    asm volatile("{\n\t" MUSER_ELECT_PRED "@e tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;\n\t}" ::"r"(tmem_addr), "l"(desc) : "memory");
}
__device__ __forceinline__ void pair_mma_nvf4_elect(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                    uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t" MUSER_ELECT_PRED
        "setp.ne.b32 p, %4, 0;\n\t"
        "@e tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}

template <bool DUAL, bool TAIL>
__global__ void __launch_bounds__(352, 1)
nvfp4_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const __grid_constant__ CUtensorMap map_b2, const GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *aligned = smem_raw + (base - smem_u32(smem_raw));
    uint64_t *bars = reinterpret_cast<uint64_t *>(aligned + kPStages * kPStageBytes);
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + kPStages);
    const uint32_t bar_acc_full = smem_u32(bars + 2 * kPStages), bar_acc_empty = smem_u32(bars + 2 * kPStages + 1);
    const uint32_t bar_sf_full = smem_u32(bars + 2 * kPStages + 2), bar_sf_empty = smem_u32(bars + 2 * kPStages + 2 + kSfBufs);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kPStages + 2 + 2 * kSfBufs);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank(), leader = rank == 0;
    const uint32_t pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const uint32_t m_blocks = (g.tokens + BM - 1) / BM;            // 128-token blocks (the rows of the scale image)
    const uint32_t m_tiles = (m_blocks + 1) / 2, n_tiles_total = g.n_tiles * m_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPStages; ++s) {
            mbar_init(bar_full + 8 * s, leader ? 2 : 1); // leader: its own copies and the follower's "landed"
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_acc_full, 1);
        mbar_init(bar_acc_empty, 16); // one arrival per epilogue warp of the pair (used in the leader)
        for (int b = 0; b < (int)kSfBufs; ++b) {
            mbar_init(bar_sf_full + 8 * b, 1);
            mbar_init(bar_sf_empty + 8 * b, 1);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    cluster_barrier(); // both CTAs' barriers exist before anything arrives on them
    if (warp == 1) {   // one warp of EACH CTA of the pair takes part in the paired allocation
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer (both CTAs; whole warp, one elected lane issues)
        {
            uint32_t it = 0, issued = 0;
            bool ok = true; PROF_DECL
            for (uint32_t tile = pair; tile < n_tiles_total && ok; tile += pairs) {
                const uint32_t tile_m = tile % m_tiles, tile_n = tile / m_tiles;
                const uint32_t m_block = 2 * tile_m + rank;
                // a follower whose 128 tokens do not exist reads zero-filled activation boxes; its scale chunks
                // come from block 0 so that the copy stays inside the scale image (the products are zero anyway)
                const uint8_t *sfa = g.a_scales + (size_t)(m_block < m_blocks ? m_block : 0) * g.kt64 * 512;
                const uint8_t *sfb0 = g.b_scales + (size_t)(DUAL ? tile_n : 2 * tile_n) * g.kt64 * 512;
                const uint8_t *sfb1 = DUAL ? g.b2_scales + (size_t)tile_n * g.kt64 * 512 : sfb0 + (size_t)g.kt64 * 512;
                // this CTA's half of the weight rows: the leader takes rows 0..127 of the tile (the gate rows of the
                // fused form), the follower rows 128..255 (the up rows)
                const CUtensorMap *mb = (DUAL && rank) ? &map_b2 : &map_b;
                const int b_row = DUAL ? (int)(tile_n * (BN / 2)) : (int)(tile_n * BN + rank * (BN / 2));
                for (uint32_t kt = 0; kt < g.k_tiles; ++kt, ++it) {
                    const uint32_t s = it % kPStages, round = it / kPStages;
                    PROF_BEGIN if (round > 0) ok = mbar_wait_pair_warp(bar_empty + 8 * s, (round - 1) & 1, abort_flag); PROF_END(0)
                    if (!ok) break;
                    const uint32_t st = base + s * kPStageBytes;
                    const uint32_t full = bar_full + 8 * s;
                    const uint32_t nkb = min(4u, g.kt64 - 4 * kt), sf_bytes = nkb * 512;
                    mbar_expect_tx_elect(full, kABytes + kPBBytes + 3 * sf_bytes);
                    tma_load_2d_elect(st, &map_a, (int)(kt * (BK / 2)), (int)(m_block * BM), full);
                    tma_load_2d_elect(st + kABytes, mb, (int)(kt * (BK / 2)), b_row, full);
                    bulk_load_elect(st + kABytes + kPBBytes, sfa + (size_t)kt * kSfaBytes, sf_bytes, full);
                    bulk_load_elect(st + kABytes + kPBBytes + kSfaBytes, sfb0 + (size_t)kt * 2048, sf_bytes, full);
                    bulk_load_elect(st + kABytes + kPBBytes + kSfaBytes + 2048, sfb1 + (size_t)kt * 2048, sf_bytes, full);
                    issued = it + 1;
                }
            }
            if (lane == 0) { PROF_FLUSH(0) }
            if (!ok) {
                if (lane == 0) {
                    *abort_flag = 1;
                    atomicCAS(g.status + 1, 0, 111);
                }
                // let the copies already in flight land before the CTA's shared memory goes away (bounded: the
                // leader's phases also need the follower's arrival)
                const uint32_t first = issued > (uint32_t)kPStages ? issued - kPStages : 0;
                for (uint32_t k = first; k < issued; ++k) mbar_wait_alone(bar_full + 8 * (k % kPStages), (k / kPStages) & 1);
            }
        }
    } else if (warp == 1) {
        if (leader) {
            // ---------------------------------------------------------------- MMA issuer (leader, for the pair; whole warp)
            // M = 256 (128 rows in each CTA), N = 256: N >> 3 at bit 17, M >> 4 at bit 24
            const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
            const uint32_t peer_empty = map_to_rank(bar_empty, 1), peer_acc_full = map_to_rank(bar_acc_full, 1);
            uint32_t it = 0, local = 0;
            bool ok = true; PROF_DECL
            for (uint32_t tile = pair; tile < n_tiles_total && ok; tile += pairs, ++local) {
                if (local > 0) {
                    PROF_BEGIN ok = mbar_wait_pair_warp(bar_acc_empty, (local - 1) & 1, abort_flag); PROF_END(0)
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                }
                for (uint32_t kt = 0; kt < g.k_tiles; ++kt, ++it) {
                    const uint32_t s = it % kPStages, round = it / kPStages;
                    PROF_BEGIN ok = mbar_wait_pair_warp(bar_full + 8 * s, round & 1, abort_flag); PROF_END(1)
                    if (!ok) break;
                    const uint32_t st = base + s * kPStageBytes;
                    const uint64_t da = operand_desc(st), db = operand_desc(st + kABytes);
                    const uint32_t nkb = min(4u, g.kt64 - 4 * kt);
                    const uint32_t buf = it % kSfBufs, sf = tmem + kSfCol + buf * kSfBufCols;
                    PROF_BEGIN ok = mbar_wait_warp(bar_sf_full + 8 * buf, (it / kSfBufs) & 1, abort_flag); PROF_END(2)
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    for (uint32_t kb = 0; kb < nkb; ++kb)
                        pair_mma_nvf4_elect(tmem, da + 2 * kb, db + 2 * kb, idesc, sf + 4 * kb, sf + 16 + 8 * kb, (kt | kb) != 0);
                    pair_commit_elect(bar_sf_empty + 8 * buf);
                    pair_commit_elect(bar_empty + 8 * s);   // both CTAs may overwrite the stage once these MMAs have read it
                    pair_commit_elect(peer_empty + 8 * s);
                }
                if (ok) {
                    pair_commit_elect(bar_acc_full);
                    pair_commit_elect(peer_acc_full);
                }
            }
            if (lane == 0) { PROF_FLUSH(1) }
            if (!ok && lane == 0) {
                *abort_flag = 1;
                atomicCAS(g.status + 1, 0, 112);
            }
        } else {
            // ---------------------------------------------------------------- follower: "my stage has landed"
            const uint32_t leader_full = map_to_rank(bar_full, 0);
            uint32_t it = 0;
            bool ok = true; PROF_DECL
            for (uint32_t tile = pair; tile < n_tiles_total && ok; tile += pairs) {
                for (uint32_t kt = 0; kt < g.k_tiles; ++kt, ++it) {
                    const uint32_t s = it % kPStages, round = it / kPStages;
                    PROF_BEGIN ok = mbar_wait_warp(bar_full + 8 * s, round & 1, abort_flag); PROF_END(0)
                    if (!ok) break;
                    mbar_arrive_cluster_elect(leader_full + 8 * s);
                }
            }
            if (lane == 0) { PROF_FLUSH(3) }
            if (!ok && lane == 0) {
                *abort_flag = 1;
                atomicCAS(g.status + 1, 0, 116);
            }
        }
    } else if (warp == 10) {
        // ---------------------------------------------------------------- scale copier (leader, for the pair)
        if (leader) { // whole warp
            uint32_t it = 0;
            bool ok = true; PROF_DECL
            for (uint32_t tile = pair; tile < n_tiles_total && ok; tile += pairs) {
                for (uint32_t kt = 0; kt < g.k_tiles; ++kt, ++it) {
                    const uint32_t s = it % kPStages, round = it / kPStages, buf = it % kSfBufs;
                    PROF_BEGIN ok = mbar_wait_pair_warp(bar_full + 8 * s, round & 1, abort_flag); PROF_END(0)
                    PROF_BEGIN if (ok && it >= kSfBufs) ok = mbar_wait_warp(bar_sf_empty + 8 * buf, ((it / kSfBufs) - 1) & 1, abort_flag); PROF_END(1)
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t st = base + s * kPStageBytes, sfa = st + kABytes + kPBBytes, sfb = sfa + kSfaBytes;
                    const uint32_t sf = tmem + kSfCol + buf * kSfBufCols, nkb = min(4u, g.kt64 - 4 * kt);
                    for (uint32_t kb = 0; kb < nkb; ++kb) { // each CTA copies from its own shared memory into its own tensor memory
                        pair_cp_scales_elect(sf + 4 * kb, scale_desc(sfa + 512 * kb));
                        pair_cp_scales_elect(sf + 16 + 8 * kb, scale_desc(sfb + 512 * kb));
                        pair_cp_scales_elect(sf + 16 + 8 * kb + 4, scale_desc(sfb + 2048 + 512 * kb));
                    }
                    pair_commit_elect(bar_sf_full + 8 * buf);
                }
            }
            if (lane == 0) { PROF_FLUSH(2) }
            if (!ok && lane == 0) {
                *abort_flag = 1;
                atomicCAS(g.status + 1, 0, 115);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..9 of both CTAs)
        const uint32_t quad = warp & 3;
        const uint32_t part = (uint32_t)(warp - 2) >> 2;
        constexpr uint32_t kOutCols = DUAL ? BN / 2 : BN, kPartCols = kOutCols / 2;
        const uint32_t leader_acc_empty = map_to_rank(bar_acc_empty, 0);
        uint32_t local = 0;
        for (uint32_t tile = pair; tile < n_tiles_total; tile += pairs, ++local) {
            const uint32_t tile_m = tile % m_tiles, tile_n = tile / m_tiles;
            const bool ok = __all_sync(0xffffffffu, mbar_wait_pair(bar_acc_full, local & 1, abort_flag));
            if (!ok) {
                if (lane == 0) {
                    *abort_flag = 1;
                    atomicCAS(g.status + 1, 0, 113);
                }
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tok = (2 * tile_m + rank) * BM + quad * 32 + lane;
            const float rs = (g.row_scale && tok < g.tokens) ? g.row_scale[tok] : 1.0f;
            const bool vec_ok = (g.n_out & 7) == 0;
            const uint32_t lane_base = tmem + ((quad * 32) << 16), col0 = part * kPartCols;
            uint32_t r[4][32]; // as in the single-CTA kernel: everything to registers, then the accumulator goes back
#pragma unroll
            for (uint32_t s = 0; s < 4; ++s)
                tmem_ld32(lane_base + col0 + (DUAL ? (s & 1) * 32 + (s >> 1) * kOutCols : 32 * s), r[s]);
            tmem_ld_wait();
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_acc_empty);
#pragma unroll
            for (uint32_t s = 0; s < kPartCols / 32; ++s) {
                const uint32_t c0 = col0 + 32 * s;
                uint32_t(&cur)[32] = r[s];
                uint32_t(&r_up)[32] = r[DUAL ? 2 + s : s];
                const uint32_t n0 = tile_n * kOutCols + c0;
                if (tok < g.tokens && n0 < g.n_out) {
                    const size_t o = (size_t)tok * g.n_out + n0;
                    const uint32_t valid = min(32u, g.n_out - n0);
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        v[i] = __fmul_rn(__fmul_rn(__uint_as_float(cur[i]), g.scale2), g.inv_input_scale);
                        if constexpr (DUAL) {
                            const float gate = __half2float(__float2half_rn(v[i]));
                            const float up = __half2float(__float2half_rn(
                                __fmul_rn(__fmul_rn(__uint_as_float(r_up[i]), g.scale2_up), g.inv_input_scale)));
                            v[i] = __fdiv_rn(gate, 1.0f + expf(-gate)) * up;
                        }
                        v[i] *= rs;
                        if constexpr (TAIL) v[i] = logit_tail(v[i], g.out_scale, g.softcap);
                    }
                    if (g.y_dtype == MUSER_DTYPE_F32)
                        store_strip<float>(v, reinterpret_cast<float *>(g.y) + o,
                                           g.residual ? reinterpret_cast<const float *>(g.residual) + o : nullptr, valid, vec_ok);
                    else if (g.y_dtype == MUSER_DTYPE_BF16)
                        store_strip<__nv_bfloat16>(v, reinterpret_cast<__nv_bfloat16 *>(g.y) + o,
                                                   g.residual ? reinterpret_cast<const __nv_bfloat16 *>(g.residual) + o : nullptr, valid, vec_ok);
                    else
                        store_strip<__half>(v, reinterpret_cast<__half *>(g.y) + o,
                                            g.residual ? reinterpret_cast<const __half *>(g.residual) + o : nullptr, valid, vec_ok);
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_barrier(); // nothing of the pair is in flight towards this CTA any more
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// Tensor-pipe ceiling for this instruction: every SM issues `iters` x 4 block-scaled FP4 MMAs (128 x 256 x 64 each)
// on whatever its shared and tensor memory hold, with no loads, no scale copies and no epilogue.  The time of this
// kernel is the denominator for the GEMM's roofline fraction.
__global__ void __launch_bounds__(192, 1) nvfp4_peak_kernel(uint32_t iters, int *status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *aligned = smem_raw + (base - smem_u32(smem_raw));
    uint64_t *bars = reinterpret_cast<uint64_t *>(aligned + kStageBytes);
    const uint32_t bar_done = smem_u32(bars);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (uint32_t i = threadIdx.x; i < kStageBytes / 16; i += blockDim.x) reinterpret_cast<uint4 *>(aligned)[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) {
        mbar_init(bar_done, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    if (warp == 1) { // whole warp, one elected lane issues
        const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
        const uint64_t da = operand_desc(base), db = operand_desc(base + kABytes);
        // scale factors: one copy of zeroed chunks so that the accumulator stays finite
        for (uint32_t kb = 0; kb < 4; ++kb) {
            tmem_cp_scales_elect(tmem + kSfCol + 4 * kb, scale_desc(base + kABytes + kBBytes));
            tmem_cp_scales_elect(tmem + kSfCol + 16 + 8 * kb, scale_desc(base + kABytes + kBBytes));
            tmem_cp_scales_elect(tmem + kSfCol + 16 + 8 * kb + 4, scale_desc(base + kABytes + kBBytes));
        }
        for (uint32_t i = 0; i < iters; ++i)
#pragma unroll
            for (uint32_t kb = 0; kb < 4; ++kb)
                mma_nvf4_elect(tmem, da + 2 * kb, db + 2 * kb, idesc, tmem + kSfCol + 4 * kb, tmem + kSfCol + 16 + 8 * kb, (i | kb) != 0);
        mma_commit_elect(bar_done);
        if (!mbar_wait_warp(bar_done, 0, abort_flag) && lane == 0) atomicExch(status + 1, 104);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
}

// What the tensor pipe and the shared-memory ports do with the GEMM's instruction mix, measured in isolation: one
// thread per SM issues, per iteration (= one 256-value slab of a 128 x 256 tile), the slab's four MMAs and / or its
// scale-factor copies in a chosen order, on resident operands; another thread may stream bulk copies from an
// L2-resident buffer into shared memory beside it, as the GEMM's producer does.
//   mode 0: 4 MMAs                       mode 1: 12 copies (32x128b.warpx4), then 4 MMAs
//   mode 2: (3 copies, 1 MMA) x 4         mode 3: 12 copies only
//   mode 4: 6 copies of 128x256b only     mode 5: 6 copies of 128x256b, then 4 MMAs        mode 6: nothing (loads only)
constexpr int kProbeLoadRing = 6, kProbeLoadChunk = 18 * 1024;
constexpr int kProbeSmemBytes = kStageBytes + 16384 + kProbeLoadRing * kProbeLoadChunk + 2048;
__global__ void __launch_bounds__(192, 1) nvfp4_pipe_probe_kernel(uint32_t mode, uint32_t iters, uint32_t load_chunks, uint32_t random,
                                                                  const uint8_t *src, uint32_t src_chunks, int *status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *aligned = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t scales = base + kABytes + kBBytes, load_base = base + kStageBytes + 16384;
    uint64_t *bars = reinterpret_cast<uint64_t *>(aligned + kStageBytes + 16384 + kProbeLoadRing * kProbeLoadChunk);
    const uint32_t bar_done = smem_u32(bars), bar_load = smem_u32(bars + 1);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 1 + kProbeLoadRing);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (uint32_t i = threadIdx.x; i < (kStageBytes + 16384) / 16; i += blockDim.x) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (random) { // non-zero E2M1 codes; scale bytes 0x30..0x3f (E4M3 0.5 .. 1.9) so that the sums stay finite
            uint32_t h = (i + 1u) * 2654435761u + blockIdx.x * 40503u;
            auto next = [&]() { h ^= h << 13; h ^= h >> 17; h ^= h << 5; return h; };
            v = make_uint4(next(), next(), next(), next());
            if (16 * i >= (uint32_t)(kABytes + kBBytes)) v.x = (v.x & 0x0f0f0f0fu) | 0x30303030u, v.y = (v.y & 0x0f0f0f0fu) | 0x30303030u, v.z = (v.z & 0x0f0f0f0fu) | 0x30303030u, v.w = (v.w & 0x0f0f0f0fu) | 0x30303030u;
        }
        reinterpret_cast<uint4 *>(aligned)[i] = v;
    }
    if (threadIdx.x == 0) {
        mbar_init(bar_done, 1);
        for (int i = 0; i < kProbeLoadRing; ++i) mbar_init(bar_load + 8 * i, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot, sf = tmem + kSfCol, sf2 = sf + kSfBufCols;
    if (warp == 1 && mode != 6) { // whole warp, one elected lane issues: as the GEMM's roles do
        const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
        const uint64_t da = operand_desc(base), db = operand_desc(base + kABytes);
        auto wide_desc = [&](uint32_t a) { // 128 rows x 32 bytes, the two halves of a row 8 KiB apart
            return (uint64_t)((a >> 4) & 0x3FFF) | (uint64_t)(8192 >> 4) << 16 | (uint64_t)(128 >> 4) << 32 | (uint64_t)1 << 46;
        };
        for (uint32_t c = 0; c < 12; ++c) tmem_cp_scales_elect(sf + 4 * c, scale_desc(scales + 512 * c)); // what the MMAs read
        for (uint32_t i = 0; i < iters; ++i) {
            if (mode == 1 || mode == 3)
                for (uint32_t c = 0; c < 12; ++c) tmem_cp_scales_elect(sf2 + 4 * c, scale_desc(scales + 512 * c));
            if (mode == 4 || mode == 5)
                for (uint32_t c = 0; c < 6; ++c) asm volatile("{\n\t" MUSER_ELECT_PRED "@e tcgen05.cp.cta_group::1.128x256b [%0], %1;\n\t}" ::"r"(sf2 + 8 * c), "l"(wide_desc(scales + 2048 * (c % 3))) : "memory");
            if (mode == 2) {
#pragma unroll
                for (uint32_t kb = 0; kb < 4; ++kb) {
                    for (uint32_t c = 0; c < 3; ++c) tmem_cp_scales_elect(sf2 + 4 * (3 * kb + c), scale_desc(scales + 512 * (3 * kb + c)));
                    mma_nvf4_elect(tmem, da + 2 * kb, db + 2 * kb, idesc, sf + 4 * kb, sf + 16 + 8 * kb, (i | kb) != 0);
                }
            } else if (mode == 0 || mode == 1 || mode == 5) {
#pragma unroll
                for (uint32_t kb = 0; kb < 4; ++kb) mma_nvf4_elect(tmem, da + 2 * kb, db + 2 * kb, idesc, sf + 4 * kb, sf + 16 + 8 * kb, (i | kb) != 0);
            }
        }
        mma_commit_elect(bar_done);
        if (!mbar_wait_warp(bar_done, 0, abort_flag) && lane == 0) atomicExch(status + 1, 107);
    }
    if (warp == 0 && load_chunks) {
        uint32_t at = (blockIdx.x * 977u) % src_chunks;
        for (uint32_t it = 0; it < load_chunks + kProbeLoadRing; ++it) {
            const uint32_t slot = it % kProbeLoadRing, bar = bar_load + 8 * slot;
            if (it >= (uint32_t)kProbeLoadRing && !mbar_wait_warp(bar, ((it / kProbeLoadRing) - 1) & 1, abort_flag)) {
                if (lane == 0) atomicExch(status + 1, 108);
                break;
            }
            if (it < load_chunks) {
                mbar_expect_tx_elect(bar, kProbeLoadChunk);
                bulk_load_elect(load_base + slot * kProbeLoadChunk, src + (size_t)at * kProbeLoadChunk, kProbeLoadChunk, bar);
                at = (at + 149u) % src_chunks;
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
}

muser_cuda_status launch_nvfp4_pipe_probe(Ctx *ctx, uint32_t mode, uint32_t iters, uint32_t load_kib, uint32_t random, cudaStream_t stream) {
    const uint32_t chunks_per_iter = load_kib / 18, src_chunks = (uint32_t)std::min<size_t>(1024, ctx->workspace_bytes / kProbeLoadChunk);
    if (mode > 6 || load_kib % 18 || (chunks_per_iter && src_chunks < 2))
        return fail(ctx, MUSER_CUDA_BAD_ARG, "pipe probe: mode 0..6, loads in multiples of 18 KiB, and a context workspace of at least 36 KiB to read them from");
    MUSER_CUDA_TRY(ctx, ensure_dynamic_smem(reinterpret_cast<const void *>(nvfp4_pipe_probe_kernel), ctx->device, kProbeSmemBytes));
    nvfp4_pipe_probe_kernel<<<ctx->sm_count, 192, kProbeSmemBytes, stream>>>(mode, iters, chunks_per_iter * iters, random,
                                                                            reinterpret_cast<const uint8_t *>(ctx->workspace), src_chunks, ctx->dev_status);
    MUSER_CUDA_TRY(ctx, cudaGetLastError());
    return MUSER_CUDA_OK;
}

muser_cuda_status launch_nvfp4_peak(Ctx *ctx, uint32_t iters, double *flops, cudaStream_t stream) {
    MUSER_CUDA_TRY(ctx, ensure_dynamic_smem(reinterpret_cast<const void *>(nvfp4_peak_kernel), ctx->device, kStageBytes + 2048));
    nvfp4_peak_kernel<<<ctx->sm_count, 192, kStageBytes + 2048, stream>>>(iters, ctx->dev_status);
    MUSER_CUDA_TRY(ctx, cudaGetLastError());
    *flops = 2.0 * BM * BN * 64 * 4.0 * iters * ctx->sm_count;
    return MUSER_CUDA_OK;
}

// ------------------------------------------------------------------------------------------ host side
#ifdef MUSER_GEMM_WAIT_PROFILE
extern "C" __attribute__((visibility("default"))) int muser_cuda_debug_wait_profile(unsigned long long *out) {
    return (int)cudaMemcpyFromSymbol(out, g_wait_prof, sizeof(g_wait_prof));
}
#endif
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// rows x row_bytes, K contiguous; box = box_rows x box_bytes with the swizzle of the same width, zero fill outside.
bool tma_make_map(CUtensorMap *map, const void *ptr, uint64_t rows, uint64_t row_bytes, uint32_t box_rows, uint32_t box_bytes) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {row_bytes, rows};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {box_bytes, box_rows};
    cuuint32_t elem[2] = {1, 1};
    const CUtensorMapSwizzle sw = box_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                  : box_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                  : box_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(ptr), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
static bool make_map(CUtensorMap *map, const void *ptr, uint64_t rows, uint64_t row_bytes, uint32_t box_rows) {
    return tma_make_map(map, ptr, rows, row_bytes, box_rows, 128);
}

muser_cuda_status nvfp4_build_tensor_map(Ctx *ctx, Weight *w) {
    CUtensorMap *m = new CUtensorMap;
    if (!make_map(m, w->packed, w->n_out_pad, w->n_in / 2, BN)) {
        delete m;
        return fail(ctx, MUSER_CUDA_ERROR, "cuTensorMapEncodeTiled failed for the weight image");
    }
    w->tmap_cache = m;
    CUtensorMap *half = new CUtensorMap; // 128-row boxes, for the fused gate/up form
    if (!make_map(half, w->packed, w->n_out_pad, w->n_in / 2, BN / 2)) {
        delete half;
        return fail(ctx, MUSER_CUDA_ERROR, "cuTensorMapEncodeTiled failed for the weight image (128-row boxes)");
    }
    w->tmap_half = half;
    return MUSER_CUDA_OK;
}

void nvfp4_free_tensor_map(Weight *w) {
    delete reinterpret_cast<CUtensorMap *>(w->tmap_cache);
    delete reinterpret_cast<CUtensorMap *>(w->tmap_half);
    w->tmap_cache = nullptr;
    w->tmap_half = nullptr;
}

muser_cuda_status launch_nvfp4_gemm(Ctx *ctx, const Weight *w, const uint8_t *x_packed, const uint8_t *x_scales, void *y,
                                    uint32_t y_dtype, uint32_t tokens, const Epilogue &ep, cudaStream_t stream,
                                    const Weight *w_up, const NvFp4Out *qout) {
    CUtensorMap map_a;
    if (!make_map(&map_a, x_packed, tokens, w->n_in / 2, BM))
        return fail(ctx, MUSER_CUDA_ERROR, "cuTensorMapEncodeTiled failed for the activations");
    GemmArgs g;
    g.a_scales = x_scales;
    g.b_scales = w->scales;
    g.b2_scales = w_up ? w_up->scales : nullptr;
    g.y = y;
    g.row_scale = ep.row_scale;
    g.out_scale = ep.out_scale;
    g.softcap = ep.softcap;
    g.residual = ep.residual;
    g.status = ctx->dev_status;
    g.tokens = tokens;
    g.n_out = (uint32_t)w->n_out;
    g.k_tiles = (uint32_t)((w->n_in + BK - 1) / BK);
    g.kt64 = (uint32_t)(w->n_in / 64);
    g.y_dtype = y_dtype;
    g.scale2 = w->scale2;
    g.scale2_up = w_up ? w_up->scale2 : 0.0f;
    g.inv_input_scale = 1.0f / w->input_scale_inv;
    g.n_tiles = w_up ? (uint32_t)((w->n_out + BN / 2 - 1) / (BN / 2)) : (uint32_t)(w->n_out_pad / BN);
    g.q_packed = qout ? qout->packed : nullptr;
    g.q_scales = qout ? qout->scales : nullptr;
    g.q_isi = qout ? qout->input_scale_inv : 0.0f;
    g.q_kt = (uint32_t)(w->n_out / 64);
    {   // raster groups of about 32 MB of activations (at least 8 token tiles)
        const uint64_t tile_bytes = (uint64_t)BM * (w->n_in / 2 + w->n_in / 16);
        uint32_t gm = (uint32_t)std::max<uint64_t>(8, (32ull << 20) / std::max<uint64_t>(1, tile_bytes));
        if (ctx->nvfp4_group_m) gm = ctx->nvfp4_group_m;
        g.group_m = std::max<uint32_t>(1, std::min<uint32_t>(gm, (tokens + BM - 1) / BM));
    }
    if (qout && (!w_up || w->n_out % 64)) return fail(ctx, MUSER_CUDA_BAD_SHAPE, "quantized outputs come from the fused gate/up form, with n_out % 64 == 0");
    const CUtensorMap &mb = *reinterpret_cast<const CUtensorMap *>(w_up ? w->tmap_half : w->tmap_cache);
    const CUtensorMap &mb2 = w_up ? *reinterpret_cast<const CUtensorMap *>(w_up->tmap_half) : mb;
    const bool tail = ep.out_scale != 1.0f || ep.softcap > 0.0f;
    const uint32_t m_blocks = (tokens + BM - 1) / BM;
    // Pairs of SMs on 256-token tiles are opt-in: the pair halves the operand traffic per SM, but this GEMM is bound
    // by the scale-factor copies into tensor memory, which a pair does not reduce, and the pair's hand-offs cost more
    // than its traffic saves (ffn_gate at 2048 tokens: 2.4 against 2.8 PFLOP/s).
    const bool pair = ctx->nvfp4_pair == 1 && !qout;
    if (pair) {
        struct PairLimit { int n[3] = {0, 0, 0}; };
        static PerDevice<PairLimit> max_pairs; // co-resident clusters of two, asked once per device and kernel
        const void *kfn = w_up ? reinterpret_cast<const void *>(nvfp4_gemm_pair_kernel<true, false>)
                          : tail ? reinterpret_cast<const void *>(nvfp4_gemm_pair_kernel<false, true>)
                                 : reinterpret_cast<const void *>(nvfp4_gemm_pair_kernel<false, false>);
        MUSER_CUDA_TRY(ctx, ensure_dynamic_smem(kfn, ctx->device, kPSmemBytes));
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
        cfg.blockDim = dim3(352), cfg.dynamicSmemBytes = kPSmemBytes, cfg.stream = stream, cfg.attrs = attr, cfg.numAttrs = 1;
        int cached;
        {
            std::lock_guard<std::mutex> lock(max_pairs.mu);
            int &slot = max_pairs.slot[ctx->device].n[w_up ? 1 : tail ? 2 : 0];
            if (slot == 0) {
                cfg.gridDim = dim3(2 * (ctx->sm_count / 2));
                int n = 0;
                MUSER_CUDA_TRY(ctx, cudaOccupancyMaxActiveClusters(&n, kfn, &cfg));
                if (n < 1) return fail(ctx, MUSER_CUDA_ERROR, "no cluster of two CTAs of the paired NVFP4 GEMM fits on this device");
                slot = n;
            }
            cached = slot;
        }
        const uint32_t pair_tiles = g.n_tiles * ((m_blocks + 1) / 2);
        const uint32_t pairs = std::min<uint32_t>(pair_tiles, std::min<uint32_t>((uint32_t)cached, (uint32_t)ctx->sm_count / 2));
        cfg.gridDim = dim3(2 * pairs);
        // every CTA of a pair fetches 128 weight rows per slab: the maps with 128-row boxes, in both forms
        const CUtensorMap &half = *reinterpret_cast<const CUtensorMap *>(w->tmap_half);
        const CUtensorMap &half_up = w_up ? *reinterpret_cast<const CUtensorMap *>(w_up->tmap_half) : half;
        if (w_up)
            MUSER_CUDA_TRY(ctx, cudaLaunchKernelEx(&cfg, nvfp4_gemm_pair_kernel<true, false>, map_a, half, half_up, g));
        else if (tail)
            MUSER_CUDA_TRY(ctx, cudaLaunchKernelEx(&cfg, nvfp4_gemm_pair_kernel<false, true>, map_a, half, half_up, g));
        else
            MUSER_CUDA_TRY(ctx, cudaLaunchKernelEx(&cfg, nvfp4_gemm_pair_kernel<false, false>, map_a, half, half_up, g));
        return MUSER_CUDA_OK;
    }
    const uint32_t tiles = g.n_tiles * m_blocks;
    const uint32_t grid = tiles < (uint32_t)ctx->sm_count ? tiles : (uint32_t)ctx->sm_count;
    // (the attribute is per device: set where the launch happens, with the launching context's device current)
    const void *kfn = w_up ? reinterpret_cast<const void *>(nvfp4_gemm_kernel<true, false>)
                      : tail ? reinterpret_cast<const void *>(nvfp4_gemm_kernel<false, true>)
                             : reinterpret_cast<const void *>(nvfp4_gemm_kernel<false, false>);
    MUSER_CUDA_TRY(ctx, ensure_dynamic_smem(kfn, ctx->device, kSmemBytes));
    if (qout) {
        const void *qfn = reinterpret_cast<const void *>(nvfp4_gemm_kernel<true, false, true>);
        MUSER_CUDA_TRY(ctx, ensure_dynamic_smem(qfn, ctx->device, kSmemBytes));
        nvfp4_gemm_kernel<true, false, true><<<grid, 352, kSmemBytes, stream>>>(map_a, mb, mb2, mb, mb, g);
    } else if (w_up)
        nvfp4_gemm_kernel<true, false><<<grid, 352, kSmemBytes, stream>>>(map_a, mb, mb2, mb, mb, g); // (the fused FFN form has no tail)
    else if (tail)
        nvfp4_gemm_kernel<false, true><<<grid, 352, kSmemBytes, stream>>>(map_a, mb, mb2, mb, mb, g);
    else
        nvfp4_gemm_kernel<false, false><<<grid, 352, kSmemBytes, stream>>>(map_a, mb, mb2, mb, mb, g);
    MUSER_CUDA_TRY(ctx, cudaGetLastError());
    return MUSER_CUDA_OK;
}

// Up to four projections of the same quantized activations in one launch (GROUP form of the kernel).
muser_cuda_status launch_nvfp4_gemm_group(Ctx *ctx, const Weight *const *ws, uint32_t n, const uint8_t *x_packed, const uint8_t *x_scales,
                                          void *const *ys, uint32_t y_dtype, uint32_t tokens, cudaStream_t stream) {
    const Weight *w0 = ws[0];
    CUtensorMap map_a;
    if (!make_map(&map_a, x_packed, tokens, w0->n_in / 2, BM))
        return fail(ctx, MUSER_CUDA_ERROR, "cuTensorMapEncodeTiled failed for the activations");
    GemmArgs g = {};
    g.a_scales = x_scales;
    g.status = ctx->dev_status;
    g.tokens = tokens;
    g.k_tiles = (uint32_t)((w0->n_in + BK - 1) / BK);
    g.kt64 = (uint32_t)(w0->n_in / 64);
    g.y_dtype = y_dtype;
    g.out_scale = 1.0f;
    g.inv_input_scale = 1.0f / w0->input_scale_inv;
    uint32_t tiles_n = 0;
    for (uint32_t p = 0; p < 4; ++p) {
        g.grp_tile0[p] = tiles_n;
        if (p >= n) continue;
        g.grp_b_scales[p] = ws[p]->scales;
        g.grp_y[p] = ys[p];
        g.grp_n_out[p] = (uint32_t)ws[p]->n_out;
        g.grp_scale2[p] = ws[p]->scale2;
        tiles_n += (uint32_t)(ws[p]->n_out_pad / BN);
    }
    g.grp_tile0[4] = tiles_n;
    for (uint32_t p = n; p < 4; ++p) g.grp_tile0[p] = tiles_n; // no tile falls into a projection that is not there
    g.n_tiles = tiles_n;
    g.n_out = g.grp_n_out[0], g.y = g.grp_y[0], g.scale2 = g.grp_scale2[0], g.b_scales = g.grp_b_scales[0];
    {
        const uint64_t tile_bytes = (uint64_t)BM * (w0->n_in / 2 + w0->n_in / 16);
        uint32_t gm = (uint32_t)std::max<uint64_t>(8, (32ull << 20) / std::max<uint64_t>(1, tile_bytes));
        if (ctx->nvfp4_group_m) gm = ctx->nvfp4_group_m;
        g.group_m = std::max<uint32_t>(1, std::min<uint32_t>(gm, (tokens + BM - 1) / BM));
    }
    const CUtensorMap *maps[4];
    for (uint32_t p = 0; p < 4; ++p) maps[p] = reinterpret_cast<const CUtensorMap *>(ws[p < n ? p : 0]->tmap_cache);
    const uint32_t tiles = tiles_n * ((tokens + BM - 1) / BM);
    const uint32_t grid = tiles < (uint32_t)ctx->sm_count ? tiles : (uint32_t)ctx->sm_count;
    const void *kfn = reinterpret_cast<const void *>(nvfp4_gemm_kernel<false, false, false, true>);
    MUSER_CUDA_TRY(ctx, ensure_dynamic_smem(kfn, ctx->device, kSmemBytes));
    nvfp4_gemm_kernel<false, false, false, true><<<grid, 352, kSmemBytes, stream>>>(map_a, *maps[0], *maps[1], *maps[2], *maps[3], g);
    MUSER_CUDA_TRY(ctx, cudaGetLastError());
    return MUSER_CUDA_OK;
}

} // namespace muser
