// Weight-loader repack: GGUF K-quant rows and NVFP4 tensors -> the tiled device images the
// kernels read, plus the decoders that turn an image back into f32 (the bit-exact gate).
//
// Block formats follow the reference decoders: Q4_K crates/muser-engine/src/quant/k_block.rs:12-49,
// Q6_K src/quant/k_block/q6.rs:264-325, NVFP4 src/quant/nvfp4.rs:240-255.
#include "common.cuh"
#include "kquant_layout.cuh"

namespace muser {

// ------------------------------------------------------------------------------ K-quant repack
// One thread builds one 32-bit word of a quant plane (8 weights of one row), or one scale header.
__device__ __forceinline__ uint32_t q6_raw_value(const uint8_t *blk, uint32_t e, uint32_t *lo, uint32_t *hi2) {
    uint32_t h = e >> 7, r = e & 127, c = r >> 5, l = r & 31;
    *lo = (blk[64 * h + 32 * (c & 1) + l] >> (4 * (c >> 1))) & 15u;
    *hi2 = (blk[128 + 32 * h + l] >> (2 * c)) & 3u;
    return *lo | (*hi2 << 4);
}

// Tile layout: kquant_layout.cuh (a lane owns a quarter of every sub-block of its two rows).
// Q4_K and Q5_K share everything but the fifth-bit plane (Q5 blocks: d, dmin, scales[12], qh[32], qs[128];
// element e's fifth bit is bit e / 32 of qh[e % 32], quant/k_block.rs:61-105).
template <bool Q5>
__global__ void repack_q4k_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ image, KqGeom gm) {
    constexpr uint32_t kBlock = Q5 ? 176 : 144, kQsOff = Q5 ? 48 : 16, kTile = Q5 ? kQ5TileBytes : kQ4TileBytes, kHdrOff = Q5 ? kQ5OffHdr : 2048;
    const uint64_t units_per_tile = 512 + 16 + (Q5 ? 128 : 0);
    uint64_t idx = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
    if (idx >= (uint64_t)gm.row_tiles * gm.nsb * units_per_tile) return;
    uint64_t tile = idx / units_per_tile;
    uint32_t unit = (uint32_t)(idx % units_per_tile);
    uint32_t rt = (uint32_t)(tile / gm.nsb), sb = (uint32_t)(tile % gm.nsb);
    uint8_t *tile_ptr = image + tile * kTile;
    uint64_t sb_global = gm.k0 / 256 + sb;
    int64_t k_base = (int64_t)sb_global * 256;
    auto in_shard = [&](uint32_t e) {
        int64_t k = k_base + e;
        return k >= (int64_t)gm.k0 && k < (int64_t)(gm.k0 + gm.n_in);
    };
    if (unit < 512) {
        uint32_t u = unit >> 7, lane = (unit >> 2) & 31, jj = unit & 3;
        uint32_t g = lane >> 2, t = lane & 3;
        uint32_t row = rt * 16 + g + 8 * (u >> 1), j = 4 * (u & 1) + jj;
        uint32_t word = 0;
        if (row < gm.n_out) {
            const uint8_t *blk = raw + ((uint64_t)(gm.row0 + row) * gm.blocks_per_row + sb_global) * kBlock;
            for (int i = 0; i < 8; ++i) {
                uint32_t e = 32 * j + 8 * t + i;
                if (!in_shard(e)) continue;
                uint32_t grp = e >> 6, l = e & 63;
                uint8_t byte = blk[kQsOff + 32 * grp + (l & 31)];
                uint32_t nib = l < 32 ? (byte & 15u) : (byte >> 4);
                word |= nib << (4 * q4_nibble_pos(i));
            }
        }
        reinterpret_cast<uint32_t *>(tile_ptr)[(u * 32 + lane) * 4 + jj] = word;
    } else if (Q5 && unit < 512 + 128) { // one word of the fifth-bit plane: (lane, rowsel, half) -> four sub-blocks' bytes
        uint32_t v = unit - 512, lane = v >> 2, wi = v & 3;
        uint32_t g = lane >> 2, t = lane & 3;
        uint32_t row = rt * 16 + g + 8 * (wi >> 1), half = wi & 1;
        uint32_t word = 0;
        if (row < gm.n_out) {
            const uint8_t *blk = raw + ((uint64_t)(gm.row0 + row) * gm.blocks_per_row + sb_global) * kBlock;
            for (uint32_t jj = 0; jj < 4; ++jj) {
                uint32_t j = 4 * half + jj;
                for (uint32_t i = 0; i < 8; ++i) {
                    uint32_t e = 32 * j + 8 * t + i;
                    if (!in_shard(e)) continue;
                    uint32_t bit = (blk[16 + (e & 31)] >> j) & 1u;
                    // element i sits in nibble q4_nibble_pos(i) of the nibble word: byte pos / 2, low or high nibble
                    uint32_t pos = q4_nibble_pos(i), b = pos >> 1, hi = pos & 1;
                    word |= bit << (8 * jj + 4 * hi + b);
                }
            }
        }
        reinterpret_cast<uint32_t *>(tile_ptr + kQ5OffHi)[lane * 4 + wi] = word;
    } else {
        uint32_t r = unit - 512 - (Q5 ? 128 : 0), row = rt * 16 + r;
        uint8_t hdr[16];
        for (int i = 0; i < 16; ++i) hdr[i] = 0;
        if (row < gm.n_out) {
            const uint8_t *blk = raw + ((uint64_t)(gm.row0 + row) * gm.blocks_per_row + sb_global) * kBlock;
            const uint8_t *sp = blk + 4;
            uint8_t sc[8], mn[8];
            for (int j = 0; j < 8; ++j) {
                if (j < 4) {
                    sc[j] = sp[j] & 63;
                    mn[j] = sp[j + 4] & 63;
                } else {
                    sc[j] = (uint8_t)((sp[j + 4] & 15) | ((sp[j - 4] >> 6) << 4));
                    mn[j] = (uint8_t)((sp[j + 4] >> 4) | ((sp[j] >> 6) << 4));
                }
                if (!in_shard(32 * j)) sc[j] = mn[j] = 0; // a sub-block outside the shard contributes nothing
            }
            hdr[0] = blk[0], hdr[1] = blk[1], hdr[2] = blk[2], hdr[3] = blk[3];
            for (int j = 0; j < 4; ++j) {
                hdr[4 + j] = (uint8_t)(sc[j] | ((sc[j + 4] >> 4) << 6));
                hdr[8 + j] = (uint8_t)(mn[j] | ((mn[j + 4] >> 4) << 6));
                hdr[12 + j] = (uint8_t)((sc[j + 4] & 15) | ((mn[j + 4] & 15) << 4));
            }
        }
        uint4 v;
        memcpy(&v, hdr, 16);
        reinterpret_cast<uint4 *>(tile_ptr + kHdrOff)[r] = v;
    }
}

__global__ void repack_q6k_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ image, KqGeom gm) {
    const uint64_t units_per_tile = 512 + 256 + 16 + 1;
    uint64_t idx = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
    if (idx >= (uint64_t)gm.row_tiles * gm.nsb * units_per_tile) return;
    uint64_t tile = idx / units_per_tile;
    uint32_t unit = (uint32_t)(idx % units_per_tile);
    uint32_t rt = (uint32_t)(tile / gm.nsb), sb = (uint32_t)(tile % gm.nsb);
    uint8_t *tile_ptr = image + tile * kQ6TileBytes;
    uint64_t sb_global = gm.k0 / 256 + sb;
    int64_t k_base = (int64_t)sb_global * 256;
    // six-bit two's complement of q - 32 for element e of the block, 0 outside this shard
    auto v6 = [&](const uint8_t *blk, uint32_t e) -> uint32_t {
        int64_t k = k_base + e;
        if (k < (int64_t)gm.k0 || k >= (int64_t)(gm.k0 + gm.n_in)) return 0u;
        uint32_t lo, hi2;
        return q6_raw_value(blk, e, &lo, &hi2) ^ 32u;
    };
    if (unit < 512) { // T plane
        uint32_t u = unit >> 7, lane = (unit >> 2) & 31, wi = unit & 3;
        uint32_t g = lane >> 2, t = lane & 3;
        uint32_t row = rt * 16 + g + 8 * (u >> 1), s0 = 8 * (u & 1) + 2 * wi;
        uint32_t word = 0;
        if (row < gm.n_out) {
            const uint8_t *blk = raw + ((uint64_t)(gm.row0 + row) * gm.blocks_per_row + sb_global) * 210;
            for (uint32_t b = 0; b < 4; ++b) {
                word |= (v6(blk, 16 * s0 + 4 * t + b) >> 2) << (8 * b);
                word |= (v6(blk, 16 * (s0 + 1) + 4 * t + b) >> 2) << (8 * b + 4);
            }
        }
        reinterpret_cast<uint32_t *>(tile_ptr)[(u * 32 + lane) * 4 + wi] = word;
    } else if (unit < 768) { // L plane
        uint32_t v = unit - 512;
        uint32_t rowsel = v >> 7, lane = (v >> 2) & 31, wv = v & 3;
        uint32_t g = lane >> 2, t = lane & 3;
        uint32_t row = rt * 16 + g + 8 * rowsel;
        uint32_t word = 0;
        if (row < gm.n_out) {
            const uint8_t *blk = raw + ((uint64_t)(gm.row0 + row) * gm.blocks_per_row + sb_global) * 210;
            for (uint32_t x = 0; x < 4; ++x)
                for (uint32_t b = 0; b < 4; ++b) word |= (v6(blk, 16 * (4 * wv + x) + 4 * t + b) & 3u) << (8 * b + 2 * x);
        }
        reinterpret_cast<uint32_t *>(tile_ptr + kQ6OffHi)[(rowsel * 32 + lane) * 4 + wv] = word;
    } else if (unit < 784) {
        uint32_t r = unit - 768, row = rt * 16 + r;
        uint8_t sc[16];
        for (int i = 0; i < 16; ++i) sc[i] = 0;
        if (row < gm.n_out) {
            const uint8_t *blk = raw + ((uint64_t)(gm.row0 + row) * gm.blocks_per_row + sb_global) * 210;
            for (uint32_t s2 = 0; s2 < 16; ++s2) {
                int64_t k = k_base + 16 * s2;
                sc[s2] = (k >= (int64_t)gm.k0 && k < (int64_t)(gm.k0 + gm.n_in)) ? blk[192 + s2] : 0;
            }
        }
        uint4 v;
        memcpy(&v, sc, 16);
        reinterpret_cast<uint4 *>(tile_ptr + kQ6OffSc)[r] = v;
    } else {
        for (uint32_t r = 0; r < 16; ++r) {
            uint32_t row = rt * 16 + r;
            uint16_t d = 0;
            if (row < gm.n_out) {
                const uint8_t *blk = raw + ((uint64_t)(gm.row0 + row) * gm.blocks_per_row + sb_global) * 210;
                d = (uint16_t)(blk[208] | (blk[209] << 8));
            }
            reinterpret_cast<uint16_t *>(tile_ptr + kQ6OffD)[r] = d;
        }
    }
}

muser_cuda_status launch_repack_kquant(Ctx *ctx, Weight *w, const uint8_t *dev_blocks, cudaStream_t stream) {
    KqGeom gm = kq_geom(*w);
    uint64_t tiles = (uint64_t)gm.row_tiles * gm.nsb;
    if (w->dtype == MUSER_DTYPE_Q4_K)
        repack_q4k_kernel<false><<<(unsigned)((tiles * 528 + 255) / 256), 256, 0, stream>>>(dev_blocks, w->image, gm);
    else if (w->dtype == MUSER_DTYPE_Q5_K)
        repack_q4k_kernel<true><<<(unsigned)((tiles * 656 + 255) / 256), 256, 0, stream>>>(dev_blocks, w->image, gm);
    else
        repack_q6k_kernel<<<(unsigned)((tiles * 785 + 255) / 256), 256, 0, stream>>>(dev_blocks, w->image, gm);
    MUSER_CUDA_TRY(ctx, cudaGetLastError());
    return MUSER_CUDA_OK;
}

// ------------------------------------------------------------------------------ NVFP4 repack
// Values stay row-major [n_out_pad][n_in/2] (K contiguous: the shape a TMA box load wants); scales move to
// the 128-row x 4-group swizzle and lose their sign, which is folded into the 16 codes of the group
// (a negative E4M3 scale times a code equals the positive scale times the negated code, bit for bit).
__global__ void repack_nvfp4_kernel(const uint8_t *__restrict__ raw_packed, const uint8_t *__restrict__ raw_scales,
                                    uint8_t *__restrict__ packed, uint8_t *__restrict__ scales, uint64_t n_out,
                                    uint64_t n_in, uint64_t row0, uint64_t k0, uint64_t n_in_full,
                                    uint32_t kt /* 64-element tiles per row */, int *nan_flag) {
    uint64_t groups = n_in / 16;
    uint64_t idx = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
    if (idx >= n_out * groups) return;
    uint64_t row = idx / groups, grp = idx % groups;
    uint64_t src_row = row0 + row, src_grp = k0 / 16 + grp;
    uint8_t s = raw_scales[src_row * (n_in_full / 16) + src_grp];
    if ((s & 0x7f) == 0x7f) atomicOr(nan_flag, 1);
    uint64_t two = *reinterpret_cast<const uint64_t *>(raw_packed + src_row * (n_in_full / 2) + src_grp * 8);
    if (s & 0x80) two ^= 0x8888888888888888ull;
    *reinterpret_cast<uint64_t *>(packed + row * (n_in / 2) + grp * 8) = two;
    uint64_t off = (row / 128) * ((uint64_t)kt * 512) + (grp / 4) * 512 + (row % 32) * 16 + ((row % 128) / 32) * 4 + grp % 4;
    scales[off] = s & 0x7f;
}

muser_cuda_status launch_repack_nvfp4(Ctx *ctx, Weight *w, const uint8_t *dev_packed, const uint8_t *dev_scales,
                                      cudaStream_t stream) {
    uint32_t kt = (uint32_t)((w->n_in + 63) / 64);
    size_t packed_bytes = w->n_out_pad * (w->n_in / 2), scale_bytes = (w->n_out_pad / 128) * (size_t)kt * 512;
    MUSER_CUDA_TRY(ctx, cudaMemsetAsync(w->packed, 0, packed_bytes, stream));
    MUSER_CUDA_TRY(ctx, cudaMemsetAsync(w->scales, 0, scale_bytes, stream));
    MUSER_CUDA_TRY(ctx, cudaMemsetAsync(ctx->dev_status, 0, sizeof(int), stream));
    uint64_t row0 = 0, k0 = 0;
    if (w->shard.axis == MUSER_SHARD_ROWS) row0 = w->shard.rank * w->n_out;
    if (w->shard.axis == MUSER_SHARD_K) k0 = w->shard.rank * w->n_in;
    uint64_t total = w->n_out * (w->n_in / 16);
    repack_nvfp4_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
        dev_packed, dev_scales, w->packed, w->scales, w->n_out, w->n_in, row0, k0, w->n_in_full, kt, ctx->dev_status);
    MUSER_CUDA_TRY(ctx, cudaGetLastError());
    int flag = 0;
    MUSER_CUDA_TRY(ctx, cudaMemcpyAsync(&flag, ctx->dev_status, sizeof(int), cudaMemcpyDeviceToHost, stream));
    MUSER_CUDA_TRY(ctx, cudaStreamSynchronize(stream));
    if (flag) return fail(ctx, MUSER_CUDA_NAN_SCALE, "NVFP4 block scales contain an E4M3FN NaN code");
    return MUSER_CUDA_OK;
}

// ------------------------------------------------------------------------------ image -> f32
// One weight out of the repacked image: row `row`, position `kk` in the tile grid (input index + k_off).
template <bool Q5>
__device__ __forceinline__ float q4k_weight(const uint8_t *__restrict__ image, uint32_t nsb, uint32_t row, uint64_t kk) {
    uint32_t sb = (uint32_t)(kk / 256), e = (uint32_t)(kk % 256);
    const uint8_t *tile = image + ((uint64_t)(row / 16) * nsb + sb) * (Q5 ? kQ5TileBytes : kQ4TileBytes);
    uint32_t r = row % 16, g = r & 7, rowsel = r >> 3;
    uint32_t j = e >> 5, wi = (e >> 3) & 3, i = e & 7;
    uint32_t q = rowsel * 2 + (j >> 2);
    uint32_t word = reinterpret_cast<const uint32_t *>(tile)[(q * 32 + g * 4 + wi) * 4 + (j & 3)]; // lane (g, 8-element group), word = sub-block % 4
    uint32_t nib = (word >> (4 * q4_nibble_pos(i))) & 15u;
    if constexpr (Q5) { // the fifth bit: byte (j % 4) of word (2 * rowsel + j / 4) of the lane's uint4, see kquant_layout.cuh
        uint32_t hw = reinterpret_cast<const uint32_t *>(tile + kQ5OffHi)[(g * 4 + wi) * 4 + rowsel * 2 + (j >> 2)];
        uint32_t pos = q4_nibble_pos(i);
        nib |= ((hw >> (8 * (j & 3) + 4 * (pos & 1) + (pos >> 1))) & 1u) << 4;
    }
    const uint8_t *hdr = tile + (Q5 ? kQ5OffHdr : 2048) + r * 16;
    float d = __half2float(*reinterpret_cast<const __half *>(hdr));
    float dmin = __half2float(*reinterpret_cast<const __half *>(hdr + 2));
    const uint8_t *s = hdr + 4;
    uint32_t sc, mn;
    if (j < 4) {
        sc = s[j] & 63;
        mn = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 15u) | ((s[j - 4] >> 6) << 4);
        mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
    float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(dmin, (float)mn);
    return __fsub_rn(__fmul_rn(d1, (float)nib), m1); // k_block.rs:40-41
}

__device__ __forceinline__ float q6k_weight(const uint8_t *__restrict__ image, uint32_t nsb, uint32_t row, uint64_t kk) {
    uint32_t sb = (uint32_t)(kk / 256), e = (uint32_t)(kk % 256);
    const uint8_t *tile = image + ((uint64_t)(row / 16) * nsb + sb) * kQ6TileBytes;
    uint32_t r = row % 16, g = r & 7, rowsel = r >> 3;
    uint32_t s = e >> 4, el = e & 15;
    uint32_t lane = g * 4 + (el >> 2), b = el & 3;
    uint32_t t_word = reinterpret_cast<const uint32_t *>(tile)[((rowsel * 2 + (s >> 3)) * 32 + lane) * 4 + ((s & 7) >> 1)];
    uint32_t top = (t_word >> (8 * b + 4 * (s & 1))) & 15u;
    uint32_t l_word = reinterpret_cast<const uint32_t *>(tile + kQ6OffHi)[(rowsel * 32 + lane) * 4 + (s >> 2)];
    uint32_t low = (l_word >> (8 * b + 2 * (s & 3))) & 3u;
    int qv = (int)(((top << 2) | low) ^ 32u) - 32; // the image holds (q - 32) & 63
    float d = __half2float(reinterpret_cast<const __half *>(tile + kQ6OffD)[r]);
    int sc = reinterpret_cast<const int8_t *>(tile + kQ6OffSc)[r * 16 + s];
    return __fmul_rn(__fmul_rn(d, (float)sc), (float)qv); // q6.rs:305-313
}

// One thread per output element; reads the repacked image only.
template <bool Q5>
__global__ void dequant_q4k_kernel(const uint8_t *__restrict__ image, float *__restrict__ out, KqGeom gm) {
    uint64_t idx = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
    if (idx >= gm.n_out * gm.n_in) return;
    out[idx] = q4k_weight<Q5>(image, gm.nsb, (uint32_t)(idx / gm.n_in), idx % gm.n_in + gm.k_off);
}

__global__ void dequant_q6k_kernel(const uint8_t *__restrict__ image, float *__restrict__ out, KqGeom gm) {
    uint64_t idx = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
    if (idx >= gm.n_out * gm.n_in) return;
    out[idx] = q6k_weight(image, gm.nsb, (uint32_t)(idx / gm.n_in), idx % gm.n_in + gm.k_off);
}

// ------------------------------------------------------------------------------ selected rows
// weights::matmul_rows (src/weights.rs:425-449): out[t][i] = dot(W_rows[i], x_t) for a list of output rows, the way
// the reference scores a handful of LM-head rows.  One warp per listed row; lanes stride over the inputs, decode
// each weight from the image and keep up to eight token sums; a butterfly adds the lanes (fixed order).
template <int DT, bool XF32>
__global__ void __launch_bounds__(256) kquant_rows_kernel(const uint8_t *__restrict__ image, KqGeom gm, const uint32_t *__restrict__ rows,
                                                          uint32_t n_rows, const void *__restrict__ x, uint32_t tokens,
                                                          float *__restrict__ out) {
    const uint32_t i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (i >= n_rows) return;
    const uint32_t row = rows[i];
    for (uint32_t t0 = 0; t0 < tokens; t0 += 8) {
        const uint32_t nt = min(8u, tokens - t0);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (row < gm.n_out) {
            for (uint64_t k = lane; k < gm.n_in; k += 32) {
                const float w = DT == MUSER_DTYPE_Q4_K ? q4k_weight<false>(image, gm.nsb, row, k + gm.k_off)
                              : DT == MUSER_DTYPE_Q5_K ? q4k_weight<true>(image, gm.nsb, row, k + gm.k_off)
                                                       : q6k_weight(image, gm.nsb, row, k + gm.k_off);
#pragma unroll
                for (uint32_t t = 0; t < 8; ++t)
                    if (t < nt) {
                        const size_t xi = (size_t)(t0 + t) * gm.n_in + k;
                        const float xv = XF32 ? reinterpret_cast<const float *>(x)[xi]
                                              : __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(x)[xi]);
                        acc[t] = fmaf(w, xv, acc[t]);
                    }
            }
        }
#pragma unroll
        for (uint32_t t = 0; t < 8; ++t) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], o);
            if (lane == 0 && t < nt) out[(size_t)(t0 + t) * n_rows + i] = row < gm.n_out ? acc[t] : __int_as_float(0x7fc00000);
        }
    }
}

muser_cuda_status launch_kquant_rows(Ctx *ctx, const Weight *w, const uint32_t *rows, uint32_t n_rows, const void *x,
                                     uint32_t x_dtype, float *out, uint32_t tokens, cudaStream_t stream) {
    const unsigned blocks = (n_rows + 7) / 8;
    const KqGeom gm = kq_geom(*w);
    const bool xf32 = x_dtype == MUSER_DTYPE_F32;
#define MUSER_ROWS(DT_)                                                                                                   \
    do {                                                                                                                   \
        if (xf32) kquant_rows_kernel<DT_, true><<<blocks, 256, 0, stream>>>(w->image, gm, rows, n_rows, x, tokens, out);   \
        else kquant_rows_kernel<DT_, false><<<blocks, 256, 0, stream>>>(w->image, gm, rows, n_rows, x, tokens, out);       \
    } while (0)
    if (w->dtype == MUSER_DTYPE_Q4_K) MUSER_ROWS(MUSER_DTYPE_Q4_K);
    else if (w->dtype == MUSER_DTYPE_Q5_K) MUSER_ROWS(MUSER_DTYPE_Q5_K);
    else MUSER_ROWS(MUSER_DTYPE_Q6_K);
#undef MUSER_ROWS
    MUSER_CUDA_TRY(ctx, cudaGetLastError());
    return MUSER_CUDA_OK;
}

__device__ __forceinline__ float e4m3_magnitude(uint32_t code) { // quant/nvfp4.rs:108-120, sign handled at repack
    uint32_t ex = (code >> 3) & 15u, man = code & 7u;
    if (ex == 0) return (float)man * (1.0f / 512.0f);
    return __fmul_rn(1.0f + (float)man * 0.125f, __uint_as_float((ex - 7 + 127) << 23));
}

__global__ void dequant_nvfp4_kernel(const uint8_t *__restrict__ packed, const uint8_t *__restrict__ scales,
                                     float *__restrict__ out, uint64_t n_out, uint64_t n_in, uint32_t kt,
                                     float scale2) {
    uint64_t idx = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
    if (idx >= n_out * n_in) return;
    uint64_t row = idx / n_in, k = idx % n_in, grp = k / 16;
    uint8_t byte = packed[row * (n_in / 2) + k / 2];
    uint32_t code = (k & 1) ? (byte >> 4) : (byte & 15u);
    uint64_t off = (row / 128) * ((uint64_t)kt * 512) + (grp / 4) * 512 + (row % 32) * 16 + ((row % 128) / 32) * 4 + grp % 4;
    const float lut[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float v = lut[code & 7];
    if (code & 8) v = -v;
    out[idx] = __fmul_rn(__fmul_rn(v, e4m3_magnitude(scales[off])), scale2); // nvfp4.rs:250-251
}

muser_cuda_status launch_dequant(Ctx *ctx, const Weight *w, float *out, cudaStream_t stream) {
    uint64_t total = w->n_out * w->n_in;
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (w->dtype == MUSER_DTYPE_NVFP4_E2M1) {
        dequant_nvfp4_kernel<<<blocks, 256, 0, stream>>>(w->packed, w->scales, out, w->n_out, w->n_in,
                                                         (uint32_t)((w->n_in + 63) / 64), w->scale2);
    } else if (w->dtype == MUSER_DTYPE_Q4_K) {
        dequant_q4k_kernel<false><<<blocks, 256, 0, stream>>>(w->image, out, kq_geom(*w));
    } else if (w->dtype == MUSER_DTYPE_Q5_K) {
        dequant_q4k_kernel<true><<<blocks, 256, 0, stream>>>(w->image, out, kq_geom(*w));
    } else {
        dequant_q6k_kernel<<<blocks, 256, 0, stream>>>(w->image, out, kq_geom(*w));
    }
    MUSER_CUDA_TRY(ctx, cudaGetLastError());
    return MUSER_CUDA_OK;
}

} // namespace muser
