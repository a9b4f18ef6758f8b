// Geometry of the repacked K-quant images, shared by the repack, dequant and matmul kernels.
//
// Q4_K tile (16 rows x 256 inputs, 2304 bytes)
//   [0, 2048)   uint4[4][32]: uint4 (q, lane) with lane = 4g + t, q = 2*rowsel + half, belongs to row
//               g + 8*rowsel; its word wi holds sub-block j = 4*half + wi, elements 32j + 8t + i (i = 0..7),
//               element i in nibble q4_nibble_pos(i).  That order puts elements (0,1), (2,3), (4,5), (6,7) in
//               nibble pairs (s, s+4), so (word >> 4s) & 0x000F000F yields one packed pair per operation.
//   [2048,2304) 16 x the block's 16-byte header (d f16, dmin f16, 12 bytes of packed 6-bit scale/min).
// Q6_K tile (3360 bytes)
//   [0, 2048)   low nibbles: uint4 (q, lane), q = 2*rowsel + half; word wi holds sub-blocks 8*half + 2wi
//               (low nibble of byte b) and 8*half + 2wi + 1 (high nibble of byte b), elements 4t + b.
//   [2048,3072) high 2 bits: uint4 (rowsel, lane); word wi holds sub-blocks 4wi + s (s = 0..3): element
//               4t + b in bits [8b + 2s, 8b + 2s + 1].
//   [3072,3328) 16 x sc[16] int8;  [3328,3360) 16 x d f16.
// A lane (g, t) therefore owns, in both formats, the weights that the m16n8k16 A fragment assigns to it:
// rows g and g + 8, MMA k-slots {2t, 2t+1, 2t+8, 2t+9}.
#pragma once
#include "common.cuh"

namespace muser {

struct KqGeom {
    uint64_t n_out, n_in;    // local (shard) geometry
    uint64_t row0, k0;       // first global row / input of this shard
    uint64_t blocks_per_row; // super-blocks per row of the stored (unsharded) tensor
    uint32_t row_tiles, nsb, k_off;
};

inline KqGeom kq_geom(const Weight &w) {
    KqGeom g;
    g.n_out = w.n_out;
    g.n_in = w.n_in;
    g.row0 = w.shard.axis == MUSER_SHARD_ROWS ? w.shard.rank * w.n_out : 0;
    g.k0 = w.shard.axis == MUSER_SHARD_K ? w.shard.rank * w.n_in : 0;
    g.blocks_per_row = w.n_in_full / 256;
    g.row_tiles = w.row_tiles;
    g.nsb = w.nsb;
    g.k_off = w.k_off;
    return g;
}

__host__ __device__ __forceinline__ int q4_nibble_pos(int i) { return (i & 1) * 4 + (i >> 1); }

} // namespace muser
