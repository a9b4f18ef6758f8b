// Geometry of the repacked K-quant images, shared by the repack, dequant and matmul kernels.
//
// Lane (g, t) of a warp (g = lane / 4, t = lane % 4) owns rows g and g + 8 of the tile and, within each row,
// WHOLE sub-blocks: Q4_K sub-blocks t and t + 4 (32 weights each), Q6_K sub-blocks t, t + 4, t + 8, t + 12
// (16 weights each).  Its bytes sit at uint4 index (q * 32 + lane) of each plane, so one warp-wide 16-byte
// load reads 512 contiguous bytes.
//
// Q4_K tile (16 rows x 256 inputs, 2304 bytes)
//   [0, 2048)   uint4 (q, lane), q = 2*rowsel + hi: row g + 8*rowsel, sub-block t + 4*hi.  Word wi holds
//               elements 8wi .. 8wi+7 of that sub-block, element i in nibble q4_nibble_pos(i): the order puts
//               elements (0,1), (2,3), (4,5), (6,7) in nibble pairs (p, p+4), so (word >> 4p) & 0x000F000F
//               yields one packed pair per operation.
//   [2048,2304) 16 x the block's 16-byte header (d f16, dmin f16, 12 bytes of packed 6-bit scale/min).
// Q6_K tile (3360 bytes)
//   [0, 2048)   low nibbles: uint4 (q, lane), q = 2*rowsel + half.  Word wi belongs to owned sub-block
//               o = 2*half + wi/2 (sub-block t + 4o) and holds its elements 8h .. 8h+7, h = wi % 2: byte b
//               carries element 8h + b in its low nibble and element 8h + 4 + b in its high nibble.
//   [2048,3072) high 2 bits: uint4 (rowsel, lane); word o holds sub-block t + 4o: element 4x + b in bits
//               [8b + 2x, 8b + 2x + 1].
//   [3072,3328) 16 x sc[16] int8;  [3328,3360) 16 x d f16.
//
// ---- The "column" layout (Weight::layout == 1), read by the decode kernel (kquant_decode.cu) ----
// Here a lane owns a QUARTER of EVERY sub-block of its two rows, which is what a tensor-core fragment of a
// sub-block-at-a-time product wants: lane (g, t) supplies rows g and g + 8 and 8 (Q4_K) or 4 (Q6_K) consecutive
// elements of each sub-block, so no regrouping is needed between the load and the MMA.
//
// Q4_K tile (2304 bytes)
//   [0, 2048)   uint4 (u, lane), u = 2*rowsel + half: row g + 8*rowsel, sub-blocks 4*half .. 4*half + 3.  Word jj
//               holds elements 8t .. 8t+7 of sub-block 4*half + jj, element i in nibble q4_nibble_pos(i): the low
//               nibbles of bytes 0..3 are elements 8t + (0, 4, 1, 5), the high nibbles 8t + (2, 6, 3, 7).
//   [2048,2304) 16 x the block's 16-byte header, as above.
// Q6_K tile (3360 bytes).  A weight is stored as v = (q - 32) & 63 (six-bit two's complement), split into its top
// four bits T = v >> 2 and low two bits L = v & 3, so that (T << 4) | (L << 2) is the signed byte 4 * (q - 32).
//   [0, 2048)   T plane: uint4 (u, lane), u = 2*rowsel + half: row g + 8*rowsel, sub-blocks 8*half .. 8*half + 7.
//               Word wi: byte b carries element 4t + b of sub-block 8*half + 2*wi in its low nibble and of
//               sub-block 8*half + 2*wi + 1 in its high nibble.
//   [2048,3072) L plane: uint4 (rowsel, lane); word v covers sub-blocks 4v .. 4v+3: bits [2x, 2x+1] of byte b are
//               L of element 4t + b of sub-block 4v + x.
//   [3072,3328) 16 x sc[16] int8;  [3328,3360) 16 x d f16.
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
