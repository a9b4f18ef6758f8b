// Geometry of the repacked K-quant images, shared by the repack, dequant and matmul kernels.
//
// A lane owns a QUARTER of EVERY sub-block of its two rows, which is what a tensor-core fragment of a
// sub-block-at-a-time product wants: lane (g, t) of a warp (g = lane / 4, t = lane % 4) supplies rows g and g + 8
// and 8 (Q4_K) or 4 (Q6_K) consecutive elements of each sub-block, so nothing is regrouped between the load and
// the MMA.  Its bytes sit at uint4 index (plane * 32 + lane), so one warp-wide 16-byte load reads 512 contiguous
// bytes and a tile is one contiguous bulk copy.
//
// Q4_K tile (16 rows x 256 inputs, 2304 bytes)
//   [0, 2048)   uint4 (u, lane), u = 2*rowsel + half: row g + 8*rowsel, sub-blocks 4*half .. 4*half + 3.  Word jj
//               holds elements 8t .. 8t+7 of sub-block 4*half + jj, element i in nibble q4_nibble_pos(i): the low
//               nibbles of bytes 0..3 are elements 8t + (0, 4, 1, 5), the high nibbles 8t + (2, 6, 3, 7), and
//               (word >> 4p) & 0x000F000F yields the pair (2p, 2p + 1) in one operation.
//   [2048,2304) 16 x the block's 16-byte header (d f16, dmin f16, 12 bytes of packed 6-bit scale/min, GGUF packing).
// Q5_K tile (2816 bytes): the Q4_K tile with a plane of fifth bits between the nibbles and the headers.
//   [0, 2048)   the low four bits of every weight, exactly as in a Q4_K tile.
//   [2048,2560) uint4 (lane): word 0 = row g, sub-blocks 0-3; word 1 = row g, sub-blocks 4-7; words 2, 3 = row g + 8.
//               Byte jj of a word holds the fifth bits of the lane's eight elements of that sub-block in the order the
//               nibble word yields them: bit b (0..3) belongs to the element in the LOW nibble of byte b, bit 4 + b to
//               the one in the HIGH nibble, so (x * 0x02040810) & 0x10101010 drops four of them onto bit 4 of four bytes.
//   [2560,2816) 16 x the block's 16-byte header (d, dmin, 6-bit scales and mins), as in Q4_K.
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
