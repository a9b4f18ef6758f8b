// The one-shot all-reduce's exchange protocol, written once for the GPU kernel (collective.cu) and for a host
// harness in which the ranks are CPU threads (tests/exchange_harness.cpp), so that the protocol's logic (slots,
// sequence numbers, rank-order sums, what a rank does when a peer never shows up) is tested without a GPU.
//
// Every rank owns a buffer of cells[2 slots][kMaxRanks senders][kMaxElems]; a cell is 8 bytes, the value's bits and
// the sequence number of the call that sent it, written by ONE store and therefore seen whole or not at all.  A call:
//   1. push: this rank stores (value, seq) into cell (seq & 1, this rank, i) of EVERY rank's buffer;
//   2. gather: for each element it polls its own buffer's cells of all senders until they carry `seq` (bounded),
//      adds the values in rank order (identical bits on every rank), and writes the sum back.
// The slot alternates with the sequence number: a cell still holds the number of two calls ago when a new value is
// due.  A rank can run at most one call ahead of the slowest reader of a slot (to get further it needs that reader's
// values of the call in between), so two slots are enough.  When a wait gives up, the element and all later
// elements of that caller keep this rank's own partial sums and the call returns kGaveUp: no stale or half-summed
// value is ever written.
#pragma once
#include <stddef.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define MUSER_XCHG __device__ __forceinline__
#else
#define MUSER_XCHG static inline
#endif

namespace muser {
namespace xchg {

constexpr uint32_t kMaxRanks = 8;
constexpr uint32_t kMaxBytes = 1536u << 10;       // f32 payload per rank and call: 64 tokens x 5120 values and some room
constexpr uint32_t kMaxElems = kMaxBytes / 4;
constexpr uint32_t kChunkElems = 256;             // values per CTA (one per thread); each chunk has its own sequence counter
constexpr uint32_t kMaxChunks = kMaxElems / kChunkElems;
constexpr int kGaveUp = 401;

struct Cell {
    uint32_t bits, seq;
};

constexpr size_t kCellBytes = (size_t)2 * kMaxRanks * kMaxElems * sizeof(Cell);
constexpr size_t kSeqBytes = kMaxChunks * sizeof(uint32_t); // this rank's own per-chunk sequence numbers, behind the cells
constexpr size_t kBufBytes = kCellBytes + kSeqBytes;

MUSER_XCHG size_t cell_index(uint32_t slot, uint32_t sender, uint32_t i) { return ((size_t)slot * kMaxRanks + sender) * kMaxElems + i; }

// Mem supplies: void store(Cell *, uint32_t bits, uint32_t seq); Cell load(const Cell *); void pause(uint32_t polls_so_far);
// float get(const float *); void put(float *, float)  (how the payload itself is read and written).
// One value of this rank into cell (seq & 1, rank, i) of every rank's buffer.
template <class Mem>
MUSER_XCHG void push_element(Mem &mem, Cell *const *peer, uint32_t rank, uint32_t world, uint32_t seq, uint32_t i, float value) {
    union { float f; uint32_t u; } v;
    v.f = value;
    for (uint32_t p = 0; p < world; ++p) mem.store(peer[p] + cell_index(seq & 1u, rank, i), v.u, seq);
}

// Elements first, first + stride, ... of [begin, end) are this caller's.  push = false: the values of this call
// were pushed earlier by whoever produced them (the projection kernel's epilogue), this rank's own included.
template <class Mem>
MUSER_XCHG int exchange_elements(Mem &mem, Cell *const *peer, uint32_t rank, uint32_t world, uint32_t seq, float *buf, uint32_t begin,
                                 uint32_t end, uint32_t first, uint32_t stride, uint32_t wait_limit, bool push = true) {
    const uint32_t slot = seq & 1u;
    if (push)
        for (uint32_t i = begin + first; i < end; i += stride) push_element(mem, peer, rank, world, seq, i, mem.get(buf + i));
    // Gather, four elements at a time: every cell of the four is read once before any is examined, so the loads are
    // in flight together (a thread that read, checked and re-read cell after cell spent one memory round trip per
    // rank and element: 25 us for an 8-rank sum of 20 KB); only cells that have not arrived yet are polled again.
    const Cell *mine = peer[rank];
    constexpr uint32_t kBatch = 4;
    for (uint32_t i0 = begin + first; i0 < end; i0 += kBatch * stride) {
        Cell c[kBatch][kMaxRanks];
#pragma unroll
        for (uint32_t k = 0; k < kBatch; ++k) {
            const uint32_t i = i0 + k * stride;
            if (i >= end) continue;
#pragma unroll
            for (uint32_t p = 0; p < kMaxRanks; ++p)
                if (p < world) c[k][p] = mem.load(mine + cell_index(slot, p, i));
        }
#pragma unroll
        for (uint32_t k = 0; k < kBatch; ++k) {
            const uint32_t i = i0 + k * stride;
            if (i >= end) continue;
            float sum = 0.0f;
#pragma unroll
            for (uint32_t p = 0; p < kMaxRanks; ++p) {
                if (p >= world) continue;
                const Cell *cell = mine + cell_index(slot, p, i);
                for (uint32_t n = 0; c[k][p].seq != seq && n < wait_limit; ++n) {
                    mem.pause(n);
                    c[k][p] = mem.load(cell);
                }
                if (c[k][p].seq != seq) return kGaveUp; // this and the caller's later elements keep their partial sums
                union { float f; uint32_t u; } v;
                v.u = c[k][p].bits;
                sum += v.f;
            }
            mem.put(buf + i, sum);
        }
    }
    return 0;
}

} // namespace xchg
} // namespace muser
