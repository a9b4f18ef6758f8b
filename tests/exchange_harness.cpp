// Host harness for the one-shot all-reduce's exchange protocol (muser_b200/csrc/oneshot_exchange.h): the ranks are CPU
// threads, the peer buffers plain host memory, a cell is read and written with one 8-byte atomic access as on the
// GPU.  Built by tests/test_exchange_protocol.py with g++; no GPU, no CUDA.
//
// Fault injection happens here, on the host: a rank can skip a call altogether (it never shows up), or join it with
// fewer elements than the others.
#include <sched.h>

#include <cstring>
#include <thread>
#include <vector>

#include "../muser_b200/csrc/oneshot_exchange.h"

using namespace muser::xchg;

struct HostCells {
    void store(Cell *p, uint32_t bits, uint32_t seq) {
        const uint64_t v = (uint64_t)seq << 32 | bits;
        __atomic_store_n(reinterpret_cast<uint64_t *>(p), v, __ATOMIC_RELAXED);
    }
    Cell load(const Cell *p) {
        const uint64_t v = __atomic_load_n(reinterpret_cast<const uint64_t *>(p), __ATOMIC_RELAXED);
        return Cell{(uint32_t)v, (uint32_t)(v >> 32)};
    }
    void pause(uint32_t n) {
        if (n > 8) sched_yield();
    }
    float get(const float *p) { return *p; }
    void put(float *p, float v) { *p = v; }
};

// One process-wide "box": world buffers, as cudaMalloc + memset(0) leaves them at communicator set-up.
struct Box {
    uint32_t world;
    std::vector<std::vector<uint64_t>> buf; // kBufBytes each
    std::vector<Cell *> peer;
};

extern "C" {

void *xchg_box_create(uint32_t world) {
    if (world < 1 || world > kMaxRanks) return nullptr;
    Box *b = new Box;
    b->world = world;
    b->buf.resize(world);
    for (auto &v : b->buf) v.assign(kBufBytes / 8, 0); // sequence number 0 is never expected
    for (auto &v : b->buf) b->peer.push_back(reinterpret_cast<Cell *>(v.data()));
    return b;
}
void xchg_box_destroy(void *box) { delete static_cast<Box *>(box); }

// One all-reduce call of every rank, each on its own thread.  data: [world][count] in, sums out (in place, as the
// kernel leaves them).  joins[r] = 0: rank r skips the call; counts[r]: how many elements rank r brings (the others
// expect `count`).  lead[r] > 0: rank r sleeps that many microseconds before it starts (to vary who runs ahead).
// status[r] receives 0 or kGaveUp.  Chunks are walked one after the other by one thread per rank.
void xchg_call(void *box, float *data, uint32_t count, const uint32_t *joins, const uint32_t *counts, const uint32_t *lead_us,
               uint32_t wait_limit, int *status) {
    Box *b = static_cast<Box *>(box);
    std::vector<std::thread> th;
    for (uint32_t r = 0; r < b->world; ++r) {
        status[r] = 0;
        if (!joins[r]) continue;
        th.emplace_back([=]() {
            if (lead_us[r]) std::this_thread::sleep_for(std::chrono::microseconds(lead_us[r]));
            HostCells mem;
            const uint32_t n = counts[r], chunks = (n + kChunkElems - 1) / kChunkElems;
            uint32_t *seqs = reinterpret_cast<uint32_t *>(reinterpret_cast<uint8_t *>(b->peer[r]) + kCellBytes);
            for (uint32_t c = 0; c < chunks; ++c) {
                const uint32_t seq = ++seqs[c];
                const uint32_t begin = c * kChunkElems, end = begin + kChunkElems < n ? begin + kChunkElems : n;
                if (exchange_elements(mem, b->peer.data(), r, b->world, seq, data + (size_t)r * count, begin, end, 0, 1, wait_limit) != 0)
                    status[r] = kGaveUp;
            }
        });
    }
    for (auto &t : th) t.join();
}

// Several calls back to back WITHOUT a join between them: every rank thread runs `calls` all-reduces in a row, so a
// fast rank runs ahead of a slow one by as much as the protocol lets it.  data: [calls][world][count].
void xchg_run(void *box, float *data, uint32_t count, uint32_t calls, const uint32_t *lead_us, uint32_t wait_limit, int *status) {
    Box *b = static_cast<Box *>(box);
    std::vector<std::thread> th;
    for (uint32_t r = 0; r < b->world; ++r) {
        status[r] = 0;
        th.emplace_back([=]() {
            HostCells mem;
            const uint32_t chunks = (count + kChunkElems - 1) / kChunkElems;
            uint32_t *seqs = reinterpret_cast<uint32_t *>(reinterpret_cast<uint8_t *>(b->peer[r]) + kCellBytes);
            for (uint32_t k = 0; k < calls; ++k) {
                if (lead_us[r] && (k % 3) == r % 3) std::this_thread::sleep_for(std::chrono::microseconds(lead_us[r]));
                float *mine = data + ((size_t)k * b->world + r) * count;
                for (uint32_t c = 0; c < chunks; ++c) {
                    const uint32_t seq = ++seqs[c];
                    const uint32_t begin = c * kChunkElems, end = begin + kChunkElems < count ? begin + kChunkElems : count;
                    if (exchange_elements(mem, b->peer.data(), r, b->world, seq, mine, begin, end, 0, 1, wait_limit) != 0) status[r] = kGaveUp;
                }
            }
        });
    }
    for (auto &t : th) t.join();
}

} // extern "C"
