// The all-reduce that follows a row-parallel projection, behind the C ABI.
//
// The reference runs one accelerator and refuses tensor parallelism (scripts/gx10/vllm/muser_vllm/connector.py:119-120),
// so nothing here has a counterpart there.  A context can be given a communicator of `world` ranks, one process per
// GPU of one box; muser_cuda_all_reduce then sums a buffer in place across the ranks on the caller's stream:
//   - payloads up to 1.5 MiB of f32 (a decode or verify step's [tokens][hidden] partial sums: 20 KB per token) take a one-shot
//     exchange over peer memory: every rank PUSHES each value, paired with the call's sequence number in one 8-byte
//     store, into a cell of every rank's buffer over NVLink, then polls (bounded) its own cells until every rank's
//     value of the call is there and adds them in rank order, so all ranks get the same bits.  No flag, no fence:
//     latency is one one-way trip.  One small kernel, no library call;
//   - everything else goes to ncclAllReduce, found at run time in the NCCL that the process already carries
//     (dlopen of libnccl.so.2), so the library itself has no link-time dependency on it.
// The peer buffers are cudaMalloc'd once per context at comm set-up and mapped into the other processes through
// CUDA IPC handles, which travel by one ncclAllGather.  No TMA and no multicast anywhere: plain st.global / ld.global.
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <cstring>
#include <new>

#include "common.cuh"
#include "oneshot_exchange.h"

namespace muser {

// Layout and protocol of the peer buffers: oneshot_exchange.h (shared with the host harness that tests the protocol).
constexpr uint32_t kMaxRanks = xchg::kMaxRanks;
constexpr uint32_t kOneShotMaxBytes = xchg::kMaxBytes;
constexpr uint32_t kOneShotChunkElems = xchg::kChunkElems;
constexpr uint32_t kOneShotWaitLimit = 1u << 21; // polls of one value (with a short sleep between) before the wait gives up: about a second
constexpr size_t kCellBytes = xchg::kCellBytes;
constexpr size_t kPeerBufBytes = xchg::kBufBytes;

struct NcclApi {
    void *lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

static NcclApi *nccl_api(std::string *why) {
    static std::mutex mu;
    static NcclApi api;
    static bool tried = false;
    std::lock_guard<std::mutex> lock(mu);
    if (!tried) {
        tried = true;
        void *lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (lib) {
            api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(lib, "ncclGetUniqueId"));
            api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(lib, "ncclCommInitRank"));
            api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(lib, "ncclCommDestroy"));
            api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(dlsym(lib, "ncclAllReduce"));
            api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(lib, "ncclAllGather"));
            api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(lib, "ncclGetErrorString"));
            if (api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce && api.AllGather && api.GetErrorString) api.lib = lib;
        }
    }
    if (!api.lib) {
        if (why) *why = "NCCL (libnccl.so.2) could not be loaded into this process";
        return nullptr;
    }
    return &api;
}

struct Comm {
    NcclApi *api = nullptr;
    ncclComm_t nccl = nullptr;
    bool own_nccl = false;
    uint32_t rank = 0, world = 1;
    uint8_t *local = nullptr;       // this rank's buffer (cudaMalloc)
    uint8_t *peer[kMaxRanks] = {};  // every rank's buffer as mapped here; peer[rank] == local
    bool oneshot = false;
    uint32_t oneshot_max_bytes = kOneShotMaxBytes;
};

struct OneShotArgs {
    uint8_t *peer[kMaxRanks];
    float *buf;
    uint32_t count, rank, world;
    uint32_t push; // 0: the values were pushed by the kernel that produced them (fused projection epilogue)
    int *status;
};

// A value travels together with its sequence number in one 8-byte store, which arrives whole or not at all: the
// receiver needs no fence and no separate flag, it polls the cell until the number is the one it expects.
struct DeviceCells {
    __device__ __forceinline__ void store(xchg::Cell *p, uint32_t bits, uint32_t seq) {
        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(bits), "r"(seq) : "memory");
    }
    __device__ __forceinline__ xchg::Cell load(const xchg::Cell *p) {
        xchg::Cell v;
        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.bits), "=r"(v.seq) : "l"(p) : "memory");
        return v;
    }
    __device__ __forceinline__ void pause(uint32_t n) {
        if (n > 32) __nanosleep(100);
    }
    __device__ __forceinline__ float get(const float *p) { return *p; }
    __device__ __forceinline__ void put(float *p, float v) { *p = v; }
};

// One CTA per 256 values, one per thread (more values per thread made every thread walk through its stores and loads
// one after the other: an 8-rank sum of 20 KB took 24 us with 2048 values per CTA).  CTA c keeps its own sequence number
// (in this rank's buffer, bumped once per launch), so
// the kernel can sit in a CUDA graph: nothing that changes from call to call is a launch argument.
__global__ void __launch_bounds__(256) oneshot_all_reduce_kernel(const OneShotArgs a) {
    __shared__ uint32_t seq_s;
    pdl_wait(); // `buf` comes from the kernel before this one; the sequence counter from the all-reduce before it
    const uint32_t c = blockIdx.x, tid = threadIdx.x;
    if (tid == 0) {
        uint32_t *seq = reinterpret_cast<uint32_t *>(a.peer[a.rank] + kCellBytes) + c;
        seq_s = __ldcg(seq) + 1; // kept in L2: the projection kernels that push for the next call read it from there
        __stcg(seq, seq_s);
    }
    __syncthreads();
    const uint32_t begin = c * kOneShotChunkElems, end = min(begin + kOneShotChunkElems, a.count);
    DeviceCells mem;
    // a thread that gives up stops there: its remaining outputs keep the rank's own partial sums
    if (xchg::exchange_elements(mem, reinterpret_cast<xchg::Cell *const *>(a.peer), a.rank, a.world, seq_s, a.buf, begin, end, tid, 256,
                                kOneShotWaitLimit, a.push != 0) != 0)
        atomicExch(a.status + 1, xchg::kGaveUp);
}

static muser_cuda_status nccl_fail(Ctx *ctx, Comm *cm, const char *what, ncclResult_t r) {
    return fail(ctx, MUSER_CUDA_NCCL_ERROR, std::string(what) + ": " + (cm && cm->api ? cm->api->GetErrorString(r) : "NCCL error"));
}

// Peer buffers: allocate, exchange IPC handles through the communicator, map.  A failure here leaves the context
// with NCCL only (the reason stays in last_error); it is not an error of the set-up call.
static void setup_oneshot(Ctx *ctx, Comm *cm, cudaStream_t stream) {
    cm->oneshot = false;
    if (cm->world > kMaxRanks) return;
    cudaIpcMemHandle_t *dev_handles = nullptr;
    cudaIpcMemHandle_t handles[kMaxRanks];
    auto give_up = [&](const std::string &why) {
        ctx->last_error = "one-shot all-reduce unavailable, NCCL serves every size: " + why;
        cudaFree(dev_handles);
    };
    cudaError_t e = cudaMalloc(&cm->local, kPeerBufBytes);
    if (e == cudaSuccess) e = cudaMemsetAsync(cm->local, 0, kPeerBufBytes, stream); // sequence number 0 is never expected
    if (e == cudaSuccess) e = cudaMalloc(&dev_handles, sizeof(handles));
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&handles[cm->rank], cm->local);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dev_handles + cm->rank, &handles[cm->rank], sizeof(cudaIpcMemHandle_t), cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return give_up(cudaGetErrorString(e));
    ncclResult_t r = cm->api->AllGather(dev_handles + cm->rank, dev_handles, sizeof(cudaIpcMemHandle_t), ncclChar, cm->nccl, stream);
    if (r != ncclSuccess) return give_up(cm->api->GetErrorString(r));
    e = cudaMemcpyAsync(handles, dev_handles, sizeof(handles), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return give_up(cudaGetErrorString(e));
    for (uint32_t p = 0; p < cm->world; ++p) {
        if (p == cm->rank) {
            cm->peer[p] = cm->local;
            continue;
        }
        void *ptr = nullptr;
        e = cudaIpcOpenMemHandle(&ptr, handles[p], cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return give_up(std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e));
        cm->peer[p] = reinterpret_cast<uint8_t *>(ptr);
    }
    cudaFree(dev_handles);
    dev_handles = nullptr;
    // every rank has zeroed its buffer before its handle left (stream order), so nobody can write into stale flags
    cm->oneshot = true;
}

static muser_cuda_status comm_install(Ctx *ctx, Comm *cm, cudaStream_t stream) {
    setup_oneshot(ctx, cm, stream);
    ctx->comm = cm;
    return MUSER_CUDA_OK;
}

void comm_destroy(Ctx *ctx) {
    Comm *cm = reinterpret_cast<Comm *>(ctx->comm);
    if (!cm) return;
    for (uint32_t p = 0; p < cm->world && p < kMaxRanks; ++p)
        if (cm->peer[p] && p != cm->rank) cudaIpcCloseMemHandle(cm->peer[p]);
    cudaFree(cm->local);
    if (cm->own_nccl && cm->nccl) cm->api->CommDestroy(cm->nccl);
    delete cm;
    ctx->comm = nullptr;
}

// For a projection that pushes its partial sums itself: where they go (null when this context cannot: no peer
// buffers, or a payload beyond the one-shot limit), and the second half of the all-reduce, which only gathers.
bool oneshot_push_target(Ctx *ctx, uint64_t count, OneShotPush *out) {
    Comm *cm = reinterpret_cast<Comm *>(ctx->comm);
    if (!cm || !cm->oneshot || count * 4 > std::min(cm->oneshot_max_bytes, ctx->oneshot_max_bytes)) return false;
    for (uint32_t p = 0; p < kMaxRanks; ++p) out->peer[p] = cm->peer[p];
    out->seq = reinterpret_cast<const uint32_t *>(cm->peer[cm->rank] + kCellBytes);
    out->rank = cm->rank, out->world = cm->world;
    return true;
}

cudaError_t launch_oneshot_gather(Ctx *ctx, float *buf, uint64_t count, cudaStream_t stream) {
    Comm *cm = reinterpret_cast<Comm *>(ctx->comm);
    OneShotArgs a;
    for (uint32_t p = 0; p < kMaxRanks; ++p) a.peer[p] = cm->peer[p];
    a.buf = buf, a.count = (uint32_t)count, a.rank = cm->rank, a.world = cm->world, a.push = 0, a.status = ctx->dev_status;
    const uint32_t ctas = ((uint32_t)count + kOneShotChunkElems - 1) / kOneShotChunkElems;
    return launch_pdl(oneshot_all_reduce_kernel, dim3(ctas), dim3(256), 0, stream, a);
}

} // namespace muser

using namespace muser;

extern "C" {

muser_cuda_status muser_cuda_comm_unique_id(uint8_t *out, size_t out_bytes) {
    if (!out || out_bytes < sizeof(ncclUniqueId)) {
        g_create_error = "the id buffer must hold 128 bytes";
        return MUSER_CUDA_BAD_ARG;
    }
    std::string why;
    NcclApi *api = nccl_api(&why);
    if (!api) {
        g_create_error = why;
        return MUSER_CUDA_NCCL_ERROR;
    }
    ncclUniqueId id;
    const ncclResult_t r = api->GetUniqueId(&id);
    if (r != ncclSuccess) {
        g_create_error = std::string("ncclGetUniqueId: ") + api->GetErrorString(r);
        return MUSER_CUDA_NCCL_ERROR;
    }
    memcpy(out, &id, sizeof(id));
    return MUSER_CUDA_OK;
}

muser_cuda_status muser_cuda_ctx_comm_init(muser_cuda_ctx *c, const uint8_t *id_bytes, uint32_t rank, uint32_t world, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (!ctx || !id_bytes || world < 2 || rank >= world) return fail(ctx, MUSER_CUDA_BAD_ARG, "a communicator needs an id and 0 <= rank < world, world >= 2");
    if (ctx->comm) return fail(ctx, MUSER_CUDA_BAD_ARG, "this context already has a communicator");
    std::string why;
    NcclApi *api = nccl_api(&why);
    if (!api) return fail(ctx, MUSER_CUDA_NCCL_ERROR, why);
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    Comm *cm = new (std::nothrow) Comm();
    if (!cm) return fail(ctx, MUSER_CUDA_ERROR, "out of host memory");
    cm->api = api, cm->rank = rank, cm->world = world, cm->own_nccl = true;
    ncclUniqueId id;
    memcpy(&id, id_bytes, sizeof(id));
    const ncclResult_t r = api->CommInitRank(&cm->nccl, (int)world, id, (int)rank);
    if (r != ncclSuccess) {
        const muser_cuda_status st = nccl_fail(ctx, cm, "ncclCommInitRank", r);
        delete cm;
        return st;
    }
    return comm_install(ctx, cm, (cudaStream_t)stream);
}

muser_cuda_status muser_cuda_ctx_comm_attach(muser_cuda_ctx *c, void *nccl_comm, uint32_t rank, uint32_t world, void *stream) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (!ctx || !nccl_comm || world < 2 || rank >= world) return fail(ctx, MUSER_CUDA_BAD_ARG, "a communicator and 0 <= rank < world, world >= 2");
    if (ctx->comm) return fail(ctx, MUSER_CUDA_BAD_ARG, "this context already has a communicator");
    std::string why;
    NcclApi *api = nccl_api(&why);
    if (!api) return fail(ctx, MUSER_CUDA_NCCL_ERROR, why);
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    Comm *cm = new (std::nothrow) Comm();
    if (!cm) return fail(ctx, MUSER_CUDA_ERROR, "out of host memory");
    cm->api = api, cm->rank = rank, cm->world = world, cm->own_nccl = false;
    cm->nccl = reinterpret_cast<ncclComm_t>(nccl_comm);
    return comm_install(ctx, cm, (cudaStream_t)stream);
}

int muser_cuda_ctx_comm_has_oneshot(const muser_cuda_ctx *c) {
    const Ctx *ctx = reinterpret_cast<const Ctx *>(c);
    const Comm *cm = ctx ? reinterpret_cast<const Comm *>(ctx->comm) : nullptr;
    return cm && cm->oneshot ? 1 : 0;
}

muser_cuda_status muser_cuda_all_reduce(muser_cuda_ctx *c, void *buf, uint64_t count, uint32_t dtype, void *stream_) {
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (!ctx || !buf || count == 0) return fail(ctx, MUSER_CUDA_BAD_ARG, "null argument");
    Comm *cm = reinterpret_cast<Comm *>(ctx->comm);
    if (!cm) return fail(ctx, MUSER_CUDA_BAD_ARG, "this context has no communicator (muser_cuda_ctx_comm_init / _attach)");
    if (dtype != MUSER_DTYPE_F32 && dtype != MUSER_DTYPE_BF16 && dtype != MUSER_DTYPE_F16)
        return fail(ctx, MUSER_CUDA_UNSUPPORTED_DTYPE, "all-reduce sums f32, f16 or bf16");
    if (!aligned16(buf)) return fail(ctx, MUSER_CUDA_BAD_ALIGN, "the buffer must be 16-byte aligned");
    cudaStream_t stream = (cudaStream_t)stream_;
    MUSER_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const uint32_t limit = std::min(cm->oneshot_max_bytes, ctx->oneshot_max_bytes);
    if (cm->oneshot && dtype == MUSER_DTYPE_F32 && count * 4 <= limit) {
        OneShotArgs a;
        for (uint32_t p = 0; p < kMaxRanks; ++p) a.peer[p] = cm->peer[p];
        a.buf = reinterpret_cast<float *>(buf);
        a.count = (uint32_t)count;
        a.rank = cm->rank;
        a.world = cm->world;
        a.push = 1;
        a.status = ctx->dev_status;
        const uint32_t ctas = ((uint32_t)count + kOneShotChunkElems - 1) / kOneShotChunkElems;
        MUSER_CUDA_TRY(ctx, launch_pdl(oneshot_all_reduce_kernel, dim3(ctas), dim3(256), 0, stream, a));
        return MUSER_CUDA_OK;
    }
    const ncclDataType_t t = dtype == MUSER_DTYPE_F32 ? ncclFloat32 : dtype == MUSER_DTYPE_F16 ? ncclFloat16 : ncclBfloat16;
    const ncclResult_t r = cm->api->AllReduce(buf, buf, (size_t)count, t, ncclSum, cm->nccl, stream);
    if (r != ncclSuccess) return nccl_fail(ctx, cm, "ncclAllReduce", r);
    return MUSER_CUDA_OK;
}

} // extern "C"
