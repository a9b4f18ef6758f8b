// Shared declarations of the muser-cuda library: handles, error plumbing, tile geometry.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>
#include <utility>

#include "../../include/muser_cuda.h"

namespace muser {

// ---- tile geometry of the repacked K-quant images -------------------------------------------
// A tile covers 16 weight rows x one 256-element super-block and is contiguous in memory; tiles
// are ordered [row_tile][super_block].  Inside a tile the quants are laid out in the order the
// 32 lanes of a warp consume them (one 16-byte load per lane), followed by the scale headers.
constexpr int kTileRows = 16;
constexpr int kQ4TileBytes = 2048 + 256;             // nibbles | 16 x (d, dmin, scales[12])
constexpr int kQ6TileBytes = 2048 + 1024 + 256 + 32; // low nibbles | high 2-bit | 16 x sc[16] | 16 x d
constexpr int kQ5TileBytes = 2048 + 512 + 256;       // nibbles | fifth bits | 16 x (d, dmin, scales[12])
constexpr int kQ5OffHi = 2048, kQ5OffHdr = 2560;
constexpr int kQ6OffHi = 2048, kQ6OffSc = 3072, kQ6OffD = 3328;

struct Ctx {
    int device = 0;
    int sm_count = 0;
    void *workspace = nullptr;
    size_t workspace_bytes = 0;
    int *dev_status = nullptr; // device-side give-up flags (bounded waits), read by sync_status
    float *gemv_partial = nullptr;        // K-slice partial sums of the decode GEMV
    size_t gemv_partial_bytes = 0;
    unsigned int *gemv_counters = nullptr; // one arrival counter per 16-row tile, zero between launches
    uint32_t gemv_counter_slots = 0;
    void *tc_scratch = nullptr;            // f16 activations + sub-block sums of the tensor-core K-quant kernel
    size_t tc_scratch_bytes = 0;
    uint32_t tc_min_tokens[2] = {17, 17};  // from how many tokens Q4_K / Q6_K calls take that kernel (tuning knobs,
    uint32_t tc_min_rows = 1024;           // and from how many output rows); fewer tokens take the decode kernel
    uint32_t dec_warps = 0, dec_ksplit = 0, dec_ring = 0, dec_wsplit = 0;
    uint32_t dec_last_plan[4] = {0, 0, 0, 0}; // (warps, ksplit, wsplit, ring) of the decode kernel's latest launch on this context // decode kernel plan overrides (0: from its cost model)
    float *norm_scratch = nullptr;         // normalized rows for the skinny K-quant kernel (fused input norm)
    size_t norm_scratch_bytes = 0;
    float *inv_rms = nullptr;              // one 1/rms per token row of a fused input norm (NVFP4 quantizer, skinny kernel)
    uint32_t inv_rms_rows = 0;
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t copy_events[32] = {};          // "this group's input has landed", made on first use of the host-group entry
    void *host_stage = nullptr; // pinned staging for matmul_host
    size_t host_stage_bytes = 0;
    void *dev_stage = nullptr;
    size_t dev_stage_bytes = 0;
    void *arena = nullptr; // device staging of matmul_host_enqueue: bumped per call, rewound by sync_status
    size_t arena_bytes = 0, arena_used = 0;
    void *comm = nullptr;                      // tensor-parallel communicator (collective.cu), or null
    unsigned long long *amax_keys = nullptr;   // fused greedy pick: one key and one flag word per token (16 each), zero between calls
    unsigned int *amax_flags = nullptr;
    uint32_t host_direct_output = 2;           // host-group entry: 2 one copy per output on the copy stream (beside the next launches), 1 a kernel
                                               // stores the outputs into mapped host buffers, 0 one copy per output on the launches' stream
    uint32_t nvfp4_pair = 0;                   // NVFP4 GEMM on pairs of SMs (cta_group::2): 0 off, 1 on
    uint32_t nvfp4_group_m = 0;                // NVFP4 GEMM: token tiles per raster group, 0 = automatic
    uint32_t oneshot_max_bytes = 1536u << 10;  // all-reduce payloads up to this size take the one-shot peer exchange
    std::string last_error;
};

void comm_destroy(Ctx *ctx);

struct Weight {
    uint32_t dtype = 0;
    int device = 0;
    uint64_t n_in = 0, n_out = 0;           // local (shard) geometry
    uint64_t n_in_full = 0, n_out_full = 0; // unsharded geometry
    muser_cuda_shard shard{0, 1, 0};
    // K-quants
    uint8_t *image = nullptr; // tiles
    uint32_t row_tiles = 0;   // ceil(n_out / 16)
    uint32_t nsb = 0;         // super-block tiles per row tile
    uint32_t k_off = 0;       // elements of the first tile that precede this shard's first input
    // NVFP4
    uint8_t *packed = nullptr; // [n_out_pad][n_in/2]
    uint8_t *scales = nullptr; // swizzled [n_out_pad/128][ceil(n_in/64)][32][4][4], unsigned magnitudes
    uint64_t n_out_pad = 0;
    float scale2 = 1.0f;
    float input_scale_inv = 0.0f;
    bool has_input_scale_inv = false;
    uint64_t image_bytes = 0;
    void *tmap_cache = nullptr; // CUtensorMap of `packed` with 256-row boxes, built at repack time
    void *tmap_half = nullptr;  // the same image with 128-row boxes (fused gate/up form)
};

inline muser_cuda_status fail(Ctx *ctx, muser_cuda_status st, const std::string &msg) {
    if (ctx) ctx->last_error = msg;
    return st;
}

extern thread_local std::string g_create_error;

#define MUSER_CUDA_TRY(ctx, expr)                                                                     \
    do {                                                                                              \
        cudaError_t e__ = (expr);                                                                     \
        if (e__ != cudaSuccess)                                                                       \
            return ::muser::fail((ctx), MUSER_CUDA_ERROR,                                             \
                                 std::string(#expr) + ": " + cudaGetErrorString(e__));                \
    } while (0)

// Programmatic dependent launch: a kernel launched through launch_pdl may begin while the kernel before it in the
// stream is still running.  It calls pdl_wait() before it touches anything an earlier kernel may have written (its
// activations, the context's scratch and counters, its output); what it does before that (barrier set-up, the first
// weight-tile copies: weights are constants) overlaps the predecessor's tail and hides the launch latency.
// pdl_release() lets the next kernel start early in turn.  Both are no-ops for ordinary launches.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
#endif

inline int kquant_tile_bytes(uint32_t dtype) {
    return dtype == MUSER_DTYPE_Q4_K ? kQ4TileBytes : dtype == MUSER_DTYPE_Q5_K ? kQ5TileBytes : kQ6TileBytes;
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Launch set-up that CUDA keeps per device.  A process may hold contexts on several GPUs and drive them from several
// host threads, so nothing of it lives in unguarded function-local statics.
constexpr int kMaxDevices = 64;
// Raises cudaFuncAttributeMaxDynamicSharedMemorySize of `kernel` on `device` (which must be current) to at least
// `bytes`; remembers what it set per (kernel, device) under a lock, so repeated calls cost a table lookup.
cudaError_t ensure_dynamic_smem(const void *kernel, int device, size_t bytes);
// One slot per device for a launcher's cached plan; lock() before touching a slot.
template <typename T> struct PerDevice {
    std::mutex mu;
    T slot[kMaxDevices];
};

// ---- launchers implemented in the .cu files ---------------------------------------------------
// Where a projection kernel pushes its f32 partial sums for the one-shot all-reduce (oneshot_exchange.h): every
// rank's cell buffer, this rank's per-chunk sequence numbers (read, not bumped: the gathering kernel does that).
struct OneShotPush {
    uint8_t *peer[8];
    const uint32_t *seq;
    uint32_t rank, world;
};
bool oneshot_push_target(Ctx *, uint64_t count, OneShotPush *out);
cudaError_t launch_oneshot_gather(Ctx *, float *buf, uint64_t count, cudaStream_t);

struct Epilogue {
    const float *row_scale = nullptr;
    const void *residual = nullptr;
    const float *norm_weight = nullptr; // fused input RMSNorm: x <- (x / rms(x)) * norm_weight before the projection
    float norm_eps = 0.0f;
    float out_scale = 1.0f;             // LM-head tail (reference.rs:559-570): y <- y * out_scale,
    float softcap = 0.0f;               // then, if > 0, y <- softcap * tanh(y / softcap)
    bool all_reduce = false;            // the output is one rank's partial sum: sum it over the context's communicator
};

#ifdef __CUDACC__
__device__ __forceinline__ float logit_tail(float v, float out_scale, float softcap) {
    v *= out_scale;
    if (softcap > 0.0f) v = softcap * tanhf(v * __fdiv_rn(1.0f, softcap));
    return v;
}
#endif

muser_cuda_status launch_repack_kquant(Ctx *, Weight *, const uint8_t *dev_blocks, cudaStream_t);
muser_cuda_status launch_repack_nvfp4(Ctx *, Weight *, const uint8_t *dev_packed, const uint8_t *dev_scales,
                                      cudaStream_t);
muser_cuda_status launch_dequant(Ctx *, const Weight *, float *out, cudaStream_t);
muser_cuda_status launch_kquant_rows(Ctx *, const Weight *w, const uint32_t *rows, uint32_t n_rows, const void *x,
                                     uint32_t x_dtype, float *out, uint32_t tokens, cudaStream_t);
muser_cuda_status launch_kquant_matmul(Ctx *, const Weight *w, const Weight *w_up, const void *x, uint32_t x_dtype,
                                       void *y, uint32_t y_dtype, uint32_t tokens, const Epilogue &,
                                       cudaStream_t);
cudaError_t launch_kquant_tc(Ctx *, const Weight *w, const void *x, uint32_t x_dtype, void *y, uint32_t y_dtype,
                             uint32_t tokens, const Epilogue &, cudaStream_t);
muser_cuda_status decode_autotune(Ctx *, const Weight *const *w, const Weight *w_up, uint32_t n_jobs, uint32_t max_tokens, cudaStream_t);
cudaError_t launch_kquant_decode(Ctx *, const Weight *const *w, const Weight *w_up, uint32_t n_jobs, const void *x,
                                 uint32_t x_dtype, void *const *y, const uint32_t *y_dtype, uint32_t tokens,
                                 const Epilogue *ep, cudaStream_t, unsigned long long *amax_keys = nullptr, unsigned int *amax_flags = nullptr,
                                 const OneShotPush *push = nullptr);
cudaError_t launch_lm_head_argmax(Ctx *, const Weight *w, const void *x, uint32_t x_dtype, void *logits, uint32_t logits_dtype,
                                  uint32_t tokens, const Epilogue &ep, uint32_t *out_index, float *out_value, uint32_t *out_nonfinite,
                                  cudaStream_t);
muser_cuda_status launch_nvfp4_quantize(Ctx *, const void *x, uint32_t x_dtype, uint32_t tokens, uint64_t n_in,
                                        float input_scale_inv, uint8_t *packed, uint8_t *scales, cudaStream_t,
                                        const float *norm_weight = nullptr, float norm_eps = 0.0f);
muser_cuda_status launch_rmsnorm_rows(Ctx *, const void *x, uint32_t x_dtype, uint32_t tokens, uint64_t n_in,
                                      const float *norm_weight, float norm_eps, float *out, cudaStream_t);
struct NvFp4Out { // where a GEMM leaves its output as NVFP4 activations for the next projection
    uint8_t *packed, *scales;
    float input_scale_inv;
};
muser_cuda_status launch_nvfp4_gemm(Ctx *, const Weight *w, const uint8_t *x_packed, const uint8_t *x_scales,
                                    void *y, uint32_t y_dtype, uint32_t tokens, const Epilogue &, cudaStream_t,
                                    const Weight *w_up = nullptr, const NvFp4Out *qout = nullptr);
muser_cuda_status launch_nvfp4_gemm_group(Ctx *, const Weight *const *ws, uint32_t n, const uint8_t *x_packed, const uint8_t *x_scales,
                                          void *const *ys, uint32_t y_dtype, uint32_t tokens, cudaStream_t);
muser_cuda_status launch_nvfp4_a16(Ctx *, const Weight *w, const void *x, uint32_t x_dtype, void *y, uint32_t y_dtype, uint32_t tokens,
                                   void *workspace, size_t workspace_bytes, cudaStream_t);
muser_cuda_status launch_nvfp4_peak(Ctx *, uint32_t iters, double *flops, cudaStream_t);
muser_cuda_status launch_f16_mma_probe(Ctx *, uint32_t n_cols, uint32_t iters, double *cycles_per_mma);
muser_cuda_status nvfp4_build_tensor_map(Ctx *, Weight *);
muser_cuda_status launch_norm_residual_norm(Ctx *, float *hidden, const float *src, float *output, const float *w1, const float *w2,
                                            uint32_t tokens, uint32_t n, float eps1, float eps2, cudaStream_t);
muser_cuda_status launch_sigmoid_gate(Ctx *, float *x, const float *gate, size_t count, cudaStream_t);
muser_cuda_status launch_head_rms_norm(Ctx *, float *x, const float *w, float eps, uint32_t tokens, uint32_t heads, uint32_t head_dim, cudaStream_t);
muser_cuda_status launch_nvfp4_pipe_probe(Ctx *, uint32_t mode, uint32_t iters, uint32_t load_kib, uint32_t random, cudaStream_t);
void nvfp4_free_tensor_map(Weight *);

} // namespace muser
