// NVFP4 W4A4 projection for callers that must not allocate.
//
// muser's forward-graph drivers own every buffer they touch: weights are views into the mapped model file and
// activations live in arenas sized once per session, and the operator they call "allocates nothing"
// (crates/muser-engine/src/decode.rs:669-731, src/metal/buffer.rs:98-120).  A driver written that way has no
// allocator to lend, and on the step path it may not take the device-wide lock that cudaMalloc and cudaFree hold.
// muser_cuda_nvfp4_matmul needs a context because a context owns the scratch that the quantized activations pass
// through; this entry point keeps that scratch in the library image instead, so it needs neither a context nor
// any allocation: the caller hands in the weight handle it made at load time, its activations and its output.
//
// The scratch is one file-scope __device__ array per GPU that loads the library (2.25 MiB, held until the
// process exits).  In host code the array's name is only a stand-in for the device object; the address that a
// kernel or a tensor map can use comes from cudaGetSymbolAddress, asked once per device with that device
// current.  The first call on a device does that set-up, so make the first call outside any stream capture.
//
// Limits: tokens <= 128 and n_in <= 32768 (decode groups and speculative-verify batches); larger calls are
// refused with MUSER_CUDA_WORKSPACE_TOO_SMALL.  All calls on a device share the one array: two calls that overlap
// on the GPU (different streams, or graphs replayed concurrently) race on it, so keep them on one stream or
// order them with events.  The array keeps whatever the previous call left; nothing in it has to start at zero,
// because every call rewrites all scale slots of its 128-row group (rows past `tokens` as zeros) and the GEMM
// never reads code bytes past `tokens` rows (its tensor map ends there).
#include <mutex>

#include "common.cuh"

namespace muser {
namespace {

constexpr uint32_t kStaticMaxTokens = 128;
constexpr uint64_t kStaticMaxNIn = 32768;
constexpr size_t kStaticPackedBytes = (size_t)kStaticMaxTokens * (kStaticMaxNIn / 2);  // E2M1 codes, 2 per byte
constexpr size_t kStaticScaleBytes = (size_t)(kStaticMaxNIn / 64) * 512;               // one 128-row group of scales

static __device__ __align__(256) uint8_t g_static_scratch[kStaticPackedBytes + kStaticScaleBytes];
static __device__ __align__(256) int g_static_status[4]; // word 1: a bounded wait inside the GEMM gave up

struct DeviceSetup {
    bool ready = false;
    uint8_t *scratch = nullptr;
    int *status = nullptr;
    int sm_count = 0;
};
constexpr int kMaxDevices = 64;
DeviceSetup g_setup[kMaxDevices];
std::mutex g_setup_mutex;

// Resolves the device addresses of the two arrays above for `device` (which must be current).
muser_cuda_status device_setup(int device, DeviceSetup **out) {
    if (device < 0 || device >= kMaxDevices) {
        g_create_error = "device index out of range for the static scratch table";
        return MUSER_CUDA_BAD_ARG;
    }
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    DeviceSetup &s = g_setup[device];
    if (!s.ready) {
        void *scratch = nullptr, *status = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&scratch, g_static_scratch);
        if (e == cudaSuccess) e = cudaGetSymbolAddress(&status, g_static_status);
        if (e != cudaSuccess) {
            g_create_error = std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(e);
            return MUSER_CUDA_ERROR;
        }
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (e != cudaSuccess || sms < 1) {
            g_create_error = "cudaDeviceGetAttribute(multiProcessorCount) failed";
            return MUSER_CUDA_ERROR;
        }
        s.sm_count = sms;
        s.scratch = reinterpret_cast<uint8_t *>(scratch);
        s.status = reinterpret_cast<int *>(status);
        s.ready = true;
    }
    *out = &s;
    return MUSER_CUDA_OK;
}

muser_cuda_status refuse(muser_cuda_status st, const std::string &why) {
    g_create_error = why;
    return st;
}

} // namespace
} // namespace muser

using namespace muser;

extern "C" muser_cuda_status muser_cuda_nvfp4_matmul_static(const muser_cuda_weight *wp, const void *x, uint32_t x_dtype,
                                                            void *y, uint32_t y_dtype, uint32_t tokens, void *stream) {
    const Weight *w = reinterpret_cast<const Weight *>(wp);
    if (!w || !x || !y) return refuse(MUSER_CUDA_BAD_ARG, "null argument");
    if (w->dtype != MUSER_DTYPE_NVFP4_E2M1 || !w->has_input_scale_inv)
        return refuse(MUSER_CUDA_UNSUPPORTED_DTYPE, "the static-scratch entry point takes NVFP4 weights with an input_scale_inv");
    if (x_dtype != MUSER_DTYPE_F32 && x_dtype != MUSER_DTYPE_BF16)
        return refuse(MUSER_CUDA_UNSUPPORTED_DTYPE, "activations must be f32 or bf16");
    if (y_dtype != MUSER_DTYPE_F32 && y_dtype != MUSER_DTYPE_BF16 && y_dtype != MUSER_DTYPE_F16)
        return refuse(MUSER_CUDA_UNSUPPORTED_DTYPE, "unsupported output dtype");
    if (tokens == 0) return refuse(MUSER_CUDA_BAD_SHAPE, "tokens must be positive");
    if (tokens > kStaticMaxTokens || w->n_in > kStaticMaxNIn)
        return refuse(MUSER_CUDA_WORKSPACE_TOO_SMALL,
                      "the static scratch serves tokens <= 128 and n_in <= 32768; this call has tokens = " +
                          std::to_string(tokens) + ", n_in = " + std::to_string(w->n_in) +
                          " (use muser_cuda_nvfp4_matmul with a context workspace)");
    if (!aligned16(x) || !aligned16(y)) return refuse(MUSER_CUDA_BAD_ALIGN, "x and y must be 16-byte aligned");
    cudaError_t e = cudaSetDevice(w->device);
    if (e != cudaSuccess) return refuse(MUSER_CUDA_ERROR, std::string("cudaSetDevice: ") + cudaGetErrorString(e));
    DeviceSetup *setup = nullptr;
    muser_cuda_status st = device_setup(w->device, &setup);
    if (st != MUSER_CUDA_OK) return st;

    Ctx call; // plumbing for the launchers only: nothing in it is allocated
    call.device = w->device;
    call.dev_status = setup->status;
    call.sm_count = setup->sm_count;
    uint8_t *packed = setup->scratch, *scales = setup->scratch + kStaticPackedBytes;
    st = launch_nvfp4_quantize(&call, x, x_dtype, tokens, w->n_in, w->input_scale_inv, packed, scales, (cudaStream_t)stream);
    if (st == MUSER_CUDA_OK)
        st = launch_nvfp4_gemm(&call, w, packed, scales, y, y_dtype, tokens, Epilogue{}, (cudaStream_t)stream);
    if (st != MUSER_CUDA_OK) g_create_error = call.last_error;
    return st;
}

// The static path's muser_cuda_sync_status: it has no context, so the give-up word of its kernels' bounded waits
// lives beside the scratch array and is read here.
extern "C" muser_cuda_status muser_cuda_static_sync_status(int device, void *stream) {
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return refuse(MUSER_CUDA_ERROR, std::string("cudaSetDevice: ") + cudaGetErrorString(e));
    DeviceSetup *setup = nullptr;
    muser_cuda_status st = device_setup(device, &setup);
    if (st != MUSER_CUDA_OK) return st;
    int flags[4] = {0, 0, 0, 0};
    e = cudaMemcpyAsync(flags, setup->status, sizeof(flags), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return refuse(MUSER_CUDA_ERROR, std::string("static status read: ") + cudaGetErrorString(e));
    if (flags[1]) {
        cudaMemsetAsync(setup->status, 0, sizeof(flags), (cudaStream_t)stream);
        return refuse(MUSER_CUDA_TIMEOUT, "a device-side bounded wait gave up on the static-scratch path (code " + std::to_string(flags[1]) + ")");
    }
    return MUSER_CUDA_OK;
}
