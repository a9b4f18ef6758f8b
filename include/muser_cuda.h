/*
 * muser-cuda: C ABI of the B200 (sm_100a) backend for muser's quantized linear layers.
 *
 * Every entry point is what a Rust `muser-cuda` crate binds 1:1 so that the engine's
 * forward-graph drivers can select this backend the way they select Metal
 * (crates/muser-engine/src/api.rs:626-631).  Each declaration cites the reference
 * interface it stands in for.  Plain pointers and sizes only; no C++ or torch types.
 *
 * Conventions (the reference's, crates/muser-engine/src/weights.rs:398-421 and
 * src/metal/encode/qkv.rs:414-424):
 *   - weights are row-major quantized rows, rows = n_out, contiguous dim = n_in;
 *   - activations are token-major [tokens][n_in], outputs token-major [tokens][n_out];
 *   - dtype ids are the GgmlType discriminants (src/gguf/types.rs:9-39).
 *
 * Unless a comment says "host", data pointers are device pointers on the context's device.
 * Calls enqueue work on the caller's stream and never synchronize; errors detected on the
 * host come back as a status, never as an abort.  `stream` is a cudaStream_t passed as void*.
 */
#ifndef MUSER_CUDA_H
#define MUSER_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MUSER_CUDA_ABI_VERSION 3u

#if defined(__GNUC__)
#define MUSER_CUDA_API __attribute__((visibility("default")))
#else
#define MUSER_CUDA_API
#endif

/* GgmlType discriminants, src/gguf/types.rs:9-39 */
#define MUSER_DTYPE_F32 0u
#define MUSER_DTYPE_F16 1u
#define MUSER_DTYPE_Q4_K 12u
#define MUSER_DTYPE_Q5_K 13u
#define MUSER_DTYPE_Q6_K 14u
#define MUSER_DTYPE_BF16 30u
#define MUSER_DTYPE_NVFP4_E2M1 1000u
#define MUSER_DTYPE_F8_E4M3FN 1001u

/* The reference's encoders return () and debug_assert / panic on misuse
 * (src/metal/encode/qkv.rs:141-145,459,627); device trouble surfaces later as
 * MetalError::{Command,Deadline} (src/metal/context.rs:8-30).  Here every call validates
 * on the host and reports one of these. */
typedef enum muser_cuda_status {
    MUSER_CUDA_OK = 0,
    MUSER_CUDA_BAD_ARG = 1,           /* null pointer, zero size, bad enum */
    MUSER_CUDA_BAD_SHAPE = 2,         /* n_in / n_out / tokens not supported by the dtype */
    MUSER_CUDA_BAD_ALIGN = 3,         /* a device pointer is not 16-byte aligned */
    MUSER_CUDA_UNSUPPORTED_DTYPE = 4, /* supports_projection() is false for it */
    MUSER_CUDA_NAN_SCALE = 5,         /* an E4M3FN NaN code or non-finite tensor scale */
    MUSER_CUDA_ERROR = 6,             /* a CUDA runtime call failed; see last_error */
    MUSER_CUDA_NCCL_ERROR = 7,
    MUSER_CUDA_TIMEOUT = 8,           /* a bounded device-side wait gave up */
    MUSER_CUDA_WORKSPACE_TOO_SMALL = 9
} muser_cuda_status;

typedef struct muser_cuda_ctx muser_cuda_ctx;       /* one per device; thread-compatible */
typedef struct muser_cuda_weight muser_cuda_weight; /* immutable repacked device image */

/* How one projection is split across tensor-parallel ranks.  The reference has no tensor
 * parallelism (scripts/gx10/vllm/muser_vllm/connector.py:119-120 refuses it), so this has no
 * counterpart there. */
#define MUSER_SHARD_NONE 0u
#define MUSER_SHARD_ROWS 1u /* column-parallel: this rank keeps n_out/world output rows */
#define MUSER_SHARD_K 2u    /* row-parallel: this rank keeps n_in/world inputs; outputs are partial sums */
typedef struct muser_cuda_shard {
    uint32_t rank, world, axis;
} muser_cuda_shard;

/* Work fused around a projection, reproducing src/reference.rs:59-80 (rms_norm, rms_norm_mul on the input
 * rows), :511-513 (silu(gate)*up, through muser_cuda_ffn_gate_up_silu) and :475-477,536-538 (residual add). */
typedef struct muser_cuda_epilogue {
    const float *row_scale; /* [tokens] multiplies every output row, or NULL */
    const void *residual;   /* [tokens][n_out] in y's dtype, added after scaling, or NULL.  On a K-sharded weight the
                             * outputs are partial sums that the ranks add afterwards: pass the residual on ONE rank
                             * only (the others NULL), or it is added `world` times.  For the same reason softcap
                             * is refused on K shards (MUSER_CUDA_BAD_SHAPE). */
    uint32_t swiglu;        /* must be 0: the fused SwiGLU takes two weights, see muser_cuda_ffn_gate_up_silu */
    float norm_eps;         /* eps of the fused input norm (used when norm_weight is set) */
    const float *norm_weight; /* [n_in] f32 on the device, or NULL.  Set: the projection reads
                               * (x * 1/sqrt(mean(x^2) + norm_eps)) * norm_weight instead of x (rms_norm_mul,
                               * reference.rs:73-80), computed inside the kernel that stages or quantizes x.  Not
                               * available on K-sharded weights (a shard sees only part of the row). */
    float out_scale;          /* LM-head tail (src/reference.rs:559-570): every output is multiplied by out_scale
                               * (0 is read as 1, so a zeroed struct changes nothing) ... */
    float softcap;            /* ... and, when softcap > 0, becomes softcap * tanh(y / softcap); both before the residual */
    uint32_t all_reduce;      /* muser_cuda_quantized_matmul on a K-sharded weight (row-parallel o_proj, down_proj): 1 = y is one
                               * rank's partial sum and the call also sums it over the context's communicator, leaving the
                               * total in y on every rank (every rank makes the same call).  Up to 16 tokens of f32 the
                               * projection kernel stores each value into all ranks' exchange cells as its row tile finishes
                               * and a small second kernel gathers them (the transfer runs beside the projection's remaining
                               * tiles); otherwise the projection is followed by muser_cuda_all_reduce.  0 elsewhere. */
} muser_cuda_epilogue;

typedef struct muser_cuda_weight_info {
    uint32_t dtype;
    uint32_t shard_axis, shard_rank, shard_world;
    uint64_t n_in, n_out;             /* geometry this image multiplies: the local shard's */
    uint64_t n_in_full, n_out_full;   /* geometry of the unsharded tensor */
    uint64_t image_bytes;             /* device bytes of the repacked image */
    uint64_t image_hash;              /* 64-bit digest of the image bytes: repacking is deterministic */
    float scale2;
    float input_scale_inv;
    uint32_t has_input_scale_inv;
    uint32_t reserved;
} muser_cuda_weight_info;

MUSER_CUDA_API uint32_t muser_cuda_abi_version(void);

/* MetalKernels::supports_projection, src/metal/encode.rs:370-385.  True for Q4_K, Q5_K, Q6_K (the K-quant calls
 * below) and NVFP4_E2M1 (the muser_cuda_nvfp4_* calls). */
MUSER_CUDA_API int muser_cuda_supports_projection(uint32_t ggml_type);

/* MetalContext::new + MetalKernels::new (src/metal/context.rs, src/metal/encode.rs:278-280).
 * workspace_bytes sizes the one scratch arena the context owns (quantized activations of
 * the NVFP4 lane); no entry point below allocates per call. */
MUSER_CUDA_API muser_cuda_status muser_cuda_ctx_create(int device, size_t workspace_bytes, muser_cuda_ctx **out);
MUSER_CUDA_API void muser_cuda_ctx_destroy(muser_cuda_ctx *ctx);
/* Text of the most recent failure on this context (or of the last create failure when ctx is NULL). */
MUSER_CUDA_API const char *muser_cuda_last_error(const muser_cuda_ctx *ctx);
/* The bounded wait of MetalContext::wait_for_completion (src/metal/context.rs:149-211):
 * synchronizes `stream` and folds asynchronous faults and device-side give-ups into a status. */
MUSER_CUDA_API muser_cuda_status muser_cuda_sync_status(muser_cuda_ctx *ctx, void *stream);

/* No counterpart in the reference (its kernel choice is compiled in, src/metal/encode/qkv.rs:425-449).  Which kernel
 * serves a K-quant call depends on the token count: up to 16 tokens the decode kernel, from 17 the tcgen05 skinny
 * kernel where the weight is large enough.  The thresholds and the decode kernel's launch plan can be moved, e.g. to
 * force one kernel in a test.  A TC_MIN_TOKENS value above 64 switches the tensor-core skinny kernel off. */
#define MUSER_TUNE_TC_MIN_TOKENS_Q4_K 1u /* Q4_K calls with at least this many tokens take the tcgen05 kernel (default 17) */
#define MUSER_TUNE_TC_MIN_TOKENS_Q6_K 2u /* likewise for Q6_K (default 17) */
#define MUSER_TUNE_TC_MIN_ROWS 3u        /* ... if the weight has at least this many output rows (default 1024) */
#define MUSER_TUNE_DECODE_WARPS 8u       /* decode kernel: warps per CTA, even (0: from its cost model) */
#define MUSER_TUNE_DECODE_KSPLIT 9u      /* decode kernel: K slices (0: from its cost model) */
#define MUSER_TUNE_DECODE_RING 10u       /* decode kernel: weight tiles in flight per warp, 2 or 4 (0: from its cost model) */
#define MUSER_TUNE_DECODE_WSPLIT 12u      /* decode kernel: warps of a CTA that share one row tile and split K between them (0: from its cost model) */
#define MUSER_TUNE_ONESHOT_MAX_BYTES 11u /* all-reduce: f32 payloads up to this many bytes take the one-shot peer exchange (default and most 1572864; 0: always NCCL) */
#define MUSER_TUNE_NVFP4_PAIR 13u         /* NVFP4 GEMM: 0 one CTA per 128-token tile (default), 1 pairs of SMs on 256-token tiles (tcgen05 cta_group::2) */
#define MUSER_TUNE_HOST_DIRECT_OUTPUT 14u /* muser_cuda_matmul_host_groups_enqueue: how the outputs reach the host buffers.  2 (default): one cudaMemcpyAsync per output on the context's copy stream, behind an event of the launch that produced it (the copy engine needs no SM and runs beside the next launches); 1: a kernel stores them into pinned, mapped host buffers; 0: one cudaMemcpyAsync per output on the launches' own stream */
#define MUSER_TUNE_NVFP4_GROUP_M 15u /* NVFP4 GEMM: 128-token tiles per raster group (the activations one group touches stay in L2 while it sweeps the weight rows); 0 (default) = about 32 MB of activations, at least 8 tiles */
MUSER_CUDA_API muser_cuda_status muser_cuda_tuning_set(muser_cuda_ctx *ctx, uint32_t key, uint32_t value);

/* The weight-loader step that MuseWeights / bind_nvfp4 views perform on the mmap'd file
 * (src/weights.rs:171-373, src/decode.rs:148-161): takes the tensor exactly as stored
 * (K-quant: rows of blocks; NVFP4: packed E2M1 [n_out][n_in/2] plus E4M3FN scales
 * [n_out][n_in/16], scale2, optional input_scale_inv) from HOST memory and builds the
 * tiled device image the kernels read.  `shard` may be NULL (unsharded).  NVFP4 NaN scale
 * codes are rejected as the loader does (src/weights.rs:244-248). */
MUSER_CUDA_API muser_cuda_status muser_cuda_weight_repack(muser_cuda_ctx *ctx, uint32_t ggml_type, const uint8_t *host_blocks,
                                           const uint8_t *host_block_scales, float scale2,
                                           int has_input_scale_inv, float input_scale_inv, uint64_t n_in,
                                           uint64_t n_out, const muser_cuda_shard *shard,
                                           muser_cuda_weight **out);
/* Same, with the stored tensor already resident on the device. */
MUSER_CUDA_API muser_cuda_status muser_cuda_weight_repack_device(muser_cuda_ctx *ctx, uint32_t ggml_type, const uint8_t *dev_blocks,
                                                  const uint8_t *dev_block_scales, float scale2,
                                                  int has_input_scale_inv, float input_scale_inv, uint64_t n_in,
                                                  uint64_t n_out, const muser_cuda_shard *shard, void *stream,
                                                  muser_cuda_weight **out);
MUSER_CUDA_API void muser_cuda_weight_free(muser_cuda_weight *w);
MUSER_CUDA_API muser_cuda_status muser_cuda_weight_info_get(const muser_cuda_weight *w, muser_cuda_weight_info *out);

/* weights::dequant_row over every row (src/weights.rs:82-108; quant/k_block.rs:12-49,
 * quant/k_block/q6.rs:283-325, quant/nvfp4.rs:240-255): decodes the repacked image back to
 * f32 [n_out][n_in].  Results are bit-identical to the reference decoders. */
MUSER_CUDA_API muser_cuda_status muser_cuda_dequant(muser_cuda_ctx *ctx, const muser_cuda_weight *w, float *out, void *stream);

/* MetalKernels::encode_quantized_matmul (src/metal/encode/qkv.rs:414-424) and its CPU twin
 * weights::matmul (src/weights.rs:398-421) for K-quant weights (Q4_K, Q5_K, Q6_K): y[t][r] = dot(W_r, x_t).
 * x_dtype is F32 or BF16, y_dtype F32 or BF16; 1 <= tokens <= 64 (decode, decode groups as in
 * encode_quantized_decode_group qkv.rs:234-244, and speculative-verify batches).  Activations are taken as 15-bit
 * fixed point per 256 inputs up to 16 tokens (error <= amax * 2^-15 per input) and as f16 beyond (Q5_K, the LM
 * head's type, always takes the fixed-point kernel, 16 tokens at a time). */
MUSER_CUDA_API muser_cuda_status muser_cuda_quantized_matmul(muser_cuda_ctx *ctx, const muser_cuda_weight *w, const void *x,
                                              uint32_t x_dtype, void *y, uint32_t y_dtype, uint32_t tokens,
                                              const muser_cuda_epilogue *epilogue, void *stream);

/* The projections that read the same activations, in ONE launch: the reference dispatches q, k, v (and gate) of a
 * decode step inside one barrier interval (src/decode.rs:5569-5598) and groups up to four sequences per dispatch
 * (MetalKernels::encode_quantized_decode_group, src/metal/encode/qkv.rs:234-281).  1 <= n_items <= 4 K-quant weights of
 * one n_in (and, when K-sharded, one shard geometry), Q4_K and Q6_K may mix, Q5_K only with Q5_K; 1 <= tokens <= 16; each item has its own
 * output and epilogue, but the fused input norm (norm_weight / norm_eps) must be the same in all of them (or absent
 * in all), since x is staged once.  Results equal n_items calls of muser_cuda_quantized_matmul up to the order in
 * which the f32 partial sums of the K slices are added (the launch plan depends on the group's total size). */
typedef struct muser_cuda_group_item {
    const muser_cuda_weight *w;
    void *y;                             /* [tokens][w.n_out] */
    uint32_t y_dtype;                    /* F32 or BF16 */
    uint32_t reserved;                   /* 0 */
    const muser_cuda_epilogue *epilogue; /* or NULL */
} muser_cuda_group_item;
MUSER_CUDA_API muser_cuda_status muser_cuda_quantized_matmul_group(muser_cuda_ctx *ctx, const muser_cuda_group_item *items,
                                                    uint32_t n_items, const void *x, uint32_t x_dtype, uint32_t tokens,
                                                    void *stream);

/* No counterpart in the reference (its Metal pipelines have fixed threadgroup shapes).  The decode kernel's launch
 * plan (warps per CTA, how K is split between CTAs and between the warps of a CTA) comes from a cost model; this
 * call measures the model's best candidates for one projection or one group (`weights`, as they will be passed to
 * muser_cuda_quantized_matmul / _group; `w_up` non-NULL for the fused gate/up form of weights[0]) at 1 .. max_tokens
 * tokens and remembers the fastest for this device, for every later call on the same geometry in this process.
 * Every candidate is timed as a CUDA graph of back-to-back launches over temporary copies of the weight images (so
 * that they stream from HBM).  Optional load-time work: it allocates scratch (up to ~350 MB), synchronizes
 * `stream`, runs on a stream of its own, and frees the scratch. */
MUSER_CUDA_API muser_cuda_status muser_cuda_decode_autotune(muser_cuda_ctx *ctx, const muser_cuda_weight *const *weights,
                                             uint32_t n_weights, const muser_cuda_weight *w_up, uint32_t max_tokens,
                                             void *stream);

/* Diagnostics: the launch plan of the decode kernel's latest launch on this context, as (warps per CTA, K slices
 * between CTAs, K parts between the warps of a CTA, weight tiles in flight per warp). */
MUSER_CUDA_API muser_cuda_status muser_cuda_decode_last_plan(const muser_cuda_ctx *ctx, uint32_t out[4]);

/* weights::matmul_rows (src/weights.rs:425-449): the projection restricted to a list of output rows, as the
 * reference scores selected LM-head rows.  rows: n_rows row indices on the device (an index >= n_out yields NaN);
 * y: f32 [tokens][n_rows].  K-quant weights, any token count. */
MUSER_CUDA_API muser_cuda_status muser_cuda_quantized_matmul_rows(muser_cuda_ctx *ctx, const muser_cuda_weight *w,
                                                   const uint32_t *rows, uint32_t n_rows, const void *x, uint32_t x_dtype,
                                                   float *y, uint32_t tokens, void *stream);

/* The LM head with the greedy pick fused in: logits = matmul(output.weight, x), times out_scale, tanh softcap
 * (src/reference.rs:559-570, through `epilogue`, which may also carry the final norm and a row scale), then per token the
 * index of the FIRST maximum (src/api.rs:1842-1850; on the GPU the two-phase reduction of
 * shaders/ferrite/argmax_f32.metal, which keeps the lower index among equal values).  The pick happens in the
 * projection kernel's epilogue: every finishing warp raises a per-token 64-bit key (ordered value bits, inverted row)
 * with an atomic max, so the 202048-row logits never have to be written or read again.  logits: [tokens][n_out] in
 * logits_dtype (F32 or BF16), or NULL when only the pick is wanted.  out_index: [tokens] u32 on the device; out_value
 * (the winning logit, f32) and out_nonfinite (1 where some logit of the token was NaN or infinite, the condition the
 * reference refuses with NonfiniteLogits, src/api.rs:1856-1861) may be NULL.  A NaN never wins; a token whose logits are
 * all NaN yields index 0.  K-quant weights (the real model's LM head is Q5_K), unsharded, 1 <= tokens <= 16. */
MUSER_CUDA_API muser_cuda_status muser_cuda_lm_head_argmax(muser_cuda_ctx *ctx, const muser_cuda_weight *w, const void *x,
                                            uint32_t x_dtype, uint32_t tokens, const muser_cuda_epilogue *epilogue,
                                            void *logits, uint32_t logits_dtype, uint32_t *out_index, float *out_value,
                                            uint32_t *out_nonfinite, void *stream);

/* MetalKernels::encode_ffn_q4k_gate_up_silu_4r2s (src/metal/encode/ffn.rs:10-19) and the CPU lane's
 * silu_fast(gate) * up (src/reference.rs:511-513, quant/helpers.rs:72):
 * y[t][j] = silu(Wgate_j . x_t) * (Wup_j . x_t), x read once, the two projections never written out.
 * `epilogue` may be NULL; only its norm_weight / norm_eps are honoured (rms_norm_mul of the FFN input,
 * reference.rs:489).  K-quant weights (Q4_K or Q6_K): 1 <= tokens <= 16.  NVFP4 weights (both with the same input_scale_inv): any token count; x is
 * quantized into the context workspace once and one tensor-core GEMM computes both projections, each rounded
 * to f16 as the W4A4 lane returns it (quant/nvfp4.rs:337) before the SwiGLU. */
MUSER_CUDA_API muser_cuda_status muser_cuda_ffn_gate_up_silu(muser_cuda_ctx *ctx, const muser_cuda_weight *w_gate,
                                              const muser_cuda_weight *w_up, const void *x, uint32_t x_dtype,
                                              void *y, uint32_t y_dtype, uint32_t tokens,
                                              const muser_cuda_epilogue *epilogue, void *stream);

/* quant::quantize_nvfp4_activation (src/quant/nvfp4.rs:221-238) with the scale layout of the
 * GB10 producer's quantizer (scripts/gx10/vllm/muser_vllm/exact_fp4_quant.py:149-162):
 * packed [tokens][n_in/2], scales swizzled [ceil(tokens/128)][ceil(n_in/64)][32][4][4].
 * Codes and scale bytes are bit-identical to the reference. */
MUSER_CUDA_API muser_cuda_status muser_cuda_quantize_nvfp4_activation(muser_cuda_ctx *ctx, const void *x, uint32_t x_dtype,
                                                       uint32_t tokens, uint64_t n_in, float input_scale_inv,
                                                       uint8_t *packed, uint8_t *scales_swizzled, void *stream);
MUSER_CUDA_API size_t muser_cuda_nvfp4_swizzled_scale_bytes(uint64_t rows, uint64_t n_in);
/* The same quantizer behind a fused rms_norm_mul (src/reference.rs:59-80): each row is first scaled by
 * 1/sqrt(mean(x^2) + norm_eps) and multiplied by norm_weight [n_in] (f32, device), in f32, inside the kernel.
 * One call serves every projection that reads the normalized row (q, k, v; or gate and up). */
MUSER_CUDA_API muser_cuda_status muser_cuda_rmsnorm_quantize_nvfp4_activation(muser_cuda_ctx *ctx, const void *x, uint32_t x_dtype,
                                                               uint32_t tokens, uint64_t n_in, const float *norm_weight,
                                                               float norm_eps, float input_scale_inv, uint8_t *packed,
                                                               uint8_t *scales_swizzled, void *stream);

/* MetalKernels::encode_nvfp4_matmul with input_scale_inv = Some(..) (src/metal/encode/qkv.rs:128-227),
 * i.e. weights::matmul's W4A4 lane (src/weights.rs:111-121, quant/nvfp4.rs:304-338): quantizes x
 * into the context workspace, then runs the block-scaled tensor-core GEMM.  y_dtype F32, F16 or BF16
 * (F16 is the reference's output boundary, nvfp4.rs:337).
 * A weight repacked WITHOUT input_scale_inv takes the reference's weight-only lane instead (input_scale_inv = None,
 * src/weights.rs:117-121, quant::dot_nvfp4_a16_q8_f32 src/quant/nvfp4.rs:348-379): activations go to int8 per 256
 * inputs, the contraction is exact integer arithmetic, and the f16-rounded result equals the reference's bit for bit
 * (an F32 output holds that f16 value).  That lane takes no epilogue, needs n_in % 256 == 0 and tokens * (n_in + 16)
 * bytes of context workspace. */
MUSER_CUDA_API muser_cuda_status muser_cuda_nvfp4_matmul(muser_cuda_ctx *ctx, const muser_cuda_weight *w, const void *x,
                                          uint32_t x_dtype, void *y, uint32_t y_dtype, uint32_t tokens,
                                          const muser_cuda_epilogue *epilogue, void *stream);

/* MetalKernels::encode_nvfp4_w4a4_prequant_m16 (src/metal/encode/qkv.rs:13-26) generalized to any
 * token count: the GEMM alone on activations quantized earlier by
 * muser_cuda_quantize_nvfp4_activation. */
MUSER_CUDA_API muser_cuda_status muser_cuda_nvfp4_matmul_prequant(muser_cuda_ctx *ctx, const muser_cuda_weight *w,
                                                   const uint8_t *x_packed, const uint8_t *x_scales_swizzled,
                                                   void *y, uint32_t y_dtype, uint32_t tokens,
                                                   const muser_cuda_epilogue *epilogue, void *stream);

/* The NVFP4 form of muser_cuda_quantized_matmul_group (MetalKernels::encode_quantized_decode_group,
 * src/metal/encode/qkv.rs:414-449: q | k | v on the same activations in one dispatch): 2..4 NVFP4 weights with the same
 * n_in and the same input_scale_inv, the activations quantized earlier, one launch whose output tiles run through
 * all of them, so the small projections fill the SMs that a launch of their own would leave idle.  Every output is
 * bit-identical to what muser_cuda_nvfp4_matmul_prequant gives for that weight.  Plain outputs (no epilogue), all of
 * y_dtype, outputs[i] [tokens][n_out of weights[i]]. */
MUSER_CUDA_API muser_cuda_status muser_cuda_nvfp4_matmul_group_prequant(muser_cuda_ctx *ctx, const muser_cuda_weight *const *weights,
                                                         uint32_t n_weights, const uint8_t *x_packed,
                                                         const uint8_t *x_scales_swizzled, void *const *outputs,
                                                         uint32_t y_dtype, uint32_t tokens, void *stream);

/* muser_cuda_ffn_gate_up_silu for NVFP4 weights on activations quantized earlier (the pre-quantized form of
 * qkv.rs:13-26 applied to the fused FFN front half). */
MUSER_CUDA_API muser_cuda_status muser_cuda_nvfp4_ffn_gate_up_silu_prequant(muser_cuda_ctx *ctx, const muser_cuda_weight *w_gate,
                                                             const muser_cuda_weight *w_up, const uint8_t *x_packed,
                                                             const uint8_t *x_scales_swizzled, void *y, uint32_t y_dtype,
                                                             uint32_t tokens, void *stream);

/* The FFN front half feeding the down projection without a detour through numbers: silu(gate) * up as above, then
 * quant::quantize_nvfp4_activation of that f32 product (src/quant/nvfp4.rs:173-238) with the DOWN projection's static
 * input_scale_inv, inside the GEMM's epilogue.  out_packed [tokens][n_out / 2] and out_scales_swizzled
 * (muser_cuda_nvfp4_swizzled_scale_bytes(tokens, n_out) bytes) are what muser_cuda_quantize_nvfp4_activation would
 * have produced from the fused call's f32 output, byte for byte; pass them to muser_cuda_nvfp4_matmul_prequant with
 * the down weight.  n_out % 64 == 0.  The reference quantizes the intermediate in a pass of its own
 * (src/weights.rs:111-121 on the CPU lane; scripts/gx10/vllm/muser_vllm/exact_fp4_quant.py on the GB10 producer). */
MUSER_CUDA_API muser_cuda_status muser_cuda_nvfp4_ffn_gate_up_silu_requant(muser_cuda_ctx *ctx, const muser_cuda_weight *w_gate,
                                                            const muser_cuda_weight *w_up, const uint8_t *x_packed,
                                                            const uint8_t *x_scales_swizzled, uint32_t tokens,
                                                            float out_input_scale_inv, uint8_t *out_packed,
                                                            uint8_t *out_scales_swizzled, void *stream);

/* No counterpart in the reference.  The same W4A4 projection as muser_cuda_nvfp4_matmul for callers that cannot
 * allocate device memory: a driver that works out of arenas it sized once has no allocator to lend and, on the
 * step path, may not stall on the device-wide lock that cudaMalloc / cudaFree take.  This call needs no context
 * and allocates nothing: the quantized activations pass through a 2.25 MiB array that lives in the library image
 * on every GPU that loads it.  `w` is a handle made earlier by muser_cuda_weight_repack*; x and y are the caller's.
 * Limits: tokens <= 128, n_in <= 32768, else MUSER_CUDA_WORKSPACE_TOO_SMALL.  All calls on a device share that
 * array, so calls that overlap on the GPU race: keep them on one stream or order them.  The first call on a device
 * looks up the array's device address; make that call before any stream capture.  Failures leave their text in
 * muser_cuda_last_error(NULL). */
MUSER_CUDA_API muser_cuda_status muser_cuda_nvfp4_matmul_static(const muser_cuda_weight *w, const void *x, uint32_t x_dtype,
                                                                void *y, uint32_t y_dtype, uint32_t tokens, void *stream);
/* No counterpart in the reference.  muser_cuda_sync_status for the call above, which has no context: synchronizes
 * `stream` on `device` and reports MUSER_CUDA_TIMEOUT if a bounded wait inside one of that path's kernels gave up
 * since the last check (the output of such a call is incomplete), then clears the record.  Allocates nothing. */
MUSER_CUDA_API muser_cuda_status muser_cuda_static_sync_status(int device, void *stream);

/* Measurement aid, no counterpart in the reference (its kernel bench prints TMAC/s without a ceiling,
 * crates/muser-bench/src/m16.rs:755-774): enqueues a kernel in which every SM issues `iters` x 4 block-scaled FP4
 * tensor-core instructions (the GEMM's, 128 x 256 x 64) with no memory traffic, and returns the flops it will have
 * done.  Timing it gives the tensor-pipe ceiling that the prefill GEMM's roofline fraction is quoted against. */
MUSER_CUDA_API muser_cuda_status muser_cuda_fp4_peak_probe(muser_cuda_ctx *ctx, uint32_t iters, double *flops, void *stream);

/* Measurement aid, no counterpart in the reference.  The instruction mix of one 256-value slab of the NVFP4 GEMM's
 * 128 x 256 tile, issued `iters` times by one thread per SM on resident operands, so that the cost of each part can
 * be timed alone: mode 0 the slab's four MMAs; 1 its twelve scale-factor copies into tensor memory (tcgen05.cp
 * 32x128b.warpx4), then the MMAs; 2 (three copies, one MMA) four times; 3 the copies alone; 4 six 128x256b copies
 * alone; 5 those, then the MMAs; 6 nothing.  load_kib (a multiple of 18, or 0): KiB per iteration that a second
 * thread streams from the context workspace (L2-resident) into shared memory beside it, as the GEMM's producer does.
 * random_data: operands and scales are pseudo-random non-zero values instead of zeros.  Enqueues one kernel. */
MUSER_CUDA_API muser_cuda_status muser_cuda_fp4_pipe_probe(muser_cuda_ctx *ctx, uint32_t mode, uint32_t iters, uint32_t load_kib,
                                            uint32_t random_data, void *stream);

/* Measurement aid, no counterpart in the reference.  Issue interval of the instruction the K-quant skinny kernel is
 * built on: every SM issues iters x 4 tcgen05.mma kind::f16 (128 rows x n_cols x 16, n_cols in {16,32,64,128,256})
 * back to back on resident operands; returns SM clock cycles per instruction.  Synchronizes the device. */
MUSER_CUDA_API muser_cuda_status muser_cuda_f16_mma_probe(muser_cuda_ctx *ctx, uint32_t n_cols, uint32_t iters, double *cycles_per_mma);

/* Test aid, no counterpart in the reference.  Runs the give-up path of the kernels' bounded waits on its own: one
 * thread polls a barrier that nobody arrives at `polls` times (1..65536), records a give-up code as the kernels do
 * and returns.  The next muser_cuda_sync_status on the context reports MUSER_CUDA_TIMEOUT once; the context stays
 * usable. */
MUSER_CUDA_API muser_cuda_status muser_cuda_wait_probe(muser_cuda_ctx *ctx, uint32_t polls, void *stream);

/* Tensor parallelism.  The reference has none (scripts/gx10/vllm/muser_vllm/connector.py:119-120 refuses it), so
 * these have no counterpart there.  One process per GPU of one box; a context gets a communicator either from an
 * id that rank 0 made and the host carried to the other ranks (comm_init: every rank calls it, it blocks until all
 * have), or from an NCCL communicator the host already owns (comm_attach; `nccl_comm` is an ncclComm_t).  NCCL is
 * looked up at run time (libnccl.so.2); MUSER_CUDA_NCCL_ERROR reports its absence or a failed call.  At most 8 ranks
 * get the one-shot path; the set-up call synchronizes `stream`. */
#define MUSER_CUDA_COMM_ID_BYTES 128u
MUSER_CUDA_API muser_cuda_status muser_cuda_comm_unique_id(uint8_t *out, size_t out_bytes);
MUSER_CUDA_API muser_cuda_status muser_cuda_ctx_comm_init(muser_cuda_ctx *ctx, const uint8_t *id, uint32_t rank, uint32_t world, void *stream);
MUSER_CUDA_API muser_cuda_status muser_cuda_ctx_comm_attach(muser_cuda_ctx *ctx, void *nccl_comm, uint32_t rank, uint32_t world, void *stream);
/* 1 when the context's communicator has its peer buffers mapped (CUDA IPC) and small payloads avoid NCCL. */
MUSER_CUDA_API int muser_cuda_ctx_comm_has_oneshot(const muser_cuda_ctx *ctx);
/* The all-reduce(sum) after a row-parallel projection (o_proj, down_proj), in place on `buf` (count elements of F32,
 * F16 or BF16), enqueued on `stream`; every rank must make the same calls in the same order.  f32 payloads up to
 * 1.5 MiB (a decode or verify step's [tokens][hidden] partial sums) take a one-shot exchange over peer memory: each rank stores
 * its values into every rank's buffer over NVLink, each paired with the call's sequence number, polls its own buffer
 * until every rank's values are there (bounded: a give-up is reported by muser_cuda_sync_status as
 * MUSER_CUDA_TIMEOUT, and the elements that were still waiting keep this rank's partial sums) and adds them in rank
 * order, so all ranks end with identical bits.  Larger payloads and 16-bit types go to ncclAllReduce on the same
 * stream. */
MUSER_CUDA_API muser_cuda_status muser_cuda_all_reduce(muser_cuda_ctx *ctx, void *buf, uint64_t count, uint32_t dtype, void *stream);

/* weights::matmul itself (src/weights.rs:398): HOST slices in, HOST slices out, f32 both ways.
 * Copies x up, runs the device path for w's dtype, copies y back and synchronizes. */
MUSER_CUDA_API muser_cuda_status muser_cuda_matmul_host(muser_cuda_ctx *ctx, const muser_cuda_weight *w, const float *x_host,
                                         uint32_t tokens, float *y_host);

/* The same with the wait left to the caller, the way the reference's drivers encode a whole step into one command
 * buffer and wait once (src/decode.rs:5448-5460, src/metal/context.rs:149-211): the copy of x up, the projection and
 * the copy of y back are enqueued on `stream` and the call returns.  x_host and y_host must stay valid until the
 * stream has been synchronized (muser_cuda_sync_status does that and also rewinds the context's staging arena); with
 * pinned host memory the copies overlap the host's next calls.  The arena (64 MiB, allocated on first use) is the
 * only allocation; a step that outgrows it makes the call wait for the stream once and start the arena over. */
MUSER_CUDA_API muser_cuda_status muser_cuda_matmul_host_enqueue(muser_cuda_ctx *ctx, const muser_cuda_weight *w,
                                                 const float *x_host, uint32_t tokens, float *y_host, void *stream);

/* The step either side of the projections, so that a layer's non-attention work can stay on the device between two
 * projection calls.  All f32, device pointers, rows 16-byte aligned.
 *
 * muser_fused_norm_residual_rms_norm_32sg (src/shaders/ferrite/rmsnorm_batch_tail.metal:147-200), the sandwich-norm
 * tail of src/reference.rs:466-490: hidden[t] += rms_norm(src[t], eps1) * weight1 (the post-norm of a projection's
 * output with its own epsilon, onto the residual stream, in place) and, when `output` is given,
 * output[t] = rms_norm(hidden[t], eps2) * weight2 (the next pre-norm).  tokens rows of n values, n % 4 == 0. */
MUSER_CUDA_API muser_cuda_status muser_cuda_fused_norm_residual_rms_norm(muser_cuda_ctx *ctx, float *hidden, const float *src, float *output,
                                                          const float *weight1, const float *weight2, uint32_t tokens,
                                                          uint32_t n, float eps1, float eps2, void *stream);
/* The attention output gate in front of o_proj (src/reference.rs:447-455; shaders/ferrite sigmoid_gate):
 * x[i] *= 1 / (1 + exp(-gate[i])), in place; count % 4 == 0. */
MUSER_CUDA_API muser_cuda_status muser_cuda_sigmoid_gate(muser_cuda_ctx *ctx, float *x, const float *gate, uint64_t count, void *stream);
/* The per-head QK norm (src/reference.rs:384-393): every head_dim-long piece of x ([tokens][heads * head_dim], in place)
 * becomes rms_norm(piece, eps) * weight, weight [head_dim]; head_dim % 4 == 0. */
MUSER_CUDA_API muser_cuda_status muser_cuda_head_rms_norm(muser_cuda_ctx *ctx, float *x, const float *weight, float eps, uint32_t tokens,
                                           uint32_t heads, uint32_t head_dim, void *stream);

/* A whole decode step's projections through host buffers in ONE call: the drivers of the reference encode a step into
 * one command buffer (src/decode.rs:5448-5460) and group the projections that read the same hidden state
 * (src/decode.rs:5569-5598, src/metal/encode/qkv.rs:234-281).  Every group is 1..4 K-quant projections of one x_host
 * ([tokens][n_in] f32, 1 <= tokens <= 16): x is copied up once, the group runs as one launch
 * (muser_cuda_quantized_matmul_group), and the outputs y_host[i] ([tokens][n_out_i] f32) leave beside the following
 * groups' launches: by default one copy each on the context's copy stream, behind an event of the launch that made
 * them (MUSER_TUNE_HOST_DIRECT_OUTPUT selects a store kernel into pinned, mapped buffers, or copies on `stream`,
 * instead).  Pinned host buffers let the copies run asynchronously.  At most 28 groups per call.  Nothing is synchronized: wait with muser_cuda_sync_status,
 * after which the outputs are complete.  Buffers must stay valid until then.  The call can be captured into a CUDA
 * graph on `stream` (after one plain call, which makes the arena and the events) and replayed step after step: the
 * graph then reads and writes the same host buffers and the same part of the arena. */
typedef struct muser_cuda_host_group {
    const muser_cuda_weight *w[4];
    float *y_host[4];
    const float *x_host;
    uint32_t n_items;
    uint32_t tokens;
} muser_cuda_host_group;
MUSER_CUDA_API muser_cuda_status muser_cuda_matmul_host_groups_enqueue(muser_cuda_ctx *ctx, const muser_cuda_host_group *groups,
                                                        uint32_t n_groups, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* MUSER_CUDA_H */
