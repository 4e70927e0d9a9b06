/*
 * bitnet_cuda.h -- C ABI of libbitnet_cuda_kernels (B200 / sm_100a).
 *
 * The BitLinear forward hot path of BitNet-Rust behind plain C entry points:
 * per-token absmax int8 activation quantisation, 2-bit ternary weights in the
 * reference's packed layout, int8 x ternary contraction with int32
 * accumulation, dequantisation by weight scale x activation scale.
 *
 * Conventions
 *   - Every function returns a bitnet_status_t (0 = ok) and never aborts; the text of
 *     the last failure on the calling thread is available from bitnet_last_error_string().
 *   - All pointers named *_dev are device pointers; kernels are enqueued on the given
 *     stream and the call returns without synchronising unless stated otherwise.
 *   - M = tokens (rows of x), K = in_features, N = out_features.
 *   - Packed weights: the ternary matrix W[N,K] is flattened row-major, code = w + 1,
 *     four codes per byte, element j of a byte in bits [2j+1:2j]
 *     (bitnet-quant/src/quantization/packing.rs:352-394, utils.rs:434-475).  The buffer
 *     holds ceil(N*K/4) bytes.  Code 3 is never produced by the reference's packers and
 *     its decoders disagree on it; kernels here require it to be absent --
 *     bitnet_sanitize_packed rewrites it to code 1 (weight 0, the majority rule of
 *     gguf.rs:1139 and weight_conversion.rs:179-182) and reports how many it found.
 *   - Citations are paths inside the reference project.
 */
#ifndef BITNET_CUDA_H
#define BITNET_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* A cudaStream_t, spelled without the CUDA headers so that any FFI can bind it. */
typedef void *bitnet_stream_t;

/* Status codes; one per variant of the reference's CudaError
 * (bitnet-cuda/src/error.rs:7-56) plus the two this library adds. */
typedef int32_t bitnet_status_t;
enum {
    BITNET_OK = 0,
    BITNET_ERR_CUDA_NOT_ENABLED = 1,     /* CudaError::CudaNotEnabled: no usable device */
    BITNET_ERR_CUDA_DRIVER = 2,          /* CudaError::CudaDriver */
    BITNET_ERR_DEVICE = 3,               /* CudaError::DeviceError */
    BITNET_ERR_MEMORY_ALLOCATION = 4,    /* CudaError::MemoryAllocation */
    BITNET_ERR_KERNEL_EXECUTION = 5,     /* CudaError::KernelExecution */
    BITNET_ERR_INVALID_CONFIG = 6,       /* CudaError::InvalidConfig */
    BITNET_ERR_UNSUPPORTED_OPERATION = 7,/* CudaError::UnsupportedOperation */
    BITNET_ERR_STREAM_SYNC = 8,          /* CudaError::StreamSync */
    BITNET_ERR_UNSUPPORTED_DTYPE = 9,    /* CudaError::UnsupportedDataType */
    BITNET_ERR_INCOMPATIBLE_SHAPES = 10, /* CudaError::IncompatibleShapes */
    BITNET_ERR_PERFORMANCE = 11,         /* CudaError::PerformanceDegradation */
    BITNET_ERR_NULL_POINTER = 12,        /* added: a required pointer was NULL */
    BITNET_ERR_WORKSPACE = 13            /* added: workspace missing, misaligned or too small */
};

/* CudaError::is_recoverable (bitnet-cuda/src/error.rs:88-103): 1 or 0. */
int32_t bitnet_is_recoverable(bitnet_status_t status);
const char *bitnet_status_string(bitnet_status_t status);
const char *bitnet_last_error_string(void);

/* Which kernel family runs a forward call. */
enum {
    BITNET_PATH_AUTO = 0,    /* decode kernel for M <= 16, cluster GEMM up to 128 tokens, persistent GEMM beyond */
    BITNET_PATH_DECODE = 1,  /* weight-streaming GEMV family, M <= 16, K % 64 == 0 */
    BITNET_PATH_PREFILL = 2, /* TMA + tcgen05 int8 GEMM, K % 128 == 0 */
    BITNET_PATH_GENERIC = 3, /* any M, K, N (rows may start mid-byte); slow, exact */
    BITNET_PATH_CLUSTER = 4  /* TMA + tcgen05 int8 GEMM with K split over a thread-block cluster, 1 <= M <= 128, K % 128 == 0 */
};

enum {
    BITNET_FLAG_PDL = 1u, /* launch with programmatic dependent launch: the kernel starts
                             fetching weights before the preceding kernel on the stream has
                             finished and only then waits for it */
    BITNET_FLAG_THROUGHPUT = 2u /* decode shapes: smaller CTAs (four consumer warps, at most two
                                   weight stages), so that CTAs of four launches share an SM.
                                   A single call gets slower; independent calls issued on
                                   several streams get about a quarter more throughput */
};

/* Options of a forward call; zero-initialise for the defaults. */
typedef struct bitnet_forward_opts {
    int32_t path;           /* BITNET_PATH_* */
    uint32_t flags;         /* BITNET_FLAG_* */
    int8_t *q_out_dev;      /* optional [M,K]: the int8 activations */
    float *a_scale_out_dev; /* optional [M]: absmax/127 per token (1 when the row is all zero) */
    int32_t *acc_out_dev;   /* optional [M,N]: the int32 accumulators */
    size_t ldy;             /* row stride of y (and acc_out) in elements; 0 means N */
    int32_t stages;         /* decode kernel: depth of the shared-memory weight ring (0 = choose) */
    int32_t n_peers;        /* 0, or the number of entries of y_peers_dev (at most BITNET_MAX_PEERS) */
    /* Output-feature-split layer on several GPUs: when n_peers > 0 the kernel's epilogue stores every
       output element into each of these buffers (this GPU's and its peers', mapped into this process:
       CUDA IPC, symmetric memory or cudaDeviceEnablePeerAccess) instead of y_dev alone, which replaces
       the all-gather of the column slices by plain peer stores over NVLink.  Each pointer addresses
       the slice's first column in that GPU's full-width output (row stride ldy).  Written by the
       decode kernel (M <= 16) and by the persistent GEMM (path BITNET_PATH_PREFILL, one weight
       matrix, no acc_out); the caller synchronises the GPUs afterwards.  No counterpart in the
       reference, which has no multi-GPU code. */
    float *y_peers_dev[8];
} bitnet_forward_opts;
#define BITNET_MAX_PEERS 8

/* Device facts (CudaBackend::validate_device_capabilities, bitnet-cuda/src/backend.rs:192-213). */
typedef struct bitnet_device_info {
    int32_t device_id;
    int32_t cc_major, cc_minor;
    int32_t sm_count;
    int32_t l2_bytes;
    int32_t max_smem_per_block;
    size_t free_bytes, total_bytes;
    char name[128];
} bitnet_device_info;

bitnet_status_t bitnet_device_count(int32_t *count);                  /* lib.rs:56-64 device_count() */
/* Device-side waits are bounded; one that runs out raises a flag instead of hanging.
 * Returns and clears the flags (bit 0: a decode-kernel stage wait gave up, bit 1: a GEMM-kernel wait;
 * the outputs of that launch are incomplete).  Synchronises the device.  The reference has no counterpart: its kernel has
 * no waits. */
bitnet_status_t bitnet_device_error_flags(uint32_t *flags_out);
bitnet_status_t bitnet_query_device(int32_t device_id, bitnet_device_info *out);

/* ---- the hot path --------------------------------------------------------------- */

/* Legacy single-token entry point: out[n] = sum_k (code(W[n,k]) - 1) * a[k], int32.
 * Replaces launch_w2a8_gemv_optimized / w2a8_gemv_kernel
 * (bitnet-cuda/src/kernels/w2a8_gemv.cu:100-106, :188-214); note the reference calls
 * n_out "m" and k_in "k".  Unlike the reference it reports launch errors. */
bitnet_status_t bitnet_w2a8_gemv(const uint8_t *weights_dev, const int8_t *activations_dev,
                                 int32_t *output_dev, size_t n_out, size_t k_in,
                                 bitnet_stream_t stream);

/* Same symbol and signature as the reference's launcher (w2a8_gemv.cu:188-195), for
 * callers that already link against it; errors are only recorded (see
 * bitnet_last_error_string), as the void return leaves no other channel. */
void launch_w2a8_gemv_optimized(const uint8_t *weights, const int8_t *activations,
                                int32_t *output, size_t m, size_t k, bitnet_stream_t stream);

/* Fused BitLinear forward: y[M,N] = dequant(contract(quant(x[M,K]), W)).
 * Semantics: TernaryProcessor::quantize_activations + ternary_matmul_generic
 * (bitnet-inference/src/engine/ternary_operations.rs:117-172, :283-338) with int32
 * accumulation and y = acc * (w_scale * absmax/127), output [M,N] row-major; it is what
 * BitLinearLayer::forward (transformer_layers.rs:119-202) and
 * BitLinearForward::forward_with_quantized_weights (bitnet-quant/src/bitlinear/forward.rs:95)
 * compute for a 2-D input.  The argument order follows the reference's only batched
 * quantised-GEMM signature (bitnet-metal/src/mps/matrix_ops.rs:318-341).
 * workspace_dev: bitnet_bitlinear_workspace_size() bytes, 256-byte aligned; may be NULL
 * when that size is 0 (the decode path needs none). */
bitnet_status_t bitnet_bitlinear_forward(const uint8_t *weights_dev, float w_scale,
                                         const float *x_dev, float *y_dev,
                                         size_t M, size_t K, size_t N,
                                         const bitnet_forward_opts *opts,
                                         void *workspace_dev, size_t workspace_bytes,
                                         bitnet_stream_t stream);
bitnet_status_t bitnet_bitlinear_workspace_size(size_t M, size_t K, size_t N, int32_t path,
                                                size_t *bytes);

/* The same forward for the decode shapes (1 <= M <= 16, K % 64 == 0, K <= 16384, or 8192 when
 * M > 8) with no workspace argument and no allocation of any kind: its scratch is a fixed
 * 136 KiB array built into the library, resident on every GPU that loads it.  It has no
 * counterpart in the reference; it exists for callers that run inside a memory budget fixed at
 * start-up, or that are called while their host forbids allocation calls, and so can neither
 * cudaMalloc nor lend a buffer.  Other shapes are refused with BITNET_ERR_UNSUPPORTED_OPERATION
 * (or BITNET_ERR_WORKSPACE if the scratch would not fit).  All calls on a device share the
 * array: calls that may overlap on the GPU race on it.  The first call on a device resolves
 * the array's address and should be made before any stream capture. */
bitnet_status_t bitnet_bitlinear_forward_static(const uint8_t *weights_dev, float w_scale,
                                                const float *x_dev, float *y_dev,
                                                size_t M, size_t K, size_t N,
                                                bitnet_stream_t stream);

/* Per-token absmax int8 quantisation on its own
 * (TernaryProcessor::quantize_activations, ternary_operations.rs:117-172):
 * q = clamp(round_half_away(x * (127/absmax)), -128, 127), a_scale = absmax/127. */
bitnet_status_t bitnet_quantize_activations(const float *x_dev, size_t M, size_t K,
                                            int8_t *q_dev, float *a_scale_dev,
                                            bitnet_stream_t stream);

/* FFN block: y = down( up(x) * relu(gate(x))^2 ), each projection a BitLinear that
 * re-quantises its input per token (FeedForwardNetwork::forward,
 * bitnet-inference/src/engine/transformer_layers.rs:603-623).
 * h_dev: caller-provided [M,ffn] fp32 buffer that receives the gated activations. */
bitnet_status_t bitnet_ffn_forward(const uint8_t *w_gate_dev, float s_gate,
                                   const uint8_t *w_up_dev, float s_up,
                                   const uint8_t *w_down_dev, float s_down,
                                   const float *x_dev, float *h_dev, float *y_dev,
                                   size_t M, size_t hidden, size_t ffn,
                                   const bitnet_forward_opts *opts,
                                   void *workspace_dev, size_t workspace_bytes,
                                   bitnet_stream_t stream);
bitnet_status_t bitnet_ffn_workspace_size(size_t M, size_t hidden, size_t ffn, int32_t path,
                                          size_t *bytes);

/* ---- decoder-layer glue fused around the projections ------------------------------------------ */

/* Row-wise operations applied to x on its way into a projection, inside the launch that quantises it
 * (TransformerBlock::forward, bitnet-inference/src/engine/transformer_layers.rs:675-709: the residual add
 * in front of a sub-layer, and SubLNNormalization::forward, :356-386: (x - mean) / sqrt(var + eps) *
 * weight + bias over the feature dimension, var with the n - 1 divisor of candle-core 0.8's var_keepdim).
 * All members optional; zero-initialise.  Needs K % 16 == 0 and K <= 16384. */
typedef struct bitnet_row_glue {
    const float *residual_dev;    /* [M,K]: the row that is normalised and quantised is x + residual */
    float *sum_out_dev;           /* [M,K]: receives x + residual (may be x itself: the hidden state updated in place) */
    const float *norm_weight_dev; /* [K]: SubLN weight; NULL = no normalisation */
    const float *norm_bias_dev;   /* [K]: SubLN bias (required with the weight) */
    float norm_eps;
    float *normed_out_dev;        /* [M,K]: receives the normalised fp32 row (for parity tests) */
} bitnet_row_glue;

/* Up to three BitLinear layers that read the same x (the q, k and v projections of
 * MultiHeadAttention::forward, transformer_layers.rs:469-475), their packed weights stacked along the
 * output features in one buffer; every member but the last must end on a 16-byte boundary of the packed
 * stream (rows * K % 64 == 0).  Each keeps its own weight scale. */
typedef struct bitnet_stack {
    int32_t n_members;   /* 1..3 */
    size_t rows[3];      /* output features of each member */
    float scales[3];
} bitnet_stack;

/* y[M, sum(rows)] = the stacked BitLinears applied to glue(x).  Same semantics as one
 * bitnet_bitlinear_forward per member on the glued row; for M <= 16 everything runs in two launches (the
 * quantiser launch carries the glue, one decode launch streams all members).  workspace_dev:
 * bitnet_bitlinear_fused_workspace_size() bytes. */
bitnet_status_t bitnet_bitlinear_forward_fused(const uint8_t *weights_dev, const bitnet_stack *stack,
                                               const float *x_dev, const bitnet_row_glue *glue, float *y_dev,
                                               size_t M, size_t K, const bitnet_forward_opts *opts,
                                               void *workspace_dev, size_t workspace_bytes, bitnet_stream_t stream);
bitnet_status_t bitnet_bitlinear_fused_workspace_size(size_t M, size_t K, size_t N_total, int32_t path, size_t *bytes);

/* bitnet_ffn_forward with row glue in front of the gate and up projections (the post-attention
 * normalisation and the attention residual of TransformerBlock::forward, transformer_layers.rs:690-701). */
bitnet_status_t bitnet_ffn_forward_fused(const uint8_t *w_gate_dev, float s_gate,
                                         const uint8_t *w_up_dev, float s_up,
                                         const uint8_t *w_down_dev, float s_down,
                                         const float *x_dev, const bitnet_row_glue *glue, float *h_dev, float *y_dev,
                                         size_t M, size_t hidden, size_t ffn,
                                         const bitnet_forward_opts *opts,
                                         void *workspace_dev, size_t workspace_bytes, bitnet_stream_t stream);
bitnet_status_t bitnet_ffn_fused_workspace_size(size_t M, size_t hidden, size_t ffn, int32_t path, size_t *bytes);

/* The glue alone: sum_out = x + residual, normed_out = SubLN(x + residual). */
bitnet_status_t bitnet_row_glue_forward(const float *x_dev, size_t M, size_t K, const bitnet_row_glue *glue,
                                        bitnet_stream_t stream);

/* ---- decode-step kernels around the projections ------------------------------------------------- */

/* Attention of ONE new token per sequence over a bf16 KV cache, grouped-query form
 * (MultiHeadAttention::forward, transformer_layers.rs:460-547: softmax(q k^T / sqrt(head_dim)) v; RoPE is
 * the identity in the reference, :278-289; cache shape [batch, kv_heads, max_seq, head_dim] as
 * KVCache::initialize_cache, bitnet-inference/src/cache/kv_cache.rs:104-121, in bf16 instead of f32).
 * qkv_dev [B, ldq] holds the new token's q at column 0 (n_heads * head_dim values), k at k_off, v at v_off
 * (n_kv_heads * head_dim each).  pos_dev[b] = tokens already cached for sequence b: the kernel stores the
 * new k and v (rounded to bf16) at that position and attends over positions 0..pos[b].  It does not
 * advance pos_dev.  out_dev [B, n_heads * head_dim].  head_dim 64 or 128; n_heads / n_kv_heads in
 * {1,2,4,8}.  n_splits: CTAs per (sequence, KV head) along the keys (bitnet_attention_splits suggests
 * one); scratch_dev: bitnet_attention_scratch_size() bytes, zero-filled once by the caller before the
 * first launch, 256-byte aligned (NULL allowed when n_splits == 1). */
bitnet_status_t bitnet_attention_decode(const float *qkv_dev, size_t ldq, size_t k_off, size_t v_off,
                                        void *k_cache_dev, void *v_cache_dev, const int32_t *pos_dev, float *out_dev,
                                        size_t B, size_t n_heads, size_t n_kv_heads, size_t head_dim, size_t max_seq,
                                        int32_t n_splits, void *scratch_dev, size_t scratch_bytes, bitnet_stream_t stream);
bitnet_status_t bitnet_attention_scratch_size(size_t B, size_t n_heads, size_t n_kv_heads, size_t head_dim,
                                              int32_t n_splits, size_t *bytes);
int32_t bitnet_attention_splits(size_t B, size_t n_kv_heads, size_t max_context);

/* SamplingConfig (bitnet-inference/src/engine/sampling.rs:11-45). */
typedef struct bitnet_sampling_config {
    float temperature;      /* 1.0 */
    uint32_t top_k;         /* 0 = off */
    float top_p;            /* 1.0 = off */
    uint64_t seed;          /* sequence i draws from a generator seeded with seed + i (BatchSampler::new, :419-426) */
    int32_t deterministic;  /* 1 = argmax */
} bitnet_sampling_config;
void bitnet_sampling_config_default(bitnet_sampling_config *cfg);

/* TokenSampler::sample for B sequences (sampling.rs:106-189): argmax (first index on ties) when
 * deterministic; otherwise logits / temperature, top-k and top-p filters (ties with the cut-off value are
 * kept), softmax, and one draw per sequence with the reference's generator (state * 1103515245 + 12345,
 * :273-276; u = bits 16..39 of the state / 2^24), taking the first index whose running probability exceeds
 * u.  The reference's filters and softmax are stubs and its draw ignores the logits; this does what its
 * doc comments describe.  rng_state_dev [B] uint64 (bitnet_seed_sampler), next_ids_dev [B] int32. */
bitnet_status_t bitnet_sample_tokens(const float *logits_dev, size_t B, size_t vocab,
                                     const bitnet_sampling_config *cfg, uint64_t *rng_state_dev,
                                     int32_t *next_ids_dev, bitnet_stream_t stream);
bitnet_status_t bitnet_seed_sampler(uint64_t *rng_state_dev, size_t B, uint64_t seed, bitnet_stream_t stream);

/* ---- packed-weight helpers (device) -------------------------------------------------- */

/* BitPacked2BitPacker::pack / unpack (packing.rs:352-394) on device buffers.
 * n_values ternary int8 values <-> ceil(n_values/4) bytes. */
bitnet_status_t bitnet_pack_ternary(const int8_t *w_dev, size_t n_values, uint8_t *packed_dev,
                                    bitnet_stream_t stream);
bitnet_status_t bitnet_unpack_ternary(const uint8_t *packed_dev, size_t n_values, int8_t *w_dev,
                                      bitnet_stream_t stream);
/* Rewrites code 3 to code 1 in place and adds the number found to *count_dev (a device
 * uint64 the caller zeroed; may be NULL). */
bitnet_status_t bitnet_sanitize_packed(uint8_t *packed_dev, size_t n_bytes,
                                       unsigned long long *count_dev, bitnet_stream_t stream);

/* absmean_quantize_weights + BitPacked2BitPacker::pack on device buffers (weights.rs:807-857,
 * packing.rs:352-388): n_values fp32 weights -> ceil(n_values/4) packed bytes and the fp32 scale
 * sum(W t) / sum(t t) in *scale_dev.  Sums run in double precision in a fixed order. */
bitnet_status_t bitnet_quantize_pack_weights(const float *w_dev, size_t n_values, uint8_t *packed_dev,
                                             float *scale_dev, void *workspace_dev, size_t workspace_bytes,
                                             bitnet_stream_t stream);
bitnet_status_t bitnet_quantize_pack_weights_workspace_size(size_t n_values, size_t *bytes);

/* One-time preparation of a packed weight buffer for the kernels of this library: the hook that
 * the reference names enable_weight_permutation / permute_weights_16x32
 * (bitnet-cuda/src/kernels/w2a8_gemv.rs:21, :259).  No permutation is needed here -- every kernel
 * consumes the canonical layout (layout_id 0, the only one accepted) -- so preparation is the
 * in-place removal of code 3 plus the shape checks of the fast paths: *fast_paths receives a mask
 * (bit 0: decode kernel usable for M <= 16, bit 1: tensor-core GEMM usable); shapes that fit
 * neither still run on the generic kernel.  count_dev as in bitnet_sanitize_packed. */
bitnet_status_t bitnet_prepare_weights(uint8_t *packed_dev, size_t N, size_t K, int32_t layout_id,
                                       unsigned long long *count_dev, uint32_t *fast_paths,
                                       bitnet_stream_t stream);

/* ---- host-side backend (handle based) ------------------------------------------------- */
/* Mirrors CudaBackend / CudaBackendConfig / W2A8GemvConfig / CudaMemoryManager /
 * CudaStream / PerformanceStats of the reference's bitnet-cuda crate
 * (backend.rs:14-37, :40-213, :262-290; kernels/w2a8_gemv.rs:15-60; memory.rs:47-186;
 * stream.rs:31-207) so that a Rust shim can stay a list of declarations. */

typedef struct bitnet_backend bitnet_backend;   /* CudaBackend */
typedef struct bitnet_weights bitnet_weights;   /* a packed, uploaded weight tensor */

enum { BITNET_GRID_FIXED = 0, BITNET_GRID_DYNAMIC = 1, BITNET_GRID_OCCUPANCY = 2 };    /* GridStrategy */
enum { BITNET_COALESCE_NONE = 0, BITNET_COALESCE_BASIC = 1, BITNET_COALESCE_AGGRESSIVE = 2 }; /* CoalescingLevel */

typedef struct bitnet_w2a8_config {     /* W2A8GemvConfig, w2a8_gemv.rs:15-38 */
    uint32_t block_size;                /* must be a non-zero multiple of 32 */
    int32_t grid_strategy;
    uint32_t grid_fixed;                /* GridStrategy::Fixed(n) */
    int32_t enable_weight_permutation;
    int32_t enable_dp4a;
    int32_t coalescing_level;
} bitnet_w2a8_config;

typedef struct bitnet_backend_config {  /* CudaBackendConfig, backend.rs:14-37 */
    size_t device_id;
    size_t memory_pool_size;
    size_t num_streams;
    int32_t enable_profiling;
    bitnet_w2a8_config w2a8_config;
} bitnet_backend_config;

typedef struct bitnet_performance_stats { /* PerformanceStats, backend.rs:262-272 */
    uint64_t total_w2a8_operations;
    float average_execution_time_us;
    float memory_utilization_percent;
    float peak_bandwidth_gbps;
} bitnet_performance_stats;

void bitnet_backend_config_default(bitnet_backend_config *cfg);       /* Default impls */
bitnet_status_t bitnet_backend_create(const bitnet_backend_config *cfg, bitnet_backend **out); /* CudaBackend::new */
void bitnet_backend_destroy(bitnet_backend *b);
bitnet_status_t bitnet_backend_stream(bitnet_backend *b, size_t index, bitnet_stream_t *out);  /* CudaBackend::stream */
bitnet_status_t bitnet_backend_synchronize(bitnet_backend *b);                                  /* CudaBackend::synchronize */
bitnet_status_t bitnet_backend_get_performance_stats(bitnet_backend *b, bitnet_performance_stats *out);

/* CudaMemoryManager::{allocate, copy_to_device, copy_to_host} (memory.rs:79,:130,:143);
 * allocations are zero-filled and charged against memory_pool_size. */
bitnet_status_t bitnet_backend_allocate(bitnet_backend *b, size_t bytes, void **dev_ptr);
bitnet_status_t bitnet_backend_free(bitnet_backend *b, void *dev_ptr);
bitnet_status_t bitnet_backend_copy_to_device(bitnet_backend *b, void *dst_dev, const void *src_host, size_t bytes);
bitnet_status_t bitnet_backend_copy_to_host(bitnet_backend *b, void *dst_host, const void *src_dev, size_t bytes);
bitnet_status_t bitnet_backend_memory_usage(bitnet_backend *b, size_t *allocated, size_t *pool_size);

/* CudaBackend::w2a8_gemv (backend.rs:129-157) with its length checks (:217-257): lengths
 * are element counts of the three device buffers; mismatches give
 * BITNET_ERR_INCOMPATIBLE_SHAPES, a bad stream index BITNET_ERR_INVALID_CONFIG. */
bitnet_status_t bitnet_backend_w2a8_gemv(bitnet_backend *b,
                                         const uint8_t *weights_dev, size_t weights_len,
                                         const int8_t *activations_dev, size_t activations_len,
                                         int32_t *output_dev, size_t output_len,
                                         size_t m, size_t k, size_t stream_idx);

/* Weight life cycle of BitLinear (bitnet-quant/src/bitlinear/layer.rs:236-326): pack and
 * upload once per weight version, launch-only afterwards, drop on update_weights. */
bitnet_status_t bitnet_backend_upload_packed(bitnet_backend *b, const uint8_t *packed_host,
                                             size_t N, size_t K, float w_scale, bitnet_weights **out);
bitnet_status_t bitnet_backend_upload_ternary(bitnet_backend *b, const int8_t *ternary_host,
                                              size_t N, size_t K, float w_scale, bitnet_weights **out);
/* Full-precision weights [N,K]: absmean ternary quantisation (absmean_quantize_weights,
 * bitnet-quant/src/quantization/weights.rs:807-857) and packing on the device; the scale it computes
 * becomes the handle's w_scale. */
bitnet_status_t bitnet_backend_upload_f32(bitnet_backend *b, const float *weights_host,
                                          size_t N, size_t K, bitnet_weights **out);
/* A ternary tensor of a GGUF file as GgufLoader::decode_ternary_weights reads it
 * (bitnet-inference/src/gguf.rs:1089-1165): 8 bytes of metadata (f32 scale, f32 offset, little endian)
 * followed by the 2-bit codes; the codes are uploaded as they are, never unpacked on the host. */
bitnet_status_t bitnet_backend_upload_gguf_ternary(bitnet_backend *b, const uint8_t *tensor_host, size_t tensor_bytes,
                                                   size_t N, size_t K, float *offset_out, bitnet_weights **out);
bitnet_status_t bitnet_backend_free_weights(bitnet_backend *b, bitnet_weights *w);
bitnet_status_t bitnet_weights_info(const bitnet_weights *w, size_t *N, size_t *K, float *w_scale,
                                    const uint8_t **packed_dev);

/* BitLinear forward on device buffers through the backend (workspace from the pool). */
bitnet_status_t bitnet_backend_bitlinear_forward(bitnet_backend *b, const bitnet_weights *w,
                                                 const float *x_dev, float *y_dev, size_t M,
                                                 const bitnet_forward_opts *opts, size_t stream_idx);
/* The call a host-side user makes (BitLinearLayer::forward on host tensors,
 * transformer_layers.rs:119-202): x and y are HOST buffers [M,K] / [M,N]; the copies in
 * and out run on the chosen stream and the call returns after y is complete. */
bitnet_status_t bitnet_backend_bitlinear_forward_host(bitnet_backend *b, const bitnet_weights *w,
                                                      const float *x_host, float *y_host, size_t M,
                                                      const bitnet_forward_opts *opts, size_t stream_idx);
/* FFN block on host buffers (FeedForwardNetwork::forward, transformer_layers.rs:603-623). */
bitnet_status_t bitnet_backend_ffn_forward_host(bitnet_backend *b, const bitnet_weights *gate,
                                                const bitnet_weights *up, const bitnet_weights *down,
                                                const float *x_host, float *y_host, size_t M,
                                                const bitnet_forward_opts *opts, size_t stream_idx);
/* Asynchronous form: the copies and launches are queued on the chosen stream and the call returns
 * (the reference's model for its stream pool: launches are asynchronous per stream and
 * CudaBackend::synchronize joins them, bitnet-cuda/src/backend.rs:129-178).  x_host may be reused at
 * once; y_host is complete after bitnet_backend_synchronize or after the next host-buffer call on
 * the same stream.  One call may be in flight per stream: spread calls over the backend's streams. */
bitnet_status_t bitnet_backend_ffn_forward_host_async(bitnet_backend *b, const bitnet_weights *gate,
                                                      const bitnet_weights *up, const bitnet_weights *down,
                                                      const float *x_host, float *y_host, size_t M,
                                                      const bitnet_forward_opts *opts, size_t stream_idx);

/* Page-locks / releases a host buffer of the caller (cudaHostRegister), so that the copies of the
 * host-buffer calls read and write it directly.  The reference's memory manager has no pinned
 * allocations (memory.rs:130-160 copies from pageable slices); this is an addition. */
bitnet_status_t bitnet_backend_pin_host(bitnet_backend *b, void *host_ptr, size_t bytes);
bitnet_status_t bitnet_backend_unpin_host(bitnet_backend *b, void *host_ptr);

/* A fixed batch of independent FFN blocks as one replayable unit: what a caller of the reference
 * writes as a loop of asynchronous launches spread over the stream pool followed by
 * CudaBackend::synchronize (bitnet-cuda/src/backend.rs:129-178), with the loop recorded once.
 * Creation binds, per call, the weights, the token count and the HOST buffers x [M,hidden] and
 * y [M,hidden]; it allocates the device buffers from the backend's pool, runs the batch once, and
 * records it as a CUDA graph: per call host->device copy of x, the block, device->host copy of y,
 * the calls dealt round-robin to n_lanes streams (0 = 8) so that independent blocks overlap on the
 * device.  Host buffers that are page-locked (bitnet_backend_pin_host, cudaMallocHost, ...) are
 * copied from and to directly; others are staged through pinned memory inside the run.
 * Calls of one shape with at most 16 tokens each run as up to three FFN groups (bitnet_ffn_group_*,
 * below) instead of per-call launches: all input copies are queued at once on the lanes, a group's
 * kernels start when its own inputs have landed, and its outputs leave while the next group computes (the
 * groups' scratch is allocated with cudaMalloc, outside the backend's pool and its byte budget).
 * bitnet_backend_ffn_plan_run replays the batch and returns when every y_host is complete; the
 * caller refreshes the bound x_host buffers between runs.  One run at a time per plan. */
typedef struct bitnet_ffn_plan bitnet_ffn_plan;
typedef struct bitnet_ffn_call {
    const bitnet_weights *gate, *up, *down;
    size_t M;
    const float *x_host;
    float *y_host;
} bitnet_ffn_call;
bitnet_status_t bitnet_backend_ffn_plan_create(bitnet_backend *b, const bitnet_ffn_call *calls, size_t n_calls,
                                               const bitnet_forward_opts *opts, size_t n_lanes,
                                               bitnet_ffn_plan **out);
bitnet_status_t bitnet_backend_ffn_plan_run(bitnet_ffn_plan *plan);
void bitnet_backend_ffn_plan_destroy(bitnet_ffn_plan *plan);

/* ---- a group of independent FFN blocks as four launches ------------------------------------------------
 * Decode-time blocks of one shape (hidden -> ffn -> hidden, at most 16 tokens each) that do not depend on one
 * another: the same computation as bitnet_ffn_forward per member (FeedForwardNetwork::forward,
 * bitnet-inference/src/engine/transformer_layers.rs:608-629), bit for bit, but the whole group runs as one
 * quantiser launch + one persistent gate/up launch + one quantiser launch + one persistent down launch, each
 * streaming the weights of ALL members (a block of a 2B-class model alone is too short a launch to bring the
 * memory system to speed).  The reference has no counterpart: its caller loops over the blocks.
 * Creation (on the current device) binds every member's device pointers and allocates the group's scratch
 * (tables, quantised-activation images, the gated intermediate); a run enqueues the four launches on `stream`
 * and may be captured into a CUDA graph.  The caller refreshes the bound x buffers between runs; one run at a
 * time per group, on the device it was created on.  Needs hidden % 64 == 0, ffn % 64 == 0 and 16-byte aligned
 * buffers; widths the grouped kernel cannot split over its warps (hidden above 7680 or ffn above 15360; from
 * nine tokens per member on, 4096 and 8192) are refused with BITNET_ERR_UNSUPPORTED_OPERATION at creation. */
typedef struct bitnet_ffn_group bitnet_ffn_group;
typedef struct bitnet_ffn_group_member {
    const uint8_t *gate_packed_dev, *up_packed_dev, *down_packed_dev; /* canonical packed [ffn,hidden/4], [ffn,hidden/4], [hidden,ffn/4] */
    float gate_scale, up_scale, down_scale;
    const float *x_dev;   /* [M, hidden] */
    float *y_dev;         /* [M, hidden] */
    size_t M;             /* 1..16 */
} bitnet_ffn_group_member;
bitnet_status_t bitnet_ffn_group_create(const bitnet_ffn_group_member *members, size_t n_members, size_t hidden,
                                        size_t ffn, bitnet_ffn_group **out);
bitnet_status_t bitnet_ffn_group_run(bitnet_ffn_group *group, cudaStream_t stream);
void bitnet_ffn_group_destroy(bitnet_ffn_group *group);

/* The same for plain BitLinear calls of one shape [N, K] (TernaryProcessor::quantize_activations +
 * ternary_matmul_generic per member, ternary_operations.rs:117-172, :283-338): a quantiser launch and ONE persistent
 * launch over the weights of every member; bit-identical to bitnet_bitlinear_forward per member.  N need not be a
 * multiple of 16; ldy = 0 means N. */
typedef struct bitnet_bitlinear_group bitnet_bitlinear_group;
typedef struct bitnet_bitlinear_group_member {
    const uint8_t *packed_dev;  /* canonical packed [N, K/4] */
    float w_scale;
    const float *x_dev;         /* [M, K] */
    float *y_dev;               /* [M, ldy] */
    size_t M;                   /* 1..16 */
    size_t ldy;
} bitnet_bitlinear_group_member;
bitnet_status_t bitnet_bitlinear_group_create(const bitnet_bitlinear_group_member *members, size_t n_members, size_t K,
                                              size_t N, bitnet_bitlinear_group **out);
bitnet_status_t bitnet_bitlinear_group_run(bitnet_bitlinear_group *group, cudaStream_t stream);
void bitnet_bitlinear_group_destroy(bitnet_bitlinear_group *group);

/* ---- exchange step of the output-feature-split layer ------------------------------------------------- */
/* Every GPU holds y[:, its column slice]; all need y[M, N].  No counterpart in the reference, which has no
 * multi-GPU code.
 * Peer-store form: this GPU's slice y_local_dev [M, n_local] (row stride ld_local) is written into every entry of
 * y_peers_dev (n_peers pointers, each to the slice's first column in one GPU's full-width output of row stride ldy,
 * mapped into this process: CUDA IPC, symmetric memory or peer access).  The caller synchronises the GPUs
 * afterwards.  (bitnet_forward_opts.y_peers_dev does the same from the decode kernel's epilogue, without this pass.) */
bitnet_status_t bitnet_allgather_output(const float *y_local_dev, size_t M, size_t n_local, size_t ld_local,
                                        float *const *y_peers_dev, int32_t n_peers, size_t ldy, bitnet_stream_t stream);
/* NCCL form.  The library finds NCCL at run time (dlopen of libnccl.so.2, the copy already in the process if there
 * is one); without it these return BITNET_ERR_UNSUPPORTED_OPERATION.  bitnet_nccl_unique_id on one rank, the 128
 * bytes handed to the others by the caller's own means, bitnet_nccl_comm_create on every rank with its device
 * current.  bitnet_allgather_output_nccl: ncclAllGather of the fp32 slices into staging_dev [n_ranks, M, n_local],
 * then the local reordering into y_full_dev [M, n_ranks * n_local] (row stride ldy). */
bitnet_status_t bitnet_nccl_unique_id(uint8_t *id_out /* 128 bytes */);
bitnet_status_t bitnet_nccl_comm_create(const uint8_t *id, int32_t n_ranks, int32_t rank, void **comm_out);
bitnet_status_t bitnet_nccl_comm_destroy(void *comm);
bitnet_status_t bitnet_allgather_output_nccl(void *comm, const float *y_local_dev, size_t M, size_t n_local,
                                             float *staging_dev, float *y_full_dev, int32_t n_ranks, size_t ldy,
                                             bitnet_stream_t stream);

/* ---- decode step of a whole model (handle based) ------------------------------------------------- */
/* ForwardPassPipeline (bitnet-inference/src/engine/forward_pass_pipeline.rs:146-362) for one new token per
 * sequence with a KV cache: token embedding, num_layers transformer blocks (TransformerBlock::forward,
 * transformer_layers.rs:675-709: SubLN -> attention -> residual -> SubLN -> FFN -> residual), the
 * language-model head (a BitLinear on the last hidden state, no final normalisation, :283-291) and the
 * sampler.  Device memory comes from the backend's pool (size it for the model: packed weights, the fp32
 * embedding table, 2 x layers x max_batch x kv_heads x max_seq x head_dim bf16 of cache, max_batch x vocab
 * fp32 logits).  All sequences of a batch advance together, one token per step. */
typedef struct bitnet_decoder bitnet_decoder;

typedef struct bitnet_decoder_config {   /* ForwardPassConfig + TransformerConfig, forward_pass_pipeline.rs:80-118 */
    size_t vocab_size, hidden_size, num_layers, num_heads, num_kv_heads, head_dim, ffn_size, max_seq_len, max_batch;
    float norm_eps;                       /* rms_norm_eps */
} bitnet_decoder_config;

typedef struct bitnet_decoder_layer {     /* one TransformerBlock's parameters, HOST pointers */
    const uint8_t *q_packed, *k_packed, *v_packed, *o_packed;   /* [heads*head_dim, hidden], [kv*head_dim, hidden] x2, [hidden, heads*head_dim] */
    const uint8_t *gate_packed, *up_packed, *down_packed;       /* [ffn, hidden] x2, [hidden, ffn] */
    float q_scale, k_scale, v_scale, o_scale, gate_scale, up_scale, down_scale;
    const float *input_norm_weight, *input_norm_bias;           /* input_layernorm, [hidden] */
    const float *post_norm_weight, *post_norm_bias;             /* post_attention_layernorm, [hidden] */
} bitnet_decoder_layer;

enum {
    BITNET_DECODER_LOGITS = 0,      /* fp32 [batch, vocab] of the last generation step */
    BITNET_DECODER_HIDDEN = 1,      /* fp32 [batch, hidden]: the last hidden state */
    BITNET_DECODER_POSITIONS = 2,   /* int32 [batch]: tokens cached per sequence */
    BITNET_DECODER_KEY_CACHE = 3,   /* bf16 [layers, max_batch, kv_heads, max_seq, head_dim] */
    BITNET_DECODER_VALUE_CACHE = 4
};

void bitnet_decoder_config_default(bitnet_decoder_config *cfg);
bitnet_status_t bitnet_decoder_create(bitnet_backend *b, const bitnet_decoder_config *cfg, bitnet_decoder **out);
void bitnet_decoder_destroy(bitnet_decoder *d);
bitnet_status_t bitnet_decoder_load_embedding(bitnet_decoder *d, const float *table_host);      /* [vocab, hidden] */
bitnet_status_t bitnet_decoder_load_layer(bitnet_decoder *d, size_t index, const bitnet_decoder_layer *weights);
bitnet_status_t bitnet_decoder_load_lm_head(bitnet_decoder *d, const uint8_t *packed_host, float scale);  /* [vocab, hidden] */
/* KVCache::reset (kv_cache.rs:168-172): forget every cached token. */
bitnet_status_t bitnet_decoder_reset(bitnet_decoder *d);
/* Steps are replayed as CUDA graphs recorded on first use (default); 0 launches kernel by kernel. */
bitnet_status_t bitnet_decoder_set_graphs(bitnet_decoder *d, int32_t enabled);
/* Context tokens: ids_host [B, T] row-major; each of the T steps caches one token per sequence, nothing
 * is sampled.  Returns when done. */
bitnet_status_t bitnet_decoder_feed(bitnet_decoder *d, const int32_t *ids_host, size_t B, size_t T);
/* Generation (ForwardPassPipeline::generate, forward_pass_pipeline.rs:311-362): ids_host [B] is the last
 * known token of each sequence; n_new steps, each feeding its sampled token to the next, without a host
 * round trip in between; out_host [B, n_new].  eos_id >= 0: a sequence that samples it is finished and
 * keeps emitting it (GenerationState::should_stop); the loop ends early once every sequence has.
 * *steps_run receives the steps taken. */
bitnet_status_t bitnet_decoder_decode(bitnet_decoder *d, const int32_t *ids_host, size_t B, size_t n_new,
                                      const bitnet_sampling_config *sampling, int32_t eos_id,
                                      int32_t *out_host, size_t *steps_run);
/* reset + feed(prompt[:, :-1]) + decode(prompt[:, -1]): prompt_host [B, prompt_len], out_host [B, max_new_tokens]. */
bitnet_status_t bitnet_decoder_generate(bitnet_decoder *d, const int32_t *prompt_host, size_t B, size_t prompt_len,
                                        size_t max_new_tokens, const bitnet_sampling_config *sampling,
                                        int32_t eos_id, int32_t *out_host, size_t *steps_run);
/* Copies an internal buffer (BITNET_DECODER_*) to the host, for parity tests. */
bitnet_status_t bitnet_decoder_read(bitnet_decoder *d, int32_t what, void *host, size_t bytes);

#ifdef __cplusplus
}
#endif
#endif /* BITNET_CUDA_H */
