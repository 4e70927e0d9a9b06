// Shared internals of libbitnet_cuda_kernels: error plumbing and the exact fp32
// arithmetic of the activation quantiser.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/bitnet_cuda.h"

namespace bitnet {

// Records the message for bitnet_last_error_string() and returns `status`.
bitnet_status_t fail(bitnet_status_t status, const char *fmt, ...);
bitnet_status_t check_cuda(cudaError_t err, const char *what);
bitnet_status_t check_launch(const char *kernel_name);

#define BITNET_TRY(expr)                                   \
    do {                                                   \
        bitnet_status_t _st = (expr);                      \
        if (_st != BITNET_OK) return _st;                  \
    } while (0)

#define BITNET_CUDA(expr) BITNET_TRY(::bitnet::check_cuda((expr), #expr))

inline cudaStream_t as_stream(bitnet_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Row-wise glue of a decoder layer that the activation quantiser applies on its way: the residual
// add in front of a sub-layer, and the sub-layer normalisation (SubLNNormalization::forward,
// bitnet-inference/src/engine/transformer_layers.rs:356-386: (x - mean) / sqrt(var + eps) * weight + bias,
// var with the n - 1 divisor of candle's var_keepdim).  All members optional.
struct RowPre {
    const float *residual;   // [M,K]: the row that is normalised and quantised is x + residual
    float *sum_out;          // [M,K]: receives x + residual (may alias x)
    const float *norm_w;     // [K]: SubLN weight; null = no normalisation
    const float *norm_b;     // [K]: SubLN bias
    float eps;
    float *normed_out;       // [M,K]: receives the normalised fp32 row (parity tests)
};

// Row-major output of the activation quantiser for the tensor-core kernels.
struct RowsOut {
    int8_t *q_perm;   // [M,K] int8, every 16-wide k group transposed (byte 4j+i holds k = 4i+j)
    int *rowsum;      // [M] sum_k q[m,k]
    float *a_scale;   // [M] absmax / 127
};

// Launchers of the kernel families (defined next to their kernels).
struct ForwardArgs {
    const uint8_t *wp;
    float w_scale;
    const float *x;      // fp32 activations [M,K] (nullptr when x_i8 is used)
    const int8_t *x_i8;  // already-quantised activations (legacy GEMV), M == 1
    float *y;            // fp32 out [M,ldy] (nullptr for the legacy GEMV)
    int32_t *acc_out;    // optional int32 out [M,ldy]
    int8_t *q_out;       // optional [M,K]
    float *a_scale_out;  // optional [M]
    // gated dual mode (FFN first half): wp = gate weights, wp2 = up weights,
    // y receives up * relu(gate)^2
    const uint8_t *wp2;
    float w_scale2;
    size_t M, K, N, ldy;
    uint32_t flags;
    int stages;          // decode kernel: weight ring depth (0 = choose)
    // per-token absmax keys exchanged between chained decode launches (FFN): [ctas][16] each
    const unsigned *amax_in;
    int n_amax_in;
    unsigned *amax_out;
    // decode path scratch for the quantised-activation image (decode_image_bytes); optional
    void *image_ws;
    size_t image_ws_bytes;
    bool force_split;    // quantise through the image even for a single token
    bool image_ready;    // image_ws already holds this launch's image (an earlier launch of the same K and plan wrote it)
    const RowPre *pre;   // decode path: residual add / normalisation done by the quantiser launch (needs image_ws)
    // several BitLinears that share x, their weights stacked along N: rows [0, seg_end[0]) use w_scale,
    // [seg_end[0], seg_end[1]) seg_scale[0], the rest seg_scale[1]; n_seg = 0 for a single matrix
    int n_seg;
    size_t seg_end[2];
    float seg_scale[2];
    // output-feature split over several GPUs: the epilogue stores to every one of these (decode kernel)
    float *y_peers[8];
    int n_peers;
};

bitnet_status_t launch_decode(const ForwardArgs &a, cudaStream_t stream);
bool decode_supports(size_t M, size_t K, size_t N);
bool decode_supports_dual(size_t M, size_t K, size_t N);   // gate and up in one launch
int decode_grid(size_t N);                                  // CTAs of a decode launch over N output features
size_t decode_image_bytes(size_t M, size_t K, size_t N, bool dual);   // 0 when the kernel quantises by itself
size_t decode_image_bytes_always(size_t M, size_t K, size_t N, bool dual);   // size of the image if one is used

bitnet_status_t launch_quantize_rows(const float *x, size_t M, size_t K, int8_t *q, float *a_scale,
                                     cudaStream_t stream);
bitnet_status_t launch_generic(const uint8_t *wp, float w_scale, const int8_t *q, const float *a_scale,
                               float *y, int32_t *acc_out, size_t M, size_t K, size_t N, size_t ldy,
                               cudaStream_t stream);
bitnet_status_t launch_gate_relu2(const float *up, const float *gate, float *h, size_t n, cudaStream_t stream);

bool prefill_supports(size_t M, size_t K, size_t N);
size_t prefill_workspace_bytes(size_t M, size_t K, size_t N);
bitnet_status_t launch_prefill(const ForwardArgs &a, void *workspace, size_t workspace_bytes, cudaStream_t stream);
bitnet_status_t prefill_take_error_flags(unsigned *flags);

// Cluster split-K tensor-core GEMM for a few dozen tokens (midm_gemm.cu).
bool midm_supports(size_t M, size_t K, size_t N);
bool midm_can_run(size_t M, size_t K, size_t N, bool pair);
size_t midm_workspace_bytes(size_t M, size_t K);
bitnet_status_t launch_midm(const ForwardArgs &a, void *workspace, size_t workspace_bytes, bool ready, cudaStream_t stream);
bitnet_status_t midm_take_error_flags(unsigned *flags);
bitnet_status_t group_take_error_flags(unsigned *flags);   // decode_group.cu

int device_sm_count();
bitnet_status_t launch_quantize_rows_glued(const float *x, size_t M, size_t K, const RowPre *pre, const RowsOut &rows,
                                           int8_t *q_out, float *a_scale_out, uint32_t flags, cudaStream_t stream);

// Stand-alone row glue (residual add and/or SubLN) for the paths whose quantiser does not take it:
// writes x + residual to pre.sum_out and the normalised row to pre.normed_out.  K % 16 == 0, K <= 16384.
bitnet_status_t launch_row_pre(const float *x, size_t M, size_t K, const RowPre &pre, uint32_t flags, cudaStream_t stream);

// Decode-step kernels around the projections (decoder_kernels.cu).
bitnet_status_t launch_embed_gather(const int *ids, const float *table, float *x, size_t M, size_t hidden, size_t vocab,
                                    cudaStream_t stream);
size_t attention_scratch_bytes(size_t B, size_t n_heads, size_t n_kv, size_t head_dim, size_t n_splits);
int attention_splits(size_t B, size_t n_kv, size_t max_context);
bitnet_status_t launch_attention_decode(const float *qkv, size_t ldq, size_t k_off, size_t v_off, void *kcache, void *vcache,
                                        const int *pos, float *out, size_t B, size_t n_heads, size_t n_kv, size_t head_dim,
                                        size_t max_seq, int n_splits, void *scratch, size_t scratch_bytes, uint32_t flags,
                                        cudaStream_t stream);
bitnet_status_t launch_sample(const float *logits, size_t B, size_t vocab, const bitnet_sampling_config &cfg,
                              unsigned long long *rng, int *next, int *ids_feed, int *pos, int *history, int *step_counter,
                              int eos_id, int *finished, uint32_t flags, cudaStream_t stream);
bitnet_status_t launch_seed_rng(unsigned long long *rng, size_t B, unsigned long long seed, cudaStream_t stream);

#ifdef __CUDACC__

// Rust f32::round / C roundf: nearest, ties away from zero, exact for every float.
// |t| < 2^23 here (the quantiser feeds values in [-127, 127] up to rounding), where
// trunc and the subtraction are exact.
__device__ __forceinline__ float round_half_away(float t)
{
    const float r = truncf(t);
    const float d = fabsf(__fsub_rn(t, r));
    return d >= 0.5f ? __fadd_rn(r, copysignf(1.0f, t)) : r;
}

// scale = 127/absmax (1 when absmax == 0): ternary_operations.rs:148-152.
__device__ __forceinline__ float quant_scale(float absmax)
{
    return absmax > 0.0f ? __fdiv_rn(127.0f, absmax) : 1.0f;
}

// a_scale = absmax/127 (1 when absmax == 0): the factor the dequantiser multiplies by.
__device__ __forceinline__ float dequant_scale(float absmax)
{
    return absmax > 0.0f ? __fdiv_rn(absmax, 127.0f) : 1.0f;
}

// q = clamp(round(x*scale), -128, 127): ternary_operations.rs:157-160.  NaN -> 0.
__device__ __forceinline__ int quantize_one(float x, float scale)
{
    float r = round_half_away(__fmul_rn(x, scale));
    if (!(r == r)) return 0;
    r = fminf(fmaxf(r, -128.0f), 127.0f);
    return __float2int_rz(r);
}

// |x| as an unsigned key that orders like the float (non-negative floats compare as ints);
// NaN maps to 0 so that, like f32::max, it never wins the fold.
__device__ __forceinline__ unsigned abs_key(float x)
{
    const unsigned b = __float_as_uint(x) & 0x7fffffffu;
    return b > 0x7f800000u ? 0u : b;
}

// The decoder-layer glue of RowPre on a row held in registers by a 512-thread CTA (thread t owns the
// 16-wide groups t and t + 512 of row m, n_groups = K / 16 <= 1024): residual add, then SubLN.
// Sums run in a fixed order (lane tree, then the sixteen warps in turn), mean first, then the centred
// sum of squares with the n - 1 divisor.  Every thread of the CTA must call it.
__device__ __forceinline__ void apply_row_pre(float4 (&f)[2][4], const RowPre &pre, int m, int K, int tid, float (&s_fsum)[2][16])
{
    const int n_groups = K / 16;
    if (pre.residual) {   // the hidden state takes the sub-layer's output before it is normalised
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int G = tid + u * 512;
            if (G < n_groups) {
                const float4 *rsrc = reinterpret_cast<const float4 *>(pre.residual + (size_t)m * K + (size_t)G * 16);
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    const float4 r4 = __ldg(rsrc + v);
                    f[u][v].x = __fadd_rn(f[u][v].x, r4.x); f[u][v].y = __fadd_rn(f[u][v].y, r4.y);
                    f[u][v].z = __fadd_rn(f[u][v].z, r4.z); f[u][v].w = __fadd_rn(f[u][v].w, r4.w);
                }
                if (pre.sum_out) {
                    float4 *dst = reinterpret_cast<float4 *>(pre.sum_out + (size_t)m * K + (size_t)G * 16);
#pragma unroll
                    for (int v = 0; v < 4; ++v) dst[v] = f[u][v];
                }
            }
        }
    }
    if (pre.norm_w) {
        auto block_sum = [&](float v, int slot) {
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
            if ((tid & 31) == 0) s_fsum[slot][tid >> 5] = v;
            __syncthreads();
            float t = 0.0f;
#pragma unroll
            for (int w = 0; w < 16; ++w) t = __fadd_rn(t, s_fsum[slot][w]);
            return t;
        };
        float part = 0.0f;
#pragma unroll
        for (int u = 0; u < 2; ++u)
            if (tid + u * 512 < n_groups) {
#pragma unroll
                for (int v = 0; v < 4; ++v)
                    part = __fadd_rn(part, __fadd_rn(__fadd_rn(f[u][v].x, f[u][v].y), __fadd_rn(f[u][v].z, f[u][v].w)));
            }
        const float mean = __fdiv_rn(block_sum(part, 0), (float)K);
        part = 0.0f;
#pragma unroll
        for (int u = 0; u < 2; ++u)
            if (tid + u * 512 < n_groups) {
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    const float a = __fsub_rn(f[u][v].x, mean), b2 = __fsub_rn(f[u][v].y, mean);
                    const float c = __fsub_rn(f[u][v].z, mean), d = __fsub_rn(f[u][v].w, mean);
                    part = __fadd_rn(part, __fadd_rn(__fadd_rn(__fmul_rn(a, a), __fmul_rn(b2, b2)), __fadd_rn(__fmul_rn(c, c), __fmul_rn(d, d))));
                }
            }
        const float var = __fdiv_rn(block_sum(part, 1), (float)(K > 1 ? K - 1 : 1));
        const float sd = __fsqrt_rn(__fadd_rn(var, pre.eps));
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int G = tid + u * 512;
            if (G < n_groups) {
                const float4 *wsrc = reinterpret_cast<const float4 *>(pre.norm_w + (size_t)G * 16);
                const float4 *bsrc = reinterpret_cast<const float4 *>(pre.norm_b + (size_t)G * 16);
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    const float4 w4 = __ldg(wsrc + v), b4 = __ldg(bsrc + v);
                    f[u][v].x = __fadd_rn(__fmul_rn(__fdiv_rn(__fsub_rn(f[u][v].x, mean), sd), w4.x), b4.x);
                    f[u][v].y = __fadd_rn(__fmul_rn(__fdiv_rn(__fsub_rn(f[u][v].y, mean), sd), w4.y), b4.y);
                    f[u][v].z = __fadd_rn(__fmul_rn(__fdiv_rn(__fsub_rn(f[u][v].z, mean), sd), w4.z), b4.z);
                    f[u][v].w = __fadd_rn(__fmul_rn(__fdiv_rn(__fsub_rn(f[u][v].w, mean), sd), w4.w), b4.w);
                }
                if (pre.normed_out) {
                    float4 *dst = reinterpret_cast<float4 *>(pre.normed_out + (size_t)m * K + (size_t)G * 16);
#pragma unroll
                    for (int v = 0; v < 4; ++v) dst[v] = f[u][v];
                }
            }
        }
    }
}

#endif  // __CUDACC__

}  // namespace bitnet
