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

int device_sm_count();

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

#endif  // __CUDACC__

}  // namespace bitnet
