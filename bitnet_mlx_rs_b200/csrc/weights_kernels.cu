// Weight preparation on the device: absmean ternary quantisation of an fp32 weight matrix straight into the
// packed 2-bit layout, and its scale.
//
// Semantics: absmean_quantize_weights (bitnet-quant/src/quantization/weights.rs:807-857): threshold =
// 0.7 * mean|W| (:829-831); t = sign(W) * (|W| > threshold) (apply_ternary_quantization, :482-496); scale =
// sum(W * t) / sum(t * t), 1 when the denominator is below f32 epsilon (compute_ternary_scale, :546-559);
// packing as BitPacked2BitPacker::pack (packing.rs:352-388): code = t + 1, four codes per byte, first in the
// low bits.  The reductions run in double precision in a fixed order (per thread, lane tree, warps in turn,
// blocks in turn), so the result does not depend on scheduling.
#include "common.cuh"

namespace bitnet {

constexpr int WQ_THREADS = 256;
constexpr int WQ_MAX_BLOCKS = 1024;

__device__ __forceinline__ double wq_block_sum(double v, double *s_part)
{
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = v;
    __syncthreads();
    double t = 0.0;
#pragma unroll
    for (int w = 0; w < WQ_THREADS / 32; ++w) t += s_part[w];
    return t;
}

// partial[b] = sum of |w| over block b's share (grid-stride over 4-element groups)
__global__ void __launch_bounds__(WQ_THREADS) wq_abs_partial_kernel(const float *__restrict__ w, size_t n, double *__restrict__ partial)
{
    __shared__ double s_part[WQ_THREADS / 32];
    double acc = 0.0;
    const size_t groups = (n + 3) / 4;
    for (size_t g = (size_t)blockIdx.x * WQ_THREADS + threadIdx.x; g < groups; g += (size_t)gridDim.x * WQ_THREADS) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const size_t idx = g * 4 + i;
            if (idx < n) acc += fabs((double)__ldg(w + idx));
        }
    }
    const double t = wq_block_sum(acc, s_part);
    if (threadIdx.x == 0) partial[blockIdx.x] = t;
}

// threshold = 0.7f * (float)(sum / n): one thread adds the block partials in order
__global__ void wq_threshold_kernel(const double *__restrict__ partial, int n_blocks, size_t n, float *__restrict__ threshold)
{
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        double s = 0.0;
        for (int b = 0; b < n_blocks; ++b) s += partial[b];
        const float mean_abs = n ? (float)(s / (double)n) : 0.0f;
        *threshold = __fmul_rn(mean_abs, 0.7f);
    }
}

// one packed byte per thread and step; partial[2b], partial[2b+1] = sum(w*t), sum(t*t) of block b's share
__global__ void __launch_bounds__(WQ_THREADS) wq_ternarize_pack_kernel(const float *__restrict__ w, size_t n, const float *__restrict__ threshold,
                                                                       uint8_t *__restrict__ packed, double *__restrict__ partial)
{
    __shared__ double s_part[WQ_THREADS / 32];
    const float thr = *threshold;
    double num = 0.0, den = 0.0;
    const size_t groups = (n + 3) / 4;
    for (size_t g = (size_t)blockIdx.x * WQ_THREADS + threadIdx.x; g < groups; g += (size_t)gridDim.x * WQ_THREADS) {
        unsigned byte = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const size_t idx = g * 4 + i;
            if (idx < n) {
                const float v = __ldg(w + idx);
                int t = 0;
                if (fabsf(v) > thr) t = (v > 0.0f) - (v < 0.0f);
                byte |= (unsigned)(t + 1) << (2 * i);
                num += (double)v * (double)t;
                den += (double)(t * t);
            }   // padding positions keep code 0, as the reference's packer pads with zeros (packing.rs:364-368)
        }
        packed[g] = (uint8_t)byte;
    }
    const double tn = wq_block_sum(num, s_part);
    const double td = wq_block_sum(den, s_part);
    if (threadIdx.x == 0) { partial[2 * blockIdx.x] = tn; partial[2 * blockIdx.x + 1] = td; }
}

__global__ void wq_scale_kernel(const double *__restrict__ partial, int n_blocks, float *__restrict__ scale)
{
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        double num = 0.0, den = 0.0;
        for (int b = 0; b < n_blocks; ++b) { num += partial[2 * b]; den += partial[2 * b + 1]; }
        *scale = fabs(den) < 1.1920929e-07 ? 1.0f : (float)(num / den);
    }
}

}  // namespace bitnet

using namespace bitnet;

extern "C" bitnet_status_t bitnet_quantize_pack_weights_workspace_size(size_t n_values, size_t *bytes)
{
    if (!bytes) return fail(BITNET_ERR_NULL_POINTER, "bitnet_quantize_pack_weights_workspace_size: null output");
    (void)n_values;
    *bytes = align_up(2 * WQ_MAX_BLOCKS * sizeof(double), 256) + 256;   // block partials, the threshold
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_quantize_pack_weights(const float *w_dev, size_t n_values, uint8_t *packed_dev,
                                                        float *scale_dev, void *workspace_dev, size_t workspace_bytes,
                                                        bitnet_stream_t stream)
{
    if (n_values == 0) return BITNET_OK;
    if (!w_dev || !packed_dev || !scale_dev) return fail(BITNET_ERR_NULL_POINTER, "bitnet_quantize_pack_weights: null buffer");
    size_t need = 0;
    bitnet_quantize_pack_weights_workspace_size(n_values, &need);
    if (!workspace_dev || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace_dev) & 255))
        return fail(BITNET_ERR_WORKSPACE, "bitnet_quantize_pack_weights needs %zu bytes of 256-byte aligned workspace", need);
    cudaStream_t s = as_stream(stream);
    double *partial = static_cast<double *>(workspace_dev);
    float *threshold = reinterpret_cast<float *>(static_cast<char *>(workspace_dev) + align_up(2 * WQ_MAX_BLOCKS * sizeof(double), 256));
    const size_t groups = (n_values + 3) / 4;
    size_t blocks = (groups + WQ_THREADS - 1) / WQ_THREADS;
    if (blocks > WQ_MAX_BLOCKS) blocks = WQ_MAX_BLOCKS;
    wq_abs_partial_kernel<<<(unsigned)blocks, WQ_THREADS, 0, s>>>(w_dev, n_values, partial);
    BITNET_TRY(check_launch("wq_abs_partial_kernel"));
    wq_threshold_kernel<<<1, 32, 0, s>>>(partial, (int)blocks, n_values, threshold);
    BITNET_TRY(check_launch("wq_threshold_kernel"));
    wq_ternarize_pack_kernel<<<(unsigned)blocks, WQ_THREADS, 0, s>>>(w_dev, n_values, threshold, packed_dev, partial);
    BITNET_TRY(check_launch("wq_ternarize_pack_kernel"));
    wq_scale_kernel<<<1, 32, 0, s>>>(partial, (int)blocks, scale_dev);
    return check_launch("wq_scale_kernel");
}
