// Stand-alone pieces of the path: per-token activation quantisation, the gating
// between the FFN projections, and packed-weight helpers.
#include "common.cuh"

namespace bitnet {

// One CTA per token row.  Pass 1 folds |x| to the row's absmax, pass 2 quantises.
// Semantics: TernaryProcessor::quantize_activations
// (bitnet-inference/src/engine/ternary_operations.rs:130-163).
__global__ void __launch_bounds__(256) quantize_rows_kernel(const float *__restrict__ x, size_t K,
                                                            int8_t *__restrict__ q,
                                                            float *__restrict__ a_scale)
{
    __shared__ unsigned s_key[8];
    const size_t m = blockIdx.x;
    const float *row = x + m * K;
    const int tid = threadIdx.x;

    unsigned key = 0;
    const bool vec = (K % 4 == 0) && ((reinterpret_cast<uintptr_t>(row) & 15) == 0);
    if (vec) {
        const float4 *row4 = reinterpret_cast<const float4 *>(row);
        for (size_t i = tid; i < K / 4; i += blockDim.x) {
            const float4 v = __ldg(row4 + i);
            key = max(max(key, abs_key(v.x)), max(abs_key(v.y), max(abs_key(v.z), abs_key(v.w))));
        }
    } else {
        for (size_t i = tid; i < K; i += blockDim.x) key = max(key, abs_key(__ldg(row + i)));
    }
    key = __reduce_max_sync(0xffffffffu, key);
    if ((tid & 31) == 0) s_key[tid >> 5] = key;
    __syncthreads();
    key = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) key = max(key, s_key[w]);

    const float absmax = __uint_as_float(key);
    const float scale = quant_scale(absmax);
    if (tid == 0 && a_scale) a_scale[m] = dequant_scale(absmax);
    if (!q) return;

    int8_t *qrow = q + m * K;
    if (vec && ((reinterpret_cast<uintptr_t>(qrow) & 3) == 0)) {
        const float4 *row4 = reinterpret_cast<const float4 *>(row);
        uint32_t *q4 = reinterpret_cast<uint32_t *>(qrow);
        for (size_t i = tid; i < K / 4; i += blockDim.x) {
            const float4 v = __ldg(row4 + i);
            const uint32_t b0 = (uint32_t)quantize_one(v.x, scale) & 0xffu;
            const uint32_t b1 = (uint32_t)quantize_one(v.y, scale) & 0xffu;
            const uint32_t b2 = (uint32_t)quantize_one(v.z, scale) & 0xffu;
            const uint32_t b3 = (uint32_t)quantize_one(v.w, scale) & 0xffu;
            q4[i] = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
        }
    } else {
        for (size_t i = tid; i < K; i += blockDim.x) qrow[i] = (int8_t)quantize_one(__ldg(row + i), scale);
    }
}

bitnet_status_t launch_quantize_rows(const float *x, size_t M, size_t K, int8_t *q, float *a_scale,
                                     cudaStream_t stream)
{
    if (M == 0) return BITNET_OK;
    if (M > 0x7fffffffull) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "too many rows: %zu", M);
    quantize_rows_kernel<<<(unsigned)M, 256, 0, stream>>>(x, K, q, a_scale);
    return check_launch("quantize_rows_kernel");
}

// h = up * relu(gate)^2 (FeedForwardNetwork::forward, transformer_layers.rs:613-618).
__global__ void gate_relu2_kernel(const float *__restrict__ up, const float *__restrict__ gate,
                                  float *__restrict__ h, size_t n)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float r = fmaxf(gate[i], 0.0f);
        h[i] = __fmul_rn(up[i], __fmul_rn(r, r));
    }
}

bitnet_status_t launch_gate_relu2(const float *up, const float *gate, float *h, size_t n, cudaStream_t stream)
{
    if (n == 0) return BITNET_OK;
    const unsigned blocks = (unsigned)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    gate_relu2_kernel<<<blocks, 256, 0, stream>>>(up, gate, h, n);
    return check_launch("gate_relu2_kernel");
}

// BitPacked2BitPacker::pack (packing.rs:352-388): code = w + 1, element j in bits [2j+1:2j].
__global__ void pack_ternary_kernel(const int8_t *__restrict__ w, size_t n, uint8_t *__restrict__ out)
{
    const size_t nbytes = (n + 3) / 4;
    for (size_t b = blockIdx.x * (size_t)blockDim.x + threadIdx.x; b < nbytes; b += (size_t)gridDim.x * blockDim.x) {
        unsigned byte = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const size_t i = b * 4 + j;
            if (i < n) byte |= ((unsigned)(w[i] + 1) & 3u) << (2 * j);
        }
        out[b] = (uint8_t)byte;
    }
}

// BitPacked2BitPacker::unpack (packing.rs:390-394); code 3 decodes to 0
// (gguf.rs:1139, weight_conversion.rs:179-182).
__global__ void unpack_ternary_kernel(const uint8_t *__restrict__ p, size_t n, int8_t *__restrict__ out)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const unsigned code = (p[i >> 2] >> (2 * (i & 3))) & 3u;
        out[i] = code == 3u ? (int8_t)0 : (int8_t)((int)code - 1);
    }
}

__global__ void sanitize_packed_kernel(uint8_t *__restrict__ p, size_t nbytes, unsigned long long *count)
{
    unsigned long long found = 0;
    for (size_t b = blockIdx.x * (size_t)blockDim.x + threadIdx.x; b < nbytes; b += (size_t)gridDim.x * blockDim.x) {
        const unsigned v = p[b];
        const unsigned both = (v >> 1) & v & 0x55u;   // low bit of every field that holds 3
        if (both) {
            p[b] = (uint8_t)(v ^ (both << 1));        // 3 -> 1
            found += __popc(both);
        }
    }
    found = __reduce_add_sync(0xffffffffu, (unsigned)found);
    if (count && (threadIdx.x & 31) == 0 && found) atomicAdd(count, found);
}

static unsigned grid_for(size_t items)
{
    const size_t blocks = (items + 255) / 256;
    return (unsigned)(blocks < 1 ? 1 : (blocks > 148 * 16 ? 148 * 16 : blocks));
}

}  // namespace bitnet

using namespace bitnet;

extern "C" bitnet_status_t bitnet_pack_ternary(const int8_t *w_dev, size_t n_values, uint8_t *packed_dev,
                                               bitnet_stream_t stream)
{
    if (n_values == 0) return BITNET_OK;
    if (!w_dev || !packed_dev) return fail(BITNET_ERR_NULL_POINTER, "bitnet_pack_ternary: null buffer");
    pack_ternary_kernel<<<grid_for((n_values + 3) / 4), 256, 0, as_stream(stream)>>>(w_dev, n_values, packed_dev);
    return check_launch("pack_ternary_kernel");
}

extern "C" bitnet_status_t bitnet_unpack_ternary(const uint8_t *packed_dev, size_t n_values, int8_t *w_dev,
                                                 bitnet_stream_t stream)
{
    if (n_values == 0) return BITNET_OK;
    if (!w_dev || !packed_dev) return fail(BITNET_ERR_NULL_POINTER, "bitnet_unpack_ternary: null buffer");
    unpack_ternary_kernel<<<grid_for(n_values), 256, 0, as_stream(stream)>>>(packed_dev, n_values, w_dev);
    return check_launch("unpack_ternary_kernel");
}

extern "C" bitnet_status_t bitnet_sanitize_packed(uint8_t *packed_dev, size_t n_bytes,
                                                  unsigned long long *count_dev, bitnet_stream_t stream)
{
    if (n_bytes == 0) return BITNET_OK;
    if (!packed_dev) return fail(BITNET_ERR_NULL_POINTER, "bitnet_sanitize_packed: null buffer");
    sanitize_packed_kernel<<<grid_for(n_bytes), 256, 0, as_stream(stream)>>>(packed_dev, n_bytes, count_dev);
    return check_launch("sanitize_packed_kernel");
}

extern "C" bitnet_status_t bitnet_quantize_activations(const float *x_dev, size_t M, size_t K, int8_t *q_dev,
                                                       float *a_scale_dev, bitnet_stream_t stream)
{
    if (M == 0) return BITNET_OK;
    if (K == 0) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "bitnet_quantize_activations: K == 0");
    if (!x_dev) return fail(BITNET_ERR_NULL_POINTER, "bitnet_quantize_activations: x is null");
    if (!q_dev && !a_scale_dev) return fail(BITNET_ERR_NULL_POINTER, "bitnet_quantize_activations: no output");
    return launch_quantize_rows(x_dev, M, K, q_dev, a_scale_dev, as_stream(stream));
}
