// Shape-agnostic BitLinear contraction: any M, K, N, including K % 4 != 0 where a row
// of the flat packed stream starts in the middle of a byte.  One warp per output
// feature, tokens in groups of 8.  Exact, not fast: the decode and prefill kernels
// cover the shapes that matter; this one covers everything else.
#include "common.cuh"

namespace bitnet {

constexpr int GEN_TOKENS = 8;

__global__ void __launch_bounds__(256) generic_contract_kernel(
    const uint8_t *__restrict__ wp, float w_scale, const int8_t *__restrict__ q,
    const float *__restrict__ a_scale, float *__restrict__ y, int32_t *__restrict__ acc_out,
    size_t M, size_t K, size_t N, size_t ldy)
{
    const int lane = threadIdx.x & 31;
    const size_t warp = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5;
    const size_t n_warps = ((size_t)gridDim.x * blockDim.x) >> 5;
    for (size_t n = warp; n < N; n += n_warps) {
        const size_t base = n * K;   // flat element index of W[n,0]
        for (size_t m0 = 0; m0 < M; m0 += GEN_TOKENS) {
            int acc[GEN_TOKENS];
#pragma unroll
            for (int t = 0; t < GEN_TOKENS; ++t) acc[t] = 0;
            for (size_t k = lane; k < K; k += 32) {
                const size_t e = base + k;
                const unsigned code = (wp[e >> 2] >> (2 * (e & 3))) & 3u;
                const int w = code == 3u ? 0 : (int)code - 1;
#pragma unroll
                for (int t = 0; t < GEN_TOKENS; ++t)
                    if (m0 + t < M) acc[t] += w * (int)q[(m0 + t) * K + k];
            }
#pragma unroll
            for (int t = 0; t < GEN_TOKENS; ++t) {
                const int s = __reduce_add_sync(0xffffffffu, acc[t]);
                if (lane == 0 && m0 + t < M) {
                    const size_t o = (m0 + t) * ldy + n;
                    if (acc_out) acc_out[o] = s;
                    if (y) y[o] = __fmul_rn((float)s, __fmul_rn(w_scale, a_scale[m0 + t]));
                }
            }
        }
    }
}

bitnet_status_t launch_generic(const uint8_t *wp, float w_scale, const int8_t *q, const float *a_scale,
                               float *y, int32_t *acc_out, size_t M, size_t K, size_t N, size_t ldy,
                               cudaStream_t stream)
{
    if (M == 0 || N == 0) return BITNET_OK;
    size_t blocks = (N + 7) / 8;
    const size_t cap = (size_t)device_sm_count() * 8;
    if (blocks > cap) blocks = cap;
    generic_contract_kernel<<<(unsigned)blocks, 256, 0, stream>>>(wp, w_scale, q, a_scale, y, acc_out, M, K, N, ldy);
    return check_launch("generic_contract_kernel");
}

}  // namespace bitnet
