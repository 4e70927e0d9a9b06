// Device primitives shared by the decode kernels (single launch and grouped launch): mbarrier and bulk-copy
// wrappers with bounded waits, the u8 x s8 tensor-core step on masked packed words, the exact fp32 quantiser and
// the row quantiser that writes the activation image those kernels fetch.
#pragma once

#include "common.cuh"

namespace bitnet {

constexpr int DEC_MAX_CWARPS = 16;                     // consumer warps: 8 (two CTAs per SM) or 16
constexpr int DEC_MAX_STAGES = 8;
constexpr int DEC_MAX_TOKENS = 16;
constexpr unsigned DEC_WAIT_LIMIT = 1u << 22;          // polls before a wait gives up
// A quantised-activation image starts with this header: int32 sums [16 warps][16 tokens], then
// fp32 absmax/127 [16 tokens], padded; the fragment-ordered int8 data follows.
constexpr unsigned DEC_IMG_HDR = 1152;

// Set when a bounded wait ran out (bit 0).  One copy per translation unit; each one's host side reads and clears
// its own (bitnet_device_error_flags collects them).
static __device__ unsigned g_decode_error_flags;

// ---- mbarrier / bulk-copy primitives ---------------------------------------------------------

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long *bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned long long *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long *bar, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait: false when the phase did not complete within DEC_WAIT_LIMIT polls.
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, unsigned parity)
{
    const unsigned addr = smem_u32(bar);
    for (unsigned n = 0; n < DEC_WAIT_LIMIT; ++n) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        __nanosleep(n < 16 ? 32 : 128);   // a waiting warp must not take issue slots from the working ones
    }
    atomicOr(&g_decode_error_flags, 1u);
    return false;
}
__device__ __forceinline__ void bulk_copy_g2s(void *dst_smem, const void *src, unsigned bytes, unsigned long long *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void mma_u8s8(int (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The same step starting an accumulator: D = A x B with a zero C that costs no register moves.
__device__ __forceinline__ void mma_u8s8_first(int (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                               unsigned b0, unsigned b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

__device__ __forceinline__ unsigned word_of(const uint4 &v, int i)
{
    return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}

// Exact round-half-away quantisation of t = x*scale for |t| <= 2^22: trunc(|t| + c) with
// c the largest float below 0.5 equals roundf(|t|) for every float (checked exhaustively),
// and adding 2^23 with round-toward-zero leaves that integer in the low mantissa bits.
__device__ __forceinline__ int quantize_fast(float x, float scale)
{
    const float t = __fmul_rn(x, scale);
    const float a = fminf(__fadd_rn(fabsf(t), 0.49999997f), 127.0f);   // |t| < 127.5 whenever x is finite
    const int mag = __float_as_int(__fadd_rz(a, 8388608.0f)) & 0xff;
    const int neg = __float_as_int(t) >> 31;          // 0 or -1
    const int q = (mag ^ neg) - neg;
    return (t == t) ? q : 0;                            // NaN quantises to 0, like the oracle
}

// The rare slow path (absmax so large or small that 127/absmax leaves the normal range) stays
// out of line: these kernels run their prologue once per CTA, so its code size is paid in
// instruction fetches.
static __device__ __noinline__ int quantize_one_slow(float x, float scale) { return quantize_one(x, scale); }

__device__ __forceinline__ int quantize_any(float x, float scale, bool fast)
{
    return fast ? quantize_fast(x, scale) : quantize_one_slow(x, scale);
}

// Quantises row m of x[.,K] for the decode kernels: one CTA of 512 threads per token, one read of the row (it
// stays in registers between the absmax fold and the rounding), and the int8 values land in global memory as
// the exact shared-memory image the consuming kernel's warps want (header: per-warp-slice sums and absmax/127;
// then fragment-ordered bytes), so that kernel fetches it with a single bulk copy.  cw/sw/nt/mrows describe the
// consuming instantiation.  Semantics: TernaryProcessor::quantize_activations (ternary_operations.rs:130-163).
// pre: the decoder-layer glue in front of the quantiser (residual add, SubLN), applied to the row while it
// sits in registers; sums run in a fixed order (lane tree, then the sixteen warps in turn).
__device__ __forceinline__ void quantize_row_to_image(const float *x, int m, int K, int cw, int sw, int nt, int mrows,
                                                      unsigned char *__restrict__ image,
                                                      const unsigned *__restrict__ amax_in, int n_amax_in,
                                                      int8_t *__restrict__ q_out, float *__restrict__ a_scale_out,
                                                      const RowPre &pre, const RowsOut &rows)
{
    __shared__ unsigned s_wkey[16];
    __shared__ int s_sum[DEC_MAX_CWARPS];
    __shared__ float s_fsum[2][16];
    const int tid = threadIdx.x;
    const int n_groups = K / 16;
    const float *row = x + (size_t)m * K;
    if (tid < DEC_MAX_CWARPS) s_sum[tid] = 0;

    float4 f[2][4];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int G = tid + u * 512;
        if (G < n_groups) {
            const float4 *src = reinterpret_cast<const float4 *>(row + (size_t)G * 16);
#pragma unroll
            for (int v = 0; v < 4; ++v) f[u][v] = src[v];   // plain loads: sum_out may alias x
        }
    }
    apply_row_pre(f, pre, m, K, tid, s_fsum);
    unsigned key = 0;
    if (amax_in) {
        for (int i = tid; i < n_amax_in; i += 512) key = max(key, __ldg(amax_in + (size_t)m * 256 + i));
    } else {
#pragma unroll
        for (int u = 0; u < 2; ++u)
            if (tid + u * 512 < n_groups) {
#pragma unroll
                for (int v = 0; v < 4; ++v)
                    key = max(max(key, abs_key(f[u][v].x)), max(abs_key(f[u][v].y), max(abs_key(f[u][v].z), abs_key(f[u][v].w))));
            }
    }
    key = __reduce_max_sync(0xffffffffu, key);
    if ((tid & 31) == 0) s_wkey[tid >> 5] = key;
    __syncthreads();
    key = 0;
#pragma unroll
    for (int w = 0; w < 16; ++w) key = max(key, s_wkey[w]);
    const float absmax = __uint_as_float(key);
    const float scale = quant_scale(absmax);
    const bool fast = scale >= 1e-30f && scale <= 1e30f;
    const int C = K / 64;
    int row_total = 0;
    const unsigned frag_blk = (unsigned)mrows * 64u;
    const unsigned region = (unsigned)sw * 4 * nt * frag_blk;

#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int G = tid + u * 512;
        if (G < n_groups) {
            int q[16];
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                q[4 * v + 0] = fast ? quantize_fast(f[u][v].x, scale) : quantize_one(f[u][v].x, scale);
                q[4 * v + 1] = fast ? quantize_fast(f[u][v].y, scale) : quantize_one(f[u][v].y, scale);
                q[4 * v + 2] = fast ? quantize_fast(f[u][v].z, scale) : quantize_one(f[u][v].z, scale);
                q[4 * v + 3] = fast ? quantize_fast(f[u][v].w, scale) : quantize_one(f[u][v].w, scale);
            }
            if (q_out) {
                uint4 canon;
                canon.x = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((unsigned)(q[3] & 0xff) << 24);
                canon.y = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((unsigned)(q[7] & 0xff) << 24);
                canon.z = (q[8] & 0xff) | ((q[9] & 0xff) << 8) | ((q[10] & 0xff) << 16) | ((unsigned)(q[11] & 0xff) << 24);
                canon.w = (q[12] & 0xff) | ((q[13] & 0xff) << 8) | ((q[14] & 0xff) << 16) | ((unsigned)(q[15] & 0xff) << 24);
                *reinterpret_cast<uint4 *>(q_out + (size_t)m * K + (size_t)G * 16) = canon;
            }
            uint4 frag;
            frag.x = (q[0] & 0xff) | ((q[4] & 0xff) << 8) | ((q[8] & 0xff) << 16) | ((unsigned)(q[12] & 0xff) << 24);
            frag.y = (q[1] & 0xff) | ((q[5] & 0xff) << 8) | ((q[9] & 0xff) << 16) | ((unsigned)(q[13] & 0xff) << 24);
            frag.z = (q[2] & 0xff) | ((q[6] & 0xff) << 8) | ((q[10] & 0xff) << 16) | ((unsigned)(q[14] & 0xff) << 24);
            frag.w = (q[3] & 0xff) | ((q[7] & 0xff) << 8) | ((q[11] & 0xff) << 16) | ((unsigned)(q[15] & 0xff) << 24);
            int sum = 0;
#pragma unroll
            for (int e = 0; e < 16; ++e) sum += q[e];
            if (rows.q_perm) {   // row-major form for the tensor-core kernels: groups stay in row order
                *reinterpret_cast<uint4 *>(rows.q_perm + (size_t)m * K + (size_t)G * 16) = frag;
                row_total += sum;
                continue;
            }
            // which consumer warp owns this chunk, and where in its region the group goes
            const int chunk = G >> 2, i = G & 3;
            const int w = (int)((((long long)chunk + 1) * cw - 1) / C);
            const int c_rel = chunk - (int)((long long)w * C / cw);
            const unsigned step = (unsigned)c_rel >> 2, ctig = (unsigned)c_rel & 3;
            const unsigned off = DEC_IMG_HDR + (unsigned)w * region + ((step * 4 + i) * nt + (m >> 3)) * frag_blk + ((m & 7) * 4 + ctig) * 16;
            *reinterpret_cast<uint4 *>(image + off) = frag;
            if (sum) atomicAdd(&s_sum[w], sum);
        }
    }
    if (rows.q_perm) {
        row_total = __reduce_add_sync(0xffffffffu, row_total);
        if ((tid & 31) == 0 && row_total) atomicAdd(&s_sum[0], row_total);
    }
    __syncthreads();
    if (rows.q_perm) {
        if (tid == 0) {
            rows.rowsum[m] = s_sum[0];
            rows.a_scale[m] = dequant_scale(absmax);
            if (a_scale_out) a_scale_out[m] = dequant_scale(absmax);
        }
        return;
    }
    if (tid < cw) reinterpret_cast<int *>(image)[tid * DEC_MAX_TOKENS + m] = s_sum[tid];
    if (tid == 0) {
        reinterpret_cast<float *>(image + DEC_MAX_CWARPS * DEC_MAX_TOKENS * 4)[m] = dequant_scale(absmax);
        if (a_scale_out) a_scale_out[m] = dequant_scale(absmax);
    }
}

}  // namespace bitnet
