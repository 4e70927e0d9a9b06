// Prefill-time BitLinear (many tokens): int8 x ternary GEMM on the 5th-generation tensor cores.
//
//   1. quantize_rows_perm_kernel: per-token absmax int8 quantisation of x[M,K] into scratch,
//      with the 16 values of every 16-wide k group stored transposed (byte 4j+i holds k = 4i+j),
//      plus the row sums sum_k q[m,k].
//   2. prefill_gemm_kernel: persistent CTAs, one 128-token x 256-feature tile at a time.
//        warp 0      TMA producer: the int8 activation tile (128 x 128 bytes, 128-byte swizzle) and
//                    the PACKED weight tile (256 rows x 32 bytes) per 128-wide k slice
//        warps 2-9   expand packed weights to int8 codes {0,1,2} in shared memory, straight into
//                    the swizzled K-major layout the tensor core reads: (w >> 2j) & 0x03030303
//                    yields the four bytes k = j, j+4, j+8, j+12 of a group, i.e. word j of the
//                    transposed group order the activations were stored in
//                    (two groups of four warps take the k slices in turn)
//        warp 1      issues tcgen05.mma kind::i8 (M=128, N=256, K=32; s8 x u8 -> s32) with the
//                    accumulator in tensor memory; two accumulators alternate between tiles
//        warps 10-13 epilogue: tcgen05.ld the accumulator, subtract the row sum
//                    (sum_k (code-1) q = sum_k code q - sum_k q), scale, store y
//      Every barrier wait is bounded; a wait that runs out raises an error flag and the CTA
//      drains and frees its tensor memory.
//
// Semantics: TernaryProcessor::quantize_activations + ternary_matmul_generic
// (bitnet-inference/src/engine/ternary_operations.rs:117-172, :283-338) with int32 accumulation
// on the packed layout of BitPacked2BitPacker (bitnet-quant/src/quantization/packing.rs:352-394).
// The reference has no tensor-core kernel; this is what its BitLinearLayer::forward
// (transformer_layers.rs:119-202) computes for a [B*S, K] input.
#include <cuda.h>

#include "common.cuh"

namespace bitnet {

// Set (bit 1) when a bounded wait of the GEMM kernel ran out -- read with bitnet_device_error_flags().
__device__ unsigned g_prefill_error_flags;

constexpr int PF_BM = 128, PF_BN = 256, PF_BK = 128;   // tile: tokens x features x k (bytes of int8)
constexpr int PF_STAGES = 4;                       // TMA ring: activations + packed weights (latency hiding)
constexpr int PF_BSTAGES = 3;                      // ring of expanded weight tiles
constexpr int PF_A_BYTES = PF_BM * PF_BK;          // 16 KB
constexpr int PF_WP_BYTES = PF_BN * PF_BK / 4;     // 8 KB packed
constexpr int PF_B_BYTES = PF_BN * PF_BK;          // 32 KB expanded
constexpr int PF_STAGE_BYTES = PF_A_BYTES + PF_WP_BYTES;
constexpr int PF_EXP_WARPS = 8;                    // warps that expand packed weights
constexpr int PF_GROUPS = 2;                       // expander groups working on alternate k slices
constexpr int PF_THREADS = (2 + PF_EXP_WARPS + 4) * 32;   // producer, MMA, expanders, epilogue
constexpr unsigned PF_WAIT_LIMIT = 1u << 22;
constexpr int PF_EPI_BYTES = 4 * 32 * 32 * 4;       // per epilogue warp a 32x32 fp32 transpose buffer
constexpr size_t PF_SMEM = (size_t)PF_STAGES * PF_STAGE_BYTES + (size_t)PF_BSTAGES * PF_B_BYTES + PF_EPI_BYTES + 1024;   // + alignment slack

// ---- quantiser for the GEMM path ----------------------------------------------------------------

// Same exact rounding as common.cuh's quantize_one for |x*scale| <= 2^22 (trunc(|t| + c) with c the
// largest float below 0.5 equals roundf(|t|) for every float; adding 2^23 toward zero leaves the
// integer in the low mantissa bits); NaN quantises to 0.
__device__ __forceinline__ int pf_quantize_fast(float x, float scale)
{
    const float t = __fmul_rn(x, scale);
    const float a = fminf(__fadd_rn(fabsf(t), 0.49999997f), 127.0f);
    const int mag = __float_as_int(__fadd_rz(a, 8388608.0f)) & 0xff;
    const int neg = __float_as_int(t) >> 31;
    return (t == t) ? (mag ^ neg) - neg : 0;
}

// One CTA per token row, one read of the row when it fits the registers (K <= 8192).
// q_perm[m, 16G + 4j + i] = q[m, 16G + 4i + j]; rowsum[m] = sum_k q[m,k].
// Semantics: TernaryProcessor::quantize_activations (ternary_operations.rs:130-163).
__global__ void __launch_bounds__(256) quantize_rows_perm_kernel(const float *__restrict__ x, size_t K,
                                                                 int8_t *__restrict__ q_perm, float *__restrict__ a_scale,
                                                                 int *__restrict__ rowsum, int8_t *__restrict__ q_out,
                                                                 float *__restrict__ a_scale_out)
{
    __shared__ unsigned s_key[8];
    __shared__ int s_sum[8];
    const size_t m = blockIdx.x;
    const float *row = x + m * K;
    const int tid = threadIdx.x;
    const size_t n_groups = K / 16;
    const bool resident = n_groups <= 512;   // two 16-wide groups per thread stay in registers

    float4 f[2][4];
    unsigned key = 0;
    if (resident) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const size_t G = tid + u * 256;
            if (G < n_groups) {
                const float4 *src = reinterpret_cast<const float4 *>(row + G * 16);
#pragma unroll
                for (int v = 0; v < 4; ++v) f[u][v] = __ldg(src + v);
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u)
            if ((size_t)(tid + u * 256) < n_groups) {
#pragma unroll
                for (int v = 0; v < 4; ++v)
                    key = max(max(key, abs_key(f[u][v].x)), max(abs_key(f[u][v].y), max(abs_key(f[u][v].z), abs_key(f[u][v].w))));
            }
    } else {
        for (size_t G = tid; G < n_groups; G += 256) {
            const float4 *src = reinterpret_cast<const float4 *>(row + G * 16);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const float4 g4 = __ldg(src + v);
                key = max(max(key, abs_key(g4.x)), max(abs_key(g4.y), max(abs_key(g4.z), abs_key(g4.w))));
            }
        }
    }
    key = __reduce_max_sync(0xffffffffu, key);
    if ((tid & 31) == 0) s_key[tid >> 5] = key;
    __syncthreads();
    key = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) key = max(key, s_key[w]);
    const float absmax = __uint_as_float(key);
    const float scale = quant_scale(absmax);
    // a huge or tiny absmax makes the scale leave the normal range; the fast rounding assumes it has not
    const bool fast = scale >= 1e-30f && scale <= 1e30f;

    int sum = 0;
    const size_t rounds = resident ? 2 : (n_groups + 255) / 256;
    for (size_t u = 0; u < rounds; ++u) {
        const size_t G = tid + u * 256;
        if (G >= n_groups) break;
        float4 g4[4];
        if (resident) {
#pragma unroll
            for (int v = 0; v < 4; ++v) g4[v] = u == 0 ? f[0][v] : f[1][v];
        } else {
            const float4 *src = reinterpret_cast<const float4 *>(row + G * 16);
#pragma unroll
            for (int v = 0; v < 4; ++v) g4[v] = __ldg(src + v);
        }
        int q[16];
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            if (fast) {
                q[4 * v + 0] = pf_quantize_fast(g4[v].x, scale);
                q[4 * v + 1] = pf_quantize_fast(g4[v].y, scale);
                q[4 * v + 2] = pf_quantize_fast(g4[v].z, scale);
                q[4 * v + 3] = pf_quantize_fast(g4[v].w, scale);
            } else {
                q[4 * v + 0] = quantize_one(g4[v].x, scale);
                q[4 * v + 1] = quantize_one(g4[v].y, scale);
                q[4 * v + 2] = quantize_one(g4[v].z, scale);
                q[4 * v + 3] = quantize_one(g4[v].w, scale);
            }
        }
#pragma unroll
        for (int e = 0; e < 16; ++e) sum += q[e];
        uint4 perm;
        perm.x = (q[0] & 0xff) | ((q[4] & 0xff) << 8) | ((q[8] & 0xff) << 16) | ((unsigned)(q[12] & 0xff) << 24);
        perm.y = (q[1] & 0xff) | ((q[5] & 0xff) << 8) | ((q[9] & 0xff) << 16) | ((unsigned)(q[13] & 0xff) << 24);
        perm.z = (q[2] & 0xff) | ((q[6] & 0xff) << 8) | ((q[10] & 0xff) << 16) | ((unsigned)(q[14] & 0xff) << 24);
        perm.w = (q[3] & 0xff) | ((q[7] & 0xff) << 8) | ((q[11] & 0xff) << 16) | ((unsigned)(q[15] & 0xff) << 24);
        *reinterpret_cast<uint4 *>(q_perm + m * K + G * 16) = perm;
        if (q_out) {
            uint4 canon;
            canon.x = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((unsigned)(q[3] & 0xff) << 24);
            canon.y = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((unsigned)(q[7] & 0xff) << 24);
            canon.z = (q[8] & 0xff) | ((q[9] & 0xff) << 8) | ((q[10] & 0xff) << 16) | ((unsigned)(q[11] & 0xff) << 24);
            canon.w = (q[12] & 0xff) | ((q[13] & 0xff) << 8) | ((q[14] & 0xff) << 16) | ((unsigned)(q[15] & 0xff) << 24);
            *reinterpret_cast<uint4 *>(q_out + m * K + G * 16) = canon;
        }
    }
    sum = __reduce_add_sync(0xffffffffu, sum);
    if ((tid & 31) == 0) s_sum[tid >> 5] = sum;
    __syncthreads();
    if (tid == 0) {
        int total = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) total += s_sum[w];
        rowsum[m] = total;
        a_scale[m] = dequant_scale(absmax);
        if (a_scale_out) a_scale_out[m] = dequant_scale(absmax);
    }
}

#ifdef BITNET_PHASE_TIMERS
__device__ unsigned long long g_pf_ts[8][128];   // [role/point][iteration] of CTA 0
#define PF_TS(point, it)                                                         \
    do {                                                                         \
        if (blockIdx.x == 0 && (it) < 128) {                                     \
            unsigned long long t_;                                               \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));               \
            g_pf_ts[point][it] = t_;                                             \
        }                                                                        \
    } while (0)
extern "C" int bitnet_debug_read_pf(unsigned long long *host) { return (int)cudaMemcpyFromSymbol(host, g_pf_ts, sizeof(g_pf_ts)); }
#else
#define PF_TS(point, it) do { } while (0)
#endif

// ---- PTX wrappers -------------------------------------------------------------------------------

__device__ __forceinline__ unsigned pf_smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void pf_mbar_init(unsigned long long *bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pf_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void pf_mbar_arrive(unsigned long long *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(pf_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void pf_mbar_expect_tx(unsigned long long *bar, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(pf_smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait; false (and the error flag) when the phase did not complete in time.
__device__ __forceinline__ bool pf_mbar_wait(unsigned long long *bar, unsigned parity)
{
    const unsigned addr = pf_smem_u32(bar);
    for (unsigned n = 0; n < PF_WAIT_LIMIT; ++n) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
#ifndef BITNET_NO_BACKOFF
        __nanosleep(n < 16 ? 32 : 128);   // a waiting warp must not take issue slots from the working ones
#endif
    }
    atomicOr(&g_prefill_error_flags, 2u);
    return false;
}
// One lane polls for the whole warp (keeps barrier polling off the shared-memory pipe).
__device__ __forceinline__ bool pf_warp_wait(unsigned long long *bar, unsigned parity)
{
    unsigned ok = 1;
    if ((threadIdx.x & 31) == 0) ok = pf_mbar_wait(bar, parity) ? 1u : 0u;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    return ok != 0;
}
__device__ __forceinline__ void pf_tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, unsigned long long *bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            pf_smem_u32(dst)),
        "l"(map), "r"(pf_smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
// K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ unsigned long long pf_smem_desc(unsigned smem_addr)
{
    return (unsigned long long)((smem_addr >> 4) & 0x3fffu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void pf_mma_i8(unsigned tmem_d, unsigned long long a_desc, unsigned long long b_desc,
                                          unsigned idesc, unsigned accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void pf_commit(unsigned long long *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(pf_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void pf_tmem_ld32(unsigned taddr, unsigned (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

struct PrefillParams {
    float *y;
    int32_t *acc_out;
    const float *a_scale;
    const int *rowsum;
    float w_scale;
    int M, K, N;
    size_t ldy;
    int m_tiles, n_tiles, k_tiles;
};

// instruction descriptor: D = s32, A = s8 (activations), B = u8 (codes), both K-major, N = 256, M = 128
constexpr unsigned PF_IDESC = (2u << 4) | (1u << 7) | (0u << 10) | ((unsigned)(PF_BN >> 3) << 17) | ((unsigned)(PF_BM >> 4) << 24);

__global__ void __launch_bounds__(PF_THREADS, 1)
prefill_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const PrefillParams p)
{
    extern __shared__ unsigned char pf_smem_raw[];
    __shared__ __align__(8) unsigned long long s_full_tma[PF_STAGES], s_empty[PF_STAGES];
    __shared__ __align__(8) unsigned long long s_full_b[PF_BSTAGES], s_empty_b[PF_BSTAGES];
    __shared__ __align__(8) unsigned long long s_acc_full[2], s_acc_empty[2];
    __shared__ unsigned s_tmem_base;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(pf_smem_raw) + 1023) & ~uintptr_t(1023));
    // expanded weight tiles first (1024-byte aligned for the swizzle), then the TMA ring
    auto stage_b = [&](int sb) { return smem + (size_t)sb * PF_B_BYTES; };
    auto stage_a = [&](int s) { return smem + (size_t)PF_BSTAGES * PF_B_BYTES + (size_t)s * PF_STAGE_BYTES; };
    auto stage_wp = [&](int s) { return smem + (size_t)PF_BSTAGES * PF_B_BYTES + (size_t)s * PF_STAGE_BYTES + PF_A_BYTES; };

    if (tid == 0) {
        for (int s = 0; s < PF_STAGES; ++s) {
            pf_mbar_init(&s_full_tma[s], 1);
            pf_mbar_init(&s_empty[s], 1);
        }
        for (int sb = 0; sb < PF_BSTAGES; ++sb) {
            pf_mbar_init(&s_full_b[sb], PF_EXP_WARPS / PF_GROUPS);
            pf_mbar_init(&s_empty_b[sb], 1);
        }
        for (int b = 0; b < 2; ++b) {
            pf_mbar_init(&s_acc_full[b], 1);
            pf_mbar_init(&s_acc_empty[b], 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // one warp allocates all 512 tensor-memory columns: two 128x256 s32 accumulators
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(pf_smem_u32(&s_tmem_base)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = s_tmem_base;

    const int n_tiles_total = p.m_tiles * p.n_tiles;

    if (warp == 0) {
        // ===================== TMA producer =====================
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles_total && ok; t += gridDim.x) {
                const int n_tile = t / p.m_tiles, m_tile = t % p.m_tiles;
                for (int kt = 0; kt < p.k_tiles; ++kt, ++it) {
                    const int s = it % PF_STAGES;
                    const unsigned ph = (unsigned)(it / PF_STAGES) & 1u;
                    PF_TS(0, it);
                    if (!pf_mbar_wait(&s_empty[s], ph ^ 1u)) { ok = false; break; }
                    PF_TS(1, it);
                    pf_mbar_expect_tx(&s_full_tma[s], PF_A_BYTES + PF_WP_BYTES);
                    pf_tma_load_2d(stage_a(s), &map_a, kt * PF_BK, m_tile * PF_BM, &s_full_tma[s]);
                    pf_tma_load_2d(stage_wp(s), &map_w, kt * (PF_BK / 4), n_tile * PF_BN, &s_full_tma[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ===================== MMA issuer =====================
        if (lane == 0) {
            int it = 0, tc = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles_total && ok; t += gridDim.x, ++tc) {
                const int buf = tc & 1;
                const unsigned acc_ph = (unsigned)(tc >> 1) & 1u;
                if (!pf_mbar_wait(&s_acc_empty[buf], acc_ph ^ 1u)) { ok = false; break; }   // epilogue drained this accumulator
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned tmem_d = tmem_base + (unsigned)buf * PF_BN;
                for (int kt = 0; kt < p.k_tiles; ++kt, ++it) {
                    const int s = it % PF_STAGES;
                    const unsigned ph = (unsigned)(it / PF_STAGES) & 1u;
                    const int sb = it % PF_BSTAGES;
                    const unsigned phb = (unsigned)(it / PF_BSTAGES) & 1u;
                    if (!pf_mbar_wait(&s_full_b[sb], phb)) { ok = false; break; }   // implies the TMA data of the slice landed
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned long long a_desc = pf_smem_desc(pf_smem_u32(stage_a(s)));
                    const unsigned long long b_desc = pf_smem_desc(pf_smem_u32(stage_b(sb)));
#pragma unroll
                    for (int ks = 0; ks < PF_BK / 32; ++ks)   // 32 bytes of k per instruction: +2 in 16-byte units
                        pf_mma_i8(tmem_d, a_desc + 2ull * ks, b_desc + 2ull * ks, PF_IDESC, (kt | ks) != 0 ? 1u : 0u);
                    pf_commit(&s_empty[s]);     // both rings' slots are free once these MMAs have read them
                    pf_commit(&s_empty_b[sb]);
                    (void)ph;
                }
                if (ok) pf_commit(&s_acc_full[buf]);
            }
        }
    } else if (warp < 2 + PF_EXP_WARPS) {
        // ===================== weight expanders: PF_GROUPS groups take the k slices in turn =====================
        // One group's wait -> expand -> publish chain is longer than the MMAs of a slice; two chains
        // side by side keep the tensor core fed.
        constexpr int GROUP_THREADS = PF_EXP_WARPS * 32 / PF_GROUPS;
        const int group = (warp - 2) / (PF_EXP_WARPS / PF_GROUPS);
        const int e = (tid - 64) - group * GROUP_THREADS;
        int it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles_total && ok; t += gridDim.x) {
            for (int kt = 0; kt < p.k_tiles && ok; ++kt, ++it) {
                if (it % PF_GROUPS != group) continue;
                const int s = it % PF_STAGES;
                const unsigned ph = (unsigned)(it / PF_STAGES) & 1u;
                const int sb = it % PF_BSTAGES;
                const unsigned phb = (unsigned)(it / PF_BSTAGES) & 1u;
                if (!pf_warp_wait(&s_full_tma[s], ph) || !pf_warp_wait(&s_empty_b[sb], phb ^ 1u)) { ok = false; break; }
                // word idx = e + r*GROUP_THREADS covers row n = idx/8, 16-wide group g = idx%8; both g and
                // n%8 are fixed per thread, so source and (swizzled) destination just step by constants
                const unsigned *wp = reinterpret_cast<const unsigned *>(stage_wp(s)) + e;
                unsigned char *bx = stage_b(sb) + (e >> 3) * 128 + (((e & 7) ^ ((e >> 3) & 7)) << 4);
                {
#pragma unroll
                    for (int r = 0; r < (PF_BN * PF_BK / 16) / GROUP_THREADS; ++r) {   // 2048 words of 16 weights
                        const unsigned w = wp[r * GROUP_THREADS];
                        uint4 v;
                        v.x = w & 0x03030303u;
                        v.y = (w >> 2) & 0x03030303u;
                        v.z = (w >> 4) & 0x03030303u;
                        v.w = (w >> 6) & 0x03030303u;
                        *reinterpret_cast<uint4 *>(bx + r * (GROUP_THREADS / 8) * 128) = v;
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the tensor core
                __syncwarp();
                if (lane == 0) pf_mbar_arrive(&s_full_b[sb]);
            }
        }
    } else {
        // ===================== epilogue (128 threads, one accumulator row each) =====================
        const int quarter = warp & 3;   // the tensor-memory lanes a warp may touch: 32 * (warp % 4)
        int tc = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles_total && ok; t += gridDim.x, ++tc) {
            const int n_tile = t / p.m_tiles, m_tile = t % p.m_tiles;
            const int buf = tc & 1;
            const unsigned acc_ph = (unsigned)(tc >> 1) & 1u;
            if (!pf_warp_wait(&s_acc_full[buf], acc_ph)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int m = m_tile * PF_BM + quarter * 32 + lane;
            const bool row_ok = m < p.M;
            const int rs = row_ok ? p.rowsum[m] : 0;
            const float scale = row_ok ? __fmul_rn(p.w_scale, p.a_scale[m]) : 0.0f;
            const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)buf * PF_BN;
            // each lane holds one token row of the accumulator; rows are far apart in y, so a 32x32
            // block goes through shared memory (XOR-swizzled 16-byte chunks, conflict-free both ways)
            // and leaves as full 128-byte row segments
            unsigned char *epi = smem + (size_t)PF_BSTAGES * PF_B_BYTES + (size_t)PF_STAGES * PF_STAGE_BYTES + (size_t)(warp & 3) * 4096;
            const int m_base = m_tile * PF_BM + quarter * 32;
#pragma unroll 1
            for (int c = 0; c < PF_BN / 32; ++c) {
                unsigned r[32];
                pf_tmem_ld32(taddr + (unsigned)c * 32, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const int n0 = n_tile * PF_BN + c * 32;
                if (n0 >= p.N) continue;   // warp-uniform
                if (p.acc_out && row_ok) {
                    int32_t *arow = p.acc_out + (size_t)m * p.ldy + n0;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (n0 + j < p.N) arow[j] = (int)r[j] - rs;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float4 o;
                    o.x = __fmul_rn((float)((int)r[4 * j + 0] - rs), scale);
                    o.y = __fmul_rn((float)((int)r[4 * j + 1] - rs), scale);
                    o.z = __fmul_rn((float)((int)r[4 * j + 2] - rs), scale);
                    o.w = __fmul_rn((float)((int)r[4 * j + 3] - rs), scale);
                    *reinterpret_cast<float4 *>(epi + lane * 128 + ((j ^ (lane & 7)) << 4)) = o;
                }
                __syncwarp();
                const bool vec_ok = n0 + 32 <= p.N && (p.ldy % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.y) & 15) == 0);
#pragma unroll
                for (int it2 = 0; it2 < 8; ++it2) {
                    const int rr = it2 * 4 + (lane >> 3), ch = lane & 7;
                    const float4 o = *reinterpret_cast<const float4 *>(epi + rr * 128 + ((ch ^ (rr & 7)) << 4));
                    const int mm = m_base + rr;
                    if (mm < p.M) {
                        float *dst = p.y + (size_t)mm * p.ldy + n0 + ch * 4;
                        if (vec_ok) {
                            *reinterpret_cast<float4 *>(dst) = o;
                        } else {
                            if (n0 + ch * 4 + 0 < p.N) dst[0] = o.x;
                            if (n0 + ch * 4 + 1 < p.N) dst[1] = o.y;
                            if (n0 + ch * 4 + 2 < p.N) dst[2] = o.z;
                            if (n0 + ch * 4 + 3 < p.N) dst[3] = o.w;
                        }
                    }
                }
                __syncwarp();
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) pf_mbar_arrive(&s_acc_empty[buf]);
        }
    }

    // everyone meets here, also after a wait that gave up, so that tensor memory is always freed
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}

bitnet_status_t prefill_take_error_flags(unsigned *flags)
{
    unsigned v = 0, zero = 0;
    BITNET_CUDA(cudaMemcpyFromSymbol(&v, g_prefill_error_flags, sizeof(v)));
    if (v) BITNET_CUDA(cudaMemcpyToSymbol(g_prefill_error_flags, &zero, sizeof(zero)));
    *flags = v;
    return BITNET_OK;
}

// ---- host side --------------------------------------------------------------------------------------

bool prefill_supports(size_t M, size_t K, size_t N)
{
    return M >= 1 && N >= 1 && K >= 128 && K % 128 == 0 && M <= (1u << 24) && N <= (1u << 24) && K <= (1u << 20);
}

static size_t pf_q_bytes(size_t M, size_t K) { return align_up(M * K, 256); }
static size_t pf_vec_bytes(size_t M) { return align_up(M * 4, 256); }

size_t prefill_workspace_bytes(size_t M, size_t K, size_t N)
{
    (void)N;
    return pf_q_bytes(M, K) + 2 * pf_vec_bytes(M);   // int8 activations, fp32 scales, int32 row sums
}

static bitnet_status_t encode_map(CUtensorMap *map, const void *base, uint64_t inner, uint64_t rows, uint64_t row_stride_bytes,
                                  uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swizzle)
{
    const cuuint64_t dims[2] = {inner, rows};
    const cuuint64_t strides[1] = {row_stride_bytes};
    const cuuint32_t box[2] = {box_inner, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    // the driver entry point is looked up through the runtime, so the library does not link
    // against libcuda and still loads on a machine without a driver
    typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                 const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        BITNET_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess)
            return fail(BITNET_ERR_CUDA_DRIVER, "cuTensorMapEncodeTiled is not available from this driver");
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(BITNET_ERR_CUDA_DRIVER, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return BITNET_OK;
}

bitnet_status_t launch_prefill(const ForwardArgs &a, void *workspace, size_t workspace_bytes, cudaStream_t stream)
{
    if (!prefill_supports(a.M, a.K, a.N))
        return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "tensor-core path needs K %% 128 == 0 (M=%zu K=%zu N=%zu)", a.M, a.K, a.N);
    if (workspace_bytes < prefill_workspace_bytes(a.M, a.K, a.N))
        return fail(BITNET_ERR_WORKSPACE, "workspace too small for the tensor-core path");
    if ((reinterpret_cast<uintptr_t>(a.wp) & 15) || (reinterpret_cast<uintptr_t>(a.x) & 15))
        return fail(BITNET_ERR_INVALID_CONFIG, "packed weights and activations must be 16-byte aligned");
    if (a.q_out && (reinterpret_cast<uintptr_t>(a.q_out) & 15)) return fail(BITNET_ERR_INVALID_CONFIG, "q_out must be 16-byte aligned");

    char *ws = static_cast<char *>(workspace);
    int8_t *q_perm = reinterpret_cast<int8_t *>(ws);
    float *a_scale = reinterpret_cast<float *>(ws + pf_q_bytes(a.M, a.K));
    int *rowsum = reinterpret_cast<int *>(ws + pf_q_bytes(a.M, a.K) + pf_vec_bytes(a.M));

    quantize_rows_perm_kernel<<<(unsigned)a.M, 256, 0, stream>>>(a.x, a.K, q_perm, a_scale, rowsum, a.q_out, a.a_scale_out);
    BITNET_TRY(check_launch("quantize_rows_perm_kernel"));

    CUtensorMap map_a, map_w;
    BITNET_TRY(encode_map(&map_a, q_perm, a.K, a.M, a.K, PF_BK, PF_BM, CU_TENSOR_MAP_SWIZZLE_128B));
    BITNET_TRY(encode_map(&map_w, a.wp, a.K / 4, a.N, a.K / 4, PF_BK / 4, PF_BN, CU_TENSOR_MAP_SWIZZLE_NONE));

    PrefillParams p = {};
    p.y = a.y; p.acc_out = a.acc_out; p.a_scale = a_scale; p.rowsum = rowsum; p.w_scale = a.w_scale;
    p.M = (int)a.M; p.K = (int)a.K; p.N = (int)a.N; p.ldy = a.ldy ? a.ldy : a.N;
    p.m_tiles = (int)((a.M + PF_BM - 1) / PF_BM);
    p.n_tiles = (int)((a.N + PF_BN - 1) / PF_BN);
    p.k_tiles = (int)(a.K / PF_BK);

    static bool attr_set = false;
    if (!attr_set) {
        BITNET_CUDA(cudaFuncSetAttribute(prefill_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PF_SMEM));
        attr_set = true;
    }
    const int tiles = p.m_tiles * p.n_tiles;
    const int sms = device_sm_count();
    const int grid = tiles < sms ? tiles : sms;
    prefill_gemm_kernel<<<grid, PF_THREADS, PF_SMEM, stream>>>(map_a, map_w, p);
    return check_launch("prefill_gemm_kernel");
}

}  // namespace bitnet
