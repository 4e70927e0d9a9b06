// Prefill-time BitLinear (many tokens): int8 x ternary GEMM on the 5th-generation tensor cores.
//
//   1. quantize_rows_perm_kernel: per-token absmax int8 quantisation of x[M,K] into scratch,
//      with the 16 values of every 16-wide k group stored transposed (byte 4j+i holds k = 4i+j),
//      plus the row sums sum_k q[m,k].
//   2. prefill_gemm_kernel: persistent CTAs; the accumulator tile is 128 output features (tensor-memory
//      lanes) x up to 192 tokens (columns), i.e. the weights are the MMA's A operand.
//        warp 0      TMA producer: per 128-wide k slice the int8 activation tile (tokens x 128 bytes,
//                    128-byte swizzle) and the PACKED weight tile (128 rows x 32 bytes); the packed
//                    weights run two slice pairs ahead of the activations
//        warps 2-9   expand packed weights to u8 codes {0,1,2} in registers and write them straight
//                    into TENSOR MEMORY (tcgen05.st), where the MMA reads its A operand: a thread
//                    owns one feature row; (w >> 2j) & 0x03030303 yields the four bytes
//                    k = j, j+4, j+8, j+12 of a group, i.e. word j of the transposed group order the
//                    activations were stored in.  Expanded weights never touch shared memory.
//                    (two groups of four warps take the slice pairs in turn)
//        warp 1      one thread issues tcgen05.mma kind::i8 (M=128, N=tokens, K=32; u8 x s8 -> s32),
//                    A from tensor memory, B (activations) from shared memory; two accumulators
//                    alternate between tiles
//        warps 10-13 epilogue: tcgen05.ld the accumulator, subtract the row sum
//                    (sum_k (code-1) q = sum_k code q - sum_k q), scale, stage 32 x 32 blocks in
//                    shared memory and write y with TMA stores
//      Work is dealt in whole tiles, or -- when whole tiles would leave most of a wave idle -- in
//      equal runs of k slices with an exact integer fix-up of the tiles shared by two CTAs.
//      Every barrier wait is bounded; a wait that runs out raises an error flag and the CTA
//      drains and frees its tensor memory.
//
// Semantics: TernaryProcessor::quantize_activations + ternary_matmul_generic
// (bitnet-inference/src/engine/ternary_operations.rs:117-172, :283-338) with int32 accumulation
// on the packed layout of BitPacked2BitPacker (bitnet-quant/src/quantization/packing.rs:352-394).
// The reference has no tensor-core kernel; this is what its BitLinearLayer::forward
// (transformer_layers.rs:119-202) computes for a [B*S, K] input.
#include <cuda.h>
#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace bitnet {

// Set (bit 1) when a bounded wait of the GEMM kernel ran out -- read with bitnet_device_error_flags().
__device__ unsigned g_prefill_error_flags;

constexpr int PF_BF = 128;                         // output features per tile (the MMA's M: tensor-memory lanes)
constexpr int PF_BT = 192;                         // tokens per tile (the MMA's N)
constexpr int PF_BK = 128;                         // k per slice (bytes of int8)
constexpr int PF_PAIR = 2;                         // k slices per hand-over between the roles (one barrier round per pair)
constexpr int PF_RING = 3;                         // activation pairs in flight (the ring holds PF_RING * PF_PAIR slices)
constexpr int PF_WLEAD = 2;                        // the packed weights run this many pairs ahead of the activations, so
                                                   // that a pair's weights are expanded before its activations land
constexpr int PF_WRING = PF_RING + PF_WLEAD;       // packed-weight pairs in flight
constexpr int PF_XSTAGES = PF_RING * PF_PAIR, PF_WSTAGES = PF_WRING * PF_PAIR;
constexpr int PF_ASLOTS = 2;                       // expanded-weight pairs in tensor memory
constexpr int PF_X_BYTES = PF_BT * PF_BK;          // 24 KB
constexpr int PF_WP_BYTES = PF_BF * PF_BK / 4;     // 4 KB packed
constexpr int PF_EXP_WARPS = 8;                    // warps that expand packed weights
constexpr int PF_GROUPS = 2;                       // expander groups working on alternate k slices
constexpr int PF_THREADS = (2 + PF_EXP_WARPS + 4) * 32;   // producer, MMA, expanders, epilogue
constexpr unsigned PF_WAIT_LIMIT = 1u << 20;
constexpr int PF_TMEM_A0 = 2 * PF_BT;              // tensor-memory columns: two accumulators, then the weight ring
constexpr int PF_A_COLS = PF_BK / 4;               // 32 columns hold 128 bytes of k per lane
static_assert(PF_TMEM_A0 + PF_ASLOTS * PF_PAIR * PF_A_COLS <= 512, "tensor memory has 512 columns");
constexpr int PF_WARP_OUT_BYTES = 32 * 32 * 4;     // epilogue staging per warp: 32 tokens x 32 features fp32, two of them
constexpr int PF_OUT_BYTES = 4 * PF_WARP_OUT_BYTES;
constexpr size_t PF_RING_BYTES = (size_t)PF_XSTAGES * PF_X_BYTES + (size_t)PF_WSTAGES * PF_WP_BYTES;
constexpr size_t PF_SMEM = PF_RING_BYTES + 2 * PF_OUT_BYTES + 1024;   // + alignment slack
constexpr size_t PF_SLOT_BYTES = (size_t)PF_BF * PF_BT * 4;   // one partial accumulator tile

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

// One CTA per token row, one read of the row when it fits the registers (two 16-wide groups per
// thread).  Short rows take 128-thread CTAs: more rows in flight per SM, which is what bounds this
// kernel (a row is one dependent chain load -> absmax -> quantise -> store).
// q_perm[m, 16G + 4j + i] = q[m, 16G + 4i + j]; rowsum[m] = sum_k q[m,k].
// Semantics: TernaryProcessor::quantize_activations (ternary_operations.rs:130-163).
template <int THREADS>
__global__ void __launch_bounds__(THREADS, THREADS == 128 ? 8 : 4) quantize_rows_perm_kernel(const float *__restrict__ x, size_t K,
                                                                 int8_t *__restrict__ q_perm, float *__restrict__ a_scale,
                                                                 int *__restrict__ rowsum, int8_t *__restrict__ q_out,
                                                                 float *__restrict__ a_scale_out, unsigned *__restrict__ counters,
                                                                 int n_counters)
{
    // the GEMM that follows may start (allocate tensor memory, fetch packed weights) while this runs;
    // it waits for this grid before it touches anything written here
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // launched with programmatic dependent launch itself (BITNET_FLAG_PDL): x and the scratch this grid
    // overwrites belong to the kernels before it until they have finished
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // the GEMM counts the parts of split tiles in these; they start at zero
    if (blockIdx.x == 0)
        for (int i = threadIdx.x; i < n_counters; i += THREADS) counters[i] = 0u;
    __shared__ unsigned s_key[THREADS / 32];
    __shared__ int s_sum[THREADS / 32];
    const size_t m = blockIdx.x;
    const float *row = x + m * K;
    const int tid = threadIdx.x;
    const size_t n_groups = K / 16;
    const bool resident = n_groups <= 2 * THREADS;   // two 16-wide groups per thread stay in registers

    float4 f[2][4];
    unsigned key = 0;
    if (resident) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const size_t G = tid + u * THREADS;
            if (G < n_groups) {
                const float4 *src = reinterpret_cast<const float4 *>(row + G * 16);
#pragma unroll
                for (int v = 0; v < 4; ++v) f[u][v] = __ldg(src + v);
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u)
            if ((size_t)(tid + u * THREADS) < n_groups) {
#pragma unroll
                for (int v = 0; v < 4; ++v)
                    key = max(max(key, abs_key(f[u][v].x)), max(abs_key(f[u][v].y), max(abs_key(f[u][v].z), abs_key(f[u][v].w))));
            }
    } else {
        for (size_t G = tid; G < n_groups; G += THREADS) {
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
    for (int w = 0; w < THREADS / 32; ++w) key = max(key, s_key[w]);
    const float absmax = __uint_as_float(key);
    const float scale = quant_scale(absmax);
    // a huge or tiny absmax makes the scale leave the normal range; the fast rounding assumes it has not
    const bool fast = scale >= 1e-30f && scale <= 1e30f;

    int sum = 0;
    const size_t rounds = resident ? 2 : (n_groups + THREADS - 1) / THREADS;
    for (size_t u = 0; u < rounds; ++u) {
        const size_t G = tid + u * THREADS;
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
        for (int w = 0; w < THREADS / 32; ++w) total += s_sum[w];
        rowsum[m] = total;
        a_scale[m] = dequant_scale(absmax);
        if (a_scale_out) a_scale_out[m] = dequant_scale(absmax);
    }
}

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
__device__ __forceinline__ bool pf_mbar_wait(unsigned long long *bar, unsigned parity, bool backoff_req = true)
{
    const unsigned addr = pf_smem_u32(bar);
    {   // the usual case: the phase completed long ago -- a plain test, not the potentially suspending wait
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
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
        (void)backoff_req; __nanosleep(n < 16 ? 32 : 128);   // a waiting warp must not take issue slots from the working ones
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

__device__ __forceinline__ void pf_mma_i8_ts(unsigned tmem_d, unsigned tmem_a, unsigned long long b_desc, unsigned idesc,
                                             unsigned accumulate)
{
    // A (expanded weights) comes from tensor memory, B (activations) from shared memory
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
        "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void pf_tmem_st32(unsigned taddr, const unsigned (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
// Barrier among the four epilogue warps that also ANDs a predicate (all leave a loop together).
__device__ __forceinline__ bool pf_epi_all(bool ok)
{
    unsigned out;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "barrier.cta.red.and.pred p, 1, 128, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(out)
        : "r"(ok ? 1u : 0u)
        : "memory");
    return out != 0;
}

__device__ __forceinline__ void pf_tma_store_2d(const CUtensorMap *map, int x, int y, const void *src)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
                 "r"(pf_smem_u32(src)), "r"(x), "r"(y)
                 : "memory");
}
struct PrefillParams {
    float *y;
    int32_t *acc_out;
    const float *a_scale;
    const int *rowsum;
    int *slots;          // partial accumulator tiles, two per CTA, [token][feature] int32
    unsigned *counters;  // per tile: k slices contributed so far (zero at launch)
    float w_scale;
    int M, K, N;
    size_t ldy;
    int m_tiles, n_tiles, k_tiles;
    int tma_store;       // y can be written with TMA (16-byte aligned rows), else plain stores
    int bt;              // tokens per tile (the MMA's N): a multiple of 32, at most PF_BT
    int whole_tiles;     // ranges end on tile boundaries (no tile is split between CTAs)
    float *y_peers[8];   // output-feature split over several GPUs: every output goes to each of these (own and peer
    int n_peers;         // memory, plain stores over NVLink; TMA is used for this GPU's memory only); 0 = write y only
};

// instruction descriptor: D = s32, A = u8 (codes, tensor memory), B = s8 (activations, K-major), N = tokens, M = 128
__host__ __device__ constexpr unsigned pf_idesc(int bt) { return (2u << 4) | (0u << 7) | (1u << 10) | ((unsigned)(bt >> 3) << 17) | ((unsigned)(PF_BF >> 4) << 24); }

// The work of the whole GEMM is the sequence of (tile, k slice) units, tile-major; CTA c takes
// the contiguous range [U*c/G, U*(c+1)/G), so every CTA has the same number of k slices whatever
// the tile count.  A segment is the part of one tile inside a range.  A CTA works through its
// segments in the order: first (often a partial tile), last (often a partial tile), then the whole
// tiles in between -- the fix-up of a tile shared with a neighbour then happens early on both
// sides and hides behind the MMAs of the whole tiles, and the kernel's tail is a plain tile.
struct PfSegment {
    int tile, kb, ke;
};
struct PfSchedule {
    int t_first, kb_first;   // tile and k position of the range's first unit
    int t_last, ke_last;     // tile of the range's last unit, end of its k range
    int n_seg;
};
__device__ __forceinline__ long long pf_range_start(long long units, int c, int ctas, int k_tiles = 0)
{
    if (k_tiles > 0) {   // whole tiles only: split the tile count, not the slice count
        const unsigned tiles = (unsigned)(units / k_tiles);
        return (long long)(unsigned)((unsigned long long)tiles * (unsigned)c / (unsigned)ctas) * k_tiles;
    }
    // 32-bit arithmetic when it fits (the usual case): 64-bit division is slow on the device
    if (units < (1ll << 31) / (ctas > 0 ? ctas : 1)) return (long long)((unsigned)units * (unsigned)c / (unsigned)ctas);
    return units * c / ctas;
}
__device__ __forceinline__ PfSchedule pf_schedule(long long u_begin, long long u_end, int k_tiles)
{
    PfSchedule sch;
    sch.n_seg = 0;
    sch.t_first = sch.kb_first = sch.t_last = sch.ke_last = 0;
    if (u_end <= u_begin) return sch;
    if (u_end < (1ll << 31)) {
        sch.t_first = (int)((unsigned)u_begin / (unsigned)k_tiles);
        sch.t_last = (int)((unsigned)(u_end - 1) / (unsigned)k_tiles);
    } else {
        sch.t_first = (int)(u_begin / k_tiles);
        sch.t_last = (int)((u_end - 1) / k_tiles);
    }
    sch.kb_first = (int)(u_begin - (long long)sch.t_first * k_tiles);
    sch.ke_last = (int)(u_end - (long long)sch.t_last * k_tiles);
    sch.n_seg = sch.t_last - sch.t_first + 1;
    return sch;
}
__device__ __forceinline__ PfSegment pf_segment(const PfSchedule &sch, int idx, int k_tiles)
{
    PfSegment sg;
    if (sch.n_seg == 1) {
        sg.tile = sch.t_first; sg.kb = sch.kb_first; sg.ke = sch.ke_last;
    } else if (idx == 0) {
        sg.tile = sch.t_first; sg.kb = sch.kb_first; sg.ke = k_tiles;
    } else if (idx == 1) {
        sg.tile = sch.t_last; sg.kb = 0; sg.ke = sch.ke_last;
    } else {
        sg.tile = sch.t_first + idx - 1; sg.kb = 0; sg.ke = k_tiles;
    }
    return sg;
}

__global__ void __launch_bounds__(PF_THREADS, 1)
prefill_gemm_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_y, const PrefillParams p)
{
    extern __shared__ unsigned char pf_smem_raw[];
    __shared__ __align__(8) unsigned long long s_full_x[PF_RING];        // a pair's activations have landed
    __shared__ __align__(8) unsigned long long s_full_w[PF_WRING];       // a pair's packed weights have landed
    __shared__ __align__(8) unsigned long long s_full_a[PF_ASLOTS];      // a pair's weights are expanded in tensor memory
    __shared__ __align__(8) unsigned long long s_done[PF_RING];          // the MMAs of a pair have read their operands
    __shared__ __align__(8) unsigned long long s_acc_full[2], s_acc_empty[2];
    __shared__ unsigned s_tmem_base;
    __shared__ unsigned s_prev_count;
    __shared__ __align__(16) int2 s_tab[4 * PF_BT];   // per epilogue warp, per token of the tile: row sum, scale bits
    __shared__ __align__(8) unsigned long long s_in[4];   // per epilogue warp: a fetched part of a split tile has landed

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // a kernel launched behind this one with programmatic dependent launch may be scheduled as CTAs here retire
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(pf_smem_raw) + 1023) & ~uintptr_t(1023));
    // activation stages start 1024-byte aligned (the 128-byte swizzle needs it); the packed weights follow
    auto stage_x = [&](int s) { return smem + (size_t)s * PF_X_BYTES; };
    auto stage_wp = [&](int s) { return smem + (size_t)PF_XSTAGES * PF_X_BYTES + (size_t)s * PF_WP_BYTES; };

    if (tid == 0) {
        for (int r = 0; r < PF_RING; ++r) pf_mbar_init(&s_full_x[r], 1);
        for (int r = 0; r < PF_WRING; ++r) pf_mbar_init(&s_full_w[r], 1);
        for (int sa = 0; sa < PF_ASLOTS; ++sa) pf_mbar_init(&s_full_a[sa], PF_EXP_WARPS / PF_GROUPS);
        for (int r = 0; r < PF_RING; ++r) pf_mbar_init(&s_done[r], 1);
        for (int w = 0; w < 4; ++w) pf_mbar_init(&s_in[w], 1);
        for (int b = 0; b < 2; ++b) {
            pf_mbar_init(&s_acc_full[b], 1);
            pf_mbar_init(&s_acc_empty[b], 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // all 512 tensor-memory columns: two 128 x 192 s32 accumulators + the weight slots
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(pf_smem_u32(&s_tmem_base)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = s_tmem_base;

    const long long units = (long long)p.m_tiles * p.n_tiles * p.k_tiles;
    const int whole_k = p.whole_tiles ? p.k_tiles : 0;
    const long long u_begin = pf_range_start(units, (int)blockIdx.x, (int)gridDim.x, whole_k);
    const long long u_end = pf_range_start(units, (int)blockIdx.x + 1, (int)gridDim.x, whole_k);
    const int n_slices = (int)(u_end - u_begin);   // k slices of this CTA, numbered it = 0.. across its segments
    const PfSchedule sch = pf_schedule(u_begin, u_end, p.k_tiles);
    // Slices are handed between the roles in pairs (pair pp = it / 2): one barrier round per pair
    // keeps the single MMA-issuing thread's waits and commits off the critical path.

    if (warp == 0) {
        // ===================== TMA producer =====================
        if (lane == 0) {
            const int n_pairs = (n_slices + PF_PAIR - 1) / PF_PAIR;
            // two cursors walk this CTA's slices in segment order: one for the activations, one for
            // the packed weights that run ahead
            struct Cursor {
                int idx, n_tile, m_tile, kt, ke;
            };
            auto cursor_seg = [&](Cursor &c, int idx) {
                c.idx = idx;
                if (idx >= sch.n_seg) return;
                const PfSegment sg = pf_segment(sch, idx, p.k_tiles);
                c.n_tile = sg.tile / p.m_tiles;
                c.m_tile = sg.tile - c.n_tile * p.m_tiles;
                c.kt = sg.kb;
                c.ke = sg.ke;
            };
            auto advance = [&](Cursor &c) {
                if (++c.kt == c.ke) cursor_seg(c, c.idx + 1);
            };
            Cursor cx, cw;
            cursor_seg(cx, 0);
            cw = cx;
            auto load_w = [&](int q) {   // packed weights of pair q (called for q = 0, 1, 2, ... in order)
                const int cnt = n_slices - q * PF_PAIR < PF_PAIR ? n_slices - q * PF_PAIR : PF_PAIR;
                if (cnt <= 0) return;
                pf_mbar_expect_tx(&s_full_w[q % PF_WRING], (unsigned)cnt * PF_WP_BYTES);
                for (int h = 0; h < cnt; ++h) {
                    pf_tma_load_2d(stage_wp((q * PF_PAIR + h) % PF_WSTAGES), &map_w, cw.kt * (PF_BK / 4), cw.n_tile * PF_BF,
                                   &s_full_w[q % PF_WRING]);
                    advance(cw);
                }
            };
            for (int q = 0; q < PF_WLEAD; ++q) load_w(q);
            asm volatile("griddepcontrol.wait;" ::: "memory");   // the int8 activations come from the quantiser grid
            for (int pp = 0; pp < n_pairs; ++pp) {
                const int cnt = n_slices - pp * PF_PAIR < PF_PAIR ? n_slices - pp * PF_PAIR : PF_PAIR;
                // the pair that used these stages PF_RING pairs ago has been consumed; its packed
                // weights (PF_WRING pairs behind the ones loaded below) as well
                if (!pf_mbar_wait(&s_done[pp % PF_RING], ((unsigned)(pp / PF_RING) & 1u) ^ 1u, false)) break;
                pf_mbar_expect_tx(&s_full_x[pp % PF_RING], (unsigned)cnt * (unsigned)(p.bt * PF_BK));
                for (int h = 0; h < cnt; ++h) {
                    pf_tma_load_2d(stage_x((pp * PF_PAIR + h) % PF_XSTAGES), &map_x, cx.kt * PF_BK, cx.m_tile * p.bt,
                                   &s_full_x[pp % PF_RING]);
                    advance(cx);
                }
                load_w(pp + PF_WLEAD);
            }
        }
    } else if (warp == 1) {
        // ===================== MMA issuer =====================
        if (lane == 0) {
            int it = 0, sc = 0;
            bool ok = true;
            const unsigned idesc = pf_idesc(p.bt);
            for (int si = 0; si < sch.n_seg && ok; ++si) {
                const PfSegment sg = pf_segment(sch, si, p.k_tiles);
                const int buf = sc & 1;
                const unsigned acc_ph = (unsigned)(sc >> 1) & 1u;
                ++sc;
                if (!pf_mbar_wait(&s_acc_empty[buf], acc_ph ^ 1u, false)) { ok = false; break; }   // epilogue drained this accumulator
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned tmem_d = tmem_base + (unsigned)buf * PF_BT;
                for (int kt = sg.kb; kt < sg.ke; ++kt, ++it) {
                    const int s = it % PF_XSTAGES;
                    const int pp = it / PF_PAIR, h = it % PF_PAIR;
                    if (h == 0) {   // the pair's expanded weights are in tensor memory and its activations have landed
                        // (the expanders wait for the pair's activations before they report, so one wait covers both)
                        if (!pf_mbar_wait(&s_full_a[pp % PF_ASLOTS], (unsigned)(pp / PF_ASLOTS) & 1u, false)) { ok = false; break; }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    }
                    const unsigned tmem_a = tmem_base + (unsigned)(PF_TMEM_A0 + ((pp % PF_ASLOTS) * PF_PAIR + h) * PF_A_COLS);
                    const unsigned long long b_desc = pf_smem_desc(pf_smem_u32(stage_x(s)));
#pragma unroll
                    for (int ks = 0; ks < PF_BK / 32; ++ks)   // 32 bytes of k per instruction: 8 columns / +2 16-byte units
                        pf_mma_i8_ts(tmem_d, tmem_a + 8u * ks, b_desc + 2ull * ks, idesc, (kt != sg.kb || ks != 0) ? 1u : 0u);
                    if (h == PF_PAIR - 1 || it == n_slices - 1) {
                        pf_commit(&s_done[pp % PF_RING]);   // TMA stages and the tensor-memory slot of the pair are free
                    }
                }
                if (ok) pf_commit(&s_acc_full[buf]);
            }
        }
    } else if (warp < 2 + PF_EXP_WARPS) {
        // ===================== weight expanders: PF_GROUPS groups take the pairs in turn =====================
        // A thread owns one feature row of the tile: 32 packed bytes per slice become the 128 code
        // bytes of its tensor-memory lane.  (w >> 2j) & 0x03030303 is word j of a 16-wide group in
        // the transposed k order the activations were stored in.
        const int group = (warp - 2) / (PF_EXP_WARPS / PF_GROUPS);
        const int quarter = warp & 3;            // the tensor-memory lanes this warp may touch
        const int row = quarter * 32 + lane;
        const int n_pairs = (n_slices + PF_PAIR - 1) / PF_PAIR;
        bool ok = true;
        for (int pp = group; pp < n_pairs && ok; pp += PF_GROUPS) {
            const int slot = pp % PF_ASLOTS;
            // expand both slices of the pair into registers first: this part does not need the
            // tensor-memory slot and overlaps the MMAs that still read it
            unsigned r[PF_PAIR][32];
            if (!pf_warp_wait(&s_full_w[pp % PF_WRING], (unsigned)(pp / PF_WRING) & 1u)) { ok = false; break; }
#pragma unroll
            for (int h = 0; h < PF_PAIR; ++h) {
                const int it = pp * PF_PAIR + h;
                if (it >= n_slices) break;
                const int s = it % PF_WSTAGES;
                const uint4 *src = reinterpret_cast<const uint4 *>(stage_wp(s) + row * (PF_BK / 4));
                const uint4 w0 = src[0], w1 = src[1];
                const unsigned w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    r[h][4 * g + 0] = w[g] & 0x03030303u;
                    r[h][4 * g + 1] = (w[g] >> 2) & 0x03030303u;
                    r[h][4 * g + 2] = (w[g] >> 4) & 0x03030303u;
                    r[h][4 * g + 3] = (w[g] >> 6) & 0x03030303u;
                }
            }
            if (!ok) break;
            if (pp >= PF_ASLOTS) {   // the MMAs that read this slot (pair pp - PF_ASLOTS) are done
                const int pd = pp - PF_ASLOTS;
                if (!pf_warp_wait(&s_done[pd % PF_RING], (unsigned)(pd / PF_RING) & 1u)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            const unsigned ta = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(PF_TMEM_A0 + slot * PF_PAIR * PF_A_COLS);
            pf_tmem_st32(ta, r[0]);
            if (pp * PF_PAIR + 1 < n_slices) pf_tmem_st32(ta + PF_A_COLS, r[1]);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            // report the pair only when its activations have landed too: the MMA thread then needs one wait
            if (!pf_warp_wait(&s_full_x[pp % PF_RING], (unsigned)(pp / PF_RING) & 1u)) { ok = false; break; }
            if (lane == 0) pf_mbar_arrive(&s_full_a[slot]);
        }
    } else {
        // ===================== epilogue (4 warps; a thread owns one feature row of the accumulator) =====================
        // Accumulator lanes are features, columns are tokens, so a warp's 32 lanes hold 32 consecutive
        // features of one token.  Each warp works on its own: a chunk of 32 tokens x 32 features goes
        // through the warp's private staging buffer ([token][feature], conflict-free) and leaves as one
        // TMA store; no barrier between the warps inside a tile.
        const int quarter = warp & 3;   // the tensor-memory lanes a warp may touch: 32 * (warp % 4)
        const int frow = quarter * 32 + lane;
        const bool epi_leader = tid == (2 + PF_EXP_WARPS) * 32;
        unsigned char *my_stage = smem + PF_RING_BYTES + (size_t)quarter * (2 * PF_WARP_OUT_BYTES);   // two 4 KB buffers
        int sc = 0, n_staged = 0, n_in = 0;
        bool ok = true;
        asm volatile("griddepcontrol.wait;" ::: "memory");   // row sums, scales and the zeroed counters come from the quantiser grid

        // the copy that read buffer (n_staged & 1) two sends ago has finished reading: lane 0 waited for it
        // right after the previous send, and the __syncwarp orders that before everybody's stores
        auto send_chunk = [&](const unsigned (&v)[32], int x, int yrow) {   // token-major, to y
            unsigned *st = reinterpret_cast<unsigned *>(my_stage + (size_t)(n_staged & 1) * PF_WARP_OUT_BYTES);
            ++n_staged;
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 32; ++j) st[j * 32 + lane] = v[j];
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                pf_tma_store_2d(&map_y, x, yrow, st);
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");   // the other buffer is free again
            }
        };
        // a part of a split tile goes to its slot feature-major: the thread's 32 values are 128
        // contiguous bytes (16-byte pieces XOR-swizzled so that the shared-memory accesses do not
        // collide); a warp's 32 rows are 4 KB contiguous in the slot
        auto send_partial = [&](const unsigned (&v)[32], int *slot_piece) {
            unsigned char *st = my_stage + (size_t)(n_staged & 1) * PF_WARP_OUT_BYTES;
            ++n_staged;
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i)
                *reinterpret_cast<uint4 *>(st + lane * 128 + ((i ^ (lane & 7)) << 4)) = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(slot_piece + quarter * 32 * 32),
                             "r"(pf_smem_u32(st)), "r"(PF_WARP_OUT_BYTES)
                             : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            }
        };
        // fetch this warp's 4 KB of another CTA's part into the staging buffer that is free, add it to v
        auto add_partial = [&](unsigned (&v)[32], const int *slot_piece) -> bool {
            unsigned char *st = my_stage + (size_t)(n_staged & 1) * PF_WARP_OUT_BYTES;
            __syncwarp();   // lane 0 has seen the last copy out of this buffer finish reading
            if (lane == 0) {
                pf_mbar_expect_tx(&s_in[quarter], PF_WARP_OUT_BYTES);
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                 pf_smem_u32(st)),
                             "l"(slot_piece + quarter * 32 * 32), "r"(PF_WARP_OUT_BYTES), "r"(pf_smem_u32(&s_in[quarter]))
                             : "memory");
            }
            const bool got = pf_warp_wait(&s_in[quarter], (unsigned)n_in & 1u);
            ++n_in;
            if (!got) return false;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint4 t = *reinterpret_cast<const uint4 *>(st + lane * 128 + ((i ^ (lane & 7)) << 4));
                v[4 * i + 0] += t.x;
                v[4 * i + 1] += t.y;
                v[4 * i + 2] += t.z;
                v[4 * i + 3] += t.w;
            }
            return true;
        };

        for (int si = 0; si < sch.n_seg && ok; ++si) {
            const PfSegment sg = pf_segment(sch, si, p.k_tiles);
            const int n_tile = sg.tile / p.m_tiles, m_tile = sg.tile % p.m_tiles;
            const int buf = sc & 1;
            const unsigned acc_ph = (unsigned)(sc >> 1) & 1u;
            ++sc;
            const bool whole = sg.kb == 0 && sg.ke == p.k_tiles;
            const int m0 = m_tile * p.bt;
            const int n = n_tile * PF_BF + frow;
            const bool n_ok = n < p.N;
            // per token of the tile: row sum and scale (each warp keeps its own copy), read back below as
            // broadcast 16-byte loads
            int2 *tab = s_tab + quarter * PF_BT;
            __syncwarp();
            for (int j = lane; j < p.bt; j += 32) {
                const int m = m0 + j;
                int2 e = make_int2(0, 0);
                if (m < p.M) {
                    e.x = __ldg(p.rowsum + m);
                    e.y = __float_as_int(__fmul_rn(p.w_scale, __ldg(p.a_scale + m)));
                }
                tab[j] = e;
            }
            ok = pf_epi_all(pf_warp_wait(&s_acc_full[buf], acc_ph));   // the four warps go on, or give up, together
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)buf * PF_BT;

            // a tile that is split between CTAs: publish this part, and whoever completes the
            // tile's k range adds the published parts to its own (integer sums: order is irrelevant)
            int c_lo = 0, c_hi = -1;   // the CTAs that hold parts of this tile (when it is split)
            bool finish = true;
            if (!whole) {
                // claim first: the CTA whose claim completes the tile's k range finishes the tile and need not
                // publish its own part; everyone else publishes and moves on
                const unsigned len = (unsigned)(sg.ke - sg.kb);
                if (epi_leader) s_prev_count = atomicAdd(p.counters + 2 * sg.tile, len);
                pf_epi_all(true);
                finish = s_prev_count + len == (unsigned)p.k_tiles;
                pf_epi_all(true);   // s_prev_count may be rewritten only after everyone has read it
                if (!finish) {
                    int *slot = p.slots + ((size_t)2 * blockIdx.x + (sg.tile != sch.t_first ? 1 : 0)) * (PF_BF * PF_BT);
#pragma unroll 1
                    for (int c = 0; c < p.bt / 32; ++c) {
                        unsigned r[32];
                        pf_tmem_ld32(taddr + (unsigned)c * 32, r);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        send_partial(r, slot + c * 32 * PF_BF);
                    }
                    if (lane == 0) {
                        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // this warp's pieces are written
                        asm volatile("fence.proxy.async;" ::: "memory");
                        __threadfence();
                    }
                    pf_epi_all(true);
                    if (epi_leader) {
                        __threadfence();
                        atomicAdd(p.counters + 2 * sg.tile + 1, len);
                    }
                } else {
                    // the other parts were claimed before this one, so their CTAs are running and publish
                    // without waiting for anybody: a short, bounded wait
                    if (epi_leader) {
                        const volatile unsigned *published = p.counters + 2 * sg.tile + 1;
                        unsigned seen = 0;
                        for (unsigned n = 0; n < PF_WAIT_LIMIT; ++n) {
                            seen = *published;
                            if (seen + len == (unsigned)p.k_tiles) break;
                            __nanosleep(64);
                        }
                        if (seen + len != (unsigned)p.k_tiles) atomicOr(&g_prefill_error_flags, 2u);
                        __threadfence();
                    }
                    pf_epi_all(true);
                    const long long t_begin = (long long)sg.tile * p.k_tiles, t_end = t_begin + p.k_tiles;
                    c_lo = (int)(((t_begin + 1) * gridDim.x - 1) / units);   // owners of the tile's first and last unit
                    c_hi = (int)((t_end * gridDim.x - 1) / units);
                }
            }
            if (finish) {
#pragma unroll 1
                for (int c = 0; c < p.bt / 32; ++c) {
                    if (m0 + c * 32 >= p.M) break;   // warp-uniform
                    unsigned r[32];
                    pf_tmem_ld32(taddr + (unsigned)c * 32, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    for (int cc = c_lo; cc <= c_hi; ++cc) {
                        if (cc == (int)blockIdx.x) continue;
                        const long long t_begin = (long long)sg.tile * p.k_tiles, t_end = t_begin + p.k_tiles;
                        const long long cb = pf_range_start(units, cc, (int)gridDim.x), ce = pf_range_start(units, cc + 1, (int)gridDim.x);
                        if ((cb > t_begin ? cb : t_begin) >= (ce < t_end ? ce : t_end)) continue;   // an empty range
                        const int *piece = p.slots + ((size_t)2 * cc + (sg.tile != (int)(cb / p.k_tiles) ? 1 : 0)) * (PF_BF * PF_BT) + (c * 32) * PF_BF;
                        if (!add_partial(r, piece)) break;
                    }
                    const int m_left = p.M - (m0 + c * 32);   // tokens of this chunk that exist
                    if (p.acc_out) {   // parity-test output of the integer sums; kept out of the loop below so that it stays branch-free
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (n_ok && j < m_left) p.acc_out[(size_t)(m0 + c * 32 + j) * p.ldy + n] = (int)r[j] - tab[c * 32 + j].x;
                    }
                    // loads first, arithmetic after: the warp issues in order, so a load placed next to
                    // its use would expose its latency 32 times
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        int4 e[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) e[i] = reinterpret_cast<const int4 *>(tab)[c * 16 + h * 8 + i];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int j = h * 16 + 2 * i;
                            r[j] = __float_as_uint(__fmul_rn((float)((int)r[j] - e[i].x), __int_as_float(e[i].y)));
                            r[j + 1] = __float_as_uint(__fmul_rn((float)((int)r[j + 1] - e[i].z), __int_as_float(e[i].w)));
                        }
                    }
                    if (p.tma_store) {
                        send_chunk(r, n_tile * PF_BF + quarter * 32, m0 + c * 32);
                    } else if (p.n_peers) {
                        // this GPU's column slice, stored into every GPU's full-width output: a warp writes 128
                        // contiguous bytes per token row and destination
                        for (int pr = 0; pr < p.n_peers; ++pr) {
                            float *ycol = p.y_peers[pr] + (size_t)(m0 + c * 32) * p.ldy + n;
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (n_ok && j < m_left) ycol[(size_t)j * p.ldy] = __uint_as_float(r[j]);
                        }
                    } else {
                        float *ycol = p.y + (size_t)(m0 + c * 32) * p.ldy + n;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (n_ok && j < m_left) ycol[(size_t)j * p.ldy] = __uint_as_float(r[j]);
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) pf_mbar_arrive(&s_acc_empty[buf]);
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // shared memory outlives the stores
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

// How a problem is cut: tokens per tile, whether tiles may be split between CTAs, and the grid.
struct PfPlan {
    int bt;
    bool whole_tiles;
    size_t tiles, grid;
};
static size_t pf_tiles(size_t M, size_t N, int bt) { return ((M + bt - 1) / bt) * ((N + PF_BF - 1) / PF_BF); }
// Estimated device cycles of a plan, from timings of the 2560/6912-wide projections at 2048 tokens:
// a k slice costs about 700 cycles at 192 tokens per tile and only 27 % of that scales with the
// tile's tokens; finishing a split tile costs about as much as 35 slices, so splitting pays only
// when whole tiles would leave most of a wave idle.
static double pf_plan_cost(size_t M, size_t K, size_t N, int bt, bool whole, size_t sms)
{
    const double k = (double)(K / PF_BK), tiles = (double)pf_tiles(M, N, bt);
    const double per_slice = 700.0 * (0.73 + 0.27 * bt / (double)PF_BT);
    const double epilogue = 900.0 * (bt / 32);
    if (tiles <= (double)sms) return k * per_slice + epilogue;
    if (whole) return (double)((size_t)((tiles + sms - 1) / sms)) * k * per_slice + epilogue;
    return tiles * k / (double)sms * per_slice + epilogue + 25000.0;
}
static PfPlan pf_plan(size_t M, size_t K, size_t N)
{
    const size_t sms = (size_t)device_sm_count();
    static const int env_bt = getenv("BITNET_PREFILL_BT") ? atoi(getenv("BITNET_PREFILL_BT")) : 0;
    static const int env_mode = getenv("BITNET_PREFILL_WHOLE") ? atoi(getenv("BITNET_PREFILL_WHOLE")) : -1;
    PfPlan best = {};
    double best_cost = 0.0;
    for (int bt = PF_BT; bt >= 64; bt -= 32) {
        if (env_bt >= 32 && env_bt <= PF_BT && env_bt % 32 == 0 && bt != env_bt) continue;
        for (int whole = 1; whole >= 0; --whole) {
            if (env_mode >= 0 && whole != (env_mode != 0)) continue;
            const double cost = pf_plan_cost(M, K, N, bt, whole != 0, sms);
            if (best.bt == 0 || cost < best_cost) {
                best.bt = bt;
                best.whole_tiles = whole != 0;
                best_cost = cost;
            }
        }
    }
    if (best.bt == 0) { best.bt = PF_BT; best.whole_tiles = false; }
    best.tiles = pf_tiles(M, N, best.bt);
    const size_t units = best.tiles * (K / PF_BK);
    if (best.tiles <= sms) { best.grid = best.tiles; best.whole_tiles = true; }
    else best.grid = best.whole_tiles ? sms : (units < sms ? units : sms);
    return best;
}
static size_t pf_counter_bytes(size_t M, size_t N) { return align_up(pf_tiles(M, N, 64) * 8, 256); }   // claimed, published (largest tile count)

size_t prefill_workspace_bytes(size_t M, size_t K, size_t N)
{
    // int8 activations, fp32 scales, int32 row sums, tile counters, two partial tiles per CTA
    (void)K;
    return pf_q_bytes(M, K) + 2 * pf_vec_bytes(M) + pf_counter_bytes(M, N) + 2 * (size_t)device_sm_count() * PF_SLOT_BYTES;
}

static bitnet_status_t encode_map(CUtensorMap *map, const void *base, uint64_t inner, uint64_t rows, uint64_t row_stride_bytes,
                                  uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swizzle,
                                  CUtensorMapDataType dtype = CU_TENSOR_MAP_DATA_TYPE_UINT8)
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
    const CUresult r = encode(map, dtype, 2, const_cast<void *>(base), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(BITNET_ERR_CUDA_DRIVER, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return BITNET_OK;
}

// The same encoder for the other tensor-core kernel of the library (uint8 elements).
bitnet_status_t tensor_map_2d(void *map_out, const void *base, uint64_t inner, uint64_t rows, uint64_t row_stride_bytes,
                              uint32_t box_inner, uint32_t box_rows, int swizzle_128b)
{
    return encode_map(static_cast<CUtensorMap *>(map_out), base, inner, rows, row_stride_bytes, box_inner, box_rows,
                      swizzle_128b ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE);
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
    ws += pf_q_bytes(a.M, a.K);
    float *a_scale = reinterpret_cast<float *>(ws);
    ws += pf_vec_bytes(a.M);
    int *rowsum = reinterpret_cast<int *>(ws);
    ws += pf_vec_bytes(a.M);
    unsigned *counters = reinterpret_cast<unsigned *>(ws);
    ws += pf_counter_bytes(a.M, a.N);
    int *slots = reinterpret_cast<int *>(ws);

    const PfPlan plan = pf_plan(a.M, a.K, a.N);
    const int tiles = (int)plan.tiles;
    {
        cudaLaunchConfig_t qcfg = {};
        cudaLaunchAttribute qattr[1];
        const bool short_rows = a.K / 16 <= 256;
        qcfg.gridDim = dim3((unsigned)a.M);
        qcfg.blockDim = dim3(short_rows ? 128 : 256);
        qcfg.stream = stream;
        qcfg.attrs = qattr;
        if (a.flags & BITNET_FLAG_PDL) {   // the caller chains launches: start while the previous kernel drains
            qattr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            qattr[0].val.programmaticStreamSerializationAllowed = 1;
            qcfg.numAttrs = 1;
        }
        const int n_counters = 2 * tiles;
        if (short_rows)
            BITNET_CUDA(cudaLaunchKernelEx(&qcfg, quantize_rows_perm_kernel<128>, a.x, a.K, q_perm, a_scale, rowsum, a.q_out,
                                           a.a_scale_out, counters, n_counters));
        else
            BITNET_CUDA(cudaLaunchKernelEx(&qcfg, quantize_rows_perm_kernel<256>, a.x, a.K, q_perm, a_scale, rowsum, a.q_out,
                                           a.a_scale_out, counters, n_counters));
    }
    BITNET_TRY(check_launch("quantize_rows_perm_kernel"));

    CUtensorMap map_x, map_w, map_y;
    BITNET_TRY(encode_map(&map_x, q_perm, a.K, a.M, a.K, PF_BK, (uint32_t)plan.bt, CU_TENSOR_MAP_SWIZZLE_128B));
    BITNET_TRY(encode_map(&map_w, a.wp, a.K / 4, a.N, a.K / 4, PF_BK / 4, PF_BF, CU_TENSOR_MAP_SWIZZLE_NONE));

    PrefillParams p = {};
    p.y = a.y; p.acc_out = a.acc_out; p.a_scale = a_scale; p.rowsum = rowsum; p.w_scale = a.w_scale;
    p.slots = slots; p.counters = counters;
    p.M = (int)a.M; p.K = (int)a.K; p.N = (int)a.N; p.ldy = a.ldy ? a.ldy : a.N;
    p.bt = plan.bt;
    p.whole_tiles = plan.whole_tiles ? 1 : 0;
    p.m_tiles = (int)((a.M + plan.bt - 1) / plan.bt);
    p.n_tiles = (int)((a.N + PF_BF - 1) / PF_BF);
    p.k_tiles = (int)(a.K / PF_BK);
    // y leaves through TMA when its rows are 16-byte aligned; any other output takes plain stores
    p.tma_store = ((reinterpret_cast<uintptr_t>(a.y) & 15) == 0 && (p.ldy % 4) == 0) ? 1 : 0;
    p.n_peers = a.n_peers;
    for (int r = 0; r < a.n_peers && r < 8; ++r) p.y_peers[r] = a.y_peers[r];
    if (a.n_peers) {
        if (a.acc_out) return fail(BITNET_ERR_INVALID_CONFIG, "peer outputs and acc_out exclude each other");
        p.tma_store = 0;   // peer memory takes plain stores
    }
    if (p.tma_store)
        BITNET_TRY(encode_map(&map_y, a.y, a.N, a.M, p.ldy * 4, 32, 32, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_DATA_TYPE_FLOAT32));
    else
        map_y = map_w;   // unused by the kernel

    {   // once per device, under a lock: host threads launch concurrently (one per stream)
        static std::mutex mu;
        static bool attr_set[64] = {false};
        int dev = 0;
        BITNET_CUDA(cudaGetDevice(&dev));
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64 || !attr_set[dev]) {
            BITNET_CUDA(cudaFuncSetAttribute(prefill_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PF_SMEM));
            if (dev >= 0 && dev < 64) attr_set[dev] = true;
        }
    }
    const int grid = (int)plan.grid;
    // programmatic dependent launch: the GEMM's prologue and weight fetch overlap the quantiser's tail
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(PF_THREADS);
    cfg.dynamicSmemBytes = PF_SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    BITNET_CUDA(cudaLaunchKernelEx(&cfg, prefill_gemm_kernel, map_x, map_w, map_y, p));
    return check_launch("prefill_gemm_kernel");
}

}  // namespace bitnet
