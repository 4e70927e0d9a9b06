// BitLinear for a few dozen tokens (17 <= M <= 128): too many for the weight-streaming decode kernel's
// register tiles, too few to fill the persistent tensor-core GEMM's 128 x 192 tiles.  The op is still
// bound by the packed weights it has to read once, so the aim is to have every SM pulling weights at once
// and to finish in a handful of microseconds:
//
//   - an output tile is 128 features (tensor-memory lanes) x all tokens (columns, padded to 16);
//   - a CLUSTER of C CTAs owns a tile and splits K between them, so that tiles x C covers the SMs even
//     for a layer with twenty tiles; a gate/up pair is one cluster of 2 x C CTAs, half on each matrix;
//   - each CTA is one shot, no rings: it requests ALL of its operands at once by TMA (packed weights 128
//     rows x 32 bytes per 128-wide k slice; int8 activations tokens x 128 bytes, 128-byte swizzle), four
//     warps expand packed weights to u8 codes straight into tensor memory (the MMA's A operand) slice by
//     slice as they land, one thread issues tcgen05.mma kind::i8 (u8 x s8 -> s32, B from shared memory);
//   - the K-partial accumulators meet through DISTRIBUTED SHARED MEMORY: every CTA leaves its int32 tile
//     in its own shared memory, the cluster synchronises, and each CTA finishes a slice of the tokens by
//     reading all partials with ld.shared::cluster -- integer sums, exact in any order -- then subtracts the
//     row sum (code = w + 1), scales and stores y (or up * relu(gate)^2 for the pair).
//
// Every mbarrier wait is bounded; a wait that runs out raises an error flag, the CTA skips its work but
// still meets the cluster's barriers and frees its tensor memory.
//
// Semantics: TernaryProcessor::quantize_activations + ternary_matmul_generic
// (bitnet-inference/src/engine/ternary_operations.rs:117-172, :283-338) with int32 accumulation on the packed
// layout of BitPacked2BitPacker (bitnet-quant/src/quantization/packing.rs:352-394); the pair form is the first
// half of FeedForwardNetwork::forward (transformer_layers.rs:603-618).
#include <cuda.h>
#include <mutex>

#include "common.cuh"

namespace bitnet {

__device__ unsigned g_midm_error_flags;   // bit 2: a bounded wait of this kernel ran out

constexpr int MM_BF = 128;                 // features per tile
constexpr int MM_BK = 128;                 // k per slice
constexpr int MM_MAX_SLICES = 12;          // k slices one CTA can hold (tensor memory: 32 columns each, plus the accumulator)
constexpr int MM_THREADS = 192;            // warp 0: TMA + tensor-memory allocation, warp 1: MMA, warps 2-5: expand, epilogue
constexpr int MM_WP_BYTES = MM_BF * MM_BK / 4;   // 4 KB of packed weights per slice
constexpr unsigned MM_WAIT_LIMIT = 1u << 20;

struct MidParams {
    float *y;
    int32_t *acc_out;
    const float *a_scale;
    const int *rowsum;
    float w_scale, w_scale2;       // pair: gate scale, up scale
    int seg_end0, seg_end1;        // stacked matrices: features below seg_end0 use w_scale, below seg_end1 seg_scale1, the rest seg_scale2
    float seg_scale1, seg_scale2;
    int M, K, N;
    size_t ldy;
    int mt;                        // token columns of the tile: M rounded up to 16
    int k_slices;                  // K / 128
    int ck;                        // CTAs that split K for one matrix
    int pair;                      // 1: cluster = 2 * ck CTAs, ranks >= ck work on the second matrix
    int tmem_cols;
    int a_slots;                   // 32-column slots of expanded weights in tensor memory; slice s uses slot s % a_slots
    int w_slots;                   // 4 KB slots of packed weights in shared memory; slice s uses slot s % w_slots
    unsigned x_bytes;              // shared memory reserved for the activation slices / the partial tile
};

__device__ __forceinline__ unsigned mm_smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mm_mbar_init(unsigned long long *bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mm_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mm_mbar_arrive(unsigned long long *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mm_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mm_mbar_expect_tx(unsigned long long *bar, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mm_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mm_mbar_wait(unsigned long long *bar, unsigned parity)
{
    const unsigned addr = mm_smem_u32(bar);
    for (unsigned n = 0; n < MM_WAIT_LIMIT; ++n) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if (n > 8) __nanosleep(n < 64 ? 32 : 128);
    }
    atomicOr(&g_midm_error_flags, 4u);
    return false;
}
__device__ __forceinline__ bool mm_warp_wait(unsigned long long *bar, unsigned parity)
{
    unsigned ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mm_mbar_wait(bar, parity) ? 1u : 0u;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ void mm_tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, unsigned long long *bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            mm_smem_u32(dst)),
        "l"(map), "r"(mm_smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
// K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ unsigned long long mm_smem_desc(unsigned smem_addr)
{
    return (unsigned long long)((smem_addr >> 4) & 0x3fffu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// D = s32, A = u8 codes (tensor memory), B = s8 activations (K-major), N = token columns, M = 128
__device__ __forceinline__ unsigned mm_idesc(int mt) { return (2u << 4) | (0u << 7) | (1u << 10) | ((unsigned)(mt >> 3) << 17) | ((unsigned)(MM_BF >> 4) << 24); }
__device__ __forceinline__ void mm_mma_i8_ts(unsigned tmem_d, unsigned tmem_a, unsigned long long b_desc, unsigned idesc, unsigned accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
        "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mm_commit(unsigned long long *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mm_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mm_tmem_st32(unsigned taddr, const unsigned (&r)[32])
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
__device__ __forceinline__ void mm_tmem_ld16(unsigned taddr, unsigned (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ unsigned mm_cluster_rank()
{
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void mm_cluster_sync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// a shared-memory address of this CTA, as seen in CTA `rank` of the cluster
__device__ __forceinline__ unsigned mm_map_to_rank(unsigned local_addr, unsigned rank)
{
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ int mm_ld_cluster(unsigned addr)
{
    int v;
    asm volatile("ld.shared::cluster.b32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}

__global__ void __launch_bounds__(MM_THREADS, 1)
midm_gemm_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_w2, const MidParams p)
{
    extern __shared__ unsigned char mm_smem_raw[];
    __shared__ __align__(8) unsigned long long s_full_w[MM_MAX_SLICES], s_full_x[MM_MAX_SLICES], s_a_ready[MM_MAX_SLICES];
    __shared__ __align__(8) unsigned long long s_a_free[MM_MAX_SLICES];   // the MMAs of a slice have read its tensor-memory slot
    __shared__ __align__(8) unsigned long long s_w_free[MM_MAX_SLICES];   // the expanders hold a slice's packed words in registers
    __shared__ __align__(8) unsigned long long s_acc_full;
    __shared__ unsigned s_tmem_base;
    __shared__ unsigned s_failed;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(mm_smem_raw) + 1023) & ~uintptr_t(1023));

    const unsigned csize = (unsigned)(p.pair ? 2 * p.ck : p.ck);
    const unsigned rank = mm_cluster_rank();
    const int tile = (int)(blockIdx.x / csize);
    const int matrix = p.pair ? (int)(rank / (unsigned)p.ck) : 0;
    const int krank = (int)(rank % (unsigned)p.ck);
    const int s0 = krank * p.k_slices / p.ck, s1 = (krank + 1) * p.k_slices / p.ck;
    const int ns = s1 - s0;                                  // k slices of this CTA (<= MM_MAX_SLICES)
    const unsigned x_slice_bytes = (unsigned)p.mt * MM_BK;
    unsigned char *x_base = smem;                            // [ns][mt rows][128 B], later the partial tile [tokens][128] int32
    unsigned char *w_base = smem + p.x_bytes;                // [ns][128 rows][32 B]

    if (tid == 0) {
        for (int s = 0; s < MM_MAX_SLICES; ++s) {
            mm_mbar_init(&s_full_w[s], 1);
            mm_mbar_init(&s_full_x[s], 1);
            mm_mbar_init(&s_a_ready[s], 4);
            mm_mbar_init(&s_a_free[s], 1);
            mm_mbar_init(&s_w_free[s], 4);
        }
        mm_mbar_init(&s_acc_full, 1);
        s_failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(mm_smem_u32(&s_tmem_base)), "r"(p.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = s_tmem_base;
    const unsigned a_col0 = (unsigned)p.mt;                  // accumulator in columns [0, mt), expanded weights after it

    if (warp == 0) {
        // ===================== TMA: everything this CTA needs, requested at once =====================
        if (lane == 0) {
            const CUtensorMap *mw = matrix ? &map_w2 : &map_w;
            const int first = ns < p.w_slots ? ns : p.w_slots;
            for (int s = 0; s < first; ++s) {   // weights do not depend on the kernel in front of this one
                mm_mbar_expect_tx(&s_full_w[s], MM_WP_BYTES);
                mm_tma_load_2d(w_base + (size_t)s * MM_WP_BYTES, mw, (s0 + s) * (MM_BK / 4), tile * MM_BF, &s_full_w[s]);
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");   // the int8 activations come from the quantiser launch
            for (int s = 0; s < ns; ++s) {
                mm_mbar_expect_tx(&s_full_x[s], x_slice_bytes);
                mm_tma_load_2d(x_base + (size_t)s * x_slice_bytes, &map_x, (s0 + s) * MM_BK, 0, &s_full_x[s]);
            }
            for (int s = first; s < ns; ++s) {  // the later slices reuse a slot once the expanders have taken its words
                if (!mm_mbar_wait(&s_w_free[s - p.w_slots], 0)) { s_failed = 1; break; }
                mm_mbar_expect_tx(&s_full_w[s], MM_WP_BYTES);
                mm_tma_load_2d(w_base + (size_t)(s % p.w_slots) * MM_WP_BYTES, mw, (s0 + s) * (MM_BK / 4), tile * MM_BF, &s_full_w[s]);
            }
        }
    } else if (warp == 1) {
        // ===================== MMA issuer =====================
        if (lane == 0) {
            const unsigned idesc = mm_idesc(p.mt);
            bool ok = true;
            for (int s = 0; s < ns && ok; ++s) {
                ok = mm_mbar_wait(&s_a_ready[s], 0) && mm_mbar_wait(&s_full_x[s], 0);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned tmem_a = tmem_base + a_col0 + (unsigned)(s % p.a_slots) * (MM_BK / 4);
                const unsigned long long b_desc = mm_smem_desc(mm_smem_u32(x_base + (size_t)s * x_slice_bytes));
#pragma unroll
                for (int ks = 0; ks < MM_BK / 32; ++ks)
                    mm_mma_i8_ts(tmem_base, tmem_a + 8u * ks, b_desc + 2ull * ks, idesc, (s != 0 || ks != 0) ? 1u : 0u);
                if (s + p.a_slots < ns) mm_commit(&s_a_free[s]);   // a later slice waits for this slot
            }
            if (ok) mm_commit(&s_acc_full);
            else s_failed = 1;
        }
    } else {
        // ===================== expanders, then epilogue: a thread owns one feature row =====================
        const int quarter = warp & 3;                        // the tensor-memory lanes this warp may touch
        const int row = quarter * 32 + lane;
        bool ok = true;
        for (int s = 0; s < ns && ok; ++s) {
            if (!mm_warp_wait(&s_full_w[s], 0)) { ok = false; break; }
            const uint4 *src = reinterpret_cast<const uint4 *>(w_base + (size_t)(s % p.w_slots) * MM_WP_BYTES + row * (MM_BK / 4));
            const uint4 w0 = src[0], w1 = src[1];
            const unsigned w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
            unsigned r[32];
#pragma unroll
            for (int g = 0; g < 8; ++g) {   // (w >> 2j) & 0x03030303 is word j of a 16-wide group in the activations' transposed order
                r[4 * g + 0] = w[g] & 0x03030303u;
                r[4 * g + 1] = (w[g] >> 2) & 0x03030303u;
                r[4 * g + 2] = (w[g] >> 4) & 0x03030303u;
                r[4 * g + 3] = (w[g] >> 6) & 0x03030303u;
            }
            if (s + p.w_slots < ns) {       // a later slice lands in this shared-memory slot
                __syncwarp();
                if (lane == 0) mm_mbar_arrive(&s_w_free[s]);
            }
            if (s >= p.a_slots) {   // the slot still feeds the MMAs of slice s - a_slots
                if (!mm_warp_wait(&s_a_free[s - p.a_slots], 0)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            mm_tmem_st32(tmem_base + ((unsigned)(quarter * 32) << 16) + a_col0 + (unsigned)(s % p.a_slots) * (MM_BK / 4), r);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mm_mbar_arrive(&s_a_ready[s]);
        }
        // the accumulator: this CTA's K-partial sums, left in its own shared memory as [token][feature]
        if (ok) ok = mm_warp_wait(&s_acc_full, 0);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            int *part = reinterpret_cast<int *>(x_base);     // the activation slices are consumed: the MMAs have completed
            for (int c = 0; c < p.mt; c += 16) {
                unsigned r[16];
                mm_tmem_ld16(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)c, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (c + j < p.M) part[(c + j) * MM_BF + row] = (int)r[j];
            }
        }
        if (!ok) s_failed = 1;
    }

    // ---- the partial tiles of the cluster meet ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    mm_cluster_sync();   // every CTA's partial tile is in its shared memory (or its failure flag is up)

    if (warp >= 2) {
        asm volatile("griddepcontrol.wait;" ::: "memory");   // row sums and scales come from the quantiser launch
        // any CTA of the cluster that gave up spoils the tile: nobody writes it
        bool bad = false;
        const unsigned flag_local = mm_smem_u32(&s_failed);
        for (unsigned c = 0; c < csize; ++c) bad = bad || mm_ld_cluster(mm_map_to_rank(flag_local, c)) != 0;
        if (!bad) {
            // This CTA finishes tokens [t0, t1) of the tile: a thread takes four consecutive features of one token
            // per pass (the 128 threads cover four token rows), reads that 16-byte piece from every CTA's partial
            // tile -- all reads of two passes are issued before the first sum, a remote read costs a round trip
            // through the cluster network -- and writes 16 bytes of y.
            const int e = tid - 64;                          // 0..127
            const int fq = (e & 31) * 4, tr = e >> 5;
            const int n = tile * MM_BF + fq;
            const int t0 = (int)((long long)rank * p.M / csize), t1 = (int)((long long)(rank + 1) * p.M / csize);
            const unsigned part_local = mm_smem_u32(x_base);
            unsigned remote[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) remote[c] = mm_map_to_rank(part_local, (unsigned)c < csize ? (unsigned)c : 0u);
            float ws4[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) ws4[i] = n + i < p.seg_end0 ? p.w_scale : (n + i < p.seg_end1 ? p.seg_scale1 : p.seg_scale2);
            const bool vec_ok = (reinterpret_cast<uintptr_t>(p.y) & 15) == 0 && (p.ldy & 3) == 0 && n + 3 < p.N;
            constexpr int U = 2;
            for (int tb = t0; tb < t1; tb += 4 * U) {
                int4 v[U][8];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int t = tb + u * 4 + tr;
                    const unsigned off = (unsigned)(t * MM_BF + fq) * 4u;
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        v[u][c] = make_int4(0, 0, 0, 0);
                        if ((unsigned)c < csize && t < t1)
                            asm volatile("ld.shared::cluster.v4.b32 {%0, %1, %2, %3}, [%4];"
                                         : "=r"(v[u][c].x), "=r"(v[u][c].y), "=r"(v[u][c].z), "=r"(v[u][c].w)
                                         : "r"(remote[c] + off));
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int t = tb + u * 4 + tr;
                    if (t >= t1) continue;
                    int s0v[4] = {0, 0, 0, 0}, s1v[4] = {0, 0, 0, 0};
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        if (p.pair && c >= p.ck) { s1v[0] += v[u][c].x; s1v[1] += v[u][c].y; s1v[2] += v[u][c].z; s1v[3] += v[u][c].w; }
                        else { s0v[0] += v[u][c].x; s0v[1] += v[u][c].y; s0v[2] += v[u][c].z; s0v[3] += v[u][c].w; }
                    }
                    const int rs = __ldcg(p.rowsum + t);
                    const float a = __ldcg(p.a_scale + t);
                    float out[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (p.pair) {
                            const float gate = __fmul_rn((float)(s0v[i] - rs), __fmul_rn(p.w_scale, a));
                            const float up = __fmul_rn((float)(s1v[i] - rs), __fmul_rn(p.w_scale2, a));
                            const float rl = fmaxf(gate, 0.0f);
                            out[i] = __fmul_rn(up, __fmul_rn(rl, rl));
                        } else {
                            out[i] = __fmul_rn((float)(s0v[i] - rs), __fmul_rn(ws4[i], a));
                        }
                    }
                    const size_t o = (size_t)t * p.ldy + n;
                    if (vec_ok) {
                        *reinterpret_cast<float4 *>(p.y + o) = make_float4(out[0], out[1], out[2], out[3]);
                        if (p.acc_out && !p.pair) *reinterpret_cast<int4 *>(p.acc_out + o) = make_int4(s0v[0] - rs, s0v[1] - rs, s0v[2] - rs, s0v[3] - rs);
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            if (n + i < p.N) {
                                p.y[o + i] = out[i];
                                if (p.acc_out && !p.pair) p.acc_out[o + i] = s0v[i] - rs;
                            }
                    }
                }
            }
        }
    }
    mm_cluster_sync();   // nobody leaves while its shared memory may still be read
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols) : "memory");
    }
}

bitnet_status_t midm_take_error_flags(unsigned *flags)
{
    unsigned v = 0, zero = 0;
    BITNET_CUDA(cudaMemcpyFromSymbol(&v, g_midm_error_flags, sizeof(v)));
    if (v) BITNET_CUDA(cudaMemcpyToSymbol(g_midm_error_flags, &zero, sizeof(zero)));
    *flags = v;
    return BITNET_OK;
}

// ---- host side --------------------------------------------------------------------------------------

bool midm_supports(size_t M, size_t K, size_t N)
{
    return M >= 1 && M <= 128 && N >= 1 && N <= (1u << 24) && K >= 128 && K % 128 == 0 && K <= 16384;
}

struct MidPlan {
    int mt, ck, tmem_cols, a_slots, w_slots;
    size_t x_bytes, smem;
    size_t tiles, ctas;
};

// K split per matrix: enough CTAs for every SM, few enough k slices per CTA for tensor memory and
// shared memory, at most 8 CTAs per cluster; the estimate counts waves x (a fixed part + slices).
static bool midm_plan(size_t M, size_t K, size_t N, bool pair, MidPlan *out)
{
    const int mt = (int)((M + 15) / 16 * 16);
    const int S = (int)(K / MM_BK);
    const size_t tiles = (N + MM_BF - 1) / MM_BF;
    const int sms = device_sm_count();
    const int max_ck = pair ? 4 : 8;
    double best = 0.0;
    bool found = false;
    for (int ck = 1; ck <= max_ck && ck <= S; ++ck) {
        const int ns = (S + ck - 1) / ck;
        if (ns > MM_MAX_SLICES) continue;
        // tensor memory: the accumulator, then 32-column slots of expanded weights; all slices of the CTA when
        // they fit 256 columns, else as many slots as do and later slices reuse them once their MMAs are through
        const int slots_256 = (256 - mt) / 32;
        const int a_slots = ns <= slots_256 ? ns : slots_256;
        if (a_slots < 2 && ns > a_slots) continue;
        const int cols = 256;
        const size_t part = (size_t)mt * MM_BF * 4;
        size_t xb = (size_t)ns * mt * MM_BK;
        if (xb < part) xb = part;
        xb = align_up(xb, 1024);
        // packed weights: a slot per slice, or fewer (at least four, reused in turn) when that lets two CTAs share an SM
        int w_slots = ns;
        const size_t two_per_sm = 110 * 1024;
        if (xb + (size_t)ns * MM_WP_BYTES + 1024 > two_per_sm && ns > 4 && xb + 4 * (size_t)MM_WP_BYTES + 1024 <= two_per_sm)
            w_slots = (int)((two_per_sm - 1024 - xb) / MM_WP_BYTES);
        size_t smem = xb + (size_t)w_slots * MM_WP_BYTES + 1024;
        if (smem > 220 * 1024) continue;
        // Shared memory is also what keeps tensor memory from being oversubscribed, so that no CTA ever waits
        // inside tcgen05.alloc for a CTA of another cluster (which could be waiting for this cluster in turn):
        // every CTA takes 256 of the 512 columns and asks for at least 77 KB of shared memory, so at most two
        // of them fit an SM (and none beside a CTA of the persistent GEMM, which fills an SM's shared memory).
        const size_t floor_bytes = 77 * 1024;
        if (smem < floor_bytes) smem = floor_bytes;
        const int per_sm = smem <= two_per_sm ? 2 : 1;
        const size_t ctas = tiles * (size_t)ck * (pair ? 2 : 1);
        const double waves = (double)((ctas + (size_t)sms * per_sm - 1) / ((size_t)sms * per_sm));
        const double cost = waves * (6.0 + ns) + 0.8 * ck;   // a wider cluster has more partial tiles to sum: measured, about 0.8 of a slice each
        if (!found || cost < best) {
            found = true;
            best = cost;
            out->mt = mt; out->ck = ck; out->tmem_cols = cols; out->a_slots = a_slots; out->w_slots = w_slots; out->x_bytes = xb; out->smem = smem; out->tiles = tiles; out->ctas = ctas;
        }
    }
    return found;
}

size_t midm_workspace_bytes(size_t M, size_t K)
{
    return align_up(M * K, 256) + 2 * align_up(M * 4, 256);   // int8 rows, row sums, scales
}

bool midm_can_run(size_t M, size_t K, size_t N, bool pair)
{
    MidPlan pl;
    return midm_supports(M, K, N) && midm_plan(M, K, N, pair, &pl);
}

bitnet_status_t tensor_map_2d(void *map_out, const void *base, uint64_t inner, uint64_t rows, uint64_t row_stride_bytes,
                              uint32_t box_inner, uint32_t box_rows, int swizzle_128b);

// a.wp2 != nullptr: gate/up pair (a.wp = gate), y receives up * relu(gate)^2.  ready = true: the workspace already
// holds this input's quantised rows (an earlier call with the same x wrote them).
bitnet_status_t launch_midm(const ForwardArgs &a, void *workspace, size_t workspace_bytes, bool ready, cudaStream_t stream)
{
    const bool pair = a.wp2 != nullptr;
    MidPlan pl;
    if (!midm_supports(a.M, a.K, a.N) || !midm_plan(a.M, a.K, a.N, pair, &pl))
        return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "cluster GEMM needs 1 <= M <= 128, K %% 128 == 0 and a K slice per CTA that fits shared and tensor memory (M=%zu K=%zu N=%zu)", a.M, a.K, a.N);
    if (workspace_bytes < midm_workspace_bytes(a.M, a.K) || (reinterpret_cast<uintptr_t>(workspace) & 255))
        return fail(BITNET_ERR_WORKSPACE, "cluster GEMM needs %zu bytes of 256-byte aligned workspace", midm_workspace_bytes(a.M, a.K));
    if ((reinterpret_cast<uintptr_t>(a.wp) & 15) || (pair && (reinterpret_cast<uintptr_t>(a.wp2) & 15)))
        return fail(BITNET_ERR_INVALID_CONFIG, "packed weights must be 16-byte aligned");
    if (pair && a.n_seg) return fail(BITNET_ERR_INVALID_CONFIG, "stacked matrices and the gate/up pair do not combine");

    char *ws = static_cast<char *>(workspace);
    RowsOut rows;
    rows.q_perm = reinterpret_cast<int8_t *>(ws);
    rows.rowsum = reinterpret_cast<int *>(ws + align_up(a.M * a.K, 256));
    rows.a_scale = reinterpret_cast<float *>(ws + align_up(a.M * a.K, 256) + align_up(a.M * 4, 256));
    if (!ready) BITNET_TRY(launch_quantize_rows_glued(a.x, a.M, a.K, a.pre, rows, a.q_out, a.a_scale_out, a.flags, stream));

    CUtensorMap map_x, map_w, map_w2;
    BITNET_TRY(tensor_map_2d(&map_x, rows.q_perm, a.K, a.M, a.K, MM_BK, (uint32_t)pl.mt, 1));
    BITNET_TRY(tensor_map_2d(&map_w, a.wp, a.K / 4, a.N, a.K / 4, MM_BK / 4, MM_BF, 0));
    if (pair) BITNET_TRY(tensor_map_2d(&map_w2, a.wp2, a.K / 4, a.N, a.K / 4, MM_BK / 4, MM_BF, 0));
    else map_w2 = map_w;

    MidParams p = {};
    p.y = a.y; p.acc_out = a.acc_out; p.a_scale = rows.a_scale; p.rowsum = rows.rowsum;
    p.w_scale = a.w_scale; p.w_scale2 = a.w_scale2;
    p.seg_end0 = p.seg_end1 = 0x7fffffff;
    if (a.n_seg > 0) {
        p.seg_end0 = (int)a.seg_end[0]; p.seg_scale1 = a.seg_scale[0];
        if (a.n_seg > 1) { p.seg_end1 = (int)a.seg_end[1]; p.seg_scale2 = a.seg_scale[1]; }
    }
    p.M = (int)a.M; p.K = (int)a.K; p.N = (int)a.N; p.ldy = a.ldy ? a.ldy : a.N;
    p.mt = pl.mt; p.k_slices = (int)(a.K / MM_BK); p.ck = pl.ck; p.pair = pair ? 1 : 0; p.tmem_cols = pl.tmem_cols;
    p.a_slots = pl.a_slots;
    p.w_slots = pl.w_slots;
    p.x_bytes = (unsigned)pl.x_bytes;

    {   // once per device, under a lock: host threads launch concurrently
        static std::mutex mu;
        static bool attr_set[64] = {false};
        int dev = 0;
        BITNET_CUDA(cudaGetDevice(&dev));
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64 || !attr_set[dev]) {
            BITNET_CUDA(cudaFuncSetAttribute(midm_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
            if (dev >= 0 && dev < 64) attr_set[dev] = true;
        }
    }
    const unsigned csize = (unsigned)(pair ? 2 * pl.ck : pl.ck);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attrs[2];
    cfg.gridDim = dim3((unsigned)(pl.tiles * csize));
    cfg.blockDim = dim3(MM_THREADS);
    cfg.dynamicSmemBytes = pl.smem;
    cfg.stream = stream;
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = csize;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 2;   // the GEMM's prologue and weight requests overlap the quantiser's tail
    BITNET_CUDA(cudaLaunchKernelEx(&cfg, midm_gemm_kernel, map_x, map_w, map_w2, p));
    return check_launch("midm_gemm_kernel");
}

}  // namespace bitnet
