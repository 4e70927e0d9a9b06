// Decode-time BitLinear (M <= 16 tokens): a weight-streaming W2A8 GEMV for sm_100a.
//
// What one launch does
//   1. every lane issues its first 128-bit loads of packed weights (they do not depend
//      on the preceding kernel, so under programmatic dependent launch they overlap it);
//   2. the CTAs of a cluster quantise the activations together: each CTA folds |x| over
//      its own K slice, the partial maxima are exchanged through distributed shared
//      memory, and each CTA writes the int8 values of its slice to its shared memory in
//      the order the tensor-core fragments want;
//   3. packed weights go from global memory straight into mma fragments: masking a
//      32-bit word with 0x03030303 << 2j leaves code << 2j in each byte, which is fed to
//      the u8 x s8 tensor-core instruction unshifted; the four j classes accumulate
//      separately and are combined exactly as acc0 + acc1/4 + acc2/16 + acc3/64.
//      sum_k (code-1)*q = sum_k code*q - sum_k q, and sum_k q is known from step 2;
//   4. the K-split partial sums of a cluster meet in the shared memory of the CTA that
//      owns the 16-row block, which dequantises and writes y.
//
// The contraction is order-independent integer arithmetic, so the result is the exact
// int32 accumulator whatever the tiling.
//
// Semantics: TernaryProcessor::quantize_activations + ternary_matmul_generic
// (bitnet-inference/src/engine/ternary_operations.rs:117-172, :283-338) on the packed
// layout of BitPacked2BitPacker (bitnet-quant/src/quantization/packing.rs:352-394);
// replaces w2a8_gemv_kernel (bitnet-cuda/src/kernels/w2a8_gemv.cu:100-182).
#include <cooperative_groups.h>

#include <map>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace bitnet {

constexpr int DEC_WARPS = 8;
constexpr int DEC_THREADS = DEC_WARPS * 32;
constexpr int DEC_MAX_TOKENS = 16;

struct DecodeParams {
    const uint8_t *wp;
    const uint8_t *wp2;
    const float *x;
    const int8_t *x_i8;
    float *y;
    int32_t *acc_out;
    int8_t *q_out;
    float *a_scale_out;
    float w_scale, w_scale2;
    int M, K, N;
    size_t ldy;
    int chunks;    // K / 64: one chunk is the 16 bytes (64 weights) a lane loads at once
    int n_blocks;  // ceil(N / 16): 16-row blocks, one per warp per round
    int steps;     // loop steps per round: ceil(ceil(chunks / S) / 4)
};

__device__ __forceinline__ uint4 ldg_stream(const uint8_t *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_u8s8(int (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ unsigned word_of(const uint4 &v, int i)
{
    return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}

// Shared memory carve-up (dynamic):
//   act   : int8 activations of this CTA's K slice, fragment order, steps*4*NT*512 bytes
//   red   : K-split exchange buffers, 2 * DEC_WARPS * NTD * 512 bytes (S > 1 only)
// plus small static arrays below.
template <int NT, int S, bool IN_I8, bool DUAL>
__global__ void __launch_bounds__(DEC_THREADS, (NT == 1 && !DUAL) ? 2 : 1) decode_kernel(const DecodeParams p)
{
    constexpr int NW = DUAL ? 2 : 1;      // weight matrices streamed together
    constexpr int D = (NW * NT >= 2) ? 2 : 4;  // loop steps of weights in flight per lane
    constexpr int NTD = NT * NW;

    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ unsigned s_key[DEC_MAX_TOKENS];       // absmax of this CTA's slice, as ordered keys
    __shared__ int s_sumq[DEC_MAX_TOKENS];           // sum of int8 activations over this CTA's slice
    __shared__ float s_ascale[DEC_MAX_TOKENS];       // absmax/127 per token
    __shared__ float s_qscale[DEC_MAX_TOKENS];       // 127/absmax per token

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tig = lane & 3;

    int rank = 0;
    if constexpr (S > 1) rank = (int)cg::this_cluster().block_rank();
    const int cluster_id = blockIdx.x / S;
    const int n_clusters = gridDim.x / S;

    const int cb = (int)((long long)rank * p.chunks / S);
    const int ce = (int)((long long)(rank + 1) * p.chunks / S);
    const int Cs = ce - cb;
    const int steps = p.steps;
    const int blk_begin = (int)((long long)cluster_id * p.n_blocks / n_clusters);
    const int blk_end = (int)((long long)(cluster_id + 1) * p.n_blocks / n_clusters);
    const int rounds = (blk_end - blk_begin + DEC_WARPS - 1) / DEC_WARPS;
    const int total = rounds * steps;
    const size_t row_bytes = (size_t)p.K / 4;

    unsigned char *s_act = smem;
    uint4 *s_red = reinterpret_cast<uint4 *>(smem + (size_t)steps * 4 * NT * 512);

    // ---- weight pipeline -----------------------------------------------------------
    uint4 wa[NW][D], wb[NW][D];   // rows g and g+8 of this warp's block, per matrix
    int l_round = 0, l_step = 0;  // position of the next load
    auto issue = [&](int d) {
        const int blk = blk_begin + l_round * DEC_WARPS + warp;
        const int ci = l_step * 4 + tig;
        const bool ok = blk < blk_end && ci < Cs;
        const int ra = blk * 16 + g, rb = ra + 8;
        const size_t col = (size_t)(cb + ci) * 16;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const uint8_t *base = w == 0 ? p.wp : p.wp2;
            wa[w][d] = (ok && ra < p.N) ? ldg_stream(base + (size_t)ra * row_bytes + col) : make_uint4(0, 0, 0, 0);
            wb[w][d] = (ok && rb < p.N) ? ldg_stream(base + (size_t)rb * row_bytes + col) : make_uint4(0, 0, 0, 0);
        }
        if (++l_step == steps) { l_step = 0; ++l_round; }
    };
#pragma unroll
    for (int d = 0; d < D; ++d) {
        if (d < total) issue(d);
        else {
#pragma unroll
            for (int w = 0; w < NW; ++w) wa[w][d] = wb[w][d] = make_uint4(0, 0, 0, 0);
        }
    }

    // Let the next kernel on the stream start its own weight fetch, then wait for the
    // kernel that produced our activations.  Both are no-ops without the launch attribute.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- activation quantisation, shared by the cluster ---------------------------------
    if (tid < DEC_MAX_TOKENS) { s_key[tid] = 0; s_sumq[tid] = 0; }
    __syncthreads();

    const unsigned groups_per_token = (unsigned)Cs * 4;   // 16-wide k groups in the slice
    const unsigned n_groups = (unsigned)p.M * groups_per_token;

    if constexpr (!IN_I8) {
        for (unsigned gid0 = 0; gid0 < n_groups; gid0 += DEC_THREADS) {
            const unsigned gid = gid0 + tid;
            unsigned key = 0, m = 0;
            if (gid < n_groups) {
                m = gid / groups_per_token;
                const unsigned l = gid - m * groups_per_token;
                const float4 *src = reinterpret_cast<const float4 *>(p.x + (size_t)m * p.K + (size_t)cb * 64 + (size_t)l * 16);
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    const float4 f = __ldg(src + v);
                    key = max(max(key, abs_key(f.x)), max(abs_key(f.y), max(abs_key(f.z), abs_key(f.w))));
                }
            }
            // a warp's 32 groups usually belong to one or two tokens: fold those in registers
            const unsigned m_lo = __shfl_sync(0xffffffffu, m, 0);
            const unsigned k_lo = __reduce_max_sync(0xffffffffu, m == m_lo ? key : 0u);
            const unsigned k_hi = __reduce_max_sync(0xffffffffu, m == m_lo + 1 ? key : 0u);
            if (lane == 0) {
                if (k_lo) atomicMax(&s_key[m_lo], k_lo);
                if (k_hi) atomicMax(&s_key[m_lo + 1], k_hi);
            }
            if (m > m_lo + 1 && key) atomicMax(&s_key[m], key);
        }
        __syncthreads();
        unsigned key = 0;
        if constexpr (S > 1) {
            cg::cluster_group cluster = cg::this_cluster();
            cluster.sync();   // every CTA of the cluster is running and has published its partial keys
            if (tid < p.M) {
#pragma unroll
                for (int r = 0; r < S; ++r) key = max(key, *cluster.map_shared_rank(&s_key[tid], r));
            }
        } else {
            if (tid < p.M) key = s_key[tid];
        }
        if (tid < p.M) {
            const float absmax = __uint_as_float(key);
            s_ascale[tid] = dequant_scale(absmax);
            s_qscale[tid] = quant_scale(absmax);
            if (p.a_scale_out && blockIdx.x == 0) p.a_scale_out[tid] = dequant_scale(absmax);
        }
        __syncthreads();
    } else {
        if constexpr (S > 1) cg::this_cluster().sync();
        if (tid < p.M) s_ascale[tid] = 1.0f;
        __syncthreads();
    }

    // pass 2: quantise this slice into fragment order
    for (unsigned gid0 = 0; gid0 < n_groups; gid0 += DEC_THREADS) {
        const unsigned gid = gid0 + tid;
        unsigned m = 0;
        int sum = 0;
        if (gid < n_groups) {
            m = gid / groups_per_token;
            const unsigned l = gid - m * groups_per_token;   // 16-wide group inside the slice
            int q[16];
            if constexpr (IN_I8) {
                const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(p.x_i8 + (size_t)m * p.K + (size_t)cb * 64 + (size_t)l * 16));
#pragma unroll
                for (int e = 0; e < 16; ++e) q[e] = (int)(int8_t)((word_of(raw, e >> 2) >> (8 * (e & 3))) & 0xffu);
            } else {
                const float scale = s_qscale[m];
                const float4 *src = reinterpret_cast<const float4 *>(p.x + (size_t)m * p.K + (size_t)cb * 64 + (size_t)l * 16);
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    const float4 f = __ldg(src + v);
                    q[4 * v + 0] = quantize_one(f.x, scale);
                    q[4 * v + 1] = quantize_one(f.y, scale);
                    q[4 * v + 2] = quantize_one(f.z, scale);
                    q[4 * v + 3] = quantize_one(f.w, scale);
                }
                if (p.q_out && cluster_id == 0) {
                    uint4 canon;
                    canon.x = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((unsigned)(q[3] & 0xff) << 24);
                    canon.y = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((unsigned)(q[7] & 0xff) << 24);
                    canon.z = (q[8] & 0xff) | ((q[9] & 0xff) << 8) | ((q[10] & 0xff) << 16) | ((unsigned)(q[11] & 0xff) << 24);
                    canon.w = (q[12] & 0xff) | ((q[13] & 0xff) << 8) | ((q[14] & 0xff) << 16) | ((unsigned)(q[15] & 0xff) << 24);
                    *reinterpret_cast<uint4 *>(p.q_out + (size_t)m * p.K + (size_t)cb * 64 + (size_t)l * 16) = canon;
                }
            }
            // word j holds k = j, j+4, j+8, j+12 of the group: the bytes the mask
            // 0x03030303 << 2j selects from a packed weight word
            uint4 frag;
            frag.x = (q[0] & 0xff) | ((q[4] & 0xff) << 8) | ((q[8] & 0xff) << 16) | ((unsigned)(q[12] & 0xff) << 24);
            frag.y = (q[1] & 0xff) | ((q[5] & 0xff) << 8) | ((q[9] & 0xff) << 16) | ((unsigned)(q[13] & 0xff) << 24);
            frag.z = (q[2] & 0xff) | ((q[6] & 0xff) << 8) | ((q[10] & 0xff) << 16) | ((unsigned)(q[14] & 0xff) << 24);
            frag.w = (q[3] & 0xff) | ((q[7] & 0xff) << 8) | ((q[11] & 0xff) << 16) | ((unsigned)(q[15] & 0xff) << 24);
#pragma unroll
            for (int e = 0; e < 16; ++e) sum += q[e];
            // slice-relative chunk c = l/4 is read by lanes with tig = c%4 in step c/4;
            // i = l%4 is the 16-wide group inside the chunk; token m sits in tile m/8, row m%8
            const unsigned c = l >> 2, i = l & 3;
            const unsigned step = c >> 2, ctig = c & 3;
            const unsigned off = (((step * 4 + i) * NT + (m >> 3)) * 32 + (m & 7) * 4 + ctig) * 16;
            *reinterpret_cast<uint4 *>(s_act + off) = frag;
        }
        const unsigned m_lo = __shfl_sync(0xffffffffu, m, 0);
        const int s_lo = __reduce_add_sync(0xffffffffu, m == m_lo ? sum : 0);
        const int s_hi = __reduce_add_sync(0xffffffffu, m == m_lo + 1 ? sum : 0);
        if (lane == 0) {
            if (s_lo) atomicAdd(&s_sumq[m_lo], s_lo);
            if (s_hi) atomicAdd(&s_sumq[m_lo + 1], s_hi);
        }
        if (m > m_lo + 1 && sum) atomicAdd(&s_sumq[m], sum);
    }
    __syncthreads();

    // ---- main loop -------------------------------------------------------------------------
    int acc[NW][NT][4][4];   // [matrix][token tile][j class][fragment register]
    auto clear_acc = [&]() {
#pragma unroll
        for (int w = 0; w < NW; ++w)
#pragma unroll
            for (int t = 0; t < NT; ++t)
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int r = 0; r < 4; ++r) acc[w][t][j][r] = 0;
    };
    clear_acc();

    int c_round = 0, c_step = 0;   // position of the step being consumed
    for (int it0 = 0; it0 < total; it0 += D) {
#pragma unroll
        for (int d = 0; d < D; ++d) {
            if (it0 + d < total) {
                // B fragments: 16 bytes per (16-wide group, token tile), conflict-free
                uint4 bw[4][NT];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int t = 0; t < NT; ++t)
                        bw[i][t] = *reinterpret_cast<const uint4 *>(s_act + ((size_t)((c_step * 4 + i) * NT + t) * 32 + lane) * 16);
#pragma unroll
                for (int w = 0; w < NW; ++w) {
#pragma unroll
                    for (int pr = 0; pr < 2; ++pr) {
                        const unsigned a_lo0 = word_of(wa[w][d], 2 * pr), a_lo1 = word_of(wa[w][d], 2 * pr + 1);
                        const unsigned a_hi0 = word_of(wb[w][d], 2 * pr), a_hi1 = word_of(wb[w][d], 2 * pr + 1);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const unsigned mask = 0x03030303u << (2 * j);
#pragma unroll
                            for (int t = 0; t < NT; ++t)
                                mma_u8s8(acc[w][t][j], a_lo0 & mask, a_hi0 & mask, a_lo1 & mask, a_hi1 & mask,
                                         word_of(bw[2 * pr][t], j), word_of(bw[2 * pr + 1][t], j));
                        }
                    }
                }

                const bool tile_done = (c_step == steps - 1);
                const int blk = blk_begin + c_round * DEC_WARPS + warp;   // this warp's block in the round
                if (++c_step == steps) { c_step = 0; ++c_round; }

                // refill this slot before the (possibly long) tile epilogue
                if (it0 + d + D < total) issue(d);

                if (tile_done) {
                    // exact partial sums of sum_k (code-1)*q over this CTA's K slice
                    int part[NTD][4];
#pragma unroll
                    for (int w = 0; w < NW; ++w)
#pragma unroll
                        for (int t = 0; t < NT; ++t) {
                            const int sq0 = s_sumq[8 * t + 2 * tig], sq1 = s_sumq[8 * t + 2 * tig + 1];
#pragma unroll
                            for (int r = 0; r < 4; ++r) {
                                const int v = acc[w][t][0][r] + (acc[w][t][1][r] >> 2) + (acc[w][t][2][r] >> 4) +
                                              (acc[w][t][3][r] >> 6);
                                part[w * NT + t][r] = v - ((r & 1) ? sq1 : sq0);
                            }
                        }
                    clear_acc();

                    int fin_blk = blk;      // block this warp finalises
                    bool fin = true;
                    if constexpr (S > 1) {
                        cg::cluster_group cluster = cg::this_cluster();
                        const int buf = (c_round + 1) & 1;   // parity of the round just finished
                        // owner of warp w's block is rank w % S, slot w / S
                        uint4 *dst = cluster.map_shared_rank(s_red, warp % S) +
                                     ((((size_t)buf * S + rank) * (DEC_WARPS / S) + warp / S) * NTD) * 32 + lane;
#pragma unroll
                        for (int u = 0; u < NTD; ++u)
                            dst[u * 32] = make_uint4((unsigned)part[u][0], (unsigned)part[u][1], (unsigned)part[u][2], (unsigned)part[u][3]);
                        cluster.sync();
                        fin = warp < DEC_WARPS / S;
                        if (fin) {
                            const int src_warp = warp * S + rank;   // the warp index whose block we own
                            fin_blk = blk - warp + src_warp;
#pragma unroll
                            for (int u = 0; u < NTD; ++u)
#pragma unroll
                                for (int r = 0; r < 4; ++r) part[u][r] = 0;
#pragma unroll
                            for (int r2 = 0; r2 < S; ++r2) {
                                const uint4 *src = s_red + ((((size_t)buf * S + r2) * (DEC_WARPS / S) + warp) * NTD) * 32 + lane;
#pragma unroll
                                for (int u = 0; u < NTD; ++u) {
                                    const uint4 v = src[u * 32];
                                    part[u][0] += (int)v.x; part[u][1] += (int)v.y; part[u][2] += (int)v.z; part[u][3] += (int)v.w;
                                }
                            }
                        }
                    }

                    if (fin && fin_blk < blk_end) {
                        const int row_a = fin_blk * 16 + g, row_b = row_a + 8;
#pragma unroll
                        for (int t = 0; t < NT; ++t)
#pragma unroll
                            for (int r = 0; r < 4; ++r) {
                                const int m = 8 * t + 2 * tig + (r & 1);
                                const int row = (r & 2) ? row_b : row_a;
                                if (m < p.M && row < p.N) {
                                    const size_t o = (size_t)m * p.ldy + row;
                                    if constexpr (DUAL) {
                                        const float a = s_ascale[m];
                                        const float gate = __fmul_rn((float)part[t][r], __fmul_rn(p.w_scale, a));
                                        const float up = __fmul_rn((float)part[NT + t][r], __fmul_rn(p.w_scale2, a));
                                        const float rl = fmaxf(gate, 0.0f);
                                        p.y[o] = __fmul_rn(up, __fmul_rn(rl, rl));
                                    } else {
                                        if (p.acc_out) p.acc_out[o] = part[t][r];
                                        if (p.y) p.y[o] = __fmul_rn((float)part[t][r], __fmul_rn(p.w_scale, s_ascale[m]));
                                    }
                                }
                            }
                    }
                }
            }
        }
    }

    // no CTA may leave while a peer can still read or write its shared memory
    if constexpr (S > 1) cg::this_cluster().sync();
}

// ---- launcher ---------------------------------------------------------------------------------

bool decode_supports(size_t M, size_t K, size_t N)
{
    return M >= 1 && M <= DEC_MAX_TOKENS && K >= 64 && K % 64 == 0 && K <= 65536 && N >= 1 && N <= (1u << 30);
}

struct DecodeChoice { int S; };

template <int NT, int S, bool IN_I8, bool DUAL>
static bitnet_status_t launch_one(const DecodeParams &p, uint32_t flags, cudaStream_t stream)
{
    auto kernel = decode_kernel<NT, S, IN_I8, DUAL>;
    constexpr int NTD = NT * (DUAL ? 2 : 1);
    const size_t smem = (size_t)p.steps * 4 * NT * 512 + (S > 1 ? (size_t)2 * DEC_WARPS * NTD * 512 : 0);
    static size_t smem_set = 0;   // per instantiation
    if (smem > 48 * 1024 && smem > smem_set) {
        BITNET_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        smem_set = smem;
    }
    if (smem > 227 * 1024) return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "decode kernel: K=%d needs %zu bytes of shared memory", p.K, smem);

    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attrs[2];
    int n_attrs = 0;
    if (S > 1) {
        attrs[n_attrs].id = cudaLaunchAttributeClusterDimension;
        attrs[n_attrs].val.clusterDim.x = S;
        attrs[n_attrs].val.clusterDim.y = 1;
        attrs[n_attrs].val.clusterDim.z = 1;
        ++n_attrs;
    }
    if (flags & BITNET_FLAG_PDL) {
        attrs[n_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[n_attrs].val.programmaticStreamSerializationAllowed = 1;
        ++n_attrs;
    }
    cfg.blockDim = dim3(DEC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attrs;
    cfg.numAttrs = n_attrs;

    // resident clusters: ask the occupancy calculator once per (instantiation, smem size)
    static std::map<size_t, int> resident;   // not thread-safe by design: one launching thread per process
    auto it = resident.find(smem);
    if (it == resident.end()) {
        int n = 0;
        if (S > 1) {
            cfg.gridDim = dim3(S * 64);
            cudaLaunchAttribute cattr = attrs[0];
            cudaLaunchConfig_t qcfg = cfg;
            qcfg.attrs = &cattr;
            qcfg.numAttrs = 1;
            BITNET_CUDA(cudaOccupancyMaxActiveClusters(&n, kernel, &qcfg));
        } else {
            int per_sm = 0;
            BITNET_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, DEC_THREADS, smem));
            n = per_sm * device_sm_count();
        }
        if (n < 1) return fail(BITNET_ERR_KERNEL_EXECUTION, "decode kernel cannot be resident (S=%d, smem=%zu)", S, smem);
        it = resident.emplace(smem, n).first;
    }
    const int cached_clusters = it->second;
    int n_clusters = cached_clusters < p.n_blocks ? cached_clusters : p.n_blocks;
    cfg.gridDim = dim3((unsigned)(n_clusters * S));
    BITNET_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
    return BITNET_OK;
}

template <int NT, bool IN_I8, bool DUAL>
static bitnet_status_t launch_s(int S, const DecodeParams &p, uint32_t flags, cudaStream_t stream)
{
    switch (S) {
        case 1: return launch_one<NT, 1, IN_I8, DUAL>(p, flags, stream);
        case 2: return launch_one<NT, 2, IN_I8, DUAL>(p, flags, stream);
        case 4: return launch_one<NT, 4, IN_I8, DUAL>(p, flags, stream);
        case 8: return launch_one<NT, 8, IN_I8, DUAL>(p, flags, stream);
    }
    return fail(BITNET_ERR_INVALID_CONFIG, "cluster_k must be 1, 2, 4 or 8 (got %d)", S);
}

// K-split factor: enough CTAs to fill the machine twice over, without slicing K thinner
// than one loop step (4 chunks) per CTA.
static int choose_cluster_k(const DecodeParams &p)
{
    const int sms = device_sm_count();
    const int row_ctas = (p.n_blocks + DEC_WARPS - 1) / DEC_WARPS;   // CTAs if K is not split
    int S = 1;
    while (S < 8 && row_ctas * S < 2 * sms && p.chunks / (S * 2) >= 4) S *= 2;
    return S;
}

bitnet_status_t launch_decode(const ForwardArgs &a, cudaStream_t stream)
{
    if (!decode_supports(a.M, a.K, a.N))
        return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "decode kernel needs 1 <= M <= 16 and K %% 64 == 0 (M=%zu K=%zu N=%zu)", a.M, a.K, a.N);
    const bool in_i8 = a.x_i8 != nullptr;
    const bool dual = a.wp2 != nullptr;
    auto misaligned = [](const void *ptr, size_t al) { return (reinterpret_cast<uintptr_t>(ptr) & (al - 1)) != 0; };
    if (misaligned(a.wp, 16) || (dual && misaligned(a.wp2, 16)))
        return fail(BITNET_ERR_INVALID_CONFIG, "packed weights must be 16-byte aligned");
    if ((!in_i8 && misaligned(a.x, 16)) || (in_i8 && misaligned(a.x_i8, 16)))
        return fail(BITNET_ERR_INVALID_CONFIG, "activations must be 16-byte aligned");
    if (a.q_out && misaligned(a.q_out, 16)) return fail(BITNET_ERR_INVALID_CONFIG, "q_out must be 16-byte aligned");
    if (in_i8 && (a.M != 1 || dual)) return fail(BITNET_ERR_INVALID_CONFIG, "int8 input is single-token only");

    DecodeParams p = {};
    p.wp = a.wp; p.wp2 = a.wp2; p.x = a.x; p.x_i8 = a.x_i8; p.y = a.y; p.acc_out = a.acc_out;
    p.q_out = a.q_out; p.a_scale_out = a.a_scale_out; p.w_scale = a.w_scale; p.w_scale2 = a.w_scale2;
    p.M = (int)a.M; p.K = (int)a.K; p.N = (int)a.N; p.ldy = a.ldy ? a.ldy : a.N;
    p.chunks = (int)(a.K / 64);
    p.n_blocks = (int)((a.N + 15) / 16);
    int S = a.cluster_k > 0 ? a.cluster_k : choose_cluster_k(p);
    if (S > p.chunks) S = 1;
    const int NT = a.M > 8 ? 2 : 1;
    // the int8 activations of a CTA's K slice must fit in shared memory
    while (S < 8 && (size_t)(((p.chunks + S - 1) / S + 3) / 4) * 4 * NT * 512 > 160 * 1024) S *= 2;
    p.steps = ((p.chunks + S - 1) / S + 3) / 4;

    if (in_i8) return launch_s<1, true, false>(S, p, a.flags, stream);
    if (dual) return NT == 1 ? launch_s<1, false, true>(S, p, a.flags, stream) : launch_s<2, false, true>(S, p, a.flags, stream);
    return NT == 1 ? launch_s<1, false, false>(S, p, a.flags, stream) : launch_s<2, false, false>(S, p, a.flags, stream);
}

}  // namespace bitnet
