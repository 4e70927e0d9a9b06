// Decode-time BitLinear (M <= 16 tokens): a weight-streaming W2A8 GEMV for sm_100a.
//
// One CTA per SM owns a contiguous range of 16-row blocks of W.  Rows are contiguous in
// the packed layout, so a block is ONE bulk-async (TMA) copy of 16*K/4 bytes into a ring
// of shared-memory stages, issued by a producer warp and tracked by mbarriers; the first
// stages are requested before the kernel waits for its predecessor on the stream
// (programmatic dependent launch), so weight traffic overlaps the previous kernel, and
// the kernel is sized so that two CTAs fit on an SM for that overlap.
//
// Eight consumer warps split K between them.  Each warp quantises its own K slice of
// the activations (per-token absmax is folded CTA-wide first, or taken from the partial
// maxima its producer kernel left behind), keeps the int8 values in tensor-core fragment
// order (in registers when a CTA has many blocks to stream), and for every block turns
// packed words into mma operands with one AND per operand: masking a 32-bit word with
// 0x03030303 << 2j leaves code << 2j in each byte, which the u8 x s8 mma.sync.m16n8k32
// consumes unshifted; the four j classes accumulate separately and combine exactly as
// acc0 + acc1/4 + acc2/16 + acc3/64.  sum_k (code-1)*q equals sum_k code*q - sum_k q, and
// sum_k q is known from the quantiser.  The eight K-partial sums of a block meet in shared
// memory; the warps take turns to dequantise a block and write y once a barrier says all
// partial sums are in.
//
// The contraction is order-independent integer arithmetic, so the int32 accumulators are
// exact whatever the tiling.
//
// Semantics: TernaryProcessor::quantize_activations + ternary_matmul_generic
// (bitnet-inference/src/engine/ternary_operations.rs:117-172, :283-338) on the packed
// layout of BitPacked2BitPacker (bitnet-quant/src/quantization/packing.rs:352-394);
// replaces w2a8_gemv_kernel (bitnet-cuda/src/kernels/w2a8_gemv.cu:100-182).
#include <mutex>

#include "decode_common.cuh"

namespace bitnet {

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
    int seg_end0, seg_end1;       // stacked matrices: rows below seg_end0 use w_scale, below seg_end1 seg_scale1, the rest seg_scale2
    float seg_scale1, seg_scale2;
    int M, K, N;
    size_t ldy;
    int chunks;          // K / 64: a chunk is the 16 bytes (64 weights) of one 128-bit load
    int n_blocks;        // ceil(N / 16)
    int stages;          // depth of the weight ring
    int stages_free;     // stages that do not overlap the activation staging area
    unsigned stage_bytes;   // one block of one matrix is 16 * K/4 contiguous bytes; a stage holds NW of them
    unsigned stage_stride;  // stage_bytes plus 128 bytes of padding
    unsigned zero_offset;   // 16 zero bytes in dynamic shared memory that no stage and no staging area ever covers
    const unsigned *amax_in;   // optional: per-token absmax keys left by the producer kernel, [16 tokens][256 CTA slots]
    int n_amax_in;
    unsigned *amax_out;        // optional: this CTA's per-token absmax keys of what it wrote, same layout
    int weights_first;         // 1: start the weight stream at once (the activations are not ready yet anyway)
    const unsigned char *image;   // optional: activations already quantised by decode_quantize_kernel
    unsigned image_bytes;
    unsigned bst_offset; // where the activation staging area starts in dynamic shared memory
    unsigned red_offset; // where the K-split sums start
    int mrows;           // token rows kept per 8-token tile of the activation staging area (1, 2, 4 or 8)
    float *y_peers[8];   // output-feature split over several GPUs: every output goes to each of these
    int n_peers;         // (own and peer memory, plain stores over NVLink); 0 = write y only
};

template <int CW>
__device__ __forceinline__ void consumer_barrier()
{
    asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");   // the consumer warps only
}

// Dynamic shared memory: the weight ring [stages x stage_bytes], the activation staging
// area (warp-private regions of SW*4*NT fragment blocks of 64 bytes per kept token row; with BREG and little shared memory
// it overlaps the last ring stages, which the producer then fills only after every warp has
// moved its activations to registers), and the K-split sums [stages x CW x NW*NT*512].
// NT: token tiles of 8; SW: loop steps per warp (a step is 4 chunks = 256 k per warp);
// BREG: activations live in registers during the main loop (pays when a CTA streams many blocks).
// CW: consumer warps (8 leaves room for a second CTA on the SM; 16 hides more latency when one CTA
// streams many blocks).
template <int CW, int NT, int SW, bool BREG, bool IN_I8, bool DUAL>
__global__ void __launch_bounds__((CW + 1) * 32, CW == 4 ? 4 : ((CW == 8 && NT * (DUAL ? 2 : 1) <= 2 && !(BREG && SW >= 4)) ? 2 : 1))
decode_kernel(const DecodeParams p)
{
    constexpr int DEC_CWARPS = CW;
    constexpr int DEC_THREADS = (CW + 1) * 32;   // plus the producer warp
    constexpr int NW = DUAL ? 2 : 1;          // weight matrices streamed together (gate and up)
    constexpr int NTD = NT * NW;
    constexpr int NP = 1;                     // accumulator sets per j class
    constexpr int U = 3;                      // 16-wide groups a lane has in flight in the quantiser
    constexpr int DEC_DEFER = 1;              // a block is finished this many blocks after its sums were handed in

    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) unsigned long long s_full[DEC_MAX_STAGES], s_done[DEC_MAX_STAGES], s_empty[DEC_MAX_STAGES];
    __shared__ __align__(8) unsigned long long s_bst_free, s_x_issued, s_img;
    __shared__ unsigned s_key[DEC_MAX_TOKENS], s_okey[DEC_MAX_TOKENS];
    __shared__ float s_ascale[DEC_MAX_TOKENS], s_qscale[DEC_MAX_TOKENS];
    __shared__ int s_sumq[DEC_MAX_CWARPS][DEC_MAX_TOKENS];

    // the next kernel on the stream may start (and fetch its own weights) from here on
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tig = lane & 3;
    const int NS = p.stages;

    // blocks are dealt round-robin: every CTA's stream of 16-row blocks is spread over the whole
    // weight matrix in the same way, so no CTA sits on a slower set of memory channels
    const int b0 = (int)blockIdx.x, bstride = (int)gridDim.x;
    const int nb = (p.n_blocks - b0 + bstride - 1) / bstride;
    const unsigned row_bytes = (unsigned)p.K / 4;

    unsigned char *s_w = smem;
    unsigned char *s_bst = smem + p.bst_offset;
    int *s_red = reinterpret_cast<int *>(smem + p.red_offset);

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&s_full[s], 1);
            mbar_init(&s_done[s], DEC_CWARPS);
            mbar_init(&s_empty[s], 1);
        }
        mbar_init(&s_bst_free, DEC_CWARPS);
        mbar_init(&s_x_issued, DEC_CWARPS);
        mbar_init(&s_img, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < DEC_MAX_TOKENS) { s_key[tid] = 0; s_okey[tid] = 0; }
    for (int i = tid; i < DEC_MAX_CWARPS * DEC_MAX_TOKENS; i += DEC_THREADS) (&s_sumq[0][0])[i] = 0;
    if (tid < 4) reinterpret_cast<unsigned *>(smem + p.zero_offset)[tid] = 0;
    __syncthreads();

    // ======================= producer warp: keep the ring full ===============================
    // Weights do not depend on the previous kernel on the stream: no grid-dependency wait here.
    if (warp == DEC_CWARPS) {
        if (lane == 0) {
            // alone on the stream the activation loads go first, so that they do not queue behind
            // the weight stream; under programmatic dependent launch the weights go first, since
            // the activations do not exist yet
            if (!p.weights_first && !mbar_wait(&s_x_issued, 0)) return;
            for (int i = 0; i < nb; ++i) {
                const int s = i % NS;
                if (i >= NS) {
                    if (!mbar_wait(&s_empty[s], (unsigned)((i / NS) - 1) & 1u)) return;
                } else if (i >= p.stages_free) {   // first use of a stage that overlaps the staging area
                    if (!mbar_wait(&s_bst_free, 0)) return;
                }
                const int row0 = (b0 + i * bstride) * 16;
                const unsigned bytes = (unsigned)min(16, p.N - row0) * row_bytes;
                mbar_arrive_expect_tx(&s_full[s], NW * bytes);
                unsigned char *stage = s_w + (size_t)s * p.stage_stride;
                bulk_copy_g2s(stage, p.wp + (size_t)row0 * row_bytes, bytes, &s_full[s]);
                if constexpr (DUAL) bulk_copy_g2s(stage + 16 * row_bytes, p.wp2 + (size_t)row0 * row_bytes, bytes, &s_full[s]);
            }
        }
        return;
    }

    // ======================= consumer warps =====================================================
    asm volatile("griddepcontrol.wait;" ::: "memory");   // activations come from the previous kernel

    const int cw0 = (int)((long long)warp * p.chunks / DEC_CWARPS);
    const int cw1 = (int)((long long)(warp + 1) * p.chunks / DEC_CWARPS);
    const int Cw = cw1 - cw0;                              // chunks of this warp's K slice (<= 4*SW)
    // a fragment block holds 16 bytes for each (token row, k quad); only the token rows that exist are kept
    const unsigned frag_blk = (unsigned)p.mrows * 64u;
    // lanes of token rows that do not exist feed accumulator columns nobody reads: they re-read lane 0's bytes
    const unsigned frag_lane_off = ((unsigned)lane < (unsigned)p.mrows * 4u ? (unsigned)lane : 0u) * 16u;
    unsigned char *bst = s_bst + DEC_IMG_HDR + (size_t)warp * (SW * 4 * NT) * frag_blk;
    const unsigned groups_per_token = (unsigned)Cw * 4;   // 16-wide k groups
    const unsigned n_groups = (unsigned)p.M * groups_per_token;
    const size_t k_base = (size_t)cw0 * 64;
    const bool single_batch = n_groups <= 32u * U;         // the whole slice fits in one batch of registers

    float4 f[U][4];                                         // fp32 activations in flight
    auto load_batch = [&](unsigned base) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const unsigned gid = base + u * 32 + lane;
            if (gid < n_groups) {
                const unsigned m = gid / groups_per_token;
                const unsigned l = gid - m * groups_per_token;
                const float4 *src = reinterpret_cast<const float4 *>(p.x + (size_t)m * p.K + k_base + (size_t)l * 16);
#pragma unroll
                for (int v = 0; v < 4; ++v) f[u][v] = __ldg(src + v);
            }
        }
    };

    if (p.image) {
        // ---- the activations were quantised once for all CTAs: fetch the ready-made image -------------
        if (tid == 0) {
            mbar_arrive_expect_tx(&s_img, p.image_bytes);
            bulk_copy_g2s(s_bst, p.image, p.image_bytes, &s_img);
        }
        if (lane == 0) mbar_arrive(&s_x_issued);   // the weight stream may start
        if (!mbar_wait(&s_img, 0)) return;
        if (tid < DEC_CWARPS * DEC_MAX_TOKENS) (&s_sumq[0][0])[tid] = reinterpret_cast<const int *>(s_bst)[tid];
        if (tid < DEC_MAX_TOKENS) s_ascale[tid] = reinterpret_cast<const float *>(s_bst + DEC_MAX_CWARPS * DEC_MAX_TOKENS * 4)[tid];
        consumer_barrier<CW>();
    } else {
        // ---- pass 1: per-token absmax, folded CTA-wide ------------------------------------------------
        if constexpr (!IN_I8) {
            if (p.amax_in) {
                // the kernel that produced x left one partial maximum per CTA and token
                if (single_batch) load_batch(0);               // overlap the fetch of x with the fold
                __syncwarp();
                if (lane == 0) mbar_arrive(&s_x_issued);
                // keys are stored [token][256 CTA slots]; only the real tokens are read, four
                // independent loads at a time
                const int total = p.M * p.n_amax_in;
                for (int i0 = tid; i0 < total; i0 += 4 * DEC_CWARPS * 32) {
                    unsigned k4[4];
                    int tok[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int i = i0 + u * DEC_CWARPS * 32;
                        tok[u] = i < total ? i / p.n_amax_in : 0;
                        k4[u] = i < total ? __ldg(p.amax_in + tok[u] * 256 + (i - tok[u] * p.n_amax_in)) : 0u;
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (k4[u]) atomicMax(&s_key[tok[u]], k4[u]);
                }
            } else {
                unsigned cur_m = 0, cur_key = 0;   // running maximum of the token this lane is in
                for (unsigned base = 0; base < n_groups; base += 32u * U) {
                    load_batch(base);
                    if (base == 0) {
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&s_x_issued);   // the weight stream may start
                    }
    #pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const unsigned gid = base + u * 32 + lane;
                        if (gid < n_groups) {
                            const unsigned m = gid / groups_per_token;
                            unsigned key = 0;
    #pragma unroll
                            for (int v = 0; v < 4; ++v)
                                key = max(max(key, abs_key(f[u][v].x)), max(abs_key(f[u][v].y), max(abs_key(f[u][v].z), abs_key(f[u][v].w))));
                            if (m != cur_m) {
                                if (cur_key) atomicMax(&s_key[cur_m], cur_key);
                                cur_m = m;
                                cur_key = 0;
                            }
                            cur_key = max(cur_key, key);
                        }
                    }
                }
                if (cur_key) atomicMax(&s_key[cur_m], cur_key);
                if (n_groups == 0 && lane == 0) mbar_arrive(&s_x_issued);
            }
            consumer_barrier<CW>();
            if (tid < p.M) {
                const float absmax = __uint_as_float(s_key[tid]);
                s_ascale[tid] = dequant_scale(absmax);
                s_qscale[tid] = quant_scale(absmax);
                if (p.a_scale_out && blockIdx.x == 0) p.a_scale_out[tid] = dequant_scale(absmax);
            }
            consumer_barrier<CW>();
        } else {
            if (tid < p.M) s_ascale[tid] = 1.0f;
            if (lane == 0) mbar_arrive(&s_x_issued);
        }

        // ---- pass 2: quantise this warp's slice into fragment order ---------------------------------------
        {
            unsigned cur_m = 0;
            int cur_sum = 0;
            for (unsigned base = 0; base < n_groups; base += 32u * U) {
                if constexpr (!IN_I8) {
                    if (!single_batch) load_batch(base);       // second read: L1/L2 resident
                }
    #pragma unroll
                for (int u = 0; u < U; ++u) {
                    const unsigned gid = base + u * 32 + lane;
                    if (gid < n_groups) {
                        const unsigned m = gid / groups_per_token;
                        const unsigned l = gid - m * groups_per_token;
                        int q[16];
                        if constexpr (IN_I8) {
                            const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(p.x_i8 + (size_t)m * p.K + k_base + (size_t)l * 16));
    #pragma unroll
                            for (int e = 0; e < 16; ++e) q[e] = (int)(int8_t)((word_of(raw, e >> 2) >> (8 * (e & 3))) & 0xffu);
                        } else {
                            const float scale = s_qscale[m];
                            // a huge absmax makes scale subnormal or zero; the fast path assumes neither
                            const bool fast = scale >= 1e-30f && scale <= 1e30f;
    #pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                q[4 * v + 0] = quantize_any(f[u][v].x, scale, fast);
                                q[4 * v + 1] = quantize_any(f[u][v].y, scale, fast);
                                q[4 * v + 2] = quantize_any(f[u][v].z, scale, fast);
                                q[4 * v + 3] = quantize_any(f[u][v].w, scale, fast);
                            }
                            if (p.q_out && blockIdx.x == 0) {
                                uint4 canon;
                                canon.x = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((unsigned)(q[3] & 0xff) << 24);
                                canon.y = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((unsigned)(q[7] & 0xff) << 24);
                                canon.z = (q[8] & 0xff) | ((q[9] & 0xff) << 8) | ((q[10] & 0xff) << 16) | ((unsigned)(q[11] & 0xff) << 24);
                                canon.w = (q[12] & 0xff) | ((q[13] & 0xff) << 8) | ((q[14] & 0xff) << 16) | ((unsigned)(q[15] & 0xff) << 24);
                                *reinterpret_cast<uint4 *>(p.q_out + (size_t)m * p.K + k_base + (size_t)l * 16) = canon;
                            }
                        }
                        // word j holds k = j, j+4, j+8, j+12 of the group: the bytes that the mask
                        // 0x03030303 << 2j selects from a packed weight word
                        uint4 frag;
                        frag.x = (q[0] & 0xff) | ((q[4] & 0xff) << 8) | ((q[8] & 0xff) << 16) | ((unsigned)(q[12] & 0xff) << 24);
                        frag.y = (q[1] & 0xff) | ((q[5] & 0xff) << 8) | ((q[9] & 0xff) << 16) | ((unsigned)(q[13] & 0xff) << 24);
                        frag.z = (q[2] & 0xff) | ((q[6] & 0xff) << 8) | ((q[10] & 0xff) << 16) | ((unsigned)(q[14] & 0xff) << 24);
                        frag.w = (q[3] & 0xff) | ((q[7] & 0xff) << 8) | ((q[11] & 0xff) << 16) | ((unsigned)(q[15] & 0xff) << 24);
                        int sum = 0;
    #pragma unroll
                        for (int e = 0; e < 16; ++e) sum += q[e];
                        if (m != cur_m) {
                            if (cur_sum) atomicAdd(&s_sumq[warp][cur_m], cur_sum);
                            cur_m = m;
                            cur_sum = 0;
                        }
                        cur_sum += sum;
                        // slice-relative chunk c = l/4 is read by lanes with tig = c%4 in step c/4; i = l%4 is
                        // the 16-wide group inside the chunk; token m sits in tile m/8, fragment row m%8
                        const unsigned c = l >> 2, i = l & 3;
                        const unsigned step = c >> 2, ctig = c & 3;
                        const unsigned off = ((step * 4 + i) * NT + (m >> 3)) * frag_blk + ((m & 7) * 4 + ctig) * 16;
                        *reinterpret_cast<uint4 *>(bst + off) = frag;
                    }
                }
            }
            if (cur_sum) atomicAdd(&s_sumq[warp][cur_m], cur_sum);
        }
    }
    __syncwarp();

    // activations of this warp's slice: registers for the whole kernel when asked for
    uint4 breg[BREG ? SW : 1][4][NT];
    if constexpr (BREG) {
#pragma unroll
        for (int s2 = 0; s2 < SW; ++s2)
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int t = 0; t < NT; ++t)
                    breg[s2][i][t] = *reinterpret_cast<const uint4 *>(bst + (size_t)((s2 * 4 + i) * NT + t) * frag_blk + frag_lane_off);
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_bst_free);   // the staging area may be overwritten by weights
    }
    int sq[NT][2];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        sq[t][0] = s_sumq[warp][8 * t + 2 * tig];
        sq[t][1] = s_sumq[warp][8 * t + 2 * tig + 1];
    }

    // ---- main loop over this CTA's blocks -----------------------------------------------------------------
    // Byte offsets of this lane's 16-byte chunks inside a stage.  A chunk beyond the slice must read
    // zeros as weights (its activation fragments were never written and hold stale bytes): it reads a
    // zero region of its own, outside every stage -- not a stage's padding, which the activation
    // staging area may cover when the ring grows over it.  Rows past N of the last block hold stale
    // bytes: they only feed accumulators of rows that are never written.
    constexpr unsigned OFF_ZERO = 0xffffffffu;
    unsigned off_a[NW][SW], off_b[NW][SW];
#pragma unroll
    for (int w = 0; w < NW; ++w)
#pragma unroll
        for (int s2 = 0; s2 < SW; ++s2) {
            const int ci = s2 * 4 + tig;
            const unsigned col = (unsigned)(cw0 + ci) * 16;
            off_a[w][s2] = ci < Cw ? (unsigned)(w * 16 + g) * row_bytes + col : OFF_ZERO;
            off_b[w][s2] = ci < Cw ? (unsigned)(w * 16 + g + 8) * row_bytes + col : OFF_ZERO;
        }

    bool alive = true;   // false once a bounded wait gave up: the CTA only drains from then on
    // a stage is refilled only after its block was finished, so the deferral must stay below the ring depth
    // (and a CTA with only a few blocks gains nothing from it: its last blocks would just end later)
    const int want_defer = nb >= 6 ? DEC_DEFER : 0;
    const int defer = NS > want_defer ? want_defer : NS - 1;
    // Finishes block j if this warp is on duty for it: waits until every warp's partial sums of the block are
    // in, adds them up, releases the stage, dequantises and stores.
    auto finish_block = [&](int j, int sj, unsigned pj) {   // sj = j % NS, pj = (j / NS) & 1, kept by the caller
        if (!alive || ((j + (int)blockIdx.x) & (DEC_CWARPS - 1)) != warp) return;
        if (!mbar_wait(&s_done[sj], pj)) { alive = false; return; }
        const int4 *red = reinterpret_cast<const int4 *>(s_red) + (size_t)sj * (DEC_CWARPS * NTD * 32);
        const int row_a = (b0 + j * bstride) * 16 + g, row_b = row_a + 8;
        int tot[NTD][4];
#pragma unroll
        for (int u = 0; u < NTD; ++u) {
            tot[u][0] = tot[u][1] = tot[u][2] = tot[u][3] = 0;
#pragma unroll
            for (int w2 = 0; w2 < DEC_CWARPS; ++w2) {
                const int4 v = red[(w2 * NTD + u) * 32 + lane];
                tot[u][0] += v.x; tot[u][1] += v.y; tot[u][2] += v.z; tot[u][3] += v.w;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_empty[sj]);   // release: the stage and its sums may be reused
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int m = 8 * t + 2 * tig + (r & 1);
                const int row = (r & 2) ? row_b : row_a;
                if (m < p.M && row < p.N) {
                    const size_t o = (size_t)m * p.ldy + row;
                    float out;
                    if constexpr (DUAL) {
                        const float a = s_ascale[m];
                        const float gate = __fmul_rn((float)tot[t][r], __fmul_rn(p.w_scale, a));
                        const float up = __fmul_rn((float)tot[NT + t][r], __fmul_rn(p.w_scale2, a));
                        const float rl = fmaxf(gate, 0.0f);
                        out = __fmul_rn(up, __fmul_rn(rl, rl));
                        p.y[o] = out;
                    } else {
                        if (p.acc_out) p.acc_out[o] = tot[t][r];
                        const float ws = row < p.seg_end0 ? p.w_scale : (row < p.seg_end1 ? p.seg_scale1 : p.seg_scale2);
                        out = __fmul_rn((float)tot[t][r], __fmul_rn(ws, s_ascale[m]));
                        if (p.n_peers) {   // this GPU's column slice, stored into every GPU's full-width output
                            for (int pr = 0; pr < p.n_peers; ++pr) p.y_peers[pr][o] = out;
                        } else if (p.y) {
                            p.y[o] = out;
                        }
                    }
                    if (p.amax_out) {
                        const unsigned key = abs_key(out);
                        if (key > s_okey[m]) atomicMax(&s_okey[m], key);
                    }
                }
            }
    };

    // stage index and barrier phase of block i and of the block being finished, advanced without divisions
    int s = 0, sj = 0, jn = 0;
    unsigned parity = 0, pj = 0;
    auto advance = [&](int &stage, unsigned &phase) {
        if (++stage == NS) { stage = 0; phase ^= 1u; }
    };
    for (int i = 0; i < nb; ++i, advance(s, parity)) {
        if (!alive) return;
        if (!mbar_wait(&s_full[s], parity)) return;
        const unsigned stage_off = (unsigned)s * p.stage_stride;

        int acc[NW][NT][NP][4][4];   // [matrix][token tile][chain][j class][fragment register]
#pragma unroll
        for (int w = 0; w < NW; ++w)
#pragma unroll
            for (int t = 0; t < NT; ++t)
#pragma unroll
                for (int c = 0; c < NP; ++c)
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                        for (int r = 0; r < 4; ++r) acc[w][t][c][j][r] = 0;

#pragma unroll
        for (int s2 = 0; s2 < SW; ++s2) {
            if (s2 * 4 < Cw) {   // warp-uniform: this step holds at least one chunk of the slice
                uint4 bw[4][NT];
#pragma unroll
                for (int i2 = 0; i2 < 4; ++i2)
#pragma unroll
                    for (int t = 0; t < NT; ++t) {
                        if constexpr (BREG) bw[i2][t] = breg[s2][i2][t];
                        else bw[i2][t] = *reinterpret_cast<const uint4 *>(bst + (size_t)((s2 * 4 + i2) * NT + t) * frag_blk + frag_lane_off);
                    }
#pragma unroll
                for (int w = 0; w < NW; ++w) {
                    const uint4 wa = *reinterpret_cast<const uint4 *>(smem + (off_a[w][s2] != OFF_ZERO ? stage_off + off_a[w][s2] : p.zero_offset));
                    const uint4 wb = *reinterpret_cast<const uint4 *>(smem + (off_b[w][s2] != OFF_ZERO ? stage_off + off_b[w][s2] : p.zero_offset));
#pragma unroll
                    for (int pr = 0; pr < 2; ++pr) {
                        const unsigned a_lo0 = word_of(wa, 2 * pr), a_lo1 = word_of(wa, 2 * pr + 1);
                        const unsigned a_hi0 = word_of(wb, 2 * pr), a_hi1 = word_of(wb, 2 * pr + 1);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const unsigned mask = 0x03030303u << (2 * j);
#pragma unroll
                            for (int t = 0; t < NT; ++t)
                                mma_u8s8(acc[w][t][pr % NP][j], a_lo0 & mask, a_hi0 & mask, a_lo1 & mask, a_hi1 & mask,
                                         word_of(bw[2 * pr][t], j), word_of(bw[2 * pr + 1][t], j));
                        }
                    }
                }
            }
        }

        // exact partial sums of sum_k (code-1)*q over this warp's K slice, left in this warp's slot
        int4 *red = reinterpret_cast<int4 *>(s_red) + (size_t)s * (DEC_CWARPS * NTD * 32);
#pragma unroll
        for (int w = 0; w < NW; ++w)
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                int v[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    v[r] = -sq[t][r & 1];
#pragma unroll
                    for (int c = 0; c < NP; ++c)
                        v[r] += acc[w][t][c][0][r] + (acc[w][t][c][1][r] >> 2) + (acc[w][t][c][2][r] >> 4) + (acc[w][t][c][3][r] >> 6);
                }
                red[(warp * NTD + w * NT + t) * 32 + lane] = make_int4(v[0], v[1], v[2], v[3]);
            }
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_done[s]);   // release: this warp's sums are in, its reads of the stage are over

        // the warps take turns to finish a block -- DEC_DEFER blocks later, so that the warp on duty finds the
        // other warps' sums already there instead of stalling its own next block behind the slowest warp
        if (i >= defer) {
            finish_block(jn, sj, pj);
            ++jn;
            advance(sj, pj);
        }
    }
    for (; jn < nb; ++jn, advance(sj, pj)) finish_block(jn, sj, pj);
    if (!alive) return;
    if (p.amax_out) {   // this CTA's share of the per-token absmax of what the launch wrote
        consumer_barrier<CW>();
        if (tid < DEC_MAX_TOKENS) p.amax_out[(size_t)tid * 256 + blockIdx.x] = s_okey[tid];   // [token][CTA slot]
    }
}

// Quantises x[M,K] once for every CTA of the decode kernel that follows: one CTA per token,
// one read of the row (it stays in registers between the absmax fold and the rounding), and
// the int8 values land in global memory as the exact shared-memory image the decode kernel's
// warps want (header: per-warp-slice sums and absmax/127; then fragment-ordered bytes), so that
// kernel fetches it with a single bulk copy.  cw/sw/nt describe the consuming instantiation.
// Semantics: TernaryProcessor::quantize_activations (ternary_operations.rs:130-163).
// pre: the decoder-layer glue in front of the quantiser (residual add, SubLN), applied to the row while it
// sits in registers; sums run in a fixed order (lane tree, then the sixteen warps in turn).
__global__ void __launch_bounds__(512) decode_quantize_kernel(const float *x, int M, int K, int cw, int sw, int nt, int mrows,
                                                              unsigned char *__restrict__ image,
                                                              const unsigned *__restrict__ amax_in, int n_amax_in,
                                                              int8_t *__restrict__ q_out, float *__restrict__ a_scale_out,
                                                              const RowPre pre, const RowsOut rows)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the decode kernel may start fetching weights
    asm volatile("griddepcontrol.wait;" ::: "memory");
    quantize_row_to_image(x, (int)blockIdx.x, K, cw, sw, nt, mrows, image, amax_in, n_amax_in, q_out, a_scale_out, pre, rows);
}

// The same quantiser writing the row-major form the tensor-core kernels read: int8 rows with every 16-wide
// k group stored transposed (byte 4j+i holds k = 4i+j), the row sums and the scales.  K % 16 == 0, K <= 16384.
bitnet_status_t launch_quantize_rows_glued(const float *x, size_t M, size_t K, const RowPre *pre, const RowsOut &rows,
                                           int8_t *q_out, float *a_scale_out, uint32_t flags, cudaStream_t stream)
{
    if (M == 0) return BITNET_OK;
    if (K == 0 || K % 16 || K > 16384) return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "row quantiser needs K %% 16 == 0 and K <= 16384 (got %zu)", K);
    auto mis = [](const void *ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) != 0; };
    const RowPre rp = pre ? *pre : RowPre{};
    if (mis(x) || mis(rows.q_perm) || mis(q_out) || mis(rp.residual) || mis(rp.sum_out) || mis(rp.norm_w) || mis(rp.norm_b) || mis(rp.normed_out))
        return fail(BITNET_ERR_INVALID_CONFIG, "row quantiser buffers must be 16-byte aligned");
    if (!rows.q_perm || !rows.rowsum || !rows.a_scale) return fail(BITNET_ERR_NULL_POINTER, "row quantiser: null output");
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attrs[1];
    cfg.gridDim = dim3((unsigned)M);
    cfg.blockDim = dim3(512);
    cfg.stream = stream;
    cfg.attrs = attrs;
    if (flags & BITNET_FLAG_PDL) {
        attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 1;
    }
    BITNET_CUDA(cudaLaunchKernelEx(&cfg, decode_quantize_kernel, x, (int)M, (int)K, 1, 1, 1, 1, static_cast<unsigned char *>(nullptr),
                                   static_cast<const unsigned *>(nullptr), 0, q_out, a_scale_out, rp, rows));
    return BITNET_OK;
}

// ---- launcher -----------------------------------------------------------------------------------------

static int steps_needed(size_t K, int cw) { return (int)(((K / 64 + cw - 1) / cw + 3) / 4); }

static bool shape_fits(size_t M, size_t K, bool dual)
{
    const int sw = steps_needed(K, 8);   // the eight-warp kernels are the ones every shape can fall back to
    const int nt = M > 8 ? 2 : 1;
    if (dual) return sw <= 2;
    return nt == 1 ? sw <= 8 : sw <= 4;
}

bool decode_supports(size_t M, size_t K, size_t N)
{
    return M >= 1 && M <= DEC_MAX_TOKENS && K >= 64 && K % 64 == 0 && N >= 1 && N <= (1u << 30) && shape_fits(M, K, false);
}

bool decode_supports_dual(size_t M, size_t K, size_t N) { return decode_supports(M, K, N) && shape_fits(M, K, true); }

// CTAs a decode launch over N output features uses (also the number of absmax partials it writes).
int decode_grid(size_t N)
{
    const int n_blocks = (int)((N + 15) / 16);
    const int sms = device_sm_count();
    return n_blocks < sms ? n_blocks : sms;
}

template <int CW, int NT, int SW, bool BREG, bool IN_I8, bool DUAL>
static bitnet_status_t launch_one(DecodeParams p, uint32_t flags, cudaStream_t stream)
{
    auto kernel = decode_kernel<CW, NT, SW, BREG, IN_I8, DUAL>;
    constexpr int NW = DUAL ? 2 : 1;
    const unsigned row_bytes = (unsigned)p.K / 4;
    const unsigned real_stage = NW * 16 * row_bytes;
    p.stage_bytes = real_stage;
    p.stage_stride = real_stage + 128;
    const size_t bst_bytes = DEC_IMG_HDR + (size_t)CW * SW * 4 * NT * (size_t)p.mrows * 64;   // image header + fragment data
    if (p.image) p.image_bytes = (unsigned)bst_bytes;
    const size_t red_per_stage = (size_t)CW * NW * NT * 512;   // one slot of partial sums per consumer warp
    const size_t budget = 208 * 1024;

    const int grid = decode_grid((size_t)p.N);
    const int max_blocks = (p.n_blocks + grid - 1) / grid;
    int want = p.stages > 0 ? p.stages : DEC_MAX_STAGES;
    if (want > DEC_MAX_STAGES) want = DEC_MAX_STAGES;
    if (want > max_blocks) want = max_blocks;
    if (CW == 4 && want > 2) want = 2;   // small CTAs: at most two stages, so that four CTAs fit an SM

    int stages = want, stages_free = want;
    size_t bst_offset = 0, smem = 0;
    if ((size_t)want * (p.stage_stride + red_per_stage) + bst_bytes <= budget) {
        // everything fits side by side
        bst_offset = (size_t)want * p.stage_stride;
        smem = bst_offset + bst_bytes + (size_t)want * red_per_stage;
    } else if (BREG) {
        // let the ring grow over the staging area; those stages open once the activations
        // are in registers
        while (stages > 1 && (size_t)stages * (p.stage_stride + red_per_stage) > budget) --stages;
        size_t ring = (size_t)stages * p.stage_stride;
        if (ring < bst_bytes + p.stage_stride) ring = bst_bytes + p.stage_stride;   // at least one stage stays free
        bst_offset = ring - bst_bytes;
        stages_free = (int)(bst_offset / p.stage_stride);
        if (stages_free > stages) stages_free = stages;
        smem = ring + (size_t)stages * red_per_stage;
    } else {
        while (stages > 1 && (size_t)stages * (p.stage_stride + red_per_stage) + bst_bytes > budget) --stages;
        stages_free = stages;
        bst_offset = (size_t)stages * p.stage_stride;
        smem = bst_offset + bst_bytes + (size_t)stages * red_per_stage;
    }
    if (smem + 16 > 227 * 1024 || stages_free < 1)
        return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "decode kernel: K=%d needs %zu bytes of shared memory", p.K, smem);
    p.stages = stages;
    p.stages_free = stages_free;
    p.bst_offset = (unsigned)bst_offset;
    p.red_offset = (unsigned)(smem - (size_t)stages * red_per_stage);
    p.zero_offset = (unsigned)smem;   // after everything else: nothing is ever copied over it
    smem += 16;

    // The attribute is raised once per instantiation and device to the most this kernel can ever ask
    // for, under a lock: host threads launch concurrently (one per stream), and a smaller value set by
    // one of them must never undercut a launch another one is about to make.
    {
        static std::mutex mu;
        static bool raised[64] = {false};
        int dev = 0;
        BITNET_CUDA(cudaGetDevice(&dev));
        const bool tracked = dev >= 0 && dev < 64;
        std::lock_guard<std::mutex> lock(mu);
        if (!tracked || !raised[dev]) {
            cudaFuncAttributes fa;
            int optin = 0;
            BITNET_CUDA(cudaFuncGetAttributes(&fa, kernel));
            BITNET_CUDA(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
            BITNET_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, optin - (int)fa.sharedSizeBytes));
            if (tracked) raised[dev] = true;
        }
    }

    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attrs[1];
    int n_attrs = 0;
    if (flags & BITNET_FLAG_PDL) {
        attrs[n_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[n_attrs].val.programmaticStreamSerializationAllowed = 1;
        ++n_attrs;
    }
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((CW + 1) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attrs;
    cfg.numAttrs = n_attrs;
    BITNET_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
    return BITNET_OK;
}

struct DecodePlan {
    int cw, sw, nt;      // consumer warps, steps per warp (template value), token tiles
    bool breg, wide;
};

static int round_sw(int sw) { return sw <= 1 ? 1 : (sw <= 2 ? 2 : (sw <= 4 ? 4 : 8)); }

static DecodePlan decode_plan(size_t M, size_t K, size_t N, bool dual, bool throughput)
{
    DecodePlan pl;
    pl.nt = M > 8 ? 2 : 1;
    const int n_blocks = (int)((N + 15) / 16);
    const int grid = decode_grid(N);
    const int blocks_per_cta = (n_blocks + grid - 1) / grid;
    // keep the activations in registers when a CTA streams enough blocks to repay the registers,
    // and use the sixteen-warp kernel when it streams many (K up to 8192)
    pl.breg = pl.nt == 1 && !dual && blocks_per_cta >= 4;
    pl.wide = pl.breg && blocks_per_cta >= 6 && steps_needed(K, 16) <= 2;
    pl.cw = pl.wide ? 16 : 8;
    pl.sw = round_sw(steps_needed(K, pl.cw));
    // throughput mode (BITNET_FLAG_THROUGHPUT): four consumer warps, so that four CTAs (of different launches) share an SM
    if (throughput && !pl.breg) {
        const int sw4 = round_sw(steps_needed(K, 4));
        if (steps_needed(K, 4) <= 8 && (sw4 <= 4 || (pl.nt == 1 && !dual))) {
            pl.cw = 4;
            pl.sw = sw4;
        }
    }
    return pl;
}

template <int NT, bool IN_I8, bool DUAL>
static bitnet_status_t launch_sw(const DecodePlan &pl, const DecodeParams &p, uint32_t flags, cudaStream_t stream)
{
    if (pl.wide) {
        // sixteen consumer warps, activations in registers: one CTA per SM streaming many blocks
        if constexpr (NT == 1 && !DUAL) {
            if (pl.sw == 1) return launch_one<16, 1, 1, true, IN_I8, false>(p, flags, stream);
            if (pl.sw == 2) return launch_one<16, 1, 2, true, IN_I8, false>(p, flags, stream);
        }
    }
    if (pl.cw == 4) {
        if (pl.sw == 1) return launch_one<4, NT, 1, false, IN_I8, DUAL>(p, flags, stream);
        if (pl.sw == 2) return launch_one<4, NT, 2, false, IN_I8, DUAL>(p, flags, stream);
        if (pl.sw == 4) return launch_one<4, NT, 4, false, IN_I8, DUAL>(p, flags, stream);
        if constexpr (NT == 1 && !DUAL) {
            if (pl.sw == 8) return launch_one<4, NT, 8, false, IN_I8, DUAL>(p, flags, stream);
        }
    }
#define BITNET_DECODE_CASE(SWV)                                                                   \
    return pl.breg ? launch_one<8, NT, SWV, true, IN_I8, DUAL>(p, flags, stream)                 \
                   : launch_one<8, NT, SWV, false, IN_I8, DUAL>(p, flags, stream)
    if (pl.sw == 1) { BITNET_DECODE_CASE(1); }
    if (pl.sw == 2) { BITNET_DECODE_CASE(2); }
    if constexpr (!DUAL) {
        if (pl.sw == 4) { BITNET_DECODE_CASE(4); }
        if constexpr (NT == 1) {
            if (pl.sw == 8) return launch_one<8, NT, 8, false, IN_I8, DUAL>(p, flags, stream);
        }
    }
#undef BITNET_DECODE_CASE
    return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "decode kernel: K=%d is too wide for this token count", p.K);
}

// Activation count (M*K) above which the activations are quantised by their own small launch
// instead of by every CTA of the decode kernel: the redundant per-CTA quantiser work grows with
// M*K, while the extra launch costs a fixed couple of microseconds in the dependency chain.
static bool use_split(size_t M, size_t K) { return M * K > 8192; }

// Token rows kept per 8-token tile of the staging area: the power of two that covers M (8 from 5 tokens on).
static int decode_mrows(size_t M) { return M > 4 ? 8 : (M > 2 ? 4 : (M > 1 ? 2 : 1)); }

size_t decode_image_bytes_always(size_t M, size_t K, size_t N, bool dual)
{
    // the larger of the two plans' images, so that one workspace serves a call with or without the throughput flag
    size_t bytes = 0;
    for (int t = 0; t < 2; ++t) {
        const DecodePlan pl = decode_plan(M, K, N, dual, t != 0);
        const size_t b = align_up(DEC_IMG_HDR + (size_t)pl.cw * pl.sw * 4 * pl.nt * (size_t)decode_mrows(M) * 64, 256);
        if (b > bytes) bytes = b;
    }
    return bytes;
}

size_t decode_image_bytes(size_t M, size_t K, size_t N, bool dual)
{
    if (!use_split(M, K)) return 0;
    return decode_image_bytes_always(M, K, N, dual);
}

bitnet_status_t launch_decode(const ForwardArgs &a, cudaStream_t stream)
{
    const bool in_i8 = a.x_i8 != nullptr;
    const bool dual = a.wp2 != nullptr;
    if (!decode_supports(a.M, a.K, a.N) || (dual && !shape_fits(a.M, a.K, true)))
        return fail(BITNET_ERR_UNSUPPORTED_OPERATION,
                    "decode kernel needs 1 <= M <= 16, K %% 64 == 0 and K <= 16384 (8192 for M > 8, 4096 for a gate/up pair) (M=%zu K=%zu N=%zu)",
                    a.M, a.K, a.N);
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
    p.stages = a.stages;
    p.amax_in = a.amax_in; p.n_amax_in = a.n_amax_in; p.amax_out = a.amax_out;
    p.weights_first = (a.flags & BITNET_FLAG_PDL) ? 1 : 0;
    p.mrows = decode_mrows(a.M);
    p.n_peers = a.n_peers;
    p.seg_end0 = p.seg_end1 = 0x7fffffff;
    if (a.n_seg > 0) {
        if (dual || a.n_seg > 2) return fail(BITNET_ERR_INVALID_CONFIG, "at most three stacked matrices, and not with the gate/up pair");
        p.seg_end0 = (int)a.seg_end[0]; p.seg_scale1 = a.seg_scale[0];
        if (a.n_seg > 1) { p.seg_end1 = (int)a.seg_end[1]; p.seg_scale2 = a.seg_scale[1]; }
    }
    for (int r = 0; r < a.n_peers && r < 8; ++r) p.y_peers[r] = a.y_peers[r];
    if (a.n_peers && dual) return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "peer outputs are not available for the gate/up pair launch");
    const DecodePlan pl = decode_plan(a.M, a.K, a.N, dual, (a.flags & BITNET_FLAG_THROUGHPUT) != 0);

    if (a.pre && (in_i8 || !a.image_ws || a.amax_in))
        return fail(BITNET_ERR_INVALID_CONFIG, "row glue (residual, normalisation) runs in the quantiser launch: it needs the image workspace");
    if (!in_i8 && a.image_ws && (a.force_split || a.pre || a.image_ready || use_split(a.M, a.K))) {
        // quantise once, then let every CTA fetch the result
        const size_t need = decode_image_bytes_always(a.M, a.K, a.N, dual);
        if (a.image_ws_bytes < need || misaligned(a.image_ws, 16))
            return fail(BITNET_ERR_WORKSPACE, "decode path needs %zu bytes of 16-byte aligned workspace", need);
        const RowPre pre = a.pre ? *a.pre : RowPre{};
        if (pre.norm_w && (!pre.norm_b || misaligned(pre.norm_w, 16) || misaligned(pre.norm_b, 16)))
            return fail(BITNET_ERR_INVALID_CONFIG, "normalisation needs 16-byte aligned weight and bias vectors");
        if ((pre.residual && misaligned(pre.residual, 16)) || (pre.sum_out && misaligned(pre.sum_out, 16)) ||
            (pre.normed_out && misaligned(pre.normed_out, 16)))
            return fail(BITNET_ERR_INVALID_CONFIG, "row glue buffers must be 16-byte aligned");
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute attrs[1];
        cfg.gridDim = dim3((unsigned)a.M);
        cfg.blockDim = dim3(512);
        cfg.stream = stream;
        cfg.attrs = attrs;
        if (a.flags & BITNET_FLAG_PDL) {
            attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attrs[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.numAttrs = 1;
        }
        if (!a.image_ready)
            BITNET_CUDA(cudaLaunchKernelEx(&cfg, decode_quantize_kernel, a.x, (int)a.M, (int)a.K, pl.cw, pl.sw, pl.nt, p.mrows,
                                           static_cast<unsigned char *>(a.image_ws), a.amax_in, a.n_amax_in, a.q_out,
                                           a.a_scale_out, pre, RowsOut{}));
        p.image = static_cast<const unsigned char *>(a.image_ws);
        p.q_out = nullptr; p.a_scale_out = nullptr; p.amax_in = nullptr;
        p.weights_first = 1;   // the image does not exist before the quantiser ends: fetch weights meanwhile
        // the decode kernel must be allowed to start while the quantiser runs
        const uint32_t flags = a.flags | BITNET_FLAG_PDL;
        if (dual) return pl.nt == 1 ? launch_sw<1, false, true>(pl, p, flags, stream) : launch_sw<2, false, true>(pl, p, flags, stream);
        return pl.nt == 1 ? launch_sw<1, false, false>(pl, p, flags, stream) : launch_sw<2, false, false>(pl, p, flags, stream);
    }
    if (in_i8) return launch_sw<1, true, false>(pl, p, a.flags, stream);
    if (dual) return pl.nt == 1 ? launch_sw<1, false, true>(pl, p, a.flags, stream) : launch_sw<2, false, true>(pl, p, a.flags, stream);
    return pl.nt == 1 ? launch_sw<1, false, false>(pl, p, a.flags, stream) : launch_sw<2, false, false>(pl, p, a.flags, stream);
}

}  // namespace bitnet

// Flags raised by device-side bounded waits since the last call (bit 0: a decode-kernel
// barrier wait ran out, bit 1: a GEMM-kernel wait, bit 2: the cluster GEMM, bit 3: the grouped decode kernel).  Synchronises the device.
extern "C" bitnet_status_t bitnet_device_error_flags(uint32_t *flags_out)
{
    if (!flags_out) return bitnet::fail(BITNET_ERR_NULL_POINTER, "bitnet_device_error_flags: null output");
    unsigned v = 0, zero = 0;
    BITNET_CUDA(cudaMemcpyFromSymbol(&v, bitnet::g_decode_error_flags, sizeof(v)));
    if (v) BITNET_CUDA(cudaMemcpyToSymbol(bitnet::g_decode_error_flags, &zero, sizeof(zero)));
    unsigned pf = 0, mm = 0, gr = 0;
    BITNET_TRY(bitnet::prefill_take_error_flags(&pf));
    BITNET_TRY(bitnet::midm_take_error_flags(&mm));
    BITNET_TRY(bitnet::group_take_error_flags(&gr));
    *flags_out = v | pf | mm | gr;
    return BITNET_OK;
}
