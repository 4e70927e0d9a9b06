// Grouped decode: many independent BitLinear calls of one width K (at most 16 tokens each), or gate/up pairs, as
// ONE persistent launch.
//
// A decode-time block of a 2B-class model moves a few megabytes of packed weights: a launch of its own is over
// before the memory system is at speed, and what a step of many such blocks costs is launches, not bytes.  When
// the blocks do not depend on one another (the same block of many model replicas or layers-in-flight, the
// per-request adapters of a serving batch, a benchmark's batch of blocks), the group kernel treats all of their
// 16-row weight blocks as one list: CTA c of a one-per-SM grid streams the c-th contiguous share of that list
// through the same shared-memory ring and the same masked-word u8 x s8 tensor-core steps as decode_kernel, and
// swaps the quantised-activation image when its share crosses from one member into the next (at most a couple of
// times per CTA).  The activations of all members are quantised by one launch in front (one CTA per token).
//
// Arithmetic per member is that of the single launch: exact int32 accumulators, the same fp32 dequantisation, so
// a grouped run and member-by-member runs give the same bits.
//
// Semantics per member: TernaryProcessor::quantize_activations + ternary_matmul_generic
// (bitnet-inference/src/engine/ternary_operations.rs:117-172, :283-338); the FFN form is
// FeedForwardNetwork::forward (bitnet-inference/src/engine/transformer_layers.rs:608-629).
#include <mutex>
#include <new>
#include <vector>

#include "decode_common.cuh"

namespace bitnet {

struct GroupMember {
    const uint8_t *wp, *wp2;     // packed weights (wp2: the up matrix of a gate/up pair)
    const float *x;              // activations [M, K], read by the group's quantiser launch
    unsigned char *image;        // quantised-activation image: written by that launch, fetched by the decode launch
    float *y;                    // [M, ldy]
    float w_scale, w_scale2;
    int M, N, ldy, mrows;
    unsigned image_bytes;
    int blk_begin;               // first of this member's 16-row blocks in the group's list
    int tok_begin;               // first of its tokens in the group's token list
};

struct GroupParams {
    const GroupMember *members;  // n + 1 entries: the last one only closes the lists (blk_begin = total_blocks)
    const int *cta_member;       // per CTA: the member that holds the first block of its share
    int total_blocks;
    int K, chunks, cw, stages;
    unsigned stage_stride, bst_offset, red_offset;
};

constexpr int GROUP_MAX_STAGES = 12;

__device__ __forceinline__ void group_barrier(int threads)
{
    asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory");   // the consumer warps only
}

// One CTA per token of the group: the member's row quantiser.
__global__ void __launch_bounds__(512) group_quantize_kernel(const GroupMember *__restrict__ members, const int *__restrict__ token_member,
                                                             int K, int cw, int sw, int nt)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the decode launch may start fetching weights
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const GroupMember mb = members[token_member[blockIdx.x]];
    quantize_row_to_image(mb.x, (int)blockIdx.x - mb.tok_begin, K, cw, sw, nt, mb.mrows, mb.image, nullptr, 0, nullptr, nullptr,
                          RowPre{}, RowsOut{});
}

// NT: token tiles of 8; SW: loop steps per warp (a step is 4 chunks = 256 k per warp); DUAL: gate/up pair with the
// ReLU^2 gating in the epilogue.  Consumer warps: p.cw (blockDim.x / 32 - 1), each owning a K slice of every block.
// Dynamic shared memory: the weight ring (every stage ends in 128 bytes of padding that no copy writes: its first
// 16 bytes are zeroed once and are what chunks past a warp's K slice read as weights), the staging area of one
// member's image, and the K-split sums per stage.
// MAXT: thread bound (384 leaves 168 registers a thread).  One CTA per SM: two smaller CTAs per SM (half the ring
// each, twice the warps) measured 15 % slower, and so did computing two blocks per pass (a stage is held longer).
template <int NT, int SW, bool DUAL, int MAXT>
__global__ void __launch_bounds__(MAXT, 1) decode_group_kernel(const GroupParams p)
{
    constexpr int NW = DUAL ? 2 : 1;
    constexpr int NTD = NT * NW;
    constexpr bool BREG = NT == 1;   // activations of the current member in registers

    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) unsigned long long s_full[GROUP_MAX_STAGES], s_done[GROUP_MAX_STAGES], s_empty[GROUP_MAX_STAGES];
    __shared__ __align__(8) unsigned long long s_img;
    __shared__ unsigned s_dead;   // a bounded wait gave up somewhere in the CTA: everybody stops at the next member

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tig = lane & 3;
    const int CW = p.cw, NS = p.stages;
    // A contiguous share of the block list per CTA, so that it meets only the few members its share crosses (dealing
    // the blocks of a run round-robin to a team of CTAs, for wider streams in DRAM, measured slower at every team size).
    const int g0 = (int)((long long)blockIdx.x * p.total_blocks / gridDim.x);
    const int g1 = (int)((long long)(blockIdx.x + 1) * p.total_blocks / gridDim.x);
    const unsigned row_bytes = (unsigned)p.K / 4;

    unsigned char *s_w = smem;
    unsigned char *s_bst = smem + p.bst_offset;
    int *s_red = reinterpret_cast<int *>(smem + p.red_offset);

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&s_full[s], 1);
            mbar_init(&s_done[s], (unsigned)CW);
            mbar_init(&s_empty[s], 1);
        }
        mbar_init(&s_img, 1);
        s_dead = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int z = tid; z < NS * 4; z += (int)blockDim.x)
        reinterpret_cast<unsigned *>(smem + (size_t)(z >> 2) * p.stage_stride + (size_t)NW * 16 * row_bytes)[z & 3] = 0;
    __syncthreads();

    // ======================= producer warp: keep the ring full, across members ===============================
    // Weights and the member table do not depend on the kernel in front of this one: no grid-dependency wait.
    if (warp == CW) {
        if (lane == 0) {
            int mi = p.cta_member[blockIdx.x];
            int begin = p.members[mi].blk_begin, end = p.members[mi + 1].blk_begin;
            const uint8_t *wp = p.members[mi].wp, *wp2 = p.members[mi].wp2;
            int N = p.members[mi].N;
            int s = 0;
            unsigned phase = 0;   // of the stage's previous use
            for (int gb = g0, i = 0; gb < g1; ++gb, ++i) {
                while (gb >= end) {
                    ++mi;
                    begin = end;
                    end = p.members[mi + 1].blk_begin;
                    wp = p.members[mi].wp; wp2 = p.members[mi].wp2; N = p.members[mi].N;
                }
                if (i >= NS && !mbar_wait(&s_empty[s], phase)) return;
                const int row0 = (gb - begin) * 16;
                const unsigned bytes = (unsigned)min(16, N - row0) * row_bytes;
                mbar_arrive_expect_tx(&s_full[s], NW * bytes);
                unsigned char *stage = s_w + (size_t)s * p.stage_stride;
                bulk_copy_g2s(stage, wp + (size_t)row0 * row_bytes, bytes, &s_full[s]);
                if constexpr (DUAL) bulk_copy_g2s(stage + 16 * row_bytes, wp2 + (size_t)row0 * row_bytes, bytes, &s_full[s]);
                if (++s == NS) { s = 0; if (i >= NS) phase ^= 1u; }
            }
        }
        return;
    }

    // ======================= consumer warps =====================================================
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the images come from the quantiser launch

    const int cw0 = (int)((long long)warp * p.chunks / CW);
    const int cw1 = (int)((long long)(warp + 1) * p.chunks / CW);
    const int Cw = cw1 - cw0;                              // chunks of this warp's K slice (<= 4*SW)

    // Byte offsets of this lane's 16-byte chunks inside a stage; a chunk beyond the slice reads the stage's zeroed
    // padding (its activation fragments were never written and hold stale bytes).
    const unsigned OFF_ZERO = (unsigned)NW * 16 * row_bytes;
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

    // ring position and barrier phase of the block being computed (i) and of the block being finished (jn):
    // they run on across members
    int s = 0, sj = 0, i = 0, jn = 0;
    unsigned parity = 0, pj = 0;
    auto advance = [&](int &stage, unsigned &phase) {
        if (++stage == NS) { stage = 0; phase ^= 1u; }
    };

    int mi = p.cta_member[blockIdx.x];
    unsigned seg = 0;
    for (int gb = g0; gb < g1; ++seg) {
        while (gb >= p.members[mi + 1].blk_begin) ++mi;
        const GroupMember mb = p.members[mi];
        const int seg_end = min(g1, p.members[mi + 1].blk_begin);

        // a fragment block holds 16 bytes for each (token row, k quad); only the token rows that exist are kept
        const unsigned frag_blk = (unsigned)mb.mrows * 64u;
        // lanes of token rows that do not exist feed accumulator columns nobody reads: they re-read lane 0's bytes
        const unsigned frag_lane_off = ((unsigned)lane < (unsigned)mb.mrows * 4u ? (unsigned)lane : 0u) * 16u;
        const size_t warp_region = DEC_IMG_HDR + (size_t)warp * (SW * 4 * NT) * frag_blk;
        const unsigned char *bst = s_bst + warp_region;
        const float *hdr_ascale = reinterpret_cast<const float *>(s_bst + DEC_MAX_CWARPS * DEC_MAX_TOKENS * 4);

        uint4 breg[BREG ? SW : 1][4][NT];
        int sq[NT][2];        // sum_k q of the whole row: the +1 of the weight code is taken out once per output
        float asc[NT][2];     // absmax / 127 of this lane's two tokens per tile
        bool ok = true;
        if constexpr (BREG) {
            // One tile of tokens: the member's image goes from global memory (L2: the quantiser launch just wrote it)
            // straight into registers, so no shared memory is spent on it and the ring gets that room.
            const unsigned char *img = mb.image;
            const int *g_sumq = reinterpret_cast<const int *>(img);
            const float *g_ascale = reinterpret_cast<const float *>(img + DEC_MAX_CWARPS * DEC_MAX_TOKENS * 4);
#pragma unroll
            for (int s2 = 0; s2 < SW; ++s2)
#pragma unroll
                for (int i2 = 0; i2 < 4; ++i2)
#pragma unroll
                    for (int t = 0; t < NT; ++t)
                        breg[s2][i2][t] = __ldg(reinterpret_cast<const uint4 *>(img + warp_region + (size_t)((s2 * 4 + i2) * NT + t) * frag_blk + frag_lane_off));
#pragma unroll
            for (int t = 0; t < NT; ++t)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    sq[t][e] = 0;
                    for (int w2 = 0; w2 < CW; ++w2) sq[t][e] += __ldg(g_sumq + w2 * DEC_MAX_TOKENS + 8 * t + 2 * tig + e);
                    asc[t][e] = __ldg(g_ascale + 8 * t + 2 * tig + e);
                }
        } else {
            group_barrier(CW * 32);                        // every warp is through with the previous member's image
            if (*reinterpret_cast<volatile unsigned *>(&s_dead)) break;
            if (tid == 0) {
                mbar_arrive_expect_tx(&s_img, mb.image_bytes);
                bulk_copy_g2s(s_bst, mb.image, mb.image_bytes, &s_img);
            }
            ok = mbar_wait(&s_img, seg & 1u);
            if (ok) {
                const int *hdr_sumq = reinterpret_cast<const int *>(s_bst);
#pragma unroll
                for (int t = 0; t < NT; ++t)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        sq[t][e] = 0;
                        for (int w2 = 0; w2 < CW; ++w2) sq[t][e] += hdr_sumq[w2 * DEC_MAX_TOKENS + 8 * t + 2 * tig + e];
                        asc[t][e] = hdr_ascale[8 * t + 2 * tig + e];
                    }
            }
        }

        const int nbs = seg_end - gb;
        const int i_end = i + nbs;
        const int local0 = gb - mb.blk_begin - i;          // block `pos` of the ring is the member's block local0 + pos
        // a stage is refilled only after its block was finished (handing it back as soon as every warp had read it,
        // with the sums guarded by a barrier of their own, measured slower), so the deferral must stay below the ring depth
        const int defer = (nbs >= 6 && NS > 1) ? 1 : 0;

        // Finishes block j if this warp is on duty for it: waits until every warp's partial sums of the block are
        // in, adds them up, releases the stage, dequantises and stores.
        auto finish_block = [&](int j) {
            if (!ok || (j + (int)blockIdx.x) % CW != warp) return;
            if (!mbar_wait(&s_done[sj], pj)) { ok = false; return; }
            const int4 *red = reinterpret_cast<const int4 *>(s_red) + (size_t)sj * (CW * NTD * 32);
            const int row_a = (local0 + j) * 16 + g, row_b = row_a + 8;
            int tot[NTD][4];
#pragma unroll
            for (int u = 0; u < NTD; ++u) tot[u][0] = tot[u][1] = tot[u][2] = tot[u][3] = 0;
            for (int w2 = 0; w2 < CW; ++w2) {
#pragma unroll
                for (int u = 0; u < NTD; ++u) {
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
                    if (m < mb.M && row < mb.N) {
                        const size_t o = (size_t)m * mb.ldy + row;
                        const float a = asc[t][r & 1];
                        const int rs = sq[t][r & 1];
                        if constexpr (DUAL) {
                            const float gate = __fmul_rn((float)((tot[t][r] >> 6) - rs), __fmul_rn(mb.w_scale, a));
                            const float up = __fmul_rn((float)((tot[NT + t][r] >> 6) - rs), __fmul_rn(mb.w_scale2, a));
                            const float rl = fmaxf(gate, 0.0f);
                            mb.y[o] = __fmul_rn(up, __fmul_rn(rl, rl));
                        } else {
                            mb.y[o] = __fmul_rn((float)((tot[t][r] >> 6) - rs), __fmul_rn(mb.w_scale, a));
                        }
                    }
                }
        };

        for (; i < i_end && ok; ++i, advance(s, parity)) {
            if (!mbar_wait(&s_full[s], parity)) { ok = false; break; }
            const unsigned stage_off = (unsigned)s * p.stage_stride;

            int acc[NW][NT][4][4];   // [matrix][token tile][j class][fragment register]; the first step starts them
#pragma unroll
            for (int s2 = 0; s2 < SW; ++s2) {
                if (s2 == 0 || s2 * 4 < Cw) {   // warp-uniform: this step holds at least one chunk of the slice
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
                        const uint4 wa = *reinterpret_cast<const uint4 *>(smem + stage_off + off_a[w][s2]);
                        const uint4 wb = *reinterpret_cast<const uint4 *>(smem + stage_off + off_b[w][s2]);
#pragma unroll
                        for (int pr = 0; pr < 2; ++pr) {
                            const unsigned a_lo0 = word_of(wa, 2 * pr), a_lo1 = word_of(wa, 2 * pr + 1);
                            const unsigned a_hi0 = word_of(wb, 2 * pr), a_hi1 = word_of(wb, 2 * pr + 1);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const unsigned mask = 0x03030303u << (2 * j);
#pragma unroll
                                for (int t = 0; t < NT; ++t) {
                                    if (s2 == 0 && pr == 0)
                                        mma_u8s8_first(acc[w][t][j], a_lo0 & mask, a_hi0 & mask, a_lo1 & mask, a_hi1 & mask,
                                                       word_of(bw[0][t], j), word_of(bw[1][t], j));
                                    else
                                        mma_u8s8(acc[w][t][j], a_lo0 & mask, a_hi0 & mask, a_lo1 & mask, a_hi1 & mask,
                                                 word_of(bw[2 * pr][t], j), word_of(bw[2 * pr + 1][t], j));
                                }
                            }
                        }
                    }
                }
            }
            // 64 x this warp's exact partial sum of sum_k code*q: class j holds 4^j times its share, so
            // ((acc0*4 + acc1)*4 + acc2)*4 + acc3 needs no division; the warp on duty divides the total once
            int4 *red = reinterpret_cast<int4 *>(s_red) + (size_t)s * (CW * NTD * 32);
#pragma unroll
            for (int w = 0; w < NW; ++w)
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    int v[4];
#pragma unroll
                    for (int r = 0; r < 4; ++r)
                        v[r] = ((acc[w][t][0][r] * 4 + acc[w][t][1][r]) * 4 + acc[w][t][2][r]) * 4 + acc[w][t][3][r];
                    red[(warp * NTD + w * NT + t) * 32 + lane] = make_int4(v[0], v[1], v[2], v[3]);
                }
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_done[s]);   // release: this warp's sums are in, its reads of the stage are over

            // the warps take turns to finish a block, one block later, so that the warp on duty finds the other
            // warps' sums already there instead of stalling its own next block behind the slowest warp
            if (i >= jn + defer) {
                finish_block(jn);
                ++jn;
                advance(sj, pj);
            }
        }
        for (; jn < i_end && ok; ++jn, advance(sj, pj)) finish_block(jn);
        if (!ok) {
            // a wait gave up: without a staging area nothing else holds the warps together, this one just stops;
            // with one, everybody stops at the next member's barrier
            if constexpr (BREG) return;
            *reinterpret_cast<volatile unsigned *>(&s_dead) = 1u;
        }
        gb = seg_end;
    }
}

// ---- host side --------------------------------------------------------------------------------------

// Set by this file's bounded waits; bit 3 of bitnet_device_error_flags.
bitnet_status_t group_take_error_flags(unsigned *flags)
{
    unsigned v = 0, zero = 0;
    BITNET_CUDA(cudaMemcpyFromSymbol(&v, g_decode_error_flags, sizeof(v)));
    if (v) BITNET_CUDA(cudaMemcpyToSymbol(g_decode_error_flags, &zero, sizeof(zero)));
    *flags = v ? 8u : 0u;
    return BITNET_OK;
}

namespace {

int group_mrows(size_t M) { return M > 4 ? 8 : (M > 2 ? 4 : (M > 1 ? 2 : 1)); }

// One launch pair (quantiser + decode) over all members: shapes, shared-memory layout and device tables.
struct GroupStage {
    int K = 0, nt = 1, sw = 1, cw = 0, stages = 0, grid = 0, total_blocks = 0, total_tokens = 0;
    bool dual = false;
    unsigned stage_stride = 0, bst_offset = 0, red_offset = 0;
    size_t smem = 0;
    size_t image_stride = 0;          // bytes between members' images
    GroupMember *members_dev = nullptr;
    int *cta_member_dev = nullptr, *token_member_dev = nullptr;
};

// Consumer warps and steps per warp for a width: the fewest steps whose warps cover K, so that no tensor-core
// step runs on padding (K = 2560: ten warps x one step; K = 6912: fourteen x two).
bitnet_status_t group_stage_plan(GroupStage &st, size_t K, size_t max_M, bool dual)
{
    if (K < 64 || K % 64 || K > 16384) return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "grouped decode needs K %% 64 == 0 and 64 <= K <= 16384 (got %zu)", K);
    st.K = (int)K;
    st.dual = dual;
    st.nt = max_M > 8 ? 2 : 1;
    const int chunks = (int)(K / 64);
    const int max_cw = st.nt == 1 ? 15 : 8;   // with the producer warp: 16 warps (128 registers each) or 9
    const int max_sw = dual ? 2 : 4;
    st.cw = 0;
    for (int sw = 1; sw <= max_sw; sw *= 2) {
        const int cw = (chunks + 4 * sw - 1) / (4 * sw);
        if (cw <= max_cw) { st.sw = sw; st.cw = cw; break; }
    }
    if (!st.cw) return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "grouped decode: K=%zu is too wide for %zu tokens%s", K, max_M, dual ? " (gate/up pair)" : "");
    const int nw = dual ? 2 : 1;
    const unsigned row_bytes = (unsigned)K / 4;
    st.stage_stride = (unsigned)nw * 16 * row_bytes + 128;
    const size_t image_bytes = align_up(DEC_IMG_HDR + (size_t)st.cw * st.sw * 4 * st.nt * (size_t)group_mrows(max_M) * 64, 128);
    st.image_stride = align_up(image_bytes, 256);
    const size_t bst_bytes = st.nt == 1 ? 0 : image_bytes;   // one token tile: the image lives in registers, not in shared memory
    const size_t red_per_stage = (size_t)st.cw * nw * st.nt * 512;
    const size_t budget = 226 * 1024;   // all of an SM's shared memory: the ring's depth is the bytes in flight
    if (bst_bytes + 2 * (st.stage_stride + red_per_stage) > budget)
        return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "grouped decode: K=%zu at %zu tokens does not fit shared memory", K, max_M);
    int stages = (int)((budget - bst_bytes) / (st.stage_stride + red_per_stage));
    if (stages > GROUP_MAX_STAGES) stages = GROUP_MAX_STAGES;
    st.stages = stages;
    st.bst_offset = (unsigned)stages * st.stage_stride;
    st.red_offset = st.bst_offset + (unsigned)bst_bytes;
    st.smem = (size_t)st.red_offset + (size_t)stages * red_per_stage;
    return BITNET_OK;
}

template <int NT, int SW, bool DUAL, int MAXT>
bitnet_status_t group_launch_one(const GroupStage &st, const GroupParams &p, cudaStream_t stream)
{
    auto kernel = decode_group_kernel<NT, SW, DUAL, MAXT>;
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
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // starts (and fetches weights) while the quantiser runs
    attrs[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = dim3((unsigned)st.grid);
    cfg.blockDim = dim3((unsigned)(st.cw + 1) * 32);
    cfg.dynamicSmemBytes = st.smem;
    cfg.stream = stream;
    cfg.attrs = attrs;
    cfg.numAttrs = 1;
    BITNET_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
    return BITNET_OK;
}

template <int NT, bool DUAL>
bitnet_status_t group_launch_sw(const GroupStage &st, const GroupParams &p, cudaStream_t stream)
{
    if constexpr (NT == 1) {
        // up to eleven warps: 168 registers a thread, room for two blocks of a gate/up pair per pass
        if ((st.cw + 1) * 32 <= 384) {
            if (st.sw == 1) return group_launch_one<1, 1, DUAL, 384>(st, p, stream);
            if (st.sw == 2) return group_launch_one<1, 2, DUAL, 384>(st, p, stream);
        }
        if constexpr (!DUAL) {
            if (st.sw == 1) return group_launch_one<1, 1, false, 512>(st, p, stream);
            if (st.sw == 2) return group_launch_one<1, 2, false, 512>(st, p, stream);
            if (st.sw == 4) return group_launch_one<1, 4, false, 512>(st, p, stream);
        } else {
            if (st.sw == 1) return group_launch_one<1, 1, true, 512>(st, p, stream);
            if (st.sw == 2) return group_launch_one<1, 2, true, 512>(st, p, stream);
        }
    } else {
        if (st.sw == 1) return group_launch_one<2, 1, DUAL, 288>(st, p, stream);
        if (st.sw == 2) return group_launch_one<2, 2, DUAL, 288>(st, p, stream);
        if constexpr (!DUAL) {
            if (st.sw == 4) return group_launch_one<2, 4, false, 288>(st, p, stream);
        }
    }
    return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "grouped decode: no kernel for this width");
}

bitnet_status_t group_stage_run(const GroupStage &st, cudaStream_t stream)
{
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attrs[1];
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = dim3((unsigned)st.total_tokens);
    cfg.blockDim = dim3(512);
    cfg.stream = stream;
    cfg.attrs = attrs;
    cfg.numAttrs = 1;
    BITNET_CUDA(cudaLaunchKernelEx(&cfg, group_quantize_kernel, (const GroupMember *)st.members_dev, (const int *)st.token_member_dev, st.K,
                                   st.cw, st.sw, st.nt));
    GroupParams p = {};
    p.members = st.members_dev;
    p.cta_member = st.cta_member_dev;
    p.total_blocks = st.total_blocks;
    p.K = st.K;
    p.chunks = st.K / 64;
    p.cw = st.cw;
    p.stages = st.stages;
    p.stage_stride = st.stage_stride;
    p.bst_offset = st.bst_offset;
    p.red_offset = st.red_offset;
    if (st.dual) return st.nt == 1 ? group_launch_sw<1, true>(st, p, stream) : group_launch_sw<2, true>(st, p, stream);
    return st.nt == 1 ? group_launch_sw<1, false>(st, p, stream) : group_launch_sw<2, false>(st, p, stream);
}

// What the caller gives for one member of a stage; images and list positions are filled in by group_stage_build.
struct StageMemberIn {
    const uint8_t *wp, *wp2;
    const float *x;
    float *y;
    float w_scale, w_scale2;
    size_t M, N, ldy;
};

size_t group_stage_table_bytes(size_t n, size_t total_tokens, int sms)
{
    return align_up((n + 1) * sizeof(GroupMember), 256) + align_up((size_t)sms * sizeof(int), 256) + align_up(total_tokens * sizeof(int), 256);
}

// Lays the stage's tables out at `dev` (device) and uploads them; images start at `images`.
bitnet_status_t group_stage_build(GroupStage &st, const std::vector<StageMemberIn> &in, unsigned char *dev, unsigned char *images)
{
    const size_t n = in.size();
    std::vector<GroupMember> members(n + 1);
    std::vector<int> token_member;
    int blocks = 0, tokens = 0;
    for (size_t i = 0; i < n; ++i) {
        GroupMember &m = members[i];
        m.wp = in[i].wp; m.wp2 = in[i].wp2; m.x = in[i].x; m.y = in[i].y;
        m.w_scale = in[i].w_scale; m.w_scale2 = in[i].w_scale2;
        m.M = (int)in[i].M; m.N = (int)in[i].N; m.ldy = (int)in[i].ldy;
        m.mrows = group_mrows(in[i].M);
        m.image = images + i * st.image_stride;
        m.image_bytes = (unsigned)(DEC_IMG_HDR + (size_t)st.cw * st.sw * 4 * st.nt * (size_t)m.mrows * 64);
        m.blk_begin = blocks;
        m.tok_begin = tokens;
        blocks += (int)((in[i].N + 15) / 16);
        tokens += (int)in[i].M;
        for (size_t t = 0; t < in[i].M; ++t) token_member.push_back((int)i);
    }
    members[n] = GroupMember{};
    members[n].blk_begin = blocks;
    members[n].tok_begin = tokens;
    st.total_blocks = blocks;
    st.total_tokens = tokens;
    const int sms = device_sm_count();
    st.grid = blocks < sms ? blocks : sms;
    std::vector<int> cta_member((size_t)sms, 0);
    size_t mi = 0;
    for (int c = 0; c < st.grid; ++c) {
        const int first = (int)((long long)c * blocks / st.grid);
        while (mi + 1 < n && first >= members[mi + 1].blk_begin) ++mi;
        cta_member[(size_t)c] = (int)mi;
    }
    st.members_dev = reinterpret_cast<GroupMember *>(dev);
    dev += align_up((n + 1) * sizeof(GroupMember), 256);
    st.cta_member_dev = reinterpret_cast<int *>(dev);
    dev += align_up((size_t)sms * sizeof(int), 256);
    st.token_member_dev = reinterpret_cast<int *>(dev);
    BITNET_CUDA(cudaMemcpy(st.members_dev, members.data(), (n + 1) * sizeof(GroupMember), cudaMemcpyHostToDevice));
    BITNET_CUDA(cudaMemcpy(st.cta_member_dev, cta_member.data(), cta_member.size() * sizeof(int), cudaMemcpyHostToDevice));
    BITNET_CUDA(cudaMemcpy(st.token_member_dev, token_member.data(), token_member.size() * sizeof(int), cudaMemcpyHostToDevice));
    return BITNET_OK;
}

bool misaligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; }

}  // namespace
}  // namespace bitnet

using namespace bitnet;

struct bitnet_ffn_group {
    int device = 0;
    void *slab = nullptr;
    GroupStage pair, down;     // gate/up with the gating, then the down projection
};

static void group_release(bitnet_ffn_group *g)
{
    if (!g) return;
    if (g->slab) {
        cudaSetDevice(g->device);
        cudaFree(g->slab);
    }
    delete g;
}

extern "C" bitnet_status_t bitnet_ffn_group_create(const bitnet_ffn_group_member *members, size_t n_members, size_t hidden,
                                                   size_t ffn, bitnet_ffn_group **out)
{
    if (!out) return fail(BITNET_ERR_NULL_POINTER, "bitnet_ffn_group_create: null output");
    *out = nullptr;
    if (!members || n_members == 0) return fail(BITNET_ERR_INVALID_CONFIG, "bitnet_ffn_group_create: no members");
    if (n_members > (1u << 20)) return fail(BITNET_ERR_INVALID_CONFIG, "bitnet_ffn_group_create: too many members");
    if (hidden == 0 || ffn == 0) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "bitnet_ffn_group_create: zero dimension");
    size_t max_M = 0, tokens = 0;
    for (size_t i = 0; i < n_members; ++i) {
        const bitnet_ffn_group_member &m = members[i];
        if (!m.gate_packed_dev || !m.up_packed_dev || !m.down_packed_dev || !m.x_dev || !m.y_dev)
            return fail(BITNET_ERR_NULL_POINTER, "FFN group: member %zu has a null pointer", i);
        if (m.M == 0 || m.M > DEC_MAX_TOKENS) return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "FFN group: member %zu has %zu tokens (1..16)", i, m.M);
        if (misaligned16(m.gate_packed_dev) || misaligned16(m.up_packed_dev) || misaligned16(m.down_packed_dev) || misaligned16(m.x_dev) || misaligned16(m.y_dev))
            return fail(BITNET_ERR_INVALID_CONFIG, "FFN group: buffers of member %zu must be 16-byte aligned", i);
        if (m.M > max_M) max_M = m.M;
        tokens += m.M;
    }
    bitnet_ffn_group *g = new (std::nothrow) bitnet_ffn_group();
    if (!g) return fail(BITNET_ERR_MEMORY_ALLOCATION, "out of host memory");
    bitnet_status_t st = group_stage_plan(g->pair, hidden, max_M, true);
    if (st == BITNET_OK) st = group_stage_plan(g->down, ffn, max_M, false);
    if (st == BITNET_OK) st = check_cuda(cudaGetDevice(&g->device), "cudaGetDevice");
    if (st != BITNET_OK) { group_release(g); return st; }

    const int sms = device_sm_count();
    const size_t tables = 2 * group_stage_table_bytes(n_members, tokens, sms);
    const size_t images_pair = n_members * g->pair.image_stride, images_down = n_members * g->down.image_stride;
    size_t h_bytes = 0;
    for (size_t i = 0; i < n_members; ++i) h_bytes += align_up(members[i].M * ffn * sizeof(float), 256);
    st = check_cuda(cudaMalloc(&g->slab, tables + images_pair + images_down + h_bytes), "cudaMalloc (FFN group)");
    if (st != BITNET_OK) { group_release(g); return st; }

    unsigned char *dev = static_cast<unsigned char *>(g->slab);
    unsigned char *tab_pair = dev, *tab_down = dev + tables / 2;
    unsigned char *img_pair = dev + tables, *img_down = img_pair + images_pair;
    unsigned char *h = img_down + images_down;
    std::vector<StageMemberIn> a(n_members), b(n_members);
    for (size_t i = 0; i < n_members; ++i) {
        const bitnet_ffn_group_member &m = members[i];
        float *h_i = reinterpret_cast<float *>(h);
        h += align_up(m.M * ffn * sizeof(float), 256);
        a[i] = StageMemberIn{m.gate_packed_dev, m.up_packed_dev, m.x_dev, h_i, m.gate_scale, m.up_scale, m.M, ffn, ffn};
        b[i] = StageMemberIn{m.down_packed_dev, nullptr, h_i, m.y_dev, m.down_scale, 0.0f, m.M, hidden, hidden};
    }
    st = group_stage_build(g->pair, a, tab_pair, img_pair);
    if (st == BITNET_OK) st = group_stage_build(g->down, b, tab_down, img_down);
    if (st != BITNET_OK) { group_release(g); return st; }
    *out = g;
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_ffn_group_run(bitnet_ffn_group *g, cudaStream_t stream)
{
    if (!g) return fail(BITNET_ERR_NULL_POINTER, "bitnet_ffn_group_run: null group");
    int dev = -1;
    BITNET_CUDA(cudaGetDevice(&dev));
    if (dev != g->device) return fail(BITNET_ERR_INVALID_CONFIG, "bitnet_ffn_group_run: the group lives on device %d, the current device is %d", g->device, dev);
    BITNET_TRY(group_stage_run(g->pair, stream));
    return group_stage_run(g->down, stream);
}

extern "C" void bitnet_ffn_group_destroy(bitnet_ffn_group *g) { group_release(g); }

// ---- a group of independent BitLinear calls of one shape -------------------------------------------------

struct bitnet_bitlinear_group {
    int device = 0;
    void *slab = nullptr;
    GroupStage stage;
};

static void linear_group_release(bitnet_bitlinear_group *g)
{
    if (!g) return;
    if (g->slab) {
        cudaSetDevice(g->device);
        cudaFree(g->slab);
    }
    delete g;
}

extern "C" bitnet_status_t bitnet_bitlinear_group_create(const bitnet_bitlinear_group_member *members, size_t n_members, size_t K,
                                                         size_t N, bitnet_bitlinear_group **out)
{
    if (!out) return fail(BITNET_ERR_NULL_POINTER, "bitnet_bitlinear_group_create: null output");
    *out = nullptr;
    if (!members || n_members == 0) return fail(BITNET_ERR_INVALID_CONFIG, "bitnet_bitlinear_group_create: no members");
    if (n_members > (1u << 20)) return fail(BITNET_ERR_INVALID_CONFIG, "bitnet_bitlinear_group_create: too many members");
    if (K == 0 || N == 0 || N > (1u << 30)) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "bitnet_bitlinear_group_create: bad dimension");
    size_t max_M = 0, tokens = 0;
    for (size_t i = 0; i < n_members; ++i) {
        const bitnet_bitlinear_group_member &m = members[i];
        if (!m.packed_dev || !m.x_dev || !m.y_dev) return fail(BITNET_ERR_NULL_POINTER, "BitLinear group: member %zu has a null pointer", i);
        if (m.M == 0 || m.M > DEC_MAX_TOKENS) return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "BitLinear group: member %zu has %zu tokens (1..16)", i, m.M);
        if (misaligned16(m.packed_dev) || misaligned16(m.x_dev) || misaligned16(m.y_dev))
            return fail(BITNET_ERR_INVALID_CONFIG, "BitLinear group: buffers of member %zu must be 16-byte aligned", i);
        if (m.ldy && m.ldy < N) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "BitLinear group: member %zu has ldy %zu < N %zu", i, m.ldy, N);
        if (m.M > max_M) max_M = m.M;
        tokens += m.M;
    }
    bitnet_bitlinear_group *g = new (std::nothrow) bitnet_bitlinear_group();
    if (!g) return fail(BITNET_ERR_MEMORY_ALLOCATION, "out of host memory");
    bitnet_status_t st = group_stage_plan(g->stage, K, max_M, false);
    if (st == BITNET_OK) st = check_cuda(cudaGetDevice(&g->device), "cudaGetDevice");
    if (st != BITNET_OK) { linear_group_release(g); return st; }
    const size_t tables = group_stage_table_bytes(n_members, tokens, device_sm_count());
    st = check_cuda(cudaMalloc(&g->slab, tables + n_members * g->stage.image_stride), "cudaMalloc (BitLinear group)");
    if (st != BITNET_OK) { linear_group_release(g); return st; }
    std::vector<StageMemberIn> in(n_members);
    for (size_t i = 0; i < n_members; ++i) {
        const bitnet_bitlinear_group_member &m = members[i];
        in[i] = StageMemberIn{m.packed_dev, nullptr, m.x_dev, m.y_dev, m.w_scale, 0.0f, m.M, N, m.ldy ? m.ldy : N};
    }
    unsigned char *dev = static_cast<unsigned char *>(g->slab);
    st = group_stage_build(g->stage, in, dev, dev + tables);
    if (st != BITNET_OK) { linear_group_release(g); return st; }
    *out = g;
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_bitlinear_group_run(bitnet_bitlinear_group *g, cudaStream_t stream)
{
    if (!g) return fail(BITNET_ERR_NULL_POINTER, "bitnet_bitlinear_group_run: null group");
    int dev = -1;
    BITNET_CUDA(cudaGetDevice(&dev));
    if (dev != g->device) return fail(BITNET_ERR_INVALID_CONFIG, "bitnet_bitlinear_group_run: the group lives on device %d, the current device is %d", g->device, dev);
    return group_stage_run(g->stage, stream);
}

extern "C" void bitnet_bitlinear_group_destroy(bitnet_bitlinear_group *g) { linear_group_release(g); }
