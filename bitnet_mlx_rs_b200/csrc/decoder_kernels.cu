// Kernels of a decode step around the BitLinear projections: token-embedding gather, the stand-alone
// row glue (residual add + SubLN), grouped-query attention of one new token per sequence over a bf16
// KV cache, and the token sampler.  All of them are one pass over their input: HBM bound, no tensor cores.
//
// Semantics followed (paths inside the reference project):
//   TokenEmbedding::forward          bitnet-inference/src/engine/forward_pass_pipeline.rs:31-77 (a row gather; the
//                                    reference's body draws random rows instead of gathering, a stub)
//   SubLNNormalization::forward      bitnet-inference/src/engine/transformer_layers.rs:356-386
//   MultiHeadAttention::forward      transformer_layers.rs:460-547: scores = q k^T / sqrt(head_dim), softmax over the
//                                    keys, weights x values; RoPE is the identity there (:278-289)
//   KVCache::{update, get}           bitnet-inference/src/cache/kv_cache.rs:125-176: cache[batch, heads, max_seq, head_dim]
//   TokenSampler::sample             bitnet-inference/src/engine/sampling.rs:106-189 (argmax / temperature, top-k, top-p;
//                                    the reference's filters are stubs that return the logits unchanged and its draw
//                                    ignores them; its linear congruential generator is kept for the draw)
#include <cuda_bf16.h>

#include <mutex>

#include "common.cuh"

namespace bitnet {

// ---- embedding gather -----------------------------------------------------------------------------------

__global__ void __launch_bounds__(256) embed_gather_kernel(const int *__restrict__ ids, const float *__restrict__ table, float *__restrict__ x,
                                                           int hidden, int vocab)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int m = blockIdx.x;
    int id = ids[m];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);   // an id outside the table reads its nearest row instead of faulting
    const float4 *src = reinterpret_cast<const float4 *>(table + (size_t)id * hidden);
    float4 *dst = reinterpret_cast<float4 *>(x + (size_t)m * hidden);
    for (int i = threadIdx.x; i < hidden / 4; i += blockDim.x) dst[i] = __ldg(src + i);
}

bitnet_status_t launch_embed_gather(const int *ids, const float *table, float *x, size_t M, size_t hidden, size_t vocab,
                                    cudaStream_t stream)
{
    if (M == 0) return BITNET_OK;
    if (hidden % 4) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "embedding width must be a multiple of 4 (got %zu)", hidden);
    embed_gather_kernel<<<(unsigned)M, 256, 0, stream>>>(ids, table, x, (int)hidden, (int)vocab);
    return check_launch("embed_gather_kernel");
}

// ---- stand-alone row glue ------------------------------------------------------------------------------

__global__ void __launch_bounds__(512) row_pre_kernel(const float *x, int K, const RowPre pre)
{
    __shared__ float s_fsum[2][16];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int m = blockIdx.x, tid = threadIdx.x;
    const int n_groups = K / 16;
    float4 f[2][4];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int G = tid + u * 512;
        if (G < n_groups) {
            const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)m * K + (size_t)G * 16);
#pragma unroll
            for (int v = 0; v < 4; ++v) f[u][v] = src[v];
        }
    }
    apply_row_pre(f, pre, m, K, tid, s_fsum);
}

bitnet_status_t launch_row_pre(const float *x, size_t M, size_t K, const RowPre &pre, uint32_t flags, cudaStream_t stream)
{
    if (M == 0) return BITNET_OK;
    if (K % 16 || K > 16384 || K == 0)
        return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "row glue needs K %% 16 == 0 and K <= 16384 (got %zu)", K);
    auto mis = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
    if (mis(x) || mis(pre.residual) || mis(pre.sum_out) || mis(pre.norm_w) || mis(pre.norm_b) || mis(pre.normed_out))
        return fail(BITNET_ERR_INVALID_CONFIG, "row glue buffers must be 16-byte aligned");
    if (pre.norm_w && !pre.norm_b) return fail(BITNET_ERR_NULL_POINTER, "normalisation needs weight and bias");
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
    BITNET_CUDA(cudaLaunchKernelEx(&cfg, row_pre_kernel, x, (int)K, pre));
    return BITNET_OK;
}

// ---- attention of one new token per sequence --------------------------------------------------------------

struct AttnParams {
    const float *qkv;        // [B, ldq]: the new token's q at column 0, k at k_off, v at v_off
    int ldq, k_off, v_off;
    __nv_bfloat16 *kcache;   // [B_cache][n_kv][max_seq][HD]
    __nv_bfloat16 *vcache;
    const int *pos;          // [B]: tokens already cached; the new token goes to position pos[b]
    float *out;              // [B, n_heads * HD]
    float *part_o;           // [B][n_heads][n_splits][HD] unnormalised partial outputs
    float *part_ml;          // [B][n_heads][n_splits][2]  running maximum and sum
    unsigned *counters;      // [B][n_kv], zero between launches
    int n_heads, n_kv, max_seq, n_splits;
    float scale;
};

__device__ __forceinline__ float bf16_lo(unsigned w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(unsigned w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ unsigned pack_bf16(float a, float b)
{
    const unsigned lo = (unsigned)__bfloat16_as_ushort(__float2bfloat16_rn(a));
    const unsigned hi = (unsigned)__bfloat16_as_ushort(__float2bfloat16_rn(b));
    return lo | (hi << 16);
}

// Sums NV values across the warp so that value i ends up in the lanes with (lane >> (5 - log2 NV)) == i:
// halves are exchanged while more than one value is left (a reduce-scatter), the rest is a butterfly.
template <int NV>
__device__ __forceinline__ float warp_reduce_scatter(float (&v)[NV], int lane)
{
    int off = 16;
#pragma unroll
    for (int n = NV; n > 1; n >>= 1) {
        const int half = n >> 1;
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < half; ++i) {
            const float send = upper ? v[i] : v[i + half];
            const float keep = upper ? v[i + half] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
        off >>= 1;
    }
#pragma unroll
    for (int o = 16 / NV; o >= 1; o >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
    return v[0];
}

// The end of an attention CTA: the four warps' partial results (running maximum, sum and unnormalised output per
// head, in shared memory) are folded; with one split the result is final, otherwise it goes to scratch and the CTA that
// arrives last at the (sequence, KV head) counter folds the splits.
template <int G, int HD>
__device__ __forceinline__ void attention_fold(const AttnParams &p, int split, int kvh, int b, int tid, float (*s_m)[8], float (*s_l)[8],
                                               float (*s_o)[G][HD], unsigned *s_last)
{
    constexpr float NEG_INF = -3.0e38f;
    const int h0 = kvh * G;
    for (int e = tid; e < G * HD; e += 128) {
        const int g = e / HD, d = e - g * HD;
        float mx = NEG_INF;
#pragma unroll
        for (int w = 0; w < 4; ++w) mx = fmaxf(mx, s_m[w][g]);
        float l = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = s_m[w][g] > NEG_INF ? expf(s_m[w][g] - mx) : 0.0f;
            l += s_l[w][g] * f;
            acc += s_o[w][g][d] * f;
        }
        if (p.n_splits == 1) {
            p.out[(size_t)b * p.n_heads * HD + (size_t)(h0 + g) * HD + d] = acc / l;
        } else {
            const size_t slot = ((size_t)b * p.n_heads + h0 + g) * p.n_splits + split;
            p.part_o[slot * HD + d] = acc;
            if (d == 0) { p.part_ml[slot * 2] = mx; p.part_ml[slot * 2 + 1] = l; }
        }
    }
    if (p.n_splits == 1) return;

    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned old = atomicAdd(p.counters + b * p.n_kv + kvh, 1u);
        *s_last = old == (unsigned)p.n_splits - 1u ? 1u : 0u;
    }
    __syncthreads();
    if (!*s_last) return;
    __threadfence();
    // the last CTA to arrive folds the splits: all maxima and sums first (one load per thread, all in flight at
    // once), a weight per split and head, then the weighted partial outputs
    float *s_w = &s_o[0][0][0];                 // [G][32] weights, then [G] sums: the warps' outputs are consumed
    float *s_lsum = s_w + G * 32;
    __syncthreads();
    for (int i = tid; i < G * p.n_splits; i += 128) {
        const int g = i / p.n_splits, s2 = i - g * p.n_splits;
        const size_t slot = ((size_t)b * p.n_heads + h0 + g) * p.n_splits + s2;
        s_w[g * 32 + s2] = __ldcg(p.part_ml + slot * 2);
        s_w[G * 32 + G + g * 32 + s2] = __ldcg(p.part_ml + slot * 2 + 1);
    }
    __syncthreads();
    if (tid < G) {
        float mx = NEG_INF;
        for (int s2 = 0; s2 < p.n_splits; ++s2) mx = fmaxf(mx, s_w[tid * 32 + s2]);
        float l = 0.0f;
        for (int s2 = 0; s2 < p.n_splits; ++s2) {
            const float ms = s_w[tid * 32 + s2];
            const float f = ms > NEG_INF ? expf(ms - mx) : 0.0f;
            l += s_w[G * 32 + G + tid * 32 + s2] * f;
            s_w[tid * 32 + s2] = f;
        }
        s_lsum[tid] = l;
    }
    __syncthreads();
    for (int e = tid; e < G * HD; e += 128) {
        const int g = e / HD, d = e - g * HD;
        const size_t slot0 = ((size_t)b * p.n_heads + h0 + g) * p.n_splits;
        float acc = 0.0f;
        int s2 = 0;
        for (; s2 + 4 <= p.n_splits; s2 += 4) {
            const float v0 = __ldcg(p.part_o + (slot0 + s2) * HD + d), v1 = __ldcg(p.part_o + (slot0 + s2 + 1) * HD + d);
            const float v2 = __ldcg(p.part_o + (slot0 + s2 + 2) * HD + d), v3 = __ldcg(p.part_o + (slot0 + s2 + 3) * HD + d);
            acc += v0 * s_w[g * 32 + s2];
            acc += v1 * s_w[g * 32 + s2 + 1];
            acc += v2 * s_w[g * 32 + s2 + 2];
            acc += v3 * s_w[g * 32 + s2 + 3];
        }
        for (; s2 < p.n_splits; ++s2) acc += __ldcg(p.part_o + (slot0 + s2) * HD + d) * s_w[g * 32 + s2];
        p.out[(size_t)b * p.n_heads * HD + (size_t)(h0 + g) * HD + d] = acc / s_lsum[g];
    }
    if (tid == 0) p.counters[b * p.n_kv + kvh] = 0u;   // ready for the next launch
}

// grid (n_splits, n_kv, B), 128 threads.  A CTA takes a contiguous range of one sequence's positions for one KV
// head and all G query heads that share it; a lane owns HD/32 dimensions of every row (coalesced 256-byte
// rows), a warp takes NB positions at a time.  Scores of a batch are reduced across the lanes in one
// reduce-scatter, the running softmax is kept per head, and probabilities go through shared memory to
// weight the value rows.  Several splits of one (sequence, KV head) meet through a counter: the CTA
// that arrives last folds the partial results.
template <int G, int HD, int NB>
__global__ void __launch_bounds__(128) attention_decode_kernel(const AttnParams p)
{
    constexpr int DPL = HD / 32;
    constexpr int NV = NB * G;
    static_assert(NV <= 32 && (NV & (NV - 1)) == 0, "positions per batch x heads must be a power of two up to 32");
    static_assert(DPL == 2 || DPL == 4, "head_dim 64 or 128");
    constexpr int SH = (NV == 32 ? 0 : NV == 16 ? 1 : NV == 8 ? 2 : NV == 4 ? 3 : NV == 2 ? 4 : 5);   // lanes per value
    constexpr float NEG_INF = -3.0e38f;

    __shared__ float s_p[4][32];
    __shared__ float s_c[4][8];
    __shared__ float s_m[4][8], s_l[4][8];
    __shared__ float s_o[4][G][HD];
    __shared__ unsigned s_last;

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int L = p.pos[b] + 1;                        // keys including the new token
    if (L > p.max_seq) L = p.max_seq;            // a full cache: the host refuses this; never index past the end
    if (L < 1) L = 1;
    const int chunk = (L + p.n_splits - 1) / p.n_splits;
    const int p0 = split * chunk;
    const int p1 = min(L, p0 + chunk);

    const float *qrow = p.qkv + (size_t)b * p.ldq + (size_t)(kvh * G) * HD + lane * DPL;
    float qr[G][DPL];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int d = 0; d < DPL; ++d) qr[g][d] = qrow[g * HD + d];

    // the new token's key and value, rounded to the cache's bf16
    const float *knew = p.qkv + (size_t)b * p.ldq + p.k_off + kvh * HD + lane * DPL;
    const float *vnew = p.qkv + (size_t)b * p.ldq + p.v_off + kvh * HD + lane * DPL;
    unsigned kn[DPL / 2], vn[DPL / 2];
#pragma unroll
    for (int d = 0; d < DPL / 2; ++d) {
        kn[d] = pack_bf16(knew[2 * d], knew[2 * d + 1]);
        vn[d] = pack_bf16(vnew[2 * d], vnew[2 * d + 1]);
    }
    const size_t row0 = ((size_t)b * p.n_kv + kvh) * (size_t)p.max_seq;
    const unsigned *kc = reinterpret_cast<const unsigned *>(p.kcache + row0 * HD) + lane * (DPL / 2);
    const unsigned *vc = reinterpret_cast<const unsigned *>(p.vcache + row0 * HD) + lane * (DPL / 2);
    if (warp == 0 && p0 <= L - 1 && L - 1 < p1) {   // the CTA whose range holds the new position appends it
        unsigned *kw = reinterpret_cast<unsigned *>(p.kcache + (row0 + (L - 1)) * HD) + lane * (DPL / 2);
        unsigned *vw = reinterpret_cast<unsigned *>(p.vcache + (row0 + (L - 1)) * HD) + lane * (DPL / 2);
#pragma unroll
        for (int d = 0; d < DPL / 2; ++d) { kw[d] = kn[d]; vw[d] = vn[d]; }
    }

    // a lane keeps the running maximum and sum of the head (lane >> SH) % G
    float m_run = NEG_INF, l_run = 0.0f;
    float o[G][DPL];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int d = 0; d < DPL; ++d) o[g][d] = 0.0f;

    // rows of NB positions: loaded one batch ahead of the arithmetic, so that a warp always has loads in flight
    auto load_batch = [&](unsigned (&kraw)[NB][DPL / 2], unsigned (&vraw)[NB][DPL / 2], int base) {
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            const int pos = base + j;
            const bool cached = pos < p1 && pos != L - 1;
#pragma unroll
            for (int d = 0; d < DPL / 2; ++d) {
                kraw[j][d] = cached ? __ldcs(kc + (size_t)pos * (HD / 2) + d) : (pos == L - 1 ? kn[d] : 0u);
                vraw[j][d] = cached ? __ldcs(vc + (size_t)pos * (HD / 2) + d) : (pos == L - 1 ? vn[d] : 0u);
            }
        }
    };
    auto process_batch = [&](const unsigned (&kraw)[NB][DPL / 2], const unsigned (&vraw)[NB][DPL / 2], int base) {
        float part[NV];
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            float kf[DPL];
#pragma unroll
            for (int d = 0; d < DPL / 2; ++d) { kf[2 * d] = bf16_lo(kraw[j][d]); kf[2 * d + 1] = bf16_hi(kraw[j][d]); }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float acc = 0.0f;
#pragma unroll
                for (int d = 0; d < DPL; ++d) acc = fmaf(qr[g][d], kf[d], acc);
                part[j * G + g] = acc;
            }
        }
        const float tot = warp_reduce_scatter<NV>(part, lane);
        const int idx = lane >> SH;                // this lane's (position, head) of the batch
        const int my_j = idx / G;
        const bool valid = base + my_j < p1;
        const float s = valid ? tot * p.scale : NEG_INF;
        float bm = s;
#pragma unroll
        for (int of = G << SH; of < 32; of <<= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, of));
        const float m_new = fmaxf(m_run, bm);      // the batch's first position always exists, so m_new is finite
        const float pj = valid ? expf(s - m_new) : 0.0f;
        const float corr = m_run > NEG_INF ? expf(m_run - m_new) : 0.0f;
        float ps = pj;
#pragma unroll
        for (int of = G << SH; of < 32; of <<= 1) ps += __shfl_xor_sync(0xffffffffu, ps, of);
        l_run = l_run * corr + ps;
        m_run = m_new;
        s_p[warp][idx] = pj;                       // lanes that share a value write the same number
        if (idx < G) s_c[warp][idx] = corr;        // idx < G: position 0 of the batch, head idx
        __syncwarp();
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float c = s_c[warp][g];
#pragma unroll
            for (int d = 0; d < DPL; ++d) o[g][d] *= c;
        }
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            float vf[DPL];
#pragma unroll
            for (int d = 0; d < DPL / 2; ++d) { vf[2 * d] = bf16_lo(vraw[j][d]); vf[2 * d + 1] = bf16_hi(vraw[j][d]); }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float pv = s_p[warp][j * G + g];
#pragma unroll
                for (int d = 0; d < DPL; ++d) o[g][d] = fmaf(pv, vf[d], o[g][d]);
            }
        }
        __syncwarp();
    };
    {
        unsigned k0[NB][DPL / 2], v0[NB][DPL / 2], k1[NB][DPL / 2], v1[NB][DPL / 2];
        int base = p0 + warp * NB;
        if (base < p1) {
            load_batch(k0, v0, base);
            while (true) {
                int next = base + 4 * NB;
                if (next < p1) load_batch(k1, v1, next);
                process_batch(k0, v0, base);
                base = next;
                if (base >= p1) break;
                next = base + 4 * NB;
                if (next < p1) load_batch(k0, v0, next);
                process_batch(k1, v1, base);
                base = next;
                if (base >= p1) break;
            }
        }
    }

    // the four warps' partial results meet in shared memory
    if ((lane & ((1 << SH) - 1)) == 0 && (lane >> SH) < G) {
        s_m[warp][lane >> SH] = m_run;
        s_l[warp][lane >> SH] = l_run;
    }
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int d = 0; d < DPL; ++d) s_o[warp][g][lane * DPL + d] = o[g][d];
    __syncthreads();

    attention_fold<G, HD>(p, split, kvh, b, tid, s_m, s_l, s_o, &s_last);
}

// ---- the same step on the tensor cores (head_dim 128) -----------------------------------------------------
//
// A warp takes tiles of 16 cached positions: the K and V rows of a tile (4 KB each, contiguous in the cache) come in
// by cp.async into a swizzled shared-memory tile, double buffered per warp.  Scores: S[heads x 16] = Q K^T with
// mma.sync.m16n8k16 (bf16 in, fp32 out), the query heads of the KV head in rows 0..G-1 of the 16-row operand.  The
// cache is bf16 already; q and the probabilities are fp32, so each goes in as two bf16 terms (x = hi + lo, the
// remainder of the first rounding), which keeps the products at fp32 accuracy.  The score fragment of a tile is
// exactly the A-operand fragment of P for O += P V, with V read through ldmatrix.trans.  Running maximum and sum per
// head as in the scalar kernel; the end of the CTA is shared with it.
constexpr int ATC_TILE = 16;                       // positions per tile
constexpr int ATC_TILE_BYTES = ATC_TILE * 256;     // one of K or V, head_dim 128 in bf16

__device__ __forceinline__ void atc_mma(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void atc_ldmatrix(unsigned (&r)[4], unsigned smem_addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr));
}
__device__ __forceinline__ void atc_ldmatrix_trans(unsigned (&r)[4], unsigned smem_addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr));
}
// x0, x1 as two packed bf16 pairs: hi holds the rounded values, lo the rounded remainders
__device__ __forceinline__ void atc_split(float x0, float x1, unsigned &hi, unsigned &lo)
{
    const __nv_bfloat16 h0 = __float2bfloat16_rn(x0), h1 = __float2bfloat16_rn(x1);
    hi = (unsigned)__bfloat16_as_ushort(h0) | ((unsigned)__bfloat16_as_ushort(h1) << 16);
    lo = pack_bf16(x0 - __bfloat162float(h0), x1 - __bfloat162float(h1));
}

template <int G>
__global__ void __launch_bounds__(128, 3) attention_decode_tc_kernel(const AttnParams p)
{
    constexpr int HD = 128;
    constexpr float NEG_INF = -3.0e38f;
    static_assert(G >= 1 && G <= 8, "query heads per KV head sit in rows 0..7 of the operand");

    extern __shared__ __align__(128) unsigned char atc_smem[];   // [warp][buffer][K tile, V tile]
    __shared__ float s_m[4][8], s_l[4][8];
    __shared__ float s_o[4][G][HD];
    __shared__ unsigned s_last;

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tig = lane & 3;
    int L = p.pos[b] + 1;                        // keys including the new token
    if (L > p.max_seq) L = p.max_seq;
    if (L < 1) L = 1;
    const int chunk = (L + p.n_splits - 1) / p.n_splits;
    const int p0 = split * chunk;
    const int p1 = min(L, p0 + chunk);

    const size_t row0 = ((size_t)b * p.n_kv + kvh) * (size_t)p.max_seq;
    const unsigned char *kc = reinterpret_cast<const unsigned char *>(p.kcache + row0 * HD);
    const unsigned char *vc = reinterpret_cast<const unsigned char *>(p.vcache + row0 * HD);
    // the CTA whose range holds the new position appends it (rounded to the cache's bf16) before any tile is fetched
    if (p0 <= L - 1 && L - 1 < p1) {
        if (warp == 0) {
            const float *knew = p.qkv + (size_t)b * p.ldq + p.k_off + kvh * HD + lane * 4;
            const float *vnew = p.qkv + (size_t)b * p.ldq + p.v_off + kvh * HD + lane * 4;
            uint2 *kw = reinterpret_cast<uint2 *>(p.kcache + (row0 + (L - 1)) * HD) + lane;
            uint2 *vw = reinterpret_cast<uint2 *>(p.vcache + (row0 + (L - 1)) * HD) + lane;
            *kw = make_uint2(pack_bf16(knew[0], knew[1]), pack_bf16(knew[2], knew[3]));
            *vw = make_uint2(pack_bf16(vnew[0], vnew[1]), pack_bf16(vnew[2], vnew[3]));
            __threadfence();
        }
        __syncthreads();
    }

    // the query heads, scaled, as A-operand fragments: row g = head g (rows G..15 are zero), two bf16 terms each
    unsigned qhi[8][2], qlo[8][2];
    {
        const float *qrow = p.qkv + (size_t)b * p.ldq + (size_t)(kvh * G + (g < G ? g : 0)) * HD;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int d = ks * 16 + h * 8 + 2 * tig;
                const float x0 = g < G ? qrow[d] * p.scale : 0.0f, x1 = g < G ? qrow[d + 1] * p.scale : 0.0f;
                atc_split(x0, x1, qhi[ks][h], qlo[ks][h]);
            }
    }

    unsigned char *wbuf = atc_smem + (size_t)warp * 4 * ATC_TILE_BYTES;
    const unsigned wbuf_u32 = (unsigned)__cvta_generic_to_shared(wbuf);
    const int n_tiles = p1 > p0 ? (p1 - p0 + ATC_TILE - 1) / ATC_TILE : 0;

    // 16-byte pieces of a tile: piece id = row * 16 + c lands at row * 256 + ((c ^ (row & 7)) * 16); rows past the
    // range are zero-filled (their scores are masked, their values weigh nothing)
    auto fetch = [&](int tile, int buf) {
        const int base = p0 + tile * ATC_TILE;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int id = i * 32 + lane, row = id >> 4, c = id & 15;
            const int pos = base + row;
            const unsigned bytes = pos < p1 ? 16u : 0u;
            const size_t src = (size_t)(pos < p1 ? pos : p1 - 1) * 256 + (size_t)c * 16;
            const unsigned dst = wbuf_u32 + (unsigned)buf * 2 * ATC_TILE_BYTES + (unsigned)row * 256 + (unsigned)((c ^ (row & 7)) * 16);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(kc + src), "r"(bytes) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + ATC_TILE_BYTES), "l"(vc + src), "r"(bytes) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float m_run = NEG_INF, l_run = 0.0f;         // of head g (all four lanes of a row hold the same)
    float o[16][4];                              // [8-dim tile][fragment register]: rows g (registers 0, 1) carry head g
#pragma unroll
    for (int dn = 0; dn < 16; ++dn) o[dn][0] = o[dn][1] = o[dn][2] = o[dn][3] = 0.0f;

    if (warp < n_tiles) fetch(warp, 0);
    int buf = 0;
    for (int tile = warp; tile < n_tiles; tile += 4, buf ^= 1) {
        if (tile + 4 < n_tiles) {
            fetch(tile + 4, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncwarp();
        const unsigned kt = wbuf_u32 + (unsigned)buf * 2 * ATC_TILE_BYTES, vt = kt + ATC_TILE_BYTES;
        const int lrow = lane & 7, lmat = lane >> 3;

        // ---- scores of 16 positions: two 8-position tiles ----
        float sc[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            // matrices: (positions 0-7, dims 16ks..+7), (0-7, +8..15), (8-15, ..+7), (8-15, +8..15)
            const int row = (lmat >> 1) * 8 + lrow, c = ks * 2 + (lmat & 1);
            unsigned kb[4];
            atc_ldmatrix(kb, kt + (unsigned)row * 256 + (unsigned)((c ^ (row & 7)) * 16));
            atc_mma(sc[0], qhi[ks][0], 0u, qhi[ks][1], 0u, kb[0], kb[1]);
            atc_mma(sc[0], qlo[ks][0], 0u, qlo[ks][1], 0u, kb[0], kb[1]);
            atc_mma(sc[1], qhi[ks][0], 0u, qhi[ks][1], 0u, kb[2], kb[3]);
            atc_mma(sc[1], qlo[ks][0], 0u, qlo[ks][1], 0u, kb[2], kb[3]);
        }
        // registers 0, 1 of tile nt: head g at positions base + 8 nt + 2 tig, + 1
        const int base = p0 + tile * ATC_TILE;
        float tmax = NEG_INF;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                if (base + nt * 8 + 2 * tig + e >= p1) sc[nt][e] = NEG_INF;
                tmax = fmaxf(tmax, sc[nt][e]);
            }
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
        const float m_new = fmaxf(m_run, tmax);    // the tile's first position always exists: finite
        const float corr = m_run > NEG_INF ? expf(m_run - m_new) : 0.0f;
        float pr[2][2], psum = 0.0f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                pr[nt][e] = sc[nt][e] > NEG_INF ? expf(sc[nt][e] - m_new) : 0.0f;
                psum += pr[nt][e];
            }
        psum += __shfl_xor_sync(0xffffffffu, psum, 1);
        psum += __shfl_xor_sync(0xffffffffu, psum, 2);
        l_run = l_run * corr + psum;
        m_run = m_new;
        // P as the A operand of the second product: k = position; rows 8..15 stay zero
        unsigned phi[2], plo[2];
        atc_split(pr[0][0], pr[0][1], phi[0], plo[0]);
        atc_split(pr[1][0], pr[1][1], phi[1], plo[1]);

        // ---- O = O * corr + P V ----
#pragma unroll
        for (int dn = 0; dn < 16; dn += 2) {
            // matrices: (positions 0-7, dims 8dn..+7), (8-15, same), (0-7, next 8 dims), (8-15, next 8 dims); transposed
            const int row = (lmat & 1) * 8 + lrow, c = dn + (lmat >> 1);
            unsigned vb[4];
            atc_ldmatrix_trans(vb, vt + (unsigned)row * 256 + (unsigned)((c ^ (row & 7)) * 16));
            o[dn][0] *= corr; o[dn][1] *= corr;
            o[dn + 1][0] *= corr; o[dn + 1][1] *= corr;
            atc_mma(o[dn], phi[0], 0u, phi[1], 0u, vb[0], vb[1]);
            atc_mma(o[dn], plo[0], 0u, plo[1], 0u, vb[0], vb[1]);
            atc_mma(o[dn + 1], phi[0], 0u, phi[1], 0u, vb[2], vb[3]);
            atc_mma(o[dn + 1], plo[0], 0u, plo[1], 0u, vb[2], vb[3]);
        }
        __syncwarp();   // every lane is through with this buffer before the next fetch overwrites it
    }

    // the four warps' partial results meet in shared memory
    if (g < G) {
        if (tig == 0) { s_m[warp][g] = m_run; s_l[warp][g] = l_run; }
#pragma unroll
        for (int dn = 0; dn < 16; ++dn) {
            s_o[warp][g][dn * 8 + 2 * tig] = o[dn][0];
            s_o[warp][g][dn * 8 + 2 * tig + 1] = o[dn][1];
        }
    }
    __syncthreads();
    attention_fold<G, HD>(p, split, kvh, b, tid, s_m, s_l, s_o, &s_last);
}

size_t attention_scratch_bytes(size_t B, size_t n_heads, size_t n_kv, size_t head_dim, size_t n_splits)
{
    if (n_splits <= 1) return 256;
    return align_up(B * n_heads * n_splits * head_dim * 4, 256) + align_up(B * n_heads * n_splits * 8, 256) + align_up(B * n_kv * 4, 256);
}

// Splits per (sequence, KV head): one when the pairs alone fill the SMs, else about two CTAs per SM in all (more
// splits cost more in partial results and their fold than they gain in balance), at least 64 keys per split at the
// longest context.
int attention_splits(size_t B, size_t n_kv, size_t max_context)
{
    const size_t pairs = B * n_kv;
    if (pairs >= (size_t)device_sm_count()) return 1;   // a CTA per pair already fills the SMs: folding splits only costs
    size_t want = (2 * (size_t)device_sm_count() + pairs - 1) / pairs;
    const size_t by_len = max_context / 64 > 0 ? max_context / 64 : 1;
    if (want > by_len) want = by_len;
    if (want > 32) want = 32;
    if (want < 1) want = 1;
    return (int)want;
}

template <int G, int HD, int NB>
static bitnet_status_t launch_attention_t(const AttnParams &p, size_t B, uint32_t flags, cudaStream_t stream)
{
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attrs[1];
    cfg.gridDim = dim3((unsigned)p.n_splits, (unsigned)p.n_kv, (unsigned)B);
    cfg.blockDim = dim3(128);
    cfg.stream = stream;
    cfg.attrs = attrs;
    if (flags & BITNET_FLAG_PDL) {
        attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 1;
    }
    BITNET_CUDA(cudaLaunchKernelEx(&cfg, attention_decode_kernel<G, HD, NB>, p));
    return BITNET_OK;
}

template <int G>
static bitnet_status_t launch_attention_tc(const AttnParams &p, size_t B, uint32_t flags, cudaStream_t stream)
{
    const size_t smem = 4 * 4 * ATC_TILE_BYTES;   // four warps x two buffers x (K tile + V tile)
    {
        static std::mutex mu;
        static bool raised[64] = {false};
        int dev = 0;
        BITNET_CUDA(cudaGetDevice(&dev));
        const bool tracked = dev >= 0 && dev < 64;
        std::lock_guard<std::mutex> lock(mu);
        if (!tracked || !raised[dev]) {
            BITNET_CUDA(cudaFuncSetAttribute(attention_decode_tc_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            if (tracked) raised[dev] = true;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attrs[1];
    cfg.gridDim = dim3((unsigned)p.n_splits, (unsigned)p.n_kv, (unsigned)B);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attrs;
    if (flags & BITNET_FLAG_PDL) {
        attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 1;
    }
    BITNET_CUDA(cudaLaunchKernelEx(&cfg, attention_decode_tc_kernel<G>, p));
    return BITNET_OK;
}

bitnet_status_t launch_attention_decode(const float *qkv, size_t ldq, size_t k_off, size_t v_off, void *kcache, void *vcache,
                                        const int *pos, float *out, size_t B, size_t n_heads, size_t n_kv, size_t head_dim,
                                        size_t max_seq, int n_splits, void *scratch, size_t scratch_bytes, uint32_t flags,
                                        cudaStream_t stream)
{
    if (B == 0) return BITNET_OK;
    if (!qkv || !kcache || !vcache || !pos || !out) return fail(BITNET_ERR_NULL_POINTER, "attention: null buffer");
    if (n_kv == 0 || n_heads % n_kv) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "heads %zu must be a multiple of KV heads %zu", n_heads, n_kv);
    if (B > 65535 || n_kv > 65535) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "attention: batch or KV head count too large");
    const size_t G = n_heads / n_kv;
    if (n_splits < 1) n_splits = 1;
    if (n_splits > 1) {
        const size_t need = attention_scratch_bytes(B, n_heads, n_kv, head_dim, (size_t)n_splits);
        if (!scratch || scratch_bytes < need || (reinterpret_cast<uintptr_t>(scratch) & 255))
            return fail(BITNET_ERR_WORKSPACE, "attention needs %zu bytes of 256-byte aligned scratch", need);
    }
    if ((reinterpret_cast<uintptr_t>(kcache) | reinterpret_cast<uintptr_t>(vcache)) & 15)
        return fail(BITNET_ERR_INVALID_CONFIG, "KV cache must be 16-byte aligned");
    AttnParams p = {};
    p.qkv = qkv; p.ldq = (int)ldq; p.k_off = (int)k_off; p.v_off = (int)v_off;
    p.kcache = static_cast<__nv_bfloat16 *>(kcache); p.vcache = static_cast<__nv_bfloat16 *>(vcache);
    p.pos = pos; p.out = out;
    p.n_heads = (int)n_heads; p.n_kv = (int)n_kv; p.max_seq = (int)max_seq; p.n_splits = n_splits;
    p.scale = 1.0f / sqrtf((float)head_dim);
    if (n_splits > 1) {
        char *s = static_cast<char *>(scratch);
        p.part_o = reinterpret_cast<float *>(s);
        s += align_up(B * n_heads * n_splits * head_dim * 4, 256);
        p.part_ml = reinterpret_cast<float *>(s);
        s += align_up(B * n_heads * n_splits * 8, 256);
        p.counters = reinterpret_cast<unsigned *>(s);
    }
    // the tensor-core form from 64 (sequence, KV head) pairs on; below that its fixed cost per CTA (query fragments,
    // the first tile's round trip) outweighs the cheaper positions (measured: 14.3 against 12.5 us at 40 pairs)
    if (head_dim == 128 && B * n_kv >= 64 && (G == 1 || G == 2 || G == 4 || G == 8)) {
        if (G == 1) return launch_attention_tc<1>(p, B, flags, stream);
        if (G == 2) return launch_attention_tc<2>(p, B, flags, stream);
        if (G == 4) return launch_attention_tc<4>(p, B, flags, stream);
        return launch_attention_tc<8>(p, B, flags, stream);
    }
#define BITNET_ATTN_CASE(GV, HDV, NBV) \
    if (G == GV && head_dim == HDV) return launch_attention_t<GV, HDV, NBV>(p, B, flags, stream)
    BITNET_ATTN_CASE(1, 128, 8); BITNET_ATTN_CASE(2, 128, 8); BITNET_ATTN_CASE(4, 128, 8); BITNET_ATTN_CASE(8, 128, 4);
    BITNET_ATTN_CASE(1, 64, 8);  BITNET_ATTN_CASE(2, 64, 8);  BITNET_ATTN_CASE(4, 64, 8);  BITNET_ATTN_CASE(8, 64, 4);
#undef BITNET_ATTN_CASE
    return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "attention covers head_dim 64 or 128 and 1, 2, 4 or 8 query heads per KV head (got %zu, %zu)",
                head_dim, G);
}

// ---- token sampler ------------------------------------------------------------------------------------

struct SampleParams {
    const float *logits;   // [B, vocab]
    int vocab;
    int deterministic;
    float temperature;
    int top_k;             // 0 = off
    float top_p;           // >= 1 = off
    unsigned long long *rng;   // [B] generator states
    int *next;             // [B] sampled ids
    int *ids_feed;         // optional [B]: also receives the ids (the next step's input)
    int *pos;              // optional [B]: incremented (the token that produced these logits is cached now)
    int *history;          // optional [steps][B]: row `*step_counter` receives the ids
    int *step_counter;     // optional, incremented by CTA 0
    int eos_id;            // -1 = none
    int *finished;         // optional [B]: set once a sequence sampled eos_id; a finished sequence keeps emitting eos_id
};

__device__ __forceinline__ unsigned float_order_key(float f)
{
    const unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // monotone: a < b  <=>  key(a) < key(b)
}

// One CTA of 1024 threads per sequence.  A thread owns a contiguous run of the vocabulary, so the
// prefix sums of the draw follow index order.
__global__ void __launch_bounds__(1024) sample_kernel(const SampleParams p)
{
    __shared__ float s_f[32];
    __shared__ int s_i[32];
    __shared__ float s_bcast;
    __shared__ int s_ibcast;
    __shared__ float s_scan[1024];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float *row = p.logits + (size_t)b * p.vocab;
    const int per = (p.vocab + 1023) / 1024;
    const int i0 = min(p.vocab, tid * per), i1 = min(p.vocab, i0 + per);

    // ---- maximum and its first index (NaN never wins) ----
    float best = -INFINITY;
    int besti = 0x7fffffff;
    for (int i = i0; i < i1; ++i) {
        const float v = __ldg(row + i);
        if (v > best) { best = v; besti = i; }
    }
    if (besti == 0x7fffffff && i0 < i1) besti = i0;   // a run of NaN or -inf: its first index stands in
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
        if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
    }
    if (lane == 0) { s_f[warp] = best; s_i[warp] = besti; }
    __syncthreads();
    if (warp == 0) {
        best = s_f[lane]; besti = s_i[lane];
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
            if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
        }
        if (lane == 0) { s_bcast = best; s_ibcast = besti == 0x7fffffff ? 0 : besti; }
    }
    __syncthreads();
    const float zmax_raw = s_bcast;
    int choice = s_ibcast;

    auto block_sum = [&](float v) {   // fixed order: lane tree, then the warps in turn
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        __syncthreads();
        if (lane == 0) s_f[warp] = v;
        __syncthreads();
        float t = 0.0f;
#pragma unroll
        for (int w = 0; w < 32; ++w) t += s_f[w];
        return t;
    };

    if (!p.deterministic) {
        const float temp = p.temperature;
        const float zmax = zmax_raw / temp;
        // keep-threshold on the order key of z = logit / temperature: the k-th largest value (top-k), then the
        // largest value whose "at least as likely" set reaches top_p of the probability mass (top-p);
        // ties with the threshold are kept, as a sort-and-cut that keeps equal values would
        unsigned thr_key = 0u;
        if (p.top_k > 0 && p.top_k < p.vocab) {
            unsigned lo = 0u, hi = 0xffffffffu;   // largest key with count(key(z) >= key) >= k
            while (lo < hi) {
                const unsigned mid = lo + (unsigned)(((unsigned long long)hi - lo + 1ull) >> 1);
                float cnt = 0.0f;
                for (int i = i0; i < i1; ++i) cnt += float_order_key(__ldg(row + i) / temp) >= mid ? 1.0f : 0.0f;
                if (block_sum(cnt) >= (float)p.top_k) lo = mid; else hi = mid - 1u;
            }
            thr_key = lo;
        }
        float total = 0.0f;
        {
            float part = 0.0f;
            for (int i = i0; i < i1; ++i) {
                const float z = __ldg(row + i) / temp;
                if (float_order_key(z) >= thr_key) part += expf(z - zmax);
            }
            total = block_sum(part);
        }
        if (p.top_p < 1.0f) {
            const float target = p.top_p * total;
            unsigned lo = thr_key, hi = float_order_key(zmax);   // largest key whose kept mass still reaches the target
            while (lo < hi) {
                const unsigned mid = lo + (unsigned)(((unsigned long long)hi - lo + 1ull) >> 1);
                float part = 0.0f;
                for (int i = i0; i < i1; ++i) {
                    const float z = __ldg(row + i) / temp;
                    if (float_order_key(z) >= mid) part += expf(z - zmax);
                }
                if (block_sum(part) >= target) lo = mid; else hi = mid - 1u;
            }
            thr_key = lo;
            float part = 0.0f;
            for (int i = i0; i < i1; ++i) {
                const float z = __ldg(row + i) / temp;
                if (float_order_key(z) >= thr_key) part += expf(z - zmax);
            }
            total = block_sum(part);
        }
        // the draw: the reference's linear congruential generator (sampling.rs:273-276), 24 bits of it as u in [0, 1)
        unsigned long long st = p.rng[b];
        st = st * 1103515245ull + 12345ull;
        const float u = (float)((st / 65536ull) & 0xffffffull) * (1.0f / 16777216.0f);
        const float target = u * total;
        // inclusive prefix sums of the kept probabilities in index order: per-thread runs, then a scan of the run sums
        float mine = 0.0f;
        for (int i = i0; i < i1; ++i) {
            const float z = __ldg(row + i) / temp;
            if (float_order_key(z) >= thr_key) mine += expf(z - zmax);
        }
        __syncthreads();
        s_scan[tid] = mine;
        __syncthreads();
        if (tid == 0) {
            float run = 0.0f;
            int owner = -1;
            float before = 0.0f;
            for (int t = 0; t < 1024; ++t) {
                const float next = run + s_scan[t];
                if (owner < 0 && next > target && s_scan[t] > 0.0f) { owner = t; before = run; }
                run = next;
            }
            if (owner < 0) {   // rounding left the target at or past the total: the last thread that kept anything owns it
                run = 0.0f;
                for (int t = 0; t < 1024; ++t) { if (s_scan[t] > 0.0f) { owner = t; before = run; } run += s_scan[t]; }
            }
            s_ibcast = owner;
            s_bcast = before;
        }
        __syncthreads();
        if (tid == s_ibcast) {
            float run = s_bcast;
            int pick = -1, last_kept = -1;
            for (int i = i0; i < i1; ++i) {
                const float z = __ldg(row + i) / temp;
                if (float_order_key(z) >= thr_key) {
                    run += expf(z - zmax);
                    last_kept = i;
                    if (run > target) { pick = i; break; }
                }
            }
            s_ibcast = pick >= 0 ? pick : last_kept;
            p.rng[b] = st;
        }
        __syncthreads();
        choice = s_ibcast;
    }

    if (tid == 0) {
        if (p.finished) {
            if (p.finished[b]) choice = p.eos_id;
            else if (p.eos_id >= 0 && choice == p.eos_id) p.finished[b] = 1;
        }
        p.next[b] = choice;
        if (p.ids_feed) p.ids_feed[b] = choice;
        if (p.pos) p.pos[b] += 1;
        if (p.history && p.step_counter) p.history[(size_t)(*p.step_counter) * gridDim.x + b] = choice;
    }
}

// The step counter that addresses the history rows is advanced by its own one-thread launch, after every
// CTA of the sampler has read it.
__global__ void advance_step_kernel(int *step_counter)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 0 && blockIdx.x == 0) *step_counter += 1;
}

bitnet_status_t launch_sample(const float *logits, size_t B, size_t vocab, const bitnet_sampling_config &cfg,
                              unsigned long long *rng, int *next, int *ids_feed, int *pos, int *history, int *step_counter,
                              int eos_id, int *finished, uint32_t flags, cudaStream_t stream)
{
    if (B == 0) return BITNET_OK;
    if (!logits || !next) return fail(BITNET_ERR_NULL_POINTER, "sampler: null buffer");
    if (vocab == 0 || vocab > (1u << 30)) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "sampler: vocabulary size %zu", vocab);
    if (!cfg.deterministic) {
        if (!(cfg.temperature > 0.0f)) return fail(BITNET_ERR_INVALID_CONFIG, "Temperature must be positive");   // sampling.rs:183-185
        if (!rng) return fail(BITNET_ERR_NULL_POINTER, "sampler: generator states missing");
    }
    SampleParams p = {};
    p.logits = logits; p.vocab = (int)vocab; p.deterministic = cfg.deterministic ? 1 : 0;
    p.temperature = cfg.temperature; p.top_k = (int)cfg.top_k; p.top_p = cfg.top_p;
    p.rng = rng; p.next = next; p.ids_feed = ids_feed; p.pos = pos; p.history = history; p.step_counter = step_counter;
    p.eos_id = eos_id; p.finished = finished;
    cudaLaunchConfig_t lc = {};
    cudaLaunchAttribute attrs[1];
    lc.gridDim = dim3((unsigned)B);
    lc.blockDim = dim3(1024);
    lc.stream = stream;
    lc.attrs = attrs;
    if (flags & BITNET_FLAG_PDL) {
        attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[0].val.programmaticStreamSerializationAllowed = 1;
        lc.numAttrs = 1;
    }
    BITNET_CUDA(cudaLaunchKernelEx(&lc, sample_kernel, p));
    if (step_counter) {
        lc.gridDim = dim3(1);
        lc.blockDim = dim3(32);
        BITNET_CUDA(cudaLaunchKernelEx(&lc, advance_step_kernel, step_counter));
    }
    return BITNET_OK;
}

__global__ void seed_rng_kernel(unsigned long long *rng, int B, unsigned long long seed)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < B) rng[i] = seed + (unsigned long long)i;   // BatchSampler::new, sampling.rs:419-426: base seed + sequence index
}

bitnet_status_t launch_seed_rng(unsigned long long *rng, size_t B, unsigned long long seed, cudaStream_t stream)
{
    if (B == 0) return BITNET_OK;
    seed_rng_kernel<<<(unsigned)((B + 255) / 256), 256, 0, stream>>>(rng, (int)B, seed);
    return check_launch("seed_rng_kernel");
}

}  // namespace bitnet
