/*
 * CPU oracle for the BitLinear forward hot path -- TEST INFRASTRUCTURE ONLY.
 * See bitlinear_oracle.h for scope and pinning status (fused path: PARITY UNPINNED).
 *
 * Build with -ffp-contract=off and without -ffast-math: the division, the
 * multiply and the rounding in the activation quantiser must stay separately
 * rounded IEEE fp32 operations, as they are in the reference's Rust.
 */
#include "bitlinear_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline size_t nz(size_t n) { return n > 0 ? n : 1; }

/* ------------------------------------------------------------------------ */
/* layout                                                                    */
/* ------------------------------------------------------------------------ */

/* bitnet-quant/src/quantization/utils.rs:434-451: values.chunks(4) -> one byte each. */
size_t orc_packed_len(size_t n_values) { return (n_values + 3) / 4; }

/* BitUtils::pack_bits, bitnet-quant/src/quantization/utils.rs:434-451.
 * value i of a chunk goes to bits [i*bits, (i+1)*bits), least significant first. */
void orc_pack_bits(const uint8_t *values, size_t n, unsigned bits, uint8_t *out)
{
    if (bits >= 8) { memcpy(out, values, n); return; }
    const size_t per_byte = 8 / bits;
    const uint8_t mask = (uint8_t)((1u << bits) - 1u);
    size_t o = 0;
    for (size_t start = 0; start < n; start += per_byte, ++o) {
        uint8_t byte = 0;
        for (size_t i = 0; i < per_byte && start + i < n; ++i)
            byte |= (uint8_t)((values[start + i] & mask) << (i * bits));
        out[o] = byte;
    }
}

/* BitUtils::unpack_bits, bitnet-quant/src/quantization/utils.rs:454-475. */
void orc_unpack_bits(const uint8_t *packed, size_t n_packed, unsigned bits,
                     size_t n_values, uint8_t *out)
{
    if (bits >= 8) { memcpy(out, packed, n_values < n_packed ? n_values : n_packed); return; }
    const size_t per_byte = 8 / bits;
    const uint8_t mask = (uint8_t)((1u << bits) - 1u);
    size_t o = 0;
    for (size_t b = 0; b < n_packed && o < n_values; ++b)
        for (size_t i = 0; i < per_byte && o < n_values; ++i)
            out[o++] = (uint8_t)((packed[b] >> (i * bits)) & mask);
}

/* BitPacked2BitPacker::pack, bitnet-quant/src/quantization/packing.rs:352-388:
 * code = w + 1, four codes per byte, metadata.padding = (4 - n % 4) % 4. */
void orc_pack_ternary(const int8_t *w, size_t n, uint8_t *out, size_t *padding)
{
    size_t o = 0;
    for (size_t start = 0; start < n; start += 4, ++o) {
        uint8_t byte = 0;
        for (size_t i = 0; i < 4 && start + i < n; ++i)
            byte |= (uint8_t)((((uint8_t)(w[start + i] + 1)) & 3u) << (2 * i));
        out[o] = byte;
    }
    if (padding) *padding = (n % 4) ? 4 - (n % 4) : 0;
}

/* BitPacked2BitPacker::unpack, packing.rs:390-394 (code - 1), with the policy for
 * the invalid code 3 chosen by the caller (see the enum in the header). */
void orc_unpack_ternary(const uint8_t *packed, size_t n_values, int8_t *out, int code3_policy)
{
    for (size_t i = 0; i < n_values; ++i) {
        const unsigned code = (packed[i >> 2] >> (2 * (i & 3))) & 3u;
        int8_t v = (int8_t)((int)code - 1);
        if (code == 3u) {
            if (code3_policy == ORC_CODE3_ZERO) v = 0;
            else if (code3_policy == ORC_CODE3_PLUS1) v = 1;
        }
        out[i] = v;
    }
}

/* ------------------------------------------------------------------------ */
/* scalar helpers                                                            */
/* ------------------------------------------------------------------------ */

/* Rust f32::round: half away from zero (ternary_operations.rs:158; pinned by
 * bitnet-quant/src/quantization/utils.rs:609-631).  C roundf has the same rule. */
float orc_round_half_away(float x) { return roundf(x); }

/* QuantizationUtils::round_clip, bitnet-quant/src/quantization/utils.rs:391-393. */
float orc_round_clip(float x, float lo, float hi)
{
    float r = roundf(x);
    if (r < lo) r = lo;
    if (r > hi) r = hi;
    return r;
}

/* ReLUSquaredActivation::forward, bitnet-inference/src/engine/transformer_layers.rs:307-315:
 * maximum(x, 0) then powf(2.0) == r*r. */
void orc_relu2(const float *x, float *y, size_t n)
{
    for (size_t i = 0; i < n; ++i) {
        const float r = x[i] > 0.0f ? x[i] : 0.0f;
        y[i] = r * r;
    }
}

/* ------------------------------------------------------------------------ */
/* reference scalar kernels                                                  */
/* ------------------------------------------------------------------------ */

/* ternary_gemv_scalar, bitnet-quant/src/simd/matrix.rs:471-490. */
void orc_ternary_gemv_f32(const int8_t *a, const float *x, float *y,
                          size_t m, size_t k, float scale)
{
    for (size_t i = 0; i < m; ++i) {
        float sum = 0.0f;
        for (size_t kk = 0; kk < k; ++kk) sum += (float)a[i * k + kk] * x[kk];
        y[i] = sum * scale;
    }
}

/* ternary_gemm_scalar, bitnet-quant/src/simd/matrix.rs:256-282 (A ternary [m,k], B [k,n]). */
void orc_ternary_gemm_f32(const int8_t *a, const float *b, float *c,
                          size_t m, size_t k, size_t n, float scale)
{
    for (size_t i = 0; i < m * n; ++i) c[i] = 0.0f;
    for (size_t i = 0; i < m; ++i)
        for (size_t kk = 0; kk < k; ++kk) {
            const int8_t av = a[i * k + kk];
            if (av != 0) {
                const float sa = (float)av * scale;
                for (size_t j = 0; j < n; ++j) c[i * n + j] += sa * b[kk * n + j];
            }
        }
}

/* ------------------------------------------------------------------------ */
/* the fused path                                                            */
/* ------------------------------------------------------------------------ */

/* TernaryProcessor::quantize_activations, bitnet-inference/src/engine/ternary_operations.rs:130-163.
 * Per row: absmax by a max-fold from 0.0 (:144-146, NaN is ignored like f32::max),
 * scale = 127/absmax or 1 (:148-152), q = clamp(round(x*scale), -128, 127) (:157-160).
 * The reference returns q/scale (:162); the true int8 values and the dequantisation
 * factor a_scale = absmax/127 (1 when absmax == 0) are what the fused path carries. */
void orc_quantize_activations(const float *x, size_t M, size_t K,
                              int8_t *q, float *a_scale, float *fake_quant)
{
    for (size_t m = 0; m < M; ++m) {
        const float *row = x + m * K;
        float absmax = 0.0f;
        for (size_t k = 0; k < K; ++k) {
            const float a = fabsf(row[k]);
            if (a > absmax) absmax = a;
        }
        const float scale = absmax > 0.0f ? 127.0f / absmax : 1.0f;
        if (a_scale) a_scale[m] = absmax > 0.0f ? absmax / 127.0f : 1.0f;
        for (size_t k = 0; k < K; ++k) {
            const float t = row[k] * scale;
            float r = roundf(t);
            if (r < -128.0f) r = -128.0f;
            if (r > 127.0f) r = 127.0f;
            if (!(r == r)) r = 0.0f; /* NaN input: Rust `as i8` of NaN saturates to 0 */
            if (q) q[m * K + k] = (int8_t)r;
            if (fake_quant) fake_quant[m * K + k] = r / scale;
        }
    }
}

/* acc[m,n] = sum_k W[n,k] * q[m,k] in int32.  Index convention of the legacy
 * kernel (bitnet-cuda/src/kernels/w2a8_gemv.cu:100-106) and of
 * ternary_gemv_scalar (matrix.rs:471-490); loop nest of
 * ternary_matmul_generic (ternary_operations.rs:314-330), which accumulates the
 * same integers in f32. */
void orc_contract_i32(const int8_t *w, const int8_t *q, int32_t *acc,
                      size_t M, size_t K, size_t N)
{
    for (size_t n = 0; n < N; ++n)
        for (size_t m = 0; m < M; ++m) {
            int32_t s = 0;
            for (size_t k = 0; k < K; ++k) s += (int32_t)w[n * K + k] * (int32_t)q[m * K + k];
            acc[m * N + n] = s;
        }
}

/* y[m,n] = float(acc) * (w_scale * a_scale[m]); formula of the reference's Metal
 * bitlinear_forward (bitnet-metal/shaders/bitlinear_operations.metal:30). */
void orc_dequantize(const int32_t *acc, const float *a_scale, float w_scale,
                    float *y, size_t M, size_t N)
{
    for (size_t m = 0; m < M; ++m) {
        const float s = w_scale * a_scale[m];
        for (size_t n = 0; n < N; ++n) y[m * N + n] = (float)acc[m * N + n] * s;
    }
}

void orc_bitlinear_forward(const uint8_t *wp, float w_scale, const float *x,
                           size_t M, size_t K, size_t N,
                           float *y, int8_t *q_out, float *a_scale_out, int32_t *acc_out)
{
    int8_t *w = (int8_t *)malloc(nz(N * K));
    int8_t *q = q_out ? q_out : (int8_t *)malloc(nz(M * K));
    float *as = a_scale_out ? a_scale_out : (float *)malloc(sizeof(float) * nz(M));
    int32_t *acc = acc_out ? acc_out : (int32_t *)malloc(sizeof(int32_t) * nz(M * N));
    orc_unpack_ternary(wp, N * K, w, ORC_CODE3_ZERO);
    orc_quantize_activations(x, M, K, q, as, NULL);
    orc_contract_i32(w, q, acc, M, K, N);
    if (y) orc_dequantize(acc, as, w_scale, y, M, N);
    free(w);
    if (!q_out) free(q);
    if (!a_scale_out) free(as);
    if (!acc_out) free(acc);
}

/* Informational: the reference's own float order.  Fake-quantised activations
 * q/scale (ternary_operations.rs:162) summed sequentially in f32 with
 * tern(w) in {-1,0,1} (:314-330), then times the weight scale. */
void orc_bitlinear_forward_float_order(const uint8_t *wp, float w_scale, const float *x,
                                       size_t M, size_t K, size_t N, float *y)
{
    int8_t *w = (int8_t *)malloc(nz(N * K));
    float *fq = (float *)malloc(sizeof(float) * nz(M * K));
    orc_unpack_ternary(wp, N * K, w, ORC_CODE3_ZERO);
    orc_quantize_activations(x, M, K, NULL, NULL, fq);
    for (size_t n = 0; n < N; ++n)
        for (size_t m = 0; m < M; ++m) {
            float sum = 0.0f;
            for (size_t k = 0; k < K; ++k) sum += (float)w[n * K + k] * fq[m * K + k];
            y[m * N + n] = sum * w_scale;
        }
    free(w);
    free(fq);
}

/* Intended semantics of the legacy entry point (w2a8_gemv.cu:100-106):
 * out[n] = sum_k (code(W[n,k]) - 1) * a[k] for ONE token, canonical flat layout. */
void orc_w2a8_gemv(const uint8_t *wp, const int8_t *a, int32_t *out, size_t n_out, size_t k_in)
{
    int8_t *w = (int8_t *)malloc(nz(n_out * k_in));
    orc_unpack_ternary(wp, n_out * k_in, w, ORC_CODE3_ZERO);
    orc_contract_i32(w, a, out, 1, k_in, n_out);
    free(w);
}

/* FeedForwardNetwork::forward gating, transformer_layers.rs:613-618: up * relu(gate)^2. */
void orc_gate_relu2(const float *up, const float *gate, float *h, size_t n)
{
    for (size_t i = 0; i < n; ++i) {
        const float r = gate[i] > 0.0f ? gate[i] : 0.0f;
        h[i] = up[i] * (r * r);
    }
}

/* FeedForwardNetwork::forward, transformer_layers.rs:603-623: up, gate -> gating -> down,
 * every projection a BitLinear that re-quantises its own input per token. */
void orc_ffn_forward(const uint8_t *wp_gate, float s_gate, const uint8_t *wp_up, float s_up,
                     const uint8_t *wp_down, float s_down, const float *x,
                     size_t M, size_t hidden, size_t ffn, float *y, float *h_out)
{
    float *g = (float *)malloc(sizeof(float) * M * ffn);
    float *u = (float *)malloc(sizeof(float) * M * ffn);
    float *h = h_out ? h_out : (float *)malloc(sizeof(float) * M * ffn);
    orc_bitlinear_forward(wp_up, s_up, x, M, hidden, ffn, u, NULL, NULL, NULL);
    orc_bitlinear_forward(wp_gate, s_gate, x, M, hidden, ffn, g, NULL, NULL, NULL);
    orc_gate_relu2(u, g, h, M * ffn);
    orc_bitlinear_forward(wp_down, s_down, h, M, ffn, hidden, y, NULL, NULL, NULL);
    free(g);
    free(u);
    if (!h_out) free(h);
}

/* ------------------------------------------------------------------------ */
/* weight preparation                                                        */
/* ------------------------------------------------------------------------ */

/* absmean_quantize_weights, bitnet-quant/src/quantization/weights.rs:807-857:
 * threshold = 0.7 * mean|w| (:829-831); t = sign(w) * (|w| > threshold) (:482-496);
 * scale = sum(w*t)/sum(t*t), 1.0 if the denominator is below f32 epsilon (:546-559).
 * The reductions are candle's; they are restated here in double and the result cast,
 * which is why tests compare this scale with a tolerance, not bit-exactly. */
float orc_absmean_quantize_weights(const float *w, size_t n, int8_t *t)
{
    double sum_abs = 0.0;
    for (size_t i = 0; i < n; ++i) sum_abs += fabs((double)w[i]);
    const float mean_abs = n ? (float)(sum_abs / (double)n) : 0.0f;
    const float thr = mean_abs * 0.7f;
    double num = 0.0, den = 0.0;
    for (size_t i = 0; i < n; ++i) {
        const float a = fabsf(w[i]);
        int8_t v = 0;
        if (a > thr) v = (int8_t)((w[i] > 0.0f) - (w[i] < 0.0f));
        t[i] = v;
        num += (double)w[i] * (double)v;
        den += (double)v * (double)v;
    }
    if (fabs(den) < 1.1920929e-07) return 1.0f;
    return (float)(num / den);
}

/* ------------------------------------------------------------------------ */
/* threaded forms, for timing only                                           */
/* ------------------------------------------------------------------------ */

int orc_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Same arithmetic as orc_bitlinear_forward, rows of W spread over host threads.
 * The reference loop (ternary_operations.rs:314-330) is single-threaded; the
 * threaded form exists so the CPU baseline can use every host core. */
void orc_bitlinear_forward_mt(const uint8_t *wp, float w_scale, const float *x,
                              size_t M, size_t K, size_t N, float *y, int threads)
{
    int8_t *q = (int8_t *)malloc(nz(M * K));
    float *as = (float *)malloc(sizeof(float) * nz(M));
    orc_quantize_activations(x, M, K, q, as, NULL);
    if (threads < 1) threads = 1;
#ifdef _OPENMP
#pragma omp parallel num_threads(threads)
#endif
    {
        int8_t *wrow = (int8_t *)malloc(nz(K));
#ifdef _OPENMP
#pragma omp for schedule(static)
#endif
        for (long n = 0; n < (long)N; ++n) {
            const size_t base = (size_t)n * K;
            for (size_t k = 0; k < K; ++k) {
                const size_t i = base + k;
                const unsigned code = (wp[i >> 2] >> (2 * (i & 3))) & 3u;
                wrow[k] = code == 3u ? 0 : (int8_t)((int)code - 1);
            }
            for (size_t m = 0; m < M; ++m) {
                const int8_t *qr = q + m * K;
                int32_t s = 0;
                for (size_t k = 0; k < K; ++k) s += (int32_t)wrow[k] * (int32_t)qr[k];
                y[m * N + (size_t)n] = (float)s * (w_scale * as[m]);
            }
        }
        free(wrow);
    }
    free(q);
    free(as);
}

/* ------------------------------------------------------------------------ */
/* seeded synthetic inputs                                                   */
/* ------------------------------------------------------------------------ */
/* Counter-based: element i of tensor `tensor_id` under `seed` depends only on
 * (seed, tensor_id, i), so any slice can be generated independently.
 * Weights: P(-1)=0.3, P(0)=0.4, P(+1)=0.3.  Activations: N(0,1) by Box-Muller
 * in double, each multiplied by 20 with probability 0.001. */

uint64_t orc_splitmix64(uint64_t z)
{
    z += 0x9e3779b97f4a7c15ULL;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
    return z ^ (z >> 31);
}

static inline uint64_t tensor_key(uint64_t seed, uint64_t tensor_id)
{
    return orc_splitmix64(orc_splitmix64(seed) ^ (tensor_id * 0xd1342543de82ef95ULL));
}

static inline double u01(uint64_t r) { return ((double)(r >> 11) + 0.5) * (1.0 / 9007199254740992.0); }

static inline int8_t ternary_from(uint64_t r)
{
    const double u = u01(r);
    return u < 0.3 ? (int8_t)-1 : (u < 0.7 ? (int8_t)0 : (int8_t)1);
}

void orc_gen_ternary(uint64_t seed, uint64_t tensor_id, size_t n, int8_t *w)
{
    const uint64_t key = tensor_key(seed, tensor_id);
    for (size_t i = 0; i < n; ++i) w[i] = ternary_from(orc_splitmix64(key + (uint64_t)i));
}

void orc_gen_ternary_packed(uint64_t seed, uint64_t tensor_id, size_t n, uint8_t *packed)
{
    const uint64_t key = tensor_key(seed, tensor_id);
    const long nbytes = (long)orc_packed_len(n);
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
    for (long b = 0; b < nbytes; ++b) {
        uint8_t byte = 0;
        for (size_t j = 0; j < 4; ++j) {
            const size_t i = (size_t)b * 4 + j;
            if (i < n) byte |= (uint8_t)((uint8_t)(ternary_from(orc_splitmix64(key + (uint64_t)i)) + 1) << (2 * j));
        }
        packed[b] = byte;
    }
}

void orc_gen_activations(uint64_t seed, uint64_t tensor_id, size_t n, float *x)
{
    const uint64_t key = tensor_key(seed, tensor_id);
    for (size_t i = 0; i < n; ++i) {
        const uint64_t r1 = orc_splitmix64(key + (uint64_t)i);
        const uint64_t r2 = orc_splitmix64(r1);
        const uint64_t r3 = orc_splitmix64(r2);
        double z = sqrt(-2.0 * log(u01(r1))) * cos(6.283185307179586476925 * u01(r2));
        if (u01(r3) < 0.001) z *= 20.0;
        x[i] = (float)z;
    }
}

float orc_gen_weight_scale(uint64_t seed, uint64_t tensor_id, size_t K)
{
    const uint64_t key = tensor_key(seed, tensor_id ^ 0x5ca1ab1eULL);
    const double u = u01(orc_splitmix64(key));
    return (float)((0.5 + u) / sqrt((double)(K ? K : 1)));
}
