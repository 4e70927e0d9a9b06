/*
 * CPU oracle for the BitLinear forward hot path -- TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the reference's CPU algorithm for the path
 *   per-token absmax int8 quantisation -> 2-bit ternary unpack ->
 *   int8 x ternary contraction (int32 accumulation) -> dequantise.
 * It exists to CHECK the CUDA kernels (tests/, the smoke run and the CPU
 * baseline leg of the benchmark).  Nothing in the product path may call it.
 *
 * Pinning status: the pieces (packing layout, unpack, scalar ternary GEMV/GEMM,
 * half-away rounding, ReLU^2) are pinned by the reference's own known-answer
 * tests, restated in tests/test_oracle_pins.py.  The reference holds no test
 * that pins a fused quantise->contract->dequantise output, and the reference
 * (Rust) cannot be built in an image without cargo/rustc, so for the fused
 * path as a whole: PARITY UNPINNED.
 *
 * Every function cites the reference file:line it follows (paths are relative
 * to the reference project root).
 */
#ifndef BITLINEAR_ORACLE_H
#define BITLINEAR_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Policy for the invalid 2-bit code 3 (the reference's decoders disagree). */
enum {
    ORC_CODE3_ZERO = 0,   /* gguf.rs:1139, weight_conversion.rs:179-182, simd/packing.rs:508-513 */
    ORC_CODE3_PLUS1 = 1,  /* bitnet-cuda w2a8_gemv.cu:38-41, w2a8_gemv.rs:299-305 (clamp) */
    ORC_CODE3_PLUS2 = 2   /* quantization/packing.rs:392 (code-1 with no clamp) */
};

/* --- layout ------------------------------------------------------------- */
size_t orc_packed_len(size_t n_values);
void orc_pack_bits(const uint8_t *values, size_t n, unsigned bits, uint8_t *out);
void orc_unpack_bits(const uint8_t *packed, size_t n_packed, unsigned bits,
                     size_t n_values, uint8_t *out);
void orc_pack_ternary(const int8_t *w, size_t n, uint8_t *out, size_t *padding);
void orc_unpack_ternary(const uint8_t *packed, size_t n_values, int8_t *out, int code3_policy);

/* --- scalar helpers ------------------------------------------------------ */
float orc_round_half_away(float x);
float orc_round_clip(float x, float lo, float hi);
void orc_relu2(const float *x, float *y, size_t n);

/* --- reference scalar kernels (f32) --------------------------------------- */
void orc_ternary_gemv_f32(const int8_t *a, const float *x, float *y,
                          size_t m, size_t k, float scale);
void orc_ternary_gemm_f32(const int8_t *a, const float *b, float *c,
                          size_t m, size_t k, size_t n, float scale);

/* --- the fused path ------------------------------------------------------ */
void orc_quantize_activations(const float *x, size_t M, size_t K,
                              int8_t *q, float *a_scale, float *fake_quant);
void orc_contract_i32(const int8_t *w, const int8_t *q, int32_t *acc,
                      size_t M, size_t K, size_t N);
void orc_dequantize(const int32_t *acc, const float *a_scale, float w_scale,
                    float *y, size_t M, size_t N);
void orc_bitlinear_forward(const uint8_t *wp, float w_scale, const float *x,
                           size_t M, size_t K, size_t N,
                           float *y, int8_t *q_out, float *a_scale_out, int32_t *acc_out);
void orc_bitlinear_forward_float_order(const uint8_t *wp, float w_scale, const float *x,
                                       size_t M, size_t K, size_t N, float *y);
void orc_w2a8_gemv(const uint8_t *wp, const int8_t *a, int32_t *out, size_t n_out, size_t k_in);
void orc_gate_relu2(const float *up, const float *gate, float *h, size_t n);
void orc_ffn_forward(const uint8_t *wp_gate, float s_gate, const uint8_t *wp_up, float s_up,
                     const uint8_t *wp_down, float s_down, const float *x,
                     size_t M, size_t hidden, size_t ffn, float *y, float *h_out);

/* --- weight preparation --------------------------------------------------- */
float orc_absmean_quantize_weights(const float *w, size_t n, int8_t *t);

/* --- threaded forms for timing the CPU baseline ---------------------------- */
int orc_max_threads(void);
void orc_bitlinear_forward_mt(const uint8_t *wp, float w_scale, const float *x,
                              size_t M, size_t K, size_t N, float *y, int threads);

/* --- seeded synthetic inputs ----------------------------------------------- */
uint64_t orc_splitmix64(uint64_t z);
void orc_gen_ternary(uint64_t seed, uint64_t tensor_id, size_t n, int8_t *w);
void orc_gen_ternary_packed(uint64_t seed, uint64_t tensor_id, size_t n, uint8_t *packed);
void orc_gen_activations(uint64_t seed, uint64_t tensor_id, size_t n, float *x);
float orc_gen_weight_scale(uint64_t seed, uint64_t tensor_id, size_t K);

#ifdef __cplusplus
}
#endif
#endif
