"""Pins the CPU oracle to every known-answer vector the reference's tests hold for
the BitLinear path (each test names the reference test it restates), then checks
the C oracle against an independent numpy restatement on seeded inputs."""
import numpy as np
import pytest

import oracle


# --- layout pins ---------------------------------------------------------------

def test_gguf_byte_0x24_decodes_minus1_0_1_minus1():
    # bitnet-inference/src/gguf.rs:2409-2438
    assert oracle.unpack_ternary([0b00100100], 4).tolist() == [-1, 0, 1, -1]


def test_weight_conversion_byte_0xE4_code3_is_zero():
    # bitnet-inference/src/engine/weight_conversion.rs:475-499
    assert oracle.unpack_ternary([0b11100100], 4).tolist() == [-1, 0, 1, 0]
    # the other two decoders of the reference, kept as selectable policies
    assert oracle.unpack_ternary([0b11100100], 4, oracle.CODE3_PLUS1).tolist() == [-1, 0, 1, 1]
    assert oracle.unpack_ternary([0b11100100], 4, oracle.CODE3_PLUS2).tolist() == [-1, 0, 1, 2]


def test_bit_packed_2bit_compression():
    # bitnet-quant/tests/packing_tests.rs:24-40
    w = [-1, 0, 1, -1, 0, 1, 0, 1]
    packed, pad = oracle.pack_ternary(w)
    assert packed.size == 2 and pad == 0
    assert oracle.unpack_ternary(packed, 8).tolist() == w


def test_bit_packed_2bit_with_padding():
    # bitnet-quant/tests/packing_tests.rs:42-53
    w = [-1, 0, 1]
    packed, pad = oracle.pack_ternary(w)
    assert packed.size == 1 and pad == 1
    assert oracle.unpack_ternary(packed, 3).tolist() == w
    assert packed[0] == (0 | (1 << 2) | (2 << 4))


def test_pack_bits_round_trip():
    # bitnet-quant/src/quantization/utils.rs:577-582
    v = [0, 1, 2, 3, 0, 1, 2, 3]
    p = oracle.pack_bits(v, 2)
    assert p.tolist() == [0b11100100, 0b11100100]
    assert oracle.unpack_bits(p, 2, 8).tolist() == v


@pytest.mark.parametrize("n", [32, 128 * 64, 512 * 256, 1024 * 512])
def test_mod3_pattern_round_trip(n):
    # bitnet-quant/tests/simd_unpacking_correctness_tests.rs:101-133 and :744-781
    w = (np.arange(n) % 3 - 1).astype(np.int8)
    packed, pad = oracle.pack_ternary(w)
    assert packed.size == (n + 3) // 4
    out = oracle.unpack_ternary(packed, n)
    assert np.array_equal(out, w)
    assert set(np.unique(out).tolist()) <= {-1, 0, 1}


def test_all_0x55_weights_are_zero():
    # bitnet-cuda/examples/w2a8_gemv_demo.rs:59-61: every code is 1, i.e. w == 0, so the
    # GEMV result must be 0 (the demo's printed expectation "~k" contradicts its own decode).
    n_out, k = 8, 64
    wp = np.full(n_out * k // 4, 0x55, dtype=np.uint8)
    a = np.ones(k, dtype=np.int8)
    assert np.array_equal(oracle.w2a8_gemv(wp, a, n_out), np.zeros(n_out, dtype=np.int32))


# --- arithmetic pins --------------------------------------------------------------

def test_ternary_matrix_vector():
    # bitnet-quant/src/simd/matrix.rs:531-558
    a = np.array([[1, -1, 0, 1], [0, 1, -1, 0], [-1, 0, 1, 1]], dtype=np.int8)
    y = oracle.ternary_gemv_f32(a, [2.0, 3.0, 1.0, -1.0], 1.0)
    assert y.tolist() == [-2.0, 2.0, -2.0]
    # the integer path gives the same numbers
    packed, _ = oracle.pack_ternary(a)
    assert oracle.w2a8_gemv(packed, [2, 3, 1, -1], 3).tolist() == [-2, 2, -2]


def test_ternary_matrix_multiply():
    # bitnet-quant/src/simd/matrix.rs:560-595
    a = np.array([[1, -1, 0], [0, 1, -1]], dtype=np.int8)
    b = np.array([[1, 2], [3, 4], [5, 6]], dtype=np.float32)
    assert oracle.ternary_gemm_f32(a, b, 1.0).tolist() == [[-2.0, -2.0], [-2.0, -2.0]]


def test_round_clip():
    # bitnet-quant/src/quantization/utils.rs:609-631
    rc = oracle.round_clip
    assert rc(1.7, -1, 1) == 1 and rc(-2.3, -1, 1) == -1 and rc(0.4, -1, 1) == 0
    assert rc(0.6, -1, 1) == 1 and rc(-0.6, -1, 1) == -1
    assert rc(0.5, -1, 1) == 1 and rc(-0.5, -1, 1) == -1        # half away from zero
    assert rc(1.5, -1, 1) == 1 and rc(-1.5, -1, 1) == -1
    assert rc(2.5, -8, 8) == 3 and rc(-2.5, -8, 8) == -3


def test_relu_squared():
    # bitnet-inference/src/engine/transformer_layers.rs:744-758
    assert oracle.relu2([2.0, -1.0, 0.0, 3.0]).tolist() == [4.0, 0.0, 0.0, 9.0]


def test_activation_quant_preserves_order_and_sign():
    # bitnet-inference/src/engine/ternary_operations.rs:444-461 (the reference's weak pin)
    x = np.array([[1.0, -2.0, 3.0, -4.0], [0.5, 0.0, -0.25, 4.0]], dtype=np.float32)
    q, s, fq = oracle.quantize_activations(x)
    assert np.all(np.sign(q) == np.sign(x))
    assert np.all(np.diff(np.argsort(x, axis=1), axis=1) == np.diff(np.argsort(fq, axis=1), axis=1))
    assert q[0].tolist() == [32, -64, 95, -127] and q[1, 3] == 127
    assert s[0] == np.float32(4.0) / np.float32(127.0)


# --- independent numpy restatement ---------------------------------------------------

def np_round_half_away(t):
    r = np.trunc(t)
    d = np.abs(t - r)
    return (r + np.where(d >= np.float32(0.5), np.sign(t), 0)).astype(np.float32)


def np_bitlinear(wp, w_scale, x, N):
    M, K = x.shape
    codes = (wp.reshape(-1)[:, None] >> (2 * np.arange(4, dtype=np.uint8))[None, :]) & 3
    w = codes.reshape(-1)[: N * K].astype(np.int32) - 1
    w[w == 2] = 0
    w = w.reshape(N, K)
    absmax = np.abs(x).max(axis=1).astype(np.float32)
    s = np.where(absmax > 0, np.float32(127.0) / np.where(absmax > 0, absmax, 1), np.float32(1.0)).astype(np.float32)
    t = (x * s[:, None]).astype(np.float32)
    q = np.clip(np_round_half_away(t), -128, 127).astype(np.int32)
    acc = q @ w.T
    a_scale = np.where(absmax > 0, absmax / np.float32(127.0), np.float32(1.0)).astype(np.float32)
    y = acc.astype(np.float32) * (np.float32(w_scale) * a_scale)[:, None]
    return y.astype(np.float32), q.astype(np.int8), a_scale, acc.astype(np.int32)


@pytest.mark.parametrize("M,K,N", [(1, 64, 16), (3, 130, 7), (8, 2560, 48), (5, 37, 29), (2, 1, 1)])
def test_oracle_matches_numpy_restatement(M, K, N):
    wp = oracle.gen_ternary_packed(7, 1, N * K)
    x = oracle.gen_activations(7, 2, (M, K))
    ws = oracle.gen_weight_scale(7, 1, K)
    ref = oracle.bitlinear_forward(wp, ws, x, N)
    y, q, a_scale, acc = np_bitlinear(wp, ws, x, N)
    assert np.array_equal(ref["q"], q)
    assert np.array_equal(ref["acc"], acc)
    assert np.array_equal(ref["a_scale"], a_scale)
    assert np.array_equal(ref["y"], y)


def test_quant_edge_cases():
    x = np.zeros((4, 8), dtype=np.float32)
    x[1, :] = [0.5, -0.5, 1.5, -1.5, 2.5, -2.5, 127.0, -127.0]      # scale == 1: exact ties
    x[2, 3] = 1e-30                                                   # tiny absmax
    x[3, :] = [3.0e38, -3.0e38, 1.0, -1.0, 0.0, 1e20, -1e20, 5.0]    # huge absmax
    q, s, _ = oracle.quantize_activations(x)
    assert np.all(q[0] == 0) and s[0] == 1.0
    assert q[1].tolist() == [1, -1, 2, -2, 3, -3, 127, -127]
    assert q[2, 3] == 127 and np.all(np.delete(q[2], 3) == 0)
    assert q[3, 0] == 127 and q[3, 1] == -127 and q[3, 2] == 0


def test_float_order_oracle_is_close():
    M, K, N = 4, 512, 64
    wp = oracle.gen_ternary_packed(3, 1, N * K)
    x = oracle.gen_activations(3, 2, (M, K))
    ws = oracle.gen_weight_scale(3, 1, K)
    y = oracle.bitlinear_forward(wp, ws, x, N)["y"]
    yf = oracle.bitlinear_forward_float_order(wp, ws, x, N)
    assert np.all(np.abs(y - yf) <= 1e-4 * np.abs(y).max(axis=1, keepdims=True))


def test_ffn_matches_composition():
    M, H, F = 3, 128, 192
    g = oracle.gen_ternary_packed(5, 1, F * H)
    u = oracle.gen_ternary_packed(5, 2, F * H)
    d = oracle.gen_ternary_packed(5, 3, H * F)
    x = oracle.gen_activations(5, 4, (M, H))
    sg, su, sd = (oracle.gen_weight_scale(5, i, k) for i, k in ((1, H), (2, H), (3, F)))
    y, h = oracle.ffn_forward(g, sg, u, su, d, sd, x, F)
    up = oracle.bitlinear_forward(u, su, x, F)["y"]
    gate = oracle.bitlinear_forward(g, sg, x, F)["y"]
    h2 = up * np.square(np.maximum(gate, 0)).astype(np.float32)
    assert np.array_equal(h, h2)
    assert np.array_equal(y, oracle.bitlinear_forward(d, sd, h2, H)["y"])


def test_generator_distribution_and_determinism():
    w = oracle.gen_ternary(0, 9, 200000)
    frac = [(w == v).mean() for v in (-1, 0, 1)]
    assert abs(frac[0] - 0.3) < 0.01 and abs(frac[1] - 0.4) < 0.01 and abs(frac[2] - 0.3) < 0.01
    assert np.array_equal(oracle.pack_ternary(w)[0], oracle.gen_ternary_packed(0, 9, 200000))
    x = oracle.gen_activations(0, 1, (200000,))
    assert abs(x.mean()) < 0.02 and 1.0 < x.std() < 1.5     # N(0,1) plus 0.1 % x20 outliers
    assert np.array_equal(x, oracle.gen_activations(0, 1, (200000,)))
    assert (np.abs(x) > 8).mean() > 1e-4


def test_absmean_weight_quantiser():
    # bitnet-quant/src/quantization/weights.rs:807-857
    rng = np.random.default_rng(0)
    w = rng.standard_normal((64, 128)).astype(np.float32)
    t, scale = oracle.absmean_quantize_weights(w)
    thr = np.abs(w).mean() * 0.7
    assert np.array_equal(t, (np.sign(w) * (np.abs(w) > thr)).astype(np.int8))
    assert scale == pytest.approx(float((w * t).sum() / (t * t).sum()), rel=1e-5)


# ---- decode-step restatements (oracle/decoder.py) ---------------------------------------------------

def test_sampler_generator_follows_the_reference_recurrence():
    # sampling.rs:273-276: state = state.wrapping_mul(1103515245).wrapping_add(12345); token = (state / 65536) % 1000
    from oracle import decoder as od
    s = 42
    seen = []
    for _ in range(4):
        s = od.lcg_next(s)
        seen.append((s // 65536) % 1000)
    assert s == (((((42 * 1103515245 + 12345) * 1103515245 + 12345) * 1103515245 + 12345) * 1103515245 + 12345) % (1 << 64))
    assert seen == [(((42 * 1103515245 + 12345) % (1 << 64)) // 65536) % 1000] + seen[1:]
    big = (1 << 64) - 1
    assert od.lcg_next(big) == (big * 1103515245 + 12345) % (1 << 64)          # wrapping arithmetic
    assert 0.0 <= od.lcg_uniform(s) < 1.0


def test_bf16_rounding_known_answers():
    from oracle import decoder as od
    x = np.array([1.0, 1.00390625, 1.001953125, 1.005859375, -2.5, 0.0], dtype=np.float32)
    # 1 + 2^-8 is exactly half way between bf16 neighbours 1 and 1 + 2^-7: ties go to the even mantissa (1.0);
    # 1 + 3 * 2^-9 rounds up; 1 + 2^-9 rounds down
    assert od.bf16_round(x).tolist() == [1.0, 1.0, 1.0, 1.0078125, -2.5, 0.0]
    import torch
    r = torch.randn(4096, dtype=torch.float32)
    assert np.array_equal(od.bf16_round(r.numpy()), r.to(torch.bfloat16).float().numpy())


def test_subln_and_attention_restatements_agree_with_torch():
    import torch
    from oracle import decoder as od
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 96)).astype(np.float32)
    w, b = rng.standard_normal(96).astype(np.float32), rng.standard_normal(96).astype(np.float32)
    t = torch.from_numpy(x).double()
    want = (t - t.mean(-1, keepdim=True)) / torch.sqrt(t.var(-1, keepdim=True, unbiased=True) + 1e-5) * torch.from_numpy(w).double() + torch.from_numpy(b).double()
    np.testing.assert_allclose(od.subln(x, w, b, 1e-5), want.float().numpy(), rtol=1e-6, atol=1e-6)
    nh, nkv, hd, L = 4, 2, 64, 9
    q = rng.standard_normal(nh * hd).astype(np.float32)
    k = od.bf16_round(rng.standard_normal((nkv, L, hd)).astype(np.float32))
    v = od.bf16_round(rng.standard_normal((nkv, L, hd)).astype(np.float32))
    got = od.attention_decode(q, k, v, nh, nkv, hd)
    for h in range(nh):
        s = torch.from_numpy(k[h // 2]).double() @ torch.from_numpy(q[h * hd:(h + 1) * hd]).double() / np.sqrt(hd)
        ref = torch.softmax(s, 0) @ torch.from_numpy(v[h // 2]).double()
        np.testing.assert_allclose(got[h * hd:(h + 1) * hd], ref.float().numpy(), rtol=1e-5, atol=1e-6)


def test_sampler_restatement_filters():
    from oracle import decoder as od
    logits = np.array([0.0, 3.0, 1.0, 3.0, -1.0, 2.0], dtype=np.float32)
    assert od.sample(logits, 1, deterministic=True)[0] == 1                      # first index on ties
    seeds = [(i * 2654435761 * 40503) % (1 << 63) for i in range(1, 401)]       # spread: small seeds give small draws
    # top_k = 2 keeps both 3.0s (ties with the cut-off stay); top_k = 3 adds the 2.0
    picks = {od.sample(logits, s, top_k=2)[0] for s in seeds[:200]}
    assert picks == {1, 3}
    picks = {od.sample(logits, s, top_k=3)[0] for s in seeds}
    assert picks == {1, 3, 5}
    # top_p: the two 3.0s hold 0.72 of the mass; 0.5 keeps them (equal values stay together), 0.8 adds the 2.0
    picks = {od.sample(logits, s, top_p=0.5)[0] for s in seeds[:200]}
    assert picks == {1, 3}
    picks = {od.sample(logits, s, top_p=0.8)[0] for s in seeds}
    assert picks == {1, 3, 5}
    picks = {od.sample(logits, s, temperature=0.05)[0] for s in seeds[:100]}
    assert picks == {1, 3}
