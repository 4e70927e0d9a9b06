"""CPU restatement (numpy) of the decode step around the BitLinear projections.  TEST INFRASTRUCTURE:
only tests/, __graft_entry__.smoke() and bench.py's CPU legs may import this; the product never does.

Each function cites the reference file:line it follows (paths inside the reference project).  The tensor
arithmetic of these reference functions lives in candle-core "0.8" (Cargo.toml:31, no lock file), which
is not vendored: its published semantics are restated (mean_keepdim = sum / n; var_keepdim = sum of
squared deviations / (n - 1); broadcast ops elementwise in f32), and because the reference's own tests at
this level check shapes only (transformer_layers.rs:744-790), the fp32 stages here are PARITY UNPINNED.
Floating-point stages are evaluated in float64 and rounded once, i.e. they give the correctly rounded
value of the reference's formula; the CUDA path is compared with a stated tolerance.  Integer stages
(quantised activations, accumulators) go through the C oracle and are compared exactly.
"""
from __future__ import annotations

import numpy as np

from . import bitlinear_forward


def bf16_round(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 (round to nearest even) -> fp32: the precision the KV cache keeps."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).reshape(np.shape(x))


def subln(x: np.ndarray, weight: np.ndarray, bias: np.ndarray, eps: float) -> np.ndarray:
    """SubLNNormalization::forward (bitnet-inference/src/engine/transformer_layers.rs:356-386):
    (x - mean) / sqrt(var + eps) * weight + bias over the last dimension; var_keepdim divides by n - 1."""
    x64 = np.asarray(x, dtype=np.float64)
    n = x64.shape[-1]
    mean = x64.mean(axis=-1, keepdims=True)
    var = ((x64 - mean) ** 2).sum(axis=-1, keepdims=True) / max(n - 1, 1)
    y = (x64 - mean) / np.sqrt(var + np.float64(np.float32(eps))) * np.asarray(weight, np.float64) + np.asarray(bias, np.float64)
    return y.astype(np.float32)


def attention_decode(q: np.ndarray, k_cache: np.ndarray, v_cache: np.ndarray, n_heads: int, n_kv: int, head_dim: int) -> np.ndarray:
    """MultiHeadAttention::forward for one query token (transformer_layers.rs:460-547): scores = q k^T *
    (1 / sqrt(head_dim)), softmax over the keys (the reference divides exp(scores) by their sum, :517-523;
    subtracting the maximum first is the same function), weights x values; grouped-query form: query head h
    reads KV head h // (n_heads / n_kv).  q [n_heads*head_dim] fp32; caches [n_kv, L, head_dim] (already
    bf16-rounded, including the new token).  RoPE is the identity in the reference (:278-289)."""
    g = n_heads // n_kv
    out = np.empty(n_heads * head_dim, dtype=np.float32)
    scale = np.float64(np.float32(1.0) / np.sqrt(np.float32(head_dim)))
    for h in range(n_heads):
        kv = h // g
        qh = q[h * head_dim:(h + 1) * head_dim].astype(np.float64)
        s = k_cache[kv].astype(np.float64) @ qh * scale
        p = np.exp(s - s.max())
        p /= p.sum()
        out[h * head_dim:(h + 1) * head_dim] = (p @ v_cache[kv].astype(np.float64)).astype(np.float32)
    return out


LCG_MUL, LCG_ADD = 1103515245, 12345


def lcg_next(state: int) -> int:
    """TokenSampler::pseudo_random_sample's generator (sampling.rs:273-276): state * 1103515245 + 12345 (wrapping u64)."""
    return (state * LCG_MUL + LCG_ADD) & 0xFFFFFFFFFFFFFFFF


def lcg_uniform(state: int) -> float:
    """24 bits of state / 65536 as u in [0, 1) (the reference takes (state / 65536) % 1000 as a token id)."""
    return float((state >> 16) & 0xFFFFFF) / 16777216.0


def sample(logits: np.ndarray, state: int, temperature=1.0, top_k=0, top_p=1.0, deterministic=False):
    """TokenSampler::sample (sampling.rs:106-189) as its doc comments describe it: argmax when deterministic
    (first index on ties); otherwise logits / temperature (:180-192), keep the top_k largest (:195-210) and the
    smallest most-likely set whose probability reaches top_p (:213-226) -- values equal to a cut-off are kept --
    softmax, one draw with the generator above, first index whose running probability exceeds u.
    Returns (token, new_state, margin) where margin is how far u * total is from the nearest boundary of the
    running sum, relative to the total (tests skip draws that sit on a boundary)."""
    logits = np.asarray(logits, dtype=np.float32)
    if deterministic:
        return int(np.argmax(logits)), state, 1.0
    z = (logits / np.float32(temperature)).astype(np.float32)
    keep = np.ones(z.shape, dtype=bool)
    if 0 < top_k < z.size:
        kth = np.sort(z)[::-1][top_k - 1]
        keep &= z >= kth
    p = np.where(keep, np.exp(z.astype(np.float64) - np.float64(z.max())), 0.0)
    total = p.sum()
    if top_p < 1.0:
        order = np.argsort(-z, kind="stable")
        cum = np.cumsum(p[order])
        target = np.float64(np.float32(top_p)) * total
        n = int(np.searchsorted(cum, target, side="left")) + 1     # smallest prefix whose mass reaches the target
        n = min(n, int(keep.sum()))
        cut = z[order[n - 1]]
        keep &= z >= cut
        p = np.where(keep, p, 0.0)
        total = p.sum()
    state = lcg_next(state)
    u = lcg_uniform(state)
    run = np.cumsum(p)
    target = u * total
    idx = int(np.searchsorted(run, target, side="right"))
    kept = np.flatnonzero(keep)
    if idx >= z.size:
        idx = int(kept[-1])
    while not keep[idx]:
        idx += 1
    below = run[idx - 1] if idx > 0 else 0.0
    margin = min(target - below, run[idx] - target) / total
    return idx, state, float(margin)


class OracleDecoder:
    """ForwardPassPipeline (forward_pass_pipeline.rs:146-362) for one new token per sequence with a bf16 KV
    cache: embedding row gather (:31-77), TransformerBlock::forward per layer (transformer_layers.rs:675-709),
    language-model head on the last hidden state (:283-291), sampler."""

    def __init__(self, cfg: dict, embedding: np.ndarray, layers: list[dict], lm_head: tuple):
        self.cfg, self.embedding, self.layers, self.lm_head = cfg, embedding, layers, lm_head
        self.reset()

    def reset(self):
        c = self.cfg
        B, L = c["max_batch"], c["num_layers"]
        self.k = [[np.zeros((c["num_kv_heads"], 0, c["head_dim"]), np.float32) for _ in range(B)] for _ in range(L)]
        self.v = [[np.zeros((c["num_kv_heads"], 0, c["head_dim"]), np.float32) for _ in range(B)] for _ in range(L)]

    def step(self, ids: np.ndarray) -> np.ndarray:
        """ids [B] -> logits [B, vocab]; every sequence's cache grows by one token."""
        c = self.cfg
        H, nh, nkv, hd, F = c["hidden_size"], c["num_heads"], c["num_kv_heads"], c["head_dim"], c["ffn_size"]
        x = self.embedding[np.asarray(ids)].astype(np.float32)
        B = x.shape[0]
        for li, lw in enumerate(self.layers):
            n1 = subln(x, lw["n1w"], lw["n1b"], c["norm_eps"])
            q = bitlinear_forward(lw["q"], lw["s_q"], n1, nh * hd)["y"]
            k = bitlinear_forward(lw["k"], lw["s_k"], n1, nkv * hd)["y"]
            v = bitlinear_forward(lw["v"], lw["s_v"], n1, nkv * hd)["y"]
            attn = np.empty((B, nh * hd), np.float32)
            for b in range(B):
                self.k[li][b] = np.concatenate([self.k[li][b], bf16_round(k[b]).reshape(nkv, 1, hd)], axis=1)
                self.v[li][b] = np.concatenate([self.v[li][b], bf16_round(v[b]).reshape(nkv, 1, hd)], axis=1)
                attn[b] = attention_decode(q[b], self.k[li][b], self.v[li][b], nh, nkv, hd)
            o = bitlinear_forward(lw["o"], lw["s_o"], attn, H)["y"]
            x = (x + o).astype(np.float32)
            n2 = subln(x, lw["n2w"], lw["n2b"], c["norm_eps"])
            up = bitlinear_forward(lw["up"], lw["s_u"], n2, F)["y"]
            gate = bitlinear_forward(lw["gate"], lw["s_g"], n2, F)["y"]
            r = np.maximum(gate, np.float32(0))
            h = (up * (r * r).astype(np.float32)).astype(np.float32)
            f = bitlinear_forward(lw["down"], lw["s_d"], h, H)["y"]
            x = (x + f).astype(np.float32)
        self.hidden = x
        return bitlinear_forward(self.lm_head[0], self.lm_head[1], x, c["vocab_size"])["y"]
