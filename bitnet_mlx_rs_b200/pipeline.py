"""Host mirror of the reference's generation pipeline over the CUDA decode step
(ForwardPassPipeline / ForwardPassConfig / SamplingConfig / SamplingPresets,
bitnet-inference/src/engine/forward_pass_pipeline.rs:80-362 and sampling.rs:11-45, :312-385).

Everything runs inside libbitnet_cuda_kernels (bitnet_decoder_*); this file only carries arguments.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib as L
from .cuda import CudaBackend, IncompatibleShapes, check


@dataclass
class SamplingConfig:
    """SamplingConfig (sampling.rs:11-45)."""
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0
    deterministic: bool = False

    def _c(self) -> L.SamplingConfig:
        return L.SamplingConfig(self.temperature, self.top_k, self.top_p, self.seed, 1 if self.deterministic else 0)


class SamplingPresets:
    """SamplingPresets (sampling.rs:312-385)."""

    @staticmethod
    def deterministic() -> SamplingConfig:
        return SamplingConfig(deterministic=True, seed=42)

    @staticmethod
    def conservative() -> SamplingConfig:
        return SamplingConfig(temperature=0.2, top_k=50, top_p=0.9)

    @staticmethod
    def balanced() -> SamplingConfig:
        return SamplingConfig(temperature=0.7, top_k=100, top_p=0.95)

    @staticmethod
    def creative() -> SamplingConfig:
        return SamplingConfig(temperature=1.2, top_k=200, top_p=0.98)

    @staticmethod
    def reproducible(seed: int) -> SamplingConfig:
        return SamplingConfig(temperature=0.8, top_k=50, top_p=0.9, seed=seed)


@dataclass
class ForwardPassConfig:
    """ForwardPassConfig + TransformerConfig (forward_pass_pipeline.rs:80-118, transformer_layers.rs:14-49), plus the
    grouped-query and batch sizes the CUDA step needs."""
    num_layers: int = 12
    vocab_size: int = 128256
    hidden_size: int = 2048
    num_heads: int = 16
    num_kv_heads: int = 16
    head_dim: int = 128
    ffn_intermediate_size: int = 5632
    max_seq_len: int = 2048
    max_batch: int = 1
    rms_norm_eps: float = 1e-5

    def _c(self) -> L.DecoderConfig:
        return L.DecoderConfig(self.vocab_size, self.hidden_size, self.num_layers, self.num_heads, self.num_kv_heads,
                               self.head_dim, self.ffn_intermediate_size, self.max_seq_len, self.max_batch, self.rms_norm_eps)


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8).reshape(-1)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32).reshape(-1)


class ForwardPassPipeline:
    """ForwardPassPipeline (forward_pass_pipeline.rs:146-362) on the CUDA decode step."""

    def __init__(self, backend: CudaBackend, config: ForwardPassConfig):
        self.backend, self.config, self._h = backend, config, None
        cfg = config._c()
        out = C.c_void_p()
        check(L.load().bitnet_decoder_create(backend._h, C.byref(cfg), C.byref(out)))
        self._h = out.value

    def close(self) -> None:
        if self._h:
            L.load().bitnet_decoder_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            if self.backend._h:
                self.close()
        except Exception:
            pass

    # ---- parameters -------------------------------------------------------------------------------
    def load_embedding(self, table) -> None:
        t = _f32(table)
        if t.size != self.config.vocab_size * self.config.hidden_size:
            raise IncompatibleShapes("embedding table must be [vocab_size, hidden_size]")
        check(L.load().bitnet_decoder_load_embedding(self._h, t.ctypes.data))

    def load_layer(self, index: int, w: dict) -> None:
        """`w`: packed uint8 arrays q, k, v, o, gate, up, down; scales s_q, s_k, s_v, s_o, s_g, s_u, s_d; SubLN
        parameters n1w, n1b (input_layernorm) and n2w, n2b (post_attention_layernorm)."""
        c = self.config
        qd, kd, H, F = c.num_heads * c.head_dim, c.num_kv_heads * c.head_dim, c.hidden_size, c.ffn_intermediate_size
        sizes = {"q": qd * H, "k": kd * H, "v": kd * H, "o": H * qd, "gate": F * H, "up": F * H, "down": H * F}
        keep = {k: _u8(w[k]) for k in sizes}
        for k, n in sizes.items():
            if keep[k].size != (n + 3) // 4:
                raise IncompatibleShapes(f"layer {index}: {k} has {keep[k].size} packed bytes, expected {(n + 3) // 4}")
        norms = {k: _f32(w[k]) for k in ("n1w", "n1b", "n2w", "n2b")}
        for k, a in norms.items():
            if a.size != H:
                raise IncompatibleShapes(f"layer {index}: {k} must have {H} values")
        s = L.DecoderLayer(keep["q"].ctypes.data, keep["k"].ctypes.data, keep["v"].ctypes.data, keep["o"].ctypes.data,
                           keep["gate"].ctypes.data, keep["up"].ctypes.data, keep["down"].ctypes.data,
                           w["s_q"], w["s_k"], w["s_v"], w["s_o"], w["s_g"], w["s_u"], w["s_d"],
                           norms["n1w"].ctypes.data, norms["n1b"].ctypes.data, norms["n2w"].ctypes.data, norms["n2b"].ctypes.data)
        check(L.load().bitnet_decoder_load_layer(self._h, index, C.byref(s)))

    def load_lm_head(self, packed, scale: float) -> None:
        p = _u8(packed)
        if p.size != (self.config.vocab_size * self.config.hidden_size + 3) // 4:
            raise IncompatibleShapes("lm_head must be [vocab_size, hidden_size] packed")
        check(L.load().bitnet_decoder_load_lm_head(self._h, p.ctypes.data, scale))

    # ---- generation --------------------------------------------------------------------------------
    def reset(self) -> None:
        check(L.load().bitnet_decoder_reset(self._h))

    def set_graphs(self, enabled: bool) -> None:
        check(L.load().bitnet_decoder_set_graphs(self._h, 1 if enabled else 0))

    def feed(self, ids) -> None:
        """Context tokens ids [B, T]: cached, nothing sampled."""
        a = np.ascontiguousarray(ids, dtype=np.int32)
        if a.ndim != 2:
            raise IncompatibleShapes("ids must be [B, T]")
        check(L.load().bitnet_decoder_feed(self._h, a.ctypes.data, a.shape[0], a.shape[1]))

    def decode(self, ids, n_new: int, sampling: SamplingConfig | None = None, eos_id: int = -1, out=None):
        """ids [B]: each sequence's last known token; returns (tokens [B, n_new], steps run)."""
        a = np.ascontiguousarray(ids, dtype=np.int32).reshape(-1)
        res = out if out is not None else np.empty((a.size, n_new), dtype=np.int32)
        sc = (sampling or SamplingConfig())._c()
        steps = C.c_size_t()
        check(L.load().bitnet_decoder_decode(self._h, a.ctypes.data, a.size, n_new, C.byref(sc), eos_id, res.ctypes.data, C.byref(steps)))
        return res, steps.value

    def generate(self, input_ids, max_new_tokens: int, sampling: SamplingConfig | None = None, eos_id: int = -1):
        """ForwardPassPipeline::generate (forward_pass_pipeline.rs:311-362): input_ids [B, prompt_len] (or [prompt_len])
        -> the prompt followed by the generated tokens, [B, prompt_len + steps]."""
        a = np.ascontiguousarray(input_ids, dtype=np.int32)
        if a.ndim == 1:
            a = a[None, :]
        out = np.empty((a.shape[0], max_new_tokens), dtype=np.int32)
        sc = (sampling or SamplingConfig())._c()
        steps = C.c_size_t()
        check(L.load().bitnet_decoder_generate(self._h, a.ctypes.data, a.shape[0], a.shape[1], max_new_tokens, C.byref(sc), eos_id,
                                               out.ctypes.data, C.byref(steps)))
        return np.concatenate([a, out[:, :steps.value]], axis=1)

    def _read(self, what: int, shape, dtype) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        check(L.load().bitnet_decoder_read(self._h, what, out.ctypes.data, out.nbytes))
        return out

    def logits(self, batch: int) -> np.ndarray:
        return self._read(L.DECODER_LOGITS, (batch, self.config.vocab_size), np.float32)

    def hidden(self, batch: int) -> np.ndarray:
        return self._read(L.DECODER_HIDDEN, (batch, self.config.hidden_size), np.float32)

    def positions(self, batch: int) -> np.ndarray:
        return self._read(L.DECODER_POSITIONS, (batch,), np.int32)


@dataclass
class BackendCapabilities:
    """BackendCapabilities (bitnet-inference/src/engine/mod.rs:140-148)."""
    supports_batching: bool
    supports_streaming: bool
    max_batch_size: int
    memory_limit: int | None
    device_type: str


class CudaInferenceBackend:
    """The product-level plug point: the reference's InferenceBackend trait (bitnet-inference/src/engine/mod.rs:126-138:
    execute_batch, optimize_model, get_memory_usage, capabilities) on top of the CUDA decode step.

    `optimize_model(model)` takes a model description -- {"config": ForwardPassConfig, "embedding": [vocab, hidden] fp32,
    "layers": [dict per layer as ForwardPassPipeline.load_layer takes], "lm_head": (packed, scale)} -- and makes it resident
    on the device.  `execute_batch(inputs)` runs each input (token ids [B, T] or [T]) through the model and returns, per
    input, the logits of its last position [B, vocab] (ForwardPassPipeline::forward followed by the narrow of
    generate(), forward_pass_pipeline.rs:245-331)."""

    def __init__(self, backend: CudaBackend | None = None, memory_pool_size: int = 8 << 30):
        from .cuda import CudaBackendConfig
        self._own = backend is None
        self.backend = backend or CudaBackend(CudaBackendConfig(memory_pool_size=memory_pool_size))
        self.pipeline: ForwardPassPipeline | None = None

    def optimize_model(self, model: dict) -> None:
        if self.pipeline is not None:
            self.pipeline.close()
        self.pipeline = ForwardPassPipeline(self.backend, model["config"])
        self.pipeline.load_embedding(model["embedding"])
        for i, lw in enumerate(model["layers"]):
            self.pipeline.load_layer(i, lw)
        self.pipeline.load_lm_head(*model["lm_head"])

    def execute_batch(self, inputs) -> list:
        if self.pipeline is None:
            raise IncompatibleShapes("no model: call optimize_model first")
        outs = []
        for ids in inputs:
            a = np.ascontiguousarray(ids, dtype=np.int32)
            if a.ndim == 1:
                a = a[None, :]
            self.pipeline.reset()
            if a.shape[1] > 1:
                self.pipeline.feed(a[:, :-1])
            self.pipeline.decode(a[:, -1], 1, SamplingConfig(deterministic=True))
            outs.append(self.pipeline.logits(a.shape[0]))
        return outs

    def get_memory_usage(self) -> int:
        mm = self.backend.memory_manager()
        return mm._usage()[0]

    def capabilities(self) -> BackendCapabilities:
        cfg = self.pipeline.config if self.pipeline else None
        return BackendCapabilities(True, True, cfg.max_batch if cfg else 0, self.backend.memory_manager()._usage()[1], "cuda")

    def close(self) -> None:
        if self.pipeline is not None:
            self.pipeline.close()
            self.pipeline = None
        if self._own:
            self.backend.close()
