"""The BitLinear operator as the reference exposes it, backed by the CUDA path.

Mirrors ``BitLinear`` / ``BitLinearConfig`` / ``BitLinearForward``
(bitnet-quant/src/bitlinear/{layer,forward}.rs), the inference engine's
``BitLinearLayer`` and ``FeedForwardNetwork``
(bitnet-inference/src/engine/transformer_layers.rs:67-202, :552-624) and the absmean weight
quantiser (bitnet-quant/src/quantization/weights.rs:807-857): same names, argument meaning
and error behaviour.  Weight preparation (ternarise, pack, upload) happens once per
weight version; every forward afterwards is launches only.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from . import ops
from .cuda import CudaError, IncompatibleShapes


class BitLinearError(CudaError):
    """bitnet-quant/src/bitlinear/error.rs."""


class ShapeMismatch(BitLinearError, IncompatibleShapes):
    def __init__(self, expected, actual):
        super().__init__(f"Shape mismatch: expected {list(expected)}, got {list(actual)}")
        self.expected, self.actual = list(expected), list(actual)


@dataclass
class BitLinearConfig:             # bitlinear/layer.rs:19-75
    in_features: int = 0
    out_features: int = 0
    use_bias: bool = False         # BitNet standard: no bias (:52)
    enable_caching: bool = True
    per_channel: bool = False      # one scale per tensor (:57)


@dataclass
class QuantizedWeight:             # quantization/weights.rs:157-175
    values: np.ndarray             # ternary int8 [N,K]
    scale: float
    original_shape: tuple


def absmean_quantize_weights(weights) -> QuantizedWeight:
    """weights.rs:807-857: threshold 0.7*mean|W|, t = sign(W)*(|W|>thr), scale = sum(W*t)/sum(t*t)."""
    w = np.asarray(weights.detach().cpu() if isinstance(weights, torch.Tensor) else weights, dtype=np.float32)
    thr = np.float32(np.abs(w).mean(dtype=np.float64)) * np.float32(0.7)
    t = (np.sign(w) * (np.abs(w) > thr)).astype(np.int8)
    den = float((t.astype(np.float64) ** 2).sum())
    scale = 1.0 if abs(den) < np.finfo(np.float32).eps else float((w.astype(np.float64) * t).sum() / den)
    return QuantizedWeight(t, float(np.float32(scale)), tuple(w.shape))


def _flatten_tokens(x: torch.Tensor, in_features: int):
    """forward.rs:63-76 and transformer_layers.rs:167: last dim must be in_features; 3-D -> [B*S,K]."""
    if x.dim() not in (2, 3) or x.shape[-1] != in_features:
        raise ShapeMismatch(["batch", in_features], list(x.shape))
    return x.reshape(-1, in_features), x.shape[:-1]


class BitLinear:
    """bitnet-quant BitLinear: keeps full-precision weights, quantises and packs on first use."""

    def __init__(self, config: BitLinearConfig, layer_name: str = "bitlinear", device="cuda", weights=None,
                 seed: int = 0):
        if config.in_features <= 0 or config.out_features <= 0:
            raise BitLinearError(f"invalid features {config.in_features}x{config.out_features}")
        self.config, self.layer_name, self.device = config, layer_name, torch.device(device)
        if weights is None:
            gen = torch.Generator().manual_seed(seed)
            weights = torch.randn((config.out_features, config.in_features), generator=gen) * 0.02
        self._weights = torch.as_tensor(weights, dtype=torch.float32).cpu()
        if tuple(self._weights.shape) != (config.out_features, config.in_features):
            raise ShapeMismatch([config.out_features, config.in_features], list(self._weights.shape))
        self.bias = torch.zeros(config.out_features, device=self.device) if config.use_bias else None
        self._packed = None        # device cache: (packed uint8 tensor, scale)
        self.cache_hits = self.cache_misses = 0

    # layer.rs:236-294
    def get_quantized_weights(self):
        if self._packed is not None and self.config.enable_caching:
            self.cache_hits += 1
            return self._packed
        self.cache_misses += 1
        # absmean quantisation and packing on the device (weights.rs:807-857, packing.rs:352-388)
        self._packed = ops.quantize_pack_weights(self._weights.to(self.device))
        return self._packed

    # layer.rs:299-326
    def update_weights(self, new_weights) -> None:
        w = torch.as_tensor(new_weights, dtype=torch.float32).cpu()
        if tuple(w.shape) != tuple(self._weights.shape):
            raise ShapeMismatch(list(self._weights.shape), list(w.shape))
        self._weights = w
        self._packed = None

    # forward.rs:55-136
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x2, lead = _flatten_tokens(x, self.config.in_features)
        wp, scale = self.get_quantized_weights()
        y = ops.bitlinear_forward(wp, scale, x2.contiguous(), self.config.out_features)
        if self.bias is not None:
            y += self.bias
        return y.reshape(*lead, self.config.out_features)

    # forward.rs:95
    def forward_with_quantized_weights(self, x: torch.Tensor, packed: torch.Tensor, scale: float) -> torch.Tensor:
        x2, lead = _flatten_tokens(x, self.config.in_features)
        y = ops.bitlinear_forward(packed, scale, x2.contiguous(), self.config.out_features)
        if self.bias is not None:
            y += self.bias
        return y.reshape(*lead, self.config.out_features)

    forward_batch = forward        # forward.rs:270-295: [B,S,K] input


class BitLinearLayer:
    """Inference-engine BitLinearLayer (transformer_layers.rs:67-202): ternary weights given
    directly as int8 [N,K] (or already packed), one fp32 scale."""

    def __init__(self, in_features: int, out_features: int, use_bias: bool = False, device="cuda",
                 ternary=None, packed=None, scale: float = 1.0):
        self.in_features, self.out_features, self.device = in_features, out_features, torch.device(device)
        self.scale = float(scale)
        if packed is not None:
            self.packed = torch.as_tensor(packed, dtype=torch.uint8).to(self.device).reshape(-1)
            if self.packed.numel() != ops.packed_len(in_features * out_features):
                raise ShapeMismatch([ops.packed_len(in_features * out_features)], [self.packed.numel()])
            ops.sanitize_packed(self.packed)
        else:
            if ternary is None:   # the reference initialises weights to zero (:94)
                ternary = torch.zeros((out_features, in_features), dtype=torch.int8)
            t = torch.as_tensor(ternary, dtype=torch.int8)
            if tuple(t.shape) != (out_features, in_features):
                raise ShapeMismatch([out_features, in_features], list(t.shape))
            self.packed = ops.pack_ternary(t.to(self.device))
        self.bias = torch.zeros(out_features, device=self.device) if use_bias else None

    def forward(self, x: torch.Tensor, **kw) -> torch.Tensor:
        x2, lead = _flatten_tokens(x, self.in_features)
        y = ops.bitlinear_forward(self.packed, self.scale, x2.contiguous(), self.out_features, **kw)
        if self.bias is not None:
            y += self.bias
        return y.reshape(*lead, self.out_features)


class FeedForwardNetwork:
    """transformer_layers.rs:552-624: y = down(up(x) * relu(gate(x))^2)."""

    def __init__(self, hidden: int, ffn: int, gate: BitLinearLayer, up: BitLinearLayer, down: BitLinearLayer):
        for lyr, (k, n) in ((gate, (hidden, ffn)), (up, (hidden, ffn)), (down, (ffn, hidden))):
            if (lyr.in_features, lyr.out_features) != (k, n):
                raise ShapeMismatch([n, k], [lyr.out_features, lyr.in_features])
        self.hidden, self.ffn, self.gate_proj, self.up_proj, self.down_proj = hidden, ffn, gate, up, down

    def forward(self, x: torch.Tensor, **kw) -> torch.Tensor:
        x2, lead = _flatten_tokens(x, self.hidden)
        y, _ = ops.ffn_forward(self.gate_proj.packed, self.gate_proj.scale, self.up_proj.packed, self.up_proj.scale,
                               self.down_proj.packed, self.down_proj.scale, x2.contiguous(), self.ffn, **kw)
        return y.reshape(*lead, self.hidden)
