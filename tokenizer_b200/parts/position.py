"""Rotary position encoding, half-split form: lane i of a head pairs with lane
i + rotary_dim/2.  inv_freq_i = 1 / theta^(2i / rotary_dim) is computed in
float64 and stored in float32; the angle float32(position) * inv_freq_i and its
cosine and sine are float32 tables of `max_positions` rows
(reference: qwen-infer/src/model.rs:138-172)."""
from __future__ import annotations

import torch

from ..config.spec import ConfigError
from ..kernels import ops
from .base import register_part


class RotaryHalfSplit:
    @staticmethod
    def tensors(spec):
        return []

    def __init__(self, spec, store, runtime):
        self.theta = float(spec.params["theta"])
        self.rotary_dim = int(spec.params["rotary_dim"])
        self.max_positions = int(spec.params["max_positions"])
        if self.rotary_dim % 2 or self.rotary_dim <= 0:
            raise ConfigError(f"rotary width {self.rotary_dim} must be even and positive")
        inv_freq = [1.0 / (self.theta ** (i / self.rotary_dim)) for i in range(0, self.rotary_dim, 2)]
        self.inv_freq = torch.tensor(inv_freq, dtype=torch.float64).to(torch.float32).to(runtime.device)
        self.cos, self.sin = ops.rope_table(self.inv_freq, self.max_positions)

    def key(self):
        return (self.theta, self.rotary_dim, self.max_positions)


class RotaryInterleaved:
    """Rotary position encoding, interleaved form: lane 2i of the rotated lanes pairs with lane
    2i + 1, i < dims / 2; the pair (u, v) at position p becomes (u cos a - v sin a, v cos a +
    u sin a), a = float32(p) * f_i, f_i = base^(-2i / dims) computed in float64 and stored in
    float32.  There are no tables and no longest position: the kernels that rotate take the
    frequencies and compute sine and cosine of the 32-bit angle themselves."""

    @staticmethod
    def tensors(spec):
        return []

    def __init__(self, spec, store, runtime):
        self.base = float(spec.params["base"])
        self.dims = int(spec.params["dims"])
        if self.dims % 2 or self.dims <= 0 or self.base <= 0:
            raise ConfigError(f"rotary width {self.dims} must be even and positive, the base positive")
        freq = [self.base ** (-2.0 * i / self.dims) for i in range(self.dims // 2)]
        self.inv_freq = torch.tensor(freq, dtype=torch.float64).to(torch.float32).to(runtime.device)


register_part("position", "rope_half_split", RotaryHalfSplit)
register_part("position", "rope_interleaved", RotaryInterleaved)
