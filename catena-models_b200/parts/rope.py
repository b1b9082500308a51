"""Rotary position encoding with per-frequency factors.

rate[i] = theta^(-2i/head_dim) / factor[i], both steps in float32 as the reference does them
(the power on the host, src/catena.rs:185-204; the division in the kernel,
src/catena/lfm3.hex:726-734); the kernel forms angle = float(position) * rate[i] and rotates
the halves of the head against each other (src/catena/lfm3.hex:706-746).  `factors_name` is
the tensor of per-frequency divisors, or None for factor 1 (sliding layers ignore the factors
and use a base of their own).
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import Position, register_part


class Rotary(Position):
    prompt_capturable = True
    fused_decode_ok = True
    supports_append = True

    def __init__(self, head_dim, theta, factors_name=None):
        self.head_dim, self.theta, self.factors_name = head_dim, float(theta), factors_name
        self._rate = None

    def tensor_specs(self):
        if self.factors_name is None:
            return []
        return [TensorSpec(self.factors_name, (self.head_dim // 2,), "rope_factors")]

    def bind(self, tensors, rt):
        half = self.head_dim // 2
        exponent = (2 * torch.arange(half, dtype=torch.float32)) / torch.tensor(float(self.head_dim), dtype=torch.float32)
        freq = torch.pow(torch.tensor(self.theta, dtype=torch.float32), -exponent)
        if self.factors_name is not None:
            freq = freq / tensors[self.factors_name].to("cpu", torch.float32)
        self._rate = freq.to(rt.device).contiguous()

    def rate_table(self):
        return self._rate


class NoPosition(Position):
    """No position encoding: the head vectors are left unrotated."""
    prompt_capturable = True
    fused_decode_ok = True
    supports_append = True


register_part("position", "rotary", Rotary)
register_part("position", "none", NoPosition)
