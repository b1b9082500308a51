"""RMSNorm: y = (x / sqrt(mean(x^2) + eps)) * w, the product with w taken in float before
the one rounding to the activation dtype (src/catena/qwen35.hex:912-946,
src/catena/fused_normalization.hex:23-39).  The weight is float32 as in the reference's
tensor list (src/spec.rs:722-735).  Fused kernels (residual sum + norms) read `weight` and
`eps` directly.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Norm, register_part


class RMSNorm(Norm):
    prompt_capturable = True
    fused_decode_ok = True
    supports_append = True
    fused_kind = "rms"          # what the fused residual kernel can absorb

    def __init__(self, name, width, eps):
        self.name, self.width, self.eps = name, width, float(eps)
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.width,), "norm")]

    def bind(self, tensors, rt):
        self.weight = tensors[self.name].to(torch.float32).contiguous()
        self._bound = [self.weight]

    def apply(self, rt, x):
        y = torch.empty_like(x)
        kernels.rmsnorm(y, x, self.weight, self.eps)
        return y


register_part("norm", "rms", RMSNorm)
