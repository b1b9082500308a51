"""Projection y = x W^T with W stored [out, in], as every matrix of the reference is
(src/spec.rs:378-426).  Several tensors with the same input width can be packed row-wise
into one matrix at bind time, so that one matrix product serves them all (the reference
concatenates q, k, v and gate by column range inside its GEMM, src/lfm3.rs:1181-1196).
Which kernel runs (tensor-core GEMM, weight-streaming GEMV, 32-bit FMA) is the runtime's
decision from dtype and row count; this part only owns the weight.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import Part


class Linear(Part):
    prompt_capturable = True
    fused_decode_ok = True
    supports_append = True

    def __init__(self, names, rows, in_features, role="matrix"):
        self.names = [names] if isinstance(names, str) else list(names)
        self.rows = [rows] if isinstance(rows, int) else list(rows)
        self.in_features = in_features
        self.out_features = sum(self.rows)
        self.role = role
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(n, (r, self.in_features), self.role) for n, r in zip(self.names, self.rows)]

    def bind(self, tensors, rt):
        parts = [tensors[n] for n in self.names]
        if len(parts) == 1:
            self.weight = parts[0]
        else:
            if len({p.dtype for p in parts}) > 1:
                parts = [p.to(torch.float32) for p in parts]
            self.weight = torch.cat(parts, dim=0).contiguous()
        self._bound = [self.weight]

    def use_weight(self, weight):
        """Share another part's matrix (a tied output head uses the embedding table)."""
        self.weight = weight
        self._bound = []

    def apply(self, rt, x, out_dtype=None, partial_ok=False):
        """x @ weight^T.  `partial_ok`: the result goes straight into a residual sum that can add
        partial sums (StepBatch.partial_sums_ok says so), so the runtime may leave it as such."""
        return rt.linear(x, self.weight, out_dtype, partial_ok)
