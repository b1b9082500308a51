"""Gated short-convolution mixer: in_proj to B | C | X, a causal depthwise convolution of
`taps` taps over B*X with a per-sequence state of the last taps-1 inputs, times C, out_proj
(src/lfm3.rs:784-812; src/catena/lfm3.hex:3-23, 905-921, 982-1046, 1105-1114; decode form
src/catena/lfm3.hex:263-366).  The state is float32 whatever the activation dtype, as the
reference's history buffer is (src/lfm3.rs:309, 327).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.spec import FixedStateSpec
from ..weights.loader import TensorSpec
from .base import Mixer, register_part
from .linear import Linear


class ShortConv(Mixer):
    prompt_capturable = True
    fused_decode_ok = True
    supports_append = True

    def __init__(self, prefix, hidden, taps, names=None):
        names = names or {}
        n = lambda key, default: prefix + names.get(key, default)
        self.hidden, self.taps = hidden, taps
        self.in_proj = Linear(n("in_proj", "shortconv.in_proj.weight"), 3 * hidden, hidden)
        self.out_proj = Linear(n("out_proj", "shortconv.out_proj.weight"), hidden, hidden)
        self.conv_name = n("conv", "shortconv.conv.weight")
        self.conv_w = self.conv_w_t = None

    def children(self):
        return [self.in_proj, self.out_proj]

    def tensor_specs(self):
        return [TensorSpec(self.conv_name, (self.hidden, self.taps), "conv")]

    def bind(self, tensors, rt):
        self.conv_w = tensors[self.conv_name].to(torch.float32).contiguous()
        self.conv_w_t = self.conv_w.t().contiguous()          # [taps, hidden]: the kernel reads 8 channels at once
        self._bound = [self.conv_w]

    def state_spec(self):
        return FixedStateSpec((self.taps - 1, self.hidden), "float32")

    def forward(self, rt, batch, x, state):
        y = torch.empty((batch.T, self.hidden), dtype=x.dtype, device=x.device)
        if batch.kind == "decode" and rt.streams_weights(x, self.in_proj.weight):
            # a decode step of a small batch: the convolution runs where in_proj's sums are formed
            kernels.gemm_skinny_shortconv(y, x, self.in_proj.weight, self.conv_w, state.tensor, batch.seq_slot)
            return self.out_proj.apply(rt, y, partial_ok=batch.partial_sums_ok)
        bcx = self.in_proj.apply(rt, x)                                   # [T, 3H]
        # an append step: outputs from the stored state, then the state, in two launches; a sequence
        # of such a step that stands at position 0 starts from an empty state
        kernels.shortconv(y, bcx, self.conv_w, state.tensor, batch.tok_seq, batch.seq_start, batch.seq_slot,
                          self.taps, from_zero=batch.prefill, one_token_each=batch.kind == "decode",
                          w_t=self.conv_w_t, seq_pos0=batch.seq_pos0 if batch.append else None)
        return self.out_proj.apply(rt, y, partial_ok=batch.partial_sums_ok)


register_part("mixer", "short_conv", ShortConv)
