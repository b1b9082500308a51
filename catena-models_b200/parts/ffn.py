"""SwiGLU feed-forward: a = (g * sigmoid(g)) * u with g = x Wgate^T, u = x Wup^T, then Wdown
(src/catena/lfm3.hex:833-845; fused epilogue src/catena/lfm3_wmma.hex:10790-10815).  Gate and up
are packed into one matrix at bind time so that one product reads x once
(src/lfm3.rs:1062-1075 fuses them in its kernel the same way).
"""
from __future__ import annotations

from .base import FeedForward, register_part
from .linear import Linear


class SwiGLU(FeedForward):
    prompt_capturable = True
    fused_decode_ok = True
    supports_append = True

    def __init__(self, prefix, hidden, intermediate, names=None):
        names = names or {}
        n = lambda key, default: prefix + names.get(key, default)
        self.hidden, self.intermediate = hidden, intermediate
        self.gate_up = Linear([n("gate", "ffn_gate.weight"), n("up", "ffn_up.weight")],
                              [intermediate, intermediate], hidden)
        self.down = Linear(n("down", "ffn_down.weight"), hidden, intermediate)

    def children(self):
        return [self.gate_up, self.down]

    def forward(self, rt, batch, x):
        a = rt.gate_up_swiglu(x, self.gate_up.weight, self.intermediate)
        return self.down.apply(rt, a, partial_ok=batch.partial_sums_ok)


register_part("feed_forward", "swiglu", SwiGLU)
