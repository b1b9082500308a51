"""The arrangement of one layer: pre-norm, mixer, (post-norm,) residual sum, pre-norm,
feed-forward, (post-norm,) residual sum (src/spec.rs:722-735; src/lfm3.rs:361-501).  Each
residual sum is one fused kernel that also applies the post-norm before it and the next
pre-norm after it (src/catena/lfm3.hex:466-574), so the block hands the normed input of
whatever runs next back to its caller instead of leaving that norm to the next block.
"""
from __future__ import annotations

import torch

from .. import kernels
from .base import Block, register_part


class SandwichBlock(Block):
    prompt_capturable = True
    fused_decode_ok = True
    supports_append = True

    def __init__(self, mixer, feed_forward, input_norm, ffn_norm, post_mixer_norm=None, post_ffn_norm=None):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.input_norm, self.ffn_norm = input_norm, ffn_norm
        self.post_mixer_norm, self.post_ffn_norm = post_mixer_norm, post_ffn_norm

    def children(self):
        return [p for p in (self.input_norm, self.mixer, self.post_mixer_norm, self.ffn_norm,
                            self.feed_forward, self.post_ffn_norm) if p is not None]

    def state_spec(self):
        return self.mixer.state_spec()

    @staticmethod
    def _fusable(norm):
        return getattr(norm, "fused_kind", None) == "rms"

    @classmethod
    def _residual(cls, rt, h, m, post, nxt):
        """h + post(m) in place of h, and next(h) when `nxt` is given.  Norms that the fused
        kernel cannot absorb (anything but an RMSNorm) run through their own `apply`."""
        if post is not None and not cls._fusable(post):
            m, post = post.apply(rt, m), None
        fuse_next = nxt is not None and cls._fusable(nxt)
        n_out = torch.empty_like(h) if fuse_next else None
        kernels.add_norm(h, n_out, m, h,
                         post.weight if post is not None else None,
                         nxt.weight if fuse_next else None,
                         post.eps if post is not None else 0.0,
                         nxt.eps if fuse_next else 0.0)
        if nxt is not None and not fuse_next:
            n_out = nxt.apply(rt, h)
        return h, n_out

    def forward(self, rt, batch, h, n, state, next_norm):
        # the fused residual kernel can add the partial sums of a product cut over K; a post-norm
        # of another kind needs the finished product
        batch.partial_sums_ok = self.post_mixer_norm is None or self._fusable(self.post_mixer_norm)
        m = self.mixer.forward(rt, batch, n, state)
        h, n2 = self._residual(rt, h, m, self.post_mixer_norm, self.ffn_norm)
        batch.partial_sums_ok = self.post_ffn_norm is None or self._fusable(self.post_ffn_norm)
        f = self.feed_forward.forward(rt, batch, n2)
        batch.partial_sums_ok = False
        return self._residual(rt, h, f, self.post_ffn_norm, next_norm)


register_part("block", "sandwich", SandwichBlock)
