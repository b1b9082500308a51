"""Next-token choice.  catena-models samples greedily only, in its graph
(src/lfm3.rs:517, src/catena/fused_argmax.hex:1-24: strict '>' so the lowest index wins
ties; its server refuses any temperature, src/server/api.rs:170-177).  This build adds
temperature sampling: softmax(logits / temperature) in float32 and an inverse-CDF draw with a
counter-based uniform keyed by (seed, sequence id, step), so that a sequence's tokens do not
depend on which other sequences share its batch.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import kernels


class Sampler:
    """Greedy when temperature is 0, else temperature sampling.  Works on device logits and
    returns host integers (one small device-to-host copy per step)."""

    def __init__(self, device, temperature=0.0, seed=0):
        if temperature < 0:
            raise ValueError("temperature must not be negative")
        self.device = torch.device(device)
        self.temperature, self.seed = float(temperature), int(seed)
        self._cap = 0

    def request(self, sequence_ids, step):
        """The record an engine with on-device sampling takes in place of a separate call."""
        from ..engine.engine import Sampling

        return Sampling(list(sequence_ids), [step] * len(sequence_ids), self.temperature, self.seed)

    @staticmethod
    def staging_ints(n):
        """int32 words copied to the device per call for n rows (ids, steps, temperatures, seed)."""
        return 3 * max(64, 2 * n) + 2

    def _buffers(self, n):
        if n > self._cap:
            cap = max(64, 2 * n)
            self._host = torch.empty(3 * cap + 2, dtype=torch.int32, pin_memory=True)
            self._dev = torch.empty(3 * cap + 2, dtype=torch.int32, device=self.device)
            self._out = torch.empty(cap, dtype=torch.int32, device=self.device)
            self._out_host = torch.empty(cap, dtype=torch.int32, pin_memory=True)
            self._cap = cap

    def sample_device(self, logits, sequence_ids, steps):
        """Tokens as a device int32 tensor [n]."""
        n = logits.shape[0]
        self._buffers(n)
        cap = self._cap
        h = self._host.numpy()
        h[0:n] = np.asarray(sequence_ids, dtype=np.int64).astype(np.int32)
        h[cap:cap + n] = np.asarray(steps, dtype=np.int64).astype(np.int32)
        h[2 * cap:2 * cap + n] = np.float32(self.temperature).view(np.int32)
        h[3 * cap] = np.uint32(self.seed & 0xFFFFFFFF).view(np.int32)
        h[3 * cap + 1] = np.uint32((self.seed >> 32) & 0xFFFFFFFF).view(np.int32)
        self._dev.copy_(self._host, non_blocking=True)
        d = self._dev
        kernels.sample(self._out, logits, d[2 * cap:2 * cap + n].view(torch.float32), d[0:n], d[cap:cap + n],
                       d[3 * cap:3 * cap + 2])
        return self._out[:n]

    def sample(self, logits, sequence_ids, steps):
        """Tokens as a list of Python ints."""
        out = self.sample_device(logits, sequence_ids, steps)
        n = out.shape[0]
        self._out_host[:n].copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self._out_host[:n].tolist()
