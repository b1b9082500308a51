"""What a mixer keeps per sequence between steps, declared to the cache.

A mixer returns one of these from `state_spec()` (or None).  The cache puts every layer with
an equal spec into one group with storage of its own:

* `KVStateSpec(kv_heads, head_dim, window=0)`: keys and values of every position (window 0)
  or of the last `window` positions only (a ring).  catena-models keeps one full-capacity
  region per attention layer and only bounds the traversal of sliding layers
  (src/lfm3.rs:317-328, 901-1046); the ring is this build's own storage choice.
* `FixedStateSpec(shape, dtype)`: a constant number of bytes per sequence, whatever its
  length, like the short convolution's last L_cache-1 inputs (src/lfm3.rs:309, 327, 365).
"""
from __future__ import annotations

import dataclasses

PAGE_TOKENS = 64


@dataclasses.dataclass(frozen=True)
class KVStateSpec:
    kv_heads: int
    head_dim: int
    window: int = 0            # 0: every position is kept

    @property
    def ring(self):
        """Entries of the ring (the window rounded up to whole pages); 0 for a growing state."""
        if self.window <= 0:
            return 0
        return (self.window + PAGE_TOKENS - 1) // PAGE_TOKENS * PAGE_TOKENS

    def entries(self, length):
        """Cache entries a sequence of `length` tokens holds."""
        return min(length, self.ring) if self.window > 0 else length

    def pages(self, length):
        return (self.entries(length) + PAGE_TOKENS - 1) // PAGE_TOKENS


@dataclasses.dataclass(frozen=True)
class FixedStateSpec:
    shape: tuple
    dtype: str = "float32"     # float32 | compute (the engine's activation dtype)
