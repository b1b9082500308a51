"""What a mixer keeps per sequence between steps, declared to the cache.

A mixer returns one of these from `state_spec()` (or None).  The cache puts every layer with
an equal spec into one group with storage of its own:

* `KVStateSpec(kv_heads, head_dim, window=0)`: keys and values of every position (window 0)
  or of the last `window` positions only (a ring).  catena-models keeps one full-capacity
  region per attention layer and only bounds the traversal of sliding layers
  (src/lfm3.rs:317-328, 901-1046); the ring is this build's own storage choice.
* `FixedStateSpec(shape, dtype)`: a constant number of bytes per sequence, whatever its
  length, like the short convolution's last L_cache-1 inputs (src/lfm3.rs:309, 327, 365).

A spec also says how the launches of a decode step depend on the sequences' length
(`length_class`), which is all the engine needs to know to decide which recorded step may be
replayed; a mixer sizes its launches from the same answer.  A spec class of another mixer
(defined beside that mixer) needs `length_class` and equality; the cache stores what it knows
(key/value pages, fixed-size rows).
"""
from __future__ import annotations

import dataclasses

from ..csrc.limits import ATTN_DECODE_CHUNK, PAGE_TOKENS


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

    def length_class(self, length):
        """A recorded decode step serves every step whose longest sequence falls into the same class
        of lengths; the class is named by its upper bound, and the kernels of such a step are
        launched for that bound.  The kernels over a key/value state work in pieces of
        ATTN_DECODE_CHUNK entries, so the classes double from there (256, 512, 1024, ...: a handful
        of recordings up to any length); a ring never holds more than its own size."""
        bound = ATTN_DECODE_CHUNK
        while bound < length:
            bound *= 2
        return min(bound, self.ring) if self.window > 0 else bound


@dataclasses.dataclass(frozen=True)
class FixedStateSpec:
    shape: tuple
    dtype: str = "float32"     # float32 | compute (the engine's activation dtype)

    def length_class(self, length):
        """A state of fixed size is handled the same way at every length: one class."""
        return 0
