"""What an architecture hands to the engine: its parts, already built from the typed
configuration, and the order in which they run.

`blocks` are the layers that own weights; `plan` is the order of execution as data: each
entry names a block and the state unit (the cache storage) it works on.  A block may appear
in several entries (it then runs more than once, each run with a state unit of its own), and
an entry may name a state unit that an earlier entry owns (`owns_state=False`: the layer
reads another layer's cache and writes none).
"""
from __future__ import annotations

import dataclasses

from ..weights.loader import TensorSpec


@dataclasses.dataclass(frozen=True)
class PlanEntry:
    block: int
    state: int
    owns_state: bool = True


@dataclasses.dataclass
class ModelDefinition:
    architecture: str
    vocab_size: int
    hidden_size: int
    embedding_name: str
    blocks: list
    plan: list
    final_norm: object
    head: object                     # a Linear with a weight of its own, or None: tied to the embedding
    stop_token_ids: tuple = ()
    max_positions: int = 0
    embedding_aliases: tuple = ()
    extra_tensors: tuple = ()        # tensors every checkpoint holds although no part may read them
    # Other names the same tensors may carry in a file: (prefix, other prefix) pairs; a tensor whose
    # name starts with `prefix` is also looked for under the name with `other prefix` in its place.
    alias_prefixes: tuple = ()
    # Constants that some architectures put around the stack of blocks; the defaults leave it as LFM3 has it.
    embedding_scale: float = 1.0     # factor on every embedding row
    logit_scale: float = 1.0         # factor on the logits
    logit_softcap: float = 0.0       # logits <- cap * tanh(logits / cap) after the scale; 0: none

    def parts(self):
        out = list(self.blocks) + [self.final_norm]
        if self.head is not None:
            out.append(self.head)
        return out

    def tensor_specs(self):
        """Every tensor the model needs, each name once (parts may share a tensor)."""
        specs = [TensorSpec(self.embedding_name, (self.vocab_size, self.hidden_size), "embedding",
                            self.embedding_aliases)]
        for part in self.parts():
            specs.extend(part.all_tensor_specs())
        specs.extend(self.extra_tensors)
        seen, out = {}, []
        for s in specs:
            if s.name in seen:
                if seen[s.name].shape != s.shape:
                    raise ValueError(f"tensor '{s.name}' is wanted with shapes {seen[s.name].shape} and {s.shape}")
                continue
            more = tuple(other + s.name[len(prefix):] for prefix, other in self.alias_prefixes
                         if s.name.startswith(prefix))
            if more:
                s = dataclasses.replace(s, aliases=tuple(s.aliases) + more)
            seen[s.name] = s
            out.append(s)
        return out

    def state_specs(self):
        """State spec per state unit, taken from the entry that owns the unit."""
        n_units = 1 + max((e.state for e in self.plan), default=-1)
        specs = [None] * n_units
        owned = set()
        for e in self.plan:
            if e.owns_state:
                if e.state in owned:
                    raise ValueError(f"state unit {e.state} has two owners in the plan")
                owned.add(e.state)
                specs[e.state] = self.blocks[e.block].state_spec()
        for e in self.plan:
            if not e.owns_state and e.state not in owned:
                raise ValueError(f"plan reads state unit {e.state}, which no entry owns")
        return specs
