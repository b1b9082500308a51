"""Interfaces of the parts that layers are put together from, and their registries.

Five kinds of part exist: `mixer` (attention, short convolution, ...), `feed_forward`,
`norm`, `position` (position encoding) and `block` (the arrangement of the others in one
layer).  A part is built from parameters only (sizes and constants come from a configuration
through the model definition, never from this package's code) and does not know which model
or which layer it is in.  A part that needs tensors lists them with full names in
`tensor_specs()` and receives them, on the device and in their kept dtype, in `bind()`.

    register_part("mixer", "my_mixer", MyMixer)     # open to tests and later architectures
    build_part("mixer", "my_mixer", **params)

Interfaces (x, h, n are [tokens, width] activations of the step's packed batch):

    Norm.apply(rt, x) -> y                      weight, eps: attributes the fused kernels read
    Position.rate_table() -> float32 [head_dim/2] or None    (angle = position * rate[i])
    Mixer.state_spec() -> KVStateSpec | FixedStateSpec | None
    Mixer.forward(rt, batch, x, state) -> y     state: the cache's view for this layer
    FeedForward.forward(rt, batch, x) -> y
    Block.input_norm                            the norm applied to h before the block runs, or None
    Block.forward(rt, batch, h, n, state, next_norm) -> (h, n_next)
        n = input_norm(h) was made by whoever ran before (None if the block names no input_norm:
        it then takes what it needs from h itself); n_next = next_norm(h) is made here (fused
        with the last residual sum) when next_norm is given and the block can, else None: whoever
        runs next then applies its norm itself.

A part sets `capturable = False` if its forward() reads device data on the host,
`prompt_capturable = True` if its prompt steps may be recorded as well, and
`supports_append = True` if it handles steps of kind "append" (see Part).

`rt` is the engine's Runtime (dtype, device, scratch), `batch` the StepBatch (token
positions, sequence boundaries, slots, prefill or decode).
"""
from __future__ import annotations

CATEGORIES = ("mixer", "feed_forward", "norm", "position", "block")
_PARTS = {c: {} for c in CATEGORIES}


def register_part(category, kind, cls, replace=False):
    if category not in _PARTS:
        raise ValueError(f"unknown part category '{category}'; one of {CATEGORIES}")
    if kind in _PARTS[category] and not replace:
        raise ValueError(f"{category} '{kind}' is already registered")
    _PARTS[category][kind] = cls


def part_kinds(category):
    return sorted(_PARTS[category])


def build_part(category, kind, **params):
    try:
        cls = _PARTS[category][kind]
    except KeyError:
        raise ValueError(f"unknown {category} '{kind}'; registered: {part_kinds(category)}") from None
    return cls(**params)


class Part:
    """Base of every part: no tensors, nothing to bind."""

    # False for a part whose forward() lets the host look at device data (a routed feed-forward
    # that gathers each expert's tokens, say): its launches differ from step to step, so decode
    # steps of a model that holds such a part are run kernel by kernel instead of being replayed
    # from a captured graph.
    capturable = True
    # True for a part whose prompt steps too launch the same kernels whenever the batch has the same
    # class of shape (number of sequences, rows, longest prompt as StepBatch.max_len, wanted places), that
    # takes everything about the real lengths from the step's device metadata, and that leaves rows of
    # padding alone (StepBatch.tok_seq is -1 there: they belong to no sequence and must touch no state; what
    # the part returns for them is never used):
    # the engine may then record a prompt step of a class into a graph and replay it for every prompt
    # of the class.  With supports_append this holds for steps of kind "append" too, whose class also
    # names the class of lengths that the longest sequence reaches (StepBatch.max_end is then that
    # class's bound, not the real end).  A part says so itself; one that does not know is not recorded.
    prompt_capturable = False
    # True for a part that can take a step of kind "append" (StepBatch.kind): sequences that stand at
    # any position and bring any number of tokens.  A part that works row by row (norm, feed-forward,
    # projection) can; a mixer with state has to say so itself, after it has made sure that its
    # forward() reads what is older than the step from its state.  A model with a part that cannot
    # is stepped with whole prompts and single tokens only.
    supports_append = False
    # True for a part whose decode steps (one token per sequence) launch nothing but this library's
    # kernels, in program order, on tensors that stay alive until the step ends: its products, residual
    # sums and convolution may then be collected and run inside one persistent kernel
    # (kernels.FusedDecode).  A part that runs torch operations of its own between kernels must leave
    # this False: those would overtake the collected calls.
    fused_decode_ok = False

    def tensor_specs(self):
        return []

    def bind(self, tensors, rt):
        """Take this part's tensors out of {name: device tensor}."""

    def children(self):
        """Parts nested in this one (their tensors are listed and bound with it)."""
        return []

    def all_tensor_specs(self):
        out = list(self.tensor_specs())
        for child in self.children():
            out.extend(child.all_tensor_specs())
        return out

    def bind_all(self, tensors, rt):
        for child in self.children():
            child.bind_all(tensors, rt)
        self.bind(tensors, rt)

    def all_capturable(self):
        return self.capturable and all(c.all_capturable() for c in self.children())

    def all_fused_decode_ok(self):
        return self.fused_decode_ok and all(c.all_fused_decode_ok() for c in self.children())

    def all_support_append(self):
        return self.supports_append and all(c.all_support_append() for c in self.children())

    def all_prompt_capturable(self):
        return self.capturable and self.prompt_capturable and all(c.all_prompt_capturable() for c in self.children())

    def weight_bytes(self):
        """Bytes of weights a step reads from this part (each tensor once)."""
        own = sum(t.numel() * t.element_size() for t in getattr(self, "_bound", ()))
        return own + sum(c.weight_bytes() for c in self.children())


class Mixer(Part):
    def state_spec(self):
        return None

    def forward(self, rt, batch, x, state):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, rt, batch, x):
        raise NotImplementedError


class Norm(Part):
    def apply(self, rt, x):
        raise NotImplementedError


class Position(Part):
    # which elements of a head form a rotation pair: "half" pairs i with i + head_dim/2 (the reference's
    # rotate-half form), "interleaved" pairs 2i with 2i + 1; rate_table()[i] is pair i's rate either way
    pairing = "half"

    def rate_table(self):
        return None


class Block(Part):
    input_norm = None

    def state_spec(self):
        return None

    def forward(self, rt, batch, h, n, state, next_norm):
        raise NotImplementedError
