"""Configuration of the LFM3 hybrid decoder.

The keys mirror the metadata that catena-models reads for this architecture
(src/checkpoint.rs:422-625: block_count, embedding_length, feed_forward_length,
attention.head_count, attention.head_count_kv[], attention.key_length,
attention.sliding_window, attention.sliding_window_pattern[], attention.layer_norm_rms_epsilon,
rope.freq_base, rope.freq_base_swa, shortconv.l_cache, context_length, vocab_size,
tokenizer.ggml.eos_token_id), written as config.json keys.  The host-side checks are those
of src/spec.rs:185-249.
"""
from __future__ import annotations

import dataclasses

from ..csrc import limits
from .base import ConfigError, Reader

LAYER_TYPES = ("conv", "full_attention", "sliding_attention")


@dataclasses.dataclass(frozen=True)
class Lfm3Config:
    architecture: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    layer_types: tuple          # per layer: conv | full_attention | sliding_attention
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    conv_L_cache: int           # taps of the short convolution; its state keeps L_cache - 1 rows
    sliding_window: int
    rope_theta: float
    rope_theta_sliding: float   # base of the sliding layers, which also ignore the rope factors
    norm_eps: float
    tie_word_embeddings: bool
    max_position_embeddings: int
    eos_token_id: tuple         # zero or more stop ids
    post_norm: bool             # RMSNorm on the mixer's and the feed-forward's output
    attn_output_gate: bool      # per-head sigmoid gate on the attention output
    layer_order: tuple          # the order in which layers run, as indices into the layers

    @classmethod
    def from_dict(cls, data, where="config.json"):
        r = Reader(data, where)
        arch = r.string("architecture", default=data.get("model_type", "lfm3"))
        layers = r.integer("num_hidden_layers", minimum=1)
        heads = r.integer("num_attention_heads", minimum=1)
        hidden = r.integer("hidden_size", minimum=1)
        default_hd = hidden // heads if hidden and heads else None
        fields = dict(
            architecture=arch,
            vocab_size=r.integer("vocab_size", minimum=1),
            hidden_size=hidden,
            intermediate_size=r.integer("intermediate_size", minimum=1),
            num_hidden_layers=layers,
            layer_types=r.string_list("layer_types", allowed=LAYER_TYPES),
            num_attention_heads=heads,
            num_key_value_heads=r.integer("num_key_value_heads", minimum=1),
            head_dim=r.integer("head_dim", default=default_hd, minimum=1),
            conv_L_cache=r.integer("conv_L_cache", minimum=2),
            sliding_window=r.integer("sliding_window", minimum=1),
            rope_theta=r.number("rope_theta", positive=True),
            rope_theta_sliding=None,
            norm_eps=r.number("norm_eps", positive=True),
            tie_word_embeddings=r.boolean("tie_word_embeddings", default=True),
            max_position_embeddings=r.integer("max_position_embeddings", minimum=1),
            eos_token_id=r.integer_list("eos_token_id", default=()),
            post_norm=r.boolean("post_norm", default=True),
            attn_output_gate=r.boolean("attn_output_gate", default=True),
            layer_order=r.integer_list("layer_order", default=None),
        )
        fields["rope_theta_sliding"] = r.number("rope_theta_sliding", default=fields["rope_theta"], positive=True)
        if fields["layer_order"] is None and layers:
            fields["layer_order"] = tuple(range(layers))
        r.finish()
        cfg = cls(**fields)
        cfg.validate(where)
        return cfg

    def validate(self, where="config"):
        problems = []
        if len(self.layer_types) != self.num_hidden_layers:
            problems.append(f"layer_types has {len(self.layer_types)} entries for {self.num_hidden_layers} layers")
        if self.num_attention_heads % self.num_key_value_heads:
            problems.append("num_attention_heads must be divisible by num_key_value_heads")
        if self.head_dim % 8 or self.head_dim > limits.MAX_HEAD_DIM:
            problems.append(f"head_dim {self.head_dim}: the kernels take multiples of 8 up to {limits.MAX_HEAD_DIM}")
        if self.hidden_size % 8 or self.intermediate_size % 8:
            problems.append("hidden_size and intermediate_size must be multiples of 8 (16-byte rows)")
        if self.hidden_size > limits.NORM_MAX_WIDTH:
            problems.append(f"hidden_size {self.hidden_size}: the norm kernels keep a row of at most "
                            f"{limits.NORM_MAX_WIDTH} in registers")
        if self.conv_L_cache > limits.MAX_CONV_TAPS:
            problems.append(f"conv_L_cache {self.conv_L_cache}: the kernels take up to {limits.MAX_CONV_TAPS} taps")
        if any(i < 0 or i >= self.num_hidden_layers for i in self.layer_order):
            problems.append("layer_order names a layer that does not exist")
        if any(t < 0 or t >= self.vocab_size for t in self.eos_token_id):
            problems.append("eos_token_id outside the vocabulary")
        if problems:
            raise ConfigError(f"{where}: " + "; ".join(problems))

    def to_dict(self):
        d = dataclasses.asdict(self)
        d["layer_types"] = list(self.layer_types)
        d["eos_token_id"] = list(self.eos_token_id)
        d["layer_order"] = list(self.layer_order)
        return d
