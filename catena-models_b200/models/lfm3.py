"""The LFM3 hybrid decoder as parts: which mixer, feed-forward, norms and position encoding
each layer gets, read from the typed configuration layer by layer.

Tensor names are the reference's `TensorSpec.name`s (src/spec.rs:714-808):
model.embed_tokens.weight; model.layers.{l}.{attn_norm,post_attention_norm,ffn_norm,
post_ffw_norm}.weight; shortconv.{in_proj,conv,out_proj}.weight on conv layers;
attn_{q,k,v,gate,output}.weight and attn_{q,k}_norm.weight on attention layers;
ffn_{gate,up,down}.weight; model.norm.weight; rope_freqs.weight; lm_head.weight when the head
is not tied.  Full-attention layers rotate with rope_theta and the per-frequency factors,
sliding layers with rope_theta_sliding and no factors (src/catena/lfm3.hex:726-734).
A file may carry the same tensors under the names the reference's GGUF checkpoints use
(`blk.{l}.*`, `token_embd.weight`, `output_norm.weight`, `output.weight`: the second name of
every entry of src/spec.rs:714-808).
"""
from __future__ import annotations

from ..config.lfm3 import Lfm3Config
from ..config.registry import register_architecture
from ..engine.definition import ModelDefinition, PlanEntry
from ..parts import build_part
from ..parts.linear import Linear
from ..weights.loader import TensorSpec


def define(cfg: Lfm3Config) -> ModelDefinition:
    H = cfg.hidden_size
    blocks = []
    for l, kind in enumerate(cfg.layer_types):
        prefix = f"model.layers.{l}."
        norm = lambda name: build_part("norm", "rms", name=prefix + name, width=H, eps=cfg.norm_eps)
        if kind == "conv":
            mixer = build_part("mixer", "short_conv", prefix=prefix, hidden=H, taps=cfg.conv_L_cache)
        else:
            sliding = kind == "sliding_attention"
            position = build_part("position", "rotary", head_dim=cfg.head_dim,
                                  theta=cfg.rope_theta_sliding if sliding else cfg.rope_theta,
                                  factors_name=None if sliding else "rope_freqs.weight")
            mixer = build_part("mixer", "gqa_attention", prefix=prefix, hidden=H,
                               heads=cfg.num_attention_heads, kv_heads=cfg.num_key_value_heads,
                               head_dim=cfg.head_dim, window=cfg.sliding_window if sliding else 0,
                               position=position, qk_norm_eps=cfg.norm_eps,
                               output_gate=cfg.attn_output_gate)
        ffn = build_part("feed_forward", "swiglu", prefix=prefix, hidden=H, intermediate=cfg.intermediate_size)
        blocks.append(build_part(
            "block", "sandwich", mixer=mixer, feed_forward=ffn,
            input_norm=norm("attn_norm.weight"), ffn_norm=norm("ffn_norm.weight"),
            post_mixer_norm=norm("post_attention_norm.weight") if cfg.post_norm else None,
            post_ffn_norm=norm("post_ffw_norm.weight") if cfg.post_norm else None))
    plan = [PlanEntry(block=b, state=i) for i, b in enumerate(cfg.layer_order)]
    head = None if cfg.tie_word_embeddings else Linear("lm_head.weight", cfg.vocab_size, H)
    definition = ModelDefinition(
        architecture=cfg.architecture, vocab_size=cfg.vocab_size, hidden_size=H,
        embedding_name="model.embed_tokens.weight", blocks=blocks, plan=plan,
        final_norm=build_part("norm", "rms", name="model.norm.weight", width=H, eps=cfg.norm_eps),
        head=head, stop_token_ids=tuple(cfg.eos_token_id), max_positions=cfg.max_position_embeddings,
        # rope_freqs.weight is part of every LFM3 checkpoint (src/spec.rs:789-794), also of one
        # whose layers are all sliding or conv and never read it
        extra_tensors=(TensorSpec("rope_freqs.weight", (cfg.head_dim // 2,), "rope_factors"),),
        alias_prefixes=(("model.layers.", "blk."), ("model.embed_tokens.weight", "token_embd.weight"),
                        ("model.norm.weight", "output_norm.weight"), ("lm_head.weight", "output.weight")))
    return definition


register_architecture("lfm3", Lfm3Config, define)
