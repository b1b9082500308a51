"""Typed configuration, its errors, and the architecture registry (no device needed)."""
import copy
import json

import pytest

import tiny
from catena_models_b200.config.base import ConfigError
from catena_models_b200.config.lfm3 import Lfm3Config
from catena_models_b200.config import registry


def test_reads_every_key_and_defaults():
    cfg = Lfm3Config.from_dict(tiny.TINY_A)
    assert cfg.hidden_size == 64 and cfg.head_dim == 16 and cfg.conv_L_cache == 3
    assert cfg.layer_types == ("conv", "sliding_attention", "conv", "full_attention")
    assert cfg.rope_theta_sliding == cfg.rope_theta == 10000.0        # default: the full layers' base
    assert cfg.eos_token_id == (7,) and cfg.layer_order == (0, 1, 2, 3)
    b = Lfm3Config.from_dict(tiny.TINY_B)
    assert b.rope_theta_sliding == 10000.0 and b.rope_theta == 1e6 and not b.tie_word_embeddings
    assert b.eos_token_id == (3, 11) and not b.attn_output_gate
    d = dict(tiny.TINY_A)
    del d["head_dim"]
    assert Lfm3Config.from_dict(d).head_dim == 64 // 4                # hidden / heads when absent


def test_round_trip_through_json():
    cfg = Lfm3Config.from_dict(tiny.TINY_B)
    again = Lfm3Config.from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert again == cfg


@pytest.mark.parametrize("change, word", [
    (dict(hidden_size=None), "hidden_size"),
    (dict(vocab_size="many"), "vocab_size"),
    (dict(layer_types=["conv", "attention", "conv", "conv"]), "unknown entries"),
    (dict(layer_types=["conv"]), "layer_types has 1"),
    (dict(num_key_value_heads=3), "divisible"),
    (dict(head_dim=20), "head_dim"),
    (dict(head_dim=264, hidden_size=1056), "head_dim 264"),
    (dict(hidden_size=8200), "hidden_size 8200"),
    (dict(conv_L_cache=17), "conv_L_cache 17"),
    (dict(conv_L_cache=1), "conv_L_cache"),
    (dict(sliding_window=0), "sliding_window"),
    (dict(rope_theta=-1.0), "rope_theta"),
    (dict(norm_eps=float("nan")), "norm_eps"),
    (dict(tie_word_embeddings="yes"), "tie_word_embeddings"),
    (dict(layer_order=[0, 9]), "layer_order"),
    (dict(eos_token_id=999), "eos_token_id"),
])
def test_bad_values_are_named(change, word):
    d = copy.deepcopy(tiny.TINY_A)
    for k, v in change.items():
        if v is None:
            d.pop(k)
        else:
            d[k] = v
    with pytest.raises(ConfigError) as err:
        Lfm3Config.from_dict(d)
    assert word in str(err.value)


def test_all_problems_in_one_error():
    d = dict(tiny.TINY_A)
    del d["vocab_size"], d["norm_eps"]
    d["intermediate_size"] = 1.5
    with pytest.raises(ConfigError) as err:
        Lfm3Config.from_dict(d)
    text = str(err.value)
    assert "vocab_size" in text and "norm_eps" in text and "intermediate_size" in text


def test_registry_resolves_and_lists():
    arch, cfg = registry.config_from_dict(tiny.TINY_A)
    assert arch.name == "lfm3" and isinstance(cfg, Lfm3Config)
    with pytest.raises(ConfigError) as err:
        registry.config_from_dict(dict(tiny.TINY_A, architecture="qwen9"))
    assert "lfm3" in str(err.value) and "qwen9" in str(err.value)
    with pytest.raises(ValueError):
        registry.register_architecture("lfm3", Lfm3Config, lambda c: None)


def test_definition_follows_the_configuration():
    from catena_models_b200.cache.spec import FixedStateSpec, KVStateSpec

    arch, cfg = registry.config_from_dict(tiny.TINY_B)
    d = arch.define(cfg)
    kinds = [type(b.mixer).__name__ for b in d.blocks]
    assert kinds == ["ShortConv", "ShortConv", "GQAttention", "ShortConv", "GQAttention", "GQAttention"]
    states = d.state_specs()
    assert states[0] == FixedStateSpec((3, 96), "float32")
    assert states[2] == KVStateSpec(1, 24, 0) and states[4] == KVStateSpec(1, 24, 8)
    names = {s.name: s for s in d.tensor_specs()}
    assert names["lm_head.weight"].shape == (384, 96)
    assert "model.layers.2.attn_gate.weight" not in names               # gate off in B
    assert names["model.layers.0.shortconv.conv.weight"].shape == (96, 4)
    assert names["rope_freqs.weight"].shape == (12,)
    a = registry.config_from_dict(tiny.TINY_A)
    da = a[0].define(a[1])
    na = {s.name for s in da.tensor_specs()}
    assert "lm_head.weight" not in na and "model.layers.1.attn_gate.weight" in na
    # sliding layers: own base, no factors
    sliding = da.blocks[1].mixer.position
    assert sliding.factors_name is None and da.blocks[3].mixer.position.factors_name == "rope_freqs.weight"


def test_layer_order_is_data():
    arch, cfg = registry.config_from_dict(dict(tiny.TINY_A, layer_order=[0, 1, 1, 3, 2]))
    d = arch.define(cfg)
    assert [e.block for e in d.plan] == [0, 1, 1, 3, 2]
    assert len(d.state_specs()) == 5                                   # a layer that runs twice has two states


def test_limits_are_the_kernels_own():
    """The sizes the configuration check refuses are read from the header the CUDA sources include;
    the numbers stand nowhere else."""
    import re

    from catena_models_b200.csrc import limits

    text = open(limits._HEADER).read()
    for name in limits.NAMES:
        assert re.search(rf"#define\s+CM_{name}\s+{getattr(limits, name)}\b", text)
    d = dict(tiny.TINY_A, hidden_size=limits.NORM_MAX_WIDTH, num_attention_heads=512, num_key_value_heads=512)
    Lfm3Config.from_dict(d)                                   # the limit itself passes
    with pytest.raises(ConfigError):
        Lfm3Config.from_dict(dict(d, hidden_size=limits.NORM_MAX_WIDTH + 8))
