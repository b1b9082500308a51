"""Safetensors by name: dtype rule, one error for everything that is wrong, random folders."""
import json
import os

import pytest
import torch

import tiny
from catena_models_b200.config import registry
from catena_models_b200.weights import loader
from catena_models_b200.weights.loader import WeightError
from catena_models_b200.weights.random_init import random_tensors, write_random_model
from catena_models_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors


def specs_of(config):
    arch, cfg = registry.config_from_dict(config)
    return arch.define(cfg).tensor_specs()


def test_random_folder_loads_with_kept_dtypes(tmp_path):
    folder = tiny.make_folder(tmp_path, "B", seed=4)
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    with open(os.path.join(folder, "config.json")) as fh:
        assert json.load(fh) == tiny.TINY_B
    tensors = loader.load_tensors(folder, specs_of(tiny.TINY_B), "cpu")
    assert tensors["model.embed_tokens.weight"].dtype == torch.bfloat16          # stored bf16 stays bf16
    assert tensors["model.layers.0.shortconv.conv.weight"].dtype == torch.float32   # stored in 32 bits stays so
    assert tensors["model.layers.0.attn_norm.weight"].dtype == torch.float32
    wide = loader.load_tensors(folder, specs_of(tiny.TINY_B), "cpu", widen=True)
    assert all(t.dtype == torch.float32 for t in wide.values())
    assert torch.equal(wide["lm_head.weight"], tensors["lm_head.weight"].float())


def test_same_seed_same_tensors_and_independent_of_other_tensors(tmp_path):
    a = random_tensors(specs_of(tiny.TINY_A), seed=5)
    b = random_tensors(specs_of(tiny.TINY_A), seed=5)
    c = random_tensors(specs_of(tiny.TINY_A), seed=6)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    fewer = random_tensors(specs_of(tiny.TINY_A)[:3], seed=5)
    assert all(torch.equal(fewer[k], a[k]) for k in fewer)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = tiny.make_folder(tmp_path, "A", seed=1)
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n) for n in f.names()}
    f.close()
    del tensors["model.layers.1.attn_q.weight"], tensors["model.norm.weight"]
    tensors["model.layers.0.ffn_up.weight"] = torch.zeros(10, 64, dtype=torch.bfloat16)
    tensors["stray.weight"] = torch.zeros(3)
    tensors["model.layers.2.ffn_down.weight"] = tensors["model.layers.2.ffn_down.weight"].to(torch.float16)
    write_safetensors(path, tensors)
    with pytest.raises(WeightError) as err:
        loader.load_tensors(folder, specs_of(tiny.TINY_A), "cpu")
    e = err.value
    assert e.missing == ["model.layers.1.attn_q.weight", "model.norm.weight"]
    assert e.unexpected == ["stray.weight"]
    assert [w[0] for w in e.wrong_shape] == ["model.layers.0.ffn_up.weight"]
    assert [w[0] for w in e.wrong_dtype] == ["model.layers.2.ffn_down.weight"]
    text = str(e)
    for word in ("missing tensors", "unexpected tensors", "wrong shapes", "[10, 64]", "[176, 64]", "F16"):
        assert word in text


def test_untied_head_is_wanted_and_tied_head_is_refused_as_unexpected(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), tiny.TINY_B, 0)
    with pytest.raises(WeightError) as err:
        loader.load_tensors(folder, specs_of(dict(tiny.TINY_B, tie_word_embeddings=True)), "cpu")
    assert err.value.unexpected == ["lm_head.weight"]


def test_float32_matrix_stays_float32(tmp_path):
    folder = tiny.make_folder(tmp_path, "A", seed=1)
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n) for n in f.names()}
    f.close()
    tensors["model.layers.0.ffn_down.weight"] = tensors["model.layers.0.ffn_down.weight"].float()
    write_safetensors(path, tensors)
    got = loader.load_tensors(folder, specs_of(tiny.TINY_A), "cpu")
    assert got["model.layers.0.ffn_down.weight"].dtype == torch.float32
    assert got["model.layers.1.ffn_down.weight"].dtype == torch.bfloat16


def test_broken_files(tmp_path):
    p = tmp_path / "x.safetensors"
    p.write_bytes(b"\x01\x00")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    p.write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    header = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(len(header).to_bytes(8, "little") + header + b"\0" * 8)
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))                                   # 8 bytes for 4 floats
    header = b'{"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},"a":{"dtype":"F32","shape":[1],"data_offsets":[4,8]}}'
    p.write_bytes(len(header).to_bytes(8, "little") + header + b"\0" * 8)
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))                                   # a name twice
    with pytest.raises(WeightError):
        loader.load_tensors(str(tmp_path / "nowhere"), [], "cpu")


def test_round_trip_values(tmp_path):
    t = {"w": torch.randn(5, 7).to(torch.bfloat16), "v": torch.arange(6, dtype=torch.float32), "i": torch.arange(4, dtype=torch.int32)}
    write_safetensors(str(tmp_path / "t.safetensors"), t)
    f = SafetensorsFile(str(tmp_path / "t.safetensors"))
    assert all(torch.equal(f.tensor(k), v) for k, v in t.items())
    from safetensors.torch import load_file
    other = load_file(str(tmp_path / "t.safetensors"))              # the reference implementation reads it too
    assert all(torch.equal(other[k], v) for k, v in t.items())


def test_the_reference_checkpoint_names_are_accepted(tmp_path):
    """The same tensors under the names of the reference's GGUF checkpoints (blk.{l}.*,
    token_embd.weight, output_norm.weight, output.weight; src/spec.rs:428-441, 714-808) load to the
    same values; a tensor present under both names leaves one of them unexpected."""
    folder = tiny.make_folder(tmp_path, "B", seed=2)
    specs = specs_of(tiny.TINY_B)
    first = loader.load_tensors(folder, specs, "cpu")
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    stored = {n: f.tensor(n) for n in f.names()}
    f.close()

    def other(name):
        if name.startswith("model.layers."):
            return "blk." + name[len("model.layers."):]
        return {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
                "lm_head.weight": "output.weight"}.get(name, name)

    renamed = {other(n): t for n, t in stored.items()}
    assert "blk.0.shortconv.in_proj.weight" in renamed and "rope_freqs.weight" in renamed
    write_safetensors(path, renamed)
    again = loader.load_tensors(folder, specs, "cpu")
    assert set(again) == set(first) and all(torch.equal(again[k], first[k]) for k in first)
    renamed["model.norm.weight"] = renamed["output_norm.weight"]
    write_safetensors(path, renamed)
    with pytest.raises(WeightError) as err:
        loader.load_tensors(folder, specs, "cpu")
    assert err.value.unexpected == ["output_norm.weight"] and not err.value.missing
