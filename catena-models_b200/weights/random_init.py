"""Random weights from a configuration and a seed.

catena-models has no random-weights mode (it always reads a checkpoint); this one exists so
that tests and benchmarks need no files from a network.  Every tensor is drawn from its own
generator, seeded by (seed, tensor name), so a tensor's values do not depend on which other
tensors the model has or in which order they are made.

Matrices and embeddings: N(0, std) in bfloat16.  Norm weights: 1, or 1 + N(0, 0.1) with
`norm_weights="random"`.  Conv taps: N(0, std) in float32.  Rope factors: 1, or uniform in
[1, 4) with `rope_factors="uniform"`.
"""
from __future__ import annotations

import hashlib
import json
import os

import torch

from .safetensors_io import write_safetensors


def _generator(seed, name, device):
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device=device)
    g.manual_seed(int.from_bytes(digest[:8], "little") & ((1 << 63) - 1))
    return g


def random_tensors(specs, seed, std=0.02, norm_weights="ones", rope_factors="ones", device="cpu"):
    """{name: tensor} for a list of TensorSpec, in the dtypes a checkpoint would store."""
    out = {}
    for spec in specs:
        g = _generator(seed, spec.name, device)
        shape = tuple(spec.shape)
        if spec.role in ("matrix", "embedding"):
            t = (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std).to(torch.bfloat16)
        elif spec.role == "norm":
            t = torch.ones(shape, device=device, dtype=torch.float32)
            if norm_weights == "random":
                t = t + 0.1 * torch.randn(shape, generator=g, device=device, dtype=torch.float32)
        elif spec.role == "conv":
            t = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std
        elif spec.role == "rope_factors":
            t = torch.ones(shape, device=device, dtype=torch.float32)
            if rope_factors == "uniform":
                t = 1.0 + 3.0 * torch.rand(shape, generator=g, device=device, dtype=torch.float32)
        elif spec.role == "table":
            t = torch.zeros(shape, device=device, dtype=torch.int32)
        else:
            t = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std
        out[spec.name] = t
    return out


def write_random_model(folder, config, seed, std=0.02, norm_weights="ones", rope_factors="ones"):
    """Write `folder/config.json` and `folder/model.safetensors` for a configuration dict."""
    from ..config.registry import config_from_dict

    arch, typed = config_from_dict(config, where="random model config")
    definition = arch.define(typed)
    tensors = random_tensors(definition.tensor_specs(), seed, std, norm_weights, rope_factors, "cpu")
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(config, fh, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": seed, "std": std})
    return folder
