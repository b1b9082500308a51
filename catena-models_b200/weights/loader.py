"""Weights by tensor name.

A model definition lists the tensors it needs (`TensorSpec`: name, shape, role); the loader
finds them in the model folder's safetensors file(s), checks the whole inventory at once and
raises a single `WeightError` that lists missing tensors, unexpected tensors, wrong shapes and
unusable dtypes (catena-models: spec list against file inventory, src/checkpoint.rs:659-729;
safetensors lookup by name, src/weights.rs:104-120).

Storage rule: a tensor stored in bfloat16 stays bfloat16, a tensor stored in 32 bits stays in
32 bits, integer tables become int32; float16 is refused as the reference refuses it
(src/model.rs:118-122).  Small float vectors that kernels read as float (norm weights, conv
taps, rope factors: roles other than "matrix") are widened to float32, which changes no value.
With `widen=True` (the 32-bit engine) every float tensor is widened to float32.
"""
from __future__ import annotations

import dataclasses
import json
import os

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile

SINGLE_FILE = "model.safetensors"
INDEX_FILE = "model.safetensors.index.json"
LISTED = 16            # names shown per category in an error


@dataclasses.dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: tuple
    role: str = "matrix"      # matrix | embedding | norm | conv | rope_factors | vector | table
    aliases: tuple = ()       # other names the same tensor may carry in a file


class WeightError(ValueError):
    """The file inventory does not match what the model needs."""

    def __init__(self, where, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=(), other=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype, self.other = list(wrong_shape), list(wrong_dtype), list(other)
        parts = []

        def show(title, items):
            if items:
                head = ", ".join(str(i) for i in items[:LISTED])
                more = f" (+{len(items) - LISTED} more)" if len(items) > LISTED else ""
                parts.append(f"{title} [{len(items)}]: {head}{more}")

        show("missing tensors", self.missing)
        show("unexpected tensors", self.unexpected)
        show("wrong shapes", [f"{n}: file {list(f)} != model {list(e)}" for n, f, e in self.wrong_shape])
        show("unusable dtypes", [f"{n}: {d}" for n, d in self.wrong_dtype])
        show("other", self.other)
        super().__init__(f"{where}: " + "; ".join(parts))


def open_folder(folder):
    """name -> (SafetensorsFile, name) for one file or an indexed set of shards."""
    single = os.path.join(folder, SINGLE_FILE)
    index = os.path.join(folder, INDEX_FILE)
    files, table = {}, {}
    if os.path.exists(index):
        with open(index) as fh:
            weight_map = json.load(fh).get("weight_map", {})
        for name, shard in weight_map.items():
            if shard not in files:
                files[shard] = SafetensorsFile(os.path.join(folder, shard))
            if name not in files[shard].entries:
                raise WeightError(folder, other=[f"index places '{name}' in {shard}, which does not hold it"])
            table[name] = files[shard]
        for shard, f in files.items():
            for name in f.names():
                if name not in table:
                    raise WeightError(folder, other=[f"{shard} holds '{name}', which the index does not list"])
    elif os.path.exists(single):
        f = SafetensorsFile(single)
        files[SINGLE_FILE] = f
        table = {name: f for name in f.names()}
    else:
        raise WeightError(folder, other=[f"neither {SINGLE_FILE} nor {INDEX_FILE} found"])
    return files, table


def _target_dtype(stored, role, widen):
    """The dtype a tensor is kept in, or None when the stored dtype cannot be used."""
    if role == "table":
        return torch.int32 if stored in ("I64", "I32", "I16", "I8", "U8") else None
    if stored == "BF16":
        return torch.float32 if (widen or role not in ("matrix", "embedding")) else torch.bfloat16
    if stored == "F32":
        return torch.float32
    return None


def check_inventory(where, specs, found, widen=False):
    """`found`: name -> (dtype string, shape).  Returns {spec name: file name}; raises one
    WeightError for everything that is wrong."""
    chosen, missing, wrong_shape, wrong_dtype = {}, [], [], []
    used = set()
    for spec in specs:
        name = next((n for n in (spec.name, *spec.aliases) if n in found), None)
        if name is None:
            missing.append(spec.name)
            continue
        used.add(name)
        dtype, shape = found[name]
        if tuple(shape) != tuple(spec.shape):
            wrong_shape.append((spec.name, shape, spec.shape))
        elif _target_dtype(dtype, spec.role, widen) is None:
            wrong_dtype.append((spec.name, f"{dtype} cannot serve as {spec.role}"))
        else:
            chosen[spec.name] = name
    unexpected = sorted(n for n in found if n not in used)
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(where, missing, unexpected, wrong_shape, wrong_dtype)
    return chosen


def load_tensors(folder, specs, device, widen=False, progress=None):
    """{spec name: tensor on `device`} for every spec, after the inventory check."""
    try:
        files, table = open_folder(folder)
    except SafetensorsError as exc:
        raise WeightError(folder, other=[str(exc)]) from exc
    try:
        found = {name: f.info(name) for name, f in table.items()}
        chosen = check_inventory(folder, specs, found, widen)
        out = {}
        for i, spec in enumerate(specs):
            src = chosen[spec.name]
            stored, _ = found[src]
            t = table[src].tensor(src).to(_target_dtype(stored, spec.role, widen))
            out[spec.name] = t.to(device)
            if progress and (i + 1) % 64 == 0:
                progress(i + 1, len(specs))
        return out
    finally:
        for f in files.values():
            f.close()


def adopt_tensors(tensors, specs, device, widen=False, where="tensors"):
    """The same checks and dtype rule for tensors that are already in memory (random weights
    made on the device): returns {spec name: tensor on `device`}."""
    from .safetensors_io import NAMES

    found = {n: (NAMES.get(t.dtype, str(t.dtype)), tuple(t.shape)) for n, t in tensors.items()}
    chosen = check_inventory(where, specs, found, widen)
    out = {}
    for spec in specs:
        t = tensors[chosen[spec.name]]
        out[spec.name] = t.to(device=device, dtype=_target_dtype(found[chosen[spec.name]][0], spec.role, widen))
    return out
