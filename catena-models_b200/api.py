"""The Python entry point, in the manner of catena-models' library API
(`Model::load_gguf`, `model.config()`, `model.logits(tokens)`, `model.next_token(tokens)`,
`model.session(capacity)` and the session's `prefill_*` / `decode_*` calls,
src/model.rs:32-60, 155-206, 429-502), plus batched generation.

    model = Model.load("folder")                        # config.json + model.safetensors
    model = Model.random(config_dict, seed=0)           # random weights, no files
    out = model.generate([[1, 2, 3], [4, 5]], max_new_tokens=20, temperature=0.8, seed=1)
    s = model.session(capacity=256); t = s.prefill_next_token([1, 2, 3]); t = s.decode_next_token(t)
"""
from __future__ import annotations

import torch

from .engine.engine import Engine
from .engine.generate import generate as _generate
from .engine.model import DecoderModel
from .sampling.sampler import Sampler

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def _dtype(d):
    try:
        return _DTYPES[d]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {d!r}") from None


class Checkpoint:
    """The state of a session that was set aside (`Session.into_checkpoint`, src/model.rs:208-246,
    431-446): it keeps the sequence's slot of the cache until it is closed.  `Model.resume_checkpoint`
    starts any number of sessions from it, each on a copy of its own."""

    def __init__(self, model, slot, capacity):
        self.model, self.slot, self.capacity = model, slot, capacity

    @property
    def position(self):
        return self.model.engine.length(self.slot)

    def close(self):
        if self.slot is not None:
            self.model.engine.release([self.slot])
            self.slot = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class Session:
    """One sequence on a slot of the model's cache (src/model.rs:420-502)."""

    def __init__(self, model, capacity, _slot=None):
        self.model, self.capacity = model, capacity
        if _slot is None:
            (_slot,) = model.engine.admit(1)
        self.slot = _slot
        self._greedy = Sampler(model.device)

    @property
    def position(self):
        return self.model.engine.length(self.slot)

    def _run(self, tokens):
        if self.position + len(tokens) > self.capacity:
            raise ValueError(f"session capacity {self.capacity} exceeded")
        return self.model.engine.step([self.slot], [list(tokens)])

    def _to_host(self, logits):
        out = logits[0].float().cpu()
        self.model.engine.check_errors()                       # the copy has synchronised: the flags are final
        return out

    def prefill_logits(self, tokens):
        return self._to_host(self._run(tokens))

    def decode_logits(self, token):
        return self._to_host(self._run([token]))

    def prefill_next_token(self, tokens):
        return self._greedy.sample(self._run(tokens), [0], [0])[0]

    def decode_next_token(self, token):
        return self._greedy.sample(self._run([token]), [0], [0])[0]

    def append_logits(self, tokens):
        """Logits after `tokens` on top of what the session holds, in one step wherever the session
        stands (`Session::forward` takes any number of tokens at any position, src/model.rs:692-731).
        A model with a part that has no append form takes them one by one."""
        tokens = list(tokens)
        if not tokens:
            raise ValueError("append needs at least one token")
        if self.position == 0 or self.model.decoder.supports_append:
            return self.prefill_logits(tokens)
        if self.position + len(tokens) > self.capacity:
            raise ValueError(f"session capacity {self.capacity} exceeded")
        for t in tokens[:-1]:
            self._run([t])
        return self.decode_logits(tokens[-1])

    def append_next_token(self, tokens):
        logits = self.append_logits(tokens)
        return int(torch.argmax(logits))                      # the first of equal maxima, as the device sampler

    def into_checkpoint(self):
        """Sets the session's state aside; the session itself is over."""
        if self.slot is None:
            raise ValueError("the session is closed")
        ckpt = Checkpoint(self.model, self.slot, self.capacity)
        self.slot = None
        return ckpt

    def close(self):
        if self.slot is not None:
            self.model.engine.release([self.slot])
            self.slot = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class Model:
    def __init__(self, decoder, max_tokens, max_seqs=None, use_graphs=True):
        self.decoder = decoder
        self.device = decoder.rt.device
        self.engine = Engine(decoder, max_tokens, max_seqs, use_graphs)

    @classmethod
    def load(cls, folder, dtype="bfloat16", device="cuda:0", max_tokens=65536, max_seqs=None, use_graphs=True):
        return cls(DecoderModel.from_folder(folder, _dtype(dtype), device), max_tokens, max_seqs, use_graphs)

    @classmethod
    def random(cls, config, seed=0, std=0.02, norm_weights="ones", rope_factors="ones", dtype="bfloat16",
               device="cuda:0", max_tokens=65536, max_seqs=None, use_graphs=True):
        """A model with random weights made directly on the device (no files)."""
        from .config.registry import config_from_dict
        from .weights.random_init import random_tensors

        arch, typed = config_from_dict(config)
        tensors = random_tensors(arch.define(typed).tensor_specs(), seed, std, norm_weights, rope_factors, device)
        return cls(DecoderModel.from_tensors(config, tensors, _dtype(dtype), device), max_tokens, max_seqs, use_graphs)

    @property
    def config(self):
        return self.decoder.config

    def parameter_count(self):
        return self.decoder.parameter_count()

    def session(self, capacity):
        return Session(self, capacity)

    def resume_checkpoint(self, checkpoint):
        """A new session that starts from a copy of the checkpoint's state.  Refused for a checkpoint
        of another model (src/model.rs:210-213)."""
        if checkpoint.model is not self:
            raise ValueError("the checkpoint belongs to another model")
        if checkpoint.slot is None:
            raise ValueError("the checkpoint is closed")
        (slot,) = self.engine.admit(1)
        try:
            self.engine.cache.copy_slot(checkpoint.slot, slot)
        except Exception:
            self.engine.release([slot])
            raise
        return Session(self, checkpoint.capacity, _slot=slot)

    def logits(self, tokens):
        """Logits after the last of `tokens`, as float32 on the host (src/model.rs:187-190)."""
        with self.session(len(tokens)) as s:
            return s.prefill_logits(tokens)

    def next_token(self, tokens):
        with self.session(len(tokens)) as s:
            return s.prefill_next_token(tokens)

    def generate(self, prompts, max_new_tokens=20, temperature=0.0, seed=0, stop_token_ids=None, ignore_eos=False,
                 max_batch=64, on_step=None):
        """Batched generation; returns a `Generation` (tokens, finish_reason) per prompt."""
        if stop_token_ids is None:
            stop_token_ids = self.decoder.definition.stop_token_ids
        sampler = Sampler(self.device, temperature, seed)
        return _generate(self.engine, sampler, prompts, max_new_tokens, stop_token_ids, ignore_eos, max_batch,
                         on_step=on_step)
