"""A decoder put together from a `ModelDefinition`: embedding, the blocks in plan order, final
norm, output head.  It is the same class for every architecture; what differs is the
definition.  The forward pass runs only the tokens of the step's batch, reads and writes the
cache through the views the cache hands out, and returns float32 logits for the wanted rows
(src/lfm3.rs:333-524 is the reference's order of the same steps).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import adopt_tensors, load_tensors
from .runtime import Runtime


class DecoderModel:
    def __init__(self, definition, config, tensors, rt: Runtime):
        self.definition, self.config, self.rt = definition, config, rt
        self.vocab_size, self.hidden_size = definition.vocab_size, definition.hidden_size
        self.embedding = tensors[definition.embedding_name]
        for part in definition.parts():
            part.bind_all(tensors, rt)
        self.blocks, self.plan = definition.blocks, definition.plan
        self.final_norm, self.head = definition.final_norm, definition.head
        self.head_weight = self.embedding if self.head is None else self.head.weight
        self.state_specs = definition.state_specs()
        self.capturable = all(part.all_capturable() for part in definition.parts())   # decode graphs allowed
        self.prompt_capturable = all(part.all_prompt_capturable() for part in definition.parts())
        self.supports_append = all(part.all_support_append() for part in definition.parts())
        self.fusable_decode = all(part.all_fused_decode_ok() for part in definition.parts())
        self.token_error = rt.token_error

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, folder, dtype=torch.bfloat16, device="cuda:0"):
        from ..config.registry import config_from_folder

        arch, config = config_from_folder(folder)
        rt = Runtime(dtype, device)
        definition = arch.define(config)
        tensors = load_tensors(folder, definition.tensor_specs(), rt.device, widen=dtype == torch.float32)
        return cls(definition, config, tensors, rt)

    @classmethod
    def from_tensors(cls, config_dict, tensors, dtype=torch.bfloat16, device="cuda:0"):
        """Build from a configuration dict and {name: tensor} already in memory."""
        from ..config.registry import config_from_dict

        arch, config = config_from_dict(config_dict)
        rt = Runtime(dtype, device)
        definition = arch.define(config)
        bound = adopt_tensors(tensors, definition.tensor_specs(), rt.device, widen=dtype == torch.float32)
        return cls(definition, config, bound, rt)

    # ------------------------------------------------------------------ sizes
    def weight_bytes_per_step(self):
        """Bytes of weights one decode step reads: every matrix and vector once, and of the
        embedding table only the head's use of it (or the untied head)."""
        total = self.head_weight.numel() * self.head_weight.element_size()
        seen = set()
        for entry in self.plan:
            if entry.block in seen:
                total += self.blocks[entry.block].weight_bytes()     # a block that runs twice reads twice
            else:
                seen.add(entry.block)
                total += self.blocks[entry.block].weight_bytes()
        total += self.final_norm.weight_bytes()
        return total

    def parameter_count(self):
        specs = self.definition.tensor_specs()
        n = 0
        for s in specs:
            k = 1
            for d in s.shape:
                k *= d
            n += k
        return n

    # ------------------------------------------------------------------ forward
    def forward(self, batch, cache):
        self.rt._in_prompt = batch.kind != "decode"
        with kernels.pinned_stream():
            fuse = self.rt.fused_decode_for(batch) if self.fusable_decode else None
            if fuse is None:
                return self._forward(batch, cache)
            with fuse:                     # the step's small products and residual sums run in few persistent launches
                return self._forward(batch, cache)

    def _forward(self, batch, cache):
        rt = self.rt
        batch.shared.clear()
        if batch.layout.U:
            kernels.scatter_i32(cache.ptab_all, batch.upd_index, batch.upd_value, batch.upd_count, batch.layout.U)
        h = torch.empty((batch.T, self.hidden_size), dtype=rt.dtype, device=rt.device)
        kernels.embed_gather(h, self.embedding, batch.tokens, self.token_error, sampled=batch.prev_sampled,
                             scale=self.definition.embedding_scale)
        plan = self.plan
        first_norm = self.blocks[plan[0].block].input_norm
        n = first_norm.apply(rt, h) if first_norm is not None else None
        # when every row is wanted in order (a decode step), the last block's fused residual kernel
        # applies the final norm too and no rows need gathering
        whole = batch.wants_every_row and batch.n_want == batch.T
        for i, entry in enumerate(plan):
            block = self.blocks[entry.block]
            next_norm = (self.blocks[plan[i + 1].block].input_norm if i + 1 < len(plan)
                         else (self.final_norm if whole else None))
            state = cache.view(entry.state)
            if state is not None:
                state.owned, state.unit = entry.owns_state, entry.state
            h, n = block.forward(rt, batch, h, n, state, next_norm)
            if n is None and next_norm is not None and i + 1 < len(plan):
                n = next_norm.apply(rt, h)             # the block left the next block's norm to its caller
        if batch.n_want == 0:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=rt.device)
        if whole and n is not None:
            logits = rt.linear(n, self.head_weight, out_dtype=torch.float32)
        else:
            rows = torch.empty((batch.n_want, self.hidden_size), dtype=rt.dtype, device=rt.device)
            kernels.gather_rows(rows, h, batch.want_rows)
            normed = self.final_norm.apply(rt, rows)
            logits = rt.linear(normed, self.head_weight, out_dtype=torch.float32)
        d = self.definition
        if d.logit_scale != 1.0 or d.logit_softcap > 0.0:
            kernels.scale_softcap(logits, d.logit_scale, d.logit_softcap)
        return logits
