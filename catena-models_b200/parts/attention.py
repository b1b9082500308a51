"""Grouped-query attention mixer with head RMSNorm on q and k, a position encoding, a full or
sliding causal mask and an optional per-head sigmoid gate on the output.

Order of operations (src/lfm3.rs:390-464): one matrix product over the packed rows
[Wq; Wk; Wv; Wgate] (src/lfm3.rs:1159-1262); head norm and rotation of q and k, k and the raw v
written to the cache (src/catena/lfm3.hex:622-781); scores scaled by 1/sqrt(head_dim), keys
hidden when k > p or, with a window W, when k + W <= p (src/catena/lfm3.hex:48-57); softmax and
the value sum in float; context times sigmoid(gate) per head (src/catena/lfm3.hex:25-46);
output projection.

A prompt step attends over the step's own keys and values (every sequence of such a step
starts at position 0); a decode step attends over the cache; an append step (several tokens on
top of started sequences) reads the keys below each sequence's first new position from the cache
and the rest from the step, and writes the step's keys and values to the cache afterwards, so
that a ring still holds what the step's windows reach back to.  All sizes and switches are
constructor parameters; the part knows neither its layer index nor its model.
"""
from __future__ import annotations


import torch

from .. import kernels
from ..cache.spec import KVStateSpec
from ..csrc.limits import ATTN_DECODE_CHUNK
from ..weights.loader import TensorSpec
from .base import Mixer, register_part
from .linear import Linear


class GQAttention(Mixer):
    prompt_capturable = True
    fused_decode_ok = True
    supports_append = True

    def __init__(self, prefix, hidden, heads, kv_heads, head_dim, window, position, qk_norm_eps,
                 output_gate, names=None, shares_kv=False):
        names = names or {}
        n = lambda key, default: prefix + names.get(key, default)
        self.hidden, self.heads, self.kv_heads, self.head_dim = hidden, heads, kv_heads, head_dim
        self.window = int(window or 0)
        self.position = position
        self.qk_norm_eps = qk_norm_eps           # None: no head norm
        self.output_gate = bool(output_gate)
        self.q_size, self.kv_size = heads * head_dim, kv_heads * head_dim
        # shares_kv: this layer has no key/value projections of its own; it attends over the keys
        # and values of the layer that owns the state unit the plan gives it
        self.shares_kv = bool(shares_kv)
        mats, rows = [n("q", "attn_q.weight")], [self.q_size]
        if not self.shares_kv:
            mats += [n("k", "attn_k.weight"), n("v", "attn_v.weight")]
            rows += [self.kv_size, self.kv_size]
        if self.output_gate:
            mats.append(n("gate", "attn_gate.weight"))
            rows.append(heads)
        self.qkvg = Linear(mats, rows, hidden)
        self.out = Linear(n("out", "attn_output.weight"), hidden, self.q_size)
        self.q_norm_name, self.k_norm_name = n("q_norm", "attn_q_norm.weight"), n("k_norm", "attn_k_norm.weight")
        self.q_norm_w = self.k_norm_w = None
        # 1/sqrt(head_dim) in float32, as the reference bakes it (src/catena/qwen35_wmma_attention.hex:3-22)
        self.scale = float(torch.tensor(1.0, dtype=torch.float32) / torch.sqrt(torch.tensor(float(head_dim), dtype=torch.float32)))

    def children(self):
        return [self.qkvg, self.out, self.position]

    def tensor_specs(self):
        if self.qk_norm_eps is None:
            return []
        specs = [TensorSpec(self.q_norm_name, (self.head_dim,), "norm")]
        if not self.shares_kv:
            specs.append(TensorSpec(self.k_norm_name, (self.head_dim,), "norm"))
        return specs

    def bind(self, tensors, rt):
        if self.qk_norm_eps is not None:
            self.q_norm_w = tensors[self.q_norm_name].to(torch.float32).contiguous()
            self._bound = [self.q_norm_w]
            if not self.shares_kv:
                self.k_norm_w = tensors[self.k_norm_name].to(torch.float32).contiguous()
                self._bound.append(self.k_norm_w)

    def state_spec(self):
        return KVStateSpec(self.kv_heads, self.head_dim, self.window)

    def forward(self, rt, batch, x, state):
        QS, KVS, QH, KVH, HD = self.q_size, self.kv_size, self.heads, self.kv_heads, self.head_dim
        if self.shares_kv != (not state.owned):
            raise ValueError("a layer that shares keys and values must be given another layer's state unit "
                             "by the plan (owns_state=False), and only such a layer")
        proj = self.qkvg.apply(rt, x)                  # [T, QS + 2 KVS (+ QH)], or [T, QS (+ QH)] when sharing
        interleaved = self.position.pairing == "interleaved"
        if self.shares_kv:
            # q only: head norm and rotation over the q heads, nothing written to the cache
            kernels.qk_prepare(proj, self.q_norm_w, None, self.position.rate_table(), batch.tok_pos, batch.tok_seq,
                               batch.seq_slot, batch.seq_end, None, 0, None, 0, QH, 0, HD, self.qk_norm_eps or 0.0,
                               interleaved=interleaved)
            gate = proj[:, QS:] if self.output_gate else None
        else:
            # an append step keeps the cache as it is until its attention has run
            pool = None if batch.append else state.pool
            kernels.qk_prepare(proj, self.q_norm_w, self.k_norm_w, self.position.rate_table(), batch.tok_pos,
                               batch.tok_seq, batch.seq_slot, batch.seq_end, pool, state.pages, state.ptab,
                               state.ring, QH, KVH, HD, self.qk_norm_eps or 0.0, interleaved=interleaved)
            gate = proj[:, QS + 2 * KVS:] if self.output_gate else None
        q = proj[:, :QS]
        ctx = torch.empty((batch.T, QS), dtype=x.dtype, device=x.device)
        if batch.prefill or batch.append:
            if self.shares_kv and batch.append and state.ring:
                raise NotImplementedError("an append step of a layer that shares the keys and values of a sliding "
                                          "layer: the owner's ring no longer holds what this layer's windows need")
            if self.shares_kv:
                # the owner left this step's keys and values for its readers; bring them beside q so
                # that the attention kernel sees one packed buffer
                k_own, v_own = batch.shared[("kv", state.unit)]
                packed = torch.empty((batch.T, QS + 2 * KVS), dtype=x.dtype, device=x.device)
                packed[:, :QS].copy_(q)
                packed[:, QS:QS + KVS].copy_(k_own)
                packed[:, QS + KVS:].copy_(v_own)
                q, k, v = packed[:, :QS], packed[:, QS:QS + KVS], packed[:, QS + KVS:]
            else:
                k, v = proj[:, QS:QS + KVS], proj[:, QS + KVS:QS + 2 * KVS]
                batch.shared[("kv", state.unit)] = (k, v)
            if batch.append:
                rt.attention_append(ctx, q, k, v, gate, batch, state, QH, KVH, HD, self.window, self.scale)
                if not self.shares_kv:
                    kernels.kv_store(proj[:, QS:QS + 2 * KVS], batch.tok_pos, batch.tok_seq, batch.seq_slot,
                                     batch.seq_end, state.pool, state.pages, state.ptab, state.ring, KVH, HD)
            else:
                rt.attention_prefill(ctx, q, k, v, gate, batch, QH, KVH, HD, self.window, self.scale)
        else:
            # launched for the longest sequence that this step's length class allows, so that a
            # recording of the step serves every step of the class
            entries = state.spec.entries(state.spec.length_class(batch.max_end))
            n_chunks = max(1, -(-entries // ATTN_DECODE_CHUNK))
            part_o, part_ml = rt.scratch_attn_decode(batch.B, QH, HD, n_chunks)
            kernels.attn_decode(ctx, q, gate, batch.seq_pos0, batch.seq_slot, state.pool, state.pages, state.ptab,
                                state.ring, self.window, QH, KVH, HD, n_chunks, self.scale, part_o, part_ml)
        return self.out.apply(rt, ctx, partial_ok=batch.partial_sums_ok)


register_part("mixer", "gqa_attention", GQAttention)
