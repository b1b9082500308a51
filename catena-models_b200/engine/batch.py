"""One step's batch as the kernels see it: packed tokens and their sequence geometry.

A step is a prompt step (`kind` "prefill": every sequence starts at position 0 and brings its
whole prompt), a decode step ("decode": every sequence brings one token) or an append step
("append": anything else, for instance several tokens on top of started sequences).  All integer
metadata travels in one int32 buffer, filled on the host in pinned memory and copied once:

    tokens[T] tok_seq[T] tok_pos[T] seq_slot[B] seq_start[B+1] seq_pos0[B] seq_end[B]
    want_rows[W] upd_count[1] upd_index[U] upd_value[U]
    samp_seq[B] samp_step[B] samp_temp[B] (float bits) samp_seed[2]

`want_rows` are rows of the packed batch whose logits are asked for; `upd_*` are page-table
entries that the cache allocated for this step (applied on the device before any layer runs).
A step may carry rows of padding behind its tokens (tok_seq = -1): they belong to no sequence,
touch no cache and change no result; recorded prompt steps use them to serve a class of shapes.
"""
from __future__ import annotations

import numpy as np
import torch


class BatchLayout:
    """Offsets of the fields in the int32 buffer for given capacities."""

    def __init__(self, T, B, W, U):
        self.T, self.B, self.W, self.U = T, B, W, U
        fields = [("tokens", T), ("tok_seq", T), ("tok_pos", T), ("seq_slot", B), ("seq_start", B + 1),
                  ("seq_pos0", B), ("seq_end", B), ("want_rows", W), ("upd_count", 1), ("upd_index", U),
                  ("upd_value", U), ("samp_seq", B), ("samp_step", B), ("samp_temp", B), ("samp_seed", 2)]
        self.offsets, off = {}, 0
        for name, n in fields:
            self.offsets[name] = (off, n)
            off += (n + 3) // 4 * 4                     # 16-byte aligned fields
        self.size = max(4, off)

    def views(self, buf):
        return {name: buf[off:off + n] for name, (off, n) in self.offsets.items()}


class StepBatch:
    """Device-side views plus the host-side facts a part may need to size a launch."""

    KINDS = ("prefill", "decode", "append")

    def __init__(self, layout, device_buf, kind, lengths, positions, n_want, n_updates, max_len=None, max_end=None):
        if kind not in self.KINDS:
            raise ValueError(f"step kind {kind!r}; one of {self.KINDS}")
        self.layout = layout
        self.buf = device_buf
        v = layout.views(device_buf)
        self.tokens, self.tok_seq, self.tok_pos = v["tokens"], v["tok_seq"], v["tok_pos"]
        self.seq_slot, self.seq_start = v["seq_slot"], v["seq_start"]
        self.seq_pos0, self.seq_end = v["seq_pos0"], v["seq_end"]
        self.want_rows = v["want_rows"][:n_want]
        self.upd_count, self.upd_index, self.upd_value = v["upd_count"], v["upd_index"], v["upd_value"]
        self.samp_seq, self.samp_step, self.samp_seed = v["samp_seq"], v["samp_step"], v["samp_seed"]
        self.samp_temp = v["samp_temp"].view(torch.float32)
        self.kind = kind
        self.prefill = kind == "prefill"                       # every sequence starts at position 0
        self.append = kind == "append"                         # sequences stand anywhere and bring any number of tokens
        self.lengths, self.positions = list(lengths), list(positions)    # host copies, per sequence
        self.B, self.T = layout.B, layout.T
        # longest run of new tokens; a step recorded for a class of shapes is launched for the class's bound
        self.max_len = max_len if max_len is not None else (max(lengths) if lengths else 0)
        # how far the longest sequence reaches with this step; recorded steps: the bound of its class of lengths
        self.max_end = max_end if max_end is not None else max((p + n for p, n in zip(positions, lengths)), default=0)
        self.n_want, self.n_updates = n_want, n_updates
        self.wants_every_row = False                           # want_rows is 0, 1, ..., T-1 (set by the decode path)
        self.prev_sampled = None                               # device int32: tokens the step before chose (decode path)
        self.shared = {}                                       # what a layer leaves for later layers of this step
        self.partial_sums_ok = False                           # set by a block around its mixer / feed-forward: their
                                                               # output may be kernels.PartialSums

def fill_sampling(layout, host, sampling):
    """The sampler's inputs of a step: sequence ids, step numbers, temperature, seed."""
    v = layout.views(host)
    n = len(sampling.sequence_ids)
    v["samp_seq"][:n] = sampling.sequence_ids
    v["samp_step"][:n] = sampling.steps
    v["samp_temp"][:n] = np.float32(sampling.temperature).view(np.int32)
    v["samp_seed"][0] = np.uint32(sampling.seed & 0xFFFFFFFF).view(np.int32)
    v["samp_seed"][1] = np.uint32((sampling.seed >> 32) & 0xFFFFFFFF).view(np.int32)


def clear_sampling(layout, host):
    """A step that samples nothing still runs the sampling kernel when it is replayed from a
    recording: give it temperature 0 and zeroed keys, whatever an earlier step left in the buffer."""
    v = layout.views(host)
    for name in ("samp_seq", "samp_step", "samp_temp", "samp_seed"):
        v[name][:] = 0


def fill_host_decode(layout, host, slots, tokens, positions, updates):
    """A decode step (one token per sequence, every row wanted) written with whole-array stores."""
    v = layout.views(host)
    B = len(slots)
    ar = np.arange(B + 1, dtype=np.int32)
    pos = np.asarray(positions, dtype=np.int32)
    v["tokens"][:B] = tokens
    v["tok_seq"][:B] = ar[:B]
    v["tok_pos"][:B] = pos
    v["seq_slot"][:B] = slots
    v["seq_start"][:B + 1] = ar
    v["seq_pos0"][:B] = pos
    v["seq_end"][:B] = pos + 1
    v["want_rows"][:B] = ar[:B]
    v["upd_count"][0] = len(updates)
    for i, (idx, page) in enumerate(updates):
        v["upd_index"][i] = idx
        v["upd_value"][i] = page


def fill_host(layout, host, slots, token_lists, positions, want, updates):
    """Write one step into the pinned int32 array `host` (numpy view).  Returns n_want."""
    v = layout.views(host)
    t = 0
    rows = []
    for b, (slot, toks, pos) in enumerate(zip(slots, token_lists, positions)):
        n = len(toks)
        v["tokens"][t:t + n] = toks
        v["tok_seq"][t:t + n] = b
        v["tok_pos"][t:t + n] = np.arange(pos, pos + n, dtype=np.int32)
        v["seq_slot"][b] = slot
        v["seq_start"][b] = t
        v["seq_pos0"][b] = pos
        v["seq_end"][b] = pos + n
        for w in want[b]:
            rows.append(t + w)
        t += n
    v["seq_start"][len(slots)] = t
    if t < layout.T:
        # rows of padding (a step recorded for a class of shapes runs layout.T rows): token 0 of no sequence
        v["tokens"][t:layout.T] = 0
        v["tok_seq"][t:layout.T] = -1
        v["tok_pos"][t:layout.T] = 0
    v["want_rows"][:len(rows)] = rows
    v["upd_count"][0] = len(updates)
    for i, (idx, page) in enumerate(updates):
        v["upd_index"][i] = idx
        v["upd_value"][i] = page
    return len(rows)
