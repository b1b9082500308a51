"""The step function and the cache it runs on.

`Engine.step(slots, tokens, want)` runs one batch of sequences that started together: their
whole prompts in the first step (unequal lengths, packed without padding), then one token
each.  It runs only the tokens it is given, reads everything older from the cache, and
returns float32 logits at the wanted places.  catena-models has the one-sequence form of
this (`Session::forward`, src/model.rs:692-731, with its errors: empty input, capacity
exceeded, token id outside the vocabulary, src/model.rs:697-710).

A step in which a sequence brings several tokens on top of what it already holds (or in which
started and new sequences meet) is an append step: it runs the same parts through their
general forms, which read what is older than the step from the cache (the reference's
`Session::forward` takes any number of tokens at any position, src/model.rs:692-731).

Decode steps of a given batch size replay a captured CUDA graph: positions, slots and new
page-table entries live in a fixed device buffer that is refreshed by one host-to-device
copy before each replay.  Which recording serves a step is decided by the batch size and by
what the model's state specs say about the sequences' length (`length_class`); the engine
knows nothing of attention chunks.  Short prompt steps whose shape repeats are recorded and
replayed the same way.
"""
from __future__ import annotations

import dataclasses

import numpy as np
import torch

from ..cache.cache import Cache
from ..cache.allocators import CacheError, CacheFull
from .. import kernels as _kernels
from ..csrc.limits import PAGE_TOKENS
from .batch import BatchLayout, StepBatch, clear_sampling, fill_host, fill_host_decode, fill_sampling


PROMPT_GRAPH_MAX_TOKENS = 1024     # longer prompt steps are bound by the device, not by their launches
# Recorded prompt steps kept.  A class is 64 tokens wide, so prompts of up to 1,024 tokens that come alone make 16
# classes (times the numbers of wanted places in use); were fewer kept than a workload cycles through, every
# class would be recorded again and again (about twice a step's cost each time) and never replayed.  The
# recordings share the engine's memory pool and keep little of their own.
PROMPT_GRAPHS_KEPT = 48
PROMPT_PAD = 64                    # recorded prompt steps run a multiple of this many rows, the rest as padding
# Recorded decode steps (batch size, length class) kept; the least recently used goes.  A batch whose
# sequences end one by one walks through every batch size below its first, and a step of a new size costs 6
# to 8 ms (1.7B-class: kernel by kernel, then the capture) where a replay costs 1.1 to 1.8 ms; the recordings
# share one memory pool, in which a recording keeps about 10 MiB of its own, so 96 of them are 1 GiB at most.
DECODE_GRAPHS_KEPT = 96


class StepError(ValueError):
    """A step was refused before anything ran (bad token id, unknown slot, mixed batch...)."""


@dataclasses.dataclass
class Sampling:
    """What the on-device sampler needs for one step: greedy when temperature is 0, else
    temperature sampling with a uniform keyed by (seed, sequence id, step) per sequence."""
    sequence_ids: list
    steps: list
    temperature: float = 0.0
    seed: int = 0


class _Staging:
    """A few pinned host buffers used in turn, each guarded by an event of its last copy."""

    def __init__(self, n=4):
        self.bufs = [None] * n
        self.events = [None] * n
        self.i = 0

    def take(self, size):
        self.i = (self.i + 1) % len(self.bufs)
        if self.events[self.i] is not None:
            self.events[self.i].synchronize()
        buf = self.bufs[self.i]
        if buf is None or buf.numel() < size:
            buf = torch.empty(max(1024, size * 2), dtype=torch.int32, pin_memory=True)
            self.bufs[self.i] = buf
        return buf, self.i

    def mark(self, i):
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev


class PendingTokens:
    """The tokens a step chose on the device, on their way to the host (`Engine.step(...,
    wait=False)`).  `tokens()` waits for the copy and returns them as Python ints."""

    def __init__(self, host, n, event, check):
        self._host, self._n, self._event, self._check = host, n, event, check

    def tokens(self):
        self._event.synchronize()
        self._check(self._host[self._n:self._n + 2].tolist())   # the device's two fault flags travel behind the tokens
        return self._host[:self._n].tolist()


class _RecordedStep:
    """A captured step: its metadata layout and device buffer, the graph, and where its outputs land."""

    def __init__(self, layout, device_buf, graph, logits, batch):
        self.layout, self.device_buf, self.graph, self.logits, self.batch = layout, device_buf, graph, logits, batch
        self.launches = 0


class Engine:
    fused_sampling = True          # step(..., sampling=...) chooses the next tokens on the device

    def __init__(self, model, max_tokens, max_seqs=None, use_graphs=True):
        self.model, self.rt = model, model.rt
        max_len = model.definition.max_positions or None
        self.cache = Cache(model.state_specs, max_tokens, self.rt.dtype, self.rt.device, max_seqs, max_len)
        self.n_kv_groups = len(self.cache.kv_specs)
        self.use_graphs = use_graphs and model.capturable
        self._staging = _Staging()
        self._graphs = {}
        self._prompt_graphs = {}                               # shape of a prompt step -> its recorded graph
        # One memory pool for every recording of this engine: a recording's scratch (what it allocates and
        # frees while it is captured) is handed on to the next capture instead of being taken from the
        # device anew, which is most of what a capture costs; what a recording still holds (its logits)
        # stays its own.  Recordings of one engine replay one after another on one stream.
        self._graph_pool = torch.cuda.graph_pool_handle() if self.use_graphs else None
        self._prompt_seen = {}
        self._sampled_host = None
        # the tokens the last sampling step chose, by position in that step's batch: the next step may
        # take its input tokens from here without the host having seen them (`token_from`)
        self._sampled = torch.zeros(self.cache.book.max_seqs, dtype=torch.int32, device=self.rt.device)
        self._sampled_count = 0                                # sequences of the last recorded decode step that sampled
        self._readback = [None, None]                          # two pinned buffers used in turn
        self._readback_i = 0
        # the distinct state specs of the model: what they say about a length picks the recording
        self._class_specs = []
        for spec in self.cache.state_specs:
            if spec is not None and spec not in self._class_specs:
                self._class_specs.append(spec)
        self.steps_run = 0
        self.kernel_launches = 0

    # ------------------------------------------------------------------ slots
    def admit(self, count=1):
        """Slots for `count` new sequences (all or none)."""
        if count > self.cache.book.slots.free_count:
            raise CacheFull(f"{count} slot(s) wanted, {self.cache.book.slots.free_count} free")
        return self.cache.admit_many(count)

    def release(self, slots):
        for s in slots:
            self.cache.release(s)

    def length(self, slot):
        return self.cache.book.length[slot]

    def check_errors(self):
        """Reads the device's fault flags (synchronises) and raises `DeviceFault` if a kernel gave up
        on a bounded wait or a token id outside the vocabulary reached the embedding.  Steps that
        sample read the flags with their tokens; a caller that takes logits calls this before it
        trusts them."""
        self.rt.check_errors()

    # ------------------------------------------------------------------ the step
    def _check(self, slots, tokens, want):
        book = self.cache.book
        if not slots:
            raise StepError("a step needs at least one sequence")
        if len(set(slots)) != len(slots):
            raise StepError("a slot appears twice in one step")
        if len(tokens) != len(slots):
            raise StepError("one token list per slot")
        for s in slots:
            if s not in book.length:
                raise StepError(f"slot {s} is not live")
        positions = [book.length[s] for s in slots]
        if any(len(t) == 0 for t in tokens):
            raise StepError("a sequence brought no tokens")
        if all(p == 0 for p in positions):
            kind = "prefill"
        elif all(len(t) == 1 for t in tokens):
            kind = "decode"
        else:
            kind = "append"
            if not self.model.supports_append:
                raise StepError("this model has a part without an append form: its sequences either all "
                                "start at their first token or all go on by one token")
        V = self.model.vocab_size
        for t in tokens:
            arr = np.asarray(t)
            if arr.min() < 0 or arr.max() >= V:
                raise StepError(f"token id outside the vocabulary of {V}")
        if want is None:
            want = [[len(t) - 1] for t in tokens]
        if len(want) != len(slots):
            raise StepError("one list of wanted places per slot")
        for w, t in zip(want, tokens):
            if any(i < 0 or i >= len(t) for i in w):
                raise StepError("a wanted place lies outside the sequence's tokens of this step")
        return positions, kind, want

    def _reserve(self, slots, positions, tokens):
        """Pages for the new tokens of every sequence; undone as a whole if one does not fit."""
        book = self.cache.book
        updates, done = [], []
        try:
            for s, p, t in zip(slots, positions, tokens):
                ups = book.reserve(s, p + len(t))
                done.append((s, ups))
                updates.extend(self.cache.flat_updates(s, ups))
        except CacheError:
            for s, ups in done:                                  # give the pages of this step back
                for g, j, page in reversed(ups):
                    book.pages[s][g].pop()
                    book.page_alloc[g].give_back([page])
            raise
        return updates

    @property
    def overlapped_decode(self):
        """True when decode steps can take their tokens from the step before on the device and hand
        their own back without waiting (`token_from`, `wait=False`)."""
        return self.fused_sampling and self.use_graphs

    def step(self, slots, tokens, want=None, sampling=None, token_from=None, wait=True):
        """Run one step.  `tokens[i]` are the next tokens of the sequence in `slots[i]`;
        `want[i]` the places among them whose logits are returned (default: the last).
        Returns float32 logits [sum(len(want[i])), vocab] on the device, in the order of
        `slots` and of `want`.  The tensor is valid until the next step of the same size.

        With `sampling` (a `Sampling` record; `want` must be left at its default) the next token
        of every sequence is chosen on the device in the same submission and the call returns
        `(logits, tokens)` with `tokens` a list of Python ints: one host-to-device copy of the
        step's inputs, one device-to-host copy of its result.

        A decode step with `sampling` may run ahead of the host (`overlapped_decode`):
        `token_from[i] = j` takes sequence i's input token from what the sampling step before this
        one chose for the j-th sequence of its batch (`tokens[i]` is then ignored; None keeps
        `tokens[i]`), and `wait=False` returns `(logits, PendingTokens)` at once, the copy of the
        chosen tokens to the host being under way."""
        book = self.cache.book
        if sampling is not None and want is not None:
            raise StepError("sampling takes the last place of every sequence; leave `want` out")
        decode = self.use_graphs and want is None and self._is_plain_decode(slots, tokens)
        if (token_from is not None or not wait) and not (decode and sampling is not None):
            raise StepError("token_from and wait=False belong to captured decode steps with sampling")
        if decode:
            positions = [book.length[s] for s in slots]
            flat = [t[0] for t in tokens]
            V = self.model.vocab_size
            if token_from is not None:
                if len(token_from) != len(slots):
                    raise StepError("one token_from entry per slot")
                known = [t for t, j in zip(flat, token_from) if j is None]
                if any(j is not None and not 0 <= j < self._sampled_count for j in token_from):
                    raise StepError("token_from points outside what the step before sampled (a recorded decode "
                                    "step with sampling must come right before)")
                flat = [t if j is None else -(1 + j) for t, j in zip(flat, token_from)]
            else:
                known = flat
            if known and (min(known) < 0 or max(known) >= V):
                raise StepError(f"token id outside the vocabulary of {V}")
            if max(positions) >= book.max_len:
                raise CacheFull(f"sequence of {max(positions) + 1} tokens exceeds the longest allowed ({book.max_len})")
            # a decode step needs a new page only when a sequence stands on a page border
            updates = self._reserve(slots, positions, tokens) if any(p % PAGE_TOKENS == 0 for p in positions) else []
            logits, sampled = self._decode_graph_step(slots, flat, positions, updates, sampling)
            for s, p in zip(slots, positions):
                book.length[s] = p + 1
        else:
            positions, kind, want = self._check(slots, tokens, want)
            updates = self._reserve(slots, positions, tokens)
            B, T = len(slots), sum(len(t) for t in tokens)
            if kind == "decode" and self.use_graphs:
                # decode with explicit wanted places: the graph computes every row, pick the wanted
                logits, sampled = self._decode_graph_step(slots, [t[0] for t in tokens], positions, updates, sampling)
                if any(w != [0] for w in want):
                    logits = logits[[b for b, w in enumerate(want) for _ in w]]
            else:
                self._sampled_count = 0                        # what this step samples does not land in `_sampled`
                logits, sampled = self._prompt_step(slots, tokens, positions, kind, want, updates, sampling)
            for s, p, t in zip(slots, positions, tokens):
                book.advance(s, p + len(t))
        self.steps_run += 1
        if sampling is None:
            return logits
        if not wait:
            return logits, self._to_host_later(sampled)
        return logits, self._to_host(sampled)

    def _is_plain_decode(self, slots, tokens):
        """Every slot live and started, one token each, no slot twice: the lean path may take it."""
        length = self.cache.book.length
        if not slots or len(tokens) != len(slots) or len(set(slots)) != len(slots):
            return False
        for s, t in zip(slots, tokens):
            if length.get(s, 0) == 0 or len(t) != 1:
                return False
        return True

    def _to_host_later(self, sampled):
        """Starts the copy of the chosen tokens to pinned memory and returns a handle to await it."""
        n = sampled.shape[0]
        self._readback_i ^= 1
        host = self._readback[self._readback_i]
        if host is None or host.numel() < n + 2:
            host = torch.empty(max(64, 2 * n + 2), dtype=torch.int32, pin_memory=True)
            self._readback[self._readback_i] = host
        host[:n].copy_(sampled, non_blocking=True)
        host[n:n + 2].copy_(self.rt.status, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return PendingTokens(host, n, event, self.rt.raise_for_status)

    def _to_host(self, sampled):
        """Sampled tokens as Python ints (pinned buffer, one copy, one synchronisation)."""
        n = sampled.shape[0]
        if self._sampled_host is None or self._sampled_host.numel() < n + 2:
            self._sampled_host = torch.empty(max(64, 2 * n + 2), dtype=torch.int32, pin_memory=True)
        self._sampled_host[:n].copy_(sampled, non_blocking=True)
        self._sampled_host[n:n + 2].copy_(self.rt.status, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.rt.raise_for_status(self._sampled_host[n:n + 2].tolist())
        return self._sampled_host[:n].tolist()

    # ------------------------------------------------------------------ prompt steps
    def _prompt_step(self, slots, tokens, positions, kind, want, updates, sampling):
        """A step with explicit tokens per sequence, launched kernel by kernel.  A short prompt step
        whose class of shapes comes a second time is recorded into a graph as it runs and replayed
        from then on: about 200 launches from Python cost more than a short prompt's kernels take.
        A class is (number of sequences, tokens rounded up to PROMPT_PAD, longest prompt rounded up
        likewise, number of wanted places; for tokens on top of held ones also the class of lengths
        that the longest sequence reaches): the step runs that many rows, the surplus as padding that
        belongs to no sequence, and everything about the real lengths travels in the step's metadata,
        so one recording serves every prompt of its class.  The few most recent classes are kept."""
        B, T = len(slots), sum(len(t) for t in tokens)
        n_want = sum(len(w) for w in want)
        key = entry = max_len = max_end = None
        T_run, U_cap = T, len(updates)
        if (kind in ("prefill", "append") and self.use_graphs and self.model.prompt_capturable
                and T <= PROMPT_GRAPH_MAX_TOKENS):
            T_run = -(-T // PROMPT_PAD) * PROMPT_PAD
            max_len = -(-max(len(t) for t in tokens) // PROMPT_PAD) * PROMPT_PAD
            U_cap = (T_run // PAGE_TOKENS + B) * max(1, self.n_kv_groups)    # no step of the class needs more pages
            key = (B, T_run, max_len, n_want, sampling is not None)
            if kind == "append":
                # tokens on top of what the sequences hold: the class also names how far the longest one
                # reaches, in the state specs' own classes of lengths, and the step is launched for their bound
                classes = self._length_classes(max(p + len(t) for p, t in zip(positions, tokens)))
                key += ("append", classes)
                max_end = max(classes) or None
            entry = self._prompt_graphs.get(key)
        layout = entry.layout if entry else BatchLayout(T_run, B, n_want, U_cap)
        host, idx = self._staging.take(layout.size)
        fill_host(layout, host.numpy(), slots, tokens, positions, want, updates)
        if sampling is not None:
            fill_sampling(layout, host.numpy(), sampling)
        if entry:
            entry.device_buf.copy_(host[:layout.size], non_blocking=True)
            self._staging.mark(idx)
            self._prompt_graphs[key] = self._prompt_graphs.pop(key)        # most recently used last
            entry.graph.replay()
            _kernels.launches += entry.launches
            # the graph writes its logits to the same place every time: the caller gets its own copy
            return entry.logits.clone(), entry.sampled
        record = False
        if key is not None:
            seen = self._prompt_seen.get(key, 0) + 1
            if len(self._prompt_seen) > 4096:
                self._prompt_seen.clear()
            self._prompt_seen[key] = seen
            record = seen >= 2
        if record:
            dev = torch.zeros(layout.size, dtype=torch.int32, device=self.rt.device)
            dev.copy_(host[:layout.size], non_blocking=True)
        else:
            dev = host[:layout.size].to(self.rt.device, non_blocking=True)
        self._staging.mark(idx)
        batch = StepBatch(layout, dev, kind, [len(t) for t in tokens], positions, n_want, len(updates), max_len=max_len,
                          max_end=max_end)
        # a decode step that wants its every row: the same launches as its recorded form
        batch.wants_every_row = kind == "decode" and all(w == [0] for w in want)
        sampled = torch.empty(B, dtype=torch.int32, device=self.rt.device) if sampling is not None else None

        def run():
            out = self.model.forward(batch, self.cache)
            if sampled is not None:
                _kernels.sample(sampled, out, batch.samp_temp[:B], batch.samp_seq[:B], batch.samp_step[:B],
                                batch.samp_seed)
            return out

        logits = run()
        if record:
            # as for decode: this run was the step's result; the capture executes nothing
            entry = _RecordedStep(layout, dev, torch.cuda.CUDAGraph(), None, batch)
            entry.sampled = sampled
            before = _kernels.launches
            with torch.cuda.graph(entry.graph, pool=self._graph_pool):
                entry.logits = run()
            entry.launches = _kernels.launches - before
            _kernels.launches = before
            while len(self._prompt_graphs) >= PROMPT_GRAPHS_KEPT:
                torch.cuda.current_stream().synchronize()      # its last replay may still be running
                self._prompt_graphs.pop(next(iter(self._prompt_graphs)))
            self._prompt_graphs[key] = entry
        return logits, sampled

    # ------------------------------------------------------------------ captured decode
    def _length_classes(self, longest):
        """What the model's state specs say about a step whose longest sequence holds `longest`
        tokens: steps with equal answers launch the same kernels with the same arguments."""
        return tuple(spec.length_class(longest) for spec in self._class_specs)

    def _decode_graph_step(self, slots, flat_tokens, positions, updates, sampling):
        B = len(slots)
        key = (B, self._length_classes(max(positions) + 1))
        entry = self._graphs.get(key)
        if entry is not None:
            self._graphs[key] = self._graphs.pop(key)          # most recently used last
        else:
            while len(self._graphs) >= DECODE_GRAPHS_KEPT:
                torch.cuda.current_stream().synchronize()      # its last replay may still be running
                self._graphs.pop(next(iter(self._graphs)))
            layout = BatchLayout(B, B, B, B * max(1, self.n_kv_groups))
            device_buf = torch.zeros(layout.size, dtype=torch.int32, device=self.rt.device)
            entry = _RecordedStep(layout, device_buf, None, None, None)
            entry.sampled = self._sampled[:B]                  # every graph leaves its tokens in the same place
            self._graphs[key] = entry
        layout = entry.layout
        host, idx = self._staging.take(layout.size)
        view = host.numpy()
        fill_host_decode(layout, view, slots, flat_tokens, positions, updates)
        if sampling is not None:
            fill_sampling(layout, view, sampling)
        else:
            clear_sampling(layout, view)
        self._sampled_count = B if sampling is not None else 0
        entry.device_buf.copy_(host[:layout.size], non_blocking=True)
        self._staging.mark(idx)
        if entry.graph is None:
            # First step of this size: run it eagerly (this is the step's result; it also loads
            # every kernel, which must not happen inside a capture), then record the same
            # launches into a graph for the steps that follow.  A capture executes nothing, so
            # the cache and the fixed-size states advance exactly once.  The graph always ends
            # with the sampling kernel; without a sampling request its inputs are zeroed (an argmax)
            # and its output is ignored.
            batch = StepBatch(layout, entry.device_buf, "decode", [1] * B, positions, B, len(updates))
            batch.wants_every_row = True                       # fill_host_decode wants every row, in order
            batch.prev_sampled = self._sampled                 # negative token entries point into it

            def run():
                out = self.model.forward(batch, self.cache)
                _kernels.sample(entry.sampled, out, batch.samp_temp[:B], batch.samp_seq[:B], batch.samp_step[:B],
                                batch.samp_seed)
                return out

            logits = run()
            graph = torch.cuda.CUDAGraph()
            before = _kernels.launches
            with torch.cuda.graph(graph, pool=self._graph_pool):
                entry.logits = run()
            entry.launches = _kernels.launches - before       # kernels one replay runs
            _kernels.launches = before                         # the capture itself ran nothing
            entry.graph, entry.batch = graph, batch
        else:
            entry.graph.replay()
            _kernels.launches += entry.launches
            logits = entry.logits
        return logits, entry.sampled
