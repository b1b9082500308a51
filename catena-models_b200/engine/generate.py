"""The generation loop above the step function.

Requests are cut into batches that start together; a batch's prompts (of unequal lengths)
run in one step, then every live sequence gets one token per step; a sequence ends at a stop
token or at its budget and gives its slot back at once, the others go on; the next batch
starts when the last sequence of this one has ended, on the slots and pages just freed.
catena-models has the one-sequence loop (src/main.rs:311-347: the first new token comes from
the prompt step, stop at eos unless --ignore-eos, at most -n tokens) and the server's
finish reasons "stop" / "length" (src/server/engine.rs:516-522).

The loop's decisions are plain Python over an engine-like object (`admit`, `release`, `step`)
and a sampler-like object (`sample`), so they can be tested without a device.
"""
from __future__ import annotations

import dataclasses

from ..cache.allocators import CacheFull
from ..csrc.limits import PAGE_TOKENS as PAGE


@dataclasses.dataclass
class Generation:
    prompt: list
    tokens: list = dataclasses.field(default_factory=list)
    finish_reason: str = None         # "stop" | "length"


def plan_batches(prompt_lens, max_new_tokens, max_batch, max_tokens, page=PAGE):
    """Cut requests, in order, into batches of at most `max_batch` sequences whose worst-case
    footprint (prompt + budget, each rounded up to whole pages) fits `max_tokens`."""
    batches, cur, used = [], [], 0
    for i, n in enumerate(prompt_lens):
        need = (n + max_new_tokens + page - 1) // page * page
        if need > max_tokens:
            raise ValueError(f"request {i} needs {need} cache tokens, the cache holds {max_tokens}")
        if cur and (len(cur) >= max_batch or used + need > max_tokens):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


def finish_reason(token, n_generated, max_new_tokens, stop_token_ids, ignore_eos):
    """Why a sequence ends after `token`, its `n_generated`-th new token; None if it goes on.
    A stop token is kept in the output, as the reference keeps it (src/main.rs:332-346)."""
    if not ignore_eos and token in stop_token_ids:
        return "stop"
    if n_generated >= max_new_tokens:
        return "length"
    return None


def run_batch(engine, sampler, requests, ids, max_new_tokens, stop_token_ids, ignore_eos, on_step=None):
    """One batch from admission to its last sequence's end.  `requests`: Generation objects,
    `ids`: their sequence ids (the sampler's key)."""
    if max_new_tokens <= 0:
        for r in requests:
            r.finish_reason = "length"
        return
    slots = engine.admit(len(requests))
    live = list(range(len(requests)))
    # An engine that samples on the device in the same submission as the step (`fused_sampling`)
    # is asked to; any other pair of engine and sampler goes the two-call way.
    fused = getattr(engine, "fused_sampling", False) and hasattr(sampler, "request")

    def run_step(step_slots, step_tokens, step):
        if fused:
            return engine.step(step_slots, step_tokens, sampling=sampler.request([ids[i] for i in live], step))[1]
        logits = engine.step(step_slots, step_tokens)
        return sampler.sample(logits, [ids[i] for i in live], [step] * len(live))

    def settle(members, tokens, step, dropped=()):
        """Book the tokens of one step; returns the members that go on.  `dropped` members had ended
        before this step was known to be unnecessary for them: their token is thrown away."""
        still = []
        for i, tok in zip(members, tokens):
            if i in dropped:
                continue
            r = requests[i]
            r.tokens.append(int(tok))
            r.finish_reason = finish_reason(int(tok), len(r.tokens), max_new_tokens, stop_token_ids, ignore_eos)
            if r.finish_reason is None:
                still.append(i)
            else:
                engine.release([slots[i]])
                slots[i] = None
        if on_step:
            on_step(step, len(members) - len(dropped))
        return still

    try:
        step = 0
        tokens = run_step(slots, [r.prompt for r in requests], step)
        if fused and getattr(engine, "overlapped_decode", False):
            _decode_ahead(engine, sampler, requests, ids, slots, settle(live, tokens, step), max_new_tokens, settle)
            return
        while True:
            live = settle(live, tokens, step)
            if not live:
                break
            step += 1
            tokens = run_step([slots[i] for i in live], [[requests[i].tokens[-1]] for i in live], step)
    finally:
        engine.release([s for s in slots if s is not None])


def _decode_ahead(engine, sampler, requests, ids, slots, live, max_new_tokens, settle):
    """Decode with the device one step ahead of the host.  Step k+1 is submitted before the tokens
    of step k have reached the host: it takes them from the device (`token_from`), for every member
    of step k that cannot end by its budget.  A member that step k's token then ends (a stop token)
    has one token too many computed; it is dropped when step k+1 is booked.  The host's work per
    step (bookkeeping, the next submission) so runs while the device computes."""
    if not live:
        return
    step = 1
    members = list(live)
    pending = engine.step([slots[i] for i in members], [[requests[i].tokens[-1]] for i in members],
                          sampling=sampler.request([ids[i] for i in members], step), wait=False)[1]
    dropped = set()
    while True:
        # who can still be running after this step's token: everyone short of the budget by more than one
        ahead = [i for i in members if i not in dropped and len(requests[i].tokens) + 1 < max_new_tokens]
        nxt = None
        if ahead:
            where = {i: k for k, i in enumerate(members)}
            try:
                nxt = engine.step([slots[i] for i in ahead], [[0]] * len(ahead),
                                  sampling=sampler.request([ids[i] for i in ahead], step + 1),
                                  token_from=[where[i] for i in ahead], wait=False)[1]
            except CacheFull:
                nxt = None                                     # no room to run ahead: wait for this step first
        still = settle(members, pending.tokens(), step, dropped)
        step += 1
        if nxt is None:
            if not still:
                return
            members, dropped = still, set()
            pending = engine.step([slots[i] for i in members], [[requests[i].tokens[-1]] for i in members],
                                  sampling=sampler.request([ids[i] for i in members], step), wait=False)[1]
            continue
        # the step that ran ahead holds `ahead`; those of them that have just ended are dropped from it
        members, dropped, pending = ahead, {i for i in ahead if i not in still}, nxt


def generate(engine, sampler, prompts, max_new_tokens, stop_token_ids=(), ignore_eos=False, max_batch=64,
             max_tokens=None, on_step=None):
    """Generate for every prompt (lists of token ids); returns a Generation per prompt."""
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError(f"prompt {i} is empty")
    requests = [Generation(list(p)) for p in prompts]
    max_tokens = max_tokens or engine.cache.book.page_budget * PAGE
    max_batch = min(max_batch, engine.cache.book.max_seqs) if hasattr(engine, "cache") else max_batch
    stop = frozenset(stop_token_ids)
    for batch in plan_batches([len(p) for p in prompts], max_new_tokens, max_batch, max_tokens):
        run_batch(engine, sampler, [requests[i] for i in batch], batch, max_new_tokens, stop, ignore_eos, on_step)
    return requests
