"""Seeded random schedules against the plain model: requests start (alone or in batches), go on by
one token, bring several tokens on top of what they hold (alone, together, beside requests that
start in the same step), end and give their slots and pages back, in any order that the engine
allows.  What a position's logits are must not depend on the schedule that led there.  Every
request's wanted rows, over all the steps that produced them, are compared with the plain model
run over the whole request, in 32-bit and in bfloat16."""
import random

import pytest
import torch

import tiny
from test_engine_gpu import check, engine_for, folders, plain, plain_logits  # noqa: F401  (fixtures)

pytestmark = pytest.mark.gpu

MAX_LEN = 260            # past every tiny configuration's window and ring, and across page borders
MAX_LIVE = 5


def _schedule(rng, vocab, steps):
    """Yields (step, ended): step = [(request, tokens, want)], ended = the requests that are given back
    after it.  A step is a start (new requests only; live ones sit it out), a decode step (every live
    request, one token) or mixed (some live requests with 1 to 70 tokens, maybe a new one beside them)."""
    live, made = [], 0

    def new_request(first):
        nonlocal made
        made += 1
        total = rng.randint(max(first, 2), MAX_LEN)
        return dict(id=made, tokens=tiny.random_prompt(total, vocab, seed=1000 * steps + made), at=0, rows=[], places=[])

    for _ in range(steps):
        room = MAX_LIVE - len(live)
        kinds = ["decode"] * 3 + ["mixed"] * 3 if live else []
        if room > 0:
            kinds += ["start"] * (3 if not live else 1)
        kind = rng.choice(kinds)
        entries = []
        if kind == "start":
            for _ in range(rng.randint(1, room)):
                first = rng.choice([1, 2, 7, 33, 64, 65, 100, 130])
                r = new_request(first)
                n = min(first, len(r["tokens"]) - 1)
                entries.append((r, n))
                live.append(r)
        elif kind == "decode":
            entries = [(r, 1) for r in live]
        else:
            for r in live:
                if rng.random() < 0.8:
                    entries.append((r, rng.choice([1, 2, 5, 31, 64, 70])))
            if room > 0 and rng.random() < 0.5:
                r = new_request(1)
                entries.append((r, min(rng.choice([1, 9, 66]), len(r["tokens"]) - 1)))
                live.append(r)
            if not entries:
                entries = [(live[0], 3)]
        step = []
        for r, n in entries:
            n = max(1, min(n, len(r["tokens"]) - r["at"]))
            want = sorted(set(rng.sample(range(n), min(n, rng.randint(0, 3))) + ([n - 1] if rng.random() < 0.7 else [])))
            step.append((r, r["tokens"][r["at"]:r["at"] + n], want))
        ended = []
        for r, toks, _ in step:
            if r["at"] + len(toks) >= len(r["tokens"]) or rng.random() < 0.05:
                ended.append(r)
        yield step, ended
        for r, toks, _ in step:
            r["at"] += len(toks)
        for r in ended:
            live.remove(r)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,seed", [("A", 1), ("A", 2), ("B", 3), ("B", 4), ("L", 5), ("C", 6)])
def test_random_schedules(folders, plain, name, dtype, seed):
    eng = engine_for(folders, name, dtype)
    vocab = plain[name][0]["vocab_size"]
    rng = random.Random(seed)
    slot_of, done = {}, {}
    kinds = set()
    for step, ended in _schedule(rng, vocab, steps=60):
        new = [r for r, _, _ in step if r["id"] not in slot_of]
        for r, s in zip(new, eng.admit(len(new))):
            slot_of[r["id"]] = s
            done[r["id"]] = r                 # every request is checked in the end, ended or not
        at = [r["at"] for r, _, _ in step]
        kinds.add("start" if all(a == 0 for a in at) else "decode" if all(len(t) == 1 for _, t, _ in step) else "mixed")
        out = eng.step([slot_of[r["id"]] for r, _, _ in step], [t for _, t, _ in step], [w for _, _, w in step])
        off = 0
        for r, toks, want in step:
            if want:
                r["rows"].append(out[off:off + len(want)].clone())
                r["places"] += [r["at"] + w for w in want]
                off += len(want)
        assert off == (0 if out is None else out.shape[0])
        for r in ended:
            eng.release([slot_of.pop(r["id"])])
    eng.release(list(slot_of.values()))
    assert not eng.cache.book.live
    assert kinds == {"start", "decode", "mixed"}
    got, exact, same = [], [], []
    for r in done.values():
        if not r["places"]:
            continue
        upto = max(r["places"]) + 1
        e, s = plain_logits(plain, name, r["tokens"][:upto], dtype)
        got.append(torch.cat(r["rows"]))
        exact.append(e[r["places"]])
        if s is not None:
            same.append(s[r["places"]])
    assert len(got) >= 5
    check(torch.cat(got), torch.cat(exact), dtype, torch.cat(same) if same else None)
