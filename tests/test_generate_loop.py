"""The generation loop's decisions, with a fake engine and sampler (no device)."""
import pytest
import torch

from catena_models_b200.engine import generate as gen


class FakeEngine:
    """Logits put all mass on (last token + 1) % vocab; tracks slots like the real engine."""

    def __init__(self, vocab=50, slots=4):
        self.vocab, self.free, self.live = vocab, list(range(slots)), {}
        self.steps, self.max_live = [], 0

    def admit(self, n):
        assert n <= len(self.free)
        out = [self.free.pop(0) for _ in range(n)]
        for s in out:
            assert s not in self.live
            self.live[s] = 0
        self.max_live = max(self.max_live, len(self.live))
        return out

    def release(self, slots):
        for s in slots:
            del self.live[s]                      # KeyError if released twice
            self.free.append(s)
            self.free.sort()

    def step(self, slots, tokens, want=None):
        prefill = all(self.live[s] == 0 for s in slots)
        assert prefill or all(len(t) == 1 for t in tokens)
        self.steps.append(("prefill" if prefill else "decode", list(slots), [len(t) for t in tokens]))
        logits = torch.zeros(len(slots), self.vocab)
        for i, (s, t) in enumerate(zip(slots, tokens)):
            self.live[s] += len(t)
            logits[i, (t[-1] + 1) % self.vocab] = 1.0
        return logits


class Greedy:
    def sample(self, logits, ids, steps):
        self.last = (list(ids), list(steps))
        return logits.argmax(dim=-1).tolist()


def test_plan_batches_respects_batch_size_and_cache():
    assert gen.plan_batches([5, 5, 5, 5, 5], 10, max_batch=2, max_tokens=10**6) == [[0, 1], [2, 3], [4]]
    # 100 + 28 -> 128 cache tokens each; 300 hold two of them
    assert gen.plan_batches([100, 100, 100], 28, max_batch=8, max_tokens=300) == [[0, 1], [2]]
    with pytest.raises(ValueError):
        gen.plan_batches([1000], 28, 8, 512)


def test_finish_reason():
    assert gen.finish_reason(7, 1, 5, {7}, False) == "stop"
    assert gen.finish_reason(7, 1, 5, {7}, True) is None
    assert gen.finish_reason(3, 5, 5, {7}, False) == "length"
    assert gen.finish_reason(7, 5, 5, {7}, False) == "stop"
    assert gen.finish_reason(3, 4, 5, {7}, False) is None


def test_unequal_prompts_stop_tokens_and_early_finishers():
    eng, smp = FakeEngine(), Greedy()
    prompts = [[1, 2, 3], [8], [20, 21]]
    out = gen.generate(eng, smp, prompts, max_new_tokens=6, stop_token_ids=[10], max_batch=4, max_tokens=10**6)
    assert out[0].tokens == [4, 5, 6, 7, 8, 9] and out[0].finish_reason == "length"
    assert out[1].tokens == [9, 10] and out[1].finish_reason == "stop"       # the stop token is kept
    assert out[2].tokens == [22, 23, 24, 25, 26, 27]
    kinds = [k for k, _, _ in eng.steps]
    assert kinds == ["prefill"] + ["decode"] * 5
    assert eng.steps[0][2] == [3, 1, 2]                                      # one step for all prompts
    assert [len(s) for _, s, _ in eng.steps] == [3, 3, 2, 2, 2, 2]           # the short one left the batch
    assert not eng.live and eng.free == [0, 1, 2, 3]


def test_batches_one_after_another_reuse_slots():
    eng, smp = FakeEngine(slots=2), Greedy()
    out = gen.generate(eng, smp, [[i] for i in range(5)], max_new_tokens=3, max_batch=2, max_tokens=10**6)
    assert [g.tokens for g in out] == [[i + 1, i + 2, i + 3] for i in range(5)]
    assert eng.max_live == 2 and not eng.live
    assert [k for k, _, _ in eng.steps].count("prefill") == 3
    assert smp.last == ([4], [2])                                            # sequence id = request index; step count


def test_ignore_eos_and_zero_budget_and_empty_prompt():
    eng, smp = FakeEngine(), Greedy()
    out = gen.generate(eng, smp, [[8]], 4, stop_token_ids=[9], ignore_eos=True, max_tokens=10**6)
    assert out[0].tokens == [9, 10, 11, 12] and out[0].finish_reason == "length"
    out = gen.generate(eng, smp, [[8]], 0, max_tokens=10**6)
    assert out[0].tokens == [] and out[0].finish_reason == "length" and not eng.steps[5:]
    with pytest.raises(ValueError):
        gen.generate(eng, smp, [[]], 4, max_tokens=10**6)


def test_slots_come_back_when_a_step_fails():
    class Failing(FakeEngine):
        def step(self, slots, tokens, want=None):
            if len(self.steps) == 2:
                raise RuntimeError("boom")
            return super().step(slots, tokens, want)

    eng = Failing()
    with pytest.raises(RuntimeError):
        gen.generate(eng, Greedy(), [[1], [2]], 5, max_tokens=10**6)
    assert not eng.live and eng.free == [0, 1, 2, 3]


class AheadEngine(FakeEngine):
    """The same model behind the interface of an engine that samples on the device and lets decode
    steps run one ahead of the host: `step(..., sampling, token_from, wait)`."""

    fused_sampling = True
    overlapped_decode = True

    def __init__(self, vocab=50, slots=4, refuse_ahead_at=None):
        super().__init__(vocab, slots)
        self.last_sampled = []
        self.refuse_ahead_at = refuse_ahead_at           # decode step number whose run-ahead submission finds no room
        self.ahead_submissions = 0

    class _Pending:
        def __init__(self, tokens):
            self._tokens = tokens

        def tokens(self):
            return list(self._tokens)

    def step(self, slots, tokens, want=None, sampling=None, token_from=None, wait=True):
        assert sampling is not None and list(sampling.sequence_ids) is not None
        if token_from is not None:
            self.ahead_submissions += 1
            if self.refuse_ahead_at is not None and self.ahead_submissions == self.refuse_ahead_at:
                raise gen.CacheFull("no room to run ahead")
            tokens = [[self.last_sampled[j]] if j is not None else t for t, j in zip(tokens, token_from)]
        for s in slots:
            assert s in self.live                         # a released slot is never stepped again
        logits = super().step(slots, tokens)
        chosen = logits.argmax(dim=-1).tolist()
        self.last_sampled = chosen
        self.requests_seen = (list(sampling.sequence_ids), list(sampling.steps))
        return (logits, chosen) if wait else (logits, self._Pending(chosen))


class Requester:
    """The sampler's side of fused sampling: it only says which draw each sequence is at."""

    def request(self, ids, step):
        class R:
            sequence_ids, steps = list(ids), [step] * len(ids)
        return R


@pytest.mark.parametrize("refuse", [None, 2])
def test_decode_ahead_gives_the_same_tokens_and_drops_what_ran_too_far(refuse):
    eng = AheadEngine(refuse_ahead_at=refuse)
    prompts = [[1, 2, 3], [8], [20, 21], [30]]
    out = gen.generate(eng, Requester(), prompts, max_new_tokens=6, stop_token_ids=[10, 33], max_batch=4,
                       max_tokens=10**6)
    assert out[0].tokens == [4, 5, 6, 7, 8, 9] and out[0].finish_reason == "length"
    assert out[1].tokens == [9, 10] and out[1].finish_reason == "stop"       # ended by the first decode step
    assert out[2].tokens == [22, 23, 24, 25, 26, 27] and out[2].finish_reason == "length"
    assert out[3].tokens == [31, 32, 33] and out[3].finish_reason == "stop"
    assert not eng.live and eng.free == [0, 1, 2, 3]
    sizes = [len(s) for k, s, _ in eng.steps if k == "decode"]
    if refuse is None:
        # the step after a stop token still carries the sequence that stopped: one row too many, once each
        assert sizes == [4, 4, 3, 2, 2]
    assert len(sizes) == 5                                                   # never a step more than needed


def test_decode_ahead_when_everyone_stops_at_once():
    eng = AheadEngine()
    out = gen.generate(eng, Requester(), [[5], [5]], max_new_tokens=9, stop_token_ids=[7], max_batch=4, max_tokens=10**6)
    assert [g.tokens for g in out] == [[6, 7], [6, 7]] and not eng.live
    # prompt step, the decode step that produced the stop tokens, and the one that had run ahead of them
    assert [k for k, _, _ in eng.steps] == ["prefill", "decode", "decode"]
