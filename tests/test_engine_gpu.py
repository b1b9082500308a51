"""The engine against the plain implementation: whole prompts, the last tokens one by one,
unequal batches with early finishers and slot reuse, long decoding, first tokens, in 32-bit
and in bfloat16."""
import pytest
import torch

import plain_lfm3
import tiny

pytestmark = pytest.mark.gpu

# Error measure: largest |engine - plain| over all logits of a comparison, relative to the
# largest |logit|.
# float32: rounding of a few thousand float32 operations against float64.
# bfloat16: the yardstick is the plain implementation run with the reference's own
# round-to-bfloat16 points (same inputs, otherwise exact arithmetic): its distance from the
# exact result is the noise that the storage format itself causes on this input.  Single
# roundings flip differently in the engine (other summation order, unrounded scores inside the
# fused attention), so the two bfloat16 results are not compared with each other; the engine
# must stay within twice the yardstick's distance from the exact result.
TOL_F32 = 2e-5
BF16_FACTOR = 2.0


def rel_err(got, ref):
    ref = ref.to(torch.float64).cpu()
    return float((got.to(torch.float64).cpu() - ref).abs().max() / ref.abs().max())


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("models")
    return {name: tiny.make_folder(tmp, name, seed=i) for i, name in enumerate(tiny.ALL)}


@pytest.fixture(scope="module")
def plain(folders):
    return {name: plain_lfm3.load_folder(f) for name, f in folders.items()}


_models = {}


def engine_for(folders, name, dtype):
    """One engine per (model, dtype) for the module, so that later tests run on slots and pages
    that earlier tests have used and given back."""
    from catena_models_b200.api import Model

    key = (name, dtype)
    if key not in _models:
        _models[key] = Model.load(folders[name], dtype=dtype, max_tokens=2048)
    return _models[key].engine


def check(got, ref_exact, dtype, ref_same=None):
    if dtype == "float32":
        assert rel_err(got, ref_exact) < TOL_F32
    else:
        assert ref_same is not None
        assert rel_err(got, ref_exact) < BF16_FACTOR * rel_err(ref_same, ref_exact)


def plain_logits(plain, name, tokens, dtype):
    cfg, tensors = plain[name]
    exact = plain_lfm3.forward(cfg, tensors, tokens)
    same = plain_lfm3.forward(cfg, tensors, tokens, bf16=True) if dtype == "bfloat16" else None
    return exact, same


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tiny.ALL))
def test_whole_prompt_all_positions(folders, plain, name, dtype):
    eng = engine_for(folders, name, dtype)
    vocab = plain[name][0]["vocab_size"]
    for n in (1, 2, 3, 37, 150):
        tokens = tiny.random_prompt(n, vocab, seed=n)
        (slot,) = eng.admit(1)
        got = eng.step([slot], [tokens], [list(range(n))])
        eng.release([slot])
        exact, same = plain_logits(plain, name, tokens, dtype)
        check(got, exact, dtype, same)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tiny.ALL))
def test_last_32_one_by_one(folders, plain, name, dtype):
    eng = engine_for(folders, name, dtype)
    vocab = plain[name][0]["vocab_size"]
    for n in (33, 100, 200):
        tokens = tiny.random_prompt(n, vocab, seed=100 + n)
        exact, same = plain_logits(plain, name, tokens, dtype)
        (slot,) = eng.admit(1)
        head = n - 32
        rows = [eng.step([slot], [tokens[:head]], [[head - 1]])]
        for t in range(head, n):
            rows.append(eng.step([slot], [[tokens[t]]]).clone())
        eng.release([slot])
        got = torch.cat(rows)
        check(got, exact[head - 1:], dtype, None if same is None else same[head - 1:])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tiny.ALL))
def test_unequal_batches_one_after_another(folders, plain, name, dtype):
    """Batches of unequal prompts; every sequence decodes a different number of given tokens, so
    the shorter ones end earlier; the next batch runs on the slots and pages just freed."""
    eng = engine_for(folders, name, dtype)
    vocab = plain[name][0]["vocab_size"]
    batches = [[(5, 8), (11, 3), (17, 12)], [(1, 12), (7, 1), (20, 6), (33, 9)], [(70, 40), (64, 2), (3, 70)]]
    seed = 0
    for batch in batches:
        seqs = []
        for prompt_len, extra in batch:
            seed += 1
            seqs.append(tiny.random_prompt(prompt_len + extra, vocab, seed=1000 + seed))
        slots = eng.admit(len(batch))
        got = [[] for _ in batch]
        out = eng.step(slots, [s[:p] for s, (p, _) in zip(seqs, batch)], [list(range(p)) for p, _ in batch])
        off = 0
        for i, (p, _) in enumerate(batch):
            got[i].append(out[off:off + p].clone())
            off += p
        live = list(range(len(batch)))
        t = 0
        while live:
            live = [i for i in live if batch[i][1] > t]
            for i in list(range(len(batch))):
                if slots[i] is not None and i not in live:
                    eng.release([slots[i]])
                    slots[i] = None
            if not live:
                break
            out = eng.step([slots[i] for i in live], [[seqs[i][batch[i][0] + t]] for i in live])
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1].clone())
            t += 1
        assert not eng.cache.book.live
        for i, s in enumerate(seqs):
            exact, same = plain_logits(plain, name, s, dtype)
            check(torch.cat(got[i]), exact, dtype, same)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_window_and_pages(folders, plain, dtype):
    """300 decoded tokens after a 3-token prompt: crosses four page borders and wraps the ring
    of the sliding layer (window 70, ring 128) more than once."""
    name = "L"
    eng = engine_for(folders, name, dtype)
    vocab = plain[name][0]["vocab_size"]
    tokens = tiny.random_prompt(303, vocab, seed=77)
    exact, same = plain_logits(plain, name, tokens, dtype)
    (slot,) = eng.admit(1)
    rows = [eng.step([slot], [tokens[:3]], [[0, 1, 2]])]
    for t in range(3, 303):
        rows.append(eng.step([slot], [[tokens[t]]]).clone())
    eng.release([slot])
    check(torch.cat(rows), exact, dtype, same)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_longer_than_ring_then_decode(folders, plain, dtype):
    """A 300-token prompt on a ring of 128 entries: only the last entries are stored, and the
    decode steps after it must see exactly the window."""
    name = "L"
    eng = engine_for(folders, name, dtype)
    vocab = plain[name][0]["vocab_size"]
    tokens = tiny.random_prompt(340, vocab, seed=78)
    exact, same = plain_logits(plain, name, tokens, dtype)
    (slot,) = eng.admit(1)
    rows = [eng.step([slot], [tokens[:300]], [[298, 299]])]
    for t in range(300, 340):
        rows.append(eng.step([slot], [[tokens[t]]]).clone())
    eng.release([slot])
    check(torch.cat(rows), exact[298:], dtype, None if same is None else same[298:])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens_of_a_sequence(folders, plain, name, dtype):
    """Prompt of one token, then decode: conv state shorter than its taps, attention over one
    and two keys."""
    eng = engine_for(folders, name, dtype)
    vocab = plain[name][0]["vocab_size"]
    tokens = tiny.random_prompt(6, vocab, seed=5)
    exact, same = plain_logits(plain, name, tokens, dtype)
    (slot,) = eng.admit(1)
    rows = [eng.step([slot], [tokens[:1]])]
    for t in range(1, 6):
        rows.append(eng.step([slot], [[tokens[t]]]).clone())
    eng.release([slot])
    check(torch.cat(rows), exact, dtype, same)


def test_padding_and_batch_mates_change_nothing(folders, plain):
    """The same sequence alone and among others, in float32: equal beyond rounding."""
    name, dtype = "B", "float32"
    eng = engine_for(folders, name, dtype)
    vocab = plain[name][0]["vocab_size"]
    a = tiny.random_prompt(29, vocab, seed=9)
    others = [tiny.random_prompt(n, vocab, seed=20 + n) for n in (2, 61, 13)]
    (slot,) = eng.admit(1)
    alone = eng.step([slot], [a], [list(range(29))]).clone()
    eng.release([slot])
    slots = eng.admit(4)
    seqs = [others[0], a, others[1], others[2]]
    out = eng.step(slots, seqs, [[], list(range(29)), [], [0]])
    eng.release(slots)
    assert rel_err(out[:29], alone) < 1e-6


def test_step_errors(folders):
    from catena_models_b200.engine.engine import StepError
    from catena_models_b200.cache.allocators import CacheFull

    eng = engine_for(folders, "A", "float32")
    (slot,) = eng.admit(1)
    with pytest.raises(StepError):
        eng.step([slot], [[]])
    with pytest.raises(StepError):
        eng.step([slot], [[256]])
    with pytest.raises(StepError):
        eng.step([slot, slot], [[1], [2]])
    with pytest.raises(StepError):
        eng.step([999], [[1]])
    eng.step([slot], [[1, 2, 3]])
    with pytest.raises(StepError):
        eng.step([slot], [[1, 2]])                  # two tokens on top of a started sequence
    with pytest.raises(CacheFull):
        (other,) = eng.admit(1)
        try:
            eng.step([other], [[1] * 4000])         # more than the cache holds
        finally:
            eng.release([other])
    eng.release([slot])
    assert not eng.cache.book.live
    assert eng.cache.book.page_alloc[0].free_count == eng.cache.book.group_pages[0]
