"""The engine against the plain implementation: whole prompts, the last tokens one by one,
unequal batches with early finishers and slot reuse, long decoding, first tokens, in 32-bit
and in bfloat16."""
import pytest
import torch

import plain_lfm3
import tiny

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# Error measure: largest |engine - plain| over all logits of a comparison, relative to the
# largest |logit|.
# float32: rounding of a few thousand float32 operations against float64.
# bfloat16: the yardstick is the plain implementation run with the reference's own
# round-to-bfloat16 points (same inputs, otherwise exact arithmetic): its distance from the
# exact result is the noise that the storage format itself causes on this input.  Single
# roundings flip differently in the engine (other summation order, unrounded scores inside the
# fused attention), so the two bfloat16 results are not compared with each other; the engine
# must stay within twice the yardstick's distance from the exact result, over the whole
# comparison and row by row.
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


def row_errs(got, ref):
    """Per row: the largest |got - ref| of the row relative to the row's own largest |ref|."""
    ref = ref.to(torch.float64).cpu()
    return (got.to(torch.float64).cpu() - ref).abs().amax(-1) / ref.abs().amax(-1)


def check(got, ref_exact, dtype, ref_same=None):
    if dtype == "float32":
        assert rel_err(got, ref_exact) < TOL_F32
        assert float(row_errs(got, ref_exact).max()) < 2 * TOL_F32
    else:
        assert ref_same is not None
        assert rel_err(got, ref_exact) < BF16_FACTOR * rel_err(ref_same, ref_exact)
        # and row by row, each against its own scale, so that a wrong row of small logits cannot hide
        # under the largest logit of the comparison; the bound is the yardstick's own worst row
        assert float(row_errs(got, ref_exact).max()) < BF16_FACTOR * float(row_errs(ref_same, ref_exact).max())


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
    eng.step([slot], [[1, 2]])                      # two tokens on top of a started sequence: an append step
    assert eng.length(slot) == 5
    with pytest.raises(CacheFull):
        (other,) = eng.admit(1)
        try:
            eng.step([other], [[1] * 4000])         # more than the cache holds
        finally:
            eng.release([other])
    eng.release([slot])
    assert not eng.cache.book.live
    assert eng.cache.book.page_alloc[0].free_count == eng.cache.book.group_pages[0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_planted_far_key_decides_the_logits(dtype):
    """Random weights can hide a key that attention never sees: among hundreds it moves the logits
    by little.  Here the weights are made so that the last token's queries point at the key of the
    very first token (600 positions back, on the first page of the cache) and at nothing else, so
    that token's value decides the output: in the prompt step and in decode steps over the cache."""
    from catena_models_b200.api import Model
    from catena_models_b200.config.registry import config_from_dict
    from catena_models_b200.engine.model import DecoderModel
    from catena_models_b200.weights.random_init import random_tensors

    cfg = dict(architecture="lfm3", vocab_size=97, hidden_size=64, intermediate_size=96, num_hidden_layers=1,
               layer_types=["full_attention"], num_attention_heads=2, num_key_value_heads=1, head_dim=32,
               conv_L_cache=3, sliding_window=64, rope_theta=10000.0, norm_eps=1e-6, tie_word_embeddings=True,
               max_position_embeddings=2048, post_norm=True, attn_output_gate=False)
    arch, typed = config_from_dict(cfg)
    t = random_tensors(arch.define(typed).tensor_specs(), 3, std=0.5)
    A, B = 7, 9                                                  # the far token and the asking token
    pre = "model.layers.0."
    emb = t["model.embed_tokens.weight"].float()
    unit = lambda v: v / v.pow(2).mean().add(1e-6).sqrt()        # the layer's input norm (weight 1)
    n_a, n_b = unit(emb[A]), unit(emb[B])
    k_a = t[pre + "attn_k.weight"].float() @ n_a                 # the key of token A, before head norm
    wq = 0.002 * torch.randn(64, 64, generator=torch.Generator().manual_seed(1))
    for h in range(2):                                           # both query heads: q(B) = k(A) + a little noise
        wq[32 * h:32 * h + 32] += torch.outer(k_a, n_b) / n_b.dot(n_b)
    t[pre + "attn_q.weight"] = wq.to(torch.bfloat16)
    t[pre + "attn_q_norm.weight"] = torch.full((32,), 4.0)       # head norms scale the scores: a match scores about 90
    t[pre + "attn_k_norm.weight"] = torch.full((32,), 4.0)
    t["rope_freqs.weight"] = torch.full((16,), 1e9)              # factors so large that no position turns anything
    g = torch.Generator().manual_seed(2)
    filler = [int(x) for x in torch.randint(10, 97, (600,), generator=g)]
    seq = [A] + filler + [B, B, B, B]
    other = [11] + filler + [B, B, B, B]                         # the same without the planted token
    tensors64 = {k: v.double() if v.is_floating_point() else v for k, v in t.items()}
    exact = plain_lfm3.forward(cfg, tensors64, seq)
    without = plain_lfm3.forward(cfg, tensors64, other)
    rng = float(exact[601:].abs().max())
    assert float((exact[601:] - without[601:]).abs().max()) > 0.2 * rng      # the planted key matters a lot

    model = Model(DecoderModel.from_tensors(cfg, t, torch.float32 if dtype == "float32" else torch.bfloat16, DEV), max_tokens=1024)
    eng = model.engine
    (slot,) = eng.admit(1)
    got = [eng.step([slot], [seq[:602]], [[600, 601]]).clone()]            # the last filler and the first B
    for tok in seq[602:]:
        got.append(eng.step([slot], [[tok]]).clone())
    eng.release([slot])
    got = torch.cat(got)
    ref = exact[600:]
    if dtype == "float32":
        assert rel_err(got, ref) < 5e-5
    else:
        same = plain_lfm3.forward(cfg, tensors64, seq, bf16=True)[600:]
        assert rel_err(got, ref) < BF16_FACTOR * rel_err(same, ref) + 1e-3
    # and far from what the sequence without the planted token gives
    assert rel_err(got[1:], without[601:]) > 0.1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_prompt_steps_of_a_repeated_shape(folders, plain, name, dtype):
    """A prompt step whose shape repeats is recorded at its second run and replayed after that.
    Six batches of the same lengths, each with other tokens and on other slots (one slot stays
    held in between so that the slots and pages move), must each match the plain implementation,
    and a result handed out earlier must not change when the graph runs again."""
    eng = engine_for(folders, name, dtype)
    vocab = plain[name][0]["vocab_size"]
    lens = (9, 70, 31)
    held, earlier = [], []
    for rep in range(6):
        prompts = [tiny.random_prompt(n, vocab, seed=1000 * rep + n) for n in lens]
        slots = eng.admit(len(lens))
        got = eng.step(slots, prompts)
        earlier.append((got, got.clone()))
        nxt = [tiny.random_prompt(1, vocab, seed=77 + rep + n) for n in lens]
        got2 = eng.step(slots, nxt).clone()                    # a decode step on what the prompt step left
        for b, (p, t) in enumerate(zip(prompts, nxt)):
            exact, same = plain_logits(plain, name, p + t, dtype)
            rows = torch.stack([got[b], got2[b]])
            check(rows, exact[-2:], dtype, None if same is None else same[-2:])
        eng.release(slots[1:])
        held.append(slots[0])
    assert len(eng._prompt_graphs) >= 1
    for handed, copy in earlier:
        assert torch.equal(handed, copy)
    eng.release(held)


def test_recorded_prompt_shapes_are_bounded_and_evicted_ones_run_again(folders, plain, monkeypatch):
    """More repeated prompt shapes than the engine keeps graphs for (eight here): the oldest recording is
    dropped, and a dropped shape that comes back runs kernel by kernel again with the same result."""
    from catena_models_b200.engine import engine as engine_module

    PROMPT_GRAPHS_KEPT = 8
    monkeypatch.setattr(engine_module, "PROMPT_GRAPHS_KEPT", PROMPT_GRAPHS_KEPT)
    name, dtype = "A", "bfloat16"
    from catena_models_b200.api import Model

    eng = Model.load(folders[name], dtype=dtype, max_tokens=2048).engine       # an engine without recordings
    vocab = plain[name][0]["vocab_size"]
    shapes = [(40 + 64 * i,) for i in range(PROMPT_GRAPHS_KEPT + 3)]       # one class of shapes each
    for rnd in range(2):
        for lens in shapes:
            for rep in range(3):
                prompts = [tiny.random_prompt(n, vocab, seed=rnd * 100 + rep * 10 + n) for n in lens]
                slots = eng.admit(len(lens))
                got = eng.step(slots, prompts)
                eng.release(slots)
                exact, same = plain_logits(plain, name, prompts[0], dtype)
                check(got, exact[-1:], dtype, same[-1:])
            assert len(eng._prompt_graphs) <= PROMPT_GRAPHS_KEPT


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "L"])
def test_one_recording_serves_a_class_of_prompt_shapes(folders, plain, name, dtype):
    """Prompt steps are recorded per class (sequences, tokens and longest prompt rounded up to 64, wanted
    places): the step runs the class's rows, the surplus as padding that belongs to no sequence.  Prompts
    of many lengths in one class, alone and in pairs of unequal lengths, each followed by a decode step,
    must all match the plain model, whether they ran kernel by kernel (the first two of a class) or were
    replayed; padding must leave cache and fixed-size state alone (the decode step would show it)."""
    eng = engine_for(folders, name, dtype)
    vocab = plain[name][0]["vocab_size"]
    all_got, all_exact, all_same = [], [], []
    for rep, lens in enumerate([(30, 50), (1, 100), (64, 64), (90, 20), (5, 70), (65,), (100,), (128,), (77,), (66,), (127,)]):
        seqs = [tiny.random_prompt(n + 1, vocab, seed=500 + 10 * rep + i) for i, n in enumerate(lens)]
        slots = eng.admit(len(lens))
        got = eng.step(slots, [s[:-1] for s in seqs], [[0, n - 1] if n > 1 else [0] for n in lens]).clone()
        got2 = eng.step(slots, [[s[-1]] for s in seqs]).clone()
        eng.release(slots)
        off = 0
        for i, (s, n) in enumerate(zip(seqs, lens)):
            exact, same = plain_logits(plain, name, s, dtype)
            places = [0, n - 1] if n > 1 else [0]
            all_got.append(torch.cat([got[off:off + len(places)], got2[i:i + 1]]))
            off += len(places)
            all_exact.append(exact[places + [n]])
            if same is not None:
                all_same.append(same[places + [n]])
    # one comparison over all rows: the bfloat16 yardstick is a maximum and needs more than two rows to be one
    check(torch.cat(all_got), torch.cat(all_exact), dtype, torch.cat(all_same) if all_same else None)
    # the six single prompts are one class (128 rows, two wanted places), recorded at its second prompt
    assert (1, 128, 128, 2, False) in eng._prompt_graphs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "L"])
def test_one_recording_serves_a_class_of_append_steps(folders, plain, name, dtype):
    """Tokens on top of held ones are recorded per class as well (the class also names the class of
    lengths that the longest sequence reaches).  Requests with heads of many lengths bring second
    pieces of 33 to 64 tokens, alone and in pairs of unequal lengths, then one more token each: the
    first of a class runs kernel by kernel, the second is recorded, the others are replayed, and all
    must match the plain model; the padding rows of a replay must leave cache and state alone."""
    eng = engine_for(folders, name, dtype)
    vocab = plain[name][0]["vocab_size"]
    all_got, all_exact, all_same = [], [], []
    cases = [((10, 40),), ((70, 64),), ((1, 33),), ((120, 50),), ((64, 64),), ((33, 45),),
             ((10, 20), (50, 30)), ((64, 1), (5, 60)), ((100, 33), (3, 31)), ((20, 40), (90, 24))]
    for rep, case in enumerate(cases):
        seqs = [tiny.random_prompt(h + n + 1, vocab, seed=900 + 10 * rep + i) for i, (h, n) in enumerate(case)]
        slots = eng.admit(len(case))
        eng.step(slots, [s[:h] for s, (h, n) in zip(seqs, case)], [[] for _ in case])
        got = eng.step(slots, [s[h:h + n] for s, (h, n) in zip(seqs, case)], [[0, n - 1] if n > 1 else [0] for h, n in case]).clone()
        got2 = eng.step(slots, [[s[-1]] for s in seqs]).clone()
        eng.release(slots)
        off = 0
        for i, (s, (h, n)) in enumerate(zip(seqs, case)):
            exact, same = plain_logits(plain, name, s, dtype)
            places = [h, h + n - 1] if n > 1 else [h]
            all_got.append(torch.cat([got[off:off + len(places)], got2[i:i + 1]]))
            off += len(places)
            all_exact.append(exact[places + [h + n]])
            if same is not None:
                all_same.append(same[places + [h + n]])
    check(torch.cat(all_got), torch.cat(all_exact), dtype, torch.cat(all_same) if all_same else None)
    assert any(len(k) > 5 and k[5] == "append" for k in eng._prompt_graphs)
    assert not eng.cache.book.live
