"""Steps that bring several tokens on top of started sequences (kind "append"), against the plain
implementation: the reference's own split (a 129-token prompt, then 144 tokens in one call,
tests/lfm3.rs:127-130), prompts cut into chunks of unequal sizes, batches whose sequences stand
at unequal positions and bring unequal numbers of tokens, a new sequence joining started ones,
a ring that wraps inside one appended chunk; and the kernels of that path alone."""
import pytest
import torch

import plain_lfm3
import tiny
from test_engine_gpu import check, plain_logits
from test_kernels_gpu import _paged_cache, _ref_attention, close, rnd

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("append")
    return {name: tiny.make_folder(tmp, name, seed=20 + i) for i, name in enumerate(tiny.ALL)}


@pytest.fixture(scope="module")
def plain(folders):
    return {name: plain_lfm3.load_folder(f) for name, f in folders.items()}


_models = {}


def engine_for(folders, name, dtype):
    from catena_models_b200.api import Model

    key = (name, dtype)
    if key not in _models:
        _models[key] = Model.load(folders[name], dtype=dtype, max_tokens=4096)
    return _models[key].engine


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tiny.ALL))
def test_a_prompt_of_129_then_144_appended_in_one_step(folders, plain, name, dtype):
    eng = engine_for(folders, name, dtype)
    vocab = plain[name][0]["vocab_size"]
    tokens = tiny.random_prompt(129 + 144 + 3, vocab, seed=5)
    exact, same = plain_logits(plain, name, tokens, dtype)
    (slot,) = eng.admit(1)
    steps0 = eng.steps_run
    rows = [eng.step([slot], [tokens[:129]], [[0, 128]]).clone()]
    rows.append(eng.step([slot], [tokens[129:273]], [list(range(144))]).clone())        # one step, every place wanted
    for t in tokens[273:]:
        rows.append(eng.step([slot], [[t]]).clone())                                    # decode on what both left
    assert eng.steps_run - steps0 == 2 + 3
    eng.release([slot])
    pos = [0, 128] + list(range(129, 276))
    check(torch.cat(rows), exact[pos], dtype, None if same is None else same[pos])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "L"])
def test_chunks_of_unequal_sizes_give_the_whole_prompts_logits(folders, plain, name, dtype):
    """Cuts at a page's edge, inside a page, chunks of one token, chunks longer than the sliding
    layers' rings (L: window 70, ring 128; a chunk of 150 overwrites every entry of the ring)."""
    eng = engine_for(folders, name, dtype)
    vocab = plain[name][0]["vocab_size"]
    tokens = tiny.random_prompt(400, vocab, seed=6)
    exact, same = plain_logits(plain, name, tokens, dtype)
    for cuts in ([64, 1, 63, 150, 2, 120], [1, 1, 70, 128, 200], [399, 1], [7, 393]):
        assert sum(cuts) == 400
        (slot,) = eng.admit(1)
        rows, at = [], 0
        for n in cuts:
            rows.append(eng.step([slot], [tokens[at:at + n]], [list(range(n))]).clone())
            at += n
        eng.release([slot])
        check(torch.cat(rows), exact, dtype, same)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C", "L"])
def test_batches_at_unequal_positions_with_a_newcomer(folders, plain, name, dtype):
    """Three sequences prefilled to unequal lengths; then a step in which each brings another number
    of tokens (one of them a single token) and a fourth sequence starts; then decode steps of all."""
    eng = engine_for(folders, name, dtype)
    vocab = plain[name][0]["vocab_size"]
    first, more, tail = [70, 3, 129], [40, 1, 90], 4
    seqs = [tiny.random_prompt(a + b + tail, vocab, seed=30 + i) for i, (a, b) in enumerate(zip(first, more))]
    late = tiny.random_prompt(33 + tail, vocab, seed=39)
    slots = eng.admit(3)
    got = [[] for _ in range(4)]
    out = eng.step(slots, [s[:a] for s, a in zip(seqs, first)], [list(range(a)) for a in first])
    off = 0
    for i, a in enumerate(first):
        got[i].append(out[off:off + a].clone())
        off += a
    slots += eng.admit(1)
    step_tokens = [s[a:a + b] for s, a, b in zip(seqs, first, more)] + [late[:33]]
    out = eng.step(slots, step_tokens, [list(range(len(t))) for t in step_tokens])
    off = 0
    for i, t in enumerate(step_tokens):
        got[i].append(out[off:off + len(t)].clone())
        off += len(t)
    everyone = seqs + [late]
    for k in range(tail):
        out = eng.step(slots, [[s[len(s) - tail + k]] for s in everyone])
        for i in range(4):
            got[i].append(out[i:i + 1].clone())
    eng.release(slots)
    assert not eng.cache.book.live
    for i, s in enumerate(everyone):
        exact, same = plain_logits(plain, name, s, dtype)
        check(torch.cat(got[i]), exact, dtype, same)


def test_session_appends_in_one_step(folders, plain):
    from catena_models_b200.api import Model

    name = "B"
    cfg, tensors = plain[name]
    model = Model.load(folders[name], dtype="float32", max_tokens=1024)
    tokens = tiny.random_prompt(90, cfg["vocab_size"], seed=8)
    exact = plain_lfm3.forward(cfg, tensors, tokens)
    with model.session(128) as s:
        s.prefill_logits(tokens[:20])
        before = model.engine.steps_run
        row = s.append_logits(tokens[20:90])
        assert model.engine.steps_run == before + 1 and s.position == 90
        assert float((row.double() - exact[89]).abs().max() / exact[89].abs().max()) < 2e-5
        with pytest.raises(ValueError):
            s.append_logits(tokens[:60])                    # beyond the session's capacity


def test_a_model_with_a_part_without_an_append_form_is_told_so(folders):
    """The engine refuses the step (nothing runs); the session falls back to single tokens."""
    from catena_models_b200.api import Model
    from catena_models_b200.engine.engine import StepError

    model = Model.load(folders["A"], dtype="float32", max_tokens=512)
    model.decoder.supports_append = False
    eng = model.engine
    (slot,) = eng.admit(1)
    eng.step([slot], [[1, 2, 3]])
    with pytest.raises(StepError):
        eng.step([slot], [[4, 5]])
    assert eng.length(slot) == 3
    eng.release([slot])
    with model.session(64) as s:
        s.prefill_logits([1, 2, 3])
        before = eng.steps_run
        s.append_logits([4, 5, 6])
        assert eng.steps_run == before + 3


# ------------------------------------------------------------------ the kernels alone
@pytest.mark.parametrize("dtype,tensor_cores", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)])
@pytest.mark.parametrize("QH,KVH,HD,window", [(4, 2, 16, 0), (6, 1, 32, 70), (8, 2, 64, 0), (2, 2, 128, 100), (3, 1, 24, 9),
                                              (2, 1, 192, 0), (5, 5, 48, 64)])
def test_attn_append_reads_the_past_from_the_pages(dtype, tensor_cores, QH, KVH, HD, window):
    """Sequences that stand at 0, inside a page, on a page's edge and beyond a ring's size bring
    1 to 150 tokens; keys below their first new position lie in shuffled pages whose unused entries
    are NaN, the rest in the step's rows.  Against float64 attention over the whole sequences."""
    from catena_models_b200 import kernels as K

    ring = (window + 63) // 64 * 64 if window else 0
    past = [0, 5, 64, 130, 200, 257]
    new = [33, 1, 70, 150, 64, 2]
    g = torch.Generator().manual_seed(HD + window)
    kv = [torch.randn(p + n, 2, KVH, HD, generator=g) for p, n in zip(past, new)]
    # the cache as the steps before left it: positions below `past` (a ring: the last `ring` of them)
    stored = [x[:p] for x, p in zip(kv, past)]
    pool, pages, ptab = _paged_cache(K, stored, KVH, HD, dtype, past, ring)
    # _paged_cache sized the tables for the past alone; an append kernel only reads, so that is enough
    T = sum(new)
    width = (QH * HD + 2 * KVH * HD + QH + 7) // 8 * 8
    buf = rnd(T, width, dtype=dtype, seed=HD)
    q = buf[:, :QH * HD]
    k, v = buf[:, QH * HD:QH * HD + KVH * HD], buf[:, QH * HD + KVH * HD:QH * HD + 2 * KVH * HD]
    gate = buf[:, QH * HD + 2 * KVH * HD:QH * HD + 2 * KVH * HD + QH]
    starts, off = [0], 0
    for b, (p, n) in enumerate(zip(past, new)):
        k[off:off + n] = kv[b][p:, 0].reshape(n, KVH * HD).to(dtype).to(DEV)
        v[off:off + n] = kv[b][p:, 1].reshape(n, KVH * HD).to(dtype).to(DEV)
        off += n
        starts.append(off)
    starts = torch.tensor(starts, dtype=torch.int32, device=DEV)
    pos0 = torch.tensor(past, dtype=torch.int32, device=DEV)
    slots = torch.arange(1, len(past) + 1, dtype=torch.int32, device=DEV)
    ctx = torch.full((T, QH * HD), float("nan"), dtype=dtype, device=DEV)
    scale = HD ** -0.5
    if tensor_cores and (HD % 16 or HD > 128):
        tensor_cores = False                              # such head sizes go to the CUDA cores
    K.attn_append(ctx, q, k, v, gate, starts, pos0, slots, pool, pages, ptab, ring, len(past), max(new), QH, KVH, HD,
                  window, scale, tensor_cores=tensor_cores)
    off = 0
    for b, (p, n) in enumerate(zip(past, new)):
        qq = torch.zeros(p + n, QH, HD)
        qq[p:] = q[off:off + n].float().cpu().view(n, QH, HD)
        gg = torch.zeros(p + n, QH)
        gg[p:] = gate[off:off + n].float().cpu()
        ref = _ref_attention(qq, kv[b][:, 0].to(dtype), kv[b][:, 1].to(dtype), window, scale, gg)[p:]
        close(ctx[off:off + n].view(n, QH, HD), ref, dtype)
        off += n


@pytest.mark.parametrize("QH,KVH,HD,window", [(8, 2, 64, 0), (2, 2, 128, 100), (4, 1, 64, 300), (3, 3, 128, 0),
                                              (2, 1, 64, 64)])
def test_attn_append_on_tcgen05_copies_pages_and_masks_what_is_not_the_sequences(QH, KVH, HD, window):
    """The tcgen05 form copies whole pages of the cache into a matrix operand.  Sequences that stand
    at 0, inside a page, on a page's edge, in the second page of a 128-key tile, beyond a ring's size
    and several tiles in; the unused entries of the cache are NaN, and so are the rows of the step's
    buffer behind the last sequence's (the kernel clears what is not the sequence's in its copy of a
    value tile).  Against float64 attention over the whole sequences; no pipeline wait may have run
    out, and the cache is left as it was."""
    _append_on_tcgen05([0, 5, 64, 130, 200, 257, 700], [33, 1, 70, 150, 64, 2, 300], QH, KVH, HD, window)


@pytest.mark.parametrize("seed,QH,KVH,HD,window", [(1, 8, 2, 64, 0), (2, 4, 2, 128, 0), (3, 6, 3, 64, 192), (4, 2, 1, 128, 64)])
def test_attn_append_on_tcgen05_with_many_sequences(seed, QH, KVH, HD, window):
    """The same with 24 to 40 sequences at positions 0 to 900 that bring 1 to 260 rows each: every block of the
    kernel walks many (query tile, head, sequence) items, of one key tile and of eight, from the cache and from
    the step, one after another."""
    import random
    rng = random.Random(seed)
    n_seq = rng.randint(24, 40)
    past = [rng.choice([0, 1, 63, 64, 65, 128, 129, rng.randint(0, 900)]) for _ in range(n_seq)]
    new = [rng.choice([1, 2, 16, 64, 65, 128, 129, rng.randint(1, 260)]) for _ in range(n_seq)]
    _append_on_tcgen05(past, new, QH, KVH, HD, window)


def _append_on_tcgen05(past, new, QH, KVH, HD, window):
    from catena_models_b200 import kernels as K

    dtype = torch.bfloat16
    ring = (window + 63) // 64 * 64 if window else 0
    g = torch.Generator().manual_seed(HD + window)
    kv = [torch.randn(p + n, 2, KVH, HD, generator=g) for p, n in zip(past, new)]
    stored = [x[:p] for x, p in zip(kv, past)]
    pool, pages, ptab = _paged_cache(K, stored, KVH, HD, dtype, past, ring)
    T = sum(new)
    width = (QH * HD + 2 * KVH * HD + QH + 7) // 8 * 8
    buf = rnd(T, width, dtype=dtype, seed=HD)
    q = buf[:, :QH * HD]
    k, v = buf[:, QH * HD:QH * HD + KVH * HD], buf[:, QH * HD + KVH * HD:QH * HD + 2 * KVH * HD]
    gate = buf[:, QH * HD + 2 * KVH * HD:QH * HD + 2 * KVH * HD + QH]
    starts, off = [0], 0
    for b, (p, n) in enumerate(zip(past, new)):
        k[off:off + n] = kv[b][p:, 0].reshape(n, KVH * HD).to(dtype).to(DEV)
        v[off:off + n] = kv[b][p:, 1].reshape(n, KVH * HD).to(dtype).to(DEV)
        off += n
        starts.append(off)
    starts = torch.tensor(starts, dtype=torch.int32, device=DEV)
    pos0 = torch.tensor(past, dtype=torch.int32, device=DEV)
    slots = torch.arange(1, len(past) + 1, dtype=torch.int32, device=DEV)
    ctx = torch.full((T, QH * HD), float("nan"), dtype=dtype, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = HD ** -0.5
    held = pool.clone()
    K.attn_append_tc(ctx, q, k, v, gate, starts, pos0, slots, pool, pages, ptab, ring, len(past), max(new), QH, KVH, HD,
                     window, scale, err=err)
    assert int(err.item()) == 0
    same = (pool == held) | (pool.isnan() & held.isnan())
    assert bool(same.all())                                # the kernel only reads the cache
    off = 0
    for b, (p, n) in enumerate(zip(past, new)):
        qq = torch.zeros(p + n, QH, HD)
        qq[p:] = q[off:off + n].float().cpu().view(n, QH, HD)
        gg = torch.zeros(p + n, QH)
        gg[p:] = gate[off:off + n].float().cpu()
        ref = _ref_attention(qq, kv[b][:, 0].to(dtype), kv[b][:, 1].to(dtype), window, scale, gg)[p:]
        close(ctx[off:off + n].view(n, QH, HD), ref, dtype)
        off += n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("KVH,HD,ring", [(2, 16, 0), (1, 24, 64), (3, 64, 128)])
def test_kv_store_writes_what_qk_prepare_would(dtype, KVH, HD, ring):
    from catena_models_b200 import kernels as K

    past, new = [0, 70, 129], [150, 3, 64]
    ends = [p + n for p, n in zip(past, new)]
    per_seq = [((min(e, ring) if ring else e) + 63) // 64 for e in ends]
    pages = sum(per_seq) + 2
    perm = torch.randperm(pages, generator=torch.Generator().manual_seed(1)).tolist()
    ptab = torch.full((len(past) + 1, max(per_seq)), -1, dtype=torch.int32)
    nxt = 0
    for b, n in enumerate(per_seq):
        for j in range(n):
            ptab[b + 1, j] = perm[nxt]
            nxt += 1
    ptab = ptab.to(DEV)
    T = sum(new)
    rows = rnd(T, 2 * KVH * HD + 8, dtype=dtype, seed=3)
    tok_pos = torch.tensor([p + i for p, n in zip(past, new) for i in range(n)], dtype=torch.int32, device=DEV)
    tok_seq = torch.tensor([b for b, n in enumerate(new) for _ in range(n)], dtype=torch.int32, device=DEV)
    slots = torch.arange(1, len(past) + 1, dtype=torch.int32, device=DEV)
    seq_end = torch.tensor(ends, dtype=torch.int32, device=DEV)
    pool = torch.full((2, pages, KVH, 64, HD), float("nan"), dtype=dtype, device=DEV)
    K.kv_store(rows[:, :2 * KVH * HD], tok_pos, tok_seq, slots, seq_end, pool, pages, ptab, ring, KVH, HD)
    want = torch.full_like(pool, float("nan"))
    t = 0
    for b, (p, n) in enumerate(zip(past, new)):
        for i in range(n):
            pos = p + i
            if not ring or pos + ring >= ends[b]:
                e = pos % ring if ring else pos
                page = int(ptab[b + 1, e // 64])
                want[0, page, :, e % 64] = rows[t, :KVH * HD].view(KVH, HD)
                want[1, page, :, e % 64] = rows[t, KVH * HD:2 * KVH * HD].view(KVH, HD)
            t += 1
    assert torch.equal(torch.nan_to_num(pool.float(), nan=-7.0), torch.nan_to_num(want.float(), nan=-7.0))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,taps", [(72, 3), (200, 4), (27, 3), (136, 7)])
def test_shortconv_in_chunks_equals_the_whole(dtype, H, taps):
    """A sequence's rows run whole (from an empty state) and in chunks on top of the stored state,
    chunks shorter than the taps among them; a second sequence of the chunked steps starts at 0
    while the first one is under way.  Outputs and the final state must be equal bit for bit."""
    from catena_models_b200 import kernels as K

    n = 90
    bcx = rnd(n, 3 * H, dtype=dtype, seed=H)
    other = rnd(40, 3 * H, dtype=dtype, seed=H + 1)
    w = rnd(H, taps, dtype=torch.float32, seed=2)

    def run(rows, state, tok_seq, seq_start, slots, pos0, from_zero):
        y = torch.full((rows.shape[0], H), float("nan"), dtype=dtype, device=DEV)
        K.shortconv(y, rows, w, state, tok_seq, seq_start, slots, taps, from_zero=from_zero, one_token_each=False,
                    seq_pos0=pos0)
        return y

    i32 = lambda xs: torch.tensor(xs, dtype=torch.int32, device=DEV)
    state = torch.full((3, taps - 1, H), float("nan"), dtype=torch.float32, device=DEV)
    whole = run(bcx, state, i32([0] * n), i32([0, n]), i32([1]), None, True)
    whole_other = run(other, state, i32([0] * 40), i32([0, 40]), i32([2]), None, True)
    final = state.clone()

    state2 = torch.full((3, taps - 1, H), float("nan"), dtype=torch.float32, device=DEV)
    state2[1:] = 0                                         # admitted slots start cleared
    outs, at = [], 0
    for step, size in enumerate([1, 2, 30, 1, 56]):
        if step == 2:                                      # the other sequence joins here, whole
            rows = torch.cat([bcx[at:at + size], other])
            y = run(rows, state2, i32([0] * size + [1] * 40), i32([0, size, size + 40]), i32([1, 2]), i32([at, 0]), False)
            outs.append(y[:size])
            assert torch.equal(y[size:], whole_other)
        else:
            outs.append(run(bcx[at:at + size].contiguous(), state2, i32([0] * size), i32([0, size]), i32([1]), i32([at]),
                            False))
        at += size
    assert torch.equal(torch.cat(outs), whole)
    assert torch.equal(state2[1:], final[1:])
