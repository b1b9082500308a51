"""Schedules and guards of the engine that the other files do not reach: head sizes above 128
through the whole engine, a checkpoint stored in 32-bit under the bfloat16 engine, the longest
allowed sequence, a cache so tight that decoding ahead has to wait, recordings that are dropped
and made again, and the device's fault flags."""
import json
import os

import pytest
import torch

import plain_lfm3
import tiny
from test_engine_gpu import check, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _plain(folder, tokens, dtype):
    cfg, tensors = plain_lfm3.load_folder(folder)
    exact = plain_lfm3.forward(cfg, tensors, tokens)
    same = plain_lfm3.forward(cfg, tensors, tokens, bf16=True) if dtype == "bfloat16" else None
    return exact, same


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("head_dim,heads,kv_heads", [(192, 2, 1), (256, 3, 3)])
def test_head_sizes_above_128(tmp_path, dtype, head_dim, heads, kv_heads):
    """Heads of 192 and 256 (the CUDA-core attention kernels in both precisions): a prompt of
    several key tiles, decode over three chunks of the cache, a ring that wraps, an appended chunk."""
    from catena_models_b200.api import Model
    from catena_models_b200.weights.random_init import write_random_model

    cfg = dict(architecture="lfm3", vocab_size=200, hidden_size=128, intermediate_size=256, num_hidden_layers=3,
               layer_types=["full_attention", "conv", "sliding_attention"], num_attention_heads=heads,
               num_key_value_heads=kv_heads, head_dim=head_dim, conv_L_cache=3, sliding_window=100, rope_theta=10000.0,
               rope_theta_sliding=500.0, norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=2048)
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=head_dim, std=0.05, norm_weights="random",
                                rope_factors="uniform")
    tokens = tiny.random_prompt(540, 200, seed=1)
    exact, same = _plain(folder, tokens, dtype)
    eng = Model.load(folder, dtype=dtype, max_tokens=1024).engine
    (slot,) = eng.admit(1)
    rows = [eng.step([slot], [tokens[:300]], [[0, 150, 299]]).clone()]
    rows.append(eng.step([slot], [tokens[300:500]], [[0, 199]]).clone())              # appended in one step
    for t in tokens[500:]:
        rows.append(eng.step([slot], [[t]]).clone())                                  # 501..540 entries: three chunks
    eng.release([slot])
    eng.check_errors()
    pos = [0, 150, 299, 300, 499] + list(range(500, 540))
    check(torch.cat(rows), exact[pos], dtype, None if same is None else same[pos])


def test_bfloat16_engine_over_a_checkpoint_stored_in_32_bit(tmp_path):
    """The embedding (tied head) and the first layers' matrices are stored in float32, with values
    that bfloat16 cannot hold: the bfloat16 engine keeps them in 32-bit, converts embedding rows as
    it gathers them and multiplies by the float matrices on the CUDA cores."""
    from catena_models_b200.api import Model
    from catena_models_b200.config.registry import config_from_dict
    from catena_models_b200.weights.random_init import random_tensors
    from catena_models_b200.weights.safetensors_io import write_safetensors

    cfg = tiny.TINY_A
    arch, typed = config_from_dict(cfg)
    tensors = random_tensors(arch.define(typed).tensor_specs(), 4, **tiny.RANDOM_A)
    g = torch.Generator().manual_seed(0)
    stored32 = ["model.embed_tokens.weight"] + [n for n in tensors if n.startswith(("model.layers.0.", "model.layers.1."))
                                                and tensors[n].dtype == torch.bfloat16]
    assert len(stored32) > 8
    for n in stored32:
        t = tensors[n].float()
        tensors[n] = t * (1.0 + 1e-3 * torch.randn(t.shape, generator=g))
    folder = tmp_path / "f32stored"
    os.makedirs(folder)
    with open(folder / "config.json", "w") as fh:
        json.dump(cfg, fh)
    write_safetensors(str(folder / "model.safetensors"), tensors)
    model = Model.load(str(folder), dtype="bfloat16", max_tokens=512)
    assert model.decoder.embedding.dtype == torch.float32
    eng = model.engine
    seqs = [tiny.random_prompt(n, cfg["vocab_size"], seed=n) for n in (40, 9)]
    slots = eng.admit(2)
    got = [eng.step(slots, [s[:-5] for s in seqs], [list(range(len(s) - 5)) for s in seqs]).clone()]
    for k in range(5, 0, -1):
        got.append(eng.step(slots, [[s[-k]] for s in seqs]).clone())
    eng.release(slots)
    for i, s in enumerate(seqs):
        exact, same = _plain(str(folder), s, "bfloat16")
        n = len(s) - 5
        first = got[0][:n] if i == 0 else got[0][len(seqs[0]) - 5:]
        rows = torch.cat([first] + [g_[i:i + 1] for g_ in got[1:]])
        check(rows, exact, "bfloat16", same)
    # the same model with everything rounded to bfloat16 gives other logits: the 32-bit values were used
    rounded = {k: (v.to(torch.bfloat16) if k in stored32 else v) for k, v in tensors.items()}
    cfg_r, t_r = plain_lfm3.load_folder(str(folder))
    exact = plain_lfm3.forward(cfg_r, t_r, seqs[0])
    t_r2 = {k: (rounded[k].double() if k in rounded and rounded[k].is_floating_point() else v) for k, v in t_r.items()}
    assert rel_err(plain_lfm3.forward(cfg_r, t_r2, seqs[0]), exact) > 1e-4


@pytest.mark.parametrize("graphs", [True, False])
def test_the_longest_allowed_sequence(tmp_path, graphs):
    """max_position_embeddings = 100 (no multiple of a page): token 100 is the last one a sequence
    may hold, on the prompt path, the append path and the lean decode path alike."""
    from catena_models_b200.api import Model
    from catena_models_b200.cache.allocators import CacheFull
    from catena_models_b200.weights.random_init import write_random_model

    cfg = dict(tiny.TINY_A, max_position_embeddings=100)
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=1, **tiny.RANDOM_A)
    eng = Model.load(folder, dtype="float32", max_tokens=512, use_graphs=graphs).engine
    (slot,) = eng.admit(1)
    with pytest.raises(CacheFull):
        eng.step([slot], [[1] * 101])
    eng.step([slot], [[1] * 90])
    with pytest.raises(CacheFull):
        eng.step([slot], [[2] * 11])
    eng.step([slot], [[2] * 8])
    eng.step([slot], [[3]])
    eng.step([slot], [[3]])
    assert eng.length(slot) == 100
    with pytest.raises(CacheFull):
        eng.step([slot], [[3]])
    assert eng.length(slot) == 100
    eng.release([slot])
    assert not eng.cache.book.live


def test_decoding_ahead_on_a_cache_too_tight_to_run_ahead(tmp_path):
    """Two sequences stand one token before a page's edge and the cache has one free page: the step
    that would run ahead cannot reserve both pages and is refused (CacheFull), the loop waits for the
    tokens of the step before, one of the sequences ends there on its stop token and gives its page
    back, and the other goes on.  Its tokens are the plain model's."""
    from catena_models_b200.api import Model
    from catena_models_b200.engine.generate import Generation, run_batch
    from catena_models_b200.sampling.sampler import Sampler

    folder = tiny.make_folder(tmp_path, "A", seed=2)
    cfg, tensors = plain_lfm3.load_folder(folder)
    V = cfg["vocab_size"]
    found = None
    for seed in range(200):
        a, b = tiny.random_prompt(62, V, seed=seed), tiny.random_prompt(62, V, seed=1000 + seed)
        ta, tb = plain_lfm3.generate(cfg, tensors, a, 3), plain_lfm3.generate(cfg, tensors, b, 8)
        stop = ta[2]
        if stop not in ta[:2] and stop not in tb:
            found = (a, b, ta, tb, stop)
            break
    assert found
    a, b, ta, tb, stop = found
    model = Model.load(folder, dtype="float32", max_tokens=192)            # three pages in all
    eng = model.engine
    assert eng.overlapped_decode
    refused = []
    real_step = eng.step

    def watching(*args, **kw):
        try:
            return real_step(*args, **kw)
        except Exception as exc:
            refused.append(type(exc).__name__)
            raise

    eng.step = watching
    reqs = [Generation(a), Generation(b)]
    run_batch(eng, Sampler(model.device), reqs, [0, 1], 8, frozenset([stop]), False)
    assert refused == ["CacheFull"]
    assert reqs[0].tokens == ta and reqs[0].finish_reason == "stop"
    assert reqs[1].tokens == tb and reqs[1].finish_reason == "length"
    assert not eng.cache.book.live and eng.cache.book.page_alloc[0].free_count == eng.cache.book.group_pages[0]


def test_dropped_recordings_are_made_again_with_the_same_result(tmp_path, monkeypatch):
    """With room for two recorded decode steps, batches of 3, 2 and 1 sequences and two length
    classes force recordings out; every step's logits equal those of an engine that keeps them all."""
    from catena_models_b200.api import Model
    from catena_models_b200.engine import engine as engine_module

    folder = tiny.make_folder(tmp_path, "B", seed=3)
    V = tiny.TINY_B["vocab_size"]
    seqs = [tiny.random_prompt(n, V, seed=n) for n in (262, 40, 20)]      # the longest crosses 256 while it decodes

    def run(kept):
        monkeypatch.setattr(engine_module, "DECODE_GRAPHS_KEPT", kept)
        eng = Model.load(folder, dtype="bfloat16", max_tokens=1024).engine
        out = []
        for rnd in range(2):
            slots = eng.admit(3)
            eng.step(slots, [s[:-12] for s in seqs])
            live = [0, 1, 2]
            for k in range(12, 0, -1):
                if k == 8:
                    live = [0, 2]
                if k == 4:
                    live = [0]
                out.append(eng.step([slots[i] for i in live], [[seqs[i][-k]] for i in live]).clone())
            eng.release(slots)
            assert len(eng._graphs) <= kept
        return out

    few, many = run(2), run(24)
    assert len(few) == len(many)
    for x, y in zip(few, many):
        assert torch.equal(x, y)


def test_fault_flags_stop_a_step_from_handing_out_its_result(tmp_path):
    """The flags are set by hand (no kernel is made to fail): a sampling step, a step that ran
    ahead, a session's logits and the explicit check all raise, the flags are cleared, and the
    engine works afterwards."""
    from catena_models_b200.api import Model
    from catena_models_b200.engine.engine import Sampling
    from catena_models_b200.engine.runtime import DeviceFault

    folder = tiny.make_folder(tmp_path, "A", seed=4)
    model = Model.load(folder, dtype="bfloat16", max_tokens=512)
    eng, rt = model.engine, model.decoder.rt
    (slot,) = eng.admit(1)
    eng.step([slot], [[1, 2, 3]])
    greedy = lambda step: Sampling([0], [step])
    rt.status[0] = 5
    with pytest.raises(DeviceFault, match="wait ran out"):
        eng.step([slot], [[4]], sampling=greedy(1))
    assert rt.status.tolist() == [0, 0]
    _, toks = eng.step([slot], [[5]], sampling=greedy(2))                  # works again
    rt.status[1] = 1
    _, pending = eng.step([slot], [[toks[0]]], sampling=greedy(3), wait=False)
    with pytest.raises(DeviceFault, match="outside the vocabulary"):
        pending.tokens()
    assert rt.status.tolist() == [0, 0]
    rt.status[0] = 1
    with pytest.raises(DeviceFault):
        eng.check_errors()
    eng.release([slot])
    with model.session(16) as s:
        rt.status[1] = 1
        with pytest.raises(DeviceFault):
            s.prefill_logits([1, 2])
        assert s.decode_logits(3).shape == (tiny.TINY_A["vocab_size"],)


def test_tokens_are_taken_from_the_step_before_only_if_it_sampled(tmp_path):
    from catena_models_b200.api import Model
    from catena_models_b200.engine.engine import Sampling, StepError

    folder = tiny.make_folder(tmp_path, "A", seed=5)
    eng = Model.load(folder, dtype="bfloat16", max_tokens=512).engine
    slots = eng.admit(2)
    eng.step(slots, [[1, 2, 3], [4]])
    samp = lambda step: Sampling([0, 1], [step, step])
    _, toks = eng.step(slots, [[5], [6]], sampling=samp(1))
    _, nxt = eng.step(slots, [[0], [0]], sampling=samp(2), token_from=[0, 1])          # fine: the step before sampled
    assert len(nxt) == 2
    with pytest.raises(StepError):
        eng.step(slots, [[0], [0]], sampling=samp(3), token_from=[0, 2])               # only two were sampled
    eng.step(slots, [[7], [8]])                                                        # a step that samples nothing
    with pytest.raises(StepError):
        eng.step(slots, [[0], [0]], sampling=samp(4), token_from=[0, 1])
    # and the step that sampled nothing ran its sampling kernel on zeroed inputs: a later sampling
    # step is not disturbed by what it left
    logits, toks = eng.step(slots, [[9], [10]], sampling=samp(5))
    assert toks == logits.argmax(-1).tolist()
    eng.release(slots)


@pytest.mark.parametrize("name", ["A", "B", "L"])
def test_decode_through_the_persistent_kernel(tmp_path, name):
    """The opt-in decode path that collects a step's products, residual sums and convolutions into a
    few persistent launches: the same logits as the plain model, replayed from a recording, over
    page borders and a wrapping ring, for one and for several sequences; far fewer launches."""
    from catena_models_b200.api import Model

    folder = tiny.make_folder(tmp_path, name, seed=6)
    cfg = tiny.ALL[name][0]
    seqs = [tiny.random_prompt(n, cfg["vocab_size"], seed=n) for n in (150, 40, 71)]
    launches = {}
    for fused in (False, True):
        model = Model.load(folder, dtype="bfloat16", max_tokens=1024)
        model.decoder.rt.fused_decode = fused
        eng = model.engine
        slots = eng.admit(3)
        got = [eng.step(slots, [s[:-90] if len(s) > 100 else s[:-30] for s in seqs]).clone()]
        heads = [len(s) - 90 if len(s) > 100 else len(s) - 30 for s in seqs]
        from catena_models_b200 import kernels
        before = kernels.launches
        for t in range(30):
            got.append(eng.step(slots, [[s[h + t]] for s, h in zip(seqs, heads)]).clone())
        launches[fused] = kernels.launches - before
        for t in range(30, 90):                                  # the longest sequence alone
            got.append(eng.step(slots[:1], [[seqs[0][heads[0] + t]]]).clone())
        eng.release(slots)
        eng.check_errors()
        for i, (s, h) in enumerate(zip(seqs, heads)):
            exact, same = _plain(folder, s, "bfloat16")
            rows = [g[i:i + 1] for g in got[:31]] + ([g[:1] for g in got[31:]] if i == 0 else [])
            check(torch.cat(rows), exact[h - 1:h - 1 + len(rows)], "bfloat16", same[h - 1:h - 1 + len(rows)])
    assert launches[True] < launches[False] / 2
