"""Generation through the Python entry point and the command line, against the plain
implementation: greedy, temperature, stop tokens, early finishers, batch after batch."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_lfm3
import tiny

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("gen")
    return {n: tiny.make_folder(tmp, n, seed=10 + i) for i, n in enumerate(("A", "B"))}


def test_greedy_float32_equals_plain_tokens(folders):
    """The first tiny model on its named workload: prompts of 5, 11 and 17 tokens, 8 greedy steps."""
    from catena_models_b200.api import Model

    cfg, tensors = plain_lfm3.load_folder(folders["A"])
    model = Model.load(folders["A"], dtype="float32", max_tokens=1024)
    prompts = [tiny.random_prompt(n, cfg["vocab_size"], seed=n) for n in (5, 11, 17)]
    out = model.generate(prompts, max_new_tokens=8, ignore_eos=True)
    for p, g in zip(prompts, out):
        assert g.tokens == plain_lfm3.generate(cfg, tensors, p, 8) and g.finish_reason == "length"
    assert not model.engine.cache.book.live


def test_greedy_bfloat16_follows_the_exact_model(folders):
    """Along the engine's own trajectory, every chosen token is (within the format's noise) a
    maximum of the exact model's logits."""
    from catena_models_b200.api import Model

    cfg, tensors = plain_lfm3.load_folder(folders["B"])
    model = Model.load(folders["B"], dtype="bfloat16", max_tokens=2048)
    prompts = [tiny.random_prompt(n, cfg["vocab_size"], seed=n) for n in (1, 7, 20, 33)]
    out = model.generate(prompts, max_new_tokens=12, ignore_eos=True)
    for p, g in zip(prompts, out):
        assert len(g.tokens) == 12
        seq = p + g.tokens
        exact = plain_lfm3.forward(cfg, tensors, seq)
        noise = float((plain_lfm3.forward(cfg, tensors, seq, bf16=True) - exact).abs().max())
        for i, tok in enumerate(g.tokens):
            row = exact[len(p) - 1 + i]
            assert float(row[tok]) >= float(row.max()) - 4 * noise


def test_temperature_sampling_is_reproducible_and_independent_of_batch_mates(folders):
    """Second tiny model, prompts 1/7/20/33, 12 steps at temperature 0.8 with a fixed seed."""
    from catena_models_b200.api import Model

    cfg, tensors = plain_lfm3.load_folder(folders["B"])
    model = Model.load(folders["B"], dtype="float32", max_tokens=2048)
    prompts = [tiny.random_prompt(n, cfg["vocab_size"], seed=n) for n in (1, 7, 20, 33)]
    a = model.generate(prompts, max_new_tokens=12, temperature=0.8, seed=42, ignore_eos=True)
    b = model.generate(prompts, max_new_tokens=12, temperature=0.8, seed=42, ignore_eos=True)
    c = model.generate(prompts, max_new_tokens=12, temperature=0.8, seed=43, ignore_eos=True)
    assert [g.tokens for g in a] == [g.tokens for g in b] != [g.tokens for g in c]
    # a sequence's draws are keyed by its own id: batches of one give the same tokens
    solo = model.generate(prompts, max_new_tokens=12, temperature=0.8, seed=42, ignore_eos=True, max_batch=1)
    assert [g.tokens for g in solo] == [g.tokens for g in a]
    # every drawn token holds its uniform in the exact model's distribution (teacher-forced)
    for sid, (p, g) in enumerate(zip(prompts, a)):
        logits = plain_lfm3.forward(cfg, tensors, p + g.tokens)
        for step, tok in enumerate(g.tokens):
            x = logits[len(p) - 1 + step] / 0.8
            cdf = torch.cumsum(torch.exp(x - x.max()), 0)
            target = plain_lfm3.uniform_draw(42, sid, step) * float(cdf[-1])
            lo = float(cdf[tok - 1]) if tok > 0 else 0.0
            slack = 1e-4 * float(cdf[-1])
            assert lo - slack <= target <= float(cdf[tok]) + slack


def test_stop_tokens_early_finishers_and_slot_reuse(folders):
    from catena_models_b200.api import Model

    cfg, tensors = plain_lfm3.load_folder(folders["A"])
    model = Model.load(folders["A"], dtype="float32", max_tokens=640)       # ten pages: batches must queue
    prompts = [tiny.random_prompt(n, cfg["vocab_size"], seed=50 + n) for n in (9, 30, 3, 70, 15, 2, 41)]
    free = [plain_lfm3.generate(cfg, tensors, p, 10) for p in prompts]
    stops = {free[0][3], free[3][0], free[5][9]}
    out = model.generate(prompts, max_new_tokens=10, stop_token_ids=sorted(stops), max_batch=3)
    for p, g in zip(prompts, out):
        ref = plain_lfm3.generate(cfg, tensors, p, 10, stop_token_ids=stops)
        assert g.tokens == ref
        assert g.finish_reason == ("stop" if ref[-1] in stops else "length")
    assert len(out[3].tokens) == 1 and not model.engine.cache.book.live
    # eos from config.json is the default stop set; --ignore-eos goes through it
    eos = cfg["eos_token_id"]
    forced = [g.tokens for g in model.generate(prompts[:2], max_new_tokens=6, ignore_eos=True)]
    assert all(len(t) == 6 for t in forced)
    default = model.generate(prompts[:2], max_new_tokens=6)
    for t, g in zip(forced, default):
        assert g.tokens == (t[:t.index(eos) + 1] if eos in t else t)


def test_session_api(folders):
    from catena_models_b200.api import Model

    cfg, tensors = plain_lfm3.load_folder(folders["A"])
    model = Model.load(folders["A"], dtype="float32", max_tokens=512)
    prompt = tiny.random_prompt(12, cfg["vocab_size"], seed=3)
    ref = plain_lfm3.generate(cfg, tensors, prompt, 5)
    with model.session(capacity=64) as s:
        tok = s.prefill_next_token(prompt)
        got = [tok]
        for _ in range(4):
            tok = s.decode_next_token(tok)
            got.append(tok)
        assert s.position == 16 and got == ref
        with pytest.raises(ValueError):
            s._run([1] * 100)
    assert model.next_token(prompt) == ref[0]
    exact = plain_lfm3.forward(cfg, tensors, prompt)[-1]
    assert float((model.logits(prompt).double() - exact).abs().max()) < 1e-4
    assert not model.engine.cache.book.live


def test_checkpoint_resume_and_append(folders):
    """A session is set aside as a checkpoint after 70 tokens (more than a page, the sliding ring
    of 8 wrapped many times, conv state in use); two sessions resumed from it go different ways and
    each must give the logits of its whole sequence, as must the append calls; closing everything
    gives every page and slot back."""
    from catena_models_b200.api import Model

    cfg, tensors = plain_lfm3.load_folder(folders["B"])
    model = Model.load(folders["B"], dtype="float32", max_tokens=1024)
    book = model.engine.cache.book
    free_pages = [a.free_count for a in book.page_alloc]
    base = tiny.random_prompt(70, cfg["vocab_size"], seed=5)
    tails = [tiny.random_prompt(6, cfg["vocab_size"], seed=6), tiny.random_prompt(4, cfg["vocab_size"], seed=7)]

    s = model.session(capacity=128)
    s.prefill_logits(base[:60])
    got = s.append_logits(base[60:])                           # ten tokens on top of a started sequence
    exact = plain_lfm3.forward(cfg, tensors, base)
    assert float((got.double() - exact[-1]).abs().max()) < 1e-4
    ckpt = s.into_checkpoint()
    assert s.slot is None and ckpt.position == 70
    with pytest.raises(ValueError):
        s.into_checkpoint()

    sessions = [model.resume_checkpoint(ckpt), model.resume_checkpoint(ckpt)]
    assert len({x.slot for x in sessions} | {ckpt.slot}) == 3 and all(x.position == 70 for x in sessions)
    outs = [[], []]
    for step in range(6):                                       # the two go on in turns, not in one batch
        for i, (x, tail) in enumerate(zip(sessions, tails)):
            if step < len(tail):
                outs[i].append(x.decode_logits(tail[step]))
    for i, tail in enumerate(tails):
        ref = plain_lfm3.forward(cfg, tensors, base + tail)[70:]
        assert float((torch.stack(outs[i]).double() - ref).abs().max()) < 1e-4
    # the checkpoint is still what it was: a third session from it gives the first tail's logits again
    third = model.resume_checkpoint(ckpt)
    tok = third.append_next_token(tails[0][:2])
    assert tok == int(plain_lfm3.argmax_first(plain_lfm3.forward(cfg, tensors, base + tails[0][:2])[-1]))

    other = Model.load(folders["B"], dtype="float32", max_tokens=256)
    with pytest.raises(ValueError, match="another model"):
        other.resume_checkpoint(ckpt)
    for x in sessions + [third]:
        x.close()
    ckpt.close()
    with pytest.raises(ValueError, match="closed"):
        model.resume_checkpoint(ckpt)
    assert not book.live and [a.free_count for a in book.page_alloc] == free_pages


def test_command_line(folders, tmp_path):
    cfg, tensors = plain_lfm3.load_folder(folders["A"])
    p1, p2 = tiny.random_prompt(6, cfg["vocab_size"], 1), tiny.random_prompt(13, cfg["vocab_size"], 2)
    cmd = [sys.executable, "-m", "catena_models_b200", "--model", folders["A"], "--dtype", "float32", "-n", "5",
           "--ignore-eos", "--prompt", " ".join(map(str, p1)), "--prompt", ",".join(map(str, p2))]
    run = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr
    lines = [list(map(int, l.split())) for l in run.stdout.strip().splitlines()]
    assert lines == [plain_lfm3.generate(cfg, tensors, p1, 5), plain_lfm3.generate(cfg, tensors, p2, 5)]
    assert "prompt eval: 19 token(s)" in run.stderr and "cached eval: 8 token(s)" in run.stderr
    conf = tmp_path / "c.json"
    conf.write_text(json.dumps(tiny.TINY_B))
    bench = subprocess.run([sys.executable, "-m", "catena_models_b200", "--random", str(conf), "--bench", "--pp", "40",
                            "--tg", "6", "--tg-context", "9", "--batch", "2"], cwd=ROOT, capture_output=True,
                           text=True, timeout=600)
    assert bench.returncode == 0, bench.stderr
    assert "pp40x2" in bench.stdout and "tg6/ctx9x2" in bench.stdout


def test_command_line_options_of_the_reference_and_this_library(folders, tmp_path):
    """--prompt-lens (synthetic prompts), --max-slots, --kernels, --no-wmma-prefill (CUDA-core prompt
    steps under the bfloat16 engine: the same tokens as with tensor cores on a model this small, and
    the plain model's in 32-bit), --pp-chunk in the bench."""
    cfg, tensors = plain_lfm3.load_folder(folders["A"])
    base = [sys.executable, "-m", "catena_models_b200", "--model", folders["A"], "-n", "4", "--ignore-eos",
            "--prompt-lens", "7 19", "--max-slots", "2"]
    outs = {}
    for name, extra in (("f32", ["--dtype", "float32", "--kernels", "fused"]), ("f32-simt", ["--dtype", "float32", "--no-wmma-prefill"]),
                        ("bf16", []), ("bf16-simt", ["--no-wmma-prefill"])):
        run = subprocess.run(base + extra, cwd=ROOT, capture_output=True, text=True, timeout=600)
        assert run.returncode == 0, run.stderr
        outs[name] = [list(map(int, l.split())) for l in run.stdout.strip().splitlines()]
        assert "cache of" in run.stderr and [len(o) for o in outs[name]] == [4, 4]
    from catena_models_b200.cli import _synthetic
    ids = _synthetic(26, cfg["vocab_size"])
    assert outs["f32"] == outs["f32-simt"] == [plain_lfm3.generate(cfg, tensors, ids[:7], 4),
                                                 plain_lfm3.generate(cfg, tensors, ids[7:], 4)]
    refused = subprocess.run(base + ["--kernels", "reference"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert refused.returncode != 0 and "fused" in refused.stderr
    conf = tmp_path / "c.json"
    conf.write_text(json.dumps(tiny.TINY_B))
    bench = subprocess.run([sys.executable, "-m", "catena_models_b200", "--random", str(conf), "--bench", "--pp", "100",
                            "--pp-chunk", "30", "--tg", "0"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert bench.returncode == 0 and "pp100/30" in bench.stdout, bench.stderr
