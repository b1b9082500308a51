"""bin/trace_run as a user drives it: a subprocess fed JSON lines on standard input.  The same
requests whole, with the last 32 tokens one by one, in unequal batches one after another
(so slots and pages are used again), and with their prompts cut into two steps (the second on
top of what the first left, while another request starts beside it), in 32-bit and in bfloat16,
against the plain model."""
import json
import os
import subprocess

import numpy as np
import pytest
import torch

import plain_lfm3
import tiny

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def replay(folder, dtype, steps, out_dir, max_tokens):
    lines = "".join(json.dumps(s) + "\n" for s in steps)
    run = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out",
                          str(out_dir), "--max-tokens", str(max_tokens)], input=lines, capture_output=True,
                         text=True, timeout=900)
    assert run.returncode == 0, run.stderr[-2000:]
    assert [l for l in run.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    return run


def read(out_dir, step, vocab):
    return torch.from_numpy(np.fromfile(os.path.join(str(out_dir), f"{step}.f32"), dtype="<f4").reshape(-1, vocab).copy())


def rel(got, ref):
    return float((got.double() - ref.double()).abs().max() / ref.double().abs().max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_replay_four_ways(tmp_path, name, dtype):
    folder = tiny.make_folder(tmp_path, name, seed=7)
    cfg, tensors = plain_lfm3.load_folder(folder)
    V = cfg["vocab_size"]
    lens = {"a": 40, "b": 97, "c": 33, "d": 130, "e": 35}
    reqs = {k: tiny.random_prompt(n, V, seed=ord(k)) for k, n in lens.items()}
    steps, expect, way_of = [], {}, {}          # expect[step] = list of (request, positions)
    n = 0
    way = "whole"

    def add(entries, end=()):
        nonlocal n
        steps.append({"step": n, "entries": entries, "end": list(end)})
        wanted = [(e["id"].split(":")[0], e["_pos"]) for e in entries if e["want"]]
        for e in entries:
            del e["_pos"]
        if wanted:
            expect[n] = wanted
            way_of[n] = way
        n += 1

    # 1) each request alone and whole, every position wanted
    for k, toks in reqs.items():
        add([{"id": f"{k}:w", "tokens": toks, "want": list(range(len(toks))), "_pos": list(range(len(toks)))}], end=[f"{k}:w"])
    # 2) the last 32 tokens one by one after a prompt step of the rest
    way = "tail"
    for k, toks in reqs.items():
        head = len(toks) - 32
        add([{"id": f"{k}:t", "tokens": toks[:head], "want": [head - 1], "_pos": [head - 1]}])
        for t in range(head, len(toks)):
            add([{"id": f"{k}:t", "tokens": [toks[t]], "want": [0], "_pos": [t]}], end=[f"{k}:t"] if t == len(toks) - 1 else [])
    # 3) batches of unequal lengths: prompts of different sizes, the shorter requests end earlier;
    #    a step with nothing wanted in between; the next batch starts on the freed slots
    way = "batch"
    for batch, prompt_lens in ((["a", "b", "c"], [8, 60, 1]), (["d", "e", "a"], [100, 3, 39])):
        ids = [f"{k}:b" for k in batch]
        add([{"id": i, "tokens": reqs[k][:p], "want": [0, p - 1] if p > 1 else [0], "_pos": [0, p - 1] if p > 1 else [0]}
             for i, k, p in zip(ids, batch, prompt_lens)])
        pos = dict(zip(batch, prompt_lens))
        live = list(batch)
        quiet = True
        while live:
            entries, ending = [], []
            for k in live:
                want = [] if (quiet and k == live[0]) else [0]
                entries.append({"id": f"{k}:b", "tokens": [reqs[k][pos[k]]], "want": want, "_pos": [pos[k]] if want else []})
                pos[k] += 1
                if pos[k] == len(reqs[k]):
                    ending.append(k)
            quiet = False
            add(entries, end=[f"{k}:b" for k in ending])
            live = [k for k in live if k not in ending]
    # 4) prompts in two chunks: every request brings its second chunk on top of its first, in one batch
    #    with unequal cuts, while a request that has not started yet joins with its whole prompt
    way = "chunks"
    cuts = {"a": 13, "b": 64, "c": 1, "d": 100}
    add([{"id": f"{k}:c", "tokens": reqs[k][:c], "want": [c - 1], "_pos": [c - 1]} for k, c in cuts.items()])
    entries = [{"id": f"{k}:c", "tokens": reqs[k][c:], "want": list(range(len(reqs[k]) - c)),
                "_pos": list(range(c, len(reqs[k])))} for k, c in cuts.items()]
    entries.append({"id": "e:c", "tokens": reqs["e"], "want": list(range(len(reqs["e"]))), "_pos": list(range(len(reqs["e"])))})
    add(entries, end=[f"{k}:c" for k in reqs])
    out = tmp_path / "out"
    # peak: the chunked batch holds 40 + 97 + 33 + 130 + 35 tokens -> 64 + 128 + 64 + 192 + 64 = 512
    replay(folder, dtype, steps, out, max_tokens=512)
    exact = {k: plain_lfm3.forward(cfg, tensors, t) for k, t in reqs.items()}
    same = {k: plain_lfm3.forward(cfg, tensors, t, bf16=True) for k, t in reqs.items()} if dtype == "bfloat16" else None
    assert sorted(int(f[:-4]) for f in os.listdir(out)) == sorted(expect)
    # Gather the rows of each (request, way) over all its steps: the bfloat16 criterion compares
    # the engine's distance from the exact model with the distance of the plain model run with
    # the reference's bfloat16 rounding points, and both are maxima over the same set of rows.
    rows = {}
    for step, wanted in expect.items():
        got = read(out, step, V)
        assert got.shape[0] == sum(len(p) for _, p in wanted)
        off = 0
        for key, positions in wanted:
            rows.setdefault((key, way_of[step]), []).append((got[off:off + len(positions)], positions))
            off += len(positions)
    assert len(rows) == 20                                   # five requests, four ways
    for (k, way), parts in rows.items():
        got = torch.cat([g for g, _ in parts])
        pos = [p for _, ps in parts for p in ps]
        ref = exact[k][pos]
        if dtype == "float32":
            assert rel(got, ref) < 2e-5, (k, way)
        else:
            assert rel(got, ref) < 2.0 * rel(same[k][pos], ref), (k, way)


def test_replay_refuses_what_does_not_fit(tmp_path):
    folder = tiny.make_folder(tmp_path, "A", seed=7)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": [1] * 200, "want": [199]}], "end": []}]
    lines = "".join(json.dumps(s) + "\n" for s in steps)
    run = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out",
                          str(tmp_path / "o"), "--max-tokens", "128"], input=lines, capture_output=True, text=True,
                         timeout=600)
    assert run.returncode != 0 and "page" in run.stderr
