#!/usr/bin/env python3
"""Decode and prefill throughput of LFM3-class models with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--config 1.7b|350m|2.6b] [--batch B]
                    [--layers L] [--impl reference] [--kernel-table] [--attention-table]

A step is one decode step of the whole batch.  Prints one JSON line: decoded tokens per second
on the device (`value`), the same through the Python entry point with host tokens in and out
(`e2e`), the prompt step of the configuration's workload (`prefill`), the decode step's memory
roofline, and further decode points (`points`, with their fractions of the copy bandwidth in
`points_frac`).  Before the line is printed, logits of the timed run are compared with the
32-bit engine on the same tokens; a mismatch ends the run with exit code 3 and no line.

`--config` names the workload: `1.7b` (the default, the headline: batch 8, a 2,048-token prompt,
decode towards a context of 4,096; decode points at batch 1, 8 and 64 at three contexts each),
`350m` (64 prompts of 16 to 2,048 tokens in one start step, then decode) and `2.6b` (a
16,384-token prompt alone, then decode of 64 sequences on a cache sized for 64 x 32,768 tokens).
`--kernel-table` runs one decode step and one prompt step kernel by kernel with a pair of CUDA
events around each launch and prints what each kernel took against its roofline, instead of the
JSON line.  `--attention-table` times the prompt-attention kernels alone (the configuration's heads, one
sequence of 2,048, 4,096 and 16,384 tokens, launches back to back in a recorded graph).  This engine runs on one GPU; for --gpus above 1 it says so and exits with 2.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def _pattern_17b(layers):
    """Two conv layers, then an attention layer, alternately full and sliding.  The pattern is this
    bench's choice; the reference fixes only that its 24-layer model has conv, full and sliding
    layers (tests/lfm3.rs:39-42)."""
    types, attn = [], 0
    for l in range(layers):
        if l % 3 == 2:
            types.append("full_attention" if attn % 2 == 0 else "sliding_attention")
            attn += 1
        else:
            types.append("conv")
    return types


def _pattern_350m(layers):
    return ["full_attention" if l in (2, 5, 8, 10, 12, 14) else "conv" for l in range(layers)]


def _pattern_26b(layers):
    """22 conv and 8 attention layers of 30, the attention layers alternately full and sliding."""
    at = (2, 6, 10, 14, 18, 22, 26, 29)
    types, attn = [], 0
    for l in range(layers):
        if l in at:
            types.append("full_attention" if attn % 2 == 0 else "sliding_attention")
            attn += 1
        else:
            types.append("conv")
    return types


# name -> sizes of the model and of its workload
CONFIGS = {
    "1.7b": dict(model="LFM3-1.7B-class", layers=24, pattern=_pattern_17b, hidden=2048, heads=32, kv_heads=8,
                 head_dim=64, ffn=8192, context=4096, batch=8, prompt_len=2048, prefill_tokens=2048),
    "350m": dict(model="LFM3-350M-class", layers=16, pattern=_pattern_350m, hidden=1024, heads=16, kv_heads=8,
                 head_dim=64, ffn=4608, context=32768, batch=64, prompt_len=None, prefill_tokens=None),
    "2.6b": dict(model="LFM3-2.6B-class", layers=30, pattern=_pattern_26b, hidden=2048, heads=32, kv_heads=8,
                 head_dim=64, ffn=10752, context=32768, batch=64, prompt_len=2048, prefill_tokens=16384),
}
VOCAB = 65536
POINT_CONTEXTS = (2048, 3072, 4016)       # prompt lengths of the headline's further decode points (context 4,096)
# After prompt steps the board's power average is high and the SM clock stays reduced for some tens of
# milliseconds: measured on B200, the first 25 to 40 decode steps after a 2,048-token prompt per sequence
# ran 12 to 18 % slower (batch 8: 1.34 against 1.14 ms, batch 64: 2.17 against 1.83 ms) and a pause of
# 0.1 s before them removed the effect.  Decode is timed in its steady state, so every run pauses here
# between its prompts and its warm-up steps.
SETTLE_SECONDS = 0.2


def model_config(name, layers=None):
    c = CONFIGS[name]
    layers = layers or c["layers"]
    return dict(architecture="lfm3", vocab_size=VOCAB, hidden_size=c["hidden"], intermediate_size=c["ffn"],
                num_hidden_layers=layers, layer_types=c["pattern"](layers), num_attention_heads=c["heads"],
                num_key_value_heads=c["kv_heads"], head_dim=c["head_dim"], conv_L_cache=3, sliding_window=4096,
                rope_theta=1000000.0, norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=c["context"])


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
    if os.path.exists(path):
        try:
            with open(path) as fh:
                data = json.load(fh)
            for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                if isinstance(data.get(k), (int, float)):
                    out[k] = float(data[k])
            out["source"] = "measured"
        except (OSError, ValueError):
            pass
    return out


def _graph_time_us(torch, fn, launches=10, replays=5):
    """Median time of one call of fn, in microseconds, over `replays` replays of a recorded graph of
    `launches` calls back to back (CUDA events around each replay; three calls first)."""
    for _ in range(3):
        fn()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(launches):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(replays):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) / launches * 1e3)
    return statistics.median(times)


def attention_table(cfg, pk, device="cuda:0", lengths=(2048, 4096, 16384), time_us=None):
    """The two tensor-core prompt-attention kernels alone, for the configuration's heads: one sequence of each
    length with a full causal mask, random bfloat16 q, k and v as column blocks of one buffer (as the q/k/v
    product leaves them), no gate.  FLOPs are counted over the causal half: 4 * heads * head size * T (T + 1) / 2."""
    import torch

    from catena_models_b200 import kernels as K

    time_us = time_us or (lambda fn: _graph_time_us(torch, fn))
    QH, KVH, HD = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    print(f"\n### prompt attention alone, {QH} query heads over {KVH} kv heads of {HD}, bfloat16, causal\n")
    print(f"| tokens | tcgen05 us | TFLOP/s | of peak ({pk['bf16_tflops']:.0f}) | mma.sync us | TFLOP/s |")
    print("|---|---|---|---|---|---|")
    err = torch.zeros(1, dtype=torch.int32, device=device)
    for T in lengths:
        width = QH * HD + 2 * KVH * HD
        buf = torch.randn(T, width, device=device).to(torch.bfloat16)
        q, k, v = buf[:, :QH * HD], buf[:, QH * HD:QH * HD + KVH * HD], buf[:, QH * HD + KVH * HD:]
        starts = torch.tensor([0, T], dtype=torch.int32, device=device)
        ctx = torch.empty(T, QH * HD, dtype=torch.bfloat16, device=device)
        scale = HD ** -0.5
        flops = 4.0 * QH * HD * T * (T + 1) / 2
        cells = []
        if HD in (64, 128):
            t = time_us(lambda: K.attn_prefill_tc(ctx, q, k, v, None, starts, 1, T, QH, KVH, HD, 0, scale, err=err))
            if int(err.item()) != 0:
                raise RuntimeError(f"attn_prefill_tc raised its error flag ({int(err.item())})")
            cells += [f"{t:.1f}", f"{flops / t / 1e6:.0f}", f"{flops / t / 1e6 / pk['bf16_tflops']:.3f}"]
        else:
            cells += ["", "", ""]
        t = time_us(lambda: K.attn_prefill_mma(ctx, q, k, v, None, starts, 1, T, QH, KVH, HD, 0, scale))
        cells += [f"{t:.1f}", f"{flops / t / 1e6:.0f}"]
        print(f"| {T:,} | " + " | ".join(cells) + " |", flush=True)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()
        # nvidia-smi's start-up (driver library initialisation, first query) stalls the GPU for tens of
        # milliseconds: a 53 ms prompt step that met it took 118 ms.  Wait until the first sample has
        # come, so that the timed work only meets the periodic queries.
        deadline = time.time() + 5.0
        while not self.rows and time.time() < deadline:
            time.sleep(0.02)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [int(r[0]) for r in self.rows if len(r) >= 6 and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) >= 6 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower() == "active"})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def synthetic_tokens(count, vocab, state=0x9E3779B97F4A7C15):
    """Uniform ids from the 64-bit LCG the reference's own bench uses (src/main.rs:447-457)."""
    out = []
    for _ in range(count):
        state = (state * 6364136223846793005 + 1442695040888963407) & ((1 << 64) - 1)
        out.append(state % vocab)
    return out, state


def workload_prompts(name, batch, prompt_len, vocab):
    """The prompts of a configuration's decode run: equal lengths, or (350m) lengths uniform in
    [16, 2048] from the same generator."""
    state = 0x9E3779B97F4A7C15
    prompts = []
    for _ in range(batch):
        n = prompt_len
        if n is None:
            (r,), state = synthetic_tokens(1, 2048 - 16 + 1, state)
            n = 16 + r
        toks, state = synthetic_tokens(n, vocab, state)
        prompts.append(toks)
    return prompts, state


def decode_run(model, prompts, steps, warmup, vocab, state, together=False, time_prompt=False):
    """Prefill the prompts (one sequence per step, or all in one start step), run `warmup` untimed
    and `steps` timed decode steps with given (synthetic) tokens and the greedy choice computed on
    the device.  Returns facts of the run, among them the last step's logits of the first and the
    last sequence with the tokens that led to them."""
    import torch

    from catena_models_b200 import kernels

    eng = model.engine
    batch = len(prompts)
    slots = eng.admit(batch)
    prompt_ms = None
    if together:
        # once untimed (the first run of a shape loads kernels and sets their attributes), then timed
        eng.step(slots, prompts, [[] for _ in prompts])
        eng.release(slots)
        slots = eng.admit(batch)
        torch.cuda.synchronize()
        time.sleep(SETTLE_SECONDS)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.step(slots, prompts, [[] for _ in prompts])
        b.record()
        torch.cuda.synchronize()
        prompt_ms = a.elapsed_time(b)
    else:
        for s, p in zip(slots, prompts):                  # one sequence per step keeps the step's memory small
            eng.step([s], [p], [[]])
    torch.cuda.synchronize()
    time.sleep(SETTLE_SECONDS)
    feed, state = synthetic_tokens((warmup + steps) * batch, vocab, state)
    feed = [feed[i * batch:(i + 1) * batch] for i in range(warmup + steps)]
    # a decode step's graph ends with the sampling kernel (greedy here), so the choice of the
    # next token is part of the timed work although the synthetic ids are what is fed
    for i in range(warmup):
        eng.step(slots, [[t] for t in feed[i]])
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = kernels.launches
    mid_bytes = None
    logits = None
    start.record()
    for i in range(warmup, warmup + steps):
        logits = eng.step(slots, [[t] for t in feed[i]])
        if i == warmup + steps // 2:
            mid_bytes = eng.cache.live_bytes()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop)
    launches = kernels.launches - launches0
    eng.check_errors()
    rows = {}
    for b in sorted({0, batch - 1}):
        rows[b] = (prompts[b] + [f[b] for f in feed], logits[b].clone())
    # the timed steps' contexts: from the shortest sequence at the first one to the longest at the last
    first, last = min(len(p) for p in prompts) + warmup, max(len(p) for p in prompts) + warmup + steps
    eng.release(slots)
    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "launches": launches,
            "cache_bytes": mid_bytes, "rows": rows, "context_first": first, "context_last": last,
            "prompt_ms": prompt_ms, "prompt_tokens": sum(len(p) for p in prompts)}


def e2e_run(model, prompts, steps, warmup):
    """The same decode through Model.generate: per step the host sends that step's inputs from
    pinned memory (positions, slots, page-table updates, sampler keys; the token ids themselves are
    taken on the device from the step before, which chose them) and reads the chosen tokens back.
    The loop keeps the device one step ahead of its own bookkeeping."""
    import torch

    batch = len(prompts)
    marks = {}

    def on_step(step, live):
        if step == 0:                                  # the prompts are done: let the clocks settle (SETTLE_SECONDS)
            torch.cuda.synchronize()
            time.sleep(SETTLE_SECONDS)
        if step == warmup:
            torch.cuda.synchronize()
            marks["t0"] = time.perf_counter()
        if step == warmup + steps:
            torch.cuda.synchronize()
            marks["t1"] = time.perf_counter()

    # Two tokens more than the marks need: with the device a step ahead, the step after each marked
    # one is in flight when its mark synchronises, so both marks see the same amount of extra work
    # and the interval holds exactly `steps` steps.
    out = model.generate(prompts, max_new_tokens=warmup + steps + 2, temperature=0.0, ignore_eos=True,
                         stop_token_ids=(), max_batch=batch, on_step=on_step)
    sec = marks["t1"] - marks["t0"]
    eng = model.engine
    layout_bytes = max((g.layout.size * 4 for key, g in eng._graphs.items() if key[0] == batch), default=0)
    return {"value": batch * steps / sec, "unit": "tok/s", "h2d_bytes_per_step": layout_bytes,
            "d2h_bytes_per_step": (batch + 2) * 4}, out


def prompt_flops(cfg, lengths, wanted_rows):
    """Floating-point operations of a prompt step over sequences of the given lengths: every matrix
    product, and the attention over the keys each query sees."""
    H, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    QS = cfg["num_attention_heads"] * cfg["head_dim"]
    KVS = cfg["num_key_value_heads"] * cfg["head_dim"]
    T = sum(lengths)
    flops = 0.0
    for kind in cfg["layer_types"]:
        if kind == "conv":
            flops += 2.0 * T * (3 * H * H + H * H)
        else:
            flops += 2.0 * T * ((QS + 2 * KVS + cfg["num_attention_heads"]) * H + QS * H)
            for n in lengths:
                W = cfg["sliding_window"] if kind == "sliding_attention" else n
                full = min(n, W)
                keys = full * (full + 1) // 2 + (n - full) * W
                flops += 4.0 * QS * keys
        flops += 2.0 * T * 3 * F * H
    flops += 2.0 * wanted_rows * V * H
    return flops


def prefill_run(model, lengths, vocab, cfg, peak_tflops, repeats=3, chunk=0):
    """One prompt step over sequences of the given lengths; with `chunk`, steps of that many tokens a
    sequence, each on top of the ones before (append steps, which read the older keys from the cache)."""
    import torch

    eng = model.engine
    prompts = []
    state = 0x9E3779B97F4A7C15
    for n in lengths:
        toks, state = synthetic_tokens(n, vocab, state)
        prompts.append(toks)
    times = []
    for i in range(repeats + 1):
        slots = eng.admit(len(prompts))
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        if chunk > 0:
            for at in range(0, max(lengths), chunk):
                part = [(s, p[at:at + chunk]) for s, p in zip(slots, prompts) if at < len(p)]
                eng.step([s for s, _ in part], [p for _, p in part])
        else:
            eng.step(slots, prompts)
        b.record()
        torch.cuda.synchronize()
        eng.release(slots)
        if i >= 1:
            times.append(a.elapsed_time(b))
    eng.check_errors()
    ms = statistics.median(times)
    T = sum(lengths)
    flops = prompt_flops(cfg, lengths, len(lengths))
    return {"value": T / (ms / 1e3), "tokens": T, "ms": ms, "frac": flops / (ms / 1e3) / (peak_tflops * 1e12),
            "flops": flops}


class Verifier:
    """The 32-bit engine on the same random weights: says whether logits that a timed run produced
    are those of the model.  The distance allowed is what bfloat16 storage costs on these models
    (0.02 to 0.06 of the largest logit), with margin; a wrong row, slot or kernel is off by order 1."""

    LIMIT = 0.12

    def __init__(self, cfg, max_len):
        from catena_models_b200.api import Model

        self.model = Model.random(cfg, seed=0, std=0.02, dtype="float32", device="cuda:0",
                                  max_tokens=(max_len + 63) // 64 * 64, max_seqs=1)

    def check(self, what, tokens, got):
        ref = self.model.logits(tokens).double()
        got = got.double().cpu()
        err = float((got - ref).abs().max() / ref.abs().max())
        top = int(got.argmax())
        slack = float(ref.max() - ref[top]) / float(ref.abs().max())
        ok = err < self.LIMIT and slack <= 2 * err
        print(f"[bench] check {what}: {len(tokens)} tokens, distance from the 32-bit engine {err:.4f} of the largest "
              f"logit, chosen token {'equal' if slack == 0 else f'{slack:.4f} below the 32-bit maximum'}: "
              f"{'ok' if ok else 'WRONG'}", file=sys.stderr, flush=True)
        return ok, err


def kernel_table(model, cfg, pk, batch, context, prompt_lengths, graph_ms):
    """One decode step of `batch` sequences at `context` tokens and one prompt step, launched kernel
    by kernel with an event pair around every call; the calls added up by kernel and operand shape."""
    import torch

    from catena_models_b200 import kernels
    from catena_models_b200.engine.engine import Engine

    vocab = cfg["vocab_size"]
    tokens_held = max(batch * (context + 64), sum(prompt_lengths) + 64 * len(prompt_lengths))
    eng = Engine(model.decoder, tokens_held, max(batch, len(prompt_lengths)), use_graphs=False)
    KVH, HD, QS = cfg["num_key_value_heads"], cfg["head_dim"], cfg["num_attention_heads"] * cfg["head_dim"]
    window = cfg["sliding_window"]
    out = {}

    def attention_costs(rows, lengths, decode):
        for r in rows:
            if not r["name"].startswith("attn_"):
                continue
            w = int(r["shape"].split("window ")[1].split(",")[0])
            if decode:
                seen = [min(n, w) if w else n for n in lengths]
                r["bytes"] = r["calls"] * sum(seen) * 2 * KVH * HD * 2
                r["flops"] = r["calls"] * sum(seen) * 4 * QS
            else:
                keys = 0
                for n in lengths:
                    full = min(n, w) if w else n
                    keys += full * (full + 1) // 2 + (n - full) * (w or 0)
                r["flops"] = r["calls"] * 4 * QS * keys
                r["bytes"] = r["calls"] * sum(lengths) * (2 * QS + 2 * KVH * HD) * 2

    # ---- decode: the calls are timed inside the recorded step (events that a captured graph may hold),
    # so that every kernel follows its predecessor as in production; the event nodes between the kernels
    # make this replay a little slower than the step without them, which is timed too
    geng = Engine(model.decoder, batch * (context + 64), batch, use_graphs=True)
    slots = geng.admit(batch)
    state = 0x9E3779B97F4A7C15
    for s in slots:
        toks, state = synthetic_tokens(context, vocab, state)
        geng.step([s], [toks], [[]])
    feed, state = synthetic_tokens(8 * batch, vocab, state)
    step = lambda i: geng.step(slots, [[t] for t in feed[i * batch:(i + 1) * batch]])
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with kernels.Timeline(in_graph=True) as tl:
        step(0)                                            # runs kernel by kernel, then records: both are collected
    tl.keep_last(len(tl.calls) // 2)                       # the recording's events
    for i in range(1, 4):
        step(i)
    torch.cuda.synchronize()
    a.record()
    step(4)
    b.record()
    torch.cuda.synchronize()
    rows = tl.rows()
    attention_costs(rows, [context + 5] * batch, True)
    out["decode"] = (rows, a.elapsed_time(b) * 1e3, f"decode step, {batch} sequences at {context} tokens, replayed from its "
                     f"recording with an event pair around every kernel")
    geng.release(slots)
    del geng
    # ---- prompt
    prompts = []
    for n in prompt_lengths:
        toks, state = synthetic_tokens(n, vocab, state)
        prompts.append(toks)
    for rep in range(3):
        slots = eng.admit(len(prompts))
        torch.cuda.synchronize()
        time.sleep(SETTLE_SECONDS)
        with kernels.Timeline() as tl:
            a.record()
            eng.step(slots, prompts)
            b.record()
        eng.release(slots)
    rows = tl.rows()
    attention_costs(rows, prompt_lengths, False)
    out["prompt"] = (rows, a.elapsed_time(b) * 1e3, f"prompt step, {len(prompts)} sequence(s), {sum(prompt_lengths)} tokens")
    eng.check_errors()

    for key in ("decode", "prompt"):
        rows, step_us, title = out[key]
        total = sum(r["us"] for r in rows)
        print(f"\n### {title}\n")
        print(f"the step takes {step_us:.0f} us on the stream; the kernels' own times add up to "
              f"{total:.0f} us ({total / step_us:.2f} of it; the rest lies between the kernels).  Peaks "
              f"({pk['source']}): {pk['hbm_gbs']:.0f} GB/s, {pk['bf16_tflops']:.0f} TFLOP/s.\n")
        print("| kernel | operands | calls | us | share | GB/s | of peak | TFLOP/s | of peak |")
        print("|---|---|---|---|---|---|---|---|---|")
        for r in sorted(rows, key=lambda r: -r["us"]):
            sec = r["us"] * 1e-6
            gbs = r["bytes"] / sec / 1e9 if r["bytes"] else 0.0
            tf = r["flops"] / sec / 1e12 if r["flops"] else 0.0
            print(f"| {r['name']} | {r['shape']} | {r['calls']} | {r['us']:.1f} | {r['us'] / total:.3f} | "
                  f"{gbs:.0f} | {gbs / pk['hbm_gbs']:.2f} | {tf:.1f} | {tf / pk['bf16_tflops']:.3f} |")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--config", default="1.7b", choices=sorted(CONFIGS))
    ap.add_argument("--batch", type=int, default=None, help="sequences of the decode run (default: the configuration's)")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has")
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the further decode points")
    ap.add_argument("--no-check", action="store_true", help="skip the comparison with the 32-bit engine")
    ap.add_argument("--prefill-tokens", type=int, default=None, help="prompt length of `--only prefill`")
    ap.add_argument("--prefill-chunk", type=int, default=0,
                    help="with `--only prefill`: run the prompt in steps of this many tokens (append steps)")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="run one part only (small captures under a profiler); prints that part's facts")
    ap.add_argument("--kernel-table", action="store_true",
                    help="time one decode step and one prompt step kernel by kernel and print the table")
    ap.add_argument("--attention-table", action="store_true",
                    help="time the prompt-attention kernels alone at 2,048, 4,096 and 16,384 tokens and print the table")
    ap.add_argument("--print-config", action="store_true",
                    help="print the configuration's config.json (for `python -m catena_models_b200 --random FILE`) and exit")
    args = ap.parse_args()

    if args.print_config:
        print(json.dumps(model_config(args.config, args.layers), indent=1))
        return 0
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "catena-models is a Rust crate whose kernel compiler is a network git dependency; "
                          "no Rust toolchain, no network and no GGUF checkpoint here, and pip finds no Python project in it"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": "this engine runs on one GPU; --gpus %d is not supported" % args.gpus,
                          "n_gpus": args.gpus}))
        return 2
    args.warmup = max(3, args.warmup)
    c = CONFIGS[args.config]
    batch = args.batch or c["batch"]
    prompt_len = args.prompt_len or c["prompt_len"]
    longest_prompt = prompt_len or 2048
    context = c["context"]
    if longest_prompt + args.warmup + args.steps + 3 > context:
        args.steps = context - longest_prompt - args.warmup - 3

    import torch

    from catena_models_b200.api import Model

    pk = peaks()
    cfg = model_config(args.config, args.layers)
    if args.attention_table:
        attention_table(cfg, pk)
        return 0
    vocab = cfg["vocab_size"]
    headline = args.config == "1.7b"
    point_batches = (1, 8, 64) if headline and not args.no_points and args.only == "all" and not args.kernel_table else ()
    # the cache: what the configuration names (64 sequences of the full context for the two large-context
    # workloads), never less than the runs below hold
    if headline:
        seqs = max((batch,) + tuple(point_batches))
        max_tokens = seqs * context
    else:
        seqs = max(batch, 64)
        max_tokens = seqs * context
    model = Model.random(cfg, seed=0, std=0.02, dtype="bfloat16", device="cuda:0", max_tokens=max_tokens, max_seqs=seqs)
    weight_bytes = model.decoder.weight_bytes_per_step()
    params = model.parameter_count()
    prompts, state = workload_prompts(args.config, batch, prompt_len, vocab)
    together = c["prompt_len"] is None and args.prompt_len is None         # the 350m workload starts all prompts in one step
    prefill_lengths = [len(p) for p in prompts] if together else [args.prefill_tokens or c["prefill_tokens"]]

    if args.kernel_table:
        kernel_table(model, cfg, pk, batch, longest_prompt, prefill_lengths, None)
        return 0
    if args.only == "decode":
        run = decode_run(model, prompts, args.steps, args.warmup, vocab, state, together)
        print(json.dumps({k: v for k, v in run.items() if k != "rows"}))
        return 0
    if args.only == "prefill":
        print(json.dumps(prefill_run(model, prefill_lengths, vocab, cfg, pk["bf16_tflops"], chunk=args.prefill_chunk)))
        return 0

    def frac_of(run, b):
        step_bytes = weight_bytes + run["cache_bytes"]
        achieved = step_bytes / (run["ms_per_step"] / 1e3) / 1e9
        return step_bytes, achieved, achieved / pk["hbm_gbs"]

    prefill = None
    if not together:
        time.sleep(SETTLE_SECONDS)
        prefill = prefill_run(model, prefill_lengths, vocab, cfg, pk["bf16_tflops"])
    clocks = ClockSampler()
    clocks.start()
    main_run = decode_run(model, prompts, args.steps, args.warmup, vocab, state, together)
    clock_info = clocks.stop()
    e2e, _ = e2e_run(model, prompts, args.steps, args.warmup)
    checks = [("decode batch %d" % batch, main_run["rows"])]
    points, points_frac, points_ms = {}, {}, {}
    if headline:
        for b in point_batches:
            for ctx in POINT_CONTEXTS:
                # eight untimed steps, then up to 64 timed ones: the last point ends at 4,088 tokens
                p, st = workload_prompts(args.config, b, ctx, vocab)
                run = decode_run(model, p, min(args.steps, 64), 8, vocab, st)
                _, _, frac = frac_of(run, b)
                key = f"decode_b{b}_c{ctx}"
                points[key] = round(run["tok_s"], 1)
                points_frac[key] = round(frac, 4)
                points_ms[key] = round(run["ms_per_step"], 4)
                if b == 64 and ctx == POINT_CONTEXTS[-1]:
                    checks.append((f"decode batch 64 at {ctx}", run["rows"]))
        if point_batches:
            points["decode_b1"] = points["decode_b1_c2048"]
            points["decode_b64"] = points["decode_b64_c2048"]
    elif not args.no_points:
        p, st = workload_prompts("1.7b", 1, 1024, vocab)
        points["decode_b1"] = round(decode_run(model, p, min(args.steps, 64), args.warmup, vocab, st)["tok_s"], 1)
        points["decode_b64"] = round(main_run["tok_s"], 1) if batch == 64 else None
    if together:
        # the start step of the workload itself: every prompt in one step
        ms = main_run["prompt_ms"]
        lengths = [len(p) for p in prompts]
        flops = prompt_flops(cfg, lengths, 0)
        prefill = {"value": sum(lengths) / (ms / 1e3), "tokens": sum(lengths), "ms": ms,
                   "frac": flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12)}

    if not args.no_check:
        longest = max(len(t) for _, rows in checks for t, _ in rows.values())
        del model
        torch.cuda.empty_cache()
        verifier = Verifier(cfg, longest)
        bad = []
        for what, rows in checks:
            for b, (tokens, got) in rows.items():
                ok, err = verifier.check(f"{what}, sequence {b}", tokens, got)
                if not ok:
                    bad.append(what)
        if bad:
            print("[bench] the timed run's logits are not the model's: no result line", file=sys.stderr)
            return 3

    step_bytes, achieved, frac = frac_of(main_run, batch)
    layers_of = CONFIGS[args.config]["layers"]
    line = {
        "metric": "%s decode tokens/s (batch %d, context %d to %d of %d)" % (
            c["model"], batch, main_run["context_first"], main_run["context_last"], context),
        "value": round(main_run["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random N(0,0.02) weights, uniform LCG token ids",
        "config": {"model": c["model"], "layers": cfg["num_hidden_layers"], "layers_of_configuration": layers_of,
                   "hidden": c["hidden"], "heads": c["heads"], "kv_heads": c["kv_heads"], "head_dim": c["head_dim"],
                   "ffn": c["ffn"], "vocab": vocab, "conv_taps": 3, "sliding_window": 4096,
                   "attention_layers": sum(t != "conv" for t in cfg["layer_types"]),
                   "sliding_layers": cfg["layer_types"].count("sliding_attention"),
                   "global_batch": batch, "seq_len": context,
                   "prompt_len": prompt_len if prompt_len else "uniform 16..2048, %d tokens in one step" % main_run["prompt_tokens"],
                   "cache_tokens": max_tokens, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (weights read per step); %.1f s pause between prompts and decode" % SETTLE_SECONDS,
                   "params": params},
        "e2e": {k: (round(v, 1) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": main_run["launches"],
        "prefill": {"value": round(prefill["value"], 1), "tokens": prefill["tokens"], "ms": round(prefill["ms"], 3),
                    "frac": round(prefill["frac"], 4), "peak": "bf16_tflops %s" % pk["source"]},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(frac, 4), "peak_source": pk["source"], "bytes_per_step": int(step_bytes)},
        "points": points,
        "points_frac": points_frac,
        "points_ms": points_ms,
        "checked": "skipped" if args.no_check else "logits of the timed runs against the 32-bit engine",
        "clocks": clock_info,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
