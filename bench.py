#!/usr/bin/env python3
"""Decode and prefill throughput of the LFM3-1.7B-class model with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl reference]

A step is one decode step of the whole batch.  Prints one JSON line: decoded tokens per
second on the device (`value`), the same through the Python entry point with host tokens in
and out (`e2e`), a 2,048-token prefill, the decode step's memory roofline, and decode at
batch 1 and 64 (`points`).  This engine runs on one GPU; for --gpus above 1 it says so and
exits with 2.
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

# The 1.7B-class model of the headline benchmark.  The layer pattern (two conv layers, then an
# attention layer, alternately full and sliding) is this bench's choice; the reference fixes
# only that its 24-layer model has conv, full and sliding layers (tests/lfm3.rs:39-42).
FULL_LAYERS = 24


def model_config(layers):
    types = []
    attn = 0
    for l in range(layers):
        if l % 3 == 2:
            types.append("full_attention" if attn % 2 == 0 else "sliding_attention")
            attn += 1
        else:
            types.append("conv")
    return dict(architecture="lfm3", vocab_size=65536, hidden_size=2048, intermediate_size=8192,
                num_hidden_layers=layers, layer_types=types, num_attention_heads=32, num_key_value_heads=8,
                head_dim=64, conv_L_cache=3, sliding_window=4096, rope_theta=1000000.0, norm_eps=1e-5,
                tie_word_embeddings=True, max_position_embeddings=4096)


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


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

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


def decode_run(model, batch, prompt_len, steps, warmup, vocab):
    """Prefill `batch` prompts, run `warmup` untimed and `steps` timed decode steps with given
    (synthetic) tokens and the greedy choice computed on the device.  Returns facts of the run."""
    import torch

    from catena_models_b200 import kernels

    eng = model.engine
    slots = eng.admit(batch)
    state = 0x9E3779B97F4A7C15
    for i in range(0, batch, 8):                          # prompts in groups of 8 sequences
        group = slots[i:i + 8]
        prompts = []
        for _ in group:
            toks, state = synthetic_tokens(prompt_len, vocab, state)
            prompts.append(toks)
        for s, p in zip(group, prompts):                  # one sequence per step keeps the step's memory small
            eng.step([s], [p])
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
    start.record()
    for i in range(warmup, warmup + steps):
        eng.step(slots, [[t] for t in feed[i]])
        if i == warmup + steps // 2:
            mid_bytes = eng.cache.live_bytes()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop)
    launches = kernels.launches - launches0
    eng.release(slots)
    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "launches": launches,
            "cache_bytes": mid_bytes}


def e2e_run(model, batch, prompt_len, steps, warmup, vocab):
    """The same decode through Model.generate: per step the host sends that step's inputs from
    pinned memory (positions, slots, page-table updates, sampler keys; the token ids themselves are
    taken on the device from the step before, which chose them) and reads the chosen tokens back.
    The loop keeps the device one step ahead of its own bookkeeping."""
    import torch

    prompts, state = [], 0x9E3779B97F4A7C15
    for _ in range(batch):
        toks, state = synthetic_tokens(prompt_len, vocab, state)
        prompts.append(toks)
    marks = {}

    def on_step(step, live):
        if step == warmup:
            torch.cuda.synchronize()
            marks["t0"] = time.perf_counter()
        if step == warmup + steps:
            torch.cuda.synchronize()
            marks["t1"] = time.perf_counter()

    # Two tokens more than the marks need: with the device a step ahead, the step after each marked
    # one is in flight when its mark synchronises, so both marks see the same amount of extra work
    # and the interval holds exactly `steps` steps.
    model.generate(prompts, max_new_tokens=warmup + steps + 2, temperature=0.0, ignore_eos=True,
                   stop_token_ids=(), max_batch=batch, on_step=on_step)
    sec = marks["t1"] - marks["t0"]
    eng = model.engine
    layout_bytes = max((g.layout.size * 4 for (b, _), g in eng._graphs.items() if b == batch), default=0)
    return {"value": batch * steps / sec, "unit": "tok/s",
            "h2d_bytes_per_step": layout_bytes,
            "d2h_bytes_per_step": batch * 4}


def prefill_run(model, tokens_n, vocab, cfg, peak_tflops):
    import torch

    eng = model.engine
    toks, _ = synthetic_tokens(tokens_n, vocab)
    times = []
    for i in range(4):
        (slot,) = eng.admit(1)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.step([slot], [toks])
        b.record()
        torch.cuda.synchronize()
        eng.release([slot])
        if i >= 1:
            times.append(a.elapsed_time(b))
    ms = statistics.median(times)
    H, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    QS = cfg["num_attention_heads"] * cfg["head_dim"]
    KVS = cfg["num_key_value_heads"] * cfg["head_dim"]
    flops = 0.0
    T = tokens_n
    for kind in cfg["layer_types"]:
        if kind == "conv":
            flops += 2.0 * T * (3 * H * H + H * H)
        else:
            flops += 2.0 * T * ((QS + 2 * KVS + cfg["num_attention_heads"]) * H + QS * H)
            W = cfg["sliding_window"] if kind == "sliding_attention" else T
            keys = sum(min(p + 1, W) for p in range(T))
            flops += 4.0 * QS * keys
        flops += 2.0 * T * 3 * F * H
    flops += 2.0 * 1 * V * H
    return {"value": T / (ms / 1e3), "tokens": T, "ms": ms, "frac": flops / (ms / 1e3) / (peak_tflops * 1e12),
            "flops": flops}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the configuration's 24")
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--prefill-tokens", type=int, default=2048,
                    help="prompt length of `--only prefill` (the full run always measures 2,048)")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="run one part only (small captures under a profiler); prints that part's facts")
    args = ap.parse_args()

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
    if args.prompt_len + args.warmup + args.steps + 1 > args.context:
        args.steps = args.context - args.prompt_len - args.warmup - 1

    import torch

    from catena_models_b200.api import Model

    pk = peaks()
    cfg = model_config(args.layers)
    vocab = cfg["vocab_size"]
    big = 64 if not (args.no_points or args.only != "all") else args.batch
    model = Model.random(cfg, seed=0, std=0.02, dtype="bfloat16", device="cuda:0",
                         max_tokens=max(big, args.batch) * args.context, max_seqs=max(big, args.batch))
    weight_bytes = model.decoder.weight_bytes_per_step()

    if args.only == "decode":
        print(json.dumps(decode_run(model, args.batch, args.prompt_len, args.steps, args.warmup, vocab)))
        return 0
    if args.only == "prefill":
        print(json.dumps(prefill_run(model, args.prefill_tokens, vocab, cfg, pk["bf16_tflops"])))
        return 0
    clocks = ClockSampler()
    clocks.start()
    main_run = decode_run(model, args.batch, args.prompt_len, args.steps, args.warmup, vocab)
    clock_info = clocks.stop()
    e2e = e2e_run(model, args.batch, args.prompt_len, args.steps, args.warmup, vocab)
    points = {}
    if not args.no_points:
        for b in (1, 64):
            steps = min(args.steps, 128)
            points[f"decode_b{b}"] = round(decode_run(model, b, args.prompt_len, steps, args.warmup, vocab)["tok_s"], 1)
    prefill = prefill_run(model, 2048, vocab, cfg, pk["bf16_tflops"])

    step_bytes = weight_bytes + main_run["cache_bytes"]
    achieved = step_bytes / (main_run["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": "LFM3-1.7B-class decode tokens/s (batch %d, context %d)" % (args.batch, args.context),
        "value": round(main_run["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random N(0,0.02) weights, uniform LCG token ids",
        "config": {"model": "LFM3-1.7B-class", "layers": args.layers, "layers_of_configuration": FULL_LAYERS,
                   "hidden": 2048, "heads": 32, "kv_heads": 8, "head_dim": 64, "ffn": 8192, "vocab": 65536,
                   "conv_taps": 3, "sliding_window": 4096, "attention_layers": cfg["layer_types"].count("full_attention") + cfg["layer_types"].count("sliding_attention"),
                   "global_batch": args.batch, "seq_len": args.context, "prompt_len": args.prompt_len,
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (weights read per step)",
                   "params": model.parameter_count()},
        "e2e": {k: (round(v, 1) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": main_run["launches"],
        "prefill": {"value": round(prefill["value"], 1), "tokens": prefill["tokens"], "ms": round(prefill["ms"], 3),
                    "frac": round(prefill["frac"], 4), "peak": "bf16_tflops %s" % pk["source"]},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peak_source": pk["source"],
                     "bytes_per_step": int(step_bytes)},
        "points": points,
        "clocks": clock_info,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
