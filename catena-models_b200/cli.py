"""Command line in the manner of catena-models' binary (src/main.rs:21-101): the same option
names with the same meanings where it has them (--model, --prompt, -n/--max-new-tokens,
--ignore-eos, --bench, --pp, --tg, --tg-context, --bench-runs), a model folder in place of a
Hub selector, token ids in place of text (this library has no tokenizer), and the options the
reference lacks (--temperature, --seed, --dtype, --random, --prompt-lens, --max-slots, --batch,
--pp-chunk).  --kernels and --wmma-prefill / --no-wmma-prefill are the reference's too.

    python -m catena_models_b200 --model DIR --prompt "5 17 3" --prompt "9 9" -n 20
    python -m catena_models_b200 --random config.json --bench --pp 512 --tg 128 --tg-context 1024
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import time


def _positive(value):
    n = int(value)
    if n <= 0:
        raise argparse.ArgumentTypeError("value must be greater than zero")
    return n


def _ids(text):
    try:
        ids = [int(x) for x in text.replace(",", " ").split()]
    except ValueError:
        raise argparse.ArgumentTypeError("a prompt is a list of token ids, e.g. \"5 17 3\"") from None
    if not ids:
        raise argparse.ArgumentTypeError("empty prompt")
    return ids


def parser():
    ap = argparse.ArgumentParser(prog="catena_models_b200", description="LFM3 generation on one B200")
    ap.add_argument("--model", metavar="DIR", help="folder with config.json and model.safetensors")
    ap.add_argument("--random", metavar="CONFIG", help="config.json to build a random-weights model from")
    ap.add_argument("--weights-seed", type=int, default=0, help="seed of the random weights")
    ap.add_argument("--write-random", metavar="DIR", help="write the random model to this folder, then exit")
    ap.add_argument("--prompt", action="append", type=_ids, metavar="IDS",
                    help="token ids of a prompt; repeat for a batch of prompts")
    ap.add_argument("-n", "--max-new-tokens", type=int, default=20, help="maximum number of tokens to generate")
    ap.add_argument("--ignore-eos", action="store_true", help="continue through EOS to a fixed length")
    ap.add_argument("--temperature", type=float, default=0.0, help="0: greedy; above: temperature sampling")
    ap.add_argument("--seed", type=int, default=0, help="seed of the sampler")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--max-tokens", type=_positive, default=None, help="cache size in tokens")
    ap.add_argument("--bench", action="store_true", help="run prompt-processing and token-generation benchmarks")
    ap.add_argument("--pp", type=int, default=512, help="prompt-processing token count; zero skips this test")
    ap.add_argument("--tg", type=int, default=128, help="token-generation count; zero skips this test")
    ap.add_argument("--tg-context", type=_positive, default=1, help="prompt context of the decode benchmark")
    ap.add_argument("--bench-runs", type=_positive, default=1, help="measured runs per benchmark test")
    ap.add_argument("--batch", type=_positive, default=1, help="sequences per step in --bench")
    ap.add_argument("--prompt-lens", type=_ids, metavar="LENGTHS",
                    help="instead of --prompt: synthetic prompts of these lengths (the bench's generator of ids)")
    ap.add_argument("--max-slots", type=_positive, default=None, help="most sequences the cache holds at once")
    ap.add_argument("--kernels", default="fused", choices=["fused", "reference"],
                    help="kernel family, as the reference names it; this library has the fused one only")
    ap.add_argument("--wmma-prefill", dest="wmma_prefill", action="store_true", default=True,
                    help="tensor-core kernels for prompt steps (the default)")
    ap.add_argument("--no-wmma-prefill", dest="wmma_prefill", action="store_false",
                    help="CUDA-core products and attention for prompt steps (bfloat16 activations all the same)")
    ap.add_argument("--pp-chunk", type=int, default=0,
                    help="run the prompt-processing test in steps of this many tokens, each on top of the ones before "
                         "(the reference's server fills its cache in blocks of 1,024, src/server/prefix_cache.rs:4); 0: one step")
    return ap


def _synthetic(count, vocab):
    """The reference's LCG ids (src/main.rs:447-457)."""
    state, out = 0x9E3779B97F4A7C15, []
    for _ in range(count):
        state = (state * 6364136223846793005 + 1442695040888963407) & ((1 << 64) - 1)
        out.append(state % vocab)
    return out


def _rate_stats(samples):
    rates = [n / s for n, s in samples]
    return statistics.mean(rates), (statistics.stdev(rates) if len(rates) > 1 else None)


def run_benchmark(model, pp, tg, tg_context, runs, batch, pp_chunk=0):
    """`pp N`: a fresh cache slot and one prompt step (or steps of `pp_chunk` tokens); `tg N / ctx C`:
    a C-token prompt, two untimed decode steps, N timed ones (src/main.rs:393-445), for `batch`
    sequences at once."""
    import torch

    vocab = model.decoder.vocab_size
    eng = model.engine
    rows = []
    if pp > 0:
        toks = _synthetic(pp, vocab)
        samples = []
        for _ in range(runs + 1):
            slots = eng.admit(batch)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            step = pp_chunk if pp_chunk > 0 else pp
            for at in range(0, pp, step):
                eng.step(slots, [toks[at:at + step]] * batch)
            torch.cuda.synchronize()
            samples.append((pp * batch, time.perf_counter() - t0))
            eng.release(slots)
        eng.check_errors()
        rows.append((f"pp{pp}" + (f"/{pp_chunk}" if pp_chunk > 0 else "") + (f"x{batch}" if batch > 1 else ""),
                     *_rate_stats(samples[1:])))
    if tg > 0:
        toks = _synthetic(tg_context + tg + 2, vocab)
        samples = []
        for _ in range(runs):
            slots = eng.admit(batch)
            eng.step(slots, [toks[:tg_context]] * batch)
            for t in toks[tg_context:tg_context + 2]:
                eng.step(slots, [[t]] * batch)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for t in toks[tg_context + 2:]:
                eng.step(slots, [[t]] * batch)
            torch.cuda.synchronize()
            samples.append((tg * batch, time.perf_counter() - t0))
            eng.release(slots)
        eng.check_errors()
        rows.append((f"tg{tg}/ctx{tg_context}" + (f"x{batch}" if batch > 1 else ""), *_rate_stats(samples)))
    params = model.parameter_count()
    size = model.decoder.weight_bytes_per_step()
    name = f"{model.decoder.definition.architecture} {params / 1e9:.2f}B {model.decoder.rt.dtype}".replace("torch.", "")
    print(f"| {'model':40} | {'size':>10} | {'params':>10} | {'test':>15} | {'t/s':>20} |")
    print(f"| {'-' * 40} | {'-' * 10} | {'-' * 10} | {'-' * 15} | {'-' * 20} |")
    for test, mean, std in rows:
        rate = f"{mean:.2f}" if std is None else f"{mean:.2f} ± {std:.2f}"
        size_s = f"{size / 2**30:.2f} GiB" if size >= 2**30 else f"{size / 2**20:.2f} MiB"
        par_s = f"{params / 1e9:.2f} B" if params >= 1e9 else f"{params / 1e6:.2f} M"
        print(f"| {name:40} | {size_s:>10} | {par_s:>10} | {test:>15} | {rate:>20} |")


def main(argv=None):
    ap = parser()
    args = ap.parse_args(argv)
    if not args.model and not args.random:
        ap.error("one of --model and --random is required")
    if args.model and args.random:
        ap.error("--model and --random exclude each other")
    if args.write_random:
        if not args.random:
            ap.error("--write-random needs --random CONFIG")
        from .weights.random_init import write_random_model

        with open(args.random) as fh:
            print(write_random_model(args.write_random, json.load(fh), args.weights_seed))
        return 0
    if args.kernels != "fused":
        ap.error("--kernels reference: LFM3 has the fused kernels only (as in the reference, src/lfm3.rs:15-18)")
    if args.prompt and args.prompt_lens:
        ap.error("--prompt and --prompt-lens exclude each other")
    if not args.bench and not args.prompt and not args.prompt_lens:
        ap.error("--prompt or --prompt-lens is required unless --bench is given")
    if args.bench and (args.prompt or args.prompt_lens):
        ap.error("--bench and --prompt exclude each other")

    from .api import Model
    from .csrc.limits import PAGE_TOKENS

    if args.bench:
        need = args.batch * (max(args.pp, args.tg_context + args.tg + 2) + PAGE_TOKENS)
    else:
        lens = args.prompt_lens or [len(p) for p in args.prompt]
        need = sum(-(-(n + args.max_new_tokens) // PAGE_TOKENS) * PAGE_TOKENS for n in lens)
    max_tokens = args.max_tokens or max(need, PAGE_TOKENS)
    t0 = time.perf_counter()
    if args.model:
        model = Model.load(args.model, dtype=args.dtype, max_tokens=max_tokens, max_seqs=args.max_slots)
    else:
        with open(args.random) as fh:
            model = Model.random(json.load(fh), seed=args.weights_seed, dtype=args.dtype, max_tokens=max_tokens,
                                 max_seqs=args.max_slots)
    model.decoder.rt.tensor_core_prompts = args.wmma_prefill
    if args.prompt_lens:
        ids = _synthetic(sum(args.prompt_lens), model.decoder.vocab_size)
        args.prompt, at = [], 0
        for n in args.prompt_lens:
            args.prompt.append(ids[at:at + n])
            at += n
    print(f"loaded {model.parameter_count() / 1e6:.2f} M parameters in {time.perf_counter() - t0:.2f}s; "
          f"cache of {max_tokens} tokens: {model.engine.cache.bytes() / 2**20:.1f} MiB", file=sys.stderr)
    if args.bench:
        run_benchmark(model, args.pp, args.tg, args.tg_context, args.bench_runs, args.batch, args.pp_chunk)
        return 0

    import torch

    marks = {}

    def on_step(step, live):
        torch.cuda.synchronize()
        marks.setdefault("first", time.perf_counter())
        marks["last"] = time.perf_counter()
        marks["decoded"] = marks.get("decoded", 0) + (live if step > 0 else 0)

    start = time.perf_counter()
    out = model.generate(args.prompt, max_new_tokens=args.max_new_tokens, temperature=args.temperature,
                         seed=args.seed, ignore_eos=args.ignore_eos, on_step=on_step)
    for g in out:
        print(" ".join(str(t) for t in g.tokens))
    if args.max_new_tokens > 0 and "first" in marks:
        prompt_tokens = sum(len(p) for p in args.prompt)
        generated = sum(len(g.tokens) for g in out)
        prompt_s, eval_s, total_s = marks["first"] - start, marks["last"] - marks["first"], marks["last"] - start
        rate = lambda n, s: n / s if s > 0 else float("inf")
        print(f"prompt eval: {prompt_tokens} token(s) in {prompt_s:.2f}s ({rate(prompt_tokens, prompt_s):.2f} tok/s)",
              file=sys.stderr)
        print(f"cached eval: {marks['decoded']} token(s) in {eval_s:.2f}s ({rate(marks['decoded'], eval_s):.2f} tok/s)",
              file=sys.stderr)
        print(f"generated {generated} token(s) in {total_s:.2f}s ({rate(generated, total_s):.2f} tok/s)", file=sys.stderr)
    return 0
