"""Each part alone (norm, position encoding, attention mixer, short-conv mixer, feed-forward,
block), built from parameters at sizes of its own and compared with the plain functions; and a
toy architecture with a toy mixer that keeps state of its own, registered from this file."""
import dataclasses

import pytest
import torch

import plain_lfm3 as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _runtime(dtype):
    from catena_models_b200.engine.runtime import Runtime
    return Runtime(dtype, DEV)


def _batch(rt, cache, slots, token_lists, positions):
    """A StepBatch for parts that are stepped outside an Engine."""
    from catena_models_b200.engine.batch import BatchLayout, StepBatch, fill_host

    updates = []
    for s, p, t in zip(slots, positions, token_lists):
        updates += cache.flat_updates(s, cache.book.reserve(s, p + len(t)))
        cache.book.advance(s, p + len(t))
    T = sum(len(t) for t in token_lists)
    layout = BatchLayout(T, len(slots), 0, len(updates))
    host = torch.zeros(layout.size, dtype=torch.int32)
    fill_host(layout, host.numpy(), slots, token_lists, positions, [[] for _ in slots], updates)
    kind = ("prefill" if all(p == 0 for p in positions) else
            "decode" if all(len(t) == 1 for t in token_lists) else "append")
    batch = StepBatch(layout, host.to(DEV), kind, [len(t) for t in token_lists], positions, 0, len(updates))
    from catena_models_b200 import kernels
    if updates:
        kernels.scatter_i32(cache.ptab_all, batch.upd_index, batch.upd_value, batch.upd_count, layout.U)
    return batch


def _bind(part, rt, seed, std=0.3):
    from catena_models_b200.weights.random_init import random_tensors
    from catena_models_b200.weights.loader import adopt_tensors

    specs = part.all_tensor_specs()
    raw = random_tensors(specs, seed, std=std, norm_weights="random", rope_factors="uniform")
    tensors = adopt_tensors(raw, specs, rt.device, widen=rt.dtype == torch.float32)
    part.bind_all(tensors, rt)
    return {k: v.double() for k, v in raw.items()}


def _close(got, ref, dtype, same=None):
    """float32: close to the exact result.  bfloat16 with `same` (the plain part run with the
    reference's bfloat16 rounding points on the same inputs): the part's largest error is at most
    twice the largest error that the rounding points alone cause."""
    got = got.double().cpu()
    if dtype == torch.float32:
        torch.testing.assert_close(got, ref, rtol=2e-5, atol=2e-5)
    elif same is None:
        torch.testing.assert_close(got, ref, rtol=3e-2, atol=3e-2)
    else:
        assert float((got - ref).abs().max()) <= 2.0 * float((same - ref).abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_and_rotary_alone(dtype):
    from catena_models_b200.parts import build_part

    rt = _runtime(dtype)
    norm = build_part("norm", "rms", name="n.weight", width=136, eps=3e-4)
    raw = _bind(norm, rt, 1)
    x = torch.randn(9, 136).to(dtype)
    _close(norm.apply(rt, x.to(DEV)), P.rms_norm(x.double(), raw["n.weight"], 3e-4), dtype)
    rot = build_part("position", "rotary", head_dim=48, theta=12345.0, factors_name="f.weight")
    raw = _bind(rot, rt, 2)
    want = P.rope_frequencies(12345.0, 48, torch.float32) / raw["f.weight"].float()
    assert torch.equal(rot.rate_table().cpu(), want)
    assert build_part("position", "none").rate_table() is None


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,gate,qk_norm", [(0, True, True), (20, False, True), (70, True, False)])
def test_attention_mixer_alone(dtype, window, gate, qk_norm):
    """Prompt step over three sequences, then decode steps, against the plain mixer."""
    from catena_models_b200.cache.cache import Cache
    from catena_models_b200.parts import build_part

    H, QH, KVH, HD = 72, 6, 2, 32
    rt = _runtime(dtype)
    pos_part = build_part("position", "rotary", head_dim=HD, theta=5000.0, factors_name=None if window else "rope_freqs.weight")
    mixer = build_part("mixer", "gqa_attention", prefix="L.", hidden=H, heads=QH, kv_heads=KVH, head_dim=HD,
                       window=window, position=pos_part, qk_norm_eps=1e-5 if qk_norm else None, output_gate=gate)
    raw = _bind(mixer, rt, 3, std=0.2)
    w = {k[2:] if k.startswith("L.") else k: v for k, v in raw.items()}
    if not qk_norm:
        w["attn_q_norm.weight"] = w["attn_k_norm.weight"] = None
    if window:
        w["rope_freqs.weight"] = torch.ones(HD // 2, dtype=torch.float64)
    cfg = dict(num_attention_heads=QH, num_key_value_heads=KVH, head_dim=HD, norm_eps=1e-5, sliding_window=window,
               rope_theta=5000.0, rope_theta_sliding=5000.0, attn_output_gate=gate)
    cache = Cache([mixer.state_spec()], 1024, dtype, DEV)
    lens, extra = [5, 90, 33], 6
    seqs = [torch.randn(n + extra, H).to(dtype) for n in lens]
    slots = [cache.admit() for _ in lens]
    batch = _batch(rt, cache, slots, [[0] * n for n in lens], [0, 0, 0])
    y = mixer.forward(rt, batch, torch.cat([s[:n] for s, n in zip(seqs, lens)]).to(DEV), cache.view(0))
    outs = [[y[a:a + n]] for a, n in zip([0, 5, 95], lens)]
    for t in range(extra):
        batch = _batch(rt, cache, slots, [[0]] * 3, [n + t for n in lens])
        y = mixer.forward(rt, batch, torch.stack([s[n + t] for s, n in zip(seqs, lens)]).to(DEV), cache.view(0))
        for b in range(3):
            outs[b].append(y[b:b + 1])

    def plain(n, r=P._identity):
        kind = "sliding_attention" if window else "full_attention"
        if qk_norm:
            return P.attention_mixer(n, w, cfg, kind, r)
        old = P.rms_norm                                  # no head norm: the plain mixer's norm becomes the identity
        P.rms_norm = lambda x, ww, eps, rr=P._identity: x if ww is None else old(x, ww, eps, rr)
        try:
            return P.attention_mixer(n, w, cfg, kind, r)
        finally:
            P.rms_norm = old

    for b, s in enumerate(seqs):
        _close(torch.cat(outs[b]), plain(s.double()), dtype, plain(s.double(), P._round_bf16))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_shortconv_ffn_and_block_alone(dtype):
    from catena_models_b200.cache.cache import Cache
    from catena_models_b200.parts import build_part

    H, F, taps = 88, 168, 5
    rt = _runtime(dtype)
    conv = build_part("mixer", "short_conv", prefix="L.", hidden=H, taps=taps)
    ffn = build_part("feed_forward", "swiglu", prefix="L.", hidden=H, intermediate=F)
    norms = {n: build_part("norm", "rms", name=f"L.{n}.weight", width=H, eps=1e-5)
             for n in ("attn_norm", "post_attention_norm", "ffn_norm", "post_ffw_norm")}
    block = build_part("block", "sandwich", mixer=conv, feed_forward=ffn, input_norm=norms["attn_norm"],
                       ffn_norm=norms["ffn_norm"], post_mixer_norm=norms["post_attention_norm"],
                       post_ffn_norm=norms["post_ffw_norm"])
    raw = _bind(block, rt, 4, std=0.15)
    w = {k[2:]: v for k, v in raw.items()}
    cfg = dict(conv_L_cache=taps, norm_eps=1e-5, post_norm=True)
    cache = Cache([block.state_spec()], 1024, dtype, DEV)
    lens, extra = [3, 40], 4
    seqs = [torch.randn(n + extra, H).to(dtype) for n in lens]
    slots = [cache.admit() for _ in lens]
    hs = torch.cat([s[:n] for s, n in zip(seqs, lens)]).to(DEV)
    batch = _batch(rt, cache, slots, [[0] * n for n in lens], [0, 0])
    # parts alone: the feed-forward and the mixer on the same rows
    _close(ffn.forward(rt, batch, hs), P.swiglu_ffn(hs.double().cpu(), w), dtype,
           P.swiglu_ffn(hs.double().cpu(), w, P._round_bf16))
    h, n_next = block.forward(rt, batch, hs.clone(), norms["attn_norm"].apply(rt, hs), cache.view(0), norms["attn_norm"])
    outs = [[h[a:a + n]] for a, n in zip([0, 3], lens)]
    _close(n_next, P.rms_norm(h.double().cpu(), w["attn_norm.weight"], 1e-5), dtype)
    for t in range(extra):
        batch = _batch(rt, cache, slots, [[0]] * 2, [n + t for n in lens])
        x = torch.stack([s[n + t] for s, n in zip(seqs, lens)]).to(DEV)
        h, none = block.forward(rt, batch, x.clone(), norms["attn_norm"].apply(rt, x), cache.view(0), None)
        assert none is None
        for b in range(2):
            outs[b].append(h[b:b + 1])
    for b, s in enumerate(seqs):
        _close(torch.cat(outs[b]), P.block(s.double(), w, cfg, "conv"), dtype, P.block(s.double(), w, cfg, "conv", P._round_bf16))


# ----------------------------------------------------------------------------- toy parts
def test_toy_mixer_with_its_own_state_registers_builds_and_steps():
    """A mixer defined here (a per-channel leaky running sum, one float vector of state per
    sequence), a layer-norm-free toy architecture around it, registered, built with random
    weights and stepped through prompt and decode steps, without touching the library."""
    from catena_models_b200 import register_architecture, register_part
    from catena_models_b200.api import Model
    from catena_models_b200.cache.spec import FixedStateSpec
    from catena_models_b200.config.base import Reader
    from catena_models_b200.engine.definition import ModelDefinition, PlanEntry
    from catena_models_b200.parts import Mixer, build_part
    from catena_models_b200.parts.linear import Linear
    from catena_models_b200.weights.loader import TensorSpec

    class LeakySum(Mixer):
        """s_t = decay * s_{t-1} + x_t ; y_t = proj(s_t * scale).  State: s, float32 [hidden]."""

        def __init__(self, prefix, hidden, decay):
            self.hidden, self.decay = hidden, decay
            self.scale_name = prefix + "scale"
            self.proj = Linear(prefix + "proj.weight", hidden, hidden)

        def children(self):
            return [self.proj]

        def tensor_specs(self):
            return [TensorSpec(self.scale_name, (self.hidden,), "norm")]

        def bind(self, tensors, rt):
            self.scale = tensors[self.scale_name].float()

        def state_spec(self):
            return FixedStateSpec((self.hidden,), "float32")

        def forward(self, rt, batch, x, state):
            slots = batch.seq_slot.long()
            out = torch.empty_like(x, dtype=torch.float32)
            if batch.prefill:
                start = 0
                for b, n in enumerate(batch.lengths):
                    s = torch.zeros(self.hidden, device=x.device)
                    for t in range(start, start + n):
                        s = self.decay * s + x[t].float()
                        out[t] = s
                    state.tensor[slots[b]] = s
                    start += n
            else:
                s = self.decay * state.tensor[slots] + x.float()
                state.tensor[slots] = s
                out = s
            return self.proj.apply(rt, (out * self.scale).to(x.dtype))

    @dataclasses.dataclass(frozen=True)
    class ToyConfig:
        vocab_size: int
        hidden_size: int
        intermediate_size: int
        layer_kinds: tuple
        decay: float
        norm_eps: float

        @classmethod
        def from_dict(cls, data, where="config.json"):
            r = Reader(data, where)
            cfg = cls(r.integer("vocab_size"), r.integer("hidden_size"), r.integer("intermediate_size"),
                      r.string_list("layer_kinds"), r.number("decay"), r.number("norm_eps"))
            r.finish()
            return cfg

    def define(cfg):
        H = cfg.hidden_size
        blocks = []
        for l, kind in enumerate(cfg.layer_kinds):
            pre = f"layers.{l}."
            mixer = (build_part("mixer", "toy_leaky_sum", prefix=pre, hidden=H, decay=cfg.decay) if kind == "leaky"
                     else build_part("mixer", "short_conv", prefix=pre, hidden=H, taps=2))
            blocks.append(build_part(
                "block", "sandwich", mixer=mixer,
                feed_forward=build_part("feed_forward", "swiglu", prefix=pre, hidden=H, intermediate=cfg.intermediate_size),
                input_norm=build_part("norm", "rms", name=pre + "in_norm.weight", width=H, eps=cfg.norm_eps),
                ffn_norm=build_part("norm", "rms", name=pre + "ffn_norm.weight", width=H, eps=cfg.norm_eps)))
        return ModelDefinition("toy", cfg.vocab_size, H, "embed.weight", blocks,
                               [PlanEntry(i, i) for i in range(len(blocks))],
                               build_part("norm", "rms", name="final_norm.weight", width=H, eps=cfg.norm_eps), None)

    register_part("mixer", "toy_leaky_sum", LeakySum, replace=True)
    register_architecture("toy", ToyConfig, define, replace=True)
    config = dict(architecture="toy", vocab_size=50, hidden_size=32, intermediate_size=48,
                  layer_kinds=["leaky", "conv", "leaky"], decay=0.75, norm_eps=1e-5)
    from catena_models_b200.engine.model import DecoderModel
    from catena_models_b200.weights.random_init import random_tensors

    raw = random_tensors(define(ToyConfig.from_dict(config)).tensor_specs(), 5, std=0.3, norm_weights="random")
    model = Model(DecoderModel.from_tensors(config, raw, torch.float32, DEV), max_tokens=512)
    eng = model.engine
    assert [type(s).__name__ for s in model.decoder.state_specs] == ["FixedStateSpec"] * 3
    assert len(eng.cache.fixed_storage) == 2                       # two groups: [32] and [1, 32]

    # the same toy model in plain torch on the CPU
    w = {k: v.double() for k, v in raw.items()}

    def plain(tokens):
        h = w["embed.weight"][tokens]
        for l, kind in enumerate(config["layer_kinds"]):
            pre = f"layers.{l}."
            n = P.rms_norm(h, w[pre + "in_norm.weight"], 1e-5)
            if kind == "leaky":
                s, rows = torch.zeros(32, dtype=torch.float64), []
                for t in range(n.shape[0]):
                    s = 0.75 * s + n[t]
                    rows.append(s)
                m = (torch.stack(rows) * w[pre + "scale"]) @ w[pre + "proj.weight"].T
            else:
                m = P.shortconv_mixer(n, {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)}, dict(conv_L_cache=2))
            h = h + m
            n2 = P.rms_norm(h, w[pre + "ffn_norm.weight"], 1e-5)
            h = h + P.swiglu_ffn(n2, {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)})
        return P.rms_norm(h, w["final_norm.weight"], 1e-5) @ w["embed.weight"].T

    seqs = [[3, 9, 27, 31, 4, 1, 49, 0, 12], [7, 7, 8, 40]]
    for round_ in range(2):                                         # twice: the slots are used again
        slots = eng.admit(2)
        got = [[], []]
        out = eng.step(slots, [seqs[0][:5], seqs[1][:2]], [[0, 1, 2, 3, 4], [0, 1]])
        got[0].append(out[:5].clone())
        got[1].append(out[5:].clone())
        for t in range(2):
            out = eng.step(slots, [[seqs[0][5 + t]], [seqs[1][2 + t]]])
            got[0].append(out[0:1].clone())
            got[1].append(out[1:2].clone())
        eng.release([slots[1]])
        for t in range(7, 9):
            got[0].append(eng.step([slots[0]], [[seqs[0][t]]]).clone())
        eng.release([slots[0]])
        for g, s in zip(got, seqs):
            torch.testing.assert_close(torch.cat(g).double().cpu(), plain(s), rtol=2e-5, atol=2e-5)


def test_a_layer_reads_another_layers_cache():
    """A toy architecture whose third layer has no key/value projections: the plan gives it the
    state unit of the first layer (owns_state=False), so it attends over that layer's keys and
    values, in the prompt step (the owner's keys of this step) and in decode steps (the cache)."""
    from catena_models_b200 import register_architecture
    from catena_models_b200.api import Model
    from catena_models_b200.config.base import Reader
    from catena_models_b200.engine.definition import ModelDefinition, PlanEntry
    from catena_models_b200.engine.model import DecoderModel
    from catena_models_b200.parts import build_part
    from catena_models_b200.weights.random_init import random_tensors

    H, QH, KVH, HD, F, V, EPS, THETA = 48, 3, 1, 16, 80, 60, 1e-5, 10000.0

    class Cfg:
        @classmethod
        def from_dict(cls, data, where="config.json"):
            r = Reader(data, where)
            r.string("architecture")
            r.finish()
            return cls()

    def attention(prefix, shares):
        return build_part("mixer", "gqa_attention", prefix=prefix, hidden=H, heads=QH, kv_heads=KVH, head_dim=HD,
                          window=0, position=build_part("position", "rotary", head_dim=HD, theta=THETA),
                          qk_norm_eps=EPS, output_gate=False, shares_kv=shares)

    def define(cfg):
        blocks = []
        for l, shares in enumerate((False, False, True)):
            pre = f"l{l}."
            blocks.append(build_part(
                "block", "sandwich", mixer=attention(pre, shares),
                feed_forward=build_part("feed_forward", "swiglu", prefix=pre, hidden=H, intermediate=F),
                input_norm=build_part("norm", "rms", name=pre + "n1", width=H, eps=EPS),
                ffn_norm=build_part("norm", "rms", name=pre + "n2", width=H, eps=EPS)))
        plan = [PlanEntry(0, 0), PlanEntry(1, 1), PlanEntry(2, 0, owns_state=False)]
        return ModelDefinition("toy_shared", V, H, "embed", blocks, plan,
                               build_part("norm", "rms", name="nf", width=H, eps=EPS), None)

    register_architecture("toy_shared", Cfg, define, replace=True)
    config = dict(architecture="toy_shared")
    raw = random_tensors(define(Cfg()).tensor_specs(), 9, std=0.2, norm_weights="random")
    assert "l2.attn_k.weight" not in raw and "l2.attn_q.weight" in raw
    w = {k: v.double() for k, v in raw.items()}
    model = Model(DecoderModel.from_tensors(config, raw, torch.float32, DEV), max_tokens=512)
    assert len(model.decoder.state_specs) == 2                    # two state units for three layers

    def plain(tokens):
        T = len(tokens)
        pos = torch.arange(T)
        ones = torch.ones(HD // 2, dtype=torch.float64)
        h = w["embed"][tokens]
        kv = {}
        for l in range(3):
            pre = f"l{l}."
            n = P.rms_norm(h, w[pre + "n1"], EPS)
            q = P.rms_norm((n @ w[pre + "attn_q.weight"].T).view(T, QH, HD), w[pre + "attn_q_norm.weight"], EPS)
            q = P.rope(q, pos, THETA, ones, sliding=True)
            if l < 2:
                k = P.rms_norm((n @ w[pre + "attn_k.weight"].T).view(T, KVH, HD), w[pre + "attn_k_norm.weight"], EPS)
                kv[l] = (P.rope(k, pos, THETA, ones, sliding=True), (n @ w[pre + "attn_v.weight"].T).view(T, KVH, HD))
            k, v = kv[0] if l == 2 else kv[l]
            ctx = torch.zeros(T, QH, HD, dtype=torch.float64)
            for hq in range(QH):
                s = (q[:, hq] @ k[:, 0].T) * HD ** -0.5
                s = s.masked_fill(P.attention_mask(T, 0), float("-inf"))
                ctx[:, hq] = torch.softmax(s, -1) @ v[:, 0]
            h = h + ctx.reshape(T, QH * HD) @ w[pre + "attn_output.weight"].T
            h = h + P.swiglu_ffn(P.rms_norm(h, w[pre + "n2"], EPS), {k2[len(pre):]: v2 for k2, v2 in w.items() if k2.startswith(pre)})
        return P.rms_norm(h, w["nf"], EPS) @ w["embed"].T

    eng = model.engine
    seqs = [[1, 5, 9, 13, 17, 21, 25, 29, 33, 37, 41], [2, 4, 6]]
    slots = eng.admit(2)
    got = [[], []]
    out = eng.step(slots, [seqs[0][:7], seqs[1][:2]], [list(range(7)), [0, 1]])
    got[0].append(out[:7].clone())
    got[1].append(out[7:].clone())
    out = eng.step(slots, [[seqs[0][7]], [seqs[1][2]]])
    got[0].append(out[0:1].clone())
    got[1].append(out[1:2].clone())
    eng.release([slots[1]])
    for t in range(8, 11):
        got[0].append(eng.step([slots[0]], [[seqs[0][t]]]).clone())
    eng.release([slots[0]])
    for g, s in zip(got, seqs):
        torch.testing.assert_close(torch.cat(g).double().cpu(), plain(s), rtol=2e-5, atol=2e-5)


def test_toy_routed_feed_forward_and_another_position_encoding():
    """Two more toy parts defined here and registered from outside the package: a feed-forward
    that routes every token to its best-scoring expert (router logits in float32) and a position
    encoding that turns only the first quarter of a head's pairs, at linearly spaced rates.  One
    toy architecture uses them in one layer and the stock parts in the other; prompt steps,
    decode steps and a batch of unequal lengths are compared with plain torch."""
    from catena_models_b200 import register_architecture, register_part
    from catena_models_b200.api import Model
    from catena_models_b200.config.base import Reader
    from catena_models_b200.engine.definition import ModelDefinition, PlanEntry
    from catena_models_b200.engine.model import DecoderModel
    from catena_models_b200.parts import build_part
    from catena_models_b200.parts.base import FeedForward, Position
    from catena_models_b200.parts.linear import Linear
    from catena_models_b200.weights.loader import TensorSpec
    from catena_models_b200.weights.random_init import random_tensors

    H, QH, KVH, HD, F, E, V, EPS = 40, 2, 2, 16, 56, 3, 70, 1e-6

    class QuarterTurn(Position):
        """angle(p, i) = p * step * (i + 1) for i < head_dim / 4, no rotation of the other pairs."""

        def __init__(self, head_dim, step):
            self.head_dim, self.step = head_dim, step
            self._table = None

        def rates(self):
            r = torch.zeros(self.head_dim // 2, dtype=torch.float32)
            q = self.head_dim // 4
            r[:q] = self.step * torch.arange(1, q + 1, dtype=torch.float32)
            return r

        def bind(self, tensors, rt):
            self._table = self.rates().to(rt.device)

        def rate_table(self):
            return self._table

    class Top1Experts(FeedForward):
        """y_t = SwiGLU_{e(t)}(x_t) * p_t, e(t) = argmax of the float32 router logits, p_t its softmax weight."""

        capturable = False            # the host gathers each expert's rows: no graph replay of decode steps

        def __init__(self, prefix, hidden, intermediate, experts):
            self.router_name = prefix + "router.weight"
            self.hidden, self.n = hidden, experts
            self.gate_up = [Linear([f"{prefix}e{e}.gate.weight", f"{prefix}e{e}.up.weight"], [intermediate, intermediate], hidden)
                            for e in range(experts)]
            self.down = [Linear(f"{prefix}e{e}.down.weight", hidden, intermediate) for e in range(experts)]
            self.intermediate = intermediate

        def children(self):
            return self.gate_up + self.down

        def tensor_specs(self):
            return [TensorSpec(self.router_name, (self.n, self.hidden), "matrix")]

        def bind(self, tensors, rt):
            self.router = tensors[self.router_name].float()

        def forward(self, rt, batch, x):
            logits = x.float() @ self.router.T                      # float32 whatever the activations are
            prob = torch.softmax(logits, dim=-1)
            best = logits.argmax(dim=-1)
            y = torch.zeros_like(x)
            for e in range(self.n):
                rows = (best == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                xe = x[rows].contiguous()
                a = rt.gate_up_swiglu(xe, self.gate_up[e].weight, self.intermediate)
                out = self.down[e].apply(rt, a).float() * prob[rows, e].unsqueeze(1)
                y[rows] = out.to(x.dtype)
            return y

    class Cfg:
        @classmethod
        def from_dict(cls, data, where="config.json"):
            r = Reader(data, where)
            r.string("architecture")
            r.finish()
            return cls()

    def define(cfg):
        blocks = []
        for l in range(2):
            pre = f"l{l}."
            position = (build_part("position", "toy_quarter_turn", head_dim=HD, step=0.05) if l == 0
                        else build_part("position", "rotary", head_dim=HD, theta=10000.0))
            ff = (build_part("feed_forward", "toy_top1", prefix=pre, hidden=H, intermediate=F, experts=E) if l == 0
                  else build_part("feed_forward", "swiglu", prefix=pre, hidden=H, intermediate=F))
            blocks.append(build_part(
                "block", "sandwich",
                mixer=build_part("mixer", "gqa_attention", prefix=pre, hidden=H, heads=QH, kv_heads=KVH, head_dim=HD,
                                 window=0, position=position, qk_norm_eps=None, output_gate=False),
                feed_forward=ff,
                input_norm=build_part("norm", "rms", name=pre + "n1", width=H, eps=EPS),
                ffn_norm=build_part("norm", "rms", name=pre + "n2", width=H, eps=EPS)))
        return ModelDefinition("toy_routed", V, H, "embed", blocks, [PlanEntry(0, 0), PlanEntry(1, 1)],
                               build_part("norm", "rms", name="nf", width=H, eps=EPS), None)

    register_part("position", "toy_quarter_turn", QuarterTurn, replace=True)
    register_part("feed_forward", "toy_top1", Top1Experts, replace=True)
    register_architecture("toy_routed", Cfg, define, replace=True)
    config = dict(architecture="toy_routed")
    raw = random_tensors(define(Cfg()).tensor_specs(), 21, std=0.3, norm_weights="random")
    assert "l0.router.weight" in raw and "l0.e2.down.weight" in raw
    w = {k: v.double() for k, v in raw.items()}
    model = Model(DecoderModel.from_tensors(config, raw, torch.float32, DEV), max_tokens=512)

    def turn(u, positions, rates):
        ang = positions.double()[:, None, None] * rates.double()[None, None, :]
        a, b = u[..., :HD // 2], u[..., HD // 2:]
        return torch.cat([a * torch.cos(ang) - b * torch.sin(ang), b * torch.cos(ang) + a * torch.sin(ang)], dim=-1)

    def plain(tokens):
        T = len(tokens)
        pos = torch.arange(T)
        h = w["embed"][tokens]
        experts_used = set()
        for l in range(2):
            pre = f"l{l}."
            rates = (QuarterTurn(HD, 0.05).rates() if l == 0
                     else P.rope_frequencies(10000.0, HD, torch.float64))
            n = P.rms_norm(h, w[pre + "n1"], EPS)
            q = turn((n @ w[pre + "attn_q.weight"].T).view(T, QH, HD), pos, rates)
            k = turn((n @ w[pre + "attn_k.weight"].T).view(T, KVH, HD), pos, rates)
            v = (n @ w[pre + "attn_v.weight"].T).view(T, KVH, HD)
            ctx = torch.zeros(T, QH, HD, dtype=torch.float64)
            for hq in range(QH):
                s = (q[:, hq] @ k[:, hq].T) * HD ** -0.5
                s = s.masked_fill(P.attention_mask(T, 0), float("-inf"))
                ctx[:, hq] = torch.softmax(s, -1) @ v[:, hq]
            h = h + ctx.reshape(T, QH * HD) @ w[pre + "attn_output.weight"].T
            n2 = P.rms_norm(h, w[pre + "n2"], EPS)
            if l == 0:
                logits = n2 @ w[pre + "router.weight"].T
                prob, best = torch.softmax(logits, -1), logits.argmax(-1)
                f = torch.zeros_like(n2)
                for t in range(T):
                    e = int(best[t])
                    experts_used.add(e)
                    g, u = n2[t] @ w[f"{pre}e{e}.gate.weight"].T, n2[t] @ w[f"{pre}e{e}.up.weight"].T
                    f[t] = ((g * torch.sigmoid(g) * u) @ w[f"{pre}e{e}.down.weight"].T) * prob[t, e]
                h = h + f
            else:
                h = h + P.swiglu_ffn(n2, {k2[len(pre):]: v2 for k2, v2 in w.items() if k2.startswith(pre)})
        return P.rms_norm(h, w["nf"], EPS) @ w["embed"].T, experts_used

    eng = model.engine
    assert not eng.use_graphs
    seqs = [[(7 * i + 3) % V for i in range(14)], [5, 11, 2]]
    refs = [plain(s) for s in seqs]
    assert len(refs[0][1]) >= 2                                   # the router really spreads tokens over experts
    slots = eng.admit(2)
    got = [[], []]
    out = eng.step(slots, [seqs[0][:9], seqs[1][:2]], [list(range(9)), [0, 1]])
    got[0].append(out[:9].clone())
    got[1].append(out[9:].clone())
    out = eng.step(slots, [[seqs[0][9]], [seqs[1][2]]])
    got[0].append(out[0:1].clone())
    got[1].append(out[1:2].clone())
    eng.release([slots[1]])
    for t in range(10, 14):
        got[0].append(eng.step([slots[0]], [[seqs[0][t]]]).clone())
    eng.release([slots[0]])
    for g, (ref, _) in zip(got, refs):
        torch.testing.assert_close(torch.cat(g).double().cpu(), ref, rtol=3e-5, atol=3e-5)


def test_a_block_without_a_pre_norm_interleaved_pairs_and_scales_around_the_stack():
    """What an architecture may want that LFM3 does not have, added from outside the package: a block
    arrangement in which mixer and feed-forward both read one norm of the residual stream and the block
    names no input norm of its own (the blocks around it then neither make nor expect one), a position
    encoding that pairs neighbouring elements (2i, 2i + 1), a factor on the embeddings, a factor and a
    soft cap on the logits.  Prompt, decode (replayed from a recording) and append steps against plain
    torch in float64."""
    from catena_models_b200 import kernels, register_architecture, register_part
    from catena_models_b200.api import Model
    from catena_models_b200.config.base import Reader
    from catena_models_b200.engine.definition import ModelDefinition, PlanEntry
    from catena_models_b200.engine.model import DecoderModel
    from catena_models_b200.parts import build_part
    from catena_models_b200.parts.base import Block, Position
    from catena_models_b200.weights.random_init import random_tensors

    H, QH, KVH, HD, F, V, EPS, TAPS = 48, 3, 1, 16, 72, 90, 1e-5, 3
    EMB, LSCALE, CAP, THETA = 8.0, 0.75, 4.0, 100.0

    class PairTurn(Position):
        pairing = "interleaved"
        prompt_capturable = True
        supports_append = True

        def __init__(self, head_dim, theta):
            self.head_dim, self.theta = head_dim, theta

        def rates(self):
            i = torch.arange(self.head_dim // 2, dtype=torch.float32)
            return torch.pow(torch.tensor(self.theta, dtype=torch.float32), -2 * i / self.head_dim)

        def bind(self, tensors, rt):
            self._table = self.rates().to(rt.device)

        def rate_table(self):
            return self._table

    class ParallelBlock(Block):
        """h <- h + mixer(norm(h)) + feed_forward(norm(h)); no input norm that others would have to make."""
        prompt_capturable = True
        supports_append = True
        input_norm = None

        def __init__(self, norm, mixer, feed_forward):
            self.norm, self.mixer, self.feed_forward = norm, mixer, feed_forward

        def children(self):
            return [self.norm, self.mixer, self.feed_forward]

        def state_spec(self):
            return self.mixer.state_spec()

        def forward(self, rt, batch, h, n, state, next_norm):
            assert n is None
            x = self.norm.apply(rt, h)
            m = self.mixer.forward(rt, batch, x, state)
            f = self.feed_forward.forward(rt, batch, x)
            kernels.add_norm(h, None, m, h, None, None, 0.0, 0.0)
            kernels.add_norm(h, None, f, h, None, None, 0.0, 0.0)
            return h, None

    class Cfg:
        @classmethod
        def from_dict(cls, data, where="config.json"):
            r = Reader(data, where)
            r.string("architecture")
            r.finish()
            return cls()

    def define(cfg):
        norm = lambda name: build_part("norm", "rms", name=name, width=H, eps=EPS)
        attn = lambda pre: build_part("mixer", "gqa_attention", prefix=pre, hidden=H, heads=QH, kv_heads=KVH, head_dim=HD,
                                      window=0, position=build_part("position", "toy_pair_turn", head_dim=HD, theta=THETA),
                                      qk_norm_eps=EPS, output_gate=False)
        ffn = lambda pre: build_part("feed_forward", "swiglu", prefix=pre, hidden=H, intermediate=F)
        blocks = [
            build_part("block", "toy_parallel", norm=norm("l0.n"), mixer=attn("l0."), feed_forward=ffn("l0.")),
            build_part("block", "sandwich", mixer=build_part("mixer", "short_conv", prefix="l1.", hidden=H, taps=TAPS),
                       feed_forward=ffn("l1."), input_norm=norm("l1.n1"), ffn_norm=norm("l1.n2")),
            build_part("block", "toy_parallel", norm=norm("l2.n"), mixer=attn("l2."), feed_forward=ffn("l2.")),
        ]
        return ModelDefinition("toy_parallel", V, H, "embed", blocks, [PlanEntry(i, i) for i in range(3)],
                               norm("nf"), None, embedding_scale=EMB, logit_scale=LSCALE, logit_softcap=CAP)

    register_part("position", "toy_pair_turn", PairTurn, replace=True)
    register_part("block", "toy_parallel", ParallelBlock, replace=True)
    register_architecture("toy_parallel", Cfg, define, replace=True)
    raw = random_tensors(define(Cfg()).tensor_specs(), 31, std=0.3, norm_weights="random")
    w = {k: v.double() for k, v in raw.items()}
    rates = PairTurn(HD, THETA).rates().double()

    def turn(u, positions):                                     # pairs (2i, 2i + 1)
        ang = positions.double()[:, None, None] * rates[None, None, :]
        a, b = u[..., 0::2], u[..., 1::2]
        out = torch.empty_like(u)
        out[..., 0::2] = a * torch.cos(ang) - b * torch.sin(ang)
        out[..., 1::2] = b * torch.cos(ang) + a * torch.sin(ang)
        return out

    def attention(pre, n):
        T = n.shape[0]
        pos = torch.arange(T)
        q = P.rms_norm((n @ w[pre + "attn_q.weight"].T).view(T, QH, HD), w[pre + "attn_q_norm.weight"], EPS)
        k = P.rms_norm((n @ w[pre + "attn_k.weight"].T).view(T, KVH, HD), w[pre + "attn_k_norm.weight"], EPS)
        q, k = turn(q, pos), turn(k, pos)
        v = (n @ w[pre + "attn_v.weight"].T).view(T, KVH, HD)
        ctx = torch.zeros(T, QH, HD, dtype=torch.float64)
        for hq in range(QH):
            s = (q[:, hq] @ k[:, 0].T) * HD ** -0.5
            s = s.masked_fill(P.attention_mask(T, 0), float("-inf"))
            ctx[:, hq] = torch.softmax(s, -1) @ v[:, 0]
        return ctx.reshape(T, QH * HD) @ w[pre + "attn_output.weight"].T

    def sub(pre):
        return {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)}

    def plain(tokens):
        h = w["embed"][tokens] * EMB
        for l in (0, 2):
            if l == 2:                                          # the sandwich block with the convolution in between
                n1 = P.rms_norm(h, w["l1.n1"], EPS)
                h = h + P.shortconv_mixer(n1, sub("l1."), dict(conv_L_cache=TAPS))
                h = h + P.swiglu_ffn(P.rms_norm(h, w["l1.n2"], EPS), sub("l1."))
            n = P.rms_norm(h, w[f"l{l}.n"], EPS)
            h = h + attention(f"l{l}.", n) + P.swiglu_ffn(n, sub(f"l{l}."))
        logits = (P.rms_norm(h, w["nf"], EPS) @ w["embed"].T) * LSCALE
        return CAP * torch.tanh(logits / CAP)

    seqs = [[(5 * i + 1) % V for i in range(30)], [7, 3, 80, 2, 9]]
    refs = [plain(s) for s in seqs]
    assert float(refs[0].abs().max()) > 0.5 * CAP               # the cap really bends the logits
    for dtype, tol in ((torch.float32, 5e-5), (torch.bfloat16, 0.08)):
        model = Model(DecoderModel.from_tensors(dict(architecture="toy_parallel"), raw, dtype, DEV), max_tokens=512)
        eng = model.engine
        assert eng.use_graphs and model.decoder.supports_append and not model.decoder.fusable_decode
        slots = eng.admit(2)
        got = [[], []]
        out = eng.step(slots, [seqs[0][:12], seqs[1][:2]], [list(range(12)), [0, 1]])
        got[0].append(out[:12].clone())
        got[1].append(out[12:].clone())
        out = eng.step(slots, [seqs[0][12:20], seqs[1][2:3]], [list(range(8)), [0]])        # an append step
        got[0].append(out[:8].clone())
        got[1].append(out[8:].clone())
        for t in range(2):                                      # decode steps: the second one replays the recording
            out = eng.step(slots, [[seqs[0][20 + t]], [seqs[1][3 + t]]])
            got[0].append(out[0:1].clone())
            got[1].append(out[1:2].clone())
        eng.release([slots[1]])
        for t in range(22, 30):
            got[0].append(eng.step([slots[0]], [[seqs[0][t]]]).clone())
        eng.release([slots[0]])
        for g, ref in zip(got, refs):
            err = float((torch.cat(g).double().cpu() - ref).abs().max() / ref.abs().max())
            assert err < tol, (dtype, err)
