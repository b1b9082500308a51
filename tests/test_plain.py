"""The plain implementation checked against itself: properties that follow from the formulas."""
import math

import pytest
import torch

import plain_lfm3 as P
import tiny


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("plain")
    return {n: P.load_folder(tiny.make_folder(tmp, n, seed=2)) for n in ("A", "B")}


def test_causal_prefix_property(models):
    for name, (cfg, t) in models.items():
        toks = tiny.random_prompt(30, cfg["vocab_size"], 3)
        whole = P.forward(cfg, t, toks)
        part = P.forward(cfg, t, toks[:19])
        assert torch.allclose(whole[:19], part, atol=1e-12)


def test_mask_edges():
    hidden = P.attention_mask(6, 3)
    assert hidden[5].tolist() == [True, True, True, False, False, False]     # keys p-2 .. p
    assert hidden[1].tolist() == [False, False, True, True, True, True]
    assert not P.attention_mask(4, 0).tril().any()


def test_sliding_window_ignores_far_tokens(models):
    cfg, t = models["B"]                          # window 8 in the sliding layer, but full layers see all
    only_sliding = dict(cfg, layer_types=["conv", "conv", "sliding_attention", "conv", "sliding_attention", "sliding_attention"])
    toks = tiny.random_prompt(40, cfg["vocab_size"], 4)
    other = list(toks)
    other[0] = (other[0] + 1) % cfg["vocab_size"]
    a, b = P.forward(only_sliding, t, toks), P.forward(only_sliding, t, other)
    # receptive field per layer: conv 3 back, sliding 7 back -> 3+3+7+3+7+7 = 30
    assert torch.equal(a[31:], b[31:]) and not torch.equal(a[30], b[30])


def test_rope_is_a_rotation_and_uses_factors():
    u = torch.randn(5, 2, 16, dtype=torch.float64)
    fac = torch.linspace(1, 4, 8, dtype=torch.float64)
    out = P.rope(u, torch.arange(5), 1e4, fac, sliding=False)
    assert torch.allclose(out.norm(dim=-1), u.norm(dim=-1))
    assert torch.equal(out[0], u[0])                                         # position 0: identity
    same = P.rope(u, torch.arange(5), 1e4, torch.ones(8, dtype=torch.float64), sliding=False)
    assert torch.equal(P.rope(u, torch.arange(5), 1e4, fac, sliding=True), same)   # sliding ignores the factors
    assert not torch.allclose(out[3], same[3])
    # pair i turns by pos * theta^(-2i/HD) / fac_i
    e = torch.zeros(1, 1, 16, dtype=torch.float64)
    e[0, 0, 2] = 1.0
    r = P.rope(e, torch.tensor([3]), 1e4, fac, sliding=False)[0, 0]
    angle = 3 * (1e4 ** (-4 / 16)) / float(fac[2])
    assert math.isclose(float(r[2]), math.cos(angle), rel_tol=1e-6) and math.isclose(float(r[10]), math.sin(angle), rel_tol=1e-6)


def test_rms_norm_and_bf16_rounding():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    y = P.rms_norm(x, torch.tensor([2.0, 1.0], dtype=torch.float64), 0.0)
    assert torch.allclose(y, torch.tensor([[6.0, 4.0]], dtype=torch.float64) / math.sqrt(12.5))
    assert float(P._round_bf16(torch.tensor(1.00390625, dtype=torch.float64))) == 1.0     # ties to even
    assert float(P._round_bf16(torch.tensor(1.01171875, dtype=torch.float64))) == 1.015625


def test_conv_taps_and_gate_order():
    cfg = dict(conv_L_cache=3)
    H = 2
    w = {"shortconv.in_proj.weight": torch.eye(6, 2, dtype=torch.float64) * 0, "shortconv.out_proj.weight": torch.eye(2, dtype=torch.float64),
         "shortconv.conv.weight": torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]], dtype=torch.float64)}
    # rows of in_proj: B (0,1), C (2,3), X (4,5).  B = x0, C = 1 via x1, X = x0 -> bx = x0^2 on channel 0
    w["shortconv.in_proj.weight"][0, 0] = 1.0
    w["shortconv.in_proj.weight"][2, 1] = 1.0
    w["shortconv.in_proj.weight"][4, 0] = 1.0
    n = torch.tensor([[1.0, 1.0], [2.0, 1.0], [3.0, 1.0]], dtype=torch.float64)
    out = P.shortconv_mixer(n, w, cfg)
    # bx on channel 0 = 1, 4, 9; the last tap multiplies the current token
    assert out[:, 0].tolist() == [100.0, 410.0, 941.0]


def test_argmax_ties_and_sampler():
    assert P.argmax_first(torch.tensor([1.0, 3.0, 3.0, 2.0])) == 1
    logits = torch.log(torch.tensor([0.1, 0.2, 0.3, 0.4], dtype=torch.float64))
    assert [P.sample_temperature(logits, 1.0, u) for u in (0.0, 0.05, 0.11, 0.29, 0.31, 0.61, 0.99)] == [0, 0, 1, 1, 2, 3, 3]
    cold = [P.sample_temperature(logits, 0.01, u) for u in (0.1, 0.5, 0.9)]
    assert cold == [3, 3, 3]
    us = [P.uniform_draw(1, s, t) for s in range(3) for t in range(3)]
    assert len(set(us)) == 9 and all(0.0 <= u < 1.0 for u in us)
    assert P.uniform_draw(1, 2, 3) == P.uniform_draw(1, 2, 3) != P.uniform_draw(2, 2, 3)


def test_generate_stops(models):
    cfg, t = models["A"]
    free = P.generate(cfg, t, [1, 2, 3], 6)
    assert len(free) == 6
    stopped = P.generate(cfg, t, [1, 2, 3], 6, stop_token_ids=(free[2],))
    assert stopped == free[:free.index(free[2]) + 1]
