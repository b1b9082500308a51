"""Plain, slow LFM3 decoder: the oracle every engine test is compared with.

This file rests on the formulas of hellas-ai/catena-models only: its LFM3 model is a
rendered Hex program (src/lfm3.rs) that needs the project's own compiler and a GPU, so
none of it can be imported or compiled on a CPU.  Each function below restates one part
and cites the file:line (paths inside the catena-models project) it was read from.

Whole sequences, no cache, no batching, one function per part, float64 by default.  It
shares no code with the product path: it reads the model folder with the `safetensors`
package and a plain `json.load`.

`bf16=True` inserts the reference's round-to-bfloat16 points (every activation that
crosses one of its kernel boundaries is stored in bfloat16, src/weights.rs:213-221); the
default leaves every one of them out, which is the exact-arithmetic form of the model.
"""
from __future__ import annotations

import json
import math
import os

import torch


# --------------------------------------------------------------------------- helpers
def _identity(x):
    return x


def _round_bf16(x):
    """Round to nearest even bfloat16 and widen again (src/weights.rs:213-221)."""
    return x.to(torch.float32).to(torch.bfloat16).to(x.dtype)


def load_folder(folder, dtype=torch.float64):
    """Read config.json and model.safetensors of a model folder into (dict, dict)."""
    from safetensors.torch import load_file

    with open(os.path.join(folder, "config.json")) as fh:
        config = json.load(fh)
    tensors = {k: v.to(dtype) for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    return config, tensors


def layer_kind(config, l):
    """conv / full_attention / sliding_attention of layer l (src/spec.rs:277-286)."""
    return config["layer_types"][l]


def head_dim(config):
    """attention.key_length, else hidden / heads (src/checkpoint.rs:422-625)."""
    return config.get("head_dim") or config["hidden_size"] // config["num_attention_heads"]


# ----------------------------------------------------------------------------- parts
def embedding(E, tokens):
    """h0[t,:] = E[tok[t],:], no scaling (src/catena/qwen35_prefill.hex:79-90, src/lfm3.rs:349)."""
    return E[torch.as_tensor(tokens, dtype=torch.long)]


def rms_norm(x, w, eps, r=_identity):
    """inv = 1/sqrt(mean(x^2)+eps); y = r((x*inv)*w): the product with w comes before the
    single rounding (src/catena/qwen35.hex:912-946, src/catena/fused_normalization.hex:23-39)."""
    inv = 1.0 / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return r((x * inv) * w)


def rope_frequencies(theta, hd, dtype):
    """theta^(-2i/HD) for i < HD/2, computed in float32 powf on the host and then used as
    float32 constants (src/catena.rs:185-204)."""
    out = []
    for i in range(hd // 2):
        exponent = torch.tensor((2 * i), dtype=torch.float32) / torch.tensor(hd, dtype=torch.float32)
        out.append(torch.pow(torch.tensor(theta, dtype=torch.float32), -exponent))
    return torch.stack(out).to(dtype)


def rope(u, positions, theta, factors, sliding, exact32=False):
    """Rotate-half over the whole head (src/catena/lfm3.hex:706-746).

    a = f32(p) * (theta^(-2i/HD) / fac_i); fac_i = rope_freqs[i] on full layers and 1 on
    sliding layers, which also use their own theta (src/catena/lfm3.hex:726-739).
    o_i = u_i cos a - u_{i+HD/2} sin a ;  o_{i+HD/2} = u_{i+HD/2} cos a + u_i sin a.
    u: [T, heads, HD]; positions: [T].
    """
    hd = u.shape[-1]
    half = hd // 2
    freq = rope_frequencies(theta, hd, torch.float32)
    fac = torch.ones(half, dtype=torch.float32) if sliding else factors.to(torch.float32)
    rate = freq / fac                                   # float32 division, as the kernel does
    pos = torch.as_tensor(positions, dtype=torch.float32)
    angle = (pos[:, None] * rate[None, :])              # float32 product, as the kernel does
    angle = angle.to(u.dtype)
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    lo, hi = u[..., :half], u[..., half:]
    return torch.cat([lo * cos - hi * sin, hi * cos + lo * sin], dim=-1)


def attention_mask(T, window):
    """Key k is hidden from query p when k > p, or when window > 0 and k + window <= p
    (src/catena/lfm3.hex:48-57): sliding layers see keys p-window+1 .. p."""
    p = torch.arange(T)[:, None]
    k = torch.arange(T)[None, :]
    hidden = k > p
    if window > 0:
        hidden = hidden | (k + window <= p)
    return hidden


def attention_mixer(n, w, config, kind, r=_identity):
    """GQA attention with QK-RMSNorm, RoPE, causal or sliding mask and a per-head sigmoid
    output gate (src/lfm3.rs:390-464; src/catena/lfm3.hex:622-781, 25-46;
    src/catena/qwen35_wmma_attention.hex:3-22 scale/round/mask, 188-258 softmax;
    src/catena/qwen35_exact_attention.hex:3-57 PV)."""
    T, _ = n.shape
    QH, KVH, HD = config["num_attention_heads"], config["num_key_value_heads"], head_dim(config)
    eps = config["norm_eps"]
    sliding = kind == "sliding_attention"
    q = r(n @ w["attn_q.weight"].T).view(T, QH, HD)
    k = r(n @ w["attn_k.weight"].T).view(T, KVH, HD)
    v = r(n @ w["attn_v.weight"].T).view(T, KVH, HD)
    # per-head RMSNorm, rounded before the rotation (src/catena/lfm3.hex:693-704, 735-746)
    q = rms_norm(q, w["attn_q_norm.weight"], eps, r)
    k = rms_norm(k, w["attn_k_norm.weight"], eps, r)
    theta = config.get("rope_theta_sliding", config["rope_theta"]) if sliding else config["rope_theta"]
    pos = torch.arange(T)
    q = r(rope(q, pos, theta, w["rope_freqs.weight"], sliding))
    k = r(rope(k, pos, theta, w["rope_freqs.weight"], sliding))
    scale = float(torch.tensor(1.0, dtype=torch.float32) / torch.sqrt(torch.tensor(float(HD), dtype=torch.float32)))
    hidden = attention_mask(T, config["sliding_window"] if sliding else 0)
    group = QH // KVH
    ctx = torch.zeros(T, QH, HD, dtype=n.dtype)
    for hq in range(QH):
        hk = hq // group                                   # GQA: q-head h uses kv-head h/(QH/KVH)
        s = r((q[:, hq, :] @ k[:, hk, :].T) * scale)
        s = s.masked_fill(hidden, float("-inf"))
        p = r(torch.softmax(s, dim=-1))
        ctx[:, hq, :] = p @ v[:, hk, :]
    if config.get("attn_output_gate", True):
        g = r(n @ w["attn_gate.weight"].T)                 # [T, QH]: one scalar per token per head
        ctx = ctx * torch.sigmoid(g)[:, :, None]           # src/catena/lfm3.hex:25-46
    ctx = r(ctx).reshape(T, QH * HD)
    return r(ctx @ w["attn_output.weight"].T)


def shortconv_mixer(n, w, config, r=_identity):
    """Gated short convolution (src/lfm3.rs:784-812; src/catena/lfm3.hex:3-23, 905-921,
    982-1046, 1105-1114).  in_proj rows are B | C | X; bx = B*X stays unrounded float32;
    z[t,c] = sum_j w_conv[c,j] * s[t+j,c] over s = concat(zeros[K-1,H], bx), so tap K-1
    multiplies the current token; y = r(z*C); out = r(y @ W_out^T)."""
    T, H = n.shape
    K = config["conv_L_cache"]
    bcx = r(n @ w["shortconv.in_proj.weight"].T)
    B, C, X = bcx[:, :H], bcx[:, H:2 * H], bcx[:, 2 * H:]
    bx = B * X
    s = torch.cat([torch.zeros(K - 1, H, dtype=n.dtype), bx], dim=0)
    z = torch.zeros(T, H, dtype=n.dtype)
    for j in range(K):
        z = z + w["shortconv.conv.weight"][:, j][None, :] * s[j:j + T]
    y = r(z * C)
    return r(y @ w["shortconv.out_proj.weight"].T)


def swiglu_ffn(n2, w, r=_identity):
    """g = r(n2 Wg^T), u = r(n2 Wu^T); a = r((g*sigmoid(g))*u); f = r(a Wd^T)
    (src/catena/lfm3.hex:833-845; src/catena/lfm3_wmma.hex:10790-10815)."""
    g = r(n2 @ w["ffn_gate.weight"].T)
    u = r(n2 @ w["ffn_up.weight"].T)
    a = r((g * torch.sigmoid(g)) * u)
    return r(a @ w["ffn_down.weight"].T)


def block(h, w, config, kind, r=_identity):
    """n = RMS(h; attn_norm) -> m = Mixer(n) -> h = r(h + r(RMS(m; post_attention_norm)))
    -> n2 = RMS(h; ffn_norm) -> f = FFN(n2) -> h = r(h + r(RMS(f; post_ffw_norm)))
    (src/spec.rs:722-735; src/lfm3.rs:361-501; src/catena/lfm3.hex:466-574).
    With post_norm off the two post-norms are left out (h = r(h + m))."""
    eps = config["norm_eps"]
    post = config.get("post_norm", True)
    n = rms_norm(h, w["attn_norm.weight"], eps, r)
    m = shortconv_mixer(n, w, config, r) if kind == "conv" else attention_mixer(n, w, config, kind, r)
    h = r(h + (rms_norm(m, w["post_attention_norm.weight"], eps, r) if post else m))
    n2 = rms_norm(h, w["ffn_norm.weight"], eps, r)
    f = swiglu_ffn(n2, w, r)
    return r(h + (rms_norm(f, w["post_ffw_norm.weight"], eps, r) if post else f))


def layer_weights(tensors, l):
    """The tensors of layer l without their `model.layers.{l}.` prefix (src/spec.rs:428-441);
    rope_freqs.weight is global (src/spec.rs:789-794)."""
    prefix = f"model.layers.{l}."
    out = {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}
    out["rope_freqs.weight"] = tensors["rope_freqs.weight"]
    return out


def lm_head_weight(config, tensors):
    """Tied head = the embedding matrix (src/spec.rs:796-806)."""
    if config.get("tie_word_embeddings", True):
        return tensors["model.embed_tokens.weight"]
    return tensors["lm_head.weight"]


def forward(config, tensors, tokens, bf16=False):
    """Logits [T, V] of one whole sequence (src/lfm3.rs:333-524 in order)."""
    r = _round_bf16 if bf16 else _identity
    h = embedding(tensors["model.embed_tokens.weight"], tokens)
    for l in config.get("layer_order", range(config["num_hidden_layers"])):     # the order of layers is data
        h = block(h, layer_weights(tensors, l), config, layer_kind(config, l), r)
    n = rms_norm(h, tensors["model.norm.weight"], config["norm_eps"], r)
    return n @ lm_head_weight(config, tensors).T          # logits stay unrounded in this build


# -------------------------------------------------------------------------- sampling
def argmax_first(logits):
    """Strict '>' scan: the lowest index wins ties (src/catena/fused_argmax.hex:1-24, 93-104)."""
    best, arg = -math.inf, 0
    for i, x in enumerate(logits.tolist()):
        if x > best:
            best, arg = x, i
    return arg


_M64 = (1 << 64) - 1


def _mix64(z):
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def uniform_draw(seed, sequence, step):
    """The engine's counter-based uniform in [0,1): three rounds of the splitmix64 finaliser
    over (seed, sequence id, step), top 24 bits.  catena-models samples greedily only
    (src/server/api.rs:170-177), so this generator is this build's own definition."""
    z = _mix64(seed & _M64)
    z = _mix64(z ^ (sequence & _M64))
    z = _mix64(z ^ (step & _M64))
    return (z >> 40) / float(1 << 24)


def sample_temperature(logits, temperature, u):
    """softmax(logits / temperature), then the first index whose running sum exceeds
    u * total (inverse CDF, index order)."""
    x = logits.to(torch.float64) / temperature
    p = torch.exp(x - x.max())
    cdf = torch.cumsum(p, dim=0)
    target = u * float(cdf[-1])
    idx = int(torch.searchsorted(cdf, torch.tensor(target, dtype=torch.float64), right=True))
    return min(idx, logits.numel() - 1)


def generate(config, tensors, prompt, max_new_tokens, temperature=0.0, seed=0, sequence=0,
             stop_token_ids=(), bf16=False):
    """Prefill, then one token at a time, re-running the whole sequence each time; the first
    new token comes from the prompt's last position; stops after a stop token unless there is
    none (src/main.rs:311-347)."""
    tokens, new = list(prompt), []
    for step in range(max_new_tokens):
        logits = forward(config, tensors, tokens, bf16=bf16)[-1]
        if temperature == 0.0:
            tok = argmax_first(logits)
        else:
            tok = sample_temperature(logits, temperature, uniform_draw(seed, sequence, step))
        tokens.append(tok)
        new.append(tok)
        if tok in stop_token_ids:
            break
    return new
