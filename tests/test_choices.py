"""The runtime's choices of tile width and of runs of K for the tiled product are arithmetic over the
shape and the number of SMs; here for a B200's 148 SMs, against what was measured to be the best or
within a few per cent of it (the figures stand in the docstrings of the two methods)."""
from catena_models_b200.engine.runtime import Runtime


def _runtime(sms=148):
    rt = Runtime.__new__(Runtime)          # the arithmetic needs no device
    rt._sm_count, rt._choices = sms, {}
    return rt


def test_tile_width_follows_rounds_over_the_sms():
    rt = _runtime()
    assert rt._tile_width(2048, 6144) == 256        # 384 tiles, three rounds: the wide tile's rounds are the cheapest
    assert rt._tile_width(1024, 6144) == 192        # 256 tiles of 192 in two rounds beat 192 tiles of 256 in two
    assert rt._tile_width(512, 6144) == 192         # one round of 128 tiles
    assert rt._tile_width(256, 6144) == 128         # everything runs at once: the narrow tile's step is the shortest
    assert rt._tile_width(2048, 2048) == 256
    assert rt._tile_width(2048, 16384, (256, 128)) == 256
    assert rt._tile_width(2048, 3104) == 192
    assert rt._tile_width(1024, 6144, (256, 128)) == 256     # a product that cannot take 192 (SwiGLU, float output)


def test_runs_of_k_fill_one_round_and_shrink_with_the_rows():
    rt = _runtime()
    assert rt._tiled_slices(256, 2048, 2048) == (4, 128)
    assert rt._tiled_slices(256, 2048, 8192) == (8, 256)
    assert rt._tiled_slices(512, 2048, 8192) == (4, 256)
    assert rt._tiled_slices(1024, 2048, 8192) == (2, 256)
    assert rt._tiled_slices(1024, 2048, 2048)[0] == 1        # two short runs do not repay the float sums
    assert rt._tiled_slices(2048, 2048, 8192)[0] == 1        # 128 tiles fill the round by themselves
    assert rt._tiled_slices(512, 2050, 8192)[0] == 1         # float rows of a run must stay 16-byte aligned
    for rows in (160, 448, 640, 1000, 1280):
        for cols, inner in ((2048, 2048), (2048, 8192), (1024, 4608), (2048, 10752), (1024, 1024)):
            runs, width = rt._tiled_slices(rows, cols, inner)
            steps = -(-inner // 64)
            per = -(-steps // runs)
            assert 1 <= runs <= 8 and width in (128, 256)
            assert runs == 1 or (per >= 2 and per * (runs - 1) < steps)      # no run without a k-slice


def test_fewer_sms_fewer_runs():
    assert _runtime(32)._tiled_slices(512, 2048, 8192)[0] <= _runtime(148)._tiled_slices(512, 2048, 8192)[0]


def _attention_choice(monkeypatch, lens, window, dtype="bfloat16", HD=64):
    """Which prompt-attention kernel the runtime calls for a step of sequences of these lengths."""
    import types
    import torch
    from catena_models_b200.engine import runtime as R

    called = []
    for name in ("attn_prefill_tc", "attn_prefill_mma", "attn_prefill_simt"):
        monkeypatch.setattr(R.kernels, name, lambda *a, _n=name, **k: called.append(_n))
    rt = _runtime()
    rt.tensor_core_prompts, rt.error_flag = True, None
    T, QH, KVH = sum(lens), 4, 2
    buf = torch.zeros(T, (QH + 2 * KVH) * HD, dtype=getattr(torch, dtype))
    q, k, v = buf[:, :QH * HD], buf[:, QH * HD:(QH + KVH) * HD], buf[:, (QH + KVH) * HD:]
    ctx = torch.zeros(T, QH * HD, dtype=buf.dtype)
    batch = types.SimpleNamespace(max_len=max(lens), B=len(lens), seq_start=None)
    rt.attention_prefill(ctx, q, k, v, None, batch, QH, KVH, HD, window, 1.0)
    assert len(called) == 1
    return called[0]


def test_prompt_attention_goes_to_tcgen05_from_768_tokens_or_with_many_rows(monkeypatch):
    assert _attention_choice(monkeypatch, [767], 0) == "attn_prefill_mma"
    assert _attention_choice(monkeypatch, [768], 0) == "attn_prefill_tc"
    assert _attention_choice(monkeypatch, [1500], 512) == "attn_prefill_mma"          # the window is what a row sees
    assert _attention_choice(monkeypatch, [1500], 768) == "attn_prefill_tc"
    assert _attention_choice(monkeypatch, [4096], 512) == "attn_prefill_tc"           # ... unless the step has 2,048 rows
    assert _attention_choice(monkeypatch, [4096], 192) == "attn_prefill_mma"
    assert _attention_choice(monkeypatch, [256] * 8, 0) == "attn_prefill_tc"          # 2,048 rows of 256 and more
    assert _attention_choice(monkeypatch, [256] * 7, 0) == "attn_prefill_mma"
    assert _attention_choice(monkeypatch, [255] * 64, 0) == "attn_prefill_mma"
    assert _attention_choice(monkeypatch, [2048] * 4, 256) == "attn_prefill_tc"
    assert _attention_choice(monkeypatch, [2048], 0, HD=128) == "attn_prefill_tc"
    assert _attention_choice(monkeypatch, [2048], 0, HD=96) == "attn_prefill_mma"     # other multiples of 16 up to 128
    assert _attention_choice(monkeypatch, [2048], 0, HD=192) == "attn_prefill_simt"
    assert _attention_choice(monkeypatch, [2048], 0, dtype="float32") == "attn_prefill_simt"
