"""Each CUDA kernel alone against a plain PyTorch float32/float64 statement of the same
operation, at sizes other than the engine's (odd widths, row counts that fill no tile)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1e-2)


def close(got, ref, dtype, **kw):
    t = tol(dtype)
    t.update(kw)
    torch.testing.assert_close(got.float().cpu(), ref.float().cpu(), **t)


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.fixture(scope="module")
def K():
    from catena_models_b200 import kernels
    kernels.lib()
    return kernels


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_gather_and_bad_token(K, dtype):
    table = rnd(37, 24, dtype=dtype)
    tokens = torch.tensor([0, 36, 5, 5, 99, -1], dtype=torch.int32, device=DEV)
    out = torch.empty(6, 24, dtype=dtype, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    K.embed_gather(out, table, tokens, err)
    assert torch.equal(out[:4], table[[0, 36, 5, 5]])
    assert int(err) == 1 and float(out[4:].abs().sum()) == 0.0          # refused ids: zeros and a flag, no fault
    # a table stored in the other type is converted row by row as it is read
    other = torch.float32 if dtype == torch.bfloat16 else torch.bfloat16
    table2 = rnd(37, 24, dtype=other, seed=1)
    K.embed_gather(out, table2, tokens[:4], err)
    assert torch.equal(out[:4], table2[[0, 36, 5, 5]].to(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,H", [(1, 8), (5, 200), (3, 1000), (2, 2056)])
def test_rmsnorm(K, dtype, rows, H):
    x, w = rnd(rows, H, dtype=dtype, scale=3.0), 1 + 0.1 * rnd(H)
    y = torch.empty_like(x)
    K.rmsnorm(y, x, w, 1e-3)
    xf = x.double()
    ref = xf / torch.sqrt((xf * xf).mean(-1, keepdim=True) + 1e-3) * w.double()
    close(y, ref, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,H", [(7, 328), (301, 328), (258, 2048), (1500, 2048), (1100, 2568), (1030, 4104)])
@pytest.mark.parametrize("post,nxt", [(True, True), (False, True), (True, False), (False, False)])
def test_add_norm(K, dtype, post, nxt, rows, H):
    """A few rows, a few hundred and more than a thousand; widths that take one, two and four chunks
    of a thread."""
    m, h = rnd(rows, H, dtype=dtype, scale=2.0, seed=1), rnd(rows, H, dtype=dtype, seed=2)
    wp, wn = 1 + 0.1 * rnd(H, seed=3), 1 + 0.1 * rnd(H, seed=4)
    h_out, n_out = torch.empty_like(h), torch.empty_like(h)
    K.add_norm(h_out, n_out if nxt else None, m, h, wp if post else None, wn if nxt else None, 1e-5, 1e-6)

    def rms(v, w, eps):
        return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * w.double()

    d = rms(m.double(), wp, 1e-5) if post else m.double()
    if dtype == torch.bfloat16 and post:
        d = d.to(torch.bfloat16).double()
    href = h.double() + d
    close(h_out, href, dtype)
    if nxt:
        close(n_out, rms(h_out.double(), wn, 1e-6), dtype)            # over the stored sum, as the kernel does
    # in place on the residual stream
    h2 = h.clone()
    K.add_norm(h2, None, m, h2, wp if post else None, None, 1e-5, 0.0)
    assert torch.equal(h2, h_out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,H,slices", [(3, 64, 1), (700, 1544, 3), (1500, 2048, 2), (2500, 264, 8), (600, 4104, 4)])
def test_add_norm_over_partial_sums_with_more_rows_than_blocks(K, dtype, rows, H, slices):
    """Over partial sums the kernel's blocks walk rows, a fixed number of blocks per SM, with the next row's
    loads in flight: fewer rows than blocks, about as many, and several rows a block; the result must be the
    bits of add_norm over the rounded total."""
    parts = rnd(slices, rows, H, seed=5)
    h = rnd(rows, H, dtype=dtype, seed=6)
    wp, wn = 1 + 0.1 * rnd(H, seed=3), 1 + 0.1 * rnd(H, seed=4)
    total = torch.zeros(rows, H, device=DEV)
    for r in range(slices):
        total += parts[r]                                            # index order, in float
    m = total.to(dtype)
    h_a, n_a, h_b, n_b = (torch.empty_like(h) for _ in range(4))
    K.add_norm(h_a, n_a, K.PartialSums(parts, dtype), h, wp, wn, 1e-5, 1e-6)
    K.add_norm(h_b, n_b, m, h, wp, wn, 1e-5, 1e-6)
    assert torch.equal(h_a, h_b) and torch.equal(n_a, n_b)
    h2 = h.clone()                                                   # in place on the residual stream, no norms
    K.add_norm(h2, None, K.PartialSums(parts, dtype), h2, None, None, 0.0, 0.0)
    assert torch.equal(h2, (h.float() + m.float()).to(dtype))


@pytest.mark.parametrize("M,N,Kin,slices", [(1, 48, 256, 4), (8, 2048, 2048, 4), (13, 200, 1000, 3), (16, 72, 8192, 8),
                                            (5, 40, 64, 2)])
def test_gemm_skinny_parts_and_add_norm_over_them(K, M, N, Kin, slices):
    """The weight-streaming product cut over K into float partial sums, and the fused residual
    kernel that adds them: each slice against the float64 product over its own k range (the kernel's
    rule: k-blocks of 32 dealt out evenly), the total against the whole product, and add_norm over
    the slices against add_norm over the rounded total (the same bits: it adds the slices in order
    and rounds once, as the product's own store would)."""
    x = rnd(M, Kin, dtype=torch.bfloat16, seed=1)
    w = rnd(N, Kin, dtype=torch.bfloat16, scale=Kin ** -0.5, seed=2)
    parts = torch.full((slices, M, N), float("nan"), device=DEV)
    K.gemm_skinny_parts(parts, x, w)
    nblk = (Kin + 31) // 32
    per = (nblk + slices - 1) // slices
    xd, wd = x.double().cpu(), w.double().cpu()
    for s_ in range(slices):
        k0, k1 = min(Kin, s_ * per * 32), min(Kin, (s_ + 1) * per * 32)
        torch.testing.assert_close(parts[s_].double().cpu(), xd[:, k0:k1] @ wd[:, k0:k1].T, rtol=1e-4, atol=1e-4)
    total = parts[0].clone()
    for s_ in range(1, slices):
        total += parts[s_]
    m = total.to(torch.bfloat16)
    h = rnd(M, N, dtype=torch.bfloat16, seed=3)
    if N % 8 == 0:
        wp, wn = 1 + 0.1 * rnd(N, seed=4), 1 + 0.1 * rnd(N, seed=5)
        h_a, n_a, h_b, n_b = (torch.empty_like(h) for _ in range(4))
        K.add_norm(h_a, n_a, K.PartialSums(parts, torch.bfloat16), h, wp, wn, 1e-5, 1e-6)
        K.add_norm(h_b, n_b, m, h, wp, wn, 1e-5, 1e-6)
        assert torch.equal(h_a, h_b) and torch.equal(n_a, n_b)
        h_c = torch.empty_like(h)
        K.add_norm(h_c, None, K.PartialSums(parts, torch.bfloat16), h, None, None, 0.0, 0.0)
        assert torch.equal(h_c, (h.float() + m.float()).to(torch.bfloat16))
    with pytest.raises(K.KernelError):
        K.gemm_skinny_parts(torch.empty(2, 17, N, device=DEV), torch.zeros(17, Kin, dtype=torch.bfloat16, device=DEV), w)


@pytest.mark.parametrize("M,N,Kin,slices", [(17, 2048, 2048, 8), (64, 200, 1000, 3), (128, 136, 8192, 8), (100, 2052, 512, 2),
                                            (33, 72, 192, 1)])
def test_gemm_tc_few_rows_parts(K, M, N, Kin, slices):
    """The tcgen05 few-rows product cut over K into float partial sums without the exchange
    between the blocks of a tile: each slice against the float64 product over its own k range
    (64-wide steps dealt out evenly), widths that end inside a tile or are no multiple of 4, and
    add_norm over the slices against add_norm over the rounded total."""
    x = rnd(M, Kin, dtype=torch.bfloat16, seed=1)
    w = rnd(N, Kin, dtype=torch.bfloat16, scale=Kin ** -0.5, seed=2)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    parts = torch.full((slices, M, N), float("nan"), device=DEV)
    K.gemm_tc_few_rows_parts(parts, x, w, err=err)
    assert int(err) == 0
    steps = (Kin + 63) // 64
    per = (steps + slices - 1) // slices
    xd, wd = x.double().cpu(), w.double().cpu()
    for s_ in range(slices):
        k0, k1 = min(Kin, s_ * per * 64), min(Kin, (s_ + 1) * per * 64)
        torch.testing.assert_close(parts[s_].double().cpu(), xd[:, k0:k1] @ wd[:, k0:k1].T, rtol=1e-4, atol=1e-4)
    if N % 8 == 0:
        total = parts[0].clone()
        for s_ in range(1, slices):
            total += parts[s_]
        m = total.to(torch.bfloat16)
        h = rnd(M, N, dtype=torch.bfloat16, seed=3)
        wp, wn = 1 + 0.1 * rnd(N, seed=4), 1 + 0.1 * rnd(N, seed=5)
        h_a, n_a, h_b, n_b = (torch.empty_like(h) for _ in range(4))
        K.add_norm(h_a, n_a, K.PartialSums(parts, torch.bfloat16), h, wp, wn, 1e-5, 1e-6)
        K.add_norm(h_b, n_b, m, h, wp, wn, 1e-5, 1e-6)
        assert torch.equal(h_a, h_b) and torch.equal(n_a, n_b)
    with pytest.raises(K.KernelError):
        K.gemm_tc_few_rows_parts(torch.empty(4, M, N, device=DEV), x[:, :64].contiguous(), w[:, :64].contiguous(), err=err)


@pytest.mark.parametrize("block_n", [128, 256])
@pytest.mark.parametrize("M,N,Kin,slices", [(200, 2048, 2048, 4), (333, 104, 520, 3), (1024, 264, 1096, 2), (129, 516, 8192, 8),
                                            (640, 2048, 448, 7), (300, 72, 192, 1)])
def test_gemm_tc_parts(K, M, N, Kin, slices, block_n):
    """The tiled tcgen05 product cut over K into float runs (work items of the persistent kernel): each
    run against the float64 product over its own k range, with row counts that end inside a row tile
    (the run below begins right there: such tiles are stored from registers, whole ones by TMA),
    widths that end inside a column tile, an inner size that ends inside a 64-wide step, and
    add_norm over the runs against add_norm over the rounded total."""
    x = rnd(M, Kin, dtype=torch.bfloat16, seed=1)
    w = rnd(N, Kin, dtype=torch.bfloat16, scale=Kin ** -0.5, seed=2)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    guard = torch.full((slices * M * N + 512,), float("nan"), device=DEV)
    parts = guard[:slices * M * N].view(slices, M, N)
    K.gemm_tc_parts(parts, x, w, err=err, block_n=block_n)
    assert int(err) == 0
    assert bool(guard[slices * M * N:].isnan().all())            # nothing written past the last run
    steps = (Kin + 63) // 64
    per = (steps + slices - 1) // slices
    xd, wd = x.double().cpu(), w.double().cpu()
    for s_ in range(slices):
        k0, k1 = min(Kin, s_ * per * 64), min(Kin, (s_ + 1) * per * 64)
        torch.testing.assert_close(parts[s_].double().cpu(), xd[:, k0:k1] @ wd[:, k0:k1].T, rtol=1e-4, atol=1e-4)
    if N % 8 == 0:
        total = parts[0].clone()
        for s_ in range(1, slices):
            total += parts[s_]
        m = total.to(torch.bfloat16)
        h = rnd(M, N, dtype=torch.bfloat16, seed=3)
        wp, wn = 1 + 0.1 * rnd(N, seed=4), 1 + 0.1 * rnd(N, seed=5)
        h_a, n_a, h_b, n_b = (torch.empty_like(h) for _ in range(4))
        K.add_norm(h_a, n_a, K.PartialSums(parts, torch.bfloat16), h, wp, wn, 1e-5, 1e-6)
        K.add_norm(h_b, n_b, m, h, wp, wn, 1e-5, 1e-6)
        assert torch.equal(h_a, h_b) and torch.equal(n_a, n_b)
    with pytest.raises(K.KernelError):                             # a run without a k-slice
        K.gemm_tc_parts(torch.empty(4, M, N, device=DEV), x[:, :128].contiguous(), w[:, :128].contiguous(), err=err)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_and_gather(K, dtype):
    gu = rnd(5, 2 * 72, dtype=dtype, scale=2.0)
    a = torch.empty(5, 72, dtype=dtype, device=DEV)
    K.swiglu(a, gu)
    g, u = gu[:, :72].double(), gu[:, 72:].double()
    close(a, g * torch.sigmoid(g) * u, dtype)
    x = rnd(9, 40, dtype=dtype)
    rows = torch.tensor([8, 0, 3, 3], dtype=torch.int32, device=DEV)
    out = torch.empty(4, 40, dtype=dtype, device=DEV)
    K.gather_rows(out, x, rows)
    assert torch.equal(out, x[[8, 0, 3, 3]])


@pytest.mark.parametrize("M,N,Kd", [(1, 64, 256), (17, 67, 256), (65, 128, 2048), (3, 5, 8), (130, 70, 24)])
@pytest.mark.parametrize("dtx,dtw,dty", [
    (torch.float32, torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16, torch.bfloat16),
    (torch.bfloat16, torch.bfloat16, torch.float32), (torch.bfloat16, torch.float32, torch.bfloat16)])
def test_gemm_simt(K, M, N, Kd, dtx, dtw, dty):
    x, w = rnd(M, Kd, dtype=dtx, seed=1), rnd(N, Kd, dtype=dtw, scale=0.1, seed=2)
    y = torch.empty(M, N, dtype=dty, device=DEV)
    K.gemm_simt(y, x, w)
    ref = x.double() @ w.double().T
    if dty == torch.float32:
        torch.testing.assert_close(y.double().cpu(), ref.cpu(), rtol=1e-5, atol=1e-5 * math.sqrt(Kd))
    else:
        close(y, ref, torch.bfloat16)


def test_gemm_simt_rows_do_not_depend_on_their_neighbours(K):
    x, w = rnd(70, 96, seed=5), rnd(50, 96, seed=6)
    y = torch.empty(70, 50, device=DEV)
    K.gemm_simt(y, x, w)
    y1 = torch.empty(1, 50, device=DEV)
    K.gemm_simt(y1, x[69:70].contiguous(), w)
    assert torch.equal(y1[0], y[69])                                   # bit-equal: fixed k order per element


@pytest.mark.parametrize("M", [1, 2, 8, 9, 16, 31, 64])
@pytest.mark.parametrize("N,Kd", [(16, 32), (100, 72), (2048, 2048), (24, 8), (515, 1000)])
@pytest.mark.parametrize("dty", [torch.bfloat16, torch.float32])
def test_gemm_skinny(K, M, N, Kd, dty):
    x, w = rnd(M, Kd, dtype=torch.bfloat16, seed=1), rnd(N, Kd, dtype=torch.bfloat16, scale=0.1, seed=2)
    y = torch.full((M, N), float("nan"), dtype=dty, device=DEV)
    K.gemm_skinny(y, x, w)
    ref = x.double() @ w.double().T
    if dty == torch.float32:
        torch.testing.assert_close(y.double().cpu(), ref.cpu(), rtol=2e-5, atol=2e-5 * math.sqrt(Kd))
    else:
        close(y, ref, torch.bfloat16)


@pytest.mark.parametrize("M", [1, 8, 13, 64])
@pytest.mark.parametrize("F,Kd", [(16, 32), (100, 72), (1000, 520)])
def test_gemm_skinny_swiglu(K, M, F, Kd):
    x, w = rnd(M, Kd, dtype=torch.bfloat16, seed=1), rnd(2 * F, Kd, dtype=torch.bfloat16, scale=0.2, seed=2)
    a = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device=DEV)
    K.gemm_skinny(a, x, w, swiglu=True)
    # the scalar form of the reference's own check (tests/lfm3_projections.rs:139-158)
    g = (x.double() @ w[:F].double().T).to(torch.bfloat16).double()
    u = (x.double() @ w[F:].double().T).to(torch.bfloat16).double()
    close(a, g / (1 + torch.exp(-g)) * u, torch.bfloat16, rtol=2e-2)


def test_gemm_skinny_batch_mates_change_nothing(K):
    x, w = rnd(8, 520, dtype=torch.bfloat16, seed=3), rnd(70, 520, dtype=torch.bfloat16, seed=4)
    y8 = torch.empty(8, 70, dtype=torch.float32, device=DEV)
    K.gemm_skinny(y8, x, w)
    y1 = torch.empty(1, 70, dtype=torch.float32, device=DEV)
    K.gemm_skinny(y1, x[5:6].contiguous(), w)
    assert torch.equal(y1[0], y8[5])


def _ref_attention(q, k, v, window, scale, gate=None):
    """float64 softmax attention with GQA, causal or sliding mask and the head gate
    (the form of the reference's own check, tests/lfm3_online_attention.rs:145-181)."""
    T, QH, HD = q.shape
    KVH = k.shape[1]
    out = torch.zeros(T, QH, HD, dtype=torch.float64)
    pos = torch.arange(T)
    hidden = pos[None, :] > pos[:, None]
    if window > 0:
        hidden |= pos[None, :] + window <= pos[:, None]
    for h in range(QH):
        s = (q[:, h].double() @ k[:, h // (QH // KVH)].double().T) * scale
        s = s.masked_fill(hidden, float("-inf"))
        out[:, h] = torch.softmax(s, -1) @ v[:, h // (QH // KVH)].double()
    if gate is not None:
        out = out * torch.sigmoid(gate.double())[:, :, None]
    return out


@pytest.mark.parametrize("dtype,impl", [(torch.float32, "simt"), (torch.bfloat16, "simt"), (torch.bfloat16, "mma")])
@pytest.mark.parametrize("QH,KVH,HD,window,gated", [(4, 2, 16, 0, True), (6, 1, 24, 5, False), (2, 2, 128, 40, True),
                                                    (3, 3, 256, 0, False), (8, 2, 64, 256, True), (4, 4, 48, 70, True),
                                                    (2, 1, 112, 0, False)])
def test_attn_prefill_varlen(K, dtype, impl, QH, KVH, HD, window, gated):
    if impl == "mma" and (HD % 16 or HD > 128):
        with pytest.raises(K.KernelError):                              # refused, not computed wrongly
            K.attn_prefill_mma(torch.empty(1, QH * HD, dtype=dtype, device=DEV), *(torch.empty(1, QH * HD, dtype=dtype, device=DEV),) * 3,
                               None, torch.zeros(2, dtype=torch.int32, device=DEV), 1, 1, QH, KVH, HD, window, 1.0)
        return
    lens = [17, 65, 1, 100]
    T = sum(lens)
    width = (QH * HD + 2 * KVH * HD + (QH if gated else 0) + 7) // 8 * 8
    buf = rnd(T, width, dtype=dtype, seed=HD)
    q, k = buf[:, :QH * HD], buf[:, QH * HD:QH * HD + KVH * HD]
    v = buf[:, QH * HD + KVH * HD:QH * HD + 2 * KVH * HD]
    gate = buf[:, QH * HD + 2 * KVH * HD:QH * HD + 2 * KVH * HD + QH] if gated else None
    starts = torch.tensor([0, 17, 82, 83, 183], dtype=torch.int32, device=DEV)
    ctx = torch.full((T, QH * HD), float("nan"), dtype=dtype, device=DEV)
    scale = HD ** -0.5
    fn = K.attn_prefill_mma if impl == "mma" else K.attn_prefill_simt
    fn(ctx, q, k, v, gate, starts, len(lens), max(lens), QH, KVH, HD, window, scale)
    off = 0
    for n in lens:
        sl = slice(off, off + n)
        ref = _ref_attention(q[sl].cpu().view(n, QH, HD), k[sl].cpu().view(n, KVH, HD), v[sl].cpu().view(n, KVH, HD),
                             window, scale, None if gate is None else gate[sl].cpu())
        close(ctx[sl].view(n, QH, HD), ref, dtype)
        off += n


def _paged_cache(K, kv, KVH, HD, dtype, lens, ring, scramble_seed=0):
    """Put per-sequence keys/values kv[b]: [len, 2, KVH, HD] into a paged pool with shuffled page
    ids the way the engine would (entry = pos, or pos % ring)."""
    pages_per_seq = [((min(n, ring) if ring else n) + 63) // 64 for n in lens]
    total = sum(pages_per_seq) + 3
    perm = torch.randperm(total, generator=torch.Generator().manual_seed(scramble_seed)).tolist()
    pool = torch.full((2, total, KVH, 64, HD), float("nan"), dtype=dtype, device=DEV)
    stride = max(pages_per_seq)
    ptab = torch.full((len(lens) + 2, stride), -1, dtype=torch.int32)
    nxt = 0
    for b, n in enumerate(lens):
        slot = b + 1                                   # slot ids differ from batch order
        for j in range(pages_per_seq[b]):
            ptab[slot, j] = perm[nxt]
            nxt += 1
        first = max(0, n - ring) if ring else 0
        for p in range(first, n):
            e = p % ring if ring else p
            page = int(ptab[slot, e // 64])
            pool[0, page, :, e % 64] = kv[b][p, 0].to(dtype)
            pool[1, page, :, e % 64] = kv[b][p, 1].to(dtype)
    return pool, total, ptab.to(DEV)


@pytest.mark.parametrize("dtype,tensor_cores", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)])
@pytest.mark.parametrize("QH,KVH,HD,window", [(4, 2, 16, 0), (4, 1, 24, 8), (5, 5, 32, 70), (32, 8, 64, 0),
                                              (16, 1, 128, 300), (2, 1, 256, 0), (40, 2, 48, 0)])
def test_attn_decode_paged(K, dtype, tensor_cores, QH, KVH, HD, window):
    K.set_decode_attention_tensor_cores(tensor_cores)
    try:
        _attn_decode_paged(K, dtype, QH, KVH, HD, window)
    finally:
        K.set_decode_attention_tensor_cores(True)


def _attn_decode_paged(K, dtype, QH, KVH, HD, window, lens=(1, 64, 65, 300, 700), n_chunks=4):
    ring = (window + 63) // 64 * 64 if window else 0
    lens = list(lens)                                  # tokens held including the new one
    B = len(lens)
    g = torch.Generator().manual_seed(HD + window)
    kv = [torch.randn(n, 2, KVH, HD, generator=g) for n in lens]
    pool, pages, ptab = _paged_cache(K, kv, KVH, HD, dtype, lens, ring)
    q = rnd(B, QH * HD, dtype=dtype, seed=7)
    gate = rnd(B, QH, dtype=dtype, seed=8)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    slots = torch.arange(1, B + 1, dtype=torch.int32, device=DEV)
    # n_chunks: more chunks than the short sequences have
    part_o, part_ml = K.attn_decode_scratch(B, QH, HD, n_chunks, DEV)
    ctx = torch.full((B, QH * HD), float("nan"), dtype=dtype, device=DEV)
    scale = HD ** -0.5
    K.attn_decode(ctx, q, gate, pos, slots, pool, pages, ptab, ring, window, QH, KVH, HD, n_chunks, scale, part_o, part_ml)
    for b, n in enumerate(lens):
        kk, vv = kv[b][:, 0].to(dtype), kv[b][:, 1].to(dtype)
        qq = torch.zeros(n, QH, HD)
        qq[-1] = q[b].float().cpu().view(QH, HD)
        gg = torch.zeros(n, QH)
        gg[-1] = gate[b].float().cpu()
        ref = _ref_attention(qq, kk, vv, window, scale, gg)[-1]
        close(ctx[b].view(QH, HD), ref, dtype)


@pytest.mark.parametrize("target_blocks", [1, 12, 40])
@pytest.mark.parametrize("QH,KVH,HD,window", [(8, 2, 64, 0), (4, 1, 32, 1000), (6, 2, 128, 1024), (20, 1, 16, 0)])
def test_attn_decode_blocks_that_walk_several_chunks(K, QH, KVH, HD, window, target_blocks):
    """With a small target of blocks every block takes chunks c, c + n_parts, ... of its sequence
    (1: one block per sequence and kv head walks them all), carrying maximum and sum from page to
    page; sequences end inside a page, at a page's edge and at a chunk's edge."""
    K.set_decode_attention_target_blocks(target_blocks)
    try:
        _attn_decode_paged(K, torch.bfloat16, QH, KVH, HD, window, lens=(1, 256, 257, 1024, 1500, 1983), n_chunks=8)
    finally:
        K.set_decode_attention_target_blocks(0)


def test_attn_decode_finds_a_far_key_and_respects_the_window_edge(K):
    """One key far back is made to dominate; it must be found among hundreds when it is inside
    the window and be invisible one step after it leaves."""
    QH = KVH = 1
    HD, n = 16, 500
    for window, far, seen in [(0, 3, True), (200, n - 200, True), (200, n - 201, False)]:
        ring = (window + 63) // 64 * 64 if window else 0
        kv = [torch.randn(n, 2, KVH, HD, generator=torch.Generator().manual_seed(1)) * 0.1]
        kv[0][far, 0, 0] = 0.0
        kv[0][far, 0, 0, 0] = 40.0                     # the key that stands out
        kv[0][far, 1, 0] = 7.0                         # its value
        pool, pages, ptab = _paged_cache(K, kv, KVH, HD, torch.float32, [n], ring)
        q = torch.zeros(1, HD, device=DEV)
        q[0, 0] = 40.0
        pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
        slots = torch.tensor([1], dtype=torch.int32, device=DEV)
        part_o, part_ml = K.attn_decode_scratch(1, QH, HD, 2, DEV)
        ctx = torch.empty(1, HD, device=DEV)
        K.attn_decode(ctx, q, None, pos, slots, pool, pages, ptab, ring, window, QH, KVH, HD, 2, HD ** -0.5, part_o, part_ml)
        if seen:
            assert torch.allclose(ctx.cpu(), torch.full((1, HD), 7.0), atol=1e-3)
        else:
            assert float(ctx.abs().max()) < 1.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("extra", [3, 8])        # 3: rows that 16-byte accesses cannot take; 8: rows they can
@pytest.mark.parametrize("QH,KVH,HD,ring,normed,rotated", [(4, 2, 16, 0, True, True), (3, 1, 24, 64, True, False),
                                                          (2, 2, 128, 0, False, True), (5, 5, 32, 128, True, True),
                                                          (7, 3, 48, 64, True, True), (9, 3, 64, 0, True, True)])
def test_qk_prepare(K, dtype, QH, KVH, HD, ring, normed, rotated, extra):
    lens, pos0 = [5, 150, 1], [0, 0, 0]
    T = sum(lens)
    width = QH * HD + 2 * KVH * HD + extra
    qkv = rnd(T, width, dtype=dtype, seed=ring + HD)
    orig = qkv.clone()
    wq, wk = 1 + 0.1 * rnd(HD, seed=1), 1 + 0.1 * rnd(HD, seed=2)
    rate = (torch.rand(HD // 2, generator=torch.Generator().manual_seed(3)) * 0.5).to(DEV)
    tok_seq = torch.tensor(sum([[b] * n for b, n in enumerate(lens)], []), dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor(sum([list(range(n)) for n in lens], []), dtype=torch.int32, device=DEV)
    slots = torch.tensor([2, 0, 1], dtype=torch.int32, device=DEV)
    seq_end = torch.tensor(lens, dtype=torch.int32, device=DEV)
    pages = 8
    pool = torch.zeros(2, pages, KVH, 64, HD, dtype=dtype, device=DEV)
    ptab = torch.tensor([[3, 1, 6], [0, 7, 7], [5, 7, 7]], dtype=torch.int32, device=DEV)   # by slot
    eps = 1e-5
    K.qk_prepare(qkv, wq if normed else None, wk if normed else None, rate if rotated else None, tok_pos, tok_seq,
                 slots, seq_end, pool, pages, ptab, ring, QH, KVH, HD, eps)

    def prepared(x, w):
        x = x.double()
        if normed:
            x = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w.double().cpu()
            if dtype == torch.bfloat16:
                x = x.to(torch.bfloat16).double()
        if rotated:
            ang = tok_pos.cpu().double()[:, None] * rate.cpu().double()[None, :]
            c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            lo, hi = x[..., :HD // 2], x[..., HD // 2:]
            x = torch.cat([lo * c - hi * s, hi * c + lo * s], -1)
        return x

    o = orig.cpu()
    q_ref = prepared(o[:, :QH * HD].view(T, QH, HD), wq)
    k_ref = prepared(o[:, QH * HD:QH * HD + KVH * HD].view(T, KVH, HD), wk)
    close(qkv[:, :QH * HD].view(T, QH, HD), q_ref, dtype)
    close(qkv[:, QH * HD:QH * HD + KVH * HD].view(T, KVH, HD), k_ref, dtype)
    assert torch.equal(qkv[:, QH * HD + KVH * HD:], orig[:, QH * HD + KVH * HD:])       # v and the rest untouched
    # cache entries of the middle sequence (slot 0: pages 3, 1, 6)
    v_ref = o[:, QH * HD + KVH * HD:QH * HD + 2 * KVH * HD].view(T, KVH, HD)
    first = max(0, 150 - ring) if ring else 0
    for p in (first, 63 if first <= 63 else first, 64 if first <= 64 else first, 149):
        e = p % ring if ring else p
        page = [3, 1, 6][e // 64]
        t = 5 + p
        close(pool[0, page, :, e % 64], k_ref[t], dtype)
        assert torch.equal(pool[1, page, :, e % 64].cpu(), v_ref[t])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,QH,KVH,HD", [(600, 6, 2, 64), (600, 3, 3, 48), (600, 2, 1, 128), (8200, 20, 4, 64)])
def test_qk_prepare_long_prompt_both_access_widths(K, dtype, T, QH, KVH, HD):
    """Prompts long enough for the kernel with 16-byte accesses (the longest also for the form in
    which one warp walks several groups of heads of its token): rows that take such accesses
    against the same values in rows that do not (one channel of padding), which run the
    one-channel-per-lane kernel checked above; cache contents included."""
    pages = (T + 63) // 64
    g = torch.Generator().manual_seed(HD)
    core = torch.randn(T, (QH + 2 * KVH) * HD, generator=g).to(dtype)
    wq, wk = 1 + 0.1 * rnd(HD, seed=1), 1 + 0.1 * rnd(HD, seed=2)
    rate = (torch.rand(HD // 2, generator=g) * 0.5).to(DEV)
    tok_seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    tok_pos = torch.arange(T, dtype=torch.int32, device=DEV)
    slots = torch.tensor([1], dtype=torch.int32, device=DEV)
    seq_end = torch.tensor([T], dtype=torch.int32, device=DEV)
    ptab = torch.stack([torch.zeros(pages, dtype=torch.int32), torch.randperm(pages, generator=g).to(torch.int32)]).to(DEV)
    out = []
    for pad in (8, 1):
        qkv = torch.zeros(T, core.shape[1] + pad, dtype=dtype, device=DEV)
        qkv[:, :core.shape[1]] = core.to(DEV)
        pool = torch.zeros(2, pages, KVH, 64, HD, dtype=dtype, device=DEV)
        K.qk_prepare(qkv, wq, wk, rate, tok_pos, tok_seq, slots, seq_end, pool, pages, ptab, 0, QH, KVH, HD, 1e-6)
        out.append((qkv[:, :core.shape[1]].clone(), pool))
    (a, pool_a), (b, pool_b) = out
    close(a, b, dtype)
    close(pool_a[0], pool_b[0], dtype)
    assert torch.equal(pool_a[1], pool_b[1])                    # the values are copied as they are
    assert pool_a[1].abs().sum() > 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,taps", [(8, 2), (72, 3), (200, 4), (136, 7), (40, 5), (27, 3)])
@pytest.mark.parametrize("longest", [30, 300])       # 300: enough tokens for blocks that cover four tokens each
def test_shortconv_prompt_then_decode(K, dtype, H, taps, longest):
    lens = [1, 2, 9, longest]
    extra = 5
    g = torch.Generator().manual_seed(H)
    w = (torch.randn(H, taps, generator=g) * 0.5).to(DEV)
    seqs = [torch.randn(n + extra, 3 * H, generator=g).to(dtype) for n in lens]
    slots = torch.tensor([3, 0, 2, 1], dtype=torch.int32, device=DEV)
    state = torch.full((5, taps - 1, H), float("nan"), device=DEV)         # stale contents must not matter

    def reference(s):
        s = s.double()
        B_, C_, X_ = s[:, :H], s[:, H:2 * H], s[:, 2 * H:]
        bx = torch.cat([torch.zeros(taps - 1, H, dtype=torch.float64), B_ * X_])
        z = sum(w.cpu().double()[:, j][None, :] * bx[j:j + s.shape[0]] for j in range(taps))
        return z * C_

    bcx = torch.cat([s[:n] for s, n in zip(seqs, lens)]).to(DEV)
    T = bcx.shape[0]
    tok_seq = torch.tensor(sum([[b] * n for b, n in enumerate(lens)], []), dtype=torch.int32, device=DEV)
    starts = torch.tensor([0, 1, 3, 12, 12 + longest], dtype=torch.int32, device=DEV)
    y = torch.empty(T, H, dtype=dtype, device=DEV)
    K.shortconv(y, bcx, w, state, tok_seq, starts, slots, taps, from_zero=True, one_token_each=False)
    got = [[y[a:b]] for a, b in zip(starts.tolist()[:-1], starts.tolist()[1:])]
    dec_seq = torch.arange(4, dtype=torch.int32, device=DEV)
    dec_start = torch.arange(5, dtype=torch.int32, device=DEV)
    for t in range(extra):
        bcx = torch.stack([s[n + t] for s, n in zip(seqs, lens)]).to(DEV)
        y = torch.empty(4, H, dtype=dtype, device=DEV)
        K.shortconv(y, bcx, w, state, dec_seq, dec_start, slots, taps, from_zero=False, one_token_each=True)
        for b in range(4):
            got[b].append(y[b:b + 1].clone())
    for b, s in enumerate(seqs):
        close(torch.cat(got[b]), reference(s), dtype)


@pytest.mark.parametrize("M,H,Kin,taps", [(1, 48, 40, 2), (5, 100, 72, 3), (8, 2048, 2048, 3), (13, 304, 1000, 4),
                                          (16, 64, 4104, 3)])
def test_gemm_skinny_shortconv_matches_the_two_kernels(K, M, H, Kin, taps):
    """in_proj and the decode form of the short convolution in one kernel: several steps on the same
    slots (the state shifts each time), against float64 formulas and against the product followed by
    the convolution kernel; widths that are no multiple of 16, a row count between the kernel's two
    tile heights, an inner size with a ragged last block.
    The fused kernel splits K four ways where the plain product splits it eight ways, so a float sum
    that lies near a bfloat16 rounding boundary may round the other way: B, C and X are each right
    to one bfloat16 step (2^-8 of the value) plus the float summation's own error (1e-5 covers sums
    of this size).  The test carries these per-element error bounds through the formulas (products,
    taps, the state of earlier steps, the output's rounding) instead of using a flat tolerance: a
    flat one would have to be loose enough for the largest element and would then hide a wrong tap
    on a small one."""
    g = torch.Generator().manual_seed(M * 1000 + H)
    w_in = (torch.randn(3 * H, Kin, generator=g) * Kin ** -0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn(H, taps, generator=g) * 0.5).to(DEV)
    slots = torch.randperm(M + 3, generator=g)[:M].to(torch.int32).to(DEV)
    start = torch.randn(M + 3, taps - 1, H, generator=g).to(DEV)
    state_a, state_b = start.clone(), start.clone()
    seq = torch.arange(M, dtype=torch.int32, device=DEV)
    seq_start = torch.arange(M + 1, dtype=torch.int32, device=DEV)
    hist = [start[slots.long()].double().cpu()[:, j] for j in range(taps - 1)]        # per slot: s[0 .. taps-2]
    hist_err = [torch.zeros_like(h) for h in hist]                                    # the given state is exact
    wd = w.double().cpu()
    step_err = lambda v: 2.0 ** -8 * v.abs() + 1e-5
    for step in range(4):
        x = torch.randn(M, Kin, generator=g).to(torch.bfloat16).to(DEV)
        y_a = torch.empty(M, H, dtype=torch.bfloat16, device=DEV)
        K.gemm_skinny_shortconv(y_a, x, w_in, w, state_a, slots)
        bcx = torch.empty(M, 3 * H, dtype=torch.bfloat16, device=DEV)
        K.gemm_skinny(bcx, x, w_in)
        y_b = torch.empty(M, H, dtype=torch.bfloat16, device=DEV)
        K.shortconv(y_b, bcx, w, state_b, seq, seq_start, slots, taps, from_zero=False, one_token_each=True)
        r = (x.double().cpu() @ w_in.double().cpu().T).to(torch.bfloat16).double()   # the product, rounded once
        B_, C_, X_ = r[:, :H], r[:, H:2 * H], r[:, 2 * H:]
        dB, dC, dX = step_err(B_), step_err(C_), step_err(X_)
        hist.append(B_ * X_)
        hist_err.append(B_.abs() * dX + X_.abs() * dB + dB * dX)
        z = sum(wd[:, j][None, :] * hist[j] for j in range(taps))
        dz = sum(wd[:, j].abs()[None, :] * hist_err[j] for j in range(taps)) + 1e-6 * sum(
            wd[:, j].abs()[None, :] * hist[j].abs() for j in range(taps))
        hist.pop(0)
        hist_err.pop(0)
        ref = z * C_
        bound = C_.abs() * dz + z.abs() * dC + dz * dC + 2.0 ** -8 * ref.abs() + 1e-30
        for name, y in (("fused", y_a), ("two kernels", y_b)):
            excess = ((y.double().cpu() - ref).abs() / bound).max()
            assert excess <= 1.0, f"{name}, step {step}: {float(excess):.2f} of the bound"
        for st in (state_a, state_b):
            new = st[slots.long()].double().cpu()
            for j in range(taps - 1):
                assert ((new[:, j] - hist[j]).abs() <= hist_err[j] + 1e-30).all(), f"state entry {j}, step {step}"
        assert (y_a != y_b).float().mean() < 0.02, "the two paths differ in more than stray roundings"
    untouched = [s for s in range(M + 3) if s not in slots.tolist()]
    assert torch.equal(state_a[untouched], start[untouched])
    with pytest.raises(K.KernelError):
        K.gemm_skinny_shortconv(torch.empty(17, H, dtype=torch.bfloat16, device=DEV),
                                torch.zeros(17, Kin, dtype=torch.bfloat16, device=DEV), w_in, w, state_a,
                                torch.zeros(17, dtype=torch.int32, device=DEV))


def test_sample_greedy_ties_and_temperature(K):
    import plain_lfm3 as P

    V = 1000
    logits = rnd(6, V, scale=2.0, seed=4)
    logits[0, 17] = logits[0, 400] = logits[0].max() + 1.0                 # a tie: the lower index wins
    logits[1, V - 1] = 50.0
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    temp = torch.tensor([0.0, 0.0, 0.8, 0.8, 1.5, 0.8], device=DEV)
    seq = torch.tensor([0, 1, 2, 3, 4, 2], dtype=torch.int32, device=DEV)
    step = torch.tensor([0, 0, 5, 5, 9, 5], dtype=torch.int32, device=DEV)
    seed = 0x1234567890ABCDEF
    words = torch.tensor([seed & 0xFFFFFFFF, seed >> 32], dtype=torch.int64).to(torch.int32).to(DEV)
    K.sample(out, logits, temp, seq, step, words)
    got = out.tolist()
    assert got[0] == 17 and got[1] == V - 1
    for r in (2, 3, 4):
        u = P.uniform_draw(seed, int(seq[r]), int(step[r]))
        x = logits[r].double().cpu() / float(temp[r])
        cdf = torch.cumsum(torch.exp(x - x.max()), 0)
        target = u * float(cdf[-1])
        lo = float(cdf[got[r] - 1]) if got[r] > 0 else 0.0
        slack = 1e-4 * float(cdf[-1])
        assert lo - slack <= target <= float(cdf[got[r]]) + slack           # the drawn index holds u
    # rows 2 and 5 differ only in their logits' row: same key -> same uniform
    many = torch.empty(4000, dtype=torch.int32, device=DEV)
    flat = torch.log(torch.tensor([0.1, 0.2, 0.3, 0.4], device=DEV)).repeat(4000, 1).contiguous()
    K.sample(many, flat, torch.full((4000,), 1.0, device=DEV), torch.arange(4000, dtype=torch.int32, device=DEV),
             torch.zeros(4000, dtype=torch.int32, device=DEV), words)
    freq = torch.bincount(many.cpu().long(), minlength=4).double() / 4000
    assert torch.allclose(freq, torch.tensor([0.1, 0.2, 0.3, 0.4], dtype=torch.float64), atol=0.03)


def test_refusals_are_errors_not_wrong_results(K):
    x = torch.zeros(2, 12, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(K.KernelError):
        K.gemm_skinny(torch.empty(2, 4, dtype=torch.bfloat16, device=DEV), x, torch.zeros(4, 12, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(K.KernelError):
        K.gemm_skinny(torch.empty(70, 4, dtype=torch.bfloat16, device=DEV), torch.zeros(70, 16, dtype=torch.bfloat16, device=DEV),
                      torch.zeros(4, 16, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(K.KernelError):
        K.rmsnorm(torch.empty(2, 4), torch.empty(2, 4), torch.ones(4), 1e-5)     # CPU tensors


@pytest.mark.parametrize("M,N,Kd", [(128, 128, 64), (100, 70, 72), (1, 8, 8), (257, 384, 520), (2048, 2048, 2048),
                                     (65, 3104, 2048), (300, 200, 1000)])
@pytest.mark.parametrize("dty,block_n", [(torch.bfloat16, 256), (torch.bfloat16, 192), (torch.bfloat16, 128),
                                         (torch.float32, 128)])
def test_gemm_tc(K, M, N, Kd, dty, block_n):
    """tcgen05/TMA GEMM: shapes that fill no tile in any dimension, K with a ragged last k-slice."""
    x, w = rnd(M, Kd, dtype=torch.bfloat16, seed=1), rnd(N, Kd, dtype=torch.bfloat16, scale=0.1, seed=2)
    y = torch.full((M, N), float("nan"), dtype=dty, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    K.gemm_tc(y, x, w, err=err, block_n=block_n)
    ref = x.double() @ w.double().T
    assert int(err) == 0
    if dty == torch.float32:
        torch.testing.assert_close(y.double().cpu(), ref.cpu(), rtol=2e-5, atol=2e-5 * math.sqrt(Kd))
    else:
        close(y, ref, torch.bfloat16)


@pytest.mark.parametrize("block_n", [128, 256])
@pytest.mark.parametrize("M,F,Kd", [(128, 64, 64), (200, 136, 520), (70, 1000, 264)])
def test_gemm_tc_swiglu(K, M, F, Kd, block_n):
    x, w = rnd(M, Kd, dtype=torch.bfloat16, seed=1), rnd(2 * F, Kd, dtype=torch.bfloat16, scale=0.2, seed=2)
    a = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    K.gemm_tc(a, x, w, swiglu=True, err=err, block_n=block_n)
    g = (x.double() @ w[:F].double().T).to(torch.bfloat16).double()
    u = (x.double() @ w[F:].double().T).to(torch.bfloat16).double()
    assert int(err) == 0
    close(a, g / (1 + torch.exp(-g)) * u, torch.bfloat16, rtol=2e-2)


@pytest.mark.parametrize("splits", [0, 1, 2, 3, 5, 8])
@pytest.mark.parametrize("M,N,Kd,dty", [(64, 2048, 2048, torch.bfloat16), (17, 200, 520, torch.bfloat16),
                                        (128, 130, 1096, torch.bfloat16), (33, 384, 4096, torch.float32),
                                        (100, 70, 72, torch.float32)])
def test_gemm_tc_few_rows(K, M, N, Kd, dty, splits):
    """K split over a cluster: every number of blocks (a share of k-slices may be empty or ragged),
    rows and columns that fill no tile."""
    x, w = rnd(M, Kd, dtype=torch.bfloat16, seed=1), rnd(N, Kd, dtype=torch.bfloat16, scale=0.1, seed=2)
    ybuf = torch.full((M, N + 8), float("nan"), dtype=dty, device=DEV)
    y = ybuf[:, :N]
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    K.gemm_tc_few_rows(y, x, w, err=err, splits=splits)
    ref = x.double() @ w.double().T
    assert int(err) == 0
    assert bool(torch.isnan(ybuf[:, N:]).all())
    if dty == torch.float32:
        torch.testing.assert_close(y.double().cpu(), ref.cpu(), rtol=2e-5, atol=2e-5 * math.sqrt(Kd))
    else:
        close(y, ref, torch.bfloat16)


@pytest.mark.parametrize("splits", [0, 1, 4, 7])
@pytest.mark.parametrize("M,F,Kd", [(64, 64, 64), (40, 136, 520), (128, 1000, 2048)])
def test_gemm_tc_few_rows_swiglu(K, M, F, Kd, splits):
    x, w = rnd(M, Kd, dtype=torch.bfloat16, seed=1), rnd(2 * F, Kd, dtype=torch.bfloat16, scale=0.2, seed=2)
    a = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    K.gemm_tc_few_rows(a, x, w, swiglu=True, err=err, splits=splits)
    g = (x.double() @ w[:F].double().T).to(torch.bfloat16).double()
    u = (x.double() @ w[F:].double().T).to(torch.bfloat16).double()
    assert int(err) == 0
    close(a, g / (1 + torch.exp(-g)) * u, torch.bfloat16, rtol=2e-2)


def test_gemm_tc_few_rows_refuses_more_rows(K):
    x, w = rnd(129, 64, dtype=torch.bfloat16), rnd(64, 64, dtype=torch.bfloat16)
    with pytest.raises(Exception, match="rows"):
        K.gemm_tc_few_rows(torch.empty(129, 64, dtype=torch.bfloat16, device=DEV), x, w)


def test_gemm_tc_strided_operands(K):
    """A is a column block of a wider buffer (the attention context inside qkv-sized rows)."""
    buf = rnd(150, 96 + 40, dtype=torch.bfloat16, seed=3)
    x = buf[:, 8:8 + 96]
    w = rnd(50, 96, dtype=torch.bfloat16, scale=0.1, seed=4)
    ybuf = torch.zeros(150, 64, dtype=torch.bfloat16, device=DEV)
    y = ybuf[:, :50]
    K.gemm_tc(y, x, w)
    close(y, x.double() @ w.double().T, torch.bfloat16)
    assert float(ybuf[:, 50:].abs().sum()) == 0.0


@pytest.mark.parametrize("window", [0, 100])
def test_attn_prefill_mma_long_and_window_edge(K, window):
    """700 queries (many key tiles, first and last tiles ragged); one key is made to dominate and
    must be seen by exactly the queries whose window holds it."""
    QH, KVH, HD, T = 2, 1, 64, 700
    buf = rnd(T, QH * HD + 2 * KVH * HD, dtype=torch.bfloat16, scale=0.3, seed=11)
    far = 250
    buf[far, QH * HD:QH * HD + HD] = 0
    buf[far, QH * HD] = 30.0                       # the key
    buf[:, 0] = 30.0                               # every query of head 0 looks for it
    q, k, v = buf[:, :QH * HD], buf[:, QH * HD:QH * HD + HD], buf[:, QH * HD + HD:]
    starts = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    ctx = torch.empty(T, QH * HD, dtype=torch.bfloat16, device=DEV)
    K.attn_prefill_mma(ctx, q, k, v, None, starts, 1, T, QH, KVH, HD, window, HD ** -0.5)
    ref = _ref_attention(q.cpu().view(T, QH, HD), k.cpu().view(T, KVH, HD), v.cpu().view(T, KVH, HD), window, HD ** -0.5)
    close(ctx.view(T, QH, HD), ref, torch.bfloat16)
    hit = (ctx.view(T, QH, HD)[:, 0].float() - v[far].float()).abs().max(dim=-1).values < 0.05
    expect = torch.arange(T, device=DEV) >= far
    if window:
        expect &= torch.arange(T, device=DEV) < far + window
    assert torch.equal(hit, expect)


@pytest.mark.parametrize("QH,KVH,HD,window,gated", [(8, 2, 64, 0, True), (4, 4, 64, 300, False), (2, 1, 128, 0, True),
                                                    (4, 2, 128, 130, True), (3, 1, 64, 128, False)])
def test_attn_prefill_tc_varlen(K, QH, KVH, HD, window, gated):
    """tcgen05 prefill attention: packed sequences that end inside a tile, at a tile's edge and
    after several tiles, so that the last tile of one runs into the next one's rows."""
    lens = [17, 128, 1, 129, 700, 256]
    T = sum(lens)
    width = (QH * HD + 2 * KVH * HD + (QH if gated else 0) + 7) // 8 * 8
    buf = rnd(T, width, dtype=torch.bfloat16, seed=HD + window)
    q, k = buf[:, :QH * HD], buf[:, QH * HD:QH * HD + KVH * HD]
    v = buf[:, QH * HD + KVH * HD:QH * HD + 2 * KVH * HD]
    gate = buf[:, QH * HD + 2 * KVH * HD:QH * HD + 2 * KVH * HD + QH] if gated else None
    bounds = [0]
    for n in lens:
        bounds.append(bounds[-1] + n)
    starts = torch.tensor(bounds, dtype=torch.int32, device=DEV)
    ctx = torch.full((T, QH * HD), float("nan"), dtype=torch.bfloat16, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = HD ** -0.5
    K.attn_prefill_tc(ctx, q, k, v, gate, starts, len(lens), max(lens), QH, KVH, HD, window, scale, err=err)
    assert int(err) == 0
    for b, n in enumerate(lens):
        sl = slice(bounds[b], bounds[b] + n)
        ref = _ref_attention(q[sl].cpu().view(n, QH, HD), k[sl].cpu().view(n, KVH, HD), v[sl].cpu().view(n, KVH, HD),
                             window, scale, None if gate is None else gate[sl].cpu())
        close(ctx[sl].view(n, QH, HD), ref, torch.bfloat16)


@pytest.mark.parametrize("impl", ["tc", "mma", "simt"])
@pytest.mark.parametrize("HD", [64, 128])
def test_attn_prefill_is_not_spoilt_by_a_batch_mate(K, HD, impl):
    """The tcgen05 kernel copies whole 128-row tiles of keys and values, so the last tile of a sequence
    holds rows of the sequence packed behind it (the other kernels read no row that no query sees).  That
    one's keys and values are NaN and infinite here; the sequences before it must come out as if it
    were not there (its own rows may be anything)."""
    QH, KVH = 4, 2
    lens = [70, 200, 129, 60]
    T = sum(lens)
    buf = rnd(T, QH * HD + 2 * KVH * HD, dtype=torch.bfloat16, seed=HD)
    q, k = buf[:, :QH * HD], buf[:, QH * HD:QH * HD + KVH * HD]
    v = buf[:, QH * HD + KVH * HD:]
    bounds = [0, 70, 270, 399, 459]
    bad = slice(bounds[2], bounds[3])                  # the third sequence is broken
    k[bad] = float("inf")
    v[bad] = float("nan")
    starts = torch.tensor(bounds, dtype=torch.int32, device=DEV)
    ctx = torch.full((T, QH * HD), float("nan"), dtype=torch.bfloat16, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    if impl == "tc":
        K.attn_prefill_tc(ctx, q, k, v, None, starts, len(lens), max(lens), QH, KVH, HD, 0, HD ** -0.5, err=err)
    else:
        fn = K.attn_prefill_mma if impl == "mma" else K.attn_prefill_simt
        fn(ctx, q, k, v, None, starts, len(lens), max(lens), QH, KVH, HD, 0, HD ** -0.5)
    assert int(err) == 0
    for b in (0, 1, 3):
        n, sl = lens[b], slice(bounds[b], bounds[b + 1])
        ref = _ref_attention(q[sl].cpu().view(n, QH, HD), k[sl].cpu().view(n, KVH, HD), v[sl].cpu().view(n, KVH, HD),
                             0, HD ** -0.5, None)
        close(ctx[sl].view(n, QH, HD), ref, torch.bfloat16)


@pytest.mark.parametrize("window", [0, 100])
def test_attn_prefill_tc_far_key_and_window_edge(K, window):
    """One key is made to dominate and must be seen by exactly the queries whose window holds it."""
    QH, KVH, HD, T = 2, 1, 64, 700
    buf = rnd(T, QH * HD + 2 * KVH * HD, dtype=torch.bfloat16, scale=0.3, seed=11)
    far = 250
    buf[far, QH * HD:QH * HD + HD] = 0
    buf[far, QH * HD] = 30.0                       # the key
    buf[:, 0] = 30.0                               # every query of head 0 looks for it
    q, k, v = buf[:, :QH * HD], buf[:, QH * HD:QH * HD + HD], buf[:, QH * HD + HD:]
    starts = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    ctx = torch.empty(T, QH * HD, dtype=torch.bfloat16, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    K.attn_prefill_tc(ctx, q, k, v, None, starts, 1, T, QH, KVH, HD, window, HD ** -0.5, err=err)
    assert int(err) == 0
    ref = _ref_attention(q.cpu().view(T, QH, HD), k.cpu().view(T, KVH, HD), v.cpu().view(T, KVH, HD), window, HD ** -0.5)
    close(ctx.view(T, QH, HD), ref, torch.bfloat16)
    hit = (ctx.view(T, QH, HD)[:, 0].float() - v[far].float()).abs().max(dim=-1).values < 0.05
    expect = torch.arange(T, device=DEV) >= far
    if window:
        expect &= torch.arange(T, device=DEV) < far + window
    assert torch.equal(hit, expect)


@pytest.mark.parametrize("HD", [64, 128])
@pytest.mark.parametrize("slope", [0.004, 0.012, 0.035])
def test_attn_prefill_tc_maxima_that_grow_tile_after_tile(K, HD, slope):
    """The kernel keeps its sums in tensor memory relative to a reference maximum that it moves only when
    a row's maximum has grown by more than a factor of 256, rescaling the sums then.  Scores that rise
    with the key's position make every row's maximum grow from tile to tile: slowly (the reference is
    moved every few tiles), faster (every other tile) or by more than the threshold in every tile."""
    QH, KVH, T = 2, 1, 1500
    buf = rnd(T, QH * HD + 2 * KVH * HD, dtype=torch.bfloat16, scale=0.3, seed=HD)
    buf[:, 0] = HD ** 0.5                                          # query component 0, so that the score is k[p, 0] + noise
    buf[:, HD] = HD ** 0.5
    buf[:, QH * HD] = (slope * torch.arange(T, device=DEV)).to(torch.bfloat16)
    q, k, v = buf[:, :QH * HD], buf[:, QH * HD:QH * HD + HD], buf[:, QH * HD + HD:]
    starts = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    ctx = torch.empty(T, QH * HD, dtype=torch.bfloat16, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    K.attn_prefill_tc(ctx, q, k, v, None, starts, 1, T, QH, KVH, HD, 0, HD ** -0.5, err=err)
    assert int(err) == 0
    ref = _ref_attention(q.cpu().view(T, QH, HD), k.cpu().view(T, KVH, HD), v.cpu().view(T, KVH, HD), 0, HD ** -0.5)
    close(ctx.view(T, QH, HD), ref, torch.bfloat16)


@pytest.mark.parametrize("seed,QH,KVH,HD,window", [(1, 8, 2, 64, 0), (2, 6, 3, 64, 200), (3, 4, 1, 128, 0), (4, 4, 2, 128, 64),
                                                   (5, 16, 8, 64, 64)])
def test_attn_prefill_tc_many_short_and_long_items(K, seed, QH, KVH, HD, window):
    """The kernel's blocks walk items (query tile, head, sequence) one after another with rings, tensor-memory
    buffers and barrier phases that run on across their borders.  Batches of 30 to 60 sequences of 1 to 700
    rows give every block dozens of items of one to six key tiles in a row, among them many of a single tile
    and sequences that are over before a block's share begins; compared with the float64 reference."""
    import random
    rng = random.Random(seed)
    lens = [rng.choice([1, 2, 63, 64, 65, 127, 128, 129, 130, rng.randint(1, 700)]) for _ in range(rng.randint(30, 60))]
    T = sum(lens)
    width = (QH * HD + 2 * KVH * HD + QH + 7) // 8 * 8
    buf = rnd(T, width, dtype=torch.bfloat16, seed=seed)
    q, k = buf[:, :QH * HD], buf[:, QH * HD:QH * HD + KVH * HD]
    v = buf[:, QH * HD + KVH * HD:QH * HD + 2 * KVH * HD]
    gate = buf[:, QH * HD + 2 * KVH * HD:QH * HD + 2 * KVH * HD + QH]
    bounds = [0]
    for n in lens:
        bounds.append(bounds[-1] + n)
    starts = torch.tensor(bounds, dtype=torch.int32, device=DEV)
    ctx = torch.full((T, QH * HD), float("nan"), dtype=torch.bfloat16, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = HD ** -0.5
    for _ in range(3):                                  # the same launch again: nothing may be left over from the last
        K.attn_prefill_tc(ctx, q, k, v, gate, starts, len(lens), max(lens), QH, KVH, HD, window, scale, err=err)
    assert int(err) == 0
    qc, kc, vc, gc = q.cpu(), k.cpu(), v.cpu(), gate.cpu()
    for b, n in enumerate(lens):
        sl = slice(bounds[b], bounds[b] + n)
        ref = _ref_attention(qc[sl].view(n, QH, HD), kc[sl].view(n, KVH, HD), vc[sl].view(n, KVH, HD), window, scale, gc[sl])
        close(ctx[sl].view(n, QH, HD), ref, torch.bfloat16)


def test_attn_prefill_tc_refuses_other_head_sizes(K):
    x = torch.empty(4, 96, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(K.KernelError, match="head size"):
        K.attn_prefill_tc(x, x, x, x, None, torch.zeros(2, dtype=torch.int32, device=DEV), 1, 4, 1, 1, 96, 0, 1.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_copy_pages(K, dtype):
    """Pages of a paged pool copied to other pages in every layer and plane; the rest untouched."""
    layers, pages, kvh, hd = 3, 11, 2, 24
    pool = rnd(layers, 2, pages, kvh, 64, hd, dtype=dtype, seed=5)
    before = pool.clone()
    src = torch.tensor([7, 0, 3], dtype=torch.int32, device=DEV)
    dst = torch.tensor([1, 10, 5], dtype=torch.int32, device=DEV)
    K.copy_pages(pool, src, dst)
    expect = before.clone()
    expect[:, :, dst.long()] = before[:, :, src.long()]
    assert torch.equal(pool, expect)


def test_more_tokens_than_a_grid_dimension_holds(K):
    """A prompt step may carry more than 65,535 tokens (64 prompts of 2,048): the per-token kernels
    must not put the token index on a grid axis that ends there."""
    T, H, taps = 70000, 8, 3
    bcx = rnd(T, 3 * H, dtype=torch.bfloat16, seed=1)
    w = rnd(H, taps, seed=2)
    state = torch.zeros(1, taps - 1, H, device=DEV)
    tok_seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    starts = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    y = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    K.shortconv(y, bcx, w, state, tok_seq, starts, torch.zeros(1, dtype=torch.int32, device=DEV), taps, True, False)
    b, c, x = bcx[:, :H].float(), bcx[:, H:2 * H].float(), bcx[:, 2 * H:].float()
    bx = torch.cat([torch.zeros(taps - 1, H, device=DEV), b * x])
    z = sum(w[:, j][None, :] * bx[j:j + T] for j in range(taps))
    close(y[-5:], (z * c)[-5:], torch.bfloat16)
    QH, KVH, HD = 2, 1, 16
    qkv = rnd(T, (QH + 2 * KVH) * HD, dtype=torch.bfloat16, seed=3)
    orig = qkv.clone()
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    rate = torch.full((HD // 2,), 0.001, device=DEV)
    K.qk_prepare(qkv, None, None, rate, pos, tok_seq, torch.zeros(1, dtype=torch.int32, device=DEV),
                 torch.tensor([T], dtype=torch.int32, device=DEV), None, 0, None, 0, QH, KVH, HD, 0.0)
    t = T - 1
    ang = t * 0.001
    lo, hi = orig[t, :HD // 2].float(), orig[t, HD // 2:HD].float()
    ref = torch.cat([lo * math.cos(ang) - hi * math.sin(ang), hi * math.cos(ang) + lo * math.sin(ang)])
    close(qkv[t, :HD], ref, torch.bfloat16)


@pytest.mark.parametrize("dtype", DTYPES)
def test_zero_slots_clears_the_named_rows_of_every_layer(K, dtype):
    """Fixed-size states [layers, slots, ...]: 70 slots in one call (two launches of at most 64),
    every other row untouched; a slot outside the storage is refused."""
    store = rnd(3, 90, 2, 10, dtype=dtype)
    before = store.clone()
    slots = [5, 0, 89] + list(range(10, 77))
    K.zero_slots(store, slots)
    keep = torch.ones(90, dtype=torch.bool)
    keep[slots] = False
    assert float(store[:, slots].abs().sum()) == 0.0
    assert torch.equal(store[:, keep], before[:, keep])
    with pytest.raises(K.KernelError):
        K.zero_slots(store, [90])


@pytest.mark.parametrize("M", [1, 8, 13, 16])
def test_fused_decode_segment_runs_collected_calls_in_order(K, M):
    """Products in all four output forms at sizes that fill no tile or stage, the residual + norm
    operation over partial sums and over a finished product, and the short convolution's decode form,
    collected and run by the persistent kernel in one launch; every result against the same call
    launched on its own.  More calls than the kernel's table holds make it launch twice."""
    bar = torch.zeros(4, dtype=torch.int32, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    H, F, taps = 200, 136, 3

    def run(fused):
        g = lambda *shape, seed, dtype=torch.bfloat16, scale=1.0: rnd(*shape, dtype=dtype, seed=seed, scale=scale)
        out = {}
        x = g(M, H, seed=1)
        w_in, w_out = g(3 * H, H, seed=2, scale=0.1), g(H, H, seed=3, scale=0.1)
        w_gu, w_down, w_head = g(2 * F, H, seed=4, scale=0.1), g(H, F, seed=5, scale=0.1), g(1000, H, seed=6, scale=0.1)
        conv_w = g(H, taps, seed=7, dtype=torch.float32)
        state = g(M + 2, taps - 1, H, seed=8, dtype=torch.float32)
        slots = torch.arange(1, M + 1, dtype=torch.int32, device=DEV)
        post, nxt = g(H, seed=9, dtype=torch.float32), g(H, seed=10, dtype=torch.float32)
        h = g(M, H, seed=11)
        ctx = K.FusedDecode(bar, err) if fused else None
        if ctx:
            ctx.__enter__()
        launches0 = K.launches
        y = torch.empty(M, H, dtype=torch.bfloat16, device=DEV)
        K.gemm_skinny_shortconv(y, x, w_in, conv_w, state, slots)                 # in_proj + convolution
        parts = torch.empty(4, M, H, dtype=torch.float32, device=DEV)
        K.gemm_skinny_parts(parts, y, w_out)                                      # out_proj as partial sums
        n = torch.empty_like(h)
        K.add_norm(h, n, K.PartialSums(parts, torch.bfloat16), h, post, nxt, 1e-5, 1e-6)
        a = torch.empty(M, F, dtype=torch.bfloat16, device=DEV)
        K.gemm_skinny(a, n, w_gu, swiglu=True)
        d = torch.empty(M, H, dtype=torch.bfloat16, device=DEV)
        K.gemm_skinny(d, a, w_down)
        n2 = torch.empty_like(h)
        K.add_norm(h, n2, d, h, None, nxt, 0.0, 1e-6)
        logits = torch.empty(M, 1000, dtype=torch.float32, device=DEV)
        K.gemm_skinny(logits, n2, w_head)
        h2 = torch.empty_like(h)
        for i in range(30):                                                       # past the table's 24 entries
            K.add_norm(h2, n2, d, h, post, nxt, 1e-5, 1e-6)
        if ctx:
            ctx.__exit__(None, None, None)
        out.update(y=y, parts=parts.sum(0), n=n, a=a, d=d, h=h, h2=h2, n2=n2, logits=logits, state=state)
        return out, K.launches - launches0

    one, n_one = run(False)
    fused, n_fused = run(True)
    assert n_fused == 2 and n_one > 30
    assert int(err) == 0 and int(bar[0]) == 0
    for name in one:
        close(fused[name], one[name], torch.bfloat16 if one[name].dtype == torch.bfloat16 else torch.float32,
              **(dict(rtol=3e-2, atol=3e-2) if name in ("h", "h2", "n2", "logits", "d", "a", "n") else {}))


def test_fused_decode_refuses_what_it_cannot_run(K):
    bar = torch.zeros(4, dtype=torch.int32, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    x = rnd(17, 64, dtype=torch.bfloat16)
    w = rnd(32, 64, dtype=torch.bfloat16)
    y = torch.empty(17, 32, dtype=torch.bfloat16, device=DEV)
    with K.FusedDecode(bar, err) as f:
        K.gemm_skinny(y, x, w)                       # 17 rows: not collected, launched on its own
        assert not f.ops
    close(y, x.float() @ w.float().T, torch.bfloat16)
