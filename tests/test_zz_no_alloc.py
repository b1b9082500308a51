"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some users of this library cannot allocate device memory around a kernel call: a plugin in a
process whose device allocator belongs to the host application, code that runs under a fixed
memory budget, or a plain C caller with no tensor library to ask for scratch buffers.  For
them `cm_attn_decode_noalloc` keeps the kernel's per-chunk partial results in an array inside
the library image.  This test calls it twice in a row (the array is shared between calls and
keeps the previous call's contents) and compares each result with the ordinary entry point,
which gets fresh scratch buffers from the caller, and with attention computed in float64 from
the same keys and values.  That nothing is allocated is checked on the device itself: the free
memory that the driver reports does not shrink over the call (torch's own counters would not
see an allocation made inside the library).

The file is named so that pytest collects it last: a run that stops at the first failure has
then already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
SCRATCH_FLOATS = 5 * 256 * 1024          # CM_NOALLOC_SCRATCH_FLOATS in csrc/attention_noalloc.h


def _symbol():
    from catena_models_b200 import kernels

    handle = ctypes.CDLL(kernels.library_path())
    fn = handle.cm_attn_decode_noalloc
    vp, i, ll, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    fn.argtypes = [i, vp, ll, vp, ll, vp, ll, vp, vp, vp, ll, vp, i, i, i, i, i, i, i, i, f, vp]
    fn.restype = i
    handle.cm_last_error.restype = ctypes.c_char_p
    return kernels, handle, fn


def _case(kernels, dtype, QH, KVH, HD, window, lens, seed):
    """A paged cache with shuffled pages, queries and gates for one decode step."""
    g = torch.Generator().manual_seed(seed)
    ring = (window + 63) // 64 * 64 if window else 0
    per_seq = [((min(n, ring) if ring else n) + 63) // 64 for n in lens]
    pages = sum(per_seq) + 2
    perm = torch.randperm(pages, generator=g).tolist()
    pool = torch.zeros(2, pages, KVH, 64, HD, dtype=dtype, device=DEV)
    ptab = torch.zeros(len(lens), max(per_seq), dtype=torch.int32)
    nxt = 0
    kvs = []
    for b, n in enumerate(lens):
        for j in range(per_seq[b]):
            ptab[b, j] = perm[nxt]
            nxt += 1
        kv = torch.randn(n, 2, KVH, HD, generator=g).to(dtype)
        kvs.append(kv)
        for p in range(max(0, n - ring) if ring else 0, n):
            e = p % ring if ring else p
            pool[:, int(ptab[b, e // 64]), :, e % 64] = kv[p].to(DEV)
    B = len(lens)
    q = torch.randn(B, QH * HD, generator=g).to(dtype).to(DEV)
    gate = torch.randn(B, QH, generator=g).to(dtype).to(DEV)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    slots = torch.arange(B, dtype=torch.int32, device=DEV)
    return dict(q=q, gate=gate, pos=pos, slots=slots, pool=pool, pages=pages, ptab=ptab.to(DEV), ring=ring,
                window=window, QH=QH, KVH=KVH, HD=HD, kv=kvs, lens=list(lens))


def _exact(c):
    """float64 attention of every sequence's newest token over all its keys and values."""
    from test_kernels_gpu import _ref_attention

    QH, HD = c["QH"], c["HD"]
    rows = []
    for b, n in enumerate(c["lens"]):
        qq = torch.zeros(n, QH, HD)
        qq[-1] = c["q"][b].float().cpu().view(QH, HD)
        gg = torch.zeros(n, QH)
        gg[-1] = c["gate"][b].float().cpu()
        rows.append(_ref_attention(qq, c["kv"][b][:, 0], c["kv"][b][:, 1], c["window"], HD ** -0.5, gg)[-1].reshape(-1))
    return torch.stack(rows)


def _run_both(kernels, fn, c, n_chunks):
    B, QH, KVH, HD = c["q"].shape[0], c["QH"], c["KVH"], c["HD"]
    scale = HD ** -0.5
    ref = torch.empty_like(c["q"])
    part_o, part_ml = kernels.attn_decode_scratch(B, QH, HD, n_chunks, DEV)
    kernels.attn_decode(ref, c["q"], c["gate"], c["pos"], c["slots"], c["pool"], c["pages"], c["ptab"], c["ring"],
                        c["window"], QH, KVH, HD, n_chunks, scale, part_o, part_ml)
    got = torch.full_like(c["q"], float("nan"))
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before, _ = torch.cuda.mem_get_info()
    rc = fn(kernels.dtype_code(c["q"].dtype), got.data_ptr(), got.stride(0), c["q"].data_ptr(), c["q"].stride(0),
            c["gate"].data_ptr(), c["gate"].stride(0), c["pos"].data_ptr(), c["slots"].data_ptr(),
            c["pool"].data_ptr(), c["pages"], c["ptab"].data_ptr(), c["ptab"].stride(0), c["ring"], c["window"],
            B, QH, KVH, HD, n_chunks, scale, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert torch.cuda.memory_allocated() == before          # no tensor was made on the way
    assert free_after >= free_before                        # and nothing was taken from the device behind torch's back
    return rc, got, ref


def test_two_calls_in_a_row_match_the_ordinary_entry_point():
    kernels, handle, fn = _symbol()
    # a long call first, then a shorter one of another shape: the second call finds the first
    # call's partial results in the shared array and must not be disturbed by them
    first = _case(kernels, torch.bfloat16, QH=8, KVH=2, HD=64, window=0, lens=[700, 3, 257, 64], seed=1)
    second = _case(kernels, torch.float32, QH=4, KVH=4, HD=32, window=70, lens=[300, 65], seed=2)
    for case, n_chunks in ((first, 4), (second, 2)):
        rc, got, ref = _run_both(kernels, fn, case, n_chunks)
        assert rc == 0, handle.cm_last_error().decode()
        tol = dict(rtol=1e-5, atol=1e-5) if got.dtype == torch.float32 else dict(rtol=1.6e-2, atol=1e-2)
        torch.testing.assert_close(got.float().cpu(), ref.float().cpu(), **tol)
        torch.testing.assert_close(got.float().cpu(), _exact(case).float(), **tol)


def test_a_call_beyond_the_built_in_array_is_refused():
    kernels, handle, fn = _symbol()
    c = _case(kernels, torch.bfloat16, QH=32, KVH=8, HD=128, window=0, lens=[5] * 64, seed=3)
    n_chunks = 8
    assert 64 * 32 * n_chunks * (128 + 2) > SCRATCH_FLOATS
    rc, got, _ = _run_both(kernels, fn, c, n_chunks)
    assert rc != 0
    message = handle.cm_last_error().decode()
    assert "scratch" in message and str(SCRATCH_FLOATS) in message
    assert bool(torch.isnan(got.float()).all())              # nothing was launched
