"""Python face of the CUDA library: one function per entry point, taking torch tensors.

Every call launches on torch's current stream, checks the entry point's return code and
raises `KernelError` with the library's message.  There is no fallback: if the library
cannot be built or loaded, importing a kernel raises.
"""
from __future__ import annotations

import ctypes
import os

import torch

from .csrc import build as _build
from .csrc import limits as _limits
from .csrc.limits import ATTN_DECODE_CHUNK, PAGE_TOKENS  # noqa: F401  (re-exported)

DT_F32, DT_BF16 = 0, 1

_vp, _i, _ll, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float

_SIGNATURES = {
    "cm_embed_gather": [_i, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp, _vp],
    "cm_scale_softcap": [_vp, _ll, _f, _f, _vp],
    "cm_rmsnorm": [_i, _vp, _vp, _vp, _i, _i, _f, _ll, _ll, _vp],
    "cm_add_norm": [_i, _vp, _vp, _vp, _vp, _i, _ll, _vp, _vp, _vp, _i, _i, _f, _f, _vp],
    "cm_gemm_tc_few_rows_parts": [_vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _i, _vp, _vp],
    "cm_gemm_skinny_parts": [_vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _ll, _i, _vp],
    "cm_swiglu": [_i, _vp, _vp, _i, _i, _vp],
    "cm_gather_rows": [_i, _vp, _vp, _vp, _i, _i, _vp],
    "cm_gemm_simt": [_i, _i, _i, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _vp],
    "cm_gemm_skinny": [_i, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _i, _vp],
    "cm_gemm_tc": [_i, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _i, _i, _vp, _vp],
    "cm_gemm_tc_few_rows": [_i, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _i, _i, _vp, _vp],
    "cm_qk_prepare": [_i, _vp, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _vp, _i, _i, _i, _i, _i,
                      _i, _f, _i, _vp],
    "cm_attn_prefill_simt": [_i, _vp, _ll, _vp, _vp, _vp, _ll, _vp, _ll, _vp, _i, _i, _i, _i, _i, _i, _f, _vp],
    "cm_attn_prefill_mma": [_vp, _ll, _vp, _vp, _vp, _ll, _vp, _ll, _vp, _i, _i, _i, _i, _i, _i, _f, _vp],
    "cm_attn_prefill_tc": [_vp, _ll, _vp, _vp, _vp, _ll, _vp, _ll, _vp, _i, _i, _ll, _i, _i, _i, _i, _f, _vp, _vp],
    "cm_attn_decode": [_i, _vp, _ll, _vp, _ll, _vp, _ll, _vp, _vp, _vp, _ll, _vp, _i, _i, _i, _i, _i, _i, _i,
                       _i, _f, _vp, _vp, _vp],
    "cm_gemm_skinny_shortconv": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _ll, _ll, _ll, _vp],
    "cm_shortconv": [_i, _vp, _vp, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "cm_attn_append_simt": [_i, _vp, _ll, _vp, _vp, _vp, _ll, _vp, _ll, _vp, _vp, _vp, _vp, _ll, _vp, _ll, _i, _i, _i, _i,
                            _i, _i, _i, _f, _vp],
    "cm_attn_append_mma": [_vp, _ll, _vp, _vp, _vp, _ll, _vp, _ll, _vp, _vp, _vp, _vp, _ll, _vp, _ll, _i, _i, _i, _i, _i,
                           _i, _i, _f, _vp],
    "cm_attn_append_tc": [_vp, _ll, _vp, _vp, _vp, _ll, _vp, _ll, _vp, _vp, _vp, _vp, _ll, _vp, _ll, _i, _i, _i, _ll, _i,
                          _i, _i, _i, _f, _vp, _vp],
    "cm_gemm_tc_parts": [_vp, _vp, _vp, _i, _i, _i, _ll, _ll, _i, _i, _vp, _vp],
    "cm_kv_store": [_i, _vp, _ll, _vp, _vp, _vp, _vp, _vp, _ll, _vp, _ll, _i, _i, _i, _i, _vp],
    "cm_sample": [_vp, _vp, _ll, _i, _i, _vp, _vp, _vp, _vp, _vp],
    "cm_scatter_i32": [_vp, _vp, _vp, _vp, _i, _vp],
    "cm_zero_slots": [_vp, _i, _ll, _ll, ctypes.POINTER(ctypes.c_int), _i, _vp],
    "cm_copy_pages": [_vp, _vp, _vp, _i, _i, _ll, _ll, _vp],
}


class KernelError(RuntimeError):
    pass


_lib = None


class Timeline:
    """Times every launch of the library between `with kernels.Timeline() as t:` and its end, with a
    pair of CUDA events around each entry-point call, and keeps what the binding knows about the
    call: its name, the operands' shape and the bytes and floating-point operations that the
    operation needs by its definition (each operand once).  `rows()` adds the calls up by name
    and shape.  catena-models prints its own phase timers on request (CATENA_COMPILE_TIMINGS,
    src/catena.rs:82-87; per-phase rates, src/main.rs:364-371); this is that habit for kernels.
    Off unless entered: an ordinary run records no events.

    `in_graph=True` makes the events of a kind that may be recorded while a CUDA graph is captured and
    read after the graph has been replayed: the calls of a decode step are then timed inside the
    recorded step (`keep_last(n)` drops what was collected before the capture), where a kernel follows
    its predecessor as it does in production, instead of after the host's pause between two launches."""

    def __init__(self, in_graph=False):
        self.calls = []            # [name, shape, bytes, flops, start event, end event, launches]
        self._start = None
        self._event = ((lambda: torch.cuda.Event(enable_timing=True, external=True)) if in_graph
                       else (lambda: torch.cuda.Event(enable_timing=True)))

    def keep_last(self, n):
        self.calls = self.calls[-n:]

    def __enter__(self):
        global _timeline
        self._before, _timeline = _timeline, self
        return self

    def __exit__(self, *exc):
        global _timeline
        _timeline = self._before

    def begin(self):
        self._start = self._event()
        self._start.record()

    def end(self, name, n, cost):
        if self._start is None:
            return
        stop = self._event()
        stop.record()
        shape, nbytes, flops = cost() if cost is not None else ("", 0, 0)
        self.calls.append([name, shape, nbytes, flops, self._start, stop, n])
        self._start = None

    def rows(self):
        """[{name, shape, calls, launches, us, bytes, flops}] by name and shape, in order of first use
        (synchronises)."""
        torch.cuda.synchronize()
        out = {}
        for name, shape, nbytes, flops, a, b, n in self.calls:
            row = out.setdefault((name, shape), dict(name=name, shape=shape, calls=0, launches=0, us=0.0, bytes=0, flops=0))
            row["calls"] += 1
            row["launches"] += n
            row["us"] += a.elapsed_time(b) * 1e3
            row["bytes"] += nbytes
            row["flops"] += flops
        return list(out.values())


_timeline = None


def _nbytes(*tensors):
    return sum(t.numel() * t.element_size() for t in tensors if t is not None)


# ------------------------------------------------------------------ fused decode segments
FD_GEMV, FD_ADD_NORM, FD_CONV = 0, 1, 2
FD_PLAIN, FD_SWIGLU, FD_PARTS, FD_F32 = 0, 1, 2, 3
FD_MAX_ROWS = 16


class _FdOp(ctypes.Structure):
    """csrc/decode_fused.h: FdOp."""
    _fields_ = ([(n, ctypes.c_int) for n in ("kind", "mode", "M", "N", "K", "ksplit", "n_parts", "taps")]
                + [(n, ctypes.c_longlong) for n in ("ldx", "ldw", "ldy", "part_stride")]
                + [(n, ctypes.c_void_p) for n in ("x", "w", "y", "aux0", "aux1", "aux2", "aux3", "idx")]
                + [("eps0", ctypes.c_float), ("eps1", ctypes.c_float), ("pad0", ctypes.c_int), ("pad1", ctypes.c_int)])


class FusedDecode:
    """While entered, the calls of a decode step that the fused kernel knows (`gemm_skinny` and its
    forms, `add_norm`, the short convolution's decode form; bfloat16, at most 16 rows) are not
    launched but collected, in program order, and run as ONE cooperative launch (`cm_fused_decode`)
    as soon as a call comes that the kernel does not know, when the kernel's table is full, or at
    the end.  Memory that the collected calls use stays referenced until they have been launched.
    `bar`: the kernel's barrier word (uint32 zero on the device); `err`: the device flag that a
    block raises when its wait at the barrier runs out."""

    def __init__(self, bar, err):
        self.bar, self.err = bar, err
        self.ops, self.keep = [], []
        self.max_ops = lib().cm_fused_decode_max_ops()
        self.max_width = lib().cm_fused_decode_max_width()
        self._flushing = False

    def __enter__(self):
        global _fuser
        self._before, _fuser = _fuser, self
        return self

    def __exit__(self, exc_type, *exc):
        global _fuser
        try:
            if exc_type is None:
                self.flush()
        finally:
            _fuser = self._before
            self.ops, self.keep = [], []

    def add(self, keep, **fields):
        op = _FdOp()
        for k, v in fields.items():
            setattr(op, k, v)
        self.ops.append(op)
        self.keep.extend(keep)
        if len(self.ops) >= self.max_ops:
            self.flush()

    def flush(self):
        if not self.ops or self._flushing:
            return
        self._flushing = True
        try:
            n = len(self.ops)
            seg = (ctypes.c_int * 4)(n, 0, 0, 0)
            blob = bytes(seg) + b"".join(bytes(op) for op in self.ops)
            blob += b"\0" * (16 + self.max_ops * ctypes.sizeof(_FdOp) - len(blob))
            ops, self.ops, self.keep = self.ops, [], []
            _check(lib().cm_fused_decode(blob, _ptr(self.bar), _ptr(self.err), _stream()), "fused_decode",
                   cost=lambda: (f"{n} operations", 0, 0))
        finally:
            self._flushing = False


_fuser = None


def _fusable_rows(x, w):
    """x @ w^T can join a fused segment: bfloat16, at most 16 rows, 16-byte aligned rows."""
    return (_fuser is not None and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] <= FD_MAX_ROWS
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.stride(1) == 1
            and w.stride(1) == 1 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def lib():
    """The loaded CUDA library, with argument types set."""
    global _lib
    if _fuser is not None and _fuser.ops and not _fuser._flushing:
        _fuser.flush()             # a call that is launched on its own: what was collected runs before it
    if _timeline is not None and _lib is not None:
        _timeline.begin()          # every binding asks for the library right before its launch
    if _lib is None:
        handle = _build.load()
        handle.cm_last_error.restype = ctypes.c_char_p
        _limits.check_library(handle)
        for name, args in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = args
            fn.restype = _i
        handle.cm_set_pdl.argtypes = [_i]
        handle.cm_set_pdl.restype = None
        handle.cm_fused_decode.argtypes = [ctypes.c_char_p, _vp, _vp, _vp]
        handle.cm_fused_decode.restype = _i
        if os.environ.get("CATENA_B200_PDL", "1") == "0":
            handle.cm_set_pdl(0)
        _lib = handle
    return _lib


def set_pdl(on):
    """Programmatic dependent launch for every kernel of the library (on by default; the
    environment variable CATENA_B200_PDL=0 turns it off at load)."""
    lib().cm_set_pdl(1 if on else 0)


def library_path():
    return lib()._name


def dtype_code(dtype):
    if dtype == torch.float32:
        return DT_F32
    if dtype == torch.bfloat16:
        return DT_BF16
    raise KernelError(f"no kernels for dtype {dtype}")


def _ptr(t):
    return None if t is None else t.data_ptr()


_pinned_stream = None


def _stream():
    if _pinned_stream is not None:
        return _pinned_stream
    return torch.cuda.current_stream().cuda_stream


class pinned_stream:
    """Within this context every kernel of the library is launched on the stream that was current
    when it was entered, looked up once instead of once per launch (the lookup costs several
    microseconds, as much as a launch).  The caller must not change the current stream inside."""

    def __enter__(self):
        global _pinned_stream
        self._before = _pinned_stream
        _pinned_stream = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _pinned_stream
        _pinned_stream = self._before


launches = 0          # kernels launched (or recorded into a graph) by this process, counted per call


def _check(code, name, n=1, cost=None):
    """`cost`: a callable that gives (shape text, bytes, floating-point operations) of the call; it is
    evaluated only while a Timeline records."""
    global launches
    launches += n
    if _timeline is not None:
        _timeline.end(name, n, cost)
    if code != 0:
        raise KernelError(f"{name} returned {code}: {_lib.cm_last_error().decode(errors='replace')}")


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels take CUDA tensors only; there is no CPU path")


# ---------------------------------------------------------------------------- row-wise
def embed_gather(out, table, tokens, err=None, sampled=None, scale=1.0):
    """out[t] = table[tokens[t]] * scale; with `sampled` (int32 device tensor) an entry -(1 + i) of
    tokens stands for sampled[i]."""
    _need_cuda(out, table, tokens)
    T, H = out.shape
    _check(lib().cm_embed_gather(dtype_code(out.dtype), dtype_code(table.dtype), _ptr(out), _ptr(table), _ptr(tokens),
                                 _ptr(sampled), T, H, table.shape[0], scale, _ptr(err), _stream()), "embed_gather",
           cost=lambda: (f"{T}x{H}", T * H * table.element_size() + _nbytes(out, tokens), 0))


def rmsnorm(out, x, w, eps):
    _need_cuda(out, x, w)
    rows, H = x.shape
    _check(lib().cm_rmsnorm(dtype_code(x.dtype), _ptr(out), _ptr(x), _ptr(w), rows, H, eps, x.stride(0),
                            out.stride(0), _stream()), "rmsnorm",
           cost=lambda: (f"{rows}x{H}", _nbytes(x, out, w), 4 * rows * H))


class PartialSums:
    """A product x @ w^T left as float partial sums over slices of its inner dimension:
    `parts` [slices, rows, width].  Whoever consumes it adds the slices in index order and rounds
    the total to the activation dtype (`add_norm` does both while it reads them)."""

    def __init__(self, parts, dtype):
        self.parts, self.dtype = parts, dtype

    @property
    def shape(self):
        return self.parts.shape[1:]


def add_norm(h_out, n_out, m, h_in, w_post, w_next, eps_post, eps_next):
    """h_out = h_in + (norm(m; w_post) or m); n_out = norm(h_out; w_next) when w_next is given.
    m: a tensor, or the PartialSums a product left."""
    if (_fuser is not None and h_in.dtype == torch.bfloat16 and h_in.shape[0] <= FD_MAX_ROWS and h_in.shape[1] % 8 == 0
            and h_in.shape[1] <= _fuser.max_width and h_in.is_contiguous() and h_out.is_contiguous()
            and (n_out is None or n_out.is_contiguous())):
        rows, H = h_in.shape
        if isinstance(m, PartialSums):
            src, n_parts, stride = m.parts, m.parts.shape[0], rows * H
            ok = src.dtype == torch.float32 and src.is_contiguous() and n_parts <= 8
        else:
            src, n_parts, stride = m, 0, 0
            ok = m.dtype == torch.bfloat16 and m.is_contiguous()
        if ok:
            _fuser.add((h_out, n_out, src, h_in, w_post, w_next), kind=FD_ADD_NORM, M=rows, N=H, n_parts=n_parts,
                       part_stride=stride, x=_ptr(h_in), y=_ptr(h_out), aux0=_ptr(src), aux1=_ptr(w_post),
                       aux2=_ptr(w_next), aux3=_ptr(n_out), eps0=eps_post, eps1=eps_next)
            return
    if isinstance(m, PartialSums):
        parts = m.parts
        _need_cuda(h_out, parts, h_in)
        n_parts, rows, H = parts.shape
        if parts.dtype != torch.float32 or not parts.is_contiguous():
            raise KernelError("add_norm: partial sums must be contiguous float32")
        _check(lib().cm_add_norm(dtype_code(h_in.dtype), _ptr(h_out), _ptr(n_out), None, _ptr(parts), n_parts, rows * H,
                                 _ptr(h_in), _ptr(w_post), _ptr(w_next), rows, H, eps_post, eps_next, _stream()),
               "add_norm", cost=lambda: (f"{rows}x{H} over {n_parts} partial sums",
                                         _nbytes(parts, h_in, h_out, n_out, w_post, w_next), (n_parts + 8) * rows * H))
        return
    _need_cuda(h_out, m, h_in)
    rows, H = m.shape
    _check(lib().cm_add_norm(dtype_code(m.dtype), _ptr(h_out), _ptr(n_out), _ptr(m), None, 0, 0, _ptr(h_in), _ptr(w_post),
                             _ptr(w_next), rows, H, eps_post, eps_next, _stream()), "add_norm",
           cost=lambda: (f"{rows}x{H}", _nbytes(m, h_in, h_out, n_out, w_post, w_next), 8 * rows * H))


def scale_softcap(logits, scale=1.0, cap=0.0):
    """logits <- cap * tanh(logits * scale / cap) (cap > 0) or logits * scale, in place; float32."""
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise KernelError("scale_softcap takes contiguous float32 logits")
    _check(lib().cm_scale_softcap(_ptr(logits), logits.numel(), scale, cap, _stream()), "scale_softcap")


def swiglu(out, gate_up):
    rows, F = out.shape
    _check(lib().cm_swiglu(dtype_code(out.dtype), _ptr(out), _ptr(gate_up), rows, F, _stream()), "swiglu")


def gather_rows(out, x, rows):
    n, H = out.shape
    _check(lib().cm_gather_rows(dtype_code(x.dtype), _ptr(out), _ptr(x), _ptr(rows), n, H, _stream()),
           "gather_rows")


# ------------------------------------------------------------------------------- gemm
def gemm_simt(y, x, w):
    """y[M,N] = x[M,K] @ w[N,K]^T on the CUDA cores (float accumulation)."""
    _need_cuda(y, x, w)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(y.shape) != (M, N):
        raise KernelError(f"gemm shapes: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
    _check(lib().cm_gemm_simt(dtype_code(x.dtype), dtype_code(w.dtype), dtype_code(y.dtype), _ptr(y), _ptr(x),
                              _ptr(w), M, N, K, x.stride(0), w.stride(0), y.stride(0), _stream()), "gemm_simt",
           cost=lambda: (f"{M}x{N}x{K}", _nbytes(x, w, y), 2 * M * N * K))


def gemm_skinny(y, x, w, swiglu=False):
    """y = x @ w^T for at most 64 bfloat16 rows, weights streamed once (mma.sync, float sums).
    swiglu: w is [gate; up] with 2F rows and y[M, F] = silu(x Wgate^T) * (x Wup^T)."""
    _need_cuda(y, x, w)
    M, K = x.shape
    N = y.shape[1]
    if w.shape[1] != K or w.shape[0] != (2 * N if swiglu else N) or y.shape[0] != M:
        raise KernelError(f"gemm_skinny shapes: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_skinny takes bfloat16 operands")
    if _fusable_rows(x, w) and y.stride(1) == 1 and (y.dtype == torch.bfloat16 or (y.dtype == torch.float32 and not swiglu)):
        mode = FD_SWIGLU if swiglu else (FD_PLAIN if y.dtype == torch.bfloat16 else FD_F32)
        _fuser.add((y, x, w), kind=FD_GEMV, mode=mode, M=M, N=N, K=K, ksplit=1, ldx=x.stride(0), ldw=w.stride(0),
                   ldy=y.stride(0), x=_ptr(x), w=_ptr(w), y=_ptr(y))
        return
    _check(lib().cm_gemm_skinny(dtype_code(y.dtype), _ptr(y), _ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0),
                                y.stride(0), int(swiglu), _stream()), "gemm_skinny" + ("_swiglu" if swiglu else ""),
           cost=lambda: (f"{M}x{w.shape[0]}x{K}", _nbytes(x, w, y), 2 * M * w.shape[0] * K))


def gemm_skinny_parts(parts, x, w):
    """parts[s] = x[:, slice s of K] @ w[:, slice s of K]^T in float, for at most 16 bfloat16 rows:
    the weight-streaming product with K cut over parts.shape[0] independent groups of blocks."""
    _need_cuda(parts, x, w)
    M, K = x.shape
    S, _, N = parts.shape
    if w.shape != (N, K) or parts.shape[1] != M or parts.dtype != torch.float32 or not parts.is_contiguous():
        raise KernelError(f"gemm_skinny_parts shapes: x {tuple(x.shape)}, w {tuple(w.shape)}, parts {tuple(parts.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_skinny_parts takes bfloat16 operands")
    if _fusable_rows(x, w) and S <= 8:
        _fuser.add((parts, x, w), kind=FD_GEMV, mode=FD_PARTS, M=M, N=N, K=K, ksplit=S, ldx=x.stride(0), ldw=w.stride(0),
                   ldy=N, part_stride=M * N, x=_ptr(x), w=_ptr(w), y=_ptr(parts))
        return
    _check(lib().cm_gemm_skinny_parts(_ptr(parts), _ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0), N, M * N, S,
                                      _stream()), "gemm_skinny_parts",
           cost=lambda: (f"{M}x{N}x{K} in {S} slices", _nbytes(x, w, parts), 2 * M * N * K))


def gemm_tc_few_rows_parts(parts, x, w, err=None):
    """The same from the tcgen05 few-rows product (at most 128 bfloat16 rows): parts[s] holds the
    float sums over the s-th slice of K; no exchange between the blocks of a column tile."""
    _need_cuda(parts, x, w)
    M, K = x.shape
    S, _, N = parts.shape
    if w.shape != (N, K) or parts.shape[1] != M or parts.dtype != torch.float32 or not parts.is_contiguous():
        raise KernelError(f"gemm_tc_few_rows_parts shapes: x {tuple(x.shape)}, w {tuple(w.shape)}, parts {tuple(parts.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError("gemm_tc_few_rows_parts takes row-major bfloat16 operands")
    _check(lib().cm_gemm_tc_few_rows_parts(_ptr(parts), _ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0), M * N, S,
                                           _ptr(err), _stream()), "gemm_tc_few_rows_parts",
           cost=lambda: (f"{M}x{N}x{K} in {S} slices", _nbytes(x, w, parts), 2 * M * N * K))


def gemm_tc_parts(parts, x, w, err=None, block_n=256):
    """parts[r] = x @ w^T over the r-th of parts.shape[0] runs of the inner dimension, float32
    [runs, rows, width] contiguous: the tiled tcgen05 product for a few hundred rows times a narrow
    output, cut over K so that its (run, tile) items occupy the device; no exchange between blocks,
    the consumer adds the runs in order (`add_norm` takes them as `PartialSums`)."""
    _need_cuda(parts, x, w)
    S, M, N = parts.shape
    if parts.dtype != torch.float32 or not parts.is_contiguous() or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc_parts: contiguous float32 partial sums of a bfloat16 product")
    if x.shape[0] != M or w.shape[0] != N or x.shape[1] != w.shape[1] or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError(f"gemm_tc_parts: shapes {tuple(x.shape)} x {tuple(w.shape)} -> {tuple(parts.shape)}")
    K = x.shape[1]
    _check(lib().cm_gemm_tc_parts(_ptr(parts), _ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0), S, block_n, _ptr(err),
                                  _stream()), "gemm_tc_parts",
           cost=lambda: (f"{M}x{N}x{K} in {S} runs", _nbytes(x, w, parts), 2 * M * N * K))


def gemm_tc(y, x, w, swiglu=False, err=None, block_n=256):
    """y = x @ w^T on the tcgen05 tensor cores (TMA-fed, accumulator in tensor memory), any
    number of bfloat16 rows.  swiglu: w is [gate; up] with 2F rows and y[M, F] = silu(g) * u.
    err: device int32 that a block raises if one of its bounded pipeline waits runs out.
    block_n: 256 (128 x 256 tiles), 128 (twice as many 128 x 128 tiles, for few rows) or 192 (plain
    bfloat16 products only)."""
    _need_cuda(y, x, w)
    M, K = x.shape
    N = y.shape[1]
    if w.shape[1] != K or w.shape[0] != (2 * N if swiglu else N) or y.shape[0] != M:
        raise KernelError(f"gemm_tc shapes: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc takes bfloat16 operands")
    if x.stride(1) != 1 or w.stride(1) != 1 or y.stride(1) != 1:
        raise KernelError("gemm_tc takes row-major operands")
    _check(lib().cm_gemm_tc(dtype_code(y.dtype), _ptr(y), _ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0),
                            y.stride(0), int(swiglu), block_n, _ptr(err), _stream()), "gemm_tc" + ("_swiglu" if swiglu else ""),
           cost=lambda: (f"{M}x{w.shape[0]}x{K}", _nbytes(x, w, y), 2 * M * w.shape[0] * K))


def gemm_tc_few_rows(y, x, w, swiglu=False, err=None, splits=0):
    """gemm_tc for at most 128 rows.  When the product has too few 128-column tiles for the
    device, K is split over a thread-block cluster of up to 8 blocks that add their partial
    sums through distributed shared memory.  splits: 0 chooses, 1..8 forces."""
    _need_cuda(y, x, w)
    M, K = x.shape
    N = y.shape[1]
    if w.shape[1] != K or w.shape[0] != (2 * N if swiglu else N) or y.shape[0] != M:
        raise KernelError(f"gemm_tc_few_rows shapes: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc_few_rows takes bfloat16 operands")
    if x.stride(1) != 1 or w.stride(1) != 1 or y.stride(1) != 1:
        raise KernelError("gemm_tc_few_rows takes row-major operands")
    _check(lib().cm_gemm_tc_few_rows(dtype_code(y.dtype), _ptr(y), _ptr(x), _ptr(w), M, N, K, x.stride(0),
                                     w.stride(0), y.stride(0), int(swiglu), splits, _ptr(err), _stream()),
           "gemm_tc_few_rows" + ("_swiglu" if swiglu else ""),
           cost=lambda: (f"{M}x{w.shape[0]}x{K}", _nbytes(x, w, y), 2 * M * w.shape[0] * K))


# -------------------------------------------------------------------------- attention
def qk_prepare(qkv, wq, wk, rate, tok_pos, tok_seq, seq_slot, seq_end, pool, pages, ptab, ring,
               QH, KVH, HD, eps, interleaved=False):
    """Head norm + rotation in place on the q and k columns of qkv; k and v go to the cache
    (pool: this layer's [2, pages, KVH, 64, HD] storage, or None to write no cache).  The rotation
    pairs element i with i + HD/2, or, with `interleaved`, 2i with 2i + 1."""
    T = qkv.shape[0]
    _check(lib().cm_qk_prepare(dtype_code(qkv.dtype), _ptr(qkv), qkv.stride(0), _ptr(wq), _ptr(wk), _ptr(rate),
                               _ptr(tok_pos), _ptr(tok_seq), _ptr(seq_slot), _ptr(seq_end), _ptr(pool), pages,
                               _ptr(ptab), 0 if ptab is None else ptab.stride(0), ring, T, QH, KVH, HD, eps,
                               int(interleaved), _stream()), "qk_prepare",
           cost=lambda: (f"{T} tokens, {QH}+{KVH} heads of {HD}",
                         T * HD * qkv.element_size() * (2 * QH + (2 * KVH if pool is None else 4 * KVH)), 0))


def attn_prefill_simt(ctx, q, k, v, gate, seq_start, B, max_len, QH, KVH, HD, window, scale):
    """q, k, v, gate are column views of one packed row-major buffer (same row stride)."""
    if not (q.stride(0) == k.stride(0) == v.stride(0)):
        raise KernelError("attn_prefill: q, k and v must share a row stride")
    _check(lib().cm_attn_prefill_simt(dtype_code(q.dtype), _ptr(ctx), ctx.stride(0), _ptr(q), _ptr(k), _ptr(v),
                                      q.stride(0), _ptr(gate), 0 if gate is None else gate.stride(0),
                                      _ptr(seq_start), B, max_len, QH, KVH, HD, window, scale, _stream()),
           "attn_prefill_simt",
           cost=lambda: (f"{B} sequences up to {max_len}, {QH}/{KVH} heads of {HD}, window {window}", 0, 0))


def attn_prefill_mma(ctx, q, k, v, gate, seq_start, B, max_len, QH, KVH, HD, window, scale):
    """The same on the tensor cores: bfloat16, head sizes that are multiples of 16 up to 128."""
    if not (q.stride(0) == k.stride(0) == v.stride(0)) or q.dtype != torch.bfloat16:
        raise KernelError("attn_prefill_mma: bfloat16 q, k and v that share a row stride")
    _check(lib().cm_attn_prefill_mma(_ptr(ctx), ctx.stride(0), _ptr(q), _ptr(k), _ptr(v), q.stride(0), _ptr(gate),
                                     0 if gate is None else gate.stride(0), _ptr(seq_start), B, max_len, QH, KVH,
                                     HD, window, scale, _stream()), "attn_prefill_mma",
           cost=lambda: (f"{B} sequences up to {max_len}, {QH}/{KVH} heads of {HD}, window {window}", 0, 0))


def attn_append(ctx, q, k, v, gate, seq_start, seq_pos0, seq_slot, pool, pages, ptab, ring, B, max_len, QH, KVH, HD,
                window, scale, tensor_cores=True):
    """Attention of a step whose sequences may stand at seq_pos0[b] > 0: keys and values below that
    position come from the paged cache `pool`, the rest from the step's own rows (q, k, v as for the
    prefill kernels), which the caller writes to the cache afterwards (`kv_store`).  bfloat16 with a
    head size that is a multiple of 16 up to 128 runs on the tensor cores unless `tensor_cores` is off."""
    if not (q.stride(0) == k.stride(0) == v.stride(0)):
        raise KernelError("attn_append: q, k and v must share a row stride")
    mma = (tensor_cores and q.dtype == torch.bfloat16 and HD % 16 == 0 and HD <= 128 and q.stride(0) % 8 == 0
           and (q.data_ptr() | k.data_ptr() | v.data_ptr() | pool.data_ptr()) % 16 == 0)
    common = (_ptr(q), _ptr(k), _ptr(v), q.stride(0), _ptr(gate), 0 if gate is None else gate.stride(0), _ptr(seq_start),
              _ptr(seq_pos0), _ptr(seq_slot), _ptr(pool), pages, _ptr(ptab), ptab.stride(0), ring, B, max_len, QH, KVH,
              HD, window, scale, _stream())
    if mma:
        _check(lib().cm_attn_append_mma(_ptr(ctx), ctx.stride(0), *common), "attn_append_mma")
    else:
        _check(lib().cm_attn_append_simt(dtype_code(q.dtype), _ptr(ctx), ctx.stride(0), *common), "attn_append_simt")


def attn_append_tc(ctx, q, k, v, gate, seq_start, seq_pos0, seq_slot, pool, pages, ptab, ring, B, max_len, QH, KVH, HD,
                   window, scale, err=None):
    """`attn_append` on the tcgen05 tensor cores: bfloat16, head size 64 or 128, the cache read page by
    page with TMA.  err: device int32 that a block raises if a bounded pipeline wait runs out."""
    if (not (q.stride(0) == k.stride(0) == v.stride(0)) or q.dtype != torch.bfloat16 or pool.dtype != torch.bfloat16
            or q.shape[0] != k.shape[0]):
        raise KernelError("attn_append_tc: bfloat16 q, k, v and cache; q, k and v share rows and a row stride")
    if not pool.is_contiguous() or tuple(pool.shape[2:]) != (KVH, PAGE_TOKENS, HD):
        raise KernelError(f"attn_append_tc: the cache must be contiguous [2, pages, {KVH}, {PAGE_TOKENS}, {HD}]")
    _check(lib().cm_attn_append_tc(_ptr(ctx), ctx.stride(0), _ptr(q), _ptr(k), _ptr(v), q.stride(0), _ptr(gate),
                                   0 if gate is None else gate.stride(0), _ptr(seq_start), _ptr(seq_pos0),
                                   _ptr(seq_slot), _ptr(pool), pages, _ptr(ptab), ptab.stride(0), ring, B, max_len,
                                   q.shape[0], QH, KVH, HD, window, scale, _ptr(err), _stream()), "attn_append_tc",
           cost=lambda: (f"{B} sequences of up to {max_len} rows, {QH}/{KVH} heads of {HD}, window {window}", 0, 0))


def kv_store(kv, tok_pos, tok_seq, seq_slot, seq_end, pool, pages, ptab, ring, KVH, HD):
    """kv: the k | v columns [T, 2 * KVH * HD] of the step's packed rows (k normed and rotated);
    writes them to the cache entries of their positions (a ring keeps the last `ring` of a sequence)."""
    T = kv.shape[0]
    _check(lib().cm_kv_store(dtype_code(kv.dtype), _ptr(kv), kv.stride(0), _ptr(tok_pos), _ptr(tok_seq), _ptr(seq_slot),
                             _ptr(seq_end), _ptr(pool), pages, _ptr(ptab), ptab.stride(0), ring, T, KVH, HD, _stream()),
           "kv_store")


def attn_prefill_tc(ctx, q, k, v, gate, seq_start, B, max_len, QH, KVH, HD, window, scale, err=None):
    """The same on the tcgen05 tensor cores (TMA-fed, scores and outputs in tensor memory): bfloat16,
    head size 64 or 128.  q, k and v are column blocks of one row-major buffer.  err: device int32
    that a block raises if one of its bounded pipeline waits runs out."""
    if not (q.stride(0) == k.stride(0) == v.stride(0)) or q.dtype != torch.bfloat16 or q.shape[0] != k.shape[0]:
        raise KernelError("attn_prefill_tc: bfloat16 q, k and v that share rows and a row stride")
    _check(lib().cm_attn_prefill_tc(_ptr(ctx), ctx.stride(0), _ptr(q), _ptr(k), _ptr(v), q.stride(0), _ptr(gate),
                                    0 if gate is None else gate.stride(0), _ptr(seq_start), B, max_len, q.shape[0],
                                    QH, KVH, HD, window, scale, _ptr(err), _stream()), "attn_prefill_tc",
           cost=lambda: (f"{B} sequences up to {max_len}, {QH}/{KVH} heads of {HD}, window {window}", 0, 0))


def set_decode_attention_target_blocks(blocks):
    """Blocks the tensor-core decode attention aims at (0: chosen from the amount of work, the
    default).  With fewer, each block walks several 256-entry chunks of a sequence."""
    lib().cm_attn_decode_set_target_blocks(int(blocks))


def set_decode_attention_tensor_cores(on):
    """bfloat16 decode attention normally runs its first stage on the tensor cores when the head
    size allows it; off forces the CUDA-core stage (tests compare the two)."""
    lib().cm_attn_decode_set_mma.argtypes = [_i]
    lib().cm_attn_decode_set_mma.restype = None
    lib().cm_attn_decode_set_mma(1 if on else 0)


def attn_decode_scratch(B, QH, HD, n_chunks, device):
    return (torch.empty(B * QH * n_chunks * HD, dtype=torch.float32, device=device),
            torch.empty(B * QH * n_chunks * 2, dtype=torch.float32, device=device))


def attn_decode(ctx, q, gate, seq_pos, seq_slot, pool, pages, ptab, ring, window, QH, KVH, HD, n_chunks,
                scale, part_o, part_ml):
    B = q.shape[0]
    _check(lib().cm_attn_decode(dtype_code(q.dtype), _ptr(ctx), ctx.stride(0), _ptr(q), q.stride(0), _ptr(gate),
                                0 if gate is None else gate.stride(0), _ptr(seq_pos), _ptr(seq_slot), _ptr(pool),
                                pages, _ptr(ptab), ptab.stride(0), ring, window, B, QH, KVH, HD, n_chunks, scale,
                                _ptr(part_o), _ptr(part_ml), _stream()), "attn_decode", 2,
           cost=lambda: (f"{B} sequences, {QH}/{KVH} heads of {HD}, window {window}, {n_chunks} chunks", 0, 0))


# -------------------------------------------------------------------------- short conv
def shortconv(y, bcx, w, state, tok_seq, seq_start, seq_slot, K, from_zero, one_token_each, w_t=None, seq_pos0=None):
    """w: taps [H, K]; w_t: the same stored [K, H] (optional, for 16-byte reads of the taps).
    from_zero: every sequence starts from an empty state; one_token_each: a decode step.  Neither:
    several tokens on top of the stored state (two launches: outputs, then the state); seq_pos0
    (first position per sequence) then lets a sequence that stands at 0 start from an empty state."""
    T, H = y.shape
    two = not from_zero and not one_token_each
    _check(lib().cm_shortconv(dtype_code(y.dtype), _ptr(y), _ptr(bcx), bcx.stride(0), _ptr(w), _ptr(w_t), _ptr(state),
                              _ptr(tok_seq), _ptr(seq_start), _ptr(seq_slot), _ptr(seq_pos0), T, H, K, int(from_zero),
                              int(one_token_each), _stream()), "shortconv", 2 if two else 1,
           cost=lambda: (f"{T}x{H}, {K} taps", _nbytes(bcx, y), 2 * (K + 1) * T * H))


def gemm_skinny_shortconv(y, x, w_in, taps, state, seq_slot):
    """A decode step's in_proj and short convolution in one kernel: x [M <= 16, K] and w_in [3H, K]
    bfloat16 (rows B | C | X), taps [H, KT] float, state [slots, KT - 1, H] float (shifted in
    place), seq_slot [M]; y [M, H] bfloat16."""
    _need_cuda(y, x, w_in)
    M, K = x.shape
    H, KT = taps.shape
    if w_in.shape != (3 * H, K) or y.shape != (M, H) or state.shape[1:] != (KT - 1, H):
        raise KernelError(f"gemm_skinny_shortconv shapes: x {tuple(x.shape)}, w {tuple(w_in.shape)}, "
                          f"y {tuple(y.shape)}, taps {tuple(taps.shape)}, state {tuple(state.shape)}")
    if not (x.dtype == w_in.dtype == y.dtype == torch.bfloat16 and taps.dtype == state.dtype == torch.float32):
        raise KernelError("gemm_skinny_shortconv takes bfloat16 operands, float taps and state")
    if not (taps.is_contiguous() and state.is_contiguous()):
        raise KernelError("gemm_skinny_shortconv: taps and state must be contiguous")
    if _fusable_rows(x, w_in) and H % 8 == 0 and y.stride(0) % 8 == 0 and y.data_ptr() % 16 == 0:
        # in the fused kernel: in_proj as a product of its own, then the convolution over its output
        bcx = torch.empty((M, 3 * H), dtype=torch.bfloat16, device=x.device)
        _fuser.add((bcx, x, w_in), kind=FD_GEMV, mode=FD_PLAIN, M=M, N=3 * H, K=K, ksplit=1, ldx=x.stride(0),
                   ldw=w_in.stride(0), ldy=3 * H, x=_ptr(x), w=_ptr(w_in), y=_ptr(bcx))
        _fuser.add((y, taps, state, seq_slot), kind=FD_CONV, M=M, N=H, taps=KT, ldx=3 * H, ldy=y.stride(0), x=_ptr(bcx),
                   y=_ptr(y), aux0=_ptr(taps), aux3=_ptr(state), idx=_ptr(seq_slot))
        return
    _check(lib().cm_gemm_skinny_shortconv(_ptr(y), _ptr(x), _ptr(w_in), _ptr(taps), _ptr(state), _ptr(seq_slot), M, H,
                                          K, KT, x.stride(0), w_in.stride(0), y.stride(0), _stream()),
           "gemm_skinny_shortconv",
           cost=lambda: (f"{M}x{3 * H}x{K}", _nbytes(x, w_in, y, taps) + 2 * M * (KT - 1) * H * 4, 2 * M * 3 * H * K))


# ---------------------------------------------------------------------------- sampling
def sample(out, logits, temperature, sequence, step, seed_words):
    n, V = logits.shape
    _check(lib().cm_sample(_ptr(out), _ptr(logits), logits.stride(0), n, V, _ptr(temperature), _ptr(sequence),
                           _ptr(step), _ptr(seed_words), _stream()), "sample",
           cost=lambda: (f"{n}x{V}", n * V * 4, 0))


# ------------------------------------------------------------------------------- cache
def scatter_i32(table, index, value, count, max_count):
    _check(lib().cm_scatter_i32(_ptr(table), _ptr(index), _ptr(value), _ptr(count), max_count, _stream()),
           "scatter_i32")


def copy_pages(pool, src, dst):
    """pool: [layers, 2, pages, ...] paged storage of one group; page src[i] is copied to page dst[i]
    in every layer and plane (int32 device tensors of equal length)."""
    n = src.numel()
    outer, pages = pool.shape[0] * pool.shape[1], pool.shape[2]
    page_bytes = pool[0, 0, 0].numel() * pool.element_size()
    _check(lib().cm_copy_pages(_ptr(pool), _ptr(src), _ptr(dst), n, outer, pages, page_bytes, _stream()), "copy_pages")


def zero_slots(store, slots):
    """store: [layers, slots, ...] fixed-size states (32-bit words or pairs of 16-bit); clears the rows
    of the given slots (Python ints) in every layer."""
    if not slots:
        return
    layers, total = store.shape[0], store.shape[1]
    row_bytes = store[0, 0].numel() * store.element_size()
    ids = (ctypes.c_int * len(slots))(*slots)
    n_launches = -(-len(slots) // 64)
    _check(lib().cm_zero_slots(_ptr(store), layers, total, row_bytes, ids, len(slots), _stream()), "zero_slots", n_launches)
