"""The engine's view of the device: activation dtype, kernel choice, scratch memory.

Parts ask the runtime for a matrix product or an attention pass and the runtime picks the
kernel from the dtype and the number of rows: the 32-bit engine runs plain FMA kernels only
(no tensor-core mode of reduced precision), the bfloat16 engine runs the tensor-core and
weight-streaming kernels.  Kernel choice never depends on which model or layer is running.
"""
from __future__ import annotations

import torch

from .. import kernels


class Runtime:
    def __init__(self, dtype, device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"engine dtype must be float32 or bfloat16, got {dtype}")
        self.dtype = dtype
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device only; there is no CPU path")
        kernels.lib()                       # build and load now: fail loudly before any model work
        self._scratch = {}
        self._retired = []
        # raised by a kernel whose bounded pipeline wait ran out (0 otherwise); see check_errors
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=self.device)

    def check_errors(self):
        """Read the device error flag (synchronises); raises if a kernel gave up on a wait."""
        code = int(self.error_flag.item())
        if code:
            self.error_flag.zero_()
            raise RuntimeError(f"a kernel's pipeline wait ran out (code {code}); its output is not valid")

    def _unused(self):
        pass

    # ------------------------------------------------------------------ scratch
    def scratch(self, key, numel, dtype=torch.float32):
        """A grow-only device buffer shared by the kernels that run one after another."""
        buf = self._scratch.get(key)
        if buf is None or buf.numel() < numel or buf.dtype != dtype:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError(f"scratch '{key}' would be allocated during graph capture")
            if buf is not None:
                self._retired.append(buf)      # captured graphs may still launch kernels on it
            buf = torch.empty(numel, dtype=dtype, device=self.device)
            self._scratch[key] = buf
        return buf

    def scratch_attn_decode(self, B, QH, HD, n_chunks):
        return (self.scratch("attn_decode_o", B * QH * n_chunks * HD),
                self.scratch("attn_decode_ml", B * QH * n_chunks * 2))

    # ------------------------------------------------------------------ matrix products
    def linear(self, x, w, out_dtype=None):
        """y = x @ w^T; y in the activation dtype unless `out_dtype` says float32."""
        y = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype or x.dtype, device=x.device)
        if self._skinny(x, w):
            kernels.gemm_skinny(y, x, w)
        elif self._tensor_core(x, w):
            kernels.gemm_tc(y, x, w, err=self.error_flag, block_n=self._tile_width(x))
        else:
            kernels.gemm_simt(y, x, w)
        return y

    def _tensor_core(self, x, w):
        """Many bfloat16 rows: the TMA-fed tcgen05 kernel (prompt steps)."""
        return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
                and x.stride(0) % 8 == 0 and x.stride(1) == 1 and x.data_ptr() % 16 == 0 and w.stride(0) % 8 == 0)

    SKINNY_ROWS = 64          # most rows the weight-streaming kernel takes
    SKINNY_SURE_ROWS = 16     # up to here it is always the better kernel
    TILED_MIN_OUT = 4096      # above SKINNY_SURE_ROWS: outputs from which 128-wide tiles fill enough SMs

    def _skinny(self, x, w):
        """Few bfloat16 rows: the weight-streaming kernel (decode steps, wanted rows of the head).
        Between 17 and 64 rows it re-reads the activations once per 16 weight rows, so wide
        products go to the tiled tensor-core kernel instead (measured at 64 rows on B200:
        16384 x 2048 with SwiGLU 39 us against 13 us)."""
        rows = x.shape[0]
        ok = (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and rows <= self.SKINNY_ROWS
              and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0)
        if ok and rows > self.SKINNY_SURE_ROWS and w.shape[0] >= self.TILED_MIN_OUT and self._tensor_core(x, w):
            return False
        return ok

    def _tile_width(self, x):
        return 256 if x.shape[0] > self.SKINNY_ROWS else 128

    def gate_up_swiglu(self, x, w_gate_up, F):
        """a = silu(x Wgate^T) * (x Wup^T) for the row-packed [Wgate; Wup]."""
        a = torch.empty((x.shape[0], F), dtype=x.dtype, device=x.device)
        if self._skinny(x, w_gate_up):
            kernels.gemm_skinny(a, x, w_gate_up, swiglu=True)
            return a
        if self._tensor_core(x, w_gate_up):
            kernels.gemm_tc(a, x, w_gate_up, swiglu=True, err=self.error_flag, block_n=self._tile_width(x))
            return a
        gu = self.linear(x, w_gate_up)
        kernels.swiglu(a, gu)
        return a

    # ------------------------------------------------------------------ attention
    def attention_prefill(self, ctx, q, k, v, gate, batch, QH, KVH, HD, window, scale):
        tensor_cores = (q.dtype == torch.bfloat16 and HD % 16 == 0 and HD <= 128 and q.stride(0) % 8 == 0
                        and q.data_ptr() % 16 == 0 and k.data_ptr() % 16 == 0 and v.data_ptr() % 16 == 0)
        fn = kernels.attn_prefill_mma if tensor_cores else kernels.attn_prefill_simt
        fn(ctx, q, k, v, gate, batch.seq_start, batch.B, batch.max_len, QH, KVH, HD, window, scale)
