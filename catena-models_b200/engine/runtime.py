"""The engine's view of the device: activation dtype, kernel choice, scratch memory.

Parts ask the runtime for a matrix product or an attention pass and the runtime picks the
kernel from the dtype and the number of rows: the 32-bit engine runs plain FMA kernels only
(no tensor-core mode of reduced precision), the bfloat16 engine runs the tensor-core and
weight-streaming kernels.  Kernel choice never depends on which model or layer is running.
"""
from __future__ import annotations

import os

import torch

from .. import kernels


class DeviceFault(RuntimeError):
    """A kernel reported on the device that its output is not valid."""


class Runtime:
    def __init__(self, dtype, device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"engine dtype must be float32 or bfloat16, got {dtype}")
        self.dtype = dtype
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device only; there is no CPU path")
        kernels.lib()                       # build and load now: fail loudly before any model work
        # False: prompt steps (more than one row a sequence) run their products and attention on the CUDA
        # cores, whatever the dtype: the reference's --no-wmma-prefill (src/main.rs:34-40)
        self.tensor_core_prompts = True
        self._in_prompt = False
        self._scratch = {}
        self._choices = {}                  # kernel choices by shape, so that a step from Python does not redo them
        self._retired = []
        self._sm_count = None
        # Two flags that kernels raise on the device (0 otherwise), side by side so that one copy
        # brings both to the host: [0] a kernel's bounded pipeline wait ran out and its output is not
        # valid; [1] the embedding met a token id outside the vocabulary (one taken on the device from
        # the step before, which the host could not check).  See check_errors / raise_for_status.
        self.status = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.error_flag = self.status[0:1]
        self.token_error = self.status[1:2]
        # On request (CATENA_B200_FUSED_DECODE=1, or this attribute set before the first decode step) decode
        # steps of up to 16 bfloat16 sequences run their products, residual sums and convolutions in a few
        # persistent kernels (kernels.FusedDecode) instead of one launch per call.  Off by default: measured
        # slower than the recorded chain of single kernels (csrc/decode_fused.cu gives the figures).
        self.fused_decode = os.environ.get("CATENA_B200_FUSED_DECODE", "0") == "1"
        self.fused_bar = torch.zeros(4, dtype=torch.int32, device=self.device)     # the fused kernel's barrier word

    def check_errors(self):
        """Read the device flags (synchronises); raises `DeviceFault` if one is set."""
        self.raise_for_status(self.status.tolist())

    def raise_for_status(self, status):
        """`status`: the two flags as the host read them.  Clears the device flags and raises if one
        is set, so that no output of a step that went wrong is handed on as if it were valid."""
        wait, token = int(status[0]), int(status[1])
        if not (wait or token):
            return
        self.status.zero_()
        self.fused_bar.zero_()             # a fused kernel that gave up has left its barrier word half-way
        what = []
        if wait:
            what.append(f"a kernel's pipeline wait ran out (code {wait})")
        if token:
            what.append("a token id outside the vocabulary reached the embedding")
        raise DeviceFault("; ".join(what) + ": the step's output is not valid")

    def fused_decode_for(self, batch):
        """The collector for this step's fusable calls, or None: decode steps of the bfloat16 engine with
        at most 16 sequences."""
        if (self.fused_decode and self.dtype == torch.bfloat16 and batch.kind == "decode"
                and batch.T <= kernels.FD_MAX_ROWS):
            return kernels.FusedDecode(self.fused_bar, self.error_flag)
        return None

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
    def linear(self, x, w, out_dtype=None, partial_ok=False):
        """y = x @ w^T; y in the activation dtype unless `out_dtype` says float32.  With `partial_ok`
        the caller can take `kernels.PartialSums` instead (the product cut over K, to be added by the
        fused residual kernel): used where it spares the product an exchange between its blocks."""
        kind = self._product_kernel(x, w)
        # Partial sums at 9 to 16 rows: the tcgen05 kernel's eight slices beat the streaming kernel's four
        # (measured on B200 at 16 rows, us: 2,048 x 2,048 5.0 -> 4.0, 2,048 x 8,192 10.4 -> 8.9, 2,048 x 10,752
        # 13.1 -> 10.1, 1,024 x 4,608 6.1 -> 5.3; at 8 rows the streaming kernel is level or ahead)
        if (partial_ok and out_dtype is None and kind == "skinny" and 8 < x.shape[0] <= self.SKINNY_BEST_ROWS
                and w.shape[1] >= 2048 and self._tma_operands(x, w) and self._few_rows_slices(w.shape[0], w.shape[1]) > 1):
            kind = "few_rows"
        # ... and so does a finished product of that size (q/k/v at 16 rows: 7.0 -> 6.0 us; in_proj keeps the
        # streaming kernel, which takes the convolution along)
        if (not partial_ok and out_dtype is None and kind == "skinny" and 8 < x.shape[0] <= self.SKINNY_BEST_ROWS
                and w.shape[1] >= 2048 and self._tma_operands(x, w)):
            kind = "few_rows"
        if partial_ok and out_dtype is None and kind == "skinny" and x.shape[0] <= self.SKINNY_BEST_ROWS:
            slices = self._skinny_slices(w.shape[0], w.shape[1])
            if slices > 1:
                parts = torch.empty((slices, x.shape[0], w.shape[0]), dtype=torch.float32, device=x.device)
                kernels.gemm_skinny_parts(parts, x, w)
                return kernels.PartialSums(parts, x.dtype)
        if partial_ok and out_dtype is None and kind == "few_rows":
            slices = self._few_rows_slices(w.shape[0], w.shape[1])
            if slices > 1:
                parts = torch.empty((slices, x.shape[0], w.shape[0]), dtype=torch.float32, device=x.device)
                kernels.gemm_tc_few_rows_parts(parts, x, w, err=self.error_flag)
                return kernels.PartialSums(parts, x.dtype)
        if partial_ok and out_dtype is None and kind == "tiled":
            slices, width = self._tiled_slices(x.shape[0], w.shape[0], w.shape[1])
            if slices > 1:
                parts = torch.empty((slices, x.shape[0], w.shape[0]), dtype=torch.float32, device=x.device)
                kernels.gemm_tc_parts(parts, x, w, err=self.error_flag, block_n=width)
                return kernels.PartialSums(parts, x.dtype)
        y = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype or x.dtype, device=x.device)
        if kind == "skinny":
            kernels.gemm_skinny(y, x, w)
        elif kind == "few_rows":
            kernels.gemm_tc_few_rows(y, x, w, err=self.error_flag)
        elif kind == "tiled":
            widths = (256, 192, 128) if y.dtype == torch.bfloat16 else (256, 128)
            kernels.gemm_tc(y, x, w, err=self.error_flag, block_n=self._tile_width(x.shape[0], w.shape[0], widths))
        else:
            kernels.gemm_simt(y, x, w)
        return y

    SKINNY_SLICES = 4

    def _skinny_slices(self, out_columns, inner):
        """Into how many slices of K the weight-streaming product is cut when its consumer adds the
        slices: products with few row tiles (at most 160 tiles of 16 output columns), whose blocks
        would otherwise leave SMs idle or exchange sums through a cluster."""
        tiles = -(-out_columns // 16)
        if tiles > 160 or inner < 64 * self.SKINNY_SLICES:
            return 1
        return self.SKINNY_SLICES

    def _few_rows_slices(self, out_columns, inner):
        """Slices of K for the few-rows product when its consumer adds them: as many blocks as 1.4
        per SM (the rule the kernel uses for its clusters), each with two 64-wide steps at least."""
        if self._sm_count is None:
            self._sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        tiles = -(-out_columns // 128)
        steps = -(-inner // 64)
        for s in range(8, 1, -1):
            if 2 * s <= steps and 5 * tiles * s <= 7 * self._sm_count:
                return s
        return 1

    def _tiled_slices(self, rows, out_columns, inner):
        """(runs of K, tile width) for the tiled product when its consumer adds the runs.  A few hundred rows
        times a narrow output are a few dozen tiles for 148 SMs, and the kernel takes (run, tile) items: the
        pair with the least estimated time, which is rounds of items over the SMs x k-steps of an item x the
        measured cost of a k-step at that width (TILE_STEP_US), plus, for more than one run, what the float
        runs cost on their way through the residual kernel (about 1 us per run and 1.5 us once, per million
        outputs).  Measured on B200 (us, with the residual kernel, best pair first): 256 x 2,048 x 2,048
        (4, 128) 11.1, (8, 256) 12.3, unsplit 12.8+; 256 x 2,048 x 8,192 (8, 256) 18.6, (4, 128) 19.2;
        1,024 x 2,048 x 8,192 (2, 256) 40.1, (4, 256) 44.0, unsplit 49.9; 1,024 x 2,048 x 2,048 unsplit 19.6,
        (2, 256) 21.7; whole steps at 1.7B-class sizes: 256 tokens 2.57 -> 2.00 ms, 512 tokens 3.08 -> 2.64."""
        known = self._choices.get(("slices", rows, out_columns, inner))
        if known is not None:
            return known
        if self._sm_count is None:
            self._sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        steps = -(-inner // 64)
        row_tiles = -(-rows // 128)
        outputs = rows * out_columns / 1e6

        def estimate(width, runs):
            items = row_tiles * -(-out_columns // width) * runs
            time = -(-items // self._sm_count) * -(-steps // runs) * self.TILE_STEP_US[width]
            return time + (outputs * (runs + 1.5) if runs > 1 else 0.0)

        best = (min(estimate(w, 1) for w in (128, 192, 256)), 1, 256)
        if out_columns % 4 == 0:
            for width in (256, 128):
                for runs in range(2, 9):
                    per = -(-steps // runs)
                    if per < 2 or per * (runs - 1) >= steps:
                        continue
                    t = estimate(width, runs)
                    if t < 0.95 * best[0]:                  # a split has to pay clearly
                        best = (t, runs, width)
        self._choices[("slices", rows, out_columns, inner)] = best[1:]
        return best[1], best[2]

    # time of one 64-wide step of K on one tile, us, measured on B200 over 72 shapes (256 to 4,096 rows):
    # a product takes about 4.5 us + rounds of tiles over the SMs x steps x this, whatever the width
    TILE_STEP_US = {128: 0.30, 192: 0.33, 256: 0.35}

    def _tile_width(self, rows, out_columns, widths=(256, 192, 128)):
        """The tile width of the tiled product: the one whose tiles need the fewest rounds over the SMs,
        weighted by what a step of K costs at that width (a 128 x 128 tile is bound by the operands'
        way from L2, not by the tensor core, so it is not half the price of a 128 x 256 one).  Measured:
        1,024 x 6,144 x 2,048 34.6 / 26.0 / 27.2 us at 128 / 192 / 256, 512 x 6,144 x 2,048 23.8 / 15.4 /
        16.3, 2,048 x 2,048 x 8,192 81.6 / 83.0 / 50.6, 256 x 6,144 x 2,048 14.0 / 14.9 / 15.6."""
        known = self._choices.get(("width", rows, out_columns, widths))
        if known is not None:
            return known
        if self._sm_count is None:
            self._sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        row_tiles = -(-rows // 128)
        cost = {w: -(-(row_tiles * -(-out_columns // w)) // self._sm_count) * self.TILE_STEP_US[w] for w in widths}
        best = min(widths, key=lambda w: (cost[w], -w))
        self._choices[("width", rows, out_columns, widths)] = best
        return best

    SKINNY_ROWS = 64          # most rows the weight-streaming kernel takes
    SKINNY_BEST_ROWS = 16     # up to here it is the fastest kernel
    FEW_ROWS = 128            # most rows of the tensor-core kernel that splits K over a cluster

    def _product_kernel(self, x, w):
        """Which kernel multiplies x by w^T.  Up to 16 bfloat16 rows: the weight-streaming mma.sync
        kernel (decode steps of small batches, wanted rows of the head).  Up to 128 rows: the
        tcgen05 kernel that splits K over a cluster when there are few column tiles (measured on
        B200 at 64 rows, 2048 x 8192: 12.4 us against 26.0 us for the streaming kernel, which
        re-reads the activations once per 16 weight rows).  More rows: the persistent tcgen05
        kernel with 128 x 256 tiles.  Operands that TMA cannot take (pitch or base not 16-byte
        aligned) fall to the streaming kernel while it takes the rows, else to the CUDA-core one,
        which is also the float32 path."""
        rows = x.shape[0]
        if self._in_prompt and not self.tensor_core_prompts:
            return "simt"
        bf16 = x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
        streams = (bf16 and rows <= self.SKINNY_ROWS and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
                   and x.data_ptr() % 16 == 0)
        tma = self._tma_operands(x, w)
        if streams and (rows <= self.SKINNY_BEST_ROWS or not tma):
            return "skinny"
        if tma:
            return "few_rows" if rows <= self.FEW_ROWS else "tiled"
        return "simt"

    @staticmethod
    def _tma_operands(x, w):
        """True if TMA can fetch both operands of x @ w^T (bfloat16, 16-byte aligned bases and row pitches)."""
        return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
                and x.stride(1) == 1 and x.data_ptr() % 16 == 0 and w.stride(0) % 8 == 0)

    def streams_weights(self, x, w):
        """True if x @ w^T goes to the weight-streaming kernel with at most 16 rows (a part may then use
        that kernel's fused forms, which take no more)."""
        return x.shape[0] <= self.SKINNY_BEST_ROWS and self._product_kernel(x, w) == "skinny"

    def gate_up_swiglu(self, x, w_gate_up, F):
        """a = silu(x Wgate^T) * (x Wup^T) for the row-packed [Wgate; Wup]."""
        a = torch.empty((x.shape[0], F), dtype=x.dtype, device=x.device)
        kind = self._product_kernel(x, w_gate_up)
        # From 9 rows on the tcgen05 few-rows kernel leads (measured on B200 at 16 rows, us, streaming /
        # few-rows: 21,504 x 2,048 weights 25.5 / 20.2, 16,384 x 2,048 15.6 / 14.2, 9,216 x 1,024 7.7 / 7.4; at 8
        # rows the streaming kernel leads everywhere).
        if kind == "skinny" and x.shape[0] > 8 and self._tma_operands(x, w_gate_up):
            kind = "few_rows"
        if kind == "skinny":
            kernels.gemm_skinny(a, x, w_gate_up, swiglu=True)
            return a
        if kind == "few_rows":
            kernels.gemm_tc_few_rows(a, x, w_gate_up, swiglu=True, err=self.error_flag)
            return a
        if kind == "tiled":
            # a 256-wide tile of the packed matrix gives 128 output columns
            kernels.gemm_tc(a, x, w_gate_up, swiglu=True, err=self.error_flag,
                            block_n=self._tile_width(x.shape[0], 2 * F, widths=(256, 128)))
            return a
        gu = self.linear(x, w_gate_up)
        kernels.swiglu(a, gu)
        return a

    # ------------------------------------------------------------------ attention
    TCGEN05_ATTENTION_MIN_LEN = 768      # shorter prompts (or windows) give an item too few key tiles to pipeline ...
    TCGEN05_ATTENTION_MIN_LEN_BATCH = 256    # ... unless there are many of them:
    TCGEN05_ATTENTION_MIN_TOKENS = 2048      # this many rows in the step

    def attention_prefill(self, ctx, q, k, v, gate, batch, QH, KVH, HD, window, scale):
        """Attention of a prompt step over the step's own keys and values.  bfloat16 with head size
        64 or 128 and long sequences: the tcgen05 kernel (measured on B200, 32 heads of 64, tcgen05 against
        mma.sync: 18 / 25 us at 768 tokens, 22 / 35 at 1,024, 40 / 96 at 2,048, 664 against 264 TFLOP/s at
        16,384; heads of 128: 871 against 286; 8 prompts of 256: 17 / 20 us, 8 of 512: 37 / 52, 16 of
        1,100: 205 / 376, 64 of 300: 155 / 160; a window of 512 on 4,096 tokens: 57 / 87, of 256: 43 / 56.
        The mma.sync kernel is ahead for a single short prompt: 512 tokens 14.2 / 14.4 us, 256 tokens 7 /
        11, 128 tokens 4 / 9).  Other bfloat16 head sizes that are multiples of 16 up to 128: mma.sync.
        Everything else, and float32: CUDA cores."""
        aligned = (q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and k.data_ptr() % 16 == 0
                   and v.data_ptr() % 16 == 0)
        bf16 = q.dtype == torch.bfloat16 and self.tensor_core_prompts
        span = min(batch.max_len, window) if window else batch.max_len
        long_enough = span >= self.TCGEN05_ATTENTION_MIN_LEN or (
            span >= self.TCGEN05_ATTENTION_MIN_LEN_BATCH and q.shape[0] >= self.TCGEN05_ATTENTION_MIN_TOKENS)
        if (bf16 and aligned and HD in (64, 128) and long_enough
                and ctx.stride(0) % 8 == 0 and ctx.data_ptr() % 16 == 0):
            kernels.attn_prefill_tc(ctx, q, k, v, gate, batch.seq_start, batch.B, batch.max_len, QH, KVH, HD, window,
                                    scale, err=self.error_flag)
            return
        fn = kernels.attn_prefill_mma if (bf16 and aligned and HD % 16 == 0 and HD <= 128) else kernels.attn_prefill_simt
        fn(ctx, q, k, v, gate, batch.seq_start, batch.B, batch.max_len, QH, KVH, HD, window, scale)

    # Measured on B200, 32 heads of 64 over 8 kv heads, mma.sync against tcgen05:
    # 128 rows on 512 held tokens 20.9 / 17.0 us, on 256 held 13.4 / 13.3; 64 rows on 256 held 12.1 / 13.2; 16 rows x 8
    # sequences on 4,096 146 / 74 us, 8 rows x 8 on 4,096 146 / 73; 1,024 rows on 8,192 429 / 149 us (with a window of
    # 512: 38 / 19 us); 64 rows x 16 sequences on 2,048 108 / 79 us, on 192 held 17 / 27; 16 rows x 8 on 300 held 16 / 17.
    TCGEN05_APPEND_MIN_ROWS = 8
    TCGEN05_APPEND_MIN_SPAN = 512

    def attention_append(self, ctx, q, k, v, gate, batch, state, QH, KVH, HD, window, scale):
        """Attention of a step whose sequences already hold tokens: keys and values below each
        sequence's first position of the step come from the paged cache, the rest from the step's own
        rows (written to the cache by the caller afterwards).  The choice of kernel follows
        `attention_prefill`, with the span counted from the longest sequence's end and the tcgen05 kernel
        from shorter spans on (its blocks walk the past as well, so they are long enough to pipeline
        sooner)."""
        aligned = (q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and k.data_ptr() % 16 == 0
                   and v.data_ptr() % 16 == 0 and state.pool.data_ptr() % 16 == 0)
        bf16 = q.dtype == torch.bfloat16 and state.pool.dtype == torch.bfloat16 and self.tensor_core_prompts
        span = min(batch.max_end, window) if window else batch.max_end
        if (bf16 and aligned and HD in (64, 128) and span >= self.TCGEN05_APPEND_MIN_SPAN
                and batch.max_len >= self.TCGEN05_APPEND_MIN_ROWS and ctx.stride(0) % 8 == 0 and ctx.data_ptr() % 16 == 0):
            kernels.attn_append_tc(ctx, q, k, v, gate, batch.seq_start, batch.seq_pos0, batch.seq_slot, state.pool,
                                   state.pages, state.ptab, state.ring, batch.B, batch.max_len, QH, KVH, HD, window,
                                   scale, err=self.error_flag)
            return
        kernels.attn_append(ctx, q, k, v, gate, batch.seq_start, batch.seq_pos0, batch.seq_slot, state.pool,
                            state.pages, state.ptab, state.ring, batch.B, batch.max_len, QH, KVH, HD, window, scale,
                            tensor_cores=self.tensor_core_prompts)
