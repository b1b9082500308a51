// The operations that cm_fused_decode (decode_fused.cu) runs in one launch, as plain C structs: the
// host fills an FdSegment and passes it by value into the kernel's parameters (kernels.py mirrors
// the layout with ctypes).
#pragma once

#define FD_MAX_OPS 24

#define FD_KIND_GEMV 0          // y = x W^T for <= 16 bfloat16 rows
#define FD_KIND_ADD_NORM 1      // h_out = h_in + (norm(m) or m); n_out = norm(h_out)
#define FD_KIND_CONV 2          // the short convolution's decode form over in_proj's output

#define FD_MODE_PLAIN 0         // y bfloat16 [M, N]
#define FD_MODE_SWIGLU 1        // w = [gate; up] (2N rows); y = silu(x gate^T) * (x up^T), bfloat16 [M, N]
#define FD_MODE_PARTS 2         // y float [ksplit][M, N]: the sums over each slice of K, added by the consumer
#define FD_MODE_F32 3           // y float [M, N]

typedef struct {
    // GEMV: M rows, N outputs, K inner, ksplit slices of K.  ADD_NORM: M rows of width N, n_parts
    // partial sums (0: m is bfloat16).  CONV: M sequences, N channels, `taps` taps.
    int kind, mode, M, N, K, ksplit, n_parts, taps;
    long long ldx, ldw, ldy, part_stride;
    const void* x;              // GEMV: activations.  ADD_NORM: h_in.  CONV: in_proj's output [M][B | C | X]
    const void* w;              // GEMV: weights [N or 2N][K]
    void* y;                    // GEMV: output.  ADD_NORM: h_out.  CONV: output [M][N]
    const void* aux0;           // ADD_NORM: m (bfloat16) or its partial sums (float).  CONV: taps [N][taps] float
    const void* aux1;           // ADD_NORM: weight of the norm on m, or null
    const void* aux2;           // ADD_NORM: weight of the norm on h_out, or null (then no n_out)
    void* aux3;                 // ADD_NORM: n_out.  CONV: state [slots][taps - 1][N] float
    const int* idx;             // CONV: slot of each sequence
    float eps0, eps1;           // ADD_NORM: eps of the two norms
    int pad0, pad1;
} FdOp;

typedef struct {
    int n_ops;
    int pad[3];
    FdOp op[FD_MAX_OPS];
} FdSegment;
