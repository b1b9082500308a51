// Sizes that the kernels are built for and that the host must know before it launches anything.
// This header is the one place where they stand: the .cu files include it, and the Python side
// reads the same lines (limits.py), so a configuration is refused when it is read, with the same
// numbers that a kernel would refuse it with later.  cm_limit() hands out the compiled values so
// that a stale library is noticed at load.
#pragma once

#define CM_PAGE_TOKENS 64          // cache entries of one page
#define CM_ATTN_DECODE_CHUNK 256   // cache entries whose partial result one decode-attention piece leaves
#define CM_NORM_MAX_WIDTH 8192     // widest row the norm kernels keep in registers (8 * 256 threads * 4 chunks)
#define CM_MAX_HEAD_DIM 256        // largest head size of the attention and rotation kernels
#define CM_MAX_CONV_TAPS 16        // most taps of the short convolution
#define CM_SKINNY_MAX_ROWS 64      // most rows of the weight-streaming product
#define CM_FEW_ROWS_MAX_ROWS 128   // most rows of the tensor-core product that splits K
