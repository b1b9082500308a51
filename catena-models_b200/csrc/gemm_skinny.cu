// Y[M,N] = X[M,K] * W[N,K]^T for a handful of rows (decode steps): the weights are streamed
// once from HBM and are the 16-row operand of mma.sync.m16n8k16, the M <= 8*NT activation
// rows are its 8-wide operand ("swap A and B"), accumulation is float.
//
// A block owns 16 consecutive rows of W and one of gridDim.y slices of K; its 8 warps split the
// slice between them and their partial sums are added through shared memory in warp order.
// The gridDim.y blocks of a row tile form a thread-block cluster: block 0 of the cluster reads
// the others' sums from their shared memory (distributed shared memory) and adds them in rank
// order.  Every order is fixed, so the result does not depend on what else runs.  Every thread loads 16 contiguous bytes (8 values of k) per row
// and k-block of 32; the two mma steps of a k-block use those 8 values in an order that is
// the same for the W and the X fragment, so the sum over k is complete and each product is
// formed once (the instruction's own k order is irrelevant to a dot product).
//
// MODE_SWIGLU: W is the row-packed [Wgate; Wup] (2F rows); a block computes 16 gate rows with
// warps 0-3 and the matching 16 up rows with warps 4-7 and stores
// a = T(silu(T(g)) * T(u)) -- the reference's rounding points (lfm3_wmma.hex:10790-10815).
#include "common.cuh"
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

#define SK_WARPS 8
#define SK_MODE_PLAIN 0
#define SK_MODE_SWIGLU 1
#define SK_MODE_PARTS 2          // float partial sums per k-slice, no exchange between the blocks of a row tile

__device__ __forceinline__ void mma_bf16_16816(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream16(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// One warp's share of the product: the k-blocks b0 .. b1 of the weight rows w0 (fragment rows g) and
// w1 (rows g + 8) against all M activation rows.  Waits for the kernel before this one after the
// first weights are requested, and lets the next one start up right after.
template <int NT, int UNROLL>
__device__ __forceinline__ void skinny_stream(float (&acc)[NT][4], const bf16* __restrict__ X, const bf16* w0,
                                              const bf16* w1, bool v0, bool v1, int b0, int b1, int M, int K,
                                              long long ldx, int g, int t) {
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[n][j] = 0.f;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    // The weights of the first k-blocks are requested before this kernel waits for the one
    // before it: they are constants, and their latency hides behind the predecessor's tail.
    uint4 wa[UNROLL], wb[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        const int k = (b0 + u) * 32 + t * 8;
        const bool kv = b0 + u < b1 && k < K;
        wa[u] = (kv && v0) ? ld_stream16(w0 + k) : zero;
        wb[u] = (kv && v1) ? ld_stream16(w1 + k) : zero;
    }
    pdl_wait();
    pdl_trigger();                                 // what follows a product is a short kernel: let it start up now

    for (int blk = b0; blk < b1; blk += UNROLL) {
        uint4 xv[UNROLL][NT], na[UNROLL], nb[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = (blk + u) * 32 + t * 8;
            const bool kv = blk + u < b1 && k < K;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const int m = n * 8 + g;
                xv[u][n] = (kv && m < M) ? __ldg(reinterpret_cast<const uint4*>(X + (long long)m * ldx + k)) : zero;
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {                 // the next group of weights, in flight during the mma
            const int k = (blk + UNROLL + u) * 32 + t * 8;
            const bool kv = blk + UNROLL + u < b1 && k < K;
            na[u] = (kv && v0) ? ld_stream16(w0 + k) : zero;
            nb[u] = (kv && v1) ? ld_stream16(w1 + k) : zero;
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                mma_bf16_16816(acc[n], wa[u].x, wb[u].x, wa[u].y, wb[u].y, xv[u][n].x, xv[u][n].y);
                mma_bf16_16816(acc[n], wa[u].z, wb[u].z, wa[u].w, wb[u].w, xv[u][n].z, xv[u][n].w);
            }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            wa[u] = na[u];
            wb[u] = nb[u];
        }
    }
}

template <int NT, typename TY, int MODE, int UNROLL>
__global__ void __launch_bounds__(SK_WARPS * 32, NT <= 2 ? 4 : 2)
gemm_skinny_kernel(TY* __restrict__ Y, const bf16* __restrict__ X, const bf16* __restrict__ W, int M, int N,
                   int K, long long ldx, long long ldw, long long ldy, long long part_stride) {
    __shared__ float red[SK_WARPS][NT][32][4];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int r0 = blockIdx.x * 16;
    // plain: all 8 warps split K; swiglu: warps 0-3 take the gate rows, 4-7 the up rows
    const int splits = MODE == SK_MODE_SWIGLU ? SK_WARPS / 2 : SK_WARPS;
    const int part = MODE == SK_MODE_SWIGLU ? (warp & 3) : warp;
    const int row_base = (MODE == SK_MODE_SWIGLU && warp >= 4) ? N + r0 : r0;     // N = F in swiglu mode
    const int row_limit = (MODE == SK_MODE_SWIGLU && warp >= 4) ? 2 * N : N;
    const int nblk = (K + 31) >> 5;
    const int ksplit = gridDim.y;
    const int per_cta = (nblk + ksplit - 1) / ksplit;
    const int c0 = blockIdx.y * per_cta, c1 = min(nblk, c0 + per_cta);
    const int per = (per_cta + splits - 1) / splits;
    const int b0 = min(c1, c0 + part * per), b1 = min(c1, b0 + per);
    const bool v0 = row_base + g < row_limit, v1 = row_base + g + 8 < row_limit;
    const bf16* w0 = W + (long long)(row_base + g) * ldw;
    const bf16* w1 = W + (long long)(row_base + g + 8) * ldw;

    float acc[NT][4];
    skinny_stream<NT, UNROLL>(acc, X, w0, w1, v0, v1, b0, b1, M, K, ldx, g, t);
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j) red[warp][n][lane][j] = acc[n][j];
    __syncthreads();
    // element (n, lane, j): W row r0 + g (+8 for j >= 2), batch row 8n + 2t + (j & 1)
    constexpr int HALVES = MODE == SK_MODE_SWIGLU ? 2 : 1;
    __shared__ float csum[HALVES][NT * 128];
    for (int e = threadIdx.x; e < NT * 128; e += SK_WARPS * 32) {
        const int n = e >> 7, l = (e >> 2) & 31, j = e & 3;
        if (MODE == SK_MODE_SWIGLU) {
            float gsum = 0.f, usum = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) gsum += red[w][n][l][j];
#pragma unroll
            for (int w = 4; w < 8; ++w) usum += red[w][n][l][j];
            csum[0][e] = gsum;
            csum[HALVES - 1][e] = usum;
        } else {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < SK_WARPS; ++w) s += red[w][n][l][j];
            csum[0][e] = s;
        }
    }
    if (MODE == SK_MODE_PARTS) {
        // every k-slice leaves its sums where whoever consumes the product adds them in slice order
        __syncthreads();
        for (int e = threadIdx.x; e < NT * 128; e += SK_WARPS * 32) {
            const int n = e >> 7, l = (e >> 2) & 31, j = e & 3;
            const int row = r0 + (l >> 2) + (j >= 2 ? 8 : 0);
            const int m = n * 8 + (l & 3) * 2 + (j & 1);
            if (row < N && m < M) Y[(long long)blockIdx.y * part_stride + (long long)m * ldy + row] = from_f32<TY>(csum[0][e]);
        }
        return;
    }
    cg::cluster_group cluster = cg::this_cluster();
    if (ksplit > 1) cluster.sync(); else __syncthreads();
    if (blockIdx.y == 0) {
        for (int e = threadIdx.x; e < NT * 128; e += SK_WARPS * 32) {
            const int n = e >> 7, l = (e >> 2) & 31, j = e & 3;
            const int row = r0 + (l >> 2) + (j >= 2 ? 8 : 0);
            const int m = n * 8 + (l & 3) * 2 + (j & 1);
            float tot[HALVES];
#pragma unroll
            for (int hlf = 0; hlf < HALVES; ++hlf) {
                tot[hlf] = csum[hlf][e];
                for (int r = 1; r < ksplit; ++r) tot[hlf] += cluster.map_shared_rank(&csum[hlf][0], r)[e];
            }
            if (row >= N || m >= M) continue;
            if (MODE == SK_MODE_SWIGLU) {
                const float gr = rounded<TY>(tot[0]), ur = rounded<TY>(tot[HALVES - 1]);
                Y[(long long)m * ldy + row] = from_f32<TY>((gr * sigmoid_f32(gr)) * ur);
            } else {
                Y[(long long)m * ldy + row] = from_f32<TY>(tot[0]);
            }
        }
    }
    // The others' shared memory must outlive the reads.  Nothing is handed over here, so the arrival needs no
    // release (which would wait for this block's stores to Y): each thread arrives after its own reads.
    if (ksplit > 1) {
        asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
    }
}

template <int NT, typename TY, int MODE>
static int launch_skinny(void* Y, const void* X, const void* W, int M, int N, int K, long long ldx, long long ldw,
                         long long ldy, cudaStream_t st) {
    const int tiles = (N + 15) / 16;
    // Few row tiles with long rows leave most SMs idle: split K over a cluster of 4 blocks then.
    // (Measured on B200: 2048 x 8192 goes from 15.3 to 10.2 us; with K = 2048 the cluster's
    // barriers cost more than the extra blocks gain.)
    const int ksplit = (tiles <= 160 && K >= 4096) ? 4 : 1;
    // Two k-blocks per step and 64 registers: four blocks per SM (measured on B200: 6144 x 2048
    // goes from 8.6 to 6.7 us against four k-blocks per step at two blocks per SM).
    constexpr int UNROLL = 2;
    cm_launch_cluster(gemm_skinny_kernel<NT, TY, MODE, UNROLL>, dim3(tiles, ksplit), SK_WARPS * 32, 0, st, ksplit, false,
                      (TY*)Y, (const bf16*)X, (const bf16*)W, M, N, K, ldx, ldw, ldy, 0LL);
    CM_CHECK_LAUNCH();
    return CM_OK;
}

template <int NT>
static int launch_skinny_parts(float* P, const void* X, const void* W, int M, int N, int K, long long ldx, long long ldw,
                               long long ldp, long long part_stride, int ksplit, cudaStream_t st) {
    const int tiles = (N + 15) / 16;
    cm_launch_cluster(gemm_skinny_kernel<NT, float, SK_MODE_PARTS, 2>, dim3(tiles, ksplit), SK_WARPS * 32, 0, st, 1, false, P,
                      (const bf16*)X, (const bf16*)W, M, N, K, ldx, ldw, ldp, part_stride);
    CM_CHECK_LAUNCH();
    return CM_OK;
}

template <typename TY, int MODE>
static int dispatch_skinny(void* Y, const void* X, const void* W, int M, int N, int K, long long ldx, long long ldw,
                           long long ldy, cudaStream_t st) {
    if (M <= 8) return launch_skinny<1, TY, MODE>(Y, X, W, M, N, K, ldx, ldw, ldy, st);
    if (M <= 16) return launch_skinny<2, TY, MODE>(Y, X, W, M, N, K, ldx, ldw, ldy, st);
    if (M <= 32) return launch_skinny<4, TY, MODE>(Y, X, W, M, N, K, ldx, ldw, ldy, st);
    static_assert(CM_SKINNY_MAX_ROWS == 64, "cm_limits.h: CM_SKINNY_MAX_ROWS");
    if (M <= CM_SKINNY_MAX_ROWS) return launch_skinny<8, TY, MODE>(Y, X, W, M, N, K, ldx, ldw, ldy, st);
    CM_REFUSE("gemm_skinny: %d rows (at most %d)", M, CM_SKINNY_MAX_ROWS);
}

// P[s][m][n] = sum over the s-th of `ksplit` slices of K of X[m,k] W[n,k], float: the product with its
// inner dimension cut over independent blocks.  The slices are part_stride elements apart; the
// consumer (cm_add_norm with m_parts) adds them in slice order.  At most 16 rows.
extern "C" int cm_gemm_skinny_parts(float* P, const void* X, const void* W, int M, int N, int K, long long ldx,
                                    long long ldw, long long ldp, long long part_stride, int ksplit, cudaStream_t st) {
    if (M <= 0 || N <= 0) return CM_OK;
    if (M > 16) CM_REFUSE("gemm_skinny_parts: %d rows (at most 16)", M);
    if (ksplit < 1 || ksplit > 8) CM_REFUSE("gemm_skinny_parts: %d slices (1 to 8)", ksplit);
    if (K <= 0 || K % 8 || ldx % 8 || ldw % 8)
        CM_REFUSE("gemm_skinny_parts: inner size %d and row strides %lld, %lld must be multiples of 8", K, ldx, ldw);
    if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W)) & 15)
        CM_REFUSE("gemm_skinny_parts: operands must be 16-byte aligned");
    if (M <= 8) return launch_skinny_parts<1>(P, X, W, M, N, K, ldx, ldw, ldp, part_stride, ksplit, st);
    return launch_skinny_parts<2>(P, X, W, M, N, K, ldx, ldw, ldp, part_stride, ksplit, st);
}

// in_proj and the gated short convolution of a decode step in one kernel (one token per sequence).
// W is the in_proj matrix [B: H rows | C: H rows | X: H rows] x K.  A block owns 16 channels: warps
// 0-3 form the B rows of these channels, 4-7 the C rows, 8-11 the X rows, each group splitting K four
// ways; the sums are rounded to bfloat16 as the unfused product's output is, and then
//     bx = B * X;  z = sum_j taps[c][j] * s[j]  with s = (state[0 .. KT-2], bx);  y = T(z * C);
//     state <- s[1 .. KT-1]
// runs once per (sequence, channel), in the same order as shortconv_kernel does it.
#define SKC_WARPS 12

template <int NT, int UNROLL>
__global__ void __launch_bounds__(SKC_WARPS * 32, 1)
gemm_skinny_conv_kernel(bf16* __restrict__ Y, const bf16* __restrict__ X, const bf16* __restrict__ W,
                        const float* __restrict__ taps, float* __restrict__ state, const int* __restrict__ seq_slot,
                        int M, int H, int K, int KT, long long ldx, long long ldw, long long ldy) {
    __shared__ float red[SKC_WARPS][NT][32][4];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int r0 = blockIdx.x * 16;
    const int set = warp >> 2, part = warp & 3;
    const int nblk = (K + 31) >> 5;
    const int per = (nblk + 3) / 4;
    const int b0 = min(nblk, part * per), b1 = min(nblk, b0 + per);
    const bool v0 = r0 + g < H, v1 = r0 + g + 8 < H;
    const bf16* w0 = W + ((long long)set * H + r0 + g) * ldw;
    const bf16* w1 = W + ((long long)set * H + r0 + g + 8) * ldw;

    // The thread that will finish element e = threadIdx.x (NT * 128 of them, fewer than the block
    // has threads) asks for its channel's taps and its sequence's state now, so that they have
    // arrived when the sums are ready (up to 4 taps; more are read at the end).
    const int e = threadIdx.x;
    const int en = e >> 7, el = (e >> 2) & 31, ej = e & 3;
    const int c = r0 + (el >> 2) + (ej >= 2 ? 8 : 0);
    const int m = en * 8 + (el & 3) * 2 + (ej & 1);
    const bool owner = e < NT * 128 && c < H && m < M;
    const bool early = KT <= 4;
    float* st = nullptr;
    const float* wc = taps + (long long)c * KT;
    float s_pre[3] = {0.f, 0.f, 0.f}, w_pre[4] = {0.f, 0.f, 0.f, 0.f};
    if (owner) {
        st = state + (long long)seq_slot[m] * (KT - 1) * H + c;
        if (early) {
#pragma unroll
            for (int q = 0; q < 3; ++q)
                if (q < KT - 1) s_pre[q] = st[(long long)q * H];
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (q < KT) w_pre[q] = wc[q];
        }
    }

    float acc[NT][4];
    skinny_stream<NT, UNROLL>(acc, X, w0, w1, v0, v1, b0, b1, M, K, ldx, g, t);
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j) red[warp][n][lane][j] = acc[n][j];
    __syncthreads();
    if (!owner) return;
    float sum[3];
#pragma unroll
    for (int q = 0; q < 3; ++q) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) v += red[q * 4 + w][en][el][ej];
        sum[q] = rounded<bf16>(v);
    }
    const float bx = sum[0] * sum[2];
    float z = 0.f;
    if (early) {
#pragma unroll
        for (int q = 0; q < 3; ++q)
            if (q < KT - 1) {
                z += w_pre[q] * s_pre[q];
                if (q > 0) st[(long long)(q - 1) * H] = s_pre[q];        // shift: entry q becomes entry q - 1
            }
#pragma unroll
        for (int q = 1; q < 4; ++q)
            if (q == KT - 1) z += w_pre[q] * bx;
    } else {
        for (int q = 0; q < KT - 1; ++q) {
            const float sv = st[(long long)q * H];
            z += wc[q] * sv;
            if (q > 0) st[(long long)(q - 1) * H] = sv;
        }
        z += wc[KT - 1] * bx;
    }
    st[(long long)(KT - 2) * H] = bx;
    Y[(long long)m * ldy + c] = from_f32<bf16>(z * sum[1]);
}

// y[M, H] = the short convolution's output for M sequences that bring one token each; x [M, K],
// w [3H, K] bfloat16, taps [H][KT] float, state [slots][KT-1][H] float, seq_slot [M].
extern "C" int cm_gemm_skinny_shortconv(void* Y, const void* X, const void* W, const float* taps, float* state,
                                        const int* seq_slot, int M, int H, int K, int KT, long long ldx,
                                        long long ldw, long long ldy, cudaStream_t st) {
    if (M <= 0 || H <= 0) return CM_OK;
    if (M > 16) CM_REFUSE("gemm_skinny_shortconv: %d rows (at most 16)", M);
    if (KT < 2 || KT > CM_MAX_CONV_TAPS) CM_REFUSE("gemm_skinny_shortconv: %d taps (2..%d)", KT, CM_MAX_CONV_TAPS);
    if (K <= 0 || K % 8 || ldx % 8 || ldw % 8)
        CM_REFUSE("gemm_skinny_shortconv: inner size %d and row strides %lld, %lld must be multiples of 8", K, ldx, ldw);
    if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W)) & 15)
        CM_REFUSE("gemm_skinny_shortconv: operands must be 16-byte aligned");
    const int tiles = (H + 15) / 16;
    // one block per SM at most (H / 16 blocks): four k-blocks of weights in flight per thread
    constexpr int UNROLL = 4;
    if (M <= 8)
        cm_launch_cluster(gemm_skinny_conv_kernel<1, UNROLL>, dim3(tiles), SKC_WARPS * 32, 0, st, 1, false, (bf16*)Y,
                          (const bf16*)X, (const bf16*)W, taps, state, seq_slot, M, H, K, KT, ldx, ldw, ldy);
    else
        cm_launch_cluster(gemm_skinny_conv_kernel<2, UNROLL>, dim3(tiles), SKC_WARPS * 32, 0, st, 1, false, (bf16*)Y,
                          (const bf16*)X, (const bf16*)W, taps, state, seq_slot, M, H, K, KT, ldx, ldw, ldy);
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// X and W bfloat16; Y bfloat16 (dty = DT_BF16) or float (DT_F32).  swiglu: W has 2N rows
// ([gate; up]) and Y is [M, N].  K, ldx and ldw must be multiples of 8 (16-byte loads).
extern "C" int cm_gemm_skinny(int dty, void* Y, const void* X, const void* W, int M, int N, int K, long long ldx,
                              long long ldw, long long ldy, int swiglu, cudaStream_t st) {
    if (M <= 0 || N <= 0) return CM_OK;
    if (K <= 0 || K % 8 || ldx % 8 || ldw % 8)
        CM_REFUSE("gemm_skinny: inner size %d and row strides %lld, %lld must be multiples of 8", K, ldx, ldw);
    if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W)) & 15)
        CM_REFUSE("gemm_skinny: operands must be 16-byte aligned");
    if (swiglu) {
        if (dty != DT_BF16) return CM_ERR_DTYPE;
        return dispatch_skinny<bf16, SK_MODE_SWIGLU>(Y, X, W, M, N, K, ldx, ldw, ldy, st);
    }
    if (dty == DT_BF16) return dispatch_skinny<bf16, SK_MODE_PLAIN>(Y, X, W, M, N, K, ldx, ldw, ldy, st);
    if (dty == DT_F32) return dispatch_skinny<float, SK_MODE_PLAIN>(Y, X, W, M, N, K, ldx, ldw, ldy, st);
    return CM_ERR_DTYPE;
}
