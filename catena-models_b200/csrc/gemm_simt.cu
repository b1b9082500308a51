// Y[M,N] = X[M,K] * W[N,K]^T on the CUDA cores, float accumulation with plain FMAs.
//
// This is the matrix product of the true 32-bit path (no tensor-core mode of reduced
// precision is involved) and the any-size fallback of the bfloat16 path.  Every output
// element is one thread's running sum over k = 0..K-1 in increasing order, so a row's
// result does not depend on M, on the tile it falls in, or on its batch-mates.
#include "common.cuh"

#define GS_BM 64
#define GS_BN 64
#define GS_BK 16

template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(TY* __restrict__ Y, const TX* __restrict__ X, const TW* __restrict__ W, int M,
                 int N, int K, long long ldx, long long ldw, long long ldy) {
    pdl_trigger();
    pdl_wait();
    __shared__ float xs[GS_BK][GS_BM + 1];
    __shared__ float ws[GS_BK][GS_BN + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // 16 x 16 threads, 4 x 4 outputs each
    const int m0 = blockIdx.y * GS_BM, n0 = blockIdx.x * GS_BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GS_BK) {
        // 64 rows x 16 k per operand = 1024 elements, 4 per thread
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = threadIdx.x + i * 256;
            const int r = e >> 4, k = e & 15;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + k;
            xs[k][r] = (gm < M && gk < K) ? to_f32(X[(long long)gm * ldx + gk]) : 0.f;
            ws[k][r] = (gn < N && gk < K) ? to_f32(W[(long long)gn * ldw + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GS_BK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) Y[(long long)gm * ldy + gn] = from_f32<TY>(acc[i][j]);
        }
    }
}

template <typename TX, typename TW, typename TY>
static int launch_simt(void* Y, const void* X, const void* W, int M, int N, int K, long long ldx,
                       long long ldw, long long ldy, cudaStream_t st) {
    dim3 grid((N + GS_BN - 1) / GS_BN, (M + GS_BM - 1) / GS_BM);
    cm_launch(gemm_simt_kernel<TX, TW, TY>, grid, 256, 0, st, (TY*)Y, (const TX*)X, (const TW*)W, M, N, K,
                                                       ldx, ldw, ldy);
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// dtx / dtw / dty: DT_F32 or DT_BF16 of X, W and Y.  Supported: all-float; bf16 X and W with
// bf16 or float Y; bf16 X with float W (a matrix that the file stores in 32 bits) and bf16 or
// float Y.
extern "C" int cm_gemm_simt(int dtx, int dtw, int dty, void* Y, const void* X, const void* W, int M,
                            int N, int K, long long ldx, long long ldw, long long ldy,
                            cudaStream_t st) {
    if (M <= 0 || N <= 0) return CM_OK;
    if (K <= 0) CM_REFUSE("gemm: inner size %d", K);
    if (dtx == DT_F32 && dtw == DT_F32 && dty == DT_F32)
        return launch_simt<float, float, float>(Y, X, W, M, N, K, ldx, ldw, ldy, st);
    if (dtx == DT_BF16 && dtw == DT_BF16 && dty == DT_BF16)
        return launch_simt<bf16, bf16, bf16>(Y, X, W, M, N, K, ldx, ldw, ldy, st);
    if (dtx == DT_BF16 && dtw == DT_BF16 && dty == DT_F32)
        return launch_simt<bf16, bf16, float>(Y, X, W, M, N, K, ldx, ldw, ldy, st);
    if (dtx == DT_BF16 && dtw == DT_F32 && dty == DT_BF16)
        return launch_simt<bf16, float, bf16>(Y, X, W, M, N, K, ldx, ldw, ldy, st);
    if (dtx == DT_BF16 && dtw == DT_F32 && dty == DT_F32)
        return launch_simt<bf16, float, float>(Y, X, W, M, N, K, ldx, ldw, ldy, st);
    return CM_ERR_DTYPE;
}
