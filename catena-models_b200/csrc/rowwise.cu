// Row-wise kernels: embedding gather, RMSNorm, fused post-norm + residual + next norm,
// SwiGLU product, row gather.  One block per row; all sums in float, in a fixed order.
#include "common.cuh"

// ------------------------------------------------------------------ embedding gather
// out[t,:] = table[tokens[t],:].  A token id outside [0,V) writes zeros and raises *err.
// With `sampled` given, a negative entry -(1 + i) stands for sampled[i]: the token that the step
// before this one chose on the device for its i-th sequence, which the host has not seen yet.
// The table may be stored in another type than the activations (a checkpoint that keeps it in
// 32-bit under a bfloat16 engine): the row is converted as it is read.
template <typename T, typename TT>
__global__ void embed_gather_kernel(T* __restrict__ out, const TT* __restrict__ table,
                                    const int* __restrict__ tokens, const int* __restrict__ sampled, int H, int V,
                                    float scale, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    int tok = tokens[t];
    if (tok < 0 && sampled) tok = sampled[-tok - 1];
    const bool ok = tok >= 0 && tok < V;
    if (!ok && threadIdx.x == 0 && err) atomicExch(err, 1);
    const TT* src = table + (long long)(ok ? tok : 0) * H;
    T* dst = out + (long long)t * H;
    // scale: the factor some architectures put on their embeddings (1 leaves the row as it is)
    for (int c = threadIdx.x; c < H; c += blockDim.x) dst[c] = from_f32<T>(ok ? to_f32(src[c]) * scale : 0.f);
}

extern "C" int cm_embed_gather(int dt, int dt_table, void* out, const void* table, const int* tokens,
                               const int* sampled, int T, int H, int V, float scale, int* err, cudaStream_t st) {
    if (T <= 0) return CM_OK;
    const int threads = H >= 1024 ? 256 : 128;
    if (dt == DT_F32 && dt_table == DT_F32)
        cm_launch(embed_gather_kernel<float, float>, T, threads, 0, st, (float*)out, (const float*)table, tokens, sampled, H, V, scale, err);
    else if (dt == DT_BF16 && dt_table == DT_BF16)
        cm_launch(embed_gather_kernel<bf16, bf16>, T, threads, 0, st, (bf16*)out, (const bf16*)table, tokens, sampled, H, V, scale, err);
    else if (dt == DT_BF16 && dt_table == DT_F32)
        cm_launch(embed_gather_kernel<bf16, float>, T, threads, 0, st, (bf16*)out, (const float*)table, tokens, sampled, H, V, scale, err);
    else if (dt == DT_F32 && dt_table == DT_BF16)
        cm_launch(embed_gather_kernel<float, bf16>, T, threads, 0, st, (float*)out, (const bf16*)table, tokens, sampled, H, V, scale, err);
    else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// ---------------------------------------------------------------- rows in registers
// The norm kernels keep a row in registers: a thread owns chunks of 8 consecutive elements,
// chunk c of thread t starts at (c * blockDim.x + t) * 8.  All global loads of a row are
// issued before the first reduction.  H must be a multiple of 8 and at most 8 * 256 * NV_MAXC.
#define NV_THREADS 256
#define NV_MAXC 4
static_assert(8 * NV_THREADS * NV_MAXC == CM_NORM_MAX_WIDTH, "cm_limits.h: CM_NORM_MAX_WIDTH");

// -------------------------------------------------------------------------- RMSNorm
// y = T((x * inv) * w), inv = 1/sqrt(mean(x^2) + eps); w is float.
template <typename T, int C>
__global__ void __launch_bounds__(NV_THREADS)
rmsnorm_kernel(T* __restrict__ y, const T* __restrict__ x, const float* __restrict__ w, int H, float eps,
               long long ldx, long long ldy) {
    __shared__ float scratch[32];
    pdl_trigger();
    float wv[C][8], xv[C][8];
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int e = (c * NV_THREADS + threadIdx.x) * 8;
        if (e < H) load8f<float>(w + e, wv[c]);
    }
    pdl_wait();
    const T* xr = x + (long long)blockIdx.x * ldx;
    T* yr = y + (long long)blockIdx.x * ldy;
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int e = (c * NV_THREADS + threadIdx.x) * 8;
        if (e < H) {
            load8f<T>(xr + e, xv[c]);
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += xv[c][i] * xv[c][i];
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)H + eps);
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int e = (c * NV_THREADS + threadIdx.x) * 8;
        if (e < H) {
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = (xv[c][i] * inv) * wv[c][i];
            store8f<T>(yr + e, o);
        }
    }
}

template <typename T>
static int launch_rmsnorm(void* y, const void* x, const float* w, int rows, int H, float eps, long long ldx,
                          long long ldy, cudaStream_t st) {
    const int chunks = (H / 8 + NV_THREADS - 1) / NV_THREADS;
    if (chunks <= 1)
        cm_launch(rmsnorm_kernel<T, 1>, rows, NV_THREADS, 0, st, (T*)y, (const T*)x, w, H, eps, ldx, ldy);
    else if (chunks <= 2)
        cm_launch(rmsnorm_kernel<T, 2>, rows, NV_THREADS, 0, st, (T*)y, (const T*)x, w, H, eps, ldx, ldy);
    else
        cm_launch(rmsnorm_kernel<T, NV_MAXC>, rows, NV_THREADS, 0, st, (T*)y, (const T*)x, w, H, eps, ldx, ldy);
    CM_CHECK_LAUNCH();
    return CM_OK;
}

extern "C" int cm_rmsnorm(int dt, void* y, const void* x, const float* w, int rows, int H,
                          float eps, long long ldx, long long ldy, cudaStream_t st) {
    if (rows <= 0) return CM_OK;
    if (H % 8 || H > 8 * NV_THREADS * NV_MAXC || ldx % 8 || ldy % 8)
        CM_REFUSE("rmsnorm: width %d (strides %lld, %lld) must be a multiple of 8, at most %d", H, ldx, ldy,
                  8 * NV_THREADS * NV_MAXC);
    if (((uintptr_t)y | (uintptr_t)x | (uintptr_t)w) & 15) CM_REFUSE("rmsnorm: operands must be 16-byte aligned");
    if (dt == DT_F32) return launch_rmsnorm<float>(y, x, w, rows, H, eps, ldx, ldy, st);
    if (dt == DT_BF16) return launch_rmsnorm<bf16>(y, x, w, rows, H, eps, ldx, ldy, st);
    return CM_ERR_DTYPE;
}

// ------------------------------------------------- residual add with both norms fused
// d      = w_post ? T((m * inv(m)) * w_post) : m          (post-norm of the part's output)
// h_out  = T(h_in + d)                                    (sum in float)
// n_out  = w_next ? T((h_out * inv(h_out)) * w_next)      (pre-norm of whatever runs next,
//                                                          taken over the stored h_out)
// h_out may alias h_in.  The row stays in registers between the passes.
template <typename T, int C>
__global__ void __launch_bounds__(NV_THREADS)
add_norm_kernel(T* __restrict__ h_out, T* __restrict__ n_out, const T* __restrict__ m,
                const T* __restrict__ h_in, const float* __restrict__ w_post,
                const float* __restrict__ w_next, int H, float eps_post, float eps_next) {
    __shared__ float scratch[32];
    pdl_trigger();
    float wp[C][8], wn[C][8], mv[C][8], hv[C][8];
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int e = (c * NV_THREADS + threadIdx.x) * 8;
        if (e < H) {
            if (w_post) load8f<float>(w_post + e, wp[c]);
            if (w_next) load8f<float>(w_next + e, wn[c]);
        }
    }
    pdl_wait();
    const long long off = (long long)blockIdx.x * H;
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int e = (c * NV_THREADS + threadIdx.x) * 8;
        if (e < H) {
            load8f<T>(m + off + e, mv[c]);
            load8f<T>(h_in + off + e, hv[c]);
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += mv[c][i] * mv[c][i];
        }
    }
    float inv_post = 1.f;
    if (w_post) {
        ss = block_sum(ss, scratch);
        inv_post = 1.f / sqrtf(ss / (float)H + eps_post);
    }
    float ss2 = 0.f;
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int e = (c * NV_THREADS + threadIdx.x) * 8;
        if (e < H) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float d = w_post ? rounded<T>((mv[c][i] * inv_post) * wp[c][i]) : mv[c][i];
                const float hn = rounded<T>(hv[c][i] + d);
                hv[c][i] = hn;
                ss2 += hn * hn;
            }
            store8f<T>(h_out + off + e, hv[c]);
        }
    }
    if (!w_next) return;
    ss2 = block_sum(ss2, scratch);
    const float inv_next = 1.f / sqrtf(ss2 / (float)H + eps_next);
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int e = (c * NV_THREADS + threadIdx.x) * 8;
        if (e < H) {
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = (hv[c][i] * inv_next) * wn[c][i];
            store8f<T>(n_out + off + e, o);
        }
    }
}

// The same with m as n_parts float partial sums [n_parts][rows][H] (a product that split its inner dimension
// over blocks left them); they are added in index order and rounded to T, which is the value the product would
// have stored itself.  A block takes the rows blockIdx.x, + gridDim.x, ...; with more rows than NV_BLOCKS_PER_SM
// blocks an SM the next row's loads are in flight while this row's two sums and stores run.  (Measured against
// the form above with the sums folded in: a decode step of 8 rows 1.117 against 1.133 ms over its 48 calls,
// 1,024 rows over two sums 10.0 against 10.7 us; for whole tensors the form above is ahead, 9.4 against 11.0 us
// at 2,048 rows.)
template <typename T, int C>
__global__ void __launch_bounds__(NV_THREADS)
add_norm_parts_kernel(T* __restrict__ h_out, T* __restrict__ n_out,
                const float* __restrict__ m_parts, int n_parts, long long part_stride,
                const T* __restrict__ h_in, const float* __restrict__ w_post,
                const float* __restrict__ w_next, int rows, int H, float eps_post, float eps_next) {
    __shared__ float scratch[32];
    pdl_trigger();
    float wp[C][8], wn[C][8], mv[C][8], hv[C][8], mv_next[C][8], hv_next[C][8];
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int e = (c * NV_THREADS + threadIdx.x) * 8;
        if (e < H) {
            if (w_post) load8f<float>(w_post + e, wp[c]);
            if (w_next) load8f<float>(w_next + e, wn[c]);
        }
    }
    pdl_wait();
    // the row's m (the partial sums added in index order and rounded) and h_in
    auto load_row = [&](int row, float (*mr)[8], float (*hr)[8]) {
        const long long off = (long long)row * H;
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int e = (c * NV_THREADS + threadIdx.x) * 8;
            if (e < H) {
                float part[8][8];
#pragma unroll
                for (int r = 0; r < 8; ++r)
                    if (r < n_parts) load8f<float>(m_parts + (long long)r * part_stride + off + e, part[r]);
                load8f<T>(h_in + off + e, hr[c]);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float acc = 0.f;
#pragma unroll
                    for (int r = 0; r < 8; ++r)
                        if (r < n_parts) acc += part[r][i];
                    mr[c][i] = rounded<T>(acc);
                }
            }
        }
    };
    int row = blockIdx.x;
    if (row >= rows) return;
    load_row(row, mv, hv);
    while (true) {
        const int next = row + gridDim.x;                         // the same for every thread of the block
        if (next < rows) load_row(next, mv_next, hv_next);
        const long long off = (long long)row * H;
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int e = (c * NV_THREADS + threadIdx.x) * 8;
            if (e < H) {
#pragma unroll
                for (int i = 0; i < 8; ++i) ss += mv[c][i] * mv[c][i];
            }
        }
        float inv_post = 1.f;
        if (w_post) {
            ss = block_sum(ss, scratch);
            inv_post = 1.f / sqrtf(ss / (float)H + eps_post);
        }
        float ss2 = 0.f;
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int e = (c * NV_THREADS + threadIdx.x) * 8;
            if (e < H) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float d = w_post ? rounded<T>((mv[c][i] * inv_post) * wp[c][i]) : mv[c][i];
                    const float hn = rounded<T>(hv[c][i] + d);
                    hv[c][i] = hn;
                    ss2 += hn * hn;
                }
                store8f<T>(h_out + off + e, hv[c]);
            }
        }
        if (w_next) {
            ss2 = block_sum(ss2, scratch);
            const float inv_next = 1.f / sqrtf(ss2 / (float)H + eps_next);
#pragma unroll
            for (int c = 0; c < C; ++c) {
                const int e = (c * NV_THREADS + threadIdx.x) * 8;
                if (e < H) {
                    float o[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[i] = (hv[c][i] * inv_next) * wn[c][i];
                    store8f<T>(n_out + off + e, o);
                }
            }
        }
        if (next >= rows) break;
        row = next;
#pragma unroll
        for (int c = 0; c < C; ++c)
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                mv[c][i] = mv_next[c][i];
                hv[c][i] = hv_next[c][i];
            }
    }
}

#define NV_BLOCKS_PER_SM 4

template <typename T>
static int launch_add_norm(void* h_out, void* n_out, const void* m, const void* h_in, const float* w_post,
                           const float* w_next, int rows, int H, float eps_post, float eps_next, cudaStream_t st) {
    const int chunks = (H / 8 + NV_THREADS - 1) / NV_THREADS;
    if (chunks <= 1)
        cm_launch(add_norm_kernel<T, 1>, rows, NV_THREADS, 0, st, (T*)h_out, (T*)n_out, (const T*)m, (const T*)h_in, w_post,
                  w_next, H, eps_post, eps_next);
    else if (chunks <= 2)
        cm_launch(add_norm_kernel<T, 2>, rows, NV_THREADS, 0, st, (T*)h_out, (T*)n_out, (const T*)m, (const T*)h_in, w_post,
                  w_next, H, eps_post, eps_next);
    else
        cm_launch(add_norm_kernel<T, NV_MAXC>, rows, NV_THREADS, 0, st, (T*)h_out, (T*)n_out, (const T*)m, (const T*)h_in,
                  w_post, w_next, H, eps_post, eps_next);
    CM_CHECK_LAUNCH();
    return CM_OK;
}

template <typename T>
static int launch_add_norm_parts(void* h_out, void* n_out, const float* m_parts, int n_parts, long long part_stride,
                                 const void* h_in, const float* w_post, const float* w_next, int rows, int H,
                                 float eps_post, float eps_next, cudaStream_t st) {
    const int chunks = (H / 8 + NV_THREADS - 1) / NV_THREADS;
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count <= 0) sm_count = 1;
    }
    const int blocks = rows < NV_BLOCKS_PER_SM * sm_count ? rows : NV_BLOCKS_PER_SM * sm_count;
    if (chunks <= 1)
        cm_launch(add_norm_parts_kernel<T, 1>, blocks, NV_THREADS, 0, st, (T*)h_out, (T*)n_out, m_parts, n_parts,
                  part_stride, (const T*)h_in, w_post, w_next, rows, H, eps_post, eps_next);
    else if (chunks <= 2)
        cm_launch(add_norm_parts_kernel<T, 2>, blocks, NV_THREADS, 0, st, (T*)h_out, (T*)n_out, m_parts, n_parts,
                  part_stride, (const T*)h_in, w_post, w_next, rows, H, eps_post, eps_next);
    else
        cm_launch(add_norm_parts_kernel<T, NV_MAXC>, blocks, NV_THREADS, 0, st, (T*)h_out, (T*)n_out, m_parts, n_parts,
                  part_stride, (const T*)h_in, w_post, w_next, rows, H, eps_post, eps_next);
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// m: [rows, H] in the activation dtype, or (m_parts given) n_parts float partial sums of it,
// part_stride elements apart, each [rows, H].
extern "C" int cm_add_norm(int dt, void* h_out, void* n_out, const void* m, const float* m_parts, int n_parts,
                           long long part_stride, const void* h_in, const float* w_post, const float* w_next,
                           int rows, int H, float eps_post, float eps_next, cudaStream_t st) {
    if (rows <= 0) return CM_OK;
    if (H % 8 || H > 8 * NV_THREADS * NV_MAXC)
        CM_REFUSE("add_norm: width %d must be a multiple of 8, at most %d", H, 8 * NV_THREADS * NV_MAXC);
    if (((uintptr_t)h_out | (uintptr_t)n_out | (uintptr_t)m | (uintptr_t)m_parts | (uintptr_t)h_in | (uintptr_t)w_post |
         (uintptr_t)w_next) & 15)
        CM_REFUSE("add_norm: operands must be 16-byte aligned");
    if (m_parts) {
        if (n_parts < 1 || n_parts > 8 || part_stride % 4)
            CM_REFUSE("add_norm: %d partial sums (1 to 8), %lld elements apart (a multiple of 4)", n_parts, part_stride);
        if (dt == DT_F32)
            return launch_add_norm_parts<float>(h_out, n_out, m_parts, n_parts, part_stride, h_in, w_post, w_next, rows, H,
                                                eps_post, eps_next, st);
        if (dt == DT_BF16)
            return launch_add_norm_parts<bf16>(h_out, n_out, m_parts, n_parts, part_stride, h_in, w_post, w_next, rows, H,
                                               eps_post, eps_next, st);
        return CM_ERR_DTYPE;
    }
    if (dt == DT_F32)
        return launch_add_norm<float>(h_out, n_out, m, h_in, w_post, w_next, rows, H, eps_post, eps_next, st);
    if (dt == DT_BF16)
        return launch_add_norm<bf16>(h_out, n_out, m, h_in, w_post, w_next, rows, H, eps_post, eps_next, st);
    return CM_ERR_DTYPE;
}

// --------------------------------------------------------------------------- SwiGLU
// a[t,f] = T((g * sigmoid(g)) * u), g = gu[t, f], u = gu[t, F + f]  (gate | up packed rows).
template <typename T>
__global__ void swiglu_kernel(T* __restrict__ a, const T* __restrict__ gu, long long total, int F) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / F;
    const int f = (int)(i - t * F);
    const float g = to_f32(gu[t * 2 * F + f]);
    const float u = to_f32(gu[t * 2 * F + F + f]);
    a[i] = from_f32<T>((g * sigmoid_f32(g)) * u);
}

extern "C" int cm_swiglu(int dt, void* a, const void* gu, int rows, int F, cudaStream_t st) {
    const long long total = (long long)rows * F;
    if (total <= 0) return CM_OK;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (dt == DT_F32)
        cm_launch(swiglu_kernel<float>, blocks, threads, 0, st, (float*)a, (const float*)gu, total, F);
    else if (dt == DT_BF16)
        cm_launch(swiglu_kernel<bf16>, blocks, threads, 0, st, (bf16*)a, (const bf16*)gu, total, F);
    else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// ------------------------------------------------------------ logit scale and soft cap
// x <- cap * tanh((x * scale) / cap), or x * scale when cap is 0: what some architectures do to
// their logits before sampling.  Float logits, in place.
__global__ void scale_softcap_kernel(float* __restrict__ x, long long total, float scale, float cap) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const float v = x[i] * scale;
    x[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
}

extern "C" int cm_scale_softcap(float* x, long long total, float scale, float cap, cudaStream_t st) {
    if (total <= 0) return CM_OK;
    cm_launch(scale_softcap_kernel, (unsigned)((total + 255) / 256), 256, 0, st, x, total, scale, cap);
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// ----------------------------------------------------------------------- row gather
template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* __restrict__ x,
                                   const int* __restrict__ rows, int H) {
    pdl_trigger();
    pdl_wait();
    const T* src = x + (long long)rows[blockIdx.x] * H;
    T* dst = out + (long long)blockIdx.x * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) dst[c] = src[c];
}

extern "C" int cm_gather_rows(int dt, void* out, const void* x, const int* rows, int n, int H,
                              cudaStream_t st) {
    if (n <= 0) return CM_OK;
    if (dt == DT_F32)
        cm_launch(gather_rows_kernel<float>, n, 128, 0, st, (float*)out, (const float*)x, rows, H);
    else if (dt == DT_BF16)
        cm_launch(gather_rows_kernel<bf16>, n, 128, 0, st, (bf16*)out, (const bf16*)x, rows, H);
    else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}
