// Row-wise kernels: embedding gather, RMSNorm, fused post-norm + residual + next norm,
// SwiGLU product, row gather.  One block per row; all sums in float, in a fixed order.
#include "common.cuh"

// ------------------------------------------------------------------ embedding gather
// out[t,:] = table[tokens[t],:].  A token id outside [0,V) writes zeros and raises *err.
template <typename T>
__global__ void embed_gather_kernel(T* __restrict__ out, const T* __restrict__ table,
                                    const int* __restrict__ tokens, int H, int V,
                                    int* __restrict__ err) {
    const int t = blockIdx.x;
    const int tok = tokens[t];
    const bool ok = tok >= 0 && tok < V;
    if (!ok && threadIdx.x == 0 && err) atomicExch(err, 1);
    const T* src = table + (long long)(ok ? tok : 0) * H;
    T* dst = out + (long long)t * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) dst[c] = ok ? src[c] : from_f32<T>(0.f);
}

extern "C" int cm_embed_gather(int dt, void* out, const void* table, const int* tokens, int T,
                               int H, int V, int* err, cudaStream_t st) {
    if (T <= 0) return CM_OK;
    const int threads = H >= 1024 ? 256 : 128;
    if (dt == DT_F32)
        embed_gather_kernel<float><<<T, threads, 0, st>>>((float*)out, (const float*)table, tokens, H, V, err);
    else if (dt == DT_BF16)
        embed_gather_kernel<bf16><<<T, threads, 0, st>>>((bf16*)out, (const bf16*)table, tokens, H, V, err);
    else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// -------------------------------------------------------------------------- RMSNorm
// y = T((x * inv) * w), inv = 1/sqrt(mean(x^2) + eps); w is float.
template <typename T>
__global__ void rmsnorm_kernel(T* __restrict__ y, const T* __restrict__ x,
                               const float* __restrict__ w, int H, float eps, long long ldx,
                               long long ldy) {
    __shared__ float scratch[32];
    const T* xr = x + (long long)blockIdx.x * ldx;
    T* yr = y + (long long)blockIdx.x * ldy;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float v = to_f32(xr[c]);
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x)
        yr[c] = from_f32<T>((to_f32(xr[c]) * inv) * w[c]);
}

extern "C" int cm_rmsnorm(int dt, void* y, const void* x, const float* w, int rows, int H,
                          float eps, long long ldx, long long ldy, cudaStream_t st) {
    if (rows <= 0) return CM_OK;
    const int threads = H >= 1024 ? 256 : 128;
    if (dt == DT_F32)
        rmsnorm_kernel<float><<<rows, threads, 0, st>>>((float*)y, (const float*)x, w, H, eps, ldx, ldy);
    else if (dt == DT_BF16)
        rmsnorm_kernel<bf16><<<rows, threads, 0, st>>>((bf16*)y, (const bf16*)x, w, H, eps, ldx, ldy);
    else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// ------------------------------------------------- residual add with both norms fused
// d      = w_post ? T((m * inv(m)) * w_post) : m          (post-norm of the part's output)
// h_out  = T(h_in + d)                                    (sum in float)
// n_out  = w_next ? T((h_out * inv(h_out)) * w_next)      (pre-norm of whatever runs next,
//                                                          taken over the stored h_out)
// h_out may alias h_in.  Row stays in shared memory as float between the passes.
template <typename T>
__global__ void add_norm_kernel(T* __restrict__ h_out, T* __restrict__ n_out,
                                const T* __restrict__ m, const T* __restrict__ h_in,
                                const float* __restrict__ w_post,
                                const float* __restrict__ w_next, int H, float eps_post,
                                float eps_next) {
    extern __shared__ float row[];   // H floats
    __shared__ float scratch[32];
    const long long off = (long long)blockIdx.x * H;
    float inv_post = 1.f;
    if (w_post) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            const float v = to_f32(m[off + c]);
            row[c] = v;
            ss += v * v;
        }
        ss = block_sum(ss, scratch);
        inv_post = 1.f / sqrtf(ss / (float)H + eps_post);
    }
    float ss2 = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float d;
        if (w_post)
            d = rounded<T>((row[c] * inv_post) * w_post[c]);
        else
            d = to_f32(m[off + c]);
        const float hn = rounded<T>(to_f32(h_in[off + c]) + d);
        h_out[off + c] = from_f32<T>(hn);
        row[c] = hn;
        ss2 += hn * hn;
    }
    if (!w_next) return;
    ss2 = block_sum(ss2, scratch);
    const float inv_next = 1.f / sqrtf(ss2 / (float)H + eps_next);
    for (int c = threadIdx.x; c < H; c += blockDim.x)
        n_out[off + c] = from_f32<T>((row[c] * inv_next) * w_next[c]);
}

extern "C" int cm_add_norm(int dt, void* h_out, void* n_out, const void* m, const void* h_in,
                           const float* w_post, const float* w_next, int rows, int H,
                           float eps_post, float eps_next, cudaStream_t st) {
    if (rows <= 0) return CM_OK;
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 160 * 1024) CM_REFUSE("add_norm: hidden size %d needs %zu bytes of shared memory", H, smem);
    const int threads = H >= 1024 ? 256 : 128;
    if (dt == DT_F32) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        add_norm_kernel<float><<<rows, threads, smem, st>>>((float*)h_out, (float*)n_out, (const float*)m,
                                                            (const float*)h_in, w_post, w_next, H,
                                                            eps_post, eps_next);
    } else if (dt == DT_BF16) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_norm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        add_norm_kernel<bf16><<<rows, threads, smem, st>>>((bf16*)h_out, (bf16*)n_out, (const bf16*)m,
                                                           (const bf16*)h_in, w_post, w_next, H,
                                                           eps_post, eps_next);
    } else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// --------------------------------------------------------------------------- SwiGLU
// a[t,f] = T((g * sigmoid(g)) * u), g = gu[t, f], u = gu[t, F + f]  (gate | up packed rows).
template <typename T>
__global__ void swiglu_kernel(T* __restrict__ a, const T* __restrict__ gu, long long total, int F) {
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
        swiglu_kernel<float><<<blocks, threads, 0, st>>>((float*)a, (const float*)gu, total, F);
    else if (dt == DT_BF16)
        swiglu_kernel<bf16><<<blocks, threads, 0, st>>>((bf16*)a, (const bf16*)gu, total, F);
    else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// ----------------------------------------------------------------------- row gather
template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* __restrict__ x,
                                   const int* __restrict__ rows, int H) {
    const T* src = x + (long long)rows[blockIdx.x] * H;
    T* dst = out + (long long)blockIdx.x * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) dst[c] = src[c];
}

extern "C" int cm_gather_rows(int dt, void* out, const void* x, const int* rows, int n, int H,
                              cudaStream_t st) {
    if (n <= 0) return CM_OK;
    if (dt == DT_F32)
        gather_rows_kernel<float><<<n, 128, 0, st>>>((float*)out, (const float*)x, rows, H);
    else if (dt == DT_BF16)
        gather_rows_kernel<bf16><<<n, 128, 0, st>>>((bf16*)out, (const bf16*)x, rows, H);
    else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}
