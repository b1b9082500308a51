// Shared device helpers for the sm_100a kernels of this library.
//
// Every kernel is templated on the storage type of activations and matrices (float for
// the true 32-bit path, __nv_bfloat16 for the serving path) and does its reductions,
// norms, softmax, rotation angles and residual sums in float.  The C entry points take
// a dtype code (DT_F32 / DT_BF16), raw device pointers and the stream to launch on;
// they return 0 or a negative code and never allocate.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "cm_limits.h"

#define DT_F32 0
#define DT_BF16 1

#define CM_OK 0
#define CM_ERR_DTYPE -1      // unknown dtype code
#define CM_ERR_SHAPE -2      // a size this kernel refuses (message via cm_last_error)
#define CM_ERR_LAUNCH -3     // cudaGetLastError() after the launch was not cudaSuccess
#define CM_ERR_DRIVER -4     // a driver entry point (tensor map encode) failed

typedef __nv_bfloat16 bf16;

// Set by the entry points when they refuse a call; read through cm_last_error().
void cm_set_error(const char* fmt, ...);

#define CM_REFUSE(...)            \
    do {                          \
        cm_set_error(__VA_ARGS__); \
        return CM_ERR_SHAPE;      \
    } while (0)

// ---- programmatic dependent launch --------------------------------------------------
// Every kernel of this library is launched with the "programmatic stream serialization"
// attribute (unless cm_set_pdl(0)): the next kernel of the stream may be scheduled once every
// block of this one has called pdl_trigger() or left, and blocks in pdl_wait() until this one
// has finished and its writes are visible.  A kernel may read constants (weights) before
// pdl_wait(), and nothing else; every block calls pdl_wait() before it reads an activation,
// writes anything, or exits, so that completion of a kernel implies completion of all kernels
// before it.
// Where to trigger, and what to launch early (all measured on B200, LFM3 1.7B-class decode):
//  - the short row-wise kernels (norms, convolution, rotation, gathers, merges) trigger at once;
//  - the TMA-fed products and the attention kernels trigger when their last loads are under way.
//    Triggered at once, kernel after kernel became resident and sat waiting, and steps of 1 and
//    8 sequences took up to 1.5 times as long as without any overlap;
//  - the weight-streaming product of small decode batches (gemm_skinny.cu) is launched in plain
//    stream order and triggers as soon as it runs: started early it made those steps 5% slower
//    (with or without reading weights ahead of its wait, with or without a cluster), while the
//    TMA-fed products gain from setting up their barriers and tensor memory early (batch 64: 7%
//    faster).  A chain of spinning kernels of the same shapes gains 40% from starting early, a
//    chain of these products alone gains nothing (34.9 against 34.1 us for a layer's four): four
//    blocks of 64 registers fill an SM, so a block that starts early finds room only when one of the
//    kernel before has left, and what a product spends between launches is mostly the ramp of its
//    own memory pipeline, which an early start does not shorten.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

int cm_pdl_enabled();

template <typename... KArgs, typename... Args>
static inline cudaError_t cm_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = cm_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same, for a grid whose blocks form clusters of (1, cluster_y, 1).  early = false launches
// in plain stream order (the kernel starts when the one before it has finished).
template <typename... KArgs, typename... Args>
static inline cudaError_t cm_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                            cudaStream_t st, int cluster_y, bool early, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (cluster_y > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1;
        attr[n].val.clusterDim.y = cluster_y;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (early && cm_pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define CM_CHECK_LAUNCH()                                              \
    do {                                                               \
        cudaError_t e_ = cudaGetLastError();                           \
        if (e_ != cudaSuccess) {                                       \
            cm_set_error("%s:%d launch failed: %s", __FILE__, __LINE__, \
                         cudaGetErrorString(e_));                      \
            return CM_ERR_LAUNCH;                                      \
        }                                                              \
    } while (0)

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(bf16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ bf16 from_f32<bf16>(float x) { return __float2bfloat16_rn(x); }

// Value as it will read back after a store in T: identity for float, a bf16 round trip else.
template <typename T>
__device__ __forceinline__ float rounded(float x) { return to_f32(from_f32<T>(x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over the block in a fixed order (lane tree, then warp 0 over the per-warp sums), so
// that a row's result never depends on how many other rows the launch carries.
// `scratch` holds at least 32 floats.  Every thread gets the total.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                 // scratch may still be read from a previous call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? scratch[lane] : 0.f;
    t = warp_sum(t);
    return t;
}

__device__ __forceinline__ float sigmoid_f32(float x) { return 1.f / (1.f + expf(-x)); }

// Eight consecutive elements as floats: one 16-byte access for bfloat16, two for float.
template <typename T>
__device__ __forceinline__ void load8f(const T* p, float* out);
template <>
__device__ __forceinline__ void load8f<float>(const float* p, float* out) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w; out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
template <>
__device__ __forceinline__ void load8f<bf16>(const bf16* p, float* out) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
    }
}
template <typename T>
__device__ __forceinline__ void store8f(T* p, const float* v);
template <>
__device__ __forceinline__ void store8f<float>(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8f<bf16>(bf16* p, const float* v) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
}

// Page-table geometry shared by the cache kernels: a page holds PAGE_TOKENS consecutive
// cache entries of one sequence for every layer of a group.
#define PAGE_TOKENS CM_PAGE_TOKENS

// Storage of one layer group: [layer][k|v][page][kv_head][PAGE_TOKENS][head_dim].
template <typename T>
__device__ __forceinline__ T* kv_tile(T* layer_base, int kv, long long pages, int page, int kvh,
                                      int KVH, int HD) {
    return layer_base + ((((long long)kv * pages + page) * KVH + kvh) * PAGE_TOKENS) * (long long)HD;
}
