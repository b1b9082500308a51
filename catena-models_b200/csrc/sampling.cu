// Next-token choice from float logits [n, V]: greedy argmax (lowest index wins ties) and
// temperature sampling by inverse CDF with a counter-based uniform keyed by
// (seed, sequence id, step), so that a sequence's draws do not depend on its batch-mates.
#include "common.cuh"
#include <math.h>

#define SM_THREADS 512

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// Uniform in [0,1) with 24 bits: mix(mix(mix(seed) ^ sequence) ^ step) >> 40.
__device__ __forceinline__ float uniform24(unsigned long long seed, unsigned long long sequence,
                                           unsigned long long step) {
    unsigned long long z = mix64(seed);
    z = mix64(z ^ sequence);
    z = mix64(z ^ step);
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

// One block per row.  temperature[row] == 0 -> argmax.  Otherwise p_i = exp((x_i - max) / t);
// thread k sums the contiguous slice k of the row, the slices are scanned in index order and
// the slice that holds u * total is walked to the first index whose running sum exceeds it.
__global__ void __launch_bounds__(SM_THREADS)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits, long long ld, int V,
              const float* __restrict__ temperature, const int* __restrict__ sequence,
              const int* __restrict__ step, const int* __restrict__ seed_words) {
    pdl_trigger();
    pdl_wait();
    __shared__ float sval[SM_THREADS];
    __shared__ int sidx[SM_THREADS];
    __shared__ float scratch[32];
    __shared__ int chosen;
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* x = logits + (long long)row * ld;
    const float temp = temperature ? temperature[row] : 0.f;

    // ---- maximum and its first index (a thread meets its indices in rising order, so a strict
    // comparison keeps the lowest); four 16-byte loads in flight per thread where the row allows
    float best = -INFINITY;
    int arg = 0x7fffffff;
    const bool vec = (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
    const int n4 = vec ? V / 4 : 0;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    for (int i = tid; i < n4; i += 4 * SM_THREADS) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = i + u * SM_THREADS;
            v[u] = j < n4 ? x4[j] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j4 = 4 * (i + u * SM_THREADS);
            if (v[u].x > best) { best = v[u].x; arg = j4; }
            if (v[u].y > best) { best = v[u].y; arg = j4 + 1; }
            if (v[u].z > best) { best = v[u].z; arg = j4 + 2; }
            if (v[u].w > best) { best = v[u].w; arg = j4 + 3; }
        }
    }
    for (int i = 4 * n4 + tid; i < V; i += SM_THREADS) {
        const float v = x[i];
        if (v > best) {
            best = v;
            arg = i;
        }
    }
    sval[tid] = best;
    sidx[tid] = arg;
    __syncthreads();
    for (int s = SM_THREADS / 2; s > 0; s >>= 1) {
        if (tid < s) {
            const float ov = sval[tid + s];
            const int oi = sidx[tid + s];
            if (ov > sval[tid] || (ov == sval[tid] && oi < sidx[tid])) {
                sval[tid] = ov;
                sidx[tid] = oi;
            }
        }
        __syncthreads();
    }
    const float mx = sval[0];
    const int amax = sidx[0] == 0x7fffffff ? 0 : sidx[0];
    if (temp <= 0.f) {
        if (tid == 0) out[row] = amax;
        return;
    }
    __syncthreads();

    // ---- slice sums
    const int per = (V + SM_THREADS - 1) / SM_THREADS;
    const int lo = min(V, tid * per), hi = min(V, lo + per);
    const float inv_t = 1.f / temp;
    float part = 0.f;
    for (int i = lo; i < hi; ++i) part += expf((x[i] - mx) * inv_t);
    sval[tid] = part;
    __syncthreads();
    // inclusive scan over the slices, in index order (one thread: 512 adds)
    if (tid == 0) {
        float run = 0.f;
        for (int k = 0; k < SM_THREADS; ++k) {
            run += sval[k];
            sval[k] = run;
        }
        const unsigned long long seed =
            ((unsigned long long)(unsigned)seed_words[1] << 32) | (unsigned long long)(unsigned)seed_words[0];
        scratch[0] = uniform24(seed, (unsigned long long)(long long)sequence[row],
                               (unsigned long long)(long long)step[row]) * run;
        chosen = amax;                      // used if rounding leaves the target above every sum
    }
    __syncthreads();
    const float target = scratch[0];
    const float before = tid == 0 ? 0.f : sval[tid - 1];
    if (target >= before && target < sval[tid] && lo < hi) {
        float run = before;
        int pick = hi - 1;
        for (int i = lo; i < hi; ++i) {
            run += expf((x[i] - mx) * inv_t);
            if (run > target) {
                pick = i;
                break;
            }
        }
        chosen = pick;
    }
    __syncthreads();
    if (tid == 0) out[row] = chosen;
}

extern "C" int cm_sample(int* out, const float* logits, long long ld, int n, int V,
                         const float* temperature, const int* sequence, const int* step,
                         const int* seed_words, cudaStream_t st) {
    if (n <= 0) return CM_OK;
    if (V <= 0) CM_REFUSE("sample: vocabulary of %d", V);
    cm_launch(sample_kernel, n, SM_THREADS, 0, st, out, logits, ld, V, temperature, sequence, step, seed_words);
    CM_CHECK_LAUNCH();
    return CM_OK;
}
