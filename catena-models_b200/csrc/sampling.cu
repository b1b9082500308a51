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
// the row is cut into slices, the slice sums are scanned in index order and the slice that holds
// u * total is walked to the first index whose running sum exceeds it.
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

    const float inv_t = 1.f / temp;
    if (vec) {
        // ---- aligned rows: slices of 128 consecutive entries, one warp-wide 16-byte load each.
        // Warp w sums slices w, w + 16, ... (a lane adds its four exponentials in order, the lanes
        // are added by a butterfly); warp 0 scans the slice sums in index order, finds the slice
        // that holds u * total and walks it with a scan over its lanes.
        constexpr int WARPS = SM_THREADS / 32;
        constexpr int MAX_SLICES = 32 * 64;                       // one warp scans them, 64 a lane
        const int n_slices = (V + 127) / 128;
        extern __shared__ float slice_sum[];                      // [n_slices]
        const int warp = tid >> 5, lane = tid & 31;
        auto exps = [&](int s, float* e) {                        // the four exponentials of this lane in slice s
            const int i0 = s * 128 + lane * 4;
            float4 v = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            if (i0 + 3 < V) {
                v = x4[i0 >> 2];
            } else {
                if (i0 < V) v.x = x[i0];
                if (i0 + 1 < V) v.y = x[i0 + 1];
                if (i0 + 2 < V) v.z = x[i0 + 2];
            }
            e[0] = __expf((v.x - mx) * inv_t);                    // exp(-inf) = 0 beyond the row
            e[1] = __expf((v.y - mx) * inv_t);
            e[2] = __expf((v.z - mx) * inv_t);
            e[3] = __expf((v.w - mx) * inv_t);
        };
        for (int s0 = warp; s0 < n_slices; s0 += 4 * WARPS) {      // four slices in flight per warp
            float part[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int sl = s0 + u * WARPS;
                float e[4] = {0.f, 0.f, 0.f, 0.f};
                if (sl < n_slices) exps(sl, e);
                part[u] = ((e[0] + e[1]) + e[2]) + e[3];
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int u = 0; u < 4; ++u) part[u] += __shfl_xor_sync(0xffffffffu, part[u], o);
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (lane == 0 && s0 + u * WARPS < n_slices) slice_sum[s0 + u * WARPS] = part[u];
        }
        __syncthreads();
        if (warp == 0) {
            // inclusive scan of the slice sums: a lane owns `per` consecutive slices
            const int per = (n_slices + 31) / 32;
            const int s_lo = min(n_slices, lane * per), s_hi = min(n_slices, s_lo + per);
            float mine = 0.f;
            for (int sl = s_lo; sl < s_hi; ++sl) mine += slice_sum[sl];
            float incl = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            const float total = __shfl_sync(0xffffffffu, incl, 31);
            float excl = __shfl_up_sync(0xffffffffu, incl, 1);     // sum of all slices before this lane's
            if (lane == 0) excl = 0.f;
            const unsigned long long seed =
                ((unsigned long long)(unsigned)seed_words[1] << 32) | (unsigned long long)(unsigned)seed_words[0];
            const float target = uniform24(seed, (unsigned long long)(long long)sequence[row],
                                           (unsigned long long)(long long)step[row]) * total;
            // the first lane whose slices reach beyond the target, then its first such slice
            const unsigned reach = __ballot_sync(0xffffffffu, incl > target && s_lo < s_hi);
            int pick = amax;                                      // used if rounding leaves the target above every sum
            if (reach) {
                const int owner = __ffs(reach) - 1;
                float run = __shfl_sync(0xffffffffu, excl, owner);            // sum of everything before the owner's slices
                const int o_lo = __shfl_sync(0xffffffffu, s_lo, owner), o_hi = __shfl_sync(0xffffffffu, s_hi, owner);
                int sl = o_lo;
                for (; sl < o_hi - 1; ++sl) {                     // uniform over the warp: every lane reads the same sums
                    const float next = run + slice_sum[sl];
                    if (next > target) break;
                    run = next;
                }
                // walk slice sl: running sums in index order over the lanes' four entries
                float e[4];
                exps(sl, e);
                const float l1 = e[0], l2 = l1 + e[1], l3 = l2 + e[2], l4 = l3 + e[3];
                float through = l4;                               // this slice up to and with this lane's entries
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const float up = __shfl_up_sync(0xffffffffu, through, o);
                    if (lane >= o) through += up;
                }
                float before = __shfl_up_sync(0xffffffffu, through, 1);
                before = run + (lane == 0 ? 0.f : before);        // everything before this lane's entries
                const unsigned hit = __ballot_sync(0xffffffffu, before + l4 > target);
                const int last = min(V, sl * 128 + 128) - 1;      // the slice's last entry, if rounding finds none
                pick = last;
                if (hit) {
                    const int hl = __ffs(hit) - 1;
                    const float hb = __shfl_sync(0xffffffffu, before, hl);
                    const float h1 = __shfl_sync(0xffffffffu, l1, hl), h2 = __shfl_sync(0xffffffffu, l2, hl),
                                h3 = __shfl_sync(0xffffffffu, l3, hl);
                    const int base = sl * 128 + hl * 4;
                    pick = hb + h1 > target ? base : hb + h2 > target ? base + 1 : hb + h3 > target ? base + 2 : base + 3;
                    pick = min(pick, last);
                }
            }
            if (lane == 0) out[row] = pick;
        }
        (void)MAX_SLICES;
        return;
    }
    // ---- rows that are not 16-byte aligned: thread k sums the contiguous slice k of the row
    const int per = (V + SM_THREADS - 1) / SM_THREADS;
    const int lo = min(V, tid * per), hi = min(V, lo + per);
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
    // one float of shared memory per slice of 128 entries (the aligned path's slice sums)
    const size_t smem = (size_t)((V + 127) / 128) * sizeof(float);
    if (smem > 48 * 1024) CM_REFUSE("sample: vocabulary of %d (at most %d)", V, 48 * 1024 / 4 * 128);
    cm_launch(sample_kernel, n, SM_THREADS, smem, st, out, logits, ld, V, temperature, sequence, step, seed_words);
    CM_CHECK_LAUNCH();
    return CM_OK;
}
