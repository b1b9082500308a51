// Attention kernels: head norm + rotation + cache write, prefill attention over the step's
// own keys, decode attention over the paged cache (split over fixed chunks, ordered merge).
//
// Masks: a key at position k is visible to a query at position p when k <= p and, for a
// window W > 0, k + W > p.  Scores, softmax and the probability-value sums are float.
#include "common.cuh"
#include <math.h>

template <typename T>
__device__ __forceinline__ void load8(const T* p, float* out);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float* out) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
    out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<bf16>(const bf16* p, float* out) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
    }
}

// =========================================================================================
// Head norm, rotation, cache write.  One warp per (token, head); q heads first, then k heads.
//   qkv row: [ q: QH*HD | k: KVH*HD | v: KVH*HD | ... ]  (row stride ld)
//   u = T((x * inv_rms(x)) * w)           when w is given (w_q for q heads, w_k for k heads)
//   o_i       = u_i cos a - u_{i+HD/2} sin a
//   o_{i+HD/2}= u_{i+HD/2} cos a + u_i sin a,   a = float(pos) * rate[i]      when rate is given
// (pairs of the two halves; with `interleaved` the pairs are neighbours, (2i, 2i+1), instead)
// Rows whose tok_seq is negative are padding (a step recorded for a class of shapes carries some):
// they are left alone.
// q and k are overwritten in place; k and the raw v also go to the cache entry of (slot, pos):
// entry = pos (growing group) or pos % ring (ring group; during a prompt longer than the ring
// only the last `ring` positions are stored, so that no two rows meet in one entry).
// =========================================================================================
template <typename T>
__global__ void qk_prepare_kernel(T* __restrict__ qkv, long long ld, const float* __restrict__ wq,
                                  const float* __restrict__ wk, const float* __restrict__ rate,
                                  const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                  const int* __restrict__ seq_slot, const int* __restrict__ seq_end,
                                  T* __restrict__ pool, long long pages, const int* __restrict__ ptab,
                                  int ptab_stride, int ring, int QH, int KVH, int HD, float eps, int T_tokens,
                                  int heads_per_warp, int interleaved) {
    pdl_trigger();
    pdl_wait();
    // One warp per token and group of `heads_per_warp` heads (grid.y walks the groups: many heads
    // per warp when tokens are plenty, one when they are few).  A lane owns the rotation pairs (i, i + HD/2)
    // for i = lane, lane + 32, ...; sine and cosine depend on the position and the pair only, so
    // they are formed once per token and serve every head.
    constexpr int MAXP = 4;                       // pairs per lane: head sizes up to 256
    const int lane = threadIdx.x;
    const int t = blockIdx.x * blockDim.y + threadIdx.y;
    if (t >= T_tokens || tok_seq[t] < 0) return;      // a row of padding belongs to no sequence
    const int pos = tok_pos[t];
    const int half = HD >> 1;
    float sn[MAXP], cs[MAXP];
#pragma unroll
    for (int p = 0; p < MAXP; ++p) {
        const int i = lane + 32 * p;
        sn[p] = 0.f;
        cs[p] = 1.f;
        if (rate && i < half) sincosf((float)pos * rate[i], &sn[p], &cs[p]);
    }
    // where this token's key and value go in the cache (if it is kept at all)
    int page = -1, row = 0;
    if (pool) {
        const int b = tok_seq[t];
        if (ring == 0 || pos + ring >= seq_end[b]) {
            const int entry = ring ? pos % ring : pos;
            page = ptab[(long long)seq_slot[b] * ptab_stride + entry / PAGE_TOKENS];
            row = entry % PAGE_TOKENS;
        }
    }
    const int head0 = blockIdx.y * heads_per_warp;
    const int head1 = min(QH + KVH, head0 + heads_per_warp);
    for (int head = head0; head < head1; ++head) {
        const bool is_q = head < QH;
        T* x = qkv + (long long)t * ld + (long long)head * HD;     // k heads follow the q heads
        const float* w = is_q ? wq : wk;
        float lo[MAXP], hi[MAXP];
        float ss = 0.f;
#pragma unroll
        for (int p = 0; p < MAXP; ++p) {
            const int i = lane + 32 * p;
            lo[p] = hi[p] = 0.f;
            if (i < half) {
                lo[p] = to_f32(x[interleaved ? 2 * i : i]);
                hi[p] = to_f32(x[interleaved ? 2 * i + 1 : i + half]);
                ss += lo[p] * lo[p] + hi[p] * hi[p];
            }
        }
        float inv = 1.f;
        if (w) {
            ss = warp_sum(ss);
            inv = 1.f / sqrtf(ss / (float)HD + eps);
        }
        T* kdst = (!is_q && page >= 0) ? kv_tile(pool, 0, pages, page, head - QH, KVH, HD) + (long long)row * HD : nullptr;
#pragma unroll
        for (int p = 0; p < MAXP; ++p) {
            const int i = lane + 32 * p;
            if (i >= half) continue;
            float a = lo[p], bq = hi[p];
            const int i_lo = interleaved ? 2 * i : i, i_hi = interleaved ? 2 * i + 1 : i + half;
            if (w) {
                a = rounded<T>((a * inv) * w[i_lo]);
                bq = rounded<T>((bq * inv) * w[i_hi]);
            }
            const T at = from_f32<T>(a * cs[p] - bq * sn[p]), bt = from_f32<T>(bq * cs[p] + a * sn[p]);
            x[i_lo] = at;
            x[i_hi] = bt;
            if (kdst) {
                kdst[i_lo] = at;
                kdst[i_hi] = bt;
            }
        }
    }
    if (page >= 0) {
        // the raw values of the key heads this warp handled
        const T* v = qkv + (long long)t * ld + (long long)(QH + KVH) * HD;
        for (int kvh = max(0, head0 - QH); kvh < head1 - QH; ++kvh) {
            T* vdst = kv_tile(pool, 1, pages, page, kvh, KVH, HD) + (long long)row * HD;
            for (int d = lane; d < HD; d += 32) vdst[d] = v[kvh * HD + d];
        }
    }
}

// The same with 16-byte accesses (head sizes that are multiples of 16, aligned rows).  A head's two
// halves are cut into runs of eight channels; LPH = HD / 16 lanes own one run of each half, so a
// warp works on 32 / LPH heads of one token at a time and walks the token's heads in such passes.
// The sum of squares of a head is added over its lanes in lane order.
template <typename T>
__global__ void __launch_bounds__(128)
qk_prepare_vec_kernel(T* __restrict__ qkv, long long ld, const float* __restrict__ wq,
                      const float* __restrict__ wk, const float* __restrict__ rate,
                      const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                      const int* __restrict__ seq_slot, const int* __restrict__ seq_end,
                      T* __restrict__ pool, long long pages, const int* __restrict__ ptab,
                      int ptab_stride, int ring, int QH, int KVH, int HD, float eps, int T_tokens,
                      int passes_per_warp) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x;
    const int t = blockIdx.x * blockDim.y + threadIdx.y;
    if (t >= T_tokens || tok_seq[t] < 0) return;      // a row of padding belongs to no sequence
    const int half = HD >> 1, LPH = half >> 3, HPP = 32 / LPH;
    const int sub = lane % LPH, hsel = lane / LPH;          // lanes past HPP * LPH idle along
    const int pos = tok_pos[t];
    float sn[8], cs[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        sn[e] = 0.f;
        cs[e] = 1.f;
        if (rate) sincosf((float)pos * rate[sub * 8 + e], &sn[e], &cs[e]);
    }
    int page = -1, row = 0;
    if (pool) {
        const int b = tok_seq[t];
        if (ring == 0 || pos + ring >= seq_end[b]) {
            const int entry = ring ? pos % ring : pos;
            page = ptab[(long long)seq_slot[b] * ptab_stride + entry / PAGE_TOKENS];
            row = entry % PAGE_TOKENS;
        }
    }
    const int n_heads = QH + KVH;
    const int pass0 = blockIdx.y * passes_per_warp;
    for (int pass = pass0; pass < pass0 + passes_per_warp; ++pass) {
        const int head = pass * HPP + hsel;
        const bool live = hsel < HPP && head < n_heads;
        const bool is_q = head < QH;
        T* x = qkv + (long long)t * ld + (long long)head * HD + sub * 8;
        const float* w = is_q ? wq : wk;
        float lo[8], hi[8];
        float ss = 0.f;
        if (live) {
            load8f<T>(x, lo);
            load8f<T>(x + half, hi);
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += lo[e] * lo[e] + hi[e] * hi[e];
        }
        float inv = 1.f;
        if (wq || wk) {                                             // the shuffles are for the whole warp
            float tot = 0.f;
            for (int j = 0; j < LPH; ++j) tot += __shfl_sync(0xffffffffu, ss, (hsel * LPH + j) & 31);
            if (w) inv = 1.f / sqrtf(tot / (float)HD + eps);
        }
        if (!live) continue;
        if (w) {
            float wl[8], wh[8];
            load8f<float>(w + sub * 8, wl);
            load8f<float>(w + half + sub * 8, wh);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                lo[e] = rounded<T>((lo[e] * inv) * wl[e]);
                hi[e] = rounded<T>((hi[e] * inv) * wh[e]);
            }
        }
        float ol[8], oh[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            ol[e] = lo[e] * cs[e] - hi[e] * sn[e];
            oh[e] = hi[e] * cs[e] + lo[e] * sn[e];
        }
        store8f<T>(x, ol);
        store8f<T>(x + half, oh);
        if (!is_q && page >= 0) {
            T* kdst = kv_tile(pool, 0, pages, page, head - QH, KVH, HD) + (long long)row * HD + sub * 8;
            store8f<T>(kdst, ol);
            store8f<T>(kdst + half, oh);
        }
    }
    // the raw values: copied by the warp that has the token's last pass
    if (page >= 0 && pass0 + passes_per_warp >= (n_heads + HPP - 1) / HPP) {
        const T* v = qkv + (long long)t * ld + (long long)(QH + KVH) * HD;
        for (int e = lane * 8; e < KVH * HD; e += 256) {
            const int kvh = e / HD, d = e - kvh * HD;
            float tmp[8];
            load8f<T>(v + e, tmp);
            store8f<T>(kv_tile(pool, 1, pages, page, kvh, KVH, HD) + (long long)row * HD + d, tmp);
        }
    }
}

extern "C" int cm_qk_prepare(int dt, void* qkv, long long ld, const float* wq, const float* wk,
                             const float* rate, const int* tok_pos, const int* tok_seq,
                             const int* seq_slot, const int* seq_end, void* pool, long long pages,
                             const int* ptab, int ptab_stride, int ring, int T, int QH, int KVH,
                             int HD, float eps, int interleaved, cudaStream_t st) {
    if (T <= 0) return CM_OK;
    if (HD % 2 || HD <= 0) CM_REFUSE("qk_prepare: head size %d is not even", HD);
    if (ring % PAGE_TOKENS) CM_REFUSE("qk_prepare: ring of %d entries is no multiple of %d", ring, PAGE_TOKENS);
    if (HD > CM_MAX_HEAD_DIM) CM_REFUSE("qk_prepare: head size %d above %d", HD, CM_MAX_HEAD_DIM);
    const size_t esz = dt == DT_F32 ? 4 : 2;
    const bool vec = HD % 16 == 0 && (ld * esz) % 16 == 0 &&
                     (((uintptr_t)qkv | (uintptr_t)pool | (uintptr_t)wq | (uintptr_t)wk) & 15) == 0;
    // Measured on B200 (32 + 8 heads of 64): 2,048 tokens 23.4 -> 12.4 us, 8,192 tokens 81.8 -> 24.2 us;
    // a decode step of 8 or 64 tokens is quicker with a channel per lane (3.2 against 3.9 us).
    if (vec && T >= 128 && !interleaved && (dt == DT_F32 || dt == DT_BF16)) {
        const int hpp = 32 / (HD / 16), passes = (QH + KVH + hpp - 1) / hpp;
        // A warp walks several passes of its token (sine and cosine are formed once per warp) when
        // the tokens alone give the SMs enough warps; with fewer tokens the passes are spread.
        int ppw = passes;
        while (ppw > 1 && (long long)T * ((passes + ppw - 1) / ppw) < 8192) ppw = (ppw + 1) / 2;
        dim3 vblock(32, 4), vgrid((T + 3) / 4, (passes + ppw - 1) / ppw);
        if (dt == DT_F32)
            cm_launch(qk_prepare_vec_kernel<float>, vgrid, vblock, 0, st, (float*)qkv, ld, wq, wk, rate, tok_pos, tok_seq,
                      seq_slot, seq_end, (float*)pool, pages, ptab, ptab_stride, ring, QH, KVH, HD, eps, T, ppw);
        else
            cm_launch(qk_prepare_vec_kernel<bf16>, vgrid, vblock, 0, st, (bf16*)qkv, ld, wq, wk, rate, tok_pos, tok_seq,
                      seq_slot, seq_end, (bf16*)pool, pages, ptab, ptab_stride, ring, QH, KVH, HD, eps, T, ppw);
        CM_CHECK_LAUNCH();
        return CM_OK;
    }
    const int hpw = T >= 512 ? 4 : 1;
    dim3 block(32, 4), grid((T + 3) / 4, (QH + KVH + hpw - 1) / hpw);
    const size_t smem = 0;
    if (dt == DT_F32)
        cm_launch(qk_prepare_kernel<float>, grid, block, smem, st, (float*)qkv, ld, wq, wk, rate, tok_pos, tok_seq,
                                                            seq_slot, seq_end, (float*)pool, pages, ptab,
                                                            ptab_stride, ring, QH, KVH, HD, eps, T, hpw, interleaved);
    else if (dt == DT_BF16)
        cm_launch(qk_prepare_kernel<bf16>, grid, block, smem, st, (bf16*)qkv, ld, wq, wk, rate, tok_pos, tok_seq,
                                                           seq_slot, seq_end, (bf16*)pool, pages, ptab,
                                                           ptab_stride, ring, QH, KVH, HD, eps, T, hpw, interleaved);
    else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// =========================================================================================
// Prefill attention on the CUDA cores (the 32-bit path, and any head size).
// One block = 32 queries of one head of one sequence; keys come in tiles of 32 from the
// step's own rows (all sequences of a prefill step start at position 0).
// Warp w owns queries 8w..8w+7; a lane is a key for the scores and a set of channels for PV.
// PAST: the sequences may stand at a position p0 > 0 (several tokens on top of a started
// sequence).  Keys and values below p0 are then read from the paged cache (entry = position, or
// position % ring), those from p0 on from the step's own rows; the step's rows are written to
// the cache only after this kernel has run, so a ring still holds every position that the
// windows of the step's queries reach.  Rows outside what the block's queries can see are not
// read at all (they may be stale or never written) and enter the sums as zeros.
// =========================================================================================
#define AP_BQ 32
#define AP_BK 32
#define AP_MAXJ 8        // head_dim <= 32 * AP_MAXJ
static_assert(32 * AP_MAXJ == CM_MAX_HEAD_DIM, "cm_limits.h: CM_MAX_HEAD_DIM");

template <typename T, bool PAST>
__global__ void __launch_bounds__(128)
attn_prefill_simt_kernel(T* __restrict__ ctx, long long ldc, const T* __restrict__ q,
                         const T* __restrict__ k, const T* __restrict__ v, long long ld,
                         const T* __restrict__ gate, long long ldg,
                         const int* __restrict__ seq_start, int QH, int KVH, int HD, int window,
                         float scale, const int* __restrict__ seq_pos0, const int* __restrict__ seq_slot,
                         const T* __restrict__ pool, long long pages, const int* __restrict__ ptab,
                         int ptab_stride, int ring) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    const int ldq = HD + 1;
    float* Qs = smem;                       // [AP_BQ][HD+1]
    float* Ks = Qs + AP_BQ * ldq;           // [AP_BK][HD+1]
    float* Vs = Ks + AP_BK * ldq;           // [AP_BK][HD]
    float* Ps = Vs + AP_BK * HD;            // [AP_BQ][AP_BK+1]
    const int b = blockIdx.z, hq = blockIdx.y, hk = hq / (QH / KVH);
    const int s0 = seq_start[b], n_new = seq_start[b + 1] - s0;
    const int p0 = PAST ? seq_pos0[b] : 0;         // position of the step's first token of this sequence
    const int len = p0 + n_new;                    // positions are absolute from here on
    const int q0 = p0 + blockIdx.x * AP_BQ;
    if (q0 >= len) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nq = min(AP_BQ, len - q0);
    const int* prow = PAST ? ptab + (long long)seq_slot[b] * ptab_stride : nullptr;

    for (int e = threadIdx.x; e < AP_BQ * HD; e += blockDim.x) {
        const int r = e / HD, d = e - r * HD;
        Qs[r * ldq + d] = r < nq ? to_f32(q[(long long)(s0 + q0 - p0 + r) * ld + (long long)hq * HD + d]) : 0.f;
    }
    float m[8], l[8], acc[8][AP_MAXJ];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        m[i] = -INFINITY;
        l[i] = 0.f;
#pragma unroll
        for (int j = 0; j < AP_MAXJ; ++j) acc[i][j] = 0.f;
    }
    const int q_last = q0 + nq - 1;
    const int k_first = window > 0 ? max(0, q0 - window + 1) : 0;    // the first key any query of the block sees
    const int k_begin = k_first / AP_BK * AP_BK;
    const int nj = (HD + 31) / 32;

    for (int k0 = k_begin; k0 <= q_last; k0 += AP_BK) {
        __syncthreads();
        for (int e = threadIdx.x; e < AP_BK * HD; e += blockDim.x) {
            const int r = e / HD, d = e - r * HD;
            const int kp = k0 + r;
            if (PAST && kp < p0) {
                const bool in = kp >= k_first;
                float kv0 = 0.f, kv1 = 0.f;
                if (in) {
                    const int entry = ring ? kp % ring : kp;
                    const long long off = (long long)(entry % PAGE_TOKENS) * HD + d;
                    const int page = prow[entry / PAGE_TOKENS];
                    kv0 = to_f32(kv_tile(pool, 0, pages, page, hk, KVH, HD)[off]);
                    kv1 = to_f32(kv_tile(pool, 1, pages, page, hk, KVH, HD)[off]);
                }
                Ks[r * ldq + d] = kv0;
                Vs[r * HD + d] = kv1;
                continue;
            }
            const bool in = kp < len;
            const long long row = (long long)(s0 + kp - p0) * ld + (long long)hk * HD + d;
            Ks[r * ldq + d] = in ? to_f32(k[row]) : 0.f;
            Vs[r * HD + d] = in ? to_f32(v[row]) : 0.f;
        }
        __syncthreads();
        const int kpos = k0 + lane;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int qi = warp * 8 + i;
            const int qpos = q0 + qi;
            const float* qr = Qs + qi * ldq;
            const float* kr = Ks + lane * ldq;
            float s = 0.f;
            for (int d = 0; d < HD; ++d) s = fmaf(qr[d], kr[d], s);
            s *= scale;
            const bool vis = qi < nq && kpos <= qpos && kpos < len && (window <= 0 || kpos + window > qpos);
            s = vis ? s : -INFINITY;
            const float mx = fmaxf(m[i], warp_max(s));
            float p = 0.f, alpha = 1.f;
            if (mx != -INFINITY) {
                p = vis ? expf(s - mx) : 0.f;
                alpha = expf(m[i] - mx);         // exp(-inf) = 0 on the first visible tile
            }
            l[i] = l[i] * alpha + warp_sum(p);
            m[i] = mx;
#pragma unroll
            for (int j = 0; j < AP_MAXJ; ++j) acc[i][j] *= alpha;
            Ps[qi * (AP_BK + 1) + lane] = p;
        }
        __syncwarp();
        for (int kk = 0; kk < AP_BK; ++kk) {
            float vv[AP_MAXJ];
#pragma unroll
            for (int j = 0; j < AP_MAXJ; ++j) vv[j] = (j < nj && lane + 32 * j < HD) ? Vs[kk * HD + lane + 32 * j] : 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float p = Ps[(warp * 8 + i) * (AP_BK + 1) + kk];
#pragma unroll
                for (int j = 0; j < AP_MAXJ; ++j) acc[i][j] = fmaf(p, vv[j], acc[i][j]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int qi = warp * 8 + i;
        if (qi >= nq) continue;
        const long long t = s0 + q0 - p0 + qi;
        float g = 1.f;
        if (gate) g = sigmoid_f32(to_f32(gate[t * ldg + hq]));
        const float inv = 1.f / l[i];
#pragma unroll
        for (int j = 0; j < AP_MAXJ; ++j) {
            const int d = lane + 32 * j;
            if (j < nj && d < HD) ctx[t * ldc + (long long)hq * HD + d] = from_f32<T>(acc[i][j] * inv * g);
        }
    }
}

template <typename T, bool PAST>
static int launch_attn_simt(void* ctx, long long ldc, const void* q, const void* k, const void* v, long long ld,
                            const void* gate, long long ldg, const int* seq_start, int B, int max_len, int QH, int KVH,
                            int HD, int window, float scale, const int* seq_pos0, const int* seq_slot, const void* pool,
                            long long pages, const int* ptab, int ptab_stride, int ring, cudaStream_t st) {
    const size_t smem = ((size_t)(AP_BQ + AP_BK) * (HD + 1) + (size_t)AP_BK * HD + AP_BQ * (AP_BK + 1)) * sizeof(float);
    dim3 grid((max_len + AP_BQ - 1) / AP_BQ, QH, B);
    cudaFuncSetAttribute(attn_prefill_simt_kernel<T, PAST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cm_launch(attn_prefill_simt_kernel<T, PAST>, grid, 128, smem, st, (T*)ctx, ldc, (const T*)q, (const T*)k, (const T*)v,
              ld, (const T*)gate, ldg, seq_start, QH, KVH, HD, window, scale, seq_pos0, seq_slot, (const T*)pool, pages,
              ptab, ptab_stride, ring);
    CM_CHECK_LAUNCH();
    return CM_OK;
}

extern "C" int cm_attn_prefill_simt(int dt, void* ctx, long long ldc, const void* q, const void* k,
                                    const void* v, long long ld, const void* gate, long long ldg,
                                    const int* seq_start, int B, int max_len, int QH, int KVH, int HD,
                                    int window, float scale, cudaStream_t st) {
    if (B <= 0 || max_len <= 0) return CM_OK;
    if (HD > 32 * AP_MAXJ) CM_REFUSE("attn_prefill: head size %d above %d", HD, 32 * AP_MAXJ);
    if (QH % KVH) CM_REFUSE("attn_prefill: %d query heads over %d key heads", QH, KVH);
    if (dt == DT_F32)
        return launch_attn_simt<float, false>(ctx, ldc, q, k, v, ld, gate, ldg, seq_start, B, max_len, QH, KVH, HD, window,
                                              scale, nullptr, nullptr, nullptr, 0, nullptr, 0, 0, st);
    if (dt == DT_BF16)
        return launch_attn_simt<bf16, false>(ctx, ldc, q, k, v, ld, gate, ldg, seq_start, B, max_len, QH, KVH, HD, window,
                                             scale, nullptr, nullptr, nullptr, 0, nullptr, 0, 0, st);
    return CM_ERR_DTYPE;
}

// The same for sequences that stand at seq_pos0[b] >= 0: keys and values below that position come
// from the paged cache of this layer (pool [2][pages][KVH][PAGE_TOKENS][HD], page table row of
// seq_slot[b]), the rest from the step's rows.  max_len: the most new tokens of a sequence.
extern "C" int cm_attn_append_simt(int dt, void* ctx, long long ldc, const void* q, const void* k,
                                   const void* v, long long ld, const void* gate, long long ldg,
                                   const int* seq_start, const int* seq_pos0, const int* seq_slot, const void* pool,
                                   long long pages, const int* ptab, long long ptab_stride, int ring, int B,
                                   int max_len, int QH, int KVH, int HD, int window, float scale, cudaStream_t st) {
    if (B <= 0 || max_len <= 0) return CM_OK;
    if (HD > 32 * AP_MAXJ) CM_REFUSE("attn_append: head size %d above %d", HD, 32 * AP_MAXJ);
    if (QH % KVH) CM_REFUSE("attn_append: %d query heads over %d key heads", QH, KVH);
    if (ring % PAGE_TOKENS) CM_REFUSE("attn_append: ring of %d entries is no multiple of %d", ring, PAGE_TOKENS);
    if (!seq_pos0 || !seq_slot || !pool || !ptab) CM_REFUSE("attn_append: positions, slots, cache and page table are needed");
    if (dt == DT_F32)
        return launch_attn_simt<float, true>(ctx, ldc, q, k, v, ld, gate, ldg, seq_start, B, max_len, QH, KVH, HD, window,
                                             scale, seq_pos0, seq_slot, pool, pages, ptab, (int)ptab_stride, ring, st);
    if (dt == DT_BF16)
        return launch_attn_simt<bf16, true>(ctx, ldc, q, k, v, ld, gate, ldg, seq_start, B, max_len, QH, KVH, HD, window,
                                            scale, seq_pos0, seq_slot, pool, pages, ptab, (int)ptab_stride, ring, st);
    return CM_ERR_DTYPE;
}

// Keys (already normed and rotated) and values of the step's tokens into the paged cache: what
// cm_qk_prepare does with a pool, as a step of its own for steps whose attention must still read
// the entries that these rows replace.  kv: the k | v columns of the packed rows (k at column 0,
// v at column KVH * HD), row pitch ld.  A ring keeps only the last `ring` positions of a sequence.
template <typename T>
__global__ void kv_store_kernel(const T* __restrict__ kv, long long ld, const int* __restrict__ tok_pos,
                                const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                                const int* __restrict__ seq_end, T* __restrict__ pool, long long pages,
                                const int* __restrict__ ptab, int ptab_stride, int ring, int KVH, int HD) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, b = tok_seq[t], pos = tok_pos[t];
    if (b < 0) return;                                  // padding
    if (ring && pos + ring < seq_end[b]) return;
    const int entry = ring ? pos % ring : pos;
    const int page = ptab[(long long)seq_slot[b] * ptab_stride + entry / PAGE_TOKENS];
    const int row = entry % PAGE_TOKENS;
    const int width = KVH * HD;
    for (int e = threadIdx.x; e < 2 * width; e += blockDim.x) {
        const int plane = e / width, c = e - plane * width, kvh = c / HD, d = c - kvh * HD;
        kv_tile(pool, plane, pages, page, kvh, KVH, HD)[(long long)row * HD + d] = kv[(long long)t * ld + e];
    }
}

extern "C" int cm_kv_store(int dt, const void* kv, long long ld, const int* tok_pos, const int* tok_seq,
                           const int* seq_slot, const int* seq_end, void* pool, long long pages, const int* ptab,
                           long long ptab_stride, int ring, int T, int KVH, int HD, cudaStream_t st) {
    if (T <= 0) return CM_OK;
    if (ring % PAGE_TOKENS) CM_REFUSE("kv_store: ring of %d entries is no multiple of %d", ring, PAGE_TOKENS);
    const int threads = 2 * KVH * HD >= 256 ? 256 : 128;
    if (dt == DT_F32)
        cm_launch(kv_store_kernel<float>, T, threads, 0, st, (const float*)kv, ld, tok_pos, tok_seq, seq_slot, seq_end,
                  (float*)pool, pages, ptab, (int)ptab_stride, ring, KVH, HD);
    else if (dt == DT_BF16)
        cm_launch(kv_store_kernel<bf16>, T, threads, 0, st, (const bf16*)kv, ld, tok_pos, tok_seq, seq_slot, seq_end,
                  (bf16*)pool, pages, ptab, (int)ptab_stride, ring, KVH, HD);
    else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// =========================================================================================
// Decode attention over the paged cache.  One new query token per sequence.
// Grid (chunk, kv head, sequence); a chunk is AD_CHUNK cache entries (4 pages), one page per
// warp.  The G = QH/KVH query heads of the kv head share every key and value that is read;
// they are taken AD_GB at a time.  Each block leaves (max, sum, unnormalised output) per head
// in scratch; cm_attn_decode's second kernel merges the chunks in index order and applies the
// head gate.  Chunk borders are fixed, so a sequence's result does not depend on its
// batch-mates.
//   growing group: entry e holds position e;          entries 0..pos
//   ring group:    entry e holds the latest position <= pos that is congruent to e (mod ring)
// =========================================================================================
#define AD_CHUNK CM_ATTN_DECODE_CHUNK
#define AD_THREADS 128

// AD_GB: query heads of a kv head that one pass handles (1, 2, 4 or 8; more heads take more passes)
template <typename T, int AD_GB>
__global__ void __launch_bounds__(AD_THREADS)
attn_decode_kernel(float* __restrict__ part_o, float* __restrict__ part_ml, const T* __restrict__ q,
                   long long ldq, const int* __restrict__ seq_pos, const int* __restrict__ seq_slot,
                   const T* __restrict__ pool, long long pages, const int* __restrict__ ptab,
                   int ptab_stride, int ring, int window, int QH, int KVH, int HD, int n_chunks,
                   float scale) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    float* qs = smem;                               // [AD_GB][HD]
    float* ss = qs + AD_GB * HD;                    // [AD_GB][AD_CHUNK]
    float* red = ss + AD_GB * AD_CHUNK;             // [groups][AD_GB][HD] partial outputs
    __shared__ float ml[AD_GB][2];
    const int c = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const int G = QH / KVH;
    const int pos = seq_pos[b];                     // position of the query token
    const int n_entries = ring ? min(pos + 1, ring) : pos + 1;
    const int e0 = c * AD_CHUNK;
    if (e0 >= n_entries) return;
    const int slot = seq_slot[b];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tpr = HD / 8;                         // threads per value row (8 channels each)
    const int groups = AD_THREADS / tpr;
    const int vg = threadIdx.x / tpr, vc = (threadIdx.x - vg * tpr) * 8;

    // page of this warp
    const int page_idx = e0 / PAGE_TOKENS + warp;
    const bool page_live = page_idx * PAGE_TOKENS < n_entries;
    const int page = page_live ? ptab[(long long)slot * ptab_stride + page_idx] : 0;

    for (int g0 = 0; g0 < G; g0 += AD_GB) {
        const int ng = min(AD_GB, G - g0);
        __syncthreads();
        for (int e = threadIdx.x; e < AD_GB * HD; e += AD_THREADS) {
            const int g = e / HD, d = e - g * HD;
            qs[e] = g < ng ? to_f32(q[(long long)b * ldq + (long long)(hk * G + g0 + g) * HD + d]) : 0.f;
        }
        __syncthreads();
        // ---- scores of this warp's page
        if ((tpr & (tpr - 1)) == 0 && tpr <= 32) {
            // head sizes 16, 32, 64, 128, 256: HD/8 lanes share a key row (16 bytes each), so a warp
            // reads 32/tpr whole rows (512 contiguous bytes) per step; the partial dot products of a
            // row are added over its lanes by xor shuffles
            const int kq = lane / tpr, dq = lane - kq * tpr, kpw = 32 / tpr;
            float qr[AD_GB][8];
#pragma unroll
            for (int g = 0; g < AD_GB; ++g)
#pragma unroll
                for (int i = 0; i < 8; ++i) qr[g][i] = qs[g * HD + dq * 8 + i];
            const T* kpage = kv_tile(pool, 0, pages, page, hk, KVH, HD);
            constexpr int SU = 4;                          // key rows in flight per lane
            for (int r0 = 0; r0 < PAGE_TOKENS; r0 += kpw * SU) {
                float kv8[SU][8];
                unsigned vis_mask = 0;
#pragma unroll
                for (int u = 0; u < SU; ++u) {
                    const int row = r0 + u * kpw + kq;
                    const int e = page_idx * PAGE_TOKENS + row;
                    bool v_u = false;
                    if (row < PAGE_TOKENS && page_live && e < n_entries) {
                        int kpos = e;
                        if (ring) {
                            int back = (pos - e) % ring;
                            if (back < 0) back += ring;
                            kpos = pos - back;
                        }
                        v_u = kpos >= 0 && kpos <= pos && (window <= 0 || kpos + window > pos);
                    }
                    if (v_u) {
                        vis_mask |= 1u << u;
                        load8<T>(kpage + (long long)row * HD + dq * 8, kv8[u]);
                    }
                }
#pragma unroll
                for (int u = 0; u < SU; ++u) {
                    const int row = r0 + u * kpw + kq;
                    if (row >= PAGE_TOKENS) continue;      // uniform over the warp: kq < kpw, rows come in whole steps
#pragma unroll
                    const bool v_u = (vis_mask >> u) & 1u;
#pragma unroll
                    for (int g = 0; g < AD_GB; ++g) {
                        float sg = 0.f;
                        if (v_u) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) sg = fmaf(qr[g][i], kv8[u][i], sg);
                        }
                        for (int o = tpr >> 1; o > 0; o >>= 1) sg += __shfl_xor_sync(0xffffffffu, sg, o);
                        if (dq == 0) ss[g * AD_CHUNK + warp * PAGE_TOKENS + row] = v_u ? sg * scale : -INFINITY;
                    }
                }
            }
        } else {
        // ---- any other head size: a lane owns entries lane and lane+32 of its warp's page
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = lane + 32 * r;
            const int e = page_idx * PAGE_TOKENS + row;
            float s[AD_GB];
#pragma unroll
            for (int g = 0; g < AD_GB; ++g) s[g] = 0.f;
            bool vis = false;
            if (page_live && e < n_entries) {
                int kpos = e;
                if (ring) {
                    int back = (pos - e) % ring;      // pos >= 0, e < ring: C remainder may be negative
                    if (back < 0) back += ring;
                    kpos = pos - back;
                }
                vis = kpos >= 0 && kpos <= pos && (window <= 0 || kpos + window > pos);
                if (vis) {
                    const T* kr = kv_tile(pool, 0, pages, page, hk, KVH, HD) + (long long)row * HD;
                    for (int d = 0; d < HD; d += 8) {
                        float kv8[8];
                        load8<T>(kr + d, kv8);
#pragma unroll
                        for (int g = 0; g < AD_GB; ++g) {
                            const float* qg = qs + g * HD + d;
#pragma unroll
                            for (int i = 0; i < 8; ++i) s[g] = fmaf(qg[i], kv8[i], s[g]);
                        }
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < AD_GB; ++g)
                ss[g * AD_CHUNK + warp * PAGE_TOKENS + row] = vis ? s[g] * scale : -INFINITY;
        }
        }
        __syncthreads();
        // ---- softmax pieces per head: warp w takes heads w, w+4
        for (int g = warp; g < AD_GB; g += AD_THREADS / 32) {
            float mx = -INFINITY;
            for (int e = lane; e < AD_CHUNK; e += 32) mx = fmaxf(mx, ss[g * AD_CHUNK + e]);
            mx = warp_max(mx);
            float sum = 0.f;
            for (int e = lane; e < AD_CHUNK; e += 32) {
                const float sv = ss[g * AD_CHUNK + e];
                const float p = (mx == -INFINITY || sv == -INFINITY) ? 0.f : expf(sv - mx);
                ss[g * AD_CHUNK + e] = p;
                sum += p;
            }
            sum = warp_sum(sum);
            if (lane == 0) {
                ml[g][0] = mx;
                ml[g][1] = sum;
            }
        }
        __syncthreads();
        // ---- PV: thread (vg, vc) sums entries vg, vg+groups, ... for 8 channels of every head
        float acc[AD_GB][8];
#pragma unroll
        for (int g = 0; g < AD_GB; ++g)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
        if (vg < groups) {
            const int n_here = min(AD_CHUNK, n_entries - e0);
            // the chunk's four pages, looked up once
            const int* prow = ptab + (long long)slot * ptab_stride + e0 / PAGE_TOKENS;
            const T* vp0 = kv_tile(pool, 1, pages, prow[0], hk, KVH, HD) + vc;
            const T* vp1 = kv_tile(pool, 1, pages, n_here > 64 ? prow[1] : 0, hk, KVH, HD) + vc;
            const T* vp2 = kv_tile(pool, 1, pages, n_here > 128 ? prow[2] : 0, hk, KVH, HD) + vc;
            const T* vp3 = kv_tile(pool, 1, pages, n_here > 192 ? prow[3] : 0, hk, KVH, HD) + vc;
            constexpr int VU = 4;                          // value rows in flight per thread
            for (int eb = vg; eb < n_here; eb += groups * VU) {
                float vv[VU][8];
#pragma unroll
                for (int u = 0; u < VU; ++u) {
                    const int e = eb + u * groups;
                    if (e < n_here) {
                        const int pi = e / PAGE_TOKENS;
                        const T* base = pi == 0 ? vp0 : (pi == 1 ? vp1 : (pi == 2 ? vp2 : vp3));
                        load8<T>(base + (long long)(e % PAGE_TOKENS) * HD, vv[u]);
                    }
                }
#pragma unroll
                for (int u = 0; u < VU; ++u) {
                    const int e = eb + u * groups;
                    if (e >= n_here) continue;
#pragma unroll
                    for (int g = 0; g < AD_GB; ++g) {
                        const float p = ss[g * AD_CHUNK + e];
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[g][i] = fmaf(p, vv[u][i], acc[g][i]);
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < AD_GB; ++g)
#pragma unroll
                for (int i = 0; i < 8; ++i) red[((long long)vg * AD_GB + g) * HD + vc + i] = acc[g][i];
        }
        __syncthreads();
        // ---- fold the entry groups in index order and leave the chunk's partial result
        for (int e = threadIdx.x; e < ng * HD; e += AD_THREADS) {
            const int g = e / HD, d = e - g * HD;
            float o = 0.f;
            for (int x = 0; x < groups; ++x) o += red[((long long)x * AD_GB + g) * HD + d];
            const long long idx = ((long long)b * QH + hk * G + g0 + g) * n_chunks + c;
            part_o[idx * HD + d] = o;
            if (d == 0) {
                part_ml[idx * 2] = ml[g][0];
                part_ml[idx * 2 + 1] = ml[g][1];
            }
        }
    }
}

// Merge of the chunks of one (sequence, head), in chunk order; gate; store.
template <typename T>
__global__ void attn_decode_merge_kernel(T* __restrict__ ctx, long long ldc,
                                         const float* __restrict__ part_o,
                                         const float* __restrict__ part_ml,
                                         const T* __restrict__ gate, long long ldg,
                                         const int* __restrict__ seq_pos, int ring, int QH, int HD,
                                         int n_chunks) {
    pdl_trigger();
    pdl_wait();
    const int hq = blockIdx.x, b = blockIdx.y;
    const int pos = seq_pos[b];
    const int n_entries = ring ? min(pos + 1, ring) : pos + 1;
    const int nc = min(n_chunks, (n_entries + AD_CHUNK - 1) / AD_CHUNK);
    const long long base = ((long long)b * QH + hq) * n_chunks;
    float mx = -INFINITY;
    for (int c = 0; c < nc; ++c) mx = fmaxf(mx, part_ml[(base + c) * 2]);
    float den = 0.f;
    for (int c = 0; c < nc; ++c) {
        const float mc = part_ml[(base + c) * 2];
        den += mc == -INFINITY ? 0.f : part_ml[(base + c) * 2 + 1] * expf(mc - mx);
    }
    float g = 1.f;
    if (gate) g = sigmoid_f32(to_f32(gate[(long long)b * ldg + hq]));
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float o = 0.f;
        for (int c = 0; c < nc; ++c) {
            const float mc = part_ml[(base + c) * 2];
            if (mc != -INFINITY) o += part_o[(base + c) * HD + d] * expf(mc - mx);
        }
        ctx[(long long)b * ldc + (long long)hq * HD + d] = from_f32<T>(o / den * g);
    }
}

int cm_attn_decode_mma_stage(float* part_o, float* part_ml, const void* q, long long ldq, const int* seq_pos,
                             const int* seq_slot, const void* pool, long long pages, const int* ptab,
                             int ptab_stride, int ring, int window, int B, int QH, int KVH, int HD, int n_chunks,
                             float scale, int* n_parts_out, cudaStream_t st);

// Scratch: part_o holds B*QH*n_chunks*HD floats, part_ml B*QH*n_chunks*2 floats.
// bfloat16 with a head size that is a multiple of 16 up to 128 runs its first stage on the
// tensor cores (attention_mma.cu); everything else on the CUDA cores.  use_mma = 0 forces the
// CUDA-core stage.
static int g_decode_mma = 1;
extern "C" void cm_attn_decode_set_mma(int on) { g_decode_mma = on; }

extern "C" int cm_attn_decode(int dt, void* ctx, long long ldc, const void* q, long long ldq,
                              const void* gate, long long ldg, const int* seq_pos, const int* seq_slot,
                              const void* pool, long long pages, const int* ptab, int ptab_stride,
                              int ring, int window, int B, int QH, int KVH, int HD, int n_chunks,
                              float scale, float* part_o, float* part_ml, cudaStream_t st) {
    if (B <= 0) return CM_OK;
    if (HD % 8 || HD < 8 || HD > CM_MAX_HEAD_DIM)
        CM_REFUSE("attn_decode: head size %d (multiples of 8 up to %d)", HD, CM_MAX_HEAD_DIM);
    if (QH % KVH) CM_REFUSE("attn_decode: %d query heads over %d key heads", QH, KVH);
    if (ring % PAGE_TOKENS) CM_REFUSE("attn_decode: ring of %d entries is no multiple of %d", ring, PAGE_TOKENS);
    if (n_chunks <= 0) CM_REFUSE("attn_decode: %d chunks", n_chunks);
    const int G = QH / KVH;
    const int gb = G >= 8 ? 8 : (G >= 4 ? 4 : (G >= 2 ? 2 : 1));
    const int groups = AD_THREADS / (HD / 8);
    const size_t smem = ((size_t)gb * HD + (size_t)gb * AD_CHUNK + (size_t)groups * gb * HD) * sizeof(float);
    dim3 grid(n_chunks, KVH, B);
    dim3 mgrid(QH, B);
    const int mthreads = HD <= 64 ? 64 : 128;
#define AD_LAUNCH(TT, GB)                                                                                          \
    do {                                                                                                           \
        cudaFuncSetAttribute(attn_decode_kernel<TT, GB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
        cm_launch(attn_decode_kernel<TT, GB>, grid, AD_THREADS, smem, st, part_o, part_ml, (const TT*)q, ldq, seq_pos, \
                  seq_slot, (const TT*)pool, pages, ptab, ptab_stride, ring, window, QH, KVH, HD, n_chunks, scale); \
    } while (0)
#define AD_DISPATCH(TT)                   \
    do {                                  \
        if (gb == 8) AD_LAUNCH(TT, 8);    \
        else if (gb == 4) AD_LAUNCH(TT, 4); \
        else if (gb == 2) AD_LAUNCH(TT, 2); \
        else AD_LAUNCH(TT, 1);            \
    } while (0)
    if (dt == DT_BF16 && g_decode_mma && HD % 16 == 0 && HD <= 128 && ldq % 2 == 0 &&
        ((uintptr_t)q & 3) == 0 && ((uintptr_t)pool & 15) == 0) {
        int n_parts = n_chunks;                    // blocks per (sequence, kv head): at most n_chunks
        const int rc = cm_attn_decode_mma_stage(part_o, part_ml, q, ldq, seq_pos, seq_slot, pool, pages, ptab,
                                                ptab_stride, ring, window, B, QH, KVH, HD, n_chunks, scale,
                                                &n_parts, st);
        if (rc != CM_OK) return rc;
        cm_launch(attn_decode_merge_kernel<bf16>, mgrid, mthreads, 0, st, (bf16*)ctx, ldc, part_o, part_ml,
                  (const bf16*)gate, ldg, seq_pos, ring, QH, HD, n_parts);
    } else if (dt == DT_F32) {
        AD_DISPATCH(float);
        CM_CHECK_LAUNCH();
        cm_launch(attn_decode_merge_kernel<float>, mgrid, mthreads, 0, st, (float*)ctx, ldc, part_o, part_ml,
                  (const float*)gate, ldg, seq_pos, ring, QH, HD, n_chunks);
    } else if (dt == DT_BF16) {
        AD_DISPATCH(bf16);
        CM_CHECK_LAUNCH();
        cm_launch(attn_decode_merge_kernel<bf16>, mgrid, mthreads, 0, st, (bf16*)ctx, ldc, part_o, part_ml,
                  (const bf16*)gate, ldg, seq_pos, ring, QH, HD, n_chunks);
    } else
        return CM_ERR_DTYPE;
#undef AD_DISPATCH
#undef AD_LAUNCH
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// =========================================================================================
// The same decode attention for callers that cannot allocate (see attention_noalloc.h).
// The per-chunk partial results live in this file-scope device array instead of in buffers
// the caller provides.  In host code `noalloc_scratch` is only a handle for the runtime, not
// a device address: the address a kernel can use comes from cudaGetSymbolAddress, looked up
// once per device with that device current.
// =========================================================================================
#include "attention_noalloc.h"
#include <mutex>

static __device__ __align__(256) float noalloc_scratch[CM_NOALLOC_SCRATCH_FLOATS];

#define CM_NOALLOC_MAX_DEVICES 64
static float* g_noalloc_ptr[CM_NOALLOC_MAX_DEVICES] = {nullptr};
static std::mutex g_noalloc_mutex;

// Device address of the scratch array on the current device (set up at the first call there).
static int noalloc_scratch_address(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= CM_NOALLOC_MAX_DEVICES) {
        cm_set_error("attn_decode_noalloc: cannot tell the current device (%s)", cudaGetErrorString(e));
        return CM_ERR_DRIVER;
    }
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_ptr[dev]) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, noalloc_scratch);
        if (e != cudaSuccess || !p) {
            cm_set_error("attn_decode_noalloc: cudaGetSymbolAddress failed on device %d (%s)", dev,
                         cudaGetErrorString(e));
            return CM_ERR_DRIVER;
        }
        g_noalloc_ptr[dev] = p;
    }
    *out = g_noalloc_ptr[dev];
    return CM_OK;
}

extern "C" int cm_attn_decode_noalloc(int dt, void* ctx, long long ldc, const void* q, long long ldq,
                                      const void* gate, long long ldg, const int* seq_pos, const int* seq_slot,
                                      const void* pool, long long pages, const int* ptab, int ptab_stride,
                                      int ring, int window, int B, int QH, int KVH, int HD, int n_chunks,
                                      float scale, cudaStream_t st) {
    if (B <= 0) return CM_OK;
    if (QH <= 0 || HD <= 0 || n_chunks <= 0) CM_REFUSE("attn_decode_noalloc: %d heads, head size %d, %d chunks", QH, HD, n_chunks);
    const long long o_floats = (long long)B * QH * n_chunks * HD;       // unnormalised outputs per chunk
    const long long ml_floats = (long long)B * QH * n_chunks * 2;       // maximum and sum per chunk
    if (o_floats + ml_floats > CM_NOALLOC_SCRATCH_FLOATS)
        CM_REFUSE("attn_decode_noalloc: %lld floats of scratch wanted (B=%d, heads=%d, chunks=%d, head size=%d), "
                  "the built-in array holds %d", o_floats + ml_floats, B, QH, n_chunks, HD, CM_NOALLOC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    const int rc = noalloc_scratch_address(&scratch);
    if (rc != CM_OK) return rc;
    // part_o first (16-byte aligned for any size since HD is a multiple of 8), then part_ml
    return cm_attn_decode(dt, ctx, ldc, q, ldq, gate, ldg, seq_pos, seq_slot, pool, pages, ptab, ptab_stride, ring,
                          window, B, QH, KVH, HD, n_chunks, scale, scratch, scratch + o_floats, st);
}
