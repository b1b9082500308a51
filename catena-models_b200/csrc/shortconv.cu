// Gated short convolution between in_proj and out_proj, with its per-sequence state.
//
//   bcx row: [ B: H | C: H | X: H ]         bx = B * X               (float, never rounded)
//   s = concat(state[K-1, H], bx[T_b, H])    z[i,c] = sum_j w[c,j] * s[i+j, c]   (j = 0..K-1)
//   y = T(z * C)                             state <- s[T_b : T_b + K-1]           (float)
// One thread per (token, channel).  A prompt step starts every sequence from an empty state
// (from_zero = 1: the stored state is not read, so a slot that is used again needs no
// clearing); a decode step has one token per sequence and shifts the state in place.
// A step that brings several tokens on top of a stored state (seq_pos0[b] > 0) runs in two
// launches, because the first tokens of a sequence read the state that its last token replaces:
// phase 1 writes the outputs only, phase 2 the state only.  With seq_pos0 given, a sequence whose
// first position is 0 starts from an empty state whatever from_zero says.  A row whose tok_seq is
// negative is padding (a step recorded for a class of shapes carries some): its output is zero.
#include "common.cuh"

#define SC_MAXK CM_MAX_CONV_TAPS

template <typename T>
__global__ void shortconv_kernel(T* __restrict__ y, const T* __restrict__ bcx, long long ld,
                                 const float* __restrict__ w, float* __restrict__ state,
                                 const int* __restrict__ tok_seq, const int* __restrict__ seq_start,
                                 const int* __restrict__ seq_slot, const int* __restrict__ seq_pos0, int H, int K,
                                 int from_zero, int phase) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int t = blockIdx.x;                     // tokens on x: a step may carry more than 65535 of them
    if (c >= H) return;
    const int b = tok_seq[t];
    if (b < 0) {                                  // a row of padding belongs to no sequence: zeros out
        if (phase != 2) y[(long long)t * H + c] = from_f32<T>(0.f);
        return;
    }
    const int s0 = seq_start[b], len = seq_start[b + 1] - s0;
    const int i = t - s0;
    if (phase == 2 && i != len - 1) return;
    if (seq_pos0 && seq_pos0[b] == 0) from_zero = 1;
    float* st = state + (long long)seq_slot[b] * (K - 1) * H + c;     // [K-1] entries, stride H
    const float* wc = w + (long long)c * K;

    float z = 0.f;
    float cur = 0.f;
    for (int j = 0; j < K; ++j) {
        const int r = i + j - (K - 1);            // row of bx; negative rows lie in the state
        float sv;
        if (r >= 0) {
            const T* row = bcx + (long long)(s0 + r) * ld;
            sv = to_f32(row[c]) * to_f32(row[2 * H + c]);
            if (j == K - 1) cur = sv;
        } else {
            sv = from_zero ? 0.f : st[(long long)(K - 1 + r) * H];
        }
        z += wc[j] * sv;
    }
    if (phase != 2) {
        const float cc = to_f32(bcx[(long long)t * ld + H + c]);
        y[(long long)t * H + c] = from_f32<T>(z * cc);
    }

    if (i == len - 1 && phase != 1) {
        // new state entry j = s[len + j]; s index below K-1 is an old state entry
        for (int j = 0; j < K - 1; ++j) {
            const int r = len + j - (K - 1);
            float sv;
            if (r == len - 1)
                sv = cur;
            else if (r >= 0) {
                const T* row = bcx + (long long)(s0 + r) * ld;
                sv = to_f32(row[c]) * to_f32(row[2 * H + c]);
            } else
                sv = from_zero ? 0.f : st[(long long)(len + j) * H];   // len + j > j: not yet overwritten
            st[(long long)j * H] = sv;
        }
    }
}

// The same, eight channels per thread with 16-byte accesses (H a multiple of 8, aligned rows).
// KT: the number of taps when it is one of the usual ones (the loops over taps are then unrolled and
// every load of a thread is in flight at once; with a loop that waits tap by tap a thread has two
// loads in flight and 2,048 tokens of 2,048 channels take 10.4 us), or 0 for any number.
template <typename T, int KT>
__global__ void __launch_bounds__(128)
shortconv_vec_kernel(T* __restrict__ y, const T* __restrict__ bcx, long long ld, const float* __restrict__ w,
                     const float* __restrict__ w_t, float* __restrict__ state, const int* __restrict__ tok_seq, const int* __restrict__ seq_start,
                     const int* __restrict__ seq_slot, const int* __restrict__ seq_pos0, int T_tokens, int H, int K_any,
                     int from_zero, int phase) {
    pdl_trigger();
    pdl_wait();
    // threadIdx.y walks consecutive tokens: the rows a token shares with its neighbours (K - 1 of
    // its K) are then read by the same block and come from L1 after the first time
    const int K = KT ? KT : K_any;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    const int t = blockIdx.x * blockDim.y + threadIdx.y;
    if (c >= H || t >= T_tokens) return;
    const int b = tok_seq[t];
    if (b < 0) {                                  // a row of padding belongs to no sequence: zeros out
        if (phase != 2) {
            const float zeros[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            store8f<T>(y + (long long)t * H + c, zeros);
        }
        return;
    }
    const int s0 = seq_start[b], len = seq_start[b + 1] - s0;
    const int i = t - s0;
    if (phase == 2 && i != len - 1) return;
    if (seq_pos0 && seq_pos0[b] == 0) from_zero = 1;
    float* st = state + (long long)seq_slot[b] * (K - 1) * H + c;
    float z[8], cur[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) z[e] = cur[e] = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) {
        const int r = i + j - (K - 1);
        float sv[8];
        if (r >= 0) {
            const T* row = bcx + (long long)(s0 + r) * ld;
            float bb[8], xx[8];
            load8f<T>(row + c, bb);
            load8f<T>(row + 2 * H + c, xx);
#pragma unroll
            for (int e = 0; e < 8; ++e) sv[e] = bb[e] * xx[e];
        } else if (from_zero) {
#pragma unroll
            for (int e = 0; e < 8; ++e) sv[e] = 0.f;
        } else {
            load8f<float>(st + (long long)(K - 1 + r) * H, sv);
        }
        float wj[8];
        if (w_t) {
            load8f<float>(w_t + (long long)j * H + c, wj);       // taps stored [K][H]: eight channels at once
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) wj[e] = w[(long long)(c + e) * K + j];
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            z[e] += wj[e] * sv[e];
            if (j == K - 1) cur[e] = sv[e];
        }
    }
    if (phase != 2) {
        float cc[8], out[8];
        load8f<T>(bcx + (long long)t * ld + H + c, cc);
#pragma unroll
        for (int e = 0; e < 8; ++e) out[e] = z[e] * cc[e];
        store8f<T>(y + (long long)t * H + c, out);
    }

    if (i == len - 1 && phase != 1) {
        for (int j = 0; j < K - 1; ++j) {
            const int r = len + j - (K - 1);
            float sv[8];
            if (r == len - 1) {
#pragma unroll
                for (int e = 0; e < 8; ++e) sv[e] = cur[e];
            } else if (r >= 0) {
                const T* row = bcx + (long long)(s0 + r) * ld;
                float bb[8], xx[8];
                load8f<T>(row + c, bb);
                load8f<T>(row + 2 * H + c, xx);
#pragma unroll
                for (int e = 0; e < 8; ++e) sv[e] = bb[e] * xx[e];
            } else if (from_zero) {
#pragma unroll
                for (int e = 0; e < 8; ++e) sv[e] = 0.f;
            } else {
                load8f<float>(st + (long long)(len + j) * H, sv);       // len + j > j: not yet overwritten
            }
            store8f<float>(st + (long long)j * H, sv);
        }
    }
}

// w: taps [H][K]; w_t: the same taps stored [K][H] (optional; lets the vector kernel read them
// eight channels at a time).
extern "C" int cm_shortconv(int dt, void* y, const void* bcx, long long ld, const float* w, const float* w_t,
                            float* state,
                            const int* tok_seq, const int* seq_start, const int* seq_slot, const int* seq_pos0,
                            int T, int H, int K, int from_zero, int one_token_each, cudaStream_t st) {
    if (T <= 0) return CM_OK;
    if (K < 2 || K > SC_MAXK) CM_REFUSE("shortconv: %d taps (2..%d)", K, SC_MAXK);
    // several tokens on top of a stored state: outputs first, then the state (see the top of the file)
    const int first_phase = (!from_zero && !one_token_each) ? 1 : 0;
    const int last_phase = first_phase ? 2 : 0;
    for (int phase = first_phase; phase <= last_phase; ++phase) {
    const bool vec = H % 8 == 0 && ld % 8 == 0 && (((uintptr_t)y | (uintptr_t)bcx | (uintptr_t)state) & 15) == 0;
    if (vec) {
        // few tokens: a token per block (128 channel groups); many: 4 consecutive tokens per block
        const int ty = T >= 256 ? 4 : 1, tx = 128 / ty;
        dim3 vblock(tx, ty), vgrid((T + ty - 1) / ty, (H / 8 + tx - 1) / tx);
#define SC_LAUNCH_VEC(TT, KT)                                                                                      \
    cm_launch(shortconv_vec_kernel<TT, KT>, vgrid, vblock, 0, st, (TT*)y, (const TT*)bcx, ld, w, w_t, state, tok_seq, \
              seq_start, seq_slot, seq_pos0, T, H, K, from_zero, phase)
#define SC_LAUNCH_TAPS(TT)                \
    do {                                  \
        switch (K) {                      \
            case 2: SC_LAUNCH_VEC(TT, 2); break; \
            case 3: SC_LAUNCH_VEC(TT, 3); break; \
            case 4: SC_LAUNCH_VEC(TT, 4); break; \
            case 7: SC_LAUNCH_VEC(TT, 7); break; \
            default: SC_LAUNCH_VEC(TT, 0); break; \
        }                                 \
    } while (0)
        if (dt == DT_F32)
            SC_LAUNCH_TAPS(float);
        else if (dt == DT_BF16)
            SC_LAUNCH_TAPS(bf16);
        else
            return CM_ERR_DTYPE;
        CM_CHECK_LAUNCH();
        continue;
    }
    dim3 grid(T, (H + 127) / 128);
    if (dt == DT_F32)
        cm_launch(shortconv_kernel<float>, grid, 128, 0, st, (float*)y, (const float*)bcx, ld, w, state, tok_seq,
                                                      seq_start, seq_slot, seq_pos0, H, K, from_zero, phase);
    else if (dt == DT_BF16)
        cm_launch(shortconv_kernel<bf16>, grid, 128, 0, st, (bf16*)y, (const bf16*)bcx, ld, w, state, tok_seq,
                                                     seq_start, seq_slot, seq_pos0, H, K, from_zero, phase);
    else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    }
    return CM_OK;
}
