// Prefill attention on the tensor cores (bfloat16, head sizes that are multiples of 16 up to
// 128): online-softmax attention over the step's own keys and values with causal or sliding
// mask, grouped-query heads, unequal sequence lengths and the per-head sigmoid gate.
//
// One block = 64 queries of one head of one sequence, 4 warps of 16 query rows.  Keys and
// values come in tiles of 64 through a two-stage cp.async ring in shared memory (rows padded
// by 16 bytes so that ldmatrix reads without bank conflicts).  S = Q K^T and O += P V run on
// mma.sync.m16n8k16 with float accumulation; the score accumulators are re-used as the
// probability operand of the second product.  Maximum, sum, rescaling and the final division
// are float; exp is taken as exp2 of log2(e)-prescaled scores.
//
// PAST: sequences may stand at a position p0 > 0 (several tokens on top of a started sequence).
// Key tiles are then cut at multiples of 64 absolute positions, which are the cache's pages: a
// row below p0 comes from the sequence's page of the cache (entry = position, or position % ring),
// a row from p0 on from the step's own rows, which reach the cache only after this kernel.  Rows
// that no query of the block can see are not read (zero-filled).
#include "common.cuh"
#include <math.h>

#define FA_BQ 64
#define FA_BK 64

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int n = valid ? 16 : 0;                 // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the special-function unit (one instruction; -inf gives 0, as the masks need)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

template <int HD, int BQ, bool PAST>
__global__ void __launch_bounds__(BQ * 2, HD <= 64 ? 512 / (BQ * 2) : 256 / (BQ * 2))
attn_prefill_mma_kernel(bf16* __restrict__ ctx, long long ldc, const bf16* __restrict__ q,
                        const bf16* __restrict__ k, const bf16* __restrict__ v, long long ld,
                        const bf16* __restrict__ gate, long long ldg, const int* __restrict__ seq_start, int QH,
                        int KVH, int window, float scale_log2, const int* __restrict__ seq_pos0,
                        const int* __restrict__ seq_slot, const bf16* __restrict__ pool, long long pages,
                        const int* __restrict__ ptab, int ptab_stride, int ring) {
    constexpr int LDS = HD + 8;                   // padded row, elements
    constexpr int CH = HD / 8;                    // 16-byte chunks per row
    extern __shared__ __align__(16) uint8_t fa_smem[];
    bf16* Qs = reinterpret_cast<bf16*>(fa_smem);              // [BQ][LDS]
    bf16* Ks = Qs + BQ * LDS;                              // [2][FA_BK][LDS]
    bf16* Vs = Ks + 2 * FA_BK * LDS;                          // [2][FA_BK][LDS]
    pdl_wait();
    const int b = blockIdx.z, hq = blockIdx.y, hk = hq / (QH / KVH);
    const int s0 = seq_start[b], n_new = seq_start[b + 1] - s0;
    const int p0 = PAST ? seq_pos0[b] : 0;                 // position of the sequence's first row of this step
    const int len = p0 + n_new;                            // positions are absolute from here on
    constexpr int THREADS = BQ * 2;
    const int q0 = p0 + (gridDim.x - 1 - blockIdx.x) * BQ; // long rows first
    if (q0 >= len) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;

    const int k_first = window > 0 ? max(0, q0 - window + 1) : 0;   // the first key a query of this block sees
    const int kt_begin = k_first / FA_BK;
    const int kt_end = min(q0 + BQ - 1, len - 1) / FA_BK;  // inclusive
    const int* prow = PAST ? ptab + (long long)seq_slot[b] * ptab_stride : nullptr;

    // a thread's share of a 64-row tile: chunks e = tid, tid + 128, ...; row and column of each
    // are the same for every tile, so they are worked out once
    constexpr int PER = (FA_BK * CH + THREADS - 1) / THREADS;
    int l_row[PER], l_off[PER];
#pragma unroll
    for (int u = 0; u < PER; ++u) {
        const int e = tid + u * THREADS;
        l_row[u] = e < FA_BK * CH ? e / CH : -1;
        l_off[u] = (e % CH) * 8;
    }
    // rows row0 .. row0 + 63 (absolute positions) of the step's own q, k or v
    auto load_tile = [&](bf16* dst, const bf16* src, int row0) {
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            if (l_row[u] < 0) continue;
            const int pos = row0 + l_row[u];
            const bool in = pos < len && pos >= p0;
            const long long row = (long long)(s0 + (in ? pos - p0 : 0));
            cp_async16(dst + l_row[u] * LDS + l_off[u], src + row * ld + l_off[u], in);
        }
    };
    // the same for keys (plane 0) or values (plane 1), rows below p0 from the cache
    auto load_kv = [&](bf16* dst, const bf16* src, int plane, int row0) {
        if (!PAST || row0 >= p0) {
            load_tile(dst, src, row0);
            return;
        }
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            if (l_row[u] < 0) continue;
            const int pos = row0 + l_row[u];
            const bf16* from = src;
            bool in = pos < len;
            if (pos >= p0) {
                from = src + (long long)(s0 + (in ? pos - p0 : 0)) * ld + l_off[u];
            } else {
                in = pos >= k_first;
                if (in) {
                    const int entry = ring ? pos % ring : pos;
                    from = kv_tile(pool, plane, pages, prow[entry / PAGE_TOKENS], hk, KVH, HD) +
                           (long long)(entry % PAGE_TOKENS) * HD + l_off[u];
                }
            }
            cp_async16(dst + l_row[u] * LDS + l_off[u], from, in);
        }
    };
    load_tile(Qs, q + (long long)hq * HD, q0);
    if (BQ > FA_BK) load_tile(Qs + FA_BK * LDS, q + (long long)hq * HD, q0 + FA_BK);
    cp_async_commit();
    load_kv(Ks, k + (long long)hk * HD, 0, kt_begin * FA_BK);
    load_kv(Vs, v + (long long)hk * HD, 1, kt_begin * FA_BK);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    // Q fragments of this warp's 16 rows
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk)
        ldmatrix_x4(qf[kk], Qs + (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + kk * 16 + 8 * (lane >> 4));

    float o[HD / 8][4];
#pragma unroll
    for (int j = 0; j < HD / 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[j][i] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int row_lo = q0 + warp * 16 + g;        // this thread's rows: row_lo and row_lo + 8

    for (int kt = kt_begin; kt <= kt_end; ++kt) {
        const int buf = (kt - kt_begin) & 1;
        if (kt + 1 <= kt_end) {
            load_kv(Ks + (buf ^ 1) * FA_BK * LDS, k + (long long)hk * HD, 0, (kt + 1) * FA_BK);
            load_kv(Vs + (buf ^ 1) * FA_BK * LDS, v + (long long)hk * HD, 1, (kt + 1) * FA_BK);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const bf16* Kt = Ks + buf * FA_BK * LDS;
        const bf16* Vt = Vs + buf * FA_BK * LDS;
        const int key0 = kt * FA_BK;
        // a tile that none of this warp's 16 rows can see (all of it after them, or all of it
        // before their windows) is only waited for
        if (key0 > q0 + warp * 16 + 15 || (window > 0 && key0 + FA_BK - 1 + window <= q0 + warp * 16)) {
            __syncthreads();
            continue;
        }

        // ---- S = Q K^T : 16 x 64 per warp, 8 tiles of 8 keys
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[j][i] = 0.f;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {      // key tiles 2jp, 2jp+1
                uint32_t kb[4];
                ldmatrix_x4(kb, Kt + (jp * 16 + (lane & 7) + 8 * (lane >> 4)) * LDS + kk * 16 + 8 * ((lane >> 3) & 1));
                mma16816(s[2 * jp], qf[kk], kb[0], kb[1]);
                mma16816(s[2 * jp + 1], qf[kk], kb[2], kb[3]);
            }
        }
        // ---- mask, running maximum
        const bool edge = key0 + FA_BK - 1 > q0 + warp * 16 || key0 + FA_BK > len ||
                          (window > 0 && key0 + window <= q0 + warp * 16 + 15);
        // raw scores stay unscaled; the scale (times log2 e) is folded into the exponent's argument
        float mx[2] = {-INFINITY, -INFINITY};
        if (edge) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int key = key0 + 8 * j + 2 * t + (i & 1);
                    const int row = row_lo + (i >> 1) * 8;
                    const bool vis = key <= row && key < len && (window <= 0 || key + window > row);
                    s[j][i] = vis ? s[j][i] : -INFINITY;
                }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) mx[i >> 1] = fmaxf(mx[i >> 1], s[j][i]);
        float alpha[2], m_use[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m_run[h], mx[h] * scale_log2);      // scale > 0: the order of scores is kept
            m_use[h] = m_new == -INFINITY ? 0.f : m_new;
            alpha[h] = fast_exp2(m_run[h] - m_use[h]);                    // 2^(-inf) = 0 on the first visible tile
            m_run[h] = m_new;
        }
        float rs[2] = {0.f, 0.f};
        uint32_t pf[4][4];                                     // P as the A operand, 4 steps of 16 keys
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float p0 = fast_exp2(fmaf(s[j][0], scale_log2, -m_use[0])), p1 = fast_exp2(fmaf(s[j][1], scale_log2, -m_use[0]));
            const float p2 = fast_exp2(fmaf(s[j][2], scale_log2, -m_use[1])), p3 = fast_exp2(fmaf(s[j][3], scale_log2, -m_use[1]));
            rs[0] += p0 + p1;
            rs[1] += p2 + p3;
            pf[j >> 1][(j & 1) * 2] = pack_bf16(p0, p1);       // rows g
            pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);   // rows g + 8
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * alpha[h] + rs[h];
#pragma unroll
        for (int j = 0; j < HD / 8; ++j) {
            o[j][0] *= alpha[0];
            o[j][1] *= alpha[0];
            o[j][2] *= alpha[1];
            o[j][3] *= alpha[1];
        }
        // ---- O += P V
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {                       // keys 16kk .. 16kk+15
#pragma unroll
            for (int dp = 0; dp < HD / 16; ++dp) {             // channel tiles 2dp, 2dp+1
                uint32_t vb[4];
                ldmatrix_x4_trans(vb, Vt + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + dp * 16 + 8 * (lane >> 4));
                mma16816(o[2 * dp], pf[kk], vb[0], vb[1]);
                mma16816(o[2 * dp + 1], pf[kk], vb[2], vb[3]);
            }
        }
        __syncthreads();                                       // the other buffer is refilled next round
    }
    cp_async_wait<0>();
    pdl_trigger();                                             // keys and values are read: the next kernel may start up

    // ---- normalise, gate, store
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = row_lo + 8 * h;
        if (row >= len) continue;
        const long long tok = s0 + row - p0;
        float f = 1.f / l_run[h];
        if (gate) f *= sigmoid_f32(__bfloat162float(gate[tok * ldg + hq]));
        bf16* dst = ctx + tok * ldc + (long long)hq * HD;
#pragma unroll
        for (int j = 0; j < HD / 8; ++j)
            *reinterpret_cast<uint32_t*>(dst + 8 * j + 2 * t) = pack_bf16(o[j][2 * h] * f, o[j][2 * h + 1] * f);
    }
}

struct FaPast {                      // where the keys and values below a sequence's first row of this step lie
    const int* seq_pos0;
    const int* seq_slot;
    const void* pool;
    long long pages;
    const int* ptab;
    int ptab_stride;
    int ring;
};

template <int HD, int BQ, bool PAST>
static int launch_fa_bq(void* ctx, long long ldc, const void* q, const void* k, const void* v, long long ld,
                        const void* gate, long long ldg, const int* seq_start, int B, int max_len, int QH, int KVH,
                        int window, float scale, const FaPast& past, cudaStream_t st) {
    const size_t smem = (size_t)(BQ + 4 * FA_BK) * (HD + 8) * sizeof(bf16);
    auto kernel = attn_prefill_mma_kernel<HD, BQ, PAST>;
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            CM_REFUSE("attn_prefill_mma: %zu bytes of shared memory refused", smem);
        }
        configured = true;
    }
    dim3 grid((max_len + BQ - 1) / BQ, QH, B);
    cm_launch(kernel, grid, BQ * 2, smem, st, (bf16*)ctx, ldc, (const bf16*)q, (const bf16*)k, (const bf16*)v, ld,
              (const bf16*)gate, ldg, seq_start, QH, KVH, window, scale * 1.4426950408889634f, past.seq_pos0,
              past.seq_slot, (const bf16*)past.pool, past.pages, past.ptab, past.ptab_stride, past.ring);
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// Query tile: 128 rows (8 warps) for long sequences, where halving the key/value copies per unit
// of work outweighs the coarser grid (measured: +6% at 16,384 tokens, -5% at 2,048); 64 rows
// (4 warps) otherwise.

template <int HD, bool PAST>
static int launch_fa(void* ctx, long long ldc, const void* q, const void* k, const void* v, long long ld,
                     const void* gate, long long ldg, const int* seq_start, int B, int max_len, int QH, int KVH,
                     int window, float scale, const FaPast& past, cudaStream_t st) {
    const int bq = max_len >= 4096 ? 128 : 64;
    if (bq == 128)
        return launch_fa_bq<HD, 128, PAST>(ctx, ldc, q, k, v, ld, gate, ldg, seq_start, B, max_len, QH, KVH, window, scale,
                                           past, st);
    return launch_fa_bq<HD, 64, PAST>(ctx, ldc, q, k, v, ld, gate, ldg, seq_start, B, max_len, QH, KVH, window, scale, past,
                                      st);
}

template <bool PAST>
static int dispatch_fa(void* ctx, long long ldc, const void* q, const void* k, const void* v, long long ld,
                       const void* gate, long long ldg, const int* seq_start, int B, int max_len, int QH, int KVH, int HD,
                       int window, float scale, const FaPast& past, cudaStream_t st) {
    if (QH % KVH) CM_REFUSE("attn_prefill_mma: %d query heads over %d key heads", QH, KVH);
    if (ld % 8 || ldc % 2 || ((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)past.pool) & 15 || (uintptr_t)ctx & 3)
        CM_REFUSE("attn_prefill_mma: row pitch %lld must be a multiple of 8 and the operands 16-byte aligned", ld);
#define FA_CASE(D) \
    case D: return launch_fa<D, PAST>(ctx, ldc, q, k, v, ld, gate, ldg, seq_start, B, max_len, QH, KVH, window, scale, past, st);
    switch (HD) {
        FA_CASE(16) FA_CASE(32) FA_CASE(48) FA_CASE(64) FA_CASE(80) FA_CASE(96) FA_CASE(112) FA_CASE(128)
        default: CM_REFUSE("attn_prefill_mma: head size %d (multiples of 16 up to 128)", HD);
    }
#undef FA_CASE
}

// bfloat16 only; head size a multiple of 16 up to 128; q, k, v column blocks of one row-major
// buffer with a row pitch that is a multiple of 8 elements and 16-byte aligned bases.
extern "C" int cm_attn_prefill_mma(void* ctx, long long ldc, const void* q, const void* k, const void* v,
                                   long long ld, const void* gate, long long ldg, const int* seq_start, int B,
                                   int max_len, int QH, int KVH, int HD, int window, float scale, cudaStream_t st) {
    if (B <= 0 || max_len <= 0) return CM_OK;
    const FaPast none = {nullptr, nullptr, nullptr, 0, nullptr, 0, 0};
    return dispatch_fa<false>(ctx, ldc, q, k, v, ld, gate, ldg, seq_start, B, max_len, QH, KVH, HD, window, scale, none, st);
}

// The same for sequences that stand at seq_pos0[b] >= 0, with the keys and values below that
// position read from this layer's paged cache (see the top of the file).
extern "C" int cm_attn_append_mma(void* ctx, long long ldc, const void* q, const void* k, const void* v,
                                  long long ld, const void* gate, long long ldg, const int* seq_start,
                                  const int* seq_pos0, const int* seq_slot, const void* pool, long long pages,
                                  const int* ptab, long long ptab_stride, int ring, int B, int max_len, int QH, int KVH,
                                  int HD, int window, float scale, cudaStream_t st) {
    if (B <= 0 || max_len <= 0) return CM_OK;
    if (ring % PAGE_TOKENS) CM_REFUSE("attn_append_mma: ring of %d entries is no multiple of %d", ring, PAGE_TOKENS);
    if (!seq_pos0 || !seq_slot || !pool || !ptab)
        CM_REFUSE("attn_append_mma: positions, slots, cache and page table are needed");
    const FaPast past = {seq_pos0, seq_slot, pool, pages, ptab, (int)ptab_stride, ring};
    return dispatch_fa<true>(ctx, ldc, q, k, v, ld, gate, ldg, seq_start, B, max_len, QH, KVH, HD, window, scale, past, st);
}

// =========================================================================================
// Decode attention over the paged cache on the tensor cores (bfloat16, head sizes that are
// multiples of 16 up to 128).  One new query token per sequence.
//
// Grid (part, kv head, sequence).  The cache entries of a sequence are cut into chunks of 256 =
// 4 pages; block `part` of n_parts walks chunks part, part + n_parts, ... and its warp w takes
// page w of each, so the entries that a sequence really holds are spread evenly over the blocks
// whatever length the grid was sized for.  The G = QH/KVH query heads that share the kv head are
// the rows of the 16-row mma operand (up to 16 per pass), so every key and value that is read
// serves all of them.  A warp keeps one page of K and one of V in its own shared-memory region
// (cp.async, rows padded by 16 bytes) and overlaps copies with arithmetic: while S = Q K^T and
// the softmax of page i run, V of page i is still arriving; K of page i+1 is requested as soon
// as S is formed, V of page i+1 as soon as O += P V is done.  Maximum, sum and O are carried
// from page to page as in the prefill kernel (float; probabilities enter the second product as
// bfloat16).  The four warps' results are merged in warp order and the block's partial result
// goes to the scratch layout that the CUDA-core kernel uses, n_parts slots per (sequence, head);
// cm_attn_decode's merge kernel finishes the job.
// =========================================================================================
#define FD_CHUNK CM_ATTN_DECODE_CHUNK
#define FD_PAGE 64

template <int HD>
__global__ void __launch_bounds__(128)
attn_decode_mma_kernel(float* __restrict__ part_o, float* __restrict__ part_ml, const bf16* __restrict__ q,
                       long long ldq, const int* __restrict__ seq_pos, const int* __restrict__ seq_slot,
                       const bf16* __restrict__ pool, long long pages, const int* __restrict__ ptab, int ptab_stride,
                       int ring, int window, int QH, int KVH, int n_parts, float scale_log2) {
    constexpr int LDS = HD + 8;
    constexpr int CH = HD / 8;
    extern __shared__ __align__(16) uint8_t fd_smem[];
    bf16* kv_s = reinterpret_cast<bf16*>(fd_smem);                       // [4 warps][K|V][64][LDS]
    float* mrg = reinterpret_cast<float*>(fd_smem);                      // [4][16][HD+2], over kv_s once it is done with
    static_assert((size_t)4 * 16 * (HD + 2) * sizeof(float) <= (size_t)4 * 2 * FD_PAGE * LDS * sizeof(bf16),
                  "the merge rows must fit the page buffers");
    pdl_wait();
    const int c = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const int G = QH / KVH;
    const int pos = seq_pos[b];
    const int n_entries = ring ? min(pos + 1, ring) : pos + 1;
    if (c * FD_CHUNK >= n_entries) return;
    const int slot = seq_slot[b];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int page_step = 4 * n_parts;                         // this warp's pages: c*4 + warp, + page_step, ...
    bf16* Ks = kv_s + (size_t)warp * 2 * FD_PAGE * LDS;
    bf16* Vs = Ks + FD_PAGE * LDS;
    const int* my_ptab = ptab + (long long)slot * ptab_stride;
    // every full page is wholly visible unless the ring is wider than the window
    const bool mask_all = window > 0 && ring != window;

    // one of a page's two halves (which: 0 keys, 1 values) into this warp's buffer
    auto request = [&](bf16* dst, int which, int page_idx) {
        const int page = my_ptab[page_idx];
        const bf16* src = pool + ((((long long)which * pages + page) * KVH + hk) * FD_PAGE) * (long long)HD;
        const int rows_here = min(FD_PAGE, n_entries - page_idx * FD_PAGE);
        for (int e = lane; e < FD_PAGE * CH; e += 32) {
            const int r = e / CH, cc = e - r * CH;
            // entries never written are zero-filled: a stale NaN times a zero probability would be NaN
            cp_async16(dst + r * LDS + cc * 8, src + (long long)r * HD + cc * 8, r < rows_here);
        }
    };

    for (int g0 = 0; g0 < G; g0 += 16) {                   // 16 query heads per pass
        const int ng = min(16, G - g0);
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
        float o[HD / 8][4];
#pragma unroll
        for (int j = 0; j < HD / 8; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[j][i] = 0.f;
        int page_idx = c * 4 + warp;
        bool live = page_idx * FD_PAGE < n_entries;
        if (live) request(Ks, 0, page_idx);
        cp_async_commit();
        if (live) request(Vs, 1, page_idx);
        cp_async_commit();
        // Q fragments: rows g and g+8 are heads g0+g and g0+g+8 of this kv head (zero beyond ng)
        uint32_t qf[HD / 16][4];
        {
            const bf16* q0 = q + (long long)b * ldq + (long long)(hk * G + g0 + g) * HD;
            const bf16* q1 = q0 + 8 * HD;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                qf[kk][0] = g < ng ? *reinterpret_cast<const uint32_t*>(q0 + kk * 16 + 2 * t) : 0u;
                qf[kk][1] = g + 8 < ng ? *reinterpret_cast<const uint32_t*>(q1 + kk * 16 + 2 * t) : 0u;
                qf[kk][2] = g < ng ? *reinterpret_cast<const uint32_t*>(q0 + kk * 16 + 8 + 2 * t) : 0u;
                qf[kk][3] = g + 8 < ng ? *reinterpret_cast<const uint32_t*>(q1 + kk * 16 + 8 + 2 * t) : 0u;
            }
        }
        while (live) {
            const int next_idx = page_idx + page_step;
            const bool next_live = next_idx * FD_PAGE < n_entries;
            cp_async_wait<1>();                                // this page's keys are here; its values may not be
            __syncwarp();
            float s[8][4];
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) s[j][i] = 0.f;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk)
#pragma unroll
                for (int jp = 0; jp < 4; ++jp) {
                    uint32_t kb[4];
                    ldmatrix_x4(kb, Ks + (jp * 16 + (lane & 7) + 8 * (lane >> 4)) * LDS + kk * 16 + 8 * ((lane >> 3) & 1));
                    mma16816(s[2 * jp], qf[kk], kb[0], kb[1]);
                    mma16816(s[2 * jp + 1], qf[kk], kb[2], kb[3]);
                }
            __syncwarp();                                      // every lane has read the keys
            if (next_live) request(Ks, 0, next_idx);
            cp_async_commit();
            // visibility of the page's entries (columns of s); raw scores, the scale goes into the exponent
            if (mask_all || (page_idx + 1) * FD_PAGE > n_entries) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int e = page_idx * FD_PAGE + 8 * j + 2 * t + (i & 1);
                        bool vis = e < n_entries;
                        if (vis) {
                            int kpos = e;
                            if (ring) {
                                int back = (pos - e) % ring;
                                if (back < 0) back += ring;
                                kpos = pos - back;
                            }
                            vis = kpos >= 0 && kpos <= pos && (window <= 0 || kpos + window > pos);
                        }
                        s[j][i] = vis ? s[j][i] : -INFINITY;
                    }
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) mx[i >> 1] = fmaxf(mx[i >> 1], s[j][i]);
            float alpha[2], m_use[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                const float m_new = fmaxf(m_run[h], mx[h] * scale_log2);
                m_use[h] = m_new == -INFINITY ? 0.f : m_new;
                alpha[h] = fast_exp2(m_run[h] - m_use[h]);
                m_run[h] = m_new;
            }
            float rs[2] = {0.f, 0.f};
            uint32_t pf[4][4];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float p0 = fast_exp2(fmaf(s[j][0], scale_log2, -m_use[0])), p1 = fast_exp2(fmaf(s[j][1], scale_log2, -m_use[0]));
                const float p2 = fast_exp2(fmaf(s[j][2], scale_log2, -m_use[1])), p3 = fast_exp2(fmaf(s[j][3], scale_log2, -m_use[1]));
                rs[0] += p0 + p1;
                rs[1] += p2 + p3;
                pf[j >> 1][(j & 1) * 2] = pack_bf16(p0, p1);
                pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * alpha[h] + rs[h];
#pragma unroll
            for (int j = 0; j < HD / 8; ++j) {
                o[j][0] *= alpha[0];
                o[j][1] *= alpha[0];
                o[j][2] *= alpha[1];
                o[j][3] *= alpha[1];
            }
            cp_async_wait<1>();                                // this page's values are here
            __syncwarp();
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
#pragma unroll
                for (int dp = 0; dp < HD / 16; ++dp) {
                    uint32_t vb[4];
                    ldmatrix_x4_trans(vb, Vs + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + dp * 16 + 8 * (lane >> 4));
                    mma16816(o[2 * dp], pf[kk], vb[0], vb[1]);
                    mma16816(o[2 * dp + 1], pf[kk], vb[2], vb[3]);
                }
            __syncwarp();                                      // every lane has read the values
            if (next_live) request(Vs, 1, next_idx);
            cp_async_commit();
            page_idx = next_idx;
            live = next_live;
        }
        cp_async_wait<0>();
        if (g0 + 16 >= G) pdl_trigger();                       // the cache is read: the next kernel may start up
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
        }
        // ---- this warp's result to shared memory: row r = head, [HD] outputs then max, sum
        __syncthreads();                                       // every warp is done with its page buffers
        float* mine = mrg + (size_t)warp * 16 * (HD + 2);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = g + 8 * h;
#pragma unroll
            for (int j = 0; j < HD / 8; ++j) {
                mine[r * (HD + 2) + 8 * j + 2 * t] = o[j][2 * h];
                mine[r * (HD + 2) + 8 * j + 2 * t + 1] = o[j][2 * h + 1];
            }
            if (t == 0) {
                mine[r * (HD + 2) + HD] = m_run[h];            // log2-scaled maximum
                mine[r * (HD + 2) + HD + 1] = l_run[h];
            }
        }
        __syncthreads();
        // ---- merge the four warps in warp order; leave the block's partial result
        for (int e = tid; e < ng * HD; e += 128) {
            const int r = e / HD, d = e - r * HD;
            float mxx = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; ++w) mxx = fmaxf(mxx, mrg[((size_t)w * 16 + r) * (HD + 2) + HD]);
            float den = 0.f, num = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float* row = mrg + ((size_t)w * 16 + r) * (HD + 2);
                const float f = row[HD] == -INFINITY ? 0.f : exp2f(row[HD] - mxx);
                den += row[HD + 1] * f;
                num += row[d] * f;
            }
            const long long idx = ((long long)b * QH + hk * G + g0 + r) * n_parts + c;
            part_o[idx * HD + d] = num;
            if (d == 0) {
                // the merge kernel works with natural-log maxima: m_ln = m_log2 * ln 2
                part_ml[idx * 2] = mxx == -INFINITY ? -INFINITY : mxx * 0.6931471805599453f;
                part_ml[idx * 2 + 1] = den;
            }
        }
        __syncthreads();                                       // the next pass copies pages over the merge rows
    }
}

// Blocks the decode grid aims at (0: chosen from the amount of work, see launch_fd).  A smaller number makes every block walk
// more chunks; tests use it to reach that path with small inputs.
static int g_fd_target_blocks = 0;
extern "C" void cm_attn_decode_set_target_blocks(int blocks) { g_fd_target_blocks = blocks > 0 ? blocks : 0; }

// n_chunks: chunks of 256 entries that cover the longest sequence.  *n_parts_out: how many blocks
// per (sequence, kv head) were launched = slots per (sequence, head) in the scratch arrays.
template <int HD>
static int launch_fd(float* part_o, float* part_ml, const void* q, long long ldq, const int* seq_pos,
                     const int* seq_slot, const void* pool, long long pages, const int* ptab, int ptab_stride,
                     int ring, int window, int B, int QH, int KVH, int n_chunks, float scale, int* n_parts_out,
                     cudaStream_t st) {
    const size_t smem = (size_t)4 * 2 * FD_PAGE * (HD + 8) * sizeof(bf16);
    auto kernel = attn_decode_mma_kernel<HD>;
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            CM_REFUSE("attn_decode_mma: %zu bytes of shared memory refused", smem);
        }
        configured = true;
    }
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count <= 0) sm_count = 1;
    }
    // A block that walks several chunks overlaps its copies with arithmetic, a block with one chunk
    // cannot; many blocks keep every SM copying.  Measured on B200 (148 SMs): 1,024 chunk-sized
    // pieces of work run fastest on about 300 blocks (one sequence of 32,768 tokens: 22 against 39
    // us), 8,192 pieces on about 1,200 (64 sequences of 3,000: 71 against 80 us).  So: a quarter
    // as many blocks as pieces, within two and eight blocks per SM.
    const long long blocks = (long long)n_chunks * KVH * B;
    long long target = blocks / 4;
    if (target < 2LL * sm_count) target = 2LL * sm_count;
    if (target > 8LL * sm_count) target = 8LL * sm_count;
    if (g_fd_target_blocks) target = g_fd_target_blocks;
    const int rounds = (int)((blocks + target - 1) / target);
    const int n_parts = (n_chunks + rounds - 1) / rounds;
    *n_parts_out = n_parts;
    cm_launch(kernel, dim3(n_parts, KVH, B), 128, smem, st, part_o, part_ml, (const bf16*)q, ldq, seq_pos, seq_slot,
              (const bf16*)pool, pages, ptab, ptab_stride, ring, window, QH, KVH, n_parts,
              scale * 1.4426950408889634f);
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// First stage of decode attention on the tensor cores; the partial results have the layout and
// meaning that cm_attn_decode's merge kernel expects.  Returns CM_ERR_SHAPE (and launches
// nothing) for head sizes it does not take.
int cm_attn_decode_mma_stage(float* part_o, float* part_ml, const void* q, long long ldq, const int* seq_pos,
                             const int* seq_slot, const void* pool, long long pages, const int* ptab,
                             int ptab_stride, int ring, int window, int B, int QH, int KVH, int HD, int n_chunks,
                             float scale, int* n_parts_out, cudaStream_t st) {
    if (ldq % 2 || ((uintptr_t)q & 3) || ((uintptr_t)pool & 15)) CM_REFUSE("attn_decode_mma: misaligned operands");
#define FD_CASE(D) \
    case D: return launch_fd<D>(part_o, part_ml, q, ldq, seq_pos, seq_slot, pool, pages, ptab, ptab_stride, ring, \
                                window, B, QH, KVH, n_chunks, scale, n_parts_out, st);
    switch (HD) {
        FD_CASE(16) FD_CASE(32) FD_CASE(48) FD_CASE(64) FD_CASE(80) FD_CASE(96) FD_CASE(112) FD_CASE(128)
        default: CM_REFUSE("attn_decode_mma: head size %d (multiples of 16 up to 128)", HD);
    }
#undef FD_CASE
}
