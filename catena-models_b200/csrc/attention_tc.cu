// Prefill attention on the 5th-generation tensor cores (bfloat16, head sizes 64 and 128): causal or
// sliding-window attention of packed sequences over their own keys and values, grouped query
// heads, optional per-head sigmoid gate.  Same result as attn_prefill_mma (attention_mma.cu).
// PAST: the sequences may stand at seq_pos0[b] > 0 (a prompt that comes in several steps); the keys
// and values below that position are read from the paged cache, page by page (a 128-key tile is two
// pages of 64 entries, each one TMA box of the cache's [k|v, page, kv head, entry, head] layout),
// before the step's own tiles.  A tile's second page that lies wholly at or above seq_pos0 is not
// the sequence's and may not be allocated: the first page is copied in its place.
// Rows of a key/value tile that are not the sequence's (beyond its end: the next sequence's rows of
// the step, padding, unwritten entries of a page) get scores of -inf by selection, so whatever the
// keys hold does not matter, and their rows of the value tile are cleared in shared memory before the
// product over them is issued, because a probability of exactly zero times NaN would not be zero.
//
// Work items are (128-query tile, query head, sequence), long rows first; one block per SM walks its share
// of them, to and fro over the blocks so that the shares come out even, and keeps its rings, its tensor-memory
// buffers and all mbarrier phases running across an item's border: the copies and first scores of the next
// item are under way while this one's rows are stored.  Twelve warps (the first group of four gives most of
// its registers to the other two, setmaxnreg 40 / 232): threads that copy with TMA (Q tiles, 128-key K and V
// tiles into shared-memory rings; 128-byte rows, 128-byte swizzle; a head of 128 is two 64-column pieces),
// threads that issue products and commit them to mbarriers (S = Q K^T, 128 x 128, K-major operands from
// shared memory; O += P V, 128 x HD, P from tensor memory, V from shared memory as the MN-major B operand:
// its rows are keys), and two softmax groups of 128 threads, one query row a thread: a thread reads its
// row's 128 scores from tensor memory into registers once, takes their maximum, and writes the exponentials
// as bfloat16 back into tensor memory, where the product reads them.
// O is never read between tiles: the exponentials are taken relative to a reference that follows the row's
// maximum only when that has grown by more than a factor of 256 since the reference was set; then the group
// waits for its products so far, scales its O in tensor memory and goes on.  Maxima settle after the first
// tiles of a row, so this is rare (and it changes no result beyond rounding: the sums are float, and a
// bfloat16 probability of up to 256 is as exact as one below 1).
// Two forms.  In this file, for heads of 128: the two groups share an item and take its key tiles in turns
// (group g the tiles g, g + 2, ...), each with its own (reference, sum) and its own O, merged at the item's
// end; P lies over the scores it came from, and one thread issues, for a tile, the product and then the
// scores of the tile that takes the buffer over, which also keeps the groups half a tile apart.  In
// attention_tc_solo.cuh, for heads of 64, where tensor memory has room for it: each group has items of its
// own, with its own copying and issuing thread, rings, and S, P and O columns.
// What bounds a tile's time is the softmax (128 exponentials a thread and tile on the SM's 16
// special-function lanes, which the two groups share) and what stands between one tile's P and the next
// tile's scores; every look at an mbarrier and every commit costs the thread that makes it a hundred cycles
// and more, so they are kept off that path (asked early, read late).
//
// Maximum, sum, exponent arguments and the rescaling are float; probabilities enter the second
// product as bfloat16.  Every wait on an mbarrier is bounded; a wait that runs out raises *err, all
// roles leave their loops, copies in flight are awaited (bounded), tensor memory is freed.
#include "tc_common.cuh"

#define FT_TILE 128
static_assert(PAGE_TOKENS * 2 == FT_TILE, "a key tile of the cache is two pages");
#define FT_THREADS 384                     // three groups of four warps: loader and issuer, softmax 0, softmax 1
#define FT_PIECE_BYTES (128 * 64 * 2)      // 128 rows of 128 bytes
#define FT_STAGES_64 3                     // K and V tiles in flight with heads of 64 (16 KB each), per pipeline ...
#define FT_STAGES_128 2                    // ... and of 128 (32 KB each)
#define FT_ERR_LOAD 111
#define FT_ERR_MMA 112
#define FT_ERR_SOFTMAX 113

__device__ __forceinline__ float ft_max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// mbar_wait with its loop not unrolled: these kernels wait in dozens of places, nearly always with success at the
// first look, and every unrolled copy of the loop is so much less instruction cache for the code that does the
// work (the kernels' code shrank by an eighth, and they ran a fifth faster).
__device__ __forceinline__ bool ft_mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort, int* err, int code) {
#pragma unroll 1
    for (int i = 0; i < TC_SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255) == 255 && *abort) return false;
    }
    *abort = 1;
    if (err) atomicCAS(err, 0, code);
    return false;
}
// Has the phase completed?  Does not block; the answer can be asked for early and read late.
__device__ __forceinline__ uint32_t ft_mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
// Two floats in one 64-bit register and arithmetic on both at once (fma and add as for single floats, round to
// nearest): half the instructions for the softmax's multiply-adds and sums.
__device__ __forceinline__ uint64_t ft_pack2(float a, float b) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(a), "f"(b));
    return d;
}
__device__ __forceinline__ void ft_unpack2(uint64_t d, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(d));
}
__device__ __forceinline__ uint64_t ft_fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t ft_add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float ft_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 32 columns of this warp's 32 lanes of tensor memory written from registers (the reverse of tmem_load32_issue)
__device__ __forceinline__ void tmem_store32_issue(uint32_t taddr, const float* v) {
    const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
// 16 columns (32 bfloat16 of a row, two to a column) of this warp's 32 lanes
__device__ __forceinline__ void tmem_store16_issue(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
// D (tensor memory) (+)= A (tensor memory: a row per lane, two bfloat16 of K per column) x B (shared memory)
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Descriptor of an MN-major operand tile with 128-byte rows and 128-byte swizzle: 64 contiguous
// elements along N, groups of 8 rows along K 1024 bytes apart, further 64-element blocks along N
// `lbo_bytes` apart.
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t smem_addr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

struct FtPast {                      // where the keys and values below a sequence's first row of this step lie
    const int* seq_pos0;
    const int* seq_slot;
    const int* ptab;
    long long ptab_stride;
    long long pages;
    int ring;
};

// One work item: a 128-query tile of one query head of one sequence, and the key tiles it takes.
struct FtItem {
    int b, hq, hk, s0, len, q0, p0, kt_begin, tp_begin, n_past, n;
};
// Item w of the launch, long rows first (the query tile falls as w rises).  n = 0: nothing to do (the
// sequence is shorter than this tile's first row).
template <bool PAST>
__device__ __forceinline__ void ft_item(int w, int tiles_x, int QH, int KVH, int B, int window,
                                        const int* __restrict__ seq_start, const FtPast& past, FtItem& it) {
    const int per_x = QH * B, x = w / per_x, rest = w - x * per_x;
    it.b = rest / QH;
    it.hq = rest - it.b * QH;
    it.hk = it.hq / (QH / KVH);
    it.s0 = seq_start[it.b];
    it.len = seq_start[it.b + 1] - it.s0;
    it.q0 = (tiles_x - 1 - x) * FT_TILE;
    it.n = 0;
    it.p0 = 0;
    it.kt_begin = it.tp_begin = it.n_past = 0;
    if (it.q0 >= it.len) return;
    it.kt_begin = window > 0 ? max(0, it.q0 - window + 1) / FT_TILE : 0;
    const int kt_end = min(it.q0 + FT_TILE - 1, it.len - 1) / FT_TILE;   // inclusive
    // positions: row r of this step stands at p0 + r; tiles of the cache come first, in steps of 128 positions
    it.p0 = PAST ? past.seq_pos0[it.b] : 0;
    if (PAST && it.p0 > 0) {
        const int a_lo = window > 0 ? max(0, it.p0 + it.q0 - window + 1) : 0;
        if (a_lo < it.p0) {
            it.tp_begin = a_lo / FT_TILE;
            it.n_past = (it.p0 - 1) / FT_TILE - it.tp_begin + 1;
        }
    }
    it.n = it.n_past + kt_end - it.kt_begin + 1;
}
// The item that block `bx` of `G` takes in its round `r`: rounds run to and fro over the blocks, so that the
// block with the longest item of one round has the shortest of the next (items are sorted by length).  -1: none.
__device__ __forceinline__ int ft_item_of_round(int r, int bx, int G, int total) {
    const int w = r * G + ((r & 1) ? G - 1 - bx : bx);
    return w < total ? w : -1;
}
// The number of key tiles alone, for the roles that need no more.
template <bool PAST>
__device__ __forceinline__ int ft_item_tiles(int w, int tiles_x, int QH, int KVH, int B, int window,
                                             const int* __restrict__ seq_start, const FtPast& past) {
    FtItem it;
    ft_item<PAST>(w, tiles_x, QH, KVH, B, window, seq_start, past, it);
    return it.n;
}

template <int HD, int STAGES, bool PAST>
__global__ void __launch_bounds__(FT_THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_pool,
                       const FtPast past, bf16* __restrict__ ctx, long long ldc,
                       const bf16* __restrict__ gate, long long ldg, const int* __restrict__ seq_start, int QH,
                       int KVH, int B, int tiles_x, int window, float scale_log2, int* err) {
    constexpr int KB = HD / 64;                                   // 64-column pieces of a head
    constexpr uint32_t Q_BYTES = KB * FT_PIECE_BYTES, KV_BYTES = KB * FT_PIECE_BYTES;
    constexpr int NP = 2;                                         // mbarriers per group for P and for O, in turns
    // tensor memory: a score buffer of 128 columns per softmax group (tile J's is buffer J % NS), then an O
    // buffer of HD columns per group: 512 columns with a head of 128
    constexpr int NS = 2;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr int NBARS = 4 + 4 * STAGES + NS + 4 * NP + 2;
    // a stage of K or V is waited for by one issuing thread and one group only: a wait that skips a phase
    // of an mbarrier reads the wrong one
    static_assert(STAGES % 2 == 0, "tiles of one stage belong to one softmax group");
    static_assert(NS * FT_TILE + 2 * HD <= 512, "tensor memory holds the S and O buffers");
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bars[NBARS];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ int issued_q, issued_k, issued_v;
    __shared__ float2 group_ml[2][2][FT_TILE];                    // [item parity][group][row]: (reference maximum, sum), for an item's end

    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total = tiles_x * QH * B, G = gridDim.x;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_s = base, k_s = q_s + 2 * Q_BYTES, v_s = k_s + STAGES * KV_BYTES;
    const uint32_t bar0 = smem_u32(&bars[0]);
    const uint32_t q_full = bar0, q_empty = q_full + 16;
    const uint32_t k_full = q_empty + 16, k_empty = k_full + 8 * STAGES, v_full = k_empty + 8 * STAGES,
                   v_empty = v_full + 8 * STAGES;
    const uint32_t s_full = v_empty + 8 * STAGES, p_full = s_full + 8 * NS, o_full = p_full + 16 * NP,
                   merge_ready = o_full + 16 * NP, o_free = merge_ready + 8;

    if (warp == 0) {
        // one lane per mbarrier.  Arrivals: p_full, merge_ready and o_free one per warp of a group (four, eight,
        // eight); all others one.
        for (int i = lane; i < NBARS; i += 32) {
            const int first_p = 4 + 4 * STAGES + NS;
            int count = 1;
            if (i >= first_p && i < first_p + 2 * NP) count = 4;
            if (i >= NBARS - 2) count = 8;
            mbar_init(bar0 + 8 * i, count);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (lane == 0) {
            abort_flag = 0;
            issued_q = 0;
            issued_k = 0;
            issued_v = 0;
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    // Every role walks the same items (ft_item_of_round), skipping those without key tiles, and
    // counts items (i) and key tiles (J) from the block's start: rings, score buffers, the two softmax groups
    // (tile J is group J & 1's) and all mbarrier phases go by these counts, so that nothing starts over at an
    // item's border and the copies and scores of the next item are under way while this one's rows are stored.
    // 384 threads x 168 registers fill the register file; the first four warps keep 40 each and the
    // eight softmax warps take 232 (4 x 32 x 40 + 8 x 32 x 232 = 64,512 of 65,536)
    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if ((warp == 0 || warp == 3) && lane == 0) {
            // ------------------------------------------------------------- TMA loaders: warp 0 for Q and K, warp 3 for V,
            // so that a V tile that waits for its place in the ring holds no K tile back
            const bool values = warp == 3;
            bool ok = true;
            int J = 0, i = 0;
            FtItem it = {};
            // the two pages of the cache that hold positions 128 tp .. 128 tp + 127, keys (which = 0) or values
            auto load_pages = [&](uint32_t dst, uint32_t bar, int tp, int which) {
                const int* row = past.ptab + (long long)past.seq_slot[it.b] * past.ptab_stride;
                for (int h = 0; h < 2; ++h) {
                    int a0 = tp * FT_TILE + h * 64;
                    if (a0 >= it.p0) a0 = tp * FT_TILE;               // not this sequence's entries: the first page again
                    const int entry = past.ring > 0 ? a0 % past.ring : a0;
                    const long long page = row[entry >> 6];
                    const long long r0 = ((which * past.pages + page) * KVH + it.hk) * 64;
                    for (int kb = 0; kb < KB; ++kb)
                        tma_load_2d(dst + kb * FT_PIECE_BYTES + h * 8192, &map_pool, bar, kb * 64, (int)r0);
                }
            };
            auto load_tile = [&](int j, uint32_t ring_s, uint32_t full, uint32_t empty, const CUtensorMap* map, int which) {
                const int s = J % STAGES;
                ok = ft_mbar_wait(empty + 8 * s, ((J / STAGES) & 1) ^ 1, &abort_flag, err, FT_ERR_LOAD);
                if (!ok) return;
                mbar_expect_tx(full + 8 * s, KV_BYTES);
                if (PAST && j < it.n_past) {
                    load_pages(ring_s + s * KV_BYTES, full + 8 * s, it.tp_begin + j, which);
                } else {
                    for (int kb = 0; kb < KB; ++kb)
                        tma_load_2d(ring_s + s * KV_BYTES + kb * FT_PIECE_BYTES, map, full + 8 * s, it.hk * HD + kb * 64,
                                    it.s0 + (it.kt_begin + j - it.n_past) * FT_TILE);
                }
            };
            for (int rnd = 0; rnd * G < total && ok; ++rnd) {
                const int w = ft_item_of_round(rnd, blockIdx.x, G, total);
                if (w < 0) continue;
                ft_item<PAST>(w, tiles_x, QH, KVH, B, window, seq_start, past, it);
                if (it.n == 0) continue;
                if (!values) {
                    ok = ft_mbar_wait(q_empty + 8 * (i & 1), ((i >> 1) & 1) ^ 1, &abort_flag, err, FT_ERR_LOAD);
                    if (!ok) break;
                    mbar_expect_tx(q_full + 8 * (i & 1), Q_BYTES);
                    for (int kb = 0; kb < KB; ++kb)
                        tma_load_2d(q_s + (i & 1) * Q_BYTES + kb * FT_PIECE_BYTES, &map_q, q_full + 8 * (i & 1), it.hq * HD + kb * 64,
                                    it.s0 + it.q0);
                    issued_q = ++i;
                }
                for (int j = 0; j < it.n && ok; ++j) {
                    if (values) {
                        load_tile(j, v_s, v_full, v_empty, &map_v, 1);
                        if (ok) issued_v = J + 1;
                    } else {
                        load_tile(j, k_s, k_full, k_empty, &map_k, 0);
                        if (ok) issued_k = J + 1;
                    }
                    ++J;
                }
            }
            pdl_trigger();                            // every tile is requested: the next kernel may start up
        } else if (warp == 1 && lane == 0) {
            // ------------------------------------------------------------- issuer of products
            // For a tile J: O (+)= P V of tile J, then S = Q K^T of tile J + NS, whose scores go where P of tile J
            // lies: both from one thread, so the tensor core takes them in that order; and the one thread's order,
            // group after group, keeps the two groups half a tile apart, not both at their exponentials at once.
            // S: float accumulator, bf16 operands, both K-major, N = 128.  O: A (P) from tensor memory, B (V)
            // MN-major (its rows are keys), N = HD.
            constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(FT_TILE >> 3) << 17) |
                                         ((uint32_t)(FT_TILE >> 4) << 24);
            constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) |
                                         ((uint32_t)(FT_TILE >> 4) << 24);
            bool ok = true;
            // Two walks over the tiles: the one whose scores are issued (sw, sn, sj, si: item, its tiles, the tile,
            // the count of items; global tile J + NS) runs NS tiles ahead of the one whose product is (pw, ...; J).
            int sr = -1, sn = 0, sj = 0, si = -1;                   // round, the item's tiles, the tile, the count of items
            int pr = -1, pn = 0, pj = 0, pi = -1;
            bool s_valid = true;
            int T0 = 0, T1 = 0;                                     // products issued per group
            // moves the score walk to the next tile; at an item's border the item just left gives its Q buffer
            // back and the next one's Q is awaited
            auto advance_s = [&]() {
                if (++sj < sn) return;
                if (si >= 0) umma_commit(q_empty + 8 * (si & 1));    // this thread's scores of the item are all issued
                do {
                    ++sr;
                    if (sr * G >= total) { s_valid = false; return; }
                    const int w = ft_item_of_round(sr, blockIdx.x, G, total);
                    sn = w < 0 ? 0 : ft_item_tiles<PAST>(w, tiles_x, QH, KVH, B, window, seq_start, past);
                } while (sn == 0);
                sj = 0;
                ++si;
                ok = ft_mbar_wait(q_full + 8 * (si & 1), (si >> 1) & 1, &abort_flag, err, FT_ERR_MMA);
            };
            auto products_s = [&](int Js) {
                const int s = Js % STAGES;
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint64_t a = umma_desc(q_s + (si & 1) * Q_BYTES + (k >> 2) * FT_PIECE_BYTES) + 2 * (k & 3);
                    const uint64_t bd = umma_desc(k_s + s * KV_BYTES + (k >> 2) * FT_PIECE_BYTES) + 2 * (k & 3);
                    umma_bf16(tmem_base + (uint32_t)((Js % NS) * FT_TILE), a, bd, idesc_s, k != 0);
                }
                umma_commit(s_full + 8 * (Js % NS));
                umma_commit(k_empty + 8 * s);
            };
            sj = -1;                                                // so that the first advance enters the first item
            sn = 0;
            advance_s();
            // the first NS tiles' scores wait for no product
            int Js = 0;
            for (; Js < NS && s_valid && ok; ++Js) {
                ok = ft_mbar_wait(k_full + 8 * (Js % STAGES), (Js / STAGES) & 1, &abort_flag, err, FT_ERR_MMA);
                if (!ok) break;
                tc_fence_after();
                products_s(Js);
                advance_s();
            }
            // Js = J + NS from here on, as long as there are tiles left to score
            int J = 0;
            while (ok) {
                // the product walk's next tile
                if (++pj >= pn) {
                    do {
                        ++pr;
                        if (pr * G >= total) break;
                        const int w = ft_item_of_round(pr, blockIdx.x, G, total);
                        pn = w < 0 ? 0 : ft_item_tiles<PAST>(w, tiles_x, QH, KVH, B, window, seq_start, past);
                    } while (pn == 0);
                    if (pr * G >= total) break;
                    pj = 0;
                    ++pi;
                    // the O buffers hold the item before until both groups have read them
                    if (pi >= 1) ok = ft_mbar_wait(o_free, (pi - 1) & 1, &abort_flag, err, FT_ERR_MMA);
                    if (!ok) break;
                }
                {
                    const int g = J & 1, s = J % STAGES, Tg = g ? T1 : T0, pb = g * NP + Tg % NP;
                    // V and the next K first: they have long been loaded, and P is what this thread really waits
                    // for; what follows P's arrival is on the path of the group that will read the next scores.
                    ok = ft_mbar_wait(v_full + 8 * s, (J / STAGES) & 1, &abort_flag, err, FT_ERR_MMA);
                    if (ok && s_valid) ok = ft_mbar_wait(k_full + 8 * (Js % STAGES), (Js / STAGES) & 1, &abort_flag, err, FT_ERR_MMA);
                    if (ok) ok = ft_mbar_wait(p_full + 8 * pb, (Tg / NP) & 1, &abort_flag, err, FT_ERR_MMA);
                    // The group's O is in order as well: when the group rescales it, it does so before it
                    // announces the P of the tile (p_full), with every earlier product finished.
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int k = 0; k < FT_TILE / 16; ++k) {            // 16 keys per instruction
                        // P lies where the tile's scores lay: 16 keys are 8 columns.  The item's first product of a group starts O anew.
                        const uint64_t bd = umma_desc_mn(v_s + s * KV_BYTES + k * 2048, FT_PIECE_BYTES);
                        umma_bf16_ts(tmem_base + (uint32_t)(NS * FT_TILE + g * HD), tmem_base + (uint32_t)((J % NS) * FT_TILE + 8 * k), bd,
                                     idesc_o, k != 0 || pj >= 2);
                    }
                    if (s_valid) products_s(Js);
                    umma_commit(o_full + 8 * pb);                        // also behind the scores just issued: nobody waits long for it
                    umma_commit(v_empty + 8 * s);
                    if (g) ++T1; else ++T0;
                }
                ++J;
                if (s_valid) {
                    ++Js;
                    advance_s();
                }
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
        // ------------------------------------------------------------- softmax groups
        const int g = (warp - 4) >> 2, quarter = warp & 3;
        const int r = quarter * 32 + lane;                        // the row of the tile this thread owns
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const uint32_t t_o = lane_base + (uint32_t)(NS * FT_TILE + g * HD);
        const uint32_t full = 0xffffffffu;
        // The group's O stays in tensor memory: every product of the group adds to it.  The exponentials are
        // taken relative to m_ref, which follows the row's running maximum only when that has grown by more
        // than RESCALE (a factor of 256 in the probabilities; bfloat16 and the float sums have the range for
        // it): then, and only then, O is read, scaled and written back, after the group's products so far are
        // done.  With maxima that settle after the first tiles a tile costs no round trip through O at all.
        constexpr float RESCALE = 8.f;
        bool ok = true;
        int J = 0, i = 0;                                         // key tiles and items so far (both groups' tiles count)
        int T = 0, products_done = 0;                             // this group's products so far; products 0 .. products_done - 1 are finished
        auto await_products = [&](int upto) {
            if (products_done >= upto) return;                    // warp-uniform: every lane counts alike
            while (ok && products_done < upto) {
                ok = ft_mbar_wait(o_full + 8 * (g * NP + products_done % NP), (products_done / NP) & 1, &abort_flag, err,
                               FT_ERR_SOFTMAX);
                ++products_done;
            }
            ok = __all_sync(full, ok);                            // what follows is warp-wide
        };
        for (int rnd = 0; rnd * G < total && ok; ++rnd) {
            const int w = ft_item_of_round(rnd, blockIdx.x, G, total);
            if (w < 0) continue;
            FtItem it;
            ft_item<PAST>(w, tiles_x, QH, KVH, B, window, seq_start, past, it);
            if (it.n == 0) continue;
            const int row_l = it.q0 + r;                          // this thread's row among the sequence's rows of this step
            const int row = it.p0 + row_l;                        // its position in the sequence
            const int J0 = J;
            float m_ref = -INFINITY, l_run = 0.f;
            int t = 0;                                            // this group's tiles of the item so far
            for (int j = 0; j < it.n && ok; ++j, ++J) {
                if ((J & 1) != g) continue;
                // first position of the tile, and the position where its sequence's entries end
                const bool from_cache = PAST && j < it.n_past;
                const int k0 = from_cache ? (it.tp_begin + j) * FT_TILE : it.p0 + (it.kt_begin + j - it.n_past) * FT_TILE;
                const int limit = from_cache ? it.p0 : it.p0 + it.len;
                ok = __all_sync(full, ft_mbar_wait(s_full + 8 * (J % NS), (J / NS) & 1, &abort_flag, err, FT_ERR_SOFTMAX));
                if (!ok) break;
                tc_fence_after();
                const uint32_t t_s = lane_base + (uint32_t)((J % NS) * FT_TILE);
                float v[FT_TILE];                                     // the row's 128 scores, read once
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_load32_issue(t_s + (uint32_t)(32 * c), v + 32 * c);
                // Asked now, read after the maxima: has the product of two tiles ago finished?  (It has, long ago; the
                // question keeps this group within one phase of its O barriers, and a look at an mbarrier costs about
                // a hundred cycles when it stands in the way.)
                uint32_t early = 1;
                if (T >= 2 && products_done == T - 2)
                    early = ft_mbar_test(o_full + 8 * (g * NP + (T - 2) % NP), (uint32_t)(((T - 2) / NP) & 1));
                tmem_load_wait();
                // the keys of the tile that this row sees are the columns lo .. hi - 1; all of them: no comparisons needed
                const int lo = window > 0 ? max(0, row - window + 1 - k0) : 0;
                const int hi = min(FT_TILE, min(row, limit - 1) - k0 + 1);
                if (lo > 0 || hi < FT_TILE) {
                    const unsigned span = (unsigned)max(hi - lo, 0);
#pragma unroll
                    for (int c = 0; c < FT_TILE; ++c) v[c] = (unsigned)(c - lo) < span ? v[c] : -INFINITY;
                }
                // four partial maxima and four partial sums: chains of 128 dependent operations would leave the
                // thread waiting on arithmetic latency
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int c = 0; c < FT_TILE; c += 2) mx4[(c >> 1) & 3] = ft_max3(mx4[(c >> 1) & 3], v[c], v[c + 1]);
                const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
                const float m_cand = fmaxf(m_ref, mx * scale_log2);   // scale > 0 keeps the order of the scores
                // A row that has seen no key yet has O = 0 and l = 0 whatever m_ref is: it takes the maximum as it is.
                if (m_ref == -INFINITY) m_ref = m_cand;
                const bool grown = m_cand - m_ref > RESCALE;
                if (t > 0 && __any_sync(full, grown)) {
                    // The warp owns its 32 lanes of tensor memory, so the warp decides; rows that have not grown
                    // much move to their own maximum as well (a factor below one).
                    await_products(T);
                    if (!ok) break;
                    const float alpha = ft_exp2(m_ref - (m_cand == -INFINITY ? 0.f : m_cand));
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < HD / 32; ++c) {
                        float o[32];
                        tmem_load32_issue(t_o + (uint32_t)(32 * c), o);
                        tmem_load_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e) o[e] *= alpha;
                        tmem_store32_issue(t_o + (uint32_t)(32 * c), o);
                    }
                    tmem_store_wait();
                    l_run *= alpha;
                    m_ref = m_cand;
                }
                const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
                // Keeps this group within one phase of its O barriers (a wait that lags two phases behind an
                // mbarrier never returns); the product of two tiles ago is long done.
                if (T >= 2 && products_done == T - 2 && __all_sync(full, early)) products_done = T - 1;
                await_products(T - 1);
                if (!ok) break;
                // two partial sums of pairs: a chain of 64 dependent additions would leave the thread waiting on their latency
                const uint64_t scale2 = ft_pack2(scale_log2, scale_log2), minus_m2 = ft_pack2(-m_use, -m_use);
                uint64_t rs2[2] = {ft_pack2(0.f, 0.f), ft_pack2(0.f, 0.f)};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t pk[16];
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        float x0, x1;
                        ft_unpack2(ft_fma2(ft_pack2(v[32 * c + 2 * e], v[32 * c + 2 * e + 1]), scale2, minus_m2), x0, x1);
                        const float e0 = ft_exp2(x0), e1 = ft_exp2(x1);
                        rs2[e & 1] = ft_add2(rs2[e & 1], ft_pack2(e0, e1));
                        __nv_bfloat162 h = __floats2bfloat162_rn(e0, e1);
                        pk[e] = *reinterpret_cast<uint32_t*>(&h);
                    }
                    // over the scores, which are in registers: 32 probabilities of the row are 16 columns
                    tmem_store16_issue(t_s + (uint32_t)(16 * c), pk);
                }
                tmem_store_wait();
                float rs_a, rs_b;
                ft_unpack2(ft_add2(rs2[0], rs2[1]), rs_a, rs_b);
                const float rs = rs_a + rs_b;
                if (k0 + FT_TILE > limit) {
                    // The tile holds rows that are not this sequence's entries (the next sequence's rows of the step,
                    // padding, unwritten entries of a page).  Their probabilities are exactly zero, but zero times a
                    // value that is not finite is not zero: thread r clears row r of the value tile before the
                    // product over it may be issued (that waits for p_full below).
                    const int s = J % STAGES;
                    ok = __all_sync(full, ft_mbar_wait(v_full + 8 * s, (J / STAGES) & 1, &abort_flag, err, FT_ERR_SOFTMAX));
                    if (!ok) break;
                    if (k0 + r >= limit) {
#pragma unroll
                        for (int kb = 0; kb < KB; ++kb)
#pragma unroll
                            for (int c = 0; c < 8; ++c)
                                st_shared16(v_s + s * KV_BYTES + kb * FT_PIECE_BYTES + r * 128 + c * 16, 0u, 0u, 0u, 0u);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the cleared rows, for the tensor core
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full + 8 * (g * NP + T % NP));   // P is in tensor memory and O is in order
                l_run += rs;
                ++T;
                ++t;
            }
            if (!ok) break;
            // ---- the item's end.  Each group leaves its rows' (reference maximum, sum) in shared memory; then every
            // thread reads half of the row's O columns of BOTH groups from tensor memory (a warp reaches its 32
            // lanes in every column), merges, normalises, gates and stores them: group 0 the lower half of the
            // head, group 1 the upper.  Once both groups have read, the O buffers are the next item's.
            await_products(T);                                    // the group's last product is done
            if (!ok) break;
            group_ml[i & 1][g][r] = make_float2(m_ref, l_run);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(merge_ready);
            ok = __all_sync(full, ft_mbar_wait(merge_ready, i & 1, &abort_flag, err, FT_ERR_SOFTMAX));
            if (!ok) break;
            tc_fence_after();
            constexpr int HALF = HD / 2;
            // the other group's tiles of this item: those of the other parity among J0 .. J0 + n - 1
            const bool other_has_tiles = (it.n + (((J0 & 1) == (g ^ 1)) ? 1 : 0)) / 2 > 0;
            float mine[HALF], theirs[HALF];
#pragma unroll
            for (int c = 0; c < HALF; ++c) mine[c] = theirs[c] = 0.f;
            if (t > 0) {
#pragma unroll
                for (int c = 0; c < HALF / 32; ++c) tmem_load32_issue(t_o + (uint32_t)(g * HALF + 32 * c), mine + 32 * c);
            }
            if (other_has_tiles) {
                const uint32_t t_other = lane_base + (uint32_t)(NS * FT_TILE + (g ^ 1) * HD);
#pragma unroll
                for (int c = 0; c < HALF / 32; ++c) tmem_load32_issue(t_other + (uint32_t)(g * HALF + 32 * c), theirs + 32 * c);
            }
            tmem_load_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(o_free);
            if (row_l < it.len) {
                const float2 other = group_ml[i & 1][g ^ 1][r];
                const float m = fmaxf(m_ref, other.x);
                const float f_mine = m_ref == -INFINITY ? 0.f : ft_exp2(m_ref - m);
                const float f_theirs = other.x == -INFINITY ? 0.f : ft_exp2(other.x - m);
                float f = 1.f / (l_run * f_mine + other.y * f_theirs);
                const long long tok = it.s0 + row_l;
                if (gate) f *= sigmoid_f32(__bfloat162float(gate[tok * ldg + it.hq]));
                bf16* dst = ctx + tok * ldc + (long long)it.hq * HD + g * HALF;
#pragma unroll
                for (int c = 0; c < HALF / 8; ++c) {
                    uint4 raw;
                    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int d = 8 * c + 2 * e;
                        h[e] = __floats2bfloat162_rn((mine[d] * f_mine + theirs[d] * f_theirs) * f,
                                                     (mine[d + 1] * f_mine + theirs[d + 1] * f_theirs) * f);
                    }
                    *reinterpret_cast<uint4*>(dst + 8 * c) = raw;
                }
            }
            ++i;
        }
    }
    // ------------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (abort_flag && threadIdx.x == 0) {
        // copies that were issued but never consumed must land before shared memory is given up
        for (int q = max(0, issued_q - 2); q < issued_q; ++q)
            for (int c = 0; c < TC_SPIN_LIMIT; ++c)
                if (mbar_try_wait(q_full + 8 * (q & 1), (q >> 1) & 1)) break;
        for (int j = max(0, issued_k - STAGES); j < issued_k; ++j)
            for (int c = 0; c < TC_SPIN_LIMIT; ++c)
                if (mbar_try_wait(k_full + 8 * (j % STAGES), (j / STAGES) & 1)) break;
        for (int j = max(0, issued_v - STAGES); j < issued_v; ++j)
            for (int c = 0; c < TC_SPIN_LIMIT; ++c)
                if (mbar_try_wait(v_full + 8 * (j % STAGES), (j / STAGES) & 1)) break;
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

#include "attention_tc_solo.cuh"

template <int HD, int STAGES, bool PAST>
static auto ft_kernel() {
    if constexpr (HD == 64)
        return attn_prefill_tc_solo_kernel<HD, STAGES, PAST>;
    else
        return attn_prefill_tc_kernel<HD, STAGES, PAST>;
}

template <int HD, int STAGES, bool PAST>
static int launch_ft(void* ctx, long long ldc, const void* q, const void* k, const void* v, long long ld,
                     const void* gate, long long ldg, const int* seq_start, int B, int max_len, long long T, int QH,
                     int KVH, int window, float scale, const FtPast& past, const void* pool, int* err, cudaStream_t st) {
    CUtensorMap map_q, map_k, map_v, map_pool;
    int rc = make_map(&map_q, q, T, (long long)QH * HD, ld, FT_TILE);
    if (rc == CM_OK) rc = make_map(&map_k, k, T, (long long)KVH * HD, ld, FT_TILE);
    if (rc == CM_OK) rc = make_map(&map_v, v, T, (long long)KVH * HD, ld, FT_TILE);
    // the cache as rows of one head: [k|v, page, kv head, entry] x head size; a box is one page of one head
    if (PAST) {
        if (rc == CM_OK) rc = make_map(&map_pool, pool, 2 * past.pages * KVH * PAGE_TOKENS, HD, HD, PAGE_TOKENS);
    } else {
        map_pool = map_k;
    }
    if (rc != CM_OK) return rc;
    constexpr int KB = HD / 64;
    // Heads of 64: two pipelines a block, each with its own query tile, Q and rings (STAGES is a pipeline's).
    // Heads of 128: one query tile a block at a time, its key tiles dealt to the two groups (two Q tiles, shared rings).
    constexpr bool SOLO = HD == 64;
    const size_t smem = SOLO ? (size_t)2 * KB * FT_PIECE_BYTES * (1 + 2 * STAGES) + 1024
                             : (size_t)KB * FT_PIECE_BYTES * (2 + 2 * STAGES) + 1024;
    auto kernel = ft_kernel<HD, STAGES, PAST>();
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            CM_REFUSE("attn_prefill_tc: %zu bytes of shared memory refused", smem);
        }
        configured = true;
    }
    // one block per SM walks the items (query tile, head, sequence), long rows first
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count <= 0) sm_count = 1;
    }
    const int tiles_x = (max_len + FT_TILE - 1) / FT_TILE;
    const long long items = (long long)tiles_x * QH * B;
    if (items > 0x7fffffffLL) CM_REFUSE("attn_prefill_tc: %lld items", items);
    const long long blocks = SOLO ? (items + 1) / 2 : items;
    dim3 grid((unsigned)(blocks < sm_count ? blocks : sm_count));
    cm_launch(kernel, grid, FT_THREADS, smem, st, map_q, map_k, map_v, map_pool, past, (bf16*)ctx, ldc, (const bf16*)gate,
              ldg, seq_start, QH, KVH, B, tiles_x, window, scale * 1.4426950408889634f, err);
    {
        cudaError_t e_ = cudaGetLastError();
        if (e_ != cudaSuccess) {
            cudaFuncAttributes fa;
            cudaFuncGetAttributes(&fa, kernel);
            cm_set_error("attn_prefill_tc launch failed: %s (registers %d, static smem %zu, dynamic %zu, max threads %d)",
                         cudaGetErrorString(e_), fa.numRegs, fa.sharedSizeBytes, smem, fa.maxThreadsPerBlock);
            return CM_ERR_LAUNCH;
        }
    }
    return CM_OK;
}

// bfloat16; head size 64 or 128; q, k, v are column blocks of one row-major buffer of T rows with
// a row pitch that is a multiple of 8 elements, every base 16-byte aligned, and so is the output's
// base and pitch.  err: device int that a block raises when one of its bounded waits runs out.
extern "C" int cm_attn_prefill_tc(void* ctx, long long ldc, const void* q, const void* k, const void* v, long long ld,
                                  const void* gate, long long ldg, const int* seq_start, int B, int max_len,
                                  long long T, int QH, int KVH, int HD, int window, float scale, int* err,
                                  cudaStream_t st) {
    if (B <= 0 || max_len <= 0) return CM_OK;
    if (QH % KVH) CM_REFUSE("attn_prefill_tc: %d query heads over %d key heads", QH, KVH);
    if (ld % 8 || ldc % 8 || (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)ctx) & 15))
        CM_REFUSE("attn_prefill_tc: row pitches %lld, %lld must be multiples of 8 and the operands 16-byte aligned", ld, ldc);
    const FtPast none = {nullptr, nullptr, nullptr, 0, 0, 0};
    if (HD == 64)
        return launch_ft<64, FT_STAGES_64, false>(ctx, ldc, q, k, v, ld, gate, ldg, seq_start, B, max_len, T, QH, KVH, window, scale,
                                       none, nullptr, err, st);
    if (HD == 128)
        return launch_ft<128, FT_STAGES_128, false>(ctx, ldc, q, k, v, ld, gate, ldg, seq_start, B, max_len, T, QH, KVH, window, scale,
                                        none, nullptr, err, st);
    CM_REFUSE("attn_prefill_tc: head size %d (64 or 128)", HD);
}

// The same for sequences that stand at seq_pos0[b] >= 0: entries below that position come from the
// paged bfloat16 cache `pool` [2, pages, KVH, PAGE_TOKENS, HD] through the page table (a ring of
// `ring` entries when ring > 0), the rest from the step's own rows.  The caller writes the step's keys
// and values to the cache afterwards.  max_len: the most rows a sequence brings to this step.
extern "C" int cm_attn_append_tc(void* ctx, long long ldc, const void* q, const void* k, const void* v, long long ld,
                                 const void* gate, long long ldg, const int* seq_start, const int* seq_pos0,
                                 const int* seq_slot, const void* pool, long long pages, const int* ptab,
                                 long long ptab_stride, int ring, int B, int max_len, long long T, int QH, int KVH,
                                 int HD, int window, float scale, int* err, cudaStream_t st) {
    if (B <= 0 || max_len <= 0) return CM_OK;
    if (QH % KVH) CM_REFUSE("attn_append_tc: %d query heads over %d key heads", QH, KVH);
    if (ring % PAGE_TOKENS) CM_REFUSE("attn_append_tc: ring of %d entries is no multiple of %d", ring, PAGE_TOKENS);
    if (!seq_pos0 || !seq_slot || !pool || !ptab)
        CM_REFUSE("attn_append_tc: positions, slots, cache and page table are needed");
    if (ld % 8 || ldc % 8 || (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)ctx | (uintptr_t)pool) & 15))
        CM_REFUSE("attn_append_tc: row pitches %lld, %lld must be multiples of 8 and the operands 16-byte aligned", ld, ldc);
    if (2 * pages * KVH * PAGE_TOKENS > 0x7fffffffLL) CM_REFUSE("attn_append_tc: a cache of %lld pages is too large", pages);
    const FtPast past = {seq_pos0, seq_slot, ptab, ptab_stride, pages, ring};
    if (HD == 64)
        return launch_ft<64, FT_STAGES_64, true>(ctx, ldc, q, k, v, ld, gate, ldg, seq_start, B, max_len, T, QH, KVH, window, scale,
                                      past, pool, err, st);
    if (HD == 128)
        return launch_ft<128, FT_STAGES_128, true>(ctx, ldc, q, k, v, ld, gate, ldg, seq_start, B, max_len, T, QH, KVH, window, scale,
                                       past, pool, err, st);
    CM_REFUSE("attn_append_tc: head size %d (64 or 128)", HD);
}
