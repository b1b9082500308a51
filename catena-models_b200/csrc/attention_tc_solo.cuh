// Prefill attention on tcgen05 for heads of 64, second form: each softmax group has a query tile of its own.
// (Included by attention_tc.cu, which has the helpers, FtItem and the first form; same operands, same result.)
//
// A block is two pipelines that share nothing but the SM: pipeline g = one thread that copies (Q, then K and V
// tiles, into rings of the pipeline's own), one thread that issues products, and the four warps of softmax group
// g, with their own 256 columns of tensor memory: S (128 columns), P (64: 128 bfloat16 a row) and O (64).
// A pipeline walks its own items (a 128-query tile of one head of one sequence), pipelines 2 x blocks in all,
// long rows first, to and fro (ft_item_of_round).  Per key tile of an item:
//   issuer   S = Q K^T into the S columns, as soon as the group has read the tile before out of them (s_read);
//            O (+)= P V once the group has announced P (p_full); commits to s_full / o_full and to the rings;
//   group    reads the row's 128 scores into registers (one row a thread), says so (s_read), takes the maximum,
//            writes the exponentials as bfloat16 into the P columns once the product before has read them
//            (o_full), announces P.  O stays in tensor memory; the reference the exponentials are taken against
//            moves only when a row's maximum has grown by a factor of 256 (see the first form).
// At an item's end the group waits for its last product, reads O, gives it back (o_free), normalises, gates and
// stores its rows; meanwhile its copier and issuer are already at the next item (its Q once the item's scores
// are all formed, its first scores once S is read out), and the other pipeline has the SM's arithmetic to itself:
// what an item costs besides its tiles (the first tile's way through copy, product and softmax, the last
// product, the store) is idle time of one pipeline only.
//
// Every wait on an mbarrier is bounded; a wait that runs out raises *err and the block's abort flag, all roles
// leave their loops, copies in flight are awaited (bounded), tensor memory is freed.

template <int HD, int STAGES, bool PAST>
__global__ void __launch_bounds__(FT_THREADS, 1)
attn_prefill_tc_solo_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_pool,
                            const FtPast past, bf16* __restrict__ ctx, long long ldc,
                            const bf16* __restrict__ gate, long long ldg, const int* __restrict__ seq_start, int QH,
                            int KVH, int B, int tiles_x, int window, float scale_log2, int* err) {
    constexpr int KB = HD / 64;                                   // 64-column pieces of a head
    constexpr uint32_t Q_BYTES = KB * FT_PIECE_BYTES, KV_BYTES = KB * FT_PIECE_BYTES;
    constexpr uint32_t PIPE_BYTES = Q_BYTES + 2 * STAGES * KV_BYTES;
    constexpr uint32_t COL_P = FT_TILE, COL_O = FT_TILE + 64, PIPE_COLS = FT_TILE + 64 + HD, TMEM_COLS = 512;
    static_assert(2 * PIPE_COLS <= TMEM_COLS, "tensor memory holds S, P and O of both pipelines");
    // per pipeline: q_full, q_empty, s_full, s_read, p_full, o_full, o_free, then k_full, k_empty, v_full, v_empty per stage
    constexpr int PIPE_BARS = 7 + 4 * STAGES;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bars[2 * PIPE_BARS];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ int issued_q[2], issued_k[2], issued_v[2];

    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total = tiles_x * QH * B, pipes = 2 * gridDim.x;
    // roles: warps 0, 1 copy for pipelines 0, 1; warps 2, 3 issue; warps 4-7 and 8-11 are the softmax groups
    const int g = warp < 4 ? (warp & 1) : (warp - 4) >> 2;
    const int pipe = 2 * blockIdx.x + g;

    const uint32_t base = ((smem_u32(smem_raw) + 1023u) & ~1023u) + (uint32_t)g * PIPE_BYTES;
    const uint32_t q_s = base, k_s = q_s + Q_BYTES, v_s = k_s + STAGES * KV_BYTES;
    const uint32_t bar0 = smem_u32(&bars[0]) + (uint32_t)(g * PIPE_BARS) * 8;
    const uint32_t q_full = bar0, q_empty = bar0 + 8, s_full = bar0 + 16, s_read = bar0 + 24, p_full = bar0 + 32,
                   o_full = bar0 + 40, o_free = bar0 + 48;
    const uint32_t k_full = bar0 + 56, k_empty = k_full + 8 * STAGES, v_full = k_empty + 8 * STAGES,
                   v_empty = v_full + 8 * STAGES;

    if (warp == 0) {
        // one lane per mbarrier; s_read, p_full and o_free take one arrival per warp of the group, all others one
        for (int i = lane; i < 2 * PIPE_BARS; i += 32) {
            const int k = i % PIPE_BARS;
            mbar_init(smem_u32(&bars[i]), k == 3 || k == 4 || k == 6 ? 4 : 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (lane == 0) {
            abort_flag = 0;
            for (int p = 0; p < 2; ++p) issued_q[p] = issued_k[p] = issued_v[p] = 0;
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
    const uint32_t tmem_pipe = tmem_slot + (uint32_t)g * PIPE_COLS;
    // Every role of a pipeline walks the pipeline's items and counts them (i) and their key tiles (J) from the
    // start: the rings and all mbarrier phases go by these counts and run on across an item's border.
    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if (warp < 2 && lane == 0) {
            // ------------------------------------------------------------- copies: Q of an item, then its K and V tiles
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
            for (int rnd = 0; rnd * pipes < total && ok; ++rnd) {
                const int w = ft_item_of_round(rnd, pipe, pipes, total);
                if (w < 0) continue;
                ft_item<PAST>(w, tiles_x, QH, KVH, B, window, seq_start, past, it);
                if (it.n == 0) continue;
                // Q's place is free once the scores of the item before are all formed
                ok = ft_mbar_wait(q_empty, (i & 1) ^ 1, &abort_flag, err, FT_ERR_LOAD);
                if (!ok) break;
                mbar_expect_tx(q_full, Q_BYTES);
                for (int kb = 0; kb < KB; ++kb)
                    tma_load_2d(q_s + kb * FT_PIECE_BYTES, &map_q, q_full, it.hq * HD + kb * 64, it.s0 + it.q0);
                issued_q[g] = ++i;
                for (int j = 0; j < it.n && ok; ++j) {
                    load_tile(j, k_s, k_full, k_empty, &map_k, 0);
                    if (ok) issued_k[g] = J + 1;
                    if (ok) load_tile(j, v_s, v_full, v_empty, &map_v, 1);
                    if (ok) issued_v[g] = J + 1;
                    ++J;
                }
            }
            pdl_trigger();                            // every tile is requested: the next kernel may start up
        } else if (warp >= 2 && lane == 0) {
            // ------------------------------------------------------------- products
            // S: float accumulator, bf16 operands from shared memory, both K-major, N = 128.  O: A (P) from tensor
            // memory, B (V) from shared memory, MN-major (its rows are keys), N = HD.
            constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(FT_TILE >> 3) << 17) |
                                         ((uint32_t)(FT_TILE >> 4) << 24);
            constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) |
                                         ((uint32_t)(FT_TILE >> 4) << 24);
            bool ok = true;
            // Two walks over the pipeline's tiles: the one whose scores are issued (round sr, the item's tiles sn,
            // the tile sj, items so far si, tiles so far Js) is one tile ahead of the one whose product is (pr, ..., J).
            int sr = -1, sn = 0, sj = -1, si = -1, Js = 0;
            int pr = -1, pn = 0, pj = 0, pi = -1, J = 0;
            bool s_valid = true;
            // moves the score walk to the next tile; the item it leaves gives its Q back
            auto advance_s = [&]() {
                if (++sj < sn) return;
                if (si >= 0) umma_commit(q_empty);                   // the item's scores are all issued
                do {
                    ++sr;
                    if (sr * pipes >= total) { s_valid = false; return; }
                    const int w = ft_item_of_round(sr, pipe, pipes, total);
                    sn = w < 0 ? 0 : ft_item_tiles<PAST>(w, tiles_x, QH, KVH, B, window, seq_start, past);
                } while (sn == 0);
                sj = 0;
                ++si;
            };
            // S of the score walk's tile; the S columns are free (nothing was in them yet, or s_read said so)
            auto scores = [&]() {
                const int s = Js % STAGES;
                if (sj == 0) ok = ft_mbar_wait(q_full, si & 1, &abort_flag, err, FT_ERR_MMA);
                if (ok) ok = ft_mbar_wait(k_full + 8 * s, (Js / STAGES) & 1, &abort_flag, err, FT_ERR_MMA);
                if (!ok) return;
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint64_t a = umma_desc(q_s + (k >> 2) * FT_PIECE_BYTES) + 2 * (k & 3);
                    const uint64_t bd = umma_desc(k_s + s * KV_BYTES + (k >> 2) * FT_PIECE_BYTES) + 2 * (k & 3);
                    umma_bf16(tmem_pipe, a, bd, idesc_s, k != 0);
                }
                umma_commit(s_full);
                umma_commit(k_empty + 8 * s);
                ++Js;
            };
            advance_s();                                             // the first item
            if (s_valid) {
                scores();
                advance_s();
            }
            while (ok) {
                // the product walk's next tile
                if (++pj >= pn) {
                    do {
                        ++pr;
                        if (pr * pipes >= total) break;
                        const int w = ft_item_of_round(pr, pipe, pipes, total);
                        pn = w < 0 ? 0 : ft_item_tiles<PAST>(w, tiles_x, QH, KVH, B, window, seq_start, past);
                    } while (pn == 0);
                    if (pr * pipes >= total) break;
                    pj = 0;
                    ++pi;
                    // O holds the item before until the group has read it
                    if (pi >= 1) ok = ft_mbar_wait(o_free, (pi - 1) & 1, &abort_flag, err, FT_ERR_MMA);
                    if (!ok) break;
                }
                // the next tile's scores as soon as this tile's are read out ...
                if (s_valid) {
                    ok = ft_mbar_wait(s_read, J & 1, &abort_flag, err, FT_ERR_MMA);
                    if (!ok) break;
                    scores();
                    if (!ok) break;
                    advance_s();
                }
                // ... and this tile's product once P is there.  V first: it has long been loaded.
                const int s = J % STAGES;
                ok = ft_mbar_wait(v_full + 8 * s, (J / STAGES) & 1, &abort_flag, err, FT_ERR_MMA);
                if (ok) ok = ft_mbar_wait(p_full, J & 1, &abort_flag, err, FT_ERR_MMA);
                // O is in order as well: when the group rescales it, it does so before it announces P, with every
                // earlier product finished.
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < FT_TILE / 16; ++k) {                // 16 keys per instruction: 8 columns of P
                    const uint64_t bd = umma_desc_mn(v_s + s * KV_BYTES + k * 2048, FT_PIECE_BYTES);
                    umma_bf16_ts(tmem_pipe + COL_O, tmem_pipe + COL_P + (uint32_t)(8 * k), bd, idesc_o, k != 0 || pj > 0);
                }
                umma_commit(o_full);
                umma_commit(v_empty + 8 * s);
                ++J;
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
        // ------------------------------------------------------------- softmax group g: one query row a thread
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;                        // the row of the tile this thread owns
        const uint32_t lane_base = tmem_pipe + ((uint32_t)(quarter * 32) << 16);
        const uint32_t t_s = lane_base, t_p = lane_base + COL_P, t_o = lane_base + COL_O;
        const uint32_t full = 0xffffffffu;
        constexpr float RESCALE = 8.f;                            // the reference follows the maximum after a factor of 256
        bool ok = true;
        int J = 0;                                                // key tiles of this pipeline so far
        int products_done = 0;                                    // products 0 .. products_done - 1 are finished
        uint32_t s_early = 0;                                     // the next tile's scores were seen to be there
        auto await_products = [&](int upto) {
            if (products_done >= upto) return;                    // warp-uniform: every lane counts alike
            while (ok && products_done < upto) {
                ok = ft_mbar_wait(o_full, products_done & 1, &abort_flag, err, FT_ERR_SOFTMAX);
                ++products_done;
            }
            ok = __all_sync(full, ok);                            // what follows is warp-wide
        };
        for (int rnd = 0; rnd * pipes < total && ok; ++rnd) {
            const int w = ft_item_of_round(rnd, pipe, pipes, total);
            if (w < 0) continue;
            FtItem it;
            ft_item<PAST>(w, tiles_x, QH, KVH, B, window, seq_start, past, it);
            if (it.n == 0) continue;
            const int row_l = it.q0 + r;                          // this thread's row among the sequence's rows of this step
            const int row = it.p0 + row_l;                        // its position in the sequence
            float m_ref = -INFINITY, l_run = 0.f;
            for (int j = 0; j < it.n && ok; ++j, ++J) {
                // first position of the tile, and the position where its sequence's entries end
                const bool from_cache = PAST && j < it.n_past;
                const int k0 = from_cache ? (it.tp_begin + j) * FT_TILE : it.p0 + (it.kt_begin + j - it.n_past) * FT_TILE;
                const int limit = from_cache ? it.p0 : it.p0 + it.len;
                // (asked at the end of the tile before: the scores are formed while the group is at its exponentials)
                if (!__all_sync(full, s_early)) ok = __all_sync(full, ft_mbar_wait(s_full, J & 1, &abort_flag, err, FT_ERR_SOFTMAX));
                if (!ok) break;
                tc_fence_after();
                float v[FT_TILE];                                     // the row's 128 scores, read once
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_load32_issue(t_s + (uint32_t)(32 * c), v + 32 * c);
                // Asked now, read after the maxima: has the product of the tile before finished?  It reads the P
                // columns that this tile's exponentials go to.  (A look at an mbarrier costs about a hundred cycles
                // when it stands in the way.)
                uint32_t early = 1;
                if (J >= 1 && products_done == J - 1) early = ft_mbar_test(o_full, (uint32_t)((J - 1) & 1));
                tmem_load_wait();
                // the scores are in registers: their columns may take the next tile's
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(s_read);
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
                if (J >= 1 && products_done == J - 1 && __all_sync(full, early)) products_done = J;
                const bool grown = m_cand - m_ref > RESCALE;
                if (j > 0 && __any_sync(full, grown)) {
                    // The warp owns its 32 lanes of tensor memory, so the warp decides; rows that have not grown
                    // much move to their own maximum as well (a factor below one).  Every product so far must be done.
                    await_products(J);
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
                // two partial sums of pairs: a chain of 64 dependent additions would leave the thread waiting on their latency
                const uint64_t scale2 = ft_pack2(scale_log2, scale_log2), minus_m2 = ft_pack2(-m_use, -m_use);
                uint64_t rs2[2] = {ft_pack2(0.f, 0.f), ft_pack2(0.f, 0.f)};
                uint32_t pk[FT_TILE / 2];                             // the row's probabilities, two bfloat16 a word
#pragma unroll
                for (int e = 0; e < FT_TILE / 2; ++e) {
                    float x0, x1;
                    ft_unpack2(ft_fma2(ft_pack2(v[2 * e], v[2 * e + 1]), scale2, minus_m2), x0, x1);
                    const float e0 = ft_exp2(x0), e1 = ft_exp2(x1);
                    rs2[e & 1] = ft_add2(rs2[e & 1], ft_pack2(e0, e1));
                    __nv_bfloat162 h = __floats2bfloat162_rn(e0, e1);
                    pk[e] = *reinterpret_cast<uint32_t*>(&h);
                }
                // The product of the tile before reads the P columns: it has had the time of the exponentials to finish.
                await_products(J);
                if (!ok) break;
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_store16_issue(t_p + (uint32_t)(16 * c), pk + 16 * c);   // 32 probabilities are 16 columns
                // asked now, read at the top of the next tile: are its scores there?
                s_early = ft_mbar_test(s_full, (uint32_t)((J + 1) & 1));
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
                if (lane == 0) mbar_arrive(p_full);               // P is in tensor memory and O is in order
                l_run += rs;
            }
            if (!ok) break;
            // ---- the item's end: the last product, then O from tensor memory, normalised, gated and stored
            await_products(J);
            if (!ok) break;
            tc_fence_after();
            float o[HD];
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) tmem_load32_issue(t_o + (uint32_t)(32 * c), o + 32 * c);
            tmem_load_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(o_free);                   // O may take the next item's first product
            if (row_l < it.len) {
                float f = 1.f / l_run;
                const long long tok = it.s0 + row_l;
                if (gate) f *= sigmoid_f32(__bfloat162float(gate[tok * ldg + it.hq]));
                bf16* dst = ctx + tok * ldc + (long long)it.hq * HD;
#pragma unroll
                for (int c = 0; c < HD / 8; ++c) {
                    uint4 raw;
                    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
                    for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(o[8 * c + 2 * e] * f, o[8 * c + 2 * e + 1] * f);
                    *reinterpret_cast<uint4*>(dst + 8 * c) = raw;
                }
            }
        }
    }
    // ------------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (abort_flag && threadIdx.x < 2) {
        // copies that were issued but never consumed must land before shared memory is given up
        const int p = threadIdx.x;
        const uint32_t pb = smem_u32(&bars[p * PIPE_BARS]);
        if (issued_q[p] > 0)
            for (int c = 0; c < TC_SPIN_LIMIT; ++c)
                if (mbar_try_wait(pb, (issued_q[p] - 1) & 1)) break;
        for (int j = max(0, issued_k[p] - STAGES); j < issued_k[p]; ++j)
            for (int c = 0; c < TC_SPIN_LIMIT; ++c)
                if (mbar_try_wait(pb + 56 + 8 * (j % STAGES), (j / STAGES) & 1)) break;
        for (int j = max(0, issued_v[p] - STAGES); j < issued_v[p]; ++j)
            for (int c = 0; c < TC_SPIN_LIMIT; ++c)
                if (mbar_try_wait(pb + 56 + 16 * STAGES + 8 * (j % STAGES), (j / STAGES) & 1)) break;
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_slot), "r"(TMEM_COLS) : "memory");
    }
}
