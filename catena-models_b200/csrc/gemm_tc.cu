// C[M,N] = A[M,K] * B[N,K]^T in bfloat16 on the 5th-generation tensor cores (prompt steps).
//
// One block per SM computes 128 x BLOCK_N tiles of C, one after another.  Roles (ten warps):
//   warp 0  one thread: TMA loads of the A and B k-slices (128 x 64 and BLOCK_N x 64 bf16,
//           128-byte swizzle) into a ring of STAGES shared-memory stages;
//   warp 1  allocates the tensor-memory columns of the accumulator; one thread issues
//           tcgen05.mma (128 x BLOCK_N x 16 per instruction, float accumulation in tensor
//           memory) and commits each stage back to the loader and the finished tile to the
//           epilogue through mbarriers;
//   warps 2-9  epilogue, two groups of four warps that take alternate 128-byte-wide pieces of
//           the tile: tcgen05.ld of the accumulator (a warp reaches the 32 lanes 32*(warp%4)..),
//           conversion, the piece into the group's 16 KB staging buffer (128-byte swizzle), and a
//           TMA store of it to C, clipped at M and N.  (Stores straight from registers, 16 bytes per row per instruction, held
//           the tensor cores back: 2048 x 6144 x 2048 took 53.6 us with them, 38.4 us with the
//           epilogue's work removed.)  Outputs whose pitch or base is not 16-byte aligned
//           keep the direct stores.
// Rows or columns beyond M, N, K are zero-filled by TMA on load and masked on store, so any
// M and N and any K that is a multiple of 8 (16-byte row pitch) is taken.
//
// MODE_SWIGLU: B is the row-packed [Wgate; Wup] with 2N rows; the B stage is two half-height boxes
// (gate rows n0.., up rows N+n0..), so the first half of the accumulator's columns is g, the second u,
// and the epilogue stores C = T(silu(T(g)) * T(u)) (catena-models' fused gate epilogue,
// src/catena/lfm3_wmma.hex:10790-10815).
//
// Every wait on an mbarrier is bounded.  A wait that runs out raises *err, every role leaves
// its loop, copies still in flight are awaited (bounded again), tensor memory is freed and the
// block returns.
#include "tc_common.cuh"
#include <cooperative_groups.h>

#define TC_BM 128
static_assert(TC_BM == CM_FEW_ROWS_MAX_ROWS, "cm_limits.h: CM_FEW_ROWS_MAX_ROWS");
#define TC_THREADS 192
#define TCP_THREADS 320          // the persistent kernel: loader, issuer, two groups of four epilogue warps
#define TC_MODE_PLAIN 0
#define TC_MODE_SWIGLU 1

template <typename TC>
__device__ __forceinline__ void store_cols(TC* dst, const float* v, int n_valid, bool aligned);
template <>
__device__ __forceinline__ void store_cols<bf16>(bf16* dst, const float* v, int n_valid, bool aligned) {
    if (n_valid >= 32 && aligned) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint4 raw;
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[8 * i + 2 * j], v[8 * i + 2 * j + 1]);
            *reinterpret_cast<uint4*>(dst + 8 * i) = raw;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)                       // unrolled: v stays in registers
            if (i < n_valid) dst[i] = __float2bfloat16_rn(v[i]);
    }
}
template <>
__device__ __forceinline__ void store_cols<float>(float* dst, const float* v, int n_valid, bool aligned) {
    if (n_valid >= 32 && aligned) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            *reinterpret_cast<float4*>(dst + 4 * i) = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i < n_valid) dst[i] = v[i];
    }
}


// Order of the output tiles: groups of TC_GROUP_M row tiles, inside a group down the rows first.
// The blocks that run at the same time then share few B tiles (and few A tiles) instead of
// touching every column tile of one or two row tiles.
#define TC_GROUP_M 8
__device__ __forceinline__ void tile_origin(int tile, int m_tiles, int n_tiles, int* m_tile, int* n_tile) {
    const int per_group = TC_GROUP_M * n_tiles;
    const int group = tile / per_group, in_group = tile - group * per_group;
    const int rows = min(TC_GROUP_M, m_tiles - group * TC_GROUP_M);
    *m_tile = group * TC_GROUP_M + in_group % rows;
    *n_tile = in_group / rows;
}

// Persistent form: gridDim.x blocks (one per SM) walk the output tiles t = blockIdx.x,
// blockIdx.x + gridDim.x, ...; tile t covers rows (t / n_tiles) * 128 and output columns
// (t % n_tiles) * OUT_COLS.  The accumulator is double-buffered in tensor memory (2 * BLOCK_N
// columns), so the epilogue of one tile runs while the next tile's products are issued; the
// shared-memory ring of k-slices keeps turning across tile borders.
template <int BLOCK_N, int STAGES, typename TC, int MODE>
__global__ void __launch_bounds__(TCP_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_c, int tma_store_ok, TC* __restrict__ C, int M, int N, int K,
               long long ldc, int ksplit, long long part_stride, int* err) {
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2;
    constexpr uint32_t B_BYTES = BLOCK_N * TC_BK * 2;
    constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int OUT_COLS = MODE == TC_MODE_SWIGLU ? BLOCK_N / 2 : BLOCK_N;
    constexpr uint32_t TMEM_COLS = 2 * BLOCK_N <= 256 ? 256 : 512;    // two accumulators; allocations are powers of two
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bars[2 * STAGES + 4];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ int issued_kb;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (K + TC_BK - 1) / TC_BK;
    const int n_tiles = (N + OUT_COLS - 1) / OUT_COLS;
    const int m_tiles = (M + TC_BM - 1) / TC_BM;
    const int num_tiles = n_tiles * m_tiles;
    // ksplit > 1: the inner dimension is cut into ksplit runs of kb_per k-slices, every (run, tile) is an
    // item of work of its own, and run r leaves its sums at C + r * part_stride (map_c: row r * M + ...)
    const int kb_per = (num_kb + ksplit - 1) / ksplit;
    const int num_items = num_tiles * ksplit;
    const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;                    // swizzle atoms need 1024-byte alignment
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t acc_full0 = smem_u32(&bars[2 * STAGES]), acc_empty0 = smem_u32(&bars[2 * STAGES + 2]);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full0 + 8 * a, 1);
            mbar_init(acc_empty0 + 8 * a, 8);                   // one arrival per epilogue warp
        }
        abort_flag = 0;
        issued_kb = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
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
    pdl_wait();                                   // A is the previous kernel's output

    if (warp == 0 && lane == 0) {
        // ------------------------------------------------------------- TMA loader
        int it = 0;                               // k-slices issued so far, over all tiles
        bool ok = true;
        for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
            const int run = item / num_tiles, tile = item - run * num_tiles;
            int m_tile, n_tile;
            tile_origin(tile, m_tiles, n_tiles, &m_tile, &n_tile);
            const int m0 = m_tile * TC_BM, n0 = n_tile * OUT_COLS;
            const int kb_end = min(num_kb, (run + 1) * kb_per);
            for (int kb = run * kb_per; kb < kb_end; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                ok = mbar_wait(empty0 + 8 * s, ph ^ 1, &abort_flag, err, TC_ERR_TIMEOUT_LOAD);
                if (!ok) break;
                const uint32_t a_dst = tiles + s * STAGE_BYTES, b_dst = a_dst + A_BYTES;
                mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                tma_load_2d(a_dst, &map_a, full0 + 8 * s, kb * TC_BK, m0);
                if (MODE == TC_MODE_SWIGLU) {
                    tma_load_2d(b_dst, &map_b, full0 + 8 * s, kb * TC_BK, n0);
                    tma_load_2d(b_dst + B_BYTES / 2, &map_b, full0 + 8 * s, kb * TC_BK, N + n0);
                } else {
                    tma_load_2d(b_dst, &map_b, full0 + 8 * s, kb * TC_BK, n0);
                }
                issued_kb = it + 1;
            }
        }
        pdl_trigger();                            // every k-slice is requested: the next kernel may start up
    } else if (warp == 1 && lane == 0) {
        // ------------------------------------------------------------- MMA issuer
        // instruction descriptor: float accumulator, bf16 A and B, both K-major, N/8 and M/16
        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BLOCK_N >> 3) << 17) |
                                   ((uint32_t)(TC_BM >> 4) << 24);
        int it = 0, local = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++local) {
            const int acc = local & 1;
            // the epilogue must have drained this accumulator (two tiles ago)
            ok = mbar_wait(acc_empty0 + 8 * acc, ((local >> 1) & 1) ^ 1, &abort_flag, err, TC_ERR_TIMEOUT_MMA);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BLOCK_N);
            const int kb_begin = (item / num_tiles) * kb_per, kb_end = min(num_kb, kb_begin + kb_per);
            for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                ok = mbar_wait(full0 + 8 * s, ph, &abort_flag, err, TC_ERR_TIMEOUT_MMA);
                if (!ok) break;
                tc_fence_after();
                const uint64_t adesc = umma_desc(tiles + s * STAGE_BYTES);
                const uint64_t bdesc = umma_desc(tiles + s * STAGE_BYTES + A_BYTES);
#pragma unroll
                for (int k = 0; k < TC_BK / 16; ++k)      // 16 values of k = 32 bytes further in the row
                    umma_bf16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, ((kb - kb_begin) | k) != 0);
                umma_commit(empty0 + 8 * s);              // stage is free once these MMAs have read it
            }
            if (ok) umma_commit(acc_full0 + 8 * acc);     // accumulator complete
        }
    } else if (warp >= 2) {
        // ------------------------------------------------------------- epilogue
        // The four warps run the same number of rounds whatever happens (a warp whose wait ran
        // out goes on without loading or storing), so that the barriers between them always meet.
        const int q = warp & 3;                           // tensor-memory lane quarter of this warp
        const bool vec_ok = (ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
        const int group = (warp - 2) >> 2;                // two groups of four warps take alternate pieces
        const bool elected = lane == 0 && q == 2;         // first warp of the group: issues and awaits its TMA stores
        constexpr int CHUNK_COLS = 128 / (int)sizeof(TC); // output columns of a staged piece: 128 bytes a row
        constexpr int SUB = CHUNK_COLS / 32;              // tensor-memory loads of 32 columns per piece
        const uint32_t sbuf = tiles + STAGES * STAGE_BYTES + (uint32_t)group * 16384u;   // the group's staging buffer
        const int r_tile = q * 32 + lane;
        int local = 0;
        for (int item = blockIdx.x; item < num_items; item += gridDim.x, ++local) {
            const int acc = local & 1;
            const int run = item / num_tiles, tile = item - run * num_tiles;
            int m_tile, n_tile;
            tile_origin(tile, m_tiles, n_tiles, &m_tile, &n_tile);
            const int m0 = m_tile * TC_BM, n0 = n_tile * OUT_COLS;
            const int row = m0 + r_tile;
            // a run's rows end at M, where the next run's begin: a row tile that crosses M is stored from registers
            const bool tma_store = tma_store_ok && (ksplit == 1 || m0 + TC_BM <= M);
            TC* const C_run = C + (long long)run * part_stride;
            const bool ok = mbar_wait(acc_full0 + 8 * acc, (local >> 1) & 1, &abort_flag, err, TC_ERR_TIMEOUT_EPILOGUE);
            tc_fence_after();
            const uint32_t t_acc = tmem_base + (uint32_t)(acc * BLOCK_N) + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
            for (int c0 = group * CHUNK_COLS; c0 < OUT_COLS; c0 += 2 * CHUNK_COLS) {
                if (tma_store) {
                    // the group's last store must be done reading the buffer
                    if (elected) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    asm volatile("bar.sync %0, 128;" ::"r"(group + 1) : "memory");
                }
#pragma unroll
                for (int h = 0; h < SUB; ++h) {
                    const int c = c0 + 32 * h;
                    float v[32];
                    if (ok) {
                        tmem_load32(t_acc + (uint32_t)c, v);
                        if (MODE == TC_MODE_SWIGLU) {
                            float u[32];
                            tmem_load32(t_acc + (uint32_t)(OUT_COLS + c), u);
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                const float g = rounded<TC>(v[i]), uu = rounded<TC>(u[i]);
                                v[i] = __fdividef(g, 1.f + __expf(-g)) * uu;
                            }
                        }
                        if (tma_store) {
                            stage_cols(sbuf, r_tile, h * (32 * (int)sizeof(TC) / 16), v, (TC*)nullptr);
                        } else {
                            const int col = n0 + c;
                            if (row < M && col < N) store_cols<TC>(C_run + (long long)row * ldc + col, v, N - col, vec_ok);
                        }
                    }
                }
                if (tma_store) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    asm volatile("bar.sync %0, 128;" ::"r"(group + 1) : "memory");
                    if (elected) {
                        if (ok && n0 + c0 < N) tma_store_2d(&map_c, sbuf, n0 + c0, run * M + m0);   // clipped at M and N
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + 8 * acc);    // this warp has read its quarter
        }
        if (elected) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
    // ------------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (abort_flag && threadIdx.x == 0) {
        // copies that were issued but never consumed must land before shared memory is given up
        const int issued = issued_kb;
        for (int kb = max(0, issued - STAGES); kb < issued; ++kb) {
            const int s = kb % STAGES;
            for (int i = 0; i < TC_SPIN_LIMIT; ++i)
                if (mbar_try_wait(full0 + 8 * s, (kb / STAGES) & 1)) break;
        }
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                     : "memory");
    }
}

__device__ __forceinline__ void store4(bf16* dst, const float* o) {
    uint2 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
    h[0] = __floats2bfloat162_rn(o[0], o[1]);
    h[1] = __floats2bfloat162_rn(o[2], o[3]);
    *reinterpret_cast<uint2*>(dst) = raw;
}
__device__ __forceinline__ void store4(float* dst, const float* o) {
    *reinterpret_cast<float4*>(dst) = make_float4(o[0], o[1], o[2], o[3]);
}

// Few rows (M <= 128), split over K: the form for decode steps of 17 to 128 sequences, where a
// product has too few 128-column tiles to put every SM to streaming weights.  Grid (column
// tile, split): the `splits` blocks of a column tile form a thread-block cluster, each takes a
// contiguous share of the k-slices through the same TMA -> tcgen05 pipeline as above (one
// accumulator, 128 columns of tensor memory) and leaves its partial sums as float rows in its own
// shared memory (the drained stage ring).  After a cluster barrier, block r of the cluster adds
// rows r, r + splits, ... over all blocks in rank order through distributed shared memory,
// applies the epilogue and stores them; a second cluster barrier keeps every block's shared
// memory alive until its peers have read it.  The weights' k-slices of the first stages are
// requested before the wait on the previous kernel, the activations' after it.
#define TCS_BN 128
#define TCS_PITCH (TCS_BN + 4)          // floats per staged row: float4 stores of 32 lanes spread over all banks

//
// A_ROWS (64 or 128) rows of activations are brought per k-slice.  With 64, the upper half of the
// 128-row operand that the tensor core reads is whatever follows in shared memory (the weights'
// tile): those accumulator rows are never read, and a row of the product depends on its own row of
// A only.  Shared memory stays under half an SM's in both forms (4 stages of 24 KB, 3 of 32 KB), so
// that two blocks share an SM and the next kernel's blocks can request their weights while this
// kernel's are still adding up.
template <typename TC, int MODE, int A_ROWS, int TCS_STAGES>
__global__ void __launch_bounds__(TC_THREADS, 2)
gemm_tc_splitk_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      TC* __restrict__ C, float* __restrict__ parts, long long part_stride, int M, int N, int K,
                      long long ldc, int splits, int* err) {
    constexpr uint32_t A_BYTES = A_ROWS * TC_BK * 2;
    constexpr uint32_t B_BYTES = TCS_BN * TC_BK * 2;
    constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int OUT_COLS = MODE == TC_MODE_SWIGLU ? TCS_BN / 2 : TCS_BN;
    static_assert((size_t)TCS_STAGES * STAGE_BYTES >= (size_t)A_ROWS * TCS_PITCH * 4, "staged rows must fit the ring");
    static_assert(TCS_STAGES * STAGE_BYTES <= 104 * 1024, "two blocks per SM");
    static_assert(STAGE_BYTES >= TC_BM * TC_BK * 2, "the 128-row operand read stays inside its stage");
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bars[2 * TCS_STAGES + 1];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ int issued_kb;

    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = blockIdx.y;                                 // clusters are (1, splits, 1) and gridDim.y == splits
    const int num_kb = (K + TC_BK - 1) / TC_BK;
    const int per = (num_kb + splits - 1) / splits;
    const int kb0 = rank * per;
    const int my_kb = max(0, min(num_kb, kb0 + per) - kb0);
    const int n0 = blockIdx.x * OUT_COLS;
    const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
    float* stage = reinterpret_cast<float*>(smem_raw + (tiles - smem_u32(smem_raw)));
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[TCS_STAGES]);
    const uint32_t acc_full = smem_u32(&bars[2 * TCS_STAGES]);

    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
        for (int s = 0; s < TCS_STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(acc_full, 1);
        abort_flag = 0;
        issued_kb = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                     "r"((uint32_t)TCS_BN)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;

    auto load_b = [&](int i) {
        const int s = i % TCS_STAGES;
        const uint32_t b_dst = tiles + s * STAGE_BYTES + A_BYTES;
        mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
        if (MODE == TC_MODE_SWIGLU) {
            tma_load_2d(b_dst, &map_b, full0 + 8 * s, (kb0 + i) * TC_BK, n0);
            tma_load_2d(b_dst + B_BYTES / 2, &map_b, full0 + 8 * s, (kb0 + i) * TC_BK, N + n0);
        } else {
            tma_load_2d(b_dst, &map_b, full0 + 8 * s, (kb0 + i) * TC_BK, n0);
        }
    };
    auto load_a = [&](int i) {
        const int s = i % TCS_STAGES;
        tma_load_2d(tiles + s * STAGE_BYTES, &map_a, full0 + 8 * s, (kb0 + i) * TC_BK, 0);
    };

    if (warp == 0 && lane == 0) {
        // ------------------------------------------------------------- TMA loader
        const int head = min(my_kb, TCS_STAGES);
        for (int i = 0; i < head; ++i) load_b(i);               // weights do not depend on the previous kernel
        pdl_wait();
        for (int i = 0; i < head; ++i) load_a(i);
        issued_kb = head;
        for (int i = head; i < my_kb; ++i) {
            const int s = i % TCS_STAGES;
            if (!mbar_wait(empty0 + 8 * s, ((i / TCS_STAGES) & 1) ^ 1, &abort_flag, err, TC_ERR_TIMEOUT_LOAD)) break;
            load_b(i);
            load_a(i);
            issued_kb = i + 1;
        }
        pdl_trigger();                            // every k-slice is requested: the next kernel may start up
    } else if (warp == 1 && lane == 0) {
        // ------------------------------------------------------------- MMA issuer
        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TCS_BN >> 3) << 17) |
                                   ((uint32_t)(TC_BM >> 4) << 24);
        bool ok = true;
        for (int i = 0; i < my_kb; ++i) {
            const int s = i % TCS_STAGES;
            ok = mbar_wait(full0 + 8 * s, (i / TCS_STAGES) & 1, &abort_flag, err, TC_ERR_TIMEOUT_MMA);
            if (!ok) break;
            tc_fence_after();
            const uint64_t adesc = umma_desc(tiles + s * STAGE_BYTES);
            const uint64_t bdesc = umma_desc(tiles + s * STAGE_BYTES + A_BYTES);
#pragma unroll
            for (int k = 0; k < TC_BK / 16; ++k) umma_bf16(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (i | k) != 0);
            umma_commit(empty0 + 8 * s);
        }
        if (ok && my_kb > 0) umma_commit(acc_full);
    } else if (warp >= 2) {
        // ------------------------------------------------------------- accumulator -> staged float rows
        pdl_wait();
        const int q = warp & 3;
        const int row = q * 32 + lane;
        bool ok = true;
        if (my_kb > 0) ok = mbar_wait(acc_full, 0, &abort_flag, err, TC_ERR_TIMEOUT_EPILOGUE);
        tc_fence_after();
        if (ok) {
            // the ring is drained: every k-slice that was requested has been multiplied
            const uint32_t t_acc = tmem_base + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < TCS_BN / 32; ++c) {
                float v[32];
                if (my_kb > 0) {
                    tmem_load32(t_acc + (uint32_t)(c * 32), v);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0.f;
                }
                if (row < M) {
                    float4* dst = reinterpret_cast<float4*>(stage + (size_t)row * TCS_PITCH + c * 32);
#pragma unroll
                    for (int i = 0; i < 8; ++i) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                }
            }
        }
        tc_fence_before();
    }
    if (warp < 2) pdl_wait();                                     // stores below must follow the previous kernel
    __syncwarp();
    const bool exchange = splits > 1 && !parts;
    if (exchange) cluster.sync(); else __syncthreads();

    // ------------------------------------------------------------------ sum over the cluster, epilogue
    if (parts) {
        // no exchange: this k-slice's sums go to where the consumer of the product adds the slices, a row of the
        // tile per warp and instruction (512 consecutive bytes; stored straight from the registers that hold a
        // row per thread, 16 bytes of 32 different rows an instruction, the same rows took longer: 64 rows
        // 4.8 -> 4.4 and 9.8 -> 9.4 us for the 2,048 x 2,048 and 2,048 x 8,192 matrices, 128 rows 6.2 -> 5.3 and
        // 11.7 -> 10.8)
        float* base = parts + (long long)rank * part_stride + n0;
        const bool vec_ok = (ldc & 3) == 0 && ((reinterpret_cast<uintptr_t>(parts) | (uintptr_t)(part_stride * 4)) & 15) == 0 &&
                            (n0 & 3) == 0;
        for (int row = warp; row < M; row += TC_THREADS / 32) {
            const float4 v = *reinterpret_cast<const float4*>(stage + (size_t)row * TCS_PITCH + lane * 4);
            float* dst = base + (long long)row * ldc + lane * 4;
            if (vec_ok && n0 + lane * 4 + 3 < N) {
                *reinterpret_cast<float4*>(dst) = v;
            } else {
                const float o[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (n0 + lane * 4 + i < N) dst[i] = o[i];
            }
        }
    } else {
        const int col = n0 + (MODE == TC_MODE_SWIGLU ? (lane & 15) * 4 : lane * 4);
        const bool vec_ok = (ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
        constexpr int ROW_STEP = TC_THREADS / 32;
        for (int row0 = rank + splits * warp; row0 < M; row0 += 2 * splits * ROW_STEP) {
          // Two rows' pieces of all ranks are requested before any is added: one round trip through
          // distributed shared memory for both instead of one per row (measured on B200 at 64 rows: q/k/v
          // 9.5 -> 8.3 us, in_proj 10.6 -> 10.1; every row of the warp in one trip needs 168 registers and
          // was slower than the start: 9.9 and 11.4 us); the sums still run in rank order.
          float4 part[2][8];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
              const int row = row0 + h * splits * ROW_STEP;
#pragma unroll
              for (int r = 0; r < 8; ++r) {
                  if (r < splits && row < M) {
                      const float* src = exchange ? cluster.map_shared_rank(stage, r) : stage;
                      part[h][r] = *reinterpret_cast<const float4*>(src + (size_t)row * TCS_PITCH + lane * 4);
                  }
              }
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int row = row0 + h * splits * ROW_STEP;
            if (row >= M) break;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                if (r < splits) {
                    acc.x += part[h][r].x; acc.y += part[h][r].y; acc.z += part[h][r].z; acc.w += part[h][r].w;
                }
            }
            float o[4] = {acc.x, acc.y, acc.z, acc.w};
            if (MODE == TC_MODE_SWIGLU) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float u = rounded<TC>(__shfl_down_sync(0xffffffffu, o[i], 16));
                    const float g = rounded<TC>(o[i]);
                    o[i] = __fdividef(g, 1.f + __expf(-g)) * u;
                }
                if (lane >= 16) continue;
            }
            TC* dst = C + (long long)row * ldc + col;
            if (vec_ok && col + 3 < N) {
                store4(dst, o);
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (col + i < N) dst[i] = from_f32<TC>(o[i]);
            }
          }
        }
    }
    // A block's shared memory must outlive its peers' reads of it.  Nothing is handed over here, so the arrival
    // needs no release (which would wait for this block's stores to the product to be performed): every
    // thread arrives once its own reads have been added up, and waits for the others'.
    if (exchange) {
        asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
    }

    // ------------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (abort_flag && threadIdx.x == 0) {
        const int issued = issued_kb;
        for (int kb = max(0, issued - TCS_STAGES); kb < issued; ++kb) {
            const int s = kb % TCS_STAGES;
            for (int i = 0; i < TC_SPIN_LIMIT; ++i)
                if (mbar_try_wait(full0 + 8 * s, (kb / TCS_STAGES) & 1)) break;
        }
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TCS_BN)
                     : "memory");
    }
}

// Tensor map of the output [M, N] (bfloat16 or float, row pitch ldc elements) for stores of
// 128-row pieces whose rows are 128 bytes, 128-byte swizzle.
template <typename TC>
static int make_map_c(CUtensorMap* map, void* base, long long M, long long N, long long ldc) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        cm_set_error("gemm_tc: cuTensorMapEncodeTiled is not available from this driver");
        return CM_ERR_DRIVER;
    }
    cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
    cuuint64_t strides[1] = {(cuuint64_t)ldc * sizeof(TC)};
    cuuint32_t box[2] = {(cuuint32_t)(128 / sizeof(TC)), TC_BM};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, sizeof(TC) == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base,
                    dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        cm_set_error("gemm_tc: tensor map for the output [%lld, %lld] pitch %lld refused (CUresult %d)", M, N, ldc, (int)r);
        return CM_ERR_DRIVER;
    }
    return CM_OK;
}

template <int BLOCK_N, int STAGES, typename TC, int MODE>
static int launch_tc(void* C, const void* A, const void* B, int M, int N, int K, long long lda, long long ldb,
                     long long ldc, int* err, cudaStream_t st, int ksplit = 1, long long part_stride = 0) {
    CUtensorMap map_a, map_b;
    const long long b_rows = MODE == TC_MODE_SWIGLU ? 2LL * N : N;
    const int b_box = MODE == TC_MODE_SWIGLU ? BLOCK_N / 2 : BLOCK_N;
    int rc = make_map(&map_a, A, M, K, lda, TC_BM);
    if (rc != CM_OK) return rc;
    rc = make_map(&map_b, B, b_rows, K, ldb, b_box);
    if (rc != CM_OK) return rc;
    constexpr int OUT_COLS = MODE == TC_MODE_SWIGLU ? BLOCK_N / 2 : BLOCK_N;
    static_assert(OUT_COLS % (128 / (int)sizeof(TC)) == 0, "a tile is a whole number of staged pieces");
    // TMA stores want a 16-byte aligned base and pitch; other outputs are stored from registers
    CUtensorMap map_c = map_a;
    const int tma_store = ((ldc * (long long)sizeof(TC)) % 16 == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) ? 1 : 0;
    if (tma_store) {
        rc = make_map_c<TC>(&map_c, C, (long long)ksplit * M, N, ldc);      // the runs of a split product lie one below the other
        if (rc != CM_OK) return rc;
    }
    const size_t smem = (size_t)STAGES * (TC_BM * TC_BK * 2 + BLOCK_N * TC_BK * 2) + 2 * 16384 + 1024;
    auto kernel = gemm_tc_kernel<BLOCK_N, STAGES, TC, MODE>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cm_set_error("gemm_tc: %zu bytes of shared memory refused", smem);
            cudaGetLastError();
            return CM_ERR_LAUNCH;
        }
        configured = true;
    }
    const int num_tiles = ((N + OUT_COLS - 1) / OUT_COLS) * ((M + TC_BM - 1) / TC_BM);
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count <= 0) sm_count = 1;
    }
    const int num_items = num_tiles * ksplit;
    dim3 grid(num_items < sm_count ? num_items : sm_count);
    cm_launch(kernel, grid, TCP_THREADS, smem, st, map_a, map_b, map_c, tma_store, (TC*)C, M, N, K, ldc, ksplit,
              part_stride, err);
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// How many clusters of `splits` blocks of this kernel the device runs at once (0: not known).
template <typename TC, int MODE, int A_ROWS, int STAGES>
static int splitk_active_clusters(int splits, size_t smem) {
    static int cached[9] = {-1, -1, -1, -1, -1, -1, -1, -1, -1};
    if (cached[splits] >= 0) return cached[splits];
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(8, splits);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = splits;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_splitk_kernel<TC, MODE, A_ROWS, STAGES>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    cached[splits] = n;
    return n;
}

// Returns CM_OK after a launch, or 1 when the product is better left to the persistent kernel
// (enough column tiles for every SM, or no room for clusters).
template <typename TC, int MODE, int A_ROWS, int STAGES>
static int launch_splitk_rows(void* C, const void* A, const void* B, int M, int N, int K, long long lda, long long ldb,
                         long long ldc, int force_splits, int* err, cudaStream_t st, float* parts = nullptr,
                         long long part_stride = 0) {
    constexpr int OUT_COLS = MODE == TC_MODE_SWIGLU ? TCS_BN / 2 : TCS_BN;
    const size_t smem = (size_t)STAGES * (A_ROWS * TC_BK * 2 + TCS_BN * TC_BK * 2) + 1024;
    auto kernel = gemm_tc_splitk_kernel<TC, MODE, A_ROWS, STAGES>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cm_set_error("gemm_tc: %zu bytes of shared memory refused", smem);
            cudaGetLastError();
            return CM_ERR_LAUNCH;
        }
        configured = true;
    }
    const int n_tiles = (N + OUT_COLS - 1) / OUT_COLS;
    const int num_kb = (K + TC_BK - 1) / TC_BK;
    int splits = 1;
    if (force_splits > 0) {
        splits = force_splits;
    } else {
        // As many blocks as 1.4 per SM (two share an SM; measured on B200 at 64 rows: 16 tiles are
        // fastest split 8 ways, 48 tiles 4 ways, 128 tiles not at all); every block keeps at least
        // four k-slices (with an inner dimension of 1,024, 24 and 17 tiles take 5.6 and 5.3 us split 4 ways,
        // 6.4 and 6.1 us split 8 ways), and the device must have room for such a cluster.
        static int sm_count = 0;
        if (!sm_count) {
            int dev = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
            if (sm_count <= 0) sm_count = 1;
        }
        // With the SwiGLU epilogue the exchange moves gate and up sums (twice the data per output), which pays
        // for fewer rows and blocks only (us, split two ways / unsplit in the persistent kernel): 72 tiles of a
        // 9,216 x 1,024 matrix 8.1 / 9.9 at 32 rows, 9.1 / 10.0 at 64, 12.1 / 10.1 at 128; 128 tiles of a
        // 16,384 x 2,048 matrix 14.6 / 16.0 at 32 rows, 21.4 / 16.2 at 64.
        const int budget = MODE != TC_MODE_SWIGLU ? 7 * sm_count / 5 : M <= 32 ? 2 * sm_count : M <= 64 ? sm_count : sm_count / 4;
        for (int s = MODE == TC_MODE_SWIGLU ? 2 : 8; s >= 2; --s) {       // SwiGLU: two ways at most (four: 10.7 against 7.4 us)
            if (4 * s > num_kb || n_tiles * s > budget) continue;
            if (splitk_active_clusters<TC, MODE, A_ROWS, STAGES>(s, smem) > 0) {
                splits = s;
                break;
            }
        }
        // One block per tile then: the persistent kernel's job, except below 32 rows, where that kernel is a
        // third slower than this one with a single slice (measured on B200, us: SwiGLU over 16,384 x 2,048
        // weights at 24 rows 19.7 against 16.0, the 65,536 x 2,048 head at 17 to 31 rows 66 to 70 against 47
        // to 49; from 32 rows on the two are level or the persistent kernel is ahead).
        // With more tiles than SMs (168 for 148) this kernel's two blocks per SM still lead at 32 to 48 rows
        // (2.6B-class gate/up: 18.9 and 20.2 us against 21.2 and 22.0 in the persistent kernel's wide tiles).
        if (splits == 1 && M >= 32 && (n_tiles <= sm_count || M >= 64)) return 1;
    }
    CUtensorMap map_a, map_b;
    int rc = make_map(&map_a, A, M, K, lda, A_ROWS);
    if (rc != CM_OK) return rc;
    rc = make_map(&map_b, B, MODE == TC_MODE_SWIGLU ? 2LL * N : N, K, ldb, MODE == TC_MODE_SWIGLU ? TCS_BN / 2 : TCS_BN);
    if (rc != CM_OK) return rc;
    // with `parts` the k-slices are independent blocks (no cluster): each leaves its sums in parts[slice]
    cm_launch_cluster(kernel, dim3(n_tiles, splits), TC_THREADS, smem, st, parts ? 1 : splits, true, map_a, map_b, (TC*)C,
                      parts, part_stride, M, N, K, ldc, splits, err);
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// A [M,K] and B [N,K] (2N rows when swiglu) bfloat16, row pitches lda/ldb multiples of 8
// elements, bases 16-byte aligned; C bfloat16 or float.  block_n: 256 (128 x 256 tiles, four
// stages: the most arithmetic per byte moved), 128 (128 x 128 tiles, six stages: twice as
// many tiles, for products with few rows where the number of tiles decides how many SMs stream
// weights) or 192 (plain bfloat16 products whose tiles then fill their rounds over the SMs better).  err: device int, raised by a block whose pipeline wait ran out; may be null.
extern "C" int cm_gemm_tc(int dtc, void* C, const void* A, const void* B, int M, int N, int K, long long lda,
                          long long ldb, long long ldc, int swiglu, int block_n, int* err, cudaStream_t st) {
    if (M <= 0 || N <= 0) return CM_OK;
    if (K <= 0 || K % 8 || lda % 8 || ldb % 8)
        CM_REFUSE("gemm_tc: inner size %d and row pitches %lld, %lld must be multiples of 8", K, lda, ldb);
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15)
        CM_REFUSE("gemm_tc: operands must be 16-byte aligned");
    if (block_n != 128 && block_n != 192 && block_n != 256) CM_REFUSE("gemm_tc: tile width %d (128, 192 or 256)", block_n);
    if (block_n == 192 && (swiglu || dtc != DT_BF16)) CM_REFUSE("gemm_tc: 192-wide tiles are for plain bfloat16 products");
    if (swiglu) {
        if (dtc != DT_BF16) return CM_ERR_DTYPE;
        if (block_n == 256) return launch_tc<256, 4, bf16, TC_MODE_SWIGLU>(C, A, B, M, N, K, lda, ldb, ldc, err, st);
        return launch_tc<128, 6, bf16, TC_MODE_SWIGLU>(C, A, B, M, N, K, lda, ldb, ldc, err, st);
    }
    if (dtc == DT_BF16 && block_n == 256)
        return launch_tc<256, 4, bf16, TC_MODE_PLAIN>(C, A, B, M, N, K, lda, ldb, ldc, err, st);
    if (dtc == DT_BF16 && block_n == 192)
        return launch_tc<192, 4, bf16, TC_MODE_PLAIN>(C, A, B, M, N, K, lda, ldb, ldc, err, st);
    if (dtc == DT_BF16) return launch_tc<128, 6, bf16, TC_MODE_PLAIN>(C, A, B, M, N, K, lda, ldb, ldc, err, st);
    if (dtc == DT_F32) return launch_tc<128, 6, float, TC_MODE_PLAIN>(C, A, B, M, N, K, lda, ldb, ldc, err, st);
    return CM_ERR_DTYPE;
}

// P[r][m][n] = the product over the r-th of `splits` runs of K (each a whole number of 64-wide k-slices),
// float, the runs part_stride = M * N elements apart: the tiled product for shapes with too few output
// tiles to occupy the device (a few hundred rows times a narrow output), with every (run, tile) a work
// item of the persistent kernel and no exchange between blocks; whoever consumes the product adds the
// runs in order (cm_add_norm with m_parts).  block_n as for cm_gemm_tc.
extern "C" int cm_gemm_tc_parts(float* P, const void* A, const void* B, int M, int N, int K, long long lda,
                                long long ldb, int splits, int block_n, int* err, cudaStream_t st) {
    if (M <= 0 || N <= 0) return CM_OK;
    if (K <= 0 || K % 8 || lda % 8 || ldb % 8)
        CM_REFUSE("gemm_tc_parts: inner size %d and row pitches %lld, %lld must be multiples of 8", K, lda, ldb);
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(P)) & 15)
        CM_REFUSE("gemm_tc_parts: operands must be 16-byte aligned");
    if (block_n != 128 && block_n != 256) CM_REFUSE("gemm_tc_parts: tile width %d (128 or 256)", block_n);
    const int num_kb = (K + TC_BK - 1) / TC_BK;
    if (splits < 1 || splits > 8 || (splits - 1) * ((num_kb + splits - 1) / splits) >= num_kb)
        CM_REFUSE("gemm_tc_parts: %d runs over %d k-slices (1 to 8 runs, none empty)", splits, num_kb);
    if (N % 4) CM_REFUSE("gemm_tc_parts: %d output columns (a multiple of 4)", N);
    if ((long long)splits * M > 0x7fffffffLL) CM_REFUSE("gemm_tc_parts: %d runs of %d rows", splits, M);
    const long long part_stride = (long long)M * N;
    if (block_n == 256)
        return launch_tc<256, 4, float, TC_MODE_PLAIN>(P, A, B, M, N, K, lda, ldb, N, err, st, splits, part_stride);
    return launch_tc<128, 6, float, TC_MODE_PLAIN>(P, A, B, M, N, K, lda, ldb, N, err, st, splits, part_stride);
}

template <typename TC, int MODE>
static int launch_splitk(void* C, const void* A, const void* B, int M, int N, int K, long long lda, long long ldb,
                         long long ldc, int force_splits, int* err, cudaStream_t st, float* parts = nullptr,
                         long long part_stride = 0) {
    if (M <= 64)
        return launch_splitk_rows<TC, MODE, 64, 4>(C, A, B, M, N, K, lda, ldb, ldc, force_splits, err, st, parts, part_stride);
    return launch_splitk_rows<TC, MODE, 128, 3>(C, A, B, M, N, K, lda, ldb, ldc, force_splits, err, st, parts, part_stride);
}

// The same product for at most 128 rows, with K split over a thread-block cluster when the
// product has too few column tiles to occupy the device (see gemm_tc_splitk_kernel); otherwise
// it is handed to cm_gemm_tc with 128-column tiles.  splits: 0 to choose, 1..8 to force.
// P[s][m][n] = the product over the s-th of `splits` slices of K, float, the slices part_stride
// elements apart and each [M, N] with row pitch N: the few-rows product without the exchange between
// the blocks of a tile (cm_add_norm with m_parts adds the slices in order).  At most 128 rows.
extern "C" int cm_gemm_tc_few_rows_parts(float* P, const void* A, const void* B, int M, int N, int K, long long lda,
                                         long long ldb, long long part_stride, int splits, int* err, cudaStream_t st) {
    if (M <= 0 || N <= 0) return CM_OK;
    if (M > TC_BM) CM_REFUSE("gemm_tc_few_rows_parts: %d rows (at most %d)", M, TC_BM);
    if (splits < 1 || splits > 8 || 2 * splits > (K + TC_BK - 1) / TC_BK)
        CM_REFUSE("gemm_tc_few_rows_parts: %d slices of an inner size of %d (1 to 8, two 64-wide steps each at least)",
                  splits, K);
    if (K <= 0 || K % 8 || lda % 8 || ldb % 8)
        CM_REFUSE("gemm_tc: inner size %d and row pitches %lld, %lld must be multiples of 8", K, lda, ldb);
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(P)) & 15)
        CM_REFUSE("gemm_tc: operands must be 16-byte aligned");
    return launch_splitk<float, TC_MODE_PLAIN>(nullptr, A, B, M, N, K, lda, ldb, N, splits, err, st, P, part_stride);
}

extern "C" int cm_gemm_tc_few_rows(int dtc, void* C, const void* A, const void* B, int M, int N, int K,
                                   long long lda, long long ldb, long long ldc, int swiglu, int splits, int* err,
                                   cudaStream_t st) {
    if (M <= 0 || N <= 0) return CM_OK;
    if (M > TC_BM) CM_REFUSE("gemm_tc_few_rows: %d rows (at most %d)", M, TC_BM);
    if (splits < 0 || splits > 8) CM_REFUSE("gemm_tc_few_rows: %d splits (0 to 8)", splits);
    if (K <= 0 || K % 8 || lda % 8 || ldb % 8)
        CM_REFUSE("gemm_tc: inner size %d and row pitches %lld, %lld must be multiples of 8", K, lda, ldb);
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15)
        CM_REFUSE("gemm_tc: operands must be 16-byte aligned");
    int rc;
    if (swiglu) {
        if (dtc != DT_BF16) return CM_ERR_DTYPE;
        rc = launch_splitk<bf16, TC_MODE_SWIGLU>(C, A, B, M, N, K, lda, ldb, ldc, splits, err, st);
    } else if (dtc == DT_BF16) {
        rc = launch_splitk<bf16, TC_MODE_PLAIN>(C, A, B, M, N, K, lda, ldb, ldc, splits, err, st);
    } else if (dtc == DT_F32) {
        rc = launch_splitk<float, TC_MODE_PLAIN>(C, A, B, M, N, K, lda, ldb, ldc, splits, err, st);
    } else {
        return CM_ERR_DTYPE;
    }
    if (rc != 1) return rc;
    // The persistent kernel with 128-wide tiles, which put the most SMs to streaming weights, unless they
    // make one round and a fraction: the few tiles of the second round then stream alone, each at one SM's
    // pace.  256-wide tiles run in one round instead (measured on B200, SwiGLU over 21,504 x 2,048 weights,
    // 168 tiles for 148 SMs, 64 rows: 26.3 us against 22.0 us; 40 to 128 rows alike).
    int sm_count = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    const int out_cols = swiglu ? 64 : 128;
    const int tiles = (N + out_cols - 1) / out_cols;
    const int width = (dtc == DT_BF16 && sm_count > 0 && tiles > sm_count && tiles <= 2 * sm_count) ? 256 : 128;
    return cm_gemm_tc(dtc, C, A, B, M, N, K, lda, ldb, ldc, swiglu, width, err, st);
}
