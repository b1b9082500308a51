// A run of decode-step operations in ONE persistent kernel (bfloat16, at most 16 rows).
//
// A decode step of a small batch is a chain of about 170 short dependent kernels, each of which
// streams a few megabytes of weights: every one of them ramps its memory pipeline up from nothing
// and drains it before the next starts, and the step reaches half of the copy bandwidth although
// its large products reach 80 % alone.  Here a segment of that chain (matrix products with their
// epilogues, the fused residual + norm kernel, the short convolution's decode form) is one
// cooperative launch of resident blocks.  Between two operations the blocks meet at a barrier in
// global memory; but the WEIGHTS of the operations ahead do not depend on any activation, so every
// block keeps requesting its share of them (cp.async into a ring in shared memory, in the order in
// which it will use them) while it waits, adds up its sums or writes its outputs.  The stream of
// weights from HBM therefore does not stop at the borders between operations.
//
//   one block of 512 threads per SM, four groups of 4 warps in each; group v of V handles the work
//   items v, v + V, v + 2V, ... of every operation, in order, and has a ring of its own (8 stages);
//   a product's work item = 16 rows of W (a "tile") x one of `ksplit` slices of K, cut into stages
//   of 16 rows x 128 values of k (4 KB); a group's 4 warps take 32 values of k of a stage each and
//   multiply them with mma.sync.m16n8k16 (weights as the 16-row operand, the <= 8 * NT activation
//   rows as the 8-wide one, float sums), then add their sums through shared memory in warp order;
//   a product's activations are read with ordinary loads (from L1 after the first touch: the acquire
//   at the barrier has dropped whatever L1 held before another block wrote them), everything else
//   that another block wrote during this launch with ld.global.cg.
//
// Measured on B200 (LFM3 1.7B-class, decode at batch 8, 2,048 tokens of context): 37 launches a step
// instead of 173, but 1.53 ms a step against 1.13 ms for the chain of single kernels replayed from a
// graph.  A barrier phase costs as much as a kernel boundary (3.2 us for the residual + norm
// operation, of which 0.8 us the fence and the arrival and 0.5 us the wait), and the ring does not
// hide it: a group's loop over 4 KB stages (two barriers of its four warps, two shared-memory
// reads, two mma) sustains about 11 KB/us, so a product whose items keep 65 % of the groups busy
// streams at 2.4 TB/s (in_proj), one that keeps all busy at 4.4 TB/s (gate and up), where the single
// kernels reach 3.6 and 4.8.  Earlier forms were slower still, for reasons worth knowing: with 64
// registers a thread (1,024 threads a block) the spills went to an L1 that the 200 KB of rings had
// left almost nothing of, and every phase took 8 us; activations read through L2 with ld.global.cg
// queued behind the 128 KB of weights that each SM has on its way, and a stage took 0.7 us.
// The engine therefore uses this kernel only on request (CATENA_B200_FUSED_DECODE=1).
//
// Every order of summation is fixed (k within a warp, warps in index order, slices of K by their
// consumer in slice order), so a row's result does not depend on what else the batch holds.
// Every wait on the barrier is bounded: a block that gives up raises *err, stops taking part and
// returns, and the others run into their own limits; nothing spins for ever.
#include "common.cuh"
#include "decode_fused.h"
#include <cooperative_groups.h>

#define FD_SUBS 4                      // groups of 4 warps per block, each with work items and a ring of its own
#define FD_SUB_THREADS 128
#define FD_THREADS (FD_SUBS * FD_SUB_THREADS)     // 512 threads, one block per SM: up to 128 registers a thread
#define FD_WARPS 4                     // warps of a group
#define FD_STAGE_K 128                 // values of k per stage
#define FD_ROWS 16                     // rows of W per stage
#define FD_PITCH 160                   // elements between rows of a stage in shared memory (320 bytes: no bank conflicts)
#define FD_STAGES 8
#define FD_XAHEAD 2                    // k-stages of activations requested ahead of their use
#define FD_RING_BYTES (FD_STAGES * FD_ROWS * FD_PITCH * 2)
#define FD_SPIN_LIMIT (1u << 22)       // polls of the barrier word (of the order of a second) before a block gives up

__device__ __forceinline__ void fd_cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;                 // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void fd_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void fd_mma(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned fd_load_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 fd_lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
// the threads of group `sub` meet (hardware barrier 1 + sub; barrier 0 is the whole block's)
__device__ __forceinline__ void fd_sub_sync(int sub) {
    asm volatile("bar.sync %0, %1;" ::"r"(sub + 1), "n"(FD_SUB_THREADS) : "memory");
}
template <typename T>
__device__ __forceinline__ void fd_load8_cg(const T* p, float* out);          // eight values through L2
template <>
__device__ __forceinline__ void fd_load8_cg<bf16>(const bf16* p, float* out) {
    const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(p));
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
    }
}
template <>
__device__ __forceinline__ void fd_load8_cg<float>(const float* p, float* out) {
    const float4 a = __ldcg(reinterpret_cast<const float4*>(p)), b = __ldcg(reinterpret_cast<const float4*>(p + 4));
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w; out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
// ---- the geometry of a product's work items, worked out once per operation ------------------------
struct FdShape {
    int tiles;            // groups of 16 rows of the output
    int per_slice;        // stages per slice of K
    int items;            // tiles x ksplit (0 for operations that stream no weights)
    int stages;           // stages of one item (twice per_slice for SwiGLU: gate and up alternate)
};

// A group's stream of weights: the stages of its items, operation after operation, in the order of use.
struct FdStream {
    int op, item, stage, stages;       // position; stages of the current item
    const bf16* base0;                 // this thread's first source address of the item
    const bf16* base1;                 // the same in the second half of the matrix (SwiGLU: the up rows)
    int k, kend;                       // this thread's k of the next stage; end of the row
    int row_ok;                        // bit (2 * half + chunk): that row of the thread exists
    long long row8;                    // 8 rows further on, in elements
    int swiglu;
};

template <int NT>
__global__ void __launch_bounds__(FD_THREADS, 1)
fused_decode_kernel(const __grid_constant__ FdSegment seg, unsigned* __restrict__ bar, int* __restrict__ err) {
    extern __shared__ __align__(16) uint8_t fd_smem[];
    __shared__ FdShape shape[FD_MAX_OPS];
    __shared__ FdOp ops[FD_MAX_OPS];            // the table, copied out of the parameters once: read many times
    __shared__ float scratch[32];
    __shared__ int gave_up;
    const int tid = threadIdx.x & (FD_SUB_THREADS - 1), sub = threadIdx.x / FD_SUB_THREADS;
    const int lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int V = gridDim.x * FD_SUBS, vb = blockIdx.x * FD_SUBS + sub;       // groups in all, this group
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(fd_smem) + sub * FD_RING_BYTES;
    float* red = reinterpret_cast<float*>(fd_smem + FD_SUBS * FD_RING_BYTES) + sub * (2 * FD_WARPS * NT * 128);
    if (threadIdx.x == 0) gave_up = 0;
    const int n_ops = seg.n_ops;
    for (int i = threadIdx.x; i < n_ops * (int)(sizeof(FdOp) / 4); i += FD_THREADS)
        reinterpret_cast<int*>(ops)[i] = reinterpret_cast<const int*>(seg.op)[i];
    if (threadIdx.x < n_ops) {
        const FdOp& op = seg.op[threadIdx.x];
        FdShape s = {0, 0, 0, 0};
        if (op.kind == FD_KIND_GEMV) {
            s.tiles = (op.N + FD_ROWS - 1) / FD_ROWS;
            const int total = (op.K + FD_STAGE_K - 1) / FD_STAGE_K;
            s.per_slice = (total + op.ksplit - 1) / op.ksplit;
            s.items = s.tiles * op.ksplit;
            s.stages = op.mode == FD_MODE_SWIGLU ? 2 * s.per_slice : s.per_slice;
        }
        shape[threadIdx.x] = s;
    }
    __syncthreads();

    // ---- producer ------------------------------------------------------------------------------
    // chunk u of a thread: row (tid >> 4) + 8u of the stage, columns (tid & 15) * 8 ..
    const int p_row = tid >> 4, p_col = (tid & 15) * 8;
    const uint32_t p_dst = ring + (p_row * FD_PITCH + p_col) * 2;
    FdStream ps;
    ps.op = -1;
    ps.item = 0;
    ps.stage = ps.stages = 0;
    int issued = 0, consumed = 0;
    auto next_item = [&]() {              // false when the stream has ended
        for (;;) {
            if (ps.op >= 0 && ps.op < n_ops) {
                ps.item += V;
                if (ps.item < shape[ps.op].items) break;
            }
            if (++ps.op >= n_ops) return false;
            ps.item = vb - V;             // the += V above makes it vb
        }
        const FdOp& op = ops[ps.op];
        const FdShape s = shape[ps.op];
        const int tile = ps.item % s.tiles, slice = ps.item / s.tiles;
        ps.swiglu = op.mode == FD_MODE_SWIGLU;
        ps.stage = 0;
        ps.stages = s.stages;
        ps.k = slice * s.per_slice * FD_STAGE_K + p_col;
        ps.kend = op.K;
        ps.row8 = 8 * op.ldw;
        const int r = tile * FD_ROWS + p_row;
        const bf16* W = reinterpret_cast<const bf16*>(op.w);
        ps.base0 = W + (long long)r * op.ldw;
        ps.base1 = W + (long long)(op.N + r) * op.ldw;
        const int ok = (r < op.N ? 1 : 0) | (r + 8 < op.N ? 2 : 0);
        ps.row_ok = ok | (ps.swiglu ? ok << 2 : 0);
        return true;
    };
    bool stream_live = next_item();
    auto fill = [&]() {                   // keep the ring full; every round commits one group (empty at the end)
        while (issued - consumed < FD_STAGES) {
            if (stream_live) {
                const int half = ps.swiglu & ps.stage;
                const bool kv = ps.k < ps.kend;
                const bf16* src = (half ? ps.base1 : ps.base0) + ps.k;
                const uint32_t dst = p_dst + (issued & (FD_STAGES - 1)) * (FD_ROWS * FD_PITCH * 2);
                const int ok = ps.row_ok >> (2 * half);
                const bool v0 = kv && (ok & 1), v1 = kv && (ok & 2);
                fd_cp_async16(dst, v0 ? src : ps.base0, v0);
                fd_cp_async16(dst + 8 * FD_PITCH * 2, v1 ? src + ps.row8 : ps.base0, v1);
                if (!ps.swiglu || half) ps.k += FD_STAGE_K;
                if (++ps.stage == ps.stages) stream_live = next_item();
            }
            fd_commit();
            ++issued;
        }
    };
    fill();

    const uint32_t c_src = ring + (g * FD_PITCH + warp * 32 + t * 8) * 2;      // this thread's fragment of a stage
    unsigned target = 0;
    for (int o = 0; o < n_ops; ++o) {
        const FdOp& op = ops[o];
        // ---- wait for the operation before this one (the first one's inputs come from earlier kernels)
        if (o > 0) {
            if (threadIdx.x == 0) {
                unsigned spins = 0;
                while (fd_load_acquire(bar) < target) {
                    if (++spins > FD_SPIN_LIMIT) {
                        atomicExch(err, 7);
                        gave_up = 1;
                        break;
                    }
                }
            }
            __syncthreads();
            if (gave_up) break;
        }
        if (op.kind == FD_KIND_GEMV) {
            const FdShape s = shape[o];
            const bool swiglu = op.mode == FD_MODE_SWIGLU;
            const bf16* X = reinterpret_cast<const bf16*>(op.x);
            const int M = op.M, K = op.K;
            for (int item = vb; item < s.items; item += V) {
                const int tile = item % s.tiles, slice = item / s.tiles;
                float acc[2][NT][4];
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int n = 0; n < NT; ++n)
#pragma unroll
                        for (int j = 0; j < 4; ++j) acc[h][n][j] = 0.f;
                // Activations are read without a predicate: a row past M repeats row 0 and its result is
                // dropped, a k past K is pulled back inside the row and meets weights that were zero-filled.
                // (A load whose value goes through a select would be waited for at once, stage after stage.)
                int k = slice * s.per_slice * FD_STAGE_K + warp * 32 + t * 8;
                const int k_last = K - 8;
                const bf16* xrow[NT];
#pragma unroll
                for (int n = 0; n < NT; ++n) xrow[n] = X + (long long)(n * 8 + g < M ? n * 8 + g : 0) * op.ldx;
                // The activations of the next FD_XAHEAD k-stages are on their way while one is multiplied.  They
                // are read with ordinary loads: the groups of an SM read the same rows again and again, and
                // from L1 these reads do not queue behind the weights that are on their way.  (The acquire
                // at the barrier has dropped whatever L1 held before another block wrote these rows.)
                uint4 xq[FD_XAHEAD][NT];
#pragma unroll
                for (int a = 0; a < FD_XAHEAD; ++a)
#pragma unroll
                    for (int n = 0; n < NT; ++n)
                        xq[a][n] = *reinterpret_cast<const uint4*>(xrow[n] + min(k + a * FD_STAGE_K, k_last));
                k += FD_XAHEAD * FD_STAGE_K;
                const int halves = swiglu ? 2 : 1;
                for (int ks = 0; ks < s.per_slice; ++ks) {
                    uint4 xv[NT], xn[NT];
#pragma unroll
                    for (int n = 0; n < NT; ++n) {
                        xv[n] = xq[0][n];
                        xn[n] = *reinterpret_cast<const uint4*>(xrow[n] + min(k, k_last));
                    }
                    k += FD_STAGE_K;
                    for (int half = 0; half < halves; ++half) {
                        asm volatile("cp.async.wait_group %0;" ::"n"(FD_STAGES - 1) : "memory");
                        fd_sub_sync(sub);
                        const uint32_t src = c_src + (consumed & (FD_STAGES - 1)) * (FD_ROWS * FD_PITCH * 2);
                        const uint4 wa = fd_lds128(src), wb = fd_lds128(src + 8 * FD_PITCH * 2);
                        fd_sub_sync(sub);                     // every warp has its fragments: the slot may be refilled
                        ++consumed;
                        fill();
#pragma unroll
                        for (int n = 0; n < NT; ++n) {
                            if (half == 0) {
                                fd_mma(acc[0][n], wa.x, wb.x, wa.y, wb.y, xv[n].x, xv[n].y);
                                fd_mma(acc[0][n], wa.z, wb.z, wa.w, wb.w, xv[n].z, xv[n].w);
                            } else {
                                fd_mma(acc[1][n], wa.x, wb.x, wa.y, wb.y, xv[n].x, xv[n].y);
                                fd_mma(acc[1][n], wa.z, wb.z, wa.w, wb.w, xv[n].z, xv[n].w);
                            }
                        }
                    }
#pragma unroll
                    for (int n = 0; n < NT; ++n) {
#pragma unroll
                        for (int a = 0; a + 1 < FD_XAHEAD; ++a) xq[a][n] = xq[a + 1][n];
                        xq[FD_XAHEAD - 1][n] = xn[n];
                    }
                }
                // ---- the warps' sums, added in warp order
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        red[((0 * FD_WARPS + warp) * NT + n) * 128 + lane * 4 + j] = acc[0][n][j];
                        if (swiglu) red[((1 * FD_WARPS + warp) * NT + n) * 128 + lane * 4 + j] = acc[1][n][j];
                    }
                fd_sub_sync(sub);
                for (int e = tid; e < NT * 128; e += FD_SUB_THREADS) {
                    const int n = e >> 7, l = (e >> 2) & 31, j = e & 3;
                    const int row = tile * FD_ROWS + (l >> 2) + (j >= 2 ? 8 : 0);
                    const int m = n * 8 + (l & 3) * 2 + (j & 1);
                    float s0 = 0.f, s1 = 0.f;
#pragma unroll
                    for (int w = 0; w < FD_WARPS; ++w) s0 += red[((0 * FD_WARPS + w) * NT + n) * 128 + l * 4 + j];
                    if (swiglu) {
#pragma unroll
                        for (int w = 0; w < FD_WARPS; ++w) s1 += red[((1 * FD_WARPS + w) * NT + n) * 128 + l * 4 + j];
                    }
                    if (row >= op.N || m >= M) continue;
                    if (op.mode == FD_MODE_PLAIN) {
                        reinterpret_cast<bf16*>(op.y)[(long long)m * op.ldy + row] = __float2bfloat16_rn(s0);
                    } else if (op.mode == FD_MODE_SWIGLU) {
                        const float gr = rounded<bf16>(s0), ur = rounded<bf16>(s1);
                        reinterpret_cast<bf16*>(op.y)[(long long)m * op.ldy + row] = __float2bfloat16_rn((gr * sigmoid_f32(gr)) * ur);
                    } else if (op.mode == FD_MODE_PARTS) {
                        reinterpret_cast<float*>(op.y)[(long long)slice * op.part_stride + (long long)m * op.ldy + row] = s0;
                    } else {
                        reinterpret_cast<float*>(op.y)[(long long)m * op.ldy + row] = s0;
                    }
                }
                fd_sub_sync(sub);                             // red is written again by the next item
            }
        } else if (op.kind == FD_KIND_ADD_NORM) {
            // h_out = h_in + (norm(m; w_post) or m); n_out = norm(h_out; w_next).  One block per row, the row
            // in registers (H <= 8 * 512), as rowwise.cu's add_norm kernel does it.
            const int H = op.N;
            const bf16* h_in = reinterpret_cast<const bf16*>(op.x);
            bf16* h_out = reinterpret_cast<bf16*>(op.y);
            bf16* n_out = reinterpret_cast<bf16*>(op.aux3);
            const float* w_post = reinterpret_cast<const float*>(op.aux1);
            const float* w_next = reinterpret_cast<const float*>(op.aux2);
            for (int row = blockIdx.x; row < op.M; row += gridDim.x) {
                const long long off = (long long)row * H;
                const int e = threadIdx.x * 8;
                float mv[8], hv[8], wp[8], wn[8];
                float ss = 0.f;
                if (e < H) {
                    if (w_post) load8f<float>(w_post + e, wp);        // requested with the row, used after the sums
                    if (w_next) load8f<float>(w_next + e, wn);
                    if (op.n_parts > 0) {
                        const float* parts = reinterpret_cast<const float*>(op.aux0);
#pragma unroll
                        for (int i = 0; i < 8; ++i) mv[i] = 0.f;
                        for (int r = 0; r < op.n_parts; ++r) {
                            float p[8];
                            fd_load8_cg<float>(parts + (long long)r * op.part_stride + off + e, p);
#pragma unroll
                            for (int i = 0; i < 8; ++i) mv[i] += p[i];
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i) mv[i] = rounded<bf16>(mv[i]);
                    } else {
                        fd_load8_cg<bf16>(reinterpret_cast<const bf16*>(op.aux0) + off + e, mv);
                    }
                    fd_load8_cg<bf16>(h_in + off + e, hv);
#pragma unroll
                    for (int i = 0; i < 8; ++i) ss += mv[i] * mv[i];
                }

                float inv_post = 1.f;
                if (w_post) {

                    ss = block_sum(ss, scratch);
                    inv_post = 1.f / sqrtf(ss / (float)H + op.eps0);
                }

                float ss2 = 0.f;
                if (e < H) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float d = w_post ? rounded<bf16>((mv[i] * inv_post) * wp[i]) : mv[i];
                        hv[i] = rounded<bf16>(hv[i] + d);
                        ss2 += hv[i] * hv[i];
                    }
                    store8f<bf16>(h_out + off + e, hv);
                }

                if (w_next) {
                    ss2 = block_sum(ss2, scratch);

                    const float inv_next = 1.f / sqrtf(ss2 / (float)H + op.eps1);
                    if (e < H) {
                        float o8[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) o8[i] = (hv[i] * inv_next) * wn[i];
                        store8f<bf16>(n_out + off + e, o8);
                    }
                }

            }
        } else if (op.kind == FD_KIND_CONV) {
            // The short convolution's decode form (one token per sequence): bcx [M][B | C | X] bfloat16,
            //   bx = B * X; z = sum_j taps[c][j] * s[j], s = (state[0 .. KT-2], bx); y = T(z * C); state <- s[1 ..]
            // eight channels of one sequence per thread.
            const int H = op.N, KT = op.taps, groups = H / 8;
            const bf16* bcx = reinterpret_cast<const bf16*>(op.x);
            const float* taps = reinterpret_cast<const float*>(op.aux0);
            float* state = reinterpret_cast<float*>(op.aux3);
            bf16* y = reinterpret_cast<bf16*>(op.y);
            for (int idx = blockIdx.x * FD_THREADS + threadIdx.x; idx < op.M * groups; idx += gridDim.x * FD_THREADS) {
                const int m = idx / groups, c = (idx - m * groups) * 8;
                float bb[8], cc[8], xx[8], z[8], bx[8];
                fd_load8_cg<bf16>(bcx + (long long)m * op.ldx + c, bb);
                fd_load8_cg<bf16>(bcx + (long long)m * op.ldx + H + c, cc);
                fd_load8_cg<bf16>(bcx + (long long)m * op.ldx + 2 * H + c, xx);
                float* st = state + (long long)op.idx[m] * (KT - 1) * H + c;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    bx[i] = bb[i] * xx[i];
                    z[i] = 0.f;
                }
                for (int q = 0; q < KT - 1; ++q) {
                    float sv[8];
                    fd_load8_cg<float>(st + (long long)q * H, sv);
#pragma unroll
                    for (int i = 0; i < 8; ++i) z[i] += taps[(long long)(c + i) * KT + q] * sv[i];
                    if (q > 0) store8f<float>(st + (long long)(q - 1) * H, sv);
                }
                float out[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    z[i] += taps[(long long)(c + i) * KT + KT - 1] * bx[i];
                    out[i] = z[i] * cc[i];
                }
                store8f<float>(st + (long long)(KT - 2) * H, bx);
                store8f<bf16>(y + (long long)m * op.ldy + c, out);
            }
        }
        // ---- this block is done with operation o
        __syncthreads();
        target += gridDim.x;
        if (threadIdx.x == 0) {
            __threadfence();
            const unsigned seen = atomicAdd(bar, 1u) + 1u;
            // the last arrival of the last operation leaves the word as the next launch expects it
            if (o == n_ops - 1 && seen == target) atomicExch(bar, 0u);
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");     // nothing of this block may still be on its way
}

static int g_fd_blocks[3] = {0, 0, 0};                        // resident blocks per launch, by NT (0: not asked yet)
static size_t fd_smem_bytes(int NT) {
    return (size_t)FD_SUBS * (FD_RING_BYTES + (size_t)2 * FD_WARPS * NT * 128 * sizeof(float));
}

template <int NT>
static int fd_launch(const FdSegment* seg, unsigned* bar, int* err, cudaStream_t st) {
    const size_t smem = fd_smem_bytes(NT);
    auto kernel = fused_decode_kernel<NT>;
    if (!g_fd_blocks[NT]) {
        int dev = 0, sms = 0, per_sm = 0;
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
            cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, FD_THREADS, smem) != cudaSuccess || per_sm < 1) {
            cudaGetLastError();
            CM_REFUSE("fused_decode: the device cannot hold the kernel's blocks");
        }
        g_fd_blocks[NT] = sms * per_sm;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(g_fd_blocks[NT]);
    cfg.blockDim = dim3(FD_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;              // all blocks resident at once, or the launch fails
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kernel, *seg, bar, err);
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// seg: the operations (host memory; copied into the launch).  bar: a device word that is 0 before the
// first launch and is left at 0 by every launch that ends normally.  err: the device flag a block
// raises (value 7) when its wait at the barrier runs out.
extern "C" int cm_fused_decode(const FdSegment* seg, unsigned* bar, int* err, cudaStream_t st) {
    if (!seg || seg->n_ops <= 0) return CM_OK;
    if (seg->n_ops > FD_MAX_OPS) CM_REFUSE("fused_decode: %d operations (at most %d)", seg->n_ops, FD_MAX_OPS);
    int rows = 0;
    for (int i = 0; i < seg->n_ops; ++i) {
        const FdOp& op = seg->op[i];
        rows = op.M > rows ? op.M : rows;
        if (op.M < 1 || op.M > 16) CM_REFUSE("fused_decode: operation %d has %d rows (1 to 16)", i, op.M);
        if (op.kind == FD_KIND_GEMV) {
            if (op.K <= 0 || op.K % 8 || op.ldx % 8 || op.ldw % 8 || op.N <= 0 || op.ksplit < 1 || op.ksplit > 8)
                CM_REFUSE("fused_decode: product %d: %d x %d, strides %lld, %lld, %d slices", i, op.N, op.K, op.ldx, op.ldw,
                          op.ksplit);
            if (((uintptr_t)op.x | (uintptr_t)op.w) & 15) CM_REFUSE("fused_decode: product %d: operands must be 16-byte aligned", i);
            if (op.ksplit > 1 && op.mode != FD_MODE_PARTS) CM_REFUSE("fused_decode: product %d: slices of K need partial sums", i);
            if (op.mode < 0 || op.mode > FD_MODE_F32) CM_REFUSE("fused_decode: product %d: mode %d", i, op.mode);
        } else if (op.kind == FD_KIND_ADD_NORM) {
            if (op.N % 8 || op.N > 8 * FD_THREADS) CM_REFUSE("fused_decode: add_norm %d: width %d (multiples of 8 up to %d)", i, op.N, 8 * FD_THREADS);
            if (op.n_parts < 0 || op.n_parts > 8 || op.part_stride % 4) CM_REFUSE("fused_decode: add_norm %d: %d partial sums", i, op.n_parts);
            if (((uintptr_t)op.x | (uintptr_t)op.y | (uintptr_t)op.aux0 | (uintptr_t)op.aux1 | (uintptr_t)op.aux2 | (uintptr_t)op.aux3) & 15)
                CM_REFUSE("fused_decode: add_norm %d: operands must be 16-byte aligned", i);
        } else if (op.kind == FD_KIND_CONV) {
            if (op.N % 8 || op.ldx % 8 || op.ldy % 8 || op.taps < 2 || op.taps > CM_MAX_CONV_TAPS)
                CM_REFUSE("fused_decode: convolution %d: width %d, %d taps", i, op.N, op.taps);
            if (((uintptr_t)op.x | (uintptr_t)op.y | (uintptr_t)op.aux3) & 15)
                CM_REFUSE("fused_decode: convolution %d: operands must be 16-byte aligned", i);
        } else {
            CM_REFUSE("fused_decode: operation %d of unknown kind %d", i, op.kind);
        }
    }
    if (rows <= 8) return fd_launch<1>(seg, bar, err, st);
    return fd_launch<2>(seg, bar, err, st);
}

extern "C" int cm_fused_decode_max_ops() { return FD_MAX_OPS; }
extern "C" int cm_fused_decode_max_width() { return 8 * FD_THREADS; }
