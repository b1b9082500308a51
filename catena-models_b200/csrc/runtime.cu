// Library-wide pieces: the last refusal message, small cache-maintenance kernels.
#include "common.cuh"
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

static thread_local char g_last_error[512] = "";

void cm_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
}

extern "C" const char* cm_last_error() { return g_last_error; }

// The compiled value of a limit of cm_limits.h by its name without the CM_ prefix; -1 if unknown.
extern "C" long long cm_limit(const char* name) {
    struct Entry { const char* name; long long value; };
    static const Entry table[] = {
        {"PAGE_TOKENS", CM_PAGE_TOKENS},       {"ATTN_DECODE_CHUNK", CM_ATTN_DECODE_CHUNK},
        {"NORM_MAX_WIDTH", CM_NORM_MAX_WIDTH}, {"MAX_HEAD_DIM", CM_MAX_HEAD_DIM},
        {"MAX_CONV_TAPS", CM_MAX_CONV_TAPS},   {"SKINNY_MAX_ROWS", CM_SKINNY_MAX_ROWS},
        {"FEW_ROWS_MAX_ROWS", CM_FEW_ROWS_MAX_ROWS},
    };
    for (const Entry& e : table)
        if (strcmp(e.name, name) == 0) return e.value;
    return -1;
}

static int g_pdl = 1;
int cm_pdl_enabled() { return g_pdl; }
// 1 (default): kernels are launched so that the next one may start while they run (see
// common.cuh); 0: plain stream order.
extern "C" void cm_set_pdl(int on) { g_pdl = on ? 1 : 0; }

// table[index[i]] = value[i] for i < *count (count lives on the device so that a captured
// graph can carry a different number of page-table updates on every replay).
__global__ void scatter_i32_kernel(int* __restrict__ table, const int* __restrict__ index,
                                   const int* __restrict__ value, const int* __restrict__ count,
                                   int max_count) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int n = min(*count, max_count);
    if (i < n) table[index[i]] = value[i];
}

extern "C" int cm_scatter_i32(int* table, const int* index, const int* value, const int* count,
                              int max_count, cudaStream_t st) {
    if (max_count <= 0) return CM_OK;
    cm_launch(scatter_i32_kernel, (max_count + 127) / 128, 128, 0, st, table, index, value, count, max_count);
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// Clears the fixed-size state of newly admitted slots: x is [layers][slots][row_words] 32-bit
// words, and row slot_ids[i] of every layer is set to zero.  The slot ids travel as a kernel
// argument (up to ZS_MAX per launch), so admitting sequences costs no copy to the device.
#define ZS_MAX 64
struct ZeroSlots {
    int id[ZS_MAX];
};

__global__ void zero_slots_kernel(uint32_t* __restrict__ x, long long slots, long long row_words, ZeroSlots ids) {
    pdl_trigger();
    pdl_wait();
    uint32_t* dst = x + ((long long)blockIdx.y * slots + ids.id[blockIdx.x]) * row_words;
    for (long long c = threadIdx.x; c < row_words; c += blockDim.x) dst[c] = 0u;
}

extern "C" int cm_zero_slots(void* x, int layers, long long slots, long long row_bytes, const int* slot_ids, int n,
                             cudaStream_t st) {
    if (n <= 0 || layers <= 0 || row_bytes <= 0) return CM_OK;
    if (row_bytes % 4 || (reinterpret_cast<uintptr_t>(x) & 3)) CM_REFUSE("zero_slots: rows of %lld bytes (multiples of 4)", row_bytes);
    if (layers > 65535) CM_REFUSE("zero_slots: %d layers", layers);
    for (int i = 0; i < n; ++i)
        if (slot_ids[i] < 0 || slot_ids[i] >= slots) CM_REFUSE("zero_slots: slot %d of %lld", slot_ids[i], slots);
    for (int first = 0; first < n; first += ZS_MAX) {
        ZeroSlots ids;
        const int count = n - first < ZS_MAX ? n - first : ZS_MAX;
        for (int i = 0; i < count; ++i) ids.id[i] = slot_ids[first + i];
        cm_launch(zero_slots_kernel, dim3(count, layers), 256, 0, st, (uint32_t*)x, slots, row_bytes / 4, ids);
        CM_CHECK_LAUNCH();
    }
    return CM_OK;
}

// Copies whole pages inside a paged pool [outer, pages, page_bytes]: page src[i] to page dst[i] for
// every outer index (layer and key/value plane).  Used to give a resumed sequence its own copy of a
// checkpointed one (catena-models copies session buffers with its copy-buffer kernel,
// src/model.rs:208-246).  page_bytes is a multiple of 16; src and dst pages do not overlap.
__global__ void copy_pages_kernel(uint4* __restrict__ pool, const int* __restrict__ src, const int* __restrict__ dst,
                                  long long pages, long long page_vec) {
    pdl_trigger();
    pdl_wait();
    const long long plane = (long long)blockIdx.y * pages;
    const uint4* from = pool + (plane + src[blockIdx.x]) * page_vec;
    uint4* to = pool + (plane + dst[blockIdx.x]) * page_vec;
    for (long long i = threadIdx.x; i < page_vec; i += blockDim.x) to[i] = from[i];
}

extern "C" int cm_copy_pages(void* pool, const int* src, const int* dst, int n, int outer, long long pages,
                             long long page_bytes, cudaStream_t st) {
    if (n <= 0 || outer <= 0) return CM_OK;
    if (page_bytes % 16 || (reinterpret_cast<uintptr_t>(pool) & 15))
        CM_REFUSE("copy_pages: pages of %lld bytes (multiples of 16, 16-byte aligned pool)", page_bytes);
    if (outer > 65535) CM_REFUSE("copy_pages: %d planes", outer);
    cm_launch(copy_pages_kernel, dim3(n, outer), 256, 0, st, (uint4*)pool, src, dst, pages, page_bytes / 16);
    CM_CHECK_LAUNCH();
    return CM_OK;
}
