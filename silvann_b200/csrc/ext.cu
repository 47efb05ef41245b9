/* ext.cu — the `silvann_b200_*` entry points declared in include/silvann_b200.h: argument checks in the manner of the
 * engine's verbs (bounds first, then the launch: engine/src/packages/nn/cpu/opcodes/attention__abi.cuh:145-150), the
 * paged-decode planner, and the counters. */
#include "../../include/silvann_b200.h"
#include "common.cuh"
#include "kernels.h"
#include "kernels_deltanet.h"
#include <atomic>
#include <algorithm>
#include <vector>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

namespace svf {
extern std::atomic<uint64_t> g_counters[SILVANN_B200_COUNTERS];
void flush();
}

#define SV_EXPORT extern "C" __attribute__((visibility("default")))

static thread_local char t_error[256];
static int fail(int code, const char* fmt, ...) {
    va_list ap; va_start(ap, fmt); vsnprintf(t_error, sizeof t_error, fmt, ap); va_end(ap);
    return code;
}
/* the same for the library's other translation units (tier.cu) */
int sv_ext_fail(int code, const char* fmt, ...) {
    va_list ap; va_start(ap, fmt); vsnprintf(t_error, sizeof t_error, fmt, ap); va_end(ap);
    return code;
}
static int cuda_fail(const char* what, cudaError_t e) {
    (void)cudaGetLastError();
    return fail(SILVANN_B200_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
}
static inline void called() { svf::g_counters[SILVANN_B200_COUNTER_EXT_CALLS].fetch_add(1, std::memory_order_relaxed); }
static inline bool dtype_ok(int dt) { return dt == SILVANN_B200_DTYPE_FP16 || dt == SILVANN_B200_DTYPE_BF16; }

SV_EXPORT const char* silvann_b200_last_error(void) { return t_error; }

SV_EXPORT int silvann_b200_counters_read(uint64_t* out, uint32_t n, int reset) {
    if (!out) return fail(SILVANN_B200_E_ARGUMENT, "counters_read: out is null");
    for (uint32_t i = 0; i < n && i < SILVANN_B200_COUNTERS; ++i)
        out[i] = reset ? svf::g_counters[i].exchange(0) : svf::g_counters[i].load();
    return SILVANN_B200_OK;
}

SV_EXPORT int silvann_b200_device_status(uint32_t* word, int clear) {
    if (!word) return fail(SILVANN_B200_E_ARGUMENT, "device_status: word is null");
    unsigned int* dev = sv::device_status_word();
    if (!dev) return fail(SILVANN_B200_E_CUDA, "device_status: no status word on this device");
    cudaError_t e = cudaStreamSynchronize(0);
    if (e != cudaSuccess) return cuda_fail("device_status: wait", e);
    unsigned int w = 0;
    if ((e = cudaMemcpy(&w, dev, sizeof w, cudaMemcpyDeviceToHost)) != cudaSuccess) return cuda_fail("device_status: read", e);
    if (clear && w != 0u && (e = cudaMemset(dev, 0, sizeof w)) != cudaSuccess) return cuda_fail("device_status: clear", e);
    unsigned int w_static = 0;                    /* silvann_b200_decode_noalloc keeps its own word in its fixed array */
    if ((e = sv::static_status_take(&w_static, clear)) != cudaSuccess) return cuda_fail("device_status: the fixed scratch's word", e);
    *word = w | w_static;
    return SILVANN_B200_OK;
}

/* ---------------------------------------------------------------------------------------------------------- */

SV_EXPORT int silvann_b200_decode(void* o, float* res, const void* q, const void* k, const void* v, uint64_t q_heads, uint64_t kv_heads,
                                  uint64_t head_dim, uint64_t length, uint32_t nsplit, int dtype, sv_fault* over, void* stream) {
    called();
    if (!q || !k || !v || (!o && !res)) return fail(SILVANN_B200_E_ARGUMENT, "decode: a null operand");
    if (!dtype_ok(dtype)) return fail(SILVANN_B200_E_ARGUMENT, "decode: dtype %d", dtype);
    if (q_heads == 0 || kv_heads == 0 || q_heads % kv_heads != 0) return fail(SILVANN_B200_E_ARGUMENT, "decode: %llu query heads do not divide over %llu kv heads", (unsigned long long)q_heads, (unsigned long long)kv_heads);
    if (length == 0 || length > 0x7FFFFFFFull) return fail(SILVANN_B200_E_ARGUMENT, "decode: length %llu", (unsigned long long)length);
    sv::DecodeCall c;
    memset(&c, 0, sizeof c);
    c.o = o; c.res = res; c.q = q; c.k = k; c.v = v; c.kv_rows = length; c.seqs = 1;
    c.q_heads = (uint32_t)q_heads; c.kv_heads = (uint32_t)kv_heads; c.head_dim = (uint32_t)head_dim; c.length = (uint32_t)length;
    c.nsplit = nsplit; c.dtype = dtype; c.over = over; c.stream = (cudaStream_t)stream;
    if (!sv::decode_fits(c)) return fail(SILVANN_B200_E_ARGUMENT, "decode: head_dim %llu, group %llu or operand alignment is outside the kernel's fit", (unsigned long long)head_dim, (unsigned long long)(q_heads / kv_heads));
    cudaError_t e = sv::decode_device_scratch(&c.scratch);
    if (e != cudaSuccess) return cuda_fail("decode: scratch", e);
    if ((e = sv::decode_launch(c)) != cudaSuccess) return cuda_fail("decode: launch", e);
    return SILVANN_B200_OK;
}

SV_EXPORT int silvann_b200_merge(float* into, const float* a, const float* b, uint64_t q_heads, uint64_t head_dim, void* stream) {
    called();
    if (!into || !a || !b || !q_heads || !head_dim) return fail(SILVANN_B200_E_ARGUMENT, "merge: a null or empty operand");
    cudaError_t e = sv::merge_launch(into, a, b, q_heads, head_dim, (cudaStream_t)stream);
    return e == cudaSuccess ? SILVANN_B200_OK : cuda_fail("merge", e);
}
SV_EXPORT int silvann_b200_finish(void* o, const float* res, uint64_t q_heads, uint64_t head_dim, int dtype, sv_fault* over, void* stream) {
    called();
    if (!o || !res || !q_heads || !head_dim || !dtype_ok(dtype)) return fail(SILVANN_B200_E_ARGUMENT, "finish: a null or empty operand, or dtype");
    cudaError_t e = sv::finish_launch((uint16_t*)o, res, q_heads, head_dim, over, dtype, (cudaStream_t)stream);
    return e == cudaSuccess ? SILVANN_B200_OK : cuda_fail("finish", e);
}

/* ---------------------------------------------------------------------------------------------------------- */
/* paged decode: the plan                                                                                       */

struct silvann_b200_plan {
    int device;
    sv::DecodeItem* items_host;     /* pinned */
    sv::DecodeItem* items_dev;
    int32_t* lens_host;             /* pinned */
    int32_t* lens_dev;
    uint32_t items_cap, lens_cap;
    sv::DecodeScratch scratch;
    cudaEvent_t uploaded;           /* the last upload has left the pinned buffers */
    uint32_t n_items, n_slots, n_tickets, seqs, q_heads, kv_heads, head_dim;
    uint64_t positions;
    uint32_t max_len;               /* the longest sequence of the last plan_decode: bounds the page-table columns a launch reads */
    bool ready;
};

static void plan_release(silvann_b200_plan* p) {
    if (p->items_host) cudaFreeHost(p->items_host);
    if (p->items_dev) cudaFree(p->items_dev);
    if (p->lens_host) cudaFreeHost(p->lens_host);
    if (p->lens_dev) cudaFree(p->lens_dev);
    if (p->scratch.partials) cudaFree(p->scratch.partials);
    if (p->scratch.tickets) cudaFree(p->scratch.tickets);
    if (p->uploaded) cudaEventDestroy(p->uploaded);
}

SV_EXPORT int silvann_b200_plan_create(silvann_b200_plan** plan) {
    if (!plan) return fail(SILVANN_B200_E_ARGUMENT, "plan_create: plan is null");
    silvann_b200_plan* p = new (std::nothrow) silvann_b200_plan();
    if (!p) return fail(SILVANN_B200_E_CUDA, "plan_create: out of host memory");
    memset(p, 0, sizeof *p);
    cudaError_t e = cudaGetDevice(&p->device);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&p->uploaded, cudaEventDisableTiming);
    if (e != cudaSuccess) { delete p; return cuda_fail("plan_create", e); }
    *plan = p;
    return SILVANN_B200_OK;
}
SV_EXPORT int silvann_b200_plan_destroy(silvann_b200_plan* p) {
    if (!p) return SILVANN_B200_OK;
    (void)cudaDeviceSynchronize();
    plan_release(p);
    delete p;
    return SILVANN_B200_OK;
}

SV_EXPORT int silvann_b200_plan_decode(silvann_b200_plan* p, const int32_t* seq_lens, uint32_t seqs, uint32_t q_heads, uint32_t kv_heads,
                                       uint32_t head_dim, uint32_t blocks_target, void* stream) {
    if (!p || !seq_lens || seqs == 0) return fail(SILVANN_B200_E_ARGUMENT, "plan_decode: a null or empty operand");
    if (kv_heads == 0 || q_heads % kv_heads != 0 || q_heads / kv_heads > 64) return fail(SILVANN_B200_E_ARGUMENT, "plan_decode: heads %u over %u", q_heads, kv_heads);
    if (head_dim != 64 && head_dim != 128 && head_dim != 256) return fail(SILVANN_B200_E_ARGUMENT, "plan_decode: head_dim %u", head_dim);
    cudaStream_t st = (cudaStream_t)stream;
    const uint32_t group = q_heads / kv_heads, hpb = group <= 8 ? 8u : 16u, hb = (group + hpb - 1) / hpb, lanes = kv_heads * hb;
    const uint32_t TILE = sv::decode_tile_positions(head_dim);
    uint64_t tiles_total = 0, positions = 0;
    uint32_t max_len = 0;
    for (uint32_t s = 0; s < seqs; ++s) {
        if (seq_lens[s] <= 0) return fail(SILVANN_B200_E_ARGUMENT, "plan_decode: sequence %u has length %d", s, seq_lens[s]);
        tiles_total += ((uint64_t)seq_lens[s] + TILE - 1) / TILE;
        positions += (uint64_t)seq_lens[s];
        max_len = std::max(max_len, (uint32_t)seq_lens[s]);
    }
    if (blocks_target == 0) blocks_target = sv::device_sm_count() * 4u;
    uint64_t chunk = (tiles_total * lanes + blocks_target - 1) / blocks_target;
    if (chunk < 4) chunk = 4;                                 /* a block should stream at least a few tiles */

    std::vector<sv::DecodeItem> items;
    uint32_t slots = 0, tickets = 0;
    for (uint32_t s = 0; s < seqs; ++s) {
        const uint32_t tiles = ((uint32_t)seq_lens[s] + TILE - 1) / TILE;
        uint32_t ns = (uint32_t)((tiles + chunk - 1) / chunk);
        if (ns > 1024u) ns = 1024u;
        const uint32_t per = (tiles + ns - 1) / ns;
        ns = (tiles + per - 1) / per;
        for (uint32_t g = 0; g < kv_heads; ++g)
            for (uint32_t b = 0; b < hb; ++b) {
                const uint32_t base = ns > 1 ? slots : 0u;
                for (uint32_t x = 0; x < ns; ++x) {
                    sv::DecodeItem it;
                    memset(&it, 0, sizeof it);
                    it.seq = (int32_t)s; it.kvh = (int32_t)g; it.head0 = (int32_t)(g * group + b * hpb);
                    it.heads = (int32_t)std::min(hpb, group - b * hpb);
                    it.tile_begin = (int32_t)(x * per); it.tile_end = (int32_t)std::min(tiles, (x + 1) * per);
                    it.split = (int32_t)x; it.nsplit = (int32_t)ns; it.slot_base = (int32_t)base; it.ticket = (int32_t)tickets;
                    items.push_back(it);
                }
                if (ns > 1) slots += ns;
                ++tickets;
            }
    }
    /* longest first, so the tail of the launch is made of short blocks */
    std::stable_sort(items.begin(), items.end(), [](const sv::DecodeItem& a, const sv::DecodeItem& b) {
        return (a.tile_end - a.tile_begin) > (b.tile_end - b.tile_begin); });

    cudaError_t e;
    const uint32_t n = (uint32_t)items.size();
    const bool grow = n > p->items_cap || seqs > p->lens_cap || slots > p->scratch.slots || tickets > p->scratch.tickets_n ||
                      head_dim + 2 > p->scratch.slot_floats;
    if (grow) {
        if ((e = cudaDeviceSynchronize()) != cudaSuccess) return cuda_fail("plan_decode: wait before growing", e);
        if (n > p->items_cap) {
            if (p->items_host) cudaFreeHost(p->items_host);
            if (p->items_dev) cudaFree(p->items_dev);
            p->items_host = nullptr; p->items_dev = nullptr; p->items_cap = 0;
            const uint32_t cap = std::max(n * 2u, 1024u);
            if ((e = cudaHostAlloc(&p->items_host, (size_t)cap * sizeof(sv::DecodeItem), cudaHostAllocDefault)) != cudaSuccess) return cuda_fail("plan_decode: pinned items", e);
            if ((e = cudaMalloc(&p->items_dev, (size_t)cap * sizeof(sv::DecodeItem))) != cudaSuccess) return cuda_fail("plan_decode: device items", e);
            p->items_cap = cap;
        }
        if (seqs > p->lens_cap) {
            if (p->lens_host) cudaFreeHost(p->lens_host);
            if (p->lens_dev) cudaFree(p->lens_dev);
            p->lens_host = nullptr; p->lens_dev = nullptr; p->lens_cap = 0;
            const uint32_t cap = std::max(seqs * 2u, 256u);
            if ((e = cudaHostAlloc(&p->lens_host, (size_t)cap * sizeof(int32_t), cudaHostAllocDefault)) != cudaSuccess) return cuda_fail("plan_decode: pinned lens", e);
            if ((e = cudaMalloc(&p->lens_dev, (size_t)cap * sizeof(int32_t))) != cudaSuccess) return cuda_fail("plan_decode: device lens", e);
            p->lens_cap = cap;
        }
        if (slots > p->scratch.slots || head_dim + 2 > p->scratch.slot_floats) {
            if (p->scratch.partials) cudaFree(p->scratch.partials);
            p->scratch.partials = nullptr; p->scratch.slots = 0;
            const uint32_t cap = std::max(slots * 2u, 1024u), sf = std::max(head_dim + 2u, p->scratch.slot_floats);
            if ((e = cudaMalloc(&p->scratch.partials, (size_t)cap * 16 * sf * sizeof(float))) != cudaSuccess) return cuda_fail("plan_decode: partials", e);
            p->scratch.slots = cap; p->scratch.slot_floats = sf;
        }
        if (tickets > p->scratch.tickets_n) {
            if (p->scratch.tickets) cudaFree(p->scratch.tickets);
            p->scratch.tickets = nullptr; p->scratch.tickets_n = 0;
            const uint32_t cap = std::max(tickets * 2u, 1024u);
            if ((e = cudaMalloc(&p->scratch.tickets, (size_t)cap * sizeof(unsigned int))) != cudaSuccess) return cuda_fail("plan_decode: tickets", e);
            if ((e = cudaMemset(p->scratch.tickets, 0, (size_t)cap * sizeof(unsigned int))) != cudaSuccess) return cuda_fail("plan_decode: tickets", e);
            p->scratch.tickets_n = cap;
        }
    } else if (p->ready) {
        /* the previous upload must have left the pinned buffers before they are rewritten */
        if ((e = cudaEventSynchronize(p->uploaded)) != cudaSuccess) return cuda_fail("plan_decode: wait for the last upload", e);
    }
    memcpy(p->items_host, items.data(), (size_t)n * sizeof(sv::DecodeItem));
    memcpy(p->lens_host, seq_lens, (size_t)seqs * sizeof(int32_t));
    if ((e = cudaMemcpyAsync(p->items_dev, p->items_host, (size_t)n * sizeof(sv::DecodeItem), cudaMemcpyHostToDevice, st)) != cudaSuccess) return cuda_fail("plan_decode: upload items", e);
    if ((e = cudaMemcpyAsync(p->lens_dev, p->lens_host, (size_t)seqs * sizeof(int32_t), cudaMemcpyHostToDevice, st)) != cudaSuccess) return cuda_fail("plan_decode: upload lens", e);
    if ((e = cudaEventRecord(p->uploaded, st)) != cudaSuccess) return cuda_fail("plan_decode: record", e);
    p->n_items = n; p->n_slots = slots; p->n_tickets = tickets; p->seqs = seqs; p->q_heads = q_heads; p->kv_heads = kv_heads;
    p->head_dim = head_dim; p->positions = positions; p->max_len = max_len; p->ready = true;
    return SILVANN_B200_OK;
}

SV_EXPORT int silvann_b200_plan_info(const silvann_b200_plan* p, uint32_t* blocks, uint32_t* slots, uint64_t* positions) {
    if (!p || !p->ready) return fail(SILVANN_B200_E_STATE, "plan_info: the plan holds no work list");
    if (blocks) *blocks = p->n_items;
    if (slots) *slots = p->n_slots;
    if (positions) *positions = p->positions;
    return SILVANN_B200_OK;
}

SV_EXPORT int silvann_b200_paged_decode(silvann_b200_plan* p, void* o, float* res, const void* q, const void* k_pool, const void* v_pool,
                                        uint64_t pool_pages, uint32_t page_positions, const int32_t* page_table, uint32_t table_stride,
                                        int dtype, sv_fault* over, void* stream) {
    called();
    if (!p || !p->ready) return fail(SILVANN_B200_E_STATE, "paged_decode: plan_decode has not run");
    if (!q || !k_pool || !v_pool || !page_table || (!o && !res)) return fail(SILVANN_B200_E_ARGUMENT, "paged_decode: a null operand");
    if (!dtype_ok(dtype)) return fail(SILVANN_B200_E_ARGUMENT, "paged_decode: dtype %d", dtype);
    if (page_positions == 0 || page_positions % sv::decode_tile_positions(p->head_dim) != 0) return fail(SILVANN_B200_E_ARGUMENT, "paged_decode: page of %u positions is not a multiple of %u", page_positions, sv::decode_tile_positions(p->head_dim));
    if (pool_pages == 0 || pool_pages * page_positions > 0x7FFFFFFFull) return fail(SILVANN_B200_E_ARGUMENT, "paged_decode: pool of %llu pages", (unsigned long long)pool_pages);
    if ((p->max_len - 1u) / page_positions >= table_stride)
        return fail(SILVANN_B200_E_ARGUMENT, "paged_decode: the longest planned sequence (%u positions) needs %u page-table columns and a row has %u", p->max_len, (p->max_len - 1u) / page_positions + 1u, table_stride);
    sv::DecodeCall c;
    memset(&c, 0, sizeof c);
    c.o = o; c.res = res; c.q = q; c.k = k_pool; c.v = v_pool; c.kv_rows = pool_pages * page_positions;
    c.page_table = page_table; c.table_stride = table_stride; c.page_pos = page_positions; c.seq_lens = p->lens_dev;
    c.items = p->items_dev; c.n_items = p->n_items; c.seqs = p->seqs; c.q_heads = p->q_heads; c.kv_heads = p->kv_heads;
    c.head_dim = p->head_dim; c.dtype = dtype; c.over = over; c.scratch = p->scratch; c.stream = (cudaStream_t)stream;
    if (!sv::decode_fits(c)) return fail(SILVANN_B200_E_ARGUMENT, "paged_decode: operand alignment is outside the kernel's fit");
    cudaError_t e = sv::decode_launch(c);
    return e == cudaSuccess ? SILVANN_B200_OK : cuda_fail("paged_decode: launch", e);
}

__global__ void __launch_bounds__(128) paged_append_kernel(uint4* k_pool, uint4* v_pool, const uint4* k_rows, const uint4* v_rows,
                                                           const int32_t* lens, const int32_t* table, uint32_t table_stride,
                                                           uint32_t page_pos, uint32_t pool_pages, uint32_t row_vec, unsigned int* status) {
    const uint32_t s = blockIdx.x;
    const int32_t pos = lens[s] - 1;
    if (pos < 0) return;
    const uint32_t col = (uint32_t)pos / page_pos;
    const int32_t page = col < table_stride ? table[(size_t)s * table_stride + col] : -1;
    if (page < 0 || (uint32_t)page >= pool_pages) {      /* a stale or short table must not become a write somewhere else */
        if (threadIdx.x == 0 && status) atomicOr(status, SV_STATUS_BAD_PAGE);
        return;
    }
    const size_t at = ((size_t)page * page_pos + (uint32_t)pos % page_pos) * row_vec;
    for (uint32_t i = threadIdx.x; i < row_vec; i += blockDim.x) {
        k_pool[at + i] = k_rows[(size_t)s * row_vec + i];
        v_pool[at + i] = v_rows[(size_t)s * row_vec + i];
    }
}

SV_EXPORT int silvann_b200_paged_append(silvann_b200_plan* p, void* k_pool, void* v_pool, const void* k_rows, const void* v_rows,
                                        uint64_t pool_pages, uint32_t page_positions, const int32_t* page_table, uint32_t table_stride, void* stream) {
    called();
    if (!p || !p->ready) return fail(SILVANN_B200_E_STATE, "paged_append: plan_decode has not run");
    if (!k_pool || !v_pool || !k_rows || !v_rows || !page_table || page_positions == 0) return fail(SILVANN_B200_E_ARGUMENT, "paged_append: a null operand");
    if (pool_pages == 0 || pool_pages * page_positions > 0x7FFFFFFFull) return fail(SILVANN_B200_E_ARGUMENT, "paged_append: pool of %llu pages", (unsigned long long)pool_pages);
    if ((p->max_len - 1u) / page_positions >= table_stride)
        return fail(SILVANN_B200_E_ARGUMENT, "paged_append: the longest planned sequence (%u positions) needs %u page-table columns and a row has %u", p->max_len, (p->max_len - 1u) / page_positions + 1u, table_stride);
    const uint32_t row_bytes = p->kv_heads * p->head_dim * 2u;
    if (row_bytes % 16u || (((uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)k_rows | (uintptr_t)v_rows) & 15u))
        return fail(SILVANN_B200_E_ARGUMENT, "paged_append: rows and pools must be 16-byte aligned");
    paged_append_kernel<<<p->seqs, 128, 0, (cudaStream_t)stream>>>((uint4*)k_pool, (uint4*)v_pool, (const uint4*)k_rows, (const uint4*)v_rows,
                                                                  p->lens_dev, page_table, table_stride, page_positions, (uint32_t)pool_pages,
                                                                  row_bytes / 16u, sv::device_status_word());
    sv::note_launch(1);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? SILVANN_B200_OK : cuda_fail("paged_append: launch", e);
}

/* ---------------------------------------------------------------------------------------------------------- */

SV_EXPORT int silvann_b200_prefill(void* o, float* res, const void* q, const void* k, const void* v, uint64_t q_heads, uint64_t kv_heads, uint64_t head_dim,
                                   uint64_t first, uint64_t rows, int dtype, sv_fault* over, void* stream) {
    called();
    if ((!o && !res) || !q || !k || !v) return fail(SILVANN_B200_E_ARGUMENT, "prefill: a null operand");
    if (!dtype_ok(dtype)) return fail(SILVANN_B200_E_ARGUMENT, "prefill: dtype %d", dtype);
    if (rows == 0 || kv_heads == 0 || q_heads % kv_heads != 0) return fail(SILVANN_B200_E_ARGUMENT, "prefill: rows %llu, heads %llu over %llu", (unsigned long long)rows, (unsigned long long)q_heads, (unsigned long long)kv_heads);
    sv::PrefillCall c;
    memset(&c, 0, sizeof c);
    c.o = o; c.res = res; c.q = q; c.k = k; c.v = v; c.q_heads = (uint32_t)q_heads; c.kv_heads = (uint32_t)kv_heads; c.head_dim = (uint32_t)head_dim;
    c.first = first; c.rows = rows; c.dtype = dtype; c.over = over; c.stream = (cudaStream_t)stream;
    if (!sv::prefill_fits(c)) return fail(SILVANN_B200_E_ARGUMENT, "prefill: head_dim %llu or operand alignment is outside the kernel's fit", (unsigned long long)head_dim);
    cudaError_t e = sv::prefill_launch(c);
    return e == cudaSuccess ? SILVANN_B200_OK : cuda_fail("prefill: launch", e);
}

SV_EXPORT int silvann_b200_mla_decode(void* o, float* res, const void* q, const void* latent, uint64_t heads, uint64_t latent_dim, uint64_t length,
                                      uint32_t blocks, int dtype, sv_fault* over, void* stream) {
    called();
    if ((!o && !res) || !q || !latent) return fail(SILVANN_B200_E_ARGUMENT, "mla_decode: a null operand");
    if (!dtype_ok(dtype)) return fail(SILVANN_B200_E_ARGUMENT, "mla_decode: dtype %d", dtype);
    if (!sv::mla_decode_fits(q, latent, heads, latent_dim, length) || ((uintptr_t)res & 3u))
        return fail(SILVANN_B200_E_ARGUMENT, "mla_decode: %llu heads (32 or 64) over a latent of %llu (512), %llu positions, or an operand's alignment is outside the kernel's fit",
                    (unsigned long long)heads, (unsigned long long)latent_dim, (unsigned long long)length);
    cudaError_t e = sv::mla_decode_launch(o, res, q, latent, heads, length, dtype, blocks, over, (cudaStream_t)stream);
    return e == cudaSuccess ? SILVANN_B200_OK : cuda_fail("mla_decode: launch", e);
}

SV_EXPORT int silvann_b200_deltanet(float* S, const void* conved, const void* z, const void* beta, const void* g, const void* w, void* out,
                                    float* readout, uint64_t k_heads, uint64_t v_heads, uint64_t head_dim, uint64_t rows, uint32_t seqs, uint32_t gate,
                                    int dtype, sv_fault* over, void* stream) {
    called();
    if (!S || !conved || !z || !beta || !g || !w || !out) return fail(SILVANN_B200_E_ARGUMENT, "deltanet: a null operand");
    if (!dtype_ok(dtype) || gate > 1u) return fail(SILVANN_B200_E_ARGUMENT, "deltanet: dtype %d or gate %u", dtype, gate);
    sv::DeltaCall c;
    memset(&c, 0, sizeof c);
    c.S = S; c.conved = (const uint16_t*)conved; c.z = (const uint16_t*)z; c.beta = (const uint16_t*)beta; c.g = (const uint16_t*)g;
    c.w = (const uint16_t*)w; c.out = (uint16_t*)out; c.readout = readout; c.k_heads = (uint32_t)k_heads; c.v_heads = (uint32_t)v_heads;
    c.head_dim = (uint32_t)head_dim; c.seqs = seqs; c.rows = rows; c.gate = (int)gate; c.dtype = dtype; c.over = over; c.stream = (cudaStream_t)stream;
    if (!sv::deltanet_fits(c)) return fail(SILVANN_B200_E_ARGUMENT, "deltanet: head_dim %llu or heads %llu over %llu are outside the kernel's fit", (unsigned long long)head_dim, (unsigned long long)v_heads, (unsigned long long)k_heads);
    cudaError_t e = sv::deltanet_launch(c);
    return e == cudaSuccess ? SILVANN_B200_OK : cuda_fail("deltanet: launch", e);
}
