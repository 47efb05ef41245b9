/* tier.cu — one-query decode over a two-tier KV cache: the oldest positions in pinned host RAM, the rest on the card.
 *
 * The reference keeps every tier of its cache on the card (age tiers, engine/src/packages/ai_qwen_3/contracts/objects/
 * mixer.cuh:93-107) and attends each tier separately — one residual a tier (attention_weights + attention_residual_mix),
 * folded with attention_merge and closed by attention_finish (ai_qwen_3 mixer__abi.cuh:383-412).  This file keeps that
 * arithmetic and adds the tier the reference does not have: host RAM.  The host range is cut into chunks; a side stream
 * copies chunk c+1 into a ring of device staging buffers (cudaMemcpyAsync, the job the sys doors side_memory_write_queued /
 * side_mark_record / mark_wait exist for, engine/src/packages/sys/contracts/abi/gpu.cuh:53-62,70-77) while the compute
 * stream attends chunk c with the split-KV decode kernel and merges its residual into the running one.  The card tier
 * is attended first, so its work hides the first copy.  The merge order is fixed (card tier, then host chunks oldest
 * first), so results repeat bit for bit.
 *
 * The host tier is PCIe-bound by nature: its roofline is the pinned host-to-device copy rate, not HBM. */
#include "../../include/silvann_b200.h"
#include "common.cuh"
#include "kernels.h"
#include "exchange.cuh"
#include <new>
#include <stdio.h>
#include <string.h>

#define SV_EXPORT extern "C" __attribute__((visibility("default")))
#define SV_TIER_STAGES_MAX 8
#define SV_TIER_COPY_BYTES (8ull << 20)      /* a plane's share of a chunk when the caller leaves the chunk size to the library */

int sv_ext_fail(int code, const char* fmt, ...);      /* ext.cu: records the message for silvann_b200_last_error */
struct silvann_b200_exchange;
int sv_exchange_begin(silvann_b200_exchange* x, uint32_t wait_ms, uint64_t bytes, sv::XfParams* P);     /* exchange.cu */
void sv_exchange_advance(silvann_b200_exchange* x);
int sv_exchange_merge_finish(silvann_b200_exchange* x, void* o, float* res, const float* res_local, uint64_t q_heads, uint64_t head_dim, int dtype,
                             sv_fault* over, uint32_t wait_ms, void* stream);      /* exchange.cu */

struct silvann_b200_tier {
    int device;
    uint32_t q_heads, kv_heads, head_dim, chunk, stages;
    int dtype;
    size_t row_bytes;
    void* k_stage[SV_TIER_STAGES_MAX];
    void* v_stage[SV_TIER_STAGES_MAX];
    cudaEvent_t full[SV_TIER_STAGES_MAX];      /* side stream: the chunk has landed in the stage */
    cudaEvent_t freed[SV_TIER_STAGES_MAX];     /* compute stream: the stage's chunk has been attended */
    bool freed_recorded[SV_TIER_STAGES_MAX];
    cudaStream_t side;
    float* acc;                                /* running residual [q_heads][head_dim + 2] */
    float* tmp;                                /* one piece's residual */
    uint64_t h2d_bytes, chunks;
};

static void tier_release(silvann_b200_tier* t) {
    for (uint32_t s = 0; s < SV_TIER_STAGES_MAX; ++s) {
        if (t->k_stage[s]) cudaFree(t->k_stage[s]);
        if (t->v_stage[s]) cudaFree(t->v_stage[s]);
        if (t->full[s]) cudaEventDestroy(t->full[s]);
        if (t->freed[s]) cudaEventDestroy(t->freed[s]);
    }
    if (t->side) cudaStreamDestroy(t->side);
    if (t->acc) cudaFree(t->acc);
    if (t->tmp) cudaFree(t->tmp);
}

SV_EXPORT int silvann_b200_tier_create(silvann_b200_tier** out, uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim, int dtype,
                                       uint32_t chunk_positions, uint32_t stages) {
    if (!out) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "tier_create: out is null");
    if (kv_heads == 0 || q_heads % kv_heads != 0 || (head_dim != 64 && head_dim != 128 && head_dim != 256))
        return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "tier_create: %u heads over %u, head_dim %u", q_heads, kv_heads, head_dim);
    if (dtype != SV_DTYPE_FP16 && dtype != SV_DTYPE_BF16) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "tier_create: dtype %d", dtype);
    if (chunk_positions == 0) {
        /* sized in bytes, not positions: a copy of a few megabytes a plane keeps the host link busy whatever the width of a
         * row is (a rank that owns one kv head has rows of 256 bytes; 8,192 of them would be a 2 MB copy) */
        const uint64_t row = (uint64_t)kv_heads * head_dim * 2u;
        uint64_t n = (SV_TIER_COPY_BYTES + row - 1) / row;
        n = (n + 127u) / 128u * 128u;
        chunk_positions = (uint32_t)(n < 1024u ? 1024u : n);
    }
    if (stages < 2 || stages > SV_TIER_STAGES_MAX || chunk_positions % 128u != 0)
        return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "tier_create: %u stages (2..%d) of %u positions (a multiple of 128)", stages, SV_TIER_STAGES_MAX, chunk_positions);
    silvann_b200_tier* t = new (std::nothrow) silvann_b200_tier();
    if (!t) return sv_ext_fail(SILVANN_B200_E_CUDA, "tier_create: out of host memory");
    memset(t, 0, sizeof *t);
    t->q_heads = q_heads; t->kv_heads = kv_heads; t->head_dim = head_dim; t->dtype = dtype; t->chunk = chunk_positions; t->stages = stages;
    t->row_bytes = (size_t)kv_heads * head_dim * 2u;
    cudaError_t e = cudaGetDevice(&t->device);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&t->side, cudaStreamNonBlocking);
    for (uint32_t s = 0; e == cudaSuccess && s < stages; ++s) {
        e = cudaMalloc(&t->k_stage[s], t->row_bytes * chunk_positions);
        if (e == cudaSuccess) e = cudaMalloc(&t->v_stage[s], t->row_bytes * chunk_positions);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&t->full[s], cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&t->freed[s], cudaEventDisableTiming);
    }
    const size_t res_bytes = (size_t)q_heads * (head_dim + 2u) * sizeof(float);
    if (e == cudaSuccess) e = cudaMalloc(&t->acc, res_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&t->tmp, res_bytes);
    if (e != cudaSuccess) {
        tier_release(t); delete t; (void)cudaGetLastError();
        return sv_ext_fail(SILVANN_B200_E_CUDA, "tier_create: %s", cudaGetErrorString(e));
    }
    *out = t;
    return SILVANN_B200_OK;
}

SV_EXPORT int silvann_b200_tier_destroy(silvann_b200_tier* t) {
    if (!t) return SILVANN_B200_OK;
    (void)cudaDeviceSynchronize();
    tier_release(t);
    delete t;
    return SILVANN_B200_OK;
}

SV_EXPORT int silvann_b200_tier_stats(const silvann_b200_tier* t, uint64_t* h2d_bytes, uint64_t* chunks) {
    if (!t) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "tier_stats: tier is null");
    if (h2d_bytes) *h2d_bytes = t->h2d_bytes;
    if (chunks) *chunks = t->chunks;
    return SILVANN_B200_OK;
}

/* One piece of the cache into `res` (m, l, acc per head), enqueued on `st`. */
static cudaError_t piece(const silvann_b200_tier* t, void* o, float* res, const void* q, const void* k, const void* v, uint64_t length, sv_fault* over,
                         cudaStream_t st, const sv::XfParams* xf = nullptr) {
    sv::DecodeCall c;
    memset(&c, 0, sizeof c);
    c.o = o; c.res = res; c.q = q; c.k = k; c.v = v; c.kv_rows = length; c.seqs = 1;
    c.q_heads = t->q_heads; c.kv_heads = t->kv_heads; c.head_dim = t->head_dim; c.length = (uint32_t)length;
    c.dtype = t->dtype; c.over = over; c.stream = st; c.xf = xf;
    if (!sv::decode_fits(c)) return cudaErrorInvalidValue;
    cudaError_t e = sv::decode_device_scratch(&c.scratch);
    if (e != cudaSuccess) return e;
    return sv::decode_launch(c);
}

static int tier_decode(silvann_b200_tier* t, silvann_b200_exchange* x, uint32_t wait_ms, void* o, float* res, const void* q, const void* k_host,
                       const void* v_host, uint64_t host_len, const void* k_dev, const void* v_dev, uint64_t dev_len, sv_fault* over, void* stream) {
    if (!t || !q || (!o && !res)) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "tier_decode: a null operand");
    if (host_len + dev_len == 0 || host_len + dev_len > 0x7FFFFFFFull) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "tier_decode: %llu positions", (unsigned long long)(host_len + dev_len));
    if ((host_len && (!k_host || !v_host)) || (dev_len && (!k_dev || !v_dev))) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "tier_decode: a tier with positions and no planes");
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaSuccess;
    bool have = false;
#define SV_TRY(call, what) do { e = (call); if (e != cudaSuccess) { (void)cudaGetLastError(); return sv_ext_fail(SILVANN_B200_E_CUDA, "tier_decode: %s: %s", what, cudaGetErrorString(e)); } } while (0)
    if (host_len == 0 && !x) {
        /* everything is on the card and nobody else holds a part of the range: the decode kernel writes the answer itself,
         * with no running residual and no finishing launch */
        SV_TRY(piece(t, o, res, q, k_dev, v_dev, dev_len, over, st), "card tier");
        return SILVANN_B200_OK;
    }
    if (host_len == 0 && x) {
        /* everything is on the card and the other members hold the rest of the range: the decode kernel's last block of a head
         * block pushes the residual to the members, folds theirs and writes the answer — the exchange step without a launch of
         * its own.  A cache too short to be split has no such block: it takes the two launches below. */
        sv::XfParams P;
        const int rc = sv_exchange_begin(x, wait_ms, (uint64_t)t->q_heads * (t->head_dim + 2u) * sizeof(float), &P);
        if (rc != SILVANN_B200_OK) return rc;
        e = piece(t, o, res, q, k_dev, v_dev, dev_len, over, st, &P);
        if (e == cudaSuccess) { sv_exchange_advance(x); return SILVANN_B200_OK; }
        (void)cudaGetLastError();
        if (e != cudaErrorNotSupported) return sv_ext_fail(SILVANN_B200_E_CUDA, "tier_decode: %s: %s", "card tier with the exchange", cudaGetErrorString(e));
    }
    const uint64_t nchunks = (host_len + t->chunk - 1) / t->chunk;
    /* queue the first copies before any compute so that they run under the card tier's kernel */
    uint64_t queued = 0;
    auto queue_copy = [&](uint64_t c) -> cudaError_t {
        const uint32_t s = (uint32_t)(c % t->stages);
        const uint64_t n = (c + 1 == nchunks) ? host_len - c * t->chunk : t->chunk;
        cudaError_t r;
        if (t->freed_recorded[s] && (r = cudaStreamWaitEvent(t->side, t->freed[s], 0)) != cudaSuccess) return r;
        const size_t off = (size_t)c * t->chunk * t->row_bytes, bytes = (size_t)n * t->row_bytes;
        if ((r = cudaMemcpyAsync(t->k_stage[s], (const char*)k_host + off, bytes, cudaMemcpyHostToDevice, t->side)) != cudaSuccess) return r;
        if ((r = cudaMemcpyAsync(t->v_stage[s], (const char*)v_host + off, bytes, cudaMemcpyHostToDevice, t->side)) != cudaSuccess) return r;
        t->h2d_bytes += 2 * bytes; t->chunks += 1;
        return cudaEventRecord(t->full[s], t->side);
    };
    for (; queued < nchunks && queued < t->stages - 1; ++queued) SV_TRY(queue_copy(queued), "copy");
    if (dev_len) {
        SV_TRY(piece(t, nullptr, t->acc, q, k_dev, v_dev, dev_len, nullptr, st), "card tier");
        have = true;
    }
    for (uint64_t c = 0; c < nchunks; ++c) {
        const uint32_t s = (uint32_t)(c % t->stages);
        const uint64_t n = (c + 1 == nchunks) ? host_len - c * t->chunk : t->chunk;
        if (queued < nchunks) { SV_TRY(queue_copy(queued), "copy"); ++queued; }
        SV_TRY(cudaStreamWaitEvent(st, t->full[s], 0), "wait for a chunk");
        SV_TRY(piece(t, nullptr, have ? t->tmp : t->acc, q, t->k_stage[s], t->v_stage[s], n, nullptr, st), "host chunk");
        SV_TRY(cudaEventRecord(t->freed[s], st), "record");
        t->freed_recorded[s] = true;
        if (have) SV_TRY(sv::merge_launch(t->acc, t->acc, t->tmp, t->q_heads, t->head_dim, st), "merge");
        have = true;
    }
    if (x) return sv_exchange_merge_finish(x, o, res, t->acc, t->q_heads, t->head_dim, t->dtype, over, wait_ms, stream);
    if (res) SV_TRY(cudaMemcpyAsync(res, t->acc, (size_t)t->q_heads * (t->head_dim + 2u) * sizeof(float), cudaMemcpyDeviceToDevice, st), "residual out");
    if (o) SV_TRY(sv::finish_launch((uint16_t*)o, t->acc, t->q_heads, t->head_dim, over, t->dtype, st), "finish");
#undef SV_TRY
    return SILVANN_B200_OK;
}

SV_EXPORT int silvann_b200_tier_decode(silvann_b200_tier* t, void* o, float* res, const void* q, const void* k_host, const void* v_host,
                                       uint64_t host_len, const void* k_dev, const void* v_dev, uint64_t dev_len, sv_fault* over, void* stream) {
    return tier_decode(t, nullptr, 0, o, res, q, k_host, v_host, host_len, k_dev, v_dev, dev_len, over, stream);
}

SV_EXPORT int silvann_b200_tier_decode_exchange(silvann_b200_tier* t, silvann_b200_exchange* x, void* o, float* res, const void* q, const void* k_host,
                                                const void* v_host, uint64_t host_len, const void* k_dev, const void* v_dev, uint64_t dev_len,
                                                sv_fault* over, uint32_t wait_ms, void* stream) {
    if (!x) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "tier_decode_exchange: exchange is null");
    return tier_decode(t, x, wait_ms, o, res, q, k_host, v_host, host_len, k_dev, v_dev, dev_len, over, stream);
}
