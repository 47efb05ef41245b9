/* family.cu — the silicon-family face of the library: the one exported entry, the seven door tables, the sys doors
 * over the CUDA runtime, and the nn doors with deferred-pair fusion.
 *
 * What the engine expects of a family is restated in include/silvann_b200.h.  Behaviour that mirrors the reference's
 * CUDA family (engine/src/silicon_families/nvidia_cuda12/sys.cuh, nn.cuh):
 *   - the device a call acts on is the one the CALLING THREAD bound with bind_device; only sm_100 cards are counted;
 *   - every door enqueues on that device's legacy default stream and returns, so memory_read / memory_write (plain
 *     cudaMemcpy) and compute_completed order against door work exactly as they do there;
 *   - a launch the runtime refuses is remembered per device; the next compute_completed on it answers false once.
 *
 * Deferred pairs.  The contract splits attention over two or three doors with an fp32 weights buffer between them.
 * Here the first door of a pair only records its arguments (per device); when the matching second door arrives next,
 * one fused kernel runs and the buffer is never written.  Any other door — including every sys door that could make
 * the buffer observable — first runs the recorded door for real, so a program that reads the weights still finds
 * them.  SILVANN_B200_FUSE=0 turns the deferral off (each door then runs as worded). */
#include "../../include/silvann_b200.h"
#include "common.cuh"
#include "kernels.h"
#include "kernels_deltanet.h"
#include <cuda_runtime.h>
#include <mutex>
#include <atomic>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <fcntl.h>
#include <unistd.h>

namespace svf {

static constexpr int DEVICES_MAX = 64;

/* ---- counters (read through silvann_b200_counters_read) ---- */
std::atomic<uint64_t> g_counters[SILVANN_B200_COUNTERS];
static inline void bump(int which) { g_counters[which].fetch_add(1, std::memory_order_relaxed); }

/* ---- refused launches, per device ---- */
static volatile unsigned int g_refused[DEVICES_MAX];
static int current_device() { int d = -1; return (cudaGetDevice(&d) == cudaSuccess) ? d : -1; }
void launch_refused(const char* door, cudaError_t e) {
    const int d = current_device();
    fprintf(stderr, "silvann nvidia_b200: %s was refused on device %d: %s\n", door, d, e == cudaSuccess ? "not answered by this family" : cudaGetErrorString(e));
    if (e != cudaSuccess) (void)cudaGetLastError();
    if (d >= 0 && d < DEVICES_MAX) g_refused[d] = 1u;
    bump(SILVANN_B200_COUNTER_REFUSED);
}
}  // namespace svf
namespace sv { void note_launch(uint32_t kernels) { svf::g_counters[SILVANN_B200_COUNTER_LAUNCHES].fetch_add(kernels, std::memory_order_relaxed); } }
namespace svf {
static inline void check(const char* door, cudaError_t e) { if (e != cudaSuccess) launch_refused(door, e); }

static bool fuse_enabled() {
    static const bool on = []() { const char* v = getenv("SILVANN_B200_FUSE"); return !(v && v[0] == '0'); }();
    return on;
}

/* ---- the deferred first door of a pair, per device ---- */
enum PendingKind { NONE = 0, SCORES, WEIGHTS, CAUSAL_RAW, CAUSAL_SOFT, WEIGHTS_ROWS, WEIGHTS_TQ, GROUPED_RAW, GROUPED_SOFT, NORM_ROWS, GATE_ROWS };
struct Pending {
    int kind;
    float* p; float* res; const uint16_t* q; const uint16_t* k;      /* WEIGHTS_TQ: k is the key codes */
    uint64_t qh, kvh, d, length, first, rows;
    const uint16_t* scales; uint64_t width;                          /* WEIGHTS_TQ only: the key rows' scales and the code width */
    /* NORM_ROWS (rmsnorm_rows recorded in case rope_rows over the same rows follows): q = x, k = w, d = n, rows, first = x_stride, length = o_stride */
    uint16_t* o16; float eps; unsigned int* over;
    /* GATE_ROWS (attention_gate_rows recorded in case hadamard_rotate of its answers follows): o16 = o, q = att, k = qg, qh = heads, d = head_dim */
};
static Pending g_pending[DEVICES_MAX];
static std::mutex g_pending_lock[DEVICES_MAX];

/* Runs the recorded door as the contract words it.  Called with the device's lock held. */
static void run_pending_locked(Pending& pd) {
    const Pending x = pd;
    pd.kind = NONE;
    switch (x.kind) {
        case SCORES:      check("attention_scores", sv::scores_launch(x.p, x.q, x.k, x.qh, x.kvh, x.d, x.length, 0, nullptr, 0)); break;
        case WEIGHTS:     check("attention_weights", sv::scores_launch(x.p, x.q, x.k, x.qh, x.kvh, x.d, x.length, 1, x.res, 0)); break;
        case CAUSAL_RAW:  check("attention_causal_scores_grouped", sv::causal_scores_launch(x.p, x.q, x.k, x.qh, x.kvh, x.d, x.first, x.rows, false, 0)); break;
        case CAUSAL_SOFT: check("attention_causal_softmax", sv::causal_scores_launch(x.p, x.q, x.k, x.qh, x.kvh, x.d, x.first, x.rows, true, 0)); break;
        case WEIGHTS_ROWS: {        /* the one-row door a row, as the contract defines the many-row form (nn/gpu/doors.cuh:406-424) */
            const uint64_t span = x.first + x.rows;
            for (uint64_t r = 0; r < x.rows; ++r)
                check("attention_weights_rows", sv::scores_launch(x.p + r * x.qh * span, x.q + r * x.qh * x.d, x.k, x.qh, x.kvh, x.d, x.first + r + 1, 1,
                                                                  x.res + r * x.qh * (x.d + 2), 0));
            break;
        }
        case GROUPED_RAW: check("attention_scores_grouped", sv::scores_launch(x.p, x.q, x.k, x.qh, x.kvh, x.d, x.length, 2, nullptr, 0)); break;
        case GROUPED_SOFT:          /* the two doors that were recorded, as worded */
            check("attention_scores_grouped", sv::scores_launch(x.p, x.q, x.k, x.qh, x.kvh, x.d, x.length, 2, nullptr, 0));
            check("attention_softmax_rows", sv::softmax_rows_launch(x.p, x.qh, x.length, 0));
            break;
        case GATE_ROWS:   check("attention_gate_rows", sv::attention_gate_rows_launch(x.o16, x.q, x.k, x.qh, x.d, x.over, 0)); break;
        case NORM_ROWS:   check("rmsnorm_rows", sv::rmsnorm_rows_launch(x.o16, x.q, x.k, x.d, x.rows, x.first, x.length, x.eps, x.over, 0)); break;
        case WEIGHTS_TQ:  check("attention_weights_tq", sv::tq_weights_launch(x.p, x.res, x.q, (const uint8_t*)x.k, x.scales, x.qh, x.kvh, x.d, x.length, x.width, x.rows, 0)); break;
        default: return;
    }
    bump(SILVANN_B200_COUNTER_FLUSHED);
}
void flush() {
    const int d = current_device();
    if (d < 0 || d >= DEVICES_MAX) return;
    if (g_pending[d].kind == NONE) return;
    std::lock_guard<std::mutex> hold(g_pending_lock[d]);
    run_pending_locked(g_pending[d]);
}

/* ================================================================================================================ */
/* sys doors                                                                                                        */

static bool takes(int ordinal) {
    int major = 0, minor = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, ordinal) != cudaSuccess) return false;
    if (cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, ordinal) != cudaSuccess) return false;
    return major == 10 && minor == 0;              /* the library carries sm_100a code only */
}
static int shown() { int n = 0; return (cudaGetDeviceCount(&n) == cudaSuccess && n > 0) ? n : 0; }
static int ordinal_of(uint32_t index) {
    uint32_t mine = 0u;
    for (int o = 0; o < shown(); ++o) { if (!takes(o)) continue; if (mine++ == index) return o; }
    return -1;
}

static bool s_memory_allocate(void** at, size_t bytes) {
    size_t free_b = 0, total_b = 0;
    if (bytes >= ((size_t)1 << 20) && cudaMemGetInfo(&free_b, &total_b) == cudaSuccess && bytes > free_b) return false;
    return cudaMalloc(at, bytes) == cudaSuccess;
}
static void s_memory_free(void* at) { flush(); if (at) (void)cudaFree(at); }
static bool s_memory_zerofill(void* at, size_t bytes) { flush(); return cudaMemset(at, 0, bytes) == cudaSuccess; }
static bool s_memory_read(void* to, const void* from, size_t bytes) { flush(); return cudaMemcpy(to, from, bytes, cudaMemcpyDeviceToHost) == cudaSuccess; }
static bool s_memory_write(void* to, const void* from, size_t bytes) { flush(); return cudaMemcpy(to, from, bytes, cudaMemcpyHostToDevice) == cudaSuccess; }
static bool s_compute_completed(void) {
    flush();
    const bool waited = cudaStreamSynchronize(0) == cudaSuccess;
    const int d = current_device();
    if (d >= 0 && d < DEVICES_MAX && g_refused[d] != 0u) { g_refused[d] = 0u; return false; }
    return waited;
}
static bool s_side_open(void** channel) { return cudaStreamCreateWithFlags((cudaStream_t*)channel, cudaStreamNonBlocking) == cudaSuccess; }
static void s_side_close(void* channel) { if (channel) (void)cudaStreamDestroy((cudaStream_t)channel); }
static bool s_side_memory_read(void* to, const void* from, size_t bytes, void* ch) {
    return cudaMemcpyAsync(to, from, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)ch) == cudaSuccess && cudaStreamSynchronize((cudaStream_t)ch) == cudaSuccess;
}
static bool s_side_memory_write(void* to, const void* from, size_t bytes, void* ch) {
    return cudaMemcpyAsync(to, from, bytes, cudaMemcpyHostToDevice, (cudaStream_t)ch) == cudaSuccess && cudaStreamSynchronize((cudaStream_t)ch) == cudaSuccess;
}
static bool s_memory_allocate_host_ram_mapped(void** at, void** card_at, size_t bytes) {
    if (cudaHostAlloc(at, bytes, cudaHostAllocMapped) != cudaSuccess) return false;
    if (cudaHostGetDevicePointer(card_at, *at, 0) == cudaSuccess) return true;
    (void)cudaFreeHost(*at); *at = nullptr;
    return false;
}
static void s_memory_free_host_ram(void* at) { if (at) (void)cudaFreeHost(at); }
static uint32_t s_device_count(void) { uint32_t n = 0u; for (int o = 0; o < shown(); ++o) if (takes(o)) ++n; return n; }
static uint32_t s_bind_device(uint32_t index) {
    flush();                                        /* a door recorded on the device this thread leaves runs there, not on the next one */
    const int o = ordinal_of(index);
    return (o >= 0 && cudaSetDevice(o) == cudaSuccess) ? 1u : 0u;
}
static uint32_t s_bound_device(void) {
    const int d = current_device();
    if (d < 0 || !takes(d)) return 0xFFFFFFFFu;
    uint32_t mine = 0u;
    for (int o = 0; o < d; ++o) if (takes(o)) ++mine;
    return mine;
}
static bool s_memory_register_host(void* at, size_t bytes, void** card_at) {
    if (cudaHostRegister(at, bytes, cudaHostRegisterMapped) != cudaSuccess) return false;
    if (cudaHostGetDevicePointer(card_at, at, 0) == cudaSuccess) return true;
    (void)cudaHostUnregister(at);
    return false;
}
static void s_memory_unregister_host(void* at) { if (at) (void)cudaHostUnregister(at); }
/* Files: a handle is the descriptor plus one (never zero); a read goes through a bounce buffer and memory_write,
 * as engine/src/packages/sys/cpu/silicon/file.cuh does for every card family. */
static bool s_file_open(const char* path, uint64_t* handle) {
    if (!path || !handle) return false;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return false;
    *handle = (uint64_t)(uint32_t)fd + 1ull;
    return true;
}
static void s_file_close(uint64_t handle) { if (handle) (void)close((int)(uint32_t)handle - 1); }
static bool s_file_read(uint64_t handle, uint64_t offset, uint64_t bytes, void* to) {
    if (!handle || (!to && bytes)) return false;
    const size_t piece = bytes < ((size_t)8 << 20) ? (size_t)bytes : ((size_t)8 << 20);
    if (piece == 0) return true;
    char* bounce = (char*)malloc(piece);
    if (!bounce) return false;
    bool ok = true;
    for (uint64_t done = 0; ok && done < bytes; ) {
        const size_t n = (size_t)(bytes - done < piece ? bytes - done : piece);
        size_t got = 0;
        while (ok && got < n) {
            const ssize_t r = pread((int)(uint32_t)handle - 1, bounce + got, n - got, (off_t)(offset + done + got));
            if (r <= 0) ok = false; else got += (size_t)r;
        }
        ok = ok && s_memory_write((char*)to + done, bounce, n);
        done += n;
    }
    free(bounce);
    return ok;
}
static bool s_memory_map_file(void*, size_t, uint64_t, uint64_t) { return false; }    /* a card's memory is not the machine's */
static bool s_memory_prefetch(const void*, size_t) { return true; }                    /* device memory is never paged out */
static bool s_peer_access(uint32_t other) {
    const int here = current_device(), there = ordinal_of(other);
    if (here < 0 || there < 0) return false;
    if (here == there) return true;
    int can = 0;
    if (cudaDeviceCanAccessPeer(&can, here, there) != cudaSuccess || !can) return false;
    const cudaError_t on = cudaDeviceEnablePeerAccess(there, 0);
    if (on == cudaErrorPeerAccessAlreadyEnabled) { (void)cudaGetLastError(); return true; }
    return on == cudaSuccess;
}
static bool s_mark_open(void** mark) { return cudaEventCreateWithFlags((cudaEvent_t*)mark, cudaEventDisableTiming) == cudaSuccess; }
static void s_mark_close(void* mark) { if (mark) (void)cudaEventDestroy((cudaEvent_t)mark); }
static bool s_mark_record(void* mark) { flush(); return cudaEventRecord((cudaEvent_t)mark, 0) == cudaSuccess; }
static bool s_mark_wait(void* mark) { return cudaStreamWaitEvent(0, (cudaEvent_t)mark, 0) == cudaSuccess; }
static bool s_side_memory_write_queued(void* to, const void* from, size_t bytes, void* ch) { return cudaMemcpyAsync(to, from, bytes, cudaMemcpyHostToDevice, (cudaStream_t)ch) == cudaSuccess; }
static bool s_side_memory_read_queued(void* to, const void* from, size_t bytes, void* ch) { return cudaMemcpyAsync(to, from, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)ch) == cudaSuccess; }
static bool s_side_mark_record(void* mark, void* ch) { return cudaEventRecord((cudaEvent_t)mark, (cudaStream_t)ch) == cudaSuccess; }
static bool s_mark_reached(void* mark) { return cudaEventSynchronize((cudaEvent_t)mark) == cudaSuccess; }

/* ================================================================================================================ */
/* nn doors: first every row as a refusal, then the rows this family answers                                        */

#define SVF_STUB(IDX, NAME, PARAMS) static void stub_##NAME PARAMS { flush(); launch_refused(#NAME, cudaSuccess); }
SILVANN_B200_NN_DOORS(SVF_STUB)
#undef SVF_STUB

static sv::DecodeCall decode_call_for(const Pending& x, void* o, float* res, const uint16_t* v, unsigned int* over) {
    sv::DecodeCall c;
    memset(&c, 0, sizeof c);
    c.o = o; c.res = res; c.q = x.q; c.k = x.k; c.v = v; c.kv_rows = x.length;
    c.seqs = 1; c.q_heads = (uint32_t)x.qh; c.kv_heads = (uint32_t)x.kvh; c.head_dim = (uint32_t)x.d; c.length = (uint32_t)x.length;
    c.dtype = SV_DTYPE_FP16; c.over = over; c.stream = 0;
    return c;
}
static bool small_enough(uint64_t qh, uint64_t kvh, uint64_t d, uint64_t length) {
    return qh && kvh && d && length && qh < (1u << 16) && kvh < (1u << 16) && d <= 1024 && length < 0x7FFFFFFFull;
}

static void d_attention_scores(float* p, const sv_h16* q, const sv_h16* k, sv_u64 qh, sv_u64 kvh, sv_u64 d, sv_u64 length) {
    flush();
    const int dev = current_device();
    if (fuse_enabled() && dev >= 0 && dev < DEVICES_MAX && small_enough(qh, kvh, d, length)) {
        std::lock_guard<std::mutex> hold(g_pending_lock[dev]);
        g_pending[dev] = Pending{SCORES, p, nullptr, q, k, qh, kvh, d, length, 0, 0};
        return;
    }
    check("attention_scores", sv::scores_launch(p, q, k, qh, kvh, d, length, 0, nullptr, 0));
}
static void d_attention_mix(sv_h16* o, const float* p, const sv_h16* v, sv_u64 qh, sv_u64 kvh, sv_u64 d, sv_u64 length, sv_fault* over) {
    const int dev = current_device();
    if (dev >= 0 && dev < DEVICES_MAX) {
        std::lock_guard<std::mutex> hold(g_pending_lock[dev]);
        Pending& x = g_pending[dev];
        if (x.kind == GROUPED_SOFT && x.p == p && x.k == v && x.qh == qh && x.kvh == kvh && x.d == d && x.length == length && ((uintptr_t)o & 1u) == 0) {
            const Pending y = x;
            x.kind = NONE;
            const cudaError_t e = sv::mla_decode_launch(o, nullptr, y.q, y.k, qh, length, SV_DTYPE_FP16, 0, over, 0);
            if (e == cudaSuccess) { bump(SILVANN_B200_COUNTER_FUSED_LATENT); return; }
            (void)cudaGetLastError();               /* the fused launch was not taken: the three doors as worded */
            x = y;
        }
        if (x.kind == SCORES && x.p == p && x.qh == qh && x.kvh == kvh && x.d == d && x.length == length) {
            sv::DecodeCall c = decode_call_for(x, o, nullptr, v, over);
            if (sv::decode_fits(c) && sv::decode_device_scratch(&c.scratch) == cudaSuccess) {
                /* a fused launch the runtime does not take (a tensor map it cannot encode, scratch too small for the shape) is
                 * not the caller's error: the recorded door and this one then run as worded */
                if (sv::decode_launch(c) == cudaSuccess) { x.kind = NONE; bump(SILVANN_B200_COUNTER_FUSED_DECODE); return; }
                (void)cudaGetLastError();
            }
        }
        run_pending_locked(x);
    }
    check("attention_mix", sv::mix_launch(o, nullptr, p, v, qh, kvh, d, length, over, 0));
}
static void d_attention_weights(float* p, float* res, const sv_h16* q, const sv_h16* k, sv_u64 qh, sv_u64 kvh, sv_u64 d, sv_u64 length) {
    flush();
    const int dev = current_device();
    if (fuse_enabled() && dev >= 0 && dev < DEVICES_MAX && small_enough(qh, kvh, d, length)) {
        std::lock_guard<std::mutex> hold(g_pending_lock[dev]);
        g_pending[dev] = Pending{WEIGHTS, p, res, q, k, qh, kvh, d, length, 0, 0};
        return;
    }
    check("attention_weights", sv::scores_launch(p, q, k, qh, kvh, d, length, 1, res, 0));
}
static void d_attention_residual_mix(float* res, const float* p, const sv_h16* v, sv_u64 qh, sv_u64 kvh, sv_u64 d, sv_u64 length) {
    const int dev = current_device();
    if (dev >= 0 && dev < DEVICES_MAX) {
        std::lock_guard<std::mutex> hold(g_pending_lock[dev]);
        Pending& x = g_pending[dev];
        if (x.kind == WEIGHTS && x.p == p && x.res == res && x.qh == qh && x.kvh == kvh && x.d == d && x.length == length) {
            sv::DecodeCall c = decode_call_for(x, nullptr, res, v, nullptr);
            if (sv::decode_fits(c) && sv::decode_device_scratch(&c.scratch) == cudaSuccess) {
                if (sv::decode_launch(c) == cudaSuccess) { x.kind = NONE; bump(SILVANN_B200_COUNTER_FUSED_RESIDUAL); return; }
                (void)cudaGetLastError();
            }
        }
        run_pending_locked(x);
    }
    check("attention_residual_mix", sv::mix_launch(nullptr, res, p, v, qh, kvh, d, length, nullptr, 0));
}
static void d_attention_merge(float* into, const float* a, const float* b, sv_u64 qh, sv_u64 d) {
    flush();
    check("attention_merge", sv::merge_launch(into, a, b, qh, d, 0));
}
static void d_attention_finish(sv_h16* o, const float* res, sv_u64 qh, sv_u64 d, sv_fault* over) {
    flush();
    check("attention_finish", sv::finish_launch(o, res, qh, d, over, SV_DTYPE_FP16, 0));
}
/* Latent attention at decode is three doors on one buffer — scores_grouped, softmax_rows, mix with the keys' rows as the
 * values (ai_z__glm_5_3 layer__abi.cuh:279-289).  The first two are recorded when the shape is the fused kernel's; if the
 * mix that follows names the same weights and the same rows, one kernel answers all three and the weights are never
 * written; any other door first runs what was recorded, as worded. */
static void d_attention_scores_grouped(float* p, const sv_h16* q, const sv_h16* k, sv_u64 qh, sv_u64 kvh, sv_u64 d, sv_u64 length) {
    flush();
    const int dev = current_device();
    if (fuse_enabled() && dev >= 0 && dev < DEVICES_MAX && kvh == 1 && sv::mla_decode_fits(q, k, qh, d, length)) {
        std::lock_guard<std::mutex> hold(g_pending_lock[dev]);
        g_pending[dev] = Pending{GROUPED_RAW, p, nullptr, q, k, qh, kvh, d, length, 0, 0};
        return;
    }
    check("attention_scores_grouped", sv::scores_launch(p, q, k, qh, kvh, d, length, 2, nullptr, 0));
}
static void d_attention_softmax_rows(float* p, sv_u64 rows, sv_u64 length) {
    const int dev = current_device();
    if (dev >= 0 && dev < DEVICES_MAX) {
        std::lock_guard<std::mutex> hold(g_pending_lock[dev]);
        Pending& x = g_pending[dev];
        if (x.kind == GROUPED_RAW && x.p == p && x.qh == rows && x.length == length) { x.kind = GROUPED_SOFT; return; }
        run_pending_locked(x);
    }
    check("attention_softmax_rows", sv::softmax_rows_launch(p, rows, length, 0));
}
static void d_attention_causal_scores(float* p, const sv_h16* q, const sv_h16* k, sv_u64 qh, sv_u64 kvh, sv_u64 d, sv_u64 first, sv_u64 rows) {
    flush();
    const int dev = current_device();
    if (fuse_enabled() && dev >= 0 && dev < DEVICES_MAX && small_enough(qh, kvh, d, first + rows)) {
        std::lock_guard<std::mutex> hold(g_pending_lock[dev]);
        g_pending[dev] = Pending{CAUSAL_SOFT, p, nullptr, q, k, qh, kvh, d, 0, first, rows};
        return;
    }
    check("attention_causal_scores", sv::causal_scores_launch(p, q, k, qh, kvh, d, first, rows, true, 0));
}
static void d_attention_causal_scores_grouped(float* p, const sv_h16* q, const sv_h16* k, sv_u64 qh, sv_u64 kvh, sv_u64 d, sv_u64 first, sv_u64 rows) {
    flush();
    const int dev = current_device();
    if (fuse_enabled() && dev >= 0 && dev < DEVICES_MAX && small_enough(qh, kvh, d, first + rows)) {
        std::lock_guard<std::mutex> hold(g_pending_lock[dev]);
        g_pending[dev] = Pending{CAUSAL_RAW, p, nullptr, q, k, qh, kvh, d, 0, first, rows};
        return;
    }
    check("attention_causal_scores_grouped", sv::causal_scores_launch(p, q, k, qh, kvh, d, first, rows, false, 0));
}
static void d_attention_causal_softmax(float* p, sv_u64 qh, sv_u64 first, sv_u64 rows) {
    const int dev = current_device();
    if (dev >= 0 && dev < DEVICES_MAX) {
        std::lock_guard<std::mutex> hold(g_pending_lock[dev]);
        Pending& x = g_pending[dev];
        if (x.kind == CAUSAL_RAW && x.p == p && x.qh == qh && x.first == first && x.rows == rows) { x.kind = CAUSAL_SOFT; return; }
        run_pending_locked(x);
    }
    check("attention_causal_softmax", sv::causal_softmax_launch(p, qh, first, rows, 0));
}
static void d_attention_causal_mix(sv_h16* o, const float* p, const sv_h16* v, sv_u64 qh, sv_u64 kvh, sv_u64 d, sv_u64 first, sv_u64 rows, sv_fault* over) {
    const int dev = current_device();
    if (dev >= 0 && dev < DEVICES_MAX) {
        std::lock_guard<std::mutex> hold(g_pending_lock[dev]);
        Pending& x = g_pending[dev];
        if (x.kind == CAUSAL_SOFT && x.p == p && x.qh == qh && x.kvh == kvh && x.d == d && x.first == first && x.rows == rows) {
            sv::PrefillCall c;
            memset(&c, 0, sizeof c);
            c.o = o; c.q = x.q; c.k = x.k; c.v = v; c.q_heads = (uint32_t)qh; c.kv_heads = (uint32_t)kvh; c.head_dim = (uint32_t)d;
            c.first = first; c.rows = rows; c.dtype = SV_DTYPE_FP16; c.over = over; c.stream = 0;
            if (sv::prefill_fits(c)) {
                if (sv::prefill_launch(c) == cudaSuccess) { x.kind = NONE; bump(SILVANN_B200_COUNTER_FUSED_PREFILL); return; }
                (void)cudaGetLastError();              /* not taken: the recorded doors and this one as worded */
            }
        }
        run_pending_locked(x);
    }
    check("attention_causal_mix", sv::causal_mix_launch(o, p, v, qh, kvh, d, first, rows, over, 0));
}
static void d_attention_weights_rows(float* p, float* res, const sv_h16* q, const sv_h16* k, sv_u64 qh, sv_u64 kvh, sv_u64 d, sv_u64 first, sv_u64 rows) {
    flush();
    const int dev = current_device();
    if (dev >= 0 && dev < DEVICES_MAX && small_enough(qh, kvh, d, first + rows) && rows) {
        std::lock_guard<std::mutex> hold(g_pending_lock[dev]);
        g_pending[dev] = Pending{WEIGHTS_ROWS, p, res, q, k, qh, kvh, d, 0, first, rows};
        if (!fuse_enabled()) run_pending_locked(g_pending[dev]);
        return;
    }
    launch_refused("attention_weights_rows", cudaSuccess);
}
static void d_attention_residual_mix_rows(float* res, const float* p, const sv_h16* v, sv_u64 qh, sv_u64 kvh, sv_u64 d, sv_u64 first, sv_u64 rows) {
    const int dev = current_device();
    if (dev >= 0 && dev < DEVICES_MAX) {
        std::lock_guard<std::mutex> hold(g_pending_lock[dev]);
        Pending& x = g_pending[dev];
        if (x.kind == WEIGHTS_ROWS && x.p == p && x.res == res && x.qh == qh && x.kvh == kvh && x.d == d && x.first == first && x.rows == rows) {
            sv::PrefillCall c;
            memset(&c, 0, sizeof c);
            c.res = res; c.q = x.q; c.k = x.k; c.v = v; c.q_heads = (uint32_t)qh; c.kv_heads = (uint32_t)kvh; c.head_dim = (uint32_t)d;
            c.first = first; c.rows = rows; c.dtype = SV_DTYPE_FP16; c.stream = 0;
            if (sv::prefill_fits(c)) {
                if (sv::prefill_launch(c) == cudaSuccess) { x.kind = NONE; bump(SILVANN_B200_COUNTER_FUSED_PREFILL); return; }
                (void)cudaGetLastError();              /* not taken: the recorded door and this one as worded */
            }
        }
        run_pending_locked(x);
    }
    const uint64_t span = first + rows;
    for (uint64_t r = 0; r < rows; ++r)
        check("attention_residual_mix_rows", sv::mix_launch(nullptr, res + r * qh * (d + 2), p + r * qh * span, v, qh, kvh, d, first + r + 1, nullptr, 0));
}
static void d_attention_scores_grouped_rows(float* p, sv_u64 p_row, const sv_h16* q, sv_u64 q_row, const sv_h16* k, sv_u64 k_row, const sv_u32* lens,
                                            sv_u64 qh, sv_u64 kvh, sv_u64 d, sv_u64 most, sv_u64 rows) {
    flush(); (void)most;
    check("attention_scores_grouped_rows", sv::scores_grouped_rows_launch(p, p_row, q, q_row, k, k_row, lens, qh, kvh, d, rows, 0));
}
static void d_attention_softmax_lens(float* p, sv_u64 p_row, const sv_u32* lens, sv_u64 heads, sv_u64 rows) {
    flush();
    check("attention_softmax_lens", sv::softmax_lens_launch(p, p_row, lens, heads, rows, 0));
}
static void d_attention_softmax_sink(float* p, const sv_h16* sink, sv_u64 rows, sv_u64 length) {
    flush();
    check("attention_softmax_sink", sv::softmax_sink_launch(p, sink, rows, length, 0));
}
static void d_attention_mix_rows(sv_h16* o, sv_u64 o_row, const float* p, sv_u64 p_row, const sv_h16* v, sv_u64 v_row, const sv_u32* lens,
                                 sv_u64 qh, sv_u64 kvh, sv_u64 d, sv_u64 rows, sv_fault* over) {
    flush();
    check("attention_mix_rows", sv::mix_rows_launch(o, o_row, p, p_row, v, v_row, lens, qh, kvh, d, rows, over, 0));
}
static void d_deltanet_gates_rows(sv_h16* beta, sv_h16* g, const sv_h16* a, const sv_h16* b, const sv_h16* a_log, const sv_h16* dt_bias,
                                  sv_u64 heads, sv_u64 rows, sv_fault* over) {
    flush();
    check("deltanet_gates_rows", sv::deltanet_gates_rows_launch(beta, g, a, b, a_log, dt_bias, heads, rows, over, 0));
}
static void d_deltanet_conv_step(sv_h16* o, sv_h16* s, const sv_h16* w, const sv_h16* x, sv_u64 ch, sv_fault* over) {
    flush();
    check("deltanet_conv_step", sv::deltanet_conv_steps_launch(o, s, w, x, ch, 1, over, 0));
}
static void d_deltanet_conv_steps(sv_h16* o, sv_h16* s, const sv_h16* w, const sv_h16* x, sv_u64 ch, sv_u64 rows, sv_fault* over) {
    flush();
    check("deltanet_conv_steps", sv::deltanet_conv_steps_launch(o, s, w, x, ch, rows, over, 0));
}
static void deltanet_door(const char* name, float* S, const sv_h16* conved, const sv_h16* z, const sv_h16* beta, const sv_h16* g, const sv_h16* w,
                          sv_h16* out, sv_u64 kh, sv_u64 vh, sv_u64 d, sv_u64 rows, unsigned gate, sv_fault* over) {
    flush();
    sv::DeltaCall c;
    memset(&c, 0, sizeof c);
    c.S = S; c.conved = conved; c.z = z; c.beta = beta; c.g = g; c.w = w; c.out = out;
    c.k_heads = (uint32_t)kh; c.v_heads = (uint32_t)vh; c.head_dim = (uint32_t)d; c.seqs = 1; c.rows = rows;
    c.gate = (int)gate; c.dtype = SV_DTYPE_FP16; c.over = over; c.stream = 0;
    if (!sv::deltanet_fits(c)) { launch_refused(name, cudaSuccess); return; }
    check(name, sv::deltanet_launch(c));
    bump(SILVANN_B200_COUNTER_DELTANET);
}
static void d_deltanet_step(float* S, const sv_h16* conved, const sv_h16* z, const sv_h16* beta, const sv_h16* g, const sv_h16* w, sv_h16* out,
                            sv_u64 kh, sv_u64 vh, sv_u64 d, sv_fault* over) {
    deltanet_door("deltanet_step", S, conved, z, beta, g, w, out, kh, vh, d, 1, SILVANN_B200_GATE_SILU, over);
}
static void d_deltanet_steps(float* S, const sv_h16* conved, const sv_h16* z, const sv_h16* beta, const sv_h16* g, const sv_h16* w, sv_h16* out,
                             sv_u64 kh, sv_u64 vh, sv_u64 d, sv_u64 rows, sv_fault* over) {
    deltanet_door("deltanet_steps", S, conved, z, beta, g, w, out, kh, vh, d, rows, SILVANN_B200_GATE_SILU, over);
}
static void d_deltanet_steps_gate(float* S, const sv_h16* conved, const sv_h16* z, const sv_h16* beta, const sv_h16* g, const sv_h16* w, sv_h16* out,
                                  sv_u64 kh, sv_u64 vh, sv_u64 d, sv_u64 rows, unsigned int gate, sv_fault* over) {
    deltanet_door("deltanet_steps_gate", S, conved, z, beta, g, w, out, kh, vh, d, rows, gate, over);
}
static void d_vector_sum(sv_h16* out, sv_vector_parts parts, sv_u64 n, sv_fault* over) {
    flush();
    check("vector_sum", sv::vector_sum_launch(out, parts.at, parts.count, n, over, 0));
}

/* ---- the small steps either side of attention (mixer_doors.cu) ---- */
static void d_vector_add(sv_h16* z, const sv_h16* x, const sv_h16* y, sv_u64 n, sv_fault* over) {
    flush();
    if (n) check("vector_add", sv::vector_add_launch(z, x, y, n, over, 0));
}
static void d_vector_copy(sv_h16* out, const sv_h16* in, sv_u64 n) {
    flush();
    if (n) check("vector_copy", sv::vector_copy_rows_launch(out, n, in, n, n, 1, 0));
}
static void d_vector_copy_rows(sv_h16* out, sv_u64 out_row, const sv_h16* in, sv_u64 in_row, sv_u64 width, sv_u64 rows) {
    flush();
    if (width * rows) check("vector_copy_rows", sv::vector_copy_rows_launch(out, out_row, in, in_row, width, rows, 0));
}
static void d_rmsnorm(sv_h16* o, const sv_h16* x, const sv_h16* w, sv_u64 n, float eps, sv_fault* over) {
    flush();
    if (n) check("rmsnorm", sv::rmsnorm_rows_launch(o, x, w, n, 1, n, n, eps, over, 0));
}
static void d_rmsnorm_rows(sv_h16* o, const sv_h16* x, const sv_h16* w, sv_u64 n, sv_u64 rows, sv_u64 x_stride, sv_u64 o_stride, float eps, sv_fault* over) {
    flush();
    if (n * rows == 0) return;
    /* A mixer norms every head's row and then turns it (rope_rows in place over the same rows): recorded, and one kernel
     * answers both if that is what follows; any other door first runs this one as worded. */
    const int dev = current_device();
    if (fuse_enabled() && dev >= 0 && dev < DEVICES_MAX && n <= 16384) {
        std::lock_guard<std::mutex> hold(g_pending_lock[dev]);
        Pending pd;
        memset(&pd, 0, sizeof pd);
        pd.kind = NORM_ROWS; pd.q = x; pd.k = w; pd.d = n; pd.rows = rows; pd.first = x_stride; pd.length = o_stride; pd.o16 = o; pd.eps = eps; pd.over = over;
        g_pending[dev] = pd;
        return;
    }
    check("rmsnorm_rows", sv::rmsnorm_rows_launch(o, x, w, n, rows, x_stride, o_stride, eps, over, 0));
}
static void d_rope(sv_h16* o, const sv_h16* x, const float* cs, sv_u64 heads, sv_u64 head_dim, sv_fault* over) {
    flush();
    if (heads * (head_dim / 2)) check("rope", sv::rope_rows_launch(o, x, cs, 1, heads, head_dim, 0, head_dim, over, 0));
}
static void d_rope_rows(sv_h16* o, const sv_h16* x, const float* cs, sv_u64 rows, sv_u64 heads, sv_u64 head_stride, sv_u64 row_stride, sv_u64 rot, sv_fault* over) {
    const int dev = current_device();
    if (dev >= 0 && dev < DEVICES_MAX) {
        std::lock_guard<std::mutex> hold(g_pending_lock[dev]);
        Pending& pd = g_pending[dev];
        /* the rows just normed, turned in place: norm row r is head r % heads of position r / heads, a head_stride apart, whole */
        if (pd.kind == NORM_ROWS && x == o && o == pd.o16 && pd.rows == rows * heads && pd.length == head_stride && row_stride == heads * head_stride
            && rot <= pd.d && rot % 2 == 0 && over == pd.over && rows * heads * (rot / 2) != 0) {
            const Pending y = pd;
            pd.kind = NONE;
            const cudaError_t e = sv::rmsnorm_rope_rows_launch(o, y.q, y.k, cs, y.d, y.rows, heads, y.first, y.length, rot, y.eps, over, 0);
            if (e == cudaSuccess) { bump(SILVANN_B200_COUNTER_FUSED_NORM_ROPE); return; }
            (void)cudaGetLastError();                 /* the fused launch was not taken: the two doors as worded */
            pd = y;
        }
        run_pending_locked(pd);
    }
    if (rows * heads * (rot / 2)) check("rope_rows", sv::rope_rows_launch(o, x, cs, rows, heads, head_stride, row_stride, rot, over, 0));
}
static void d_rope_interleaved(sv_h16* o, const sv_h16* x, const float* cs, sv_u64 heads, sv_u64 head_stride, sv_u64 rot, sv_u64 inverse, sv_fault* over) {
    flush();
    if (heads * (rot / 2)) check("rope_interleaved", sv::rope_interleaved_launch(o, x, cs, heads, head_stride, rot, inverse, over, 0));
}
static void d_rope_angles(float* cs, sv_u64 position, float theta, sv_u64 head_dim) {
    flush();
    if (head_dim / 2) check("rope_angles", sv::rope_angles_launch(cs, position, nullptr, theta, head_dim, 1, 0, 0, 0));
}
static void d_rope_angles_rows(float* cs, sv_u64 first, float theta, sv_u64 head_dim, sv_u64 rows) {
    flush();
    if (rows * (head_dim / 2)) check("rope_angles_rows", sv::rope_angles_launch(cs, first, nullptr, theta, head_dim, rows, 0, 0, 0));
}
static void d_rope_angles_mrope_rows(float* cs, const sv_u32* positions, float theta, sv_u64 head_dim, sv_u64 rows, sv_u64 sections) {
    flush();
    if (rows * (head_dim / 2)) check("rope_angles_mrope_rows", sv::rope_angles_launch(cs, 0, positions, theta, head_dim, rows, sections, 1, 0));
}
static void d_rope_angles_axial_rows(float* cs, const sv_u32* positions, float theta, sv_u64 head_dim, sv_u64 rows) {
    flush();
    if (rows * (head_dim / 2)) check("rope_angles_axial_rows", sv::rope_angles_launch(cs, 0, positions, theta, head_dim, rows, 0, 2, 0));
}
static void d_attention_gate_rows(sv_h16* o, const sv_h16* att, const sv_h16* qg, sv_u64 heads, sv_u64 head_dim, sv_fault* over) {
    flush();
    if (heads * head_dim == 0) return;
    /* a mixer gates the answers and then rotates them for the output projection: recorded, and one kernel answers both if
     * hadamard_rotate of these answers is what follows; any other door first runs this one as worded */
    const int dev = current_device();
    if (fuse_enabled() && dev >= 0 && dev < DEVICES_MAX) {
        std::lock_guard<std::mutex> hold(g_pending_lock[dev]);
        Pending pd;
        memset(&pd, 0, sizeof pd);
        pd.kind = GATE_ROWS; pd.o16 = o; pd.q = att; pd.k = qg; pd.qh = heads; pd.d = head_dim; pd.over = over;
        g_pending[dev] = pd;
        return;
    }
    check("attention_gate_rows", sv::attention_gate_rows_launch(o, att, qg, heads, head_dim, over, 0));
}

/* ---- the TurboQuant-coded tiers (tq.cu) ---- */
static void d_turboquant_decode(sv_h16* out, const sv_u8* weights, sv_u64 w_room, const sv_u8* luts, sv_u64 l_room, sv_u64 d, sv_u64 rows,
                                sv_u64 cols, sv_fault* over) {
    flush();
    if (!sv::tq_width_ok(d)) { launch_refused("turboquant_decode", cudaSuccess); return; }
    if (rows * cols == 0) return;
    check("turboquant_decode", sv::tq_decode_launch(out, weights, w_room, luts, l_room, d, rows, cols, over, 0));
}
static void d_hadamard_blocks(sv_h16* out, const sv_h16* in, const sv_h16* sign, sv_u64 n, sv_u64 block, sv_u64 inverse, sv_fault* over) {
    flush();
    if (block < 2 || block > 512 || (block & (block - 1)) != 0 || n % block != 0) { launch_refused("hadamard_blocks", cudaSuccess); return; }
    if (n == 0) return;
    check("hadamard_blocks", sv::hadamard_blocks_launch(out, in, sign, n, block, inverse, over, 0));
}
static void d_turboquant_encode_rows(sv_u8* codes, sv_h16* scales, const sv_h16* x, sv_u64 rows, sv_u64 cols, sv_u64 d, sv_fault* over) {
    flush();
    if ((d != 4 && d != 8) || cols == 0) { launch_refused("turboquant_encode_rows", cudaSuccess); return; }
    if (rows == 0) return;
    check("turboquant_encode_rows", sv::tq_encode_rows_launch(codes, scales, x, rows, cols, d, over, 0));
}
static bool tq_shape_ok(sv_u64 qh, sv_u64 kvh, sv_u64 dh, sv_u64 d) {
    return kvh != 0 && qh % kvh == 0 && dh != 0 && dh <= 8192 && sv::tq_width_ok(d) && d != 16;
}
static void d_attention_weights_tq_rows(float* p, float* res, const sv_h16* q, const sv_u8* codes, const sv_h16* scales, sv_u64 qh, sv_u64 kvh,
                                        sv_u64 dh, sv_u64 length, sv_u64 d, sv_u64 rows) {
    flush();
    if (!tq_shape_ok(qh, kvh, dh, d)) { launch_refused("attention_weights_tq", cudaSuccess); return; }
    if (rows == 0) return;
    const int dev = current_device();
    if (fuse_enabled() && dev >= 0 && dev < DEVICES_MAX && length != 0) {
        /* deferred: if the values' door follows, the pair is one kernel over the coded rows and p is never written */
        std::lock_guard<std::mutex> hold(g_pending_lock[dev]);
        Pending x{WEIGHTS_TQ, p, res, q, (const uint16_t*)codes, qh, kvh, dh, length, 0, rows};
        x.scales = scales; x.width = d;
        g_pending[dev] = x;
        return;
    }
    check("attention_weights_tq", sv::tq_weights_launch(p, res, q, codes, scales, qh, kvh, dh, length, d, rows, 0));
}
static void d_attention_residual_mix_tq_rows(float* res, const float* p, const sv_u8* codes, const sv_h16* scales, sv_u64 qh, sv_u64 kvh,
                                             sv_u64 dh, sv_u64 length, sv_u64 d, sv_u64 rows) {
    if (!tq_shape_ok(qh, kvh, dh, d)) { flush(); launch_refused("attention_residual_mix_tq", cudaSuccess); return; }
    if (rows == 0) { flush(); return; }
    const int dev = current_device();
    if (dev >= 0 && dev < DEVICES_MAX) {
        std::lock_guard<std::mutex> hold(g_pending_lock[dev]);
        Pending& x = g_pending[dev];
        if (x.kind == WEIGHTS_TQ && x.p == p && x.res == res && x.qh == qh && x.kvh == kvh && x.d == dh && x.length == length && x.width == d &&
            x.rows == rows && sv::tq_attend_fits(x.q, x.k, x.scales, codes, scales, qh, kvh, dh, length, d)) {
            const Pending w = x;
            const cudaError_t e = sv::tq_attend_launch(res, w.q, (const uint8_t*)w.k, w.scales, codes, scales, qh, kvh, dh, length, d, rows, 0);
            if (e != cudaErrorInvalidValue) {                                /* the fused kernel took the pair: a row, or a chunk's rows */
                x.kind = NONE;
                check("attention_weights_tq+attention_residual_mix_tq", e);
                bump(SILVANN_B200_COUNTER_FUSED_RESIDUAL);
                return;
            }
            (void)cudaGetLastError();
        }
        run_pending_locked(x);
    }
    check("attention_residual_mix_tq", sv::tq_residual_mix_launch(res, p, codes, scales, qh, kvh, dh, length, d, rows, 0));
}
static void d_attention_weights_tq(float* p, float* res, const sv_h16* q, const sv_u8* codes, const sv_h16* scales, sv_u64 qh, sv_u64 kvh,
                                   sv_u64 dh, sv_u64 length, sv_u64 d) {
    d_attention_weights_tq_rows(p, res, q, codes, scales, qh, kvh, dh, length, d, 1);
}
static void d_attention_residual_mix_tq(float* res, const float* p, const sv_u8* codes, const sv_h16* scales, sv_u64 qh, sv_u64 kvh, sv_u64 dh,
                                        sv_u64 length, sv_u64 d) {
    d_attention_residual_mix_tq_rows(res, p, codes, scales, qh, kvh, dh, length, d, 1);
}

/* ---- the weight path's doors a mixer verb cannot run without, as worded (tq.cu) ---- */
static void d_hadamard_rotate(sv_h16* out, const sv_h16* in, const sv_h16* sign, sv_u64 n, sv_fault* over) {
    const bool apart = !(out < in + n && in < out + n);           /* a lane reads the whole block it writes into */
    const bool shaped = n != 0 && (n < 512 || (n % 512) % 128 == 0);   /* past the whole blocks: a 256 and a 128, or a read past n */
    {
        const int dev = current_device();
        if (dev >= 0 && dev < DEVICES_MAX) {
            std::lock_guard<std::mutex> hold(g_pending_lock[dev]);
            Pending& pd = g_pending[dev];
            /* the answers just gated, rotated: one kernel (the rotated row must lie apart from everything the gate reads) */
            if (pd.kind == GATE_ROWS && in == pd.o16 && n == pd.qh * pd.d && apart && shaped && over == pd.over
                && !(out < pd.q + n && pd.q < out + n) && !(out < pd.k + 2 * n && pd.k < out + n)) {
                const Pending y = pd;
                pd.kind = NONE;
                const cudaError_t e = sv::gate_rotate_launch(out, y.o16, y.q, y.k, sign, y.qh, y.d, over, 0);
                if (e == cudaSuccess) { bump(SILVANN_B200_COUNTER_FUSED_NORM_ROPE); return; }
                (void)cudaGetLastError();
                pd = y;
            }
            run_pending_locked(pd);
        }
    }
    if (!apart || !shaped) { launch_refused("hadamard_rotate", cudaSuccess); return; }
    check("hadamard_rotate", sv::hadamard_rotate_launch(out, in, sign, n, over, 0));
}
static void d_rmsnorm_rotate(sv_h16* rot, sv_h16* o, const sv_h16* x, const sv_h16* w, const sv_h16* sign, sv_u64 n, float eps, sv_fault* over) {
    /* nn's definition: the two doors, one after the other.  One kernel with their bits where the row is the rotation door's
     * shape and the three rows lie apart (every block reads all of x while others write o) */
    const bool apart = !(rot < o + n && o < rot + n) && !(o < x + n && x < o + n) && !(rot < x + n && x < rot + n);
    const bool shaped = n != 0 && (n < 512 || (n % 512) % 128 == 0);
    if (fuse_enabled() && apart && shaped) {
        flush();
        const cudaError_t e = sv::rmsnorm_rotate_launch(rot, o, x, w, sign, n, eps, over, 0);
        if (e == cudaSuccess) return;
        (void)cudaGetLastError();
    }
    d_rmsnorm(o, x, w, n, eps, over);
    d_hadamard_rotate(rot, o, sign, n, over);
}
static bool gemv_fast_off() {
    static const bool off = [] { const char* e = getenv("SILVANN_B200_GEMV_AS_WORDED"); return e && e[0] == '1'; }();
    return off;
}
static void d_turboquant_gemv(sv_h16* out, const sv_u8* weights, sv_u64 w_room, const sv_u8* luts, sv_u64 l_room, const sv_h16* x, sv_u64 d,
                              sv_u64 rows, sv_u64 cols, sv_fault* over) {
    flush();
    if (!sv::tq_width_ok(d)) { launch_refused("turboquant_gemv", cudaSuccess); return; }
    if (rows == 0 || cols == 0) return;
    sv_tq_groups g;
    memset(&g, 0, sizeof g);
    g.codes[0] = (sv_u64)(uintptr_t)weights; g.luts[0] = (sv_u64)(uintptr_t)luts; g.rows[0] = rows; g.d[0] = d; g.out_at[0] = 0; g.count = 1;
    if (!gemv_fast_off() && sv::tq_gemv_fast_fits(&g, cols, 1)) {
        const sv_u64 row_bytes = cols * d / 8;
        sv_u64 cap = rows;                                                  /* a row its rooms do not hold is left alone */
        if (w_room / row_bytes < cap) cap = w_room / row_bytes;
        if (l_room / 2 < cap) cap = l_room / 2;
        const cudaError_t e = sv::tq_gemv_fast_launch(out, &g, &cap, x, cols, 1, 0, over, 0);
        if (e != cudaErrorInvalidValue) { if (e == cudaSuccess) bump(SILVANN_B200_COUNTER_GEMV_FAST); check("turboquant_gemv", e); return; }
        (void)cudaGetLastError();
    }
    check("turboquant_gemv", sv::tq_gemv_groups_launch(out, &g, w_room ? w_room : 1, l_room ? l_room : 1, x, cols, over, 0));
}
static void d_turboquant_gemv_groups_n(sv_h16* out, sv_tq_groups g, const sv_h16* x, sv_u64 cols, sv_u64 n, sv_u64 out_stride, sv_fault* over) {
    flush();
    if (g.count == 0 || cols == 0 || n == 0) return;
    if (g.count > 12) { launch_refused("turboquant_gemv_groups", cudaSuccess); return; }
    if (!gemv_fast_off() && sv::tq_gemv_fast_fits(&g, cols, n)) {
        const cudaError_t e = sv::tq_gemv_fast_launch(out, &g, nullptr, x, cols, n, out_stride, over, 0);
        if (e != cudaErrorInvalidValue) { if (e == cudaSuccess) bump(SILVANN_B200_COUNTER_GEMV_FAST); check("turboquant_gemv_groups", e); return; }
        (void)cudaGetLastError();
    }
    for (sv_u64 k = 0; k < n; ++k) {                                        /* as worded: the one-input door an input at a time */
        sv_tq_groups gk = g;
        sv_h16* o = out;
        if (out_stride != 0) o += k * out_stride;
        else for (sv_u64 i = 0; i < gk.count; ++i) gk.out_at[i] += k * gk.rows[i];
        const cudaError_t e = sv::tq_gemv_groups_launch(o, &gk, 0, 0, x + k * cols, cols, over, 0);
        if (e == cudaErrorInvalidValue) { (void)cudaGetLastError(); launch_refused("turboquant_gemv_groups", cudaSuccess); return; }
        check("turboquant_gemv_groups", e);
    }
}
static void d_turboquant_gemv_groups(sv_h16* out, sv_tq_groups g, const sv_h16* x, sv_u64 cols, sv_fault* over) {
    d_turboquant_gemv_groups_n(out, g, x, cols, 1, 0, over);
}

/* ---- the expert-major GEMM doors a prompt's projections go through (expert.cu) ---- */
static bool expert_fast_off() {
    static const bool off = [] { const char* e = getenv("SILVANN_B200_EXPERT_AS_WORDED"); return e && e[0] == '1'; }();
    return off;
}
static void expert_rows_any(const char* door, sv_h16* out, float* acc, const sv_u8* weights, sv_u64 w_room, const sv_u8* luts, sv_u64 l_room, const sv_h16* x,
                            const sv_u32* rows, const sv_h16* w, sv_u64 count, sv_u64 d, sv_u64 out_rows, sv_u64 cols, sv_fault* over) {
    flush();
    if (!sv::expert_width_ok(d)) { launch_refused(door, cudaSuccess); return; }
    if (count == 0 || out_rows == 0 || cols == 0) return;
    sv_expert_groups g;
    memset(&g, 0, sizeof g);
    g.codes[0] = (sv_u64)(uintptr_t)weights; g.luts[0] = (sv_u64)(uintptr_t)luts; g.out_rows[0] = out_rows; g.d[0] = d; g.pairs[0] = count; g.count = 1;
    if (!expert_fast_off() && sv::expert_fast_fits(&g, x, cols)) {
        const sv_u64 row_bytes = cols * d / 8;
        sv_u64 held = w_room / row_bytes;                                   /* a row its rooms do not hold is computed and not written */
        if (d != 16 && l_room / 2 < held) held = l_room / 2;
        if (held == 0) return;
        const cudaError_t e = sv::expert_fast_launch(out, acc, &g, &held, x, rows, w, cols, over, 0);
        if (e == cudaSuccess) bump(SILVANN_B200_COUNTER_EXPERT_FAST);
        check(door, e);
        return;
    }
    check(door, sv::expert_rows_launch(out, acc, weights, w_room, luts, l_room, x, rows, w, count, d, out_rows, cols, over, 0));
}
static void d_expert_rows(sv_h16* out, const sv_u8* weights, sv_u64 w_room, const sv_u8* luts, sv_u64 l_room, const sv_h16* x, const sv_u32* rows, sv_u64 count,
                          sv_u64 d, sv_u64 out_rows, sv_u64 cols, sv_fault* over) {
    expert_rows_any("expert_rows", out, nullptr, weights, w_room, luts, l_room, x, rows, nullptr, count, d, out_rows, cols, over);
}
static void d_expert_rows_sum(float* acc, const sv_u8* weights, sv_u64 w_room, const sv_u8* luts, sv_u64 l_room, const sv_h16* x, const sv_u32* rows,
                              const sv_h16* w, sv_u64 count, sv_u64 d, sv_u64 out_rows, sv_u64 cols) {
    expert_rows_any("expert_rows_sum", nullptr, acc, weights, w_room, luts, l_room, x, rows, w, count, d, out_rows, cols, nullptr);
}
static void d_expert_groups(sv_h16* out, sv_expert_groups g, const sv_h16* x, const sv_u32* rows, sv_u64 cols, sv_fault* over) {
    flush();
    if (g.count == 0 || cols == 0) return;
    if (g.count > 12) { launch_refused("expert_groups", cudaSuccess); return; }
    for (sv_u64 i = 0; i < g.count; ++i)
        if (!sv::expert_width_ok(g.d[i])) { launch_refused("expert_groups", cudaSuccess); return; }
    sv_expert_groups live = g;                                              /* groups with rows and pairs */
    live.count = 0;
    for (sv_u64 i = 0; i < g.count; ++i)
        if (g.out_rows[i] != 0 && g.pairs[i] != 0) {
            const sv_u64 k = live.count++;
            live.codes[k] = g.codes[i]; live.luts[k] = g.luts[i]; live.out_rows[k] = g.out_rows[i]; live.d[k] = g.d[i]; live.out_at[k] = g.out_at[i];
            live.pairs_at[k] = g.pairs_at[i]; live.pairs[k] = g.pairs[i];
        }
    if (live.count == 0) return;
    if (!expert_fast_off() && sv::expert_fast_fits(&live, x, cols)) {
        const cudaError_t e = sv::expert_fast_launch(out, nullptr, &live, nullptr, x, rows, nullptr, cols, over, 0);
        if (e == cudaSuccess) bump(SILVANN_B200_COUNTER_EXPERT_FAST);
        check("expert_groups", e);
        return;
    }
    for (sv_u64 i = 0; i < live.count; ++i) {                               /* as worded: the one-matrix door a group at a time */
        const sv_u64 row_bytes = ((cols + 16 / live.d[i] - 1) / (16 / live.d[i])) * 2;
        check("expert_groups", sv::expert_rows_launch(out + live.out_at[i], nullptr, (const sv_u8*)(uintptr_t)live.codes[i], live.out_rows[i] * row_bytes,
                                                      (const sv_u8*)(uintptr_t)live.luts[i], live.out_rows[i] * 2, x, rows + 2 * live.pairs_at[i], nullptr,
                                                      live.pairs[i], live.d[i], live.out_rows[i], cols, over, 0));
    }
}
static void d_expert_rows_finish(sv_h16* out, float* acc, const sv_h16* residual, sv_u64 n, sv_fault* over) {
    flush();
    if (n) check("expert_rows_finish", sv::expert_rows_finish_launch(out, acc, residual, n, over, 0));
}
static void d_expert_rows_reduce(sv_h16* out, float* acc, const sv_h16* residual, sv_u64 n, sv_u64 k, sv_u64 cols, sv_fault* over) {
    flush();
    if (n * cols) check("expert_rows_reduce", sv::expert_rows_reduce_launch(out, acc, residual, n, k, cols, over, 0));
}
static void d_expert_pairs_rows(sv_u32* pairs, sv_u64 n, sv_u64 x_step, sv_u64 x_at, sv_u64 out_step, sv_u64 out_at) {
    flush();
    if (n) check("expert_pairs_rows", sv::expert_pairs_rows_launch(pairs, n, x_step, x_at, out_step, out_at, 0));
}
/* A 16-bit matrix times one vector, or n of them, is the coded door at width 16: the codes are the halves, the scale is 1. */
static void d_expert_multiply_fp16_rows(sv_h16* out, const sv_h16* W, const sv_h16* x, sv_u64 rows, sv_u64 cols, sv_u64 n, sv_fault* over) {
    if (rows == 0 || cols == 0 || n == 0) { flush(); return; }
    sv_tq_groups g;
    memset(&g, 0, sizeof g);
    g.codes[0] = (sv_u64)(uintptr_t)W; g.luts[0] = 0; g.rows[0] = rows; g.d[0] = 16; g.out_at[0] = 0; g.count = 1;
    d_turboquant_gemv_groups_n(out, g, x, cols, n, 0, over);
}
static void d_expert_multiply_fp16(sv_h16* out, const sv_h16* W, const sv_h16* x, sv_u64 rows, sv_u64 cols, sv_fault* over) {
    d_expert_multiply_fp16_rows(out, W, x, rows, cols, 1, over);
}

/* ---- the GLM mixer's doors (glm_doors.cu): KDA, the latent's absorb and expand, the indexer ---- */
static void d_kda_steps(float* S, const sv_h16* conved, const sv_h16* f, const sv_h16* b, const sv_h16* dt, const sv_h16* a_log, const sv_h16* gate,
                        const sv_h16* w, sv_h16* out, sv_u64 heads, sv_u64 head_dim, float lower, float eps, sv_u64 rows, sv_fault* over) {
    flush();
    if (heads == 0 || head_dim == 0 || rows == 0) return;
    check("kda_steps", sv::kda_steps_launch(S, conved, f, nullptr, b, dt, a_log, gate, w, out, heads, head_dim, lower, eps, rows, over, 0));
}
static void d_kda_step(float* S, const sv_h16* conved, const sv_h16* f, const sv_h16* b, const sv_h16* dt, const sv_h16* a_log, const sv_h16* gate,
                       const sv_h16* w, sv_h16* out, sv_u64 heads, sv_u64 head_dim, float lower, float eps, sv_fault* over) {
    d_kda_steps(S, conved, f, b, dt, a_log, gate, w, out, heads, head_dim, lower, eps, 1, over);      /* one row: q, k, v side by side */
}
static void d_kda_decays(float* eg, const sv_h16* f, const sv_h16* dt, const sv_h16* a_log, sv_u64 heads, sv_u64 head_dim, float lower, sv_u64 rows) {
    flush();
    if (heads * head_dim * rows == 0) return;
    check("kda_decays", sv::kda_decays_launch(eg, f, dt, a_log, heads, head_dim, lower, rows, 0));
}
static void d_kda_steps_decayed(float* S, const sv_h16* conved, const float* eg, const sv_h16* b, const sv_h16* gate, const sv_h16* w, sv_h16* out,
                                sv_u64 heads, sv_u64 head_dim, float eps, sv_u64 rows, sv_fault* over) {
    flush();
    if (heads == 0 || head_dim == 0 || rows == 0) return;
    if (eg == nullptr) { launch_refused("kda_steps_decayed", cudaSuccess); return; }
    check("kda_steps_decayed", sv::kda_steps_launch(S, conved, nullptr, eg, b, nullptr, nullptr, gate, w, out, heads, head_dim, 0.f, eps, rows, over, 0));
}
static void d_attention_absorb_rows(sv_h16* out, const sv_h16* q, const sv_h16* W, sv_u64 heads, sv_u64 nope, sv_u64 latent, sv_u64 stride, float scale,
                                    sv_u64 rows, sv_fault* over) {
    flush();
    if (heads * latent * rows == 0) return;
    const cudaError_t e = sv::absorb_launch(out, q, W, heads, nope, latent, stride, scale, rows, over, 0);
    if (e == cudaErrorInvalidValue) { (void)cudaGetLastError(); launch_refused("attention_absorb", cudaSuccess); return; }
    check("attention_absorb", e);
}
static void d_attention_absorb(sv_h16* out, const sv_h16* q, const sv_h16* W, sv_u64 heads, sv_u64 nope, sv_u64 latent, sv_u64 stride, float scale,
                               sv_fault* over) {
    d_attention_absorb_rows(out, q, W, heads, nope, latent, stride, scale, 1, over);
}
static void d_attention_expand_rows(sv_h16* out, const sv_h16* o, const sv_h16* W, sv_u64 heads, sv_u64 width, sv_u64 latent, sv_u64 stride, sv_u64 offset,
                                    sv_u64 rows, sv_fault* over) {
    flush();
    if (heads * width * rows == 0) return;
    check("attention_expand", sv::expand_launch(out, o, W, heads, width, latent, stride, offset, rows, over, 0));
}
static void d_attention_expand(sv_h16* out, const sv_h16* o, const sv_h16* W, sv_u64 heads, sv_u64 width, sv_u64 latent, sv_u64 stride, sv_u64 offset,
                               sv_fault* over) {
    d_attention_expand_rows(out, o, W, heads, width, latent, stride, offset, 1, over);
}
static void d_index_layernorm(sv_h16* o, const sv_h16* x, const sv_h16* w, const sv_h16* b, sv_u64 n, float eps, sv_fault* over) {
    flush();
    if (n == 0) return;
    check("index_layernorm", sv::index_layernorm_launch(o, x, w, b, n, eps, over, 0));
}
static void d_index_pool(sv_h16* pooled, const sv_h16* keys, const sv_h16* gates, const sv_h16* ape, sv_u64 first, sv_u64 pools, sv_u64 dim, sv_u64 kpool,
                         sv_fault* over) {
    flush();
    if (pools * dim == 0) return;
    check("index_pool", sv::index_pool_launch(pooled, keys, gates, ape, first, pools, dim, kpool, over, 0));
}
static void d_index_scores(float* scores, const sv_h16* q, const sv_h16* w, const sv_h16* pooled, sv_u64 heads, sv_u64 dim, sv_u64 pools, float scale) {
    flush();
    if (pools == 0) return;
    check("index_scores", sv::index_scores_launch(scores, 0, q, w, pooled, heads, dim, pools, 0, 1, 0, scale, 0));
}
static void d_index_scores_rows(float* scores, sv_u64 scores_row, const sv_h16* q, const sv_h16* w, const sv_h16* pooled, sv_u64 heads, sv_u64 dim,
                                sv_u64 len0, sv_u64 kpool, sv_u64 rows, float scale) {
    flush();
    if (rows == 0 || kpool == 0 || (len0 + rows - 1) / kpool == 0) return;
    check("index_scores_rows", sv::index_scores_launch(scores, scores_row, q, w, pooled, heads, dim, 0, len0, kpool, rows, scale, 0));
}
static void d_index_select(sv_u32* index, sv_u32* count, const float* scores, sv_u64 pools, sv_u64 k, sv_u64 kpool, sv_u64 tail_first, sv_u64 tail) {
    flush();
    check("index_select", sv::index_select_launch(index, 0, count, scores, 0, pools, k, kpool, tail_first, tail, 0, 0, 0));
}
static void d_index_select_rows(sv_u32* index, sv_u64 index_row, sv_u32* counts, const float* scores, sv_u64 scores_row, sv_u64 k, sv_u64 kpool, sv_u64 len0,
                                sv_u64 rows) {
    flush();
    if (rows == 0) return;
    if (kpool == 0) { launch_refused("index_select_rows", cudaSuccess); return; }
    check("index_select_rows", sv::index_select_launch(index, index_row, counts, scores, scores_row, 0, k, kpool, 0, 0, len0, rows, 0));
}
static void d_index_blocks(float* out, const float* scores, sv_u64 pools, sv_u64 block) {
    flush();
    if (pools == 0) return;
    if (block == 0) { launch_refused("index_blocks", cudaSuccess); return; }
    check("index_blocks", sv::index_blocks_launch(out, scores, pools, block, 0));
}
static void d_index_gather(sv_h16* out, const sv_h16* src, const sv_u32* index, sv_u64 n, sv_u64 row) {
    flush();
    if (n * row == 0) return;
    check("index_gather", sv::index_gather_launch(out, 0, src, index, 0, nullptr, n, row, 1, 0));
}
static void d_index_gather_rows(sv_h16* out, sv_u64 out_row, const sv_h16* src, const sv_u32* index, sv_u64 index_row, const sv_u32* counts, sv_u64 most,
                                sv_u64 row, sv_u64 rows) {
    flush();
    if (rows * most * row == 0) return;
    check("index_gather_rows", sv::index_gather_launch(out, out_row, src, index, index_row, counts, most, row, rows, 0));
}

/* ================================================================================================================ */
/* tables and the entry                                                                                             */

#define SVF_SYS_FILL(IDX, RET, NAME, PARAMS) s_##NAME,
static silvann_b200_sys_doors g_sys = {(uint32_t)sizeof(silvann_b200_sys_doors), SILVANN_B200_SYS_DOORS(SVF_SYS_FILL)};
#undef SVF_SYS_FILL
#define SVF_NN_FILL(IDX, NAME, PARAMS) stub_##NAME,
static silvann_b200_nn_doors g_nn = {(uint32_t)sizeof(silvann_b200_nn_doors), SILVANN_B200_NN_DOORS(SVF_NN_FILL)};
#undef SVF_NN_FILL
static const silvann_b200_empty_doors g_empty = {(uint32_t)sizeof(silvann_b200_empty_doors)};
static const void* const g_packages[SILVANN_B200_PACKAGES] = {&g_sys, &g_nn, &g_empty, &g_empty, &g_empty, &g_empty, &g_empty};
static const silvann_b200_family g_family = {SILVANN_B200_ABI_VERSION, (uint32_t)sizeof(silvann_b200_family), SILVANN_B200_FAMILY_ID,
                                             SILVANN_B200_PACKAGES, SILVANN_B200_FAMILY_NAME, g_packages};

static void install_doors() {
    g_nn.attention_scores = d_attention_scores;
    g_nn.attention_mix = d_attention_mix;
    g_nn.attention_weights = d_attention_weights;
    g_nn.attention_residual_mix = d_attention_residual_mix;
    g_nn.attention_merge = d_attention_merge;
    g_nn.attention_finish = d_attention_finish;
    g_nn.attention_scores_grouped = d_attention_scores_grouped;
    g_nn.attention_softmax_rows = d_attention_softmax_rows;
    g_nn.attention_causal_scores = d_attention_causal_scores;
    g_nn.attention_causal_scores_grouped = d_attention_causal_scores_grouped;
    g_nn.attention_causal_softmax = d_attention_causal_softmax;
    g_nn.attention_causal_mix = d_attention_causal_mix;
    g_nn.deltanet_step = d_deltanet_step;
    g_nn.deltanet_steps = d_deltanet_steps;
    g_nn.deltanet_steps_gate = d_deltanet_steps_gate;
    g_nn.vector_sum = d_vector_sum;
    g_nn.attention_weights_rows = d_attention_weights_rows;
    g_nn.attention_residual_mix_rows = d_attention_residual_mix_rows;
    g_nn.attention_scores_grouped_rows = d_attention_scores_grouped_rows;
    g_nn.attention_softmax_lens = d_attention_softmax_lens;
    g_nn.attention_softmax_sink = d_attention_softmax_sink;
    g_nn.attention_mix_rows = d_attention_mix_rows;
    g_nn.deltanet_gates_rows = d_deltanet_gates_rows;
    g_nn.deltanet_conv_step = d_deltanet_conv_step;
    g_nn.deltanet_conv_steps = d_deltanet_conv_steps;
    g_nn.vector_add = d_vector_add;
    g_nn.vector_copy = d_vector_copy;
    g_nn.vector_copy_rows = d_vector_copy_rows;
    g_nn.rmsnorm = d_rmsnorm;
    g_nn.rmsnorm_rows = d_rmsnorm_rows;
    g_nn.rope = d_rope;
    g_nn.rope_rows = d_rope_rows;
    g_nn.rope_interleaved = d_rope_interleaved;
    g_nn.rope_angles = d_rope_angles;
    g_nn.rope_angles_rows = d_rope_angles_rows;
    g_nn.rope_angles_mrope_rows = d_rope_angles_mrope_rows;
    g_nn.rope_angles_axial_rows = d_rope_angles_axial_rows;
    g_nn.attention_gate_rows = d_attention_gate_rows;
    g_nn.kda_step = d_kda_step;
    g_nn.kda_steps = d_kda_steps;
    g_nn.kda_decays = d_kda_decays;
    g_nn.kda_steps_decayed = d_kda_steps_decayed;
    g_nn.attention_absorb = d_attention_absorb;
    g_nn.attention_absorb_rows = d_attention_absorb_rows;
    g_nn.attention_expand = d_attention_expand;
    g_nn.attention_expand_rows = d_attention_expand_rows;
    g_nn.index_layernorm = d_index_layernorm;
    g_nn.index_pool = d_index_pool;
    g_nn.index_scores = d_index_scores;
    g_nn.index_scores_rows = d_index_scores_rows;
    g_nn.index_select = d_index_select;
    g_nn.index_select_rows = d_index_select_rows;
    g_nn.index_blocks = d_index_blocks;
    g_nn.index_gather = d_index_gather;
    g_nn.index_gather_rows = d_index_gather_rows;
    g_nn.hadamard_rotate = d_hadamard_rotate;
    g_nn.rmsnorm_rotate = d_rmsnorm_rotate;
    g_nn.turboquant_gemv = d_turboquant_gemv;
    g_nn.expert_rows = d_expert_rows;
    g_nn.expert_rows_sum = d_expert_rows_sum;
    g_nn.expert_groups = d_expert_groups;
    g_nn.expert_rows_finish = d_expert_rows_finish;
    g_nn.expert_rows_reduce = d_expert_rows_reduce;
    g_nn.expert_pairs_rows = d_expert_pairs_rows;
    g_nn.expert_multiply_fp16 = d_expert_multiply_fp16;
    g_nn.expert_multiply_fp16_rows = d_expert_multiply_fp16_rows;
    g_nn.turboquant_gemv_groups = d_turboquant_gemv_groups;
    g_nn.turboquant_gemv_groups_n = d_turboquant_gemv_groups_n;
    g_nn.turboquant_decode = d_turboquant_decode;
    g_nn.hadamard_blocks = d_hadamard_blocks;
    g_nn.turboquant_encode_rows = d_turboquant_encode_rows;
    g_nn.attention_weights_tq = d_attention_weights_tq;
    g_nn.attention_residual_mix_tq = d_attention_residual_mix_tq;
    g_nn.attention_weights_tq_rows = d_attention_weights_tq_rows;
    g_nn.attention_residual_mix_tq_rows = d_attention_residual_mix_tq_rows;
}

}  // namespace svf

static_assert(sizeof(silvann_b200_sys_doors) == 256, "sys door table must be 4 + 31 pointers, padded: 256 bytes");
static_assert(sizeof(silvann_b200_nn_doors) == 1104, "nn door table must be 4 + 137 pointers, padded: 1104 bytes");
static_assert(sizeof(sv_tq_groups) == 488 && sizeof(sv_expert_groups) == 680 && sizeof(sv_vector_parts) == 72, "by-value door structs");

extern "C" __attribute__((visibility("default")))
const silvann_b200_family* silvann_silicon_family_get(uint32_t abi_version) {
    static std::once_flag once;
    std::call_once(once, svf::install_doors);
    return abi_version == SILVANN_B200_ABI_VERSION ? &svf::g_family : nullptr;
}
