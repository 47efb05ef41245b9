/* exchange.cu — the exchange step of a sharded path as ONE kernel over peer memory: push, signal, wait, combine.
 *
 * Two places of the path end in an exchange among the cards of a box:
 *   - one long sequence whose KV RANGE is split over the cards that share a kv head: each card's split-KV decode leaves a
 *     residual (m, l, acc) per head and the residuals are folded with attention_merge's arithmetic and closed by
 *     attention_finish (engine/src/packages/nn/gpu/kernels/kernels.cuh:1243-1267);
 *   - the tensor-parallel sum that follows head-sharded attention: every card's 16-bit partial of the hidden vector is
 *     added in rank order in fp32 and rounded once (vector_sum, kernels.cuh:117-126; its caller
 *     engine/src/packages/nn/cpu/opcodes/partials__abi.cuh:110-163).
 * The reference does the second inside a kernel that LOADS the peers' partials in place after host-side marks
 * (engine/src/silicon_families/nvidia_cuda12/overrides/vector.cuh:292-331).  Here the data is PUSHED instead: a card
 * stores its piece into a slot of every member's buffer with plain peer stores, as tagged words that carry the exchange's
 * generation number beside their payload (exchange.cuh), and then reads only its own memory, polling — bounded — each word
 * it needs until the tag is the generation.  One launch a card and no host in the loop; the answer is computed redundantly
 * on every member in the same order, so all members hold the same bits.
 *
 * Buffers.  Every member owns one device buffer of [2 parities][members][slot_words] tagged words.  Two parities are
 * enough: a member can run at most one exchange ahead of the slowest (it needs that member's words of exchange t to finish
 * t), so while anyone still reads parity t nobody writes it; a word left from exchange t-2 carries an older tag and reads
 * as not there yet.  Members call the exchange entry points in the same order the same number of times (a collective's
 * contract); the generation counter is the number of exchanges so far and lives on the host.
 *
 * No multicast, no TMA, no library kernel touches peer memory: ordinary st.global / ld.global only.  Every wait is bounded
 * by the wall clock (%globaltimer); when it runs out the block raises "B2TO" in the device status word and stops: the fold
 * writes none of its outputs, a sum none past the word that did not come. */
#include "../../include/silvann_b200.h"
#include "common.cuh"
#include "kernels.h"
#include "residual.cuh"
#include "exchange.cuh"
#include <new>
#include <string.h>

#define SV_EXPORT extern "C" __attribute__((visibility("default")))
#define XF_HEADS_PER_BLOCK 8u                /* heads a block of the fold owns, fewer when a head is longer than 256 */
#define XF_FOLD_ELEMENTS 2048u              /* elements of those heads: 8 a thread, held in registers until all have come */
#define XF_SUM_BLOCKS 592u

int sv_ext_fail(int code, const char* fmt, ...);      /* ext.cu */

struct silvann_b200_exchange {
    int device;
    uint32_t members, index;
    uint64_t slot_bytes;                    /* payload bytes a member's piece may have */
    uint64_t slot_words;                    /* tagged words a slot holds: one a 16-bit value at the least, a multiple of 4 */
    uint8_t* peer[XF_MEMBERS_MAX];          /* every member's buffer as this process addresses it; peer[index] is the local one */
    bool opened[XF_MEMBERS_MAX];            /* mapped here from an inter-process handle (to be closed), not given as an address */
    bool connected;
    uint32_t gen;                           /* exchanges so far */
};

namespace sv {

/* Residuals of the members' ranges -> the whole range's residual and/or its 16-bit output.  A block owns `hb` heads (at most
 * XF_FOLD_ELEMENTS elements).  A word is one fp32 of the residual, at the index it has there. */
template <int DT>
__global__ void __launch_bounds__(256, 1) exchange_merge_kernel(const XfParams P, uint16_t* o, float* res_out, const float* res_local,
                                                             uint32_t q_heads, uint32_t d, uint32_t hb, unsigned int* over) {
    using E = Elem<DT>;
    constexpr uint32_t K = XF_FOLD_ELEMENTS / 256u;
    __shared__ float ms_s[XF_HEADS_PER_BLOCK][XF_MEMBERS_MAX], ls_s[XF_HEADS_PER_BLOCK][XF_MEMBERS_MAX];
    __shared__ float fa_s[XF_HEADS_PER_BLOCK][XF_MEMBERS_MAX], fb_s[XF_HEADS_PER_BLOCK][XF_MEMBERS_MAX], l_s[XF_HEADS_PER_BLOCK], m_s[XF_HEADS_PER_BLOCK];
    const uint32_t parity = P.gen & 1u, w = d + 2u;
    const uint32_t h0 = blockIdx.x * hb, heads = min(hb, q_heads - h0);
    const uint32_t nw = heads * w;
    const size_t off = (size_t)h0 * w;

    /* push: this card's residual of these heads into its slot on every member (its own included) */
    for (uint32_t i = threadIdx.x; i < nw; i += blockDim.x) {
        const uint32_t x = __float_as_uint(res_local[off + i]);
        for (uint32_t m = 0; m < P.members; ++m) xf_store(xf_slot(P.peer[m], parity, P.index, P.slot_words, P.members) + off + i, x, P.gen);
    }

    /* gather: every member's words of this thread's elements, and (the first threads) of the heads' scalars */
    unsigned long long t0 = 0ull;
    bool ok = true;
    uint32_t acc[K][XF_MEMBERS_MAX];
#pragma unroll
    for (uint32_t k = 0; k < K; ++k) {
        const uint32_t i = threadIdx.x + k * 256u;
        if (i < heads * d) { const uint32_t h = i / d; xf_gather(P, parity, off + (size_t)h * w + 2u + (i - h * d), acc[k], t0, ok); }
    }
    if (threadIdx.x < heads * P.members) {
        const uint32_t h = threadIdx.x / P.members, m = threadIdx.x - h * P.members;
        const uint2* at = xf_slot(P.peer[P.index], parity, m, P.slot_words, P.members) + off + (size_t)h * w;
        uint32_t mv = 0u, lv = 0u;
        ok = ok && xf_await(at, P.gen, P.wait_ns, t0, mv);
        ok = ok && xf_await(at + 1, P.gen, P.wait_ns, t0, lv);
        ms_s[h][m] = __uint_as_float(mv); ls_s[h][m] = __uint_as_float(lv);
    }
    if (__syncthreads_or(ok ? 0 : 1)) {                                      /* a word never came: say so, write nothing */
        if (threadIdx.x == 0 && P.status) atomicOr(P.status, SV_STATUS_TIMEOUT);
        return;
    }

    /* every member's residual of these heads is in registers and shared memory now; fold them in member order */
    if (threadIdx.x < heads) {
        const uint32_t h = threadIdx.x;
        float m = ms_s[h][0], l = ls_s[h][0];
        for (uint32_t s = 1; s < P.members; ++s) {
            float fa, fb;
            merge_scalars(m, l, ms_s[h][s], ls_s[h][s], fa, fb);
            fa_s[h][s] = fa; fb_s[h][s] = fb;
        }
        m_s[h] = m; l_s[h] = l;
    }
    __syncthreads();
    bool hit = false;
#pragma unroll
    for (uint32_t k = 0; k < K; ++k) {
        const uint32_t i = threadIdx.x + k * 256u;
        if (i >= heads * d) continue;
        const uint32_t h = i / d, e = i - h * d;
        const size_t at = off + (size_t)h * w + 2u + e;
        float a = __uint_as_float(acc[k][0]);
#pragma unroll
        for (uint32_t s = 1; s < XF_MEMBERS_MAX; ++s)
            if (s < P.members) a = merge_element(a, fa_s[h][s], __uint_as_float(acc[k][s]), fb_s[h][s]);
        if (res_out) { res_out[at] = a; if (e == 0) { res_out[at - 2] = m_s[h]; res_out[at - 1] = l_s[h]; } }
        if (o) o[(size_t)(h0 + h) * d + e] = E::from_float(a / l_s[h], hit);
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* 16-bit partials of the members -> their fp32 sum in member order, rounded once.  A word is a pair of neighbouring values;
 * a thread moves eight values (four words, two 16-byte stores a member) a turn. */
template <int DT>
__global__ void __launch_bounds__(256, 1) exchange_sum_kernel(const XfParams P, uint16_t* out, const uint16_t* partial, uint64_t n, unsigned int* over) {
    using E = Elem<DT>;
    const uint32_t parity = P.gen & 1u;
    const bool wide = ((uintptr_t)partial & 15u) == 0, wide_out = ((uintptr_t)out & 15u) == 0;
    const uint64_t first = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8u, stride = (uint64_t)gridDim.x * blockDim.x * 8u;
    for (uint64_t i = first; i < n; i += stride) {
        uint32_t x[4];
        if (wide && i + 8 <= n) *reinterpret_cast<uint4*>(x) = *reinterpret_cast<const uint4*>(partial + i);
        else for (int u = 0; u < 4; ++u) x[u] = (i + 2 * u < n ? (uint32_t)partial[i + 2 * u] : 0u) | (i + 2 * u + 1 < n ? (uint32_t)partial[i + 2 * u + 1] << 16 : 0u);
        for (uint32_t m = 0; m < P.members; ++m) {
            uint2* to = xf_slot(P.peer[m], parity, P.index, P.slot_words, P.members) + i / 2u;     /* i/2 is a multiple of 4: on 32 bytes */
            xf_store2(to, x[0], x[1], P.gen);
            xf_store2(to + 2, x[2], x[3], P.gen);
        }
    }
    unsigned long long t0 = 0ull;
    bool hit = false;
    uint8_t* local = P.peer[P.index];
    for (uint64_t i = first; i < n; i += stride) {
        uint4 v[XF_MEMBERS_MAX][2];
#pragma unroll
        for (uint32_t m = 0; m < XF_MEMBERS_MAX; ++m)
            if (m < P.members) {
                const uint2* from = xf_slot(local, parity, m, P.slot_words, P.members) + i / 2u;
                v[m][0] = xf_load2(from); v[m][1] = xf_load2(from + 2);
            }
        float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        bool ok = true;
#pragma unroll
        for (uint32_t m = 0; m < XF_MEMBERS_MAX; ++m) {
            if (m >= P.members) continue;
            uint32_t pay[4] = {v[m][0].x, v[m][0].z, v[m][1].x, v[m][1].z};
            const uint32_t tag[4] = {v[m][0].y, v[m][0].w, v[m][1].y, v[m][1].w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (tag[u] != P.gen && ok) ok = xf_await(xf_slot(local, parity, m, P.slot_words, P.members) + i / 2u + u, P.gen, P.wait_ns, t0, pay[u]);
                s[2 * u] += E::to_float((uint16_t)(pay[u] & 0xffffu));
                s[2 * u + 1] += E::to_float((uint16_t)(pay[u] >> 16));
            }
        }
        if (!ok) { if (P.status) atomicOr(P.status, SV_STATUS_TIMEOUT); break; }
        uint16_t y[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) y[u] = E::from_float(s[u], hit);
        if (wide_out && i + 8 <= n) *reinterpret_cast<uint4*>(out + i) = *reinterpret_cast<const uint4*>(y);
        else for (int u = 0; u < 8 && i + u < n; ++u) out[i + u] = y[u];
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* Stands in for a member on a machine with fewer cards than members: its piece as the words of the NEXT exchange.  `unit`
 * is the payload a word carries: 4 bytes (a residual's fp32, or a pair of 16-bit values) or 2 (one 16-bit value a word, the
 * coded projection's rows). */
__global__ void __launch_bounds__(256) exchange_deposit_kernel(uint8_t* local, uint32_t members, uint32_t member, uint64_t slot_words, uint32_t gen,
                                                               const uint16_t* data, uint64_t halves, uint32_t unit) {
    uint2* slot = xf_slot(local, gen & 1u, member, slot_words, members);
    const uint64_t words = unit == 2u ? halves : ((halves + 7u) / 8u) * 4u;                   /* (the sum moves four words a thread, zeros past the end) */
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < words; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t x = unit == 2u ? (uint32_t)data[i] : (2 * i < halves ? (uint32_t)data[2 * i] : 0u) | (2 * i + 1 < halves ? (uint32_t)data[2 * i + 1] << 16 : 0u);
        xf_store(slot + i, x, gen);
    }
}

}  // namespace sv

/* ---------------------------------------------------------------------------------------------------------------------- */

static size_t xf_bytes(const silvann_b200_exchange* x) { return 2u * (size_t)x->members * x->slot_words * 8u; }

SV_EXPORT int silvann_b200_exchange_create(silvann_b200_exchange** out, uint32_t members, uint32_t index, uint64_t slot_bytes) {
    if (!out) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_create: out is null");
    if (members < 1 || members > XF_MEMBERS_MAX || index >= members) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_create: member %u of %u (1..%d members)", index, members, XF_MEMBERS_MAX);
    if (slot_bytes == 0 || slot_bytes > (1ull << 30)) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_create: a slot of %llu bytes", (unsigned long long)slot_bytes);
    silvann_b200_exchange* x = new (std::nothrow) silvann_b200_exchange();
    if (!x) return sv_ext_fail(SILVANN_B200_E_CUDA, "exchange_create: out of host memory");
    memset(x, 0, sizeof *x);
    x->members = members; x->index = index; x->slot_bytes = (slot_bytes + 15u) & ~(uint64_t)15u;
    x->slot_words = x->slot_bytes / 2u;
    cudaError_t e = cudaGetDevice(&x->device);
    void* p = nullptr;
    if (e == cudaSuccess) e = cudaMalloc(&p, xf_bytes(x));
    if (e == cudaSuccess) e = cudaMemset(p, 0, xf_bytes(x));
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        if (p) cudaFree(p);
        delete x; (void)cudaGetLastError();
        return sv_ext_fail(SILVANN_B200_E_CUDA, "exchange_create: %s", cudaGetErrorString(e));
    }
    x->peer[index] = (uint8_t*)p;
    x->connected = members == 1;
    *out = x;
    return SILVANN_B200_OK;
}

SV_EXPORT int silvann_b200_exchange_destroy(silvann_b200_exchange* x) {
    if (!x) return SILVANN_B200_OK;
    (void)cudaDeviceSynchronize();
    for (uint32_t m = 0; m < x->members; ++m)
        if (m != x->index && x->opened[m] && x->peer[m]) cudaIpcCloseMemHandle(x->peer[m]);
    if (x->peer[x->index]) cudaFree(x->peer[x->index]);
    delete x;
    return SILVANN_B200_OK;
}

SV_EXPORT int silvann_b200_exchange_local(const silvann_b200_exchange* x, uint64_t* address, uint64_t* bytes) {
    if (!x) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_local: exchange is null");
    if (address) *address = (uint64_t)(uintptr_t)x->peer[x->index];
    if (bytes) *bytes = xf_bytes(x);
    return SILVANN_B200_OK;
}

SV_EXPORT int silvann_b200_exchange_handle(const silvann_b200_exchange* x, void* handle, uint32_t handle_bytes) {
    if (!x || !handle) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_handle: a null operand");
    if (handle_bytes < sizeof(cudaIpcMemHandle_t)) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_handle: a handle is %u bytes", (unsigned)sizeof(cudaIpcMemHandle_t));
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, x->peer[x->index]);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return sv_ext_fail(SILVANN_B200_E_CUDA, "exchange_handle: %s", cudaGetErrorString(e)); }
    memcpy(handle, &h, sizeof h);
    return SILVANN_B200_OK;
}

SV_EXPORT int silvann_b200_exchange_connect_handles(silvann_b200_exchange* x, const void* handles, uint32_t handle_bytes) {
    if (!x || !handles) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_connect_handles: a null operand");
    if (handle_bytes < sizeof(cudaIpcMemHandle_t)) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_connect_handles: a handle is %u bytes", (unsigned)sizeof(cudaIpcMemHandle_t));
    if (x->connected) return sv_ext_fail(SILVANN_B200_E_STATE, "exchange_connect_handles: already connected");
    for (uint32_t m = 0; m < x->members; ++m) {
        if (m == x->index) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char*)handles + (size_t)m * handle_bytes, sizeof h);
        void* p = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) { (void)cudaGetLastError(); return sv_ext_fail(SILVANN_B200_E_CUDA, "exchange_connect_handles: member %u: %s", m, cudaGetErrorString(e)); }
        x->peer[m] = (uint8_t*)p; x->opened[m] = true;
    }
    x->connected = true;
    return SILVANN_B200_OK;
}

SV_EXPORT int silvann_b200_exchange_connect_addresses(silvann_b200_exchange* x, const uint64_t* addresses) {
    if (!x || !addresses) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_connect_addresses: a null operand");
    if (x->connected) return sv_ext_fail(SILVANN_B200_E_STATE, "exchange_connect_addresses: already connected");
    for (uint32_t m = 0; m < x->members; ++m) {
        if (m == x->index) continue;
        if (!addresses[m]) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_connect_addresses: member %u has no address", m);
        x->peer[m] = (uint8_t*)(uintptr_t)addresses[m];
    }
    x->connected = true;
    return SILVANN_B200_OK;
}

static int xf_params(silvann_b200_exchange* x, const char* who, uint32_t wait_ms, sv::XfParams* P) {
    if (!x->connected) return sv_ext_fail(SILVANN_B200_E_STATE, "%s: the exchange is not connected to its members", who);
    int d = -1;
    if (cudaGetDevice(&d) != cudaSuccess || d != x->device) return sv_ext_fail(SILVANN_B200_E_STATE, "%s: the exchange lives on device %d and device %d is bound", who, x->device, d);
    memset(P, 0, sizeof *P);
    for (uint32_t m = 0; m < x->members; ++m) P->peer[m] = x->peer[m];
    P->members = x->members; P->index = x->index; P->gen = x->gen + 1u; P->slot_words = x->slot_words;
    P->wait_ns = (unsigned long long)(wait_ms ? wait_ms : 1000u) * 1000000ull;
    P->status = sv::device_status_word();
    return SILVANN_B200_OK;
}

SV_EXPORT int silvann_b200_exchange_merge_finish(silvann_b200_exchange* x, void* o, float* res, const float* res_local, uint64_t q_heads, uint64_t head_dim,
                                                 int dtype, sv_fault* over, uint32_t wait_ms, void* stream) {
    if (!x || !res_local || (!o && !res)) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_merge_finish: a null operand");
    if (dtype != SV_DTYPE_FP16 && dtype != SV_DTYPE_BF16) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_merge_finish: dtype %d", dtype);
    if (q_heads == 0 || head_dim == 0 || head_dim % 2u || ((uintptr_t)res_local & 7u)) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_merge_finish: %llu heads of %llu (even), residual on 8 bytes", (unsigned long long)q_heads, (unsigned long long)head_dim);
    if (head_dim > XF_FOLD_ELEMENTS) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_merge_finish: heads of %llu (at most %u)", (unsigned long long)head_dim, XF_FOLD_ELEMENTS);
    const uint64_t hb = XF_FOLD_ELEMENTS / head_dim < XF_HEADS_PER_BLOCK ? XF_FOLD_ELEMENTS / head_dim : XF_HEADS_PER_BLOCK;
    const uint64_t bytes = q_heads * (head_dim + 2u) * sizeof(float), blocks = (q_heads + hb - 1) / hb;
    if (bytes > x->slot_bytes) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_merge_finish: a residual of %llu bytes and a slot holds %llu", (unsigned long long)bytes, (unsigned long long)x->slot_bytes);
    sv::XfParams P;
    int rc = xf_params(x, "exchange_merge_finish", wait_ms, &P);
    if (rc != SILVANN_B200_OK) return rc;
    if (dtype == SV_DTYPE_BF16) sv::exchange_merge_kernel<SV_DTYPE_BF16><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(P, (uint16_t*)o, res, res_local, (uint32_t)q_heads, (uint32_t)head_dim, (uint32_t)hb, over);
    else sv::exchange_merge_kernel<SV_DTYPE_FP16><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(P, (uint16_t*)o, res, res_local, (uint32_t)q_heads, (uint32_t)head_dim, (uint32_t)hb, over);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return sv_ext_fail(SILVANN_B200_E_CUDA, "exchange_merge_finish: %s", cudaGetErrorString(e));
    sv::note_launch(1);
    x->gen += 1u;
    return SILVANN_B200_OK;
}

SV_EXPORT int silvann_b200_exchange_vector_sum(silvann_b200_exchange* x, void* out, const void* partial, uint64_t n, int dtype, sv_fault* over,
                                               uint32_t wait_ms, void* stream) {
    if (!x || !out || !partial || n == 0) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_vector_sum: a null or empty operand");
    if (dtype != SV_DTYPE_FP16 && dtype != SV_DTYPE_BF16) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_vector_sum: dtype %d", dtype);
    if (((uintptr_t)out | (uintptr_t)partial) & 1u) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_vector_sum: operands on 2 bytes");
    if (((n * 2u + 15u) & ~(uint64_t)15u) > x->slot_bytes) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_vector_sum: %llu elements and a slot holds %llu bytes", (unsigned long long)n, (unsigned long long)x->slot_bytes);
    sv::XfParams P;
    int rc = xf_params(x, "exchange_vector_sum", wait_ms, &P);
    if (rc != SILVANN_B200_OK) return rc;
    const unsigned blocks = (unsigned)((n + 2047u) / 2048u > XF_SUM_BLOCKS ? XF_SUM_BLOCKS : (n + 2047u) / 2048u);
    if (dtype == SV_DTYPE_BF16) sv::exchange_sum_kernel<SV_DTYPE_BF16><<<blocks, 256, 0, (cudaStream_t)stream>>>(P, (uint16_t*)out, (const uint16_t*)partial, n, over);
    else sv::exchange_sum_kernel<SV_DTYPE_FP16><<<blocks, 256, 0, (cudaStream_t)stream>>>(P, (uint16_t*)out, (const uint16_t*)partial, n, over);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return sv_ext_fail(SILVANN_B200_E_CUDA, "exchange_vector_sum: %s", cudaGetErrorString(e));
    sv::note_launch(1);
    x->gen += 1u;
    return SILVANN_B200_OK;
}

/* A coded matrix times a vector on every member, the members' answers added in member order, in ONE launch a member: the
 * output projection of a head-sharded mixer (turboquant_gemv over the card's share of the columns) and the sum the reference
 * makes afterwards with nn__partials__reduce_onto (ai_qwen_3 mixer__abi.cuh:254-257, nn partials__abi.cuh:110-163).  The
 * kernel's epilogue rounds a row's answer to 16 bits — the partial the reference would have written — and pushes it to the
 * members; each block then adds its own rows over the members in fp32 and rounds once, which is vector_sum's arithmetic. */
SV_EXPORT int silvann_b200_exchange_gemv_sum(silvann_b200_exchange* x, void* out, const void* codes, const void* scales, const void* vec, uint64_t width,
                                             uint64_t rows, uint64_t cols, sv_fault* over, uint32_t wait_ms, void* stream) {
    if (!x || !out || !codes || !scales || !vec || rows == 0) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_gemv_sum: a null or empty operand");
    struct { uint64_t codes[12], luts[12], rows[12], d[12], out_at[12], count; } g;
    memset(&g, 0, sizeof g);
    g.codes[0] = (uint64_t)(uintptr_t)codes; g.luts[0] = (uint64_t)(uintptr_t)scales; g.rows[0] = rows; g.d[0] = width; g.count = 1;
    if (!sv::tq_gemv_fast_fits(&g, cols, 1) || rows * 2u > x->slot_bytes)
        return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_gemv_sum: %llu rows of %llu codes at %llu bits are outside the kernel's fit, or more than a slot of %llu bytes holds",
                           (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)width, (unsigned long long)x->slot_bytes);
    sv::XfParams P;
    int rc = xf_params(x, "exchange_gemv_sum", wait_ms, &P);
    if (rc != SILVANN_B200_OK) return rc;
    const cudaError_t e = sv::tq_gemv_fast_launch((uint16_t*)out, &g, nullptr, (const uint16_t*)vec, cols, 1, 0, over, (cudaStream_t)stream, &P);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return sv_ext_fail(SILVANN_B200_E_CUDA, "exchange_gemv_sum: %s", cudaGetErrorString(e)); }
    x->gen += 1u;
    return SILVANN_B200_OK;
}

SV_EXPORT int silvann_b200_exchange_deposit(silvann_b200_exchange* x, uint32_t member, const void* data, uint64_t bytes, uint32_t unit_bytes, void* stream) {
    if (!x || !data || bytes == 0) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_deposit: a null or empty operand");
    if (member >= x->members || member == x->index) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_deposit: member %u (this is member %u of %u)", member, x->index, x->members);
    if ((unit_bytes != 2u && unit_bytes != 4u) || bytes % 2u || ((uintptr_t)data & 1u)) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_deposit: words of %u bytes (2 or 4), an even count of bytes on 2 bytes", unit_bytes);
    if (bytes > x->slot_bytes) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_deposit: %llu bytes and a slot holds %llu", (unsigned long long)bytes, (unsigned long long)x->slot_bytes);
    const unsigned blocks = (unsigned)((bytes + 4095u) / 4096u > 64u ? 64u : (bytes + 4095u) / 4096u);
    sv::exchange_deposit_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(x->peer[x->index], x->members, member, x->slot_words, x->gen + 1u, (const uint16_t*)data, bytes / 2u, unit_bytes);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return sv_ext_fail(SILVANN_B200_E_CUDA, "exchange_deposit: %s", cudaGetErrorString(e));
    sv::note_launch(1);
    return SILVANN_B200_OK;
}

/* for tier.cu: a launch of another kernel that does the exchange step itself (the decode kernel's last block) — the members'
 * buffers, this exchange's generation and the wait's limit; `advance` counts the exchange once that launch is queued */
int sv_exchange_begin(silvann_b200_exchange* x, uint32_t wait_ms, uint64_t bytes, sv::XfParams* P) {
    if (!x || !P) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange: a null operand");
    if (bytes > x->slot_bytes) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange: a residual of %llu bytes and a slot holds %llu", (unsigned long long)bytes, (unsigned long long)x->slot_bytes);
    return xf_params(x, "tier_decode_exchange", wait_ms, P);
}
void sv_exchange_advance(silvann_b200_exchange* x) { x->gen += 1u; }

/* for tier.cu: the same launch from inside the library */
int sv_exchange_merge_finish(silvann_b200_exchange* x, void* o, float* res, const float* res_local, uint64_t q_heads, uint64_t head_dim, int dtype,
                             sv_fault* over, uint32_t wait_ms, void* stream) {
    return silvann_b200_exchange_merge_finish(x, o, res, res_local, q_heads, head_dim, dtype, over, wait_ms, stream);
}
