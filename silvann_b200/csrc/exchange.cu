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
 * stores its piece into a slot of every member's buffer with plain peer stores, publishes a generation number in a flag
 * beside it (release at system scope), waits — bounded — until every member's flag shows the same generation, and then
 * reads only its own memory.  One launch a card and no host in the loop; the answer is computed redundantly on every
 * member in the same order, so all members hold the same bits.
 *
 * Buffers.  Every member owns one device buffer: flags [2 parities][members][XF_BLOCKS] then slots
 * [2 parities][members][slot_bytes].  Two parities are enough: a member can run at most one exchange ahead of the slowest
 * (it needs that member's flag of exchange t to finish t), so while anyone still reads parity t nobody writes it.
 * Members call the exchange entry points in the same order the same number of times (a collective's contract); the
 * generation counter is the number of exchanges so far and lives on the host.
 *
 * No multicast, no TMA, no library kernel touches peer memory: ordinary st.global / ld.global only.  Every wait is bounded
 * by the wall clock (%globaltimer); when it runs out the block raises "B2TO" in the device status word and returns
 * without writing its outputs. */
#include "../../include/silvann_b200.h"
#include "common.cuh"
#include "kernels.h"
#include "residual.cuh"
#include "exchange.cuh"
#include <new>
#include <string.h>

#define SV_EXPORT extern "C" __attribute__((visibility("default")))
#define XF_HEADS_PER_BLOCK 8u
#define XF_SUM_PIECE 4096u                  /* bytes of a partial a block of the sum kernel moves: 16 bytes a thread */

int sv_ext_fail(int code, const char* fmt, ...);      /* ext.cu */

struct silvann_b200_exchange {
    int device;
    uint32_t members, index;
    uint64_t slot_bytes;                    /* a multiple of 16 */
    uint8_t* peer[XF_MEMBERS_MAX];          /* every member's buffer as this process addresses it; peer[index] is the local one */
    bool opened[XF_MEMBERS_MAX];            /* mapped here from an inter-process handle (to be closed), not given as an address */
    bool connected;
    uint32_t gen;                           /* exchanges so far */
};

namespace sv {

/* After the block's pushes: publish this block's flag on every member, then wait until every member's flag for this block
 * shows the generation.  Answers false (to every thread of the block) when a wait ran out. */
__device__ __forceinline__ bool xf_signal_and_wait(const XfParams& P, uint32_t parity, uint32_t block, uint32_t* fail_s) {
    __threadfence_system();                   /* this thread's pushes are ordered before the flag below */
    if (threadIdx.x == 0) *fail_s = 0u;
    __syncthreads();
    if (threadIdx.x < P.members) {
        st_release_sys(xf_flag(P.peer[threadIdx.x], parity, P.index, block), P.gen);
        const unsigned int* mine = xf_flag(P.peer[P.index], parity, threadIdx.x, block);
        if (ld_acquire_sys(mine) != P.gen) {
            const unsigned long long t0 = wall_ns();
            bool ok = false;
            while (!ok) {
                for (int i = 0; i < 64 && !ok; ++i) ok = ld_acquire_sys(mine) == P.gen;
                if (!ok && wall_ns() - t0 > P.wait_ns) break;
            }
            if (!ok) { *fail_s = 1u; if (P.status) atomicOr(P.status, SV_STATUS_TIMEOUT); }
        }
    }
    __syncthreads();
    return *fail_s == 0u;
}

/* Residuals of the members' ranges -> the whole range's residual and/or its 16-bit output.  A block owns 8 heads. */
template <int DT>
__global__ void __launch_bounds__(256) exchange_merge_kernel(const XfParams P, uint16_t* o, float* res_out, const float* res_local,
                                                             uint32_t q_heads, uint32_t d, unsigned int* over) {
    using E = Elem<DT>;
    __shared__ uint32_t fail_s;
    __shared__ float fa_s[XF_HEADS_PER_BLOCK][XF_MEMBERS_MAX], fb_s[XF_HEADS_PER_BLOCK][XF_MEMBERS_MAX], l_s[XF_HEADS_PER_BLOCK], m_s[XF_HEADS_PER_BLOCK];
    const uint32_t parity = P.gen & 1u, w = d + 2u;
    const uint32_t h0 = blockIdx.x * XF_HEADS_PER_BLOCK, heads = min(XF_HEADS_PER_BLOCK, q_heads - h0);
    const uint32_t n2 = heads * w / 2u;                                      /* float2s of this block's heads (w is even) */
    const size_t off2 = (size_t)h0 * w / 2u;

    /* push: this card's residual of these heads into its slot on every member (its own included) */
    for (uint32_t i = threadIdx.x; i < n2; i += blockDim.x) {
        const float2 x = reinterpret_cast<const float2*>(res_local)[off2 + i];
        for (uint32_t m = 0; m < P.members; ++m)
            reinterpret_cast<float2*>(xf_slot(P.peer[m], parity, P.index, P.slot_bytes, P.members))[off2 + i] = x;
    }
    if (!xf_signal_and_wait(P, parity, blockIdx.x, &fail_s)) return;

    /* every member's residual of these heads is in this card's memory now; fold them in member order */
    uint8_t* local = P.peer[P.index];
    if (threadIdx.x < heads) {
        const uint32_t h = threadIdx.x;
        const float* r0 = reinterpret_cast<const float*>(xf_slot(local, parity, 0, P.slot_bytes, P.members)) + (size_t)(h0 + h) * w;
        float m = __ldcg(r0), l = __ldcg(r0 + 1);
        for (uint32_t s = 1; s < P.members; ++s) {
            const float* rs = reinterpret_cast<const float*>(xf_slot(local, parity, s, P.slot_bytes, P.members)) + (size_t)(h0 + h) * w;
            float fa, fb;
            merge_scalars(m, l, __ldcg(rs), __ldcg(rs + 1), fa, fb);
            fa_s[h][s] = fa; fb_s[h][s] = fb;
        }
        m_s[h] = m; l_s[h] = l;
    }
    __syncthreads();
    bool hit = false;
    for (uint32_t i = threadIdx.x; i < heads * d; i += blockDim.x) {
        const uint32_t h = i / d, e = i - h * d;
        const size_t at = (size_t)(h0 + h) * w + 2u + e;
        float acc = __ldcg(reinterpret_cast<const float*>(xf_slot(local, parity, 0, P.slot_bytes, P.members)) + at);
        for (uint32_t s = 1; s < P.members; ++s)
            acc = merge_element(acc, fa_s[h][s], __ldcg(reinterpret_cast<const float*>(xf_slot(local, parity, s, P.slot_bytes, P.members)) + at), fb_s[h][s]);
        if (res_out) { res_out[at] = acc; if (e == 0) { res_out[at - 2] = m_s[h]; res_out[at - 1] = l_s[h]; } }
        if (o) o[(size_t)(h0 + h) * d + e] = E::from_float(acc / l_s[h], hit);
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* 16-bit partials of the members -> their fp32 sum in member order, rounded once.  A block owns XF_SUM_PIECE bytes times
 * `pieces` (a launch has at most XF_BLOCKS blocks). */
template <int DT>
__global__ void __launch_bounds__(256) exchange_sum_kernel(const XfParams P, uint16_t* out, const uint16_t* partial, uint64_t n, uint32_t per_block,
                                                           unsigned int* over) {
    using E = Elem<DT>;
    __shared__ uint32_t fail_s;
    const uint32_t parity = P.gen & 1u;
    const uint64_t lo = (uint64_t)blockIdx.x * per_block, hi = min(n, lo + per_block);      /* elements; per_block is a multiple of 8 */
    const bool wide = ((uintptr_t)partial & 15u) == 0;
    for (uint64_t i = lo + (uint64_t)threadIdx.x * 8u; i < hi; i += (uint64_t)blockDim.x * 8u) {
        uint16_t x[8];
        if (wide && i + 8 <= hi) *reinterpret_cast<uint4*>(x) = *reinterpret_cast<const uint4*>(partial + i);
        else for (int u = 0; u < 8; ++u) x[u] = i + u < hi ? partial[i + u] : (uint16_t)0;
        for (uint32_t m = 0; m < P.members; ++m)                                                /* a slot starts on 16 bytes and i is a multiple of 8 */
            *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(xf_slot(P.peer[m], parity, P.index, P.slot_bytes, P.members)) + i) = *reinterpret_cast<const uint4*>(x);
    }
    if (!xf_signal_and_wait(P, parity, blockIdx.x, &fail_s)) return;
    uint8_t* local = P.peer[P.index];
    bool hit = false;
    const bool wide_out = ((uintptr_t)out & 15u) == 0;
    for (uint64_t i = lo + (uint64_t)threadIdx.x * 8u; i < hi; i += (uint64_t)blockDim.x * 8u) {
        float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (uint32_t m = 0; m < P.members; ++m) {
            const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(xf_slot(local, parity, m, P.slot_bytes, P.members)) + i));
            const uint16_t* x = reinterpret_cast<const uint16_t*>(&raw);
#pragma unroll
            for (int u = 0; u < 8; ++u) s[u] += E::to_float(x[u]);
        }
        uint16_t y[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) y[u] = E::from_float(s[u], hit);
        if (wide_out && i + 8 <= hi) *reinterpret_cast<uint4*>(out + i) = *reinterpret_cast<const uint4*>(y);
        else for (int u = 0; u < 8 && i + u < hi; ++u) out[i + u] = y[u];
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* Stands in for a member on a machine with fewer cards than members: its piece and its flags for the NEXT exchange. */
__global__ void __launch_bounds__(256) exchange_deposit_kernel(uint8_t* local, uint32_t members, uint32_t member, uint64_t slot_bytes, uint32_t gen,
                                                               const uint8_t* data, uint64_t bytes) {
    const uint32_t parity = gen & 1u;
    uint8_t* slot = xf_slot(local, parity, member, slot_bytes, members);
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < bytes; i += (uint64_t)gridDim.x * blockDim.x) slot[i] = data[i];
    __threadfence();
    __syncthreads();
    if (blockIdx.x == 0) for (uint32_t b = threadIdx.x; b < XF_BLOCKS; b += blockDim.x) *xf_flag(local, parity, member, b) = gen;
}

}  // namespace sv

/* ---------------------------------------------------------------------------------------------------------------------- */

static size_t xf_bytes(const silvann_b200_exchange* x) { return (size_t)XF_FLAG_BYTES + 2u * (size_t)x->members * x->slot_bytes; }

SV_EXPORT int silvann_b200_exchange_create(silvann_b200_exchange** out, uint32_t members, uint32_t index, uint64_t slot_bytes) {
    if (!out) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_create: out is null");
    if (members < 1 || members > XF_MEMBERS_MAX || index >= members) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_create: member %u of %u (1..%d members)", index, members, XF_MEMBERS_MAX);
    if (slot_bytes == 0 || slot_bytes > (1ull << 30)) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_create: a slot of %llu bytes", (unsigned long long)slot_bytes);
    silvann_b200_exchange* x = new (std::nothrow) silvann_b200_exchange();
    if (!x) return sv_ext_fail(SILVANN_B200_E_CUDA, "exchange_create: out of host memory");
    memset(x, 0, sizeof *x);
    x->members = members; x->index = index; x->slot_bytes = (slot_bytes + 15u) & ~(uint64_t)15u;
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
    P->members = x->members; P->index = x->index; P->gen = x->gen + 1u; P->slot_bytes = x->slot_bytes;
    P->wait_ns = (unsigned long long)(wait_ms ? wait_ms : 1000u) * 1000000ull;
    P->status = sv::device_status_word();
    return SILVANN_B200_OK;
}

SV_EXPORT int silvann_b200_exchange_merge_finish(silvann_b200_exchange* x, void* o, float* res, const float* res_local, uint64_t q_heads, uint64_t head_dim,
                                                 int dtype, sv_fault* over, uint32_t wait_ms, void* stream) {
    if (!x || !res_local || (!o && !res)) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_merge_finish: a null operand");
    if (dtype != SV_DTYPE_FP16 && dtype != SV_DTYPE_BF16) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_merge_finish: dtype %d", dtype);
    if (q_heads == 0 || head_dim == 0 || head_dim % 2u || ((uintptr_t)res_local & 7u)) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_merge_finish: %llu heads of %llu (even), residual on 8 bytes", (unsigned long long)q_heads, (unsigned long long)head_dim);
    const uint64_t bytes = q_heads * (head_dim + 2u) * sizeof(float), blocks = (q_heads + XF_HEADS_PER_BLOCK - 1) / XF_HEADS_PER_BLOCK;
    if (bytes > x->slot_bytes || blocks > XF_BLOCKS) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_merge_finish: a residual of %llu bytes and a slot holds %llu", (unsigned long long)bytes, (unsigned long long)x->slot_bytes);
    sv::XfParams P;
    int rc = xf_params(x, "exchange_merge_finish", wait_ms, &P);
    if (rc != SILVANN_B200_OK) return rc;
    if (dtype == SV_DTYPE_BF16) sv::exchange_merge_kernel<SV_DTYPE_BF16><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(P, (uint16_t*)o, res, res_local, (uint32_t)q_heads, (uint32_t)head_dim, over);
    else sv::exchange_merge_kernel<SV_DTYPE_FP16><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(P, (uint16_t*)o, res, res_local, (uint32_t)q_heads, (uint32_t)head_dim, over);
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
    uint64_t per_block = XF_SUM_PIECE / 2u;
    while ((n + per_block - 1) / per_block > XF_BLOCKS) per_block *= 2u;
    sv::XfParams P;
    int rc = xf_params(x, "exchange_vector_sum", wait_ms, &P);
    if (rc != SILVANN_B200_OK) return rc;
    const unsigned blocks = (unsigned)((n + per_block - 1) / per_block);
    if (dtype == SV_DTYPE_BF16) sv::exchange_sum_kernel<SV_DTYPE_BF16><<<blocks, 256, 0, (cudaStream_t)stream>>>(P, (uint16_t*)out, (const uint16_t*)partial, n, (uint32_t)per_block, over);
    else sv::exchange_sum_kernel<SV_DTYPE_FP16><<<blocks, 256, 0, (cudaStream_t)stream>>>(P, (uint16_t*)out, (const uint16_t*)partial, n, (uint32_t)per_block, over);
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

SV_EXPORT int silvann_b200_exchange_deposit(silvann_b200_exchange* x, uint32_t member, const void* data, uint64_t bytes, void* stream) {
    if (!x || !data || bytes == 0) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_deposit: a null or empty operand");
    if (member >= x->members || member == x->index) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_deposit: member %u (this is member %u of %u)", member, x->index, x->members);
    if (bytes > x->slot_bytes) return sv_ext_fail(SILVANN_B200_E_ARGUMENT, "exchange_deposit: %llu bytes and a slot holds %llu", (unsigned long long)bytes, (unsigned long long)x->slot_bytes);
    const unsigned blocks = (unsigned)((bytes + 4095u) / 4096u > 64u ? 64u : (bytes + 4095u) / 4096u);
    sv::exchange_deposit_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(x->peer[x->index], x->members, member, x->slot_bytes, x->gen + 1u, (const uint8_t*)data, bytes);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return sv_ext_fail(SILVANN_B200_E_CUDA, "exchange_deposit: %s", cudaGetErrorString(e));
    sv::note_launch(1);
    return SILVANN_B200_OK;
}

/* for tier.cu: the same launch from inside the library */
int sv_exchange_merge_finish(silvann_b200_exchange* x, void* o, float* res, const float* res_local, uint64_t q_heads, uint64_t head_dim, int dtype,
                             sv_fault* over, uint32_t wait_ms, void* stream) {
    return silvann_b200_exchange_merge_finish(x, o, res, res_local, q_heads, head_dim, dtype, over, wait_ms, stream);
}
