/* common.cuh — device helpers shared by every kernel of the B200 attention family.
 *
 * Half/bf16 bit conversions with the engine's overflow rule, mbarrier + TMA wrappers whose waits are all bounded,
 * legacy-MMA fragment helpers for the HBM-bound decode kernels, and the device status word.
 *
 * A bounded wait that runs out never traps: it ORs SV_STATUS_TIMEOUT into the device status word, raises a
 * block-local error flag so that every other warp of the block leaves its loops, and the kernel returns normally. */
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define SV_DTYPE_FP16 0
#define SV_DTYPE_BF16 1

#define SV_FAULT_OVERFLOW 0x4E504F56u   /* "NPOV" — engine/src/packages/nn/contracts/objects/primitives.cuh:57 */
#define SV_STATUS_TIMEOUT 0x4232544Fu   /* "B2TO" — a bounded device-side wait gave up */
#define SV_STATUS_BAD_PAGE 0x80000000u  /* a page-table entry inside a sequence's length named no page of the pool (a bit the code above leaves clear) */

/* How long a device-side wait may spin before giving up: tries of mbarrier.try_wait (each suspends for a
 * hardware-chosen slice) — in the order of a second at worst, far beyond any healthy TMA or MMA latency. */
#define SV_WAIT_TRIES (1u << 22)

namespace sv {

/* ------------------------------------------------------------------------------------------------------------ */
/* 16-bit element types as raw bits                                                                              */

template <int DT> struct Elem;
template <> struct Elem<SV_DTYPE_FP16> {
    static __device__ __forceinline__ float to_float(uint16_t b) { return __half2float(__ushort_as_half(b)); }
    /* fp32 -> fp16 round-to-nearest-even; a finite input that lands on infinity is an overflow (the engine's
     * rule, engine/src/packages/nn/gpu/kernels/kernels.cuh:2766-2808); inf/NaN inputs pass through unflagged. */
    static __device__ __forceinline__ uint16_t from_float(float f, bool& over) {
        const uint16_t h = __half_as_ushort(__float2half_rn(f));
        if ((h & 0x7FFFu) == 0x7C00u && !isinf(f)) over = true;
        return h;
    }
    /* the smallest magnitude that rounds to infinity (half an ulp above the largest finite value, a tie that goes up) */
    static __device__ __forceinline__ float over_from() { return 65520.0f; }
    static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
        const __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
    static __device__ __forceinline__ float2 unpack2(uint32_t u) {
        return __half22float2(*reinterpret_cast<const __half2*>(&u));
    }
};
template <> struct Elem<SV_DTYPE_BF16> {
    static __device__ __forceinline__ float to_float(uint16_t b) { return __uint_as_float(((uint32_t)b) << 16); }
    static __device__ __forceinline__ uint16_t from_float(float f, bool& over) {
        const uint16_t h = __bfloat16_as_ushort(__float2bfloat16_rn(f));
        if ((h & 0x7FFFu) == 0x7F80u && !isinf(f)) over = true;
        return h;
    }
    static __device__ __forceinline__ float over_from() { return __uint_as_float(0x7F7F8000u); }
    static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
    static __device__ __forceinline__ float2 unpack2(uint32_t u) {
        return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xFFFF0000u));
    }
};

/* ------------------------------------------------------------------------------------------------------------ */
/* shared-memory addresses, mbarriers, TMA                                                                        */

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0u;
}
/* Waits for the phase with the given parity to complete, at most SV_WAIT_TRIES tries.  `abort_flag` is a
 * block-shared word any warp raises when it gave up; a raised flag ends this wait too.  Answers false when the wait
 * did not complete (the caller then leaves its loop and falls through to the kernel's common exit). */
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          unsigned int* status) {
    if (mbar_try_wait(bar, parity)) return true;          /* the common case costs one try (about 100 cycles) and no loop */
    for (uint32_t i = 0; i < SV_WAIT_TRIES; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag != 0u) return false;
    }
    *abort_flag = 1u;
    if (status) atomicOr(status, SV_STATUS_TIMEOUT);
    return false;
}

/* One 2-D tile, shared -> global, as part of this thread's current bulk group; rows and columns past the tensor's extent
 * are not written.  x (the innermost coordinate) times the element size must be a multiple of 16 bytes, and neither
 * coordinate may be negative.  The writes to shared memory that the tile is made of must have been followed by
 * tma_store_fence() in the threads that made them, before the synchronisation that lets this thread go. */
__device__ __forceinline__ void tma_store_2d(const void* tmap, const void* src, int32_t x, int32_t y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(tmap), "r"(smem_u32(src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_store_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
/* closes the bulk group and waits until its tiles have been READ from shared memory (the memory may then be given back;
 * the writes to global memory complete on their own) */
__device__ __forceinline__ void tma_store_commit_and_wait_read() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

/* One 2-D tile, global -> shared, completion counted in bytes on `bar`.  x is the innermost (element) coordinate and
 * must be a multiple of 16 bytes' worth of elements; y is the row.  No multicast: the tile lands in this CTA only. */
__device__ __forceinline__ void tma_load_2d(void* dst, const void* tmap, uint64_t* bar, int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
/* The same with an L2 eviction-priority hint (a 64-bit policy made by `l2_policy_evict_first/last`). */
__device__ __forceinline__ void tma_load_2d_hint(void* dst, const void* tmap, uint64_t* bar, int32_t x, int32_t y,
                                                 uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(smem_u32(dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y), "l"(policy) : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
/* Makes generic-proxy writes to shared memory visible to the async proxy (TMA stores, tcgen05 operand reads). */
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

/* ------------------------------------------------------------------------------------------------------------ */
/* The 128-byte swizzle TMA applies to a tile whose rows are 128 bytes: the 16-byte chunk index is XORed with the */
/* row index modulo 8.  `row` counts 128-byte rows from a 1024-byte-aligned tile base.                              */
__device__ __forceinline__ uint32_t swz128(uint32_t row, uint32_t chunk) {
    return row * 128u + ((chunk ^ (row & 7u)) << 4);
}

/* ------------------------------------------------------------------------------------------------------------ */
/* warp-level matrix pieces for the decode kernels (fp32 accumulate)                                              */

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ uint32_t movm_t(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
template <int DT>
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    if (DT == SV_DTYPE_FP16) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

/* ------------------------------------------------------------------------------------------------------------ */
/* thread-block clusters: rank and size, the hardware barrier over all blocks of a cluster, a float read from a    */
/* peer block's shared memory (the address is this block's own address of the same variable)                       */
__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t cluster_nctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(const float* local, uint32_t rank) {
    uint32_t remote; float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

#define SV_LOG2E 1.4426950408889634f
#define SV_LN2   0.6931471805599453f

}  // namespace sv
