/* exchange.cuh — what a kernel needs to take part in an exchange over peer memory (see exchange.cu): the members' buffers,
 * where a member's flag and slot lie in one, and the two memory operations of the protocol.  Included by the exchange
 * kernels and by producers that push their results straight from their epilogue. */
#pragma once
#include "common.cuh"

#define XF_MEMBERS_MAX 8
#define XF_BLOCKS 256u                      /* flags a member and parity: one a thread block of an exchange kernel */
#define XF_FLAG_BYTES (2u * XF_MEMBERS_MAX * XF_BLOCKS * 4u)

namespace sv {

struct XfParams {
    uint8_t* peer[XF_MEMBERS_MAX];
    uint32_t members, index, gen;
    uint64_t slot_bytes;
    unsigned long long wait_ns;
    unsigned int* status;
};

__device__ __forceinline__ unsigned int* xf_flag(uint8_t* base, uint32_t parity, uint32_t member, uint32_t block) {
    return reinterpret_cast<unsigned int*>(base) + ((size_t)parity * XF_MEMBERS_MAX + member) * XF_BLOCKS + block;
}
__device__ __forceinline__ uint8_t* xf_slot(uint8_t* base, uint32_t parity, uint32_t member, uint64_t slot_bytes, uint32_t members) {
    return base + XF_FLAG_BYTES + ((size_t)parity * members + member) * slot_bytes;
}
__device__ __forceinline__ void st_release_sys(unsigned int* at, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(at), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* at) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(at) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long wall_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

}  // namespace sv
