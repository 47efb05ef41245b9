/* exchange.cuh — what a kernel needs to take part in an exchange over peer memory (see exchange.cu): the members' buffers,
 * where a member's slot lies in one, and the two memory operations of the protocol.  Included by the exchange kernels and
 * by producers that push their results straight from their epilogue.
 *
 * A piece travels as TAGGED WORDS: 8 bytes = 4 bytes of payload and the generation number of the exchange, written with one
 * 8-byte store and read with one 8-byte load, both single memory transactions.  A reader that sees the generation it waits
 * for in a word therefore sees that word's payload too: no fence between data and flag, no separate flag, and a reader
 * starts on the first words while the last are still on the wire.  (A system-scope fence between the data stores and a
 * flag store costs several microseconds on this part, more than the whole transfer.) */
#pragma once
#include "common.cuh"

#define XF_MEMBERS_MAX 8

namespace sv {

struct XfParams {
    uint8_t* peer[XF_MEMBERS_MAX];
    uint32_t members, index, gen;
    uint64_t slot_words;                    /* tagged words a member's slot holds */
    unsigned long long wait_ns;
    unsigned int* status;
};

/* member `member`'s slot of one parity inside a buffer: [2 parities][members][slot_words] tagged words */
__device__ __forceinline__ uint2* xf_slot(uint8_t* base, uint32_t parity, uint32_t member, uint64_t slot_words, uint32_t members) {
    return reinterpret_cast<uint2*>(base) + ((size_t)parity * members + member) * slot_words;
}
__device__ __forceinline__ void xf_store(uint2* at, uint32_t payload, uint32_t gen) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(at), "r"(payload), "r"(gen) : "memory");
}
__device__ __forceinline__ void xf_store2(uint2* at, uint32_t p0, uint32_t p1, uint32_t gen) {         /* two words; `at` on 16 bytes */
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %2};" ::"l"(at), "r"(p0), "r"(gen), "r"(p1) : "memory");
}
__device__ __forceinline__ uint2 xf_load(const uint2* at) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(at) : "memory");
    return v;
}
__device__ __forceinline__ uint4 xf_load2(const uint2* at) {                                            /* two words; `at` on 16 bytes */
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(at) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long wall_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

/* Poll one word until it carries `gen`, bounded by the wall clock from `t0` (0 = not started: the clock is read only once a
 * first look failed).  Answers false when the time ran out. */
__device__ __forceinline__ bool xf_await(const uint2* at, uint32_t gen, unsigned long long wait_ns, unsigned long long& t0, uint32_t& payload) {
    for (;;) {
        for (int i = 0; i < 64; ++i) {
            const uint2 v = xf_load(at);
            if (v.y == gen) { payload = v.x; return true; }
        }
        if (t0 == 0ull) t0 = wall_ns();
        else if (wall_ns() - t0 > wait_ns) return false;
    }
}

/* The same word of every member's slot in this card's own buffer: all loads first, then a look at the tags, and a bounded
 * poll only of those not there yet.  `ok` is cleared when a wait ran out. */
__device__ __forceinline__ void xf_gather(const XfParams& P, uint32_t parity, size_t word, uint32_t (&payload)[XF_MEMBERS_MAX], unsigned long long& t0, bool& ok) {
    uint8_t* local = P.peer[P.index];
    uint2 v[XF_MEMBERS_MAX];
#pragma unroll
    for (uint32_t m = 0; m < XF_MEMBERS_MAX; ++m)
        if (m < P.members) v[m] = xf_load(xf_slot(local, parity, m, P.slot_words, P.members) + word);
#pragma unroll
    for (uint32_t m = 0; m < XF_MEMBERS_MAX; ++m) {
        if (m >= P.members) continue;
        payload[m] = v[m].x;
        if (v[m].y != P.gen && ok) ok = xf_await(xf_slot(local, parity, m, P.slot_words, P.members) + word, P.gen, P.wait_ns, t0, payload[m]);
    }
}

}  // namespace sv
