/* tq_decode.cu — one query's residual over a TurboQuant-coded tier of the cache, codes expanded in flight.
 *
 * The pair attention_weights_tq + attention_residual_mix_tq (engine/src/packages/nn/gpu/kernels/kernels.cuh:2904-2986) as
 * ONE kernel: the fp32 weights buffer between the two doors is never written, the coded keys and values cross HBM once.
 * A coded row is head_dim codes of 4 or 8 bits plus one fp16 scale, so the kernel moves 2-4 times fewer bytes a position
 * than the 16-bit decode kernel and is bound by the same thing, HBM — provided the codes become tensor-core operands
 * without a detour.  They do:
 *   · code tiles (128 positions of one kv head, raw bytes) arrive by TMA into a ring of stages, swizzled;
 *   · a level is fetched from a table in shared memory that holds every entry 32 times, once a bank, so that a warp's 32
 *     lookups never collide whatever the codes are; at 4 bits an entry is indexed by a whole byte and answers both of its
 *     levels at once;
 *   · the looked-up halves are packed straight into the A fragments of mma.sync.m16n8k16 in registers.  No 16-bit tile is
 *     ever written: the contraction index of an MMA may be permuted freely as long as both operands agree, and so may
 *     the rows of an output tile, so every lane reads ONE contiguous run of a coded row — a quarter of a key row for the
 *     scores (its query fragments are loaded in the same order), an eighth of a value row for the mix (its accumulator
 *     rows are mapped back to value columns when the result is written);
 *   · the row scales never touch the operands: a key's scale multiplies its score after the MMA, a value's scale is
 *     folded into its softmax weight before the second MMA.  The levels are exact fp16 numbers, so the products the
 *     tensor core sees are the reference's level values bit for bit.
 * Splits, the fold of a block's warps, the atomic ticket and the last block's merge in a fixed order are the decode
 * kernel's (decode.cu); the result leaves as the reference's residual (m, l, acc[head_dim]) a head.
 *
 * Algorithmic bytes a position and kv head: 2 · (head_dim · width / 8 + 2).
 * Every mbarrier wait is bounded; a wait that runs out ORs "B2TO" into the device's status word and the block leaves. */
#include "common.cuh"
#include <atomic>
#include "kernels.h"
#include "tensormap.cuh"
#include <stdio.h>
#include <string.h>

namespace sv {

static __device__ const uint16_t g_tq_levels_fused[318] = {
#include "tq_levels.inc"
};

template <int DH, int W> struct TqCfg {
    static constexpr int RB = DH * W / 8;                 /* bytes a coded row */
    /* consumer warps, 16 positions of a tile each.  The kernel is bound by instruction issue with few warps to pick from,
     * so as many as registers (query fragments live in shared memory for this) and the ring allow: fifteen and the producer
     * fill the four schedulers' register files at 128 registers a thread (a scheduler's warps share 16 K registers); eight
     * where a 256-byte row makes the tiles too large for two stages of 240 positions. */
    static constexpr int NW = RB > 128 ? 8 : 15;
    static constexpr int BT = 16 * NW;
    static constexpr int BOX = RB > 128 ? 128 : RB;       /* bytes a TMA box row; the swizzle's span */
    static constexpr int BOXES = RB / BOX;
    static constexpr int TILE = BT * RB;                  /* a K (or V) tile */
    static constexpr int STAGE = 2 * TILE;
    static constexpr int RING = RB > 128 ? 128 * 1024 : 120 * 1024;
    static constexpr int STAGES = RING / STAGE > 8 ? 8 : RING / STAGE;
    static constexpr int QROW = DH * 2 + 16;              /* bytes a query head in shared memory: 16 bytes of padding spread the heads over the banks */
    static constexpr int LUT_BYTES = 256 * 256;             /* 256 entries, each 32 copies (a bank each) in a 256-byte slot */
    static constexpr int QB = RB / 4;                     /* bytes of a key row a lane reads (its quarter) */
    static constexpr int EB = RB / 8;                     /* bytes of a value row a lane reads (its eighth) */
    static constexpr int KS = DH / 16;                    /* k-steps of the score product = m-tiles of the value product */
};

struct TqParams {
    float* res;
    const uint16_t* q;
    const uint16_t *kscales, *vscales;
    float* partials;
    unsigned int* tickets;
    unsigned int* status;
    uint32_t q_heads, kv_heads, group, length, nsplit, head_blocks, heads_per_block, slot_floats;
    uint32_t vgroup;                             /* rows · group: a kv head's query heads over every row of a prompt chunk, as one list */
    float scale_log2;
};

/* byte address of 16-byte chunk `c` of row `r` in a tile at shared address `tile` (boxes of BOX bytes, swizzled) */
template <int BOX, int BT>
__device__ __forceinline__ uint32_t code_chunk(uint32_t tile, int r, int c) {
    constexpr int CPB = BOX / 16;
    const int box = c / CPB;
    int cc = c % CPB;
    if (BOX == 128) cc ^= (r & 7);
    else if (BOX == 64) cc ^= ((r >> 1) & 3);
    else if (BOX == 32) cc ^= ((r >> 2) & 1);
    return tile + box * (BT * BOX) + r * BOX + cc * 16;
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v; asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a)); return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v; asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a)); return v;
}
/* The table entry of byte `idx` of word `w` for this lane.  An entry is 256 bytes apart from the next (its 32 copies, one
 * a bank, then padding), so the byte moved into bits 8..15 by ONE byte-permute is the entry's offset.  Not volatile: the
 * table never changes while tiles are walked, and the address depends on code words that were read after the tile's
 * barrier, so the compiler may schedule the lookups of several MMA steps together but never ahead of the data. */
__device__ __forceinline__ uint32_t lut_at(uint32_t lut_lane, uint32_t w, int idx) {
    uint32_t v;
    const uint32_t off = __byte_perm(w, 0u, 0x4404u | ((uint32_t)idx << 4));
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(lut_lane + off));
    return v;
}
__device__ __forceinline__ uint32_t lo_lo(uint32_t a, uint32_t b) { return __byte_perm(a, b, 0x5410); }   /* (a.lo, b.lo) */
__device__ __forceinline__ uint32_t hi_hi(uint32_t a, uint32_t b) { return __byte_perm(a, b, 0x7632); }   /* (a.hi, b.hi) */

template <int DH, int W, int NHT>
__global__ void __launch_bounds__((TqCfg<DH, W>::NW + 1) * 32, 1)
tq_attend_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, const TqParams P) {
    using Cfg = TqCfg<DH, W>;
    constexpr int NW = Cfg::NW, BT = Cfg::BT, KS = Cfg::KS, HPB = 8 * NHT, THREADS = (NW + 1) * 32;
    constexpr int QW = Cfg::QB / 4, EW = Cfg::EB / 4;       /* 32-bit words of codes a lane holds: a key row's quarter, a value row's eighth */
    constexpr int DT = SV_DTYPE_FP16;
    static_assert(Cfg::QB >= 16 && Cfg::EB >= 8, "head_dim 128 or 256 at 4 or 8 bits");

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* stage_base = smem;
    uint32_t* lut = (uint32_t*)(smem + Cfg::STAGES * Cfg::STAGE);
    uint8_t* q_s = (uint8_t*)lut + Cfg::LUT_BYTES;          /* [HPB] query heads, zero past `heads` */
    uint64_t* full = (uint64_t*)(q_s + HPB * Cfg::QROW);
    uint64_t* empty = full + Cfg::STAGES;
    volatile uint32_t* abort_flag = (volatile uint32_t*)(empty + Cfg::STAGES);
    uint32_t* ticket_s = (uint32_t*)abort_flag + 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g8 = lane >> 2, t4 = lane & 3;
    const int hb = blockIdx.x % P.head_blocks, rest = blockIdx.x / P.head_blocks;
    const int kvh = rest % P.kv_heads, split = rest / P.kv_heads, nsplit = P.nsplit;
    /* this block's query heads: entries v0 .. v0 + heads of the kv head's list — row v / group, head v % group of its group */
    const int v0 = hb * P.heads_per_block;
    const int heads = min((int)P.heads_per_block, (int)P.vgroup - v0);
    auto head_at = [&](int h) { const int v = v0 + h; return (size_t)(v / (int)P.group) * P.q_heads + (size_t)kvh * P.group + (size_t)(v % (int)P.group); };
    const int len = (int)P.length;
    const int tiles = (len + BT - 1) / BT, chunk = (tiles + nsplit - 1) / nsplit;
    const int tile_begin = split * chunk, tile_end = min(tiles, tile_begin + chunk), nt = max(tile_end - tile_begin, 0);
    const int slot_base = kvh * P.head_blocks + hb, slot_stride = P.kv_heads * P.head_blocks, ticket = slot_base;

    if (tid == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], NW); }
        *abort_flag = 0u;
        mbar_fence_init();
        /* Programmatic dependent launch (a no-op for a launch without the attribute): the block may have been scheduled while
         * the grid ahead on the stream was still running — a tier's codes may be that grid's work (the mixer re-codes rows
         * just before it attends), so nothing is read before this wait; the launch's latency and this set-up are off the path. */
        asm volatile("griddepcontrol.wait;" ::: "memory");
        /* the ring's first fill is asked for here, ahead of the table and the block's first barrier: the codes are what the
         * work waits for, and nothing has to be free for them yet */
        if (nt > 0) {
            tma_prefetch_desc(&kmap); tma_prefetch_desc(&vmap);
            const uint64_t pol = l2_policy_evict_first();
            for (int it = 0; it < Cfg::STAGES && it < nt; ++it) {
                const int pos0 = (tile_begin + it) * BT;
                uint8_t* st = stage_base + it * Cfg::STAGE;
                mbar_expect_tx(&full[it], Cfg::STAGE);
#pragma unroll
                for (int c = 0; c < Cfg::BOXES; ++c)
                    tma_load_2d_hint(st + c * (BT * Cfg::BOX), &kmap, &full[it], kvh * Cfg::RB + c * Cfg::BOX, pos0, pol);
#pragma unroll
                for (int c = 0; c < Cfg::BOXES; ++c)
                    tma_load_2d_hint(st + Cfg::TILE + c * (BT * Cfg::BOX), &vmap, &full[it], kvh * Cfg::RB + c * Cfg::BOX, pos0, pol);
            }
        }
    }
    /* the level table, every entry once a bank: [byte][bank], 256 bytes an entry.  8 bits: the byte's level in both halves.  4 bits: the
     * low nibble's level in the low half, the high nibble's in the high half.  A thread's levels are all asked for before the
     * first is stored: one trip to memory, not one a word. */
    {
        constexpr int PER = (256 * 32 + THREADS - 1) / THREADS;
        uint32_t e[PER];
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int b = min((tid + k * THREADS) >> 5, 255);
            if (W == 8) { const uint32_t l = g_tq_levels_fused[62 + b]; e[k] = l | (l << 16); }
            else e[k] = (uint32_t)g_tq_levels_fused[14 + (b & 15)] | ((uint32_t)g_tq_levels_fused[14 + (b >> 4)] << 16);
        }
#pragma unroll
        for (int k = 0; k < PER; ++k) { const int i = tid + k * THREADS; if (i < 256 * 32) lut[(i >> 5) * 64 + (i & 31)] = e[k]; }
    }
    for (int i = tid; i < HPB * (DH / 4); i += THREADS) {           /* 8 bytes a step */
        const int h = i / (DH / 4), e = (i % (DH / 4)) * 4;
        uint2 v = make_uint2(0u, 0u);
        if (h < heads) v = *reinterpret_cast<const uint2*>(P.q + head_at(h) * DH + e);
        *reinterpret_cast<uint2*>(q_s + h * Cfg::QROW + e * 2) = v;
    }
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   /* the launch behind this one may be scheduled once every block has got this far */

    float m_run[NHT][2], l_run[NHT][2];
    float oacc[NHT][KS][4];
#pragma unroll
    for (int n = 0; n < NHT; ++n) {
        m_run[n][0] = m_run[n][1] = -INFINITY; l_run[n][0] = l_run[n][1] = 0.f;
#pragma unroll
        for (int k = 0; k < KS; ++k) { oacc[n][k][0] = oacc[n][k][1] = oacc[n][k][2] = oacc[n][k][3] = 0.f; }
    }

    if (warp == NW) {
        /* ---- producer: one lane issues every TMA load of this block ---- */
        if (lane == 0 && nt > 0) {
            const uint64_t pol = l2_policy_evict_first();
            int issued = min((int)Cfg::STAGES, nt);                 /* the first fill is on its way */
            for (int it = issued; it < nt; ++it, ++issued) {
                const int s = it % Cfg::STAGES;
                if (it >= Cfg::STAGES && !mbar_wait(&empty[s], ((it / Cfg::STAGES) - 1) & 1, abort_flag, P.status)) break;
                const int pos0 = (tile_begin + it) * BT;
                uint8_t* st = stage_base + s * Cfg::STAGE;
                mbar_expect_tx(&full[s], Cfg::STAGE);
#pragma unroll
                for (int c = 0; c < Cfg::BOXES; ++c)
                    tma_load_2d_hint(st + c * (BT * Cfg::BOX), &kmap, &full[s], kvh * Cfg::RB + c * Cfg::BOX, pos0, pol);
#pragma unroll
                for (int c = 0; c < Cfg::BOXES; ++c)
                    tma_load_2d_hint(st + Cfg::TILE + c * (BT * Cfg::BOX), &vmap, &full[s], kvh * Cfg::RB + c * Cfg::BOX, pos0, pol);
            }
            /* a wait gave up somewhere in the block: the copies already asked for get a bounded chance to land before the
             * block's memory is given back */
            if (*abort_flag != 0u)
                for (int it = issued > Cfg::STAGES ? issued - Cfg::STAGES : 0; it < issued; ++it)
                    for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&full[it % Cfg::STAGES], (it / Cfg::STAGES) & 1); ++i) {}
        }
    } else {
        /* ---- consumers.  For k-step kk this lane's four contraction slots are elements t4·DH/4 + 4kk .. +3 of its head
         * (g8) — the order in which it reads the coded keys — so a query fragment is 8 bytes of the staged head. ---- */
        const uint32_t q_lane = smem_u32(q_s) + g8 * Cfg::QROW + t4 * (DH / 2);
        const uint32_t lut_lane = smem_u32(lut) + lane * 4;
        const int rowA = warp * 16 + g8, rowB = rowA + 8;          /* this lane's score rows (positions of the tile) */
        const int pv0 = warp * 16 + 2 * t4;                        /* its value positions: pv0, pv0+1, pv0+8, pv0+9 */
        /* The rows' scales run one tile ahead in registers: they are single halves scattered 2·kv_heads bytes apart, a trip
         * to L2 or HBM each, and nothing else in the loop waits that long once the ring is full. */
        uint16_t n_ksA = 0, n_ksB = 0, n_vsA = 0, n_vsB = 0;
        auto fetch_scales = [&](int tile_it) {
            const int p0 = (tile_begin + tile_it) * BT;
            const bool a = p0 + rowA < len, b = p0 + rowB < len;
            const size_t at_a = (size_t)(p0 + rowA) * P.kv_heads + kvh, at_b = (size_t)(p0 + rowB) * P.kv_heads + kvh;
            n_ksA = a ? P.kscales[at_a] : (uint16_t)0; n_ksB = b ? P.kscales[at_b] : (uint16_t)0;
            n_vsA = a ? P.vscales[at_a] : (uint16_t)0; n_vsB = b ? P.vscales[at_b] : (uint16_t)0;
        };
        if (nt > 0) fetch_scales(0);
        for (int it = 0; it < nt; ++it) {
            const int s = it % Cfg::STAGES;
            const int pos0 = (tile_begin + it) * BT;
            const bool vA = pos0 + rowA < len, vB = pos0 + rowB < len;
            const uint16_t ksA = n_ksA, ksB = n_ksB, vsA = n_vsA, vsB = n_vsB;
            if (it + 1 < nt) fetch_scales(it + 1);
            if (!mbar_wait(&full[s], (it / Cfg::STAGES) & 1, abort_flag, P.status)) break;
            const uint32_t kt = smem_u32(stage_base + s * Cfg::STAGE), vt = kt + Cfg::TILE;

            /* S^T[16 positions][heads] = levels(K) · Q^T */
            uint32_t kc0[QW], kc1[QW];
#pragma unroll
            for (int c = 0; c < Cfg::QB / 16; ++c) {
                const uint4 a = lds128(code_chunk<Cfg::BOX, BT>(kt, rowA, t4 * (Cfg::QB / 16) + c));
                const uint4 b = lds128(code_chunk<Cfg::BOX, BT>(kt, rowB, t4 * (Cfg::QB / 16) + c));
                kc0[4 * c] = a.x; kc0[4 * c + 1] = a.y; kc0[4 * c + 2] = a.z; kc0[4 * c + 3] = a.w;
                kc1[4 * c] = b.x; kc1[4 * c + 1] = b.y; kc1[4 * c + 2] = b.z; kc1[4 * c + 3] = b.w;
            }
            float sa[NHT][4], sb[NHT][4];
#pragma unroll
            for (int n = 0; n < NHT; ++n) { sa[n][0] = sa[n][1] = sa[n][2] = sa[n][3] = 0.f; sb[n][0] = sb[n][1] = sb[n][2] = sb[n][3] = 0.f; }
#pragma unroll
            for (int kk = 0; kk < KS; ++kk) {
                uint32_t a0, a1, a2, a3;
                if (W == 8) {
                    const uint32_t w0 = kc0[kk], w1 = kc1[kk];
                    a0 = lo_lo(lut_at(lut_lane, w0, 0), lut_at(lut_lane, w0, 1)); a2 = lo_lo(lut_at(lut_lane, w0, 2), lut_at(lut_lane, w0, 3));
                    a1 = lo_lo(lut_at(lut_lane, w1, 0), lut_at(lut_lane, w1, 1)); a3 = lo_lo(lut_at(lut_lane, w1, 2), lut_at(lut_lane, w1, 3));
                } else {
                    const uint32_t w0 = kc0[kk >> 1], w1 = kc1[kk >> 1];
                    a0 = lut_at(lut_lane, w0, 2 * (kk & 1)); a2 = lut_at(lut_lane, w0, 2 * (kk & 1) + 1);
                    a1 = lut_at(lut_lane, w1, 2 * (kk & 1)); a3 = lut_at(lut_lane, w1, 2 * (kk & 1) + 1);
                }
#pragma unroll
                for (int n = 0; n < NHT; ++n) {
                    uint32_t b0, b1;
                    asm("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(q_lane + n * 8 * Cfg::QROW + kk * 8));
                    if (kk & 1) mma16816<DT>(sb[n], a0, a1, a2, a3, b0, b1);
                    else        mma16816<DT>(sa[n], a0, a1, a2, a3, b0, b1);
                }
            }

            /* online softmax over positions (accumulator rows), per head (accumulator columns); a key's scale joins its
             * score here, a value's scale its weight */
            const float kA = Elem<DT>::to_float(ksA) * P.scale_log2, kB = Elem<DT>::to_float(ksB) * P.scale_log2;
            const float wA = Elem<DT>::to_float(vsA), wB = Elem<DT>::to_float(vsB);
            uint32_t pb0[NHT], pb1[NHT];
#pragma unroll
            for (int n = 0; n < NHT; ++n) {
                float t0 = vA ? (sa[n][0] + sb[n][0]) * kA : -INFINITY;
                float t1 = vA ? (sa[n][1] + sb[n][1]) * kA : -INFINITY;
                float t2 = vB ? (sa[n][2] + sb[n][2]) * kB : -INFINITY;
                float t3 = vB ? (sa[n][3] + sb[n][3]) * kB : -INFINITY;
                float ma = fmaxf(t0, t2), mb = fmaxf(t1, t3);
#pragma unroll
                for (int x = 4; x < 32; x <<= 1) {
                    ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, x));
                    mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, x));
                }
                const float na = fmaxf(m_run[n][0], ma), nb = fmaxf(m_run[n][1], mb);
                const float ua = (na == -INFINITY) ? 0.f : na, ub = (nb == -INFINITY) ? 0.f : nb;
                const float fa = fast_exp2(m_run[n][0] - ua), fb = fast_exp2(m_run[n][1] - ub);
                m_run[n][0] = na; m_run[n][1] = nb;
                const float p0 = fast_exp2(t0 - ua), p1 = fast_exp2(t1 - ub), p2 = fast_exp2(t2 - ua), p3 = fast_exp2(t3 - ub);
                l_run[n][0] = l_run[n][0] * fa + p0 + p2;
                l_run[n][1] = l_run[n][1] * fb + p1 + p3;
                if (__any_sync(0xffffffffu, fa != 1.f || fb != 1.f)) {
#pragma unroll
                    for (int k = 0; k < KS; ++k) { oacc[n][k][0] *= fa; oacc[n][k][2] *= fa; oacc[n][k][1] *= fb; oacc[n][k][3] *= fb; }
                }
                pb0[n] = movm_t(Elem<DT>::pack2(p0 * wA, p1 * wA));
                pb1[n] = movm_t(Elem<DT>::pack2(p2 * wB, p3 * wB));
            }

            /* O^T[value column][head] += levels(V)^T · (P ⊙ scale)^T.  Row g8 of m-tile mt is value column g8·DH/8 + 2mt,
             * row g8+8 the column after it: the lane's eighth of a value row, in order. */
            uint32_t vc[4][EW];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int r = pv0 + (j & 1) + (j >> 1) * 8;
                if constexpr (Cfg::EB >= 16) {
#pragma unroll
                    for (int c = 0; c < Cfg::EB / 16; ++c) {
                        const uint4 a = lds128(code_chunk<Cfg::BOX, BT>(vt, r, g8 * (Cfg::EB / 16) + c));
                        vc[j][4 * c] = a.x; vc[j][4 * c + 1] = a.y; vc[j][4 * c + 2] = a.z; vc[j][4 * c + 3] = a.w;
                    }
                } else {
                    const uint2 a = lds64(code_chunk<Cfg::BOX, BT>(vt, r, g8 >> 1) + (g8 & 1) * 8);
                    vc[j][0] = a.x; vc[j][1] = a.y;
                }
            }
#pragma unroll
            for (int mt = 0; mt < KS; ++mt) {
                uint32_t a0, a1, a2, a3;
                if (W == 8) {
                    /* bytes 2mt and 2mt+1 of each position's run: the two columns of this m-tile */
                    const int w = mt >> 1, b = 2 * (mt & 1);
                    const uint32_t l0 = lut_at(lut_lane, vc[0][w], b), l1 = lut_at(lut_lane, vc[1][w], b);
                    const uint32_t l2 = lut_at(lut_lane, vc[2][w], b), l3 = lut_at(lut_lane, vc[3][w], b);
                    const uint32_t h0 = lut_at(lut_lane, vc[0][w], b + 1), h1 = lut_at(lut_lane, vc[1][w], b + 1);
                    const uint32_t h2 = lut_at(lut_lane, vc[2][w], b + 1), h3 = lut_at(lut_lane, vc[3][w], b + 1);
                    a0 = lo_lo(l0, l1); a1 = lo_lo(h0, h1); a2 = lo_lo(l2, l3); a3 = lo_lo(h2, h3);
                } else {
                    /* byte mt holds both columns: low nibble the first, high nibble the second */
                    const int w = mt >> 2, b = mt & 3;
                    const uint32_t l0 = lut_at(lut_lane, vc[0][w], b), l1 = lut_at(lut_lane, vc[1][w], b);
                    const uint32_t l2 = lut_at(lut_lane, vc[2][w], b), l3 = lut_at(lut_lane, vc[3][w], b);
                    a0 = lo_lo(l0, l1); a1 = hi_hi(l0, l1); a2 = lo_lo(l2, l3); a3 = hi_hi(l2, l3);
                }
#pragma unroll
                for (int n = 0; n < NHT; ++n) mma16816<DT>(oacc[n][mt], a0, a1, a2, a3, pb0[n], pb1[n]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        /* the lanes that share a head column hold disjoint positions: fold their sums */
#pragma unroll
        for (int n = 0; n < NHT; ++n)
#pragma unroll
            for (int x = 4; x < 32; x <<= 1) {
                l_run[n][0] += __shfl_xor_sync(0xffffffffu, l_run[n][0], x);
                l_run[n][1] += __shfl_xor_sync(0xffffffffu, l_run[n][1], x);
            }
    }

    /* ---- fold the warps' partials through shared memory (the ring and the table are free now) ---- */
    __syncthreads();
    float* wm = (float*)stage_base;                   /* [NW][HPB] */
    float* wl = wm + NW * HPB;                        /* [NW][HPB] */
    float* wo = wl + NW * HPB;                        /* [NW][HPB][DH] */
    static_assert((size_t)NW * HPB * (DH + 2) * 4 <= (size_t)Cfg::STAGES * Cfg::STAGE + Cfg::LUT_BYTES, "the fold fits in the ring and the table");
    static_assert(Cfg::STAGES >= 2, "at least two stages in the ring");
    if (warp < NW) {
        const int c2 = t4 * 2;
#pragma unroll
        for (int n = 0; n < NHT; ++n) {
            const int ha = n * 8 + c2;
            if (g8 == 0) {
                wm[warp * HPB + ha] = m_run[n][0]; wm[warp * HPB + ha + 1] = m_run[n][1];
                wl[warp * HPB + ha] = l_run[n][0]; wl[warp * HPB + ha + 1] = l_run[n][1];
            }
#pragma unroll
            for (int k = 0; k < KS; ++k) {
                float* base = wo + (size_t)(warp * HPB) * DH + g8 * (DH / 8) + 2 * k;      /* this lane's two value columns of m-tile k */
                base[(ha) * DH] = oacc[n][k][0];
                base[(ha + 1) * DH] = oacc[n][k][1];
                base[(ha) * DH + 1] = oacc[n][k][2];
                base[(ha + 1) * DH + 1] = oacc[n][k][3];
            }
        }
    }
    __syncthreads();

    const uint32_t SF = P.slot_floats;                /* floats a head in scratch: DH + 2 */
    const bool single = (nsplit == 1);
    float* my_slot = P.partials + (size_t)(slot_base + split * slot_stride) * HPB * SF;
    for (int i = tid; i < heads * DH; i += THREADS) {
        const int h = i / DH, e = i % DH;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) m = fmaxf(m, wm[w * HPB + h]);
        float acc = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float mw = wm[w * HPB + h];
            if (mw != -INFINITY) { const float f = fast_exp2(mw - m); acc += wo[(size_t)(w * HPB + h) * DH + e] * f; l += wl[w * HPB + h] * f; }
        }
        if (single) {
            float* r = P.res + head_at(h) * (DH + 2);
            r[2 + e] = acc;
            if (e == 0) { r[0] = m * SV_LN2; r[1] = l; }
        } else {
            my_slot[(size_t)h * DH + e] = acc;
            if (e == 0) { my_slot[HPB * DH + 2 * h] = m; my_slot[HPB * DH + 2 * h + 1] = l; }
        }
    }
    if (single) return;

    /* ---- arrive; the block that arrives last merges the splits, everything it needs asked of L2 at once (decode.cu) ---- */
    __threadfence();
    __syncthreads();
    if (tid == 0) *ticket_s = atomicAdd(&P.tickets[ticket], 1u);
    __syncthreads();
    if (*ticket_s != (uint32_t)(nsplit - 1)) return;
    __threadfence();
    constexpr int RUN_MAX = 16;
    float* fac = (float*)stage_base;                  /* [heads][nsplit] */
    float* mh = fac + HPB * nsplit;
    float* lh = mh + HPB;
    float4* part = (float4*)(lh + HPB + ((4 - ((2 * HPB + HPB * nsplit) & 3)) & 3));
    const int e4n = heads * (DH / 4);
    int runs = THREADS / e4n;
    if (runs < 1) runs = 1;
    if (runs > nsplit) runs = nsplit;
    const int run_len = (nsplit + runs - 1) / runs;
    const size_t slot_f = (size_t)HPB * SF, step = (size_t)slot_stride * slot_f;
    const float* base = P.partials + (size_t)slot_base * slot_f;
    const bool one_pass = run_len <= RUN_MAX && runs * e4n <= THREADS;
    float4 x[RUN_MAX];
    int my_e4 = 0, my_run = 0, s0 = 0, s1 = 0;
    if (one_pass && tid < runs * e4n) {
        my_e4 = tid % e4n; my_run = tid / e4n; s0 = my_run * run_len; s1 = min(nsplit, s0 + run_len);
        const float* r = base + (size_t)(my_e4 / (DH / 4)) * DH + (my_e4 % (DH / 4)) * 4;
#pragma unroll
        for (int u = 0; u < RUN_MAX; ++u) x[u] = __ldcg(reinterpret_cast<const float4*>(r + (size_t)min(s0 + u, nsplit - 1) * step));
    }
    for (int h = warp; h < heads; h += NW + 1) {
        float m = -INFINITY;
        for (int sp = lane; sp < nsplit; sp += 32) m = fmaxf(m, __ldcg(base + (size_t)sp * step + HPB * DH + 2 * h));
        for (int xo = 16; xo > 0; xo >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, xo));
        float l = 0.f;
        for (int sp = lane; sp < nsplit; sp += 32) {
            const float* r = base + (size_t)sp * step + HPB * DH + 2 * h;
            const float ms = __ldcg(r);
            const float f = (ms == -INFINITY) ? 0.f : fast_exp2(ms - m);
            fac[h * nsplit + sp] = f;
            l += __ldcg(r + 1) * f;
        }
        for (int xo = 16; xo > 0; xo >>= 1) l += __shfl_xor_sync(0xffffffffu, l, xo);
        if (lane == 0) { mh[h] = m; lh[h] = l; }
    }
    __syncthreads();
    if (one_pass) {
        if (tid < runs * e4n) {
            const float* f = fac + (my_e4 / (DH / 4)) * nsplit;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int u = 0; u < RUN_MAX; ++u)
                if (s0 + u < s1) { const float w = f[s0 + u]; acc.x += x[u].x * w; acc.y += x[u].y * w; acc.z += x[u].z * w; acc.w += x[u].w * w; }
            part[my_run * e4n + my_e4] = acc;
        }
        __syncthreads();
    }
    for (int i4 = tid; i4 < e4n; i4 += THREADS) {
        const int h = i4 / (DH / 4), e = (i4 % (DH / 4)) * 4;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (one_pass) {
            for (int g = 0; g < runs; ++g) { const float4 p4 = part[g * e4n + i4]; acc.x += p4.x; acc.y += p4.y; acc.z += p4.z; acc.w += p4.w; }
        } else {
            const float* r = base + (size_t)h * DH + e;
            const float* f = fac + h * nsplit;
            int sp = 0;
            for (; sp + 8 <= nsplit; sp += 8) {
                float4 y[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) y[u] = __ldcg(reinterpret_cast<const float4*>(r + (size_t)(sp + u) * step));
#pragma unroll
                for (int u = 0; u < 8; ++u) { const float w = f[sp + u]; acc.x += y[u].x * w; acc.y += y[u].y * w; acc.z += y[u].z * w; acc.w += y[u].w * w; }
            }
            for (; sp < nsplit; ++sp) {
                const float4 y = __ldcg(reinterpret_cast<const float4*>(r + (size_t)sp * step));
                const float w = f[sp]; acc.x += y.x * w; acc.y += y.y * w; acc.z += y.z * w; acc.w += y.w * w;
            }
        }
        float* ro = P.res + head_at(h) * (DH + 2);
        ro[2 + e] = acc.x; ro[3 + e] = acc.y; ro[4 + e] = acc.z; ro[5 + e] = acc.w;
        if (e == 0) { ro[0] = mh[h] * SV_LN2; ro[1] = lh[h]; }
    }
    if (tid == 0) P.tickets[ticket] = 0u;             /* ready for the next launch */
}

/* ---------------------------------------------------------------------------------------------------------- */

bool tq_attend_fits(const void* q, const void* kcodes, const void* kscales, const void* vcodes, const void* vscales, uint64_t qh, uint64_t kvh,
                    uint64_t dh, uint64_t length, uint64_t d) {
    if ((dh != 128 && dh != 256) || (d != 4 && d != 8)) return false;
    if (kvh == 0 || qh % kvh != 0 || qh / kvh > 64 || length == 0 || length > 0x7FFFFF00ull) return false;
    if ((((uintptr_t)kcodes | (uintptr_t)vcodes) & 15u) || ((uintptr_t)q & 7u) || (((uintptr_t)kscales | (uintptr_t)vscales) & 1u)) return false;
    return encode_tiled_fn() != nullptr;
}

template <int DH, int W, int NHT>
static cudaError_t tq_launch_one(const CUtensorMap& km, const CUtensorMap& vm, const TqParams& P, uint32_t blocks, cudaStream_t st) {
    using Cfg = TqCfg<DH, W>;
    const size_t smem = 1024 + (size_t)Cfg::STAGES * Cfg::STAGE + Cfg::LUT_BYTES + (size_t)8 * NHT * Cfg::QROW + 2 * Cfg::STAGES * 8 + 64;
    static std::atomic<bool> attr_set[64];
    int dev = 0; cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(tq_attend_kernel<DH, W, NHT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        attr_set[dev].store(true, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks); cfg.blockDim = dim3((Cfg::NW + 1) * 32); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = pdl_allowed() ? 1u : 0u;
    const cudaError_t ke = cudaLaunchKernelEx(&cfg, tq_attend_kernel<DH, W, NHT>, km, vm, P);
    if (ke != cudaSuccess) return ke;
    note_launch(1);
    cudaError_t le = cudaGetLastError();           /* a refusal names what was asked for: the message the door prints has no room for it */
    if (le != cudaSuccess) {
        cudaFuncAttributes fa;
        if (cudaFuncGetAttributes(&fa, tq_attend_kernel<DH, W, NHT>) == cudaSuccess)
            fprintf(stderr, "tq_attend<%d,%d,%d>: regs %d maxThreads %d static smem %zu max dyn %d asked %zu threads %d\n", DH, W, NHT, fa.numRegs,
                    fa.maxThreadsPerBlock, fa.sharedSizeBytes, fa.maxDynamicSharedSizeBytes, smem, (Cfg::NW + 1) * 32);
    }
    return le;
}

cudaError_t tq_attend_launch(float* res, const uint16_t* q, const uint8_t* kcodes, const uint16_t* kscales, const uint8_t* vcodes,
                             const uint16_t* vscales, uint64_t qh, uint64_t kvh, uint64_t dh, uint64_t length, uint64_t d, uint64_t rows, cudaStream_t st) {
    DecodeScratch scratch;
    cudaError_t e = decode_device_scratch(&scratch);
    if (e != cudaSuccess) return e;
    /* the rows of a prompt chunk see the same tier: their heads are more heads of the same kv head */
    if (rows == 0 || rows * (qh / kvh) > 4096) return cudaErrorInvalidValue;
    const uint32_t group = (uint32_t)(qh / kvh), vgroup = (uint32_t)rows * group;
    const uint32_t hpb = (vgroup > 8u && dh == 128) ? 16u : 8u, hb = (vgroup + hpb - 1) / hpb;
    const uint32_t rb = (uint32_t)(dh * d / 8), box = rb > 128 ? 128u : rb;
    const uint32_t BT = rb > 128 ? 128u : 240u;            /* TqCfg::BT */
    CUtensorMap km, vm;
    if (!make_map_2d_bytes(&km, kcodes, (uint64_t)kvh * rb, length, (uint64_t)kvh * rb, box, BT) ||
        !make_map_2d_bytes(&vm, vcodes, (uint64_t)kvh * rb, length, (uint64_t)kvh * rb, box, BT)) return cudaErrorInvalidValue;
    TqParams P;
    memset(&P, 0, sizeof P);
    P.res = res; P.q = q; P.kscales = kscales; P.vscales = vscales;
    P.partials = scratch.partials; P.tickets = scratch.tickets; P.status = device_status_word();
    P.q_heads = (uint32_t)qh; P.kv_heads = (uint32_t)kvh; P.group = group; P.vgroup = vgroup; P.length = (uint32_t)length;
    P.head_blocks = hb; P.heads_per_block = hpb; P.slot_floats = (uint32_t)dh + 2u;
    P.scale_log2 = (1.0f / sqrtf((float)dh)) * SV_LOG2E;
    const uint32_t tiles = (uint32_t)((length + BT - 1) / BT), lanes = (uint32_t)kvh * hb;
    uint32_t ns = device_sm_count() / lanes;
    if (ns < 1u) ns = 1u;
    if (tiles / ns >= 64u) ns *= 2u;
    if (ns > tiles) ns = tiles;
    const uint32_t chunk = (tiles + ns - 1) / ns;
    ns = (tiles + chunk - 1) / chunk;
    if (ns > 1024u) ns = 1024u;
    while ((uint64_t)ns * lanes > scratch.slots && ns > 1u) --ns;
    if ((uint64_t)lanes > scratch.tickets_n || (size_t)hpb * P.slot_floats > (size_t)16 * scratch.slot_floats) return cudaErrorInvalidValue;
    P.nsplit = ns;
    const uint32_t blocks = ns * lanes;
#define SV_TQ_CASE(DD, WW, NN) return tq_launch_one<DD, WW, NN>(km, vm, P, blocks, st)
    if (dh == 128) {
        if (d == 8) { if (hpb == 8) SV_TQ_CASE(128, 8, 1); else SV_TQ_CASE(128, 8, 2); }
        else        { if (hpb == 8) SV_TQ_CASE(128, 4, 1); else SV_TQ_CASE(128, 4, 2); }
    } else {
        if (d == 8) SV_TQ_CASE(256, 8, 1); else SV_TQ_CASE(256, 4, 1);
    }
#undef SV_TQ_CASE
    return cudaErrorInvalidValue;
}

}  // namespace sv
