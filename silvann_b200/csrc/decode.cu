/* decode.cu — split-KV grouped-query decode attention for sm_100a.
 *
 * Replaces, in one launch, the reference's two-door decode: `attention_scores` (scores + softmax into an fp32 buffer,
 * engine/src/packages/nn/gpu/kernels/kernels.cuh:894-915,1133-1141) followed by `attention_mix` (:1144-1164), and
 * equally the range-residual pair `attention_weights` + `attention_residual_mix` (:1186-1241) with the split merge
 * `attention_merge` (:1243-1255) and `attention_finish` (:1258-1267).  The fp32 weights buffer is never materialised.
 *
 * Shape of the work.  The cache is [position][kv_head][head_dim] 16-bit; query head h reads kv head h / group.  A
 * block owns one kv head's slice of KV tiles (64 positions each) for up to 8 or 16 query heads of its group, streams
 * K and V through a ring of TMA-filled shared-memory stages (128-byte swizzle, one 64-column box per 128 bytes of a
 * row), and keeps an online softmax in registers.  Heads are the N dimension of the warp MMAs (S^T = K·Q^T and
 * O^T = V^T·P^T), so a group of 8 heads wastes nothing and K/V bytes are read from HBM exactly once per group.
 * One extra warp does nothing but issue TMA loads.  Partials (m, l, acc) of the splits of a group meet in scratch in
 * the reference's residual layout; the block that arrives last (an atomic ticket, no spinning) merges them in split
 * order — so the result does not depend on which block was last — and writes the answer.
 *
 * Algorithmic bytes: 2 · positions · kv_heads · head_dim · 2 per pass (K and V once); everything else is O(heads). */
#include "common.cuh"
#include "kernels.h"
#include "tensormap.cuh"
#include "exchange.cuh"
#include "residual.cuh"
#include <atomic>
#include <mutex>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

namespace sv {

/* Consumer warps a block, each owning 16 positions of a tile: 4 at head_dim 256 (tiles of 64 positions, 64 KB a stage),
 * 8 at head_dim 128 and 64 (tiles of 128 positions), so that the per-tile softmax work keeps pace with a stage's bytes. */
template <int D> struct DecodeCfg {
    static constexpr int NW = (D >= 256) ? 4 : 8;
    static constexpr int BT = 16 * NW;                   /* positions per tile */
    static constexpr int BOXES = D / 64;                 /* 64-column (128-byte) boxes per row */
    static constexpr int BOX_BYTES = BT * 128;
    static constexpr int K_BYTES = BOXES * BOX_BYTES;
    static constexpr int STAGE_BYTES = 2 * K_BYTES;      /* K then V */
    static constexpr int STAGES = (D == 64) ? 6 : 3;     /* 192 KB in flight per SM */
};

struct DecodeParams {
    void* o;
    float* res;
    const uint16_t* q;
    float* partials;
    unsigned int* tickets;
    const DecodeItem* items;
    const int32_t* page_table;
    const int32_t* seq_lens;
    unsigned int* over;
    unsigned int* status;
    uint32_t table_stride, page_pos, pool_pages;
    uint32_t q_heads, kv_heads, group;
    uint32_t length, nsplit, head_blocks, heads_per_block;
    uint32_t slot_floats;
    uint32_t l1, l1_groups, l2_slot0, l1_ticket0;   /* one-sequence calls with many splits meet in two levels: l1 splits a first-level group (0: one level) */
    float scale_log2;
    /* with an exchange (xf.members > 0; one sequence, its splits meeting through scratch): the block that holds a head block's
     * whole residual pushes it to the members and folds theirs — this card's share of a KV range split, finished in the launch */
    XfParams xf;
};


template <int D, int DT, int NHT>
__global__ void __launch_bounds__((DecodeCfg<D>::NW + 1) * 32, 1)
decode_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
              const DecodeParams P) {
    using Cfg = DecodeCfg<D>;
    using E = Elem<DT>;
    constexpr int NW = Cfg::NW, BT = Cfg::BT;
    constexpr int HPB = 8 * NHT;            /* heads per block */
    constexpr int KS = D / 16;              /* k-steps of the score product = m-tiles of the value product */
    constexpr bool QREG = !(NHT == 2 && D >= 128);   /* 16 heads at head_dim >= 128: query fragments are re-read from shared memory */
    constexpr int Q_BYTES = Cfg::BOXES * HPB * 128;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* stage_base = smem;
    uint8_t* q_base = smem + Cfg::STAGES * Cfg::STAGE_BYTES;
    uint64_t* full = (uint64_t*)(q_base + Q_BYTES);
    uint64_t* empty = full + Cfg::STAGES;
    volatile uint32_t* abort_flag = (volatile uint32_t*)(empty + Cfg::STAGES);
    uint32_t* ticket_s = (uint32_t*)abort_flag + 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    /* blocks a cluster (1 when the launch has none): the splits of a cluster meet in shared memory, clusters in scratch */
    const int CL = (int)cluster_nctarank(), crank = (int)cluster_ctarank();

    /* ---- which work is this block's ---- */
    int seq, kvh, head0, heads, tile_begin, tile_end, split, nsplit, slot_base, slot_stride, ticket;
    if (P.items) {
        const DecodeItem it = P.items[blockIdx.x];
        seq = it.seq; kvh = it.kvh; head0 = it.head0; heads = it.heads; tile_begin = it.tile_begin; tile_end = it.tile_end;
        split = it.split; nsplit = it.nsplit; slot_base = it.slot_base; slot_stride = 1; ticket = it.ticket;
    } else {
        /* without clusters the splits of a group are spread over the grid (head blocks fastest); with clusters the splits are
         * fastest, so that the blocks of a cluster are neighbouring splits of one group */
        int hb;
        if (CL > 1) { split = blockIdx.x % P.nsplit; const int rest = blockIdx.x / P.nsplit; hb = rest % P.head_blocks; kvh = rest / P.head_blocks; }
        else { hb = blockIdx.x % P.head_blocks; const int rest = blockIdx.x / P.head_blocks; kvh = rest % P.kv_heads; split = rest / P.kv_heads; }
        nsplit = P.nsplit; seq = 0;
        head0 = kvh * P.group + hb * P.heads_per_block;
        heads = min((int)P.heads_per_block, (int)P.group - hb * (int)P.heads_per_block);
        const int tiles = (P.length + BT - 1) / BT, chunk = (tiles + nsplit - 1) / nsplit;
        tile_begin = split * chunk; tile_end = min(tiles, tile_begin + chunk);
        slot_base = kvh * P.head_blocks + hb; slot_stride = P.kv_heads * P.head_blocks; ticket = slot_base;
    }
    const int len = P.seq_lens ? P.seq_lens[seq] : (int)P.length;
    const int nt = max(tile_end - tile_begin, 0);

    if (tid == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], NW); }
        *abort_flag = 0u;
        mbar_fence_init();
    }
    __syncthreads();

    /* per-thread softmax state for the 2·NHT heads this lane's accumulator columns belong to (log2 units) */
    float m_run[NHT][2], l_run[NHT][2];
    float oacc[NHT][KS][4];
#pragma unroll
    for (int n = 0; n < NHT; ++n) {
        m_run[n][0] = m_run[n][1] = -INFINITY; l_run[n][0] = l_run[n][1] = 0.f;
#pragma unroll
        for (int k = 0; k < KS; ++k) { oacc[n][k][0] = oacc[n][k][1] = oacc[n][k][2] = oacc[n][k][3] = 0.f; }
    }

    /* Programmatic dependent launch (a no-op for a launch without the attribute).  The next launch on the stream may be
     * scheduled as soon as every block of this one has got this far, so its blocks take SMs as this grid's blocks leave them
     * instead of waiting for the whole grid and a launch latency.  What such an early block may do before the grid ahead of
     * it has completed is limited to what that grid cannot have written: this kernel only ever READS the K and V planes, so
     * a following launch of it may stream K and V at once; everything else — the query, scratch, tickets, outputs — is
     * touched only after griddepcontrol.wait, which returns when the grid ahead has completed and its writes are visible. */
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (warp == NW) {
        /* ---- producer: one lane issues every TMA load of this block ---- */
        if (lane == 0 && nt > 0) {
            tma_prefetch_desc(&kmap); tma_prefetch_desc(&vmap);
            const uint64_t pol = l2_policy_evict_first();
            const int32_t* pt = P.page_table ? P.page_table + (size_t)seq * P.table_stride : nullptr;
            for (int it = 0; it < nt; ++it) {
                const int s = it % Cfg::STAGES;
                if (it >= Cfg::STAGES && !mbar_wait(&empty[s], ((it / Cfg::STAGES) - 1) & 1, abort_flag, P.status)) break;
                const int pos0 = (tile_begin + it) * BT;
                int32_t y = pos0;
                if (pt) {
                    /* an entry outside the pool (the -1 padding, a stale table) is never made into an address: the tile is
                     * asked for past the pool's last row, where TMA answers zeros, and the status word says so */
                    const int32_t page = pt[pos0 / (int)P.page_pos];
                    if (page < 0 || page >= (int32_t)P.pool_pages) { y = (int32_t)P.pool_pages * (int)P.page_pos; if (P.status) atomicOr(P.status, SV_STATUS_BAD_PAGE); }
                    else y = page * (int)P.page_pos + pos0 % (int)P.page_pos;
                }
                uint8_t* st = stage_base + s * Cfg::STAGE_BYTES;
                mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
#pragma unroll
                for (int c = 0; c < Cfg::BOXES; ++c)
                    tma_load_2d_hint(st + c * Cfg::BOX_BYTES, &kmap, &full[s], kvh * D + c * 64, y, pol);
#pragma unroll
                for (int c = 0; c < Cfg::BOXES; ++c)
                    tma_load_2d_hint(st + Cfg::K_BYTES + c * Cfg::BOX_BYTES, &vmap, &full[s], kvh * D + c * 64, y, pol);
            }
        }
        asm volatile("griddepcontrol.wait;" ::: "memory");
    } else {
        /* ---- consumers: stage the query heads (zero rows past `heads`), then walk the tiles ---- */
        const uint16_t* qsrc = P.q + ((size_t)seq * P.q_heads + head0) * D;
        /* the query may be the work of the grid ahead, so it is read after the wait; asking L2 for its lines beforehand is
         * harmless (L2 is where writes meet) and takes a trip to memory off the path */
        if (tid < heads * (D / 64)) asm volatile("prefetch.global.L2 [%0];" ::"l"(qsrc + (size_t)tid * 64));
        asm volatile("griddepcontrol.wait;" ::: "memory");
        for (int i = tid; i < HPB * (D / 8); i += NW * 32) {
            const int r = i / (D / 8), j = i % (D / 8);
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (r < heads) val = *reinterpret_cast<const uint4*>(qsrc + (size_t)r * D + j * 8);
            *reinterpret_cast<uint4*>(q_base + (j / 8) * (HPB * 128) + swz128(r, j % 8)) = val;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");

        uint32_t qf[QREG ? NHT : 1][QREG ? KS : 1][2];
        const uint32_t q_u32 = smem_u32(q_base);
        auto load_qfrag = [&](int n, int kk, uint32_t& b0, uint32_t& b1) {
            /* B fragment of Q^T for heads n*8..n*8+7, columns kk*16..+15: two 8x8 blocks (chunks 2kk, 2kk+1) */
            const int chunk = 2 * kk + ((lane >> 3) & 1), row = n * 8 + (lane & 7);
            uint32_t r0, r1, r2, r3;
            ldsm_x4(q_u32 + (chunk / 8) * (HPB * 128) + swz128(row, chunk % 8), r0, r1, r2, r3);
            b0 = r0; b1 = r1; (void)r2; (void)r3;
        };
        if (QREG) {
#pragma unroll
            for (int n = 0; n < NHT; ++n)
#pragma unroll
                for (int kk = 0; kk < KS; ++kk) load_qfrag(n, kk, qf[n][kk][0], qf[n][kk][1]);
        }

        const int r_lo = lane >> 2;                 /* accumulator row (position or value column) of c0/c1 */
        for (int it = 0; it < nt; ++it) {
            const int s = it % Cfg::STAGES;
            if (!mbar_wait(&full[s], (it / Cfg::STAGES) & 1, abort_flag, P.status)) break;
            const uint32_t kst = smem_u32(stage_base + s * Cfg::STAGE_BYTES), vst = kst + Cfg::K_BYTES;
            const int pos0 = (tile_begin + it) * BT + warp * 16;

            /* rows of V past the sequence end may hold anything (a pool page's tail): make them zero so that a
             * zero weight times a NaN cannot reach the accumulator */
            if (pos0 + 16 > len) {
                for (int i = lane; i < 16 * (D / 8); i += 32) {
                    const int r = i / (D / 8), j = i % (D / 8);
                    if (pos0 + r >= len)
                        *reinterpret_cast<uint4*>(stage_base + s * Cfg::STAGE_BYTES + Cfg::K_BYTES + (j / 8) * Cfg::BOX_BYTES +
                                                  swz128(warp * 16 + r, j % 8)) = make_uint4(0u, 0u, 0u, 0u);
                }
                __syncwarp();
            }

            /* S^T[16 positions][heads] = K_tile · Q^T, two interleaved accumulators per head tile */
            float sa[NHT][4], sb[NHT][4];
#pragma unroll
            for (int n = 0; n < NHT; ++n) { sa[n][0] = sa[n][1] = sa[n][2] = sa[n][3] = 0.f; sb[n][0] = sb[n][1] = sb[n][2] = sb[n][3] = 0.f; }
#pragma unroll
            for (int kk = 0; kk < KS; ++kk) {
                const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, chunk = 2 * kk + (lane >> 4);
                uint32_t a0, a1, a2, a3;
                ldsm_x4(kst + (chunk / 8) * Cfg::BOX_BYTES + swz128(row, chunk % 8), a0, a1, a2, a3);
#pragma unroll
                for (int n = 0; n < NHT; ++n) {
                    uint32_t b0, b1;
                    if (QREG) { b0 = qf[n][kk][0]; b1 = qf[n][kk][1]; } else load_qfrag(n, kk, b0, b1);
                    if (kk & 1) mma16816<DT>(sb[n], a0, a1, a2, a3, b0, b1);
                    else        mma16816<DT>(sa[n], a0, a1, a2, a3, b0, b1);
                }
            }

            /* online softmax over positions (accumulator rows), per head (accumulator columns) */
            uint32_t pb0[NHT], pb1[NHT];
            const bool v0 = pos0 + r_lo < len, v1 = pos0 + r_lo + 8 < len;
#pragma unroll
            for (int n = 0; n < NHT; ++n) {
                float t0 = v0 ? (sa[n][0] + sb[n][0]) * P.scale_log2 : -INFINITY;   /* pos r_lo,   head A */
                float t1 = v0 ? (sa[n][1] + sb[n][1]) * P.scale_log2 : -INFINITY;   /* pos r_lo,   head B */
                float t2 = v1 ? (sa[n][2] + sb[n][2]) * P.scale_log2 : -INFINITY;   /* pos r_lo+8, head A */
                float t3 = v1 ? (sa[n][3] + sb[n][3]) * P.scale_log2 : -INFINITY;   /* pos r_lo+8, head B */
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
                const uint32_t w0 = E::pack2(fast_exp2(t0 - ua), fast_exp2(t1 - ub));
                const uint32_t w1 = E::pack2(fast_exp2(t2 - ua), fast_exp2(t3 - ub));
                /* the row sum uses the weights as rounded for the MMA, so weights and normaliser stay consistent */
                const float2 f0 = E::unpack2(w0), f1 = E::unpack2(w1);
                l_run[n][0] = l_run[n][0] * fa + f0.x + f1.x;
                l_run[n][1] = l_run[n][1] * fb + f0.y + f1.y;
                if (__any_sync(0xffffffffu, fa != 1.f || fb != 1.f)) {
#pragma unroll
                    for (int k = 0; k < KS; ++k) { oacc[n][k][0] *= fa; oacc[n][k][2] *= fa; oacc[n][k][1] *= fb; oacc[n][k][3] *= fb; }
                }
                pb0[n] = movm_t(w0); pb1[n] = movm_t(w1);
            }

            /* O^T[value column][head] += V_tile^T · P^T */
#pragma unroll
            for (int mt = 0; mt < KS; ++mt) {
                const int j = lane >> 3, row = warp * 16 + (lane & 7) + (j >> 1) * 8, chunk = 2 * mt + (j & 1);
                uint32_t a0, a1, a2, a3;
                ldsm_x4_t(vst + (chunk / 8) * Cfg::BOX_BYTES + swz128(row, chunk % 8), a0, a1, a2, a3);
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

    /* ---- fold the four warps' partials through shared memory (the stage ring is free now) ---- */
    __syncthreads();
    if (*abort_flag != 0u) {
        /* a wait gave up: copies this block asked for may still be on their way into the ring, so one thread gives every
         * stage a bounded chance to land before the ring is written over and the block leaves (the answer is not
         * meaningful any more — the status word says so — but the arrival protocol below is kept whole) */
        if (tid == 0)
            for (int s = 0; s < Cfg::STAGES && s < nt; ++s) {
                const int last = (nt - 1 - s) / Cfg::STAGES;            /* the last use of stage s */
                for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&full[s], last & 1); ++i) {}
            }
        __syncthreads();
    }
    float* wm = (float*)stage_base;                   /* [NW][HPB] */
    float* wl = wm + NW * HPB;                        /* [NW][HPB] */
    float* wo = wl + NW * HPB;                        /* [NW][HPB][D] */
    if (warp < NW) {
        const int r_lo = lane >> 2, c2 = (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < NHT; ++n) {
            const int ha = n * 8 + c2;
            if (r_lo == 0) {
                wm[warp * HPB + ha] = m_run[n][0]; wm[warp * HPB + ha + 1] = m_run[n][1];
                wl[warp * HPB + ha] = l_run[n][0]; wl[warp * HPB + ha + 1] = l_run[n][1];
            }
#pragma unroll
            for (int k = 0; k < KS; ++k) {
                float* base = wo + (size_t)(warp * HPB) * D + k * 16 + r_lo;
                base[(ha) * D] = oacc[n][k][0];
                base[(ha + 1) * D] = oacc[n][k][1];
                base[(ha) * D + 8] = oacc[n][k][2];
                base[(ha + 1) * D + 8] = oacc[n][k][3];
            }
        }
    }
    __syncthreads();

    const uint32_t SF = P.slot_floats;                /* floats per head in scratch: D + 2 */
    const bool single = (nsplit == 1);
    bool hit = false;
    const bool two_level = CL == 1 && P.l1 != 0u && !P.items && nsplit > (int)P.l1;
    if (CL > 1) {
        /* ---- the splits of this cluster meet in shared memory ----
         * Every block leaves its (m, l, acc) in its own shared memory; after the cluster's barrier block r of the cluster
         * folds columns [r D/CL, (r+1) D/CL) of every head over all CL blocks — read from the peers' shared memory, every
         * load asked for before the first is used, summed in split order — and writes that slice: straight to the answer
         * when the cluster holds all of the group's splits, else to the cluster's slot in scratch, where the clusters of
         * the group meet as single blocks do.  A second barrier keeps every block alive until its peers have read it. */
        float* bacc = wo + (size_t)NW * HPB * D;          /* [HPB][D] */
        float* bm = bacc + HPB * D;                      /* [HPB] log2 units */
        float* bl = bm + HPB;                            /* [HPB] */
        for (int i = tid; i < HPB * D; i += (NW + 1) * 32) {
            const int h = i / D, e = i % D;
            float m = -INFINITY;
#pragma unroll
            for (int w = 0; w < NW; ++w) m = fmaxf(m, wm[w * HPB + h]);
            float acc = 0.f, l = 0.f;
#pragma unroll
            for (int w = 0; w < NW; ++w) {
                const float mw = wm[w * HPB + h];
                if (mw != -INFINITY) { const float f = fast_exp2(mw - m); acc += wo[(size_t)(w * HPB + h) * D + e] * f; l += wl[w * HPB + h] * f; }
            }
            bacc[i] = acc;
            if (e == 0) { bm[h] = m; bl[h] = l; }
        }
        cluster_sync_all();
        const int DS = D / CL;                            /* columns of a head this block folds (CL divides D: it is a power of two <= 16) */
        const int ecl = nsplit / CL, cidx = split / CL;   /* clusters in the group, and which of them this is */
        float* cslot = P.partials + (size_t)(slot_base + cidx * slot_stride) * HPB * SF;
        for (int i = tid; i < heads * DS; i += (NW + 1) * 32) {
            const int h = i / DS, e = crank * DS + i % DS;
            float pm[16], pl[16], pa[16];
#pragma unroll
            for (int r = 0; r < 16; ++r)
                if (r < CL) { pm[r] = ld_cluster_f32(bm + h, (uint32_t)r); pl[r] = ld_cluster_f32(bl + h, (uint32_t)r); pa[r] = ld_cluster_f32(bacc + h * D + e, (uint32_t)r); }
            float m = -INFINITY;
#pragma unroll
            for (int r = 0; r < 16; ++r) if (r < CL) m = fmaxf(m, pm[r]);
            float acc = 0.f, l = 0.f;
#pragma unroll
            for (int r = 0; r < 16; ++r)
                if (r < CL && pm[r] != -INFINITY) { const float f = fast_exp2(pm[r] - m); acc += pa[r] * f; l += pl[r] * f; }
            if (ecl == 1) {
                const size_t hq = (size_t)seq * P.q_heads + head0 + h;
                if (P.o) ((uint16_t*)P.o)[hq * D + e] = E::from_float(acc / l, hit);
                if (P.res) {
                    float* r = P.res + hq * (D + 2);
                    r[2 + e] = acc;
                    if (e == 0) { r[0] = m * SV_LN2; r[1] = l; }
                }
            } else {
                cslot[(size_t)h * D + e] = acc;
                if (e == 0) { cslot[HPB * D + 2 * h] = m; cslot[HPB * D + 2 * h + 1] = l; }
            }
        }
        if (ecl > 1) __threadfence();
        cluster_sync_all();
        if (hit && P.over) atomicOr(P.over, SV_FAULT_OVERFLOW);
        if (ecl == 1 || crank != 0) return;
        /* the cluster's first block carries the cluster's partial to the meeting of the group's clusters */
        nsplit = ecl; split = cidx; hit = false;
        if (tid == 0) *ticket_s = atomicAdd(&P.tickets[ticket], 1u);
        __syncthreads();
        if (*ticket_s != (uint32_t)(nsplit - 1)) return;
        __threadfence();
    } else {
    float* my_slot = P.partials + (size_t)(slot_base + split * slot_stride) * HPB * SF;
    for (int i = tid; i < heads * D; i += (NW + 1) * 32) {
        const int h = i / D, e = i % D;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) m = fmaxf(m, wm[w * HPB + h]);
        float acc = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float mw = wm[w * HPB + h];
            if (mw != -INFINITY) { const float f = fast_exp2(mw - m); acc += wo[(size_t)(w * HPB + h) * D + e] * f; l += wl[w * HPB + h] * f; }
        }
        if (single) {
            const size_t hq = (size_t)seq * P.q_heads + head0 + h;
            if (P.o) ((uint16_t*)P.o)[hq * D + e] = E::from_float(acc / l, hit);
            if (P.res) {
                float* r = P.res + hq * (D + 2);
                r[2 + e] = acc;
                if (e == 0) { r[0] = m * SV_LN2; r[1] = l; }
            }
        } else {
            /* a slot: the heads' accumulators, D floats each on a 16-byte boundary, then (m, l) pairs a head */
            my_slot[(size_t)h * D + e] = acc;
            if (e == 0) { my_slot[HPB * D + 2 * h] = m; my_slot[HPB * D + 2 * h + 1] = l; }
        }
    }
    if (single) {
        if (hit && P.over) atomicOr(P.over, SV_FAULT_OVERFLOW);
        return;
    }

    /* ---- arrive; the last block of the group merges all splits in split order ----
     * With many splits a group meets in two levels: the splits in first-level groups of P.l1, whose last arrivals each merge
     * their group into one partial (side by side, on different SMs), and those partials at the group's own ticket. */
    __threadfence();
    __syncthreads();
    if (two_level) {
        const int g1 = split / (int)P.l1, n1 = min((int)P.l1, nsplit - g1 * (int)P.l1);
        if (tid == 0) *ticket_s = atomicAdd(&P.tickets[P.l1_ticket0 + ticket * P.l1_groups + g1], 1u);
        __syncthreads();
        if (*ticket_s != (uint32_t)(n1 - 1)) return;
    } else {
        if (tid == 0) *ticket_s = atomicAdd(&P.tickets[ticket], 1u);
        __syncthreads();
        if (*ticket_s != (uint32_t)(nsplit - 1)) return;
    }
    __threadfence();
    }
    /* The block is alone with its group by now and bound by trips to L2, so everything it needs is asked for at once:
     * a thread owns four neighbouring elements of a head over one run of splits and has that run's accumulators in
     * flight (16 bytes a load, no branch between the loads) while the warps that own a head fetch the splits' (m, l) and
     * make the factors e^(m_s - m); then the run is summed in split order, the runs in run order — a fixed order, so
     * results repeat bit for bit. */
    constexpr int THREADS = (NW + 1) * 32, RUN_MAX = 16;
    const size_t slot_f = (size_t)HPB * SF;
    const int g1 = two_level ? split / (int)P.l1 : 0;
    const int nsplit_all = nsplit;
    /* what this pass merges and where its answer goes: a first-level group into its second-level slot, or everything into
     * the answer */
    const float* base = P.partials + (size_t)slot_base * slot_f;
    size_t step = (size_t)slot_stride * slot_f;
    float* to_slot = nullptr;
    if (two_level) {
        base += (size_t)g1 * P.l1 * step;
        nsplit = min((int)P.l1, nsplit_all - g1 * (int)P.l1);
        to_slot = P.partials + (size_t)(P.l2_slot0 + ticket * P.l1_groups + g1) * slot_f;
    }
  for (int level = 0;; ++level) {
    float* fac = (float*)stage_base;                  /* [heads][nsplit] */
    float* mh = fac + HPB * nsplit;                   /* [heads] merged m (log2 units), then merged l */
    float* lh = mh + HPB;
    float4* part = (float4*)(lh + HPB + ((4 - ((2 * HPB + HPB * nsplit) & 3)) & 3));   /* [runs][heads * D / 4] */
    const int e4n = heads * (D / 4);
    int runs = THREADS / e4n;                         /* thread groups that share the splits of an element */
    if (runs < 1) runs = 1;
    if (runs > nsplit) runs = nsplit;
    int run_len = (nsplit + runs - 1) / runs;
    const bool one_pass = run_len <= RUN_MAX && runs * e4n <= THREADS;
    /* the (m, l) of a split a lane, asked for ahead of the accumulators so that they are back first */
    const bool ml_lanes = nsplit <= 32 && warp < heads;
    float ms_l = -INFINITY, ls_l = 0.f;
    if (ml_lanes && lane < nsplit) {
        const float* r = base + (size_t)lane * step + HPB * D + 2 * warp;
        ms_l = __ldcg(r); ls_l = __ldcg(r + 1);
    }
    float4 x[RUN_MAX];
    int my_e4 = 0, my_run = 0, s0 = 0, s1 = 0;
    if (one_pass && tid < runs * e4n) {
        my_e4 = tid % e4n; my_run = tid / e4n; s0 = my_run * run_len; s1 = min(nsplit, s0 + run_len);
        const float* r = base + (size_t)(my_e4 / (D / 4)) * D + (my_e4 % (D / 4)) * 4;
#pragma unroll
        for (int u = 0; u < RUN_MAX; ++u) x[u] = __ldcg(reinterpret_cast<const float4*>(r + (size_t)min(s0 + u, nsplit - 1) * step));
    }
    if (ml_lanes) {
        const int h = warp;
        float m = ms_l;
        for (int xo = 16; xo > 0; xo >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, xo));
        const float f = (ms_l == -INFINITY) ? 0.f : fast_exp2(ms_l - m);
        if (lane < nsplit) fac[h * nsplit + lane] = f;
        float l = ls_l * f;
        for (int xo = 16; xo > 0; xo >>= 1) l += __shfl_xor_sync(0xffffffffu, l, xo);
        if (lane == 0) { mh[h] = m; lh[h] = l; }
    }
    for (int h = warp + (ml_lanes ? NW + 1 : 0); h < heads; h += NW + 1) {      /* the heads no warp took above */
        float m = -INFINITY;
        for (int sp = lane; sp < nsplit; sp += 32) m = fmaxf(m, __ldcg(base + (size_t)sp * step + HPB * D + 2 * h));
        for (int xo = 16; xo > 0; xo >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, xo));
        float l = 0.f;
        for (int sp = lane; sp < nsplit; sp += 32) {
            const float* r = base + (size_t)sp * step + HPB * D + 2 * h;
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
            const float* f = fac + (my_e4 / (D / 4)) * nsplit;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int u = 0; u < RUN_MAX; ++u)
                if (s0 + u < s1) { const float w = f[s0 + u]; acc.x += x[u].x * w; acc.y += x[u].y * w; acc.z += x[u].z * w; acc.w += x[u].w * w; }
            part[my_run * e4n + my_e4] = acc;
        }
        __syncthreads();
    }
    for (int i4 = tid; i4 < e4n; i4 += THREADS) {
        const int h = i4 / (D / 4), e = (i4 % (D / 4)) * 4;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (one_pass) {
            for (int g = 0; g < runs; ++g) { const float4 p4 = part[g * e4n + i4]; acc.x += p4.x; acc.y += p4.y; acc.z += p4.z; acc.w += p4.w; }
        } else {
            /* many splits, or more elements than threads: eight loads in flight at a time */
            const float* r = base + (size_t)h * D + e;
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
        const float m = mh[h], l = lh[h];
        if (to_slot) {                                   /* a first-level group's partial, in a slot's layout (m in log2 units) */
            *reinterpret_cast<float4*>(to_slot + (size_t)h * D + e) = acc;
            if (e == 0) { to_slot[HPB * D + 2 * h] = m; to_slot[HPB * D + 2 * h + 1] = l; }
            continue;
        }
        const size_t hq = (size_t)seq * P.q_heads + head0 + h;
        if (P.xf.members != 0u) {
            /* ---- the exchange step in the same launch: this card's residual of the head (m, l, these four sums) goes to every
             * member as tagged words, the members' words are polled (bounded) where they land in this card's own memory, and the
             * ranges are folded in member order with the merge door's arithmetic and finished — the bits of the separate
             * exchange kernel, without its launch ---- */
            const XfParams& X = P.xf;
            const uint32_t parity = X.gen & 1u;
            const size_t wbase = hq * (size_t)(D + 2);
            const float m_ln = m * SV_LN2;
            for (uint32_t mm = 0; mm < X.members; ++mm) {
                uint2* slot = xf_slot(X.peer[mm], parity, X.index, X.slot_words, X.members) + wbase;
                xf_store2(slot + 2 + e, __float_as_uint(acc.x), __float_as_uint(acc.y), X.gen);
                xf_store2(slot + 4 + e, __float_as_uint(acc.z), __float_as_uint(acc.w), X.gen);
                if (e == 0) xf_store2(slot, __float_as_uint(m_ln), __float_as_uint(l), X.gen);
            }
            float tm = 0.f, tl = 0.f;
            float4 ta = make_float4(0.f, 0.f, 0.f, 0.f);
            unsigned long long t0 = 0ull;
            bool ok = true;
            for (uint32_t sm_ = 0; sm_ < X.members; ++sm_) {
                float bm_ = m_ln, bl_ = l;
                float4 ba = acc;
                if (sm_ != X.index) {
                    const uint2* from = xf_slot(X.peer[X.index], parity, sm_, X.slot_words, X.members) + wbase;
                    const uint4 w0 = xf_load2(from), w1 = xf_load2(from + 2 + e), w2 = xf_load2(from + 4 + e);
                    uint32_t pay[6] = {w0.x, w0.z, w1.x, w1.z, w2.x, w2.z};
                    const uint32_t tag[6] = {w0.y, w0.w, w1.y, w1.w, w2.y, w2.w};
                    const uint2* at[6] = {from, from + 1, from + 2 + e, from + 3 + e, from + 4 + e, from + 5 + e};
#pragma unroll
                    for (int u = 0; u < 6; ++u)
                        if (tag[u] != X.gen && ok) ok = xf_await(at[u], X.gen, X.wait_ns, t0, pay[u]);
                    bm_ = __uint_as_float(pay[0]); bl_ = __uint_as_float(pay[1]);
                    ba = make_float4(__uint_as_float(pay[2]), __uint_as_float(pay[3]), __uint_as_float(pay[4]), __uint_as_float(pay[5]));
                }
                if (sm_ == 0u) { tm = bm_; tl = bl_; ta = ba; }
                else {
                    float fa, fb;
                    merge_scalars(tm, tl, bm_, bl_, fa, fb);
                    ta.x = merge_element(ta.x, fa, ba.x, fb); ta.y = merge_element(ta.y, fa, ba.y, fb);
                    ta.z = merge_element(ta.z, fa, ba.z, fb); ta.w = merge_element(ta.w, fa, ba.w, fb);
                }
            }
            if (!ok) { if (P.status) atomicOr(P.status, SV_STATUS_TIMEOUT); continue; }     /* a member never came: said, and nothing written */
            if (P.o) {
                uint16_t* op = (uint16_t*)P.o + hq * D + e;
                op[0] = E::from_float(ta.x / tl, hit); op[1] = E::from_float(ta.y / tl, hit);
                op[2] = E::from_float(ta.z / tl, hit); op[3] = E::from_float(ta.w / tl, hit);
            }
            if (P.res) {
                float* ro = P.res + hq * (D + 2);
                ro[2 + e] = ta.x; ro[3 + e] = ta.y; ro[4 + e] = ta.z; ro[5 + e] = ta.w;
                if (e == 0) { ro[0] = tm; ro[1] = tl; }
            }
            continue;
        }
        if (P.o) {
            uint16_t* op = (uint16_t*)P.o + hq * D + e;
            op[0] = E::from_float(acc.x / l, hit); op[1] = E::from_float(acc.y / l, hit);
            op[2] = E::from_float(acc.z / l, hit); op[3] = E::from_float(acc.w / l, hit);
        }
        if (P.res) {
            float* ro = P.res + hq * (D + 2);
            ro[2 + e] = acc.x; ro[3 + e] = acc.y; ro[4 + e] = acc.z; ro[5 + e] = acc.w;
            if (e == 0) { ro[0] = m * SV_LN2; ro[1] = l; }
        }
    }
    if (!to_slot) break;
    /* the first-level group is one partial now: its ticket is cleared for the next launch, and it goes to the meeting of the
     * group's first-level groups */
    __threadfence();
    __syncthreads();
    if (tid == 0) { P.tickets[P.l1_ticket0 + ticket * P.l1_groups + g1] = 0u; *ticket_s = atomicAdd(&P.tickets[ticket], 1u); }
    __syncthreads();
    if (*ticket_s != P.l1_groups - 1u) return;
    __threadfence();
    base = P.partials + (size_t)(P.l2_slot0 + ticket * P.l1_groups) * slot_f; step = slot_f; nsplit = (int)P.l1_groups; to_slot = nullptr;
    __syncthreads();                                  /* the shared arrays of the pass above are free */
  }
    if (hit && P.over) atomicOr(P.over, SV_FAULT_OVERFLOW);
    if (tid == 0) P.tickets[ticket] = 0u;             /* ready for the next launch */
}

/* ---------------------------------------------------------------------------------------------------------- */
/* host side                                                                                                    */

/* Per-device state made on first use.  Doors are called from up to eight worker threads at once, a thread a device,
 * through the one table, so first use is decided under a lock; after that the values never change. */
static constexpr int DEVICES_MAX = 64;
static std::mutex g_once;
static DecodeScratch g_scratch[DEVICES_MAX];
static unsigned int* g_status[DEVICES_MAX];
static std::atomic<uint32_t> g_sms[DEVICES_MAX];

bool pdl_allowed() {
    static const bool on = []() { const char* v = getenv("SILVANN_B200_PDL"); return !(v && v[0] == '0'); }();
    return on;
}

uint32_t device_sm_count() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= DEVICES_MAX) return 148u;
    uint32_t n = g_sms[d].load(std::memory_order_relaxed);
    if (n == 0u) {
        int v = 0;
        n = (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, d) == cudaSuccess && v > 0) ? (uint32_t)v : 148u;
        g_sms[d].store(n, std::memory_order_relaxed);
    }
    return n;
}

unsigned int* device_status_word() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= DEVICES_MAX) return nullptr;
    std::lock_guard<std::mutex> hold(g_once);
    if (!g_status[d]) {
        unsigned int* p = nullptr;
        if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
        if (cudaMemset(p, 0, 256) != cudaSuccess) { cudaFree(p); return nullptr; }
        g_status[d] = p;
    }
    return g_status[d];
}

cudaError_t decode_device_scratch(DecodeScratch* out) {
    int d = 0;
    cudaError_t e = cudaGetDevice(&d);
    if (e != cudaSuccess) return e;
    if (d < 0 || d >= DEVICES_MAX) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> hold(g_once);
    DecodeScratch& s = g_scratch[d];
    if (!s.partials) {
        const uint32_t slot_floats = 256 + 2;
        const size_t bytes = (size_t)SV_DECODE_MAX_SLOTS * 16 * slot_floats * sizeof(float);
        float* p = nullptr; unsigned int* t = nullptr;
        if ((e = cudaMalloc(&p, bytes)) != cudaSuccess) return e;
        if ((e = cudaMalloc(&t, SV_DECODE_MAX_TICKETS * sizeof(unsigned int))) != cudaSuccess) { cudaFree(p); return e; }
        if ((e = cudaMemset(t, 0, SV_DECODE_MAX_TICKETS * sizeof(unsigned int))) != cudaSuccess) { cudaFree(p); cudaFree(t); return e; }
        s.partials = p; s.tickets = t; s.slots = SV_DECODE_MAX_SLOTS; s.tickets_n = SV_DECODE_MAX_TICKETS; s.slot_floats = slot_floats;
    }
    *out = s;
    return cudaSuccess;
}

static inline uint32_t heads_per_block_for(uint32_t group) { return group <= 8u ? 8u : 16u; }

bool decode_fits(const DecodeCall& c) {
    if (c.head_dim != 64 && c.head_dim != 128 && c.head_dim != 256) return false;
    if (c.kv_heads == 0 || c.q_heads % c.kv_heads != 0) return false;
    if (c.q_heads / c.kv_heads > 64) return false;
    if (((uintptr_t)c.q | (uintptr_t)c.k | (uintptr_t)c.v) & 15u) return false;
    if ((c.kv_heads * c.head_dim * 2u) % 16u != 0) return false;
    if (c.kv_rows == 0 || c.kv_rows > 0x7FFFFFFFull) return false;
    if (c.page_table && (c.page_pos == 0 || c.page_pos % decode_tile_positions(c.head_dim) != 0)) return false;
    return encode_tiled_fn() != nullptr;
}

void decode_auto_split(uint32_t length, uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim, uint32_t sms,
                       uint32_t* nsplit, uint32_t* head_blocks) {
    const uint32_t BT = decode_tile_positions(head_dim);
    const uint32_t group = q_heads / kv_heads, hpb = heads_per_block_for(group), hb = (group + hpb - 1) / hpb;
    const uint32_t tiles = (length + BT - 1) / BT, lanes = kv_heads * hb;
    /* one wave of blocks when the cache is short, up to four when each block still gets a long run of tiles */
    uint32_t want = sms / lanes;
    if (want < 1u) want = 1u;
    if (tiles / want >= 64u) want *= 2u;
    uint32_t ns = want < tiles ? want : tiles;
    if (ns < 1u) ns = 1u;
    const uint32_t chunk = (tiles + ns - 1) / ns;
    ns = (tiles + chunk - 1) / chunk;                       /* no empty split */
    if (ns > 1024u) ns = 1024u;                                /* the merge keeps heads x splits factors in shared memory */
    while (ns * lanes > SV_DECODE_MAX_SLOTS && ns > 1u) --ns;
    *nsplit = ns; *head_blocks = hb;
}

template <int D, int DT, int NHT>
static cudaError_t launch_one(const CUtensorMap& km, const CUtensorMap& vm, const DecodeParams& P, uint32_t blocks,
                              cudaStream_t st, uint32_t cluster = 1u, bool pdl = false) {
    using Cfg = DecodeCfg<D>;
    const size_t smem = 1024 + (size_t)Cfg::STAGES * Cfg::STAGE_BYTES + Cfg::BOXES * 8 * NHT * 128 + 2 * Cfg::STAGES * 8 + 64;
    static std::atomic<bool> attr_set[DEVICES_MAX];       /* setting the attribute twice is harmless; the flag only saves the call */
    int d = 0; cudaGetDevice(&d);
    if (d >= 0 && d < DEVICES_MAX && !attr_set[d].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(decode_kernel<D, DT, NHT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        attr_set[d].store(true, std::memory_order_release);
    }
    if (cluster > 1u || pdl) {
        static std::atomic<bool> wide_set[DEVICES_MAX];   /* clusters of 16 blocks are beyond the portable size of 8 */
        if (cluster > 8u && d >= 0 && d < DEVICES_MAX && !wide_set[d].load(std::memory_order_acquire)) {
            cudaError_t e = cudaFuncSetAttribute(decode_kernel<D, DT, NHT>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            if (e != cudaSuccess) return e;
            wide_set[d].store(true, std::memory_order_release);
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(blocks); cfg.blockDim = dim3((Cfg::NW + 1) * 32); cfg.dynamicSmemBytes = smem; cfg.stream = st;
        cudaLaunchAttribute at[2];
        unsigned na = 0;
        if (cluster > 1u) {
            at[na].id = cudaLaunchAttributeClusterDimension;
            at[na].val.clusterDim.x = cluster; at[na].val.clusterDim.y = 1; at[na].val.clusterDim.z = 1;
            ++na;
        }
        if (pdl) { at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[na].val.programmaticStreamSerializationAllowed = 1; ++na; }
        cfg.attrs = at; cfg.numAttrs = na;
        cudaError_t e = cudaLaunchKernelEx(&cfg, decode_kernel<D, DT, NHT>, km, vm, P);
        if (e != cudaSuccess) return e;
        note_launch(1);
        return cudaGetLastError();
    }
    decode_kernel<D, DT, NHT><<<blocks, (Cfg::NW + 1) * 32, smem, st>>>(km, vm, P);
    note_launch(1);
    return cudaGetLastError();
}

/* How many neighbouring splits of a group share a thread-block cluster (1: none).  SILVANN_B200_DECODE_CLUSTER overrides
 * the choice (1, 2, 4, 8 or 16), SILVANN_B200_DECODE_SPLITS the split count of one-sequence calls that leave it open. */
static uint32_t env_u32(const char* name) {
    const char* v = getenv(name);
    return v ? (uint32_t)strtoul(v, nullptr, 10) : 0u;
}
/* One-sequence calls over a short cache are bound by how the splits meet, not by the stream.  When a kv head's whole
 * cache is at most four tiles a block for a cluster's worth of blocks, the group's splits are ONE cluster and meet in
 * shared memory: no scratch, no ticket, no second pass through L2 (configuration 1: 10.3 -> 8.6 microseconds a launch,
 * 7.7 with the launch overlapped).  Answers the cluster size, or 1. */
static uint32_t decode_cluster_for(uint32_t tiles, uint32_t lanes, uint32_t sms, uint32_t* ns) {
    static const uint32_t forced = env_u32("SILVANN_B200_DECODE_CLUSTER");
    if (forced == 1u) return 1u;
    if (forced == 2u || forced == 4u || forced == 8u || forced == 16u) {
        uint32_t c = forced;
        while (c > 1u && c > *ns) c >>= 1;
        if (c > 1u) *ns = (*ns + c - 1u) / c * c;          /* whole clusters: splits past the last tile are empty and fold as nothing */
        return c;
    }
    uint32_t c = 16u;
    while (c > 1u && (c * lanes > sms || c > tiles)) c >>= 1;
    if (c >= 4u && (tiles + c - 1u) / c <= 4u) { *ns = c; return c; }
    return 1u;
}

cudaError_t decode_launch(const DecodeCall& c) {
    const uint32_t group = c.q_heads / c.kv_heads, hpb = heads_per_block_for(group), hb = (group + hpb - 1) / hpb;
    CUtensorMap km, vm;
    const uint32_t BT = decode_tile_positions(c.head_dim);
    const uint64_t cols = (uint64_t)c.kv_heads * c.head_dim, stride = cols * 2u;
    const bool bf = c.dtype == SV_DTYPE_BF16;
    if (!make_map_2d_sw128(&km, c.k, cols, c.kv_rows, stride, 64u, BT, bf)) return cudaErrorInvalidValue;
    if (!make_map_2d_sw128(&vm, c.v, cols, c.kv_rows, stride, 64u, BT, bf)) return cudaErrorInvalidValue;

    DecodeParams P;
    P.o = c.o; P.res = c.res; P.q = (const uint16_t*)c.q;
    P.partials = c.scratch.partials; P.tickets = c.scratch.tickets; P.items = c.items;
    P.page_table = c.page_table; P.seq_lens = c.seq_lens; P.over = c.over; P.status = device_status_word();
    P.table_stride = c.table_stride; P.page_pos = c.page_pos; P.pool_pages = c.page_pos ? (uint32_t)(c.kv_rows / c.page_pos) : 0u;
    P.q_heads = c.q_heads; P.kv_heads = c.kv_heads; P.group = group;
    P.length = c.length; P.head_blocks = hb; P.heads_per_block = hpb;
    P.slot_floats = c.head_dim + 2u;
    P.l1 = 0; P.l1_groups = 0; P.l2_slot0 = 0; P.l1_ticket0 = 0;
    P.scale_log2 = (1.0f / sqrtf((float)c.head_dim)) * SV_LOG2E;
    memset(&P.xf, 0, sizeof P.xf);
    if (c.xf && (c.items || c.seqs != 1u || c.page_table)) return cudaErrorNotSupported;     /* the exchange step rides on one contiguous sequence's meeting of splits */
    uint32_t blocks, cluster = 1u;
    /* one-sequence calls are a few microseconds long and often follow each other (a layer after a layer): they are launched
     * as programmatic dependents; SILVANN_B200_DECODE_PDL=0 turns that off */
    static const bool pdl_on = []() { const char* v = getenv("SILVANN_B200_DECODE_PDL"); return !(v && v[0] == '0'); }();
    const bool pdl = pdl_on && pdl_allowed() && !c.items;
    if (c.items) { blocks = c.n_items; P.nsplit = 0; }
    else {
        static const uint32_t splits_forced = env_u32("SILVANN_B200_DECODE_SPLITS");
        uint32_t ns = c.nsplit, hb2 = hb;
        if (ns == 0 && splits_forced) ns = splits_forced;
        if (ns == 0) decode_auto_split(c.length, c.q_heads, c.kv_heads, c.head_dim, device_sm_count(), &ns, &hb2);
        const uint32_t tiles = (c.length + BT - 1) / BT;
        if (ns > tiles) ns = tiles;
        if (ns > 1024u) ns = 1024u;
        const uint32_t chunk = (tiles + ns - 1) / ns;
        ns = (tiles + chunk - 1) / chunk;
        if ((c.nsplit == 0 || splits_forced) && !c.xf) cluster = decode_cluster_for(tiles, c.kv_heads * hb, device_sm_count(), &ns);
        if (c.xf) {                                              /* (a cache of one split has no meeting to ride on: the caller exchanges in a launch of its own) */
            if (ns < 2u) return cudaErrorNotSupported;
            P.xf = *static_cast<const XfParams*>(c.xf);
        }
        if ((uint64_t)(ns / cluster) * c.kv_heads * hb > c.scratch.slots || (uint64_t)c.kv_heads * hb > c.scratch.tickets_n) return cudaErrorInvalidValue;
        P.nsplit = ns; blocks = ns * c.kv_heads * hb;
        /* many splits of few groups (one long sequence, a kv head or two a card): the last arrival would merge them all on one
         * SM through L2 — in two levels the first is done side by side */
        const uint32_t lanes = c.kv_heads * hb;
        if (cluster == 1u && ns > 48u && c.nsplit == 0u) {       /* (a caller that names its split count gets exactly that meeting) */
            uint32_t g1 = 8u;
            while (g1 * g1 < ns) ++g1;
            const uint32_t groups = (ns + g1 - 1u) / g1;
            if ((uint64_t)ns * lanes + (uint64_t)groups * lanes <= c.scratch.slots && (uint64_t)lanes + (uint64_t)groups * lanes <= c.scratch.tickets_n) {
                P.l1 = g1; P.l1_groups = groups; P.l2_slot0 = ns * lanes; P.l1_ticket0 = lanes;
            }
        }
    }
    if (blocks == 0) return cudaSuccess;
    if ((size_t)hpb * P.slot_floats > (size_t)16 * c.scratch.slot_floats) return cudaErrorInvalidValue;

    const int nht = hpb == 8 ? 1 : 2;
    if (cluster > 1u) {
        /* a cluster the card cannot place (its size, the blocks' shared memory) is an error of the launch, not of the call:
         * the same work goes out again as single blocks that meet in scratch */
        cudaError_t e = cudaErrorInvalidValue;
#define SV_DECODE_TRY(DD, TT) e = (nht == 1) ? launch_one<DD, TT, 1>(km, vm, P, blocks, c.stream, cluster, pdl) : launch_one<DD, TT, 2>(km, vm, P, blocks, c.stream, cluster, pdl)
        if (c.dtype == SV_DTYPE_FP16) { if (c.head_dim == 64) SV_DECODE_TRY(64, SV_DTYPE_FP16); else if (c.head_dim == 128) SV_DECODE_TRY(128, SV_DTYPE_FP16); else SV_DECODE_TRY(256, SV_DTYPE_FP16); }
        else { if (c.head_dim == 64) SV_DECODE_TRY(64, SV_DTYPE_BF16); else if (c.head_dim == 128) SV_DECODE_TRY(128, SV_DTYPE_BF16); else SV_DECODE_TRY(256, SV_DTYPE_BF16); }
#undef SV_DECODE_TRY
        if (e == cudaSuccess) return e;
        (void)cudaGetLastError();
        cluster = 1u;
        if ((uint64_t)P.nsplit * c.kv_heads * hb > c.scratch.slots) return cudaErrorInvalidValue;
    }
#define SV_DECODE_CASE(DD, TT, NN) return launch_one<DD, TT, NN>(km, vm, P, blocks, c.stream, cluster, pdl)
    if (c.dtype == SV_DTYPE_FP16) {
        if (c.head_dim == 64)  { if (nht == 1) SV_DECODE_CASE(64, SV_DTYPE_FP16, 1);  else SV_DECODE_CASE(64, SV_DTYPE_FP16, 2); }
        if (c.head_dim == 128) { if (nht == 1) SV_DECODE_CASE(128, SV_DTYPE_FP16, 1); else SV_DECODE_CASE(128, SV_DTYPE_FP16, 2); }
        if (c.head_dim == 256) { if (nht == 1) SV_DECODE_CASE(256, SV_DTYPE_FP16, 1); else SV_DECODE_CASE(256, SV_DTYPE_FP16, 2); }
    } else {
        if (c.head_dim == 64)  { if (nht == 1) SV_DECODE_CASE(64, SV_DTYPE_BF16, 1);  else SV_DECODE_CASE(64, SV_DTYPE_BF16, 2); }
        if (c.head_dim == 128) { if (nht == 1) SV_DECODE_CASE(128, SV_DTYPE_BF16, 1); else SV_DECODE_CASE(128, SV_DTYPE_BF16, 2); }
        if (c.head_dim == 256) { if (nht == 1) SV_DECODE_CASE(256, SV_DTYPE_BF16, 1); else SV_DECODE_CASE(256, SV_DTYPE_BF16, 2); }
    }
#undef SV_DECODE_CASE
    return cudaErrorInvalidValue;
}

}  // namespace sv

namespace sv {

/* ================================================================================================================ */
/* A decode entry point that allocates nothing                                                                        */
/*
 * Who needs it.  SiLVANN sizes its buffer pools from the card's free memory when a machine boots and from then on
 * expects every byte to be spoken for: a door that discovers, on its first call in the middle of a turn, that it wants
 * a few more megabytes may be told there are none left — or may stall the whole device, because cudaMalloc waits for
 * the device to go idle.  Hosts that replay work from a captured stream are in the same position: an allocation is not
 * something a capture can contain.  For those callers the split-KV decode is offered once more with its scratch
 * (split partials, arrival tickets and the status word) living in a fixed array that is part of the library image
 * itself, so the kernel's scratch exists as soon as the library is loaded on a device and no call ever asks the
 * runtime for memory.
 *
 * The price is a ceiling and a shared array.  The array is SV_STATIC_SLOTS partial slots (about 5 MB); every device
 * that loads the library carries it until the process ends.  A call whose (splits x kv heads x head blocks) does not
 * fit is refused with a message, never truncated.  Every call on a device uses the same array and finds whatever the
 * previous call left: the tickets are cleared on the caller's stream before each launch (the partials need no
 * clearing: each split writes its slot before anyone reads it), and two calls that overlap in time on one device —
 * different streams, different threads — would race on it.  Serialise them.
 *
 * The array's name means something different on the two sides of the compiler: device code can name `g_static_scratch`
 * directly, but in host code the same identifier is only a handle for the runtime — passing it to a kernel would hand
 * the kernel a host address.  So the host asks the runtime where the array lives on the CURRENT device
 * (cudaGetSymbolAddress), once per device, and passes that address to the kernel.  That lookup happens in the first
 * call on each device; make that first call outside any stream capture. */

#define SV_STATIC_SLOTS 304u                        /* two waves of 148 blocks, and a little */
#define SV_STATIC_TICKETS 256u
#define SV_STATIC_SLOT_FLOATS (16u * (256u + 2u))   /* a slot: up to 16 heads of (m, l, acc[256]) */
#define SV_STATIC_FLOATS (SV_STATIC_SLOTS * SV_STATIC_SLOT_FLOATS)

static __device__ __align__(256) float g_static_scratch[SV_STATIC_FLOATS + SV_STATIC_TICKETS + 64];

struct StaticScratch { float* base; std::atomic<bool> ready; };
static StaticScratch g_static[DEVICES_MAX];

/* The device address of the array on the current device, looked up once per device. */
static cudaError_t static_scratch_address(float** out) {
    int d = 0;
    cudaError_t e = cudaGetDevice(&d);
    if (e != cudaSuccess) return e;
    if (d < 0 || d >= DEVICES_MAX) return cudaErrorInvalidDevice;
    if (!g_static[d].ready.load(std::memory_order_acquire)) {
        void* ptr = nullptr;
        if ((e = cudaGetSymbolAddress(&ptr, g_static_scratch)) != cudaSuccess) return e;
        g_static[d].base = (float*)ptr;                    /* two threads racing here write the same address */
        g_static[d].ready.store(true, std::memory_order_release);
    }
    *out = g_static[d].base;
    return cudaSuccess;
}

/* The allocation-free decode keeps its time-out word inside the fixed array (it may not allocate one).  This reads it
 * for silvann_b200_device_status, which ORs it into its answer; a device on which that entry point has never run has
 * no such word yet and answers 0.  The caller has already waited for the device's default queue. */
cudaError_t static_status_take(unsigned int* word, int clear) {
    *word = 0u;
    int d = 0;
    cudaError_t e = cudaGetDevice(&d);
    if (e != cudaSuccess) return e;
    if (d < 0 || d >= DEVICES_MAX || !g_static[d].ready.load(std::memory_order_acquire)) return cudaSuccess;
    unsigned int* at = (unsigned int*)(g_static[d].base + SV_STATIC_FLOATS) + SV_STATIC_TICKETS;
    if ((e = cudaMemcpy(word, at, sizeof *word, cudaMemcpyDeviceToHost)) != cudaSuccess) return e;
    if (clear && *word != 0u) e = cudaMemset(at, 0, sizeof *word);
    return e;
}

/* 0 ok · 1 the shapes are outside the kernel's fit · 2 the work does not fit the fixed scratch · 3 the runtime refused;
 * `detail` receives the runtime's error or the slots that would have been needed. */
int decode_launch_static(const DecodeCall& c0, uint32_t* detail) {
    DecodeCall c = c0;
    c.items = nullptr; c.page_table = nullptr; c.seq_lens = nullptr; c.seqs = 1; c.kv_rows = c.length;
    if (!decode_fits(c)) return 1;
    const uint32_t group = c.q_heads / c.kv_heads, hpb = heads_per_block_for(group), hb = (group + hpb - 1) / hpb;
    const uint32_t BT = decode_tile_positions(c.head_dim);
    const uint32_t lanes = c.kv_heads * hb, tiles = (c.length + BT - 1) / BT;
    if (lanes > SV_STATIC_TICKETS || lanes > SV_STATIC_SLOTS) { *detail = lanes; return 2; }
    uint32_t ns = c.nsplit, hb2 = hb;
    if (ns == 0) {
        decode_auto_split(c.length, c.q_heads, c.kv_heads, c.head_dim, device_sm_count(), &ns, &hb2);
        if (ns * lanes > SV_STATIC_SLOTS) ns = SV_STATIC_SLOTS / lanes;      /* fewer, longer splits still fit */
    }
    if (ns > tiles) ns = tiles;
    if (ns < 1u) ns = 1u;
    const uint32_t chunk = (tiles + ns - 1) / ns;
    ns = (tiles + chunk - 1) / chunk;
    if (ns > 1024u || (uint64_t)ns * lanes > SV_STATIC_SLOTS) { *detail = ns * lanes; return 2; }

    float* base = nullptr;
    cudaError_t e = static_scratch_address(&base);
    if (e != cudaSuccess) { *detail = (uint32_t)e; return 3; }
    unsigned int* tickets = (unsigned int*)(base + SV_STATIC_FLOATS);
    unsigned int* status = tickets + SV_STATIC_TICKETS;
    /* whatever an earlier call left in the tickets (a launch that failed half way, say) must not count as arrivals */
    if ((e = cudaMemsetAsync(tickets, 0, SV_STATIC_TICKETS * sizeof(unsigned int), c.stream)) != cudaSuccess) { *detail = (uint32_t)e; return 3; }

    CUtensorMap km, vm;
    const uint64_t cols = (uint64_t)c.kv_heads * c.head_dim, stride = cols * 2u;
    const bool bf = c.dtype == SV_DTYPE_BF16;
    if (!make_map_2d_sw128(&km, c.k, cols, c.kv_rows, stride, 64u, BT, bf) || !make_map_2d_sw128(&vm, c.v, cols, c.kv_rows, stride, 64u, BT, bf)) {
        *detail = (uint32_t)cudaErrorInvalidValue; return 3;
    }
    DecodeParams P;
    P.o = c.o; P.res = c.res; P.q = (const uint16_t*)c.q;
    P.partials = base; P.tickets = tickets; P.items = nullptr; P.page_table = nullptr; P.seq_lens = nullptr;
    P.over = c.over; P.status = status;
    P.table_stride = 0; P.page_pos = 0; P.pool_pages = 0;
    P.q_heads = c.q_heads; P.kv_heads = c.kv_heads; P.group = group;
    P.length = c.length; P.nsplit = ns; P.head_blocks = hb; P.heads_per_block = hpb;
    P.slot_floats = c.head_dim + 2u;
    P.l1 = 0; P.l1_groups = 0; P.l2_slot0 = 0; P.l1_ticket0 = 0;
    P.scale_log2 = (1.0f / sqrtf((float)c.head_dim)) * SV_LOG2E;
    memset(&P.xf, 0, sizeof P.xf);
    const uint32_t blocks = ns * lanes;
    const int nht = hpb == 8 ? 1 : 2;
    e = cudaErrorInvalidValue;
#define SV_STATIC_CASE(DD, TT) e = (nht == 1) ? launch_one<DD, TT, 1>(km, vm, P, blocks, c.stream) : launch_one<DD, TT, 2>(km, vm, P, blocks, c.stream)
    if (c.dtype == SV_DTYPE_FP16) {
        if (c.head_dim == 64) SV_STATIC_CASE(64, SV_DTYPE_FP16); else if (c.head_dim == 128) SV_STATIC_CASE(128, SV_DTYPE_FP16); else SV_STATIC_CASE(256, SV_DTYPE_FP16);
    } else {
        if (c.head_dim == 64) SV_STATIC_CASE(64, SV_DTYPE_BF16); else if (c.head_dim == 128) SV_STATIC_CASE(128, SV_DTYPE_BF16); else SV_STATIC_CASE(256, SV_DTYPE_BF16);
    }
#undef SV_STATIC_CASE
    if (e != cudaSuccess) { *detail = (uint32_t)e; return 3; }
    return 0;
}

}  // namespace sv

/* Declared in include/silvann_b200.h.  It lives in this file because the scratch array does: only a translation unit
 * that defines a __device__ array can ask the runtime for its address. */
extern "C" __attribute__((visibility("default")))
int silvann_b200_decode_noalloc(void* o, float* res, const void* q, const void* k, const void* v, uint64_t q_heads, uint64_t kv_heads,
                                uint64_t head_dim, uint64_t length, uint32_t nsplit, int dtype, unsigned int* over, void* stream,
                                char* message, uint32_t message_bytes) {
    auto say = [&](const char* fmt, unsigned long long a, unsigned long long b) {
        if (message && message_bytes) snprintf(message, message_bytes, fmt, a, b);
    };
    if (message && message_bytes) message[0] = 0;
    if (!q || !k || !v || (!o && !res)) { say("decode_noalloc: a null operand", 0, 0); return 1; }
    if (dtype != SV_DTYPE_FP16 && dtype != SV_DTYPE_BF16) { say("decode_noalloc: dtype %llu", (unsigned long long)dtype, 0); return 1; }
    if (q_heads == 0 || kv_heads == 0 || q_heads % kv_heads != 0 || q_heads > 65535) { say("decode_noalloc: %llu query heads do not divide over %llu kv heads", q_heads, kv_heads); return 1; }
    if (length == 0 || length > 0x7FFFFFFFull) { say("decode_noalloc: length %llu", length, 0); return 1; }
    sv::DecodeCall c;
    memset(&c, 0, sizeof c);
    c.o = o; c.res = res; c.q = q; c.k = k; c.v = v;
    c.q_heads = (uint32_t)q_heads; c.kv_heads = (uint32_t)kv_heads; c.head_dim = (uint32_t)head_dim; c.length = (uint32_t)length;
    c.nsplit = nsplit; c.dtype = dtype; c.over = over; c.stream = (cudaStream_t)stream;
    uint32_t detail = 0;
    switch (sv::decode_launch_static(c, &detail)) {
        case 0: return 0;
        case 1: say("decode_noalloc: head_dim %llu, a group of %llu heads, or an operand's alignment is outside the kernel's fit", head_dim, q_heads / kv_heads); return 1;
        case 2: say("decode_noalloc: this call needs %llu scratch slots and the fixed scratch holds %llu; use fewer splits or silvann_b200_decode", detail, (unsigned long long)SV_STATIC_SLOTS); return 1;
        default: say("decode_noalloc: the CUDA runtime answered error %llu", detail, 0); (void)cudaGetLastError(); return 2;
    }
}

