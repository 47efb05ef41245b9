/* mla_decode.cu — one query position of latent attention (MLA) on the 5th-generation tensor cores: many heads over ONE
 * 512-wide latent row a key that is both the key and the value.
 *
 * The reference runs GLM's decode attention as three doors on that latent — attention_scores_grouped (raw scaled scores
 * of 64 heads, engine/src/packages/nn/gpu/kernels/kernels.cuh:931-950), attention_softmax_rows (:1085-1100) and
 * attention_mix (:1144-1164), in engine/src/packages/ai_z__glm_5_3/cpu/opcodes/layer__abi.cuh:279-289 — with an fp32
 * weights buffer between them and the latent read twice.  Its CUDA family has a shared-memory tiled kernel for the scores
 * (engine/src/silicon_families/nvidia_cuda12/overrides/attention.cuh:960-1137).  Here the three are one pass: a latent
 * tile crosses HBM once, sits in shared memory once, and serves both products.
 *
 * The work is 128 flop a byte — a contraction, so it runs on tcgen05 — and the shapes are awkward for it: 64 heads would
 * fill half of an M = 128 accumulator.  So the products are taken TRANSPOSED, keys as the M dimension:
 *     S^T [128 keys x heads]      = C [128 keys x 512] . Q^T          A = the latent tile, K-major;  B = Q, K-major
 *     O^T [512 x heads] (4 x 128) = C^T [512 x 128 keys] . P^T        A = the SAME tile read MN-major; B = P^T, K-major
 * with N = heads (32 or 64) and nothing padded.  TMEM holds S^T (heads columns) and the four blocks of O^T (4 x heads
 * columns) for the whole run of tiles.
 *
 * A block walks a range of 128-key tiles.  Roles: warp 0 loads (Q once; a tile as eight 64-column boxes of 16 KB into an
 * eight-slot ring — a box is refilled as soon as the value product that read it has completed, so the ring is one tile
 * deep but never drains at once); warp 1 issues every MMA; warps 2-9 are the softmax, a thread a key and 32 of the heads: it reads
 * its key's scores from its TMEM lane, the tile's maximum a head is found across threads (an integer-ordered
 * redux.sync a warp, then four values a head through shared memory), the reference maximum is kept unless a tile exceeds
 * it by 2^8 (the weights and the normaliser are relative to the same reference, which is exact), the 16-bit weights go to
 * shared memory transposed as the B operand, and each thread carries its own share of every head's normaliser, summed in
 * a fixed order at the end.  The block's (m, l, acc) leaves in the reference's residual layout — straight to the answer
 * when the block had the whole range, else to scratch, where a second small kernel folds the blocks' partials in range
 * order with attention_merge's arithmetic (kernels.cuh:1243-1255) and finishes.
 *
 * A short range (a few thousand keys: what the sparse attention gathers) gives the card fewer tiles than SMs, and a block's
 * time is then one chain: copies, scores, softmax, value MMAs, the write-out of 131 KB at one SM's store rate.  Where SMs
 * are to spare a share of the range is therefore given to four (or two) blocks, each answering for a quarter (a half) of
 * O^T's columns: all take the scores and the softmax, each issues a quarter of the value MMAs and writes a quarter of the
 * partial answer.
 *
 * Algorithmic bytes: positions x 512 x 2 (the latent once) + 2 x heads x 512 x 2.  Every mbarrier wait is bounded; a wait
 * that runs out raises "B2TO" in the device status word and every role falls through to the exit, where TMEM is released.
 * No cluster, no multicast. */
#include "common.cuh"
#include "kernels.h"
#include "residual.cuh"
#include "tcgen05.cuh"
#include "tensormap.cuh"
#include <atomic>
#include <mutex>

namespace sv {

static constexpr int ML_D = 512;            /* latent width */
static constexpr int ML_BK = 128;           /* keys a tile */
static constexpr int ML_BOXES = ML_D / 64;  /* 64-column boxes a tile */
static constexpr int ML_BOX_BYTES = ML_BK * 128;

struct MlaParams {
    uint16_t* o;              /* [heads][512] or null */
    float* res;               /* [heads][514] or null */
    float* partials;          /* [blocks][heads][514] when blocks > 1 */
    const void* latent;       /* the rows themselves, for L2 prefetches */
    unsigned int* over;
    unsigned int* status;
    uint32_t length, tiles, blocks;   /* blocks: the shares the key range is cut into */
    uint32_t csplit;                  /* blocks a share of the range (1, 2 or 4): each takes 4 / csplit of the answer's four 128-column blocks */
    float scale_log2;
};

template <int NH> struct MlaCfg {
    static constexpr int Q_BOX_BYTES = NH * 128;
    static constexpr int Q_BYTES = ML_BOXES * Q_BOX_BYTES;
    static constexpr int C_BYTES = ML_BOXES * ML_BOX_BYTES;          /* 128 KB: one tile */
    static constexpr int P_BOX_BYTES = NH * 128;                     /* P^T: heads rows of 64 keys */
    static constexpr int P_BYTES = 2 * P_BOX_BYTES;
    static constexpr int HALVES = NH / 32;                           /* softmax warps a TMEM lane quadrant: a thread owns 32 heads of its key */
    static constexpr int SOFT = 128 * HALVES;                        /* softmax threads */
    static constexpr int THREADS = 64 + SOFT;                        /* warp 0 loads, warp 1 issues the MMAs */
    static constexpr int T_S = 0, T_O = NH;                          /* TMEM columns: S^T, then O^T blocks NH apart */
    static constexpr int TMEM_COLS = (5 * NH <= 256) ? 256 : 512;
    static constexpr size_t SMEM = 1024 + Q_BYTES + C_BYTES + P_BYTES + 512 /*barriers*/ + (4 * NH + 5 * NH) * 4;
};

__device__ __forceinline__ int ordered_int(float x) { const int i = __float_as_int(x); return i ^ ((i >> 31) & 0x7FFFFFFF); }
__device__ __forceinline__ float ordered_float(int i) { return __int_as_float(i ^ ((i >> 31) & 0x7FFFFFFF)); }
__device__ __forceinline__ int warp_max_s32(int v) {
    int r;
    asm volatile("redux.sync.max.s32 %0, %1, 0xffffffff;" : "=r"(r) : "r"(v));
    return r;
}
template <int N> __device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, %0;" ::"n"(N) : "memory"); }
/* the same barrier, answering whether any thread brought a true */
template <int N> __device__ __forceinline__ bool softmax_bar_or(bool mine) {
    uint32_t r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 q, %1, 0;\n\tbar.red.or.pred p, 1, %2, q;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(r) : "r"((uint32_t)mine), "n"(N) : "memory");
    return r != 0u;
}
/* asks L2 for a box ahead of its load, so that the load that refills a ring slot is a trip to L2 and not to memory */
__device__ __forceinline__ void tma_prefetch_l2_2d(const void* tmap, int32_t x, int32_t y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(tmap), "r"(x), "r"(y) : "memory");
}

template <int NH, int DT>
__global__ void __launch_bounds__(MlaCfg<NH>::THREADS, 1)
mla_decode_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap cmap, const MlaParams P) {
    using Cfg = MlaCfg<NH>;
    using E = Elem<DT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_s = smem;
    uint8_t* c_s = q_s + Cfg::Q_BYTES;
    uint8_t* p_s = c_s + Cfg::C_BYTES;
    uint64_t* bars = (uint64_t*)(p_s + Cfg::P_BYTES);
    uint64_t* full = bars;                    /* 8: a box has landed */
    uint64_t* empty = full + ML_BOXES;        /* 8: the value product that read the box has completed */
    uint64_t* q_full = empty + ML_BOXES;
    uint64_t* s_full = q_full + 1;            /* the tile's scores are in TMEM */
    uint64_t* p_full = s_full + 1;            /* the tile's weights are in shared memory (4 warps arrive) */
    uint64_t* pv_done = p_full + 1;           /* the tile's value products have completed */
    uint32_t* tmem_slot = (uint32_t*)(pv_done + 1);
    volatile uint32_t* abort_flag = (volatile uint32_t*)(tmem_slot + 1);
    float* wmax = (float*)((uint8_t*)bars + 512);      /* [4 quadrants][NH] a warp's maximum a head (log2 units) */
    float* mref = wmax + 4 * NH;                        /* [NH] the reference maximum a head, log2 units */
    float* fac = mref + NH;                             /* [NH] this tile's rescale factor a head */
    float* lsum = fac + NH;                             /* [NH] the normaliser, at the end */
    float* lhalf = lsum + NH;                           /* [2][NH] its two halves */

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    /* this block's tiles: a contiguous share of the range, as even as whole tiles allow */
    const uint32_t share = blockIdx.x / P.csplit;
    const int j0 = (int)(blockIdx.x % P.csplit) * (4 / (int)P.csplit), j1 = j0 + 4 / (int)P.csplit;   /* this block's column blocks of O^T */
    const int tile0 = (int)(((uint64_t)share * P.tiles) / P.blocks), tile1 = (int)(((uint64_t)(share + 1) * P.tiles) / P.blocks);
    const int nt = tile1 - tile0;

    if (tid == 0) {
        for (int i = 0; i < ML_BOXES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        mbar_init(q_full, 1); mbar_init(s_full, 1); mbar_init(p_full, 4 * Cfg::HALVES); mbar_init(pv_done, 1);
        *abort_flag = 0u;
        mbar_fence_init();
        /* Programmatic dependent launch (a no-op for a launch without the attribute): the block may have been scheduled while
         * the grid ahead on the stream — the fold of the call before, or whatever gathered this latent — was still running;
         * nothing of that grid's is read, and nothing it reads is overwritten, before this wait has returned. */
        asm volatile("griddepcontrol.wait;" ::: "memory");
        /* Q and the first tile are asked for here, ahead of the TMEM allocation and the block's first barrier: they head the
         * block's chain of dependent steps */
        if (nt > 0) {
            tma_prefetch_desc(&qmap); tma_prefetch_desc(&cmap);
            mbar_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
            for (int i = 0; i < ML_BOXES; ++i) tma_load_2d(q_s + i * Cfg::Q_BOX_BYTES, &qmap, q_full, i * 64, 0);
            const uint64_t pol0 = l2_policy_evict_first();
#pragma unroll
            for (int i = 0; i < ML_BOXES; ++i) {
                mbar_expect_tx(&full[i], ML_BOX_BYTES);
                tma_load_2d_hint(c_s + i * ML_BOX_BYTES, &cmap, &full[i], i * 64, tile0 * ML_BK, pol0);
            }
        }
    }
    if (tid < NH) mref[tid] = -INFINITY;
    if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    if (warp == 0) {
        /* ---------------- loads: Q once, then the tiles, a box at a time as its slot comes free ----------------
         * One lane drives the copies.  After a tile's copies are on their way the whole warp asks L2 for the NEXT tile with
         * plain prefetches (a tile is 128 KB of consecutive memory: 1,024 lines, 32 a lane), so that the copies that refill the
         * ring later are trips to L2, not to memory — and cost the copy engine nothing, which a tensor prefetch would. */
        bool ok = true;
        const uint8_t* base = (const uint8_t*)P.latent;
        const uint64_t end = (uint64_t)P.length * (ML_D * 2);
        const uint64_t pol = l2_policy_evict_first();
        int last_t = nt > 0 ? 0 : -1, last_i = nt > 0 ? ML_BOXES - 1 : -1;   /* lane 0: the last box asked for (tile, box); tile 0 is on its way */
        for (int t = 0; t < nt; ++t) {
            if (lane == 0 && ok && t > 0)
                for (int i = 0; i < ML_BOXES; ++i) {
                    if (!mbar_wait(&empty[i], (t - 1) & 1, abort_flag, P.status)) { ok = false; break; }
                    mbar_expect_tx(&full[i], ML_BOX_BYTES);
                    tma_load_2d_hint(c_s + i * ML_BOX_BYTES, &cmap, &full[i], i * 64, (tile0 + t) * ML_BK, pol);
                    last_t = t; last_i = i;
                }
            __syncwarp();
            if (t + 1 < nt) {
                const uint64_t at = (uint64_t)(tile0 + t + 1) * (ML_BK * ML_D * 2);
#pragma unroll 4
                for (int i = 0; i < 32; ++i) {
                    const uint64_t off = at + ((uint64_t)(i * 32 + lane) << 7);
                    if (off < end) asm volatile("prefetch.global.L2 [%0];" ::"l"(base + off));
                }
            }
        }
        /* a wait gave up somewhere in the block: the copies already asked for get a bounded chance to land before the
         * block's memory is given back (a box's barrier has one phase a tile) */
        if (lane == 0 && *abort_flag != 0u) {
            for (int i = 0; i < ML_BOXES; ++i) {
                const int asked = i <= last_i ? last_t + 1 : last_t;         /* tiles whose box i has been asked for */
                if (asked > 0)
                    for (uint32_t k = 0; k < (1u << 16) && !mbar_try_wait(&full[i], (asked - 1) & 1); ++k) {}
            }
            if (nt > 0) for (uint32_t k = 0; k < (1u << 16) && !mbar_try_wait(q_full, 0); ++k) {}
        }
    } else if (warp == 1) {
        /* ---------------- every MMA: S^T(t) as the boxes land, then — the weights written — the four blocks of O^T ------- */
        if (lane == 0 && nt > 0) {
            constexpr uint32_t IDESC_S = idesc_f16(DT == SV_DTYPE_BF16, 0, ML_BK, NH);
            constexpr uint32_t IDESC_O = idesc_f16_a_mn(DT == SV_DTYPE_BF16, 0, 128, NH);
            const uint64_t qd = smem_desc_sw128(smem_u32(q_s), 16, 1024), cd = smem_desc_sw128(smem_u32(c_s), 16, 1024);
            const uint64_t ct = smem_desc_sw128(smem_u32(c_s), ML_BOX_BYTES, 1024);       /* the tile read transposed: 64-column groups a box apart */
            const uint64_t pd = smem_desc_sw128(smem_u32(p_s), 16, 1024);
            const uint32_t qd_lo = (uint32_t)qd, qd_hi = (uint32_t)(qd >> 32), cd_lo = (uint32_t)cd, cd_hi = (uint32_t)(cd >> 32);
            const uint32_t ct_lo = (uint32_t)ct, ct_hi = (uint32_t)(ct >> 32), pd_lo = (uint32_t)pd, pd_hi = (uint32_t)(pd >> 32);
            bool ok = mbar_wait(q_full, 0, abort_flag, P.status);
            for (int t = 0; ok && t < nt; ++t) {
                for (int i = 0; ok && i < ML_BOXES; ++i) {
                    if (!mbar_wait(&full[i], t & 1, abort_flag, P.status)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)            /* 16 latent columns a step: 32 bytes inside the box's 128-byte rows */
                        tc_mma_ss2(tmem + Cfg::T_S, cd_lo + i * (ML_BOX_BYTES >> 4) + kk * 2, cd_hi, qd_lo + i * (Cfg::Q_BOX_BYTES >> 4) + kk * 2, qd_hi,
                                   IDESC_S, (i > 0 || kk > 0) ? 1u : 0u);
                }
                if (!ok) break;
                tc_commit(s_full);
                /* the boxes whose columns another block of this share answers for are read by the score MMAs only: free now
                 * (this block's own boxes stay until its value MMAs have read them, so a tile's scores still cannot complete
                 * before the value products of the tile before it have) */
                for (int i = 0; i < ML_BOXES; ++i)
                    if (i < 2 * j0 || i >= 2 * j1) tc_commit(&empty[i]);
                if (!mbar_wait(p_full, t & 1, abort_flag, P.status)) break;
                tc_fence_after();
#pragma unroll 1
                for (int j = j0; j < j1; ++j) {
                    /* O^T block j: latent columns 128 j .. 128 j + 127 = boxes 2j and 2j + 1; sixteen keys a step = two 8-key groups */
#pragma unroll
                    for (int kk = 0; kk < ML_BK / 16; ++kk)
                        tc_mma_ss2(tmem + Cfg::T_O + j * NH, ct_lo + (2 * j) * (ML_BOX_BYTES >> 4) + kk * (2048 >> 4), ct_hi,
                                   pd_lo + (kk / 4) * (Cfg::P_BOX_BYTES >> 4) + (kk % 4) * 2, pd_hi, IDESC_O, (t > 0 || kk > 0) ? 1u : 0u);
                    tc_commit(&empty[2 * j]);
                    tc_commit(&empty[2 * j + 1]);
                }
                tc_commit(pv_done);
            }
        }
    } else {
        /* ---------------- softmax: a thread a key of the tile and 32 of the heads ---------------- */
        constexpr int SOFT = Cfg::SOFT;
        const int quad = warp & 3, half = (warp - 2) >> 2;           /* TMEM lane quadrant; which 32 heads */
        const int r = quad * 32 + lane;                              /* key within the tile = TMEM lane */
        const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
        const int st = (warp - 2) * 32 + lane;                       /* 0..SOFT-1 among the softmax threads */
        const int h0 = half * 32;
        float lpart[32];
#pragma unroll
        for (int x = 0; x < 32; ++x) lpart[x] = 0.f;
        /* The softmax warps meet at two block barriers a tile, so they walk the tiles together whatever happens: a warp whose
         * wait ran out goes on as a bystander (it keeps the barriers' count whole and touches nothing else). */
        bool alive = nt > 0;
        for (int t = 0; t < nt; ++t) {
            if (alive && !__all_sync(0xffffffffu, mbar_wait(s_full, t & 1, abort_flag, P.status))) alive = false;
            uint32_t sv[32];
            if (alive) {
                tc_fence_after();
                tmem_ld32(tmem + Cfg::T_S + h0 + lane_off, sv);
                tmem_wait_ld();
                tc_fence_before();
                const bool valid = (uint32_t)((tile0 + t) * ML_BK + r) < P.length;   /* rows past the end arrive as zeros: not scores */
                /* the tile's maximum a head: over the warp's 32 keys here, over the four quadrants through shared memory */
                /* (all 32 reductions are asked for before any answer is used: they pipeline, a dependent chain would not) */
                int mine = 0;
#pragma unroll
                for (int x = 0; x < 32; ++x) {
                    const float sc = valid ? __uint_as_float(sv[x]) * P.scale_log2 : -INFINITY;
                    sv[x] = __float_as_uint(sc);
                }
                int wm[32];
#pragma unroll
                for (int x = 0; x < 32; ++x) wm[x] = warp_max_s32(ordered_int(__uint_as_float(sv[x])));
#pragma unroll
                for (int x = 0; x < 32; ++x) mine = (x == lane) ? wm[x] : mine;
                wmax[quad * NH + h0 + lane] = ordered_float(mine);
            }
            softmax_bar<SOFT>();
            bool grew = false;
            if (st < NH) {
                const float mx = fmaxf(fmaxf(wmax[st], wmax[NH + st]), fmaxf(wmax[2 * NH + st], wmax[3 * NH + st]));
                const float old = mref[st];
                float f = 1.f;
                if ((mx > old + 8.f) || (old == -INFINITY && mx != -INFINITY)) { f = (old == -INFINITY) ? 0.f : fast_exp2(old - mx); mref[st] = mx; grew = true; }
                fac[st] = f;
            }
            const bool rescale = softmax_bar_or<SOFT>(grew);          /* any head's reference moved: the rare path below */
            if (!alive) continue;
            const int kb = r >> 6, kr = r & 63;
            uint8_t* prow = p_s + kb * Cfg::P_BOX_BYTES + (kr & 7) * 2;
            if (rescale) {
#pragma unroll
                for (int x = 0; x < 32; ++x) lpart[x] *= fac[h0 + x];
            }
            /* eight heads at a time, every stage of the eight before the next stage: loads, exponentials, roundings and stores
             * of different heads overlap instead of forming one chain a head (two warps a scheduler hide little on their own) */
            /* A head's row of P^T is 128 bytes whose 16-byte chunks are XORed with the row number mod 8: with c16 = chunk * 16,
             * row h's chunk sits at h * 128 + (c16 ^ ((h & 7) * 16)) — eight XORs serve all 32 rows. */
            const uint32_t c16 = (uint32_t)(kr >> 3) << 4;
            uint32_t cx[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) cx[u] = c16 ^ ((uint32_t)u << 4);
            /* (a head's reference is finite here: the first tile of a block has a key inside the range, and the reference
             * was brought up to date above)  Eight heads at a time, each stage of the eight before the next. */
#pragma unroll
            for (int x0 = 0; x0 < 32; x0 += 8) {
                float pv[8];
                const float4 m0 = *reinterpret_cast<const float4*>(mref + h0 + x0), m1 = *reinterpret_cast<const float4*>(mref + h0 + x0 + 4);
                const float mu[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
#pragma unroll
                for (int u = 0; u < 8; ++u) pv[u] = fast_exp2(__uint_as_float(sv[x0 + u]) - mu[u]);
                uint32_t w[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) w[u] = E::pack2(pv[2 * u], pv[2 * u + 1]);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float2 back = E::unpack2(w[u]);            /* the normaliser sums what the MMA will see */
                    lpart[x0 + 2 * u] += back.x;
                    lpart[x0 + 2 * u + 1] += back.y;
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {                        /* (h0 + x0 is a multiple of 8, so row h's low bits are 2u and 2u + 1) */
                    *reinterpret_cast<uint16_t*>(prow + (h0 + x0 + 2 * u) * 128 + cx[2 * u]) = (uint16_t)(w[u] & 0xFFFFu);
                    *reinterpret_cast<uint16_t*>(prow + (h0 + x0 + 2 * u + 1) * 128 + cx[2 * u + 1]) = (uint16_t)(w[u] >> 16);
                }
            }
            if (t > 0 && rescale) {
                /* s_full(t) is behind every box of tile t, and every box was refilled only after the value product of t - 1
                 * that read it had completed: O^T is settled.  A thread scales its lane (a latent column) and its 32 heads of
                 * the four blocks. */
#pragma unroll 1
                for (int j = j0; j < j1; ++j) {
                    uint32_t ov[32];
                    tmem_ld32(tmem + Cfg::T_O + j * NH + h0 + lane_off, ov);
                    tmem_wait_ld();
#pragma unroll
                    for (int x = 0; x < 32; ++x) ov[x] = __float_as_uint(__uint_as_float(ov[x]) * fac[h0 + x]);
                    tmem_st32(tmem + Cfg::T_O + j * NH + h0 + lane_off, ov);
                }
                tmem_wait_st();
            }
            fence_proxy_async_smem();                                /* the weights, for the MMA's reads */
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
        }
        /* ---- the block's (m, l, acc): the normaliser in a fixed order, O^T out of TMEM ---- */
        if (alive && !__all_sync(0xffffffffu, mbar_wait(pv_done, (nt - 1) & 1, abort_flag, P.status))) alive = false;
        tc_fence_after();
        /* the fold that follows is launched as a programmatic dependent: once every block has streamed its tiles it may be
         * scheduled — its launch then overlaps the blocks' write-out — and it waits, at its first instruction, for this grid to
         * have completed (a no-op when nothing of the kind follows) */
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        float* red = (float*)c_s;                                     /* [NH][129]: the ring is free now; a head's row is one word
                                                                         longer than its 128 shares so that the threads that sum
                                                                         different heads below read different banks */
        if (alive) {
#pragma unroll
            for (int x = 0; x < 32; ++x) red[(h0 + x) * 129 + r] = lpart[x];
        }
        softmax_bar<SOFT>();
        if (st < 2 * NH) {
            /* a head's 128 shares: two threads take 64 each, four running sums apiece (the order is fixed, the chain short) */
            const int h = st % NH, part = st / NH;
            const float* src = red + h * 129 + part * 64;
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
            for (int x = 0; x < 64; x += 4) { a0 += src[x]; a1 += src[x + 1]; a2 += src[x + 2]; a3 += src[x + 3]; }
            lhalf[part * NH + h] = (a0 + a1) + (a2 + a3);
        }
        softmax_bar<SOFT>();
        if (st < NH) lsum[st] = lhalf[st] + lhalf[NH + st];
        softmax_bar<SOFT>();
        if (alive) {
            const bool whole = P.blocks == 1u;
            float* out = whole ? P.res : P.partials + (size_t)share * NH * (ML_D + 2);
            bool hit = false;
            if (out && st < NH && j0 == 0) {                          /* every block of a share holds the same (m, l): the first writes them */ out[(size_t)st * (ML_D + 2)] = mref[st] * SV_LN2; out[(size_t)st * (ML_D + 2) + 1] = lsum[st]; }
#pragma unroll 1
            for (int j = j0; j < j1; ++j) {
                uint32_t ov[32];
                tmem_ld32(tmem + Cfg::T_O + j * NH + h0 + lane_off, ov);
                tmem_wait_ld();
                const int e = j * 128 + r;                            /* this lane's latent column */
#pragma unroll
                for (int x = 0; x < 32; ++x) {
                    const int h = h0 + x;
                    const float a = __uint_as_float(ov[x]);
                    if (out) out[(size_t)h * (ML_D + 2) + 2 + e] = a;
                    if (whole && P.o) P.o[(size_t)h * ML_D + e] = E::from_float(a / lsum[h], hit);
                }
            }
            if (hit && P.over) atomicOr(P.over, SV_FAULT_OVERFLOW);
            tc_fence_before();
        }
    }
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, Cfg::TMEM_COLS); }
}

/* The blocks' partial residuals folded in range order (attention_merge's arithmetic with the common maximum taken first,
 * so the order of the sums is fixed), then attention_finish: a block a head and a quarter of its columns. */
template <int DT>
__global__ void __launch_bounds__(128) mla_fold_kernel(uint16_t* o, float* res, const float* partials, uint32_t heads, uint32_t blocks, unsigned int* over) {
    using E = Elem<DT>;
    __shared__ float ms_s[160], ls_s[160], fs_s[160];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   /* a call behind this one may set up beside the fold; it reads nothing before its own wait */
    asm volatile("griddepcontrol.wait;" ::: "memory");          /* the partials are the grid ahead's */
    const uint32_t h = blockIdx.x / 4u, e = (blockIdx.x % 4u) * 128u + threadIdx.x, w = ML_D + 2;
    const size_t step = (size_t)heads * w;
    const float* base = partials + (size_t)h * w;
    /* a thread folds one element over the blocks in range order.  The first 32 blocks' accumulators are asked for before
     * anything else and the blocks' (m, l) right behind them, so that a short range costs ONE trip to memory; a long one
     * goes on 32 loads at a time (a trip's latency, not the bytes, is what a step of this loop costs) */
    constexpr uint32_t FB = 32u;
    float a[FB];
#pragma unroll
    for (uint32_t u = 0; u < FB; ++u) a[u] = (u < blocks) ? __ldcg(base + u * step + 2 + e) : 0.f;
    for (uint32_t s = threadIdx.x; s < blocks; s += 128u) { ms_s[s] = __ldcg(base + s * step); ls_s[s] = __ldcg(base + s * step + 1); }
    __syncthreads();
    float m = -INFINITY;
    for (uint32_t s = 0; s < blocks; ++s) m = fmaxf(m, ms_s[s]);
    /* a block's weight is the same for every element of the head: taken once, not once a thread */
    for (uint32_t s = threadIdx.x; s < blocks; s += 128u) fs_s[s] = ms_s[s] == -INFINITY ? 0.f : expf(ms_s[s] - m);
    __syncthreads();
    float acc = 0.f, l = 0.f;
    for (uint32_t s0 = 0; s0 < blocks; s0 += FB) {
        if (s0 != 0u) {
#pragma unroll
            for (uint32_t u = 0; u < FB; ++u) a[u] = (s0 + u < blocks) ? __ldcg(base + (s0 + u) * step + 2 + e) : 0.f;
        }
#pragma unroll
        for (uint32_t u = 0; u < FB; ++u) {
            if (s0 + u >= blocks || ms_s[s0 + u] == -INFINITY) continue;
            const float f = fs_s[s0 + u];
            acc = __fmaf_rn(a[u], f, acc);
            l = __fmaf_rn(ls_s[s0 + u], f, l);
        }
    }
    bool hit = false;
    if (res) { res[(size_t)h * w + 2 + e] = acc; if (e == 0) { res[(size_t)h * w] = m; res[(size_t)h * w + 1] = l; } }
    if (o) o[(size_t)h * ML_D + e] = E::from_float(acc / l, hit);
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* ---------------------------------------------------------------------------------------------------------------------- */

static std::mutex g_mla_lock;
static float* g_mla_partials[64];
static size_t g_mla_floats[64];

bool mla_decode_fits(const void* q, const void* latent, uint64_t heads, uint64_t head_dim, uint64_t length) {
    if (head_dim != ML_D || (heads != 32 && heads != 64)) return false;
    if (length == 0 || length > 0x7FFFFF00ull) return false;
    if (((uintptr_t)q | (uintptr_t)latent) & 15u) return false;
    return encode_tiled_fn() != nullptr;
}

template <int NH, int DT>
static cudaError_t launch_mla(uint16_t* o, float* res, const void* q, const void* latent, uint64_t length, uint32_t blocks_want, unsigned int* over, cudaStream_t st) {
    using Cfg = MlaCfg<NH>;
    const bool bf = DT == SV_DTYPE_BF16;
    CUtensorMap qm, cm;
    if (!make_map_2d_sw128(&qm, q, ML_D, NH, ML_D * 2, 64u, NH, bf)) return cudaErrorInvalidValue;
    if (!make_map_2d_sw128(&cm, latent, ML_D, length, ML_D * 2, 64u, ML_BK, bf)) return cudaErrorInvalidValue;
    MlaParams P;
    P.o = o; P.res = res; P.over = over; P.status = device_status_word(); P.latent = latent;
    P.length = (uint32_t)length; P.tiles = (uint32_t)((length + ML_BK - 1) / ML_BK);
    uint32_t blocks = blocks_want ? blocks_want : device_sm_count();
    if (blocks > P.tiles) blocks = P.tiles;
    if (blocks > 160u) blocks = 160u;                  /* the fold keeps the blocks' (m, l) in shared memory */
    P.blocks = blocks;
    /* A short range leaves most of the card idle, and a block's time is then its chain of one or two tiles: the value MMAs
     * and the write-out of the partial answer (which goes at the one SM's store rate) are a third of it.  Two or four blocks
     * a share, each with a half or a quarter of the answer's columns, cut both wherever every block still finds an SM of its
     * own; the scores and the softmax are then taken two or four times, on SMs that had nothing to do. */
    const uint32_t sms = device_sm_count();
    P.csplit = blocks * 4u <= sms ? 4u : (blocks * 2u <= sms ? 2u : 1u);
    P.scale_log2 = (1.0f / sqrtf((float)ML_D)) * SV_LOG2E;
    P.partials = nullptr;
    int d = 0;
    cudaError_t e = cudaGetDevice(&d);
    if (e != cudaSuccess) return e;
    if (d < 0 || d >= 64) return cudaErrorInvalidDevice;
    if (blocks > 1u) {
        std::lock_guard<std::mutex> hold(g_mla_lock);
        const size_t want = (size_t)device_sm_count() * 64 * (ML_D + 2);
        if (g_mla_floats[d] < want) {
            if ((e = cudaMalloc(&g_mla_partials[d], want * sizeof(float))) != cudaSuccess) return e;
            g_mla_floats[d] = want;
        }
        if ((size_t)blocks * NH * (ML_D + 2) > g_mla_floats[d]) return cudaErrorInvalidValue;
        P.partials = g_mla_partials[d];
    }
    static std::atomic<bool> attr_set[64];
    if (!attr_set[d].load(std::memory_order_acquire)) {
        if ((e = cudaFuncSetAttribute(mla_decode_kernel<NH, DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM)) != cudaSuccess) return e;
        attr_set[d].store(true, std::memory_order_release);
    }
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(blocks * P.csplit); cfg.blockDim = dim3(Cfg::THREADS); cfg.dynamicSmemBytes = Cfg::SMEM; cfg.stream = st;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at; cfg.numAttrs = pdl_allowed() ? 1u : 0u;
        if ((e = cudaLaunchKernelEx(&cfg, mla_decode_kernel<NH, DT>, qm, cm, P)) != cudaSuccess) return e;
    }
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    note_launch(1);
    if (blocks > 1u) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(NH * 4); cfg.blockDim = dim3(128); cfg.dynamicSmemBytes = 0; cfg.stream = st;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at; cfg.numAttrs = pdl_allowed() ? 1u : 0u;
        e = cudaLaunchKernelEx(&cfg, mla_fold_kernel<DT>, o, res, (const float*)P.partials, (uint32_t)NH, blocks, over);
        if (e != cudaSuccess) return e;
        note_launch(1);
        e = cudaGetLastError();
    }
    return e;
}

/* q [heads][512]; latent [length][512] (key and value); o [heads][512] 16-bit and/or res [heads][514] (m, l, acc).
 * blocks 0 = as many as the card has SMs (at most one a tile). */
cudaError_t mla_decode_launch(void* o, float* res, const void* q, const void* latent, uint64_t heads, uint64_t length, int dtype, uint32_t blocks,
                              unsigned int* over, cudaStream_t st) {
#define SV_ML(NN) (dtype == SV_DTYPE_BF16 ? launch_mla<NN, SV_DTYPE_BF16>((uint16_t*)o, res, q, latent, length, blocks, over, st) \
                                          : launch_mla<NN, SV_DTYPE_FP16>((uint16_t*)o, res, q, latent, length, blocks, over, st))
    if (heads == 64) return SV_ML(64);
    if (heads == 32) return SV_ML(32);
#undef SV_ML
    return cudaErrorInvalidValue;
}

}  // namespace sv
