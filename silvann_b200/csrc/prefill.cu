/* prefill.cu — causal grouped-query prefill attention on the 5th-generation tensor cores (tcgen05, TMEM), sm_100a.
 *
 * One kernel replaces the reference's three prompt doors — attention_causal_scores_grouped, attention_causal_softmax,
 * attention_causal_mix (engine/src/packages/nn/gpu/kernels/kernels.cuh:1028-1081, 2051-2060) — and never writes the
 * rows x (first + rows) fp32 weights buffer they pass between them.  Row r of the call is position first + r and attends
 * cache rows 0 .. first + r; query head h reads kv head h / (q_heads / kv_heads).
 *
 * A block owns 128 query rows of one head; 20 warps in five roles.
 *   warp 0      TMA: Q once (128 x head_dim, kept in shared memory for the whole block; asked for with the first K tile
 *               by the thread that initialises the barriers, ahead of the block's first barrier), then rings of K tiles and V
 *               tiles of 64 keys (128-byte swizzle; 3 + 2 stages at head_dim 256, 4 + 4 below).
 *   warp 1      one thread issues the score MMAs S = Q.K^T (M 128, N 64, K = head_dim in steps of 16, both operands in
 *               shared memory) into one of three (four below head_dim 256) score buffers in TMEM, so scores run tiles
 *               ahead of the softmax.  There are as many K stages as score buffers and the two rings turn together: a K
 *               stage's barrier takes two arrivals, the tile's bytes and the completion of the value MMAs that read the
 *               score buffer of the same index, so this thread has ONE wait and ONE commit a tile — and at head_dim 256
 *               the wait is not its own either (warp 3).
 *   warp 2      one thread issues the value MMAs O += P.V (M 128, N = head_dim, K 64; A from TMEM, B MN-major from
 *               shared memory) with O resident in TMEM for the whole row block.
 *   warp 3      the score thread's scout: takes that thread's mbarrier waits a tile ahead and hands them over on a
 *               hardware barrier (an mbarrier try costs the issuing thread 100-200 cycles while MMAs read their operands).
 *   warps 4-19  the online softmax, four warps a TMEM lane quadrant: a thread owns 16 of its row's 64 scores (read with
 *               tcgen05.ld); the four exchange their maxima, and at the end their sums, through spare TMEM columns and a
 *               hardware barrier.  The weights go back INTO TMEM, 16-bit, over the scores they came from (tcgen05.st), and
 *               are the A operand of the value MMA there: P never touches shared memory.  O is rescaled in TMEM only when
 *               a row's maximum has grown by more than 2^8 (the reference maximum is otherwise kept, which is exact:
 *               every weight and the normaliser are relative to the same reference).
 * Two issuing threads because the MMA queue is shallow: with one thread every wait for the softmax was a bubble in the
 * tensor pipe.  TMEM columns: O in [0, head_dim), score buffer b at head_dim + 64 b, then 8 columns for the softmax's
 * exchanges.  The epilogue divides by the row sum and rounds; the 16-bit rows are staged in the K ring (free by then, in the
 * swizzled box layout TMA reads) and leave as one TMA store a 64-column box — or (m ln 2, l, acc) a row is left in the
 * reference's residual layout (the many-row residual doors).
 *
 * Every mbarrier wait is bounded; a wait that runs out raises the block's abort flag, ORs "B2TO" into the device status
 * word, and the role goes on without touching anything else until the common exit, where TMEM is released.  The hardware
 * barriers have no bound of their own: the warps that meet at one go through it the same number of times whatever
 * happens.  No multicast, no cluster.
 *
 * Algorithmic flops: 4 · q_heads · head_dim · rows·(rows+1)/2 (+ first·rows terms) — QK^T and PV, 2 flop a MAC. */
#include "common.cuh"
#include <atomic>
#include "kernels.h"
#include "tensormap.cuh"
#include "tcgen05.cuh"

namespace sv {

static constexpr int PF_BM = 128;      /* query rows per block */
static constexpr int PF_BN = 64;       /* keys per tile */
static constexpr int PF_THREADS = 640; /* warp 0 TMA, warp 1 score MMAs, warp 2 value MMAs, warp 3 the score thread's scout, warps 4-19 softmax (four per TMEM lane quadrant) */

template <int D> struct PrefillCfg {
    static constexpr int BOXES = D / 64;
    static constexpr int Q_BYTES = PF_BM * D * 2;
    static constexpr int Q_BOX_BYTES = PF_BM * 128;
    static constexpr int KV_TILE_BYTES = PF_BN * D * 2;              /* one K or one V tile */
    static constexpr int KV_BOX_BYTES = PF_BN * 128;
    static constexpr int KST = (D >= 256) ? 3 : 4;                   /* K ring: scores run two tiles ahead of the values */
    static constexpr int VST = (D >= 256) ? 2 : 4;                   /* V ring */
    static constexpr int NSB = (D >= 256) ? 3 : 4;                   /* score buffers in TMEM: as many as K stages, so that the two rings turn together */
    /* TMEM columns: O [0, D) fp32, then NSB score buffers of PF_BN columns whose first PF_BN/2 columns are overwritten
     * in place by the 16-bit weights P */
    static constexpr int T_S = D;
    static constexpr int TMEM_COLS = (T_S + NSB * PF_BN <= 256) ? 256 : 512;
    static_assert(KST == NSB, "the K ring and the score buffers turn together");
    static constexpr int T_X = T_S + NSB * PF_BN;                    /* 8 columns (two tiles' worth of 4) through which a row's four softmax threads exchange maxima and sums */
    static_assert(T_X + 8 <= TMEM_COLS, "TMEM columns");
    static constexpr size_t SMEM = 1024 + Q_BYTES + (KST + VST) * KV_TILE_BYTES + 320 + 2 * PF_BM * 4;
};

struct PrefillParams {
    const uint16_t* q;        /* the queries themselves, for L2 prefetches (the loads go through the tensor map) */
    uint16_t* o;
    float* res;
    unsigned int* over;
    unsigned int* status;
    uint32_t q_heads, kv_heads, group;
    uint32_t first, rows, q_tiles;
    uint32_t ahead;           /* a block asks L2 for the queries of the block this many further on (the SM count) */
    float scale_log2;
};

template <int D, int DT>
__global__ void __launch_bounds__(PF_THREADS, 1)
prefill_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
               const __grid_constant__ CUtensorMap vmap, const __grid_constant__ CUtensorMap omap, const PrefillParams P) {
    using Cfg = PrefillCfg<D>;
    using E = Elem<DT>;
    constexpr int KST = Cfg::KST, VST = Cfg::VST, NSB = Cfg::NSB;
    constexpr bool SCOUT = D >= 256;         /* the score thread's waits are taken by another warp (see warp 1) */

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_s = smem;
    uint8_t* k_s = q_s + Cfg::Q_BYTES;
    uint8_t* v_s = k_s + KST * Cfg::KV_TILE_BYTES;
    uint64_t* bars = (uint64_t*)(v_s + VST * Cfg::KV_TILE_BYTES);
    uint64_t* k_full = bars;                 /* KST */
    uint64_t* v_full = k_full + KST;         /* VST */
    uint64_t* k_empty = v_full + VST;        /* KST: the S MMA that read the stage has completed */
    uint64_t* pv_done = k_empty + KST;       /* VST: the PV MMA of the stage's tile has completed (V stage free, O settled) */
    uint64_t* s_full = pv_done + VST;        /* NSB */
    uint64_t* p_full = s_full + NSB;         /* NSB */
    uint64_t* s_free = p_full + NSB;         /* NSB: the PV MMA that read the buffer's weights has completed */
    uint64_t* q_full = s_free + NSB;         /* 1 */
    uint64_t* o_staged = q_full + 1;           /* 1: the sixteen softmax warps have put their share of the output rows into shared memory */
    uint32_t* tmem_slot = (uint32_t*)(o_staged + 1);
    volatile uint32_t* abort_flag = (volatile uint32_t*)(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int qt = (int)P.q_tiles - 1 - (int)(blockIdx.x / P.q_heads);       /* heaviest row blocks first */
    const int h = blockIdx.x % P.q_heads, g = h / P.group;
    const int row0 = qt * PF_BM;
    const int keys_total = (int)(P.first + P.rows);
    int last_key = (int)P.first + row0 + PF_BM - 1;                          /* the last row's own position */
    if (last_key > keys_total - 1) last_key = keys_total - 1;
    const int nt = last_key / PF_BN + 1;                                     /* KV tiles this row block walks */

    if (tid == 0) {
        for (int s = 0; s < KST; ++s) { mbar_init(&k_full[s], KST == NSB ? 2 : 1); mbar_init(&k_empty[s], 1); }
        for (int s = 0; s < VST; ++s) { mbar_init(&v_full[s], 1); mbar_init(&pv_done[s], 1); }
        for (int b = 0; b < NSB; ++b) { mbar_init(&s_full[b], 1); mbar_init(&p_full[b], 16); mbar_init(&s_free[b], 1); }
        mbar_init(q_full, 1);
        mbar_init(o_staged, 16);
        *abort_flag = 0u;
        mbar_fence_init();
        /* Programmatic dependent launch (a no-op for a launch without the attribute): this block may have been scheduled
         * while the grid ahead of it on the stream was still running — its launch latency and this set-up are then off the
         * path — and nothing of that grid's may be read or overwritten before the wait below has returned.  Everything
         * else the block does follows from the copies asked for after it. */
        asm volatile("griddepcontrol.wait;" ::: "memory");
        /* Q and the first K tile are asked for here, ahead of the TMEM allocation and the block's first barrier: the
         * first score MMA waits for nothing else */
        tma_prefetch_desc(&qmap); tma_prefetch_desc(&kmap); tma_prefetch_desc(&vmap);
        mbar_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
        for (int c = 0; c < Cfg::BOXES; ++c) tma_load_2d(q_s + c * Cfg::Q_BOX_BYTES, &qmap, q_full, h * D + c * 64, row0);
        mbar_expect_tx(&k_full[0], Cfg::KV_TILE_BYTES);
        if (KST == NSB) mbar_arrive(&k_full[0]);
#pragma unroll
        for (int c = 0; c < Cfg::BOXES; ++c) tma_load_2d(k_s + c * Cfg::KV_BOX_BYTES, &kmap, &k_full[0], g * D + c * 64, 0);
    }
    if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    /* the launch behind this one on the stream may be scheduled once every block has got this far */
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t t_o = tmem, t_s0 = tmem + Cfg::T_S;

    if (warp == 0) {
        /* ---------------- TMA producer: a ring of K tiles and a ring of V tiles (Q and K(0) are on their way) ---------------- */
        {
            /* the whole warp asks L2 for the queries of a block that starts about when this one ends, so that its first
             * wait is a trip to L2 and not to memory: 128 rows of D elements, a row's share of this head contiguous */
            const uint32_t nb = blockIdx.x + P.ahead;
            if (P.ahead != 0u && nb < gridDim.x) {
                const int nrow0 = ((int)P.q_tiles - 1 - (int)(nb / P.q_heads)) * PF_BM, nh = (int)(nb % P.q_heads);
                constexpr int LINES = D * 2 / 128;                       /* 128-byte lines a row */
                for (int i = lane; i < PF_BM * LINES; i += 32) {
                    const int rr = nrow0 + i / LINES;
                    if (rr < (int)P.rows)
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(P.q + ((size_t)rr * P.q_heads + nh) * D + (i % LINES) * 64));
                }
            }
        }
        if (lane == 0) {
            /* K runs ahead of V by the depth of the score pipeline: K(j + KST - VST) is requested with V(j) */
            int jk = 1;
            auto load_k = [&]() -> bool {
                const int s = jk % KST, use = jk / KST;
                /* with as many K stages as score buffers the two rings turn together: the scores' own barrier says the stage is read */
                if (use > 0 && !mbar_wait(KST == NSB ? &s_full[s] : &k_empty[s], (use - 1) & 1, abort_flag, P.status)) return false;
                mbar_expect_tx(&k_full[s], Cfg::KV_TILE_BYTES);
                if (KST == NSB && jk < NSB) mbar_arrive(&k_full[s]);       /* no value MMA NSB tiles back to say that the score buffer is free */
#pragma unroll
                for (int c = 0; c < Cfg::BOXES; ++c)
                    tma_load_2d(k_s + s * Cfg::KV_TILE_BYTES + c * Cfg::KV_BOX_BYTES, &kmap, &k_full[s], g * D + c * 64, jk * PF_BN);
                ++jk;
                return true;
            };
            bool ok = true;
            int jv = 0;                                      /* value tiles asked for */
            while (ok && jk < KST - 1 && jk < nt) ok = load_k();
            for (int j = 0; ok && j < nt; ++j) {
                if (jk < nt && !load_k()) break;
                const int s = j % VST, use = j / VST;
                if (use > 0 && !mbar_wait(&pv_done[s], (use - 1) & 1, abort_flag, P.status)) break;
                mbar_expect_tx(&v_full[s], Cfg::KV_TILE_BYTES);
#pragma unroll
                for (int c = 0; c < Cfg::BOXES; ++c)
                    tma_load_2d(v_s + s * Cfg::KV_TILE_BYTES + c * Cfg::KV_BOX_BYTES, &vmap, &v_full[s], g * D + c * 64, j * PF_BN);
                jv = j + 1;
            }
            /* a wait gave up somewhere in the block: the copies already asked for get a bounded chance to land before the
             * block's memory is given back */
            if (*abort_flag != 0u) {
                for (int t = jk > KST ? jk - KST : 0; t < jk; ++t)
                    for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&k_full[t % KST], (t / KST) & 1); ++i) {}
                for (int t = jv > VST ? jv - VST : 0; t < jv; ++t)
                    for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&v_full[t % VST], (t / VST) & 1); ++i) {}
            }
        }
    } else if (warp == 1) {
        /* ---------------- score MMAs: S(j) = Q · K(j)^T ----------------
         * Two threads issue MMAs, this one the scores and one of warp 2 the values, because a thread that waits on an
         * mbarrier (about a hundred cycles even when the phase is long complete) feeds the tensor pipe nothing meanwhile
         * and the pipe's queue is short: with one issuer every wait is a bubble.  Scores run up to NSB tiles ahead; a
         * buffer is reused once the value MMA that read its weights has completed, which the K stage's barrier also waits
         * for (measured: each wait or commit taken off this thread's tile was worth 2-4 % of the whole kernel). */
        /* This thread's own waits are not on mbarriers at all.  Any access of its to shared memory — an mbarrier try, a plain load
         * — takes 100-200 cycles while the MMAs' operand reads own the port, and nothing is issued meanwhile.  The scout (warp 3)
         * takes the tile's mbarrier waits a tile ahead and says so on a hardware barrier (bar 1: the scout arrives, this warp
         * syncs); this warp says on bar 2 that it has taken the word, which lets the scout go on to the next tile.  A barrier's
         * generation is the scout's 32 threads and this warp's 32, and neither side can be two generations ahead of the other.
         * Should a wait of the scout's run out it still arrives, for every tile left, so that nothing here waits for ever: the
         * status word says "B2TO" and the block's answer is void. */
        constexpr uint32_t IDESC_S = idesc_f16(DT == SV_DTYPE_BF16, 0, PF_BM, PF_BN);
        /* descriptors of stage 0; a stage further is KV_TILE_BYTES >> 4 more in the start-address field */
        const uint64_t qd0 = smem_desc_sw128(smem_u32(q_s), 16, 1024), kd0 = smem_desc_sw128(smem_u32(k_s), 16, 1024);
        const uint32_t qd_lo = (uint32_t)qd0, qd_hi = (uint32_t)(qd0 >> 32), kd_lo = (uint32_t)kd0, kd_hi = (uint32_t)(kd0 >> 32);
        for (int j = 0; j < nt; ++j) {
            const int s = j % KST, b = j % NSB;
            if (SCOUT) {
                asm volatile("bar.sync 1, 64;" ::: "memory");
                asm volatile("bar.arrive 2, 64;" ::: "memory");
            } else if (lane == 0) {
                /* (below head_dim 256 the softmax, not this thread, paces the block, and the plain wait measured as fast) */
                if (j == 0) (void)mbar_wait(q_full, 0, abort_flag, P.status);
                (void)mbar_wait(&k_full[s], (j / KST) & 1, abort_flag, P.status);
            }
            if (lane == 0) {
                tc_fence_after();
                const uint32_t lo = kd_lo + (uint32_t)s * (Cfg::KV_TILE_BYTES >> 4), d_s = t_s0 + b * PF_BN;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk)      /* 16 columns a step: box kk/4, 32 bytes a step inside the 128-byte row */
                    tc_mma_ss2(d_s, qd_lo + (kk / 4) * (Cfg::Q_BOX_BYTES >> 4) + (kk % 4) * 2, qd_hi,
                               lo + (kk / 4) * (Cfg::KV_BOX_BYTES >> 4) + (kk % 4) * 2, kd_hi, IDESC_S, kk > 0 ? 1u : 0u);
                tc_commit(&s_full[b]);
            }
            __syncwarp();
        }
    } else if (warp == 3) {
        /* ---------------- the score thread's scout: Q, then a tile's K stage (its bytes, and the score buffer free) ---------------- */
        bool ok = true;
        if (SCOUT && lane == 0) ok = mbar_wait(q_full, 0, abort_flag, P.status);
        for (int j = 0; SCOUT && j < nt; ++j) {
            if (lane == 0 && ok) ok = mbar_wait(&k_full[j % KST], (j / KST) & 1, abort_flag, P.status);
            __syncwarp();
            asm volatile("bar.arrive 1, 64;" ::: "memory");
            asm volatile("bar.sync 2, 64;" ::: "memory");
        }
    } else if (warp == 2) {
        /* ---------------- value MMAs: O += P(j) · V(j), P read from TMEM in place over the scores ---------------- */
        if (lane == 0) {
            constexpr uint32_t IDESC_O = idesc_f16(DT == SV_DTYPE_BF16, 1, PF_BM, D);
            const uint64_t vd0 = smem_desc_sw128(smem_u32(v_s), Cfg::KV_BOX_BYTES, 1024);
            const uint32_t vd_lo = (uint32_t)vd0, vd_hi = (uint32_t)(vd0 >> 32);
            for (int j = 0; j < nt; ++j) {
                const int s = j % VST, b = j % NSB;
                if (!mbar_wait(&v_full[s], (j / VST) & 1, abort_flag, P.status)) break;
                if (!mbar_wait(&p_full[b], (j / NSB) & 1, abort_flag, P.status)) break;
                tc_fence_after();
                /* V is [key][value column]: MN-major for B; 64-column groups are a box apart (LBO), 8-key groups
                 * 1024 bytes apart (SBO); sixteen keys a step.  P: sixteen keys = 8 packed columns a step. */
                const uint32_t lo = vd_lo + (uint32_t)s * (Cfg::KV_TILE_BYTES >> 4), a_p = t_s0 + b * PF_BN;
#pragma unroll
                for (int kk = 0; kk < PF_BN / 16; ++kk)
                    tc_mma_ts2(t_o, a_p + kk * 8, lo + kk * (2048 >> 4), vd_hi, IDESC_O, (j > 0 || kk > 0) ? 1u : 0u);
                tc_commit(&pv_done[s]);
                /* the score buffer is free again.  With as many K stages as score buffers that is the second of the two arrivals the
                 * K stage's barrier waits for (tile j + NSB lands in stage b), so the score thread has ONE wait a tile */
                if (KST != NSB) tc_commit(&s_free[b]);
                else if (j + NSB < nt) tc_commit(&k_full[b]);
            }
        }
    } else {
        /* ---------------- softmax, correction, epilogue ----------------
         * Sixteen warps: a warp may touch only the 32 TMEM lanes of its quadrant (warp id mod 4), so four warps share each
         * quadrant and a thread owns 16 of its row's 64 scores.  The row maximum needs all 64: each thread leaves the
         * maximum of its 16 in a TMEM column of its own lane, the quadrant's four warps meet at a hardware barrier, and each
         * reads the four (neither shared memory nor an mbarrier is touched: both cost 100-200 cycles a visit while the
         * MMAs' operand reads own the shared-memory port).  The same barrier says that every warp has read its scores, so
         * the weights may go over them.  The exponentials are what bounds this role (sixteen a cycle an SM), and four warps
         * a scheduler keep that unit busy where two left it idle a third of the time.  A thread carries the normaliser of
         * its 16 columns and owns a quarter of O's columns when a rescale or the final store is due.
         * The quadrant's barrier is not bounded, so its four warps go through it together whatever happens: a warp whose
         * wait ran out walks the remaining tiles as a bystander, touching nothing but the barrier. */
        const int sw = warp - 4;                                    /* 0..15 */
        const int quad = warp & 3, part = sw >> 2;
        const int r = quad * 32 + lane;                             /* row within the block */
        const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
        const uint32_t t_x = tmem + Cfg::T_X + lane_off;
        const int grow_ = row0 + r;                                 /* row of the call */
        const int pos = (int)P.first + grow_;                       /* this row's position: keys 0..pos */
        const uint32_t qbar = 3u + (uint32_t)quad;                  /* bars 1 and 2 are the score thread's */
        constexpr int OC = D / 4;                                   /* O's columns a thread */
        constexpr int CH = OC >= 32 ? 32 : 16;                      /* ... read 32 (or 16) at a time */

        float m_ref = -INFINITY, l = 0.f;
        bool alive = true;
        for (int j = 0; j < nt; ++j) {
            const int b = j % NSB;
            /* the TMEM accesses below are warp-collective: the warp goes on together or stands by together */
            if (alive && !__all_sync(0xffffffffu, mbar_wait(&s_full[b], (j / NSB) & 1, abort_flag, P.status))) alive = false;
            uint32_t sv[16];
            if (alive) {
                tc_fence_after();
                tmem_ld16(t_s0 + b * PF_BN + part * 16 + lane_off, sv);
                tmem_wait_ld();
                const int key0 = j * PF_BN + part * 16;
                if (key0 + 15 > pos) {                              /* keys of this tile lie past the row's position */
#pragma unroll
                    for (int c = 0; c < 16; ++c) if (key0 + c > pos) sv[c] = 0xFF800000u;   /* -inf */
                }
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int c = 0; c < 16; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sv[c]));
                tmem_st1(t_x + (j & 1) * 4 + part, __float_as_uint(fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]))));
                tmem_wait_st();
                tc_fence_before();
            }
            asm volatile("bar.sync %0, 128;" ::"r"(qbar) : "memory");
            if (!alive) continue;
            tc_fence_after();
            uint32_t xm[4];
            tmem_ld4(t_x + (j & 1) * 4, xm);
            tmem_wait_ld();
            const float mx = fmaxf(fmaxf(__uint_as_float(xm[0]), __uint_as_float(xm[1])), fmaxf(__uint_as_float(xm[2]), __uint_as_float(xm[3]))) * P.scale_log2;
            /* keep the reference maximum unless this tile's exceeds it by more than 8 (weights then stay <= 2^8) */
            float f = 1.f;
            const bool grow = (mx > m_ref + 8.f) || (m_ref == -INFINITY && mx != -INFINITY);
            if (grow) { f = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - mx); m_ref = mx; }
            const float mu = (m_ref == -INFINITY) ? 0.f : m_ref;
            uint32_t pk[8];
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < 16; c += 2) {
                const float p0 = fast_exp2(fmaf(__uint_as_float(sv[c]), P.scale_log2, -mu));
                const float p1 = fast_exp2(fmaf(__uint_as_float(sv[c + 1]), P.scale_log2, -mu));
                const uint32_t w = E::pack2(p0, p1);
                const float2 back = E::unpack2(w);                  /* the normaliser sums what the MMA will see */
                sum4[(c >> 1) & 3] += back.x + back.y;
                pk[c >> 1] = w;
            }
            l = l * f + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));

            if (j > 0 && __any_sync(0xffffffffu, f != 1.f)) {
                /* O may be rescaled only between PV MMAs: the previous one must have completed, the next waits for us */
                if (!__all_sync(0xffffffffu, mbar_wait(&pv_done[(j - 1) % VST], ((j - 1) / VST) & 1, abort_flag, P.status))) { alive = false; continue; }
                tc_fence_after();
#pragma unroll 1
                for (int c0 = part * OC; c0 < (part + 1) * OC; c0 += CH) {      /* each warp of the four a quarter of O's columns */
                    uint32_t ov[CH];
                    if (CH == 32) tmem_ld32(t_o + c0 + lane_off, *reinterpret_cast<uint32_t(*)[32]>(ov)); else tmem_ld16(t_o + c0 + lane_off, *reinterpret_cast<uint32_t(*)[16]>(ov));
                    tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < CH; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * f);
                    if (CH == 32) tmem_st32(t_o + c0 + lane_off, *reinterpret_cast<uint32_t(*)[32]>(ov)); else tmem_st16(t_o + c0 + lane_off, *reinterpret_cast<uint32_t(*)[16]>(ov));
                }
                tmem_wait_st();
            }
            /* P over the scores, in place: 16 weights = 8 packed columns at this part's place (every warp of the quadrant has
             * read its scores: the barrier above) */
            tmem_st8(t_s0 + b * PF_BN + part * 8 + lane_off, pk);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[b]);
        }
        /* epilogue: the row's normaliser is the sum of its four parts' (through the same TMEM columns, in a fixed order);
         * O / l, rounded, to global — each warp of the four a quarter of the row */
        const bool fin = alive && __all_sync(0xffffffffu, mbar_wait(&pv_done[(nt - 1) % VST], ((nt - 1) / VST) & 1, abort_flag, P.status));
        if (fin) {
            tc_fence_after();
            tmem_st1(t_x + (nt & 1) * 4 + part, __float_as_uint(l));
            tmem_wait_st();
            tc_fence_before();
        }
        asm volatile("bar.sync %0, 128;" ::"r"(qbar) : "memory");
        if (fin) {
            tc_fence_after();
            uint32_t xl[4];
            tmem_ld4(t_x + (nt & 1) * 4, xl);
            tmem_wait_ld();
            const float l_row = (__uint_as_float(xl[0]) + __uint_as_float(xl[1])) + (__uint_as_float(xl[2]) + __uint_as_float(xl[3]));
            const float inv = 1.0f / l_row;
            bool hit = false;
            /* The 16-bit rows leave through shared memory and one TMA store a 64-column box: written straight from the
             * registers, a warp's store would touch 32 rows (32 lines for 512 bytes) and the block's 4,096 such line visits
             * took longer than three tiles of attention.  The K ring is free: every MMA has completed and every copy has
             * landed.  The boxes are laid out as TMA reads them (128-byte rows, the 16-byte piece index XOR the row's low
             * three bits), which also keeps the lanes of a warp, a row each, out of each other's banks. */
            uint8_t* stage = k_s;
            static_assert(Cfg::Q_BYTES <= KST * Cfg::KV_TILE_BYTES, "the staged output fits the K ring");
            /* the residual form of the answer: (m, l, acc) as attention_weights_rows + attention_residual_mix_rows leave
             * it — m is the reference the weights were taken against (natural-log units), acc is not divided */
            float* rrow = P.res ? P.res + ((size_t)grow_ * P.q_heads + h) * (D + 2) : nullptr;
            if (rrow && part == 0 && grow_ < (int)P.rows) { rrow[0] = m_ref * SV_LN2; rrow[1] = l_row; }
#pragma unroll 1
            for (int c0 = part * OC; c0 < (part + 1) * OC; c0 += CH) {
                uint32_t ov[CH];
                if (CH == 32) tmem_ld32(t_o + c0 + lane_off, *reinterpret_cast<uint32_t(*)[32]>(ov)); else tmem_ld16(t_o + c0 + lane_off, *reinterpret_cast<uint32_t(*)[16]>(ov));
                tmem_wait_ld();
                if (rrow && grow_ < (int)P.rows) {
#pragma unroll
                    for (int c = 0; c < CH; c += 2) *reinterpret_cast<float2*>(rrow + 2 + c0 + c) = make_float2(__uint_as_float(ov[c]), __uint_as_float(ov[c + 1]));
                }
                if (P.o && grow_ < (int)P.rows) {
                    /* rounded two at a time; the overflow rule (a finite value that lands on infinity) is looked at a value
                     * at a time only when the largest magnitude of the chunk says that it can have happened */
                    float top = 0.f;
#pragma unroll
                    for (int c = 0; c < CH; c += 8) {
                        uint32_t w[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const float x0 = __uint_as_float(ov[c + 2 * u]) * inv, x1 = __uint_as_float(ov[c + 2 * u + 1]) * inv;
                            top = fmaxf(top, fmaxf(fabsf(x0), fabsf(x1)));
                            w[u] = E::pack2(x0, x1);
                        }
                        *reinterpret_cast<uint4*>(stage + ((c0 + c) >> 6) * Cfg::Q_BOX_BYTES + r * 128 + (((((c0 + c) & 63) >> 3) ^ (r & 7)) << 4)) =
                            make_uint4(w[0], w[1], w[2], w[3]);
                    }
                    if (top >= E::over_from()) {
#pragma unroll
                        for (int c = 0; c < CH; ++c) (void)E::from_float(__uint_as_float(ov[c]) * inv, hit);
                    }
                }
            }
            if (hit && P.over) atomicOr(P.over, SV_FAULT_OVERFLOW);
            tc_fence_before();
            if (P.o) {
                tma_store_fence();
                __syncwarp();
                if (lane == 0) mbar_arrive(o_staged);
                /* one thread sends the boxes once all sixteen warps have staged theirs; rows past the call's end are cut off
                 * by the tensor map (they were not staged either) */
                if (sw == 0 && lane == 0 && mbar_wait(o_staged, 0, abort_flag, P.status)) {
#pragma unroll
                    for (int c = 0; c < Cfg::BOXES; ++c) tma_store_2d(&omap, stage + c * Cfg::Q_BOX_BYTES, h * D + c * 64, row0);
                    tma_store_commit_and_wait_read();
                }
            }
        }
    }

    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, Cfg::TMEM_COLS); }
}

/* ---------------------------------------------------------------------------------------------------------- */

bool prefill_fits(const PrefillCall& c) {
    if (c.head_dim != 64 && c.head_dim != 128 && c.head_dim != 256) return false;
    if (c.kv_heads == 0 || c.q_heads % c.kv_heads != 0) return false;
    if (((uintptr_t)c.q | (uintptr_t)c.k | (uintptr_t)c.v | (uintptr_t)c.o) & 15u) return false;
    if ((!c.o && !c.res) || ((uintptr_t)c.res & 7u)) return false;
    if (c.rows == 0 || c.first + c.rows > 0x7FFFFF00ull) return false;
    if ((uint64_t)((c.rows + PF_BM - 1) / PF_BM) * c.q_heads > 0x7FFFFFFFull) return false;
    return encode_tiled_fn() != nullptr;
}

template <int D, int DT>
static cudaError_t launch_prefill(const PrefillCall& c) {
    using Cfg = PrefillCfg<D>;
    const bool bf = DT == SV_DTYPE_BF16;
    CUtensorMap qm, km, vm, om;
    const uint64_t qcols = (uint64_t)c.q_heads * D, kcols = (uint64_t)c.kv_heads * D;
    if (!make_map_2d_sw128(&qm, c.q, qcols, c.rows, qcols * 2, 64u, PF_BM, bf)) return cudaErrorInvalidValue;
    if (!make_map_2d_sw128(&km, c.k, kcols, c.first + c.rows, kcols * 2, 64u, PF_BN, bf)) return cudaErrorInvalidValue;
    if (!make_map_2d_sw128(&vm, c.v, kcols, c.first + c.rows, kcols * 2, 64u, PF_BN, bf)) return cudaErrorInvalidValue;
    if (!c.o) om = qm;                                      /* not used then */
    else if (!make_map_2d_sw128(&om, c.o, qcols, c.rows, qcols * 2, 64u, PF_BM, bf)) return cudaErrorInvalidValue;
    PrefillParams P;
    P.q = (const uint16_t*)c.q; P.ahead = device_sm_count();
    P.o = (uint16_t*)c.o; P.res = c.res; P.over = c.over; P.status = device_status_word();
    P.q_heads = c.q_heads; P.kv_heads = c.kv_heads; P.group = c.q_heads / c.kv_heads;
    P.first = (uint32_t)c.first; P.rows = (uint32_t)c.rows; P.q_tiles = (uint32_t)((c.rows + PF_BM - 1) / PF_BM);
    P.scale_log2 = (1.0f / sqrtf((float)D)) * SV_LOG2E;
    static std::atomic<bool> attr_set[64];
    int d = 0; cudaGetDevice(&d);
    if (d >= 0 && d < 64 && !attr_set[d].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(prefill_kernel<D, DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM);
        if (e != cudaSuccess) return e;
        attr_set[d].store(true, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(P.q_tiles * c.q_heads); cfg.blockDim = dim3(PF_THREADS); cfg.dynamicSmemBytes = Cfg::SMEM; cfg.stream = c.stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = pdl_allowed() ? 1u : 0u;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, prefill_kernel<D, DT>, qm, km, vm, om, P);
    if (e != cudaSuccess) return e;
    note_launch(1);
    return cudaGetLastError();
}


cudaError_t prefill_launch(const PrefillCall& c) {
#define SV_PF(DD) (c.dtype == SV_DTYPE_BF16 ? launch_prefill<DD, SV_DTYPE_BF16>(c) : launch_prefill<DD, SV_DTYPE_FP16>(c))
    if (c.head_dim == 64) return SV_PF(64);
    if (c.head_dim == 128) return SV_PF(128);
    if (c.head_dim == 256) return SV_PF(256);
#undef SV_PF
    return cudaErrorInvalidValue;
}

}  // namespace sv
