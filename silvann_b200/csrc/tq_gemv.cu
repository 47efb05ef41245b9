/* tq_gemv.cu — a TurboQuant-coded matrix times up to eight 16-bit vectors, HBM-bound: the weight path of a decode step.
 *
 * The reference's door (engine/src/packages/nn/gpu/kernels/kernels.cuh:1405-1447; groups :1453-1461; n inputs :1462-1472)
 * is out[r] = half(scale_r · sum_c level(code[r][c]) · x[c]) and its own note calls its body "the reference shape, not the
 * fast one": a family answers it with a kernel of its own.  A decode step reads every weight once, so the door is bound
 * by the bytes of the codes: cols·d/8 a row.  What stands between the codes and that bound is the expansion: a level is a
 * table entry, and a table lookup is one shared-memory load a BYTE of codes whatever the width (at 4 bits the table holds
 * both nibbles' levels as a pair of halves), 32 lookups a clock an SM.  Everything else is arranged to cost nothing next
 * to it:
 *   · the products and sums run on the tensor cores (mma.sync m16n8k16, fp16 levels × fp16 x, fp32 accumulate): the levels
 *     never pass through fp32 registers, and the eight columns of the B operand are eight INPUT VECTORS — the groups-over-
 *     n-inputs door reads a matrix once for all of them;
 *   · a sum does not care about its order, so the MMA's k index is permuted to follow the bytes as they lie: lane (g, t)
 *     of a warp takes 16 neighbouring bytes of rows g and g + 8 as its A fragments; the matching x values sit in registers
 *     as B fragments for the whole kernel;
 *   · the codes come through a ring of shared-memory stages filled by bulk copies (a row a copy, rows 64 bytes further apart
 *     than they are long, so the 16-byte reads of a quarter-warp never share a bank) that complete on mbarriers: loads held
 *     in registers serialised on the few register scoreboards (a wait for an old load waited for the newest too), copies
 *     by the async proxy do not;
 *   · the table is 256 bytes an entry — 32 copies of the 4-bit pair table, then 32 of the 8-bit table, one a bank — so a
 *     lookup never conflicts and its offset is ONE byte-permute of the code word;
 *   · a block is sixteen working warps that split a row's bytes 64 at a time, and a seventeenth that only fetches (a copy's
 *     issue waits until the memory system takes it: a warp that both fetched and worked held the whole block up at the
 *     next barrier).  A block walks a run of neighbouring tiles of 16 rows in steps of up to four; the working warps'
 *     partial sums of a step meet in shared memory, double-buffered, one barrier a step.
 * Shapes it takes: widths 4 and 8, row bytes a multiple of 64 and at most 4,096 (a row longer than 2,048 bytes goes through
 * the ring in two halves), codes 16-byte aligned, at most 8 inputs.  Anything else stays with the as-worded kernel in
 * tq.cu.  Every mbarrier wait is bounded; one that runs out ORs "B2TO" into the device's status word and the block leaves.
 *
 * Where the time goes (16,384 x 4,096 at 4 bits, 33.6 MB, 16.8 us a call: 2.0 TB/s): a block has a run of seven tiles; a
 * working warp spends 1,790 cycles on a tile's two pieces against the 1,280 the shared-memory pipe needs for the tile's 1,024
 * lookups and 256 fetch wavefronts, after 2.7 us of prologue and first landing (every SM's first three slots, 14 MB over the
 * card, are asked for at once). */
#include "common.cuh"
#include "exchange.cuh"
#include <atomic>
#include "kernels.h"
#include <string.h>

namespace sv {

using H = Elem<SV_DTYPE_FP16>;

static __device__ const uint16_t g_tq_levels_gemv[318] = {
#include "tq_levels.inc"
};

constexpr int GV_WARPS = 16, GV_THREADS = GV_WARPS * 32, GV_LUT_BYTES = 256 * 256;

constexpr int GV_STAGES_MAX = 4, GV_ROW_PAD = 64, GV_TS_MAX = 4;       /* slots of the ring at most; a row's padding; tiles a step at most */

/* The table as a block holds it (256 entries of 256 bytes: 32 copies of the 4-bit pair, then 32 of the 8-bit level twice),
 * made once a device and copied into every block by one bulk copy instead of being built again by each. */
__device__ uint4 g_gv_lut_image[GV_LUT_BYTES / 16];
__global__ void __launch_bounds__(256) gv_lut_image_kernel() {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < 256 * 16; i += gridDim.x * blockDim.x) {
        const int b = i >> 4, q = i & 15;
        const uint32_t l8 = g_tq_levels_gemv[62 + b];
        const uint32_t e = q < 8 ? ((uint32_t)g_tq_levels_gemv[14 + (b & 15)] | ((uint32_t)g_tq_levels_gemv[14 + (b >> 4)] << 16)) : (l8 | (l8 << 16));
        g_gv_lut_image[i] = make_uint4(e, e, e, e);
    }
}

cudaError_t tq_gemv_fast_launch(uint16_t* out, const void* groups, const uint64_t* rows_cap, const uint16_t* x, uint64_t cols, uint64_t inputs,
                                uint64_t out_stride, unsigned int* over, cudaStream_t st, const XfParams* xf);

struct GemvFast {
    const uint8_t* codes[12];
    const uint16_t* scales[12];
    uint32_t rows[12], d[12], halves[12], tile0[13];   /* group i's tiles of 16 rows are [tile0[i], tile0[i+1]); halves: slots a tile */
    uint64_t out_at[12];
    uint32_t count, cols, inputs, x_wide;      /* x_wide: x may be read 16 bytes at a time */
    uint32_t ts, pi, stage_bytes, smem_bytes;  /* tiles a step at most; inputs rounded up to a power of two; bytes a slot; the block's shared memory */
    uint64_t out_stride;
    unsigned int* status;
    /* with an exchange (xf.members > 0; one group, one input): the rounded answers are pushed to the members' slots instead
     * of `out`, and the block then adds every member's answers of its own rows in member order (exchange.cuh) */
    XfParams xf;
};

/* The table entry of byte `idx` of word `w` for this lane.  The table starts on a 64 KB boundary of the shared window and
 * an entry is 256 bytes, so the address is ONE byte-permute: bytes 3, 2 and 0 of `lane_at` (the table's base, and this
 * lane's bank within an entry) around the code byte. */
__device__ __forceinline__ uint32_t gv_lut(uint32_t lane_at, uint32_t w, int idx) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(__byte_perm(w, lane_at, 0x7604u | ((uint32_t)idx << 4))));
    return v;
}
__device__ __forceinline__ uint4 gv_lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
/* `bytes` (a multiple of 16) from global to shared, both 16-byte aligned, completion counted on `bar` */
__device__ __forceinline__ void gv_bulk(uint32_t dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy) : "memory");
}

/* m16n8k16, fp16 operands, fp32 sums; not volatile, so that the compiler may move it among the lookups around it */
__device__ __forceinline__ void gv_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

/* One 64-byte piece of rows g and g + 8 through the table and the tensor cores: 8 MMAs at 4 bits (bytes 2m, 2m+1 are four
 * codes a row), 4 at 8 bits (bytes 4m .. 4m+3), alternating between two accumulators so that an MMA does not wait for the
 * one before it.  The sixteen lookups of half a piece are all asked for before the first MMA that needs one: a lookup is a
 * shared-memory round trip, and four at a time (an MMA's worth) left the warp waiting for each. */
__device__ __forceinline__ void gv_piece(float (&c0)[4], float (&c1)[4], const uint4& wa, const uint4& wb, const uint32_t* xr, uint32_t d, uint32_t at4,
                                         uint32_t at8) {
    const uint32_t wsa[4] = {wa.x, wa.y, wa.z, wa.w}, wsb[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        uint32_t la[8], lb[8];                                               /* the eight bytes of this half of row g, of row g + 8 */
        if (d == 4) {
#pragma unroll
            for (int b = 0; b < 8; ++b) { la[b] = gv_lut(at4, wsa[half * 2 + (b >> 2)], b & 3); lb[b] = gv_lut(at4, wsb[half * 2 + (b >> 2)], b & 3); }
#pragma unroll
            for (int m = 0; m < 4; ++m)                                      /* bytes 2m, 2m + 1 of the half */
                gv_mma((m & 1) ? c1 : c0, la[2 * m], lb[2 * m], la[2 * m + 1], lb[2 * m + 1], xr[half * 8 + 2 * m], xr[half * 8 + 2 * m + 1]);
        } else {
#pragma unroll
            for (int b = 0; b < 8; ++b) { la[b] = gv_lut(at8, wsa[half * 2 + (b >> 2)], b & 3); lb[b] = gv_lut(at8, wsb[half * 2 + (b >> 2)], b & 3); }
#pragma unroll
            for (int m = 0; m < 2; ++m)                                      /* bytes 4m .. 4m + 3 of the half */
                gv_mma((m & 1) ? c1 : c0, __byte_perm(la[4 * m], la[4 * m + 1], 0x5410), __byte_perm(lb[4 * m], lb[4 * m + 1], 0x5410),
                                        __byte_perm(la[4 * m + 2], la[4 * m + 3], 0x5410), __byte_perm(lb[4 * m + 2], lb[4 * m + 3], 0x5410),
                                        xr[half * 4 + 2 * m], xr[half * 4 + 2 * m + 1]);
        }
    }
}

/* NIW: the 64-byte pieces of a row one warp owns at most (pieces warp, warp + 16, ...); x registers a thread: 16·NIW.
 * W: the one width of every group (4 or 8), so that the other width's code is not in the loop at all; 0: groups of both.
 *
 * Sixteen warps work the codes and a seventeenth only fetches: a copy's issue waits for the memory system to take it, and
 * a warp that both fetched and worked made the whole block wait for that at the next barrier.  The ring's slots are
 * handed back and forth on mbarriers (`full`: the copies' bytes; `empty`: one arrival a working warp).
 * A block takes a run of neighbouring tiles of 16 rows (every block as many, to within one) and walks it in steps of up to
 * `ts` tiles: a tile is one slot of the ring — two, a half row each, where 16 whole rows are more than a slot holds — and
 * the working warps meet ONCE a step, when their partial sums of the step's tiles are written (the sums are kept for as
 * many inputs as there are, rounded up to a power of two, so that a decode step's take little room and are kept twice). */
template <int NIW, int W>
__global__ void __launch_bounds__(GV_THREADS + 32, 1) tq_gemv_fast_kernel(uint16_t* out, GemvFast a, const uint16_t* x, unsigned int* over) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint32_t stage_at_s[GV_STAGES_MAX];
    __shared__ uint32_t stages_s;
    /* The table sits on the first 64 KB boundary of the shared window inside this block's memory; the partial sums, the
     * barriers and the ring's slots are carved from what lies before it and after it. */
    const uint32_t ts = a.ts, pi = a.pi;
    const uint32_t base = smem_u32(smem), lut = (base + 0xFFFFu) & ~0xFFFFu, end = base + a.smem_bytes;
    const uint32_t tile_floats = GV_WARPS * 16u * pi;                        /* a tile's partial sums: [warp][row][input] */
    const uint32_t part_bytes = 2u * ts * tile_floats * (uint32_t)sizeof(float), small = part_bytes + 128u;
    uint32_t before = base, after = lut + (uint32_t)GV_LUT_BYTES;            /* the next free byte either side */
    uint32_t part_at;
    if (lut - before >= small) { part_at = before; before += small; } else { part_at = after; after += small; }
    float* part = reinterpret_cast<float*>(smem + (part_at - base));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + (part_at - base) + part_bytes);
    uint64_t* empty = full + GV_STAGES_MAX;
    uint64_t* table_bar = empty + GV_STAGES_MAX;
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(table_bar + 1);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    if (tid == 0) {
        uint32_t n = 0;
        for (; n < (uint32_t)GV_STAGES_MAX && before + a.stage_bytes <= lut; ++n, before += a.stage_bytes) stage_at_s[n] = before;
        for (; n < (uint32_t)GV_STAGES_MAX && after + a.stage_bytes <= end; ++n, after += a.stage_bytes) stage_at_s[n] = after;
        stages_s = n;
        for (uint32_t st = 0; st < (uint32_t)GV_STAGES_MAX; ++st) { mbar_init(&full[st], 1); mbar_init(&empty[st], GV_WARPS); }
        mbar_init(table_bar, 1);
        *abort_flag = 0u;
        mbar_fence_init();
    }
    __syncthreads();
    /* Programmatic dependent launch (no-ops for a launch without the attribute).  A decode step is a run of these calls
     * back to back, each taking the answer of a kernel before it as its input: the launch behind this one may be scheduled
     * as soon as every block has got this far, and a block scheduled early may stream its CODES and build its table at
     * once — a layer's coded weights are not what the grid ahead writes — while everything that touches the input vector
     * or the answers comes after the wait the working warps take below. */
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t S = stages_s;
    if (S < 2) return;                                                       /* the launcher sized the block's memory so that two fit */
    /* this block's run of tiles: every block as many, to within one */
    const uint32_t tiles = a.tile0[a.count];
    const uint32_t run_lo = (uint32_t)(((uint64_t)blockIdx.x * tiles) / gridDim.x), run_hi = (uint32_t)(((uint64_t)(blockIdx.x + 1) * tiles) / gridDim.x);

    if (warp == GV_WARPS) {
        /* ---- the fetching warp: the table, then slot after slot as the working warps hand them back ---- */
        const uint64_t policy = l2_policy_evict_first();
        uint32_t m = 0;                                                      /* slots filled so far */
        int gi = -1;
        uint32_t hi = 0, lo = 0, row_bytes = 0, rows = 0, halves = 1, seg = 0;
        const uint8_t* codes = nullptr;
        for (uint32_t tile = run_lo; tile < run_hi; ++tile) {
            while (tile >= hi) {                                             /* a group's numbers are read once, as its first tile comes */
                ++gi; lo = a.tile0[gi]; hi = a.tile0[gi + 1];
                row_bytes = a.cols * a.d[gi] / 8u; rows = a.rows[gi]; halves = a.halves[gi]; seg = row_bytes / halves; codes = a.codes[gi];
            }
            const uint32_t row0 = (tile - lo) * 16u, there = min(16u, rows - row0);
            for (uint32_t h = 0; h < halves; ++h, ++m) {
                const uint32_t slot = m % S;
                if (m >= S && !mbar_wait(&empty[slot], ((m / S) - 1u) & 1u, abort_flag, a.status)) { tile = run_hi; break; }
                if (lane == 0) mbar_expect_tx(&full[slot], there * seg);
                __syncwarp();
                const uint32_t dst = stage_at_s[slot];
                for (uint32_t r = (uint32_t)lane; r < there; r += 32u)
                    gv_bulk(dst + r * (seg + GV_ROW_PAD), codes + (size_t)(row0 + r) * row_bytes + (size_t)h * seg, seg, &full[slot], policy);
            }
        }
        return;                                                              /* nothing after this point waits for the fetching warp */
    }

    /* ---- the sixteen working warps ----
     * They make the table themselves while the first slots are on their way: eight 16-byte stores a thread, where a copy of
     * the 64 KB image would take the block's first 1,150 cycles of copy-in (copies enter an SM at about 57 B/clk) ahead of
     * the codes that the work waits for. */
    {
        static_assert(256 * 16 % GV_THREADS == 0, "a whole number of entries' pieces a thread");
        constexpr int PER = 256 * 16 / GV_THREADS;
        uint32_t e[PER];
#pragma unroll
        for (int k = 0; k < PER; ++k) {                                      /* the levels first, all asked for at once */
            const uint32_t i = (uint32_t)tid + (uint32_t)k * GV_THREADS, b = i >> 4, q = i & 15u;
            const uint32_t lo16 = g_tq_levels_gemv[q < 8u ? 14u + (b & 15u) : 62u + b], hi16 = g_tq_levels_gemv[q < 8u ? 14u + (b >> 4) : 62u + b];
            e[k] = lo16 | (hi16 << 16);
        }
#pragma unroll
        for (int k = 0; k < PER; ++k)
            asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(lut + ((uint32_t)tid + (uint32_t)k * GV_THREADS) * 16u), "r"(e[k]) : "memory");
    }
    asm volatile("bar.sync 1, %0;" ::"n"(GV_THREADS) : "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");                      /* the input vector may be the work of the grid ahead */
    const uint32_t at4 = lut | ((uint32_t)lane * 4u), at8 = at4 + 128u;     /* the 4-bit pair table, then the 8-bit one, in every entry */
    uint32_t xr[NIW][16];                                                    /* this lane's B fragments: input g, the columns of its bytes */
    uint32_t have_d = 0, n = 0, m = 0;
    bool failed = false;
    int buf = 0;
    bool hit = false;
    int gi = -1;
    uint32_t lo = 0, hi = 0, d = 0, rows = 0, row_bytes = 0, halves = 1, seg = 0, pieces = 0;
    const uint16_t* sc = nullptr;
    uint64_t out_row = 0, out_input = 0;                                     /* an answer's place: out_row + row + input · out_input */
    for (uint32_t tile = run_lo; tile < run_hi; ++n, buf ^= 1) {
        while (tile >= hi) {                                                 /* a group's numbers are read once, as its first tile comes */
            ++gi; lo = a.tile0[gi]; hi = a.tile0[gi + 1];
            d = W != 0 ? (uint32_t)W : a.d[gi]; rows = a.rows[gi]; row_bytes = a.cols * d / 8u; halves = a.halves[gi]; seg = row_bytes / halves; pieces = row_bytes / 64u;
            sc = a.scales[gi];
            out_row = a.out_at[gi]; out_input = a.out_stride != 0 ? a.out_stride : (uint64_t)rows;
        }
        const uint32_t nt = min(ts, min(hi, run_hi) - tile);                 /* the tiles of this step: of one group, of this block's run */
        const uint32_t row0 = (tile - lo) * 16u;
        const uint32_t per_lane = (W != 0 ? (uint32_t)W : d) == 4 ? 32u : 16u;       /* columns a lane's 16 bytes hold */
        if (d != have_d) {                                                   /* the columns a lane owns depend on the width */
            have_d = d;
#pragma unroll
            for (int i = 0; i < NIW; ++i) {
                const uint32_t piece = (uint32_t)warp + (uint32_t)i * GV_WARPS;
                const uint32_t c0 = piece * (64u * 8u / d) + (uint32_t)t * per_lane;
                const bool live = piece < pieces && (uint32_t)g < a.inputs;
                const uint16_t* src = x + (size_t)g * a.cols + c0;
#pragma unroll
                for (int e = 0; e < 16; e += 4) {
                    uint4 v = make_uint4(0, 0, 0, 0);
                    if (live && (uint32_t)e * 2u < per_lane) {
                        if (a.x_wide) v = *reinterpret_cast<const uint4*>(src + e * 2);
                        else { const uint32_t* p = reinterpret_cast<const uint32_t*>(src + e * 2); v = make_uint4(p[0], p[1], p[2], p[3]); }
                    }
                    xr[i][e] = v.x; xr[i][e + 1] = v.y; xr[i][e + 2] = v.z; xr[i][e + 3] = v.w;
                }
            }
        }
        /* the answer this thread will write after the step's barrier: tile o / (16·pi), row (o / pi) % 16, input o % pi; its
         * row's scale is on its way while the step is worked */
        const uint32_t o = (uint32_t)tid, o_tile = o / (16u * pi), o_row = row0 + o_tile * 16u + (o / pi) % 16u, o_in = o % pi;
        const bool o_live = o_tile < nt && o_row < rows && o_in < a.inputs;
        uint16_t scale = 0;
        if (o_live) asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(scale) : "l"(sc + o_row));
        float* mine = part + (size_t)buf * ts * tile_floats + (size_t)warp * 16u * pi;
        for (uint32_t tq = 0; tq < nt; ++tq) {
            float c[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
            for (uint32_t h = 0; h < halves; ++h, ++m) {
                const uint32_t slot = m % S;
                bool landed = failed ? false : mbar_wait(&full[slot], (m / S) & 1u, abort_flag, a.status);
                if (!landed) { failed = true; continue; }                    /* said at the step's barrier: every warp leaves there, or none */
                const uint32_t stride = seg + GV_ROW_PAD, at_a = stage_at_s[slot] + (uint32_t)t * 16u + (uint32_t)g * stride, at_b = at_a + 8u * stride;
#pragma unroll
                for (int i = 0; i < NIW; ++i) {
                    const uint32_t piece = (uint32_t)warp + (uint32_t)i * GV_WARPS;
                    if (piece >= pieces || (piece * 64u) / seg != h) continue;                       /* the whole warp together */
                    const uint32_t off = piece * 64u - h * seg;
                    const uint4 ua = gv_lds128(at_a + off), ub = gv_lds128(at_b + off);
                    gv_piece(c, c1, ua, ub, xr[i], W != 0 ? (uint32_t)W : d, at4, at8);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[slot]);                    /* this warp has read the slot */
            }
            /* c0, c1: (row g, inputs 2t, 2t+1) · c2, c3: (row g + 8, the same inputs): kept for the inputs there are */
            float* to = mine + (size_t)tq * tile_floats;
            if (2u * (uint32_t)t < pi) {
                to[(uint32_t)g * pi + 2u * t] = c[0] + c1[0];
                to[((uint32_t)g + 8u) * pi + 2u * t] = c[2] + c1[2];
                if (pi > 1u) { to[(uint32_t)g * pi + 2u * t + 1u] = c[1] + c1[1]; to[((uint32_t)g + 8u) * pi + 2u * t + 1u] = c[3] + c1[3]; }
            }
        }
        {   /* the working warps' partial sums are whole; and a vote: a warp whose wait gave up takes every warp out */
            uint32_t any;
            asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbarrier.cta.red.or.pred p, 1, 512, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(any) : "r"(failed ? 1u : 0u) : "memory");
            if (any) { failed = true; break; }
        }
        if (o_live) {                                                        /* sixteen warps' parts of one answer, in warp order */
            const float* from = part + (size_t)buf * ts * tile_floats + (size_t)o_tile * tile_floats + ((o / pi) % 16u) * pi + o_in;
            float sum = 0.f;
#pragma unroll
            for (uint32_t w = 0; w < (uint32_t)GV_WARPS; ++w) sum += from[w * 16u * pi];
            const uint16_t y = H::from_float(sum * H::to_float(scale), hit);
            if (a.xf.members == 0u) out[out_row + o_row + o_in * out_input] = y;
            else
                for (uint32_t mm = 0; mm < a.xf.members; ++mm)                   /* this card's partial of the row, to every member: a tagged word */
                    xf_store(xf_slot(a.xf.peer[mm], a.xf.gen & 1u, a.xf.index, a.xf.slot_words, a.xf.members) + o_row, (uint32_t)y, a.xf.gen);
        }
        tile += nt;
    }
    /* After a wait gave up, copies may still be on their way into this block's memory: the first working thread waits
     * (bounded) for every slot's barrier to settle before the memory is given back. */
    if (failed && tid == 0)
        for (uint32_t st = 0; st < S; ++st) for (uint32_t i = 0; i < 4096u && !mbar_try_wait(&full[st], 0u) && !mbar_try_wait(&full[st], 1u); ++i) { }
    if (a.xf.members != 0u) {
        /* ---- the exchange: the block's rows are on their way to every member; take the members' same rows as they come ----
         * Every member runs this kernel over a matrix of the same shape, so block b owns the same rows everywhere: no block
         * waits for another block of its own card.  A row is one tagged word, so nothing is fenced or flagged: a thread
         * polls (bounded) the words of the row it adds. */
        const uint32_t parity = a.xf.gen & 1u;
        if (!failed) {
            const uint32_t r_lo = run_lo * 16u, r_hi = min(run_hi * 16u, a.rows[0]);
            unsigned long long t0 = 0ull;
            bool ok = true;
            for (uint32_t r = r_lo + (uint32_t)tid; r < r_hi; r += GV_THREADS) {
                uint32_t part16[XF_MEMBERS_MAX];
                xf_gather(a.xf, parity, r, part16, t0, ok);
                if (!ok) { if (a.status) atomicOr(a.status, SV_STATUS_TIMEOUT); break; }
                float sum = 0.f;
#pragma unroll
                for (uint32_t mm = 0; mm < XF_MEMBERS_MAX; ++mm)
                    if (mm < a.xf.members) sum += H::to_float((uint16_t)part16[mm]);
                out[a.out_at[0] + r] = H::from_float(sum, hit);
            }
        }
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* Whether the fast kernel takes these groups; `rows_cap` trims a single group to the rows its rooms hold. */
bool tq_gemv_fast_fits(const void* groups, uint64_t cols, uint64_t inputs) {
    struct G { uint64_t codes[12], luts[12], rows[12], d[12], out_at[12], count; } g;
    memcpy(&g, groups, sizeof g);
    if (g.count == 0 || g.count > 12 || inputs == 0 || inputs > 8 || cols == 0 || cols > 8192) return false;
    for (uint64_t i = 0; i < g.count; ++i) {
        if (g.d[i] != 4 && g.d[i] != 8) return false;
        if ((cols * g.d[i] / 8) % 64 != 0 || cols * g.d[i] % 8 != 0 || cols * g.d[i] / 8 > 4096) return false;
        if (g.codes[i] % 16 != 0 || g.luts[i] % 2 != 0 || g.rows[i] > 0x0fffffffu) return false;
    }
    return true;
}

cudaError_t tq_gemv_fast_launch(uint16_t* out, const void* groups, const uint64_t* rows_cap, const uint16_t* x, uint64_t cols, uint64_t inputs,
                                uint64_t out_stride, unsigned int* over, cudaStream_t st, const XfParams* xf) {
    struct G { uint64_t codes[12], luts[12], rows[12], d[12], out_at[12], count; } g;
    memcpy(&g, groups, sizeof g);
    if ((uintptr_t)x % 4 != 0 || (inputs > 1 && cols % 2 != 0)) return cudaErrorInvalidValue;
    uint32_t most_pieces = 0, least_bytes = 0xffffffffu, most_bytes = 0;
    for (uint64_t i = 0; i < g.count; ++i) {
        const uint32_t row_bytes = (uint32_t)(cols * g.d[i] / 8);
        if (row_bytes / 64 > most_pieces) most_pieces = row_bytes / 64;
        if (row_bytes < least_bytes) least_bytes = row_bytes;
        if (row_bytes > most_bytes) most_bytes = row_bytes;
    }
    const int niw = (int)((most_pieces + GV_WARPS - 1) / GV_WARPS);
    if (niw < 1 || niw > 4) return cudaErrorInvalidValue;
    /* A slot of the ring holds 16 rows of at most 2,048 bytes (a longer row is cut in two halves, a slot each): up to 33 KB.
     * A step is up to four tiles, fewer when there are many inputs (the partial sums of a step — 16 warps x 16 rows x the
     * inputs rounded up to a power of two — are kept twice in at most 16 KB).  The block takes all the shared memory there
     * is; the table lands on a 64 KB boundary somewhere in its first 64 KB, and what is left either side of it holds the
     * partial sums and two to four slots wherever it lands. */
    uint32_t pi = 1;
    while (pi < inputs) pi *= 2;
    uint32_t ts = 8u / pi;
    ts = ts < 1 ? 1 : (ts > (uint32_t)GV_TS_MAX ? (uint32_t)GV_TS_MAX : ts);
    const uint32_t smem_bytes = 227u * 1024u - 1024u;
    uint32_t stage_bytes = 0;
    for (uint64_t i = 0; i < g.count; ++i) {
        const uint32_t row_bytes = (uint32_t)(cols * g.d[i] / 8), seg = row_bytes > 2048u ? row_bytes / 2u : row_bytes;
        if (row_bytes > 2048u && (row_bytes / 64u) % 32u != 0) return cudaErrorInvalidValue;              /* halves of whole sixteen-piece groups */
        const uint32_t need = 16u * (seg + GV_ROW_PAD);
        if (need > stage_bytes) stage_bytes = need;
    }
    (void)least_bytes;
    GemvFast a;
    memset(&a, 0, sizeof a);
    uint32_t tiles = 0, n = 0;
    for (uint64_t i = 0; i < g.count; ++i) {
        uint64_t rows = g.rows[i];
        if (rows_cap && rows_cap[i] < rows) rows = rows_cap[i];
        if (rows == 0) continue;                                             /* a group with no row to write */
        /* with several inputs and no stride an input's answers sit `rows` apart: the NAMED rows, not the trimmed ones */
        if (rows != g.rows[i] && inputs > 1 && out_stride == 0) return cudaErrorInvalidValue;
        a.codes[n] = (const uint8_t*)(uintptr_t)g.codes[i];
        a.scales[n] = (const uint16_t*)(uintptr_t)g.luts[i];
        a.rows[n] = (uint32_t)rows; a.d[n] = (uint32_t)g.d[i]; a.out_at[n] = g.out_at[i];
        a.halves[n] = cols * g.d[i] / 8 > 2048 ? 2u : 1u;
        a.tile0[n] = tiles;
        tiles += (uint32_t)((rows + 15) / 16);
        ++n;
    }
    if (n == 0) return cudaSuccess;
    a.tile0[n] = tiles;
    const uint32_t steps = tiles;                                            /* the grid's size: a block has a tile at least */
    a.count = n; a.cols = (uint32_t)cols; a.inputs = (uint32_t)inputs; a.out_stride = out_stride;
    a.x_wide = ((uintptr_t)x % 16 == 0 && cols % 8 == 0) ? 1u : 0u;
    a.ts = ts; a.pi = pi; a.stage_bytes = stage_bytes; a.smem_bytes = smem_bytes;
    if (xf) {
        if (n != 1 || inputs != 1 || rows_cap || (uint64_t)a.rows[0] > xf->slot_words) return cudaErrorInvalidValue;
        a.xf = *xf;
    }
    a.status = device_status_word();
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    {   /* the table's image, once a device; making it twice (two threads' first calls at once) writes the same bytes */
        static std::atomic<bool> made[64];
        if (!made[dev].load(std::memory_order_acquire)) {
            gv_lut_image_kernel<<<16, 256, 0, st>>>();
            const cudaError_t e = cudaGetLastError();
            if (e != cudaSuccess) return e;
            note_launch(1);
            made[dev].store(true, std::memory_order_release);
        }
    }
    const size_t smem = smem_bytes;
    const unsigned grid = steps < 148u ? steps : 148u;
#define SV_GV2(N, WW)                                                                                                               \
    do {                                                                                                                             \
        static std::atomic<bool> ready[64];      /* a function's attribute is a device's: once a device, at the kernel's ceiling */ \
        if (!ready[dev].load(std::memory_order_acquire)) {                                                                           \
            const cudaError_t e = cudaFuncSetAttribute(tq_gemv_fast_kernel<N, WW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return e;                                                                                          \
            ready[dev].store(true, std::memory_order_release);                                                                       \
        }                                                                                                                            \
        cudaLaunchConfig_t cfg = {};                                                                                                 \
        cfg.gridDim = dim3(grid); cfg.blockDim = dim3(GV_THREADS + 32); cfg.dynamicSmemBytes = smem; cfg.stream = st;                \
        cudaLaunchAttribute at[1];                                                                                                   \
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;         \
        cfg.attrs = at; cfg.numAttrs = pdl_allowed() ? 1u : 0u;                                                                      \
        const cudaError_t le = cudaLaunchKernelEx(&cfg, tq_gemv_fast_kernel<N, WW>, out, a, x, over);                                \
        if (le != cudaSuccess) return le;                                                                                            \
    } while (0)
#define SV_GV(N) do { if (one_width == 4) SV_GV2(N, 4); else if (one_width == 8) SV_GV2(N, 8); else SV_GV2(N, 0); } while (0)
    uint32_t one_width = a.d[0];
    for (uint32_t i = 1; i < n; ++i) if (a.d[i] != one_width) one_width = 0;
    if (niw == 1) SV_GV(1);
    else if (niw == 2) SV_GV(2);
    else if (niw == 3) SV_GV(3);
    else SV_GV(4);
#undef SV_GV2
#undef SV_GV
    note_launch(1);
    return cudaGetLastError();
}

}  // namespace sv
