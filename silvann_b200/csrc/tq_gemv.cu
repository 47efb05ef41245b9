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
 *     of a warp loads 16 neighbouring bytes of rows g and g + 8 straight into registers (no staging in shared memory) and
 *     uses them as its A fragments; the matching x values sit in registers as B fragments for the whole kernel;
 *   · the table is 256 bytes an entry — 32 copies of the 4-bit pair table, then 32 of the 8-bit table, one a bank — so a
 *     lookup never conflicts and its offset is ONE byte-permute of the code word;
 *   · a block is 16 warps that split a row's bytes 64 at a time; their partial sums for a tile of 16 rows meet in shared
 *     memory, double-buffered, one barrier a tile.
 * Shapes it takes: widths 4 and 8, row bytes a multiple of 64, codes 16-byte aligned, at most 8 inputs, at most
 * 64 x registers a thread (cols ≤ 8,192).  Anything else stays with the as-worded kernel in tq.cu. */
#include "common.cuh"
#include "kernels.h"
#include <string.h>

namespace sv {

using H = Elem<SV_DTYPE_FP16>;

static __device__ const uint16_t g_tq_levels_gemv[318] = {
#include "tq_levels.inc"
};

constexpr int GV_WARPS = 16, GV_THREADS = GV_WARPS * 32, GV_LUT_BYTES = 256 * 256;

struct GemvFast {
    const uint8_t* codes[12];
    const uint16_t* scales[12];
    uint32_t rows[12], d[12], tile0[13];       /* group i's tiles of 16 rows are [tile0[i], tile0[i+1]) */
    uint64_t out_at[12];
    uint32_t count, cols, inputs;
    uint64_t out_stride;
};

__device__ __forceinline__ uint32_t gv_lut(uint32_t lut, uint32_t lane4, uint32_t w, int idx) {
    uint32_t v;
    const uint32_t off = __byte_perm(w, lane4, 0x5504u | ((uint32_t)idx << 4));        /* (code byte) << 8 | lane · 4 */
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(lut + off));
    return v;
}
__device__ __forceinline__ uint4 gv_ldg(const uint8_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

/* NIW: the 64-byte pieces of a row one warp owns at most (pieces warp, warp + 16, ...).  x registers a thread: 16·NIW. */
template <int NIW>
__global__ void __launch_bounds__(GV_THREADS, 1) tq_gemv_fast_kernel(uint16_t* out, GemvFast a, const uint16_t* x, unsigned int* over) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint32_t* lut_w = reinterpret_cast<uint32_t*>(smem);
    float* part = reinterpret_cast<float*>(smem + GV_LUT_BYTES);              /* [2][GV_WARPS][16 rows][8 inputs] */
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    for (int i = tid; i < 256 * 32; i += GV_THREADS) {
        const int b = i >> 5, l = i & 31;
        const uint32_t l8 = g_tq_levels_gemv[62 + b];
        lut_w[b * 64 + l] = (uint32_t)g_tq_levels_gemv[14 + (b & 15)] | ((uint32_t)g_tq_levels_gemv[14 + (b >> 4)] << 16);
        lut_w[b * 64 + 32 + l] = l8 | (l8 << 16);
    }
    __syncthreads();
    const uint32_t lut4 = smem_u32(smem), lut8 = lut4 + 128u, lane4 = (uint32_t)lane * 4u;
    const uint32_t tiles = a.tile0[a.count];
    uint32_t xr[NIW][16];                                                    /* this lane's B fragments: input g, the columns of its bytes */
    uint32_t have_d = 0;
    int buf = 0;
    bool hit = false;
    for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x, buf ^= 1) {
        int gi = 0;
        while (tile >= a.tile0[gi + 1]) ++gi;
        const uint32_t d = a.d[gi], rows = a.rows[gi], row0 = (tile - a.tile0[gi]) * 16u;
        const uint32_t row_bytes = a.cols * d / 8u, pieces = row_bytes / 64u, per_lane = d == 4 ? 32u : 16u;     /* columns a lane's 16 bytes hold */
        if (d != have_d) {                                                   /* the columns a lane owns depend on the width */
            have_d = d;
#pragma unroll
            for (int i = 0; i < NIW; ++i) {
                const uint32_t piece = (uint32_t)warp + (uint32_t)i * GV_WARPS;
                const uint32_t c0 = piece * (64u * 8u / d) + (uint32_t)t * per_lane;
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    uint32_t v = 0u;
                    if (piece < pieces && (uint32_t)g < a.inputs && (uint32_t)e * 2u < per_lane)
                        v = *reinterpret_cast<const uint32_t*>(x + (size_t)g * a.cols + c0 + e * 2);
                    xr[i][e] = v;
                }
            }
        }
        const uint32_t ra = min(row0 + (uint32_t)g, rows - 1u), rb = min(row0 + (uint32_t)g + 8u, rows - 1u);
        const uint8_t* pa = a.codes[gi] + (size_t)ra * row_bytes + (size_t)t * 16u;
        const uint8_t* pb = a.codes[gi] + (size_t)rb * row_bytes + (size_t)t * 16u;
        uint4 wa[NIW], wb[NIW];
#pragma unroll
        for (int i = 0; i < NIW; ++i) {
            const uint32_t piece = (uint32_t)warp + (uint32_t)i * GV_WARPS;
            if (piece < pieces) { wa[i] = gv_ldg(pa + (size_t)piece * 64u); wb[i] = gv_ldg(pb + (size_t)piece * 64u); }
            else { wa[i] = make_uint4(0, 0, 0, 0); wb[i] = wa[i]; }
        }
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < NIW; ++i) {
            const uint32_t piece = (uint32_t)warp + (uint32_t)i * GV_WARPS;
            if (piece >= pieces) continue;                                   /* the whole warp together */
            const uint32_t wsa[4] = {wa[i].x, wa[i].y, wa[i].z, wa[i].w}, wsb[4] = {wb[i].x, wb[i].y, wb[i].z, wb[i].w};
            if (d == 4) {
#pragma unroll
                for (int m = 0; m < 8; ++m) {                                /* bytes 2m, 2m+1: four codes a row */
                    const uint32_t ua = wsa[m >> 1], ub = wsb[m >> 1];
                    const int b0 = (m & 1) * 2;
                    mma16816<SV_DTYPE_FP16>(c, gv_lut(lut4, lane4, ua, b0), gv_lut(lut4, lane4, ub, b0), gv_lut(lut4, lane4, ua, b0 + 1),
                                            gv_lut(lut4, lane4, ub, b0 + 1), xr[i][2 * m], xr[i][2 * m + 1]);
                }
            } else {
#pragma unroll
                for (int m = 0; m < 4; ++m) {                                /* bytes 4m .. 4m+3: four codes a row */
                    const uint32_t ua = wsa[m], ub = wsb[m];
                    const uint32_t a0 = __byte_perm(gv_lut(lut8, lane4, ua, 0), gv_lut(lut8, lane4, ua, 1), 0x5410);
                    const uint32_t a1 = __byte_perm(gv_lut(lut8, lane4, ub, 0), gv_lut(lut8, lane4, ub, 1), 0x5410);
                    const uint32_t a2 = __byte_perm(gv_lut(lut8, lane4, ua, 2), gv_lut(lut8, lane4, ua, 3), 0x5410);
                    const uint32_t a3 = __byte_perm(gv_lut(lut8, lane4, ub, 2), gv_lut(lut8, lane4, ub, 3), 0x5410);
                    mma16816<SV_DTYPE_FP16>(c, a0, a1, a2, a3, xr[i][2 * m], xr[i][2 * m + 1]);
                }
            }
        }
        /* c0, c1: (row g, inputs 2t, 2t+1) · c2, c3: (row g + 8, the same inputs) */
        float* mine = part + ((size_t)buf * GV_WARPS + warp) * 128;
        *reinterpret_cast<float2*>(mine + g * 8 + t * 2) = make_float2(c[0], c[1]);
        *reinterpret_cast<float2*>(mine + (g + 8) * 8 + t * 2) = make_float2(c[2], c[3]);
        __syncthreads();                                                     /* one a tile: the other buffer is free again by the next */
        if (tid < 128) {
            const uint32_t r = (uint32_t)tid >> 3, k = (uint32_t)tid & 7u;
            if (row0 + r < rows && k < a.inputs) {
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < GV_WARPS; ++w) sum += part[((size_t)buf * GV_WARPS + w) * 128 + tid];
                const float scale = H::to_float(a.scales[gi][row0 + r]);
                const uint64_t at = a.out_stride != 0 ? k * a.out_stride + a.out_at[gi] + row0 + r : a.out_at[gi] + (uint64_t)k * rows + row0 + r;
                out[at] = H::from_float(sum * scale, hit);
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
        if ((cols * g.d[i] / 8) % 64 != 0 || cols * g.d[i] % 8 != 0) return false;
        if (g.codes[i] % 16 != 0 || g.luts[i] % 2 != 0 || g.rows[i] > 0x0fffffffu) return false;
    }
    return true;
}

cudaError_t tq_gemv_fast_launch(uint16_t* out, const void* groups, const uint64_t* rows_cap, const uint16_t* x, uint64_t cols, uint64_t inputs,
                                uint64_t out_stride, unsigned int* over, cudaStream_t st) {
    struct G { uint64_t codes[12], luts[12], rows[12], d[12], out_at[12], count; } g;
    memcpy(&g, groups, sizeof g);
    if ((uintptr_t)x % 4 != 0 || (inputs > 1 && cols % 2 != 0)) return cudaErrorInvalidValue;
    GemvFast a;
    memset(&a, 0, sizeof a);
    uint32_t tiles = 0, most_pieces = 0;
    uint32_t n = 0;
    for (uint64_t i = 0; i < g.count; ++i) {
        uint64_t rows = g.rows[i];
        if (rows_cap && rows_cap[i] < rows) rows = rows_cap[i];
        if (rows == 0) continue;                                             /* a group with no row to write */
        a.codes[n] = (const uint8_t*)(uintptr_t)g.codes[i];
        a.scales[n] = (const uint16_t*)(uintptr_t)g.luts[i];
        a.rows[n] = (uint32_t)rows; a.d[n] = (uint32_t)g.d[i]; a.out_at[n] = g.out_at[i];
        /* with several inputs and no stride an input's answers sit `rows` apart: the NAMED rows, not the trimmed ones */
        if (rows != g.rows[i] && inputs > 1 && out_stride == 0) return cudaErrorInvalidValue;
        a.tile0[n] = tiles;
        tiles += (uint32_t)((rows + 15) / 16);
        const uint32_t pieces = (uint32_t)(cols * g.d[i] / 8 / 64);
        if (pieces > most_pieces) most_pieces = pieces;
        ++n;
    }
    if (n == 0) return cudaSuccess;
    a.tile0[n] = tiles;
    a.count = n; a.cols = (uint32_t)cols; a.inputs = (uint32_t)inputs; a.out_stride = out_stride;
    const int niw = (int)((most_pieces + GV_WARPS - 1) / GV_WARPS);
    const size_t smem = GV_LUT_BYTES + 2 * GV_WARPS * 128 * sizeof(float);
    const unsigned grid = tiles < 148u ? tiles : 148u;
#define SV_GV(N)                                                                                                                     \
    do {                                                                                                                             \
        static bool ready = false;                                                                                                   \
        if (!ready) {                                                                                                                \
            const cudaError_t e = cudaFuncSetAttribute(tq_gemv_fast_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return e;                                                                                          \
            ready = true;                                                                                                            \
        }                                                                                                                            \
        tq_gemv_fast_kernel<N><<<grid, GV_THREADS, smem, st>>>(out, a, x, over);                                                     \
    } while (0)
    if (niw <= 1) SV_GV(1);
    else if (niw == 2) SV_GV(2);
    else if (niw == 3) SV_GV(3);
    else if (niw == 4) SV_GV(4);
    else return cudaErrorInvalidValue;
#undef SV_GV
    note_launch(1);
    return cudaGetLastError();
}

}  // namespace sv
