/* expert.cu — the expert-major GEMM: a coded matrix applied to several rows of `x` at once (a prompt chunk's projections).
 *
 * The reference's doors (engine/src/packages/nn/gpu/kernels/kernels.cuh:1513-1624 the shared body; expert_rows :1626-1633,
 * expert_rows_sum :1640-1648, expert_groups :1650-1660, expert_rows_finish :1662-1672, expert_rows_reduce :1676-1692,
 * expert_pairs_rows :3864-3871; declared in engine/src/packages/nn/contracts/abi/gpu.cuh) read a list of PAIRS: pair j is
 * (row of x it reads, row of out it writes), and
 *     out[pair's out row][r] = half(scale_r · sum_c level(code[r][c]) · x[pair's x row][c])
 * for every row r of the matrix the rooms hold; at 16 bits the codes are the halves themselves and the scale is 1.  The
 * levels are fp16 table entries and x is fp16, so every product is exact in fp32 and only the order of the sum is a family's
 * own.  The prompt path of a mixer (engine/src/packages/ai_qwen_3/cpu/opcodes/prefill__abi.cuh:135-237) makes its q, k, v
 * and o projections through these doors, up to 256 rows a call.
 *
 * Two kernels.  `expert_rows_kernel` is the door as worded — any width, any shape, a block a matrix row, eight pairs a pass.
 * `expert_fast_kernel` is the one a prompt runs on: a block owns 128 matrix rows and up to 128 pairs and walks the columns
 * through a ring of stages of TWO 64-column blocks each (a hand-over between its roles costs a few hundred cycles on either
 * side whatever hangs on it, so it is paid once a 128 columns).  Three roles, each a chain of its own:
 *   · eight COPIER warps gather the pairs' rows of x as the B operand (K-major, 128-byte swizzle) and bring the codes, as
 *     they lie in memory, into a small padded ring — cp.async, the threads laid along a row (whole lines from DRAM), as far
 *     ahead as the slots allow (four stages where every group is 4 bits wide, three where one is 8);
 *   · sixteen EXPANDER warps turn the codes into fp16 straight in TENSOR MEMORY as the A operand — a thread owns one matrix
 *     row (its lane) and 32 of the stage's columns, a code byte is ONE shared-memory lookup in a table of 256 entries of 128
 *     bytes (a lane reads its own bank, so no lookup ever conflicts; at 4 bits an entry is the byte's two levels, packed as
 *     the MMA wants them; at 8 bits the level twice), and the 16 packed words go out with one tcgen05.st — so the matrix's
 *     expanded rows never pass through the shared-memory pipe, which is what a block runs out of;
 *   · one thread issues tcgen05.mma with A in tensor memory (M 128, N = the pairs rounded up to 16, K 16 a step, eight a
 *     stage), accumulating in tensor memory, and gives a stage back by a commit on its mbarrier.
 * The expanders then read the accumulator out of tensor memory, scale a row by its fp16 scale, round once and store — or,
 * for expert_rows_sum, add weight · value onto the fp32 running sum.  The roles meet only on mbarriers (no block barrier
 * inside the loop), so a wait that runs out raises the block's flag and every role leaves by itself.
 * Shapes the fast kernel takes: widths 4, 8 and 16, columns a multiple of 64, codes and x on 16 bytes.  Every mbarrier wait
 * is bounded; one that runs out ORs "B2TO" into the device's status word and the block leaves through the common exit
 * (copies in flight waited for, tensor memory given back). */
#include "common.cuh"
#include "tcgen05.cuh"
#include "kernels.h"
#include <atomic>
#include <string.h>

namespace sv {

using H = Elem<SV_DTYPE_FP16>;

static __device__ const uint16_t g_tq_levels_expert[318] = {
#include "tq_levels.inc"
};

struct ExpertGroups { uint64_t codes[12], luts[12], out_rows[12], d[12], out_at[12], pairs_at[12], pairs[12], count; };

__host__ __device__ __forceinline__ bool ex_width_known(uint64_t d) { return d == 1 || d == 2 || d == 3 || d == 4 || d == 5 || d == 8 || d == 16; }
__host__ __device__ __forceinline__ uint32_t ex_table_at(uint64_t d) { return d == 1 ? 0u : d == 2 ? 2u : d == 3 ? 6u : d == 4 ? 14u : d == 5 ? 30u : 62u; }
__host__ __device__ __forceinline__ uint64_t ex_row_bytes(uint64_t d, uint64_t cols) { const uint64_t per = 16 / d; return ((cols + per - 1) / per) * 2; }
__device__ __forceinline__ float ex_level(uint64_t d, uint32_t code) {
    return d == 16 ? H::to_float((uint16_t)code) : H::to_float(g_tq_levels_expert[ex_table_at(d) + code]);
}

/* ---- the door as worded: a block a matrix row, eight pairs a pass ------------------------------------------------------ */
__global__ void __launch_bounds__(128) expert_rows_kernel(uint16_t* out, float* acc, const uint8_t* weights, uint64_t held, const uint8_t* luts,
                                                          const uint16_t* x, const uint32_t* pairs, const uint16_t* w, uint64_t count, uint64_t d,
                                                          uint64_t out_rows, uint64_t cols, unsigned int* over) {
    __shared__ float sh[4][8];
    const uint64_t per = 16 / d, row_bytes = ex_row_bytes(d, cols), units = (cols + per - 1) / per;
    const uint32_t mask = (uint32_t)((1ull << d) - 1ull);
    bool hit = false;
    for (uint64_t r = blockIdx.x; r < out_rows && r < held; r += gridDim.x) {
        const uint8_t* row = weights + r * row_bytes;
        const float scale = d == 16 ? 1.0f : H::to_float((uint16_t)((uint32_t)luts[r * 2] | ((uint32_t)luts[r * 2 + 1] << 8)));
        for (uint64_t j0 = 0; j0 < count; j0 += 8) {
            const uint16_t* xr[8];
#pragma unroll
            for (int b = 0; b < 8; ++b) xr[b] = j0 + b < count ? x + (uint64_t)pairs[2 * (j0 + b)] * cols : nullptr;
            float part[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (uint64_t u = threadIdx.x; u < units; u += blockDim.x) {
                const uint32_t unit = (uint32_t)row[u * 2] | ((uint32_t)row[u * 2 + 1] << 8);
                const uint64_t c0 = u * per;
                for (uint64_t s = 0; s < per && c0 + s < cols; ++s) {
                    const float lv = ex_level(d, (unit >> (uint32_t)(d * s)) & mask);
#pragma unroll
                    for (int b = 0; b < 8; ++b)
                        if (xr[b]) part[b] += lv * H::to_float(xr[b][c0 + s]);
                }
            }
#pragma unroll
            for (int b = 0; b < 8; ++b)
                for (int o = 16; o > 0; o >>= 1) part[b] += __shfl_xor_sync(0xffffffffu, part[b], o);
            if ((threadIdx.x & 31) == 0)
#pragma unroll
                for (int b = 0; b < 8; ++b) sh[threadIdx.x >> 5][b] = part[b];
            __syncthreads();
            if (threadIdx.x < 8 && j0 + threadIdx.x < count) {
                const uint64_t j = j0 + threadIdx.x;
                const float v = ((sh[0][threadIdx.x] + sh[1][threadIdx.x]) + (sh[2][threadIdx.x] + sh[3][threadIdx.x])) * scale;
                const uint64_t at = (uint64_t)pairs[2 * j + 1] * out_rows + r;
                if (out) out[at] = H::from_float(v, hit);
                else acc[at] += v * H::to_float(w[pairs[2 * j]]);
            }
            __syncthreads();
        }
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* expert_rows_finish: out[i] = half(residual[i] + acc[i]), acc[i] back to zero (residual may be out) */
__global__ void __launch_bounds__(256) expert_rows_finish_kernel(uint16_t* out, float* acc, const uint16_t* residual, uint64_t n, unsigned int* over) {
    bool hit = false;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        out[i] = H::from_float(H::to_float(residual[i]) + acc[i], hit);
        acc[i] = 0.0f;
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}
/* expert_rows_reduce: acc is n rows of k picks of cols floats; out[t][c] = half(residual[t][c] + the picks added in their order) */
__global__ void __launch_bounds__(256) expert_rows_reduce_kernel(uint16_t* out, float* acc, const uint16_t* residual, uint64_t n, uint64_t k, uint64_t cols,
                                                                 unsigned int* over) {
    bool hit = false;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n * cols; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t t = i / cols, c = i - t * cols;
        float s = 0.0f;
        for (uint64_t j = 0; j < k; ++j) {
            float* a = acc + (t * k + j) * cols + c;
            s += *a;
            *a = 0.0f;
        }
        out[i] = H::from_float(H::to_float(residual[i]) + s, hit);
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}
/* expert_pairs_rows: pair t = (x_step · t + x_at, out_step · t + out_at), written on the card */
__global__ void __launch_bounds__(256) expert_pairs_rows_kernel(uint32_t* pairs, uint64_t n, uint64_t x_step, uint64_t x_at, uint64_t out_step, uint64_t out_at) {
    for (uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; t < n; t += (uint64_t)gridDim.x * blockDim.x) {
        pairs[2 * t] = (uint32_t)(x_step * t + x_at);
        pairs[2 * t + 1] = (uint32_t)(out_step * t + out_at);
    }
}

/* ---- the fast kernel ---------------------------------------------------------------------------------------------------- */

constexpr int EX_COPIERS = 256, EX_THREADS = 800, EX_PRODUCERS = 512, EX_BM = 128, EX_BN = 128, EX_KC = 64;
constexpr int EX_STAGES_MAX = 4;                                      /* stages of two column blocks: four, or three where a group's codes are 8 bits wide (its ring slots are larger) */
constexpr uint32_t EX_ATOM = 16384;                                   /* a tile of 128 rows x 64 columns of halves, 128-byte rows, swizzled */
constexpr uint32_t EX_STAGE_BYTES = 2 * EX_ATOM;                      /* a stage's x: two column blocks (the matrix's rows live in tensor memory) */
constexpr uint32_t EX_RAW_PITCH4 = 80, EX_RAW_PITCH8 = 144;          /* a stage's codes as they lie in memory, rows padded apart: a ring slot is 128 rows of these */
constexpr uint32_t EX_T_ACC = 0, EX_T_A = 128, EX_T_A_STAGE = 64, EX_T_COLS = 512;   /* tensor memory: the sums, then a stage's A operand, 64 packed columns each */
constexpr uint32_t EX_LUT_BYTES = 256 * 128;
__host__ __device__ constexpr uint32_t ex_smem_bytes(uint32_t stages, uint32_t raw_bytes) { return 1024u + EX_LUT_BYTES + stages * (EX_STAGE_BYTES + raw_bytes) + 2u * EX_BN * 4u + 256u; }
constexpr uint32_t EX_SMEM_MAX = ex_smem_bytes(4, 128 * EX_RAW_PITCH4) > ex_smem_bytes(3, 128 * EX_RAW_PITCH8) ? ex_smem_bytes(4, 128 * EX_RAW_PITCH4) : ex_smem_bytes(3, 128 * EX_RAW_PITCH8);

struct ExpertFast {
    const uint8_t* codes[12];
    const uint16_t* scales[12];
    uint32_t out_rows[12], held[12], d[12], pairs_at[12], pairs[12], tile0[13];   /* group i's blocks of 128 rows are [tile0[i], tile0[i+1]) */
    uint64_t out_at[12];
    uint32_t count, cols, stages, raw_bytes;   /* stages: 3 or 4; raw_bytes: a ring slot */
    const uint16_t* x;
    const uint32_t* rows;
    const uint16_t* w;
    uint16_t* out;
    float* acc;
    unsigned int* status;
    unsigned int* over;
};

__device__ __forceinline__ void ex_cp16(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ uint4 ex_ldg128(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void ex_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void ex_cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t ex_lds32(uint32_t a) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));     /* (the table is written once, before the first lookup: not volatile, the compiler may move it) */
    return v;
}
__device__ __forceinline__ uint4 ex_lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ void ex_sts128(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

__global__ void __launch_bounds__(EX_THREADS, 1) expert_fast_kernel(const ExpertFast a) {
    extern __shared__ uint8_t ex_smem_raw[];
    const uint32_t base = (smem_u32(ex_smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = ex_smem_raw + (base - smem_u32(ex_smem_raw));
    const uint32_t S = a.stages, RAW = a.raw_bytes;                          /* stages (and ring slots); bytes a ring slot */
    const uint32_t lut_at = base, stage_at = lut_at + EX_LUT_BYTES, raw_at = stage_at + S * EX_STAGE_BYTES;
    uint32_t* xrow_s = reinterpret_cast<uint32_t*>(smem + EX_LUT_BYTES + S * (EX_STAGE_BYTES + RAW));
    uint32_t* orow_s = xrow_s + EX_BN;
    uint64_t* full = reinterpret_cast<uint64_t*>(orow_s + EX_BN);
    uint64_t* empty = full + EX_STAGES_MAX;
    uint64_t* raw_full = empty + EX_STAGES_MAX;
    uint64_t* acc_full = raw_full + EX_STAGES_MAX;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint32_t g = 0;
    while (g + 1 < a.count && blockIdx.x >= a.tile0[g + 1]) ++g;
    const uint32_t r0 = (blockIdx.x - a.tile0[g]) * EX_BM, j0 = blockIdx.y * EX_BN;
    if (j0 >= a.pairs[g]) return;                                           /* the whole block: this group has fewer pairs than the widest */
    const uint32_t nb = min((uint32_t)EX_BN, a.pairs[g] - j0), N = (nb + 15u) & ~15u;
    const uint32_t d = a.d[g], cols = a.cols, nk = cols / EX_KC, nst = (nk + 1u) / 2u, out_rows = a.out_rows[g], held = a.held[g];
    const uint64_t row_bytes = (uint64_t)cols * d / 8u;

    if (tid == 0) {
        for (int s = 0; s < EX_STAGES_MAX; ++s) { mbar_init(&full[s], (EX_PRODUCERS + EX_COPIERS) / 32); mbar_init(&empty[s], 1); mbar_init(&raw_full[s], EX_COPIERS / 32); }
        mbar_init(acc_full, 1);
        *abort_flag = 0u;
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, EX_T_COLS);
    else if (warp <= EX_PRODUCERS / 32) {
        const int p = tid - 32;
        for (int j = p; j < EX_BN; j += EX_PRODUCERS) {
            const uint32_t* pr = a.rows + 2ull * (a.pairs_at[g] + j0 + min((uint32_t)j, nb - 1u));
            xrow_s[j] = pr[0]; orow_s[j] = pr[1];
        }
        if (d != 16u) {                                                      /* entry e, 32 copies: two threads an entry, half the copies each */
            const uint32_t e = (uint32_t)p & 255u, l8 = g_tq_levels_expert[62 + e];
            const uint32_t v = d == 4u ? ((uint32_t)g_tq_levels_expert[14 + (e & 15u)] | ((uint32_t)g_tq_levels_expert[14 + (e >> 4)] << 16)) : (l8 | (l8 << 16));
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) ex_sts128(lut_at + e * 128u + ((uint32_t)p >> 8) * 64u + i * 16u, v, v, v, v);
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        /* ---------------- every MMA ---------------- */
        if (lane == 0) {
            const uint32_t idesc = idesc_f16(0, 0, EX_BM, (int)N);
            uint32_t s = 0, ph = 0;
            for (uint32_t st = 0; st < nst; ++st) {                          /* a stage: two column blocks (one at an odd end), eight MMAs a hand-over */
                if (!mbar_wait(&full[s], ph, abort_flag, a.status)) break;
                tc_fence_after();
                const uint32_t blocks = min(2u, nk - 2u * st);
                for (uint32_t h = 0; h < blocks; ++h) {                        /* A: this stage's rows in tensor memory, 8 packed columns a step of 16 */
                    const uint64_t bd = smem_desc_sw128(stage_at + s * EX_STAGE_BYTES + h * EX_ATOM, 16, 1024);
                    const uint32_t at = tmem + EX_T_A + s * EX_T_A_STAGE + h * 32u;
#pragma unroll
                    for (uint32_t kk = 0; kk < 4; ++kk) tc_mma_ts(tmem + EX_T_ACC, at + kk * 8u, bd + kk * 2u, idesc, (st | h | kk) != 0u ? 1u : 0u);
                }
                tc_commit(&empty[s]);
                if (++s == S) { s = 0; ph ^= 1u; }
            }
            tc_commit(acc_full);
        }
    } else if (warp > EX_PRODUCERS / 32) {
        /* ---------------- copiers: the pairs' rows of x -> B tiles, the codes as they lie -> the ring ----------------
         * Eight warps that only copy, two stages ahead: what a warp does for a stage is one chain of waits, so the copies have
         * a chain of their own beside the expanders'.  A thread takes one chunk column of the stage's 16 and the rows 16 apart
         * (N / 16 pieces of 16 bytes), and two or four 16-byte pieces of the codes, its addresses carried from stage to stage.  A slot of x is written again once the MMAs of
         * three stages ago have completed (their commit); that also frees the ring slot of four stages ago, which the
         * expanders had read before they handed that stage over. */
        const uint32_t cp = (uint32_t)(tid - 32 - EX_PRODUCERS);              /* 0 .. 255 */
        const uint32_t xc = cp & 15u, xj = cp >> 4;                            /* chunk column; first row (rows xj, xj + 16, ...) */
        const uint32_t x_off = (xc >> 3) * EX_ATOM + swz128(xj, xc & 7u), x_count = N / 16u;
        const uint16_t* x_src[8];
        uint32_t x_bytes[8];
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) {
            const uint32_t j = xj + 16u * i;
            x_src[i] = a.x + (uint64_t)xrow_s[j] * cols + xc * 8u;
            x_bytes[i] = j < nb ? 16u : 0u;
        }
        const uint32_t code_step = d == 4u ? 64u : d == 8u ? 128u : 256u, pitch = d == 4u ? EX_RAW_PITCH4 : EX_RAW_PITCH8;
        const uint32_t per_row = code_step / 16u, c_count = d == 16u ? 0u : 128u * per_row / EX_COPIERS;   /* 16-byte pieces of codes a row; a thread (2 or 4) */
        const uint32_t c_q = cp & (per_row - 1u), c_row0 = cp / per_row, c_rows = EX_COPIERS / per_row;   /* its piece of a row; its rows c_row0, + c_rows, ... */
        const uint8_t* c_src[4];
        uint32_t c_dst[4], c_bytes[4];
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
            const uint32_t crow = c_row0 + c_rows * i;
            const bool live = i < c_count && r0 + crow < held && r0 + crow < out_rows;
            c_src[i] = a.codes[g] + (live ? (uint64_t)(r0 + crow) * row_bytes : 0ull) + c_q * 16u;
            c_dst[i] = raw_at + crow * pitch + c_q * 16u;
            c_bytes[i] = live ? 16u : 0u;
        }
        const uint32_t LAG = S - 2u;                                          /* stages its copies run ahead of their hand-over: the slots less the one the MMA reads and one to spare */
        bool ok = true;
        uint32_t sx = 0, phx = 1, sr = 0;                                      /* the slot of the stage asked for, the parity of its last release; the slot handed over next */
        for (uint32_t c = 0; c < nst + LAG; ++c) {
            if (c < nst) {
                if (c >= S && ok) ok = mbar_wait(&empty[sx], phx, abort_flag, a.status);
                if (ok) {
                    const bool second = 2u * c + 1u < nk;                      /* the stage's second column block exists */
                    if (second || xc < 8u) {
                        const uint32_t at = stage_at + sx * EX_STAGE_BYTES + x_off;
#pragma unroll
                        for (uint32_t i = 0; i < 8; ++i)
                            if (i < x_count) ex_cp16(at + i * 2048u, x_src[i], x_bytes[i]);
                    }
                    if (second || c_q * 2u < per_row) {
                        const uint32_t to = sx * RAW;
#pragma unroll
                        for (uint32_t i = 0; i < 4; ++i)
                            if (i < c_count) ex_cp16(c_dst[i] + to, c_src[i], c_bytes[i]);
                    }
                }
#pragma unroll
                for (uint32_t i = 0; i < 8; ++i) x_src[i] += 2 * EX_KC;
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i) c_src[i] += code_step;
                if (++sx == S) { sx = 0; phx ^= 1u; }
            }
            ex_cp_commit();
            if (c >= LAG) {                                                  /* stage c - LAG: this thread's copies have landed */
                if (LAG == 2u) ex_cp_wait<2>(); else ex_cp_wait<1>();
                fence_proxy_async_smem();                                    /* x, for the MMA's reads */
                __syncwarp();
                if (lane == 0 && ok) { mbar_arrive(&raw_full[sr]); mbar_arrive(&full[sr]); }
                if (++sr == S) sr = 0;
            }
            if (!ok) break;
        }
        ex_cp_wait<0>();
    } else {
        /* ---------------- expanders: codes -> the A operand in tensor memory; then the read-out ----------------
         * A stage is TWO column blocks (128 columns): a hand-over between the producers and the issuing thread — the waits,
         * the fences, the arrivals, the commit — costs a few hundred cycles on either side whatever hangs on it, so it is paid
         * once a 128 columns.  The shared-memory pipe is what a block runs out of, so the matrix's expanded rows never touch
         * it: a thread owns ONE matrix row (its lane of tensor memory; a warp its quadrant's 32 rows) and 32 of the stage's
         * columns (the four warps of a quadrant a quarter each), reads its 16 or 32 bytes of codes from the ring (rows padded
         * apart: no bank conflict), looks them up — a 4-bit byte's entry is already two neighbouring halves packed as the MMA
         * wants them — and stores the 16 packed words with one tcgen05.st; the MMA takes A from tensor memory. */
        const uint32_t quad = (uint32_t)warp & 3u, part = (uint32_t)(warp - 1) >> 2, row = quad * 32u + (uint32_t)lane;
        const bool own_ok = r0 + row < held && r0 + row < out_rows;          /* the row this thread expands */
        const uint32_t code_step = d == 4u ? 64u : d == 8u ? 128u : 256u;    /* bytes of a row a stage covers */
        const uint32_t pitch = d == 4u ? EX_RAW_PITCH4 : EX_RAW_PITCH8;
        const uint32_t my_raw = raw_at + row * pitch + part * (code_step / 4u);   /* this thread's 32 columns of its row */
        const uint8_t* my_halves = a.codes[g] + (own_ok ? (uint64_t)(r0 + row) * row_bytes : 0ull) + part * 64u;   /* (16 bits: read straight from memory) */
        const uint32_t lane_lut = lut_at + (uint32_t)lane * 4u;
        const uint32_t my_tile = part >> 1;                                  /* which of the stage's two column blocks this thread's columns are in */
        const uint32_t a_at = tmem + EX_T_A + part * 16u + ((quad * 32u) << 16);   /* + the slot's 64 columns */
        bool ok = true;
        uint32_t s = 0, ph = 1;                                               /* the slot of the stage being expanded; the parity of its last release */
        for (uint32_t st = 0; st < nst && ok; ++st) {
            uint32_t words[16];                                              /* 32 columns of this row: 16 words of two halves */
            if (d == 16u) {
#pragma unroll
                for (uint32_t i = 0; i < 16; ++i) words[i] = 0u;
                if (own_ok && 2u * st + my_tile < nk) {
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        const uint4 v = ex_ldg128(my_halves + (uint64_t)st * code_step + i * 16u);
                        words[4 * i] = v.x; words[4 * i + 1] = v.y; words[4 * i + 2] = v.z; words[4 * i + 3] = v.w;
                    }
                }
            } else {
                if (!mbar_wait(&raw_full[s], ph ^ 1u, abort_flag, a.status)) { ok = false; break; }
                const uint32_t raw = my_raw + s * RAW;
                if (d == 4u) {                                               /* a byte: two codes, one word — every lookup asked for before the first is used */
                    const uint4 cw = ex_lds128(raw);
                    const uint32_t ws[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        const uint32_t w = ws[i];
                        words[4 * i] = ex_lds32(lane_lut + ((w << 7) & 0x7F80u)); words[4 * i + 1] = ex_lds32(lane_lut + ((w >> 1) & 0x7F80u));
                        words[4 * i + 2] = ex_lds32(lane_lut + ((w >> 9) & 0x7F80u)); words[4 * i + 3] = ex_lds32(lane_lut + ((w >> 17) & 0x7F80u));
                    }
                } else {                                                     /* a byte: one code; two lookups make a word */
                    const uint4 c0 = ex_lds128(raw), c1 = ex_lds128(raw + 16u);
                    const uint32_t ws[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                    uint32_t v[32];
#pragma unroll
                    for (uint32_t u = 0; u < 8; ++u) {
                        const uint32_t w = ws[u];
                        v[4 * u] = ex_lds32(lane_lut + ((w << 7) & 0x7F80u)); v[4 * u + 1] = ex_lds32(lane_lut + ((w >> 1) & 0x7F80u));
                        v[4 * u + 2] = ex_lds32(lane_lut + ((w >> 9) & 0x7F80u)); v[4 * u + 3] = ex_lds32(lane_lut + ((w >> 17) & 0x7F80u));
                    }
#pragma unroll
                    for (uint32_t i = 0; i < 16; ++i) words[i] = __byte_perm(v[2 * i], v[2 * i + 1], 0x5410);
                }
                if (!own_ok) {
#pragma unroll
                    for (uint32_t i = 0; i < 16; ++i) words[i] = 0u;
                }
            }
            /* the slot of tensor memory is free once the MMAs of three stages ago have read it */
            if (st >= S && !mbar_wait(&empty[s], ph, abort_flag, a.status)) { ok = false; break; }
            tmem_st16(a_at + s * EX_T_A_STAGE, words);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[s]);
            if (++s == S) { s = 0; ph ^= 1u; }
        }

        /* the read-out: a thread a matrix row (its lane of tensor memory), four warps a quadrant splitting the pairs 32 at a time */
        if (ok) {
            uint32_t got = 1u;
            if (lane == 0) got = mbar_wait(acc_full, 0u, abort_flag, a.status) ? 1u : 0u;
            ok = __shfl_sync(0xffffffffu, got, 0) != 0u;
        }
        tc_fence_after();
        if (ok) {
            const uint32_t quad = (uint32_t)warp & 3u, grp = (uint32_t)(warp - 1) >> 2;
            const uint32_t orow = r0 + quad * 32u + (uint32_t)lane;
            const bool live = orow < held && orow < out_rows;
            const float scale = d == 16u || !live ? 1.0f : H::to_float(a.scales[g][orow]);
            bool hit = false;
            for (uint32_t cb = grp; cb * 32u < N; cb += (uint32_t)EX_PRODUCERS / 128u) {
                uint32_t v[32];
                tmem_ld32(tmem + ((quad * 32u) << 16) + cb * 32u, v);
                tmem_wait_ld();
                if (!live) continue;
#pragma unroll
                for (uint32_t c = 0; c < 32; ++c) {
                    const uint32_t j = cb * 32u + c;
                    if (j >= nb) break;
                    const float val = __uint_as_float(v[c]) * scale;
                    const uint64_t at = (uint64_t)orow_s[j] * out_rows + orow;
                    if (a.out) a.out[a.out_at[g] + at] = H::from_float(val, hit);
                    else a.acc[at] += val * H::to_float(a.w[xrow_s[j]]);
                }
            }
            if (hit && a.over) atomicOr(a.over, SV_FAULT_OVERFLOW);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, EX_T_COLS);
}

/* ---------------------------------------------------------------------------------------------------------------------------- */

static inline unsigned ex_grid(uint64_t items, unsigned cap = 4096u) { return (unsigned)(items < 1 ? 1 : (items > cap ? cap : items)); }

bool expert_width_ok(uint64_t d) { return ex_width_known(d); }

cudaError_t expert_rows_launch(uint16_t* out, float* acc, const uint8_t* weights, uint64_t w_room, const uint8_t* luts, uint64_t l_room, const uint16_t* x,
                               const uint32_t* pairs, const uint16_t* w, uint64_t count, uint64_t d, uint64_t out_rows, uint64_t cols, unsigned int* over,
                               cudaStream_t st) {
    const uint64_t row_bytes = ex_row_bytes(d, cols);
    uint64_t held = row_bytes == 0 ? 0 : w_room / row_bytes;
    if (d != 16 && l_room / 2 < held) held = l_room / 2;
    if (held == 0 || count == 0 || out_rows == 0) return cudaSuccess;
    expert_rows_kernel<<<ex_grid(out_rows < held ? out_rows : held), 128, 0, st>>>(out, acc, weights, held, luts, x, pairs, w, count, d, out_rows, cols, over);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t expert_rows_finish_launch(uint16_t* out, float* acc, const uint16_t* residual, uint64_t n, unsigned int* over, cudaStream_t st) {
    expert_rows_finish_kernel<<<ex_grid((n + 255) / 256), 256, 0, st>>>(out, acc, residual, n, over);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t expert_rows_reduce_launch(uint16_t* out, float* acc, const uint16_t* residual, uint64_t n, uint64_t k, uint64_t cols, unsigned int* over,
                                      cudaStream_t st) {
    expert_rows_reduce_kernel<<<ex_grid((n * cols + 255) / 256), 256, 0, st>>>(out, acc, residual, n, k, cols, over);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t expert_pairs_rows_launch(uint32_t* pairs, uint64_t n, uint64_t x_step, uint64_t x_at, uint64_t out_step, uint64_t out_at, cudaStream_t st) {
    expert_pairs_rows_kernel<<<ex_grid((n + 255) / 256, 64u), 256, 0, st>>>(pairs, n, x_step, x_at, out_step, out_at);
    note_launch(1);
    return cudaGetLastError();
}

/* Whether the fast kernel takes these groups (an sv_expert_groups by address) over rows of `cols` columns. */
bool expert_fast_fits(const void* groups, const void* x, uint64_t cols) {
    ExpertGroups g;
    memcpy(&g, groups, sizeof g);
    if (g.count == 0 || g.count > 12 || cols == 0 || cols % EX_KC != 0 || cols > (1ull << 20) || ((uintptr_t)x & 15u)) return false;
    uint64_t tiles = 0;
    for (uint64_t i = 0; i < g.count; ++i) {
        if (g.d[i] != 4 && g.d[i] != 8 && g.d[i] != 16) return false;
        if (g.codes[i] % 16 != 0 || g.luts[i] % 2 != 0 || g.out_rows[i] == 0 || g.out_rows[i] > 0x0fffffffu || g.pairs[i] == 0 || g.pairs[i] > 0x0fffffffu) return false;
        tiles += (g.out_rows[i] + EX_BM - 1) / EX_BM;
    }
    return tiles <= 0x7fffffffu;
}

/* `held`: for a single group, the rows its rooms hold (null: every row).  `out` or `acc` (with `w`), as the door has them. */
cudaError_t expert_fast_launch(uint16_t* out, float* acc, const void* groups, const uint64_t* held, const uint16_t* x, const uint32_t* rows,
                               const uint16_t* w, uint64_t cols, unsigned int* over, cudaStream_t st) {
    ExpertGroups g;
    memcpy(&g, groups, sizeof g);
    ExpertFast a;
    memset(&a, 0, sizeof a);
    uint32_t tiles = 0, widest = 0;
    for (uint64_t i = 0; i < g.count; ++i) {
        a.codes[i] = (const uint8_t*)(uintptr_t)g.codes[i]; a.scales[i] = (const uint16_t*)(uintptr_t)g.luts[i];
        a.out_rows[i] = (uint32_t)g.out_rows[i]; a.d[i] = (uint32_t)g.d[i]; a.pairs_at[i] = (uint32_t)g.pairs_at[i]; a.pairs[i] = (uint32_t)g.pairs[i];
        a.held[i] = held && *held < g.out_rows[i] ? (uint32_t)*held : (uint32_t)g.out_rows[i];
        a.out_at[i] = g.out_at[i];
        a.tile0[i] = tiles;
        tiles += (uint32_t)((g.out_rows[i] + EX_BM - 1) / EX_BM);
        if (a.pairs[i] > widest) widest = a.pairs[i];
    }
    a.tile0[g.count] = tiles;
    bool wide = false;                                                      /* a group at 8 bits: larger ring slots, one stage fewer */
    for (uint64_t i = 0; i < g.count; ++i) wide = wide || g.d[i] == 8;
    a.stages = wide ? 3u : 4u;
    a.raw_bytes = 128u * (wide ? EX_RAW_PITCH8 : EX_RAW_PITCH4);
    a.count = (uint32_t)g.count; a.cols = (uint32_t)cols; a.x = x; a.rows = rows; a.w = w; a.out = out; a.acc = acc; a.over = over;
    a.status = device_status_word();
    static std::atomic<bool> ready[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!ready[dev].load(std::memory_order_acquire)) {
        e = cudaFuncSetAttribute(expert_fast_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)EX_SMEM_MAX);
        if (e != cudaSuccess) return e;
        ready[dev].store(true, std::memory_order_release);
    }
    const dim3 grid(tiles, (widest + EX_BN - 1) / EX_BN);
    expert_fast_kernel<<<grid, EX_THREADS, ex_smem_bytes(a.stages, a.raw_bytes), st>>>(a);
    note_launch(1);
    return cudaGetLastError();
}

}  // namespace sv
