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
 * through a ring of three stages of TWO 64-column blocks each (a hand-over between the producers and the issuing thread
 * costs a few hundred cycles on either side whatever hangs on it, so it is paid once a 128 columns);
 *   · sixteen producer warps expand the codes to fp16 straight into TENSOR MEMORY as the A operand — a thread owns one
 *     matrix row (its lane) and 32 of the stage's columns, a code byte is ONE shared-memory lookup in a table of 256 entries
 *     of 128 bytes (a lane reads its own bank, so no lookup ever conflicts; at 4 bits an entry is the byte's two levels,
 *     packed as the MMA wants them; at 8 bits the level twice), and the 16 packed words go out with one tcgen05.st — so
 *     the matrix's expanded rows never pass through the shared-memory pipe, which is what a block runs out of;
 *   · the codes reach their row's owner through a small padded ring in shared memory, copied two stages ahead by cp.async
 *     with the threads laid along a row (whole lines from DRAM); the pairs' rows of x are gathered as the B operand
 *     (K-major, 128-byte swizzle) by cp.async one stage ahead;
 *   · one thread issues tcgen05.mma with A in tensor memory (M 128, N = the pairs rounded up to 16, K 16 a step, eight a
 *     stage), accumulating in tensor memory, and gives a stage back to the producers by a commit on its mbarrier;
 *   · the producers then read the accumulator out of tensor memory, scale a row by its fp16 scale, round once and store —
 *     or, for expert_rows_sum, add weight · value onto the fp32 running sum.
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

constexpr int EX_THREADS = 544, EX_PRODUCERS = 512, EX_BM = 128, EX_BN = 128, EX_KC = 64;
constexpr int EX_STAGES = 3;                                          /* stages of two column blocks; the copies of x run one ahead */
constexpr uint32_t EX_ATOM = 16384;                                   /* a tile of 128 rows x 64 columns of halves, 128-byte rows, swizzled */
constexpr uint32_t EX_STAGE_BYTES = 2 * EX_ATOM;                      /* a stage's x: two column blocks (the matrix's rows live in tensor memory) */
constexpr uint32_t EX_RAWS = 4, EX_RAW_PITCH4 = 80, EX_RAW_PITCH8 = 144, EX_RAW_BYTES = 128 * EX_RAW_PITCH8;   /* a stage's codes as they lie in memory, rows padded apart */
constexpr uint32_t EX_T_ACC = 0, EX_T_A = 128, EX_T_A_STAGE = 64, EX_T_COLS = 512;   /* tensor memory: the sums, then a stage's A operand, 64 packed columns each */
constexpr uint32_t EX_LUT_BYTES = 256 * 128;
constexpr uint32_t EX_SMEM_BYTES = 1024 + EX_LUT_BYTES + EX_STAGES * EX_STAGE_BYTES + EX_RAWS * EX_RAW_BYTES + 2 * EX_BN * 4 + 256;

struct ExpertFast {
    const uint8_t* codes[12];
    const uint16_t* scales[12];
    uint32_t out_rows[12], held[12], d[12], pairs_at[12], pairs[12], tile0[13];   /* group i's blocks of 128 rows are [tile0[i], tile0[i+1]) */
    uint64_t out_at[12];
    uint32_t count, cols;
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
/* A spinning wait (test_wait, no suspension) for the one thread whose wake-up latency is the whole pipeline's: bounded like mbar_wait. */
__device__ __forceinline__ bool ex_spin_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, unsigned int* status) {
    for (uint32_t i = 0; i < (SV_WAIT_TRIES << 4); ++i) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
        if (done) return true;
        if ((i & 1023u) == 1023u && *abort_flag != 0u) return false;
    }
    *abort_flag = 1u;
    if (status) atomicOr(status, SV_STATUS_TIMEOUT);
    return false;
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
    const uint32_t lut_at = base, stage_at = lut_at + EX_LUT_BYTES, raw_at = stage_at + EX_STAGES * EX_STAGE_BYTES;
    uint32_t* xrow_s = reinterpret_cast<uint32_t*>(smem + EX_LUT_BYTES + EX_STAGES * EX_STAGE_BYTES + EX_RAWS * EX_RAW_BYTES);
    uint32_t* orow_s = xrow_s + EX_BN;
    uint64_t* full = reinterpret_cast<uint64_t*>(orow_s + EX_BN);
    uint64_t* empty = full + EX_STAGES;
    uint64_t* acc_full = empty + EX_STAGES;
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
        for (int s = 0; s < EX_STAGES; ++s) { mbar_init(&full[s], EX_PRODUCERS / 32); mbar_init(&empty[s], 1); }
        mbar_init(acc_full, 1);
        *abort_flag = 0u;
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, EX_T_COLS);
    else {
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
                if (!ex_spin_wait(&full[s], ph, abort_flag, a.status)) break;
                tc_fence_after();
                const uint32_t blocks = min(2u, nk - 2u * st);
                for (uint32_t h = 0; h < blocks; ++h) {                        /* A: this stage's rows in tensor memory, 8 packed columns a step of 16 */
                    const uint64_t bd = smem_desc_sw128(stage_at + s * EX_STAGE_BYTES + h * EX_ATOM, 16, 1024);
                    const uint32_t at = tmem + EX_T_A + s * EX_T_A_STAGE + h * 32u;
#pragma unroll
                    for (uint32_t kk = 0; kk < 4; ++kk) tc_mma_ts(tmem + EX_T_ACC, at + kk * 8u, bd + kk * 2u, idesc, (st | h | kk) != 0u ? 1u : 0u);
                }
                tc_commit(&empty[s]);
                if (++s == (uint32_t)EX_STAGES) { s = 0; ph ^= 1u; }
            }
            tc_commit(acc_full);
        }
    } else {
        /* ---------------- producers: codes -> the A operand in tensor memory, the pairs' rows of x -> B tiles; then the read-out ----
         * A stage is TWO column blocks (128 columns): a hand-over between the producers and the issuing thread — the wait, the
         * fences, the arrivals, the commit — costs a few hundred cycles on either side whatever hangs on it, so it is paid once a
         * 128 columns.  The shared-memory pipe is what a block runs out of (tiles stored, copied and read by the MMA all pass
         * through it), so the matrix's expanded rows never touch it: a thread owns ONE matrix row (its lane of tensor memory; a
         * warp its quadrant's 32 rows) and 32 of the stage's columns (the four warps of a quadrant a quarter each), looks its
         * codes up — a 4-bit byte's entry is already two neighbouring halves packed as the MMA wants them — and stores the 16
         * packed words with one tcgen05.st; the MMA takes A from tensor memory and only x from shared memory.
         * The codes come through a small ring as they lie in memory: copied two stages ahead by cp.async with the threads laid
         * along a row (a row's 64 or 128 bytes of a stage in one go: whole lines from DRAM), read back by the row's owner
         * (rows padded apart, so neither side meets a bank conflict).  A slot is written again four stages later, after a wait
         * every thread makes first: for the release of the x slot of three stages ago, which every warp's hand-over preceded.
         * A thread also copies up to four 16-byte pieces of the x tiles (one chunk column, rows 32 apart) one stage ahead. */
        const int p = tid - 32;
        const uint32_t quad = (uint32_t)warp & 3u, part = (uint32_t)(warp - 1) >> 2, row = quad * 32u + (uint32_t)lane;
        const bool own_ok = r0 + row < held && r0 + row < out_rows;          /* the row this thread expands */
        const uint32_t code_step = d == 4u ? 64u : d == 8u ? 128u : 256u;    /* bytes of a row a stage covers */
        const uint32_t pitch = d == 4u ? EX_RAW_PITCH4 : EX_RAW_PITCH8;
        /* the copying side: thread p takes 16 bytes of row p / 4 (4 bits) or 32 bytes of it (8 bits) */
        const uint32_t c_row = (uint32_t)p >> 2, c_q = (uint32_t)p & 3u, c_bytes = d == 4u ? 16u : 32u;
        const bool c_ok = r0 + c_row < held && r0 + c_row < out_rows;
        const uint8_t* c_src = a.codes[g] + (c_ok ? (uint64_t)(r0 + c_row) * row_bytes : 0ull) + c_q * c_bytes;
        const uint32_t c_dst = raw_at + c_row * pitch + c_q * c_bytes;
        const uint32_t my_raw = raw_at + row * pitch + part * (code_step / 4u);   /* the reading side: this thread's 32 columns of its row */
        const uint8_t* my_halves = a.codes[g] + (own_ok ? (uint64_t)(r0 + row) * row_bytes : 0ull) + part * 64u;   /* (16 bits: read straight from memory) */
        const uint32_t lane_lut = lut_at + (uint32_t)lane * 4u;
        const uint32_t my_tile = part >> 1;                                  /* which of the stage's two column blocks this thread's columns are in */
        const uint32_t a_at = tmem + EX_T_A + part * 16u + ((quad * 32u) << 16);   /* + the slot's 64 columns */
        const uint32_t xc = (uint32_t)p & 15u, xj = (uint32_t)p >> 4;        /* this thread's chunk column of the stage's 16; its first row of the x tiles */
        const uint32_t x_tile = xc >> 3;
        const uint16_t* x_src[4];
        uint32_t x_bytes[4];
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
            const uint32_t j = xj + 32u * i;
            x_src[i] = a.x + (uint64_t)xrow_s[j] * cols + xc * 8u;
            x_bytes[i] = j < nb ? 16u : 0u;
        }
        const uint32_t x_off = x_tile * EX_ATOM + swz128(xj, xc & 7u), x_count = N / 32u + ((N & 31u) > xj ? 1u : 0u);
        bool ok = true;
        uint32_t s_iss = 0, ph_iss = 1, st_iss = 0;                           /* the next stage of x to ask for: its slot, the parity of the slot's last release */
        uint32_t s = 0;                                                       /* the slot of the stage being expanded */
        /* whether column block `tile` of stage `st` exists (the last stage of an odd count of blocks has one) */
        auto has = [&](uint32_t st, uint32_t tile) { return 2u * st + tile < nk; };

        auto issue_x = [&]() {                                                /* x of the next stage, once the MMAs that read the slot have completed */
            if (st_iss >= (uint32_t)EX_STAGES && ok) ok = mbar_wait(&empty[s_iss], ph_iss, abort_flag, a.status);
            if (ok && has(st_iss, x_tile)) {
                const uint32_t at = stage_at + s_iss * EX_STAGE_BYTES;
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i)
                    if (i < x_count) ex_cp16(at + x_off + i * 4096u, x_src[i], x_bytes[i]);
            }
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) x_src[i] += 2 * EX_KC;
            ++st_iss;
            if (++s_iss == (uint32_t)EX_STAGES) { s_iss = 0; ph_iss ^= 1u; }
        };
        auto issue_codes = [&](uint32_t st) {                                 /* stage st's codes into the ring (nothing at 16 bits, nothing past the end) */
            if (d == 16u || st >= nst || !ok) return;
            const uint32_t to = c_dst + (st & (EX_RAWS - 1u)) * EX_RAW_BYTES, bytes = c_ok ? 16u : 0u;
            const uint8_t* from = c_src + (uint64_t)st * code_step;
            /* (the second column block of an odd last stage lies past the row's end: the upper half of the stage's bytes is not read) */
            const bool second = has(st, 1u);
            if (d == 4u) { if (second || c_q < 2u) ex_cp16(to, from, bytes); }
            else if (second || c_q < 2u) { ex_cp16(to, from, bytes); ex_cp16(to + 16u, from + 16, bytes); }
        };
        /* the stage's x of this thread has landed, its row of A is in tensor memory: the slot goes to the issuing thread */
        auto hand_over = [&]() {
            fence_proxy_async_smem();                                        /* the landed copies of x, for the MMA's reads */
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[s]);
            if (++s == (uint32_t)EX_STAGES) s = 0;
        };

        issue_codes(0u);
        if (nst > 0u) issue_x();
        ex_cp_commit();
        issue_codes(1u);
        ex_cp_commit();
        for (uint32_t st = 0; st < nst && ok; ++st) {
            if (st + 1u < nst) issue_x();                                    /* (waits for the release of stage st - 2's slot: every warp has handed st - 2 over) */
            issue_codes(st + 2u);                                            /* over the codes of stage st - 2 */
            ex_cp_commit();                                                  /* (an empty group past the end keeps the count below uniform) */
            ex_cp_wait<1>();                                                 /* this thread's copies for stage st — its x, and its share of the codes — have landed */
            /* the producers meet: every thread's share of the stage's codes has landed — and a thread whose wait ran out takes
             * all of them out together, so nobody is left at this barrier */
            {
                uint32_t any;
                asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbarrier.cta.red.or.pred p, 1, %2, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                             : "=r"(any) : "r"(ok ? 0u : 1u), "n"(EX_PRODUCERS) : "memory");
                if (any) { ok = false; break; }
            }
            uint32_t words[16];                                              /* 32 columns of this row: 16 words of two halves */
            if (d == 16u) {
#pragma unroll
                for (uint32_t i = 0; i < 16; ++i) words[i] = 0u;
                if (own_ok && has(st, my_tile)) {
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        const uint4 v = ex_ldg128(my_halves + (uint64_t)st * code_step + i * 16u);
                        words[4 * i] = v.x; words[4 * i + 1] = v.y; words[4 * i + 2] = v.z; words[4 * i + 3] = v.w;
                    }
                }
            } else {
                const uint32_t raw = my_raw + (st & (EX_RAWS - 1u)) * EX_RAW_BYTES;
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
            tmem_st16(a_at + s * EX_T_A_STAGE, words);
            hand_over();
        }
        ex_cp_wait<0>();

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
    a.count = (uint32_t)g.count; a.cols = (uint32_t)cols; a.x = x; a.rows = rows; a.w = w; a.out = out; a.acc = acc; a.over = over;
    a.status = device_status_word();
    static std::atomic<bool> ready[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!ready[dev].load(std::memory_order_acquire)) {
        e = cudaFuncSetAttribute(expert_fast_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)EX_SMEM_BYTES);
        if (e != cudaSuccess) return e;
        ready[dev].store(true, std::memory_order_release);
    }
    const dim3 grid(tiles, (widest + EX_BN - 1) / EX_BN);
    expert_fast_kernel<<<grid, EX_THREADS, EX_SMEM_BYTES, st>>>(a);
    note_launch(1);
    return cudaGetLastError();
}

}  // namespace sv
