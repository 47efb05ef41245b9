/* tq.cu — the TurboQuant-coded tiers of the KV cache: rotation, encoding, decoding, and attention over coded rows.
 *
 * The reference keeps a head's key and value rotated (R·k, R·v with R a signed Hadamard rotation over the head's width,
 * so q·k = (R·q)·(R·k)) and, as positions age, re-codes the rotated rows at 8 and then 4 bits an element
 * (engine/src/packages/nn/gpu/kernels/kernels.cuh:2819-2826).  A coded row is `head_dim` codes packed into 16-bit
 * containers (16/width codes a container, code s at bits width·s, little-endian bytes) plus ONE fp16 scale; an element
 * is `scale · level[code]` with the fixed level tables of tq_levels.inc (:2650-2653, :2897-2901).  The doors answered
 * here (engine/src/packages/nn/contracts/abi/gpu.cuh:161-164, 197-198 and the decode row):
 *     hadamard_blocks            R or R^T over blocks of a power of two                      (kernels.cuh:2829-2855)
 *     turboquant_encode_rows     rotated rows -> codes + scale (scale = fp16(clip · rms))     (:2886-2931)
 *     turboquant_decode          codes + scales -> halves                                     (:1281-1298)
 *     attention_weights_tq       a residual's first pass over coded keys                      (:2904-2961)
 *     attention_residual_mix_tq  its second pass over coded values                            (:2967-2986)
 *     ..._tq_rows                the same a row of a prompt chunk at a time                   (nn/gpu/doors.cuh:433-450)
 * This file holds the doors AS WORDED — any shape, any alignment, the reference's order of operations — and the table.
 * The fast path (one fused kernel for the weights/mix pair, codes expanded in flight) is tq_decode.cu. */
#include "common.cuh"
#include "kernels.h"
#include <string.h>

namespace sv {

__device__ const uint16_t g_tq_levels[318] = {
#include "tq_levels.inc"
};

__host__ __device__ __forceinline__ bool tq_width_known(uint64_t d) { return d == 1 || d == 2 || d == 3 || d == 4 || d == 5 || d == 8 || d == 16; }
__host__ __device__ __forceinline__ uint32_t tq_table_at(uint64_t d) { return d == 1 ? 0u : d == 2 ? 2u : d == 3 ? 6u : d == 4 ? 14u : d == 5 ? 30u : 62u; }
__host__ __device__ __forceinline__ uint64_t tq_row_bytes(uint64_t d, uint64_t cols) { const uint64_t per = 16 / d; return ((cols + per - 1) / per) * 2; }

using H = Elem<SV_DTYPE_FP16>;

__device__ __forceinline__ float tq_level(uint64_t d, uint32_t code) {
    return d == 16 ? H::to_float((uint16_t)code) : H::to_float(g_tq_levels[tq_table_at(d) + code]);
}
__device__ __forceinline__ uint32_t tq_code(const uint8_t* row, uint64_t d, uint64_t c) {
    const uint64_t per = 16 / d;
    const uint32_t unit = (uint32_t)row[(c / per) * 2] | ((uint32_t)row[(c / per) * 2 + 1] << 8);
    return (unit >> (uint32_t)(d * (c % per))) & ((1u << (uint32_t)d) - 1u);
}
__device__ __forceinline__ float tq_element(const uint8_t* row, float scale, uint64_t d, uint64_t c) {
    return scale * tq_level(d, tq_code(row, d, c));
}

/* ---- turboquant_decode: element (r, c) of a coded matrix as a half; a row its room does not hold is skipped -------- */
__global__ void __launch_bounds__(256) tq_decode_kernel(uint16_t* out, const uint8_t* weights, uint64_t w_room, const uint8_t* luts,
                                                        uint64_t l_room, uint64_t d, uint64_t rows, uint64_t cols, unsigned int* over) {
    const uint64_t n = rows * cols, need = tq_row_bytes(d, cols);
    bool hit = false;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t r = i / cols, c = i - r * cols;
        if (need == 0 || need > w_room || r + 1 > w_room / need) continue;
        float scale = 1.0f;
        if (d != 16) {
            if (l_room < 2 || r + 1 > l_room / 2) continue;
            scale = H::to_float((uint16_t)((uint32_t)luts[r * 2] | ((uint32_t)luts[r * 2 + 1] << 8)));
        }
        const float lv = tq_level(d, tq_code(weights + r * need, d, c));
        out[i] = H::from_float(d == 16 ? lv : lv * scale, hit);
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* ---- hadamard_blocks: out = R·in (inverse 0: H·(S ⊙ u)) or R^T·in (inverse 1: S ⊙ H·u) per block; sums in the reference's
 * order (even and odd columns apart, ascending), so the halves that come out are the reference's bit for bit ---------- */
__global__ void __launch_bounds__(256) hadamard_blocks_kernel(uint16_t* out, const uint16_t* in, const uint16_t* sign, uint64_t n,
                                                              uint64_t block, uint64_t inverse, unsigned int* over) {
    const float norm = 1.0f / sqrtf((float)(uint32_t)block);
    bool hit = false;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t a = i - i % block, r = i - a;
        float s0 = 0.f, s1 = 0.f;
        for (uint64_t c = 0; c < block; c += 2) {
            float v0 = H::to_float(in[a + c]), v1 = H::to_float(in[a + c + 1]);
            if (inverse == 0) { v0 *= H::to_float(sign[c]); v1 *= H::to_float(sign[c + 1]); }
            s0 += (__popcll(r & c) & 1) ? -v0 : v0;
            s1 += (__popcll(r & (c + 1)) & 1) ? -v1 : v1;
        }
        float sum = (s0 + s1) * norm;
        if (inverse != 0) sum *= H::to_float(sign[r]);
        out[i] = H::from_float(sum, hit);
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* ---- turboquant_encode_rows: a block a row ------------------------------------------------------------------------ */
#define SV_TQ_CLIP_4 2.7325895709952577f        /* the codec's clip for a width: a row's scale is fp16(clip · rms) */
#define SV_TQ_CLIP_8 4.6036453045214065f
#define SV_TQ_FP16_MIN_NORMAL 6.103515625e-05f

/* how many of the level table's midpoints lie below v */
__device__ __forceinline__ uint32_t tq_nearest(uint64_t d, float v) {
    uint32_t lo = 0u, hi = (1u << (uint32_t)d) - 1u;
    while (lo < hi) {
        const uint32_t mid = (lo + hi) >> 1;
        const float m = 0.5f * (tq_level(d, mid) + tq_level(d, mid + 1u));
        if (m < v) lo = mid + 1u; else hi = mid;
    }
    return lo;
}

__global__ void __launch_bounds__(128) tq_encode_rows_kernel(uint8_t* codes, uint16_t* scales, const uint16_t* x, uint64_t rows,
                                                             uint64_t cols, uint64_t d, unsigned int* over) {
    __shared__ double part_s[4];
    __shared__ float scale_s;
    __shared__ uint16_t sh_s;
    const uint64_t per = 16 / d, row_bytes = tq_row_bytes(d, cols), units = row_bytes / 2;
    const float clip = d == 4 ? SV_TQ_CLIP_4 : SV_TQ_CLIP_8;
    bool hit = false;
    for (uint64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const uint16_t* xr = x + r * cols;
        /* the row's sum of squares in double: the reference adds it in fp32 in one order, this in another, and the nearer
         * both are to the exact sum the rarer a scale that rounds to the other side of an fp16 step */
        double part = 0.0;
        for (uint64_t c = threadIdx.x; c < cols; c += blockDim.x) { const double v = (double)H::to_float(xr[c]); part += v * v; }
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        if ((threadIdx.x & 31) == 0) part_s[threadIdx.x >> 5] = part;
        __syncthreads();
        if (threadIdx.x == 0) {
            const float sumsq = (float)(part_s[0] + part_s[1] + part_s[2] + part_s[3]);
            const float rms = sqrtf(sumsq / (float)cols);
            uint16_t sh = H::from_float(clip * rms, hit);
            float scale = H::to_float(sh);
            if (scale < SV_TQ_FP16_MIN_NORMAL) { sh = 0u; scale = 0.f; }       /* a dead row is stored as zeros */
            scales[r] = sh; sh_s = sh; scale_s = scale;
        }
        __syncthreads();
        const float scale = scale_s;
        const bool dead = sh_s == 0u;
        uint8_t* cr = codes + r * row_bytes;
        for (uint64_t u = threadIdx.x; u < units; u += blockDim.x) {
            uint32_t unit = 0u;
            for (uint64_t s = 0; s < per; ++s) {
                const uint64_t c = u * per + s;
                if (c >= cols || dead) continue;
                unit |= tq_nearest(d, H::to_float(xr[c]) / scale) << (uint32_t)(d * s);
            }
            cr[u * 2] = (uint8_t)(unit & 0xffu);
            cr[u * 2 + 1] = (uint8_t)((unit >> 8) & 0xffu);
        }
        __syncthreads();
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* ---- attention_weights_tq[_rows]: a block a (row, head): p[t] = e^(s_t - top), res = (top, sum) -------------------- */
__device__ __forceinline__ float block_max(float v, float* sh) {
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float m = sh[0];
    for (unsigned w = 1; w < blockDim.x / 32; ++w) m = fmaxf(m, sh[w]);
    __syncthreads();
    return m;
}
__device__ __forceinline__ float block_sum(float v, float* sh) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.f;
    for (unsigned w = 0; w < blockDim.x / 32; ++w) s += sh[w];
    __syncthreads();
    return s;
}

__global__ void __launch_bounds__(256) tq_weights_kernel(float* p, float* res, const uint16_t* q, const uint8_t* codes, const uint16_t* scales,
                                                         uint64_t qh, uint64_t kvh, uint64_t d_head, uint64_t length, uint64_t d, uint64_t rows) {
    extern __shared__ float qs[];                  /* the head's query as floats */
    __shared__ float sh[8];
    const uint64_t group = qh / kvh, row_bytes = tq_row_bytes(d, d_head);
    const float inv = 1.0f / sqrtf((float)(uint32_t)d_head);
    for (uint64_t i = blockIdx.x; i < rows * qh; i += gridDim.x) {
        const uint64_t h = i % qh, g = h / group;
        float* ph = p + i * length;
        for (uint64_t e = threadIdx.x; e < d_head; e += blockDim.x) qs[e] = H::to_float(q[i * d_head + e]);
        __syncthreads();
        float top = -INFINITY;
        for (uint64_t t = threadIdx.x; t < length; t += blockDim.x) {
            const uint64_t row = t * kvh + g;
            const uint8_t* kr = codes + row * row_bytes;
            const float scale = H::to_float(scales[row]);
            float dot = 0.f;
            for (uint64_t e = 0; e < d_head; ++e) dot += qs[e] * tq_element(kr, scale, d, e);
            const float s = dot * inv;
            ph[t] = s;
            top = fmaxf(top, s);
        }
        top = block_max(top, sh);
        float part = 0.f;
        for (uint64_t t = threadIdx.x; t < length; t += blockDim.x) { const float w = expf(ph[t] - top); ph[t] = w; part += w; }
        const float sum = block_sum(part, sh);
        if (threadIdx.x == 0) { res[i * (d_head + 2)] = top; res[i * (d_head + 2) + 1] = sum; }
        __syncthreads();
    }
}

/* ---- attention_residual_mix_tq[_rows]: a block a (row, head), a thread an element, positions in order ---------------- */
__global__ void __launch_bounds__(256) tq_residual_mix_kernel(float* res, const float* p, const uint8_t* codes, const uint16_t* scales,
                                                              uint64_t qh, uint64_t kvh, uint64_t d_head, uint64_t length, uint64_t d, uint64_t rows) {
    const uint64_t group = qh / kvh, row_bytes = tq_row_bytes(d, d_head);
    for (uint64_t i = blockIdx.x; i < rows * qh; i += gridDim.x) {
        const uint64_t h = i % qh, g = h / group;
        const float* ph = p + i * length;
        for (uint64_t e = threadIdx.x; e < d_head; e += blockDim.x) {
            float sum = 0.f;
            for (uint64_t t = 0; t < length; ++t) {
                const uint64_t row = t * kvh + g;
                sum += ph[t] * tq_element(codes + row * row_bytes, H::to_float(scales[row]), d, e);
            }
            res[i * (d_head + 2) + 2 + e] = sum;
        }
    }
}

/* ---- the weight path's three doors a mixer cannot run without, AS WORDED (block a row; not a fast path) -------------
 * hadamard_rotate (kernels.cuh:2189-2231): the rotation over a row of n in blocks of 512, then a 256 and a 128 for what
 * is left (a row shorter than 512 is one block); a lane an output, four running sums as the reference adds them.
 * turboquant_gemv (:1405-1447): out[r] = half(scale_r · sum_c level(code[r][c]) · x[c]), a row its room does not hold
 * skipped.  turboquant_gemv_groups (:1453-1461): the gemv once a group over one shared x. */
__global__ void __launch_bounds__(256) hadamard_rotate_kernel(uint16_t* out, const uint16_t* in, const uint16_t* sign, uint64_t n, unsigned int* over) {
    const uint64_t whole = n < 512 ? 0 : (n / 512) * 512, rest = n - whole;
    bool hit = false;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t a = 0, b = n;
        if (i < whole) { a = i - i % 512; b = 512; }
        else if (whole != 0) {
            if (rest >= 256 && i < whole + 256) { a = whole; b = 256; }
            else { a = whole + (rest >= 256 ? 256 : 0); b = 128; }
        }
        const uint64_t r = i - a;
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        uint64_t c = 0;
        for (; c + 4 <= b; c += 4)
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const float v = H::to_float(in[a + c + x]) * H::to_float(sign[c + x]);
                s[x] += (__popcll(r & (c + x)) & 1) ? -v : v;
            }
        for (; c < b; ++c) { const float v = H::to_float(in[a + c]) * H::to_float(sign[c]); s[0] += (__popcll(r & c) & 1) ? -v : v; }
        out[i] = H::from_float(((s[0] + s[1]) + (s[2] + s[3])) / sqrtf((float)b), hit);
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* rmsnorm_rotate (the norm of a row, then its rotation: nn's definition is the two doors one after the other) as ONE kernel: a
 * block a rotation block of the row.  Every block folds the whole row's sum of squares itself, with the norm door's own block
 * size and order (so the scale has the norm door's bits), norms its block into shared memory and `o`, and rotates it with the
 * rotation door's four running sums. */
__global__ void __launch_bounds__(256) rmsnorm_rotate_kernel(uint16_t* rot, uint16_t* o, const uint16_t* x, const uint16_t* w, const uint16_t* sign, uint64_t n,
                                                             float eps, unsigned int* over) {
    __shared__ float sh[8];
    __shared__ uint16_t seg[512];
    bool hit = false;
    float part = 0.f;
    for (uint64_t i = threadIdx.x; i < n; i += blockDim.x) { const float v = H::to_float(x[i]); part += v * v; }
    for (int s = 16; s > 0; s >>= 1) part += __shfl_xor_sync(0xffffffffu, part, s);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = part;
    __syncthreads();
    float sum = 0.f;
    for (unsigned k = 0; k < blockDim.x / 32; ++k) sum += sh[k];
    const float scale = 1.0f / sqrtf(sum / (float)n + eps);
    /* this block's rotation block [a, a + b): the whole 512s, then a 256 and a 128 of what is left; a row under 512 is one block */
    const uint64_t whole = n < 512 ? 0 : (n / 512) * 512, rest = n - whole;
    uint64_t a = 0, b = n;
    if (n >= 512) {
        if (blockIdx.x < whole / 512) { a = (uint64_t)blockIdx.x * 512; b = 512; }
        else if (blockIdx.x == whole / 512 && rest >= 256) { a = whole; b = 256; }
        else { a = whole + (rest >= 256 ? 256 : 0); b = 128; }
    }
    for (uint64_t i = threadIdx.x; i < b; i += blockDim.x) {
        const uint16_t h = H::from_float((H::to_float(x[a + i]) * scale) * H::to_float(w[a + i]), hit);
        seg[i] = h;
        o[a + i] = h;
    }
    __syncthreads();
    for (uint64_t r = threadIdx.x; r < b; r += blockDim.x) {
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        uint64_t c = 0;
        for (; c + 4 <= b; c += 4)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float v = H::to_float(seg[c + q]) * H::to_float(sign[c + q]);
                s[q] += (__popcll(r & (c + q)) & 1) ? -v : v;
            }
        for (; c < b; ++c) { const float v = H::to_float(seg[c]) * H::to_float(sign[c]); s[0] += (__popcll(r & c) & 1) ? -v : v; }
        rot[a + r] = H::from_float(((s[0] + s[1]) + (s[2] + s[3])) / sqrtf((float)b), hit);
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* attention_gate_rows followed by hadamard_rotate over the gated answers, as ONE kernel: a block a rotation block — the gate door's
 * arithmetic element for element into shared memory and `o`, then the rotation door's four running sums over those halves. */
__global__ void __launch_bounds__(256) gate_rotate_kernel(uint16_t* rot, uint16_t* o, const uint16_t* att, const uint16_t* qg, const uint16_t* sign,
                                                          uint64_t heads, uint64_t head_dim, unsigned int* over) {
    __shared__ uint16_t seg[512];
    bool hit = false;
    const uint64_t n = heads * head_dim, whole = n < 512 ? 0 : (n / 512) * 512, rest = n - whole;
    uint64_t a = 0, b = n;
    if (n >= 512) {
        if (blockIdx.x < whole / 512) { a = (uint64_t)blockIdx.x * 512; b = 512; }
        else if (blockIdx.x == whole / 512 && rest >= 256) { a = whole; b = 256; }
        else { a = whole + (rest >= 256 ? 256 : 0); b = 128; }
    }
    for (uint64_t k = threadIdx.x; k < b; k += blockDim.x) {
        const uint64_t i = a + k, h = i / head_dim, e = i - h * head_dim;
        const float v = H::to_float(qg[h * 2 * head_dim + head_dim + e]);
        const uint16_t gate = H::from_float(1.0f / (1.0f + expf(-v)), hit);
        const uint16_t y = H::from_float(H::to_float(att[i]) * H::to_float(gate), hit);
        seg[k] = y;
        o[i] = y;
    }
    __syncthreads();
    for (uint64_t r = threadIdx.x; r < b; r += blockDim.x) {
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        uint64_t c = 0;
        for (; c + 4 <= b; c += 4)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float v = H::to_float(seg[c + q]) * H::to_float(sign[c + q]);
                s[q] += (__popcll(r & (c + q)) & 1) ? -v : v;
            }
        for (; c < b; ++c) { const float v = H::to_float(seg[c]) * H::to_float(sign[c]); s[0] += (__popcll(r & c) & 1) ? -v : v; }
        rot[a + r] = H::from_float(((s[0] + s[1]) + (s[2] + s[3])) / sqrtf((float)b), hit);
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

struct GemvGroups { uint64_t codes[12], luts[12], rows[12], d[12], out_at[12], count; };

__global__ void __launch_bounds__(128) tq_gemv_groups_kernel(uint16_t* out, GemvGroups g, uint64_t w_room0, uint64_t l_room0, const uint16_t* x,
                                                             uint64_t cols, unsigned int* over) {
    __shared__ float sh[4];
    bool hit = false;
    uint64_t row0 = 0;
    for (uint64_t i = 0; i < g.count && i < 12; ++i) {
        const uint64_t d = g.d[i], per = 16 / d, row_bytes = tq_row_bytes(d, cols), units = (cols + per - 1) / per;
        const uint8_t* weights = (const uint8_t*)g.codes[i];
        const uint8_t* luts = (const uint8_t*)g.luts[i];
        const uint64_t w_room = g.count == 1 && w_room0 ? w_room0 : g.rows[i] * row_bytes, l_room = g.count == 1 && l_room0 ? l_room0 : g.rows[i] * 2;
        const uint64_t rows_held = row_bytes == 0 ? 0 : w_room / row_bytes, scales_held = l_room / 2;
        const uint32_t mask = (uint32_t)((1ull << d) - 1ull);
        for (uint64_t r = blockIdx.x; r < g.rows[i]; r += gridDim.x) {
            if (r >= rows_held || (d != 16 && r >= scales_held)) continue;        /* the whole block skips it together */
            const uint8_t* row = weights + r * row_bytes;
            float part = 0.f;
            for (uint64_t u = threadIdx.x; u < units; u += blockDim.x) {
                const uint32_t unit = (uint32_t)row[u * 2] | ((uint32_t)row[u * 2 + 1] << 8);
                const uint64_t c0 = u * per;
                for (uint64_t s = 0; s < per && c0 + s < cols; ++s) part += tq_level(d, (unit >> (uint32_t)(d * s)) & mask) * H::to_float(x[c0 + s]);
            }
            for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = part;
            __syncthreads();
            if (threadIdx.x == 0) {
                const float scale = d == 16 ? 1.0f : H::to_float((uint16_t)((uint32_t)luts[r * 2] | ((uint32_t)luts[r * 2 + 1] << 8)));
                out[g.out_at[i] + r] = H::from_float(((sh[0] + sh[1]) + (sh[2] + sh[3])) * scale, hit);
            }
            __syncthreads();
        }
        row0 += g.rows[i];
    }
    (void)row0;
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* ---------------------------------------------------------------------------------------------------------- */

static inline unsigned tq_grid(uint64_t items, unsigned cap = 4096u) { return (unsigned)(items < 1 ? 1 : (items > cap ? cap : items)); }

bool tq_width_ok(uint64_t d) { return tq_width_known(d); }

cudaError_t tq_decode_launch(uint16_t* out, const uint8_t* weights, uint64_t w_room, const uint8_t* luts, uint64_t l_room, uint64_t d,
                             uint64_t rows, uint64_t cols, unsigned int* over, cudaStream_t st) {
    tq_decode_kernel<<<tq_grid((rows * cols + 255) / 256), 256, 0, st>>>(out, weights, w_room, luts, l_room, d, rows, cols, over);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t hadamard_blocks_launch(uint16_t* out, const uint16_t* in, const uint16_t* sign, uint64_t n, uint64_t block, uint64_t inverse,
                                   unsigned int* over, cudaStream_t st) {
    hadamard_blocks_kernel<<<tq_grid((n + 255) / 256), 256, 0, st>>>(out, in, sign, n, block, inverse, over);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t tq_encode_rows_launch(uint8_t* codes, uint16_t* scales, const uint16_t* x, uint64_t rows, uint64_t cols, uint64_t d,
                                  unsigned int* over, cudaStream_t st) {
    tq_encode_rows_kernel<<<tq_grid(rows, 65535u), 128, 0, st>>>(codes, scales, x, rows, cols, d, over);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t tq_weights_launch(float* p, float* res, const uint16_t* q, const uint8_t* codes, const uint16_t* scales, uint64_t qh, uint64_t kvh,
                              uint64_t d_head, uint64_t length, uint64_t d, uint64_t rows, cudaStream_t st) {
    if (d_head * sizeof(float) > 48 * 1024) return cudaErrorInvalidValue;
    tq_weights_kernel<<<tq_grid(rows * qh), 256, d_head * sizeof(float), st>>>(p, res, q, codes, scales, qh, kvh, d_head, length, d, rows);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t tq_residual_mix_launch(float* res, const float* p, const uint8_t* codes, const uint16_t* scales, uint64_t qh, uint64_t kvh,
                                   uint64_t d_head, uint64_t length, uint64_t d, uint64_t rows, cudaStream_t st) {
    const unsigned threads = d_head >= 256 ? 256u : (d_head >= 128 ? 128u : 64u);
    tq_residual_mix_kernel<<<tq_grid(rows * qh), threads, 0, st>>>(res, p, codes, scales, qh, kvh, d_head, length, d, rows);
    note_launch(1);
    return cudaGetLastError();
}

/* n as the rotation door takes it: under 512, or what is left after the whole 512s is 0, 128, 256 or 384 */
cudaError_t rmsnorm_rotate_launch(uint16_t* rot, uint16_t* o, const uint16_t* x, const uint16_t* w, const uint16_t* sign, uint64_t n, float eps,
                                  unsigned int* over, cudaStream_t st) {
    if (n == 0 || (n >= 512 && (n % 512) % 128 != 0)) return cudaErrorInvalidValue;
    const uint64_t rest = n % 512;
    const unsigned blocks = n < 512 ? 1u : (unsigned)(n / 512 + (rest >= 256 ? 1 : 0) + ((rest % 256) >= 128 ? 1 : 0));
    const unsigned threads = n >= 2048 ? 256u : (n >= 512 ? 128u : 64u);   /* the norm door's own block: the same partial sums in the same order */
    rmsnorm_rotate_kernel<<<blocks, threads, 0, st>>>(rot, o, x, w, sign, n, eps, over);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t gate_rotate_launch(uint16_t* rot, uint16_t* o, const uint16_t* att, const uint16_t* qg, const uint16_t* sign, uint64_t heads, uint64_t head_dim,
                               unsigned int* over, cudaStream_t st) {
    const uint64_t n = heads * head_dim;
    if (n == 0 || (n >= 512 && (n % 512) % 128 != 0)) return cudaErrorInvalidValue;
    const uint64_t rest = n % 512;
    const unsigned blocks = n < 512 ? 1u : (unsigned)(n / 512 + (rest >= 256 ? 1 : 0) + ((rest % 256) >= 128 ? 1 : 0));
    gate_rotate_kernel<<<blocks, 256, 0, st>>>(rot, o, att, qg, sign, heads, head_dim, over);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t hadamard_rotate_launch(uint16_t* out, const uint16_t* in, const uint16_t* sign, uint64_t n, unsigned int* over, cudaStream_t st) {
    hadamard_rotate_kernel<<<tq_grid((n + 255) / 256), 256, 0, st>>>(out, in, sign, n, over);
    note_launch(1);
    return cudaGetLastError();
}
/* `g` is the by-value groups struct of the door (codes, luts, rows, d, out_at a group, then the count); one group with the
 * rooms given is turboquant_gemv itself */
cudaError_t tq_gemv_groups_launch(uint16_t* out, const void* g, uint64_t w_room, uint64_t l_room, const uint16_t* x, uint64_t cols,
                                  unsigned int* over, cudaStream_t st) {
    GemvGroups gg;
    memcpy(&gg, g, sizeof gg);
    uint64_t most = 1;
    for (uint64_t i = 0; i < gg.count && i < 12; ++i) { if (!tq_width_known(gg.d[i])) return cudaErrorInvalidValue; if (gg.rows[i] > most) most = gg.rows[i]; }
    tq_gemv_groups_kernel<<<tq_grid(most, 148u * 16u), 128, 0, st>>>(out, gg, w_room, l_room, x, cols, over);
    note_launch(1);
    return cudaGetLastError();
}

}  // namespace sv
