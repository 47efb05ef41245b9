/* attn_doors.cu — the attention doors exactly as the contract words them, for any shape and alignment.
 *
 * These kernels materialise the fp32 weights buffer `p` the way the reference does, so they serve (a) a door call
 * whose partner never arrives (a program that reads `p` itself), (b) shapes or addresses the TMA kernels refuse, and
 * (c) the small doors that are real work in the tiered path: `attention_merge`, `attention_finish`.  They are
 * correct-first, not the fast path: the fused kernels in decode.cu / prefill.cu are what a matching door pair runs.
 *
 * Arithmetic follows engine/src/packages/nn/gpu/kernels/kernels.cuh — scores :894-915, mix :1144-1164, weights and
 * residual mix :1189-1241, merge :1243-1255, finish :1258-1267, causal forms :1028-1081 and :2036-2060, row softmax
 * :1085-1099, vector_sum :117-126 — with precise expf and a fixed (block-shape dependent, run-to-run identical)
 * summation order. */
#include "common.cuh"
#include "kernels.h"
#include "residual.cuh"

namespace sv {

using H = Elem<SV_DTYPE_FP16>;

__device__ __forceinline__ float block_max(float v, float* sh) {
    for (int x = 16; x > 0; x >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, x));
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (l == 0) sh[w] = v;
    __syncthreads();
    float r = sh[0];
    for (int i = 1; i < nw; ++i) r = fmaxf(r, sh[i]);
    return r;
}
__device__ __forceinline__ float block_sum(float v, float* sh) {
    for (int x = 16; x > 0; x >>= 1) v += __shfl_xor_sync(0xffffffffu, v, x);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (l == 0) sh[w] = v;
    __syncthreads();
    float r = 0.f;
    for (int i = 0; i < nw; ++i) r += sh[i];
    return r;
}

/* One query head's scaled scores over `length` positions into ph; a warp a position, lanes across head_dim. */
__device__ __forceinline__ void head_scores(float* ph, const uint16_t* qh, const uint16_t* kh, uint64_t row, uint64_t d,
                                            uint64_t length, float scale) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (uint64_t t = warp; t < length; t += nw) {
        const uint16_t* kr = kh + t * row;
        float dot = 0.f;
        for (uint64_t e = lane; e < d; e += 32) dot += H::to_float(qh[e]) * H::to_float(kr[e]);
        for (int x = 16; x > 0; x >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, x);
        if (lane == 0) ph[t] = dot * scale;
    }
}

/* In place: ph <- exp(ph - max) (and, normalise = true, divided by the sum).  Answers max and sum. */
__device__ __forceinline__ void head_softmax(float* ph, uint64_t length, bool normalise, float* sh, float& top, float& sum) {
    float m = -INFINITY;
    for (uint64_t t = threadIdx.x; t < length; t += blockDim.x) m = fmaxf(m, ph[t]);
    top = block_max(m, sh);
    float part = 0.f;
    for (uint64_t t = threadIdx.x; t < length; t += blockDim.x) { const float w = expf(ph[t] - top); ph[t] = w; part += w; }
    sum = block_sum(part, sh);
    if (normalise) {
        const float inv = 1.0f / sum;
        for (uint64_t t = threadIdx.x; t < length; t += blockDim.x) ph[t] *= inv;
    }
}

/* mode 0: softmax (attention_scores) · 1: unnormalised weights + (m, l) into res (attention_weights) ·
 * 2: raw scaled scores (attention_scores_grouped) */
__global__ void __launch_bounds__(256) scores_kernel(float* p, const uint16_t* q, const uint16_t* k, uint64_t qh, uint64_t kvh,
                                                     uint64_t d, uint64_t length, int mode, float* res) {
    __shared__ float sh[8];
    const uint64_t group = qh / kvh, row = kvh * d;
    const float scale = 1.0f / sqrtf((float)d);
    for (uint64_t h = blockIdx.x; h < qh; h += gridDim.x) {
        float* ph = p + h * length;
        head_scores(ph, q + h * d, k + (h / group) * d, row, d, length, scale);
        __syncthreads();
        if (mode == 2) continue;
        float top, sum;
        head_softmax(ph, length, mode == 0, sh, top, sum);
        if (mode == 1 && threadIdx.x == 0) { res[h * (d + 2)] = top; res[h * (d + 2) + 1] = sum; }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(256) softmax_rows_kernel(float* p, uint64_t rows, uint64_t length) {
    __shared__ float sh[8];
    for (uint64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        float top, sum;
        head_softmax(p + r * length, length, true, sh, top, sum);
        __syncthreads();
    }
}

/* One head's weighted sum of values; a thread an output element, positions in order from 0. */
__device__ __forceinline__ float head_mix(const float* ph, const uint16_t* vh, uint64_t row, uint64_t e, uint64_t length) {
    float sum = 0.f;
    for (uint64_t t = 0; t < length; ++t) sum += ph[t] * H::to_float(vh[t * row + e]);
    return sum;
}

/* res == null: o = half(sum) (attention_mix) · else acc into res (attention_residual_mix) */
__global__ void __launch_bounds__(256) mix_kernel(uint16_t* o, float* res, const float* p, const uint16_t* v, uint64_t qh,
                                                  uint64_t kvh, uint64_t d, uint64_t length, unsigned int* over) {
    const uint64_t group = qh / kvh, row = kvh * d;
    const uint64_t h = blockIdx.x;
    bool hit = false;
    for (uint64_t e = (uint64_t)blockIdx.y * blockDim.x + threadIdx.x; e < d; e += (uint64_t)gridDim.y * blockDim.x) {
        const float sum = head_mix(p + h * length, v + (h / group) * d, row, e, length);
        if (res) res[h * (d + 2) + 2 + e] = sum;
        else o[h * d + e] = H::from_float(sum, hit);
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

__global__ void __launch_bounds__(128) merge_kernel(float* into, const float* a, const float* b, uint64_t qh, uint64_t d) {
    const uint64_t w = d + 2;
    for (uint64_t h = blockIdx.x; h < qh; h += gridDim.x) {
        /* every thread reads the head's four scalars before any thread writes them: `into` may be `a` or `b` */
        float m = a[h * w], l = a[h * w + 1], fa, fb;
        merge_scalars(m, l, b[h * w], b[h * w + 1], fa, fb);
        __syncthreads();
        for (uint64_t e = threadIdx.x; e < d; e += blockDim.x) into[h * w + 2 + e] = merge_element(a[h * w + 2 + e], fa, b[h * w + 2 + e], fb);
        if (threadIdx.x == 0) { into[h * w] = m; into[h * w + 1] = l; }
        __syncthreads();
    }
}

template <int DT>
__global__ void __launch_bounds__(256) finish_kernel(uint16_t* o, const float* res, uint64_t qh, uint64_t d, unsigned int* over) {
    const uint64_t w = d + 2, n = qh * d;
    bool hit = false;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t h = i / d;
        o[i] = Elem<DT>::from_float(res[h * w + 2 + i % d] / res[h * w + 1], hit);
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* Row r (position first + r) of head h over cache rows 0..first+r; weights at p + (r·qh + h)·(first + rows). */
__global__ void __launch_bounds__(256) causal_scores_kernel(float* p, const uint16_t* q, const uint16_t* k, uint64_t qh, uint64_t kvh,
                                                            uint64_t d, uint64_t first, uint64_t rows, int softmax) {
    __shared__ float sh[8];
    const uint64_t group = qh / kvh, row = kvh * d, span = first + rows;
    const float scale = 1.0f / sqrtf((float)d);
    for (uint64_t i = blockIdx.x; i < rows * qh; i += gridDim.x) {
        const uint64_t r = i / qh, h = i - r * qh, length = first + r + 1;
        float* ph = p + i * span;
        head_scores(ph, q + i * d, k + (h / group) * d, row, d, length, scale);
        __syncthreads();
        if (softmax) { float top, sum; head_softmax(ph, length, true, sh, top, sum); __syncthreads(); }
    }
}

__global__ void __launch_bounds__(256) causal_softmax_kernel(float* p, uint64_t qh, uint64_t first, uint64_t rows) {
    __shared__ float sh[8];
    const uint64_t span = first + rows;
    for (uint64_t i = blockIdx.x; i < rows * qh; i += gridDim.x) {
        float top, sum;
        head_softmax(p + i * span, first + i / qh + 1, true, sh, top, sum);
        __syncthreads();
    }
}

__global__ void __launch_bounds__(256) causal_mix_kernel(uint16_t* o, const float* p, const uint16_t* v, uint64_t qh, uint64_t kvh,
                                                         uint64_t d, uint64_t first, uint64_t rows, unsigned int* over) {
    const uint64_t group = qh / kvh, row = kvh * d, span = first + rows;
    bool hit = false;
    for (uint64_t i = blockIdx.x; i < rows * qh; i += gridDim.x) {
        const uint64_t r = i / qh, h = i - r * qh;
        for (uint64_t e = threadIdx.x; e < d; e += blockDim.x)
            o[i * d + e] = H::from_float(head_mix(p + i * span, v + (h / group) * d, row, e, first + r + 1), hit);
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

struct SumParts { uint64_t at[8]; uint64_t count; };
__global__ void __launch_bounds__(256) vector_sum_kernel(uint16_t* out, SumParts parts, uint64_t n, unsigned int* over) {
    bool hit = false;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        float s = 0.f;
        for (uint64_t k = 0; k < parts.count; ++k) s += H::to_float(((const uint16_t*)parts.at[k])[i]);
        out[i] = H::from_float(s, hit);
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* ---------------------------------------------------------------------------------------------------------- */

static inline unsigned grid_for(uint64_t items, unsigned cap = 65535u) { return (unsigned)(items < 1 ? 1 : (items > cap ? cap : items)); }

cudaError_t scores_launch(float* p, const uint16_t* q, const uint16_t* k, uint64_t qh, uint64_t kvh, uint64_t d, uint64_t length,
                          int mode, float* res, cudaStream_t st) {
    scores_kernel<<<grid_for(qh), 256, 0, st>>>(p, q, k, qh, kvh, d, length, mode, res);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t softmax_rows_launch(float* p, uint64_t rows, uint64_t length, cudaStream_t st) {
    softmax_rows_kernel<<<grid_for(rows), 256, 0, st>>>(p, rows, length);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t mix_launch(uint16_t* o, float* res, const float* p, const uint16_t* v, uint64_t qh, uint64_t kvh, uint64_t d,
                       uint64_t length, unsigned int* over, cudaStream_t st) {
    const unsigned threads = d >= 128 ? 128u : 64u;
    dim3 grid((unsigned)qh, (unsigned)((d + threads - 1) / threads));
    mix_kernel<<<grid, threads, 0, st>>>(o, res, p, v, qh, kvh, d, length, over);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t merge_launch(float* into, const float* a, const float* b, uint64_t qh, uint64_t d, cudaStream_t st) {
    merge_kernel<<<grid_for(qh), 128, 0, st>>>(into, a, b, qh, d);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t finish_launch(uint16_t* o, const float* res, uint64_t qh, uint64_t d, unsigned int* over, int dtype, cudaStream_t st) {
    const unsigned blocks = grid_for((qh * d + 255) / 256);
    if (dtype == SV_DTYPE_BF16) finish_kernel<SV_DTYPE_BF16><<<blocks, 256, 0, st>>>(o, res, qh, d, over);
    else finish_kernel<SV_DTYPE_FP16><<<blocks, 256, 0, st>>>(o, res, qh, d, over);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t causal_scores_launch(float* p, const uint16_t* q, const uint16_t* k, uint64_t qh, uint64_t kvh, uint64_t d, uint64_t first,
                                 uint64_t rows, bool softmax, cudaStream_t st) {
    causal_scores_kernel<<<grid_for(rows * qh), 256, 0, st>>>(p, q, k, qh, kvh, d, first, rows, softmax ? 1 : 0);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t causal_softmax_launch(float* p, uint64_t qh, uint64_t first, uint64_t rows, cudaStream_t st) {
    causal_softmax_kernel<<<grid_for(rows * qh), 256, 0, st>>>(p, qh, first, rows);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t causal_mix_launch(uint16_t* o, const float* p, const uint16_t* v, uint64_t qh, uint64_t kvh, uint64_t d, uint64_t first,
                              uint64_t rows, unsigned int* over, cudaStream_t st) {
    const unsigned threads = d >= 256 ? 256u : (d >= 128 ? 128u : 64u);
    causal_mix_kernel<<<grid_for(rows * qh), threads, 0, st>>>(o, p, v, qh, kvh, d, first, rows, over);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t vector_sum_launch(uint16_t* out, const uint64_t* parts, uint64_t count, uint64_t n, unsigned int* over, cudaStream_t st) {
    SumParts sp;
    for (int i = 0; i < 8; ++i) sp.at[i] = (uint64_t)i < count ? parts[i] : 0ull;
    sp.count = count > 8 ? 8 : count;
    vector_sum_kernel<<<grid_for((n + 255) / 256, 4096u), 256, 0, st>>>(out, sp, n, over);
    note_launch(1);
    return cudaGetLastError();
}

}  // namespace sv
