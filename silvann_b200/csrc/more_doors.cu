/* more_doors.cu — the doors either side of the hot kernels, as the contract words them: the per-row (gathered key set)
 * forms of grouped scores / softmax / mix that GLM's sparse attention calls, the sink softmax, and the two small doors
 * that make DeltaNet's inputs (gates, causal conv).  Simple, any shape, fixed summation order.
 *
 * Arithmetic follows engine/src/packages/nn/gpu/kernels/kernels.cuh: scores_grouped_rows :957-972, softmax_lens
 * :1104-1110, softmax_sink :1115-1131, mix_rows :1169-1178, deltanet gates_rows :2081-2101, conv_step(s) :627-645 and
 * :2106-2125 (four taps, a window of three kept per channel, silu). */
#include "common.cuh"
#include "kernels.h"

namespace sv {

using H = Elem<SV_DTYPE_FP16>;

__device__ __forceinline__ float blk_max(float v, float* sh) {
    for (int x = 16; x > 0; x >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, x));
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (l == 0) sh[w] = v;
    __syncthreads();
    float r = sh[0];
    for (int i = 1; i < nw; ++i) r = fmaxf(r, sh[i]);
    return r;
}
__device__ __forceinline__ float blk_sum(float v, float* sh) {
    for (int x = 16; x > 0; x >>= 1) v += __shfl_xor_sync(0xffffffffu, v, x);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (l == 0) sh[w] = v;
    __syncthreads();
    float r = 0.f;
    for (int i = 0; i < nw; ++i) r += sh[i];
    return r;
}

/* Row u's query heads at q + u·q_row, its lens[u] key rows at k + u·k_row, its raw scaled scores at p + u·p_row, a query
 * head's lens[u] apart.  A block a (row, head); a warp a position, lanes across head_dim. */
__global__ void __launch_bounds__(256) scores_grouped_rows_kernel(float* p, uint64_t p_row, const uint16_t* q, uint64_t q_row, const uint16_t* k,
                                                                  uint64_t k_row, const uint32_t* lens, uint64_t qh, uint64_t kvh, uint64_t d,
                                                                  uint64_t rows) {
    const uint64_t group = qh / kvh, row = kvh * d;
    const float scale = 1.0f / sqrtf((float)d);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (uint64_t i = blockIdx.x; i < rows * qh; i += gridDim.x) {
        const uint64_t u = i / qh, h = i - u * qh, length = lens[u];
        const uint16_t* qv = q + u * q_row + h * d;
        const uint16_t* kv = k + u * k_row + (h / group) * d;
        float* ph = p + u * p_row + h * length;
        for (uint64_t t = warp; t < length; t += nw) {
            float dot = 0.f;
            for (uint64_t e = lane; e < d; e += 32) dot += H::to_float(qv[e]) * H::to_float(kv[t * row + e]);
            for (int x = 16; x > 0; x >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, x);
            if (lane == 0) ph[t] = dot * scale;
        }
    }
}

/* Each of rows·heads rows of p its softmax in place; row (u, h) at p + u·p_row + h·lens[u], lens[u] long.  With `sink`
 * (rows·heads halves, one a row — lens null, every row `length` long): the sum takes one more term, exp(sink), that
 * weighs nothing, and the maximum includes it. */
__global__ void __launch_bounds__(256) softmax_lens_kernel(float* p, uint64_t p_row, const uint32_t* lens, uint64_t heads, uint64_t rows,
                                                           const uint16_t* sink, uint64_t length_all) {
    __shared__ float sh[8];
    for (uint64_t b = blockIdx.x; b < rows * heads; b += gridDim.x) {
        const uint64_t u = b / heads, h = b - u * heads;
        const uint64_t length = lens ? lens[u] : length_all;
        float* ph = lens ? p + u * p_row + h * length : p + b * length_all;
        const float sk = sink ? H::to_float(sink[b]) : -INFINITY;
        float m = sk;
        for (uint64_t t = threadIdx.x; t < length; t += blockDim.x) m = fmaxf(m, ph[t]);
        const float top = blk_max(m, sh);
        float part = 0.f;
        for (uint64_t t = threadIdx.x; t < length; t += blockDim.x) { const float w = expf(ph[t] - top); ph[t] = w; part += w; }
        float sum = blk_sum(part, sh);
        if (sink) sum += expf(sk - top);
        const float inv = 1.0f / sum;
        for (uint64_t t = threadIdx.x; t < length; t += blockDim.x) ph[t] *= inv;
        __syncthreads();
    }
}

/* Row u's heads' answers at o + u·o_row from its weights at p + u·p_row and its lens[u] value rows at v + u·v_row. */
__global__ void __launch_bounds__(256) mix_rows_kernel(uint16_t* o, uint64_t o_row, const float* p, uint64_t p_row, const uint16_t* v, uint64_t v_row,
                                                       const uint32_t* lens, uint64_t qh, uint64_t kvh, uint64_t d, uint64_t rows, unsigned int* over) {
    const uint64_t group = qh / kvh, row = kvh * d;
    bool hit = false;
    for (uint64_t i = blockIdx.x; i < rows * qh; i += gridDim.x) {
        const uint64_t u = i / qh, h = i - u * qh, length = lens[u];
        const float* ph = p + u * p_row + h * length;
        const uint16_t* vh = v + u * v_row + (h / group) * d;
        for (uint64_t e = threadIdx.x; e < d; e += blockDim.x) {
            float sum = 0.f;
            for (uint64_t t = 0; t < length; ++t) sum += ph[t] * H::to_float(vh[t * row + e]);
            o[u * o_row + h * d + e] = H::from_float(sum, hit);
        }
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* beta = half(sigmoid(b)); g = -half(half(softplus(half(a + dt_bias[h]))) · half(exp(a_log[h]))), every intermediate
 * rounded to a half where the reference rounds it. */
__global__ void __launch_bounds__(256) deltanet_gates_rows_kernel(uint16_t* beta, uint16_t* g, const uint16_t* a, const uint16_t* b,
                                                                  const uint16_t* a_log, const uint16_t* dt_bias, uint64_t heads, uint64_t rows,
                                                                  unsigned int* over) {
    const uint64_t n = heads * rows;
    bool hit = false;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t h = i % heads;
        beta[i] = H::from_float(1.0f / (1.0f + expf(-H::to_float(b[i]))), hit);
        const float sum = H::to_float(H::from_float(H::to_float(a[i]) + H::to_float(dt_bias[h]), hit));
        const float mag = sum < 0.f ? -sum : sum, top = sum > 0.f ? sum : 0.f;
        const float sp = H::to_float(H::from_float(top + logf(1.0f + expf(-mag)), hit));
        const float ea = H::to_float(H::from_float(expf(H::to_float(a_log[h])), hit));
        const float prod = H::to_float(H::from_float(sp * ea, hit));
        g[i] = H::from_float(prod * -1.0f, hit);
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* The causal conv over `rows` positions in order: a thread a channel, its window of three its own. */
__global__ void __launch_bounds__(256) deltanet_conv_steps_kernel(uint16_t* o, uint16_t* s, const uint16_t* w, const uint16_t* x, uint64_t ch,
                                                                  uint64_t rows, unsigned int* over) {
    bool hit = false;
    for (uint64_t c = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; c < ch; c += (uint64_t)gridDim.x * blockDim.x) {
        const float w0 = H::to_float(w[c * 4]), w1 = H::to_float(w[c * 4 + 1]), w2 = H::to_float(w[c * 4 + 2]), w3 = H::to_float(w[c * 4 + 3]);
        uint16_t s0 = s[c * 3], s1 = s[c * 3 + 1], s2 = s[c * 3 + 2];
        for (uint64_t t = 0; t < rows; ++t) {
            const uint16_t xt = x[t * ch + c];
            float acc = 0.f;
            acc += w0 * H::to_float(s0);
            acc += w1 * H::to_float(s1);
            acc += w2 * H::to_float(s2);
            acc += w3 * H::to_float(xt);
            o[t * ch + c] = H::from_float(acc / (1.0f + expf(-acc)), hit);
            s0 = s1; s1 = s2; s2 = xt;
        }
        s[c * 3] = s0; s[c * 3 + 1] = s1; s[c * 3 + 2] = s2;
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* ---------------------------------------------------------------------------------------------------------- */

static inline unsigned grid_cap(uint64_t items, unsigned cap = 65535u) { return (unsigned)(items < 1 ? 1 : (items > cap ? cap : items)); }

cudaError_t scores_grouped_rows_launch(float* p, uint64_t p_row, const uint16_t* q, uint64_t q_row, const uint16_t* k, uint64_t k_row,
                                       const uint32_t* lens, uint64_t qh, uint64_t kvh, uint64_t d, uint64_t rows, cudaStream_t st) {
    scores_grouped_rows_kernel<<<grid_cap(rows * qh), 256, 0, st>>>(p, p_row, q, q_row, k, k_row, lens, qh, kvh, d, rows);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t softmax_lens_launch(float* p, uint64_t p_row, const uint32_t* lens, uint64_t heads, uint64_t rows, cudaStream_t st) {
    softmax_lens_kernel<<<grid_cap(rows * heads), 256, 0, st>>>(p, p_row, lens, heads, rows, nullptr, 0);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t softmax_sink_launch(float* p, const uint16_t* sink, uint64_t rows, uint64_t length, cudaStream_t st) {
    softmax_lens_kernel<<<grid_cap(rows), 256, 0, st>>>(p, 0, nullptr, 1, rows, sink, length);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t mix_rows_launch(uint16_t* o, uint64_t o_row, const float* p, uint64_t p_row, const uint16_t* v, uint64_t v_row, const uint32_t* lens,
                            uint64_t qh, uint64_t kvh, uint64_t d, uint64_t rows, unsigned int* over, cudaStream_t st) {
    const unsigned threads = d >= 256 ? 256u : (d >= 128 ? 128u : 64u);
    mix_rows_kernel<<<grid_cap(rows * qh), threads, 0, st>>>(o, o_row, p, p_row, v, v_row, lens, qh, kvh, d, rows, over);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t deltanet_gates_rows_launch(uint16_t* beta, uint16_t* g, const uint16_t* a, const uint16_t* b, const uint16_t* a_log,
                                       const uint16_t* dt_bias, uint64_t heads, uint64_t rows, unsigned int* over, cudaStream_t st) {
    deltanet_gates_rows_kernel<<<grid_cap((heads * rows + 255) / 256, 4096u), 256, 0, st>>>(beta, g, a, b, a_log, dt_bias, heads, rows, over);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t deltanet_conv_steps_launch(uint16_t* o, uint16_t* s, const uint16_t* w, const uint16_t* x, uint64_t ch, uint64_t rows,
                                       unsigned int* over, cudaStream_t st) {
    deltanet_conv_steps_kernel<<<grid_cap((ch + 127) / 128, 4096u), 128, 0, st>>>(o, s, w, x, ch, rows, over);
    note_launch(1);
    return cudaGetLastError();
}

}  // namespace sv
