/* mixer_doors.cu — the small steps either side of attention inside a layer's mixer, as the doors word them.
 *
 * A decode step of the reference's Qwen mixer runs, around the attention doors, a norm of the query and key heads, the
 * rotary position encoding, the output gate, a residual add and a few copies (engine/src/packages/ai_qwen_3/contracts/
 * objects/mixer__abi.cuh:229-247); a prompt runs the many-row forms.  These are elementwise or one reduction a row, a few
 * kilobytes each: bound by launch latency, not by anything on the card.  They are answered here so that a program's
 * attention path stays on one family; each follows the reference body it cites, same operations in the same order.
 *     vector_add, vector_copy, vector_copy_rows          kernels.cuh:103-113, 3855-3857, 3874-3881
 *     rmsnorm, rmsnorm_rows                               :158-176, 1700-1705   (the sum's order is the block's, as the reference allows)
 *     rope, rope_rows, rope_interleaved                   :843-858, 1710-1727, 1733-1749
 *     rope_angles, rope_angles_rows, _mrope_rows, _axial_rows   :871-886, 1754-1767, 1770-1784, 1789-1803
 *     attention_gate_rows                                 :2062-2076 */
#include "common.cuh"
#include "kernels.h"

namespace sv {

using H = Elem<SV_DTYPE_FP16>;

#define SV_EACH(i, n) for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < (n); i += (uint64_t)gridDim.x * blockDim.x)

__global__ void __launch_bounds__(256) vector_add_kernel(uint16_t* z, const uint16_t* x, const uint16_t* y, uint64_t n, unsigned int* over) {
    bool hit = false;
    SV_EACH(i, n) z[i] = H::from_float(H::to_float(x[i]) + H::to_float(y[i]), hit);
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}
__global__ void __launch_bounds__(256) vector_copy_rows_kernel(uint16_t* out, uint64_t out_row, const uint16_t* in, uint64_t in_row, uint64_t width,
                                                               uint64_t rows) {
    SV_EACH(i, rows * width) { const uint64_t t = i / width, j = i - t * width; out[t * out_row + j] = in[t * in_row + j]; }
}

/* a block a row: sum of squares folded over the block, then each thread its own elements */
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(uint16_t* o, const uint16_t* x, const uint16_t* w, uint64_t n, uint64_t rows,
                                                           uint64_t x_stride, uint64_t o_stride, float eps, unsigned int* over) {
    __shared__ float sh[8];
    bool hit = false;
    for (uint64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const uint16_t* xr = x + r * x_stride;
        float part = 0.f;
        for (uint64_t i = threadIdx.x; i < n; i += blockDim.x) { const float v = H::to_float(xr[i]); part += v * v; }
        for (int s = 16; s > 0; s >>= 1) part += __shfl_xor_sync(0xffffffffu, part, s);
        if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = part;
        __syncthreads();
        float sum = 0.f;
        for (unsigned k = 0; k < blockDim.x / 32; ++k) sum += sh[k];
        const float scale = 1.0f / sqrtf(sum / (float)n + eps);
        for (uint64_t i = threadIdx.x; i < n; i += blockDim.x) o[r * o_stride + i] = H::from_float((H::to_float(xr[i]) * scale) * H::to_float(w[i]), hit);
        __syncthreads();
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* rmsnorm_rows followed by rope_rows over the same rows, in one pass: a block a (position, head) row — its norm as the door
 * above makes it, rounded to a half, kept in shared memory — and then the rotation of the row's first `rot` elements by the
 * position's angles, reading those halves: the bits of the two doors one after the other.  Row r of the norm is head r %
 * heads of position r / heads; the angles of a position are at cs + position·rot. */
__global__ void __launch_bounds__(256) rmsnorm_rope_rows_kernel(uint16_t* o, const uint16_t* x, const uint16_t* w, const float* cs, uint64_t n, uint64_t rows,
                                                                uint64_t heads, uint64_t x_stride, uint64_t o_stride, uint64_t rot, float eps,
                                                                unsigned int* over) {
    extern __shared__ uint16_t nr_row[];
    __shared__ float sh[8];
    const uint64_t pairs = rot / 2;
    bool hit = false;
    for (uint64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const uint16_t* xr = x + r * x_stride;
        float part = 0.f;
        for (uint64_t i = threadIdx.x; i < n; i += blockDim.x) { const float v = H::to_float(xr[i]); part += v * v; }
        for (int s = 16; s > 0; s >>= 1) part += __shfl_xor_sync(0xffffffffu, part, s);
        if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = part;
        __syncthreads();
        float sum = 0.f;
        for (unsigned k = 0; k < blockDim.x / 32; ++k) sum += sh[k];
        const float scale = 1.0f / sqrtf(sum / (float)n + eps);
        for (uint64_t i = threadIdx.x; i < n; i += blockDim.x) nr_row[i] = H::from_float((H::to_float(xr[i]) * scale) * H::to_float(w[i]), hit);
        __syncthreads();
        const float* ang = cs + (r / heads) * rot;
        uint16_t* orow = o + r * o_stride;
        for (uint64_t k = threadIdx.x; k < pairs; k += blockDim.x) {         /* the turn, worded as rope_rows words it */
            const float a = H::to_float(nr_row[k]), b = H::to_float(nr_row[k + pairs]);
            const float c = ang[k], s = ang[pairs + k];
            orow[k] = H::from_float(a * c - b * s, hit);
            orow[k + pairs] = H::from_float(b * c + a * s, hit);
        }
        for (uint64_t i = rot + threadIdx.x; i < n; i += blockDim.x) orow[i] = nr_row[i];
        __syncthreads();
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* rotate_half on the first `rot` elements of every head of every row; row r's angles at cs + r·rot (cosines then sines) */
__global__ void __launch_bounds__(256) rope_rows_kernel(uint16_t* o, const uint16_t* x, const float* cs, uint64_t rows, uint64_t heads,
                                                        uint64_t head_stride, uint64_t row_stride, uint64_t rot, unsigned int* over) {
    const uint64_t pairs = rot / 2, per_row = heads * pairs;
    bool hit = false;
    SV_EACH(i, rows * per_row) {
        const uint64_t r = i / per_row, rest = i - r * per_row, e = rest / pairs, k = rest - e * pairs;
        const uint64_t at = r * row_stride + e * head_stride + k;
        const float a = H::to_float(x[at]), b = H::to_float(x[at + pairs]);
        const float c = cs[r * rot + k], s = cs[r * rot + pairs + k];
        o[at] = H::from_float(a * c - b * s, hit);
        o[at + pairs] = H::from_float(b * c + a * s, hit);
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}
/* the same turn on adjacent pairs (2k, 2k+1); `inverse` negates the sines */
__global__ void __launch_bounds__(256) rope_interleaved_kernel(uint16_t* o, const uint16_t* x, const float* cs, uint64_t heads, uint64_t head_stride,
                                                               uint64_t rot, uint64_t inverse, unsigned int* over) {
    const uint64_t pairs = rot / 2;
    bool hit = false;
    SV_EACH(i, heads * pairs) {
        const uint64_t h = i / pairs, k = i - h * pairs, at = h * head_stride + 2 * k;
        const float a = H::to_float(x[at]), b = H::to_float(x[at + 1]);
        const float c = cs[k], sn = inverse != 0 ? -cs[pairs + k] : cs[pairs + k];
        o[at] = H::from_float(a * c - b * sn, hit);
        o[at + 1] = H::from_float(b * c + a * sn, hit);
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* Angles.  The frequency of pair k is r^k with r = theta^(-2/width), MULTIPLIED UP as the reference does it (an ulp of the
 * frequency is multiplied by the position), the angle position · frequency, precise cosf and sinf.
 * mode 0: every row at position first + row.  1: M-RoPE — a row's three positions, pair k taking the row's when k % 3 == 1
 * and k < 3·(sections & 0xffff), the column's when k % 3 == 2 and k < 3·(sections >> 16 & 0xffff), the time's otherwise.
 * 2: axial — the first half of the pairs a patch's row, the second its column, each half its own ladder over width/2. */
__global__ void __launch_bounds__(256) rope_angles_kernel(float* cs, uint64_t first, const uint32_t* positions, float theta, uint64_t head_dim,
                                                          uint64_t rows, uint64_t sections, int mode) {
    const uint64_t pairs = head_dim / 2, per_axis = pairs / 2;
    /* r as the host's libm makes it: its logf and expf are correctly rounded, the card's single-precision ones are within an
     * ulp or two, and an ulp of r is k ulps of the frequency and position·k ulps of an angle — 4e-3 rad at position 100,000.
     * So each is taken in double and rounded once; the fp32 steps between them are the reference's. */
    const float lg = (float)log((double)theta);
    const float r = (float)exp((double)(-2.0f / (float)(uint32_t)(mode == 2 ? pairs : head_dim) * lg));
    SV_EACH(i, rows * pairs) {
        const uint64_t row = i / pairs, k = i - row * pairs;
        uint64_t steps = k, pos = first + row;
        if (mode == 1) {
            const uint64_t third = k % 3, by_row = sections & 0xFFFFull, by_column = (sections >> 16) & 0xFFFFull;
            const uint64_t which = (third == 1 && k < 3 * by_row) ? 1 : (third == 2 && k < 3 * by_column) ? 2 : 0;
            pos = positions[3 * row + which];
        } else if (mode == 2) {
            const uint64_t axis = k < per_axis ? 0 : 1;
            steps = k - axis * per_axis;
            pos = positions[2 * row + axis];
        }
        float frequency = 1.0f;
        for (uint64_t m = 0; m < steps; ++m) frequency = __fmul_rn(frequency, r);        /* one rounding a step, never fused or regrouped */
        const float angle = __fmul_rn((float)pos, frequency);
        cs[row * head_dim + k] = cosf(angle);
        cs[row * head_dim + pairs + k] = sinf(angle);
    }
}

/* o = att · half(sigmoid(gate)), the gate the second half of each head's [query · gate] pair in qg */
__global__ void __launch_bounds__(256) attention_gate_rows_kernel(uint16_t* o, const uint16_t* att, const uint16_t* qg, uint64_t heads, uint64_t head_dim,
                                                                  unsigned int* over) {
    bool hit = false;
    SV_EACH(i, heads * head_dim) {
        const uint64_t h = i / head_dim, e = i - h * head_dim;
        const float v = H::to_float(qg[h * 2 * head_dim + head_dim + e]);
        const uint16_t gate = H::from_float(1.0f / (1.0f + expf(-v)), hit);
        o[i] = H::from_float(H::to_float(att[i]) * H::to_float(gate), hit);
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* ---------------------------------------------------------------------------------------------------------- */

static inline unsigned each_grid(uint64_t n) { const uint64_t b = (n + 255) / 256; return (unsigned)(b < 1 ? 1 : (b > 148u * 8u ? 148u * 8u : b)); }
#define SV_DONE() do { note_launch(1); return cudaGetLastError(); } while (0)

cudaError_t vector_add_launch(uint16_t* z, const uint16_t* x, const uint16_t* y, uint64_t n, unsigned int* over, cudaStream_t st) {
    vector_add_kernel<<<each_grid(n), 256, 0, st>>>(z, x, y, n, over); SV_DONE();
}
cudaError_t vector_copy_rows_launch(uint16_t* out, uint64_t out_row, const uint16_t* in, uint64_t in_row, uint64_t width, uint64_t rows, cudaStream_t st) {
    vector_copy_rows_kernel<<<each_grid(rows * width), 256, 0, st>>>(out, out_row, in, in_row, width, rows); SV_DONE();
}
cudaError_t rmsnorm_rows_launch(uint16_t* o, const uint16_t* x, const uint16_t* w, uint64_t n, uint64_t rows, uint64_t x_stride, uint64_t o_stride,
                                float eps, unsigned int* over, cudaStream_t st) {
    const unsigned threads = n >= 2048 ? 256u : (n >= 512 ? 128u : 64u);
    rmsnorm_rows_kernel<<<(unsigned)(rows < 1 ? 1 : (rows > 65535 ? 65535 : rows)), threads, 0, st>>>(o, x, w, n, rows, x_stride, o_stride, eps, over); SV_DONE();
}
cudaError_t rmsnorm_rope_rows_launch(uint16_t* o, const uint16_t* x, const uint16_t* w, const float* cs, uint64_t n, uint64_t rows, uint64_t heads,
                                     uint64_t x_stride, uint64_t o_stride, uint64_t rot, float eps, unsigned int* over, cudaStream_t st) {
    if (n == 0 || n > 16384 || rot > n || rot % 2 != 0 || heads == 0) return cudaErrorInvalidValue;
    const unsigned threads = n >= 2048 ? 256u : (n >= 512 ? 128u : 64u);    /* the norm door's own block: the same partial sums in the same order */
    rmsnorm_rope_rows_kernel<<<(unsigned)(rows < 1 ? 1 : (rows > 65535 ? 65535 : rows)), threads, n * sizeof(uint16_t), st>>>(o, x, w, cs, n, rows, heads, x_stride,
                                                                                                                         o_stride, rot, eps, over); SV_DONE();
}
cudaError_t rope_rows_launch(uint16_t* o, const uint16_t* x, const float* cs, uint64_t rows, uint64_t heads, uint64_t head_stride, uint64_t row_stride,
                             uint64_t rot, unsigned int* over, cudaStream_t st) {
    rope_rows_kernel<<<each_grid(rows * heads * (rot / 2)), 256, 0, st>>>(o, x, cs, rows, heads, head_stride, row_stride, rot, over); SV_DONE();
}
cudaError_t rope_interleaved_launch(uint16_t* o, const uint16_t* x, const float* cs, uint64_t heads, uint64_t head_stride, uint64_t rot, uint64_t inverse,
                                    unsigned int* over, cudaStream_t st) {
    rope_interleaved_kernel<<<each_grid(heads * (rot / 2)), 256, 0, st>>>(o, x, cs, heads, head_stride, rot, inverse, over); SV_DONE();
}
cudaError_t rope_angles_launch(float* cs, uint64_t first, const uint32_t* positions, float theta, uint64_t head_dim, uint64_t rows, uint64_t sections,
                               int mode, cudaStream_t st) {
    rope_angles_kernel<<<each_grid(rows * (head_dim / 2)), 256, 0, st>>>(cs, first, positions, theta, head_dim, rows, sections, mode); SV_DONE();
}
cudaError_t attention_gate_rows_launch(uint16_t* o, const uint16_t* att, const uint16_t* qg, uint64_t heads, uint64_t head_dim, unsigned int* over,
                                       cudaStream_t st) {
    attention_gate_rows_kernel<<<each_grid(heads * head_dim), 256, 0, st>>>(o, att, qg, heads, head_dim, over); SV_DONE();
}

}  // namespace sv
