/* glm_doors.cu — the doors of the reference's GLM mixer: Kimi Delta Attention, the latent attention's absorb and expand,
 * and the sparse attention's indexer.
 *
 * KDA (engine/src/packages/nn/gpu/kernels/kernels.cuh:3301-3470) is Gated DeltaNet's recurrence with the decay a VECTOR a
 * head, one number a key channel:   S <- diag(e^g) S;  delta = (v - S^T kn) beta;  S <- S + kn delta^T;  o = S^T qs, then an
 * RMS norm and a sigmoid gate.  The reference walks a head's rows with a block, a lane a column of the state, the state
 * in memory.  Here a head is one block of 1,024 threads and the state lives in registers for the whole run of rows: a
 * thread owns one column j and a slice of D²/1024 key rows i of it, the two sums over i (S^T kn and S^T qs) are folded
 * across the slices through shared memory, and the state is read once and written once a launch — 2·D²·4 bytes a head,
 * which at one row a launch (decode) is the traffic that bounds it.
 *
 * Latent attention (:3596-3664): a head's query is absorbed into the latent by the head's key rows of W (a column sum) and
 * the answer expanded by its value rows (a row sum): both are reads of W, once, 16 bytes a lane.
 *
 * The indexer (:3666-3846): a LayerNorm, the pooled keys, a pool's score, the top k pools as positions, block maxima and
 * row gathers — small, as worded; the choice keeps the reference's order exactly (keys above the cut, then ties by lowest
 * index, written in index order). */
#include "common.cuh"
#include "kernels.h"

namespace sv {

using H = Elem<SV_DTYPE_FP16>;

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

/* ---- KDA ------------------------------------------------------------------------------------------------------------ */

/* eg[t][h][i] = exp(lower · sigmoid(e^{a_log[h]} · (f + dt)))   (kernels.cuh:3400-3409) */
__global__ void __launch_bounds__(256) kda_decays_kernel(float* eg, const uint16_t* f, const uint16_t* dt, const uint16_t* a_log, uint64_t heads,
                                                         uint64_t head_dim, float lower, uint64_t rows) {
    const uint64_t width = heads * head_dim, all = rows * width;
    for (uint64_t x = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; x < all; x += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t c = x % width, h = c / head_dim;
        const float a = expf(H::to_float(a_log[h]));
        const float gi = lower / (1.0f + expf(-a * (H::to_float(f[x]) + H::to_float(dt[c]))));
        eg[x] = expf(gi);
    }
}

/* One block a head, the state in registers across `rows` rows.  D in {64, 128} (a 256-wide head's state is every register
 * of an SM: it takes the kernel after this one): CG = D/32 column groups of a warp's
 * width, SL = 32/CG slices of RPS = D/SL key rows; warp w holds column group w % CG of slice w / CG.
 * DECAYED: the decays are read from `eg` (made by kda_decays) instead of made from f, dt and a_log. */
template <int D, bool DECAYED>
__global__ void __launch_bounds__(1024, 1) kda_steps_kernel(float* S, const uint16_t* conved, const uint16_t* f, const float* eg, const uint16_t* b,
                                                            const uint16_t* dt, const uint16_t* a_log, const uint16_t* gate, const uint16_t* w,
                                                            uint16_t* out, uint64_t heads, float lower, float eps, uint64_t rows, unsigned int* over) {
    constexpr int CG = D / 32, SL = 32 / CG, RPS = D / SL;
    __shared__ float sk[D], sq[D], seg[D], red[SL][D], part[2][CG], spart[CG];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int j = (warp % CG) * 32 + lane, slice = warp / CG, i0 = slice * RPS;
    const uint64_t h = blockIdx.x, width = heads * D;
    float* Sh = S + h * D * D;
    const uint16_t* q = conved;
    const uint16_t* k = conved + rows * width;
    const uint16_t* v = conved + 2ull * rows * width;
    float st[RPS];
#pragma unroll
    for (int r = 0; r < RPS; ++r) st[r] = Sh[(uint64_t)(i0 + r) * D + j];
    const float a = DECAYED ? 0.f : expf(H::to_float(a_log[h]));
    const float dti = (!DECAYED && tid < D) ? H::to_float(dt[h * D + tid]) : 0.f;
    const float wj = H::to_float(w[j]);
    bool hit = false;
    for (uint64_t t = 0; t < rows; ++t) {
        const uint64_t at = t * width + h * D;
        if (tid < D) {                                                     /* this row's q, k and decays, and the two norms */
            const float qi = H::to_float(q[at + tid]), ki = H::to_float(k[at + tid]);
            sq[tid] = qi; sk[tid] = ki;
            seg[tid] = DECAYED ? eg[at + tid] : expf(lower / (1.0f + expf(-a * (H::to_float(f[at + tid]) + dti))));
            float qq = qi * qi, kk = ki * ki;
            for (int o = 16; o > 0; o >>= 1) { qq += __shfl_xor_sync(0xffffffffu, qq, o); kk += __shfl_xor_sync(0xffffffffu, kk, o); }
            if (lane == 0) { part[0][warp] = qq; part[1][warp] = kk; }
        }
        const float beta = sigmoidf_(H::to_float(b[t * heads + h]));
        const float vj = H::to_float(v[at + j]), gz = H::to_float(gate[at + j]);
        __syncthreads();
        float qq = 0.f, kk = 0.f;
#pragma unroll
        for (int c = 0; c < CG; ++c) { qq += part[0][c]; kk += part[1][c]; }
        const float inv_q = 1.0f / sqrtf(qq + 1e-6f) / sqrtf((float)D), inv_k = 1.0f / sqrtf(kk + 1e-6f);
        float kv = 0.f;
#pragma unroll
        for (int r = 0; r < RPS; ++r) { st[r] *= seg[i0 + r]; kv += st[r] * sk[i0 + r] * inv_k; }
        red[slice][j] = kv;
        __syncthreads();
        kv = 0.f;
#pragma unroll
        for (int s = 0; s < SL; ++s) kv += red[s][j];
        const float delta = (vj - kv) * beta;
        float o = 0.f;
#pragma unroll
        for (int r = 0; r < RPS; ++r) { const float s = st[r] + sk[i0 + r] * inv_k * delta; st[r] = s; o += s * sq[i0 + r]; }
        __syncthreads();                                                   /* every slice has read red before it is written again */
        red[slice][j] = o;
        __syncthreads();
        float oj = 0.f;
        if (slice == 0) {
            o = 0.f;
#pragma unroll
            for (int s = 0; s < SL; ++s) o += red[s][j];
            oj = H::to_float(H::from_float(o * inv_q, hit));
            float oo = oj * oj;
            for (int x = 16; x > 0; x >>= 1) oo += __shfl_xor_sync(0xffffffffu, oo, x);
            if (lane == 0) spart[warp] = oo;
        }
        __syncthreads();
        if (slice == 0) {
            float oo = 0.f;
#pragma unroll
            for (int c = 0; c < CG; ++c) oo += spart[c];
            const float scale = 1.0f / sqrtf(oo / (float)D + eps);
            out[at + j] = H::from_float(oj * scale * wj / (1.0f + expf(-gz)), hit);
        }
    }
#pragma unroll
    for (int r = 0; r < RPS; ++r) Sh[(uint64_t)(i0 + r) * D + j] = st[r];
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* Any other head_dim: a block a head, a thread a column, the state in memory — the reference's own shape. */
template <bool DECAYED>
__global__ void __launch_bounds__(256) kda_steps_any_kernel(float* S, const uint16_t* conved, const uint16_t* f, const float* eg, const uint16_t* b,
                                                            const uint16_t* dt, const uint16_t* a_log, const uint16_t* gate, const uint16_t* w,
                                                            uint16_t* out, uint64_t heads, uint64_t d, float lower, float eps, uint64_t rows,
                                                            unsigned int* over) {
    __shared__ float sh[3][8];
    const uint64_t h = blockIdx.x, width = heads * d;
    float* Sh = S + h * d * d;
    const uint16_t* q = conved;
    const uint16_t* k = conved + rows * width;
    const uint16_t* v = conved + 2ull * rows * width;
    const float a = DECAYED ? 0.f : expf(H::to_float(a_log[h]));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    bool hit = false;
    auto fold = [&](float x, int slot) {
        for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
        if (lane == 0) sh[slot][warp] = x;
        __syncthreads();
        float s = 0.f;
        for (int c = 0; c < 8; ++c) s += sh[slot][c];
        return s;
    };
    for (uint64_t t = 0; t < rows; ++t) {
        const uint64_t at = t * width + h * d;
        float qq = 0.f, kk = 0.f;
        for (uint64_t i = threadIdx.x; i < d; i += blockDim.x) { const float qi = H::to_float(q[at + i]), ki = H::to_float(k[at + i]); qq += qi * qi; kk += ki * ki; }
        const float inv_q = 1.0f / sqrtf(fold(qq, 0) + 1e-6f) / sqrtf((float)d), inv_k = 1.0f / sqrtf(fold(kk, 1) + 1e-6f);
        const float beta = sigmoidf_(H::to_float(b[t * heads + h]));
        float oo = 0.f;
        for (uint64_t j = threadIdx.x; j < d; j += blockDim.x) {
            float kv = 0.f;
            for (uint64_t i = 0; i < d; ++i) {
                const float e = DECAYED ? eg[at + i] : expf(lower / (1.0f + expf(-a * (H::to_float(f[at + i]) + H::to_float(dt[h * d + i])))));
                const float s = Sh[i * d + j] * e;
                Sh[i * d + j] = s;
                kv += s * H::to_float(k[at + i]) * inv_k;
            }
            const float delta = (H::to_float(v[at + j]) - kv) * beta;
            float o = 0.f;
            for (uint64_t i = 0; i < d; ++i) { const float s = Sh[i * d + j] + H::to_float(k[at + i]) * inv_k * delta; Sh[i * d + j] = s; o += s * H::to_float(q[at + i]); }
            out[at + j] = H::from_float(o * inv_q, hit);
            const float oj = H::to_float(out[at + j]);
            oo += oj * oj;
        }
        const float scale = 1.0f / sqrtf(fold(oo, 2) / (float)d + eps);
        for (uint64_t j = threadIdx.x; j < d; j += blockDim.x)
            out[at + j] = H::from_float(H::to_float(out[at + j]) * scale * H::to_float(w[j]) / (1.0f + expf(-H::to_float(gate[at + j]))), hit);
        __syncthreads();
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* ---- latent attention: absorb and expand ------------------------------------------------------------------------------ */

/* out[t][h][c] = scale · sum_i W[(h·stride + i)·latent + c] · q[t][h][i]   (kernels.cuh:3608-3627).  A block a (row, head):
 * a thread owns 8 neighbouring columns (one 16-byte load a key row) when the latent's width and W's address allow, and
 * the block's threads past the columns split the nope rows between them; their sums meet in shared memory. */
template <bool WIDE>
__global__ void __launch_bounds__(512) absorb_kernel(uint16_t* out, const uint16_t* q, const uint16_t* W, uint64_t heads, uint64_t nope, uint64_t latent,
                                                     uint64_t stride, float scale, uint64_t rows, uint64_t parts, unsigned int* over) {
    extern __shared__ float acc[];                                         /* [slices][columns of a part] */
    constexpr int PER = WIDE ? 8 : 1;
    const uint64_t chunks = latent / PER / parts;                          /* chunks of a part (WIDE only where 8 divides the latent's width; `parts` divides the chunks) */
    const uint64_t pcols = chunks * PER;                                   /* columns of a part */
    const uint64_t across = chunks < blockDim.x ? chunks : blockDim.x;     /* threads side by side over the columns */
    const uint64_t slices = blockDim.x / across;                           /* and the rest of the block over the key rows */
    bool hit = false;
    /* a block a (row, head, part of the latent's columns): with few heads and one row, whole heads would leave most of the card idle */
    for (uint64_t bhp = blockIdx.x; bhp < rows * heads * parts; bhp += gridDim.x) {
        const uint64_t bh = bhp / parts, part = bhp - bh * parts;
        const uint64_t t = bh / heads, h = bh - t * heads;
        const uint16_t* qh = q + (t * heads + h) * nope;
        const uint16_t* Wh = W + h * stride * latent + part * pcols;
        const uint64_t slice = threadIdx.x / across, first = threadIdx.x - slice * across;
        if (slice < slices)
            for (uint64_t chunk = first; chunk < chunks; chunk += across) {
                float s[PER];
#pragma unroll
                for (int e = 0; e < PER; ++e) s[e] = 0.f;
                if (WIDE) {
                    /* eight key rows' 16 bytes asked for before any is used: a column sum is one long chain of loads otherwise */
                    uint64_t i = slice;
                    for (; i + 7 * slices < nope; i += 8 * slices) {
                        uint4 u[8];
                        float qv[8];
#pragma unroll
                        for (int k = 0; k < 8; ++k) { u[k] = __ldg(reinterpret_cast<const uint4*>(Wh + (i + k * slices) * latent + chunk * 8)); qv[k] = H::to_float(qh[i + k * slices]); }
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            const uint32_t ws[4] = {u[k].x, u[k].y, u[k].z, u[k].w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) { const float2 p = H::unpack2(ws[e]); s[2 * e] += p.x * qv[k]; s[2 * e + 1] += p.y * qv[k]; }
                        }
                    }
                    for (; i < nope; i += slices) {
                        const float qi = H::to_float(qh[i]);
                        const uint4 u = __ldg(reinterpret_cast<const uint4*>(Wh + i * latent + chunk * 8));
                        const uint32_t ws[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) { const float2 p = H::unpack2(ws[e]); s[2 * e] += p.x * qi; s[2 * e + 1] += p.y * qi; }
                    }
                } else {
                    for (uint64_t i = slice; i < nope; i += slices) s[0] += H::to_float(Wh[i * latent + chunk]) * H::to_float(qh[i]);
                }
#pragma unroll
                for (int e = 0; e < PER; ++e) acc[slice * pcols + chunk * PER + e] = s[e];
            }
        __syncthreads();
        for (uint64_t c = threadIdx.x; c < pcols; c += blockDim.x) {
            float sum = 0.f;
            for (uint64_t sl = 0; sl < slices; ++sl) sum += acc[sl * pcols + c];
            out[(t * heads + h) * latent + part * pcols + c] = H::from_float(sum * scale, hit);
        }
        __syncthreads();
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* out[t][h][j] = sum_c W[(h·stride + offset + j)·latent + c] · o[t][h][c]   (kernels.cuh:3629-3664): a warp an output */
__global__ void __launch_bounds__(256) expand_kernel(uint16_t* out, const uint16_t* o, const uint16_t* W, uint64_t heads, uint64_t width, uint64_t latent,
                                                     uint64_t stride, uint64_t offset, uint64_t rows, unsigned int* over) {
    const uint64_t per = heads * width, all = rows * per;
    const int lane = threadIdx.x & 31;
    const bool wide = latent % 8 == 0 && ((uintptr_t)W % 16 == 0) && ((uintptr_t)o % 16 == 0);
    bool hit = false;
    for (uint64_t x = (uint64_t)blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5); x < all; x += (uint64_t)gridDim.x * (blockDim.x / 32)) {
        const uint64_t t = x / per, r = x - t * per, h = r / width;
        const uint16_t* row = W + (h * stride + offset + r % width) * latent;
        const uint16_t* in = o + (t * heads + h) * latent;
        float part = 0.f;
        if (wide) {
            for (uint64_t c = (uint64_t)lane * 8; c < latent; c += 256) {
                const uint4 a = *reinterpret_cast<const uint4*>(row + c), bb = *reinterpret_cast<const uint4*>(in + c);
                const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) { const float2 p = H::unpack2(aw[e]), qv = H::unpack2(bw[e]); part += p.x * qv.x; part += p.y * qv.y; }
            }
        } else {
            for (uint64_t c = lane; c < latent; c += 32) part += H::to_float(row[c]) * H::to_float(in[c]);
        }
        for (int s = 16; s > 0; s >>= 1) part += __shfl_xor_sync(0xffffffffu, part, s);
        if (lane == 0) out[x] = H::from_float(part, hit);
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* ---- the sparse attention's indexer ------------------------------------------------------------------------------------ */

/* o = (x - mean) / sqrt(var + eps) · w + b over one row of n: one block   (kernels.cuh:3670-3688) */
__global__ void __launch_bounds__(256) index_layernorm_kernel(uint16_t* o, const uint16_t* x, const uint16_t* w, const uint16_t* b, uint64_t n, float eps,
                                                              unsigned int* over) {
    __shared__ float sh[2][8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float sum = 0.f;
    for (uint64_t i = threadIdx.x; i < n; i += blockDim.x) sum += H::to_float(x[i]);
    for (int s = 16; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
    if (lane == 0) sh[0][warp] = sum;
    __syncthreads();
    sum = 0.f;
    for (int c = 0; c < 8; ++c) sum += sh[0][c];
    const float mean = sum / (float)n;
    float sq = 0.f;
    for (uint64_t i = threadIdx.x; i < n; i += blockDim.x) { const float d = H::to_float(x[i]) - mean; sq += d * d; }
    for (int s = 16; s > 0; s >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, s);
    if (lane == 0) sh[1][warp] = sq;
    __syncthreads();
    sq = 0.f;
    for (int c = 0; c < 8; ++c) sq += sh[1][c];
    const float inv = 1.0f / sqrtf(sq / (float)n + eps);
    bool hit = false;
    for (uint64_t i = threadIdx.x; i < n; i += blockDim.x) o[i] = H::from_float((H::to_float(x[i]) - mean) * inv * H::to_float(w[i]) + H::to_float(b[i]), hit);
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* pooled[p][c] = sum_i softmax_i(gate + ape) · key over pool p's kpool positions, a channel a thread   (:3693-3716) */
__global__ void __launch_bounds__(256) index_pool_kernel(uint16_t* pooled, const uint16_t* keys, const uint16_t* gates, const uint16_t* ape, uint64_t first,
                                                         uint64_t pools, uint64_t dim, uint64_t kpool, unsigned int* over) {
    bool hit = false;
    for (uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; e < pools * dim; e += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t p = first + e / dim, c = e % dim;
        float top = -INFINITY;
        for (uint64_t i = 0; i < kpool; ++i) { const float l = H::to_float(gates[(p * kpool + i) * dim + c]) + H::to_float(ape[i * dim + c]); if (l > top) top = l; }
        float den = 0.f, num = 0.f;
        for (uint64_t i = 0; i < kpool; ++i) {
            const float wgt = expf(H::to_float(gates[(p * kpool + i) * dim + c]) + H::to_float(ape[i * dim + c]) - top);
            den += wgt;
            num += wgt * H::to_float(keys[(p * kpool + i) * dim + c]);
        }
        pooled[p * dim + c] = H::from_float(num / den, hit);
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* scores[u][p] = sum_h w[u][h] / sqrt(heads) · relu(q[u][h] · K_p · scale), a warp a (row, pool), a lane its heads
 * (:3718-3757).  rows = 0 is the one-row door: every one of `pools` pools scored; else row u scores (len0 + u) / kpool. */
__global__ void __launch_bounds__(256) index_scores_kernel(float* scores, uint64_t scores_row, const uint16_t* q, const uint16_t* w, const uint16_t* pooled,
                                                           uint64_t heads, uint64_t dim, uint64_t pools, uint64_t len0, uint64_t kpool, uint64_t rows, float scale) {
    const int lane = threadIdx.x & 31;
    const uint64_t most = rows == 0 ? pools : (len0 + rows - 1) / kpool, count = (rows == 0 ? 1 : rows) * most;
    const float per_head = 1.0f / sqrtf((float)heads);
    for (uint64_t x = (uint64_t)blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5); x < count; x += (uint64_t)gridDim.x * (blockDim.x / 32)) {
        const uint64_t u = x / most, p = x - u * most;
        if (rows != 0 && p >= (len0 + u) / kpool) continue;
        const uint16_t* qu = q + u * heads * dim;
        const uint16_t* kp = pooled + p * dim;
        float part = 0.f;
        for (uint64_t h = lane; h < heads; h += 32) {
            float dot = 0.f;
            for (uint64_t c = 0; c < dim; ++c) dot += H::to_float(qu[h * dim + c]) * H::to_float(kp[c]);
            dot *= scale;
            part += (dot > 0.f ? dot : 0.f) * H::to_float(w[u * heads + h]) * per_head;
        }
        for (int s = 16; s > 0; s >>= 1) part += __shfl_xor_sync(0xffffffffu, part, s);
        if (lane == 0) scores[u * scores_row + p] = part;
    }
}

/* The same scores with the row's queries staged in shared memory once a block (a head's row one word longer than it is, so
 * that the lanes — a head each — read different banks) and a pool's key staged once a warp: the sums run over the columns in
 * the reference's order, from shared memory instead of 32 strided streams of global loads.  dim even; blockIdx.y is the row. */
__global__ void __launch_bounds__(256) index_scores_staged_kernel(float* scores, uint64_t scores_row, const uint16_t* q, const uint16_t* w,
                                                                  const uint16_t* pooled, uint32_t heads, uint32_t dim, uint64_t pools, uint64_t len0,
                                                                  uint64_t kpool, uint64_t rows, float scale) {
    extern __shared__ uint32_t ix_s[];
    const uint32_t half_dim = dim / 2, qstride = half_dim + 1;
    uint32_t* q_s = ix_s;                                    /* [heads][dim/2 + 1] words */
    uint32_t* k_s = ix_s + heads * qstride + (threadIdx.x >> 5) * half_dim;   /* this warp's pool key */
    const uint64_t u = blockIdx.y, mine = rows == 0 ? pools : (len0 + u) / kpool;
    const uint32_t* qu = reinterpret_cast<const uint32_t*>(q + u * heads * dim);
    for (uint32_t i = threadIdx.x; i < heads * half_dim; i += blockDim.x) q_s[(i / half_dim) * qstride + i % half_dim] = qu[i];
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float per_head = 1.0f / sqrtf((float)heads);
    for (uint64_t p = (uint64_t)blockIdx.x * 8 + warp; p < mine; p += (uint64_t)gridDim.x * 8) {
        const uint32_t* kp = reinterpret_cast<const uint32_t*>(pooled + p * dim);
        __syncwarp();
        for (uint32_t c = lane; c < half_dim; c += 32) k_s[c] = kp[c];
        __syncwarp();
        float part = 0.f;
        for (uint32_t h = lane; h < heads; h += 32) {
            const uint32_t* qh = q_s + h * qstride;
            float dot = 0.f;
            for (uint32_t c = 0; c < half_dim; ++c) {
                const float2 a = H::unpack2(qh[c]), b = H::unpack2(k_s[c]);
                dot += a.x * b.x;
                dot += a.y * b.y;
            }
            dot *= scale;
            part += (dot > 0.f ? dot : 0.f) * H::to_float(w[u * heads + h]) * per_head;
        }
        for (int x = 16; x > 0; x >>= 1) part += __shfl_xor_sync(0xffffffffu, part, x);
        if (lane == 0) scores[u * scores_row + p] = part;
    }
}

__device__ __forceinline__ uint32_t index_key(float f) {                   /* orders as the score does (:3759-3764) */
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) != 0u ? ~u : (u | 0x80000000u);
}

/* The top k of a row's pools as positions, a block a row (:3766-3818): the k-th largest key found a bit at a time from the
 * top, then, in index order, the pools above it and the first ties until k are chosen; a chosen pool is its kpool
 * positions, and the row's unfinished pool's positions follow.  rows = 0 is the one-row door (tail given by the caller). */
__global__ void __launch_bounds__(1024) index_select_kernel(uint32_t* index, uint64_t index_row, uint32_t* counts, const float* scores, uint64_t scores_row,
                                                            uint64_t pools1, uint64_t k, uint64_t kpool, uint64_t tail_first1, uint64_t tail1, uint64_t len0,
                                                            uint64_t rows) {
    __shared__ unsigned int hist[256], found[2];
    __shared__ unsigned int warp_sum[2][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (uint64_t u = blockIdx.x; u < (rows == 0 ? 1 : rows); u += gridDim.x) {
        const uint64_t len = len0 + u, pools = rows == 0 ? pools1 : len / kpool;
        const uint64_t tail_first = rows == 0 ? tail_first1 : pools * kpool, tail = rows == 0 ? tail1 : len - pools * kpool;
        const float* sc = scores + u * scores_row;
        uint32_t* out = index + u * index_row;
        /* the k-th largest key, a byte at a time from the top: a 256-bin count of the keys that carry the bytes found so far,
         * walked down from the top bin until k keys are covered (the value the reference finds a bit at a time) */
        uint32_t cut = 0u;
        if (pools > k) {
            uint32_t known = 0u, need = (uint32_t)k;
            for (int shift = 24; shift >= 0; shift -= 8) {
                for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0u;
                __syncthreads();
                for (uint64_t first = 0; first < pools; first += blockDim.x) {             /* whole warps together: lanes that count the */
                    const uint64_t p = first + threadIdx.x;                                    /* same bin add once, through their first */
                    const uint32_t key = p < pools ? index_key(sc[p]) : 0u;
                    const bool live = p < pools && (key & known) == cut;
                    const uint32_t bin = live ? ((key >> shift) & 255u) : 256u;
                    const unsigned same = __match_any_sync(0xffffffffu, bin);
                    if (live && lane == __ffs(same) - 1) atomicAdd(&hist[bin], (unsigned int)__popc(same));
                }
                __syncthreads();
                if (warp == 0) {
                    /* walked down from the top bin, eight bins a lane: the lane whose bins take the count past `need` walks them */
                    uint32_t mine8 = 0u;
#pragma unroll
                    for (int b = 0; b < 8; ++b) mine8 += hist[255 - 8 * lane - b];
                    uint32_t upto = mine8;                                  /* this lane's bins and every lane's above */
                    for (int d = 1; d < 32; d <<= 1) { const uint32_t o = __shfl_up_sync(0xffffffffu, upto, d); if (lane >= d) upto += o; }
                    const unsigned reached = __ballot_sync(0xffffffffu, upto >= need);
                    const int who = reached ? __ffs(reached) - 1 : 31;
                    if (lane == who) {
                        uint32_t covered = upto - mine8, bin = 255u - 8u * (uint32_t)lane;
                        for (int b = 0; b < 8; ++b, --bin) { const uint32_t here = hist[bin]; if (covered + here >= need || b == 7) break; covered += here; }
                        found[0] = bin; found[1] = need - covered;
                    }
                }
                __syncthreads();
                cut |= found[0] << shift; need = found[1]; known |= 255u << shift;
                __syncthreads();
            }
        }
        /* in index order: thread t owns the contiguous pools [t·per, (t+1)·per); an exclusive scan of (above, equal) counts
         * over the threads gives each its ties already spent and its place in the output */
        const uint64_t per = (pools + blockDim.x - 1) / blockDim.x, lo = threadIdx.x * per, hi = lo + per < pools ? lo + per : pools;
        unsigned int above = 0, equal = 0;
        if (pools > k)
            for (uint64_t p = lo; p < hi; ++p) { const uint32_t key = index_key(sc[p]); above += key > cut; equal += key == cut; }
        unsigned int a_in = above, e_in = equal;
        for (int s = 1; s < 32; s <<= 1) {
            const unsigned int a2 = __shfl_up_sync(0xffffffffu, a_in, s), e2 = __shfl_up_sync(0xffffffffu, e_in, s);
            if (lane >= s) { a_in += a2; e_in += e2; }
        }
        if (lane == 31) { warp_sum[0][warp] = a_in; warp_sum[1][warp] = e_in; }
        __syncthreads();
        unsigned int a_before = a_in - above, e_before = e_in - equal, a_all = 0, e_all = 0;
        for (int x = 0; x < warps; ++x) {
            if (x < warp) { a_before += warp_sum[0][x]; e_before += warp_sum[1][x]; }
            a_all += warp_sum[0][x]; e_all += warp_sum[1][x];
        }
        (void)e_all;
        const uint64_t ties = pools > k ? k - a_all : 0;                    /* how many of the equal keys are taken, lowest index first */
        uint64_t n;
        if (pools <= k) n = lo < pools ? lo : pools;                       /* every pool is chosen */
        else n = a_before + (e_before < ties ? e_before : ties);
        uint64_t spent = e_before;
        for (uint64_t p = lo; p < hi; ++p) {
            bool take = pools <= k;
            if (!take) {
                const uint32_t key = index_key(sc[p]);
                if (key > cut) take = true;
                else if (key == cut) { take = spent < ties; ++spent; }
            }
            if (take) { for (uint64_t i = 0; i < kpool; ++i) out[n * kpool + i] = (uint32_t)(p * kpool + i); ++n; }
        }
        const uint64_t chosen = pools <= k ? pools : k;
        for (uint64_t i = threadIdx.x; i < tail; i += blockDim.x) out[chosen * kpool + i] = (uint32_t)(tail_first + i);
        if (threadIdx.x == 0) counts[u] = (uint32_t)(chosen * kpool + tail);
        __syncthreads();
    }
}

/* out[b] = the largest of block b's scores (:3820-3829) */
__global__ void __launch_bounds__(256) index_blocks_kernel(float* out, const float* scores, uint64_t pools, uint64_t block) {
    const uint64_t blocks = (pools + block - 1) / block;
    for (uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; b < blocks; b += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t end = (b + 1) * block < pools ? (b + 1) * block : pools;
        float best = scores[b * block];
        for (uint64_t p = b * block + 1; p < end; ++p) best = scores[p] > best ? scores[p] : best;
        out[b] = best;
    }
}

/* row u's counts[u] rows of src, by index, one after another (:3831-3846); counts = null is the one-row door with n = most */
__global__ void __launch_bounds__(256) index_gather_kernel(uint16_t* out, uint64_t out_row, const uint16_t* src, const uint32_t* index, uint64_t index_row,
                                                           const uint32_t* counts, uint64_t most, uint64_t row, uint64_t rows) {
    const uint64_t per = most * row;
    for (uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; e < rows * per; e += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t u = e / per, f = e - u * per, i = f / row;
        if (counts == nullptr || i < (uint64_t)counts[u]) out[u * out_row + f] = src[(uint64_t)index[u * index_row + i] * row + f % row];
    }
}

/* ---------------------------------------------------------------------------------------------------------------------- */

static inline unsigned glm_grid(uint64_t items, uint64_t per_block, unsigned cap = 148u * 8u) {
    const uint64_t b = (items + per_block - 1) / per_block;
    return (unsigned)(b < 1 ? 1 : (b > cap ? cap : b));
}
#define SV_GLM_DONE() do { note_launch(1); return cudaGetLastError(); } while (0)

cudaError_t kda_decays_launch(float* eg, const uint16_t* f, const uint16_t* dt, const uint16_t* a_log, uint64_t heads, uint64_t head_dim, float lower,
                              uint64_t rows, cudaStream_t st) {
    kda_decays_kernel<<<glm_grid(rows * heads * head_dim, 256), 256, 0, st>>>(eg, f, dt, a_log, heads, head_dim, lower, rows);
    SV_GLM_DONE();
}

/* eg = null: the decays are made from f, dt and a_log (kda_step, kda_steps); else read (kda_steps_decayed) */
cudaError_t kda_steps_launch(float* S, const uint16_t* conved, const uint16_t* f, const float* eg, const uint16_t* b, const uint16_t* dt,
                             const uint16_t* a_log, const uint16_t* gate, const uint16_t* w, uint16_t* out, uint64_t heads, uint64_t head_dim, float lower,
                             float eps, uint64_t rows, unsigned int* over, cudaStream_t st) {
    if (heads == 0 || heads > 65535) return cudaErrorInvalidValue;
    const unsigned g = (unsigned)heads;
#define SV_KDA(D)                                                                                                                                   \
    do {                                                                                                                                            \
        if (eg) kda_steps_kernel<D, true><<<g, 1024, 0, st>>>(S, conved, f, eg, b, dt, a_log, gate, w, out, heads, lower, eps, rows, over);         \
        else kda_steps_kernel<D, false><<<g, 1024, 0, st>>>(S, conved, f, eg, b, dt, a_log, gate, w, out, heads, lower, eps, rows, over);           \
    } while (0)
    if (head_dim == 64) SV_KDA(64);
    else if (head_dim == 128) SV_KDA(128);
    else if (eg) kda_steps_any_kernel<true><<<g, 256, 0, st>>>(S, conved, f, eg, b, dt, a_log, gate, w, out, heads, head_dim, lower, eps, rows, over);
    else kda_steps_any_kernel<false><<<g, 256, 0, st>>>(S, conved, f, eg, b, dt, a_log, gate, w, out, heads, head_dim, lower, eps, rows, over);
#undef SV_KDA
    SV_GLM_DONE();
}

cudaError_t absorb_launch(uint16_t* out, const uint16_t* q, const uint16_t* W, uint64_t heads, uint64_t nope, uint64_t latent, uint64_t stride, float scale,
                          uint64_t rows, unsigned int* over, cudaStream_t st) {
    const bool wide = latent % 8 == 0 && (uintptr_t)W % 16 == 0;
    const uint64_t all = wide ? latent / 8 : latent;
    /* few (row, head) pairs: a head's columns are cut over up to four blocks so that the card has a block an SM or so */
    uint64_t parts = 1;
    while (parts < 4 && rows * heads * parts < 148 && all % (parts * 2) == 0 && all / (parts * 2) >= 8) parts *= 2;
    const uint64_t chunks = all / parts, across = chunks < 512 ? chunks : 512, slices = 512 / across;
    const size_t smem = (size_t)slices * (latent / parts) * sizeof(float);
    if (smem > 48 * 1024) return cudaErrorInvalidValue;
    const unsigned g = glm_grid(rows * heads * parts, 1, 148u * 16u);
    if (wide) absorb_kernel<true><<<g, 512, smem, st>>>(out, q, W, heads, nope, latent, stride, scale, rows, parts, over);
    else absorb_kernel<false><<<g, 512, smem, st>>>(out, q, W, heads, nope, latent, stride, scale, rows, parts, over);
    SV_GLM_DONE();
}
cudaError_t expand_launch(uint16_t* out, const uint16_t* o, const uint16_t* W, uint64_t heads, uint64_t width, uint64_t latent, uint64_t stride,
                          uint64_t offset, uint64_t rows, unsigned int* over, cudaStream_t st) {
    expand_kernel<<<glm_grid(rows * heads * width, 8, 148u * 16u), 256, 0, st>>>(out, o, W, heads, width, latent, stride, offset, rows, over);
    SV_GLM_DONE();
}

cudaError_t index_layernorm_launch(uint16_t* o, const uint16_t* x, const uint16_t* w, const uint16_t* b, uint64_t n, float eps, unsigned int* over,
                                   cudaStream_t st) {
    index_layernorm_kernel<<<1, 256, 0, st>>>(o, x, w, b, n, eps, over);
    SV_GLM_DONE();
}
cudaError_t index_pool_launch(uint16_t* pooled, const uint16_t* keys, const uint16_t* gates, const uint16_t* ape, uint64_t first, uint64_t pools, uint64_t dim,
                              uint64_t kpool, unsigned int* over, cudaStream_t st) {
    index_pool_kernel<<<glm_grid(pools * dim, 256), 256, 0, st>>>(pooled, keys, gates, ape, first, pools, dim, kpool, over);
    SV_GLM_DONE();
}
cudaError_t index_scores_launch(float* scores, uint64_t scores_row, const uint16_t* q, const uint16_t* w, const uint16_t* pooled, uint64_t heads, uint64_t dim,
                                uint64_t pools, uint64_t len0, uint64_t kpool, uint64_t rows, float scale, cudaStream_t st) {
    const uint64_t most = rows == 0 ? pools : (len0 + rows - 1) / kpool;
    const size_t smem = ((size_t)heads * (dim / 2 + 1) + 8 * (dim / 2)) * 4;
    if (dim % 2 == 0 && smem <= 48 * 1024 && heads < (1u << 16) && dim < (1u << 16) && rows <= 65535 && (uintptr_t)q % 4 == 0 && (uintptr_t)pooled % 4 == 0 &&
        (heads * dim) % 2 == 0) {
        const uint64_t urows = rows == 0 ? 1 : rows;
        unsigned gx = glm_grid(most, 8, 148u * 8u);
        if (urows > 1) { const unsigned per = (unsigned)((148u * 8u + urows - 1) / urows); if (gx > per) gx = per < 1 ? 1 : per; }
        index_scores_staged_kernel<<<dim3(gx, (unsigned)urows), 256, smem, st>>>(scores, scores_row, q, w, pooled, (uint32_t)heads, (uint32_t)dim, pools, len0,
                                                                                  kpool, rows, scale);
        SV_GLM_DONE();
    }
    index_scores_kernel<<<glm_grid((rows == 0 ? 1 : rows) * most, 8, 148u * 16u), 256, 0, st>>>(scores, scores_row, q, w, pooled, heads, dim, pools, len0, kpool,
                                                                                                 rows, scale);
    SV_GLM_DONE();
}
cudaError_t index_select_launch(uint32_t* index, uint64_t index_row, uint32_t* counts, const float* scores, uint64_t scores_row, uint64_t pools, uint64_t k,
                                uint64_t kpool, uint64_t tail_first, uint64_t tail, uint64_t len0, uint64_t rows, cudaStream_t st) {
    index_select_kernel<<<glm_grid(rows == 0 ? 1 : rows, 1, 4096u), 1024, 0, st>>>(index, index_row, counts, scores, scores_row, pools, k, kpool, tail_first,
                                                                                    tail, len0, rows);
    SV_GLM_DONE();
}
cudaError_t index_blocks_launch(float* out, const float* scores, uint64_t pools, uint64_t block, cudaStream_t st) {
    index_blocks_kernel<<<glm_grid((pools + block - 1) / block, 256), 256, 0, st>>>(out, scores, pools, block);
    SV_GLM_DONE();
}
cudaError_t index_gather_launch(uint16_t* out, uint64_t out_row, const uint16_t* src, const uint32_t* index, uint64_t index_row, const uint32_t* counts,
                                uint64_t most, uint64_t row, uint64_t rows, cudaStream_t st) {
    index_gather_kernel<<<glm_grid(rows * most * row, 256), 256, 0, st>>>(out, out_row, src, index, index_row, counts, most, row, rows);
    SV_GLM_DONE();
}

}  // namespace sv
