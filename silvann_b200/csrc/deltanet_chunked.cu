/* deltanet_chunked.cu — Gated DeltaNet over a run of positions, 64 at a time.
 *
 * The recurrence the doors word (engine/src/packages/nn/gpu/kernels/kernels.cuh:650-691, walked a position at a time by
 * deltanet_steps, :2131-2155) is, with kn = k/|k|, qs = q/|q|/sqrt(d), a = e^g:
 *     S_t = a_t S_{t-1} + kn_t d_t^T,      d_t = beta_t (v_t - a_t S_{t-1}^T kn_t),      o_t = S_t^T qs_t.
 * Unrolled inside a chunk that starts from state S_0, with G_t the running sum of g (so the decay from s to t is
 * e^(G_t - G_s)), every d_t is a combination of the chunk's own rows:
 *     (I + L) D = diag(beta) (V - diag(e^G) Kn S_0),        L[t][s] = beta_t e^(G_t - G_s) (kn_t · kn_s)   for s < t
 *     O = diag(e^G) Qs S_0 + M D,                           M[t][s] = e^(G_t - G_s) (qs_t · kn_s)          for s <= t
 *     S_C = e^(G_C) S_0 + Kn^T diag(e^(G_C - G)) D.
 * L, M and the inverse A = (I + L)^-1 diag(beta) depend on k, q, beta, g only — not on the state and not on the values —
 * so a first kernel makes them for every chunk of the run at once (a block a chunk and value head), and only the three
 * products with the state are left on the serial path, where a block owns 32 value columns of one head as in the
 * position-at-a-time kernel.  Everything is fp32 FMA: the state is an fp32 quantity and its parity bar is relative 1e-3
 * after thousands of positions, so no operand is rounded to a tensor-core input type.
 *
 * The read-out leaves here rounded to 16 bits with each block's sum of squares beside it, exactly as the recurrent
 * kernel leaves it, and the same norm-and-gate kernel finishes it. */
#include "common.cuh"
#include "kernels.h"
#include "kernels_deltanet.h"

namespace sv {

static constexpr int CH = 64;            /* positions a chunk */
static constexpr int CNC = 32;           /* value columns a block of the serial kernel */
/* per (sequence, chunk, value head), in floats: A [64][64], M [64][64], then the row vectors and the chunk's decay */
static constexpr int PREP_A = 0, PREP_M = CH * CH, PREP_VA = 2 * CH * CH, PREP_VB = PREP_VA + CH, PREP_VC = PREP_VB + CH,
                     PREP_GC = PREP_VC + CH, PREP_FLOATS = PREP_GC + 64;

struct ChunkParams {
    float* S;
    const uint16_t *conved, *beta, *g;
    uint16_t* out;
    float* ss;
    float* prep;
    unsigned int* over;
    uint32_t k_heads, v_heads, seqs;
    uint64_t rows, row0, seg_rows;       /* the call's rows; this launch covers [row0, row0 + seg_rows) */
    uint32_t chunks;                     /* chunks in this segment */
};

/* ---- kernel 1: everything about a chunk that does not depend on the state ------------------------------------ */
template <int D, int DT>
__global__ void __launch_bounds__(128) deltanet_prep_kernel(const ChunkParams P) {
    using E = Elem<DT>;
    constexpr int LD = D + 4;
    extern __shared__ float sm[];
    float* kf = sm;                      /* [64][LD] raw k */
    float* qf = kf + CH * LD;            /* [64][LD] raw q */
    float* Lm = qf + CH * LD;            /* [64][65] L, then X */
    float* Xm = Lm + CH * 65;            /* [64][65] */
    float* vk = Xm + CH * 65;            /* inv_k[64], inv_q[64], G[64], beta[64] */
    float* vq = vk + CH; float* vG = vq + CH; float* vb = vG + CH;
    const int tid = threadIdx.x;
    const uint32_t c = blockIdx.x % P.chunks, h = (blockIdx.x / P.chunks) % P.v_heads, b = blockIdx.x / (P.chunks * P.v_heads);
    const uint32_t rep = P.v_heads / P.k_heads, kh = h / rep;
    const uint64_t ch = (uint64_t)(2 * P.k_heads + P.v_heads) * D;
    const uint64_t t0 = P.row0 + (uint64_t)c * CH;
    const int n = (int)((P.row0 + P.seg_rows - t0) < CH ? (P.row0 + P.seg_rows - t0) : CH);
    const uint16_t* cv = P.conved + ((uint64_t)b * P.rows + t0) * ch;

    for (int i = tid; i < CH * D; i += 128) {
        const int t = i / D, e = i % D;
        kf[t * LD + e] = t < n ? E::to_float(cv[(uint64_t)t * ch + (P.k_heads + kh) * D + e]) : 0.f;
        qf[t * LD + e] = t < n ? E::to_float(cv[(uint64_t)t * ch + kh * D + e]) : 0.f;
    }
    __syncthreads();
    if (tid < CH) {
        float kk = 0.f, qq = 0.f;
        for (int e = 0; e < D; ++e) { kk += kf[tid * LD + e] * kf[tid * LD + e]; qq += qf[tid * LD + e] * qf[tid * LD + e]; }
        vk[tid] = 1.0f / sqrtf(kk + 1e-6f);
        vq[tid] = 1.0f / sqrtf(qq + 1e-6f) / sqrtf((float)D);
        const uint64_t hh = ((uint64_t)b * P.rows + t0 + tid) * P.v_heads + h;
        vb[tid] = tid < n ? E::to_float(P.beta[hh]) : 0.f;
        vG[tid] = tid < n ? E::to_float(P.g[hh]) : 0.f;
    }
    __syncthreads();
    if (tid == 0) { float run = 0.f; for (int t = 0; t < CH; ++t) { run += vG[t]; vG[t] = run; } }   /* G_t, flat past the chunk's end */
    __syncthreads();
    float* out = P.prep + (((uint64_t)b * P.chunks + c) * P.v_heads + h) * PREP_FLOATS;
    /* L (strictly lower) into shared memory, M (lower with its diagonal) straight to scratch */
    for (int i = tid; i < CH * CH; i += 128) {
        const int t = i / CH, s = i % CH;
        float kk = 0.f, qk = 0.f;
        if (s <= t && t < n) {
            const float* ks = kf + s * LD; const float* kt = kf + t * LD; const float* qt = qf + t * LD;
#pragma unroll 4
            for (int e = 0; e < D; e += 4) {
                const float4 a = *reinterpret_cast<const float4*>(ks + e), k4 = *reinterpret_cast<const float4*>(kt + e), q4 = *reinterpret_cast<const float4*>(qt + e);
                kk += a.x * k4.x + a.y * k4.y + a.z * k4.z + a.w * k4.w;
                qk += a.x * q4.x + a.y * q4.y + a.z * q4.z + a.w * q4.w;
            }
        }
        const float dec = (s <= t && t < n) ? expf(vG[t] - vG[s]) : 0.f;
        Lm[t * 65 + s] = s < t ? vb[t] * dec * vk[t] * vk[s] * kk : 0.f;
        out[PREP_M + i] = dec * vq[t] * vk[s] * qk;
    }
    __syncthreads();
    /* X = (I + L)^-1 by forward substitution, a thread a column: X[t][c] = [t == c] - sum_{s < t} L[t][s] X[s][c] */
    if (tid < CH) {
        const int col = tid;
        for (int t = 0; t < CH; ++t) {
            float x = (t == col) ? 1.f : 0.f;
            for (int s = col; s < t; ++s) x -= Lm[t * 65 + s] * Xm[s * 65 + col];
            Xm[t * 65 + col] = (t >= col) ? x : 0.f;
        }
    }
    __syncthreads();
    for (int i = tid; i < CH * CH; i += 128) {
        const int t = i / CH, s = i % CH;
        out[PREP_A + i] = (t < n && s < n) ? Xm[t * 65 + s] * vb[s] : 0.f;        /* A = X diag(beta) */
    }
    if (tid < CH) {
        const float Gn = vG[CH - 1];
        out[PREP_VA + tid] = expf(vG[tid]) * vk[tid];                 /* scales Kn S_0 rows: e^G_t / |k_t| */
        out[PREP_VB + tid] = expf(vG[tid]) * vq[tid];                 /* scales Q S_0 rows */
        out[PREP_VC + tid] = tid < n ? expf(Gn - vG[tid]) * vk[tid] : 0.f;   /* scales D rows into the state */
        if (tid == 0) out[PREP_GC] = expf(Gn);
    }
}

/* ---- kernel 2: the serial walk, a block a (sequence, value head, 32 columns) ------------------------------------- */
template <int D, int DT>
__global__ void __launch_bounds__(256, 1) deltanet_chunk_kernel(const ChunkParams P) {
    using E = Elem<DT>;
    constexpr int LD = D + 4, CB = D / CNC;
    extern __shared__ float sm[];
    float* Ss = sm;                      /* [D][32] the state block */
    float* kf = Ss + D * CNC;            /* [64][LD] raw k */
    float* qf = kf + CH * LD;            /* [64][LD] raw q */
    float* Am = qf + CH * LD;            /* [64][65] */
    float* Mm = Am + CH * 65;            /* [64][65] */
    float* Rm = Mm + CH * 65;            /* [64][32]: V - scaled Kn S_0, then D scaled for the state update */
    float* Dm = Rm + CH * CNC;           /* [64][32]: D */
    float* va = Dm + CH * CNC; float* vb = va + CH; float* vc = vb + CH; float* gc = vc + CH;
    const int tid = threadIdx.x;
    const uint32_t cb = blockIdx.x % CB, h = (blockIdx.x / CB) % P.v_heads, b = blockIdx.x / (CB * P.v_heads);
    const uint32_t rep = P.v_heads / P.k_heads, kh = h / rep;
    const uint64_t ch = (uint64_t)(2 * P.k_heads + P.v_heads) * D, vd = (uint64_t)P.v_heads * D;
    const int j0 = cb * CNC;
    float* Sg = P.S + ((uint64_t)b * P.v_heads + h) * D * D;
    for (int i = tid; i < D * CNC; i += 256) Ss[i] = Sg[(uint64_t)(i / CNC) * D + j0 + i % CNC];
    bool hit = false;
    const int ty = tid >> 3, tx = tid & 7;           /* 32 x 8: two rows and four columns of a 64 x 32 product a thread */

    for (uint32_t c = 0; c < P.chunks; ++c) {
        const uint64_t t0 = P.row0 + (uint64_t)c * CH;
        const int n = (int)((P.row0 + P.seg_rows - t0) < CH ? (P.row0 + P.seg_rows - t0) : CH);
        const uint16_t* cv = P.conved + ((uint64_t)b * P.rows + t0) * ch;
        const float* pr = P.prep + (((uint64_t)b * P.chunks + c) * P.v_heads + h) * PREP_FLOATS;
        __syncthreads();                              /* the previous chunk's readers are done with the buffers */
        for (int i = tid; i < CH * D; i += 256) {
            const int t = i / D, e = i % D;
            kf[t * LD + e] = t < n ? E::to_float(cv[(uint64_t)t * ch + (P.k_heads + kh) * D + e]) : 0.f;
            qf[t * LD + e] = t < n ? E::to_float(cv[(uint64_t)t * ch + kh * D + e]) : 0.f;
        }
        for (int i = tid; i < CH * CH; i += 256) { Am[(i / CH) * 65 + i % CH] = pr[PREP_A + i]; Mm[(i / CH) * 65 + i % CH] = pr[PREP_M + i]; }
        if (tid < CH) { va[tid] = pr[PREP_VA + tid]; vb[tid] = pr[PREP_VB + tid]; vc[tid] = pr[PREP_VC + tid]; if (tid == 0) gc[0] = pr[PREP_GC]; }
        for (int i = tid; i < CH * CNC; i += 256) {
            const int t = i / CNC, jj = i % CNC;
            Rm[i] = t < n ? E::to_float(cv[(uint64_t)t * ch + (uint64_t)2 * P.k_heads * D + (uint64_t)h * D + j0 + jj]) : 0.f;
        }
        __syncthreads();

        /* (1) K S_0 and Q S_0 together: rows 2ty, 2ty+1; columns 4tx..4tx+3 */
        float ks[2][4] = {}, qs[2][4] = {};
        {
            const float* k0 = kf + (2 * ty) * LD; const float* k1 = k0 + LD;
            const float* q0 = qf + (2 * ty) * LD; const float* q1 = q0 + LD;
#pragma unroll 2
            for (int i = 0; i < D; i += 4) {
                const float4 a0 = *reinterpret_cast<const float4*>(k0 + i), a1 = *reinterpret_cast<const float4*>(k1 + i);
                const float4 b0 = *reinterpret_cast<const float4*>(q0 + i), b1 = *reinterpret_cast<const float4*>(q1 + i);
                const float ka0[4] = {a0.x, a0.y, a0.z, a0.w}, ka1[4] = {a1.x, a1.y, a1.z, a1.w};
                const float qa0[4] = {b0.x, b0.y, b0.z, b0.w}, qa1[4] = {b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float4 s4 = *reinterpret_cast<const float4*>(Ss + (i + u) * CNC + 4 * tx);
                    const float sv4[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        ks[0][x] += ka0[u] * sv4[x]; ks[1][x] += ka1[u] * sv4[x];
                        qs[0][x] += qa0[u] * sv4[x]; qs[1][x] += qa1[u] * sv4[x];
                    }
                }
            }
        }
        /* R = V - diag(e^G / |k|) K S_0 */
#pragma unroll
        for (int rr = 0; rr < 2; ++rr)
#pragma unroll
            for (int x = 0; x < 4; ++x) Rm[(2 * ty + rr) * CNC + 4 * tx + x] -= va[2 * ty + rr] * ks[rr][x];
        __syncthreads();
        /* (2) D = A R, A lower triangular */
        float dd[2][4] = {};
        for (int s = 0; s <= 2 * ty + 1; ++s) {
            const float4 r4 = *reinterpret_cast<const float4*>(Rm + s * CNC + 4 * tx);
            const float a0 = Am[(2 * ty) * 65 + s], a1 = Am[(2 * ty + 1) * 65 + s];
            dd[0][0] += a0 * r4.x; dd[0][1] += a0 * r4.y; dd[0][2] += a0 * r4.z; dd[0][3] += a0 * r4.w;
            dd[1][0] += a1 * r4.x; dd[1][1] += a1 * r4.y; dd[1][2] += a1 * r4.z; dd[1][3] += a1 * r4.w;
        }
#pragma unroll
        for (int rr = 0; rr < 2; ++rr)
#pragma unroll
            for (int x = 0; x < 4; ++x) Dm[(2 * ty + rr) * CNC + 4 * tx + x] = dd[rr][x];
        __syncthreads();
        /* (3) O = diag(e^G / |q| / sqrt d) Q S_0 + M D, rounded, with the block's sum of squares for the norm */
        float oo[2][4];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr)
#pragma unroll
            for (int x = 0; x < 4; ++x) oo[rr][x] = vb[2 * ty + rr] * qs[rr][x];
        for (int s = 0; s <= 2 * ty + 1; ++s) {
            const float4 d4 = *reinterpret_cast<const float4*>(Dm + s * CNC + 4 * tx);
            const float m0 = Mm[(2 * ty) * 65 + s], m1 = Mm[(2 * ty + 1) * 65 + s];
            oo[0][0] += m0 * d4.x; oo[0][1] += m0 * d4.y; oo[0][2] += m0 * d4.z; oo[0][3] += m0 * d4.w;
            oo[1][0] += m1 * d4.x; oo[1][1] += m1 * d4.y; oo[1][2] += m1 * d4.z; oo[1][3] += m1 * d4.w;
        }
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            const int t = 2 * ty + rr;
            float sq = 0.f;
            uint16_t w[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) { w[x] = E::from_float(oo[rr][x], hit); const float f = E::to_float(w[x]); sq += f * f; }
            for (int x = 1; x < 8; x <<= 1) sq += __shfl_xor_sync(0xffffffffu, sq, x);
            if (t < n) {
                uint16_t* orow = P.out + ((uint64_t)b * P.rows + t0 + t) * vd + (uint64_t)h * D + j0 + 4 * tx;
                *reinterpret_cast<uint2*>(orow) = make_uint2((uint32_t)w[0] | ((uint32_t)w[1] << 16), (uint32_t)w[2] | ((uint32_t)w[3] << 16));
                if (tx == 0) P.ss[(((uint64_t)b * P.rows + t0 + t) * P.v_heads + h) * CB + cb] = sq;
            }
        }
        /* the state update reads D scaled by e^(G_C - G_t) / |k_t|: scale it in place (every reader of D is past) */
        __syncthreads();
        for (int i = tid; i < CH * CNC; i += 256) Dm[i] *= vc[i / CNC];
        __syncthreads();
        /* (4) S = e^(G_C) S_0 + K^T D': rows 4(tid/8)..+3 of the state for D = 128 (D/32 rows a thread), columns 4tx..+3 */
        {
            constexpr int RP = D / 32;                 /* state rows a thread */
            const int i0 = (tid >> 3) * RP;
            float acc[RP][4];
            const float g = gc[0];
#pragma unroll
            for (int a = 0; a < RP; ++a) {
                const float4 s4 = *reinterpret_cast<const float4*>(Ss + (i0 + a) * CNC + 4 * tx);
                acc[a][0] = g * s4.x; acc[a][1] = g * s4.y; acc[a][2] = g * s4.z; acc[a][3] = g * s4.w;
            }
#pragma unroll 4
            for (int t = 0; t < CH; ++t) {
                const float4 d4 = *reinterpret_cast<const float4*>(Dm + t * CNC + 4 * tx);
#pragma unroll
                for (int a = 0; a < RP; ++a) {
                    const float kv = kf[t * LD + i0 + a];
                    acc[a][0] += kv * d4.x; acc[a][1] += kv * d4.y; acc[a][2] += kv * d4.z; acc[a][3] += kv * d4.w;
                }
            }
            __syncthreads();                           /* every thread has read the old state */
#pragma unroll
            for (int a = 0; a < RP; ++a) *reinterpret_cast<float4*>(Ss + (i0 + a) * CNC + 4 * tx) = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
        }
    }
    __syncthreads();
    for (int i = tid; i < D * CNC; i += 256) Sg[(uint64_t)(i / CNC) * D + j0 + i % CNC] = Ss[i];
    if (hit && P.over) atomicOr(P.over, SV_FAULT_OVERFLOW);
}

/* ---------------------------------------------------------------------------------------------------------- */

bool deltanet_chunked_fits(const DeltaCall& c) {
    return (c.head_dim == 64 || c.head_dim == 128) && c.rows >= 32 && ((uintptr_t)c.out & 7u) == 0 && ((uintptr_t)c.S & 15u) == 0;
}

size_t deltanet_chunked_scratch_floats(const DeltaCall& c) {
    const uint64_t seg = c.rows < 2048 ? c.rows : 2048;
    return (size_t)c.seqs * ((seg + CH - 1) / CH) * c.v_heads * PREP_FLOATS;
}

template <int D, int DT>
static cudaError_t launch_chunked(const DeltaCall& c, float* ss, float* prep) {
    constexpr int LD = D + 4;
    const size_t smem1 = (size_t)(2 * CH * LD + 2 * CH * 65 + 4 * CH) * sizeof(float);
    const size_t smem2 = (size_t)(D * CNC + 2 * CH * LD + 2 * CH * 65 + 2 * CH * CNC + 4 * CH) * sizeof(float);
    static bool attr_set[64] = {};
    int dev = 0; cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(deltanet_prep_kernel<D, DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(deltanet_chunk_kernel<D, DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    ChunkParams P;
    P.S = c.S; P.conved = c.conved; P.beta = c.beta; P.g = c.g; P.out = c.out; P.ss = ss; P.prep = prep; P.over = c.over;
    P.k_heads = c.k_heads; P.v_heads = c.v_heads; P.seqs = c.seqs; P.rows = c.rows;
    for (uint64_t row0 = 0; row0 < c.rows; row0 += 2048) {
        P.row0 = row0; P.seg_rows = (c.rows - row0) < 2048 ? (c.rows - row0) : 2048; P.chunks = (uint32_t)((P.seg_rows + CH - 1) / CH);
        deltanet_prep_kernel<D, DT><<<c.seqs * c.v_heads * P.chunks, 128, smem1, c.stream>>>(P);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
        deltanet_chunk_kernel<D, DT><<<c.seqs * c.v_heads * (D / CNC), 256, smem2, c.stream>>>(P);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
        note_launch(2);
    }
    return cudaSuccess;
}

cudaError_t deltanet_chunked_launch(const DeltaCall& c, float* ss, float* prep) {
#define SV_DC(DD) (c.dtype == SV_DTYPE_BF16 ? launch_chunked<DD, SV_DTYPE_BF16>(c, ss, prep) : launch_chunked<DD, SV_DTYPE_FP16>(c, ss, prep))
    if (c.head_dim == 64) return SV_DC(64);
    if (c.head_dim == 128) return SV_DC(128);
#undef SV_DC
    return cudaErrorInvalidValue;
}

}  // namespace sv
