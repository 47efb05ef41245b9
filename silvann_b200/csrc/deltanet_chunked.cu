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

/* 16-byte asynchronous copies global -> shared; `bytes` of 0 writes zeros and reads nothing */
__device__ __forceinline__ void cp_async16(void* dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int DT> __device__ __forceinline__ void unpack4(uint2 u, float* f) {
    const float2 a = Elem<DT>::unpack2(u.x), b = Elem<DT>::unpack2(u.y);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

/* ---- kernel 1: everything about a chunk that does not depend on the state ------------------------------------
 * A block a (sequence, chunk, KEY head), 256 threads.  The two Gram products K K^T and Q K^T belong to the key head and
 * are made once, register-tiled (a thread owns rows ti, ti+16, ti+32, ti+48 against si, si+16, ..., so that the 16
 * lanes that differ in si read 16 consecutive rows of shared memory); then, two value heads of the key head at a time,
 * L is built transposed, (I + L)^-1 comes out of a right-looking substitution that lives in registers (a thread a
 * column, 64 running rows, the loop fully unrolled so that L is read four rows at a load), and A, M and the row vectors
 * go to scratch. */
template <int D, int DT>
__global__ void __launch_bounds__(256, 2) deltanet_prep_kernel(const ChunkParams P) {
    using E = Elem<DT>;
    constexpr int LD = D + 4, GL = CH + 1, TL = CH + 4, CPR = D / 8;
    extern __shared__ __align__(16) float sm[];
    float* kf = sm;                      /* [64][LD] raw k */
    float* qf = kf + CH * LD;            /* [64][LD] raw q */
    float* KK = qf + CH * LD;            /* [64][65] k_t . k_s, s <= t */
    float* QK = KK + CH * GL;            /* [64][65] q_t . k_s, s <= t */
    float* ik = QK + CH * GL;            /* 1 / |k_t| */
    float* iq = ik + CH;                 /* 1 / |q_t| / sqrt(d) */
    float* vb = iq + CH;                 /* [2][64] beta */
    float* vG = vb + 2 * CH;             /* [2][64] running sums of g */
    float* LT = sm;                      /* [2][64][TL]: L transposed, over k and q once the Gram products are done */
    static_assert(2 * CH * TL <= 2 * CH * LD, "L transposed fits where k and q were");
    const int tid = threadIdx.x, lane = tid & 31;
    const uint32_t c = blockIdx.x % P.chunks, kh = (blockIdx.x / P.chunks) % P.k_heads, b = blockIdx.x / (P.chunks * P.k_heads);
    const uint32_t rep = P.v_heads / P.k_heads;
    const uint64_t ch = (uint64_t)(2 * P.k_heads + P.v_heads) * D;
    const uint64_t t0 = P.row0 + (uint64_t)c * CH;
    const int n = (int)((P.row0 + P.seg_rows - t0) < CH ? (P.row0 + P.seg_rows - t0) : CH);
    const uint16_t* cv = P.conved + ((uint64_t)b * P.rows + t0) * ch;

    /* k and q as fp32, with each row's sum of squares folded over the lanes that share the row */
    for (int i = tid; i < 2 * CH * CPR; i += 256) {
        const int which = i / (CH * CPR), r = (i / CPR) % CH, p = i % CPR;
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (r < n) raw = *reinterpret_cast<const uint4*>(cv + (uint64_t)r * ch + (uint64_t)(which ? kh : P.k_heads + kh) * D + p * 8);
        float f[8];
        unpack4<DT>(make_uint2(raw.x, raw.y), f); unpack4<DT>(make_uint2(raw.z, raw.w), f + 4);
        float* dst = (which ? qf : kf) + r * LD + p * 8;
        *reinterpret_cast<float4*>(dst) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(f[4], f[5], f[6], f[7]);
        float ssq = 0.f;
#pragma unroll
        for (int x = 0; x < 8; ++x) ssq += f[x] * f[x];
#pragma unroll
        for (int x = 1; x < CPR; x <<= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, x);
        if (p == 0) {
            if (which) iq[r] = 1.0f / sqrtf(ssq + 1e-6f) / sqrtf((float)D);
            else       ik[r] = 1.0f / sqrtf(ssq + 1e-6f);
        }
    }
    __syncthreads();
    {
        const int ti = tid >> 4, si = tid & 15;
        float kk[4][4] = {}, qk[4][4] = {};
#pragma unroll 2
        for (int e = 0; e < D; e += 4) {
            float4 kt[4], qt[4], ks[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                kt[a] = *reinterpret_cast<const float4*>(kf + (ti + 16 * a) * LD + e);
                qt[a] = *reinterpret_cast<const float4*>(qf + (ti + 16 * a) * LD + e);
                ks[a] = *reinterpret_cast<const float4*>(kf + (si + 16 * a) * LD + e);
            }
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int bb = 0; bb <= a; ++bb) {       /* rows ti+16a against si+16bb: below the diagonal when a > bb */
                    kk[a][bb] += kt[a].x * ks[bb].x + kt[a].y * ks[bb].y + kt[a].z * ks[bb].z + kt[a].w * ks[bb].w;
                    qk[a][bb] += qt[a].x * ks[bb].x + qt[a].y * ks[bb].y + qt[a].z * ks[bb].z + qt[a].w * ks[bb].w;
                }
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int bb = 0; bb <= a; ++bb) {
                KK[(ti + 16 * a) * GL + si + 16 * bb] = kk[a][bb];
                QK[(ti + 16 * a) * GL + si + 16 * bb] = qk[a][bb];
            }
    }

    for (uint32_t p0 = 0; p0 < rep; p0 += 2) {
        const int nh = (int)((rep - p0) < 2u ? (rep - p0) : 2u);
        const int hh = (tid >> 6) & 1, t = tid & 63;
        const uint32_t h = kh * rep + p0 + hh;
        __syncthreads();                  /* the Gram products are written; the last pass's readers are done */
        if (tid < 128) {
            float gsum = 0.f, be = 0.f;
            if (hh < nh && t < n) {
                const uint64_t at = ((uint64_t)b * P.rows + t0 + t) * P.v_heads + h;
                be = E::to_float(P.beta[at]); gsum = E::to_float(P.g[at]);
            }
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const float y = __shfl_up_sync(0xffffffffu, gsum, o); if (lane >= o) gsum += y; }
            vb[tid] = be; vG[tid] = gsum;
        }
        __syncthreads();
        if (tid < 128 && (tid & 32)) vG[tid] += vG[(tid & ~63) + 31];      /* G_t, flat past the chunk's end */
        __syncthreads();
        /* L transposed into shared memory (t runs fastest), M straight to scratch (s runs fastest) */
        for (int i = tid; i < nh * CH * CH; i += 256) {
            const int hq = i / (CH * CH), s = (i / CH) % CH, tt = i % CH;
            float l = 0.f;
            if (s < tt && tt < n) l = vb[hq * CH + tt] * expf(vG[hq * CH + tt] - vG[hq * CH + s]) * ik[tt] * ik[s] * KK[tt * GL + s];
            LT[(hq * CH + s) * TL + tt] = l;
        }
        for (int i = tid; i < nh * CH * CH; i += 256) {
            const int hq = i / (CH * CH), tt = (i / CH) % CH, s = i % CH;
            float m = 0.f;
            if (s <= tt && tt < n) m = expf(vG[hq * CH + tt] - vG[hq * CH + s]) * iq[tt] * ik[s] * QK[tt * GL + s];
            P.prep[(((uint64_t)b * P.chunks + c) * P.v_heads + kh * rep + p0 + hq) * PREP_FLOATS + PREP_M + tt * CH + s] = m;
        }
        __syncthreads();
        float* out = P.prep + (((uint64_t)b * P.chunks + c) * P.v_heads + h) * PREP_FLOATS;
        if (tid < 128) {
            if (hh < nh) {
                /* X = (I + L)^-1, column t of it: x_s is final once every s' < s has been taken out of the rows below */
                float x[CH];
#pragma unroll
                for (int r = 0; r < CH; ++r) x[r] = (r == t) ? 1.f : 0.f;
#pragma unroll
                for (int s = 0; s < CH - 1; ++s) {
                    const float xs = x[s];
                    const float* row = LT + (hh * CH + s) * TL;
#pragma unroll
                    for (int tg = ((s + 1) / 4) * 4; tg < CH; tg += 4) {
                        const float4 l = *reinterpret_cast<const float4*>(row + tg);
                        if (tg + 0 > s) x[tg + 0] -= l.x * xs;
                        if (tg + 1 > s) x[tg + 1] -= l.y * xs;
                        if (tg + 2 > s) x[tg + 2] -= l.z * xs;
                        if (tg + 3 > s) x[tg + 3] -= l.w * xs;
                    }
                }
                const float be = vb[hh * CH + t];
#pragma unroll
                for (int r = 0; r < CH; ++r) out[PREP_A + r * CH + t] = x[r] * be;       /* A = X diag(beta) */
            }
        } else if (hh < nh) {
            const float G = vG[hh * CH + t], Gn = vG[hh * CH + CH - 1];
            out[PREP_VA + t] = expf(G) * ik[t];                        /* scales Kn S_0 rows: e^G_t / |k_t| */
            out[PREP_VB + t] = expf(G) * iq[t];                        /* scales Q S_0 rows */
            out[PREP_VC + t] = t < n ? expf(Gn - G) * ik[t] : 0.f;     /* scales D rows into the state */
            if (t == 0) out[PREP_GC] = expf(Gn);
        }
    }
}

/* ---- kernel 2: the serial walk, a block a (sequence, value head, 32 columns) -------------------------------------
 * What a chunk needs — its k, q and v rows as they lie in the cache (16 bits), A, M and the row vectors from kernel 1 —
 * is fetched with 16-byte asynchronous copies into one of two stages while the chunk before it is being computed, so the
 * serial path waits on arithmetic and not on memory.  k and q stay 16-bit in shared memory and widen as they are read. */
template <int D> struct ChunkSmem {
    static constexpr int LDH = D + 8;                      /* halves a k or q row: 16-byte rows, 8 banks apart for row pairs */
    static constexpr int TL = CH + 4;                      /* floats an A or M row */
    static constexpr size_t STATE = (size_t)D * CNC * 4, RD = (size_t)CH * CNC * 4;
    static constexpr size_t KQ = (size_t)CH * LDH * 2, V = (size_t)CH * CNC * 2, AM = (size_t)CH * TL * 4, VEC = 4 * CH * 4;
    static constexpr size_t STAGE = 2 * KQ + V + 2 * AM + VEC;
    static constexpr size_t TOTAL = STATE + 2 * RD + 2 * STAGE;
};

template <int D, int DT>
__global__ void __launch_bounds__(256, 1) deltanet_chunk_kernel(const ChunkParams P) {
    using E = Elem<DT>;
    using L = ChunkSmem<D>;
    constexpr int LDH = L::LDH, TL = L::TL, CB = D / CNC, CPR = D / 8;
    extern __shared__ __align__(16) unsigned char smb[];
    float* Ss = reinterpret_cast<float*>(smb);                       /* [D][32] the state block */
    float* Rm = reinterpret_cast<float*>(smb + L::STATE);            /* [64][32]: V - scaled Kn S_0 */
    float* Dm = Rm + CH * CNC;                                       /* [64][32]: D, then D scaled for the state update */
    unsigned char* stage0 = smb + L::STATE + 2 * L::RD;
    const int tid = threadIdx.x;
    const uint32_t cb = blockIdx.x % CB, h = (blockIdx.x / CB) % P.v_heads, b = blockIdx.x / (CB * P.v_heads);
    const uint32_t rep = P.v_heads / P.k_heads, kh = h / rep;
    const uint64_t ch = (uint64_t)(2 * P.k_heads + P.v_heads) * D, vd = (uint64_t)P.v_heads * D;
    const int j0 = cb * CNC;
    float* Sg = P.S + ((uint64_t)b * P.v_heads + h) * D * D;

    auto fetch = [&](uint32_t c) {
        unsigned char* st = stage0 + (size_t)(c & 1u) * L::STAGE;
        uint16_t* kr = reinterpret_cast<uint16_t*>(st);
        uint16_t* qr = reinterpret_cast<uint16_t*>(st + L::KQ);
        uint16_t* vr = reinterpret_cast<uint16_t*>(st + 2 * L::KQ);
        float* Am = reinterpret_cast<float*>(st + 2 * L::KQ + L::V);
        float* Mm = Am + CH * TL;
        float* vec = Mm + CH * TL;
        const uint64_t t0 = P.row0 + (uint64_t)c * CH;
        const int n = (int)((P.row0 + P.seg_rows - t0) < CH ? (P.row0 + P.seg_rows - t0) : CH);
        const uint16_t* cv = P.conved + ((uint64_t)b * P.rows + t0) * ch;
        const float* pr = P.prep + (((uint64_t)b * P.chunks + c) * P.v_heads + h) * PREP_FLOATS;
        for (int i = tid; i < 2 * CH * CPR; i += 256) {
            const int which = i / (CH * CPR), r = (i / CPR) % CH, p = i % CPR;
            const int rr = r < n ? r : 0;
            cp_async16((which ? qr : kr) + r * LDH + p * 8, cv + (uint64_t)rr * ch + (uint64_t)(which ? kh : P.k_heads + kh) * D + p * 8, r < n ? 16u : 0u);
        }
        for (int i = tid; i < CH * (CNC / 8); i += 256) {
            const int r = i / (CNC / 8), p = i % (CNC / 8);
            const int rr = r < n ? r : 0;
            cp_async16(vr + r * CNC + p * 8, cv + (uint64_t)rr * ch + (uint64_t)2 * P.k_heads * D + (uint64_t)h * D + j0 + p * 8, r < n ? 16u : 0u);
        }
        for (int i = tid; i < 2 * CH * (CH / 4); i += 256) {
            const int which = i / (CH * (CH / 4)), r = (i / (CH / 4)) % CH, p = i % (CH / 4);
            cp_async16((which ? Mm : Am) + r * TL + p * 4, pr + (which ? PREP_M : PREP_A) + r * CH + p * 4, 16u);
        }
        if (tid < CH) cp_async16(vec + tid * 4, pr + PREP_VA + tid * 4, 16u);
    };

    fetch(0);
    cp_async_commit();
    for (int i = tid; i < D * CNC; i += 256) Ss[i] = Sg[(uint64_t)(i / CNC) * D + j0 + i % CNC];
    bool hit = false;
    const int ty = tid >> 3, tx = tid & 7;           /* 32 x 8: two rows and four columns of a 64 x 32 product a thread */

    for (uint32_t c = 0; c < P.chunks; ++c) {
        const uint64_t t0 = P.row0 + (uint64_t)c * CH;
        const int n = (int)((P.row0 + P.seg_rows - t0) < CH ? (P.row0 + P.seg_rows - t0) : CH);
        unsigned char* st = stage0 + (size_t)(c & 1u) * L::STAGE;
        const uint16_t* kr = reinterpret_cast<const uint16_t*>(st);
        const uint16_t* qr = reinterpret_cast<const uint16_t*>(st + L::KQ);
        const uint16_t* vr = reinterpret_cast<const uint16_t*>(st + 2 * L::KQ);
        const float* Am = reinterpret_cast<const float*>(st + 2 * L::KQ + L::V);
        const float* Mm = Am + CH * TL;
        const float* va = Mm + CH * TL; const float* vb = va + CH; const float* vc = vb + CH; const float* gc = vc + CH;
        /* the other stage's last readers passed the barrier ahead of the state write of the chunk before: refill it */
        if (c + 1 < P.chunks) fetch(c + 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();

        /* (1) K S_0 and Q S_0 together: rows 2ty, 2ty+1; columns 4tx..4tx+3 */
        float ks[2][4] = {}, qs[2][4] = {};
        {
            const uint16_t* k0 = kr + (2 * ty) * LDH; const uint16_t* k1 = k0 + LDH;
            const uint16_t* q0 = qr + (2 * ty) * LDH; const uint16_t* q1 = q0 + LDH;
#pragma unroll 2
            for (int i = 0; i < D; i += 4) {
                float ka0[4], ka1[4], qa0[4], qa1[4];
                unpack4<DT>(*reinterpret_cast<const uint2*>(k0 + i), ka0); unpack4<DT>(*reinterpret_cast<const uint2*>(k1 + i), ka1);
                unpack4<DT>(*reinterpret_cast<const uint2*>(q0 + i), qa0); unpack4<DT>(*reinterpret_cast<const uint2*>(q1 + i), qa1);
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
        for (int rr = 0; rr < 2; ++rr) {
            float v4[4];
            unpack4<DT>(*reinterpret_cast<const uint2*>(vr + (2 * ty + rr) * CNC + 4 * tx), v4);
            const float a = va[2 * ty + rr];
            *reinterpret_cast<float4*>(Rm + (2 * ty + rr) * CNC + 4 * tx) =
                make_float4(v4[0] - a * ks[rr][0], v4[1] - a * ks[rr][1], v4[2] - a * ks[rr][2], v4[3] - a * ks[rr][3]);
        }
        __syncthreads();
        /* (2) D = A R, A lower triangular */
        float dd[2][4] = {};
        for (int s = 0; s <= 2 * ty + 1; ++s) {
            const float4 r4 = *reinterpret_cast<const float4*>(Rm + s * CNC + 4 * tx);
            const float a0 = Am[(2 * ty) * TL + s], a1 = Am[(2 * ty + 1) * TL + s];
            dd[0][0] += a0 * r4.x; dd[0][1] += a0 * r4.y; dd[0][2] += a0 * r4.z; dd[0][3] += a0 * r4.w;
            dd[1][0] += a1 * r4.x; dd[1][1] += a1 * r4.y; dd[1][2] += a1 * r4.z; dd[1][3] += a1 * r4.w;
        }
#pragma unroll
        for (int rr = 0; rr < 2; ++rr)
            *reinterpret_cast<float4*>(Dm + (2 * ty + rr) * CNC + 4 * tx) = make_float4(dd[rr][0], dd[rr][1], dd[rr][2], dd[rr][3]);
        __syncthreads();
        /* (3) O = diag(e^G / |q| / sqrt d) Q S_0 + M D, rounded, with the block's sum of squares for the norm */
        float oo[2][4];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr)
#pragma unroll
            for (int x = 0; x < 4; ++x) oo[rr][x] = vb[2 * ty + rr] * qs[rr][x];
        for (int s = 0; s <= 2 * ty + 1; ++s) {
            const float4 d4 = *reinterpret_cast<const float4*>(Dm + s * CNC + 4 * tx);
            const float m0 = Mm[(2 * ty) * TL + s], m1 = Mm[(2 * ty + 1) * TL + s];
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
        /* (4) S = e^(G_C) S_0 + K^T D': D/32 rows of the state a thread, columns 4tx..+3 */
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
                float kv[4];
                if constexpr (RP == 4) unpack4<DT>(*reinterpret_cast<const uint2*>(kr + t * LDH + i0), kv);
                else { const float2 k2 = E::unpack2(*reinterpret_cast<const uint32_t*>(kr + t * LDH + i0)); kv[0] = k2.x; kv[1] = k2.y; }
#pragma unroll
                for (int a = 0; a < RP; ++a) {
                    acc[a][0] += kv[a] * d4.x; acc[a][1] += kv[a] * d4.y; acc[a][2] += kv[a] * d4.z; acc[a][3] += kv[a] * d4.w;
                }
            }
            __syncthreads();                           /* every thread has read the old state and this chunk's stage */
#pragma unroll
            for (int a = 0; a < RP; ++a) *reinterpret_cast<float4*>(Ss + (i0 + a) * CNC + 4 * tx) = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
        }
    }
    cp_async_wait<0>();
    __syncthreads();
    for (int i = tid; i < D * CNC; i += 256) Sg[(uint64_t)(i / CNC) * D + j0 + i % CNC] = Ss[i];
    if (hit && P.over) atomicOr(P.over, SV_FAULT_OVERFLOW);
}

/* ---------------------------------------------------------------------------------------------------------- */

bool deltanet_chunked_fits(const DeltaCall& c) {
    return (c.head_dim == 64 || c.head_dim == 128) && c.rows >= 32 && ((uintptr_t)c.out & 7u) == 0 && ((uintptr_t)c.S & 15u) == 0 &&
           ((uintptr_t)c.conved & 15u) == 0;       /* rows of the cache are fetched 16 bytes at a time */
}

size_t deltanet_chunked_scratch_floats(const DeltaCall& c) {
    const uint64_t seg = c.rows < 2048 ? c.rows : 2048;
    return (size_t)c.seqs * ((seg + CH - 1) / CH) * c.v_heads * PREP_FLOATS;
}

template <int D, int DT>
static cudaError_t launch_chunked(const DeltaCall& c, float* ss, float* prep) {
    constexpr int LD = D + 4;
    const size_t smem1 = (size_t)(2 * CH * LD + 2 * CH * (CH + 1) + 6 * CH) * sizeof(float);
    const size_t smem2 = ChunkSmem<D>::TOTAL;
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
        deltanet_prep_kernel<D, DT><<<c.seqs * c.k_heads * P.chunks, 256, smem1, c.stream>>>(P);
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
