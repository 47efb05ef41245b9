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
 * position-at-a-time kernel.  The state is an fp32 quantity held to a relative 1e-3 after thousands of positions, so
 * nothing of it is rounded to a 16-bit tensor-core type: the Gram products and the triangular products are fp32 FMA, and
 * the two products with the state run on the tensor cores in TF32 with the state (or D) split into two terms — k and q
 * are exact in TF32, the pair of terms carries 21 significand bits.
 *
 * The read-out leaves here rounded to 16 bits with each block's sum of squares beside it, exactly as the recurrent
 * kernel leaves it, and the same norm-and-gate kernel finishes it. */
#include "common.cuh"
#include <atomic>
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
    float* readout;
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

/* D (16 x 8, fp32) += A (16 x 8) · B (8 x 8), TF32 inputs: the warp MMA of the two products with the state */
__device__ __forceinline__ void mma_tf32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
/* a 16-bit input as TF32 bits: exact, both types have at most 10 significand bits */
template <int DT> __device__ __forceinline__ uint32_t tf32_of(uint16_t h) { return __float_as_uint(Elem<DT>::to_float(h)); }
/* an fp32 number as two TF32 terms, hi + lo: hi its top 19 bits, lo the rest (the MMA reads lo's top 19 bits), so the
 * pair carries 21 significand bits — a relative 2^-21 against the 1e-3 the state is held to */
__device__ __forceinline__ void tf32_split(float x, uint32_t& hi, uint32_t& lo) {
    hi = __float_as_uint(x) & 0xffffe000u;
    lo = __float_as_uint(x - __uint_as_float(hi));
}

/* ---- kernel 1: everything about a chunk that does not depend on the state ------------------------------------
 * A block a (sequence, chunk, KEY head), 256 threads.  The two Gram products K K^T and Q K^T belong to the key head and
 * are made once, below the diagonal, on the tensor cores (TF32 holds k and q exactly; the sums are fp32); then, two
 * value heads of the key head at a time, L is built transposed, (I + L)^-1 comes out of a right-looking substitution
 * that lives in registers (a thread a column, 64 running rows, the loop fully unrolled so that L is read four rows at a
 * load), and A, M and the row vectors
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
        /* K K^T and Q K^T below the diagonal on the tensor cores: k and q are exact in TF32 and the sums are fp32, so the
         * products are the fp32 ones.  A warp owns 16 rows t and every other 8-column tile s up to its diagonal. */
        const int warp = tid >> 5, g8 = lane >> 2, t4 = lane & 3;
        const int r1 = (warp & 3) * 16;
        const float* kA = kf + (r1 + g8) * LD + t4; const float* kB = kA + 8 * LD;
        const float* qA = qf + (r1 + g8) * LD + t4; const float* qB = qA + 8 * LD;
        for (int nt = (warp >> 2); nt * 8 <= r1 + 15; nt += 2) {
            float ck[4] = {}, cq[4] = {};
            const float* sB = kf + (nt * 8 + g8) * LD + t4;                  /* B[k][n = s] = K[s][k] */
#pragma unroll 4
            for (int k0 = 0; k0 < D; k0 += 8) {
                const uint32_t b0 = __float_as_uint(sB[k0]), b1 = __float_as_uint(sB[k0 + 4]);
                mma_tf32(ck, __float_as_uint(kA[k0]), __float_as_uint(kB[k0]), __float_as_uint(kA[k0 + 4]), __float_as_uint(kB[k0 + 4]), b0, b1);
                mma_tf32(cq, __float_as_uint(qA[k0]), __float_as_uint(qB[k0]), __float_as_uint(qA[k0 + 4]), __float_as_uint(qB[k0 + 4]), b0, b1);
            }
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                float* kd = KK + (r1 + g8 + 8 * hh) * GL + nt * 8 + 2 * t4;
                float* qd = QK + (r1 + g8 + 8 * hh) * GL + nt * 8 + 2 * t4;
                kd[0] = ck[2 * hh]; kd[1] = ck[2 * hh + 1];
                qd[0] = cq[2 * hh]; qd[1] = cq[2 * hh + 1];
            }
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
    static constexpr int SP = CNC + 8;                     /* floats a row of the state block and of the 64 x 32 products: rows 8 banks apart,
                                                            * so the B fragments of an MMA (4 rows x 8 columns a load) touch 32 banks */
    static constexpr size_t STATE = (size_t)D * SP * 4, RD = (size_t)CH * SP * 4;
    static constexpr size_t KQ = (size_t)CH * LDH * 2, V = (size_t)CH * CNC * 2, AM = (size_t)CH * TL * 4, VEC = 4 * CH * 4;
    static constexpr size_t STAGE = 2 * KQ + V + 2 * AM + VEC;
    static constexpr size_t SQ = 2 * CH * 4;               /* two warps' halves of a row's sum of squares */
    static constexpr size_t TOTAL = STATE + 3 * RD + SQ + 2 * STAGE;
};

template <int D, int DT>
__global__ void __launch_bounds__(256, 1) deltanet_chunk_kernel(const ChunkParams P) {
    using E = Elem<DT>;
    using L = ChunkSmem<D>;
    constexpr int LDH = L::LDH, TL = L::TL, SP = L::SP, CB = D / CNC, CPR = D / 8;
    extern __shared__ __align__(16) unsigned char smb[];
    float* Ss = reinterpret_cast<float*>(smb);                       /* [D][SP] the state block */
    float* Rm = reinterpret_cast<float*>(smb + L::STATE);            /* [64][SP]: V - scaled Kn S_0 */
    float* Dm = Rm + CH * SP;                                        /* [64][SP]: D, then D scaled for the state update */
    float* Qm = Dm + CH * SP;                                        /* [64][SP]: Q S_0 */
    float* Qs = Qm + CH * SP;                                        /* [2][64]: a row's sum of squares, the two column halves */
    unsigned char* stage0 = smb + L::STATE + 3 * L::RD + L::SQ;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g8 = lane >> 2, t4 = lane & 3;
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
    for (int i = tid; i < D * CNC; i += 256) Ss[(i / CNC) * SP + i % CNC] = Sg[(uint64_t)(i / CNC) * D + j0 + i % CNC];
    bool hit = false;
    /* the state products on the tensor cores: a warp owns 16 rows by 16 columns of K S_0 and of Q S_0 ... */
    const int r1 = (warp & 3) * 16, c1 = (warp >> 2) * 16;
    /* ... and, for the update, 16 rows of the state by all 32 columns (head_dim 128) or by 16 of them (head_dim 64) */
    constexpr int NT4 = (D / 16 >= 8) ? 4 : 2;       /* 8-column tiles a warp in the update */
    const int i4 = (D / 16 >= 8) ? warp * 16 : (warp & 3) * 16, c4 = (D / 16 >= 8) ? 0 : (warp >> 2) * 16;

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

        /* (1) K S_0 and Q S_0: k and q are exact in TF32, the state goes in as two terms */
        {
            float ak[2][4] = {}, aq[2][4] = {};
            const uint16_t* kA = kr + (r1 + g8) * LDH + t4; const uint16_t* kB = kA + 8 * LDH;
            const uint16_t* qA = qr + (r1 + g8) * LDH + t4; const uint16_t* qB = qA + 8 * LDH;
            const float* sB = Ss + t4 * SP + c1 + g8;
#pragma unroll 4
            for (int k0 = 0; k0 < D; k0 += 8) {
                const uint32_t k_0 = tf32_of<DT>(kA[k0]), k_1 = tf32_of<DT>(kB[k0]), k_2 = tf32_of<DT>(kA[k0 + 4]), k_3 = tf32_of<DT>(kB[k0 + 4]);
                const uint32_t q_0 = tf32_of<DT>(qA[k0]), q_1 = tf32_of<DT>(qB[k0]), q_2 = tf32_of<DT>(qA[k0 + 4]), q_3 = tf32_of<DT>(qB[k0 + 4]);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    uint32_t h0, l0, h1, l1;
                    tf32_split(sB[k0 * SP + 8 * j], h0, l0);
                    tf32_split(sB[(k0 + 4) * SP + 8 * j], h1, l1);
                    mma_tf32(ak[j], k_0, k_1, k_2, k_3, h0, h1); mma_tf32(ak[j], k_0, k_1, k_2, k_3, l0, l1);
                    mma_tf32(aq[j], q_0, q_1, q_2, q_3, h0, h1); mma_tf32(aq[j], q_0, q_1, q_2, q_3, l0, l1);
                }
            }
            /* R = V - diag(e^G / |k|) K S_0, and Q S_0 kept for the read-out */
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int row = r1 + g8 + 8 * hh, col = c1 + 8 * j + 2 * t4;
                    const float2 v2 = E::unpack2(*reinterpret_cast<const uint32_t*>(vr + row * CNC + col));
                    const float a = va[row];
                    *reinterpret_cast<float2*>(Rm + row * SP + col) = make_float2(v2.x - a * ak[j][2 * hh], v2.y - a * ak[j][2 * hh + 1]);
                    *reinterpret_cast<float2*>(Qm + row * SP + col) = make_float2(aq[j][2 * hh], aq[j][2 * hh + 1]);
                }
        }
        __syncthreads();
        /* (2) D = A R, A lower triangular: both operands fp32, so three MMAs a step (hi·hi, hi·lo, lo·hi); a warp's 16 rows need
         * only the k-steps up to their diagonal */
        {
            float ad[2][4] = {};
            const float* aA = Am + (r1 + g8) * TL + t4; const float* aB = aA + 8 * TL;
            const float* rB = Rm + t4 * SP + c1 + g8;
            for (int k0 = 0; k0 < r1 + 16; k0 += 8) {
                uint32_t ah[4], al[4];
                tf32_split(aA[k0], ah[0], al[0]); tf32_split(aB[k0], ah[1], al[1]);
                tf32_split(aA[k0 + 4], ah[2], al[2]); tf32_split(aB[k0 + 4], ah[3], al[3]);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    uint32_t h0, l0, h1, l1;
                    tf32_split(rB[k0 * SP + 8 * j], h0, l0);
                    tf32_split(rB[(k0 + 4) * SP + 8 * j], h1, l1);
                    mma_tf32(ad[j], ah[0], ah[1], ah[2], ah[3], h0, h1);
                    mma_tf32(ad[j], ah[0], ah[1], ah[2], ah[3], l0, l1);
                    mma_tf32(ad[j], al[0], al[1], al[2], al[3], h0, h1);
                }
            }
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh)
                    *reinterpret_cast<float2*>(Dm + (r1 + g8 + 8 * hh) * SP + c1 + 8 * j + 2 * t4) = make_float2(ad[j][2 * hh], ad[j][2 * hh + 1]);
        }
        __syncthreads();
        /* (3) O = diag(e^G / |q| / sqrt d) Q S_0 + M D the same way, rounded, with the block's sum of squares for the norm */
        {
            float ao[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int row = r1 + g8 + 8 * hh;
                    const float2 q2 = *reinterpret_cast<const float2*>(Qm + row * SP + c1 + 8 * j + 2 * t4);
                    ao[j][2 * hh] = vb[row] * q2.x; ao[j][2 * hh + 1] = vb[row] * q2.y;
                }
            const float* mA = Mm + (r1 + g8) * TL + t4; const float* mB = mA + 8 * TL;
            const float* dB = Dm + t4 * SP + c1 + g8;
            for (int k0 = 0; k0 < r1 + 16; k0 += 8) {
                uint32_t ah[4], al[4];
                tf32_split(mA[k0], ah[0], al[0]); tf32_split(mB[k0], ah[1], al[1]);
                tf32_split(mA[k0 + 4], ah[2], al[2]); tf32_split(mB[k0 + 4], ah[3], al[3]);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    uint32_t h0, l0, h1, l1;
                    tf32_split(dB[k0 * SP + 8 * j], h0, l0);
                    tf32_split(dB[(k0 + 4) * SP + 8 * j], h1, l1);
                    mma_tf32(ao[j], ah[0], ah[1], ah[2], ah[3], h0, h1);
                    mma_tf32(ao[j], ah[0], ah[1], ah[2], ah[3], l0, l1);
                    mma_tf32(ao[j], al[0], al[1], al[2], al[3], h0, h1);
                }
            }
            /* a row's 32 columns are spread over two warps (16 each) and the four lanes of a group: fold in that order */
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int t = r1 + g8 + 8 * hh;
                float sq = 0.f;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const uint16_t w0 = E::from_float(ao[j][2 * hh], hit), w1 = E::from_float(ao[j][2 * hh + 1], hit);
                    const float f0 = E::to_float(w0), f1 = E::to_float(w1);
                    sq += f0 * f0 + f1 * f1;
                    if (t < n) {
                        uint16_t* orow = P.out + ((uint64_t)b * P.rows + t0 + t) * vd + (uint64_t)h * D + j0 + c1 + 8 * j + 2 * t4;
                        *reinterpret_cast<uint32_t*>(orow) = (uint32_t)w0 | ((uint32_t)w1 << 16);
                        if (P.readout) {
                            float* frow = P.readout + ((uint64_t)b * P.rows + t0 + t) * vd + (uint64_t)h * D + j0 + c1 + 8 * j + 2 * t4;
                            frow[0] = ao[j][2 * hh]; frow[1] = ao[j][2 * hh + 1];
                        }
                    }
                }
                sq += __shfl_xor_sync(0xffffffffu, sq, 1);
                sq += __shfl_xor_sync(0xffffffffu, sq, 2);
                if (t4 == 0) Qs[(warp >> 2) * CH + t] = sq;
            }
        }
        __syncthreads();
        if (tid < n) P.ss[(((uint64_t)b * P.rows + t0 + tid) * P.v_heads + h) * CB + cb] = Qs[tid] + Qs[CH + tid];
        /* the state update reads D scaled by e^(G_C - G_t) / |k_t|: scale it in place (every reader of D passed the barrier above) */
        for (int i = tid; i < CH * CNC; i += 256) Dm[(i / CNC) * SP + i % CNC] *= vc[i / CNC];
        __syncthreads();
        /* (4) S = e^(G_C) S_0 + K^T D' on the tensor cores: a warp owns its rows of the state, reads and writes nobody else's */
        {
            float acc[NT4][4];
            const float g = gc[0];
#pragma unroll
            for (int j = 0; j < NT4; ++j)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const float2 s2 = *reinterpret_cast<const float2*>(Ss + (i4 + g8 + 8 * hh) * SP + c4 + 8 * j + 2 * t4);
                    acc[j][2 * hh] = g * s2.x; acc[j][2 * hh + 1] = g * s2.y;
                }
            const uint16_t* kT = kr + t4 * LDH + i4 + g8;           /* K^T[i][p] = K[p][i] */
            const float* dB = Dm + t4 * SP + c4 + g8;
#pragma unroll 2
            for (int p0 = 0; p0 < CH; p0 += 8) {
                const uint32_t a0 = tf32_of<DT>(kT[p0 * LDH]), a1 = tf32_of<DT>(kT[p0 * LDH + 8]);
                const uint32_t a2 = tf32_of<DT>(kT[(p0 + 4) * LDH]), a3 = tf32_of<DT>(kT[(p0 + 4) * LDH + 8]);
#pragma unroll
                for (int j = 0; j < NT4; ++j) {
                    uint32_t h0, l0, h1, l1;
                    tf32_split(dB[p0 * SP + 8 * j], h0, l0);
                    tf32_split(dB[(p0 + 4) * SP + 8 * j], h1, l1);
                    mma_tf32(acc[j], a0, a1, a2, a3, h0, h1); mma_tf32(acc[j], a0, a1, a2, a3, l0, l1);
                }
            }
#pragma unroll
            for (int j = 0; j < NT4; ++j)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh)
                    *reinterpret_cast<float2*>(Ss + (i4 + g8 + 8 * hh) * SP + c4 + 8 * j + 2 * t4) = make_float2(acc[j][2 * hh], acc[j][2 * hh + 1]);
        }
        __syncthreads();                               /* every warp is done with this chunk's stage before the next fetch overwrites it */
    }
    cp_async_wait<0>();
    __syncthreads();
    for (int i = tid; i < D * CNC; i += 256) Sg[(uint64_t)(i / CNC) * D + j0 + i % CNC] = Ss[(i / CNC) * SP + i % CNC];
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
    static std::atomic<bool> attr_set[64];
    int dev = 0; cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(deltanet_prep_kernel<D, DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(deltanet_chunk_kernel<D, DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
        if (e != cudaSuccess) return e;
        attr_set[dev].store(true, std::memory_order_release);
    }
    ChunkParams P;
    P.S = c.S; P.conved = c.conved; P.beta = c.beta; P.g = c.g; P.out = c.out; P.readout = c.readout; P.ss = ss; P.prep = prep; P.over = c.over;
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
