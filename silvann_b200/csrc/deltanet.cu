/* deltanet.cu — Gated DeltaNet: the recurrent state update for one position (decode) and for a run of positions.
 *
 * The doors this answers: `deltanet_step`, `deltanet_steps`, `deltanet_steps_gate`
 * (engine/src/packages/nn/contracts/abi/gpu.cuh:128,160,227); the arithmetic is the reference's
 * nn__deltanet__zzprivate_step_head (engine/src/packages/nn/gpu/kernels/kernels.cuh:650-691): per value head h with
 * key head h / (v_heads / k_heads), per position,
 *     kn = k / sqrt(|k|^2 + 1e-6)      qs = q / sqrt(|q|^2 + 1e-6) / sqrt(d)      decay = exp(g)
 *     delta = (v - decay · S^T kn) · beta            S <- decay · S + kn delta^T            o = half(S^T qs)
 *     out = half(o · rsqrt(mean(o^2) + 1e-6) · w · gate(z))          gate = silu or sigmoid, z clamped to ±88
 * with S[key i][value j] fp32, updated in place.
 *
 * Mapping.  The columns j of a head's state never interact inside the recurrence, so a head is cut into blocks of 32
 * columns and every (sequence, head, column block) is an independent thread block: 4 blocks a head at d = 128, which
 * puts 128 blocks on the card for one sequence of 32 heads where a block per head would light 32 SMs.  A thread owns
 * one column's d/4 consecutive keys, keeps that slice of S in registers across all positions of the call, and the
 * state crosses HBM exactly once in and once out.  Two block barriers a position.  The read-out's RMS norm needs the
 * whole head, so the loop leaves the rounded read-out in `out` and each block's sum of squares in scratch; a second,
 * elementwise kernel norms and gates.  Scratch: positions · v_heads · (d/32) floats per sequence.
 *
 * Algorithmic bytes a position (decode, state round trip): 2·v_heads·d²·4 + inputs (see bench). */
#include "common.cuh"
#include "kernels_deltanet.h"
#include "kernels.h"
#include <atomic>
#include <mutex>
#include <stdlib.h>

namespace sv {

static constexpr int DN_COLS = 32;     /* state columns per block */
static constexpr int DN_RG = 4;        /* row groups: threads sharing a column */
static constexpr int DN_THREADS = DN_COLS * DN_RG;

struct DeltaParams {
    float* S;
    const uint16_t *conved, *z, *beta, *g, *w;
    uint16_t* out;
    float* readout;            /* null, or the fp32 read-out of every position before its first rounding */
    float* ss;                 /* scratch [seqs][rows][v_heads][d/32] */
    const float4* sc;          /* with PRE: per (seq, row, value head) {1/|q|/sqrt(d), 1/|k|, e^g, beta}, made by the scalars kernel */
    unsigned int* over;
    uint32_t k_heads, v_heads, seqs;
    uint64_t rows;
    int gate;
};


/* the blocks of a head as a thread-block cluster: the two halves of a barrier over all of them, and a float written into a peer's shared memory */
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void st_cluster_f32(float* local, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

/* FUSE (one position): the kernel is launched with the d/32 blocks of a head as one cluster; each block PUSHES its sum of
 * squares into every block's shared memory, arrives at the cluster barrier, stores its slice of the state while the
 * barrier completes, waits, and finishes the read-out (norm, weight, gate) from its own shared memory — one launch a
 * step, which is what a decode step of one sequence is bound by, and no block reads a peer after the barrier, so none
 * has to wait for the others before it leaves.  The sums are added in block order, as the norm kernel adds them. */
template <int D, int DT, bool PRE, bool FUSE>
__global__ void __launch_bounds__(DN_THREADS) deltanet_steps_kernel(const DeltaParams P) {
    using E = Elem<DT>;
    constexpr int CB = D / DN_COLS;            /* column blocks per head */
    constexpr int R = D / DN_RG;               /* keys per thread */
    const int tid = threadIdx.x, rg = tid / DN_COLS, c = tid % DN_COLS;
    const int cb = blockIdx.x % CB, h = (blockIdx.x / CB) % P.v_heads, b = blockIdx.x / (CB * P.v_heads);
    const int rep = P.v_heads / P.k_heads, kh = h / rep;
    const int j = cb * DN_COLS + c;            /* this thread's value column */
    const uint64_t ch = (uint64_t)(2 * P.k_heads + P.v_heads) * D, vd = (uint64_t)P.v_heads * D;

    __shared__ __align__(16) float qk[2][2][D];   /* [buffer][q|k][i] as fp32 */
    __shared__ float red1[DN_RG][DN_COLS + 2];     /* first fold, per row group: S^T k partials, then |q|^2 and |k|^2 */
    __shared__ float red2[DN_RG][DN_COLS];         /* second fold: read-out partials */
    __shared__ float cl_ss[8];                     /* FUSE: every block of the head's sum of squares, pushed here by its owner */

    float* Sh = P.S + ((uint64_t)b * P.v_heads + h) * D * D;
    float s[R];
#pragma unroll
    for (int i = 0; i < R; ++i) s[i] = Sh[(uint64_t)(rg * R + i) * D + j];

    const uint16_t* cv = P.conved + (uint64_t)b * P.rows * ch;
    const uint16_t* bb = P.beta + (uint64_t)b * P.rows * P.v_heads;
    const uint16_t* gg = P.g + (uint64_t)b * P.rows * P.v_heads;
    uint16_t* oo = P.out + (uint64_t)b * P.rows * vd;
    float* ss = P.ss + (uint64_t)b * P.rows * P.v_heads * CB;

    /* Inputs run one position ahead in registers so that no global-load latency sits on the serial path: during
     * position t the thread already holds position t's value/beta/g and position t+1's q,k elements (both loaded during
     * t-1); it parks the q,k elements in the other shared buffer and issues the loads for t+1 and t+2. */
    constexpr int NQ = (2 * D + DN_THREADS - 1) / DN_THREADS;      /* q,k elements this thread stages per position */
    /* raw bits are kept until use: converting at load time would stall the thread on the load */
    auto qk_src = [&](const uint16_t* row, int i) -> uint16_t {
        const int which = i / D, e = i % D;
        return row[(which == 0 ? kh * D : (P.k_heads + kh) * D) + e];
    };
    for (int i = tid; i < 2 * D; i += DN_THREADS) (&qk[0][0][0])[i] = E::to_float(qk_src(cv, i));
    uint16_t n_v = cv[(uint64_t)2 * P.k_heads * D + (uint64_t)h * D + j], n_beta = bb[h], n_g = gg[h];
    const float4* sc = PRE ? P.sc + (uint64_t)b * P.rows * P.v_heads + h : nullptr;
    float4 n_sc = PRE ? sc[0] : make_float4(0.f, 0.f, 0.f, 0.f);
    uint16_t n_qk[NQ];
#pragma unroll
    for (int u = 0; u < NQ; ++u) {
        const int i = tid + u * DN_THREADS;
        n_qk[u] = (P.rows > 1 && i < 2 * D) ? qk_src(cv + ch, i) : (uint16_t)0;
    }
    __syncthreads();

    const float inv_sqrt_d = 1.0f / sqrtf((float)D);
    bool hit = false;
    for (uint64_t t = 0; t < P.rows; ++t) {
        const int buf = (int)(t & 1);
        const float vj = E::to_float(n_v);
        const float4 c_sc = n_sc;
        const float beta = PRE ? c_sc.w : E::to_float(n_beta), decay = PRE ? c_sc.z : expf(E::to_float(n_g));
        if (t + 1 < P.rows) {
#pragma unroll
            for (int u = 0; u < NQ; ++u) {
                const int i = tid + u * DN_THREADS;
                if (i < 2 * D) (&qk[buf ^ 1][0][0])[i] = E::to_float(n_qk[u]);
            }
            const uint16_t* nrow = cv + (t + 1) * ch;
            n_v = nrow[(uint64_t)2 * P.k_heads * D + (uint64_t)h * D + j];
            if (PRE) n_sc = sc[(t + 1) * P.v_heads];
            else { n_beta = bb[(t + 1) * P.v_heads + h]; n_g = gg[(t + 1) * P.v_heads + h]; }
            if (t + 2 < P.rows) {
#pragma unroll
                for (int u = 0; u < NQ; ++u) {
                    const int i = tid + u * DN_THREADS;
                    if (i < 2 * D) n_qk[u] = qk_src(nrow + ch, i);
                }
            }
        }
        /* FUSE: the gate's input and the norm's weight are on their way while the state is worked */
        const uint16_t z_bits = (FUSE && rg == 0) ? P.z[((uint64_t)b * P.rows + t) * vd + (uint64_t)h * D + j] : (uint16_t)0;
        const uint16_t w_bits = (FUSE && rg == 0) ? P.w[j] : (uint16_t)0;
        const float* qv = qk[buf][0] + rg * R;
        const float* kv_ = qk[buf][1] + rg * R;
        float kvp = 0.f, qq = 0.f, kk = 0.f;
        float kv4[4] = {0.f, 0.f, 0.f, 0.f};          /* four chains instead of one: the sums are latency-bound */
#pragma unroll
        for (int i = 0; i < R; i += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(kv_ + i);
            const float4 q4 = *reinterpret_cast<const float4*>(qv + i);
            kv4[(i >> 2) & 3] += s[i] * k4.x + s[i + 1] * k4.y + s[i + 2] * k4.z + s[i + 3] * k4.w;
            if (!PRE) {
                kk += k4.x * k4.x + k4.y * k4.y + k4.z * k4.z + k4.w * k4.w;
                qq += q4.x * q4.x + q4.y * q4.y + q4.z * q4.z + q4.w * q4.w;
            }
        }
        kvp = (kv4[0] + kv4[1]) + (kv4[2] + kv4[3]);
        red1[rg][c] = kvp;
        if (!PRE && c == 0) { red1[rg][DN_COLS] = qq; red1[rg][DN_COLS + 1] = kk; }
        __syncthreads();
        float kvsum = 0.f, qsum = 0.f, ksum = 0.f;
#pragma unroll
        for (int r = 0; r < DN_RG; ++r) { kvsum += red1[r][c]; if (!PRE) { qsum += red1[r][DN_COLS]; ksum += red1[r][DN_COLS + 1]; } }
        const float inv_k = PRE ? c_sc.y : 1.0f / sqrtf(ksum + 1e-6f);
        const float inv_q = PRE ? c_sc.x : 1.0f / sqrtf(qsum + 1e-6f) * inv_sqrt_d;
        const float delta = (vj - decay * kvsum * inv_k) * beta;
        const float kd = inv_k * delta;
        float op4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < R; i += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(kv_ + i);
            const float4 q4 = *reinterpret_cast<const float4*>(qv + i);
            s[i]     = decay * s[i]     + k4.x * kd; op4[0] += s[i]     * q4.x;
            s[i + 1] = decay * s[i + 1] + k4.y * kd; op4[1] += s[i + 1] * q4.y;
            s[i + 2] = decay * s[i + 2] + k4.z * kd; op4[2] += s[i + 2] * q4.z;
            s[i + 3] = decay * s[i + 3] + k4.w * kd; op4[3] += s[i + 3] * q4.w;
        }
        red2[rg][c] = (op4[0] + op4[1]) + (op4[2] + op4[3]);
        __syncthreads();
        uint16_t oh = 0;
        if (rg == 0) {
            const float o = (red2[0][c] + red2[1][c] + red2[2][c] + red2[3][c]) * inv_q;
            oh = E::from_float(o, hit);
            if (P.readout) P.readout[((uint64_t)b * P.rows + t) * vd + (uint64_t)h * D + j] = o;
            float sq = E::to_float(oh); sq *= sq;
            for (int x = 16; x > 0; x >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, x);
            if (!FUSE) {
                oo[t * vd + (uint64_t)h * D + j] = oh;
                if (c == 0) ss[(t * P.v_heads + h) * CB + cb] = sq;
            } else if (c < CB) st_cluster_f32(&cl_ss[cb], (uint32_t)c, sq);        /* lane r tells block r of the head */
        }
        if (FUSE) {
            cluster_arrive();
            /* the state goes home while the barrier completes */
#pragma unroll
            for (int i = 0; i < R; ++i) Sh[(uint64_t)(rg * R + i) * D + j] = s[i];
            cluster_wait();
            if (rg == 0) {
                float sum = 0.f;
#pragma unroll
                for (int r = 0; r < CB; ++r) sum += cl_ss[r];
                const float scale = 1.0f / sqrtf(sum / (float)D + 1e-6f);
                const float zr = E::to_float(z_bits);
                const float zc = zr < -88.0f ? -88.0f : (zr > 88.0f ? 88.0f : zr);
                const float sg = 1.0f / (1.0f + expf(-zc));
                const float gz = P.gate == 1 ? sg : zc * sg;
                oo[t * vd + (uint64_t)h * D + j] = E::from_float(E::to_float(oh) * scale * E::to_float(w_bits) * gz, hit);
            }
        }
        /* Two barriers a position are enough because the folds use separate arrays: red1 is rewritten after this
         * position's second barrier, which follows every read of it; red2 is rewritten after the next position's first
         * barrier, which the readers above reach only after reading; qk[buf] is rewritten by the next position's
         * prefetch, after the second barrier that follows its last read. */
    }
    if (!FUSE) {
#pragma unroll
        for (int i = 0; i < R; ++i) Sh[(uint64_t)(rg * R + i) * D + j] = s[i];
    }
    if (hit && P.over) atomicOr(P.over, SV_FAULT_OVERFLOW);
}

/* One position of MANY sequences in one launch: a block a (sequence, head) with the head's whole state in its registers —
 * 4 row groups x D columns of threads, the same slice a thread and the same order of every sum as the cluster form above, so
 * a sequence's answer has the same bits whether it is stepped alone or in a batch — and, because the block holds all D
 * read-outs of the head, the RMS norm, weight and gate are finished here: no second launch, no scratch.  The state crosses
 * HBM once in and once out; 64 KB of loads a block are in flight before the first sum. */
template <int D, int DT>
__global__ void __launch_bounds__(4 * D, 2) deltanet_step_head_kernel(const DeltaParams P) {
    using E = Elem<DT>;
    constexpr int CB = D / DN_COLS, R = D / DN_RG;
    const int tid = threadIdx.x, rg = tid / D, j = tid % D, c = j % DN_COLS, cb = j / DN_COLS;
    const int h = blockIdx.x % P.v_heads, b = blockIdx.x / P.v_heads;
    const int rep = P.v_heads / P.k_heads, kh = h / rep;
    const uint64_t ch = (uint64_t)(2 * P.k_heads + P.v_heads) * D, vd = (uint64_t)P.v_heads * D;

    __shared__ __align__(16) float qk[2][D];
    __shared__ float red1[DN_RG][D], red2[DN_RG][D], nq[DN_RG], nk[DN_RG], ssq[CB];

    float* Sh = P.S + ((uint64_t)b * P.v_heads + h) * D * D;
    float s[R];
#pragma unroll
    for (int i = 0; i < R; ++i) s[i] = Sh[(uint64_t)(rg * R + i) * D + j];
    const uint16_t* cv = P.conved + (uint64_t)b * ch;
    if (tid < 2 * D) {
        const int which = tid / D, e = tid % D;
        (&qk[0][0])[tid] = E::to_float(cv[(which == 0 ? kh * D : (P.k_heads + kh) * D) + e]);
    }
    const float vj = E::to_float(cv[(uint64_t)2 * P.k_heads * D + (uint64_t)h * D + j]);
    const float beta = E::to_float(P.beta[(uint64_t)b * P.v_heads + h]), decay = expf(E::to_float(P.g[(uint64_t)b * P.v_heads + h]));
    const uint16_t z_bits = rg == 0 ? P.z[(uint64_t)b * vd + (uint64_t)h * D + j] : (uint16_t)0;
    const uint16_t w_bits = rg == 0 ? P.w[j] : (uint16_t)0;
    __syncthreads();

    const float inv_sqrt_d = 1.0f / sqrtf((float)D);
    const float* qv = qk[0] + rg * R;
    const float* kv_ = qk[1] + rg * R;
    float qq = 0.f, kk = 0.f;
    float kv4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < R; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kv_ + i);
        const float4 q4 = *reinterpret_cast<const float4*>(qv + i);
        kv4[(i >> 2) & 3] += s[i] * k4.x + s[i + 1] * k4.y + s[i + 2] * k4.z + s[i + 3] * k4.w;
        kk += k4.x * k4.x + k4.y * k4.y + k4.z * k4.z + k4.w * k4.w;
        qq += q4.x * q4.x + q4.y * q4.y + q4.z * q4.z + q4.w * q4.w;
    }
    red1[rg][j] = (kv4[0] + kv4[1]) + (kv4[2] + kv4[3]);
    if (j == 0) { nq[rg] = qq; nk[rg] = kk; }
    __syncthreads();
    float kvsum = 0.f, qsum = 0.f, ksum = 0.f;
#pragma unroll
    for (int r = 0; r < DN_RG; ++r) { kvsum += red1[r][j]; qsum += nq[r]; ksum += nk[r]; }
    const float inv_k = 1.0f / sqrtf(ksum + 1e-6f);
    const float inv_q = 1.0f / sqrtf(qsum + 1e-6f) * inv_sqrt_d;
    const float delta = (vj - decay * kvsum * inv_k) * beta;
    const float kd = inv_k * delta;
    float op4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < R; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kv_ + i);
        const float4 q4 = *reinterpret_cast<const float4*>(qv + i);
        s[i]     = decay * s[i]     + k4.x * kd; op4[0] += s[i]     * q4.x;
        s[i + 1] = decay * s[i + 1] + k4.y * kd; op4[1] += s[i + 1] * q4.y;
        s[i + 2] = decay * s[i + 2] + k4.z * kd; op4[2] += s[i + 2] * q4.z;
        s[i + 3] = decay * s[i + 3] + k4.w * kd; op4[3] += s[i + 3] * q4.w;
    }
    red2[rg][j] = (op4[0] + op4[1]) + (op4[2] + op4[3]);
    /* the state goes home while the read-out is folded */
#pragma unroll
    for (int i = 0; i < R; ++i) Sh[(uint64_t)(rg * R + i) * D + j] = s[i];
    __syncthreads();
    bool hit = false;
    uint16_t oh = 0;
    if (rg == 0) {
        const float o = (red2[0][j] + red2[1][j] + red2[2][j] + red2[3][j]) * inv_q;
        oh = E::from_float(o, hit);
        if (P.readout) P.readout[(uint64_t)b * vd + (uint64_t)h * D + j] = o;
        float sq = E::to_float(oh); sq *= sq;
        for (int x = 16; x > 0; x >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, x);
        if (c == 0) ssq[cb] = sq;
    }
    __syncthreads();
    if (rg == 0) {
        float sum = 0.f;
#pragma unroll
        for (int r = 0; r < CB; ++r) sum += ssq[r];
        const float scale = 1.0f / sqrtf(sum / (float)D + 1e-6f);
        const float zr = E::to_float(z_bits);
        const float zc = zr < -88.0f ? -88.0f : (zr > 88.0f ? 88.0f : zr);
        const float sg = 1.0f / (1.0f + expf(-zc));
        const float gz = P.gate == 1 ? sg : zc * sg;
        P.out[(uint64_t)b * vd + (uint64_t)h * D + j] = E::from_float(E::to_float(oh) * scale * E::to_float(w_bits) * gz, hit);
    }
    if (hit && P.over) atomicOr(P.over, SV_FAULT_OVERFLOW);
}

/* The per-position scalars of a run of positions, off the serial path: a warp a (sequence, position, key head) folds
 * |q|^2 and |k|^2 and writes {1/sqrt(|q|^2 + 1e-6)/sqrt(d), 1/sqrt(|k|^2 + 1e-6), e^g, beta} for each of its value heads. */
template <int D, int DT>
__global__ void __launch_bounds__(128) deltanet_scalars_kernel(float4* sc, const uint16_t* conved, const uint16_t* beta, const uint16_t* g,
                                                               uint32_t k_heads, uint32_t v_heads, uint64_t items) {
    using E = Elem<DT>;
    const int lane = threadIdx.x & 31;
    const uint32_t rep = v_heads / k_heads;
    const uint64_t ch = (uint64_t)(2 * k_heads + v_heads) * D;
    for (uint64_t it = (uint64_t)blockIdx.x * 4 + (threadIdx.x >> 5); it < items; it += (uint64_t)gridDim.x * 4) {
        const uint64_t bt = it / k_heads; const uint32_t kh = (uint32_t)(it % k_heads);
        const uint16_t* row = conved + bt * ch;
        float qq = 0.f, kk = 0.f;
        for (int e = lane; e < D; e += 32) {
            const float qe = E::to_float(row[kh * D + e]), ke = E::to_float(row[(k_heads + kh) * D + e]);
            qq += qe * qe; kk += ke * ke;
        }
        for (int x = 16; x > 0; x >>= 1) { qq += __shfl_xor_sync(0xffffffffu, qq, x); kk += __shfl_xor_sync(0xffffffffu, kk, x); }
        const float inv_q = 1.0f / sqrtf(qq + 1e-6f) / sqrtf((float)D), inv_k = 1.0f / sqrtf(kk + 1e-6f);
        for (uint32_t x = lane; x < rep; x += 32) {
            const uint64_t hh = bt * v_heads + kh * rep + x;
            sc[hh] = make_float4(inv_q, inv_k, expf(E::to_float(g[hh])), E::to_float(beta[hh]));
        }
    }
}

/* out <- half(out · rsqrt(mean(out^2) + 1e-6) · w · gate(z)), the head's sum of squares read from the blocks' parts.
 * Eight neighbouring elements a thread (16 bytes of out, of z and of w a load): the kernel moves 6 bytes an element and
 * is bound by how many loads are in flight, which two-byte loads kept low. */
template <int D, int DT>
__global__ void __launch_bounds__(256) deltanet_norm_kernel(uint16_t* out, const float* ss, const uint16_t* z, const uint16_t* w,
                                                            uint64_t heads_total, int gate, unsigned int* over) {
    using E = Elem<DT>;
    constexpr int CB = D / DN_COLS;
    bool hit = false;
    const uint64_t n8 = heads_total * (D / 8);
    const bool wide = (((uintptr_t)out | (uintptr_t)z | (uintptr_t)w) & 15u) == 0;
    for (uint64_t i8 = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i8 < n8; i8 += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t hh = i8 / (D / 8); const int e0 = (int)(i8 % (D / 8)) * 8;
        const uint64_t i0 = hh * D + e0;
        float sum = 0.f;
#pragma unroll
        for (int k = 0; k < CB; ++k) sum += ss[hh * CB + k];
        const float scale = 1.0f / sqrtf(sum / (float)D + 1e-6f);
        uint16_t ov[8], zv[8], wv[8];
        if (wide) {
            *reinterpret_cast<uint4*>(ov) = *reinterpret_cast<const uint4*>(out + i0);
            *reinterpret_cast<uint4*>(zv) = *reinterpret_cast<const uint4*>(z + i0);
            *reinterpret_cast<uint4*>(wv) = *reinterpret_cast<const uint4*>(w + e0);
        } else {
#pragma unroll
            for (int x = 0; x < 8; ++x) { ov[x] = out[i0 + x]; zv[x] = z[i0 + x]; wv[x] = w[e0 + x]; }
        }
#pragma unroll
        for (int x = 0; x < 8; ++x) {
            const float zr = E::to_float(zv[x]);
            const float zc = zr < -88.0f ? -88.0f : (zr > 88.0f ? 88.0f : zr);
            const float sg = 1.0f / (1.0f + expf(-zc));
            const float gz = gate == 1 ? sg : zc * sg;
            ov[x] = E::from_float(E::to_float(ov[x]) * scale * E::to_float(wv[x]) * gz, hit);
        }
        if (wide) *reinterpret_cast<uint4*>(out + i0) = *reinterpret_cast<const uint4*>(ov);
        else {
#pragma unroll
            for (int x = 0; x < 8; ++x) out[i0 + x] = ov[x];
        }
    }
    if (hit && over) atomicOr(over, SV_FAULT_OVERFLOW);
}

/* ---------------------------------------------------------------------------------------------------------- */

static float* g_ss[64];
static size_t g_ss_floats[64];

static cudaError_t ss_scratch(size_t floats, float** out) {
    int d = 0;
    cudaError_t e = cudaGetDevice(&d);
    if (e != cudaSuccess) return e;
    if (d < 0 || d >= 64) return cudaErrorInvalidDevice;
    static std::mutex lock;                        /* a device's worker thread is the only grower of its block, but first use is not ordered */
    std::lock_guard<std::mutex> hold(lock);
    if (g_ss_floats[d] < floats) {
        /* grow-only; the old block is released once the queue that may still read it has drained */
        if (g_ss[d]) { if ((e = cudaDeviceSynchronize()) != cudaSuccess) return e; cudaFree(g_ss[d]); g_ss[d] = nullptr; g_ss_floats[d] = 0; }
        size_t want = floats < (1u << 20) ? (1u << 20) : floats;
        if ((e = cudaMalloc(&g_ss[d], want * sizeof(float))) != cudaSuccess) return e;
        g_ss_floats[d] = want;
    }
    *out = g_ss[d];
    return cudaSuccess;
}

bool deltanet_fits(const DeltaCall& c) {
    if (c.head_dim != 64 && c.head_dim != 128 && c.head_dim != 256) return false;
    if (c.k_heads == 0 || c.v_heads % c.k_heads != 0) return false;
    return ((uintptr_t)c.S & 3u) == 0;
}

static unsigned fuse_blocks_max() {
    static const unsigned v = []() { const char* e = getenv("SILVANN_B200_DELTANET_FUSE_BLOCKS"); return e ? (unsigned)strtoul(e, nullptr, 10) : 1024u; }();
    return v;
}

template <int D, int DT>
static cudaError_t launch_dn(const DeltaCall& c, float* ss) {
    DeltaParams P;
    P.S = c.S; P.conved = c.conved; P.z = c.z; P.beta = c.beta; P.g = c.g; P.w = c.w; P.out = c.out; P.readout = c.readout; P.ss = ss; P.over = c.over;
    P.k_heads = c.k_heads; P.v_heads = c.v_heads; P.seqs = c.seqs; P.rows = c.rows; P.gate = c.gate;
    const unsigned blocks = c.seqs * c.v_heads * (D / DN_COLS);
    cudaError_t e;
    if (c.rows > 1) {
        /* a run of positions: the norms, decays and betas of every position first, in parallel */
        float4* sc = reinterpret_cast<float4*>(ss + (((size_t)c.seqs * c.rows * c.v_heads * (D / DN_COLS) + 3) & ~(size_t)3));
        const uint64_t items = (uint64_t)c.seqs * c.rows * c.k_heads;
        uint64_t nb = (items + 3) / 4; if (nb > 148 * 32) nb = 148 * 32;
        deltanet_scalars_kernel<D, DT><<<(unsigned)nb, 128, 0, c.stream>>>(sc, c.conved, c.beta, c.g, c.k_heads, c.v_heads, items);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
        note_launch(1);
        P.sc = sc;
        deltanet_steps_kernel<D, DT, true, false><<<blocks, DN_THREADS, 0, c.stream>>>(P);
    } else if (blocks > fuse_blocks_max() && D <= 128) {
        /* one position of many sequences: a block a (sequence, head), the read-out finished in the same launch */
        P.sc = nullptr;
        deltanet_step_head_kernel<(D <= 128 ? D : 128), DT><<<c.seqs * c.v_heads, 4 * (D <= 128 ? D : 128), 0, c.stream>>>(P);
        note_launch(1);
        return cudaGetLastError();
    } else if (blocks > fuse_blocks_max()) {
        P.sc = nullptr;
        deltanet_steps_kernel<D, DT, false, false><<<blocks, DN_THREADS, 0, c.stream>>>(P);
    } else {
        /* one position of a few sequences: the d/32 blocks of a head as a cluster, the read-out finished in the same
         * launch.  With many sequences the card is full either way and the cluster barrier costs more than a launch. */
        P.sc = nullptr;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(blocks); cfg.blockDim = dim3(DN_THREADS); cfg.dynamicSmemBytes = 0; cfg.stream = c.stream;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = D / DN_COLS; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        e = cudaLaunchKernelEx(&cfg, deltanet_steps_kernel<D, DT, false, true>, P);
        if (e != cudaSuccess) return e;
        note_launch(1);
        return cudaGetLastError();
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const uint64_t heads_total = (uint64_t)c.seqs * c.rows * c.v_heads;
    /* z and out are laid out [seq][row][head][d], so one flat pass covers every sequence */
    uint64_t nb = (heads_total * (D / 8) + 255) / 256; if (nb > 148 * 16) nb = 148 * 16;
    deltanet_norm_kernel<D, DT><<<(unsigned)nb, 256, 0, c.stream>>>(c.out, ss, c.z, c.w, heads_total, c.gate, c.over);
    note_launch(2);
    return cudaGetLastError();
}

template <int D, int DT>
static cudaError_t launch_norm(const DeltaCall& c, const float* ss) {
    const uint64_t heads_total = (uint64_t)c.seqs * c.rows * c.v_heads;
    uint64_t nb = (heads_total * (D / 8) + 255) / 256; if (nb > 148 * 16) nb = 148 * 16;
    deltanet_norm_kernel<D, DT><<<(unsigned)nb, 256, 0, c.stream>>>(c.out, ss, c.z, c.w, heads_total, c.gate, c.over);
    note_launch(1);
    return cudaGetLastError();
}
cudaError_t deltanet_norm_launch(const DeltaCall& c, const float* ss) {
    if (c.head_dim == 64) return c.dtype == SV_DTYPE_BF16 ? launch_norm<64, SV_DTYPE_BF16>(c, ss) : launch_norm<64, SV_DTYPE_FP16>(c, ss);
    if (c.head_dim == 128) return c.dtype == SV_DTYPE_BF16 ? launch_norm<128, SV_DTYPE_BF16>(c, ss) : launch_norm<128, SV_DTYPE_FP16>(c, ss);
    return cudaErrorInvalidValue;
}

static bool chunked_enabled() {
    static const bool on = []() { const char* v = getenv("SILVANN_B200_DELTANET_CHUNKED"); return !(v && v[0] == '0'); }();
    return on;
}

cudaError_t deltanet_launch(const DeltaCall& c) {
    if (c.rows == 0 || c.seqs == 0) return cudaSuccess;
    if (chunked_enabled() && deltanet_chunked_fits(c)) {
        /* a run of positions: 64 at a time */
        const size_t ss_floats = (((size_t)c.seqs * c.rows * c.v_heads * (c.head_dim / DN_COLS)) + 3) & ~(size_t)3;
        float* buf = nullptr;
        cudaError_t e = ss_scratch(ss_floats + deltanet_chunked_scratch_floats(c), &buf);
        if (e != cudaSuccess) return e;
        if ((e = deltanet_chunked_launch(c, buf, buf + ss_floats)) != cudaSuccess) return e;
        return deltanet_norm_launch(c, buf);
    }
    float* ss = nullptr;
    /* per-block sums of squares, then (for a run of positions) four scalars per position and value head */
    cudaError_t e = ss_scratch((size_t)c.seqs * c.rows * c.v_heads * (c.head_dim / DN_COLS) + 4 + (c.rows > 1 ? 4 * (size_t)c.seqs * c.rows * c.v_heads : 0), &ss);
    if (e != cudaSuccess) return e;
#define SV_DN(DD) (c.dtype == SV_DTYPE_BF16 ? launch_dn<DD, SV_DTYPE_BF16>(c, ss) : launch_dn<DD, SV_DTYPE_FP16>(c, ss))
    if (c.head_dim == 64) return SV_DN(64);
    if (c.head_dim == 128) return SV_DN(128);
    if (c.head_dim == 256) return SV_DN(256);
#undef SV_DN
    return cudaErrorInvalidValue;
}

}  // namespace sv
