/* silvann_oracle.c — TEST INFRASTRUCTURE, NOT PRODUCT.  A plain-C, CPU restatement of the arithmetic of SiLVANN's
 * attention and Gated-DeltaNet doors, used only as the checker in tests/, in __graft_entry__.smoke() and as the
 * `cpu_baseline` of bench.py when the reference's own CPU family could not be built.  Nothing in silvann_b200/ may
 * call it.
 *
 * Each function names the reference body it restates (paths under engine/src/ of the reference tree).  The loops are
 * serial in the order the reference's one-lane host build would take; dtype 0 reads and rounds IEEE fp16 (the only
 * type the reference has), dtype 1 reads and rounds bf16 (this library's extension).  Parity is pinned against the
 * reference's own x86_avx2 family: tests/golden/ holds outputs of that family, produced in a container that had the
 * reference sources, by tests/golden/make_golden.py. */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_FAULT_OVERFLOW 0x4E504F56u   /* packages/nn/contracts/objects/primitives.cuh:57 */

/* ---- 16-bit conversions --------------------------------------------------------------------------------------- */

static float f16_to_f32(uint16_t h) {                      /* packages/nn/gpu/kernels/kernels.cuh:2733-2759 */
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const int exp = (h >> 10) & 31;
    const uint32_t man = h & 0x3FFu;
    if (exp == 31) { union { uint32_t u; float f; } c; c.u = sign | 0x7F800000u | (man << 13); return c.f; }
    float v = exp == 0 ? ldexpf((float)man, -24) : ldexpf((float)(man | 0x400u), exp - 25);
    return sign ? -v : v;
}
static uint16_t f32_to_f16(float f, int* over) {           /* kernels.cuh:2766-2808: RNE; a finite value that does not fit flags */
    union { float f; uint32_t u; } c; c.f = f;
    const uint32_t sign = (c.u >> 16) & 0x8000u, e = (c.u >> 23) & 0xFFu;
    uint32_t m = c.u & 0x7FFFFFu;
    if (e == 0xFFu) return (uint16_t)(sign | 0x7C00u | (m ? ((m >> 13) | 0x200u) : 0u));
    int he = (int)e - 112;
    if (he >= 31) { if (over) *over = 1; return (uint16_t)(sign | 0x7C00u); }
    if (he > 0) {
        uint32_t mh = m >> 13; const uint32_t rem = m & 0x1FFFu;
        if (rem > 0x1000u || (rem == 0x1000u && (mh & 1u))) {
            if (++mh == 0x400u) { mh = 0; if (++he >= 31) { if (over) *over = 1; return (uint16_t)(sign | 0x7C00u); } }
        }
        return (uint16_t)(sign | ((uint32_t)he << 10) | mh);
    }
    if (he < -10) return (uint16_t)sign;
    m |= 0x800000u;
    const uint32_t shift = (uint32_t)(14 - he), half = 1u << (shift - 1);
    uint32_t mh = m >> shift; const uint32_t rem = m & ((1u << shift) - 1u);
    if (rem > half || (rem == half && (mh & 1u))) ++mh;
    return (uint16_t)(sign | mh);
}
static float bf16_to_f32(uint16_t h) { union { uint32_t u; float f; } c; c.u = (uint32_t)h << 16; return c.f; }
static uint16_t f32_to_bf16(float f, int* over) {
    union { float f; uint32_t u; } c; c.f = f;
    if ((c.u & 0x7F800000u) == 0x7F800000u) return (uint16_t)((c.u >> 16) | ((c.u & 0xFFFFu) ? 0x40u : 0u));
    const uint32_t r = c.u + 0x7FFFu + ((c.u >> 16) & 1u);
    if ((r & 0x7F800000u) == 0x7F800000u && over) *over = 1;
    return (uint16_t)(r >> 16);
}
static inline float ld16(uint16_t h, int dtype) { return dtype ? bf16_to_f32(h) : f16_to_f32(h); }
static inline uint16_t st16(float f, int dtype, int* over) { return dtype ? f32_to_bf16(f, over) : f32_to_f16(f, over); }

uint16_t oracle_f32_to_f16(float f) { return f32_to_f16(f, 0); }
float oracle_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
uint16_t oracle_f32_to_bf16(float f) { return f32_to_bf16(f, 0); }

/* ---- one query position ------------------------------------------------------------------------------------------ */

/* scaled scores of one head: dot over head_dim in element order, times 1/sqrt(head_dim) (kernels.cuh:894-905) */
static void head_scores(float* ph, const uint16_t* qh, const uint16_t* kh, uint64_t row, uint64_t d, uint64_t len, int dt) {
    const float scale = 1.0f / sqrtf((float)d);
    for (uint64_t t = 0; t < len; ++t) {
        float dot = 0.0f;
        for (uint64_t e = 0; e < d; ++e) dot += ld16(qh[e], dt) * ld16(kh[t * row + e], dt);
        ph[t] = dot * scale;
    }
}
/* in place: exp(x - max), optionally over the sum (kernels.cuh:906-914, 1085-1099) */
static void head_softmax(float* ph, uint64_t len, int normalise, float* top_out, float* sum_out) {
    float top = -INFINITY, sum = 0.0f;
    for (uint64_t t = 0; t < len; ++t) if (ph[t] > top) top = ph[t];
    for (uint64_t t = 0; t < len; ++t) { ph[t] = expf(ph[t] - top); sum += ph[t]; }
    if (normalise) { const float inv = 1.0f / sum; for (uint64_t t = 0; t < len; ++t) ph[t] *= inv; }
    if (top_out) *top_out = top;
    if (sum_out) *sum_out = sum;
}

/* attention_scores: p[h][t] = softmax_t(q_h · k_{t, h/group} / sqrt(d))  (kernels.cuh:1133-1141) */
void oracle_attention_scores(float* p, const uint16_t* q, const uint16_t* k, uint64_t qh, uint64_t kvh, uint64_t d, uint64_t len, int dt) {
    const uint64_t group = qh / kvh, row = kvh * d;
    for (uint64_t h = 0; h < qh; ++h) {
        head_scores(p + h * len, q + h * d, k + (h / group) * d, row, d, len, dt);
        head_softmax(p + h * len, len, 1, 0, 0);
    }
}
/* attention_scores_grouped: the same without the softmax (kernels.cuh:931-952) */
void oracle_attention_scores_grouped(float* p, const uint16_t* q, const uint16_t* k, uint64_t qh, uint64_t kvh, uint64_t d, uint64_t len, int dt) {
    const uint64_t group = qh / kvh, row = kvh * d;
    for (uint64_t h = 0; h < qh; ++h) head_scores(p + h * len, q + h * d, k + (h / group) * d, row, d, len, dt);
}
/* attention_softmax_rows (kernels.cuh:1085-1101) */
void oracle_attention_softmax_rows(float* p, uint64_t rows, uint64_t len) {
    for (uint64_t r = 0; r < rows; ++r) head_softmax(p + r * len, len, 1, 0, 0);
}
/* attention_mix: o[h][e] = half(sum_t p[h][t] · v[t][h/group][e]), positions in order (kernels.cuh:1144-1164) */
void oracle_attention_mix(uint16_t* o, const float* p, const uint16_t* v, uint64_t qh, uint64_t kvh, uint64_t d, uint64_t len, int dt, unsigned* over) {
    const uint64_t group = qh / kvh, row = kvh * d;
    int hit = 0;
    for (uint64_t h = 0; h < qh; ++h)
        for (uint64_t e = 0; e < d; ++e) {
            float sum = 0.0f;
            for (uint64_t t = 0; t < len; ++t) sum += p[h * len + t] * ld16(v[t * row + (h / group) * d + e], dt);
            o[h * d + e] = st16(sum, dt, &hit);
        }
    if (hit && over) *over = ORACLE_FAULT_OVERFLOW;
}
/* attention_weights: unnormalised e^(s-m) into p; m and l into res[h][0..1]  (kernels.cuh:1189-1222) */
void oracle_attention_weights(float* p, float* res, const uint16_t* q, const uint16_t* k, uint64_t qh, uint64_t kvh, uint64_t d, uint64_t len, int dt) {
    const uint64_t group = qh / kvh, row = kvh * d;
    for (uint64_t h = 0; h < qh; ++h) {
        head_scores(p + h * len, q + h * d, k + (h / group) * d, row, d, len, dt);
        head_softmax(p + h * len, len, 0, &res[h * (d + 2)], &res[h * (d + 2) + 1]);
    }
}
/* attention_residual_mix: acc into res[h][2..]  (kernels.cuh:1225-1241) */
void oracle_attention_residual_mix(float* res, const float* p, const uint16_t* v, uint64_t qh, uint64_t kvh, uint64_t d, uint64_t len, int dt) {
    const uint64_t group = qh / kvh, row = kvh * d;
    for (uint64_t h = 0; h < qh; ++h)
        for (uint64_t e = 0; e < d; ++e) {
            float sum = 0.0f;
            for (uint64_t t = 0; t < len; ++t) sum += p[h * len + t] * ld16(v[t * row + (h / group) * d + e], dt);
            res[h * (d + 2) + 2 + e] = sum;
        }
}
/* attention_merge: both scaled to the common maximum, then added; `into` may be a or b (kernels.cuh:1243-1255) */
void oracle_attention_merge(float* into, const float* a, const float* b, uint64_t qh, uint64_t d) {
    const uint64_t w = d + 2;
    for (uint64_t h = 0; h < qh; ++h) {
        const float ma = a[h * w], la = a[h * w + 1], mb = b[h * w], lb = b[h * w + 1];
        const float m = ma > mb ? ma : mb, fa = expf(ma - m), fb = expf(mb - m);
        for (uint64_t e = 0; e < d; ++e) into[h * w + 2 + e] = a[h * w + 2 + e] * fa + b[h * w + 2 + e] * fb;
        into[h * w] = m;
        into[h * w + 1] = la * fa + lb * fb;
    }
}
/* attention_finish: half(acc / l)  (kernels.cuh:1258-1267) */
void oracle_attention_finish(uint16_t* o, const float* res, uint64_t qh, uint64_t d, int dt, unsigned* over) {
    const uint64_t w = d + 2;
    int hit = 0;
    for (uint64_t i = 0; i < qh * d; ++i) o[i] = st16(res[(i / d) * w + 2 + i % d] / res[(i / d) * w + 1], dt, &hit);
    if (hit && over) *over = ORACLE_FAULT_OVERFLOW;
}

/* ---- a prompt's rows ------------------------------------------------------------------------------------------------ */

/* attention_causal_scores_grouped: row r (position first + r), head h over cache rows 0..first+r, unnormalised, at
 * p + (r·qh + h)·(first + rows)  (kernels.cuh:1028-1062; per-element order of nn__attention__zzprivate_dots, :975-995) */
void oracle_attention_causal_scores_grouped(float* p, const uint16_t* q, const uint16_t* k, uint64_t qh, uint64_t kvh, uint64_t d, uint64_t first, uint64_t rows, int dt) {
    const uint64_t group = qh / kvh, row = kvh * d, span = first + rows;
    for (uint64_t i = 0; i < rows * qh; ++i) {
        const uint64_t r = i / qh, h = i % qh;
        head_scores(p + i * span, q + i * d, k + (h / group) * d, row, d, first + r + 1, dt);
    }
}
/* attention_causal_softmax (kernels.cuh:1066-1081) */
void oracle_attention_causal_softmax(float* p, uint64_t qh, uint64_t first, uint64_t rows) {
    const uint64_t span = first + rows;
    for (uint64_t i = 0; i < rows * qh; ++i) head_softmax(p + i * span, first + i / qh + 1, 1, 0, 0);
}
/* attention_causal_mix (kernels.cuh:2051-2060) */
void oracle_attention_causal_mix(uint16_t* o, const float* p, const uint16_t* v, uint64_t qh, uint64_t kvh, uint64_t d, uint64_t first, uint64_t rows, int dt, unsigned* over) {
    const uint64_t group = qh / kvh, row = kvh * d, span = first + rows;
    int hit = 0;
    for (uint64_t i = 0; i < rows * qh; ++i) {
        const uint64_t r = i / qh, h = i % qh, len = first + r + 1;
        for (uint64_t e = 0; e < d; ++e) {
            float sum = 0.0f;
            for (uint64_t t = 0; t < len; ++t) sum += p[i * span + t] * ld16(v[t * row + (h / group) * d + e], dt);
            o[i * d + e] = st16(sum, dt, &hit);
        }
    }
    if (hit && over) *over = ORACLE_FAULT_OVERFLOW;
}
/* The three causal doors for a run of rows without the rows·(first+rows) buffer: one row's weights at a time.  Also
 * answers the fp32 value before rounding (o32, may be null).  Same arithmetic and order as the three above. */
void oracle_prefill(uint16_t* o, float* o32, const uint16_t* q, const uint16_t* k, const uint16_t* v, uint64_t qh, uint64_t kvh, uint64_t d,
                    uint64_t first, uint64_t rows, int dt, unsigned* over) {
    const uint64_t group = qh / kvh, row = kvh * d;
    int hit = 0;
#pragma omp parallel for schedule(dynamic, 4) reduction(| : hit)
    for (int64_t i = 0; i < (int64_t)(rows * qh); ++i) {
        const uint64_t r = (uint64_t)i / qh, h = (uint64_t)i % qh, len = first + r + 1;
        float* ph = (float*)malloc(len * sizeof(float));
        head_scores(ph, q + (uint64_t)i * d, k + (h / group) * d, row, d, len, dt);
        head_softmax(ph, len, 1, 0, 0);
        for (uint64_t e = 0; e < d; ++e) {
            float sum = 0.0f;
            for (uint64_t t = 0; t < len; ++t) sum += ph[t] * ld16(v[t * row + (h / group) * d + e], dt);
            int one = 0;
            o[(uint64_t)i * d + e] = st16(sum, dt, &one);
            hit |= one;
            if (o32) o32[(uint64_t)i * d + e] = sum;
        }
        free(ph);
    }
    if (hit && over) *over = ORACLE_FAULT_OVERFLOW;
}

/* ---- Gated DeltaNet -------------------------------------------------------------------------------------------------- */

/* One value head, one position (nn__deltanet__zzprivate_step_head, kernels.cuh:650-691).  The reference walks a column j
 * of the state at a time (its inner loops run over the key index i); here i is the outer loop and j the inner one so that
 * memory is walked with unit stride — every sum still receives its terms in the order i = 0, 1, ..., so each result is the
 * same float.  `readout` (may be null) receives the read-out of the position before its first rounding to 16 bits. */
static void deltanet_head(float* S, const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* z, float beta, float g,
                          const uint16_t* w, uint16_t* out, float* readout, uint64_t d, unsigned gate, int dt, int* hit) {
    float qq = 0.0f, kk = 0.0f;
    for (uint64_t i = 0; i < d; ++i) { const float qi = ld16(q[i], dt), ki = ld16(k[i], dt); qq += qi * qi; kk += ki * ki; }
    const float inv_q = 1.0f / sqrtf(qq + 1e-6f) / sqrtf((float)d), inv_k = 1.0f / sqrtf(kk + 1e-6f), decay = expf(g);
    float kv[512], o[512], delta[512];
    for (uint64_t j = 0; j < d; ++j) { kv[j] = 0.0f; o[j] = 0.0f; }
    for (uint64_t i = 0; i < d; ++i) {
        const float ki = ld16(k[i], dt);
        const float* row = S + i * d;
        for (uint64_t j = 0; j < d; ++j) kv[j] += row[j] * ki;
    }
    for (uint64_t j = 0; j < d; ++j) delta[j] = (ld16(v[j], dt) - decay * kv[j] * inv_k) * beta;
    for (uint64_t i = 0; i < d; ++i) {
        const float kn = ld16(k[i], dt) * inv_k, qi = ld16(q[i], dt);
        float* row = S + i * d;
        for (uint64_t j = 0; j < d; ++j) {
            const float s = decay * row[j] + kn * delta[j];
            row[j] = s;
            o[j] += s * qi;
        }
    }
    float oo = 0.0f;
    for (uint64_t j = 0; j < d; ++j) {
        if (readout) readout[j] = o[j] * inv_q;
        out[j] = st16(o[j] * inv_q, dt, hit);              /* the read-out is rounded before its norm */
        const float oj = ld16(out[j], dt);
        oo += oj * oj;
    }
    const float scale = 1.0f / sqrtf(oo / (float)d + 1e-6f);
    for (uint64_t j = 0; j < d; ++j) {
        const float zr = ld16(z[j], dt), zc = zr < -88.0f ? -88.0f : (zr > 88.0f ? 88.0f : zr);
        const float gz = gate == 1u ? 1.0f / (1.0f + expf(-zc)) : zc / (1.0f + expf(-zc));
        out[j] = st16(ld16(out[j], dt) * scale * ld16(w[j], dt) * gz, dt, hit);
    }
}
/* deltanet_steps_gate (kernels.cuh:2131-2165); rows = 1 and gate = 0 is deltanet_step (:707-718).
 * conved row = q heads, k heads, v heads; value head h reads key head h / (vh / kh).  head_dim <= 512.
 * `readout`: null, or [rows][vh*d] fp32 (see deltanet_head). */
void oracle_deltanet_steps_readout(float* S, const uint16_t* conved, const uint16_t* z, const uint16_t* beta, const uint16_t* g, const uint16_t* w,
                                   uint16_t* out, float* readout, uint64_t kh, uint64_t vh, uint64_t d, uint64_t rows, unsigned gate, int dt, unsigned* over) {
    const uint64_t rep = vh / kh, ch = (2 * kh + vh) * d, vd = vh * d;
    int hit = 0;
    if (d > 512) return;
#pragma omp parallel for schedule(static) reduction(| : hit)
    for (int64_t h = 0; h < (int64_t)vh; ++h)
        for (uint64_t t = 0; t < rows; ++t) {
            const uint16_t* c = conved + t * ch;
            int one = 0;
            deltanet_head(S + (uint64_t)h * d * d, c + ((uint64_t)h / rep) * d, c + kh * d + ((uint64_t)h / rep) * d, c + 2 * kh * d + (uint64_t)h * d,
                          z + t * vd + (uint64_t)h * d, ld16(beta[t * vh + (uint64_t)h], dt), ld16(g[t * vh + (uint64_t)h], dt), w,
                          out + t * vd + (uint64_t)h * d, readout ? readout + t * vd + (uint64_t)h * d : 0, d, gate, dt, &one);
            hit |= one;
        }
    if (hit && over) *over = ORACLE_FAULT_OVERFLOW;
}
void oracle_deltanet_steps(float* S, const uint16_t* conved, const uint16_t* z, const uint16_t* beta, const uint16_t* g, const uint16_t* w,
                           uint16_t* out, uint64_t kh, uint64_t vh, uint64_t d, uint64_t rows, unsigned gate, int dt, unsigned* over) {
    oracle_deltanet_steps_readout(S, conved, z, beta, g, w, out, 0, kh, vh, d, rows, gate, dt, over);
}

/* vector_sum: parts added in the order given, one rounding (kernels.cuh:117-126) */
void oracle_vector_sum(uint16_t* out, const uint16_t* const* parts, uint64_t count, uint64_t n, int dt, unsigned* over) {
    int hit = 0;
    for (uint64_t i = 0; i < n; ++i) {
        float s = 0.0f;
        for (uint64_t k = 0; k < count; ++k) s += ld16(parts[k][i], dt);
        out[i] = st16(s, dt, &hit);
    }
    if (hit && over) *over = ORACLE_FAULT_OVERFLOW;
}

/* ---- the per-row (gathered key set) forms, the sink softmax, and DeltaNet's input doors ------------------------------ */

/* attention_scores_grouped_rows (kernels.cuh:957-972): row u's heads at q + u·q_row, its lens[u] keys at k + u·k_row, raw
 * scaled scores at p + u·p_row, a head's lens[u] apart */
void oracle_attention_scores_grouped_rows(float* p, uint64_t p_row, const uint16_t* q, uint64_t q_row, const uint16_t* k, uint64_t k_row,
                                          const uint32_t* lens, uint64_t qh, uint64_t kvh, uint64_t d, uint64_t rows, int dt) {
    const uint64_t group = qh / kvh, row = kvh * d;
    for (uint64_t u = 0; u < rows; ++u)
        for (uint64_t h = 0; h < qh; ++h)
            head_scores(p + u * p_row + h * lens[u], q + u * q_row + h * d, k + u * k_row + (h / group) * d, row, d, lens[u], dt);
}
/* attention_softmax_lens (kernels.cuh:1104-1110) */
void oracle_attention_softmax_lens(float* p, uint64_t p_row, const uint32_t* lens, uint64_t heads, uint64_t rows) {
    for (uint64_t u = 0; u < rows; ++u)
        for (uint64_t h = 0; h < heads; ++h) head_softmax(p + u * p_row + h * lens[u], lens[u], 1, 0, 0);
}
/* attention_softmax_sink (kernels.cuh:1115-1131): one more term exp(sink[r]) in the sum, and in the maximum */
void oracle_attention_softmax_sink(float* p, const uint16_t* sink, uint64_t rows, uint64_t len) {
    for (uint64_t r = 0; r < rows; ++r) {
        float* ph = p + r * len;
        const float sk = f16_to_f32(sink[r]);
        float top = sk, sum = 0.0f;
        for (uint64_t t = 0; t < len; ++t) if (ph[t] > top) top = ph[t];
        for (uint64_t t = 0; t < len; ++t) { ph[t] = expf(ph[t] - top); sum += ph[t]; }
        const float inv = 1.0f / (sum + expf(sk - top));
        for (uint64_t t = 0; t < len; ++t) ph[t] *= inv;
    }
}
/* attention_mix_rows (kernels.cuh:1169-1178) */
void oracle_attention_mix_rows(uint16_t* o, uint64_t o_row, const float* p, uint64_t p_row, const uint16_t* v, uint64_t v_row, const uint32_t* lens,
                               uint64_t qh, uint64_t kvh, uint64_t d, uint64_t rows, int dt, unsigned* over) {
    const uint64_t group = qh / kvh, row = kvh * d;
    int hit = 0;
    for (uint64_t u = 0; u < rows; ++u)
        for (uint64_t h = 0; h < qh; ++h)
            for (uint64_t e = 0; e < d; ++e) {
                float sum = 0.0f;
                for (uint64_t t = 0; t < lens[u]; ++t) sum += p[u * p_row + h * lens[u] + t] * ld16(v[u * v_row + t * row + (h / group) * d + e], dt);
                o[u * o_row + h * d + e] = st16(sum, dt, &hit);
            }
    if (hit && over) *over = ORACLE_FAULT_OVERFLOW;
}
/* deltanet_gates_rows (kernels.cuh:2081-2101): every intermediate rounded to a half where the reference rounds it */
void oracle_deltanet_gates_rows(uint16_t* beta, uint16_t* g, const uint16_t* a, const uint16_t* b, const uint16_t* a_log, const uint16_t* dt_bias,
                                uint64_t heads, uint64_t rows) {
    for (uint64_t i = 0; i < heads * rows; ++i) {
        const uint64_t h = i % heads;
        beta[i] = f32_to_f16(1.0f / (1.0f + expf(-f16_to_f32(b[i]))), 0);
        const float sum = f16_to_f32(f32_to_f16(f16_to_f32(a[i]) + f16_to_f32(dt_bias[h]), 0));
        const float mag = sum < 0.0f ? -sum : sum, top = sum > 0.0f ? sum : 0.0f;
        const float sp = f16_to_f32(f32_to_f16(top + logf(1.0f + expf(-mag)), 0));
        const float ea = f16_to_f32(f32_to_f16(expf(f16_to_f32(a_log[h])), 0));
        const float prod = f16_to_f32(f32_to_f16(sp * ea, 0));
        g[i] = f32_to_f16(prod * -1.0f, 0);
    }
}
/* deltanet_conv_steps (kernels.cuh:2106-2125; rows = 1 is deltanet_conv_step, :627-645): four taps over a kept window of
 * three and the new input, silu, then the window slides */
void oracle_deltanet_conv_steps(uint16_t* o, uint16_t* s, const uint16_t* w, const uint16_t* x, uint64_t ch, uint64_t rows) {
    for (uint64_t c = 0; c < ch; ++c)
        for (uint64_t t = 0; t < rows; ++t) {
            const uint16_t xt = x[t * ch + c];
            float acc = 0.0f;
            for (int k = 0; k < 3; ++k) acc += f16_to_f32(w[c * 4 + k]) * f16_to_f32(s[c * 3 + k]);
            acc += f16_to_f32(w[c * 4 + 3]) * f16_to_f32(xt);
            o[t * ch + c] = f32_to_f16(acc / (1.0f + expf(-acc)), 0);
            s[c * 3] = s[c * 3 + 1]; s[c * 3 + 1] = s[c * 3 + 2]; s[c * 3 + 2] = xt;
        }
}

/* ---- the TurboQuant-coded tiers of the cache (kernels.cuh:2819-2986) ------------------------------------------------
 * The level tables are the format's: Lloyd-Max levels of a standard normal, regenerated by
 * silvann_b200/csrc/gen_tq_levels.py and pinned to the reference's own turboquant_decode door by tests/test_tq_levels.py. */
static const uint16_t tq_levels[318] = {
#include "../silvann_b200/csrc/tq_levels.inc"
};
static uint32_t tq_table_at(uint64_t d) { return d == 1 ? 0u : d == 2 ? 2u : d == 3 ? 6u : d == 4 ? 14u : d == 5 ? 30u : 62u; }
static float tq_level(uint64_t d, uint32_t code) {                                     /* kernels.cuh:2650-2653 */
    return d == 16 ? f16_to_f32((uint16_t)code) : f16_to_f32(tq_levels[tq_table_at(d) + code]);
}
static uint64_t tq_row_bytes(uint64_t d, uint64_t cols) { const uint64_t per = 16 / d; return ((cols + per - 1) / per) * 2; }   /* :2814-2817 */
static float tq_element(const uint8_t* row, float scale, uint64_t d, uint64_t c) {     /* :2897-2901 */
    const uint64_t per = 16 / d;
    const uint32_t unit = (uint32_t)row[(c / per) * 2] | ((uint32_t)row[(c / per) * 2 + 1] << 8);
    return scale * tq_level(d, (unit >> (uint32_t)(d * (c % per))) & ((1u << (uint32_t)d) - 1u));
}
/* turboquant_decode (kernels.cuh:1281-1298) for a matrix whose rooms hold every row */
void oracle_turboquant_decode(uint16_t* out, const uint8_t* weights, const uint8_t* luts, uint64_t d, uint64_t rows, uint64_t cols) {
    const uint64_t need = tq_row_bytes(d, cols);
    for (uint64_t r = 0; r < rows; ++r) {
        const float scale = d == 16 ? 1.0f : f16_to_f32((uint16_t)((uint32_t)luts[r * 2] | ((uint32_t)luts[r * 2 + 1] << 8)));
        for (uint64_t c = 0; c < cols; ++c) out[r * cols + c] = f32_to_f16(tq_element(weights + r * need, scale, d, c), 0);
    }
}
/* hadamard_blocks (kernels.cuh:2829-2855): R = H·(S ⊙ u) a block, or its transpose S ⊙ H·u; even and odd columns summed apart */
void oracle_hadamard_blocks(uint16_t* out, const uint16_t* in, const uint16_t* sign, uint64_t n, uint64_t block, uint64_t inverse) {
    const float norm = 1.0f / sqrtf((float)(uint32_t)block);
    for (uint64_t i = 0; i < n; ++i) {
        const uint64_t a = i - i % block, r = i - a;
        float s0 = 0.0f, s1 = 0.0f;
        for (uint64_t c = 0; c < block; c += 2) {
            float v0 = f16_to_f32(in[a + c]), v1 = f16_to_f32(in[a + c + 1]);
            if (!inverse) { v0 *= f16_to_f32(sign[c]); v1 *= f16_to_f32(sign[c + 1]); }
            s0 += (__builtin_popcountll(r & c) & 1) ? -v0 : v0;
            s1 += (__builtin_popcountll(r & (c + 1)) & 1) ? -v1 : v1;
        }
        float sum = (s0 + s1) * norm;
        if (inverse) sum *= f16_to_f32(sign[r]);
        out[i] = f32_to_f16(sum, 0);
    }
}
/* turboquant_encode_rows (kernels.cuh:2857-2895): scale = fp16(clip · rms), a code = how many midpoints lie below x / scale */
void oracle_turboquant_encode_rows(uint8_t* codes, uint16_t* scales, const uint16_t* x, uint64_t rows, uint64_t cols, uint64_t d) {
    const uint64_t per = 16 / d, row_bytes = tq_row_bytes(d, cols), units = row_bytes / 2;
    const float clip = d == 4 ? 2.7325895709952577f : 4.6036453045214065f;
    for (uint64_t r = 0; r < rows; ++r) {
        const uint16_t* xr = x + r * cols;
        float part = 0.0f;
        for (uint64_t c = 0; c < cols; ++c) { const float v = f16_to_f32(xr[c]); part += v * v; }
        uint16_t sh = f32_to_f16(clip * sqrtf(part / (float)cols), 0);
        float scale = f16_to_f32(sh);
        const int dead = scale < 6.103515625e-05f;
        if (dead) { sh = 0; scale = 0.0f; }
        scales[r] = sh;
        for (uint64_t u = 0; u < units; ++u) {
            uint32_t unit = 0;
            for (uint64_t s = 0; s < per; ++s) {
                const uint64_t c = u * per + s;
                if (c >= cols || dead) continue;
                const float v = f16_to_f32(xr[c]) / scale;
                uint32_t lo = 0, hi = (1u << (uint32_t)d) - 1u;
                while (lo < hi) {
                    const uint32_t mid = (lo + hi) >> 1;
                    if (0.5f * (tq_level(d, mid) + tq_level(d, mid + 1)) < v) lo = mid + 1; else hi = mid;
                }
                unit |= lo << (uint32_t)(d * s);
            }
            codes[r * row_bytes + u * 2] = (uint8_t)(unit & 0xff);
            codes[r * row_bytes + u * 2 + 1] = (uint8_t)(unit >> 8);
        }
    }
}
/* attention_weights_tq + attention_residual_mix_tq (kernels.cuh:2904-2986): the residual of one query over coded rows */
void oracle_attention_residual_tq(float* p, float* res, const uint16_t* q, const uint8_t* kcodes, const uint16_t* kscales,
                                  const uint8_t* vcodes, const uint16_t* vscales, uint64_t qh, uint64_t kvh, uint64_t dh, uint64_t len, uint64_t d) {
    const uint64_t group = qh / kvh, row_bytes = tq_row_bytes(d, dh);
    const float inv = 1.0f / sqrtf((float)(uint32_t)dh);
    for (uint64_t h = 0; h < qh; ++h) {
        const uint64_t g = h / group;
        float* ph = p + h * len;
        float top = -INFINITY;
        for (uint64_t t = 0; t < len; ++t) {
            const uint64_t row = t * kvh + g;
            const float scale = f16_to_f32(kscales[row]);
            float dot = 0.0f;
            for (uint64_t e = 0; e < dh; ++e) dot += f16_to_f32(q[h * dh + e]) * tq_element(kcodes + row * row_bytes, scale, d, e);
            ph[t] = dot * inv;
            if (ph[t] > top) top = ph[t];
        }
        float sum = 0.0f;
        for (uint64_t t = 0; t < len; ++t) { ph[t] = expf(ph[t] - top); sum += ph[t]; }
        res[h * (dh + 2)] = top; res[h * (dh + 2) + 1] = sum;
        for (uint64_t e = 0; e < dh; ++e) {
            float acc = 0.0f;
            for (uint64_t t = 0; t < len; ++t) {
                const uint64_t row = t * kvh + g;
                acc += ph[t] * tq_element(vcodes + row * row_bytes, f16_to_f32(vscales[row]), d, e);
            }
            res[h * (dh + 2) + 2 + e] = acc;
        }
    }
}

/* ---- the small steps either side of attention in a mixer ------------------------------------------------------------ */
void oracle_vector_add(uint16_t* z, const uint16_t* x, const uint16_t* y, uint64_t n) {                  /* kernels.cuh:103-113 */
    for (uint64_t i = 0; i < n; ++i) z[i] = f32_to_f16(f16_to_f32(x[i]) + f16_to_f32(y[i]), 0);
}
void oracle_vector_copy_rows(uint16_t* out, uint64_t out_row, const uint16_t* in, uint64_t in_row, uint64_t width, uint64_t rows) {   /* :3874-3881 */
    for (uint64_t t = 0; t < rows; ++t) for (uint64_t j = 0; j < width; ++j) out[t * out_row + j] = in[t * in_row + j];
}
void oracle_rmsnorm_rows(uint16_t* o, const uint16_t* x, const uint16_t* w, uint64_t n, uint64_t rows, uint64_t x_stride, uint64_t o_stride, float eps) {
    for (uint64_t r = 0; r < rows; ++r) {                                                                  /* :158-176, 1700-1705 */
        const uint16_t* xr = x + r * x_stride;
        float part = 0.0f;
        for (uint64_t i = 0; i < n; ++i) { const float v = f16_to_f32(xr[i]); part += v * v; }
        const float scale = 1.0f / sqrtf(part / (float)n + eps);
        for (uint64_t i = 0; i < n; ++i) o[r * o_stride + i] = f32_to_f16((f16_to_f32(xr[i]) * scale) * f16_to_f32(w[i]), 0);
    }
}
void oracle_rope_rows(uint16_t* o, const uint16_t* x, const float* cs, uint64_t rows, uint64_t heads, uint64_t head_stride, uint64_t row_stride, uint64_t rot) {
    const uint64_t pairs = rot / 2;                                                                        /* :1710-1727; rows = 1 is :843-858 */
    for (uint64_t r = 0; r < rows; ++r) for (uint64_t e = 0; e < heads; ++e) for (uint64_t k = 0; k < pairs; ++k) {
        const uint64_t at = r * row_stride + e * head_stride + k;
        const float a = f16_to_f32(x[at]), b = f16_to_f32(x[at + pairs]), c = cs[r * rot + k], s = cs[r * rot + pairs + k];
        o[at] = f32_to_f16(a * c - b * s, 0); o[at + pairs] = f32_to_f16(b * c + a * s, 0);
    }
}
void oracle_rope_interleaved(uint16_t* o, const uint16_t* x, const float* cs, uint64_t heads, uint64_t head_stride, uint64_t rot, uint64_t inverse) {
    const uint64_t pairs = rot / 2;                                                                        /* :1733-1749 */
    for (uint64_t h = 0; h < heads; ++h) for (uint64_t k = 0; k < pairs; ++k) {
        const uint64_t at = h * head_stride + 2 * k;
        const float a = f16_to_f32(x[at]), b = f16_to_f32(x[at + 1]), c = cs[k], sn = inverse ? -cs[pairs + k] : cs[pairs + k];
        o[at] = f32_to_f16(a * c - b * sn, 0); o[at + 1] = f32_to_f16(b * c + a * sn, 0);
    }
}
/* mode 0: rows from position `first` (:871-886, 1754-1767) · 1: M-RoPE (:1770-1784) · 2: axial (:1789-1803) */
void oracle_rope_angles(float* cs, uint64_t first, const uint32_t* positions, float theta, uint64_t head_dim, uint64_t rows, uint64_t sections, int mode) {
    const uint64_t pairs = head_dim / 2, per_axis = pairs / 2;
    const float r = expf(-2.0f / (float)(uint32_t)(mode == 2 ? pairs : head_dim) * logf(theta));
    for (uint64_t row = 0; row < rows; ++row) for (uint64_t k = 0; k < pairs; ++k) {
        uint64_t steps = k, pos = first + row;
        if (mode == 1) {
            const uint64_t third = k % 3, by_row = sections & 0xFFFF, by_column = (sections >> 16) & 0xFFFF;
            pos = positions[3 * row + ((third == 1 && k < 3 * by_row) ? 1 : (third == 2 && k < 3 * by_column) ? 2 : 0)];
        } else if (mode == 2) { const uint64_t axis = k < per_axis ? 0 : 1; steps = k - axis * per_axis; pos = positions[2 * row + axis]; }
        float frequency = 1.0f;
        for (uint64_t m = 0; m < steps; ++m) frequency *= r;
        const float angle = (float)pos * frequency;
        cs[row * head_dim + k] = cosf(angle); cs[row * head_dim + pairs + k] = sinf(angle);
    }
}
void oracle_attention_gate_rows(uint16_t* o, const uint16_t* att, const uint16_t* qg, uint64_t heads, uint64_t head_dim) {   /* :2062-2076 */
    for (uint64_t i = 0; i < heads * head_dim; ++i) {
        const uint64_t h = i / head_dim, e = i - h * head_dim;
        const uint16_t gate = f32_to_f16(1.0f / (1.0f + expf(-f16_to_f32(qg[h * 2 * head_dim + head_dim + e]))), 0);
        o[i] = f32_to_f16(f16_to_f32(att[i]) * f16_to_f32(gate), 0);
    }
}

/* ---- the weight path's doors a mixer runs around its attention ------------------------------------------------------
 * hadamard_rotate (kernels.cuh:2189-2231): the block rotation H·(S ⊙ u)/sqrt(b) over a row of n — blocks of 512, then one of
 * 256 and one of 128 for what is left; a row shorter than 512 is one block of n.  Four running sums, columns c mod 4. */
void oracle_hadamard_rotate(uint16_t* out, const uint16_t* in, const uint16_t* sign, uint64_t n) {
    const uint64_t whole = n < 512 ? 0 : (n / 512) * 512, rest = n - whole;
    for (uint64_t i = 0; i < n; ++i) {
        uint64_t a = 0, b = n;
        if (i < whole) { a = i - i % 512; b = 512; }
        else if (whole != 0) {
            if (rest >= 256 && i < whole + 256) { a = whole; b = 256; }
            else { a = whole + (rest >= 256 ? 256 : 0); b = 128; }
        }
        const uint64_t r = i - a;
        float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        uint64_t c = 0;
        for (; c + 4 <= b; c += 4)
            for (int k = 0; k < 4; ++k) {
                const float v = f16_to_f32(in[a + c + k]) * f16_to_f32(sign[c + k]);
                s[k] += (__builtin_popcountll(r & (c + k)) & 1) ? -v : v;
            }
        for (; c < b; ++c) { const float v = f16_to_f32(in[a + c]) * f16_to_f32(sign[c]); s[0] += (__builtin_popcountll(r & c) & 1) ? -v : v; }
        out[i] = f32_to_f16(((s[0] + s[1]) + (s[2] + s[3])) / sqrtf((float)b), 0);
    }
}
/* turboquant_gemv (kernels.cuh:1405-1447): out[r] = half(scale_r · sum_c level(code[r][c]) · x[c]); the sum in column order */
void oracle_turboquant_gemv(uint16_t* out, const uint8_t* weights, const uint8_t* luts, const uint16_t* x, uint64_t d, uint64_t rows, uint64_t cols) {
    const uint64_t need = tq_row_bytes(d, cols);
    for (uint64_t r = 0; r < rows; ++r) {
        float part = 0.0f;
        for (uint64_t c = 0; c < cols; ++c) part += tq_element(weights + r * need, 1.0f, d, c) * f16_to_f32(x[c]);
        const float scale = d == 16 ? 1.0f : f16_to_f32((uint16_t)((uint32_t)luts[r * 2] | ((uint32_t)luts[r * 2 + 1] << 8)));
        out[r] = f32_to_f16(part * scale, 0);
    }
}

/* ---- the GLM mixer's doors: Kimi Delta Attention, the latent's absorb and expand, the sparse attention's indexer --------
 * KDA (kernels.cuh:3301-3470): DeltaNet's recurrence with a decay a key channel.  `eg` null: the decays are made from f, dt
 * and a_log (kda_step, kda_steps); else read (kda_steps_decayed, with kda_decays before it).  conved is the rows' q, then
 * their k, then their v, each `heads·d` wide a row. */
static float kda_decay(float lower, float a, uint16_t f, uint16_t dt) { return expf(lower / (1.0f + expf(-a * (f16_to_f32(f) + f16_to_f32(dt))))); }
void oracle_kda_decays(float* eg, const uint16_t* f, const uint16_t* dt, const uint16_t* a_log, uint64_t heads, uint64_t d, float lower, uint64_t rows) {
    const uint64_t width = heads * d;                                                                     /* :3400-3409 */
    for (uint64_t x = 0; x < rows * width; ++x) { const uint64_t c = x % width; eg[x] = kda_decay(lower, expf(f16_to_f32(a_log[c / d])), f[x], dt[c]); }
}
void oracle_kda_steps(float* S, const uint16_t* conved, const uint16_t* f, const float* eg, const uint16_t* b, const uint16_t* dt, const uint16_t* a_log,
                      const uint16_t* gate, const uint16_t* w, uint16_t* out, uint64_t heads, uint64_t d, float lower, float eps, uint64_t rows) {
    const uint64_t width = heads * d;
    const uint16_t *q = conved, *k = conved + rows * width, *v = conved + 2 * rows * width;
    for (uint64_t h = 0; h < heads; ++h) {
        float* Sh = S + h * d * d;
        const float a = eg ? 0.0f : expf(f16_to_f32(a_log[h]));
        for (uint64_t t = 0; t < rows; ++t) {                                                             /* :3312-3347 a row of a head */
            const uint64_t at = t * width + h * d;
            const float beta = 1.0f / (1.0f + expf(-f16_to_f32(b[t * heads + h])));
            float qq = 0.0f, kk = 0.0f;
            for (uint64_t i = 0; i < d; ++i) { const float qi = f16_to_f32(q[at + i]), ki = f16_to_f32(k[at + i]); qq += qi * qi; kk += ki * ki; }
            const float inv_q = 1.0f / sqrtf(qq + 1e-6f) / sqrtf((float)d), inv_k = 1.0f / sqrtf(kk + 1e-6f);
            float oo = 0.0f;
            for (uint64_t j = 0; j < d; ++j) {
                float kv = 0.0f;
                for (uint64_t i = 0; i < d; ++i) {
                    Sh[i * d + j] *= eg ? eg[at + i] : kda_decay(lower, a, f[at + i], dt[h * d + i]);
                    kv += Sh[i * d + j] * f16_to_f32(k[at + i]) * inv_k;
                }
                const float delta = (f16_to_f32(v[at + j]) - kv) * beta;
                float o = 0.0f;
                for (uint64_t i = 0; i < d; ++i) { const float s = Sh[i * d + j] + f16_to_f32(k[at + i]) * inv_k * delta; Sh[i * d + j] = s; o += s * f16_to_f32(q[at + i]); }
                out[at + j] = f32_to_f16(o * inv_q, 0);
                const float oj = f16_to_f32(out[at + j]);
                oo += oj * oj;
            }
            const float scale = 1.0f / sqrtf(oo / (float)d + eps);                                        /* :3350-3359 */
            for (uint64_t j = 0; j < d; ++j)
                out[at + j] = f32_to_f16(f16_to_f32(out[at + j]) * scale * f16_to_f32(w[j]) / (1.0f + expf(-f16_to_f32(gate[at + j]))), 0);
        }
    }
}
/* attention_absorb_rows (:3596-3627), attention_expand_rows (:3629-3664) */
void oracle_attention_absorb_rows(uint16_t* out, const uint16_t* q, const uint16_t* W, uint64_t heads, uint64_t nope, uint64_t latent, uint64_t stride,
                                  float scale, uint64_t rows) {
    for (uint64_t t = 0; t < rows; ++t) for (uint64_t h = 0; h < heads; ++h) for (uint64_t c = 0; c < latent; ++c) {
        float sum = 0.0f;
        for (uint64_t i = 0; i < nope; ++i) sum += f16_to_f32(W[(h * stride + i) * latent + c]) * f16_to_f32(q[(t * heads + h) * nope + i]);
        out[(t * heads + h) * latent + c] = f32_to_f16(sum * scale, 0);
    }
}
void oracle_attention_expand_rows(uint16_t* out, const uint16_t* o, const uint16_t* W, uint64_t heads, uint64_t width, uint64_t latent, uint64_t stride,
                                  uint64_t offset, uint64_t rows) {
    for (uint64_t t = 0; t < rows; ++t) for (uint64_t r = 0; r < heads * width; ++r) {
        const uint64_t h = r / width;
        float sum = 0.0f;
        for (uint64_t c = 0; c < latent; ++c) sum += f16_to_f32(W[(h * stride + offset + r % width) * latent + c]) * f16_to_f32(o[(t * heads + h) * latent + c]);
        out[t * heads * width + r] = f32_to_f16(sum, 0);
    }
}
/* the indexer (:3666-3846) */
void oracle_index_layernorm(uint16_t* o, const uint16_t* x, const uint16_t* w, const uint16_t* b, uint64_t n, float eps) {
    float sum = 0.0f, sq = 0.0f;
    for (uint64_t i = 0; i < n; ++i) sum += f16_to_f32(x[i]);
    const float mean = sum / (float)n;
    for (uint64_t i = 0; i < n; ++i) { const float dd = f16_to_f32(x[i]) - mean; sq += dd * dd; }
    const float inv = 1.0f / sqrtf(sq / (float)n + eps);
    for (uint64_t i = 0; i < n; ++i) o[i] = f32_to_f16((f16_to_f32(x[i]) - mean) * inv * f16_to_f32(w[i]) + f16_to_f32(b[i]), 0);
}
void oracle_index_pool(uint16_t* pooled, const uint16_t* keys, const uint16_t* gates, const uint16_t* ape, uint64_t first, uint64_t pools, uint64_t dim,
                       uint64_t kpool) {
    for (uint64_t e = 0; e < pools * dim; ++e) {
        const uint64_t p = first + e / dim, c = e % dim;
        float top = -INFINITY, den = 0.0f, num = 0.0f;
        for (uint64_t i = 0; i < kpool; ++i) { const float l = f16_to_f32(gates[(p * kpool + i) * dim + c]) + f16_to_f32(ape[i * dim + c]); if (l > top) top = l; }
        for (uint64_t i = 0; i < kpool; ++i) {
            const float wgt = expf(f16_to_f32(gates[(p * kpool + i) * dim + c]) + f16_to_f32(ape[i * dim + c]) - top);
            den += wgt; num += wgt * f16_to_f32(keys[(p * kpool + i) * dim + c]);
        }
        pooled[p * dim + c] = f32_to_f16(num / den, 0);
    }
}
static void index_score(float* scores, const uint16_t* q, const uint16_t* w, const uint16_t* pooled, uint64_t heads, uint64_t dim, uint64_t p, float scale) {
    const float per_head = 1.0f / sqrtf((float)heads);
    float part = 0.0f;
    for (uint64_t h = 0; h < heads; ++h) {
        float dot = 0.0f;
        for (uint64_t c = 0; c < dim; ++c) dot += f16_to_f32(q[h * dim + c]) * f16_to_f32(pooled[p * dim + c]);
        dot *= scale;
        part += (dot > 0.0f ? dot : 0.0f) * f16_to_f32(w[h]) * per_head;
    }
    scores[p] = part;
}
/* rows = 0: the one-row door over `pools` pools; else row u, position len0 + u - 1, scores its (len0 + u) / kpool finished pools */
void oracle_index_scores_rows(float* scores, uint64_t scores_row, const uint16_t* q, const uint16_t* w, const uint16_t* pooled, uint64_t heads, uint64_t dim,
                              uint64_t pools, uint64_t len0, uint64_t kpool, uint64_t rows, float scale) {
    if (rows == 0) { for (uint64_t p = 0; p < pools; ++p) index_score(scores, q, w, pooled, heads, dim, p, scale); return; }
    for (uint64_t u = 0; u < rows; ++u) for (uint64_t p = 0; p < (len0 + u) / kpool; ++p)
        index_score(scores + u * scores_row, q + u * heads * dim, w + u * heads, pooled, heads, dim, p, scale);
}
static uint32_t index_key(float f) { uint32_t u; memcpy(&u, &f, 4); return (u & 0x80000000u) ? ~u : (u | 0x80000000u); }
/* the k largest scores' pools (ties by lowest index) as positions in index order, then the tail's positions (:3789-3818) */
void oracle_index_select(uint32_t* index, uint32_t* count, const float* scores, uint64_t pools, uint64_t k, uint64_t kpool, uint64_t tail_first, uint64_t tail) {
    uint32_t cut = 0;
    if (pools > k)
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t want = cut | (1u << bit);
            uint64_t have = 0;
            for (uint64_t p = 0; p < pools; ++p) have += index_key(scores[p]) >= want;
            if (have >= k) cut = want;
        }
    uint64_t above = 0, n = 0;
    if (pools > k) for (uint64_t p = 0; p < pools; ++p) above += index_key(scores[p]) > cut;
    uint64_t ties = pools > k ? k - above : 0;
    for (uint64_t p = 0; p < pools; ++p) {
        int take = pools <= k;
        if (!take) { const uint32_t key = index_key(scores[p]); if (key > cut) take = 1; else if (key == cut && ties != 0) { take = 1; --ties; } }
        if (take) for (uint64_t i = 0; i < kpool; ++i) index[n++] = (uint32_t)(p * kpool + i);
    }
    for (uint64_t i = 0; i < tail; ++i) index[n++] = (uint32_t)(tail_first + i);
    count[0] = (uint32_t)n;
}
void oracle_index_select_rows(uint32_t* index, uint64_t index_row, uint32_t* counts, const float* scores, uint64_t scores_row, uint64_t k, uint64_t kpool,
                              uint64_t len0, uint64_t rows) {
    for (uint64_t u = 0; u < rows; ++u) {
        const uint64_t len = len0 + u, pools = len / kpool;
        oracle_index_select(index + u * index_row, counts + u, scores + u * scores_row, pools, k, kpool, pools * kpool, len - pools * kpool);
    }
}
void oracle_index_blocks(float* out, const float* scores, uint64_t pools, uint64_t block) {
    for (uint64_t b = 0; b < (pools + block - 1) / block; ++b) {
        const uint64_t end = (b + 1) * block < pools ? (b + 1) * block : pools;
        float best = scores[b * block];
        for (uint64_t p = b * block + 1; p < end; ++p) best = scores[p] > best ? scores[p] : best;
        out[b] = best;
    }
}
/* counts null: one row of `most` positions (index_gather); else row u's counts[u] positions (index_gather_rows) */
void oracle_index_gather_rows(uint16_t* out, uint64_t out_row, const uint16_t* src, const uint32_t* index, uint64_t index_row, const uint32_t* counts,
                              uint64_t most, uint64_t row, uint64_t rows) {
    for (uint64_t u = 0; u < rows; ++u) for (uint64_t i = 0; i < (counts ? counts[u] : most); ++i) for (uint64_t e = 0; e < row; ++e)
        out[u * out_row + i * row + e] = src[(uint64_t)index[u * index_row + i] * row + e];
}
