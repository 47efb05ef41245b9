/* kernels.h — host-side launchers of this library's kernels; the doors (family.cu) and the `silvann_b200_*`
 * entry points (ext.cu) are thin callers of these.  Every launcher validates nothing the caller has not already
 * validated except what only it can know (kernel fit), enqueues on the given stream and returns the runtime's error.
 * None of them synchronises the device. */
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace sv {

/* ---- split-KV decode (decode.cu) ------------------------------------------------------------------------ */

/* One unit of decode work: query heads [head0, head0+heads) of sequence `seq`, all sharing kv head `kvh`, over KV
 * tiles [tile_begin, tile_end) of decode_tile_positions(head_dim) positions.  Split `split` of `nsplit` for that (seq, head block); the partial
 * of split s is written to scratch slot `slot_base + s`, and `ticket` indexes the arrival counter of the group. */
struct DecodeItem {
    int32_t seq, kvh, head0, heads;
    int32_t tile_begin, tile_end, split, nsplit;
    int32_t slot_base, ticket, pad0, pad1;
};

/* Positions per KV tile of the decode kernel: 64 at head_dim 256, 128 at head_dim 128 and 64. */
inline uint32_t decode_tile_positions(uint32_t head_dim) { return head_dim >= 256u ? 64u : 128u; }
#define SV_DECODE_MAX_SLOTS 2048   /* scratch partial slots per device (per plan) */
#define SV_DECODE_MAX_TICKETS 8192

struct DecodeScratch {
    float* partials;        /* [slots][16][head_dim_max + 2] fp32 */
    unsigned int* tickets;  /* zero between launches: the last block of a group resets its ticket */
    uint32_t slots, tickets_n, slot_floats;
};

struct DecodeCall {
    void* o;                 /* [seqs][q_heads][head_dim] 16-bit, or null */
    float* res;              /* [seqs][q_heads][head_dim + 2] fp32 (m, l, acc), or null */
    const void* q;           /* [seqs][q_heads][head_dim] 16-bit */
    const void* k;           /* contiguous: [length][kv_heads][head_dim]; paged: pool [pages][page_pos][kv_heads][head_dim] */
    const void* v;
    uint64_t kv_rows;        /* rows the K/V maps span: length (contiguous) or pages * page_pos (paged) */
    const int32_t* page_table;  /* device [seqs][table_stride], or null for a contiguous cache */
    uint32_t table_stride, page_pos;
    const int32_t* seq_lens;    /* device [seqs] (paged), or null: every sequence is `length` long */
    const DecodeItem* items;    /* device work list, `n_items` long, or null for one sequence split evenly */
    uint32_t n_items;
    uint32_t seqs, q_heads, kv_heads, head_dim, length;
    uint32_t nsplit;            /* with items == null: 0 = choose */
    int dtype;                  /* SV_DTYPE_* */
    unsigned int* over;         /* device fault word or null */
    DecodeScratch scratch;
    cudaStream_t stream;
    const void* xf;             /* an XfParams (exchange.cuh) or null: the exchange step of a KV range split done in this launch — one contiguous
                                   sequence of at least two splits, else cudaErrorNotSupported and the caller exchanges in a launch of its own */
};

/* Whether the TMA kernel can take these shapes and addresses (head_dim 64/128/256, 16-byte aligned q/k/v, rows a
 * multiple of 16 bytes, whole query groups of at most 64 heads on a kv head). */
bool decode_fits(const DecodeCall& c);
/* Blocks the launch will use and scratch slots it needs, for a one-sequence call with items == null. */
void decode_auto_split(uint32_t length, uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim, uint32_t sms,
                       uint32_t* nsplit, uint32_t* head_blocks);
cudaError_t decode_launch(const DecodeCall& c);
/* Per-device scratch for calls that bring none (the doors): allocated once on first use, kept until exit. */
cudaError_t decode_device_scratch(DecodeScratch* out);
uint32_t device_sm_count();
/* Whether kernels that follow each other closely are launched as programmatic dependents (the default);
 * SILVANN_B200_PDL=0 turns it off for every kernel of the library, for a caller that cannot keep to what such a kernel
 * reads before it waits for the grid ahead (the one-sequence decode: the K and V planes; the coded GEMV: the codes and
 * their scales; every other kernel: nothing). */
bool pdl_allowed();
void note_launch(uint32_t kernels);    /* adds to the library's launch counter (family.cu) */
unsigned int* device_status_word();   /* device address of the bound device's status word (allocated on first use) */
cudaError_t static_status_take(unsigned int* word, int clear);   /* the allocation-free decode's own status word (decode.cu) */

/* ---- contract-faithful attention doors, any shape (attn_doors.cu) ------------------------------------------- */
cudaError_t scores_launch(float* p, const uint16_t* q, const uint16_t* k, uint64_t qh, uint64_t kvh, uint64_t d,
                          uint64_t length, int mode /*0 softmax, 1 weights+res, 2 raw grouped*/, float* res,
                          cudaStream_t st);
cudaError_t softmax_rows_launch(float* p, uint64_t rows, uint64_t length, cudaStream_t st);
cudaError_t mix_launch(uint16_t* o, float* res, const float* p, const uint16_t* v, uint64_t qh, uint64_t kvh,
                       uint64_t d, uint64_t length, unsigned int* over, cudaStream_t st);
cudaError_t merge_launch(float* into, const float* a, const float* b, uint64_t qh, uint64_t d, cudaStream_t st);
cudaError_t finish_launch(uint16_t* o, const float* res, uint64_t qh, uint64_t d, unsigned int* over, int dtype,
                          cudaStream_t st);
cudaError_t causal_scores_launch(float* p, const uint16_t* q, const uint16_t* k, uint64_t qh, uint64_t kvh, uint64_t d,
                                 uint64_t first, uint64_t rows, bool softmax, cudaStream_t st);
cudaError_t causal_softmax_launch(float* p, uint64_t qh, uint64_t first, uint64_t rows, cudaStream_t st);
cudaError_t causal_mix_launch(uint16_t* o, const float* p, const uint16_t* v, uint64_t qh, uint64_t kvh, uint64_t d,
                              uint64_t first, uint64_t rows, unsigned int* over, cudaStream_t st);
/* ---- the doors either side of the hot kernels (more_doors.cu) ------------------------------------------------ */
cudaError_t scores_grouped_rows_launch(float* p, uint64_t p_row, const uint16_t* q, uint64_t q_row, const uint16_t* k, uint64_t k_row,
                                       const uint32_t* lens, uint64_t qh, uint64_t kvh, uint64_t d, uint64_t rows, cudaStream_t st);
cudaError_t softmax_lens_launch(float* p, uint64_t p_row, const uint32_t* lens, uint64_t heads, uint64_t rows, cudaStream_t st);
cudaError_t softmax_sink_launch(float* p, const uint16_t* sink, uint64_t rows, uint64_t length, cudaStream_t st);
cudaError_t mix_rows_launch(uint16_t* o, uint64_t o_row, const float* p, uint64_t p_row, const uint16_t* v, uint64_t v_row, const uint32_t* lens,
                            uint64_t qh, uint64_t kvh, uint64_t d, uint64_t rows, unsigned int* over, cudaStream_t st);
cudaError_t deltanet_gates_rows_launch(uint16_t* beta, uint16_t* g, const uint16_t* a, const uint16_t* b, const uint16_t* a_log,
                                       const uint16_t* dt_bias, uint64_t heads, uint64_t rows, unsigned int* over, cudaStream_t st);
cudaError_t deltanet_conv_steps_launch(uint16_t* o, uint16_t* s, const uint16_t* w, const uint16_t* x, uint64_t ch, uint64_t rows,
                                       unsigned int* over, cudaStream_t st);
cudaError_t vector_sum_launch(uint16_t* out, const uint64_t* parts, uint64_t count, uint64_t n, unsigned int* over,
                              cudaStream_t st);
/* ---- the small steps either side of attention in a mixer (mixer_doors.cu) ------------------------------------- */
cudaError_t vector_add_launch(uint16_t* z, const uint16_t* x, const uint16_t* y, uint64_t n, unsigned int* over, cudaStream_t st);
cudaError_t vector_copy_rows_launch(uint16_t* out, uint64_t out_row, const uint16_t* in, uint64_t in_row, uint64_t width, uint64_t rows, cudaStream_t st);
cudaError_t rmsnorm_rows_launch(uint16_t* o, const uint16_t* x, const uint16_t* w, uint64_t n, uint64_t rows, uint64_t x_stride, uint64_t o_stride,
                                float eps, unsigned int* over, cudaStream_t st);
/* rmsnorm_rows then rope_rows over the same rows as one kernel (rows = positions x heads; the bits of the two doors in turn) */
cudaError_t rmsnorm_rope_rows_launch(uint16_t* o, const uint16_t* x, const uint16_t* w, const float* cs, uint64_t n, uint64_t rows, uint64_t heads,
                                     uint64_t x_stride, uint64_t o_stride, uint64_t rot, float eps, unsigned int* over, cudaStream_t st);
cudaError_t rope_rows_launch(uint16_t* o, const uint16_t* x, const float* cs, uint64_t rows, uint64_t heads, uint64_t head_stride, uint64_t row_stride,
                             uint64_t rot, unsigned int* over, cudaStream_t st);
cudaError_t rope_interleaved_launch(uint16_t* o, const uint16_t* x, const float* cs, uint64_t heads, uint64_t head_stride, uint64_t rot, uint64_t inverse,
                                    unsigned int* over, cudaStream_t st);
cudaError_t rope_angles_launch(float* cs, uint64_t first, const uint32_t* positions, float theta, uint64_t head_dim, uint64_t rows, uint64_t sections,
                               int mode /*0 plain, 1 M-RoPE, 2 axial*/, cudaStream_t st);
cudaError_t attention_gate_rows_launch(uint16_t* o, const uint16_t* att, const uint16_t* qg, uint64_t heads, uint64_t head_dim, unsigned int* over,
                                       cudaStream_t st);
/* ---- a coded matrix times up to eight vectors on the tensor cores, codes expanded in flight (tq_gemv.cu) ---- */
bool tq_gemv_fast_fits(const void* groups /*the door's by-value groups struct*/, uint64_t cols, uint64_t inputs);
/* rows_cap: null, or a group's rows trimmed to what its rooms hold */
struct XfParams;    /* exchange.cuh: with one, the answers are exchanged among the cards and added in member order in the same launch */
cudaError_t tq_gemv_fast_launch(uint16_t* out, const void* groups, const uint64_t* rows_cap, const uint16_t* x, uint64_t cols, uint64_t inputs,
                                uint64_t out_stride, unsigned int* over, cudaStream_t st, const XfParams* xf = nullptr);
/* ---- the GLM mixer's doors: Kimi Delta Attention, latent absorb / expand, the sparse attention's indexer (glm_doors.cu) ---- */
cudaError_t kda_decays_launch(float* eg, const uint16_t* f, const uint16_t* dt, const uint16_t* a_log, uint64_t heads, uint64_t head_dim, float lower,
                              uint64_t rows, cudaStream_t st);
cudaError_t kda_steps_launch(float* S, const uint16_t* conved, const uint16_t* f, const float* eg /*null: made from f, dt, a_log*/, const uint16_t* b,
                             const uint16_t* dt, const uint16_t* a_log, const uint16_t* gate, const uint16_t* w, uint16_t* out, uint64_t heads,
                             uint64_t head_dim, float lower, float eps, uint64_t rows, unsigned int* over, cudaStream_t st);
cudaError_t absorb_launch(uint16_t* out, const uint16_t* q, const uint16_t* W, uint64_t heads, uint64_t nope, uint64_t latent, uint64_t stride, float scale,
                          uint64_t rows, unsigned int* over, cudaStream_t st);
cudaError_t expand_launch(uint16_t* out, const uint16_t* o, const uint16_t* W, uint64_t heads, uint64_t width, uint64_t latent, uint64_t stride,
                          uint64_t offset, uint64_t rows, unsigned int* over, cudaStream_t st);
cudaError_t index_layernorm_launch(uint16_t* o, const uint16_t* x, const uint16_t* w, const uint16_t* b, uint64_t n, float eps, unsigned int* over,
                                   cudaStream_t st);
cudaError_t index_pool_launch(uint16_t* pooled, const uint16_t* keys, const uint16_t* gates, const uint16_t* ape, uint64_t first, uint64_t pools, uint64_t dim,
                              uint64_t kpool, unsigned int* over, cudaStream_t st);
/* rows = 0: the one-row doors (every one of `pools` pools; the caller's tail) */
cudaError_t index_scores_launch(float* scores, uint64_t scores_row, const uint16_t* q, const uint16_t* w, const uint16_t* pooled, uint64_t heads, uint64_t dim,
                                uint64_t pools, uint64_t len0, uint64_t kpool, uint64_t rows, float scale, cudaStream_t st);
cudaError_t index_select_launch(uint32_t* index, uint64_t index_row, uint32_t* counts, const float* scores, uint64_t scores_row, uint64_t pools, uint64_t k,
                                uint64_t kpool, uint64_t tail_first, uint64_t tail, uint64_t len0, uint64_t rows, cudaStream_t st);
cudaError_t index_blocks_launch(float* out, const float* scores, uint64_t pools, uint64_t block, cudaStream_t st);
cudaError_t index_gather_launch(uint16_t* out, uint64_t out_row, const uint16_t* src, const uint32_t* index, uint64_t index_row, const uint32_t* counts /*null: all*/,
                                uint64_t most, uint64_t row, uint64_t rows, cudaStream_t st);
/* ---- the TurboQuant-coded tiers of the cache, as worded (tq.cu) ------------------------------------------------ */
bool tq_width_ok(uint64_t d);
cudaError_t tq_decode_launch(uint16_t* out, const uint8_t* weights, uint64_t w_room, const uint8_t* luts, uint64_t l_room, uint64_t d,
                             uint64_t rows, uint64_t cols, unsigned int* over, cudaStream_t st);
cudaError_t hadamard_blocks_launch(uint16_t* out, const uint16_t* in, const uint16_t* sign, uint64_t n, uint64_t block, uint64_t inverse,
                                   unsigned int* over, cudaStream_t st);
cudaError_t tq_encode_rows_launch(uint8_t* codes, uint16_t* scales, const uint16_t* x, uint64_t rows, uint64_t cols, uint64_t d,
                                  unsigned int* over, cudaStream_t st);
cudaError_t tq_weights_launch(float* p, float* res, const uint16_t* q, const uint8_t* codes, const uint16_t* scales, uint64_t qh, uint64_t kvh,
                              uint64_t d_head, uint64_t length, uint64_t d, uint64_t rows, cudaStream_t st);
cudaError_t hadamard_rotate_launch(uint16_t* out, const uint16_t* in, const uint16_t* sign, uint64_t n, unsigned int* over, cudaStream_t st);
/* attention_gate_rows then hadamard_rotate over the gated answers in one kernel, the bits of the two doors in turn */
cudaError_t gate_rotate_launch(uint16_t* rot, uint16_t* o, const uint16_t* att, const uint16_t* qg, const uint16_t* sign, uint64_t heads, uint64_t head_dim,
                               unsigned int* over, cudaStream_t st);
/* the norm of a row and its rotation in one kernel, the bits of the two doors in turn */
cudaError_t rmsnorm_rotate_launch(uint16_t* rot, uint16_t* o, const uint16_t* x, const uint16_t* w, const uint16_t* sign, uint64_t n, float eps,
                                  unsigned int* over, cudaStream_t st);
cudaError_t tq_gemv_groups_launch(uint16_t* out, const void* groups /* sv_tq_groups */, uint64_t w_room, uint64_t l_room, const uint16_t* x,
                                  uint64_t cols, unsigned int* over, cudaStream_t st);
/* ---- the expert-major GEMM: a coded matrix over several rows of x named by pairs (expert.cu) ---------------------- */
bool expert_width_ok(uint64_t d);
cudaError_t expert_rows_launch(uint16_t* out, float* acc, const uint8_t* weights, uint64_t w_room, const uint8_t* luts, uint64_t l_room, const uint16_t* x,
                               const uint32_t* pairs, const uint16_t* w, uint64_t count, uint64_t d, uint64_t out_rows, uint64_t cols, unsigned int* over,
                               cudaStream_t st);
cudaError_t expert_rows_finish_launch(uint16_t* out, float* acc, const uint16_t* residual, uint64_t n, unsigned int* over, cudaStream_t st);
cudaError_t expert_rows_reduce_launch(uint16_t* out, float* acc, const uint16_t* residual, uint64_t n, uint64_t k, uint64_t cols, unsigned int* over,
                                      cudaStream_t st);
cudaError_t expert_pairs_rows_launch(uint32_t* pairs, uint64_t n, uint64_t x_step, uint64_t x_at, uint64_t out_step, uint64_t out_at, cudaStream_t st);
bool expert_fast_fits(const void* groups /* sv_expert_groups */, const void* x, uint64_t cols);
cudaError_t expert_fast_launch(uint16_t* out, float* acc, const void* groups, const uint64_t* held /*one group: rows its rooms hold; null: all*/, const uint16_t* x,
                               const uint32_t* rows, const uint16_t* w, uint64_t cols, unsigned int* over, cudaStream_t st);
/* the pair weights_tq + residual_mix_tq as one kernel, codes expanded in flight (tq_decode.cu) */
bool tq_attend_fits(const void* q, const void* kcodes, const void* kscales, const void* vcodes, const void* vscales, uint64_t qh, uint64_t kvh,
                    uint64_t dh, uint64_t length, uint64_t d);
cudaError_t tq_attend_launch(float* res, const uint16_t* q, const uint8_t* kcodes, const uint16_t* kscales, const uint8_t* vcodes,
                             const uint16_t* vscales, uint64_t qh, uint64_t kvh, uint64_t dh, uint64_t length, uint64_t d, uint64_t rows /*of a prompt chunk; 1: one query*/, cudaStream_t st);
cudaError_t tq_residual_mix_launch(float* res, const float* p, const uint8_t* codes, const uint16_t* scales, uint64_t qh, uint64_t kvh,
                                   uint64_t d_head, uint64_t length, uint64_t d, uint64_t rows, cudaStream_t st);

}  // namespace sv

/* ---- latent attention at decode on tcgen05 / TMEM: many heads over one 512-wide latent that is key and value (mla_decode.cu) ---- */
namespace sv {
bool mla_decode_fits(const void* q, const void* latent, uint64_t heads, uint64_t head_dim, uint64_t length);
cudaError_t mla_decode_launch(void* o, float* res, const void* q, const void* latent, uint64_t heads, uint64_t length, int dtype, uint32_t blocks,
                              unsigned int* over, cudaStream_t st);
}  // namespace sv

/* ---- causal GQA prefill on tcgen05 / TMEM (prefill.cu) ------------------------------------------------------- */
namespace sv {
struct PrefillCall {
    void* o;                  /* [rows][q_heads][head_dim] 16-bit, or null */
    float* res;               /* [rows][q_heads][head_dim + 2] fp32 residuals (m, l, acc), or null */
    const void* q;            /* [rows][q_heads][head_dim] */
    const void* k;            /* [first + rows][kv_heads][head_dim] */
    const void* v;
    uint32_t q_heads, kv_heads, head_dim;
    uint64_t first, rows;     /* row r is position first + r and attends cache rows 0..first+r */
    int dtype;
    unsigned int* over;
    cudaStream_t stream;
};
bool prefill_fits(const PrefillCall& c);
cudaError_t prefill_launch(const PrefillCall& c);
}  // namespace sv
