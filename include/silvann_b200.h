/* silvann_b200.h — the C boundary of the B200 (sm_100a) attention silicon family for SiLVANN.
 *
 * One shared library, libsilvann_nvidia_b200.so, is loaded by an unmodified SiLVANN engine the way it loads any
 * silicon family: it looks up the single entry `silvann_silicon_family_get`, asks for ABI version 9 and receives a
 * table of per-package "door" tables — plain C function pointers over raw device addresses and sizes.  Everything in
 * the first half of this header restates that contract so that the library and its tests build without the engine's
 * sources; the field order and every signature must stay byte-compatible with the engine's own headers:
 *
 *   family table            engine/src/packages/sys/contracts/abi/silicon_family.cuh:33-59
 *   sys doors (31)          engine/src/packages/sys/contracts/abi/gpu.cuh:46-77 (meaning of each: :79-150)
 *   nn doors (137)          engine/src/packages/nn/contracts/abi/gpu.cuh:93-240
 *   by-value door structs   engine/src/packages/nn/contracts/abi/gpu.cuh:13-61
 *   the exported symbol     engine/src/silicon_families/entry.cuh:68-80
 *
 * The second half declares what the door ABI cannot express — bf16 element type, the paged KV pool with its page
 * table and pinned host tier, a one-call fused decode / causal prefill / DeltaNet, counters — as ordinary exported C
 * functions named `silvann_b200_*`.  They have no `__` in their names, so the engine's "one entry point and nothing
 * else of ours" build gate (engine/scripts/build_silicon_families.sh:73-79 counts only `<prefix>__` names) still holds.
 *
 * Conventions shared by every entry point: pointers named `*_dev` or passed to a door are device addresses of the
 * device bound to the calling thread; a "half" is 16 raw bits (IEEE fp16, or bf16 where a dtype argument says so);
 * all accumulation is fp32; nothing here throws, aborts or allocates behind the caller's back unless it says so. */
#ifndef SILVANN_B200_H
#define SILVANN_B200_H

#include <stddef.h>
#include <stdint.h>
#include <stdbool.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef uint16_t sv_h16;      /* 16 raw bits of an fp16 (door ABI) or bf16 (extension, by dtype) value */
typedef uint8_t  sv_u8;
typedef uint32_t sv_u32;
typedef uint64_t sv_u64;
typedef unsigned int sv_fault; /* a worker's device-resident fault word; doors OR a four-letter code into it */

/* ---- constants of the engine's contract ------------------------------------------------------------------ */
#define SILVANN_B200_ABI_VERSION     9u            /* silicon_family.cuh:31 */
#ifndef SILVANN_B200_FAMILY_ID                     /* both may be given at build time to answer to another roster name */
#define SILVANN_B200_FAMILY_ID       310u          /* a free roster slot above nvidia_cuda12 (300); ids < 1024 */
#endif
#ifndef SILVANN_B200_FAMILY_NAME
#define SILVANN_B200_FAMILY_NAME     "nvidia_b200"
#endif
#define SILVANN_B200_PACKAGES        7u            /* sys, nn, and five model packages with empty door tables */
#define SILVANN_B200_FAULT_OVERFLOW  0x4E504F56u   /* "NPOV": an fp32 result did not fit a half (primitives.cuh:57) */
#define SILVANN_B200_RESIDUAL_FLOATS(head_dim) ((head_dim) + 2u)  /* per head: m, l, acc[head_dim] (kernels.cuh:1186) */
#define SILVANN_B200_GATE_SILU       0u            /* deltanet.cuh:14-15 */
#define SILVANN_B200_GATE_SIGMOID    1u

/* ---- by-value structs some doors take (layout only; this family does not implement those doors) ----------- */
typedef struct sv_tq_groups     { sv_u64 codes[12], luts[12], rows[12], d[12], out_at[12], count; } sv_tq_groups;
typedef struct sv_expert_groups { sv_u64 codes[12], luts[12], out_rows[12], d[12], out_at[12], pairs_at[12], pairs[12], count; } sv_expert_groups;
typedef struct sv_vector_parts  { sv_u64 at[8], count; } sv_vector_parts;

/* ---- package 0: sys doors — memory, copies, queues, devices (sys/contracts/abi/gpu.cuh:46-77) ------------- */
#define SILVANN_B200_SYS_DOORS(D) \
    D( 0, bool,     memory_allocate,                 (void** at, size_t bytes)) \
    D( 1, void,     memory_free,                     (void* at)) \
    D( 2, bool,     memory_zerofill,                 (void* at, size_t bytes)) \
    D( 3, bool,     memory_read,                     (void* to, const void* from, size_t bytes)) \
    D( 4, bool,     memory_write,                    (void* to, const void* from, size_t bytes)) \
    D( 5, bool,     compute_completed,               (void)) \
    D( 6, bool,     side_open,                       (void** channel)) \
    D( 7, void,     side_close,                      (void* channel)) \
    D( 8, bool,     side_memory_read,                (void* to, const void* from, size_t bytes, void* channel)) \
    D( 9, bool,     side_memory_write,               (void* to, const void* from, size_t bytes, void* channel)) \
    D(10, bool,     memory_allocate_host_ram_mapped, (void** at, void** card_at, size_t bytes)) \
    D(11, void,     memory_free_host_ram,            (void* at)) \
    D(12, uint32_t, device_count,                    (void)) \
    D(13, uint32_t, bind_device,                     (uint32_t index)) \
    D(14, uint32_t, bound_device,                    (void)) \
    D(15, bool,     memory_register_host,            (void* at, size_t bytes, void** card_at)) \
    D(16, void,     memory_unregister_host,          (void* at)) \
    D(17, bool,     file_open,                       (const char* path, uint64_t* handle)) \
    D(18, void,     file_close,                      (uint64_t handle)) \
    D(19, bool,     file_read,                       (uint64_t handle, uint64_t offset, uint64_t bytes, void* to)) \
    D(20, bool,     memory_map_file,                 (void* at, size_t bytes, uint64_t handle, uint64_t offset)) \
    D(21, bool,     memory_prefetch,                 (const void* at, size_t bytes)) \
    D(22, bool,     peer_access,                     (uint32_t other)) \
    D(23, bool,     mark_open,                       (void** mark)) \
    D(24, void,     mark_close,                      (void* mark)) \
    D(25, bool,     mark_record,                     (void* mark)) \
    D(26, bool,     mark_wait,                       (void* mark)) \
    D(27, bool,     side_memory_write_queued,        (void* to, const void* from, size_t bytes, void* channel)) \
    D(28, bool,     side_memory_read_queued,         (void* to, const void* from, size_t bytes, void* channel)) \
    D(29, bool,     side_mark_record,                (void* mark, void* channel)) \
    D(30, bool,     mark_reached,                    (void* mark))

#define SILVANN_B200_FIELD_SYS(IDX, RET, NAME, PARAMS) RET (*NAME) PARAMS;
typedef struct silvann_b200_sys_doors {
    uint32_t size;                       /* sizeof(this) as the library was built: 256 */
    SILVANN_B200_SYS_DOORS(SILVANN_B200_FIELD_SYS)
} silvann_b200_sys_doors;

/* ---- package 1: nn doors, in the engine's append-only order (nn/contracts/abi/gpu.cuh:93-230) ------------- *
 * Every door returns void, enqueues work on the bound device's default queue and returns.  This family answers the
 * attention and Gated-DeltaNet rows (25, 26, 28-31, 34, 61, 62, 66, 95-98, 133) with its own sm_100a kernels; the
 * other rows are present, never null, and refuse: they print one line, and the device's next `compute_completed`
 * answers false once, which the engine raises as the fault "SEWK" (nvidia_cuda12/sys.cuh:41-61 does the same for a
 * launch the runtime refused). */
#define SILVANN_B200_NN_DOORS(D) \
    D(  0, vector_zero, (sv_h16* v, sv_u64 n)) \
    D(  1, vector_exp, (sv_h16* o, const sv_h16* x, sv_u64 n, sv_fault* over)) \
    D(  2, vector_softplus, (sv_h16* o, const sv_h16* x, sv_u64 n, sv_fault* over)) \
    D(  3, vector_scale, (sv_h16* o, const sv_h16* x, sv_u64 n, float factor, sv_fault* over)) \
    D(  4, vector_add, (sv_h16* z, const sv_h16* x, const sv_h16* y, sv_u64 n, sv_fault* over)) \
    D(  5, vector_pointwise_mul, (sv_h16* z, const sv_h16* x, const sv_h16* y, sv_u64 n, sv_fault* over)) \
    D(  6, rmsnorm, (sv_h16* o, const sv_h16* x, const sv_h16* w, sv_u64 n, float eps, sv_fault* over)) \
    D(  7, vector_l2norm, (sv_h16* o, const sv_h16* x, sv_u64 n, sv_fault* over)) \
    D(  8, softmax, (sv_h16* o, const sv_h16* x, sv_u64 n, sv_fault* over)) \
    D(  9, sigmoid, (sv_h16* o, const sv_h16* x, sv_u64 n, sv_fault* over)) \
    D( 10, vector_scale_at, (sv_h16* o, const sv_h16* x, const sv_h16* a, sv_u64 which, sv_u64 n, sv_fault* over)) \
    D( 11, matrix_transpose, (sv_h16* d, const sv_h16* s, sv_u64 rows, sv_u64 cols)) \
    D( 12, matrix_matvec_transposed, (sv_h16* out, const sv_h16* W, const sv_h16* x, sv_u64 rows, sv_u64 cols, sv_fault* over)) \
    D( 13, argmax, (sv_u64* out, sv_u64 stamp, const sv_h16* x, sv_u64 n)) \
    D( 14, vector_dot_product, (sv_u64* out, sv_u64 stamp, const sv_h16* a, const sv_h16* b, sv_u64 n)) \
    D( 15, vector_at, (sv_u64* out, sv_u64 stamp, const sv_h16* x, sv_u64 i)) \
    D( 16, swiglu_combine, (sv_h16* o, const sv_h16* g, const sv_h16* u, sv_u64 n, sv_fault* over)) \
    D( 17, deltanet_rank_1_update, (float* S, const sv_h16* k, const sv_h16* d, float g, sv_u64 k_dim, sv_u64 v_dim)) \
    D( 18, deltanet_readout, (sv_h16* o, const float* S, const sv_h16* x, sv_u64 k_dim, sv_u64 v_dim, sv_fault* over)) \
    D( 19, deltanet_conv_step, (sv_h16* o, sv_h16* s, const sv_h16* w, const sv_h16* x, sv_u64 ch, sv_fault* over)) \
    D( 20, expert_multiply_fp16, (sv_h16* out, const sv_h16* W, const sv_h16* x, sv_u64 rows, sv_u64 cols, sv_fault* over)) \
    D( 21, turboquant_decode, (sv_h16* out, const sv_u8* weights, sv_u64 w_room, const sv_u8* luts, sv_u64 l_room, sv_u64 d, sv_u64 rows, sv_u64 cols, sv_fault* over)) \
    D( 22, turboquant_gemv, (sv_h16* out, const sv_u8* weights, sv_u64 w_room, const sv_u8* luts, sv_u64 l_room, const sv_h16* x, sv_u64 d, sv_u64 rows, sv_u64 cols, sv_fault* over)) \
    D( 23, hadamard_rotate, (sv_h16* out, const sv_h16* in, const sv_h16* sign, sv_u64 n, sv_fault* over)) \
    D( 24, rope, (sv_h16* o, const sv_h16* x, const float* cs, sv_u64 heads, sv_u64 head_dim, sv_fault* over)) \
    D( 25, attention_scores, (float* p, const sv_h16* q, const sv_h16* k, sv_u64 q_heads, sv_u64 kv_heads, sv_u64 head_dim, sv_u64 length)) \
    D( 26, attention_mix, (sv_h16* o, const float* p, const sv_h16* v, sv_u64 q_heads, sv_u64 kv_heads, sv_u64 head_dim, sv_u64 length, sv_fault* over)) \
    D( 27, rope_angles, (float* cs, sv_u64 position, float theta, sv_u64 head_dim)) \
    D( 28, attention_weights, (float* p, float* res, const sv_h16* q, const sv_h16* k, sv_u64 q_heads, sv_u64 kv_heads, sv_u64 head_dim, sv_u64 length)) \
    D( 29, attention_residual_mix, (float* res, const float* p, const sv_h16* v, sv_u64 q_heads, sv_u64 kv_heads, sv_u64 head_dim, sv_u64 length)) \
    D( 30, attention_merge, (float* into, const float* a, const float* b, sv_u64 q_heads, sv_u64 head_dim)) \
    D( 31, attention_finish, (sv_h16* o, const float* res, sv_u64 q_heads, sv_u64 head_dim, sv_fault* over)) \
    D( 32, vector_top_k, (sv_u64* values, sv_u64 stride, sv_h16* weights, const sv_h16* x, sv_u64 n, sv_u64 k)) \
    D( 33, turboquant_gemv_int8, (sv_h16* out, const sv_u8* weights, sv_u64 w_room, const sv_u8* luts, sv_u64 l_room, const sv_h16* x, sv_u64 d, sv_u64 rows, sv_u64 cols, sv_fault* over)) \
    D( 34, deltanet_step, (float* S, const sv_h16* conved, const sv_h16* z, const sv_h16* beta, const sv_h16* g, const sv_h16* w, sv_h16* out, sv_u64 k_heads, sv_u64 v_heads, sv_u64 head_dim, sv_fault* over)) \
    D( 35, turboquant_gemv_groups, (sv_h16* out, sv_tq_groups g, const sv_h16* x, sv_u64 cols, sv_fault* over)) \
    D( 36, turboquant_gemv_groups_sum, (sv_h16* out, sv_tq_groups g, const sv_h16* x, const sv_h16* w, const sv_h16* residual, sv_u64 rows, sv_u64 cols, sv_fault* over)) \
    D( 37, turboquant_gemv_groups_int8, (sv_h16* out, sv_tq_groups g, const sv_h16* x, sv_u64 cols, sv_fault* over)) \
    D( 38, turboquant_gemv_groups_sum_int8, (sv_h16* out, sv_tq_groups g, const sv_h16* x, const sv_h16* w, const sv_h16* residual, sv_u64 rows, sv_u64 cols, sv_fault* over)) \
    D( 39, swiglu_pairs, (sv_h16* o, const sv_h16* gu, sv_u64 pairs, sv_u64 n, sv_fault* over)) \
    D( 40, expert_rows, (sv_h16* out, const sv_u8* weights, sv_u64 w_room, const sv_u8* luts, sv_u64 l_room, const sv_h16* x, const sv_u32* rows, sv_u64 count, sv_u64 d, sv_u64 out_rows, sv_u64 cols, sv_fault* over)) \
    D( 41, expert_rows_sum, (float* acc, const sv_u8* weights, sv_u64 w_room, const sv_u8* luts, sv_u64 l_room, const sv_h16* x, const sv_u32* rows, const sv_h16* w, sv_u64 count, sv_u64 d, sv_u64 out_rows, sv_u64 cols)) \
    D( 42, expert_groups, (sv_h16* out, sv_expert_groups g, const sv_h16* x, const sv_u32* rows, sv_u64 cols, sv_fault* over)) \
    D( 43, expert_rows_finish, (sv_h16* out, float* acc, const sv_h16* residual, sv_u64 n, sv_fault* over)) \
    D( 44, expert_rows_reduce, (sv_h16* out, float* acc, const sv_h16* residual, sv_u64 n, sv_u64 k, sv_u64 cols, sv_fault* over)) \
    D( 45, rmsnorm_rows, (sv_h16* o, const sv_h16* x, const sv_h16* w, sv_u64 n, sv_u64 rows, sv_u64 x_stride, sv_u64 o_stride, float eps, sv_fault* over)) \
    D( 46, rope_rows, (sv_h16* o, const sv_h16* x, const float* cs, sv_u64 rows, sv_u64 heads, sv_u64 head_stride, sv_u64 row_stride, sv_u64 rot, sv_fault* over)) \
    D( 47, rope_angles_rows, (float* cs, sv_u64 first, float theta, sv_u64 head_dim, sv_u64 rows)) \
    D( 48, rope_angles_mrope_rows, (float* cs, const sv_u32* positions, float theta, sv_u64 head_dim, sv_u64 rows, sv_u64 sections)) \
    D( 49, rope_angles_axial_rows, (float* cs, const sv_u32* positions, float theta, sv_u64 head_dim, sv_u64 rows)) \
    D( 50, layernorm_rows, (sv_h16* o, const sv_h16* x, const sv_h16* w, const sv_h16* b, sv_u64 n, sv_u64 rows, sv_u64 x_stride, sv_u64 o_stride, float eps, sv_fault* over)) \
    D( 51, vector_bias_rows, (sv_h16* o, const sv_h16* x, const sv_h16* b, sv_u64 n, sv_u64 rows, sv_fault* over)) \
    D( 52, vector_gelu, (sv_h16* o, const sv_h16* x, sv_u64 n, sv_u64 exact, sv_fault* over)) \
    D( 53, attention_set, (sv_h16* o, const sv_h16* qkv, sv_u64 rows, sv_u64 heads, sv_u64 head_dim, sv_fault* over)) \
    D( 54, attention_limits, (sv_h16* o, const sv_h16* q, const sv_h16* k, const sv_h16* v, const sv_u32* limits, sv_u64 rows, sv_u64 heads, sv_u64 head_dim, sv_u64 q_stride, sv_u64 kv_stride, sv_fault* over)) \
    D( 55, vector_gated_add_rows, (sv_h16* o, const sv_h16* x, const sv_h16* y, const sv_h16* g, sv_u64 n, sv_u64 rows, sv_fault* over)) \
    D( 56, vector_tanh, (sv_h16* o, const sv_h16* x, sv_u64 n, sv_fault* over)) \
    D( 57, vector_silu, (sv_h16* o, const sv_h16* x, sv_u64 n, sv_fault* over)) \
    D( 58, unfold_rows, (sv_h16* o, const sv_h16* x, sv_u64 H, sv_u64 W, sv_u64 C, sv_u64 kh, sv_u64 kw, sv_u64 stride, sv_u64 pad_top, sv_u64 pad_left, sv_u64 up, sv_u64 Wo, sv_u64 r0, sv_u64 rows)) \
    D( 59, depth_to_space_rows, (sv_h16* o, const sv_h16* x, sv_u64 H, sv_u64 W, sv_u64 C, sv_u64 f)) \
    D( 60, hadamard_ladder_rows, (sv_h16* out, const sv_h16* in, const sv_h16* sign, sv_u64 cols, sv_u64 rows, sv_fault* over)) \
    D( 61, attention_causal_scores, (float* p, const sv_h16* q, const sv_h16* k, sv_u64 q_heads, sv_u64 kv_heads, sv_u64 head_dim, sv_u64 first, sv_u64 rows)) \
    D( 62, attention_causal_mix, (sv_h16* o, const float* p, const sv_h16* v, sv_u64 q_heads, sv_u64 kv_heads, sv_u64 head_dim, sv_u64 first, sv_u64 rows, sv_fault* over)) \
    D( 63, attention_gate_rows, (sv_h16* o, const sv_h16* att, const sv_h16* qg, sv_u64 heads, sv_u64 head_dim, sv_fault* over)) \
    D( 64, deltanet_gates_rows, (sv_h16* beta, sv_h16* g, const sv_h16* a, const sv_h16* b, const sv_h16* a_log, const sv_h16* dt_bias, sv_u64 heads, sv_u64 rows, sv_fault* over)) \
    D( 65, deltanet_conv_steps, (sv_h16* o, sv_h16* s, const sv_h16* w, const sv_h16* x, sv_u64 ch, sv_u64 rows, sv_fault* over)) \
    D( 66, deltanet_steps, (float* S, const sv_h16* conved, const sv_h16* z, const sv_h16* beta, const sv_h16* g, const sv_h16* w, sv_h16* out, sv_u64 k_heads, sv_u64 v_heads, sv_u64 head_dim, sv_u64 rows, sv_fault* over)) \
    D( 67, hadamard_blocks, (sv_h16* out, const sv_h16* in, const sv_h16* sign, sv_u64 n, sv_u64 block, sv_u64 inverse, sv_fault* over)) \
    D( 68, turboquant_encode_rows, (sv_u8* codes, sv_h16* scales, const sv_h16* x, sv_u64 rows, sv_u64 cols, sv_u64 d, sv_fault* over)) \
    D( 69, attention_weights_tq, (float* p, float* res, const sv_h16* q, const sv_u8* codes, const sv_h16* scales, sv_u64 q_heads, sv_u64 kv_heads, sv_u64 head_dim, sv_u64 length, sv_u64 d)) \
    D( 70, attention_residual_mix_tq, (float* res, const float* p, const sv_u8* codes, const sv_h16* scales, sv_u64 q_heads, sv_u64 kv_heads, sv_u64 head_dim, sv_u64 length, sv_u64 d)) \
    D( 71, hyper_logits, (float* lg, const sv_h16* streams, const sv_h16* fn, sv_u64 hidden, sv_u64 mult, float norm_eps)) \
    D( 72, hyper_pre, (sv_h16* out, float* mix, const sv_h16* streams, const sv_h16* base, const sv_h16* scale, sv_u64 hidden, sv_u64 mult, sv_u64 iters, float eps, sv_fault* over)) \
    D( 73, hyper_post, (sv_h16* out, const sv_h16* streams, const sv_h16* y, const float* mix, sv_u64 hidden, sv_u64 mult, sv_fault* over)) \
    D( 74, kda_step, (float* S, const sv_h16* conved, const sv_h16* f, const sv_h16* b, const sv_h16* dt, const sv_h16* a_log, const sv_h16* gate, const sv_h16* w, sv_h16* out, sv_u64 heads, sv_u64 head_dim, float lower, float eps, sv_fault* over)) \
    D( 75, vector_top_k_biased, (sv_u64* values, sv_u64 stride, sv_h16* weights, const sv_h16* x, const sv_h16* bias, sv_u64 n, sv_u64 k, float scale)) \
    D( 76, swiglu_clamped, (sv_h16* act, const sv_h16* gu, sv_u64 pairs, sv_u64 n, float limit, sv_fault* over)) \
    D( 77, attention_absorb, (sv_h16* out, const sv_h16* q, const sv_h16* W, sv_u64 heads, sv_u64 nope, sv_u64 latent, sv_u64 stride, float scale, sv_fault* over)) \
    D( 78, attention_expand, (sv_h16* out, const sv_h16* o, const sv_h16* W, sv_u64 heads, sv_u64 width, sv_u64 latent, sv_u64 stride, sv_u64 offset, sv_fault* over)) \
    D( 79, index_layernorm, (sv_h16* o, const sv_h16* x, const sv_h16* w, const sv_h16* b, sv_u64 n, float eps, sv_fault* over)) \
    D( 80, index_pool, (sv_h16* pooled, const sv_h16* keys, const sv_h16* gates, const sv_h16* ape, sv_u64 first, sv_u64 pools, sv_u64 dim, sv_u64 kpool, sv_fault* over)) \
    D( 81, index_scores, (float* scores, const sv_h16* q, const sv_h16* w, const sv_h16* pooled, sv_u64 heads, sv_u64 dim, sv_u64 pools, float scale)) \
    D( 82, index_select, (sv_u32* index, sv_u32* count, const float* scores, sv_u64 pools, sv_u64 k, sv_u64 kpool, sv_u64 tail_first, sv_u64 tail)) \
    D( 83, index_gather, (sv_h16* out, const sv_h16* src, const sv_u32* index, sv_u64 n, sv_u64 row)) \
    D( 84, index_blocks, (float* out, const float* scores, sv_u64 pools, sv_u64 block)) \
    D( 85, vector_copy, (sv_h16* out, const sv_h16* in, sv_u64 n)) \
    D( 86, hyper_logits_rows, (float* lg, const sv_h16* streams, const sv_h16* fn, sv_u64 hidden, sv_u64 mult, float norm_eps, sv_u64 rows, sv_u64 lg_stride)) \
    D( 87, hyper_pre_rows, (sv_h16* out, float* mix, const sv_h16* streams, const sv_h16* base, const sv_h16* scale, sv_u64 hidden, sv_u64 mult, sv_u64 iters, float eps, sv_u64 rows, sv_u64 mix_stride, sv_fault* over)) \
    D( 88, hyper_post_rows, (sv_h16* out, const sv_h16* streams, const sv_h16* y, const float* mix, sv_u64 hidden, sv_u64 mult, sv_u64 rows, sv_u64 mix_stride, sv_fault* over)) \
    D( 89, kda_steps, (float* S, const sv_h16* conved, const sv_h16* f, const sv_h16* b, const sv_h16* dt, const sv_h16* a_log, const sv_h16* gate, const sv_h16* w, sv_h16* out, sv_u64 heads, sv_u64 head_dim, float lower, float eps, sv_u64 rows, sv_fault* over)) \
    D( 90, expert_groups_int8, (sv_h16* out, sv_expert_groups g, const sv_h16* x, const sv_u32* rows, sv_u64 cols, sv_fault* over)) \
    D( 91, expert_rows_sum_int8, (float* acc, const sv_u8* weights, sv_u64 w_room, const sv_u8* luts, sv_u64 l_room, const sv_h16* x, const sv_u32* rows, const sv_h16* w, sv_u64 count, sv_u64 d, sv_u64 out_rows, sv_u64 cols)) \
    D( 92, rank1_dots, (float* s, const sv_h16* v, const sv_u32* which, const sv_h16* x, const sv_h16* w, const sv_u32* w_at, sv_u64 n, sv_u64 cols, sv_u64 x_stride, sv_u64 w_stride)) \
    D( 93, rank1_add, (sv_h16* out, const sv_h16* r, const float* s, sv_u64 n, sv_u64 per, sv_u64 rows, sv_u64 out_stride, sv_fault* over)) \
    D( 94, rank1_spread, (float* acc, const sv_h16* r, const float* s, const sv_u32* row_of, sv_u64 n, sv_u64 rows, sv_u64 row_stride)) \
    D( 95, attention_scores_grouped, (float* p, const sv_h16* q, const sv_h16* k, sv_u64 q_heads, sv_u64 kv_heads, sv_u64 head_dim, sv_u64 length)) \
    D( 96, attention_softmax_rows, (float* p, sv_u64 rows, sv_u64 length)) \
    D( 97, attention_causal_scores_grouped, (float* p, const sv_h16* q, const sv_h16* k, sv_u64 q_heads, sv_u64 kv_heads, sv_u64 head_dim, sv_u64 first, sv_u64 rows)) \
    D( 98, attention_causal_softmax, (float* p, sv_u64 q_heads, sv_u64 first, sv_u64 rows)) \
    D( 99, vector_penalize, (sv_h16* x, sv_u64 n, const sv_u64* ids, sv_u64 stride, sv_u64 count, float penalty, sv_fault* over)) \
    D(100, vector_draw, (sv_u64* out, sv_u64 stamp, const sv_h16* w, sv_u64 k, float top_p, sv_u64 seed, sv_u64 pos)) \
    D(101, attention_weights_rows, (float* p, float* res, const sv_h16* q, const sv_h16* k, sv_u64 q_heads, sv_u64 kv_heads, sv_u64 head_dim, sv_u64 first, sv_u64 rows)) \
    D(102, attention_residual_mix_rows, (float* res, const float* p, const sv_h16* v, sv_u64 q_heads, sv_u64 kv_heads, sv_u64 head_dim, sv_u64 first, sv_u64 rows)) \
    D(103, attention_weights_tq_rows, (float* p, float* res, const sv_h16* q, const sv_u8* codes, const sv_h16* scales, sv_u64 q_heads, sv_u64 kv_heads, sv_u64 head_dim, sv_u64 length, sv_u64 d, sv_u64 rows)) \
    D(104, attention_residual_mix_tq_rows, (float* res, const float* p, const sv_u8* codes, const sv_h16* scales, sv_u64 q_heads, sv_u64 kv_heads, sv_u64 head_dim, sv_u64 length, sv_u64 d, sv_u64 rows)) \
    D(105, vector_sum, (sv_h16* out, sv_vector_parts parts, sv_u64 n, sv_fault* over)) \
    D(106, rope_interleaved, (sv_h16* o, const sv_h16* x, const float* cs, sv_u64 heads, sv_u64 head_stride, sv_u64 rot, sv_u64 inverse, sv_fault* over)) \
    D(107, attention_softmax_sink, (float* p, const sv_h16* sink, sv_u64 rows, sv_u64 length)) \
    D(108, hyper_collapse_fp32, (float* out, const float* mix, const float* streams, sv_u64 hidden, sv_u64 mult)) \
    D(109, vector_top_k_scored, (sv_u64* values, sv_u64 stride, sv_h16* weights, const sv_h16* x, const sv_h16* bias, sv_u64 n, sv_u64 k, float scale, sv_u64 score)) \
    D(110, engram_gate_fp32, (float* streams, const sv_h16* kv, const sv_h16* w, sv_u64 hidden, sv_u64 mult, float eps)) \
    D(111, turboquant_gemv_groups_n, (sv_h16* out, sv_tq_groups g, const sv_h16* x, sv_u64 cols, sv_u64 n, sv_u64 out_stride, sv_fault* over)) \
    D(112, rmsnorm_rotate, (sv_h16* rot, sv_h16* o, const sv_h16* x, const sv_h16* w, const sv_h16* sign, sv_u64 n, float eps, sv_fault* over)) \
    D(113, hyper_logits_fp32, (float* lg, const float* streams, const sv_h16* fn, sv_u64 hidden, sv_u64 mult, float norm_eps)) \
    D(114, hyper_pre_fp32, (float* out, float* mix, const float* streams, const sv_h16* base, const sv_h16* scale, sv_u64 hidden, sv_u64 mult, sv_u64 iters, float eps)) \
    D(115, hyper_post_fp32, (float* out, const float* streams, const sv_h16* y, const float* mix, sv_u64 hidden, sv_u64 mult)) \
    D(116, rmsnorm_fp32, (sv_h16* o, const float* x, const sv_h16* w, sv_u64 n, float eps, sv_fault* over)) \
    D(117, vector_widen, (float* out, const sv_h16* x, sv_u64 n)) \
    D(118, vector_copy_rows, (sv_h16* out, sv_u64 out_row, const sv_h16* in, sv_u64 in_row, sv_u64 width, sv_u64 rows)) \
    D(119, expert_multiply_fp16_rows, (sv_h16* out, const sv_h16* W, const sv_h16* x, sv_u64 rows, sv_u64 cols, sv_u64 n, sv_fault* over)) \
    D(120, vector_top_k_biased_rows, (sv_u64* values, sv_u64 stride, sv_u64 values_row, sv_h16* weights, sv_u64 weights_row, const sv_h16* x, const sv_h16* bias, sv_u64 n, sv_u64 k, float scale, sv_u64 rows)) \
    D(121, attention_absorb_rows, (sv_h16* out, const sv_h16* q, const sv_h16* W, sv_u64 heads, sv_u64 nope, sv_u64 latent, sv_u64 stride, float scale, sv_u64 rows, sv_fault* over)) \
    D(122, attention_expand_rows, (sv_h16* out, const sv_h16* o, const sv_h16* W, sv_u64 heads, sv_u64 width, sv_u64 latent, sv_u64 stride, sv_u64 offset, sv_u64 rows, sv_fault* over)) \
    D(123, kda_decays, (float* eg, const sv_h16* f, const sv_h16* dt, const sv_h16* a_log, sv_u64 heads, sv_u64 head_dim, float lower, sv_u64 rows)) \
    D(124, kda_steps_decayed, (float* S, const sv_h16* conved, const float* eg, const sv_h16* b, const sv_h16* gate, const sv_h16* w, sv_h16* out, sv_u64 heads, sv_u64 head_dim, float eps, sv_u64 rows, sv_fault* over)) \
    D(125, index_scores_rows, (float* scores, sv_u64 scores_row, const sv_h16* q, const sv_h16* w, const sv_h16* pooled, sv_u64 heads, sv_u64 dim, sv_u64 len0, sv_u64 kpool, sv_u64 rows, float scale)) \
    D(126, index_select_rows, (sv_u32* index, sv_u64 index_row, sv_u32* counts, const float* scores, sv_u64 scores_row, sv_u64 k, sv_u64 kpool, sv_u64 len0, sv_u64 rows)) \
    D(127, index_gather_rows, (sv_h16* out, sv_u64 out_row, const sv_h16* src, const sv_u32* index, sv_u64 index_row, const sv_u32* counts, sv_u64 most, sv_u64 row, sv_u64 rows)) \
    D(128, attention_scores_grouped_rows, (float* p, sv_u64 p_row, const sv_h16* q, sv_u64 q_row, const sv_h16* k, sv_u64 k_row, const sv_u32* lens, sv_u64 q_heads, sv_u64 kv_heads, sv_u64 head_dim, sv_u64 most, sv_u64 rows)) \
    D(129, attention_softmax_lens, (float* p, sv_u64 p_row, const sv_u32* lens, sv_u64 heads, sv_u64 rows)) \
    D(130, attention_mix_rows, (sv_h16* o, sv_u64 o_row, const float* p, sv_u64 p_row, const sv_h16* v, sv_u64 v_row, const sv_u32* lens, sv_u64 q_heads, sv_u64 kv_heads, sv_u64 head_dim, sv_u64 rows, sv_fault* over)) \
    D(131, vector_top_k_rows, (sv_u64* values, sv_u64 stride, sv_u64 values_row, sv_h16* weights, sv_u64 weights_row, const sv_h16* x, sv_u64 n, sv_u64 k, sv_u64 rows)) \
    D(132, expert_pairs_rows, (sv_u32* pairs, sv_u64 n, sv_u64 x_step, sv_u64 x_at, sv_u64 out_step, sv_u64 out_at)) \
    D(133, deltanet_steps_gate, (float* S, const sv_h16* conved, const sv_h16* z, const sv_h16* beta, const sv_h16* g, const sv_h16* w, sv_h16* out, sv_u64 k_heads, sv_u64 v_heads, sv_u64 head_dim, sv_u64 rows, unsigned int gate, sv_fault* over)) \
    D(134, rmsnorm_fp32_rows, (sv_h16* o, const float* x, const sv_h16* w, sv_u64 n, sv_u64 rows, sv_u64 period, float eps, sv_fault* over)) \
    D(135, gated_rank, (sv_h16* rot, sv_h16* act, const sv_h16* a, const sv_h16* sign, sv_u64 rank, float scale, sv_fault* over)) \
    D(136, gated_mean, (sv_h16* into, sv_h16* inj, const sv_h16* gt, const sv_h16* an, const sv_h16* ij, sv_u64 hidden, sv_u64 streams, float mean, sv_fault* over))

#define SILVANN_B200_FIELD_NN(IDX, NAME, PARAMS) void (*NAME) PARAMS;
typedef struct silvann_b200_nn_doors {
    uint32_t size;                       /* sizeof(this) as the library was built: 1104 */
    SILVANN_B200_NN_DOORS(SILVANN_B200_FIELD_NN)
} silvann_b200_nn_doors;

/* ---- packages 2..6: model packages whose door tables are a size word only (the ai_<model> packages, contracts/abi/gpu.cuh) */
typedef struct silvann_b200_empty_doors { uint32_t size; } silvann_b200_empty_doors;

/* ---- the family table and the one symbol the engine binds (silicon_family.cuh:48-59, entry.cuh:68-80) ------ */
typedef struct silvann_b200_family {
    uint32_t            abi_version;     /* 9 */
    uint32_t            size;            /* sizeof(this) */
    uint32_t            id;              /* SILVANN_B200_FAMILY_ID */
    uint32_t            package_count;   /* 7 */
    const char*         name;            /* "nvidia_b200" */
    const void* const*  package_doors;   /* [package id] -> that package's door table */
} silvann_b200_family;

/* Answers the family table when `abi_version` is 9 and a null pointer otherwise. */
const silvann_b200_family* silvann_silicon_family_get(uint32_t abi_version);

/* ================================================================================================================
 * Extension entry points — what the door ABI cannot say.
 *
 * Every function returns SILVANN_B200_OK or an error code and leaves a one-line message for
 * silvann_b200_last_error() (per thread).  `stream` is a cudaStream_t passed as void*, null meaning the bound
 * device's default queue.  `dtype` selects how 16-bit operands are read and results rounded.  `over` is a device
 * fault word (may be null): a finite result that does not fit the 16-bit type ORs SILVANN_B200_FAULT_OVERFLOW there.
 * Unless a function says otherwise it only enqueues work and does not wait for the device.
 * ================================================================================================================ */
#define SILVANN_B200_DTYPE_FP16 0
#define SILVANN_B200_DTYPE_BF16 1

#define SILVANN_B200_OK          0
#define SILVANN_B200_E_ARGUMENT  1   /* a shape, size or address the kernels cannot take; nothing was enqueued */
#define SILVANN_B200_E_CUDA      2   /* the CUDA runtime refused an allocation, copy or launch */
#define SILVANN_B200_E_TIMEOUT   3   /* a bounded device-side wait ran out; see silvann_b200_device_status */
#define SILVANN_B200_E_STATE     4   /* an object used before it was prepared, or after it was destroyed */

/* Indexes into the counter array of silvann_b200_counters_read. */
#define SILVANN_B200_COUNTER_FUSED_DECODE    0   /* attention_scores + attention_mix answered by one kernel */
#define SILVANN_B200_COUNTER_FUSED_RESIDUAL  1   /* attention_weights + attention_residual_mix answered by one kernel */
#define SILVANN_B200_COUNTER_FUSED_PREFILL   2   /* the three causal doors answered by one kernel */
#define SILVANN_B200_COUNTER_FLUSHED         3   /* a deferred door that had to run as worded */
#define SILVANN_B200_COUNTER_REFUSED         4   /* refused doors and refused launches */
#define SILVANN_B200_COUNTER_DELTANET        5   /* DeltaNet door calls */
#define SILVANN_B200_COUNTER_LAUNCHES        6   /* kernels of this library launched, all paths */
#define SILVANN_B200_COUNTER_EXT_CALLS       7   /* silvann_b200_* compute entry points called */
#define SILVANN_B200_COUNTER_GEMV_FAST       8   /* coded matrix-vector doors answered by the tensor-core kernel */
#define SILVANN_B200_COUNTER_FUSED_LATENT     9   /* scores_grouped + softmax_rows + mix over one latent answered by one kernel */
#define SILVANN_B200_COUNTER_EXPERT_FAST     10   /* expert-major GEMM doors answered by the tcgen05 kernel */
#define SILVANN_B200_COUNTER_FUSED_NORM_ROPE 11   /* neighbours of attention answered two doors a kernel: rmsnorm_rows + rope_rows over the same rows, attention_gate_rows + hadamard_rotate */
#define SILVANN_B200_COUNTERS                12

const char* silvann_b200_last_error(void);
/* Copies min(n, SILVANN_B200_COUNTERS) process-wide counters into out; reset != 0 zeroes them afterwards. */
int silvann_b200_counters_read(uint64_t* out, uint32_t n, int reset);
/* Waits for the bound device's default queue, then answers its status word: 0 when nothing went wrong; "B2TO"
 * (0x4232544F) ORed in when a kernel gave up on a bounded wait; SILVANN_B200_STATUS_BAD_PAGE ORed in when a paged decode
 * or append met a page-table entry, inside a sequence's length, that names no page of the pool (the tile was read as
 * zeros, the row was not written).  The word of silvann_b200_decode_noalloc — which lives in that entry point's fixed
 * array, because it may not allocate one — is ORed into the same answer.  clear != 0 zeroes both words. */
#define SILVANN_B200_STATUS_TIMEOUT  0x4232544Fu
#define SILVANN_B200_STATUS_BAD_PAGE 0x80000000u
int silvann_b200_device_status(uint32_t* word, int clear);

/* Fused split-KV decode of one query position over a contiguous cache — the work of attention_scores +
 * attention_mix (kernels.cuh:1133-1164), or of attention_weights + attention_residual_mix (:1189-1241) when `res`
 * is given.  q [q_heads][head_dim]; k, v [length][kv_heads][head_dim]; o [q_heads][head_dim] (may be null);
 * res [q_heads][head_dim + 2] fp32 = (m, l, acc) per head, unnormalised (may be null).  nsplit 0 lets the library
 * choose how many blocks share a kv head.  Uses the bound device's split scratch: calls on different streams of one
 * device must not overlap. */
int silvann_b200_decode(void* o, float* res, const void* q, const void* k, const void* v, uint64_t q_heads,
                        uint64_t kv_heads, uint64_t head_dim, uint64_t length, uint32_t nsplit, int dtype,
                        sv_fault* over, void* stream);

/* The same decode for callers that must not cause an allocation.  It has no counterpart in the reference: the
 * reference's doors never own memory, because the engine carves every buffer from pools it sized at boot — and that is
 * exactly the kind of caller this is for.  A host that has committed all of the card's memory up front, or that is
 * recording its work into a stream capture, cannot afford a library that reaches for cudaMalloc on first use (the call
 * may fail, and it stalls the device while it waits for it to go idle).  Here the split-KV scratch is a fixed array
 * inside the library image (about 5 MB on every device that loads the library, until the process ends), so:
 *   - nothing is allocated or freed, by this call or on its behalf;
 *   - work that needs more than 304 scratch slots (splits x kv_heads x head blocks of 8 or 16 query heads) is refused
 *     with a message; nsplit 0 chooses a split count that fits;
 *   - all calls on a device share that one array: calls that overlap in time on a device race with each other, so
 *     keep them on one stream or otherwise serialised; tickets are re-zeroed on `stream` before each launch;
 *   - the first call on each device looks up the array's device address; make that first call before any stream
 *     capture begins;
 *   - a bounded device-side wait that runs out is recorded in a word of the same array (nothing is allocated for it);
 *     silvann_b200_device_status reads and clears that word together with the device's ordinary status word.
 * Operands and results are silvann_b200_decode's.  Returns 0, 1 (refused: shapes, alignment or size) or 2 (the CUDA
 * runtime refused); a one-line reason is written to `message` (may be null) — this entry keeps no error state. */
int silvann_b200_decode_noalloc(void* o, float* res, const void* q, const void* k, const void* v, uint64_t q_heads,
                                uint64_t kv_heads, uint64_t head_dim, uint64_t length, uint32_t nsplit, int dtype,
                                sv_fault* over, void* stream, char* message, uint32_t message_bytes);

/* Two residuals into one, and a residual into 16-bit output — attention_merge / attention_finish with a dtype. */
int silvann_b200_merge(float* into, const float* a, const float* b, uint64_t q_heads, uint64_t head_dim, void* stream);
int silvann_b200_finish(void* o, const float* res, uint64_t q_heads, uint64_t head_dim, int dtype, sv_fault* over, void* stream);

/* Batched decode over a paged KV pool.  The pool is [pages][page_positions][kv_heads][head_dim] for K and the same
 * for V; sequence s owns pages page_table[s][0 .. ceil(len_s / page_positions)) in order.  A plan turns the host's
 * view of the sequence lengths into a balanced device work list (and owns the split scratch), once per decoding step;
 * every layer of that step then calls silvann_b200_paged_decode with it.  page_positions must be a multiple of 64. */
typedef struct silvann_b200_plan silvann_b200_plan;
int silvann_b200_plan_create(silvann_b200_plan** plan);
int silvann_b200_plan_destroy(silvann_b200_plan* plan);
/* seq_lens is a HOST array; the call copies what it needs before it returns (it waits for `stream` when it has to
 * grow its buffers).  blocks_target 0 = a few waves of the device's SMs. */
int silvann_b200_plan_decode(silvann_b200_plan* plan, const int32_t* seq_lens, uint32_t seqs, uint32_t q_heads,
                             uint32_t kv_heads, uint32_t head_dim, uint32_t blocks_target, void* stream);
/* What the last plan_decode produced: thread blocks, scratch slots, and the positions summed over sequences. */
int silvann_b200_plan_info(const silvann_b200_plan* plan, uint32_t* blocks, uint32_t* slots, uint64_t* positions);
/* q, o [seqs][q_heads][head_dim]; res [seqs][q_heads][head_dim + 2] or null; page_table is a DEVICE array
 * [seqs][table_stride] of int32 page numbers; columns past a sequence's last page may hold anything (-1 by custom)
 * and are never read.  Refused when the longest planned sequence needs more columns than table_stride.  An entry
 * inside a sequence's length that names no page of the pool is never used as an address: its positions read as zeros
 * and SILVANN_B200_STATUS_BAD_PAGE is raised in the device status word. */
int silvann_b200_paged_decode(silvann_b200_plan* plan, void* o, float* res, const void* q, const void* k_pool,
                              const void* v_pool, uint64_t pool_pages, uint32_t page_positions,
                              const int32_t* page_table, uint32_t table_stride, int dtype, sv_fault* over, void* stream);

/* Writes each sequence's newest K and V row into its place in the pools: sequence s's row goes to position
 * len_s - 1 (the lengths of the last plan_decode), i.e. page page_table[s][(len_s-1) / page_positions].  k_rows and
 * v_rows are DEVICE arrays [seqs][kv_heads][head_dim] of 16-bit elements.  This is the pool-side half of what the
 * engine's mixer does when it projects k and v "straight into the cache row" (ai_qwen_3 mixer__abi.cuh:229-239).
 * Refused like paged_decode when the table's rows are too short for the plan; a sequence whose entry names no page of
 * the pool (< 0 or >= pool_pages) is skipped and SILVANN_B200_STATUS_BAD_PAGE is raised in the device status word. */
int silvann_b200_paged_append(silvann_b200_plan* plan, void* k_pool, void* v_pool, const void* k_rows, const void* v_rows,
                              uint64_t pool_pages, uint32_t page_positions, const int32_t* page_table, uint32_t table_stride,
                              void* stream);

/* One query position over a two-tier cache: the oldest host_len positions in pinned host RAM (k_host, v_host are HOST
 * addresses of [host_len][kv_heads][head_dim] planes), the next dev_len positions on the card.  The reference has no
 * host tier; its tiered mixer attends each on-card tier into a residual and merges them (ai_qwen_3 mixer__abi.cuh:383-412),
 * and this does the same with one more tier: host chunks of `chunk_positions` are copied by cudaMemcpyAsync on a side
 * stream into a ring of `stages` staging buffers while `stream` attends the previous chunk; the card tier is attended
 * first.  o [q_heads][head_dim] and/or res [q_heads][head_dim + 2] (the merged residual, for a further merge across
 * devices).  The tier object owns the staging ring (2 * stages * chunk_positions * kv_heads * head_dim * 2 bytes);
 * chunk_positions 0 lets the library size a chunk in bytes (8 MB a plane), which keeps the host link busy at any row
 * width.  With no host positions the decode kernel writes the answer itself: one launch. */
typedef struct silvann_b200_tier silvann_b200_tier;
int silvann_b200_tier_create(silvann_b200_tier** tier, uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim, int dtype,
                             uint32_t chunk_positions, uint32_t stages);
int silvann_b200_tier_destroy(silvann_b200_tier* tier);
int silvann_b200_tier_decode(silvann_b200_tier* tier, void* o, float* res, const void* q, const void* k_host, const void* v_host,
                             uint64_t host_len, const void* k_dev, const void* v_dev, uint64_t dev_len, sv_fault* over, void* stream);
/* Bytes copied host to device and chunks staged since the tier was created. */
int silvann_b200_tier_stats(const silvann_b200_tier* tier, uint64_t* h2d_bytes, uint64_t* chunks);

/* The exchange step of a sharded path among up to 8 cards of one box, as one kernel a card over peer memory.
 *
 * It replaces the reference's in-process collective — a `vector_sum` kernel that loads the other cards' partials in place
 * after host-side marks (engine/src/silicon_families/nvidia_cuda12/overrides/vector.cuh:292-331, driven by
 * nn__partials__reduce_onto, engine/src/packages/nn/cpu/opcodes/partials__abi.cuh:110-163, with its bounded patience
 * :42-56) — and carries the residual fold of a KV range split over cards (attention_merge + attention_finish,
 * engine/src/packages/nn/gpu/kernels/kernels.cuh:1243-1267).  A member PUSHES its piece into a slot of every member's
 * buffer with plain stores, publishes a generation number beside it, waits (at most wait_ms, 0 = one second) for every
 * member's number, then combines from its own memory in member order — so every member computes the same bits.
 *
 * An exchange object is one member's end: `members` cards, this one is `index` (the order of the fold / the sum);
 * slot_bytes is the largest piece a member will push.  create allocates the member's buffer on the bound device.  The
 * members then learn each other's buffers once: between processes (a process a card) each passes the 64-byte handle of
 * exchange_handle to the others by any means and calls connect_handles with all members' handles in member order (its own
 * entry is ignored); inside one process (the engine's model: a worker thread a card, peer_access granted) each calls
 * connect_addresses with the addresses exchange_local answers.  After that every member calls the same exchange entry
 * points in the same order.  A wait that runs out raises "B2TO" in the device status word and leaves the outputs
 * unwritten; the object stays usable. */
typedef struct silvann_b200_exchange silvann_b200_exchange;
#define SILVANN_B200_EXCHANGE_HANDLE_BYTES 64u
int silvann_b200_exchange_create(silvann_b200_exchange** exchange, uint32_t members, uint32_t index, uint64_t slot_bytes);
int silvann_b200_exchange_destroy(silvann_b200_exchange* exchange);
int silvann_b200_exchange_local(const silvann_b200_exchange* exchange, uint64_t* address, uint64_t* bytes);
int silvann_b200_exchange_handle(const silvann_b200_exchange* exchange, void* handle, uint32_t handle_bytes);
int silvann_b200_exchange_connect_handles(silvann_b200_exchange* exchange, const void* handles, uint32_t handle_bytes);
int silvann_b200_exchange_connect_addresses(silvann_b200_exchange* exchange, const uint64_t* addresses);
/* res_local [q_heads][head_dim + 2] is this member's residual of its range; o [q_heads][head_dim] and/or res receive the
 * whole range's answer: ((r_0 + r_1) + r_2) + ... with attention_merge's arithmetic, then attention_finish's. */
int silvann_b200_exchange_merge_finish(silvann_b200_exchange* exchange, void* o, float* res, const float* res_local, uint64_t q_heads,
                                       uint64_t head_dim, int dtype, sv_fault* over, uint32_t wait_ms, void* stream);
/* out[i] = round16(sum over members, in member order, of fp32(partial_member[i])) — vector_sum (kernels.cuh:117-126). */
int silvann_b200_exchange_vector_sum(silvann_b200_exchange* exchange, void* out, const void* partial, uint64_t n, int dtype,
                                     sv_fault* over, uint32_t wait_ms, void* stream);
/* The output projection of a head-sharded mixer and the sum over the cards that follows it, in one launch a card: `codes`
 * [rows][cols·width/8] and `scales` [rows] are this card's share of a TurboQuant-coded matrix (width 4 or 8; turboquant_gemv's
 * operands, kernels.cuh:1405-1447), vec [cols] its share of the input; every member's 16-bit partial out_m[r] is pushed from
 * the kernel's epilogue and out[r] = round16(sum over members, in member order, of fp32(out_m[r])) — what turboquant_gemv
 * followed by nn__partials__reduce_onto leaves (nn partials__abi.cuh:110-163).  fp16; rows * 2 bytes must fit a slot. */
int silvann_b200_exchange_gemv_sum(silvann_b200_exchange* exchange, void* out, const void* codes, const void* scales, const void* vec,
                                   uint64_t width, uint64_t rows, uint64_t cols, sv_fault* over, uint32_t wait_ms, void* stream);
/* Stands in for an absent member where there are fewer cards than members (a one-card walk of a many-card plan): puts
 * `data` where that member's push of the NEXT exchange would land, in the form that exchange moves it: `unit_bytes` 4 for a
 * residual (merge_finish) or a 16-bit vector (vector_sum), 2 for the rows of gemv_sum.  Same stream as the exchange. */
int silvann_b200_exchange_deposit(silvann_b200_exchange* exchange, uint32_t member, const void* data, uint64_t bytes, uint32_t unit_bytes, void* stream);
/* silvann_b200_tier_decode for a member of a range split: the member's residual over its two tiers, then the exchange,
 * as one call — and as one launch when every position is on the card and the share is long enough to be split: the decode
 * kernel's last block of a head block does the exchange step itself (the same bits). */
int silvann_b200_tier_decode_exchange(silvann_b200_tier* tier, silvann_b200_exchange* exchange, void* o, float* res, const void* q,
                                      const void* k_host, const void* v_host, uint64_t host_len, const void* k_dev, const void* v_dev,
                                      uint64_t dev_len, sv_fault* over, uint32_t wait_ms, void* stream);

/* Causal grouped-query prefill in one kernel — attention_causal_scores_grouped + attention_causal_softmax +
 * attention_causal_mix (kernels.cuh:1028-1081, 2051-2060): row r is position first + r and attends cache rows
 * 0..first+r.  q, o [rows][q_heads][head_dim]; k, v [first + rows][kv_heads][head_dim].  With `res` (may be null, as may
 * `o`, not both) every row's heads also leave their residual (m, l, acc) at res + row·q_heads·(head_dim + 2), the
 * answer of attention_weights_rows + attention_residual_mix_rows (nn/gpu/doors.cuh:406-431) for a later merge. */
int silvann_b200_prefill(void* o, float* res, const void* q, const void* k, const void* v, uint64_t q_heads, uint64_t kv_heads,
                         uint64_t head_dim, uint64_t first, uint64_t rows, int dtype, sv_fault* over, void* stream);

/* One query position of latent attention in one pass — attention_scores_grouped + attention_softmax_rows + attention_mix
 * when the keys and the values are the SAME rows (kernels.cuh:931-950, 1085-1100, 1144-1164; the sequence GLM's decode runs,
 * ai_z__glm_5_3 layer__abi.cuh:279-289): `heads` (32 or 64) query heads over one kv head whose rows are `latent_dim` (512)
 * wide.  q [heads][512]; latent [length][512]; o [heads][512] 16-bit and/or res [heads][514] fp32 (m, l, acc).  blocks 0 lets
 * the library cut the positions over the card's SMs; with more than one block the blocks' partial residuals meet in scratch
 * the library keeps a device (allocated on first use) and a second small kernel folds them. */
int silvann_b200_mla_decode(void* o, float* res, const void* q, const void* latent, uint64_t heads, uint64_t latent_dim,
                            uint64_t length, uint32_t blocks, int dtype, sv_fault* over, void* stream);

/* Gated DeltaNet over `rows` positions of `seqs` independent sequences (deltanet_steps_gate, kernels.cuh:650-718,
 * 2131-2165, with a dtype and a batch).  S [seqs][v_heads][d][d] fp32 in place; conved [seqs][rows][(2·k_heads +
 * v_heads)·d]; z, out [seqs][rows][v_heads·d]; beta, g [seqs][rows][v_heads]; w [d].  `readout` (may be null) receives
 * [seqs][rows][v_heads·d] fp32: every position's read-out S^T qs as summed, before the first of the two roundings to
 * 16 bits the door applies (kernels.cuh:677-688) — what a caller compares when it wants the recurrence's own error
 * rather than the rounding's. */
int silvann_b200_deltanet(float* S, const void* conved, const void* z, const void* beta, const void* g, const void* w,
                          void* out, float* readout, uint64_t k_heads, uint64_t v_heads, uint64_t head_dim, uint64_t rows,
                          uint32_t seqs, uint32_t gate, int dtype, sv_fault* over, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SILVANN_B200_H */
