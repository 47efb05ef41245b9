/* kernels_deltanet.h — launcher of the Gated DeltaNet kernels (deltanet.cu). */
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace sv {

/* `seqs` independent sequences, each with its own state and `rows` positions.  Sequence b's operands follow
 * sequence b-1's contiguously: S [seqs][v_heads][d][d] fp32; conved [seqs][rows][(2·k_heads + v_heads)·d] (query
 * heads, key heads, value heads); z and out [seqs][rows][v_heads·d]; beta and g [seqs][rows][v_heads]; w [d]. */
struct DeltaCall {
    float* S;
    const uint16_t *conved, *z, *beta, *g, *w;
    uint16_t* out;
    float* readout;      /* null, or [seqs][rows][v_heads·d] fp32: S^T qs of every position before its first rounding to 16 bits */
    uint32_t k_heads, v_heads, head_dim, seqs;
    uint64_t rows;
    int gate;      /* 0 silu(z), 1 sigmoid(z) */
    int dtype;     /* SV_DTYPE_* of every 16-bit operand */
    unsigned int* over;
    cudaStream_t stream;
};
bool deltanet_fits(const DeltaCall& c);
/* the 64-position chunked form (deltanet_chunked.cu): runs of at least 32 positions at head_dim 64 or 128 */
bool deltanet_chunked_fits(const DeltaCall& c);
size_t deltanet_chunked_scratch_floats(const DeltaCall& c);
cudaError_t deltanet_chunked_launch(const DeltaCall& c, float* ss, float* prep);
/* the read-out's norm and gate over what either form left in `out` and `ss` (deltanet.cu) */
cudaError_t deltanet_norm_launch(const DeltaCall& c, const float* ss);
cudaError_t deltanet_launch(const DeltaCall& c);

}  // namespace sv
