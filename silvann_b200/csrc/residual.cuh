/* residual.cuh — the arithmetic of attention_merge on one head (engine/src/packages/nn/gpu/kernels/kernels.cuh:1243-1255),
 * written once so that every kernel that folds residuals — the merge door, the exchange kernel — rounds identically:
 * with m = max(m_a, m_b), f_a = e^(m_a - m), f_b = e^(m_b - m):  l = l_a f_a + l_b f_b,  acc = acc_a f_a + acc_b f_b.
 * The sum of two products is fixed as one multiply and one fused multiply-add, so the compiler has no choice to make. */
#pragma once
#include <cuda_runtime.h>

namespace sv {

__device__ __forceinline__ float merge_element(float a, float fa, float b, float fb) { return __fmaf_rn(a, fa, __fmul_rn(b, fb)); }

/* (m, l) <- merged with (mb, lb); answers the two factors for the head's elements. */
__device__ __forceinline__ void merge_scalars(float& m, float& l, float mb, float lb, float& fa, float& fb) {
    const float top = m > mb ? m : mb;
    fa = expf(m - top); fb = expf(mb - top);
    l = merge_element(l, fa, lb, fb);
    m = top;
}

}  // namespace sv
