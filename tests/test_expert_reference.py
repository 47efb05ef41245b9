"""The checker's expert-major GEMM helpers, pinned on the CPU: the reference's x86_avx2 family called through
oracle.expert_rows / expert_groups / expert_rows_sum must equal numpy's product of the decoded matrix and the named rows of
x (engine/src/packages/nn/gpu/kernels/kernels.cuh:1513-1660) — so that the GPU tests, which compare this library with those
helpers, compare it with the definition."""
import numpy as np
import pytest

import oracle
from oracle import from_bits, to_bits

FP16 = 0


def decoded(reference, codes, luts, d, rows, cols):
    if d == 16:
        return from_bits(codes.view(np.uint16).reshape(rows, cols), FP16).astype(np.float64)
    levels = from_bits(oracle.tq_decode(reference, codes, np.full(rows, 0x3C00, np.uint16).view(np.uint8).copy(), d, rows, cols), FP16).astype(np.float64)
    return levels * from_bits(luts, FP16).astype(np.float64)[:, None]


@pytest.mark.parametrize("d,out_rows,cols,count", [(4, 96, 256, 11), (8, 64, 192, 5), (16, 40, 128, 9), (3, 33, 96, 4)])
def test_reference_expert_rows_is_the_definition(reference, d, out_rows, cols, count):
    if reference is None:
        pytest.skip("the reference family is not built here")
    rng = np.random.default_rng(d + count)
    w = to_bits((rng.standard_normal((out_rows, cols)) / np.sqrt(cols)).astype(np.float32), FP16)
    codes, luts = (w.view(np.uint8).reshape(out_rows, cols * 2).copy(), None) if d == 16 else oracle.tq_encode_rows(reference, w, d)
    x = to_bits(rng.standard_normal((count + 2, cols)).astype(np.float32), FP16)
    pairs = np.stack([rng.integers(0, count + 2, count), rng.permutation(count + 3)[:count]], 1).astype(np.uint32)
    out = np.full((count + 3, out_rows), 0x1234, np.uint16)
    oracle.expert_rows(reference, out, codes, luts, x, pairs, count, d, out_rows, cols)
    W, X = decoded(reference, codes, luts, d, out_rows, cols), from_bits(x, FP16).astype(np.float64)
    named = np.zeros(count + 3, bool)
    for j in range(count):
        want = W @ X[pairs[j, 0]]
        got = from_bits(out[pairs[j, 1]], FP16)
        assert np.abs(got - want).max() <= 2e-3 * max(1.0, np.abs(want).max()), f"pair {j}"
        named[pairs[j, 1]] = True
    assert (out[~named] == 0x1234).all()
    # the groups door over the same matrix is the same answer; the running sum adds weight x value
    again = np.zeros((count + 3) * out_rows, np.uint16)
    oracle.expert_groups(reference, again, [(codes, luts, out_rows, d, 0, 0, count)], x, pairs, cols)
    assert np.array_equal(again.reshape(count + 3, out_rows)[named], out[named])
    wts = to_bits(rng.uniform(0.2, 1.0, count + 2).astype(np.float32), FP16)
    acc = np.ones((count + 3, out_rows), np.float32)
    oracle.expert_rows_sum(reference, acc, codes, luts, x, pairs, wts, count, d, out_rows, cols)
    for j in range(count):
        want = 1.0 + from_bits(wts, FP16)[pairs[j, 0]] * (W @ X[pairs[j, 0]])
        assert np.abs(acc[pairs[j, 1]] - want).max() <= 2e-3 * max(1.0, np.abs(want).max())
