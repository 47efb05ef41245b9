"""The expert-major GEMM doors — expert_rows, expert_rows_sum, expert_groups, expert_rows_finish, expert_rows_reduce,
expert_pairs_rows, expert_multiply_fp16(_rows) — on a B200 against the reference's CPU family run on the host
(engine/src/packages/nn/gpu/kernels/kernels.cuh:1513-1692, 3864-3871): the same codes, scales, rows of x and pairs through
both.  Every product level x value is exact in fp32 in both, so the two differ by the order of an fp32 sum and by one
rounding to fp16: the bar is one fp16 step, nearly everywhere zero.  Shapes the tcgen05 kernel takes and shapes only the
as-worded kernel takes are both here; the counter says which ran."""
import numpy as np
import pytest

import oracle
from oracle import from_bits, to_bits
from silvann_b200 import ext
from util import OnCard

pytestmark = pytest.mark.gpu
FP16 = 0


def coded(reference, rng, rows, cols, d):
    w = to_bits((rng.standard_normal((rows, cols)) / np.sqrt(cols)).astype(np.float32), FP16)
    if d == 16:
        return w.view(np.uint8).reshape(rows, cols * 2).copy(), None
    return oracle.tq_encode_rows(reference, w, d)


def pairs_of(rng, count, x_rows, out_rows_n):
    """`count` pairs: x rows drawn with repeats, out rows distinct and shuffled."""
    p = np.empty((count, 2), np.uint32)
    p[:, 0] = rng.integers(0, x_rows, count)
    p[:, 1] = rng.permutation(out_rows_n)[:count]
    return p


def steps_apart(got, want):
    """fp16 steps between two arrays of bit patterns (sign-magnitude -> a line)."""
    line = lambda b: np.where(b & 0x8000, -(b & 0x7FFF).astype(np.int32), (b & 0x7FFF).astype(np.int32))
    return np.abs(line(got) - line(want))


def close(got, want, what):
    """At most one fp16 step apart — or, near zero where a step is smaller than an fp32 sum's own noise, 2e-5 — and nearly
    everywhere the same bits."""
    s = steps_apart(got, want)
    err = np.abs(from_bits(got, FP16) - from_bits(want, FP16))
    bad = (s > 1) & (err > 2e-5)
    assert np.isfinite(from_bits(got, FP16)).all(), f"{what}: non-finite"
    assert not bad.any(), f"{what}: {int(bad.sum())} values more than one fp16 step from the reference (worst {int(s.max())} steps, {err.max():.3e})"
    assert (s == 0).mean() > 0.9, f"{what}: only {(s == 0).mean():.3f} of the values are the reference's bits"


@pytest.mark.parametrize("d,out_rows,cols,count,fast", [
    (4, 256, 512, 16, True), (8, 256, 512, 16, True), (16, 256, 512, 16, True),
    (4, 384, 1024, 100, True), (8, 1000, 2048, 256, True), (4, 128, 64, 1, True), (8, 200, 192, 130, True), (16, 130, 320, 37, True),
    (4, 1024, 5120, 256, True), (8, 512, 4096, 200, True),
    (3, 96, 256, 9, False), (5, 64, 200, 5, False), (4, 100, 40, 11, False), (2, 33, 512, 20, False),
])
def test_expert_rows(cuda, fam, reference, d, out_rows, cols, count, fast):
    rng = np.random.default_rng(d * 1000 + out_rows + count)
    codes, luts = coded(reference, rng, out_rows, cols, d)
    x_rows, out_n = max(count, 7) + 3, count + 5
    x = to_bits(rng.standard_normal((x_rows, cols)).astype(np.float32), FP16)
    pairs = pairs_of(rng, count, x_rows, out_n)
    want = np.full((out_n, out_rows), 0x1234, np.uint16)
    oracle.expert_rows(reference, want, codes, luts, x, pairs, count, d, out_rows, cols)
    got = np.full((out_n, out_rows), 0x1234, np.uint16)
    before = ext.counters()
    oracle.expert_rows(OnCard(cuda, fam), got, codes, luts, x, pairs, count, d, out_rows, cols)
    after = ext.counters()
    assert after["refused"] == before["refused"] and ext.device_status() == 0
    assert (after["expert_fast"] - before["expert_fast"] == 1) == fast, "which kernel answered"
    untouched = np.ones(out_n, bool); untouched[pairs[:, 1]] = False
    assert (got[untouched] == 0x1234).all(), "a row no pair names was written"
    close(got, want, f"expert_rows d={d} {out_rows}x{cols} pairs={count}")


@pytest.mark.parametrize("d,held", [(4, 100), (8, 129), (16, 1)])
def test_rows_the_rooms_do_not_hold_are_left_alone(cuda, fam, reference, d, held):
    rng = np.random.default_rng(d + held)
    out_rows, cols, count = 256, 256, 20
    codes, luts = coded(reference, rng, out_rows, cols, d)
    x = to_bits(rng.standard_normal((count, cols)).astype(np.float32), FP16)
    pairs = pairs_of(rng, count, count, count)
    row_bytes = oracle.tq_row_bytes(d, cols) if d != 16 else cols * 2
    want = np.full((count, out_rows), 0x1234, np.uint16)
    oracle.expert_rows(reference, want, codes, luts, x, pairs, count, d, out_rows, cols, w_room=held * row_bytes)
    got = np.full((count, out_rows), 0x1234, np.uint16)
    oracle.expert_rows(OnCard(cuda, fam), got, codes, luts, x, pairs, count, d, out_rows, cols, w_room=held * row_bytes)
    assert (got[:, held:] == 0x1234).all() and (want[:, held:] == 0x1234).all()
    close(got[:, :held], want[:, :held], "held rows")
    assert ext.device_status() == 0


def test_expert_groups_like_a_layers_q_and_k(cuda, fam, reference):
    """Two matrices of different widths and heights over the same pairs, their outputs one after the other — and a third over
    a different run of pairs — in one launch."""
    rng = np.random.default_rng(77)
    cols, T = 1024, 150
    q_rows, k_rows, v_rows = 768, 256, 200
    qc, ql = coded(reference, rng, q_rows, cols, 4)
    kc, kl = coded(reference, rng, k_rows, cols, 8)
    vc, vl = coded(reference, rng, v_rows, cols, 4)
    x = to_bits(rng.standard_normal((T, cols)).astype(np.float32), FP16)
    pairs = np.concatenate([np.stack([np.arange(T), np.arange(T)], 1), np.stack([np.arange(40)[::-1], np.arange(40)], 1)]).astype(np.uint32)
    groups = lambda: [(qc, ql, q_rows, 4, 0, 0, T), (kc, kl, k_rows, 8, T * q_rows, 0, T), (vc, vl, v_rows, 4, T * (q_rows + k_rows), T, 40)]
    n = T * (q_rows + k_rows) + 40 * v_rows
    want = np.zeros(n, np.uint16)
    oracle.expert_groups(reference, want, groups(), x, pairs, cols)
    got = np.zeros(n, np.uint16)
    before = ext.counters()
    oracle.expert_groups(OnCard(cuda, fam), got, groups(), x, pairs, cols)
    after = ext.counters()
    assert after["expert_fast"] - before["expert_fast"] == 1 and after["refused"] == before["refused"] and ext.device_status() == 0
    close(got, want, "expert_groups")


@pytest.mark.parametrize("d,cols,fast", [(4, 512, True), (8, 200, False)])
def test_rows_sum_then_finish_and_reduce(cuda, fam, reference, d, cols, fast):
    """The MoE's down: an expert's picks weighted onto a running fp32 sum, rounded once by rows_finish; and rows_reduce over
    per-pick slots."""
    rng = np.random.default_rng(d + cols)
    out_rows, count, T = 192, 24, 30
    codes, luts = coded(reference, rng, out_rows, cols, d)
    x = to_bits(rng.standard_normal((T, cols)).astype(np.float32), FP16)
    w = to_bits(rng.uniform(0.1, 1.0, T).astype(np.float32), FP16)
    pairs = pairs_of(rng, count, T, T)
    start = rng.standard_normal((T, out_rows)).astype(np.float32)
    residual = to_bits(rng.standard_normal((T, out_rows)).astype(np.float32), FP16)
    outs = []
    for impl in (reference, OnCard(cuda, fam)):
        P = getattr(impl, "ptr", oracle._p)
        acc = start.copy()
        oracle.expert_rows_sum(impl, acc, codes, luts, x, pairs, w, count, d, out_rows, cols)
        summed = acc.copy()
        out = np.zeros((T, out_rows), np.uint16)
        over = np.zeros(4, np.uint32)
        impl.nn.expert_rows_finish(P(out), P(acc), P(residual), T * out_rows, P(over))
        impl.wait()
        assert not acc.any(), "rows_finish leaves the sum at zero"
        k = 3
        acc3 = rng.standard_normal((T // k, k, out_rows)).astype(np.float32) if impl is reference else outs[0][3].copy()
        slots = acc3.copy()
        red = np.zeros((T // k, out_rows), np.uint16)
        impl.nn.expert_rows_reduce(P(red), P(slots), P(residual), T // k, k, out_rows, P(over))
        impl.wait()
        assert not slots.any()
        outs.append((summed, out, red, acc3))
    np.testing.assert_allclose(outs[1][0], outs[0][0], rtol=2e-5, atol=2e-5)
    close(outs[1][1], outs[0][1], "rows_finish")
    assert np.array_equal(outs[1][2], outs[0][2]), "rows_reduce adds the picks in their order: the same bits"


def test_pairs_rows_and_the_16_bit_multiplies(cuda, fam, reference):
    rng = np.random.default_rng(5)
    for impl in (reference, OnCard(cuda, fam)):
        P = getattr(impl, "ptr", oracle._p)
        pairs = np.zeros((37, 2), np.uint32)
        impl.nn.expert_pairs_rows(P(pairs), 37, 2, 5, 3, 1)
        impl.wait()
        assert np.array_equal(pairs[:, 0], 2 * np.arange(37) + 5) and np.array_equal(pairs[:, 1], 3 * np.arange(37) + 1)
    rows, cols, n = 96, 320, 5
    W = to_bits((rng.standard_normal((rows, cols)) / np.sqrt(cols)).astype(np.float32), FP16)
    x = to_bits(rng.standard_normal((n, cols)).astype(np.float32), FP16)
    outs = []
    for impl in (reference, OnCard(cuda, fam)):
        P = getattr(impl, "ptr", oracle._p)
        over = np.zeros(4, np.uint32)
        one = np.zeros(rows, np.uint16)
        many = np.zeros((n, rows), np.uint16)
        impl.nn.expert_multiply_fp16(P(one), P(W), P(x), rows, cols, P(over))
        impl.nn.expert_multiply_fp16_rows(P(many), P(W), P(x), rows, cols, n, P(over))
        impl.wait()
        outs.append((one, many))
    close(outs[1][0], outs[0][0], "multiply_fp16")
    close(outs[1][1], outs[0][1], "multiply_fp16_rows")
    assert np.array_equal(outs[1][0], outs[1][1][0]), "the rows door's first row is the one-row door's answer"


def test_empty_calls_write_nothing_and_an_unknown_width_is_refused(cuda, fam, reference):
    rng = np.random.default_rng(3)
    codes, luts = coded(reference, rng, 64, 128, 4)
    x = cuda.from_numpy(rng.standard_normal((4, 128)).astype(np.float16).view(np.int16)).cuda()
    pairs = cuda.from_numpy(np.array([[0, 0], [1, 1]], np.int32)).cuda()
    tc = cuda.from_numpy(codes.copy()).cuda()
    tl = cuda.from_numpy(luts.view(np.int16).copy()).cuda()
    out = cuda.full((2, 64), 0x1234, dtype=cuda.int16, device="cuda")
    before = ext.counters()
    fam.nn.expert_rows(out.data_ptr(), tc.data_ptr(), codes.nbytes, tl.data_ptr(), luts.nbytes, x.data_ptr(), pairs.data_ptr(), 0, 4, 64, 128, None)     # no pairs
    fam.nn.expert_rows(out.data_ptr(), tc.data_ptr(), 0, tl.data_ptr(), luts.nbytes, x.data_ptr(), pairs.data_ptr(), 2, 4, 64, 128, None)                # rooms that hold no row
    assert fam.sys.compute_completed()
    assert (out == 0x1234).all() and ext.counters()["launches"] == before["launches"]
    fam.nn.expert_rows(out.data_ptr(), tc.data_ptr(), codes.nbytes, tl.data_ptr(), luts.nbytes, x.data_ptr(), pairs.data_ptr(), 2, 7, 64, 128, None)     # no such width
    assert not fam.sys.compute_completed(), "a refused door makes the next wait answer false once"
    assert fam.sys.compute_completed()
    assert (out == 0x1234).all() and ext.counters()["refused"] == before["refused"] + 1
