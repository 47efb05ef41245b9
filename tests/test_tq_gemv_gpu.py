"""A TurboQuant-coded matrix times up to eight vectors on a B200 — the tensor-core kernel that answers turboquant_gemv,
turboquant_gemv_groups and turboquant_gemv_groups_n at the shapes it takes — against the restatement of the reference's
door (pinned to the reference's CPU family by tests/test_oracle.py), a row its rooms do not hold left alone."""
import numpy as np
import pytest

import oracle
from oracle import FP16, from_bits, to_bits
from silvann_b200 import ext
from silvann_b200.abi import TqGroups
from util import dev, host_bits

pytestmark = pytest.mark.gpu


def coded(port, rng, rows, cols, d):
    w = to_bits((rng.standard_normal((rows, cols)) / np.sqrt(cols)).astype(np.float32), FP16)
    return oracle.tq_encode_rows(port, w, d)


def near(got, want, what):
    """within one fp16 step of the restatement, or 2e-3 where a step is smaller than that: the sums differ in order"""
    g, w = from_bits(got, FP16), from_bits(want, FP16)
    steps = np.abs(got.astype(np.int32) - want.astype(np.int32))
    bad = (steps > 1) & (np.abs(g - w) > 1e-3)
    assert not bad.any(), f"{what}: {int(bad.sum())} outputs off, worst {np.abs(g - w).max():.3e}"


@pytest.mark.parametrize("d,rows,cols", [(4, 1000, 2048), (8, 513, 4096), (4, 37, 4096), (8, 2048, 2048), (4, 16, 128), (8, 5, 64), (4, 4096, 8192)])
def test_one_matrix(cuda, fam, port, d, rows, cols):
    rng = np.random.default_rng(300 + d + rows)
    codes, scales = coded(port, rng, rows, cols, d)
    x = to_bits(rng.standard_normal(cols).astype(np.float32), FP16)
    want = oracle.tq_gemv(port, codes, scales.view(np.uint8).copy(), x, d, rows, cols)
    tc, ts, tx = dev(cuda, codes), dev(cuda, scales), dev(cuda, x)
    out = cuda.full((rows,), 0x1234, dtype=cuda.int16, device="cuda")
    before = ext.counters()
    fam.nn.turboquant_gemv(out.data_ptr(), tc.data_ptr(), codes.nbytes, ts.data_ptr(), scales.nbytes, tx.data_ptr(), d, rows, cols, None)
    assert fam.sys.compute_completed()
    after = ext.counters()
    assert after["gemv_fast"] - before["gemv_fast"] == 1 and ext.device_status() == 0
    near(host_bits(out), want, f"{rows} x {cols} at {d} bits")
    # rooms that hold fewer rows than named: the rows past them keep what they held
    if rows > 20:
        out2 = cuda.full((rows,), 0x1234, dtype=cuda.int16, device="cuda")
        fam.nn.turboquant_gemv(out2.data_ptr(), tc.data_ptr(), (rows - 3) * codes.shape[1], ts.data_ptr(), (rows - 7) * 2, tx.data_ptr(), d, rows, cols, None)
        assert fam.sys.compute_completed()
        got = host_bits(out2)
        near(got[: rows - 7], want[: rows - 7], "short rooms")
        assert (got[rows - 7:] == 0x1234).all()


@pytest.mark.parametrize("n,stride", [(1, 0), (3, 0), (8, 0), (4, 5000), (2, 3000)])
def test_groups_over_n_inputs(cuda, fam, port, n, stride):
    """Four matrices of two widths over n inputs in one launch — a DeltaNet mixer's projections for a draft's rows."""
    cols = 2048
    rng = np.random.default_rng(400 + n)
    shapes = [(1100, 4), (512, 8), (33, 8), (32, 4)]
    mats = [coded(port, rng, r, cols, d) for r, d in shapes]
    x = to_bits(rng.standard_normal((n, cols)).astype(np.float32), FP16)
    tx = dev(cuda, x)
    held = [(dev(cuda, c), dev(cuda, s)) for c, s in mats]
    g = TqGroups()
    placed = 0
    for i, ((r, d), (tc, ts)) in enumerate(zip(shapes, held)):
        g.codes[i], g.luts[i], g.rows[i], g.d[i], g.out_at[i] = tc.data_ptr(), ts.data_ptr(), r, d, placed
        placed += r * (n if stride == 0 else 1)
    g.count = len(shapes)
    total = placed if stride == 0 else n * stride
    out = cuda.full((total,), 0x1234, dtype=cuda.int16, device="cuda")
    before = ext.counters()
    if n == 1 and stride == 0:
        fam.nn.turboquant_gemv_groups(out.data_ptr(), g, tx.data_ptr(), cols, None)
    else:
        fam.nn.turboquant_gemv_groups_n(out.data_ptr(), g, tx.data_ptr(), cols, n, stride, None)
    assert fam.sys.compute_completed()
    assert ext.counters()["gemv_fast"] - before["gemv_fast"] == 1 and ext.device_status() == 0
    got = host_bits(out)
    seen = np.zeros(total, bool)
    for i, ((r, d), (codes, scales)) in enumerate(zip(shapes, mats)):
        for k in range(n):
            want = oracle.tq_gemv(port, codes, scales.view(np.uint8).copy(), x[k].copy(), d, r, cols)
            at = int(g.out_at[i]) + (k * stride if stride else k * r)
            near(got[at: at + r], want, f"group {i}, input {k}")
            seen[at: at + r] = True
    assert (got[~seen] == 0x1234).all(), "nothing outside the groups' answers was written"


def test_shapes_the_fast_kernel_leaves_to_the_worded_one(cuda, fam, port):
    rng = np.random.default_rng(500)
    for d, rows, cols in ((5, 40, 256), (4, 40, 200), (8, 9, 100)):
        codes, scales = coded(port, rng, rows, cols, d) if d != 5 else (
            rng.integers(0, 256, (rows, oracle.tq_row_bytes(5, cols)), dtype=np.uint8), to_bits(rng.uniform(0.01, 0.1, rows).astype(np.float32), FP16))
        x = to_bits(rng.standard_normal(cols).astype(np.float32), FP16)
        want = oracle.tq_gemv(port, codes, scales.view(np.uint8).copy(), x, d, rows, cols)
        tc, ts, tx = dev(cuda, codes), dev(cuda, scales), dev(cuda, x)
        out = cuda.zeros(rows, dtype=cuda.int16, device="cuda")
        before = ext.counters()
        fam.nn.turboquant_gemv(out.data_ptr(), tc.data_ptr(), codes.nbytes, ts.data_ptr(), scales.nbytes, tx.data_ptr(), d, rows, cols, None)
        assert fam.sys.compute_completed()
        assert ext.counters()["gemv_fast"] == before["gemv_fast"]
        near(host_bits(out), want, f"{rows} x {cols} at {d} bits, as worded")
