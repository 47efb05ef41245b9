"""Causal GQA prefill on a B200: the fused tcgen05 kernel through the extension and through the three causal doors the
engine's verbs call, against the reference's CPU family / the C restatement.  Bars: 16-bit outputs within 2e-3 (or half
an output ulp more where bf16's ulp is larger); exact structural properties at the benchmark's full size."""
import numpy as np
import pytest

import oracle
from oracle import from_bits, to_bits
from silvann_b200 import ext, verbs, workloads
from util import assert_close16, dev, host_bits

pytestmark = pytest.mark.gpu


def case(seed, qh, kvh, d, first, rows, dtype, scale=0.5):
    rng = np.random.default_rng(seed)
    mk = lambda s: to_bits(oracle.fp16_exact_bf16(rng.standard_normal(s, dtype=np.float32) * scale), dtype)
    return mk((rows, qh, d)), mk((first + rows, kvh, d)), mk((first + rows, kvh, d))


SHAPES = [  # qh, kvh, d, first, rows
    (4, 2, 64, 0, 128), (4, 2, 64, 0, 100), (8, 2, 128, 0, 300), (2, 1, 256, 0, 257), (16, 2, 256, 0, 384),
    (4, 1, 128, 70, 200), (2, 2, 256, 333, 64), (3, 1, 64, 5, 1),
]


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("qh,kvh,d,first,rows", SHAPES)
def test_ext_prefill_matches_oracle(cuda, port, qh, kvh, d, first, rows, dtype):
    q, k, v = case(rows + d, qh, kvh, d, first, rows, dtype)
    _, want = port.prefill(q, k, v, qh, kvh, d, first, rows, dtype)
    o = cuda.zeros((rows, qh, d), dtype=cuda.int16, device="cuda")
    ext.prefill(o, dev(cuda, q), dev(cuda, k), dev(cuda, v), qh, kvh, d, first, rows, dtype)
    cuda.cuda.synchronize()
    assert ext.device_status() == 0
    assert_close16(host_bits(o), want, dtype, f"prefill {qh}/{kvh} d{d} first{first} rows{rows}")


@pytest.mark.parametrize("tag", ["cau_a", "cau_b"])
def test_golden_rows_through_the_three_doors(cuda, fam, golden, tag):
    qh, kvh, d, first, rows = (int(x) for x in golden[f"{tag}_shape"])
    V = verbs.Verbs(fam)
    tq, tk, tv = (dev(cuda, golden[f"{tag}_{n}"]) for n in "qkv")
    scores = cuda.zeros((rows * qh, first + rows), dtype=cuda.float32, device="cuda")
    out = cuda.zeros((rows, qh, d), dtype=cuda.int16, device="cuda")
    before = ext.counters()["fused_prefill"]
    V.attention_causal_rows(tq, tk, tv, scores, out, qh, kvh, d, first, rows)
    assert fam.sys.compute_completed()
    assert ext.counters()["fused_prefill"] == before + 1
    assert_close16(host_bits(out), from_bits(golden[f"{tag}_o"], 0), 0, tag)


def test_passes_sized_by_the_scores_room_equal_one_pass(cuda, fam, port):
    """The layer verb attends as many rows a pass as its scores buffer holds; every pass is one fused launch."""
    qh, kvh, d, first, rows = 8, 2, 128, 40, 300
    q, k, v = case(1, qh, kvh, d, first, rows, 0)
    _, want = port.prefill(q, k, v, qh, kvh, d, first, rows, 0)
    V = verbs.Verbs(fam)
    tq, tk, tv = dev(cuda, q), dev(cuda, k), dev(cuda, v)
    small = cuda.zeros((qh * (first + rows) * 70,), dtype=cuda.float32, device="cuda")       # room for 70 rows a pass
    out = cuda.zeros((rows, qh, d), dtype=cuda.int16, device="cuda")
    before = ext.counters()["fused_prefill"]
    V.attention_causal_rows(tq, tk, tv, small, out, qh, kvh, d, first, rows)
    assert fam.sys.compute_completed()
    assert ext.counters()["fused_prefill"] == before + 5
    assert_close16(host_bits(out), want, 0, "five passes")


def test_worded_causal_doors_for_an_unfit_head_dim(cuda, fam, port):
    qh, kvh, d, first, rows = 4, 2, 96, 3, 20
    q, k, v = case(2, qh, kvh, d, first, rows, 0)
    _, want = port.prefill(q, k, v, qh, kvh, d, first, rows, 0)
    V = verbs.Verbs(fam)
    scores = cuda.zeros((rows * qh, first + rows), dtype=cuda.float32, device="cuda")
    out = cuda.zeros((rows, qh, d), dtype=cuda.int16, device="cuda")
    V.attention_causal_rows(dev(cuda, q), dev(cuda, k), dev(cuda, v), scores, out, qh, kvh, d, first, rows)
    assert fam.sys.compute_completed()
    assert_close16(host_bits(out), want, 0, "worded causal doors")


def test_config2_shape_at_a_quarter_against_the_reference(cuda, port, reference):
    """16 q heads on 2 kv heads, head_dim 256, bf16 0.5·N(0,1) that fp16 holds exactly, 1,024 rows; the reference is
    driven in 256-row chunks as its runtime drives it."""
    w = workloads.config2(rows=1024)
    if reference is not None:
        to16 = lambda b: to_bits(from_bits(b, 1), 0)
        want = from_bits(reference.prefill(to16(w.q), to16(w.k), to16(w.v), 16, 2, 256, 1024), 0)
        slack = 2.0 ** -11 * np.maximum(np.abs(want), 2.0 ** -14)          # the reference's own fp16 output rounding
    else:
        _, want = port.prefill(w.q, w.k, w.v, 16, 2, 256, 0, 1024, 1)
        slack = 0.0
    o = cuda.zeros((1024, 16, 256), dtype=cuda.int16, device="cuda")
    ext.prefill(o, dev(cuda, w.q), dev(cuda, w.k), dev(cuda, w.v), 16, 2, 256, 0, 1024, 1)
    cuda.cuda.synchronize()
    got = from_bits(host_bits(o), 1).reshape(want.shape)
    ulp = 2.0 ** -8 * np.maximum(np.abs(want), 2.0 ** -14)                  # half a bf16 ulp at most 2^-8 |x|
    assert (np.abs(got - want) <= np.maximum(2e-3, ulp + 1e-3) + slack).all(), np.abs(got - want).max()


def test_config2_full_size_structure(cuda):
    """Size-independent properties at 4,096 rows: the first row is its own value row exactly; a shorter prompt is a
    bit-exact prefix of a longer one (causality); the launch is bit-repeatable."""
    w = workloads.config2()
    tq, tk, tv = dev(cuda, w.q), dev(cuda, w.k), dev(cuda, w.v)
    full = cuda.zeros((4096, 16, 256), dtype=cuda.int16, device="cuda")
    ext.prefill(full, tq, tk, tv, 16, 2, 256, 0, 4096, 1)
    again = cuda.zeros_like(full)
    ext.prefill(again, tq, tk, tv, 16, 2, 256, 0, 4096, 1)
    half = cuda.zeros((2048, 16, 256), dtype=cuda.int16, device="cuda")
    ext.prefill(half, tq, tk, tv, 16, 2, 256, 0, 2048, 1)
    tail = cuda.zeros((2048, 16, 256), dtype=cuda.int16, device="cuda")
    ext.prefill(tail, tq[2048:], tk, tv, 16, 2, 256, 2048, 2048, 1)         # the second half as a chunk with first = 2048
    cuda.cuda.synchronize()
    assert ext.device_status() == 0
    assert cuda.equal(full, again)
    assert cuda.equal(full[:2048], half)
    assert cuda.equal(full[2048:], tail)
    got0 = host_bits(full[0])                                                # [16][256]
    assert np.array_equal(got0, np.repeat(w.v[0], 8, axis=0))
    assert np.isfinite(from_bits(host_bits(full), 1)).all()


def test_refusals(cuda):
    t = cuda.zeros(4096, dtype=cuda.int16, device="cuda")
    with pytest.raises(ext.B200Error):
        ext.prefill(t, t, t, t, 4, 2, 96, 0, 4)
    with pytest.raises(ext.B200Error):
        ext.prefill(t, t, t, t, 4, 3, 64, 0, 4)
    with pytest.raises(ext.B200Error):
        ext.prefill(t, t, t, t, 4, 2, 64, 0, 0)
