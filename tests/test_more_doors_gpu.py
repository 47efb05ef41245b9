"""The doors either side of the hot kernels on a B200, against outputs of the reference's CPU family (tests/golden/):
a residual a row through the fused prefill kernel, the per-row gathered forms, the sink softmax, DeltaNet's gates and
causal conv."""
import numpy as np
import pytest

from oracle import from_bits
from silvann_b200 import ext
from util import dev, host_bits

pytestmark = pytest.mark.gpu


def close16(got_bits, want_bits, what, ulps=1):
    want = from_bits(want_bits, 0)
    err = np.abs(from_bits(got_bits, 0).reshape(want.shape) - want)
    assert (err <= np.maximum(2e-3, ulps * 2.0 ** -10 * np.abs(want))).all(), f"{what}: {err.max()}"


def test_row_residuals_through_the_doors_and_the_extension(cuda, fam, golden):
    qh, kvh, d, first, rows = (int(x) for x in golden["rr_shape"])
    want = golden["rr_res"][:, :, 2:] / golden["rr_res"][:, :, 1:2]
    tq, tk, tv = (dev(cuda, golden[f"rr_{n}"]) for n in "qkv")
    p = cuda.zeros((rows * qh, first + rows), dtype=cuda.float32, device="cuda")
    res = cuda.zeros((rows, qh, d + 2), dtype=cuda.float32, device="cuda")
    before = ext.counters()["fused_prefill"]
    fam.nn.attention_weights_rows(p.data_ptr(), res.data_ptr(), tq.data_ptr(), tk.data_ptr(), qh, kvh, d, first, rows)
    fam.nn.attention_residual_mix_rows(res.data_ptr(), p.data_ptr(), tv.data_ptr(), qh, kvh, d, first, rows)
    assert fam.sys.compute_completed()
    assert ext.counters()["fused_prefill"] == before + 1
    got = res.cpu().numpy()
    np.testing.assert_allclose(got[:, :, 2:] / got[:, :, 1:2], want, rtol=0, atol=2e-3)
    # each row's residual finishes to that row's causal answer, and merges like any other
    o = cuda.zeros((qh, d), dtype=cuda.int16, device="cuda")
    fam.nn.attention_finish(o.data_ptr(), res[rows - 1].data_ptr(), qh, d, None)
    assert fam.sys.compute_completed()
    assert np.abs(from_bits(host_bits(o), 0) - want[rows - 1]).max() <= 2e-3
    # the same pair as worded (weights left in p because something else came between)
    res2 = cuda.zeros_like(res)
    fam.nn.attention_weights_rows(p.data_ptr(), res2.data_ptr(), tq.data_ptr(), tk.data_ptr(), qh, kvh, d, first, rows)
    assert fam.sys.compute_completed()
    fam.nn.attention_residual_mix_rows(res2.data_ptr(), p.data_ptr(), tv.data_ptr(), qh, kvh, d, first, rows)
    assert fam.sys.compute_completed()
    np.testing.assert_allclose(res2.cpu().numpy(), golden["rr_res"], rtol=1e-4, atol=1e-5)
    # and through the extension, with the 16-bit answer beside the residual
    o_all = cuda.zeros((rows, qh, d), dtype=cuda.int16, device="cuda")
    res3 = cuda.zeros_like(res)
    ext.prefill(o_all, tq, tk, tv, qh, kvh, d, first, rows, 0, res=res3)
    cuda.cuda.synchronize()
    got3 = res3.cpu().numpy()
    np.testing.assert_allclose(got3[:, :, 2:] / got3[:, :, 1:2], want, rtol=0, atol=2e-3)
    assert np.abs(from_bits(host_bits(o_all), 0) - want).max() <= 2e-3


def test_gathered_rows_doors(cuda, fam, golden):
    qh, kvh, d, most = (int(x) for x in golden["gr_shape"])
    lens = golden["gr_lens"]
    rows = len(lens)
    tq, tk, tv = (dev(cuda, golden[f"gr_{n}"]) for n in "qkv")
    tl = dev(cuda, lens)
    p = cuda.zeros((rows, qh * most), dtype=cuda.float32, device="cuda")
    o = cuda.zeros((rows, qh, d), dtype=cuda.int16, device="cuda")
    fam.nn.attention_scores_grouped_rows(p.data_ptr(), qh * most, tq.data_ptr(), qh * d, tk.data_ptr(), most * kvh * d, tl.data_ptr(), qh, kvh, d, most, rows)
    fam.nn.attention_softmax_lens(p.data_ptr(), qh * most, tl.data_ptr(), qh, rows)
    fam.nn.attention_mix_rows(o.data_ptr(), qh * d, p.data_ptr(), qh * most, tv.data_ptr(), most * kvh * d, tl.data_ptr(), qh, kvh, d, rows, None)
    assert fam.sys.compute_completed()
    got = p.cpu().numpy()
    for u, n in enumerate(lens):
        np.testing.assert_allclose(got[u, :qh * n], golden["gr_p"][u, :qh * n], rtol=1e-4, atol=1e-7)
    close16(host_bits(o), golden["gr_o"], "mix_rows")


def test_softmax_sink_door(cuda, fam, golden):
    p = dev(cuda, golden["sink_scores"].copy())
    rows, length = golden["sink_scores"].shape
    sink = dev(cuda, golden["sink_sink"])
    fam.nn.attention_softmax_sink(p.data_ptr(), sink.data_ptr(), rows, length)
    assert fam.sys.compute_completed()
    np.testing.assert_allclose(p.cpu().numpy(), golden["sink_p"], rtol=1e-4, atol=1e-8)


def test_deltanet_gates_and_conv_doors(cuda, fam, golden):
    heads, rows, ch = (int(x) for x in golden["dni_shape"])
    beta = cuda.zeros((rows, heads), dtype=cuda.int16, device="cuda"); g = cuda.zeros_like(beta)
    ta, tb, tal, tdt = (dev(cuda, golden[f"dni_{n}"]) for n in ("a", "b", "a_log", "dt_bias"))     # kept alive until the doors ran
    fam.nn.deltanet_gates_rows(beta.data_ptr(), g.data_ptr(), ta.data_ptr(), tb.data_ptr(), tal.data_ptr(), tdt.data_ptr(), heads, rows, None)
    window = dev(cuda, golden["dni_window0"].copy())
    o = cuda.zeros((rows, ch), dtype=cuda.int16, device="cuda")
    tw, tx = dev(cuda, golden["dni_w"]), dev(cuda, golden["dni_x"])
    fam.nn.deltanet_conv_steps(o.data_ptr(), window.data_ptr(), tw.data_ptr(), tx.data_ptr(), ch, rows - 1, None)
    # the last row through the one-position door: same window, same bits as the many-row door would give
    fam.nn.deltanet_conv_step(o.data_ptr() + 2 * (rows - 1) * ch, window.data_ptr(), tw.data_ptr(), tx.data_ptr() + 2 * (rows - 1) * ch, ch, None)
    assert fam.sys.compute_completed()
    close16(host_bits(beta), golden["dni_beta"], "beta")
    close16(host_bits(g), golden["dni_g"], "g", ulps=2)
    close16(host_bits(o), golden["dni_o"], "conv")
    assert np.array_equal(host_bits(window), golden["dni_window"])
