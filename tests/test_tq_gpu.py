"""The TurboQuant-coded tiers of the cache on a B200 against the reference's CPU family (tests/golden/, and the family
itself where oracle/_ref holds it): level tables, rotation, encoding, and the residual over coded keys and values — as the
doors word them, a row of a prompt chunk at a time, and at a tier's real size against the reference run on the host."""
import numpy as np
import pytest

import oracle
from oracle import FP16, from_bits, to_bits
from silvann_b200 import ext
from util import dev, host_bits

pytestmark = pytest.mark.gpu


def gpu_decode(cuda, fam, codes, scales, d, rows, cols):
    tc, ts = dev(cuda, codes), dev(cuda, scales)
    out = cuda.zeros((rows, cols), dtype=cuda.int16, device="cuda")
    fam.nn.turboquant_decode(out.data_ptr(), tc.data_ptr(), codes.nbytes, ts.data_ptr(), scales.nbytes, d, rows, cols, None)
    assert fam.sys.compute_completed()
    return host_bits(out)


def test_level_tables_on_the_card(cuda, fam, golden):
    for d in (1, 2, 3, 4, 5, 8):
        n, per = 1 << d, 16 // d
        units = np.zeros((n + per - 1) // per, np.uint16)
        for c in range(n):
            units[c // per] |= np.uint16(c << (d * (c % per)))
        got = gpu_decode(cuda, fam, units.view(np.uint8).copy(), np.array([0x3C00], np.uint16), d, 1, n)
        assert np.array_equal(got.reshape(n), golden[f"tq_levels_{d}"]), f"width {d}"


def test_rotation_is_the_references_bit_for_bit(cuda, fam, golden):
    sign, x = dev(cuda, golden["tq_sign"]), dev(cuda, golden["tq_x"])
    rot, back = cuda.zeros_like(x), cuda.zeros_like(x)
    fam.nn.hadamard_blocks(rot.data_ptr(), x.data_ptr(), sign.data_ptr(), x.numel(), 128, 0, None)
    fam.nn.hadamard_blocks(back.data_ptr(), rot.data_ptr(), sign.data_ptr(), x.numel(), 128, 1, None)
    assert fam.sys.compute_completed()
    assert np.array_equal(host_bits(rot), golden["tq_rot"])
    assert np.array_equal(host_bits(back), golden["tq_unrot"])


@pytest.mark.parametrize("d", [4, 8])
def test_encode_rows(cuda, fam, golden, d):
    rows = golden["tq_rows"]
    n, cols = rows.shape
    x = dev(cuda, rows)
    codes = cuda.zeros((n, oracle.tq_row_bytes(d, cols)), dtype=cuda.uint8, device="cuda")
    scales = cuda.zeros(n, dtype=cuda.int16, device="cuda")
    fam.nn.turboquant_encode_rows(codes.data_ptr(), scales.data_ptr(), x.data_ptr(), n, cols, d, None)
    assert fam.sys.compute_completed()
    got_s, got_c = host_bits(scales), codes.cpu().numpy()
    want_s, want_c = golden[f"tq_scales_{d}"], golden[f"tq_codes_{d}"]
    # a row's scale is fp16(clip · rms); the rms is summed in another order here, so a scale may land on the neighbouring
    # half once in a long while.  Where the scale is the reference's, so must every code be.
    same = got_s == want_s
    assert same.mean() >= 0.95 and (np.abs(got_s.astype(np.int32) - want_s.astype(np.int32)) <= 1).all()
    assert np.array_equal(got_c[same], want_c[same])
    assert got_s[7] == 0 and got_s[8] == 0 and not got_c[7].any() and not got_c[8].any()


@pytest.mark.parametrize("d", [4, 8])
def test_residual_over_coded_rows_as_the_doors_word_it(cuda, fam, golden, port, d):
    qh, kvh, dh, L = (int(v) for v in golden["tq_res_shape"])
    kc, ks = oracle.tq_encode_rows(port, golden["tq_res_k"], d)
    vc, vs = oracle.tq_encode_rows(port, golden["tq_res_v"], d)
    want = golden[f"tq_res_{d}"]
    tq_, tkc, tks, tvc, tvs = (dev(cuda, a) for a in (golden["tq_res_q"], kc, ks, vc, vs))
    p = cuda.zeros((qh, L), dtype=cuda.float32, device="cuda")
    res = cuda.zeros((qh, dh + 2), dtype=cuda.float32, device="cuda")
    fam.nn.attention_weights_tq(p.data_ptr(), res.data_ptr(), tq_.data_ptr(), tkc.data_ptr(), tks.data_ptr(), qh, kvh, dh, L, d)
    assert fam.sys.compute_completed()          # something between the two doors: each runs as worded
    fam.nn.attention_residual_mix_tq(res.data_ptr(), p.data_ptr(), tvc.data_ptr(), tvs.data_ptr(), qh, kvh, dh, L, d)
    assert fam.sys.compute_completed()
    got = res.cpu().numpy()
    np.testing.assert_allclose(got[:, 0], want[:, 0], rtol=0, atol=2e-5)
    np.testing.assert_allclose(got[:, 1], want[:, 1], rtol=1e-4)
    np.testing.assert_allclose(got[:, 2:], want[:, 2:], rtol=0, atol=1e-4 * np.abs(want[:, 2:]).max())
    # the pair back to back (whatever path the family takes for it) finishes to the same attention
    res2 = cuda.zeros_like(res)
    fam.nn.attention_weights_tq(p.data_ptr(), res2.data_ptr(), tq_.data_ptr(), tkc.data_ptr(), tks.data_ptr(), qh, kvh, dh, L, d)
    fam.nn.attention_residual_mix_tq(res2.data_ptr(), p.data_ptr(), tvc.data_ptr(), tvs.data_ptr(), qh, kvh, dh, L, d)
    assert fam.sys.compute_completed()
    got2 = res2.cpu().numpy()
    np.testing.assert_allclose(got2[:, 2:] / got2[:, 1:2], want[:, 2:] / want[:, 1:2], rtol=0, atol=2e-3)
    # a prompt chunk's rows over the same tier: row r's residual is the one-row door's for query r
    rows = 3
    q3 = np.concatenate([golden["tq_res_q"]] * rows).reshape(rows, qh, dh).copy()
    q3[1] = to_bits(from_bits(q3[1], FP16) * 0.5, FP16)
    t3 = dev(cuda, q3)
    p3 = cuda.zeros((rows * qh, L), dtype=cuda.float32, device="cuda")
    r3 = cuda.zeros((rows, qh, dh + 2), dtype=cuda.float32, device="cuda")
    fam.nn.attention_weights_tq_rows(p3.data_ptr(), r3.data_ptr(), t3.data_ptr(), tkc.data_ptr(), tks.data_ptr(), qh, kvh, dh, L, d, rows)
    fam.nn.attention_residual_mix_tq_rows(r3.data_ptr(), p3.data_ptr(), tvc.data_ptr(), tvs.data_ptr(), qh, kvh, dh, L, d, rows)
    assert fam.sys.compute_completed()
    g3 = r3.cpu().numpy()
    np.testing.assert_allclose(g3[0, :, 2:] / g3[0, :, 1:2], want[:, 2:] / want[:, 1:2], rtol=0, atol=2e-3)
    np.testing.assert_allclose(g3[2, :, 2:] / g3[2, :, 1:2], want[:, 2:] / want[:, 1:2], rtol=0, atol=2e-3)
    half = oracle.residual_tq(port, q3[1], kc, ks, vc, vs, qh, kvh, dh, L, d)
    np.testing.assert_allclose(g3[1, :, 2:] / g3[1, :, 1:2], half[:, 2:] / half[:, 1:2], rtol=0, atol=2e-3)


@pytest.mark.parametrize("d,dh,qh,kvh,L", [(8, 128, 16, 4, 3000), (4, 128, 16, 4, 5000), (4, 256, 16, 2, 2500), (8, 256, 8, 2, 1111), (4, 64, 8, 8, 700),
                                           (4, 128, 32, 2, 4000), (8, 128, 32, 2, 129), (8, 256, 24, 2, 40000), (4, 256, 3, 1, 7), (8, 128, 4, 4, 128)])
def test_a_tier_at_size_against_the_reference_run_here(cuda, fam, reference, port, d, dh, qh, kvh, L):
    """Rows rotated, encoded ON THE CARD, attended on the card; the oracle attends the card's codes on the host."""
    impl = reference if reference is not None else port
    rng = np.random.default_rng(900 + d + dh + L)
    q = to_bits(rng.standard_normal((qh, dh), dtype=np.float32), FP16)
    kr = to_bits(rng.standard_normal((L * kvh, dh), dtype=np.float32), FP16)
    vr = to_bits(rng.standard_normal((L * kvh, dh), dtype=np.float32), FP16)
    tq_, tk, tv = dev(cuda, q), dev(cuda, kr), dev(cuda, vr)
    rb = oracle.tq_row_bytes(d, dh)
    kc, vc = (cuda.zeros((L * kvh, rb), dtype=cuda.uint8, device="cuda") for _ in range(2))
    ks, vs = (cuda.zeros(L * kvh, dtype=cuda.int16, device="cuda") for _ in range(2))
    fam.nn.turboquant_encode_rows(kc.data_ptr(), ks.data_ptr(), tk.data_ptr(), L * kvh, dh, d, None)
    fam.nn.turboquant_encode_rows(vc.data_ptr(), vs.data_ptr(), tv.data_ptr(), L * kvh, dh, d, None)
    p = cuda.zeros((qh, L), dtype=cuda.float32, device="cuda")
    res = cuda.zeros((qh, dh + 2), dtype=cuda.float32, device="cuda")
    o = cuda.zeros((qh, dh), dtype=cuda.int16, device="cuda")
    before = ext.counters()
    fam.nn.attention_weights_tq(p.data_ptr(), res.data_ptr(), tq_.data_ptr(), kc.data_ptr(), ks.data_ptr(), qh, kvh, dh, L, d)
    fam.nn.attention_residual_mix_tq(res.data_ptr(), p.data_ptr(), vc.data_ptr(), vs.data_ptr(), qh, kvh, dh, L, d)
    fam.nn.attention_finish(o.data_ptr(), res.data_ptr(), qh, dh, None)
    assert fam.sys.compute_completed()
    after = ext.counters()
    assert after["refused"] == before["refused"] and ext.device_status() == 0
    assert after["fused_residual"] - before["fused_residual"] == (1 if dh in (128, 256) else 0), "the pair is one kernel at head_dim 128 and 256"
    want = oracle.residual_tq(impl, q, kc.cpu().numpy(), host_bits(ks), vc.cpu().numpy(), host_bits(vs), qh, kvh, dh, L, d)
    got = res.cpu().numpy()
    np.testing.assert_allclose(got[:, 2:] / got[:, 1:2], want[:, 2:] / want[:, 1:2], rtol=0, atol=2e-3)
    want_o = want[:, 2:] / want[:, 1:2]
    assert np.abs(from_bits(host_bits(o), FP16) - want_o).max() <= 2e-3
    # and a residual over coded rows merges with one over plain rows like any other: m and l are on the same footing
    lse_got = got[:, 0] + np.log(got[:, 1])
    lse_want = want[:, 0] + np.log(want[:, 1])
    np.testing.assert_allclose(lse_got, lse_want, rtol=0, atol=2e-3)


@pytest.mark.parametrize("d,dh,qh,kvh,L,rows", [(8, 128, 16, 2, 3000, 5), (4, 128, 32, 4, 1500, 3), (4, 256, 16, 2, 2000, 3), (8, 256, 8, 2, 700, 7), (8, 128, 8, 8, 333, 2)])
def test_a_prompt_chunks_rows_over_a_tier_in_one_launch(cuda, fam, reference, port, d, dh, qh, kvh, L, rows):
    """attention_weights_tq_rows + attention_residual_mix_tq_rows: the rows of a chunk see the same tier, so they are more
    query heads of the same kv heads to the fused kernel; row r's residual is the one-row doors' for query r."""
    impl = reference if reference is not None else port
    rng = np.random.default_rng(1200 + d + dh + L + rows)
    q = to_bits(rng.standard_normal((rows, qh, dh), dtype=np.float32), FP16)
    kr = to_bits(rng.standard_normal((L * kvh, dh), dtype=np.float32), FP16)
    vr = to_bits(rng.standard_normal((L * kvh, dh), dtype=np.float32), FP16)
    kc, ks = oracle.tq_encode_rows(port, kr, d)
    vc, vs = oracle.tq_encode_rows(port, vr, d)
    tq_, tkc, tks, tvc, tvs = (dev(cuda, a) for a in (q, kc, ks, vc, vs))
    p = cuda.zeros((rows * qh, L), dtype=cuda.float32, device="cuda")
    res = cuda.zeros((rows, qh, dh + 2), dtype=cuda.float32, device="cuda")
    before = ext.counters()
    fam.nn.attention_weights_tq_rows(p.data_ptr(), res.data_ptr(), tq_.data_ptr(), tkc.data_ptr(), tks.data_ptr(), qh, kvh, dh, L, d, rows)
    fam.nn.attention_residual_mix_tq_rows(res.data_ptr(), p.data_ptr(), tvc.data_ptr(), tvs.data_ptr(), qh, kvh, dh, L, d, rows)
    assert fam.sys.compute_completed()
    after = ext.counters()
    assert after["refused"] == before["refused"] and ext.device_status() == 0
    assert after["fused_residual"] - before["fused_residual"] == 1, "the rows pair is one kernel"
    got = res.cpu().numpy()
    for r in range(rows):
        want = oracle.residual_tq(impl, q[r].copy(), kc, ks, vc, vs, qh, kvh, dh, L, d)
        np.testing.assert_allclose(got[r, :, 2:] / got[r, :, 1:2], want[:, 2:] / want[:, 1:2], rtol=0, atol=2e-3, err_msg=f"row {r}")
        np.testing.assert_allclose(got[r, :, 0] + np.log(got[r, :, 1]), want[:, 0] + np.log(want[:, 1]), rtol=0, atol=2e-3, err_msg=f"row {r} lse")
