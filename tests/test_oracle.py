"""Pins the checker itself: the C restatement against outputs of the reference's own CPU family (tests/golden/, and
live where oracle/_ref is present) and against fp64 numpy."""
import numpy as np
import pytest

import oracle
from oracle import FP16, from_bits, to_bits

DEC = ["dec_a", "dec_b", "dec_c", "dec_d"]


@pytest.mark.parametrize("tag", DEC)
def test_decode_matches_reference_golden(golden, port, tag):
    qh, kvh, d, L = (int(x) for x in golden[f"{tag}_shape"])
    q, k, v = golden[f"{tag}_q"], golden[f"{tag}_k"], golden[f"{tag}_v"]
    p = port.scores(q, k, qh, kvh, d, L)
    np.testing.assert_allclose(p, golden[f"{tag}_p"], rtol=2e-5, atol=1e-7)
    o, _ = port.mix(p, v, qh, kvh, d, L)
    # fp16 outputs: identical up to one unit in the last place where summation order differs
    assert np.abs(from_bits(o, 0) - from_bits(golden[f"{tag}_o"], 0)).max() <= 2.0 ** -10 * max(1.0, np.abs(from_bits(o, 0)).max())


@pytest.mark.parametrize("tag", DEC)
def test_residual_merge_finish_match_reference_golden(golden, port, tag):
    qh, kvh, d, L = (int(x) for x in golden[f"{tag}_shape"])
    q, k, v = golden[f"{tag}_q"], golden[f"{tag}_k"], golden[f"{tag}_v"]
    cut = int(golden[f"{tag}_cut"][0])
    ra = port.residual(q, np.ascontiguousarray(k[:cut]), np.ascontiguousarray(v[:cut]), qh, kvh, d, cut)
    rb = port.residual(q, np.ascontiguousarray(k[cut:]), np.ascontiguousarray(v[cut:]), qh, kvh, d, L - cut)
    np.testing.assert_allclose(ra, golden[f"{tag}_res_a"], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(rb, golden[f"{tag}_res_b"], rtol=1e-4, atol=1e-5)
    rm = port.merge(ra, rb, qh, d)
    np.testing.assert_allclose(rm, golden[f"{tag}_res_m"], rtol=1e-4, atol=1e-5)
    o, _ = port.finish(rm, qh, d)
    want = from_bits(golden[f"{tag}_o_merged"], 0)
    assert np.abs(from_bits(o, 0) - want).max() <= 2.0 ** -10 * max(1.0, np.abs(want).max())
    # and the merged answer is the one-call answer (the reference's exactness claim, kernels.cuh:1180-1184)
    assert np.abs(want - from_bits(golden[f"{tag}_o"], 0)).max() <= 2e-3


@pytest.mark.parametrize("tag", ["cau_a", "cau_b"])
def test_causal_matches_reference_golden(golden, port, tag):
    qh, kvh, d, first, rows = (int(x) for x in golden[f"{tag}_shape"])
    q, k, v = golden[f"{tag}_q"], golden[f"{tag}_k"], golden[f"{tag}_v"]
    want = from_bits(golden[f"{tag}_o"], 0)
    three = port.causal_three_doors(q, k, v, qh, kvh, d, first, rows)
    fused, o32 = port.prefill(q, k, v, qh, kvh, d, first, rows)
    assert np.array_equal(three, fused)
    assert np.abs(from_bits(fused, 0) - want).max() <= 2.0 ** -10 * max(1.0, np.abs(want).max())
    assert np.abs(o32 - want).max() <= 1e-3


@pytest.mark.parametrize("tag", ["dn_a", "dn_b"])
def test_deltanet_matches_reference_golden(golden, port, tag):
    kh, vh, d, rows, gate = (int(x) for x in golden[f"{tag}_shape"])
    conved, z, beta, g, w = (golden[f"{tag}_{n}"] for n in ("conved", "z", "beta", "g", "w"))
    S = golden[f"{tag}_S0"].copy()
    o_rows = port.deltanet(S, conved[:rows], z[:rows], beta[:rows], g[:rows], w, kh, vh, d, rows, gate)
    ref_S = golden[f"{tag}_S_rows"]
    assert np.abs(S - ref_S).max() <= 1e-3 * np.abs(ref_S).max()
    assert np.abs(from_bits(o_rows, 0) - from_bits(golden[f"{tag}_o_rows"], 0)).max() <= 2e-3
    o_step = port.deltanet(S, np.ascontiguousarray(conved[rows:]), np.ascontiguousarray(z[rows:]), np.ascontiguousarray(beta[rows:]),
                           np.ascontiguousarray(g[rows:]), w, kh, vh, d, 1, gate)
    assert np.abs(S - golden[f"{tag}_S_step"]).max() <= 1e-3 * np.abs(golden[f"{tag}_S_step"]).max()
    assert np.abs(from_bits(o_step, 0) - from_bits(golden[f"{tag}_o_step"], 0)).max() <= 2e-3


def test_decode_against_fp64(port):
    rng = np.random.default_rng(7)
    qh, kvh, d, L = 8, 2, 64, 257
    q, k, v = (to_bits(rng.standard_normal(s, dtype=np.float32), 0) for s in ((qh, d), (L, kvh, d), (L, kvh, d)))
    _, o32 = port.decode(q, k, v, qh, kvh, d, L)
    qf, kf, vf = (from_bits(x, 0).astype(np.float64) for x in (q, k, v))
    want = np.zeros((qh, d))
    for h in range(qh):
        s = kf[:, h // (qh // kvh), :] @ qf[h] / np.sqrt(d)
        w = np.exp(s - s.max())
        want[h] = (w / w.sum()) @ vf[:, h // (qh // kvh), :]
    assert np.abs(o32 - want).max() < 1e-5


def test_bf16_inputs_are_fp16_exact_and_port_agrees_across_dtypes(port):
    """The bridge used for every bf16 configuration: the same real numbers, read as fp16 by the reference and as bf16 by
    the kernels, give the same fp32 result in the restatement."""
    rng = np.random.default_rng(11)
    qh, kvh, d, L = 8, 1, 64, 100
    vals = [oracle.fp16_exact_bf16(rng.standard_normal(s, dtype=np.float32)) for s in ((qh, d), (L, kvh, d), (L, kvh, d))]
    as16 = [to_bits(x, 0) for x in vals]
    asbf = [to_bits(x, 1) for x in vals]
    for a, b, x in zip(as16, asbf, vals):
        assert np.array_equal(from_bits(a, 0), x) and np.array_equal(from_bits(b, 1), x)
    _, o16 = port.decode(*as16, qh, kvh, d, L, 0)
    _, obf = port.decode(*asbf, qh, kvh, d, L, 1)
    assert np.array_equal(o16, obf)


def test_half_conversion_edges(port):
    lib = port.lib
    import ctypes as C
    lib.oracle_f32_to_f16.restype, lib.oracle_f32_to_f16.argtypes = C.c_uint16, [C.c_float]
    lib.oracle_f16_to_f32.restype, lib.oracle_f16_to_f32.argtypes = C.c_float, [C.c_uint16]
    for x in [0.0, -0.0, 1.0, 65504.0, 65520.0, 1e-8, 6e-8, 6.1e-5, -3.14159, 0.1, 2049.0, 2051.0]:
        want = np.float32(x).astype(np.float16)
        got = lib.oracle_f32_to_f16(x)
        assert got == int(want.view(np.uint16)) or (np.isinf(want) and got & 0x7FFF == 0x7C00), x
    for h in [0, 1, 0x03FF, 0x0400, 0x3C00, 0x7BFF, 0x8001, 0xFBFF]:
        assert lib.oracle_f16_to_f32(h) == float(np.array([h], np.uint16).view(np.float16)[0])


def test_live_reference_agrees_with_golden(golden, reference):
    if reference is None:
        pytest.skip("oracle/_ref holds no reference family on this machine")
    qh, kvh, d, L = (int(x) for x in golden["dec_a_shape"])
    o = reference.decode(golden["dec_a_q"], golden["dec_a_k"], golden["dec_a_v"], qh, kvh, d, L)
    assert np.array_equal(o, golden["dec_a_o"])


def test_gathered_rows_sink_and_deltanet_inputs_match_reference_golden(golden, port):
    qh, kvh, d, most = (int(x) for x in golden["gr_shape"])
    p, o = oracle.gathered_rows(port, golden["gr_q"], golden["gr_k"], golden["gr_v"], golden["gr_lens"], qh, kvh, d)
    for u, n in enumerate(golden["gr_lens"]):                      # a row's weights occupy heads x its own length
        np.testing.assert_allclose(p[u, :qh * n], golden["gr_p"][u, :qh * n], rtol=2e-5, atol=1e-7)
    assert np.abs(from_bits(o, 0) - from_bits(golden["gr_o"], 0)).max() <= 2.0 ** -10
    np.testing.assert_allclose(oracle.softmax_sink(port, golden["sink_scores"], golden["sink_sink"]), golden["sink_p"], rtol=2e-5, atol=1e-8)
    heads, rows, ch = (int(x) for x in golden["dni_shape"])
    window = golden["dni_window0"].copy()
    beta, g, out = oracle.deltanet_inputs(port, golden["dni_a"], golden["dni_b"], golden["dni_a_log"], golden["dni_dt_bias"], golden["dni_w"],
                                          golden["dni_x"], window, heads, rows, ch)
    for got, want in ((beta, golden["dni_beta"]), (g, golden["dni_g"]), (out, golden["dni_o"])):
        assert np.abs(from_bits(got, 0) - from_bits(want, 0)).max() <= 2.0 ** -10 * max(1.0, np.abs(from_bits(want, 0)).max())
    assert np.array_equal(window, golden["dni_window"])


def test_row_residuals_golden_stand_for_the_causal_answer(golden, port):
    qh, kvh, d, first, rows = (int(x) for x in golden["rr_shape"])
    res = golden["rr_res"]
    _, want = port.prefill(golden["rr_q"], golden["rr_k"], golden["rr_v"], qh, kvh, d, first, rows)
    np.testing.assert_allclose(res[:, :, 2:] / res[:, :, 1:2], want, rtol=0, atol=1e-5)


# ---- the TurboQuant-coded tiers ------------------------------------------------------------------------------------

def test_port_rotation_both_ways(golden, port):
    sign, x = golden["tq_sign"], golden["tq_x"]
    rot = oracle.hadamard_blocks(port, x, sign, 128, 0)
    assert np.array_equal(rot, golden["tq_rot"])
    assert np.array_equal(oracle.hadamard_blocks(port, rot, sign, 128, 1), golden["tq_unrot"])
    # R^T R = I up to the two roundings to 16 bits
    back = oracle.from_bits(golden["tq_unrot"], FP16)
    assert np.abs(back - oracle.from_bits(x, FP16)).max() < 4e-3


@pytest.mark.parametrize("d", [4, 8])
def test_port_encode_rows(golden, port, d):
    codes, scales = oracle.tq_encode_rows(port, golden["tq_rows"], d)
    assert np.array_equal(scales, golden[f"tq_scales_{d}"])
    assert np.array_equal(codes, golden[f"tq_codes_{d}"])
    assert scales[7] == 0 and scales[8] == 0 and not codes[7].any() and not codes[8].any(), "dead rows are stored as zeros"
    # and what was stored is the input to within the code's step: decode and compare
    x = oracle.from_bits(golden["tq_rows"], FP16)
    back = oracle.from_bits(oracle.tq_decode(port, codes, scales.view(np.uint8).copy(), d, *x.shape), FP16)
    live = np.ones(len(x), bool); live[[7, 8]] = False
    err = np.sqrt(((back[live] - x[live]) ** 2).mean(axis=1) / (x[live] ** 2).mean(axis=1))      # rms error over rms, a row
    assert err.max() < (0.15 if d == 4 else 0.02), err.max()


@pytest.mark.parametrize("d", [4, 8])
def test_port_residual_over_coded_rows(golden, port, d):
    qh, kvh, dh, L = (int(v) for v in golden["tq_res_shape"])
    kc, ks = oracle.tq_encode_rows(port, golden["tq_res_k"], d)
    vc, vs = oracle.tq_encode_rows(port, golden["tq_res_v"], d)
    res = oracle.residual_tq(port, golden["tq_res_q"], kc, ks, vc, vs, qh, kvh, dh, L, d)
    want = golden[f"tq_res_{d}"]
    assert np.allclose(res[:, 0], want[:, 0], rtol=0, atol=2e-5) and np.allclose(res[:, 1], want[:, 1], rtol=2e-5)
    assert np.abs(res[:, 2:] - want[:, 2:]).max() <= 2e-5 * np.abs(want[:, 2:]).max() + 1e-6


# ---- the small steps either side of attention in a mixer -----------------------------------------------------------

def test_port_mixer_steps(golden, port):
    P, L = oracle._p, port.lib
    g = golden
    z = np.zeros_like(g["mx_add_z"]); L.oracle_vector_add(P(z), P(g["mx_add_x"]), P(g["mx_add_y"]), z.size)
    assert np.array_equal(z, g["mx_add_z"])
    o = np.zeros_like(g["mx_norm_o"]); L.oracle_rmsnorm_rows(P(o), P(g["mx_norm_x"]), P(g["mx_norm_w"]), 256, 5, 300, 256, 1e-6)
    assert (np.abs(o.astype(np.int32) - g["mx_norm_o"].astype(np.int32)) <= 1).all()           # the sum's order is the family's own
    o1 = np.zeros_like(g["mx_norm1_o"]); L.oracle_rmsnorm_rows(P(o1), P(g["mx_norm1_x"]), P(g["mx_norm1_w"]), 2048, 1, 2048, 2048, 1e-5)
    assert (np.abs(o1.astype(np.int32) - g["mx_norm1_o"].astype(np.int32)) <= 1).all()
    for tag in "abc":
        theta, hd, pos = g[f"mx_ang_{tag}_args"]
        cs = np.zeros(int(hd), np.float32); L.oracle_rope_angles(P(cs), int(pos), None, theta, int(hd), 1, 0, 0)
        assert np.array_equal(cs, g[f"mx_ang_{tag}"])
    cs = np.zeros((4, 64), np.float32); L.oracle_rope_angles(P(cs), 100000, None, 1e7, 64, 4, 0, 0)
    assert np.array_equal(cs, g["mx_ang_rows"])
    csm = np.zeros((4, 64), np.float32); L.oracle_rope_angles(P(csm), 0, P(g["mx_ang_mrope_pos"]), 1e7, 64, 4, 11 | (10 << 16), 1)
    assert np.array_equal(csm, g["mx_ang_mrope"])
    csa = np.zeros((3, 72), np.float32); L.oracle_rope_angles(P(csa), 0, P(g["mx_ang_axial_pos"]), 1e4, 72, 3, 0, 2)
    assert np.array_equal(csa, g["mx_ang_axial"])
    oh = np.zeros_like(g["mx_rope_o"]); L.oracle_rope_rows(P(oh), P(g["mx_rope_x"]), P(g["mx_ang_a"]), 1, 4, 64, 0, 64)
    assert np.array_equal(oh, g["mx_rope_o"])
    orr = g["mx_rope_rows_x"].copy(); L.oracle_rope_rows(P(orr), P(g["mx_rope_rows_x"]), P(g["mx_ang_rows"]), 3, 2, 128, 256, 64)
    assert np.array_equal(orr, g["mx_rope_rows_o"])
    for inv in (0, 1):
        xi = g["mx_rope_il_x"]; oi = xi.copy()
        L.oracle_rope_interleaved(P(oi[:, 32:]), P(xi[:, 32:]), P(g["mx_ang_a"]), 3, 96, 64, inv)
        assert np.array_equal(oi, g[f"mx_rope_il_{inv}"])
    og = np.zeros_like(g["mx_gate_o"]); L.oracle_attention_gate_rows(P(og), P(g["mx_gate_att"]), P(g["mx_gate_qg"]), 6, 64)
    assert np.array_equal(og, g["mx_gate_o"])
    dst = np.zeros_like(g["mx_copy_dst"]); L.oracle_vector_copy_rows(P(dst), 40, P(g["mx_copy_src"]), 50, 33, 4)
    assert np.array_equal(dst, g["mx_copy_dst"])


def test_port_weight_path_doors(golden, port):
    """The whole-row rotation and a coded matrix times a vector, restated, against the reference's CPU family bit for bit."""
    g = golden
    for n in (96, 512, 896, 1152):
        assert np.array_equal(oracle.hadamard_rotate(port, g[f"wp_rot_x_{n}"], g["wp_sign"]), g[f"wp_rot_o_{n}"]), f"a row of {n}"
    x, cols = g["wp_gemv_x"], g["wp_gemv_x"].size
    outs = {}
    for d in (4, 8, 5):
        codes, scales = g[f"wp_gemv_codes_{d}"], g[f"wp_gemv_scales_{d}"]
        outs[d] = oracle.tq_gemv(port, codes, scales.view(np.uint8).copy(), x, d, codes.shape[0], cols)
        assert np.array_equal(outs[d], g[f"wp_gemv_o_{d}"]), f"width {d}"
    assert np.array_equal(np.concatenate([outs[4], outs[8]]), g["wp_groups_o"])          # groups: the gemv once a group
    # rmsnorm_rotate: the norm, then the rotation of what the norm stored
    h = np.zeros(896, np.uint16)
    port.lib.oracle_rmsnorm_rows(oracle._p(h), oracle._p(g["wp_nr_x"]), oracle._p(g["wp_nr_w"]), 896, 1, 896, 896, np.float32(1e-6))
    assert np.array_equal(h, g["wp_nr_h"])
    assert np.array_equal(oracle.hadamard_rotate(port, h, g["wp_sign"]), g["wp_nr_hrot"])


def test_port_glm_doors(golden, port):
    """Kimi Delta Attention, the latent's absorb and expand and the indexer, restated, against the reference's CPU family."""
    import glm_cases
    glm_cases.check_kda(golden, lambda S, **kw: oracle.kda_steps(port, S, **kw), state_rtol=1e-6, out_atol=2e-4)
    glm_cases.check_mla(golden, lambda *a: oracle.absorb_rows(port, *a), lambda *a: oracle.expand_rows(port, *a), steps=0)
    glm_cases.check_indexer(golden, lambda **kw: oracle.indexer(port, **kw))

    def select(scores, pools, k, kpool, tail_first, tail):
        index, count = np.zeros(min(k, pools) * kpool + tail, np.uint32), np.zeros(1, np.uint32)
        port.lib.oracle_index_select(oracle._p(index), oracle._p(count), oracle._p(scores), pools, k, kpool, tail_first, tail)
        return index[: int(count[0])]
    glm_cases.check_select(golden, select)
