"""Generates tests/golden/reference_x86_avx2.npz: outputs of the REFERENCE's own CPU silicon family (x86_avx2, built
unmodified by oracle/build.py from the mounted reference tree) on small seeded inputs, for every door on the hot path.

Run where the reference tree is mounted:  python tests/golden/make_golden.py
The fixtures travel with the repository; the reference tree does not.  Inputs are stored as bit patterns, so the
fixture does not depend on how this script's numpy rounds.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

import oracle  # noqa: E402
from oracle import to_bits  # noqa: E402


def main():
    R = oracle.reference()
    if R is None:
        raise SystemExit("the reference tree is not mounted and oracle/_ref holds no earlier build")
    rng = np.random.default_rng(20260901)
    out = {}

    def bits(shape, scale=1.0):
        return to_bits(rng.standard_normal(shape, dtype=np.float32) * np.float32(scale), 0)

    # one query position: decode, residual over two ranges, merge, finish
    for tag, (qh, kvh, d, L) in {"dec_a": (8, 2, 64, 200), "dec_b": (8, 2, 128, 150), "dec_c": (4, 4, 32, 17), "dec_d": (6, 1, 96, 70)}.items():
        q, k, v = bits((qh, d)), bits((L, kvh, d)), bits((L, kvh, d))
        out[f"{tag}_shape"] = np.array([qh, kvh, d, L])
        out[f"{tag}_q"], out[f"{tag}_k"], out[f"{tag}_v"] = q, k, v
        out[f"{tag}_p"] = R.scores(q, k, qh, kvh, d, L)
        out[f"{tag}_o"] = R.decode(q, k, v, qh, kvh, d, L)
        cut = L // 3
        ra = R.residual(q, k[:cut], v[:cut], qh, kvh, d, cut)
        rb = R.residual(q, np.ascontiguousarray(k[cut:]), np.ascontiguousarray(v[cut:]), qh, kvh, d, L - cut)
        rm = R.merge(ra, rb, qh, d)
        out[f"{tag}_cut"] = np.array([cut])
        out[f"{tag}_res_a"], out[f"{tag}_res_b"], out[f"{tag}_res_m"] = ra, rb, rm
        out[f"{tag}_o_merged"] = R.finish(rm, qh, d)

    # a prompt's rows through the three causal doors
    for tag, (qh, kvh, d, first, rows) in {"cau_a": (8, 2, 64, 0, 24), "cau_b": (4, 1, 128, 9, 7)}.items():
        q, k, v = bits((rows, qh, d), 0.5), bits((first + rows, kvh, d), 0.5), bits((first + rows, kvh, d), 0.5)
        out[f"{tag}_shape"] = np.array([qh, kvh, d, first, rows])
        out[f"{tag}_q"], out[f"{tag}_k"], out[f"{tag}_v"] = q, k, v
        out[f"{tag}_o"] = R.causal(q, k, v, qh, kvh, d, first, rows)

    # Gated DeltaNet: a run of rows then one more step, both gates
    for tag, (kh, vh, d, rows, gate) in {"dn_a": (1, 2, 64, 6, 0), "dn_b": (1, 1, 128, 3, 1)}.items():
        conved = bits((rows + 1, (2 * kh + vh) * d))
        z = bits((rows + 1, vh * d))
        beta = to_bits(1.0 / (1.0 + np.exp(-rng.standard_normal((rows + 1, vh), dtype=np.float32))), 0)
        g = to_bits(-np.log1p(np.exp(rng.standard_normal((rows + 1, vh), dtype=np.float32))), 0)
        w = bits((d,))
        S = (rng.standard_normal((vh, d, d), dtype=np.float32) * 0.05).astype(np.float32)
        out[f"{tag}_shape"] = np.array([kh, vh, d, rows, gate])
        for name, arr in (("conved", conved), ("z", z), ("beta", beta), ("g", g), ("w", w), ("S0", S.copy())):
            out[f"{tag}_{name}"] = arr
        o_rows = R.deltanet(S, conved[:rows], z[:rows], beta[:rows], g[:rows], w, kh, vh, d, rows, gate)
        out[f"{tag}_S_rows"], out[f"{tag}_o_rows"] = S.copy(), o_rows
        o_step = R.deltanet(S, conved[rows:], z[rows:], beta[rows:], g[rows:], w, kh, vh, d, 1, gate)
        out[f"{tag}_S_step"], out[f"{tag}_o_step"] = S.copy(), o_step

    # a residual a row (the tiered prompt path), and the per-row gathered forms, the sink softmax, DeltaNet's input doors
    qh, kvh, d, first, rows = 4, 2, 64, 5, 6
    q, k, v = bits((rows, qh, d), 0.5), bits((first + rows, kvh, d), 0.5), bits((first + rows, kvh, d), 0.5)
    out["rr_shape"] = np.array([qh, kvh, d, first, rows])
    out["rr_q"], out["rr_k"], out["rr_v"] = q, k, v
    out["rr_res"] = R.residual_rows(q, k, v, qh, kvh, d, first, rows)
    qh, kvh, d, most = 8, 1, 64, 20
    lens = np.array([20, 7, 1, 13], np.uint32)
    q, k, v = bits((4, qh, d), 0.5), bits((4, most, kvh, d), 0.5), bits((4, most, kvh, d), 0.5)
    p, o = oracle.gathered_rows(R, q, k, v, lens, qh, kvh, d)
    out["gr_shape"] = np.array([qh, kvh, d, most])
    out["gr_lens"], out["gr_q"], out["gr_k"], out["gr_v"], out["gr_p"], out["gr_o"] = lens, q, k, v, p, o
    sc = rng.standard_normal((5, 33), dtype=np.float32) * 2
    sink = bits((5,), 2.0)
    out["sink_scores"], out["sink_sink"], out["sink_p"] = sc, sink, oracle.softmax_sink(R, sc, sink)
    heads, rows, ch = 6, 5, 48
    a, b, a_log, dt_bias = bits((rows, heads)), bits((rows, heads)), bits((heads,)), bits((heads,))
    w, x, window = bits((ch, 4), 0.5), bits((rows, ch)), bits((ch, 3))
    out["dni_shape"] = np.array([heads, rows, ch])
    for name, arr in (("a", a), ("b", b), ("a_log", a_log), ("dt_bias", dt_bias), ("w", w), ("x", x), ("window0", window.copy())):
        out[f"dni_{name}"] = arr
    beta, g, o = oracle.deltanet_inputs(R, a, b, a_log, dt_bias, w, x, window, heads, rows, ch)
    out["dni_beta"], out["dni_g"], out["dni_o"], out["dni_window"] = beta, g, o, window

    # the TurboQuant-coded tiers: the level tables, the rotation both ways, rows encoded at 8 and 4 bits, a residual over them
    for d in (1, 2, 3, 4, 5, 8):
        out[f"tq_levels_{d}"] = oracle.tq_levels(R, d)
    dh = 128
    sign = to_bits(np.where(rng.random(dh) < 0.5, -1.0, 1.0).astype(np.float32), 0)
    x = bits((6, dh))
    rot = oracle.hadamard_blocks(R, x, sign, dh, 0)
    out["tq_sign"], out["tq_x"], out["tq_rot"], out["tq_unrot"] = sign, x, rot, oracle.hadamard_blocks(R, rot, sign, dh, 1)
    rows = bits((40, dh))
    rows[7] = 0                                              # a dead row: stored as zeros with a zero scale
    rows[8] = to_bits(np.full(dh, 1e-6, np.float32), 0)      # below a normal half once scaled: dead as well
    out["tq_rows"] = rows
    for d in (4, 8):
        out[f"tq_codes_{d}"], out[f"tq_scales_{d}"] = oracle.tq_encode_rows(R, rows, d)
    qh, kvh, L = 8, 2, 50
    q = bits((qh, dh))
    kr, vr = bits((L * kvh, dh)), bits((L * kvh, dh))
    out["tq_res_shape"] = np.array([qh, kvh, dh, L])
    out["tq_res_q"], out["tq_res_k"], out["tq_res_v"] = q, kr, vr
    for d in (4, 8):
        kc, ks = oracle.tq_encode_rows(R, kr, d)
        vc, vs = oracle.tq_encode_rows(R, vr, d)
        out[f"tq_res_{d}"] = oracle.residual_tq(R, q, kc, ks, vc, vs, qh, kvh, dh, L, d)

    # the small steps either side of attention in a mixer
    P_ = oracle._p
    over = R.over
    n = 1000
    x, y = bits((n,)), bits((n,))
    z = np.zeros(n, np.uint16)
    R.nn.vector_add(P_(z), P_(x), P_(y), n, P_(over)); R.wait()
    out["mx_add_x"], out["mx_add_y"], out["mx_add_z"] = x, y, z
    xr, w = bits((5, 300)), bits((256,))
    o = np.zeros((5, 256), np.uint16)
    R.nn.rmsnorm_rows(P_(o), P_(xr), P_(w), 256, 5, 300, 256, np.float32(1e-6), P_(over)); R.wait()
    out["mx_norm_x"], out["mx_norm_w"], out["mx_norm_o"] = xr, w, o
    x1, w1 = bits((2048,)), bits((2048,))
    o1 = np.zeros(2048, np.uint16)
    R.nn.rmsnorm(P_(o1), P_(x1), P_(w1), 2048, np.float32(1e-5), P_(over)); R.wait()
    out["mx_norm1_x"], out["mx_norm1_w"], out["mx_norm1_o"] = x1, w1, o1
    for tag, theta, hd, pos in (("a", 1e7, 64, 123456), ("b", 1e4, 128, 77), ("c", 1e6, 256, 4095)):
        cs = np.zeros(hd, np.float32)
        R.nn.rope_angles(P_(cs), pos, np.float32(theta), hd); R.wait()
        out[f"mx_ang_{tag}"] = cs
        out[f"mx_ang_{tag}_args"] = np.array([theta, hd, pos], np.float64)
    csr = np.zeros((4, 64), np.float32)
    R.nn.rope_angles_rows(P_(csr), 100000, np.float32(1e7), 64, 4); R.wait()
    out["mx_ang_rows"] = csr
    pos3 = np.array([[5, 2, 9], [1000, 17, 3], [7, 7, 7], [65000, 40, 41]], np.uint32)
    csm = np.zeros((4, 64), np.float32)
    R.nn.rope_angles_mrope_rows(P_(csm), P_(pos3), np.float32(1e7), 64, 4, 11 | (10 << 16)); R.wait()
    out["mx_ang_mrope_pos"], out["mx_ang_mrope"] = pos3, csm
    pos2 = np.array([[3, 8], [30, 1], [0, 0]], np.uint32)
    csa = np.zeros((3, 72), np.float32)
    R.nn.rope_angles_axial_rows(P_(csa), P_(pos2), np.float32(1e4), 72, 3); R.wait()
    out["mx_ang_axial_pos"], out["mx_ang_axial"] = pos2, csa
    xh = bits((4, 64))
    oh = np.zeros_like(xh)
    R.nn.rope(P_(oh), P_(xh), P_(out["mx_ang_a"]), 4, 64, P_(over)); R.wait()
    out["mx_rope_x"], out["mx_rope_o"] = xh, oh
    xrr = bits((3, 256))
    orr = xrr.copy()
    R.nn.rope_rows(P_(orr), P_(xrr), P_(csr), 3, 2, 128, 256, 64, P_(over)); R.wait()
    out["mx_rope_rows_x"], out["mx_rope_rows_o"] = xrr, orr
    xi = bits((3, 96))
    for inv in (0, 1):
        oi = xi.copy()
        R.nn.rope_interleaved(P_(oi[:, 32:]), P_(xi[:, 32:]), P_(out["mx_ang_a"]), 3, 96, 64, inv, P_(over)); R.wait()
        out[f"mx_rope_il_{inv}"] = oi
    out["mx_rope_il_x"] = xi
    att, qg = bits((6, 64)), bits((6, 128), 2.0)
    og = np.zeros_like(att)
    R.nn.attention_gate_rows(P_(og), P_(att), P_(qg), 6, 64, P_(over)); R.wait()
    out["mx_gate_att"], out["mx_gate_qg"], out["mx_gate_o"] = att, qg, og
    src = bits((4, 50))
    dst = np.zeros((4, 40), np.uint16)
    R.nn.vector_copy_rows(P_(dst), 40, P_(src), 50, 33, 4); R.wait()
    out["mx_copy_src"], out["mx_copy_dst"] = src, dst

    # the weight path's doors a mixer runs around its attention: the whole-row rotation, a coded matrix times a vector
    # (alone and as groups over one vector), the norm and rotation in one door
    from silvann_b200.abi import TqGroups
    sign512 = to_bits(np.where(rng.random(512) < 0.5, -1.0, 1.0).astype(np.float32), 0)
    out["wp_sign"] = sign512
    for n in (96, 512, 896, 1152):
        x = bits((n,))
        out[f"wp_rot_x_{n}"], out[f"wp_rot_o_{n}"] = x, oracle.hadamard_rotate(R, x, sign512)
    cols = 384
    xv = bits((cols,))
    out["wp_gemv_x"] = xv
    mats = {}
    for d, rows_ in ((4, 48), (8, 20), (5, 9)):
        codes, scales = oracle.tq_encode_rows(R, bits((rows_, cols), 0.05), d)
        mats[d] = (codes, scales, rows_)
        out[f"wp_gemv_codes_{d}"], out[f"wp_gemv_scales_{d}"] = codes, scales
        out[f"wp_gemv_o_{d}"] = oracle.tq_gemv(R, codes, scales.view(np.uint8).copy(), xv, d, rows_, cols)
    g = TqGroups()
    og = np.zeros(48 + 20, np.uint16)
    for i, d in enumerate((4, 8)):
        codes, scales, rows_ = mats[d]
        g.codes[i], g.luts[i], g.rows[i], g.d[i], g.out_at[i] = codes.ctypes.data, scales.ctypes.data, rows_, d, (0, 48)[i]
    g.count = 2
    R.nn.turboquant_gemv_groups(P_(og), g, P_(xv), cols, P_(over)); R.wait()
    out["wp_groups_o"] = og
    xn, wn = bits((896,)), bits((896,))
    hn, hr = np.zeros(896, np.uint16), np.zeros(896, np.uint16)
    R.nn.rmsnorm_rotate(P_(hr), P_(hn), P_(xn), P_(wn), P_(sign512), 896, np.float32(1e-6), P_(over)); R.wait()
    out["wp_nr_x"], out["wp_nr_w"], out["wp_nr_h"], out["wp_nr_hrot"] = xn, wn, hn, hr

    # the GLM mixer's doors: Kimi Delta Attention (rows from an empty state, then one more row; made and ready-made decays;
    # a head width no register form covers), the latent's absorb and expand, the indexer's doors one after another
    for tag, (heads, d, rows_) in {"kda_a": (2, 128, 4), "kda_b": (3, 64, 3), "kda_c": (1, 96, 2)}.items():
        W = heads * d
        inp = dict(conved=bits((3, rows_ + 1, W)), f=bits((rows_ + 1, W)), b=bits((rows_ + 1, heads)), dt=bits((W,)), a_log=bits((heads,), 0.3),
                   gate=bits((rows_ + 1, W)), w=bits((d,)))
        for k_, v_ in inp.items():
            out[f"{tag}_{k_}"] = v_
        out[f"{tag}_shape"] = np.array([heads, d, rows_])
        first = dict(inp, conved=np.ascontiguousarray(inp["conved"][:, :rows_]), f=inp["f"][:rows_].copy(), b=inp["b"][:rows_].copy(), gate=inp["gate"][:rows_].copy())
        last = dict(inp, conved=np.ascontiguousarray(inp["conved"][:, rows_:]), f=inp["f"][rows_:].copy(), b=inp["b"][rows_:].copy(), gate=inp["gate"][rows_:].copy())
        S0 = np.zeros((heads, d, d), np.float32)
        S1, o1 = oracle.kda_steps(R, S0, heads=heads, d=d, lower=-5.0, eps=1e-5, rows=rows_, **first)
        S1d, o1d = oracle.kda_steps(R, S0, heads=heads, d=d, lower=-5.0, eps=1e-5, rows=rows_, decayed=True, **first)
        assert np.array_equal(S1, S1d) and np.array_equal(o1, o1d), "ready-made decays are the same bits"
        S2, o2 = oracle.kda_steps(R, S1, heads=heads, d=d, lower=-5.0, eps=1e-5, rows=1, **last)
        out[f"{tag}_S1"], out[f"{tag}_o1"], out[f"{tag}_S2"], out[f"{tag}_o2"] = S1, o1, S2, o2
    heads, nope, vd, lat, rows_ = 4, 48, 40, 128, 3
    Wm, qa, oa = bits((heads * (nope + vd), lat), 0.1), bits((rows_, heads * nope)), bits((rows_, heads * lat))
    out["mla_shape"] = np.array([heads, nope, vd, lat, rows_])
    out["mla_W"], out["mla_q"], out["mla_o"] = Wm, qa, oa
    out["mla_absorbed"] = oracle.absorb_rows(R, qa, Wm, heads, nope, lat, nope + vd, 0.125, rows_)
    out["mla_absorbed_1"] = oracle.absorb_rows(R, qa[:1].copy(), Wm, heads, nope, lat, nope + vd, 0.125, 1)
    out["mla_expanded"] = oracle.expand_rows(R, oa, Wm, heads, vd, lat, nope + vd, nope, rows_)
    out["mla_expanded_1"] = oracle.expand_rows(R, oa[:1].copy(), Wm, heads, vd, lat, nope + vd, nope, 1)
    dim, kpool, ih, k_, len0, rows_, block = 32, 4, 8, 5, 45, 6, 3
    n_pos = len0 + rows_ - 1
    ix = dict(x=bits((dim,)), lw=bits((dim,)), lb=bits((dim,)), keys=bits((n_pos, dim)), gates=bits((n_pos, dim)), ape=bits((kpool, dim)),
              q=bits((rows_, ih * dim)), w=bits((rows_, ih)), src=bits((n_pos, 24)))
    ix["keys"][8:12] = ix["keys"][16:20]            # two pools alike in every number: a tie, settled by the lower index
    ix["gates"][8:12] = ix["gates"][16:20]
    out["ix_shape"] = np.array([dim, kpool, ih, k_, len0, rows_, block])
    for name, arr in ix.items():
        out[f"ix_in_{name}"] = arr
    got = oracle.indexer(R, dim=dim, kpool=kpool, heads=ih, k=k_, len0=len0, rows=rows_, scale=0.17, block=block, **ix)
    for name, arr in got.items():
        out[f"ix_{name}"] = arr
    # the choice alone on scores full of ties (and both zeros, which order apart): the cut falls inside a run of equals
    tied = rng.integers(-3, 4, 64).astype(np.float32) * np.float32(0.5)
    tied[5], tied[9] = np.float32(-0.0), np.float32(0.0)
    out["ixsel_scores"] = tied
    for k_ in (1, 7, 20, 63, 64, 80):
        index = np.zeros(min(k_, 64) * 2 + 3, np.uint32)
        count = np.zeros(1, np.uint32)
        R.nn.index_select(P_(index), P_(count), P_(tied), 64, k_, 2, 128, 3); R.wait()
        out[f"ixsel_{k_}"] = index[: int(count[0])].copy()

    path = Path(__file__).with_name("reference_x86_avx2.npz")
    np.savez_compressed(path, **out)
    print(path, path.stat().st_size, "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
