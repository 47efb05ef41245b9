"""The GLM mixer's doors — Kimi Delta Attention, the latent's absorb and expand, the sparse attention's indexer — on the
inputs tests/golden/ holds for them, through any implementation that words them as oracle/__init__.py's helpers do (the C
restatement, the reference's CPU family, or this family on a card through tests/test_glm_doors_gpu.py's adapter)."""
import numpy as np

import oracle
from oracle import FP16, from_bits

KDA_TAGS = ("kda_a", "kda_b", "kda_c")


def kda_inputs(g, tag):
    heads, d, rows = (int(v) for v in g[f"{tag}_shape"])
    inp = {k: g[f"{tag}_{k}"] for k in ("conved", "f", "b", "dt", "a_log", "gate", "w")}
    first = dict(inp, conved=np.ascontiguousarray(inp["conved"][:, :rows]), f=inp["f"][:rows].copy(), b=inp["b"][:rows].copy(), gate=inp["gate"][:rows].copy())
    last = dict(inp, conved=np.ascontiguousarray(inp["conved"][:, rows:]), f=inp["f"][rows:].copy(), b=inp["b"][rows:].copy(), gate=inp["gate"][rows:].copy())
    return heads, d, rows, first, last


def check_kda(g, run, state_rtol=1e-3, out_atol=2e-3):
    """run(S, rows=, decayed=, heads=, d=, lower=, eps=, **inputs) -> (state, out).  The state within 1e-3 of its largest
    element's size, the 16-bit outputs within 2e-3."""
    for tag in KDA_TAGS:
        heads, d, rows, first, last = kda_inputs(g, tag)
        S0 = np.zeros((heads, d, d), np.float32)
        for decayed in (False, True):
            S1, o1 = run(S0, heads=heads, d=d, lower=-5.0, eps=1e-5, rows=rows, decayed=decayed, **first)
            np.testing.assert_allclose(S1, g[f"{tag}_S1"], rtol=0, atol=state_rtol * np.abs(g[f"{tag}_S1"]).max(), err_msg=f"{tag} state, decayed={decayed}")
            assert np.abs(from_bits(o1, FP16) - from_bits(g[f"{tag}_o1"], FP16)).max() <= out_atol, f"{tag} out, decayed={decayed}"
        S2, o2 = run(g[f"{tag}_S1"], heads=heads, d=d, lower=-5.0, eps=1e-5, rows=1, decayed=False, **last)
        np.testing.assert_allclose(S2, g[f"{tag}_S2"], rtol=0, atol=state_rtol * np.abs(g[f"{tag}_S2"]).max(), err_msg=f"{tag} state after one more row")
        assert np.abs(from_bits(o2, FP16) - from_bits(g[f"{tag}_o2"], FP16)).max() <= out_atol, f"{tag} one more row"


def check_mla(g, absorb, expand, steps=1):
    """absorb(q, W, heads, nope, latent, stride, scale, rows), expand(o, W, heads, width, latent, stride, offset, rows):
    within `steps` fp16 steps (a sum's order)."""
    heads, nope, vd, lat, rows = (int(v) for v in g["mla_shape"])
    W, q, o = g["mla_W"], g["mla_q"], g["mla_o"]

    def near(got, want, what):
        d = np.abs(got.astype(np.int32) - want.astype(np.int32))
        assert (d <= steps).all(), f"{what}: {int(d.max())} fp16 steps"

    near(absorb(q, W, heads, nope, lat, nope + vd, 0.125, rows), g["mla_absorbed"], "absorb_rows")
    near(absorb(q[:1].copy(), W, heads, nope, lat, nope + vd, 0.125, 1), g["mla_absorbed_1"], "absorb")
    near(expand(o, W, heads, vd, lat, nope + vd, nope, rows), g["mla_expanded"], "expand_rows")
    near(expand(o[:1].copy(), W, heads, vd, lat, nope + vd, nope, 1), g["mla_expanded_1"], "expand")


def check_indexer(g, run):
    """run(**inputs) -> the dict oracle.indexer answers.  Scores to 1e-5 of their size; every integer exactly."""
    dim, kpool, ih, k, len0, rows, block = (int(v) for v in g["ix_shape"])
    inp = {name: g[f"ix_in_{name}"] for name in ("x", "lw", "lb", "keys", "gates", "ape", "q", "w", "src")}
    got = run(dim=dim, kpool=kpool, heads=ih, k=k, len0=len0, rows=rows, scale=0.17, block=block, **inp)
    for name in ("ln", "pooled"):
        d = np.abs(got[name].astype(np.int32) - g[f"ix_{name}"].astype(np.int32))
        assert (d <= 1).all(), f"{name}: {int(d.max())} fp16 steps"
    for name in ("scores", "blocks", "scores_rows"):
        np.testing.assert_allclose(got[name], g[f"ix_{name}"], rtol=0, atol=1e-5 * np.abs(g["ix_scores_rows"]).max(), err_msg=name)
    for name in ("index", "count", "index_rows", "counts", "gathered", "gathered_rows"):
        assert np.array_equal(got[name], g[f"ix_{name}"]), name


def check_select(g, select):
    """select(scores, pools, k, kpool, tail_first, tail) -> the positions chosen.  The tie rule, exactly."""
    for k in (1, 7, 20, 63, 64, 80):
        assert np.array_equal(select(g["ixsel_scores"], 64, k, 2, 128, 3), g[f"ixsel_{k}"]), f"k = {k}"
