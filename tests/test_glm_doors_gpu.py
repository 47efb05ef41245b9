"""The GLM mixer's doors on a B200 — Kimi Delta Attention (the register-resident form at head widths 64 and 128, the
in-memory form at 96), the latent's absorb and expand, the sparse attention's indexer — against outputs of the reference's
CPU family (tests/golden/), and Kimi Delta Attention at a model's size against the reference run here."""
import numpy as np
import pytest

import glm_cases
import oracle
from oracle import FP16, from_bits, to_bits
from util import OnCard

pytestmark = pytest.mark.gpu


def test_kda(cuda, fam, golden):
    glm_cases.check_kda(golden, lambda S, **kw: oracle.kda_steps(OnCard(cuda, fam), S, **kw))


def test_absorb_and_expand(cuda, fam, golden):
    glm_cases.check_mla(golden, lambda *a: oracle.absorb_rows(OnCard(cuda, fam), *a), lambda *a: oracle.expand_rows(OnCard(cuda, fam), *a))


def test_indexer(cuda, fam, golden):
    glm_cases.check_indexer(golden, lambda **kw: oracle.indexer(OnCard(cuda, fam), **kw))

    def select(scores, pools, k, kpool, tail_first, tail):
        card = OnCard(cuda, fam)
        index, count = np.zeros(min(k, pools) * kpool + tail, np.uint32), np.zeros(1, np.uint32)
        fam.nn.index_select(card.ptr(index), card.ptr(count), card.ptr(scores), pools, k, kpool, tail_first, tail)
        card.wait()
        return index[: int(count[0])]
    glm_cases.check_select(golden, select)


def test_select_over_many_pools(cuda, fam, port):
    """More pools than the block has threads, ties everywhere: the integer answer is the restatement's exactly."""
    rng = np.random.default_rng(77)
    for pools, k in ((5000, 512), (16384, 2048), (1025, 1024), (3, 8)):
        scores = np.round(rng.standard_normal(pools).astype(np.float32) * 4) / 4
        index, count = np.zeros(min(k, pools) * 4 + 2, np.uint32), np.zeros(1, np.uint32)
        port.lib.oracle_index_select(oracle._p(index), oracle._p(count), oracle._p(scores), pools, k, 4, pools * 4, 2)
        card = OnCard(cuda, fam)
        got, n = np.zeros_like(index), np.zeros(1, np.uint32)
        fam.nn.index_select(card.ptr(got), card.ptr(n), card.ptr(scores), pools, k, 4, pools * 4, 2)
        card.wait()
        assert n[0] == count[0] and np.array_equal(got, index), f"{pools} pools, the top {k}"


def test_kda_at_a_models_size(cuda, fam, reference, port):
    """64 heads of 128, a decode step and a run of rows, from a state that is not empty."""
    impl = reference if reference is not None else port
    heads, d = 64, 128
    rng = np.random.default_rng(78)
    W = heads * d
    bits = lambda shape, s=1.0: to_bits((rng.standard_normal(shape) * s).astype(np.float32), FP16)
    S = (rng.standard_normal((heads, d, d)) * 0.05).astype(np.float32)
    for rows in (1, 6):
        inp = dict(conved=bits((3, rows, W)), f=bits((rows, W)), b=bits((rows, heads)), dt=bits((W,)), a_log=bits((heads,), 0.3), gate=bits((rows, W)),
                   w=bits((d,)))
        want_S, want_o = oracle.kda_steps(impl, S, heads=heads, d=d, lower=-5.0, eps=1e-5, rows=rows, **inp)
        for decayed in ((False, True) if rows > 1 else (False,)):
            got_S, got_o = oracle.kda_steps(OnCard(cuda, fam), S, heads=heads, d=d, lower=-5.0, eps=1e-5, rows=rows, decayed=decayed, **inp)
            np.testing.assert_allclose(got_S, want_S, rtol=0, atol=1e-3 * np.abs(want_S).max())
            assert np.abs(from_bits(got_o, FP16) - from_bits(want_o, FP16)).max() <= 2e-3
