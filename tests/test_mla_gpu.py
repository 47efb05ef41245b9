"""Latent attention at decode — many heads over ONE 512-wide latent that is both key and value — as one tcgen05 kernel, on a
B200, against the reference's CPU family (its three doors' arithmetic: scores_grouped, softmax_rows, mix) and the C
restatement.  Bars: 16-bit outputs within 2e-3 (or half a unit in the last place of bf16 where that is larger); the fp32
answer before rounding within 1e-3."""
import numpy as np
import pytest

import oracle
from oracle import from_bits, to_bits
from silvann_b200 import ext
from util import assert_close16, dev, host_bits

pytestmark = pytest.mark.gpu


def case(seed, heads, L, dtype, scale=1.0):
    rng = np.random.default_rng(seed)
    mk = lambda s, f=1.0: to_bits(oracle.fp16_exact_bf16(rng.standard_normal(s, dtype=np.float32) * np.float32(f)), dtype)
    return mk((heads, 512), scale), mk((L, 1, 512))


def want_for(impl, port, q, c, heads, L, dtype):
    if impl is not None:            # the reference has no bf16: the same real numbers as fp16
        to16 = (lambda b: to_bits(from_bits(b, 1), 0)) if dtype == 1 else (lambda b: b)
        r = impl.residual(to16(q), to16(c), to16(c), heads, 1, 512, L)
    else:
        r = port.residual(q, c, c, heads, 1, 512, L, dtype)
    return r[:, 2:] / r[:, 1:2]


@pytest.mark.parametrize("heads,L", [(64, 37), (64, 128), (64, 640), (64, 2048), (32, 1000), (64, 65536), (32, 5000)])
def test_the_three_doors_as_one_kernel(cuda, fam, reference, port, heads, L):
    q, c = case(heads + L, heads, L, 0, 2.0)
    p = cuda.zeros((heads, L), dtype=cuda.float32, device="cuda")
    o = cuda.zeros((heads, 512), dtype=cuda.int16, device="cuda")
    tq, tc = dev(cuda, q), dev(cuda, c)
    before = ext.counters()
    fam.nn.attention_scores_grouped(p.data_ptr(), tq.data_ptr(), tc.data_ptr(), heads, 1, 512, L)
    fam.nn.attention_softmax_rows(p.data_ptr(), heads, L)
    fam.nn.attention_mix(o.data_ptr(), p.data_ptr(), tc.data_ptr(), heads, 1, 512, L, None)
    assert fam.sys.compute_completed()
    after = ext.counters()
    assert after["fused_latent"] == before["fused_latent"] + 1 and after["flushed"] == before["flushed"] and ext.device_status() == 0
    impl = reference if (reference is not None or L > 5000) else None
    assert_close16(host_bits(o), want_for(impl, port, q, c, heads, L, 0), 0, f"{heads} heads over {L} latents")


@pytest.mark.parametrize("dtype", [0, 1])
def test_extension_entry_residual_and_block_counts(cuda, reference, port, dtype):
    """The fp32 answer before rounding, for one block and for many (the partials folded by the second kernel), and the same
    bits on a second run."""
    heads, L = 64, 3000
    q, c = case(7 + dtype, heads, L, dtype)
    want = want_for(reference, port, q, c, heads, L, dtype)
    tq, tc = dev(cuda, q), dev(cuda, c)
    outs = []
    for blocks in (1, 0, 5, 0):
        o = cuda.zeros((heads, 512), dtype=cuda.int16, device="cuda")
        res = cuda.zeros((heads, 514), dtype=cuda.float32, device="cuda")
        ext.mla_decode(o, res, tq, tc, heads, L, dtype, blocks)
        cuda.cuda.synchronize()
        assert ext.device_status() == 0
        r = res.cpu().numpy()
        np.testing.assert_allclose(r[:, 2:] / r[:, 1:2], want, rtol=0, atol=1e-3)
        assert_close16(host_bits(o), want, dtype, f"blocks {blocks}")
        outs.append(host_bits(o).copy())
    assert np.array_equal(outs[1], outs[3])


def test_a_reader_of_the_weights_still_finds_them(cuda, fam, port):
    """The first two doors are only recorded; a door that could observe the weights runs them as worded first."""
    heads, L = 64, 300
    q, c = case(11, heads, L, 0)
    p = cuda.zeros((heads, L), dtype=cuda.float32, device="cuda")
    tq, tc = dev(cuda, q), dev(cuda, c)
    fam.nn.attention_scores_grouped(p.data_ptr(), tq.data_ptr(), tc.data_ptr(), heads, 1, 512, L)
    fam.nn.attention_softmax_rows(p.data_ptr(), heads, L)
    assert fam.sys.compute_completed()
    got = p.cpu().numpy()
    want = port.scores(q, c, heads, 1, 512, L, 0)
    np.testing.assert_allclose(got, want, rtol=0, atol=2e-6 + 1e-4 * want.max())
    # and a mix over OTHER rows than the keys' is not the latent case: the doors as worded
    other = dev(cuda, case(12, heads, L, 0)[1])
    o = cuda.zeros((heads, 512), dtype=cuda.int16, device="cuda")
    before = ext.counters()["fused_latent"]
    fam.nn.attention_scores_grouped(p.data_ptr(), tq.data_ptr(), tc.data_ptr(), heads, 1, 512, L)
    fam.nn.attention_softmax_rows(p.data_ptr(), heads, L)
    fam.nn.attention_mix(o.data_ptr(), p.data_ptr(), other.data_ptr(), heads, 1, 512, L, None)
    assert fam.sys.compute_completed()
    assert ext.counters()["fused_latent"] == before


def test_refusals(cuda):
    t = cuda.zeros(64 * 514, dtype=cuda.float32, device="cuda")
    with pytest.raises(ext.B200Error):
        ext.mla_decode(t, None, t, t, 48, 100)              # a head count the kernel does not take
    with pytest.raises(ext.B200Error):
        ext.mla_decode(t, None, t, t, 64, 100, latent_dim=256)
    with pytest.raises(ext.B200Error):
        ext.mla_decode(None, None, t, t, 64, 100)
