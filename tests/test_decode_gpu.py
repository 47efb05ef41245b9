"""Parity of the decode path on a B200, through the C boundary: the door pair the engine's verbs call, the residual
doors with merge and finish, and the one-call extension — against the reference's CPU family where it is present and
against the C restatement everywhere.  Tolerance: max abs error <= 2e-3 on 16-bit outputs (half an output ulp more
where bf16's ulp exceeds that), fp32 residuals to 1e-4 relative of the head's largest magnitude."""
import numpy as np
import pytest

import oracle
from oracle import FP16, from_bits, to_bits
from silvann_b200 import ext, verbs, workloads
from util import assert_close16, dev, host_bits

pytestmark = pytest.mark.gpu


def rand_case(seed, qh, kvh, d, L, dtype, scale=1.0):
    rng = np.random.default_rng(seed)
    mk = (lambda s: to_bits(oracle.fp16_exact_bf16(rng.standard_normal(s, dtype=np.float32) * scale), dtype)) if dtype else \
         (lambda s: to_bits(rng.standard_normal(s, dtype=np.float32) * scale, 0))
    return mk((qh, d)), mk((L, kvh, d)), mk((L, kvh, d))


def oracle_o32(port, q, k, v, qh, kvh, d, L, dtype):
    res = port.residual(q, k, v, qh, kvh, d, L, dtype)
    return res, res[:, 2:] / res[:, 1:2]


SHAPES = [  # qh, kvh, d, L
    (16, 4, 128, 1), (16, 4, 128, 63), (16, 4, 128, 64), (16, 4, 128, 65), (16, 4, 128, 1000),
    (8, 8, 64, 300), (8, 1, 64, 129), (16, 2, 256, 777), (32, 4, 128, 2049), (16, 1, 128, 500),
    (2, 1, 256, 4097), (24, 1, 128, 200), (48, 1, 64, 333),
]


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("qh,kvh,d,L", SHAPES)
def test_ext_decode_matches_oracle(cuda, port, qh, kvh, d, L, dtype):
    q, k, v = rand_case(100 + L, qh, kvh, d, L, dtype)
    want_res, want = oracle_o32(port, q, k, v, qh, kvh, d, L, dtype)
    tq, tk, tv = dev(cuda, q), dev(cuda, k), dev(cuda, v)
    o = cuda.zeros((qh, d), dtype=cuda.int16, device="cuda")
    res = cuda.zeros((qh, d + 2), dtype=cuda.float32, device="cuda")
    ext.decode(o, res, tq, tk, tv, qh, kvh, d, L, dtype)
    cuda.cuda.synchronize()
    assert ext.device_status() == 0
    assert_close16(host_bits(o), want, dtype, f"decode {qh}/{kvh} d{d} L{L}")
    got = res.cpu().numpy()
    # the residual is the reference's (m, l, acc): compare what it stands for, and m itself
    np.testing.assert_allclose(got[:, 0], want_res[:, 0], rtol=0, atol=1e-4)
    np.testing.assert_allclose(got[:, 2:] / got[:, 1:2], want, rtol=0, atol=1e-3)
    np.testing.assert_allclose(got[:, 1], want_res[:, 1], rtol=2e-3)


@pytest.mark.parametrize("nsplit", [1, 2, 3, 7, 32])
def test_every_split_count_gives_the_same_answer(cuda, port, nsplit):
    qh, kvh, d, L = 16, 4, 128, 3000
    q, k, v = rand_case(5, qh, kvh, d, L, 0)
    _, want = oracle_o32(port, q, k, v, qh, kvh, d, L, 0)
    o = cuda.zeros((qh, d), dtype=cuda.int16, device="cuda")
    ext.decode(o, None, dev(cuda, q), dev(cuda, k), dev(cuda, v), qh, kvh, d, L, 0, nsplit=nsplit)
    cuda.cuda.synchronize()
    assert_close16(host_bits(o), want, 0, f"nsplit {nsplit}")


def test_decode_is_bit_repeatable(cuda):
    qh, kvh, d, L = 16, 4, 128, 8192
    q, k, v = rand_case(9, qh, kvh, d, L, 0)
    tq, tk, tv = dev(cuda, q), dev(cuda, k), dev(cuda, v)
    outs = []
    for _ in range(5):
        o = cuda.zeros((qh, d), dtype=cuda.int16, device="cuda")
        ext.decode(o, None, tq, tk, tv, qh, kvh, d, L, 0)
        outs.append(host_bits(o).copy())
    assert all(np.array_equal(outs[0], x) for x in outs[1:])


def test_config1_through_the_door_pair_against_the_reference(cuda, fam, port, reference):
    """Configuration 1 (16 query heads on 4 kv heads of 128, 8,192 positions, fp16), driven exactly as (nn__attention__decode q k v scores out 16 4 128 0 8192)."""
    w = workloads.config1()
    want_bits = reference.decode(w.q, w.k, w.v, 16, 4, 128, 8192) if reference is not None else port.decode(w.q, w.k, w.v, 16, 4, 128, 8192, 0)[0]
    want = from_bits(want_bits, 0)
    before = ext.counters()
    over = cuda.zeros(1, dtype=cuda.int32, device="cuda")
    V = verbs.Verbs(fam, over)
    tq, tk, tv = dev(cuda, w.q), dev(cuda, w.k), dev(cuda, w.v)
    scores = cuda.full((16, 8192), 7.0, dtype=cuda.float32, device="cuda")
    out = cuda.zeros((16, 128), dtype=cuda.int16, device="cuda")
    V.attention_decode(tq, tk, tv, scores, out, 16, 4, 128, 0, 8192)
    assert fam.sys.compute_completed()
    after = ext.counters()
    assert after["fused_decode"] == before["fused_decode"] + 1 and after["flushed"] == before["flushed"]
    assert_close16(host_bits(out), want, 0, "config 1 via doors")
    assert int(over.item()) == 0
    # a range that does not start at zero: the verb hands the doors the cache from row `from`
    V.attention_decode(tq, tk, tv, scores, out, 16, 4, 128, 4096, 8192)
    assert fam.sys.compute_completed()
    want2 = port.residual(w.q, np.ascontiguousarray(w.k[4096:]), np.ascontiguousarray(w.v[4096:]), 16, 4, 128, 4096, 0)
    assert_close16(host_bits(out), want2[:, 2:] / want2[:, 1:2], 0, "range 4096..8192")


def test_a_scores_door_left_alone_still_writes_its_weights(cuda, fam, port):
    """The deferred door runs as worded as soon as anything else could observe its buffer."""
    qh, kvh, d, L = 8, 2, 64, 200
    q, k, v = rand_case(3, qh, kvh, d, L, 0)
    p = cuda.zeros((qh, L), dtype=cuda.float32, device="cuda")
    tq, tk = dev(cuda, q), dev(cuda, k)
    before = ext.counters()["flushed"]
    fam.nn.attention_scores(p.data_ptr(), tq.data_ptr(), tk.data_ptr(), qh, kvh, d, L)
    host = np.empty((qh, L), np.float32)
    assert fam.sys.memory_read(host.ctypes.data, p.data_ptr(), host.nbytes)     # a sys door: flushes first
    assert ext.counters()["flushed"] == before + 1
    np.testing.assert_allclose(host, port.scores(q, k, qh, kvh, d, L, 0), rtol=1e-4, atol=1e-7)
    np.testing.assert_allclose(host.sum(axis=1), 1.0, rtol=1e-5)


def test_worded_doors_without_fusion_match(cuda, fam, port):
    """mix with weights that did not come from a deferred scores call (so: the contract-worded kernels)."""
    qh, kvh, d, L = 6, 2, 96, 150          # head_dim 96 is outside the fused kernel's fit as well
    q, k, v = rand_case(4, qh, kvh, d, L, 0)
    want_res, want = oracle_o32(port, q, k, v, qh, kvh, d, L, 0)
    tq, tk, tv = dev(cuda, q), dev(cuda, k), dev(cuda, v)
    p = cuda.zeros((qh, L), dtype=cuda.float32, device="cuda")
    o = cuda.zeros((qh, d), dtype=cuda.int16, device="cuda")
    res = cuda.zeros((qh, d + 2), dtype=cuda.float32, device="cuda")
    fam.nn.attention_scores(p.data_ptr(), tq.data_ptr(), tk.data_ptr(), qh, kvh, d, L)
    fam.nn.attention_mix(o.data_ptr(), p.data_ptr(), tv.data_ptr(), qh, kvh, d, L, None)
    fam.nn.attention_weights(p.data_ptr(), res.data_ptr(), tq.data_ptr(), tk.data_ptr(), qh, kvh, d, L)
    fam.nn.attention_residual_mix(res.data_ptr(), p.data_ptr(), tv.data_ptr(), qh, kvh, d, L)
    assert fam.sys.compute_completed()
    assert_close16(host_bits(o), want, 0, "worded scores+mix")
    np.testing.assert_allclose(res.cpu().numpy(), want_res, rtol=1e-4, atol=1e-5)


def test_residual_ranges_merge_and_finish_like_the_tiered_mixer(cuda, fam, port, golden):
    """Four ranges of one cache, one residual each, merged into the first and finished — the door sequence of
    ai_qwen_3__attention_tiered (mixer__abi.cuh:383-412) — equals one call over the whole cache."""
    qh, kvh, d, L = 16, 4, 128, 5000
    q, k, v = rand_case(6, qh, kvh, d, L, 0)
    _, want = oracle_o32(port, q, k, v, qh, kvh, d, L, 0)
    V = verbs.Verbs(fam)
    tq, tk, tv = dev(cuda, q), dev(cuda, k), dev(cuda, v)
    scores = cuda.zeros((qh, L), dtype=cuda.float32, device="cuda")
    cuts = [0, 256, 1300, 4352, 5000]
    res = [cuda.zeros((qh, d + 2), dtype=cuda.float32, device="cuda") for _ in range(4)]
    before = ext.counters()["fused_residual"]
    for i in range(4):
        V.attention_residual(tq, tk, tv, scores, res[i], qh, kvh, d, cuts[i], cuts[i + 1])
        if i:
            V.attention_merge(res[0], res[i], res[0], qh, d)
    out = cuda.zeros((qh, d), dtype=cuda.int16, device="cuda")
    V.attention_finish(res[0], out, qh, d)
    assert fam.sys.compute_completed()
    assert ext.counters()["fused_residual"] == before + 4
    assert_close16(host_bits(out), want, 0, "four ranges merged")
    # the reference's own merged residual of the golden case, through our merge + finish doors
    gqh, gkvh, gd, gL = (int(x) for x in golden["dec_b_shape"])
    ra, rb = dev(cuda, golden["dec_b_res_a"]), dev(cuda, golden["dec_b_res_b"])
    V.attention_merge(ra, rb, ra, gqh, gd)
    go = cuda.zeros((gqh, gd), dtype=cuda.int16, device="cuda")
    V.attention_finish(ra, go, gqh, gd)
    assert fam.sys.compute_completed()
    np.testing.assert_allclose(ra.cpu().numpy(), golden["dec_b_res_m"], rtol=1e-5, atol=1e-6)
    assert np.abs(from_bits(host_bits(go), 0) - from_bits(golden["dec_b_o_merged"], 0)).max() <= 1e-3


def test_golden_decode_cases_through_the_doors(cuda, fam, golden):
    V = verbs.Verbs(fam)
    for tag in ("dec_a", "dec_b", "dec_c", "dec_d"):
        qh, kvh, d, L = (int(x) for x in golden[f"{tag}_shape"])
        tq, tk, tv = (dev(cuda, golden[f"{tag}_{n}"]) for n in "qkv")
        scores = cuda.zeros((qh, L), dtype=cuda.float32, device="cuda")
        out = cuda.zeros((qh, d), dtype=cuda.int16, device="cuda")
        V.attention_decode(tq, tk, tv, scores, out, qh, kvh, d, 0, L)
        assert fam.sys.compute_completed()
        assert_close16(host_bits(out), from_bits(golden[f"{tag}_o"], 0), 0, tag)


def test_overflow_sets_the_fault_word(cuda, fam):
    qh, kvh, d, L = 8, 2, 64, 70
    q = to_bits(np.ones((qh, d), np.float32), 0)
    k = to_bits(np.ones((L, kvh, d), np.float32), 0)
    v = to_bits(np.full((L, kvh, d), 60000.0, np.float32), 0)
    v[0] = to_bits(np.full((kvh, d), 65504.0, np.float32), 0)
    over = cuda.zeros(1, dtype=cuda.int32, device="cuda")
    res = cuda.zeros((qh, d + 2), dtype=cuda.float32, device="cuda")
    o = cuda.zeros((qh, d), dtype=cuda.int16, device="cuda")
    ext.decode(o, res, dev(cuda, q), dev(cuda, k), dev(cuda, v), qh, kvh, d, L, 0, over=over)
    cuda.cuda.synchronize()
    assert int(over.item()) == 0                      # 60070-ish fits a half
    big = res.clone(); big[:, 2:] *= 2.0              # acc / l now exceeds 65504
    ext.finish(o, big, qh, d, 0, over=over)
    cuda.cuda.synchronize()
    assert int(over.item()) & 0xFFFFFFFF == 0x4E504F56
    assert (host_bits(o) & 0x7FFF == 0x7C00).all()


def test_argument_refusals(cuda):
    t = cuda.zeros(64, dtype=cuda.int16, device="cuda")
    with pytest.raises(ext.B200Error) as e:
        ext.decode(t, None, t, t, t, 16, 4, 96, 10, 0)            # head_dim outside the fit
    assert e.value.code == ext.E_ARGUMENT
    with pytest.raises(ext.B200Error):
        ext.decode(t, None, t, t, t, 16, 5, 128, 10, 0)           # heads do not divide
    with pytest.raises(ext.B200Error):
        ext.decode(t, None, t, t, t, 16, 4, 128, 0, 0)            # empty range
    with pytest.raises(ext.B200Error):
        ext.decode(None, None, t, t, t, 16, 4, 128, 10, 0)        # nowhere to put the answer


def test_latent_attention_shaped_decode(cuda, fam, reference, port):
    """GLM's latent attention at decode: 64 query heads on ONE kv head 512 wide, the cached latent both keys and values
    (the same plane handed to both doors).  Wider than the fused kernel's heads: the doors run as worded, and must."""
    impl = reference if reference is not None else port
    qh, kvh, d, L = 64, 1, 512, 1500
    rng = np.random.default_rng(91)
    q = to_bits(rng.standard_normal((qh, d)).astype(np.float32) * 0.25, FP16)
    lat = to_bits(rng.standard_normal((L, kvh, d)).astype(np.float32) * 0.5, FP16)
    tq_, tl = dev(cuda, q), dev(cuda, lat)
    p = cuda.zeros((qh, L), dtype=cuda.float32, device="cuda")
    o = cuda.zeros((qh, d), dtype=cuda.int16, device="cuda")
    before = ext.counters()
    fam.nn.attention_scores(p.data_ptr(), tq_.data_ptr(), tl.data_ptr(), qh, kvh, d, L)
    fam.nn.attention_mix(o.data_ptr(), p.data_ptr(), tl.data_ptr(), qh, kvh, d, L, None)
    assert fam.sys.compute_completed()
    assert ext.counters()["refused"] == before["refused"] and ext.device_status() == 0
    want = impl.decode(q, lat, lat, qh, kvh, d, L)
    assert_close16(host_bits(o), from_bits(want, FP16), FP16, "64 heads over one 512-wide latent")
