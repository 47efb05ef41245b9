"""The five benchmark configurations at their FULL sizes on a B200 against the reference's own CPU family (oracle/_ref,
fp16 doors; bf16 inputs are generated fp16-exact so both sides read the same real numbers).

Bars, as the path's contract states them: 16-bit outputs within 2e-3 absolute, or half a unit in the last place of the
output type where that is larger (bf16 above magnitude 0.5) plus the reference's own fp16 output rounding; the DeltaNet
fp32 state within 1e-3 relative of its largest magnitude after 8,192 + 512 positions.  The CPU side costs seconds
(configuration 2 about five, the others about one each)."""
import numpy as np
import pytest

import oracle
from oracle import from_bits, to_bits
from silvann_b200 import ext, sharded, workloads
from util import assert_close16, dev, half_ulp, host_bits

pytestmark = pytest.mark.gpu


def as_fp16(bits_bf16):
    """The same real numbers as fp16 bits (the inputs are fp16-exact by construction)."""
    x = from_bits(bits_bf16, 1)
    b = to_bits(x, 0)
    assert np.array_equal(from_bits(b, 0), x), "an input is not fp16-exact"
    return b


@pytest.fixture(scope="module")
def ref(reference):
    if reference is None:
        pytest.skip("oracle/_ref holds no reference CPU family (build it where the reference tree is mounted)")
    return reference


def test_config1_full_size(cuda, ref):
    w = workloads.config1()
    want = from_bits(ref.decode(w.q, w.k, w.v, 16, 4, 128, 8192), 0)
    o = cuda.zeros((16, 128), dtype=cuda.int16, device="cuda")
    ext.decode(o, None, dev(cuda, w.q), dev(cuda, w.k), dev(cuda, w.v), 16, 4, 128, 8192, 0)
    cuda.cuda.synchronize()
    assert_close16(host_bits(o), want, 0, "configuration 1")


def test_config2_full_size(cuda, ref):
    """4,096 rows, 16 query heads on 2 kv heads, head_dim 256, bf16; the reference is driven in 256-row chunks as its
    runtime drives it (runtime/silvann_runtime/qwen3_5.py:584-586)."""
    w = workloads.config2()
    want = from_bits(ref.prefill(as_fp16(w.q), as_fp16(w.k), as_fp16(w.v), 16, 2, 256, 4096), 0)
    o = cuda.zeros((4096, 16, 256), dtype=cuda.int16, device="cuda")
    res = cuda.zeros((4096, 16, 258), dtype=cuda.float32, device="cuda")
    tq, tk, tv = dev(cuda, w.q), dev(cuda, w.k), dev(cuda, w.v)
    ext.prefill(o, tq, tk, tv, 16, 2, 256, 0, 4096, 1)
    ext.prefill(None, tq, tk, tv, 16, 2, 256, 0, 4096, 1, res=res)
    cuda.cuda.synchronize()
    assert ext.device_status() == 0
    slack = half_ulp(want, 0)                                               # the reference's own fp16 output rounding
    got = from_bits(host_bits(o), 1).reshape(want.shape)
    assert (np.abs(got - want) <= np.maximum(2e-3, half_ulp(want, 1) + 1e-3) + slack).all(), np.abs(got - want).max()
    r = res.cpu().numpy()
    before_rounding = r[:, :, 2:] / r[:, :, 1:2]                            # this kernel's answer before its bf16 rounding
    assert (np.abs(before_rounding - want) <= 2e-3 + slack).all(), np.abs(before_rounding - want).max()


def test_config3_full_size(cuda, ref):
    """All 32 sequences, lengths uniform in [1,024, 100,000], 3.3 GB of bf16 KV in a permuted pool of 256-position pages;
    the reference attends each sequence gathered to the contiguous planes its doors take."""
    L = workloads.config3_layout()
    q, k_pool, v_pool = workloads.config3_fill(L)
    plan = ext.Plan()
    plan.plan(L.seq_lens, L.q_heads, L.kv_heads, L.head_dim)
    o = cuda.zeros((32, L.q_heads, L.head_dim), dtype=cuda.int16, device="cuda")
    res = cuda.zeros((32, L.q_heads, L.head_dim + 2), dtype=cuda.float32, device="cuda")
    plan.decode(o, res, dev(cuda, q), dev(cuda, k_pool), dev(cuda, v_pool), L.pool_pages, workloads.PAGE_POSITIONS, dev(cuda, L.page_table),
                L.page_table.shape[1], 1)
    cuda.cuda.synchronize()
    assert ext.device_status() == 0
    assert plan.info()["positions"] == L.positions == int(L.seq_lens.sum())
    got, r = host_bits(o), res.cpu().numpy()
    for s in range(32):
        n = int(L.seq_lens[s])
        ks, vs = workloads.gather_sequence(L, k_pool, s), workloads.gather_sequence(L, v_pool, s)
        want = ref.residual(as_fp16(q[s]), as_fp16(ks), as_fp16(vs), L.q_heads, L.kv_heads, L.head_dim, n)
        want = want[:, 2:] / want[:, 1:2]
        assert_close16(got[s], want, 1, f"sequence {s} of {n} positions")
        np.testing.assert_allclose(r[s][:, 2:] / r[s][:, 1:2], want, rtol=0, atol=1e-3)
    plan.close()


def test_config4_full_size_two_tiers_and_every_rank_plan(cuda, ref):
    """One sequence of 262,144 positions, 32 query heads on 4 kv heads, head_dim 128, bf16, its first 65,536 positions in
    pinned host RAM.  One GPU attends it whole; then the plans for 2, 4 and 8 ranks are walked rank by rank on the one GPU —
    each rank's residual from the same calls a real run makes, the range halves of the 8-rank plan folded by the exchange
    kernel with the absent partner's push deposited."""
    qh, kvh, d, L, HOST = 32, 4, 128, 262144, 65536
    w = workloads.config4()
    want = ref.residual(as_fp16(w.q), as_fp16(w.k), as_fp16(w.v), qh, kvh, d, L)
    want = want[:, 2:] / want[:, 1:2]
    pin = lambda a: cuda.from_numpy(np.ascontiguousarray(a).view(np.int16)).pin_memory()
    for world in (1, 2, 4, 8):
        plan = sharded.shard_plan(qh, kvh, L, world)
        out = np.zeros((qh, d), np.uint16)
        piece = {}
        for s in plan:
            k = np.ascontiguousarray(w.k[s.pos_lo:s.pos_hi, s.kv_head_lo:s.kv_head_hi])
            v = np.ascontiguousarray(w.v[s.pos_lo:s.pos_hi, s.kv_head_lo:s.kv_head_hi])
            h_len = max(0, min(HOST, s.pos_hi) - s.pos_lo)
            tier = ext.Tier(s.q_heads, s.kv_heads, d, 1)
            tq = dev(cuda, w.q[s.q_head_lo:s.q_head_hi])
            args = (tq, pin(k[:h_len]) if h_len else None, pin(v[:h_len]) if h_len else None, h_len,
                    dev(cuda, k[h_len:]) if s.positions > h_len else None, dev(cuda, v[h_len:]) if s.positions > h_len else None, s.positions - h_len)
            if len(s.group) == 1:
                o = cuda.zeros((s.q_heads, d), dtype=cuda.int16, device="cuda")
                tier.decode(o, None, *args)
                cuda.cuda.synchronize()
                out[s.q_head_lo:s.q_head_hi] = host_bits(o)
            else:
                res = cuda.zeros((s.q_heads, d + 2), dtype=cuda.float32, device="cuda")
                tier.decode(None, res, *args)
                cuda.cuda.synchronize()
                piece[s.rank] = res
            tier.close()
        for s in plan:
            if len(s.group) == 1:
                continue
            me = s.group.index(s.rank)
            x = ext.Exchange(len(s.group), me, s.q_heads * (d + 2) * 4)
            x.connect_alone()
            for m, r in enumerate(s.group):
                if r != s.rank:
                    x.deposit(m, piece[r], s.q_heads * (d + 2) * 4)
            o = cuda.zeros((s.q_heads, d), dtype=cuda.int16, device="cuda")
            x.merge_finish(o, None, piece[s.rank], s.q_heads, d, 1, wait_ms=200)
            cuda.cuda.synchronize()
            if me == 0:
                out[s.q_head_lo:s.q_head_hi] = host_bits(o)
            else:                                                           # every member of a group holds the same bits
                assert np.array_equal(out[s.q_head_lo:s.q_head_hi], host_bits(o))
            x.close()
        assert ext.device_status() == 0
        assert_close16(out, want, 1, f"{world} rank(s)")


def deltanet_epilogue(readout, z, w, dtype):
    """What the door does to a position's fp32 read-out (kernels.cuh:677-691): round to 16 bits, RMS-norm over the head with
    eps 1e-6, times w, times silu(z) with z clamped to +-88, round again.  numpy fp32, for comparing a kernel's own 16-bit
    output with its own read-out."""
    rows, heads, d = readout.shape
    o16 = from_bits(to_bits(readout, dtype), dtype)
    scale = (1.0 / np.sqrt((o16 * o16).sum(-1, keepdims=True, dtype=np.float32) / np.float32(d) + np.float32(1e-6))).astype(np.float32)
    zc = np.clip(from_bits(z, dtype).reshape(rows, heads, d), -88.0, 88.0).astype(np.float32)
    gz = (zc / (1.0 + np.exp(-zc))).astype(np.float32)
    return o16 * scale * from_bits(w, dtype)[None, None, :] * gz


def test_config5_full_size(cuda, ref, port):
    """32 heads of 128: a prompt of 8,192 positions through the chunked kernel, then 512 single steps through the
    recurrent one, bf16.  The fp32 state is compared with the reference family's (which reads the same numbers as fp16)
    after the prompt and again after the last step; the fp32 read-out of every position — before any rounding to 16
    bits — with the checker's; the 16-bit output with the door's epilogue applied to this kernel's own read-out (the
    epilogue's own exactness), and with the checker's output up to one flip of the first rounding."""
    T, STEPS, kh, vh, d = 8192, 512, 32, 32, 128
    w = workloads.config5()
    assert w.rows == T + STEPS
    c16, z16, b16, g16, w16 = (as_fp16(x) for x in (w.conved, w.z, w.beta, w.g, w.w))
    S_ref = np.zeros((vh, d, d), np.float32)
    ref.deltanet(S_ref, c16[:T], z16[:T], b16[:T], g16[:T], w16, kh, vh, d, T)
    S_ref_prompt = S_ref.copy()
    for i in range(T, T + STEPS):
        ref.deltanet(S_ref, c16[i:i + 1], z16[i:i + 1], b16[i:i + 1], g16[i:i + 1], w16, kh, vh, d, 1)
    S_port = np.zeros((vh, d, d), np.float32)
    ro_want = np.zeros((T + STEPS, vh * d), np.float32)
    o_want = port.deltanet(S_port, w.conved, w.z, w.beta, w.g, w.w, kh, vh, d, T + STEPS, 0, 1, readout=ro_want)

    S = cuda.zeros((vh, d, d), dtype=cuda.float32, device="cuda")
    tc, tz, tb, tg, tw = (dev(cuda, x) for x in (w.conved, w.z, w.beta, w.g, w.w))
    out = cuda.zeros((T + STEPS, vh * d), dtype=cuda.int16, device="cuda")
    ro = cuda.zeros((T + STEPS, vh * d), dtype=cuda.float32, device="cuda")
    ch = (2 * kh + vh) * d
    ext.deltanet(S, tc, tz, tb, tg, tw, out, kh, vh, d, T, 1, 0, 1, readout=ro)
    cuda.cuda.synchronize()
    S_prompt = S.cpu().numpy()
    for r in range(T, T + STEPS):
        ext.deltanet(S, tc.data_ptr() + 2 * r * ch, tz.data_ptr() + 2 * r * vh * d, tb.data_ptr() + 2 * r * vh, tg.data_ptr() + 2 * r * vh,
                     tw, out.data_ptr() + 2 * r * vh * d, kh, vh, d, 1, 1, 0, 1, readout=ro.data_ptr() + 4 * r * vh * d)
    cuda.cuda.synchronize()
    assert ext.device_status() == 0
    S_end = S.cpu().numpy()
    for name, got, want in (("after the prompt", S_prompt, S_ref_prompt), ("after the steps", S_end, S_ref)):
        rel = np.abs(got - want).max() / np.abs(want).max()
        assert rel <= 1e-3, f"state {name}: {rel:.3e} relative"
    assert np.abs(S_port - S_ref).max() <= 1e-5 * np.abs(S_ref).max()       # the two CPU witnesses agree with each other

    got_ro = ro.cpu().numpy()
    assert np.abs(got_ro - ro_want).max() <= 2e-3, np.abs(got_ro - ro_want).max()
    assert np.abs(got_ro - ro_want).max() <= 1e-3 * np.abs(ro_want).max()
    got = from_bits(host_bits(out), 1).reshape(T + STEPS, vh, d)
    own = deltanet_epilogue(got_ro.reshape(T + STEPS, vh, d), w.z, w.w, 1)
    # the same read-out through the same epilogue: only the last rounding can fall the other way (the norm's sum is added
    # in another order), which is one unit in the last place
    assert (np.abs(got - own) <= np.maximum(2e-3, 2.0 * half_ulp(own, 1))).all(), "the epilogue on this kernel's own read-out"
    # against the checker's 16-bit output a flip of the FIRST rounding (read-outs that agree to 1e-6 on either side of a
    # tie) moves the input of the norm by a unit in the last place, so: two units where that exceeds 2e-3, and such
    # elements must be rare
    want = from_bits(o_want, 1).reshape(T + STEPS, vh, d)
    err = np.abs(got - want)
    assert (err <= np.maximum(2e-3, 4.0 * half_ulp(want, 1))).all(), err.max()
    assert (err > np.maximum(2e-3, half_ulp(want, 1) + 1e-3)).mean() <= 0.01
