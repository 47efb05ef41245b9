"""The two-tier (pinned host RAM + card) decode and the KV-range sharding arithmetic on one B200, against the checker.
The 8-rank plan of configuration 4 is walked rank by rank on the one GPU: every rank's residual from the kernel, the
fold from the library's merge — the same calls a real 8-GPU run makes, minus the all-gather."""
import numpy as np
import pytest

import oracle
from oracle import to_bits
from silvann_b200 import ext, sharded, workloads
from util import assert_close16, dev, host_bits

pytestmark = pytest.mark.gpu


def pinned(cuda, bits):
    t = cuda.from_numpy(np.ascontiguousarray(bits).view(np.int16)).pin_memory()
    return t


@pytest.mark.parametrize("host_len,dev_len,chunk", [(3000, 5000, 1024), (1024, 0, 512), (0, 700, 512), (2500, 1, 1024), (8192, 8192, 2048)])
@pytest.mark.parametrize("dtype", [0, 1])
def test_tier_decode_matches_one_call_over_the_whole_cache(cuda, port, host_len, dev_len, chunk, dtype):
    qh, kvh, d = 16, 2, 128
    L = host_len + dev_len
    rng = np.random.default_rng(L)
    mk = lambda s: to_bits(oracle.fp16_exact_bf16(rng.standard_normal(s, dtype=np.float32)), dtype)
    q, k, v = mk((qh, d)), mk((L, kvh, d)), mk((L, kvh, d))
    want_res = port.residual(q, k, v, qh, kvh, d, L, dtype)
    want = want_res[:, 2:] / want_res[:, 1:2]
    kh, vh = pinned(cuda, k[:host_len]) if host_len else None, pinned(cuda, v[:host_len]) if host_len else None
    kd, vd = (dev(cuda, k[host_len:]), dev(cuda, v[host_len:])) if dev_len else (None, None)
    tier = ext.Tier(qh, kvh, d, dtype, chunk, 3)
    o = cuda.zeros((qh, d), dtype=cuda.int16, device="cuda")
    res = cuda.zeros((qh, d + 2), dtype=cuda.float32, device="cuda")
    outs = []
    for _ in range(2):                       # the second call reuses the staging ring
        tier.decode(o, res, dev(cuda, q), kh, vh, host_len, kd, vd, dev_len)
        cuda.cuda.synchronize()
        outs.append(host_bits(o).copy())
    assert np.array_equal(outs[0], outs[1])
    assert_close16(outs[0], want, dtype, f"tier {host_len}+{dev_len}")
    got = res.cpu().numpy()
    np.testing.assert_allclose(got[:, 2:] / got[:, 1:2], want, rtol=0, atol=1e-3)
    st = tier.stats()
    assert st["h2d_bytes"] == 2 * 2 * host_len * kvh * d * 2 and st["chunks"] == 2 * ((host_len + chunk - 1) // chunk)
    assert ext.device_status() == 0
    tier.close()


def test_config4_plan_of_eight_ranks_walked_on_one_gpu(cuda, port):
    """32 q heads on 4 kv heads, head_dim 128, bf16; the sequence shortened to 16,384 positions with its first quarter
    in host RAM, as configuration 4 has it."""
    qh, kvh, d, L, host = 32, 4, 128, 16384, 4096
    w = workloads.config4(length=L)
    want_res = port.residual(w.q, w.k, w.v, qh, kvh, d, L, 1)
    want = want_res[:, 2:] / want_res[:, 1:2]
    for world in (2, 8):
        plan = sharded.shard_plan(qh, kvh, L, world)
        out = np.zeros((qh, d), np.uint16)
        residuals = {}
        for s in plan:
            k = np.ascontiguousarray(w.k[s.pos_lo:s.pos_hi, s.kv_head_lo:s.kv_head_hi])
            v = np.ascontiguousarray(w.v[s.pos_lo:s.pos_hi, s.kv_head_lo:s.kv_head_hi])
            h_len = max(0, min(host, s.pos_hi) - s.pos_lo)
            tier = ext.Tier(s.q_heads, s.kv_heads, d, 1, 2048, 2)
            res = cuda.zeros((s.q_heads, d + 2), dtype=cuda.float32, device="cuda")
            tier.decode(None, res, dev(cuda, w.q[s.q_head_lo:s.q_head_hi]), pinned(cuda, k[:h_len]) if h_len else None,
                        pinned(cuda, v[:h_len]) if h_len else None, h_len, dev(cuda, k[h_len:]) if s.positions > h_len else None,
                        dev(cuda, v[h_len:]) if s.positions > h_len else None, s.positions - h_len)
            cuda.cuda.synchronize()
            residuals[s.rank] = res
            tier.close()
        for s in plan:
            if s.rank != s.group[0]:
                continue
            def merge(a, b):
                ext.merge(a, a, b, s.q_heads, d)
                return a
            total = sharded.fold([residuals[r].clone() for r in s.group], merge)
            o = cuda.zeros((s.q_heads, d), dtype=cuda.int16, device="cuda")
            ext.finish(o, total, s.q_heads, d, 1)
            cuda.cuda.synchronize()
            out[s.q_head_lo:s.q_head_hi] = host_bits(o)
        assert_close16(out, want, 1, f"{world} ranks")


def test_tier_refusals(cuda):
    with pytest.raises(ext.B200Error):
        ext.Tier(16, 2, 128, 0, 1000, 3)          # chunk not a multiple of 128
    with pytest.raises(ext.B200Error):
        ext.Tier(16, 2, 128, 0, 1024, 1)          # a ring needs two stages
    tier = ext.Tier(16, 2, 128, 0, 1024, 2)
    t = cuda.zeros(4096, dtype=cuda.int16, device="cuda")
    with pytest.raises(ext.B200Error):
        tier.decode(t, None, t, None, None, 0, None, None, 0)
    with pytest.raises(ext.B200Error):
        tier.decode(t, None, t, None, None, 100, t, t, 10)     # host positions without host planes
    tier.close()
