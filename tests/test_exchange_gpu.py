"""The exchange kernels (push, bounded wait, combine in member order) on ONE B200: the absent members' pushes are stood in
for by `deposit`, which puts a piece where that member's stores would have landed, as the same tagged words — the kernel
under test then runs its own push, its polls and its fold exactly as it does among real cards.

Bars: the fold equals attention_merge applied in member order and attention_finish (this library's own doors, which are
checked against the reference elsewhere) bit for bit, and the checker's merge within fp32 rounding; the sum equals the
fp32-sum-rounded-once definition bit for bit.  A wait that nothing answers ends by itself with "B2TO" in the status word."""
import numpy as np
import pytest

import oracle
from oracle import from_bits, to_bits
from silvann_b200 import ext
from util import dev, host_bits

pytestmark = pytest.mark.gpu
B2TO = 0x4232544F


def residuals(rng, members, qh, d):
    """Plausible range residuals: m anywhere, l positive, acc of the size l allows."""
    out = []
    for _ in range(members):
        r = np.empty((qh, d + 2), np.float32)
        r[:, 0] = rng.standard_normal(qh) * 3.0
        r[:, 1] = rng.uniform(0.5, 900.0, qh)
        r[:, 2:] = rng.standard_normal((qh, d)) * r[:, 1:2] * 0.3
        out.append(r)
    return out


@pytest.mark.parametrize("members,index,qh,d,dtype", [(2, 0, 8, 128, 1), (2, 1, 8, 128, 1), (3, 1, 32, 128, 0), (4, 3, 20, 256, 1), (8, 5, 16, 64, 0), (1, 0, 8, 128, 0)])
def test_fold_equals_the_merge_door_in_member_order(cuda, port, members, index, qh, d, dtype):
    rng = np.random.default_rng(members * 100 + index)
    x = ext.Exchange(members, index, qh * (d + 2) * 4)
    if members > 1:
        x.connect_alone()
    for call in range(3):                                                  # three in a row: both parities, and one reused
        parts = residuals(rng, members, qh, d)
        t = [dev(cuda, p) for p in parts]
        for m in range(members):
            if m != index:
                x.deposit(m, t[m], parts[m].nbytes)
        o = cuda.zeros((qh, d), dtype=cuda.int16, device="cuda")
        res = cuda.zeros((qh, d + 2), dtype=cuda.float32, device="cuda")
        x.merge_finish(o, res, t[index], qh, d, dtype, wait_ms=200)
        # the same fold through the doors' kernels
        acc = t[0].clone()
        for m in range(1, members):
            ext.merge(acc, acc, t[m], qh, d)
        o_want = cuda.zeros((qh, d), dtype=cuda.int16, device="cuda")
        ext.finish(o_want, acc, qh, d, dtype)
        cuda.cuda.synchronize()
        assert ext.device_status() == 0
        assert cuda.equal(res, acc), f"call {call}: residual"
        assert cuda.equal(o, o_want), f"call {call}: output"
        # and the checker's merge, within fp32 rounding of the factors
        want = parts[0]
        for m in range(1, members):
            want = port.merge(want, parts[m], qh, d)
        got = res.cpu().numpy()
        np.testing.assert_allclose(got[:, 2:] / got[:, 1:2], want[:, 2:] / want[:, 1:2], rtol=2e-5, atol=1e-6)
    x.close()


@pytest.mark.parametrize("members,index,n,dtype", [(2, 0, 5120, 0), (2, 1, 5121, 0), (8, 3, 5120, 1), (4, 0, 7, 0), (3, 2, 256 * 5120, 0)])
def test_sum_is_fp32_in_member_order_rounded_once(cuda, members, index, n, dtype):
    rng = np.random.default_rng(n + members)
    x = ext.Exchange(members, index, 2 * n)
    x.connect_alone()
    for call in range(2):
        parts = [to_bits(rng.standard_normal(n, dtype=np.float32), dtype) for _ in range(members)]
        t = [dev(cuda, p) for p in parts]
        for m in range(members):
            if m != index:
                x.deposit(m, t[m], 2 * n)
        out = cuda.zeros(n, dtype=cuda.int16, device="cuda")
        x.vector_sum(out, t[index], n, dtype, wait_ms=200)
        cuda.cuda.synchronize()
        assert ext.device_status() == 0
        s = np.zeros(n, np.float32)
        for p in parts:
            s += from_bits(p, dtype)
        assert np.array_equal(host_bits(out), to_bits(s, dtype)), f"call {call}"
    x.close()


def test_a_member_that_never_arrives_ends_the_wait_with_a_status(cuda):
    """Two members, and the other one never pushes: the kernel gives up after its limit, says so, writes nothing — and the
    object serves the next exchange."""
    qh, d = 8, 128
    rng = np.random.default_rng(5)
    x = ext.Exchange(2, 0, qh * (d + 2) * 4)
    x.connect_alone()
    mine, theirs = (dev(cuda, r) for r in residuals(rng, 2, qh, d))
    o = cuda.full((qh, d), 0x1234, dtype=cuda.int16, device="cuda")
    assert ext.device_status() == 0
    x.merge_finish(o, None, mine, qh, d, 0, wait_ms=20)
    cuda.cuda.synchronize()
    assert ext.device_status() == B2TO
    assert (o == 0x1234).all()
    assert ext.device_status() == 0                                         # reading cleared it
    part = cuda.zeros(5, dtype=cuda.int16, device="cuda")
    with pytest.raises(ext.B200Error):
        x.vector_sum(part, part, 4096, 0)                                   # more than a slot holds: refused, no exchange counted
    x.deposit(1, theirs, qh * (d + 2) * 4)
    x.merge_finish(o, None, mine, qh, d, 0, wait_ms=200)
    acc = mine.clone()
    ext.merge(acc, acc, theirs, qh, d)
    want = cuda.zeros((qh, d), dtype=cuda.int16, device="cuda")
    ext.finish(want, acc, qh, d, 0)
    cuda.cuda.synchronize()
    assert ext.device_status() == 0 and cuda.equal(o, want)
    x.close()


def test_refusals(cuda):
    with pytest.raises(ext.B200Error):
        ext.Exchange(9, 0, 1024)
    with pytest.raises(ext.B200Error):
        ext.Exchange(2, 2, 1024)
    x = ext.Exchange(2, 0, 1024)
    t = cuda.zeros(4096, dtype=cuda.float32, device="cuda")
    with pytest.raises(ext.B200Error) as e:
        x.merge_finish(t, None, t, 1, 128, 0)                               # not connected to its other member yet
    assert e.value.code == ext.E_STATE
    x.connect_addresses([0, x.local()[0]])                                  # (its own buffer stands in: only the wiring is under test)
    with pytest.raises(ext.B200Error):
        x.merge_finish(t, None, t, 8, 128, 0)                               # a residual larger than a slot
    with pytest.raises(ext.B200Error):
        x.deposit(0, t, 16)                                                 # a member does not deposit for itself
    x.close()


@pytest.mark.parametrize("members,index,width,rows,cols", [(2, 0, 4, 5120, 2048), (2, 1, 8, 5120, 1024), (4, 2, 4, 1000, 4096), (8, 7, 8, 2048, 512)])
def test_coded_projection_and_sum_in_one_launch(cuda, fam, port, members, index, width, rows, cols):
    """The output projection of a head-sharded mixer with the sum over the cards in its epilogue: this card's share of a coded
    matrix times its share of the input, pushed as the 16-bit partial the reference's turboquant_gemv would have written, the
    absent members' partials deposited; the bits must be those of the door followed by the exchange's vector_sum."""
    rng = np.random.default_rng(members * 10 + index + width)
    w = to_bits((rng.standard_normal((rows, cols)) / np.sqrt(cols * members)).astype(np.float32), 0)
    codes, scales = oracle.tq_encode_rows(port, w, width)
    vec = to_bits(rng.standard_normal(cols).astype(np.float32), 0)
    tc, ts, tv = dev(cuda, codes), dev(cuda, scales), dev(cuda, vec)
    others = {m: to_bits(rng.standard_normal(rows).astype(np.float32) * 0.5, 0) for m in range(members) if m != index}
    x = ext.Exchange(members, index, 2 * rows)
    x.connect_alone()
    # the unfused pair: the door, then the exchange's sum
    mine = cuda.zeros(rows, dtype=cuda.int16, device="cuda")
    fam.nn.turboquant_gemv(mine.data_ptr(), tc.data_ptr(), codes.nbytes, ts.data_ptr(), scales.nbytes, tv.data_ptr(), width, rows, cols, None)
    assert fam.sys.compute_completed()
    t_others = {m: dev(cuda, p) for m, p in others.items()}
    for m, t in t_others.items():
        x.deposit(m, t, 2 * rows)
    want = cuda.zeros(rows, dtype=cuda.int16, device="cuda")
    x.vector_sum(want, mine, rows, 0, wait_ms=200)
    for call in range(2):
        for m, t in t_others.items():
            x.deposit(m, t, 2 * rows, unit=2)
        got = cuda.full((rows,), 0x1234, dtype=cuda.int16, device="cuda")
        x.gemv_sum(got, tc, ts, tv, width, rows, cols, wait_ms=200)
        cuda.cuda.synchronize()
        assert ext.device_status() == 0
        assert cuda.equal(got, want), f"call {call}"
    # and against the checker: the restatement's gemv for this card, the members added in order
    s = np.zeros(rows, np.float32)
    part = {index: oracle.tq_gemv(port, codes, scales.view(np.uint8).copy(), vec, width, rows, cols), **others}
    for m in range(members):
        s += from_bits(part[m], 0)
    diff = np.abs(from_bits(host_bits(want), 0) - from_bits(to_bits(s, 0), 0))
    assert diff.max() <= 4e-3, diff.max()
    x.close()


@pytest.mark.parametrize("members,index,length,dtype", [(2, 0, 40000, 1), (2, 1, 131072, 1), (4, 2, 9000, 0), (2, 0, 3000, 1), (2, 1, 100, 0)])
def test_a_range_share_and_its_exchange_in_one_launch(cuda, members, index, length, dtype):
    """A member's share of a KV range split with every position on the card: the decode kernel's last block does the exchange
    step itself (one launch), and the answer has the bits of the decode followed by the exchange kernel wherever the two
    meet their splits the same way (long shares; a short share's separate decode meets in a cluster, and a share of one split
    has no meeting to ride on and takes the two launches)."""
    qh, kvh, d = 8, 1, 128
    rng = np.random.default_rng(length + index)
    mk = lambda shape, s: to_bits((rng.standard_normal(shape) * s).astype(np.float32), dtype)
    q, k, v = dev(cuda, mk((qh, d), 0.5)), dev(cuda, mk((length, kvh, d), 0.5)), dev(cuda, mk((length, kvh, d), 0.5))
    parts = residuals(rng, members, qh, d)
    t_parts = [dev(cuda, p) for p in parts]
    tier = ext.Tier(qh, kvh, d, dtype)
    # apart: the share's residual, then the exchange kernel
    mine = cuda.zeros((qh, d + 2), dtype=cuda.float32, device="cuda")
    tier.decode(None, mine, q, None, None, 0, k, v, length)
    x1 = ext.Exchange(members, index, qh * (d + 2) * 4)
    x1.connect_alone()
    for m in range(members):
        if m != index:
            x1.deposit(m, t_parts[m], parts[m].nbytes)
    o_want = cuda.zeros((qh, d), dtype=cuda.int16, device="cuda")
    r_want = cuda.zeros((qh, d + 2), dtype=cuda.float32, device="cuda")
    x1.merge_finish(o_want, r_want, mine, qh, d, dtype, wait_ms=200)
    # together
    x2 = ext.Exchange(members, index, qh * (d + 2) * 4)
    x2.connect_alone()
    for call in range(2):                                                  # twice: both parities of the slots
        for m in range(members):
            if m != index:
                x2.deposit(m, t_parts[m], parts[m].nbytes)
        o = cuda.full((qh, d), 0x1234, dtype=cuda.int16, device="cuda")
        r = cuda.zeros((qh, d + 2), dtype=cuda.float32, device="cuda")
        before = ext.counters()["launches"]
        tier.decode_exchange(x2, o, r, q, None, None, 0, k, v, length, wait_ms=200)
        cuda.cuda.synchronize()
        launches = ext.counters()["launches"] - before
        assert ext.device_status() == 0
        assert launches == (2 if length <= 128 else 1), launches
        if length >= 9000 or length <= 128:
            assert cuda.equal(o, o_want) and cuda.equal(r, r_want), f"call {call}"
        else:
            got, want = from_bits(host_bits(o), dtype), from_bits(host_bits(o_want), dtype)
            assert np.abs(got - want).max() <= 2e-3 * max(1.0, np.abs(want).max())
    # a member that never comes: the wait runs out, nothing is written, the status says so
    if length >= 9000:
        o = cuda.full((qh, d), 0x1234, dtype=cuda.int16, device="cuda")
        tier.decode_exchange(x2, o, None, q, None, None, 0, k, v, length, wait_ms=20)
        cuda.cuda.synchronize()
        assert ext.device_status() == B2TO and (o == 0x1234).all()
    x1.close(); x2.close(); tier.close()
