"""Two cards in ONE process, as the reference's engine drives them (a worker thread a card, one shared door table,
engine/src/packages/nn/cpu/opcodes/partials__abi.cuh:110-163): the doors that cross cards read a peer's memory with plain
loads.  `vector_sum` adds partial results that live on two cards (the tensor-parallel sum that follows head-sharded
attention); a long cache split by position has each card attend its range into a residual, and one card merges its own
residual with the peer's through `attention_merge` and finishes — the reference's residual arithmetic as the wire format.
Skipped where fewer than two B200s are visible."""
import numpy as np
import pytest

import oracle
from oracle import FP16, from_bits, to_bits
from util import assert_close16

pytestmark = pytest.mark.gpu


@pytest.fixture()
def two(cuda, fam):
    if fam.sys.device_count() < 2:
        pytest.skip("one card visible")
    assert fam.sys.bind_device(0) == 1 and fam.sys.peer_access(1)
    assert fam.sys.bind_device(1) == 1 and fam.sys.peer_access(0)
    yield fam
    fam.sys.bind_device(0)
    cuda.cuda.set_device(0)


def on(cuda, fam, index, array):
    """`array` (numpy) on card `index`, through the family's own bind."""
    assert fam.sys.bind_device(index) == 1
    cuda.cuda.set_device(index)
    a = np.ascontiguousarray(array)
    view = {np.dtype(np.uint16): np.int16, np.dtype(np.uint32): np.int32}.get(a.dtype)
    return cuda.from_numpy(a.view(view) if view else a).to(f"cuda:{index}")


def test_partial_sums_across_cards(cuda, two, port):
    fam = two
    n = 5120
    rng = np.random.default_rng(31)
    parts = [to_bits(rng.standard_normal(n).astype(np.float32), FP16) for _ in range(2)]
    t = [on(cuda, fam, i, parts[i]) for i in range(2)]
    assert fam.sys.bind_device(0) == 1
    cuda.cuda.set_device(0)
    out = cuda.zeros(n, dtype=cuda.int16, device="cuda:0")

    from silvann_b200.abi import VectorParts
    p = VectorParts()
    p.at[0], p.at[1], p.count = t[0].data_ptr(), t[1].data_ptr(), 2
    fam.nn.vector_sum(out.data_ptr(), p, n, None)
    assert fam.sys.compute_completed()
    want = to_bits(from_bits(parts[0], FP16) + from_bits(parts[1], FP16), FP16)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want)


def test_one_cache_split_by_position_over_two_cards(cuda, two, reference, port):
    fam = two
    impl = reference if reference is not None else port
    qh, kvh, d, n, cut = 16, 4, 128, 6000, 3072
    rng = np.random.default_rng(32)
    q = to_bits(rng.standard_normal((qh, d)).astype(np.float32) * 0.5, FP16)
    k = to_bits(rng.standard_normal((n, kvh, d)).astype(np.float32) * 0.5, FP16)
    v = to_bits(rng.standard_normal((n, kvh, d)).astype(np.float32) * 0.5, FP16)
    spans = [(0, cut), (cut, n)]
    res = []
    for i, (lo, hi) in enumerate(spans):
        tq, tk, tv = on(cuda, fam, i, q), on(cuda, fam, i, k[lo:hi]), on(cuda, fam, i, v[lo:hi])
        p = cuda.zeros((qh, hi - lo), dtype=cuda.float32, device=f"cuda:{i}")
        r = cuda.zeros((qh, d + 2), dtype=cuda.float32, device=f"cuda:{i}")
        fam.nn.attention_weights(p.data_ptr(), r.data_ptr(), tq.data_ptr(), tk.data_ptr(), qh, kvh, d, hi - lo)
        fam.nn.attention_residual_mix(r.data_ptr(), p.data_ptr(), tv.data_ptr(), qh, kvh, d, hi - lo)
        assert fam.sys.compute_completed()
        res.append((r, p, tq, tk, tv))
    # card 0 merges its residual with card 1's, read in place over the link, and finishes
    assert fam.sys.bind_device(0) == 1
    cuda.cuda.set_device(0)
    o = cuda.zeros((qh, d), dtype=cuda.int16, device="cuda:0")
    fam.nn.attention_merge(res[0][0].data_ptr(), res[0][0].data_ptr(), res[1][0].data_ptr(), qh, d)
    fam.nn.attention_finish(o.data_ptr(), res[0][0].data_ptr(), qh, d, None)
    assert fam.sys.compute_completed()
    want = impl.decode(q, k, v, qh, kvh, d, n)
    assert_close16(o.cpu().numpy().view(np.uint16), from_bits(want, FP16), FP16, "two ranges on two cards, merged over the link")


def test_exchange_between_two_cards_of_one_process(cuda, two, port):
    """The exchange kernels with both members REAL: one process, a card each, the members wired by address (peer access is
    granted by the fixture).  Both launches are queued before either is waited for; each card waits on the device for the
    other's push.  Range residuals are folded, then partial sums added — the same object, consecutive generations."""
    from silvann_b200 import ext
    fam = two
    qh, kvh, d, n, cut = 16, 4, 128, 6000, 3072
    rng = np.random.default_rng(33)
    q = to_bits(rng.standard_normal((qh, d)).astype(np.float32) * 0.5, FP16)
    k = to_bits(rng.standard_normal((n, kvh, d)).astype(np.float32) * 0.5, FP16)
    v = to_bits(rng.standard_normal((n, kvh, d)).astype(np.float32) * 0.5, FP16)
    hidden = 5120
    parts = [to_bits(rng.standard_normal(hidden).astype(np.float32), FP16) for _ in range(2)]
    xs, res, outs, sums, tparts = [], [], [], [], []
    for i, (lo, hi) in enumerate([(0, cut), (cut, n)]):
        tq, tk, tv = on(cuda, fam, i, q), on(cuda, fam, i, k[lo:hi]), on(cuda, fam, i, v[lo:hi])
        r = cuda.zeros((qh, d + 2), dtype=cuda.float32, device=f"cuda:{i}")
        ext.decode(None, r, tq, tk, tv, qh, kvh, d, hi - lo, 0)
        cuda.cuda.synchronize()
        res.append(r)
        outs.append(cuda.zeros((qh, d), dtype=cuda.int16, device=f"cuda:{i}"))
        sums.append(cuda.zeros(hidden, dtype=cuda.int16, device=f"cuda:{i}"))
        tparts.append(on(cuda, fam, i, parts[i]))
        xs.append(ext.Exchange(2, i, max(qh * (d + 2) * 4, 2 * hidden)))
    addresses = [x.local()[0] for x in xs]
    for i in range(2):
        assert fam.sys.bind_device(i) == 1
        cuda.cuda.set_device(i)
        xs[i].connect_addresses(addresses)
    for step in ("fold", "sum"):
        for i in range(2):
            assert fam.sys.bind_device(i) == 1
            cuda.cuda.set_device(i)
            if step == "fold":
                xs[i].merge_finish(outs[i], None, res[i], qh, d, 0, wait_ms=2000)
            else:
                xs[i].vector_sum(sums[i], tparts[i], hidden, 0, wait_ms=2000)
        for i in range(2):
            cuda.cuda.synchronize(i)
    for i in range(2):
        assert fam.sys.bind_device(i) == 1
        cuda.cuda.set_device(i)
        assert ext.device_status() == 0
    want = port.residual(q, k, v, qh, kvh, d, n, 0)
    assert cuda.equal(outs[0].cpu(), outs[1].cpu())
    assert_close16(outs[0].cpu().numpy().view(np.uint16), want[:, 2:] / want[:, 1:2], FP16, "two ranges folded by the exchange kernel")
    total = to_bits(from_bits(parts[0], FP16) + from_bits(parts[1], FP16), FP16)
    assert np.array_equal(sums[0].cpu().numpy().view(np.uint16), total) and np.array_equal(sums[1].cpu().numpy().view(np.uint16), total)
    for i in range(2):
        assert fam.sys.bind_device(i) == 1
        cuda.cuda.set_device(i)
        xs[i].close()
