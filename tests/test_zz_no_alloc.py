"""The allocation-free decode entry point, silvann_b200_decode_noalloc, through the C boundary.

Some hosts cannot let a library allocate: SiLVANN commits the card's memory to its own pools at boot, and a host that
records its work into a stream capture cannot have cudaMalloc appear in the middle of it.  For them the split-KV decode
exists once more with its scratch in a fixed array inside the library.  This file checks that it answers what the
ordinary entry point answers — twice in a row, because the second call finds the first call's leftovers in the shared
scratch — that it really allocates nothing, and that it refuses what does not fit.

It is named to be collected last: a run that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest

import oracle
from oracle import to_bits
from silvann_b200 import ext
from util import dev, host_bits

pytestmark = pytest.mark.gpu

CASES = [  # q_heads, kv_heads, head_dim, length, dtype
    (16, 4, 128, 8192, 0),
    (16, 2, 256, 5000, 1),
    (32, 4, 128, 70000, 1),
    (8, 8, 64, 100, 0),
]


def make(cuda, qh, kvh, d, L, dtype, seed):
    rng = np.random.default_rng(seed)
    mk = lambda s: dev(cuda, to_bits(rng.standard_normal(s, dtype=np.float32), dtype))
    return mk((qh, d)), mk((L, kvh, d)), mk((L, kvh, d))


@pytest.mark.parametrize("qh,kvh,d,L,dtype", CASES)
def test_same_answer_as_the_allocating_entry_point_twice_in_a_row(cuda, port, qh, kvh, d, L, dtype):
    first = None
    for call in range(2):
        q, k, v = make(cuda, qh, kvh, d, L, dtype, 40 + call)       # different inputs each call: leftovers would show
        want_o = cuda.zeros((qh, d), dtype=cuda.int16, device="cuda")
        want_res = cuda.zeros((qh, d + 2), dtype=cuda.float32, device="cuda")
        ext.decode(want_o, want_res, q, k, v, qh, kvh, d, L, dtype)
        got_o = cuda.zeros((qh, d), dtype=cuda.int16, device="cuda")
        got_res = cuda.zeros((qh, d + 2), dtype=cuda.float32, device="cuda")
        ext.decode_noalloc(got_o, got_res, q, k, v, qh, kvh, d, L, dtype)
        cuda.cuda.synchronize()
        got, want = oracle.from_bits(host_bits(got_o), dtype), oracle.from_bits(host_bits(want_o), dtype)
        assert np.isfinite(got).all()
        # the two entry points may cut the cache into a different number of splits, so the bar is the decode tests' own
        # tolerance (2e-3, or half an output ulp of bf16 where that is larger), not bit equality
        ulp = (2.0 ** -8 if dtype else 2.0 ** -11) * np.maximum(np.abs(want), 2.0 ** -14)
        assert (np.abs(got - want) <= np.maximum(2e-3, ulp)).all(), f"call {call}: max abs diff {np.abs(got - want).max()}"
        rg, rw = got_res.cpu().numpy(), want_res.cpu().numpy()
        np.testing.assert_allclose(rg[:, 2:] / rg[:, 1:2], rw[:, 2:] / rw[:, 1:2], rtol=0, atol=1e-3)
        np.testing.assert_allclose(rg[:, 0], rw[:, 0], rtol=0, atol=1e-4)
        if L <= 8192:                                               # and once against the CPU checker itself
            r = port.residual(host_bits(q), host_bits(k), host_bits(v), qh, kvh, d, L, dtype)
            assert (np.abs(got - r[:, 2:] / r[:, 1:2]) <= np.maximum(2e-3, 2 * ulp)).all(), f"call {call}: against the checker"
        if first is not None:
            assert not np.array_equal(first, host_bits(got_o))      # the second call really computed its own inputs
        first = host_bits(got_o).copy()
    # this entry point's time-out word lives in its own fixed array; device_status reads that word too
    assert ext.device_status() == 0


def test_it_allocates_nothing(cuda):
    qh, kvh, d, L = 16, 4, 128, 4096
    q, k, v = make(cuda, qh, kvh, d, L, 0, 7)
    o = cuda.zeros((qh, d), dtype=cuda.int16, device="cuda")
    ext.decode_noalloc(o, None, q, k, v, qh, kvh, d, L, 0)          # first call on the device: address lookup only
    cuda.cuda.synchronize()
    free0, _ = cuda.cuda.mem_get_info()
    for _ in range(20):
        ext.decode_noalloc(o, None, q, k, v, qh, kvh, d, L, 0)
    cuda.cuda.synchronize()
    free1, _ = cuda.cuda.mem_get_info()
    assert free1 == free0


def test_explicit_splits_and_refusals(cuda):
    qh, kvh, d, L = 16, 4, 128, 38912            # 304 tiles of 128 positions = 76 splits of 4 tiles
    q, k, v = make(cuda, qh, kvh, d, L, 0, 9)
    want = cuda.zeros((qh, d), dtype=cuda.int16, device="cuda")
    got = cuda.zeros((qh, d), dtype=cuda.int16, device="cuda")
    ext.decode(want, None, q, k, v, qh, kvh, d, L, 0, nsplit=76)
    ext.decode_noalloc(got, None, q, k, v, qh, kvh, d, L, 0, nsplit=76)      # 76 x 4 = 304 slots: exactly the ceiling
    cuda.cuda.synchronize()
    assert np.array_equal(host_bits(got), host_bits(want))                    # same splits, same bits
    with pytest.raises(ext.B200Error) as e:
        ext.decode_noalloc(got, None, q, k, v, qh, kvh, d, L, 0, nsplit=152)  # 152 splits of 2 tiles x 4 kv heads = 608 slots
    assert e.value.code == ext.E_ARGUMENT and "304" in str(e.value)
    with pytest.raises(ext.B200Error):
        ext.decode_noalloc(got, None, q, k, v, qh, kvh, 96, L, 0)            # outside the kernel's fit
    with pytest.raises(ext.B200Error):
        ext.decode_noalloc(None, None, q, k, v, qh, kvh, d, L, 0)            # nowhere to put the answer
