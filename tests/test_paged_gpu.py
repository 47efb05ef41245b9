"""Batched decode over the paged pool (configuration 3) against the reference path: gather a sequence's pages into the
contiguous planes the reference doors take, then attention_scores + attention_mix per sequence."""
import numpy as np
import pytest

import oracle
from oracle import from_bits
from silvann_b200 import ext, workloads
from util import assert_close16, dev, host_bits

pytestmark = pytest.mark.gpu


def run_paged(cuda, layout, q, k_pool, v_pool, blocks_target=0):
    L = layout
    plan = ext.Plan()
    plan.plan(L.seq_lens, L.q_heads, L.kv_heads, L.head_dim, blocks_target)
    seqs = len(L.seq_lens)
    o = cuda.zeros((seqs, L.q_heads, L.head_dim), dtype=cuda.int16, device="cuda")
    res = cuda.zeros((seqs, L.q_heads, L.head_dim + 2), dtype=cuda.float32, device="cuda")
    table = dev(cuda, L.page_table)                  # the -1 padding goes to the card as it is
    plan.decode(o, res, dev(cuda, q), dev(cuda, k_pool), dev(cuda, v_pool), L.pool_pages, workloads.PAGE_POSITIONS,
                table, L.page_table.shape[1], L.dtype)
    cuda.cuda.synchronize()
    assert ext.device_status() == 0
    info = plan.info()
    plan.close()
    return host_bits(o), res.cpu().numpy(), info


@pytest.mark.parametrize("blocks_target", [0, 8, 4000])
def test_small_batch_against_the_oracle(cuda, port, blocks_target):
    L = workloads.config3_layout(seqs=6, lo=1, hi=2500)
    L.seq_lens[0] = 1; L.seq_lens[1] = 256; L.seq_lens[2] = 257          # page-boundary cases
    q, k_pool, v_pool = workloads.config3_fill(L)
    o, res, info = run_paged(cuda, L, q, k_pool, v_pool, blocks_target)
    assert info["positions"] == L.positions
    for s in range(len(L.seq_lens)):
        n = int(L.seq_lens[s])
        ks, vs = workloads.gather_sequence(L, k_pool, s), workloads.gather_sequence(L, v_pool, s)
        want_res = port.residual(q[s], ks, vs, L.q_heads, L.kv_heads, L.head_dim, n, L.dtype)
        want = want_res[:, 2:] / want_res[:, 1:2]
        assert_close16(o[s], want, L.dtype, f"sequence {s} of {n}")
        np.testing.assert_allclose(res[s][:, 2:] / res[s][:, 1:2], want, rtol=0, atol=1e-3)


def test_config3_shape_at_one_eighth_against_the_reference(cuda, port, reference):
    """32 sequences, 16 q heads on 2 kv heads, head_dim 256, bf16 values that fp16 holds exactly, a permuted pool —
    lengths an eighth of the benchmark's so the CPU side stays in seconds."""
    L = workloads.config3_layout(seqs=32, lo=128, hi=12500)
    q, k_pool, v_pool = workloads.config3_fill(L)
    o, _, info = run_paged(cuda, L, q, k_pool, v_pool)
    assert info["blocks"] >= 148
    for s in range(0, 32, 3):
        n = int(L.seq_lens[s])
        ks, vs = workloads.gather_sequence(L, k_pool, s), workloads.gather_sequence(L, v_pool, s)
        if reference is not None:       # the same real numbers as fp16 bits for the reference (it has no bf16)
            to16 = lambda b: oracle.to_bits(oracle.from_bits(b, 1), 0)
            res = reference.residual(to16(q[s]), to16(ks), to16(vs), L.q_heads, L.kv_heads, L.head_dim, n)
        else:
            res = port.residual(q[s], ks, vs, L.q_heads, L.kv_heads, L.head_dim, n, 1)
        assert_close16(o[s], res[:, 2:] / res[:, 1:2], 1, f"sequence {s} of {n}")


def test_page_order_does_not_matter(cuda):
    """Size-independent property: permuting which pool page holds which rows leaves every output bit unchanged."""
    L = workloads.config3_layout(seqs=8, lo=300, hi=6000)
    q, k_pool, v_pool = workloads.config3_fill(L)
    o1, _, _ = run_paged(cuda, L, q, k_pool, v_pool)
    rng = np.random.default_rng(5)
    perm = rng.permutation(L.pool_pages).astype(np.int32)          # old page i moves to new page perm[i]
    k2, v2 = np.empty_like(k_pool), np.empty_like(v_pool)
    k2[perm], v2[perm] = k_pool, v_pool
    L2 = workloads.PagedLayout(L.seq_lens, np.where(L.page_table >= 0, perm[np.maximum(L.page_table, 0)], -1).astype(np.int32),
                               L.pool_pages, L.q_heads, L.kv_heads, L.head_dim, L.dtype)
    o2, _, _ = run_paged(cuda, L2, q, k2, v2)
    assert np.array_equal(o1, o2)


def test_plan_refusals(cuda):
    plan = ext.Plan()
    with pytest.raises(ext.B200Error):
        plan.plan([10, 0, 5], 16, 2, 256)                  # an empty sequence
    with pytest.raises(ext.B200Error):
        plan.plan([10], 16, 3, 256)                        # heads do not divide
    with pytest.raises(ext.B200Error) as e:
        plan.info()
    assert e.value.code == ext.E_STATE
    plan.plan([10], 16, 2, 256)
    t = cuda.zeros(16 * 256, dtype=cuda.int16, device="cuda")
    with pytest.raises(ext.B200Error):
        plan.decode(t, None, t, t, t, 1, 100, t, 1, 1)     # page size not a multiple of 64
    plan.close()


def test_append_writes_each_sequences_newest_row_and_nothing_else(cuda):
    L = workloads.config3_layout(seqs=5, lo=1, hi=900)
    L.seq_lens[0] = 1; L.seq_lens[1] = 256; L.seq_lens[2] = 257
    q, k_pool, v_pool = workloads.config3_fill(L)
    row = L.kv_heads * L.head_dim
    rng = np.random.default_rng(8)
    k_rows = oracle.to_bits(rng.standard_normal((5, row), dtype=np.float32), 1)
    v_rows = oracle.to_bits(rng.standard_normal((5, row), dtype=np.float32), 1)
    plan = ext.Plan()
    plan.plan(L.seq_lens, L.q_heads, L.kv_heads, L.head_dim)
    tk, tv = dev(cuda, k_pool), dev(cuda, v_pool)
    plan.append(tk, tv, dev(cuda, k_rows), dev(cuda, v_rows), L.pool_pages, workloads.PAGE_POSITIONS, dev(cuda, L.page_table), L.page_table.shape[1])
    cuda.cuda.synchronize()
    assert ext.device_status() == 0
    want_k, want_v = k_pool.copy(), v_pool.copy()
    for s, n in enumerate(L.seq_lens):
        page, at = L.page_table[s, (int(n) - 1) // 256], (int(n) - 1) % 256
        want_k[page, at] = k_rows[s].reshape(L.kv_heads, L.head_dim)
        want_v[page, at] = v_rows[s].reshape(L.kv_heads, L.head_dim)
    assert np.array_equal(host_bits(tk).reshape(want_k.shape), want_k) and np.array_equal(host_bits(tv).reshape(want_v.shape), want_v)
    plan.close()


def test_a_table_that_names_no_page_is_never_made_into_an_address(cuda):
    """A short table is refused on the host; an entry outside the pool is skipped on the card and the status word says so."""
    L = workloads.config3_layout(seqs=3, lo=300, hi=900)
    q, k_pool, v_pool = workloads.config3_fill(L)
    plan = ext.Plan()
    plan.plan(L.seq_lens, L.q_heads, L.kv_heads, L.head_dim)
    seqs, stride = 3, L.page_table.shape[1]
    o = cuda.zeros((seqs, L.q_heads, L.head_dim), dtype=cuda.int16, device="cuda")
    tq, tk, tv, tt = dev(cuda, q), dev(cuda, k_pool), dev(cuda, v_pool), dev(cuda, L.page_table)
    with pytest.raises(ext.B200Error) as e:
        plan.decode(o, None, tq, tk, tv, L.pool_pages, 256, tt, 1, 1)                         # rows of one column for sequences of several pages
    assert e.value.code == ext.E_ARGUMENT
    rows = cuda.zeros((2, seqs, L.kv_heads * L.head_dim), dtype=cuda.int16, device="cuda")
    with pytest.raises(ext.B200Error):
        plan.append(tk, tv, rows[0], rows[1], L.pool_pages, 256, tt, 1)
    bad = L.page_table.copy()
    last = (int(L.seq_lens[1]) - 1) // 256
    bad[1, last] = L.pool_pages + 7                                                              # sequence 1's newest page: outside the pool
    before = host_bits(tk).copy()
    plan.append(tk, tv, rows[0], rows[1], L.pool_pages, 256, dev(cuda, bad), stride)
    cuda.cuda.synchronize()
    assert ext.device_status() == 0x80000000
    after = host_bits(tk).reshape(k_pool.shape)
    changed = np.flatnonzero((after != before.reshape(k_pool.shape)).any(axis=(1, 2, 3)))
    assert set(changed) <= {int(L.page_table[0, (int(L.seq_lens[0]) - 1) // 256]), int(L.page_table[2, (int(L.seq_lens[2]) - 1) // 256])}
    bad[1, last] = -1
    plan.decode(o, None, tq, tk, tv, L.pool_pages, 256, dev(cuda, bad), stride, 1)              # read as zeros, flagged, no fault
    cuda.cuda.synchronize()
    assert ext.device_status() == 0x80000000
    assert ext.device_status() == 0
    plan.close()
