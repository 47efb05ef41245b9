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
    table = dev(cuda, np.maximum(L.page_table, 0))
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
