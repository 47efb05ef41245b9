"""The tensor-parallel partial sum with one PROCESS a card (NCCL between them): every rank gathers the others' 16-bit
partials and adds them in rank order through the family's `vector_sum` door — the same bits on every rank, and the bits
the fp32-sum-rounded-once definition gives.  Skipped where fewer than two B200s are visible."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def _rank(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    import oracle
    import silvann_b200
    from silvann_b200 import sharded
    torch.cuda.set_device(rank)
    fam = silvann_b200.family()
    assert fam.sys.bind_device(rank) == 1
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    n = 5120
    parts = [oracle.to_bits(np.random.default_rng(60 + r).standard_normal(n, dtype=np.float32), 0) for r in range(world)]
    mine = torch.from_numpy(parts[rank].view(np.int16)).cuda()
    total = sharded.sum_over_ranks(mine, dist, sharded.family_vector_sum(torch, fam))
    assert fam.sys.compute_completed()
    np.save(Path(tmp) / f"s{rank}.npy", total.cpu().numpy().view(np.uint16))
    # the same sum as one launch a rank over peer memory, twice (both parities of the exchange)
    from silvann_b200 import ext
    peer = sharded.PeerSum(torch, ext, dist, n, 0)
    for _ in range(2):
        pushed = peer.sum(mine, wait_ms=5000)
    torch.cuda.synchronize()
    assert ext.device_status() == 0
    np.save(Path(tmp) / f"p{rank}.npy", pushed.cpu().numpy().view(np.uint16))
    # the same sum with its producer: each rank's share of a coded output projection, the partials exchanged in the epilogue
    rows, cols, width = 5120, 1024, 4
    P = oracle.port()
    grng = np.random.default_rng(80 + rank)
    codes, scales = oracle.tq_encode_rows(P, oracle.to_bits((grng.standard_normal((rows, cols)) / np.sqrt(cols * world)).astype(np.float32), 0), width)
    vec = oracle.to_bits(grng.standard_normal(cols).astype(np.float32), 0)
    up16 = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16 if a.dtype == np.uint16 else np.uint8)).cuda()
    tc, ts, tv = up16(codes), up16(scales), up16(vec)
    fused = torch.zeros(rows, dtype=torch.int16, device="cuda")
    for _ in range(2):
        peer.exchange.gemv_sum(fused, tc, ts, tv, width, rows, cols, wait_ms=5000)
    part = torch.zeros(rows, dtype=torch.int16, device="cuda")
    fam.nn.turboquant_gemv(part.data_ptr(), tc.data_ptr(), codes.nbytes, ts.data_ptr(), scales.nbytes, tv.data_ptr(), width, rows, cols, None)
    assert fam.sys.compute_completed()
    unfused = peer.sum(part, wait_ms=5000)
    torch.cuda.synchronize()
    assert ext.device_status() == 0
    assert torch.equal(fused, unfused), "the fused projection + sum differs from the door followed by the sum"
    np.save(Path(tmp) / f"g{rank}.npy", fused.cpu().numpy().view(np.uint16))
    # and a KV range split over the two ranks: each attends its half, the exchange kernel folds
    qh, kvh, d, L = 8, 1, 128, 4096
    rng = np.random.default_rng(70)
    q, k, v = (oracle.to_bits(rng.standard_normal(s, dtype=np.float32), 0) for s in ((qh, d), (L, kvh, d), (L, kvh, d)))
    shard = sharded.shard_plan(qh, kvh, L, world)[rank]
    x = sharded.connect_exchange(torch, ext, dist, shard.group, rank, qh * (d + 2) * 4)
    up = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda()
    runner = sharded.LongContextRank(torch, ext, shard, d, 0, None, None, 0, up(k[shard.pos_lo:shard.pos_hi]), up(v[shard.pos_lo:shard.pos_hi]), shard.positions,
                                     dist, None, exchange=x)
    for _ in range(2):
        o = runner.step(up(q))
    torch.cuda.synchronize()
    assert ext.device_status() == 0
    np.save(Path(tmp) / f"o{rank}.npy", o.cpu().numpy().view(np.uint16))
    if rank == 0:
        r = oracle.port().residual(q, k, v, qh, kvh, d, L, 0)
        np.save(Path(tmp) / "o_want.npy", r[:, 2:] / r[:, 1:2])
    dist.barrier()
    runner.close(); x.close(); peer.close()
    if rank == 0:
        s = np.zeros(n, np.float32)
        for p in parts:
            s += oracle.from_bits(p, 0)
        np.save(Path(tmp) / "want.npy", oracle.to_bits(s, 0))
    dist.barrier()
    dist.destroy_process_group()


def test_partial_sums_over_two_processes(cuda, tmp_path):
    if cuda.cuda.device_count() < 2:
        pytest.skip("one card visible")
    import torch.multiprocessing as mp
    port = 32500 + os.getpid() % 2000
    mp.spawn(_rank, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    s0, s1, want = (np.load(tmp_path / f) for f in ("s0.npy", "s1.npy", "want.npy"))
    assert np.array_equal(s0, s1) and np.array_equal(s0, want)
    assert np.array_equal(np.load(tmp_path / "g0.npy"), np.load(tmp_path / "g1.npy"))
    p0, p1 = np.load(tmp_path / "p0.npy"), np.load(tmp_path / "p1.npy")
    assert np.array_equal(p0, want) and np.array_equal(p1, want)
    import oracle
    o0, o1, o_want = np.load(tmp_path / "o0.npy"), np.load(tmp_path / "o1.npy"), np.load(tmp_path / "o_want.npy")
    assert np.array_equal(o0, o1) and np.abs(oracle.from_bits(o0, 0) - o_want).max() <= 2e-3
