"""Host logic of the multi-GPU long-context path, on CPU: the shard plan, and the residual exchange + fold among the
ranks of a kv head over a real process group (gloo, world size 2) with the checker's merge standing in for the kernel."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

from silvann_b200 import sharded

ROOT = Path(__file__).resolve().parents[1]


def test_plan_by_heads_needs_no_exchange():
    for world in (1, 2, 4):
        plan = sharded.shard_plan(32, 4, 262144, world)
        assert len(plan) == world
        assert all(len(s.group) == 1 and (s.pos_lo, s.pos_hi) == (0, 262144) for s in plan)
        assert sorted(h for s in plan for h in range(s.kv_head_lo, s.kv_head_hi)) == [0, 1, 2, 3]
        assert sum(s.q_heads for s in plan) == 32
        for s in plan:
            assert (s.q_head_lo, s.q_head_hi) == (s.kv_head_lo * 8, s.kv_head_hi * 8)


def test_plan_splits_the_range_when_ranks_outnumber_kv_heads():
    plan = sharded.shard_plan(32, 4, 262144, 8)
    assert [(s.kv_head_lo, s.pos_lo, s.pos_hi) for s in plan] == [(h, p * 131072, (p + 1) * 131072) for h in range(4) for p in range(2)]
    assert [s.group for s in plan] == [[0, 1], [0, 1], [2, 3], [2, 3], [4, 5], [4, 5], [6, 7], [6, 7]]
    ragged = sharded.shard_plan(8, 1, 1000, 4)
    assert [(s.pos_lo, s.pos_hi) for s in ragged] == [(0, 256), (256, 512), (512, 768), (768, 1000)]
    tiny = sharded.shard_plan(8, 1, 200, 4)              # fewer tiles than ranks: the empty ranks are left out of the group
    assert [(s.pos_lo, s.pos_hi) for s in tiny] == [(0, 128), (128, 200), (200, 200), (200, 200)]
    assert tiny[0].group == [0, 1]


def test_plan_refusals():
    for args in [(32, 4, 100, 3), (32, 4, 100, 6), (30, 4, 100, 2), (32, 4, 0, 2)]:
        with pytest.raises(ValueError):
            sharded.shard_plan(*args)


def _rank_main(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist
    import oracle
    from silvann_b200 import sharded as sh
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    P = oracle.port()
    qh, kvh, d, L = 8, 1, 64, 1000
    rng = np.random.default_rng(3)
    q, k, v = (oracle.to_bits(rng.standard_normal(s, dtype=np.float32), 0) for s in ((qh, d), (L, kvh, d), (L, kvh, d)))
    shard = sh.shard_plan(qh, kvh, L, world)[rank]
    mine = P.residual(q, np.ascontiguousarray(k[shard.pos_lo:shard.pos_hi]), np.ascontiguousarray(v[shard.pos_lo:shard.pos_hi]), qh, kvh, d, shard.positions)
    merge = lambda a, b: torch.from_numpy(P.merge(a.numpy(), b.numpy(), qh, d))
    total = sh.gather_and_fold(torch.from_numpy(mine), shard, dist, merge)
    o, _ = P.finish(total.numpy(), qh, d)
    np.save(Path(tmp) / f"o{rank}.npy", o)
    if rank == 0:
        whole = P.residual(q, k, v, qh, kvh, d, L)
        np.save(Path(tmp) / "want.npy", whole[:, 2:] / whole[:, 1:2])
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_exchange_and_fold_over_gloo(tmp_path):
    import torch.multiprocessing as mp
    port = 29500 + os.getpid() % 2000
    mp.spawn(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    import oracle
    o0, o1 = np.load(tmp_path / "o0.npy"), np.load(tmp_path / "o1.npy")
    assert np.array_equal(o0, o1)                                        # every rank of the group folds the same bits
    assert np.abs(oracle.from_bits(o0, 0) - np.load(tmp_path / "want.npy")).max() <= 2e-3


def _sum_main(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist
    import oracle
    from silvann_b200 import sharded as sh
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n = 5120
    parts = [oracle.to_bits(np.random.default_rng(40 + r).standard_normal(n, dtype=np.float32), 0) for r in range(world)]

    def vector_sum(pieces):                                  # the door's arithmetic: fp32 in the order given, rounded once
        s = np.zeros(n, np.float32)
        for p in pieces:
            s += oracle.from_bits(p.numpy().view(np.uint16), 0)
        return torch.from_numpy(oracle.to_bits(s, 0).view(np.int16))
    total = sh.sum_over_ranks(torch.from_numpy(parts[rank].view(np.int16)), dist, vector_sum)
    np.save(Path(tmp) / f"s{rank}.npy", total.numpy().view(np.uint16))
    if rank == 0:
        s = np.zeros(n, np.float32)
        for p in parts:
            s += oracle.from_bits(p, 0)
        np.save(Path(tmp) / "want.npy", oracle.to_bits(s, 0))
    dist.barrier()
    dist.destroy_process_group()


def test_partial_sums_over_two_ranks_are_the_same_bits_everywhere(tmp_path):
    import torch.multiprocessing as mp
    port = 31500 + os.getpid() % 2000
    mp.spawn(_sum_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    s0, s1, want = (np.load(tmp_path / f) for f in ("s0.npy", "s1.npy", "want.npy"))
    assert np.array_equal(s0, s1) and np.array_equal(s0, want)


class _FakeExchange:
    """Stands in for ext.Exchange on a machine without a GPU: a handle that says whose it is, and a record of the wiring."""
    def __init__(self, members, index, slot_bytes):
        self.members, self.index, self.slot_bytes, self.wired = members, index, slot_bytes, None
        self.me = int(os.environ["RANK_FOR_FAKE"])

    def ipc_handle(self):
        return bytes([self.me]) * 64

    def connect_handles(self, handles):
        self.wired = [h[0] for h in handles]


class _FakeExt:
    Exchange = _FakeExchange


def _wire_main(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist
    from silvann_b200 import sharded as sh
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK_FOR_FAKE=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    shard = sh.shard_plan(8, 1, 1000, world)[rank]                 # one kv head over two ranks: a range split, group [0, 1]
    x = sh.connect_exchange(torch, _FakeExt, dist, shard.group, rank, 8 * 66 * 4)
    alone = sh.connect_exchange(torch, _FakeExt, dist, [rank], rank, 64)       # a rank without partners still takes part in the gather
    np.save(Path(tmp) / f"w{rank}.npy", np.array([x.members, x.index] + x.wired + [alone.members, -1 if alone.wired is None else 1]))

    calls = []

    class Tier:
        def __init__(self, *a): pass
        def decode(self, *a): calls.append("decode")
        def decode_exchange(self, ex, *a): calls.append(("decode_exchange", ex is x))
        def close(self): pass

    class Ext:
        pass
    Ext.Tier = Tier

    class Torch:
        float32, int16 = None, None
        @staticmethod
        def zeros(*a, **k): return None
    runner = sh.LongContextRank(Torch, Ext, shard, 64, 0, None, None, 0, None, None, shard.positions, dist, None, exchange=x)
    runner.step(None)
    lone = sh.LongContextRank(Torch, Ext, sh.shard_plan(8, 2, 1000, world)[rank], 64, 0, None, None, 0, None, None, 1000, dist, None, exchange=None)
    lone.step(None)
    assert calls == [("decode_exchange", True), "decode"], calls
    dist.barrier()
    dist.destroy_process_group()


def test_exchange_handles_reach_the_members_of_a_group_over_gloo(tmp_path):
    """The one-time wiring of the exchange: every rank's buffer handle gathered over the world, each rank connecting the
    handles of ITS group in group order; and the step's dispatch — a rank in a range split makes one decode_exchange call, a
    rank alone on its heads one decode call."""
    import torch.multiprocessing as mp
    port = 33500 + os.getpid() % 2000
    mp.spawn(_wire_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    w0, w1 = np.load(tmp_path / "w0.npy"), np.load(tmp_path / "w1.npy")
    assert list(w0) == [2, 0, 0, 1, 1, -1] and list(w1) == [2, 1, 0, 1, 1, -1]
