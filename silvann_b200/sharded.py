"""One long sequence over several GPUs: which rank attends what, and how the pieces meet.

The reference shards a model over cards by heads — each card gets a table with its share of the heads, and the
attention doors never know (runtime/silvann_runtime/qwen3_5.py:112-134) — and replicates a kv head when there are more
cards than kv heads.  Here a replicated kv head is put to work instead: the ranks that share it split its KV RANGE, each
produces the residual (m, l, acc) of its range with the same decode kernel, and the residuals are folded with the
reference's merge arithmetic (engine/src/packages/nn/gpu/kernels/kernels.cuh:1243-1255).  The residual is the wire
format: q_heads_local * (head_dim + 2) floats a rank.  On GPUs the exchange is the library's own kernel over peer memory
(push, signal, bounded wait, fold in range order: one launch a rank, connect_exchange wires the ranks once); under gloo in
the CPU tests it is one small all-gather and a fold here.  There is no exchange at all while ranks <= kv heads.

This module is host logic only: it decides shards and drives the exchange; arithmetic is the library's (ext.merge,
ext.finish), injected so that the plumbing can be exercised without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field

RANGE_ALIGN = 128     # a rank's range starts on a multiple of the decode kernel's largest tile


@dataclass
class Shard:
    rank: int
    kv_head_lo: int
    kv_head_hi: int
    q_head_lo: int
    q_head_hi: int
    pos_lo: int
    pos_hi: int
    group: list = field(default_factory=list)   # the ranks that share these heads, in range order (len 1: no exchange)

    @property
    def kv_heads(self) -> int:
        return self.kv_head_hi - self.kv_head_lo

    @property
    def q_heads(self) -> int:
        return self.q_head_hi - self.q_head_lo

    @property
    def positions(self) -> int:
        return self.pos_hi - self.pos_lo


def shard_plan(q_heads: int, kv_heads: int, length: int, world: int) -> list[Shard]:
    """Every rank's share of one sequence of `length` cached positions.

    world <= kv_heads: whole kv heads per rank (kv_heads must divide evenly), full range, no exchange.
    world >  kv_heads: world / kv_heads ranks per kv head, each a contiguous range of positions cut on multiples of 128.
    """
    if q_heads <= 0 or kv_heads <= 0 or q_heads % kv_heads or length <= 0 or world <= 0:
        raise ValueError(f"shard_plan: {q_heads} query heads, {kv_heads} kv heads, {length} positions, {world} ranks")
    group = q_heads // kv_heads
    shards = []
    if world <= kv_heads:
        if kv_heads % world:
            raise ValueError(f"shard_plan: {kv_heads} kv heads do not divide over {world} ranks")
        per = kv_heads // world
        for r in range(world):
            shards.append(Shard(r, r * per, (r + 1) * per, r * per * group, (r + 1) * per * group, 0, length, [r]))
        return shards
    if world % kv_heads:
        raise ValueError(f"shard_plan: {world} ranks do not divide over {kv_heads} kv heads")
    parts = world // kv_heads
    step = -(-length // parts)
    step = -(-step // RANGE_ALIGN) * RANGE_ALIGN
    for r in range(world):
        head, part = divmod(r, parts)
        lo, hi = min(part * step, length), min((part + 1) * step, length)
        members = [head * parts + x for x in range(parts) if min(x * step, length) < min((x + 1) * step, length)]
        shards.append(Shard(r, head, head + 1, head * group, (head + 1) * group, lo, hi, members))
    return shards


def fold(parts, merge):
    """Folds residuals in the order given: ((p0 + p1) + p2) + ...; `merge(a, b)` answers the merged residual."""
    acc = parts[0]
    for nxt in parts[1:]:
        acc = merge(acc, nxt)
    return acc


def gather_and_fold(residual, shard: Shard, dist, merge, process_group=None, empty_like=None):
    """The residual of the whole range, on every rank of the shard's group.

    `residual` is this rank's piece (a tensor the backend of `dist` can move); `dist` is torch.distributed (or anything
    with its all_gather); ranks outside the group must not call.  Ranks fold in range order, so every rank of the group
    computes the same bits.  A rank whose range is empty is not a member of the group.
    """
    if len(shard.group) == 1:
        return residual
    empty_like = empty_like or (lambda t: t.new_empty(t.shape))
    pieces = [empty_like(residual) for _ in shard.group]
    dist.all_gather(pieces, residual, group=process_group)
    return fold(pieces, merge)


def connect_exchange(torch, ext, dist, members, rank, slot_bytes, device=None):
    """This rank's end of an exchange among the ranks `members` (world ranks, in fold / sum order), connected.

    Every rank of the WORLD must call this together (with its own `members`; a rank that belongs to no group of more than
    one passes [rank]): the 64-byte buffer handles travel by one all_gather over the whole world — once, at set-up — so
    no sub-group communicator is ever made.  `device`: where the gathered bytes live ("cuda" under NCCL, "cpu" under gloo).
    """
    x = ext.Exchange(len(members), members.index(rank), slot_bytes)
    device = device or ("cuda" if dist.get_backend() == "nccl" else "cpu")
    mine = torch.frombuffer(bytearray(x.ipc_handle()), dtype=torch.uint8).to(device)
    world = dist.get_world_size()
    every = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(every, mine)
    if len(members) > 1:
        x.connect_handles([bytes(every[r].cpu().numpy().tobytes()) for r in members])
    return x


class LongContextRank:
    """A rank's share of the long-context decode (configuration 4): its heads, its range, its two tiers.

    k_host/v_host: pinned host planes [host_len][kv_heads_local][head_dim] (this rank's positions that live in host RAM),
    k_dev/v_dev: device planes [dev_len][kv_heads_local][head_dim].  step(q_local) answers the rank's output heads
    [q_heads_local][head_dim] as a device tensor of 16-bit patterns.
    """

    def __init__(self, torch, ext, shard: Shard, head_dim, dtype, k_host, v_host, host_len, k_dev, v_dev, dev_len,
                 dist=None, process_group=None, chunk_positions=0, stages=3, exchange=None):
        self.torch, self.ext, self.shard, self.d, self.dtype = torch, ext, shard, head_dim, dtype
        self.k_host, self.v_host, self.host_len, self.k_dev, self.v_dev, self.dev_len = k_host, v_host, host_len, k_dev, v_dev, dev_len
        self.dist, self.pg, self.exchange = dist, process_group, exchange
        self.tier = ext.Tier(shard.q_heads, shard.kv_heads, head_dim, dtype, chunk_positions, stages)
        self.res = torch.zeros((shard.q_heads, head_dim + 2), dtype=torch.float32, device="cuda")
        self.out = torch.zeros((shard.q_heads, head_dim), dtype=torch.int16, device="cuda")

    def _merge(self, a, b):
        self.ext.merge(a, a, b, self.shard.q_heads, self.d)       # `into` may be `a`: the gathered pieces are ours to overwrite
        return a

    def step(self, q_local):
        """One query position.  Alone on its heads: one call, and one launch when every position is on the card.  In a
        range split with an exchange object (connect_exchange): one call — the rank's residual, then the library's
        push-wait-fold kernel.  Without one (gloo on CPU, or by choice): the residuals are all-gathered and folded here."""
        if len(self.shard.group) == 1:
            self.tier.decode(self.out, None, q_local, self.k_host, self.v_host, self.host_len, self.k_dev, self.v_dev, self.dev_len)
        elif self.exchange is not None:
            self.tier.decode_exchange(self.exchange, self.out, None, q_local, self.k_host, self.v_host, self.host_len, self.k_dev, self.v_dev, self.dev_len)
        else:
            self.tier.decode(None, self.res, q_local, self.k_host, self.v_host, self.host_len, self.k_dev, self.v_dev, self.dev_len)
            merged = gather_and_fold(self.res, self.shard, self.dist, self._merge, self.pg)
            self.ext.finish(self.out, merged, self.shard.q_heads, self.d, self.dtype)
        return self.out

    def close(self):
        self.tier.close()


class PeerSum:
    """The tensor-parallel sum that follows head-sharded attention as ONE launch a rank: every rank pushes its 16-bit
    partial into the others' memory, and each adds the pieces in rank order in fp32 and rounds once — the reference's
    vector_sum over the cards' partials (engine/src/packages/nn/gpu/kernels/kernels.cuh:117-126, the fan-in of
    nn/cpu/opcodes/partials__abi.cuh:110-163), so every rank holds the same bits.  `n`: the longest vector to be summed."""

    def __init__(self, torch, ext, dist, n, dtype=0):
        self.torch, self.ext, self.dtype = torch, ext, dtype
        world, rank = dist.get_world_size(), dist.get_rank()
        self.exchange = connect_exchange(torch, ext, dist, list(range(world)), rank, 2 * n)

    def sum(self, partial, out=None, wait_ms=0):
        out = self.torch.empty_like(partial) if out is None else out
        self.exchange.vector_sum(out, partial, partial.numel(), self.dtype, wait_ms=wait_ms)
        return out

    def close(self):
        self.exchange.close()


def sum_over_ranks(partial, dist, vector_sum, process_group=None, world=None, empty_like=None):
    """The tensor-parallel sum that follows head-sharded attention, for ranks that are PROCESSES (one a card, NCCL between
    them): every rank's 16-bit partial is gathered and the pieces are added in rank order by one launch of the family's
    `vector_sum` door — `vector_sum(pieces) -> tensor`, fp32 sum over the pieces in the order given, rounded once — so every
    rank holds the same bits, the bits the reference's in-process form makes when it reads the other cards' partials in
    place (engine/src/packages/nn/gpu/kernels/kernels.cuh:117-126; nn/cpu/opcodes/partials__abi.cuh: the fan-in is in rank
    order there too).  An all-reduce would round a partial sum at every hop in an order the library chooses; this costs
    world-1 more copies of a vector of a few KB and keeps the answer the reference's.
    """
    world = world if world is not None else dist.get_world_size(process_group)
    if world == 1:
        return partial
    import torch
    as_bytes = partial.contiguous().view(torch.uint8)         # 16-bit patterns travel as bytes: neither NCCL nor gloo moves int16
    empty_like = empty_like or (lambda t: t.new_empty(t.shape))
    pieces = [empty_like(as_bytes) for _ in range(world)]
    dist.all_gather(pieces, as_bytes, group=process_group)
    return vector_sum([p.view(partial.dtype).view(partial.shape) for p in pieces])


def family_vector_sum(torch, fam):
    """`vector_sum` for sum_over_ranks through a bound family's door: the pieces are device tensors of 16-bit patterns."""
    from .abi import VectorParts

    def run(pieces):
        n = pieces[0].numel()
        out = torch.empty_like(pieces[0])
        parts = VectorParts()
        for i, p in enumerate(pieces):
            parts.at[i] = p.data_ptr()
        parts.count = len(pieces)
        fam.nn.vector_sum(out.data_ptr(), parts, n, None)
        return out
    return run
