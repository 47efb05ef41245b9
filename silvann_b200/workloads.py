"""Seeded synthetic inputs for the five benchmark configurations (numpy, host side).

The reference publishes no dataset for this path; these generators stand in for one.  Every array is produced by
numpy.random.default_rng(seed) (PCG64) in C order; seeds are fixed per configuration (1001..1005).  16-bit operands are
returned as uint16 bit patterns.  bf16 operands are made fp16-exact (rounded to bf16, magnitudes under 2^-17 flushed
to zero) so that the fp16-only reference and a bf16 kernel read the same real numbers.

A `scale` argument shrinks the long axis (positions, sequences) for tests; scale=1 is the benchmark's size.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

FP16, BF16 = 0, 1
PAGE_POSITIONS = 256


def _bits(x: np.ndarray, dtype: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    if dtype == FP16:
        return x.astype(np.float16).view(np.uint16)
    u = x.view(np.uint32)
    b = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    small = (b & 0x7F80) < ((127 - 17) << 7)          # |value| < 2^-17, read off the exponent field
    b[small] &= 0x8000
    return b


def normal_bits(rng, shape, dtype, scale=1.0) -> np.ndarray:
    return _bits(rng.standard_normal(shape, dtype=np.float32) * np.float32(scale), dtype)


@dataclass
class Decode:
    q: np.ndarray
    k: np.ndarray
    v: np.ndarray
    q_heads: int
    kv_heads: int
    head_dim: int
    length: int
    dtype: int

    @property
    def kv_bytes(self) -> int:
        return 2 * self.length * self.kv_heads * self.head_dim * 2


def config1(length: int = 8192) -> Decode:
    """Single-sequence GQA decode: 16 query heads on 4 kv heads, head_dim 128, fp16 N(0,1)."""
    rng = np.random.default_rng(1001)
    qh, kvh, d = 16, 4, 128
    return Decode(normal_bits(rng, (qh, d), FP16), normal_bits(rng, (length, kvh, d), FP16),
                  normal_bits(rng, (length, kvh, d), FP16), qh, kvh, d, length, FP16)


@dataclass
class Prefill:
    q: np.ndarray
    k: np.ndarray
    v: np.ndarray
    q_heads: int
    kv_heads: int
    head_dim: int
    rows: int
    dtype: int

    @property
    def flops(self) -> float:
        return 4.0 * self.q_heads * self.head_dim * self.rows * (self.rows + 1) / 2.0


def config2(rows: int = 4096, dtype: int = BF16) -> Prefill:
    """Causal GQA prefill: 16 query heads on 2 kv heads, head_dim 256, 0.5·N(0,1)."""
    rng = np.random.default_rng(1002)
    qh, kvh, d = 16, 2, 256
    return Prefill(normal_bits(rng, (rows, qh, d), dtype, 0.5), normal_bits(rng, (rows, kvh, d), dtype, 0.5),
                   normal_bits(rng, (rows, kvh, d), dtype, 0.5), qh, kvh, d, rows, dtype)


@dataclass
class PagedLayout:
    seq_lens: np.ndarray        # int32 [seqs]
    page_table: np.ndarray      # int32 [seqs][max_pages], -1 padded
    pool_pages: int
    q_heads: int
    kv_heads: int
    head_dim: int
    dtype: int

    @property
    def positions(self) -> int:
        return int(self.seq_lens.sum())

    @property
    def kv_bytes(self) -> int:
        return self.positions * 2 * self.kv_heads * self.head_dim * 2


def config3_layout(seqs: int = 32, lo: int = 1024, hi: int = 100000) -> PagedLayout:
    """Batched paged decode: sequence lengths uniform in [lo, hi], pages of 256 positions handed out in order and then
    the pool randomly permuted (same generator), int32 page table padded with -1."""
    rng = np.random.default_rng(1003)
    lens = rng.integers(lo, hi + 1, size=seqs).astype(np.int32)
    pages = (lens + PAGE_POSITIONS - 1) // PAGE_POSITIONS
    total = int(pages.sum())
    perm = rng.permutation(total).astype(np.int32)
    table = np.full((seqs, int(pages.max())), -1, np.int32)
    at = 0
    for s in range(seqs):
        table[s, :pages[s]] = perm[at:at + pages[s]]
        at += int(pages[s])
    return PagedLayout(lens, table, total, 16, 2, 256, BF16)


FILL_CHUNK = 1 << 24


def normal_bits_into(seed: int, stream: int, out: np.ndarray, dtype: int) -> None:
    """Fills `out` (uint16, C order) with N(0,1) bit patterns, FILL_CHUNK elements at a time on a few threads: chunk c is
    drawn from PCG64(seed) jumped (stream * 4096 + c + 1) times, so the values depend on nothing but (seed, stream, index)
    and a 1.6-billion-element pool takes seconds, not minutes."""
    from concurrent.futures import ThreadPoolExecutor
    import os
    flat = out.reshape(-1)

    def one(c):
        rng = np.random.Generator(np.random.PCG64(seed).jumped(stream * 4096 + c + 1))
        at = c * FILL_CHUNK
        n = min(FILL_CHUNK, flat.size - at)
        flat[at:at + n] = _bits(rng.standard_normal(n, dtype=np.float32), dtype)
    chunks = (flat.size + FILL_CHUNK - 1) // FILL_CHUNK
    with ThreadPoolExecutor(max_workers=max(1, min(8, os.cpu_count() or 1))) as pool:
        list(pool.map(one, range(chunks)))


def config3_fill(layout: PagedLayout, seed: int = 1003):
    """q and the two pools for a layout, on the host.  Pool rows past a sequence's end are filled with NaN bit patterns
    on purpose: a kernel must not let them reach its output."""
    rng = np.random.default_rng(seed + 1)
    L = layout
    q = normal_bits(rng, (len(L.seq_lens), L.q_heads, L.head_dim), L.dtype)
    shape = (L.pool_pages, PAGE_POSITIONS, L.kv_heads, L.head_dim)
    k_pool, v_pool = np.empty(shape, np.uint16), np.empty(shape, np.uint16)
    normal_bits_into(seed + 1, 1, k_pool, L.dtype)
    normal_bits_into(seed + 1, 2, v_pool, L.dtype)
    for s, n in enumerate(L.seq_lens):
        tail = int(n) % PAGE_POSITIONS
        if tail:
            last = L.page_table[s, (int(n) - 1) // PAGE_POSITIONS]
            k_pool[last, tail:] = 0x7FC1
            v_pool[last, tail:] = 0x7FC1
    return q, k_pool, v_pool


def gather_sequence(layout: PagedLayout, pool: np.ndarray, s: int) -> np.ndarray:
    """Sequence s's rows as one contiguous [len][kv_heads][head_dim] plane — the layout the reference doors take."""
    n = int(layout.seq_lens[s])
    pages = layout.page_table[s, :(n + PAGE_POSITIONS - 1) // PAGE_POSITIONS]
    return np.ascontiguousarray(pool[pages].reshape(-1, layout.kv_heads, layout.head_dim)[:n])


def config4(length: int = 262144) -> Decode:
    """Long-context decode: one sequence, 32 query heads on 4 kv heads, head_dim 128, bf16 N(0,1)."""
    rng = np.random.default_rng(1004)
    qh, kvh, d = 32, 4, 128
    return Decode(normal_bits(rng, (qh, d), BF16), normal_bits(rng, (length, kvh, d), BF16),
                  normal_bits(rng, (length, kvh, d), BF16), qh, kvh, d, length, BF16)


@dataclass
class DeltaNet:
    conved: np.ndarray   # [rows][(2·k_heads + v_heads)·d]: query heads, key heads, value heads
    z: np.ndarray        # [rows][v_heads·d]
    beta: np.ndarray     # [rows][v_heads]
    g: np.ndarray        # [rows][v_heads]  log decay, negative
    w: np.ndarray        # [d]
    k_heads: int
    v_heads: int
    head_dim: int
    rows: int
    dtype: int


def config5(rows: int = 8192 + 512, heads: int = 32, d: int = 128, dtype: int = BF16) -> DeltaNet:
    """Gated DeltaNet: q,k rows L2-normalised N(0,1); v N(0,1); beta = sigmoid(N(0,1)); g = -softplus(N(0,1)) (so the
    decay gate is exp(g)); z N(0,1); w = 1."""
    rng = np.random.default_rng(1005)
    q = rng.standard_normal((rows, heads, d), dtype=np.float32)
    k = rng.standard_normal((rows, heads, d), dtype=np.float32)
    q /= np.linalg.norm(q, axis=-1, keepdims=True)
    k /= np.linalg.norm(k, axis=-1, keepdims=True)
    v = rng.standard_normal((rows, heads, d), dtype=np.float32)
    conved = np.concatenate([q.reshape(rows, -1), k.reshape(rows, -1), v.reshape(rows, -1)], axis=1)
    beta = 1.0 / (1.0 + np.exp(-rng.standard_normal((rows, heads), dtype=np.float32)))
    g = -np.log1p(np.exp(rng.standard_normal((rows, heads), dtype=np.float32)))
    z = rng.standard_normal((rows, heads * d), dtype=np.float32)
    return DeltaNet(_bits(conved, dtype), _bits(z, dtype), _bits(beta, dtype), _bits(g, dtype),
                    _bits(np.ones(d, np.float32), dtype), heads, heads, d, rows, dtype)
