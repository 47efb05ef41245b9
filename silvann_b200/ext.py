"""ctypes bindings of the `silvann_b200_*` entry points (include/silvann_b200.h, second half).

Arguments that are device buffers may be torch tensors (their data_ptr() is used), integers (raw device addresses) or
None.  Every call raises B200Error with the library's own message when it answers anything but SILVANN_B200_OK.
"""
from __future__ import annotations

import ctypes as C

from . import library_path

FP16, BF16 = 0, 1
OK, E_ARGUMENT, E_CUDA, E_TIMEOUT, E_STATE = 0, 1, 2, 3, 4
COUNTERS = ("fused_decode", "fused_residual", "fused_prefill", "flushed", "refused", "deltanet", "launches", "ext_calls", "gemv_fast", "fused_latent", "expert_fast", "fused_norm_rope")
EXPORTS = (
    "silvann_silicon_family_get", "silvann_b200_last_error", "silvann_b200_counters_read", "silvann_b200_device_status",
    "silvann_b200_decode", "silvann_b200_decode_noalloc", "silvann_b200_merge", "silvann_b200_finish", "silvann_b200_plan_create",
    "silvann_b200_plan_destroy", "silvann_b200_plan_decode", "silvann_b200_plan_info", "silvann_b200_paged_decode", "silvann_b200_paged_append",
    "silvann_b200_prefill", "silvann_b200_deltanet", "silvann_b200_tier_create", "silvann_b200_tier_destroy",
    "silvann_b200_tier_decode", "silvann_b200_tier_stats", "silvann_b200_tier_decode_exchange",
    "silvann_b200_exchange_create", "silvann_b200_exchange_destroy", "silvann_b200_exchange_local", "silvann_b200_exchange_handle",
    "silvann_b200_exchange_connect_handles", "silvann_b200_exchange_connect_addresses", "silvann_b200_exchange_merge_finish",
    "silvann_b200_exchange_vector_sum", "silvann_b200_exchange_deposit", "silvann_b200_mla_decode", "silvann_b200_exchange_gemv_sum",
)


class B200Error(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"silvann_b200 error {code}: {message}")
        self.code = code


def addr(x) -> int | None:
    if x is None:
        return None
    if isinstance(x, int):
        return x
    return x.data_ptr()


_lib = None


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(str(library_path()), mode=C.RTLD_LOCAL)
        vp, u64, u32, i32 = C.c_void_p, C.c_uint64, C.c_uint32, C.c_int
        L.silvann_b200_last_error.restype = C.c_char_p
        sigs = {
            "silvann_b200_counters_read": [vp, u32, i32],
            "silvann_b200_device_status": [vp, i32],
            "silvann_b200_decode": [vp, vp, vp, vp, vp, u64, u64, u64, u64, u32, i32, vp, vp],
            "silvann_b200_decode_noalloc": [vp, vp, vp, vp, vp, u64, u64, u64, u64, u32, i32, vp, vp, C.c_char_p, u32],
            "silvann_b200_merge": [vp, vp, vp, u64, u64, vp],
            "silvann_b200_finish": [vp, vp, u64, u64, i32, vp, vp],
            "silvann_b200_plan_create": [vp],
            "silvann_b200_plan_destroy": [vp],
            "silvann_b200_plan_decode": [vp, vp, u32, u32, u32, u32, u32, vp],
            "silvann_b200_plan_info": [vp, vp, vp, vp],
            "silvann_b200_paged_decode": [vp, vp, vp, vp, vp, vp, u64, u32, vp, u32, i32, vp, vp],
            "silvann_b200_paged_append": [vp, vp, vp, vp, vp, u64, u32, vp, u32, vp],
            "silvann_b200_tier_create": [vp, u32, u32, u32, i32, u32, u32],
            "silvann_b200_tier_destroy": [vp],
            "silvann_b200_tier_decode": [vp, vp, vp, vp, vp, vp, u64, vp, vp, u64, vp, vp],
            "silvann_b200_tier_stats": [vp, vp, vp],
            "silvann_b200_tier_decode_exchange": [vp, vp, vp, vp, vp, vp, vp, u64, vp, vp, u64, vp, u32, vp],
            "silvann_b200_mla_decode": [vp, vp, vp, vp, u64, u64, u64, u32, i32, vp, vp],
            "silvann_b200_exchange_create": [vp, u32, u32, u64],
            "silvann_b200_exchange_destroy": [vp],
            "silvann_b200_exchange_local": [vp, vp, vp],
            "silvann_b200_exchange_handle": [vp, vp, u32],
            "silvann_b200_exchange_connect_handles": [vp, vp, u32],
            "silvann_b200_exchange_connect_addresses": [vp, vp],
            "silvann_b200_exchange_merge_finish": [vp, vp, vp, vp, u64, u64, i32, vp, u32, vp],
            "silvann_b200_exchange_vector_sum": [vp, vp, vp, u64, i32, vp, u32, vp],
            "silvann_b200_exchange_deposit": [vp, u32, vp, u64, u32, vp],
            "silvann_b200_exchange_gemv_sum": [vp, vp, vp, vp, vp, u64, u64, u64, vp, u32, vp],
            "silvann_b200_prefill": [vp, vp, vp, vp, vp, u64, u64, u64, u64, u64, i32, vp, vp],
            "silvann_b200_deltanet": [vp, vp, vp, vp, vp, vp, vp, vp, u64, u64, u64, u64, u32, u32, i32, vp, vp],
        }
        for name, args in sigs.items():
            fn = getattr(L, name)
            fn.argtypes, fn.restype = args, i32
        _lib = L
    return _lib


def _check(code: int):
    if code != OK:
        raise B200Error(code, lib().silvann_b200_last_error().decode())


def counters(reset: bool = False) -> dict:
    out = (C.c_uint64 * len(COUNTERS))()
    _check(lib().silvann_b200_counters_read(out, len(COUNTERS), int(reset)))
    return dict(zip(COUNTERS, out))


def device_status(clear: bool = True) -> int:
    w = C.c_uint32(0)
    _check(lib().silvann_b200_device_status(C.byref(w), int(clear)))
    return w.value


def decode(o, res, q, k, v, q_heads, kv_heads, head_dim, length, dtype=FP16, nsplit=0, over=None, stream=None):
    _check(lib().silvann_b200_decode(addr(o), addr(res), addr(q), addr(k), addr(v), q_heads, kv_heads, head_dim, length,
                                     nsplit, dtype, addr(over), stream))


def decode_noalloc(o, res, q, k, v, q_heads, kv_heads, head_dim, length, dtype=FP16, nsplit=0, over=None, stream=None):
    """silvann_b200_decode_noalloc: the same decode with its scratch in a fixed array inside the library, for callers
    that cannot let a library allocate.  Raises B200Error with the entry point's own message when it refuses."""
    msg = C.create_string_buffer(256)
    code = lib().silvann_b200_decode_noalloc(addr(o), addr(res), addr(q), addr(k), addr(v), q_heads, kv_heads, head_dim, length,
                                             nsplit, dtype, addr(over), stream, msg, 256)
    if code != OK:
        raise B200Error(code, msg.value.decode())


def merge(into, a, b, q_heads, head_dim, stream=None):
    _check(lib().silvann_b200_merge(addr(into), addr(a), addr(b), q_heads, head_dim, stream))


def finish(o, res, q_heads, head_dim, dtype=FP16, over=None, stream=None):
    _check(lib().silvann_b200_finish(addr(o), addr(res), q_heads, head_dim, dtype, addr(over), stream))


class Plan:
    """A paged-decode plan (work list + split scratch) on the current device."""

    def __init__(self):
        self.handle = C.c_void_p()
        _check(lib().silvann_b200_plan_create(C.byref(self.handle)))

    def close(self):
        if self.handle:
            lib().silvann_b200_plan_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def plan(self, seq_lens, q_heads, kv_heads, head_dim, blocks_target=0, stream=None):
        # a contiguous int32 numpy array is handed over as it lies (the planner copies what it keeps before it returns)
        dt, fl = getattr(seq_lens, "dtype", None), getattr(seq_lens, "flags", None)
        if dt is not None and fl is not None and str(dt) == "int32" and fl["C_CONTIGUOUS"] and getattr(seq_lens, "ndim", 0) == 1:
            arr = seq_lens.ctypes.data
        else:
            arr = (C.c_int32 * len(seq_lens))(*[int(x) for x in seq_lens])
        _check(lib().silvann_b200_plan_decode(self.handle, arr, len(seq_lens), q_heads, kv_heads, head_dim, blocks_target, stream))

    def info(self) -> dict:
        b, s, p = C.c_uint32(), C.c_uint32(), C.c_uint64()
        _check(lib().silvann_b200_plan_info(self.handle, C.byref(b), C.byref(s), C.byref(p)))
        return {"blocks": b.value, "slots": s.value, "positions": p.value}

    def decode(self, o, res, q, k_pool, v_pool, pool_pages, page_positions, page_table, table_stride, dtype=FP16, over=None, stream=None):
        _check(lib().silvann_b200_paged_decode(self.handle, addr(o), addr(res), addr(q), addr(k_pool), addr(v_pool), pool_pages,
                                               page_positions, addr(page_table), table_stride, dtype, addr(over), stream))


    def append(self, k_pool, v_pool, k_rows, v_rows, pool_pages, page_positions, page_table, table_stride, stream=None):
        _check(lib().silvann_b200_paged_append(self.handle, addr(k_pool), addr(v_pool), addr(k_rows), addr(v_rows), pool_pages, page_positions,
                                               addr(page_table), table_stride, stream))


class Tier:
    """Decode over a cache whose oldest positions live in pinned host RAM (see silvann_b200_tier_decode)."""

    def __init__(self, q_heads, kv_heads, head_dim, dtype=FP16, chunk_positions=0, stages=3):
        self.handle = C.c_void_p()
        _check(lib().silvann_b200_tier_create(C.byref(self.handle), q_heads, kv_heads, head_dim, dtype, chunk_positions, stages))

    def close(self):
        if self.handle:
            lib().silvann_b200_tier_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def decode(self, o, res, q, k_host, v_host, host_len, k_dev, v_dev, dev_len, over=None, stream=None):
        _check(lib().silvann_b200_tier_decode(self.handle, addr(o), addr(res), addr(q), addr(k_host), addr(v_host), host_len,
                                              addr(k_dev), addr(v_dev), dev_len, addr(over), stream))

    def decode_exchange(self, exchange, o, res, q, k_host, v_host, host_len, k_dev, v_dev, dev_len, over=None, wait_ms=0, stream=None):
        """This member's residual over its two tiers, then the exchange with the members that hold the rest of the range."""
        _check(lib().silvann_b200_tier_decode_exchange(self.handle, exchange.handle, addr(o), addr(res), addr(q), addr(k_host), addr(v_host), host_len,
                                                       addr(k_dev), addr(v_dev), dev_len, addr(over), wait_ms, stream))

    def stats(self) -> dict:
        b, c = C.c_uint64(), C.c_uint64()
        _check(lib().silvann_b200_tier_stats(self.handle, C.byref(b), C.byref(c)))
        return {"h2d_bytes": b.value, "chunks": c.value}


HANDLE_BYTES = 64


class Exchange:
    """One member's end of an exchange among the cards that share a piece of work (see silvann_b200_exchange_create)."""

    def __init__(self, members, index, slot_bytes):
        self.handle = C.c_void_p()
        self.members, self.index = members, index
        _check(lib().silvann_b200_exchange_create(C.byref(self.handle), members, index, slot_bytes))

    def close(self):
        if self.handle:
            lib().silvann_b200_exchange_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def local(self) -> tuple:
        a, b = C.c_uint64(), C.c_uint64()
        _check(lib().silvann_b200_exchange_local(self.handle, C.byref(a), C.byref(b)))
        return a.value, b.value

    def ipc_handle(self) -> bytes:
        buf = C.create_string_buffer(HANDLE_BYTES)
        _check(lib().silvann_b200_exchange_handle(self.handle, buf, HANDLE_BYTES))
        return buf.raw

    def connect_handles(self, handles):
        """handles: every member's ipc_handle() in member order (this member's own entry is ignored)."""
        blob = b"".join(bytes(h) for h in handles)
        assert len(blob) == HANDLE_BYTES * self.members
        _check(lib().silvann_b200_exchange_connect_handles(self.handle, blob, HANDLE_BYTES))

    def connect_addresses(self, addresses):
        arr = (C.c_uint64 * self.members)(*[int(a) for a in addresses])
        _check(lib().silvann_b200_exchange_connect_addresses(self.handle, arr))

    def connect_alone(self):
        """For a one-card walk of a many-card plan: this member's own buffer stands in for every absent member's, so the
        kernel's pushes land somewhere real; the absent members' pieces arrive by deposit()."""
        self.connect_addresses([self.local()[0]] * self.members)

    def merge_finish(self, o, res, res_local, q_heads, head_dim, dtype=FP16, over=None, wait_ms=0, stream=None):
        _check(lib().silvann_b200_exchange_merge_finish(self.handle, addr(o), addr(res), addr(res_local), q_heads, head_dim, dtype, addr(over), wait_ms, stream))

    def vector_sum(self, out, partial, n, dtype=FP16, over=None, wait_ms=0, stream=None):
        _check(lib().silvann_b200_exchange_vector_sum(self.handle, addr(out), addr(partial), n, dtype, addr(over), wait_ms, stream))

    def gemv_sum(self, out, codes, scales, vec, width, rows, cols, over=None, wait_ms=0, stream=None):
        """This card's share of a coded matrix times its share of the input, the cards' answers added in member order: one launch."""
        _check(lib().silvann_b200_exchange_gemv_sum(self.handle, addr(out), addr(codes), addr(scales), addr(vec), width, rows, cols, addr(over), wait_ms, stream))

    def deposit(self, member, data, nbytes, unit=4, stream=None):
        """An absent member's piece of the next exchange; unit 4 for merge_finish and vector_sum, 2 for gemv_sum's rows."""
        _check(lib().silvann_b200_exchange_deposit(self.handle, member, addr(data), nbytes, unit, stream))


def prefill(o, q, k, v, q_heads, kv_heads, head_dim, first, rows, dtype=FP16, over=None, stream=None, res=None):
    _check(lib().silvann_b200_prefill(addr(o), addr(res), addr(q), addr(k), addr(v), q_heads, kv_heads, head_dim, first, rows, dtype, addr(over), stream))


def mla_decode(o, res, q, latent, heads, length, dtype=FP16, blocks=0, latent_dim=512, over=None, stream=None):
    _check(lib().silvann_b200_mla_decode(addr(o), addr(res), addr(q), addr(latent), heads, latent_dim, length, blocks, dtype, addr(over), stream))


def deltanet(S, conved, z, beta, g, w, out, k_heads, v_heads, head_dim, rows, seqs=1, gate=0, dtype=FP16, over=None, stream=None, readout=None):
    _check(lib().silvann_b200_deltanet(addr(S), addr(conved), addr(z), addr(beta), addr(g), addr(w), addr(out), addr(readout), k_heads, v_heads,
                                       head_dim, rows, seqs, gate, dtype, addr(over), stream))
