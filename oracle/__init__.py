"""The checker — TEST INFRASTRUCTURE, NOT PRODUCT.

Two CPU witnesses of the attention / Gated-DeltaNet door arithmetic, both driven with numpy arrays:

  * `port`       the plain-C restatement in silvann_oracle.c (fp16 and bf16), always available after oracle/build.py;
  * `reference`  the reference's own CPU silicon family (x86_avx2, fp16 only), compiled unmodified from the reference
                 tree into oracle/_ref/ where that tree is mounted; None elsewhere unless an earlier build travelled.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference legs may import this package.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
FP16, BF16 = 0, 1


# ---- 16-bit helpers (numpy has no bf16) -------------------------------------------------------------------------

def to_bits(x: np.ndarray, dtype: int) -> np.ndarray:
    """fp32 array -> uint16 bit patterns of fp16 (dtype 0) or bf16 (dtype 1), round to nearest even."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if dtype == FP16:
        return x.astype(np.float16).view(np.uint16)
    u = x.view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def from_bits(b: np.ndarray, dtype: int) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint16)
    if dtype == FP16:
        return b.view(np.float16).astype(np.float32)
    return (b.astype(np.uint32) << 16).view(np.float32)


def fp16_exact_bf16(x: np.ndarray) -> np.ndarray:
    """Rounds to bf16 and flushes |x| < 2^-17 to zero, so every value is exactly representable in fp16 as well: the
    reference (fp16 only) and a bf16 kernel then see the same real numbers."""
    y = from_bits(to_bits(x, BF16), BF16)
    y[np.abs(y) < 2.0 ** -17] = 0.0
    y = np.clip(y, -65504.0, 65504.0)
    assert np.array_equal(y.astype(np.float16).astype(np.float32), y)
    return y


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


# ---- the C restatement -------------------------------------------------------------------------------------------

class Port:
    def __init__(self):
        so = HERE / "liboracle.so"
        if not so.exists():
            from . import build
            build.build_port()
        self.lib = C.CDLL(str(so))
        u64, vp, i32 = C.c_uint64, C.c_void_p, C.c_int
        sig = {
            "oracle_attention_scores": [vp, vp, vp, u64, u64, u64, u64, i32],
            "oracle_attention_scores_grouped": [vp, vp, vp, u64, u64, u64, u64, i32],
            "oracle_attention_softmax_rows": [vp, u64, u64],
            "oracle_attention_mix": [vp, vp, vp, u64, u64, u64, u64, i32, vp],
            "oracle_attention_weights": [vp, vp, vp, vp, u64, u64, u64, u64, i32],
            "oracle_attention_residual_mix": [vp, vp, vp, u64, u64, u64, u64, i32],
            "oracle_attention_merge": [vp, vp, vp, u64, u64],
            "oracle_attention_finish": [vp, vp, u64, u64, i32, vp],
            "oracle_attention_causal_scores_grouped": [vp, vp, vp, u64, u64, u64, u64, u64, i32],
            "oracle_attention_causal_softmax": [vp, u64, u64, u64],
            "oracle_attention_causal_mix": [vp, vp, vp, u64, u64, u64, u64, u64, i32, vp],
            "oracle_prefill": [vp, vp, vp, vp, vp, u64, u64, u64, u64, u64, i32, vp],
            "oracle_deltanet_steps": [vp, vp, vp, vp, vp, vp, vp, u64, u64, u64, u64, C.c_uint, i32, vp],
            "oracle_deltanet_steps_readout": [vp, vp, vp, vp, vp, vp, vp, vp, u64, u64, u64, u64, C.c_uint, i32, vp],
            "oracle_attention_scores_grouped_rows": [vp, u64, vp, u64, vp, u64, vp, u64, u64, u64, u64, i32],
            "oracle_attention_softmax_lens": [vp, u64, vp, u64, u64],
            "oracle_attention_softmax_sink": [vp, vp, u64, u64],
            "oracle_attention_mix_rows": [vp, u64, vp, u64, vp, u64, vp, u64, u64, u64, u64, i32, vp],
            "oracle_deltanet_gates_rows": [vp, vp, vp, vp, vp, vp, u64, u64],
            "oracle_deltanet_conv_steps": [vp, vp, vp, vp, u64, u64],
            "oracle_vector_add": [vp, vp, vp, u64],
            "oracle_vector_copy_rows": [vp, u64, vp, u64, u64, u64],
            "oracle_rmsnorm_rows": [vp, vp, vp, u64, u64, u64, u64, C.c_float],
            "oracle_rope_rows": [vp, vp, vp, u64, u64, u64, u64, u64],
            "oracle_rope_interleaved": [vp, vp, vp, u64, u64, u64, u64],
            "oracle_rope_angles": [vp, u64, vp, C.c_float, u64, u64, u64, i32],
            "oracle_attention_gate_rows": [vp, vp, vp, u64, u64],
            "oracle_turboquant_decode": [vp, vp, vp, u64, u64, u64],
            "oracle_hadamard_blocks": [vp, vp, vp, u64, u64, u64],
            "oracle_turboquant_encode_rows": [vp, vp, vp, u64, u64, u64],
            "oracle_attention_residual_tq": [vp, vp, vp, vp, vp, vp, vp, u64, u64, u64, u64, u64],
            "oracle_hadamard_rotate": [vp, vp, vp, u64],
            "oracle_kda_decays": [vp, vp, vp, vp, u64, u64, C.c_float, u64],
            "oracle_kda_steps": [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, u64, u64, C.c_float, C.c_float, u64],
            "oracle_attention_absorb_rows": [vp, vp, vp, u64, u64, u64, u64, C.c_float, u64],
            "oracle_attention_expand_rows": [vp, vp, vp, u64, u64, u64, u64, u64, u64],
            "oracle_index_layernorm": [vp, vp, vp, vp, u64, C.c_float],
            "oracle_index_pool": [vp, vp, vp, vp, u64, u64, u64, u64],
            "oracle_index_scores_rows": [vp, u64, vp, vp, vp, u64, u64, u64, u64, u64, u64, C.c_float],
            "oracle_index_select": [vp, vp, vp, u64, u64, u64, u64, u64],
            "oracle_index_select_rows": [vp, u64, vp, vp, u64, u64, u64, u64, u64],
            "oracle_index_blocks": [vp, vp, u64, u64],
            "oracle_index_gather_rows": [vp, u64, vp, vp, u64, vp, u64, u64, u64],
            "oracle_turboquant_gemv": [vp, vp, vp, vp, u64, u64, u64],
        }
        for name, args in sig.items():
            fn = getattr(self.lib, name)
            fn.argtypes, fn.restype = args, None

    # one query position ------------------------------------------------------------------------------------------
    def scores(self, q, k, qh, kvh, d, length, dtype=FP16):
        p = np.empty((qh, length), np.float32)
        self.lib.oracle_attention_scores(_p(p), _p(q), _p(k), qh, kvh, d, length, dtype)
        return p

    def mix(self, p, v, qh, kvh, d, length, dtype=FP16):
        o = np.empty((qh, d), np.uint16)
        over = np.zeros(1, np.uint32)
        self.lib.oracle_attention_mix(_p(o), _p(p), _p(v), qh, kvh, d, length, dtype, _p(over))
        return o, int(over[0])

    def residual(self, q, k, v, qh, kvh, d, length, dtype=FP16):
        """(m, l, acc) per head, [qh][d + 2] fp32: attention_weights then attention_residual_mix."""
        p = np.empty((qh, length), np.float32)
        res = np.zeros((qh, d + 2), np.float32)
        self.lib.oracle_attention_weights(_p(p), _p(res), _p(q), _p(k), qh, kvh, d, length, dtype)
        self.lib.oracle_attention_residual_mix(_p(res), _p(p), _p(v), qh, kvh, d, length, dtype)
        return res

    def merge(self, a, b, qh, d):
        out = np.empty_like(a)
        self.lib.oracle_attention_merge(_p(out), _p(a), _p(b), qh, d)
        return out

    def finish(self, res, qh, d, dtype=FP16):
        o = np.empty((qh, d), np.uint16)
        over = np.zeros(1, np.uint32)
        self.lib.oracle_attention_finish(_p(o), _p(res), qh, d, dtype, _p(over))
        return o, int(over[0])

    def decode(self, q, k, v, qh, kvh, d, length, dtype=FP16):
        """attention_scores + attention_mix.  Answers (o bits, fp32 value before rounding)."""
        res = self.residual(q, k, v, qh, kvh, d, length, dtype)
        p = self.scores(q, k, qh, kvh, d, length, dtype)
        o, _ = self.mix(p, v, qh, kvh, d, length, dtype)
        return o, res[:, 2:] / res[:, 1:2]

    # a prompt's rows -------------------------------------------------------------------------------------------
    def causal_three_doors(self, q, k, v, qh, kvh, d, first, rows, dtype=FP16):
        span = first + rows
        p = np.zeros((rows * qh, span), np.float32)
        o = np.empty((rows, qh, d), np.uint16)
        over = np.zeros(1, np.uint32)
        self.lib.oracle_attention_causal_scores_grouped(_p(p), _p(q), _p(k), qh, kvh, d, first, rows, dtype)
        self.lib.oracle_attention_causal_softmax(_p(p), qh, first, rows)
        self.lib.oracle_attention_causal_mix(_p(o), _p(p), _p(v), qh, kvh, d, first, rows, dtype, _p(over))
        return o

    def prefill(self, q, k, v, qh, kvh, d, first, rows, dtype=FP16):
        o = np.empty((rows, qh, d), np.uint16)
        o32 = np.empty((rows, qh, d), np.float32)
        over = np.zeros(1, np.uint32)
        self.lib.oracle_prefill(_p(o), _p(o32), _p(q), _p(k), _p(v), qh, kvh, d, first, rows, dtype, _p(over))
        return o, o32

    # Gated DeltaNet ------------------------------------------------------------------------------------------------
    def deltanet(self, S, conved, z, beta, g, w, kh, vh, d, rows, gate=0, dtype=FP16, readout=None):
        """Updates S in place; answers out [rows][vh*d] bits.  `readout`: a float32 [rows][vh*d] array that receives every
        position's read-out before its first rounding to 16 bits."""
        out = np.empty((rows, vh * d), np.uint16)
        over = np.zeros(1, np.uint32)
        self.lib.oracle_deltanet_steps_readout(_p(S), _p(conved), _p(z), _p(beta), _p(g), _p(w), _p(out), None if readout is None else _p(readout),
                                               kh, vh, d, rows, gate, dtype, _p(over))
        return out


def gathered_rows(impl, q, k, v, lens, qh, kvh, d, dtype=FP16):
    """The per-row (gathered key set) door sequence GLM's sparse attention runs — attention_scores_grouped_rows,
    attention_softmax_lens, attention_mix_rows (ai_z__glm_5_3 layer__abi.cuh:861-1055) — on either checker.
    q [rows][qh][d]; k, v [rows][most][kvh][d]; lens uint32 [rows].  Answers (weights buffer, o bits)."""
    rows, most = len(lens), k.shape[1]
    p = np.zeros((rows, qh * most), np.float32)
    o = np.zeros((rows, qh, d), np.uint16)
    over = np.zeros(1, np.uint32)
    lens = np.ascontiguousarray(lens, np.uint32)
    if isinstance(impl, Port):
        impl.lib.oracle_attention_scores_grouped_rows(_p(p), qh * most, _p(q), qh * d, _p(k), most * kvh * d, _p(lens), qh, kvh, d, rows, dtype)
        impl.lib.oracle_attention_softmax_lens(_p(p), qh * most, _p(lens), qh, rows)
        impl.lib.oracle_attention_mix_rows(_p(o), qh * d, _p(p), qh * most, _p(v), most * kvh * d, _p(lens), qh, kvh, d, rows, dtype, _p(over))
    else:
        impl.nn.attention_scores_grouped_rows(_p(p), qh * most, _p(q), qh * d, _p(k), most * kvh * d, _p(lens), qh, kvh, d, most, rows)
        impl.nn.attention_softmax_lens(_p(p), qh * most, _p(lens), qh, rows)
        impl.nn.attention_mix_rows(_p(o), qh * d, _p(p), qh * most, _p(v), most * kvh * d, _p(lens), qh, kvh, d, rows, _p(over))
        impl.wait()
    return p, o


def softmax_sink(impl, scores, sink):
    p = np.ascontiguousarray(scores, np.float32).copy()
    rows, length = p.shape
    if isinstance(impl, Port):
        impl.lib.oracle_attention_softmax_sink(_p(p), _p(sink), rows, length)
    else:
        impl.nn.attention_softmax_sink(_p(p), _p(sink), rows, length)
        impl.wait()
    return p


def deltanet_inputs(impl, a, b, a_log, dt_bias, w, x, window, heads, rows, ch):
    """deltanet_gates_rows, then deltanet_conv_steps over `rows` rows (window updated in place)."""
    beta, g = np.zeros((rows, heads), np.uint16), np.zeros((rows, heads), np.uint16)
    o = np.zeros((rows, ch), np.uint16)
    over = np.zeros(1, np.uint32)
    if isinstance(impl, Port):
        impl.lib.oracle_deltanet_gates_rows(_p(beta), _p(g), _p(a), _p(b), _p(a_log), _p(dt_bias), heads, rows)
        impl.lib.oracle_deltanet_conv_steps(_p(o), _p(window), _p(w), _p(x), ch, rows)
    else:
        impl.nn.deltanet_gates_rows(_p(beta), _p(g), _p(a), _p(b), _p(a_log), _p(dt_bias), heads, rows, _p(over))
        impl.nn.deltanet_conv_steps(_p(o), _p(window), _p(w), _p(x), ch, rows, _p(over))
        impl.wait()
    return beta, g, o


# ---- the reference's own CPU family --------------------------------------------------------------------------------

class Reference:
    """Door calls into the reference's x86_avx2 family; a CPU family's "device" addresses are host addresses."""

    def __init__(self, path: Path):
        from silvann_b200.abi import Family
        os.environ.setdefault("SILVANN_CPU_AVX512", "0")     # pin the AVX2 bodies so runs are comparable across hosts
        self.family = Family(path)
        self.nn = self.family.nn
        self.over = np.zeros(4, np.uint32)
        # How many threads the family's pool takes beside the caller is decided from the machine's load when the pool starts
        # (at binding or on the first launch) and is only ever told through SILVANN_CPU_POOL_REPORT=1 on stderr
        # (x86_avx2/primitives/pool.cuh:282-289 of the reference tree): bind and make a first launch with stderr caught.
        import re
        import tempfile
        os.environ["SILVANN_CPU_POOL_REPORT"] = "1"
        q = np.zeros((16, 128), np.uint16); k = np.zeros((512, 4, 128), np.uint16); p = np.zeros((16, 512), np.float32)
        with tempfile.TemporaryFile() as tmp:
            keep = os.dup(2)
            os.dup2(tmp.fileno(), 2)
            try:
                self.family.sys.bind_device(0)
                self.nn.attention_scores(_p(p), _p(q), _p(k), 16, 4, 128, 512)
                self.nn.attention_mix(_p(np.zeros((16, 128), np.uint16)), _p(p), _p(k), 16, 4, 128, 512, _p(self.over))
                self.family.sys.compute_completed()
            finally:
                os.dup2(keep, 2)
                os.close(keep)
            tmp.seek(0)
            self.pool_line = tmp.read().decode(errors="replace").strip()
        m = re.search(r"a pool of (\d+) thread", self.pool_line)
        self.pool_threads = int(m.group(1)) if m else None      # threads beside the caller, who works too

    def wait(self):
        self.family.sys.compute_completed()

    def pool(self):
        """(threads the pool took beside the caller, or None when the family did not say; the family's own line)."""
        return self.pool_threads, self.pool_line

    def scores(self, q, k, qh, kvh, d, length):
        p = np.empty((qh, length), np.float32)
        self.nn.attention_scores(_p(p), _p(q), _p(k), qh, kvh, d, length)
        self.wait()
        return p

    def decode(self, q, k, v, qh, kvh, d, length, p=None):
        p = np.empty((qh, length), np.float32) if p is None else p
        o = np.empty((qh, d), np.uint16)
        self.nn.attention_scores(_p(p), _p(q), _p(k), qh, kvh, d, length)
        self.nn.attention_mix(_p(o), _p(p), _p(v), qh, kvh, d, length, _p(self.over))
        self.wait()
        return o

    def residual(self, q, k, v, qh, kvh, d, length, p=None):
        p = np.empty((qh, length), np.float32) if p is None else p
        res = np.zeros((qh, d + 2), np.float32)
        self.nn.attention_weights(_p(p), _p(res), _p(q), _p(k), qh, kvh, d, length)
        self.nn.attention_residual_mix(_p(res), _p(p), _p(v), qh, kvh, d, length)
        self.wait()
        return res

    def merge(self, a, b, qh, d):
        out = np.empty_like(a)
        self.nn.attention_merge(_p(out), _p(a), _p(b), qh, d)
        self.wait()
        return out

    def finish(self, res, qh, d):
        o = np.empty((qh, d), np.uint16)
        self.nn.attention_finish(_p(o), _p(res), qh, d, _p(self.over))
        self.wait()
        return o

    def causal(self, q, k, v, qh, kvh, d, first, rows, p=None):
        """One chunk of rows through the three causal doors, as the runtime drives them (<= 256 rows a call)."""
        span = first + rows
        p = np.empty((rows * qh, span), np.float32) if p is None else p
        o = np.empty((rows, qh, d), np.uint16)
        self.nn.attention_causal_scores_grouped(_p(p), _p(q), _p(k), qh, kvh, d, first, rows)
        self.nn.attention_causal_softmax(_p(p), qh, first, rows)
        self.nn.attention_causal_mix(_p(o), _p(p), _p(v), qh, kvh, d, first, rows, _p(self.over))
        self.wait()
        return o

    def prefill(self, q, k, v, qh, kvh, d, rows, chunk=256):
        o = np.empty((rows, qh, d), np.uint16)
        p = np.empty(chunk * qh * rows, np.float32)
        for first in range(0, rows, chunk):
            n = min(chunk, rows - first)
            o[first:first + n] = self.causal(q[first:first + n], k, v, qh, kvh, d, first, n, p)
        return o

    def residual_rows(self, q, k, v, qh, kvh, d, first, rows):
        """attention_weights_rows + attention_residual_mix_rows: a residual a row, [rows][qh][d + 2]."""
        span = first + rows
        p = np.zeros((rows * qh, span), np.float32)
        res = np.zeros((rows, qh, d + 2), np.float32)
        self.nn.attention_weights_rows(_p(p), _p(res), _p(q), _p(k), qh, kvh, d, first, rows)
        self.nn.attention_residual_mix_rows(_p(res), _p(p), _p(v), qh, kvh, d, first, rows)
        self.wait()
        return res

    def deltanet(self, S, conved, z, beta, g, w, kh, vh, d, rows, gate=0):
        out = np.empty((rows, vh * d), np.uint16)
        if rows == 1 and gate == 0:
            self.nn.deltanet_step(_p(S), _p(conved), _p(z), _p(beta), _p(g), _p(w), _p(out), kh, vh, d, _p(self.over))
        else:
            self.nn.deltanet_steps_gate(_p(S), _p(conved), _p(z), _p(beta), _p(g), _p(w), _p(out), kh, vh, d, rows, gate, _p(self.over))
        self.wait()
        return out


# ---- the TurboQuant-coded tiers: the same four operations through either implementation --------------------------------

def tq_row_bytes(d: int, cols: int) -> int:
    per = 16 // d
    return ((cols + per - 1) // per) * 2


def tq_levels(impl, d: int) -> np.ndarray:
    """The 2^d levels of width d as fp16 bit patterns: every code decoded at scale 1."""
    n = 1 << d
    per = 16 // d
    units = np.zeros((n + per - 1) // per, np.uint16)
    for c in range(n):
        units[c // per] |= np.uint16(c << (d * (c % per)))
    codes = units.view(np.uint8).copy()
    lut = np.array([0x3C00], np.uint16).view(np.uint8).copy()
    return tq_decode(impl, codes, lut, d, 1, n).reshape(n)


def tq_decode(impl, codes, luts, d, rows, cols):
    out = np.zeros((rows, cols), np.uint16)
    if isinstance(impl, Port):
        impl.lib.oracle_turboquant_decode(_p(out), _p(codes), _p(luts), d, rows, cols)
    else:
        impl.nn.turboquant_decode(_p(out), _p(codes), codes.nbytes, _p(luts), luts.nbytes, d, rows, cols, _p(impl.over))
        impl.wait()
    return out


def hadamard_blocks(impl, x, sign, block, inverse):
    out = np.zeros_like(x)
    if isinstance(impl, Port):
        impl.lib.oracle_hadamard_blocks(_p(out), _p(x), _p(sign), x.size, block, inverse)
    else:
        impl.nn.hadamard_blocks(_p(out), _p(x), _p(sign), x.size, block, inverse, _p(impl.over))
        impl.wait()
    return out


def tq_encode_rows(impl, x, d):
    rows, cols = x.shape
    codes = np.zeros((rows, tq_row_bytes(d, cols)), np.uint8)
    scales = np.zeros(rows, np.uint16)
    if isinstance(impl, Port):
        impl.lib.oracle_turboquant_encode_rows(_p(codes), _p(scales), _p(x), rows, cols, d)
    else:
        impl.nn.turboquant_encode_rows(_p(codes), _p(scales), _p(x), rows, cols, d, _p(impl.over))
        impl.wait()
    return codes, scales


def residual_tq(impl, q, kcodes, kscales, vcodes, vscales, qh, kvh, dh, length, d):
    """attention_weights_tq + attention_residual_mix_tq: (m, l, acc) a head over `length` coded positions."""
    p = np.zeros((qh, length), np.float32)
    res = np.zeros((qh, dh + 2), np.float32)
    if isinstance(impl, Port):
        impl.lib.oracle_attention_residual_tq(_p(p), _p(res), _p(q), _p(kcodes), _p(kscales), _p(vcodes), _p(vscales), qh, kvh, dh, length, d)
    else:
        impl.nn.attention_weights_tq(_p(p), _p(res), _p(q), _p(kcodes), _p(kscales), qh, kvh, dh, length, d)
        impl.nn.attention_residual_mix_tq(_p(res), _p(p), _p(vcodes), _p(vscales), qh, kvh, dh, length, d)
        impl.wait()
    return res


def hadamard_rotate(impl, x, sign):
    """The rotation over a whole row (hadamard_rotate): blocks of 512, then a 256 and a 128."""
    P = getattr(impl, "ptr", _p)
    out = np.zeros_like(x)
    if isinstance(impl, Port):
        impl.lib.oracle_hadamard_rotate(_p(out), _p(x), _p(sign), x.size)
    else:
        impl.nn.hadamard_rotate(P(out), P(x), P(sign), x.size, P(impl.over))
        impl.wait()
    return out


def tq_gemv(impl, codes, luts, x, d, rows, cols):
    """turboquant_gemv: a coded matrix of `rows` rows times the 16-bit vector x."""
    P = getattr(impl, "ptr", _p)
    out = np.zeros(rows, np.uint16)
    if isinstance(impl, Port):
        impl.lib.oracle_turboquant_gemv(_p(out), _p(codes), _p(luts), _p(x), d, rows, cols)
    else:
        impl.nn.turboquant_gemv(P(out), P(codes), codes.nbytes, P(luts), luts.nbytes, P(x), d, rows, cols, P(impl.over))
        impl.wait()
    return out


# ---- the expert-major GEMM doors (a coded matrix over rows of x named by pairs) through a family ---------------------

def _address(p) -> int:
    return int(p.value or 0) if isinstance(p, C.c_void_p) else int(p or 0)


def expert_groups_struct(groups, ptr):
    """groups: [(codes, luts, out_rows, d, out_at, pairs_at, pairs)] -> the by-value struct the door takes."""
    from silvann_b200.abi import ExpertGroups
    g = ExpertGroups()
    for i, (codes, luts, out_rows, d, out_at, pairs_at, pairs) in enumerate(groups):
        g.codes[i] = _address(ptr(codes))
        g.luts[i] = _address(ptr(luts)) if luts is not None else 0
        g.out_rows[i], g.d[i], g.out_at[i], g.pairs_at[i], g.pairs[i] = out_rows, d, out_at, pairs_at, pairs
    g.count = len(groups)
    return g


def expert_rows(impl, out, codes, luts, x, pairs, count, d, out_rows, cols, w_room=None, l_room=None):
    """expert_rows into `out` (a 16-bit array [out rows][out_rows], written in place): a family's door (the restatement has none)."""
    P = getattr(impl, "ptr", _p)
    over = impl.over if getattr(impl, "over", None) is not None else None
    impl.nn.expert_rows(P(out), P(codes), codes.nbytes if w_room is None else w_room, P(luts) if luts is not None else None,
                        (luts.nbytes if luts is not None else 0) if l_room is None else l_room,
                        P(x), P(pairs), count, d, out_rows, cols, P(over) if over is not None else None)
    impl.wait()
    return out


def expert_rows_sum(impl, acc, codes, luts, x, pairs, w, count, d, out_rows, cols):
    P = getattr(impl, "ptr", _p)
    impl.nn.expert_rows_sum(P(acc), P(codes), codes.nbytes, P(luts) if luts is not None else None, luts.nbytes if luts is not None else 0, P(x), P(pairs), P(w), count, d, out_rows, cols)
    impl.wait()
    return acc


def expert_groups(impl, out, groups, x, pairs, cols):
    P = getattr(impl, "ptr", _p)
    over = impl.over if getattr(impl, "over", None) is not None else None
    impl.nn.expert_groups(P(out), expert_groups_struct(groups, P), P(x), P(pairs), cols, P(over) if over is not None else None)
    impl.wait()
    return out


# ---- the GLM mixer's doors through either implementation ------------------------------------------------------------

def kda_steps(impl, S, conved, f, b, dt, a_log, gate, w, heads, d, lower, eps, rows, decayed=False):
    """Kimi Delta Attention over `rows` rows (kda_steps; rows = 1 through kda_step; decayed: kda_decays then
    kda_steps_decayed).  conved is the rows' q, then their k, then their v.  Answers (state after, out)."""
    P = getattr(impl, "ptr", _p)
    S = S.copy()
    out = np.zeros((rows, heads * d), np.uint16)
    f32 = lambda v: C.c_float(float(v))
    if isinstance(impl, Port):
        eg = None
        if decayed:
            eg = np.zeros((rows, heads * d), np.float32)
            impl.lib.oracle_kda_decays(_p(eg), _p(f), _p(dt), _p(a_log), heads, d, f32(lower), rows)
        impl.lib.oracle_kda_steps(_p(S), _p(conved), _p(f), _p(eg) if decayed else None, _p(b), _p(dt), _p(a_log), _p(gate), _p(w), _p(out), heads, d,
                                  f32(lower), f32(eps), rows)
    elif decayed:
        eg = np.zeros((rows, heads * d), np.float32)
        impl.nn.kda_decays(P(eg), P(f), P(dt), P(a_log), heads, d, f32(lower), rows)
        impl.nn.kda_steps_decayed(P(S), P(conved), P(eg), P(b), P(gate), P(w), P(out), heads, d, f32(eps), rows, P(impl.over))
        impl.wait()
    elif rows == 1:
        impl.nn.kda_step(P(S), P(conved), P(f), P(b), P(dt), P(a_log), P(gate), P(w), P(out), heads, d, f32(lower), f32(eps), P(impl.over))
        impl.wait()
    else:
        impl.nn.kda_steps(P(S), P(conved), P(f), P(b), P(dt), P(a_log), P(gate), P(w), P(out), heads, d, f32(lower), f32(eps), rows, P(impl.over))
        impl.wait()
    return S, out


def absorb_rows(impl, q, W, heads, nope, latent, stride, scale, rows):
    P = getattr(impl, "ptr", _p)
    out = np.zeros((rows, heads * latent), np.uint16)
    if isinstance(impl, Port):
        impl.lib.oracle_attention_absorb_rows(_p(out), _p(q), _p(W), heads, nope, latent, stride, C.c_float(scale), rows)
    else:
        if rows == 1:
            impl.nn.attention_absorb(P(out), P(q), P(W), heads, nope, latent, stride, C.c_float(scale), P(impl.over))
        else:
            impl.nn.attention_absorb_rows(P(out), P(q), P(W), heads, nope, latent, stride, C.c_float(scale), rows, P(impl.over))
        impl.wait()
    return out


def expand_rows(impl, o, W, heads, width, latent, stride, offset, rows):
    P = getattr(impl, "ptr", _p)
    out = np.zeros((rows, heads * width), np.uint16)
    if isinstance(impl, Port):
        impl.lib.oracle_attention_expand_rows(_p(out), _p(o), _p(W), heads, width, latent, stride, offset, rows)
    else:
        if rows == 1:
            impl.nn.attention_expand(P(out), P(o), P(W), heads, width, latent, stride, offset, P(impl.over))
        else:
            impl.nn.attention_expand_rows(P(out), P(o), P(W), heads, width, latent, stride, offset, rows, P(impl.over))
        impl.wait()
    return out


def indexer(impl, x, lw, lb, keys, gates, ape, q, w, dim, kpool, heads, k, len0, rows, scale, src, block):
    """The indexer's doors one after another on one set of inputs: the LayerNorm of x; the pooled keys of every whole pool of
    the len0 + rows - 1 positions; the one-row scores, choice, block maxima and gather at position len0 - 1; and the rows
    forms for `rows` rows from it.  Answers a dict of every door's output."""
    P = getattr(impl, "ptr", _p)
    g = {}
    port = isinstance(impl, Port)
    nn, lib = (None, impl.lib) if port else (impl.nn, None)
    over = None if port else P(impl.over)
    n_pos = len0 + rows - 1
    pools_all, pools1 = n_pos // kpool, len0 // kpool
    g["ln"] = np.zeros_like(x)
    g["pooled"] = np.zeros((pools_all, dim), np.uint16)
    g["scores"] = np.zeros(max(pools1, 1), np.float32)
    g["index"] = np.zeros(min(k, max(pools1, 1)) * kpool + kpool, np.uint32)
    g["count"] = np.zeros(1, np.uint32)
    nblocks = (pools1 + block - 1) // block
    g["blocks"] = np.zeros(max(nblocks, 1), np.float32)
    srow = max(pools_all, 1)
    g["scores_rows"] = np.zeros((rows, srow), np.float32)
    irow = min(k, max(pools_all, 1)) * kpool + kpool
    g["index_rows"] = np.zeros((rows, irow), np.uint32)
    g["counts"] = np.zeros(rows, np.uint32)
    row = src.shape[1]
    tail = len0 - pools1 * kpool
    if port:
        lib.oracle_index_layernorm(_p(g["ln"]), _p(x), _p(lw), _p(lb), x.size, C.c_float(1e-5))
        lib.oracle_index_pool(_p(g["pooled"]), _p(keys), _p(gates), _p(ape), 0, pools_all, dim, kpool)
        lib.oracle_index_scores_rows(_p(g["scores"]), 0, _p(q), _p(w), _p(g["pooled"]), heads, dim, pools1, 0, 1, 0, C.c_float(scale))
        lib.oracle_index_select(_p(g["index"]), _p(g["count"]), _p(g["scores"]), pools1, k, kpool, pools1 * kpool, tail)
        lib.oracle_index_blocks(_p(g["blocks"]), _p(g["scores"]), pools1, block)
        lib.oracle_index_scores_rows(_p(g["scores_rows"]), srow, _p(q), _p(w), _p(g["pooled"]), heads, dim, 0, len0, kpool, rows, C.c_float(scale))
        lib.oracle_index_select_rows(_p(g["index_rows"]), irow, _p(g["counts"]), _p(g["scores_rows"]), srow, k, kpool, len0, rows)
    else:
        nn.index_layernorm(P(g["ln"]), P(x), P(lw), P(lb), x.size, C.c_float(1e-5), over)
        nn.index_pool(P(g["pooled"]), P(keys), P(gates), P(ape), 0, pools_all, dim, kpool, over)
        impl.wait()
        nn.index_scores(P(g["scores"]), P(q), P(w), P(g["pooled"]), heads, dim, pools1, C.c_float(scale))
        impl.wait()
        nn.index_select(P(g["index"]), P(g["count"]), P(g["scores"]), pools1, k, kpool, pools1 * kpool, tail)
        nn.index_blocks(P(g["blocks"]), P(g["scores"]), pools1, block)
        nn.index_scores_rows(P(g["scores_rows"]), srow, P(q), P(w), P(g["pooled"]), heads, dim, len0, kpool, rows, C.c_float(scale))
        impl.wait()
        nn.index_select_rows(P(g["index_rows"]), irow, P(g["counts"]), P(g["scores_rows"]), srow, k, kpool, len0, rows)
        impl.wait()
    n1 = int(g["count"][0])
    most = int(g["counts"].max())
    g["gathered"] = np.zeros((n1, row), np.uint16)
    g["gathered_rows"] = np.zeros((rows, most * row), np.uint16)
    if port:
        lib.oracle_index_gather_rows(_p(g["gathered"]), 0, _p(src), _p(g["index"]), 0, None, n1, row, 1)
        lib.oracle_index_gather_rows(_p(g["gathered_rows"]), most * row, _p(src), _p(g["index_rows"]), irow, _p(g["counts"]), most, row, rows)
    else:
        nn.index_gather(P(g["gathered"]), P(src), P(g["index"]), n1, row)
        nn.index_gather_rows(P(g["gathered_rows"]), most * row, P(src), P(g["index_rows"]), irow, P(g["counts"]), most, row, rows)
        impl.wait()
    return g


_port = None
_reference = None
_reference_tried = False


class OnCard:
    """This family on a card, worded as oracle/__init__.py's helpers word an implementation: `ptr(array)` is the address
    of the array's copy in device memory (made at first sight), `nn` the family's doors, `wait()` the family's
    compute_completed followed by every copy read back into its array — so a helper written for host pointers drives the
    card's doors unchanged."""

    def __init__(self, torch, fam):
        self.torch, self.fam, self.nn, self.over = torch, fam, fam.nn, None
        self.held = {}

    def ptr(self, a):
        if a is None:
            return None
        key = id(a)
        if key not in self.held:
            assert a.flags["C_CONTIGUOUS"]
            self.held[key] = (a, self.torch.from_numpy(a.view(np.uint8).reshape(-1)).cuda())
        return self.held[key][1].data_ptr()

    def wait(self):
        assert self.fam.sys.compute_completed(), "a door refused its launch"
        for a, t in self.held.values():
            if a.flags["WRITEABLE"] and a.size:
                a.view(np.uint8).reshape(-1)[:] = t.cpu().numpy()


def port() -> Port:
    global _port
    if _port is None:
        _port = Port()
    return _port


def reference() -> Reference | None:
    global _reference, _reference_tried
    if not _reference_tried:
        _reference_tried = True
        from . import build
        so = build.build_reference()
        if so is not None and so.exists():
            _reference = Reference(so)
    return _reference


_reference_cuda = None
_reference_cuda_tried = False


def reference_cuda():
    """The reference's own CUDA family (oracle/_ref/libsilvann_nvidia_cuda12.so, built by oracle/build.py) as a table of
    doors that take DEVICE addresses, bound to device 0 of the cards it counts — the same-card baseline.  None when the
    library is not there or counts no card on this machine."""
    global _reference_cuda, _reference_cuda_tried
    if not _reference_cuda_tried:
        _reference_cuda_tried = True
        from . import build
        so = build.build_reference_cuda()
        if so is not None and so.exists():
            from silvann_b200.abi import Family
            fam = Family(so)
            if fam.sys.device_count() >= 1 and fam.sys.bind_device(0) == 1:
                _reference_cuda = fam
    return _reference_cuda
