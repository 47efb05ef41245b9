"""The engine's attention and DeltaNet verbs, restated over a family's doors.

In SiLVANN a verb is the host half of an operation: it checks arity, types and buffer room, then calls doors in a
fixed order (engine/src/packages/nn/cpu/opcodes/attention__abi.cuh:129-272, deltanet__abi.cuh:99-131).  The same
checks and the same door order are written here against `abi.Family`, so a test can say
`verbs.attention_decode(q, k, v, scores, out, 16, 4, 128, 0, 8192)` exactly as a Lisp program says
`(nn__attention__decode q k v scores out 16 4 128 0 8192)` — and the doors underneath are this library's.

A buffer is anything with data_ptr(), numel() and element_size() (a torch tensor).  Room is counted in halves, as the
engine counts it: an fp32 buffer of n floats has room for 2n halves.  Refusals raise VerbFault carrying the engine's
four-letter fault word.
"""
from __future__ import annotations

FAULT_ARITY = 0x4F504341      # "OPCA"
FAULT_TYPE = 0x4F504354       # "OPCT"
FAULT_BOUNDS = 0x4E50424E     # "NPBN"
FAULT_NO_DEVICE = 0x4E504E44  # "NPND"
GATE_SILU, GATE_SIGMOID = 0, 1


class VerbFault(RuntimeError):
    def __init__(self, word: int, verb: str):
        super().__init__(f"{verb}: fault {word.to_bytes(4, 'big').decode()}")
        self.word = word


def _room(buf) -> int:
    return buf.numel() * buf.element_size() // 2


def _dim(x, verb) -> int:
    if not isinstance(x, int) or isinstance(x, bool) or x <= 0:
        raise VerbFault(FAULT_TYPE, verb)
    return x


class Verbs:
    def __init__(self, family, fault_word=None):
        """`family` is an abi.Family; `fault_word` a 4-byte device buffer the doors OR overflow codes into."""
        self.family = family
        self.nn = family.nn
        self.fault_word = fault_word

    def _over(self):
        return self.fault_word.data_ptr() if self.fault_word is not None else None

    def _range(self, verb, q, k, v, scores, out_room, q_heads, kv_heads, head_dim, lo, hi):
        q_heads, kv_heads, head_dim, hi = (_dim(x, verb) for x in (q_heads, kv_heads, head_dim, hi))
        if not isinstance(lo, int) or lo < 0:
            raise VerbFault(FAULT_TYPE, verb)
        row = kv_heads * head_dim
        if lo >= hi:                      # an empty range has no softmax
            raise VerbFault(FAULT_BOUNDS, verb)
        length, cached = hi - lo, hi * row
        if (q_heads % kv_heads != 0 or q_heads * head_dim > _room(q) or out_room is False or cached > _room(k)
                or cached > _room(v) or 2 * q_heads * length > _room(scores)):
            raise VerbFault(FAULT_BOUNDS, verb)
        if self.nn is None:
            raise VerbFault(FAULT_NO_DEVICE, verb)
        return length, lo * row * 2

    def attention_decode(self, q, k, v, scores, out, q_heads, kv_heads, head_dim, lo, hi):
        """(nn__attention__decode q k v scores out q_heads kv_heads head_dim from to) — attention__abi.cuh:129-160."""
        verb = "nn__attention__decode"
        length, skip = self._range(verb, q, k, v, scores, q_heads * head_dim <= _room(out), q_heads, kv_heads, head_dim, lo, hi)
        self.nn.attention_scores(scores.data_ptr(), q.data_ptr(), k.data_ptr() + skip, q_heads, kv_heads, head_dim, length)
        self.nn.attention_mix(out.data_ptr(), scores.data_ptr(), v.data_ptr() + skip, q_heads, kv_heads, head_dim, length, self._over())
        return out

    def attention_residual(self, q, k, v, scores, res, q_heads, kv_heads, head_dim, lo, hi):
        """(nn__attention__residual q k v scores res q_heads kv_heads head_dim from to) — attention__abi.cuh:181-213."""
        verb = "nn__attention__residual"
        ok = 2 * q_heads * (head_dim + 2) <= _room(res)
        length, skip = self._range(verb, q, k, v, scores, ok, q_heads, kv_heads, head_dim, lo, hi)
        self.nn.attention_weights(scores.data_ptr(), res.data_ptr(), q.data_ptr(), k.data_ptr() + skip, q_heads, kv_heads, head_dim, length)
        self.nn.attention_residual_mix(res.data_ptr(), scores.data_ptr(), v.data_ptr() + skip, q_heads, kv_heads, head_dim, length)
        return res

    def attention_merge(self, a, b, into, q_heads, head_dim):
        """(nn__attention__merge a b into q_heads head_dim) — attention__abi.cuh:217-233; `into` may be a or b."""
        verb = "nn__attention__merge"
        q_heads, head_dim = _dim(q_heads, verb), _dim(head_dim, verb)
        need = 2 * q_heads * (head_dim + 2)
        if any(need > _room(x) for x in (a, b, into)):
            raise VerbFault(FAULT_BOUNDS, verb)
        self.nn.attention_merge(into.data_ptr(), a.data_ptr(), b.data_ptr(), q_heads, head_dim)
        return into

    def attention_finish(self, res, out, q_heads, head_dim):
        """(nn__attention__finish res out q_heads head_dim) — attention__abi.cuh:236-250."""
        verb = "nn__attention__finish"
        q_heads, head_dim = _dim(q_heads, verb), _dim(head_dim, verb)
        if 2 * q_heads * (head_dim + 2) > _room(res) or q_heads * head_dim > _room(out):
            raise VerbFault(FAULT_BOUNDS, verb)
        self.nn.attention_finish(out.data_ptr(), res.data_ptr(), q_heads, head_dim, self._over())
        return out

    def attention_causal_rows(self, q, k, v, scores, out, q_heads, kv_heads, head_dim, first, rows):
        """The attention step of a prompt chunk as the layer verbs run it (attention__abi.cuh:397-405,
        ai_qwen_3 prefill__abi.cuh:213-217): as many rows a pass as the scores' room holds, each pass the three causal
        doors in order.  q, out [rows][q_heads][head_dim]; k, v hold rows 0..first+rows."""
        verb = "nn__attention__rows"
        q_heads, kv_heads, head_dim, rows = (_dim(x, verb) for x in (q_heads, kv_heads, head_dim, rows))
        to = first + rows
        qw, kvw = q_heads * head_dim, kv_heads * head_dim
        if q_heads % kv_heads != 0 or rows * qw > _room(q) or rows * qw > _room(out) or to * kvw > _room(k) or to * kvw > _room(v):
            raise VerbFault(FAULT_BOUNDS, verb)
        floats = _room(scores) // 2
        if floats < q_heads * to:
            raise VerbFault(FAULT_BOUNDS, verb)
        per_pass = min(rows, floats // (q_heads * to))
        for r0 in range(0, rows, per_pass):
            n = min(per_pass, rows - r0)
            self.nn.attention_causal_scores_grouped(scores.data_ptr(), q.data_ptr() + 2 * r0 * qw, k.data_ptr(), q_heads, kv_heads, head_dim, first + r0, n)
            self.nn.attention_causal_softmax(scores.data_ptr(), q_heads, first + r0, n)
            self.nn.attention_causal_mix(out.data_ptr() + 2 * r0 * qw, scores.data_ptr(), v.data_ptr(), q_heads, kv_heads, head_dim, first + r0, n, self._over())
        return out

    def deltanet_step(self, S, conved, z, beta, g, w, out, k_heads, v_heads, head_dim, gate=GATE_SILU):
        """(nn__deltanet__step S conved z beta g w out k_heads v_heads head_dim [gate]) — deltanet__abi.cuh:78-127."""
        verb = "nn__deltanet__step"
        k_heads, v_heads, d = _dim(k_heads, verb), _dim(v_heads, verb), _dim(head_dim, verb)
        if v_heads % k_heads != 0 or k_heads > v_heads or gate not in (GATE_SILU, GATE_SIGMOID):
            raise VerbFault(FAULT_BOUNDS, verb)
        if (2 * d * d * v_heads > _room(S) or (2 * k_heads + v_heads) * d > _room(conved) or v_heads * d > _room(z)
                or v_heads > _room(beta) or v_heads > _room(g) or d > _room(w) or v_heads * d > _room(out)):
            raise VerbFault(FAULT_BOUNDS, verb)
        if gate == GATE_SILU:
            self.nn.deltanet_step(S.data_ptr(), conved.data_ptr(), z.data_ptr(), beta.data_ptr(), g.data_ptr(), w.data_ptr(), out.data_ptr(),
                                  k_heads, v_heads, d, self._over())
        else:
            self.nn.deltanet_steps_gate(S.data_ptr(), conved.data_ptr(), z.data_ptr(), beta.data_ptr(), g.data_ptr(), w.data_ptr(), out.data_ptr(),
                                        k_heads, v_heads, d, 1, gate, self._over())
        return out

    def deltanet_rows(self, S, conved, z, beta, g, w, out, k_heads, v_heads, head_dim, rows, gate=GATE_SILU):
        """The recurrence over a prompt chunk, as ai_qwen_3__deltanet_rows ends (prefill__abi.cuh:109-116)."""
        verb = "ai_qwen_3__deltanet_rows"
        k_heads, v_heads, d, rows = (_dim(x, verb) for x in (k_heads, v_heads, head_dim, rows))
        if v_heads % k_heads != 0 or gate not in (GATE_SILU, GATE_SIGMOID):
            raise VerbFault(FAULT_BOUNDS, verb)
        if (2 * d * d * v_heads > _room(S) or rows * (2 * k_heads + v_heads) * d > _room(conved) or rows * v_heads * d > _room(z)
                or rows * v_heads > _room(beta) or rows * v_heads > _room(g) or d > _room(w) or rows * v_heads * d > _room(out)):
            raise VerbFault(FAULT_BOUNDS, verb)
        if gate == GATE_SILU:
            self.nn.deltanet_steps(S.data_ptr(), conved.data_ptr(), z.data_ptr(), beta.data_ptr(), g.data_ptr(), w.data_ptr(), out.data_ptr(),
                                   k_heads, v_heads, d, rows, self._over())
        else:
            self.nn.deltanet_steps_gate(S.data_ptr(), conved.data_ptr(), z.data_ptr(), beta.data_ptr(), g.data_ptr(), w.data_ptr(), out.data_ptr(),
                                        k_heads, v_heads, d, rows, gate, self._over())
        return out
