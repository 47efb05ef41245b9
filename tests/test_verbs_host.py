"""The verbs' refusals, with no device: the same checks and fault words as the engine's
(engine/src/packages/nn/cpu/opcodes/attention__abi.cuh:129-250)."""
import pytest

from silvann_b200 import verbs
from silvann_b200.verbs import FAULT_BOUNDS, FAULT_TYPE, VerbFault


class Buf:
    def __init__(self, halves, width=2):
        self.n, self.w = halves * 2 // width, width

    def numel(self): return self.n
    def element_size(self): return self.w
    def data_ptr(self): return 0x1000


class Recorder:
    """Stands in for a family: records which doors were called, in order."""
    def __init__(self):
        self.calls = []
        self.nn = self
    def __getattr__(self, name):
        def door(*a):
            self.calls.append(name)
        return door


def make():
    rec = Recorder()
    return rec, verbs.Verbs(rec)


def test_decode_calls_scores_then_mix():
    rec, v = make()
    v.attention_decode(Buf(16 * 128), Buf(100 * 512), Buf(100 * 512), Buf(2 * 16 * 100), Buf(16 * 128), 16, 4, 128, 0, 100)
    assert rec.calls == ["attention_scores", "attention_mix"]


def test_decode_refuses_an_empty_range_and_short_buffers():
    rec, v = make()
    args = dict(q=Buf(16 * 128), k=Buf(100 * 512), v=Buf(100 * 512), scores=Buf(2 * 16 * 100), out=Buf(16 * 128))
    with pytest.raises(VerbFault) as e:
        v.attention_decode(*args.values(), 16, 4, 128, 50, 50)
    assert e.value.word == FAULT_BOUNDS
    with pytest.raises(VerbFault) as e:
        v.attention_decode(*args.values(), 16, 4, 128, 0, 101)          # cache too short
    assert e.value.word == FAULT_BOUNDS
    with pytest.raises(VerbFault) as e:
        v.attention_decode(*args.values(), 16, 5, 128, 0, 100)          # heads do not divide
    assert e.value.word == FAULT_BOUNDS
    with pytest.raises(VerbFault) as e:
        v.attention_decode(*args.values(), 16, 4, 0, 0, 100)            # a dimension must be a positive integer
    assert e.value.word == FAULT_TYPE
    assert rec.calls == []


def test_residual_merge_finish_order_and_room():
    rec, v = make()
    res = Buf(2 * 16 * 130)
    v.attention_residual(Buf(16 * 128), Buf(100 * 512), Buf(100 * 512), Buf(2 * 16 * 60), res, 16, 4, 128, 40, 100)
    v.attention_merge(res, res, res, 16, 128)
    v.attention_finish(res, Buf(16 * 128), 16, 128)
    assert rec.calls == ["attention_weights", "attention_residual_mix", "attention_merge", "attention_finish"]
    with pytest.raises(VerbFault):
        v.attention_merge(res, Buf(10), res, 16, 128)
    with pytest.raises(VerbFault):
        v.attention_finish(res, Buf(16 * 128 - 1), 16, 128)


def test_causal_rows_pass_size_follows_the_scores_room():
    rec, v = make()
    qh, kvh, d, first, rows = 4, 2, 64, 10, 8
    scores = Buf(2 * qh * (first + rows) * 3)          # room for three rows a pass
    v.attention_causal_rows(Buf(rows * qh * d), Buf(18 * kvh * d), Buf(18 * kvh * d), scores, Buf(rows * qh * d), qh, kvh, d, first, rows)
    assert rec.calls == ["attention_causal_scores_grouped", "attention_causal_softmax", "attention_causal_mix"] * 3


def test_deltanet_step_gate_picks_the_door():
    rec, v = make()
    S, c, z, b, g, w, o = Buf(2 * 4 * 64 * 64), Buf(12 * 64), Buf(4 * 64), Buf(4), Buf(4), Buf(64), Buf(4 * 64)
    v.deltanet_step(S, c, z, b, g, w, o, 4, 4, 64)
    v.deltanet_step(S, c, z, b, g, w, o, 4, 4, 64, gate=1)
    assert rec.calls == ["deltanet_step", "deltanet_steps_gate"]
    with pytest.raises(VerbFault):
        v.deltanet_step(S, c, z, b, g, w, o, 3, 4, 64)
