"""The drop-in claim, tested with the reference's own engine: its evaluator and its nn verbs, unmodified, load a family
by path (engine/src/pybind.cuh:399-406), boot on it and run `(nn__attention__decode ...)`, `(nn__attention__residual ...)`,
`(nn__attention__merge ...)`, `(nn__attention__finish ...)`, `(nn__attention__residual_tq ...)`, `(nn__deltanet__step ...)` and
`(nn__deltanet__conv_step ...)`
(engine/src/packages/nn/cpu/opcodes/attention__abi.cuh:120-243, deltanet__abi.cuh:55-125).

Without a GPU the family is the reference's own x86_avx2, and the answers must equal, bit for bit, the same doors called
directly — that pins the driver.  With a GPU the family is this repository's library, and the answers must be within 2e-3
of the reference family's; the library's own counters must show that the verb's two doors ran as ONE fused launch.
"""
import time

import numpy as np
import pytest

import oracle
import oracle.build
from oracle import FP16, to_bits
from tests import engine_driver
from tests.util import assert_close16

QH, KVH, D, N = 16, 4, 128, 8192


def _inputs(seed):
    rng = np.random.default_rng(seed)
    q = to_bits(rng.standard_normal((QH, D)).astype(np.float32) * 0.5, FP16)
    k = to_bits(rng.standard_normal((N, KVH, D)).astype(np.float32) * 0.5, FP16)
    v = to_bits(rng.standard_normal((N, KVH, D)).astype(np.float32) * 0.5, FP16)
    return q, k, v


def _u16(b, shape):
    return np.frombuffer(b, np.uint16).reshape(shape).copy()


def _f32(b, shape):
    return np.frombuffer(b, np.float32).reshape(shape).copy()


def _attention_forms(s, reference, exact):
    q, k, v = _inputs(41)
    qb, kb, vb = s.buffer(q.nbytes, q.tobytes()), s.buffer(k.nbytes, k.tobytes()), s.buffer(v.nbytes, v.tobytes())
    sb = s.buffer(QH * N * 4)
    ob = s.buffer(QH * D * 2)
    kind, value = s.run("nn__attention__decode", qb, kb, vb, sb, ob, QH, KVH, D, 0, N)
    assert kind == s.OBJ, "the verb answers its output buffer"
    got = _u16(ob.read(), (QH, D))
    want = reference.decode(q, k, v, QH, KVH, D, N)
    if exact:
        assert np.array_equal(got, want)
    else:
        assert_close16(got, oracle.from_bits(want, FP16), FP16, "decode through the engine")

    # a range that does not start at zero: the verb offsets K and V by `from` rows
    lo, hi = 1000, 5000
    s.run("nn__attention__decode", qb, kb, vb, sb, ob, QH, KVH, D, lo, hi)
    got = _u16(ob.read(), (QH, D))
    want = reference.decode(q, np.ascontiguousarray(k[lo:hi]), np.ascontiguousarray(v[lo:hi]), QH, KVH, D, hi - lo)
    if exact:
        assert np.array_equal(got, want)
    else:
        assert_close16(got, oracle.from_bits(want, FP16), FP16, "decode of a range through the engine")

    # two ranges as residuals, merged and finished: the tiered form (ai_qwen_3 mixer__abi.cuh:383-412)
    ra, rb = s.buffer(QH * (D + 2) * 4), s.buffer(QH * (D + 2) * 4)
    cut = 3000
    s.run("nn__attention__residual", qb, kb, vb, sb, ra, QH, KVH, D, 0, cut)
    s.run("nn__attention__residual", qb, kb, vb, sb, rb, QH, KVH, D, cut, N)
    s.run("nn__attention__merge", ra, rb, ra, QH, D)
    s.run("nn__attention__finish", ra, ob, QH, D)
    got = _u16(ob.read(), (QH, D))
    wa = reference.residual(q, np.ascontiguousarray(k[:cut]), np.ascontiguousarray(v[:cut]), QH, KVH, D, cut)
    wb = reference.residual(q, np.ascontiguousarray(k[cut:]), np.ascontiguousarray(v[cut:]), QH, KVH, D, N - cut)
    want = reference.finish(reference.merge(wa, wb, QH, D), QH, D)
    if exact:
        assert np.array_equal(got, want)
    else:
        assert_close16(got, oracle.from_bits(want, FP16), FP16, "residual, merge, finish through the engine")
    s.release_buffers()


def _deltanet_forms(s, reference, exact):
    kh, vh, d = 4, 8, 128
    rng = np.random.default_rng(43)
    S0 = (rng.standard_normal((vh, d, d)) * 0.1).astype(np.float32)
    conved = to_bits(rng.standard_normal((2 * kh + vh) * d).astype(np.float32), FP16)
    z = to_bits(rng.standard_normal(vh * d).astype(np.float32), FP16)
    beta = to_bits(rng.uniform(0.1, 0.9, vh).astype(np.float32), FP16)
    g = to_bits(-rng.uniform(0.01, 0.5, vh).astype(np.float32), FP16)
    w = to_bits((1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32), FP16)
    for gate in (0, 1):
        Sb = s.buffer(S0.nbytes, S0.tobytes())
        bufs = [s.buffer(a.nbytes, a.tobytes()) for a in (conved, z, beta, g, w)]
        out = s.buffer(vh * d * 2)
        args = [Sb] + bufs + [out, kh, vh, d] + ([gate] if gate else [])
        s.run("nn__deltanet__step", *args)
        got_o, got_S = _u16(out.read(), (1, vh * d)), _f32(Sb.read(), S0.shape)
        want_S = S0.copy()
        want_o = reference.deltanet(want_S, conved, z, beta, g, w, kh, vh, d, 1, gate)
        if exact:
            assert np.array_equal(got_o, want_o) and np.array_equal(got_S, want_S)
        else:
            assert_close16(got_o, oracle.from_bits(want_o, FP16), FP16, f"deltanet step, gate {gate}", tol=4e-3)
            scale = np.abs(want_S).max()
            assert np.abs(got_S - want_S).max() <= 1e-3 * scale, "deltanet state"
        s.release_buffers()

    # the convolution step ahead of it: (nn__deltanet__conv_step w state x out channels), four taps over a window of three
    ch = 2048
    wc = to_bits((rng.standard_normal(ch * 4) * 0.3).astype(np.float32), FP16)
    st = to_bits(rng.standard_normal(ch * 3).astype(np.float32), FP16)
    x = to_bits(rng.standard_normal(ch).astype(np.float32), FP16)
    wb, sb, xb, ob = s.buffer(wc.nbytes, wc.tobytes()), s.buffer(st.nbytes, st.tobytes()), s.buffer(x.nbytes, x.tobytes()), s.buffer(ch * 2)
    s.run("nn__deltanet__conv_step", wb, sb, xb, ob, ch)
    got_o, got_s = _u16(ob.read(), (ch,)), _u16(sb.read(), (ch * 3,))
    want_o, want_s = np.empty(ch, np.uint16), st.copy()
    reference.nn.deltanet_conv_step(oracle._p(want_o), oracle._p(want_s), oracle._p(wc), oracle._p(x), ch, oracle._p(reference.over))
    reference.wait()
    assert np.array_equal(got_s, want_s), "the window holds inputs, moved and not computed"
    if exact:
        assert np.array_equal(got_o, want_o)
    else:
        assert_close16(got_o, oracle.from_bits(want_o, FP16), FP16, "deltanet conv step")
    s.release_buffers()


def _tq_forms(s, reference, exact):
    """`(nn__attention__residual_tq q kcodes kscales vcodes vscales scores res q_heads kv_heads head_dim d count)`
    (attention__abi.cuh:245-272): the residual over a coded tier, finished with the plain verb."""
    qh, kvh, dh, L = 16, 4, 128, 2000
    rng = np.random.default_rng(47)
    q = to_bits(rng.standard_normal((qh, dh)).astype(np.float32), FP16)
    kr = to_bits(rng.standard_normal((L * kvh, dh)).astype(np.float32), FP16)
    vr = to_bits(rng.standard_normal((L * kvh, dh)).astype(np.float32), FP16)
    for d in (8, 4):
        kc, ks = oracle.tq_encode_rows(reference, kr, d)
        vc, vs = oracle.tq_encode_rows(reference, vr, d)
        bufs = [s.buffer(a.nbytes, a.tobytes()) for a in (q, kc, ks, vc, vs)]
        scores, res, out = s.buffer(2 * qh * L * 4), s.buffer(2 * qh * (dh + 2) * 4), s.buffer(qh * dh * 2)
        s.run("nn__attention__residual_tq", *bufs, scores, res, qh, kvh, dh, d, L)
        s.run("nn__attention__finish", res, out, qh, dh)
        got = _u16(out.read(), (qh, dh))
        want_res = oracle.residual_tq(reference, q, kc, ks, vc, vs, qh, kvh, dh, L, d)
        want = reference.finish(want_res, qh, dh)
        if exact:
            assert np.array_equal(got, want)
        else:
            assert_close16(got, oracle.from_bits(want, FP16), FP16, f"residual over a {d}-bit tier through the engine")
        s.release_buffers()


# the tiered mixer's table (engine/src/packages/ai_qwen_3/contracts/objects/mixer.cuh:56-107): seventeen planes, eleven
# numbers, eleven planes of the tiers, three tier sizes
MIX = dict(H=512, QH=4, KVH=2, HD=128, ROT=64, D_Q=4, D_K=8, D_V=4, D_O=8, THETA=10000, SINK=4, HOT=8, WARM=8, STEPS=30)


def _coded(reference, rng, rows, cols, d):
    w = to_bits((rng.standard_normal((rows, cols)) / np.sqrt(cols)).astype(np.float32), FP16)
    return oracle.tq_encode_rows(reference, w, d)


def _tiered_mixer(s, reference):
    """`(ai_qwen_3__attention_tiered x planes pos h1)` (engine/src/packages/ai_qwen_3/cpu/opcodes/mixer__abi.cuh:262-432), a
    position at a time from an empty cache until the sink, the hot ring and the warm ring are full and the cold tier has
    rows: the reference's whole attention mixer — norm and rotation, four coded projections, head norms, RoPE, the tiers'
    bookkeeping (rotate, encode at 8 bits, decode and encode again at 4), a residual a tier merged into one softmax, the
    gate, the out projection, the residual add — about forty door calls a position.  Answers h1 of every position and the
    tiers as they stand at the end."""
    m = MIX
    H, qh, kvh, hd, rot = m["H"], m["QH"], m["KVH"], m["HD"], m["ROT"]
    qw, kvw = qh * hd, kvh * hd
    rng = np.random.default_rng(53)
    mats = [_coded(reference, rng, 2 * qw, H, m["D_Q"]), _coded(reference, rng, kvw, H, m["D_K"]),
            _coded(reference, rng, kvw, H, m["D_V"]), _coded(reference, rng, H, qw, m["D_O"])]
    norms = [to_bits((1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32), FP16) for n in (H, hd, hd)]
    signs = to_bits(np.where(rng.random(512) < 0.5, -1.0, 1.0).astype(np.float32), FP16)
    xs = to_bits(rng.standard_normal((m["STEPS"], H)).astype(np.float32), FP16)
    cold_rows = m["STEPS"] - m["SINK"] - m["HOT"] - m["WARM"]
    rb8, rb4 = oracle.tq_row_bytes(8, hd), oracle.tq_row_bytes(4, hd)
    rw = 4 * qh * (hd + 2)

    def filled(a):
        return s.buffer(a.nbytes, a.tobytes())

    def room(nbytes):
        return s.buffer(nbytes, bytes(nbytes))

    planes = [filled(norms[0]),
              filled(mats[0][0]), filled(mats[0][1]), filled(mats[1][0]), filled(mats[1][1]),
              filled(mats[2][0]), filled(mats[2][1]), filled(mats[3][0]), filled(mats[3][1]),
              filled(norms[1]), filled(norms[2]),
              room(2 * m["SINK"] * kvw), room(2 * m["SINK"] * kvw),                           # the sink's keys and values
              room(4 * rot),                                                                   # this position's angles
              room(4 * qh * max(m["SINK"], m["HOT"], m["WARM"], cold_rows)),                   # scores
              filled(signs),
              room(2 * (2 * H + 2 * qw + kvw + 5 * qw + H))]                                    # the attention's scratch
    numbers = [H, qh, kvh, hd, rot, m["D_Q"], m["D_K"], m["D_V"], m["D_O"], m["THETA"], 0]
    tiers = [room(2 * m["HOT"] * kvw), room(2 * m["HOT"] * kvw),
             room(m["WARM"] * kvh * rb8), room(2 * m["WARM"] * kvh), room(m["WARM"] * kvh * rb8), room(2 * m["WARM"] * kvh),
             room(cold_rows * kvh * rb4), room(2 * cold_rows * kvh), room(cold_rows * kvh * rb4), room(2 * cold_rows * kvh),
             room(4 * rw + 2 * (2 * qw + 3 * kvw))]
    table = s.table(planes + numbers + tiers + [m["SINK"], m["HOT"], m["WARM"]])
    xb, hb = room(2 * H), room(2 * H)
    angles = planes[13]
    pairs = rot // 2
    freq = np.float64(m["THETA"]) ** (-2.0 * np.arange(pairs) / rot)
    h1 = np.zeros((m["STEPS"], H), np.uint16)
    seconds = []                                             # a position through the engine, its answer read back
    for pos in range(m["STEPS"]):
        a = pos * freq
        angles.write(np.concatenate([np.cos(a), np.sin(a)]).astype(np.float32).tobytes())
        xb.write(xs[pos].tobytes())
        t0 = time.perf_counter()
        kind, _ = s.run_cells("ai_qwen_3__attention_tiered", [s.buf(xb.ref), s.buf(table), s.integer(pos), s.buf(hb.ref)])
        assert kind == s.OBJ, f"position {pos}: the verb answers h1"
        h1[pos] = _u16(hb.read(), (H,))
        seconds.append(time.perf_counter() - t0)
    state = {"x": xs, "sink_k": _u16(planes[11].read(), (m["SINK"], kvw)), "hot_k": _u16(tiers[0].read(), (m["HOT"], kvw)),
             "warm_ks": _u16(tiers[3].read(), (m["WARM"] * kvh,)), "cold_ks": _u16(tiers[7].read(), (cold_rows * kvh,)),
             "warm_kc": np.frombuffer(tiers[2].read(), np.uint8).copy(), "cold_kc": np.frombuffer(tiers[6].read(), np.uint8).copy(),
             "seconds": seconds}
    s.release(table)
    s.release_buffers()
    return h1, state


ROWS_MIX = dict(H=512, QH=4, KVH=2, HD=128, ROT=64, D_Q=4, D_K=4, D_V=8, D_O=8, THETA=10000, CHUNKS=(64, 40, 1))


def _rows_mixer(s, reference):
    """`(ai_qwen_3__attention_rows x planes first h1 rows)` (engine/src/packages/ai_qwen_3/cpu/opcodes/prefill__abi.cuh:135-237): a
    prompt through the attention mixer a chunk of rows at a time — norm and rotation of every row, q and k through
    `expert_groups`, v and o through `expert_rows`, head norms and RoPE over the rows, the keys and values written into the
    cache, the three causal doors, the gate, the residual add.  Answers h1 of every row and the caches at the end."""
    m = ROWS_MIX
    H, qh, kvh, hd, rot = m["H"], m["QH"], m["KVH"], m["HD"], m["ROT"]
    qw, kvw = qh * hd, kvh * hd
    total, most = sum(m["CHUNKS"]), max(m["CHUNKS"])
    rng = np.random.default_rng(61)
    mats = [_coded(reference, rng, 2 * qw, H, m["D_Q"]), _coded(reference, rng, kvw, H, m["D_K"]),
            _coded(reference, rng, kvw, H, m["D_V"]), _coded(reference, rng, H, qw, m["D_O"])]
    norms = [to_bits((1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32), FP16) for n in (H, hd, hd)]
    signs = to_bits(np.where(rng.random(512) < 0.5, -1.0, 1.0).astype(np.float32), FP16)
    xs = to_bits(rng.standard_normal((total, H)).astype(np.float32), FP16)

    def filled(a):
        return s.buffer(a.nbytes, a.tobytes())

    def room(nbytes):
        return s.buffer(nbytes, bytes(nbytes))

    planes = [filled(norms[0]),
              filled(mats[0][0]), filled(mats[0][1]), filled(mats[1][0]), filled(mats[1][1]),
              filled(mats[2][0]), filled(mats[2][1]), filled(mats[3][0]), filled(mats[3][1]),
              filled(norms[1]), filled(norms[2]),
              room(2 * total * kvw), room(2 * total * kvw),                                    # the caches
              room(4 * most * rot),                                                            # the rows' angles
              room(4 * most * qh * total),                                                     # the rows' scores
              filled(signs),
              room(2 * most * (3 * H + 7 * qw + kvw) + 16 * 256 + 4096)]                        # pairs, then the rows' scratch
    numbers = [H, qh, kvh, hd, rot, m["D_Q"], m["D_K"], m["D_V"], m["D_O"], m["THETA"], 0]
    table = s.table(planes + numbers)
    h1 = np.zeros((total, H), np.uint16)
    seconds, first = [], 0
    for T in m["CHUNKS"]:
        xb, hb = filled(xs[first:first + T]), room(2 * T * H)
        t0 = time.perf_counter()
        kind, _ = s.run_cells("ai_qwen_3__attention_rows", [s.buf(xb.ref), s.buf(table), s.integer(first), s.buf(hb.ref), s.integer(T)])
        assert kind == s.OBJ, f"rows {first}..{first + T}: the verb answers h1"
        h1[first:first + T] = _u16(hb.read(), (T, H))
        seconds.append(time.perf_counter() - t0)
        first += T
    state = {"x": xs, "k": _u16(planes[11].read(), (total, kvw)), "v": _u16(planes[12].read(), (total, kvw)), "seconds": seconds}
    s.release(table)
    s.release_buffers()
    return h1, state


DN_MIX = dict(H=512, KH=2, VH=4, HD=128, D_QKV=4, D_Z=8, D_A=8, D_B=8, D_OUT=4, STEPS=12)


def _deltanet_mixer(s, reference):
    """`(ai_qwen_3__deltanet x planes h1)` (engine/src/packages/ai_qwen_3/cpu/opcodes/mixer__abi.cuh:15-90), a position at a
    time from an empty state: the norm and rotation, the four coded projections as one grouped launch, the gates, the
    conv over its window, every head's recurrence, the rotation and the out projection, the residual add.  Answers h1 of
    every position, and the state and the window as they stand at the end."""
    m = DN_MIX
    H, kh, vh, hd = m["H"], m["KH"], m["VH"], m["HD"]
    vdim, ch = vh * hd, 2 * kh * hd + vh * hd
    rng = np.random.default_rng(59)
    mats = [_coded(reference, rng, ch, H, m["D_QKV"]), _coded(reference, rng, vdim, H, m["D_Z"]), _coded(reference, rng, vh, H, m["D_A"]),
            _coded(reference, rng, vh, H, m["D_B"]), _coded(reference, rng, H, vdim, m["D_OUT"])]
    half = lambda a: to_bits(np.asarray(a, np.float32), FP16)
    norm_in, norm_w = half(1.0 + 0.1 * rng.standard_normal(H)), half(1.0 + 0.1 * rng.standard_normal(hd))
    conv_w = half(rng.standard_normal((ch, 4)) * 0.5)
    a_log, dt_bias = half(rng.uniform(-1.0, 1.0, vh)), half(rng.standard_normal(vh) * 0.5)
    signs = half(np.where(rng.random(512) < 0.5, -1.0, 1.0))
    xs = half(rng.standard_normal((m["STEPS"], H)))

    def filled(a):
        return s.buffer(a.nbytes, a.tobytes())

    def room(nbytes):
        return s.buffer(nbytes, bytes(nbytes))

    proj = ch + vdim + 2 * vh
    state, window = room(4 * vh * hd * hd), room(2 * ch * 3)
    planes = [filled(norm_in)]
    for codes, scales in mats[:4]:
        planes += [filled(codes), filled(scales)]
    planes += [filled(conv_w), filled(a_log), filled(dt_bias), filled(norm_w), filled(mats[4][0]), filled(mats[4][1]), state, window, filled(signs),
               filled(half([-1.0])), room(2 * (2 * H + proj + 2 * vh + ch + 2 * vdim + H))]
    numbers = [H, kh, vh, hd, m["D_QKV"], m["D_Z"], m["D_A"], m["D_B"], m["D_OUT"]]
    table = s.table(planes + numbers)
    xb, hb = room(2 * H), room(2 * H)
    h1 = np.zeros((m["STEPS"], H), np.uint16)
    seconds = []
    for pos in range(m["STEPS"]):
        xb.write(xs[pos].tobytes())
        t0 = time.perf_counter()
        kind, _ = s.run_cells("ai_qwen_3__deltanet", [s.buf(xb.ref), s.buf(table), s.buf(hb.ref)])
        assert kind == s.OBJ, f"position {pos}: the verb answers h1"
        h1[pos] = _u16(hb.read(), (H,))
        seconds.append(time.perf_counter() - t0)
    end = {"x": xs, "seconds": seconds, "state": _f32(state.read(4 * vh * hd * hd), (vh, hd, hd)), "window": _u16(window.read(2 * ch * 3), (ch, 3))}
    s.release(table)
    s.release_buffers()
    return h1, end


@pytest.fixture(scope="module")
def cpu_session(reference):
    if reference is None or engine_driver.engine_module() is None:
        pytest.skip("oracle/_ref holds no reference engine and family (built where the reference tree is mounted)")
    s = engine_driver.Session(oracle.build.REF, "x86_avx2")
    yield s
    s.close()


def test_engine_runs_reference_family(cpu_session, reference):
    _attention_forms(cpu_session, reference, exact=True)
    _deltanet_forms(cpu_session, reference, exact=True)
    _tq_forms(cpu_session, reference, exact=True)
    h1, state = _tiered_mixer(cpu_session, reference)
    again, _ = _tiered_mixer(cpu_session, reference)
    assert np.array_equal(h1, again), "the same program on the same family twice"
    assert np.isfinite(oracle.from_bits(h1, FP16)).all() and (h1 != state["x"]).mean() > 0.9, "every position's answer was written"
    assert state["warm_ks"].all() and state["cold_ks"].all() and state["hot_k"].any(axis=1).all(), "every tier holds rows at the end"
    h1, end = _deltanet_mixer(cpu_session, reference)
    again, _ = _deltanet_mixer(cpu_session, reference)
    assert np.array_equal(h1, again) and np.isfinite(oracle.from_bits(h1, FP16)).all() and (h1 != end["x"]).mean() > 0.9
    assert np.abs(end["state"]).max() > 1e-3 and end["window"].any(), "the state and the window were written"


@pytest.fixture(scope="module")
def mixer_on_reference_family(cuda, reference):
    """The tiered mixer run on the reference's own CPU family through the same engine, before this family's session boots
    (one machine is up at a time in a process): what the drop-in's answers are compared with."""
    if reference is None or engine_driver.engine_module() is None:
        pytest.fail("oracle/_ref holds no reference engine and family: build them where the reference tree is mounted")
    s = engine_driver.Session(oracle.build.REF, "x86_avx2")
    try:
        return _tiered_mixer(s, reference), _deltanet_mixer(s, reference), _rows_mixer(s, reference)
    finally:
        s.close()


@pytest.fixture(scope="module")
def gpu_session(cuda, mixer_on_reference_family):
    import silvann_b200
    if engine_driver.engine_module() is None:
        pytest.fail("oracle/_ref holds no reference engine: build it where the reference tree is mounted")
    s = engine_driver.Session(silvann_b200.library_path(), "nvidia_b200")
    yield s
    s.close()


@pytest.mark.gpu
def test_engine_runs_this_family(gpu_session, reference):
    from silvann_b200 import ext
    assert reference is not None
    before = ext.counters()
    _attention_forms(gpu_session, reference, exact=False)
    mid = ext.counters()
    assert mid["fused_decode"] - before["fused_decode"] == 2, "each decode verb is one fused launch"
    assert mid["fused_residual"] - before["fused_residual"] == 2, "each residual verb is one fused launch"
    _deltanet_forms(gpu_session, reference, exact=False)
    after = ext.counters()
    assert after["deltanet"] - mid["deltanet"] == 2
    _tq_forms(gpu_session, reference, exact=False)
    assert ext.counters()["refused"] == before["refused"]
    assert ext.device_status() == 0


@pytest.mark.gpu
def test_engine_runs_the_tiered_mixer_on_this_family(gpu_session, mixer_on_reference_family, reference):
    """The reference's whole attention mixer, a position at a time across every tier boundary, on this family against the
    same program on the reference's CPU family.  The tiers quantise what earlier positions wrote, so the two families'
    caches are compared too: a scale may differ by one fp16 step, and nearly every code must be the same."""
    from silvann_b200 import ext
    want, want_state = mixer_on_reference_family[0]
    before = ext.counters()
    got, state = _tiered_mixer(gpu_session, reference)
    after = ext.counters()
    print(f"tiered mixer through the engine: median {1e6 * np.median(state['seconds'][8:]):.0f} us a position on this family "
          f"({(after['launches'] - before['launches']) / MIX['STEPS']:.1f} launches a position), "
          f"{1e6 * np.median(want_state['seconds'][8:]):.0f} us on the reference's CPU family")
    assert after["refused"] == before["refused"] and ext.device_status() == 0
    m = MIX
    cold_steps = m["STEPS"] - m["SINK"] - m["HOT"] - m["WARM"]
    assert after["fused_residual"] - before["fused_residual"] >= m["STEPS"] + cold_steps, "the tiers' door pairs ran fused"
    err = np.abs(oracle.from_bits(got, FP16) - oracle.from_bits(want, FP16))
    print("tiered mixer: max |h1 - reference| a position:", np.round(err.max(axis=1), 5).tolist())
    assert err.max() <= 2e-3 * max(1.0, float(np.abs(oracle.from_bits(want, FP16)).max())), f"h1 differs by {err.max()}"
    for name in ("sink_k", "hot_k"):
        d = np.abs(oracle.from_bits(state[name], FP16) - oracle.from_bits(want_state[name], FP16))
        assert d.max() <= 4e-3, f"{name} differs by {d.max()}"
    for name in ("warm_ks", "cold_ks"):
        d = np.abs(state[name].astype(np.int32) - want_state[name].astype(np.int32))
        assert d.max() <= 1, f"{name}: a scale {d.max()} fp16 steps away"
    for name in ("warm_kc", "cold_kc"):
        same = (state[name] == want_state[name]).mean()
        assert same >= 0.97, f"{name}: only {same:.3f} of the code bytes are the reference's"


@pytest.mark.gpu
def test_engine_runs_the_deltanet_mixer_on_this_family(gpu_session, mixer_on_reference_family, reference):
    """The reference's Gated DeltaNet mixer, a position at a time from an empty state, on this family against the same
    program on the reference's CPU family: every position's answer, and the recurrent state and the conv window at the end."""
    from silvann_b200 import ext
    want, want_end = mixer_on_reference_family[1]
    before = ext.counters()
    got, end = _deltanet_mixer(gpu_session, reference)
    after = ext.counters()
    print(f"deltanet mixer through the engine: median {1e6 * np.median(end['seconds'][2:]):.0f} us a position on this family "
          f"({(after['launches'] - before['launches']) / DN_MIX['STEPS']:.1f} launches a position), "
          f"{1e6 * np.median(want_end['seconds'][2:]):.0f} us on the reference's CPU family")
    assert after["refused"] == before["refused"] and ext.device_status() == 0
    assert after["deltanet"] - before["deltanet"] == DN_MIX["STEPS"]
    err = np.abs(oracle.from_bits(got, FP16) - oracle.from_bits(want, FP16))
    print("deltanet mixer: max |h1 - reference| a position:", np.round(err.max(axis=1), 5).tolist())
    assert err.max() <= 2e-3 * max(1.0, float(np.abs(oracle.from_bits(want, FP16)).max())), f"h1 differs by {err.max()}"
    np.testing.assert_allclose(end["state"], want_end["state"], rtol=0, atol=1e-3 * np.abs(want_end["state"]).max())
    assert np.abs(oracle.from_bits(end["window"], FP16) - oracle.from_bits(want_end["window"], FP16)).max() <= 2e-3


@pytest.mark.gpu
def test_engine_runs_a_prompt_through_the_rows_mixer_on_this_family(gpu_session, mixer_on_reference_family, reference):
    """The reference's prompt path of the attention mixer, three chunks of rows (the second and third over a cache the earlier
    ones filled), on this family against the same program on the reference's CPU family: the projections are the expert-major
    GEMM doors and the attention is the three causal doors, which this family answers with one tcgen05 kernel each."""
    from silvann_b200 import ext
    want, want_state = mixer_on_reference_family[2]
    before = ext.counters()
    got, state = _rows_mixer(gpu_session, reference)
    after = ext.counters()
    chunks = len(ROWS_MIX["CHUNKS"])
    print(f"rows mixer through the engine: {[round(1e6 * t) for t in state['seconds']]} us a chunk of {list(ROWS_MIX['CHUNKS'])} rows on this family "
          f"({(after['launches'] - before['launches']) / chunks:.1f} launches a chunk), {[round(1e6 * t) for t in want_state['seconds']]} us on the reference's CPU family")
    assert after["refused"] == before["refused"] and ext.device_status() == 0
    assert after["expert_fast"] - before["expert_fast"] == 3 * chunks, "q and k in one launch, v, o: the projections ran on the tcgen05 kernel"
    assert after["fused_prefill"] - before["fused_prefill"] == chunks, "the three causal doors ran as one kernel a chunk"
    err = np.abs(oracle.from_bits(got, FP16) - oracle.from_bits(want, FP16))
    print("rows mixer: max |h1 - reference| a chunk:", [float(np.round(err[a:b].max(), 5)) for a, b in zip(np.cumsum((0,) + ROWS_MIX["CHUNKS"][:-1]), np.cumsum(ROWS_MIX["CHUNKS"]))])
    assert err.max() <= 2e-3 * max(1.0, float(np.abs(oracle.from_bits(want, FP16)).max())), f"h1 differs by {err.max()}"
    for name in ("k", "v"):
        d = np.abs(oracle.from_bits(state[name], FP16) - oracle.from_bits(want_state[name], FP16))
        assert d.max() <= 4e-3, f"the {name} cache differs by {d.max()}"
