"""The small steps either side of attention in a layer's mixer on a B200 — add, copies, RMS norm, the rotary angles and the
three rotations, the output gate — against outputs of the reference's CPU family (tests/golden/)."""
import ctypes as C

import numpy as np
import pytest

from oracle import from_bits
from util import dev, host_bits

pytestmark = pytest.mark.gpu


def one_ulp(got, want, what):
    d = np.abs(got.astype(np.int32) - want.astype(np.int32))
    assert (d <= 1).all(), f"{what}: {int(d.max())} fp16 steps"


def test_add_copy_norm_gate(cuda, fam, golden):
    g = golden
    x, y = dev(cuda, g["mx_add_x"]), dev(cuda, g["mx_add_y"])
    z = cuda.zeros_like(x)
    fam.nn.vector_add(z.data_ptr(), x.data_ptr(), y.data_ptr(), x.numel(), None)
    xr, w = dev(cuda, g["mx_norm_x"]), dev(cuda, g["mx_norm_w"])
    o = cuda.zeros((5, 256), dtype=cuda.int16, device="cuda")
    fam.nn.rmsnorm_rows(o.data_ptr(), xr.data_ptr(), w.data_ptr(), 256, 5, 300, 256, C.c_float(1e-6), None)
    x1, w1 = dev(cuda, g["mx_norm1_x"]), dev(cuda, g["mx_norm1_w"])
    o1 = cuda.zeros(2048, dtype=cuda.int16, device="cuda")
    fam.nn.rmsnorm(o1.data_ptr(), x1.data_ptr(), w1.data_ptr(), 2048, C.c_float(1e-5), None)
    att, qg = dev(cuda, g["mx_gate_att"]), dev(cuda, g["mx_gate_qg"])
    og = cuda.zeros_like(att)
    fam.nn.attention_gate_rows(og.data_ptr(), att.data_ptr(), qg.data_ptr(), 6, 64, None)
    src = dev(cuda, g["mx_copy_src"])
    dst = cuda.zeros((4, 40), dtype=cuda.int16, device="cuda")
    fam.nn.vector_copy_rows(dst.data_ptr(), 40, src.data_ptr(), 50, 33, 4)
    flat = cuda.zeros(200, dtype=cuda.int16, device="cuda")
    fam.nn.vector_copy(flat.data_ptr(), src.data_ptr(), 200)
    assert fam.sys.compute_completed()
    assert np.array_equal(host_bits(z), g["mx_add_z"])
    one_ulp(host_bits(o), g["mx_norm_o"], "rmsnorm_rows")          # the sum of squares is folded in the block's order
    one_ulp(host_bits(o1), g["mx_norm1_o"], "rmsnorm")
    one_ulp(host_bits(og), g["mx_gate_o"], "attention_gate_rows")  # expf on the card against libm's, then two roundings
    assert np.array_equal(host_bits(dst), g["mx_copy_dst"])
    assert np.array_equal(host_bits(flat), g["mx_copy_src"].reshape(-1))


def test_rotary_angles(cuda, fam, golden):
    g = golden
    for tag in "abc":
        theta, hd, pos = g[f"mx_ang_{tag}_args"]
        cs = cuda.zeros(int(hd), dtype=cuda.float32, device="cuda")
        fam.nn.rope_angles(cs.data_ptr(), int(pos), C.c_float(theta), int(hd))
        assert fam.sys.compute_completed()
        # same fp32 angle as the reference (r is made exactly as libm makes it); cosf/sinf on the card are within 2 ulps
        np.testing.assert_allclose(cs.cpu().numpy(), g[f"mx_ang_{tag}"], rtol=0, atol=5e-7)
    cs = cuda.zeros((4, 64), dtype=cuda.float32, device="cuda")
    fam.nn.rope_angles_rows(cs.data_ptr(), 100000, C.c_float(1e7), 64, 4)
    pos3 = dev(cuda, g["mx_ang_mrope_pos"])
    csm = cuda.zeros((4, 64), dtype=cuda.float32, device="cuda")
    fam.nn.rope_angles_mrope_rows(csm.data_ptr(), pos3.data_ptr(), C.c_float(1e7), 64, 4, 11 | (10 << 16))
    pos2 = dev(cuda, g["mx_ang_axial_pos"])
    csa = cuda.zeros((3, 72), dtype=cuda.float32, device="cuda")
    fam.nn.rope_angles_axial_rows(csa.data_ptr(), pos2.data_ptr(), C.c_float(1e4), 72, 3)
    assert fam.sys.compute_completed()
    np.testing.assert_allclose(cs.cpu().numpy(), g["mx_ang_rows"], rtol=0, atol=5e-7)
    np.testing.assert_allclose(csm.cpu().numpy(), g["mx_ang_mrope"], rtol=0, atol=5e-7)
    np.testing.assert_allclose(csa.cpu().numpy(), g["mx_ang_axial"], rtol=0, atol=5e-7)


def test_rotations(cuda, fam, golden):
    g = golden
    cs_a = cuda.from_numpy(g["mx_ang_a"]).cuda()
    cs_r = cuda.from_numpy(g["mx_ang_rows"]).cuda()
    xh = dev(cuda, g["mx_rope_x"])
    oh = cuda.zeros_like(xh)
    fam.nn.rope(oh.data_ptr(), xh.data_ptr(), cs_a.data_ptr(), 4, 64, None)
    xr = dev(cuda, g["mx_rope_rows_x"])
    fam.nn.rope_rows(xr.data_ptr(), xr.data_ptr(), cs_r.data_ptr(), 3, 2, 128, 256, 64, None)       # in place, partial: 64 of 128
    outs = []
    for inv in (0, 1):
        xi = dev(cuda, g["mx_rope_il_x"])
        at = xi.data_ptr() + 32 * 2                                                                  # a head's tail is what turns
        fam.nn.rope_interleaved(at, at, cs_a.data_ptr(), 3, 96, 64, inv, None)
        outs.append(xi)
    assert fam.sys.compute_completed()
    assert np.array_equal(host_bits(oh), g["mx_rope_o"])
    assert np.array_equal(host_bits(xr), g["mx_rope_rows_o"])
    for inv in (0, 1):
        assert np.array_equal(host_bits(outs[inv]), g[f"mx_rope_il_{inv}"])
    # turning one way and back is the identity up to two roundings
    back = from_bits(host_bits(outs[0]), 0)
    assert np.isfinite(back).all()


def test_weight_path_doors(cuda, fam, golden):
    """The whole-row rotation, a coded matrix times a vector (alone and as groups over one vector), the norm and rotation in
    one door.  The rotation's four sums are the reference's own, so it is bit for bit; a gemv's sum is folded over a block."""
    from silvann_b200.abi import TqGroups
    g = golden
    sign = dev(cuda, g["wp_sign"])
    for n in (96, 512, 896, 1152):
        x = dev(cuda, g[f"wp_rot_x_{n}"])
        o = cuda.zeros_like(x)
        fam.nn.hadamard_rotate(o.data_ptr(), x.data_ptr(), sign.data_ptr(), n, None)
        assert fam.sys.compute_completed()
        assert np.array_equal(host_bits(o), g[f"wp_rot_o_{n}"]), f"a row of {n}"
    xv = dev(cuda, g["wp_gemv_x"])
    cols = xv.numel()
    held = {}
    for d in (4, 8, 5):
        codes, scales = dev(cuda, g[f"wp_gemv_codes_{d}"]), dev(cuda, g[f"wp_gemv_scales_{d}"])
        rows = codes.shape[0]
        held[d] = (codes, scales, rows)
        o = cuda.zeros(rows, dtype=cuda.int16, device="cuda")
        fam.nn.turboquant_gemv(o.data_ptr(), codes.data_ptr(), codes.numel(), scales.data_ptr(), scales.numel() * 2, xv.data_ptr(), d, rows, cols, None)
        assert fam.sys.compute_completed()
        one_ulp(host_bits(o), g[f"wp_gemv_o_{d}"], f"gemv at {d} bits")
        # a room that holds fewer rows than named: those past it are left alone
        o2 = cuda.full((rows,), 0x1234, dtype=cuda.int16, device="cuda")
        short = (rows - 3) * (codes.numel() // rows)
        fam.nn.turboquant_gemv(o2.data_ptr(), codes.data_ptr(), short, scales.data_ptr(), scales.numel() * 2, xv.data_ptr(), d, rows, cols, None)
        assert fam.sys.compute_completed()
        got = host_bits(o2)
        one_ulp(got[:rows - 3], g[f"wp_gemv_o_{d}"][:rows - 3], "a short room")
        assert (got[rows - 3:] == 0x1234).all()
    gr = TqGroups()
    for i, d in enumerate((4, 8)):
        codes, scales, rows = held[d]
        gr.codes[i], gr.luts[i], gr.rows[i], gr.d[i], gr.out_at[i] = codes.data_ptr(), scales.data_ptr(), rows, d, (0, 48)[i]
    gr.count = 2
    og = cuda.zeros(68, dtype=cuda.int16, device="cuda")
    fam.nn.turboquant_gemv_groups(og.data_ptr(), gr, xv.data_ptr(), cols, None)
    assert fam.sys.compute_completed()
    one_ulp(host_bits(og), g["wp_groups_o"], "two groups over one vector")
    xn, wn = dev(cuda, g["wp_nr_x"]), dev(cuda, g["wp_nr_w"])
    h, hrot = cuda.zeros_like(xn), cuda.zeros_like(xn)
    fam.nn.rmsnorm_rotate(hrot.data_ptr(), h.data_ptr(), xn.data_ptr(), wn.data_ptr(), sign.data_ptr(), 896, C.c_float(1e-6), None)
    assert fam.sys.compute_completed()
    one_ulp(host_bits(h), g["wp_nr_h"], "the norm of rmsnorm_rotate")
    want = from_bits(g["wp_nr_hrot"], 0)
    assert np.abs(from_bits(host_bits(hrot), 0) - want).max() <= 2e-3 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("positions,heads,n,rot,x_stride", [(1, 16, 128, 64, 256), (1, 2, 256, 64, 256), (40, 4, 128, 128, 128), (7, 3, 64, 32, 80), (3, 2, 2048, 64, 2048)])
def test_norm_then_rope_over_the_same_rows_is_one_kernel_with_the_two_doors_bits(cuda, fam, positions, heads, n, rot, x_stride):
    """A mixer norms every head's row (rmsnorm_rows) and turns it in place (rope_rows): the pair is answered by one kernel,
    and its bits are those of the two doors run one after the other (a wait between them makes each run as worded)."""
    from silvann_b200 import ext
    rng = np.random.default_rng(positions * 100 + heads)
    rows = positions * heads
    x = cuda.from_numpy(rng.standard_normal((rows, x_stride)).astype(np.float16).view(np.int16)).cuda()
    w = cuda.from_numpy((1.0 + 0.1 * rng.standard_normal(n)).astype(np.float16).view(np.int16)).cuda()
    ang = rng.uniform(0, 6.28, (positions, rot // 2))
    cs = cuda.from_numpy(np.concatenate([np.cos(ang), np.sin(ang)], 1).astype(np.float32)).cuda()
    eps = C.c_float(1e-6)
    # as worded: a wait after the norm runs it alone
    want = cuda.zeros((rows, n), dtype=cuda.int16, device="cuda")
    fam.nn.rmsnorm_rows(want.data_ptr(), x.data_ptr(), w.data_ptr(), n, rows, x_stride, n, eps, None)
    assert fam.sys.compute_completed()
    normed = want.clone()
    fam.nn.rope_rows(want.data_ptr(), want.data_ptr(), cs.data_ptr(), positions, heads, n, heads * n, rot, None)
    assert fam.sys.compute_completed()
    # the pair as a mixer issues it
    before = ext.counters()
    got = cuda.zeros((rows, n), dtype=cuda.int16, device="cuda")
    fam.nn.rmsnorm_rows(got.data_ptr(), x.data_ptr(), w.data_ptr(), n, rows, x_stride, n, eps, None)
    fam.nn.rope_rows(got.data_ptr(), got.data_ptr(), cs.data_ptr(), positions, heads, n, heads * n, rot, None)
    assert fam.sys.compute_completed()
    after = ext.counters()
    assert after["fused_norm_rope"] - before["fused_norm_rope"] == 1 and after["refused"] == before["refused"]
    assert cuda.equal(got, want), "the fused pair's bits differ from the two doors'"
    assert not cuda.equal(got, normed), "the turn was applied"
    # a norm that nothing turns still runs, when the next door asks
    alone = cuda.zeros((rows, n), dtype=cuda.int16, device="cuda")
    other = cuda.zeros((rows, n), dtype=cuda.int16, device="cuda")
    fam.nn.rmsnorm_rows(alone.data_ptr(), x.data_ptr(), w.data_ptr(), n, rows, x_stride, n, eps, None)
    fam.nn.rope_rows(other.data_ptr(), normed.data_ptr(), cs.data_ptr(), positions, heads, n, heads * n, rot, None)   # not in place over the normed rows
    assert fam.sys.compute_completed()
    assert cuda.equal(alone, normed) and cuda.equal(other[:, :rot], want[:, :rot])      # (rope_rows writes the turned elements only)


@pytest.mark.parametrize("n", [128, 384, 512, 2048 + 384, 5120, 640])
def test_rmsnorm_rotate_is_one_kernel_with_the_two_doors_bits(cuda, fam, n):
    """rmsnorm_rotate is nn's rmsnorm followed by hadamard_rotate; here one kernel, and its two outputs must be the bits of the
    two doors called one after the other."""
    from silvann_b200 import ext
    rng = np.random.default_rng(n)
    x = cuda.from_numpy(rng.standard_normal(n).astype(np.float16).view(np.int16)).cuda()
    w = cuda.from_numpy((1.0 + 0.1 * rng.standard_normal(n)).astype(np.float16).view(np.int16)).cuda()
    sign = cuda.from_numpy(np.where(rng.random(512) < 0.5, -1.0, 1.0).astype(np.float16).view(np.int16)).cuda()
    eps = C.c_float(1e-6)
    o_want = cuda.zeros(n, dtype=cuda.int16, device="cuda")
    r_want = cuda.zeros(n, dtype=cuda.int16, device="cuda")
    fam.nn.rmsnorm(o_want.data_ptr(), x.data_ptr(), w.data_ptr(), n, eps, None)
    fam.nn.hadamard_rotate(r_want.data_ptr(), o_want.data_ptr(), sign.data_ptr(), n, None)
    assert fam.sys.compute_completed()
    o = cuda.zeros(n, dtype=cuda.int16, device="cuda")
    r = cuda.zeros(n, dtype=cuda.int16, device="cuda")
    before = ext.counters()["launches"]
    fam.nn.rmsnorm_rotate(r.data_ptr(), o.data_ptr(), x.data_ptr(), w.data_ptr(), sign.data_ptr(), n, eps, None)
    assert fam.sys.compute_completed()
    assert ext.counters()["launches"] == before + 1, "one kernel"
    assert cuda.equal(o, o_want), "the normed row"
    assert cuda.equal(r, r_want), "the rotated row"


@pytest.mark.parametrize("heads,hd", [(4, 128), (16, 128), (3, 128), (2, 256), (1, 64)])
def test_gate_then_rotation_is_one_kernel_with_the_two_doors_bits(cuda, fam, heads, hd):
    """A mixer gates its answers (attention_gate_rows) and rotates them for the output projection (hadamard_rotate): the pair
    is answered by one kernel with the bits of the two doors run apart."""
    from silvann_b200 import ext
    rng = np.random.default_rng(heads * 10 + hd)
    n = heads * hd
    att = cuda.from_numpy(rng.standard_normal(n).astype(np.float16).view(np.int16)).cuda()
    qg = cuda.from_numpy((rng.standard_normal((heads, 2 * hd)) * 2).astype(np.float16).view(np.int16)).cuda()
    sign = cuda.from_numpy(np.where(rng.random(512) < 0.5, -1.0, 1.0).astype(np.float16).view(np.int16)).cuda()
    g_want = cuda.zeros(n, dtype=cuda.int16, device="cuda")
    r_want = cuda.zeros(n, dtype=cuda.int16, device="cuda")
    fam.nn.attention_gate_rows(g_want.data_ptr(), att.data_ptr(), qg.data_ptr(), heads, hd, None)
    assert fam.sys.compute_completed()                                     # (a wait: the gate runs as worded)
    fam.nn.hadamard_rotate(r_want.data_ptr(), g_want.data_ptr(), sign.data_ptr(), n, None)
    assert fam.sys.compute_completed()
    g = cuda.zeros(n, dtype=cuda.int16, device="cuda")
    r = cuda.zeros(n, dtype=cuda.int16, device="cuda")
    before = ext.counters()
    fam.nn.attention_gate_rows(g.data_ptr(), att.data_ptr(), qg.data_ptr(), heads, hd, None)
    fam.nn.hadamard_rotate(r.data_ptr(), g.data_ptr(), sign.data_ptr(), n, None)
    assert fam.sys.compute_completed()
    after = ext.counters()
    shaped = n < 512 or (n % 512) % 128 == 0
    assert after["launches"] - before["launches"] == (1 if shaped else 2) and after["refused"] == before["refused"] + (0 if shaped else 1)
    assert cuda.equal(g, g_want), "the gated answers"
    if shaped:
        assert cuda.equal(r, r_want), "the rotated answers"
