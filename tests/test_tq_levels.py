"""The level tables of the TurboQuant codes are part of the format.  Three witnesses must agree: the committed table the
kernels compile in (silvann_b200/csrc/tq_levels.inc), the construction that generates it (gen_tq_levels.py: Lloyd-Max
levels of a standard normal, 50,000 sweeps from levels evenly spaced over [-3, 3]), and what the reference's own
turboquant_decode door answers for every code (the golden fixture; the reference family itself where it is present)."""
import re
import sys
from pathlib import Path

import numpy as np

import oracle

ROOT = Path(__file__).resolve().parents[1]
INC = ROOT / "silvann_b200" / "csrc" / "tq_levels.inc"
WIDTHS = (1, 2, 3, 4, 5, 8)


def committed():
    text = re.sub(r"/\*.*?\*/", "", INC.read_text(), flags=re.S)
    bits = np.array([int(x, 16) for x in re.findall(r"0x([0-9A-Fa-f]{4})", text)], np.uint16)
    assert bits.size == 318
    out, at = {}, 0
    for w in WIDTHS:
        out[w] = bits[at:at + (1 << w)]
        at += 1 << w
    return out


def test_committed_table_equals_the_reference_doors_answers(golden, port, reference):
    table = committed()
    for w in WIDTHS:
        assert np.array_equal(table[w], golden[f"tq_levels_{w}"]), f"width {w}: committed table against the reference's decode door"
        assert np.array_equal(oracle.tq_levels(port, w), golden[f"tq_levels_{w}"]), f"width {w}: the C restatement"
        if reference is not None:
            assert np.array_equal(oracle.tq_levels(reference, w), table[w]), f"width {w}: the reference family, run here"


def test_the_construction_regenerates_the_committed_table():
    sys.path.insert(0, str(INC.parent))
    import gen_tq_levels
    table = committed()
    for w in WIDTHS:                     # width 8 is most of the minute this takes
        assert np.array_equal(gen_tq_levels.levels(w), table[w]), f"width {w}"
    assert gen_tq_levels.render(np.concatenate([table[w] for w in WIDTHS])) == INC.read_text()


def test_tables_are_mirrored_and_span_one():
    for w, lv in committed().items():
        f = oracle.from_bits(lv, oracle.FP16)
        assert f[0] == -1.0 and f[-1] == 1.0 and np.all(np.diff(f) > 0)
        assert np.array_equal(f, -f[::-1])
