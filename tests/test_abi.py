"""The C boundary without a GPU: the library loads, exports what include/silvann_b200.h declares, and lays its tables
out the way the engine reads them."""
import ctypes as C
import re
import shutil
import subprocess
from pathlib import Path

import pytest

import silvann_b200
from silvann_b200 import abi, ext

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "silvann_b200.h"
REFERENCE = __import__("oracle.build", fromlist=["REFERENCE_TREE"]).REFERENCE_TREE / "engine" / "src"   # where the reference tree is mounted, if it is


def test_library_is_built_and_loads():
    lib = C.CDLL(str(silvann_b200.library_path()))
    assert lib.silvann_silicon_family_get


def test_every_declared_symbol_is_exported():
    text = HEADER.read_text()
    declared = set(re.findall(r"\b(silvann_b200_[a-z_0-9]+|silvann_silicon_family_get)\s*\(", text))
    declared -= {"silvann_b200_family"}
    assert declared == set(ext.EXPORTS), declared ^ set(ext.EXPORTS)
    lib = C.CDLL(str(silvann_b200.library_path()))
    for name in sorted(declared):
        assert getattr(lib, name), name


def test_no_package_style_symbol_leaks():
    """The engine's build gate counts dynamic symbols shaped `<prefix>__...` (build_silicon_families.sh:73-79)."""
    out = subprocess.run(["nm", "-D", "--defined-only", str(silvann_b200.library_path())], capture_output=True, text=True, check=True).stdout
    names = [l.split()[-1] for l in out.splitlines() if l.strip()]
    assert "silvann_silicon_family_get" in names
    assert [n for n in names if re.match(r"^[a-z][a-z0-9_]*__", n)] == []


def test_family_table():
    f = silvann_b200.family()
    assert (f.table.abi_version, f.id, f.name, f.package_count) == (9, 310, "nvidia_b200", 7)
    assert f.table.size == C.sizeof(abi.FamilyTable) == 32
    assert f.package_sizes == [256, 1104, 4, 4, 4, 4, 4]
    assert f.refuses_other_versions


def test_no_door_is_null():
    f = silvann_b200.family()
    assert len(abi.SYS_DOORS) == 31 and len(abi.NN_DOORS) == 137
    for _, _, name, _ in abi.SYS_DOORS:
        assert getattr(f.sys, name) is not None, name
    for _, _, name, _ in abi.NN_DOORS:
        assert getattr(f.nn, name) is not None, name


def test_hot_door_indexes_match_the_contract():
    want = {"attention_scores": 25, "attention_mix": 26, "attention_weights": 28, "attention_residual_mix": 29,
            "attention_merge": 30, "attention_finish": 31, "deltanet_step": 34, "attention_causal_scores": 61,
            "attention_causal_mix": 62, "deltanet_steps": 66, "attention_scores_grouped": 95, "attention_softmax_rows": 96,
            "attention_causal_scores_grouped": 97, "attention_causal_softmax": 98, "vector_sum": 105, "deltanet_steps_gate": 133}
    for name, idx in want.items():
        assert abi.NN_INDEX[name] == idx, name


@pytest.mark.skipif(not REFERENCE.exists() or shutil.which("g++") is None, reason="needs the reference headers")
def test_layout_equals_the_reference_headers(tmp_path):
    """Every field of both door tables at the same offset with the same signature as the engine's own headers."""
    # doors that take a struct by value name the engine's struct type there and ours here: same layout (checked by
    # sizeof below), different C++ type, so their signatures are compared by offset only
    by_value = (abi.TqGroups, abi.ExpertGroups, abi.VectorParts)
    fields_nn = "\n".join(f"  static_assert(offsetof(nn__doors, {n}) == offsetof(silvann_b200_nn_doors, {n}), \"{n}\");\n"
                          + ("" if any(a in by_value for a in args) else
                             f"  static_assert(std::is_same<decltype(nn__doors::{n}), decltype(silvann_b200_nn_doors::{n})>::value, \"{n} signature\");")
                          for _, _, n, args in abi.NN_DOORS)
    fields_sys = "\n".join(f"  static_assert(offsetof(sys__doors, {n}) == offsetof(silvann_b200_sys_doors, {n}), \"{n}\");\n"
                           f"  static_assert(std::is_same<decltype(sys__doors::{n}), decltype(silvann_b200_sys_doors::{n})>::value, \"{n} signature\");"
                           for _, _, n, _ in abi.SYS_DOORS)
    src = tmp_path / "layout.cpp"
    src.write_text(f"""
#include <cstddef>
#include <type_traits>
#define SYS__SILICON_FAMILY__THIS layout_check
#define __device__
#include "packages/sys/contracts/abi/silicon_family.cuh"
#include "packages/sys/contracts/abi/gpu.cuh"
#include "packages/nn/contracts/abi/gpu.cuh"
#include "{HEADER}"
static_assert(sizeof(nn__doors) == sizeof(silvann_b200_nn_doors), "nn table size");
static_assert(sizeof(sys__doors) == sizeof(silvann_b200_sys_doors), "sys table size");
static_assert(sizeof(sys__silicon_family) == sizeof(silvann_b200_family), "family size");
static_assert(offsetof(sys__silicon_family, package_doors) == offsetof(silvann_b200_family, package_doors), "family");
static_assert(sizeof(nn__turboquant__groups) == sizeof(sv_tq_groups) && sizeof(nn__expert__groups) == sizeof(sv_expert_groups)
              && sizeof(nn__vector__parts) == sizeof(sv_vector_parts), "by-value structs");
static_assert(SYS__SILICON_FAMILY__ABI_VERSION == SILVANN_B200_ABI_VERSION, "abi version");
void check() {{
{fields_nn}
{fields_sys}
}}
""")
    r = subprocess.run(["g++", "-std=c++17", "-fsyntax-only", "-I", str(REFERENCE), str(src)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
