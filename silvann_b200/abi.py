"""ctypes view of the silicon-family C boundary declared in include/silvann_b200.h.

The door lists are read from the header itself, so the Python side cannot drift from the C side: `Family(path)` loads
any library that exports `silvann_silicon_family_get` — this repository's libsilvann_nvidia_b200.so, or any family the
SiLVANN engine builds — asks for ABI version 9 and exposes `family.sys.<door>` / `family.nn.<door>` as callables whose
argument types follow the header (reference contract: engine/src/packages/sys/contracts/abi/gpu.cuh:46-77 and
engine/src/packages/nn/contracts/abi/gpu.cuh:93-230).
"""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

HEADER = Path(__file__).resolve().parent.parent / "include" / "silvann_b200.h"
ABI_VERSION = 9
FAULT_OVERFLOW = 0x4E504F56


class TqGroups(C.Structure):
    _fields_ = [(n, C.c_uint64 * 12) for n in ("codes", "luts", "rows", "d", "out_at")] + [("count", C.c_uint64)]


class ExpertGroups(C.Structure):
    _fields_ = [(n, C.c_uint64 * 12) for n in ("codes", "luts", "out_rows", "d", "out_at", "pairs_at", "pairs")] + [("count", C.c_uint64)]


class VectorParts(C.Structure):
    _fields_ = [("at", C.c_uint64 * 8), ("count", C.c_uint64)]


class FamilyTable(C.Structure):
    _fields_ = [("abi_version", C.c_uint32), ("size", C.c_uint32), ("id", C.c_uint32), ("package_count", C.c_uint32),
                ("name", C.c_char_p), ("package_doors", C.POINTER(C.c_void_p))]


_SCALARS = {
    "sv_u64": C.c_uint64, "uint64_t": C.c_uint64, "size_t": C.c_size_t, "uint32_t": C.c_uint32, "unsigned int": C.c_uint32,
    "float": C.c_float, "bool": C.c_bool, "void": None, "sv_tq_groups": TqGroups, "sv_expert_groups": ExpertGroups,
    "sv_vector_parts": VectorParts,
}


def _ctype(decl: str):
    decl = decl.strip()
    if decl == "void":
        return None
    if "*" in decl:
        return C.c_char_p if decl.startswith("const char") else C.c_void_p
    words = decl.split()
    base = " ".join(words[:-1]) if len(words) > 1 else words[0]
    if base in _SCALARS:
        return _SCALARS[base]
    if decl in _SCALARS:
        return _SCALARS[decl]
    raise ValueError(f"unknown parameter type in door list: {decl!r}")


def _parse_doors(macro: str):
    """[(index, return type or None, name, [argument ctypes])] for one door-list macro of the header."""
    text = HEADER.read_text()
    start = text.index(f"#define {macro}(D)")
    body = text[start:text.index("\n\n", start)]
    doors = []
    for m in re.finditer(r"D\(\s*(\d+),\s*(?:(bool|void|uint32_t),\s*)?(\w+),\s*\((.*?)\)\)\s*\\?\s*$", body, re.M):
        idx, ret, name, params = int(m.group(1)), m.group(2), m.group(3), m.group(4)
        args = [a for a in (_ctype(p) for p in params.split(",")) if a is not None]
        doors.append((idx, _ctype(ret) if ret else None, name, args))
    doors.sort()
    assert [d[0] for d in doors] == list(range(len(doors))), f"{macro}: door indexes are not 0..n-1"
    return doors


SYS_DOORS = _parse_doors("SILVANN_B200_SYS_DOORS")
NN_DOORS = _parse_doors("SILVANN_B200_NN_DOORS")
NN_INDEX = {name: idx for idx, _, name, _ in NN_DOORS}
SYS_TABLE_BYTES = 8 + 8 * len(SYS_DOORS)
NN_TABLE_BYTES = 8 + 8 * len(NN_DOORS)


class _Doors:
    def __init__(self, table_addr: int, doors):
        self.size = C.c_uint32.from_address(table_addr).value
        self.names = [d[2] for d in doors]
        for idx, ret, name, args in doors:
            if 8 + 8 * (idx + 1) > self.size:
                continue
            fn_addr = C.c_void_p.from_address(table_addr + 8 + 8 * idx).value
            setattr(self, name, C.CFUNCTYPE(ret, *args)(fn_addr) if fn_addr else None)


class Family:
    """A loaded silicon family: its table, and its sys and nn doors as Python callables."""

    def __init__(self, path: str | Path):
        self.path = str(path)
        self.lib = C.CDLL(self.path, mode=C.RTLD_LOCAL)
        get = self.lib.silvann_silicon_family_get
        get.restype = C.POINTER(FamilyTable)
        get.argtypes = [C.c_uint32]
        self.refuses_other_versions = not bool(get(ABI_VERSION + 1)) and not bool(get(0))
        table = get(ABI_VERSION)
        if not table:
            raise RuntimeError(f"{path}: silvann_silicon_family_get({ABI_VERSION}) answered nothing")
        self.table = table.contents
        self.id = self.table.id
        self.name = self.table.name.decode()
        self.package_count = self.table.package_count
        self.package_sizes = [C.c_uint32.from_address(self.table.package_doors[i]).value for i in range(self.package_count)]
        self.sys = _Doors(self.table.package_doors[0], SYS_DOORS)
        self.nn = _Doors(self.table.package_doors[1], NN_DOORS)
