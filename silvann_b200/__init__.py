"""silvann_b200 — a B200 (sm_100a) attention silicon family for the SiLVANN engine.

The product is one shared library, lib/libsilvann_nvidia_b200.so (built from csrc/ by silvann_b200.build), whose C
boundary is include/silvann_b200.h.  This package is the thin host side used by the tests and the benchmark:

  abi     the door tables of any silicon family as ctypes callables
  ext     the `silvann_b200_*` extension entry points over raw device addresses
  verbs   the engine's attention / DeltaNet verbs (argument checks, door order) restated over those doors

There is no CPU fallback anywhere in this package: if the library is missing, loading raises.
"""
from __future__ import annotations

from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libsilvann_nvidia_b200.so"


class LibraryMissing(RuntimeError):
    pass


def library_path() -> Path:
    if not LIB_PATH.exists():
        raise LibraryMissing(
            f"{LIB_PATH} is not built. Run `python -m silvann_b200.build` (needs nvcc; no GPU needed to build). "
            "There is no CPU path in this package.")
    return LIB_PATH


_family = None


def family():
    """This library as a loaded silicon family (abi.Family)."""
    global _family
    if _family is None:
        from .abi import Family
        _family = Family(library_path())
    return _family
