"""A minimal driver of the reference's own engine, built unmodified into oracle/_ref/ (oracle/build.py: build_engine).

TEST INFRASTRUCTURE.  The engine's Python module offers the calls of engine/src/pybind.cuh of the reference tree:
load_silicon_family(path) (399-406), choose_silicon(name) (370-374), boot(config=...) (334-361), kinds() / verbs(),
bindings_create, create_executable(cells), freeze, execute, release, and the byte movers nn.write / nn.read.  The
reference drives them from its Python runtime (runtime/silvann_runtime/machine.py: Machine.boot 230-253, Machine.buffer
625-640), which composes Lisp text into cells; that runtime does not travel with this repository, and none of it is
needed for what is tested here: one verb a program, its arguments numbers and buffers.  So a program is built directly
as the list of cells `(kind, verb, value)` that create_executable takes — a standard verb's cell first, then a value cell
for a number and an object reference for a buffer — and run the way Composer.run runs one (composer.py:583-594):
frozen into a picture, executed in the session's bindings, released.
"""
from __future__ import annotations

import importlib
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
REF_DIR = ROOT / "oracle" / "_ref"

# What nn's package init sizes its rooms from at a boot; a boot with any of these lines left out is refused.  The
# classes are small except `main`, which holds the K and V planes of the cases below.
_DEVICE_POOLS = {"resid": (4096, 48), "main": (16 << 20, 10), "attn_out": (1 << 20, 16), "logits": (8192, 8), "partials": (65536, 32)}
_RAM_POOLS = {"result": (65536, 16), "experts": (4096, 1), "table": (128, 1)}
_CARTRIDGES = {"sink": 4, "tq4": 16, "tq6": 16, "fp32": 16}


def _boot_text(alloc_mb: int) -> str:
    lines = []
    for name, (size, qty) in _DEVICE_POOLS.items():
        lines += [f"nn__buffer_{name}__size_bytes:{size}", f"nn__buffer_{name}__qty:{qty}"]
    for name, (size, qty) in _RAM_POOLS.items():
        lines += [f"nn__ram_buffer_{name}__size_bytes:{size}", f"nn__ram_buffer_{name}__qty:{qty}"]
    for name, tokens in _CARTRIDGES.items():
        lines += [f"nn__cartridge_{name}__tokens:{tokens}", f"nn__cartridge_{name}__bytes_per_token_layer:512"]
    lines += ["nn__expert_cache_l1__size_mb:8", "nn__model__kv_cache_layers_fullattn:1", "nn__model__kv_cache_layers_deltanet:3",
              "nn__conversation__text_size_kb:4", "nn__deltanet_state__bytes_per_layer:4096", "nn__model__layer_types:dddf"]
    return "boot_commands{\nsys__alloc_size_mb:%d\n}\ndevice_params{\n%s\n}\n" % (alloc_mb, "\n".join(lines))


def engine_module():
    """The reference engine's module, or None when oracle/_ref does not hold it."""
    if not any(REF_DIR.glob("silvann_engine_cpu*")):
        return None
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    return importlib.import_module("silvann_engine_cpu")


_loaded: dict[str, str] = {}


class Session:
    """One booted machine on one silicon family.  Only one can be up in a process at a time: close() before the next."""

    def __init__(self, family_path, silicon: str, alloc_mb: int = 64):
        self.e = e = engine_module()
        if e is None:
            raise RuntimeError("the reference engine is not built (python -m oracle.build where the reference tree is mounted)")
        path = str(family_path)
        if path not in _loaded:                      # a family is offered once a process; a second offer is refused
            _loaded[path] = e.load_silicon_family(path)
        if _loaded[path] != silicon:
            raise RuntimeError(f"{path} answered silicon {_loaded[path]!r}, not {silicon!r}")
        self.devices = e.devices(silicon)
        if self.devices < 1:
            raise RuntimeError(f"family {silicon} counts no device on this machine")
        e.choose_silicon(silicon)
        self.geometry = e.boot(config=_boot_text(alloc_mb))
        self.K, self.V = e.kinds(), e.verbs()
        self.env = e.bindings_create(512)
        self.OBJ = self.K["sys__object_reference"]
        self.held = []

    # cells
    def verb(self, name):
        return (self.K["sys__standard"], self.V[name], 0)

    def integer(self, n):
        return (self.K["sys__value_int"], 0, int(n))

    def buf(self, ref):
        return (self.OBJ, 0, ref)

    def run(self, name, *args, keep=False):
        """Runs `(name args...)`; an int argument is a number, a Buffer an object reference.  Answers (kind, value) and
        raises when the machine's fault channel says a door or the verb refused.  An answer that is an object arrives with
        a hold of its own (nothing the engine's interface hands out frees itself, pybind.cuh:510-512): it is given back
        here unless the caller keeps the object — a verb that answers its output buffer would otherwise pin that buffer
        out of its pool for good."""
        return self.run_cells(name, [self.buf(a.ref) if isinstance(a, Buffer) else self.integer(a) for a in args], keep=keep)

    def buffer(self, nbytes: int, payload: bytes | None = None) -> "Buffer":
        kind, ref = self.run("nn__buffer__getnew", nbytes, keep=True)
        if kind != self.OBJ:
            raise RuntimeError(f"a {nbytes}-byte buffer was refused: {self.e.sys.fault()}")
        at = self.e.sys.peek(self.e.sys.full_address(ref))[2][0]
        b = Buffer(self, ref, at, nbytes)
        if payload is not None:
            b.write(payload)
        self.held.append(b)
        return b

    def table(self, cells) -> int:
        """A node array of `cells` — a Buffer is an object reference, an int a number — as a model's verbs take their
        planes (the reference builds one with `(sys__create kind n)` and `(sys__node_array__set t i cell)`, machine.py:642-647).
        Answers the table's reference; release it with `release()`."""
        kind, ref = self._run_cells([self.verb("sys__create"), self.integer(self.K["sys__node_array"]), self.integer(len(cells))])
        if kind != self.K["sys__quoted_list"]:       # a constructor answers a datum: the reference, tagged quoted
            raise RuntimeError(f"a table of {len(cells)} cells was refused: ({kind}, {ref}) {self.e.sys.fault()}")
        for i, c in enumerate(cells):
            cell = self.buf(c.ref) if isinstance(c, Buffer) else self.integer(c)
            got = self._run_cells([self.verb("sys__node_array__set"), self.buf(ref), self.integer(i), cell])
            fault = self.e.sys.fault()
            if fault["raised"] != 0:
                self.e.sys.fault_clear()
                raise RuntimeError(f"cell {i} of the table was refused: {got} {fault}")
            if got[0] == self.OBJ:
                self.e.release(got[1])                   # the verb answers the value set, with a hold of the answer's own
        return ref

    def run_cells(self, name, cells, keep=False):
        """`(name cells...)` with the cells given as (kind, verb, value) triples already."""
        got = self._run_cells([self.verb(name)] + list(cells))
        fault = self.e.sys.fault()
        if fault["raised"] != 0:
            self.e.sys.fault_clear()
            raise RuntimeError(f"({name} ...) raised {fault}; answered {got}")
        if not keep and got[0] in (self.OBJ, self.K["sys__quoted_list"]):
            self.e.release(got[1])
        return got

    def _run_cells(self, cells):
        e = self.e
        prog = e.create_executable(cells)
        pic = e.freeze(prog)
        try:
            return e.execute((self.OBJ, 0, self.env), pic)
        finally:
            e.release(pic[2])
            e.release(prog[2])

    def release(self, ref):
        self.e.release(ref)

    def release_buffers(self):
        for b in self.held:
            self.e.release(b.ref)
        self.held = []

    def close(self):
        self.release_buffers()
        self.e.shutdown()


class Buffer:
    def __init__(self, session, ref, at, nbytes):
        self.s, self.ref, self.at, self.nbytes = session, ref, at, nbytes

    def write(self, data: bytes):
        self.s.e.nn.write(self.at, bytes(data))

    def read(self, nbytes: int | None = None) -> bytes:
        return self.s.e.nn.read(self.at, self.nbytes if nbytes is None else nbytes)
