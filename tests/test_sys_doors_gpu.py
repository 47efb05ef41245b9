"""The sys doors over the CUDA runtime: memory, copies, the side channel, marks, and the refused-launch rule."""
import ctypes as C

import numpy as np
import pytest

from silvann_b200 import ext

pytestmark = pytest.mark.gpu


def test_devices(fam):
    assert fam.sys.device_count() >= 1
    assert fam.sys.bind_device(0) == 1 and fam.sys.bound_device() == 0
    assert fam.sys.bind_device(1000) == 0
    assert fam.sys.peer_access(0)


def test_memory_round_trip_and_zerofill(fam):
    at = C.c_void_p()
    assert fam.sys.memory_allocate(C.byref(at), 1 << 20)
    src = np.arange(1 << 18, dtype=np.uint32)
    assert fam.sys.memory_write(at, src.ctypes.data, src.nbytes)
    back = np.zeros_like(src)
    assert fam.sys.memory_read(back.ctypes.data, at, src.nbytes) and np.array_equal(src, back)
    assert fam.sys.memory_zerofill(at, src.nbytes)
    assert fam.sys.memory_read(back.ctypes.data, at, src.nbytes) and not back.any()
    assert not fam.sys.memory_allocate(C.byref(C.c_void_p()), 1 << 50)        # past what the card has free
    fam.sys.memory_free(at)


def test_side_channel_and_marks(fam):
    dev_at, chan, mark = C.c_void_p(), C.c_void_p(), C.c_void_p()
    host, card = C.c_void_p(), C.c_void_p()
    n = 1 << 22
    assert fam.sys.memory_allocate(C.byref(dev_at), n)
    assert fam.sys.memory_allocate_host_ram_mapped(C.byref(host), C.byref(card), n)
    assert fam.sys.side_open(C.byref(chan)) and fam.sys.mark_open(C.byref(mark))
    src = np.ctypeslib.as_array(C.cast(host, C.POINTER(C.c_uint8)), shape=(n,))
    src[:] = np.arange(n, dtype=np.uint8)
    assert fam.sys.side_memory_write_queued(dev_at, host, n, chan)             # pinned tier -> card, not waited for
    assert fam.sys.side_mark_record(mark, chan)
    assert fam.sys.mark_wait(mark)                                             # the compute queue waits on the device
    assert fam.sys.mark_reached(mark)                                          # and the caller can wait too
    back = np.zeros(n, np.uint8)
    assert fam.sys.side_memory_read(back.ctypes.data, dev_at, n, chan) and np.array_equal(back, src)
    assert fam.sys.mark_record(mark) and fam.sys.mark_reached(mark)
    fam.sys.mark_close(mark); fam.sys.side_close(chan)
    fam.sys.memory_free_host_ram(host); fam.sys.memory_free(dev_at)


def test_file_read_lands_in_device_memory(fam, tmp_path):
    data = np.random.default_rng(0).integers(0, 255, size=300000, dtype=np.uint8)
    path = tmp_path / "blob.bin"; path.write_bytes(data.tobytes())
    h, at = C.c_uint64(), C.c_void_p()
    assert fam.sys.file_open(str(path).encode(), C.byref(h)) and h.value != 0
    assert fam.sys.memory_allocate(C.byref(at), 200000)
    assert fam.sys.file_read(h.value, 1234, 200000, at)
    back = np.zeros(200000, np.uint8)
    assert fam.sys.memory_read(back.ctypes.data, at, 200000) and np.array_equal(back, data[1234:201234])
    assert not fam.sys.file_read(h.value, 250000, 200000, at)                   # past the end of the file
    fam.sys.file_close(h.value); fam.sys.memory_free(at)
    assert not fam.sys.file_open(b"/nonexistent/file", C.byref(h))
    assert not fam.sys.memory_map_file(at, 4096, 1, 0) and fam.sys.memory_prefetch(at, 4096)


def test_an_unanswered_door_refuses_once_and_the_device_stays_usable(fam, cuda):
    """A door this family does not answer prints a line and makes the device's next compute_completed answer false
    once — the engine raises that as SEWK and carries on (nvidia_cuda12/sys.cuh:41-61)."""
    before = ext.counters()["refused"]
    t = cuda.zeros(64, dtype=cuda.int16, device="cuda")
    fam.nn.vector_zero(t.data_ptr(), 64)
    assert ext.counters()["refused"] == before + 1
    assert fam.sys.compute_completed() is False
    assert fam.sys.compute_completed() is True


def test_vector_sum_in_the_given_order(fam, cuda):
    from silvann_b200.abi import VectorParts
    rng = np.random.default_rng(1)
    parts = [cuda.from_numpy(rng.standard_normal(1000).astype(np.float16)).cuda() for _ in range(5)]
    out = cuda.zeros(1000, dtype=cuda.float16, device="cuda")
    vp = VectorParts()
    for i, p in enumerate(parts):
        vp.at[i] = p.data_ptr()
    vp.count = 5
    fam.nn.vector_sum(out.data_ptr(), vp, 1000, None)
    assert fam.sys.compute_completed()
    want = sum(p.float() for p in parts).half()
    assert cuda.equal(out, want)
