"""Helpers shared by the GPU tests: numpy bit arrays <-> device tensors, and error measures."""
import numpy as np

import oracle


def dev(torch, bits_or_array):
    a = np.ascontiguousarray(bits_or_array)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).cuda()
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).cuda()
    return torch.from_numpy(a).cuda()


def host_bits(t):
    return t.cpu().numpy().view(np.uint16)


def f32(bits, dtype):
    return oracle.from_bits(bits, dtype)


def half_ulp(ref, dtype):
    """Half a unit in the last place of the 16-bit type at |ref| (elementwise), for the rounding-aware bound."""
    mant = 10 if dtype == 0 else 7
    a = np.maximum(np.abs(ref), 2.0 ** -14)
    return 2.0 ** (np.floor(np.log2(a)) - mant - 1)


def assert_close16(got_bits, want_f32, dtype, what, tol=2e-3):
    """max abs error <= tol, or <= half an ulp of the output type where that is larger (bf16 at |x| >= 1)."""
    got = f32(got_bits, dtype).reshape(want_f32.shape)
    err = np.abs(got - want_f32)
    bound = np.maximum(tol, half_ulp(want_f32, dtype) + tol / 2)
    worst = float((err - bound).max())
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    assert worst <= 0, f"{what}: max abs err {err.max():.3e} exceeds bound by {worst:.3e}"
    return float(err.max())


class OnCard:
    """This family on a card, worded as oracle/__init__.py's helpers word an implementation: `ptr(array)` is the address
    of the array's copy in device memory (made at first sight), `nn` the family's doors, `wait()` the family's
    compute_completed followed by every copy read back into its array — so a helper written for host pointers drives the
    card's doors unchanged."""

    def __init__(self, torch, fam):
        self.torch, self.fam, self.nn, self.over = torch, fam, fam.nn, None
        self.held = {}

    def ptr(self, a):
        if a is None:
            return None
        key = id(a)
        if key not in self.held:
            assert a.flags["C_CONTIGUOUS"]
            self.held[key] = (a, self.torch.from_numpy(a.view(np.uint8).reshape(-1)).cuda())
        return self.held[key][1].data_ptr()

    def wait(self):
        assert self.fam.sys.compute_completed(), "a door refused its launch"
        for a, t in self.held.values():
            if a.flags["WRITEABLE"] and a.size:
                a.view(np.uint8).reshape(-1)[:] = t.cpu().numpy()
