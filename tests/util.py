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


OnCard = oracle.OnCard
