"""Shared helpers for the GPU parity tests (everything goes through the C ABI)."""
import numpy as np
import pytest

import oracle as O


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def assert_bit_equal(got, want, what=""):
    got, want = np.asarray(got, np.float32), np.asarray(want, np.float32)
    assert got.shape == want.shape, (got.shape, want.shape)
    same = bits(got) == bits(want)
    if not same.all():
        bad = np.argwhere(~same)
        i = tuple(bad[0])
        raise AssertionError(f"{what}: {len(bad)} of {same.size} values differ in their bits; first at {i}: got {got[i]!r} want {want[i]!r}")


def rel_err(got, want, magnitude):
    """max |got - want| relative to the term magnitude (sum |w*x|), the reference's own yardstick."""
    return float(np.max(np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64)) / np.maximum(magnitude, 1e-6)))


@pytest.fixture(scope="session")
def backend():
    import orangu_b200

    be = orangu_b200.CudaBackend.init(0)  # raises with the reason: a GPU test never falls back
    yield be
    be.close()
