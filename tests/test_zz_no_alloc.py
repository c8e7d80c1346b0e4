"""Allocation-free gradient-norm entry point (collected last on purpose).

ane_op_sumsq_noalloc exists for hosts that cannot let a library allocate device memory (they own
the whole device through their own arena, or they are inside a loop where an allocation would
stall the GPU).  It must give the same squared norm as ane_op_sumsq, on repeated calls that reuse
the library's fixed scratch array, and must refuse inputs larger than that array covers."""
import ctypes

import numpy as np
import pytest

import ane
from ane import _ffi

pytestmark = pytest.mark.gpu
lib = _ffi.lib


def _upload(a):
    p = lib.ane_dev_malloc(a.nbytes)
    assert lib.ane_dev_h2d(p, a.ctypes.data, a.nbytes) == 0
    return p


def _read_double(p):
    out = np.zeros(1, dtype=np.float64)
    assert lib.ane_dev_d2h(out.ctypes.data, p, 8) == 0
    return float(out[0])


def test_noalloc_matches_allocating_entry_point_twice():
    rng = np.random.default_rng(123)
    d_out = lib.ane_dev_malloc(8)
    # Two calls in a row with different sizes and contents: the second call sees the scratch the
    # first one left behind (more chunks than it needs) and must not be affected by it.
    for n, scale in ((3_000_001, 1.0 / 256.0), (70_001, 0.5)):
        g = rng.standard_normal(n).astype(np.float32)
        d_g = _upload(g)
        assert lib.ane_op_sumsq(d_g, n, scale, d_out) == 0, lib.ane_ops_last_error()
        assert lib.ane_dev_sync() == 0
        want = _read_double(d_out)
        assert lib.ane_dev_memset(d_out, 0, 8) == 0
        assert lib.ane_op_sumsq_noalloc(d_g, n, scale, d_out) == 0, lib.ane_op_sumsq_noalloc_last_error()
        assert lib.ane_dev_sync() == 0
        got = _read_double(d_out)
        host = float(np.sum((g.astype(np.float64) * np.float32(scale)) ** 2))
        # both sums run in double; they differ only by summation order
        assert abs(got - want) <= 1e-10 * abs(want)
        assert abs(got - host) <= 1e-6 * abs(host)
        lib.ane_dev_free(d_g)
    lib.ane_dev_free(d_out)


def test_noalloc_rejects_oversized_input_and_handles_empty():
    d_out = lib.ane_dev_malloc(8)
    d_g = lib.ane_dev_malloc(16)
    too_many = (1 << 28) + 1
    assert lib.ane_op_sumsq_noalloc(d_g, too_many, 1.0, d_out) == -1
    assert b"exceeds" in lib.ane_op_sumsq_noalloc_last_error()
    assert lib.ane_op_sumsq_noalloc(d_g, 0, 1.0, d_out) == 0
    assert lib.ane_dev_sync() == 0
    assert _read_double(d_out) == 0.0
    lib.ane_dev_free(d_g)
    lib.ane_dev_free(d_out)
