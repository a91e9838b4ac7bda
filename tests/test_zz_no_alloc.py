"""The non-allocating decode entry point, htp_b200_mul_mat_static_scratch.

It exists for hosts that cannot call cudaMalloc while running - a server whose memory pools own
all of device memory, or a decode loop that cannot take an allocation's device-wide
synchronisation - and keeps its kernel scratch in a static device array shared by every call.
This test calls it through the C ABI twice in a row (the second call finds the first call's
leftovers in the array) and compares each result with the ordinary entry point's on the same
inputs.  It lives in the last-collected file so that a failure here cannot hide other tests.
"""
from __future__ import annotations

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(dev, fn, x, wq, n, wtype):
    lib = dev.lib
    m, k = x.shape
    fw, fx, fy = dev.put(wq), dev.put(x), dev.buf(m * n * 4)
    st = lib.htp_session_stream()
    rc = fn(lib.htp_buf_ptr(fy), lib.htp_buf_ptr(fx), lib.htp_buf_ptr(fw), m, k, n, wtype,
            1 if x.dtype == np.float16 else 0, st)
    assert rc == 0, rc
    assert lib.htp_session_synchronize() == 0
    y = dev.get(fy, (m, n))
    dev.free(fw, fx, fy)
    return y


def test_static_scratch_entry_point_matches_allocating_one(dev, oracle, wl):
    lib = dev.lib
    # two different shapes back to back: tiles cut by CTA boundaries in both, different formats
    # (the third and fourth: fp32 tokens on the wide integer path, which both entry points plan alike)
    cases = [(2, False, 1, 4096, 1024), (8, True, 5, 2048, 4000 // 32 * 32), (2, False, 8, 4096, 1024),
             (8, False, 7, 2048, 992), (20, False, 3, 1024, 224)]
    for wtype, act_f16, m, k, n in cases:
        wq, x = wl.random_case(500 + m, wtype, act_f16, m, k, n)
        ref = _run(dev, lib.htp_b200_mul_mat, x, wq, n, wtype)
        for _ in range(2):  # two calls in a row share the static array
            y = _run(dev, lib.htp_b200_mul_mat_static_scratch, x, wq, n, wtype)
            assert np.abs(y - ref).max() <= (1e-3 if act_f16 else 1e-5) * np.abs(ref).max()
            assert (y == ref).all()  # same kernel, same work split: the bytes agree too
        o = oracle.mul_mat_f64(x, wq, n, wtype)
        assert oracle.error_metrics(y, o)["max_rel_to_max"] <= (1e-3 if act_f16 else 1e-5)


def test_static_scratch_entry_point_rejects_what_it_cannot_hold(dev, wl):
    lib = dev.lib
    wq, x = wl.random_case(7, 2, False, 1, 256, 32)
    fw, fx, fy = dev.put(wq), dev.put(x), dev.buf(4096)
    w, a, y, st = lib.htp_buf_ptr(fw), lib.htp_buf_ptr(fx), lib.htp_buf_ptr(fy), lib.htp_session_stream()
    fn = lib.htp_b200_mul_mat_static_scratch
    assert fn(y, a, w, 9, 256, 32, 2, 0, st) == -3  # m beyond the decode range
    assert fn(y, a, w, 1, 96, 32, 2, 0, st) == -3  # k not a multiple of 256
    assert fn(y, a, w, 8, 14336, 32, 2, 0, st) == -3  # fragments of the whole k do not fit
    # the limits the header states: one K range only.  Q4_0, fp32: k = 14336 fits at m = 1, not at m = 2;
    # three to eight tokens: k <= 5632 (Q4_0, IQ4_NL) / 5888 (Q8_0)
    big = dev.buf(14336 // 32 * 34 * 32)
    wb = lib.htp_buf_ptr(big)
    xb = lib.htp_buf_ptr(dev.buf(8 * 14336 * 4))
    assert fn(y, xb, wb, 1, 14336, 32, 2, 0, st) == 0
    assert fn(y, xb, wb, 2, 14336, 32, 2, 0, st) == -3
    assert fn(y, xb, wb, 2, 9472, 32, 2, 0, st) == 0
    assert fn(y, xb, wb, 8, 5632, 32, 2, 0, st) == 0
    assert fn(y, xb, wb, 8, 5888, 32, 2, 0, st) == -3
    assert fn(y, xb, wb, 8, 5888, 32, 8, 0, st) == 0
    assert fn(y, xb, wb, 8, 6144, 32, 8, 0, st) == -3
    assert fn(y, xb, wb, 3, 5632, 32, 20, 1, st) == 0
    assert fn(y, a, w, 1, 256, 40, 2, 0, st) == -1  # the ordinary argument checks still apply
    assert fn(None, a, w, 1, 256, 32, 2, 0, st) == -1
    assert fn(y, a, w, 1, 256, 32, 2, 0, st) == 0
    assert lib.htp_session_synchronize() == 0
    dev.free(fw, fx, fy)
