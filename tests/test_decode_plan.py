"""Host logic of the decode kernel's launch plan (no GPU): token padding, K ranges and ring depth as the
library computes them for a 227 KB shared-memory budget - the limits that include/htp_ops_b200.h states
for the non-allocating entry point, the configurations' shapes, and the argument checks."""
from __future__ import annotations

import ctypes

import pytest

Q4, Q8, IQ4 = 2, 8, 20
F32, F16 = 0, 1


def plan(lib, m, k, wt, at):
    r, rk, st = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    rc = lib.htp_b200_decode_plan(m, k, wt, at, ctypes.byref(r), ctypes.byref(rk), ctypes.byref(st))
    return rc, r.value, rk.value, st.value


def test_one_range_limits_match_the_header(lib):
    """Largest k that runs as ONE K range per (tokens, format, activation type), and the next one up."""
    table = [  # (tokens, format, activations, largest one-range k)
        (1, Q4, F32, 18944), (1, IQ4, F16, 18944), (1, Q8, F32, 23040), (1, Q8, F16, 46080),
        (2, Q4, F32, 9472), (2, IQ4, F32, 9472), (2, Q8, F32, 11520), (2, Q8, F16, 23040),
        (3, Q4, F32, 5632), (8, Q4, F16, 5632), (5, IQ4, F32, 5632), (8, Q8, F32, 5888), (3, Q8, F16, 5888),
    ]
    for m, wt, at, kmax in table:
        rc, ranges, range_k, stages = plan(lib, m, kmax, wt, at)
        assert (rc, ranges, range_k) == (0, 1, kmax) and stages >= 2, (m, wt, at, kmax, ranges, stages)
        rc, ranges, range_k, stages = plan(lib, m, kmax + 256, wt, at)
        assert rc == 0 and ranges >= 2 and range_k < kmax + 256, (m, wt, at, kmax)


def test_configuration_shapes(lib):
    # one token: every configuration's K is one range; K = 4096 with eight tokens rides a three-stage ring
    for k in (4096, 14336):
        assert plan(lib, 1, k, Q4, F32)[1] == 1
    assert plan(lib, 8, 4096, Q4, F32) == (0, 1, 4096, 3)
    assert plan(lib, 1, 4096, Q8, F16)[1:3] == (1, 4096)
    # config 3's down projection with eight tokens: four ranges of whole 2048-weight stages
    rc, ranges, range_k, stages = plan(lib, 8, 14336, Q4, F32)
    assert (rc, ranges, range_k) == (0, 4, 4096) and stages >= 2 and range_k % 2048 == 0
    rc, ranges, range_k, _ = plan(lib, 8, 14336, Q8, F32)
    assert rc == 0 and ranges * range_k >= 14336 and range_k % 1024 == 0  # Q8_0 stages hold 1024 weights


def test_plan_rejects_what_the_decode_kernel_does_not_take(lib):
    assert plan(lib, 0, 4096, Q4, F32)[0] == -1
    assert plan(lib, 9, 4096, Q4, F32)[0] == -1
    assert plan(lib, 1, 4000, Q4, F32)[0] == -1  # k % 256
    assert plan(lib, 1, 4096, 3, F32)[0] == -1  # unknown format
    assert plan(lib, 1, 4096, 1, F32)[0] == -1  # tile-order formats have their own kernel
    assert plan(lib, 1, 4096, Q4, 7)[0] == -1
    assert lib.htp_b200_decode_plan(1, 4096, Q4, F32, None, None, None) == 0
