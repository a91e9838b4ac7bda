"""GPU parity of RMSNorm (fp32), the op that sits before every matmul of a decoder layer.  The
reference's own test (src/host/test.c:82-140) draws inputs from [-20, 20], compares with its scalar
statement and accepts an absolute difference of 1e-5; the same gate is used here against the
double-accumulating oracle, through the raw entry point, the op registry and the RPC-named call."""
from __future__ import annotations

import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SHAPES = [(4096, 1), (4096, 8), (32, 3), (100, 5), (14336, 4), (8192, 2), (8196, 2), (20000, 3), (1, 7), (4, 300)]


def _input(ne0, ne1, seed):
    rng = np.random.Generator(np.random.PCG64([seed, ne0, ne1]))
    return (rng.random((ne1, ne0), dtype=np.float32) * 40.0 - 20.0).astype(np.float32)


def _request(pkg, dst, src, ne0, ne1):
    req = pkg.pack_rms_norm_request(dst, src, ne0, ne1)[8:]
    return ctypes.create_string_buffer(req, len(req))


@pytest.mark.parametrize("ne0,ne1", SHAPES)
def test_rms_norm_matches_oracle(dev, oracle, ne0, ne1):
    x = _input(ne0, ne1, 11)
    fx, fy = dev.put(x), dev.buf(x.nbytes)
    before = dev.lib.htp_b200_launch_count()
    buf = _request(dev.pkg, (fy, 0), (fx, 0), ne0, ne1)
    assert dev.lib.execute_op_simple(ctypes.cast(buf, ctypes.c_void_p)) == 0
    assert dev.lib.htp_b200_launch_count() == before + 1
    y = dev.get(fy, (ne1, ne0))
    ref = oracle.rms_norm_f32(x)
    assert np.isfinite(y).all()
    assert np.abs(y - ref).max() <= 1e-5, np.abs(y - ref).max()
    # the reference's float-accumulating scalar statement is within its own tolerance too
    assert np.abs(y - oracle.rms_norm_f32(x, wide=False)).max() <= 1e-5
    dev.free(fx, fy)


def test_rms_norm_in_place_and_zero_row(dev, oracle):
    """dst == src is what a decoder does; an all-zero row gives zeros (scale = 1/sqrt(eps))."""
    x = _input(4096, 4, 12)
    x[2] = 0.0
    fx = dev.put(x)
    buf = _request(dev.pkg, (fx, 0), (fx, 0), 4096, 4)
    assert dev.lib.execute_op_simple(ctypes.cast(buf, ctypes.c_void_p)) == 0
    y = dev.get(fx, (4, 4096))
    assert np.abs(y - oracle.rms_norm_f32(x)).max() <= 1e-5 and (y[2] == 0).all()
    dev.free(fx)


def test_rms_norm_rpc_named_call_and_rejections(dev, oracle):
    lib = dev.lib
    x = _input(512, 2, 13)
    fx, fy = dev.put(x), dev.buf(x.nbytes)
    h = lib.get_global_handle()
    assert lib.htp_ops_rms_norm_f32(h, fy, 0, fx, 0, 512, 2) == 0
    assert np.abs(dev.get(fy, (2, 512)) - oracle.rms_norm_f32(x)).max() <= 1e-5
    assert lib.htp_ops_rpc_rms_norm_f32(fy, 0, fx, 0, 512, 2) == 0
    before = lib.htp_b200_launch_count()
    assert lib.htp_ops_rms_norm_f32(h, fy, 0, fx, 0, 0, 2) != 0  # ne0 == 0 (rms_norm.c:69)
    assert lib.htp_ops_rms_norm_f32(h, fy, 0, fx, 0, 512, 0) != 0  # ne1 == 0
    assert lib.htp_ops_rms_norm_f32(h, fy, 4, fx, 0, 256, 2) != 0  # offset breaks the 128-byte alignment (:72)
    assert lib.htp_ops_rms_norm_f32(h, fy, 0, fx, 0, 512, 3) != 0  # region leaves its buffer
    assert lib.htp_ops_rms_norm_f32(h, 9999, 0, fx, 0, 512, 2) != 0  # unknown handle
    assert lib.htp_b200_launch_count() == before


def test_rms_norm_then_matmul_in_one_message(dev, oracle, wl):
    """A norm followed by the mat-vec that reads its output, as two requests of one message: the
    servicer keeps them in order."""
    pkg = dev.pkg
    wq, x = wl.random_case(31, 2, False, 1, 4096, 256)
    fx, fn, fw, fy = dev.put(x), dev.buf(x.nbytes), dev.put(wq), dev.buf(256 * 4)
    chan = pkg.MessageChannel(4096)
    try:
        states = chan.submit([
            pkg.pack_rms_norm_request((fn, 0), (fx, 0), 4096, 1),
            pkg.pack_matmul_request(pkg.HTP_OPS_MAT_MUL_PERMUTED_W4D16A32, (fy, 0), (fn, 0), (fw, 0), 1, 4096, 256),
        ])
    finally:
        chan.close()
    assert states == [0, 0]
    xn = oracle.rms_norm_f32(x)
    ref, absdot = oracle.mul_mat_f64(xn, wq, 256, 2, want_absdot=True)
    e = oracle.error_metrics(dev.get(fy, (1, 256)), ref, absdot)
    assert e["max_rel_to_max"] <= 2e-5 and e["max_cond_rel"] <= 2e-5, e
    dev.free(fx, fn, fw, fy)
