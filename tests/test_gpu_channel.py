"""The drop-in boundary on the GPU: session, buffer table, execute_op_simple and the message
channel, exercised the way the reference's host test drives its channel
(src/host/test.c:166-204: compose, publish state.v[0], spin on state.v[1], read per-request state)."""
from __future__ import annotations

import ctypes
import struct

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_session_lifecycle(pkg, lib):
    assert lib.get_global_handle() == 2**64 - 1
    assert lib.htp_buf_alloc(64) == -1  # no session yet
    h = ctypes.c_uint64(0)
    assert lib.htp_ops_open(b"file:///libhtp_ops_skel.so?htp_ops_skel_handle_invoke&_modver=1.0&_dom=0",
                            ctypes.byref(h)) == 0
    assert h.value == lib.get_global_handle() != 2**64 - 1
    assert lib.execute_op_simple(None) == -1
    assert lib.htp_ops_init_backend(h) == 0
    assert lib.htp_ops_test_ops(h) == 0
    assert lib.htp_ops_rms_norm_f32(h, 0, 0, 0, 0, 32, 1) != 0  # handle 0 names no buffer
    assert lib.htp_ops_rpc_mat_mul_permuted_w16a32(0, 0, 0, 0, 0, 0, 1, 32, 32) != 0
    fd = lib.htp_buf_alloc(1000)
    assert fd > 0 and lib.htp_buf_size(fd) == 1000 and lib.htp_buf_is_host(fd) == 0
    assert lib.htp_buf_ptr(fd) % 256 == 0
    src = np.arange(250, dtype=np.int32)
    dst = np.zeros_like(src)
    assert lib.htp_buf_upload(fd, 0, src.ctypes.data, 1000) == 0
    assert lib.htp_buf_upload(fd, 8, src.ctypes.data, 1000) == -1  # beyond the buffer
    assert lib.htp_buf_download(fd, 0, dst.ctypes.data, 1000) == 0 and (src == dst).all()
    assert lib.htp_buf_free(fd) == 0 and lib.htp_buf_free(fd) == -1
    assert lib.htp_ops_close(h) == 0
    assert lib.get_global_handle() == 2**64 - 1


def test_execute_op_simple_rejections(dev, wl):
    """Every rejection the reference makes (-1 from mat_mul.c:878-892, unknown fd -> null pointer
    -> -1 via op_executor.cc:57-61) plus the bounds this library adds; nothing is launched."""
    lib, pkg = dev.lib, dev.pkg
    wq, x = wl.random_case(2, 2, False, 1, 256, 32)
    fw, fx, fy = dev.put(wq), dev.put(x), dev.buf(4096)
    op = pkg.HTP_OPS_MAT_MUL_PERMUTED_W4D16A32
    before = lib.htp_b200_launch_count()
    assert dev.execute(op, (fy, 0), (fx, 0), (fw, 0), 1, 256, 32) == 0
    assert lib.htp_b200_launch_count() == before + 1
    bad = [
        (op, (9999, 0), (fx, 0), (fw, 0), 1, 256, 32),  # unknown handle
        (op, (fy, 0), (fx, 0), (fw, 128), 1, 256, 32),  # weight region leaves its buffer
        (op, (fy, -4), (fx, 0), (fw, 0), 1, 256, 32),  # negative offset
        (op, (fy, 64), (fx, 0), (fw, 0), 1, 256, 32),  # offset breaks the 128-byte alignment
        (op, (fy, 0), (fx, 0), (fw, 0), 1, 250, 32),  # k % 32
        (op, (fy, 0), (fx, 0), (fw, 0), 1, 256, 40),  # n % 32
        (op, (fy, 0), (fx, 0), (fw, 0), 0, 256, 32),  # m == 0
        (op, (fy, 0), (fx, 0), (fw, 0), 2, 256, 32),  # activation region too small for m = 2
        (pkg.HTP_OPS_FLASH_ATTN_QO_F32_KV_F16, (fy, 0), (fx, 0), (fw, 0), 1, 256, 32),  # not built
        (77, (fy, 0), (fx, 0), (fw, 0), 1, 256, 32),  # unknown op index
    ]
    for args in bad:
        assert dev.execute(*args) == -1, args
    assert lib.htp_b200_launch_count() == before + 1
    dev.free(fw, fx, fy)


def test_message_channel_round_trip(dev, oracle, wl):
    """One message with five requests: two good matmuls (Q4_0 fp32-act, Q8_0 fp16-act), one invalid
    matmul, one map request, one no-op; all executed in order, each with its own return code."""
    lib, pkg = dev.lib, dev.pkg
    wq4, x4 = wl.random_case(41, 2, False, 3, 1024, 96)
    wq8, x8 = wl.random_case(42, 8, True, 1, 512, 64)
    f = {k: dev.put(v) for k, v in dict(w4=wq4, x4=x4, w8=wq8, x8=x8).items()}
    fy4, fy8 = dev.buf(3 * 96 * 4), dev.buf(64 * 4)
    chan = pkg.MessageChannel(4096)
    try:
        # a second channel while one is active is refused (reference commu.c:253-255)
        other = lib.htp_buf_alloc_host(4096)
        assert lib.create_htp_message_channel(other, 4096) != 0
        assert lib.htp_ops_create_channel(lib.get_global_handle(), other, 4096) != 0
        lib.htp_buf_free(other)
        reqs = [
            pkg.pack_matmul_request(pkg.HTP_OPS_MAT_MUL_PERMUTED_W4D16A32, (fy4, 0), (f["x4"], 0), (f["w4"], 0), 3,
                                    1024, 96),
            pkg.pack_matmul_request(pkg.HTP_OPS_MAT_MUL_PERMUTED_W4D16A32, (fy4, 0), (f["x4"], 0), (f["w4"], 0), 3,
                                    1000, 96),
            pkg.pack_map_request([f["x4"], f["w4"]]),
            struct.pack("<ii", 123, pkg.REQUEST_TYPE_NO_OP),
            pkg.pack_matmul_request(pkg.HTP_OPS_MAT_MUL_W8D16A16, (fy8, 0), (f["x8"], 0), (f["w8"], 0), 1, 512, 64),
        ]
        states = chan.submit(reqs)
        assert states == [0, -1, 0, 123, 0]
        y4, y8 = dev.get(fy4, (3, 96)), dev.get(fy8, (1, 64))
        assert oracle.error_metrics(y4, oracle.mul_mat_f64(x4, wq4, 96, 2))["max_rel_to_max"] <= 1e-5
        assert oracle.error_metrics(y8, oracle.mul_mat_f64(x8, wq8, 64, 8))["max_rel_to_max"] <= 1e-3
        # the channel is reusable: same message again, same bytes out
        assert chan.submit(reqs) == [0, -1, 0, 123, 0]
        assert (dev.get(fy4, (3, 96)) == y4).all()
        # a message whose offset table leaves the buffer is answered without executing anything
        chan.state.value = 0
        struct.pack_into("<Iii", chan.view, 8, 0, 1, 20)
        struct.pack_into("<i", chan.view, 24, 1 << 20)
        v = (ctypes.c_uint8 * 8).from_address(chan.base)
        v[0] = 1
        n = 0
        while v[1] != 1 and n < 100_000_000:
            n += 1
        assert v[1] == 1
    finally:
        chan.close()
    # after destroy a new channel can be created
    chan2 = pkg.MessageChannel(1024)
    assert chan2.submit([struct.pack("<ii", 5, pkg.REQUEST_TYPE_NO_OP)]) == [5]
    chan2.close()
    dev.free(*f.values(), fy4, fy8)


def test_chained_ops_in_one_message(dev, oracle, wl):
    """The output of one matmul is the activation of the next inside one message: stream order
    must hold although the second kernel prefetches its weights early."""
    lib, pkg = dev.lib, dev.pkg
    wa, x = wl.random_case(51, 2, False, 2, 1024, 512)
    wb, _ = wl.random_case(52, 2, False, 2, 512, 256)
    fwa, fwb, fx = dev.put(wa), dev.put(wb), dev.put(x)
    fh, fy = dev.buf(2 * 512 * 4), dev.buf(2 * 256 * 4)
    chan = pkg.MessageChannel(4096)
    try:
        op = pkg.HTP_OPS_MAT_MUL_PERMUTED_W4D16A32
        states = chan.submit([pkg.pack_matmul_request(op, (fh, 0), (fx, 0), (fwa, 0), 2, 1024, 512),
                              pkg.pack_matmul_request(op, (fy, 0), (fh, 0), (fwb, 0), 2, 512, 256)])
        assert states == [0, 0]
    finally:
        chan.close()
    h = dev.get(fh, (2, 512))
    y = dev.get(fy, (2, 256))
    ref = oracle.mul_mat_f64(h, wb, 256, 2)  # second stage checked on the first stage's GPU output
    assert oracle.error_metrics(h, oracle.mul_mat_f64(x, wa, 512, 2))["max_rel_to_max"] <= 1e-5
    assert oracle.error_metrics(y, ref)["max_rel_to_max"] <= 1e-5
    dev.free(fwa, fwb, fx, fh, fy)


def test_direct_calls_while_messages_are_in_flight(dev, oracle, wl):
    """The reference's host test mixes FastRPC-style direct calls with channel messages in one session
    (src/host/test.c).  A thread keeps posting messages of several matmuls while this thread issues
    htp_ops_rpc_rms_norm_f32 and execute_op_simple: the two share the session's operator state, which
    one lock serialises - every request state is 0 and every result stays right."""
    import threading
    lib, pkg = dev.lib, dev.pkg
    op = pkg.HTP_OPS_MAT_MUL_PERMUTED_W4D16A32
    shapes = [(1024, 256), (2048, 96), (512, 512), (1024, 64)]
    cases = [wl.random_case(2100 + i, 2, False, 2, k, n) for i, (k, n) in enumerate(shapes)]
    fw = [dev.put(wq) for wq, _ in cases]
    fx = [dev.put(x) for _, x in cases]
    fy = [dev.buf(2 * n * 4) for _, n in shapes]
    reqs = [pkg.pack_matmul_request(op, (fy[i], 0), (fx[i], 0), (fw[i], 0), 2, k, n) for i, (k, n) in enumerate(shapes)]
    src = (np.random.default_rng(5).random((16, 1024), dtype=np.float32) * 40 - 20).astype(np.float32)
    fsrc, fdst = dev.put(src), dev.buf(src.nbytes)
    wd, xd = wl.random_case(2200, 8, False, 3, 1024, 160)
    fwd, fxd, fyd = dev.put(wd), dev.put(xd), dev.buf(3 * 160 * 4)
    chan = pkg.MessageChannel(4096)
    bad = []

    def poster():
        for _ in range(60):
            st = chan.submit(reqs)
            if st != [0] * len(reqs):
                bad.append(st)
    t = threading.Thread(target=poster)
    try:
        t.start()
        for _ in range(60):
            assert lib.htp_ops_rpc_rms_norm_f32(fdst, 0, fsrc, 0, 1024, 16) == 0
            assert dev.execute(pkg.HTP_OPS_MAT_MUL_PERMUTED_W8D16A32, (fyd, 0), (fxd, 0), (fwd, 0), 3, 1024, 160) == 0
    finally:
        t.join()
        chan.close()
    assert not bad, bad[:2]
    for i, ((k, n), (wq, x)) in enumerate(zip(shapes, cases)):
        e = oracle.error_metrics(dev.get(fy[i], (2, n)), oracle.mul_mat_f64(x, wq, n, 2))
        assert e["max_rel_to_max"] <= 1e-5, e
    e = oracle.error_metrics(dev.get(fyd, (3, 160)), oracle.mul_mat_f64(xd, wd, 160, 8))
    assert e["max_rel_to_max"] <= 1e-5, e
    got = dev.get(fdst, src.shape)
    ref = src / np.sqrt((src.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-5)
    assert np.abs(got - ref).max() <= 1e-5
    dev.free(*fw, *fx, *fy, fsrc, fdst, fwd, fxd, fyd)


def test_shared_output_buffer_is_read_in_place(dev, oracle, wl):
    """A shared buffer - pinned host memory the device addresses, the counterpart of the reference's
    rpcmem buffers (src/host/test.c:30-53) - as the operator's OUTPUT: when the message is done the host
    reads the results through the buffer's own address, no download.  Decode and GEMM paths, and the
    buffer as an activation source as well."""
    import ctypes
    lib, pkg = dev.lib, dev.pkg
    for m, k, n, act_f16 in ((1, 1024, 2048, False), (8, 2048, 512, False), (64, 512, 256, True)):
        wq, x = wl.random_case(3100 + m, 2, act_f16, m, k, n)
        fw, fx = dev.put(wq), lib.htp_buf_alloc_shared(x.nbytes)
        fy = lib.htp_buf_alloc_shared(m * n * 4)
        assert fx > 0 and fy > 0 and lib.htp_buf_is_host(fy) == 2
        ctypes.memmove(lib.htp_buf_ptr(fx), x.ctypes.data, x.nbytes)  # the host writes the activations in place
        host_y = np.ctypeslib.as_array(ctypes.cast(lib.htp_buf_ptr(fy), ctypes.POINTER(ctypes.c_float)), shape=(m, n))
        host_y[:] = np.nan
        op = pkg.HTP_OPS_MAT_MUL_W4D16A16 if act_f16 else pkg.HTP_OPS_MAT_MUL_PERMUTED_W4D16A32
        chan = pkg.MessageChannel(4096)
        try:
            assert chan.submit([pkg.pack_matmul_request(op, (fy, 0), (fx, 0), (fw, 0), m, k, n)]) == [0]
        finally:
            chan.close()
        ref, absdot = oracle.mul_mat_f64(x, wq, n, 2, want_absdot=True)
        e = oracle.error_metrics(np.array(host_y), ref, absdot)
        tol = 1e-3 if act_f16 else 1e-5
        assert np.isfinite(host_y).all() and e["max_rel_to_max"] <= tol and e["max_cond_rel"] <= tol, e
        # the synchronous download of a shared buffer is a plain copy of the same bytes
        back = np.empty((m, n), dtype=np.float32)
        assert lib.htp_buf_download(fy, 0, back.ctypes.data, back.nbytes) == 0
        assert (back == host_y).all()
        dev.free(fw)
        assert lib.htp_buf_free(fx) == 0 and lib.htp_buf_free(fy) == 0
