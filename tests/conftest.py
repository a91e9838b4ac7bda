"""Shared fixtures.  Tests marked `gpu` need a CUDA device and call through the C ABI of
libhtp_ops_b200.so; everything else runs on CPU only."""
from __future__ import annotations

import ctypes
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    return entry.load_package()


@pytest.fixture(scope="session")
def wl(pkg):
    from htp_ops_lib_b200 import workloads
    return workloads


@pytest.fixture(scope="session")
def oracle():
    mod = entry.load_oracle()
    mod.load()
    return mod


@pytest.fixture(scope="session")
def lib(pkg):
    """The loaded shared library (no session opened)."""
    return pkg.load()


class Device:
    """Small convenience layer over the C host API for the GPU tests: buffers in, buffers out."""

    def __init__(self, pkg, lib):
        self.pkg, self.lib = pkg, lib
        self.fds = []

    def buf(self, nbytes: int) -> int:
        fd = self.lib.htp_buf_alloc(max(int(nbytes), 1))
        assert fd > 0
        self.fds.append(fd)
        return fd

    def put(self, arr: np.ndarray) -> int:
        arr = np.ascontiguousarray(arr)
        fd = self.buf(arr.nbytes)
        assert self.lib.htp_buf_upload(fd, 0, arr.ctypes.data, arr.nbytes) == 0
        return fd

    def get(self, fd: int, shape, dtype=np.float32, offset: int = 0) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        assert self.lib.htp_buf_download(fd, offset, out.ctypes.data, out.nbytes) == 0
        return out

    def free(self, *fds):
        for fd in fds:
            self.lib.htp_buf_free(fd)
            if fd in self.fds:
                self.fds.remove(fd)

    def free_all(self):
        self.free(*list(self.fds))

    def op_index(self, wtype: int, act_f16: bool) -> int:
        p = self.pkg
        return {(2, False): p.HTP_OPS_MAT_MUL_PERMUTED_W4D16A32, (8, False): p.HTP_OPS_MAT_MUL_PERMUTED_W8D16A32,
                (2, True): p.HTP_OPS_MAT_MUL_W4D16A16, (8, True): p.HTP_OPS_MAT_MUL_W8D16A16}[(wtype, act_f16)]

    def execute(self, op: int, out, act, weight, m, k, n) -> int:
        """execute_op_simple on one MatMulParams request; out/act/weight are (fd, offset)."""
        req = self.pkg.pack_matmul_request(op, out, act, weight, m, k, n)[8:]
        buf = ctypes.create_string_buffer(req, len(req))
        return self.lib.execute_op_simple(ctypes.cast(buf, ctypes.c_void_p))

    def matmul(self, x: np.ndarray, wq: np.ndarray, n: int, wtype: int) -> np.ndarray:
        m, k = x.shape
        fw, fx, fy = self.put(wq), self.put(x), self.buf(m * n * 4)
        rc = self.execute(self.op_index(wtype, x.dtype == np.float16), (fy, 0), (fx, 0), (fw, 0), m, k, n)
        assert rc == 0, f"execute_op_simple -> {rc}"
        y = self.get(fy, (m, n))
        self.free(fw, fx, fy)
        return y


@pytest.fixture(scope="module")
def dev(pkg, lib):
    """An open session on device 0 with the backend initialised; closed after the module."""
    assert lib.open_dsp_session(0, 1) == 0, "no usable CUDA device: the library has no CPU fallback"
    lib.init_htp_backend()
    d = Device(pkg, lib)
    yield d
    d.free_all()
    lib.close_dsp_session()
