"""Python face of libhtp_ops_b200.so: a ctypes loader plus a thin mirror of the C host API.

The compute lives in the shared library (hand-written sm_100a CUDA behind a C ABI); nothing here
computes.  Importing the package never builds anything; `load()` raises when the library has not
been built (`python htp-ops-lib_b200/build.py`) - there is no CPU or pure-Python fallback.

The directory name is not a Python identifier; load the package with importlib under the name
`htp_ops_lib_b200` (see `__graft_entry__.load_package`).
"""
from __future__ import annotations

import ctypes
import struct
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "libhtp_ops_b200.so"
INCLUDE_DIR = PKG_DIR.parent / "include"

# enum HtpOpsIndex (include/op_reg.h)
HTP_OPS_RMS_NORM_F32 = 0
HTP_OPS_MAT_MUL_PERMUTED_W16A32 = 1
HTP_OPS_MAT_MUL_PERMUTED_W4D16A32 = 2
HTP_OPS_MAT_MUL_PERMUTED_W8D16A32 = 3
HTP_OPS_MAT_MUL_PERMUTED_W4D16A32_IQ4_NL = 4
HTP_OPS_FLASH_ATTN_QO_F32_KV_F16 = 5
HTP_OPS_MAT_MUL_W4D16A16 = 6
HTP_OPS_MAT_MUL_W8D16A16 = 7
HTP_OPS_COUNT = 8

# enum RequestType (include/message.h)
REQUEST_TYPE_NO_OP = 0
REQUEST_TYPE_RPCMEM_MAP = 1
REQUEST_TYPE_OP_COMPUTE = 2

TYPE_Q4_0 = 2
TYPE_Q8_0 = 8
TYPE_IQ4_NL = 20
WT_F16_TILED = 1  # fp16 weights in the reference's tile order (HTP_B200_WT_F16_TILED)
WT_PERMUTED = 0x100  # | TYPE_*: the reference-private permuted super-blocks (HTP_B200_WT_PERMUTED)
ACT_F32 = 0
ACT_F16 = 1
BLOCK_BYTES = {TYPE_Q4_0: 18, TYPE_Q8_0: 34, TYPE_IQ4_NL: 18}

# every symbol include/*.h declares, with (restype, argtypes)
_vp, _i, _u, _sz, _i64, _u64 = (ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_size_t, ctypes.c_int64,
                                ctypes.c_uint64)
EXPORTS = {
    # include/htp_ops_b200.h
    "htp_b200_mul_mat": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "htp_b200_mul_mat_batch": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "htp_b200_mul_mat_static_scratch": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "htp_b200_block_sums": (_i, [_vp, _vp, _vp, _i64, _i, _vp]),
    "htp_b200_decode_plan": (_i, [_i, _i, _i, _i, ctypes.POINTER(_i), ctypes.POINTER(_i), ctypes.POINTER(_i)]),
    "htp_b200_rms_norm_f32": (_i, [_vp, _vp, _i, _i, _vp]),
    "htp_b200_mul_mat_multi_dst": (_i, [_vp, _i, _i64, _i64, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "htp_b200_mul_mat_multi_dst_signal": (_i, [_vp, _i, _i64, _i64, _vp, _vp, _i, _i, _i, _i, _i, _vp, ctypes.c_uint32,
                                               _vp]),
    "htp_b200_mul_mat_gather_step": (_i, [_vp, _i, _i64, _i64, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, ctypes.c_uint32,
                                          _vp]),
    "htp_b200_wait_flags": (_i, [_vp, _i, ctypes.c_uint32, _vp]),
    "htp_b200_weight_bytes": (_sz, [_i, _i64, _i64]),
    "htp_b200_stream_status": (_i, [_vp]),
    "htp_b200_set_option": (_i, [ctypes.c_char_p, _i]),
    "htp_b200_launch_count": (_u64, []),
    "htp_b200_version": (ctypes.c_char_p, []),
    # include/host/session.h
    "open_dsp_session": (_i, [_i, _i]),
    "close_dsp_session": (None, []),
    "get_global_handle": (_u64, []),
    "init_htp_backend": (None, []),
    "create_htp_message_channel": (_i, [_i, _u]),
    # include/host/op_export.h
    "htp_ops_rpc_rms_norm_f32": (_i, [_i] * 6),
    "htp_ops_rpc_mat_mul_permuted_w16a32": (_i, [_i] * 9),
    # include/htp_ops.h
    "htp_ops_open": (_i, [ctypes.c_char_p, ctypes.POINTER(_u64)]),
    "htp_ops_close": (_i, [_u64]),
    "htp_ops_init_backend": (_i, [_u64]),
    "htp_ops_create_channel": (_i, [_u64, ctypes.c_int32, ctypes.c_uint32]),
    "htp_ops_destroy_channel": (_i, [_u64]),
    "htp_ops_rms_norm_f32": (_i, [_u64] + [ctypes.c_int32] * 6),
    "htp_ops_mat_mul_permuted_w16a32": (_i, [_u64] + [ctypes.c_int32] * 9),
    "htp_ops_test_ops": (_i, [_u64]),
    # include/dsp/op_executor.h
    "execute_op_simple": (_i, [_vp]),
    # include/host/buffers.h
    "htp_buf_alloc": (_i, [_sz]),
    "htp_buf_alloc_host": (_i, [_sz]),
    "htp_buf_alloc_shared": (_i, [_sz]),
    "htp_buf_wrap": (_i, [_vp, _sz]),
    "htp_buf_free": (_i, [_i]),
    "htp_buf_upload": (_i, [_i, _sz, _vp, _sz]),
    "htp_buf_download": (_i, [_i, _sz, _vp, _sz]),
    "htp_buf_upload_async": (_i, [_i, _sz, _vp, _sz]),
    "htp_buf_download_async": (_i, [_i, _sz, _vp, _sz]),
    "htp_buf_ptr": (_vp, [_i]),
    "htp_buf_is_host": (_i, [_i]),
    "htp_buf_size": (_sz, [_i]),
    "htp_session_stream": (_vp, []),
    "htp_session_synchronize": (_i, []),
}

_lib = None


def load() -> ctypes.CDLL:
    """dlopen the library and declare every exported signature.  Raises if it is not built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python {PKG_DIR / 'build.py'}`; "
                               "there is no fallback implementation")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in EXPORTS.items():
            fn = getattr(lib, name)  # AttributeError if the library lost a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


# ------------------------------------------------------------------------------------------------
# wire helpers (include/message.h, include/op_reg.h) - byte-level, no ctypes structs needed

def pack_matmul_request(op: int, out: tuple[int, int], act: tuple[int, int], weight: tuple[int, int], m: int, k: int,
                        n: int) -> bytes:
    """RequestHeader{state=0,type=OP_COMPUTE} || OpComputeRequest{op} || MatMulParams - 48 bytes."""
    return struct.pack("<iiI9i", 0, REQUEST_TYPE_OP_COMPUTE, op, out[0], out[1], act[0], act[1], weight[0], weight[1],
                       m, k, n)


def pack_rms_norm_request(dst: tuple[int, int], src: tuple[int, int], ne0: int, ne1: int) -> bytes:
    """RequestHeader{state=0,type=OP_COMPUTE} || OpComputeRequest{RMS_NORM_F32} || RmsNormF32Params - 36 bytes."""
    return struct.pack("<iiI6i", 0, REQUEST_TYPE_OP_COMPUTE, HTP_OPS_RMS_NORM_F32, dst[0], dst[1], src[0], src[1], ne0,
                       ne1)


def pack_map_request(puts: list[int], gets: list[int] | None = None) -> bytes:
    gets = gets or []
    fds = list(puts) + list(gets)
    return struct.pack(f"<iiii{len(fds)}i", 0, REQUEST_TYPE_RPCMEM_MAP, len(puts), len(gets), *fds)


def compose_message(requests: list[bytes]) -> bytes:
    """MessageHeader with state = 0 followed by the request table and the requests, as the
    reference's host test composes it (src/host/test.c:181-193)."""
    n = len(requests)
    hdr_size = 16 + 4 * (n + 1)
    offs = [hdr_size]
    for r in requests:
        offs.append(offs[-1] + len(r))
    return struct.pack(f"<QIi{n + 1}i", 0, 0, n, *offs) + b"".join(requests)


class MessageChannel:
    """Host side of the message protocol on a pinned host buffer (reference test.c:166-204)."""

    def __init__(self, max_msg_size: int = 4096):
        lib = load()
        self.lib = lib
        self.size = max_msg_size
        self.fd = lib.htp_buf_alloc_host(max_msg_size)
        if self.fd < 0:
            raise RuntimeError("htp_buf_alloc_host failed")
        rc = lib.create_htp_message_channel(self.fd, max_msg_size)
        if rc != 0:
            lib.htp_buf_free(self.fd)
            raise RuntimeError(f"create_htp_message_channel failed: {rc}")
        self.base = lib.htp_buf_ptr(self.fd)
        self.view = (ctypes.c_uint8 * max_msg_size).from_address(self.base)
        self.state = ctypes.c_uint64.from_address(self.base)

    def submit(self, requests: list[bytes], spin_limit: int = 200_000_000) -> list[int]:
        """Publish one message, spin until the servicer marks it done, return the per-request states."""
        return self.submit_composed(compose_message(requests), [len(r) for r in requests], spin_limit)

    def submit_composed(self, msg: bytes, request_sizes: list[int], spin_limit: int = 200_000_000) -> list[int]:
        """The same for a message composed beforehand (compose_message): a host that re-issues the same
        requests every step - a decoder's layer stack - builds the bytes once, as a C host would in a few
        microseconds, and pays only the copy into the channel per step."""
        if len(msg) > self.size:
            raise ValueError("message does not fit the channel buffer")
        self.state.value = 0
        ctypes.memmove(self.base + 8, msg[8:], len(msg) - 8)
        v = (ctypes.c_uint8 * 8).from_address(self.base)
        v[0] = 1  # publish (x86 stores are not reordered with earlier stores)
        n = 0
        while v[1] != 1:
            n += 1
            if n > spin_limit:
                raise TimeoutError("message channel servicer did not answer")
        hdr = 16 + 4 * (len(request_sizes) + 1)
        states, off = [], hdr
        for size in request_sizes:
            states.append(struct.unpack_from("<i", self.view, off)[0])
            off += size
        return states

    def close(self):
        self.lib.htp_ops_destroy_channel(self.lib.get_global_handle())
        self.lib.htp_buf_free(self.fd)
