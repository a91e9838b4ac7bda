"""ctypes front-end of the CPU oracle (oracle.c) plus an independent numpy restatement.

TEST INFRASTRUCTURE ONLY.  The shipped library never imports this module; it is used by the
test-suite, by the smoke check and by the CPU-baseline leg of the benchmark.

PARITY UNPINNED: the reference holds no golden vectors for Q4_0/Q8_0 matmul and its
implementation cannot be built without the Hexagon toolchain; see the header of oracle.c for
the reference lines each rule is restated from.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
TYPE_Q4_0 = 2
TYPE_Q8_0 = 8
TYPE_IQ4_NL = 20
BLOCK_BYTES = {TYPE_Q4_0: 18, TYPE_Q8_0: 34, TYPE_IQ4_NL: 18}
IQ4_NL_VALUES = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], dtype=np.int8)

_lib = None


def build(outdir: str | os.PathLike | None = None, arch: str | None = None) -> Path:
    """Compile oracle.c with the Makefile beside it; returns the path of the shared object."""
    outdir = Path(outdir) if outdir else HERE / "_ref"
    cmd = ["make", "-s", "-C", str(HERE), f"OUTDIR={outdir}"]
    if arch:
        cmd.append(f"ARCH={arch}")
    subprocess.run(cmd, check=True)
    return outdir / "liboracle.so"


def load(path: str | os.PathLike | None = None):
    """Load (building first if absent) the oracle shared object and declare its signatures."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    so = Path(path) if path else HERE / "_ref" / "liboracle.so"
    if not so.exists():
        build(so.parent)
    lib = ctypes.CDLL(str(so))
    vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    lib.htp_oracle_usable_cores.restype = i32
    lib.htp_oracle_quantize.restype = i64
    lib.htp_oracle_quantize.argtypes = [vp, vp, i64, i64, i32, i32]
    lib.htp_oracle_dequantize.restype = i32
    lib.htp_oracle_dequantize.argtypes = [vp, vp, i64, i64, i32]
    lib.htp_oracle_block_sums.restype = i32
    lib.htp_oracle_block_sums.argtypes = [vp, vp, vp, i64, i32]
    lib.htp_oracle_mul_mat_f64.restype = i32
    lib.htp_oracle_mul_mat_f64.argtypes = [vp, vp, vp, i32, vp, i64, i64, i64, i32, i32]
    lib.htp_oracle_rms_norm_f32.restype = i32
    lib.htp_oracle_rms_norm_f32.argtypes = [vp, vp, i64, i64, i32]
    lib.htp_oracle_mul_mat_f32.restype = i32
    lib.htp_oracle_mul_mat_f32.argtypes = [vp, vp, i32, vp, i64, i64, i64, i32, i32]
    lib.htp_oracle_tiled_dequantize.restype = i32
    lib.htp_oracle_tiled_dequantize.argtypes = [vp, vp, i64, i64, i32]
    lib.htp_oracle_tiled_group_sums.restype = i32
    lib.htp_oracle_tiled_group_sums.argtypes = [vp, vp, vp, i64, i32]
    lib.htp_oracle_mul_mat_dense_f64.restype = i32
    lib.htp_oracle_mul_mat_dense_f64.argtypes = [vp, vp, vp, i32, vp, i64, i64, i64, i32]
    if path is None:
        _lib = lib
    return lib


def _ptr(a: np.ndarray) -> int:
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


def usable_cores() -> int:
    return int(load().htp_oracle_usable_cores())


def quantize(w: np.ndarray, wtype: int, threads: int = 0) -> np.ndarray:
    """fp32 [N][K] -> packed block bytes (uint8, N * K/32 * block_bytes)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = w.shape
    out = np.empty(n * (k // 32) * BLOCK_BYTES[wtype], dtype=np.uint8)
    r = load().htp_oracle_quantize(_ptr(w), _ptr(out), n, k, wtype, threads)
    if r != out.size:
        raise ValueError("htp_oracle_quantize rejected the shape")
    return out


def dequantize(wq: np.ndarray, n: int, k: int, wtype: int) -> np.ndarray:
    out = np.empty((n, k), dtype=np.float32)
    if load().htp_oracle_dequantize(_ptr(wq), _ptr(out), n, k, wtype) != 0:
        raise ValueError("bad arguments")
    return out


def block_sums(wq: np.ndarray, wtype: int) -> tuple[np.ndarray, np.ndarray]:
    nb = wq.size // BLOCK_BYTES[wtype]
    s = np.empty(nb, dtype=np.int32)
    t = np.empty(nb, dtype=np.int32)
    if load().htp_oracle_block_sums(_ptr(wq), _ptr(s), _ptr(t), nb, wtype) != 0:
        raise ValueError("bad arguments")
    return s, t


def _act_args(act: np.ndarray):
    if act.dtype == np.float16:
        return np.ascontiguousarray(act).view(np.uint16), 1
    return np.ascontiguousarray(act, dtype=np.float32), 0


def mul_mat_f64(act: np.ndarray, wq: np.ndarray, n: int, wtype: int, threads: int = 0, want_absdot: bool = False):
    """The parity oracle: y[m][n] in fp64.  act is [M][K] float32 or float16."""
    m, k = act.shape
    a, is16 = _act_args(act)
    y = np.empty((m, n), dtype=np.float64)
    ad = np.empty((m, n), dtype=np.float64) if want_absdot else None
    r = load().htp_oracle_mul_mat_f64(_ptr(y), _ptr(ad) if want_absdot else None, _ptr(a), is16, _ptr(wq), m, k, n,
                                      wtype, threads)
    if r != 0:
        raise ValueError("bad arguments")
    return (y, ad) if want_absdot else y


def mul_mat_f32(act: np.ndarray, wq: np.ndarray, n: int, wtype: int, threads: int = 0, lib=None) -> np.ndarray:
    """The timed CPU baseline: fp32 dequantise-then-dot, threads over output rows."""
    m, k = act.shape
    a, is16 = _act_args(act)
    y = np.empty((m, n), dtype=np.float32)
    r = (lib or load()).htp_oracle_mul_mat_f32(_ptr(y), _ptr(a), is16, _ptr(wq), m, k, n, wtype, threads)
    if r != 0:
        raise ValueError("bad arguments")
    return y


def tiled_dequantize(w: np.ndarray, k: int, n: int, fmt: int) -> np.ndarray:
    """Weights in the reference's tile order (fmt = the library's weight_type code: 1 fp16 tiles, 0x102 /
    0x108 / 0x114 permuted Q4_0 / Q8_0 / IQ4_NL super-blocks) -> dense fp32 [n][k], slot by slot."""
    out = np.empty((n, k), dtype=np.float32)
    if load().htp_oracle_tiled_dequantize(_ptr(w), _ptr(out), k, n, fmt) != 0:
        raise ValueError("bad arguments")
    return out


def tiled_group_sums(w: np.ndarray, fmt: int) -> tuple[np.ndarray, np.ndarray]:
    """(S, T) per scale group (32 slots, eight per super-block) of a permuted super-block buffer."""
    sbb = {0x102: 144, 0x108: 272, 0x114: 144}[fmt]
    n_sb = w.size // sbb
    s = np.empty(n_sb * 8, dtype=np.int32)
    t = np.empty(n_sb * 8, dtype=np.int32)
    if load().htp_oracle_tiled_group_sums(_ptr(w), _ptr(s), _ptr(t), n_sb, fmt) != 0:
        raise ValueError("bad arguments")
    return s, t


def tiled_mul_mat_f64(act: np.ndarray, w: np.ndarray, n: int, fmt: int, threads: int = 0, want_absdot: bool = False):
    """The parity oracle for tile-order weights: dequantise exactly, then the fp64 dot."""
    m, k = act.shape
    wd = tiled_dequantize(w, k, n, fmt)
    a, is16 = _act_args(act)
    y = np.empty((m, n), dtype=np.float64)
    ad = np.empty((m, n), dtype=np.float64) if want_absdot else None
    r = load().htp_oracle_mul_mat_dense_f64(_ptr(y), _ptr(ad) if want_absdot else None, _ptr(a), is16, _ptr(wd), m, k,
                                            n, threads)
    if r != 0:
        raise ValueError("bad arguments")
    return (y, ad) if want_absdot else y


# ----------------------------------------------------------------------------------------------
# Independent numpy restatement (small cases): cross-checks the C code above in the CPU tests.

def rms_norm_f32(x: np.ndarray, wide: bool = True) -> np.ndarray:
    """RMSNorm of every row of x (fp32), eps 1e-5, as the reference's scalar statement
    (src/host/test.c:60-80); wide=True accumulates the sum of squares in double."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    assert x.ndim == 2
    y = np.empty_like(x)
    rc = load().htp_oracle_rms_norm_f32(_ptr(y), _ptr(x), x.shape[1], x.shape[0], 1 if wide else 0)
    assert rc == 0
    return y


def np_rms_norm_f32(x: np.ndarray) -> np.ndarray:
    """Independent numpy restatement (double arithmetic, rounded once at the end)."""
    xd = np.asarray(x, dtype=np.float64)
    scale = 1.0 / np.sqrt((xd * xd).mean(axis=1, keepdims=True) + np.float64(np.float32(1e-5)))
    return (xd * scale.astype(np.float32).astype(np.float64)).astype(np.float32)


def np_unpack(wq: np.ndarray, n: int, k: int, wtype: int):
    """-> (values int8 [N][K], scales float32 [N][K/32]) from packed bytes."""
    bb = BLOCK_BYTES[wtype]
    blocks = np.ascontiguousarray(wq, dtype=np.uint8).reshape(n, k // 32, bb)
    scales = blocks[:, :, :2].copy().view(np.float16).astype(np.float32)[:, :, 0]
    qs = blocks[:, :, 2:]
    if wtype == TYPE_Q4_0:
        lo = (qs & 0x0F).astype(np.int8) - 8
        hi = (qs >> 4).astype(np.int8) - 8
        vals = np.concatenate([lo, hi], axis=2)
    elif wtype == TYPE_IQ4_NL:
        vals = np.concatenate([IQ4_NL_VALUES[qs & 0x0F], IQ4_NL_VALUES[qs >> 4]], axis=2)
    else:
        vals = qs.view(np.int8)
    return vals.reshape(n, k), scales


def np_mul_mat_f64(act: np.ndarray, wq: np.ndarray, n: int, wtype: int) -> np.ndarray:
    m, k = act.shape
    vals, scales = np_unpack(wq, n, k, wtype)
    w = vals.astype(np.float64) * np.repeat(scales.astype(np.float64), 32, axis=1)
    return act.astype(np.float64) @ w.T


def error_metrics(y: np.ndarray, ref: np.ndarray, absdot: np.ndarray | None = None) -> dict:
    """max|y-o|/max|o| (the gated figure) and, when absdot is given, max|y-o|/sum|x_l w_l|."""
    y = np.asarray(y, dtype=np.float64)
    err = np.abs(y - ref)
    out = {"max_rel_to_max": float(err.max() / max(np.abs(ref).max(), 1e-300))}
    if absdot is not None:
        out["max_cond_rel"] = float((err / np.maximum(absdot, 1e-300)).max())
    return out
