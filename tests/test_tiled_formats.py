"""CPU checks of the tile-order weight formats: the fp16 tile buffer of the W16A32 op against the
index formula of the reference's host test (src/host/test.c:303-313), and the permuted Q4_0 / Q8_0 /
IQ4_NL super-blocks (include/dsp/quants.h:16-31) - hand-built known-answer blocks for the slot order
read off src/dsp/ops/mat_mul.c:373-405 and :472-506, the C restatement against an independent numpy
one, and packer -> reader round trips.  No reference test or fixture holds these formats, so the
permuted ones stay "parity unpinned"."""
from __future__ import annotations

import importlib.util
import json
from pathlib import Path

import numpy as np
import pytest

GOLDEN_DIR = Path(__file__).parent / "golden"
GOLDEN = json.loads((GOLDEN_DIR / "golden_tiled.json").read_text())


def golden_module():
    spec = importlib.util.spec_from_file_location("make_golden_tiled", GOLDEN_DIR / "make_golden_tiled.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


Q4, Q8, IQ4 = 2, 8, 20
PERM = 0x100
IQ4_TABLE = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], dtype=np.float32)


def _np_tiled_dequantize(buf: np.ndarray, k: int, n: int, fmt: int) -> np.ndarray:
    """Vectorised restatement, written without looking at slots one by one: decode every super-block
    into [row pair][slot] values, then undo the tile order with one transpose.  Returns [n][k]."""
    nt, kt = n // 32, k // 32
    if fmt == 1:
        slots = buf.view(np.float16).astype(np.float32).reshape(nt, kt, 4, 4, 64)
    else:
        sbb = 272 if fmt == (PERM | Q8) else 144
        sb = buf.reshape(nt * kt * 4, sbb)
        d = sb[:, :16].copy().view(np.float16).astype(np.float32)  # [sb][8]
        if fmt == (PERM | Q8):
            q = sb[:, 16:].copy().view(np.int8).astype(np.float32).reshape(-1, 4, 64)
        else:
            qs = sb[:, 16:].reshape(-1, 64, 2)
            nib = np.stack([qs[:, :, 0] & 15, qs[:, :, 1] & 15, qs[:, :, 0] >> 4, qs[:, :, 1] >> 4], axis=1)
            q = nib.astype(np.float32) - 8 if fmt == (PERM | Q4) else IQ4_TABLE[nib]
        scale = np.repeat(d.reshape(-1, 4, 2), 32, axis=2)  # slot t of row pair v uses scales[2v + (t % 64) / 32]
        slots = (q * scale).reshape(nt, kt, 4, 4, 64)
    a = slots.reshape(nt, kt, 4, 4, 32, 2)  # n-tile, k-tile, super-block, row pair, column, parity
    return np.ascontiguousarray(a.transpose(0, 4, 1, 2, 3, 5)).reshape(n, k)


def test_f16_tile_buffer_follows_the_reference_index_formula(wl, oracle):
    k, n = 96, 64
    rng = np.random.default_rng(5)
    w = rng.standard_normal((k, n)).astype(np.float32)
    buf = wl.pack_f16_tiles(w)
    assert buf.size == wl.weight_bytes(wl.WT_F16_TILED, k, n) == k * n * 2
    want = np.zeros(k * n, dtype=np.float16)
    for i in range(k):  # the loop of test.c:303-313
        for j in range(n):
            i0, i1, j0, j1 = i // 32, i % 32, j // 32, j % 32
            want[(j0 * (k // 32) + i0) * 1024 + (i1 & ~1) * 32 + j1 * 2 + (i1 & 1)] = np.float16(w[i, j])
    assert (buf == want.view(np.uint8)).all()
    dense = oracle.tiled_dequantize(buf, k, n, wl.WT_F16_TILED)
    assert (dense == w.astype(np.float16).astype(np.float32).T).all()


def _one_tile(sb_bytes: int) -> np.ndarray:
    t = np.zeros((4, sb_bytes), dtype=np.uint8)
    t[:, :16] = np.full(8, 1.0, dtype=np.float16).view(np.uint8)  # all scales 1.0
    return t


def test_permuted_q8_known_answer(oracle):
    """Slot t of a super-block is k-row 2 * (t / 64) + (t & 1), column (t % 64) / 2, scale t / 32."""
    tile = _one_tile(272)
    tile[1, 16 + 70] = np.uint8(0xFB)  # -5 at super-block 1, slot 70: k = 8 + 2 + 0 = 10, n = 3, scale index 2
    tile[1, 4:6] = np.array([0.5], dtype=np.float16).view(np.uint8)
    tile[3, 16 + 255] = 100  # super-block 3, slot 255: k = 24 + 6 + 1 = 31, n = 31
    dense = oracle.tiled_dequantize(tile.reshape(-1), 32, 32, PERM | Q8)
    want = np.zeros((32, 32), dtype=np.float32)
    want[3, 10] = -2.5
    want[31, 31] = 100.0
    assert (dense == want).all()


def test_permuted_q4_known_answer(oracle):
    """Byte 2s / 2s+1 of the quants: low nibbles are row pairs 0 / 1, high nibbles row pairs 2 / 3."""
    tile = _one_tile(144)
    tile[:, 16:] = 0x88  # every nibble 8 -> value 0
    tile[2, 16 + 13] = 0x9F  # odd byte of slot s = 6 (column 3, even k): low 15 -> +7 at pair 1, high 9 -> +1 at pair 3
    tile[2, 2:4] = np.array([2.0], dtype=np.float16).view(np.uint8)    # scales[1]: slots 32..63 (pair 0, columns 16..31)
    tile[2, 4:6] = np.array([0.25], dtype=np.float16).view(np.uint8)   # scales[2]: pair 1, columns 0..15
    tile[0, 16 + 2 * 63] = 0x80  # even byte of slot 63 (column 31, odd k): low 0 -> -8 at pair 0 of super-block 0
    dense = oracle.tiled_dequantize(tile.reshape(-1), 32, 32, PERM | Q4)
    want = np.zeros((32, 32), dtype=np.float32)
    want[3, 16 + 2] = 7 * 0.25  # k = 16 + 2 * 1 + 0
    want[3, 16 + 6] = 1.0       # k = 16 + 2 * 3 + 0, scales[6] = 1
    want[31, 1] = -8.0          # k = 0 + 0 + 1, scales[1] of super-block 0 = 1
    assert (dense == want).all()
    iq = oracle.tiled_dequantize(tile.reshape(-1), 32, 32, PERM | IQ4)
    assert iq[3, 18] == 113 * 0.25 and iq[3, 22] == 13.0 and iq[31, 1] == -127.0
    assert iq[0, 0] == 1.0  # nibble 8 -> table value 1


@pytest.mark.parametrize("wtype", [Q4, Q8, IQ4])
def test_permuted_c_restatement_matches_numpy_and_round_trips(wl, oracle, wtype):
    k, n = 128, 96
    rng = np.random.default_rng(7 + wtype)
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    buf = wl.quantize_permuted(w, wtype)
    fmt = PERM | wtype
    assert buf.size == wl.weight_bytes(fmt, k, n)
    dense = oracle.tiled_dequantize(buf, k, n, fmt)
    assert (dense == _np_tiled_dequantize(buf, k, n, fmt)).all()
    # the packer's scale groups are the reader's: errors stay within one quantisation step of each group
    step = np.abs(w).max() / (127 if wtype == Q8 else 7)
    assert np.abs(dense - w.T).max() <= (0.51 if wtype == Q8 else 1.05) * step * (3.0 if wtype == IQ4 else 1.0)
    # random bytes (every nibble / byte value in every position) decode identically in both restatements
    junk = rng.integers(0, 256, size=buf.size, dtype=np.uint8).reshape(-1, buf.size // (n // 32 * k // 32 * 4))
    junk[:, :16] = buf.reshape(junk.shape)[:, :16]  # keep finite scales
    assert (oracle.tiled_dequantize(junk.reshape(-1), k, n, fmt) == _np_tiled_dequantize(junk.reshape(-1), k, n, fmt)).all()


def test_tiled_oracle_matmul_equals_dense_fp64(wl, oracle):
    m, k, n = 3, 64, 64
    for fmt in (wl.WT_F16_TILED, PERM | Q4, PERM | Q8, PERM | IQ4):
        wq, x = wl.tiled_random_case(9, fmt, False, m, k, n)
        y, absdot = oracle.tiled_mul_mat_f64(x, wq, n, fmt, want_absdot=True)
        dense = _np_tiled_dequantize(wq, k, n, fmt).astype(np.float64)
        ref = x.astype(np.float64) @ dense.T
        assert np.abs(y - ref).max() <= 1e-12 * np.abs(ref).max() + 1e-300
        assert (absdot >= np.abs(y) - 1e-12).all()
    with pytest.raises(ValueError):
        oracle.tiled_dequantize(wq, 48, 64, fmt)


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_golden_tile_order_cases(name):
    """Packer and oracle reproduce the committed fixtures bit for bit (hashes) / to 1e-12 (fp64 samples)."""
    g = golden_module().entry_of(name)
    want = GOLDEN[name]
    assert g["w_sha256"] == want["w_sha256"] and g["x_sha256"] == want["x_sha256"]
    for key in ("head", "tail"):
        assert np.allclose(np.array(g[key]), np.array(want[key]), rtol=1e-12, atol=0)
    assert abs(g["abs_sum"] - want["abs_sum"]) <= 1e-10 * want["abs_sum"]


@pytest.mark.parametrize("wtype", [Q4, Q8, IQ4])
def test_permuted_group_sums_match_numpy(wl, oracle, wtype):
    """S = sum q and T = sum (j + 1) q per scale group (32 consecutive slots), the integer invariant the GPU
    decode is held to bit for bit: the C loop against a vectorised count on random bytes."""
    fmt = PERM | wtype
    sbb = 272 if wtype == Q8 else 144
    rng = np.random.default_rng(30 + wtype)
    buf = rng.integers(0, 256, size=24 * sbb, dtype=np.uint8)
    s, t = oracle.tiled_group_sums(buf, fmt)
    sb = buf.reshape(-1, sbb)
    if wtype == Q8:
        q = sb[:, 16:].copy().view(np.int8).astype(np.int64).reshape(-1, 8, 32)
    else:
        qs = sb[:, 16:].reshape(-1, 64, 2)
        nib = np.stack([qs[:, :, 0] & 15, qs[:, :, 1] & 15, qs[:, :, 0] >> 4, qs[:, :, 1] >> 4], axis=1)  # [sb][pair][slot]
        q = (nib.astype(np.int64) - 8 if wtype == Q4 else IQ4_TABLE[nib].astype(np.int64)).reshape(-1, 8, 32)
    assert (s == q.sum(axis=2).reshape(-1)).all()
    assert (t == (q * np.arange(1, 33)).sum(axis=2).reshape(-1)).all()
    assert s.dtype == np.int32 and s.size == 24 * 8
