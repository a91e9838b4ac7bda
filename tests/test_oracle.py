"""CPU tests of the oracle itself: C code vs an independent numpy restatement, the packer,
known-answer blocks, and the committed golden fixtures (tests/golden/golden.json)."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import pytest

GOLDEN = json.loads((Path(__file__).parent / "golden" / "golden.json").read_text())


def f16(v: float) -> bytes:
    return np.float16(v).tobytes()


def test_q4_0_known_answer_block(oracle):
    """All sixteen nibble values at known positions: element j < 16 is the LOW nibble of byte j,
    element j + 16 the HIGH nibble (reference mat_mul.c:266-271), value = nibble - 8 (:25-27)."""
    qs = bytes(((15 - j) << 4) | j for j in range(16))
    blk = np.frombuffer(f16(0.5) + qs, dtype=np.uint8)
    w = oracle.dequantize(blk, 1, 32, 2)[0]
    expect = np.array([j - 8 for j in range(16)] + [(15 - j) - 8 for j in range(16)], dtype=np.float32) * 0.5
    assert (w == expect).all()
    s, t = oracle.block_sums(blk, 2)
    assert s[0] == int(sum(expect / 0.5)) and t[0] == int(sum((i + 1) * v for i, v in enumerate(expect / 0.5)))
    vals, scales = oracle.np_unpack(blk, 1, 32, 2)
    assert (vals[0] * scales[0, 0] == expect).all()


def test_q8_0_known_answer_block(oracle):
    """Bytes are signed (reference mat_mul.c:300-301) although the struct declares uint8_t."""
    q = np.array([-128, -127, -1, 0, 1, 127] + list(range(-13, 13)), dtype=np.int8)
    blk = np.frombuffer(f16(-0.25) + q.tobytes(), dtype=np.uint8)
    w = oracle.dequantize(blk, 1, 32, 8)[0]
    assert (w == q.astype(np.float32) * -0.25).all()
    s, t = oracle.block_sums(blk, 8)
    assert s[0] == int(q.astype(int).sum()) and t[0] == int(((np.arange(32) + 1) * q.astype(int)).sum())


def test_all_byte_values_block_sums(oracle):
    """Every byte value in every position: 256 Q8_0 blocks with a sliding window of byte values."""
    blocks = []
    for b in range(256):
        q = ((np.arange(32) * 7 + b) % 256).astype(np.uint8)
        blocks.append(f16(1.0) + q.tobytes())
    wq = np.frombuffer(b"".join(blocks), dtype=np.uint8)
    s, t = oracle.block_sums(wq, 8)
    vals, _ = oracle.np_unpack(wq, 256, 32, 8)
    assert (s == vals.astype(np.int32).sum(axis=1)).all()
    assert (t == (vals.astype(np.int32) * (np.arange(32) + 1)).sum(axis=1)).all()


def test_q4_0_signed_scale_rule(oracle, wl):
    """d = (signed value at max |w|) / -8: a negative extreme maps to nibble 0 with positive d, a
    positive extreme maps to nibble 0 with negative d."""
    w = np.zeros((1, 64), dtype=np.float32)
    w[0, 3], w[0, 5] = -1.0, 0.5
    w[0, 32 + 7], w[0, 32 + 9] = 2.0, -1.0
    for packer in (lambda a: oracle.quantize(a, 2), wl.quantize_q4_0):
        wq = packer(w)
        vals, scales = oracle.np_unpack(wq, 1, 64, 2)
        assert scales[0, 0] == 0.125 and vals[0, 3] == -8 and vals[0, 5] == 4 and vals[0, 0] == 0
        assert scales[0, 1] == -0.25 and vals[0, 39] == -8 and vals[0, 41] == 4


@pytest.mark.parametrize("wtype", [2, 8])
def test_c_packer_equals_numpy_packer(oracle, wl, wtype):
    rng = np.random.default_rng(7)
    w = rng.standard_normal((96, 512), dtype=np.float32) * np.float32(0.02)
    w[0, :32] = 0.0  # zero block
    w[1, :32] = np.float32(0.01)  # all equal
    w[2, 5] = np.float32(65504.0)  # large
    w[3, :64] = rng.integers(-8, 8, 64).astype(np.float32) * np.float32(0.5)  # exact ties at .5 steps
    a = oracle.quantize(w, wtype)
    b = wl.quantize(w, wtype)
    assert a.shape == b.shape and (a == b).all()


@pytest.mark.parametrize("wtype,act_f16,m,k,n", [(2, False, 1, 256, 32), (8, False, 3, 512, 64), (2, True, 8, 1024, 96),
                                                 (8, True, 5, 96, 32)])
def test_c_oracle_equals_numpy_restatement(oracle, wl, wtype, act_f16, m, k, n):
    wq, x = wl.random_case(11, wtype, act_f16, m, k, n)
    y, absdot = oracle.mul_mat_f64(x, wq, n, wtype, want_absdot=True)
    ref = oracle.np_mul_mat_f64(x, wq, n, wtype)
    assert np.abs(y - ref).max() <= 1e-12 * np.abs(ref).max()
    assert (absdot >= np.abs(y) - 1e-12).all()
    y32 = oracle.mul_mat_f32(x, wq, n, wtype)
    assert oracle.error_metrics(y32, y)["max_rel_to_max"] < 1e-5


def test_oracle_rejects_bad_shapes(oracle):
    lib = oracle.load()
    assert lib.htp_oracle_mul_mat_f64(None, None, None, 0, None, 1, 48, 32, 2, 1) == -1
    assert lib.htp_oracle_quantize(None, None, 1, 48, 2, 1) == -1
    assert lib.htp_oracle_quantize(None, None, 1, 64, 3, 1) == -1


def _check_sample(y, g):
    head, tail = np.array(g["head"]), np.array(g["tail"])
    assert abs(y.sum() - g["sum"]) <= 1e-9 * g["abs_sum"]
    assert abs(np.abs(y).sum() - g["abs_sum"]) <= 1e-9 * g["abs_sum"]
    y = y[g["rows"]]
    assert np.allclose(y[:, :head.shape[1]], head, rtol=0, atol=1e-12 * g["max_abs"])
    assert np.allclose(y[:, -tail.shape[1]:], tail, rtol=0, atol=1e-12 * g["max_abs"])


@pytest.mark.parametrize("name", ["cfg0", "cfg1"])
def test_golden_small_configs(oracle, wl, name):
    """Configs 0 and 1 regenerated from their seeds: input hashes, oracle outputs, block sums."""
    cfg, g = wl.CONFIGS[name], GOLDEN[name]
    op = cfg.ops[0]
    wq = wl.make_weight(cfg, quantizer=lambda w, t: oracle.quantize(w, t))
    x = wl.make_activation(cfg, g["m"])
    assert wl.sha256(wq) == g["w_sha256"] and wl.sha256(x) == g["x_sha256"]
    _check_sample(oracle.mul_mat_f64(x, wq, op.n, op.wtype), g["oracle"])
    s, t = oracle.block_sums(wq, op.wtype)
    assert wl.sha256(s) == g["block_sum_s_sha256"] and wl.sha256(t) == g["block_sum_t_sha256"]


def test_golden_cfg3_layer0_small_matrices(oracle, wl):
    """Config 3: the k and v projections of layer 0 (1024 x 4096) against the fixtures."""
    cfg, g = wl.CONFIGS["cfg3"], GOLDEN["cfg3"]
    for i, op in enumerate(cfg.ops):
        if op.name not in ("k", "v"):
            continue
        wq = wl.make_weight(cfg, i, 0, quantizer=lambda w, t: oracle.quantize(w, t))
        assert wl.sha256(wq) == g["layers"]["0"][op.name]
        for m in cfg.ms:
            x = wl.make_activation(cfg, m, i, 0)
            e = g["oracle_layer0"][f"{op.name}_m{m}"]
            assert wl.sha256(x) == e["x_sha256"]
            _check_sample(oracle.mul_mat_f64(x, wq, op.n, op.wtype), e["oracle"])


def test_golden_cfg4_first_chunk(oracle, wl):
    """Config 4: the first 8192-row chunk of the lm_head weight, as a shard would generate it."""
    cfg, g = wl.CONFIGS["cfg4"], GOLDEN["cfg4"]
    part = wl.make_weight(cfg, rows=(0, wl.ROW_CHUNK), quantizer=lambda w, t: oracle.quantize(w, t))
    assert wl.sha256(part) == g["w_chunk_sha256"][0]
    x = wl.make_activation(cfg, 1)
    assert wl.sha256(x) == g["m1"]["x_sha256"]
    y = oracle.mul_mat_f64(x, part, wl.ROW_CHUNK, cfg.ops[0].wtype)
    head = np.array(g["m1"]["oracle"]["head"])
    assert np.allclose(y[:, :head.shape[1]], head, rtol=0, atol=1e-12 * g["m1"]["oracle"]["max_abs"])


def test_rms_norm_oracle_restatements_agree(oracle):
    """C oracle (double accumulation), the reference's float loop and the numpy restatement on the
    reference test's input range [-20, 20] (src/host/test.c:100-102), plus a known answer."""
    rng = np.random.Generator(np.random.PCG64(5))
    x = (rng.random((6, 1000), dtype=np.float32) * 40.0 - 20.0).astype(np.float32)
    a, b, c = oracle.rms_norm_f32(x), oracle.np_rms_norm_f32(x), oracle.rms_norm_f32(x, wide=False)
    assert np.abs(a - b).max() <= 2e-7 and np.abs(a - c).max() <= 1e-5
    ones = np.full((1, 64), 3.0, dtype=np.float32)  # mean of squares 9 -> scale 1/sqrt(9.00001)
    assert np.allclose(oracle.rms_norm_f32(ones), 3.0 / np.sqrt(9.0 + 1e-5), rtol=0, atol=1e-7)
    assert (oracle.rms_norm_f32(np.zeros((2, 8), dtype=np.float32)) == 0).all()


def test_iq4_nl_unpack_known_answer_and_restatements(oracle, wl):
    """IQ4_NL = the Q4_0 block with the reference's value table (src/dsp/ops/mat_mul.c:29-32) in the
    same nibble order: every nibble value at a known position, C against numpy, packers agree."""
    table = [-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113]
    blk = np.zeros(18, dtype=np.uint8)
    blk[:2] = np.array([2.0], dtype=np.float16).view(np.uint8)
    blk[2:] = np.arange(16, dtype=np.uint8) | ((15 - np.arange(16, dtype=np.uint8)) << 4)
    w = oracle.dequantize(blk, 1, 32, 20)[0]
    assert w[:16].tolist() == [2.0 * v for v in table]  # element j < 16: low nibble of byte j
    assert w[16:].tolist() == [2.0 * v for v in table[::-1]]  # element j + 16: high nibble of byte j
    s, t = oracle.block_sums(blk, 20)
    vals = table + table[::-1]
    assert s[0] == sum(vals) and t[0] == sum((i + 1) * v for i, v in enumerate(vals))
    rng = np.random.Generator(np.random.PCG64(21))
    wf = rng.standard_normal((48, 512), dtype=np.float32) * np.float32(0.02)
    assert (wl.quantize(wf, 20) == oracle.quantize(wf, 20)).all()
    wq, x = wl.random_case(22, 20, False, 3, 512, 48)
    assert np.abs(oracle.mul_mat_f64(x, wq, 48, 20) - oracle.np_mul_mat_f64(x, wq, 48, 20)).max() < 1e-12
