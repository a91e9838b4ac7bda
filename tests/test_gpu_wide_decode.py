"""GPU parity of the decode kernel's wide integer path (three to eight tokens per launch, every
weight format, either activation type) and of the launches built on it: K ranges that accumulate,
batched launches whose operators have different K, and config 3's decoder stack issued as ONE
message per token count - the way the benchmark drives it (reference host test,
src/host/test.c:166-204: compose, publish, spin, read the per-request states).

Gate: max|y - o| / max|o| <= 1e-5 (fp32 activations) / 1e-3 (fp16 activations) against the fp64
oracle on the same packed bytes, and the same bound on the condition-normalised error."""
from __future__ import annotations

import ctypes
import json
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GOLDEN = json.loads((Path(__file__).parent / "golden" / "golden.json").read_text())
TOL = {False: 1e-5, True: 1e-3}


def check(oracle, y, x, wq, n, wtype):
    ref, absdot = oracle.mul_mat_f64(x, wq, n, wtype, want_absdot=True)
    e = oracle.error_metrics(y, ref, absdot)
    tol = TOL[x.dtype == np.float16]
    assert np.isfinite(y).all()
    assert e["max_rel_to_max"] <= tol, e
    assert e["max_cond_rel"] <= tol, e
    return e


def raw(dev, x, wq, n, wtype):
    """htp_b200_mul_mat on device copies of the arrays."""
    import torch
    m, k = x.shape
    tw, tx = torch.from_numpy(wq).cuda(), torch.from_numpy(x).cuda()
    ty = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    assert dev.lib.htp_b200_mul_mat(ty.data_ptr(), tx.data_ptr(), tw.data_ptr(), m, k, n, wtype,
                                    1 if x.dtype == np.float16 else 0, st) == 0
    torch.cuda.synchronize()
    assert dev.lib.htp_b200_stream_status(st) == 0
    return ty.cpu().numpy()


# K = 5632 / 5888: the largest K whose fragments fit one launch (Q4_0 / Q8_0); 6144, 14336: K ranges
# that accumulate; 2048 x 4000: tiles cut by CTA range boundaries; 256 x 32: a single, partial stage;
# 4352: a two-stage ring; 4096: three stages
SHAPES = [(256, 32), (2048, 4000 // 32 * 32), (4096, 1024), (4352, 64), (5632, 96), (5888, 64), (6144, 64), (14336, 96)]


@pytest.mark.parametrize("wtype", [2, 8, 20])
@pytest.mark.parametrize("act_f16", [False, True])
@pytest.mark.parametrize("k,n", SHAPES)
def test_wide_path_matches_oracle(dev, oracle, wl, wtype, act_f16, k, n):
    for m in (3, 6, 8):
        wq, x = wl.random_case(1300 + m, wtype, act_f16, m, k, n)
        check(oracle, raw(dev, x, wq, n, wtype), x, wq, n, wtype)


@pytest.mark.parametrize("wtype", [2, 8, 20])
def test_wide_path_token_magnitudes(dev, oracle, wl, wtype):
    """Tokens of very different magnitude in one launch, a token with one dominant element, a zero
    token: every token has its own power-of-two scale, so each meets the gate on its own."""
    wq, x = wl.random_case(1400, wtype, False, 8, 2048, 96)
    x[0] *= 3.0e5
    x[1] *= 1.0e-6
    x[2, 17] = 7.5e7
    x[3] = 0.0
    x[4] = -x[4]
    y = raw(dev, x, wq, 96, wtype)
    ref = oracle.mul_mat_f64(x, wq, 96, wtype)
    assert (y[3] == 0.0).all()
    for m in (0, 1, 2, 4, 5, 6, 7):
        assert np.abs(y[m] - ref[m]).max() <= 1e-5 * np.abs(ref[m]).max()


def test_wide_path_exhaustive_values(dev, oracle, wl):
    """Every byte value of a Q8_0 block and every nibble of a Q4_0 block at known positions, eight
    basis-like tokens: a misplaced element or a wrong sign changes a result by O(1)."""
    k, n = 256, 32
    for wtype in (2, 8):
        bb = wl.BLOCK_BYTES[wtype]
        raw_w = np.zeros((n, k // 32, bb), dtype=np.uint8)
        raw_w[:, :, :2] = np.frombuffer(np.float16(0.25).tobytes(), dtype=np.uint8)
        for r in range(n):
            for b in range(k // 32):
                raw_w[r, b, 2:] = (np.arange(bb - 2) * 5 + r * 8 + b * 37) % 256
        wq = raw_w.reshape(-1)
        x = np.zeros((8, k), dtype=np.float32)
        for m in range(8):
            x[m, m::8] = np.arange(1, k // 8 + 1, dtype=np.float32)
        y = raw(dev, x, wq, n, wtype)
        ref = oracle.mul_mat_f64(x, wq, n, wtype)
        assert np.abs(y - ref).max() <= 1e-6 * np.abs(ref).max()


@pytest.mark.parametrize("wtype,act_f16,m", [(2, False, 8), (8, False, 5), (20, True, 3)])
def test_batched_launch_with_k_ranges(dev, oracle, wl, wtype, act_f16, m):
    """Operators of different K in one batch, three of them with more K than one launch's fragments
    hold: such an operator is entered once per K range, every range writes a slab of its own, and one
    small kernel adds the slabs in range order.  Two launches: the persistent one and the sums."""
    lib = dev.lib
    shapes = [(14336, 64), (4096, 1024), (1024, 32), (14336, 160), (6144, 96)]
    cases = [wl.random_case(1500 + i, wtype, act_f16, m, k, n) for i, (k, n) in enumerate(shapes)]
    fw = [dev.put(wq) for wq, _ in cases]
    fx = [dev.put(x) for _, x in cases]
    fy = [dev.buf(m * n * 4) for _, n in shapes]
    n_ops = len(shapes)
    arr = lambda fds: (ctypes.c_void_p * n_ops)(*[lib.htp_buf_ptr(f) for f in fds])  # noqa: E731
    ks = (ctypes.c_int * n_ops)(*[k for k, _ in shapes])
    ns = (ctypes.c_int * n_ops)(*[n for _, n in shapes])
    before = lib.htp_b200_launch_count()
    assert lib.htp_b200_mul_mat_batch(n_ops, arr(fy), arr(fx), arr(fw), ks, ns, m, wtype, 1 if act_f16 else 0,
                                      lib.htp_session_stream()) == 0
    assert lib.htp_session_synchronize() == 0
    assert lib.htp_b200_launch_count() == before + 2
    for i, ((k, n), (wq, x)) in enumerate(zip(shapes, cases)):
        check(oracle, dev.get(fy[i], (m, n)), x, wq, n, wtype)
    dev.free(*fw, *fx, *fy)


@pytest.mark.parametrize("m", [1, 8])
def test_config3_layers_as_one_message(dev, oracle, wl, m):
    """Config 3 as the benchmark issues it: the seven matrices of decoder layers 0 and 31 as ONE
    message of fourteen requests through the channel - the servicer forms one batch of them (when
    m = 8 the down projections run as four K ranges each, summed by one small kernel), every request
    state is 0 and every output meets the oracle gate; layer 0 also meets the committed samples."""
    lib, pkg = dev.lib, dev.pkg
    cfg, g = wl.CONFIGS["cfg3"], GOLDEN["cfg3"]
    opi = pkg.HTP_OPS_MAT_MUL_PERMUTED_W4D16A32
    items = []
    for layer in (0, 31):
        for i, op in enumerate(cfg.ops):
            wq = wl.make_weight(cfg, i, layer, quantizer=lambda w, t: oracle.quantize(w, t))
            if str(layer) in g["layers"]:
                assert wl.sha256(wq) == g["layers"][str(layer)][op.name]
            x = wl.make_activation(cfg, m, i, layer)
            items.append((layer, op, wq, x, dev.put(wq), dev.put(x), dev.buf(m * op.n * 4)))
    reqs = [pkg.pack_matmul_request(opi, (fy, 0), (fx, 0), (fw, 0), m, op.k, op.n)
            for _, op, _, _, fw, fx, fy in items]
    chan = pkg.MessageChannel(4096)
    try:
        before = lib.htp_b200_launch_count()
        assert chan.submit(reqs) == [0] * len(reqs)
        launches = lib.htp_b200_launch_count() - before
    finally:
        chan.close()
    assert launches == (1 if m == 1 else 2)
    for layer, op, wq, x, fw, fx, fy in items:
        y = dev.get(fy, (m, op.n))
        check(oracle, y, x, wq, op.n, op.wtype)
        if layer == 0:
            e = g["oracle_layer0"][f"{op.name}_m{m}"]["oracle"]
            head, tail = np.array(e["head"]), np.array(e["tail"])
            ys = y[e["rows"]]
            assert np.abs(ys[:, :head.shape[1]] - head).max() <= 1e-5 * e["max_abs"]
            assert np.abs(ys[:, -tail.shape[1]:] - tail).max() <= 1e-5 * e["max_abs"]
            assert abs(float(y.astype(np.float64).sum()) - e["sum"]) <= 1e-5 * e["abs_sum"]
        dev.free(fw, fx, fy)
