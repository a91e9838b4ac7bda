"""GPU parity: the CUDA path, called through the C ABI, against the fp64 oracle on the same seeded
inputs.  Gate: max|y - o| / max|o| <= 1e-5 for fp32 activations, <= 1e-3 for fp16 activations;
integer block sums bit-exact."""
from __future__ import annotations

import ctypes
import json
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GOLDEN = json.loads((Path(__file__).parent / "golden" / "golden.json").read_text())
TOL = {False: 1e-5, True: 1e-3}


def check(oracle, y, x, wq, n, wtype, tol=None):
    ref, absdot = oracle.mul_mat_f64(x, wq, n, wtype, want_absdot=True)
    e = oracle.error_metrics(y, ref, absdot)
    tol = TOL[x.dtype == np.float16] if tol is None else tol
    assert np.isfinite(y).all()
    assert e["max_rel_to_max"] <= tol, e
    assert e["max_cond_rel"] <= tol, e
    return e


def near(y, g, tol):
    """GPU output against a fixture: sampled outputs and the whole-matrix checksum."""
    head, tail = np.array(g["head"]), np.array(g["tail"])
    ys = y[g["rows"]]
    assert np.abs(ys[:, :head.shape[1]] - head).max() <= tol * g["max_abs"]
    assert np.abs(ys[:, -tail.shape[1]:] - tail).max() <= tol * g["max_abs"]
    assert abs(float(y.astype(np.float64).sum()) - g["sum"]) <= tol * g["abs_sum"]


# ------------------------------------------------------------------ integer unpack probe

@pytest.mark.parametrize("wtype", [2, 8])
def test_block_sums_bit_exact(dev, oracle, wl, wtype):
    """S_b = sum v_i and T_b = sum (i+1) v_i of every block, computed on the GPU with the unpack
    routines the matmul kernels use, equal the oracle's bit for bit.  (The reference has no integer
    path; this is the checkable integer invariant of the unpack: value, sign and element order.)"""
    rng = np.random.default_rng(3)
    nb = 4096 + 17
    raw = rng.integers(0, 256, nb * wl.BLOCK_BYTES[wtype], dtype=np.uint8)
    if wtype == 8:  # all byte values in sliding positions up front
        for b in range(256):
            raw[b * 34 + 2:b * 34 + 34] = (np.arange(32) * 7 + b) % 256
    fw = dev.put(raw)
    fs, ft = dev.buf(nb * 4), dev.buf(nb * 4)
    lib = dev.lib
    assert lib.htp_b200_block_sums(lib.htp_buf_ptr(fw), lib.htp_buf_ptr(fs), lib.htp_buf_ptr(ft), nb, wtype,
                                   lib.htp_session_stream()) == 0
    assert lib.htp_session_synchronize() == 0
    s, t = dev.get(fs, nb, np.int32), dev.get(ft, nb, np.int32)
    so, to = oracle.block_sums(raw, wtype)
    assert (s == so).all() and (t == to).all()
    dev.free(fw, fs, ft)


@pytest.mark.parametrize("name", ["cfg0", "cfg1"])
def test_block_sums_of_config_weights(dev, oracle, wl, name):
    cfg, g = wl.CONFIGS[name], GOLDEN[name]
    op = cfg.ops[0]
    wq = wl.make_weight(cfg, quantizer=lambda w, t: oracle.quantize(w, t))
    nb = wq.size // wl.BLOCK_BYTES[op.wtype]
    fw, fs, ft = dev.put(wq), dev.buf(nb * 4), dev.buf(nb * 4)
    lib = dev.lib
    assert lib.htp_b200_block_sums(lib.htp_buf_ptr(fw), lib.htp_buf_ptr(fs), lib.htp_buf_ptr(ft), nb, op.wtype,
                                   lib.htp_session_stream()) == 0
    assert lib.htp_session_synchronize() == 0
    assert wl.sha256(dev.get(fs, nb, np.int32)) == g["block_sum_s_sha256"]
    assert wl.sha256(dev.get(ft, nb, np.int32)) == g["block_sum_t_sha256"]
    dev.free(fw, fs, ft)


# ------------------------------------------------------------------ small shapes, every M

SHAPES = [(256, 32), (512, 64), (1024, 96), (1280, 32), (2048, 160), (4096, 1024), (14336, 64), (96, 32), (736, 64)]


@pytest.mark.parametrize("wtype", [2, 8])
@pytest.mark.parametrize("act_f16", [False, True])
@pytest.mark.parametrize("k,n", SHAPES)
def test_small_shapes_all_m(dev, oracle, wl, wtype, act_f16, k, n):
    """M = 1..9 (decode kernel, with the M > 8 split), shapes that exercise a single stage, a
    partial last stage, tiles cut by CTA boundaries, K chunking, and K % 256 != 0 (fallback)."""
    for m in (1, 2, 3, 4, 5, 7, 8, 9):
        wq, x = wl.random_case(100 + m, wtype, act_f16, m, k, n)
        y = dev.matmul(x, wq, n, wtype)
        check(oracle, y, x, wq, n, wtype)


@pytest.mark.parametrize("wtype", [2, 8])
def test_exhaustive_values_tiny(dev, oracle, wl, wtype):
    """K = 256, N = 32: every nibble / byte value appears, activations are basis-like so that a
    misplaced element changes the result by O(1)."""
    k, n = 256, 32
    rng = np.random.default_rng(5)
    bb = wl.BLOCK_BYTES[wtype]
    raw = rng.integers(0, 256, n * (k // 32) * bb, dtype=np.uint8).reshape(n, k // 32, bb)
    raw[:, :, :2] = np.frombuffer(np.float16(0.25).tobytes(), dtype=np.uint8)
    for r in range(n):
        for b in range(k // 32):
            raw[r, b, 2:] = (np.arange(bb - 2) * 5 + r * 8 + b) % 256
    wq = raw.reshape(-1)
    x = np.zeros((8, k), dtype=np.float32)
    for m in range(8):
        x[m, m::8] = np.arange(1, k // 8 + 1, dtype=np.float32)
    y = dev.matmul(x, wq, n, wtype)
    ref = oracle.mul_mat_f64(x, wq, n, wtype)
    assert np.abs(y - ref).max() <= 1e-6 * np.abs(ref).max()


def test_large_magnitude_fp32_activations(dev, oracle, wl):
    """fp32 activations beyond the fp16 range: the per-token power-of-two pre-scale keeps 1e-5."""
    wq, x = wl.random_case(9, 2, False, 4, 1024, 64)
    x[0] *= 3.0e5
    x[1] *= 1.0e-6
    x[2, 17] = 7.5e7
    y = dev.matmul(x, wq, 64, 2)
    ref = oracle.mul_mat_f64(x, wq, 64, 2)
    for m in range(4):
        assert np.abs(y[m] - ref[m]).max() <= 1e-5 * np.abs(ref[m]).max()


def test_repeat_runs_are_bit_identical(dev, wl):
    wq, x = wl.random_case(21, 2, False, 1, 4096, 1024)
    a = dev.matmul(x, wq, 1024, 2)
    for _ in range(3):
        assert (dev.matmul(x, wq, 1024, 2) == a).all()


# ------------------------------------------------------------------ the benchmark configurations

@pytest.mark.parametrize("name", ["cfg0", "cfg1"])
def test_config_gemv(dev, oracle, wl, name):
    cfg, g = wl.CONFIGS[name], GOLDEN[name]
    op, m = cfg.ops[0], g["m"]
    wq = wl.make_weight(cfg, quantizer=lambda w, t: oracle.quantize(w, t))
    x = wl.make_activation(cfg, m)
    assert wl.sha256(wq) == g["w_sha256"] and wl.sha256(x) == g["x_sha256"]
    y = dev.matmul(x, wq, op.n, op.wtype)
    check(oracle, y, x, wq, op.n, op.wtype)
    near(y, g["oracle"], TOL[op.act_f16])


def test_config2_prefill(dev, oracle, wl):
    cfg, g = wl.CONFIGS["cfg2"], GOLDEN["cfg2"]
    op, m = cfg.ops[0], 512
    wq = wl.make_weight(cfg, quantizer=lambda w, t: oracle.quantize(w, t))
    x = wl.make_activation(cfg, m)
    assert wl.sha256(wq) == g["w_sha256"] and wl.sha256(x) == g["x_sha256"]
    y = dev.matmul(x, wq, op.n, op.wtype)
    near(y, g["oracle"], 1e-3)
    # full comparison on a band of 2048 output columns (the oracle is a scalar fp64 loop)
    c0 = 6144
    rows = wq.reshape(op.n, -1)[c0:c0 + 2048].reshape(-1)
    ref = oracle.mul_mat_f64(x, rows, 2048, op.wtype)
    assert oracle.error_metrics(y[:, c0:c0 + 2048], ref)["max_rel_to_max"] <= 1e-3


@pytest.mark.parametrize("m", [1, 8])
def test_config3_layer0(dev, oracle, wl, m):
    """All seven matrices of decoder layer 0, issued in order, against oracle and fixtures."""
    cfg, g = wl.CONFIGS["cfg3"], GOLDEN["cfg3"]
    for i, op in enumerate(cfg.ops):
        wq = wl.make_weight(cfg, i, 0, quantizer=lambda w, t: oracle.quantize(w, t))
        assert wl.sha256(wq) == g["layers"]["0"][op.name]
        x = wl.make_activation(cfg, m, i, 0)
        y = dev.matmul(x, wq, op.n, op.wtype)
        check(oracle, y, x, wq, op.n, op.wtype)
        e = g["oracle_layer0"][f"{op.name}_m{m}"]
        near(y, e["oracle"], 1e-5)


def test_config4_lm_head_single_gpu(dev, oracle, wl):
    """The whole 128256 x 4096 Q8_0 lm_head on one GPU at M = 1 (full oracle) and M = 256 (fixture
    samples, a column band against the oracle, and linearity as the size-independent property)."""
    cfg, g = wl.CONFIGS["cfg4"], GOLDEN["cfg4"]
    op = cfg.ops[0]
    wq = wl.make_weight(cfg, quantizer=lambda w, t: oracle.quantize(w, t))
    assert wl.sha256(wq) == g["w_sha256"]
    fw = dev.put(wq)
    opi = dev.op_index(op.wtype, True)
    for m in (1, 256):
        x = wl.make_activation(cfg, m)
        assert wl.sha256(x) == g[f"m{m}"]["x_sha256"]
        fx, fy = dev.put(x), dev.buf(m * op.n * 4)
        assert dev.execute(opi, (fy, 0), (fx, 0), (fw, 0), m, op.k, op.n) == 0
        y = dev.get(fy, (m, op.n))
        e = g[f"m{m}"]["oracle"]
        near(y, e, 1e-3)
        if m == 1:
            check(oracle, y, x, wq, op.n, op.wtype)
        else:
            c0 = 64128 - 512
            rows = wq.reshape(op.n, -1)[c0:c0 + 1024].reshape(-1)
            ref = oracle.mul_mat_f64(x, rows, 1024, op.wtype)
            assert oracle.error_metrics(y[:, c0:c0 + 1024], ref)["max_rel_to_max"] <= 1e-3
            # linearity: rows of y for x0 + x1 (exactly representable sums) = y0 + y1
            x2 = (x[:128].astype(np.float32) * 0.5 + x[128:].astype(np.float32) * 0.5).astype(np.float16)
            fx2, fy2 = dev.put(x2), dev.buf(128 * op.n * 4)
            assert dev.execute(opi, (fy2, 0), (fx2, 0), (fw, 0), 128, op.k, op.n) == 0
            y2 = dev.get(fy2, (128, op.n))
            lin = 0.5 * (y[:128].astype(np.float64) + y[128:].astype(np.float64))
            assert np.abs(y2 - lin).max() <= 2e-3 * np.abs(lin).max()
            dev.free(fx2, fy2)
        dev.free(fx, fy)
    dev.free(fw)


# ------------------------------------------------------------------ the raw compute entry point

def test_raw_entry_point_checks_arguments(dev, wl):
    """htp_b200_mul_mat keeps the reference's checks (mat_mul.c:878-892): -1, nothing launched."""
    lib = dev.lib
    wq, x = wl.random_case(1, 2, False, 1, 256, 32)
    fw, fx, fy = dev.put(wq), dev.put(x), dev.buf(4096)
    w, a, y, st = lib.htp_buf_ptr(fw), lib.htp_buf_ptr(fx), lib.htp_buf_ptr(fy), lib.htp_session_stream()
    before = lib.htp_b200_launch_count()
    assert lib.htp_b200_mul_mat(None, a, w, 1, 256, 32, 2, 0, st) == -1
    assert lib.htp_b200_mul_mat(y, a, w, 0, 256, 32, 2, 0, st) == -1
    assert lib.htp_b200_mul_mat(y, a, w, 1, 250, 32, 2, 0, st) == -1
    assert lib.htp_b200_mul_mat(y, a, w, 1, 256, 48, 2, 0, st) == -1
    assert lib.htp_b200_mul_mat(y, a + 64, w, 1, 256, 32, 2, 0, st) == -1
    assert lib.htp_b200_mul_mat(y, a, w, 1, 256, 32, 3, 0, st) == -1
    assert lib.htp_b200_mul_mat(y, a, w, 1, 256, 32, 2, 5, st) == -1
    assert lib.htp_b200_launch_count() == before
    assert lib.htp_b200_mul_mat(y, a, w, 1, 256, 32, 2, 0, st) == 0
    assert lib.htp_b200_stream_status(st) == 0
    assert lib.htp_b200_launch_count() == before + 1
    dev.free(fw, fx, fy)


def test_generic_kernel_matches_streaming_kernel(dev, oracle, wl):
    lib = dev.lib
    wq, x = wl.random_case(33, 8, True, 6, 1024, 128)
    y_fast = dev.matmul(x, wq, 128, 8)
    assert lib.htp_b200_set_option(b"force_generic", 1) == 0
    try:
        y_gen = dev.matmul(x, wq, 128, 8)
    finally:
        lib.htp_b200_set_option(b"force_generic", 0)
    check(oracle, y_gen, x, wq, 128, 8)
    assert np.abs(y_gen - y_fast).max() <= 1e-3 * np.abs(y_fast).max()


# ------------------------------------------------------------------ batched decode launches

@pytest.mark.parametrize("wtype,act_f16,m", [(2, False, 1), (8, True, 1), (2, False, 3), (2, True, 8)])
def test_batched_independent_ops(dev, oracle, wl, wtype, act_f16, m):
    """Several independent mat-vecs of different shapes as ONE launch (htp_b200_mul_mat_batch):
    every operator's result meets the oracle gate and agrees with its single-launch result to fp32
    rounding (tiles are cut at different places, so the fp32 summation order differs).
    Shapes chosen so that CTA ranges cross operator boundaries inside and between tiles."""
    import ctypes
    lib = dev.lib
    shapes = [(1024, 256), (1024, 32), (4096, 1024), (256, 96), (2048, 4096), (4096, 128), (1024, 2016)]
    cases = [wl.random_case(700 + i, wtype, act_f16, m, k, n) for i, (k, n) in enumerate(shapes)]
    fw = [dev.put(wq) for wq, _ in cases]
    fx = [dev.put(x) for _, x in cases]
    fy = [dev.buf(m * n * 4) for _, n in shapes]
    n_ops = len(shapes)
    arr = lambda fds: (ctypes.c_void_p * n_ops)(*[lib.htp_buf_ptr(f) for f in fds])
    ks = (ctypes.c_int * n_ops)(*[k for k, _ in shapes])
    ns = (ctypes.c_int * n_ops)(*[n for _, n in shapes])
    before = lib.htp_b200_launch_count()
    rc = lib.htp_b200_mul_mat_batch(n_ops, arr(fy), arr(fx), arr(fw), ks, ns, m, wtype, 1 if act_f16 else 0,
                                    lib.htp_session_stream())
    assert rc == 0
    assert lib.htp_session_synchronize() == 0
    assert lib.htp_b200_launch_count() == before + 1
    for i, ((k, n), (wq, x)) in enumerate(zip(shapes, cases)):
        y = dev.get(fy[i], (m, n))
        check(oracle, y, x, wq, n, wtype)
        y1 = dev.matmul(x, wq, n, wtype)
        assert np.abs(y - y1).max() <= 2e-6 * np.abs(y1).max()
    # an operator that cannot join a batch is refused, nothing is launched
    ks_bad = (ctypes.c_int * n_ops)(*([96] + [k for k, _ in shapes][1:]))
    assert lib.htp_b200_mul_mat_batch(n_ops, arr(fy), arr(fx), arr(fw), ks_bad, ns, m, wtype, 1 if act_f16 else 0,
                                      lib.htp_session_stream()) == -1
    dev.free(*fw, *fx, *fy)


def test_channel_batches_independent_requests(dev, oracle, wl):
    """A message of twelve independent requests plus one that reads an earlier output: the servicer
    issues the independent ones as one launch and the dependent one after it."""
    lib, pkg = dev.lib, dev.pkg
    op = pkg.HTP_OPS_MAT_MUL_PERMUTED_W4D16A32
    shapes = [(1024, 512), (1024, 64), (2048, 256)] * 4
    cases = [wl.random_case(800 + i, 2, False, 1, k, n) for i, (k, n) in enumerate(shapes)]
    fw = [dev.put(wq) for wq, _ in cases]
    fx = [dev.put(x) for _, x in cases]
    fy = [dev.buf(n * 4) for _, n in shapes]
    wdep, _ = wl.random_case(899, 2, False, 1, 512, 128)
    fwd, fyd = dev.put(wdep), dev.buf(128 * 4)
    reqs = [pkg.pack_matmul_request(op, (fy[i], 0), (fx[i], 0), (fw[i], 0), 1, k, n) for i, (k, n) in enumerate(shapes)]
    reqs.append(pkg.pack_matmul_request(op, (fyd, 0), (fy[0], 0), (fwd, 0), 1, 512, 128))  # reads output 0
    chan = pkg.MessageChannel(4096)
    try:
        before = lib.htp_b200_launch_count()
        assert chan.submit(reqs) == [0] * 13
        assert lib.htp_b200_launch_count() == before + 2
    finally:
        chan.close()
    for i, ((k, n), (wq, x)) in enumerate(zip(shapes, cases)):
        check(oracle, dev.get(fy[i], (1, n)), x, wq, n, 2)
    h = dev.get(fy[0], (1, 512))
    check(oracle, dev.get(fyd, (1, 128)), h, wdep, 128, 2)
    dev.free(*fw, *fx, *fy, fwd, fyd)


@pytest.mark.parametrize("wtype,act_f16,m", [(2, False, 1), (2, True, 2), (8, True, 1), (8, False, 3), (2, False, 8)])
def test_decode_multi_destination_band(dev, oracle, wl, wtype, act_f16, m):
    """Decode output as the column band [col0, col0 + n) of several destination matrices (on a
    multi-GPU box: every rank's copy of a row-sharded output): each band equals the plain result bit
    for bit, nothing else is touched."""
    import ctypes

    import torch
    k, n, ld, col0 = 1024, 608, 1536, 352
    wq, x = wl.random_case(960 + m, wtype, act_f16, m, k, n)
    plain = dev.matmul(x, wq, n, wtype)
    tw, tx = torch.from_numpy(wq).cuda(), torch.from_numpy(x).cuda()
    dsts = [torch.full((m, ld), -7.0, dtype=torch.float32, device="cuda") for _ in range(3)]
    ptrs = (ctypes.c_void_p * 3)(*[d.data_ptr() for d in dsts])
    st = torch.cuda.current_stream().cuda_stream
    assert dev.lib.htp_b200_mul_mat_multi_dst(ptrs, 3, ld, col0, tx.data_ptr(), tw.data_ptr(), m, k, n, wtype,
                                              1 if act_f16 else 0, st) == 0
    torch.cuda.synchronize()
    assert dev.lib.htp_b200_stream_status(st) == 0
    for d in dsts:
        h = d.cpu().numpy()
        assert (h[:, col0:col0 + n] == plain).all()
        assert (h[:, :col0] == -7.0).all() and (h[:, col0 + n:] == -7.0).all()


def test_decode_completion_flags(dev, wl):
    """The signalling form: after the launch every destination's flag word holds the epoch; the wait
    kernel passes for an epoch that has been reached and, for one that nothing raises, gives up
    after its bounded wait with error 103 in the stream's error word (no hang, context intact)."""
    import ctypes

    import torch
    m, k, n, ld = 1, 1024, 608, 1536
    wq, x = wl.random_case(970, 8, True, m, k, n)
    plain = dev.matmul(x, wq, n, 8)
    tw, tx = torch.from_numpy(wq).cuda(), torch.from_numpy(x).cuda()
    dsts = [torch.zeros((m, ld), dtype=torch.float32, device="cuda") for _ in range(2)]
    flags = torch.zeros(32, dtype=torch.int32, device="cuda")
    ptrs = (ctypes.c_void_p * 2)(*[d.data_ptr() for d in dsts])
    fptrs = (ctypes.c_void_p * 2)(flags.data_ptr(), flags.data_ptr() + 4)
    st = torch.cuda.current_stream().cuda_stream
    lib = dev.lib
    for epoch in (1, 2, 3):
        assert lib.htp_b200_mul_mat_multi_dst_signal(ptrs, 2, ld, 0, tx.data_ptr(), tw.data_ptr(), m, k, n, 8, 1, fptrs,
                                                     epoch, st) == 0
        assert lib.htp_b200_wait_flags(flags.data_ptr(), 2, epoch, st) == 0
        torch.cuda.synchronize()
        assert flags[:2].tolist() == [epoch, epoch]
    assert lib.htp_b200_stream_status(st) == 0
    assert all((d.cpu().numpy()[:, :n] == plain).all() for d in dsts)
    assert lib.htp_b200_wait_flags(flags.data_ptr(), 2, 4, st) == 0  # nobody raises epoch 4
    assert lib.htp_b200_stream_status(st) == 103
    assert lib.htp_b200_stream_status(st) == 0  # cleared; the stream still works
    assert lib.htp_b200_wait_flags(flags.data_ptr(), 2, 3, st) == 0 and lib.htp_b200_stream_status(st) == 0
