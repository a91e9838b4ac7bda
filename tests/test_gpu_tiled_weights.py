"""GPU parity of the matmul over weights in the reference's tile order: the fp16 tiles of
hmx_mat_mul_permuted_w16a32 (op index 1 and the RPC-named call; the shape of the reference's own
test, src/host/test.c:275-317, is among the cases) and the permuted Q4_0 / Q8_0 / IQ4_NL
super-blocks that the reference's ops 2, 3 and 4 consume (option "permuted_weights").  Gates as for
the standard-layout path: 1e-5 (fp32 activations) / 1e-3 (fp16) against the fp64 oracle, relative to
the largest output and to sum |x w| per output."""
from __future__ import annotations

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

Q4, Q8, IQ4 = 2, 8, 20
PERM = 0x100
FMTS = [1, PERM | Q4, PERM | Q8, PERM | IQ4]
SHAPES = [(1, 1024, 1024), (1, 256, 32), (2, 2048, 480), (3, 1024, 224), (7, 512, 96), (8, 4096, 256),
          (1, 14336, 64), (20, 512, 64), (1, 96, 64), (5, 32, 32)]


def _check(oracle, y, x, wq, n, fmt, tol):
    ref, absdot = oracle.tiled_mul_mat_f64(x, wq, n, fmt, want_absdot=True)
    e = oracle.error_metrics(y, ref, absdot)
    assert np.isfinite(y).all()
    assert e["max_rel_to_max"] <= tol and e["max_cond_rel"] <= tol, e


def _raw(dev, x, wq, n, fmt):
    import torch
    m, k = x.shape
    tw = torch.from_numpy(wq).cuda()
    tx = torch.from_numpy(x).cuda()
    ty = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    before = dev.lib.htp_b200_launch_count()
    rc = dev.lib.htp_b200_mul_mat(ty.data_ptr(), tx.data_ptr(), tw.data_ptr(), m, k, n, fmt,
                                  1 if x.dtype == np.float16 else 0, st)
    assert rc == 0
    # one launch; fp32 activations on their way to the tensor-core GEMM take a conversion launch first
    assert dev.lib.htp_b200_launch_count() == before + (2 if _gemm_path(fmt, x) and x.dtype == np.float32 else 1)
    assert dev.lib.htp_b200_stream_status(st) == 0
    return ty.cpu().numpy()


def _gemm_path(fmt, x) -> bool:
    """Every tile-order format with many tokens runs on the tensor-core GEMM (fp16 activations from 9
    tokens, fp32 from 17, k % 128 == 0): weights and activations rounded to fp16, gate 1e-3."""
    m, k = x.shape
    return k % 128 == 0 and m >= (9 if x.dtype == np.float16 else 17)


@pytest.mark.parametrize("act_f16", [False, True])
@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("m,k,n", SHAPES)
def test_tile_order_matmul_matches_oracle(dev, oracle, wl, fmt, act_f16, m, k, n):
    wq, x = wl.tiled_random_case(50, fmt, act_f16, m, k, n)
    assert wq.size == dev.lib.htp_b200_weight_bytes(fmt, k, n)
    _check(oracle, _raw(dev, x, wq, n, fmt), x, wq, n, fmt, 1e-3 if act_f16 or _gemm_path(fmt, x) else 1e-5)


@pytest.mark.parametrize("act_f16", [False, True])
@pytest.mark.parametrize("m,k,n", [(17, 128, 32), (64, 1024, 1024), (200, 2048, 480), (512, 4096, 2240), (300, 1152, 19360 // 32 * 32)])
def test_fp16_tiles_many_tokens_on_the_tensor_cores(dev, oracle, wl, act_f16, m, k, n):
    """The reference's W16A32 op takes any m (src/dsp/ops/mat_mul.c:758-855): many tokens over fp16 tiles
    run as ONE tensor-core GEMM launch that reads the tiles as they lie - full and ragged tiles in M and
    N, one and many K steps, K a multiple of 128 but not of 256, more tiles than one wave."""
    wq, x = wl.tiled_random_case(60 + m, 1, act_f16, m, k, n)
    if not act_f16:
        x[0] *= 1.0e5  # beyond the fp16 range: absorbed by the per-token scale
    y = _raw(dev, x, wq, n, 1)
    ref = oracle.tiled_mul_mat_f64(x, wq, n, 1)
    assert np.isfinite(y).all()
    for r in range(m):
        assert np.abs(y[r] - ref[r]).max() <= 1e-3 * np.abs(ref[r]).max(), r
    # through the op registry (index 1) as well: same bytes
    if not act_f16:
        fw, fx, fy = dev.put(wq), dev.put(x), dev.buf(m * n * 4)
        assert dev.execute(dev.pkg.HTP_OPS_MAT_MUL_PERMUTED_W16A32, (fy, 0), (fx, 0), (fw, 0), m, k, n) == 0
        assert (dev.get(fy, (m, n)) == y).all()
        dev.free(fw, fx, fy)


@pytest.mark.parametrize("act_f16", [False, True])
@pytest.mark.parametrize("wtype", [Q4, Q8, IQ4])
@pytest.mark.parametrize("m,k,n", [(17, 128, 32), (64, 1024, 1024), (200, 2176, 480), (512, 4096, 2240), (300, 1152, 19360 // 32 * 32)])
def test_permuted_super_blocks_many_tokens_on_the_tensor_cores(dev, oracle, wl, wtype, act_f16, m, k, n):
    """The reference's quantised ops take any m over its permuted super-blocks
    (src/dsp/ops/mat_mul.c:875-1005, expansion to fp16 at :308-510): many tokens run as ONE tensor-core
    GEMM launch whose unpack reads the super-blocks as they lie, value * scale rounded to fp16 once as
    the reference does - full and ragged tiles in M and N, one and many K steps, K a multiple of 128 but
    not of 256, more tiles than one wave.  Also through op indices 2, 3, 4 with the option set."""
    fmt = PERM | wtype
    wq, x = wl.tiled_random_case(70 + m, fmt, act_f16, m, k, n)
    if not act_f16:
        x[0] *= 1.0e5  # beyond the fp16 range: absorbed by the per-token scale
    y = _raw(dev, x, wq, n, fmt)
    ref = oracle.tiled_mul_mat_f64(x, wq, n, fmt)
    assert np.isfinite(y).all()
    for r in range(m):
        assert np.abs(y[r] - ref[r]).max() <= 1e-3 * np.abs(ref[r]).max(), r
    if not act_f16 and m <= 200:
        op = {Q4: dev.pkg.HTP_OPS_MAT_MUL_PERMUTED_W4D16A32, Q8: dev.pkg.HTP_OPS_MAT_MUL_PERMUTED_W8D16A32,
              IQ4: dev.pkg.HTP_OPS_MAT_MUL_PERMUTED_W4D16A32_IQ4_NL}[wtype]
        fw, fx, fy = dev.put(wq), dev.put(x), dev.buf(m * n * 4)
        old = dev.lib.htp_b200_set_option(b"permuted_weights", 1)
        try:
            assert dev.execute(op, (fy, 0), (fx, 0), (fw, 0), m, k, n) == 0
        finally:
            dev.lib.htp_b200_set_option(b"permuted_weights", old)
        assert (dev.get(fy, (m, n)) == y).all()
        dev.free(fw, fx, fy)


def test_tile_order_matmul_matches_committed_golden_samples(dev):
    """The committed fixtures (tests/golden/golden_tiled.json): same seeded inputs, GPU output against the
    stored fp64 samples."""
    import json
    from pathlib import Path

    from test_tiled_formats import golden_module
    gm = golden_module()
    golden = json.loads((Path(__file__).parent / "golden" / "golden_tiled.json").read_text())
    for name, want in golden.items():
        fmt, n, wq, x = gm.make_case(name)
        assert gm.wl.sha256(wq) == want["w_sha256"]
        y = _raw(dev, x, wq, n, fmt)
        tol = 1e-3 if x.dtype == np.float16 else 1e-5
        scale = max(np.abs(np.array(want["head"])).max(), np.abs(np.array(want["tail"])).max())
        assert np.abs(y[:, :16] - np.array(want["head"])).max() <= tol * scale
        assert np.abs(y[:, -16:] - np.array(want["tail"])).max() <= tol * scale


@pytest.mark.parametrize("wtype", [Q4, Q8, IQ4])
def test_permuted_group_sums_bit_exact(dev, oracle, wtype):
    """Integer sums per scale group through the decode routines the matmul kernel uses, on random bytes
    (every nibble / byte value in every position): bit-exact against the oracle."""
    import torch
    fmt = PERM | wtype
    sbb = 272 if wtype == Q8 else 144
    rng = np.random.default_rng(60 + wtype)
    buf = rng.integers(0, 256, size=1000 * sbb, dtype=np.uint8)
    tw = torch.from_numpy(buf).cuda()
    s = torch.empty(8000, dtype=torch.int32, device="cuda")
    t = torch.empty(8000, dtype=torch.int32, device="cuda")
    assert dev.lib.htp_b200_block_sums(tw.data_ptr(), s.data_ptr(), t.data_ptr(), 8000, fmt, None) == 0
    torch.cuda.synchronize()
    so, to = oracle.tiled_group_sums(buf, fmt)
    assert (s.cpu().numpy() == so).all() and (t.cpu().numpy() == to).all()
    assert dev.lib.htp_b200_block_sums(tw.data_ptr(), s.data_ptr(), t.data_ptr(), 12, fmt, None) == -1  # not whole super-blocks
    assert dev.lib.htp_b200_block_sums(tw.data_ptr(), s.data_ptr(), t.data_ptr(), 8, 1, None) == -1  # fp16 tiles: no integers


def test_w16a32_rpc_named_call_on_the_reference_test_shape(dev, oracle, wl):
    """m = 1, k = 1024, n = 1024, inputs uniform in [0, 1) as in src/host/test.c:281-313; the call is the
    one that test makes (htp_ops_mat_mul_permuted_w16a32 on three mapped buffers)."""
    m, k, n = 1, 1024, 1024
    rng = np.random.Generator(np.random.PCG64(51))
    x = rng.random((m, k), dtype=np.float32)
    w = rng.random((k, n), dtype=np.float32)
    wq = wl.pack_f16_tiles(w)
    fw, fx, fy = dev.put(wq), dev.put(x), dev.buf(m * n * 4)
    assert dev.lib.htp_ops_mat_mul_permuted_w16a32(dev.lib.get_global_handle(), fy, 0, fx, 0, fw, 0, m, k, n) == 0
    y = dev.get(fy, (m, n))
    _check(oracle, y, x, wq, n, 1, 1e-5)
    # and against plain fp64 on the fp16-rounded matrix, the reference test's own "f32" column
    ref = x.astype(np.float64) @ w.astype(np.float16).astype(np.float64)
    assert np.abs(y - ref).max() <= 1e-5 * np.abs(ref).max()
    # the wrapper of include/host/op_export.h and the op registry give the same bytes
    fz = dev.buf(m * n * 4)
    assert dev.lib.htp_ops_rpc_mat_mul_permuted_w16a32(fz, 0, fx, 0, fw, 0, m, k, n) == 0
    assert (dev.get(fz, (m, n)) == y).all()
    assert dev.execute(dev.pkg.HTP_OPS_MAT_MUL_PERMUTED_W16A32, (fz, 0), (fx, 0), (fw, 0), m, k, n) == 0
    assert (dev.get(fz, (m, n)) == y).all()
    # the reference's argument rules: k % 32, n % 32, buffer sizes
    assert dev.lib.htp_ops_mat_mul_permuted_w16a32(dev.lib.get_global_handle(), fy, 0, fx, 0, fw, 0, m, k, n + 16) != 0
    assert dev.lib.htp_ops_mat_mul_permuted_w16a32(dev.lib.get_global_handle(), fy, 0, fx, 0, fw, 0, m, k + 8, n) != 0
    assert dev.lib.htp_ops_mat_mul_permuted_w16a32(dev.lib.get_global_handle(), fy, 0, fx, 0, fw, 0, m, k, 2 * n) != 0
    dev.free(fw, fx, fy, fz)


@pytest.mark.parametrize("wtype,op_name", [(Q4, "HTP_OPS_MAT_MUL_PERMUTED_W4D16A32"),
                                           (Q8, "HTP_OPS_MAT_MUL_PERMUTED_W8D16A32"),
                                           (IQ4, "HTP_OPS_MAT_MUL_PERMUTED_W4D16A32_IQ4_NL")])
def test_ops_2_3_4_read_permuted_super_blocks_when_asked(dev, oracle, wl, wtype, op_name):
    m, k, n = 2, 1024, 256
    wq, x = wl.tiled_random_case(52, PERM | wtype, False, m, k, n)
    fw, fx, fy = dev.put(wq), dev.put(x), dev.buf(m * n * 4)
    op = getattr(dev.pkg, op_name)
    prev = dev.lib.htp_b200_set_option(b"permuted_weights", 1)
    try:
        assert dev.execute(op, (fy, 0), (fx, 0), (fw, 0), m, k, n) == 0
        y = dev.get(fy, (m, n))
    finally:
        dev.lib.htp_b200_set_option(b"permuted_weights", prev)
    _check(oracle, y, x, wq, n, PERM | wtype, 1e-5)
    dev.free(fw, fx, fy)


def test_tile_order_formats_are_rejected_where_not_supported(dev, wl):
    import torch
    m, k, n = 1, 256, 64
    wq, x = wl.tiled_random_case(53, 1, False, m, k, n)
    tw, tx = torch.from_numpy(wq).cuda(), torch.from_numpy(x).cuda()
    ty = torch.empty((m, n), dtype=torch.float32, device="cuda")
    lib = dev.lib
    assert lib.htp_b200_mul_mat_static_scratch(ty.data_ptr(), tx.data_ptr(), tw.data_ptr(), m, k, n, 1, 0, None) != 0
    assert lib.htp_b200_mul_mat(ty.data_ptr(), tx.data_ptr(), tw.data_ptr(), m, k, n, PERM | 3, 0, None) == -1
    assert lib.htp_b200_mul_mat(ty.data_ptr(), tx.data_ptr(), tw.data_ptr(), m, k + 16, n, 1, 0, None) == -1
    assert lib.htp_b200_weight_bytes(1, 256, 48) == 0 and lib.htp_b200_weight_bytes(PERM | 8, 256, 64) == 16 * 1088
    torch.cuda.synchronize()
