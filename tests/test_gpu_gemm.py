"""GPU parity of the prefill GEMM (tcgen05 / TMEM): fp16 activations (M >= 9) or fp32 activations
converted to fp16 on the way in (M >= 17), against the fp64 oracle.  Gate: max|y - o| / max|o| <= 1e-3
(weights - and fp32 activations - are rounded to fp16 once, as the reference's dequantisation and
activation transfer do, src/dsp/ops/mat_mul.c:117, 290, 304; accumulation and output are fp32)."""
from __future__ import annotations

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def run(dev, oracle, wl, wtype, m, k, n, seed=0, tol=1e-3):
    wq, x = wl.random_case(900 + seed, wtype, True, m, k, n)
    before = dev.lib.htp_b200_launch_count()
    y = dev.matmul(x, wq, n, wtype)
    assert dev.lib.htp_b200_launch_count() == before + 1  # one GEMM launch, not token slices
    ref, absdot = oracle.mul_mat_f64(x, wq, n, wtype, want_absdot=True)
    e = oracle.error_metrics(y, ref, absdot)
    assert np.isfinite(y).all()
    assert e["max_rel_to_max"] <= tol and e["max_cond_rel"] <= tol, e
    return y


@pytest.mark.parametrize("wtype", [2, 8])
@pytest.mark.parametrize("m,k,n", [(128, 256, 256), (64, 256, 32), (128, 512, 224), (200, 1024, 480),
                                   (512, 2048, 1024), (65, 768, 96), (384, 4096, 2240)])
def test_gemm_shapes(dev, oracle, wl, wtype, m, k, n):
    """Full and ragged tiles in M and N, one and many K steps, more tiles than one wave has."""
    run(dev, oracle, wl, wtype, m, k, n)


@pytest.mark.parametrize("wtype", [2, 8])
@pytest.mark.parametrize("tile_n", [128, 256])
def test_gemm_many_tiles_per_cta(dev, oracle, wl, wtype, tile_n):
    """More tiles than SMs, so every CTA walks several tiles back to back with its rings full -
    the regime in which a raw-weight stage released too early was overwritten while still being
    read.  Three runs must agree bit for bit and match the oracle."""
    lib = dev.lib
    assert lib.htp_b200_set_option(b"gemm_tile_n", tile_n) == 0
    try:
        ys = [run(dev, oracle, wl, wtype, tile_n, 1024, 128 * 500, seed=9) for _ in range(3)]
    finally:
        lib.htp_b200_set_option(b"gemm_tile_n", 0)
    assert (ys[0] == ys[1]).all() and (ys[0] == ys[2]).all()


@pytest.mark.parametrize("wtype", [2, 8])
@pytest.mark.parametrize("m,k,n", [(300, 1024, 19360), (100, 2048, 128 * 190 + 96)])
def test_gemm_split_tiles(dev, oracle, wl, wtype, m, k, n):
    """Tile counts that do not divide among the SMs: the work is cut into equal K ranges and the
    tiles cut in two are finished through scratch.  Ragged in M and N; repeatable bit for bit;
    equal to the unsplit schedule up to fp32 summation order."""
    lib = dev.lib
    c = run(dev, oracle, wl, wtype, m, k, n, seed=5)  # whole tiles only (the default)
    old = lib.htp_b200_set_option(b"gemm_split", 1)
    try:
        a = run(dev, oracle, wl, wtype, m, k, n, seed=5)
        b = run(dev, oracle, wl, wtype, m, k, n, seed=5)
    finally:
        lib.htp_b200_set_option(b"gemm_split", old)
    assert (a == b).all()
    assert np.abs(a - c).max() <= 1e-5 * np.abs(c).max()


def test_gemm_is_deterministic(dev, oracle, wl):
    a = run(dev, oracle, wl, 2, 256, 1024, 512, seed=3)
    b = run(dev, oracle, wl, 2, 256, 1024, 512, seed=3)
    assert (a == b).all()


def test_gemm_matches_decode_kernel(dev, wl):
    """The same product through the decode kernel (token slices, exact integer weights) and the
    GEMM (fp16-rounded weights) agrees to the fp16 rounding of the weights."""
    lib = dev.lib
    wq, x = wl.random_case(77, 8, True, 128, 1024, 256)
    y_gemm = dev.matmul(x, wq, 256, 8)
    old = lib.htp_b200_set_option(b"gemm_min_m", 1 << 30)
    assert old == 9
    try:
        y_gemv = dev.matmul(x, wq, 256, 8)
    finally:
        lib.htp_b200_set_option(b"gemm_min_m", old)
    assert np.abs(y_gemm - y_gemv).max() <= 1e-3 * np.abs(y_gemv).max()


@pytest.mark.parametrize("wtype", [2, 8])
def test_gemm_multi_destination_band(dev, oracle, wl, wtype):
    """The fused form of "matmul on a row shard, then all-gather": the result goes into the column band
    [col0, col0 + n) of several destination matrices of ld floats per token.  Here both destinations
    are buffers of this GPU (on a multi-GPU box they are the ranks' logits buffers): each band must
    equal the plain result bit for bit and nothing outside the band may be touched."""
    import ctypes

    import torch
    m, k, n, ld, col0 = 200, 1024, 736, 2048, 512
    wq, x = wl.random_case(950, wtype, True, m, k, n)
    plain = dev.matmul(x, wq, n, wtype)
    tw, tx = torch.from_numpy(wq).cuda(), torch.from_numpy(x).cuda()
    dsts = [torch.full((m, ld), -7.0, dtype=torch.float32, device="cuda") for _ in range(3)]
    ptrs = (ctypes.c_void_p * 3)(*[d.data_ptr() for d in dsts])
    st = torch.cuda.current_stream().cuda_stream
    lib = dev.lib
    assert lib.htp_b200_mul_mat_multi_dst(ptrs, 3, ld, col0, tx.data_ptr(), tw.data_ptr(), m, k, n, wtype, 1, st) == 0
    torch.cuda.synchronize()
    assert lib.htp_b200_stream_status(st) == 0
    for d in dsts:
        h = d.cpu().numpy()
        assert (h[:, col0:col0 + n] == plain).all()
        assert (h[:, :col0] == -7.0).all() and (h[:, col0 + n:] == -7.0).all()
    # outside the kernel's range: rejected, nothing launched
    before = lib.htp_b200_launch_count()
    assert lib.htp_b200_mul_mat_multi_dst(ptrs, 3, ld, col0 + 16, tx.data_ptr(), tw.data_ptr(), m, k, n, wtype, 1, st) == -1
    assert lib.htp_b200_mul_mat_multi_dst(ptrs, 3, ld, ld - 32, tx.data_ptr(), tw.data_ptr(), m, k, n, wtype, 1, st) == -1
    assert lib.htp_b200_mul_mat_multi_dst(ptrs, 9, ld, col0, tx.data_ptr(), tw.data_ptr(), m, k, n, wtype, 1, st) == -1
    # fp32 activations beyond the decode kernel's range (m <= 8)
    assert lib.htp_b200_mul_mat_multi_dst(ptrs, 3, ld, col0, tx.data_ptr(), tw.data_ptr(), 12, k, n, wtype, 0, st) == -1
    assert lib.htp_b200_launch_count() == before


@pytest.mark.parametrize("wtype", [2, 8, 20])
@pytest.mark.parametrize("m,k,n", [(17, 256, 64), (32, 1024, 480), (64, 2048, 1024), (512, 4096, 2240), (100, 14336, 96)])
def test_gemm_fp32_activations(dev, oracle, wl, wtype, m, k, n):
    """The reference's own A32 ops (indices 2, 3, 4) at prefill sizes: ONE conversion launch (fp32 ->
    per-token scaled fp16) and ONE GEMM launch, never token slices through the decode kernel."""
    import torch
    wq, x = wl.random_case(990, wtype, False, m, k, n)
    x[0] *= 3.0e5  # beyond the fp16 range: the per-token power-of-two scale must absorb it
    x[1] *= 1.0e-6
    tw, tx = torch.from_numpy(wq).cuda(), torch.from_numpy(x).cuda()
    ty = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    before = dev.lib.htp_b200_launch_count()
    assert dev.lib.htp_b200_mul_mat(ty.data_ptr(), tx.data_ptr(), tw.data_ptr(), m, k, n, wtype, 0, st) == 0
    torch.cuda.synchronize()
    assert dev.lib.htp_b200_stream_status(st) == 0
    assert dev.lib.htp_b200_launch_count() == before + 2
    y = ty.cpu().numpy()
    ref = oracle.mul_mat_f64(x, wq, n, wtype)
    assert np.isfinite(y).all()
    for r in range(m):  # per token: the tokens differ by eleven orders of magnitude
        assert np.abs(y[r] - ref[r]).max() <= 1e-3 * np.abs(ref[r]).max(), r
    # the exact path stays available: decode kernel in slices of eight tokens, gate 1e-5
    old = dev.lib.htp_b200_set_option(b"a32_exact", 1)
    try:
        assert dev.lib.htp_b200_mul_mat(ty.data_ptr(), tx.data_ptr(), tw.data_ptr(), m, k, n, wtype, 0, st) == 0
        torch.cuda.synchronize()
    finally:
        dev.lib.htp_b200_set_option(b"a32_exact", old)
    y = ty.cpu().numpy()
    for r in range(m):
        assert np.abs(y[r] - ref[r]).max() <= 1e-5 * np.abs(ref[r]).max(), r


@pytest.mark.parametrize("wtype,m,k,n", [(2, 1024, 1024, 480), (8, 2500, 512, 256), (20, 4096, 256, 96)])
def test_gemm_thousands_of_tokens(dev, oracle, wl, wtype, m, k, n):
    """Token counts at which the reference switches to its pipelined schedule (m >= 1024,
    src/dsp/ops/mat_mul.c:925, 1006-1139): here the same GEMM launch walks more token tiles - full and
    ragged - through op indices 2 / 3 / 4 (fp32 activations) and through the fp16-activation entry."""
    if wtype != 20:  # (IQ4_NL has no fp16-activation op index)
        assert run(dev, oracle, wl, wtype, m, k, n, seed=5).shape == (m, n)
    wq, x = wl.random_case(995, wtype, False, m, k, n)
    fw, fx, fy = dev.put(wq), dev.put(x), dev.buf(m * n * 4)
    op = {2: dev.pkg.HTP_OPS_MAT_MUL_PERMUTED_W4D16A32, 8: dev.pkg.HTP_OPS_MAT_MUL_PERMUTED_W8D16A32,
          20: dev.pkg.HTP_OPS_MAT_MUL_PERMUTED_W4D16A32_IQ4_NL}[wtype]
    before = dev.lib.htp_b200_launch_count()
    assert dev.execute(op, (fy, 0), (fx, 0), (fw, 0), m, k, n) == 0
    assert dev.lib.htp_b200_launch_count() == before + 2  # conversion + GEMM
    y = dev.get(fy, (m, n))
    dev.free(fw, fx, fy)
    ref, absdot = oracle.mul_mat_f64(x, wq, n, wtype, want_absdot=True)
    e = oracle.error_metrics(y, ref, absdot)
    assert np.isfinite(y).all()
    assert e["max_rel_to_max"] <= 1e-3 and e["max_cond_rel"] <= 1e-3, e


@pytest.mark.parametrize("m", [9, 16, 24, 48, 63])
def test_gemm_fp16_between_decode_and_full_tiles(dev, oracle, wl, m):
    """9 .. 63 tokens: one GEMM launch on a padded 128-token tile (cheaper than one pass over the
    weights per eight tokens)."""
    run(dev, oracle, wl, 2, m, 1024, 992, seed=m)
