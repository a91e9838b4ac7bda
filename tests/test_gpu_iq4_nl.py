"""GPU parity of the IQ4_NL variant (op index 4): the Q4_0 block with the reference's non-linear
value table (src/dsp/ops/mat_mul.c:29-32, selected at :316 and :583).  Same gates as Q4_0: block sums
bit-exact, decode 1e-5 (fp32 activations) / 1e-3 (fp16), prefill GEMM 1e-3, against the fp64 oracle."""
from __future__ import annotations

import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
IQ4 = 20


def _check(dev, oracle, y, x, wq, n, tol):
    ref, absdot = oracle.mul_mat_f64(x, wq, n, IQ4, want_absdot=True)
    e = oracle.error_metrics(y, ref, absdot)
    assert np.isfinite(y).all()
    assert e["max_rel_to_max"] <= tol and e["max_cond_rel"] <= tol, e


def _raw(dev, x, wq, n):
    import torch
    m, k = x.shape
    tw = torch.from_numpy(wq).cuda()
    tx = torch.from_numpy(x).cuda()
    ty = torch.empty((m, n), dtype=torch.float32, device="cuda")
    rc = dev.lib.htp_b200_mul_mat(ty.data_ptr(), tx.data_ptr(), tw.data_ptr(), m, k, n, IQ4,
                                  1 if x.dtype == np.float16 else 0, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert dev.lib.htp_b200_stream_status(torch.cuda.current_stream().cuda_stream) == 0
    return ty.cpu().numpy()


def test_iq4_nl_block_sums_bit_exact(dev, oracle, wl):
    import torch
    wq, _ = wl.random_case(40, IQ4, False, 1, 1024, 96)
    nb = wq.size // 18
    tw = torch.from_numpy(wq).cuda()
    s = torch.empty(nb, dtype=torch.int32, device="cuda")
    t = torch.empty(nb, dtype=torch.int32, device="cuda")
    assert dev.lib.htp_b200_block_sums(tw.data_ptr(), s.data_ptr(), t.data_ptr(), nb, IQ4, None) == 0
    torch.cuda.synchronize()
    so, to = oracle.block_sums(wq, IQ4)
    assert (s.cpu().numpy() == so).all() and (t.cpu().numpy() == to).all()


@pytest.mark.parametrize("act_f16", [False, True])
@pytest.mark.parametrize("m,k,n", [(1, 256, 32), (1, 4096, 4096), (2, 2048, 480), (3, 1024, 224), (7, 512, 96),
                                   (1, 14336, 1024), (2, 96, 64)])
def test_iq4_nl_decode_matches_oracle(dev, oracle, wl, act_f16, m, k, n):
    """One and two tokens per launch on the integer tensor-core path, more tokens in slices of two,
    K % 256 != 0 through the shape-agnostic kernel."""
    wq, x = wl.random_case(41, IQ4, act_f16, m, k, n)
    _check(dev, oracle, _raw(dev, x, wq, n), x, wq, n, 1e-3 if act_f16 else 1e-5)


@pytest.mark.parametrize("m,k,n", [(128, 512, 256), (300, 1024, 1312), (64, 256, 32)])
def test_iq4_nl_prefill_gemm_matches_oracle(dev, oracle, wl, m, k, n):
    wq, x = wl.random_case(42, IQ4, True, m, k, n)
    _check(dev, oracle, _raw(dev, x, wq, n), x, wq, n, 1e-3)


def test_iq4_nl_through_the_op_registry(dev, oracle, wl):
    """Op index 4 of the reference's registry (include/op_reg.h:10), fp32 activations."""
    pkg = dev.pkg
    wq, x = wl.random_case(43, IQ4, False, 1, 2048, 512)
    fw, fx, fy = dev.put(wq), dev.put(x), dev.buf(512 * 4)
    rc = dev.execute(pkg.HTP_OPS_MAT_MUL_PERMUTED_W4D16A32_IQ4_NL, (fy, 0), (fx, 0), (fw, 0), 1, 2048, 512)
    assert rc == 0
    _check(dev, oracle, dev.get(fy, (1, 512)), x, wq, 512, 1e-5)
    dev.free(fw, fx, fy)
