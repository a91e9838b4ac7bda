"""The fused decode exchange across TWO GPUs of one process (skipped with fewer): each device holds
half of the weight rows, multiplies, stores its band into BOTH devices' logits with the kernel's
16-byte peer stores, raises its flag on both, and waits for the other's - one call per device and
step (htp_b200_mul_mat_gather_step).  Both copies of the logits must meet the oracle gate and equal
the single-device result bit for bit."""
from __future__ import annotations

import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _two_gpus() -> bool:
    import torch
    return torch.cuda.is_available() and torch.cuda.device_count() >= 2 and torch.cuda.can_device_access_peer(0, 1) \
        and torch.cuda.can_device_access_peer(1, 0)


@pytest.mark.parametrize("wtype,act_f16,m", [(8, True, 1), (2, False, 1), (2, False, 8)])
def test_gather_step_across_two_devices(lib, oracle, wl, wtype, act_f16, m):
    import torch
    if not _two_gpus():
        pytest.skip("needs two GPUs with peer access")
    k, n, world = 4096, 2048, 2
    n_loc = n // world
    wq, x = wl.random_case(1700 + m, wtype, act_f16, m, k, n)
    row_bytes = (k // 32) * wl.BLOCK_BYTES[wtype]
    devs = [torch.device("cuda", r) for r in range(world)]
    logits = [torch.full((m, n), float("nan"), dtype=torch.float32, device=d) for d in devs]
    flags = [torch.zeros(32, dtype=torch.int32, device=d) for d in devs]
    # a copy between the devices makes torch enable peer access in both directions
    logits[0][:, :1].copy_(logits[1][:, :1])
    logits[1][:, :1].copy_(logits[0][:, :1])
    tw = [torch.from_numpy(wq[r * n_loc * row_bytes:(r + 1) * n_loc * row_bytes].copy()).to(devs[r])
          for r in range(world)]
    tx = [torch.from_numpy(x).to(d) for d in devs]
    for d in devs:
        torch.cuda.synchronize(d)
    single = None
    for epoch in (1, 2):
        for r in range(world):
            torch.cuda.set_device(r)
            order = [r] + [q for q in range(world) if q != r]  # own copy first
            dsts = (ctypes.c_void_p * world)(*[logits[q].data_ptr() for q in order])
            fl = (ctypes.c_void_p * world)(*[flags[q].data_ptr() + 4 * r for q in order])
            st = torch.cuda.current_stream(devs[r]).cuda_stream
            assert lib.htp_b200_mul_mat_gather_step(dsts, world, n, r * n_loc, tx[r].data_ptr(), tw[r].data_ptr(), m, k,
                                                    n_loc, wtype, 1 if act_f16 else 0, fl, flags[r].data_ptr(), epoch,
                                                    st) == 0
        for r in range(world):
            torch.cuda.set_device(r)
            torch.cuda.synchronize(devs[r])
            assert lib.htp_b200_stream_status(torch.cuda.current_stream(devs[r]).cuda_stream) == 0
            assert flags[r][:world].tolist() == [epoch] * world
    torch.cuda.set_device(0)
    ty = torch.empty((m, n), dtype=torch.float32, device=devs[0])
    twf = torch.from_numpy(wq).to(devs[0])
    st = torch.cuda.current_stream(devs[0]).cuda_stream
    assert lib.htp_b200_mul_mat(ty.data_ptr(), tx[0].data_ptr(), twf.data_ptr(), m, k, n, wtype, 1 if act_f16 else 0,
                                st) == 0
    torch.cuda.synchronize(devs[0])
    single = ty.cpu().numpy()
    ref, absdot = oracle.mul_mat_f64(x, wq, n, wtype, want_absdot=True)
    tol = 1e-3 if act_f16 else 1e-5
    for r in range(world):
        got = logits[r].cpu().numpy()
        e = oracle.error_metrics(got, ref, absdot)
        assert e["max_rel_to_max"] <= tol and e["max_cond_rel"] <= tol, e
        # whole tiles per CTA on both sides of the comparison (few tiles): the same sums, bit for bit
        assert (got == single).all()
