"""The multi-GPU path on CPU: two gloo ranks shard the weight rows, each computes its slab (here
with the oracle standing in for the kernel), the logits are assembled with the library's
all-gather helper, and every rank must hold the single-process result."""
from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, m: int, n: int, k: int, out_dir: str):
    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as entry
    entry.load_package()
    from htp_ops_lib_b200 import sharding
    from htp_ops_lib_b200 import workloads as wl
    oracle = entry.load_oracle()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        wq, x = wl.random_case(77, 8, True, m, k, n)
        r0, r1 = sharding.row_range(n, rank, world)
        row_bytes = (k // 32) * 34
        slab = wq[r0 * row_bytes:r1 * row_bytes]
        y_loc = torch.from_numpy(oracle.mul_mat_f64(x, slab, r1 - r0, 8).astype(np.float32)) if r1 > r0 else \
            torch.empty((m, 0), dtype=torch.float32)
        logits = torch.full((m, n), float("nan"), dtype=torch.float32)
        sharding.all_gather_logits(dist, logits, y_loc, m, n, world)
        np.save(os.path.join(out_dir, f"rank{rank}.npy"), logits.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("m,n", [(1, 128), (4, 128), (1, 96), (3, 160)])
def test_two_rank_row_sharding(tmp_path, m, n):
    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as entry
    entry.load_package()
    from htp_ops_lib_b200 import workloads as wl
    oracle = entry.load_oracle()
    k, world = 256, 2
    mp.spawn(_worker, args=(world, _free_port(), m, n, k, str(tmp_path)), nprocs=world, join=True)
    wq, x = wl.random_case(77, 8, True, m, k, n)
    ref = oracle.mul_mat_f64(x, wq, n, 8).astype(np.float32)
    for r in range(world):
        got = np.load(tmp_path / f"rank{r}.npy")
        assert (got == ref).all()


def test_row_ranges_cover_and_align():
    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as entry
    entry.load_package()
    from htp_ops_lib_b200 import sharding
    for n in (32, 96, 4096, 128256, 14336):
        for world in (1, 2, 3, 4, 8):
            pos = 0
            for r in range(world):
                r0, r1 = sharding.row_range(n, r, world)
                assert r0 == pos and r0 % 32 == 0 and (r1 - r0) % 32 == 0
                pos = r1
            assert pos == n
    assert [sharding.row_range(128256, r, 8) for r in (0, 7)] == [(0, 16032), (112224, 128256)]
    with pytest.raises(ValueError):
        sharding.row_range(100, 0, 2)
