"""Generates tests/golden/golden.json: hashes of the seeded inputs of the five configurations and
samples of the fp64 oracle's outputs on them.

    python tests/golden/make_golden.py            # a few minutes, ~6 GB of host memory

The reference holds no golden vectors for this path (its tests never issue a quantised matmul),
so these fixtures pin THIS repository's generator, packer and oracle against drift; they are not
reference outputs.  Inputs come from htp-ops-lib_b200/workloads.py (packed with the oracle's C
quantiser, which the CPU tests prove bit-identical to the numpy packer).
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

entry.load_package()
from htp_ops_lib_b200 import workloads as wl  # noqa: E402

oracle = entry.load_oracle()
CQ = lambda w, t: oracle.quantize(w, t)  # noqa: E731

SAMPLE_ROWS = 32  # first and last output columns kept per matrix


def sample(y: np.ndarray) -> dict:
    """First/last SAMPLE_ROWS outputs of (up to eight) token rows plus whole-matrix checksums."""
    m = y.shape[0]
    rows = list(range(m)) if m <= 8 else [0, 1, 2, 3, m - 4, m - 3, m - 2, m - 1]
    return {
        "rows": rows,
        "head": y[rows, :SAMPLE_ROWS].tolist(),
        "tail": y[rows, -SAMPLE_ROWS:].tolist(),
        "sum": float(y.sum()),
        "abs_sum": float(np.abs(y).sum()),
        "max_abs": float(np.abs(y).max()),
    }


def main():
    out = {}
    for name in ("cfg0", "cfg1", "cfg2"):
        cfg = wl.CONFIGS[name]
        op, m = cfg.ops[0], cfg.ms[0]
        wq = wl.make_weight(cfg, quantizer=CQ)
        x = wl.make_activation(cfg, m)
        y = oracle.mul_mat_f64(x, wq, op.n, op.wtype)
        s, t = oracle.block_sums(wq, op.wtype)
        out[name] = {"w_sha256": wl.sha256(wq), "x_sha256": wl.sha256(x), "m": m, "oracle": sample(y),
                     "block_sum_s_sha256": wl.sha256(s), "block_sum_t_sha256": wl.sha256(t)}
        print(name, "done", flush=True)
    # config 3: hashes of every matrix of layers 0 and 31, oracle samples for layer 0 at M = 1 and 8
    cfg = wl.CONFIGS["cfg3"]
    c3 = {"layers": {}, "oracle_layer0": {}}
    for layer in (0, 31):
        c3["layers"][str(layer)] = {}
        for i, op in enumerate(cfg.ops):
            wq = wl.make_weight(cfg, i, layer, quantizer=CQ)
            c3["layers"][str(layer)][op.name] = wl.sha256(wq)
            if layer == 0:
                for m in cfg.ms:
                    x = wl.make_activation(cfg, m, i, layer)
                    y = oracle.mul_mat_f64(x, wq, op.n, op.wtype)
                    c3["oracle_layer0"][f"{op.name}_m{m}"] = {"x_sha256": wl.sha256(x), "oracle": sample(y)}
        print("cfg3 layer", layer, "done", flush=True)
    out["cfg3"] = c3
    # config 4: weight hash per 8192-row chunk (so a shard can check its own rows), oracle samples
    cfg = wl.CONFIGS["cfg4"]
    op = cfg.ops[0]
    chunks = []
    parts = []
    for c0 in range(0, op.n, wl.ROW_CHUNK):
        part = wl.make_weight(cfg, rows=(c0, min(op.n, c0 + wl.ROW_CHUNK)), quantizer=CQ)
        chunks.append(wl.sha256(part))
        parts.append(part)
    wq = np.concatenate(parts)
    del parts
    c4 = {"w_chunk_sha256": chunks, "w_sha256": wl.sha256(wq)}
    for m in cfg.ms:
        x = wl.make_activation(cfg, m)
        y = oracle.mul_mat_f64(x, wq, op.n, op.wtype)
        c4[f"m{m}"] = {"x_sha256": wl.sha256(x), "oracle": sample(y)}
        print("cfg4 m", m, "done", flush=True)
    out["cfg4"] = c4
    path = Path(__file__).with_name("golden.json")
    path.write_text(json.dumps(out))
    print("wrote", path, path.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
