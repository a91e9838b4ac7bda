"""Generates tests/golden/golden_tiled.json: seeded cases in the tile-order weight formats (fp16 tiles
of the W16A32 op, permuted Q4_0 / Q8_0 / IQ4_NL super-blocks) - hashes of the packed buffers and
samples of the fp64 oracle's outputs.

    python tests/golden/make_golden_tiled.py      # seconds

Like golden.json these pin THIS repository's packer and oracle against drift; they are not reference
outputs (the reference holds no vectors for these formats)."""
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

CASES = {  # name -> (seed, weight_type code, fp16 activations, m, k, n)
    "w16_tiled_m1_k1024_n1024": (70, wl.WT_F16_TILED, False, 1, 1024, 1024),
    "permuted_q4_0_m2_k1024_n256": (71, wl.WT_PERMUTED | wl.TYPE_Q4_0, False, 2, 1024, 256),
    "permuted_q8_0_m2_k1024_n256": (72, wl.WT_PERMUTED | wl.TYPE_Q8_0, False, 2, 1024, 256),
    "permuted_iq4_nl_m3_k512_n128": (73, wl.WT_PERMUTED | wl.TYPE_IQ4_NL, True, 3, 512, 128),
}


def make_case(name: str):
    seed, fmt, a16, m, k, n = CASES[name]
    wq, x = wl.tiled_random_case(seed, fmt, a16, m, k, n)
    return fmt, n, wq, x


def entry_of(name: str) -> dict:
    fmt, n, wq, x = make_case(name)
    y = oracle.tiled_mul_mat_f64(x, wq, n, fmt)
    return {"w_sha256": wl.sha256(wq), "x_sha256": wl.sha256(x), "head": y[:, :16].tolist(), "tail": y[:, -16:].tolist(),
            "sum": float(y.sum()), "abs_sum": float(np.abs(y).sum())}


if __name__ == "__main__":
    out = {name: entry_of(name) for name in CASES}
    (Path(__file__).parent / "golden_tiled.json").write_text(json.dumps(out, indent=1))
    print("wrote", len(out), "cases")
