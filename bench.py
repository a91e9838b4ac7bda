"""Benchmark of the quantised MUL_MAT path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Headline workload (every N): the lm_head configuration - Q8_0 weights 128256 x 4096, fp16
activations, M = 1 - the one configuration that is sharded by output rows over 1/2/4/8 GPUs with
an NCCL all-gather of the fp32 logits.  One step = one pass: every rank runs the decode mat-vec on
its row slab, then the slabs are gathered.  `value` = algorithmic bytes of the WHOLE matrix per
step / max-over-ranks device time (strong scaling), inputs resident in HBM; `e2e` = the same
through the message channel with host buffers (activation upload and logits download inside the
timed region).  The other configurations are measured briefly on one GPU and reported under
`configs` in the same JSON line (decode GB/s for configs 0, 1, 3; prefill TFLOP/s for configs 2
and 4 at M = 256).

Timing: CUDA events on the launching stream, >= 3 warm-up steps, max over ranks; decode weights are
rotated through enough distinct copies that every pass reads from HBM, not L2; SM clocks and
throttle reasons are sampled with nvidia-smi during the timed region.

`--impl reference` times the CPU restatement of the reference's dequantise-then-dot semantics
(oracle/, fp32, all host threads) on a bounded sample of the same workload: the reference's own
implementation is Hexagon HVX/HMX code and cannot be built for a host CPU.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

L2_BYTES = 126 * 1024 * 1024


def read_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "tflops": float(d["bf16_tflops"]),
                "tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


def read_traffic(key: str):
    """DRAM bytes per launch of the dominant kernel from the committed ncu summary, if any."""
    p = ROOT / "profiles" / "ncu_traffic.json"
    if p.exists():
        e = json.loads(p.read_text()).get(key)
        return e["bytes_per_launch"] if isinstance(e, dict) else e
    return None


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.rows, self.proc = gpu_index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.idx)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0.0, set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx = max(mx, float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                              ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------

def rows_of_rank(n: int, rank: int, world: int) -> tuple[int, int]:
    from htp_ops_lib_b200 import sharding
    return sharding.row_range(n, rank, world)


def seeded_weight_slab(torch, wl, cfg, dev, rows):
    """Rows [rows[0], rows[1]) of the configuration's SEEDED weight matrix, packed, in device memory:
    the fp32 values come from the same PCG64 streams as workloads.make_weight (drawn on the host, one
    8192-row chunk at a time), the packing runs on the device with the same rule as the numpy packer,
    so the bytes are the ones the committed fixtures were computed from."""
    import numpy as np
    op = cfg.ops[0]
    r0, r1 = rows
    row_bytes = (op.k // 32) * wl.BLOCK_BYTES[op.wtype]
    out = torch.empty((r1 - r0) * row_bytes, dtype=torch.uint8, device=dev)
    pos = 0
    for c in range(r0 // wl.ROW_CHUNK, (r1 + wl.ROW_CHUNK - 1) // wl.ROW_CHUNK):
        c0, c1 = c * wl.ROW_CHUNK, min(op.n, (c + 1) * wl.ROW_CHUNK)
        w = wl._rng(cfg.seed, 0, 0, 0, c).standard_normal((c1 - c0, op.k), dtype=np.float32) * np.float32(0.02)
        lo, hi = max(r0, c0) - c0, min(r1, c1) - c0
        q = wl.quantize_torch(torch.from_numpy(w[lo:hi]).to(dev), op.wtype)
        out[pos:pos + q.numel()] = q
        pos += q.numel()
    return out


def golden_fixture(name: str, key: str):
    p = ROOT / "tests" / "golden" / "golden.json"
    return json.loads(p.read_text())[name][key]["oracle"] if p.exists() else None


def matches_fixture(y, g, tol: float) -> bool:
    """Logits (numpy [m][n]) against the committed oracle samples: sampled token rows (head and tail
    columns) and the whole-matrix checksum, relative to the oracle's largest magnitude / absolute sum."""
    import numpy as np
    head, tail = np.array(g["head"]), np.array(g["tail"])
    ys = y[g["rows"]]
    return bool(np.isfinite(y).all()
                and np.abs(ys[:, :head.shape[1]] - head).max() <= tol * g["max_abs"]
                and np.abs(ys[:, -tail.shape[1]:] - tail).max() <= tol * g["max_abs"]
                and abs(float(y.astype(np.float64).sum()) - g["sum"]) <= tol * g["abs_sum"])


def time_region(torch, fn, steps: int, stream) -> float:
    """Milliseconds for `steps` calls of fn, CUDA events on `stream`, synchronised on both sides."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record(stream)
    for i in range(steps):
        fn(i)
    e1.record(stream)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def graph_time(torch, lib, launch, n_in_graph: int, replays: int):
    """Milliseconds per launch when `n_in_graph` launches (launch(i, stream_ptr), i = 0 ..) are captured
    into ONE CUDA graph and the graph is replayed `replays` times: the host cost of issuing each
    operator is paid at capture time, not per launch.  None when the capture fails."""
    side = torch.cuda.Stream()
    try:
        with torch.cuda.stream(side):
            for i in range(2):  # first use of the stream: scratch allocation, attribute set-up - not capturable
                launch(i, side.cuda_stream)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for i in range(n_in_graph):
                launch(i, side.cuda_stream)
        for _ in range(2):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        assert lib.htp_b200_stream_status(side.cuda_stream) == 0
        return e0.elapsed_time(e1) / (replays * n_in_graph)
    except Exception as e:  # noqa: BLE001 - reported as absent, the stream-launch number stands
        sys.stderr.write(f"graph capture failed: {type(e).__name__}: {e}\n")
        return None


def cpu_baseline(wl, cfg_name: str, m: int, seconds: float = 12.0, sample_rows: int = 8192):
    """The CPU restatement (fp32, threaded) timed on a bounded row sample of the workload."""
    import numpy as np
    oracle = entry.load_oracle()
    lib = None
    try:  # a build tuned to this machine, outside the repository
        tmp = Path(tempfile.mkdtemp(prefix="htp_oracle_native_"))
        lib = oracle.load(oracle.build(tmp, arch="native"))
        kind_note = "-O3 -march=native"
    except Exception:  # noqa: BLE001
        lib = oracle.load()
        kind_note = "-O3 -march=x86-64-v3 (prebuilt)"
    cfg = wl.CONFIGS[cfg_name]
    op = cfg.ops[-1] if cfg_name == "cfg3" else cfg.ops[0]
    rows = min(sample_rows, op.n)
    wq = wl.make_weight(cfg, 0 if cfg_name != "cfg3" else len(cfg.ops) - 1, rows=(0, rows),
                        quantizer=lambda w, t: oracle.quantize(w, t))
    x = wl.make_activation(cfg, m, 0 if cfg_name != "cfg3" else len(cfg.ops) - 1)
    cores = oracle.usable_cores()
    oracle.mul_mat_f32(x, wq, rows, op.wtype, lib=lib)  # warm-up
    t0, n = time.perf_counter(), 0
    while True:
        oracle.mul_mat_f32(x, wq, rows, op.wtype, lib=lib)
        n += 1
        dt = time.perf_counter() - t0
        if dt >= seconds or n >= 100000:
            break
    per = dt / n
    return {"seconds_per_sample": per, "rows": rows, "cores": cores, "op": op, "build": kind_note,
            "gbps": wl.algorithmic_bytes(op, m, rows) / per / 1e9, "tflops": wl.flops(op, m, rows) / per / 1e12,
            "iters": n}


# ------------------------------------------------------------------------------------------------

def workload_name(world: int) -> str:
    """config.workload of both arms."""
    return f"cfg4 lm_head Q8_0 128256x4096, fp16 activations, M=1, rows sharded over {world} GPU(s)"


def run_reference(args):
    """CPU arm: rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    entry.load_package()
    from htp_ops_lib_b200 import workloads as wl
    steps, warm = args.steps, args.warmup
    cfg_name, m = "cfg4", 1
    secs = max(2.0, min(60.0, 0.5 * (steps + warm)))
    b = cpu_baseline(wl, cfg_name, m, seconds=secs, sample_rows=16384)
    line = {
        "impl": "reference", "metric": "decode_GBps", "value": round(b["gbps"], 3), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": round(b["seconds_per_sample"] * 1e3, 4),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args.gpus),
                   "implementation": "CPU restatement of the reference's dequantise-then-dot (fp32, all host threads); "
                                     "the reference's own HVX/HMX code cannot be built for a host CPU",
                   "sample": f"first {b['rows']} of 128256 weight rows per step; GB/s does not depend on the row count"},
        "cpu_baseline": {"value": round(b["gbps"], 3), "unit": "GB/s", "cores": b["cores"], "kind": "port",
                         "sample": f"first {b['rows']} of 128256 weight rows per step, {b['iters']} steps, "
                                   f"{b['build']}"},
        "e2e": {"value": round(b["gbps"], 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def measure_single_gpu_configs(torch, pkg, lib, wl, peaks, stream_ptr, quick: bool):
    """Configs 0-3 and config 4 at M = 256 on this GPU: brief, device-resident, rotating copies."""
    out = {}
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream()

    def run_case(name, cfg, op_idx, m, steps):
        op = cfg.ops[op_idx]
        slab = wl.weight_bytes(op.wtype, op.k, op.n)
        copies = max(2, -(-L2_BYTES // slab) + 1) if m <= 8 else 1
        w0 = wl.make_weight_torch(cfg, dev, op_idx)
        ws = [w0] + [w0.clone() for _ in range(copies - 1)]
        x = torch.randn((m, op.k), device=dev, dtype=torch.float32)
        x = x.to(torch.float16) if op.act_f16 else x
        y = torch.empty((m, op.n), device=dev, dtype=torch.float32)
        act_t = pkg.ACT_F16 if op.act_f16 else pkg.ACT_F32

        def launch(i, sp_):
            rc = lib.htp_b200_mul_mat(y.data_ptr(), x.data_ptr(), ws[i % copies].data_ptr(), m, op.k, op.n, op.wtype,
                                      act_t, sp_)
            assert rc == 0

        def step(i):
            launch(i, stream_ptr)
        for i in range(3):
            step(i)
        ms = time_region(torch, step, steps, stream) / steps
        assert lib.htp_b200_stream_status(stream_ptr) == 0
        r = {"ms": round(ms, 5), "m": m, "k": op.k, "n": op.n, "weight_copies": copies}
        if m <= 8:
            gb = wl.algorithmic_bytes(op, m) / (ms * 1e-3) / 1e9
            r.update(GBps=round(gb, 1), frac_of_hbm_peak=round(gb / peaks["hbm_gbs"], 4))
            # a small mat-vec is bound by the HOST's launch rate (about 5 us per call from Python): the
            # same launches replayed from a CUDA graph show what the device does
            msg = graph_time(torch, lib, launch, max(copies, 8), max(5, steps // 4))
            if msg is not None:
                gbg = wl.algorithmic_bytes(op, m) / (msg * 1e-3) / 1e9
                r.update(ms_graph=round(msg, 5), GBps_graph=round(gbg, 1),
                         frac_of_hbm_peak_graph=round(gbg / peaks["hbm_gbs"], 4))
        else:
            tf = wl.flops(op, m) / (ms * 1e-3) / 1e12
            r.update(TFLOPs=round(tf, 2), frac_of_tensor_peak=round(tf / peaks["tflops"], 4))
        out[name] = r
        del ws, w0

    steps = 20 if quick else 100
    run_case("cfg0_q4_0_gemv_4096x4096_m1", wl.CONFIGS["cfg0"], 0, 1, steps)
    run_case("cfg1_q8_0_gemv_11008x4096_m1", wl.CONFIGS["cfg1"], 0, 1, steps)
    run_case("cfg2_q4_0_prefill_14336x4096_m512", wl.CONFIGS["cfg2"], 0, 512, max(20, steps // 2))
    run_case("cfg2_shape_q4_0_prefill_14336x4096_m128", wl.CONFIGS["cfg2"], 0, 128, max(20, steps // 2))
    run_case("cfg4_q8_0_lm_head_m256", wl.CONFIGS["cfg4"], 0, 256, max(10, steps // 4))
    out["rms_norm_f32_4096x32768"] = measure_rms_norm(torch, lib, peaks, stream_ptr, stream, max(5, steps // 5))
    out.update(measure_large_decode_and_iq4(torch, pkg, lib, wl, peaks, stream_ptr, stream, max(5, steps // 5)))
    out.update(measure_tile_order_decode(torch, pkg, lib, wl, peaks, stream_ptr, stream, max(5, steps // 5)))
    out.update(measure_decoder_stack(torch, pkg, lib, wl, peaks, quick))
    return out


def measure_large_decode_and_iq4(torch, pkg, lib, wl, peaks, stream_ptr, stream, steps):
    """Decode mat-vecs long enough (151 MB of 4-bit weights, two rotating copies) that launch and
    pipeline fill stop dominating - Q4_0 and IQ4_NL - and the IQ4_NL prefill GEMM on config 2's shape.
    Timing does not depend on the weight values: random block bytes with a small fp16 scale."""
    dev = torch.device("cuda", torch.cuda.current_device())
    out = {}

    def blocks(wtype, k, n):
        bb = wl.BLOCK_BYTES[wtype]
        w = torch.randint(0, 256, (n * (k // 32), bb), dtype=torch.uint8, device=dev)
        w[:, 0], w[:, 1] = 0, 0x20  # fp16 scale 2^-7
        return w.reshape(-1)

    for name, wtype, a16, m, k, n in (("q4_0_gemv_65536x4096_m1", wl.TYPE_Q4_0, False, 1, 4096, 65536),
                                      ("q4_0_gemv_65536x4096_m8", wl.TYPE_Q4_0, False, 8, 4096, 65536),
                                      ("q8_0_gemv_32768x4096_m8", wl.TYPE_Q8_0, False, 8, 4096, 32768),
                                      ("iq4_nl_gemv_65536x4096_m1", wl.TYPE_IQ4_NL, False, 1, 4096, 65536),
                                      ("iq4_nl_gemv_65536x4096_m8", wl.TYPE_IQ4_NL, False, 8, 4096, 65536),
                                      ("iq4_nl_prefill_14336x4096_m512", wl.TYPE_IQ4_NL, True, 512, 4096, 14336),
                                      ("q4_0_prefill_f32act_14336x4096_m512", wl.TYPE_Q4_0, False, 512, 4096, 14336),
                                      ("q4_0_prefill_f32act_14336x4096_m32", wl.TYPE_Q4_0, False, 32, 4096, 14336)):
        op = wl.MatMul(name, wtype, a16, k, n)
        copies = 2 if m <= 8 else 1
        ws = [blocks(wtype, k, n) for _ in range(copies)]
        x = torch.randn((m, k), device=dev, dtype=torch.float16 if a16 else torch.float32)
        y = torch.empty((m, n), device=dev, dtype=torch.float32)

        def launch(i, sp_):
            assert lib.htp_b200_mul_mat(y.data_ptr(), x.data_ptr(), ws[i % copies].data_ptr(), m, k, n, wtype,
                                        pkg.ACT_F16 if a16 else pkg.ACT_F32, sp_) == 0

        def step(i):
            launch(i, stream_ptr)
        for i in range(3):
            step(i)
        ms = time_region(torch, step, steps, stream) / steps
        assert lib.htp_b200_stream_status(stream_ptr) == 0
        r = {"ms": round(ms, 5), "m": m, "k": k, "n": n, "weight_copies": copies}
        if m <= 8:
            gb = wl.algorithmic_bytes(op, m) / (ms * 1e-3) / 1e9
            r.update(GBps=round(gb, 1), frac_of_hbm_peak=round(gb / peaks["hbm_gbs"], 4))
            msg = graph_time(torch, lib, launch, 8, max(5, steps // 2))
            if msg is not None:
                gbg = wl.algorithmic_bytes(op, m) / (msg * 1e-3) / 1e9
                r.update(ms_graph=round(msg, 5), GBps_graph=round(gbg, 1),
                         frac_of_hbm_peak_graph=round(gbg / peaks["hbm_gbs"], 4))
        else:
            tf = wl.flops(op, m) / (ms * 1e-3) / 1e12
            r.update(TFLOPs=round(tf, 2), frac_of_tensor_peak=round(tf / peaks["tflops"], 4))
        out[name] = r
        del ws
    return out


def tile_order_device_weights(torch, wl, fmt: int, k: int, n: int, dev):
    """A device-resident weight buffer in one of the tile-order formats.  Timing does not depend on the
    values: fp16 tiles hold N(0, 0.02^2), super-blocks hold random quant bytes under scales of 2^-7."""
    nbytes = wl.weight_bytes(fmt, k, n)
    if fmt == wl.WT_F16_TILED:
        return (torch.randn(nbytes // 2, device=dev, dtype=torch.float16) * 0.02).view(torch.uint8)
    sbb = wl.TILE_BYTES[fmt] // 4
    w = torch.randint(0, 256, (nbytes // sbb, sbb), dtype=torch.uint8, device=dev)
    w[:, 0:16:2], w[:, 1:16:2] = 0, 0x20
    return w.reshape(-1)


def measure_tile_order_decode(torch, pkg, lib, wl, peaks, stream_ptr, stream, steps):
    """One-token mat-vecs over weights in the reference's tile order, read in place: the fp16 tiles of the
    W16A32 op (32768 x 4096, 268 MB) and the permuted Q4_0 / Q8_0 super-blocks (65536 x 4096, 151 / 285 MB),
    two rotating copies each.  Algorithmic bytes = weight buffer + activation + output.  The 512-token
    lines are config 2's shape on the same formats (fp32 activations, as the reference's ops take them):
    conversion launch + tensor-core GEMM, flops = 2 m n k."""
    dev = torch.device("cuda", torch.cuda.current_device())
    out = {}
    for name, fmt, m, k, n in (("w16a32_tiled_gemv_32768x4096_m1", wl.WT_F16_TILED, 1, 4096, 32768),
                               ("w16a32_tiled_prefill_f32act_14336x4096_m512", wl.WT_F16_TILED, 512, 4096, 14336),
                               ("permuted_q4_0_gemv_65536x4096_m1", wl.WT_PERMUTED | wl.TYPE_Q4_0, 1, 4096, 65536),
                               ("permuted_q8_0_gemv_65536x4096_m1", wl.WT_PERMUTED | wl.TYPE_Q8_0, 1, 4096, 65536),
                               ("permuted_q4_0_prefill_f32act_14336x4096_m512", wl.WT_PERMUTED | wl.TYPE_Q4_0, 512, 4096, 14336),
                               ("permuted_q8_0_prefill_f32act_14336x4096_m512", wl.WT_PERMUTED | wl.TYPE_Q8_0, 512, 4096, 14336)):
        nbytes = wl.weight_bytes(fmt, k, n)
        assert nbytes == lib.htp_b200_weight_bytes(fmt, k, n)
        copies = 2 if m == 1 else 1
        ws = [tile_order_device_weights(torch, wl, fmt, k, n, dev) for _ in range(copies)]
        x = torch.randn((m, k), device=dev, dtype=torch.float32)
        y = torch.empty((m, n), device=dev, dtype=torch.float32)

        def step(i):
            assert lib.htp_b200_mul_mat(y.data_ptr(), x.data_ptr(), ws[i % copies].data_ptr(), m, k, n, fmt, pkg.ACT_F32,
                                        stream_ptr) == 0
        for i in range(3):
            step(i)
        ms = time_region(torch, step, steps, stream) / steps
        assert lib.htp_b200_stream_status(stream_ptr) == 0
        r = {"ms": round(ms, 5), "m": m, "k": k, "n": n, "weight_copies": copies}
        if m == 1:
            gb = (nbytes + 4 * k + 4 * n) / (ms * 1e-3) / 1e9
            r.update(GBps=round(gb, 1), frac_of_hbm_peak=round(gb / peaks["hbm_gbs"], 4))
        else:
            tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
            r.update(TFLOPs=round(tf, 2), frac_of_tensor_peak=round(tf / peaks["tflops"], 4))
        out[name] = r
        del ws
    return out


def measure_rms_norm(torch, lib, peaks, stream_ptr, stream, steps):
    """RMSNorm over 32768 rows of 4096 floats (512 MB read + 512 MB written per launch, far beyond L2):
    algorithmic bytes = 2 * 4 * ne0 * ne1."""
    ne0, ne1 = 4096, 32768
    dev = torch.device("cuda", torch.cuda.current_device())
    x = torch.randn((ne1, ne0), device=dev, dtype=torch.float32)
    y = torch.empty_like(x)

    def step(i):
        assert lib.htp_b200_rms_norm_f32(y.data_ptr(), x.data_ptr(), ne0, ne1, stream_ptr) == 0
    for i in range(3):
        step(i)
    ms = time_region(torch, step, steps, stream) / steps
    gb = 2.0 * 4 * ne0 * ne1 / (ms * 1e-3) / 1e9
    return {"ms": round(ms, 5), "ne0": ne0, "ne1": ne1, "GBps": round(gb, 1),
            "frac_of_hbm_peak": round(gb / peaks["hbm_gbs"], 4)}


def measure_decoder_stack(torch, pkg, lib, wl, peaks, quick: bool, layers: int = 32, ms_list=None):
    """Config 3: 32 layers x 7 Q4_0 matmuls issued in order through the message channel (one message
    of 224 requests per pass); 3.9 GB of weights per pass, so every pass streams from HBM."""
    cfg = wl.CONFIGS["cfg3"]
    dev = torch.device("cuda", torch.cuda.current_device())
    out = {}
    if lib.open_dsp_session(torch.cuda.current_device(), 1) != 0:
        return {"cfg3": {"error": "open_dsp_session failed"}}
    lib.init_htp_backend()
    try:
        # one distinct weight set per layer (generated once per matrix kind, then perturbed per layer
        # by copying: the bytes differ in address, which is what matters for HBM traffic)
        base = [wl.make_weight_torch(cfg, dev, i, 0) for i in range(len(cfg.ops))]
        weights = [[b if l == 0 else b.clone() for b in base] for l in range(layers)]
        wfd = [[lib.htp_buf_wrap(w.data_ptr(), w.numel()) for w in lw] for lw in weights]
        total_w = sum(w.numel() for lw in weights for w in lw)
        chan = pkg.MessageChannel(16384)
        try:
            for m in (ms_list or cfg.ms):
                # independent N(0,1) activations per matrix kind, one output buffer per (layer, matrix):
                # no request reads or overwrites what another one writes
                xs = [torch.randn((m, op.k), device=dev, dtype=torch.float32) for op in cfg.ops]
                ys = [[torch.empty((m, op.n), device=dev, dtype=torch.float32) for op in cfg.ops]
                      for _ in range(layers)]
                xfd = [lib.htp_buf_wrap(x.data_ptr(), x.numel() * 4) for x in xs]
                yfd = [lib.htp_buf_wrap(y.data_ptr(), y.numel() * 4) for ly in ys for y in ly]
                reqs = []
                for l in range(layers):
                    for i, op in enumerate(cfg.ops):
                        reqs.append(pkg.pack_matmul_request(pkg.HTP_OPS_MAT_MUL_PERMUTED_W4D16A32,
                                                            (yfd[l * len(cfg.ops) + i], 0), (xfd[i], 0),
                                                            (wfd[l][i], 0), m, op.k, op.n))
                launches0 = lib.htp_b200_launch_count()
                # the 224 requests are the same every pass: the message bytes are composed once (a C host
                # fills them in a few microseconds; Python's struct packing would cost ~0.1 ms per pass)
                msg, sizes = pkg.compose_message(reqs), [len(r) for r in reqs]
                for _ in range(2):
                    st = chan.submit_composed(msg, sizes)
                    assert all(s == 0 for s in st), st
                n_pass = 5 if quick else 20
                # device time of the same passes: events on the session stream around each message
                sstream = torch.cuda.ExternalStream(lib.htp_session_stream())
                ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_pass)]
                t0 = time.perf_counter()
                for i in range(n_pass):
                    ev[i][0].record(sstream)
                    chan.submit_composed(msg, sizes)
                    ev[i][1].record(sstream)
                ms = (time.perf_counter() - t0) / n_pass * 1e3
                torch.cuda.synchronize()
                ms_dev = statistics.median(a.elapsed_time(b) for a, b in ev)
                algo = total_w + layers * sum(m * op.k * 4 + m * op.n * 4 for op in cfg.ops)
                gb = algo / (ms * 1e-3) / 1e9
                out[f"cfg3_llama8b_stack_q4_0_m{m}"] = {
                    "ms_per_pass": round(ms, 4), "ops_per_pass": len(reqs), "GBps": round(gb, 1),
                    "frac_of_hbm_peak": round(gb / peaks["hbm_gbs"], 4),
                    "ms_per_pass_on_device": round(ms_dev, 4),
                    "frac_of_hbm_peak_on_device": round(algo / (ms_dev * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
                    "layers": layers,
                    "kernel_launches_per_pass": (lib.htp_b200_launch_count() - launches0) // (n_pass + 2),
                    "timed": "ms_per_pass: host wall clock around message-channel round trips (224 requests per "
                             "message, composed once); on_device: CUDA events on the session stream around a message"}
                for fd in xfd + yfd:
                    lib.htp_buf_free(fd)
        finally:
            chan.close()
    finally:
        lib.close_dsp_session()
    return out


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    pkg = entry.load_package()
    from htp_ops_lib_b200 import sharding
    from htp_ops_lib_b200 import workloads as wl
    lib = pkg.load()  # raises if the CUDA library is not built: there is no fallback

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; the library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
    peaks = read_peaks()
    steps, warm = args.steps, max(3, args.warmup)

    cfg = wl.CONFIGS["cfg4"]
    op, m = cfg.ops[0], 1
    r0, r1 = sharding.row_range(op.n, rank, world)
    n_loc = r1 - r0
    slab = wl.weight_bytes(op.wtype, op.k, n_loc)
    copies = max(2, -(-L2_BYTES // slab) + 1)
    w0 = seeded_weight_slab(torch, wl, cfg, dev, (r0, r1))
    ws = [w0] + [w0.clone() for _ in range(copies - 1)]
    x_host = torch.from_numpy(wl.make_activation(cfg, m)).pin_memory()  # the configuration's seeded tokens
    x = x_host.to(dev)
    logits = torch.empty((m, op.n), device=dev, dtype=torch.float32)  # every rank ends with all of it
    y_loc = logits[:, r0:r1] if world == 1 else torch.empty((m, n_loc), device=dev, dtype=torch.float32)
    stream = torch.cuda.current_stream()
    sp = stream.cuda_stream

    def kernel(i):
        rc = lib.htp_b200_mul_mat(y_loc.data_ptr(), x.data_ptr(), ws[i % copies].data_ptr(), m, op.k, n_loc,
                                  op.wtype, pkg.ACT_F16, sp)
        assert rc == 0

    def step_gather(i):
        kernel(i)
        if world > 1:
            sharding.all_gather_logits(dist, logits, y_loc, m, op.n, world)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Fused exchange (N > 1): the kernel's tile completion stores each rank's slice of the logits
    # straight into EVERY rank's logits vector (peer pointers from torch's symmetric memory); a
    # cross-rank barrier replaces the all-gather.  Used for the timed step when it is available and
    # reproduces the gathered result bit for bit on every rank; otherwise the NCCL all-gather is.
    step, exchange = step_gather, ("none" if world == 1 else "NCCL all-gather of fp32 logits")
    fused_logits = None  # this rank's copy of the logits the fused exchange assembles
    fused_e2e = None     # two sets of symmetric logits for the end-to-end loop
    if world > 1 and not args.no_fused:
        try:

            import torch.distributed._symmetric_memory as symm
            ranges = [sharding.row_range(op.n, r, world) for r in range(world)]
            if all(b - a == n_loc for a, b in ranges):
                sym = symm.empty((m, op.n), dtype=torch.float32, device=dev)
                hdl = symm.rendezvous(sym, dist.group.WORLD)
                symf = symm.empty((32,), dtype=torch.int32, device=dev)  # completion flags, one word per rank
                hdlf = symm.rendezvous(symf, dist.group.WORLD)
                order = [rank] + [r for r in range(world) if r != rank]  # own copy first
                arr = (ctypes.c_void_p * world)(*[int(hdl.buffer_ptrs[r]) for r in order])
                # a second set of logits for the end-to-end loop: a rank downloads step e from one set while
                # its peers' step e + 1 already stores into the other
                sym_b = symm.empty((m, op.n), dtype=torch.float32, device=dev)
                hdl_b = symm.rendezvous(sym_b, dist.group.WORLD)
                arr_b = (ctypes.c_void_p * world)(*[int(hdl_b.buffer_ptrs[r]) for r in order])
                fused_e2e = {"syms": (sym, sym_b), "arrs": (arr, arr_b)}
                # this rank's flag word in every destination GPU's flag array
                farr = (ctypes.c_void_p * world)(*[int(hdlf.buffer_ptrs[r]) + 4 * rank for r in order])
                epoch = [0]

                def step_fused(i):
                    # ONE call: the kernel stores this rank's slice into every rank's logits (16-byte peer
                    # stores) and raises its flag on every GPU; a small wait kernel behind it returns when
                    # all ranks' flags of this step are here - no all-gather, no separate barrier
                    epoch[0] += 1
                    assert lib.htp_b200_mul_mat_gather_step(arr, world, op.n, r0, x.data_ptr(),
                                                            ws[i % copies].data_ptr(), m, op.k, n_loc, op.wtype,
                                                            pkg.ACT_F16, farr, symf.data_ptr(), epoch[0], sp) == 0
                sym.zero_()
                symf.zero_()
                torch.cuda.synchronize()
                hdl.barrier()
                step_gather(0)
                step_fused(0)
                torch.cuda.synchronize()
                hdl.barrier()
                fused_logits = sym
                same = torch.tensor([1 if bool((sym == logits).all().item()) else 0], device=dev)
                dist.all_reduce(same, op=dist.ReduceOp.MIN)
                faster = False
                if int(same[0]) == 1:
                    # both paths give the same logits: take the faster one (agreed between the ranks)
                    for f in (step_fused, step_gather):
                        for i in range(3):
                            f(i)
                    barrier()
                    tt = torch.tensor([time_region(torch, step_fused, 50, stream),
                                       time_region(torch, step_gather, 50, stream)], device=dev, dtype=torch.float64)
                    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                    faster = float(tt[0]) < float(tt[1])
                    if rank == 0:
                        sys.stderr.write(f"exchange: fused {float(tt[0]) / 50 * 1e3:.1f} us per step, NCCL all-gather "
                                         f"{float(tt[1]) / 50 * 1e3:.1f} us per step\n")
                if faster:
                    step, exchange = step_fused, ("fused: tile completion stores into every rank's logits (16-byte peer "
                                      "stores), completion flags raised by the last CTA, bounded flag wait on every "
                                      "rank; one library call per step")
        except Exception as e:  # noqa: BLE001 - symmetric memory is optional plumbing
            sys.stderr.write(f"fused exchange unavailable: {type(e).__name__}: {e}\n")

    # Parity of what is about to be timed: the assembled logits of BOTH exchanges on every rank against
    # the committed oracle samples of config 4 (seeded weights and tokens), gate 1e-3 as for any fp16
    # activation result.
    g1 = golden_fixture("cfg4", "m1")
    parity = {"decode_m1": None}
    if g1 is not None:
        step_gather(0)
        torch.cuda.synchronize()
        ok = matches_fixture(logits.cpu().numpy(), g1, 1e-3)
        if fused_logits is not None:
            ok = ok and matches_fixture(fused_logits.cpu().numpy(), g1, 1e-3)
        t = torch.tensor([1 if ok else 0], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
        parity["decode_m1"] = bool(int(t[0]))
    for i in range(warm):
        step(i)
    barrier()
    l0 = lib.htp_b200_launch_count()
    with ClockSampler(local) as clk:
        # The first region is the reported one (EXACTLY `steps` steps).  It is then repeated so that
        # the whole lasts long enough (~0.5 s) for nvidia-smi to sample clocks under load; the number
        # of repeats is agreed between the ranks (max over ranks of the first region's time).
        barrier()
        first_ms = time_region(torch, step, steps, stream)
        first_launches = lib.htp_b200_launch_count() - l0
        t = torch.tensor([first_ms], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        reps = int(min(400, max(1, 500.0 / max(float(t[0]), 1e-3))))
        ms_total, k_total = first_ms, steps
        for _ in range(reps - 1):
            barrier()
            ms_total += time_region(torch, step, steps, stream)
            k_total += steps
    barrier()
    assert lib.htp_b200_stream_status(sp) == 0
    t = torch.tensor([first_ms, ms_total / k_total * steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t[0]) / steps  # EXACTLY `steps` steps, max over ranks
    ms_step_long = float(t[1]) / steps
    total_bytes = wl.algorithmic_bytes(op, m)
    value = total_bytes / (ms_step * 1e-3) / 1e9

    # the NCCL all-gather path beside the fused one, for comparison
    gather_ms = None
    if world > 1 and step is not step_gather:
        barrier()
        t = torch.tensor([time_region(torch, step_gather, steps, stream) / steps], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        gather_ms = float(t[0])

    # The dominant kernel's launch duration for the roofline.  One GPU: a step IS one launch of it, so
    # the timed region above is the measurement (CUDA events around exactly `steps` launches).  Sharded:
    # the kernel alone (no exchange) in a region of its own, max over ranks.
    if world == 1:
        k_ms = ms_step
    else:
        barrier()
        k_ms = time_region(torch, kernel, steps, stream) / steps
        t = torch.tensor([k_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        k_ms = float(t[0])
    k_bytes = wl.algorithmic_bytes(op, m, n_loc)
    achieved = k_bytes / (k_ms * 1e-3) / 1e9

    # ---- end to end through the message channel with host buffers
    e2e = None
    if lib.open_dsp_session(local, 1) == 0:
        lib.init_htp_backend()
        chan = pkg.MessageChannel(4096)
        try:
            fx = lib.htp_buf_alloc(x.numel() * 2)
            fw = [lib.htp_buf_wrap(w.data_ptr(), w.numel()) for w in ws]
            # One GPU: the operator writes the logits into a SHARED buffer - pinned host memory the device
            # addresses, the counterpart of the reference's rpcmem output buffer - so the device->host
            # transfer of the result is the kernel's own stores and the host reads them in place when the
            # message is done.  Sharded: the band goes to device memory, is gathered, then downloaded.
            shared_out = world == 1
            if shared_out:
                fy = lib.htp_buf_alloc_shared(m * op.n * 4)
                assert fy > 0
                out_host = torch.from_numpy(np.ctypeslib.as_array(
                    ctypes.cast(lib.htp_buf_ptr(fy), ctypes.POINTER(ctypes.c_float)), shape=(m, op.n)))
            else:
                fy = lib.htp_buf_wrap(y_loc.data_ptr(), m * n_loc * 4)
                out_host = torch.empty((m, op.n), dtype=torch.float32).pin_memory()
            reqs = [[pkg.pack_matmul_request(pkg.HTP_OPS_MAT_MUL_W8D16A16, (fy, 0), (fx, 0), (f, 0), m, op.k, n_loc)]
                    for f in fw]

            use_fused = world > 1 and step is not step_gather and fused_e2e is not None
            if use_fused:
                fl = [lib.htp_buf_wrap(t_.data_ptr(), m * op.n * 4) for t_ in fused_e2e["syms"]]
                ss = lib.htp_session_stream()
                xs = lib.htp_buf_ptr(fx)

            def e2e_step(i):
                # upload is only enqueued (pinned source): what follows is ordered behind it on the session stream
                assert lib.htp_buf_upload_async(fx, 0, x_host.data_ptr(), x_host.numel() * 2) == 0
                if use_fused:
                    # sharded, fused exchange: ONE library call whose kernel stores this rank's band into every
                    # rank's logits and ends when all bands are here; then the download of the full logits
                    epoch[0] += 1
                    assert lib.htp_b200_mul_mat_gather_step(fused_e2e["arrs"][i & 1], world, op.n, r0, xs,
                                                            ws[i % copies].data_ptr(), m, op.k, n_loc, op.wtype,
                                                            pkg.ACT_F16, farr, symf.data_ptr(), epoch[0], ss) == 0
                    assert lib.htp_buf_download_async(fl[i & 1], 0, out_host.data_ptr(), m * op.n * 4) == 0
                    assert lib.htp_session_synchronize() == 0
                    return
                st = chan.submit(reqs[i % copies])
                assert st == [0], st
                if not shared_out:
                    sharding.all_gather_logits(dist, logits, y_loc, m, op.n, world)
                    out_host.copy_(logits, non_blocking=True)
                    torch.cuda.current_stream().synchronize()
            for i in range(warm):
                e2e_step(i)
            e2e_steps = max(steps, 200)
            per_step = []
            barrier()
            t0 = time.perf_counter()
            for i in range(e2e_steps):
                t1 = time.perf_counter()
                e2e_step(i)
                per_step.append(time.perf_counter() - t1)
            barrier()
            dt = (time.perf_counter() - t0) / e2e_steps
            t = torch.tensor([dt, statistics.median(per_step)], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt, med = float(t[0]), float(t[1])
            # the check reads what ONE more step delivers into a cleared host buffer
            out_host.zero_()
            e2e_step(e2e_steps)
            e2e_ok = g1 is None or matches_fixture(out_host.numpy(), g1, 1e-3)
            direct_ms = None
            if shared_out:
                # beside it (one GPU): the same step without the message channel - upload, ONE direct library
                # call on the session stream into the shared output buffer, stream synchronise
                ss, xs, yo = lib.htp_session_stream(), lib.htp_buf_ptr(fx), lib.htp_buf_ptr(fy)

                def direct_step(i):
                    assert lib.htp_buf_upload_async(fx, 0, x_host.data_ptr(), x_host.numel() * 2) == 0
                    assert lib.htp_b200_mul_mat(yo, xs, ws[i % copies].data_ptr(), m, op.k, op.n, op.wtype, pkg.ACT_F16, ss) == 0
                    assert lib.htp_session_synchronize() == 0
                for i in range(warm):
                    direct_step(i)
                t0 = time.perf_counter()
                for i in range(e2e_steps):
                    direct_step(i)
                direct_ms = (time.perf_counter() - t0) / e2e_steps * 1e3
                out_host.zero_()
                direct_step(0)
                e2e_ok = e2e_ok and (g1 is None or matches_fixture(out_host.numpy(), g1, 1e-3))
            e2e = {"value": round(total_bytes / dt / 1e9, 2), "unit": "GB/s", "ms_per_step": round(dt * 1e3, 4),
                   "ms_per_step_median": round(med * 1e3, 4), "steps": e2e_steps,
                   "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": m * op.n * 4,
                   "downloaded_logits_match_fixture": bool(e2e_ok),
                   "ms_per_step_direct_call": None if direct_ms is None else round(direct_ms, 4),
                   "path": "htp_buf_upload_async (pinned host memory) -> " + (
                       "htp_b200_mul_mat_gather_step on the session stream (the kernel stores this rank's band into "
                       "every rank's logits, raises its flags and ends when all bands are here; two sets of logits "
                       "used in turn) -> htp_buf_download_async of the full fp32 logits -> htp_session_synchronize; "
                       if use_fused else
                       "message channel (1 request) -> NCCL all-gather -> download of the fp32 logits; " if world > 1 else
                       "message channel (1 request) -> the kernel stores the fp32 logits into a shared (pinned, "
                       "device-addressable) output buffer, read in place when the message is done; ")
                   + "weights stay resident, as the reference's mapped weight buffers do"}
        finally:
            chan.close()
            lib.close_dsp_session()

    line = None
    if rank == 0:
        clocks = clk.summary()
        line = {
            "metric": "decode_GBps", "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": steps,
            "warmup": warm, "ms_per_step": round(ms_step, 5), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16 x int8 -> f32", "data": "synthetic",
            "config": {"workload": workload_name(world), "exchange": exchange,
                       "l2": f"rotating {copies} distinct weight copies per rank "
                             f"({slab * copies / 1e6:.0f} MB > 126 MB L2): every pass reads HBM",
                       "algorithmic_bytes_per_step": total_bytes,
                       "ms_per_step_over_long_run": round(ms_step_long, 5),
                       **({"ms_per_step_with_nccl_all_gather": round(gather_ms, 5)} if gather_ms else {})},
            "roofline": {"bound": "hbm", "kernel": "gemv_mma_kernel<Q8_0,f16,M=1>", "achieved": round(achieved, 1),
                         "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4),
                         # the same kernel inside the long (~0.5 s) step loop, clocks under the power cap
                         "frac_sustained": (round(total_bytes / (ms_step_long * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
                                            if world == 1 else None),
                         "peak_source": f"{peaks['source']} (copy bandwidth)", "ms_per_launch": round(k_ms, 5),
                         "algorithmic_bytes_per_launch": k_bytes,
                         # the committed capture is of the whole matrix on one GPU; a rank's launch covers its
                         # share of the rows, and the kernel's DRAM traffic is proportional to rows
                         "traffic": (None if read_traffic("cfg4_m1_q8_0") is None
                                     else int(read_traffic("cfg4_m1_q8_0") * k_bytes / total_bytes))},
            "e2e": e2e, "gpu_launches": int(first_launches), "clocks": clocks,
            "parity_ok": parity["decode_m1"],
            "parity": "assembled logits of every rank (NCCL all-gather and fused exchange) against the committed "
                      "fp64-oracle samples of config 4, gate 1e-3",
        }
    # the sharded prefill case of config 4 (M = 256): each rank multiplies its row shard on the tensor
    # cores, then the [256][N / R] slabs are gathered into [256][N] on every rank
    if world > 1:
        m2, steps2 = 256, max(5, min(20, steps))
        x2 = torch.from_numpy(wl.make_activation(cfg, m2)).to(dev)  # the configuration's seeded tokens
        y2 = torch.empty((m2, n_loc), device=dev, dtype=torch.float32)
        logits2 = torch.empty((m2, op.n), device=dev, dtype=torch.float32)

        def kernel2(i):
            assert lib.htp_b200_mul_mat(y2.data_ptr(), x2.data_ptr(), ws[i % copies].data_ptr(), m2, op.k, n_loc,
                                        op.wtype, pkg.ACT_F16, sp) == 0

        def step2(i):
            kernel2(i)
            sharding.all_gather_logits(dist, logits2, y2, m2, op.n, world)
        for i in range(3):
            step2(i)
        barrier()
        t = torch.tensor([time_region(torch, step2, steps2, stream) / steps2,
                          time_region(torch, kernel2, steps2, stream) / steps2], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert lib.htp_b200_stream_status(sp) == 0
        # Fused exchange: the GEMM's epilogue stores each rank's column band straight into EVERY rank's
        # logits buffer (peer pointers from torch's symmetric memory); a cross-rank barrier replaces the
        # all-gather and the copy.  Checked against the gathered result above.
        fused = None
        try:

            import torch.distributed._symmetric_memory as symm
            r0_all = [sharding.row_range(op.n, r, world) for r in range(world)]
            equal = all(b - a == n_loc for a, b in r0_all)
            if equal:
                sym = symm.empty((m2, op.n), dtype=torch.float32, device=dev)
                hdl = symm.rendezvous(sym, dist.group.WORLD)
                ptrs = [int(pp) for pp in hdl.buffer_ptrs]
                order = [rank] + [r for r in range(world) if r != rank]  # own copy first
                arr = (ctypes.c_void_p * world)(*[ptrs[r] for r in order])
                col0 = r0_all[rank][0]

                def step3(i):
                    assert lib.htp_b200_mul_mat_multi_dst(arr, world, op.n, col0, x2.data_ptr(),
                                                          ws[i % copies].data_ptr(), m2, op.k, n_loc, op.wtype,
                                                          pkg.ACT_F16, sp) == 0
                    hdl.barrier()
                sym.zero_()
                hdl.barrier()
                step3(0)
                torch.cuda.synchronize()
                same = bool((sym == logits2).all().item())
                g256 = golden_fixture("cfg4", "m256")
                if g256 is not None:
                    okp = matches_fixture(logits2.cpu().numpy(), g256, 1e-3) and matches_fixture(sym.cpu().numpy(), g256,
                                                                                                 1e-3)
                    tp = torch.tensor([1 if okp else 0], device=dev)
                    dist.all_reduce(tp, op=dist.ReduceOp.MIN)
                    parity["prefill_m256"] = bool(int(tp[0]))
                for i in range(3):
                    step3(i)
                barrier()
                t3 = torch.tensor([time_region(torch, step3, steps2, stream) / steps2], device=dev,
                                  dtype=torch.float64)
                dist.all_reduce(t3, op=dist.ReduceOp.MAX)
                ok_all = torch.tensor([1 if same else 0], device=dev)
                dist.all_reduce(ok_all, op=dist.ReduceOp.MIN)
                assert lib.htp_b200_stream_status(sp) == 0
                fused = {"ms_per_step": round(float(t3[0]), 5),
                         "TFLOPs": round(wl.flops(op, m2) / (float(t3[0]) * 1e-3) / 1e12, 2),
                         "equals_gathered_result": bool(int(ok_all[0])),
                         "exchange": "epilogue TMA stores into every rank's logits (peer memory) + barrier"}
            else:
                fused = {"skipped": "row shards of unequal size"}
        except Exception as e:  # noqa: BLE001 - symmetric memory is optional plumbing
            fused = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
        if rank == 0:
            fl = wl.flops(op, m2)
            line["prefill_m256"] = {
                "ms_per_step": round(float(t[0]), 5), "TFLOPs": round(fl / (float(t[0]) * 1e-3) / 1e12, 2),
                "kernel_ms_per_launch": round(float(t[1]), 5),
                "kernel_TFLOPs_per_gpu": round(wl.flops(op, m2, n_loc) / (float(t[1]) * 1e-3) / 1e12, 2),
                "frac_of_tensor_peak_per_gpu": round(wl.flops(op, m2, n_loc) / (float(t[1]) * 1e-3) / 1e12
                                                     / peaks["tflops"], 4),
                "gathered_bytes_per_step": m2 * op.n * 4, "fused_exchange": fused,
                "parity_ok": parity.get("prefill_m256"),
                "note": "whole-job TFLOP/s = 2*256*128256*4096 / max-over-ranks time of GEMM + all-gather"}
        del x2, y2, logits2
    # single-GPU extras and the CPU baseline: rank 0 at N = 1 only
    if world == 1:
        del ws, w0
        torch.cuda.empty_cache()
        if not args.no_extras:
            line["configs"] = measure_single_gpu_configs(torch, pkg, lib, wl, peaks, sp, args.quick)
        if not args.no_cpu:
            b = cpu_baseline(wl, "cfg4", 1, seconds=12.0, sample_rows=16384)
            line["cpu_baseline"] = {"value": round(b["gbps"], 3), "unit": "GB/s", "cores": b["cores"], "kind": "port",
                                    "sample": f"first {b['rows']} of 128256 weight rows, {b['iters']} repeats over "
                                              f"{b['seconds_per_sample'] * b['iters']:.1f} s, fp32, {b['build']}"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_case(args):
    """One matmul shape, device-resident, rotating weight copies: the small case the ncu captures
    use (`--case q8_0,f16,1,4096,32768`; weight kinds q4_0, q8_0, and the tile-order ones w16_tiled, pq4_0, pq8_0,
    piq4_nl)."""
    import torch

    pkg = entry.load_package()
    from htp_ops_lib_b200 import workloads as wl
    lib = pkg.load()
    wt_s, act_s, m, k, n = args.case.split(",")
    m, k, n = int(m), int(k), int(n)
    wtype = {"q4_0": wl.TYPE_Q4_0, "q8_0": wl.TYPE_Q8_0, "w16_tiled": wl.WT_F16_TILED,
             "pq4_0": wl.WT_PERMUTED | wl.TYPE_Q4_0, "pq8_0": wl.WT_PERMUTED | wl.TYPE_Q8_0,
             "piq4_nl": wl.WT_PERMUTED | wl.TYPE_IQ4_NL}[wt_s]
    a16 = act_s == "f16"
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    cfg = wl.Config("case", 99, (m,), (wl.MatMul("case", wtype, a16, k, n),))
    op = cfg.ops[0]
    slab = wl.weight_bytes(wtype, k, n)
    copies = max(2, -(-L2_BYTES // slab) + 1) if m <= 8 else 1
    w0 = tile_order_device_weights(torch, wl, wtype, k, n, dev) if wtype in wl.TILE_BYTES else wl.make_weight_torch(cfg, dev)
    ws = [w0] + [w0.clone() for _ in range(copies - 1)]
    x = torch.randn((m, k), device=dev, dtype=torch.float32)
    x = x.to(torch.float16) if a16 else x
    y = torch.empty((m, n), device=dev, dtype=torch.float32)
    stream = torch.cuda.current_stream()

    def step(i):
        assert lib.htp_b200_mul_mat(y.data_ptr(), x.data_ptr(), ws[i % copies].data_ptr(), m, k, n, wtype,
                                    pkg.ACT_F16 if a16 else pkg.ACT_F32, stream.cuda_stream) == 0
    for i in range(args.warmup):
        step(i)
    ms = time_region(torch, step, args.steps, stream) / args.steps
    assert lib.htp_b200_stream_status(stream.cuda_stream) == 0
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(args.steps):
        step(i)
    enqueue_us = (time.perf_counter() - t0) / args.steps * 1e6  # host time to issue one op
    torch.cuda.synchronize()

    def launch(i, sp_):
        assert lib.htp_b200_mul_mat(y.data_ptr(), x.data_ptr(), ws[i % copies].data_ptr(), m, k, n, wtype,
                                    pkg.ACT_F16 if a16 else pkg.ACT_F32, sp_) == 0
    ms_graph = graph_time(torch, lib, launch, max(copies, 8), max(3, args.steps // 4)) if args.graph else None
    peaks = read_peaks()
    r = {"case": args.case, "ms": round(ms, 5), "host_enqueue_us": round(enqueue_us, 2), "weight_copies": copies,
         "GBps": round(wl.algorithmic_bytes(op, m) / (ms * 1e-3) / 1e9, 1),
         "TFLOPs": round(wl.flops(op, m) / (ms * 1e-3) / 1e12, 2)}
    r["frac_hbm"] = round(r["GBps"] / peaks["hbm_gbs"], 4)
    r["frac_tensor"] = round(r["TFLOPs"] / peaks["tflops"], 4)
    if ms_graph is not None:
        r["ms_graph"] = round(ms_graph, 5)
        r["frac_hbm_graph"] = round(wl.algorithmic_bytes(op, m) / (ms_graph * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
    print(json.dumps(r), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the brief single-GPU runs of the other configs")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--quick", action="store_true", help="fewer repeats in the extra runs")
    ap.add_argument("--no-fused", action="store_true",
                    help="N > 1: assemble the logits with an NCCL all-gather instead of the kernel's own peer stores")
    ap.add_argument("--case", default=None, help="wtype,act,m,k,n: time one shape only (profiling aid)")
    ap.add_argument("--graph", action="store_true", help="--case: also time the launches replayed from a CUDA graph")
    ap.add_argument("--stack", default=None, help="m[,layers]: time config 3's decoder stack only, through the message "
                                                  "channel, with that many tokens and layers (profiling aid)")
    args = ap.parse_args()
    if args.stack:
        import torch
        pkg = entry.load_package()
        from htp_ops_lib_b200 import workloads as wl
        parts = [int(v) for v in args.stack.split(",")]
        torch.cuda.set_device(0)
        print(json.dumps(measure_decoder_stack(torch, pkg, pkg.load(), wl, read_peaks(), True,
                                               layers=parts[1] if len(parts) > 1 else 32, ms_list=[parts[0]])), flush=True)
    elif args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
