"""Synthetic workloads of the quantised MUL_MAT path and the host-side weight packer.

The five configurations are the benchmark's own (seeded, synthetic - no dataset, checkpoint or
tokenizer is involved; configs 3 and 4 borrow only the matrix SHAPES of an 8B-parameter decoder).
`quantize_q4_0` / `quantize_q8_0` are the packer a host integration would run once per weight
matrix: fp32 rows -> standard ggml blocks (include/quants.h).  The packing rule is the workload's:
  Q4_0: d = (signed value of max |w|) / -8 as fp16, q = clamp(round(w / d) + 8, 0, 15)
  Q8_0: d = max |w| / 127 as fp16,                  q = round(w / d)
with the division by the fp16-rounded d, round-half-away-from-zero, q = 8 / 0 for a zero block,
and Q8_0 q clamped to [-128, 127].
"""
from __future__ import annotations

import dataclasses
import hashlib

import numpy as np

TYPE_Q4_0 = 2
TYPE_Q8_0 = 8
TYPE_IQ4_NL = 20
BLOCK_BYTES = {TYPE_Q4_0: 18, TYPE_Q8_0: 34, TYPE_IQ4_NL: 18}
IQ4_NL_VALUES = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], dtype=np.float32)


def _round_half_away(x: np.ndarray) -> np.ndarray:
    r = np.trunc(x)
    frac = x - r  # exact in floating point
    return r + np.where(np.abs(frac) >= 0.5, np.sign(x), 0.0).astype(x.dtype)


def quantize_q4_0(w: np.ndarray) -> np.ndarray:
    """fp32 [N][K] -> uint8 [N * K/32 * 18]."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = w.shape
    assert k % 32 == 0
    blk = w.reshape(n, k // 32, 32)
    idx = np.abs(blk).argmax(axis=2)  # first occurrence of the largest magnitude
    vmax = np.take_along_axis(blk, idx[..., None], axis=2)[..., 0]
    d16 = (vmax / np.float32(-8.0)).astype(np.float16)
    d = d16.astype(np.float32)
    safe = np.where(d == 0, np.float32(1), d)
    q = _round_half_away(blk / safe[..., None]).astype(np.int32) + 8
    q = np.where(d[..., None] == 0, 8, np.clip(q, 0, 15)).astype(np.uint8)
    out = np.empty((n, k // 32, 18), dtype=np.uint8)
    out[..., :2] = d16.view(np.uint8).reshape(n, k // 32, 2)
    out[..., 2:] = q[..., :16] | (q[..., 16:] << 4)
    return out.reshape(-1)


def quantize_q8_0(w: np.ndarray) -> np.ndarray:
    """fp32 [N][K] -> uint8 [N * K/32 * 34]."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = w.shape
    assert k % 32 == 0
    blk = w.reshape(n, k // 32, 32)
    amax = np.abs(blk).max(axis=2)
    d16 = (amax / np.float32(127.0)).astype(np.float16)
    d = d16.astype(np.float32)
    safe = np.where(d == 0, np.float32(1), d)
    q = _round_half_away(blk / safe[..., None]).astype(np.int32)
    q = np.where(d[..., None] == 0, 0, np.clip(q, -128, 127)).astype(np.int8)
    out = np.empty((n, k // 32, 34), dtype=np.uint8)
    out[..., :2] = d16.view(np.uint8).reshape(n, k // 32, 2)
    out[..., 2:] = q.view(np.uint8)
    return out.reshape(-1)


def quantize_iq4_nl(w: np.ndarray) -> np.ndarray:
    """fp32 [N][K] -> uint8 [N * K/32 * 18]: d = (signed value of max |w|) / -127 as fp16, every element
    takes the table entry nearest to w / d (first one on ties); the Q4_0 nibble order."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = w.shape
    assert k % 32 == 0
    blk = w.reshape(n, k // 32, 32)
    idx = np.abs(blk).argmax(axis=2)
    vmax = np.take_along_axis(blk, idx[..., None], axis=2)[..., 0]
    d16 = (vmax / np.float32(-127.0)).astype(np.float16)
    d = d16.astype(np.float32)
    safe = np.where(d == 0, np.float32(1), d)
    t = blk / safe[..., None]
    q = np.abs(t[..., None] - IQ4_NL_VALUES).argmin(axis=-1)
    q = np.where(d[..., None] == 0, 8, q).astype(np.uint8)
    out = np.empty((n, k // 32, 18), dtype=np.uint8)
    out[..., :2] = d16.view(np.uint8).reshape(n, k // 32, 2)
    out[..., 2:] = q[..., :16] | (q[..., 16:] << 4)
    return out.reshape(-1)


def quantize(w: np.ndarray, wtype: int, row_chunk: int = 4096) -> np.ndarray:
    """Packs in row chunks so that a 128256 x 4096 matrix does not need tens of GB of temporaries."""
    fn = {TYPE_Q4_0: quantize_q4_0, TYPE_Q8_0: quantize_q8_0, TYPE_IQ4_NL: quantize_iq4_nl}[wtype]
    n = w.shape[0]
    if n <= row_chunk:
        return fn(w)
    return np.concatenate([fn(w[i:i + row_chunk]) for i in range(0, n, row_chunk)])


def weight_bytes(wtype: int, k: int, n: int) -> int:
    if wtype in TILE_BYTES:
        return (n // 32) * (k // 32) * TILE_BYTES[wtype]
    return n * (k // 32) * BLOCK_BYTES[wtype]


# ----------------------------------------------------------------------------------------------
# Weights in the reference's 32 x 32 tile order (weight_type codes of include/htp_ops_b200.h).
# Tile (n/32, k/32) is tile number (n/32) * (K/32) + k/32; element (k, n) of a tile is halfword slot
# (k & ~1) * 32 + n * 2 + (k & 1) (reference src/host/test.c:303-313).

WT_F16_TILED = 1
WT_PERMUTED = 0x100
TILE_BYTES = {WT_F16_TILED: 2048, WT_PERMUTED | TYPE_Q4_0: 576, WT_PERMUTED | TYPE_Q8_0: 1088,
              WT_PERMUTED | TYPE_IQ4_NL: 576}


def _tile_slots(w_kn: np.ndarray) -> np.ndarray:
    """[K][N] -> [N/32][K/32][super-block 4][k-row pair 4][slot 64], slot = 2 * column + (k & 1)."""
    k, n = w_kn.shape
    assert k % 32 == 0 and n % 32 == 0
    a = w_kn.reshape(k // 32, 4, 4, 2, n // 32, 32)  # k-tile, super-block, row pair, parity, n-tile, column
    return np.ascontiguousarray(a.transpose(4, 0, 1, 2, 5, 3)).reshape(n // 32, k // 32, 4, 4, 64)


def pack_f16_tiles(w_kn: np.ndarray) -> np.ndarray:
    """fp16-representable weights W[K][N] -> the fp16 tile buffer of the W16A32 op (uint8 view)."""
    return _tile_slots(np.asarray(w_kn).astype(np.float16)).view(np.uint8).reshape(-1)


def quantize_permuted(w_kn: np.ndarray, wtype: int) -> np.ndarray:
    """fp32 W[K][N] -> the reference-private permuted super-blocks (my_block_q4_0 144 B / my_block_q8_0
    272 B, four per tile; wtype = TYPE_Q4_0, TYPE_Q8_0 or TYPE_IQ4_NL).  A scale group is 32 consecutive
    slots = 2 k-rows x 16 columns; each group is quantised by the same rule as a standard block, then the
    quants are laid out as the reference's expansion reads them (src/dsp/ops/mat_mul.c:373-405, 472-506)."""
    slots = _tile_slots(np.asarray(w_kn, dtype=np.float32))
    groups = slots.reshape(-1, 32)
    blocks = quantize(groups, wtype).reshape(groups.shape[0], BLOCK_BYTES[wtype])
    n_sb = groups.shape[0] // 8
    scales = blocks[:, :2].reshape(n_sb, 16)
    if wtype == TYPE_Q8_0:
        return np.concatenate([scales, blocks[:, 2:].reshape(n_sb, 256)], axis=1).reshape(-1)
    qs = blocks[:, 2:]
    q = np.concatenate([qs & 15, qs >> 4], axis=1).reshape(n_sb, 4, 64)  # [super-block][row pair][slot]
    out = np.empty((n_sb, 64, 2), dtype=np.uint8)
    out[:, :, 0] = q[:, 0] | (q[:, 2] << 4)
    out[:, :, 1] = q[:, 1] | (q[:, 3] << 4)
    return np.concatenate([scales, out.reshape(n_sb, 128)], axis=1).reshape(-1)


def tiled_random_case(seed: int, fmt: int, act_f16: bool, m: int, k: int, n: int, scale: float = 0.02):
    """Seeded case in a tile-order format: (weight buffer, activations [m][k])."""
    rng = _rng(seed, fmt, int(act_f16), m, k, n)
    w = rng.standard_normal((k, n), dtype=np.float32) * np.float32(scale)
    x = rng.standard_normal((m, k), dtype=np.float32)
    wq = pack_f16_tiles(w) if fmt == WT_F16_TILED else quantize_permuted(w, fmt & 0xFF)
    return wq, (x.astype(np.float16) if act_f16 else x)


@dataclasses.dataclass(frozen=True)
class MatMul:
    """One quantised matmul: y[m][n] = x[m][k] . W[n][k]^T."""
    name: str
    wtype: int
    act_f16: bool
    k: int
    n: int


@dataclasses.dataclass(frozen=True)
class Config:
    name: str
    seed: int
    ms: tuple[int, ...]  # token counts the config is run at
    ops: tuple[MatMul, ...]  # one entry for configs 0, 1, 2, 4; one decoder layer for config 3
    layers: int = 1
    sharded: bool = False


_LAYER = (("q", 4096, 4096), ("k", 4096, 1024), ("v", 4096, 1024), ("o", 4096, 4096), ("gate", 4096, 14336),
          ("up", 4096, 14336), ("down", 14336, 4096))

CONFIGS = {
    "cfg0": Config("cfg0", 0, (1,), (MatMul("gemv_q4_0", TYPE_Q4_0, False, 4096, 4096),)),
    "cfg1": Config("cfg1", 1, (1,), (MatMul("gemv_q8_0", TYPE_Q8_0, False, 4096, 11008),)),
    "cfg2": Config("cfg2", 2, (512,), (MatMul("prefill_q4_0", TYPE_Q4_0, True, 4096, 14336),)),
    "cfg3": Config("cfg3", 3, (1, 8), tuple(MatMul(nm, TYPE_Q4_0, False, k, n) for nm, k, n in _LAYER), layers=32),
    "cfg4": Config("cfg4", 4, (1, 256), (MatMul("lm_head_q8_0", TYPE_Q8_0, True, 4096, 128256),), sharded=True),
}


ROW_CHUNK = 8192  # rows per independently seeded chunk of a weight matrix


def _rng(*key: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(list(key)))


def make_weight(cfg: Config, op_idx: int = 0, layer: int = 0, rows: tuple[int, int] | None = None,
                quantizer=None) -> np.ndarray:
    """Packed weights of rows [rows[0], rows[1]) of matrix (layer, op_idx) of a configuration.

    W ~ N(0, 0.02^2) in fp32, drawn in chunks of ROW_CHUNK rows, chunk c of matrix (layer, op) from
    the PCG64 stream seeded with [cfg.seed, 0, layer, op, c]: any row range (a rank's shard) can be
    produced without drawing the rest.  `quantizer(w, wtype)` defaults to the numpy packer above.
    """
    op = cfg.ops[op_idx]
    r0, r1 = rows if rows is not None else (0, op.n)
    quantizer = quantizer or quantize
    row_bytes = (op.k // 32) * BLOCK_BYTES[op.wtype]
    parts = []
    for c in range(r0 // ROW_CHUNK, (r1 + ROW_CHUNK - 1) // ROW_CHUNK):
        c0, c1 = c * ROW_CHUNK, min(op.n, (c + 1) * ROW_CHUNK)
        w = _rng(cfg.seed, 0, layer, op_idx, c).standard_normal((c1 - c0, op.k), dtype=np.float32) * np.float32(0.02)
        q = quantizer(w, op.wtype)
        lo, hi = max(r0, c0) - c0, min(r1, c1) - c0
        parts.append(q[lo * row_bytes:hi * row_bytes])
    return np.concatenate(parts) if len(parts) != 1 else np.ascontiguousarray(parts[0])


def make_activation(cfg: Config, m: int, op_idx: int = 0, layer: int = 0) -> np.ndarray:
    """x[m][k] ~ N(0, 1) from the PCG64 stream [cfg.seed, 1, layer, op, m]; fp16-rounded where the
    configuration feeds fp16 activations."""
    op = cfg.ops[op_idx]
    x = _rng(cfg.seed, 1, layer, op_idx, m).standard_normal((m, op.k), dtype=np.float32)
    return x.astype(np.float16) if op.act_f16 else x


def random_case(seed: int, wtype: int, act_f16: bool, m: int, k: int, n: int, scale: float = 0.02):
    """A free-form seeded case for the small-shape tests: (packed weights, activations)."""
    rng = _rng(seed, wtype, int(act_f16), m, k, n)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(scale)
    x = rng.standard_normal((m, k), dtype=np.float32)
    return quantize(w, wtype), (x.astype(np.float16) if act_f16 else x)


def sha256(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def algorithmic_bytes(op: MatMul, m: int, n: int | None = None) -> int:
    """Weight bytes once + activations + outputs."""
    n = n if n is not None else op.n
    return weight_bytes(op.wtype, op.k, n) + m * op.k * (2 if op.act_f16 else 4) + m * n * 4


def flops(op: MatMul, m: int, n: int | None = None) -> int:
    return 2 * m * (n if n is not None else op.n) * op.k


# ------------------------------------------------------------------------------------------------
# torch packer: the same rule as the numpy packer, on whatever device the tensor lives on.  Used to
# produce benchmark-sized weights directly in device memory.

def quantize_torch(w, wtype: int):
    """float32 tensor [N][K] -> uint8 tensor [N * K/32 * block_bytes] on the same device."""
    import torch

    n, k = w.shape
    blk = w.reshape(n, k // 32, 32)

    def round_half_away(x):
        r = torch.trunc(x)
        frac = x - r
        return r + torch.where(frac.abs() >= 0.5, torch.sign(x), torch.zeros_like(x))

    if wtype == TYPE_Q4_0:
        idx = blk.abs().argmax(dim=2, keepdim=True)
        vmax = torch.gather(blk, 2, idx)[..., 0]
        d16 = (vmax / -8.0).to(torch.float16)
        d = d16.to(torch.float32)
        safe = torch.where(d == 0, torch.ones_like(d), d)
        q = round_half_away(blk / safe[..., None]).to(torch.int32) + 8
        q = torch.where(d[..., None] == 0, torch.full_like(q, 8), q.clamp(0, 15)).to(torch.uint8)
        out = torch.empty((n, k // 32, 18), dtype=torch.uint8, device=w.device)
        out[..., :2] = d16.view(torch.uint8).reshape(n, k // 32, 2)
        out[..., 2:] = q[..., :16] | (q[..., 16:] << 4)
    else:
        amax = blk.abs().amax(dim=2)
        d16 = (amax / 127.0).to(torch.float16)
        d = d16.to(torch.float32)
        safe = torch.where(d == 0, torch.ones_like(d), d)
        q = round_half_away(blk / safe[..., None]).to(torch.int32)
        q = torch.where(d[..., None] == 0, torch.zeros_like(q), q.clamp(-128, 127)).to(torch.int8)
        out = torch.empty((n, k // 32, 34), dtype=torch.uint8, device=w.device)
        out[..., :2] = d16.view(torch.uint8).reshape(n, k // 32, 2)
        out[..., 2:] = q.view(torch.uint8)
    return out.reshape(-1)


def make_weight_torch(cfg: Config, device, op_idx: int = 0, layer: int = 0, rows: tuple[int, int] | None = None):
    """Device-resident packed weights with the configuration's distribution (N(0, 0.02^2), seeded
    per 8192-row chunk by (cfg.seed, layer, op, chunk) through torch's generator - the same
    distribution as make_weight, not the same bytes)."""
    import torch

    op = cfg.ops[op_idx]
    r0, r1 = rows if rows is not None else (0, op.n)
    row_bytes = (op.k // 32) * BLOCK_BYTES[op.wtype]
    out = torch.empty((r1 - r0) * row_bytes, dtype=torch.uint8, device=device)
    gen = torch.Generator(device=device)
    pos = 0
    for c in range(r0 // ROW_CHUNK, (r1 + ROW_CHUNK - 1) // ROW_CHUNK):
        c0, c1 = c * ROW_CHUNK, min(op.n, (c + 1) * ROW_CHUNK)
        gen.manual_seed(((cfg.seed * 64 + layer) * 16 + op_idx) * 4096 + c)
        w = torch.randn((c1 - c0, op.k), generator=gen, device=device, dtype=torch.float32) * 0.02
        q = quantize_torch(w, op.wtype)
        lo, hi = max(r0, c0) - c0, min(r1, c1) - c0
        nbytes = (hi - lo) * row_bytes
        out[pos:pos + nbytes] = q[lo * row_bytes:hi * row_bytes]
        pos += nbytes
    return out
