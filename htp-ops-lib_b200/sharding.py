"""Row sharding of a large weight matrix over the GPUs of one box, and assembly of the logits.

Every output column y[:, j] depends on weight row j only, so W[N][K] is cut into contiguous row
ranges, one per rank (each a contiguous byte range of the block array), the activations are
replicated, and the only exchange is an all-gather of the fp32 outputs.  One process per GPU;
the collective is torch.distributed's (NCCL over NVLink on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

ROW_ALIGN = 32  # the matmul contract: n % 32 == 0 for every shard


def shard_rows(n: int, world: int) -> int:
    """Rows per rank: N / world rounded up to a multiple of 32 (the last ranks may hold fewer)."""
    per = -(-n // world)
    return -(-per // ROW_ALIGN) * ROW_ALIGN


def row_range(n: int, rank: int, world: int) -> tuple[int, int]:
    """Half-open row range [r0, r1) of `rank`; empty for ranks past the end of a small matrix."""
    if n % ROW_ALIGN:
        raise ValueError("n must be a multiple of 32")
    per = shard_rows(n, world)
    r0 = min(n, rank * per)
    return r0, min(n, r0 + per)


def all_gather_logits(dist, logits, y_local, m: int, n: int, world: int) -> None:
    """Assembles logits[m][n] on every rank from the per-rank slabs y_local[m][rows of the rank].

    M = 1 with equal shards gathers in place (the slabs are contiguous in the output vector).
    Otherwise each rank's slab is a strided column band of the row-major output, so the slabs are
    gathered as [world][m][per] and copied into place.
    """
    import torch

    per = shard_rows(n, world)
    equal = per * world == n
    if m == 1 and equal:
        flat_out, flat_in = logits.view(-1), y_local.reshape(-1)
        if dist.get_backend() == "gloo":
            dist.all_gather(list(flat_out.split(per)), flat_in)
        else:
            dist.all_gather_into_tensor(flat_out, flat_in)
        return
    mine = y_local
    if y_local.shape[1] != per:  # ragged last shard: pad to the common width
        mine = torch.zeros((m, per), dtype=y_local.dtype, device=y_local.device)
        mine[:, :y_local.shape[1]] = y_local
    tmp = torch.empty((world, m, per), dtype=logits.dtype, device=logits.device)
    if dist.get_backend() == "gloo":
        dist.all_gather(list(tmp.unbind(0)), mine.contiguous())
    else:
        dist.all_gather_into_tensor(tmp, mine.contiguous())
    if equal:
        # one strided copy [world][m][per] -> [m][world][per] (the row-major output seen per rank band)
        logits.view(m, world, per).copy_(tmp.permute(1, 0, 2))
        return
    for r in range(world):
        r0, r1 = row_range(n, r, world)
        if r1 > r0:
            logits[:, r0:r1] = tmp[r, :, :r1 - r0]
