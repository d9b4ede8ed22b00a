"""Row sharding of a quantized weight matrix over the ranks of one node.

Output rows are independent, so rank r owns the contiguous rows [begin, end) and, because
the GGUF layout is row-major blocks, the contiguous byte range [begin, end) * row_bytes of
the tensor: a shard is a byte-range upload, no re-quantisation, content bit-identical.
The activation vector is replicated; the only exchange is the all-gather of the FP32
results (brotensor has no sharded form; its P2P bring-up is src/cuda/register.cu:90-103).

These helpers are host logic only and run on any torch.distributed backend; the CPU tests
drive them with gloo ranks.
"""
from __future__ import annotations

from . import synth


def row_range(n_rows: int, world: int, rank: int, align: int = 1):
    """Rows [begin, end) of rank `rank`: an even split in units of `align` rows, the
    remainder units going to the lowest ranks; the last shard takes the ragged tail."""
    if not (0 <= rank < world) or n_rows < 0 or align < 1:
        raise ValueError("row_range: bad arguments")
    units = (n_rows + align - 1) // align
    base, rem = divmod(units, world)
    b = (rank * base + min(rank, rem)) * align
    e = ((rank + 1) * base + min(rank + 1, rem)) * align
    return min(b, n_rows), min(e, n_rows)


def byte_range(fmt: int, n_rows: int, K: int, world: int, rank: int, align: int = 1):
    b, e = row_range(n_rows, world, rank, align)
    rb = synth.packed_bytes(fmt, 1, K)
    return b * rb, e * rb


def all_gather_rows(local, n_rows: int, world: int, rank: int, group=None, align: int = 1):
    """Gathers per-rank result vectors (length = that rank's row count) into the full
    vector of n_rows entries, in row order. Equal shards use one all_gather_into_tensor;
    ragged ones are padded to the largest shard."""
    import torch
    import torch.distributed as dist
    if world == 1:
        return local.reshape(-1)[:n_rows]
    sizes = [row_range(n_rows, world, r, align) for r in range(world)]
    lens = [e - b for b, e in sizes]
    flat = local.reshape(-1)
    assert flat.numel() == lens[rank], "local result does not match this rank's shard"
    mx = max(lens)
    if min(lens) == mx:
        full = torch.empty(world * mx, dtype=flat.dtype, device=flat.device)
        dist.all_gather_into_tensor(full, flat.contiguous(), group=group)
        return full
    pad = torch.zeros(mx, dtype=flat.dtype, device=flat.device)
    pad[:lens[rank]] = flat
    full = torch.empty(world * mx, dtype=flat.dtype, device=flat.device)
    dist.all_gather_into_tensor(full, pad, group=group)
    return torch.cat([full[r * mx:r * mx + lens[r]] for r in range(world)])
