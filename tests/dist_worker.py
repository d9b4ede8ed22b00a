"""One rank of the CPU multi-process test of the row-sharded LM head (gloo).

Every rank cuts its shard out of the same seeded weight bytes by byte range, computes its
rows with the CPU oracle (the GPU kernel's stand-in here: this test is about the shard and
gather logic), all-gathers, and rank 0 compares with the unsharded oracle result."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import oracle  # noqa: E402
from brotensor_b200 import shard, synth  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    cpu = oracle.cpu()
    bad = 0
    for fmt, N, K, align in ((synth.Q6_K, 96, 512, 16), (synth.Q4_K, 70, 256, 1), (synth.Q8_0, 33, 64, 16)):
        W = synth.make_blocks(fmt, N, K, seed=7)            # same bytes on every rank
        x = synth.make_activations(1, K, seed=8)
        b, e = shard.row_range(N, world, rank, align)
        bb, be = shard.byte_range(fmt, N, K, world, rank, align)
        Wb = W.reshape(-1)
        assert be - bb == (e - b) * synth.packed_bytes(fmt, 1, K)
        local = cpu.matmul(fmt, np.ascontiguousarray(Wb[bb:be]), x, threads=1) if e > b else np.zeros((1, 0), np.float32)
        full = shard.all_gather_rows(torch.from_numpy(np.ascontiguousarray(local)), N, world, rank, align=align)
        ref = cpu.matmul(fmt, W, x, threads=1).reshape(-1)
        if not np.array_equal(full.numpy(), ref):
            bad += 1
    t = torch.tensor([bad])
    dist.all_reduce(t)
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("DIST_OK" if t.item() == 0 else f"DIST_FAIL {t.item()}")
    sys.exit(0 if t.item() == 0 else 1)


if __name__ == "__main__":
    main()
