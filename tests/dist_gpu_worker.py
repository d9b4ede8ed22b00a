"""One rank (one GPU) of the multi-GPU test of the fused row-sharded LM head.

Compares, bitwise, the full result vector every rank holds after ShardedHead.run with the
NCCL all-gather of the plain per-shard GEMV results, over several calls including calls
issued back to back without a host synchronisation in between; and the candidate (top-k) form
against the sorted gathered logits."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from brotensor_b200 import hostapi, ops, shard, synth  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("cpu:gloo,cuda:nccl", device_id=torch.device("cuda", local))
    hostapi.init()
    bad = 0
    for fmt, N, K in ((synth.Q6_K, 16 * 40 * world, 2048), (synth.Q4_K, 16 * 7 * world, 512)):
        W = synth.make_blocks(fmt, N, K, seed=3)              # same bytes on every rank
        b, e = shard.row_range(N, world, rank, align=16)
        bb, be = shard.byte_range(fmt, N, K, world, rank, align=16)
        Wsh = np.ascontiguousarray(W.reshape(-1)[bb:be])
        w = hostapi.Weight(fmt, Wsh, e - b, K, local)

        def exchange(h):
            out = [None] * world
            dist.all_gather_object(out, h)
            return out

        head = hostapi.ShardedHead(w, b, N, rank, world, exchange)
        Wd = torch.from_numpy(Wsh).cuda()
        xs = [torch.from_numpy(synth.make_activations(1, K, seed=20 + i)).cuda() for i in range(6)]
        torch.cuda.synchronize()
        dist.barrier()
        # one call at a time
        for i in range(3):
            head.run(xs[i].data_ptr(), K, 0)
            got = head.logits()
            local_y = ops.gemv(fmt, Wd, xs[i], e - b).reshape(-1)
            ref = shard.all_gather_rows(local_y, N, world, rank, align=16).cpu().numpy()
            if not np.array_equal(got, ref):
                bad += 1
        # three calls back to back: the ranks drift apart and the alternating vectors must hold
        for i in range(3, 6):
            head.run(xs[i].data_ptr(), K, 0)
        got = head.logits()
        local_y = ops.gemv(fmt, Wd, xs[5], e - b).reshape(-1)
        ref = shard.all_gather_rows(local_y, N, world, rank, align=16).cpu().numpy()
        if not np.array_equal(got, ref):
            bad += 1
        # candidate form, mixed with the full form on the same exchange memory: every rank must end up
        # with the k best rows of the WHOLE matrix (largest first, equal values: lower row first)
        for k in (1, 5, 8):
            head.run_topk(xs[k % 6].data_ptr(), K, k, 0)
            vals, rows = head.top(k)
            local_y = ops.gemv(fmt, Wd, xs[k % 6], e - b).reshape(-1)
            full = shard.all_gather_rows(local_y, N, world, rank, align=16).cpu().numpy()
            order = np.lexsort((np.arange(N), -full))[:k]
            if not (np.array_equal(rows, order.astype(np.int32)) and np.array_equal(vals, full[order])):
                bad += 1
            head.run(xs[0].data_ptr(), K, 0)  # and a full forward after it still delivers every row
            if not np.array_equal(head.logits(), shard.all_gather_rows(ops.gemv(fmt, Wd, xs[0], e - b).reshape(-1), N, world, rank, align=16).cpu().numpy()):
                bad += 1
        if ops.device_status() != 0:
            bad += 1
        torch.cuda.synchronize()
        dist.barrier()       # nobody unmaps while a peer may still be storing
        head.close()
    t = torch.tensor([bad], device="cuda")
    dist.all_reduce(t)
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("HEAD_OK" if t.item() == 0 else f"HEAD_FAIL {t.item()}")
    sys.exit(0 if t.item() == 0 else 1)


if __name__ == "__main__":
    main()
