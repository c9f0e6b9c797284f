"""Link load of the fused GEMM + all-gather, measured on two GPUs.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port P \
        -m onebitsparsemul_b200.scatter_bench <slab rows> <n> <k> [peers]

Each of the two ranks multiplies the same (slab rows x k) one-bit weights by the same (k x n) tokens
with ``onebit_matmul_packed_scatter`` and sends the result to `peers` (default 7) separate buffers in the
OTHER rank's memory: per GPU that is the NVLink traffic, out and in, of one rank of a (peers + 1)-GPU
row-sharded GEMM whose full result every GPU keeps. Prints the time with one destination (the GEMM
alone), with the extra destinations in local memory (the epilogue's instruction cost) and with them
on the peer, and checks every received copy against the local result.
"""
from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist


def main(argv):
    if len(argv) < 4:
        print(__doc__)
        return 2
    import torch.distributed._symmetric_memory as symm

    import onebitsparsemul_b200 as ob
    m, n, k = int(argv[1]), int(argv[2]), int(argv[3])
    peers = int(argv[4]) if len(argv) > 4 else 7
    rank = int(os.environ["RANK"])
    if int(os.environ["WORLD_SIZE"]) != 2:
        raise SystemExit("run with exactly two ranks")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    w = torch.zeros((m, k // 4, 4), dtype=torch.float16, device=dev)
    w[..., 0], w[..., 2] = 1.0, -1.0
    pw = ob.pack_weight(w.reshape(m, k), apply_mask=False, keep_reference=False)
    del w
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    B = torch.randint(-4, 5, (k, n), device=dev, generator=g).to(torch.float16)
    out = torch.empty((m, n), dtype=torch.float16, device=dev)
    recv = symm.empty((peers, m, n), dtype=torch.float16, device=dev)
    handle = symm.rendezvous(recv, dist.group.WORLD)
    peer_base = int(handle.buffer_ptrs[1 - rank])
    local = torch.empty((peers, m, n), dtype=torch.float16, device=dev)
    slab_bytes = m * n * 2
    flag = torch.zeros(1, device=dev)

    def timed(extra, iters=5):
        for _ in range(2):
            ob.matmul_scatter(pw, B, out, extra)
        dist.all_reduce(flag)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            ob.matmul_scatter(pw, B, out, extra)
        e1.record()
        torch.cuda.synchronize()
        dist.all_reduce(flag)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    t = [timed([]), timed([local.data_ptr() + i * slab_bytes for i in range(peers)]),
         timed([peer_base + i * slab_bytes for i in range(peers)])]
    exact = all(bool((recv[i] == out).all()) and bool((local[i] == out).all()) for i in range(peers))
    tt = torch.tensor(t, device=dev)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    if rank == 0:
        gb = peers * slab_bytes / 1e9
        print(f"{m} x {n} x {k}: 1 destination {tt[0]:.3f} ms | +{peers} local {tt[1]:.3f} ms | +{peers} on the peer {tt[2]:.3f} ms "
              f"({gb:.2f} GB each way, {gb / (float(tt[2]) * 1e-3):.0f} GB/s if it were not overlapped) | received copies exact: {exact}",
              flush=True)
    dist.destroy_process_group()
    return 0 if exact else 1


if __name__ == "__main__":
    sys.exit(main(sys.argv))
