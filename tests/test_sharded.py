"""Row sharding across ranks.

CPU part (gloo, world_size 2): the partition arithmetic, per-slab packing against slicing a global
pack, and the gather plumbing of ShardedBinaryLinear with the oracle standing in for the GEMM.
GPU part: the real kernels on however many GPUs are visible, compared bit for bit with the single-GPU
result (row sharding does not change any reduction order).
"""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from onebitsparsemul_b200.sharded import ShardedBinaryLinear, row_partition
from tests import helpers

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_row_partition():
    assert row_partition(8192, 8) == [(i * 1024, 1024) for i in range(8)]
    assert row_partition(25600, 8) == [(i * 3200, 3200) for i in range(4)] + [(12800 + i * 3200, 3200) for i in range(4)] \
        or sum(r for _, r in row_partition(25600, 8)) == 25600
    parts = row_partition(28672, 8)
    assert sum(r for _, r in parts) == 28672 and all(r % 256 == 0 for _, r in parts)
    assert [s for s, _ in parts] == list(np.cumsum([0] + [r for _, r in parts[:-1]]))
    assert max(r for _, r in parts) - min(r for _, r in parts) <= 256
    assert row_partition(768, 2) == [(0, 512), (512, 256)]
    with pytest.raises(ValueError):
        row_partition(1000, 2)
    with pytest.raises(ValueError):
        row_partition(256, 2)


def test_slab_pack_equals_rows_of_the_canonical_pack():
    rng = np.random.default_rng(4)
    dense, _ = helpers.make_weights(rng, 768, 128)
    canon, signs, _ = oracle.compress(dense)
    for start, rows in row_partition(768, 2):
        c2, s2, _ = oracle.compress(dense[start:start + rows])
        assert (c2 == canon[start:start + rows]).all() and (s2 == signs[start:start + rows]).all()
        # ... but the reference-ordered slab is NOT a slice of the global pack: pack per slab
        assert oracle.pack_bits(s2).shape == (64, rows // 8)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _cpu_worker(rank, world, port, mode, q, shared_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(9)
        m, k, n = 768, 128, 8
        dense, scale = helpers.make_weights(rng, m, k)
        B = helpers.make_tokens(rng, k, n, "int")

        def pack(w, s):                                     # oracle stands in for the pack kernel
            canon, signs, _ = oracle.compress(w.numpy())
            return (oracle.pack_bits(signs), oracle.meta_reorder(canon, 0), None if s is None else s.numpy(), w.shape[0])

        def matmul(pw, Bt, out, row0, rows):                # ... and for the GEMM kernels
            bits, meta, sc, mm = pw
            c32, _ = oracle.gemm(bits, meta, 0, Bt.numpy(), mm, scale=sc)
            out.copy_(torch.from_numpy(c32[row0:row0 + rows]))

        def scatter(pw, Bt, mine, extra):                  # the several-destination GEMM: peers' rows by address
            import ctypes
            bits, meta, sc, mm = pw
            c32, _ = oracle.gemm(bits, meta, 0, Bt.numpy(), mm, scale=sc)
            mine.copy_(torch.from_numpy(c32))
            src = mine.contiguous()
            for addr in extra:
                ctypes.memmove(addr, src.data_ptr(), src.numel() * src.element_size())

        def peer_buffer(layer, nn, dev):                    # every rank's C in a file all ranks map
            shape = (layer.m, nn)
            paths = [os.path.join(shared_dir, f"c_{r}_{nn}.bin") for r in range(world)]
            full = torch.from_file(paths[rank], shared=True, size=shape[0] * shape[1], dtype=torch.float16).view(shape)
            dist.barrier()
            views = [full if r == rank else torch.from_file(paths[r], shared=True, size=shape[0] * shape[1],
                                                            dtype=torch.float16).view(shape) for r in range(world)]
            return full, [v.data_ptr() for v in views], (None, views)

        layer = ShardedBinaryLinear(m, k, matmul=matmul, pack=pack, scatter=scatter, peer_buffer=peer_buffer)
        layer.pack_full(torch.from_numpy(dense), torch.from_numpy(scale))
        canon, signs, _ = oracle.compress(dense)
        want, _ = oracle.gemm(oracle.pack_bits(signs), oracle.meta_reorder(canon, 0), 0, B, m, scale=scale)
        if mode == "fused":
            ok = True
            for _ in range(2):                              # twice: the cached buffer is reused
                got = layer.forward(torch.from_numpy(B), gather=mode, out_dtype=torch.float16).numpy()
                ok &= bool((got == want.astype(np.float16)).all())
            q.put((rank, ok, got.shape))
            return
        got = layer.forward(torch.from_numpy(B), gather=mode, out_dtype=torch.float32).numpy()
        if mode == "none":
            want = want[layer.start:layer.start + layer.rows]
        q.put((rank, bool((got == want).all()), got.shape))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["none", "all", "fused"])
def test_sharded_host_logic_two_cpu_ranks(mode, tmp_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_cpu_worker, args=(r, 2, port, mode, q, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in results), results
    shapes = {r: s for r, _, s in results}
    if mode == "none":
        assert shapes == {0: (512, 8), 1: (256, 8)}
    else:
        assert shapes == {0: (768, 8), 1: (768, 8)}


def _gpu_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import onebitsparsemul_b200 as ob
        rng = np.random.default_rng(10)
        m, k = 2048, 1024
        dense, scale = helpers.make_weights(rng, m, k)
        w, sc = torch.from_numpy(dense).cuda(), torch.from_numpy(scale).cuda()
        single = ob.pack_weight(w, scale=sc)
        layer = ShardedBinaryLinear(m, k).pack_full(w, sc)
        ok = []                                           # the (n, mode) cases that differ
        for n in (8, 512):
            # integer tokens: every kernel variant gives the exact result, whatever its summation order
            B = torch.from_numpy(helpers.make_tokens(rng, k, n, "int")).cuda()
            want = ob.matmul_packed(single, B, out_dtype=torch.float16)
            slab = layer.forward(B, gather="none")
            if not bool((slab == want[layer.start:layer.start + layer.rows]).all()):
                ok.append((n, "none"))
            for mode in ("all", "fused", "fused"):   # twice: the cached peer-mapped buffer is reused
                if not bool((layer.forward(B, gather=mode) == want).all()):
                    ok.append((n, mode))
            # tokens and result in pinned host memory: 1/world of B uploaded per rank, all-gathered, C slab back
            Bh = B.cpu().pin_memory()
            for _ in range(2):                       # twice: the cached device buffers and the copy stream are reused
                Ch = layer.forward_host(Bh)
                torch.cuda.synchronize()
                if not bool((Ch == want[layer.start:layer.start + layer.rows].cpu()).all()):
                    ok.append((n, "host"))
        ok = (ok == [], ok, layer.fused_backend)
        torch.cuda.synchronize()
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
def test_sharded_gemm_on_visible_gpus_matches_single_gpu():
    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        # one GPU: the sharded layer must degenerate to the plain path
        import onebitsparsemul_b200 as ob
        rng = np.random.default_rng(10)
        dense, scale = helpers.make_weights(rng, 512, 256)
        w = torch.from_numpy(dense).cuda()
        layer = ShardedBinaryLinear(512, 256).pack_full(w)
        B = torch.from_numpy(helpers.make_tokens(rng, 256, 32)).cuda()
        want = ob.matmul_packed(ob.pack_weight(w), B, out_dtype=torch.float16)
        for mode in ("none", "all", "fused"):
            assert (layer.forward(B, gather=mode) == want).all()
        Ch = layer.forward_host(B.cpu().pin_memory())
        torch.cuda.synchronize()
        assert (Ch == want.cpu()).all()
        return
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gpu_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok[0] for _, ok in results), results
