"""The on-disk format of packed weights (packed_file.py).

CPU part: header and payload round trip, damage detection, one file per row slab on two `gloo` ranks where
every rank reads only its own. GPU part: save -> load -> the GEMM gives identical bits.
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
from onebitsparsemul_b200 import packed_file
from tests import helpers

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _tile_operands(seed, m, k):
    rng = np.random.default_rng(seed)
    dense, scale = helpers.make_weights(rng, m, k)
    canon, signs, _ = oracle.compress(dense)
    bt, mt = helpers.tile_order_from_canonical(canon, signs)
    return dense, scale, torch.from_numpy(bt.copy()), torch.from_numpy(mt.copy())


def test_round_trip_and_header(tmp_path):
    m, k = 256, 384
    _, scale, bits, meta = _tile_operands(1, m, k)
    bias = torch.arange(m, dtype=torch.float16)
    path = str(tmp_path / "w.ob24")
    packed_file.save_packed(path, bits, meta, m, k, scale=torch.from_numpy(scale), bias=bias, row0=512, rows_total=1024, slab=2, slabs=4)
    info = packed_file.read_header(path)
    assert (info.order, info.m, info.k, info.row0, info.rows_total, info.slab, info.slabs) == (packed_file.ORDER_TILE, m, k, 512, 1024, 2, 4)
    assert os.path.getsize(path) % 256 == 0
    info2, b2, m2, s2, bias2 = packed_file.load_packed(path)
    assert info2 == info and torch.equal(b2, bits) and torch.equal(m2, meta)
    assert torch.equal(s2, torch.from_numpy(scale)) and torch.equal(bias2, bias)


def test_reference_order_payload(tmp_path):
    # the exchange format of the reference packer: (k/2, m/8) sign bytes and int16 (m, k/16) metadata
    m, k = 128, 256
    rng = np.random.default_rng(2)
    dense, _ = helpers.make_weights(rng, m, k)
    a_bits, e_meta = oracle.pack(dense, oracle.META_PYTHON)
    path = str(tmp_path / "ref.ob24")
    packed_file.save_packed(path, torch.from_numpy(a_bits), torch.from_numpy(e_meta.copy()), m, k, order=packed_file.ORDER_PYTHON)
    info, b2, m2, s2, bias2 = packed_file.load_packed(path)
    assert info.order == packed_file.ORDER_PYTHON and s2 is None and bias2 is None
    assert b2.shape == (k // 2, m // 8) and m2.shape == (m, k // 16) and m2.dtype == torch.int16
    assert (b2.numpy() == a_bits).all() and (m2.numpy() == e_meta).all()


def test_damage_is_detected(tmp_path):
    m, k = 128, 128
    _, scale, bits, meta = _tile_operands(3, m, k)
    path = str(tmp_path / "w.ob24")
    packed_file.save_packed(path, bits, meta, m, k, scale=torch.from_numpy(scale))
    raw = bytearray(open(path, "rb").read())
    flipped = bytearray(raw)
    flipped[256 + 100] ^= 0x10                                   # one bit of the sign section
    open(path, "wb").write(flipped)
    with pytest.raises(packed_file.PackedFileError, match="checksum"):
        packed_file.load_packed(path)
    open(path, "wb").write(raw[:1000])
    with pytest.raises(packed_file.PackedFileError):
        packed_file.load_packed(path)
    open(path, "wb").write(b"not a weight file" * 40)
    with pytest.raises(packed_file.PackedFileError, match="not a packed"):
        packed_file.read_header(path)
    with pytest.raises(ValueError):
        packed_file.save_packed(path, bits, meta, 100, 128)        # not whole tiles
    with pytest.raises(ValueError):
        packed_file.save_packed(path, bits[:-1], meta, m, k)       # payload of the wrong size


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _rank_worker(rank, world, port, directory, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import onebitsparsemul_b200 as ob
        from onebitsparsemul_b200.sharded import ShardedBinaryLinear
        m, k, n = 768, 256, 8
        rng = np.random.default_rng(21)
        dense, scale = helpers.make_weights(rng, m, k)
        B = helpers.make_tokens(rng, k, n, "int")

        def pack(w, s):                                     # the oracle stands in for the pack kernel: tile order on CPU
            canon, signs, _ = oracle.compress(w.numpy())
            bt, mt = helpers.tile_order_from_canonical(canon, signs)
            return ob.PackedWeight(w.shape[0], w.shape[1], torch.from_numpy(bt.copy()), torch.from_numpy(mt.copy()), s)

        def matmul(pw, Bt, out, row0, rows):                # ... and for the GEMM: dense weights rebuilt from the tiles
            want = _gemm_from_tiles(pw, Bt.numpy())
            out.copy_(torch.from_numpy(want[row0:row0 + rows]))

        layer = ShardedBinaryLinear(m, k, matmul=matmul, pack=pack).pack_full(torch.from_numpy(dense), torch.from_numpy(scale))
        before = layer.forward(torch.from_numpy(B), gather="all", out_dtype=torch.float32).numpy()
        layer.save(directory, "proj")
        dist.barrier()
        fresh = ShardedBinaryLinear(m, k, matmul=matmul, pack=pack).load(directory, "proj", device="cpu")
        after = fresh.forward(torch.from_numpy(B), gather="all", out_dtype=torch.float32).numpy()
        canon, signs, _ = oracle.compress(dense)
        want, _ = oracle.gemm(oracle.pack_bits(signs), oracle.meta_reorder(canon, 0), 0, B, m, scale=scale)
        mine = packed_file.slab_path(directory, "proj", rank, world)
        other = packed_file.slab_path(directory, "proj", 1 - rank, world)
        # a layer cut differently must refuse these files
        refused = False
        try:
            ShardedBinaryLinear(m + 256, k, matmul=matmul, pack=pack).load(directory, "proj", device="cpu")
        except (packed_file.PackedFileError, FileNotFoundError):
            refused = True
        q.put((rank, bool((before == want).all()), bool((after == want).all()), os.path.exists(mine) and os.path.exists(other), refused,
               packed_file.read_header(mine).row0 == layer.start))
    finally:
        dist.destroy_process_group()


def _gemm_from_tiles(pw, B):
    """Dense {-1, 0, +1} weights from tile-ordered operands (numpy restatement of the tile order), times B."""
    m, k = pw.m, pw.k
    bits = pw.bits_tile.numpy().view(np.uint32).reshape(m // 128, k // 128, 128, 2)
    meta = pw.meta_tile.numpy().view(np.uint16).reshape(m // 128, k // 128, 128, 8)
    W = np.zeros((m, k), np.float32)
    for r in range(128):
        r0, r1, r2 = r & 7, (r >> 3) & 1, r >> 4
        for c in range(8):
            c1, c2 = c & 1, c >> 1
            word = meta[:, :, r0 + 8 * c1 + 16 * r2, 2 * c2 + r1].astype(np.int64)     # (mt, kt)
            for t in range(8):                                    # kept value t of the chunk: group t // 2, position from the nibble
                pos = (t // 2) * 4 + ((word >> (2 * t)) & 3)
                v = c * 8 + t
                bit = (bits[:, :, r, v // 32] >> np.uint32((v % 32) // 2 + 16 * (v % 2))) & 1
                val = np.where(bit == 1, 1.0, -1.0).astype(np.float32)
                mt_i, kt_i = np.meshgrid(np.arange(m // 128), np.arange(k // 128), indexing="ij")
                W[mt_i * 128 + r, kt_i * 128 + c * 16 + pos] = val
    out = W @ B.astype(np.float32)
    if pw.scale is not None:
        out = out * pw.scale.numpy().astype(np.float32)[:, None]
    return out


def test_one_file_per_slab_two_cpu_ranks(tmp_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_worker, args=(r, 2, port, str(tmp_path), q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, before, after, files, refused, row0_ok in results:
        assert before and after and files and refused and row0_ok, results


@pytest.mark.gpu
def test_save_load_gemm_bit_identical_on_gpu(tmp_path):
    import onebitsparsemul_b200 as ob
    rng = np.random.default_rng(31)
    m, k = 512, 1024
    dense, scale = helpers.make_weights(rng, m, k)
    layer = ob.BinaryLinear_2_4(k, m, out_dtype=torch.float16, bias=True).cuda()
    layer.pack(torch.from_numpy(dense).cuda(), scale=torch.from_numpy(scale).cuda(), bias=torch.linspace(-1, 1, m))
    path = str(tmp_path / "layer.ob24")
    layer.save_packed(path)
    again = ob.BinaryLinear_2_4.from_packed_file(path)
    for n in (1, 8, 64, 512):
        x = torch.from_numpy(helpers.make_tokens(rng, k, n).T.copy()).cuda()
        assert torch.equal(layer.forward_tokens(x), again.forward_tokens(x))
        B = x.t().contiguous()
        assert torch.equal(layer(B), again(B))
    # a reference-ordered file (the exchange format) loads into the same tiles
    ref_path = str(tmp_path / "ref.ob24")
    packed_file.save_packed(ref_path, layer.packed_binary_sparse, layer.meta, m, k, order=packed_file.ORDER_PYTHON, scale=layer.scale)
    pw, _, info = ob.PackedWeight.load(ref_path)
    assert info.order == packed_file.ORDER_PYTHON
    assert torch.equal(pw.bits_tile, layer.bits_tile) and torch.equal(pw.meta_tile, layer.meta_tile)
