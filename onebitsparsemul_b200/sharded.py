"""Row-sharded one-bit 2:4 sparse GEMM across the GPUs of one node.

The path shards by output rows with no exchange during compute: rank g owns the weight rows
``[start_g, start_g + rows_g)`` -- its own sign bits, metadata and scale, packed per slab (a slab of
a global pack is not contiguous: the reference bitfield is column-major in m and its metadata rows
are shuffled in groups of 64) -- every rank holds the tokens B, and rank g writes the C rows of its
slab. The reference has no multi-GPU code; this module is the only place a collective appears, and
only when the caller asks for the full C on every rank:

  gather="none"     each rank returns its (rows_g, n) slab                      (no collective)
  gather="all"      one NCCL all-gather after the GEMM (one grouped send/recv exchange when the slabs
                    are of unequal height)
  gather="fused"    no collective kernel at all: the GEMM's epilogue stores every output tile into this
                    rank's C and, through peer-mapped memory, into the same rows of every other rank's C
                    while the next tile is multiplied (``onebit_matmul_packed_scatter``). C lives in a
                    buffer all ranks have mapped (symmetric memory, else CUDA IPC handles); two tiny
                    all-reduces order the ranks before peers are overwritten and before C is read.
                    The returned tensor is that cached buffer: the next fused call of the same shape
                    overwrites it.

One process per GPU, ``torch.distributed`` for the plumbing. Slabs are whole 256-row blocks so that
every rank runs the same kernel variants as a single GPU would; results are bit-identical to the
single-GPU run because no reduction crosses a slab boundary.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

ROW_BLOCK = 256


def row_partition(m: int, world: int, block: int = ROW_BLOCK) -> List[Tuple[int, int]]:
    """Split m rows into `world` contiguous slabs of whole blocks, as even as possible.
    Returns [(start, rows)] per rank; needs m % block == 0 and m // block >= world."""
    if m % block != 0:
        raise ValueError(f"m = {m} must be a multiple of {block}")
    blocks = m // block
    if blocks < world:
        raise ValueError(f"{blocks} row blocks cannot be spread over {world} ranks")
    base, extra = divmod(blocks, world)
    out, start = [], 0
    for r in range(world):
        rows = (base + (1 if r < extra else 0)) * block
        out.append((start, rows))
        start += rows
    return out


class ShardedBinaryLinear:
    """One rank's share of a row-sharded one-bit 2:4 layer.

    `matmul` computes C_slab = W_slab @ B for a packed slab; it defaults to the library's GEMM and is
    injectable so that the host-side logic can be exercised on CPU ranks.
    """

    def __init__(self, outfeatures: int, infeatures: int, group: Optional[dist.ProcessGroup] = None,
                 matmul: Optional[Callable] = None, pack: Optional[Callable] = None, scatter: Optional[Callable] = None,
                 peer_buffer: Optional[Callable] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.m, self.k = outfeatures, infeatures
        self.partition = row_partition(outfeatures, self.world)
        self.start, self.rows = self.partition[self.rank]
        self._matmul, self._pack = matmul, pack
        self.packed = None
        self._scatter = scatter
        self._peer_buffer = peer_buffer  # (layer, n, device) -> what _peer_mapped_buffer returns; for CPU ranks
        self._fused = {}                 # n -> (full C, peers' base addresses, keep-alive objects)
        self._flag = None
        self.fused_backend = None        # "symmetric_memory" or "ipc", once a fused buffer exists

    # -- weights ---------------------------------------------------------------------------------------
    def pack_slab(self, weight_slab, scale_slab=None, apply_mask=True):
        """weight_slab: this rank's (rows_g, k) rows of the dense weight."""
        if tuple(weight_slab.shape) != (self.rows, self.k):
            raise ValueError(f"rank {self.rank} expects a slab of shape ({self.rows}, {self.k})")
        if self._pack is not None:
            self.packed = self._pack(weight_slab, scale_slab)
        else:
            from . import pack_weight
            self.packed = pack_weight(weight_slab, scale=scale_slab, apply_mask=apply_mask, keep_reference=False)
        return self

    def pack_full(self, weight, scale=None, apply_mask=True):
        """weight: the whole (m, k) matrix, available on every rank; each rank packs only its slab."""
        sl = slice(self.start, self.start + self.rows)
        return self.pack_slab(weight[sl], None if scale is None else scale[sl], apply_mask)

    # -- persistence: one file per row slab, every rank touches only its own ------------------------------------
    def save(self, directory: str, name: str):
        """Write this rank's slab to `directory` (packed_file.slab_path names the file)."""
        from . import packed_file
        self.packed.save(packed_file.slab_path(directory, name, self.rank, self.world), row0=self.start, rows_total=self.m,
                         slab=self.rank, slabs=self.world)

    def load(self, directory: str, name: str, device="cuda"):
        """Read this rank's slab; the file must have been written for the same partition."""
        from . import PackedWeight, packed_file
        path = packed_file.slab_path(directory, name, self.rank, self.world)
        pw, _, info = PackedWeight.load(path, device)
        if (info.row0, info.m, info.k, info.rows_total, info.slabs) != (self.start, self.rows, self.k, self.m, self.world):
            raise packed_file.PackedFileError(f"{path} was written for another partition of the matrix")
        self.packed = pw
        return self

    # -- GEMM ---------------------------------------------------------------------------------------------
    def _gemm(self, B, out, row0=0, rows=None):
        rows = self.rows if rows is None else rows
        if self._matmul is not None:
            return self._matmul(self.packed, B, out, row0, rows)
        from . import matmul_rows
        return matmul_rows(self.packed, B, out, row0, rows)

    def forward(self, B, gather: str = "none", out_dtype=torch.float16):
        n = B.shape[1]
        dev = B.device
        if gather == "none" or self.world == 1:
            out = torch.empty((self.rows, n), dtype=out_dtype, device=dev)
            self._gemm(B, out)
            return out
        if gather == "fused":
            return self._forward_fused(B, out_dtype)
        if gather != "all":
            raise ValueError(f"unknown gather mode {gather!r}")
        full = torch.empty((self.m, n), dtype=out_dtype, device=dev)
        mine = full[self.start:self.start + self.rows]
        self._gemm(B, mine)
        if len({r for _, r in self.partition}) == 1:
            dist.all_gather_into_tensor(full, mine, group=self.group)
            return full
        # unequal slabs: every rank sends its slab to, and receives the other slabs from, every peer
        ops = []
        for peer, (ps, prows) in enumerate(self.partition):
            if peer == self.rank:
                continue
            ops.append(dist.P2POp(dist.isend, mine, peer, group=self.group))
            ops.append(dist.P2POp(dist.irecv, full[ps:ps + prows], peer, group=self.group))
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        return full

    # -- fused GEMM + all-gather ------------------------------------------------------------------------
    def _peer_mapped_buffer(self, n, dev):
        """A (m, n) fp16 buffer on every rank that all ranks can store to: returns (tensor, [base address
        of rank p's buffer as seen from this process], (handle, [tensor aliasing rank p's buffer]))."""
        shape = (self.m, n)
        if self._peer_buffer is not None:
            self.fused_backend = "injected"
            return self._peer_buffer(self, n, dev)
        try:
            import torch.distributed._symmetric_memory as symm
            group = self.group if self.group is not None else dist.group.WORLD
            full = symm.empty(shape, dtype=torch.float16, device=dev)
            handle = symm.rendezvous(full, group)
            ptrs = [int(p) for p in handle.buffer_ptrs]
            views = [full if p == self.rank else handle.get_buffer(p, shape, torch.float16) for p in range(self.world)]
            self.fused_backend = "symmetric_memory"
            return full, ptrs, (handle, views)
        except Exception:                                # fall back to plain CUDA IPC handles
            full = torch.empty(shape, dtype=torch.float16, device=dev)
            mine = full.untyped_storage()._share_cuda_()
            handles = [None] * self.world
            dist.all_gather_object(handles, (mine, full.storage_offset() * 2), group=self.group)
            ptrs, views = [], []
            for p, (h, off) in enumerate(handles):
                if p == self.rank:
                    ptrs.append(full.data_ptr())
                    views.append(full)
                    continue
                st = torch.UntypedStorage._new_shared_cuda(*h)
                peer = torch.empty(0, dtype=torch.float16, device=st.device).set_(st, off // 2, shape)
                peer[:1, :1].to(dev)                     # a first copy makes torch enable peer access dev -> peer
                ptrs.append(peer.data_ptr())
                views.append(peer)
            self.fused_backend = "ipc"
            return full, ptrs, (None, views)

    def _rank_barrier(self, dev):
        """Stream-ordered barrier: no rank's later work starts before every rank's earlier work is done."""
        if self._flag is None:
            self._flag = torch.zeros(1, dtype=torch.float32, device=dev)
        dist.all_reduce(self._flag, group=self.group)

    def _forward_fused(self, B, out_dtype):
        if out_dtype != torch.float16:
            raise ValueError("gather='fused' produces float16")
        n, dev = B.shape[1], B.device
        if n not in self._fused:
            self._fused[n] = self._peer_mapped_buffer(n, dev)
        full, ptrs, _ = self._fused[n]
        mine = full[self.start:self.start + self.rows]
        extra = [ptrs[p] + self.start * n * 2 for p in range(self.world) if p != self.rank]
        self._rank_barrier(dev)                          # every rank is done reading the previous result
        if self._scatter is not None:
            self._scatter(self.packed, B, mine, extra)
        else:
            from . import matmul_scatter
            matmul_scatter(self.packed, B, mine, extra)
        self._rank_barrier(dev)                          # every rank's stores have landed
        return full
