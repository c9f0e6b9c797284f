"""Row-sharded one-bit 2:4 sparse GEMM across the GPUs of one node.

The path shards by output rows with no exchange during compute: rank g owns the weight rows
``[start_g, start_g + rows_g)`` -- its own sign bits, metadata and scale, packed per slab (a slab of
a global pack is not contiguous: the reference bitfield is column-major in m and its metadata rows
are shuffled in groups of 64) -- every rank holds the tokens B, and rank g writes the C rows of its
slab. The reference has no multi-GPU code; this module is the only place a collective appears, and
only when the caller asks for the full C on every rank:

  gather="none"     each rank returns its (rows_g, n) slab                      (no collective)
  gather="all"      one NCCL all-gather after the GEMM
  gather="overlap"  the slab is computed in row chunks; chunk c travels (grouped send/recv into the
                    right rows of the full C) on a side stream while chunk c+1 is computed

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


def chunk_rows(rows: int, chunks: int, block: int = ROW_BLOCK) -> List[Tuple[int, int]]:
    """Split a slab into at most `chunks` row chunks of whole blocks."""
    chunks = max(1, min(chunks, rows // block))
    return row_partition(rows, chunks, block)


class ShardedBinaryLinear:
    """One rank's share of a row-sharded one-bit 2:4 layer.

    `matmul` computes C_slab = W_slab @ B for a packed slab; it defaults to the library's GEMM and is
    injectable so that the host-side logic can be exercised on CPU ranks.
    """

    def __init__(self, outfeatures: int, infeatures: int, group: Optional[dist.ProcessGroup] = None,
                 matmul: Optional[Callable] = None, pack: Optional[Callable] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.m, self.k = outfeatures, infeatures
        self.partition = row_partition(outfeatures, self.world)
        self.start, self.rows = self.partition[self.rank]
        self._matmul, self._pack = matmul, pack
        self.packed = None
        self._side = None

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

    # -- GEMM ---------------------------------------------------------------------------------------------
    def _gemm(self, B, out, row0=0, rows=None):
        rows = self.rows if rows is None else rows
        if self._matmul is not None:
            return self._matmul(self.packed, B, out, row0, rows)
        from . import matmul_rows
        return matmul_rows(self.packed, B, out, row0, rows)

    def forward(self, B, gather: str = "none", out_dtype=torch.float16, chunks: int = 4):
        n = B.shape[1]
        dev = B.device
        if gather == "none" or self.world == 1:
            out = torch.empty((self.rows, n), dtype=out_dtype, device=dev)
            self._gemm(B, out)
            return out
        full = torch.empty((self.m, n), dtype=out_dtype, device=dev)
        mine = full[self.start:self.start + self.rows]
        if gather == "all" and len({r for _, r in self.partition}) == 1:
            self._gemm(B, mine)
            dist.all_gather_into_tensor(full, mine, group=self.group)
            return full
        if gather == "all":
            chunks = 1                 # unequal slabs: one grouped send/recv exchange after the GEMM
            gather = "overlap"
        if gather != "overlap":
            raise ValueError(f"unknown gather mode {gather!r}")
        # every rank must cut its slab into the same number of chunks
        nchunks = max(1, min(chunks, min(r for _, r in self.partition) // ROW_BLOCK))
        my_chunks = chunk_rows(self.rows, nchunks)
        cuda = dev.type == "cuda"
        if cuda and self._side is None:
            self._side = torch.cuda.Stream(device=dev)
        pending = []
        for c, (c0, crows) in enumerate(my_chunks):
            self._gemm(B, mine[c0:c0 + crows], c0, crows)
            ops = []
            for peer, (ps, prows) in enumerate(self.partition):
                if peer == self.rank:
                    continue
                pc0, pcrows = chunk_rows(prows, nchunks)[c]
                ops.append(dist.P2POp(dist.isend, mine[c0:c0 + crows], peer, group=self.group))
                ops.append(dist.P2POp(dist.irecv, full[ps + pc0:ps + pc0 + pcrows], peer, group=self.group))
            if cuda:
                ready = torch.cuda.Event()
                ready.record()
                with torch.cuda.stream(self._side):
                    self._side.wait_event(ready)
                    pending += dist.batch_isend_irecv(ops)
            else:
                pending += dist.batch_isend_irecv(ops)
        for w in pending:
            w.wait()
        if cuda:
            torch.cuda.current_stream().wait_stream(self._side)
        return full
