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

``forward_host`` is the same GEMM for tokens and result in pinned host memory: in column panels, every rank uploads
1/world of a panel, the shares are all-gathered over NVLink, and the panel of C goes back to the host while the next
panels travel and multiply.

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
        self._host_state = {}            # n -> device copies of B and of this rank's C, and the copy stream (forward_host)
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

    # -- tokens and result in host memory -----------------------------------------------------------------
    def forward_host(self, B_host, out_host=None, out_dtype=torch.float16, panels: int = 8):
        """C_slab = W_slab @ B for tokens B (k, n) in pinned HOST memory -- the same B on every rank -- with this
        rank's (rows_g, n) slab of the result written to pinned host memory.

        One rank: the library's host-buffer pipeline (``onebit_matmul_packed_host``). Several ranks: B crosses
        PCIe once per NODE, not once per rank. The tokens are cut into column panels (whole 256-token blocks); for
        every panel each rank uploads only its 1/world share of the panel's rows (a pitched copy), one NCCL
        all-gather over NVLink completes the panel in place, the slab GEMM runs on it, and the panel of the result
        goes back to the host. Three slots rotate on three streams, so panel p + 1 travels in while panel p is
        multiplied and panel p - 1 travels out: PCIe carries both directions at once and a call costs about
        max(H2D, D2H) / world. Needs k % world == 0 and n % 8 == 0 (otherwise every rank uploads all of B, unpipelined).
        The work is queued on the current stream; synchronise it before reading the result."""
        from . import _lib, matmul_packed_host
        n = B_host.shape[1]
        if out_host is None:
            out_host = torch.empty((self.rows, n), dtype=out_dtype).pin_memory()
        if self.world == 1:
            return matmul_packed_host(self.packed, B_host, out_host, out_dtype)
        if B_host.is_cuda or not B_host.is_pinned() or B_host.dtype != torch.float16 or tuple(B_host.shape) != (self.k, n) \
                or not B_host.is_contiguous():
            raise ValueError("B_host must be a contiguous pinned CPU float16 tensor of shape (k, n)")
        if out_host.is_cuda or not out_host.is_pinned() or tuple(out_host.shape) != (self.rows, n) or not out_host.is_contiguous():
            raise ValueError("out_host must be a contiguous pinned CPU tensor of shape (rows of this rank, n)")
        dev = self.packed.bits_tile.device
        main = torch.cuda.current_stream(dev)
        esz = out_host.element_size()
        if self.k % self.world != 0 or n % 8 != 0:
            # every rank uploads all of B; no pipeline
            Bd = B_host.to(dev, non_blocking=True)
            Cd = torch.empty((self.rows, n), dtype=out_host.dtype, device=dev)
            self._gemm(Bd, Cd)
            out_host.copy_(Cd, non_blocking=True)
            return out_host
        lib = _lib.load()
        blocks = (n + ROW_BLOCK - 1) // ROW_BLOCK
        width = ((blocks + panels - 1) // max(1, panels)) * ROW_BLOCK          # tokens per panel: whole 256-token blocks
        slots = 3
        st = self._host_state.get((n, out_host.dtype))
        if st is None:
            st = self._host_state[(n, out_host.dtype)] = dict(
                B=[torch.empty(self.k * width, dtype=torch.float16, device=dev) for _ in range(slots)],
                C=[torch.empty(self.rows * width, dtype=out_host.dtype, device=dev) for _ in range(slots)],
                up=torch.cuda.Stream(device=dev), down=torch.cuda.Stream(device=dev))
        up, down = st["up"], st["down"]
        up.wait_stream(main)                                    # earlier work of the caller (and of the previous call) first
        down.wait_stream(main)
        share = self.k // self.world
        r0 = self.rank * share
        multiplied, drained = [None] * slots, [None] * slots
        c0 = 0
        p = 0
        while c0 < n:
            w = min(width, n - c0)
            s = p % slots
            Bp = st["B"][s][:self.k * w].view(self.k, w)
            Cp = st["C"][s][:self.rows * w].view(self.rows, w)
            mine = Bp[r0:r0 + share]
            with torch.cuda.stream(up):
                if multiplied[s] is not None:
                    up.wait_event(multiplied[s])                # the GEMM that read this slot's tokens is done
                _lib.check(lib.onebit_copy_2d_async(mine.data_ptr(), w * 2, B_host.data_ptr() + (r0 * n + c0) * 2, n * 2,
                                                    w * 2, share, up.cuda_stream))
                loaded = torch.cuda.Event()
                loaded.record(up)
            main.wait_event(loaded)
            dist.all_gather_into_tensor(Bp, mine, group=self.group)     # in place: the share already sits at its offset
            if drained[s] is not None:
                main.wait_event(drained[s])                     # this slot's previous result has left
            self._gemm(Bp, Cp)
            multiplied[s] = torch.cuda.Event()
            multiplied[s].record(main)
            with torch.cuda.stream(down):
                down.wait_event(multiplied[s])
                _lib.check(lib.onebit_copy_2d_async(out_host.data_ptr() + c0 * esz, n * esz, Cp.data_ptr(), w * esz,
                                                    w * esz, self.rows, down.cuda_stream))
                drained[s] = torch.cuda.Event()
                drained[s].record(down)
            c0 += w
            p += 1
        main.wait_stream(down)
        main.wait_stream(up)
        return out_host

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
