"""Multi-GPU partitioner for the matmul path: one process per GPU, torch.distributed
for the plumbing.

The reference has no distributed layer at all; "multi-device" there is a
``Device{backend,id}`` tag and a ``cudaSetDevice`` before each launch
(include/tt/device.h:37-51, backend/cuda/kernel_launch.cuh:20), and a cross-device
copy bounces through the host (autograd/unary_ops.cpp:67-83).  This module adds the
one thing the matmul path needs on an 8-GPU box:

* batched products (B > 1) are sharded over the batch dim -- batches are independent,
  so there is no data-path collective; each rank keeps its slice of the result
  (``gather=True`` all-gathers the slices, which are contiguous chunks of [B,N,M]);
* a single large product (B == 1) is sharded over output-column blocks: rank r computes
  ``lhs . rhs[:, c0:c1]`` -- a strided view of rhs consumed directly by the kernels --
  into its column block of C, and one all-gather of C follows (the only exchange step).

The split itself is computed by the C ABI (``ttb_partition``) so that the C++ shim
and this module agree.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import backend

# Column blocks are cut on multiples of the tensor-core kernel's tile width so that no
# rank gets a partial tile in the middle of the matrix, and block starts stay 16-byte
# aligned for TMA.
COL_ALIGN = 128


@dataclass(frozen=True)
class Partition:
    kind: str  # "batch" or "columns"
    begin: int
    end: int

    @property
    def size(self) -> int:
        return self.end - self.begin


def partition(B: int, N: int, K: int, M: int, world: int, rank: int, col_align: int = COL_ALIGN) -> Partition:
    b, e = ctypes.c_int64(), ctypes.c_int64()
    rc = backend.lib().ttb_partition(B, N, K, M, world, rank, col_align, ctypes.byref(b), ctypes.byref(e))
    if rc < 0:
        backend._raise(rc)
    return Partition("columns" if rc == 1 else "batch", b.value, e.value)


class ShardedMatmul:
    """Callable ``(lhs, rhs) -> out`` that splits one batched product over the ranks of a
    process group.  Every rank passes the FULL operands (replicated on its own device;
    placing them is set-up, not part of the product) and computes only its share.

    ``local_matmul(lhs3, rhs3, out3)`` does the per-rank product; it defaults to the CUDA
    kernels and exists so the host logic can be exercised on CPU ranks (gloo) in tests.
    """

    def __init__(self, group: Optional[dist.ProcessGroup] = None,
                 local_matmul: Optional[Callable[[torch.Tensor, torch.Tensor, torch.Tensor], None]] = None,
                 col_align: int = COL_ALIGN, exchange: str = "auto"):
        # exchange of the fused column-block product: "multicast" = one multimem store per tile
        # through NVSwitch, "peer" = one store per peer GPU, "auto" = multicast when the
        # symmetric buffer has a multicast mapping
        self.exchange = exchange
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.col_align = col_align
        self._local = local_matmul or (lambda a, b, o: backend.batched_matmul(a, b, out=o))
        self._stage: Optional[torch.Tensor] = None
        self._gathered: Optional[torch.Tensor] = None
        self._host_lhs: Optional[torch.Tensor] = None
        self._host_rhs: Optional[torch.Tensor] = None
        self._host_out: Optional[torch.Tensor] = None
        self._kernel_done: Optional[torch.cuda.Event] = None
        self._symm = {}          # storage pointer -> (tensor, symmetric-memory handle) of the fused path's C buffers
        self._last_fused = None  # storage pointer of the C the previous fused product wrote

    # -- fused exchange: C lives in symmetric memory so that every rank can store into every C
    def symmetric_output(self, shape, dtype: torch.dtype, device) -> torch.Tensor:
        """Allocates one C buffer of this rank in ``torch.distributed`` symmetric memory and
        exchanges the peer mappings (a collective: every rank must call it with the same shape).
        A product whose `out` is such a tensor uses the fused GEMM + all-gather kernel: the column
        block is computed into it and stored, tile by tile from inside the kernel, into the peers'
        C over NVLink; one symmetric-memory barrier per product replaces the NCCL all-gather and
        the re-layout pass.

        Ordering rule.  The kernel of rank s writes into rank r's C.  After the product's barrier
        every rank holds the complete C and may read it with work enqueued on the same stream.
        The NEXT product must not start writing into that C while some rank still reads it.  Two
        ways, both handled by ``__call__``: call this method twice and alternate the two buffers
        as `out` -- a rank then reaches the product that overwrites a buffer only after every
        rank has passed the barrier of the product in between, i.e. after all their reads of that
        buffer, which precede it on their streams; or keep one buffer, and ``__call__`` puts a
        second barrier in FRONT of every product that writes the buffer the previous one wrote."""
        import torch.distributed._symmetric_memory as symm

        t = symm.empty(tuple(shape), dtype=dtype, device=device)
        group = self.group if self.group is not None else dist.group.WORLD
        hdl = symm.rendezvous(t, group.group_name)
        if int(hdl.buffer_ptrs[hdl.rank]) != t.untyped_storage().data_ptr():
            raise backend.TTBError("symmetric buffer does not start at the tensor's storage")
        self._symm[t.untyped_storage().data_ptr()] = (t, hdl)
        return t

    def multicast_available(self, out: torch.Tensor) -> bool:
        """True if `out` is a symmetric C buffer of this object with an NVSwitch multicast mapping."""
        entry = self._symm.get(out.untyped_storage().data_ptr())
        return bool(entry is not None and getattr(entry[1], "has_multicast_support", False))

    def _fused_handle(self, lhs: torch.Tensor, out: Optional[torch.Tensor]):
        """The symmetric-memory handle of `out` if the fused exchange applies, else None."""
        if out is None or lhs.dtype != torch.float32:
            return None
        entry = self._symm.get(out.untyped_storage().data_ptr())
        return entry[1] if entry is not None else None

    def plan(self, lhs: torch.Tensor, rhs: torch.Tensor) -> Partition:
        B, N, K = lhs.shape
        M = rhs.shape[2]
        return partition(B, N, K, M, self.world, self.rank, self.col_align)

    def _buffer(self, name: str, shape, like: torch.Tensor) -> torch.Tensor:
        cur = getattr(self, name)
        n = 1
        for s in shape:
            n *= s
        if cur is None or cur.numel() < n or cur.dtype != like.dtype or cur.device != like.device:
            cur = torch.empty(n, dtype=like.dtype, device=like.device)
            setattr(self, name, cur)
        return cur[:n].view(*shape)

    def __call__(self, lhs: torch.Tensor, rhs: torch.Tensor, out: Optional[torch.Tensor] = None,
                 gather: bool = True, kernel_done: Optional[torch.cuda.Event] = None) -> torch.Tensor:
        """`kernel_done`, if given, is recorded on the current stream right after this rank's
        product kernel and before any exchange or barrier (for timing breakdowns)."""
        if lhs.dim() != 3 or rhs.dim() != 3:
            raise backend.TTBError("ShardedMatmul expects rank-3 operands")
        B, N, K = lhs.shape
        M = rhs.shape[2]
        part = self.plan(lhs, rhs)
        self._kernel_done = kernel_done
        if part.kind == "batch":
            return self._batch(lhs, rhs, out, part, gather)
        return self._columns(lhs, rhs, out, part, gather)

    def _mark_kernel_done(self):
        ev = getattr(self, "_kernel_done", None)
        if ev is not None:
            ev.record()
            self._kernel_done = None

    def host_shards(self, N: int, K: int, M: int):
        """How ``columns_from_host`` splits lhs [N,K] . rhs [K,M] over the ranks: this rank's
        half-open row range of lhs and column range of rhs / out."""
        part = partition(1, N, K, M, self.world, self.rank, self.col_align)
        rows = (N + self.world - 1) // self.world
        return (min(self.rank * rows, N), min((self.rank + 1) * rows, N)), (part.begin, part.end)

    def columns_from_host(self, lhs_rows_host: torch.Tensor, rhs_block_host: torch.Tensor,
                          out_block_host: torch.Tensor, N: int) -> None:
        """One column-sharded product whose operands and result live in (pinned) HOST memory, the
        multi-GPU form of ``batched_matmul_host`` for one process per GPU, where every process
        holds a shard of the data: `lhs_rows_host` [rows_r, K] is this rank's row range of lhs,
        `rhs_block_host` [K, cols_r] its column block of rhs (both as ``host_shards`` cuts them,
        contiguous), `out_block_host` [N, cols_r] receives its column block of the result.  Each
        rank uploads only its shards over its own PCIe link; the rows of lhs are all-gathered over
        NVLink (NCCL) so that every GPU holds all of lhs; the block product runs; the block of C
        is downloaded.  Each operand byte crosses PCIe once in the whole job, not once per rank.
        Synchronises."""
        K = rhs_block_host.shape[0]
        cols = rhs_block_host.shape[1]
        dev = torch.device("cuda", torch.cuda.current_device())
        like = torch.empty(0, dtype=lhs_rows_host.dtype, device=dev)
        rows = (N + self.world - 1) // self.world
        full = self._buffer("_host_lhs", (self.world * rows, K), like)
        mine = full[self.rank * rows:self.rank * rows + rows]
        if lhs_rows_host.shape[0] > 0:
            mine[:lhs_rows_host.shape[0]].copy_(lhs_rows_host, non_blocking=True)
        if self.world > 1:
            dist.all_gather_into_tensor(full.view(-1), mine.reshape(-1), group=self.group)
        if cols > 0:
            blk = self._buffer("_host_rhs", (1, K, cols), like)
            blk[0].copy_(rhs_block_host, non_blocking=True)
            res = self._buffer("_host_out", (1, N, cols), like)
            self._local(full[:N].unsqueeze(0), blk, res)
            out_block_host.copy_(res[0], non_blocking=True)
        torch.cuda.synchronize()

    # -- batch sharding: no exchange unless the caller wants the full result everywhere
    def _batch(self, lhs, rhs, out, part: Partition, gather: bool):
        B, N, _ = lhs.shape
        M = rhs.shape[2]
        if out is None:
            out = torch.empty((B, N, M), dtype=lhs.dtype, device=lhs.device)
        if part.size > 0:
            self._local(lhs[part.begin:part.end], rhs[part.begin:part.end], out[part.begin:part.end])
        self._mark_kernel_done()
        if gather and self.world > 1:
            # Slices are contiguous chunks of [B,N,M]; sizes may differ by one batch.
            chunks = []
            for r in range(self.world):
                p = partition(B, N, lhs.shape[2], M, self.world, r, self.col_align)
                chunks.append(out[p.begin:p.end])
            if len({c.shape[0] for c in chunks}) == 1 and out.is_contiguous():
                dist.all_gather_into_tensor(out.view(-1), chunks[self.rank].reshape(-1), group=self.group)
            else:
                for r, c in enumerate(chunks):
                    if c.numel():
                        dist.broadcast(c, src=dist.get_global_rank(self.group, r) if self.group else r,
                                       group=self.group)
        return out if gather or self.world == 1 else out[part.begin:part.end]

    # -- column sharding: compute the block, then all-gather C
    def _columns(self, lhs, rhs, out, part: Partition, gather: bool):
        _, N, _ = lhs.shape
        M = rhs.shape[2]
        if out is None:
            out = torch.empty((1, N, M), dtype=lhs.dtype, device=lhs.device)
        if self.world == 1 or not gather:
            if part.size > 0:
                self._local(lhs, rhs[:, :, part.begin:part.end], out[:, :, part.begin:part.end])
            self._mark_kernel_done()
            return out
        hdl = self._fused_handle(lhs, out)
        if hdl is not None:
            # One kernel computes the block and pushes it to every peer; then the ranks meet.
            key = out.untyped_storage().data_ptr()
            if self._last_fused == key:
                # Same C as the product before: every rank must be done reading it before any
                # rank's kernel stores into it again (see symmetric_output).
                hdl.barrier()
            self._last_fused = key
            block = out[:, :, part.begin:part.end]
            mc = int(hdl.multicast_ptr) if (self.exchange != "peer" and getattr(hdl, "has_multicast_support", False)) else 0
            # multimem.st moves 16 bytes: the block's rows must be 16-byte aligned, 4 columns at a time
            mc_ok = mc != 0 and part.size % 4 == 0 and out.stride(1) % 4 == 0 and out.stride(2) == 1 and \
                (out.storage_offset() + part.begin) % 4 == 0
            if self.exchange == "multicast" and not mc_ok:
                raise backend.TTBError("multicast exchange asked for, but the symmetric buffer has no multicast "
                                       "mapping or the block is not 16-byte aligned")
            if part.size > 0:
                if mc_ok:
                    backend.matmul_allgather_multicast(lhs, rhs[:, :, part.begin:part.end], block, mc)
                else:
                    # peers in ring order starting after this rank, so that at any moment the
                    # ranks' stores are spread over all receivers instead of converging on one
                    peers = [int(hdl.buffer_ptrs[(self.rank + i) % self.world]) for i in range(1, self.world)]
                    backend.matmul_allgather(lhs, rhs[:, :, part.begin:part.end], block, peers)
            self._mark_kernel_done()
            hdl.barrier()
            return out
        parts = [partition(1, N, lhs.shape[2], M, self.world, r, self.col_align) for r in range(self.world)]
        width = max(p.size for p in parts)
        equal = all(p.size == width for p in parts)
        # NCCL concatenates contiguous per-rank chunks, so the block is computed into a
        # contiguous [N, width] staging buffer, gathered as [world, N, width], and then laid
        # out row-major.
        stage = self._buffer("_stage", (1, N, width), lhs)
        if part.size > 0:
            self._local(lhs, rhs[:, :, part.begin:part.end], stage[:, :, :part.size])
        self._mark_kernel_done()
        gathered = self._buffer("_gathered", (self.world, N, width), lhs)
        dist.all_gather_into_tensor(gathered.view(-1), stage.reshape(-1), group=self.group)
        if equal:
            out.view(N, self.world, width).copy_(gathered.permute(1, 0, 2))
        else:
            for r, p in enumerate(parts):
                if p.size:
                    out[0, :, p.begin:p.end].copy_(gathered[r, :, :p.size])
        return out
