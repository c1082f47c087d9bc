"""Host side of the tensor-parallel exchange kernel (csrc/tp_exchange.cu).

The reference has no multi-GPU code; a tensor-parallel port of it would end every row-parallel GEMM with
an NCCL all-reduce and an elementwise residual update.  ``PeerExchange`` replaces that pair by one kernel
that reads the ranks' partial results straight from their memory over NVLink and pushes the updated
residual into every rank's buffer:

    ex = PeerExchange(group, device, rows, cols, torch.bfloat16)
    gemm(..., out=ex.partial[a:b])          # this rank's partial sums
    ex.exchange(gate0, gate1, split_row)     # ex.residual += gate * sum_over_ranks(partial), on every rank

Buffers: each rank allocates one block holding [partial | residual | flag pad] and maps the other ranks'
blocks into its address space through torch's symmetric memory (virtual-memory handles exchanged over the
group's store, every peer's block mapped for this rank's device).  A mapping through torch's storage-sharing
IPC handles is deliberately not offered: such a storage is opened in the owning device's context, and a
kernel on another device may only touch it once peer access between the two devices is enabled in this
process, which nothing on that route guarantees.  Nothing here is NCCL; the process group is used for the
one-time rendezvous and for host-side barriers only.
"""
from __future__ import annotations

import ctypes
import os

import torch

from comfy_kitchen import _native


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class PeerExchange:
    """One rank's view of the shared buffers of a tensor-parallel group, and the launch of the fused
    all-reduce + residual kernel.  World size 1 works too (the kernel then only applies the residual update),
    which is what the single-GPU tests exercise."""

    def __init__(self, group, device, rows: int, cols: int, dtype: torch.dtype = torch.bfloat16, mode: str | None = None,
                 extra_bytes: int = 0):
        import torch.distributed as dist

        assert dtype in (torch.bfloat16, torch.float16) and cols % 8 == 0
        self.device = torch.device(device)
        self.rows, self.cols, self.dtype = rows, cols, dtype
        self._dist, self.group = dist, group
        live = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if live else 1
        self.rank = dist.get_rank(group) if live else 0
        lib = _native.load()
        # the partial region holds either the whole [rows, cols] partial result (exchange / reduce_rows by peer loads)
        # or, in the scattered layout, one slab per source rank with that rank's partial rows of MY row range
        # (written by the peers' GEMM epilogues): world slabs of the largest range
        tiles = (rows + 127) // 128
        slab_rows = max(min(rows, 128 * (tiles * (r + 1) // self.world)) - min(rows, 128 * (tiles * r // self.world))
                        for r in range(self.world)) if self.world > 1 else rows
        self._slab_bytes = _align(max(slab_rows, 1) * cols * 2)
        mat = _align(max(rows * cols * 2, self.world * self._slab_bytes))
        self._pad_bytes = _align(int(lib.ck_tp_pad_bytes()))
        # one block per rank: [partial | residual | NVFP4 codes of the activation | its tiled block scales | flag pad]
        rows_pad, sf_cols = (rows + 127) // 128 * 128, (cols // 16 + 3) // 4 * 4
        q_bytes, sf_bytes = _align(rows * (cols // 2)), _align(rows_pad * sf_cols)
        extra_bytes = _align(extra_bytes)     # a caller-defined region every rank can push slices of (gather_extra)
        self._offsets = (0, mat, 2 * mat + q_bytes + sf_bytes + extra_bytes)
        self._q_off, self._sf_off = 2 * mat, 2 * mat + q_bytes
        self._extra_off, self._extra_bytes = 2 * mat + q_bytes + sf_bytes, extra_bytes
        total = self._offsets[2] + self._pad_bytes
        mode = mode or os.environ.get("CK_TP_PEER_MEMORY", "auto")
        self._keep = []          # objects that own the mappings
        bases = None
        if self.world == 1:
            self._block = torch.zeros(total, dtype=torch.uint8, device=self.device)
            bases, self.mode = [self._block.data_ptr()], "local"
        else:
            if mode not in ("auto", "symm"):
                raise ValueError(f"unknown peer memory mode {mode!r} (only torch symmetric memory is supported)")
            bases, self.mode = self._map_symmetric(total), "symm"
        self._block.zero_()
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=group)   # every pad is zero before anyone's first launch
        n = rows * cols
        self.partial = self._block[:n * 2].view(dtype).view(rows, cols)
        self.residual = self._block[mat:mat + n * 2].view(dtype).view(rows, cols)
        # sequence-parallel pieces: the quantized activation every rank assembles from all ranks' rows, and the row
        # ranges (whole 128-row scale tiles, as even as they come) each rank is responsible for
        self.qx = self._block[self._q_off:self._q_off + rows * (cols // 2)].view(rows, cols // 2)
        self.sx = self._block[self._sf_off:self._sf_off + rows_pad * sf_cols].view(rows_pad, sf_cols)
        self._sf_cols = sf_cols
        self.extra = self._block[self._extra_off:self._extra_off + extra_bytes]
        tiles = rows_pad // 128
        cuts = [min(rows, 128 * (tiles * r // self.world)) for r in range(self.world)] + [rows]
        self.row_bounds = cuts
        self.row_lo, self.row_hi = cuts[self.rank], cuts[self.rank + 1]
        arr = ctypes.c_void_p * self.world
        self._partials = arr(*[b + self._offsets[0] for b in bases])
        self._residuals = arr(*[b + self._offsets[1] for b in bases])
        self._pads = arr(*[b + self._offsets[2] for b in bases])
        self._bases = arr(*bases)
        # scattered layout: where MY partial rows of rank d's range go (d's slab number `rank`), the bounds as the
        # GEMM launcher wants them, and this rank's slabs addressed so that "pointer + global vector index" lands in them
        self._scatter_dests = arr(*[b + self._offsets[0] + self.rank * self._slab_bytes for b in bases])
        self._scatter_bounds = (ctypes.c_int64 * (self.world + 1))(*self.row_bounds)
        back = self.row_lo * cols * 2
        self._slab_partials = arr(*[bases[self.rank] + self._offsets[0] + i * self._slab_bytes - back for i in range(self.world)])
        # NVLink-switch multicast address of the block, when the symmetric allocation has one (0 = none)
        mc = int(getattr(self, "_multicast_base", 0) or 0)
        # Off unless asked for (CK_TP_MULTIMEM=1): measured on 8 B200s the switch path takes the same 107 us per
        # 28 MB exchange as plain peer loads and stores, and on 2 it is slower (101 against 64 us).
        if os.environ.get("CK_TP_MULTIMEM", "0") != "1":
            mc = 0
        self.multimem = mc != 0
        self._mc_partial = ctypes.c_void_p(mc + self._offsets[0] if mc else 0)
        self._mc_residual = ctypes.c_void_p(mc + self._offsets[1] if mc else 0)
        self.calls = 0

    # ---- ways of making one allocation per rank visible to all ranks

    def _map_symmetric(self, total: int):
        import torch.distributed._symmetric_memory as symm_mem

        self._block = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
        group = self.group if self.group is not None else self._dist.group.WORLD
        handle = symm_mem.rendezvous(self._block, group)
        self._keep.append(handle)
        self._multicast_base = int(getattr(handle, "multicast_ptr", 0) or 0)
        ptrs = [int(p) for p in handle.buffer_ptrs]
        assert len(ptrs) == self.world and ptrs[self.rank] == self._block.data_ptr()
        return ptrs

    # ---- the exchange

    def exchange(self, gate0: torch.Tensor, gate1: torch.Tensor | None = None, split_row: int = 0, blocks: int = 0) -> torch.Tensor:
        """residual <- residual + gate * sum_over_ranks(partial), on every rank (rows below split_row use gate0,
        the rest gate1).  Every rank of the group must make the same sequence of calls."""
        g0 = gate0.reshape(-1)
        assert g0.numel() == self.cols and g0.dtype == self.dtype and g0.is_contiguous()
        g1 = None
        if gate1 is not None:
            g1 = gate1.reshape(-1)
            assert g1.numel() == self.cols and g1.dtype == self.dtype and g1.is_contiguous()
        code = 2 if self.dtype == torch.bfloat16 else 1
        _native.call("launch_tp_exchange_kernel", self._partials, self._residuals, self._pads, self._mc_partial,
                     self._mc_residual, self.world, self.rank,
                     ctypes.c_void_p(g0.data_ptr()), ctypes.c_void_p(0 if g1 is None else g1.data_ptr()),
                     int(split_row), self.rows, self.cols, code, int(blocks),
                     ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))
        self.calls += 1
        return self.residual

    # ---- sequence-parallel form: reduce my rows only, then distribute what I derived from them

    def scatter_args(self, row_offset: int):
        """The ``scatter=`` argument of ``scaled_mm_nvfp4`` for a row-parallel GEMM whose first output row is row
        ``row_offset`` of the group's matrix: its tile rows go straight into the slabs of the ranks that sum them."""
        return (self._scatter_dests, self._scatter_bounds, self.world, int(row_offset))

    def reduce_rows(self, gate0: torch.Tensor, gate1: torch.Tensor | None = None, split_row: int = 0, blocks: int = 0,
                    scattered: bool = False) -> None:
        """residual[row_lo:row_hi] += gate * sum_over_ranks(partial[row_lo:row_hi]) in this rank's buffer only.
        ``scattered``: the partial rows were delivered into this rank's slabs by the peers' GEMMs (scatter_args), so
        the sum reads local memory only; otherwise they are read from the peers' partial buffers."""
        g0 = gate0.reshape(-1)
        g1 = None if gate1 is None else gate1.reshape(-1)
        assert g0.numel() == self.cols and g0.dtype == self.dtype and g0.is_contiguous()
        code = 2 if self.dtype == torch.bfloat16 else 1
        _native.call("launch_tp_reduce_rows_kernel", self._slab_partials if scattered else self._partials, self._residuals,
                     self._pads, self.world, self.rank,
                     ctypes.c_void_p(g0.data_ptr()), ctypes.c_void_p(0 if g1 is None else g1.data_ptr()), int(split_row),
                     self.rows, self.cols, self.row_lo, self.row_hi, code, int(blocks),
                     ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))
        self.calls += 1

    def _gather(self, r0, r1, blocks: int = 0) -> None:
        _native.call("launch_tp_gather_kernel", self._bases, self._pads, self.world, self.rank, r0[0], r0[1], r1[0], r1[1],
                     int(blocks), ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))

    def gather_quantized(self) -> None:
        """Every rank's rows of ``qx`` (codes) and ``sx`` (whole scale tiles) reach every rank's copy."""
        lo, hi = self.row_lo, self.row_hi
        half = self.cols // 2
        tile_lo, tile_hi = lo // 128, (hi + 127) // 128
        self._gather((self._q_off + lo * half, self._q_off + hi * half),
                     (self._sf_off + tile_lo * 128 * self._sf_cols, self._sf_off + tile_hi * 128 * self._sf_cols))

    def gather_extra(self, lo: int, hi: int) -> None:
        """Bytes [lo, hi) (multiples of 16) of this rank's ``extra`` region reach every rank's copy."""
        assert 0 <= lo <= hi <= self._extra_bytes and lo % 16 == 0 and hi % 16 == 0
        self._gather((self._extra_off + lo, self._extra_off + hi), (0, 0))

    def gather_residual(self) -> None:
        """Every rank's rows of the residual stream reach every rank's copy (end of a sequence-parallel forward)."""
        row = self.cols * 2
        self._gather((self._offsets[1] + self.row_lo * row, self._offsets[1] + self.row_hi * row), (0, 0))

    def status(self) -> int:
        """Synchronise and read (then clear) the kernel's status word: 0, or -6 after a wait for a peer ran out."""
        return int(_native.load().ck_tp_device_status())
