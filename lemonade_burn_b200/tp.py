"""Tensor-parallel sharding of packed ternary projections (one process per GPU, torch.distributed).

The reference has no multi-device path; the closest thing is its two-socket row split
(crates/lb-model/src/ops.rs:255-297, crates/lb-ternary/src/numa.rs:122-124), which this
generalises:

* column-parallel (q/k/v, gate, up): each rank holds a contiguous range of the packed ROWS -- no
  repacking, rows are contiguous in the lb-ternary layout (pack.rs:46-49). The input is
  replicated, every rank quantises the whole token row itself (identical on all ranks), outputs
  are sharded along features. No collective.
* row-parallel (o, down): each rank holds a range of the COLUMNS, a multiple of 128 so that the
  cut falls on packed-block boundaries (a contiguous byte range of every row, copied once at
  load). Per-token quantisation needs the maximum over the whole row, so ranks all-reduce (MAX)
  their slice maxima first; then every rank has the same scale, quantises its slice, computes
  exact int32 partial dots, and the partial dots are all-reduced with an integer SUM, which is
  exact and order independent. The scale epilogue runs after the reduction. Results are
  bit-identical to the single-GPU op for any world size.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import numpy as np

from .pack import BLOCK, row_bytes


# ---- pure host-side slicing (numpy or torch tensors; no GPU needed) -----------------------

def shard_rows(packed, world: int, rank: int):
    """Rows [rank*rows/world, (rank+1)*rows/world) of a packed [rows, row_bytes] matrix."""
    rows = packed.shape[0]
    if rows % world:
        raise ValueError(f"{rows} rows do not divide over {world} ranks")
    n = rows // world
    return packed[rank * n:(rank + 1) * n]


def shard_cols(packed, cols: int, world: int, rank: int):
    """Columns [rank*cols/world, (rank+1)*cols/world) of a packed matrix as a packed matrix of
    cols/world columns: a byte range of every row. Returns (slice view, local cols)."""
    if cols % world or (cols // world) % BLOCK:
        raise ValueError(f"{cols} columns over {world} ranks do not fall on 128-column blocks")
    if packed.shape[1] != row_bytes(cols):
        raise ValueError("packed data length mismatch")
    lc = cols // world
    lb = lc // 4
    return packed[:, rank * lb:(rank + 1) * lb], lc


# ---- peer-memory communicator for the fused row-parallel kernels --------------------------------

class TpComm:
    """One region of device memory per rank, opened in every rank through CUDA IPC handles that
    travel over the torch.distributed group (any transport would do), for lbk_tp_quantize /
    lbk_tp_reduce_scale. Plain NVLink peer loads and stores; NCCL is not involved in the data path."""

    def __init__(self, ctx, world: int, rank: int, group=None):
        import torch.distributed as dist
        from . import _lib
        self.ctx, self.world, self.rank = ctx, world, rank
        lib = ctx._lib
        self._lib = lib
        self.max_tokens = int(lib.lbk_tp_max_tokens())
        self.partial_bytes = int(lib.lbk_tp_partial_bytes())
        mine = C.c_void_p()
        handle = (C.c_ubyte * 64)()
        _lib.check(lib.lbk_tp_region_alloc(ctx.handle, C.byref(mine), handle))
        self._mine = mine
        handles = [None] * world
        if world > 1:
            dist.all_gather_object(handles, bytes(handle), group=group)
        else:
            handles[0] = bytes(handle)
        self._opened = []
        regions = []
        for r in range(world):
            if r == rank:
                regions.append(mine.value)
                continue
            ptr = C.c_void_p()
            buf = (C.c_ubyte * 64).from_buffer_copy(handles[r])
            _lib.check(lib.lbk_tp_region_open(ctx.handle, buf, C.byref(ptr)))
            self._opened.append(ptr)
            regions.append(ptr.value)
        arr, self._keep = _lib.ptr_array(regions)
        h = C.c_void_p()
        _lib.check(lib.lbk_tp_comm_create(ctx.handle, world, rank, arr, C.byref(h)))
        self.handle = h
        self.partial_ptr = int(lib.lbk_tp_partial_buffer(h))
        if world > 1:
            dist.barrier(group=group)  # every rank has opened every region before anyone launches

    def close(self):
        """Call on every rank once no kernel of the group is in flight."""
        if getattr(self, "handle", None):
            self._lib.lbk_tp_comm_destroy(self.handle)
            self.handle = None
            for ptr in self._opened:
                self._lib.lbk_tp_region_close(self.ctx.handle, ptr)
            self._lib.lbk_tp_region_free(self.ctx.handle, self._mine)


# ---- device-resident layers -------------------------------------------------------------------

class ColumnParallelTernary:
    """One or several matrices sharing an input (q/k/v, gate/up), rows split across ranks."""

    def __init__(self, packed_list, scales, cols: int, world: int, rank: int, ctx=None):
        import torch
        from . import ops
        self.lins = [ops.TernaryLinear(shard_rows(p, world, rank).contiguous().cuda() if isinstance(p, torch.Tensor)
                                       else torch.from_numpy(np.ascontiguousarray(shard_rows(p, world, rank))).cuda(),
                                       float(s), cols, ctx) for p, s in zip(packed_list, scales)]

    def forward(self, x):
        from . import ops
        return ops.ternary_linear_multi(x, self.lins)


class RowParallelTernary:
    """One matrix with its columns split across ranks; forward returns the full [m, rows] output
    on every rank after an exact integer all-reduce."""

    def __init__(self, packed, scale: float, cols: int, world: int, rank: int, group=None, ctx=None, comm: Optional[TpComm] = None):
        import torch
        from . import ops
        self.comm = comm  # with a TpComm, small batches take the two fused peer-memory kernels instead of NCCL
        sl, self.local_cols = shard_cols(packed, cols, world, rank)
        dev = sl.contiguous().cuda() if isinstance(sl, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(sl)).cuda()
        self.lin = ops.TernaryLinear(dev, float(scale), self.local_cols, ctx)
        self.world, self.group = world, group
        self.rows, self.scale = self.lin.rows, float(scale)
        self.ctx = self.lin.ctx

    def forward(self, x_local):
        """x_local: f32 CUDA [m, cols/world], this rank's column slice of the input."""
        import torch
        import torch.distributed as dist
        from . import _lib
        if x_local.dtype != torch.float32 or x_local.dim() != 2 or x_local.shape[1] != self.local_cols:
            raise ValueError("inner dimension mismatch")
        x_local = x_local.contiguous()
        m = x_local.shape[0]
        lib, h = self.ctx._lib, self.ctx.handle
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        dev = x_local.device
        if (self.comm is not None and self.world > 1 and 0 < m <= self.comm.max_tokens and self.rows % 4 == 0
                and m * self.rows * 4 <= self.comm.partial_bytes):
            return self._forward_fused(x_local, m, st, dev)
        amax = torch.empty(m, dtype=torch.float32, device=dev)
        _lib.check(lib.lbk_absmax_dev(h, C.c_void_p(x_local.data_ptr()), m, self.local_cols, C.c_void_p(amax.data_ptr()), st))
        if self.world > 1:
            dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=self.group)
        kp = (self.local_cols + BLOCK - 1) // BLOCK * BLOCK
        q = torch.empty((m, kp), dtype=torch.int8, device=dev)
        scale = torch.empty(m, dtype=torch.float32, device=dev)
        ssum = torch.empty(m, dtype=torch.int32, device=dev)
        _lib.check(lib.lbk_quantize_acts_amax_dev(h, C.c_void_p(x_local.data_ptr()), m, self.local_cols,
                                                  C.c_void_p(amax.data_ptr()), C.c_void_p(q.data_ptr()),
                                                  C.c_void_p(scale.data_ptr()), C.c_void_p(ssum.data_ptr()), st))
        dots = torch.empty((m, self.rows), dtype=torch.int32, device=dev)
        wp, _k1 = _lib.ptr_array([self.lin.weight.handle.value])
        ip, _k2 = _lib.ptr_array([dots.data_ptr()])
        _lib.check(lib.lbk_ternary_gemm_dev(h, wp, 1, C.c_void_p(q.data_ptr()), None, C.c_void_p(ssum.data_ptr()), m,
                                            None, ip, st))
        if self.world > 1:
            dist.all_reduce(dots, op=dist.ReduceOp.SUM, group=self.group)
        out = torch.empty((m, self.rows), dtype=torch.float32, device=dev)
        _lib.check(lib.lbk_scale_epilogue_dev(h, C.c_void_p(dots.data_ptr()), C.c_void_p(scale.data_ptr()),
                                              C.c_float(self.scale), m, self.rows, C.c_void_p(out.data_ptr()), st))
        return out, dots

    def _forward_fused(self, x_local, m, st, dev):
        """quantise with the all-rank maximum (one kernel) -> int32 partial dots into this rank's
        region -> sum of all ranks' dots + scale (one kernel)."""
        import torch
        from . import _lib
        lib, h, comm = self.ctx._lib, self.ctx.handle, self.comm
        kp = (self.local_cols + BLOCK - 1) // BLOCK * BLOCK
        q = torch.empty((m, kp), dtype=torch.int8, device=dev)
        scale = torch.empty(m, dtype=torch.float32, device=dev)
        ssum = torch.empty(m, dtype=torch.int32, device=dev)
        _lib.check(lib.lbk_tp_quantize(comm.handle, C.c_void_p(x_local.data_ptr()), m, self.local_cols, C.c_void_p(q.data_ptr()),
                                       C.c_void_p(scale.data_ptr()), C.c_void_p(ssum.data_ptr()), st))
        wp, _k1 = _lib.ptr_array([self.lin.weight.handle.value])
        ip, _k2 = _lib.ptr_array([comm.partial_ptr])
        _lib.check(lib.lbk_ternary_gemm_dev(h, wp, 1, C.c_void_p(q.data_ptr()), None, C.c_void_p(ssum.data_ptr()), m, None, ip, st))
        out = torch.empty((m, self.rows), dtype=torch.float32, device=dev)
        dots = torch.empty((m, self.rows), dtype=torch.int32, device=dev)
        _lib.check(lib.lbk_tp_reduce_scale(comm.handle, C.c_void_p(scale.data_ptr()), C.c_float(self.scale), m, self.rows,
                                           C.c_void_p(out.data_ptr()), C.c_void_p(dots.data_ptr()), st))
        return out, dots
