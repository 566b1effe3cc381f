"""Device-resident ops on torch CUDA tensors: the B200 side of lb-model's op boundary.

Mirrors `ternary_linear`, `ternary_linear2`, `ternary_linear3`, `bf16_linear`
(crates/lb-model/src/ops.rs:332-397) and `TernaryLinear` (crates/lb-model/src/model.rs:38-83).
torch is used for device memory and streams only; all arithmetic is in liblbk.so.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from . import _lib
from .pack import row_bytes
from .ternary import Context, DeviceWeight, default_context


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


class TernaryLinear:
    """A packed ternary projection resident on the GPU (model.rs:38-63).

    `packed` is a uint8 CUDA tensor [rows, row_bytes(cols)] in the lb-ternary layout (what
    `<linear>.qweight` holds in model.lbt.safetensors); `scale` is `<linear>.wscale`."""

    def __init__(self, packed: torch.Tensor, scale: float, cols: int, ctx: Optional[Context] = None):
        if packed.dtype != torch.uint8:  # ops.rs:228
            raise TypeError("ternary_linear expects u8 packed weights")
        if packed.dim() != 2:
            raise ValueError("expected a rank-2 tensor")
        if not packed.is_cuda:
            raise ValueError("packed weights must live on the GPU")
        self.ctx = ctx or default_context()
        self.packed = packed.contiguous()
        self.rows = int(packed.shape[0])
        self.cols = int(cols)
        self.scale = float(scale)
        if packed.shape[1] != row_bytes(cols):  # pack.rs:40
            raise ValueError("packed data length mismatch")
        self.weight = DeviceWeight.wrap(self.ctx, self.rows, self.cols, self.packed.data_ptr(), self.scale)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ternary_linear_multi(x, [self])[0]

    __call__ = forward


def ternary_linear_multi(x: torch.Tensor, linears: Sequence[TernaryLinear], want_i32: bool = False):
    """flex_ternary_multi (ops.rs:301-329): quantise `x` once, one fused launch over all
    matrices. x: f32 CUDA [m, cols]. Returns a list of f32 [m, rows_i] (and the exact int32
    dots when want_i32)."""
    if x.dtype != torch.float32:  # ops.rs:306
        raise TypeError("ternary_linear expects f32 activations")
    if x.dim() != 2:
        raise ValueError("expected a rank-2 tensor")
    ctx = linears[0].ctx
    x = x.contiguous()
    m, k = x.shape
    for l in linears:
        if l.cols != k:  # ops.rs:308
            raise ValueError("inner dimension mismatch")
    outs = [torch.empty((m, l.rows), dtype=torch.float32, device=x.device) for l in linears]
    iouts = [torch.empty((m, l.rows), dtype=torch.int32, device=x.device) for l in linears] if want_i32 else None
    wp, _k1 = _lib.ptr_array([l.weight.handle.value for l in linears])
    op, _k2 = _lib.ptr_array([o.data_ptr() for o in outs])
    ip, _k3 = _lib.ptr_array([o.data_ptr() for o in iouts]) if iouts else (None, None)
    _lib.check(ctx._lib.lbk_ternary_linear_n(ctx.handle, C.c_void_p(x.data_ptr()), m, wp, len(linears), op, ip,
                                             C.c_void_p(_stream_ptr())))
    return (outs, iouts) if want_i32 else outs


PRE_RMS, PRE_ADD_RMS, PRE_RELU2_MUL_RMS = 1, 2, 3


def pre_supported(m: int, cols: int) -> bool:
    """Whether ternary_linear_pre can take m token rows of `cols` columns."""
    return bool(_lib.load().lbk_ternary_linear_pre_supported(m, cols))


def ternary_linear_pre(pre: int, x: torch.Tensor, y: Optional[torch.Tensor], w: torch.Tensor, eps: float,
                       linears: Sequence[TernaryLinear], xout: Optional[torch.Tensor] = None) -> List[torch.Tensor]:
    """The projection group of ternary_linear_multi with the decoder step's element-wise work in
    front of it done by the same kernel (model.rs:331-366): PRE_RMS rms_norm(x)*w, PRE_ADD_RMS
    rms_norm(x + y)*w with x + y stored in `xout`, PRE_RELU2_MUL_RMS rms_norm(relu(x)^2 * y)*w."""
    ctx = linears[0].ctx
    m, k = x.shape
    outs = [torch.empty((m, l.rows), dtype=torch.float32, device=x.device) for l in linears]
    wp, _k1 = _lib.ptr_array([l.weight.handle.value for l in linears])
    op, _k2 = _lib.ptr_array([o.data_ptr() for o in outs])
    ptr = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None
    _lib.check(ctx._lib.lbk_ternary_linear_pre(ctx.handle, pre, ptr(x), ptr(y), ptr(w), C.c_float(eps), ptr(xout), m, wp,
                                               len(linears), op, None, C.c_void_p(_stream_ptr())))
    return outs


def norm_quant_supported(width: int) -> bool:
    return bool(_lib.load().lbk_norm_quant_supported(width))


def norm_quant(pre: int, x: torch.Tensor, y: Optional[torch.Tensor], w: torch.Tensor, eps: float, q8: torch.Tensor,
               scale: torch.Tensor, qsum: torch.Tensor, ctx: Optional[Context] = None) -> None:
    """The norm in front of a projection (PRE_* as for ternary_linear_pre; PRE_ADD_RMS updates x) with
    the activation quantiser inside: fills q8 int8 [m, padded(k)], scale [m], qsum [m] for ternary_gemm_q."""
    ctx = ctx or default_context()
    m, k = x.shape
    ptr = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None
    _lib.check(ctx._lib.lbk_norm_quant(ctx.handle, pre, ptr(x), ptr(y), ptr(w), m, k, C.c_float(eps), ptr(q8), ptr(scale), ptr(qsum),
                                       C.c_void_p(_stream_ptr())))


def ternary_gemm_q(q8: torch.Tensor, scale: torch.Tensor, qsum: torch.Tensor, m: int,
                   linears: Sequence[TernaryLinear]) -> List[torch.Tensor]:
    """ternary_gemm_multi (gemm.rs:128-195) on rows that are quantised already (norm_quant)."""
    ctx = linears[0].ctx
    outs = [torch.empty((m, l.rows), dtype=torch.float32, device=q8.device) for l in linears]
    wp, _k1 = _lib.ptr_array([l.weight.handle.value for l in linears])
    op, _k2 = _lib.ptr_array([o.data_ptr() for o in outs])
    _lib.check(ctx._lib.lbk_ternary_gemm_dev(ctx.handle, wp, len(linears), C.c_void_p(q8.data_ptr()), C.c_void_p(scale.data_ptr()),
                                             C.c_void_p(qsum.data_ptr()), m, op, None, C.c_void_p(_stream_ptr())))
    return outs


def ternary_linear(x: torch.Tensor, lin: TernaryLinear) -> torch.Tensor:
    """ops.rs:332-339"""
    return ternary_linear_multi(x, [lin])[0]


def ternary_linear2(x: torch.Tensor, p: Sequence[TernaryLinear]) -> List[torch.Tensor]:
    """ops.rs:342-345 (gate/up)"""
    if len(p) != 2:
        raise ValueError("ternary_linear2 takes two matrices")
    return ternary_linear_multi(x, p)


def ternary_linear3(x: torch.Tensor, p: Sequence[TernaryLinear]) -> List[torch.Tensor]:
    """ops.rs:348-358 (q/k/v)"""
    if len(p) != 3:
        raise ValueError("ternary_linear3 takes three matrices")
    return ternary_linear_multi(x, p)


def bf16_linear(x: torch.Tensor, w: torch.Tensor, ctx: Optional[Context] = None) -> torch.Tensor:
    """ops.rs:391-397 / 199-218: x f32 [m, k] @ w^T with w bf16 [n, k] -> f32 [m, n]."""
    ctx = ctx or default_context()
    if x.dtype != torch.float32:
        raise TypeError("bf16_linear expects f32 activations")
    if w.dtype != torch.bfloat16:  # ops.rs:204
        raise TypeError("bf16_linear expects bf16 weights")
    if x.dim() != 2 or w.dim() != 2:
        raise ValueError("expected rank-2 tensors")
    if x.shape[1] != w.shape[1]:  # ops.rs:207
        raise ValueError("inner dimension mismatch")
    x, w = x.contiguous(), w.contiguous()
    m, k = x.shape
    n = w.shape[0]
    out = torch.empty((m, n), dtype=torch.float32, device=x.device)
    _lib.check(ctx._lib.lbk_bf16_linear(ctx.handle, C.c_void_p(x.data_ptr()), m, C.c_void_p(w.data_ptr()), n, k,
                                        C.c_void_p(out.data_ptr()), C.c_void_p(_stream_ptr())))
    return out


class Plan:
    """A recorded sequence of fused decode groups replayed with one call (lbk_plan_*)."""

    def __init__(self, ctx: Optional[Context] = None):
        self.ctx = ctx or default_context()
        h = C.c_void_p()
        _lib.check(self.ctx._lib.lbk_plan_create(self.ctx.handle, C.byref(h)))
        self.handle = h
        self._keep = []

    def add(self, x: torch.Tensor, linears: Sequence[TernaryLinear], outs: Sequence[torch.Tensor],
            iouts: Optional[Sequence[torch.Tensor]] = None):
        if x.dtype != torch.float32 or x.numel() != linears[0].cols:
            raise ValueError("plan groups take one f32 token row of `cols` elements")
        wp, k1 = _lib.ptr_array([l.weight.handle.value for l in linears])
        op, k2 = _lib.ptr_array([o.data_ptr() for o in outs])
        ip, k3 = _lib.ptr_array([o.data_ptr() for o in iouts]) if iouts else (None, None)
        _lib.check(self.ctx._lib.lbk_plan_add(self.handle, C.c_void_p(x.data_ptr()), wp, len(linears), op, ip))
        self._keep.append((x, list(linears), list(outs), list(iouts) if iouts else None))

    def add_arena(self, linears: Sequence[TernaryLinear]):
        """Append a group whose input row and outputs live in the plan's own arenas."""
        wp, k1 = _lib.ptr_array([l.weight.handle.value for l in linears])
        _lib.check(self.ctx._lib.lbk_plan_add(self.handle, None, wp, len(linears), None, None))
        self._keep.append((None, list(linears), None, None))

    def run_host(self, x_host: torch.Tensor, y_host: torch.Tensor):
        """One step on host buffers (pinned for speed): H2D inputs, run, D2H outputs, sync."""
        _lib.check(self.ctx._lib.lbk_plan_run_host(self.handle, C.c_void_p(x_host.data_ptr()), x_host.numel(),
                                                   C.c_void_p(y_host.data_ptr()), y_host.numel(),
                                                   C.c_void_p(_stream_ptr())))

    def input_elems(self) -> int:
        return int(self.ctx._lib.lbk_plan_input_elems(self.handle))

    def output_elems(self) -> int:
        return int(self.ctx._lib.lbk_plan_output_elems(self.handle))

    def input_arena_ptr(self) -> int:
        return int(self.ctx._lib.lbk_plan_input_arena(self.handle) or 0)

    def output_arena_ptr(self) -> int:
        return int(self.ctx._lib.lbk_plan_output_arena(self.handle) or 0)

    def finalize(self):
        _lib.check(self.ctx._lib.lbk_plan_finalize(self.handle))

    def run(self):
        _lib.check(self.ctx._lib.lbk_plan_run(self.handle, C.c_void_p(_stream_ptr())))

    def weight_bytes(self) -> int:
        return int(self.ctx._lib.lbk_plan_weight_bytes(self.handle))

    def close(self):
        if getattr(self, "handle", None):
            self.ctx._lib.lbk_plan_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
