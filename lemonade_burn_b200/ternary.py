"""Host mirror of lb-ternary's public API over the CUDA C ABI (numpy host buffers).

Same names, argument meaning and error behaviour as the Rust crate
(crates/lb-ternary/src/lib.rs:19-21): `quantize_acts`, `QuantActs`, `ternary_gemm_i32`,
`ternary_gemm`, `ternary_gemm_multi`, `bf16_gemv`, `Kernel`. Where the reference asserts
(shape mismatch), these raise. Every call goes to the GPU through liblbk.so; there is no
CPU path here.
"""
from __future__ import annotations

import ctypes as C
import enum
import os
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np

from . import _lib
from .pack import PackedTernary, TernaryView, padded_cols, row_bytes


class Kernel(enum.Enum):
    """Kernel selector (crates/lb-ternary/src/gemm.rs:25-92). The reference picks a CPU ISA;
    here there is exactly one implementation, the sm_100a CUDA path."""
    Sm100 = "sm100"

    def name_str(self) -> str:
        return self.value

    @staticmethod
    def parse(s: str) -> Optional["Kernel"]:
        return Kernel.Sm100 if s in ("sm100", "sm_100a", "cuda") else None

    @staticmethod
    def available() -> List["Kernel"]:
        return [Kernel.Sm100]

    @staticmethod
    def detect() -> "Kernel":
        """`LB_KERNEL` is honoured as in gemm.rs:76-91; any value but the CUDA path is
        reported and ignored (there is nothing else to fall back to)."""
        want = os.environ.get("LB_KERNEL")
        if want is not None and Kernel.parse(want) is None:
            import sys
            print(f"lb-ternary: LB_KERNEL={want} not usable here, using sm100", file=sys.stderr)
        return Kernel.Sm100


class Context:
    """One lbk context (one CUDA device)."""

    def __init__(self, device: int = 0):
        self._lib = _lib.load()
        h = C.c_void_p()
        _lib.check(self._lib.lbk_init(device, C.byref(h)))
        self.handle = h
        self.device = device

    def close(self):
        if getattr(self, "handle", None):
            self._lib.lbk_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check_device_error(self):
        _lib.check(self._lib.lbk_check_device_error(self.handle))

    def launch_count(self) -> int:
        return int(self._lib.lbk_launch_count(self.handle))

    def int8_peak_tops(self, token_rows: int = 192, iterations: int = 20000) -> float:
        """Measured rate of the int8 tensor-core instruction with resident operands (lbk_int8_peak_probe)."""
        out = C.c_double()
        _lib.check(self._lib.lbk_int8_peak_probe(self.handle, token_rows, iterations, C.byref(out)))
        return float(out.value)

    def set_gemv_rows(self, rows: int) -> None:
        """0: the measured rule decides between the fused few-row kernel and quantise + GEMM;
        n: the fused kernel takes every call of at most n token rows (same bits either way)."""
        _lib.check(self._lib.lbk_set_gemv_rows(self.handle, rows))


_default_ctx: Optional[Context] = None


def default_context() -> Context:
    global _default_ctx
    if _default_ctx is None:
        _default_ctx = Context(0)
    return _default_ctx


class DeviceWeight:
    """A packed matrix uploaded to the GPU (lbk_weight). Built from a TernaryView."""

    def __init__(self, view: TernaryView, ctx: Optional[Context] = None):
        self.ctx = ctx or default_context()
        self.rows, self.cols, self.scale = view.rows, view.cols, float(view.scale)
        h = C.c_void_p()
        data = np.ascontiguousarray(view.data, dtype=np.uint8)
        _lib.check(self.ctx._lib.lbk_weight_upload(self.ctx.handle, view.rows, view.cols,
                                                   data.ctypes.data, data.size, C.c_float(view.scale), C.byref(h)))
        self.handle = h

    @classmethod
    def wrap(cls, ctx: Context, rows: int, cols: int, dev_ptr: int, scale: float) -> "DeviceWeight":
        """Borrow device memory that already holds packed rows (lbk_weight_wrap)."""
        self = cls.__new__(cls)
        self.ctx, self.rows, self.cols, self.scale = ctx, rows, cols, float(scale)
        h = C.c_void_p()
        _lib.check(ctx._lib.lbk_weight_wrap(ctx.handle, rows, cols, C.c_void_p(dev_ptr), C.c_float(scale), C.byref(h)))
        self.handle = h
        return self

    def data_ptr(self) -> int:
        return int(self.ctx._lib.lbk_weight_data(self.handle) or 0)

    def close(self):
        if getattr(self, "handle", None):
            self.ctx._lib.lbk_weight_free(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _as_device(w, ctx: Context) -> DeviceWeight:
    if isinstance(w, DeviceWeight):
        return w
    if isinstance(w, PackedTernary):
        w = w.view()
    return DeviceWeight(w, ctx)


@dataclass
class QuantActs:
    """crates/lb-ternary/src/quant.rs:19-34"""
    m: int
    k: int
    kp: int
    q: np.ndarray      # int8 [m * kp], zero padded rows
    scale: np.ndarray  # f32 [m] = 127 / max|x|
    sum: np.ndarray    # i32 [m] = sum of q per row

    def row(self, i: int) -> np.ndarray:
        return self.q[i * self.kp:(i + 1) * self.kp]


def quantize_acts(x, m: int, k: int, ctx: Optional[Context] = None) -> QuantActs:
    """quantize_acts (quant.rs:37-75) on the GPU."""
    ctx = ctx or default_context()
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    if x.size != m * k:  # quant.rs:46
        raise ValueError(f"x has {x.size} elements, expected m*k = {m * k}")
    kp = padded_cols(k)
    q = np.zeros(m * kp, dtype=np.int8)
    scale = np.zeros(m, dtype=np.float32)
    ssum = np.zeros(m, dtype=np.int32)
    _lib.check(ctx._lib.lbk_quantize_acts(ctx.handle, x.ctypes.data, m, k, q.ctypes.data, scale.ctypes.data, ssum.ctypes.data))
    return QuantActs(m, k, kp, q, scale, ssum)


def _check(w, x: QuantActs):
    """gemm.rs:197-200"""
    if w.cols != x.k:
        raise ValueError("inner dimension mismatch")
    if padded_cols(w.cols) != x.kp:
        raise ValueError("padded width mismatch")


def ternary_gemm_i32(w, x: QuantActs, kernel: Kernel = Kernel.Sm100, ctx: Optional[Context] = None) -> np.ndarray:
    """ternary_gemm_i32 (gemm.rs:95-114): exact out[t*rows + r] = sum_k w[r,k] * q[t,k]."""
    ctx = ctx or default_context()
    _check(w, x)
    dw = _as_device(w, ctx)
    out = np.zeros(x.m * dw.rows, dtype=np.int32)
    _lib.check(ctx._lib.lbk_ternary_gemm_i32(ctx.handle, dw.handle, x.q.ctypes.data, x.sum.ctypes.data, x.m, out.ctypes.data))
    return out


def ternary_gemm_multi(ws: Sequence, x: QuantActs, kernel: Kernel, outs: Sequence[np.ndarray],
                       ctx: Optional[Context] = None) -> None:
    """ternary_gemm_multi (gemm.rs:128-195): outs[i][t*rows_i + r] = (x @ ws[i]^T)[t, r]."""
    ctx = ctx or default_context()
    if len(ws) != len(outs):  # gemm.rs:129
        raise ValueError("ws and outs differ in length")
    dws = []
    for w, o in zip(ws, outs):
        _check(w, x)
        if o.size != x.m * w.rows or o.dtype != np.float32 or not o.flags.c_contiguous:  # gemm.rs:133
            raise ValueError("output buffer has the wrong size/dtype")
        dws.append(_as_device(w, ctx))
    wp, _keep1 = _lib.ptr_array([d.handle.value for d in dws])
    op, _keep2 = _lib.ptr_array([o.ctypes.data for o in outs])
    _lib.check(ctx._lib.lbk_ternary_gemm_multi(ctx.handle, wp, len(dws), x.q.ctypes.data, x.scale.ctypes.data,
                                               x.sum.ctypes.data, x.m, op))


def ternary_gemm(w, x: QuantActs, kernel: Kernel, out: np.ndarray, ctx: Optional[Context] = None) -> None:
    """ternary_gemm (gemm.rs:117-119)."""
    ternary_gemm_multi([w], x, kernel, [out], ctx)


def ternary_linear_host(x: np.ndarray, ws: Sequence, want_i32: bool = False, ctx: Optional[Context] = None):
    """The fused op on host buffers (crates/lb-model/src/ops.rs:301-329): quantise x once,
    run every matrix. Returns (list of f32 [m, rows_i], list of i32 or None)."""
    ctx = ctx or default_context()
    x = np.ascontiguousarray(x, dtype=np.float32)
    if x.ndim != 2:
        raise ValueError("expected a rank-2 tensor")  # ops.rs:104
    m, k = x.shape
    dws = [_as_device(w, ctx) for w in ws]
    for d in dws:
        if d.cols != k:  # ops.rs:308
            raise ValueError("inner dimension mismatch")
    outs = [np.zeros((m, d.rows), dtype=np.float32) for d in dws]
    iouts = [np.zeros((m, d.rows), dtype=np.int32) for d in dws] if want_i32 else None
    wp, _k1 = _lib.ptr_array([d.handle.value for d in dws])
    op, _k2 = _lib.ptr_array([o.ctypes.data for o in outs])
    ip, _k3 = _lib.ptr_array([o.ctypes.data for o in iouts]) if iouts else (None, None)
    _lib.check(ctx._lib.lbk_ternary_linear_host(ctx.handle, x.ctypes.data, m, wp, len(dws), op, ip))
    return outs, iouts


def bf16_gemv(w: np.ndarray, rows: int, cols: int, x: np.ndarray, out: np.ndarray,
              kernel: Kernel = Kernel.Sm100, ctx: Optional[Context] = None) -> None:
    """bf16_gemv (crates/lb-ternary/src/bf16.rs:14-27): w is raw bf16 bits [rows*cols]."""
    ctx = ctx or default_context()
    w = np.ascontiguousarray(w, dtype=np.uint16).reshape(-1)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    if w.size != rows * cols or x.size != cols or out.size != rows:  # bf16.rs:15-17
        raise ValueError("bf16_gemv: size mismatch")
    _lib.check(ctx._lib.lbk_bf16_gemv_host(ctx.handle, w.ctypes.data, rows, cols, x.ctypes.data, out.ctypes.data))
