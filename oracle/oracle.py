"""ctypes/numpy front end of the CPU oracle (test infrastructure only).

Only the tests, the smoke check and the benchmark's CPU-baseline leg may import this
module. The product package never does: it fails loudly when its CUDA library is missing
instead of falling back to anything in here.

Each function forwards to the plain-C restatement in ``lbt_oracle.c`` (scalar definition,
following crates/lb-ternary/src/{pack,quant,gemm,bf16}.rs and
crates/ternary-kernels/src/{pack,quant,reference}.rs) or to the threaded SIMD port in
``lbt_simd.c`` (the timed CPU baseline, following crates/lb-ternary/src/gemm.rs:364-588).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "_build" / "liblbt_oracle.so"

BLOCK = 128
BLOCK_BYTES = 32


def build(force: bool = False) -> Path:
    """Compile the oracle with the committed Makefile (gcc)."""
    srcs = [_HERE / n for n in ("lbt_oracle.c", "lbt_simd.c", "lbt_testgen.c", "lbt_oracle.h", "Makefile")]
    stale = not _SO.exists() or any(s.stat().st_mtime > _SO.stat().st_mtime for s in srcs)
    if force or stale:
        env = dict(os.environ)
        env.pop("CC", None)
        subprocess.run(["make", "-C", str(_HERE), "-B"], check=True, env=env,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not _SO.exists():
            build()
        _lib = C.CDLL(str(_SO))
        _lib.lbt_padded_cols.restype = C.c_size_t
        _lib.lbt_padded_cols.argtypes = [C.c_size_t]
        _lib.lbt_absmean_f32.restype = C.c_float
        _lib.lbt_ternarize_absmean.restype = C.c_float
        _lib.lbt_argmax.restype = C.c_uint32
        _lib.lbt_simd_kernel_name.restype = C.c_char_p
        _lib.lbt_gen_xorshift_next.restype = C.c_uint64
        _lib.lbt_gen_xorshift_f.restype = C.c_float
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def padded_cols(cols: int) -> int:
    return (cols + BLOCK - 1) // BLOCK * BLOCK


def row_bytes(cols: int) -> int:
    return padded_cols(cols) // 4


# ---- pack.rs --------------------------------------------------------------------------

def pack_matrix(values: np.ndarray) -> np.ndarray:
    """PackedTernary::from_ternary (pack.rs:69-78): int8 [rows, cols] -> u8 [rows, rb]."""
    values = np.ascontiguousarray(values, dtype=np.int8)
    rows, cols = values.shape
    out = np.empty((rows, row_bytes(cols)), dtype=np.uint8)
    lib().lbt_pack_matrix(_p(values), C.c_size_t(rows), C.c_size_t(cols), _p(out))
    return out


def tk_pack_ternary(values: np.ndarray) -> np.ndarray:
    """ternary-kernels pack_ternary (pack.rs:46-69), the second statement of the layout."""
    values = np.ascontiguousarray(values, dtype=np.int8)
    n, k = values.shape
    out = np.empty((n, row_bytes(k)), dtype=np.uint8)
    lib().lbt_tk_pack_ternary(_p(values), C.c_size_t(n), C.c_size_t(k), _p(out))
    return out


def unpack_matrix(packed: np.ndarray, cols: int, tk: bool = False) -> np.ndarray:
    """unpack_row per row (pack.rs:106-116 or ternary-kernels pack.rs:72-81), padded width."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    rows = packed.shape[0]
    kp = padded_cols(cols)
    out = np.empty((rows, kp), dtype=np.int8)
    fn = lib().lbt_tk_unpack_row if tk else lib().lbt_unpack_row
    for r in range(rows):
        fn(_p(packed[r]), C.c_size_t(kp), _p(out[r]))
    return out


def absmean_f32(w: np.ndarray) -> float:
    w = np.ascontiguousarray(w, dtype=np.float32).ravel()
    return float(lib().lbt_absmean_f32(_p(w), C.c_size_t(w.size)))


def ternarize_absmean(w: np.ndarray):
    """pack.rs:129-142 -> (int8 values of w's shape, f32 scale = 1/max(mean|w|,1e-5))."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    out = np.empty(w.shape, dtype=np.int8)
    s = lib().lbt_ternarize_absmean(_p(w), C.c_size_t(w.size), _p(out))
    return out, np.float32(s)


def ternarize_with_scale(w: np.ndarray, scale: float) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.float32)
    out = np.empty(w.shape, dtype=np.int8)
    lib().lbt_ternarize_with_scale(_p(w), C.c_size_t(w.size), C.c_float(scale), _p(out))
    return out


# ---- quant.rs -------------------------------------------------------------------------

def quantize_acts(x: np.ndarray):
    """quantize_acts (quant.rs:37-75): f32 [m,k] -> (q int8 [m,kp], scale f32[m], sum i32[m])."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    kp = padded_cols(k)
    q = np.empty((m, kp), dtype=np.int8)
    scale = np.empty(m, dtype=np.float32)
    ssum = np.empty(m, dtype=np.int32)
    lib().lbt_quantize_acts(_p(x), C.c_size_t(m), C.c_size_t(k), _p(q), _p(scale), _p(ssum))
    return q, scale, ssum


# ---- gemm.rs / reference.rs -----------------------------------------------------------

def ternary_gemm_i32(packed: np.ndarray, cols: int, q: np.ndarray, ssum: np.ndarray) -> np.ndarray:
    """ternary_gemm_i32 (gemm.rs:95-114): exact int32 [m, rows]."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    q = np.ascontiguousarray(q, dtype=np.int8)
    ssum = np.ascontiguousarray(ssum, dtype=np.int32)
    rows, m = packed.shape[0], q.shape[0]
    assert packed.shape[1] == row_bytes(cols) and q.shape[1] == padded_cols(cols)
    out = np.empty((m, rows), dtype=np.int32)
    lib().lbt_ternary_gemm_i32(_p(packed), C.c_size_t(rows), C.c_size_t(cols), _p(q), _p(ssum),
                               C.c_size_t(m), _p(out))
    return out


def gemv_i32_reference(packed: np.ndarray, kp: int, q_row: np.ndarray) -> np.ndarray:
    """gemv_i32_reference (ternary-kernels reference.rs:7-16): one token, unpack every weight."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    q_row = np.ascontiguousarray(q_row, dtype=np.int8)
    n = packed.shape[0]
    out = np.empty(n, dtype=np.int32)
    lib().lbt_gemv_i32_reference(_p(packed), C.c_size_t(n), C.c_size_t(kp), _p(q_row), _p(out))
    return out


def ternary_gemm(packed: np.ndarray, cols: int, wscale: float, q, scale, ssum) -> np.ndarray:
    """ternary_gemm (gemm.rs:117-195): f32 [m, rows] = dot as f32 * (1/(s_a*s_w))."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    q = np.ascontiguousarray(q, dtype=np.int8)
    scale = np.ascontiguousarray(scale, dtype=np.float32)
    ssum = np.ascontiguousarray(ssum, dtype=np.int32)
    rows, m = packed.shape[0], q.shape[0]
    out = np.empty((m, rows), dtype=np.float32)
    lib().lbt_ternary_gemm(_p(packed), C.c_size_t(rows), C.c_size_t(cols), C.c_float(wscale), _p(q),
                           _p(scale), _p(ssum), C.c_size_t(m), _p(out))
    return out


def ternary_linear(x: np.ndarray, packed: np.ndarray, wscale: float, cols: int):
    """The op (ops.rs:301-329) for one matrix: quantize then gemm. Returns (f32, i32)."""
    q, s, ssum = quantize_acts(x)
    return ternary_gemm(packed, cols, wscale, q, s, ssum), ternary_gemm_i32(packed, cols, q, ssum)


def bf16_gemv(w_bits: np.ndarray, x: np.ndarray) -> np.ndarray:
    """bf16_gemv with dot_scalar (bf16.rs:14-51): w u16 [rows, cols], x f32 [cols]."""
    w_bits = np.ascontiguousarray(w_bits, dtype=np.uint16)
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = w_bits.shape
    out = np.empty(rows, dtype=np.float32)
    lib().lbt_bf16_gemv(_p(w_bits), C.c_size_t(rows), C.c_size_t(cols), _p(x), _p(out))
    return out


def argmax(logits: np.ndarray) -> int:
    logits = np.ascontiguousarray(logits, dtype=np.float32).ravel()
    return int(lib().lbt_argmax(_p(logits), C.c_size_t(logits.size)))


# ---- timed SIMD baseline --------------------------------------------------------------

def simd_best_kernel() -> int:
    return int(lib().lbt_simd_best_kernel())


def simd_kernel_name(k: int) -> str:
    return lib().lbt_simd_kernel_name(C.c_int(k)).decode()


def simd_max_threads() -> int:
    return int(lib().lbt_simd_max_threads())


def simd_gemm_multi(packed_list, wscales, q, scale, ssum, kernel=None, threads=0,
                    want_f32=True, want_i32=False):
    """Threaded SIMD port of ternary_gemm_multi (gemm.rs:128-195) on quantised inputs."""
    if kernel is None:
        kernel = simd_best_kernel()
    q = np.ascontiguousarray(q, dtype=np.int8)
    scale = np.ascontiguousarray(scale, dtype=np.float32)
    ssum = np.ascontiguousarray(ssum, dtype=np.int32)
    m, kp = q.shape
    n = len(packed_list)
    packed_list = [np.ascontiguousarray(p, dtype=np.uint8) for p in packed_list]
    rows = (C.c_size_t * n)(*[p.shape[0] for p in packed_list])
    ws = (C.c_float * n)(*[float(w) for w in wscales])
    pp = (C.c_void_p * n)(*[p.ctypes.data for p in packed_list])
    outs = [np.empty((m, p.shape[0]), dtype=np.float32) for p in packed_list] if want_f32 else None
    iouts = [np.empty((m, p.shape[0]), dtype=np.int32) for p in packed_list] if want_i32 else None
    op = (C.c_void_p * n)(*[o.ctypes.data for o in outs]) if outs else None
    ip = (C.c_void_p * n)(*[o.ctypes.data for o in iouts]) if iouts else None
    lib().lbt_simd_gemm_multi(C.c_int(kernel), C.c_int(threads), C.c_size_t(n), pp, rows, ws,
                              C.c_size_t(kp), _p(q), _p(scale), _p(ssum), C.c_size_t(m), op, ip)
    return outs, iouts


def simd_quantize_acts(x: np.ndarray, threads=0):
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    kp = padded_cols(k)
    q = np.empty((m, kp), dtype=np.int8)
    scale = np.empty(m, dtype=np.float32)
    ssum = np.empty(m, dtype=np.int32)
    lib().lbt_simd_quantize_acts(C.c_int(threads), _p(x), C.c_size_t(m), C.c_size_t(k), C.c_size_t(kp),
                                 _p(q), _p(scale), _p(ssum))
    return q, scale, ssum


# ---- the reference tests' seeded generators (lbt_testgen.c) ---------------------------

class GoldenRng:
    """xorshift64 of crates/lb-ternary/tests/golden.rs:12-23."""

    def __init__(self, seed: int):
        self.state = C.c_uint64(seed)

    def next(self) -> int:
        return int(lib().lbt_gen_xorshift_next(C.byref(self.state)))

    def f(self) -> float:
        return float(lib().lbt_gen_xorshift_f(C.byref(self.state)))

    def weights(self, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        lib().lbt_gen_golden_weights(C.byref(self.state), C.c_size_t(n), _p(out))
        return out

    def acts(self, n: int, period: int, phase: int, gain: float) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        lib().lbt_gen_golden_acts(C.byref(self.state), C.c_size_t(n), C.c_size_t(period),
                                  C.c_size_t(phase), C.c_float(gain), _p(out))
        return out

    def ternary(self, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.int8)
        lib().lbt_gen_xorshift_ternary(C.byref(self.state), C.c_size_t(n), _p(out))
        return out


class XssRng:
    """xorshift64* of crates/lb-ternary-gpu/tests/gpu_matches_scalar.rs:8-24."""

    def __init__(self, seed: int):
        self.state = C.c_uint64(seed)

    def ternary(self, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.int8)
        lib().lbt_gen_xss_ternary(C.byref(self.state), C.c_size_t(n), _p(out))
        return out

    def acts(self, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        lib().lbt_gen_xss_acts(C.byref(self.state), C.c_size_t(n), _p(out))
        return out


def golden_case(rows: int, cols: int, m: int, seed: int):
    """Inputs of golden.rs `case` (:25-35): (ternary int8 [rows,cols], wscale, packed, x f32 [m,cols])."""
    rng = GoldenRng(seed)
    wf = rng.weights(rows * cols)
    t, wscale = ternarize_absmean(wf)
    t = t.reshape(rows, cols)
    x = rng.acts(m * cols, 97, 3, 20.0).reshape(m, cols)
    return t, wscale, pack_matrix(t), x


def gpu_case(rows: int, cols: int, m: int, seed: int):
    """Inputs of gpu_matches_scalar.rs `check` (:26-31): (ternary, packed, x)."""
    rng = XssRng(seed)
    t = rng.ternary(rows * cols).reshape(rows, cols)
    x = rng.acts(m * cols).reshape(m, cols)
    return t, pack_matrix(t), x
