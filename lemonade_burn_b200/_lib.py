"""ctypes binding of liblbk.so, the C ABI declared in include/lbk.h.

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "liblbk.so"

LBK_OK = 0
STATUS_NAMES = {0: "OK", 1: "INVALID", 2: "SHAPE", 3: "CUDA", 4: "UNSUPPORTED", 5: "TIMEOUT", 6: "NOMEM"}
MAX_GROUP = 4
GEMV_MAX_M = 16

# Every symbol include/lbk.h declares: (name, restype, argtypes)
_vp, _sz, _i, _f = C.c_void_p, C.c_size_t, C.c_int, C.c_float
_pp = C.POINTER(C.c_void_p)
SYMBOLS = [
    ("lbk_last_error", C.c_char_p, []),
    ("lbk_abi_version", _i, []),
    ("lbk_init", _i, [_i, _pp]),
    ("lbk_destroy", _i, [_vp]),
    ("lbk_check_device_error", _i, [_vp]),
    ("lbk_launch_count", C.c_uint64, [_vp]),
    ("lbk_set_gemv_rows", _i, [_vp, _i]),
    ("lbk_int8_peak_probe", _i, [_vp, _sz, _sz, _vp]),
    ("lbk_padded_cols", _sz, [_sz]),
    ("lbk_row_bytes", _sz, [_sz]),
    ("lbk_weight_upload", _i, [_vp, _sz, _sz, _vp, _sz, _f, _pp]),
    ("lbk_weight_wrap", _i, [_vp, _sz, _sz, _vp, _f, _pp]),
    ("lbk_weight_free", _i, [_vp]),
    ("lbk_weight_rows", _sz, [_vp]),
    ("lbk_weight_cols", _sz, [_vp]),
    ("lbk_weight_scale", _f, [_vp]),
    ("lbk_weight_data", _vp, [_vp]),
    ("lbk_weight_download", _i, [_vp, _vp, _sz]),
    ("lbk_quantize_acts", _i, [_vp, _vp, _sz, _sz, _vp, _vp, _vp]),
    ("lbk_ternary_gemm_i32", _i, [_vp, _vp, _vp, _vp, _sz, _vp]),
    ("lbk_ternary_gemm_multi", _i, [_vp, _pp, _sz, _vp, _vp, _vp, _sz, _pp]),
    ("lbk_ternary_linear_host", _i, [_vp, _vp, _sz, _pp, _sz, _pp, _pp]),
    ("lbk_bf16_gemv_host", _i, [_vp, _vp, _sz, _sz, _vp, _vp]),
    ("lbk_ternary_linear_n", _i, [_vp, _vp, _sz, _pp, _sz, _pp, _pp, _vp]),
    ("lbk_ternary_linear_prefill_static", _i, [_vp, _vp, _sz, _pp, _sz, _pp, _pp, _vp]),
    ("lbk_quantize_acts_dev", _i, [_vp, _vp, _sz, _sz, _vp, _vp, _vp, _vp]),
    ("lbk_absmax_dev", _i, [_vp, _vp, _sz, _sz, _vp, _vp]),
    ("lbk_quantize_acts_amax_dev", _i, [_vp, _vp, _sz, _sz, _vp, _vp, _vp, _vp, _vp]),
    ("lbk_scale_epilogue_dev", _i, [_vp, _vp, _vp, _f, _sz, _sz, _vp, _vp]),
    ("lbk_ternary_gemm_dev", _i, [_vp, _pp, _sz, _vp, _vp, _vp, _sz, _pp, _pp, _vp]),
    ("lbk_bf16_linear", _i, [_vp, _vp, _sz, _vp, _sz, _sz, _vp, _vp]),
    ("lbk_embed_bf16", _i, [_vp, _vp, _vp, _sz, _sz, _vp, _vp]),
    ("lbk_rms_norm", _i, [_vp, _vp, _vp, _sz, _sz, _f, _vp, _vp]),
    ("lbk_rope_kv_append", _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _vp, _vp, _vp]),
    ("lbk_attn_decode", _i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _vp, _vp, _vp]),
    ("lbk_relu2_mul", _i, [_vp, _vp, _vp, _sz, _vp, _vp]),
    ("lbk_add_inplace", _i, [_vp, _vp, _vp, _sz, _vp]),
    ("lbk_add_rms_norm", _i, [_vp, _vp, _vp, _vp, _sz, _sz, _f, _vp, _vp]),
    ("lbk_relu2_mul_rms_norm", _i, [_vp, _vp, _vp, _vp, _sz, _sz, _f, _vp, _vp]),
    ("lbk_rope_kv_append_rows", _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _vp, _vp, _vp]),
    ("lbk_attn_prefill", _i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _vp, _vp]),
    ("lbk_attn_decode_fused_supported", _i, [_sz, _sz, _sz, _sz]),
    ("lbk_attn_decode_fused", _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _vp, _vp, _vp, _vp, _vp, _vp]),
    ("lbk_ternary_linear_pre_supported", _i, [_sz, _sz]),
    ("lbk_ternary_linear_pre", _i, [_vp, _i, _vp, _vp, _vp, _f, _vp, _sz, _pp, _sz, _pp, _pp, _vp]),
    ("lbk_argmax", _i, [_vp, _vp, _sz, _sz, _vp, _vp]),
    ("lbk_advance_pos", _i, [_vp, _vp, _vp]),
    ("lbk_tp_region_bytes", _sz, []),
    ("lbk_tp_max_tokens", _sz, []),
    ("lbk_tp_partial_bytes", _sz, []),
    ("lbk_tp_region_alloc", _i, [_vp, _pp, _vp]),
    ("lbk_tp_region_open", _i, [_vp, _vp, _pp]),
    ("lbk_tp_region_close", _i, [_vp, _vp]),
    ("lbk_tp_region_free", _i, [_vp, _vp]),
    ("lbk_tp_comm_create", _i, [_vp, _i, _i, _pp, _pp]),
    ("lbk_tp_comm_destroy", _i, [_vp]),
    ("lbk_tp_comm_set_wait_limit", _i, [_vp, C.c_uint32]),
    ("lbk_tp_partial_buffer", _vp, [_vp]),
    ("lbk_tp_quantize", _i, [_vp, _vp, _sz, _sz, _vp, _vp, _vp, _vp]),
    ("lbk_tp_reduce_scale", _i, [_vp, _vp, _f, _sz, _sz, _vp, _vp, _vp]),
    ("lbk_tp_max_rows", _sz, []),
    ("lbk_tp_max_width", _sz, []),
    ("lbk_tp_max_f32_rows", _sz, []),
    ("lbk_tp_token_range", _i, [_vp, _sz, _vp, _vp]),
    ("lbk_tp_norm_quant", _i, [_vp, _i, _vp, _vp, _vp, _sz, _sz, _sz, _f, _vp, _vp, _vp, _vp]),
    ("lbk_tp_reduce_norm_gather", _i, [_vp, _i, _vp, _f, _vp, _vp, _f, _sz, _sz, _vp, _vp]),
    ("lbk_tp_gemm_scatter", _i, [_vp, _vp, _vp, _vp, _sz, _vp]),
    ("lbk_tp_gather_q", _vp, [_vp]),
    ("lbk_tp_gather_scale", _vp, [_vp]),
    ("lbk_tp_gather_sum", _vp, [_vp]),
    ("lbk_tp_gather_f32", _vp, [_vp]),
    ("lbk_tp_argmax", _i, [_vp, _vp, _vp, _sz, _sz, _vp, _vp]),
    ("lbk_model_load", _i, [_vp, C.c_char_p, _pp]),
    ("lbk_model_load_shard", _i, [_vp, C.c_char_p, _i, _i, _pp]),
    ("lbk_model_load_stats", _i, [_vp, _vp]),
    ("lbk_model_linear", _vp, [_vp, _sz, _i]),
    ("lbk_model_norm", _vp, [_vp, _sz, _i]),
    ("lbk_model_embedding", _vp, [_vp]),
    ("lbk_model_rope_cos", _vp, [_vp]),
    ("lbk_model_rope_sin", _vp, [_vp]),
    ("lbk_model_get_config", _i, [_vp, _vp]),
    ("lbk_model_free", _i, [_vp]),
    ("lbk_model_new_cache", _i, [_vp, _sz, _sz, _pp]),
    ("lbk_kv_cache_len", _sz, [_vp]),
    ("lbk_kv_cache_reset", _i, [_vp]),
    ("lbk_kv_cache_free", _i, [_vp]),
    ("lbk_model_forward", _i, [_vp, _vp, _vp, _sz, _i, _vp]),
    ("lbk_model_decode", _i, [_vp, _vp, _vp, _vp, _vp, _vp]),
    ("lbk_norm_quant_supported", _i, [_sz]),
    ("lbk_norm_quant", _i, [_vp, _i, _vp, _vp, _vp, _sz, _sz, _f, _vp, _vp, _vp, _vp]),
    ("lbk_model_set_prefill_rows", _i, [_vp, _sz]),
    ("lbk_kv_cache_len_seq", _sz, [_vp, _sz]),
    ("lbk_batcher_create", _i, [_vp, _sz, _sz, _pp]),
    ("lbk_batcher_submit", _i, [_vp, _vp, _sz, _sz, _i, _vp]),
    ("lbk_batcher_step", _i, [_vp, _vp]),
    ("lbk_batcher_poll", _i, [_vp, C.c_uint64, _vp, _sz, _vp, _vp]),
    ("lbk_batcher_forget", _i, [_vp, C.c_uint64]),
    ("lbk_batcher_destroy", _i, [_vp]),
    ("lbk_rope_kv_append_seq", _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _vp, _vp, _vp]),
    ("lbk_attn_decode_seq", _i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _vp, _vp, _vp]),
    ("lbk_attn_decode_fused_seq", _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _vp, _vp, _vp, _vp, _vp, _vp]),
    ("lbk_advance_pos_seq", _i, [_vp, _vp, _vp, _sz, _vp]),
    ("lbk_convert_bitlinear", _i, [_vp, _vp, _sz, _i, _vp, _vp, _vp, _vp]),
    ("lbk_plan_create", _i, [_vp, _pp]),
    ("lbk_plan_add", _i, [_vp, _vp, _pp, _sz, _pp, _pp]),
    ("lbk_plan_finalize", _i, [_vp]),
    ("lbk_plan_run", _i, [_vp, _vp]),
    ("lbk_plan_run_host", _i, [_vp, _vp, _sz, _vp, _sz, _vp]),
    ("lbk_plan_input_elems", _sz, [_vp]),
    ("lbk_plan_output_elems", _sz, [_vp]),
    ("lbk_plan_input_arena", _vp, [_vp]),
    ("lbk_plan_output_arena", _vp, [_vp]),
    ("lbk_plan_weight_bytes", _sz, [_vp]),
    ("lbk_plan_destroy", _i, [_vp]),
]


class LbkError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"lbk status {status} ({STATUS_NAMES.get(status, '?')}): {message}")
        self.status = status
        self.message = message


_lib = None


def load() -> C.CDLL:
    """Load liblbk.so and bind every declared symbol. Raises if it is not built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m lemonade_burn_b200.build` "
                "(there is no CPU fallback)")
        lib = C.CDLL(str(LIB_PATH))
        for name, res, args in SYMBOLS:
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(status: int) -> None:
    if status != LBK_OK:
        raise LbkError(status, load().lbk_last_error().decode(errors="replace"))


def ptr_array(ptrs):
    """void*[n] from ints/None."""
    arr = (C.c_void_p * len(ptrs))(*[C.c_void_p(p) if p else C.c_void_p(0) for p in ptrs])
    return C.cast(arr, _pp), arr
