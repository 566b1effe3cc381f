"""BitNet b1.58 decoder on the GPU: the device-side mirror of lb-model's `BitNet`
(crates/lb-model/src/model.rs). Same names and meaning: `Config`, `BitNet.load`,
`BitNet.new_cache`, `BitNet.forward`, checkpoint format "lemonade-burn-ternary" v1
(crates/lb-convert/src/lib.rs:1-16). Differences, all stated: the KV cache is bf16 (the
reference keeps f32, model.rs:245), `forward` takes one new token per sequence (decode; `b`
independent sequences advance together), and every op runs in liblbk.so.

Per layer (model.rs:331-366):
    n1 = rms(x); q,k,v = ternary3(n1); rope(q), rope(k); cache k,v; a = gqa(q, K, V)
    x += o(rms(a, attn_sub_norm)); n2 = rms(x)
    g,u = ternary2(n2); x += down(rms(relu(g)^2 * u, ffn_sub_norm))
then final norm, bf16 LM head (tied embedding), greedy argmax.
"""
from __future__ import annotations

import ctypes as C
import json
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Optional

import numpy as np
import torch

from . import _lib, ops
from .pack import row_bytes
from .ternary import Context, default_context

FORMAT = "lemonade-burn-ternary"      # lb-convert/src/lib.rs:14
FILE_NAME = "model.lbt.safetensors"   # lb-convert/src/lib.rs:16
LINEARS = ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
           "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"]  # lb-convert/src/lib.rs:18-26


@dataclass
class Config:
    """model.rs:23-42"""
    hidden_size: int
    intermediate_size: int
    num_attention_heads: int
    num_key_value_heads: int
    num_hidden_layers: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    hidden_act: str = "relu2"
    tie_word_embeddings: bool = True
    bos_token_id: int = 0

    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @staticmethod
    def bitnet_2b4t(layers: int = 30, max_pos: int = 4352) -> "Config":
        return Config(2560, 6912, 20, 5, layers, 128256, 1e-5, 500000.0, max_pos)


def rope_tables(cfg: Config):
    """model.rs:213-230: inv_freq in f32, freq = pos as f32 * inv (f32), sin/cos in f64, stored
    f32, duplicated to both halves."""
    hd = cfg.head_dim()
    inv = np.array([1.0 / cfg.rope_theta ** ((2 * i) / hd) for i in range(hd // 2)], dtype=np.float64).astype(np.float32)
    pos = np.arange(cfg.max_position_embeddings, dtype=np.float32)
    f = (pos[:, None] * inv[None, :]).astype(np.float32).astype(np.float64)
    cos = np.concatenate([np.cos(f), np.cos(f)], axis=1).astype(np.float32)
    sin = np.concatenate([np.sin(f), np.sin(f)], axis=1).astype(np.float32)
    return cos, sin


class KvCache:
    """model.rs:136-141, here fixed capacity, bf16, [layers][b][kv_heads][cap][head_dim]."""

    def __init__(self, cfg: Config, b: int, cap: int, device):
        if cap < 1 or cap > cfg.max_position_embeddings:  # the RoPE tables end there (model.rs:213-230, 309)
            raise ValueError(f"capacity {cap} is outside 1..max_position_embeddings ({cfg.max_position_embeddings})")
        if b < 1:
            raise ValueError("a cache serves at least one sequence")
        shape = (cfg.num_hidden_layers, b, cfg.num_key_value_heads, cap, cfg.head_dim())
        self.k = torch.zeros(shape, dtype=torch.bfloat16, device=device)
        self.v = torch.zeros(shape, dtype=torch.bfloat16, device=device)
        self.pos = torch.zeros(1, dtype=torch.int32, device=device)  # cache.len, on the device
        self.b, self.cap = b, cap
        self.host_len = 0  # the same length on the host: `forward` refuses a step that would not fit

    @property
    def len(self) -> int:
        return int(self.pos.item())

    def reserve(self, n: int = 1) -> None:
        """Raises unless `n` more positions fit (model.rs:309 asserts pos0 + m <= rope_len). Called by
        `BitNet.forward` before anything is launched; the kernels check the device-side position too."""
        if self.host_len + n > self.cap:
            raise ValueError(f"the cache is full: {self.host_len} of {self.cap} positions are used, {n} more do not fit")


class BitNet:
    def __init__(self, cfg: Config, tensors: Dict[str, torch.Tensor], ctx: Optional[Context] = None, device="cuda:0"):
        if cfg.hidden_act != "relu2" or not cfg.tie_word_embeddings:  # model.rs:151-153
            raise ValueError(f"unsupported config: act={cfg.hidden_act} tied={cfg.tie_word_embeddings}")
        self.cfg, self.ctx, self.device = cfg, ctx or default_context(), torch.device(device)
        dev = self.device
        H, I = cfg.hidden_size, cfg.intermediate_size

        def linear(name, cols):
            qw = tensors[f"{name}.qweight"]
            if qw.dtype != torch.uint8 or qw.shape[1] != row_bytes(cols):
                raise ValueError(f"{name}: unexpected dtype/shape")
            scale = float(tensors[f"{name}.wscale"].reshape(-1)[0])
            return ops.TernaryLinear(qw.to(dev), scale, cols, self.ctx)

        def vec(name):
            t = tensors[name]
            if t.dtype != torch.float32:
                raise ValueError(f"{name}: expected F32")  # model.rs:165
            return t.to(dev).contiguous()

        self.layers = []
        for i in range(cfg.num_hidden_layers):
            p = f"model.layers.{i}"
            self.layers.append(dict(
                input_norm=vec(f"{p}.input_layernorm.weight"), post_attn_norm=vec(f"{p}.post_attention_layernorm.weight"),
                attn_sub_norm=vec(f"{p}.self_attn.attn_sub_norm.weight"), ffn_sub_norm=vec(f"{p}.mlp.ffn_sub_norm.weight"),
                q=linear(f"{p}.self_attn.q_proj", H), k=linear(f"{p}.self_attn.k_proj", H), v=linear(f"{p}.self_attn.v_proj", H),
                o=linear(f"{p}.self_attn.o_proj", H), gate=linear(f"{p}.mlp.gate_proj", H), up=linear(f"{p}.mlp.up_proj", H),
                down=linear(f"{p}.mlp.down_proj", I)))
        self.final_norm = vec("model.norm.weight")
        emb = tensors["model.embed_tokens.weight"]
        if emb.dtype != torch.bfloat16 or tuple(emb.shape) != (cfg.vocab_size, H):  # model.rs:204
            raise ValueError("embed_tokens: unexpected dtype/shape")
        self.lm_head = emb.to(dev).contiguous()
        cos, sin = rope_tables(cfg)
        self.cos, self.sin = torch.from_numpy(cos).to(dev), torch.from_numpy(sin).to(dev)
        self._bufs = {}

    # ---- checkpoint --------------------------------------------------------------------------
    @classmethod
    def load(cls, directory, ctx: Optional[Context] = None, device="cuda:0") -> "BitNet":
        """model.rs:149-232: config.json + model.lbt.safetensors with metadata format check."""
        from safetensors import safe_open
        directory = Path(directory)
        raw = json.loads((directory / "config.json").read_text())
        for key in ("hidden_act", "tie_word_embeddings"):  # required fields of the reference's Config (model.rs:22-36)
            if key not in raw:
                raise ValueError(f"{directory / 'config.json'}: missing field {key}")
        cfg = Config(**{k: raw[k] for k in Config.__dataclass_fields__ if k in raw})
        path = directory / FILE_NAME
        tensors = {}
        with safe_open(str(path), framework="pt", device="cpu") as f:
            meta = f.metadata() or {}
            if meta.get("format") != FORMAT:  # model.rs:158-161
                raise ValueError(f"{path} is not a lemonade-burn ternary file (format={meta.get('format')!r})")
            for k in f.keys():
                tensors[k] = f.get_tensor(k)
        return cls(cfg, tensors, ctx, device)

    def new_cache(self, b: int = 1, cap: Optional[int] = None) -> KvCache:
        """model.rs:234-236. The capacity cannot exceed the RoPE tables (max_position_embeddings)."""
        return KvCache(self.cfg, b, cap or self.cfg.max_position_embeddings, self.device)

    # ---- one decode step -------------------------------------------------------------------------
    def _buf(self, name, shape, dtype=torch.float32):
        key = (name, tuple(shape), dtype)
        if key not in self._bufs:
            self._bufs[key] = torch.empty(shape, dtype=dtype, device=self.device)
        return self._bufs[key]

    def forward(self, tokens: torch.Tensor, cache: KvCache, splits: Optional[int] = None) -> torch.Tensor:
        """One new token per sequence at position cache.len (model.rs:305-374 with m = 1).
        tokens: int32 CUDA [b]. Returns logits f32 [b, vocab] and advances the cache."""
        cfg, lib, h = self.cfg, self.ctx._lib, self.ctx.handle
        b = tokens.shape[0]
        if b != cache.b:
            raise ValueError("batch size differs from the cache's")
        cache.reserve(1)
        if splits is None:
            splits = attention_splits(cache.cap)
        H, I, nh, kvh, hd = cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim()
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        P = lambda t: C.c_void_p(t.data_ptr())
        eps = C.c_float(cfg.rms_norm_eps)
        x = self._buf("x", (b, H))
        x2 = self._buf("x2", (b, H))
        n = self._buf("n", (b, H))
        attn = self._buf("attn", (b, nh * hd))
        act = self._buf("act", (b, I))
        scratch = self._buf("attn_part", (b * nh * splits * (hd + 4),))
        chk = _lib.check
        e = cfg.rms_norm_eps
        fused = H % 4 == 0 and H <= 8192 and I % 4 == 0 and I <= 8192
        # Where the decode kernel can hold the input row in registers (small batches), the norms, the
        # residual adds and the gate run inside the projection kernels: 7 launches a layer, not 13.
        pre_h, pre_a, pre_i = ops.pre_supported(b, H), ops.pre_supported(b, nh * hd), ops.pre_supported(b, I)
        attn_fused = bool(lib.lbk_attn_decode_fused_supported(nh, kvh, hd, splits))
        key = ("attn_counters", (b * kvh,), torch.int32)
        if key not in self._bufs:
            self._bufs[key] = torch.zeros(b * kvh, dtype=torch.int32, device=self.device)  # zero once; the kernel keeps them zero
        counters = self._bufs[key]

        def add_norm(xin, y, w, xout):  # xout = xin + y; n = rms_norm(xout) * w
            if fused and xin is xout:
                chk(lib.lbk_add_rms_norm(h, P(xin), P(y), P(w), b, H, eps, P(n), st))
            else:
                if xin is not xout:
                    xout.copy_(xin)
                chk(lib.lbk_add_inplace(h, P(xout), P(y), b * H, st))
                chk(lib.lbk_rms_norm(h, P(xout), P(w), b, H, eps, P(n), st))
            return n

        # From 9 sequences on every projection takes the quantise + GEMM path; the norm in front of it
        # then writes the quantised rows itself (lbk_norm_quant): no f32 copy, no quantise kernel.
        nq = b >= 9 and all(ops.norm_quant_supported(wd) for wd in (H, I, nh * hd))
        if nq:
            q8 = self._buf("q8", (b, row_bytes(max(H, I, nh * hd)) * 4), torch.int8)
            qs, qsum = self._buf("qs", (b,)), self._buf("qsum", (b,), torch.int32)
            normq = lambda pre, xx, yy, w: ops.norm_quant(pre, xx, yy, w, e, q8, qs, qsum, self.ctx)
            projq = lambda lins: ops.ternary_gemm_q(q8, qs, qsum, b, lins)

        chk(lib.lbk_embed_bf16(h, P(self.lm_head), P(tokens), b, H, P(x), st))
        d = None  # output of the previous layer's down projection, not yet added to the residual x
        for li, l in enumerate(self.layers):
            qkv_l = [l["q"], l["k"], l["v"]]
            if nq:
                if d is None:
                    normq(ops.PRE_RMS, x, None, l["input_norm"])
                else:
                    normq(ops.PRE_ADD_RMS, x, d, l["input_norm"])
                q, k, v = projq(qkv_l)
            elif d is None:
                if pre_h:
                    q, k, v = ops.ternary_linear_pre(ops.PRE_RMS, x, None, l["input_norm"], e, qkv_l)
                else:
                    chk(lib.lbk_rms_norm(h, P(x), P(l["input_norm"]), b, H, eps, P(n), st))
                    q, k, v = ops.ternary_linear3(n, qkv_l)
            elif pre_h:
                q, k, v = ops.ternary_linear_pre(ops.PRE_ADD_RMS, x, d, l["input_norm"], e, qkv_l, xout=x2)
                x, x2 = x2, x
            else:
                q, k, v = ops.ternary_linear3(add_norm(x, d, l["input_norm"], x), qkv_l)
            if attn_fused:  # RoPE, KV append, attention slices and their merge in one launch
                chk(lib.lbk_attn_decode_fused(h, P(q), P(k), P(v), P(self.cos), P(self.sin), P(cache.pos), b, nh, kvh, hd, cache.cap,
                                              splits, P(cache.k[li]), P(cache.v[li]), P(scratch), P(counters), P(attn), st))
            else:
                chk(lib.lbk_rope_kv_append(h, P(q), P(k), P(v), P(self.cos), P(self.sin), P(cache.pos), b, nh, kvh, hd, cache.cap,
                                           P(cache.k[li]), P(cache.v[li]), st))
                chk(lib.lbk_attn_decode(h, P(q), P(cache.k[li]), P(cache.v[li]), P(cache.pos), b, nh, kvh, hd, cache.cap, splits,
                                        P(scratch), P(attn), st))
            if nq:
                normq(ops.PRE_RMS, attn, None, l["attn_sub_norm"])
                o = projq([l["o"]])[0]
                normq(ops.PRE_ADD_RMS, x, o, l["post_attn_norm"])
                g, u = projq([l["gate"], l["up"]])
                normq(ops.PRE_RELU2_MUL_RMS, g, u, l["ffn_sub_norm"])
                d = projq([l["down"]])[0]
                continue
            if pre_a:
                o = ops.ternary_linear_pre(ops.PRE_RMS, attn, None, l["attn_sub_norm"], e, [l["o"]])[0]
            else:
                chk(lib.lbk_rms_norm(h, P(attn), P(l["attn_sub_norm"]), b, nh * hd, eps, P(attn), st))
                o = ops.ternary_linear(attn, l["o"])
            if pre_h:
                g, u = ops.ternary_linear_pre(ops.PRE_ADD_RMS, x, o, l["post_attn_norm"], e, [l["gate"], l["up"]], xout=x2)
                x, x2 = x2, x
            else:
                g, u = ops.ternary_linear2(add_norm(x, o, l["post_attn_norm"], x), [l["gate"], l["up"]])
            if pre_i:
                d = ops.ternary_linear_pre(ops.PRE_RELU2_MUL_RMS, g, u, l["ffn_sub_norm"], e, [l["down"]])[0]
            else:
                if fused:
                    chk(lib.lbk_relu2_mul_rms_norm(h, P(g), P(u), P(l["ffn_sub_norm"]), b, I, eps, P(act), st))
                else:
                    chk(lib.lbk_relu2_mul(h, P(g), P(u), b * I, P(act), st))
                    chk(lib.lbk_rms_norm(h, P(act), P(l["ffn_sub_norm"]), b, I, eps, P(act), st))
                d = ops.ternary_linear(act, l["down"])
        if d is None:
            chk(lib.lbk_rms_norm(h, P(x), P(self.final_norm), b, H, eps, P(n), st))
        else:
            add_norm(x, d, self.final_norm, x)
        logits = ops.bf16_linear(n, self.lm_head, self.ctx)
        chk(lib.lbk_advance_pos(h, P(cache.pos), st))
        cache.host_len += 1
        return logits

    def argmax(self, logits: torch.Tensor) -> torch.Tensor:
        """sample.rs:17-25 on the device."""
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        _lib.check(self.ctx._lib.lbk_argmax(self.ctx.handle, C.c_void_p(logits.data_ptr()), logits.shape[0], logits.shape[1],
                                            C.c_void_p(out.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return out


def attention_splits(cap: int) -> int:
    """Slices of the key range per attention problem (sequence x KV head): 32 positions each, at most
    256. Fewer, longer slices were measured at batches 4 to 16 (8 to 130 slices at 4096 positions):
    equal within 5 % at batch 16, slower below, so the rule does not look at the batch. The native
    runtime uses the same rule, so the two produce the same bits."""
    return max(1, min(256, (cap + 31) // 32))


def random_checkpoint(cfg: Config, seed: int = 0, device="cpu") -> Dict[str, torch.Tensor]:
    """Random-init weights in checkpoint naming (there is no real checkpoint where this is built):
    valid ternary codes, scales near 1/mean|N(0,0.02)|, norm gains near 1, bf16 embedding N(0,0.02)."""
    g = torch.Generator(device=device).manual_seed(seed)
    H, I, hd = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim()
    rows = {"self_attn.q_proj": (cfg.num_attention_heads * hd, H), "self_attn.k_proj": (cfg.num_key_value_heads * hd, H),
            "self_attn.v_proj": (cfg.num_key_value_heads * hd, H), "self_attn.o_proj": (H, cfg.num_attention_heads * hd),
            "mlp.gate_proj": (I, H), "mlp.up_proj": (I, H), "mlp.down_proj": (H, I)}
    t: Dict[str, torch.Tensor] = {}
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        for name, (r, c) in rows.items():
            b = torch.randint(0, 256, (r, row_bytes(c)), dtype=torch.uint8, generator=g, device=device)
            t[f"{p}.{name}.qweight"] = b & ~((b >> 1) & b & 0x55)   # code 3 -> 1: valid ternary
            t[f"{p}.{name}.wscale"] = torch.tensor([60.0 + 5.0 * torch.rand(1, generator=g, device=device).item()], dtype=torch.float32)
        for nm, sz in (("input_layernorm", H), ("post_attention_layernorm", H), ("self_attn.attn_sub_norm", H), ("mlp.ffn_sub_norm", I)):
            t[f"{p}.{nm}.weight"] = (1.0 + 0.05 * torch.randn(sz, generator=g, device=device)).float()
    t["model.norm.weight"] = (1.0 + 0.05 * torch.randn(H, generator=g, device=device)).float()
    t["model.embed_tokens.weight"] = (0.02 * torch.randn(cfg.vocab_size, H, generator=g, device=device)).to(torch.bfloat16)
    return t


def save_checkpoint(directory, cfg: Config, tensors: Dict[str, torch.Tensor]) -> None:
    """Writes config.json + model.lbt.safetensors with the metadata lb-convert writes
    (crates/lb-convert/src/main.rs:111-115)."""
    from safetensors.torch import save_file
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    (directory / "config.json").write_text(json.dumps(cfg.__dict__))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(directory / FILE_NAME),
              metadata={"format": FORMAT, "version": "1", "quant": "absmean-ternary", "layout": "lb-ternary-128x2bit"})


class _ModelConfig(C.Structure):
    _fields_ = [(n, C.c_size_t) for n in ("hidden_size", "intermediate_size", "num_attention_heads", "num_key_value_heads",
                                          "num_hidden_layers", "vocab_size", "max_position_embeddings")] + \
               [("rms_norm_eps", C.c_float), ("rope_theta", C.c_float), ("bos_token_id", C.c_int)]


class _LoadStats(C.Structure):
    _fields_ = [("seconds", C.c_double), ("bytes_read", C.c_size_t), ("bytes_to_device", C.c_size_t), ("staging_bytes", C.c_size_t)]


class NativeBitNet:
    """The same decoder driven entirely by liblbk.so (lbk_model_load / new_cache / forward / decode):
    what a host without a tensor framework binds. Same checkpoint, same kernels, same results as
    `BitNet`; this class only marshals pointers."""

    def __init__(self, directory, ctx: Optional[Context] = None, rank: int = 0, world: int = 1):
        """world > 1: this rank's shard only (rows of q/k/v/gate/up, 128-aligned column ranges of
        o/down); such a model serves the tensor-parallel step, not `new_cache` / `forward`."""
        self.ctx = ctx or default_context()
        self._lib = self.ctx._lib
        self.rank, self.world = rank, world
        h = C.c_void_p()
        if world == 1:
            _lib.check(self._lib.lbk_model_load(self.ctx.handle, str(directory).encode(), C.byref(h)))
        else:
            _lib.check(self._lib.lbk_model_load_shard(self.ctx.handle, str(directory).encode(), rank, world, C.byref(h)))
        self.handle = h
        raw = _ModelConfig()
        _lib.check(self._lib.lbk_model_get_config(h, C.byref(raw)))
        self.cfg = Config(raw.hidden_size, raw.intermediate_size, raw.num_attention_heads, raw.num_key_value_heads,
                          raw.num_hidden_layers, raw.vocab_size, raw.rms_norm_eps, raw.rope_theta, raw.max_position_embeddings,
                          bos_token_id=raw.bos_token_id)
        self._caches = []

    LINEAR_IDS = {"q": 0, "k": 1, "v": 2, "o": 3, "gate": 4, "up": 5, "down": 6}
    NORM_IDS = {"input_norm": 0, "post_attn_norm": 1, "attn_sub_norm": 2, "ffn_sub_norm": 3, "final_norm": 4}

    def load_stats(self) -> dict:
        """Seconds, bytes read, bytes copied to the device and pinned staging bytes of the load."""
        s = _LoadStats()
        _lib.check(self._lib.lbk_model_load_stats(self.handle, C.byref(s)))
        return {"seconds": s.seconds, "bytes_read": s.bytes_read, "bytes_to_device": s.bytes_to_device, "staging_bytes": s.staging_bytes}

    def linear_handle(self, layer: int, name: str) -> int:
        h = self._lib.lbk_model_linear(self.handle, layer, self.LINEAR_IDS[name])
        if not h:
            raise ValueError(f"no linear {name} in layer {layer}")
        return h

    def linear_bytes(self, layer: int, name: str) -> np.ndarray:
        """The packed rows this model (or shard) holds for one projection, copied to the host."""
        h = self.linear_handle(layer, name)
        rows, cols = self._lib.lbk_weight_rows(h), self._lib.lbk_weight_cols(h)
        out = np.empty((rows, row_bytes(cols)), dtype=np.uint8)
        _lib.check(self._lib.lbk_weight_download(h, out.ctypes.data_as(C.c_void_p), out.size))
        return out

    def norm_ptr(self, layer: int, name: str) -> int:
        return int(self._lib.lbk_model_norm(self.handle, layer, self.NORM_IDS[name]))

    def new_cache(self, b: int = 1, cap: int = 0):
        c = C.c_void_p()
        _lib.check(self._lib.lbk_model_new_cache(self.handle, b, cap, C.byref(c)))
        self._caches.append(c)
        return c

    def cache_len(self, cache) -> int:
        return int(self._lib.lbk_kv_cache_len(cache))

    def set_prefill_rows(self, rows: int) -> None:
        """Rows a prompt pass takes at once (default 4096)."""
        _lib.check(self._lib.lbk_model_set_prefill_rows(self.handle, rows))

    def reset_cache(self, cache) -> None:
        """Back to an empty sequence; the buffers and the recorded step are kept."""
        _lib.check(self._lib.lbk_kv_cache_reset(cache))

    def forward(self, tokens, cache, all_logits: bool = False) -> np.ndarray:
        """model.rs:305: logits [n, vocab] (all_logits) or [vocab] of the last token, on the host."""
        toks = np.ascontiguousarray(tokens, dtype=np.uint32)
        out = np.empty((len(toks) if all_logits else 1, self.cfg.vocab_size), dtype=np.float32)
        _lib.check(self._lib.lbk_model_forward(self.handle, cache, toks.ctypes.data_as(C.c_void_p), len(toks), int(all_logits),
                                               out.ctypes.data_as(C.c_void_p)))
        return out if all_logits else out[0]

    def decode(self, tokens_dev: torch.Tensor, cache):
        """One token per sequence; returns (logits [b, vocab], greedy next tokens [b]) on the device."""
        b = tokens_dev.shape[0]
        logits = torch.empty((b, self.cfg.vocab_size), dtype=torch.float32, device=tokens_dev.device)
        nxt = torch.empty(b, dtype=torch.int32, device=tokens_dev.device)
        _lib.check(self._lib.lbk_model_decode(self.handle, cache, C.c_void_p(tokens_dev.data_ptr()), C.c_void_p(logits.data_ptr()),
                                              C.c_void_p(nxt.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return logits, nxt

    def batcher(self, slots: int, capacity: int = 0) -> "Batcher":
        return Batcher(self, slots, capacity)

    def close(self):
        if getattr(self, "handle", None):
            for bt in list(getattr(self, "_batchers", [])):
                bt.close()
            for c in self._caches:
                self._lib.lbk_kv_cache_free(c)
            self._caches = []
            self._lib.lbk_model_free(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Batcher:
    """Continuous batching in front of the batched decode step (lbk_batcher_*): requests queue up, take
    free slots of one shared cache (prompt pass into the slot), advance together one greedy token per
    step, and leave as soon as they finish. The reference's server runs its requests one at a time
    (crates/lb-server/src/main.rs:92-166)."""

    def __init__(self, net: NativeBitNet, slots: int, capacity: int = 0):
        self.net = net
        self._lib = net._lib
        h = C.c_void_p()
        _lib.check(self._lib.lbk_batcher_create(net.handle, slots, capacity, C.byref(h)))
        self.handle = h
        if not hasattr(net, "_batchers"):
            net._batchers = []
        net._batchers.append(self)

    def submit(self, prompt, max_new_tokens: int, eos: int = -1) -> int:
        toks = np.ascontiguousarray(prompt, dtype=np.uint32)
        rid = C.c_uint64()
        _lib.check(self._lib.lbk_batcher_submit(self.handle, toks.ctypes.data_as(C.c_void_p), len(toks), max_new_tokens, eos, C.byref(rid)))
        return int(rid.value)

    def step(self) -> int:
        """One scheduling step; returns how many requests are still queued or running."""
        pending = C.c_size_t()
        _lib.check(self._lib.lbk_batcher_step(self.handle, C.byref(pending)))
        return int(pending.value)

    def poll(self, rid: int):
        """(tokens generated so far, finished?)"""
        n, done = C.c_size_t(), C.c_int()
        _lib.check(self._lib.lbk_batcher_poll(self.handle, rid, None, 0, C.byref(n), C.byref(done)))
        out = np.empty(n.value, dtype=np.uint32)
        _lib.check(self._lib.lbk_batcher_poll(self.handle, rid, out.ctypes.data_as(C.c_void_p), len(out), C.byref(n), C.byref(done)))
        return out.tolist(), bool(done.value)

    def forget(self, rid: int) -> None:
        _lib.check(self._lib.lbk_batcher_forget(self.handle, rid))

    def run(self, max_steps: int = 1 << 30) -> int:
        """Steps until nothing is queued or running; returns the number of steps."""
        steps = 0
        while steps < max_steps:
            steps += 1
            if self.step() == 0:
                break
        return steps

    def close(self):
        if getattr(self, "handle", None):
            self._lib.lbk_batcher_destroy(self.handle)
            self.handle = None
            if self in getattr(self.net, "_batchers", []):
                self.net._batchers.remove(self)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
