"""CPU restatement of one decode step of lb-model's BitNet::forward (test infrastructure only).

Follows crates/lb-model/src/model.rs:305-374 with m = 1: rms_norm (:267-272), fused q/k/v, rotate-half
RoPE with the tables of :213-230 (:295-303), cache append, grouped-query attention with softmax in
f32 (:350-357), attn_sub_norm, o, residual, post-norm, gate/up, relu^2 * up (:363), ffn_sub_norm,
down, residual, final norm, bf16 head (crates/lb-ternary/src/bf16.rs:14-51), argmax
(crates/lb-model/src/sample.rs:17-25). Projections go through the integer oracle (lbt_oracle.c).
The K/V cache holds bf16 values (round-to-nearest-even), as the benchmark configuration asks; the
reference keeps f32 there. PARITY UNPINNED: the reference has no test or fixture for
BitNet::forward, and its float ops run inside a tensor library whose summation order is not
visible, so agreement is to rounding, judged by greedy-token equality and max |delta logit|.
"""
from __future__ import annotations

import numpy as np

from . import oracle as o


def _bf16_round(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return (u.astype(np.uint32) << 16).view(np.float32)


def _rms(x, w, eps):
    var = np.mean(x.astype(np.float32) ** 2, axis=-1, keepdims=True, dtype=np.float32)
    return (x * (np.float32(1.0) / np.sqrt(var + np.float32(eps))) * w).astype(np.float32)


def _linear(x, packed, scale, cols):
    return o.ternary_linear(x.astype(np.float32), packed, np.float32(scale), cols)[0]


def rope_tables(hd, theta, max_pos):
    inv = np.array([1.0 / theta ** ((2 * i) / hd) for i in range(hd // 2)], dtype=np.float64).astype(np.float32)
    f = (np.arange(max_pos, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float32).astype(np.float64)
    return (np.concatenate([np.cos(f), np.cos(f)], 1).astype(np.float32), np.concatenate([np.sin(f), np.sin(f)], 1).astype(np.float32))


def _rope(x, cos, sin):  # x [heads, hd]
    half = x.shape[-1] // 2
    rot = np.concatenate([-x[:, half:], x[:, :half]], axis=-1)
    return (x * cos + rot * sin).astype(np.float32)


def decode_step(cfg, w, token, kc, vc, pos):
    """cfg: dict-like with the Config fields; w: name -> numpy (qweight u8, wscale f32, norms f32,
    embed as uint16 bf16 bits); kc/vc: [layers][kvh][cap][hd] f32 arrays holding bf16-rounded values,
    updated in place at `pos`. Returns logits f32 [vocab]."""
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    nh, kvh = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd, eps = H // nh, cfg["rms_norm_eps"]
    group = nh // kvh
    cos, sin = w["_cos"][pos], w["_sin"][pos]
    emb = w["model.embed_tokens.weight"]
    x = (emb[token].astype(np.uint32) << 16).view(np.float32)[None, :].copy()
    for li in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{li}"
        lin = lambda name, inp, cols: _linear(inp, w[f"{p}.{name}.qweight"], w[f"{p}.{name}.wscale"][0], cols)
        n1 = _rms(x, w[f"{p}.input_layernorm.weight"], eps)
        q = _rope(lin("self_attn.q_proj", n1, H).reshape(nh, hd), cos, sin)
        k = _rope(lin("self_attn.k_proj", n1, H).reshape(kvh, hd), cos, sin)
        v = lin("self_attn.v_proj", n1, H).reshape(kvh, hd)
        kc[li][:, pos] = _bf16_round(k)
        vc[li][:, pos] = _bf16_round(v)
        keys, vals = kc[li][:, :pos + 1], vc[li][:, :pos + 1]          # [kvh, total, hd]
        qg = q.reshape(kvh, group, hd)
        scores = np.einsum("kgd,ktd->kgt", qg, keys).astype(np.float32) * np.float32(hd ** -0.5)
        scores = scores - scores.max(axis=-1, keepdims=True)
        pr = np.exp(scores).astype(np.float32)
        pr = pr / pr.sum(axis=-1, keepdims=True, dtype=np.float32)
        attn = np.einsum("kgt,ktd->kgd", pr, vals).astype(np.float32).reshape(1, nh * hd)
        attn = _rms(attn, w[f"{p}.self_attn.attn_sub_norm.weight"], eps)
        x = x + lin("self_attn.o_proj", attn, nh * hd)
        n2 = _rms(x, w[f"{p}.post_attention_layernorm.weight"], eps)
        g, u = lin("mlp.gate_proj", n2, H), lin("mlp.up_proj", n2, H)
        a = _rms(np.maximum(g, 0) ** 2 * u, w[f"{p}.mlp.ffn_sub_norm.weight"], eps)
        x = (x + lin("mlp.down_proj", a, I)).astype(np.float32)
    xn = _rms(x, w["model.norm.weight"], eps)
    return o.bf16_gemv(emb, xn[0])
