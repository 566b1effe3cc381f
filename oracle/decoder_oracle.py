"""CPU restatement of one decode step of lb-model's BitNet::forward (test infrastructure only).

Follows crates/lb-model/src/model.rs:305-374 with m = 1: rms_norm (:267-272), fused q/k/v, rotate-half
RoPE with the tables of :213-230 (:295-303), cache append, grouped-query attention with softmax in
f32 (:350-357), attn_sub_norm, o, residual, post-norm, gate/up, relu^2 * up (:363), ffn_sub_norm,
down, residual, final norm, bf16 head (crates/lb-ternary/src/bf16.rs:14-51), argmax
(crates/lb-model/src/sample.rs:17-25). Projections go through the integer oracle (lbt_oracle.c).
The K/V cache holds bf16 values (round-to-nearest-even), as the benchmark configuration asks; the
reference keeps f32 there (`kv_bf16=False` gives the reference's f32 cache).

Pinned against a second, independent statement: tests/golden/hf_bitnet_decoder.npz holds logits of
the installed `transformers` BitNetForCausalLM (random init, float32) on a seeded sequence, written
by tests/golden/make_decoder_fixture.py; tests/test_decoder_oracle_pin.py holds this restatement to
them by the reference's own end-to-end metrics (crates/lb-model/src/bin/lb-run.rs:223-259: top-1
agreement, agreement where the margin is clear, max / mean |delta logit|). That is the library the
reference itself validates against (scripts/hf_reference.py:41-58). The reference has no in-repo
test or fixture for BitNet::forward, and its float ops run inside a tensor library whose summation
order is not visible, so agreement is to rounding, not bit for bit.

`fast=True` sends the projections through the threaded SIMD port (lbt_simd.c; its integers equal the
scalar restatement's, tested) so that a full-size model (30 layers, 128256-entry vocabulary) takes
about a second per token on a few cores.
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


def _linear(x, packed, scale, cols, fast=False):
    if fast:
        q, s, ssum = o.quantize_acts(x.astype(np.float32))
        return o.simd_gemm_multi([packed], [np.float32(scale)], q, s, ssum)[0][0]
    return o.ternary_linear(x.astype(np.float32), packed, np.float32(scale), cols)[0]


def rope_tables(hd, theta, max_pos):
    inv = np.array([1.0 / theta ** ((2 * i) / hd) for i in range(hd // 2)], dtype=np.float64).astype(np.float32)
    f = (np.arange(max_pos, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float32).astype(np.float64)
    return (np.concatenate([np.cos(f), np.cos(f)], 1).astype(np.float32), np.concatenate([np.sin(f), np.sin(f)], 1).astype(np.float32))


def _rope(x, cos, sin):  # x [heads, hd]
    half = x.shape[-1] // 2
    rot = np.concatenate([-x[:, half:], x[:, :half]], axis=-1)
    return (x * cos + rot * sin).astype(np.float32)


def decode_step(cfg, w, token, kc, vc, pos, kv_bf16=True, fast=False):
    """cfg: dict-like with the Config fields; w: name -> numpy (qweight u8, wscale f32, norms f32,
    embed as uint16 bf16 bits); kc/vc: [layers][kvh][cap][hd] f32 arrays (holding bf16-rounded values
    when kv_bf16), updated in place at `pos`. Returns logits f32 [vocab]."""
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    nh, kvh = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd, eps = H // nh, cfg["rms_norm_eps"]
    group = nh // kvh
    cos, sin = w["_cos"][pos], w["_sin"][pos]
    emb = w["model.embed_tokens.weight"]
    x = (emb[token].astype(np.uint32) << 16).view(np.float32)[None, :].copy()
    for li in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{li}"
        lin = lambda name, inp, cols: _linear(inp, w[f"{p}.{name}.qweight"], w[f"{p}.{name}.wscale"][0], cols, fast)
        n1 = _rms(x, w[f"{p}.input_layernorm.weight"], eps)
        q = _rope(lin("self_attn.q_proj", n1, H).reshape(nh, hd), cos, sin)
        k = _rope(lin("self_attn.k_proj", n1, H).reshape(kvh, hd), cos, sin)
        v = lin("self_attn.v_proj", n1, H).reshape(kvh, hd)
        kc[li][:, pos] = _bf16_round(k) if kv_bf16 else k
        vc[li][:, pos] = _bf16_round(v) if kv_bf16 else v
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


def greedy_decode(cfg, w, prompt, n_new, kv_bf16=True, fast=False):
    """The reference's generation loop with greedy sampling (crates/lb-server/src/main.rs:102-166,
    sample.rs:17-25): the prompt token by token, then n_new tokens, each the first maximum of the
    previous step's logits. Returns the generated tokens."""
    kvh, hd = cfg["num_key_value_heads"], cfg["hidden_size"] // cfg["num_attention_heads"]
    cap = len(prompt) + n_new
    kc = [np.zeros((kvh, cap, hd), np.float32) for _ in range(cfg["num_hidden_layers"])]
    vc = [np.zeros((kvh, cap, hd), np.float32) for _ in range(cfg["num_hidden_layers"])]
    logits = None
    for pos, tok in enumerate(prompt):
        logits = decode_step(cfg, w, int(tok), kc, vc, pos, kv_bf16, fast)
    out = []
    for i in range(n_new):
        nxt = o.argmax(logits)
        out.append(nxt)
        if i + 1 < n_new:
            logits = decode_step(cfg, w, nxt, kc, vc, len(prompt) + i, kv_bf16, fast)
    return out


def compare_logits(got, ref, margin=0.5):
    """The reference's end-to-end report (lb-run.rs:223-259): top-1 agreement over rows, agreement
    restricted to rows where the reference's top-1 leads its runner-up by more than `margin`, and
    max / mean |delta logit|. got, ref: [rows, vocab]."""
    got, ref = np.atleast_2d(got), np.atleast_2d(ref)
    top_g, top_r = got.argmax(axis=1), ref.argmax(axis=1)
    srt = np.sort(ref, axis=1)
    clear = (srt[:, -1] - srt[:, -2]) > margin
    d = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    return {"rows": int(ref.shape[0]), "top1_agree": int((top_g == top_r).sum()), "clear_rows": int(clear.sum()),
            "clear_agree": int(((top_g == top_r) & clear).sum()), "max_abs_delta": float(d.max()), "mean_abs_delta": float(d.mean()),
            "max_abs_logit": float(np.abs(ref).max())}


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def check_step(cfg, w, tokens, k_bits, v_bits, pos, fast=True):
    """One decode step for each of b independent sequences that already hold `pos` cached positions
    (the reference has no batch dimension: b single-token forwards, model.rs:305-374 with m = 1).
    k_bits / v_bits: uint16 bf16 bits [layers][b][kvh][cap][hd], the device cache as it was BEFORE the
    step. Returns logits f32 [b, vocab]."""
    L = cfg["num_hidden_layers"]
    out = []
    for bi, tok in enumerate(tokens):
        kc = [bf16_bits_to_f32(k_bits[li][bi]) for li in range(L)]
        vc = [bf16_bits_to_f32(v_bits[li][bi]) for li in range(L)]
        out.append(decode_step(cfg, w, int(tok), kc, vc, pos, kv_bf16=True, fast=fast))
    return np.stack(out)
