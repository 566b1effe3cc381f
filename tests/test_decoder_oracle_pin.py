"""Pins oracle/decoder_oracle.py (the CPU restatement of lb-model's BitNet::forward,
crates/lb-model/src/model.rs:305-374) against logits of the installed transformers
BitNetForCausalLM, the library the reference validates itself against
(scripts/hf_reference.py:41-58, docs/BENCHMARKS.md:9-13). The fixture and the script that wrote it
are tests/golden/hf_bitnet_decoder.npz and tests/golden/make_decoder_fixture.py; this test needs
neither torch nor transformers.

Bar, in the reference's own terms (lb-run.rs:223-259: top-1 agreement, agreement where the margin
is clear, max / mean |delta logit|):
  * at least 10 of the 14 rows agree with the library to 1e-5 absolute (max|logit| is 1.16): the two
    statements are the same arithmetic up to float32 summation order (measured: 11 rows within 9e-7);
  * every row within 5e-2 of max|logit|, and top-1 equal wherever the library's margin exceeds that.
Why not one tight bound for all rows: per-token int8 quantisation makes the model discontinuous. A
last-bit difference in a normalised activation that sits on a rounding boundary changes one int8
code, and relu^2 followed by the sub-norm (a gain near 100 on this random model) turns that into
1e-2 on the logits of that token and, through the K/V rows it wrote, of the ones after it (measured:
rows 11-13, 1.5e-2 at most). The reference reports the same effect against this library on the real
checkpoint: max |delta logit| 1.556 with full agreement where the margin is clear
(docs/BENCHMARKS.md:9-13)."""
from pathlib import Path

import numpy as np

GOLDEN = Path(__file__).resolve().parent / "golden" / "hf_bitnet_decoder.npz"
TIGHT = 1e-5   # absolute, rows without a flipped activation code
LOOSE = 5e-2   # of max|logit|, every row


def _load():
    fx = np.load(GOLDEN)
    cfg = {k[4:]: fx[k].item() for k in fx.files if k.startswith("cfg_")}
    w = {k: fx[k] for k in fx.files if k.startswith("model.")}
    return cfg, w, fx["tokens"], fx["logits"]


def test_restatement_meets_transformers_bitnet_logits(oracle):
    from oracle import decoder_oracle as D
    cfg, w, tokens, want = _load()
    hd = cfg["hidden_size"] // cfg["num_attention_heads"]
    w["_cos"], w["_sin"] = D.rope_tables(hd, cfg["rope_theta"], cfg["max_position_embeddings"])
    kvh, L, n = cfg["num_key_value_heads"], cfg["num_hidden_layers"], len(tokens)
    kc = [np.zeros((kvh, n, hd), np.float32) for _ in range(L)]
    vc = [np.zeros((kvh, n, hd), np.float32) for _ in range(L)]
    got = np.stack([D.decode_step(cfg, w, int(t), kc, vc, pos, kv_bf16=False) for pos, t in enumerate(tokens)])
    scale = float(np.abs(want).max())
    rep = D.compare_logits(got, want, margin=LOOSE * scale)
    per_row = np.abs(got - want).max(axis=1)
    assert rep["rows"] == n and int((per_row < TIGHT).sum()) >= 10, (per_row, rep)
    assert rep["clear_rows"] >= n // 2 and rep["clear_agree"] == rep["clear_rows"], rep
    assert rep["max_abs_delta"] < LOOSE * scale, rep
    # the SIMD route through the projections gives the same logits bit for bit (same integers, same epilogue)
    kc2 = [np.zeros((kvh, n, hd), np.float32) for _ in range(L)]
    vc2 = [np.zeros((kvh, n, hd), np.float32) for _ in range(L)]
    fast = np.stack([D.decode_step(cfg, w, int(t), kc2, vc2, pos, kv_bf16=False, fast=True) for pos, t in enumerate(tokens)])
    assert np.array_equal(fast.view(np.uint32), got.view(np.uint32))
    print("decoder restatement vs transformers BitNetForCausalLM:", rep)


def test_bf16_cache_stays_close_to_the_f32_cache(oracle):
    """The benchmark configuration keeps the K/V cache in bf16 (the reference and the library keep
    f32). The same sequence with rounded cache rows stays within 5e-2 of max|logit| of the library's
    f32-cache logits (measured 3.3e-2: the rounding moves activation codes, see the module text), with
    top-1 equal where the margin is clear. This bounds what the cache format alone explains."""
    from oracle import decoder_oracle as D
    cfg, w, tokens, want = _load()
    hd = cfg["hidden_size"] // cfg["num_attention_heads"]
    w["_cos"], w["_sin"] = D.rope_tables(hd, cfg["rope_theta"], cfg["max_position_embeddings"])
    kvh, L, n = cfg["num_key_value_heads"], cfg["num_hidden_layers"], len(tokens)
    kc = [np.zeros((kvh, n, hd), np.float32) for _ in range(L)]
    vc = [np.zeros((kvh, n, hd), np.float32) for _ in range(L)]
    got = np.stack([D.decode_step(cfg, w, int(t), kc, vc, pos, kv_bf16=True) for pos, t in enumerate(tokens)])
    scale = float(np.abs(want).max())
    rep = D.compare_logits(got, want, margin=LOOSE * scale)
    assert rep["max_abs_delta"] < LOOSE * scale and rep["clear_agree"] == rep["clear_rows"], rep


def test_greedy_decode_follows_argmax(oracle):
    from oracle import decoder_oracle as D
    cfg, w, tokens, _ = _load()
    hd = cfg["hidden_size"] // cfg["num_attention_heads"]
    w["_cos"], w["_sin"] = D.rope_tables(hd, cfg["rope_theta"], cfg["max_position_embeddings"])
    out = D.greedy_decode(cfg, w, tokens[:5], 4)
    assert len(out) == 4 and all(0 <= t < cfg["vocab_size"] for t in out)
    again = D.greedy_decode(cfg, w, tokens[:5], 4, fast=True)
    assert out == again
