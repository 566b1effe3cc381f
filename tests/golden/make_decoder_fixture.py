"""Generates tests/golden/hf_bitnet_decoder.npz: logits of the installed `transformers`
BitNetForCausalLM (random init, CPU, float32, eager attention) on a seeded token sequence, together
with the weights it was run on, already in lb-ternary's packed form.

This is the second, independent statement of the decoder step that pins oracle/decoder_oracle.py:
the reference validates lb-model against exactly this library (scripts/hf_reference.py:41-58,81,
docs/BENCHMARKS.md:9-13; crates/lb-model/src/model.rs:1 calls itself its mirror). The library is
imported and run; none of its source is copied.

How the two sides get the same model: master weights are drawn here (N(0, 0.02), rounded to bf16 like
a released checkpoint). The library's linear layers are swapped for its own AutoBitLinear with
online quantisation, so it ternarises the masters (WeightQuant) and quantises activations (ActQuant)
inside its forward. The packed weights stored for the oracle come from the oracle's own ternariser
on the same masters, and the script checks that both ternarisations give the same ternary values,
element for element, before it writes anything (the per-tensor scale can differ in its last bits:
the library averages |w| in float32, the reference in float64).

Run once where transformers + torch are installed:  python tests/golden/make_decoder_fixture.py
TORCHDYNAMO_DISABLE=1 makes the library's torch.compile-decorated quantisers run eagerly.
"""
import os
import sys

os.environ["TORCHDYNAMO_DISABLE"] = "1"

from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
OUT = Path(__file__).resolve().parent / "hf_bitnet_decoder.npz"

CFG = dict(hidden_size=256, intermediate_size=384, num_attention_heads=2, num_key_value_heads=1, num_hidden_layers=2,
           vocab_size=320, rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=32)
N_TOKENS = 14
LINEARS = ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"]


def build_model():
    """The library's model on seeded weights, and the same weights in the oracle's form."""
    from transformers import BitNetConfig, BitNetForCausalLM
    from transformers.integrations.bitnet import AutoBitLinear, WeightQuant
    from oracle import oracle as o
    o.build()

    torch.manual_seed(1234)
    torch.set_num_threads(1)  # one thread: the library's float sums are then reproducible run to run
    hf_cfg = BitNetConfig(hidden_size=CFG["hidden_size"], intermediate_size=CFG["intermediate_size"],
                          num_attention_heads=CFG["num_attention_heads"], num_key_value_heads=CFG["num_key_value_heads"],
                          num_hidden_layers=CFG["num_hidden_layers"], vocab_size=CFG["vocab_size"], rms_norm_eps=CFG["rms_norm_eps"],
                          max_position_embeddings=CFG["max_position_embeddings"], hidden_act="relu2", tie_word_embeddings=True,
                          rope_parameters={"rope_theta": CFG["rope_theta"], "rope_type": "default"}, attention_bias=False)
    hf_cfg._attn_implementation = "eager"
    model = BitNetForCausalLM(hf_cfg).float().eval()

    g = torch.Generator().manual_seed(77)
    worst_scale = 0.0
    fx = {f"cfg_{k}": np.array(v) for k, v in CFG.items()}

    def bf16_valued(t):
        return t.to(torch.bfloat16).to(torch.float32)

    # swap every projection for the library's online-quantising linear and give it seeded masters
    for li, layer in enumerate(model.model.layers):
        for name in LINEARS:
            parent = layer
            parts = name.split(".")
            for p in parts[:-1]:
                parent = getattr(parent, p)
            old = getattr(parent, parts[-1])
            new = AutoBitLinear(old.in_features, old.out_features, bias=False, online_quant=True)
            master = bf16_valued(torch.randn(old.out_features, old.in_features, generator=g) * 0.02)
            with torch.no_grad():
                new.weight.copy_(master)
            setattr(parent, parts[-1], new)
            # the oracle's ternariser on the same masters (pack.rs:129-142), and the proof that the
            # library's WeightQuant produces the same ternary values and the same scale
            tern, scale = o.ternarize_absmean(master.numpy())
            lib_deq = WeightQuant.apply(master.clone()).numpy()
            assert np.array_equal(np.sign(lib_deq).astype(np.int8), tern), f"layer {li} {name}: WeightQuant and the oracle's ternariser disagree"
            # the library sums |w| in float32, the reference in float64 (pack.rs:131-134): the scale may differ in its last bits
            lib_scale = 1.0 / np.abs(lib_deq).max()
            worst_scale = max(worst_scale, abs(lib_scale / float(scale) - 1.0))
            key = f"model.layers.{li}.{name}"
            fx[key + ".qweight"] = o.pack_matrix(tern)
            fx[key + ".wscale"] = np.array([scale], dtype=np.float32)
        for nm, mod in (("input_layernorm", layer.input_layernorm), ("post_attention_layernorm", layer.post_attention_layernorm),
                        ("self_attn.attn_sub_norm", layer.self_attn.attn_sub_norm), ("mlp.ffn_sub_norm", layer.mlp.ffn_sub_norm)):
            w = (1.0 + 0.1 * torch.randn(mod.weight.shape, generator=g)).float()
            with torch.no_grad():
                mod.weight.copy_(w)
            fx[f"model.layers.{li}.{nm}.weight"] = w.numpy().copy()
    w = (1.0 + 0.1 * torch.randn(model.model.norm.weight.shape, generator=g)).float()
    emb = bf16_valued(torch.randn(CFG["vocab_size"], CFG["hidden_size"], generator=g) * 0.02)
    with torch.no_grad():
        model.model.norm.weight.copy_(w)
        model.model.embed_tokens.weight.copy_(emb)
    model.tie_weights()
    assert model.lm_head.weight.data_ptr() == model.model.embed_tokens.weight.data_ptr(), "the head is not tied to the embedding"
    fx["model.norm.weight"] = w.numpy().copy()
    fx["model.embed_tokens.weight"] = (emb.numpy().view(np.uint32) >> 16).astype(np.uint16)  # bf16 bits

    tokens = torch.randint(0, CFG["vocab_size"], (1, N_TOKENS), generator=g)
    print("largest relative difference between the library's weight scale and the oracle's:", worst_scale)
    return model, fx, tokens


def main():
    model, fx, tokens = build_model()
    with torch.no_grad():
        logits = model(tokens).logits[0].float().numpy()
    fx["tokens"] = tokens[0].numpy().astype(np.int32)
    fx["logits"] = logits.astype(np.float32)
    fx["versions"] = np.array([f"torch {torch.__version__}", f"transformers {__import__('transformers').__version__}"])
    np.savez_compressed(OUT, **fx)
    print("wrote", OUT, OUT.stat().st_size, "bytes; logits", logits.shape, "max |logit|", float(np.abs(logits).max()))


if __name__ == "__main__":
    main()
