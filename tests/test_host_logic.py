"""Host-side logic that needs no GPU: the converter's tensor naming (crates/lb-convert/src/lib.rs:18-47),
its command line (crates/lb-convert/src/main.rs:19-28), and the attention slicing rule that the Python
mirror and the native runtime share."""
import pytest


def test_bitlinear_names():
    from lemonade_burn_b200 import convert
    yes = ["model.layers.0.self_attn.q_proj.weight", "model.layers.29.mlp.down_proj.weight", "model.layers.3.mlp.gate_proj.weight",
           "model.layers.7.self_attn.o_proj.weight"]
    no = ["model.embed_tokens.weight", "model.norm.weight", "model.layers.0.input_layernorm.weight",
          "model.layers.0.self_attn.attn_sub_norm.weight", "model.layers.0.mlp.ffn_sub_norm.weight",
          "layers.0.self_attn.q_proj.weight", "model.layers.0.self_attn.q_proj.bias", "model.layers.0.self_attn.q_proj.qweight"]
    assert all(convert.is_bitlinear_weight(n) for n in yes)
    assert not any(convert.is_bitlinear_weight(n) for n in no)
    assert len(convert.LINEAR_SUFFIXES) == 7
    assert (convert.FORMAT, convert.VERSION, convert.FILE_NAME) == ("lemonade-burn-ternary", "1", "model.lbt.safetensors")


def test_converter_command_line(monkeypatch):
    from lemonade_burn_b200 import convert
    seen = {}
    monkeypatch.setattr(convert, "convert_checkpoint", lambda src, dst, check=None: seen.update(src=src, dst=dst, check=check))
    assert convert.main(["--src", "a", "--dst", "b"]) == 0 and seen == {"src": "a", "dst": "b", "check": None}
    assert convert.main(["--src", "a", "--dst", "b", "--check", "q.json"]) == 0 and seen["check"] == "q.json"
    with pytest.raises(SystemExit):
        convert.main(["--src", "a"])          # --dst is required, as in the reference's parser
    assert convert.convert_bitlinear([]) == []  # nothing to do needs no device


def test_attention_slices():
    from lemonade_burn_b200 import model
    assert model.attention_splits(1) == 1 and model.attention_splits(32) == 1 and model.attention_splits(33) == 2
    assert model.attention_splits(4160) == 130 and model.attention_splits(1 << 20) == 256


def test_cache_refuses_positions_beyond_its_capacity():
    """BitNet::forward asserts pos0 + m <= rope_len (model.rs:309). Here: a cache cannot be larger than
    the RoPE tables, and the host-side length refuses the step that would not fit, before any launch."""
    from lemonade_burn_b200 import model
    cfg = model.Config(256, 384, 2, 1, 1, 100, 1e-5, 500000.0, 8)
    with pytest.raises(ValueError, match="max_position_embeddings"):
        model.KvCache(cfg, 1, 9, "cpu")
    with pytest.raises(ValueError):
        model.KvCache(cfg, 0, 4, "cpu")
    cache = model.KvCache(cfg, 2, 3, "cpu")
    for _ in range(3):
        cache.reserve(1)
        cache.host_len += 1
    with pytest.raises(ValueError, match="cache is full"):
        cache.reserve(1)
    assert cache.host_len == 3


def test_config_json_needs_the_reference_fields(tmp_path):
    """hidden_act and tie_word_embeddings are required members of the reference's Config
    (model.rs:22-36): a config.json without them is refused, like one with another activation."""
    import json
    from lemonade_burn_b200 import model
    cfg = model.Config(256, 384, 2, 1, 1, 100, 1e-5, 500000.0, 8)
    for drop in ("hidden_act", "tie_word_embeddings"):
        raw = dict(cfg.__dict__)
        del raw[drop]
        (tmp_path / "config.json").write_text(json.dumps(raw))
        with pytest.raises(ValueError, match=drop):
            model.BitNet.load(tmp_path, ctx=object())
