"""The converter on the GPU (lbk_convert_bitlinear, lemonade_burn_b200.convert) against the CPU
restatement of lb-ternary's ternariser and packer (oracle: pack.rs:88-103,129-142) and against
hashlib's sha256 of the int8 ternary array, the value lb-convert's --check compares
(crates/lb-convert/src/main.rs:73-78,141-170). Everything here is integer or a single correctly
rounded f32: the bar is bit equality (scale bits, packed bytes, counts, digest)."""
import hashlib
import json

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _check(oracle, ctx, w_t, sha=True):
    """w_t: list of torch CPU tensors (f32 or bf16)."""
    import torch
    from lemonade_burn_b200 import convert
    res = convert.convert_bitlinear([w.cuda() for w in w_t], ctx, sha=sha)
    assert len(res) == len(w_t)
    for w, c in zip(w_t, res):
        wf = w.float().numpy()
        t, scale = oracle.ternarize_absmean(wf)
        assert np.float32(c.scale).tobytes() == np.float32(scale).tobytes(), (c.scale, scale, w.shape)
        assert np.array_equal(c.packed.cpu().numpy(), oracle.pack_matrix(t)), w.shape
        assert c.counts == (int((t == -1).sum()), int((t == 0).sum()), int((t == 1).sum()))
        if sha:
            assert c.sha256 == hashlib.sha256(t.tobytes()).hexdigest(), w.shape
        else:
            assert c.sha256 is None
    return res


def test_ternarize_matches_torch_semantics(oracle, ctx):
    """pack.rs:164-170: mean|w| = 1 -> scale 1; 0.5 -> 0 (half to even), 1.5 -> 2 -> clamp 1, -0.5 -> -0."""
    import torch
    w = torch.tensor([[0.5, 1.5, -0.5, -2.0, 0.0, 1.5]], dtype=torch.float32)
    (c,) = _check(oracle, ctx, [w])
    assert float(c.scale) == 1.0
    assert oracle.unpack_matrix(c.packed.cpu().numpy(), 6)[0, :6].tolist() == [0, 1, 0, -1, 0, 1]
    assert not oracle.unpack_matrix(c.packed.cpu().numpy(), 6)[0, 6:].any()   # padding decodes to zero weights (pack.rs:158-160)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_ragged_shapes_one_call(oracle, ctx, dtype):
    """Widths that are no multiple of 4, 32 or 128 (the pack round trip's cols of pack.rs:151), one
    row and many, all in ONE call (the tensors hash side by side), message lengths around the sha256
    padding boundaries (55, 56, 63, 64, 119 bytes)."""
    import torch
    g = torch.Generator().manual_seed(7)
    shapes = [(3, 1), (3, 31), (1, 55), (1, 56), (7, 9), (1, 64), (7, 17), (3, 128), (5, 129), (7, 300), (3, 512), (64, 2560), (9, 6912)]
    ws = [(0.02 * torch.randn(r, c, generator=g)) for r, c in shapes]
    if dtype == "bf16":
        ws = [w.bfloat16() for w in ws]
    _check(oracle, ctx, ws)
    _check(oracle, ctx, ws[:3], sha=False)


def test_zero_and_tie_tensors(oracle, ctx):
    """All zeros: mean 0 -> scale 1/1e-5 (pack.rs:131), all codes zero. Exact ties: values k/2 * m
    with mean|w| = m a power of two, so w * scale lands on .5 exactly and must round to even."""
    import torch
    z = torch.zeros(4, 200)
    (cz,) = _check(oracle, ctx, [z])
    assert np.float32(cz.scale) == np.float32(1.0) / np.float32(1e-5) and cz.counts == (0, 800, 0)
    base = torch.tensor([0.5, -0.5, 1.5, -1.5, 2.5, -2.5, 1.0, -1.0, 1.0, 0.0, 0.0, 0.0])   # mean|.| = 1
    w = (base * 0.25).repeat(50).reshape(20, 30)
    (ct,) = _check(oracle, ctx, [w])
    assert float(ct.scale) == 4.0


def test_bitnet_shapes_bf16(oracle, ctx):
    """Full projection shapes of the 2B4T architecture from bf16 masters N(0, 0.02): q (2560x2560)
    with its digest, gate (6912x2560) and down (2560x6912) without (the digest chain of 17.7 M
    weights is a second of one GPU thread)."""
    import torch
    g = torch.Generator().manual_seed(11)
    q = (0.02 * torch.randn(2560, 2560, generator=g)).bfloat16()
    _check(oracle, ctx, [q])
    gate = (0.02 * torch.randn(6912, 2560, generator=g)).bfloat16()
    down = (0.02 * torch.randn(2560, 6912, generator=g)).bfloat16()
    res = _check(oracle, ctx, [gate, down], sha=False)
    tot = sum(res[0].counts)
    assert tot == 6912 * 2560 and 0.25 < res[0].counts[1] / tot < 0.5   # roughly a third zeros


def test_convert_checkpoint_end_to_end(oracle, ctx, tmp_path):
    """A bf16 source checkpoint in the source naming -> model.lbt.safetensors: every tensor as the
    format says (lb-convert/src/lib.rs:1-16), --check against a summary (identical; then one
    digest spoiled -> exit status 2 as main.rs:166-168), an unexpected tensor refused
    (main.rs:105), and the result loads and runs in the native runtime."""
    import torch
    from safetensors.torch import load_file, save_file
    from lemonade_burn_b200 import convert, model
    cfg = model.Config(512, 768, 4, 2, 2, 1000, 1e-5, 500000.0, 32)
    g = torch.Generator().manual_seed(3)
    hd = cfg.head_dim()
    shapes = {"self_attn.q_proj": (cfg.num_attention_heads * hd, 512), "self_attn.k_proj": (cfg.num_key_value_heads * hd, 512),
              "self_attn.v_proj": (cfg.num_key_value_heads * hd, 512), "self_attn.o_proj": (512, cfg.num_attention_heads * hd),
              "mlp.gate_proj": (768, 512), "mlp.up_proj": (768, 512), "mlp.down_proj": (512, 768)}
    src = {}
    for i in range(cfg.num_hidden_layers):
        for nm, (r, c) in shapes.items():
            src[f"model.layers.{i}.{nm}.weight"] = (0.02 * torch.randn(r, c, generator=g)).bfloat16()
        for nm, sz in (("input_layernorm", 512), ("post_attention_layernorm", 512), ("self_attn.attn_sub_norm", 512), ("mlp.ffn_sub_norm", 768)):
            src[f"model.layers.{i}.{nm}.weight"] = (1.0 + 0.05 * torch.randn(sz, generator=g)).bfloat16()
    src["model.norm.weight"] = (1.0 + 0.05 * torch.randn(512, generator=g)).bfloat16()
    src["model.embed_tokens.weight"] = (0.02 * torch.randn(cfg.vocab_size, 512, generator=g)).bfloat16()
    sdir, ddir = tmp_path / "src", tmp_path / "dst"
    sdir.mkdir()
    save_file(src, str(sdir / "model.safetensors"))
    (sdir / "config.json").write_text(json.dumps(cfg.__dict__))
    summary = {}
    for name, w in src.items():
        if convert.is_bitlinear_weight(name):
            t, scale = oracle.ternarize_absmean(w.float().numpy())
            summary[name] = {"scale": float(scale), "sha256": hashlib.sha256(t.tobytes()).hexdigest()}
    (tmp_path / "quant_summary.json").write_text(json.dumps(summary))
    import io
    log = io.StringIO()
    qinfo = convert.convert_checkpoint(sdir, ddir, check=tmp_path / "quant_summary.json", ctx=ctx, log=log)
    assert f"check vs torch: {len(summary)}/{len(summary)} identical, 0 scale mismatches, 0 ternary mismatches" in log.getvalue()
    assert set(qinfo) == set(summary)
    out = load_file(str(ddir / convert.FILE_NAME))
    for name, w in src.items():
        if convert.is_bitlinear_weight(name):
            lin = name[:-len(".weight")]
            t, scale = oracle.ternarize_absmean(w.float().numpy())
            assert np.array_equal(out[lin + ".qweight"].numpy(), oracle.pack_matrix(t))
            assert out[lin + ".wscale"].dtype == torch.float32 and out[lin + ".wscale"].numpy().tobytes() == np.float32(scale).tobytes()
        elif name.endswith("norm.weight"):
            assert out[name].dtype == torch.float32 and torch.equal(out[name], w.float())
        else:
            assert out[name].dtype == torch.bfloat16 and torch.equal(out[name], w)
    assert (ddir / "config.json").exists()
    nat = model.NativeBitNet(ddir, ctx)
    logits = nat.forward([1, 2, 3], nat.new_cache(1, 32))
    assert logits.shape == (cfg.vocab_size,) and np.isfinite(logits).all()
    nat.close()
    first = next(iter(summary))
    summary[first]["sha256"] = "0" * 64
    (tmp_path / "bad.json").write_text(json.dumps(summary))
    with pytest.raises(SystemExit) as e:
        convert.convert_checkpoint(sdir, tmp_path / "dst2", check=tmp_path / "bad.json", ctx=ctx, log=io.StringIO())
    assert e.value.code == 2
    src["lm_head.weight"] = src["model.embed_tokens.weight"].clone()
    save_file(src, str(sdir / "model.safetensors"))
    with pytest.raises(ValueError, match="unexpected tensor"):
        convert.convert_checkpoint(sdir, tmp_path / "dst3", ctx=ctx, log=io.StringIO())
    ctx.check_device_error()
