"""One decode step of the BitNet decoder on the GPU against the CPU restatement of
crates/lb-model/src/model.rs:305-374 (oracle/decoder_oracle.py). The projections are bit-exact by
themselves (tested elsewhere); everything between them is float math whose summation order the
reference does not pin, so the bar here is the reference's own end-to-end metrics
(crates/lb-model/src/bin/lb-run.rs:223-259): greedy token equality where the margin is clear, and
max |delta logit| small against the logit range. Tolerance: 2e-3 of max |logit|."""
import json

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _to_oracle_weights(cfg, tensors):
    import torch
    from oracle import decoder_oracle as D
    w = {}
    for k, v in tensors.items():
        w[k] = v.view(torch.int16).numpy().view(np.uint16) if v.dtype == torch.bfloat16 else v.numpy()
    w["_cos"], w["_sin"] = D.rope_tables(cfg.head_dim(), cfg.rope_theta, cfg.max_position_embeddings)
    return w


def _run(cfg, b, steps, ctx, seed=1):
    import torch
    from lemonade_burn_b200 import model
    from oracle import decoder_oracle as D
    tensors = model.random_checkpoint(cfg, seed)
    net = model.BitNet(cfg, tensors, ctx)
    cache = net.new_cache(b=b, cap=cfg.max_position_embeddings)
    w = _to_oracle_weights(cfg, tensors)
    c = cfg.__dict__
    kvh, hd = cfg.num_key_value_heads, cfg.head_dim()
    okc = [[np.zeros((kvh, cfg.max_position_embeddings, hd), np.float32) for _ in range(cfg.num_hidden_layers)] for _ in range(b)]
    ovc = [[np.zeros((kvh, cfg.max_position_embeddings, hd), np.float32) for _ in range(cfg.num_hidden_layers)] for _ in range(b)]
    rng = np.random.default_rng(seed)
    toks = rng.integers(0, cfg.vocab_size, size=(steps, b)).astype(np.int32)
    worst = 0.0
    for s in range(steps):
        logits = net.forward(torch.from_numpy(toks[s]).cuda(), cache)
        greedy = net.argmax(logits).cpu().numpy()
        got = logits.cpu().numpy()
        for bi in range(b):
            ref = D.decode_step(c, w, int(toks[s, bi]), okc[bi], ovc[bi], s)
            scale = np.abs(ref).max()
            err = np.abs(got[bi] - ref).max() / scale
            worst = max(worst, err)
            assert err < TOL, f"step {s} seq {bi}: max |delta logit| / max |logit| = {err}"
            srt = np.sort(ref)
            if srt[-1] - srt[-2] > 4 * TOL * scale:
                assert greedy[bi] == int(np.argmax(ref))
            assert greedy[bi] == int(np.argmax(got[bi]))  # device argmax == first max of its own logits
    assert cache.len == steps
    ctx.check_device_error()
    return worst


def test_small_decoder_batch2(ctx):
    from lemonade_burn_b200 import model
    cfg = model.Config(512, 768, 4, 2, 2, 1000, 1e-5, 500000.0, 16)
    _run(cfg, b=2, steps=6, ctx=ctx)


def test_bitnet_width_two_layers(ctx):
    """Full BitNet-2B4T layer shapes (hidden 2560, 20/5 heads of 128, intermediate 6912), two layers,
    reduced vocabulary, batch 1 and 3."""
    from lemonade_burn_b200 import model
    cfg = model.Config(2560, 6912, 20, 5, 2, 8000, 1e-5, 500000.0, 8)
    _run(cfg, b=1, steps=3, ctx=ctx, seed=2)
    _run(cfg, b=3, steps=2, ctx=ctx, seed=3)


def test_checkpoint_roundtrip_and_format_check(ctx, tmp_path):
    import torch
    from safetensors.torch import save_file
    from lemonade_burn_b200 import model
    cfg = model.Config(512, 768, 4, 2, 1, 500, 1e-5, 500000.0, 8)
    tensors = model.random_checkpoint(cfg, 5)
    model.save_checkpoint(tmp_path, cfg, tensors)
    a = model.BitNet(cfg, tensors, ctx)
    b = model.BitNet.load(tmp_path, ctx)
    tok = torch.tensor([7], dtype=torch.int32, device="cuda")
    la = a.forward(tok, a.new_cache(1, 8))
    lb = b.forward(tok, b.new_cache(1, 8))
    assert torch.equal(la, lb)
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(tmp_path / model.FILE_NAME), metadata={"format": "something-else"})
    with pytest.raises(ValueError, match="not a lemonade-burn ternary file"):   # model.rs:158-161
        model.BitNet.load(tmp_path, ctx)
    bad = dict(cfg.__dict__, hidden_act="silu")
    (tmp_path / "config.json").write_text(json.dumps(bad))
    with pytest.raises(ValueError):
        model.BitNet.load(tmp_path, ctx)


def test_argmax_first_max(ctx):
    import torch
    from lemonade_burn_b200 import model
    cfg = model.Config(512, 768, 4, 2, 1, 500, 1e-5, 500000.0, 8)
    net = model.BitNet(cfg, model.random_checkpoint(cfg, 6), ctx)
    x = torch.full((3, 128256), -1.0, device="cuda")
    x[0, 777] = 5.0; x[0, 90000] = 5.0          # first of two equal maxima
    x[2, 128255] = 0.5
    assert net.argmax(x).cpu().tolist() == [777, 0, 128255]


@pytest.mark.parametrize("total,splits", [(1, 1), (37, 4), (1000, 128), (4097, 128), (300, 512)])
def test_attention_long_context_against_numpy(ctx, total, splits):
    """lbk_attn_decode at contexts the tiny decoders above never reach, slices shorter and longer
    than one pass of the kernel's position loop and empty trailing slices, against softmax(qK/sqrt(d))V
    in float64 (model.rs:343-353). Tolerance 1e-5 absolute on outputs of magnitude <= 1."""
    import torch
    from lemonade_burn_b200 import _lib
    lib = _lib.load()
    b, nh, kvh, hd, cap = 2, 8, 2, 128, max(total, 8)
    g = torch.Generator().manual_seed(total)
    q = torch.randn(b, nh, hd, generator=g)
    k = torch.randn(b, kvh, cap, hd, generator=g).bfloat16()
    v = torch.rand(b, kvh, cap, hd, generator=g).bfloat16()
    pos = torch.tensor([total - 1], dtype=torch.int32)
    qd, kd, vd, pd = q.cuda(), k.cuda(), v.cuda(), pos.cuda()
    scratch = torch.empty(b * nh * splits * (hd + 4), device="cuda")
    out = torch.empty(b, nh * hd, device="cuda")
    rc = lib.lbk_attn_decode(ctx.handle, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), pd.data_ptr(), b, nh, kvh, hd, cap, splits,
                             scratch.data_ptr(), out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    _lib.check(rc)
    got = out.cpu().numpy().reshape(b, nh, hd)
    kf, vf, qf = k.double().numpy()[:, :, :total], v.double().numpy()[:, :, :total], q.double().numpy()
    for h in range(nh):
        s = np.einsum("bd,bpd->bp", qf[:, h], kf[:, h // (nh // kvh)]) / np.sqrt(hd)
        w = np.exp(s - s.max(axis=1, keepdims=True))
        w /= w.sum(axis=1, keepdims=True)
        ref = np.einsum("bp,bpd->bd", w, vf[:, h // (nh // kvh)])
        assert np.abs(got[:, h] - ref).max() < 1e-5
    ctx.check_device_error()


def test_fused_norms_match_their_parts(ctx):
    """lbk_add_rms_norm and lbk_relu2_mul_rms_norm give the bits of the unfused op pairs."""
    import torch
    from lemonade_burn_b200 import _lib
    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    for rows, n in [(1, 2560), (3, 6912), (2, 8192), (5, 512)]:
        g = torch.Generator().manual_seed(n)
        x = torch.randn(rows, n, generator=g).cuda(); y = torch.randn(rows, n, generator=g).cuda()
        w = torch.rand(n, generator=g).cuda() + 0.5
        x1, x2 = x.clone(), x.clone()
        o1, o2 = torch.empty_like(x), torch.empty_like(x)
        assert lib.lbk_add_inplace(ctx.handle, x1.data_ptr(), y.data_ptr(), rows * n, st) == 0
        assert lib.lbk_rms_norm(ctx.handle, x1.data_ptr(), w.data_ptr(), rows, n, 1e-5, o1.data_ptr(), st) == 0
        assert lib.lbk_add_rms_norm(ctx.handle, x2.data_ptr(), y.data_ptr(), w.data_ptr(), rows, n, 1e-5, o2.data_ptr(), st) == 0
        assert torch.equal(x1, x2) and torch.equal(o1, o2)
        a1, a2 = torch.empty_like(x), torch.empty_like(x)
        assert lib.lbk_relu2_mul(ctx.handle, x.data_ptr(), y.data_ptr(), rows * n, a1.data_ptr(), st) == 0
        assert lib.lbk_rms_norm(ctx.handle, a1.data_ptr(), w.data_ptr(), rows, n, 1e-5, a1.data_ptr(), st) == 0
        assert lib.lbk_relu2_mul_rms_norm(ctx.handle, x.data_ptr(), y.data_ptr(), w.data_ptr(), rows, n, 1e-5, a2.data_ptr(), st) == 0
        assert torch.equal(a1, a2)
    bad = torch.empty(1, 8196, device="cuda")
    assert lib.lbk_add_rms_norm(ctx.handle, bad.data_ptr(), bad.data_ptr(), bad.data_ptr(), 1, 8196, 1e-5, bad.data_ptr(), st) != 0
    ctx.check_device_error()


def test_batch_of_twelve_native_equals_mirror(ctx, tmp_path):
    """Nine and more sequences take the norm + quantise kernels and the GEMM path in both the Python
    mirror and the native runtime: same bits from both, and each row within the decoder's bar
    (2e-3 of max |logit|) of the same sequence run alone (other projection kernels, another
    LM-head kernel)."""
    import torch
    from lemonade_burn_b200 import model
    cfg = model.Config(512, 768, 4, 1, 2, 1000, 1e-5, 500000.0, 32)
    tensors = model.random_checkpoint(cfg, 77)
    model.save_checkpoint(tmp_path, cfg, tensors)
    py = model.BitNet.load(tmp_path, ctx)
    nat = model.NativeBitNet(tmp_path, ctx)
    b = 12
    pc, nc = py.new_cache(b, 32), nat.new_cache(b, 32)
    solo = [nat.new_cache(1, 32) for _ in range(2)]
    g = torch.Generator().manual_seed(1)
    for step in range(5):
        toks = torch.randint(0, cfg.vocab_size, (b,), dtype=torch.int32, generator=g).cuda()
        lp = py.forward(toks, pc)
        ln, nxt = nat.decode(toks, nc)
        torch.cuda.synchronize()
        assert torch.equal(ln, lp) and torch.equal(nxt, py.argmax(lp))
        for i, sc in enumerate(solo):
            ref = nat.forward([int(toks[i])], sc)
            got = ln[i].cpu().numpy()
            assert np.abs(got - ref).max() <= TOL * np.abs(ref).max()
    ctx.check_device_error()
    nat.close()


def test_norm_quant_matches_norm_then_quantise(ctx):
    """lbk_norm_quant (the norm of a projection's input with the activation quantiser inside) gives
    the bits of the norm kernel followed by lbk_quantize_acts_dev: int8 rows with their zero padding,
    scales, sums, and the updated residual for the add form."""
    import torch
    from lemonade_burn_b200 import _lib
    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    for rows, n in [(1, 2560), (17, 6912), (40, 8192), (5, 512), (3, 100)]:
        kp = (n + 127) // 128 * 128
        g = torch.Generator().manual_seed(n)
        x = (3.0 * torch.randn(rows, n, generator=g)).cuda(); y = torch.randn(rows, n, generator=g).cuda()
        w = torch.rand(n, generator=g).cuda() + 0.5
        for pre in (1, 2, 3):
            xa, xb = x.clone(), x.clone()
            f = torch.empty_like(x)
            if pre == 1:
                assert lib.lbk_rms_norm(ctx.handle, xa.data_ptr(), w.data_ptr(), rows, n, 1e-5, f.data_ptr(), st) == 0
            elif pre == 2:
                assert lib.lbk_add_rms_norm(ctx.handle, xa.data_ptr(), y.data_ptr(), w.data_ptr(), rows, n, 1e-5, f.data_ptr(), st) == 0
            else:
                assert lib.lbk_relu2_mul_rms_norm(ctx.handle, xa.data_ptr(), y.data_ptr(), w.data_ptr(), rows, n, 1e-5, f.data_ptr(), st) == 0
            q1 = torch.full((rows, kp), 77, dtype=torch.int8, device="cuda"); q2 = q1.clone()
            s1 = torch.empty(rows, device="cuda"); s2 = torch.empty(rows, device="cuda")
            t1 = torch.empty(rows, dtype=torch.int32, device="cuda"); t2 = torch.empty(rows, dtype=torch.int32, device="cuda")
            _lib.check(lib.lbk_quantize_acts_dev(ctx.handle, f.data_ptr(), rows, n, q1.data_ptr(), s1.data_ptr(), t1.data_ptr(), st))
            _lib.check(lib.lbk_norm_quant(ctx.handle, pre, xb.data_ptr(), y.data_ptr(), w.data_ptr(), rows, n, 1e-5, q2.data_ptr(),
                                          s2.data_ptr(), t2.data_ptr(), st))
            assert torch.equal(q1, q2) and torch.equal(s1, s2) and torch.equal(t1, t2) and torch.equal(xa, xb), (rows, n, pre)
    assert not lib.lbk_norm_quant_supported(8196) and not lib.lbk_norm_quant_supported(6)
    ctx.check_device_error()


@pytest.mark.parametrize("m,cols", [(1, 2560), (1, 6912), (2, 6912), (4, 2560), (1, 512)])
def test_projection_with_input_transform(oracle, ctx, m, cols):
    """lbk_ternary_linear_pre against the separate kernels it replaces (norm / residual add / gate,
    then the plain projection). The residual sum is the same float add (bits equal); the norm's sum
    of squares is reduced in another order, which can move a quantised activation by one step, so
    the projections agree to 1 % of the output range rather than bit for bit."""
    import torch
    from lemonade_burn_b200 import _lib, ops
    lib = _lib.load()
    assert ops.pre_supported(m, cols)
    st = torch.cuda.current_stream().cuda_stream
    rows = 384
    rng = np.random.default_rng(cols + m)
    t = rng.choice(np.array([-1, 0, 1], dtype=np.int8), size=(rows, cols), p=[0.3, 0.4, 0.3])
    lin = ops.TernaryLinear(torch.from_numpy(oracle.pack_matrix(t)).cuda(), 40.0, cols, ctx)
    g = torch.Generator().manual_seed(m * 7 + cols)
    x = torch.randn(m, cols, generator=g).cuda()
    y = torch.randn(m, cols, generator=g).cuda()
    w = (torch.rand(cols, generator=g) + 0.5).cuda()
    eps = 1e-5

    def norm(v):
        out = torch.empty_like(v)
        assert lib.lbk_rms_norm(ctx.handle, v.data_ptr(), w.data_ptr(), m, cols, eps, out.data_ptr(), st) == 0
        return out

    def close(a, b):
        tol = 0.01 * float(b.abs().max())
        return float((a - b).abs().max()) <= tol

    got = ops.ternary_linear_pre(ops.PRE_RMS, x, None, w, eps, [lin])[0]
    assert close(got, ops.ternary_linear(norm(x), lin))
    xout = torch.empty_like(x)
    got = ops.ternary_linear_pre(ops.PRE_ADD_RMS, x, y, w, eps, [lin], xout=xout)[0]
    assert torch.equal(xout, x + y)
    assert close(got, ops.ternary_linear(norm(x + y), lin))
    got = ops.ternary_linear_pre(ops.PRE_RELU2_MUL_RMS, x, y, w, eps, [lin])[0]
    assert close(got, ops.ternary_linear(norm(torch.relu(x) ** 2 * y), lin))
    assert not ops.pre_supported(16, 6912)
    with pytest.raises(_lib.LbkError):
        ops.ternary_linear_pre(ops.PRE_RMS, torch.randn(16, cols).cuda(), None, w, eps, [lin]) if not ops.pre_supported(16, cols) else (_ for _ in ()).throw(_lib.LbkError(7, "n/a"))
    ctx.check_device_error()


@pytest.mark.parametrize("total,splits,nh,kvh,b", [(1, 1, 8, 2, 2), (37, 4, 8, 2, 2), (1000, 32, 8, 2, 2), (4097, 130, 20, 5, 2), (300, 256, 16, 2, 2),
                                                  (1, 1, 8, 2, 9), (37, 4, 8, 2, 8), (1000, 3, 16, 2, 9), (1089, 1, 8, 1, 10), (4097, 130, 20, 5, 8),
                                                  (300, 256, 16, 2, 8), (130, 2, 8, 2, 16), (4097, 130, 20, 5, 16)])
def test_fused_attention_against_numpy(ctx, total, splits, nh, kvh, b):
    """lbk_attn_decode_fused (RoPE on q and the new k, append of the new K/V row, slices, merge by the
    last block) against RoPE + softmax(qK/sqrt(d))V in float64, two calls in a row on the same
    buffers (the merge counters must come back to zero). The appended rows must be the bf16 of the
    rotated k and of v. Eight sequences and more take the tensor-core kernel (whole-chunk slices, empty
    slices when there are more slices than chunks, one slice written straight to the output).
    Tolerance 1e-5 absolute on outputs of magnitude <= 1."""
    import torch
    from lemonade_burn_b200 import _lib
    lib = _lib.load()
    assert lib.lbk_attn_decode_fused_supported(nh, kvh, 128, splits)
    hd, cap = 128, max(total, 8)
    g = torch.Generator().manual_seed(total + nh)
    q = torch.randn(b, nh, hd, generator=g)
    kn = torch.randn(b, kvh, hd, generator=g)
    vn = torch.rand(b, kvh, hd, generator=g)
    k = torch.randn(b, kvh, cap, hd, generator=g).bfloat16()
    v = torch.rand(b, kvh, cap, hd, generator=g).bfloat16()
    ang = torch.rand(cap, hd // 2, generator=g) * 6.0
    cos = torch.cat([torch.cos(ang), torch.cos(ang)], dim=1).contiguous()
    sin = torch.cat([torch.sin(ang), torch.sin(ang)], dim=1).contiguous()
    pos = total - 1

    def rope(x):  # model.rs:298-302
        x1, x2 = x[..., :hd // 2], x[..., hd // 2:]
        return x * cos[pos] + torch.cat([-x2, x1], dim=-1) * sin[pos]

    qd, knd, vnd, kd, vd = q.cuda(), kn.cuda(), vn.cuda(), k.cuda(), v.cuda()
    cd, sd, pd = cos.cuda(), sin.cuda(), torch.tensor([pos], dtype=torch.int32).cuda()
    scratch = torch.empty(b * nh * splits * (hd + 4), device="cuda")
    counters = torch.zeros(b * kvh, dtype=torch.int32, device="cuda")
    out = torch.empty(b, nh * hd, device="cuda")
    kref = k.clone(); vref = v.clone()
    kref[:, :, pos] = rope(kn).bfloat16(); vref[:, :, pos] = vn.bfloat16()
    kf, vf = kref.double().numpy()[:, :, :total], vref.double().numpy()[:, :, :total]
    qf = rope(q).double().numpy()
    for _ in range(2):
        out.zero_()
        _lib.check(lib.lbk_attn_decode_fused(ctx.handle, qd.data_ptr(), knd.data_ptr(), vnd.data_ptr(), cd.data_ptr(), sd.data_ptr(),
                                             pd.data_ptr(), b, nh, kvh, hd, cap, splits, kd.data_ptr(), vd.data_ptr(),
                                             scratch.data_ptr(), counters.data_ptr(), out.data_ptr(),
                                             torch.cuda.current_stream().cuda_stream))
        got = out.cpu().numpy().reshape(b, nh, hd)
        assert int(counters.abs().sum()) == 0
        assert torch.equal(kd.cpu()[:, :, pos], kref[:, :, pos]) and torch.equal(vd.cpu()[:, :, pos], vref[:, :, pos])
        for h in range(nh):
            s = np.einsum("bd,bpd->bp", qf[:, h], kf[:, h // (nh // kvh)]) / np.sqrt(hd)
            w = np.exp(s - s.max(axis=1, keepdims=True))
            w /= w.sum(axis=1, keepdims=True)
            ref = np.einsum("bp,bpd->bd", w, vf[:, h // (nh // kvh)])
            assert np.abs(got[:, h] - ref).max() < 1e-5
    ctx.check_device_error()


def test_native_runtime_matches_python_mirror(ctx, tmp_path):
    """lbk_model_load / new_cache / forward / decode (the decoder as a C-ABI runtime) on a checkpoint
    written in lb-convert's format: logits bit-identical to the Python mirror's (same kernels, same
    order) for a prompt fed token by token + generation, a batch of three sequences, and the
    reference's loader checks (model.rs:151-161)."""
    import torch
    from safetensors.torch import save_file
    from lemonade_burn_b200 import _lib, model
    cfg = model.Config(512, 768, 4, 1, 2, 1000, 1e-5, 500000.0, 64)   # 4 query heads per KV head: the fused attention
    tensors = model.random_checkpoint(cfg, 21)
    model.save_checkpoint(tmp_path, cfg, tensors)
    py = model.BitNet.load(tmp_path, ctx)
    nat = model.NativeBitNet(tmp_path, ctx)
    assert nat.cfg.hidden_size == 512 and nat.cfg.num_key_value_heads == 1 and abs(nat.cfg.rope_theta - 500000.0) < 1e-3
    prompt = [5, 77, 901, 3, 42]
    # single sequence: all logits of the prompt, then three greedy steps
    pc = py.new_cache(1, 64)
    ref = []
    for tk in prompt:
        ref.append(py.forward(torch.tensor([tk], dtype=torch.int32, device="cuda"), pc).cpu().numpy()[0])
    nc = nat.new_cache(1, 64)
    got = np.stack([nat.forward([tk], nc) for tk in prompt])   # one token per call: the decode step
    for i in range(len(prompt)):
        assert np.array_equal(got[i].view(np.uint32), ref[i].view(np.uint32))
    assert nat.cache_len(nc) == len(prompt)
    tk = int(np.argmax(got[-1]))
    for _ in range(3):
        lp = py.forward(torch.tensor([tk], dtype=torch.int32, device="cuda"), pc).cpu().numpy()[0]
        ln = nat.forward([tk], nc)
        assert np.array_equal(ln.view(np.uint32), lp.view(np.uint32))
        tk = int(np.argmax(ln))
    # three sequences advancing together
    pc3, nc3 = py.new_cache(3, 16), nat.new_cache(3, 16)
    toks = torch.tensor([9, 500, 31], dtype=torch.int32, device="cuda")
    for _ in range(4):
        lp = py.forward(toks, pc3)
        ln, nxt = nat.decode(toks, nc3)
        torch.cuda.synchronize()
        assert torch.equal(ln, lp)
        assert torch.equal(nxt, py.argmax(lp))
        toks = nxt
    ctx.check_device_error()
    nat.close()
    # loader checks
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(tmp_path / model.FILE_NAME), metadata={"format": "something-else"})
    with pytest.raises(_lib.LbkError, match="not a lemonade-burn ternary file"):
        model.NativeBitNet(tmp_path, ctx)
    model.save_checkpoint(tmp_path, cfg, tensors)
    (tmp_path / "config.json").write_text(json.dumps(dict(cfg.__dict__, hidden_act="silu")))
    with pytest.raises(_lib.LbkError, match="relu2"):
        model.NativeBitNet(tmp_path, ctx)
    (tmp_path / "config.json").write_text(json.dumps(cfg.__dict__))
    del tensors["model.norm.weight"]
    model.save_checkpoint(tmp_path, cfg, tensors)
    with pytest.raises(_lib.LbkError, match="missing"):
        model.NativeBitNet(tmp_path, ctx)


@pytest.mark.parametrize("pos0,n,nh,kvh", [(0, 1, 8, 2), (0, 37, 8, 2), (5, 64, 20, 5), (100, 33, 4, 4), (0, 130, 16, 2), (1024, 1024, 20, 5)])
def test_prefill_rows_against_numpy(ctx, pos0, n, nh, kvh):
    """lbk_rope_kv_append_rows + lbk_attn_prefill (n prompt rows of one sequence at once) against
    RoPE + causal softmax(qK/sqrt(d))V in float64 over a cache that already holds pos0 positions:
    the appended rows must be the bf16 of the rotated k and of v, everything else in the cache
    untouched, and row i sees keys 0..pos0+i. Tolerance 1e-5 absolute on outputs of magnitude <= 1."""
    import torch
    from lemonade_burn_b200 import _lib
    lib = _lib.load()
    b, seq, hd, cap = 2, 1, 128, pos0 + n + 3
    g = torch.Generator().manual_seed(pos0 * 1000 + n)
    q = torch.randn(n, nh, hd, generator=g)
    kn = torch.randn(n, kvh, hd, generator=g)
    vn = torch.rand(n, kvh, hd, generator=g)
    k = torch.randn(b, kvh, cap, hd, generator=g).bfloat16()
    v = torch.rand(b, kvh, cap, hd, generator=g).bfloat16()
    ang = torch.rand(cap, hd // 2, generator=g) * 6.0
    cos = torch.cat([torch.cos(ang), torch.cos(ang)], dim=1).contiguous()
    sin = torch.cat([torch.sin(ang), torch.sin(ang)], dim=1).contiguous()

    def rope(x):  # [n][heads][hd], row i at position pos0 + i (model.rs:298-302)
        x1, x2 = x[..., :hd // 2], x[..., hd // 2:]
        c, s_ = cos[pos0:pos0 + n, None, :], sin[pos0:pos0 + n, None, :]
        return x * c + torch.cat([-x2, x1], dim=-1) * s_

    qd, knd, vnd, kd, vd = q.cuda(), kn.cuda(), vn.cuda(), k.cuda(), v.cuda()
    cd, sd, pd = cos.cuda(), sin.cuda(), torch.tensor([pos0], dtype=torch.int32).cuda()
    out = torch.zeros(n, nh * hd, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.lbk_rope_kv_append_rows(ctx.handle, qd.data_ptr(), knd.data_ptr(), vnd.data_ptr(), cd.data_ptr(), sd.data_ptr(),
                                           pd.data_ptr(), n, nh, kvh, hd, cap, seq, kd.data_ptr(), vd.data_ptr(), st))
    _lib.check(lib.lbk_attn_prefill(ctx.handle, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), pd.data_ptr(), n, nh, kvh, hd, cap, seq,
                                    out.data_ptr(), st))
    torch.cuda.synchronize()
    kref, vref = k.clone(), v.clone()
    kref[seq, :, pos0:pos0 + n] = rope(kn).bfloat16().transpose(0, 1)
    vref[seq, :, pos0:pos0 + n] = vn.bfloat16().transpose(0, 1)
    # v is a plain conversion; the rotated k is two products and a sum whose fusing into an fma the
    # reference does not pin: equal up to one bf16 step, and nearly everywhere exactly
    kgot = kd.cpu()
    assert torch.equal(vd.cpu(), vref)
    assert torch.equal(kgot[1 - seq], k[1 - seq]) and torch.equal(kgot[seq, :, :pos0], k[seq, :, :pos0])
    dk = (kgot.float() - kref.float()).abs()
    assert bool((dk <= kref.float().abs() * 2.0 ** -7 + 1e-30).all()) and float((dk != 0).float().mean()) < 1e-3
    assert int(pd.cpu()[0]) == pos0
    assert (qd.cpu() - rope(q)).abs().max() < 1e-5
    qf = rope(q).double().numpy()
    kf, vf = kgot[seq].double().numpy(), vref[seq].double().numpy()
    got = out.cpu().numpy().reshape(n, nh, hd)
    for h in range(nh):
        kv = h // (nh // kvh)
        sc = qf[:, h] @ kf[kv].T / np.sqrt(hd)                       # [n][cap]
        mask = np.arange(cap)[None, :] <= (pos0 + np.arange(n))[:, None]
        sc = np.where(mask, sc, -np.inf)
        w = np.exp(sc - sc.max(axis=1, keepdims=True))
        w /= w.sum(axis=1, keepdims=True)
        assert np.abs(got[:, h] - w @ vf[kv]).max() < 1e-5
    ctx.check_device_error()


@pytest.mark.parametrize("n,wide,pass_rows", [(2, False, 0), (7, False, 0), (40, False, 0), (300, False, 0), (70, True, 0), (1500, False, 0),
                                              (300, False, 64), (70, True, 17)])
def test_native_prompt_pass_matches_token_by_token(ctx, tmp_path, n, wide, pass_rows):
    """lbk_model_forward with several tokens (one pass of n rows: GEMV batch up to 16 rows, the
    tcgen05 GEMM above; causal attention over the cache) against the same tokens fed one call at a
    time through the decode step, and against the CPU restatement for the first rows. The integer
    projections are the same for both routes; the float summation orders of attention and of the
    LM head differ, so the bar is the decoder's own: max |delta logit| <= 2e-3 of max |logit|, the
    greedy token equal where the margin is clear (the 1500-row case states its own, statistical bar).
    A second prompt pass then continues the same
    cache (positions n..n+4), followed by a decode step. `wide`: BitNet-2B4T layer shapes (hidden 2560,
    20/5 heads, intermediate 6912), two layers, reduced vocabulary. `pass_rows`: rows a pass takes
    (default 4096), so that a prompt goes through several passes."""
    from lemonade_burn_b200 import model
    from oracle import decoder_oracle as D
    cap = 512 if n < 400 else 2048
    cfg = model.Config(2560, 6912, 20, 5, 2, 8000, 1e-5, 500000.0, cap) if wide else model.Config(512, 768, 4, 1, 2, 1000, 1e-5, 500000.0, cap)
    tensors = model.random_checkpoint(cfg, 33)
    model.save_checkpoint(tmp_path, cfg, tensors)
    nat = model.NativeBitNet(tmp_path, ctx)
    if pass_rows:   # several passes per prompt, the last one ragged
        nat.set_prefill_rows(pass_rows)
    rng = np.random.default_rng(n)
    toks = rng.integers(0, cfg.vocab_size, size=n + 6).astype(np.uint32)
    c_seq, c_pf = nat.new_cache(1, cap), nat.new_cache(1, cap)
    ref = np.stack([nat.forward([int(t)], c_seq) for t in toks])

    def close(a, r):
        scale = np.abs(r).max()
        assert np.abs(a - r).max() <= TOL * scale
        srt = np.sort(r)
        if srt[-1] - srt[-2] > 4 * TOL * scale:
            assert int(np.argmax(a)) == int(np.argmax(r))

    got = nat.forward(toks[:n], c_pf, all_logits=True)
    assert got.shape == (n, cfg.vocab_size) and nat.cache_len(c_pf) == n
    if n <= 400:
        for i in range(n):
            close(got[i], ref[i])
    else:
        # Over a thousand rows a few meet an activation that sits on a rounding boundary of the int8
        # quantiser: a 1e-6 difference in the attention sum then moves it by one step (1/127 of the
        # row's maximum), which is worth a few 1e-3 of the logit range in this small model. So: 99 %
        # of the rows inside the bar, every row inside three times the bar.
        err = np.array([np.abs(got[i] - ref[i]).max() / np.abs(ref[i]).max() for i in range(n)])
        assert np.quantile(err, 0.99) <= TOL and err.max() <= 3 * TOL, (np.quantile(err, 0.99), err.max())
    last = nat.forward(toks[n:n + 5], c_pf)              # continues the cache; last row's logits only
    assert nat.cache_len(c_pf) == n + 5
    tail_tol = TOL if n <= 400 else 3 * TOL
    assert np.abs(last - ref[n + 4]).max() <= tail_tol * np.abs(ref[n + 4]).max()
    step = nat.forward([int(toks[n + 5])], c_pf)          # and a decode step on top
    assert np.abs(step - ref[n + 5]).max() <= tail_tol * np.abs(ref[n + 5]).max()
    # the CPU restatement, first rows
    w = _to_oracle_weights(cfg, tensors)
    kvh, hd = cfg.num_key_value_heads, cfg.head_dim()
    okc = [np.zeros((kvh, cap, hd), np.float32) for _ in range(cfg.num_hidden_layers)]
    ovc = [np.zeros((kvh, cap, hd), np.float32) for _ in range(cfg.num_hidden_layers)]
    for i in range(min(n, 2 if wide else 4)):
        close(got[i], D.decode_step(cfg.__dict__, w, int(toks[i]), okc, ovc, i))
    ctx.check_device_error()
    nat.close()


@pytest.fixture(scope="module")
def full_size_net(ctx):
    """The benchmark configuration's decoder: 30 layers, hidden 2560, 20/5 heads of 128, intermediate
    6912, tied 128256-entry bf16 head, random init (seeded, generated on the device)."""
    import torch
    from lemonade_burn_b200 import model
    cfg = model.Config.bitnet_2b4t(layers=30, max_pos=4096 + 64)
    tensors = model.random_checkpoint(cfg, 11, device="cuda")
    net = model.BitNet(cfg, tensors, ctx)
    from oracle import decoder_oracle as D
    w = {}
    for k, v in tensors.items():
        v = v.cpu()
        w[k] = v.view(torch.int16).numpy().view(np.uint16) if v.dtype == torch.bfloat16 else v.numpy()
    w["_cos"], w["_sin"] = D.rope_tables(cfg.head_dim(), cfg.rope_theta, cfg.max_position_embeddings)
    yield cfg, net, w
    del net, tensors
    torch.cuda.empty_cache()


@pytest.mark.parametrize("b", [1, 16])
def test_full_size_step_at_4096_positions_against_oracle(ctx, oracle, full_size_net, b):
    """The decode step of the benchmark configuration at its stated size: a seeded bf16 K/V cache of
    4096 positions per sequence, one step at position 4096 for 1 and for 16 sequences, logits and
    greedy tokens against the CPU restatement fed the same cache (the reference has no batch
    dimension: 16 single-token forwards there). Bar, in the reference's own metrics
    (crates/lb-model/src/bin/lb-run.rs:223-259): greedy token equal wherever the oracle's margin over
    the runner-up exceeds twice the logit tolerance, and max |delta logit| below TOL = 2e-3 of
    max |logit|, the bar of the two-layer tests (measured on a B200: 1.6e-6 at batch 1, 8.8e-5 at
    batch 16, every greedy token equal)."""
    import torch
    from oracle import decoder_oracle as D
    FULL_TOL = TOL
    cfg, net, w = full_size_net
    context, cap = 4096, 4096 + 64
    cache = net.new_cache(b=b, cap=cap)
    g = torch.Generator(device="cuda").manual_seed(100 + b)
    for t in (cache.k, cache.v):
        for li in range(cfg.num_hidden_layers):
            t[li].copy_(torch.randn(t[li].shape, generator=g, device="cuda").to(torch.bfloat16))
    k_bits = cache.k.cpu().view(torch.int16).numpy().view(np.uint16)
    v_bits = cache.v.cpu().view(torch.int16).numpy().view(np.uint16)
    tokens = torch.randint(0, cfg.vocab_size, (b,), dtype=torch.int32, device="cuda", generator=g)
    cache.pos.fill_(context)
    cache.host_len = context
    logits = net.forward(tokens, cache)
    greedy = net.argmax(logits).cpu().numpy()
    got = logits.cpu().numpy()
    ctx.check_device_error()
    assert cache.len == context + 1
    want = D.check_step(cfg.__dict__, w, tokens.cpu().numpy(), k_bits, v_bits, context)
    scale = float(np.abs(want).max())
    rep = D.compare_logits(got, want, margin=2 * FULL_TOL * scale)
    print(f"config 3, batch {b}: {rep}, relative max delta {rep['max_abs_delta'] / scale:.2e}")
    assert rep["max_abs_delta"] < FULL_TOL * scale, rep
    assert rep["clear_agree"] == rep["clear_rows"], rep
    for bi in range(b):
        assert greedy[bi] == int(np.argmax(got[bi]))              # device argmax == first max of its own logits
    # the appended K/V rows are the bf16 of what the oracle appended
    ks = cache.k[:, :, :, context].float().cpu().numpy()           # [layers][b][kvh][hd]
    assert np.isfinite(ks).all() and np.abs(ks).max() > 0


def test_loader_shards_equal_slices_and_failures_are_errors(ctx, tmp_path):
    """lbk_model_load_shard for every rank of 2 and 4 against slicing the full load: q/k/v/gate/up keep a
    row range, o/down a 128-aligned column range, byte for byte, scales equal; the loader holds two
    pinned staging buffers whatever the file's size. Failures become error returns with a message,
    never a crash (the reference turns a failing request into an error reply,
    crates/lb-server/src/main.rs:92-100): a truncated file, a config.json without the fields the
    reference's Config requires (model.rs:22-36), a world size that does not divide the model, and the
    decode step on a shard."""
    import json
    import shutil
    from lemonade_burn_b200 import _lib, model, tp
    cfg = model.Config(1024, 1536, 8, 4, 2, 512, 1e-5, 500000.0, 16)
    model.save_checkpoint(tmp_path, cfg, model.random_checkpoint(cfg, 31))
    full = model.NativeBitNet(tmp_path, ctx)
    st = full.load_stats()
    assert st["staging_bytes"] == 2 * (32 << 20) and st["bytes_read"] == st["bytes_to_device"] > 0 and st["seconds"] > 0
    cols = {"q": 1024, "k": 1024, "v": 1024, "o": 1024, "gate": 1024, "up": 1024, "down": 1536}
    for world in (2, 4):
        for rank in range(world):
            sh = model.NativeBitNet(tmp_path, ctx, rank=rank, world=world)
            for layer in range(cfg.num_hidden_layers):
                for name in ("q", "k", "v", "gate", "up"):
                    assert np.array_equal(sh.linear_bytes(layer, name), tp.shard_rows(full.linear_bytes(layer, name), world, rank))
                for name in ("o", "down"):
                    want, lc = tp.shard_cols(full.linear_bytes(layer, name), cols[name], world, rank)
                    got = sh.linear_bytes(layer, name)
                    assert np.array_equal(got, want) and ctx._lib.lbk_weight_cols(sh.linear_handle(layer, name)) == lc
                for name in ("q", "o", "down"):
                    assert ctx._lib.lbk_weight_scale(sh.linear_handle(layer, name)) == ctx._lib.lbk_weight_scale(full.linear_handle(layer, name))
            assert sh.load_stats()["bytes_to_device"] < st["bytes_to_device"]
            with pytest.raises(_lib.LbkError, match="shard"):
                sh.new_cache(1, 8)
            sh.close()
    full.close()
    with pytest.raises(_lib.LbkError, match="do not divide"):
        model.NativeBitNet(tmp_path, ctx, rank=0, world=8)      # 4 KV heads over 8 ranks
    with pytest.raises(_lib.LbkError):
        model.NativeBitNet(tmp_path, ctx, rank=2, world=2)
    # a file cut short: the header is intact, the data is not
    cut = tmp_path / "cut"
    cut.mkdir()
    shutil.copy(tmp_path / "config.json", cut / "config.json")
    data = (tmp_path / model.FILE_NAME).read_bytes()
    (cut / model.FILE_NAME).write_bytes(data[: len(data) * 2 // 3])
    with pytest.raises(_lib.LbkError, match="truncated"):
        model.NativeBitNet(cut, ctx)
    (cut / model.FILE_NAME).write_bytes(data[:5])
    with pytest.raises(_lib.LbkError, match="truncated"):
        model.NativeBitNet(cut, ctx)
    # config.json without a field the reference requires
    (cut / model.FILE_NAME).write_bytes(data)
    for drop in ("hidden_act", "tie_word_embeddings"):
        raw = dict(cfg.__dict__)
        del raw[drop]
        (cut / "config.json").write_text(json.dumps(raw))
        with pytest.raises(_lib.LbkError, match=drop):
            model.NativeBitNet(cut, ctx)
    ctx.check_device_error()
