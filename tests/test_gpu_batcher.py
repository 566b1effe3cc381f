"""Continuous batching (lbk_batcher_*) and the per-sequence positions under it. The batched decode
step computes every sequence's row independently (per-row quantisation, integer dots, row-wise
norms, one attention problem per sequence), so a request must produce the same tokens whether it
shares the step with others or not: the bar is token equality. Against the single-sequence runtime
(another LM-head kernel: one row instead of several) the first token, which comes from the same
prompt pass, must be equal."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("nh,kvh,splits,b", [(8, 2, 4, 3), (4, 4, 3, 3), (8, 2, 4, 9), (8, 1, 1, 12)])
def test_attention_with_a_position_per_sequence(ctx, nh, kvh, splits, b):
    """lbk_attn_decode_fused_seq (4 query heads per KV head) / lbk_rope_kv_append_seq + lbk_attn_decode_seq
    (one per KV head) with positions 0, 36 and 130 in one batch against RoPE + softmax(qK/sqrt(d))V
    in float64 per sequence; lbk_advance_pos_seq moves only the active ones. Tolerance 1e-5 absolute."""
    import torch
    from lemonade_burn_b200 import _lib
    lib = _lib.load()
    hd, cap = 128, 160
    posv = [0, 36, 130, 63, 64, 65, 1, 159, 100, 17, 128, 5][:b]
    g = torch.Generator().manual_seed(nh)
    q = torch.randn(b, nh, hd, generator=g)
    kn = torch.randn(b, kvh, hd, generator=g)
    vn = torch.rand(b, kvh, hd, generator=g)
    k = torch.randn(b, kvh, cap, hd, generator=g).bfloat16()
    v = torch.rand(b, kvh, cap, hd, generator=g).bfloat16()
    ang = torch.rand(cap, hd // 2, generator=g) * 6.0
    cos = torch.cat([torch.cos(ang), torch.cos(ang)], dim=1).contiguous()
    sin = torch.cat([torch.sin(ang), torch.sin(ang)], dim=1).contiguous()

    def rope(x, pos):
        x1, x2 = x[..., :hd // 2], x[..., hd // 2:]
        return x * cos[pos] + torch.cat([-x2, x1], dim=-1) * sin[pos]

    qd, knd, vnd, kd, vd = q.cuda(), kn.cuda(), vn.cuda(), k.cuda(), v.cuda()
    cd, sd, pd = cos.cuda(), sin.cuda(), torch.tensor(posv, dtype=torch.int32).cuda()
    scratch = torch.empty(b * nh * splits * (hd + 4), device="cuda")
    counters = torch.zeros(b * kvh, dtype=torch.int32, device="cuda")
    out = torch.zeros(b, nh * hd, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    if nh // kvh >= 4:
        _lib.check(lib.lbk_attn_decode_fused_seq(ctx.handle, qd.data_ptr(), knd.data_ptr(), vnd.data_ptr(), cd.data_ptr(), sd.data_ptr(),
                                                 pd.data_ptr(), b, nh, kvh, hd, cap, splits, kd.data_ptr(), vd.data_ptr(),
                                                 scratch.data_ptr(), counters.data_ptr(), out.data_ptr(), st))
    else:
        _lib.check(lib.lbk_rope_kv_append_seq(ctx.handle, qd.data_ptr(), knd.data_ptr(), vnd.data_ptr(), cd.data_ptr(), sd.data_ptr(),
                                              pd.data_ptr(), b, nh, kvh, hd, cap, kd.data_ptr(), vd.data_ptr(), st))
        _lib.check(lib.lbk_attn_decode_seq(ctx.handle, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), pd.data_ptr(), b, nh, kvh, hd, cap,
                                           splits, scratch.data_ptr(), out.data_ptr(), st))
    got = out.cpu().numpy().reshape(b, nh, hd)
    kgot, vgot = kd.cpu(), vd.cpu()
    for bi, pos in enumerate(posv):
        assert torch.equal(vgot[bi, :, pos], vn[bi].bfloat16())
        dk = (kgot[bi, :, pos].float() - rope(kn[bi], pos).bfloat16().float()).abs()
        assert float(dk.max()) <= 2.0 ** -7 * float(kn[bi].abs().max()) * 2
        untouched = [p for p in range(cap) if p != pos]
        assert torch.equal(kgot[bi][:, untouched], k[bi][:, untouched])
        kf, vf = kgot[bi, :, :pos + 1].double().numpy(), vgot[bi, :, :pos + 1].double().numpy()
        qf = rope(q[bi], pos).double().numpy()
        for h in range(nh):
            kv = h // (nh // kvh)
            sc = kf[kv] @ qf[h] / np.sqrt(hd)
            w = np.exp(sc - sc.max())
            w /= w.sum()
            assert np.abs(got[bi, h] - w @ vf[kv]).max() < 1e-5
    act = ([1, 0, 1] + [0] * b)[:b]
    active = torch.tensor(act, dtype=torch.int32).cuda()
    _lib.check(lib.lbk_advance_pos_seq(ctx.handle, pd.data_ptr(), active.data_ptr(), b, st))
    assert pd.cpu().tolist() == [p + a for p, a in zip(posv, act)]
    _lib.check(lib.lbk_advance_pos_seq(ctx.handle, pd.data_ptr(), None, b, st))
    assert pd.cpu().tolist() == [p + a + 1 for p, a in zip(posv, act)]
    ctx.check_device_error()


def test_batcher_tokens_do_not_depend_on_company(ctx, tmp_path):
    """Seven requests of different prompt lengths (1..70 tokens: GEMV and GEMM prompt passes) and
    budgets through three slots: (1) all submitted at once (slots are refilled as requests finish),
    (2) one at a time. Same tokens both ways, the first of each equal to the single-sequence
    runtime's greedy token after the prompt; budgets, the end token and the cache capacity end a
    request; a finished record can be dropped, a running one cannot."""
    from lemonade_burn_b200 import _lib, model
    cfg = model.Config(512, 768, 4, 1, 2, 1000, 1e-5, 500000.0, 96)
    model.save_checkpoint(tmp_path, cfg, model.random_checkpoint(cfg, 5))
    nat = model.NativeBitNet(tmp_path, ctx)
    rng = np.random.default_rng(9)
    lens, budgets = [1, 5, 17, 70, 3, 40, 2], [6, 12, 4, 9, 1, 30, 7]
    prompts = [rng.integers(0, cfg.vocab_size, size=n).astype(np.uint32) for n in lens]

    bt = nat.batcher(3, 96)
    ids = [bt.submit(p, m) for p, m in zip(prompts, budgets)]
    with pytest.raises(_lib.LbkError, match="still running"):
        bt.forget(ids[0])
    steps = bt.run(1000)
    together = []
    for rid, m in zip(ids, budgets):
        toks, done = bt.poll(rid)
        assert done and len(toks) == m
        together.append(toks)
        bt.forget(rid)
    with pytest.raises(_lib.LbkError, match="no request"):
        bt.poll(ids[0])
    assert steps < sum(budgets)           # the requests really shared steps
    alone = []
    for p, m in zip(prompts, budgets):
        rid = bt.submit(p, m)
        bt.run(1000)
        toks, done = bt.poll(rid)
        assert done
        alone.append(toks)
    assert together == alone
    # a prompt that enters its slot in several passes (32 rows at a time, the last one ragged) gives the
    # same bits: every row's projections, attention and norms are computed independently of its neighbours
    nat.set_prefill_rows(32)
    for i in (3, 5, 2):
        rid = bt.submit(prompts[i], budgets[i])
        bt.run(1000)
        assert bt.poll(rid)[0] == together[i]
    nat.set_prefill_rows(4096)
    single = nat.new_cache(1, 96)
    for p, toks in zip(prompts, together):
        nat.reset_cache(single)
        assert int(np.argmax(nat.forward(p, single))) == toks[0]
    # the end token stops a request early; the capacity stops one that asks for too much
    eos = together[5][3]
    rid = bt.submit(prompts[5], 30, eos=eos)
    bt.run(1000)
    toks, done = bt.poll(rid)
    assert done and toks == together[5][:together[5].index(eos) + 1]
    rid = bt.submit(prompts[3], 1000)
    bt.run(1000)
    toks, done = bt.poll(rid)
    assert done and len(toks) == 96 - 70 + 1 and toks[:9] == together[3]
    with pytest.raises(_lib.LbkError, match="does not fit"):
        bt.submit(np.zeros(97, dtype=np.uint32), 1)
    with pytest.raises(_lib.LbkError, match="vocabulary"):
        bt.submit(np.array([cfg.vocab_size], dtype=np.uint32), 1)
    ctx.check_device_error()
    bt.close()
    nat.close()


def test_batcher_tokens_against_the_oracle(ctx, oracle, tmp_path):
    """Requests served by the batcher against the CPU restatement of the reference's generation loop
    (crates/lb-server/src/main.rs:102-166 with greedy sampling, sample.rs:17-25; decoder step
    oracle/decoder_oracle.py). Six slots: batches of 5..8 sequences take the quantise + GEMM route for
    the long-row projection inside the recorded step, and prompts of mixed lengths (1..40 tokens) run
    their own prompt passes on the same context in between, so the recorded step's buffers must stay
    valid while other calls come and go. Teacher-forced check: the oracle is fed the batcher's own
    tokens; at every step the batcher's token must be the oracle's first maximum, or, where float
    rounding could decide (the oracle's lead over the batcher's token is below 2e-3 of max |logit|, the
    decoder tests' bar), at least within that margin."""
    import torch
    from lemonade_burn_b200 import model
    from oracle import decoder_oracle as D
    cfg = model.Config(512, 768, 4, 1, 2, 1000, 1e-5, 500000.0, 64)
    tensors = model.random_checkpoint(cfg, 21)
    model.save_checkpoint(tmp_path, cfg, tensors)
    nat = model.NativeBitNet(tmp_path, ctx)
    w = {k: (v.view(torch.int16).numpy().view(np.uint16) if v.dtype == torch.bfloat16 else v.numpy()) for k, v in tensors.items()}
    w["_cos"], w["_sin"] = D.rope_tables(cfg.head_dim(), cfg.rope_theta, cfg.max_position_embeddings)
    rng = np.random.default_rng(4)
    lens, budgets = [1, 9, 40, 3, 17, 2, 25, 6], [5, 7, 4, 8, 6, 9, 3, 5]
    prompts = [rng.integers(0, cfg.vocab_size, size=n).astype(np.uint32) for n in lens]
    bt = nat.batcher(6, 64)
    ids = [bt.submit(p, m) for p, m in zip(prompts, budgets)]
    bt.run(1000)
    c = cfg.__dict__
    kvh, hd = cfg.num_key_value_heads, cfg.head_dim()
    checked = 0
    for p, m, rid in zip(prompts, budgets, ids):
        toks, done = bt.poll(rid)
        assert done and len(toks) == m
        kc = [np.zeros((kvh, 64, hd), np.float32) for _ in range(cfg.num_hidden_layers)]
        vc = [np.zeros((kvh, 64, hd), np.float32) for _ in range(cfg.num_hidden_layers)]
        seq = [int(t) for t in p] + [int(t) for t in toks[:-1]]
        for pos, tok in enumerate(seq):
            logits = D.decode_step(c, w, tok, kc, vc, pos)
            if pos >= len(p) - 1:
                mine = toks[pos - (len(p) - 1)]
                best = int(np.argmax(logits))
                if mine != best:
                    assert logits[best] - logits[mine] < 2e-3 * np.abs(logits).max(), (rid, pos, mine, best)
                checked += 1
    assert checked == sum(budgets)
    ctx.check_device_error()
    bt.close()
    nat.close()
