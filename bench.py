#!/usr/bin/env python
"""Benchmark of the packed-ternary x int8 decode path: one JSON line per run.

Workload at N=1 ("bitnet2b_decode_sweep"): the BitNet-b1.58-2B4T-shaped decode weight
stream at batch 1 -- 30 layers x (QKV 2560->3840, O 2560->2560, gate/up 2560->2x6912,
down 6912->2560), every group with its own fused per-token int8 activation quantisation,
distinct seeded weights per layer (521 011 200 packed bytes, larger than L2, so every step
streams them from HBM). One step = one whole-model sweep = one token-equivalent, which is how
the reference's own microbenchmark times it (crates/lb-ternary/benches/kbench.rs:148-194).
Weights are i.i.d. ternary with P(-1)=P(+1)=0.3, P(0)=0.4; activations N(0,1); synthetic.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

`value`   tok/s with inputs resident in HBM (CUDA events around exactly K steps)
`e2e`     tok/s through the host-buffer C-ABI call (H2D inputs, sweep, D2H outputs per step)
`roofline` algorithmic bytes per sweep / measured time, against the measured HBM copy peak
`cpu_baseline` the C port of the reference's SIMD kernels on this box's host cores
`--impl reference` times only that CPU port (the reference itself is Rust and cannot be
built where there is no Rust toolchain) and prints the same line with "impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

HIDDEN, INTER, LAYERS = 2560, 6912, 30
GROUPS = [  # (cols, [rows...]) per layer, in the model's order (model.rs:333,359,362,365)
    (HIDDEN, [2560, 640, 640]),
    (HIDDEN, [2560]),
    (HIDDEN, [INTER, INTER]),
    (INTER, [2560]),
]
WSCALE = float(np.float32(1.0) / np.float32(0.02 * np.sqrt(2.0 / np.pi)))  # 1/mean|N(0,0.02)|
METRIC = "decode tok/s (BitNet-2B shape)"
WORKLOAD = "bitnet2b_decode_sweep"


def bench_config(world: int) -> dict:
    """The `config` object of the JSON line, the same keys and values for both arms."""
    return {"workload": WORKLOAD, "layers": LAYERS, "hidden": HIDDEN, "intermediate": INTER, "batch": 1,
            "groups_per_step": LAYERS * len(GROUPS), "packed_weight_bytes": weight_bytes_per_sweep(),
            "l2": "inputs larger than L2 (521 MB of distinct weights per step)",
            "parallelism": "replicas" if world > 1 else "single"}


def weight_bytes_per_sweep() -> int:
    return LAYERS * sum(sum(rows) * cols // 4 for cols, rows in GROUPS)


def algorithmic_bytes_per_sweep() -> int:
    """Packed weights once + f32 input row per group + f32 outputs."""
    io = LAYERS * sum(cols * 4 + sum(rows) * 4 for cols, rows in GROUPS)
    return weight_bytes_per_sweep() + io


# DRAM bytes one sweep moves, from an ncu capture of this same workload (dram__bytes_read.sum +
# dram__bytes_write.sum of one sweep_kernel launch; the summary is kept with the other profile notes).
NCU_TRAFFIC_BYTES_PER_SWEEP = 532_251_904 + 5_107_712


def config0_gemv(torch, ops, ctx, device, copies: int = 64, reps: int = 20):
    """Config 0 (K=2560, N=6912, M=1) as single fused launches, rotating over `copies`
    distinct weight buffers (283 MB, larger than L2) inside one CUDA graph."""
    g = torch.Generator(device=device).manual_seed(4321)
    lins = []
    for _ in range(copies):
        u = torch.rand((4, INTER, HIDDEN // 4), generator=g, device=device)
        codes = (u > 0.3).to(torch.uint8) + (u > 0.7).to(torch.uint8)
        lins.append(ops.TernaryLinear((codes[0] | (codes[1] << 2) | (codes[2] << 4) | (codes[3] << 6)).contiguous(),
                                      WSCALE, HIDDEN, ctx))
        del u, codes
    x = torch.randn(1, HIDDEN, generator=g, device=device)
    for l in lins[:2]:
        ops.ternary_linear(x, l)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for l in lins:
                ops.ternary_linear(x, l)
    torch.cuda.synchronize()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (reps * copies)
    nbytes = INTER * HIDDEN // 4 + HIDDEN * 4 + INTER * 4
    return {"workload": "single fused GEMV K=2560 N=6912 M=1, 64 cold weight copies in one CUDA graph",
            "us_per_call": us, "GBps": nbytes / us / 1e3, "algorithmic_bytes_per_call": nbytes}


def int8_peak(ctx):
    """The int8 tensor-core rate with nothing to load or store (lbk_int8_peak_probe: one kernel, a few
    milliseconds), at the GEMM's token-tile widths. The best of them is the denominator of every
    "fraction of measured int8 peak" in this run; the nominal dense figure of the part is 4500 TOPS."""
    rates = {str(n): ctx.int8_peak_tops(n, 20000) for n in (64, 128, 192, 256)}
    return {"workload": "tcgen05.mma kind::i8, M=128 x N token rows x K=32, operands resident, 20000 x 4 MMAs per SM",
            "TOPS_by_token_rows": rates, "TOPS": max(rates.values()), "nominal_dense_TOPS": 4500.0}


def config2_prefill(torch, ops, ctx, device, peak_tops, ms=(64, 256, 1024, 2048), reps=5, per_graph=10):
    """Config 2: prefill ternary GEMM at the BitNet-2B projections, per token count. One call =
    per-token int8 quantisation kernel + tcgen05 GEMM kernel (`us`, the operator as the decoder calls
    it on f32 activations); beside it the GEMM alone on rows that are quantised already (`gemm_only_us`:
    in the decoder the norm in front of a projection writes the quantised rows itself, so this is the
    projection's cost there). Timed as CUDA-graph replays."""
    import ctypes as C
    from lemonade_burn_b200 import _lib
    g = torch.Generator(device=device).manual_seed(2222)
    out = []

    def timed(call):
        for _ in range(2):
            call(torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for _ in range(per_graph):
                    call(side.cuda_stream)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (reps * per_graph)

    for rows, cols in ((INTER, HIDDEN), (HIDDEN, INTER)):
        u = torch.rand((4, rows, cols // 4), generator=g, device=device)
        codes = (u > 0.3).to(torch.uint8) + (u > 0.7).to(torch.uint8)
        lin = ops.TernaryLinear((codes[0] | (codes[1] << 2) | (codes[2] << 4) | (codes[3] << 6)).contiguous(), WSCALE, cols, ctx)
        del u, codes
        for m in ms:
            x = torch.randn(m, cols, generator=g, device=device)
            y = torch.empty(m, rows, device=device)
            q8 = torch.empty((m, cols), dtype=torch.int8, device=device)
            qs = torch.empty(m, device=device)
            qsum = torch.empty(m, dtype=torch.int32, device=device)
            wp, _k1 = _lib.ptr_array([lin.weight.handle.value])
            op, _k2 = _lib.ptr_array([y.data_ptr()])

            def call(stream):
                _lib.check(ctx._lib.lbk_ternary_linear_n(ctx.handle, C.c_void_p(x.data_ptr()), m, wp, 1, op, None, C.c_void_p(stream)))

            def call_gemm(stream):
                _lib.check(ctx._lib.lbk_ternary_gemm_dev(ctx.handle, wp, 1, C.c_void_p(q8.data_ptr()), C.c_void_p(qs.data_ptr()),
                                                         C.c_void_p(qsum.data_ptr()), m, op, None, C.c_void_p(stream)))

            us = timed(call)
            _lib.check(ctx._lib.lbk_quantize_acts_dev(ctx.handle, C.c_void_p(x.data_ptr()), m, cols, C.c_void_p(q8.data_ptr()), C.c_void_p(qs.data_ptr()),
                                                      C.c_void_p(qsum.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
            us_gemm = timed(call_gemm)
            ops_n = 2.0 * m * rows * cols
            tops = ops_n / us / 1e6
            out.append({"k": cols, "n": rows, "m": m, "us": us, "int8_TOPS": tops,
                        "frac_of_measured_int8_peak": tops / peak_tops, "frac_of_nominal_4500": tops / 4500.0,
                        "gemm_only_us": us_gemm, "gemm_only_int8_TOPS": ops_n / us_gemm / 1e6,
                        "gemm_only_frac_of_measured_int8_peak": ops_n / us_gemm / 1e6 / peak_tops})
    return {"workload": "prefill ternary GEMM, quantise + tcgen05 kernel per call", "peak_TOPS_measured": peak_tops,
            "cases": out}


def config3_decode(torch, ctx, device, batches=(1, 16), steps=20, context=4096, check=True):
    """Config 3: full decode step of a random-init BitNet-b1.58-2B4T-architecture decoder (30 layers,
    20/5 heads of 128, tied 128256-token bf16 head) at position `context` of a seeded bf16 KV cache,
    greedy next token on the device. One CUDA graph per step, replayed `steps` times. Outside the timed
    region the step at position `context` is compared with the CPU restatement of the reference's
    decoder fed the same weights and cache (logits and greedy tokens, the reference's own metrics,
    crates/lb-model/src/bin/lb-run.rs:223-259); at the larger batch the first two sequences are checked."""
    from lemonade_burn_b200 import model
    cfg = model.Config.bitnet_2b4t(max_pos=context + 64)
    tensors = model.random_checkpoint(cfg, 11, device=device)
    net = model.BitNet(cfg, tensors, ctx, device)
    peak, _ = measured_peaks()
    w = None
    if check:
        from oracle import decoder_oracle as D
        w = {}
        for k, v in tensors.items():
            v = v.cpu()
            w[k] = v.view(torch.int16).numpy().view(np.uint16) if v.dtype == torch.bfloat16 else v.numpy()
        w["_cos"], w["_sin"] = D.rope_tables(cfg.head_dim(), cfg.rope_theta, cfg.max_position_embeddings)
    del tensors
    res = []
    for b in batches:
        cache = net.new_cache(b=b, cap=context + 64)
        g = torch.Generator(device=device).manual_seed(100 + b)
        for t in (cache.k, cache.v):  # seeded cache contents, in slabs to bound temporary memory
            for li in range(cfg.num_hidden_layers):
                t[li].copy_(torch.randn(t[li].shape, generator=g, device=device).to(torch.bfloat16))
        tokens = torch.randint(0, cfg.vocab_size, (b,), dtype=torch.int32, device=device, generator=g)
        nxt = torch.zeros(b, dtype=torch.int32, device=device)
        logits_keep = torch.zeros((b, cfg.vocab_size), device=device)
        n_chk = min(b, 2)
        k_bits = v_bits = None
        if check:  # the cache as it is before the step, for the sequences that are checked
            k_bits = cache.k[:, :n_chk].cpu().view(torch.int16).numpy().view(np.uint16)
            v_bits = cache.v[:, :n_chk].cpu().view(torch.int16).numpy().view(np.uint16)

        def step():
            logits = net.forward(tokens, cache)
            logits_keep.copy_(logits)
            nxt.copy_(net.argmax(logits))

        def rewind():
            cache.pos.fill_(context)
            cache.host_len = context

        rewind()
        step()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        rewind()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                step()
        torch.cuda.synchronize()
        rewind()
        graph.replay()
        torch.cuda.synchronize()
        report = None
        if check:
            from oracle import decoder_oracle as D
            want = D.check_step(cfg.__dict__, w, tokens[:n_chk].cpu().numpy(), k_bits, v_bits, context)
            got = logits_keep[:n_chk].cpu().numpy()
            report = D.compare_logits(got, want, margin=4e-3 * float(np.abs(want).max()))
            report["greedy_equal"] = bool(np.array_equal(nxt[:n_chk].cpu().numpy(), want.argmax(axis=1)))
            report["sequences_checked"] = n_chk
            report["relative_max_delta"] = report["max_abs_delta"] / report["max_abs_logit"]
        rewind()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ctx.check_device_error()
        ms = e0.elapsed_time(e1) / steps
        kv_bytes = cfg.num_hidden_layers * 2 * cfg.num_key_value_heads * (context + steps // 2) * cfg.head_dim() * 2 * b
        head_bytes = cfg.vocab_size * cfg.hidden_size * 2 * ((b + 15) // 16)   # the head streams W once per 16 token rows
        nbytes = weight_bytes_per_sweep() + head_bytes + kv_bytes
        gbs = nbytes / (ms * 1e-3) / 1e9
        res.append({"batch": b, "ms_per_step": ms, "tok_per_s": b / (ms * 1e-3), "context": context,
                    "algorithmic_bytes_per_step": nbytes, "GBps": gbs,
                    "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                                 "algorithmic_bytes": {"packed_weights": weight_bytes_per_sweep(), "bf16_head": head_bytes, "bf16_kv_cache": kv_bytes}},
                    "next_tokens": nxt.cpu().tolist()[:4], "check_against_cpu_restatement": report})
        del cache, graph
        torch.cuda.empty_cache()
    return {"workload": "BitNet-2B4T-architecture decode step, random init, bf16 KV cache, greedy", "cases": res}


def config3_prompt(torch, ctx, lengths=(128, 1024, 2048), reps=3):
    """Config 3's other half: a prompt of n tokens through the native runtime (lbk_model_forward:
    checkpoint on disk in the converter's format, up to 4096 rows per pass through the tcgen05 GEMM,
    tensor-core causal attention, last row's logits back on the host). Wall clock around the
    synchronous call, best of `reps`, fresh cache each time."""
    from lemonade_burn_b200 import model
    cfg = model.Config.bitnet_2b4t(max_pos=max(lengths) + 64)
    res = []
    with tempfile.TemporaryDirectory() as d:
        model.save_checkpoint(d, cfg, model.random_checkpoint(cfg, 11))

        def rss_kb(field):
            for line in open("/proc/self/status"):
                if line.startswith(field):
                    return int(line.split()[1])
            return 0

        rss0 = rss_kb("VmRSS:")
        nat = model.NativeBitNet(d, ctx)
        loader = nat.load_stats()
        loader.update(file_bytes=os.path.getsize(os.path.join(d, model.FILE_NAME)), host_rss_growth_bytes=(rss_kb("VmRSS:") - rss0) * 1024,
                      GBps=loader["bytes_read"] / loader["seconds"] / 1e9,
                      note="file -> two 32 MiB pinned buffers -> device; the reference's loader peaks at twice the model in host memory")
        rng = np.random.default_rng(5)
        cache = nat.new_cache(1, max(lengths) + 64)
        for n in lengths:
            toks = rng.integers(0, cfg.vocab_size, size=n).astype(np.uint32)
            times = []
            for _ in range(reps + 1):   # the first pass allocates the work buffers and is not counted
                nat.reset_cache(cache)
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                logits = nat.forward(toks, cache)
                times.append(time.perf_counter() - t0)
            best = min(times[1:])
            res.append({"prompt_tokens": n, "ms": best * 1e3, "tok_per_s": n / best, "next_token": int(np.argmax(logits))})
        serving = batcher_case(torch, nat, rng, cfg)
        nat.close()
    return {"workload": "BitNet-2B4T-architecture prompt pass, native runtime, random init", "cases": res, "batcher": serving, "loader": loader}


def batcher_case(torch, nat, rng, cfg, slots=16, requests=48, prompt=128, new_tokens=64):
    """Continuous batching (lbk_batcher_*): `requests` prompts of `prompt` tokens, `new_tokens` greedy
    tokens each, through `slots` slots; wall clock from the first step to the last. Beside it the same
    requests one after the other through one slot (what the reference's single worker does)."""
    out = {}
    for name, nslots, nreq in (("batched", slots, requests), ("one_at_a_time", 1, max(requests // 8, 2))):
        bt = nat.batcher(nslots, prompt + new_tokens)
        warm = bt.submit(rng.integers(0, cfg.vocab_size, size=prompt).astype(np.uint32), 2)
        bt.run()
        bt.forget(warm)
        ids = [bt.submit(rng.integers(0, cfg.vocab_size, size=prompt).astype(np.uint32), new_tokens) for _ in range(nreq)]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        steps = bt.run()
        dt = time.perf_counter() - t0
        gen = sum(len(bt.poll(i)[0]) for i in ids)
        out[name] = {"slots": nslots, "requests": nreq, "prompt_tokens": prompt, "new_tokens": new_tokens, "steps": steps,
                     "seconds": dt, "generated_tok_per_s": gen / dt, "requests_per_s": nreq / dt}
        bt.close()
    return out


def converter_pass(torch, ctx, device, layers=30):
    """The converter's arithmetic for a whole BitNet-2B4T-shaped model: 7 x `layers` bf16 master
    tensors N(0, 0.02) resident on the device -> scales, packed rows and counts (two launches per
    tensor: f64 absmean, then ternarise + pack). Algorithmic bytes: the masters are read twice and a
    quarter byte per weight is written. The digests are timed apart (a chain per tensor, one GPU
    thread each). Beside it the CPU restatement of the same work on one tensor, one thread."""
    from lemonade_burn_b200 import convert
    from oracle import oracle as O
    shapes = [(2560, 2560), (640, 2560), (640, 2560), (2560, 2560), (6912, 2560), (6912, 2560), (2560, 6912)]
    g = torch.Generator(device=device).manual_seed(17)
    ws = [(0.02 * torch.randn(r, c, generator=g, device=device)).to(torch.bfloat16) for _ in range(layers) for r, c in shapes]
    weights = sum(w.numel() for w in ws)
    convert.convert_bitlinear(ws[:7], ctx, sha=False)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    res = convert.convert_bitlinear(ws, ctx, sha=False)
    dt = time.perf_counter() - t0
    t0 = time.perf_counter()
    convert.convert_bitlinear(ws, ctx, sha=True)
    dt_sha = time.perf_counter() - t0
    w0 = ws[4].float().cpu().numpy()
    t0 = time.perf_counter()
    t, scale = O.ternarize_absmean(w0)
    packed = O.pack_matrix(t)
    dt_cpu = time.perf_counter() - t0
    same = bool(np.array_equal(res[4].packed.cpu().numpy(), packed)) and np.float32(scale).tobytes() == np.float32(res[4].scale).tobytes()
    nbytes = weights * 4.25
    return {"workload": f"{len(ws)} bf16 tensors, {weights} weights", "ms": dt * 1e3, "GBps": nbytes / dt / 1e9,
            "algorithmic_bytes": nbytes, "weights_per_s": weights / dt, "ms_with_sha256": dt_sha * 1e3,
            "cpu_port_one_thread_weights_per_s": w0.size / dt_cpu, "matches_cpu_port": same}


# ---------------------------------------------------------------------------------------
# config 4: 70B-shaped ternary decoder, tensor parallel (column-parallel q/k/v/gate/up,
# row-parallel o/down with an exact int32 all-reduce), batch-64 decode weight sweep
# ---------------------------------------------------------------------------------------
TP_HIDDEN, TP_INTER, TP_LAYERS, TP_KV = 8192, 28672, 80, 1024
TP_BATCH = 64


def tp70b_sweep(torch, dist, ctx, device, world, rank, steps=5, warmup=2, layers=TP_LAYERS, batch=TP_BATCH,
                prefill_tokens=2048, prefill_layers=8):
    """One step = every projection of every layer once at `batch` token rows (no attention / FFN
    math between them, like the reference's KB_MODEL sweep). Row-parallel layers run through the
    two fused peer-memory kernels and, for comparison, through NCCL all-reduces; a 2048-token
    prefill of `prefill_layers` layers (NCCL: the partial dots are too large for the one-shot
    exchange) is timed as well. Returns a dict for the JSON line."""
    from lemonade_burn_b200 import tp

    def rand_packed(rows, rb, gen):  # i.i.d. codes, P(-1) = P(+1) = 0.3, P(0) = 0.4
        v = torch.randint(0, 10, (4, rows, rb), dtype=torch.uint8, device=device, generator=gen)
        codes = (v >= 3).to(torch.uint8) + (v >= 7).to(torch.uint8)
        return codes[0] | (codes[1] << 2) | (codes[2] << 4) | (codes[3] << 6)

    gen = torch.Generator(device=device).manual_seed(777 + rank)
    H, I = TP_HIDDEN, TP_INTER
    lays = []
    for _ in range(layers):
        # shards are generated directly at their local size (no need to build the full matrices)
        lays.append({
            "qkv": [rand_packed(H // world, H // 4, gen), rand_packed(TP_KV // world, H // 4, gen), rand_packed(TP_KV // world, H // 4, gen)],
            "o": rand_packed(H, H // world // 4, gen),
            "gu": [rand_packed(I // world, H // 4, gen), rand_packed(I // world, H // 4, gen)],
            "down": rand_packed(H, I // world // 4, gen),
        })
    comm = tp.TpComm(ctx, world, rank) if world > 1 else None
    mods = []
    for L in lays:
        mods.append((tp.ColumnParallelTernary(L["qkv"], [WSCALE] * 3, H, 1, 0, ctx),
                     tp.RowParallelTernary(L["o"], WSCALE, H // world, 1, 0, ctx=ctx),
                     tp.ColumnParallelTernary(L["gu"], [WSCALE] * 2, H, 1, 0, ctx),
                     tp.RowParallelTernary(L["down"], WSCALE, I // world, 1, 0, ctx=ctx)))
    for _, o_, _, d_ in mods:  # the layers were built from local shards; give them the real world size
        o_.world = world
        d_.world = world
    del lays
    g2 = torch.Generator(device=device).manual_seed(5)

    def timed(tokens, n_layers, use_comm, n_steps):
        x_h = torch.randn(tokens, H, device=device, generator=g2)
        x_o = torch.randn(tokens, H // world, device=device, generator=g2)
        x_d = torch.randn(tokens, I // world, device=device, generator=g2)
        for _, o_, _, d_ in mods:
            o_.comm = comm if use_comm else None
            d_.comm = comm if use_comm else None

        def sweep():
            for qkv, o_, gu, d_ in mods[:n_layers]:
                qkv.forward(x_h)
                o_.forward(x_o)
                gu.forward(x_h)
                d_.forward(x_d)

        for _ in range(warmup):
            sweep()
        torch.cuda.synchronize()
        # one CUDA graph per sweep (kernels and collectives) strips ~1000 host-side launches
        run, mode = sweep, "eager"
        try:
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    sweep()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph.replay()
            torch.cuda.synchronize()
            run, mode = graph.replay, "cuda graph"
        except Exception as exc:  # capture is an optimisation only
            mode = f"eager (graph capture failed: {type(exc).__name__})"
            torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_steps):
            run()
        e1.record()
        torch.cuda.synchronize()
        ctx.check_device_error()
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms[0]) / n_steps, mode

    per_layer = (H + 2 * TP_KV) * H // 4 + H * H // 4 + 2 * I * H // 4 + H * I // 4
    packed_total = layers * per_layer
    ms_step, mode = timed(batch, layers, True, steps)
    res = {"workload": "ternary70b_tp_decode_sweep", "layers": layers, "hidden": H, "intermediate": I, "batch": batch,
           "parallelism": f"tp{world}", "scaling": "strong", "ms_per_step": ms_step,
           "tok_per_s": batch / (ms_step * 1e-3), "int8_TOPS": 2.0 * batch * packed_total * 4 / (ms_step * 1e-3) / 1e12,
           "packed_weight_bytes_total": packed_total, "allreduce_int32_bytes_per_layer": 2 * batch * H * 4,
           "collectives": "two fused peer-memory kernels per row-parallel layer (NVLink loads/stores)" if world > 1 else "none (one rank)",
           "launch": mode, "weights": "i.i.d. ternary codes, P(0)=0.4, drawn per rank at shard size",
           "ms_per_80_layers": ms_step * TP_LAYERS / layers}
    if world > 1:
        ms_nccl, _ = timed(batch, layers, False, steps)
        res["ms_per_step_nccl_allreduce"] = ms_nccl
        res["ms_per_80_layers_nccl_allreduce"] = ms_nccl * TP_LAYERS / layers
    pl = min(prefill_layers, layers)
    ms_pf, mode_pf = timed(prefill_tokens, pl, False, 3)
    res["prefill"] = {"tokens": prefill_tokens, "layers_timed": pl, "ms_per_layer": ms_pf / pl,
                      "ms_per_80_layers": ms_pf / pl * TP_LAYERS,
                      "int8_TOPS_per_gpu": 2.0 * prefill_tokens * per_layer * 4 * pl / world / (ms_pf * 1e-3) / 1e12,
                      "collectives": "NCCL all-reduce (MAX of 2048 floats, SUM of int32 [2048, 8192])" if world > 1 else "none (one rank)",
                      "launch": mode_pf}
    if comm is not None:
        dist.barrier()
        comm.close()
    return res


def tp70b_decoder(torch, dist, ctx, device, world, rank, layers=TP_LAYERS, batch=TP_BATCH, context=1024, steps=5, warmup=2,
                  prefill_tokens=2048):
    """Config 4 as a decoder: hidden 8192, intermediate 28672, 64 Q / 8 KV heads of 128, `layers` layers,
    random init with P(0) = 0.4 (every rank holds slices of the same seeded model). One decode step for
    `batch` sequences at position `context` of a seeded bf16 K/V cache (one CUDA graph per step), and one
    prompt pass of `prefill_tokens` tokens. Sharding: q/k/v/gate/up by rows, o/down by 128-aligned columns,
    attention and K/V cache by heads, the head by vocabulary rows; the exchanges are the library's own
    peer-memory kernels (strong scaling: the work is fixed, the ranks split it). Before the timing one
    row-parallel projection (layer 0's down, all 28672 columns) is compared with the CPU port of the
    reference's kernels on this rank's token rows."""
    from lemonade_burn_b200 import _lib, model, tp
    import ctypes as C
    cap = context + 64
    cfg = model.Config(TP_HIDDEN, TP_INTER, 64, 8, layers, 128256, 1e-5, 500000.0, max(cap, prefill_tokens + 64))
    comm = tp.TpComm(ctx, world, rank)
    t_build = time.perf_counter()
    net = tp.TpBitNet.random_init(cfg, 70, comm, ctx, device, p_zero=0.4)
    torch.cuda.synchronize()
    t_build = time.perf_counter() - t_build
    lib, h = ctx._lib, ctx.handle
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- check: layer 0's down projection through the row-parallel path against the CPU port -------
    from oracle import oracle as o
    o.build()
    H, I = TP_HIDDEN, TP_INTER
    lc = I // world
    full = net._packed_for_check(H, I, 70 * 100003 + 6).cpu().numpy()
    gx = torch.Generator(device=device).manual_seed(4242)
    x = torch.randn(batch, I, generator=gx, device=device)
    xl = x[:, rank * lc:(rank + 1) * lc].contiguous()
    q8 = torch.empty((batch, lc), dtype=torch.int8, device=device)
    sc = torch.empty(batch, device=device)
    sm = torch.empty(batch, dtype=torch.int32, device=device)
    _lib.check(lib.lbk_tp_quantize(comm.handle, C.c_void_p(xl.data_ptr()), batch, lc, C.c_void_p(q8.data_ptr()), C.c_void_p(sc.data_ptr()),
                                   C.c_void_p(sm.data_ptr()), st))
    down = net.layers[0]["down"]
    wp, _k1 = _lib.ptr_array([down.handle])
    ip, _k2 = _lib.ptr_array([comm.partial_ptr])
    _lib.check(lib.lbk_ternary_gemm_dev(h, wp, 1, C.c_void_p(q8.data_ptr()), None, C.c_void_p(sm.data_ptr()), batch, None, ip, st))
    t0, cnt = tp.token_range(batch, world, rank)
    xres = torch.zeros((max(cnt, 1), H), device=device)
    y = torch.zeros((max(cnt, 1), H), device=device)
    gain = torch.ones(H, device=device)
    _lib.check(lib.lbk_tp_reduce_norm_gather(comm.handle, 0, C.c_void_p(sc.data_ptr()), C.c_float(down.scale), C.c_void_p(xres.data_ptr()),
                                             C.c_void_p(gain.data_ptr()), C.c_float(1e-5), batch, H, C.c_void_p(y.data_ptr()), st))
    torch.cuda.synchronize()
    xq, xs, xsum = o.quantize_acts(x.cpu().numpy())
    want = o.simd_gemm_multi([full], [down.scale], xq[t0:t0 + max(cnt, 1)], xs[t0:t0 + max(cnt, 1)], xsum[t0:t0 + max(cnt, 1)])[0][0]
    same = bool(cnt == 0 or np.array_equal(y.cpu().numpy()[:cnt].view(np.uint32), want[:cnt].view(np.uint32)))
    flag = torch.tensor([1 if same else 0], device=device)
    if world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    del full, x, xl, q8, y, xres
    ctx.check_device_error()

    # ---- decode: `batch` sequences at position `context` ----------------------------------------------
    cache = net.new_cache(batch, cap)
    g = torch.Generator(device=device).manual_seed(300 + rank)
    for tsr in (cache["k"], cache["v"]):
        for li in range(layers):
            tsr[li].copy_(torch.randn(tsr[li].shape, generator=g, device=device).to(torch.bfloat16))
    gt = torch.Generator(device=device).manual_seed(9)
    tokens = torch.randint(0, cfg.vocab_size, (batch,), dtype=torch.int32, device=device, generator=gt)

    def rewind():
        cache["pos"].fill_(context)
        cache["host_len"] = [context] * batch

    for _ in range(warmup):
        rewind()
        net.forward(tokens, cache)
    sync_all()
    # per-operation breakdown of one eager step (events between the calls; the graph below has no gaps)
    rewind()
    trace = []
    net.forward(tokens, cache, trace=trace)
    torch.cuda.synchronize()
    by_op = {}
    for (n0, e0_), (n1, e1_) in zip(trace[:-1], trace[1:]):
        by_op[n1] = by_op.get(n1, 0.0) + e0_.elapsed_time(e1_)
    sync_all()
    rewind()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            net.forward(tokens, cache)
    torch.cuda.current_stream().wait_stream(side)
    sync_all()
    rewind()
    graph.replay()
    sync_all()
    rewind()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        graph.replay()
    e1.record()
    sync_all()
    ctx.check_device_error()
    tms = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    ms_step = float(tms[0])
    del graph
    # ---- prompt pass -------------------------------------------------------------------------------------
    pc = net.new_cache(1, prefill_tokens + 64)
    ptoks = torch.randint(0, cfg.vocab_size, (prefill_tokens,), dtype=torch.int32, device=device, generator=gt)

    def prewind():
        pc["pos"].zero_()
        pc["host_len"] = [0]

    prewind()
    net.forward(ptoks, pc, prompt=True)  # eager once: buffers exist before anything is recorded
    sync_all()
    prun, pmode = (lambda: net.forward(ptoks, pc, prompt=True)), "eager"
    try:
        prewind()
        pgraph = torch.cuda.CUDAGraph()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(pgraph, stream=side):
                net.forward(ptoks, pc, prompt=True)
        torch.cuda.current_stream().wait_stream(side)
        prun, pmode = pgraph.replay, "cuda graph"
    except Exception as exc:  # recording is an optimisation only
        pmode = f"eager (graph capture failed: {type(exc).__name__})"
    sync_all()
    times = []
    for rep in range(3):
        prewind()
        sync_all()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        prun()
        p1.record()
        sync_all()
        times.append(p0.elapsed_time(p1))
    ctx.check_device_error()
    # per-operation breakdown of one eager prompt pass
    prewind()
    ptrace = []
    net.forward(ptoks, pc, prompt=True, trace=ptrace)
    torch.cuda.synchronize()
    p_by_op = {}
    for (n0, e0_), (n1, e1_) in zip(ptrace[:-1], ptrace[1:]):
        p_by_op[n1] = p_by_op.get(n1, 0.0) + e0_.elapsed_time(e1_)
    sync_all()
    pms = torch.tensor([min(times[1:])], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(pms, op=dist.ReduceOp.MAX)
    per_layer = (H + 2 * TP_KV) * H // 4 + H * H // 4 + 2 * I * H // 4 + H * I // 4
    kv_bytes = layers * 2 * 8 * (context + 1) * 128 * 2 * batch
    head_bytes = cfg.vocab_size * H * 2 * ((batch + 15) // 16)
    dec_bytes = layers * per_layer + kv_bytes + head_bytes
    peak, _ = measured_peaks()
    res = {"workload": "ternary70b_tp_decoder", "layers": layers, "hidden": H, "intermediate": I, "heads": "64 Q / 8 KV of 128", "vocab": cfg.vocab_size,
           "batch": batch, "context": context, "parallelism": f"tp{world}", "scaling": "strong",
           "decode": {"ms_per_step": ms_step, "tok_per_s": batch / (ms_step * 1e-3), "launch": "cuda graph",
                      "algorithmic_bytes_per_step_all_ranks": dec_bytes, "GBps_per_gpu": dec_bytes / world / (ms_step * 1e-3) / 1e9,
                      "frac_of_measured_hbm_per_gpu": dec_bytes / world / (ms_step * 1e-3) / 1e9 / peak,
                      "eager_step_ms_by_operation_rank0": {k: round(v, 4) for k, v in by_op.items()},
                      "eager_step_ms_rank0": round(sum(by_op.values()), 4)},
           "prefill": {"tokens": prefill_tokens, "ms": float(pms[0]), "tok_per_s": prefill_tokens / (float(pms[0]) * 1e-3),
                       "int8_TOPS_per_gpu": 2.0 * prefill_tokens * per_layer * 4 * layers / world / (float(pms[0]) * 1e-3) / 1e12,
                       "launch": pmode, "eager_ms_by_operation_rank0": {k: round(v, 3) for k, v in p_by_op.items()}},
           "exchange": ("reduce-scatter of int32 partial dots by token rows + all-gather of int8 rows, peer loads/stores in the library's kernels "
                        f"({(world - 1) * batch * H * 4 // world} + {(world - 1) * batch * H // world} bytes per rank and row-parallel layer at decode)") if world > 1
                       else "none (one rank)",
           "check_down_proj_rows_equal_cpu_port_bits": bool(int(flag[0])), "weights": "i.i.d. ternary P(0)=0.4, shared seeds, sliced per rank",
           "build_seconds": t_build}
    del cache, pc, net
    torch.cuda.empty_cache()
    sync_all()
    comm.close()
    return res


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ---------------------------------------------------------------------------------------
# clocks sampling (nvidia-smi in the background during the timed regions)
# ---------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,utilization.gpu,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile(prefix="lbk_clocks_", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.idx)], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def lines(self) -> int:
        try:
            return sum(1 for _ in open(self.path))
        except Exception:
            return 0

    def ensure(self, min_samples: int, load, max_s: float = 3.0) -> bool:
        """A timed region shorter than the sampling period leaves no sample: keep the same load
        running (untimed) until nvidia-smi has reported `min_samples` times. Returns whether the
        load had to be continued."""
        if not self.proc or self.lines() >= min_samples:
            return False
        t0 = time.perf_counter()
        while self.lines() < min_samples and time.perf_counter() - t0 < max_s:
            load()
        return True

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.proc:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = []
        try:
            for line in Path(self.path).read_text().splitlines():
                parts = [p.strip() for p in line.split(",")]
                if len(parts) >= 10:
                    rows.append(parts)
            os.unlink(self.path)
        except Exception:
            pass
        if not rows:
            return out
        def num(v):
            try:
                return float(v)
            except Exception:
                return None
        busy = [r for r in rows if (num(r[4]) or 0) > 0] or rows
        sm = sorted(v for v in (num(r[1]) for r in busy) if v is not None)
        mx = [v for v in (num(r[2]) for r in rows) if v is not None]
        reasons = set()
        for r in busy:
            for name, col in (("hw_slowdown", 6), ("hw_thermal_slowdown", 7), ("sw_thermal_slowdown", 8), ("sw_power_cap", 9)):
                if r[col].lower().startswith("active"):
                    reasons.add(name)
        out.update(sm_mhz=sm[len(sm) // 2] if sm else None, sm_max_mhz=max(mx) if mx else None,
                   reasons=sorted(reasons), samples=len(busy))
        return out


# ---------------------------------------------------------------------------------------
# CPU baseline: the C port of the reference's SIMD kernels (oracle/lbt_simd.c)
# ---------------------------------------------------------------------------------------
def cpu_sweep_baseline(packed_layers, xs, budget_s: float = 12.0, max_layers: int = 30):
    """Times whole-layer passes of the SIMD port on the host cores over a bounded sample of
    the sweep's layers. Returns (tok_per_s, cores, kernel, sample description)."""
    from oracle import oracle as o
    o.build()
    kern = o.simd_best_kernel()
    # every core this process may run on, whatever OMP_NUM_THREADS says (torchrun sets it to 1)
    try:
        threads = len(os.sched_getaffinity(0))
    except AttributeError:
        threads = os.cpu_count() or 1
    n_layers = min(len(packed_layers), max_layers)

    def one_pass():
        for li in range(n_layers):
            for gi, (cols, rows) in enumerate(GROUPS):
                x = xs[li * len(GROUPS) + gi]
                q, s, ssum = o.simd_quantize_acts(x.reshape(1, cols))
                o.simd_gemm_multi(packed_layers[li][gi], [WSCALE] * len(rows), q, s, ssum, kernel=kern, threads=threads)

    one_pass()  # warm (page in)
    t0 = time.perf_counter()
    reps = 0
    while True:
        one_pass()
        reps += 1
        dt = time.perf_counter() - t0
        if dt > budget_s or reps >= 20:
            break
    per_sweep = dt / reps * (LAYERS / n_layers)
    sample = (f"{reps} passes over {n_layers} of {LAYERS} layers "
              f"({n_layers * weight_bytes_per_sweep() // LAYERS} packed bytes per pass), "
              f"{o.simd_kernel_name(kern)} kernel, scaled to a full sweep")
    return 1.0 / per_sweep, threads, o.simd_kernel_name(kern), sample


def host_weights(seed: int, n_layers: int):
    """Seeded packed weights and inputs on the host (for --impl reference, no GPU needed).
    Packed bytes are drawn so that every 2-bit code is i.i.d. with P = (0.3, 0.4, 0.3)."""
    rng = np.random.default_rng(seed)
    layers, xs = [], []
    for li in range(n_layers):
        groups = []
        for cols, rows in GROUPS:
            mats = []
            for r in rows:
                u = rng.random((4, r, cols // 4), dtype=np.float32)
                codes = (u > 0.3).astype(np.uint8) + (u > 0.7).astype(np.uint8)
                mats.append(np.ascontiguousarray(codes[0] | (codes[1] << 2) | (codes[2] << 4) | (codes[3] << 6)))
            groups.append(mats)
            xs.append(rng.standard_normal(cols).astype(np.float32))
        layers.append(groups)
    return layers, xs


def run_reference(args):
    """The reference arm: the CPU implementation of the path on this box's host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    n_layers = 6  # bounded sample: 104 MB of packed weights per pass, well beyond host caches
    layers, xs = host_weights(1234, n_layers)
    budget = min(60.0, max(2.0, 0.05 * args.steps))
    toks, cores, kern, sample = cpu_sweep_baseline(layers, xs, budget_s=budget, max_layers=n_layers)
    line = {
        "impl": "reference", "metric": METRIC, "value": toks, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / toks, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 x ternary -> int32", "data": "synthetic",
        "config": bench_config(int(os.environ.get("WORLD_SIZE", "1"))),
        "cpu_baseline": {"value": toks, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": toks, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "C port of lb-ternary's SIMD kernels (the Rust reference cannot be built: no rustc/cargo here)",
    }
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------------
# ours
# ---------------------------------------------------------------------------------------
def build_sweep(torch, ops, ctx, device, seed: int):
    """Seeded packed weights on the device + a plan of 120 fused groups using plan arenas."""
    g = torch.Generator(device=device).manual_seed(seed)
    plan = ops.Plan(ctx)
    linears = []
    for li in range(LAYERS):
        for cols, rows in GROUPS:
            lins = []
            for r in rows:
                u = torch.rand((4, r, cols // 4), generator=g, device=device)
                codes = (u > 0.3).to(torch.uint8) + (u > 0.7).to(torch.uint8)
                packed = codes[0] | (codes[1] << 2) | (codes[2] << 4) | (codes[3] << 6)
                lins.append(ops.TernaryLinear(packed.contiguous(), WSCALE, cols, ctx))
                del u, codes
            plan.add_arena(lins)
            linears.append(lins)
    plan.finalize()
    return plan, linears


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        # a rank that fails must not leave the others waiting for ten minutes: collectives give up after five
        from datetime import timedelta
        dist.init_process_group("nccl", device_id=device, timeout=timedelta(seconds=300))

    from lemonade_burn_b200 import ops, ternary
    ctx = ternary.Context(local)
    plan, linears = build_sweep(torch, ops, ctx, device, 1234 + rank)
    nx, ny = plan.input_elems(), plan.output_elems()
    x_host = torch.randn(nx, generator=torch.Generator().manual_seed(99 + rank)).pin_memory()
    y_host = torch.empty(ny, dtype=torch.float32).pin_memory()
    torch.cuda.synchronize()
    plan.run_host(x_host, y_host)  # also fills the arena; warms everything once
    ctx.check_device_error()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()

    # ---- device-timed: inputs resident, exactly K steps ---------------------------------
    torch.cuda.profiler.start()  # `ncu --profile-from-start off` skips the set-up; use --extras none to list the sweep alone
    for _ in range(args.warmup):
        plan.run()
    barrier()
    launches0 = ctx.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        plan.run()
    e1.record()
    barrier()
    launches = ctx.launch_count() - launches0
    dev_ms = e0.elapsed_time(e1)
    ctx.check_device_error()

    # ---- end to end: host buffers through the C ABI, copies inside the timed region --------
    for _ in range(min(args.warmup, 10)):
        plan.run_host(x_host, y_host)
    barrier()
    e2e_steps = args.steps
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        plan.run_host(x_host, y_host)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier()

    continued = False
    if rank == 0:
        def same_load():
            for _ in range(200):
                plan.run()
            torch.cuda.synchronize()
        continued = sampler.ensure(4, same_load)
    clocks = sampler.stop() if rank == 0 else {}
    if rank == 0:
        clocks["sampled"] = ("during the timed region and an untimed continuation of the same load"
                             if continued else "during the timed region")

    sustained = None
    if rank == 0 and "sustained" in args.extras:
        # The headline's timed region is a burst of a few milliseconds. The same launch repeated for more
        # than two seconds shows what the part holds once the power cap has had time to act.
        n_sus = max(1000, int(2.5 / (dev_ms * 1e-3 / args.steps)))
        sus = ClockSampler(local)
        sus.start()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(n_sus):
            plan.run()
        s1.record()
        torch.cuda.synchronize()
        sus_clocks = sus.stop()
        sus_ms = s0.elapsed_time(s1) / n_sus
        sus_gbs = algorithmic_bytes_per_sweep() / (sus_ms * 1e-3) / 1e9
        sustained = {"steps": n_sus, "seconds": sus_ms * n_sus * 1e-3, "ms_per_step": sus_ms, "tok_per_s": 1e3 / sus_ms, "GBps": sus_gbs,
                     "clocks": sus_clocks,
                     "us_times_median_sm_mhz": (sus_ms * 1e3 * sus_clocks["sm_mhz"]) if sus_clocks.get("sm_mhz") else None}

    times = torch.tensor([dev_ms, e2e_s * 1e3], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = float(times[0]), float(times[1])

    if rank == 0:
        tok_s = world * args.steps / (dev_ms * 1e-3)
        e2e_tok_s = world * e2e_steps / (e2e_ms * 1e-3)
        peak, peak_kind = measured_peaks()
        sweep_s = dev_ms * 1e-3 / args.steps
        achieved = algorithmic_bytes_per_sweep() / sweep_s / 1e9
        # CPU baseline on this box's host cores: same weights, a bounded sample of layers
        n_cpu_layers = 6
        packed_layers = []
        xs = []
        xh = x_host.numpy()
        off = 0
        for li in range(n_cpu_layers):
            groups = []
            for gi, (cols, rows) in enumerate(GROUPS):
                groups.append([l.packed.cpu().numpy() for l in linears[li * len(GROUPS) + gi]])
            packed_layers.append(groups)
        for li in range(LAYERS):
            for cols, rows in GROUPS:
                xs.append(xh[off:off + cols].copy())
                off += cols
        cpu_toks, cores, kern, sample = cpu_sweep_baseline(packed_layers, xs, budget_s=10.0, max_layers=n_cpu_layers)
        extra = {}
        if sustained is not None:
            sustained["frac_of_measured_hbm"] = sustained["GBps"] / peak
            sustained["frac_of_nominal_8TBs"] = sustained["GBps"] / 8000.0
            sustained["burst_us_times_median_sm_mhz"] = (sweep_s * 1e6 * clocks["sm_mhz"]) if clocks.get("sm_mhz") else None
            extra["sustained"] = sustained

        def side(name, fn):
            """A side measurement must not cost the headline line (measured above): its failure is reported in its place."""
            try:
                extra[name] = fn()
            except Exception as exc:  # e.g. no room for the prompt case's checkpoint in the temp directory
                extra[name] = {"error": f"{type(exc).__name__}: {exc}"}
            torch.cuda.empty_cache()

        if "config0" in args.extras:
            side("config0_gemv", lambda: config0_gemv(torch, ops, ctx, device))
        if "config2" in args.extras:
            side("int8_peak", lambda: int8_peak(ctx))
            peak_tops = extra["int8_peak"].get("TOPS", 4500.0) if isinstance(extra.get("int8_peak"), dict) else 4500.0
            side("config2_prefill", lambda: config2_prefill(torch, ops, ctx, device, peak_tops))
    del plan, linears
    torch.cuda.empty_cache()
    if rank == 0 and world == 1 and "config3" in args.extras:
        side("config3_decode", lambda: config3_decode(torch, ctx, device, batches=tuple(args.decode_batches)))
        side("config3_prompt", lambda: config3_prompt(torch, ctx))
    if rank == 0 and world == 1 and "convert" in args.extras:
        side("converter", lambda: converter_pass(torch, ctx, device))
    tp_res = tp_dec = None
    if "tp" in args.extras:
        # config 4 at every N (N = 1 is the base of the strong-scaling curve): the decoder with the
        # library's own exchanges, then the projection sweep through NCCL all-reduces beside it
        try:
            tp_dec = tp70b_decoder(torch, dist, ctx, device, world, rank, layers=args.tp_layers)
        except Exception as exc:
            tp_dec = {"error": f"{type(exc).__name__}: {exc}"}
        torch.cuda.empty_cache()
        if args.tp70b or world > 1:
            try:
                tp_res = tp70b_sweep(torch, dist, ctx, device, world, rank, layers=min(args.tp_layers, 16), prefill_layers=4)
            except Exception as exc:
                tp_res = {"error": f"{type(exc).__name__}: {exc}"}
    if rank == 0:
        if tp_dec is not None:
            extra["tp70b"] = tp_dec
        if tp_res is not None:
            extra["tp70b_projection_sweep_nccl"] = tp_res
        line = {
            "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8 x ternary -> int32", "data": "synthetic",
            "config": bench_config(world),
            "e2e": {"value": e2e_tok_s, "unit": "tok/s", "h2d_bytes_per_step": nx * 4, "d2h_bytes_per_step": ny * 4},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": NCU_TRAFFIC_BYTES_PER_SWEEP, "peak_kind": peak_kind,
                         "kernel": "sweep_kernel (one launch per step)",
                         "algorithmic_bytes_per_step": algorithmic_bytes_per_sweep(),
                         "frac_of_nominal_8TBs": achieved / 8000.0},
            "cpu_baseline": {"value": cpu_toks, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
            "extra": extra,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--tp70b", action="store_true", help="also time the 70B-shaped tensor-parallel sweep at N=1")
    ap.add_argument("--tp-layers", type=int, default=TP_LAYERS)
    ap.add_argument("--extras", default="sustained,config0,config2,config3,convert,tp",
                    help="side measurements to add under `extra` (comma list of sustained, config0, config2, config3, convert, tp; "
                         "'none' for a profiler run)")
    ap.add_argument("--decode-batches", type=int, nargs="+", default=[1, 16], help="batch sizes of the config-3 decode step")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    args.extras = set(args.extras.split(","))
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
