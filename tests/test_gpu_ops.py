"""Device-resident ops (torch CUDA tensors in, CUDA tensors out) against the oracle:
ternary_linear / ternary_linear2 / ternary_linear3 / bf16_linear (crates/lb-model/src/ops.rs)
and a recorded plan of decode groups (the reference's per-token loop of fused ops)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def make_linear(o, rows, cols, seed, ctx, scale=None):
    import torch
    from lemonade_burn_b200 import ops
    rng = np.random.default_rng(seed)
    t = rng.choice(np.array([-1, 0, 1], dtype=np.int8), size=(rows, cols), p=[0.3, 0.4, 0.3])
    p = o.pack_matrix(t)
    ws = np.float32(scale if scale is not None else 1.0 / (0.02 * 0.8))
    lin = ops.TernaryLinear(torch.from_numpy(p).cuda(), float(ws), cols, ctx)
    return lin, p, ws


@pytest.mark.parametrize("m", [1, 2, 8, 9, 16])
def test_ternary_linear3_qkv(oracle, ctx, m):
    import torch
    from lemonade_burn_b200 import ops
    cols = 2560
    lins = [make_linear(oracle, r, cols, 10 + i, ctx, sc) for i, (r, sc) in enumerate([(2560, 41.0), (640, 57.5), (640, 63.25)])]
    x = np.random.default_rng(m).standard_normal((m, cols)).astype(np.float32)
    outs, iouts = ops.ternary_linear_multi(torch.from_numpy(x).cuda(), [l for l, _, _ in lins], want_i32=True)
    torch.cuda.synchronize()
    q, s, ssum = oracle.quantize_acts(x)
    wf, wi = oracle.simd_gemm_multi([p for _, p, _ in lins], [w for _, _, w in lins], q, s, ssum, want_i32=True)
    for o_, i_, ef, ei in zip(outs, iouts, wf, wi):
        assert np.array_equal(i_.cpu().numpy(), ei)
        assert np.array_equal(o_.cpu().numpy().view(np.uint32), ef.view(np.uint32))
    three = ops.ternary_linear3(torch.from_numpy(x).cuda(), [l for l, _, _ in lins])
    single = ops.ternary_linear(torch.from_numpy(x).cuda(), lins[1][0])
    assert torch.equal(three[1], single)  # fused == separate, bit for bit (ops.rs:27-29)
    ctx.check_device_error()


@pytest.mark.parametrize("cols", [2560, 6912])
@pytest.mark.parametrize("m", [5, 9, 12, 16])
def test_fused_kernel_forced_up_to_16_rows(oracle, ctx, m, cols):
    """By default 9..16 token rows (and 5..8 of long rows) go to quantise + GEMM; lbk_set_gemv_rows(16)
    sends them to the fused few-row kernel's second token tile instead. Both must give the oracle's
    bits, and the setting must be undone by 0."""
    import torch
    from lemonade_burn_b200 import ops
    lins = [make_linear(oracle, r, cols, 40 + i, ctx, sc) for i, (r, sc) in enumerate([(1040, 41.0), (656, 57.5)])]
    x = np.random.default_rng(m + cols).standard_normal((m, cols)).astype(np.float32)
    q, s, ssum = oracle.quantize_acts(x)
    wf, wi = oracle.simd_gemm_multi([p for _, p, _ in lins], [w for _, _, w in lins], q, s, ssum, want_i32=True)
    xd = torch.from_numpy(x).cuda()
    try:
        for forced in (16, 0):
            ctx.set_gemv_rows(forced)
            before = ctx.launch_count()
            outs, iouts = ops.ternary_linear_multi(xd, [l for l, _, _ in lins], want_i32=True)
            torch.cuda.synchronize()
            launches = ctx.launch_count() - before
            fused_by_default = m <= 4 or (m <= 8 and cols < 4096)   # the measured rule of lbk_ternary_linear_n
            assert (launches == 1) if (forced or fused_by_default) else (launches >= 2), "one fused launch, or quantise + GEMM"
            for o_, i_, ef, ei in zip(outs, iouts, wf, wi):
                assert np.array_equal(i_.cpu().numpy(), ei)
                assert np.array_equal(o_.cpu().numpy().view(np.uint32), ef.view(np.uint32))
    finally:
        ctx.set_gemv_rows(0)
    with pytest.raises(Exception):
        ctx.set_gemv_rows(17)
    ctx.check_device_error()


def test_ternary_linear2_gate_up_and_down(oracle, ctx):
    import torch
    from lemonade_burn_b200 import ops
    g, pg, wg = make_linear(oracle, 6912, 2560, 21, ctx, 50.0)
    u, pu, wu = make_linear(oracle, 6912, 2560, 22, ctx, 52.0)
    d, pd, wd = make_linear(oracle, 2560, 6912, 23, ctx, 49.0)
    x = np.random.default_rng(7).standard_normal((1, 2560)).astype(np.float32)
    a, b = ops.ternary_linear2(torch.from_numpy(x).cuda(), [g, u])
    q, s, ssum = oracle.quantize_acts(x)
    wf, _ = oracle.simd_gemm_multi([pg, pu], [wg, wu], q, s, ssum)
    assert np.array_equal(a.cpu().numpy().view(np.uint32), wf[0].view(np.uint32))
    assert np.array_equal(b.cpu().numpy().view(np.uint32), wf[1].view(np.uint32))
    x2 = np.random.default_rng(8).standard_normal((3, 6912)).astype(np.float32)
    y = ops.ternary_linear(torch.from_numpy(x2).cuda(), d)
    q, s, ssum = oracle.quantize_acts(x2)
    wf, _ = oracle.simd_gemm_multi([pd], [wd], q, s, ssum)
    assert np.array_equal(y.cpu().numpy().view(np.uint32), wf[0].view(np.uint32))


def test_dtype_and_shape_errors(oracle, ctx):
    import torch
    from lemonade_burn_b200 import ops
    lin, _, _ = make_linear(oracle, 16, 256, 1, ctx)
    with pytest.raises(TypeError, match="f32 activations"):       # ops.rs:306
        ops.ternary_linear(torch.zeros(1, 256, dtype=torch.float16, device="cuda"), lin)
    with pytest.raises(ValueError, match="inner dimension mismatch"):  # ops.rs:308
        ops.ternary_linear(torch.zeros(1, 128, device="cuda"), lin)
    with pytest.raises(TypeError, match="u8 packed weights"):     # ops.rs:228
        ops.TernaryLinear(torch.zeros(4, 64, dtype=torch.int8, device="cuda"), 1.0, 256, ctx)
    with pytest.raises(TypeError, match="bf16 weights"):          # ops.rs:204
        ops.bf16_linear(torch.zeros(1, 8, device="cuda"), torch.zeros(4, 8, device="cuda"))


@pytest.mark.parametrize("m,rows,cols", [(1, 1000, 2560), (3, 1000, 2560), (4, 1000, 2560), (7, 1000, 2560), (16, 1003, 2560),
                                         (19, 37, 512), (2, 1000, 2568), (5, 64, 40), (20, 530, 8192), (3, 100, 6912), (2, 64, 3104),
                                         (64, 300, 2560), (65, 260, 1024), (130, 129, 512), (3, 50, 36), (6, 40, 2562)])
def test_bf16_linear(oracle, ctx, m, rows, cols):
    """One token row takes the FMA kernel, two or more the tcgen05 kernel (activations split into two
    bf16 terms; 64 token rows per pass over the table, so 65 and 130 rows take two and three passes),
    ragged row counts, a ragged last K block (2568, 40 columns) and long rows (8192: the 70B-shaped
    head) included; rows that are not whole 16-byte units (36, 2562 columns) take the FMA kernel."""
    import torch
    from lemonade_burn_b200 import ops
    g = torch.Generator().manual_seed(m)
    w = (torch.randn(rows, cols, generator=g) * 0.02).to(torch.bfloat16)
    x = torch.randn(m, cols, generator=g)
    out = ops.bf16_linear(x.cuda(), w.cuda()).cpu().numpy()
    bits = w.view(torch.int16).numpy().view(np.uint16)
    for t in range(m):
        ref = oracle.bf16_gemv(bits, x[t].numpy())
        assert np.abs(out[t] - ref).max() < 1e-4  # bf16.rs:113-136 bound
        # and relative to the row's range: the two-term bf16 split of the activations leaves 2^-17 per
        # product and the tensor core's own f32 accumulation adds an error that grows with the column
        # count (measured 3e-6 / 7e-6 / 1.0e-5 of max |out| at 2560 / 6912 / 8192 columns)
        assert np.abs(out[t] - ref).max() <= 2e-5 * np.abs(ref).max()


def test_plan_replays_groups(oracle, ctx):
    """Two layers' worth of decode groups (q/k/v, o, gate/up, down), recorded once and run as
    one unit, equal to the oracle group by group."""
    import torch
    from lemonade_burn_b200 import ops
    shapes = [[(256, 512), (64, 512), (64, 512)], [(512, 512)], [(640, 512), (640, 512)], [(512, 640)]]
    plan = ops.Plan(ctx)
    recs = []
    seed = 100
    for layer in range(2):
        for grp in shapes:
            cols = grp[0][1]
            lins = []
            for rows, _ in grp:
                seed += 1
                lins.append(make_linear(oracle, rows, cols, seed, ctx, 40.0 + seed % 7))
            x = np.random.default_rng(seed).standard_normal((1, cols)).astype(np.float32)
            xd = torch.from_numpy(x).cuda()
            outs = [torch.zeros(1, l.rows, device="cuda") for l, _, _ in lins]
            iouts = [torch.zeros(1, l.rows, dtype=torch.int32, device="cuda") for l, _, _ in lins]
            plan.add(xd, [l for l, _, _ in lins], outs, iouts)
            recs.append((x, lins, outs, iouts))
    plan.finalize()
    assert plan.weight_bytes() == sum(p.size for _, lins, _, _ in recs for _, p, _ in lins)
    for _ in range(2):
        plan.run()
    torch.cuda.synchronize()
    ctx.check_device_error()
    for x, lins, outs, iouts in recs:
        q, s, ssum = oracle.quantize_acts(x)
        wf, wi = oracle.simd_gemm_multi([p for _, p, _ in lins], [w for _, _, w in lins], q, s, ssum, want_i32=True)
        for o_, i_, ef, ei in zip(outs, iouts, wf, wi):
            assert np.array_equal(i_.cpu().numpy(), ei)
            assert np.array_equal(o_.cpu().numpy().view(np.uint32), ef.view(np.uint32))


@pytest.mark.parametrize("n_groups", [2, 9])
def test_plan_host_arenas(oracle, ctx, n_groups):
    """lbk_plan_run_host: groups added without buffers live in the plan's arenas; one call copies the
    inputs in, runs the plan and copies the outputs out. With nine groups the call is pipelined in
    segments (inputs of one segment arrive while another computes); with two it is sequential. Both
    against the oracle, twice with different inputs."""
    import torch
    from lemonade_burn_b200 import ops
    plan = ops.Plan(ctx)
    lins_all = []
    for gi in range(n_groups):
        cols = 512 if gi % 3 else 640
        lins = [make_linear(oracle, rows, cols, 300 + gi * 5 + j, ctx, 30.0 + gi) for j, rows in enumerate([96, 40][: 1 + gi % 2])]
        plan.add_arena([l for l, _, _ in lins])
        lins_all.append((cols, lins))
    plan.finalize()
    nx, ny = plan.input_elems(), plan.output_elems()
    assert nx == sum(c for c, _ in lins_all) and ny == sum(l.rows for _, lins in lins_all for l, _, _ in lins)
    for rep in range(2):
        x_host = torch.from_numpy(np.random.default_rng(rep).standard_normal(nx).astype(np.float32)).pin_memory()
        y_host = torch.zeros(ny).pin_memory()
        plan.run_host(x_host, y_host)
        xo = yo = 0
        for cols, lins in lins_all:
            x = x_host.numpy()[xo:xo + cols][None, :]
            xo += cols
            q, s, ssum = oracle.quantize_acts(x)
            wf = oracle.simd_gemm_multi([p for _, p, _ in lins], [w for _, _, w in lins], q, s, ssum)[0]
            for (l, _, _), ef in zip(lins, wf):
                assert np.array_equal(y_host.numpy()[yo:yo + l.rows].view(np.uint32), np.ascontiguousarray(ef).reshape(-1).view(np.uint32))
                yo += l.rows
    ctx.check_device_error()
