"""Prefill path (more than 16 token rows -> tcgen05 int8 GEMM) against the oracle, through the
C ABI. Integers bit-exact, f32 bit-exact (same epilogue order as gemm.rs:158,178), 1e-3 relative
as the documented bound. Shapes are the BitNet-2B projections (K=2560->N=6912, K=6912->N=2560) plus
the reference's padded / token-tile / extreme cases (crates/lb-ternary/tests/golden.rs)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
REL_TOL = 1e-3


def T():
    from lemonade_burn_b200 import ternary
    return ternary


def run_case(o, ctx, t, ws, p, x):
    rows, cols = t.shape
    m = x.shape[0]
    dw = T().DeviceWeight(T().TernaryView(rows, cols, p.reshape(-1), float(ws)), ctx)
    outs, iouts = T().ternary_linear_host(x, [dw], want_i32=True, ctx=ctx)
    q, s, ssum = o.quantize_acts(x)
    wf, wi = o.simd_gemm_multi([p], [ws], q, s, ssum, want_i32=True)
    assert np.array_equal(iouts[0], wi[0])
    assert np.array_equal(outs[0].view(np.uint32), wf[0].view(np.uint32))
    assert np.allclose(outs[0], wf[0], rtol=REL_TOL, atol=0)
    ctx.check_device_error()


@pytest.mark.parametrize("rows,cols,m,seed", [(23, 384, 17, 1), (37, 2560, 40, 78), (300, 640, 64, 3), (257, 128, 129, 4),
                                               (5, 300, 33, 5), (5, 1, 20, 6), (130, 300, 130, 2)])
def test_small_and_padded(oracle, ctx, rows, cols, m, seed):
    run_case(oracle, ctx, *oracle.golden_case(rows, cols, m, seed))


def random_case(rows, cols, m, seed, oracle):
    rng = np.random.default_rng(seed)
    t = rng.choice(np.array([-1, 0, 1], dtype=np.int8), size=(rows, cols), p=[0.3, 0.4, 0.3])
    x = rng.standard_normal((m, cols)).astype(np.float32)
    return t, np.float32(62.66), oracle.pack_matrix(t), x


@pytest.mark.parametrize("m", [64, 256, 1024, 2048])
@pytest.mark.parametrize("rows,cols", [(6912, 2560), (2560, 6912)])
def test_config2_shapes(oracle, ctx, rows, cols, m):
    """Both BitNet-2B prefill projections at every token count of the benchmark configuration, every
    output element against the oracle: int32 sums and f32 bits. K = 6912 at the larger token counts is
    where the GEMM cuts K into parts that add their sums (`choose_ksplit`); the host-buffer entry
    point and the device-resident one are both driven."""
    import torch
    from lemonade_burn_b200 import ops
    t, ws, p, x = random_case(rows, cols, m, rows + m, oracle)
    q, s, ssum = oracle.quantize_acts(x)
    wf, wi = oracle.simd_gemm_multi([p], [ws], q, s, ssum, want_i32=True)
    if m <= 256:
        run_case(oracle, ctx, t, ws, p, x)
    lin = ops.TernaryLinear(torch.from_numpy(p).cuda(), float(ws), cols, ctx)
    outs, iouts = ops.ternary_linear_multi(torch.from_numpy(x).cuda(), [lin], want_i32=True)
    assert np.array_equal(iouts[0].cpu().numpy(), wi[0])
    assert np.array_equal(outs[0].cpu().numpy().view(np.uint32), wf[0].view(np.uint32))
    # f32 outputs alone (no int32 buffer): the epilogue variant the decoder uses
    only_f = ops.ternary_linear_multi(torch.from_numpy(x).cuda(), [lin])[0]
    assert np.array_equal(only_f.cpu().numpy().view(np.uint32), wf[0].view(np.uint32))
    ctx.check_device_error()


def test_extreme_long_rows(oracle, ctx):
    # golden.rs:181-194 at a prefill token count: all +1 weights, +-1 activations, K = 13824
    rows, cols, m = 3, 6912 * 2, 40
    p = oracle.pack_matrix(np.ones((rows, cols), dtype=np.int8))
    dw = T().DeviceWeight(T().TernaryView(rows, cols, p.reshape(-1), 1.0), ctx)
    for sign in (1.0, -1.0):
        outs, iouts = T().ternary_linear_host(np.full((m, cols), sign, dtype=np.float32), [dw], want_i32=True, ctx=ctx)
        assert (iouts[0] == int(sign) * 127 * cols).all()
        assert (outs[0] == np.float32(sign * cols)).all()


def test_code3_and_multi(oracle, ctx):
    """Random packed bytes (code 3 decodes to +2, pack.rs:7-8) in a fused q/k/v-like group."""
    rng = np.random.default_rng(11)
    cols, m = 640, 70
    mats = []
    for rows, sc in [(96, 0.7), (24, 1.3), (300, 2.1)]:
        p = rng.integers(0, 256, size=(rows, cols // 4), dtype=np.uint8)
        mats.append((p, np.float32(sc), T().DeviceWeight(T().TernaryView(rows, cols, p.reshape(-1), sc), ctx)))
    x = rng.standard_normal((m, cols)).astype(np.float32)
    outs, iouts = T().ternary_linear_host(x, [d for _, _, d in mats], want_i32=True, ctx=ctx)
    q, s, ssum = oracle.quantize_acts(x)
    for (p, sc, _), of, oi in zip(mats, outs, iouts):
        assert np.array_equal(oi, oracle.ternary_gemm_i32(p, cols, q, ssum))
        assert np.array_equal(of.view(np.uint32), oracle.ternary_gemm(p, cols, sc, q, s, ssum).view(np.uint32))


@pytest.mark.parametrize("m", [1024, 2048])
def test_full_size_fused_group_and_permutation(oracle, ctx, m):
    """The fused gate/up group (two 6912 x 2560 matrices sharing one quantised input) at full prefill
    token counts, every element against the oracle, and a size-independent property: permuting the
    token rows permutes the output rows."""
    import torch
    from lemonade_burn_b200 import ops
    rows, cols = 6912, 2560
    ta, wsa, pa, x = random_case(rows, cols, m, 4242 + m, oracle)
    tb, wsb, pb, _ = random_case(rows, cols, 1, 99 + m, oracle)
    wsb = np.float32(47.5)
    la = ops.TernaryLinear(torch.from_numpy(pa).cuda(), float(wsa), cols, ctx)
    lb = ops.TernaryLinear(torch.from_numpy(pb).cuda(), float(wsb), cols, ctx)
    xd = torch.from_numpy(x).cuda()
    outs, iouts = ops.ternary_linear_multi(xd, [la, lb], want_i32=True)
    q, s, ssum = oracle.quantize_acts(x)
    wf, wi = oracle.simd_gemm_multi([pa, pb], [wsa, wsb], q, s, ssum, want_i32=True)
    for k in range(2):
        assert np.array_equal(iouts[k].cpu().numpy(), wi[k])
        assert np.array_equal(outs[k].cpu().numpy().view(np.uint32), wf[k].view(np.uint32))
    perm = torch.randperm(m, generator=torch.Generator().manual_seed(1)).cuda()
    o3 = ops.ternary_linear_multi(xd[perm].contiguous(), [la, lb])
    assert torch.equal(o3[0], outs[0][perm]) and torch.equal(o3[1], outs[1][perm])
    ctx.check_device_error()


def test_int8_peak_probe_is_plausible(ctx):
    """lbk_int8_peak_probe: the no-load rate of the tensor-core instruction the GEMM is built on. The
    nominal dense int8 figure of the part is 4500 TOPS; the probe must land within a factor of two of
    it at 192 and 256 token rows and must not report more at 64 rows than at 256."""
    r64, r192, r256 = ctx.int8_peak_tops(64, 5000), ctx.int8_peak_tops(192, 5000), ctx.int8_peak_tops(256, 5000)
    assert 2250.0 < r192 < 9000.0 and 2250.0 < r256 < 9000.0, (r64, r192, r256)
    assert r64 <= r256 * 1.05
    ctx.check_device_error()
    from lemonade_burn_b200 import _lib
    with pytest.raises(_lib.LbkError):
        ctx.int8_peak_tops(100, 10)
