"""Parity of the CUDA path with the CPU oracle, through the C ABI (liblbk.so).

Integers must be bit-exact; f32 outputs are compared bit for bit as well, because the
epilogue follows the reference's operation order ((float)dot * (1/(s_a*s_w)), gemm.rs:141),
with 1e-3 relative (the bar the path is held to) as the documented fallback bound.
Cases are the reference's own: crates/lb-ternary/tests/golden.rs and
crates/lb-ternary-gpu/tests/gpu_matches_scalar.rs, same generators and seeds.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

REL_TOL = 1e-3  # float outputs after scaling: within 1e-3 relative


def lbt():
    from lemonade_burn_b200 import ternary
    return ternary


def check_case(o, ctx, t, wscale, packed, x, want_bits=True):
    T = lbt()
    rows, cols = t.shape
    m = x.shape[0]
    view = T.TernaryView(rows, cols, packed.reshape(-1), float(wscale))
    dw = T.DeviceWeight(view, ctx)
    # quantize_acts
    qa = T.quantize_acts(x, m, cols, ctx)
    q, s, ssum = o.quantize_acts(x)
    assert np.array_equal(qa.q.reshape(m, -1), q)
    assert np.array_equal(qa.scale.view(np.uint32), s.view(np.uint32))
    assert np.array_equal(qa.sum, ssum)
    # ternary_gemm_i32: bit exact
    want_i = o.ternary_gemm_i32(packed, cols, q, ssum)
    got_i = T.ternary_gemm_i32(dw, qa, ctx=ctx).reshape(m, rows)
    assert np.array_equal(got_i, want_i)
    # ternary_gemm
    want_f = o.ternary_gemm(packed, cols, wscale, q, s, ssum)
    out = np.zeros((m, rows), dtype=np.float32)
    T.ternary_gemm(dw, qa, T.Kernel.Sm100, out, ctx)
    if want_bits:
        assert np.array_equal(out.view(np.uint32), want_f.view(np.uint32))
    assert np.allclose(out, want_f, rtol=REL_TOL, atol=0)
    # fused op from f32 activations
    outs, iouts = T.ternary_linear_host(x, [dw], want_i32=True, ctx=ctx)
    assert np.array_equal(iouts[0], want_i)
    assert np.array_equal(outs[0].view(np.uint32), want_f.view(np.uint32))
    dw.close()


GEMV_SHAPES = [(1, 128), (7, 128), (33, 256), (17, 384), (64, 640), (40, 2560), (9, 6912)]


@pytest.mark.parametrize("rows,cols", GEMV_SHAPES)
def test_gemv_shapes(oracle, ctx, rows, cols):
    t, ws, p, x = oracle.golden_case(rows, cols, 1, rows * 31 + cols)
    check_case(oracle, ctx, t, ws, p, x)


@pytest.mark.parametrize("m", list(range(1, 10)) + [13, 16])
def test_token_tiles(oracle, ctx, m):
    t, ws, p, x = oracle.golden_case(23, 384, m, 1000 + m)
    check_case(oracle, ctx, t, ws, p, x)


def test_token_tiles_big(oracle, ctx):
    check_case(oracle, ctx, *oracle.golden_case(48, 2560, 5, 77))
    check_case(oracle, ctx, *oracle.golden_case(37, 2560, 13, 78))


@pytest.mark.parametrize("cols", [1, 100, 129, 300])
def test_padded_columns(oracle, ctx, cols):
    check_case(oracle, ctx, *oracle.golden_case(5, cols, 3, cols))


def test_extreme_values(oracle, ctx):
    T = lbt()
    rows, cols = 4, 6912
    p = oracle.pack_matrix(np.ones((rows, cols), dtype=np.int8))
    dw = T.DeviceWeight(T.TernaryView(rows, cols, p.reshape(-1), 1.0), ctx)
    for sign in (1.0, -1.0):
        qa = T.quantize_acts(np.full((1, cols), sign, dtype=np.float32), 1, cols, ctx)
        got = T.ternary_gemm_i32(dw, qa, ctx=ctx)
        assert (got == int(sign) * 127 * cols).all()


def test_extreme_long_rows(oracle, ctx):
    # golden.rs:181-194: K = 13824, m = 5, all-ones weights, +-1 activations -> exactly +-K
    T = lbt()
    rows, cols, m = 3, 6912 * 2, 5
    p = oracle.pack_matrix(np.ones((rows, cols), dtype=np.int8))
    dw = T.DeviceWeight(T.TernaryView(rows, cols, p.reshape(-1), 1.0), ctx)
    for sign in (1.0, -1.0):
        x = np.full((m, cols), sign, dtype=np.float32)
        outs, _ = T.ternary_linear_host(x, [dw], ctx=ctx)
        assert (outs[0] == np.float32(sign * cols)).all()


def test_never_emitted_code_3_decodes_to_plus_2(oracle, ctx):
    # pack.rs:7-8: code 3 decodes to +2 in the reference; the kernels must agree
    T = lbt()
    rng = np.random.default_rng(3)
    rows, cols = 20, 512
    p = rng.integers(0, 256, size=(rows, cols // 4), dtype=np.uint8)
    x = rng.standard_normal((3, cols)).astype(np.float32)
    q, s, ssum = oracle.quantize_acts(x)
    want = oracle.ternary_gemm_i32(p, cols, q, ssum)
    dw = T.DeviceWeight(T.TernaryView(rows, cols, p.reshape(-1), 1.0), ctx)
    _, iouts = T.ternary_linear_host(x, [dw], want_i32=True, ctx=ctx)
    assert np.array_equal(iouts[0], want)


def test_multi_matches_separate_bit_for_bit(oracle, ctx):
    # golden.rs:128-176
    T = lbt()
    o = oracle
    cols = 640
    rng = o.GoldenRng(4242)
    mats = []
    for rows, sc in [(96, 0.7), (24, 1.3), (200, 2.1)]:
        t = rng.ternary(rows * cols).reshape(rows, cols)
        p = o.pack_matrix(t)
        mats.append((p, np.float32(sc), T.DeviceWeight(T.TernaryView(rows, cols, p.reshape(-1), sc), ctx)))
    for m in (1, 2, 5, 16):
        x = rng.acts(m * cols, 89, 1, 30.0).reshape(m, cols)
        q, s, ssum = o.quantize_acts(x)
        qa = T.QuantActs(m, cols, o.padded_cols(cols), q.reshape(-1), s, ssum)
        bufs = [np.zeros((m, p.shape[0]), dtype=np.float32) for p, _, _ in mats]
        T.ternary_gemm_multi([d for _, _, d in mats], qa, T.Kernel.Sm100, bufs, ctx)
        for (p, sc, d), b in zip(mats, bufs):
            e = o.ternary_gemm(p, cols, sc, q, s, ssum)
            assert np.array_equal(b.view(np.uint32), e.view(np.uint32))
            single = np.zeros_like(b)
            T.ternary_gemm(d, qa, T.Kernel.Sm100, single, ctx)
            assert np.array_equal(single.view(np.uint32), e.view(np.uint32))


@pytest.mark.parametrize("rows,cols,m,seed", [(64, 128, 1, 1), (130, 300, 3, 2), (2560, 2560, 1, 3), (6912, 2560, 4, 4)])
def test_gpu_matches_scalar(oracle, ctx, rows, cols, m, seed):
    # crates/lb-ternary-gpu/tests/gpu_matches_scalar.rs:37-54, checked against the oracle
    T = lbt()
    t, packed, x = oracle.gpu_case(rows, cols, m, seed)
    q, s, ssum = oracle.quantize_acts(x)
    _, want = oracle.simd_gemm_multi([packed], [1.0], q, s, ssum, want_f32=False, want_i32=True)
    dw = T.DeviceWeight(T.TernaryView(rows, cols, packed.reshape(-1), 1.0), ctx)
    qa = T.quantize_acts(x, m, cols, ctx)
    got = T.ternary_gemm_i32(dw, qa, ctx=ctx).reshape(m, rows)
    assert np.array_equal(got, want[0])


def test_quant_special_values(oracle, ctx):
    # quant.rs:234-264 on the GPU quantiser (standalone and fused)
    T = lbt()
    cases = []
    for seed, n in [(1, 2560), (2, 6912), (3, 31), (4, 33), (5, 7), (6, 1), (7, 130)]:
        cases.append(oracle.GoldenRng(seed).acts(n, 53, 7, 40.0))
    ties = np.concatenate([np.arange(96, dtype=np.float32) - 48.0 + 0.5, [np.float32(127.0)]]).astype(np.float32)
    cases.append(ties)
    odd = oracle.GoldenRng(9).acts(70, 53, 7, 40.0)
    odd[3] = np.nan; odd[40] = np.nan; odd[5] = 1e-42; odd[6] = -0.0
    cases.append(odd)
    inf = oracle.GoldenRng(10).acts(64, 53, 7, 40.0)
    inf[10] = np.inf; inf[50] = -np.inf
    cases.append(inf)
    cases.append(np.zeros(40, dtype=np.float32))
    cases.append(np.full(40, 1e-30, dtype=np.float32))
    for x in cases:
        n = x.size
        q, s, ssum = oracle.quantize_acts(x[None])
        qa = T.quantize_acts(x, 1, n, ctx)
        assert np.array_equal(qa.scale.view(np.uint32), s.view(np.uint32)), n
        assert np.array_equal(qa.q.reshape(1, -1), q), n
        assert np.array_equal(qa.sum, ssum), n
        # fused kernel sees the same codes: identity-like matrix rows pick out sum and q
        w = np.ones((2, n), dtype=np.int8); w[1] = -1
        p = oracle.pack_matrix(w)
        dw = T.DeviceWeight(T.TernaryView(2, n, p.reshape(-1), 1.0), ctx)
        _, iouts = T.ternary_linear_host(x[None], [dw], want_i32=True, ctx=ctx)
        assert iouts[0][0, 0] == ssum[0] and iouts[0][0, 1] == -ssum[0]


def test_error_behaviour(oracle, ctx):
    T = lbt()
    from lemonade_burn_b200._lib import LbkError
    t, ws, p, x = oracle.golden_case(5, 256, 1, 1)
    dw = T.DeviceWeight(T.TernaryView(5, 256, p.reshape(-1), ws), ctx)
    qa = T.quantize_acts(np.zeros((1, 384), dtype=np.float32), 1, 384, ctx)
    with pytest.raises(ValueError, match="inner dimension mismatch"):   # gemm.rs:198
        T.ternary_gemm_i32(dw, qa, ctx=ctx)
    with pytest.raises(ValueError, match="packed data length mismatch"):  # pack.rs:40
        T.TernaryView(5, 256, p.reshape(-1)[:-1], ws)
    # the same mistakes made directly at the C boundary come back as status codes
    import ctypes as C
    h = C.c_void_p()
    st = ctx._lib.lbk_weight_upload(ctx.handle, 5, 256, p.ctypes.data, p.size - 1, C.c_float(1.0), C.byref(h))
    assert st == 2 and b"length mismatch" in ctx._lib.lbk_last_error()
    with pytest.raises(ValueError, match="inner dimension mismatch"):   # ops.rs:308
        T.ternary_linear_host(np.zeros((1, 128), dtype=np.float32), [dw], ctx=ctx)
    # ... and a mismatch that only the library can see (two matrices of different widths)
    t2, ws2, p2, _ = oracle.golden_case(5, 384, 1, 2)
    dw2 = T.DeviceWeight(T.TernaryView(5, 384, p2.reshape(-1), ws2), ctx)
    from lemonade_burn_b200 import _lib as L
    wp, _k = L.ptr_array([dw.handle.value, dw2.handle.value])
    xz = np.zeros((1, 256), dtype=np.float32)
    o1 = np.zeros((1, 5), dtype=np.float32)
    op, _k2 = L.ptr_array([o1.ctypes.data, o1.ctypes.data])
    st = ctx._lib.lbk_ternary_linear_host(ctx.handle, xz.ctypes.data, 1, wp, 2, op, None)
    assert st == 2 and b"inner dimension mismatch" in ctx._lib.lbk_last_error()
    assert issubclass(LbkError, RuntimeError)


def test_config0_gate_proj(oracle, ctx):
    """K=2560, N=6912, M=1 with P(-1)=P(+1)=0.3, P(0)=0.4 weights and N(0,1) activations."""
    T = lbt()
    rng = np.random.default_rng(0x5EED0)
    rows, cols = 6912, 2560
    t = rng.choice(np.array([-1, 0, 1], dtype=np.int8), size=(rows, cols), p=[0.3, 0.4, 0.3])
    latent = (rng.standard_normal(4096) * 0.02).astype(np.float32)
    wscale = np.float32(1.0) / np.float32(np.abs(latent.astype(np.float64)).mean())
    x = rng.standard_normal((1, cols)).astype(np.float32)
    p = oracle.pack_matrix(t)
    q, s, ssum = oracle.quantize_acts(x)
    outs_f, outs_i = oracle.simd_gemm_multi([p], [wscale], q, s, ssum, want_i32=True)
    assert np.array_equal(oracle.gemv_i32_reference(p[:64], cols, q[0]), outs_i[0][0, :64])
    dw = T.DeviceWeight(T.TernaryView(rows, cols, p.reshape(-1), float(wscale)), ctx)
    outs, iouts = T.ternary_linear_host(x, [dw], want_i32=True, ctx=ctx)
    assert np.array_equal(iouts[0], outs_i[0])
    assert np.array_equal(outs[0].view(np.uint32), outs_f[0].view(np.uint32))
    assert np.allclose(outs[0], outs_f[0], rtol=REL_TOL, atol=0)


def test_bf16_gemv(oracle, ctx):
    # crates/lb-ternary/src/bf16.rs:113-136: within 1e-4 abs of an f64 dot (37 x 2584)
    T = lbt()
    rows, cols = 37, 2560 + 24
    rng = oracle.GoldenRng(12345)
    wf = np.array([rng.f() * 0.05 for _ in range(rows * cols)], dtype=np.float32)
    w = (wf.view(np.uint32) >> 16).astype(np.uint16)
    x = np.array([rng.f() for _ in range(cols)], dtype=np.float32)
    wd = (w.astype(np.uint32) << 16).view(np.float32).astype(np.float64).reshape(rows, cols)
    ref = wd @ x.astype(np.float64)
    out = np.zeros(rows, dtype=np.float32)
    T.bf16_gemv(w, rows, cols, x, out, ctx=ctx)
    assert np.abs(out.astype(np.float64) - ref).max() < 1e-4
    assert np.abs(out - oracle.bf16_gemv(w.reshape(rows, cols), x)).max() < 1e-4
