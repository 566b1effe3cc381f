"""The oracle against every known-answer vector the reference's own tests hold."""
import numpy as np
import pytest

GOLD = __import__("pathlib").Path(__file__).resolve().parent / "golden"


def test_quantizes_like_actquant(oracle):
    # crates/lb-ternary/src/quant.rs:201-209
    q, s, ssum = oracle.quantize_acts(np.array([[1.0, -0.5, 0.25, 0.0, -1.0]], dtype=np.float32))
    assert s[0] == np.float32(127.0)
    assert q[0, :5].tolist() == [127, -64, 32, 0, -127]   # 63.5 -> 64 (half-even), 31.75 -> 32
    assert not q[0, 5:].any() and q.shape[1] == 128
    assert ssum[0] == 127 - 64 + 32 - 127


def test_zero_row_is_safe(oracle):
    # quant.rs:212-216
    q, s, ssum = oracle.quantize_acts(np.zeros((1, 4), dtype=np.float32))
    assert s[0] == np.float32(127.0) / np.float32(1e-5)
    assert not q.any() and ssum[0] == 0


def test_ternary_kernels_quant_basic(oracle):
    # crates/ternary-kernels/src/quant.rs:34-42
    q, s, ssum = oracle.quantize_acts(np.array([[1.0, -2.0, 0.5, 0.0]], dtype=np.float32))
    assert s[0] == np.float32(63.5)
    assert q[0, :6].tolist() == [64, -127, 32, 0, 0, 0]
    assert ssum[0] == 64 - 127 + 32


def test_quant_special_values(oracle):
    # quant.rs:234-264: ties, NaN, denormal, -0.0, +-inf, zeros, tiny
    ties = np.concatenate([np.arange(96, dtype=np.float32) - 48.0 + 0.5, [np.float32(127.0)]]).astype(np.float32)
    q, s, _ = oracle.quantize_acts(ties[None])
    assert s[0] == 1.0
    want = np.rint(ties).astype(np.int8)  # ties to even
    assert np.array_equal(q[0, :97], want)
    odd = np.linspace(-1, 1, 70, dtype=np.float32)
    odd[3] = np.nan; odd[40] = np.nan; odd[5] = 1e-42; odd[6] = -0.0
    q, s, ssum = oracle.quantize_acts(odd[None])
    assert s[0] == np.float32(127.0)            # NaN ignored by the max
    assert q[0, 3] == 0 and q[0, 40] == 0       # NaN as i8 -> 0
    assert q[0, 5] == 0 and q[0, 6] == 0
    assert ssum[0] == int(q[0].astype(np.int64).sum())
    inf = np.ones(64, dtype=np.float32); inf[10] = np.inf; inf[50] = -np.inf
    q, s, _ = oracle.quantize_acts(inf[None])
    assert s[0] == 0.0                          # 127 / inf
    assert q[0, 10] == 0 and q[0, 50] == 0      # inf * 0 = NaN -> 0
    assert not q.any()


def test_pack_roundtrip_with_padding(oracle):
    # crates/lb-ternary/src/pack.rs:149-162
    for cols in [1, 31, 128, 129, 300, 512]:
        rows = 3
        vals = np.array([((i * 7 + i // 3) % 3) - 1 for i in range(rows * cols)], dtype=np.int8).reshape(rows, cols)
        p = oracle.pack_matrix(vals)
        assert p.shape == (rows, oracle.row_bytes(cols))
        full = oracle.unpack_matrix(p, cols)
        assert np.array_equal(full[:, :cols], vals)
        assert not full[:, cols:].any()          # padding decodes to zero weights


def test_tk_pack_roundtrip(oracle):
    # crates/ternary-kernels/src/pack.rs:86-99, and the two packers agree byte for byte
    n, k = 3, 300
    t = np.array([((i * 7 + i // 5) % 3) - 1 for i in range(n * k)], dtype=np.int8).reshape(n, k)
    p = oracle.tk_pack_ternary(t)
    assert p.shape == (n, 384 // 4)
    u = oracle.unpack_matrix(p, k, tk=True)
    assert np.array_equal(u[:, :k], t) and not u[:, k:].any()
    assert np.array_equal(p, oracle.pack_matrix(t))


def test_ternarize_matches_torch_semantics(oracle):
    # pack.rs:164-170
    t, s = oracle.ternarize_absmean(np.array([0.5, 1.5, -0.5, -2.0, 0.0, 1.5], dtype=np.float32))
    assert s == np.float32(1.0)
    assert t.tolist() == [0, 1, 0, -1, 0, 1]
    # ternary-kernels/src/pack.rs:101-107
    t = oracle.ternarize_with_scale(np.array([0.5, -0.5, 1.5, -1.5, 0.0, 1.0, -1.0, 2.0], dtype=np.float32), 1.0)
    assert t.tolist() == [0, 0, 1, -1, 0, 1, -1, 1]


def test_extreme_values(oracle):
    # crates/lb-ternary/tests/golden.rs:108-122: all +1 weights x all +-127 activations
    rows, cols = 4, 6912
    p = oracle.pack_matrix(np.ones((rows, cols), dtype=np.int8))
    for sign in (1.0, -1.0):
        q, s, ssum = oracle.quantize_acts(np.full((1, cols), sign, dtype=np.float32))
        got = oracle.ternary_gemm_i32(p, cols, q, ssum)
        assert (got == int(sign) * 127 * cols).all()
        assert (oracle.gemv_i32_reference(p, cols, q[0]) == int(sign) * 127 * cols).all()


def test_prefill_extreme_long_rows(oracle):
    # golden.rs:181-194: K = 13824, five tokens, output exactly +-K
    rows, cols, m = 3, 6912 * 2, 5
    p = oracle.pack_matrix(np.ones((rows, cols), dtype=np.int8))
    for sign in (1.0, -1.0):
        q, s, ssum = oracle.quantize_acts(np.full((m, cols), sign, dtype=np.float32))
        out = oracle.ternary_gemm(p, cols, 1.0, q, s, ssum)
        assert (out == np.float32(sign * 127.0 * cols / 127.0)).all()
        outs, iouts = oracle.simd_gemm_multi([p], [1.0], q, s, ssum, want_i32=True)
        assert (outs[0] == np.float32(sign * cols)).all() and (iouts[0] == int(sign) * 127 * cols).all()


def test_bf16_against_f64(oracle):
    # crates/lb-ternary/src/bf16.rs:113-136: within 1e-4 abs of an f64 dot (37 x 2584)
    rows, cols = 37, 2560 + 24
    rng = oracle.GoldenRng(12345)
    wf = np.array([rng.f() * 0.05 for _ in range(rows * cols)], dtype=np.float32)
    w = (wf.view(np.uint32) >> 16).astype(np.uint16).reshape(rows, cols)
    x = np.array([rng.f() for _ in range(cols)], dtype=np.float32)
    wd = (w.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    ref = wd @ x.astype(np.float64)
    out = oracle.bf16_gemv(w, x)
    assert np.abs(out.astype(np.float64) - ref).max() < 1e-4


def test_argmax_first_max_wins(oracle):
    # crates/lb-model/src/sample.rs:17-25
    assert oracle.argmax(np.array([1.0, 3.0, 3.0, 2.0], dtype=np.float32)) == 1
    assert oracle.argmax(np.array([-1.0], dtype=np.float32)) == 0


def test_hf_actquant_fixture(oracle):
    """The oracle quantiser against transformers' ActQuant outputs (committed fixture).

    transformers writes `127 / amax` with a Python scalar on the left, which torch evaluates
    as `amax.reciprocal() * 127`; the reference divides directly (quant.rs:105). The two
    scales can differ by one ulp. Rows whose scales are bit-equal must match the library bit
    for bit; on the others a code may move only where x*scale sits within an ulp of a tie."""
    fx = np.load(GOLD / "hf_bitnet_quant.npz")
    x = fx["act_x"]
    q, s, ssum = oracle.quantize_acts(x)
    hf_s, hf_q, hf_deq = fx["act_scale"], fx["act_q"], fx["act_dequant"]
    ulps = np.abs(s.view(np.int32).astype(np.int64) - hf_s.view(np.int32).astype(np.int64))
    assert ulps.max() <= 1
    same = ulps == 0
    assert same.sum() >= 4
    assert np.array_equal(q[same][:, : x.shape[1]], hf_q[same])
    deq = q[:, : x.shape[1]].astype(np.float32) / s[:, None]
    assert np.array_equal(deq[same], hf_deq[same])  # by value: the library keeps -0.0 for rounded-away negatives
    diff = np.abs(q[~same][:, : x.shape[1]].astype(np.int32) - hf_q[~same].astype(np.int32))
    assert diff.max(initial=0) <= 1 and (diff != 0).mean() < 0.01
    assert np.array_equal(ssum, q.astype(np.int64).sum(axis=1))


def test_hf_weightquant_fixture(oracle):
    """The oracle ternariser against transformers' WeightQuant outputs (committed fixture)."""
    fx = np.load(GOLD / "hf_bitnet_quant.npz")
    for i in range(3):
        w, deq, ts = fx[f"w{i}"], fx[f"w{i}_dequant"], np.float32(fx[f"w{i}_scale"])
        t = oracle.ternarize_with_scale(w, ts)
        assert np.array_equal(t.astype(np.float32) / ts, deq)  # by value (-0.0 == 0.0)
        # the reference sums |w| in f64 where torch sums in f32: scales agree to 1 ulp
        # (crates/lb-ternary/src/pack.rs:126-128)
        _, s = oracle.ternarize_absmean(w)
        assert abs(int(np.float32(s).view(np.uint32)) - int(ts.view(np.uint32))) <= 1
