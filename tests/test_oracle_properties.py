"""The reference's golden property tests (crates/lb-ternary/tests/golden.rs) run on the oracle,
with the same xorshift generator, seeds and shapes: the code-offset path, the
unpack-every-weight path (ternary-kernels' reference) and the threaded SIMD port must all give
the integers of a naive sum over unpacked values."""
import numpy as np
import pytest

GEMV_SHAPES = [(1, 128), (7, 128), (33, 256), (17, 384), (64, 640), (40, 2560), (9, 6912)]  # golden.rs:83


def naive(t, q, cols):
    """golden.rs:37-58: i64 sum over unpacked values."""
    return q[:, :cols].astype(np.int64) @ t.astype(np.int64).T


def run_case(o, rows, cols, m, seed):
    t, ws, packed, x = o.golden_case(rows, cols, m, seed)
    q, s, ssum = o.quantize_acts(x)
    ref_i = naive(t, q, cols)
    got = o.ternary_gemm_i32(packed, cols, q, ssum)
    assert np.array_equal(got.astype(np.int64), ref_i)
    kp = o.padded_cols(cols)
    for tk in range(m):
        assert np.array_equal(o.gemv_i32_reference(packed, kp, q[tk]).astype(np.int64), ref_i[tk])
    # f32 after scaling within 1e-5 * sum|terms| of the f64 evaluation (golden.rs:5-7,65-72)
    qa = q[:, :cols].astype(np.float64) / s[:, None].astype(np.float64)
    wa = t.astype(np.float64) / np.float64(ws)
    ref_f = qa @ wa.T
    ref_abs = np.abs(qa) @ np.abs(wa).T
    out = o.ternary_gemm(packed, cols, ws, q, s, ssum)
    assert (np.abs(out.astype(np.float64) - ref_f) <= 1e-5 * np.maximum(ref_abs, 1e-6)).all()
    # the SIMD port: every kernel this CPU has
    for kern in range(o.simd_best_kernel() + 1):
        for threads in (1, 3):
            outs, iouts = o.simd_gemm_multi([packed], [ws], q, s, ssum, kernel=kern, threads=threads, want_i32=True)
            assert np.array_equal(iouts[0], got), (o.simd_kernel_name(kern), threads)
            assert np.array_equal(outs[0].view(np.uint32), out.view(np.uint32))


@pytest.mark.parametrize("rows,cols", GEMV_SHAPES)
def test_gemv_shapes(oracle, rows, cols):
    run_case(oracle, rows, cols, 1, rows * 31 + cols)


@pytest.mark.parametrize("m", list(range(1, 10)))
def test_gemm_token_tiles(oracle, m):
    run_case(oracle, 23, 384, m, 1000 + m)  # golden.rs:91-93


def test_gemm_token_tiles_big(oracle):
    run_case(oracle, 48, 2560, 5, 77)   # golden.rs:94
    run_case(oracle, 37, 2560, 13, 78)  # golden.rs:96


@pytest.mark.parametrize("cols", [1, 100, 129, 300])
def test_padded_columns(oracle, cols):
    run_case(oracle, 5, cols, 3, cols)  # golden.rs:100-105


def test_multi_matches_separate_bit_for_bit(oracle):
    # golden.rs:128-176: fused == separate, f32 bit-equal, several thread counts, m in {1,2,5,64}
    o = oracle
    cols = 640
    rng = o.GoldenRng(4242)
    mats = []
    for rows, sc in [(96, 0.7), (24, 1.3), (200, 2.1)]:
        t = rng.ternary(rows * cols).reshape(rows, cols)
        mats.append((o.pack_matrix(t), np.float32(sc)))
    for m in (1, 2, 5, 64):
        x = rng.acts(m * cols, 89, 1, 30.0).reshape(m, cols)
        q, s, ssum = o.quantize_acts(x)
        expect = []
        for p, sc in mats:
            ints = o.ternary_gemm_i32(p, cols, q, ssum)
            inv = (np.float32(1.0) / (s * sc)).astype(np.float32)
            expect.append((ints.astype(np.float32) * inv[:, None]).astype(np.float32))
        for threads in (1, 3, 8):
            outs, _ = o.simd_gemm_multi([p for p, _ in mats], [sc for _, sc in mats], q, s, ssum, threads=threads)
            for got, e in zip(outs, expect):
                assert np.array_equal(got.view(np.uint32), e.view(np.uint32))
        for (p, sc), e in zip(mats, expect):
            single = o.ternary_gemm(p, cols, sc, q, s, ssum)
            assert np.array_equal(single.view(np.uint32), e.view(np.uint32))


def test_parallel_rows_match(oracle):
    # crates/lb-ternary/src/quant.rs:268-281: threaded rows == scalar rows
    o = oracle
    for m, k in [(64, 2560), (5, 6912), (3, 100), (17, 1000)]:
        rng = o.GoldenRng(m * 31 + k)
        x = rng.acts(m * k, 53, 7, 40.0).reshape(m, k)
        a = o.quantize_acts(x)
        b = o.simd_quantize_acts(x)
        for u, v in zip(a, b):
            assert np.array_equal(u, v)


@pytest.mark.parametrize("rows,cols,m,seed", [(64, 128, 1, 1), (130, 300, 3, 2), (2560, 2560, 1, 3), (6912, 2560, 4, 4)])
def test_gpu_matches_scalar_cases_on_oracle(oracle, rows, cols, m, seed):
    # crates/lb-ternary-gpu/tests/gpu_matches_scalar.rs:37-54 inputs: both oracle paths and the
    # SIMD port agree (the CUDA tests run the same four cases against the oracle)
    o = oracle
    t, packed, x = o.gpu_case(rows, cols, m, seed)
    q, s, ssum = o.quantize_acts(x)
    _, iouts = o.simd_gemm_multi([packed], [1.0], q, s, ssum, want_f32=False, want_i32=True)
    assert np.array_equal(iouts[0].astype(np.int64), naive(t, q, cols))
    if rows <= 130:
        assert np.array_equal(o.ternary_gemm_i32(packed, cols, q, ssum), iouts[0])
