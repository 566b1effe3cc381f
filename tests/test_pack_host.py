"""Host-side pack module (the lb-ternary `pack` mirror) against the oracle and the reference's
unit tests (crates/lb-ternary/src/pack.rs:149-170)."""
import numpy as np
import pytest

from lemonade_burn_b200 import pack


def test_pack_roundtrip_with_padding():
    for cols in [1, 31, 128, 129, 300, 512]:
        rows = 3
        vals = np.array([((i * 7 + i // 3) % 3) - 1 for i in range(rows * cols)], dtype=np.int8)
        p = pack.PackedTernary.from_ternary(rows, cols, vals, 1.0)
        for r in range(rows):
            assert np.array_equal(p.view().unpack_row(r), vals[r * cols:(r + 1) * cols])
        full = pack.unpack_row(p.view().row(0), pack.padded_cols(cols))
        assert not full[cols:].any()


def test_ternarize_matches_torch_semantics():
    t, s = pack.ternarize_absmean(np.array([0.5, 1.5, -0.5, -2.0, 0.0, 1.5], dtype=np.float32))
    assert s == np.float32(1.0) and t.tolist() == [0, 1, 0, -1, 0, 1]


def test_view_length_assert():
    with pytest.raises(ValueError, match="packed data length mismatch"):  # pack.rs:40
        pack.TernaryView(3, 128, np.zeros(95, dtype=np.uint8), 1.0)
    with pytest.raises(ValueError):
        pack.pack_rows(np.array([[2, 0]], dtype=np.int8))


def test_matches_oracle(oracle):
    rng = np.random.default_rng(5)
    for rows, cols in [(1, 1), (3, 127), (9, 128), (4, 700), (2, 6912)]:
        v = rng.integers(-1, 2, size=(rows, cols)).astype(np.int8)
        assert np.array_equal(pack.pack_rows(v), oracle.pack_matrix(v))
        assert np.array_equal(pack.pack_rows(v), oracle.tk_pack_ternary(v))
    w = (rng.standard_normal((64, 640)) * 0.02).astype(np.float32)
    t, s = pack.ternarize_absmean(w)
    t2, s2 = oracle.ternarize_absmean(w)
    assert np.array_equal(t, t2) and np.float32(s) == np.float32(s2)
