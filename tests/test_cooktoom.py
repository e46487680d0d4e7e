"""Cook-Toom generator: exact identity and equality with the reference generator's output
(fixtures made by tests/golden/make_golden.py from wincnn.showCookToomFilter and the
reference's hand-written tables, matrix_convnd.py:14-36)."""
import os
from fractions import Fraction

import numpy as np
import pytest

from pytorch_winoconv_b200 import cooktoom

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "cooktoom_golden.npz"))


@pytest.mark.parametrize("m,r", [(2, 1), (2, 2), (2, 3), (4, 3), (2, 5), (2, 7), (6, 3), (4, 2), (1, 1), (3, 3)])
def test_identity_exact(m, r):
    at, g, bt = cooktoom.cook_toom(m, r)
    assert cooktoom.verify_identity(at, g, bt)


@pytest.mark.parametrize("m,r", [(2, 3), (2, 4), (2, 5), (2, 6), (2, 7), (2, 9), (2, 11), (9, 5), (4, 3), (2, 2)])
def test_matches_reference_generator(m, r):
    pts = [Fraction(int(n), int(d)) for n, d in zip(GOLD[f"F{m}_{r}_points_num"], GOLD[f"F{m}_{r}_points_den"])]
    at, g, bt = cooktoom.cook_toom(m, r, pts)
    np.testing.assert_allclose(cooktoom.as_float64(at), GOLD[f"F{m}_{r}_AT"], rtol=0, atol=1e-15 * max(1, np.abs(GOLD[f"F{m}_{r}_AT"]).max()))
    np.testing.assert_allclose(cooktoom.as_float64(g), GOLD[f"F{m}_{r}_G"], rtol=1e-15, atol=0)
    np.testing.assert_allclose(cooktoom.as_float64(bt), GOLD[f"F{m}_{r}_BT"], rtol=1e-15, atol=0)


@pytest.mark.parametrize("r", [1, 2, 3])
def test_reference_tables(r):
    at, g, bt = cooktoom.reference_table(2, r)
    np.testing.assert_array_equal(at, GOLD[f"table2_{r}_AT"])
    np.testing.assert_array_equal(g, GOLD[f"table2_{r}_G"])
    np.testing.assert_array_equal(bt, GOLD[f"table2_{r}_BT"])
    assert cooktoom.verify_identity(at.tolist(), g.tolist(), bt.tolist())


def test_default_points_f43():
    at, g, bt = cooktoom.cook_toom(4, 3)
    np.testing.assert_array_equal(cooktoom.as_float64(bt)[0], [4, 0, -5, 0, 1, 0])
    assert g[3] == [Fraction(1, 24), Fraction(1, 12), Fraction(1, 6)]


def test_bad_points_rejected():
    with pytest.raises(ValueError):
        cooktoom.cook_toom(2, 3, (0, 1))
    with pytest.raises(ValueError):
        cooktoom.cook_toom(2, 3, (0, 1, 1))
