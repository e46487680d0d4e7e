"""Exact Cook-Toom (Winograd minimal filtering) matrix generator.

F(m, r) computes m outputs of an r-tap correlation from alpha = m + r - 1 inputs:

    y = AT @ ((G @ g) * (BT @ d))

The construction is the transposed Toom-Cook linear convolution: pick alpha - 1 finite
interpolation points a_j plus the point at infinity, let E_n be the alpha x n evaluation
matrix (row j = a_j^0 .. a_j^(n-1); the infinity row selects the leading coefficient), then

    AT = E_m^T,   G = diag(1/f) E_r,   BT = diag(f) (E_alpha^-1)^T,
    f_j = prod_{l != j} (a_j - a_l)  (f_inf = 1; f_0 is made positive)

All arithmetic is in ``fractions.Fraction`` so the matrices are exact rationals.  This is the
same parametrisation the reference obtains from its vendored generator
(``wincnn.py:49-70``: ``cookToomFilter`` with fractions in G), written independently from the
Lagrange / Vandermonde definition; ``tests/test_cooktoom.py`` pins it against matrices that
generator produced for the point sets the reference uses (``matrix_conv.py:12-40``).

The hard-coded F(2,1), F(2,2) and F(2,3) triples of the reference (``matrix_conv.py:15-30``,
``matrix_convnd.py:14-36``; they carry the sign convention of the device code in
``calculation_kernels.cu:786-802,1543-1551``) are exposed through :func:`reference_table`.
"""
from __future__ import annotations

from fractions import Fraction
from typing import Iterable, List, Sequence, Tuple

import numpy as np

Matrix = List[List[Fraction]]

# Interpolation points used by the reference for each (m, r) it tabulates
# (matrix_conv.py:31-40).  F(4,3) is not tabulated there; (0, 1, -1, 2, -2) is the
# customary choice and what the reference's generator would be fed (the engine's device
# code uses ENGINE_F43_POINTS below instead).
_LONG_POINTS = (0, 1, -1, Fraction(1, 2), -Fraction(1, 2), Fraction(1, 3), -Fraction(1, 3),
                Fraction(3, 2), -Fraction(3, 2), -3, 2, -2)


# Points of the engine's F(4,3) device code (wino_common.cuh, Xf<4,3>): symmetric and dyadic,
# chosen for low fp16 error (see the comment there).
ENGINE_F43_POINTS = (Fraction(0), Fraction(5, 8), -Fraction(5, 8), Fraction(3, 2), -Fraction(3, 2))


def default_points(m: int, r: int) -> Tuple[Fraction, ...]:
    alpha = m + r - 1
    need = alpha - 1
    if need <= 5:
        pts = (0, 1, -1, 2, -2)[:need]
    else:
        pts = _LONG_POINTS[:need]
    if len(pts) < need:
        raise ValueError(f"no default point set for F({m},{r})")
    return tuple(Fraction(p) for p in pts)


def _eval_matrix(points: Sequence[Fraction], n: int) -> Matrix:
    """alpha x n evaluation matrix with the point at infinity as last row."""
    rows = [[Fraction(p) ** k for k in range(n)] for p in points]
    rows.append([Fraction(int(k == n - 1)) for k in range(n)])
    return rows


def _inverse(mat: Matrix) -> Matrix:
    n = len(mat)
    aug = [list(row) + [Fraction(int(i == j)) for j in range(n)] for i, row in enumerate(mat)]
    for col in range(n):
        piv = next(i for i in range(col, n) if aug[i][col] != 0)
        aug[col], aug[piv] = aug[piv], aug[col]
        inv = 1 / aug[col][col]
        aug[col] = [v * inv for v in aug[col]]
        for i in range(n):
            if i != col and aug[i][col] != 0:
                fac = aug[i][col]
                aug[i] = [vi - fac * vc for vi, vc in zip(aug[i], aug[col])]
    return [row[n:] for row in aug]


def cook_toom(m: int, r: int, points: Iterable | None = None) -> Tuple[Matrix, Matrix, Matrix]:
    """Exact (AT, G, BT) for F(m, r); shapes m x alpha, alpha x r, alpha x alpha."""
    if m < 1 or r < 1:
        raise ValueError("m and r must be positive")
    alpha = m + r - 1
    pts = tuple(Fraction(p) for p in (points if points is not None else default_points(m, r)))
    if len(pts) != alpha - 1:
        raise ValueError(f"F({m},{r}) needs {alpha - 1} finite points, got {len(pts)}")
    if len(set(pts)) != len(pts):
        raise ValueError("interpolation points must be distinct")
    f = []
    for j, aj in enumerate(pts):
        prod = Fraction(1)
        for l, al in enumerate(pts):
            if l != j:
                prod *= aj - al
        f.append(prod)
    if f and f[0] < 0:
        f[0] = -f[0]
    f.append(Fraction(1))
    e_m = _eval_matrix(pts, m)
    e_r = _eval_matrix(pts, r)
    e_a_inv = _inverse(_eval_matrix(pts, alpha))
    at = [[e_m[j][i] for j in range(alpha)] for i in range(m)]
    g = [[e_r[j][k] / f[j] for k in range(r)] for j in range(alpha)]
    bt = [[f[j] * e_a_inv[l][j] for l in range(alpha)] for j in range(alpha)]
    return at, g, bt


def as_float64(mat: Matrix) -> np.ndarray:
    return np.array([[float(v) for v in row] for row in mat], dtype=np.float64)


def reference_table(m: int, r: int) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """(AT, G, BT) as float64 in the reference's own convention.

    r <= 3 with m == 2 returns the hand-written tables of matrix_conv.py:15-30 /
    matrix_convnd.py:14-36 (identity for r = 1, Lavin's signs for r = 3); every other
    (m, r) comes from :func:`cook_toom`.
    """
    if m == 2 and r == 1:
        return np.eye(2), np.ones((2, 1)), np.eye(2)
    if m == 2 and r == 2:
        return (np.array([[1., 1., 0.], [0., 1., 1.]]),
                np.array([[1., 0.], [1., 1.], [0., 1.]]),
                np.array([[1., -1., 0.], [0., 1., 0.], [0., -1., 1.]]))
    if m == 2 and r == 3:
        return (np.array([[1., 1., 1., 0.], [0., 1., -1., -1.]]),
                np.array([[1., 0., 0.], [.5, .5, .5], [.5, -.5, .5], [0., 0., 1.]]),
                np.array([[1., 0., -1., 0.], [0., 1., 1., 0.], [0., -1., 1., 0.], [0., 1., 0., -1.]]))
    if m == 1 and r == 1:
        one = np.ones((1, 1))
        return one, one.copy(), one.copy()
    at, g, bt = cook_toom(m, r)
    return as_float64(at), as_float64(g), as_float64(bt)


def verify_identity(at: Matrix, g: Matrix, bt: Matrix) -> bool:
    """Exact check that sum_j AT[i][j] G[j][k] BT[j][l] == [l == i + k]."""
    m, alpha, r = len(at), len(bt), len(g[0])
    for i in range(m):
        for k in range(r):
            for l in range(alpha):
                s = sum(Fraction(at[i][j]) * Fraction(g[j][k]) * Fraction(bt[j][l]) for j in range(alpha))
                if s != (1 if l == i + k else 0):
                    return False
    return True
