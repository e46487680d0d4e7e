"""Generate the golden fixtures in this directory from the reference's own Python code.

Run where a checkout of the reference project is available, pointing ``WINOCONV_REFERENCE_DIR`` at it:

    WINOCONV_REFERENCE_DIR=<reference checkout> python tests/golden/make_golden.py

It imports the only two reference modules that run on CPU -- ``wincnn`` (the vendored
Cook-Toom generator) and ``matrix_convnd`` (``conv`` / ``base_conv32``, matrix_convnd.py:99-153)
-- and stores their outputs on seeded inputs.  ``wincnn.py:56,61`` divides a sympy Matrix by a
Matrix, which current sympy rejects; the harness-side shim below restores the old meaning
(multiply by the inverse; the divisor is diagonal).  Nothing of the reference is copied: only
inputs and the numbers it computed are stored.

Fixtures:
  cooktoom_golden.npz      AT/G/BT for the (points, m, r) the reference tabulates
                           (matrix_conv.py:31-40) plus F(4,3) on (0,1,-1,2,-2)
  tile_algebra_golden.npz  matrix_convnd.conv outputs for 1-D/2-D/3-D tiles, r in {1,2,3,5,7}
  split_control_golden.npz the piece boxes of every kernel shape in the reference's splitControl()
                           look-up table (src/base_conv_launchers.h:58-388), read from the source text:
                           shapes [n,3] = (kD,kH,kW), offsets [n+1], boxes [sum pieces, 6] =
                           (D_s, D_e, H_s, H_e, W_s, W_e); a branch's piece count is the length of its
                           D_s array, as the C code computes it (`sizeof(D_s) / sizeof(D_s[0])`)
"""
import os
import sys
import warnings

import numpy as np
import torch

HERE_EARLY = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("WINOCONV_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE_EARLY))), "reference")
HERE = os.path.dirname(os.path.abspath(__file__))


def _install_sympy_shim():
    from sympy.matrices.matrixbase import MatrixBase
    orig = MatrixBase.__truediv__

    def truediv(self, other):
        if isinstance(other, MatrixBase):
            return self * other.inv()
        return orig(self, other)

    MatrixBase.__truediv__ = truediv


def parse_split_control(header_path):
    """[( (kD,kH,kW), [(D_s,D_e,H_s,H_e,W_s,W_e), ...] ), ...] from the text of splitControl()."""
    import re
    text = open(header_path).read()
    text = text[text.index("static void splitControl"):]
    out = []
    branches = re.split(r"if ?\(D == (\d+) && H == (\d+) && W == (\d+)\)", text)
    for i in range(1, len(branches), 4):
        shape = tuple(int(v) for v in branches[i:i + 3])
        body = branches[i + 3]
        arrs = {}
        for name in ("D_s", "D_e", "H_s", "H_e", "W_s", "W_e"):
            m = re.search(r"int %s\[\] = \{([^}]*)\}" % name, body)
            arrs[name] = [int(v) for v in m.group(1).split(",")]
        n = len(arrs["D_s"])
        out.append((shape, [tuple(arrs[k][j] for k in ("D_s", "D_e", "H_s", "H_e", "W_s", "W_e")) for j in range(n)]))
    return out


def main():
    warnings.filterwarnings("ignore")
    _install_sympy_shim()
    sys.path.insert(0, REF)
    import wincnn                     # noqa: E402  (reference module)
    import matrix_convnd              # noqa: E402  (reference module)
    from sympy import Rational

    long_pts = (0, 1, -1, Rational(1, 2), -Rational(1, 2), Rational(1, 3), -Rational(1, 3),
                Rational(3, 2), -Rational(3, 2), -3, 2, -2)
    cases = [((0, 1, -1), 2, 3), ((0, 1, -1, 2), 2, 4), ((0, 1, -1, 2, -2), 2, 5),
             (long_pts, 2, 6), (long_pts, 2, 7), (long_pts, 2, 9), (long_pts, 2, 11),
             (long_pts, 9, 5), ((0, 1, -1, 2, -2), 4, 3), ((0, 1), 2, 2)]
    blob = {}
    for pts, m, r in cases:
        at, g, bt = wincnn.showCookToomFilter(pts, m, r)
        alpha = m + r - 1
        used = pts[:alpha - 1]
        blob[f"F{m}_{r}_points_num"] = np.array([int(Rational(p).p) for p in used], dtype=np.int64)
        blob[f"F{m}_{r}_points_den"] = np.array([int(Rational(p).q) for p in used], dtype=np.int64)
        blob[f"F{m}_{r}_AT"], blob[f"F{m}_{r}_G"], blob[f"F{m}_{r}_BT"] = at, g, bt
    # the reference's hand-written tables (matrix_convnd.py:14-36)
    for r in (1, 2, 3):
        blob[f"table2_{r}_AT"] = matrix_convnd.A[(2, r)]
        blob[f"table2_{r}_G"] = matrix_convnd.G[(2, r)]
        blob[f"table2_{r}_BT"] = matrix_convnd.B[(2, r)]
    np.savez_compressed(os.path.join(HERE, "cooktoom_golden.npz"), **blob)

    blob = {}
    gen = torch.Generator().manual_seed(20240611)
    tile_cases = [("1d_r3", 1, (3,)), ("2d_r3", 2, (3, 3)), ("3d_r3", 3, (3, 3, 3)),
                  ("2d_r2x3", 2, (2, 3)), ("2d_r1x3", 2, (1, 3)), ("2d_r5", 2, (5, 5)),
                  ("2d_r7", 2, (7, 7)), ("3d_r3x2x1", 3, (3, 2, 1))]
    for name, n, r in tile_cases:
        t, c, k = 5, 6, 4
        alpha = [rr + 1 for rr in r]
        x = torch.randn([t, c] + alpha, generator=gen, dtype=torch.float64)
        w = torch.randn([k, c] + list(r), generator=gen, dtype=torch.float64)
        y = matrix_convnd.conv(x.clone(), w.clone(), n)          # [T, K, 2, ...]
        blob[f"{name}_x"], blob[f"{name}_w"], blob[f"{name}_y"] = x.numpy(), w.numpy(), y.numpy()
    np.savez_compressed(os.path.join(HERE, "tile_algebra_golden.npz"), **blob)
    lut = parse_split_control(os.path.join(REF, "src", "base_conv_launchers.h"))
    shapes = np.array([sh for sh, _ in lut], dtype=np.int64)
    offsets = np.cumsum([0] + [len(b) for _, b in lut]).astype(np.int64)
    boxes = np.array([b for _, bs in lut for b in bs], dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "split_control_golden.npz"), shapes=shapes, offsets=offsets, boxes=boxes)
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


if __name__ == "__main__":
    main()
