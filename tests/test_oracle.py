"""The CPU oracle against (a) outputs of the reference's matrix_convnd.conv stored as golden
fixtures, (b) an independent numpy direct convolution, (c) the float64 direct convolution for
every decomposition it restates (tiles, DWM pieces, stride-2 polyphase, F(4,3))."""
import os

import numpy as np
import pytest
import torch

from oracle import winograd_oracle as wo

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "tile_algebra_golden.npz"))


@pytest.mark.parametrize("name", ["1d_r3", "2d_r3", "3d_r3", "2d_r2x3", "2d_r1x3", "3d_r3x2x1"])
def test_tile_algebra_matches_reference_output(name):
    x, w, y = (torch.from_numpy(GOLD[f"{name}_{k}"]) for k in "xwy")
    got = wo.base_conv(x, w, [2] * (x.dim() - 2))
    assert got.shape == y.shape
    assert (got - y).abs().max().item() < 1e-12


@pytest.mark.parametrize("name", ["2d_r5", "2d_r7"])
def test_dwm_on_one_tile_matches_reference_direct_large_r(name):
    # the reference evaluates r = 5, 7 with one large F(2,r); the DWM decomposition of the
    # same tile must agree (dwm_convnd.py:7-40 states this identity).
    x, w, y = (torch.from_numpy(GOLD[f"{name}_{k}"]) for k in "xwy")
    got = wo.winograd_conv_cpu(x, w, dtype=torch.float64)
    assert (got - y).abs().max().item() < 1e-10


def test_direct_conv_torch_vs_numpy():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(2, 3, 9, 8, generator=g)
    w = torch.randn(4, 3, 5, 3, generator=g)
    a = wo.direct_conv_f64(x, w, stride=(2, 1), padding=(2, 1)).numpy()
    b = wo.direct_conv_numpy(x.numpy(), w.numpy(), stride=(2, 1), padding=(2, 1))
    np.testing.assert_allclose(a, b, atol=1e-12)
    x3 = torch.randn(1, 2, 5, 6, 7, generator=g)
    w3 = torch.randn(3, 2, 3, 3, 3, generator=g)
    np.testing.assert_allclose(wo.direct_conv_f64(x3, w3, padding=1).numpy(),
                               wo.direct_conv_numpy(x3.numpy(), w3.numpy(), padding=1), atol=1e-12)


CASES = [
    # N, C, K, spatial, kernel, stride, pad, tile_m
    (2, 5, 4, (9, 10), (3, 3), 1, 1, 2),
    (2, 5, 4, (9, 10), (3, 3), 1, 1, 4),
    (1, 3, 2, (11, 7), (5, 5), 1, 2, 2),
    (1, 3, 2, (13, 12), (7, 7), 1, 3, 2),
    (2, 3, 4, (17, 16), (7, 7), 2, 3, 2),
    (1, 2, 3, (9, 9), (4, 4), 1, 0, 2),
    (1, 2, 3, (10, 9), (3, 3), 2, 1, 2),
    (1, 3, 2, (5, 6, 7), (3, 3, 3), 1, 1, 2),
    (1, 2, 2, (6, 6, 6), (5, 3, 2), 1, 0, 2),
    (1, 2, 2, (12, 12), (9, 9), 1, 4, 2),
]


@pytest.mark.parametrize("n,c,k,sp,ks,stride,pad,m", CASES)
def test_winograd_cpu_equals_direct(n, c, k, sp, ks, stride, pad, m):
    g = torch.Generator().manual_seed(7)
    x = torch.randn((n, c) + sp, generator=g, dtype=torch.float64)
    w = torch.randn((k, c) + ks, generator=g, dtype=torch.float64)
    y = wo.winograd_conv_cpu(x, w, stride=stride, padding=pad, tile_m=m, dtype=torch.float64)
    o = wo.direct_conv_f64(x, w, stride=stride, padding=pad)
    assert y.shape == o.shape
    assert (y - o).abs().max().item() < 1e-10


def test_dwm_cut_rule():
    # base_conv_launchers.h:58-388: 4 -> 2+2, 5 -> 3+2, 7 -> 3+3+1, 8 -> 3+3+2, 10 -> 3+3+3+1
    assert wo.dwm_cuts(4) == [(0, 2), (2, 2)]
    assert wo.dwm_cuts(5) == [(0, 3), (3, 2)]
    assert wo.dwm_cuts(7) == [(0, 3), (3, 3), (6, 1)]
    assert wo.dwm_cuts(8) == [(0, 3), (3, 3), (6, 2)]
    assert wo.dwm_cuts(10) == [(0, 3), (3, 3), (6, 3), (9, 1)]
    assert len(wo.dwm_pieces((7, 7), (2, 2))) == 9
    assert len(wo.dwm_pieces((5, 5), (1, 1))) == 4


def test_split_concat_roundtrip_and_mask():
    x = torch.arange(2 * 3 * 7 * 5, dtype=torch.float64).reshape(2, 3, 7, 5)
    tiles = wo.wino_split_cpu(x, (3, 3), (2, 2))          # out 5x3 -> 3x2 tiles
    assert tiles.shape == (2 * 3 * 2, 3, 4, 4)
    assert torch.equal(tiles[0, :, :, :], x[0, :, 0:4, 0:4])
    # last tile column reads past the edge: zero filled
    assert torch.equal(tiles[1, :, :, 3], torch.zeros(3, 4, dtype=torch.float64))
    y = torch.randn(12, 4, 2, 2, dtype=torch.float64)
    out = wo.wino_concat_cpu(y, (5, 3), (2, 2), 2)
    assert out.shape == (2, 4, 5, 3)
    assert torch.equal(out[0, :, 0:2, 0:2], y[0])
    assert torch.equal(out[0, :, 4, 2], y[5][:, 0, 0])


def test_fp16_emulation_error_is_reported_not_zero():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(1, 16, 12, 12, generator=g).half().float()
    w = wo.kaiming_normal((8, 16, 3, 3), 4).half().float()
    o = wo.direct_conv_f64(x, w, padding=1)
    e32 = wo.error_metrics(wo.winograd_conv_cpu(x, w, padding=1), o)["E_B"]
    e16 = wo.error_metrics(wo.winograd_conv_cpu(x, w, padding=1, fp16=True), o)["E_B"]
    assert e32 < 1e-5 < e16 < 5e-2


@pytest.mark.parametrize("n,c,k,sp,ks,pad", [
    (2, 3, 4, (9, 10), (3, 3), 1),
    (1, 5, 2, (8, 11), (5, 5), 2),        # two windows along W, the second with two taps
    (1, 2, 3, (7, 9), (7, 7), 3),         # three windows, the last with one tap
    (1, 3, 2, (6, 7), (1, 3), 0),
    (1, 2, 2, (5, 6, 7), (3, 3, 3), 1),   # 3-D: depth and row taps are identity pieces
    (1, 2, 2, (9, 9), (4, 4), 0),
])
def test_row_piece_decomposition_equals_direct(n, c, k, sp, ks, pad):
    """1 x 3 DWM pieces (F(2,3) along W, identity pieces along the other dimensions) summed in the Winograd
    domain give the direct convolution: the algebra of the engine's row kernel."""
    g = torch.Generator().manual_seed(3)
    x = torch.randn(n, c, *sp, generator=g, dtype=torch.float64)
    w = torch.randn(k, c, *ks, generator=g, dtype=torch.float64)
    y = wo.row_piece_conv_cpu(x, w, padding=pad)
    o = wo.direct_conv_f64(x, w, padding=pad)
    assert y.shape == o.shape
    assert (y - o).abs().max().item() < 1e-11


@pytest.mark.parametrize("n,c,k,sp,ks,stride,pad", [
    (2, 3, 4, (15, 14), (7, 7), 2, 3),             # the 7x7 stride-2 case: 4x4, 4x3, 3x4, 3x3 parts
    (1, 2, 3, (9, 10), (3, 3), 2, 1),
    (1, 4, 2, (11, 8), (5, 5), 2, 0),              # odd extents, no padding
    (1, 2, 2, (7, 8, 9), (3, 3, 3), 2, 1),         # 3-D: eight phases
    (1, 2, 2, (9, 12), (3, 5), (1, 2), (1, 2)),    # stride 2 along W only
])
def test_stride2_as_stride1_over_phase_channels(n, c, k, sp, ks, stride, pad):
    """Folding the polyphase parts of a stride-2 convolution into channels leaves a stride-1, unpadded
    convolution with the same result (how the engine runs stride 2 on its stride-1 kernel)."""
    g = torch.Generator().manual_seed(4)
    x = torch.randn(n, c, *sp, generator=g, dtype=torch.float64)
    w = torch.randn(k, c, *ks, generator=g, dtype=torch.float64)
    xs, ws = wo.phases_to_channels_cpu(x, w, stride, pad)
    o = wo.direct_conv_f64(x, w, stride=stride, padding=pad)
    y = wo.direct_conv_f64(xs, ws)
    assert y.shape == o.shape and (y - o).abs().max().item() < 1e-11
    # and through the row-piece decomposition, as the device does
    assert (wo.row_piece_conv_cpu(xs, ws) - o).abs().max().item() < 1e-10
