"""Host-side checks that need no GPU: the C-ABI library loads, exports every symbol the header
declares, plans shapes the way the oracle's restatement of the reference does, and reports
errors as status codes instead of exiting the process."""
import os
import re

import pytest
import torch

from oracle import winograd_oracle as wo
from pytorch_winoconv_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "winoconv_b200.h")).read()
    declared = set(re.findall(r"WINOCONV_API\s+[\w\s\*]+?\b(winoconv_\w+)\s*\(", header))
    assert declared == set(capi.EXPORTED_SYMBOLS)
    L = capi.lib()
    for name in declared:
        assert getattr(L, name) is not None
    assert L.winoconv_abi_version() == 1
    assert L.winoconv_status_string(capi.ERR_UNSUPPORTED) == b"unsupported configuration"


BASELINE_CONFIGS = [
    # name, kwargs, expected (positions, pieces, tiles)
    ("cfg1", dict(ndim=2, batch=8, c_in=64, k_out=64, in_size=(56, 56), ker_size=3, pad=1, tile_m=2, dtype=capi.F32), (16, 1, 6272)),
    ("cfg2", dict(ndim=2, batch=32, c_in=256, k_out=256, in_size=(28, 28), ker_size=3, pad=1, tile_m=4), (36, 1, 1568)),
    ("cfg1 as F(6x6,3x3)", dict(ndim=2, batch=8, c_in=64, k_out=64, in_size=(56, 56), ker_size=3, pad=1, tile_m=6, dtype=capi.F32), (64, 1, 800)),
    ("cfg3a", dict(ndim=2, batch=64, c_in=3, k_out=64, in_size=(224, 224), ker_size=7, stride=2, pad=3, algo=capi.ALGO_STAGED), (100, 9, 200704)),
    ("cfg3b", dict(ndim=2, batch=32, c_in=128, k_out=128, in_size=(56, 56), ker_size=5, pad=2, algo=capi.ALGO_STAGED), (49, 4, 25088)),
    ("cfg4", dict(ndim=3, batch=8, c_in=64, k_out=64, in_size=(16, 56, 56), ker_size=3, pad=1, algo=capi.ALGO_STAGED), (64, 1, 50176)),
]


@pytest.mark.parametrize("name,kw,expect", BASELINE_CONFIGS)
def test_plan_matches_hand_computed_figures(name, kw, expect):
    info = capi.plan(capi.make_desc(**kw))
    assert (info.positions, info.n_pieces, info.tiles) == expect
    d = capi.make_desc(**kw)
    n_out = 1
    for o in info.conv_out_size:
        n_out *= o
    ks = 1
    for k in d.ker_size:
        ks *= k
    assert info.direct_flops == pytest.approx(2.0 * d.batch * d.k_out * d.c_in * ks * n_out)
    assert info.gemm_flops == pytest.approx(2.0 * info.positions * info.tiles * d.c_in * d.k_out)
    assert info.algo == capi.ALGO_STAGED


def test_auto_takes_f43_where_it_was_measured_to_win():
    """AUTO on a 16-bit 3x3 stride-1 layer: the row-piece kernel, except 512 -> 512 channels with 4-wide tiles that cover
    the output exactly and at least 4096 of them -- there staged F(4x4,3x3) (36 positions, V and M scratch)."""
    def plan(n, c, k, hw, **kw):
        return capi.plan(capi.make_desc(ndim=2, batch=n, c_in=c, k_out=k, in_size=(hw, hw), ker_size=3, pad=1, **kw))
    big = plan(256, 512, 512, 28)
    assert big.algo == capi.ALGO_STAGED and big.positions == 36 and list(big.tile_m) == [1, 4, 4] and big.tiles == 256 * 49
    assert big.input_ws_bytes == 36 * 256 * 49 * 512 * 2 and big.product_ws_bytes == 36 * 256 * 49 * 512 * 4
    for n, c, k, hw in ((32, 512, 512, 28),       # too few tiles to fill the GPU
                        (256, 512, 512, 14),      # 4-wide tiles would cover 16 x 16
                        (256, 256, 512, 28),      # fewer input channels
                        (256, 256, 256, 56)):
        i = plan(n, c, k, hw)
        assert i.algo == capi.ALGO_ROW and i.positions == 4 and i.input_ws_bytes == 0, (n, c, k, hw)
    assert plan(256, 512, 512, 28, tile_m=2).algo == capi.ALGO_ROW          # an explicit tile keeps its algorithm
    assert plan(256, 512, 512, 28, algo=capi.ALGO_ROW).algo == capi.ALGO_ROW


@pytest.mark.parametrize("kw,windows,tiles", [
    (dict(ndim=2, batch=64, c_in=3, k_out=64, in_size=(224, 224), ker_size=7, stride=2, pad=3), 9, 64 * 56 * 56),
    (dict(ndim=2, batch=32, c_in=128, k_out=128, in_size=(56, 56), ker_size=5, pad=2), 4, 32 * 28 * 28),
    (dict(ndim=3, batch=8, c_in=64, k_out=64, in_size=(16, 56, 56), ker_size=3, pad=1), 3, 8 * 16 * 28 * 28),
    (dict(ndim=2, batch=2, c_in=16, k_out=16, in_size=(9, 9), ker_size=3, pad=1, tile_m=2), 1, 2 * 5 * 5),
])
def test_fused_plan(kw, windows, tiles):
    """The 3x3-piece fused kernel: 16 positions, every piece a 3x3 window in the GEMM reduction, depth taps
    applied directly, no scratch."""
    d = capi.make_desc(**{**kw, "algo": capi.ALGO_FUSED})
    info = capi.plan(d)
    assert info.algo == capi.ALGO_FUSED
    assert (info.positions, info.n_pieces, info.tiles) == (16, windows, tiles)
    assert info.input_ws_bytes == 0 and info.product_ws_bytes == 0
    assert info.filter_bytes == 16 * d.k_out * windows * info.c_pad * 2
    assert info.gemm_flops == pytest.approx(2.0 * 16 * tiles * windows * d.c_in * d.k_out)


def test_row_piece_plan():
    """AUTO picks the row-piece kernel for 16-bit stride-1 convolutions: 4 positions, kD*kH*ceil(kW/3) pieces."""
    d = capi.make_desc(ndim=2, batch=32, c_in=128, k_out=128, in_size=(56, 56), ker_size=5, pad=2)
    info = capi.plan(d)
    assert info.algo == capi.ALGO_ROW and (info.positions, info.n_pieces) == (4, 10)
    assert info.tiles == 32 * 56 * 28 and info.input_ws_bytes == 0 and info.product_ws_bytes == 0
    assert info.filter_bytes == 10 * 4 * 128 * 128 * 2
    assert info.gemm_flops == pytest.approx(2.0 * 4 * info.tiles * 10 * 128 * 128)
    d3 = capi.make_desc(ndim=3, batch=8, c_in=64, k_out=64, in_size=(16, 56, 56), ker_size=3, pad=1)
    i3 = capi.plan(d3)
    assert i3.algo == capi.ALGO_ROW and i3.n_pieces == 9
    rgb = capi.plan(capi.make_desc(ndim=2, batch=4, c_in=3, k_out=64, in_size=(224, 224), ker_size=3, pad=1, tile_m=2))
    # RGB with W * C a multiple of eight is read as it lies: no padded copy, no scratch
    assert rgb.algo == capi.ALGO_ROW and rgb.c_pad == 8 and rgb.input_ws_bytes == 0
    odd = capi.plan(capi.make_desc(ndim=2, batch=4, c_in=3, k_out=64, in_size=(224, 225), ker_size=3, pad=1, tile_m=2))
    assert odd.algo == capi.ALGO_ROW and odd.input_ws_bytes == 4 * 224 * 225 * 8 * 2      # 225 x 3 elements: padded copy
    s2 = capi.plan(capi.make_desc(ndim=2, batch=4, c_in=16, k_out=64, in_size=(64, 64), ker_size=7, stride=2, pad=3))
    # stride 2 runs on the row kernel as a stride-1 problem: 4 phases x 16 channels, 4 x 4 kernel (4 rows x 2 windows),
    # input gathered into scratch as [4, 32 + 3, 32 + 3, 64]
    assert s2.algo == capi.ALGO_ROW and s2.n_pieces == 8 and s2.input_ws_bytes == 4 * 35 * 35 * 64 * 2
    assert s2.gemm_flops == pytest.approx(2.0 * 4 * s2.tiles * 8 * 64 * 64)
    s2f = capi.plan(capi.make_desc(ndim=2, batch=4, c_in=16, k_out=64, in_size=(64, 64), ker_size=7, stride=2, pad=3, algo=capi.ALGO_FUSED))
    assert s2f.algo == capi.ALGO_FUSED                      # the 3x3-piece kernel on request
    with pytest.raises(capi.WinoconvError) as ei:           # stride 3 is no Winograd / DWM case of either single-kernel path
        capi.plan(capi.make_desc(ndim=2, batch=4, c_in=16, k_out=64, in_size=(64, 64), ker_size=7, stride=3, pad=3, algo=capi.ALGO_ROW))
    assert ei.value.status in (capi.ERR_UNSUPPORTED, capi.ERR_INVALID_ARGUMENT)


def test_fused_refused_where_it_does_not_apply():
    for kw in (dict(dtype=capi.F32), dict(tile_m=4), dict(gemm_engine=capi.GEMM_SIMT), dict(product_dtype=capi.F16)):
        base = dict(ndim=2, batch=1, c_in=8, k_out=8, in_size=(16, 16), ker_size=3, algo=capi.ALGO_FUSED)
        base.update(kw)
        with pytest.raises(capi.WinoconvError) as ei:
            capi.plan(capi.make_desc(**base))
        assert ei.value.status == capi.ERR_UNSUPPORTED
    auto = capi.plan(capi.make_desc(ndim=2, batch=1, c_in=8, k_out=8, in_size=(16, 16), ker_size=3, dtype=capi.F32))
    assert auto.algo == capi.ALGO_STAGED


@pytest.mark.parametrize("ks,stride", [((5, 5), 1), ((7, 7), 1), ((7, 7), 2), ((9, 9), 1), ((4, 4), 1), ((3, 4), 1),
                                       ((10, 3), 1), ((8, 4), 1), ((3, 3), 2), ((1, 1), 1), ((2, 2), 1)])
def test_piece_table_matches_oracle_rule(ks, stride):
    d = capi.make_desc(ndim=2, batch=1, c_in=8, k_out=8, in_size=(32, 32), ker_size=ks, stride=stride, tile_m=2)
    got = capi.plan_pieces(d)
    want = wo.dwm_pieces((1,) + ks, (1, stride, stride))
    want = [(tuple(p[0] for p in piece), tuple(p[1] for p in piece), tuple(p[2] for p in piece)) for piece in want]
    assert got == want


def _split_control_golden():
    import os
    import numpy as np
    d = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "split_control_golden.npz"))
    for i, shape in enumerate(d["shapes"].tolist()):
        yield tuple(shape), [tuple(b) for b in d["boxes"][d["offsets"][i]:d["offsets"][i + 1]].tolist()]


def test_piece_table_reproduces_every_box_of_the_reference_lut():
    """All 36 kernel shapes of splitControl() (src/base_conv_launchers.h:58-388), read from the reference's source
    by tests/golden/make_golden.py: the library's rule and the oracle's rule give the same boxes in the same order."""
    n = 0
    for shape, boxes in _split_control_golden():
        if shape[0] == 1:
            d = capi.make_desc(ndim=2, batch=1, c_in=8, k_out=8, in_size=(16, 16), ker_size=shape[1:], tile_m=2)
        else:
            d = capi.make_desc(ndim=3, batch=1, c_in=8, k_out=8, in_size=(16, 16, 16), ker_size=shape, tile_m=2)
        got = [(st[0], st[0] + r[0], st[1], st[1] + r[1], st[2], st[2] + r[2]) for ph, st, r in capi.plan_pieces(d)]
        assert all(ph == (0, 0, 0) for ph, _, _ in capi.plan_pieces(d))
        assert got == boxes, (shape, got, boxes)
        want = wo.dwm_pieces(shape, (1, 1, 1))
        assert [(p[0][1], p[0][1] + p[0][2], p[1][1], p[1][1] + p[1][2], p[2][1], p[2][1] + p[2][2]) for p in want] == boxes, shape
        n += 1
    assert n == 36


def test_piece_table_3d():
    d = capi.make_desc(ndim=3, batch=1, c_in=8, k_out=8, in_size=(12, 12, 12), ker_size=(5, 7, 7))
    got = capi.plan_pieces(d)
    want = wo.dwm_pieces((5, 7, 7), (1, 1, 1))
    assert len(got) == len(want) == 18
    assert [g[2] for g in got] == [tuple(p[2] for p in piece) for piece in want]


def test_tile_counts_and_output_sizes():
    info = capi.plan(capi.make_desc(ndim=2, batch=2, c_in=8, k_out=8, in_size=(13, 10), ker_size=3, pad=1, tile_m=4))
    assert list(info.out_size) == [1, 13, 10] and list(info.tiles_per_dim) == [1, 4, 3] and info.tiles == 24
    info = capi.plan(capi.make_desc(ndim=2, batch=2, c_in=8, k_out=8, in_size=(13, 10), ker_size=3, pad=1,
                                    epilogue=capi.EPI_POOL2 | capi.EPI_RELU))
    assert list(info.out_size) == [1, 6, 5] and list(info.conv_out_size) == [1, 13, 10]
    info = capi.plan(capi.make_desc(ndim=2, batch=1, c_in=3, k_out=8, in_size=(224, 224), ker_size=7, stride=2, pad=3))
    assert list(info.out_size) == [1, 112, 112] and info.c_pad == 8


@pytest.mark.parametrize("kw,status", [
    (dict(ndim=4), capi.ERR_UNSUPPORTED),
    (dict(ker_size=11), capi.ERR_UNSUPPORTED),
    (dict(stride=3), capi.ERR_UNSUPPORTED),
    (dict(tile_m=4, ker_size=5), capi.ERR_UNSUPPORTED),
    (dict(tile_m=3), capi.ERR_UNSUPPORTED),
    (dict(batch=0), capi.ERR_INVALID_ARGUMENT),
    (dict(dtype=7), capi.ERR_INVALID_ARGUMENT),
    (dict(in_size=(2, 2), ker_size=5), capi.ERR_INVALID_ARGUMENT),
    (dict(dtype=capi.F32, gemm_engine=capi.GEMM_TCGEN05), capi.ERR_UNSUPPORTED),
    (dict(dtype=capi.F16, product_dtype=capi.BF16), capi.ERR_UNSUPPORTED),
    (dict(epilogue=64), capi.ERR_INVALID_ARGUMENT),
    (dict(algo=9), capi.ERR_INVALID_ARGUMENT),
])
def test_bad_descriptors_return_status_not_exit(kw, status):
    base = dict(ndim=2, batch=1, c_in=8, k_out=8, in_size=(16, 16), ker_size=3)
    base.update(kw)
    if base["ndim"] == 4:
        d = capi.make_desc(**{**base, "ndim": 2})
        d.ndim = 4
    else:
        d = capi.make_desc(**base)
    with pytest.raises(capi.WinoconvError) as ei:
        capi.plan(d)
    assert ei.value.status == status
    assert str(ei.value)


def test_null_pointers_rejected_before_any_device_call():
    d = capi.make_desc(ndim=2, batch=1, c_in=8, k_out=8, in_size=(16, 16), ker_size=3)
    with pytest.raises(capi.WinoconvError) as ei:
        capi.forward(d, None, None, None, None, None, 0, None, 0)
    assert ei.value.status == capi.ERR_INVALID_ARGUMENT
    with pytest.raises(capi.WinoconvError) as ei:
        capi.gemm_batched(capi.F16, capi.F32, capi.GEMM_AUTO, 1, 1, 12, 8, 16, 16, 16)
    assert ei.value.status == capi.ERR_INVALID_ARGUMENT   # c_pad not a multiple of 8


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU error path")
def test_no_device_is_an_error_not_a_fallback():
    d = capi.make_desc(ndim=2, batch=1, c_in=8, k_out=8, in_size=(16, 16), ker_size=3)
    with pytest.raises(capi.WinoconvError) as ei:
        capi.filter_transform(d, 16, 16)
    assert ei.value.status == capi.ERR_NO_DEVICE
    from pytorch_winoconv_b200 import engine
    with pytest.raises(RuntimeError):
        engine.WinoConv((1, 16, 16, 8), torch.zeros(8, 8, 3, 3))


def test_reference_named_modules_import():
    import MakePytorchPlusPlus as mpp
    import MakePytorchBackend as backend
    assert set(mpp.__all__) == {"AddGPU", "Foo", "WinoSplit", "WinoConcat", "DWM", "add_gpu", "wino_split", "wino_concat"}
    f = backend.Foo()
    f.setKey(7)
    assert f.getKey() == 7 and "7" in repr(f)
    from pytorch_winoconv_b200 import WinoConv, dwm, dwm_convnd, matrix_conv, matrix_conv3d, matrix_convnd
    for mod, names in [(dwm, ["dwm2d", "dwm3d", "dwm2d_", "dwm3d_"]),
                       (matrix_conv, ["conv16", "conv32", "conv", "base_conv32", "matrix_alloc"]),
                       (matrix_conv3d, ["conv16", "conv32", "conv", "base_conv32", "matrix_alloc"]),
                       (matrix_convnd, ["conv32", "conv", "base_conv32", "matrix_alloc"]),
                       (dwm_convnd, ["conv32"]), (WinoConv, ["Wino"])]:
        for n in names:
            assert hasattr(mod, n), (mod.__name__, n)
    with pytest.raises(RuntimeError):
        dwm.dwm2d(torch.zeros(1, 4, 8, 8), torch.zeros(4, 4, 3, 3))     # CPU tensors: no CPU path
