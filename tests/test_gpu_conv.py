"""Parity of the forward convolution (through the C ABI) with the float64 direct-convolution
oracle: the BASELINE configurations at full size, small cases covering every edge the reference
handles (odd output extents -> masked last tile, zero-fill padding, every DWM piece shape) and
the ones it does not (stride 2, F(4x4,3x3), channel counts that are not vector multiples),
plus size-independent properties at full size."""
import pytest
import torch

from oracle import winograd_oracle as wo
from pytorch_winoconv_b200 import capi
from tests.gpu_util import TOL, check_against_oracle, run_engine, seeded

pytestmark = pytest.mark.gpu

SMALL = [
    # N, C, K, spatial, kernel, stride, pad, tile_m
    (2, 8, 8, (9, 10), (3, 3), 1, 1, 2),
    (2, 8, 8, (9, 10), (3, 3), 1, 1, 4),
    (1, 16, 8, (13, 13), (3, 3), 1, 0, 4),       # odd outputs, no padding
    (2, 3, 5, (12, 11), (3, 3), 1, 1, 4),        # C, K not vector multiples
    (1, 7, 9, (10, 10), (3, 3), 1, 1, 2),
    (1, 8, 8, (11, 9), (5, 5), 1, 2, 0),         # 5x5 -> 4 pieces
    (1, 6, 4, (15, 14), (7, 7), 1, 3, 0),        # 7x7 -> 9 pieces
    (2, 3, 8, (33, 32), (7, 7), 2, 3, 0),        # stride-2 polyphase
    (1, 8, 8, (12, 13), (3, 3), 2, 1, 0),
    (1, 4, 4, (12, 12), (9, 9), 1, 4, 0),
    (1, 8, 8, (9, 9), (4, 4), 1, 0, 0),          # 4 -> 2 + 2
    (1, 8, 8, (10, 9), (3, 4), 1, 0, 0),
    (1, 8, 8, (9, 9), (1, 1), 1, 0, 0),
    (1, 8, 8, (9, 12), (1, 3), 1, 0, 0),
    (1, 8, 8, (5, 6, 7), (3, 3, 3), 1, 1, 0),    # 3-D
    (1, 4, 6, (6, 7, 6), (5, 3, 2), 1, 0, 0),
    (1, 4, 4, (4, 9, 9), (1, 3, 3), 1, 1, 0),    # depth kernel of 1 in a 3-D tensor
    (1, 4, 4, (7, 8, 9), (3, 3, 3), 2, 1, 0),    # 3-D stride 2
    (1, 4, 4, (12, 4, 4), (10, 3, 3), 1, 1, 0),  # 10 -> 3+3+3+1
]


@pytest.mark.parametrize("n,c,k,sp,ks,stride,pad,m", SMALL)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_small_cases(n, c, k, sp, ks, stride, pad, m, dtype):
    x = seeded((n, c) + sp, 11, dtype=dtype)
    w = wo.kaiming_normal((k, c) + ks, 12).to(dtype)
    y, _ = run_engine(x, w, stride=stride, padding=pad, tile_m=m)
    check_against_oracle(x, w, y, stride=stride, padding=pad)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("eng", [capi.GEMM_SIMT, capi.GEMM_TCGEN05])
def test_both_gemm_engines(dtype, eng):
    x = seeded((2, 24, 14, 14), 21, dtype=dtype)
    w = wo.kaiming_normal((40, 24, 3, 3), 22).to(dtype)
    y, conv = run_engine(x, w, padding=1, gemm_engine=eng)
    assert conv.info.gemm_engine == eng
    check_against_oracle(x, w, y, padding=1)


def test_epilogue_bias_relu_pool():
    x = seeded((2, 8, 13, 14), 31, dtype=torch.float16)
    w = wo.kaiming_normal((16, 8, 3, 3), 32).half()
    b = seeded((16,), 33, dtype=torch.float16)
    o = wo.direct_conv_f64(x, w, padding=1) + b.double().view(1, -1, 1, 1)
    for m in (2, 4):
        y, _ = run_engine(x, w, padding=1, tile_m=m, bias=b, relu=True)
        assert wo.error_metrics(y, torch.relu(o))["E_A"] < 5e-3
        y, _ = run_engine(x, w, padding=1, tile_m=m, bias=b, relu=True, pool2=True)
        op = torch.nn.functional.max_pool2d(torch.relu(o), 2)
        assert tuple(y.shape) == tuple(op.shape) == (2, 16, 6, 7)
        assert wo.error_metrics(y, op)["E_A"] < 5e-3


def test_blocked_passes_equal_single_pass():
    # scratch for 256 tiles forces several passes over the 2 x 11 x 11 = 242... tiles of a bigger image
    from pytorch_winoconv_b200 import engine
    x = seeded((3, 16, 40, 44), 41, dtype=torch.float16)
    w = wo.kaiming_normal((16, 16, 3, 3), 42).half()
    dev = torch.device("cuda", 0)
    xl = x.permute(0, 2, 3, 1).contiguous().to(dev)
    conv = engine.WinoConv(xl.shape, w.to(dev), padding=1)
    y_full = conv(xl).clone()
    v = torch.empty(int(conv.info.input_ws_bytes_min) * 2, dtype=torch.uint8, device=dev)
    m = torch.empty(int(conv.info.product_ws_bytes_min) * 2, dtype=torch.uint8, device=dev)
    y_blk = torch.empty_like(y_full)
    capi.forward(conv.desc, xl.data_ptr(), conv.u.data_ptr(), None, y_blk.data_ptr(), v.data_ptr(), v.numel(),
                 m.data_ptr(), m.numel(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert conv.info.tiles > 256
    assert torch.equal(y_full, y_blk)
    with pytest.raises(capi.WinoconvError) as ei:
        capi.forward(conv.desc, xl.data_ptr(), conv.u.data_ptr(), None, y_blk.data_ptr(), v.data_ptr(), 1024,
                     m.data_ptr(), m.numel(), torch.cuda.current_stream().cuda_stream)
    assert ei.value.status == capi.ERR_WORKSPACE


# ---- BASELINE.json configurations at full size -------------------------------------------------
def test_cfg1_fp32_f23():
    x = seeded((8, 64, 56, 56), 0)
    w = wo.kaiming_normal((64, 64, 3, 3), 1)
    y, conv = run_engine(x, w, padding=1, tile_m=2)
    assert conv.info.positions == 16
    err = check_against_oracle(x, w, y, padding=1)
    ref = wo.error_metrics(wo.winograd_conv_cpu(x, w, padding=1, tile_m=2), wo.direct_conv_f64(x, w, padding=1))
    print("cfg1 engine", err, "reference algebra (CPU fp32)", ref)


@pytest.mark.parametrize("product_dtype", [None, torch.float16])
def test_cfg2_fp16_f43(product_dtype):
    x = seeded((32, 256, 28, 28), 0, dtype=torch.float16)
    w = wo.kaiming_normal((256, 256, 3, 3), 1).half()
    y, conv = run_engine(x, w, padding=1, tile_m=4, product_dtype=product_dtype)
    assert conv.info.positions == 36 and conv.info.gemm_engine == capi.GEMM_TCGEN05
    err = check_against_oracle(x, w, y, padding=1)
    print("cfg2 engine", product_dtype, err)


def test_cfg3a_fp16_7x7_stride2():
    x = seeded((64, 3, 224, 224), 0, dist="uniform", dtype=torch.float16)
    w = wo.kaiming_normal((64, 3, 7, 7), 1).half()
    y, conv = run_engine(x, w, stride=2, padding=3)
    assert conv.info.n_pieces == 9 and conv.info.positions == 100
    print("cfg3a engine", check_against_oracle(x, w, y, stride=2, padding=3))


def test_cfg3b_fp16_5x5():
    x = seeded((32, 128, 56, 56), 0, dtype=torch.float16)
    w = wo.kaiming_normal((128, 128, 5, 5), 1).half()
    y, conv = run_engine(x, w, padding=2)
    assert conv.info.n_pieces == 4 and conv.info.positions == 49
    print("cfg3b engine", check_against_oracle(x, w, y, padding=2))


def test_cfg4_fp16_3d():
    x = seeded((8, 64, 16, 56, 56), 0, dtype=torch.float16)
    w = wo.kaiming_normal((64, 64, 3, 3, 3), 1).half()
    y, conv = run_engine(x, w, padding=1)
    assert conv.info.positions == 64
    print("cfg4 engine", check_against_oracle(x, w, y, padding=1))


def test_linearity_at_full_size():
    # conv(a x1 + x2, w) == a conv(x1, w) + conv(x2, w) up to rounding, at config 2's size
    x1 = seeded((32, 256, 28, 28), 5, dtype=torch.float16)
    x2 = seeded((32, 256, 28, 28), 6, dtype=torch.float16)
    w = wo.kaiming_normal((256, 256, 3, 3), 7).half()
    xs = (2.0 * x1.float() + x2.float()).half()
    y1, _ = run_engine(x1, w, padding=1)
    y2, _ = run_engine(x2, w, padding=1)
    ys, _ = run_engine(xs, w, padding=1)
    comb = 2.0 * y1.double() + y2.double()
    assert wo.error_metrics(ys, comb)["E_B"] < 2 * TOL[torch.float16]


def test_translation_equivariance():
    # shifting the input by one tile (4 px) shifts the output: catches tile / halo indexing slips
    x = seeded((1, 16, 36, 36), 8, dtype=torch.float16)
    w = wo.kaiming_normal((16, 16, 3, 3), 9).half()
    y, _ = run_engine(x, w, padding=0)
    ys, _ = run_engine(x[:, :, 4:, 4:].contiguous(), w, padding=0)
    assert torch.equal(y[:, :, 4:, 4:], ys)
