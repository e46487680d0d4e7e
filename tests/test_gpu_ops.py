"""The reference's operator surface on the GPU: MakePytorchBackend.DWM / WinoSplit / WinoConcat /
AddGPU and the Python wrappers dwm, matrix_conv, matrix_conv3d, matrix_convnd, dwm_convnd,
Split_and_Concat -- each checked against the oracle's restatement of what the reference computes."""
import pytest
import torch

from oracle import winograd_oracle as wo
from tests.gpu_util import TOL, seeded

pytestmark = pytest.mark.gpu


def test_add_gpu_and_foo():
    import MakePytorchPlusPlus as mpp
    a, b = seeded((1000,), 1).cuda(), seeded((1000,), 2).cuda()
    c = mpp.add_gpu(a, b)
    assert torch.equal(c, a + b)
    assert mpp.Foo().getKey() == 0


@pytest.mark.parametrize("m", [2, 4])
def test_split_and_concat_match_restatement(m):
    from pytorch_winoconv_b200.Split_and_Concat import wino_concat, wino_split
    x = seeded((2, 37, 11, 13), 3)
    tiles = wino_split(x.cuda(), (8, 37, 3, 3), m)
    want = wo.wino_split_cpu(x, (3, 3), (m, m))
    assert tuple(tiles.shape) == tuple(want.shape)
    assert torch.equal(tiles.cpu(), want)
    t = seeded((want.shape[0], 5, m, m), 4)
    out = wino_concat(t.cuda(), (9, 11), m)
    assert torch.equal(out.cpu(), wo.wino_concat_cpu(t, (9, 11), (m, m), 2))


def test_split_and_concat_3d():
    from pytorch_winoconv_b200.Split_and_Concat import wino_concat, wino_split
    x = seeded((1, 6, 7, 8, 9), 5)
    tiles = wino_split(x.cuda(), (4, 6, 3, 3, 3), 2)
    want = wo.wino_split_cpu(x, (3, 3, 3), (2, 2, 2))
    assert torch.equal(tiles.cpu(), want)
    t = seeded((want.shape[0], 4, 2, 2, 2), 6)
    out = wino_concat(t.cuda(), (5, 6, 7), 2)
    assert torch.equal(out.cpu(), wo.wino_concat_cpu(t, (5, 6, 7), (2, 2, 2), 1))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_dwm_op_direct(dtype):
    """DWM(Input NDHWC, Weight [kD,kH,kW,C,K], Output, stride, scratch...) as dwm.py:129-135 calls it,
    with caller-provided scratch of the reference's sizes."""
    import MakePytorchBackend as backend
    B, C, K, H, W, k = 2, 16, 24, 14, 15, 5
    x = seeded((B, C, H, W), 7, dtype=dtype)
    w = wo.kaiming_normal((K, C, k, k), 8).to(dtype)
    oh, ow = H - k + 1, W - k + 1
    nh, nw = (oh + 1) // 2, (ow + 1) // 2
    ksz = (k + 1 + (k - 1) // 3) ** 2 * 2
    dev = "cuda"
    tmp_in = torch.empty(ksz, B, 1, nh, nw, C, dtype=dtype, device=dev)
    tmp_w = torch.empty(ksz, C, K, dtype=dtype, device=dev)
    tmp_p = torch.empty(ksz * nh * nw * B * K, dtype=dtype, device=dev)
    tmp_ptr = torch.empty(3 * ksz, dtype=torch.long, device=dev)
    out = torch.zeros(B, 1, oh, ow, K, dtype=dtype, device=dev)
    xl = x.to(dev).unsqueeze(2).permute(0, 2, 3, 4, 1).contiguous()
    wl = w.to(dev).unsqueeze(2).permute(2, 3, 4, 1, 0).contiguous()
    backend.DWM(xl, wl, out, 1, tmp_in, tmp_w, tmp_p, tmp_ptr)
    y = out[:, 0].permute(0, 3, 1, 2).cpu()
    err = wo.error_metrics(y, wo.direct_conv_f64(x, w))
    assert err["E_B"] <= TOL[dtype], err
    with pytest.raises(RuntimeError):
        backend.DWM(xl, wl, out[:, :, :-1].contiguous(), 1, tmp_in, tmp_w, tmp_p, tmp_ptr)   # wrong output shape
    with pytest.raises(RuntimeError):
        backend.DWM(xl, wl, out, 3, tmp_in, tmp_w, tmp_p, tmp_ptr)                            # stride 3


def test_dwm2d_matches_example_shape():
    """example.py:99-109: x [1,224,10,10] uniform, w [32,224,7,7]; dwm2d vs float64 conv."""
    from pytorch_winoconv_b200 import dwm
    x = seeded((1, 224, 10, 10), 9, dist="uniform")
    w = seeded((32, 224, 7, 7), 10, dist="uniform")
    y = dwm.dwm2d(x.cuda(), w.cuda()).cpu()
    o = wo.direct_conv_f64(x, w)
    rel = ((y.double() - o).abs() / o.abs()).mean().item()     # the reference's printed metric
    assert rel < 1e-5
    b = seeded((32,), 11)
    yb = dwm.dwm2d(x.cuda(), w.cuda(), bias=b.cuda(), padding=(3, 3), stride=(2, 2)).cpu()
    ob = wo.direct_conv_f64(x, w, stride=2, padding=3) + b.double().view(1, -1, 1, 1)
    assert wo.error_metrics(yb, ob)["E_B"] < 1e-3


def test_dwm3d_matches_example_shape():
    """example.py:111-119: x [1,32,10,10,10], w [32,32,3,3,3]."""
    from pytorch_winoconv_b200 import dwm
    x = seeded((1, 32, 10, 10, 10), 12, dist="uniform")
    w = seeded((32, 32, 3, 3, 3), 13, dist="uniform")
    y = dwm.dwm3d(x.cuda(), w.cuda(), padding=1).cpu()
    assert wo.error_metrics(y, wo.direct_conv_f64(x, w, padding=1))["E_B"] < 1e-3
    yh = dwm.dwm3d(x.half().cuda(), w.half().cuda(), padding=(1, 1, 1)).cpu()
    assert wo.error_metrics(yh, wo.direct_conv_f64(x.half(), w.half(), padding=1))["E_B"] < 2e-2


@pytest.mark.parametrize("chain", [False, True])
@pytest.mark.parametrize("block", [2, 4])
def test_matrix_conv_routes(chain, block):
    from pytorch_winoconv_b200 import matrix_conv
    x = seeded((2, 16, 13, 12), 14)
    w = wo.kaiming_normal((8, 16, 3, 3), 15)
    b = seeded((8,), 16)
    o = wo.direct_conv_f64(x, w, padding=1) + b.double().view(1, -1, 1, 1)
    matrix_conv.USE_SPLIT_CHAIN = chain
    try:
        y32 = matrix_conv.conv32(x.cuda(), w.cuda(), bias=b.cuda(), padding=(1, 1), output_block=block).cpu()
        y16 = matrix_conv.conv16(x.cuda(), w.cuda(), bias=b.cuda(), padding=(1, 1), output_block=block).cpu()
    finally:
        matrix_conv.USE_SPLIT_CHAIN = False
    assert y32.dtype == torch.float32 and y16.dtype == torch.float32
    assert wo.error_metrics(y32, o)["E_B"] < 1e-3
    assert wo.error_metrics(y16, o)["E_B"] < 2e-2


def test_matrix_conv_output_block_6_is_fp32_only():
    from pytorch_winoconv_b200 import capi, matrix_conv
    x = seeded((2, 16, 13, 12), 14)
    w = wo.kaiming_normal((8, 16, 3, 3), 15)
    o = wo.direct_conv_f64(x, w, padding=1)
    y32 = matrix_conv.conv32(x.cuda(), w.cuda(), padding=(1, 1), output_block=6).cpu()
    assert wo.error_metrics(y32, o)["E_B"] < 1e-3
    with pytest.raises(capi.WinoconvError):      # F(6x6,3x3) over fp16 operands cannot hold the 2e-2 bound: refused, not approximated
        matrix_conv.conv16(x.cuda(), w.cuda(), padding=(1, 1), output_block=6)


def test_matrix_conv3d_and_nd_and_dwm_convnd():
    from pytorch_winoconv_b200 import dwm_convnd, matrix_conv3d, matrix_convnd
    x = seeded((1, 8, 6, 7, 8), 17)
    w = wo.kaiming_normal((8, 8, 3, 3, 3), 18)
    y = matrix_conv3d.conv32(x.cuda(), w.cuda(), padding=(1, 1, 1)).cpu()
    assert wo.error_metrics(y, wo.direct_conv_f64(x, w, padding=1))["E_B"] < 1e-3
    matrix_conv3d.USE_SPLIT_CHAIN = True
    try:
        y = matrix_conv3d.conv32(x.cuda(), w.cuda(), padding=(1, 1, 1)).cpu()
    finally:
        matrix_conv3d.USE_SPLIT_CHAIN = False
    assert wo.error_metrics(y, wo.direct_conv_f64(x, w, padding=1))["E_B"] < 1e-3
    # convnd.py:156-195: single tile [1,1,6^n] * kernel 5^n, n = 1..3
    for n in (1, 2, 3):
        xt = seeded((1, 8) + (6,) * n, 19 + n)
        wt = seeded((8, 8) + (5,) * n, 29 + n)
        o = wo.direct_conv_f64(xt, wt)
        y = dwm_convnd.conv32(xt.cuda(), wt.cuda(), n).cpu()
        assert tuple(y.shape) == (1, 8) + (2,) * n
        assert wo.error_metrics(y, o)["E_B"] < 1e-3
    # tile algebra on pre-split tiles equals the oracle's restatement of base_conv32
    tiles = seeded((10, 8, 4, 4), 40)
    wk = seeded((8, 8, 3, 3), 41)
    got = matrix_convnd.base_conv32(tiles.cuda(), wk.cuda(), False, 2, [3, 3], 2).cpu()
    assert (got.double() - wo.base_conv(tiles.double(), wk.double(), [2, 2])).abs().max().item() < 1e-4
    # n > 3 (matrix_convnd.py:110-153, convnd.py:156-195): 4-D and 5-D tiles against the sliding-window float64 oracle
    # and against the oracle's restatement of the reference's n-D tile algebra
    for n, r in ((4, 3), (5, 3), (4, 5)):
        xt = seeded((3, 8) + (r + 1,) * n, 50 + n)
        wt = seeded((8, 8) + (r,) * n, 60 + n + r) * (1.0 / (8 * r ** n)) ** 0.5
        o = torch.from_numpy(wo.direct_conv_numpy(xt.numpy(), wt.numpy()))
        y = (dwm_convnd.conv32 if r > 3 else matrix_convnd.conv32)(xt.cuda(), wt.cuda(), n).cpu()
        assert tuple(y.shape) == (3, 8) + (2,) * n
        assert wo.error_metrics(y, o)["E_B"] < 1e-3
        if r == 3:
            assert wo.error_metrics(y, wo.base_conv(xt.double(), wt.double(), [2] * n))["E_B"] < 1e-3


def test_wino_class():
    from pytorch_winoconv_b200.WinoConv import Wino
    x = seeded((1, 8, 10, 10), 50)
    w = wo.kaiming_normal((8, 8, 3, 3), 51)
    y = Wino().conv32(x.cuda(), w.cuda(), padding=(1, 1)).cpu()
    assert wo.error_metrics(y, wo.direct_conv_f64(x, w, padding=1))["E_B"] < 1e-3
