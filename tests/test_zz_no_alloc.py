"""winoconv_forward_static -- the forward for callers that may not allocate device memory -- against
winoconv_forward on the same inputs.  The built-in scratch array is shared by all calls and keeps the
previous call's contents, so the check runs two different layers back to back, then the first again.
Collected last on purpose (file name), and self-contained so it also passes alone in a fresh process."""
import pytest
import torch

from oracle import winograd_oracle as wo
from pytorch_winoconv_b200 import capi, engine

pytestmark = pytest.mark.gpu

TOL = {torch.float16: 2e-2, torch.float32: 1e-3}     # the E_B bounds of tests/gpu_util.py


def _layer(seed, n, c, k, hw, ks, pad, dtype, tile_m=0, stride=1):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, hw, hw, c, generator=g).to(dtype).cuda()
    w = (torch.randn(k, c, ks, ks, generator=g) * (2.0 / (c * ks * ks)) ** 0.5).to(dtype).cuda()
    conv = engine.WinoConv(x.shape, w, stride=stride, padding=pad, tile_m=tile_m)
    conv.test_w, conv.test_stride, conv.test_pad = w, stride, pad
    return x, conv


def _both(x, conv):
    y_ref = conv(x).clone()                                    # existing entry point, caller scratch
    y = torch.full_like(y_ref, float("nan"))
    capi.forward_static(conv.desc, x.data_ptr(), conv.u.data_ptr(), None, y.data_ptr(),
                        torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert capi.read_device_error() == 0
    assert torch.isfinite(y).all()
    d = (y.double() - y_ref.double()).abs()
    rms = y_ref.double().pow(2).mean().sqrt()
    e_b = (d / torch.maximum(y_ref.double().abs(), rms)).max().item()
    assert e_b <= TOL[x.dtype], e_b
    # and against the float64 direct convolution of the same rounded inputs, so the check stands by itself
    o = wo.direct_conv_f64(x.permute(0, 3, 1, 2).cpu(), conv.test_w.cpu(), stride=conv.test_stride, padding=conv.test_pad)
    err = wo.error_metrics(y.permute(0, 3, 1, 2).cpu(), o)
    assert err["E_B"] <= TOL[x.dtype], err
    return e_b


def test_static_scratch_forward_matches_on_consecutive_calls():
    # layer A needs several passes through the 32 MiB array; layer B is a different shape and dtype
    xa, ca = _layer(1, 16, 64, 96, 56, 3, 1, torch.float16, tile_m=4)     # F(4x4,3x3): the staged flow, which needs scratch
    xb, cb = _layer(2, 2, 24, 40, 21, 5, 2, torch.float32)
    assert ca.info.algo == capi.ALGO_STAGED and cb.info.algo == capi.ALGO_STAGED
    need_a = int(ca.info.tiles) * (int(ca.info.input_ws_bytes_min) + int(ca.info.product_ws_bytes_min)) // 128
    assert need_a > capi.STATIC_SCRATCH_BYTES            # so the array is reused within one call
    errs = [_both(xa, ca), _both(xb, cb), _both(xa, ca)]
    print("forward_static vs forward, E_B:", errs)


def test_static_scratch_serves_the_single_kernel_paths():
    # the row kernel's only scratch: channel padding (3 -> 8; a row of 41 x 3 elements is not a multiple of eight, so
    # the input cannot be read as it lies) and the stride-2 phase gather (4 x 3 -> 16 channels)
    xa, ca = _layer(3, 4, 3, 32, 41, 3, 1, torch.float16)
    xb, cb = _layer(4, 4, 3, 32, 41, 7, 3, torch.float16, stride=2)
    assert ca.info.algo == capi.ALGO_ROW and cb.info.algo == capi.ALGO_ROW
    assert 0 < int(ca.info.input_ws_bytes) <= capi.STATIC_SCRATCH_BYTES
    assert 0 < int(cb.info.input_ws_bytes) <= capi.STATIC_SCRATCH_BYTES
    errs = [_both(xa, ca), _both(xb, cb), _both(xa, ca)]
    print("forward_static vs forward (row kernel), E_B:", errs)


def test_static_scratch_refuses_oversized_layers():
    # 3-D 3x3x3 with 1024 -> 1024 channels: 64 positions x (1024*2 + 1024*4) B x 128 tiles = 48 MiB > 32 MiB (512 tiles in all)
    d = capi.make_desc(ndim=3, batch=1, c_in=1024, k_out=1024, in_size=(16, 16, 16), ker_size=3, pad=1, algo=capi.ALGO_STAGED)
    with pytest.raises(capi.WinoconvError) as ei:
        capi.forward_static(d, 256, 256, None, 256)
    assert ei.value.status == capi.ERR_WORKSPACE
    assert "33554432" in str(ei.value)


def test_static_scratch_refuses_an_oversized_row_layer_and_names_the_way_out():
    # 7x7 stride-2 stem, 3 -> 64 at 225 x 225 (rows of 675 elements cannot be read as they lie), batch 96: the
    # phase-gathered copy of the input (116 x 116 x 16 channels per image) is 41 MB > 32 MiB
    d = capi.make_desc(ndim=2, batch=96, c_in=3, k_out=64, in_size=(225, 225), ker_size=7, stride=2, pad=3)
    assert capi.plan(d).algo == capi.ALGO_ROW and capi.plan(d).input_ws_bytes > capi.STATIC_SCRATCH_BYTES
    with pytest.raises(capi.WinoconvError) as ei:
        capi.forward_static(d, 256, 256, None, 256)
    assert ei.value.status == capi.ERR_WORKSPACE
    assert "WINOCONV_ALGO_FUSED" in str(ei.value) and "33554432" in str(ei.value)
