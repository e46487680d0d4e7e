"""VGG-16 convolution stack (BASELINE config 5) on the device against the float64 stack."""
import pytest
import torch

from oracle import winograd_oracle as wo
from pytorch_winoconv_b200 import capi, engine

pytestmark = pytest.mark.gpu


def _weights(dtype):
    return [wo.kaiming_normal((k, c, 3, 3), 100 + i).to(dtype) for i, (c, k) in enumerate(wo.VGG16_CHANNELS)]


def test_vgg16_stack_matches_float64_stack():
    batch = 2
    g = torch.Generator().manual_seed(0)
    x = torch.rand(batch, 3, 224, 224, generator=g).half()
    ws = _weights(torch.float16)
    stack = engine.VGG16ConvStack([w.cuda() for w in ws], batch)
    xl = x.permute(0, 2, 3, 1).contiguous().cuda()
    y = stack(xl).permute(0, 3, 1, 2).float().cpu()
    torch.cuda.synchronize()
    assert capi.read_device_error() == 0
    assert tuple(y.shape) == (batch, 512, 7, 7)
    # errors compound over 13 layers; compare with the float64 stack fed the same fp16 inputs
    o = wo.vgg16_conv_stack_f64(x, ws)
    err = wo.error_metrics(y, o)
    print("vgg16 stack error vs float64", err)
    assert err["E_A"] < 3e-2, err
    # per-layer check: layer i of the engine against float64 on the engine's own layer input
    h = xl
    for i, conv in enumerate(stack.layers):
        out = conv(h)
        hin = h.permute(0, 3, 1, 2).cpu()
        ref = torch.relu(wo.direct_conv_f64(hin, ws[i], padding=1))
        if i in wo.VGG16_POOL_AFTER:
            ref = torch.nn.functional.max_pool2d(ref, 2)
        e = wo.error_metrics(out.permute(0, 3, 1, 2).cpu(), ref)
        assert e["E_A"] < 1e-2 and e["E_B"] <= 2e-2, (i, e)     # the fp16 gate of every other config, per layer
        h = out.clone()
    # CUDA-graph replay gives the same bits as eager
    stack.capture(xl)
    yg = stack.replay(xl).permute(0, 3, 1, 2).float().cpu()
    assert torch.equal(yg, y)
    # default path: one row-piece kernel per layer (the RGB input of layer 1 is read as it lies: no padding pass)
    assert all(c.info.algo == capi.ALGO_ROW for c in stack.layers) and stack.launches_per_call == 13


def test_vgg16_stack_staged_f43_matches_float64_stack():
    """The same stack through input transform -> GEMM -> output transform with F(4x4,3x3) tiles."""
    batch = 2
    g = torch.Generator().manual_seed(0)
    x = torch.rand(batch, 3, 224, 224, generator=g).half()
    ws = _weights(torch.float16)
    stack = engine.VGG16ConvStack([w.cuda() for w in ws], batch, tile_m=4, algo=capi.ALGO_STAGED)
    xl = x.permute(0, 2, 3, 1).contiguous().cuda()
    y = stack(xl).permute(0, 3, 1, 2).float().cpu()
    torch.cuda.synchronize()
    assert capi.read_device_error() == 0
    assert all(c.info.algo == capi.ALGO_STAGED and c.info.positions == 36 for c in stack.layers)
    assert stack.launches_per_call >= 39
    err = wo.error_metrics(y, wo.vgg16_conv_stack_f64(x, ws))
    print("vgg16 staged F(4,3) stack error vs float64", err)
    assert err["E_A"] < 3e-2, err


def test_graph_replay_survives_growth_of_the_shared_scratch_pool():
    """A captured stack holds raw scratch addresses; a larger layer run later on the same device makes the
    shared pool grow, and the replay must still read and write memory that is its own."""
    batch = 1
    x = torch.rand(batch, 3, 224, 224, generator=torch.Generator().manual_seed(3)).half()
    ws = _weights(torch.float16)
    pool = engine.ScratchPool()                      # its own pool, so earlier tests cannot have grown it already
    stack = engine.VGG16ConvStack([w.cuda() for w in ws], batch, tile_m=4, algo=capi.ALGO_STAGED, pool=pool)
    xl = x.permute(0, 2, 3, 1).contiguous().cuda()
    stack.capture(xl)
    y0 = stack.replay(xl).clone()
    before = (pool.v.data_ptr(), pool.v.numel())
    big_x = torch.randn(8, 224, 224, 64, generator=torch.Generator().manual_seed(4)).half().cuda()
    big = engine.WinoConv(big_x.shape, ws[1].cuda(), padding=1, tile_m=4, algo=capi.ALGO_STAGED, pool=pool)
    big(big_x)
    filler = [torch.full((before[1],), 0x5A, dtype=torch.uint8, device=xl.device) for _ in range(3)]   # would reuse a freed block
    assert pool.v.numel() > before[1] and any(t.data_ptr() == before[0] for t in pool._outgrown)
    y1 = stack.replay(xl)
    torch.cuda.synchronize()
    assert capi.read_device_error() == 0
    assert torch.equal(y0, y1)
    del filler
