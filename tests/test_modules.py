"""torch.nn modules over the engine (the caller layer, reference conv.py:305-340,446-481): constructor and
state_dict compatibility and argument checks on CPU; parity, the filter-transform cache, channels-last
zero-copy I/O and the fused epilogue on the GPU."""
import pytest
import torch

from oracle import winograd_oracle as wo
from pytorch_winoconv_b200 import conv as wconv


def test_constructor_and_state_dict_match_torch():
    ref = torch.nn.Conv2d(8, 12, 5, stride=1, padding=2, bias=True)
    m = wconv.Conv2d(8, 12, 5, stride=1, padding=2, bias=True)
    assert set(m.state_dict()) == set(ref.state_dict())
    m.load_state_dict(ref.state_dict())
    assert torch.equal(m.weight, ref.weight) and torch.equal(m.bias, ref.bias)
    m3 = wconv.Conv3d(4, 6, 3, padding=1, bias=False)
    assert m3.bias is None and tuple(m3.weight.shape) == (6, 4, 3, 3, 3)
    assert "compute_dtype" in repr(m)


def test_unsupported_arguments_raise():
    with pytest.raises(NotImplementedError):
        wconv.Conv2d(4, 4, 3, dilation=2)
    with pytest.raises(NotImplementedError):
        wconv.Conv2d(4, 4, 3, groups=2)
    with pytest.raises(NotImplementedError):
        wconv.Conv2d(4, 4, 3, padding=1, padding_mode="reflect")
    with pytest.raises(ValueError):
        wconv.Conv2d(4, 4, 3, activation="gelu")
    with pytest.raises(ValueError):
        wconv.Conv2d(4, 4, 3, pool=3)
    with pytest.raises(ValueError):
        wconv.Conv3d(4, 4, 3, pool=2)          # the epilogue pool is 2-D


def test_cpu_input_is_refused_loudly():
    m = wconv.Conv2d(4, 4, 3, padding=1).eval()
    with pytest.raises(RuntimeError, match="CUDA"):
        m(torch.zeros(1, 4, 8, 8))
    with pytest.raises(ValueError):
        m(torch.zeros(4, 8, 8))


@pytest.mark.gpu
@pytest.mark.parametrize("ks,stride,pad", [(3, 1, 1), (5, 1, 2), (7, 2, 3)])
def test_conv2d_module_parity(ks, stride, pad):
    torch.manual_seed(5)
    m = wconv.Conv2d(16, 24, ks, stride=stride, padding=pad, bias=True).cuda().eval()
    x = torch.randn(3, 16, 30, 28).half()
    y = m(x.cuda())
    o = wo.direct_conv_f64(x, m.weight.detach().cpu().half(), stride=stride, padding=pad) \
        + m.bias.detach().cpu().half().double().view(1, -1, 1, 1)
    assert y.dtype == torch.float16 and tuple(y.shape) == tuple(o.shape)
    assert wo.error_metrics(y.cpu().double(), o)["E_B"] < 2e-2          # the fp16 bound of the parity tests


@pytest.mark.gpu
def test_conv3d_module_parity_and_fp32():
    torch.manual_seed(6)
    m = wconv.Conv3d(8, 8, 3, padding=1, bias=False, compute_dtype=None).cuda().eval()
    x = torch.randn(1, 8, 6, 9, 10)
    y = m(x.cuda())                                                      # fp32 in -> fp32 path
    o = wo.direct_conv_f64(x, m.weight.detach().cpu(), padding=1)
    assert y.dtype == torch.float32
    assert wo.error_metrics(y.cpu().double(), o)["E_B"] < 1e-3


@pytest.mark.gpu
def test_channels_last_io_is_zero_copy_and_cache_follows_the_weight():
    torch.manual_seed(7)
    m = wconv.Conv2d(32, 32, 3, padding=1, bias=False, activation="relu", pool=2).cuda().half().eval()
    x = torch.randn(4, 32, 16, 16, device="cuda").half().contiguous(memory_format=torch.channels_last)
    y = m(x)
    assert y.is_contiguous(memory_format=torch.channels_last) and tuple(y.shape) == (4, 32, 8, 8)
    o = torch.nn.functional.max_pool2d(torch.relu(wo.direct_conv_f64(x.cpu(), m.weight.detach().cpu(), padding=1)), 2)
    assert wo.error_metrics(y.cpu().double(), o)["E_A"] < 5e-3
    assert list(m.planned_algorithms.values()) == ["row"]
    plan = next(iter(m._plans.values()))
    u_before = plan.u.clone()
    assert m(x).data_ptr() != 0 and next(iter(m._plans.values())) is plan      # second call: same plan, same U
    assert torch.equal(plan.u, u_before)
    with torch.no_grad():
        m.weight.mul_(2.0)                                                # in-place update bumps the version counter
    y2 = m(x)
    assert next(iter(m._plans.values())) is not plan                      # stale transforms were dropped
    assert wo.error_metrics(y2.cpu().double(), 2.0 * o)["E_A"] < 5e-3


def _grads_f64(x, w, b, gy, stride, pad, relu):
    """float64 torch.autograd.grad of F.conv2d / conv3d on the same rounded tensors."""
    xd, wd = x.double().requires_grad_(True), w.double().requires_grad_(True)
    bd = None if b is None else b.double().requires_grad_(True)
    conv = torch.nn.functional.conv2d if w.dim() == 4 else torch.nn.functional.conv3d
    y = conv(xd, wd, bd, stride=stride, padding=pad)
    if relu:
        y = torch.relu(y)
    return torch.autograd.grad(y, [xd, wd] + ([bd] if bd is not None else []), gy.double())


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [
    # n, c, k, hw, kernel, stride, pad, relu
    (4, 32, 48, 20, 3, 1, 1, False),
    (2, 16, 24, 18, 5, 1, 2, True),
    (2, 8, 16, 23, 7, 2, 3, False),          # stride 2, and (23 + 6 - 7) % 2 == 0
    (2, 8, 16, 24, 3, 2, 1, False),          # stride 2 with an input row the forward never reads
])
def test_backward_matches_float64_autograd(shape):
    n, c, k, hw, ks, stride, pad, relu = shape
    torch.manual_seed(11)
    m = wconv.Conv2d(c, k, ks, stride=stride, padding=pad, bias=True, activation="relu" if relu else None).cuda()
    x = torch.randn(n, c, hw, hw).half()
    xg = x.cuda().requires_grad_(True)
    y = m(xg)
    gy = torch.randn(y.shape, generator=torch.Generator().manual_seed(12)).half()
    y.backward(gy.cuda())
    w16, b16 = m.weight.detach().cpu().half(), m.bias.detach().cpu().half()
    gx, gw, gb = _grads_f64(x, w16, b16, gy, stride, pad, relu)
    # the ReLU mask of the engine's fp16 output can differ from the float64 one where y is within rounding of zero
    tol = 2e-2 if not relu else 4e-2
    assert wo.error_metrics(xg.grad.cpu(), gx)["E_B"] < tol
    assert wo.error_metrics(m.weight.grad.cpu(), gw)["E_B"] < tol
    assert wo.error_metrics(m.bias.grad.cpu(), gb)["E_B"] < tol


@pytest.mark.gpu
def test_data_gradient_at_the_baseline_shapes():
    """grad_x of configs[1] (3x3, 256 -> 256 at 28 x 28) and configs[2]b (5x5, 128 -> 128 at 56 x 56) against float64."""
    for n, c, k, hw, ks, pad in [(32, 256, 256, 28, 3, 1), (8, 128, 128, 56, 5, 2)]:
        torch.manual_seed(13)
        m = wconv.Conv2d(c, k, ks, padding=pad, bias=False).cuda().eval()
        x = torch.randn(n, c, hw, hw).half()
        xg = x.cuda().requires_grad_(True)
        y = m(xg)
        gy = torch.randn(y.shape, generator=torch.Generator().manual_seed(14)).half()
        (gx,) = torch.autograd.grad(y, [xg], gy.cuda())
        ref = _grads_f64(x, m.weight.detach().cpu().half(), None, gy, 1, pad, False)[0]
        assert wo.error_metrics(gx.cpu(), ref)["E_B"] < 2e-2


@pytest.mark.gpu
def test_conv3d_backward_and_pool_refusal():
    torch.manual_seed(15)
    m = wconv.Conv3d(8, 8, 3, padding=1, bias=False).cuda()
    x = torch.randn(1, 8, 6, 9, 10).half()
    xg = x.cuda().requires_grad_(True)
    y = m(xg)
    gy = torch.randn(y.shape, generator=torch.Generator().manual_seed(16)).half()
    y.backward(gy.cuda())
    gx, gw = _grads_f64(x, m.weight.detach().cpu().half(), None, gy, 1, 1, False)
    assert wo.error_metrics(xg.grad.cpu(), gx)["E_B"] < 2e-2
    assert wo.error_metrics(m.weight.grad.cpu(), gw)["E_B"] < 2e-2
    mp = wconv.Conv2d(8, 8, 3, padding=1, pool=2).cuda()
    with pytest.raises(NotImplementedError):
        mp(torch.randn(1, 8, 8, 8, device="cuda"))                        # train mode: the fused pool has no gradient
    with torch.no_grad():
        assert tuple(mp(torch.randn(1, 8, 8, 8, device="cuda")).shape) == (1, 8, 4, 4)
