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


@pytest.mark.gpu
def test_training_mode_call_that_needs_grad_raises():
    m = wconv.Conv2d(8, 8, 3, padding=1).cuda()
    x = torch.randn(1, 8, 8, 8, device="cuda")
    with pytest.raises(NotImplementedError):
        m(x)                                                              # train mode, grad enabled
    with torch.no_grad():
        assert tuple(m(x).shape) == (1, 8, 8, 8)
