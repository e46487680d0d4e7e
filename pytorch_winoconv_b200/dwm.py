"""``dwm2d`` / ``dwm3d`` with the reference's signatures (``dwm.py:5-40``), on the engine's DWM op.

Same call pattern as the reference -- pad, permute to channels last, call ``DWM`` with
caller-allocated output and scratch, permute back, add bias -- with its gaps closed: integer
padding is honoured (the reference pads only for tuples, ``dwm.py:26-28``), ``stride`` may be 1
or 2 (the reference ignores the argument and its op exits on stride 2,
``src/winograd_conv.cpp:122-126``), half / bfloat16 tensors run natively (the reference binds
float only, ``pybind/bind.cpp:23-24``), no per-call prints or device synchronisations
(``dwm.py:44-107``), and scratch is ``torch.empty`` rather than ``torch.zeros``.
``groups`` is accepted and ignored, as in the reference.
"""
import torch

from . import capi
from ._backend import load as _load


def _pad_tuple(padding, n):
    if isinstance(padding, int):
        return (padding,) * n
    padding = tuple(int(p) for p in padding)
    if len(padding) != n:
        raise ValueError(f"padding must have {n} entries")
    return padding


def _stride_int(stride, n):
    if isinstance(stride, int):
        return stride
    stride = tuple(int(s) for s in stride)
    if len(set(stride)) != 1 or len(stride) != n:
        raise ValueError("dwm takes one stride for all dimensions (1 or 2)")
    return stride[0]


def _dwm(x, w, stride, nd):
    """x [B,C,*sp] (already padded), w [K,C,*k] -> [B,K,*out] through the native DWM op."""
    if not x.is_cuda:
        raise RuntimeError("dwm needs CUDA tensors: the engine has no CPU path")
    w = w.to(device=x.device, dtype=x.dtype)
    sp = [int(s) for s in x.shape[2:]]
    ks = [int(s) for s in w.shape[2:]]
    B, K = int(x.shape[0]), int(w.shape[0])
    out_sp = [(s - k) // stride + 1 for s, k in zip(sp, ks)]
    if nd == 2:
        xl = x.unsqueeze(2).permute(0, 2, 3, 4, 1).contiguous()
        wl = w.unsqueeze(2).permute(2, 3, 4, 1, 0).contiguous()
        out = torch.empty(B, 1, out_sp[0], out_sp[1], K, dtype=x.dtype, device=x.device)
    else:
        xl = x.permute(0, 2, 3, 4, 1).contiguous()
        wl = w.permute(2, 3, 4, 1, 0).contiguous()
        out = torch.empty(B, *out_sp, K, dtype=x.dtype, device=x.device)
    empty = torch.empty(0, dtype=x.dtype, device=x.device)       # scratch comes from the op itself
    ptrs = torch.empty(0, dtype=torch.long, device=x.device)
    _load().DWM(xl, wl, out, int(stride), empty, empty, empty, ptrs)
    if nd == 2:
        return out[:, 0].permute(0, 3, 1, 2).contiguous()
    return out.permute(0, 4, 1, 2, 3).contiguous()


def dwm2d_(x, w, stride=1):
    return _dwm(x, w, stride, 2)


def dwm3d_(x, w, stride=1):
    return _dwm(x, w, stride, 3)


def dwm2d(input, kernel, bias=None, stride=(1, 1), padding=0, groups=1):
    ph, pw = _pad_tuple(padding, 2)
    if ph or pw:
        input = torch.nn.functional.pad(input, (pw, pw, ph, ph))
    out = dwm2d_(input, kernel, _stride_int(stride, 2))
    if bias is not None:
        out = out + bias.type_as(out).view(1, -1, 1, 1)
    return out


def dwm3d(input, kernel, bias=None, stride=(1, 1, 1), padding=0, groups=1):
    pd, ph, pw = _pad_tuple(padding, 3)
    if pd or ph or pw:
        input = torch.nn.functional.pad(input, (pw, pw, ph, ph, pd, pd))
    out = dwm3d_(input, kernel, _stride_int(stride, 3))
    if bias is not None:
        out = out + bias.type_as(out).view(1, -1, 1, 1, 1)
    return out
