"""3-D twin of :mod:`matrix_conv` with the reference's names (``matrix_conv3d.py:42-290``)."""
import torch

from . import matrix_convnd
from .engine import conv_forward
from .Split_and_Concat import wino_concat, wino_split

USE_SPLIT_CHAIN = False
A, G, B = matrix_convnd.A, matrix_convnd.G, matrix_convnd.B
_ND = 3


def matrix_alloc(m, r):
    return matrix_convnd.matrix_alloc(m, r)


def base_conv32(input, kernel, fp16, m, r):
    return matrix_convnd.base_conv32(input, kernel, fp16, m, r, _ND)


def conv(input, kernel, output_block, stride, fp16=False):
    ks = [int(s) for s in kernel.shape[2:]]
    out_shape = [int(s) - k + 1 for s, k in zip(input.shape[2:], ks)]
    tiles = wino_split(input, list(kernel.shape), output_block)
    out = base_conv32(tiles, kernel, fp16, [output_block] * _ND, ks)
    return wino_concat(out.float(), out_shape, output_block)


def _run(input, kernel, bias, stride, padding, output_block, fp16):
    if not input.is_cuda:
        input = input.cuda()
    kernel = kernel.to(input.device)
    strides = (stride,) * _ND if isinstance(stride, int) else tuple(stride)
    pads = (padding,) * _ND if isinstance(padding, int) else tuple(padding)
    dt = torch.float16 if fp16 else torch.float32
    x, w = input.to(dt), kernel.to(dt)
    if any(pads):
        x = torch.nn.functional.pad(x, (pads[2], pads[2], pads[1], pads[1], pads[0], pads[0]))
    if USE_SPLIT_CHAIN and all(s == 1 for s in strides):
        out = conv(x.float(), w.float(), output_block, strides, fp16)
    else:
        out = conv_forward(x, w, stride=strides, padding=0, tile_m=2)
    out = out.float()
    if bias is not None:
        out = out + bias.to(out).view(1, -1, 1, 1, 1)
    return out


def conv32(input, kernel, bias=None, stride=(1, 1, 1), padding=0, groups=1, output_block=2):
    return _run(input, kernel, bias, stride, padding, output_block, False)


def conv16(input, kernel, bias=None, stride=(1, 1, 1), padding=0, groups=1, output_block=2):
    return _run(input, kernel, bias, stride, padding, output_block, True)
