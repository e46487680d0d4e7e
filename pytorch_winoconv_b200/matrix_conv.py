"""2-D torch-level Winograd route with the reference's names (``matrix_conv.py:42-254``).

``conv`` keeps the reference's three steps -- ``wino_split`` -> ``base_conv32`` -> ``wino_concat``
-- each now a kernel of this engine.  ``conv32`` / ``conv16`` go straight to the fused forward
(no tile tensor in HBM) unless ``USE_SPLIT_CHAIN`` is set.  ``output_block`` may be 2 or 4
(the reference has no F(4,3) table entry and exits, ``matrix_conv.py:50-52``).  Stride 2 runs on
the engine too (the reference falls back to cuDNN, ``matrix_conv.py:71-75,93-95``).
"""
import torch

from . import matrix_convnd
from .engine import conv_forward
from .Split_and_Concat import wino_concat, wino_split

USE_SPLIT_CHAIN = False
A, G, B = matrix_convnd.A, matrix_convnd.G, matrix_convnd.B
_ND = 2


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


def _pad(input, padding):
    pads = (padding,) * _ND if isinstance(padding, int) else tuple(padding)
    if any(pads):
        spec = []
        for p in reversed(pads):
            spec += [p, p]
        input = torch.nn.functional.pad(input, spec)
    return input


def _run(input, kernel, bias, stride, padding, output_block, fp16):
    if not input.is_cuda:
        input = input.cuda()
    kernel = kernel.to(input.device)
    strides = (stride,) * _ND if isinstance(stride, int) else tuple(stride)
    dt = torch.float16 if fp16 else torch.float32
    x, w = _pad(input, padding).to(dt), kernel.to(dt)
    if USE_SPLIT_CHAIN and all(s == 1 for s in strides):
        out = conv(x.float(), w.float(), output_block, strides, fp16)
    else:
        ks = tuple(int(s) for s in kernel.shape[2:])
        tile_m = output_block if (output_block == 2 or (ks == (3, 3) and all(s == 1 for s in strides))) else 2
        out = conv_forward(x, w, stride=strides, padding=0, tile_m=tile_m)
    out = out.float()
    if bias is not None:
        out = out + bias.to(out).view(1, -1, *([1] * _ND))
    return out


def conv32(input, kernel, bias=None, stride=(1, 1), padding=0, groups=1, output_block=2):
    return _run(input, kernel, bias, stride, padding, output_block, False)


def conv16(input, kernel, bias=None, stride=(1, 1), padding=0, groups=1, output_block=2):
    return _run(input, kernel, bias, stride, padding, output_block, True)
