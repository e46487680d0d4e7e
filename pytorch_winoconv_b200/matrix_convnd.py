"""n-D Winograd tile algebra with the reference's names (``matrix_convnd.py:87-153``).

``base_conv32`` takes pre-split tiles ``[T, C, *alpha]`` and a kernel ``[K, C, *r]`` and returns
``[T, K, *m]``: every tile is a VALID convolution of an alpha-sized image, so it runs on the
engine as a batch of T one-tile images.  The engine's kernels are 2-D and 3-D; for n > 3
(``matrix_convnd.py:110-153`` and ``convnd.py:43-153`` run any n in torch) the leading n - 3 dimensions are
evaluated directly -- their taps are folded into the channels, which the engine sums in its reduction, once
per leading output position -- and the last three go through the 3-D Winograd / DWM kernels.
"""
import itertools

import torch

from . import cooktoom
from .engine import WinoConv

A, G, B = {}, {}, {}
for _r in (1, 2, 3):
    A[(2, _r)], G[(2, _r)], B[(2, _r)] = cooktoom.reference_table(2, _r)
A[(4, 3)], G[(4, 3)], B[(4, 3)] = cooktoom.reference_table(4, 3)


def matrix_alloc(m, r):
    """Per-dimension (A^T, B^T, G) as float64 tensors, like matrix_convnd.py:45-66."""
    mm = [m] * len(r) if isinstance(m, int) else list(m)
    a_, b_, g_ = [], [], []
    for mi, ri in zip(mm, r):
        at, g, bt = cooktoom.reference_table(int(mi), int(ri))
        a_.append(torch.from_numpy(at)); b_.append(torch.from_numpy(bt)); g_.append(torch.from_numpy(g))
    return a_, b_, g_


def base_conv32(input, kernel, fp16, m, r, n):
    mm = int(m if isinstance(m, int) else m[0])
    if n > 3:
        return _base_conv_leading_direct(input, kernel, fp16, mm, n)
    dt = torch.float16 if fp16 else input.dtype
    x, w = input.to(dt), kernel.to(device=input.device, dtype=dt)
    if n == 1:                                   # carry 1-D as 2-D with a unit row
        x, w = x.unsqueeze(2), w.unsqueeze(2)
    nd = max(n, 2)
    xl = x.permute(0, *range(2, 2 + nd), 1).contiguous()
    conv = WinoConv(xl.shape, w, tile_m=mm)
    y = conv(xl).permute(0, nd + 1, *range(1, nd + 1))
    if n == 1:
        y = y[:, :, 0]
    return y.contiguous()


def _base_conv_leading_direct(input, kernel, fp16, mm, n):
    """n > 3: y[t, k, o_lead, o_last3] = sum over leading taps j and channels c of
    x[t, c, o_lead + j, .] * w[k, c, j, .] convolved over the last three dimensions.  The (j, c) pairs become the
    channels of one 3-D convolution per leading output position."""
    lead = n - 3
    r_lead = [int(v) for v in kernel.shape[2:2 + lead]]
    out_lead = [int(input.shape[2 + i]) - r_lead[i] + 1 for i in range(lead)]
    if min(out_lead) < 1:
        raise ValueError("kernel larger than the tile")
    t, c, k = int(input.shape[0]), int(input.shape[1]), int(kernel.shape[0])
    taps = 1
    for v in r_lead:
        taps *= v
    # w [K, C, r_lead..., r3] -> [K, (r_lead..., C), r3]
    w3 = kernel.permute(0, *range(2, 2 + lead), 1, *range(2 + lead, 2 + n)).reshape(k, taps * c, *kernel.shape[2 + lead:])
    out = None
    for o in itertools.product(*[range(v) for v in out_lead]):
        win = (slice(None), slice(None)) + tuple(slice(oi, oi + ri) for oi, ri in zip(o, r_lead))
        xs = input[win]                                              # [T, C, r_lead..., a3]
        x3 = xs.permute(0, *range(2, 2 + lead), 1, *range(2 + lead, 2 + n)).reshape(t, taps * c, *input.shape[2 + lead:])
        y3 = base_conv32(x3.contiguous(), w3.contiguous(), fp16, mm, list(kernel.shape[2 + lead:]), 3)     # [T, K, o3]
        if out is None:
            out = y3.new_empty((t, k, *out_lead, *y3.shape[2:]))
        out[(slice(None), slice(None)) + o] = y3
    return out


def conv(input, kernel, n, output_block=2, fp16=False):
    r = list(kernel.shape[2:])
    return base_conv32(input, kernel, fp16, output_block, r, n)


def conv32(input, kernel, n, output_block=2):
    return conv(input.cuda().float(), kernel.cuda().float(), n, output_block, False).float()
