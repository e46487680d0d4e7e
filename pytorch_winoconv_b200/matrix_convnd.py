"""n-D Winograd tile algebra with the reference's names (``matrix_convnd.py:87-153``).

``base_conv32`` takes pre-split tiles ``[T, C, *alpha]`` and a kernel ``[K, C, *r]`` and returns
``[T, K, *m]``: every tile is a VALID convolution of an alpha-sized image, so it runs on the
engine as a batch of T one-tile images.  n <= 3 (the engine's kernels); the reference's n > 3
research path is out of scope.
"""
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
    if n > 3:
        raise NotImplementedError("Winograd tiles of more than 3 dimensions are outside this engine")
    mm = int(m if isinstance(m, int) else m[0])
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


def conv(input, kernel, n, output_block=2, fp16=False):
    r = list(kernel.shape[2:])
    return base_conv32(input, kernel, fp16, output_block, r, n)


def conv32(input, kernel, n, output_block=2):
    return conv(input.cuda().float(), kernel.cuda().float(), n, output_block, False).float()
