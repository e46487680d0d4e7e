"""``wino_split`` / ``wino_concat`` with the reference's signatures and tile arithmetic
(``Split_and_Concat.py:4-82``), running the engine's WinoSplit / WinoConcat kernels.

Differences from the reference, all supersets: the window stride equals ``output_block_size``
(the reference's kernels hard-code 2, ``src/split_and_concat_kernels.cu:20-22,87-88``), the tile
count is ``ceil(outputs / block)`` written as ``(H + m - 1 - bH) // m + 1`` (the reference's
``(H + 1 - bH) / m + 1`` is the m = 2 case, ``Split_and_Concat.py:24-26,40-41``), and the results
stay on the input's device instead of a bare ``.cuda()``.
"""
import torch

from ._backend import load as _load


def wino_split(a, w_shape, output_block_size):
    m = int(output_block_size)
    a = a.float()
    if len(w_shape) == 5:
        B, C, D, H, W = (int(s) for s in a.shape)
        bD, bH, bW = (int(w_shape[i]) + m - 1 for i in (2, 3, 4))
        nD = (D + m - 1 - bD) // m + 1
        nH = (H + m - 1 - bH) // m + 1
        nW = (W + m - 1 - bW) // m + 1
        out = torch.empty(B * nD * nH * nW, C, bD, bH, bW, dtype=torch.float32, device=a.device)
        a = a.permute(0, 2, 3, 4, 1).contiguous()
        _load().WinoSplit(a, out, bD, bH, bW, m, nD, nH, nW, False)
    else:
        B, C, H, W = (int(s) for s in a.shape)
        bH, bW = int(w_shape[2]) + m - 1, int(w_shape[3]) + m - 1
        nH = (H + m - 1 - bH) // m + 1
        nW = (W + m - 1 - bW) // m + 1
        out = torch.empty(B * nH * nW, C, bH, bW, dtype=torch.float32, device=a.device)
        a = a.permute(0, 2, 3, 1).contiguous()
        _load().WinoSplit(a, out, 0, bH, bW, m, 0, nH, nW, True)
    return out


def wino_concat(a, output_size, output_block_size):
    m = int(output_block_size)
    a = a.float().contiguous()
    N, K = int(a.shape[0]), int(a.shape[1])
    if len(output_size) == 3:
        oD, oH, oW = (int(s) for s in output_size)
        nD, nH, nW = (int((o + m - 1) / m) for o in (oD, oH, oW))
        B = int(N / (nD * nH * nW))
        out = torch.empty(B, oD, oH, oW, K, dtype=torch.float32, device=a.device)
        _load().WinoConcat(a, out, m, False)
        out = out.permute(0, 4, 1, 2, 3).contiguous()
    else:
        oH, oW = (int(s) for s in output_size)
        nH, nW = (int((o + m - 1) / m) for o in (oH, oW))
        B = int(N / (nH * nW))
        out = torch.empty(B, oH, oW, K, dtype=torch.float32, device=a.device)
        _load().WinoConcat(a, out, m, True)
        out = out.permute(0, 3, 1, 2).contiguous()
    return out
