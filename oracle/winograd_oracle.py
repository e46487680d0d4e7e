"""CPU oracle for the Winograd / DWM forward-convolution path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product (``pytorch_winoconv_b200``) imports this module.  It is used by
``tests/``, by ``__graft_entry__.smoke()`` and by the ``cpu_baseline`` / ``--impl reference``
legs of ``bench.py`` as the checker and as the timed CPU restatement of the reference.

Two things live here:

1. The float64 direct-convolution oracle every result is compared with -- the same yardstick the
   reference uses in its own print-only checks (``example.py:104,115``: ``F.conv2d`` /
   ``F.conv3d`` on ``.double()`` tensors).  ``direct_conv_numpy`` is an independent sliding
   window restatement used to cross-check torch on small cases.

2. A CPU restatement of the reference's torch-level Winograd algebra and of its DWM
   decomposition, so that "the reference's own error" can be reported on the same inputs and
   the reference path can be timed on host cores:

   * tile split / concat        after ``src/split_and_concat_kernels.cu:77-129`` (overlapping
                                windows, tile stride = output block, zero fill, edge mask) and
                                ``Split_and_Concat.py:28-48,68-81`` (tile counts);
   * transforms + batched GEMM  after ``matrix_convnd.py:110-153`` (``base_conv32``: G g G^T,
                                B^T d B, one matmul per Winograd position, A^T m A), with the
                                output block selectable (the reference hard-codes 2,
                                ``matrix_convnd.py:54-57``);
   * fp16 emulation             after ``matrix_conv.py:127-143`` (tiles, weights and matrices
                                cast to half, every product rounded in half);
   * DWM piece rule             after ``src/base_conv_launchers.h:58-388`` (cut each kernel
                                extent at multiples of 3, remainder last, 4 -> 2+2) and
                                ``dwm_convnd.py:10-35`` (input window shifted by the piece start,
                                partial outputs summed);
   * stride-2 polyphase         the scheme the reference scaffolds but never finishes
                                (``src/winograd_conv.cpp:45-51,61-68``; LUT entries 4x4, 4x3, 3x4
                                at ``base_conv_launchers.h:68-94``).

Parity status: the reference holds no golden vectors (it has no test suite), so results are
pinned (a) against outputs of the reference's own ``matrix_convnd.conv`` and ``wincnn``
generated in the build container and committed under ``tests/golden/`` (see
``tests/golden/make_golden.py``) and (b) against the float64 direct convolution.
"""
from __future__ import annotations

import itertools
import math
from typing import List, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from pytorch_winoconv_b200 import cooktoom


# --------------------------------------------------------------------------------------
# float64 direct convolution
# --------------------------------------------------------------------------------------
def direct_conv_f64(x: torch.Tensor, w: torch.Tensor, stride=1, padding=0) -> torch.Tensor:
    """float64 direct convolution on CPU (example.py:104,115). x: [N,C,*sp], w: [K,C,*k]."""
    nd = x.dim() - 2
    xd, wd = x.detach().cpu().double(), w.detach().cpu().double()
    fn = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[nd]
    return fn(xd, wd, stride=stride, padding=padding)


def direct_conv_numpy(x: np.ndarray, w: np.ndarray, stride=1, padding=0) -> np.ndarray:
    """Independent sliding-window float64 correlation (2-D or 3-D, small shapes only)."""
    nd = x.ndim - 2
    stride = (stride,) * nd if isinstance(stride, int) else tuple(stride)
    padding = (padding,) * nd if isinstance(padding, int) else tuple(padding)
    x = np.pad(x.astype(np.float64), [(0, 0), (0, 0)] + [(p, p) for p in padding])
    w = w.astype(np.float64)
    ks = w.shape[2:]
    outs = [(x.shape[2 + i] - ks[i]) // stride[i] + 1 for i in range(nd)]
    y = np.zeros((x.shape[0], w.shape[0]) + tuple(outs))
    for taps in itertools.product(*[range(k) for k in ks]):
        sl = tuple(slice(taps[i], taps[i] + stride[i] * (outs[i] - 1) + 1, stride[i]) for i in range(nd))
        xs = x[(slice(None), slice(None)) + sl]                  # [N, C, *out]
        wt = w[(slice(None), slice(None)) + taps]                # [K, C]
        y += np.einsum('nc...,kc->nk...', xs, wt)
    return y


# --------------------------------------------------------------------------------------
# error metrics
# --------------------------------------------------------------------------------------
def error_metrics(y: torch.Tensor, oracle: torch.Tensor, percentile: bool = False) -> dict:
    """E_B gates: max |y-o| / max(|o|, rms(o)).  E_A = max|d|/max|o|, E_C = mean(|d|/|o|)
    (the quantity the reference prints, example.py:105-108; taken over the non-zero oracle values, since
    a ReLU output has exact zeros).  ``percentile`` adds P999, the 99.9th percentile of the E_B ratio."""
    yd, od = y.detach().cpu().double(), oracle.detach().cpu().double()
    d = (yd - od).abs()
    rms = od.pow(2).mean().sqrt().clamp_min(1e-300)
    ratio = d / torch.maximum(od.abs(), rms)
    e_b = ratio.max().item()
    e_a = (d.max() / od.abs().max().clamp_min(1e-300)).item()
    nz = od != 0
    e_c = (d[nz] / od[nz].abs()).mean().item() if bool(nz.any()) else 0.0
    out = {"E_B": e_b, "E_A": e_a, "E_C": e_c}
    if percentile:
        flat = ratio.flatten()
        kth = max(1, int(math.ceil(0.999 * flat.numel())))
        out["P999"] = torch.kthvalue(flat, kth).values.item()
    return out


# --------------------------------------------------------------------------------------
# tile split / concat (split_and_concat_kernels.cu:77-129, generalised to any output block)
# --------------------------------------------------------------------------------------
def tile_counts(in_sizes: Sequence[int], r: Sequence[int], m: Sequence[int]) -> List[int]:
    """Tiles per dim for a VALID op: ceil(out / m) (Split_and_Concat.py:40-41 for m = 2)."""
    return [-(-(s - k + 1) // mm) for s, k, mm in zip(in_sizes, r, m)]


def wino_split_cpu(x: torch.Tensor, r: Sequence[int], m: Sequence[int]) -> torch.Tensor:
    """[N,C,*sp] -> [N*prod(tiles), C, *alpha]; windows start at m*t, zero filled past the edge."""
    nd = x.dim() - 2
    alpha = [mm + k - 1 for mm, k in zip(m, r)]
    nt = tile_counts(x.shape[2:], r, m)
    need = [mm * (t - 1) + a for mm, t, a in zip(m, nt, alpha)]
    padspec = []
    for i in reversed(range(nd)):
        padspec += [0, max(0, need[i] - x.shape[2 + i])]
    xp = F.pad(x, padspec)
    t = xp
    for i in range(nd):
        t = t.unfold(2 + i, alpha[i], m[i])                      # [N,C,t0..,a0..]
    # -> [N, t0..t(nd-1), C, a0..]
    perm = [0] + list(range(2, 2 + nd)) + [1] + list(range(2 + nd, 2 + 2 * nd))
    t = t.permute(perm).contiguous()
    return t.reshape([-1, x.shape[1]] + alpha)


def wino_concat_cpu(tiles: torch.Tensor, out_sizes: Sequence[int], m: Sequence[int], batch: int) -> torch.Tensor:
    """[N*prod(tiles), K, *m] -> [N,K,*out]; the last tile of an odd extent is masked."""
    nd = len(out_sizes)
    nt = [-(-o // mm) for o, mm in zip(out_sizes, m)]
    k = tiles.shape[1]
    t = tiles.reshape([batch] + nt + [k] + list(m))
    perm = [0, 1 + nd]
    for i in range(nd):
        perm += [1 + i, 2 + nd + i]
    t = t.permute(perm).contiguous().reshape([batch, k] + [n * mm for n, mm in zip(nt, m)])
    sl = (slice(None), slice(None)) + tuple(slice(0, o) for o in out_sizes)
    return t[sl].contiguous()


# --------------------------------------------------------------------------------------
# Winograd tile algebra (matrix_convnd.py:110-153)
# --------------------------------------------------------------------------------------
def _apply(t: torch.Tensor, mat: torch.Tensor, axis: int) -> torch.Tensor:
    """Multiply ``mat`` [p,q] into axis ``axis`` (length q) of t."""
    t = t.movedim(axis, -1)
    t = t @ mat.transpose(0, 1)
    return t.movedim(-1, axis)


def base_conv(tiles: torch.Tensor, kernel: torch.Tensor, m: Sequence[int], fp16: bool = False) -> torch.Tensor:
    """tiles [T,C,*alpha], kernel [K,C,*r] -> [T,K,*m].

    fp16=True rounds tiles, weights, matrices and every intermediate to half the way the
    reference's conv16 does (matrix_conv.py:127-143); half matmuls are evaluated through float
    and rounded, since CPU half matmul is what the reference would get from cuBLAS Hgemm.
    """
    nd = tiles.dim() - 2
    r = list(kernel.shape[2:])
    mats = [cooktoom.reference_table(mm, rr) for mm, rr in zip(m, r)]
    dt = tiles.dtype

    def rnd(t):
        return t.half().to(dt) if fp16 else t

    tiles, kernel = rnd(tiles), rnd(kernel)
    u, v = kernel, tiles
    for i in range(nd):
        at, g, bt = (rnd(torch.from_numpy(a).to(dt)) for a in mats[i])
        u = rnd(_apply(u, g, 2 + i))
        v = rnd(_apply(v, bt, 2 + i))
    n_tiles, c = tiles.shape[0], tiles.shape[1]
    k = kernel.shape[0]
    pos = u.shape[2:].numel()
    u = u.reshape(k, c, pos).permute(2, 0, 1)                    # [pos, K, C]
    v = v.reshape(n_tiles, c, pos).permute(2, 1, 0)              # [pos, C, T]
    prod = rnd(torch.matmul(u, v))                               # [pos, K, T]
    alpha = [mm + rr - 1 for mm, rr in zip(m, r)]
    prod = prod.permute(2, 1, 0).reshape([n_tiles, k] + alpha)
    for i in range(nd):
        at = rnd(torch.from_numpy(mats[i][0]).to(dt))
        prod = rnd(_apply(prod, at, 2 + i))
    return prod


# --------------------------------------------------------------------------------------
# DWM piece rule and stride-2 polyphase
# --------------------------------------------------------------------------------------
def dwm_cuts(k: int) -> List[Tuple[int, int]]:
    """Per-dimension pieces (start, length) of a k-tap kernel (base_conv_launchers.h:58-388)."""
    if k <= 3:
        return [(0, k)]
    if k == 4:
        return [(0, 2), (2, 2)]
    cuts, s = [], 0
    while s < k:
        cuts.append((s, min(3, k - s)))
        s += 3
    return cuts


def dwm_pieces(ksize: Sequence[int], stride: Sequence[int]):
    """All pieces of a kernel: list of (phase, start, length) triples per dimension."""
    per_dim = []
    for k, s in zip(ksize, stride):
        opts = []
        for phase in range(s):
            taps = len(range(phase, k, s))
            if taps == 0:
                continue
            for st, ln in dwm_cuts(taps):
                opts.append((phase, st, ln))
        per_dim.append(opts)
    return list(itertools.product(*per_dim))


def choose_m(ksize: Sequence[int], stride: Sequence[int], tile_m: int = 2) -> List[int]:
    """Output block per dim: 1 where the kernel extent is 1 and stride 1 (a 2-D conv carried
    with depth 1 needs no dummy depth transform), else ``tile_m``."""
    return [1 if (k == 1 and s == 1) else tile_m for k, s in zip(ksize, stride)]


def winograd_conv_cpu(x: torch.Tensor, w: torch.Tensor, stride=1, padding=0, tile_m: int = 2,
                      fp16: bool = False, dtype=torch.float32) -> torch.Tensor:
    """Reference-style Winograd / DWM forward on CPU: pad -> (polyphase) -> pieces ->
    split -> tile algebra -> concat -> sum.  x [N,C,*sp], w [K,C,*k]; returns [N,K,*out]."""
    nd = x.dim() - 2
    stride = [stride] * nd if isinstance(stride, int) else list(stride)
    padding = [padding] * nd if isinstance(padding, int) else list(padding)
    x = x.detach().cpu().to(dtype)
    w = w.detach().cpu().to(dtype)
    padspec = []
    for p in reversed(padding):
        padspec += [p, p]
    xp = F.pad(x, padspec)
    ks = list(w.shape[2:])
    outs = [(xp.shape[2 + i] - ks[i]) // stride[i] + 1 for i in range(nd)]
    m = [tile_m] * nd
    nt = [-(-o // mm) for o, mm in zip(outs, m)]
    y = None
    for piece in dwm_pieces(ks, stride):
        w_idx = [slice(None), slice(None)]
        x_idx = [slice(None), slice(None)]
        r = []
        for i, (phase, st, ln) in enumerate(piece):
            w_idx.append(slice(phase + stride[i] * st, phase + stride[i] * (st + ln - 1) + 1, stride[i]))
            x_idx.append(slice(phase + stride[i] * st, None, stride[i]))
            r.append(ln)
        wp = w[tuple(w_idx)]
        xs = xp[tuple(x_idx)]
        # exactly the window the piece's tiles cover; zero filled beyond the image
        need = [mm * (t - 1) + mm + rr - 1 for mm, t, rr in zip(m, nt, r)]
        crop = (slice(None), slice(None)) + tuple(slice(0, n) for n in need)
        xs = xs[crop]
        pad2 = []
        for i in reversed(range(nd)):
            pad2 += [0, need[i] - xs.shape[2 + i]]
        xs = F.pad(xs, pad2)
        tiles = wino_split_cpu(xs, r, m)
        part = wino_concat_cpu(base_conv(tiles, wp, m, fp16), outs, m, x.shape[0])
        y = part if y is None else y + part
    return y


# --------------------------------------------------------------------------------------
# the two rearrangements the engine's single-kernel path makes (restated to pin their algebra)
# --------------------------------------------------------------------------------------
def phases_to_channels_cpu(x: torch.Tensor, w: torch.Tensor, stride, padding):
    """A stride-{1,2} convolution as a stride-1, unpadded one: y[o] = sum_t xpad[s o + t] w[t] with
    t = s a + phase becomes, per strided dimension, a sum over `phase` (carried as extra channels,
    channel = phase_index * C + c, phases ordered depth-major) and over a < ceil(k / s).
    The reference scaffolds this polyphase scheme (``src/winograd_conv.cpp:45-51,61-68`` and the 4x4,
    4x3, 3x4 parts of ``base_conv_launchers.h:68-94``) without finishing it.
    x [N,C,*sp], w [K,C,*k] -> (xs [N, P*C, *(out + k' - 1)], ws [K, P*C, *k'])."""
    nd = x.dim() - 2
    stride = [stride] * nd if isinstance(stride, int) else list(stride)
    padding = [padding] * nd if isinstance(padding, int) else list(padding)
    x = x.detach().cpu().double()
    w = w.detach().cpu().double()
    n, c = x.shape[:2]
    k_out = w.shape[0]
    ks = list(w.shape[2:])
    outs = [(x.shape[2 + i] + 2 * padding[i] - ks[i]) // stride[i] + 1 for i in range(nd)]
    k2 = [-(-ks[i] // stride[i]) for i in range(nd)]
    ext = [outs[i] + k2[i] - 1 for i in range(nd)]
    # pad on the left by `padding`, on the right up to the last element any phase touches
    padspec = []
    for i in reversed(range(nd)):
        right = stride[i] * ext[i] - padding[i] - x.shape[2 + i]
        padspec += [padding[i], max(right, 0)]
    xp = F.pad(x, padspec)
    phases = list(itertools.product(*[range(s) for s in stride]))
    xs = torch.zeros((n, len(phases) * c, *ext), dtype=torch.float64)
    ws = torch.zeros((k_out, len(phases) * c, *k2), dtype=torch.float64)
    for pi, ph in enumerate(phases):
        xi = (slice(None), slice(None)) + tuple(slice(ph[i], ph[i] + stride[i] * ext[i], stride[i]) for i in range(nd))
        xs[:, pi * c:(pi + 1) * c] = xp[xi]
        wi = (slice(None), slice(None)) + tuple(slice(ph[i], None, stride[i]) for i in range(nd))
        part = w[wi]
        dst = (slice(None), slice(pi * c, (pi + 1) * c)) + tuple(slice(0, part.shape[2 + i]) for i in range(nd))
        ws[dst] = part
    return xs, ws


def row_piece_conv_cpu(x: torch.Tensor, w: torch.Tensor, padding=0, dtype=torch.float64) -> torch.Tensor:
    """Stride-1 convolution by 1 x 3 DWM pieces, the decomposition of the engine's row kernel: along the last
    dimension every run of three taps is an F(2,3) window (zero taps where the kernel ends; the piece rule
    of ``src/base_conv_launchers.h:58-388`` cuts at multiples of 3 too), along every other dimension each
    tap is its own piece, for which F(m,1) is the identity.  All pieces share the four Winograd positions
    of a 1 x 2 output tile, so they are summed before the output transform:
        M[j] = sum_{taps, window} (B^T d)[j] * (G g)[j],   y = A^T M
    with the F(2,3) matrices of ``matrix_conv.py:12-29`` (B^T rows (1,0,-1,0), (0,1,1,0), (0,-1,1,0), (0,1,0,-1);
    G rows (1,0,0), (.5,.5,.5), (.5,-.5,.5), (0,0,1); A^T rows (1,1,1,0), (0,1,-1,-1))."""
    nd = x.dim() - 2
    padding = [padding] * nd if isinstance(padding, int) else list(padding)
    x = x.detach().cpu().to(dtype)
    w = w.detach().cpu().to(dtype)
    padspec = []
    for p in reversed(padding):
        padspec += [p, p]
    xp = F.pad(x, padspec)
    ks = list(w.shape[2:])
    outs = [xp.shape[2 + i] - ks[i] + 1 for i in range(nd)]
    n_pairs = -(-outs[-1] // 2)
    n_win = -(-ks[-1] // 3)
    bt = torch.tensor([[1, 0, -1, 0], [0, 1, 1, 0], [0, -1, 1, 0], [0, 1, 0, -1]], dtype=dtype)
    g = torch.tensor([[1, 0, 0], [.5, .5, .5], [.5, -.5, .5], [0, 0, 1]], dtype=dtype)
    at = torch.tensor([[1, 1, 1, 0], [0, 1, -1, -1]], dtype=dtype)
    # zero-extend the last dimension so every window of every column pair is inside the tensor
    need_w = 2 * n_pairs + 3 * n_win - 1
    xp = F.pad(xp, [0, max(need_w - xp.shape[-1], 0)])
    m = torch.zeros((x.shape[0], w.shape[0], *outs[:-1], n_pairs, 4), dtype=dtype)
    for taps in itertools.product(*[range(k) for k in ks[:-1]]):
        for win in range(n_win):
            gw = torch.zeros((w.shape[0], w.shape[1], 3), dtype=dtype)
            hi = min(3 * win + 3, ks[-1])
            gw[..., :hi - 3 * win] = w[(slice(None), slice(None)) + taps + (slice(3 * win, hi),)]
            u = torch.einsum("jt,kct->kcj", g, gw)                                   # [K, C, 4]
            xi = (slice(None), slice(None)) + tuple(slice(t, t + o) for t, o in zip(taps, outs[:-1]))
            rows = xp[xi]                                                            # [N, C, *outs[:-1], W]
            d = torch.stack([rows[..., 2 * q + 3 * win: 2 * q + 3 * win + 4] for q in range(n_pairs)], dim=-2)
            v = torch.einsum("ji,...qi->...qj", bt, d)                               # [N, C, ..., pairs, 4]
            m += torch.einsum("nc...qj,kcj->nk...qj", v, u)
    y = torch.einsum("oj,...qj->...qo", at, m).reshape(*m.shape[:-2], 2 * n_pairs)
    return y[..., :outs[-1]]


# --------------------------------------------------------------------------------------
# workload descriptions shared by tests and the bench
# --------------------------------------------------------------------------------------
VGG16_CHANNELS = [(3, 64), (64, 64), (64, 128), (128, 128), (128, 256), (256, 256), (256, 256),
                  (256, 512), (512, 512), (512, 512), (512, 512), (512, 512), (512, 512)]
VGG16_POOL_AFTER = (1, 3, 6, 9, 12)     # zero-based conv indices followed by a 2x2 max-pool


def kaiming_normal(shape, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    fan_in = math.prod(shape[1:])
    return torch.randn(shape, generator=g) * math.sqrt(2.0 / fan_in)


def vgg16_conv_stack_f64(x: torch.Tensor, weights: Sequence[torch.Tensor], round_to=None) -> torch.Tensor:
    """float64 VGG-16 conv stack (3x3/s1/p1 + ReLU, 2x2 max-pool after convs 2,4,7,10,13).
    ``round_to`` (e.g. torch.float16) rounds each layer's activations the way a half-precision
    engine stores them, so layer inputs match what the device path sees."""
    h = x.detach().cpu().double()
    for i, wt in enumerate(weights):
        h = F.relu(F.conv2d(h, wt.detach().cpu().double(), padding=1))
        if i in VGG16_POOL_AFTER:
            h = F.max_pool2d(h, 2)
        if round_to is not None:
            h = h.to(round_to).double()
    return h


def vgg16_winograd_cpu(x: torch.Tensor, weights: Sequence[torch.Tensor], tile_m: int = 2) -> torch.Tensor:
    """The VGG-16 conv stack evaluated the reference's way on CPU: every 3x3 convolution through
    pad -> tile split -> F(tile_m,3) algebra in fp32 -> concat (matrix_conv.py:92-135 ->
    matrix_convnd.py:110-153), then ReLU and the max-pools in torch.  This is the timed CPU
    baseline; fp16 shapes are run in fp32 here, as a CPU has no half GEMM worth timing."""
    h = x.detach().cpu().float()
    for i, wt in enumerate(weights):
        h = F.relu(winograd_conv_cpu(h, wt, padding=1, tile_m=tile_m))
        if i in VGG16_POOL_AFTER:
            h = F.max_pool2d(h, 2)
    return h
