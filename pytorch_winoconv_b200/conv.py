"""``torch.nn`` modules over the engine: the caller layer of the forward path.

The reference patches a copy of torch's ``conv.py`` so that ``Conv2d`` / ``Conv3d`` send large stride-1
kernels to ``dwm.dwm2d`` / ``dwm.dwm3d`` (or ``matrix_conv.conv16``) in half precision and everything
else to cuDNN (reference: ``conv.py:324-340`` and ``conv.py:465-481``).  These classes keep that
interface -- same constructor as ``torch.nn.Conv2d`` / ``Conv3d``, same parameters and ``state_dict``,
half-precision compute by default -- and run *every* supported shape on the engine: 3x3 kernels and
stride 2 included, no cuDNN branch.  What the reference pays per call and these do not:

* the filter transform: U = G g G^T is cached and recomputed only when the weight tensor changes
  (its version counter, storage, dtype or device), not on every forward;
* the layout copies of ``dwm.py:129-133,144``: an input in ``torch.channels_last`` (``channels_last_3d``)
  memory format is handed to the kernels as it lies, and the result comes back as an NCHW-shaped
  view of the channels-last buffer the kernels wrote (any other input is copied once);
* separate bias / ReLU / max-pool passes: ``activation="relu"`` and ``pool=2`` run in the
  convolution's epilogue.

Backward (the reference left only traces of one: ``include/splitstrideone/split_functions_grad.h:1-7``,
``backwardAssign`` at ``src/back/utils.cu:16``) runs on the engine's kernels too:

* data gradient: the forward engine on the flipped, transposed filter -- ``grad_x = conv(grad_y, flip(w)^T)``
  with padding ``k - 1 - p``; a stride-2 layer first spreads ``grad_y`` onto the stride grid (zeros between);
* weight gradient: one tensor-core GEMM per filter tap, ``dW[:, :, tap] = grad_y^T  x_shifted(tap)`` with the
  batch and output pixels as the reduction (``winoconv_gemm_batched``, fp32 accumulate);
* bias gradient: a sum.

A fused ReLU is differentiated through the stored output; the fused max-pool is forward only.
``groups != 1`` and dilation raise (the reference accepts ``groups`` and silently computes groups = 1).
"""
from __future__ import annotations

import itertools
import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import capi, engine

__all__ = ["Conv2d", "Conv3d"]


class _WinoConvMixin:
    """Shared forward of :class:`Conv2d` and :class:`Conv3d` (``self`` is a ``torch.nn._ConvNd``)."""

    _nd: int = 2
    MAX_CACHED_PLANS = 8      # distinct input shapes (and backward shapes) kept per module; the oldest is dropped

    def _init_wino(self, compute_dtype, activation, pool, tile_m, algo):
        if activation not in (None, "relu"):
            raise ValueError("activation must be None or 'relu'")
        if pool not in (None, 1, 2):
            raise ValueError("pool must be None or 2 (2x2 max-pool fused into the epilogue)")
        if any(int(d) != 1 for d in self.dilation):
            raise NotImplementedError("dilated convolution is not a Winograd / DWM case")
        if self.groups != 1:
            raise NotImplementedError("groups != 1 is not supported (the reference ignores the argument)")
        if self.padding_mode != "zeros" or isinstance(self.padding, str):
            raise NotImplementedError("only explicit zero padding")
        self.compute_dtype = compute_dtype
        self.activation = activation
        self.pool = 2 if pool == 2 else None
        self.tile_m = int(tile_m)
        self.algo = int(algo)
        self._plans = {}          # input shape (or backward key) -> engine.WinoConv, most recently used last
        self._weight_key = None   # identity of the weight the cached plans were built from

    # -- cache -------------------------------------------------------------------------------------
    def _current_weight_key(self, dtype, device):
        w, b = self.weight, self.bias
        return (w.data_ptr(), w._version, None if b is None else (b.data_ptr(), b._version), dtype, device)

    def _plan_for(self, in_shape_cl: Tuple[int, ...], dtype, device) -> engine.WinoConv:
        key = self._current_weight_key(dtype, device)
        if key != self._weight_key:            # the parameters changed: every cached filter transform is stale
            self._plans.clear()
            self._weight_key = key
        plan = self._plans.pop(in_shape_cl, None)
        if plan is not None:
            self._plans[in_shape_cl] = plan            # most recently used last
        if plan is None:
            w = self.weight.detach().to(device=device, dtype=dtype)
            b = None if self.bias is None else self.bias.detach().to(device=device, dtype=dtype)
            plan = engine.WinoConv(in_shape_cl, w, stride=tuple(int(s) for s in self.stride),
                                   padding=tuple(int(p) for p in self.padding), tile_m=self.tile_m, bias=b,
                                   relu=self.activation == "relu", pool2=self.pool == 2, algo=self.algo)
            self._plans[in_shape_cl] = plan
            while len(self._plans) > self.MAX_CACHED_PLANS:      # each plan holds its own transformed filter
                self._plans.pop(next(iter(self._plans)))
        return plan

    # -- forward -----------------------------------------------------------------------------------
    def forward(self, input: torch.Tensor) -> torch.Tensor:      # noqa: A002  (torch's argument name)
        nd = self._nd
        if input.dim() != nd + 2:
            raise ValueError(f"expected a {nd + 2}-D input [N, C, {'D, ' if nd == 3 else ''}H, W]")
        if not input.is_cuda:
            raise RuntimeError("the Winograd engine runs on CUDA devices only: there is no CPU or cuDNN path")
        if torch.is_grad_enabled() and (input.requires_grad or self.weight.requires_grad and self.training):
            if self.pool:
                raise NotImplementedError("the fused max-pool is forward only: use pool=None and a separate "
                                          "torch.nn.MaxPool2d where a gradient is needed")
            return _WinoConvFn.apply(self, input, self.weight, self.bias)
        return self._forward_no_grad(input)

    def _forward_no_grad(self, input: torch.Tensor) -> torch.Tensor:      # noqa: A002
        nd = self._nd
        dtype = self.compute_dtype if self.compute_dtype is not None else input.dtype
        x = input.detach()
        if x.dtype != dtype:
            x = x.to(dtype)
        # channels-last view of the input: free when the tensor already lies that way
        perm_in = (0, *range(2, 2 + nd), 1)
        x_cl = x.permute(*perm_in)
        if not x_cl.is_contiguous():
            x_cl = x_cl.contiguous()
        plan = self._plan_for(tuple(int(s) for s in x_cl.shape), dtype, x.device)
        y_cl = plan(x_cl)
        # NCHW-shaped view of the channels-last result (torch.channels_last memory format): no copy
        return y_cl.permute(0, nd + 1, *range(1, nd + 1))

    # -- backward ----------------------------------------------------------------------------------
    def _grad_input(self, gy_cl: torch.Tensor, in_shape_cl: Tuple[int, ...]) -> torch.Tensor:
        """grad_x, channels last, from the channels-last ``grad_y`` in the compute dtype."""
        nd = self._nd
        ks = tuple(int(k) for k in self.weight.shape[2:])
        st = tuple(int(v) for v in self.stride)
        pd = tuple(int(v) for v in self.padding)
        in_sp = in_shape_cl[1:-1]
        left = [k - 1 - p for k, p in zip(ks, pd)]
        if min(left) < 0:
            raise NotImplementedError("data gradient needs padding <= kernel - 1")
        extra = [(n + 2 * p - k) % s for n, p, k, s in zip(in_sp, pd, ks, st)]     # input rows the strided forward never read
        z = gy_cl
        if any(s > 1 for s in st):       # spread grad_y onto the stride grid
            full = [(o - 1) * s + 1 for o, s in zip(gy_cl.shape[1:-1], st)]
            z = gy_cl.new_zeros((gy_cl.shape[0], *full, gy_cl.shape[-1]))
            z[(slice(None), *[slice(None, None, s) for s in st], slice(None))] = gy_cl
        pad_arg = tuple(left)
        if any(extra) or any(s > 1 for s in st):
            spec = [0, 0]
            for l, e in zip(reversed(left), reversed(extra)):
                spec += [l, l + e]
            z = F.pad(z, spec).contiguous()
            pad_arg = (0,) * nd
        key = ("bwd", tuple(z.shape), z.dtype, z.device)
        wkey = self._current_weight_key(z.dtype, z.device)
        if wkey != self._weight_key:
            self._plans.clear()
            self._weight_key = wkey
        plan = self._plans.get(key)
        if plan is None:
            wt = self.weight.detach().to(device=z.device, dtype=z.dtype).flip(*range(2, 2 + nd)).transpose(0, 1).contiguous()
            plan = engine.WinoConv(tuple(z.shape), wt, stride=1, padding=pad_arg)
            self._plans[key] = plan
        gx = plan(z)
        assert tuple(gx.shape) == tuple(in_shape_cl), (gx.shape, in_shape_cl)
        return gx

    def _grad_weight(self, gy_cl: torch.Tensor, x_cl: torch.Tensor) -> torch.Tensor:
        """dW [K, C, *k] in fp32: per filter tap, grad_y^T [K, R] times the shifted input [R, C] on the engine's
        batched GEMM (R = batch x output pixels, zero-extended to a multiple of 8)."""
        nd = self._nd
        ks = tuple(int(k) for k in self.weight.shape[2:])
        st = tuple(int(v) for v in self.stride)
        pd = tuple(int(v) for v in self.padding)
        n, out_sp, k_out = int(gy_cl.shape[0]), tuple(int(v) for v in gy_cl.shape[1:-1]), int(gy_cl.shape[-1])
        c_in = int(x_cl.shape[-1])
        r = n * math.prod(out_sp)
        rp = (r + 7) // 8 * 8
        dcode = engine.dtype_code(gy_cl.dtype)
        spec = [0, 0]
        for p in reversed(pd):
            spec += [p, p]
        xp = F.pad(x_cl, spec)
        gyt = gy_cl.new_zeros((k_out, rp))
        gyt[:, :r] = gy_cl.reshape(r, k_out).t()
        xt = x_cl.new_zeros((c_in, rp))
        dw = torch.empty((k_out, c_in, *ks), dtype=torch.float32, device=gy_cl.device)
        m = torch.empty((k_out, c_in), dtype=torch.float32, device=gy_cl.device)
        stream = torch.cuda.current_stream(gy_cl.device).cuda_stream
        with torch.cuda.device(gy_cl.device):
            for tap in itertools.product(*[range(k) for k in ks]):
                win = (slice(None), *[slice(t, t + (o - 1) * s + 1, s) for t, o, s in zip(tap, out_sp, st)], slice(None))
                xt[:, :r] = xp[win].reshape(r, c_in).t()
                capi.gemm_batched(dcode, capi.F32, capi.GEMM_AUTO, 1, k_out, rp, c_in, gyt.data_ptr(), xt.data_ptr(),
                                  m.data_ptr(), stream)
                dw[(slice(None), slice(None), *tap)] = m
        return dw

    def extra_repr(self) -> str:
        s = super().extra_repr()
        s += f", compute_dtype={self.compute_dtype}"
        if self.activation:
            s += f", activation={self.activation}"
        if self.pool:
            s += f", pool={self.pool}"
        return s

    @property
    def planned_algorithms(self):
        """Algorithm the engine chose for every input shape seen so far: {shape: 'row' | 'fused' | 'staged'}."""
        names = {capi.ALGO_ROW: "row", capi.ALGO_FUSED: "fused", capi.ALGO_STAGED: "staged"}
        return {shape: names.get(int(p.info.algo), str(p.info.algo)) for shape, p in self._plans.items()}


class _WinoConvFn(torch.autograd.Function):
    """Autograd node of the module forward: every arithmetic kernel of the three gradients is the engine's."""

    @staticmethod
    def forward(ctx, module, x, weight, bias):
        y = module._forward_no_grad(x)
        ctx.module = module
        ctx.save_for_backward(x, y if module.activation == "relu" else None)
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, gy):
        module = ctx.module
        x, y = ctx.saved_tensors
        nd = module._nd
        dtype = module.compute_dtype if module.compute_dtype is not None else x.dtype
        perm_in = (0, *range(2, 2 + nd), 1)
        to_nchw = (0, nd + 1, *range(1, nd + 1))
        if y is not None:
            gy = gy * (y > 0).to(gy.dtype)
        gy_cl = gy.detach().to(dtype).permute(*perm_in).contiguous()
        x_cl = x.detach().to(dtype).permute(*perm_in).contiguous()
        gx = gw = gb = None
        if ctx.needs_input_grad[1]:
            gx = module._grad_input(gy_cl, tuple(int(v) for v in x_cl.shape)).permute(*to_nchw).to(x.dtype)
        if ctx.needs_input_grad[2]:
            gw = module._grad_weight(gy_cl, x_cl).to(module.weight.dtype)
        if ctx.has_bias and ctx.needs_input_grad[3]:
            gb = gy_cl.float().sum(dim=tuple(range(0, nd + 1))).to(module.bias.dtype)
        return None, gx, gw, gb


class Conv2d(_WinoConvMixin, nn.Conv2d):
    """``torch.nn.Conv2d`` whose forward is the Winograd / DWM engine (reference: ``conv.py:305-340``).

    Extra keyword arguments: ``compute_dtype`` (default ``torch.float16`` as upstream, ``None`` keeps the
    input's dtype; fp32 runs its products as three tf32 tensor-core products of a hi / lo split), ``activation`` (``None`` / ``"relu"``),
    ``pool`` (``None`` / ``2``), ``tile_m`` (0 auto, 2, 4; 6 for fp32 layers) and ``algo`` (``capi.ALGO_*``).
    """

    _nd = 2

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True,
                 padding_mode="zeros", device=None, dtype=None, *, compute_dtype: Optional[torch.dtype] = torch.float16,
                 activation: Optional[str] = None, pool: Optional[int] = None, tile_m: int = 0,
                 algo: int = capi.ALGO_AUTO):
        nn.Conv2d.__init__(self, in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias,
                           padding_mode, device=device, dtype=dtype)
        self._init_wino(compute_dtype, activation, pool, tile_m, algo)


class Conv3d(_WinoConvMixin, nn.Conv3d):
    """``torch.nn.Conv3d`` on the engine (reference: ``conv.py:446-481``); arguments as :class:`Conv2d`,
    except ``pool``: the epilogue's 2x2 max-pool is a 2-D operation and is refused here."""

    _nd = 3

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True,
                 padding_mode="zeros", device=None, dtype=None, *, compute_dtype: Optional[torch.dtype] = torch.float16,
                 activation: Optional[str] = None, pool: Optional[int] = None, tile_m: int = 0,
                 algo: int = capi.ALGO_AUTO):
        if pool == 2:
            raise ValueError("pool=2 is the 2-D epilogue max-pool: not available on Conv3d")
        nn.Conv3d.__init__(self, in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias,
                           padding_mode, device=device, dtype=dtype)
        self._init_wino(compute_dtype, activation, pool, tile_m, algo)
