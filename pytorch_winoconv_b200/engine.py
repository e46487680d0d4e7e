"""Torch-tensor front end of the C ABI: one :class:`WinoConv` per (shape, weight), a shared
scratch pool per device, and the VGG-16 convolution stack used by the benchmark.

PyTorch is used here for device memory and streams only; every arithmetic kernel is the
library's own (``libwinoconv_b200.so``).  Activations are channels-last: ``[N, H, W, C]`` for
2-D, ``[N, D, H, W, C]`` for 3-D -- the layout the reference's native op takes
(``dwm.py:129-133``).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import capi

_DTYPE_CODE = {torch.float32: capi.F32, torch.float16: capi.F16, torch.bfloat16: capi.BF16}
_CODE_DTYPE = {v: k for k, v in _DTYPE_CODE.items()}


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise TypeError(f"winoconv supports float32, float16 and bfloat16, not {dt}") from None


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class _NoScratch:
    """Stands in for a scratch tensor when the algorithm needs none."""
    @staticmethod
    def data_ptr():
        return None

    @staticmethod
    def numel():
        return 0


_NO_SCRATCH = _NoScratch()


class ScratchPool:
    """Grow-only V / M scratch per device, shared by every WinoConv on that device.

    Kernels of consecutive layers run on one stream, so sharing is safe; callers using several
    streams on one device should give each its own pool (``WinoConv(..., pool=ScratchPool())``).

    A block that is outgrown is kept, not freed: a CUDA graph captured earlier holds its raw address
    (``VGG16ConvStack.capture``), and handing the block back to the caching allocator would let a later
    tensor land on memory the graph still reads and writes on replay.
    """
    _default: Dict[int, "ScratchPool"] = {}

    def __init__(self):
        self.v: Optional[torch.Tensor] = None
        self.m: Optional[torch.Tensor] = None
        self._outgrown: List[torch.Tensor] = []

    @classmethod
    def default(cls, device: torch.device) -> "ScratchPool":
        idx = device.index if device.index is not None else torch.cuda.current_device()
        return cls._default.setdefault(idx, cls())

    def get(self, device, v_bytes: int, m_bytes: int) -> Tuple[torch.Tensor, torch.Tensor]:
        if self.v is None or self.v.numel() < v_bytes or self.v.device != device:
            if self.v is not None:
                self._outgrown.append(self.v)
            self.v = torch.empty(v_bytes, dtype=torch.uint8, device=device)
        if self.m is None or self.m.numel() < m_bytes or self.m.device != device:
            if self.m is not None:
                self._outgrown.append(self.m)
            self.m = torch.empty(m_bytes, dtype=torch.uint8, device=device)
        return self.v, self.m


class WinoConv:
    """A planned forward convolution with its transformed filter resident on the device.

    weight: ``[K, C, (kD,) kH, kW]`` (torch order).  ``in_shape`` is the channels-last input
    shape.  ``tile_m``: 0 auto (2-wide tiles where a single-kernel path takes the layer -- 16-bit layers, except
    3x3 stride-1 layers of >= 512 -> >= 512 channels with >= 4096 exactly-covering 4-wide tiles, which run as staged
    F(4x4,3x3) -- else F(4x4,3x3) for 2-D 3x3 stride 1 and F(2,r) pieces otherwise), 2, 4, or 6 (F(6x6,3x3), fp32 layers only).
    """

    def __init__(self, in_shape: Sequence[int], weight: torch.Tensor, *, stride=1, padding=0, tile_m: int = 0,
                 bias: Optional[torch.Tensor] = None, relu: bool = False, pool2: bool = False,
                 gemm_engine: int = capi.GEMM_AUTO, product_dtype: Optional[torch.dtype] = None,
                 pool: Optional[ScratchPool] = None, algo: int = capi.ALGO_AUTO):
        if not weight.is_cuda:
            raise RuntimeError("WinoConv needs CUDA tensors: the engine has no CPU path")
        nd = weight.dim() - 2
        if nd not in (2, 3) or len(in_shape) != nd + 2:
            raise ValueError("weight must be [K,C,kH,kW] or [K,C,kD,kH,kW] and in_shape channels-last of matching rank")
        self.ndim = nd
        self.device = weight.device
        self.dtype = weight.dtype
        self.in_shape = tuple(int(s) for s in in_shape)
        k, c = int(weight.shape[0]), int(weight.shape[1])
        if self.in_shape[-1] != c:
            raise ValueError(f"input has {self.in_shape[-1]} channels, weight expects {c}")
        epi = (capi.EPI_BIAS if bias is not None else 0) | (capi.EPI_RELU if relu else 0) | (capi.EPI_POOL2 if pool2 else 0)
        pdt = capi.F32 if product_dtype is None else dtype_code(product_dtype)
        self.desc = capi.make_desc(ndim=nd, batch=self.in_shape[0], c_in=c, k_out=k, in_size=self.in_shape[1:-1],
                                   ker_size=tuple(weight.shape[2:]), stride=stride, pad=padding, tile_m=tile_m,
                                   dtype=dtype_code(weight.dtype), weight_layout=capi.W_KCRS, epilogue=epi,
                                   gemm_engine=gemm_engine, product_dtype=pdt, algo=algo)
        self.info = capi.plan(self.desc)
        out_sp = list(self.info.out_size)[3 - nd:]
        self.out_shape = (self.in_shape[0], *out_sp, k)
        self.bias = None if bias is None else bias.to(device=self.device, dtype=self.dtype).contiguous()
        self.pool = pool if pool is not None else ScratchPool.default(self.device)
        self.u = torch.empty(int(self.info.filter_bytes), dtype=torch.uint8, device=self.device)
        self.set_weight(weight)

    def set_weight(self, weight: torch.Tensor) -> None:
        """(Re)compute U = G g G^T; done once per weight, outside the per-call path."""
        w = weight.to(device=self.device, dtype=self.dtype).contiguous()
        with torch.cuda.device(self.device):
            capi.filter_transform(self.desc, w.data_ptr(), self.u.data_ptr(), _stream_ptr(self.device))
        self._w_keepalive = w

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if tuple(x.shape) != self.in_shape or x.dtype != self.dtype or x.device != self.device:
            raise ValueError(f"expected {self.in_shape} {self.dtype} on {self.device}, got {tuple(x.shape)} {x.dtype} on {x.device}")
        if not x.is_contiguous():
            raise ValueError("input must be contiguous channels-last ([N,(D,)H,W,C])")
        if out is None:
            out = torch.empty(self.out_shape, dtype=self.dtype, device=self.device)
        elif tuple(out.shape) != self.out_shape or out.dtype != self.dtype or not out.is_contiguous():
            raise ValueError(f"out must be contiguous {self.out_shape} {self.dtype}")
        v, m = self._scratch()
        with torch.cuda.device(self.device):
            capi.forward(self.desc, x.data_ptr(), self.u.data_ptr(), None if self.bias is None else self.bias.data_ptr(),
                         out.data_ptr(), v.data_ptr(), v.numel(), m.data_ptr(), m.numel(), _stream_ptr(self.device))
        return out

    def _scratch(self):
        """V / M scratch for the staged algorithm; the fused kernel needs none."""
        if self.info.algo == capi.ALGO_FUSED or (self.info.algo == capi.ALGO_ROW and self.info.input_ws_bytes == 0):
            return _NO_SCRATCH, _NO_SCRATCH
        if self.info.algo == capi.ALGO_ROW:          # channel-padding buffer only
            v, _ = self.pool.get(self.device, int(self.info.input_ws_bytes), 16)
            return v, _NO_SCRATCH
        return self.pool.get(self.device, int(self.info.input_ws_bytes), int(self.info.product_ws_bytes))

    def timed(self, x: torch.Tensor, out: Optional[torch.Tensor] = None):
        """Forward with CUDA events around the three stages: (y, [ms_in, ms_gemm, ms_out], launches)."""
        if out is None:
            out = torch.empty(self.out_shape, dtype=self.dtype, device=self.device)
        v, m = self._scratch()
        with torch.cuda.device(self.device):
            ms, n = capi.forward_timed(self.desc, x.data_ptr(), self.u.data_ptr(),
                                       None if self.bias is None else self.bias.data_ptr(), out.data_ptr(),
                                       v.data_ptr(), v.numel(), m.data_ptr(), m.numel(), _stream_ptr(self.device))
        return out, ms, n

    @property
    def launches_per_call(self) -> int:
        """Kernels this forward launches: three per pass over a block of tiles."""
        if self.info.algo == capi.ALGO_FUSED:
            return 1
        if self.info.algo == capi.ALGO_ROW:
            return 2 if self.info.input_ws_bytes else 1
        blocks = -(-int(self.info.tiles) // int(self.info.block_tiles))
        return 3 * blocks


def conv_forward(x: torch.Tensor, weight: torch.Tensor, *, stride=1, padding=0, tile_m: int = 0,
                 bias: Optional[torch.Tensor] = None, channels_last_in: bool = False, **kw) -> torch.Tensor:
    """One-shot convolution.  ``x`` is ``[N,C,*sp]`` (torch order) unless ``channels_last_in``;
    the result has the same convention.  Plans and transforms the filter on every call -- use
    :class:`WinoConv` to amortise that."""
    nd = weight.dim() - 2
    if channels_last_in:
        xc = x.contiguous()
    else:
        xc = x.permute(0, *range(2, 2 + nd), 1).contiguous()
    conv = WinoConv(xc.shape, weight, stride=stride, padding=padding, tile_m=tile_m, bias=bias, **kw)
    y = conv(xc)
    if channels_last_in:
        return y
    return y.permute(0, nd + 1, *range(1, nd + 1)).contiguous()


# ------------------------------------------------------------------------------------------
# VGG-16 convolution stack (13 3x3/s1/p1 convs + ReLU, 2x2 max-pool after convs 2,4,7,10,13)
# ------------------------------------------------------------------------------------------
VGG16_CHANNELS = [(3, 64), (64, 64), (64, 128), (128, 128), (128, 256), (256, 256), (256, 256),
                  (256, 512), (512, 512), (512, 512), (512, 512), (512, 512), (512, 512)]
VGG16_POOL_AFTER = (1, 3, 6, 9, 12)


class VGG16ConvStack:
    """The 13 convolutions of VGG-16 with ReLU and the five max-pools fused into the output
    transforms.  Input ``[N, H, W, 3]`` channels-last; output ``[N, H/32, W/32, 512]``."""

    def __init__(self, weights: Sequence[torch.Tensor], batch: int, height: int = 224, width: int = 224,
                 tile_m: int = 0, product_dtype: Optional[torch.dtype] = None, gemm_engine: int = capi.GEMM_AUTO,
                 algo: int = capi.ALGO_AUTO, pool: Optional[ScratchPool] = None):
        if len(weights) != 13:
            raise ValueError("VGG-16 has 13 convolutions")
        self.layers: List[WinoConv] = []
        self.acts: List[torch.Tensor] = []
        h, w = height, width
        dev, dt = weights[0].device, weights[0].dtype
        self.in_shape = (batch, h, w, 3)
        for i, wt in enumerate(weights):
            cin = int(wt.shape[1])
            conv = WinoConv((batch, h, w, cin), wt, padding=1, tile_m=tile_m, relu=True,
                            pool2=i in VGG16_POOL_AFTER, product_dtype=product_dtype, gemm_engine=gemm_engine,
                            algo=algo, pool=pool)
            self.layers.append(conv)
            self.acts.append(torch.empty(conv.out_shape, dtype=dt, device=dev))
            h, w = conv.out_shape[1], conv.out_shape[2]
        self.out_shape = self.layers[-1].out_shape
        self._graph = None
        self._graph_in = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = x
        for conv, buf in zip(self.layers, self.acts):
            h = conv(h, out=buf)
        return h

    __call__ = forward

    def capture(self, x: torch.Tensor) -> None:
        """Record the whole stack into a CUDA graph reading from a static copy of ``x``."""
        self._graph_in = x.clone()
        s = torch.cuda.Stream(device=x.device)
        s.wait_stream(torch.cuda.current_stream(x.device))
        with torch.cuda.stream(s):
            self.forward(self._graph_in)          # warm-up outside capture (function attributes, pool growth)
        torch.cuda.current_stream(x.device).wait_stream(s)
        torch.cuda.synchronize(x.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.forward(self._graph_in)
        self._graph = g

    def replay(self, x: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self._graph is None:
            raise RuntimeError("call capture() first")
        if x is not None:
            self._graph_in.copy_(x, non_blocking=True)
        self._graph.replay()
        return self.acts[-1]

    @property
    def launches_per_call(self) -> int:
        return sum(c.launches_per_call for c in self.layers)

    @property
    def direct_flops(self) -> float:
        return sum(c.info.direct_flops for c in self.layers)
