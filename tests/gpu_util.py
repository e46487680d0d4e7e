"""Helpers shared by the GPU parity tests (the oracle is the checker, never the thing run)."""
import torch

from oracle import winograd_oracle as wo
from pytorch_winoconv_b200 import capi, engine

TOL = {torch.float32: 1e-3, torch.float16: 2e-2, torch.bfloat16: 1.2e-1}   # E_B bounds; bf16 has 8 mantissa bits


def seeded(shape, seed, dist="normal", dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    t = torch.randn(shape, generator=g) if dist == "normal" else torch.rand(shape, generator=g)
    return t.to(dtype)


def run_engine(x, w, *, stride=1, padding=0, tile_m=0, bias=None, relu=False, pool2=False, gemm_engine=capi.GEMM_AUTO,
               product_dtype=None, algo=capi.ALGO_AUTO):
    """x [N,C,*sp], w [K,C,*k] on CPU in the target dtype -> device result as [N,K,*out] on CPU."""
    nd = w.dim() - 2
    dev = torch.device("cuda", 0)
    xl = x.permute(0, *range(2, 2 + nd), 1).contiguous().to(dev)
    conv = engine.WinoConv(xl.shape, w.to(dev), stride=stride, padding=padding, tile_m=tile_m,
                           bias=None if bias is None else bias.to(dev), relu=relu, pool2=pool2,
                           gemm_engine=gemm_engine, product_dtype=product_dtype, algo=algo)
    y = conv(xl)
    torch.cuda.synchronize()
    assert capi.read_device_error() == 0
    return y.permute(0, nd + 1, *range(1, nd + 1)).contiguous().cpu(), conv


def check_against_oracle(x, w, y, *, stride=1, padding=0, tol=None):
    o = wo.direct_conv_f64(x, w, stride=stride, padding=padding)
    assert tuple(y.shape) == tuple(o.shape), (y.shape, o.shape)
    err = wo.error_metrics(y, o)
    tol = TOL[x.dtype] if tol is None else tol
    assert err["E_B"] <= tol, err
    return err
