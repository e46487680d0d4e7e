"""ctypes binding of ``libwinoconv_b200.so`` (the C ABI declared in ``include/winoconv_b200.h``).

This is the only door from Python to the kernels.  There is no fallback: if the library is
missing, :func:`lib` raises with the build command; if it is called without a B200 the C ABI
returns ``WINOCONV_ERR_NO_DEVICE`` and :class:`WinoconvError` is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import (POINTER, Structure, byref, c_char_p, c_double, c_int, c_int32, c_int64, c_size_t, c_uint32,
                    c_uint64, c_void_p, create_string_buffer)

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
# WINOCONV_LIB points at another build of the library (e.g. one compiled with different kernel switches)
LIB_PATH = os.environ.get("WINOCONV_LIB") or os.path.join(_PKG_DIR, "libwinoconv_b200.so")

OK, ERR_INVALID_ARGUMENT, ERR_UNSUPPORTED, ERR_WORKSPACE, ERR_CUDA, ERR_TIMEOUT, ERR_NO_DEVICE = range(7)
F32, F16, BF16 = 0, 1, 2
W_KCRS, W_RSCK = 0, 1
GEMM_AUTO, GEMM_SIMT, GEMM_TCGEN05, GEMM_TF32, GEMM_TF32X3 = 0, 1, 2, 3, 4
EPI_BIAS, EPI_RELU, EPI_POOL2 = 1, 2, 4
ALGO_AUTO, ALGO_STAGED, ALGO_FUSED, ALGO_ROW = 0, 1, 2, 3
MAX_PIECES = 64

# every symbol include/winoconv_b200.h declares
EXPORTED_SYMBOLS = (
    "winoconv_abi_version", "winoconv_status_string", "winoconv_last_error", "winoconv_device_check",
    "winoconv_plan", "winoconv_plan_pieces", "winoconv_filter_transform", "winoconv_forward",
    "winoconv_forward_timed", "winoconv_forward_static", "winoconv_gemm_batched", "winoconv_split",
    "winoconv_concat", "winoconv_add", "winoconv_read_device_error", "winoconv_probe_mma_rate",
)


class Desc(Structure):
    _fields_ = [("ndim", c_int32), ("batch", c_int32), ("c_in", c_int32), ("k_out", c_int32),
                ("in_size", c_int32 * 3), ("ker_size", c_int32 * 3), ("stride", c_int32 * 3), ("pad", c_int32 * 3),
                ("tile_m", c_int32), ("dtype", c_int32), ("weight_layout", c_int32), ("epilogue", c_uint32),
                ("gemm_engine", c_int32), ("product_dtype", c_int32), ("algo", c_int32), ("reserved", c_int32 * 5)]


class PlanInfo(Structure):
    _fields_ = [("out_size", c_int32 * 3), ("conv_out_size", c_int32 * 3), ("tile_m", c_int32 * 3),
                ("tiles_per_dim", c_int32 * 3), ("n_pieces", c_int32), ("positions", c_int32), ("c_pad", c_int32),
                ("gemm_engine", c_int32), ("algo", c_int32), ("reserved0", c_int32), ("tiles", c_int64), ("filter_bytes", c_uint64),
                ("input_ws_bytes", c_uint64), ("product_ws_bytes", c_uint64), ("input_ws_bytes_min", c_uint64),
                ("product_ws_bytes_min", c_uint64), ("block_tiles", c_int64), ("direct_flops", c_double),
                ("gemm_flops", c_double), ("algorithmic_bytes", c_double)]


class WinoconvError(RuntimeError):
    def __init__(self, status: int, what: str, detail: str):
        self.status = status
        super().__init__(f"{what}: {detail}" if detail else what)


_lib = None


def lib() -> ctypes.CDLL:
    """Load the C-ABI library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} is missing: the CUDA library is not built. "
                           "Run `python -m pytorch_winoconv_b200.build` (needs nvcc); there is no fallback path.")
    L = ctypes.CDLL(LIB_PATH)
    L.winoconv_abi_version.restype = c_int
    L.winoconv_status_string.restype = c_char_p
    L.winoconv_status_string.argtypes = [c_int]
    L.winoconv_last_error.restype = c_size_t
    L.winoconv_last_error.argtypes = [c_char_p, c_size_t]
    L.winoconv_device_check.restype = c_int
    L.winoconv_plan.argtypes = [POINTER(Desc), POINTER(PlanInfo)]
    L.winoconv_plan_pieces.argtypes = [POINTER(Desc), POINTER(c_int32), c_int32, POINTER(c_int32)]
    L.winoconv_filter_transform.argtypes = [POINTER(Desc), c_void_p, c_void_p, c_void_p]
    L.winoconv_forward.argtypes = [POINTER(Desc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                   c_void_p, c_size_t, c_void_p]
    L.winoconv_forward_timed.argtypes = [POINTER(Desc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                         c_void_p, c_size_t, c_void_p, POINTER(ctypes.c_float), POINTER(c_int32)]
    L.winoconv_forward_static.argtypes = [POINTER(Desc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
    L.winoconv_gemm_batched.argtypes = [c_int, c_int, c_int, c_int, c_int64, c_int, c_int, c_void_p, c_void_p,
                                        c_void_p, c_void_p]
    L.winoconv_split.argtypes = [c_void_p, c_void_p] + [c_int] * 14 + [c_void_p]
    L.winoconv_concat.argtypes = [c_void_p, c_void_p] + [c_int] * 8 + [c_void_p]
    L.winoconv_add.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_void_p]
    L.winoconv_read_device_error.argtypes = [c_void_p, POINTER(c_uint32)]
    L.winoconv_probe_mma_rate.argtypes = [c_int, c_int, c_int, c_int, c_int, POINTER(ctypes.c_float),
                                          POINTER(ctypes.c_float), c_void_p]
    L.winoconv_probe_mma_rate.restype = c_int
    for name in ("winoconv_plan", "winoconv_plan_pieces", "winoconv_filter_transform", "winoconv_forward",
                 "winoconv_forward_timed", "winoconv_forward_static", "winoconv_gemm_batched", "winoconv_split",
                 "winoconv_concat", "winoconv_add", "winoconv_read_device_error"):
        getattr(L, name).restype = c_int
    _lib = L
    return L


def last_error() -> str:
    buf = create_string_buffer(1024)
    lib().winoconv_last_error(buf, 1024)
    return buf.value.decode("utf-8", "replace")


def check(status: int, what: str) -> None:
    if status != OK:
        name = lib().winoconv_status_string(status).decode()
        raise WinoconvError(status, f"{what} failed ({name})", last_error())


def make_desc(*, ndim, batch, c_in, k_out, in_size, ker_size, stride=1, pad=0, tile_m=0, dtype=F16,
              weight_layout=W_KCRS, epilogue=0, gemm_engine=GEMM_AUTO, product_dtype=F32, algo=ALGO_AUTO) -> Desc:
    """Fill a descriptor.  ``in_size`` / ``ker_size`` / ``stride`` / ``pad`` have ``ndim`` entries
    (ints are broadcast); 2-D descriptors get depth 1 in slot 0."""
    def triple(v, fill):
        vals = [v] * ndim if isinstance(v, int) else list(v)
        if len(vals) != ndim:
            raise ValueError(f"expected {ndim} values, got {vals}")
        return ([fill] * (3 - ndim)) + [int(a) for a in vals]
    d = Desc()
    d.ndim, d.batch, d.c_in, d.k_out = ndim, batch, c_in, k_out
    d.in_size[:] = triple(in_size, 1)
    d.ker_size[:] = triple(ker_size, 1)
    d.stride[:] = triple(stride, 1)
    d.pad[:] = triple(pad, 0)
    d.tile_m, d.dtype, d.weight_layout = tile_m, dtype, weight_layout
    d.epilogue, d.gemm_engine, d.product_dtype, d.algo = epilogue, gemm_engine, product_dtype, algo
    return d


def plan(desc: Desc) -> PlanInfo:
    info = PlanInfo()
    check(lib().winoconv_plan(byref(desc), byref(info)), "winoconv_plan")
    return info


def plan_pieces(desc: Desc):
    arr = (c_int32 * (9 * MAX_PIECES))()
    n = c_int32(0)
    check(lib().winoconv_plan_pieces(byref(desc), arr, MAX_PIECES, byref(n)), "winoconv_plan_pieces")
    return [(tuple(arr[i * 9:i * 9 + 3]), tuple(arr[i * 9 + 3:i * 9 + 6]), tuple(arr[i * 9 + 6:i * 9 + 9]))
            for i in range(n.value)]


def filter_transform(desc: Desc, w_ptr: int, u_ptr: int, stream: int = 0) -> None:
    check(lib().winoconv_filter_transform(byref(desc), w_ptr, u_ptr, stream), "winoconv_filter_transform")


def forward(desc: Desc, x_ptr: int, u_ptr: int, bias_ptr, y_ptr: int, v_ptr: int, v_bytes: int, m_ptr: int,
            m_bytes: int, stream: int = 0) -> None:
    check(lib().winoconv_forward(byref(desc), x_ptr, u_ptr, bias_ptr, y_ptr, v_ptr, v_bytes, m_ptr, m_bytes, stream),
          "winoconv_forward")


STATIC_SCRATCH_BYTES = 32 << 20


def forward_static(desc: Desc, x_ptr: int, u_ptr: int, bias_ptr, y_ptr: int, stream: int = 0) -> None:
    """winoconv_forward_static: the forward with the library's built-in 32 MiB scratch array -- for callers
    that may not allocate device memory.  Calls on one device share that array, so they must not overlap."""
    check(lib().winoconv_forward_static(byref(desc), x_ptr, u_ptr, bias_ptr, y_ptr, stream), "winoconv_forward_static")


def forward_timed(desc: Desc, x_ptr: int, u_ptr: int, bias_ptr, y_ptr: int, v_ptr: int, v_bytes: int, m_ptr: int,
                  m_bytes: int, stream: int = 0):
    """Returns ([input_transform_ms, gemm_ms, output_transform_ms], kernels_launched)."""
    ms = (ctypes.c_float * 3)()
    n = c_int32(0)
    check(lib().winoconv_forward_timed(byref(desc), x_ptr, u_ptr, bias_ptr, y_ptr, v_ptr, v_bytes, m_ptr, m_bytes,
                                       stream, ms, byref(n)), "winoconv_forward_timed")
    return [float(v) for v in ms], int(n.value)


def gemm_batched(dtype, product_dtype, engine, positions, tiles, c_pad, k_out, v_ptr, u_ptr, m_ptr, stream=0) -> None:
    check(lib().winoconv_gemm_batched(dtype, product_dtype, engine, positions, tiles, c_pad, k_out, v_ptr, u_ptr,
                                      m_ptr, stream), "winoconv_gemm_batched")


def read_device_error(stream: int = 0) -> int:
    code = c_uint32(0)
    st = lib().winoconv_read_device_error(stream, byref(code))
    if st not in (OK, ERR_TIMEOUT):
        check(st, "winoconv_read_device_error")
    return code.value


def probe_mma_rate(cta_pair: bool, a_in_tmem: bool, n_cols: int, n_threads: int, n_mma: int = 512, stream: int = 0):
    """(clocks per MMA over all issuing threads, issue clocks per MMA of one thread) -- winoconv_probe_mma_rate."""
    total, issue = ctypes.c_float(0), ctypes.c_float(0)
    check(lib().winoconv_probe_mma_rate(int(cta_pair), int(a_in_tmem), n_cols, n_threads, n_mma, byref(total),
                                        byref(issue), stream), "winoconv_probe_mma_rate")
    return float(total.value), float(issue.value)
