"""The per-position batched GEMM through the C ABI (winoconv_gemm_batched) against a float64
matmul: both engines, ragged tile counts, output-channel counts that do not fill a block,
reductions that do not fill a 64-wide slab, fp32 / fp16 / bf16 products."""
import pytest
import torch

from pytorch_winoconv_b200 import capi, engine

pytestmark = pytest.mark.gpu

CASES = [
    # positions, tiles, c_pad, k_out
    (1, 128, 64, 64),
    (3, 128, 64, 128),
    (2, 256, 128, 256),
    (4, 300, 64, 64),        # ragged last row block
    (2, 100, 64, 64),        # fewer rows than one block
    (3, 257, 256, 512),      # two column blocks of 256
    (2, 130, 8, 64),         # reduction shorter than a slab (C = 3 padded to 8)
    (2, 200, 72, 96),        # slab tail, K not a block multiple
    (36, 1568, 256, 256),    # BASELINE config 2's GEMM
    (1, 129, 320, 40),       # K multiple of 8 but < 64
    (2, 140, 64, 30),        # K not a multiple of 8: element-wise store path
]


def _operands(pos, tiles, c_pad, k_out, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    v = torch.randn(pos, tiles, c_pad, generator=g).to(dtype)
    u = (torch.randn(pos, k_out, c_pad, generator=g) / c_pad ** 0.5).to(dtype)
    return v, u


def _run(engine_code, dtype, pdtype, pos, tiles, c_pad, k_out, tol_override=None):
    v, u = _operands(pos, tiles, c_pad, k_out, dtype)
    ref = torch.matmul(v.double(), u.double().transpose(1, 2))
    vd, ud = v.cuda(), u.cuda()
    m = torch.full((pos, tiles, k_out), float("nan"), dtype=pdtype, device="cuda")
    capi.gemm_batched(engine.dtype_code(dtype), engine.dtype_code(pdtype), engine_code, pos, tiles, c_pad, k_out,
                      vd.data_ptr(), ud.data_ptr(), m.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert capi.read_device_error() == 0
    got = m.double().cpu()
    assert torch.isfinite(got).all(), "output not fully written"
    scale = ref.abs().max().item()
    err = (got - ref).abs().max().item() / scale
    tol = {torch.float32: 2e-5, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}[pdtype]
    if dtype != torch.float32 and pdtype == torch.float32:
        tol = 2e-5     # exact products of rounded inputs, fp32 accumulation
    if tol_override is not None:
        tol = tol_override
    assert err <= tol, (err, tol)
    return err


@pytest.mark.parametrize("pos,tiles,c_pad,k_out", CASES)
def test_tf32x3_gemm_holds_the_fp32_tolerance(pos, tiles, c_pad, k_out):
    """fp32 operands on the tensor cores as three tf32 products of a hi / lo split: the same 2e-5 as the FMA kernel."""
    _run(capi.GEMM_TF32X3, torch.float32, torch.float32, pos, tiles, c_pad, k_out)


@pytest.mark.parametrize("pos,tiles,c_pad,k_out", CASES)
def test_plain_tf32_gemm(pos, tiles, c_pad, k_out):
    """one tf32 product per multiply: operands keep 10 mantissa bits, so the bound is 2^-10-class, not fp32-class"""
    _run(capi.GEMM_TF32, torch.float32, torch.float32, pos, tiles, c_pad, k_out, tol_override=3e-3)


def test_tf32_engines_refuse_16bit_operands():
    with pytest.raises(capi.WinoconvError) as ei:
        capi.gemm_batched(capi.F16, capi.F32, capi.GEMM_TF32X3, 1, 128, 64, 64, 256, 256, 256)
    assert ei.value.status == capi.ERR_UNSUPPORTED


@pytest.mark.parametrize("pos,tiles,c_pad,k_out", CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_simt_gemm(pos, tiles, c_pad, k_out, dtype):
    _run(capi.GEMM_SIMT, dtype, torch.float32, pos, tiles, c_pad, k_out)


@pytest.mark.parametrize("pos,tiles,c_pad,k_out", CASES)
@pytest.mark.parametrize("dtype,pdtype", [(torch.float16, torch.float32), (torch.bfloat16, torch.float32),
                                          (torch.float16, torch.float16), (torch.bfloat16, torch.bfloat16)])
def test_tcgen05_gemm(pos, tiles, c_pad, k_out, dtype, pdtype):
    _run(capi.GEMM_TCGEN05, dtype, pdtype, pos, tiles, c_pad, k_out)


def test_tcgen05_gemm_does_not_touch_neighbouring_memory():
    pos, tiles, c_pad, k_out = 2, 130, 64, 72
    v, u = _operands(pos, tiles, c_pad, k_out, torch.float16, seed=3)
    guard = 1024
    buf = torch.full((pos * tiles * k_out + 2 * guard,), 7.0, dtype=torch.float32, device="cuda")
    m = buf[guard:guard + pos * tiles * k_out]
    vd, ud = v.cuda(), u.cuda()
    capi.gemm_batched(capi.F16, capi.F32, capi.GEMM_TCGEN05, pos, tiles, c_pad, k_out, vd.data_ptr(), ud.data_ptr(),
                      m.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert capi.read_device_error() == 0
    assert (buf[:guard] == 7.0).all() and (buf[-guard:] == 7.0).all()


def test_engines_agree_bitwise_inputs():
    pos, tiles, c_pad, k_out = 4, 384, 128, 128
    v, u = _operands(pos, tiles, c_pad, k_out, torch.float16, seed=5)
    vd, ud = v.cuda(), u.cuda()
    outs = []
    for eng in (capi.GEMM_SIMT, capi.GEMM_TCGEN05):
        m = torch.empty(pos, tiles, k_out, dtype=torch.float32, device="cuda")
        capi.gemm_batched(capi.F16, capi.F32, eng, pos, tiles, c_pad, k_out, vd.data_ptr(), ud.data_ptr(),
                          m.data_ptr(), torch.cuda.current_stream().cuda_stream)
        outs.append(m)
    torch.cuda.synchronize()
    assert (outs[0] - outs[1]).abs().max().item() <= 1e-4 * outs[0].abs().max().item()


def test_mma_rate_probe_reports_the_figures_the_planner_relies_on():
    """A 128-column MMA from shared memory runs at the tensor pipe's rate (64 clocks); a 64-column one does not
    (the 4 KB A-operand read keeps it above ~40 clocks) unless A sits in tensor memory."""
    full, _ = capi.probe_mma_rate(False, False, 128, 2)
    narrow_smem, _ = capi.probe_mma_rate(False, False, 64, 4)
    narrow_tmem, _ = capi.probe_mma_rate(False, True, 64, 4)
    pair_narrow, _ = capi.probe_mma_rate(True, False, 64, 4)
    print("clocks per MMA: N=128 smem", full, "N=64 smem", narrow_smem, "N=64 tmem", narrow_tmem, "N=64 smem pair", pair_narrow)
    assert 56 <= full <= 80
    assert narrow_smem >= 38 and pair_narrow >= 38
    assert narrow_tmem <= 40
    with pytest.raises(capi.WinoconvError):
        capi.probe_mma_rate(False, False, 256, 4)       # four 256-column accumulators do not fit 512 columns
