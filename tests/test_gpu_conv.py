"""Parity of the forward convolution (through the C ABI) with the float64 direct-convolution
oracle: the BASELINE configurations at full size, small cases covering every edge the reference
handles (odd output extents -> masked last tile, zero-fill padding, every DWM piece shape) and
the ones it does not (stride 2, F(4x4,3x3), channel counts that are not vector multiples),
plus size-independent properties at full size."""
import pytest
import torch

from oracle import winograd_oracle as wo
from pytorch_winoconv_b200 import capi
from tests.gpu_util import TOL, check_against_oracle, run_engine, seeded

pytestmark = pytest.mark.gpu

SMALL = [
    # N, C, K, spatial, kernel, stride, pad, tile_m
    (2, 8, 8, (9, 10), (3, 3), 1, 1, 2),
    (2, 8, 8, (9, 10), (3, 3), 1, 1, 4),
    (1, 16, 8, (13, 13), (3, 3), 1, 0, 4),       # odd outputs, no padding
    (2, 3, 5, (12, 11), (3, 3), 1, 1, 4),        # C, K not vector multiples
    (1, 7, 9, (10, 10), (3, 3), 1, 1, 2),
    (1, 8, 8, (11, 9), (5, 5), 1, 2, 0),         # 5x5 -> 4 pieces
    (1, 6, 4, (15, 14), (7, 7), 1, 3, 0),        # 7x7 -> 9 pieces
    (2, 3, 8, (33, 32), (7, 7), 2, 3, 0),        # stride-2 polyphase
    (1, 8, 8, (12, 13), (3, 3), 2, 1, 0),
    (1, 4, 4, (12, 12), (9, 9), 1, 4, 0),
    (1, 8, 8, (9, 9), (4, 4), 1, 0, 0),          # 4 -> 2 + 2
    (1, 8, 8, (10, 9), (3, 4), 1, 0, 0),
    (1, 8, 8, (9, 9), (1, 1), 1, 0, 0),
    (1, 8, 8, (9, 12), (1, 3), 1, 0, 0),
    (1, 8, 8, (5, 6, 7), (3, 3, 3), 1, 1, 0),    # 3-D
    (1, 4, 6, (6, 7, 6), (5, 3, 2), 1, 0, 0),
    (1, 4, 4, (4, 9, 9), (1, 3, 3), 1, 1, 0),    # depth kernel of 1 in a 3-D tensor
    (1, 4, 4, (7, 8, 9), (3, 3, 3), 2, 1, 0),    # 3-D stride 2
    (1, 4, 4, (12, 4, 4), (10, 3, 3), 1, 1, 0),  # 10 -> 3+3+3+1
    (1, 4, 4, (7, 10, 11), (5, 7, 7), 1, 0, 0),  # asymmetric 3-D shapes of the reference's piece table: 18 pieces
    (1, 4, 4, (10, 7, 8), (8, 4, 4), 1, 0, 0),   # 8 -> 3+3+2, 4 -> 2+2: 12 pieces
]


@pytest.mark.parametrize("n,c,k,sp,ks,stride,pad,m", SMALL)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_small_cases(n, c, k, sp, ks, stride, pad, m, dtype):
    """Staged algorithm (input transform -> batched GEMM -> output transform)."""
    x = seeded((n, c) + sp, 11, dtype=dtype)
    w = wo.kaiming_normal((k, c) + ks, 12).to(dtype)
    y, conv = run_engine(x, w, stride=stride, padding=pad, tile_m=m, algo=capi.ALGO_STAGED)
    assert conv.info.algo == capi.ALGO_STAGED
    check_against_oracle(x, w, y, stride=stride, padding=pad)


FUSED_EXTRA = [
    (3, 64, 64, (20, 24), (3, 3), 1, 1, 2),        # several work items, two channel blocks
    (2, 72, 40, (17, 15), (3, 3), 1, 1, 2),        # reduction slab tail, K not a block multiple
    (1, 160, 96, (12, 12), (5, 5), 1, 2, 2),       # windows straddling 64-wide slabs
    (5, 16, 8, (30, 31), (3, 3), 1, 1, 2),         # tiles not a multiple of 128
    (1, 8, 36, (9, 9), (3, 3), 1, 1, 2),           # K = 36: 16-byte stores with a partial last block
    (1, 8, 30, (9, 9), (3, 3), 1, 1, 2),           # K not a multiple of 8: element-wise stores
    (2, 3, 64, (30, 28), (3, 3), 1, 1, 2),         # RGB first layer: few-channel FMA variant
    (1, 4, 10, (11, 12), (5, 5), 1, 2, 2),         # few channels, K not a multiple of 4
    (1, 1, 520, (9, 9), (3, 3), 1, 1, 2),          # too many output channels for the few-channel variant
]


@pytest.mark.parametrize("n,c,k,sp,ks,stride,pad,m", [c for c in SMALL if c[7] != 4] + FUSED_EXTRA)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fused_cases(n, c, k, sp, ks, stride, pad, m, dtype):
    """Fused single-kernel algorithm on the same shapes (every DWM piece shape, stride 2, 3-D, ragged edges)."""
    x = seeded((n, c) + sp, 11, dtype=dtype)
    w = wo.kaiming_normal((k, c) + ks, 12).to(dtype)
    y, conv = run_engine(x, w, stride=stride, padding=pad, tile_m=2, algo=capi.ALGO_FUSED)
    assert conv.info.algo == capi.ALGO_FUSED and conv.info.positions == 16
    check_against_oracle(x, w, y, stride=stride, padding=pad)


ROW_CASES = [c for c in SMALL + FUSED_EXTRA if c[7] != 4] + [
    (2, 32, 64, (16, 64), (3, 3), 1, 1, 2),        # exactly one 8 x 16 block per image, one channel slab
    (1, 64, 128, (40, 70), (3, 3), 1, 1, 2),       # N = 128 accumulators, ragged blocks in both directions
    (2, 96, 192, (14, 14), (3, 3), 1, 1, 2),       # 16 x 8 block shape, two channel blocks, slab tail
    (1, 40, 72, (9, 50), (3, 3), 1, 0, 2),         # no padding, K not a block multiple
    (1, 16, 16, (12, 12), (7, 7), 1, 3, 2),
    (2, 16, 32, (20, 24), (9, 9), 1, 4, 2),        # 9 x 9 (the tallest 2-D shape of the reference's table): 9 rows x 3 windows
    (1, 8, 16, (14, 26), (10, 10), 1, 5, 2),       # tallest kernel the engine takes
    (3, 64, 128, (20, 36), (3, 3), 1, 1, 2),       # CTA pairs, odd batch: the last pair holds one image
    (5, 24, 64, (17, 23), (3, 3), 1, 1, 2),        # CTA pairs at 64-wide accumulators (two TMEM buffers), odd batch
    (4, 256, 256, (28, 28), (3, 3), 1, 1, 2),      # eight channel slabs, filter slabs streamed through the ring
    (2, 512, 128, (14, 14), (3, 3), 1, 1, 2),      # sixteen channel slabs, one channel block
    (3, 3, 64, (61, 57), (7, 7), 2, 3, 2),         # stride 2: four polyphase parts as 12 channels, 4 x 4 stride-1 kernel
    (2, 40, 72, (23, 30), (3, 3), 2, 1, 2),        # stride 2, 3 x 3: parts of 2 x 2, 2 x 1, 1 x 2, 1 x 1 taps
    (1, 16, 32, (20, 21), (5, 5), 2, 0, 2),        # stride 2 without padding, odd extents
    (1, 8, 16, (9, 12, 11), (3, 3, 3), 2, 1, 2),   # 3-D stride 2: eight phases
]

# fewer than eight channels with W * C a multiple of eight: x is read as it lies (no padded copy), the producers gather
# the channels; (C, padding) pairs that put the first patch pixel 0, 3, 5 and 6 elements past a multiple of eight
RAW_FEW_CHANNEL_CASES = [
    (2, 3, 64, (30, 32), (3, 3), 1, 1, 2),         # RGB, element offset 5
    (3, 3, 16, (45, 40), (5, 5), 1, 2, 2),         # RGB 5x5: two windows, odd batch, offset 2
    (1, 2, 8, (20, 24), (3, 3), 1, 0, 2),          # two channels, no padding: offset 0
    (2, 5, 8, (18, 16), (3, 3), 1, 1, 2),          # five channels: offset 3
    (1, 6, 8, (16, 20), (7, 7), 1, 3, 2),          # six channels, 7x7: three windows, offset 6, the widest raw row
    (1, 4, 4, (5, 9, 8), (3, 3, 3), 1, 1, 2),      # 3-D
    # stride 2 over few channels: the phase channels are gathered from the raw rows in the kernel (no phase-gathered copy)
    (2, 3, 64, (60, 56), (7, 7), 2, 3, 2),         # RGB stem: 4 phases x 3 channels, 4 x 4 stride-1 kernel
    (3, 3, 16, (31, 32), (3, 3), 2, 1, 2),         # 3 x 3 at stride 2, odd batch, odd height
    (1, 4, 16, (35, 36), (5, 5), 2, 0, 2),         # four channels: 16 phase channels fill both vectors (16 x 8 tile blocks)
    (1, 3, 8, (18, 24), (3, 3), (1, 2), 1, 2),     # stride 2 along W only
    (1, 2, 8, (19, 20), (5, 3), (2, 1), (2, 1), 2),  # stride 2 along H only
    # stride 2 over a multiple of 32 channels: each 32-channel step is one polyphase part, loaded from the caller's tensor
    # through an element-strided tensor map (no phase-gathered copy)
    (2, 32, 64, (23, 30), (3, 3), 2, 1, 2),        # odd extents, padding
    (3, 64, 64, (28, 28), (3, 3), 2, 1, 2),        # a ResNet-style downsampling layer, odd batch
    (2, 64, 128, (30, 32), (7, 7), 2, 3, 2),       # 7 x 7: 4 x 4 stride-1 kernel over 256 phase channels
    (1, 32, 32, (17, 20), (3, 3), (2, 1), 1, 2),   # stride 2 along H only
    (1, 32, 16, (5, 12, 11), (3, 3, 3), (1, 2, 2), 1, 2),   # 3-D, stride 2 in the plane
    # ... and over a multiple of 8: each part's channels are padded to 32 by the map's zero fill and zero filter channels
    (2, 24, 32, (23, 30), (3, 3), 2, 1, 2),        # 24 of 32
    (1, 48, 64, (20, 22), (3, 3), 2, 1, 2),        # 48 of 64: a full step and a half one per part
    (1, 72, 16, (17, 18), (5, 5), 2, 2, 2),        # 72 of 96, 5 x 5
]
ROW_CASES = ROW_CASES + RAW_FEW_CHANNEL_CASES


@pytest.mark.parametrize("n,c,k,sp,ks,stride,pad,m", ROW_CASES)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_row_piece_cases(n, c, k, sp, ks, stride, pad, m, dtype):
    """Row-piece kernel (1 x 3 DWM pieces; F(2,3) along W, taps along H / depth summed in TMEM)."""
    x = seeded((n, c) + sp, 11, dtype=dtype)
    w = wo.kaiming_normal((k, c) + ks, 12).to(dtype)
    y, conv = run_engine(x, w, stride=stride, padding=pad, tile_m=2, algo=capi.ALGO_ROW)
    assert conv.info.algo == capi.ALGO_ROW and conv.info.positions == 4
    if (n, c, k, sp, ks, stride, pad, m) in RAW_FEW_CHANNEL_CASES:
        assert conv.info.input_ws_bytes == 0 and conv.launches_per_call == 1      # no padded copy of x
    check_against_oracle(x, w, y, stride=stride, padding=pad)


def test_row_piece_epilogue_bias_relu_pool():
    for nb, hw in ((2, (13, 14)), (2, (32, 64)), (2, (16, 16)), (3, (16, 24)), (1, (16, 24))):
        x = seeded((nb, 16) + hw, 31, dtype=torch.float16)
        w = wo.kaiming_normal((72, 16, 3, 3), 32).half()
        b = seeded((72,), 33, dtype=torch.float16)
        o = wo.direct_conv_f64(x, w, padding=1) + b.double().view(1, -1, 1, 1)
        y, conv = run_engine(x, w, padding=1, tile_m=2, bias=b, relu=True, algo=capi.ALGO_ROW)
        assert conv.info.algo == capi.ALGO_ROW
        assert wo.error_metrics(y, torch.relu(o))["E_A"] < 5e-3
        y, _ = run_engine(x, w, padding=1, tile_m=2, bias=b, relu=True, pool2=True, algo=capi.ALGO_ROW)
        op = torch.nn.functional.max_pool2d(torch.relu(o), 2)
        assert tuple(y.shape) == tuple(op.shape)
        assert wo.error_metrics(y, op)["E_A"] < 5e-3


def test_fused_epilogue_bias_relu_pool():
    x = seeded((2, 16, 13, 14), 31, dtype=torch.float16)
    w = wo.kaiming_normal((40, 16, 3, 3), 32).half()
    b = seeded((40,), 33, dtype=torch.float16)
    o = wo.direct_conv_f64(x, w, padding=1) + b.double().view(1, -1, 1, 1)
    y, conv = run_engine(x, w, padding=1, tile_m=2, bias=b, relu=True, algo=capi.ALGO_FUSED)
    assert conv.info.algo == capi.ALGO_FUSED
    assert wo.error_metrics(y, torch.relu(o))["E_A"] < 5e-3
    y, _ = run_engine(x, w, padding=1, tile_m=2, bias=b, relu=True, pool2=True, algo=capi.ALGO_FUSED)
    op = torch.nn.functional.max_pool2d(torch.relu(o), 2)
    assert tuple(y.shape) == tuple(op.shape) == (2, 40, 6, 7)
    assert wo.error_metrics(y, op)["E_A"] < 5e-3


def test_fused_and_staged_agree():
    x = seeded((4, 64, 28, 28), 71, dtype=torch.float16)
    w = wo.kaiming_normal((64, 64, 3, 3), 72).half()
    yf, _ = run_engine(x, w, padding=1, tile_m=2, algo=capi.ALGO_FUSED)
    ys, _ = run_engine(x, w, padding=1, tile_m=2, algo=capi.ALGO_STAGED)
    assert wo.error_metrics(yf, ys.double())["E_B"] < 5e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("eng", [capi.GEMM_SIMT, capi.GEMM_TCGEN05])
def test_both_gemm_engines(dtype, eng):
    x = seeded((2, 24, 14, 14), 21, dtype=dtype)
    w = wo.kaiming_normal((40, 24, 3, 3), 22).to(dtype)
    y, conv = run_engine(x, w, padding=1, gemm_engine=eng)
    assert conv.info.gemm_engine == eng
    check_against_oracle(x, w, y, padding=1)


def test_epilogue_bias_relu_pool():
    x = seeded((2, 8, 13, 14), 31, dtype=torch.float16)
    w = wo.kaiming_normal((16, 8, 3, 3), 32).half()
    b = seeded((16,), 33, dtype=torch.float16)
    o = wo.direct_conv_f64(x, w, padding=1) + b.double().view(1, -1, 1, 1)
    for m in (2, 4):
        y, _ = run_engine(x, w, padding=1, tile_m=m, bias=b, relu=True)
        assert wo.error_metrics(y, torch.relu(o))["E_A"] < 5e-3
        y, _ = run_engine(x, w, padding=1, tile_m=m, bias=b, relu=True, pool2=True)
        op = torch.nn.functional.max_pool2d(torch.relu(o), 2)
        assert tuple(y.shape) == tuple(op.shape) == (2, 16, 6, 7)
        assert wo.error_metrics(y, op)["E_A"] < 5e-3


def test_blocked_passes_equal_single_pass():
    # scratch for 256 tiles forces several passes over the 2 x 11 x 11 = 242... tiles of a bigger image
    from pytorch_winoconv_b200 import engine
    x = seeded((3, 16, 40, 44), 41, dtype=torch.float16)
    w = wo.kaiming_normal((16, 16, 3, 3), 42).half()
    dev = torch.device("cuda", 0)
    xl = x.permute(0, 2, 3, 1).contiguous().to(dev)
    conv = engine.WinoConv(xl.shape, w.to(dev), padding=1, tile_m=4)      # F(4x4,3x3): staged
    y_full = conv(xl).clone()
    v = torch.empty(int(conv.info.input_ws_bytes_min) * 2, dtype=torch.uint8, device=dev)
    m = torch.empty(int(conv.info.product_ws_bytes_min) * 2, dtype=torch.uint8, device=dev)
    y_blk = torch.empty_like(y_full)
    capi.forward(conv.desc, xl.data_ptr(), conv.u.data_ptr(), None, y_blk.data_ptr(), v.data_ptr(), v.numel(),
                 m.data_ptr(), m.numel(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert conv.info.tiles > 256
    assert torch.equal(y_full, y_blk)
    with pytest.raises(capi.WinoconvError) as ei:
        capi.forward(conv.desc, xl.data_ptr(), conv.u.data_ptr(), None, y_blk.data_ptr(), v.data_ptr(), 1024,
                     m.data_ptr(), m.numel(), torch.cuda.current_stream().cuda_stream)
    assert ei.value.status == capi.ERR_WORKSPACE


# ---- BASELINE.json configurations at full size -------------------------------------------------
def test_cfg1_fp32_f23():
    x = seeded((8, 64, 56, 56), 0)
    w = wo.kaiming_normal((64, 64, 3, 3), 1)
    y, conv = run_engine(x, w, padding=1, tile_m=2)
    assert conv.info.positions == 16
    err = check_against_oracle(x, w, y, padding=1)
    ref = wo.error_metrics(wo.winograd_conv_cpu(x, w, padding=1, tile_m=2), wo.direct_conv_f64(x, w, padding=1))
    print("cfg1 engine", err, "reference algebra (CPU fp32)", ref)


def test_cfg1_fp32_product_arithmetic_table():
    """configs[0] with the three ways of forming the fp32 products: fp32 FMA, one tf32 product, three tf32 products of
    a hi / lo split.  The 1e-3 bound of the fp32 path holds for the first and the last; the measured E_B of each is
    printed (and quoted in the design notes)."""
    x = seeded((8, 64, 56, 56), 0)
    w = wo.kaiming_normal((64, 64, 3, 3), 1)
    o = wo.direct_conv_f64(x, w, padding=1)
    table = {}
    for name, eng in (("fp32 fma", capi.GEMM_SIMT), ("tf32", capi.GEMM_TF32), ("tf32 x3", capi.GEMM_TF32X3)):
        for tm in (2, 4):
            y, conv = run_engine(x, w, padding=1, tile_m=tm, gemm_engine=eng)
            assert conv.info.gemm_engine == eng
            table[(name, tm)] = wo.error_metrics(y, o)["E_B"]
    print("cfg1 E_B by product arithmetic and tile:", {f"{k[0]} F({k[1]}x{k[1]},3x3)": "%.3g" % v for k, v in table.items()})
    for tm in (2, 4):
        assert table[("fp32 fma", tm)] <= 1e-3 and table[("tf32 x3", tm)] <= 1e-3
        assert table[("tf32 x3", tm)] <= 4 * table[("fp32 fma", tm)] + 1e-6
        assert table[("tf32", tm)] <= 2e-2          # bounded, but (measured) over the fp32 tolerance


@pytest.mark.parametrize("dtype,product", [(torch.bfloat16, None), (torch.bfloat16, torch.bfloat16), (torch.float16, torch.float16)])
@pytest.mark.parametrize("n,c,k,sp,pad", [(3, 64, 72, (20, 24), 1),       # whole tiles, K not a multiple of 64
                                          (2, 136, 64, (30, 27), 1),      # ragged tiles in both directions, three channel blocks
                                          (1, 8, 8, (9, 41), 0)])         # no padding, one channel vector, a wide strip
def test_staged_f43_tma_transforms(dtype, product, n, c, k, sp, pad):
    """F(4x4,3x3) with both transforms staged through shared memory by TMA (channels a multiple of eight), in the
    dtype and product combinations the BASELINE configurations do not reach; bias and ReLU in the output transform."""
    x = seeded((n, c) + sp, 41, dtype=dtype)
    w = wo.kaiming_normal((k, c, 3, 3), 42).to(dtype)
    b = seeded((k,), 43, dtype=dtype)
    y, conv = run_engine(x, w, padding=pad, tile_m=4, bias=b, relu=True, product_dtype=product)
    assert conv.info.algo == capi.ALGO_STAGED and conv.info.positions == 36
    o = torch.relu(wo.direct_conv_f64(x, w, padding=pad) + b.double().view(1, -1, 1, 1))
    err = wo.error_metrics(y, o)
    tol = {torch.float16: 3e-2, torch.bfloat16: 1.6e-1}[dtype]     # 16-bit products on top of the 16-bit operands
    assert err["E_B"] <= tol, err


def test_auto_f43_on_a_512_channel_layer():
    """The one place AUTO leaves the row-piece kernel: 512 -> 512 at 28 x 28 with >= 4096 tiles runs as staged
    F(4x4,3x3) with both transforms staged through shared memory by TMA.  Checked against the float64 direct
    convolution on the first and the last image (the whole batch would take the CPU minutes)."""
    n = 84                                             # 84 x 49 = 4116 tiles
    g = torch.Generator().manual_seed(5)
    x = torch.randn(n, 512, 28, 28, generator=g).half()
    w = wo.kaiming_normal((512, 512, 3, 3), 6).half()
    b = seeded((512,), 7, dtype=torch.float16)
    y, conv = run_engine(x, w, padding=1, bias=b, relu=True)
    assert conv.info.algo == capi.ALGO_STAGED and conv.info.positions == 36 and conv.launches_per_call == 3
    for i in (0, n - 1):
        o = torch.relu(wo.direct_conv_f64(x[i:i + 1], w, padding=1) + b.double().view(1, -1, 1, 1))
        err = wo.error_metrics(y[i:i + 1], o)
        print("AUTO -> F(4x4,3x3), image", i, err)
        assert err["E_B"] <= TOL[torch.float16], err
    y2, conv2 = run_engine(x[:8], w, padding=1, bias=b, relu=True)       # a small batch stays on the row-piece kernel
    assert conv2.info.algo == capi.ALGO_ROW
    assert wo.error_metrics(y2, y[:8].double())["E_A"] < 2e-2            # the two algorithms agree to fp16 accuracy


F63_CASES = [
    # N, C, K, spatial, padding
    (2, 8, 8, (12, 12), 1),            # 2 x 2 whole tiles
    (1, 16, 8, (13, 17), 0),           # no padding, ragged last tiles (11 x 15 outputs)
    (2, 3, 5, (9, 20), 1),             # C, K not vector multiples; a single tile row
    (1, 7, 9, (30, 7), (2, 1)),        # wider padding than the kernel needs, narrow image
    (8, 64, 64, (56, 56), 1),          # configs[0]'s layer
]


@pytest.mark.parametrize("n,c,k,sp,pad", F63_CASES)
@pytest.mark.parametrize("eng", [capi.GEMM_SIMT, capi.GEMM_TF32X3])
def test_f63_fp32(n, c, k, sp, pad, eng):
    """F(6x6,3x3) (64 positions, 1.78 multiplies per output; the reference stops at F(2,3)): fp32 operands with fp32 FMA
    or three-tf32 products hold the fp32 bound."""
    x = seeded((n, c) + sp, 21)
    w = wo.kaiming_normal((k, c, 3, 3), 22)
    y, conv = run_engine(x, w, padding=pad, tile_m=6, gemm_engine=eng)
    assert conv.info.algo == capi.ALGO_STAGED and conv.info.positions == 64 and list(conv.info.tile_m) == [1, 6, 6]
    err = check_against_oracle(x, w, y, padding=pad)
    print("F(6x6,3x3)", (n, c, k, sp), "engine", eng, err)
    assert err["E_B"] <= 2e-4, err       # measured 1e-5-class; well inside the 1e-3 contract


def test_f63_epilogue_and_refusals():
    x = seeded((2, 16, 14, 16), 23)
    w = wo.kaiming_normal((24, 16, 3, 3), 24)
    b = seeded((24,), 25)
    o = torch.relu(wo.direct_conv_f64(x, w, padding=1) + b.double().view(1, -1, 1, 1))
    y, _ = run_engine(x, w, padding=1, tile_m=6, bias=b, relu=True)
    assert wo.error_metrics(y, o)["E_A"] < 1e-4
    y, _ = run_engine(x, w, padding=1, tile_m=6, bias=b, relu=True, pool2=True)
    op = torch.nn.functional.max_pool2d(o, 2)
    assert tuple(y.shape) == tuple(op.shape) and wo.error_metrics(y, op)["E_A"] < 1e-4
    for kw in (dict(dtype=capi.F16), dict(dtype=capi.F32, gemm_engine=capi.GEMM_TF32), dict(dtype=capi.F32, ker_size=5),
               dict(dtype=capi.F32, stride=2)):
        args = dict(ndim=2, batch=1, c_in=8, k_out=8, in_size=(12, 12), ker_size=3, stride=1, pad=1, tile_m=6)
        args.update(kw)
        with pytest.raises(capi.WinoconvError) as ei:
            capi.plan(capi.make_desc(**args))
        assert ei.value.status == capi.ERR_UNSUPPORTED


@pytest.mark.parametrize("product_dtype", [None, torch.float16])
@pytest.mark.parametrize("seed", [0, 17])
def test_cfg2_fp16_f43(product_dtype, seed):
    x = seeded((32, 256, 28, 28), seed, dtype=torch.float16)
    w = wo.kaiming_normal((256, 256, 3, 3), seed + 1).half()
    y, conv = run_engine(x, w, padding=1, tile_m=4, product_dtype=product_dtype)
    assert conv.info.positions == 36 and conv.info.gemm_engine == capi.GEMM_TCGEN05
    err = check_against_oracle(x, w, y, padding=1)
    print("cfg2 engine", product_dtype, "seed", seed, err)


ALGOS = [(capi.ALGO_STAGED, "staged"), (capi.ALGO_FUSED, "fused"), (capi.ALGO_ROW, "row")]


@pytest.mark.parametrize("algo,name", ALGOS)
def test_cfg3a_fp16_7x7_stride2(algo, name):
    x = seeded((64, 3, 224, 224), 0, dist="uniform", dtype=torch.float16)
    w = wo.kaiming_normal((64, 3, 7, 7), 1).half()
    y, conv = run_engine(x, w, stride=2, padding=3, algo=algo)
    # staged: 9 polyphase / DWM pieces, 100 positions; 3x3-piece kernel: the same 9 pieces at 16 positions;
    # row kernel: 4 phases as channels, a 4 x 4 stride-1 kernel = 4 rows x 2 windows of 4 positions
    expect = {capi.ALGO_STAGED: (9, 100), capi.ALGO_FUSED: (9, 16), capi.ALGO_ROW: (8, 4)}[algo]
    assert (conv.info.n_pieces, conv.info.positions) == expect
    print("cfg3a engine", name, check_against_oracle(x, w, y, stride=2, padding=3))


@pytest.mark.parametrize("algo,name", ALGOS)
def test_cfg3b_fp16_5x5(algo, name):
    x = seeded((32, 128, 56, 56), 0, dtype=torch.float16)
    w = wo.kaiming_normal((128, 128, 5, 5), 1).half()
    y, conv = run_engine(x, w, padding=2, algo=algo)
    assert (conv.info.n_pieces, conv.info.positions) == {capi.ALGO_STAGED: (4, 49), capi.ALGO_FUSED: (4, 16), capi.ALGO_ROW: (10, 4)}[algo]
    print("cfg3b engine", name, check_against_oracle(x, w, y, padding=2))


@pytest.mark.parametrize("algo,name", ALGOS)
def test_cfg4_fp16_3d(algo, name):
    x = seeded((8, 64, 16, 56, 56), 0, dtype=torch.float16)
    w = wo.kaiming_normal((64, 64, 3, 3, 3), 1).half()
    y, conv = run_engine(x, w, padding=1, algo=algo)
    assert (conv.info.n_pieces, conv.info.positions) == {capi.ALGO_STAGED: (1, 64), capi.ALGO_FUSED: (3, 16), capi.ALGO_ROW: (9, 4)}[algo]
    print("cfg4 engine", name, check_against_oracle(x, w, y, padding=1))


def test_auto_resolves_to_row_for_16bit_and_staged_otherwise():
    x = seeded((1, 8, 12, 12), 1, dtype=torch.float16)
    w5 = wo.kaiming_normal((8, 8, 5, 5), 2).half()
    w3 = wo.kaiming_normal((8, 8, 3, 3), 3).half()
    assert run_engine(x, w5, padding=2)[1].info.algo == capi.ALGO_ROW
    assert run_engine(x, w5, padding=2, stride=2)[1].info.algo == capi.ALGO_ROW     # stride 2: phases folded into channels
    assert run_engine(x, w5, padding=2, stride=2, algo=capi.ALGO_FUSED)[1].info.algo == capi.ALGO_FUSED
    assert run_engine(x, w3, padding=1)[1].info.algo == capi.ALGO_ROW             # 16-bit: 2-wide tiles, one kernel
    assert run_engine(x, w3, padding=1, tile_m=2)[1].info.algo == capi.ALGO_ROW
    c4 = run_engine(x, w3, padding=1, tile_m=4)[1]                                # F(4x4,3x3) on request: staged
    assert c4.info.algo == capi.ALGO_STAGED and c4.info.positions == 36
    cs = run_engine(x, w3, padding=1, algo=capi.ALGO_STAGED)[1]                   # staged on request: auto tile is 4
    assert cs.info.algo == capi.ALGO_STAGED and cs.info.positions == 36
    c32 = run_engine(x.float(), w3.float(), padding=1)[1]                         # fp32: staged F(4x4,3x3)
    assert c32.info.algo == capi.ALGO_STAGED and c32.info.positions == 36
    assert run_engine(x.float(), w3.float(), padding=1, tile_m=2)[1].info.algo == capi.ALGO_STAGED


def test_linearity_at_full_size():
    # conv(a x1 + x2, w) == a conv(x1, w) + conv(x2, w) up to rounding, at config 2's size
    x1 = seeded((32, 256, 28, 28), 5, dtype=torch.float16)
    x2 = seeded((32, 256, 28, 28), 6, dtype=torch.float16)
    w = wo.kaiming_normal((256, 256, 3, 3), 7).half()
    xs = (2.0 * x1.float() + x2.float()).half()
    y1, _ = run_engine(x1, w, padding=1)
    y2, _ = run_engine(x2, w, padding=1)
    ys, _ = run_engine(xs, w, padding=1)
    comb = 2.0 * y1.double() + y2.double()
    assert wo.error_metrics(ys, comb)["E_B"] < 2 * TOL[torch.float16]


def test_translation_equivariance():
    # shifting the input by one tile (4 px) shifts the output: catches tile / halo indexing slips
    x = seeded((1, 16, 36, 36), 8, dtype=torch.float16)
    w = wo.kaiming_normal((16, 16, 3, 3), 9).half()
    y, _ = run_engine(x, w, padding=0)
    ys, _ = run_engine(x[:, :, 4:, 4:].contiguous(), w, padding=0)
    assert torch.equal(y[:, :, 4:, 4:], ys)
