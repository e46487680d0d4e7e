// C ABI of libwinoconv_b200: descriptor validation, the DWM piece rule, scratch sizing and the
// forward driver that walks the tiles in cache-sized blocks.  See include/winoconv_b200.h.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "wino_common.cuh"
#include "wino_launch.h"

namespace wino {
namespace {

thread_local std::string t_last_error;

int fail(int status, const std::string &msg) {
  t_last_error = msg;
  return status;
}

int cuda_fail(cudaError_t e, const char *what, const char *detail = "") {
  return fail(WINOCONV_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e) + (detail && *detail ? std::string(" (") + detail + ")" : std::string()));
}

size_t dtype_size(int dt) { return dt == WINOCONV_F32 ? 4 : 2; }

// Per-dimension cut of a k-tap kernel into Winograd pieces: at multiples of 3, remainder last, and 4 -> 2 + 2
// (the rule behind the look-up table of src/base_conv_launchers.h:58-388).
void dwm_cuts(int taps, std::vector<std::pair<int, int>> &out) {
  out.clear();
  if (taps <= 3) { out.push_back({0, taps}); return; }
  if (taps == 4) { out.push_back({0, 2}); out.push_back({2, 2}); return; }
  for (int s = 0; s < taps; s += 3) out.push_back({s, std::min(3, taps - s)});
}

struct DimPiece { int phase, start, r; };

struct Plan {
  Geom g;
  FGeom fg;      // filled when fused
  bool fused;
  bool row;      // row-piece kernel
  RowDesc rd;
  RowPlan rp;
  winoconv_plan_info_t info;
  int dtype, product_dtype, engine;
};

// Tiles are walked in passes of `block` tiles; V and M of a pass live in the caller's scratch.  Measured on
// B200, passes small enough to keep V + M inside the 126 MB L2 lose more to launch gaps and under-filled
// single-wave kernels than they save in HBM traffic (VGG-16, N = 256: 29.3 ms with 48 MB passes, 23.9 ms
// with one pass per layer), so the default is one pass per layer up to a 16 GB scratch budget.
// WINOCONV_BLOCK_MB / WINOCONV_WHOLE_MB override the pass budget / the whole-layer limit (read once).
unsigned long long env_mb(const char *name, unsigned long long dflt_mb) {
  const char *v = getenv(name);
  const long long mb = (v && *v) ? atoll(v) : 0;
  return (mb > 0 ? (unsigned long long)mb : dflt_mb) << 20;
}
unsigned long long block_bytes_target() { static const unsigned long long v = env_mb("WINOCONV_BLOCK_MB", 16384); return v; }
unsigned long long whole_bytes_limit() { static const unsigned long long v = env_mb("WINOCONV_WHOLE_MB", 16384); return v; }

int build_plan(const winoconv_desc_t *d, Plan *plan) {
  if (!d || !plan) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "null descriptor");
  if (d->ndim != 2 && d->ndim != 3) return fail(WINOCONV_ERR_UNSUPPORTED, "ndim must be 2 or 3");
  if (d->batch <= 0 || d->c_in <= 0 || d->k_out <= 0) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "batch, c_in and k_out must be positive");
  if (d->dtype < WINOCONV_F32 || d->dtype > WINOCONV_BF16) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "bad dtype");
  if (d->weight_layout != WINOCONV_W_KCRS && d->weight_layout != WINOCONV_W_RSCK) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "bad weight_layout");
  int pdt = d->product_dtype;
  if (pdt != WINOCONV_F32 && pdt != d->dtype) return fail(WINOCONV_ERR_UNSUPPORTED, "product_dtype must be F32 or equal to dtype");
  for (int i = 0; i < 3; ++i) {
    const bool unused = (d->ndim == 2 && i == 0);
    if (unused) {
      if (d->in_size[0] > 1 || d->ker_size[0] > 1 || d->stride[0] > 1 || d->pad[0] != 0)
        return fail(WINOCONV_ERR_INVALID_ARGUMENT, "ndim = 2 needs depth extent, kernel, stride <= 1 and pad 0");
      continue;
    }
    if (d->in_size[i] <= 0) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "input extents must be positive");
    if (d->ker_size[i] < 1 || d->ker_size[i] > 10) return fail(WINOCONV_ERR_UNSUPPORTED, "kernel extents must be 1..10");
    if (d->stride[i] != 1 && d->stride[i] != 2) return fail(WINOCONV_ERR_UNSUPPORTED, "stride must be 1 or 2");
    if (d->pad[i] < 0 || d->pad[i] > 64) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "bad padding");
    if (d->in_size[i] + 2 * d->pad[i] < d->ker_size[i]) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "kernel larger than the padded input");
  }
  Geom &g = plan->g;
  std::memset(&g, 0, sizeof(g));
  std::memset(&plan->info, 0, sizeof(plan->info));
  g.N = d->batch; g.C = d->c_in; g.K = d->k_out; g.Cp = (d->c_in + 7) / 8 * 8;
  int in[3], ks[3], st[3], pd[3];
  for (int i = 0; i < 3; ++i) {
    const bool unused = (d->ndim == 2 && i == 0);
    in[i] = unused ? 1 : d->in_size[i];
    ks[i] = unused ? 1 : d->ker_size[i];
    st[i] = unused ? 1 : d->stride[i];
    pd[i] = unused ? 0 : d->pad[i];
  }
  // F(4x4,3x3): 2-D, 3x3, stride 1.  With tile_m = 0 it is chosen where the staged flow runs anyway (fp32, the
  // SIMT engine, 16-bit products, algo = STAGED); a 16-bit layer that one of the single-kernel paths can take gets
  // 2-wide tiles instead: measured on B200 the row-piece kernel runs the 256 -> 256 layer at 28 x 28, N = 32 in
  // 35 us against 58 us for staged F(4x4,3x3), and its fp16 error is four times smaller.
  const bool f43_ok = ks[0] == 1 && in[0] == 1 && ks[1] == 3 && ks[2] == 3 && st[1] == 1 && st[2] == 1;
  const bool single_kernel_candidate = d->dtype != WINOCONV_F32 && d->algo != WINOCONV_ALGO_STAGED &&
                                       d->gemm_engine != WINOCONV_GEMM_SIMT && d->product_dtype == WINOCONV_F32;
  // Where F(4x4,3x3) pays for its intermediates: at 512 -> 512 channels the contraction outweighs the V and M traffic,
  // and with the tiles covering the output exactly and enough of them to fill the GPU the staged flow beats the
  // row-piece kernel (measured on B200, 512 -> 512 at 28 x 28, N = 256: 0.60 ms against 0.70 ms; at 14 x 14, where 4-wide
  // tiles cover 16 x 16, 0.23 against 0.18 ms; 256 -> 256 at 56 x 56: 1.03 against 0.69 ms).  AUTO takes it there, within
  // the same 2e-2 bound (E_B 1.2e-2 against 2.8e-3).  WINOCONV_AUTO_F43=0 keeps the row-piece kernel everywhere.
  static const int auto_f43_env = [] { const char *v = getenv("WINOCONV_AUTO_F43"); return v && *v ? atoi(v) : 1; }();
  bool f43_wins = false;
  if (f43_ok && single_kernel_candidate && d->algo == WINOCONV_ALGO_AUTO && d->tile_m == 0 && auto_f43_env != 0 &&
      d->gemm_engine != WINOCONV_GEMM_SIMT && d->c_in >= 512 && d->k_out >= 512 && d->c_in % 8 == 0 && d->k_out % 8 == 0) {
    const int oh = in[1] + 2 * pd[1] - 2, ow = in[2] + 2 * pd[2] - 2;
    f43_wins = oh > 0 && ow > 0 && oh % 4 == 0 && ow % 4 == 0 && (long long)d->batch * (oh / 4) * (ow / 4) >= 4096;
  }
  int tile_m = d->tile_m;
  if (tile_m == 0) tile_m = (f43_ok && (!single_kernel_candidate || f43_wins)) ? 4 : 2;
  if (tile_m != 2 && tile_m != 4 && tile_m != 6) return fail(WINOCONV_ERR_UNSUPPORTED, "tile_m must be 0, 2, 4 or 6");
  if (tile_m == 4 && !f43_ok) return fail(WINOCONV_ERR_UNSUPPORTED, "tile_m = 4 is F(4x4,3x3): 2-D, 3x3 kernel, stride 1 only");
  if (tile_m == 6 && !f43_ok) return fail(WINOCONV_ERR_UNSUPPORTED, "tile_m = 6 is F(6x6,3x3): 2-D, 3x3 kernel, stride 1 only");
  // F(6x6,3x3) with 16-bit or single-tf32 operands sits at 5e-2 of the output scale (measured), beyond the 2e-2 bound
  if (tile_m == 6 && (d->dtype != WINOCONV_F32 || d->gemm_engine == WINOCONV_GEMM_TF32))
    return fail(WINOCONV_ERR_UNSUPPORTED, "tile_m = 6 (F(6x6,3x3)) takes f32 operands with fp32-class products (SIMT or TF32X3 engine)");
  int m[3], out[3], nt[3];
  // A depth of one tap at stride 1 (every 2-D conv) is not tiled: no dummy F(2,1) along depth, which is
  // what doubles the positions of every 2-D call in the reference (dwm.py:117).
  m[0] = (ks[0] == 1 && st[0] == 1) ? 1 : 2;
  m[1] = tile_m; m[2] = tile_m;
  if (m[0] == 2 && tile_m != 2) return fail(WINOCONV_ERR_UNSUPPORTED, "tile_m = 4 or 6 with a depth kernel");
  for (int i = 0; i < 3; ++i) {
    out[i] = (in[i] + 2 * pd[i] - ks[i]) / st[i] + 1;
    nt[i] = (out[i] + m[i] - 1) / m[i];
  }
  g.D = in[0]; g.H = in[1]; g.W = in[2];
  g.oD = out[0]; g.oH = out[1]; g.oW = out[2];
  g.nD = nt[0]; g.nH = nt[1]; g.nW = nt[2];
  g.mD = m[0]; g.mH = m[1]; g.mW = m[2];
  g.sD = st[0]; g.sH = st[1]; g.sW = st[2];
  g.pD = pd[0]; g.pH = pd[1]; g.pW = pd[2];
  g.kD = ks[0]; g.kH = ks[1]; g.kW = ks[2];
  g.epilogue = d->epilogue;
  g.weight_layout = d->weight_layout;
  g.yD = g.oD; g.yH = g.oH; g.yW = g.oW;
  if (d->epilogue & ~(WINOCONV_EPI_BIAS | WINOCONV_EPI_RELU | WINOCONV_EPI_POOL2)) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "unknown epilogue bits");
  if (d->epilogue & WINOCONV_EPI_POOL2) {
    if (m[0] != 1 || g.oD != 1) return fail(WINOCONV_ERR_UNSUPPORTED, "POOL2 is for 2-D convolutions");
    if (g.oH < 2 || g.oW < 2) return fail(WINOCONV_ERR_UNSUPPORTED, "POOL2 needs at least a 2x2 output");
    g.yH = g.oH / 2; g.yW = g.oW / 2;
  }
  // pieces: per dimension every (polyphase part, cut) pair; the product over dimensions, depth slowest
  std::vector<DimPiece> per_dim[3];
  std::vector<std::pair<int, int>> cuts;
  for (int i = 0; i < 3; ++i) {
    for (int phase = 0; phase < st[i]; ++phase) {
      const int taps = (ks[i] - phase + st[i] - 1) / st[i];
      if (taps <= 0) continue;
      dwm_cuts(taps, cuts);
      for (auto &c : cuts) per_dim[i].push_back({phase, c.first, c.second});
    }
  }
  const size_t n_pieces = per_dim[0].size() * per_dim[1].size() * per_dim[2].size();
  if (n_pieces > WINOCONV_MAX_PIECES) return fail(WINOCONV_ERR_UNSUPPORTED, "kernel decomposes into more than 64 pieces");
  int pos = 0, np = 0;
  for (auto &a : per_dim[0]) for (auto &b : per_dim[1]) for (auto &c : per_dim[2]) {
    Piece &p = g.pieces[np++];
    const DimPiece *dp[3] = {&a, &b, &c};
    int n_pos = 1;
    for (int i = 0; i < 3; ++i) {
      p.phase[i] = (int8_t)dp[i]->phase; p.start[i] = (int8_t)dp[i]->start; p.r[i] = (int8_t)dp[i]->r;
      n_pos *= (m[i] + dp[i]->r - 1);
    }
    p.type = (int8_t)((a.r - 1) * 9 + (b.r - 1) * 3 + (c.r - 1));
    p.pos_base = (int16_t)pos; p.n_pos = (int16_t)n_pos;
    pos += n_pos;
  }
  g.n_pieces = np; g.positions = pos;
  g.T = (long long)g.N * g.nD * g.nH * g.nW;

  int engine = d->gemm_engine;
  // f32: three tf32 tensor-core products of a hi / lo split hold the fp32 tolerance (measured E_B 2.4e-6 on the
  // 64 -> 64 56 x 56 layer, against 1.8e-6 for fp32 FMA and 3.1e-3 for a single tf32 product) and run the batched GEMM
  // of that layer in 23 us against 34 us for the FMA kernel.
  if (engine == WINOCONV_GEMM_AUTO) engine = (d->dtype == WINOCONV_F32) ? WINOCONV_GEMM_TF32X3 : WINOCONV_GEMM_TCGEN05;
  if (engine < WINOCONV_GEMM_SIMT || engine > WINOCONV_GEMM_TF32X3) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "bad gemm_engine");
  if (engine == WINOCONV_GEMM_TCGEN05 && d->dtype == WINOCONV_F32) return fail(WINOCONV_ERR_UNSUPPORTED, "the f16 tcgen05 GEMM takes f16 / bf16; f32 runs on SIMT, TF32 or TF32X3");
  if ((engine == WINOCONV_GEMM_TF32 || engine == WINOCONV_GEMM_TF32X3) && d->dtype != WINOCONV_F32)
    return fail(WINOCONV_ERR_UNSUPPORTED, "the tf32 GEMM engines take f32 inputs");
  plan->dtype = d->dtype; plan->product_dtype = pdt; plan->engine = engine;

  // Algorithm: the fused single-kernel path covers 16-bit F(2x2,3x3)-piece convolutions; everything else
  // (fp32, F(4x4,3x3), the SIMT engine) runs as input transform -> batched GEMM -> output transform.
  const bool fused_ok = d->dtype != WINOCONV_F32 && tile_m == 2 && engine == WINOCONV_GEMM_TCGEN05 &&
                        pdt == WINOCONV_F32;
  if (d->algo < WINOCONV_ALGO_AUTO || d->algo > WINOCONV_ALGO_ROW) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "bad algo");
  plan->row = false;
  if (fused_ok && (d->algo == WINOCONV_ALGO_AUTO || d->algo == WINOCONV_ALGO_ROW)) {
    RowDesc &r = plan->rd;
    std::memset(&r, 0, sizeof(r));
    r.N = g.N; r.K = g.K; r.oD = g.oD; r.oH = g.oH; r.oW = g.oW; r.yH = g.yH; r.yW = g.yW;
    r.epilogue = g.epilogue; r.weight_layout = g.weight_layout;
    r.C0 = g.C; r.D0 = g.D; r.H0 = g.H; r.W0 = g.W; r.pD0 = g.pD; r.pH0 = g.pH; r.pW0 = g.pW;
    r.kD0 = g.kD; r.kH0 = g.kH; r.kW0 = g.kW;
    const bool strides_ok = (g.sD == 1 || g.sD == 2) && (g.sH == 1 || g.sH == 2) && (g.sW == 1 || g.sW == 2);
    r.fD = g.sD; r.fH = g.sH; r.fW = g.sW;
    r.phases = strides_ok ? g.sD * g.sH * g.sW : 0;
    if (r.phases == 1) {
      r.C = g.C; r.D = g.D; r.H = g.H; r.W = g.W; r.pD = g.pD; r.pH = g.pH; r.pW = g.pW; r.kD = g.kD; r.kH = g.kH; r.kW = g.kW;
    } else if (r.phases > 1) {
      // stride 2: y[o] = sum_t x[2 o + t] w[t] with t = 2 a + phase is a stride-1 convolution over the two
      // polyphase parts of x taken as extra channels, kernel ceil(k / 2), input extent out + k' - 1, no padding
      r.C = r.phases * g.C;
      r.kD = (g.kD + g.sD - 1) / g.sD; r.kH = (g.kH + g.sH - 1) / g.sH; r.kW = (g.kW + g.sW - 1) / g.sW;
      r.D = g.oD + r.kD - 1; r.H = g.oH + r.kH - 1; r.W = g.oW + r.kW - 1;
      r.pD = r.pH = r.pW = 0;
    }
    r.sD = r.sH = r.sW = 1;
    plan->row = r.phases >= 1 && rowfused_plan(r, &plan->rp);
  }
  if (d->algo == WINOCONV_ALGO_ROW && !plan->row)
    return fail(WINOCONV_ERR_UNSUPPORTED, "the row-piece kernel needs f16 / bf16, tile_m = 2, strides of 1 or 2, a patch and slab set that fit shared memory, the tcgen05 engine and fp32 products");
  if (d->algo == WINOCONV_ALGO_FUSED && !fused_ok)
    return fail(WINOCONV_ERR_UNSUPPORTED, "the fused path needs f16 / bf16, tile_m = 2 (or 0 with a kernel other than 2-D 3x3 stride 1), the tcgen05 engine and fp32 products");
  plan->fused = fused_ok && !plan->row && d->algo != WINOCONV_ALGO_STAGED && d->algo != WINOCONV_ALGO_ROW;
  if (plan->fused) {
    FGeom &f = plan->fg;
    std::memset(&f, 0, sizeof(f));
    f.N = g.N; f.C = g.C; f.K = g.K; f.Cp = g.Cp;
    f.D = g.D; f.H = g.H; f.W = g.W; f.oD = g.oD; f.oH = g.oH; f.oW = g.oW; f.yH = g.yH; f.yW = g.yW;
    f.nH = (g.oH + 1) / 2; f.nW = (g.oW + 1) / 2;
    f.sD = g.sD; f.sH = g.sH; f.sW = g.sW; f.pD = g.pD; f.pH = g.pH; f.pW = g.pW; f.kD = g.kD; f.kH = g.kH; f.kW = g.kW;
    f.epilogue = g.epilogue; f.weight_layout = g.weight_layout;
    f.T = (long long)g.N * g.oD * f.nH * f.nW;
    // windows per dimension: every polyphase part cut into 3-tap windows (the last one zero padded)
    std::vector<std::pair<int, int>> win[2];
    for (int i = 1; i < 3; ++i)
      for (int phase = 0; phase < st[i]; ++phase) {
        const int taps = (ks[i] - phase + st[i] - 1) / st[i];
        for (int s0 = 0; s0 < taps; s0 += 3) win[i - 1].push_back({phase, s0});
      }
    const size_t np_f = (size_t)ks[0] * win[0].size() * win[1].size();
    if (np_f > (size_t)kMaxFusedPieces) {
      if (d->algo == WINOCONV_ALGO_FUSED) return fail(WINOCONV_ERR_UNSUPPORTED, "kernel decomposes into more than 160 windows");
      plan->fused = false;
    } else {
      int q = 0;
      for (int kd = 0; kd < ks[0]; ++kd) for (auto &a : win[0]) for (auto &b : win[1]) {
        FPiece &fp = f.pieces[q++];
        fp.kd = (int8_t)kd; fp.ph_h = (int8_t)a.first; fp.st_h = (int8_t)a.second; fp.ph_w = (int8_t)b.first; fp.st_w = (int8_t)b.second;
      }
      f.P = q; f.R = q * g.Cp;
    }
  }

  winoconv_plan_info_t &I = plan->info;
  for (int i = 0; i < 3; ++i) { I.conv_out_size[i] = out[i]; I.tile_m[i] = m[i]; I.tiles_per_dim[i] = nt[i]; }
  I.out_size[0] = g.yD; I.out_size[1] = g.yH; I.out_size[2] = g.yW;
  I.n_pieces = np; I.positions = pos; I.c_pad = g.Cp; I.gemm_engine = engine; I.tiles = g.T;
  const unsigned long long esz = dtype_size(d->dtype), psz = dtype_size(pdt);
  I.filter_bytes = (unsigned long long)pos * g.K * g.Cp * esz;
  const unsigned long long v_tile = (unsigned long long)pos * g.Cp * esz, m_tile = (unsigned long long)pos * g.K * psz;
  long long block = (long long)(block_bytes_target() / (v_tile + m_tile));
  block = std::max(128LL, block / 128 * 128);
  if ((unsigned long long)g.T * (v_tile + m_tile) <= whole_bytes_limit() || block > g.T) block = g.T;
  I.block_tiles = block;
  I.input_ws_bytes = v_tile * (unsigned long long)block;
  I.product_ws_bytes = m_tile * (unsigned long long)block;
  const long long min_block = std::min<long long>(128, g.T);
  I.input_ws_bytes_min = v_tile * (unsigned long long)min_block;
  I.product_ws_bytes_min = m_tile * (unsigned long long)min_block;
  I.algo = plan->fused ? WINOCONV_ALGO_FUSED : WINOCONV_ALGO_STAGED;
  if (plan->fused) {
    const FGeom &f = plan->fg;
    I.tile_m[0] = 1; I.tiles_per_dim[0] = g.oD; I.tiles_per_dim[1] = f.nH; I.tiles_per_dim[2] = f.nW;
    I.n_pieces = f.P; I.positions = 16; I.tiles = f.T;
    I.filter_bytes = 16ull * g.K * f.R * esz;
    I.input_ws_bytes = I.product_ws_bytes = I.input_ws_bytes_min = I.product_ws_bytes_min = 0;
    I.block_tiles = f.T;
  }
  if (plan->row) {
    const RowPlan &rp = plan->rp;
    I.algo = WINOCONV_ALGO_ROW;
    I.tile_m[0] = 1; I.tile_m[1] = 1; I.tile_m[2] = 2;
    I.tiles_per_dim[0] = g.oD; I.tiles_per_dim[1] = g.oH; I.tiles_per_dim[2] = (g.oW + 1) / 2;
    I.n_pieces = plan->rd.kD * plan->rd.kH * rp.PW; I.positions = 4;
    I.tiles = (long long)g.N * g.oD * g.oH * ((g.oW + 1) / 2);
    I.filter_bytes = (unsigned long long)rp.filter_elems * esz;
    // scratch only to zero-pad the channels of x to a multiple of 8 (TMA needs 16-byte pixel strides), or to hold
    // the input with its stride-2 phases gathered into channels
    const RowDesc &rd = plan->rd;
    I.input_ws_bytes = I.input_ws_bytes_min =
        ((rd.phases > 1 || rp.Cp != g.C) && !rp.raw_c && !rp.s2_chunks) ? (unsigned long long)rd.N * rd.D * rd.H * rd.W * rp.Cp * esz : 0ull;
    I.product_ws_bytes = I.product_ws_bytes_min = 0;
    I.block_tiles = I.tiles;
  }
  I.direct_flops = 2.0 * g.N * g.K * g.C * (double)ks[0] * ks[1] * ks[2] * (double)out[0] * out[1] * out[2];
  I.gemm_flops = plan->fused ? 2.0 * 16 * (double)plan->fg.T * plan->fg.P * g.C * g.K : 2.0 * pos * (double)g.T * g.C * g.K;
  if (plan->row) I.gemm_flops = 2.0 * 4 * (double)I.tiles * I.n_pieces * plan->rd.C * g.K;
  I.algorithmic_bytes = (double)esz * ((double)g.N * g.D * g.H * g.W * g.C + (double)g.K * g.C * ks[0] * ks[1] * ks[2] +
                                       (double)g.N * g.yD * g.yH * g.yW * g.K);
  return WINOCONV_OK;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int run_gemm(int dtype, int pdt, int engine, int positions, long long tiles, int c_pad, int k_out, const void *v,
             const void *u, void *m, cudaStream_t s) {
  if (engine == WINOCONV_GEMM_TCGEN05) {
    const char *detail = "";
    cudaError_t e = launch_gemm_tcgen05(dtype, pdt, positions, tiles, c_pad, k_out, v, u, m, s, &detail);
    if (e != cudaSuccess) return cuda_fail(e, "tcgen05 GEMM launch", detail);
    return WINOCONV_OK;
  }
  if (engine == WINOCONV_GEMM_TF32 || engine == WINOCONV_GEMM_TF32X3) {
    const char *detail = "";
    cudaError_t e = launch_gemm_tf32(engine == WINOCONV_GEMM_TF32X3 ? 1 : 0, positions, tiles, c_pad, k_out, v, u, m, s, &detail);
    if (e != cudaSuccess) return cuda_fail(e, "tf32 GEMM launch", detail);
    return WINOCONV_OK;
  }
  cudaError_t e = launch_gemm_simt(dtype, pdt, positions, tiles, c_pad, k_out, v, u, m, s);
  if (e != cudaSuccess) return cuda_fail(e, "SIMT GEMM launch");
  return WINOCONV_OK;
}

}  // namespace
}  // namespace wino

using namespace wino;

extern "C" {

int winoconv_abi_version(void) { return WINOCONV_ABI_VERSION; }

const char *winoconv_status_string(int status) {
  switch (status) {
    case WINOCONV_OK: return "ok";
    case WINOCONV_ERR_INVALID_ARGUMENT: return "invalid argument";
    case WINOCONV_ERR_UNSUPPORTED: return "unsupported configuration";
    case WINOCONV_ERR_WORKSPACE: return "scratch buffer too small";
    case WINOCONV_ERR_CUDA: return "CUDA error";
    case WINOCONV_ERR_TIMEOUT: return "device-side wait timed out";
    case WINOCONV_ERR_NO_DEVICE: return "no sm_100 device";
    default: return "unknown status";
  }
}

size_t winoconv_last_error(char *buf, size_t buf_size) {
  if (buf && buf_size) {
    const size_t n = std::min(buf_size - 1, t_last_error.size());
    std::memcpy(buf, t_last_error.data(), n);
    buf[n] = '\0';
  }
  return t_last_error.size();
}

int winoconv_device_check(void) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { cudaGetLastError(); return fail(WINOCONV_ERR_NO_DEVICE, std::string("cudaGetDevice: ") + cudaGetErrorString(e)); }
  int major = 0;
  e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (e != cudaSuccess) { cudaGetLastError(); return fail(WINOCONV_ERR_NO_DEVICE, std::string("cudaDeviceGetAttribute: ") + cudaGetErrorString(e)); }
  if (major != 10) return fail(WINOCONV_ERR_NO_DEVICE, "the kernels are built for sm_100a only; current device has compute capability major " + std::to_string(major));
  return WINOCONV_OK;
}

int winoconv_plan(const winoconv_desc_t *desc, winoconv_plan_info_t *info) {
  if (!info) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "null info");
  Plan plan;
  const int st = build_plan(desc, &plan);
  if (st != WINOCONV_OK) return st;
  *info = plan.info;
  return WINOCONV_OK;
}

int winoconv_plan_pieces(const winoconv_desc_t *desc, int32_t *pieces, int32_t max_pieces, int32_t *n_pieces) {
  if (!pieces || !n_pieces) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "null output");
  Plan plan;
  const int st = build_plan(desc, &plan);
  if (st != WINOCONV_OK) return st;
  if (plan.g.n_pieces > max_pieces) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "pieces array too small");
  for (int i = 0; i < plan.g.n_pieces; ++i)
    for (int j = 0; j < 3; ++j) {
      pieces[i * 9 + j] = plan.g.pieces[i].phase[j];
      pieces[i * 9 + 3 + j] = plan.g.pieces[i].start[j];
      pieces[i * 9 + 6 + j] = plan.g.pieces[i].r[j];
    }
  *n_pieces = plan.g.n_pieces;
  return WINOCONV_OK;
}

int winoconv_filter_transform(const winoconv_desc_t *desc, const void *weights, void *u, void *stream) {
  Plan plan;
  int st = build_plan(desc, &plan);
  if (st != WINOCONV_OK) return st;
  if (!weights || !u) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "null weights or u");
  if ((st = winoconv_device_check()) != WINOCONV_OK) return st;
  cudaError_t e = plan.row     ? launch_rowfused_filter_transform(plan.rd, plan.rp, plan.dtype, weights, u, (cudaStream_t)stream)
                  : plan.fused ? launch_fused_filter_transform(plan.fg, plan.dtype, weights, u, (cudaStream_t)stream)
                               : launch_filter_transform(plan.g, plan.dtype, weights, u, (cudaStream_t)stream);
  if (e != cudaSuccess) return cuda_fail(e, "filter transform launch");
  return WINOCONV_OK;
}

static int forward_impl(const winoconv_desc_t *desc, const void *x, const void *u, const void *bias, void *y,
                        void *v_ws, size_t v_ws_bytes, void *m_ws, size_t m_ws_bytes, void *stream, float *stage_ms,
                        int32_t *launches) {
  Plan plan;
  int st = build_plan(desc, &plan);
  if (st != WINOCONV_OK) return st;
  if (!x || !u || !y) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "null tensor pointer");
  if ((desc->epilogue & WINOCONV_EPI_BIAS) && !bias) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "EPI_BIAS set but bias is null");
  if (!aligned16(x) || !aligned16(u) || !aligned16(y)) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "tensors must be 16-byte aligned");
  if (plan.row && plan.info.input_ws_bytes_min > 0) {
    if (!v_ws || !aligned16(v_ws)) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "channel-padding scratch (v_ws) must be a 16-byte aligned pointer");
    if (v_ws_bytes < plan.info.input_ws_bytes_min)
      return fail(WINOCONV_ERR_WORKSPACE, "v_ws holds " + std::to_string(v_ws_bytes) + " bytes; padding the input channels needs " +
                                              std::to_string(plan.info.input_ws_bytes_min));
  }
  if (plan.fused || plan.row) {   // one kernel, no V / M scratch
    if ((st = winoconv_device_check()) != WINOCONV_OK) return st;
    cudaStream_t fs = (cudaStream_t)stream;
    struct EventPair {   // destroyed on every way out
      cudaEvent_t a = nullptr, b = nullptr;
      ~EventPair() { if (a) cudaEventDestroy(a); if (b) cudaEventDestroy(b); }
    } ev;
    cudaEvent_t &e0 = ev.a, &e1 = ev.b;
    cudaError_t e = cudaSuccess;
    if (stage_ms) {
      e = cudaEventCreate(&e0);
      if (e == cudaSuccess) e = cudaEventCreate(&e1);
      if (e == cudaSuccess) e = cudaEventRecord(e0, fs);
      if (e != cudaSuccess) return cuda_fail(e, "event record");
    }
    const char *detail = "";
    e = plan.row ? launch_rowfused_forward(plan.rd, plan.rp, plan.dtype, x, u, bias, y, v_ws, fs, &detail)
                 : launch_fused_forward(plan.fg, plan.dtype, x, u, bias, y, fs, &detail);
    if (e != cudaSuccess) return cuda_fail(e, "fused forward launch", detail);
    if (launches) *launches = (plan.row && plan.info.input_ws_bytes_min > 0) ? 2 : 1;
    if (stage_ms) {
      stage_ms[0] = stage_ms[2] = 0.f;
      e = cudaEventRecord(e1, fs);
      if (e == cudaSuccess) e = cudaEventSynchronize(e1);
      if (e == cudaSuccess) e = cudaEventElapsedTime(&stage_ms[1], e0, e1);
      if (e != cudaSuccess) return cuda_fail(e, "event timing");
    }
    return WINOCONV_OK;
  }
  if (!v_ws || !m_ws) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "null scratch pointer");
  if (!aligned16(v_ws) || !aligned16(m_ws)) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "scratch must be 16-byte aligned");
  if ((st = winoconv_device_check()) != WINOCONV_OK) return st;
  const Geom &g = plan.g;
  const unsigned long long esz = dtype_size(plan.dtype), psz = dtype_size(plan.product_dtype);
  const unsigned long long v_tile = (unsigned long long)g.positions * g.Cp * esz, m_tile = (unsigned long long)g.positions * g.K * psz;
  long long block = (long long)std::min<unsigned long long>(v_ws_bytes / v_tile, m_ws_bytes / m_tile);
  block = std::min(block, (long long)plan.info.block_tiles);  // never exceed the cache-sized block
  if (block < std::min<long long>(128, g.T))
    return fail(WINOCONV_ERR_WORKSPACE, "scratch holds " + std::to_string(block) + " tiles; need at least " +
                                            std::to_string(std::min<long long>(128, g.T)) + " (see winoconv_plan)");
  if (block < g.T) block = block / 128 * 128;
  cudaStream_t s = (cudaStream_t)stream;
  std::vector<cudaEvent_t> ev;  // four events per pass when stage times are wanted
  auto mark = [&]() -> cudaError_t {
    if (!stage_ms) return cudaSuccess;
    cudaEvent_t e;
    cudaError_t r = cudaEventCreate(&e);
    if (r != cudaSuccess) return r;
    ev.push_back(e);
    return cudaEventRecord(e, s);
  };
  int n_launch = 0;
  int result = WINOCONV_OK;
  for (long long t0 = 0; t0 < g.T && result == WINOCONV_OK; t0 += block) {
    const int n = (int)std::min<long long>(block, g.T - t0);
    cudaError_t e = mark();
    if (e == cudaSuccess) {
      static const int xt_env = [] { const char *v = getenv("WINOCONV_XF_TMA"); return v && *v ? atoi(v) : 1; }();
      if (xt_env != 0 && input_f43_tma_applies(g, plan.dtype, x, t0, n)) {
        const char *detail = "";
        e = launch_input_f43_tma(g, plan.dtype, x, v_ws, s, &detail);
        if (e != cudaSuccess) { result = cuda_fail(e, detail && *detail ? detail : "input transform launch"); break; }
      } else {
        e = launch_input_transform(g, plan.dtype, x, v_ws, t0, n, s);
      }
    }
    if (e != cudaSuccess) { result = cuda_fail(e, "input transform launch"); break; }
    if ((e = mark()) != cudaSuccess) { result = cuda_fail(e, "event record"); break; }
    result = run_gemm(plan.dtype, plan.product_dtype, plan.engine, g.positions, n, g.Cp, g.K, v_ws, u, m_ws, s);
    if (result != WINOCONV_OK) break;
    if ((e = mark()) != cudaSuccess) { result = cuda_fail(e, "event record"); break; }
    {
      static const int yt_env = [] { const char *v = getenv("WINOCONV_XF_TMA"); return v && *v ? atoi(v) : 1; }();
      if (yt_env != 0 && output_f43_tma_applies(g, plan.dtype, plan.product_dtype, m_ws, t0, n)) {
        const char *detail = "";
        e = launch_output_f43_tma(g, plan.dtype, plan.product_dtype, m_ws, y, bias, s, &detail);
        if (e != cudaSuccess) { result = cuda_fail(e, detail && *detail ? detail : "output transform launch"); break; }
      } else {
        e = launch_output_transform(g, plan.dtype, plan.product_dtype, m_ws, y, bias, t0, n, s);
      }
    }
    if (e != cudaSuccess) { result = cuda_fail(e, "output transform launch"); break; }
    if ((e = mark()) != cudaSuccess) { result = cuda_fail(e, "event record"); break; }
    n_launch += 3;
  }
  if (launches) *launches = n_launch;
  if (stage_ms) {
    stage_ms[0] = stage_ms[1] = stage_ms[2] = 0.f;
    if (result == WINOCONV_OK) {
      cudaError_t e = cudaStreamSynchronize(s);
      if (e != cudaSuccess) result = cuda_fail(e, "stream synchronize");
      for (size_t i = 0; result == WINOCONV_OK && i + 3 < ev.size(); i += 4)
        for (int j = 0; j < 3; ++j) {
          float ms = 0.f;
          if ((e = cudaEventElapsedTime(&ms, ev[i + j], ev[i + j + 1])) != cudaSuccess) { result = cuda_fail(e, "event elapsed"); break; }
          stage_ms[j] += ms;
        }
    }
    for (cudaEvent_t e : ev) cudaEventDestroy(e);
  }
  return result;
}

int winoconv_forward(const winoconv_desc_t *desc, const void *x, const void *u, const void *bias, void *y, void *v_ws,
                     size_t v_ws_bytes, void *m_ws, size_t m_ws_bytes, void *stream) {
  return forward_impl(desc, x, u, bias, y, v_ws, v_ws_bytes, m_ws, m_ws_bytes, stream, nullptr, nullptr);
}

int winoconv_forward_timed(const winoconv_desc_t *desc, const void *x, const void *u, const void *bias, void *y,
                           void *v_ws, size_t v_ws_bytes, void *m_ws, size_t m_ws_bytes, void *stream,
                           float *stage_ms, int32_t *launches) {
  if (!stage_ms) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "null stage_ms");
  return forward_impl(desc, x, u, bias, y, v_ws, v_ws_bytes, m_ws, m_ws_bytes, stream, stage_ms, launches);
}

// ---- scratch that is part of the library image (winoconv_forward_static) ---------------------------------
// In host code the name below is only a handle for cudaGetSymbolAddress; the address kernels may use is
// looked up once per device and kept in g_static_scratch_addr.  The cache (like the launch-attribute caches of the
// kernels) is keyed by device ordinal and assumes the device's primary context lives as long as the process: a
// program that calls cudaDeviceReset must not use the library afterwards.
static __device__ __align__(256) unsigned char g_static_scratch[WINOCONV_STATIC_SCRATCH_BYTES];
static void *g_static_scratch_addr[64] = {};
static std::mutex g_static_scratch_mu;

static int static_scratch_of_current_device(unsigned char **out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= 64) return fail(WINOCONV_ERR_UNSUPPORTED, "device ordinal beyond 63");
  std::lock_guard<std::mutex> lock(g_static_scratch_mu);
  if (!g_static_scratch_addr[dev]) {
    void *p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
    g_static_scratch_addr[dev] = p;
  }
  *out = static_cast<unsigned char *>(g_static_scratch_addr[dev]);
  return WINOCONV_OK;
}

int winoconv_forward_static(const winoconv_desc_t *desc, const void *x, const void *u, const void *bias, void *y,
                            void *stream) {
  Plan plan;
  int st = build_plan(desc, &plan);
  if (st != WINOCONV_OK) return st;
  if ((st = winoconv_device_check()) != WINOCONV_OK) return st;
  const winoconv_plan_info_t &I = plan.info;
  if (plan.fused || (plan.row && I.input_ws_bytes_min == 0))
    return forward_impl(desc, x, u, bias, y, nullptr, 0, nullptr, 0, stream, nullptr, nullptr);
  if (plan.row) {   // the built-in array serves as the channel-padding buffer
    if (I.input_ws_bytes_min > WINOCONV_STATIC_SCRATCH_BYTES)
      return fail(WINOCONV_ERR_WORKSPACE, "the row kernel's channel-padded / phase-gathered copy of the input needs " +
                                              std::to_string(I.input_ws_bytes_min) + " bytes; the built-in array holds " +
                                              std::to_string(WINOCONV_STATIC_SCRATCH_BYTES) +
                                              " (plan and filter-transform this layer with algo = WINOCONV_ALGO_FUSED, which needs"
                                              " no scratch, or WINOCONV_ALGO_STAGED, and call again)");
    unsigned char *pad = nullptr;
    if ((st = static_scratch_of_current_device(&pad)) != WINOCONV_OK) return st;
    return forward_impl(desc, x, u, bias, y, pad, WINOCONV_STATIC_SCRATCH_BYTES, nullptr, 0, stream, nullptr, nullptr);
  }
  const unsigned long long tiles_min = (unsigned long long)std::min<long long>(128, I.tiles);
  const unsigned long long v_tile = I.input_ws_bytes_min / tiles_min, m_tile = I.product_ws_bytes_min / tiles_min;
  const unsigned long long usable = WINOCONV_STATIC_SCRATCH_BYTES - 256;  // V is rounded up to the M alignment
  if (tiles_min * (v_tile + m_tile) > usable)
    return fail(WINOCONV_ERR_WORKSPACE, "this layer needs " + std::to_string(tiles_min * (v_tile + m_tile)) +
                                            " bytes of scratch for its smallest pass; the built-in array holds " +
                                            std::to_string(WINOCONV_STATIC_SCRATCH_BYTES) +
                                            " (use winoconv_forward with caller scratch)");
  unsigned long long block = std::min<unsigned long long>(usable / (v_tile + m_tile), (unsigned long long)I.tiles);
  if (block < (unsigned long long)I.tiles) block = block / 128 * 128;
  const size_t v_bytes = (size_t)((block * v_tile + 255) / 256 * 256);
  unsigned char *base = nullptr;
  if ((st = static_scratch_of_current_device(&base)) != WINOCONV_OK) return st;
  return forward_impl(desc, x, u, bias, y, base, v_bytes, base + v_bytes, WINOCONV_STATIC_SCRATCH_BYTES - v_bytes, stream,
                      nullptr, nullptr);
}

int winoconv_gemm_batched(int dtype, int product_dtype, int gemm_engine, int positions, int64_t tiles, int c_pad,
                          int k_out, const void *v, const void *u, void *m, void *stream) {
  if (!v || !u || !m) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "null operand");
  if (positions <= 0 || tiles <= 0 || c_pad <= 0 || k_out <= 0) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "sizes must be positive");
  if (c_pad % 8 != 0) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "c_pad must be a multiple of 8");
  if (dtype < WINOCONV_F32 || dtype > WINOCONV_BF16) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "bad dtype");
  if (product_dtype != WINOCONV_F32 && product_dtype != dtype) return fail(WINOCONV_ERR_UNSUPPORTED, "product_dtype must be F32 or equal to dtype");
  if (!aligned16(v) || !aligned16(u) || !aligned16(m)) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "operands must be 16-byte aligned");
  int engine = gemm_engine;
  if (engine == WINOCONV_GEMM_AUTO) engine = dtype == WINOCONV_F32 ? WINOCONV_GEMM_TF32X3 : WINOCONV_GEMM_TCGEN05;
  if (engine < WINOCONV_GEMM_SIMT || engine > WINOCONV_GEMM_TF32X3) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "bad gemm_engine");
  if (engine == WINOCONV_GEMM_TCGEN05 && dtype == WINOCONV_F32) return fail(WINOCONV_ERR_UNSUPPORTED, "the f16 tcgen05 GEMM takes f16 / bf16");
  if ((engine == WINOCONV_GEMM_TF32 || engine == WINOCONV_GEMM_TF32X3) && (dtype != WINOCONV_F32 || product_dtype != WINOCONV_F32))
    return fail(WINOCONV_ERR_UNSUPPORTED, "the tf32 GEMM engines take f32 operands and write f32 products");
  int st = winoconv_device_check();
  if (st != WINOCONV_OK) return st;
  return run_gemm(dtype, product_dtype, engine, positions, tiles, c_pad, k_out, v, u, m, (cudaStream_t)stream);
}

int winoconv_split(const float *x, float *out, int batch, int d, int h, int w, int c, int block_d, int block_h,
                   int block_w, int out_block_d, int out_block_h, int out_block_w, int n_d, int n_h, int n_w,
                   void *stream) {
  if (!x || !out) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "null tensor");
  if (batch <= 0 || d <= 0 || h <= 0 || w <= 0 || c <= 0 || block_d <= 0 || block_h <= 0 || block_w <= 0 ||
      out_block_d <= 0 || out_block_h <= 0 || out_block_w <= 0 || n_d <= 0 || n_h <= 0 || n_w <= 0)
    return fail(WINOCONV_ERR_INVALID_ARGUMENT, "sizes must be positive");
  if ((size_t)block_d * block_h * block_w * 33 * sizeof(float) > 48 * 1024)
    return fail(WINOCONV_ERR_UNSUPPORTED, "tile volume too large for the split kernel (max 372 elements)");
  int st = winoconv_device_check();
  if (st != WINOCONV_OK) return st;
  cudaError_t e = launch_split(x, out, batch, d, h, w, c, block_d, block_h, block_w, out_block_d, out_block_h,
                               out_block_w, n_d, n_h, n_w, (cudaStream_t)stream);
  if (e != cudaSuccess) return cuda_fail(e, "split launch");
  return WINOCONV_OK;
}

int winoconv_concat(const float *tiles, float *y, int batch, int out_d, int out_h, int out_w, int k, int out_block_d,
                    int out_block_h, int out_block_w, void *stream) {
  if (!tiles || !y) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "null tensor");
  if (batch <= 0 || out_d <= 0 || out_h <= 0 || out_w <= 0 || k <= 0 || out_block_d <= 0 || out_block_h <= 0 || out_block_w <= 0)
    return fail(WINOCONV_ERR_INVALID_ARGUMENT, "sizes must be positive");
  if ((size_t)out_block_d * out_block_h * out_block_w * 33 * sizeof(float) > 48 * 1024)
    return fail(WINOCONV_ERR_UNSUPPORTED, "output block too large for the concat kernel");
  int st = winoconv_device_check();
  if (st != WINOCONV_OK) return st;
  cudaError_t e = launch_concat(tiles, y, batch, out_d, out_h, out_w, k, out_block_d, out_block_h, out_block_w, (cudaStream_t)stream);
  if (e != cudaSuccess) return cuda_fail(e, "concat launch");
  return WINOCONV_OK;
}

int winoconv_add(const float *a, const float *b, float *c, int64_t n, void *stream) {
  if (n < 0) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "negative length");
  if (n == 0) return WINOCONV_OK;
  if (!a || !b || !c) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "null tensor");
  int st = winoconv_device_check();
  if (st != WINOCONV_OK) return st;
  cudaError_t e = launch_add(a, b, c, (long long)n, (cudaStream_t)stream);
  if (e != cudaSuccess) return cuda_fail(e, "add launch");
  return WINOCONV_OK;
}

int winoconv_read_device_error(void *stream, uint32_t *code) {
  if (!code) return fail(WINOCONV_ERR_INVALID_ARGUMENT, "null code");
  unsigned int host = 0, host2 = 0;
  cudaError_t e = read_and_clear_device_error((cudaStream_t)stream, &host);
  unsigned int host3 = 0;
  if (e == cudaSuccess) e = read_and_clear_fused_error((cudaStream_t)stream, &host2);
  if (e == cudaSuccess) e = read_and_clear_row_error((cudaStream_t)stream, &host3);
  if (e != cudaSuccess) return cuda_fail(e, "reading the device error word");
  if (host == 0) host = host2 ? host2 : host3;
  *code = host;
  if (host != 0) return fail(WINOCONV_ERR_TIMEOUT, "a bounded device wait gave up, code 0x" + [&] { char b[16]; snprintf(b, sizeof b, "%x", host); return std::string(b); }());
  return WINOCONV_OK;
}

}  // extern "C"
