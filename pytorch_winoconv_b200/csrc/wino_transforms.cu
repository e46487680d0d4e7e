// Filter, input and output transforms of the Winograd / DWM engine, plus the stand-alone tile
// split / concat and the elementwise add kept for the reference's operator surface.
//
// One thread owns VEC consecutive channels of one tile.  Consecutive threads own consecutive
// channel vectors, then consecutive tiles, so every global access of a warp is a run of whole
// 128-byte lines: channels are innermost in x (NDHWC), in V [position][tile][C], in
// M [position][tile][K] and in y (NDHWK).  The patch of a tile lives in registers; the 2-D/3-D
// transform is applied one axis at a time with the 1-D Cook-Toom kernels of wino_common.cuh.
//
// Reference counterparts: wNorm2WinoTransform / inputNorm2WinoTransform /
// outputWino2NormTransform / outputAggregate (src/split_kernel.cu:14-203) with the unrolled
// arithmetic of src/calculation_kernels.cu; winoSplitKernel(2d) / winoConcatKernel(2d)
// (src/split_and_concat_kernels.cu:9-129); sum (src/add.cu:7-13).
#include "wino_common.cuh"
#include "wino_launch.h"

namespace wino {

// MODE selects the output block per dimension (uniform for a launch):
//   0: (1,2,2)  2-D F(2,r) pieces        1: (2,2,2)  3-D F(2,r) pieces        2: (1,4,4)  2-D F(4x4,3x3)
//   3: (1,6,6)  2-D F(6x6,3x3), fp32 only
template <int MODE> struct ModeM;
template <> struct ModeM<0> { static constexpr int MD = 1, MH = 2, MW = 2; };
template <> struct ModeM<1> { static constexpr int MD = 2, MH = 2, MW = 2; };
template <> struct ModeM<2> { static constexpr int MD = 1, MH = 4, MW = 4; };
template <> struct ModeM<3> { static constexpr int MD = 1, MH = 6, MW = 6; };

// Nested switch over the taps of a piece; BODY(RD, RH, RW) is expanded with literals.
#define WINO_SW_W(RD, RH, BODY)                                   \
  switch (rw) {                                                   \
    case 1: BODY(RD, RH, 1); break;                               \
    case 2: BODY(RD, RH, 2); break;                               \
    default: BODY(RD, RH, 3); break;                              \
  }
#define WINO_SW_H(RD, BODY)                                       \
  switch (rh) {                                                   \
    case 1: WINO_SW_W(RD, 1, BODY) break;                         \
    case 2: WINO_SW_W(RD, 2, BODY) break;                         \
    default: WINO_SW_W(RD, 3, BODY) break;                        \
  }
#define WINO_SW_D(BODY)                                           \
  switch (rd) {                                                   \
    case 1: WINO_SW_H(1, BODY) break;                             \
    case 2: WINO_SW_H(2, BODY) break;                             \
    default: WINO_SW_H(3, BODY) break;                            \
  }

struct TileCoord { int n, td, th, tw; };

// Tile indices fit 32 bits (2^31 tiles would be more outputs than the device holds): unsigned 32-bit divisions, a
// fraction of the instructions of 64-bit ones -- the index arithmetic, not the transform, was most of these kernels.
__device__ __forceinline__ TileCoord decode_tile(const Geom &g, long long t64) {
  unsigned t = (unsigned)t64;
  TileCoord tc;
  unsigned q = t / (unsigned)g.nW; tc.tw = (int)(t - q * (unsigned)g.nW); t = q;
  q = t / (unsigned)g.nH; tc.th = (int)(t - q * (unsigned)g.nH); t = q;
  q = t / (unsigned)g.nD; tc.td = (int)(t - q * (unsigned)g.nD);
  tc.n = (int)q;
  return tc;
}

// ------------------------------------------------------------------------------------------
// input transform:  V[pos][tile][c] = (B^T d B)[pos]
// ------------------------------------------------------------------------------------------
template <typename T, int VEC, int MD, int RD, int MH, int RH, int MW, int RW>
__device__ __forceinline__ void input_piece(const T *__restrict__ x, T *__restrict__ v, const Geom &g,
                                            const Piece &pc, const TileCoord &tc, int c0, long long v_row,
                                            long long v_pos_stride) {
  using XD = Xf<MD, RD>; using XH = Xf<MH, RH>; using XW = Xf<MW, RW>;
  constexpr int AD = XD::ALPHA, AH = XH::ALPHA, AW = XW::ALPHA;
  float p[AD * AH * AW * VEC];
  // in = stride * (m * tile + start + i) + phase - pad
  const int zd = g.sD * (MD * tc.td + pc.start[0]) + pc.phase[0] - g.pD;
  const int zh = g.sH * (MH * tc.th + pc.start[1]) + pc.phase[1] - g.pH;
  const int zw = g.sW * (MW * tc.tw + pc.start[2]) + pc.phase[2] - g.pW;
  // one 64-bit base per image, 32-bit pixel indices inside it, validity per row and per column
  const T *xb = x + (long long)tc.n * g.D * g.H * g.W * g.C + c0;
  bool okw[AW];
  int colofs[AW];      // element offset of a patch column within its image row
#pragma unroll
  for (int k = 0; k < AW; ++k) {
    const int iw = zw + g.sW * k;
    okw[k] = (unsigned)iw < (unsigned)g.W;
    colofs[k] = iw * g.C;
  }
#pragma unroll
  for (int i = 0; i < AD; ++i) {
    const int id = zd + g.sD * i;
    const bool okd = (unsigned)id < (unsigned)g.D;
#pragma unroll
    for (int j = 0; j < AH; ++j) {
      const int ih = zh + g.sH * j;
      const bool okr = okd && (unsigned)ih < (unsigned)g.H;
      const T *rowp = xb + (long long)((id * g.H + ih) * g.W) * g.C;      // one 64-bit product per patch row
#pragma unroll
      for (int k = 0; k < AW; ++k) {
        float(&dst)[VEC] = *reinterpret_cast<float(*)[VEC]>(&p[((i * AH + j) * AW + k) * VEC]);
        if (okr && okw[k]) {
          VecIO<T, VEC>::load(rowp + colofs[k], dst);
        } else {
#pragma unroll
          for (int l = 0; l < VEC; ++l) dst[l] = 0.f;
        }
      }
    }
  }
  if constexpr (VEC == 2 && MD == 1 && MH == 4 && MW == 4 && RH == 3 && RW == 3) {
    // F(4x4,3x3) over a channel pair: both passes on packed fp32 pairs (half the arithmetic instructions, same roundings)
    uint64_t q[AH * AW];
#pragma unroll
    for (int i = 0; i < AH * AW; ++i) q[i] = f2_pack(p[2 * i], p[2 * i + 1]);
#pragma unroll
    for (int i = 0; i < AH; ++i) XW::template bt2<1>(&q[i * AW]);
#pragma unroll
    for (int k = 0; k < AW; ++k) XH::template bt2<AW>(&q[k]);
    T *dstq = v + (long long)pc.pos_base * v_pos_stride + v_row * g.Cp + c0;
#pragma unroll
    for (int i = 0; i < AH * AW; ++i) {   // a running pointer: one 64-bit add per position, no 64-bit product
      float o[2];
      f2_unpack(q[i], o[0], o[1]);
      VecIO<T, 2>::store(dstq, o);
      dstq += v_pos_stride;
    }
  } else {
  // along W (stride VEC), H (stride AW*VEC), D (stride AH*AW*VEC)
#pragma unroll
  for (int i = 0; i < AD * AH; ++i)
#pragma unroll
    for (int l = 0; l < VEC; ++l) XW::template bt<VEC>(&p[i * AW * VEC + l]);
#pragma unroll
  for (int i = 0; i < AD; ++i)
#pragma unroll
    for (int k = 0; k < AW * VEC; ++k) XH::template bt<AW * VEC>(&p[i * AH * AW * VEC + k]);
#pragma unroll
  for (int k = 0; k < AH * AW * VEC; ++k) XD::template bt<AH * AW * VEC>(&p[k]);

  T *dst = v + (long long)pc.pos_base * v_pos_stride + v_row * g.Cp + c0;
#pragma unroll
  for (int q = 0; q < AD * AH * AW; ++q) {
    float(&src)[VEC] = *reinterpret_cast<float(*)[VEC]>(&p[q * VEC]);
    VecIO<T, VEC>::store(dst, src);
    dst += v_pos_stride;
  }
  }   // generic path
}

template <typename T, int VEC, int MODE>
__global__ void __launch_bounds__(256) input_transform_kernel(const T *__restrict__ x, T *__restrict__ v,
                                                              const __grid_constant__ Geom g, long long t0,
                                                              int n_tiles) {
  constexpr int MD = ModeM<MODE>::MD, MH = ModeM<MODE>::MH, MW = ModeM<MODE>::MW;
  const unsigned cvs = (unsigned)(g.Cp / VEC);
  const unsigned idx = blockIdx.x * blockDim.x + threadIdx.x;      // tiles x channel vectors of a pass fit 32 bits
  const unsigned row_u = idx / cvs;
  if (row_u >= (unsigned)n_tiles) return;
  const long long row = row_u;
  const int c0 = (int)(idx - row_u * cvs) * VEC;
  const Piece &pc = g.pieces[blockIdx.y];
  const long long v_pos_stride = (long long)n_tiles * g.Cp;
  if (c0 >= g.C) {  // padding channels of V are zero so the GEMM can run over c_pad
    T *dst = v + (long long)pc.pos_base * v_pos_stride + row * g.Cp + c0;
    float z[VEC];
#pragma unroll
    for (int l = 0; l < VEC; ++l) z[l] = 0.f;
    for (int q = 0; q < pc.n_pos; ++q) VecIO<T, VEC>::store(dst + (long long)q * v_pos_stride, z);
    return;
  }
  const TileCoord tc = decode_tile(g, t0 + row);
  const int rd = pc.r[0], rh = pc.r[1], rw = pc.r[2];
#define WINO_IN_BODY(RD_, RH_, RW_) \
  input_piece<T, VEC, MD, RD_, MH, RH_, MW, RW_>(x, v, g, pc, tc, c0, row, v_pos_stride)
  if constexpr (MODE == 0) {
    (void)rd;
    WINO_SW_H(1, WINO_IN_BODY)
  } else if constexpr (MODE == 1) {
    WINO_SW_D(WINO_IN_BODY)
  } else {
    (void)rd; (void)rh; (void)rw;
    WINO_IN_BODY(1, 3, 3);
  }
#undef WINO_IN_BODY
}

// ------------------------------------------------------------------------------------------
// filter transform:  U[pos][k][c] = (G g G^T)[pos]
// ------------------------------------------------------------------------------------------
template <typename T, int MD, int RD, int MH, int RH, int MW, int RW>
__device__ __forceinline__ void filter_piece(const T *__restrict__ w, T *__restrict__ u, const Geom &g,
                                             const Piece &pc, int k, int c) {
  using XD = Xf<MD, RD>; using XH = Xf<MH, RH>; using XW = Xf<MW, RW>;
  constexpr int AD = XD::ALPHA, AH = XH::ALPHA, AW = XW::ALPHA;
  float a[RD * RH * RW];
#pragma unroll
  for (int i = 0; i < RD; ++i)
#pragma unroll
    for (int j = 0; j < RH; ++j)
#pragma unroll
      for (int l = 0; l < RW; ++l) {
        const int kd = pc.phase[0] + g.sD * (pc.start[0] + i);
        const int kh = pc.phase[1] + g.sH * (pc.start[1] + j);
        const int kw = pc.phase[2] + g.sW * (pc.start[2] + l);
        long long off;
        if (g.weight_layout == WINOCONV_W_KCRS)
          off = ((((long long)k * g.C + c) * g.kD + kd) * g.kH + kh) * g.kW + kw;
        else
          off = ((((long long)kd * g.kH + kh) * g.kW + kw) * g.C + c) * g.K + k;
        a[(i * RH + j) * RW + l] = Elem<T>::load(w + off);
      }
  float b[RD * RH * AW];   // W expanded
#pragma unroll
  for (int i = 0; i < RD * RH; ++i) XW::template g<1, 1>(&a[i * RW], &b[i * AW]);
  float cbuf[RD * AH * AW];  // H expanded
#pragma unroll
  for (int i = 0; i < RD; ++i)
#pragma unroll
    for (int l = 0; l < AW; ++l) XH::template g<AW, AW>(&b[i * RH * AW + l], &cbuf[i * AH * AW + l]);
  float d[AD * AH * AW];  // D expanded
#pragma unroll
  for (int l = 0; l < AH * AW; ++l) XD::template g<AH * AW, AH * AW>(&cbuf[l], &d[l]);
  const long long pos_stride = (long long)g.K * g.Cp;
  T *dst = u + (long long)pc.pos_base * pos_stride + (long long)k * g.Cp + c;
#pragma unroll
  for (int q = 0; q < AD * AH * AW; ++q) Elem<T>::store(dst + q * pos_stride, d[q]);
}

template <typename T, int MODE>
__global__ void __launch_bounds__(256) filter_transform_kernel(const T *__restrict__ w, T *__restrict__ u,
                                                               const __grid_constant__ Geom g) {
  constexpr int MD = ModeM<MODE>::MD, MH = ModeM<MODE>::MH, MW = ModeM<MODE>::MW;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)g.K * g.Cp) return;
  const int k = (int)(idx / g.Cp), c = (int)(idx % g.Cp);
  const Piece &pc = g.pieces[blockIdx.y];
  if (c >= g.C) {
    const long long pos_stride = (long long)g.K * g.Cp;
    T *dst = u + (long long)pc.pos_base * pos_stride + (long long)k * g.Cp + c;
    for (int q = 0; q < pc.n_pos; ++q) Elem<T>::store(dst + q * pos_stride, 0.f);
    return;
  }
  const int rd = pc.r[0], rh = pc.r[1], rw = pc.r[2];
#define WINO_F_BODY(RD_, RH_, RW_) filter_piece<T, MD, RD_, MH, RH_, MW, RW_>(w, u, g, pc, k, c)
  if constexpr (MODE == 0) {
    (void)rd;
    WINO_SW_H(1, WINO_F_BODY)
  } else if constexpr (MODE == 1) {
    WINO_SW_D(WINO_F_BODY)
  } else {
    (void)rd; (void)rh; (void)rw;
    WINO_F_BODY(1, 3, 3);
  }
#undef WINO_F_BODY
}

// ------------------------------------------------------------------------------------------
// output transform:  y = sum_pieces A^T M A  (+ bias, ReLU, 2x2 max-pool), one store per output
// ------------------------------------------------------------------------------------------
template <typename TM, int VEC, int MD, int RD, int MH, int RH, int MW, int RW>
__device__ __forceinline__ void output_piece(const TM *__restrict__ m, float *acc, const Geom &g, const Piece &pc,
                                             int k0, long long m_row, long long m_pos_stride) {
  using XD = Xf<MD, RD>; using XH = Xf<MH, RH>; using XW = Xf<MW, RW>;
  constexpr int AD = XD::ALPHA, AH = XH::ALPHA, AW = XW::ALPHA;
  const TM *src = m + (long long)pc.pos_base * m_pos_stride + m_row * g.K + k0;
  float t1[AD * AH * MW * VEC];
#pragma unroll
  for (int i = 0; i < AD * AH; ++i) {
    float row[AW * VEC];
#pragma unroll
    for (int k = 0; k < AW; ++k) {
      float(&dst)[VEC] = *reinterpret_cast<float(*)[VEC]>(&row[k * VEC]);
      VecIO<TM, VEC>::load(src, dst);
      src += m_pos_stride;      // positions are consecutive: a running pointer instead of a 64-bit product per load
    }
#pragma unroll
    for (int l = 0; l < VEC; ++l) XW::template at<VEC, VEC>(&row[l], &t1[i * MW * VEC + l]);
  }
  float t2[AD * MH * MW * VEC];
#pragma unroll
  for (int i = 0; i < AD; ++i)
#pragma unroll
    for (int k = 0; k < MW * VEC; ++k)
      XH::template at<MW * VEC, MW * VEC>(&t1[i * AH * MW * VEC + k], &t2[i * MH * MW * VEC + k]);
#pragma unroll
  for (int k = 0; k < MH * MW * VEC; ++k) {
    float o[MD];
    XD::template at<MH * MW * VEC, 1>(&t2[k], o);
#pragma unroll
    for (int i = 0; i < MD; ++i) acc[i * MH * MW * VEC + k] += o[i];
  }
}

template <typename T, typename TM, int VEC, int MODE>
__global__ void __launch_bounds__(256) output_transform_kernel(const TM *__restrict__ m, T *__restrict__ y,
                                                               const T *__restrict__ bias,
                                                               const __grid_constant__ Geom g, long long t0,
                                                               int n_tiles) {
  constexpr int MD = ModeM<MODE>::MD, MH = ModeM<MODE>::MH, MW = ModeM<MODE>::MW;
  const unsigned kvs = (unsigned)(g.K / VEC);
  const unsigned idx = blockIdx.x * blockDim.x + threadIdx.x;      // tiles x channel vectors of a pass fit 32 bits
  const unsigned row_u = idx / kvs;
  if (row_u >= (unsigned)n_tiles) return;
  const long long row = row_u;
  const int k0 = (int)(idx - row_u * kvs) * VEC;
  const long long m_pos_stride = (long long)n_tiles * g.K;
  float acc[MD * MH * MW * VEC];
#pragma unroll
  for (int i = 0; i < MD * MH * MW * VEC; ++i) acc[i] = 0.f;
  for (int p = 0; p < g.n_pieces; ++p) {
    const Piece &pc = g.pieces[p];
    const int rd = pc.r[0], rh = pc.r[1], rw = pc.r[2];
#define WINO_O_BODY(RD_, RH_, RW_) \
  output_piece<TM, VEC, MD, RD_, MH, RH_, MW, RW_>(m, acc, g, pc, k0, row, m_pos_stride)
    if constexpr (MODE == 0) {
      (void)rd;
      WINO_SW_H(1, WINO_O_BODY)
    } else if constexpr (MODE == 1) {
      WINO_SW_D(WINO_O_BODY)
    } else {
      (void)rd; (void)rh; (void)rw;
      WINO_O_BODY(1, 3, 3);
    }
#undef WINO_O_BODY
  }
  float bv[VEC];
#pragma unroll
  for (int l = 0; l < VEC; ++l) bv[l] = 0.f;
  if (g.epilogue & WINOCONV_EPI_BIAS) VecIO<T, VEC>::load(bias + k0, bv);
  const bool relu = (g.epilogue & WINOCONV_EPI_RELU) != 0;
  const TileCoord tc = decode_tile(g, t0 + row);
  if (g.epilogue & WINOCONV_EPI_POOL2) {
    // 2x2 windows never straddle tiles (MH, MW even); bias and ReLU commute with max.
    if constexpr (MD == 1 && MH % 2 == 0 && MW % 2 == 0) {
#pragma unroll
      for (int a = 0; a < MH / 2; ++a)
#pragma unroll
        for (int b = 0; b < MW / 2; ++b) {
          const int ph = tc.th * (MH / 2) + a, pw = tc.tw * (MW / 2) + b;
          if (ph < g.yH && pw < g.yW) {
            float o[VEC];
#pragma unroll
            for (int l = 0; l < VEC; ++l) {
              float v0 = acc[((2 * a) * MW + 2 * b) * VEC + l], v1 = acc[((2 * a) * MW + 2 * b + 1) * VEC + l];
              float v2 = acc[((2 * a + 1) * MW + 2 * b) * VEC + l], v3 = acc[((2 * a + 1) * MW + 2 * b + 1) * VEC + l];
              float r = fmaxf(fmaxf(v0, v1), fmaxf(v2, v3)) + bv[l];
              o[l] = relu ? fmaxf(r, 0.f) : r;
            }
            VecIO<T, VEC>::store(y + (((long long)tc.n * g.yH + ph) * g.yW + pw) * g.K + k0, o);
          }
        }
    }
    return;
  }
#pragma unroll
  for (int a = 0; a < MD; ++a) {
    const int od = tc.td * MD + a;
#pragma unroll
    for (int b = 0; b < MH; ++b) {
      const int oh = tc.th * MH + b;
#pragma unroll
      for (int c = 0; c < MW; ++c) {
        const int ow = tc.tw * MW + c;
        if (od < g.oD && oh < g.oH && ow < g.oW) {  // last tile of an odd extent is masked
          float o[VEC];
#pragma unroll
          for (int l = 0; l < VEC; ++l) {
            float r = acc[((a * MH + b) * MW + c) * VEC + l] + bv[l];
            o[l] = relu ? fmaxf(r, 0.f) : r;
          }
          VecIO<T, VEC>::store(y + ((((long long)tc.n * g.oD + od) * g.oH + oh) * g.oW + ow) * g.K + k0, o);
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// host launchers
// ------------------------------------------------------------------------------------------
// The transform kernels index threads, tiles and the pixels of one image with 32 bits.
static inline bool fits_32bit_indexing(const Geom &g, long long n_threads) {
  return n_threads + 256 < (1LL << 32) && g.T < (1LL << 31) && (long long)g.D * g.H * g.W < (1LL << 31);
}

static inline int mode_of(const Geom &g) { return g.mH == 6 ? 3 : (g.mH == 4 ? 2 : (g.mD == 2 ? 1 : 0)); }

// F(6x6,3x3) is instantiated for fp32 only (the planner refuses it for 16-bit operands)
template <typename T> constexpr bool kHasF63 = false;
template <> constexpr bool kHasF63<float> = true;

template <typename T>
static cudaError_t launch_filter_t(const Geom &g, const void *w, void *u, cudaStream_t s) {
  const long long n = (long long)g.K * g.Cp;
  dim3 grid((unsigned)((n + 255) / 256), g.n_pieces), block(256);
  switch (mode_of(g)) {
    case 0: filter_transform_kernel<T, 0><<<grid, block, 0, s>>>((const T *)w, (T *)u, g); break;
    case 1: filter_transform_kernel<T, 1><<<grid, block, 0, s>>>((const T *)w, (T *)u, g); break;
    case 2: filter_transform_kernel<T, 2><<<grid, block, 0, s>>>((const T *)w, (T *)u, g); break;
    default:
      if constexpr (kHasF63<T>) filter_transform_kernel<T, 3><<<grid, block, 0, s>>>((const T *)w, (T *)u, g);
      else return cudaErrorInvalidValue;
      break;
  }
  return cudaGetLastError();
}

cudaError_t launch_filter_transform(const Geom &g, int dtype, const void *w, void *u, cudaStream_t s) {
  switch (dtype) {
    case WINOCONV_F32: return launch_filter_t<float>(g, w, u, s);
    case WINOCONV_F16: return launch_filter_t<__half>(g, w, u, s);
    default: return launch_filter_t<__nv_bfloat16>(g, w, u, s);
  }
}

// 2-D F(2,r) pieces with four channels per thread (16-byte accesses in fp32): the patch is 16 x 4 floats, still in registers
template <typename T>
static cudaError_t launch_input_v4_2d(const Geom &g, const void *x, void *v, long long t0, int n_tiles, cudaStream_t s) {
  const long long n = (long long)n_tiles * (g.Cp / 4);
  if (!fits_32bit_indexing(g, n)) return cudaErrorInvalidValue;
  dim3 grid((unsigned)((n + 255) / 256), g.n_pieces), block(256);
  input_transform_kernel<T, 4, 0><<<grid, block, 0, s>>>((const T *)x, (T *)v, g, t0, n_tiles);
  return cudaGetLastError();
}

template <typename T, int VEC>
static cudaError_t launch_input_tv(const Geom &g, const void *x, void *v, long long t0, int n_tiles, cudaStream_t s) {
  const long long n = (long long)n_tiles * (g.Cp / VEC);
  if (!fits_32bit_indexing(g, n)) return cudaErrorInvalidValue;
  dim3 grid((unsigned)((n + 255) / 256), g.n_pieces), block(256);
  switch (mode_of(g)) {
    case 0: input_transform_kernel<T, VEC, 0><<<grid, block, 0, s>>>((const T *)x, (T *)v, g, t0, n_tiles); break;
    case 1: input_transform_kernel<T, VEC, 1><<<grid, block, 0, s>>>((const T *)x, (T *)v, g, t0, n_tiles); break;
    case 2: input_transform_kernel<T, VEC, 2><<<grid, block, 0, s>>>((const T *)x, (T *)v, g, t0, n_tiles); break;
    default:
      if constexpr (kHasF63<T>) input_transform_kernel<T, VEC, 3><<<grid, block, 0, s>>>((const T *)x, (T *)v, g, t0, n_tiles);
      else return cudaErrorInvalidValue;
      break;
  }
  return cudaGetLastError();
}

cudaError_t launch_input_transform(const Geom &g, int dtype, const void *x, void *v, long long t0, int n_tiles,
                                   cudaStream_t s) {
  // F(6x6,3x3) keeps an 8 x 8 patch per channel in registers: one channel per thread (two would leave one block per SM)
  const bool vec = (g.C % 2 == 0) && mode_of(g) != 3;
  if (mode_of(g) == 0 && g.C % 4 == 0 && g.Cp % 4 == 0) {
    switch (dtype) {
      case WINOCONV_F32: return launch_input_v4_2d<float>(g, x, v, t0, n_tiles, s);
      case WINOCONV_F16: return launch_input_v4_2d<__half>(g, x, v, t0, n_tiles, s);
      default: return launch_input_v4_2d<__nv_bfloat16>(g, x, v, t0, n_tiles, s);
    }
  }
  switch (dtype) {
    case WINOCONV_F32:
      return vec ? launch_input_tv<float, 2>(g, x, v, t0, n_tiles, s) : launch_input_tv<float, 1>(g, x, v, t0, n_tiles, s);
    case WINOCONV_F16:
      return vec ? launch_input_tv<__half, 2>(g, x, v, t0, n_tiles, s) : launch_input_tv<__half, 1>(g, x, v, t0, n_tiles, s);
    default:
      return vec ? launch_input_tv<__nv_bfloat16, 2>(g, x, v, t0, n_tiles, s)
                 : launch_input_tv<__nv_bfloat16, 1>(g, x, v, t0, n_tiles, s);
  }
}

template <typename T, typename TM, int VEC>
static cudaError_t launch_output_tv(const Geom &g, const void *m, void *y, const void *bias, long long t0, int n_tiles,
                                    cudaStream_t s) {
  const long long n = (long long)n_tiles * (g.K / VEC);
  if (!fits_32bit_indexing(g, n)) return cudaErrorInvalidValue;
  dim3 grid((unsigned)((n + 255) / 256)), block(256);
  switch (mode_of(g)) {
    case 0:
      output_transform_kernel<T, TM, VEC, 0><<<grid, block, 0, s>>>((const TM *)m, (T *)y, (const T *)bias, g, t0, n_tiles);
      break;
    case 1:
      output_transform_kernel<T, TM, VEC, 1><<<grid, block, 0, s>>>((const TM *)m, (T *)y, (const T *)bias, g, t0, n_tiles);
      break;
    case 2:
      output_transform_kernel<T, TM, VEC, 2><<<grid, block, 0, s>>>((const TM *)m, (T *)y, (const T *)bias, g, t0, n_tiles);
      break;
    default:
      if constexpr (kHasF63<T>)
        output_transform_kernel<T, TM, VEC, 3><<<grid, block, 0, s>>>((const TM *)m, (T *)y, (const T *)bias, g, t0, n_tiles);
      else
        return cudaErrorInvalidValue;
      break;
  }
  return cudaGetLastError();
}

template <typename T, typename TM>
static cudaError_t launch_output_t(const Geom &g, const void *m, void *y, const void *bias, long long t0, int n_tiles,
                                   cudaStream_t s) {
  if (mode_of(g) == 0 && g.K % 4 == 0) {   // 2-D F(2,r): four channels per thread
    const long long n = (long long)n_tiles * (g.K / 4);
    if (!fits_32bit_indexing(g, n)) return cudaErrorInvalidValue;
    dim3 grid((unsigned)((n + 255) / 256)), block(256);
    output_transform_kernel<T, TM, 4, 0><<<grid, block, 0, s>>>((const TM *)m, (T *)y, (const T *)bias, g, t0, n_tiles);
    return cudaGetLastError();
  }
  if (g.K % 2 == 0 && mode_of(g) != 3) return launch_output_tv<T, TM, 2>(g, m, y, bias, t0, n_tiles, s);
  return launch_output_tv<T, TM, 1>(g, m, y, bias, t0, n_tiles, s);
}

cudaError_t launch_output_transform(const Geom &g, int dtype, int product_dtype, const void *m, void *y,
                                    const void *bias, long long t0, int n_tiles, cudaStream_t s) {
  // product dtype is f32 or the activation dtype
  switch (dtype) {
    case WINOCONV_F32: return launch_output_t<float, float>(g, m, y, bias, t0, n_tiles, s);
    case WINOCONV_F16:
      if (product_dtype == WINOCONV_F32) return launch_output_t<__half, float>(g, m, y, bias, t0, n_tiles, s);
      return launch_output_t<__half, __half>(g, m, y, bias, t0, n_tiles, s);
    default:
      if (product_dtype == WINOCONV_F32) return launch_output_t<__nv_bfloat16, float>(g, m, y, bias, t0, n_tiles, s);
      return launch_output_t<__nv_bfloat16, __nv_bfloat16>(g, m, y, bias, t0, n_tiles, s);
  }
}

// ------------------------------------------------------------------------------------------
// stand-alone tile split / concat (fp32) and add
// ------------------------------------------------------------------------------------------
constexpr int SC_CH = 32;  // channels staged per block

// x [N,D,H,W,C] -> out [tiles, C, bD, bH, bW]; one block = one tile x 32 channels, staged through
// shared memory so both the channel-innermost read and the channel-outermost write are coalesced.
__global__ void __launch_bounds__(256) split_kernel(const float *__restrict__ x, float *__restrict__ out, int D,
                                                    int H, int W, int C, int bD, int bH, int bW, int oD, int oH,
                                                    int oW, int nD, int nH, int nW) {
  extern __shared__ float sm[];
  const int vol = bD * bH * bW;
  long long t = blockIdx.x;
  const int tw = (int)(t % nW); t /= nW;
  const int th = (int)(t % nH); t /= nH;
  const int td = (int)(t % nD); t /= nD;
  const int n = (int)t;
  const int c0 = blockIdx.y * SC_CH;
  for (int e = threadIdx.x; e < vol * SC_CH; e += blockDim.x) {
    const int c = e % SC_CH, pix = e / SC_CH;
    const int k = pix % bW, j = (pix / bW) % bH, i = pix / (bW * bH);
    const int id = td * oD + i, ih = th * oH + j, iw = tw * oW + k;
    float val = 0.f;
    if (c0 + c < C && id < D && ih < H && iw < W)
      val = x[((((long long)n * D + id) * H + ih) * W + iw) * C + c0 + c];
    sm[pix * (SC_CH + 1) + c] = val;
  }
  __syncthreads();
  const int nc = min(SC_CH, C - c0);
  float *dst = out + ((long long)blockIdx.x * C + c0) * vol;
  for (int e = threadIdx.x; e < vol * nc; e += blockDim.x) {
    const int c = e / vol, pix = e % vol;
    dst[e] = sm[pix * (SC_CH + 1) + c];
  }
}

// tiles [tiles, K, mD, mH, mW] -> y [N,oD,oH,oW,K]
__global__ void __launch_bounds__(256) concat_kernel(const float *__restrict__ tiles, float *__restrict__ y, int oD,
                                                     int oH, int oW, int K, int mD, int mH, int mW, int nD, int nH,
                                                     int nW) {
  extern __shared__ float sm[];
  const int vol = mD * mH * mW;
  long long t = blockIdx.x;
  const int tw = (int)(t % nW); t /= nW;
  const int th = (int)(t % nH); t /= nH;
  const int td = (int)(t % nD); t /= nD;
  const int n = (int)t;
  const int k0 = blockIdx.y * SC_CH;
  const int nk = min(SC_CH, K - k0);
  const float *src = tiles + ((long long)blockIdx.x * K + k0) * vol;
  for (int e = threadIdx.x; e < vol * nk; e += blockDim.x) {
    const int k = e / vol, pix = e % vol;
    sm[pix * (SC_CH + 1) + k] = src[e];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < vol * SC_CH; e += blockDim.x) {
    const int k = e % SC_CH, pix = e / SC_CH;
    const int c = pix % mW, b = (pix / mW) % mH, a = pix / (mW * mH);
    const int od = td * mD + a, oh = th * mH + b, ow = tw * mW + c;
    if (k < nk && od < oD && oh < oH && ow < oW)
      y[((((long long)n * oD + od) * oH + oh) * oW + ow) * K + k0 + k] = sm[pix * (SC_CH + 1) + k];
  }
}

__global__ void __launch_bounds__(256) add_kernel(const float *__restrict__ a, const float *__restrict__ b,
                                                  float *__restrict__ c, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) c[i] = a[i] + b[i];
}

cudaError_t launch_split(const float *x, float *out, int N, int D, int H, int W, int C, int bD, int bH, int bW,
                         int oD, int oH, int oW, int nD, int nH, int nW, cudaStream_t s) {
  const long long tiles = (long long)N * nD * nH * nW;
  const size_t smem = (size_t)bD * bH * bW * (SC_CH + 1) * sizeof(float);
  dim3 grid((unsigned)tiles, (C + SC_CH - 1) / SC_CH), block(256);
  split_kernel<<<grid, block, smem, s>>>(x, out, D, H, W, C, bD, bH, bW, oD, oH, oW, nD, nH, nW);
  return cudaGetLastError();
}

cudaError_t launch_concat(const float *tiles, float *y, int N, int oD, int oH, int oW, int K, int mD, int mH, int mW,
                          cudaStream_t s) {
  const int nD = ceil_div(oD, mD), nH = ceil_div(oH, mH), nW = ceil_div(oW, mW);
  const long long nt = (long long)N * nD * nH * nW;
  const size_t smem = (size_t)mD * mH * mW * (SC_CH + 1) * sizeof(float);
  dim3 grid((unsigned)nt, (K + SC_CH - 1) / SC_CH), block(256);
  concat_kernel<<<grid, block, smem, s>>>(tiles, y, oD, oH, oW, K, mD, mH, mW, nD, nH, nW);
  return cudaGetLastError();
}

cudaError_t launch_add(const float *a, const float *b, float *c, long long n, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  add_kernel<<<(unsigned)blocks, 256, 0, s>>>(a, b, c, n);
  return cudaGetLastError();
}

}  // namespace wino
