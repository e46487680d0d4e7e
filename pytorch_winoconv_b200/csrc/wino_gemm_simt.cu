// Per-position batched GEMM with fp32 FMA accumulation: the engine's fp32 path (TF32 tensor-core
// products would not hold the 1e-3 bound of an fp32 convolution) and a cross-check for the
// tcgen05 kernel.  m[p][t][k] = sum_c v[p][t][c] * u[p][k][c].
//
// Stands in for cublasSgemmBatched as called from src/base_conv_launchers.cu:362-367.
// 64x64 output tile per 256-thread block, 16-deep reduction slabs staged in shared memory
// (transposed on the way in so the inner loop reads conflict-free float4s), 4x4 register tile.
#include "wino_common.cuh"
#include "wino_launch.h"

namespace wino {

constexpr int SG_BM = 64, SG_BN = 64, SG_BK = 16;

template <typename T, typename TM>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const T *__restrict__ v, const T *__restrict__ u,
                                                        TM *__restrict__ m, long long tiles, int c_pad, int k_out) {
  __shared__ __align__(16) float As[SG_BK][SG_BM + 4];
  __shared__ __align__(16) float Bs[SG_BK][SG_BN + 4];
  const int pos = blockIdx.z;
  const long long row0 = (long long)blockIdx.x * SG_BM;
  const int col0 = blockIdx.y * SG_BN;
  const T *vp = v + (long long)pos * tiles * c_pad;
  const T *up = u + (long long)pos * k_out * c_pad;
  const int tid = threadIdx.x;
  const int lr = tid >> 2;            // 0..63: row of the slab this thread stages
  const int lc = (tid & 3) * 4;       // 0,4,8,12: first of its 4 reduction indices
  const int ty = tid >> 4, tx = tid & 15;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int c0 = 0; c0 < c_pad; c0 += SG_BK) {
    float a4[4] = {0.f, 0.f, 0.f, 0.f}, b4[4] = {0.f, 0.f, 0.f, 0.f};
    if (row0 + lr < tiles && c0 + lc < c_pad) VecIO<T, 4>::load(vp + (row0 + lr) * c_pad + c0 + lc, a4);
    if (col0 + lr < k_out && c0 + lc < c_pad) VecIO<T, 4>::load(up + (long long)(col0 + lr) * c_pad + c0 + lc, b4);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      As[lc + i][lr] = a4[i];
      Bs[lc + i][lr] = b4[i];
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < SG_BK; ++kk) {
      const float4 a = *reinterpret_cast<const float4 *>(&As[kk][ty * 4]);
      const float4 b = *reinterpret_cast<const float4 *>(&Bs[kk][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bw[j], acc[i][j]);
    }
    __syncthreads();
  }
  TM *mp = m + (long long)pos * tiles * k_out;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long r = row0 + ty * 4 + i;
    if (r >= tiles) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + tx * 4 + j;
      if (c < k_out) Elem<TM>::store(mp + r * k_out + c, acc[i][j]);
    }
  }
}

template <typename T, typename TM>
static cudaError_t run(int positions, long long tiles, int c_pad, int k_out, const void *v, const void *u, void *m,
                       cudaStream_t s) {
  dim3 grid((unsigned)((tiles + SG_BM - 1) / SG_BM), (k_out + SG_BN - 1) / SG_BN, positions), block(256);
  gemm_simt_kernel<T, TM><<<grid, block, 0, s>>>((const T *)v, (const T *)u, (TM *)m, tiles, c_pad, k_out);
  return cudaGetLastError();
}

cudaError_t launch_gemm_simt(int dtype, int product_dtype, int positions, long long tiles, int c_pad, int k_out,
                             const void *v, const void *u, void *m, cudaStream_t s) {
  if (positions <= 0 || tiles <= 0) return cudaSuccess;
  if ((tiles + SG_BM - 1) / SG_BM > 0x7fffffffLL || positions > 65535) return cudaErrorInvalidConfiguration;
  switch (dtype) {
    case WINOCONV_F32: return run<float, float>(positions, tiles, c_pad, k_out, v, u, m, s);
    case WINOCONV_F16:
      return product_dtype == WINOCONV_F32 ? run<__half, float>(positions, tiles, c_pad, k_out, v, u, m, s)
                                           : run<__half, __half>(positions, tiles, c_pad, k_out, v, u, m, s);
    default:
      return product_dtype == WINOCONV_F32
                 ? run<__nv_bfloat16, float>(positions, tiles, c_pad, k_out, v, u, m, s)
                 : run<__nv_bfloat16, __nv_bfloat16>(positions, tiles, c_pad, k_out, v, u, m, s);
  }
}

}  // namespace wino
