// Host-side launch functions shared between the translation units of libwinoconv_b200.
#pragma once

#include <cuda_runtime.h>

#include "wino_common.cuh"

namespace wino {

cudaError_t launch_filter_transform(const Geom &g, int dtype, const void *w, void *u, cudaStream_t s);
cudaError_t launch_input_transform(const Geom &g, int dtype, const void *x, void *v, long long t0, int n_tiles,
                                   cudaStream_t s);
cudaError_t launch_output_transform(const Geom &g, int dtype, int product_dtype, const void *m, void *y,
                                    const void *bias, long long t0, int n_tiles, cudaStream_t s);
cudaError_t launch_split(const float *x, float *out, int N, int D, int H, int W, int C, int bD, int bH, int bW,
                         int oD, int oH, int oW, int nD, int nH, int nW, cudaStream_t s);
cudaError_t launch_concat(const float *tiles, float *y, int N, int oD, int oH, int oW, int K, int mD, int mH, int mW,
                          cudaStream_t s);
cudaError_t launch_add(const float *a, const float *b, float *c, long long n, cudaStream_t s);

// m[p][t][k] = sum_c v[p][t][c] u[p][k][c]; fp32 accumulate.
cudaError_t launch_gemm_simt(int dtype, int product_dtype, int positions, long long tiles, int c_pad, int k_out,
                             const void *v, const void *u, void *m, cudaStream_t s);
// tcgen05 / TMEM / TMA version (f16 / bf16).  `detail` receives a message on failure.
cudaError_t launch_gemm_tcgen05(int dtype, int product_dtype, int positions, long long tiles, int c_pad, int k_out,
                                const void *v, const void *u, void *m, cudaStream_t s, const char **detail);

// fp32 operands on the tensor cores (kind::tf32): split = 0 plain tf32 products, split = 1 three products of a
// hi / lo split made in shared memory (fp32-class accuracy).  m in fp32.
cudaError_t launch_gemm_tf32(int split, int positions, long long tiles, int c_pad, int k_out, const void *v,
                             const void *u, void *m, cudaStream_t s, const char **detail);

// F(4x4,3x3) input transform of a whole 16-bit layer with the raw patches staged through shared memory by TMA
// (channels a multiple of eight, one pass over all tiles); `applies` says whether a call qualifies.
bool input_f43_tma_applies(const Geom &g, int dtype, const void *x, long long t0, long long n_tiles);
cudaError_t launch_input_f43_tma(const Geom &g, int dtype, const void *x, void *v, cudaStream_t s, const char **detail);

// The matching output transform (output channels a multiple of eight, bias / ReLU epilogue, one pass over all tiles).
bool output_f43_tma_applies(const Geom &g, int dtype, int product_dtype, const void *m, long long t0, long long n_tiles);
cudaError_t launch_output_f43_tma(const Geom &g, int dtype, int product_dtype, const void *m, void *y, const void *bias,
                                  cudaStream_t s, const char **detail);

// Fused F(2x2,3x3) path (f16 / bf16): transformed filter u [16][K][R], then one kernel for the whole layer.
cudaError_t launch_fused_filter_transform(const FGeom &g, int dtype, const void *w, void *u, cudaStream_t s);
cudaError_t launch_fused_forward(const FGeom &g, int dtype, const void *x, const void *u, const void *bias, void *y,
                                 cudaStream_t s, const char **detail);
cudaError_t read_and_clear_fused_error(cudaStream_t s, unsigned int *code);

// Row-piece DWM kernel (f16 / bf16, stride 1): 1 x 3 pieces, F(2,3) along W, taps along H / depth summed in TMEM.
struct RowDesc {
  int N, C, K, D, H, W, oD, oH, oW, yH, yW;
  int sD, sH, sW, pD, pH, pW, kD, kH, kW;
  unsigned epilogue;
  int weight_layout;
  // Stride 2 as a stride-1 problem (polyphase parts folded into the channels): when `phases` > 1 the fields above
  // describe the stride-1 convolution the kernel runs -- C = phases x C0 channels, kernel ceil(k0 / 2) per strided
  // dimension, no padding, input extent out + k - 1 -- and the fields below the tensor the caller passes in.
  int phases;                 // 1: plain stride-1 problem
  int fD, fH, fW;             // phase count per dimension (1 or 2)
  int C0, D0, H0, W0;         // caller's input [N, D0, H0, W0, C0]
  int pD0, pH0, pW0;          // caller's padding
  int kD0, kH0, kW0;          // caller's kernel
};
struct RowPlan {
  int Cp, PW, BN, MB, CBW, RB, n_rb, n_cb, slab_rows, patch_h, patch_w, n_chunks, n_nblocks, slabs;
  long long filter_elems, n_items;
  int raw_bytes, a_bytes, b_stage_bytes, n_b_stages, n_a_bufs, smem_total;
  int b_group;   // filter stages per barrier group (1, or 3 = all rows of a 3-row kernel)
  int s2_chunks;   // > 0: a stride-2 layer read from the caller's tensor through an element-strided tensor map (ceil(C0 / 32) chunks per phase)
  int raw_c, raw_off, raw_row_el;   // raw_c > 0: few-channel x is read as it lies (rows of W * C elements)
  int raw_seg, raw_fh, raw_pd, raw_ph, raw_pw;   // elements per pixel and raw row, raw rows per patch row, padding in x's own coordinates
  int pair;   // 1: CTA pairs (two images per work item, one M = 256 MMA over both SMs, filter slabs split between them)
};
bool rowfused_plan(const RowDesc &d, RowPlan *out);
cudaError_t launch_rowfused_filter_transform(const RowDesc &d, const RowPlan &p, int dtype, const void *w, void *u, cudaStream_t s);
cudaError_t launch_rowfused_forward(const RowDesc &d, const RowPlan &p, int dtype, const void *x, const void *u,
                                    const void *bias, void *y, void *pad_ws, cudaStream_t s, const char **detail);
cudaError_t read_and_clear_row_error(cudaStream_t s, unsigned int *code);

// Reads the error word of the bounded device waits, clears it and synchronises the stream.
cudaError_t read_and_clear_device_error(cudaStream_t s, unsigned int *code);

}  // namespace wino
