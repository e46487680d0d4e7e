/*
 * winoconv_b200 -- C ABI of the B200 (sm_100a) Winograd / DWM forward-convolution engine.
 *
 * Plain pointers, sizes and a CUDA stream handle; no torch types, no exceptions, no process
 * exits.  Every entry point returns a winoconv_status_t; winoconv_last_error() gives the
 * detail text of the calling thread's last failure.  All device memory is owned by the
 * caller.  No entry point allocates or frees device memory and none synchronises the device;
 * work is enqueued on the stream passed in (NULL = the legacy default stream).  The library keeps
 * per-device state (kernel attributes, the address of its built-in scratch array) for the life of
 * the process: do not call cudaDeviceReset while it is in use.
 *
 * Data layout (all contiguous, channels last, as the reference's native op takes them):
 *   activations  x [N, D, H, W, C]     (D = 1 for 2-D convolutions)
 *   output       y [N, oD, oH, oW, K]  (oH, oW halved when WINOCONV_EPI_POOL2 is set)
 *   weights      [K, C, kD, kH, kW] (WINOCONV_W_KCRS, torch order) or
 *                [kD, kH, kW, C, K] (WINOCONV_W_RSCK, the order dwm.py:130-133 passes)
 *
 * The reference interface each entry point stands in for is cited beside it
 * (paths are relative to the huangdi95/pytorch_winoconv checkout).
 */
#ifndef WINOCONV_B200_H_
#define WINOCONV_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WINOCONV_ABI_VERSION 1
#if defined(__GNUC__)
#define WINOCONV_API __attribute__((visibility("default")))
#else
#define WINOCONV_API
#endif
#define WINOCONV_MAX_PIECES 64

typedef enum winoconv_status {
  WINOCONV_OK = 0,
  WINOCONV_ERR_INVALID_ARGUMENT = 1, /* NULL pointer, bad enum, non-positive size               */
  WINOCONV_ERR_UNSUPPORTED = 2,      /* shape / stride / dtype outside what the engine covers   */
  WINOCONV_ERR_WORKSPACE = 3,        /* scratch buffers too small for even one block of tiles   */
  WINOCONV_ERR_CUDA = 4,             /* a CUDA runtime / driver call failed                     */
  WINOCONV_ERR_TIMEOUT = 5,          /* a bounded device-side wait gave up (see error word)     */
  WINOCONV_ERR_NO_DEVICE = 6         /* current device is not compute capability 10.x           */
} winoconv_status_t;

typedef enum winoconv_dtype { WINOCONV_F32 = 0, WINOCONV_F16 = 1, WINOCONV_BF16 = 2 } winoconv_dtype_t;
typedef enum winoconv_wlayout { WINOCONV_W_KCRS = 0, WINOCONV_W_RSCK = 1 } winoconv_wlayout_t;
typedef enum winoconv_gemm {
  WINOCONV_GEMM_AUTO = 0,    /* tcgen05 for f16/bf16 inputs, TF32X3 for f32 inputs        */
  WINOCONV_GEMM_SIMT = 1,    /* fp32-accumulate FMA kernel (any dtype; the f32 path)      */
  WINOCONV_GEMM_TCGEN05 = 2, /* tcgen05.mma + TMEM + TMA (f16 / bf16 inputs only)         */
  WINOCONV_GEMM_TF32 = 3,    /* f32 inputs, tcgen05 kind::tf32: 10-bit operand mantissas   */
  WINOCONV_GEMM_TF32X3 = 4   /* f32 inputs, three tf32 products of a hi / lo operand split */
                             /* made in shared memory: fp32-class accuracy on tensor cores */
} winoconv_gemm_t;

typedef enum winoconv_algo {
  WINOCONV_ALGO_AUTO = 0,   /* ROW where it applies, else FUSED where it applies, else STAGED; with      */
                            /* tile_m = 0 a 16-bit 3x3 stride-1 layer of >= 512 input and output channels */
                            /* whose 4-wide tiles cover the output exactly (>= 4096 of them) runs as       */
                            /* STAGED F(4x4,3x3) instead (measured faster; needs the V / M scratch)        */
  WINOCONV_ALGO_STAGED = 1, /* input transform -> batched GEMM -> output transform through V / M scratch  */
  WINOCONV_ALGO_FUSED = 2,  /* one tcgen05 kernel, 3x3 pieces as F(2x2,3x3); f16 / bf16, any stride       */
  WINOCONV_ALGO_ROW = 3     /* one tcgen05 kernel, 1x3 pieces: F(2,3) along W, taps along H / depth summed */
                            /* in TMEM; f16 / bf16, strides 1 or 2 (stride 2 runs as a stride-1 problem    */
                            /* over phase channels), any kernel of 1..10 taps per dimension.  Scratch only  */
                            /* where x cannot be read as it lies: to hold the phase-gathered input of a    */
                            /* stride-2 layer (read in place when C is a multiple of 32, or few channels   */
                            /* with W * C a multiple of 8), or to pad C to a multiple of 8 (few channels   */
                            /* with W * C a multiple of 8 need no padding) (v_ws: input_ws_bytes)          */
} winoconv_algo_t;

/* epilogue bits, applied inside the output transform */
#define WINOCONV_EPI_BIAS 1u  /* y += bias[k]                                  */
#define WINOCONV_EPI_RELU 2u  /* y = max(y, 0)                                 */
#define WINOCONV_EPI_POOL2 4u /* 2x2/stride-2 max pool over (H, W), 2-D only   */

/* One forward convolution.  Zero-initialise, then fill. */
typedef struct winoconv_desc {
  int32_t ndim;          /* 2 or 3 spatial dimensions                                        */
  int32_t batch;         /* N                                                                */
  int32_t c_in;          /* C                                                                */
  int32_t k_out;         /* K                                                                */
  int32_t in_size[3];    /* D, H, W of the input as stored (before padding); D = 1 if ndim=2 */
  int32_t ker_size[3];   /* kD, kH, kW (each 1..10);  kD = 1 if ndim = 2                     */
  int32_t stride[3];     /* 1 or 2 per dimension                                             */
  int32_t pad[3];        /* symmetric zero padding per dimension, applied in-kernel          */
  int32_t tile_m;        /* Winograd output block: 0 = auto (2 where a single-kernel path
                          * takes the layer, else 4 for 2-D 3x3 stride 1), 2 = F(2,r),
                          * 4 = F(4x4,3x3), 6 = F(6x6,3x3) (f32 operands with the SIMT or
                          * TF32X3 engine only: 64 positions, 1.78 multiplies per output) */
  int32_t dtype;         /* winoconv_dtype_t of x, weights, y and of the transformed filter  */
  int32_t weight_layout; /* winoconv_wlayout_t                                               */
  uint32_t epilogue;     /* WINOCONV_EPI_* bits                                              */
  int32_t gemm_engine;   /* winoconv_gemm_t                                                  */
  int32_t product_dtype; /* dtype of the Winograd-domain products: F32 (default), F16, BF16  */
  int32_t algo;          /* winoconv_algo_t                                                  */
  int32_t reserved[5];
} winoconv_desc_t;

/* What winoconv_plan() derives from a descriptor. */
typedef struct winoconv_plan_info {
  int32_t out_size[3];        /* oD, oH, oW of y (after pooling if requested)                 */
  int32_t conv_out_size[3];   /* convolution output extents before pooling                    */
  int32_t tile_m[3];          /* output block per dimension (1 where that extent is not tiled)*/
  int32_t tiles_per_dim[3];   /* nD, nH, nW                                                   */
  int32_t n_pieces;           /* DWM pieces (x polyphase parts for stride 2)                  */
  int32_t positions;          /* Winograd positions summed over pieces                        */
  int32_t c_pad;              /* channel stride of the transformed operands (C rounded to 8)  */
  int32_t gemm_engine;        /* engine AUTO resolves to                                      */
  int32_t algo;               /* algorithm AUTO resolves to (winoconv_algo_t)                 */
  int32_t reserved0;
  int64_t tiles;              /* N * nD * nH * nW                                             */
  uint64_t filter_bytes;      /* size of the transformed filter U [positions][K][c_pad]       */
  uint64_t input_ws_bytes;    /* preferred size of the transformed-input scratch V            */
  uint64_t product_ws_bytes;  /* preferred size of the product scratch M                      */
  uint64_t input_ws_bytes_min;   /* smallest V scratch the forward accepts (128 tiles)        */
  uint64_t product_ws_bytes_min; /* smallest M scratch the forward accepts (128 tiles)        */
  int64_t block_tiles;        /* tiles per pass with the preferred scratch sizes              */
  double direct_flops;        /* 2 N K C prod(k) prod(out): effective-TFLOP/s numerator        */
  double gemm_flops;          /* 2 positions tiles C K: Winograd-domain multiply-adds x 2      */
  double algorithmic_bytes;   /* bytes(x) + bytes(w) + bytes(y)                                */
} winoconv_plan_info_t;

/* Library / device. */
WINOCONV_API int winoconv_abi_version(void);
WINOCONV_API const char *winoconv_status_string(int status);
/* Copies the calling thread's last error detail into buf (NUL terminated); returns its length. */
WINOCONV_API size_t winoconv_last_error(char *buf, size_t buf_size);
/* WINOCONV_OK when the current CUDA device can run the kernels (compute capability 10.x). */
WINOCONV_API int winoconv_device_check(void);

/*
 * Shape inference, DWM piece table and scratch sizes.  Pure host code; needs no GPU.
 * Replaces the host-side sizing in dwm.py:109-127 (dwm2d_), dwm.py:43-75 (dwm3d_), the output
 * extent arithmetic of src/winograd_conv.cpp:20-90 and the splitControl() look-up table
 * (src/base_conv_launchers.h:58-388; here a rule, so every kernel extent 1..10 is accepted,
 * including the 2-D 3x3 the table lacks) and adds what the reference refuses: stride 2
 * (src/winograd_conv.cpp:122-126) as polyphase parts, and F(4x4,3x3).
 */
WINOCONV_API int winoconv_plan(const winoconv_desc_t *desc, winoconv_plan_info_t *info);

/* Fills pieces[i*9 + {0..2}] = phase(d,h,w), {3..5} = start, {6..8} = taps, for i < n_pieces. */
WINOCONV_API int winoconv_plan_pieces(const winoconv_desc_t *desc, int32_t *pieces, int32_t max_pieces, int32_t *n_pieces);

/*
 * U = G g G^T for every piece: weights -> u [positions][K][c_pad] in desc->dtype (computed in
 * fp32, rounded once; channels C..c_pad-1 are written as zero).
 * Replaces wNorm2WinoTransform (src/split_kernel.cu:14-53 with calculation_kernels.cu:1-760),
 * launched from convLauncherStrideOneLarge (src/base_conv_launchers.cu:340-347), and the
 * torch-level G @ w @ G^T (matrix_conv.py:150-153).  Unlike the reference it can be done once
 * per weight and reused across calls.
 */
WINOCONV_API int winoconv_filter_transform(const winoconv_desc_t *desc, const void *weights, void *u, void *stream);

/*
 * y = conv(x, w) by the algorithm the plan names (winoconv_plan_info_t.algo):
 *   ROW / FUSED  one kernel: input tiles are transformed in shared memory, multiplied on the tensor
 *                cores with the DWM pieces summed in the accumulator, and written through the output
 *                transform with the bias / ReLU / 2x2 max-pool epilogue; v_ws and m_ws are not used
 *                (ROW pads C to a multiple of 8 into v_ws when it is not one already).
 *   STAGED       input transform (B^T d B with in-kernel zero padding, DWM piece offsets and stride-2
 *                polyphase addressing) -> one GEMM per Winograd position -> output transform (A^T m A,
 *                summed over pieces in registers, same epilogue, one store per output element).  Tiles
 *                are processed in blocks sized to the scratch given: v_ws holds
 *                [positions][block][c_pad] in desc->dtype, m_ws [positions][block][K] in
 *                desc->product_dtype.
 * Replaces DWM<T> (src/winograd_conv.cpp:16-127; bound at pybind/bind.cpp:23) and everything it
 * launches: inputNorm2WinoTransform, forwardAssign, cublasSgemmBatched / cublasHgemmBatched,
 * outputWino2NormTransform, outputAggregate (src/base_conv_launchers.cu:282-399,
 * src/base_conv_launchers_half.cu:151-268, src/split_kernel.cu:60-203, src/utils.cu:5-12);
 * and the torch-level chain wino_split -> base_conv32 -> wino_concat (matrix_conv.py:112-254).
 * bias may be NULL unless WINOCONV_EPI_BIAS is set (then K values of desc->dtype).
 */
WINOCONV_API int winoconv_forward(const winoconv_desc_t *desc, const void *x, const void *u, const void *bias, void *y,
                     void *v_ws, size_t v_ws_bytes, void *m_ws, size_t m_ws_bytes, void *stream);

/*
 * winoconv_forward with CUDA events around its three stages.  Synchronises the stream, then
 * writes the summed device time of the input transforms, GEMMs and output transforms (ms) to
 * stage_ms[0..2] and the number of kernels launched to *launches (may be NULL).
 * The counterpart of the per-stage perf_counter prints inside dwm3d_ (dwm.py:44-107).
 */
WINOCONV_API int winoconv_forward_timed(const winoconv_desc_t *desc, const void *x, const void *u, const void *bias,
                                        void *y, void *v_ws, size_t v_ws_bytes, void *m_ws, size_t m_ws_bytes,
                                        void *stream, float *stage_ms, int32_t *launches);

/*
 * winoconv_forward for callers that may not allocate device memory at all -- a plugin inside a host
 * application that has handed the whole device to its own memory pool, or a latency-critical loop that
 * cannot afford the device-wide stall of cudaMalloc.  The caller passes only inputs and outputs; the V and
 * M scratch of the pass live in a WINOCONV_STATIC_SCRATCH_BYTES array that is part of the library image, so
 * every GPU that loads the library holds those 32 MiB until the process exits.  Nothing here calls
 * cudaMalloc, cudaFree or any allocating library routine.
 *   - Limit: 128 tiles of scratch (winoconv_plan: input_ws_bytes_min + product_ws_bytes_min) must fit the
 *     array; larger layers are refused with WINOCONV_ERR_WORKSPACE and a message stating both sizes.
 *     Layers that fit are walked in as many passes as the array allows.  A ROW layer uses the array for
 *     its whole channel-padded or phase-gathered copy of the input (winoconv_plan: input_ws_bytes; e.g. a
 *     7x7 stride-2 stem on 225 x 225 RGB images, whose rows cannot be read as they lie, passes 32 MiB from batch 78 on) and is refused the same way beyond that:
 *     the transformed filter is laid out per algorithm, so re-plan that layer with algo =
 *     WINOCONV_ALGO_FUSED (no scratch at all) or WINOCONV_ALGO_STAGED, transform its filter again and call.
 *   - The first call on each device looks up the array's device address (with that device current) and
 *     keeps it; make that first call before starting any stream capture.
 *   - All calls on a device share the one array, and it keeps whatever the previous call left.  Nothing
 *     needs clearing: every scratch element a pass reads was written earlier in the same pass.  Two calls
 *     whose kernels can overlap on the GPU (different streams, no dependency) race on the array -- order them.
 * No counterpart in the reference, whose launcher allocates and frees on every call
 * (src/base_conv_launchers.cu:323-336,376,384-391).
 */
#define WINOCONV_STATIC_SCRATCH_BYTES (32u << 20)
WINOCONV_API int winoconv_forward_static(const winoconv_desc_t *desc, const void *x, const void *u, const void *bias,
                                         void *y, void *stream);

/*
 * The per-position batched GEMM on its own: m[p][t][k] = sum_c v[p][t][c] * u[p][k][c],
 * fp32 accumulate.  v [positions][tiles][c_pad], u [positions][k_out][c_pad] in `dtype`,
 * m [positions][tiles][k_out] in `product_dtype`.  c_pad must be a multiple of 8.
 * Replaces forwardAssign + cublasSgemmBatched / cublasHgemmBatched
 * (src/base_conv_launchers.cu:349-367, src/base_conv_launchers_half.cu:218-236) and the
 * torch.matmul of matrix_conv.py:205.
 */
WINOCONV_API int winoconv_gemm_batched(int dtype, int product_dtype, int gemm_engine, int positions, int64_t tiles, int c_pad,
                          int k_out, const void *v, const void *u, void *m, void *stream);

/*
 * Overlapping-tile extraction and re-assembly, kept so the reference's torch-level route keeps
 * working.  fp32, channels last.
 *   split : x [N, D, H, W, C] -> out [N*nD*nH*nW, C, bD, bH, bW], window origin = out_block * tile,
 *           zero filled beyond the input.  2-D: pass D = bD = nD = 1.
 *   concat: in [N*nD*nH*nW, K, mD, mH, mW] -> y [N, oD, oH, oW, K], last tile masked.
 * Replace WinoSplit<float> / WinoConcat<float> (src/split_and_concat.cpp:14-78,
 * src/split_and_concat_kernels.cu:9-129; bound at pybind/bind.cpp:21-22).  The reference's
 * kernels hard-code a window stride of 2 (split_and_concat_kernels.cu:20-22,87-88); here the
 * stride is the output block, so F(4x4,3x3) tiles work too.
 */
WINOCONV_API int winoconv_split(const float *x, float *out, int batch, int d, int h, int w, int c, int block_d, int block_h,
                   int block_w, int out_block_d, int out_block_h, int out_block_w, int n_d, int n_h, int n_w,
                   void *stream);
WINOCONV_API int winoconv_concat(const float *tiles, float *y, int batch, int out_d, int out_h, int out_w, int k,
                    int out_block_d, int out_block_h, int out_block_w, void *stream);

/*
 * c = a + b over n floats.  Replaces AddGPU<float> (src/add.cpp:10-34, src/add.cu:7-29; bound at
 * pybind/bind.cpp:19) -- without its off-by-one (add.cu:10 tests i <= N).
 */
WINOCONV_API int winoconv_add(const float *a, const float *b, float *c, int64_t n, void *stream);

/*
 * Calibration probe: clocks per tcgen05.mma (M = 128 rows per SM, K = 16, f16 operands, fp32 accumulate) for an
 * accumulator n_cols wide (a multiple of 16, <= 256), issued by n_threads (1, 2 or 4) threads with their own
 * accumulators, with the A operand in shared memory (a_in_tmem = 0) or tensor memory (1), on one SM or across a
 * CTA pair (cta_pair = 1: M = 256 over both).  Writes the span from first issue to last completion divided by
 * the MMAs issued, and (optionally) the issuing cost per MMA seen by one thread.  Synchronises the stream.  The
 * planner's preference for 128-column accumulators and the design notes' bandwidth figures come from this probe
 * (`python bench.py --workload mma-rate` prints the table).  No counterpart in the reference.
 */
WINOCONV_API int winoconv_probe_mma_rate(int cta_pair, int a_in_tmem, int n_cols, int n_threads, int n_mma,
                                         float *clocks_per_mma, float *issue_clocks_per_mma, void *stream);

/*
 * Device error word of the tcgen05 GEMM: bounded mbarrier waits store a code here instead of
 * spinning forever.  Reads and clears it (synchronises the stream).  0 = no error.
 */
WINOCONV_API int winoconv_read_device_error(void *stream, uint32_t *code);

#ifdef __cplusplus
}
#endif
#endif /* WINOCONV_B200_H_ */
