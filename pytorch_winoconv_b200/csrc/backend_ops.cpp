// Host glue between torch tensors and the winoconv_b200 C ABI for the reference's operator names.
// Everything is enqueued on torch's current stream; nothing synchronises, nothing exits the process:
// every failure becomes a Python exception carrying the C ABI's error text.
#include "backend_ops.h"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <atomic>

#include "winoconv_b200.h"

namespace {

std::atomic<int> g_dwm_block{2};

std::string abi_error() {
  char buf[1024];
  winoconv_last_error(buf, sizeof buf);
  return std::string(buf);
}

#define WINO_CHECK(call, what)                                                                     \
  do {                                                                                             \
    const int st_ = (call);                                                                        \
    TORCH_CHECK(st_ == WINOCONV_OK, what, " failed (", winoconv_status_string(st_), "): ", abi_error()); \
  } while (0)

int dtype_code(const at::Tensor &t, const char *name) {
  switch (t.scalar_type()) {
    case at::kFloat: return WINOCONV_F32;
    case at::kHalf: return WINOCONV_F16;
    case at::kBFloat16: return WINOCONV_BF16;
    default: TORCH_CHECK(false, name, " must be float32, float16 or bfloat16, got ", t.scalar_type());
  }
  return -1;
}

void check_cuda_contig(const at::Tensor &t, const char *name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

void *stream_of() { return (void *)at::cuda::getCurrentCUDAStream().stream(); }

bool usable(const at::Tensor &t, const at::Tensor &like, at::ScalarType want, size_t bytes) {
  return t.defined() && t.is_cuda() && t.is_contiguous() && t.device() == like.device() && t.scalar_type() == want &&
         (size_t)t.numel() * t.element_size() >= bytes && (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15u) == 0;
}

}  // namespace

void set_dwm_output_block(int m) {
  TORCH_CHECK(m == 0 || m == 2 || m == 4, "output block must be 0 (auto), 2 or 4");
  g_dwm_block = m;
}
int get_dwm_output_block() { return g_dwm_block; }

// reference: src/add.cpp:10-34 (resizes the output like in_a, then adds)
void AddGPU(at::Tensor in_a, at::Tensor in_b, at::Tensor out_c) {
  check_cuda_contig(in_a, "in_a");
  check_cuda_contig(in_b, "in_b");
  TORCH_CHECK(in_a.scalar_type() == at::kFloat && in_b.scalar_type() == at::kFloat, "AddGPU takes float32 tensors");
  TORCH_CHECK(in_a.numel() == in_b.numel(), "AddGPU: element counts differ");
  c10::cuda::CUDAGuard guard(in_a.device());
  out_c.resize_(in_a.sizes());
  TORCH_CHECK(out_c.is_cuda() && out_c.scalar_type() == at::kFloat && out_c.is_contiguous(), "out_c must be a contiguous float32 CUDA tensor");
  WINO_CHECK(winoconv_add(in_a.data_ptr<float>(), in_b.data_ptr<float>(), out_c.data_ptr<float>(), in_a.numel(), stream_of()), "AddGPU");
}

// reference: src/split_and_concat.cpp:14-42.  in_a channels last ([B,H,W,C] or [B,D,H,W,C]),
// out [B*tiles, C, (bD,) bH, bW] pre-allocated by the caller.
void WinoSplit(at::Tensor in_a, at::Tensor out, int block_D, int block_H, int block_W, int output_block_size, int nD,
               int nH, int nW, bool two_dimension) {
  check_cuda_contig(in_a, "in_a");
  check_cuda_contig(out, "out");
  TORCH_CHECK(in_a.scalar_type() == at::kFloat && out.scalar_type() == at::kFloat, "WinoSplit takes float32 tensors");
  TORCH_CHECK(in_a.dim() == (two_dimension ? 4 : 5), "WinoSplit: in_a must be ", two_dimension ? "[B,H,W,C]" : "[B,D,H,W,C]");
  c10::cuda::CUDAGuard guard(in_a.device());
  const int B = in_a.size(0);
  int D = 1, H, W, C, bD = 1, oD = 1, tD = 1;
  if (two_dimension) {
    H = in_a.size(1); W = in_a.size(2); C = in_a.size(3);
  } else {
    D = in_a.size(1); H = in_a.size(2); W = in_a.size(3); C = in_a.size(4);
    bD = block_D; oD = output_block_size; tD = nD;
  }
  TORCH_CHECK(out.numel() == (int64_t)B * tD * nH * nW * C * bD * block_H * block_W, "WinoSplit: out has the wrong number of elements");
  WINO_CHECK(winoconv_split(in_a.data_ptr<float>(), out.data_ptr<float>(), B, D, H, W, C, bD, block_H, block_W, oD,
                            output_block_size, output_block_size, tD, nH, nW, stream_of()), "WinoSplit");
}

// reference: src/split_and_concat.cpp:44-78.  in_a [B*tiles, K, (m,) m, m]; out channels last, pre-allocated.
void WinoConcat(at::Tensor in_a, at::Tensor out, int output_block_size, bool two_dimension) {
  check_cuda_contig(in_a, "in_a");
  check_cuda_contig(out, "out");
  TORCH_CHECK(in_a.scalar_type() == at::kFloat && out.scalar_type() == at::kFloat, "WinoConcat takes float32 tensors");
  TORCH_CHECK(out.dim() == (two_dimension ? 4 : 5), "WinoConcat: out must be ", two_dimension ? "[B,H,W,K]" : "[B,D,H,W,K]");
  c10::cuda::CUDAGuard guard(in_a.device());
  const int m = output_block_size;
  const int N = in_a.size(0), K = in_a.size(1);
  int oD = 1, oH, oW, mD = 1;
  if (two_dimension) { oH = out.size(1); oW = out.size(2); }
  else { oD = out.size(1); oH = out.size(2); oW = out.size(3); mD = m; }
  const int nD = (oD + mD - 1) / mD, nH = (oH + m - 1) / m, nW = (oW + m - 1) / m;
  TORCH_CHECK(N % (nD * nH * nW) == 0, "WinoConcat: tile count is not a multiple of tiles per image");
  const int B = N / (nD * nH * nW);
  TORCH_CHECK(out.numel() == (int64_t)B * oD * oH * oW * K, "WinoConcat: out has the wrong number of elements");
  TORCH_CHECK(in_a.numel() == (int64_t)N * K * mD * m * m, "WinoConcat: in_a has the wrong number of elements");
  WINO_CHECK(winoconv_concat(in_a.data_ptr<float>(), out.data_ptr<float>(), B, oD, oH, oW, K, mD, m, m, stream_of()), "WinoConcat");
}

// reference: src/winograd_conv.cpp:16-127.  Input [B,D,H,W,C] already padded (the op is VALID-only),
// Weight [kD,kH,kW,C,K], Output [B,oD,oH,oW,K] allocated by the caller.  The three scratch tensors are
// used when they are large enough for this engine's layouts, otherwise scratch comes from torch's
// caching allocator; tmp_ptr_buffer (pointer tables for cuBLAS batched GEMM) is not needed.
void DWM(at::Tensor Input, at::Tensor Weight, at::Tensor Output, int stride, at::Tensor tmp_input_buffer,
         at::Tensor tmp_weight_buffer, at::Tensor tmp_product_buffer, at::Tensor /*tmp_ptr_buffer*/) {
  check_cuda_contig(Input, "Input");
  check_cuda_contig(Weight, "Weight");
  check_cuda_contig(Output, "Output");
  TORCH_CHECK(Input.dim() == 5 && Weight.dim() == 5 && Output.dim() == 5, "DWM takes Input [B,D,H,W,C], Weight [kD,kH,kW,C,K], Output [B,oD,oH,oW,K]");
  TORCH_CHECK(Weight.scalar_type() == Input.scalar_type() && Output.scalar_type() == Input.scalar_type(), "DWM: Input, Weight and Output must share a dtype");
  TORCH_CHECK(Weight.size(3) == Input.size(4), "DWM: channel mismatch between Input and Weight");
  TORCH_CHECK(stride == 1 || stride == 2, "DWM: stride must be 1 or 2");
  c10::cuda::CUDAGuard guard(Input.device());

  winoconv_desc_t d;
  memset(&d, 0, sizeof d);
  const bool flat = Input.size(1) == 1 && Weight.size(0) == 1;
  d.ndim = flat ? 2 : 3;
  d.batch = Input.size(0); d.c_in = Input.size(4); d.k_out = Weight.size(4);
  for (int i = 0; i < 3; ++i) {
    d.in_size[i] = Input.size(1 + i);
    d.ker_size[i] = Weight.size(i);
    d.stride[i] = (flat && i == 0) ? 1 : stride;
    d.pad[i] = 0;
  }
  d.tile_m = g_dwm_block.load();
  if (d.tile_m == 4 && !(flat && d.ker_size[1] == 3 && d.ker_size[2] == 3 && stride == 1)) d.tile_m = 2;
  d.dtype = dtype_code(Input, "Input");
  d.weight_layout = WINOCONV_W_RSCK;
  d.gemm_engine = WINOCONV_GEMM_AUTO;
  d.product_dtype = WINOCONV_F32;
  winoconv_plan_info_t info;
  WINO_CHECK(winoconv_plan(&d, &info), "DWM (plan)");
  TORCH_CHECK(Output.size(0) == d.batch && Output.size(1) == info.out_size[0] && Output.size(2) == info.out_size[1] &&
                  Output.size(3) == info.out_size[2] && Output.size(4) == d.k_out,
              "DWM: Output must be [", d.batch, ",", info.out_size[0], ",", info.out_size[1], ",", info.out_size[2], ",", d.k_out, "]");

  const auto act = Input.scalar_type();
  auto opts_act = Input.options();
  at::Tensor u = usable(tmp_weight_buffer, Input, act, info.filter_bytes)
                     ? tmp_weight_buffer
                     : at::empty({(int64_t)(info.filter_bytes / Input.element_size())}, opts_act);
  at::Tensor v = usable(tmp_input_buffer, Input, act, info.input_ws_bytes_min)
                     ? tmp_input_buffer
                     : at::empty({(int64_t)(info.input_ws_bytes / Input.element_size())}, opts_act);
  // products are fp32; a caller-provided buffer of any dtype will do if it is large enough
  at::Tensor m;
  if (tmp_product_buffer.defined() && tmp_product_buffer.is_cuda() && tmp_product_buffer.is_contiguous() &&
      tmp_product_buffer.device() == Input.device() &&
      (size_t)tmp_product_buffer.numel() * tmp_product_buffer.element_size() >= info.product_ws_bytes_min &&
      (reinterpret_cast<uintptr_t>(tmp_product_buffer.data_ptr()) & 15u) == 0)
    m = tmp_product_buffer;
  else
    m = at::empty({(int64_t)(info.product_ws_bytes / 4)}, opts_act.dtype(at::kFloat));

  void *s = stream_of();
  WINO_CHECK(winoconv_filter_transform(&d, Weight.data_ptr(), u.data_ptr(), s), "DWM (filter transform)");
  WINO_CHECK(winoconv_forward(&d, Input.data_ptr(), u.data_ptr(), nullptr, Output.data_ptr(), v.data_ptr(),
                              (size_t)v.numel() * v.element_size(), m.data_ptr(), (size_t)m.numel() * m.element_size(), s),
             "DWM (forward)");
}
