// Operator surface of the reference's pybind module (pybind/extern.hpp:1-9, src/common.hpp:8-19),
// re-implemented on the winoconv_b200 C ABI.  The reference templates these on the element type and
// binds only <float> (pybind/bind.cpp:19-24); here one function per op dispatches on the tensor dtype.
#pragma once

#include <string>

#include <torch/extension.h>

class Foo {
 public:
  void setKey(int key) { key_ = key; }
  int getKey() const { return key_; }
  std::string toString() const { return "< Foo, key: " + std::to_string(key_) + " > "; }

 private:
  int key_ = 0;
};

void AddGPU(at::Tensor in_a, at::Tensor in_b, at::Tensor out_c);
void WinoSplit(at::Tensor in_a, at::Tensor out, int block_D, int block_H, int block_W, int output_block_size, int nD,
               int nH, int nW, bool two_dimension);
void WinoConcat(at::Tensor in_a, at::Tensor out, int output_block_size, bool two_dimension);
void DWM(at::Tensor Input, at::Tensor Weight, at::Tensor Output, int stride, at::Tensor tmp_input_buffer,
         at::Tensor tmp_weight_buffer, at::Tensor tmp_product_buffer, at::Tensor tmp_ptr_buffer);

// Output block the DWM op uses: 2 (the reference's only block size, default) or 4 / 0 (= F(4x4,3x3)
// wherever it applies).  Not part of the reference surface.
void set_dwm_output_block(int m);
int get_dwm_output_block();
