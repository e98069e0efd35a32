// Host-side interface of the tcgen05 GEMM (no device code: safe to include from plain C++).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace cw {

enum Act : int { kActNone = 0, kActGelu = 1, kActRelu = 2 };

struct GemmArgs {
  const void* a;
  const void* b;
  void* out;
  void* z_out = nullptr;
  const float* bias = nullptr;
  int M, N, K;
  bool trans_a, trans_b;
  bool is_bf16 = true;
  bool out_f32 = false;
  int act = kActNone;
  bool allow_split_k = true;
  int num_sms = 148;
  int* status = nullptr;
};

void gemm_launch(const GemmArgs& g, cudaStream_t stream);

}  // namespace cw
