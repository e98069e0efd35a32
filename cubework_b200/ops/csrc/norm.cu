// Layer-norm kernels (forward, backward, and the two-pass pieces used when the hidden dimension is
// split over a process group).  One CTA per row, the row held in registers (16-byte loads), statistics in
// fp32.  Backward is persistent over rows so each thread keeps partial dgamma / dbeta for its columns in
// registers; partials are written to a scratch buffer [ctas, H] and summed by a second kernel.
//
// Replaces nn.LayerNorm in LayerNorm1D (cubework/module/parallel_1d/module.py:72-87), the elementwise
// chains of _Layernorm_2D (parallel_2d/_operation.py:307-347 + module.py:142-171) and _Layernorm3D
// (parallel_3d/_operation.py:252-313).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAException.h>
#include <torch/extension.h>

#include "common.cuh"

namespace cw {

constexpr int kNT = 256;
constexpr int kMaxVPT = 8;   // 8 vectors x 8 elements x 256 threads = 16384 columns; kernels are compiled for 1, 2, 4, 8

template <typename T, int VPT>
__device__ __forceinline__ int load_row(const T* row, int H, float (&x)[VPT][8]) {
  int n = 0;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int c = (v * kNT + threadIdx.x) * 8;
    if (c < H) {
      Vec8<T> t;
      t.load(row + c);
      t.unpack(x[v]);
      n = v + 1;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) x[v][i] = 0.f;
    }
  }
  return n;
}

// MODE 0: local statistics (plain layer norm).  MODE 1: statistics supplied (sharded, pass 2).
template <typename T, int MODE, int VPT>
__global__ void __launch_bounds__(kNT) ln_fwd_kernel(const T* __restrict__ x, const float* __restrict__ gamma,
                                                     const float* __restrict__ beta, T* __restrict__ y,
                                                     float* __restrict__ mean_io, float* __restrict__ rstd_io, int rows,
                                                     int H, float eps) {
  __shared__ float red[64];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    float xv[VPT][8];
    load_row(x + static_cast<size_t>(row) * H, H, xv);
    float mean, rstd;
    if (MODE == 0) {
      float s = 0.f, dummy = 0.f;
#pragma unroll
      for (int v = 0; v < VPT; ++v)
#pragma unroll
        for (int i = 0; i < 8; ++i) s += xv[v][i];
      block_sum2<kNT>(s, dummy, red);
      mean = s / H;
      float q = 0.f;
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        const int c = (v * kNT + threadIdx.x) * 8;
        if (c < H) {
#pragma unroll
          for (int i = 0; i < 8; ++i) { const float d = xv[v][i] - mean; q += d * d; }
        }
      }
      block_sum2<kNT>(q, dummy, red);
      rstd = rsqrtf(q / H + eps);
      if (threadIdx.x == 0) { mean_io[row] = mean; rstd_io[row] = rstd; }
    } else {
      mean = mean_io[row];
      rstd = rstd_io[row];
    }
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int c = (v * kNT + threadIdx.x) * 8;
      if (c < H) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float n = (xv[v][i] - mean) * rstd;
          if (gamma != nullptr) n = n * __ldg(gamma + c + i) + __ldg(beta + c + i);
          o[i] = n;
        }
        Vec8<T> t;
        t.pack(o);
        t.store(y + static_cast<size_t>(row) * H + c);
      }
    }
  }
}

// Per-row [sum x, sum x^2] for the sharded layer norm (pass 1).
template <typename T, int VPT>
__global__ void __launch_bounds__(kNT) row_moments_kernel(const T* __restrict__ x, float* __restrict__ mom, int rows,
                                                          int H) {
  __shared__ float red[64];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    float xv[VPT][8];
    load_row(x + static_cast<size_t>(row) * H, H, xv);
    float s = 0.f, q = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v)
#pragma unroll
      for (int i = 0; i < 8; ++i) { s += xv[v][i]; q += xv[v][i] * xv[v][i]; }
    block_sum2<kNT>(s, q, red);
    if (threadIdx.x == 0) { mom[2 * row] = s; mom[2 * row + 1] = q; }
  }
}

// Backward.  MODE 0: everything local.  MODE 1: only row sums [sum g, sum g*xhat] + parameter partials.
// MODE 2: only dx, row sums supplied (already reduced over the group) and divided by `hidden`.
template <typename T, int MODE, int VPT>
__global__ void __launch_bounds__(kNT) ln_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                     const float* __restrict__ mean, const float* __restrict__ rstd,
                                                     const float* __restrict__ gamma, T* __restrict__ dx,
                                                     float* __restrict__ row_sums, float* __restrict__ part_dgamma,
                                                     float* __restrict__ part_dbeta, int rows, int H, float hidden) {
  __shared__ float red[64];
  float dg[VPT][8], db[VPT][8];
#pragma unroll
  for (int v = 0; v < VPT; ++v)
#pragma unroll
    for (int i = 0; i < 8; ++i) { dg[v][i] = 0.f; db[v][i] = 0.f; }

  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    float xv[VPT][8], gv[VPT][8];
    load_row(x + static_cast<size_t>(row) * H, H, xv);
    load_row(dy + static_cast<size_t>(row) * H, H, gv);
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int c = (v * kNT + threadIdx.x) * 8;
      if (c < H) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xhat = (xv[v][i] - mu) * rs;
          const float d = gv[v][i];
          if (MODE != 2) { dg[v][i] += d * xhat; db[v][i] += d; }
          const float g = gamma != nullptr ? d * __ldg(gamma + c + i) : d;
          xv[v][i] = xhat;
          gv[v][i] = g;
          s1 += g;
          s2 += g * xhat;
        }
      }
    }
    if (MODE == 2) {
      s1 = row_sums[2 * row];
      s2 = row_sums[2 * row + 1];
    } else {
      block_sum2<kNT>(s1, s2, red);
      if (MODE == 1 && threadIdx.x == 0) { row_sums[2 * row] = s1; row_sums[2 * row + 1] = s2; }
    }
    if (MODE != 1) {
      const float m1 = s1 / hidden, m2 = s2 / hidden;
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        const int c = (v * kNT + threadIdx.x) * 8;
        if (c < H) {
          float o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = (gv[v][i] - m1 - xv[v][i] * m2) * rs;
          Vec8<T> t;
          t.pack(o);
          t.store(dx + static_cast<size_t>(row) * H + c);
        }
      }
    }
  }
  if (MODE != 2) {
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int c = (v * kNT + threadIdx.x) * 8;
      if (c < H) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          part_dgamma[static_cast<size_t>(blockIdx.x) * H + c + i] = dg[v][i];
          part_dbeta[static_cast<size_t>(blockIdx.x) * H + c + i] = db[v][i];
        }
      }
    }
  }
}

// out[c] = sum_p part[p, c] for two partial buffers at once.
__global__ void colsum2_kernel(const float* __restrict__ pa, const float* __restrict__ pb, float* __restrict__ oa,
                               float* __restrict__ ob, int P, int H) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float a = 0.f, b = 0.f;
  for (int p = 0; p < P; ++p) {
    a += pa[static_cast<size_t>(p) * H + c];
    b += pb[static_cast<size_t>(p) * H + c];
  }
  oa[c] = a;
  ob[c] = b;
}

// ---------------------------------------------------------------------------------------- host side
static void check_rows(const torch::Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous(), "expected a contiguous 2-D CUDA tensor");
  TORCH_CHECK(x.size(1) % 8 == 0 && x.size(1) <= kNT * 8 * kMaxVPT, "hidden size must be a multiple of 8 and <= 16384");
  TORCH_CHECK(x.scalar_type() == torch::kBFloat16 || x.scalar_type() == torch::kFloat16, "expected bf16 / fp16");
}
static int row_grid(int rows) {
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return std::max(1, std::min(rows, sms * 8));
}
static const float* fptr(const c10::optional<torch::Tensor>& t) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->scalar_type() == torch::kFloat32 && t->is_contiguous(), "norm parameters must be contiguous fp32");
  return t->data_ptr<float>();
}

#define DISPATCH_VPT(H, ...)                                        \
  {                                                                 \
    const int need_ = ((H) / 8 + kNT - 1) / kNT;                    \
    if (need_ <= 1) { constexpr int VPT = 1; __VA_ARGS__ }          \
    else if (need_ <= 2) { constexpr int VPT = 2; __VA_ARGS__ }     \
    else if (need_ <= 4) { constexpr int VPT = 4; __VA_ARGS__ }     \
    else { constexpr int VPT = 8; __VA_ARGS__ }                     \
  }
#define DISPATCH_16(x, ...)                                         \
  if ((x).scalar_type() == torch::kBFloat16) {                      \
    using T = __nv_bfloat16;                                        \
    DISPATCH_VPT((x).size(1), __VA_ARGS__)                          \
  } else {                                                          \
    using T = __half;                                               \
    DISPATCH_VPT((x).size(1), __VA_ARGS__)                          \
  }

std::vector<torch::Tensor> layer_norm_fwd(torch::Tensor x, torch::Tensor gamma, torch::Tensor beta, double eps) {
  check_rows(x);
  const int rows = x.size(0), H = x.size(1);
  auto y = torch::empty_like(x);
  auto mean = torch::empty({rows}, x.options().dtype(torch::kFloat32));
  auto rstd = torch::empty({rows}, x.options().dtype(torch::kFloat32));
  if (rows == 0) return {y, mean, rstd};
  auto stream = at::cuda::getCurrentCUDAStream();
  DISPATCH_16(x, ln_fwd_kernel<T, 0, VPT><<<row_grid(rows), kNT, 0, stream>>>(
                     reinterpret_cast<const T*>(x.data_ptr()), fptr(gamma), fptr(beta), reinterpret_cast<T*>(y.data_ptr()),
                     mean.data_ptr<float>(), rstd.data_ptr<float>(), rows, H, static_cast<float>(eps));)
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {y, mean, rstd};
}

torch::Tensor norm_apply(torch::Tensor x, torch::Tensor mean, torch::Tensor rstd, c10::optional<torch::Tensor> gamma,
                         c10::optional<torch::Tensor> beta) {
  check_rows(x);
  const int rows = x.size(0), H = x.size(1);
  auto y = torch::empty_like(x);
  if (rows == 0) return y;
  auto stream = at::cuda::getCurrentCUDAStream();
  DISPATCH_16(x, ln_fwd_kernel<T, 1, VPT><<<row_grid(rows), kNT, 0, stream>>>(
                     reinterpret_cast<const T*>(x.data_ptr()), fptr(gamma), fptr(beta), reinterpret_cast<T*>(y.data_ptr()),
                     mean.data_ptr<float>(), rstd.data_ptr<float>(), rows, H, 0.f);)
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return y;
}

torch::Tensor row_moments(torch::Tensor x) {
  check_rows(x);
  const int rows = x.size(0), H = x.size(1);
  auto mom = torch::empty({rows, 2}, x.options().dtype(torch::kFloat32));
  if (rows == 0) return mom;
  auto stream = at::cuda::getCurrentCUDAStream();
  DISPATCH_16(x, row_moments_kernel<T, VPT><<<row_grid(rows), kNT, 0, stream>>>(reinterpret_cast<const T*>(x.data_ptr()),
                                                                             mom.data_ptr<float>(), rows, H);)
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return mom;
}

// Launches the backward kernel on caller-provided scratch: part_dgamma / part_dbeta are [grid, H] fp32.
template <int MODE>
static void ln_bwd_launch(const torch::Tensor& dy, const torch::Tensor& x, const float* mean, const float* rstd,
                          const float* gamma, void* dx, float* row_sums, float* pdg, float* pdb, int grid, float hidden,
                          cudaStream_t stream) {
  const int rows = x.size(0), H = x.size(1);
  DISPATCH_16(x, ln_bwd_kernel<T, MODE, VPT><<<grid, kNT, 0, stream>>>(
                     reinterpret_cast<const T*>(dy.data_ptr()), reinterpret_cast<const T*>(x.data_ptr()), mean, rstd, gamma,
                     reinterpret_cast<T*>(dx), row_sums, pdg, pdb, rows, H, hidden);)
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

static int bwd_grid(int rows) {
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return std::max(1, std::min(rows, sms * 2));
}

std::vector<torch::Tensor> layer_norm_bwd(torch::Tensor dy, torch::Tensor x, torch::Tensor mean, torch::Tensor rstd,
                                          torch::Tensor gamma) {
  check_rows(x);
  check_rows(dy);
  const int rows = x.size(0), H = x.size(1);
  auto dx = torch::empty_like(x);
  auto f32 = x.options().dtype(torch::kFloat32);
  auto dgamma = torch::zeros({H}, f32), dbeta = torch::zeros({H}, f32);
  if (rows == 0) return {dx, dgamma, dbeta};
  const int grid = bwd_grid(rows);
  auto scratch = torch::empty({2, grid, H}, f32);
  auto stream = at::cuda::getCurrentCUDAStream();
  float* pdg = scratch.data_ptr<float>();
  float* pdb = pdg + static_cast<size_t>(grid) * H;
  ln_bwd_launch<0>(dy, x, mean.data_ptr<float>(), rstd.data_ptr<float>(), fptr(gamma), dx.data_ptr(), nullptr, pdg, pdb,
                   grid, static_cast<float>(H), stream);
  colsum2_kernel<<<(H + 255) / 256, 256, 0, stream>>>(pdg, pdb, dgamma.data_ptr<float>(), dbeta.data_ptr<float>(), grid, H);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {dx, dgamma, dbeta};
}

std::vector<torch::Tensor> norm_bwd_partials(torch::Tensor dy, torch::Tensor x, torch::Tensor mean, torch::Tensor rstd,
                                             c10::optional<torch::Tensor> gamma) {
  check_rows(x);
  check_rows(dy);
  const int rows = x.size(0), H = x.size(1);
  auto f32 = x.options().dtype(torch::kFloat32);
  auto sums = torch::empty({rows, 2}, f32);
  auto dgamma = torch::zeros({H}, f32), dbeta = torch::zeros({H}, f32);
  if (rows == 0) return {sums, dgamma, dbeta};
  const int grid = bwd_grid(rows);
  auto scratch = torch::empty({2, grid, H}, f32);
  auto stream = at::cuda::getCurrentCUDAStream();
  float* pdg = scratch.data_ptr<float>();
  float* pdb = pdg + static_cast<size_t>(grid) * H;
  ln_bwd_launch<1>(dy, x, mean.data_ptr<float>(), rstd.data_ptr<float>(), fptr(gamma), nullptr, sums.data_ptr<float>(), pdg,
                   pdb, grid, 1.f, stream);
  colsum2_kernel<<<(H + 255) / 256, 256, 0, stream>>>(pdg, pdb, dgamma.data_ptr<float>(), dbeta.data_ptr<float>(), grid, H);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {sums, dgamma, dbeta};
}

torch::Tensor norm_bwd_apply(torch::Tensor dy, torch::Tensor x, torch::Tensor mean, torch::Tensor rstd,
                             c10::optional<torch::Tensor> gamma, torch::Tensor sums, double hidden) {
  check_rows(x);
  check_rows(dy);
  TORCH_CHECK(sums.scalar_type() == torch::kFloat32 && sums.is_contiguous());
  const int rows = x.size(0);
  auto dx = torch::empty_like(x);
  if (rows == 0) return dx;
  auto stream = at::cuda::getCurrentCUDAStream();
  ln_bwd_launch<2>(dy, x, mean.data_ptr<float>(), rstd.data_ptr<float>(), fptr(gamma), dx.data_ptr(), sums.data_ptr<float>(),
                   nullptr, nullptr, row_grid(rows), static_cast<float>(hidden), stream);
  return dx;
}

}  // namespace cw
