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

// ---------------------------------------------------------------------------------------------------------
// Warp-per-row layer norm for hidden sizes up to 2048: a row lives in one warp's registers (NV 16-byte vectors
// per lane), the two statistics are warp shuffles, and nothing synchronises the CTA, so eight rows per CTA are in
// flight with all their loads outstanding.  Optionally fused with the residual add in front of the norm
// (reference: `x = x + dropout(...)` followed by `norm(x)`, benchmark/gpt2/gpt2.py:179-186): forward writes the sum
// and its normalised value, backward adds the gradient that reaches the sum directly.
constexpr int kWarpRows = 8;                 // warps (rows in flight) per CTA

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
  const T* h = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = to_f(h[i]);
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 raw;
  T* h = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < 8; ++i) h[i] = from_f<T>(f[i]);
  return raw;
}

template <typename T, int NV, bool HAS_RES>
__global__ void __launch_bounds__(32 * kWarpRows)
ln_fwd_warp_kernel(const T* __restrict__ x, const T* __restrict__ res, const float* __restrict__ gamma,
                   const float* __restrict__ beta, T* __restrict__ sum_out, T* __restrict__ y, float* __restrict__ mean_o,
                   float* __restrict__ rstd_o, int rows, int H, float eps) {
  const int lane = threadIdx.x & 31;
  const int warp = blockIdx.x * kWarpRows + (threadIdx.x >> 5);
  const int nwarps = gridDim.x * kWarpRows;
  const float inv_h = 1.0f / H;
  for (int row = warp; row < rows; row += nwarps) {
    const size_t base = static_cast<size_t>(row) * H;
    uint4 raw[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c = (v * 32 + lane) * 8;
      raw[v] = c < H ? *reinterpret_cast<const uint4*>(x + base + c) : make_uint4(0, 0, 0, 0);
    }
    // the next row of this warp goes to L2 while this one is processed (costs no registers)
    if (row + nwarps < rows) {
      const size_t nbase = static_cast<size_t>(row + nwarps) * H;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const int c = (v * 32 + lane) * 8;
        if (c < H) {
          asm volatile("prefetch.global.L2 [%0];" ::"l"(x + nbase + c));
          if (HAS_RES) asm volatile("prefetch.global.L2 [%0];" ::"l"(res + nbase + c));
        }
      }
    }
    if (HAS_RES) {
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const int c = (v * 32 + lane) * 8;
        if (c < H) {
          const uint4 r = *reinterpret_cast<const uint4*>(res + base + c);
          float a[8], b[8];
          unpack8<T>(raw[v], a);
          unpack8<T>(r, b);
#pragma unroll
          for (int i = 0; i < 8; ++i) a[i] += b[i];
          raw[v] = pack8<T>(a);                       // the normalised value is that of the stored (rounded) sum
          *reinterpret_cast<uint4*>(sum_out + base + c) = raw[v];
        }
      }
    }
    float s = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      float f[8];
      unpack8<T>(raw[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) s += f[i];
    }
    const float mean = warp_sum(s) * inv_h;
    float q = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      if ((v * 32 + lane) * 8 < H) {
        float f[8];
        unpack8<T>(raw[v], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) { const float d = f[i] - mean; q += d * d; }
      }
    }
    const float rstd = rsqrtf(warp_sum(q) * inv_h + eps);
    if (lane == 0) { mean_o[row] = mean; rstd_o[row] = rstd; }
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c = (v * 32 + lane) * 8;
      if (c < H) {
        float f[8];
        unpack8<T>(raw[v], f);
        const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma + c)), g1 = __ldg(reinterpret_cast<const float4*>(gamma + c + 4));
        const float4 b0 = __ldg(reinterpret_cast<const float4*>(beta + c)), b1 = __ldg(reinterpret_cast<const float4*>(beta + c + 4));
        const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = (f[i] - mean) * rstd * gg[i] + bb[i];
        *reinterpret_cast<uint4*>(y + base + c) = pack8<T>(f);
      }
    }
  }
}

// Backward of the above.  Each warp keeps the dgamma / dbeta partial sums of its rows in a shared-memory strip of its
// own (in registers they cost 112 registers per thread at H = 1600 and held the kernel at eight warps per SM, where it
// was bound by latency); the warps of a CTA are added up at the end and the CTA writes one partial row (summed by
// colsum2).
template <typename T, int NV, bool HAS_RES>
__global__ void __launch_bounds__(32 * kWarpRows, 2)
ln_bwd_warp_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ mean,
                   const float* __restrict__ rstd, const float* __restrict__ gamma, const T* __restrict__ dres,
                   T* __restrict__ dx, float* __restrict__ part_dgamma, float* __restrict__ part_dbeta, int rows, int H) {
  extern __shared__ __align__(16) float sacc[];            // [kWarpRows][2][H]
  const int lane = threadIdx.x & 31;
  const int warp = blockIdx.x * kWarpRows + (threadIdx.x >> 5);
  const int nwarps = gridDim.x * kWarpRows;
  const float inv_h = 1.0f / H;
  float* wdg = sacc + static_cast<size_t>(threadIdx.x >> 5) * 2 * H;
  float* wdb = wdg + H;
  for (int i = lane * 4; i < 2 * H; i += 128) *reinterpret_cast<float4*>(wdg + i) = make_float4(0.f, 0.f, 0.f, 0.f);
  __syncwarp();

  for (int row = warp; row < rows; row += nwarps) {
    const size_t base = static_cast<size_t>(row) * H;
    uint4 xr[NV], gr[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c = (v * 32 + lane) * 8;
      const bool ok = c < H;
      xr[v] = ok ? *reinterpret_cast<const uint4*>(x + base + c) : make_uint4(0, 0, 0, 0);
      gr[v] = ok ? *reinterpret_cast<const uint4*>(dy + base + c) : make_uint4(0, 0, 0, 0);
    }
    // requests that cost no registers: this row's residual gradient (read in the second pass) and the next row's
    // operands go to L2 while the first pass runs
    {
      const size_t nbase = static_cast<size_t>(row + nwarps) * H;
      const bool has_next = row + nwarps < rows;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const int c = (v * 32 + lane) * 8;
        if (c < H) {
          if (HAS_RES) asm volatile("prefetch.global.L2 [%0];" ::"l"(dres + base + c));
          if (has_next) {
            asm volatile("prefetch.global.L2 [%0];" ::"l"(x + nbase + c));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(dy + nbase + c));
          }
        }
      }
    }
    const float mu = mean[row], rs = rstd[row];
    const float nmr = -mu * rs;
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c = (v * 32 + lane) * 8;
      if (c < H) {
        float xf[8], df[8];
        unpack8<T>(xr[v], xf);
        unpack8<T>(gr[v], df);
        const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma + c)), g1 = __ldg(reinterpret_cast<const float4*>(gamma + c + 4));
        const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        float4* pg = reinterpret_cast<float4*>(wdg + c);
        float4* pb = reinterpret_cast<float4*>(wdb + c);
        float4 a0 = pg[0], a1 = pg[1], b0 = pb[0], b1 = pb[1];
        float ag[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        float ab[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xhat = fmaf(xf[i], rs, nmr);
          ag[i] = fmaf(df[i], xhat, ag[i]);
          ab[i] += df[i];
          const float g = df[i] * gg[i];
          s1 += g;
          s2 = fmaf(g, xhat, s2);
        }
        pg[0] = make_float4(ag[0], ag[1], ag[2], ag[3]);
        pg[1] = make_float4(ag[4], ag[5], ag[6], ag[7]);
        pb[0] = make_float4(ab[0], ab[1], ab[2], ab[3]);
        pb[1] = make_float4(ab[4], ab[5], ab[6], ab[7]);
      }
    }
    const float m1 = warp_sum(s1) * inv_h, m2 = warp_sum(s2) * inv_h;
    // dx = rs * (dy * gamma - m1 - xhat * m2) = dy * (rs * gamma) + x * kx + k0
    const float kx = -rs * rs * m2, k0 = rs * (mu * rs * m2 - m1);
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c = (v * 32 + lane) * 8;
      if (c < H) {
        float xf[8], df[8], o[8];
        unpack8<T>(xr[v], xf);
        unpack8<T>(gr[v], df);
        const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma + c)), g1 = __ldg(reinterpret_cast<const float4*>(gamma + c + 4));
        const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = fmaf(df[i], rs * gg[i], fmaf(xf[i], kx, k0));
        if (HAS_RES) {
          float rf[8];
          unpack8<T>(*reinterpret_cast<const uint4*>(dres + base + c), rf);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += rf[i];
        }
        *reinterpret_cast<uint4*>(dx + base + c) = pack8<T>(o);
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int w = 0; w < kWarpRows; ++w) {
      a += sacc[static_cast<size_t>(w) * 2 * H + i];
      b += sacc[static_cast<size_t>(w) * 2 * H + H + i];
    }
    part_dgamma[static_cast<size_t>(blockIdx.x) * H + i] = a;
    part_dbeta[static_cast<size_t>(blockIdx.x) * H + i] = b;
  }
}

template <typename T, int NV, bool HAS_RES>
static void launch_ln_bwd_warp(int grid, size_t smem, cudaStream_t stream, const void* dy, const void* x, const float* mean,
                               const float* rstd, const float* gamma, const void* dres, void* dx, float* pdg, float* pdb,
                               int rows, int H) {
  auto kern = ln_bwd_warp_kernel<T, NV, HAS_RES>;
  static bool done = false;
  if (!done) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kWarpRows * 2 * 2048 * 4));
    done = true;
  }
  kern<<<grid, 32 * kWarpRows, smem, stream>>>(reinterpret_cast<const T*>(dy), reinterpret_cast<const T*>(x), mean, rstd, gamma,
                                               reinterpret_cast<const T*>(dres), reinterpret_cast<T*>(dx), pdg, pdb, rows, H);
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

// ---- warp-per-row path (hidden <= 2048) --------------------------------------------------------------------
constexpr int kWarpMaxH = 2048;
#define DISPATCH_NV(H, ...)                                        \
  {                                                                \
    const int need_ = ((H) / 8 + 31) / 32;                         \
    if (need_ <= 1) { constexpr int NV = 1; __VA_ARGS__ }          \
    else if (need_ <= 2) { constexpr int NV = 2; __VA_ARGS__ }     \
    else if (need_ <= 4) { constexpr int NV = 4; __VA_ARGS__ }     \
    else if (need_ <= 7) { constexpr int NV = 7; __VA_ARGS__ }     \
    else { constexpr int NV = 8; __VA_ARGS__ }                     \
  }
#define DISPATCH_16_NV(x, ...)                                     \
  if ((x).scalar_type() == torch::kBFloat16) {                     \
    using T = __nv_bfloat16;                                       \
    DISPATCH_NV((x).size(1), __VA_ARGS__)                          \
  } else {                                                         \
    using T = __half;                                              \
    DISPATCH_NV((x).size(1), __VA_ARGS__)                          \
  }

static bool warp_path(const torch::Tensor& x) { return x.size(1) <= kWarpMaxH; }

// y = LN(x (+ residual)); returns {y, mean, rstd, sum}: `sum` is x + residual (undefined without a residual).
std::vector<torch::Tensor> layer_norm_fwd_res(torch::Tensor x, c10::optional<torch::Tensor> residual, torch::Tensor gamma,
                                              torch::Tensor beta, double eps) {
  check_rows(x);
  const bool has_res = residual.has_value() && residual->defined();
  const int rows = x.size(0), H = x.size(1);
  TORCH_CHECK(gamma.scalar_type() == torch::kFloat32 && beta.scalar_type() == torch::kFloat32 && gamma.is_contiguous() &&
              beta.is_contiguous() && gamma.numel() == H && beta.numel() == H, "norm parameters must be contiguous fp32 [H]");
  torch::Tensor sum;
  if (has_res) {
    check_rows(*residual);
    TORCH_CHECK(residual->sizes() == x.sizes() && residual->scalar_type() == x.scalar_type());
    if (!warp_path(x)) {                       // wide rows: separate add, then the CTA-per-row kernel
      sum = x + *residual;
      auto r = layer_norm_fwd(sum, gamma, beta, eps);
      r.push_back(sum);
      return r;
    }
    sum = torch::empty_like(x);
  } else if (!warp_path(x)) {
    auto r = layer_norm_fwd(x, gamma, beta, eps);
    r.push_back(torch::Tensor());
    return r;
  }
  auto y = torch::empty_like(x);
  auto mean = torch::empty({rows}, x.options().dtype(torch::kFloat32));
  auto rstd = torch::empty({rows}, x.options().dtype(torch::kFloat32));
  if (rows == 0) return {y, mean, rstd, sum};
  auto stream = at::cuda::getCurrentCUDAStream();
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const int grid = std::max(1, std::min((rows + kWarpRows - 1) / kWarpRows, sms * 6));
  if (has_res) {
    DISPATCH_16_NV(x, ln_fwd_warp_kernel<T, NV, true><<<grid, 32 * kWarpRows, 0, stream>>>(
                          reinterpret_cast<const T*>(x.data_ptr()), reinterpret_cast<const T*>(residual->data_ptr()),
                          gamma.data_ptr<float>(), beta.data_ptr<float>(), reinterpret_cast<T*>(sum.data_ptr()),
                          reinterpret_cast<T*>(y.data_ptr()), mean.data_ptr<float>(), rstd.data_ptr<float>(), rows, H,
                          static_cast<float>(eps));)
  } else {
    DISPATCH_16_NV(x, ln_fwd_warp_kernel<T, NV, false><<<grid, 32 * kWarpRows, 0, stream>>>(
                          reinterpret_cast<const T*>(x.data_ptr()), nullptr, gamma.data_ptr<float>(), beta.data_ptr<float>(),
                          nullptr, reinterpret_cast<T*>(y.data_ptr()), mean.data_ptr<float>(), rstd.data_ptr<float>(), rows, H,
                          static_cast<float>(eps));)
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {y, mean, rstd, sum};
}

// {dx, dgamma, dbeta} with dx = LN'(dy) (+ dres, the gradient that reaches the normalised tensor directly).
std::vector<torch::Tensor> layer_norm_bwd_res(torch::Tensor dy, torch::Tensor x, torch::Tensor mean, torch::Tensor rstd,
                                              torch::Tensor gamma, c10::optional<torch::Tensor> dres) {
  check_rows(x);
  check_rows(dy);
  const bool has_res = dres.has_value() && dres->defined();
  if (!warp_path(x)) {
    auto r = layer_norm_bwd(dy, x, mean, rstd, gamma);
    if (has_res) r[0].add_(*dres);
    return r;
  }
  const int rows = x.size(0), H = x.size(1);
  TORCH_CHECK(gamma.scalar_type() == torch::kFloat32 && gamma.is_contiguous() && gamma.numel() == H);
  if (has_res) {
    check_rows(*dres);
    TORCH_CHECK(dres->sizes() == x.sizes() && dres->scalar_type() == x.scalar_type());
  }
  auto dx = torch::empty_like(x);
  auto f32 = x.options().dtype(torch::kFloat32);
  auto dgamma = torch::zeros({H}, f32), dbeta = torch::zeros({H}, f32);
  if (rows == 0) return {dx, dgamma, dbeta};
  auto stream = at::cuda::getCurrentCUDAStream();
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const int grid = std::max(1, std::min((rows + kWarpRows - 1) / kWarpRows, 2 * sms));
  auto scratch = torch::empty({2, grid, H}, f32);
  float* pdg = scratch.data_ptr<float>();
  float* pdb = pdg + static_cast<size_t>(grid) * H;
  const size_t smem = static_cast<size_t>(kWarpRows) * 2 * H * sizeof(float);
  if (has_res) {
    DISPATCH_16_NV(x, (launch_ln_bwd_warp<T, NV, true>(grid, smem, stream, dy.data_ptr(), x.data_ptr(), mean.data_ptr<float>(),
                                                       rstd.data_ptr<float>(), gamma.data_ptr<float>(), dres->data_ptr(),
                                                       dx.data_ptr(), pdg, pdb, rows, H));)
  } else {
    DISPATCH_16_NV(x, (launch_ln_bwd_warp<T, NV, false>(grid, smem, stream, dy.data_ptr(), x.data_ptr(), mean.data_ptr<float>(),
                                                        rstd.data_ptr<float>(), gamma.data_ptr<float>(), nullptr, dx.data_ptr(),
                                                        pdg, pdb, rows, H));)
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  colsum2_kernel<<<(H + 255) / 256, 256, 0, stream>>>(pdg, pdb, dgamma.data_ptr<float>(), dbeta.data_ptr<float>(), grid, H);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {dx, dgamma, dbeta};
}

}  // namespace cw
