// Bandwidth-bound kernels: vocab-parallel softmax cross-entropy pieces, activation backward fused with the
// bias gradient, column sums, masked embedding lookup and its scatter-add backward.
//
// Replace: the fp32 elementwise chain of _VocabParallelCrossEntropy{1,2,3}D (cubework/module/loss/
// loss_1d.py:14-79), F.gelu / ReLU backward + bias-gradient sums after dense_1 / fc1
// (benchmark/gpt2/gpt2.py:116-117, opt/opt.py:199-200), F.embedding + masking in the vocab-parallel
// embeddings (parallel_1d/module.py:441-455).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAException.h>
#include <torch/extension.h>

#include "common.cuh"

namespace cw {

constexpr int kCeThreads = 256;

// ---- cross-entropy -------------------------------------------------------------------------------------
// stats[row] = (max, sum exp(x - max), logit of the target if it falls in [vocab_start, vocab_start + V))
template <typename T>
__global__ void __launch_bounds__(kCeThreads) ce_stats_kernel(const T* __restrict__ logits,
                                                              const int64_t* __restrict__ targets,
                                                              float* __restrict__ stats, int rows, int V,
                                                              int64_t vocab_start) {
  __shared__ float red[64];
  const int row = blockIdx.x;
  if (row >= rows) return;
  const T* x = logits + static_cast<size_t>(row) * V;
  float m = -INFINITY, s = 0.f;
  const bool vec = (V % 8 == 0);
  if (vec) {
    for (int c = threadIdx.x * 8; c < V; c += kCeThreads * 8) {
      Vec8<T> t;
      t.load(x + c);
      float f[8];
      t.unpack(f);
      float lm = f[0];
#pragma unroll
      for (int i = 1; i < 8; ++i) lm = fmaxf(lm, f[i]);
      const float nm = fmaxf(m, lm);
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc += __expf(f[i] - nm);
      s = s * __expf(m - nm) + acc;
      m = nm;
    }
  } else {
    for (int c = threadIdx.x; c < V; c += kCeThreads) {
      const float f = to_f(x[c]);
      const float nm = fmaxf(m, f);
      s = s * __expf(m - nm) + __expf(f - nm);
      m = nm;
    }
  }
  const float gm = block_max<kCeThreads>(m, red);
  float part = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  float dummy = 0.f;
  block_sum2<kCeThreads>(part, dummy, red);
  if (threadIdx.x == 0) {
    const int64_t t = targets[row] - vocab_start;
    stats[3 * row + 0] = gm;
    stats[3 * row + 1] = part;
    stats[3 * row + 2] = (t >= 0 && t < V) ? to_f(x[t]) : 0.f;
  }
}

// grad[row, c] = (exp(x - gmax) / gsum - [c == target]) * scale[row]
template <typename T>
__global__ void __launch_bounds__(kCeThreads) ce_grad_kernel(const T* __restrict__ logits,
                                                             const int64_t* __restrict__ targets,
                                                             const float* __restrict__ gmax,
                                                             const float* __restrict__ gsum,
                                                             const float* __restrict__ scale, T* __restrict__ grad,
                                                             int rows, int V, int64_t vocab_start) {
  const int row = blockIdx.x;
  if (row >= rows) return;
  const T* x = logits + static_cast<size_t>(row) * V;
  T* g = grad + static_cast<size_t>(row) * V;
  const float mx = gmax[row], inv = 1.f / gsum[row], sc = scale[row];
  const int64_t t = targets[row] - vocab_start;
  if (V % 8 == 0) {
    for (int c = threadIdx.x * 8; c < V; c += kCeThreads * 8) {
      Vec8<T> v;
      v.load(x + c);
      float f[8];
      v.unpack(f);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float p = __expf(f[i] - mx) * inv;
        if (c + i == t) p -= 1.f;
        f[i] = p * sc;
      }
      v.pack(f);
      v.store(g + c);
    }
  } else {
    for (int c = threadIdx.x; c < V; c += kCeThreads) {
      float p = __expf(to_f(x[c]) - mx) * inv;
      if (c == t) p -= 1.f;
      g[c] = from_f<T>(p * sc);
    }
  }
}

// ---- activation backward + column sums --------------------------------------------------------------------
// d/dx of x * Phi(x) = Phi(x) + x * phi(x), with the error function from Abramowitz & Stegun 7.1.26 (absolute error
// below 1.5e-7, far below the resolution of a 16-bit gradient).  Its exp(-x^2 / 2) is the density's exponential as
// well, so one exponential, one reciprocal and a few multiply-adds serve both terms; erff alone costs more than that.
__device__ __forceinline__ float gelu_grad_fast(float x) {
  const float ax = fabsf(x) * 0.70710678118654752f;
  const float t = __fdividef(1.0f, fmaf(0.3275911f, ax, 1.0f));
  float poly = fmaf(t, 1.061405429f, -1.453152027f);
  poly = fmaf(t, poly, 1.421413741f);
  poly = fmaf(t, poly, -0.284496736f);
  poly = fmaf(t, poly, 0.254829592f);
  poly *= t;
  const float e = __expf(-ax * ax);
  const float cdf = 0.5f * (1.0f + copysignf(1.0f - poly * e, x));
  return fmaf(x, 0.3989422804014327f * e, cdf);
}

// Each CTA owns a stripe of 2048 columns (256 threads x 8) and a range of rows; per-thread column sums stay
// in registers and are written as partials[blockIdx.y, N].  Two rows are in flight per thread.
template <typename T, int ACT, bool WRITE_DZ, bool WANT_SUM>
__global__ void __launch_bounds__(256) act_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ z,
                                                      T* __restrict__ dz, float* __restrict__ partials, int M, int N,
                                                      int rows_per_cta) {
  const int c = (blockIdx.x * 256 + threadIdx.x) * 8;
  if (c >= N) return;
  const int r0 = blockIdx.y * rows_per_cta;
  const int r1 = min(r0 + rows_per_cta, M);
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  auto one_row = [&](const Vec8<T>& vd, const Vec8<T>& vz, size_t off) {
    float d[8];
    vd.unpack(d);
    if (ACT != 0) {
      float zz[8];
      vz.unpack(zz);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (ACT == 1) d[i] *= gelu_grad_fast(zz[i]);
        else d[i] = zz[i] > 0.f ? d[i] : 0.f;
      }
    }
    if (WRITE_DZ) {
      Vec8<T> vo;
      vo.pack(d);
      vo.store(dz + off);
      if (WANT_SUM) vo.unpack(d);   // sum what was stored, so db matches the rounded dz
    }
    if (WANT_SUM) {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += d[i];
    }
  };
  int r = r0;
  for (; r + 1 < r1; r += 2) {
    const size_t off0 = static_cast<size_t>(r) * N + c, off1 = off0 + N;
    if (r + 9 < r1) {
      // the rows this thread reads four iterations from now go to L2 (costs no registers)
      const size_t offp = off0 + static_cast<size_t>(8) * N;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(dy + offp));
      asm volatile("prefetch.global.L2 [%0];" ::"l"(dy + offp + N));
      if (ACT != 0) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(z + offp));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(z + offp + N));
      }
    }
    Vec8<T> vd0, vd1, vz0, vz1;
    vd0.load(dy + off0);
    vd1.load(dy + off1);
    if (ACT != 0) {
      vz0.load(z + off0);
      vz1.load(z + off1);
    }
    one_row(vd0, vz0, off0);
    one_row(vd1, vz1, off1);
  }
  if (r < r1) {
    const size_t off = static_cast<size_t>(r) * N + c;
    Vec8<T> vd, vz;
    vd.load(dy + off);
    if (ACT != 0) vz.load(z + off);
    one_row(vd, vz, off);
  }
  if (WANT_SUM) {
#pragma unroll
    for (int i = 0; i < 8; ++i) partials[static_cast<size_t>(blockIdx.y) * N + c + i] = acc[i];
  }
}

// out[c] = sum_p part[p, c].  A CTA of 64 columns x 4 row groups: every thread keeps four loads in flight, the row
// groups meet in shared memory (one thread per column over all P rows left a handful of CTAs waiting on one load each).
__global__ void __launch_bounds__(256) colsum1_kernel(const float* __restrict__ part, float* __restrict__ out, int P, int N) {
  __shared__ float red[4][64];
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  const int c = blockIdx.x * 64 + tx;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  if (c < N) {
    int p = ty;
    for (; p + 12 < P; p += 16) {
      a0 += part[static_cast<size_t>(p) * N + c];
      a1 += part[static_cast<size_t>(p + 4) * N + c];
      a2 += part[static_cast<size_t>(p + 8) * N + c];
      a3 += part[static_cast<size_t>(p + 12) * N + c];
    }
    for (; p < P; p += 4) a0 += part[static_cast<size_t>(p) * N + c];
  }
  red[ty][tx] = (a0 + a1) + (a2 + a3);
  __syncthreads();
  if (ty == 0 && c < N) out[c] = (red[0][tx] + red[1][tx]) + (red[2][tx] + red[3][tx]);
}

// ---- embedding -------------------------------------------------------------------------------------------------
template <typename W, typename O>
__global__ void embedding_fwd_kernel(const int64_t* __restrict__ ids, const W* __restrict__ weight, O* __restrict__ out,
                                     int64_t n_tokens, int H, int64_t vocab_start, int64_t n_rows) {
  const int64_t tok = blockIdx.x;
  if (tok >= n_tokens) return;
  const int64_t r = ids[tok] - vocab_start;
  O* o = out + tok * H;
  if (r < 0 || r >= n_rows) {
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = from_f<O>(0.f);
  } else {
    const W* w = weight + r * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = from_f<O>(to_f(w[c]));
  }
}

template <typename G>
__global__ void embedding_bwd_kernel(const int64_t* __restrict__ ids, const G* __restrict__ dout,
                                     float* __restrict__ dweight, int64_t n_tokens, int H, int64_t vocab_start,
                                     int64_t n_rows) {
  const int64_t tok = blockIdx.x;
  if (tok >= n_tokens) return;
  const int64_t r = ids[tok] - vocab_start;
  if (r < 0 || r >= n_rows) return;
  const G* g = dout + tok * H;
  float* w = dweight + r * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x) atomicAdd(w + c, to_f(g[c]));
}

// ---------------------------------------------------------------------------------------------- host side
#define DISPATCH_T(tensor, ...)                                     \
  if ((tensor).scalar_type() == torch::kBFloat16) {                 \
    using T = __nv_bfloat16;                                        \
    __VA_ARGS__                                                     \
  } else if ((tensor).scalar_type() == torch::kFloat16) {           \
    using T = __half;                                               \
    __VA_ARGS__                                                     \
  } else {                                                          \
    TORCH_CHECK(false, "expected bf16 / fp16");                     \
  }

torch::Tensor ce_local_stats(torch::Tensor logits, torch::Tensor targets, int64_t vocab_start) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous());
  TORCH_CHECK(targets.scalar_type() == torch::kInt64 && targets.is_contiguous() && targets.numel() == logits.size(0));
  const int rows = logits.size(0), V = logits.size(1);
  auto stats = torch::empty({rows, 3}, logits.options().dtype(torch::kFloat32));
  if (rows == 0) return stats;
  auto stream = at::cuda::getCurrentCUDAStream();
  DISPATCH_T(logits, ce_stats_kernel<T><<<rows, kCeThreads, 0, stream>>>(reinterpret_cast<const T*>(logits.data_ptr()),
                                                                         targets.data_ptr<int64_t>(),
                                                                         stats.data_ptr<float>(), rows, V, vocab_start);)
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return stats;
}

torch::Tensor ce_grad(torch::Tensor logits, torch::Tensor targets, int64_t vocab_start, torch::Tensor gmax,
                      torch::Tensor gsum, torch::Tensor scale, bool inplace) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous());
  const int rows = logits.size(0), V = logits.size(1);
  TORCH_CHECK(gmax.scalar_type() == torch::kFloat32 && gsum.scalar_type() == torch::kFloat32 &&
              scale.scalar_type() == torch::kFloat32 && gmax.numel() == rows && gsum.numel() == rows &&
              scale.numel() == rows);
  auto grad = inplace ? logits : torch::empty_like(logits);
  if (rows == 0) return grad;
  auto stream = at::cuda::getCurrentCUDAStream();
  DISPATCH_T(logits, ce_grad_kernel<T><<<rows, kCeThreads, 0, stream>>>(
                         reinterpret_cast<const T*>(logits.data_ptr()), targets.data_ptr<int64_t>(),
                         gmax.contiguous().data_ptr<float>(), gsum.contiguous().data_ptr<float>(),
                         scale.contiguous().data_ptr<float>(), reinterpret_cast<T*>(grad.data_ptr()), rows, V,
                         vocab_start);)
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return grad;
}

// returns (dz, db or undefined)
std::vector<torch::Tensor> act_backward(torch::Tensor dy, c10::optional<torch::Tensor> z, int64_t act, bool want_dz,
                                        bool want_sum) {
  TORCH_CHECK(dy.is_cuda() && dy.dim() == 2 && dy.is_contiguous());
  const int M = dy.size(0), N = dy.size(1);
  TORCH_CHECK(N % 8 == 0, "column count must be a multiple of 8");
  if (act != 0) TORCH_CHECK(z.has_value() && z->sizes() == dy.sizes() && z->is_contiguous() && z->dtype() == dy.dtype());
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const int gx = (N + 2047) / 2048;
  int gy = std::max(1, std::min((M + 15) / 16, (sms * 8 + gx - 1) / gx));
  const int rows_per = (M + gy - 1) / gy;
  gy = (M + rows_per - 1) / std::max(rows_per, 1);
  torch::Tensor dz, db, partials;
  if (want_dz) dz = torch::empty_like(dy);
  auto f32 = dy.options().dtype(torch::kFloat32);
  if (want_sum) {
    partials = torch::empty({std::max(gy, 1), N}, f32);
    db = torch::zeros({N}, f32);
  }
  if (M == 0) return {dz, db};
  auto stream = at::cuda::getCurrentCUDAStream();
  dim3 grid(gx, gy);
#define LAUNCH_ACT(ACT, WDZ, WSUM)                                                                                  \
  act_bwd_kernel<T, ACT, WDZ, WSUM><<<grid, 256, 0, stream>>>(                                                      \
      reinterpret_cast<const T*>(dy.data_ptr()), act != 0 ? reinterpret_cast<const T*>(z->data_ptr()) : nullptr,    \
      want_dz ? reinterpret_cast<T*>(dz.data_ptr()) : nullptr, want_sum ? partials.data_ptr<float>() : nullptr, M, N, \
      rows_per)
  DISPATCH_T(dy, {
    if (act == 1) {
      if (want_sum) LAUNCH_ACT(1, true, true); else LAUNCH_ACT(1, true, false);
    } else if (act == 2) {
      if (want_sum) LAUNCH_ACT(2, true, true); else LAUNCH_ACT(2, true, false);
    } else {
      TORCH_CHECK(!want_dz && want_sum, "identity activation is only used for column sums");
      LAUNCH_ACT(0, false, true);
    }
  })
#undef LAUNCH_ACT
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  if (want_sum) {
    colsum1_kernel<<<(N + 63) / 64, 256, 0, stream>>>(partials.data_ptr<float>(), db.data_ptr<float>(), gy, N);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  }
  return {dz, db};
}

torch::Tensor embedding_fwd(torch::Tensor ids, torch::Tensor weight, int64_t vocab_start, torch::ScalarType out_dtype) {
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == torch::kInt64 && weight.is_cuda() && weight.dim() == 2 &&
              weight.is_contiguous());
  auto idc = ids.contiguous();
  const int64_t n = idc.numel();
  const int H = weight.size(1);
  auto shape = idc.sizes().vec();
  shape.push_back(H);
  auto out = torch::empty(shape, weight.options().dtype(out_dtype));
  if (n == 0) return out;
  auto stream = at::cuda::getCurrentCUDAStream();
  const int threads = H >= 1024 ? 256 : 128;
#define LAUNCH_EMB(W, O)                                                                                            \
  embedding_fwd_kernel<W, O><<<n, threads, 0, stream>>>(idc.data_ptr<int64_t>(), reinterpret_cast<const W*>(weight.data_ptr()), \
                                                        reinterpret_cast<O*>(out.data_ptr()), n, H, vocab_start, weight.size(0))
  const auto wt = weight.scalar_type();
  if (out_dtype == torch::kBFloat16) {
    if (wt == torch::kFloat32) LAUNCH_EMB(float, __nv_bfloat16);
    else if (wt == torch::kBFloat16) LAUNCH_EMB(__nv_bfloat16, __nv_bfloat16);
    else TORCH_CHECK(false, "unsupported embedding weight dtype");
  } else if (out_dtype == torch::kFloat16) {
    if (wt == torch::kFloat32) LAUNCH_EMB(float, __half);
    else if (wt == torch::kFloat16) LAUNCH_EMB(__half, __half);
    else TORCH_CHECK(false, "unsupported embedding weight dtype");
  } else {
    TORCH_CHECK(false, "embedding output must be bf16 / fp16");
  }
#undef LAUNCH_EMB
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

torch::Tensor embedding_bwd(torch::Tensor dout, torch::Tensor ids, int64_t vocab_start, int64_t num_rows) {
  TORCH_CHECK(dout.is_cuda() && dout.is_contiguous() && ids.scalar_type() == torch::kInt64);
  auto idc = ids.contiguous();
  const int64_t n = idc.numel();
  const int H = dout.size(-1);
  auto dw = torch::zeros({num_rows, H}, dout.options().dtype(torch::kFloat32));
  if (n == 0) return dw;
  auto stream = at::cuda::getCurrentCUDAStream();
  const int threads = H >= 1024 ? 256 : 128;
  DISPATCH_T(dout, embedding_bwd_kernel<T><<<n, threads, 0, stream>>>(idc.data_ptr<int64_t>(),
                                                                     reinterpret_cast<const T*>(dout.data_ptr()),
                                                                     dw.data_ptr<float>(), n, H, vocab_start, num_rows);)
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return dw;
}

}  // namespace cw
