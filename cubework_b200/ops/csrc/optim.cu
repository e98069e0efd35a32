// Multi-tensor optimizer kernels: AdamW / SGD updates of fp32 master parameters that also refresh the
// 16-bit shadow copy used by the GEMMs, sum of squared gradients (for the global-norm clip) and in-place
// gradient scaling.  One launch covers up to kPack tensors: the pointer table travels as a kernel argument,
// each CTA owns one 16K-element chunk of one tensor.
//
// Replace torch.optim.AdamW (benchmark/gpt2/gpt2.py:440), torch.optim.SGD (benchmark/opt/opt.py:623) and the
// per-parameter norm / mul_ loops of cubework/utils/clip_grad.py:36-68.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAException.h>
#include <torch/extension.h>

#include "common.cuh"

namespace cw {

constexpr int kPack = 24;
constexpr int kChunk = 16384;
constexpr int kOptThreads = 256;

struct Pack {
  void* p[kPack];
  void* g[kPack];
  void* m[kPack];
  void* v[kPack];
  void* s[kPack];          // 16-bit shadow or nullptr
  float w[kPack];          // per-tensor weight (sum of squares)
  long long n[kPack];
  int first_block[kPack + 1];
  int count;
};

__device__ __forceinline__ bool locate(const Pack& pk, int& t, long long& begin, long long& end) {
  const int b = blockIdx.x;
  t = 0;
  while (t + 1 < pk.count && b >= pk.first_block[t + 1]) ++t;
  begin = static_cast<long long>(b - pk.first_block[t]) * kChunk;
  end = min(begin + kChunk, pk.n[t]);
  return begin < end;
}

// grad dtype G, shadow kind: 0 none / 1 bf16 / 2 fp16 (runtime)
template <typename G>
__global__ void __launch_bounds__(kOptThreads) adamw_kernel(Pack pk, float lr, float beta1, float beta2, float eps,
                                                            float wd, float bc1, float bc2_sqrt, const float* gscale,
                                                            int shadow_kind) {
  int t;
  long long b, e;
  if (!locate(pk, t, b, e)) return;
  float* p = static_cast<float*>(pk.p[t]);
  const G* g = static_cast<const G*>(pk.g[t]);
  float* m = static_cast<float*>(pk.m[t]);
  float* v = static_cast<float*>(pk.v[t]);
  const float gs = gscale != nullptr ? *gscale : 1.f;
  for (long long i = b + threadIdx.x; i < e; i += kOptThreads) {
    const float gr = to_f(g[i]) * gs;
    float pv = p[i] * (1.f - lr * wd);
    const float mv = m[i] + (gr - m[i]) * (1.f - beta1);
    const float vv = beta2 * v[i] + (1.f - beta2) * gr * gr;
    const float denom = sqrtf(vv) / bc2_sqrt + eps;
    pv -= (lr / bc1) * (mv / denom);
    p[i] = pv;
    m[i] = mv;
    v[i] = vv;
    if (pk.s[t] != nullptr) {
      if (shadow_kind == 1) static_cast<__nv_bfloat16*>(pk.s[t])[i] = __float2bfloat16(pv);
      else static_cast<__half*>(pk.s[t])[i] = __float2half(pv);
    }
  }
}

template <typename G>
__global__ void __launch_bounds__(kOptThreads) sgd_kernel(Pack pk, float lr, float momentum, float wd, int first,
                                                          const float* gscale, int shadow_kind) {
  int t;
  long long b, e;
  if (!locate(pk, t, b, e)) return;
  float* p = static_cast<float*>(pk.p[t]);
  const G* g = static_cast<const G*>(pk.g[t]);
  float* buf = static_cast<float*>(pk.m[t]);
  const float gs = gscale != nullptr ? *gscale : 1.f;
  for (long long i = b + threadIdx.x; i < e; i += kOptThreads) {
    float gr = to_f(g[i]) * gs + wd * p[i];
    if (buf != nullptr) {
      gr = first ? gr : momentum * buf[i] + gr;
      buf[i] = gr;
    }
    const float pv = p[i] - lr * gr;
    p[i] = pv;
    if (pk.s[t] != nullptr) {
      if (shadow_kind == 1) static_cast<__nv_bfloat16*>(pk.s[t])[i] = __float2bfloat16(pv);
      else static_cast<__half*>(pk.s[t])[i] = __float2half(pv);
    }
  }
}

template <typename G>
__global__ void __launch_bounds__(kOptThreads) sumsq_kernel(Pack pk, float* out) {
  __shared__ float red[64];
  int t;
  long long b, e;
  float acc = 0.f;
  if (locate(pk, t, b, e)) {
    const G* g = static_cast<const G*>(pk.g[t]);
    for (long long i = b + threadIdx.x; i < e; i += kOptThreads) {
      const float x = to_f(g[i]);
      acc += x * x;
    }
    acc *= pk.w[t];
  }
  float dummy = 0.f;
  block_sum2<kOptThreads>(acc, dummy, red);
  if (threadIdx.x == 0 && acc != 0.f) atomicAdd(out, acc);
}

template <typename G>
__global__ void __launch_bounds__(kOptThreads) scale_kernel(Pack pk, const float* coef) {
  int t;
  long long b, e;
  if (!locate(pk, t, b, e)) return;
  G* g = static_cast<G*>(pk.g[t]);
  const float c = *coef;
  if (c == 1.f) return;
  for (long long i = b + threadIdx.x; i < e; i += kOptThreads) g[i] = from_f<G>(to_f(g[i]) * c);
}

// ---------------------------------------------------------------------------------------------- host side
using TensorList = std::vector<torch::Tensor>;
using OptList = std::vector<c10::optional<torch::Tensor>>;

template <typename F>
static void for_each_pack(const TensorList& grads, F&& body) {
  // group by gradient dtype so one launch has one template instantiation
  for (auto dt : {torch::kFloat32, torch::kBFloat16, torch::kFloat16}) {
    std::vector<int> idx;
    for (int i = 0; i < static_cast<int>(grads.size()); ++i)
      if (grads[i].scalar_type() == dt && grads[i].numel() > 0) idx.push_back(i);
    for (size_t s = 0; s < idx.size(); s += kPack) {
      std::vector<int> sub(idx.begin() + s, idx.begin() + std::min(idx.size(), s + kPack));
      body(dt, sub);
    }
  }
}

static int fill_blocks(Pack& pk, const TensorList& ref, const std::vector<int>& sub) {
  int blocks = 0;
  pk.count = static_cast<int>(sub.size());
  for (int j = 0; j < pk.count; ++j) {
    pk.n[j] = ref[sub[j]].numel();
    pk.first_block[j] = blocks;
    blocks += static_cast<int>((pk.n[j] + kChunk - 1) / kChunk);
  }
  pk.first_block[pk.count] = blocks;
  return blocks;
}

#define DISPATCH_G(dt, ...)                                                   \
  if (dt == torch::kFloat32) { using G = float; __VA_ARGS__ }                 \
  else if (dt == torch::kBFloat16) { using G = __nv_bfloat16; __VA_ARGS__ }   \
  else { using G = __half; __VA_ARGS__ }

static int shadow_kind_of(const OptList& shadows) {
  int kind = 0;
  for (auto& s : shadows) {
    if (s.has_value() && s->defined()) {
      const int k = s->scalar_type() == torch::kBFloat16 ? 1 : 2;
      TORCH_CHECK(kind == 0 || kind == k, "all shadows must share one 16-bit dtype");
      kind = k;
    }
  }
  return kind;
}

void multi_adamw(TensorList params, TensorList grads, TensorList exp_avg, TensorList exp_avg_sq, OptList shadows, double lr,
                 double beta1, double beta2, double eps, double wd, int64_t step, c10::optional<torch::Tensor> gscale) {
  TORCH_CHECK(params.size() == grads.size() && params.size() == exp_avg.size() && params.size() == exp_avg_sq.size() &&
              params.size() == shadows.size());
  const float bc1 = 1.f - static_cast<float>(std::pow(beta1, static_cast<double>(step)));
  const float bc2s = std::sqrt(1.0 - std::pow(beta2, static_cast<double>(step)));
  const int kind = shadow_kind_of(shadows);
  const float* gs = (gscale.has_value() && gscale->defined()) ? gscale->data_ptr<float>() : nullptr;
  auto stream = at::cuda::getCurrentCUDAStream();
  for_each_pack(grads, [&](torch::ScalarType dt, const std::vector<int>& sub) {
    Pack pk;
    const int blocks = fill_blocks(pk, params, sub);
    for (int j = 0; j < pk.count; ++j) {
      const int i = sub[j];
      TORCH_CHECK(params[i].scalar_type() == torch::kFloat32 && params[i].is_contiguous() && grads[i].is_contiguous(),
                  "fused AdamW updates contiguous fp32 parameters");
      pk.p[j] = params[i].data_ptr();
      pk.g[j] = grads[i].data_ptr();
      pk.m[j] = exp_avg[i].data_ptr();
      pk.v[j] = exp_avg_sq[i].data_ptr();
      pk.s[j] = (shadows[i].has_value() && shadows[i]->defined()) ? shadows[i]->data_ptr() : nullptr;
    }
    DISPATCH_G(dt, adamw_kernel<G><<<blocks, kOptThreads, 0, stream>>>(pk, static_cast<float>(lr), static_cast<float>(beta1),
                                                                     static_cast<float>(beta2), static_cast<float>(eps),
                                                                     static_cast<float>(wd), bc1, bc2s, gs, kind);)
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  });
}

void multi_sgd(TensorList params, TensorList grads, c10::optional<TensorList> bufs, OptList shadows, double lr,
               double momentum, double wd, bool first, c10::optional<torch::Tensor> gscale) {
  TORCH_CHECK(params.size() == grads.size() && params.size() == shadows.size());
  const int kind = shadow_kind_of(shadows);
  const float* gs = (gscale.has_value() && gscale->defined()) ? gscale->data_ptr<float>() : nullptr;
  auto stream = at::cuda::getCurrentCUDAStream();
  for_each_pack(grads, [&](torch::ScalarType dt, const std::vector<int>& sub) {
    Pack pk;
    const int blocks = fill_blocks(pk, params, sub);
    for (int j = 0; j < pk.count; ++j) {
      const int i = sub[j];
      TORCH_CHECK(params[i].scalar_type() == torch::kFloat32 && params[i].is_contiguous() && grads[i].is_contiguous(),
                  "fused SGD updates contiguous fp32 parameters");
      pk.p[j] = params[i].data_ptr();
      pk.g[j] = grads[i].data_ptr();
      pk.m[j] = bufs.has_value() ? (*bufs)[i].data_ptr() : nullptr;
      pk.v[j] = nullptr;
      pk.s[j] = (shadows[i].has_value() && shadows[i]->defined()) ? shadows[i]->data_ptr() : nullptr;
    }
    DISPATCH_G(dt, sgd_kernel<G><<<blocks, kOptThreads, 0, stream>>>(pk, static_cast<float>(lr), static_cast<float>(momentum),
                                                                   static_cast<float>(wd), first ? 1 : 0, gs, kind);)
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  });
}

torch::Tensor multi_sumsq(TensorList grads, std::vector<double> weights) {
  TORCH_CHECK(!grads.empty() && grads.size() == weights.size());
  auto out = torch::zeros({1}, grads[0].options().dtype(torch::kFloat32));
  auto stream = at::cuda::getCurrentCUDAStream();
  for_each_pack(grads, [&](torch::ScalarType dt, const std::vector<int>& sub) {
    Pack pk;
    const int blocks = fill_blocks(pk, grads, sub);
    for (int j = 0; j < pk.count; ++j) {
      TORCH_CHECK(grads[sub[j]].is_contiguous());
      pk.g[j] = grads[sub[j]].data_ptr();
      pk.w[j] = static_cast<float>(weights[sub[j]]);
    }
    DISPATCH_G(dt, sumsq_kernel<G><<<blocks, kOptThreads, 0, stream>>>(pk, out.data_ptr<float>());)
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  });
  return out;
}

void multi_scale(TensorList grads, torch::Tensor coef) {
  TORCH_CHECK(coef.scalar_type() == torch::kFloat32 && coef.numel() == 1 && coef.is_cuda());
  auto stream = at::cuda::getCurrentCUDAStream();
  for_each_pack(grads, [&](torch::ScalarType dt, const std::vector<int>& sub) {
    Pack pk;
    const int blocks = fill_blocks(pk, grads, sub);
    for (int j = 0; j < pk.count; ++j) {
      TORCH_CHECK(grads[sub[j]].is_contiguous());
      pk.g[j] = grads[sub[j]].data_ptr();
    }
    DISPATCH_G(dt, scale_kernel<G><<<blocks, kOptThreads, 0, stream>>>(pk, coef.data_ptr<float>());)
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  });
}

}  // namespace cw
