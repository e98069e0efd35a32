// Python bindings of the sm_100a kernels.  Everything launches on the current CUDA stream of the
// calling thread; nothing here synchronises the device.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "gemm_api.h"

namespace cw {

// norm.cu
std::vector<torch::Tensor> layer_norm_fwd(torch::Tensor x, torch::Tensor gamma, torch::Tensor beta, double eps);
std::vector<torch::Tensor> layer_norm_bwd(torch::Tensor dy, torch::Tensor x, torch::Tensor mean, torch::Tensor rstd,
                                          torch::Tensor gamma);
std::vector<torch::Tensor> layer_norm_fwd_res(torch::Tensor x, c10::optional<torch::Tensor> residual, torch::Tensor gamma,
                                              torch::Tensor beta, double eps);
std::vector<torch::Tensor> layer_norm_bwd_res(torch::Tensor dy, torch::Tensor x, torch::Tensor mean, torch::Tensor rstd,
                                              torch::Tensor gamma, c10::optional<torch::Tensor> dres);
torch::Tensor norm_apply(torch::Tensor x, torch::Tensor mean, torch::Tensor rstd, c10::optional<torch::Tensor> gamma,
                         c10::optional<torch::Tensor> beta);
torch::Tensor row_moments(torch::Tensor x);
std::vector<torch::Tensor> norm_bwd_partials(torch::Tensor dy, torch::Tensor x, torch::Tensor mean, torch::Tensor rstd,
                                             c10::optional<torch::Tensor> gamma);
torch::Tensor norm_bwd_apply(torch::Tensor dy, torch::Tensor x, torch::Tensor mean, torch::Tensor rstd,
                             c10::optional<torch::Tensor> gamma, torch::Tensor sums, double hidden);
// loss_elementwise.cu
torch::Tensor ce_local_stats(torch::Tensor logits, torch::Tensor targets, int64_t vocab_start);
torch::Tensor ce_grad(torch::Tensor logits, torch::Tensor targets, int64_t vocab_start, torch::Tensor gmax,
                      torch::Tensor gsum, torch::Tensor scale, bool inplace);
std::vector<torch::Tensor> act_backward(torch::Tensor dy, c10::optional<torch::Tensor> z, int64_t act, bool want_dz,
                                        bool want_sum);
torch::Tensor embedding_fwd(torch::Tensor ids, torch::Tensor weight, int64_t vocab_start, torch::ScalarType out_dtype);
torch::Tensor embedding_bwd(torch::Tensor dout, torch::Tensor ids, int64_t vocab_start, int64_t num_rows);
// optim.cu
void multi_adamw(std::vector<torch::Tensor> params, std::vector<torch::Tensor> grads, std::vector<torch::Tensor> exp_avg,
                 std::vector<torch::Tensor> exp_avg_sq, std::vector<c10::optional<torch::Tensor>> shadows, double lr,
                 double beta1, double beta2, double eps, double wd, int64_t step, c10::optional<torch::Tensor> gscale);
void multi_sgd(std::vector<torch::Tensor> params, std::vector<torch::Tensor> grads,
               c10::optional<std::vector<torch::Tensor>> bufs, std::vector<c10::optional<torch::Tensor>> shadows, double lr,
               double momentum, double wd, bool first, c10::optional<torch::Tensor> gscale);
torch::Tensor multi_sumsq(std::vector<torch::Tensor> grads, std::vector<double> weights);
void multi_scale(std::vector<torch::Tensor> grads, torch::Tensor coef);
// attention_sm100.cu
std::vector<torch::Tensor> attention_fwd(torch::Tensor qkv, bool causal, c10::optional<torch::Tensor> key_bias,
                                         double scale, int64_t status_ptr, c10::optional<torch::Tensor> trace);
torch::Tensor attention_bwd(torch::Tensor dout, torch::Tensor qkv, torch::Tensor out, torch::Tensor lse, bool causal,
                            c10::optional<torch::Tensor> key_bias, double scale, int64_t status_ptr,
                            c10::optional<torch::Tensor> packed, c10::optional<torch::Tensor> trace);
bool attention_ready();
// comm.cu
void register_comm(pybind11::module& m);

// Host-mapped status words: kernels record a bounded-wait failure here and the host can read it at any time.
static int* g_status_host = nullptr;
static int* g_status_dev = nullptr;

static void ensure_status() {
  if (g_status_host == nullptr) {
    C10_CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&g_status_host), 64 * sizeof(int), cudaHostAllocMapped));
    for (int i = 0; i < 64; ++i) g_status_host[i] = 0;
    C10_CUDA_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&g_status_dev), g_status_host, 0));
  }
}
int64_t status_device_ptr() {
  ensure_status();
  return reinterpret_cast<int64_t>(g_status_dev);
}
std::vector<int64_t> read_status(bool clear) {
  ensure_status();
  std::vector<int64_t> v = {g_status_host[0], g_status_host[1], g_status_host[2]};
  if (clear) g_status_host[0] = g_status_host[1] = g_status_host[2] = 0;
  return v;
}

static int act_code(const std::string& a) {
  if (a.empty() || a == "none") return kActNone;
  if (a == "gelu") return kActGelu;
  if (a == "relu") return kActRelu;
  TORCH_CHECK(false, "unknown activation ", a);
}

// C = act(op(A) op(B) + bias); returns (C, Z) with Z the pre-activation tensor when requested.
std::vector<torch::Tensor> gemm(torch::Tensor a, torch::Tensor b, bool trans_a, bool trans_b,
                                c10::optional<torch::Tensor> bias, const std::string& act, bool out_f32, bool want_z) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.dim() == 2 && b.dim() == 2 && a.is_contiguous() && b.is_contiguous());
  TORCH_CHECK(a.scalar_type() == b.scalar_type() &&
              (a.scalar_type() == torch::kBFloat16 || a.scalar_type() == torch::kFloat16));
  c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = trans_a ? a.size(1) : a.size(0);
  const int64_t K = trans_a ? a.size(0) : a.size(1);
  const int64_t Kb = trans_b ? b.size(1) : b.size(0);
  const int64_t N = trans_b ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "inner dimensions differ: ", K, " vs ", Kb);
  auto out = torch::empty({M, N}, a.options().dtype(out_f32 ? torch::kFloat32 : a.scalar_type()));
  torch::Tensor z;
  if (want_z) z = torch::empty({M, N}, a.options());
  if (M == 0 || N == 0) return {out, z};
  if (K == 0) { out.zero_(); return {out, z}; }
  torch::Tensor bias_f;
  if (bias.has_value() && bias->defined()) {
    bias_f = bias->to(torch::kFloat32).contiguous();
    TORCH_CHECK(bias_f.numel() == N, "bias must have one value per output column");
  }
  ensure_status();
  GemmArgs g;
  g.a = a.data_ptr(); g.b = b.data_ptr(); g.out = out.data_ptr();
  g.z_out = want_z ? z.data_ptr() : nullptr;
  g.bias = bias_f.defined() ? bias_f.data_ptr<float>() : nullptr;
  g.M = static_cast<int>(M); g.N = static_cast<int>(N); g.K = static_cast<int>(K);
  g.trans_a = trans_a; g.trans_b = trans_b;
  g.is_bf16 = a.scalar_type() == torch::kBFloat16;
  g.out_f32 = out_f32;
  g.act = act_code(act);
  g.allow_split_k = g.act == kActNone && !want_z;
  g.num_sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  g.status = g_status_dev;
  gemm_launch(g, at::cuda::getCurrentCUDAStream());
  return {out, z};
}

}  // namespace cw

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &cw::gemm);
  m.def("status_device_ptr", &cw::status_device_ptr);
  m.def("read_status", &cw::read_status);
  m.def("layer_norm_fwd", &cw::layer_norm_fwd);
  m.def("layer_norm_bwd", &cw::layer_norm_bwd);
  m.def("layer_norm_fwd_res", &cw::layer_norm_fwd_res);
  m.def("layer_norm_bwd_res", &cw::layer_norm_bwd_res);
  m.def("norm_apply", &cw::norm_apply);
  m.def("row_moments", &cw::row_moments);
  m.def("norm_bwd_partials", &cw::norm_bwd_partials);
  m.def("norm_bwd_apply", &cw::norm_bwd_apply);
  m.def("ce_local_stats", &cw::ce_local_stats);
  m.def("ce_grad", &cw::ce_grad);
  m.def("act_backward", &cw::act_backward);
  m.def("embedding_fwd", &cw::embedding_fwd);
  m.def("embedding_bwd", &cw::embedding_bwd);
  m.def("multi_adamw", &cw::multi_adamw);
  m.def("multi_sgd", &cw::multi_sgd);
  m.def("multi_sumsq", &cw::multi_sumsq);
  m.def("multi_scale", &cw::multi_scale);
  m.def("attention_fwd", &cw::attention_fwd);
  m.def("attention_bwd", &cw::attention_bwd);
  m.def("attention_ready", &cw::attention_ready);
  cw::register_comm(m);
}
