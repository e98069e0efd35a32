#include <torch/extension.h>
namespace cw {
std::vector<torch::Tensor> attention_fwd(torch::Tensor qkv, bool causal, c10::optional<torch::Tensor> key_bias,
                                         double scale, int64_t status_ptr) { TORCH_CHECK(false, "not built"); }
torch::Tensor attention_bwd(torch::Tensor dout, torch::Tensor qkv, torch::Tensor out, torch::Tensor lse, bool causal,
                            c10::optional<torch::Tensor> key_bias, double scale, int64_t status_ptr) { TORCH_CHECK(false, "not built"); }
}
