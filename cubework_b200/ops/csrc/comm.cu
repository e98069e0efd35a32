// Peer-memory plumbing: buffers that every rank of a process group can address (CUDA IPC), and the
// fused GEMM + collective launches that use them (fused_gemm_sm100.cu).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAException.h>
#include <pybind11/pybind11.h>
#include <torch/extension.h>

#include "sm100.cuh"

namespace py = pybind11;

namespace cw {

void register_fused(py::module& m);

// Allocate `nbytes` with cudaMalloc (outside the caching allocator, so the IPC handle maps exactly this
// buffer) and return (device pointer, IPC handle bytes).
static py::tuple ipc_alloc(int64_t nbytes, bool zero) {
  void* p = nullptr;
  C10_CUDA_CHECK(cudaMalloc(&p, static_cast<size_t>(nbytes)));
  if (zero) C10_CUDA_CHECK(cudaMemset(p, 0, static_cast<size_t>(nbytes)));
  cudaIpcMemHandle_t h;
  C10_CUDA_CHECK(cudaIpcGetMemHandle(&h, p));
  C10_CUDA_CHECK(cudaDeviceSynchronize());
  return py::make_tuple(reinterpret_cast<int64_t>(p), py::bytes(reinterpret_cast<const char*>(&h), sizeof(h)));
}

static int64_t ipc_open(py::bytes handle) {
  std::string s = handle;
  TORCH_CHECK(s.size() == sizeof(cudaIpcMemHandle_t), "bad IPC handle size");
  cudaIpcMemHandle_t h;
  memcpy(&h, s.data(), sizeof(h));
  void* p = nullptr;
  C10_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  return reinterpret_cast<int64_t>(p);
}

static void ipc_close(int64_t ptr) { cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr)); }
static void ipc_free(int64_t ptr) { cudaFree(reinterpret_cast<void*>(ptr)); }

// View a raw device region as a tensor (no ownership).
static torch::Tensor as_tensor(int64_t ptr, std::vector<int64_t> shape, torch::ScalarType dtype, int64_t device) {
  auto opts = torch::TensorOptions().dtype(dtype).device(torch::kCUDA, static_cast<int>(device));
  return torch::from_blob(reinterpret_cast<void*>(ptr), shape, opts);
}

void register_comm(py::module& m) {
  m.def("ipc_alloc", &ipc_alloc);
  m.def("ipc_open", &ipc_open);
  m.def("ipc_close", &ipc_close);
  m.def("ipc_free", &ipc_free);
  m.def("as_tensor", &as_tensor);
  register_fused(m);
}

}  // namespace cw
