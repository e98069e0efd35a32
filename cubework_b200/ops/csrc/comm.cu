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
void register_ggs(py::module& m);

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

// One thread waits (bounded by `limit_ns`) for *flag >= epoch and records the outcome: 0 = arrived, code 5 = gave up.
// Used by the failure-detection tests: a wait whose partner never writes must end with a status, not a hang.
__global__ void probe_wait_kernel(const int* flag, int epoch, unsigned long long limit_ns, int* result) {
  const unsigned long long t0 = globaltimer_ns();
  int outcome = kErrPeerFlagTimeout;
  for (unsigned spin = 0;; ++spin) {
    int v;
    asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= epoch) { outcome = kOk; break; }
    if ((spin & 63u) == 0) {
      __nanosleep(200);
      if (globaltimer_ns() - t0 > limit_ns) break;
    }
  }
  result[0] = outcome;
  result[1] = static_cast<int>((globaltimer_ns() - t0) / 1000000ull);
}

static torch::Tensor probe_wait(torch::Tensor flag, int64_t epoch, double limit_ms) {
  TORCH_CHECK(flag.is_cuda() && flag.scalar_type() == torch::kInt32 && flag.numel() >= 1);
  auto result = torch::zeros({2}, flag.options());
  probe_wait_kernel<<<1, 1, 0, at::cuda::getCurrentCUDAStream()>>>(
      flag.data_ptr<int>(), static_cast<int>(epoch), static_cast<unsigned long long>(limit_ms * 1e6), result.data_ptr<int>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return result;
}

// Streaming copy src -> dst through shared memory with bulk copies only (one issuing thread per CTA, `kDepth`
// chunks in flight).  Either pointer may be a peer mapping, which makes this the measuring stick for what the
// bulk-copy data path of the fused kernels can reach over NVLink.
constexpr int kCopyDepth = 4;
__global__ void __launch_bounds__(32) bulk_copy_kernel(uint8_t* dst, const uint8_t* src, size_t bytes, int chunk) {
  extern __shared__ __align__(128) uint8_t cp_smem[];
  __shared__ uint64_t bars[kCopyDepth];
  if (threadIdx.x != 0) return;
  for (int i = 0; i < kCopyDepth; ++i) mbar_init(&bars[i], 1);
  fence_barrier_init();
  const size_t n_chunks = bytes / chunk;
  volatile int abort_flag = 0;
  size_t issued = 0, done = 0;
  uint32_t phase[kCopyDepth] = {0, 0, 0, 0};
  // chunk ids of this CTA: blockIdx.x, + gridDim.x, ...
  auto chunk_id = [&](size_t k) { return blockIdx.x + k * gridDim.x; };
  while (chunk_id(done) < n_chunks) {
    while (issued < done + kCopyDepth && chunk_id(issued) < n_chunks) {
      const int s = issued % kCopyDepth;
      if (issued >= kCopyDepth) {
        // the store that last used this slot must have finished reading it
        asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kCopyDepth - 1) : "memory");
      }
      mbar_expect_tx(&bars[s], chunk);
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                       smem_u32(cp_smem + s * chunk)),
                   "l"(src + chunk_id(issued) * chunk), "r"(chunk), "r"(smem_u32(&bars[s]))
                   : "memory");
      ++issued;
    }
    const int s = done % kCopyDepth;
    if (!mbar_wait(&bars[s], phase[s], &abort_flag, nullptr, 0, 0)) return;
    phase[s] ^= 1;
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst + chunk_id(done) * chunk),
                 "r"(smem_u32(cp_smem + s * chunk)), "r"(chunk)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    ++done;
  }
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

static void bulk_copy(int64_t dst, int64_t src, int64_t bytes, int64_t chunk, int64_t ctas) {
  TORCH_CHECK(bytes % chunk == 0 && chunk % 16 == 0 && chunk * kCopyDepth <= 200 * 1024);
  static bool configured = false;
  if (!configured) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(bulk_copy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    configured = true;
  }
  bulk_copy_kernel<<<static_cast<int>(ctas), 32, chunk * kCopyDepth, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<uint8_t*>(dst), reinterpret_cast<const uint8_t*>(src), static_cast<size_t>(bytes),
      static_cast<int>(chunk));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void register_comm(py::module& m) {
  m.def("bulk_copy", &bulk_copy);
  m.def("probe_wait", &probe_wait);
  m.def("ipc_alloc", &ipc_alloc);
  m.def("ipc_open", &ipc_open);
  m.def("ipc_close", &ipc_close);
  m.def("ipc_free", &ipc_free);
  m.def("as_tensor", &as_tensor);
  register_fused(m);
  register_ggs(m);
}

}  // namespace cw
