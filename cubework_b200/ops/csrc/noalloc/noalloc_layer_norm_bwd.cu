// Allocation-free layer-norm backward: see noalloc_layer_norm_bwd.h for who needs it and for the contract.
// Same arithmetic as the package's regular backward (one CTA walks rows, keeps per-column partial sums of
// dgamma / dbeta in registers, a second kernel adds the partials), but the partials go to a fixed array in
// this library's image instead of a freshly allocated tensor.
#include "noalloc_layer_norm_bwd.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include <mutex>

namespace {

constexpr int kThreads = 256;
constexpr int kVPT = CW_NOALLOC_MAX_HIDDEN / (8 * kThreads);   // 16-byte vectors per thread per row

// [2][CW_NOALLOC_MAX_CTAS][CW_NOALLOC_MAX_HIDDEN] fp32: partial dgamma, then partial dbeta.
// In host code this name is only a handle for cudaGetSymbolAddress, never a pointer to pass to a kernel.
static __device__ __align__(256) float g_partials[2 * CW_NOALLOC_MAX_CTAS * CW_NOALLOC_MAX_HIDDEN];

__device__ __forceinline__ float tof(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float tof(__half v) { return __half2float(v); }
__device__ __forceinline__ void fromf(__nv_bfloat16& o, float v) { o = __float2bfloat16(v); }
__device__ __forceinline__ void fromf(__half& o, float v) { o = __float2half(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void block_sum2(float& a, float& b, float* red) {
  a = warp_sum(a);
  b = warp_sum(b);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) { red[warp] = a; red[32 + warp] = b; }
  __syncthreads();
  float x = lane < kThreads / 32 ? red[lane] : 0.f;
  float y = lane < kThreads / 32 ? red[32 + lane] : 0.f;
  a = warp_sum(x);
  b = warp_sum(y);
}

template <typename T>
__global__ void __launch_bounds__(kThreads) ln_bwd_noalloc_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                                  const float* __restrict__ mean,
                                                                  const float* __restrict__ rstd,
                                                                  const float* __restrict__ gamma, T* __restrict__ dx,
                                                                  float* __restrict__ partials, int rows, int H) {
  __shared__ float red[64];
  float dg[kVPT][8], db[kVPT][8];
#pragma unroll
  for (int v = 0; v < kVPT; ++v)
#pragma unroll
    for (int i = 0; i < 8; ++i) { dg[v][i] = 0.f; db[v][i] = 0.f; }

  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    float xh[kVPT][8], g[kVPT][8];
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int v = 0; v < kVPT; ++v) {
      const int c = (v * kThreads + threadIdx.x) * 8;
      if (c < H) {
        const uint4 rx = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * H + c);
        const uint4 rd = *reinterpret_cast<const uint4*>(dy + static_cast<size_t>(row) * H + c);
        const T* px = reinterpret_cast<const T*>(&rx);
        const T* pd = reinterpret_cast<const T*>(&rd);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xhat = (tof(px[i]) - mu) * rs;
          const float d = tof(pd[i]);
          dg[v][i] += d * xhat;
          db[v][i] += d;
          const float gg = d * __ldg(gamma + c + i);
          xh[v][i] = xhat;
          g[v][i] = gg;
          s1 += gg;
          s2 += gg * xhat;
        }
      }
    }
    block_sum2(s1, s2, red);
    const float m1 = s1 / H, m2 = s2 / H;
#pragma unroll
    for (int v = 0; v < kVPT; ++v) {
      const int c = (v * kThreads + threadIdx.x) * 8;
      if (c < H) {
        uint4 out;
        T* po = reinterpret_cast<T*>(&out);
#pragma unroll
        for (int i = 0; i < 8; ++i) fromf(po[i], (g[v][i] - m1 - xh[v][i] * m2) * rs);
        *reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * H + c) = out;
      }
    }
  }
  float* pg = partials + static_cast<size_t>(blockIdx.x) * H;
  float* pb = partials + static_cast<size_t>(CW_NOALLOC_MAX_CTAS) * CW_NOALLOC_MAX_HIDDEN + static_cast<size_t>(blockIdx.x) * H;
#pragma unroll
  for (int v = 0; v < kVPT; ++v) {
    const int c = (v * kThreads + threadIdx.x) * 8;
    if (c < H) {
#pragma unroll
      for (int i = 0; i < 8; ++i) { pg[c + i] = dg[v][i]; pb[c + i] = db[v][i]; }
    }
  }
}

__global__ void ln_bwd_noalloc_finish(const float* __restrict__ partials, float* __restrict__ dgamma,
                                      float* __restrict__ dbeta, int ctas, int H) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  const float* pg = partials;
  const float* pb = partials + static_cast<size_t>(CW_NOALLOC_MAX_CTAS) * CW_NOALLOC_MAX_HIDDEN;
  float a = 0.f, b = 0.f;
  for (int p = 0; p < ctas; ++p) {
    a += pg[static_cast<size_t>(p) * H + c];
    b += pb[static_cast<size_t>(p) * H + c];
  }
  dgamma[c] = a;
  dbeta[c] = b;
}

constexpr int kMaxDevices = 64;
float* g_partials_addr[kMaxDevices] = {};
std::mutex g_setup_mutex;

// Device address of g_partials on the current device (looked up once per device).
int partials_address(float** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return CW_NOALLOC_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_partials_addr[dev] == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_partials) != cudaSuccess || p == nullptr)
      return CW_NOALLOC_ERR_CUDA;
    g_partials_addr[dev] = p;
  }
  *out = g_partials_addr[dev];
  return CW_NOALLOC_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

extern "C" int cw_layer_norm_bwd_noalloc(const void* dy, const void* x, const float* mean, const float* rstd,
                                         const float* gamma, void* dx, float* dgamma, float* dbeta, int rows, int hidden,
                                         int is_bf16, cudaStream_t stream) {
  if (hidden > CW_NOALLOC_MAX_HIDDEN) return CW_NOALLOC_ERR_TOO_LARGE;
  if (!dy || !x || !mean || !rstd || !gamma || !dx || !dgamma || !dbeta || rows < 1 || hidden < 8 || hidden % 8 != 0 ||
      !aligned16(dy) || !aligned16(x) || !aligned16(dx))
    return CW_NOALLOC_ERR_BAD_ARGUMENT;
  float* partials = nullptr;
  const int rc = partials_address(&partials);
  if (rc != CW_NOALLOC_OK) return rc;
  const int ctas = rows < CW_NOALLOC_MAX_CTAS ? rows : CW_NOALLOC_MAX_CTAS;
  if (is_bf16) {
    ln_bwd_noalloc_kernel<__nv_bfloat16><<<ctas, kThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), mean, rstd, gamma,
        static_cast<__nv_bfloat16*>(dx), partials, rows, hidden);
  } else {
    ln_bwd_noalloc_kernel<__half><<<ctas, kThreads, 0, stream>>>(static_cast<const __half*>(dy),
                                                                  static_cast<const __half*>(x), mean, rstd, gamma,
                                                                  static_cast<__half*>(dx), partials, rows, hidden);
  }
  if (cudaPeekAtLastError() != cudaSuccess) return CW_NOALLOC_ERR_CUDA;
  ln_bwd_noalloc_finish<<<(hidden + 255) / 256, 256, 0, stream>>>(partials, dgamma, dbeta, ctas, hidden);
  if (cudaPeekAtLastError() != cudaSuccess) return CW_NOALLOC_ERR_CUDA;
  return CW_NOALLOC_OK;
}
