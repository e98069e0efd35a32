// Shared declarations of the tcgen05 GEMM family (plain and fused-with-collective variants).
#pragma once
#include <c10/cuda/CUDAException.h>
#include <torch/extension.h>

#include <algorithm>

#include "gemm_api.h"
#include "sm100.cuh"

namespace cw {

constexpr int kBM = 128;          // rows of C per tile == TMEM lanes
constexpr int kBK = 64;           // K elements per stage == one 128-byte swizzle row of 16-bit data
constexpr int kGemmThreads = 192; // producer warp + MMA warp + 4 epilogue warps

template <int BN>
struct GemmCfg {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kTmemCols = 2 * BN;                 // two accumulators
  static constexpr int kBarrierBytes = (2 * kStages + 4) * 8 + 16;
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + 1024;   // + alignment slack
};

struct GemmParams {
  int M, N, K;
  void* out;          // [M, ldo] OutT
  void* z_out;        // optional pre-activation copy, input dtype
  const float* bias;  // optional [N]
  int ldo;
  int act;
  int splits;         // split-K factor (fp32 red.add epilogue when > 1)
  int is_bf16;
  uint32_t mn_lbo, mn_sbo;   // descriptor offsets of MN-major operands
  int* status;        // host-visible error word
};

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

CUtensorMap make_tma_2d(const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows);
CUtensorMap make_tma_2d_plain(const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
                              uint32_t box_rows);
CUtensorMap make_tma_4d(const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3, uint64_t s1, uint64_t s2,
                        uint64_t s3);

template <typename InT, bool OUT_F32>
struct OutType { using type = InT; };
template <typename InT>
struct OutType<InT, true> { using type = float; };

// Work item -> (tile_m, tile_n, k-block range).  Tiles are walked in groups of 16 row-blocks so the CTAs
// that run concurrently share A and B panels in L2.
__device__ __forceinline__ void decode_work(int w, int num_tiles, int tiles_m, int tiles_n, int kb_total, int splits,
                                            int& tile_m, int& tile_n, int& kb0, int& kb1) {
  const int split = w / num_tiles;
  const int t = w - split * num_tiles;
  constexpr int kGroup = 16;
  const int per_group = kGroup * tiles_n;
  const int group = t / per_group;
  const int first_m = group * kGroup;
  const int gsz = min(tiles_m - first_m, kGroup);
  const int in_group = t - group * per_group;
  tile_m = first_m + in_group % gsz;
  tile_n = in_group / gsz;
  const int per = (kb_total + splits - 1) / splits;
  kb0 = split * per;
  kb1 = min(kb0 + per, kb_total);
}

__device__ __forceinline__ float gelu_f(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f)); }

__device__ __forceinline__ uint32_t pack2(float a, float b, __nv_bfloat16) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack2(float a, float b, __half) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void store_scalar(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }
__device__ __forceinline__ void store_scalar(__half* p, float v) { *p = __float2half(v); }
__device__ __forceinline__ void store_scalar(float* p, float v) { *p = v; }

// 32 consecutive outputs of one row.  `vec` = the chunk is complete and 16-byte aligned.
template <typename T>
__device__ __forceinline__ void store_row(T* dst, const float (&v)[32], bool vec, int remaining) {
  if (vec) {
    if constexpr (sizeof(T) == 2) {
      uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 u;
        u.x = pack2(v[q * 8 + 0], v[q * 8 + 1], T());
        u.y = pack2(v[q * 8 + 2], v[q * 8 + 3], T());
        u.z = pack2(v[q * 8 + 4], v[q * 8 + 5], T());
        u.w = pack2(v[q * 8 + 6], v[q * 8 + 7], T());
        d4[q] = u;
      }
    } else {
      float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
      for (int q = 0; q < 8; ++q) d4[q] = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < remaining) store_scalar(dst + j, v[j]);
  }
}

// fp32 accumulate into global memory (split-K partial sums).
__device__ __forceinline__ void red_row(float* dst, const float (&v)[32], bool vec, int remaining) {
  if (vec) {
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + q * 4), "f"(v[q * 4]), "f"(v[q * 4 + 1]),
                   "f"(v[q * 4 + 2]), "f"(v[q * 4 + 3])
                   : "memory");
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < remaining) atomicAdd(dst + j, v[j]);
  }
}

}  // namespace cw
