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

// The plain GEMM: producer warp + MMA warp + 8 epilogue warps, and a 32 KB staging area for TMA tile stores.
constexpr int kEpiWarps = 8;
constexpr int kGemmThreadsV2 = 64 + 32 * kEpiWarps;
constexpr int kEpiBlockBytes = 32 * 128;            // one warp's staging block: 32 rows x 128 bytes
constexpr uint32_t kGemmMnLbo = 8192, kGemmMnSbo = 1024;    // descriptor offsets of MN-major operands (see make_smem_desc)

template <int BN>
struct GemmCfgV2 {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kTmemCols = 2 * BN;                 // two accumulators
  static constexpr int kBarrierBytes = (2 * kStages + 4) * 8 + 16;
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiWarps * kEpiBlockBytes + kBarrierBytes + 1024;
  static_assert(kSmemBytes <= 227 * 1024, "GEMM exceeds the shared memory of one SM");
};

struct GemmParams {
  int M, N, K;
  void* out;          // [M, ldo] OutT
  void* z_out;        // optional pre-activation copy, input dtype
  const float* bias;  // optional [N]
  int ldo;
  int act;
  int splits;         // split-K factor (fp32 reduce-add epilogue when > 1)
  int is_bf16;
  int tma_store;      // outputs are written by TMA tile stores (16-byte aligned base and row pitch)
  int* status;        // host-visible error word
};

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

CUtensorMap make_tma_2d(const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows);
CUtensorMap make_tma_2d_plain(const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
                              uint32_t box_rows);
CUtensorMap make_tma_2d_store(const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, int elem_bytes, bool is_bf16);
CUtensorMap make_tma_4d(const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3, uint64_t s1, uint64_t s2,
                        uint64_t s3);

template <typename InT, bool OUT_F32>
struct OutType { using type = InT; };
template <typename InT>
struct OutType<InT, true> { using type = float; };

// x / d for 0 <= x < 2^22 and d >= 1 through a float reciprocal and one correction step: a handful of instructions
// where the integer division by a run-time divisor is a long dependent chain.  Every role of the persistent kernels
// decodes its tiles with several such divisions, on the critical path between two tiles.
__device__ __forceinline__ int fast_div(int x, int d) {
  int q = __float2int_rz(__int2float_rn(x) * __frcp_rn(__int2float_rn(d)));
  const int r = x - q * d;
  q += (r >= d ? 1 : 0) - (r < 0 ? 1 : 0);
  return q;
}

// Work item -> (tile_m, tile_n, k-block range).  Tiles are walked in groups of 16 row-blocks so the CTAs
// that run concurrently share A and B panels in L2.
__device__ __forceinline__ void decode_work(int w, int num_tiles, int tiles_m, int tiles_n, int kb_total, int splits,
                                            int& tile_m, int& tile_n, int& kb0, int& kb1) {
  const int split = splits > 1 ? fast_div(w, num_tiles) : 0;
  const int t = w - split * num_tiles;
  constexpr int kGroup = 16;
  const int per_group = kGroup * tiles_n;
  const int group = fast_div(t, per_group);
  const int first_m = group * kGroup;
  const int gsz = min(tiles_m - first_m, kGroup);
  const int in_group = t - group * per_group;
  tile_n = gsz == kGroup ? in_group >> 4 : fast_div(in_group, gsz);
  tile_m = first_m + in_group - tile_n * gsz;
  const int per = splits > 1 ? fast_div(kb_total + splits - 1, splits) : kb_total;
  kb0 = split * per;
  kb1 = min(kb0 + per, kb_total);
}

__device__ __forceinline__ float gelu_f(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f)); }

// GELU with the error function from Abramowitz & Stegun 7.1.26 (absolute error of erf below 1.5e-7, i.e. far below
// the resolution of a 16-bit output): one reciprocal, one exponential and six multiply-adds instead of erff's
// two-branch polynomial.  The GEMM epilogue is bound by this arithmetic when the activation is fused.
__device__ __forceinline__ float gelu_fast(float x) {
  const float ax = fabsf(x) * 0.70710678118654752f;
  const float t = __fdividef(1.0f, fmaf(0.3275911f, ax, 1.0f));
  float poly = fmaf(t, 1.061405429f, -1.453152027f);
  poly = fmaf(t, poly, 1.421413741f);
  poly = fmaf(t, poly, -0.284496736f);
  poly = fmaf(t, poly, 0.254829592f);
  poly *= t;
  const float erf_abs = 1.0f - poly * __expf(-ax * ax);
  return 0.5f * x * (1.0f + copysignf(erf_abs, x));
}

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

// ---- epilogue staging -------------------------------------------------------------------------------------
// A warp's 32 x 128-byte block in the TMA 128-byte swizzle: the 16-byte chunk j of row r sits at chunk j ^ (r & 7).
// Lane = row, so the eight lanes of a quarter-warp hit eight different bank groups with every 16-byte store.
template <typename T>
__device__ __forceinline__ void stage_row_16bit(uint8_t* block, int lane, const float (&v)[64]) {
  uint8_t* rowp = block + lane * 128;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint4 u;
    u.x = pack2(v[j * 8 + 0], v[j * 8 + 1], T());
    u.y = pack2(v[j * 8 + 2], v[j * 8 + 3], T());
    u.z = pack2(v[j * 8 + 4], v[j * 8 + 5], T());
    u.w = pack2(v[j * 8 + 6], v[j * 8 + 7], T());
    *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = u;
  }
}
template <typename T>
__device__ __forceinline__ void stage_row_16bit(uint8_t*, int, const float (&)[32]) {}   // 4-byte outputs never stage 16-bit rows
__device__ __forceinline__ void stage_row_f32(uint8_t* block, int lane, const float (&v)[32]) {
  uint8_t* rowp = block + lane * 128;
#pragma unroll
  for (int j = 0; j < 8; ++j)
    *reinterpret_cast<float4*>(rowp + ((j ^ (lane & 7)) << 4)) = make_float4(v[j * 4], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]);
}
__device__ __forceinline__ void stage_row_f32(uint8_t*, int, const float (&)[64]) {}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* ssrc, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(smem_u32(ssrc)),
               "r"(x), "r"(y)
               : "memory");
}
// global[tile] += shared[tile] element-wise (fp32): split-K partial sums without per-thread atomics
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* ssrc, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
               "r"(smem_u32(ssrc)), "r"(x), "r"(y)
               : "memory");
}


}  // namespace cw
