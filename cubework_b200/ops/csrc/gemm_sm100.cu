// Persistent warp-specialised GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma -> TMEM -> epilogue.
//
//   C[M,N] = act( op(A)[M,K] * op(B)[K,N] + bias[N] )        fp32 accumulation, 16-bit inputs
//
// * warp 0   : TMA producer (one lane), kStages-deep ring of {A tile 128xBK, B tile BNxBK}
// * warp 1   : MMA issuer (one lane) + TMEM owner; two accumulators (2*BN columns) so the epilogue of
//              tile i overlaps the main loop of tile i+1
// * warps 2-9: epilogue, two warps per TMEM lane quarter (one per half of the tile's columns): tcgen05.ld of
//              128 bytes of output per row -> bias / GELU / ReLU -> a 32-row x 128-byte staging block in shared
//              memory (128-byte swizzle, bank-conflict free) -> one TMA tile store (or TMA reduce-add in fp32
//              for split-K), which writes whole 128-byte lines and clips at the matrix edge.  The accumulator
//              is handed back to the MMA warp as soon as its last column has been read.  Outputs whose row
//              pitch is not a multiple of 16 bytes take a direct-store path instead.
//
// Both operands may be K-major (row-major [rows, K]) or MN-major (row-major [K, rows]); the four
// combinations cover forward (X * W^T), data gradient (dY * W) and weight gradient (dY^T * X) without any
// transposition pass.  The library equivalents replaced are the cuBLAS calls behind F.linear /
// torch.matmul / addmm in cubework/module/parallel_{1d,2d,3d}.
#include <cmath>

#include "gemm_sm100.cuh"

namespace cw {

static PFN_encodeTiled g_encode = nullptr;

static PFN_encodeTiled get_encode() {
  if (g_encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    TORCH_CHECK(e == cudaSuccess && fn != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
    g_encode = reinterpret_cast<PFN_encodeTiled>(fn);
  }
  return g_encode;
}

// 2-D map over a row-major 16-bit matrix [rows, cols] (leading dimension `ld` elements), box = 64 x box_rows.
CUtensorMap make_tma_2d(const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  TORCH_CHECK((reinterpret_cast<uintptr_t>(ptr) & 15) == 0, "TMA operand must be 16-byte aligned");
  TORCH_CHECK((ld * 2) % 16 == 0, "TMA operand needs a leading dimension that is a multiple of 8 elements");
  CUtensorMap m;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = get_encode()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", static_cast<int>(r));
  return m;
}

// 2-D map without swizzle over a row-major 16-bit matrix, box = box_cols x box_rows (dense rows in shared memory);
// used for tile stores, which clip the box against the matrix extent.
CUtensorMap make_tma_2d_plain(const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
                              uint32_t box_rows) {
  TORCH_CHECK((reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && (ld * 2) % 16 == 0, "TMA store target must be 16-byte aligned");
  CUtensorMap m;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = get_encode()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (plain) failed with code ", static_cast<int>(r));
  return m;
}

// 2-D map for epilogue tile stores: row-major [rows, cols] of 2- or 4-byte elements, box = 128 bytes x 32 rows,
// 128-byte swizzle (the staging block in shared memory is written in that pattern).
CUtensorMap make_tma_2d_store(const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, int elem_bytes, bool is_bf16) {
  TORCH_CHECK((reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && (ld * elem_bytes) % 16 == 0,
              "TMA store target must be 16-byte aligned with a 16-byte multiple row pitch");
  CUtensorMap m;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / elem_bytes), 32};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                 : (is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  CUresult r = get_encode()(&m, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (store) failed with code ", static_cast<int>(r));
  return m;
}

// 4-D map over 16-bit data [d3][d2][d1][d0] (d0 innermost, strides in bytes for d1..d3), box = 64 x 128 x 1 x 1.
// Reads past any extent are zero-filled, which is how tiles get their padding.
CUtensorMap make_tma_4d(const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3, uint64_t s1, uint64_t s2,
                        uint64_t s3) {
  TORCH_CHECK((reinterpret_cast<uintptr_t>(ptr) & 15) == 0, "TMA operand must be 16-byte aligned");
  TORCH_CHECK(s1 % 16 == 0 && s2 % 16 == 0 && s3 % 16 == 0, "TMA strides must be multiples of 16 bytes");
  CUtensorMap m;
  cuuint64_t dims[4] = {d0, d1, d2, d3};
  cuuint64_t strides[3] = {s1, s2, s3};
  cuuint32_t box[4] = {64, 128, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = get_encode()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (4-D) failed with code ", static_cast<int>(r));
  return m;
}

template <int BN, bool A_KMAJOR, bool B_KMAJOR, typename InT, bool OUT_F32>
__global__ void __launch_bounds__(kGemmThreadsV2, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
            const __grid_constant__ CUtensorMap tma_out, const __grid_constant__ CUtensorMap tma_z, GemmParams p) {
  using Cfg = GemmCfgV2<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_out = smem + Cfg::kStages * Cfg::kStageBytes;                     // 8 x 4 KB, 1024-byte aligned
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(stage_out + kEpiWarps * kEpiBlockBytes);
  uint64_t* empty_bar = full_bar + Cfg::kStages;
  uint64_t* tfull_bar = empty_bar + Cfg::kStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], kEpiWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
    if (p.tma_store) {
      tma_prefetch_desc(&tma_out);
      if (p.z_out != nullptr) tma_prefetch_desc(&tma_z);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_m = (p.M + kBM - 1) / kBM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int kb_total = (p.K + kBK - 1) / kBK;
  const int total_work = num_tiles * p.splits;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int w = blockIdx.x; w < total_work && !*abort_flag; w += gridDim.x) {
        int tile_m, tile_n, kb0, kb1;
        decode_work(w, num_tiles, tiles_m, tiles_n, kb_total, p.splits, tile_m, tile_n, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kErrEmptyBarrierTimeout, w)) break;
          mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kABytes;
          if (A_KMAJOR) {
            tma_load_2d(sa, &tma_a, &full_bar[stage], kb * kBK, tile_m * kBM);
          } else {
#pragma unroll
            for (int g = 0; g < kBM / 64; ++g)
              tma_load_2d(sa + g * 8192, &tma_a, &full_bar[stage], tile_m * kBM + g * 64, kb * kBK);
          }
          if (B_KMAJOR) {
            tma_load_2d(sb, &tma_b, &full_bar[stage], kb * kBK, tile_n * BN);
          } else {
#pragma unroll
            for (int g = 0; g < BN / 64; ++g)
              tma_load_2d(sb + g * 8192, &tma_b, &full_bar[stage], tile_n * BN + g * 64, kb * kBK);
          }
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(kBM, BN, !A_KMAJOR, !B_KMAJOR, sizeof(InT) == 2 && p.is_bf16);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int w = blockIdx.x; w < total_work && !*abort_flag; w += gridDim.x, ++it) {
        int tile_m, tile_n, kb0, kb1;
        decode_work(w, num_tiles, tiles_m, tiles_n, kb_total, p.splits, tile_m, tile_n, kb0, kb1);
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status, kErrTmemEmptyTimeout, w)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kErrFullBarrierTimeout, w)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t sb = sa + Cfg::kABytes;
#pragma unroll
          for (int k16 = 0; k16 < kBK / 16; ++k16) {
            const uint64_t da = A_KMAJOR ? make_smem_desc(sa + k16 * 32, 16, 1024)
                                         : make_smem_desc(sa + k16 * 2048, kGemmMnLbo, kGemmMnSbo);
            const uint64_t db = B_KMAJOR ? make_smem_desc(sb + k16 * 32, 16, 1024)
                                         : make_smem_desc(sb + k16 * 2048, kGemmMnLbo, kGemmMnSbo);
            tc_mma_f16(d_tmem, da, db, idesc, (kb > kb0 || k16 > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);   // frees the stage once these MMAs have consumed it
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(&tfull_bar[acc]);        // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (8 warps)
    using OutT = typename OutType<InT, OUT_F32>::type;
    const int ew = warp - 2;                 // 0..7
    const int quarter = warp & 3;            // TMEM lanes [32*quarter, 32*quarter + 32) (fixed by the hardware)
    const int half = ew >> 2;                // which half of the tile's columns
    constexpr int kHalfCols = BN / 2;
    constexpr int kChunk = 128 / static_cast<int>(sizeof(OutT));   // columns per 128-byte staging row
    constexpr int kLoads = kChunk / 32;                            // tcgen05.ld (32 columns) per chunk
    uint8_t* sbuf = stage_out + ew * kEpiBlockBytes;
    OutT* out = reinterpret_cast<OutT*>(p.out);
    InT* zout = reinterpret_cast<InT*>(p.z_out);
    int it = 0;
    for (int w = blockIdx.x; w < total_work && !*abort_flag; w += gridDim.x, ++it) {
      int tile_m, tile_n, kb0, kb1;
      decode_work(w, num_tiles, tiles_m, tiles_n, kb_total, p.splits, tile_m, tile_n, kb0, kb1);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, kErrTmemFullTimeout, w)) break;
      tc_fence_after();
      const int row0 = tile_m * kBM + quarter * 32;
      const int row = row0 + lane;
      const bool add_bias = p.bias != nullptr && kb0 == 0;   // split-K: only the first split adds it
      const uint32_t t_addr = tmem_base + acc * BN + half * kHalfCols + (static_cast<uint32_t>(quarter * 32) << 16);
      const int colbase = tile_n * BN + half * kHalfCols;
      if (p.tma_store) {
#pragma unroll 1
        for (int c = 0; c < kHalfCols / kChunk; ++c) {
          const int col0 = colbase + c * kChunk;
          const bool live = col0 < p.N;       // warp-uniform; dead chunks are still read so the hand-back below is uniform
          float v[kChunk];
          {
            uint32_t r0[32];
            tmem_ld_32x32(t_addr + c * kChunk, r0);
            if constexpr (kLoads == 2) {
              uint32_t r1[32];
              tmem_ld_32x32(t_addr + c * kChunk + 32, r1);
              tmem_wait_ld();
#pragma unroll
              for (int j = 0; j < 32; ++j) v[32 + j] = __uint_as_float(r1[j]);
            } else {
              tmem_wait_ld();
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r0[j]);
          }
          if (c == kHalfCols / kChunk - 1) {
            // every column of this warp's part has been read: the MMA warp may overwrite the accumulator
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty_bar[acc]);
          }
          if (!live) continue;
          if (add_bias) {
#pragma unroll
            for (int j = 0; j < kChunk; ++j) v[j] += (col0 + j < p.N) ? __ldg(p.bias + col0 + j) : 0.f;
          }
          if constexpr (!OUT_F32) {
            if (p.z_out != nullptr) {
              if (lane == 0) bulk_wait_group_read0();
              __syncwarp();
              stage_row_16bit<InT>(sbuf, lane, v);
              fence_proxy_async();
              __syncwarp();
              if (lane == 0) {
                tma_store_2d(&tma_z, sbuf, col0, row0);
                bulk_commit_group();
              }
            }
          }
          if (p.act == kActGelu) {
#pragma unroll
            for (int j = 0; j < kChunk; ++j) v[j] = gelu_fast(v[j]);
          } else if (p.act == kActRelu) {
#pragma unroll
            for (int j = 0; j < kChunk; ++j) v[j] = fmaxf(v[j], 0.f);
          }
          if (lane == 0) bulk_wait_group_read0();       // the previous store of this warp has finished reading sbuf
          __syncwarp();
          if constexpr (OUT_F32) stage_row_f32(sbuf, lane, v);
          else stage_row_16bit<InT>(sbuf, lane, v);
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            if (OUT_F32 && p.splits > 1) tma_reduce_add_2d(&tma_out, sbuf, col0, row0);
            else tma_store_2d(&tma_out, sbuf, col0, row0);
            bulk_commit_group();
          }
        }
      } else {
        // direct stores: row pitch or base not 16-byte aligned
        const bool row_ok = row < p.M;
#pragma unroll 1
        for (int c = 0; c < kHalfCols / 32; ++c) {
          const int col0 = colbase + c * 32;
          uint32_t r[32];
          tmem_ld_32x32(t_addr + c * 32, r);
          tmem_wait_ld();
          if (c == kHalfCols / 32 - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty_bar[acc]);
          }
          if (col0 >= p.N) continue;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          if (add_bias) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) v[j] += __ldg(p.bias + col0 + j);
          }
          if (row_ok) {
            if (p.z_out != nullptr) store_row<InT>(zout + static_cast<size_t>(row) * p.ldo + col0, v, false, p.N - col0);
            if (p.act == kActGelu) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = gelu_fast(v[j]);
            } else if (p.act == kActRelu) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
            }
            OutT* dst = out + static_cast<size_t>(row) * p.ldo + col0;
            if (OUT_F32 && p.splits > 1) red_row(reinterpret_cast<float*>(dst), v, false, p.N - col0);
            else store_row<OutT>(dst, v, false, p.N - col0);
          }
        }
      }
    }
    if (lane == 0) bulk_wait_group0();     // the tile stores must have left shared memory (and landed) before exit
  }

  // ---------------------------------------------------------------------- teardown
  if (*abort_flag) {
    // give copies that are still in flight time to land before shared memory and TMEM are released
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int BN, bool AK, bool BK_, typename InT, bool OUT_F32>
static void launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to, const CUtensorMap& tz,
                   const GemmParams& p, int grid, cudaStream_t stream) {
  using Cfg = GemmCfgV2<BN>;
  auto kern = gemm_kernel<BN, AK, BK_, InT, OUT_F32>;
  static bool configured = false;
  if (!configured) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    configured = true;
  }
  kern<<<grid, kGemmThreadsV2, Cfg::kSmemBytes, stream>>>(ta, tb, to, tz, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

template <int BN, typename InT, bool OUT_F32>
static void dispatch_major(bool ak, bool bk, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to,
                           const CUtensorMap& tz, const GemmParams& p, int grid, cudaStream_t s) {
  if (ak && bk) launch<BN, true, true, InT, OUT_F32>(ta, tb, to, tz, p, grid, s);
  else if (ak && !bk) launch<BN, true, false, InT, OUT_F32>(ta, tb, to, tz, p, grid, s);
  else if (!ak && bk) launch<BN, false, true, InT, OUT_F32>(ta, tb, to, tz, p, grid, s);
  else launch<BN, false, false, InT, OUT_F32>(ta, tb, to, tz, p, grid, s);
}

// Host entry.  a: [M,K] (trans_a=false) or [K,M]; b: [K,N] (trans_b=false) or [N,K]; both contiguous 2-D.
void gemm_launch(const GemmArgs& g, cudaStream_t stream) {
  const bool a_kmajor = !g.trans_a;
  const bool b_kmajor = g.trans_b;
  // 128-wide tiles read 128 B of shared memory per tensor-core clock against 96 B for 256-wide ones and lose even
  // where they waste fewer columns (N = 800: 115 us with 7 tiles of 128, 83 us with 4 tiles of 256)
  const int bn = g.N <= 128 ? 128 : 256;
  const int tiles = ((g.M + kBM - 1) / kBM) * ((g.N + bn - 1) / bn);
  const int kb_total = (g.K + kBK - 1) / kBK;
  int sms = g.num_sms;
  int splits = 1;
  if (g.out_f32 && g.allow_split_k && tiles * 2 <= sms && kb_total >= 16) {
    splits = std::min(std::min(sms / tiles, kb_total / 8), 32);
    if (splits < 1) splits = 1;
  } else if (g.out_f32 && g.allow_split_k && kb_total >= 64) {
    // A weight gradient has few, very long tiles (K = tokens): 350 tiles on 148 SMs leave the third wave 36 % full.
    // Splitting K evens the waves out: take the smallest factor (each one costs a pass of fp32 red.add over the
    // output) whose last wave is at least 93 % full, else the fullest of 1..8.
    double best = 0.0;
    for (int sp = 1; sp <= 8 && kb_total / sp >= 32; ++sp) {
      const double waves = static_cast<double>(tiles) * sp / sms;
      const double eff = waves / std::ceil(waves);
      if (eff > best + 1e-9) { best = eff; splits = sp; }
      if (eff >= 0.93) break;
    }
  }
  {
    // no split may be empty: an accumulator that no MMA wrote holds stale TMEM contents
    const int per = (kb_total + splits - 1) / splits;
    splits = (kb_total + per - 1) / per;
  }
  if (splits > 1) {
    TORCH_CHECK(g.out_f32 && g.act == kActNone && g.z_out == nullptr, "split-K needs an fp32 output and no activation");
    C10_CUDA_CHECK(cudaMemsetAsync(g.out, 0, static_cast<size_t>(g.M) * g.N * sizeof(float), stream));
  }
  CUtensorMap ta = a_kmajor ? make_tma_2d(g.a, g.M, g.K, g.K, kBM) : make_tma_2d(g.a, g.K, g.M, g.M, 64);
  CUtensorMap tb = b_kmajor ? make_tma_2d(g.b, g.N, g.K, g.K, bn) : make_tma_2d(g.b, g.K, g.N, g.N, 64);
  GemmParams p;
  p.M = g.M; p.N = g.N; p.K = g.K;
  p.out = g.out; p.z_out = g.z_out; p.bias = g.bias; p.ldo = g.N;
  p.act = g.act; p.splits = splits; p.is_bf16 = g.is_bf16 ? 1 : 0;
  p.status = g.status;
  // tile stores through TMA need a 16-byte aligned base and row pitch; anything else takes the direct-store path
  const int out_bytes = g.out_f32 ? 4 : 2;
  const bool out_ok = (reinterpret_cast<uintptr_t>(g.out) & 15) == 0 && (static_cast<size_t>(g.N) * out_bytes) % 16 == 0;
  const bool z_ok = g.z_out == nullptr || ((reinterpret_cast<uintptr_t>(g.z_out) & 15) == 0 && (static_cast<size_t>(g.N) * 2) % 16 == 0);
  p.tma_store = (out_ok && z_ok) ? 1 : 0;
  CUtensorMap to = ta, tz = ta;      // placeholders when unused
  if (p.tma_store) {
    to = make_tma_2d_store(g.out, g.M, g.N, g.N, out_bytes, g.is_bf16);
    if (g.z_out != nullptr) tz = make_tma_2d_store(g.z_out, g.M, g.N, g.N, 2, g.is_bf16);
  }
  const int grid = std::min(tiles * splits, sms);
  if (g.is_bf16) {
    if (bn == 256) {
      if (g.out_f32) dispatch_major<256, __nv_bfloat16, true>(a_kmajor, b_kmajor, ta, tb, to, tz, p, grid, stream);
      else dispatch_major<256, __nv_bfloat16, false>(a_kmajor, b_kmajor, ta, tb, to, tz, p, grid, stream);
    } else {
      if (g.out_f32) dispatch_major<128, __nv_bfloat16, true>(a_kmajor, b_kmajor, ta, tb, to, tz, p, grid, stream);
      else dispatch_major<128, __nv_bfloat16, false>(a_kmajor, b_kmajor, ta, tb, to, tz, p, grid, stream);
    }
  } else {
    if (bn == 256) {
      if (g.out_f32) dispatch_major<256, __half, true>(a_kmajor, b_kmajor, ta, tb, to, tz, p, grid, stream);
      else dispatch_major<256, __half, false>(a_kmajor, b_kmajor, ta, tb, to, tz, p, grid, stream);
    } else {
      if (g.out_f32) dispatch_major<128, __half, true>(a_kmajor, b_kmajor, ta, tb, to, tz, p, grid, stream);
      else dispatch_major<128, __half, false>(a_kmajor, b_kmajor, ta, tb, to, tz, p, grid, stream);
    }
  }
}

}  // namespace cw
