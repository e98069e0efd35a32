// GEMM fused with the all-reduce that follows it (1D row-parallel forward, column-parallel backward,
// Classifier1D): ONE kernel per rank computes the local partial product on tcgen05 tensor cores and moves
// the tiles over NVLink peer memory while later tiles are still being multiplied.
//
//   out = sum over ranks( op(A_r) * op(B_r) ) + bias          identical on every rank of the group
//
// Grid = G GEMM CTAs + R communication CTAs, all co-resident (one CTA per SM).
//  * GEMM CTAs: the persistent TMA -> tcgen05 -> TMEM pipeline of gemm_sm100.cu; each epilogue warp converts
//    its 32 rows of the partial tile to 16-bit in shared memory and sends them with one 16 KB bulk copy
//    straight into the *owner's* staging buffer through its peer pointer (tile t is owned by rank t mod n),
//    then publishes an arrival flag there.
//  * communication CTAs, tile by tile in production order; warp 0 issues, warps 1-5 work:
//      owner:  wait for the n partials, sum them in fp32 (+ bias), write the result tile to its own output
//              and to its result buffer, publish a "done" flag to every peer;
//      others: warp 0 waits for "done" and bulk-copies the result tile from the owner's result buffer into one
//              of three shared-memory slots (running up to three tiles ahead); the workers copy it to the output.
// Flags hold a call epoch that only grows, so nothing is ever reset.  Every wait is bounded and reports to
// the status word.  Remote accesses are bulk copies and ordinary ld/st through IPC-mapped pointers; no TMA
// tensor map ever covers peer memory.
//
// The reference issues a cuBLAS GEMM and then a blocking NCCL all-reduce (cubework/module/parallel_1d/
// module.py:331-346 -> _utils.py:73-74; backward _utils.py:63-64).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/pybind11.h>
#include <torch/extension.h>

#include "gemm_sm100.cuh"

namespace py = pybind11;

namespace cw {

constexpr int kFusedBN = 256;
constexpr int kMaxRanks = 8;
constexpr int kTileElems = kBM * kFusedBN;          // 16-bit elements per staged tile

struct FusedParams {
  int M, N, K;
  int n, me, epoch;
  int num_gemm_ctas, num_comm_ctas;
  int is_bf16;
  uint32_t mn_lbo, mn_sbo;
  void* stage[kMaxRanks];        // peer pointers: [owned tiles][n sources][128 x 256] 16-bit
  void* result[kMaxRanks];       // peer pointers: [owned tiles][128 x 256] 16-bit
  int* flags[kMaxRanks];         // peer pointers: [done_cap] "done" epochs, then [owned tiles][n sources][4] arrivals
  int done_cap;
  void* out;                     // local [M, N] 16-bit
  const float* bias;             // optional [N]
  int* status;
};

__device__ __forceinline__ float tof(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float tof(__half v) { return __half2float(v); }
// 16-byte load that bypasses L1 (the data was written by another GPU, or by another SM of this one)
__device__ __forceinline__ uint4 ld_cg16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Wait until *flag >= epoch.  Bounded; returns false on timeout (after recording it).
__device__ __forceinline__ bool wait_flag(const int* flag, int epoch, int* status, int detail) {
  if (ld_acquire_sys(flag) >= epoch) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (uint32_t spin = 1;; ++spin) {
    if (ld_acquire_sys(flag) >= epoch) return true;
    if ((spin & 63u) == 0) {
      __nanosleep(200);
      if (globaltimer_ns() - t0 > kWaitLimitNs) {
        report_error(status, kErrPeerFlagTimeout, detail);
        return false;
      }
    }
  }
}

constexpr int kFusedStages = 3;
constexpr int kSlabBytes = 32 * kFusedBN * 2;                 // one epilogue warp's 32 rows of a tile (16 KB)
constexpr int kEpiBytes = 4 * kSlabBytes;                      // 64 KB
constexpr int kPullSlots = 3;
constexpr int kTileBytes = kTileElems * 2;                     // 64 KB
constexpr int kFusedSmemBytes = kFusedStages * GemmCfg<kFusedBN>::kStageBytes + kEpiBytes + 256 + 1024;
static_assert(kPullSlots * kTileBytes + 256 + 1024 <= kFusedSmemBytes, "pull slots must fit the same allocation");
constexpr int kWorkers = kGemmThreads - 32;                    // communication CTA: warp 0 issues, warps 1-5 work

__device__ __forceinline__ void bulk_store(void* gdst, const void* ssrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(ssrc)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_load(void* sdst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(sdst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void worker_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kWorkers) : "memory"); }

// Element offset of 16-byte chunk j (0..31) of row r inside a staged 128 x 256 tile.  The chunk position is
// XOR-ed with the row so the epilogue's row-per-lane shared-memory writes are bank-conflict free; the staged tile
// is copied verbatim to the owner, whose reducer applies the same mapping when it reads.
__device__ __forceinline__ int staged_off(int r, int j) { return r * kFusedBN + ((j ^ (r & 31)) << 3); }

template <bool A_KMAJOR, bool B_KMAJOR, typename InT>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_allreduce_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                      FusedParams p) {
  constexpr int BN = kFusedBN;
  using Cfg = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (p.M + kBM - 1) / kBM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int kb_total = (p.K + kBK - 1) / kBK;
  const bool is_comm = static_cast<int>(blockIdx.x) >= p.num_gemm_ctas;

  if (is_comm) {
    // =============================================================== communication CTA
    uint8_t* slots = smem;                                            // kPullSlots x 64 KB
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kPullSlots * kTileBytes);
    uint64_t* empty_bar = full_bar + kPullSlots;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + kPullSlots);
    if (threadIdx.x == 0) {
      for (int s = 0; s < kPullSlots; ++s) {
        mbar_init(&full_bar[s], 1);
        mbar_init(&empty_bar[s], kWorkers / 32);
      }
      *abort_flag = 0;
      fence_barrier_init();
    }
    __syncthreads();
    const int c = blockIdx.x - p.num_gemm_ctas;
    if (warp == 0) {
      // ---- issuer: runs ahead of the workers, fetching finished tiles of other owners into free slots
      if (lane == 0) {
        int slot = 0;
        uint32_t phase = 0;
        for (int t = c; t < num_tiles && !*abort_flag; t += p.num_comm_ctas) {
          const int owner = t % p.n;
          if (owner == p.me) continue;
          if (!mbar_wait(&empty_bar[slot], phase ^ 1, abort_flag, p.status, kErrPeerFlagTimeout, t)) break;
          if (!wait_flag(p.flags[p.me] + t, p.epoch, p.status, t)) { *abort_flag = 1; break; }
          const uint8_t* src = reinterpret_cast<const uint8_t*>(p.result[owner]) + static_cast<size_t>(t / p.n) * kTileBytes;
          mbar_expect_tx(&full_bar[slot], kTileBytes);
#pragma unroll
          for (int q = 0; q < 4; ++q)
            bulk_load(slots + slot * kTileBytes + q * (kTileBytes / 4), src + q * (kTileBytes / 4), kTileBytes / 4,
                      &full_bar[slot]);
          if (++slot == kPullSlots) { slot = 0; phase ^= 1; }
        }
      }
      return;
    }
    // ---- workers
    const int wid = threadIdx.x - 32;
    InT* out = reinterpret_cast<InT*>(p.out);
    int slot = 0;
    uint32_t phase = 0;
    for (int t = c; t < num_tiles; t += p.num_comm_ctas) {
      if (*abort_flag) break;
      int tile_m, tile_n, kb0, kb1;
      decode_work(t, num_tiles, tiles_m, tiles_n, kb_total, 1, tile_m, tile_n, kb0, kb1);
      const int owner = t % p.n;
      const int li = t / p.n;
      const int rows = min(kBM, p.M - tile_m * kBM);
      const int cols = min(BN, p.N - tile_n * BN);
      const int vec_per_row = cols >> 3;                    // 16-byte vectors (N is a multiple of 8)
      const int total_vec = rows * vec_per_row;
      InT* out_tile = out + static_cast<size_t>(tile_m * kBM) * p.N + tile_n * BN;
      if (owner == p.me) {
        // wait for the n x 4 arrival words of this tile, then sum the n staged partials
        if (warp == 1) {
          const int nflags = p.n * 4;
          for (int f = lane; f < nflags; f += 32)
            if (!wait_flag(p.flags[p.me] + p.done_cap + static_cast<size_t>(li) * nflags + f, p.epoch, p.status, t))
              *abort_flag = 1;
        }
        worker_sync();
        if (*abort_flag) break;
        const InT* stage = reinterpret_cast<const InT*>(p.stage[p.me]) + static_cast<size_t>(li) * p.n * kTileElems;
        InT* res = reinterpret_cast<InT*>(p.result[p.me]) + static_cast<size_t>(li) * kTileElems;
        for (int v = wid; v < total_vec; v += kWorkers) {
          const int r = v / vec_per_row, j = v - r * vec_per_row;
          float acc[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = 0.f;
          const int off = staged_off(r, j);
          for (int src = 0; src < p.n; ++src) {
            const uint4 raw = ld_cg16(stage + static_cast<size_t>(src) * kTileElems + off);
            const InT* h = reinterpret_cast<const InT*>(&raw);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] += tof(h[i]);
          }
          const int gcol = tile_n * BN + j * 8;
          if (p.bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] += __ldg(p.bias + gcol + i);
          }
          uint4 o;
          o.x = pack2(acc[0], acc[1], InT());
          o.y = pack2(acc[2], acc[3], InT());
          o.z = pack2(acc[4], acc[5], InT());
          o.w = pack2(acc[6], acc[7], InT());
          *reinterpret_cast<uint4*>(res + r * BN + j * 8) = o;
          *reinterpret_cast<uint4*>(out_tile + static_cast<size_t>(r) * p.N + j * 8) = o;
        }
        worker_sync();
        if (wid < p.n && wid != p.me) {
          __threadfence_system();
          st_release_sys(p.flags[wid] + t, p.epoch);
        }
      } else {
        if (!mbar_wait(&full_bar[slot], phase, abort_flag, p.status, kErrPeerFlagTimeout, t)) break;
        const InT* tile = reinterpret_cast<const InT*>(slots + slot * kTileBytes);
        for (int v = wid; v < total_vec; v += kWorkers) {
          const int r = v / vec_per_row, j = v - r * vec_per_row;
          *reinterpret_cast<uint4*>(out_tile + static_cast<size_t>(r) * p.N + j * 8) =
              *reinterpret_cast<const uint4*>(tile + r * BN + j * 8);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[slot]);
        if (++slot == kPullSlots) { slot = 0; phase ^= 1; }
      }
    }
    return;
  }

  // ================================================================= GEMM CTA
  uint8_t* epi = smem + kFusedStages * Cfg::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(epi + kEpiBytes);
  uint64_t* empty_bar = full_bar + kFusedStages;
  uint64_t* tfull_bar = empty_bar + kFusedStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  if (threadIdx.x == 0) {
    for (int s = 0; s < kFusedStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int G = p.num_gemm_ctas;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int w = blockIdx.x; w < num_tiles && !*abort_flag; w += G) {
        int tile_m, tile_n, kb0, kb1;
        decode_work(w, num_tiles, tiles_m, tiles_n, kb_total, 1, tile_m, tile_n, kb0, kb1);
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
          if (++stage == kFusedStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(kBM, BN, !A_KMAJOR, !B_KMAJOR, p.is_bf16);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int w = blockIdx.x; w < num_tiles && !*abort_flag; w += G, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status, kErrTmemEmptyTimeout, w)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kErrFullBarrierTimeout, w)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t sb = sa + Cfg::kABytes;
#pragma unroll
          for (int k16 = 0; k16 < kBK / 16; ++k16) {
            const uint64_t da = A_KMAJOR ? make_smem_desc(sa + k16 * 32, 16, 1024)
                                         : make_smem_desc(sa + k16 * 2048, p.mn_lbo, p.mn_sbo);
            const uint64_t db = B_KMAJOR ? make_smem_desc(sb + k16 * 32, 16, 1024)
                                         : make_smem_desc(sb + k16 * 2048, p.mn_lbo, p.mn_sbo);
            tc_mma_f16(d_tmem, da, db, idesc, (kb > 0 || k16 > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == kFusedStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(&tfull_bar[acc]);
      }
    }
  } else {
    // ---- epilogue: TMEM -> 16-bit -> this warp's shared slab -> ONE 16 KB bulk copy into the owner's staging
    //      slot (peer memory), then the arrival flag
    const int quarter = warp & 3;
    uint8_t* slab = epi + quarter * kSlabBytes;
    int it = 0;
    for (int w = blockIdx.x; w < num_tiles && !*abort_flag; w += G, ++it) {
      int tile_m, tile_n, kb0, kb1;
      decode_work(w, num_tiles, tiles_m, tiles_n, kb_total, 1, tile_m, tile_n, kb0, kb1);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, kErrTmemFullTimeout, w)) break;
      tc_fence_after();
      const int owner = w % p.n;
      const int li = w / p.n;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        if (tile_n * BN + c * 32 >= p.N) break;
        uint32_t raw[32];
        tmem_ld_32x32(tmem_base + acc * BN + c * 32 + (static_cast<uint32_t>(quarter * 32) << 16), raw);
        tmem_wait_ld();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 u;
          u.x = pack2(__uint_as_float(raw[q * 8 + 0]), __uint_as_float(raw[q * 8 + 1]), InT());
          u.y = pack2(__uint_as_float(raw[q * 8 + 2]), __uint_as_float(raw[q * 8 + 3]), InT());
          u.z = pack2(__uint_as_float(raw[q * 8 + 4]), __uint_as_float(raw[q * 8 + 5]), InT());
          u.w = pack2(__uint_as_float(raw[q * 8 + 6]), __uint_as_float(raw[q * 8 + 7]), InT());
          *reinterpret_cast<uint4*>(slab + staged_off(lane, c * 4 + q) * 2) = u;
        }
      }
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&tempty_bar[acc]);           // the accumulator can be refilled while the copy is in flight
        InT* slot = reinterpret_cast<InT*>(p.stage[owner]) + (static_cast<size_t>(li) * p.n + p.me) * kTileElems;
        bulk_store(slot + quarter * 32 * BN, slab, kSlabBytes);
        bulk_commit_group();
        bulk_wait_group0();                      // written, not merely read: the flag must not overtake the data
        __threadfence_system();
        st_release_sys(p.flags[owner] + p.done_cap + (static_cast<size_t>(li) * p.n + p.me) * 4 + quarter, p.epoch);
      }
      __syncwarp();                              // the slab is free again
    }
  }

  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <bool AK, bool BK_, typename InT>
static void launch_fused(const CUtensorMap& ta, const CUtensorMap& tb, const FusedParams& p, cudaStream_t stream) {
  auto kern = gemm_allreduce_kernel<AK, BK_, InT>;
  static bool configured = false;
  if (!configured) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kFusedSmemBytes));
    configured = true;
  }
  kern<<<p.num_gemm_ctas + p.num_comm_ctas, kGemmThreads, kFusedSmemBytes, stream>>>(ta, tb, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// out (pre-allocated [M, N], same dtype as a) = all-reduce over the group of op(a) op(b), + bias.
// stage / result / flags: device pointers of every rank's workspace buffers, indexed by group rank.
static void fused_gemm_all_reduce(torch::Tensor a, torch::Tensor b, bool trans_a, bool trans_b,
                                  c10::optional<torch::Tensor> bias, torch::Tensor out, std::vector<int64_t> stage,
                                  std::vector<int64_t> result, std::vector<int64_t> flags, int64_t done_cap, int64_t me,
                                  int64_t epoch, int64_t num_comm_ctas, int64_t status_ptr) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.dim() == 2 && b.dim() == 2 && a.is_contiguous() && b.is_contiguous());
  TORCH_CHECK(a.scalar_type() == b.scalar_type() && out.scalar_type() == a.scalar_type() && out.is_contiguous());
  const int n = static_cast<int>(stage.size());
  TORCH_CHECK(n >= 2 && n <= kMaxRanks && result.size() == stage.size() && flags.size() == stage.size());
  c10::cuda::CUDAGuard guard(a.device());
  const int M = trans_a ? a.size(1) : a.size(0);
  const int K = trans_a ? a.size(0) : a.size(1);
  const int N = trans_b ? b.size(0) : b.size(1);
  TORCH_CHECK((trans_b ? b.size(1) : b.size(0)) == K && out.size(0) == M && out.size(1) == N);
  TORCH_CHECK(N % 8 == 0, "the fused all-reduce moves 16-byte vectors: N must be a multiple of 8");
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  FusedParams p{};
  p.M = M; p.N = N; p.K = K;
  p.n = n; p.me = static_cast<int>(me); p.epoch = static_cast<int>(epoch);
  p.num_comm_ctas = std::max(1, std::min(static_cast<int>(num_comm_ctas), sms - 1));
  p.num_gemm_ctas = sms - p.num_comm_ctas;
  p.is_bf16 = a.scalar_type() == torch::kBFloat16;
  p.mn_lbo = 8192; p.mn_sbo = 1024;
  for (int i = 0; i < n; ++i) {
    p.stage[i] = reinterpret_cast<void*>(stage[i]);
    p.result[i] = reinterpret_cast<void*>(result[i]);
    p.flags[i] = reinterpret_cast<int*>(flags[i]);
  }
  p.done_cap = static_cast<int>(done_cap);
  p.out = out.data_ptr();
  torch::Tensor bias_f;
  if (bias.has_value() && bias->defined()) {
    bias_f = bias->to(torch::kFloat32).contiguous();
    p.bias = bias_f.data_ptr<float>();
  }
  p.status = reinterpret_cast<int*>(status_ptr);
  const bool ak = !trans_a, bk = trans_b;
  CUtensorMap ta = ak ? make_tma_2d(a.data_ptr(), M, K, K, kBM) : make_tma_2d(a.data_ptr(), K, M, M, 64);
  CUtensorMap tb = bk ? make_tma_2d(b.data_ptr(), N, K, K, kFusedBN) : make_tma_2d(b.data_ptr(), K, N, N, 64);
  auto stream = at::cuda::getCurrentCUDAStream();
#define FUSED_DISPATCH(T)                                                  \
  if (ak && bk) launch_fused<true, true, T>(ta, tb, p, stream);            \
  else if (ak && !bk) launch_fused<true, false, T>(ta, tb, p, stream);     \
  else if (!ak && bk) launch_fused<false, true, T>(ta, tb, p, stream);     \
  else launch_fused<false, false, T>(ta, tb, p, stream);
  if (p.is_bf16) { FUSED_DISPATCH(__nv_bfloat16) } else { FUSED_DISPATCH(__half) }
#undef FUSED_DISPATCH
}

void register_fused(py::module& m) { m.def("fused_gemm_all_reduce", &fused_gemm_all_reduce); }

}  // namespace cw
