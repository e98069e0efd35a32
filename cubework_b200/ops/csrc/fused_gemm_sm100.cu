// GEMM fused with the all-reduce that follows it (1D row-parallel forward, column-parallel backward,
// Classifier1D): ONE kernel per rank computes the local partial product on tcgen05 tensor cores and moves
// the tiles over NVLink peer memory while later tiles are still being multiplied.
//
//   out = sum over ranks( op(A_r) * op(B_r) ) + bias          identical on every rank of the group
//
// Grid = G GEMM CTAs + R communication CTAs, all co-resident (one CTA per SM).
//  * GEMM CTAs: the persistent TMA -> tcgen05 -> TMEM pipeline of gemm_sm100.cu.  Tile t is owned by rank
//    t mod n.  "Push" CTAs compute tiles of other owners: each epilogue warp converts 32 rows x 128 columns to
//    16-bit in shared memory and sends them with one 8 KB bulk copy straight into the owner's staging buffer
//    (peer pointer).  "Own" CTAs compute this rank's tiles: the epilogue waits for the n-1 staged partials, adds
//    them to the accumulator (+ bias) and writes the rows to the output and to the result buffer - the
//    reduction rides in the GEMM epilogue, there is no separate pass.  Flags (arrival of a partial, result
//    done) are written by one publisher thread per CTA that batches them behind a single system-scope fence.
//  * communication CTAs (a few): wait for "done" flags, bulk-load finished tiles of other owners from the
//    owner's result buffer into shared-memory slots (three in flight) and bulk-store their rows into the output.
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

#include "fused_common.cuh"

namespace py = pybind11;

namespace cw {

struct FusedParams {
  int M, N, K;
  int n, me, epoch;
  int num_gemm_ctas, num_comm_ctas;
  int is_bf16;
  uint32_t mn_lbo, mn_sbo;
  void* stage[kMaxRanks];        // peer pointers: [owned tiles][n sources][128 x 256] 16-bit
  void* result[kMaxRanks];       // peer pointers: [owned tiles][128 x 256] 16-bit
  int* flags[kMaxRanks];         // peer pointers: [done_cap][8] "done" epochs, then [owned tiles][n sources][8] arrivals
  int done_cap;
  void* out;                     // local [M, N] 16-bit
  const float* bias;             // optional [N]
  int* status;
  long long* trace;              // optional [ctas][kTraceLen][2] (event, globaltimer) for performance debugging
};

// Tile schedule.  Tile t is owned by rank t mod n.  GEMM CTAs are split into "push" CTAs, which compute tiles of
// other owners and never wait for anybody, and "own" CTAs, which compute this rank's tiles and wait for the other
// ranks' partials.  Push item p -> group p / (n-1), and inside the group the (p mod (n-1))-th owner after `me`.
__device__ __forceinline__ int push_item_tile(int p, int n, int me, int num_tiles) {
  const int g = p / (n - 1), j = p - g * (n - 1);
  const int t = g * n + (me + 1 + j) % n;
  return t < num_tiles ? t : -1;
}

template <bool A_KMAJOR, bool B_KMAJOR, typename InT>
__global__ void __launch_bounds__(kFusedThreads, 1)
gemm_allreduce_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                      const __grid_constant__ CUtensorMap tma_out, FusedParams p) {
  constexpr int BN = kFusedBN;
  using Cfg = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (p.M + kBM - 1) / kBM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_groups = (num_tiles + p.n - 1) / p.n;
  const int kb_total = (p.K + kBK - 1) / kBK;
  const bool is_comm = static_cast<int>(blockIdx.x) >= p.num_gemm_ctas;

  if (is_comm) {
    // =============================================================== communication CTA: pull finished tiles
    // warp 0 lane 0: waits for "done" flags and bulk-loads result tiles (dense [128][256]) of other owners into one
    // of three slots; warp 1: bulk-stores the rows of a landed slot into the output.  No thread touches the data.
    uint8_t* slots = smem;                                            // kPullSlots x 64 KB
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kPullSlots * kTileBytes);
    uint64_t* empty_bar = full_bar + kPullSlots;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + kPullSlots);
    if (threadIdx.x == 0) {
      for (int s = 0; s < kPullSlots; ++s) {
        mbar_init(&full_bar[s], 1);
        mbar_init(&empty_bar[s], 1);
      }
      *abort_flag = 0;
      fence_barrier_init();
    }
    __syncthreads();
    const int c = blockIdx.x - p.num_gemm_ctas;
    if (warp > 1) return;
    int slot = 0, k = 0, ntr = 0;
    uint32_t phase = 0;
    int pending_slot = -1;                                            // warp 1: slot whose stores are in flight
    for (int t = 0; t < num_tiles; ++t) {
      if (t % p.n == p.me) continue;
      if ((k++) % p.num_comm_ctas != c) continue;
      if (*abort_flag) break;
      int tile_m, tile_n, kb0, kb1;
      decode_work(t, num_tiles, tiles_m, tiles_n, kb_total, 1, tile_m, tile_n, kb0, kb1);
      const int cols = min(BN, p.N - tile_n * BN);
      if (warp == 0) {
        bool ok = true;
        if (lane == 0) ok = mbar_wait(&empty_bar[slot], phase ^ 1, abort_flag, p.status, kErrPeerFlagTimeout, t);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        if (lane == 0) trace_ev(p.trace, ntr, 10, t);
        const bool second_half = cols > 128;                          // an edge tile may have no second column half
        if (lane < 8 && ((lane & 1) == 0 || second_half)) {           // one "done" word per (32-row slab, half)
          if (!wait_flag(p.flags[p.me] + t * 8 + lane, p.epoch, p.status, t)) *abort_flag = 1;
        }
        __syncwarp();
        if (*abort_flag) break;
        if (lane == 0) {
          trace_ev(p.trace, ntr, 11, t);
          const int owner = t % p.n;
          const uint8_t* src = reinterpret_cast<const uint8_t*>(p.result[owner]) + static_cast<size_t>(t / p.n) * kTileBytes;
          mbar_expect_tx(&full_bar[slot], kTileBytes);
#pragma unroll
          for (int q = 0; q < 4; ++q)
            bulk_load(slots + slot * kTileBytes + q * kSlabBytes, src + q * kSlabBytes, kSlabBytes, &full_bar[slot]);
        }
      } else {
        if (!mbar_wait(&full_bar[slot], phase, abort_flag, p.status, kErrPeerFlagTimeout, t)) break;
        // the rows of the previous slot have been read out of shared memory: hand that slot back
        // (each lane waits for its own stores; the warp then agrees)
        bulk_wait_group_read_n<0>();
        __syncwarp();
        if (pending_slot >= 0 && lane == 0) mbar_arrive(&empty_bar[pending_slot]);
        if (lane == 0) {
          // one TMA tile store: the box is clipped against the output's extent, so edge tiles need no special case
          tma_store_2d(&tma_out, slots + slot * kTileBytes, tile_n * BN, tile_m * kBM);
          bulk_commit_group();
        }
        pending_slot = slot;
      }
      if (++slot == kPullSlots) { slot = 0; phase ^= 1; }
    }
    if (warp == 1) {
      bulk_wait_group0();
      __syncwarp();
      if (pending_slot >= 0 && lane == 0) mbar_arrive(&empty_bar[pending_slot]);
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
  __shared__ Mailbox mailbox;
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
    for (int q = 0; q < 4; ++q) { mailbox.tail[q] = 0; mailbox.head[q] = 0; }
    mailbox.finished = 0;
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

  // role of this CTA and its tile list: tile(k), k = 0, 1, ... until -2
  const int G = p.num_gemm_ctas;
  int g_push = (G * (p.n - 1) + p.n / 2) / p.n;
  g_push = max(1, min(G - 1, g_push));
  const int g_own = G - g_push;
  const bool push_role = static_cast<int>(blockIdx.x) < g_push;
  const int n_push_items = num_groups * (p.n - 1);
  auto tile_of = [&](int k) -> int {             // -1: skip, -2: finished
    if (push_role) {
      const int item = blockIdx.x + k * g_push;
      return item < n_push_items ? push_item_tile(item, p.n, p.me, num_tiles) : -2;
    }
    const int grp = (blockIdx.x - g_push) + k * g_own;
    if (grp >= num_groups) return -2;
    const int t = grp * p.n + p.me;
    return t < num_tiles ? t : -1;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int k = 0; !*abort_flag; ++k) {
        const int t = tile_of(k);
        if (t == -2) break;
        if (t < 0) continue;
        int tile_m, tile_n, kb0, kb1;
        decode_work(t, num_tiles, tiles_m, tiles_n, kb_total, 1, tile_m, tile_n, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kErrEmptyBarrierTimeout, t)) break;
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
      for (int k = 0; !*abort_flag; ++k) {
        const int t = tile_of(k);
        if (t == -2) break;
        if (t < 0) continue;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ++it;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status, kErrTmemEmptyTimeout, t)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kErrFullBarrierTimeout, t)) { ok = false; break; }
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
  } else if (warp == kPublisherWarp) {
    if (lane == 0) {
      // ---- publisher: batches completed copies, one system-scope fence per batch, then the flags
      int head[4] = {0, 0, 0, 0};
      const unsigned long long t_start = globaltimer_ns();
      for (;;) {
        int batch[32];
        int nb = 0;
        const int fin = mailbox.finished;
        for (int q = 0; q < 4; ++q) {
          const int tail = mailbox.tail[q];
          while (head[q] < tail && nb < 32) {
            batch[nb++] = mailbox.item[q][head[q] % kMailboxDepth];
            ++head[q];
          }
          mailbox.head[q] = head[q];
        }
        if (nb == 0) {
          if (fin == 4 || *abort_flag) {
            bool drained = true;
            for (int q = 0; q < 4; ++q) drained = drained && head[q] == mailbox.tail[q];
            if (drained) break;
            continue;
          }
          if (globaltimer_ns() - t_start > 4 * kWaitLimitNs) break;      // never spin forever
          __nanosleep(100);
          continue;
        }
        __threadfence_block();
        __threadfence_system();
        for (int b = 0; b < nb; ++b) {
          const int t = batch[b] >> 3, qh = batch[b] & 7;
          const int owner = t % p.n, li = t / p.n;
          if (owner == p.me) {
            for (int peer = 0; peer < p.n; ++peer)
              if (peer != p.me) st_relaxed_sys(p.flags[peer] + t * 8 + qh, p.epoch);
          } else {
            st_relaxed_sys(p.flags[owner] + p.done_cap * 8 + (static_cast<size_t>(li) * p.n + p.me) * 8 + qh, p.epoch);
          }
        }
      }
    }
  } else {
    // ---- epilogue, per tile in two column halves of 128 (half-slabs of 8 KB per warp, used alternately).
    //  push role: 16-bit partial -> half-slab -> one bulk copy into the owner's staging slot (peer memory); the copy
    //             is recorded for publication once `wait_group 1` shows it has completed.
    //  own role : wait for the n-1 staged partials of these rows, add them (+ bias), write the rows to the output
    //             and to the (dense) result buffer with coalesced stores, record the half for publication.
    const int quarter = warp & 3;
    uint8_t* buf = epi + quarter * kHalfSlabBytes;             // this warp's 32 x 128 half-slab
    InT* out = reinterpret_cast<InT*>(p.out);
    int pend = -1;                                             // lane 0, push role: the copy issued last, not yet published
    int mb_tail = 0;
    int it = 0, ntr = 0;
    const bool tr = quarter == 0 && lane == 0;
    bool failed = false;
    for (int k = 0; !*abort_flag && !failed; ++k) {
      const int t = tile_of(k);
      if (t == -2) break;
      if (t < 0) continue;
      int tile_m, tile_n, kb0, kb1;
      decode_work(t, num_tiles, tiles_m, tiles_n, kb_total, 1, tile_m, tile_n, kb0, kb1);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ++it;
      if (tr) trace_ev(p.trace, ntr, 1, t);
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, kErrTmemFullTimeout, t)) break;
      tc_fence_after();
      if (tr) trace_ev(p.trace, ntr, 2, t);
      const int owner = t % p.n;
      const int li = t / p.n;
      const bool mine = owner == p.me;
      const InT* stage = reinterpret_cast<const InT*>(p.stage[p.me]) + static_cast<size_t>(li) * p.n * kTileElems;
      const int r = quarter * 32 + lane;                       // row inside the tile
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        const int colh = tile_n * BN + h * 128;
        if (colh >= p.N) break;                                // warp-uniform: this half is entirely out of range
        if (!mine && lane == 0) {
          bulk_wait_group_read_n<0>();                         // the previous copy has finished reading `buf`
          if (tr) trace_ev(p.trace, ntr, 3, t * 2 + h);
        }
        if (mine) {
          bool ok = true;                                      // the other ranks' half-slabs of these rows have landed
          if (lane < p.n && lane != p.me)
            ok = wait_flag(p.flags[p.me] + p.done_cap * 8 + (static_cast<size_t>(li) * p.n + lane) * 8 + quarter * 2 + h,
                           p.epoch, p.status, t);
          if (__any_sync(0xffffffffu, !ok)) { failed = true; break; }
          if (tr) trace_ev(p.trace, ntr, 4, t * 2 + h);
        }
        __syncwarp();
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          const int col0 = colh + c * 32;
          if (col0 >= p.N) break;
          uint32_t raw[32];
          tmem_ld_32x32(tmem_base + acc * BN + h * 128 + c * 32 + (static_cast<uint32_t>(quarter * 32) << 16), raw);
          tmem_wait_ld();
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
          if (mine) {
            for (int src = 0; src < p.n; ++src) {
              if (src == p.me) continue;
              uint4 part[4];
#pragma unroll
              for (int q = 0; q < 4; ++q)
                part[q] = ld_cg16(stage + static_cast<size_t>(src) * kTileElems + staged_off(r, h * 16 + c * 4 + q));
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const InT* hh = reinterpret_cast<const InT*>(&part[q]);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[q * 8 + e] += tof(hh[e]);
              }
            }
            if (p.bias != nullptr) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) v[j] += __ldg(p.bias + col0 + j);
            }
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 u;
            u.x = pack2(v[q * 8 + 0], v[q * 8 + 1], InT());
            u.y = pack2(v[q * 8 + 2], v[q * 8 + 3], InT());
            u.z = pack2(v[q * 8 + 4], v[q * 8 + 5], InT());
            u.w = pack2(v[q * 8 + 6], v[q * 8 + 7], InT());
            *reinterpret_cast<uint4*>(buf + (lane * 128 + (((c * 4 + q) ^ (lane & 15)) << 3)) * 2) = u;
          }
        }
        __syncwarp();
        if (mine) {
          // rows -> output and dense result tile: two 256-byte row halves per step (lane>>4 = row, lane&15 = chunk)
          const int cols = min(128, p.N - colh);
          const int rows_here = min(32, p.M - tile_m * kBM - quarter * 32);
          InT* out_rows = out + static_cast<size_t>(tile_m * kBM + quarter * 32) * p.N + colh;
          InT* res_rows = reinterpret_cast<InT*>(p.result[p.me]) + static_cast<size_t>(li) * kTileElems +
                          (quarter * 32) * BN + h * 128;
          const int jj = lane & 15;
          for (int rr = lane >> 4; rr < 32; rr += 2) {
            const uint4 val = *reinterpret_cast<const uint4*>(buf + (rr * 128 + ((jj ^ (rr & 15)) << 3)) * 2);
            *reinterpret_cast<uint4*>(res_rows + rr * BN + jj * 8) = val;
            if (rr < rows_here && jj * 8 < cols) *reinterpret_cast<uint4*>(out_rows + static_cast<size_t>(rr) * p.N + jj * 8) = val;
          }
          __syncwarp();
          if (lane == 0) {
            mailbox_put(&mailbox, quarter, mb_tail, 0, (t << 3) | (quarter << 1) | h);
            if (tr) trace_ev(p.trace, ntr, 5, t * 2 + h);
          }
          __syncwarp();
        } else {
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            InT* dst = reinterpret_cast<InT*>(p.stage[owner]) + (static_cast<size_t>(li) * p.n + p.me) * kTileElems;
            bulk_store(dst + h * (kBM * 128) + quarter * 32 * 128, buf, kHalfSlabBytes);
            bulk_commit_group();
            if (tr) trace_ev(p.trace, ntr, 5, t * 2 + h);
            bulk_wait_group_1();                               // everything but the copy just issued has completed
            if (pend >= 0) mailbox_put(&mailbox, quarter, mb_tail, 0, pend);
            pend = (t << 3) | (quarter << 1) | h;
          }
        }
      }
      if (failed) break;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);            // the accumulator can be refilled from here on
    }
    if (failed) *abort_flag = 1;
    if (lane == 0) {
      bulk_wait_group0();
      if (pend >= 0) mailbox_put(&mailbox, quarter, mb_tail, 0, pend);
      __threadfence_block();
      atomicAdd(const_cast<int*>(&mailbox.finished), 1);
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
static void launch_fused(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tout, const FusedParams& p,
                         cudaStream_t stream) {
  auto kern = gemm_allreduce_kernel<AK, BK_, InT>;
  static bool configured = false;
  if (!configured) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kFusedSmemBytes));
    configured = true;
  }
  kern<<<p.num_gemm_ctas + p.num_comm_ctas, kFusedThreads, kFusedSmemBytes, stream>>>(ta, tb, tout, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// out (pre-allocated [M, N], same dtype as a) = all-reduce over the group of op(a) op(b), + bias.
// stage / result / flags: device pointers of every rank's workspace buffers, indexed by group rank.
static void fused_gemm_all_reduce(torch::Tensor a, torch::Tensor b, bool trans_a, bool trans_b,
                                  c10::optional<torch::Tensor> bias, torch::Tensor out, std::vector<int64_t> stage,
                                  std::vector<int64_t> result, std::vector<int64_t> flags, int64_t done_cap, int64_t me,
                                  int64_t epoch, int64_t num_comm_ctas, int64_t status_ptr,
                                  c10::optional<torch::Tensor> trace) {
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
  p.trace = (trace.has_value() && trace->defined()) ? reinterpret_cast<long long*>(trace->data_ptr<int64_t>()) : nullptr;
  const bool ak = !trans_a, bk = trans_b;
  CUtensorMap ta = ak ? make_tma_2d(a.data_ptr(), M, K, K, kBM) : make_tma_2d(a.data_ptr(), K, M, M, 64);
  CUtensorMap tb = bk ? make_tma_2d(b.data_ptr(), N, K, K, kFusedBN) : make_tma_2d(b.data_ptr(), K, N, N, 64);
  CUtensorMap tout = make_tma_2d_plain(out.data_ptr(), M, N, N, kFusedBN, kBM);
  auto stream = at::cuda::getCurrentCUDAStream();
#define FUSED_DISPATCH(T)                                                  \
  if (ak && bk) launch_fused<true, true, T>(ta, tb, tout, p, stream);            \
  else if (ak && !bk) launch_fused<true, false, T>(ta, tb, tout, p, stream);     \
  else if (!ak && bk) launch_fused<false, true, T>(ta, tb, tout, p, stream);     \
  else launch_fused<false, false, T>(ta, tb, tout, p, stream);
  if (p.is_bf16) { FUSED_DISPATCH(__nv_bfloat16) } else { FUSED_DISPATCH(__half) }
#undef FUSED_DISPATCH
}

void register_fused(py::module& m) { m.def("fused_gemm_all_reduce", &fused_gemm_all_reduce); }

}  // namespace cw
