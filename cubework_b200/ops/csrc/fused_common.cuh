// Pieces shared by the GEMM kernels that are fused with a collective over NVLink peer memory:
// system-scope flag accesses with bounded waits, bulk-copy wrappers, the staged tile layout and the
// batched flag publisher.
#pragma once
#include "gemm_sm100.cuh"

namespace cw {

constexpr int kFusedBN = 256;
constexpr int kMaxRanks = 8;
constexpr int kTileElems = kBM * kFusedBN;          // 16-bit elements per staged tile

constexpr int kTraceLen = 192;
__device__ __forceinline__ void trace_ev(long long* trace, int& n, int code, int tile) {
  if (trace != nullptr && n < kTraceLen) {
    long long* e = trace + (static_cast<size_t>(blockIdx.x) * kTraceLen + n) * 2;
    e[0] = (static_cast<long long>(code) << 32) | static_cast<unsigned>(tile);
    e[1] = static_cast<long long>(globaltimer_ns());
    ++n;
  }
}

__device__ __forceinline__ float tof(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float tof(__half v) { return __half2float(v); }
// 16-byte load that bypasses L1 (the data was written by another GPU, or by another SM of this one)
__device__ __forceinline__ uint4 ld_cg16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(int* p, int v) {
  asm volatile("st.relaxed.sys.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group_read_n() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
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

// Fused kernels run the six warps of the plain GEMM plus one publisher warp: the thread that publishes flags sits
// in system-scope fences for tens of microseconds at a time and must not share a warp with the TMA producer or
// the MMA issuer, whose instruction issue it would hold up.
constexpr int kFusedThreads = kGemmThreads + 32;
constexpr int kPublisherWarp = kGemmThreads / 32;
constexpr int kFusedStages = 4;
constexpr int kSlabBytes = 32 * kFusedBN * 2;                 // one epilogue warp's 32 rows of a tile (16 KB)
constexpr int kEpiBytes = 4 * 32 * 128 * 2;                    // 32 KB: one 32 x 128 half-slab per epilogue warp
constexpr int kPullSlots = 3;
constexpr int kTileBytes = kTileElems * 2;                     // 64 KB
constexpr int kFusedSmemBytes = kFusedStages * GemmCfg<kFusedBN>::kStageBytes + kEpiBytes + 256 + 1024;
static_assert(kFusedSmemBytes <= 227 * 1024, "fused kernel exceeds the shared memory of one SM");
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
__device__ __forceinline__ void bulk_wait_group_1() { asm volatile("cp.async.bulk.wait_group 1;" ::: "memory"); }
__device__ __forceinline__ void worker_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kWorkers) : "memory"); }

// Staged tile layout (staging slots, result buffer, pull slots): two column halves of [128 rows][128 cols], so
// the 32 rows x 128 columns that one epilogue warp produces per step are 8 KB of contiguous memory and travel as
// one bulk copy.  Inside a row the 16-byte chunk position is XOR-ed with the row so the row-per-lane shared-memory
// writes are bank-conflict free; readers apply the same mapping.  Returns the element offset of chunk j (0..31).
__device__ __forceinline__ int staged_off(int r, int j) {
  return (j >> 4) * (kBM * 128) + r * 128 + (((j & 15) ^ (r & 15)) << 3);
}
constexpr int kHalfSlabBytes = 32 * 128 * 2;                   // 8 KB: one warp, one column half

// ---- flag publication -------------------------------------------------------------------------------------
// A system-scope release towards another GPU costs tens of microseconds while the links are busy, far too much to
// pay on the epilogue's critical path once per copy.  Epilogue warps therefore only *record* completed copies in a
// per-warp mailbox in shared memory; one thread of a warp of its own collects
// whatever has accumulated, issues ONE system-scope fence and then writes all the corresponding flags.
constexpr int kMailboxDepth = 16;
struct Mailbox {
  volatile int item[4][kMailboxDepth];   // (tile << 3) | (quarter << 1) | half
  volatile int tail[4];                  // written by epilogue warp q
  volatile int head[4];                  // written by the publisher
  volatile int finished;                 // number of epilogue warps that have left their loop
};

__device__ __forceinline__ void mailbox_put(Mailbox* mb, int q, int& tail, int head_hint_unused, int value) {
  // the publisher may lag by one fence; wait (bounded) if the ring is full
  for (int spin = 0; tail - mb->head[q] >= kMailboxDepth && spin < (1 << 22); ++spin) __nanosleep(50);
  mb->item[q][tail % kMailboxDepth] = value;
  __threadfence_block();
  ++tail;
  mb->tail[q] = tail;
}


}  // namespace cw
