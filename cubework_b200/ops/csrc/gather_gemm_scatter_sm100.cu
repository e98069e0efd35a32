// All-gather -> GEMM -> reduce-scatter as ONE kernel per rank: the parallel matmul of the 2D (SUMMA) and 3D
// layouts, with both collectives moved into the tcgen05 GEMM and carried over NVLink peer memory.
//
//   out = reduce-scatter_s( op(gather_a(A)) * op(gather_b(B)) ) + bias
//
// Every part is optional: a gathered A and/or B (each over its own process group, concatenated along the
// rows or the columns of the stored shard), and a reduce-scatter of the product along its rows or columns
// over a third group.
//
// Grid = C communication CTAs + G GEMM CTAs, all co-resident (one CTA per SM).
//  * communication CTAs push this rank's shard, panel by panel (a panel = a block of stored rows), into the
//    gather buffer of every other rank of the operand's group with bulk copies global -> shared -> peer, and
//    publish one arrival flag per (destination, panel).  They wait for nobody.  The own shard is read in place
//    by the GEMM CTAs (it is copied into the own buffer only when TMA boxes could straddle two sources).
//  * GEMM CTAs run the persistent TMA -> tcgen05 -> TMEM pipeline.  The TMA producer reads a gathered
//    operand from the *local* gather buffer [sources][rows][cols]; before the first load of a tile it waits
//    for the flags of the (source, panel) pairs the tile reads (remembered in a shared-memory bitmap
//    afterwards), so tiles whose operands are local start at once.  The K loop starts at the k-blocks of the
//    local shard.
//  * with a reduce-scatter, tile ownership follows the output shard: every GEMM CTA first computes its share
//    of the tiles of other owners and sends the 16-bit partials into the owner's staging buffer (4 KB bulk
//    copies, flags batched behind one system-scope fence by a publisher thread), then its share of this
//    rank's tiles, to whose accumulators it adds the other ranks' partials in fp32 (+ bias) before storing
//    the output shard.
// Gather and staging buffers are used in two halves that alternate with the call epoch: a rank can run at
// most one call ahead of a peer (it needs that peer's data of the current call to finish), so the half
// written now was last read two calls ago.  Flags hold epochs that only grow.  Every wait is bounded and
// reports to the status word.  TMA tensor maps cover local memory only; peer memory is touched by bulk
// copies and plain stores.
//
// The reference runs these as separate NCCL collectives around cuBLAS GEMMs: q rounds of broadcast + addmm in
// cubework/module/parallel_2d/_operation.py:15-239, all_gather / matmul / reduce_scatter in
// cubework/module/parallel_3d/_operation.py:12-68.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/pybind11.h>
#include <torch/extension.h>

#include "fused_common.cuh"

namespace py = pybind11;

namespace cw {

// Thread layout of a GEMM CTA: warp 0 TMA producer, warp 1 MMA issuer, warps 2-9 epilogue (two per TMEM lane
// quarter, one per half of the tile's columns), warp 10 publisher of the flags of pushed partial tiles.
constexpr int kGgsEpiWarps = 8;
constexpr int kGgsThreads = 64 + 32 * kGgsEpiWarps + 32;
constexpr int kGgsPublisherWarp = 2 + kGgsEpiWarps;
constexpr int kGgsSmemBytes = kFusedStages * GemmCfg<kFusedBN>::kStageBytes + kGgsEpiWarps * kEpiBlockBytes + 256 + 1024;
static_assert(kGgsSmemBytes <= 227 * 1024, "gather/scatter kernel exceeds the shared memory of one SM");

// Staged partial tile (staging slots of the reduce-scatter): four column quarters of [128 rows][64 columns]; inside a
// quarter a row is 128 bytes and its 16-byte chunk j sits at chunk j ^ (row & 7).  The 32 rows x 64 columns that
// one epilogue warp produces per step are therefore 4 KB of contiguous memory in exactly the pattern of its
// shared-memory staging block, and travel as one bulk copy; readers apply the same mapping.
__device__ __forceinline__ int staged_off_v2(int r, int cq, int j) {      // element offset of chunk j (0..7)
  return cq * (kBM * 64) + r * 64 + ((j ^ (r & 7)) << 3);
}

struct Mailbox8 {
  volatile int item[kGgsEpiWarps][kMailboxDepth];   // (staging slot << 3) | (quarter << 1) | half
  volatile int tail[kGgsEpiWarps];                  // written by epilogue warp e
  volatile int head[kGgsEpiWarps];                  // written by the publisher
  volatile int finished;                            // number of epilogue warps that have left their loop
};
__device__ __forceinline__ void mailbox8_put(Mailbox8* mb, int e, int& tail, int value) {
  // the publisher may lag by one fence; wait (bounded) if the ring is full
  for (int spin = 0; tail - mb->head[e] >= kMailboxDepth && spin < (1 << 22); ++spin) __nanosleep(50);
  mb->item[e][tail % kMailboxDepth] = value;
  __threadfence_block();
  ++tail;
  mb->tail[e] = tail;
}

constexpr int kKnownWords = 64;            // 2048 (source, panel) arrival bits per operand
constexpr int kPiece = 32 * 1024;          // bytes per bulk copy of the gather pushers
constexpr int kPushSlots = 6;              // shared-memory pieces in flight per communication CTA
constexpr int kPendItems = 16;
constexpr int kPushInflight = 12;          // bulk stores a communication CTA keeps in flight before it waits
static_assert(kPushSlots * kPiece + 1024 + 256 <= kGgsSmemBytes, "push slots must fit the GEMM allocation");

struct GatherView {          // how the TMA producer sees one operand
  int live;                  // 0: an ordinary local tensor, nothing to wait for
  int n;                     // sources
  int g;                     // stored dimension along which the shards are concatenated (0 rows, 1 columns)
  int R, C;                  // extent of one stored shard
  int panel_rows, panels;    // one arrival flag per `panel_rows` stored rows of a source
  int epoch;
  int me;                    // this rank's position among the sources
  int own_direct;            // this rank's own shard is read from the tensor itself, not from the gather buffer
  const int* flags;          // local [n][panels]
};

struct GatherPush {          // what the communication CTAs do for one operand
  int live, n, me, panels, epoch;
  int dests;                 // destinations per panel: n, or n - 1 when the own shard is read in place
  long long shard_bytes, panel_bytes;
  const uint8_t* src;        // this rank's shard, dense [R][C] 16-bit
  uint8_t* dst[kMaxRanks];   // every rank's gather buffer (own included): [n][R][C]
  int* flags[kMaxRanks];     // every rank's flag array [n][panels]
};

struct GgsParams {
  int M, N, K;               // the product this rank computes: [M, K] x [K, N]
  int num_comm_ctas, num_gemm_ctas;
  int is_bf16;
  uint32_t mn_lbo, mn_sbo;
  int k_start;               // first k-block of the loop (the local shard's, when K is gathered)
  int b_first;               // push B's panels before A's
  GatherView va, vb;
  GatherPush pa, pb;
  int sc_dim;                // reduce-scatter of the product: -1 none, 0 rows, 1 columns
  int sn, sme, sepoch;
  int Ms, Ns;                // extent of one owner's part of the product
  int tiles_m, tiles_n;      // tile grid of one owner's part
  void* stage[kMaxRanks];    // [owned tiles][sn][128 x 256] 16-bit, this call's half
  int* sflags[kMaxRanks];    // [owned tiles][sn][8]
  void* out;                 // local [Ms or M][ldo]
  int ldo;
  const float* bias;         // optional, indexed by output column
  int tma_store;             // the output (and z_out) is written with TMA tile stores (16-byte aligned base and pitch)
  int act;                   // activation applied by the tile's owner after the bias (kActNone / Gelu / Relu)
  void* z_out;               // optional copy of the value before the activation, input dtype, same layout as `out`
  // Row-block order of a product whose A operand is gathered along its rows (and is not scattered): this rank's
  // own rows first, then panel by panel over the other sources in the order their pushes arrive.
  int m_remap, m_rps;        // enabled; row blocks per source
  long long* trace;          // optional [CTAs * 3][kGgsTraceLen][2] (event, globaltimer): performance debugging
  int* status;
};

// Event trace: three writers per CTA (0: TMA producer / push loader, 1: epilogue warp 0 / push storer, 2: MMA issuer).
constexpr int kGgsTraceLen = 512;
__device__ __forceinline__ void ggs_trace(long long* trace, int role, int& n, int code, int tile) {
  if (trace != nullptr && n < kGgsTraceLen) {
    long long* e = trace + ((static_cast<size_t>(blockIdx.x) * 3 + role) * kGgsTraceLen + n) * 2;
    e[0] = (static_cast<long long>(code) << 32) | static_cast<unsigned>(tile);
    e[1] = static_cast<long long>(globaltimer_ns());
    ++n;
  }
}

__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_group_n() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// Completed pushes waiting for their flag: written by the storing thread, drained by the publisher.
struct PushBox {
  int* volatile item[kPendItems * 2];
  volatile int tail, head, finished;
};

struct TileInfo {
  int row0, col0;     // position in the product
  int rows, cols;     // valid extent
  int orow, ocol;     // position in the local output
};

__device__ __forceinline__ TileInfo tile_info(const GgsParams& p, int owner, int li, int kb_total) {
  int tm, tn, kb0, kb1;
  decode_work(li, p.tiles_m * p.tiles_n, p.tiles_m, p.tiles_n, kb_total, 1, tm, tn, kb0, kb1);
  if (p.m_remap) {
    // logical position -> row block: [own source's blocks][block 0 of every other source][block 1 ...] ...
    // source s pushes to this rank in step (me - s - 1) mod n of each of its panel rounds
    const int n = p.va.n, me = p.va.me;
    if (tm < p.m_rps) {
      tm += me * p.m_rps;
    } else {
      const int q = tm - p.m_rps;
      const int pnl = fast_div(q, n - 1), si = q - pnl * (n - 1);
      int src = me + n - 1 - si;                      // in [me, me + n - 1]
      if (src >= n) src -= n;
      tm = src * p.m_rps + pnl;
    }
  }
  TileInfo t;
  t.orow = tm * kBM;
  t.ocol = tn * kFusedBN;
  t.row0 = (p.sc_dim == 0 ? owner * p.Ms : 0) + t.orow;
  t.col0 = (p.sc_dim == 1 ? owner * p.Ns : 0) + t.ocol;
  t.rows = min(kBM, p.Ms - t.orow);
  t.cols = min(kFusedBN, p.Ns - t.ocol);
  return t;
}

// The producer thread's record of what has arrived: one bit per (source, panel) in shared memory, and their count.
struct Known {
  uint32_t* bits;
  int count, total;
  __device__ __forceinline__ bool all() const { return count >= total; }
};

// rows [r0, r1) of source s must have arrived
__device__ __forceinline__ bool ensure_panels(const GatherView& v, Known& kn, int s, int r0, int r1, int* status) {
  uint32_t* known = kn.bits;
  if (r1 <= r0) return true;
  for (int pnl = r0 / v.panel_rows; pnl <= (r1 - 1) / v.panel_rows; ++pnl) {
    const int idx = s * v.panels + pnl;
    if ((known[idx >> 5] >> (idx & 31)) & 1u) continue;
    if (!wait_flag(v.flags + idx, v.epoch, status, idx)) return false;
    fence_proxy_async_all();                      // the TMA reads that follow must see what the flag announced
    known[idx >> 5] |= 1u << (idx & 31);
    ++kn.count;
  }
  return true;
}
// rows [y0, y1) of the concatenation along the rows (g == 0)
__device__ __forceinline__ bool ensure_stacked(const GatherView& v, Known& known, int y0, int y1, int* status) {
  y1 = min(y1, v.n * v.R);
  while (y0 < y1) {
    const int s = y0 / v.R, r = y0 - s * v.R;
    const int len = min(v.R - r, y1 - y0);
    if (!ensure_panels(v, known, s, r, r + len, status)) return false;
    y0 += len;
  }
  return true;
}

// ---- what the TMA producer needs to know about one operand for one tile ---------------------------------------
// All divisions happen once per tile; the k loop only adds and compares.  A box is 64 columns wide; along a
// column-wise concatenation it never straddles two sources (the host checks the divisibility that guarantees it).
//
// Arrival is checked per tile, before its first load: every (source, panel) the tile will read must have landed.
// (Tiles whose operands are entirely local therefore start at once; the others start when their panels are in.)
template <bool KMAJOR, int BOXES>
struct OperandTile {
  int x[BOXES], ybase[BOXES];      // MN-major: column and row offset of box g (row = ybase + k)
  bool local[BOXES];               // box g comes from this rank's own tensor
  int s, xin;                      // K-major, column-wise concatenation: source and column of the current k block
  int y;                           // K-major: row of the box (in the gather buffer, or in the own tensor if local[0])
};

__device__ __forceinline__ bool ensure_source(const GatherView& v, Known& known, int s, int r0, int r1, int* status) {
  if (s >= v.n || (v.own_direct && s == v.me)) return true;
  return ensure_panels(v, known, s, r0, r1, status);
}

// mn0 .. mn0 + len: the rows (A) or columns (B) of the product this tile covers
template <bool KMAJOR, int BOXES>
__device__ __forceinline__ bool begin_tile(const GatherView& v, Known& known, int mn0, int len, int kb_first,
                                           OperandTile<KMAJOR, BOXES>& t, int* status) {
  if (KMAJOR) {
    t.y = mn0; t.local[0] = false; t.s = 0; t.xin = kb_first * kBK;
    if (!v.live) return true;
    if (v.g == 0) {                                          // rows of the concatenation = MN
      if (v.own_direct && mn0 >= v.me * v.R && mn0 < (v.me + 1) * v.R) {
        t.y = mn0 - v.me * v.R;
        t.local[0] = true;
        return true;
      }
      return known.all() || ensure_stacked(v, known, mn0, mn0 + len, status);
    }
    t.s = t.xin / v.C;                                       // K is concatenated: every source, these rows
    t.xin -= t.s * v.C;
    for (int s = 0; s < v.n && !known.all(); ++s)
      if (!ensure_source(v, known, s, min(mn0, v.R), min(mn0 + len, v.R), status)) return false;
    return true;
  }
#pragma unroll
  for (int g = 0; g < BOXES; ++g) {
    t.x[g] = mn0 + g * 64; t.ybase[g] = 0; t.local[g] = false;
  }
  if (!v.live) return true;
  if (v.g == 0) {                                            // rows of the concatenation = K: everything is needed
    for (int s = 0; s < v.n && !known.all(); ++s)
      if (!ensure_source(v, known, s, 0, v.R, status)) return false;
    return true;
  }
#pragma unroll
  for (int g = 0; g < BOXES; ++g) {                          // MN is concatenated by columns: the sources of the boxes
    const int s = t.x[g] / v.C;
    if (s >= v.n) continue;                                  // beyond the operand: zero-filled
    t.x[g] -= s * v.C;
    if (v.own_direct && s == v.me) {
      t.local[g] = true;
    } else {
      t.ybase[g] = s * v.R;
      if (!known.all() && !ensure_panels(v, known, s, 0, v.R, status)) return false;
    }
  }
  return true;
}

// Coordinates of box g for k block `kb`; `local` tells which tensor map to use.
template <bool KMAJOR, int BOXES>
__device__ __forceinline__ void box_at(const GatherView& v, const OperandTile<KMAJOR, BOXES>& t, int g, int kb, int& x,
                                       int& y, bool& local) {
  if (KMAJOR) {
    x = kb * kBK; y = t.y; local = t.local[0];
    if (v.live && v.g == 1) {
      x = t.xin;
      local = v.own_direct && t.s == v.me;
      if (!local) y = t.s * v.R + t.y;
    }
    return;
  }
  x = t.x[g]; y = kb * kBK + t.ybase[g]; local = t.local[g];
  if (v.live && v.g == 0 && v.own_direct && y >= v.me * v.R && y < (v.me + 1) * v.R) {
    y -= v.me * v.R;
    local = true;
  }
}

// advance to the next k block (K-major operand whose K is concatenated: follow the source boundaries)
template <bool KMAJOR, int BOXES>
__device__ __forceinline__ void next_kb(const GatherView& v, OperandTile<KMAJOR, BOXES>& t, bool wrapped) {
  if (!KMAJOR || !v.live || v.g != 1) return;
  if (wrapped) { t.s = 0; t.xin = 0; return; }
  t.xin += kBK;
  if (t.xin >= v.C) { t.xin = 0; ++t.s; }
}

template <bool A_KMAJOR, bool B_KMAJOR, typename InT, bool OUT_F32>
__global__ void __launch_bounds__(kGgsThreads, 1)
gather_gemm_scatter_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                           const __grid_constant__ CUtensorMap tma_a_own, const __grid_constant__ CUtensorMap tma_b_own,
                           const __grid_constant__ CUtensorMap tma_out, const __grid_constant__ CUtensorMap tma_z,
                           const __grid_constant__ GgsParams p) {
  constexpr int BN = kFusedBN;
  using Cfg = GemmCfg<BN>;
  using OutT = typename OutType<InT, OUT_F32>::type;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kb_total = (p.K + kBK - 1) / kBK;
  const bool is_comm = static_cast<int>(blockIdx.x) < p.num_comm_ctas;
  if (p.trace != nullptr && threadIdx.x == 32 * 3 + 1) {      // entry stamp of the CTA
    int n0 = kGgsTraceLen - 2;
    ggs_trace(p.trace, 0, n0, 30, 0);
  }

  if (is_comm) {
    // =========================================================== communication CTA: push this rank's shards
    // three single threads: loader (global -> shared), storer (shared -> destination), publisher (flags)
    uint8_t* slots = smem;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kPushSlots * kPiece);
    uint64_t* empty_bar = full_bar + kPushSlots;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + kPushSlots);
    __shared__ PushBox box;
    if (threadIdx.x == 0) {
      for (int s = 0; s < kPushSlots; ++s) {
        mbar_init(&full_bar[s], 1);
        mbar_init(&empty_bar[s], 1);
      }
      *abort_flag = 0;
      box.tail = 0; box.head = 0; box.finished = 0;
      fence_barrier_init();
    }
    __syncthreads();
    if (warp > 2 || lane != 0) return;
    const int c = blockIdx.x;
    const GatherPush& first = p.b_first ? p.pb : p.pa;
    const GatherPush& second = p.b_first ? p.pa : p.pb;
    const int n_first = first.live ? first.panels * first.dests : 0;
    const int n_second = second.live ? second.panels * second.dests : 0;

    if (warp == 2) {
      // ---- publisher
      const unsigned long long t_start = globaltimer_ns();
      int head = 0;
      for (;;) {
        const int fin = box.finished;
        const int tail = box.tail;
        if (head == tail) {
          if (fin || *abort_flag) {
            if (head == box.tail) break;
            continue;
          }
          if (globaltimer_ns() - t_start > 4 * kWaitLimitNs) break;
          __nanosleep(100);
          continue;
        }
        __threadfence_block();
        __threadfence_system();
        for (; head < tail; ++head) {
          int* f = box.item[head % (kPendItems * 2)];
          const GatherPush& op = (reinterpret_cast<uintptr_t>(f) & 1) ? second : first;
          st_relaxed_sys(reinterpret_cast<int*>(reinterpret_cast<uintptr_t>(f) & ~uintptr_t(1)), op.epoch);
        }
        box.head = head;
      }
      return;
    }

    int slot = 0;
    uint32_t phase = 0;
    int seq = -1;                                   // storer: index of the bulk group committed last
    int box_tail = 0;
    bool ok = true;
    int ntr = 0;
    ggs_trace(p.trace, warp, ntr, 20, 0);
    // storer: panels whose last store has been committed but may still be in flight: (last group, flag) pairs
    constexpr int kDone = 8;
    int done_seq[kDone];
    int* done_flag[kDone];
    int done_head = 0, done_tail = 0;
    auto hand_over = [&](int upto) {               // flags of the panels whose stores are complete -> publisher
      while (done_head < done_tail && done_seq[done_head % kDone] <= upto) {
        for (int spin = 0; box_tail - box.head >= kPendItems * 2 && spin < (1 << 22); ++spin) __nanosleep(50);
        box.item[box_tail % (kPendItems * 2)] = done_flag[done_head % kDone];
        __threadfence_block();
        box.tail = ++box_tail;
        ++done_head;
      }
    };
    for (int i = c; i < n_first + n_second && ok; i += p.num_comm_ctas) {
      const bool is_second = i >= n_first;
      const GatherPush& op = is_second ? second : first;
      const int idx = is_second ? i - n_first : i;
      const int panel = idx / op.dests;
      const int dest = (op.me + (op.n - op.dests) + idx % op.dests) % op.n;
      const long long off0 = static_cast<long long>(panel) * op.panel_bytes;
      const long long bytes = min(op.panel_bytes, op.shard_bytes - off0);
      const uint8_t* src = op.src + off0;
      uint8_t* dst = op.dst[dest] + static_cast<long long>(op.me) * op.shard_bytes + off0;
      for (long long off = 0; off < bytes; off += kPiece) {
        const uint32_t len = static_cast<uint32_t>(min(static_cast<long long>(kPiece), bytes - off));
        if (warp == 0) {
          if (!mbar_wait(&empty_bar[slot], phase ^ 1, abort_flag, p.status, kErrEmptyBarrierTimeout, i)) { ok = false; break; }
          mbar_expect_tx(&full_bar[slot], len);
          bulk_load(slots + slot * kPiece, src + off, len, &full_bar[slot]);
        } else {
          if (!mbar_wait(&full_bar[slot], phase, abort_flag, p.status, kErrFullBarrierTimeout, i)) { ok = false; break; }
          bulk_store(dst + off, slots + slot * kPiece, len);
          bulk_commit_group();
          ++seq;
          bulk_wait_group_read_n<2>();              // groups <= seq-2 no longer read their slot: hand it back
          if (seq >= 2) mbar_arrive(&empty_bar[(slot + kPushSlots - 2) % kPushSlots]);
          bulk_wait_group_n<kPushInflight>();       // groups <= seq-kPushInflight have landed at their destination
          hand_over(seq - kPushInflight);
        }
        if (++slot == kPushSlots) { slot = 0; phase ^= 1; }
      }
      if (warp == 1 && ok) {
        // every store of the panel is committed; its flag goes to the publisher once they have landed, which the
        // stores of the following panels reveal (no drain of the pipeline per panel)
        if (done_tail - done_head == kDone) {
          ggs_trace(p.trace, 1, ntr, 21, i);
          bulk_wait_group0();
          ggs_trace(p.trace, 1, ntr, 22, i);
          hand_over(seq);
        }
        int* f = op.flags[dest] + op.me * op.panels + panel;
        done_seq[done_tail % kDone] = seq;
        done_flag[done_tail % kDone] = reinterpret_cast<int*>(reinterpret_cast<uintptr_t>(f) | (is_second ? 1u : 0u));
        ++done_tail;
      }
    }
    if (warp == 1) {
      bulk_wait_group0();
      hand_over(seq);
      ggs_trace(p.trace, 1, ntr, 22, 0);
      __threadfence_block();
      box.finished = 1;
    }
    return;
  }

  // ================================================================= GEMM CTA
  uint8_t* epi = smem + kFusedStages * Cfg::kStageBytes;         // 8 staging blocks of 4 KB, 1024-byte aligned
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(epi + kGgsEpiWarps * kEpiBlockBytes);
  uint64_t* empty_bar = full_bar + kFusedStages;
  uint64_t* tfull_bar = empty_bar + kFusedStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  __shared__ Mailbox8 mailbox;
  __shared__ uint32_t known_a[kKnownWords], known_b[kKnownWords];
  if (threadIdx.x == 0) {
    for (int s = 0; s < kFusedStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], kGgsEpiWarps);
    }
    *abort_flag = 0;
    for (int q = 0; q < kGgsEpiWarps; ++q) { mailbox.tail[q] = 0; mailbox.head[q] = 0; }
    mailbox.finished = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
    tma_prefetch_desc(&tma_a_own);
    tma_prefetch_desc(&tma_b_own);
    if (p.tma_store) {
      tma_prefetch_desc(&tma_out);
      if (p.z_out != nullptr) tma_prefetch_desc(&tma_z);
    }
  }
  if (threadIdx.x >= 32 && threadIdx.x < 32 + kKnownWords) {
    known_a[threadIdx.x - 32] = 0;
    known_b[threadIdx.x - 32] = 0;
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // role of this CTA and its tile list
  const bool scat = p.sc_dim >= 0;
  const int G = p.num_gemm_ctas;
  const int bid = blockIdx.x - p.num_comm_ctas;
  const int tpo = p.tiles_m * p.tiles_n;                     // tiles per owner
  // Tile order of a GEMM CTA under a reduce-scatter.  Tiles of other owners ("push": the partial leaves for its
  // owner) and this rank's own tiles (the peers' partials are added) are interleaved: pushes keep the links busy
  // from the first to the last tile while the own tiles' arithmetic and stores run in their shadow.  An own tile is
  // taken only when this CTA is kLead pushes past the point where, by symmetry, the peers pushed their partials of
  // that tile, so its flags are normally up when it looks (and waits cannot chain: every wait is for a push that
  // was issued strictly earlier in the common order).  Without a reduce-scatter every tile is an own tile.
  constexpr int kLead = 3;
  const int n_push_items = scat ? tpo * (p.sn - 1) : 0;
  const int np = bid < n_push_items ? (n_push_items - bid + G - 1) / G : 0;    // pushes of this CTA
  const int own0 = (bid + G - n_push_items % G) % G;                            // round robin continues after the pushes
  const int no = own0 < tpo ? (tpo - own0 + G - 1) / G : 0;                     // own tiles of this CTA
  struct Sched { int ip, io; };
  bool push_tile = false;
  auto next_tile = [&](Sched& sc, int& owner, int& li) -> bool {              // false: finished; sets push_tile
    if (sc.ip < np && (sc.io >= no || sc.ip < (sc.io + 1) * (p.sn - 1) + kLead)) {
      const int v = bid + sc.ip * G;
      ++sc.ip;
      push_tile = true;
      li = fast_div(v, p.sn - 1);
      owner = p.sme + 1 + (v - li * (p.sn - 1));    // in [sme + 1, sme + sn - 1]
      if (owner >= p.sn) owner -= p.sn;
      return true;
    }
    if (sc.io >= no) return false;
    push_tile = false;
    li = own0 + sc.io * G;
    ++sc.io;
    owner = scat ? p.sme : 0;
    return true;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int owner, li;
      Known ka{known_a, 0, p.va.live ? (p.va.n - p.va.own_direct) * p.va.panels : 0};
      Known kb_{known_b, 0, p.vb.live ? (p.vb.n - p.vb.own_direct) * p.vb.panels : 0};
      int ntr = 0;
      Sched sched{0, 0};
      while (!*abort_flag && next_tile(sched, owner, li)) {
        const TileInfo ti = tile_info(p, owner, li, kb_total);
        OperandTile<A_KMAJOR, kBM / 64> ta;
        OperandTile<B_KMAJOR, BN / 64> tb;
        ggs_trace(p.trace, 0, ntr, 1, li);
        bool ok = begin_tile(p.va, ka, ti.row0, kBM, p.k_start, ta, p.status) &&
                  begin_tile(p.vb, kb_, ti.col0, BN, p.k_start, tb, p.status);
        ggs_trace(p.trace, 0, ntr, 2, li);
        if (!ok) { *abort_flag = 1; break; }
        int kb = p.k_start;
        for (int kbi = 0; kbi < kb_total; ++kbi) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kErrEmptyBarrierTimeout, li)) { ok = false; break; }
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kABytes;
          mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          int x, y;
          bool local;
#pragma unroll
          for (int g = 0; g < (A_KMAJOR ? 1 : kBM / 64); ++g) {
            box_at(p.va, ta, g, kb, x, y, local);
            tma_load_2d(sa + g * 8192, local ? &tma_a_own : &tma_a, &full_bar[stage], x, y);
          }
#pragma unroll
          for (int g = 0; g < (B_KMAJOR ? 1 : BN / 64); ++g) {
            box_at(p.vb, tb, g, kb, x, y, local);
            tma_load_2d(sb + g * 8192, local ? &tma_b_own : &tma_b, &full_bar[stage], x, y);
          }
          const bool wrapped = ++kb == kb_total;
          if (wrapped) kb = 0;
          next_kb(p.va, ta, wrapped);
          next_kb(p.vb, tb, wrapped);
          if (++stage == kFusedStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(kBM, BN, !A_KMAJOR, !B_KMAJOR, p.is_bf16);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      int owner, li;
      int ntr = 0;
      Sched sched{0, 0};
      while (!*abort_flag && next_tile(sched, owner, li)) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ++it;
        ggs_trace(p.trace, 2, ntr, 10, li);
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status, kErrTmemEmptyTimeout, li)) break;
        ggs_trace(p.trace, 2, ntr, 11, li);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kErrFullBarrierTimeout, li)) { ok = false; break; }
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
        ggs_trace(p.trace, 2, ntr, 12, li);
      }
    }
  } else if (warp == kGgsPublisherWarp) {
    if (lane == 0 && scat) {
      // ---- publisher of the partial tiles this CTA pushed: one system-scope fence per batch, then the flags
      int head[kGgsEpiWarps];
      for (int q = 0; q < kGgsEpiWarps; ++q) head[q] = 0;
      const unsigned long long t_start = globaltimer_ns();
      for (;;) {
        int batch[32];
        int nb = 0;
        const int fin = mailbox.finished;
        for (int q = 0; q < kGgsEpiWarps; ++q) {
          const int tail = mailbox.tail[q];
          while (head[q] < tail && nb < 32) {
            batch[nb++] = mailbox.item[q][head[q] % kMailboxDepth];
            ++head[q];
          }
          mailbox.head[q] = head[q];
        }
        if (nb == 0) {
          if (fin == kGgsEpiWarps || *abort_flag) {
            bool drained = true;
            for (int q = 0; q < kGgsEpiWarps; ++q) drained = drained && head[q] == mailbox.tail[q];
            if (drained) break;
            continue;
          }
          if (globaltimer_ns() - t_start > 4 * kWaitLimitNs) break;
          __nanosleep(100);
          continue;
        }
        __threadfence_block();
        __threadfence_system();
        for (int b = 0; b < nb; ++b) {
          const int slot_id = batch[b] >> 3, qh = batch[b] & 7;
          const int owner = slot_id % p.sn, li = slot_id / p.sn;
          st_relaxed_sys(p.sflags[owner] + (static_cast<size_t>(li) * p.sn + p.sme) * 8 + qh, p.sepoch);
        }
      }
    }
  } else {
    // ---- epilogue: 8 warps; warp (quarter, half) owns 32 accumulator rows x 128 columns of every tile and walks
    //      them in two steps of 64 columns.
    //  push role: 16-bit partial -> 4 KB staging block -> one bulk copy into the owner's staging slot
    //  own role : (wait for and add the other ranks' partials) + bias (+ activation) -> staging block -> TMA tile
    //             store into the output (direct stores when the output's row pitch is not a multiple of 16 bytes)
    const int ew = warp - 2;
    const int quarter = warp & 3;            // TMEM lanes [32*quarter, +32): fixed by the hardware per warp
    const int half = ew >> 2;
    uint8_t* sbuf = epi + ew * kEpiBlockBytes;
    OutT* out = reinterpret_cast<OutT*>(p.out);
    int pend = -1;
    int mb_tail = 0;
    int it = 0;
    bool failed = false;
    int owner, li;
    int ntr = 0;
    const bool tr = ew == 0 && lane == 0;
    const int r = quarter * 32 + lane;
    Sched sched{0, 0};
    int gseq = 0, pend_seq = 0;            // lane 0: bulk groups committed so far; value after the pending push's last
    while (!*abort_flag && !failed && next_tile(sched, owner, li)) {
      const TileInfo ti = tile_info(p, owner, li, kb_total);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ++it;
      if (tr) ggs_trace(p.trace, 1, ntr, 3, li);
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, kErrTmemFullTimeout, li)) break;
      if (tr) ggs_trace(p.trace, 1, ntr, 4, li);
      tc_fence_after();
      const bool mine = !push_tile;
      if (mine && scat && sched.ip >= np && pend >= 0) {
        // no push will follow: the last pushed tile must not wait for a later tile to be announced (its owner
        // may need it for the very tile this CTA is about to wait on, and vice versa)
        if (lane == 0) {
          bulk_wait_group0();
          mailbox8_put(&mailbox, ew, mb_tail, pend);
        }
        pend = -1;
      }
      const bool half_live = half * 128 < ti.cols;             // warp-uniform
      const InT* stage = reinterpret_cast<const InT*>(p.stage[scat ? p.sme : 0]) + static_cast<size_t>(li) * p.sn * kTileElems;
      if (mine && scat && half_live) {
        bool ok = true;
        if (lane < p.sn && lane != p.sme)
          ok = wait_flag(p.sflags[p.sme] + (static_cast<size_t>(li) * p.sn + lane) * 8 + quarter * 2 + half, p.sepoch,
                         p.status, li);
        if (__any_sync(0xffffffffu, !ok)) { failed = true; break; }
        if (tr) ggs_trace(p.trace, 1, ntr, 5, li);
      }
      __syncwarp();
      const uint32_t t_addr = tmem_base + acc * BN + half * 128 + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
      for (int i = 0; i < 2; ++i) {
        const int cq = half * 2 + i;
        const int c0 = cq * 64;
        float v[64];
        {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(t_addr + i * 64, r0);
          tmem_ld_32x32(t_addr + i * 64 + 32, r1);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) { v[j] = __uint_as_float(r0[j]); v[32 + j] = __uint_as_float(r1[j]); }
        }
        if (i == 1) {
          // this warp has read all its columns: the MMA warp may reuse the accumulator
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty_bar[acc]);
        }
        const bool live = c0 < ti.cols;                          // warp-uniform
        if (!mine) {
          // ---- push: this step's 32 x 64 block of the partial tile goes to its owner (always one bulk group per
          // step, empty for dead columns, so that "all but the latest two groups" means "the previous tile")
          if (live) {
            if (lane == 0) bulk_wait_group_read0();              // the previous copy has finished reading sbuf
            __syncwarp();
            stage_row_16bit<InT>(sbuf, lane, v);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
              InT* dst = reinterpret_cast<InT*>(p.stage[owner]) + (static_cast<size_t>(li) * p.sn + p.sme) * kTileElems;
              bulk_store(dst + cq * (kBM * 64) + quarter * (32 * 64), sbuf, kEpiBlockBytes);
            }
          }
          if (lane == 0) { bulk_commit_group(); ++gseq; }
          continue;
        }
        if (!live) continue;
        if (scat) {
          // the peers' partials: the loads of the next source are in flight while the current one is added
          uint4 pa[8], pb[8];
          auto next_src = [&](int s) { ++s; return s == p.sme ? s + 1 : s; };
          auto fetch = [&](uint4 (&dst)[8], int s) {
#pragma unroll
            for (int j = 0; j < 8; ++j) dst[j] = ld_cg16(stage + static_cast<size_t>(s) * kTileElems + staged_off_v2(r, cq, j));
          };
          auto add = [&](const uint4 (&srcv)[8]) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const InT* hh = reinterpret_cast<const InT*>(&srcv[j]);
#pragma unroll
              for (int e = 0; e < 8; ++e) v[j * 8 + e] += tof(hh[e]);
            }
          };
          int s0 = next_src(-1);
          fetch(pa, s0);
          for (;;) {
            const int s1 = next_src(s0);
            if (s1 < p.sn) fetch(pb, s1);
            add(pa);
            if (s1 >= p.sn) break;
            s0 = next_src(s1);
            if (s0 < p.sn) fetch(pa, s0);
            add(pb);
            if (s0 >= p.sn) break;
          }
        }
        if (p.bias != nullptr) {
#pragma unroll
          for (int j = 0; j < 64; ++j) v[j] += (c0 + j < ti.cols) ? __ldg(p.bias + ti.ocol + c0 + j) : 0.f;
        }
        const int gx = ti.ocol + c0, gy = ti.orow + quarter * 32;
        if (p.tma_store) {
          if (p.z_out != nullptr) {
            if (lane == 0) bulk_wait_group_read0();
            __syncwarp();
            stage_row_16bit<InT>(sbuf, lane, v);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) { tma_store_2d(&tma_z, sbuf, gx, gy); bulk_commit_group(); ++gseq; }
          }
          if (p.act == kActGelu) {
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] = gelu_fast(v[j]);
          } else if (p.act == kActRelu) {
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] = fmaxf(v[j], 0.f);
          }
          if constexpr (OUT_F32) {
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              if (c0 + hh * 32 >= ti.cols) break;
              float w32[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) w32[j] = v[hh * 32 + j];
              if (lane == 0) bulk_wait_group_read0();
              __syncwarp();
              stage_row_f32(sbuf, lane, w32);
              fence_proxy_async();
              __syncwarp();
              if (lane == 0) { tma_store_2d(&tma_out, sbuf, gx + hh * 32, gy); bulk_commit_group(); ++gseq; }
            }
          } else {
            if (lane == 0) bulk_wait_group_read0();
            __syncwarp();
            stage_row_16bit<InT>(sbuf, lane, v);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) { tma_store_2d(&tma_out, sbuf, gx, gy); bulk_commit_group(); ++gseq; }
          }
        } else if (r < ti.rows) {
          const size_t o = static_cast<size_t>(ti.orow + r) * p.ldo + gx;
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            if (c0 + hh * 32 >= ti.cols) break;
            float w32[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) w32[j] = v[hh * 32 + j];
            if (p.z_out != nullptr)
              store_row<InT>(reinterpret_cast<InT*>(p.z_out) + o + hh * 32, w32, false, ti.cols - c0 - hh * 32);
            if (p.act == kActGelu) {
#pragma unroll
              for (int j = 0; j < 32; ++j) w32[j] = gelu_fast(w32[j]);
            } else if (p.act == kActRelu) {
#pragma unroll
              for (int j = 0; j < 32; ++j) w32[j] = fmaxf(w32[j], 0.f);
            }
            store_row(out + o + hh * 32, w32, false, ti.cols - c0 - hh * 32);
          }
        }
      }
      if (lane == 0) {
        // a pushed tile is announced once its copies have landed, which is known without draining the pipeline as
        // soon as this warp has committed two more groups: "all but the latest two have completed"
        if (pend >= 0 && gseq - pend_seq >= 2) {
          bulk_wait_group_n<2>();
          mailbox8_put(&mailbox, ew, mb_tail, pend);
          pend = -1;
        }
        if (!mine) {
          if (pend >= 0) {                 // (only when a tile committed fewer than two groups in between)
            bulk_wait_group_n<2>();
            mailbox8_put(&mailbox, ew, mb_tail, pend);
          }
          pend = half_live ? (((li * p.sn + owner) << 3) | (quarter << 1) | half) : -1;
          pend_seq = gseq;
        }
      }
      if (tr) ggs_trace(p.trace, 1, ntr, 6, li);
    }
    if (failed) *abort_flag = 1;
    if (lane == 0) {
      bulk_wait_group0();
      if (pend >= 0) mailbox8_put(&mailbox, ew, mb_tail, pend);
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
  if (p.trace != nullptr && threadIdx.x == 32 * 3 + 1) {
    int n1 = kGgsTraceLen - 1;
    ggs_trace(p.trace, 0, n1, 31, 0);
  }
}

template <bool AK, bool BK_, typename InT, bool F32>
static void launch_ggs(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tao, const CUtensorMap& tbo,
                       const CUtensorMap& to, const CUtensorMap& tz, const GgsParams& p, cudaStream_t stream) {
  auto kern = gather_gemm_scatter_kernel<AK, BK_, InT, F32>;
  static bool configured = false;
  if (!configured) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kGgsSmemBytes));
    configured = true;
  }
  // Co-residency: GEMM CTAs spin (bounded) on flags that the communication CTAs of the peers' launches write, and
  // the peers' GEMM CTAs on this launch's.  The grid is exactly one CTA per SM and every CTA takes the SM's whole
  // shared memory, so all CTAs are resident at once as long as no other kernel holds SMs while this one starts; a
  // concurrent kernel on another stream turns into a stall that the bounded waits report through the status word.
  kern<<<p.num_gemm_ctas + p.num_comm_ctas, kGgsThreads, kGgsSmemBytes, stream>>>(ta, tb, tao, tbo, to, tz, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

template <typename InT, bool F32>
static void dispatch_ggs(bool ak, bool bk, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tao,
                         const CUtensorMap& tbo, const CUtensorMap& to, const CUtensorMap& tz, const GgsParams& p,
                         cudaStream_t stream) {
  if (ak && bk) launch_ggs<true, true, InT, F32>(ta, tb, tao, tbo, to, tz, p, stream);
  else if (ak && !bk) launch_ggs<true, false, InT, F32>(ta, tb, tao, tbo, to, tz, p, stream);
  else if (!ak && bk) launch_ggs<false, true, InT, F32>(ta, tb, tao, tbo, to, tz, p, stream);
  else launch_ggs<false, false, InT, F32>(ta, tb, tao, tbo, to, tz, p, stream);
}

// One operand's gather, as the host describes it: cfg = [] (not gathered) or [n, me, g, panel_rows, epoch];
// bufs / flags = every rank's gather buffer (this call's half) and flag array, indexed by group rank.
static void fill_gather(const torch::Tensor& t, const std::vector<int64_t>& cfg, const std::vector<int64_t>& bufs,
                        const std::vector<int64_t>& flags, GatherView& v, GatherPush& q) {
  v = GatherView{};
  q = GatherPush{};
  if (cfg.empty()) return;
  TORCH_CHECK(cfg.size() == 5 && bufs.size() == static_cast<size_t>(cfg[0]) && flags.size() == bufs.size());
  const int n = static_cast<int>(cfg[0]), me = static_cast<int>(cfg[1]);
  TORCH_CHECK(n >= 2 && n <= kMaxRanks && me >= 0 && me < n);
  v.live = 1; v.n = n; v.g = static_cast<int>(cfg[2]);
  v.R = static_cast<int>(t.size(0)); v.C = static_cast<int>(t.size(1));
  v.panel_rows = static_cast<int>(cfg[3]);
  v.panels = (v.R + v.panel_rows - 1) / v.panel_rows;
  v.epoch = static_cast<int>(cfg[4]);
  v.me = me;
  v.own_direct = 0;
  v.flags = reinterpret_cast<const int*>(flags[me]);
  TORCH_CHECK(v.C % 8 == 0 && n * v.panels <= kKnownWords * 32, "gathered operand: bad shard shape or too many panels");
  TORCH_CHECK(v.g == 0 || v.C % 64 == 0, "column-wise gather needs shard columns in multiples of 64");
  q.live = 1; q.n = n; q.me = me; q.panels = v.panels; q.epoch = v.epoch; q.dests = n;
  q.shard_bytes = static_cast<long long>(v.R) * v.C * 2;
  q.panel_bytes = static_cast<long long>(v.panel_rows) * v.C * 2;
  q.src = reinterpret_cast<const uint8_t*>(t.data_ptr());
  TORCH_CHECK((reinterpret_cast<uintptr_t>(q.src) & 15) == 0, "gathered operand must be 16-byte aligned");
  for (int i = 0; i < n; ++i) {
    q.dst[i] = reinterpret_cast<uint8_t*>(bufs[i]);
    q.flags[i] = reinterpret_cast<int*>(flags[i]);
  }
}

// out = reduce-scatter( op(gather(a)) op(gather(b)) ) + bias; see the head of this file.  `a`, `b` are this rank's
// stored shards; `out` is pre-allocated with the shape of this rank's part of the product (fp32 or the input type).
// sc = [] or [dim, n, me, epoch] with every rank's staging buffer (this call's half) and flag array.
static void gather_gemm_scatter(torch::Tensor a, torch::Tensor b, bool trans_a, bool trans_b,
                                c10::optional<torch::Tensor> bias, torch::Tensor out, std::vector<int64_t> ga,
                                std::vector<int64_t> ga_bufs, std::vector<int64_t> ga_flags, std::vector<int64_t> gb,
                                std::vector<int64_t> gb_bufs, std::vector<int64_t> gb_flags, std::vector<int64_t> sc,
                                std::vector<int64_t> sc_stage, std::vector<int64_t> sc_flags, int64_t num_comm_ctas,
                                int64_t status_ptr, int64_t act, c10::optional<torch::Tensor> z_out,
                                c10::optional<torch::Tensor> trace) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.dim() == 2 && b.dim() == 2 && a.is_contiguous() && b.is_contiguous());
  TORCH_CHECK(a.scalar_type() == b.scalar_type() && out.is_contiguous() && out.dim() == 2);
  TORCH_CHECK(a.scalar_type() == torch::kBFloat16 || a.scalar_type() == torch::kFloat16);
  const bool f32 = out.scalar_type() == torch::kFloat32;
  TORCH_CHECK(f32 || out.scalar_type() == a.scalar_type());
  c10::cuda::CUDAGuard guard(a.device());
  GgsParams p{};
  fill_gather(a, ga, ga_bufs, ga_flags, p.va, p.pa);
  fill_gather(b, gb, gb_bufs, gb_flags, p.vb, p.pb);
  // full stored extents
  const int64_t a_rows = a.size(0) * (p.va.live && p.va.g == 0 ? p.va.n : 1);
  const int64_t a_cols = a.size(1) * (p.va.live && p.va.g == 1 ? p.va.n : 1);
  const int64_t b_rows = b.size(0) * (p.vb.live && p.vb.g == 0 ? p.vb.n : 1);
  const int64_t b_cols = b.size(1) * (p.vb.live && p.vb.g == 1 ? p.vb.n : 1);
  const int M = static_cast<int>(trans_a ? a_cols : a_rows);
  const int K = static_cast<int>(trans_a ? a_rows : a_cols);
  const int N = static_cast<int>(trans_b ? b_rows : b_cols);
  TORCH_CHECK((trans_b ? b_cols : b_rows) == K, "inner dimensions differ");
  const bool ak = !trans_a, bk = trans_b;
  // a gathered operand whose rows are the K dimension is concatenated without padding: K blocks may straddle
  // sources only when the concatenation is along the rows (it is then contiguous); a column-wise concatenation of
  // an MN-major operand would read the next source's rows past the end of K
  if (p.va.live && p.va.g == 1 && !ak) TORCH_CHECK(p.va.R % kBK == 0, "A: K rows of a column-gathered operand must be a multiple of 64");
  if (p.vb.live && p.vb.g == 1 && !bk) TORCH_CHECK(p.vb.R % kBK == 0, "B: K rows of a column-gathered operand must be a multiple of 64");
  p.M = M; p.N = N; p.K = K;
  p.is_bf16 = a.scalar_type() == torch::kBFloat16;
  p.mn_lbo = 8192; p.mn_sbo = 1024;
  p.sc_dim = -1; p.sn = 1; p.sme = 0; p.Ms = M; p.Ns = N;
  if (!sc.empty()) {
    TORCH_CHECK(sc.size() == 4 && sc_stage.size() == static_cast<size_t>(sc[1]) && sc_flags.size() == sc_stage.size());
    p.sc_dim = static_cast<int>(sc[0]); p.sn = static_cast<int>(sc[1]); p.sme = static_cast<int>(sc[2]);
    p.sepoch = static_cast<int>(sc[3]);
    TORCH_CHECK(p.sn >= 2 && p.sn <= kMaxRanks && (p.sc_dim == 0 || p.sc_dim == 1));
    if (p.sc_dim == 0) { TORCH_CHECK(M % p.sn == 0); p.Ms = M / p.sn; }
    else { TORCH_CHECK(N % p.sn == 0 && (N / p.sn) % 8 == 0); p.Ns = N / p.sn; }
    for (int i = 0; i < p.sn; ++i) {
      p.stage[i] = reinterpret_cast<void*>(sc_stage[i]);
      p.sflags[i] = reinterpret_cast<int*>(sc_flags[i]);
    }
    // boxes of a column-gathered MN-major operand must stay inside one source for every owner's tiles
    if (p.sc_dim == 0 && !ak) TORCH_CHECK(p.Ms % 8 == 0, "row shards of an MN-major A must start on 16-byte boundaries");
    if (p.sc_dim == 0 && p.va.live && p.va.g == 1 && !ak) TORCH_CHECK(p.Ms % 64 == 0);
    if (p.sc_dim == 1 && p.vb.live && p.vb.g == 1 && bk == false) TORCH_CHECK(p.Ns % 64 == 0);
  }
  TORCH_CHECK(out.size(0) == p.Ms && out.size(1) == p.Ns, "output must have the shape of this rank's part");
  // The own shard is read in place (and not copied into the own gather buffer) whenever no TMA box can cover rows
  // of two sources: always for a column-wise concatenation; for a row-wise one when the shard extent and every
  // box origin are multiples of the box height.
  if (p.va.live) {
    const int h = ak ? kBM : kBK;
    const bool origins = !ak || p.sc_dim != 0 || p.Ms % kBM == 0;
    p.va.own_direct = (p.va.g == 1 || (p.va.R % h == 0 && origins)) ? 1 : 0;
    if (p.va.own_direct) p.pa.dests = p.pa.n - 1;
  }
  if (p.vb.live) {
    const int h = bk ? kFusedBN : kBK;
    const bool origins = !bk || p.sc_dim != 1 || p.Ns % kFusedBN == 0;
    p.vb.own_direct = (p.vb.g == 1 || (p.vb.R % h == 0 && origins)) ? 1 : 0;
    if (p.vb.own_direct) p.pb.dests = p.pb.n - 1;
  }
  p.tiles_m = (p.Ms + kBM - 1) / kBM;
  p.tiles_n = (p.Ns + kFusedBN - 1) / kFusedBN;
  p.out = out.data_ptr();
  p.ldo = static_cast<int>(out.size(1));
  torch::Tensor bias_f;
  if (bias.has_value() && bias->defined()) {
    bias_f = bias->to(torch::kFloat32).contiguous();
    TORCH_CHECK(bias_f.numel() == p.Ns);
    p.bias = bias_f.data_ptr<float>();
  }
  p.status = reinterpret_cast<int*>(status_ptr);
  p.act = static_cast<int>(act);
  p.z_out = nullptr;
  if (z_out.has_value() && z_out->defined()) {
    TORCH_CHECK(z_out->scalar_type() == a.scalar_type() && z_out->is_contiguous() && z_out->sizes() == out.sizes(),
                "pre-activation output must match the output's shape and the operands' dtype");
    p.z_out = z_out->data_ptr();
  }
  p.trace = nullptr;
  if (trace.has_value() && trace->defined()) {
    TORCH_CHECK(trace->scalar_type() == torch::kInt64 && trace->is_contiguous() &&
                trace->numel() >= static_cast<int64_t>(at::cuda::getCurrentDeviceProperties()->multiProcessorCount) * 3 *
                                      kGgsTraceLen * 2, "trace tensor too small");
    p.trace = reinterpret_cast<long long*>(trace->data_ptr<int64_t>());
  }
  p.m_remap = 0; p.m_rps = 0;
  if (p.va.live && p.va.g == 0 && ak && p.sc_dim < 0 && p.va.own_direct && p.va.panel_rows == kBM &&
      p.va.R % kBM == 0) {
    p.m_remap = 1;
    p.m_rps = p.va.R / kBM;
  }
  // start the K loop at the local shard when K is the gathered dimension
  const int kb_total = (K + kBK - 1) / kBK;
  p.k_start = 0;
  if (p.va.live && ((ak && p.va.g == 1) || (!ak && p.va.g == 0)))
    p.k_start = static_cast<int>(static_cast<int64_t>(p.pa.me) * (K / p.va.n) / kBK);
  else if (p.vb.live && ((bk && p.vb.g == 1) || (!bk && p.vb.g == 0)))
    p.k_start = static_cast<int>(static_cast<int64_t>(p.pb.me) * (K / p.vb.n) / kBK);
  p.k_start = std::min(p.k_start, kb_total - 1);
  p.b_first = (p.pb.live && (!p.pa.live || p.pb.shard_bytes < p.pa.shard_bytes)) ? 1 : 0;
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  p.num_comm_ctas = (p.pa.live || p.pb.live) ? std::max(1, std::min(static_cast<int>(num_comm_ctas), sms / 2)) : 0;
  p.num_gemm_ctas = sms - p.num_comm_ctas;
  TORCH_CHECK(p.num_gemm_ctas >= 2);

  const void* a_ptr = p.va.live ? reinterpret_cast<const void*>(ga_bufs[p.pa.me]) : a.data_ptr();
  const void* b_ptr = p.vb.live ? reinterpret_cast<const void*>(gb_bufs[p.pb.me]) : b.data_ptr();
  const uint64_t ar = p.va.live ? static_cast<uint64_t>(p.va.n) * a.size(0) : a.size(0);
  const uint64_t br = p.vb.live ? static_cast<uint64_t>(p.vb.n) * b.size(0) : b.size(0);
  CUtensorMap ta = make_tma_2d(a_ptr, ar, a.size(1), a.size(1), ak ? kBM : 64);
  CUtensorMap tb = make_tma_2d(b_ptr, br, b.size(1), b.size(1), bk ? kFusedBN : 64);
  CUtensorMap tao = make_tma_2d(a.data_ptr(), a.size(0), a.size(1), a.size(1), ak ? kBM : 64);
  CUtensorMap tbo = make_tma_2d(b.data_ptr(), b.size(0), b.size(1), b.size(1), bk ? kFusedBN : 64);
  // tile stores through TMA need a 16-byte aligned base and row pitch; anything else takes the direct-store path
  const int out_bytes = f32 ? 4 : 2;
  const bool out_ok = (reinterpret_cast<uintptr_t>(p.out) & 15) == 0 && (static_cast<size_t>(p.ldo) * out_bytes) % 16 == 0;
  const bool z_ok = p.z_out == nullptr || ((reinterpret_cast<uintptr_t>(p.z_out) & 15) == 0 && (static_cast<size_t>(p.ldo) * 2) % 16 == 0);
  p.tma_store = (out_ok && z_ok) ? 1 : 0;
  CUtensorMap to = tao, tz = tao;     // placeholders when unused
  if (p.tma_store) {
    to = make_tma_2d_store(p.out, p.Ms, p.Ns, p.ldo, out_bytes, p.is_bf16);
    if (p.z_out != nullptr) tz = make_tma_2d_store(p.z_out, p.Ms, p.Ns, p.ldo, 2, p.is_bf16);
  }
  auto stream = at::cuda::getCurrentCUDAStream();
  if (p.is_bf16) {
    if (f32) dispatch_ggs<__nv_bfloat16, true>(ak, bk, ta, tb, tao, tbo, to, tz, p, stream);
    else dispatch_ggs<__nv_bfloat16, false>(ak, bk, ta, tb, tao, tbo, to, tz, p, stream);
  } else {
    if (f32) dispatch_ggs<__half, true>(ak, bk, ta, tb, tao, tbo, to, tz, p, stream);
    else dispatch_ggs<__half, false>(ak, bk, ta, tb, tao, tbo, to, tz, p, stream);
  }
}

void register_ggs(py::module& m) { m.def("gather_gemm_scatter", &gather_gemm_scatter); }

}  // namespace cw
