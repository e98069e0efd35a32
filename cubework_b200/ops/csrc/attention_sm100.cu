// Fused (flash-style) self-attention for sm_100a on tcgen05 tensor cores, forward and backward, over a packed
// QKV tensor [B, T, heads, 3*dh] whose per-head layout is [q | k | v] (the layout the GPT-2 / OPT / ViT models of
// this package and of the reference use: benchmark/gpt2/gpt2.py:66-96, vit/vit.py:74-89, opt/opt.py:70-128).
// Scores never reach HBM; the reference materialises [b, heads, T, T] several times per layer.
//
// Forward, one CTA per (128-query block, head, batch), 128 threads, thread r owns query row r:
//   S = Q K^T         tcgen05.mma, both operands K-major in shared memory, accumulator in TMEM (128 columns)
//   softmax           rows read back with tcgen05.ld, online max / sum in the exp2 domain, P written to shared
//                     memory as 16-bit in the MMA's swizzled layout
//   O_blk = P V       tcgen05.mma, V consumed as an MN-major operand straight from its row-major image
//   O = O*alpha+O_blk in registers
// Backward, one work item per (128-key block, head, batch) looping over query blocks: S and dP = dO V^T in TMEM,
// P / dS written to shared memory, dV += P^T dO and dK += dS^T Q accumulate in TMEM across the loop,
// dQ = dS K is added to an fp32 scratch buffer (several key blocks contribute to one query block).  Head dims up
// to 64 run as a persistent warp-specialised kernel (attn_bwd_ws_kernel), larger ones with one CTA per work item.
//
// Head dims are zero-padded to DP in {32, 64, 96, 128}.  Q / K / V / dO tiles arrive by TMA (4-D maps over
// [dh, T, heads, B] with a 64 x 128 box, 128-byte swizzle; columns past dh and rows past T are zero-filled by
// the out-of-bounds rule).  When dh is not a multiple of 8 a head's rows are not 16-byte aligned in the packed
// tensor (dh = 25), so a small pre-pass copies them into a padded [part][B, heads, T, 64*NB] buffer first.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAException.h>
#include <torch/extension.h>

#include "common.cuh"
#include "gemm_sm100.cuh"
#include "sm100.cuh"

namespace cw {

constexpr int kAttnThreads = 128;
constexpr int kBlk = 128;                 // queries per CTA == keys per step
constexpr float kLog2e = 1.4426950408889634f;
// Descriptor offsets of an operand read "MN-major" from a row-major [rows, 64*NB] swizzled image.
constexpr uint32_t kMnSbo = 1024;         // between groups of 8 rows (the MMA's K direction)
constexpr uint32_t kMnLbo = kBlk * 128;   // between 64-column blocks (the MMA's M/N direction)

// Byte offset of element (r, c) in a [128 rows x (64*NB) cols] 16-bit image: 64-column blocks of 128 rows,
// rows of 128 bytes, 16-byte chunks XOR-swizzled with the row index inside each 8-row group.
__device__ __forceinline__ uint32_t img_off(int r, int c) {
  const int cb = c >> 6, cc = c & 63;
  return cb * (kBlk * 128) + (r >> 3) * 1024 + (r & 7) * 128 + ((((cc >> 3) ^ (r & 7)) & 7) << 4) + ((cc & 7) << 1);
}

template <typename T>
__device__ __forceinline__ uint32_t pack_pair(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack_pair<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Write 32 consecutive columns [c0, c0+32) of row r of a [128 x 128] 16-bit image.
template <typename T>
__device__ __forceinline__ void store_p_chunk(uint8_t* img, int r, int c0, const float (&v)[32]) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint4 u;
    u.x = pack_pair<T>(v[q * 8 + 0], v[q * 8 + 1]);
    u.y = pack_pair<T>(v[q * 8 + 2], v[q * 8 + 3]);
    u.z = pack_pair<T>(v[q * 8 + 4], v[q * 8 + 5]);
    u.w = pack_pair<T>(v[q * 8 + 6], v[q * 8 + 7]);
    *reinterpret_cast<uint4*>(img + img_off(r, c0 + q * 8)) = u;
  }
}

// K-major descriptor for the k16-th 16-column slice of an image (A or B operand whose MMA-K runs along columns).
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t img_addr, int k16) {
  return make_smem_desc(img_addr + (k16 >> 2) * (kBlk * 128) + (k16 & 3) * 32, 16, 1024);
}
// MN-major descriptor for rows [16*k16, 16*k16+16) of an image (MMA-K runs along rows).
__device__ __forceinline__ uint64_t mnmajor_desc(uint32_t img_addr, int k16) {
  return make_smem_desc(img_addr + k16 * 2048, kMnLbo, kMnSbo);
}

struct AttnParams {
  void* out;            // [B, T, H, dh]
  float* lse;           // [B, H, T]   (log2 domain: m + log2(l))
  const float* key_bias;  // [B, T] or nullptr
  int B, T, H, dh;
  float scale;
  int causal;
  int is_bf16;
  int* status;
  // backward only
  const float* delta;   // [B, H, T]  rowsum(dO * O)
  float* dq_acc;        // [B, H, T, DP] fp32 scratch, zero-initialised (DP = padded head dim)
  void* dqkv;           // [B, T, H, 3*dh]
  int* work_counter;    // zero-initialised: next work item of the persistent backward
  long long* trace;     // optional [3][4096][2]: (event, globaltimer) stamps of CTA 0 (row 0: softmax group 0 / compute thread 0,
                        // row 1: MMA issuer); the persistent backward adds per-CTA totals in row 2
};
__device__ __forceinline__ void attn_trace(long long* trace, int row, int& n, int code) {
  if (trace != nullptr && blockIdx.x == 0 && n < 4096) {
    long long* e = trace + (static_cast<size_t>(row) * 4096 + n) * 2;
    e[0] = code;
    e[1] = static_cast<long long>(globaltimer_ns());
    ++n;
  }
}

// One [128 x 64*NB] tile = NB boxes of 64 columns; arrives on `bar` (expect_tx must cover NB * 16 KB).
template <int NB>
__device__ __forceinline__ void tma_tile(uint8_t* img, const CUtensorMap* map, uint64_t* bar, int row0, int h, int b) {
#pragma unroll
  for (int cb = 0; cb < NB; ++cb) tma_load_4d(img + cb * (kBlk * 128), map, bar, cb * 64, row0, h, b);
}

template <typename T, int DP>
__global__ void __launch_bounds__(kAttnThreads)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, AttnParams p) {
  constexpr int NB = (DP + 63) / 64;
  constexpr int kImg = NB * kBlk * 128;          // bytes of a [128 x DP] image
  constexpr uint32_t kTmemCols = 256;             // S: [0,128)  O_blk: [128, 128+DP)
  constexpr bool kOnePass = DP <= 64;             // scores of the whole block fit in registers
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_img = smem;
  uint8_t* k_img = q_img + kImg;
  uint8_t* v_img = k_img + kImg;
  uint8_t* p_img = v_img + kImg;                  // [128 x 128] 16-bit = 32 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_img + 2 * kBlk * 128);   // 0:S 1:O 2:Q 3:K 4:V
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_bias = reinterpret_cast<float*>(tmem_slot + 2);                 // [2][128] key bias (log2 domain) of a block

  const int r = threadIdx.x, warp = r >> 5;
  const int qb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q0 = qb * kBlk;
  const float* kbias = p.key_bias != nullptr ? p.key_bias + static_cast<int64_t>(b) * p.T : nullptr;
  if (kbias != nullptr) s_bias[r] = r < p.T ? kbias[r] * kLog2e : 0.f;

  if (r == 0) {
    for (int i = 0; i < 5; ++i) mbar_init(&bars[i], 1);
    *abort_flag = 0;
    fence_barrier_init();
    mbar_expect_tx(&bars[2], kImg);
    tma_tile<NB>(q_img, &map_q, &bars[2], q0, h, b);
    mbar_expect_tx(&bars[3], kImg);
    tma_tile<NB>(k_img, &map_k, &bars[3], 0, h, b);
    mbar_expect_tx(&bars[4], kImg);
    tma_tile<NB>(v_img, &map_v, &bars[4], 0, h, b);
  }
  if (warp == 0) {
    __syncwarp();   // lane 0 just left the set-up branch: the allocation is warp-collective
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  const uint32_t idesc_s = make_idesc_f16(kBlk, kBlk, false, false, p.is_bf16);
  const uint32_t idesc_o = make_idesc_f16(kBlk, DP, false, true, p.is_bf16);

  const int q_idx = q0 + r;
  const float sc2 = p.scale * kLog2e;
  float m_run = -INFINITY, l_run = 0.f;
  float o_acc[DP];
#pragma unroll
  for (int i = 0; i < DP; ++i) o_acc[i] = 0.f;

  const int n_kv = p.causal ? min((p.T + kBlk - 1) / kBlk, qb + 1) : (p.T + kBlk - 1) / kBlk;
  bool ok = true;
  for (int j = 0; j < n_kv && ok; ++j) {
    const int k0 = j * kBlk;
    if (r == 0) {
      bool good = true;
      if (j == 0) good = mbar_wait(&bars[2], 0, abort_flag, p.status, kErrAttnBarrierTimeout, blockIdx.x);
      good = good && mbar_wait(&bars[3], j & 1, abort_flag, p.status, kErrAttnBarrierTimeout, blockIdx.x);
      if (good) {
        tc_fence_after();
#pragma unroll
        for (int k16 = 0; k16 < DP / 16; ++k16)
          tc_mma_f16(tmem, kmajor_desc(smem_u32(q_img), k16), kmajor_desc(smem_u32(k_img), k16), idesc_s, k16 > 0);
        tc_commit(&bars[0]);
      }
    }
    if (!mbar_wait(&bars[0], j & 1, abort_flag, p.status, kErrAttnBarrierTimeout, blockIdx.x)) { ok = false; break; }
    tc_fence_after();
    if (r == 0 && j + 1 < n_kv) {                 // K is free again: fetch the next block behind the softmax
      mbar_expect_tx(&bars[3], kImg);
      tma_tile<NB>(k_img, &map_k, &bars[3], k0 + kBlk, h, b);
    }
    const bool diag = (p.causal && j == qb) || (k0 + kBlk > p.T);   // block needs element-wise masking
    const float* bias_j = s_bias + (j & 1) * kBlk;
    if (kbias != nullptr && j + 1 < n_kv) {       // bias of the next block; published by this iteration's __syncthreads
      const int key = k0 + kBlk + r;
      s_bias[((j + 1) & 1) * kBlk + r] = key < p.T ? kbias[key] * kLog2e : 0.f;
    }
    float alpha, l_blk = 0.f, m_use;
    if (kOnePass) {
      float sv[kBlk];
      float m_blk = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t raw[32];
        tmem_ld_32x32(tmem + lane_base + c * 32, raw);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int key = k0 + c * 32 + i;
          float sx = __uint_as_float(raw[i]) * sc2;
          if (kbias != nullptr) sx += bias_j[c * 32 + i];
          if (diag && (key >= p.T || (p.causal && key > q_idx))) sx = -INFINITY;
          sv[c * 32 + i] = sx;
          m_blk = fmaxf(m_blk, sx);
        }
      }
      const float m_new = fmaxf(m_run, m_blk);
      m_use = (m_new == -INFINITY) ? 0.f : m_new;
      alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_use);
      m_run = m_new;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float pv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float e = exp2f(sv[c * 32 + i] - m_use);
          pv[i] = e;
          l_blk += e;
        }
        store_p_chunk<T>(p_img, r, c * 32, pv);
      }
    } else {
      float m_blk = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t raw[32];
        tmem_ld_32x32(tmem + lane_base + c * 32, raw);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int key = k0 + c * 32 + i;
          float sx = __uint_as_float(raw[i]) * sc2;
          if (kbias != nullptr) sx += bias_j[c * 32 + i];
          if (diag && (key >= p.T || (p.causal && key > q_idx))) sx = -INFINITY;
          m_blk = fmaxf(m_blk, sx);
        }
      }
      const float m_new = fmaxf(m_run, m_blk);
      m_use = (m_new == -INFINITY) ? 0.f : m_new;
      alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_use);
      m_run = m_new;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t raw[32];
        tmem_ld_32x32(tmem + lane_base + c * 32, raw);
        tmem_wait_ld();
        float pv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int key = k0 + c * 32 + i;
          float sx = __uint_as_float(raw[i]) * sc2;
          if (kbias != nullptr) sx += bias_j[c * 32 + i];
          if (diag && (key >= p.T || (p.causal && key > q_idx))) sx = -INFINITY;
          const float e = exp2f(sx - m_use);
          pv[i] = e;
          l_blk += e;
        }
        store_p_chunk<T>(p_img, r, c * 32, pv);
      }
    }
    l_run = l_run * alpha + l_blk;
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (r == 0) {
      if (mbar_wait(&bars[4], j & 1, abort_flag, p.status, kErrAttnBarrierTimeout, blockIdx.x)) {
        tc_fence_after();
#pragma unroll
        for (int k16 = 0; k16 < kBlk / 16; ++k16)
          tc_mma_f16(tmem + 128, kmajor_desc(smem_u32(p_img), k16), mnmajor_desc(smem_u32(v_img), k16), idesc_o, k16 > 0);
        tc_commit(&bars[1]);
      }
    }
    if (!mbar_wait(&bars[1], j & 1, abort_flag, p.status, kErrAttnBarrierTimeout, blockIdx.x)) { ok = false; break; }
    tc_fence_after();
    if (r == 0 && j + 1 < n_kv) {                 // V is free again
      mbar_expect_tx(&bars[4], kImg);
      tma_tile<NB>(v_img, &map_v, &bars[4], k0 + kBlk, h, b);
    }
#pragma unroll
    for (int c = 0; c < DP / 32; ++c) {
      uint32_t raw[32];
      tmem_ld_32x32(tmem + 128 + lane_base + c * 32, raw);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] = o_acc[c * 32 + i] * alpha + __uint_as_float(raw[i]);
    }
    tc_fence_before();
  }

  if (ok && q_idx < p.T) {
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    T* o = reinterpret_cast<T*>(p.out) + ((static_cast<int64_t>(b) * p.T + q_idx) * p.H + h) * p.dh;
#pragma unroll
    for (int d = 0; d < DP; ++d)
      if (d < p.dh) o[d] = from_f<T>(o_acc[d] * inv);
    p.lse[(static_cast<int64_t>(b) * p.H + h) * p.T + q_idx] = (l_run > 0.f) ? m_run + log2f(l_run) : -INFINITY;
  }
  if (*abort_flag) {
    for (int i = 0; i < 32; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------------------
// Warp-specialised forward for head dims up to 64: persistent CTAs (one per SM) of ten warps.
//   warps 0-3 / 4-7  two softmax groups; group w owns the key blocks j = w, w+2, ... of the current query tile,
//                    with its own running max / sum and its own output accumulator, merged at the end of the tile
//   warp 8           issues every tcgen05.mma: S_w = Q K_j^T into group w's score columns, O_w += P_w V_j
//   warp 9           TMA producer: Q (two buffers), K and V (rings of three), key bias (ring of six)
// While one group runs its exponentials the tensor core works for the other, and the next score block of a group
// is issued as soon as its P has been handed over, so no group waits for a tensor-core round trip with nothing
// else resident on the SM.  O accumulates in TMEM across key blocks; the owning group rescales it in place
// (tcgen05.ld / st) before handing over the next P.  All hand-overs are mbarriers with bounded waits.
// TMEM: S_0 [0,128)  S_1 [128,256)  O_0 [256,256+DP)  O_1 [320,320+DP).
// ---------------------------------------------------------------------------------------------------------
// Warp-specialised forward for head dims up to 64: persistent CTAs (one per SM) of twelve warps that run TWO
// independent query tiles at a time ("lanes" w = 0, 1), each with its own
//   softmax group   warps 4w .. 4w+3: thread r owns query row r; two passes over the scores in TMEM (maximum, then
//                   exponentials), P to shared memory, O rescaled in TMEM, the tile's output written at the end
//   MMA issuer      warp 8 + w:  S = Q K_j^T, then after the group hands over P_j: O += P_j V_j and S for block j+1
//   TMA producer    warp 10 + w: Q, K (ring of two), V, key bias (ring of four)
// While one lane waits for a tensor-core round trip or writes its output, the other lane's group computes, and the
// MMA / TMA threads never sit on a softmax warp's critical path.  O accumulates in TMEM across key blocks; the group
// rescales it in place (tcgen05.ld / st) before handing over the next P.  All hand-overs are mbarriers with bounded
// waits.  TMEM: S_w at 128 w, O_w at 256 + 64 w.
template <bool MASKED, bool BIAS>
__device__ __forceinline__ float chunk_max(const uint32_t (&raw)[32], const float* bias, float sc2, int key0, int q_idx, int T,
                                           bool causal, float m) {
  float mm[4] = {m, -INFINITY, -INFINITY, -INFINITY};      // four chains: the maximum is not one long dependency
  float bv[32];
  if (BIAS) {
#pragma unroll
    for (int q = 0; q < 8; ++q) {                           // eight 16-byte broadcast loads instead of 32 scalar ones
      const float4 t = reinterpret_cast<const float4*>(bias)[q];
      bv[q * 4] = t.x; bv[q * 4 + 1] = t.y; bv[q * 4 + 2] = t.z; bv[q * 4 + 3] = t.w;
    }
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float sx = BIAS ? fmaf(__uint_as_float(raw[i]), sc2, bv[i]) : __uint_as_float(raw[i]);
    if (MASKED) {
      const int key = key0 + i;
      if (key >= T || (causal && key > q_idx)) sx = -INFINITY;
    }
    mm[i & 3] = fmaxf(mm[i & 3], sx);
  }
  return fmaxf(fmaxf(mm[0], mm[1]), fmaxf(mm[2], mm[3]));
}
// exponentials of one chunk relative to m_use (log2 domain); returns their sum
template <bool MASKED, bool BIAS>
__device__ __forceinline__ float chunk_exp(const uint32_t (&raw)[32], const float* bias, float sc2, float m_use, int key0,
                                           int q_idx, int T, bool causal, float (&pv)[32]) {
  float ll[4] = {0.f, 0.f, 0.f, 0.f};
  float bv[32];
  if (BIAS) {
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float4 t = reinterpret_cast<const float4*>(bias)[q];
      bv[q * 4] = t.x; bv[q * 4 + 1] = t.y; bv[q * 4 + 2] = t.z; bv[q * 4 + 3] = t.w;
    }
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float e = ex2_approx(fmaf(__uint_as_float(raw[i]), sc2, BIAS ? bv[i] - m_use : -m_use));
    if (MASKED) {
      const int key = key0 + i;
      if (key >= T || (causal && key > q_idx)) e = 0.f;
    }
    pv[i] = e;
    ll[i & 3] += e;
  }
  return (ll[0] + ll[1]) + (ll[2] + ll[3]);
}

// Bounded wait whose polling loop is kept out of line: the persistent kernels wait in many places, and their
// instruction footprint decides how often the warps of the different roles miss the instruction cache.
__device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int detail) {
  return mbar_wait(bar, parity, abort_flag, status, kErrAttnBarrierTimeout, detail);
}
__device__ __forceinline__ bool mbar_wait_ol(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int detail) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, status, detail);
}
constexpr int kWsThreads = 384;
constexpr int kWsKRing = 2, kWsBiasRing = 4;
template <int DP>
constexpr int fwd_ws_smem() {
  return 2 * ((1 + kWsKRing + 1) * kBlk * 128 + 2 * kBlk * 128 + kWsBiasRing * kBlk * 4) + 768 + 1024;
}

struct WsLaneBars {
  uint64_t q_full, q_empty;
  uint64_t k_full[kWsKRing], k_empty[kWsKRing];
  uint64_t v_full, v_empty;
  uint64_t s_full, s_free, p_ready, o_full;
  int bias_nz[kWsBiasRing];        // the key bias of this ring slot has a non-zero entry
};

template <typename T, int DP>
__global__ void __launch_bounds__(kWsThreads, 1)
attn_fwd_ws_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, AttnParams p) {
  static_assert(DP <= 64, "one 64-column image per operand");
  constexpr int kImg = kBlk * 128;                 // 16 KB: a [128 x 64] 16-bit image
  constexpr int kPImg = 2 * kBlk * 128;            // 32 KB: a [128 x 128] 16-bit image
  constexpr int kLaneBytes = (1 + kWsKRing + 1) * kImg + kPImg + kWsBiasRing * kBlk * 4;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  WsLaneBars* all_bars = reinterpret_cast<WsLaneBars*>(smem + 2 * kLaneBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(all_bars + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int w = 0; w < 2; ++w) {
      WsLaneBars* bb = all_bars + w;
      mbar_init(&bb->q_full, 1); mbar_init(&bb->q_empty, 1);
      for (int i = 0; i < kWsKRing; ++i) { mbar_init(&bb->k_full[i], 1); mbar_init(&bb->k_empty[i], 1); }
      mbar_init(&bb->v_full, 1); mbar_init(&bb->v_empty, 1);
      mbar_init(&bb->s_full, 1); mbar_init(&bb->s_free, kBlk); mbar_init(&bb->p_ready, kBlk); mbar_init(&bb->o_full, 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 8) {
    __syncwarp();
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // this thread's lane and that lane's buffers
  const int w = warp < 8 ? warp >> 2 : (warp - 8) & 1;
  uint8_t* lane_smem = smem + w * kLaneBytes;
  uint8_t* q_img = lane_smem;
  uint8_t* k_img = q_img + kImg;                   // [kWsKRing]
  uint8_t* v_img = k_img + kWsKRing * kImg;
  uint8_t* p_img = v_img + kImg;
  float* s_bias = reinterpret_cast<float*>(p_img + kPImg);          // [kWsBiasRing][128], log2 domain
  WsLaneBars* bars = all_bars + w;
  const uint32_t tm_s = tmem + w * 128, tm_o = tmem + 256 + w * 64;

  const int n_qb = (p.T + kBlk - 1) / kBlk;
  const int bh_total = p.B * p.H;
  const int tiles = n_qb * bh_total;
  auto n_kv_of = [&](int qb) { return p.causal ? min(n_qb, qb + 1) : n_qb; };
  // tiles of this lane, heaviest (most key blocks) first: t = first, first + stride, ...
  const int first = blockIdx.x + w * gridDim.x, stride = 2 * gridDim.x;

  if (warp >= 10) {
    // =========================================================================== TMA producer (+ key bias)
    int kcount = 0, vcount = 0, tile_it = 0;
    for (int t = first; t < tiles; t += stride, ++tile_it) {
      if (__shfl_sync(0xffffffffu, lane == 0 ? *abort_flag : 0, 0)) break;     // one decision for the whole warp
      const int qb = n_qb - 1 - t / bh_total, bh = t % bh_total;
      const int h = bh % p.H, b = bh / p.H;
      const int n_kv = n_kv_of(qb);
      bool ok = true;
      if (lane == 0) {
        ok = mbar_wait_ol(&bars->q_empty, (tile_it & 1) ^ 1, abort_flag, p.status, t);
        if (ok) {
          mbar_expect_tx(&bars->q_full, kImg);
          tma_load_4d(q_img, &map_q, &bars->q_full, 0, qb * kBlk, h, b);
        }
      }
      for (int j = 0; j < n_kv; ++j) {
        const int ks = kcount % kWsKRing;
        if (lane == 0)
          ok = ok && mbar_wait_ol(&bars->k_empty[ks], ((kcount / kWsKRing) & 1) ^ 1, abort_flag, p.status, t);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        if (p.key_bias != nullptr) {
          float* dst = s_bias + (kcount % kWsBiasRing) * kBlk;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int key = j * kBlk + lane * 4 + i;
            dst[lane * 4 + i] = key < p.T ? p.key_bias[static_cast<int64_t>(b) * p.T + key] * kLog2e : 0.f;
          }
          // an all-zero bias (no padding in this key block) lets the softmax warps skip it
          const bool nz = dst[lane * 4] != 0.f || dst[lane * 4 + 1] != 0.f || dst[lane * 4 + 2] != 0.f || dst[lane * 4 + 3] != 0.f;
          const bool any_nz = __any_sync(0xffffffffu, nz);
          if (lane == 0) bars->bias_nz[kcount % kWsBiasRing] = any_nz ? 1 : 0;
          __threadfence_block();
        }
        __syncwarp();
        if (lane == 0) {
          mbar_expect_tx(&bars->k_full[ks], kImg);
          tma_load_4d(k_img + ks * kImg, &map_k, &bars->k_full[ks], 0, j * kBlk, h, b);
          ok = mbar_wait_ol(&bars->v_empty, (vcount & 1) ^ 1, abort_flag, p.status, t);
          if (ok) {
            mbar_expect_tx(&bars->v_full, kImg);
            tma_load_4d(v_img, &map_v, &bars->v_full, 0, j * kBlk, h, b);
          }
        }
        ++kcount; ++vcount;
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
    }
  } else if (warp >= 8) {
    // =========================================================================== MMA issuer of lane w
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_f16(kBlk, kBlk, false, false, p.is_bf16);
      const uint32_t idesc_o = make_idesc_f16(kBlk, DP, false, true, p.is_bf16);
      int kcount = 0, vcount = 0, pcount = 0, fcount = 0, tile_it = 0;
      bool ok = true;
      auto issue_s = [&](bool last) -> bool {
        const int ks = kcount % kWsKRing;
        if (!mbar_wait_ol(&bars->k_full[ks], (kcount / kWsKRing) & 1, abort_flag, p.status, kcount)) return false;
        tc_fence_after();
#pragma unroll
        for (int k16 = 0; k16 < DP / 16; ++k16)
          tc_mma_f16(tm_s, kmajor_desc(smem_u32(q_img), k16), kmajor_desc(smem_u32(k_img + ks * kImg), k16), idesc_s, k16 > 0);
        tc_commit(&bars->k_empty[ks]);
        tc_commit(&bars->s_full);
        if (last) tc_commit(&bars->q_empty);
        ++kcount;
        return true;
      };
      for (int t = first; t < tiles && ok && !*abort_flag; t += stride, ++tile_it) {
        const int qb = n_qb - 1 - t / bh_total;
        const int n_kv = n_kv_of(qb);
        ok = mbar_wait_ol(&bars->q_full, tile_it & 1, abort_flag, p.status, t);
        ok = ok && issue_s(n_kv == 1);
        for (int j = 0; j < n_kv && ok; ++j) {
          // the group has read S_j for the last time: S_{j+1} goes first, it is what the group needs soonest
          ok = mbar_wait_ol(&bars->s_free, fcount & 1, abort_flag, p.status, t);
          if (!ok) break;
          ++fcount;
          if (j + 1 < n_kv) {
            tc_fence_after();
            ok = issue_s(j + 1 == n_kv - 1);
            if (!ok) break;
          }
          ok = mbar_wait_ol(&bars->p_ready, pcount & 1, abort_flag, p.status, t);
          if (!ok) break;
          ++pcount;
          ok = mbar_wait_ol(&bars->v_full, vcount & 1, abort_flag, p.status, t);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int k16 = 0; k16 < kBlk / 16; ++k16)
            tc_mma_f16(tm_o, kmajor_desc(smem_u32(p_img), k16), mnmajor_desc(smem_u32(v_img), k16), idesc_o,
                       (j > 0 || k16 > 0) ? 1u : 0u);
          tc_commit(&bars->v_empty);
          tc_commit(&bars->o_full);
          ++vcount;
        }
      }
    }
  } else {
    // =========================================================================== softmax group of lane w
    const int r = threadIdx.x & 127;                 // query row inside the tile == TMEM lane
    const int wq = warp & 3;                         // this warp's 32-row block
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    const float sc2 = p.scale * kLog2e;
    int scount = 0, ocount = 0, kbase = 0;           // uses of s_full / o_full; key blocks before this tile
    bool ok = true;
    int ntr = 0;
    long long* tr = threadIdx.x == 0 ? p.trace : nullptr;
    for (int t = first; t < tiles && ok; t += stride) {
      const int qb = n_qb - 1 - t / bh_total, bh = t % bh_total;
      const int h = bh % p.H, b = bh / p.H;
      const int n_kv = n_kv_of(qb);
      const int q_idx = qb * kBlk + r;
      float m_run = -INFINITY, l_run = 0.f;
      for (int j = 0; j < n_kv; ++j) {
        const int k0 = j * kBlk;
        attn_trace(tr, 0, ntr, 1);
        if (!mbar_wait_ol(&bars->s_full, scount & 1, abort_flag, p.status, t)) { ok = false; break; }
        ++scount;
        tc_fence_after();
        attn_trace(tr, 0, ntr, 2);
        const bool tail = k0 + kBlk > p.T;
        const bool cdiag = p.causal && j == qb;
        const float* bias_j = s_bias + ((kbase + j) % kWsBiasRing) * kBlk;
        const bool has_bias = p.key_bias != nullptr && bars->bias_nz[(kbase + j) % kWsBiasRing] != 0;
        const uint32_t s_addr = tm_s + lane_base;
        uint32_t ra[32], rb[32];
        float m_blk = -INFINITY;
        // ---- pass 1: the row maximum.  The next chunk's TMEM load is in flight while the current one is reduced.
        if (!tail && !cdiag) {
          // all four chunk loads are issued before the first is used: one TMEM round trip for the pass
          uint32_t rc[32], rd[32];
          tmem_ld_32x32(s_addr, ra);
          tmem_ld_32x32(s_addr + 32, rb);
          tmem_ld_32x32(s_addr + 64, rc);
          tmem_ld_32x32(s_addr + 96, rd);
          tmem_wait_ld_for(ra);
          tmem_wait_ld_for(rb);
          tmem_wait_ld_for(rc);
          tmem_wait_ld_for(rd);
#define CW_MAX_STEP(CUR, C)                                                                                   \
          m_blk = has_bias ? chunk_max<false, true>(CUR, bias_j + (C) * 32, sc2, 0, 0, 0, false, m_blk)        \
                           : chunk_max<false, false>(CUR, nullptr, sc2, 0, 0, 0, false, m_blk);
          CW_MAX_STEP(ra, 0)
          CW_MAX_STEP(rb, 1)
          CW_MAX_STEP(rc, 2)
          CW_MAX_STEP(rd, 3)
#undef CW_MAX_STEP
        } else {
          // diagonal block of a causal mask: chunks left of this warp's rows are plain, the chunk on the diagonal is
          // tested key by key, chunks to the right contribute nothing.  A sequence tail is tested everywhere.
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            if (!tail && c > wq) break;
            tmem_ld_32x32(s_addr + c * 32, ra);
            tmem_wait_ld_for(ra);
            if (!tail && c < wq)
              m_blk = has_bias ? chunk_max<false, true>(ra, bias_j + c * 32, sc2, 0, 0, 0, false, m_blk)
                               : chunk_max<false, false>(ra, nullptr, sc2, 0, 0, 0, false, m_blk);
            else
              m_blk = has_bias ? chunk_max<true, true>(ra, bias_j + c * 32, sc2, k0 + c * 32, q_idx, p.T, cdiag, m_blk)
                               : chunk_max<true, false>(ra, nullptr, sc2, k0 + c * 32, q_idx, p.T, cdiag, m_blk);
          }
        }
        if (!has_bias) m_blk *= sc2;                  // scale > 0: the maximum commutes with the scaling
        attn_trace(tr, 0, ntr, 3);
        const float m_new = fmaxf(m_run, m_blk);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = (m_run == -INFINITY) ? 0.f : ex2_approx(m_run - m_use);
        m_run = m_new;
        if (j > 0) {
          // the previous P V has landed in O: rescale it in place before more is added
          if (!mbar_wait_ol(&bars->o_full, ocount & 1, abort_flag, p.status, t)) { ok = false; break; }
          ++ocount;
          tc_fence_after();
          attn_trace(tr, 0, ntr, 4);
          if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
            for (int c = 0; c < DP / 32; ++c) {
              uint32_t raw[32];
              tmem_ld_32x32(tm_o + lane_base + c * 32, raw);
              tmem_wait_ld_for(raw);
#pragma unroll
              for (int i = 0; i < 32; ++i) raw[i] = __float_as_uint(__uint_as_float(raw[i]) * alpha);
              tmem_st_32x32(tm_o + lane_base + c * 32, raw);
            }
            tmem_wait_st();
          }
        }
        // ---- pass 2: exponentials, P to shared memory
        float l_blk = 0.f;
        attn_trace(tr, 0, ntr, 5);
        if (!tail && !cdiag) {
          // chunks 0 and 1 are requested together; chunk c + 2 is requested before chunk c is processed
          uint32_t rc[32];
          tmem_ld_32x32(s_addr, ra);
          tmem_ld_32x32(s_addr + 32, rb);
          tmem_wait_ld_for(ra);
          tmem_wait_ld_for(rb);
#define CW_EXP_STEP(CUR, C)                                                                                   \
          {                                                                                                    \
            float pv[32];                                                                                      \
            l_blk += has_bias ? chunk_exp<false, true>(CUR, bias_j + (C) * 32, sc2, m_use, 0, 0, 0, false, pv) \
                              : chunk_exp<false, false>(CUR, nullptr, sc2, m_use, 0, 0, 0, false, pv);         \
            store_p_chunk<T>(p_img, r, (C) * 32, pv);                                                          \
          }
          tmem_ld_32x32(s_addr + 64, rc);
          CW_EXP_STEP(ra, 0)
          tmem_wait_ld_for(rc);
          tmem_ld_32x32(s_addr + 96, ra);
          CW_EXP_STEP(rb, 1)
          tmem_wait_ld_for(ra);
          tc_fence_before();
          mbar_arrive(&bars->s_free);                 // last read of the scores: the next block's S may overwrite them
          CW_EXP_STEP(rc, 2)
          CW_EXP_STEP(ra, 3)
#undef CW_EXP_STEP
        } else {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            float pv[32];
            if (!tail && c > wq) {
#pragma unroll
              for (int i = 0; i < 32; ++i) pv[i] = 0.f;
            } else {
              tmem_ld_32x32(s_addr + c * 32, ra);
              tmem_wait_ld_for(ra);
              if (!tail && c < wq)
                l_blk += has_bias ? chunk_exp<false, true>(ra, bias_j + c * 32, sc2, m_use, 0, 0, 0, false, pv)
                                  : chunk_exp<false, false>(ra, nullptr, sc2, m_use, 0, 0, 0, false, pv);
              else
                l_blk += has_bias ? chunk_exp<true, true>(ra, bias_j + c * 32, sc2, m_use, k0 + c * 32, q_idx, p.T, cdiag, pv)
                                  : chunk_exp<true, false>(ra, nullptr, sc2, m_use, k0 + c * 32, q_idx, p.T, cdiag, pv);
            }
            store_p_chunk<T>(p_img, r, c * 32, pv);
          }
          tc_fence_before();
          mbar_arrive(&bars->s_free);
        }
        l_run = l_run * alpha + l_blk;
        attn_trace(tr, 0, ntr, 6);
        fence_proxy_async();
        tc_fence_before();
        mbar_arrive(&bars->p_ready);
        attn_trace(tr, 0, ntr, 7);
      }
      if (!ok) break;
      // ---- the tile's output: the last P V has landed
      if (!mbar_wait_ol(&bars->o_full, ocount & 1, abort_flag, p.status, t)) { ok = false; break; }
      ++ocount;
      tc_fence_after();
      attn_trace(tr, 0, ntr, 8);
      {
        // rows go through shared memory (the P image is free now) so that each global store instruction writes one
        // row's contiguous bytes instead of one column of 32 rows that lie kilobytes apart
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        T* stage = reinterpret_cast<T*>(p_img) + wq * 32 * DP;          // this warp's [32][DP]
#pragma unroll
        for (int c = 0; c < DP / 32; ++c) {
          uint32_t raw[32];
          tmem_ld_32x32(tm_o + lane_base + c * 32, raw);
          tmem_wait_ld_for(raw);
          uint4* dst = reinterpret_cast<uint4*>(stage + lane * DP + c * 32);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 u;
            u.x = pack_pair<T>(__uint_as_float(raw[q * 8 + 0]) * inv, __uint_as_float(raw[q * 8 + 1]) * inv);
            u.y = pack_pair<T>(__uint_as_float(raw[q * 8 + 2]) * inv, __uint_as_float(raw[q * 8 + 3]) * inv);
            u.z = pack_pair<T>(__uint_as_float(raw[q * 8 + 4]) * inv, __uint_as_float(raw[q * 8 + 5]) * inv);
            u.w = pack_pair<T>(__uint_as_float(raw[q * 8 + 6]) * inv, __uint_as_float(raw[q * 8 + 7]) * inv);
            dst[q] = u;
          }
        }
        if (q_idx < p.T)
          p.lse[(static_cast<int64_t>(b) * p.H + h) * p.T + q_idx] = (l_run > 0.f) ? m_run + log2f(l_run) : -INFINITY;
        tc_fence_before();
        __syncwarp();
        const int row0 = qb * kBlk + wq * 32;
        T* o = reinterpret_cast<T*>(p.out) + ((static_cast<int64_t>(b) * p.T + row0) * p.H + h) * p.dh;
        const int64_t row_pitch = static_cast<int64_t>(p.H) * p.dh;
        const int rows = min(32, p.T - row0);
        for (int d = lane; d < p.dh; d += 32) {
          for (int r0 = 0; r0 < rows; r0 += 8) {
            T v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = stage[min(r0 + u, 31) * DP + d];
#pragma unroll
            for (int u = 0; u < 8; ++u)
              if (r0 + u < rows) o[(r0 + u) * row_pitch + d] = v[u];
          }
        }
        __syncwarp();
      }
      attn_trace(tr, 0, ntr, 9);
      kbase += n_kv;
    }
    if (!ok) *abort_flag = 1;
  }

  if (*abort_flag) {
    for (int i = 0; i < 32; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// Copy `parts` consecutive [dh] slices per (token, head) of src [B, T, H, parts*dh] into zero-padded rows
// dst [parts][B, H, T, W] (W a multiple of 8 elements): makes every row 16-byte aligned for TMA.
template <typename T>
__global__ void attn_pack_kernel(const T* __restrict__ src, T* __restrict__ dst, int B, int Tn, int H, int dh, int parts,
                                 int W) {
  // One thread per (b, t, h, part) slice.  A warp's 32 slices are 32 * dh consecutive source elements: they are
  // fetched with coalesced 16-byte loads into shared memory (when the chunk is 16-byte aligned, i.e. dh even),
  // and each thread then assembles its zero-padded row from there.
  extern __shared__ __align__(16) uint8_t pack_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  T* stage = reinterpret_cast<T*>(pack_smem) + static_cast<size_t>(warp) * 32 * dh;
  const int64_t total = static_cast<int64_t>(B) * Tn * H * parts;
  const int64_t first = (static_cast<int64_t>(blockIdx.x) * blockDim.x + warp * 32);
  if (first >= total) return;
  const int rows = static_cast<int>(min(static_cast<int64_t>(32), total - first));
  const T* chunk = src + first * dh;
  const int n_el = rows * dh;
  if ((reinterpret_cast<uintptr_t>(chunk) & 15) == 0) {
    const int n16 = n_el / 8;
    for (int i = lane; i < n16; i += 32)
      reinterpret_cast<uint4*>(stage)[i] = reinterpret_cast<const uint4*>(chunk)[i];
    for (int i = n16 * 8 + lane; i < n_el; i += 32) stage[i] = chunk[i];
  } else {
    for (int i = lane; i < n_el; i += 32) stage[i] = chunk[i];
  }
  __syncwarp();
  if (lane >= rows) return;
  const int64_t idx = first + lane;
  const int part = idx % parts;
  const int64_t bth = idx / parts;
  const int h = bth % H;
  const int64_t bt = bth / H;
  const int t = bt % Tn, b = bt / Tn;
  const T* s = stage + lane * dh;
  T* d = dst + (((static_cast<int64_t>(part) * B + b) * H + h) * Tn + t) * W;
  for (int c0 = 0; c0 < W; c0 += 8) {
    T tmp[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) tmp[i] = (c0 + i < dh) ? s[c0 + i] : from_f<T>(0.f);
    *reinterpret_cast<uint4*>(d + c0) = *reinterpret_cast<const uint4*>(tmp);
  }
}

// delta[b, h, t] = sum_d dO[b,t,h,d] * O[b,t,h,d]
// A warp takes 32 consecutive (b, t, h) rows, i.e. 32 * dh consecutive elements of both tensors: it reads them with
// coalesced 16-byte loads (the chunk starts on a 16-byte boundary for every dh), leaves the products in shared memory
// and each lane sums one row.
template <typename T>
__global__ void attn_delta_kernel(const T* __restrict__ dout, const T* __restrict__ out, float* __restrict__ delta, int B,
                                  int Tn, int H, int dh) {
  extern __shared__ __align__(16) uint8_t delta_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* prod = reinterpret_cast<float*>(delta_smem) + static_cast<size_t>(warp) * 32 * dh;
  const int64_t total = static_cast<int64_t>(B) * Tn * H;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * blockDim.x + warp * 32;
  if (first >= total) return;
  const int rows = static_cast<int>(min(static_cast<int64_t>(32), total - first));
  const int n_el = rows * dh;
  const T* a = dout + first * dh;
  const T* o = out + first * dh;
  const int n16 = n_el / 8;
  for (int i = lane; i < n16; i += 32) {
    const uint4 va = reinterpret_cast<const uint4*>(a)[i], vo = reinterpret_cast<const uint4*>(o)[i];
    const T* ha = reinterpret_cast<const T*>(&va);
    const T* ho = reinterpret_cast<const T*>(&vo);
#pragma unroll
    for (int e = 0; e < 8; ++e) prod[i * 8 + e] = to_f(ha[e]) * to_f(ho[e]);
  }
  for (int i = n16 * 8 + lane; i < n_el; i += 32) prod[i] = to_f(a[i]) * to_f(o[i]);
  __syncwarp();
  if (lane >= rows) return;
  float s = 0.f;
  for (int d = 0; d < dh; ++d) s += prod[lane * dh + d];
  const int64_t idx = first + lane;
  const int h = idx % H;
  const int64_t bt = idx / H;
  const int t = bt % Tn, b = bt / Tn;
  delta[(static_cast<int64_t>(b) * H + h) * Tn + t] = s;
}

// dqkv[b, t, h, 0:dh] = dq_acc[b, h, t, 0:dh]   (fp32 accumulator, padded to DP columns, head-major)
// One thread per (b, t, h) row: it reads its 4*DP contiguous bytes, converts, and the warp writes the 32 rows one
// after the other with the lanes along the row (contiguous bytes per store instruction).
template <typename T>
__global__ void attn_dq_store_kernel(const float* __restrict__ dq_acc, T* __restrict__ dqkv, int B, int Tn, int H, int dh,
                                     int DP) {
  extern __shared__ __align__(16) uint8_t dq_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  T* stage = reinterpret_cast<T*>(dq_smem) + static_cast<size_t>(warp) * 32 * DP;
  const int64_t total = static_cast<int64_t>(B) * Tn * H;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * blockDim.x + warp * 32;
  if (first >= total) return;
  const int rows = static_cast<int>(min(static_cast<int64_t>(32), total - first));
  // eight lanes read one accumulator row (DP floats, contiguous), so an instruction touches four rows' full lines
  // instead of 16 bytes of 32 different ones
  {
    const int sub = lane >> 3, qv = lane & 7;
    for (int r0 = 0; r0 < rows; r0 += 4) {
      const int rr = r0 + sub;
      if (rr < rows) {
        const int64_t bth = first + rr;
        const int h = bth % H;
        const int64_t bt = bth / H;
        const int t = bt % Tn, b = bt / Tn;
        const float4* srow = reinterpret_cast<const float4*>(dq_acc + ((static_cast<int64_t>(b) * H + h) * Tn + t) * DP);
        for (int q = qv; q < DP / 4; q += 8) {
          const float4 v = srow[q];
          T* o = stage + rr * DP + q * 4;
          o[0] = from_f<T>(v.x); o[1] = from_f<T>(v.y); o[2] = from_f<T>(v.z); o[3] = from_f<T>(v.w);
        }
      }
    }
  }
  __syncwarp();
  T* dst = dqkv + first * 3 * dh;
  for (int d = lane; d < dh; d += 32)
    for (int r0 = 0; r0 < rows; r0 += 8) {
      T v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = stage[min(r0 + u, 31) * DP + d];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (r0 + u < rows) dst[static_cast<int64_t>(r0 + u) * 3 * dh + d] = v[u];
    }
}

// P and dS of one 32-score chunk of a row.  p = exp2(s*sc2 + bias - lse), ds = p * (dp - delta) * scale.
template <bool MASKED, bool BIAS, typename T>
__device__ __forceinline__ void bwd_chunk(const uint32_t (&rs)[32], const uint32_t (&rp)[32], const float* bias, float sc2,
                                          float lse2, float scale, float nds, int key0, int q_idx, int Tn, bool causal,
                                          uint8_t* p_img, uint8_t* ds_img, int r, int c0) {
  float pv[32], dsv[32];
  float bv[32];
  if (BIAS) {
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float4 t = reinterpret_cast<const float4*>(bias)[q];
      bv[q * 4] = t.x; bv[q * 4 + 1] = t.y; bv[q * 4 + 2] = t.z; bv[q * 4 + 3] = t.w;
    }
  }
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    float pr = ex2_approx(fmaf(__uint_as_float(rs[j]), sc2, BIAS ? bv[j] - lse2 : -lse2));
    if (MASKED) {
      const int key = key0 + j;
      if (key >= Tn || q_idx >= Tn || (causal && key > q_idx)) pr = 0.f;
    }
    pv[j] = pr;
    dsv[j] = pr * fmaf(__uint_as_float(rp[j]), scale, nds);
  }
  store_p_chunk<T>(p_img, r, c0, pv);
  store_p_chunk<T>(ds_img, r, c0, dsv);
}

constexpr int kBwdThreads = 256;   // two threads per query row: each handles 64 of the 128 keys of a block

template <typename T, int DP>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do, AttnParams p) {
  constexpr int NB = (DP + 63) / 64;
  constexpr int kImg = NB * kBlk * 128;
  constexpr uint32_t kTmemCols = 512;
  // TMEM columns.  DP <= 64: S [0,128) dP [128,256) dV [256,..) dK [320,..) dQ [384,..) and [448,..): dQ has two
  // column sets of its own, used alternately, so the scores of the next query block are multiplied right behind this
  // block's products and a block's dQ is written out one iteration later, while the next products run.
  // DP > 64: S/dQ [0,128) dP [128,256) dV [256,..) dK [384,..) (dQ reuses the score columns).
  constexpr bool kSep = DP <= 64;
  constexpr uint32_t kColDV = 256, kColDK = kSep ? 320 : 384, kColDQ = kSep ? 384 : 0;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_img = smem;
  uint8_t* v_img = k_img + kImg;
  constexpr int kBufs = NB == 1 ? 2 : 1;          // Q and dO are double-buffered when shared memory allows
  uint8_t* q_img0 = v_img + kImg;
  uint8_t* do_img0 = q_img0 + kBufs * kImg;
  uint8_t* p_img = do_img0 + kBufs * kImg;
  uint8_t* ds_img = p_img + 2 * kBlk * 128;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ds_img + 2 * kBlk * 128);   // 0: S,dP  1: dQ  2: K,V  3,4: Q,dO  5: dV,dK
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_bias = reinterpret_cast<float*>(tmem_slot + 4);                 // [128] key bias (log2 domain) of this block
  // [128][DP] fp32 staging of dQ: a region of its own for DP <= 64 (it is filled while the MMAs still read P / dS),
  // otherwise it aliases P / dS between their uses
  float* dq_stage = kSep ? s_bias + kBlk : reinterpret_cast<float*>(p_img);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int r = tid & 127;                         // query row inside a block == TMEM lane
  const int half = tid >> 7;                       // which 64 keys of the block this thread handles
  const int kb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int k0 = kb * kBlk;
  const int64_t ld = static_cast<int64_t>(p.H) * 3 * p.dh;
  const float* kbias = p.key_bias != nullptr ? p.key_bias + static_cast<int64_t>(b) * p.T : nullptr;
  int bias_nz = 0;                                  // this thread's bias entry is non-zero
  if (kbias != nullptr && tid < kBlk) {
    s_bias[tid] = k0 + tid < p.T ? kbias[k0 + tid] * kLog2e : 0.f;
    bias_nz = s_bias[tid] != 0.f;
  }
  const int n_q = (p.T + kBlk - 1) / kBlk;
  const int i0 = p.causal ? kb : 0;

  if (tid == 0) {
    for (int i = 0; i < 6; ++i) mbar_init(&bars[i], 1);
    *abort_flag = 0;
    fence_barrier_init();
    mbar_expect_tx(&bars[2], 2 * kImg);
    tma_tile<NB>(k_img, &map_k, &bars[2], k0, h, b);
    tma_tile<NB>(v_img, &map_v, &bars[2], k0, h, b);
    if (i0 < n_q) {
      mbar_expect_tx(&bars[3], 2 * kImg);
      tma_tile<NB>(q_img0, &map_q, &bars[3], i0 * kBlk, h, b);
      tma_tile<NB>(do_img0, &map_do, &bars[3], i0 * kBlk, h, b);
    }
    if (kBufs == 2 && i0 + 1 < n_q) {
      mbar_expect_tx(&bars[4], 2 * kImg);
      tma_tile<NB>(q_img0 + kImg, &map_q, &bars[4], (i0 + 1) * kBlk, h, b);
      tma_tile<NB>(do_img0 + kImg, &map_do, &bars[4], (i0 + 1) * kBlk, h, b);
    }
  }
  if (warp == 0) {
    __syncwarp();   // lane 0 just left the set-up branch: the allocation is warp-collective
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  // an all-zero bias (no padding among these keys) is skipped altogether
  const bool has_bias = __syncthreads_or(bias_nz) != 0;
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  const uint32_t idesc_s = make_idesc_f16(kBlk, kBlk, false, false, p.is_bf16);     // Q K^T, dO V^T
  const uint32_t idesc_tt = make_idesc_f16(kBlk, DP, true, true, p.is_bf16);        // P^T dO, dS^T Q
  const uint32_t idesc_dq = make_idesc_f16(kBlk, DP, false, true, p.is_bf16);       // dS K
  const float sc2 = p.scale * kLog2e;

  // S = Q K^T and dP = dO V^T of the query block held in buffer `sb` (thread 0 only)
  auto issue_scores = [&](int it, int sb) -> bool {
    const uint32_t parity = kBufs == 2 ? ((it >> 1) & 1) : (it & 1);
    bool good = true;
    if (it == 0) good = mbar_wait(&bars[2], 0, abort_flag, p.status, kErrAttnBarrierTimeout, blockIdx.x);
    good = good && mbar_wait(&bars[3 + sb], parity, abort_flag, p.status, kErrAttnBarrierTimeout, blockIdx.x);
    if (!good) return false;
    tc_fence_after();
    const uint32_t qa = smem_u32(q_img0 + sb * kImg), da = smem_u32(do_img0 + sb * kImg);
#pragma unroll
    for (int k16 = 0; k16 < DP / 16; ++k16)
      tc_mma_f16(tmem, kmajor_desc(qa, k16), kmajor_desc(smem_u32(k_img), k16), idesc_s, k16 > 0);
#pragma unroll
    for (int k16 = 0; k16 < DP / 16; ++k16)
      tc_mma_f16(tmem + 128, kmajor_desc(da, k16), kmajor_desc(smem_u32(v_img), k16), idesc_s, k16 > 0);
    tc_commit(&bars[0]);
    return true;
  };

  bool ok = true;
  int it = 0, ntr = 0;
  const bool trb = tid == 0 && blockIdx.y == 0 && blockIdx.z == 0;
  if (trb) attn_trace(p.trace, 0, ntr, 0);
  if (kSep && tid == 0 && i0 < n_q) issue_scores(0, 0);
  for (int i = i0; i < n_q && ok; ++i, ++it) {
    const int q0 = i * kBlk;
    const int sb = kBufs == 2 ? (it & 1) : 0;
    uint8_t* q_img = q_img0 + sb * kImg;
    uint8_t* do_img = do_img0 + sb * kImg;
    const int q_idx = q0 + r;
    const int64_t stat = (static_cast<int64_t>(b) * p.H + h) * p.T + q_idx;
    const float lse2 = q_idx < p.T ? p.lse[stat] : 0.f;
    const float nds = q_idx < p.T ? -p.delta[stat] * p.scale : 0.f;
    if (!kSep) {
      // every thread has finished reading dQ of the previous query block, and the bulk reduction of that block has
      // finished reading its staging area (aliased with P / dS)
      if (tid == 0) bulk_wait_group_read0();
      tc_fence_before();
      __syncthreads();
      if (tid == 0) issue_scores(it, sb);
    }
    if (trb) attn_trace(p.trace, 0, ntr, 1);
    if (!mbar_wait(&bars[0], it & 1, abort_flag, p.status, kErrAttnBarrierTimeout, blockIdx.x)) { ok = false; break; }
    tc_fence_after();
    if (trb) attn_trace(p.trace, 0, ntr, 2);
    const bool tail = (k0 + kBlk > p.T) || (q0 + kBlk > p.T);
    const bool cdiag = p.causal && i == kb;
    const int wq = warp & 3;                       // this warp's 32-row block
    const int c_a = half * 2, c_b = half * 2 + 1;  // this thread's two 32-key chunks
    if (!tail && !cdiag) {
      // the second pair of TMEM loads is in flight while the first is processed
      uint32_t rs_a[32], rp_a[32], rs_b[32], rp_b[32];
      tmem_ld_32x32(tmem + lane_base + c_a * 32, rs_a);
      tmem_ld_32x32(tmem + 128 + lane_base + c_a * 32, rp_a);
      tmem_wait_ld_for(rs_a);
      tmem_wait_ld_for(rp_a);
      tmem_ld_32x32(tmem + lane_base + c_b * 32, rs_b);
      tmem_ld_32x32(tmem + 128 + lane_base + c_b * 32, rp_b);
      if (has_bias) bwd_chunk<false, true, T>(rs_a, rp_a, s_bias + c_a * 32, sc2, lse2, p.scale, nds, 0, 0, 0, false, p_img, ds_img, r, c_a * 32);
      else bwd_chunk<false, false, T>(rs_a, rp_a, nullptr, sc2, lse2, p.scale, nds, 0, 0, 0, false, p_img, ds_img, r, c_a * 32);
      tmem_wait_ld_for(rs_b);
      tmem_wait_ld_for(rp_b);
      if (has_bias) bwd_chunk<false, true, T>(rs_b, rp_b, s_bias + c_b * 32, sc2, lse2, p.scale, nds, 0, 0, 0, false, p_img, ds_img, r, c_b * 32);
      else bwd_chunk<false, false, T>(rs_b, rp_b, nullptr, sc2, lse2, p.scale, nds, 0, 0, 0, false, p_img, ds_img, r, c_b * 32);
    } else {
      // diagonal block of a causal mask: key chunks left of this warp's rows are plain, the chunk on the diagonal is
      // tested key by key, chunks to the right are zero.  Blocks that reach past the sequence end are tested everywhere.
#pragma unroll 1
      for (int cc = 0; cc < 2; ++cc) {
        const int c = half * 2 + cc;
        if (!tail && c > wq) {
          float z[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) z[j] = 0.f;
          store_p_chunk<T>(p_img, r, c * 32, z);
          store_p_chunk<T>(ds_img, r, c * 32, z);
          continue;
        }
        uint32_t rs[32], rp[32];
        tmem_ld_32x32(tmem + lane_base + c * 32, rs);
        tmem_ld_32x32(tmem + 128 + lane_base + c * 32, rp);
        tmem_wait_ld_for(rs);
        tmem_wait_ld_for(rp);
        if (!tail && c < wq) {
          if (has_bias) bwd_chunk<false, true, T>(rs, rp, s_bias + c * 32, sc2, lse2, p.scale, nds, 0, 0, 0, false, p_img, ds_img, r, c * 32);
          else bwd_chunk<false, false, T>(rs, rp, nullptr, sc2, lse2, p.scale, nds, 0, 0, 0, false, p_img, ds_img, r, c * 32);
        } else {
          if (has_bias) bwd_chunk<true, true, T>(rs, rp, s_bias + c * 32, sc2, lse2, p.scale, nds, k0 + c * 32, q_idx, p.T, cdiag, p_img, ds_img, r, c * 32);
          else bwd_chunk<true, false, T>(rs, rp, nullptr, sc2, lse2, p.scale, nds, k0 + c * 32, q_idx, p.T, cdiag, p_img, ds_img, r, c * 32);
        }
      }
    }
    if (trb) attn_trace(p.trace, 0, ntr, 3);
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (trb) attn_trace(p.trace, 0, ntr, 4);
    // dQ of (query block, key block): TMEM -> registers -> shared staging -> one bulk fp32 reduction into the
    // [B, H, T, DP] accumulator (several key blocks add into the same query rows)
    auto drain_dq = [&](uint32_t col, int q_first) {
#pragma unroll
      for (int c = 0; c < DP / 32; ++c) {
        if ((c & 1) != half && DP > 32) continue;            // the two threads of a row share the chunks
        if (DP == 32 && half != 0) continue;
        uint32_t raw[32];
        tmem_ld_32x32(tmem + col + lane_base + c * 32, raw);
        tmem_wait_ld_for(raw);
        float4* dst = reinterpret_cast<float4*>(dq_stage + r * DP + c * 32);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          dst[j] = make_float4(__uint_as_float(raw[4 * j]), __uint_as_float(raw[4 * j + 1]),
                               __uint_as_float(raw[4 * j + 2]), __uint_as_float(raw[4 * j + 3]));
      }
      fence_proxy_async();
      tc_fence_before();
      __syncthreads();
      if (tid == 0) {
        const int qvalid = min(kBlk, p.T - q_first);
        float* gdst = p.dq_acc + ((static_cast<int64_t>(b) * p.H + h) * p.T + q_first) * DP;
        bulk_reduce_add_f32(gdst, dq_stage, static_cast<uint32_t>(qvalid) * DP * 4);
        bulk_commit_group();
      }
    };
    const uint32_t col_dq = kSep ? kColDQ + (it & 1) * 64 : kColDQ;
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int k16 = 0; k16 < kBlk / 16; ++k16)   // dQ[q, d] = sum_key dS[q, key] K[key, d]
        tc_mma_f16(tmem + col_dq, kmajor_desc(smem_u32(ds_img), k16), mnmajor_desc(smem_u32(k_img), k16), idesc_dq, k16 > 0);
      tc_commit(&bars[1]);
      // the scores of the next query block, right behind this block's products
      if (kSep && i + 1 < n_q) issue_scores(it + 1, kBufs == 2 ? (sb ^ 1) : 0);
    } else if (tid == kBlk) {
      // a thread of another warp issues the other two products at the same time (issuing takes about a microsecond)
      tc_fence_after();
      const uint32_t acc = it > 0 ? 1u : 0u;
#pragma unroll
      for (int k16 = 0; k16 < kBlk / 16; ++k16)   // dV[key, d] += sum_q P[q, key] dO[q, d]
        tc_mma_f16(tmem + kColDV, mnmajor_desc(smem_u32(p_img), k16), mnmajor_desc(smem_u32(do_img), k16), idesc_tt,
                   (k16 > 0) ? 1u : acc);
#pragma unroll
      for (int k16 = 0; k16 < kBlk / 16; ++k16)   // dK[key, d] += sum_q dS[q, key] Q[q, d]
        tc_mma_f16(tmem + kColDK, mnmajor_desc(smem_u32(ds_img), k16), mnmajor_desc(smem_u32(q_img), k16), idesc_tt,
                   (k16 > 0) ? 1u : acc);
      tc_commit(&bars[5]);
    }
    if (trb) attn_trace(p.trace, 0, ntr, 5);
    if (kSep && it > 0) {
      // while those run: write out the previous block's dQ (its MMAs were waited for at the end of that iteration)
      if (tid == 0) bulk_wait_group_read0();               // the staging area has been read by the reduction before it
      __syncthreads();
      drain_dq(kColDQ + ((it - 1) & 1) * 64, q0 - kBlk);
    }
    if (trb) attn_trace(p.trace, 0, ntr, 6);
    if (!mbar_wait(&bars[1], it & 1, abort_flag, p.status, kErrAttnBarrierTimeout, blockIdx.x) ||
        !mbar_wait(&bars[5], it & 1, abort_flag, p.status, kErrAttnBarrierTimeout, blockIdx.x)) { ok = false; break; }
    tc_fence_after();
    if (trb) attn_trace(p.trace, 0, ntr, 7);
    // every MMA that read this block's Q / dO buffer (and P / dS) is done: refill the buffer
    {
      const int nxt = kBufs == 2 ? i + 2 : i + 1;
      if (tid == 0 && nxt < n_q) {
        mbar_expect_tx(&bars[3 + sb], 2 * kImg);
        tma_tile<NB>(q_img0 + sb * kImg, &map_q, &bars[3 + sb], nxt * kBlk, h, b);
        tma_tile<NB>(do_img0 + sb * kImg, &map_do, &bars[3 + sb], nxt * kBlk, h, b);
      }
    }
    if (!kSep) drain_dq(kColDQ, q0);
  }
  if (kSep && ok && it > 0) {
    // the last block's dQ
    const int q_last = (i0 + it - 1) * kBlk;
    if (tid == 0) bulk_wait_group_read0();
    __syncthreads();
    {
#pragma unroll
      for (int c = 0; c < DP / 32; ++c) {
        if ((c & 1) != half && DP > 32) continue;
        if (DP == 32 && half != 0) continue;
        uint32_t raw[32];
        tmem_ld_32x32(tmem + kColDQ + ((it - 1) & 1) * 64 + lane_base + c * 32, raw);
        tmem_wait_ld_for(raw);
        float4* dst = reinterpret_cast<float4*>(dq_stage + r * DP + c * 32);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          dst[j] = make_float4(__uint_as_float(raw[4 * j]), __uint_as_float(raw[4 * j + 1]),
                               __uint_as_float(raw[4 * j + 2]), __uint_as_float(raw[4 * j + 3]));
      }
      fence_proxy_async();
      tc_fence_before();
      __syncthreads();
      if (tid == 0) {
        const int qvalid = min(kBlk, p.T - q_last);
        float* gdst = p.dq_acc + ((static_cast<int64_t>(b) * p.H + h) * p.T + q_last) * DP;
        bulk_reduce_add_f32(gdst, dq_stage, static_cast<uint32_t>(qvalid) * DP * 4);
        bulk_commit_group();
      }
    }
  }
  if (trb) attn_trace(p.trace, 0, ntr, 8);
  if (tid == 0) bulk_wait_group0();
  __syncthreads();          // the last reduction has read its staging area, which the rows below may reuse
  if (trb) attn_trace(p.trace, 0, ntr, 9);

  if (ok && it > 0) {
    // dK (threads of half 0) and dV (half 1): rows go through shared memory (P / dS are free now) so that each global
    // store instruction writes one row's contiguous bytes instead of one column of 32 rows that lie kilobytes apart
    const int wq = warp & 3, lane = tid & 31;
    T* stage = reinterpret_cast<T*>(half == 0 ? p_img : ds_img) + wq * 32 * DP;      // this warp's [32][DP]
    const uint32_t col = half == 0 ? kColDK : kColDV;
#pragma unroll
    for (int c = 0; c < DP / 32; ++c) {
      uint32_t raw[32];
      tmem_ld_32x32(tmem + col + lane_base + c * 32, raw);
      tmem_wait_ld_for(raw);
      uint4* d4 = reinterpret_cast<uint4*>(stage + lane * DP + c * 32);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 u;
        u.x = pack_pair<T>(__uint_as_float(raw[q * 8 + 0]), __uint_as_float(raw[q * 8 + 1]));
        u.y = pack_pair<T>(__uint_as_float(raw[q * 8 + 2]), __uint_as_float(raw[q * 8 + 3]));
        u.z = pack_pair<T>(__uint_as_float(raw[q * 8 + 4]), __uint_as_float(raw[q * 8 + 5]));
        u.w = pack_pair<T>(__uint_as_float(raw[q * 8 + 6]), __uint_as_float(raw[q * 8 + 7]));
        d4[q] = u;
      }
    }
    __syncwarp();
    const int row0 = k0 + wq * 32;
    const int rows = min(32, p.T - row0);
    T* dst = reinterpret_cast<T*>(p.dqkv) + (static_cast<int64_t>(b) * p.T + row0) * ld + h * 3 * p.dh + (half == 0 ? p.dh : 2 * p.dh);
    for (int d = lane; d < p.dh; d += 32) {
      for (int r0 = 0; r0 < rows; r0 += 8) {
        T v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = stage[min(r0 + u, 31) * DP + d];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (r0 + u < rows) dst[(r0 + u) * ld + d] = v[u];
      }
    }
  } else if (ok && half == 0 && k0 + r < p.T) {
    // no query block attends to this key block (cannot happen for causal / full attention, kept for safety)
    T* dst = reinterpret_cast<T*>(p.dqkv) + (static_cast<int64_t>(b) * p.T + k0 + r) * ld + h * 3 * p.dh;
    for (int d = 0; d < p.dh; ++d) { dst[p.dh + d] = from_f<T>(0.f); dst[2 * p.dh + d] = from_f<T>(0.f); }
  }
  if (*abort_flag) {
    for (int i = 0; i < 32; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (trb) attn_trace(p.trace, 0, ntr, 10);
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// P and dS of 16 scores of a row as packed 16-bit pairs, kept in registers: p = exp2(s*sc2 + bias - lse),
// ds = p * (dp - delta) * scale.  `pk` / `dk` point at the 8 words of this half of the thread's chunk.
template <bool MASKED, bool BIAS, typename T>
__device__ __forceinline__ void bwd_half_regs(const uint32_t (&rs)[16], const uint32_t (&rp)[16], const float* bias, float sc2,
                                              float lse2, float scale, float nds, int key0, int q_idx, int Tn, bool causal,
                                              uint32_t* pk, uint32_t* dk) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    float bv[4] = {0.f, 0.f, 0.f, 0.f};
    if (BIAS) {
      const float4 t = reinterpret_cast<const float4*>(bias)[q];    // a broadcast load: all lanes read the same keys
      bv[0] = t.x; bv[1] = t.y; bv[2] = t.z; bv[3] = t.w;
    }
    float pr[4], ds[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int e = 4 * q + u;
      float v = ex2_approx(fmaf(__uint_as_float(rs[e]), sc2, BIAS ? bv[u] - lse2 : -lse2));
      if (MASKED) {
        const int key = key0 + e;
        if (key >= Tn || q_idx >= Tn || (causal && key > q_idx)) v = 0.f;
      }
      pr[u] = v;
      ds[u] = v * fmaf(__uint_as_float(rp[e]), scale, nds);
    }
    pk[2 * q] = pack_pair<T>(pr[0], pr[1]);
    pk[2 * q + 1] = pack_pair<T>(pr[2], pr[3]);
    dk[2 * q] = pack_pair<T>(ds[0], ds[1]);
    dk[2 * q + 1] = pack_pair<T>(ds[2], ds[3]);
  }
}
// Write 32 consecutive columns [c0, c0+32) of row r of a [128 x 128] 16-bit image from packed pairs.
__device__ __forceinline__ void store_packed_chunk(uint8_t* img, int r, int c0, const uint32_t (&pk)[16]) {
#pragma unroll
  for (int q = 0; q < 4; ++q)
    *reinterpret_cast<uint4*>(img + img_off(r, c0 + q * 8)) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
}

// ------------------------------------------------------------------------------------------------
// Backward for head dims up to 64: persistent, warp-specialised.  Sixteen compute warps (four threads per query row,
// one per 32-key chunk: four warps per scheduler cover each other's TMEM and exponential latencies), two MMA-issuing
// warps and one TMA warp per CTA; CTAs take (key block, head, batch) work items from a global counter in
// (batch, head)-major order, so the key blocks that add into the same dQ rows run at about the same time and the
// fp32 accumulator stays in L2.  Per (query block, key block) pair nobody meets at a CTA-wide barrier:
//   MMA warp A:  S_{i+1}, dP_{i+1} are issued as soon as the compute warps have read S_i, dP_i out of TMEM (for the
//                last block of an item: the first scores of the next item, whose K / V sit in the other buffer), ahead
//                of dQ_i = dS K, which waits for dS_i in shared memory.
//   MMA warp B:  dV += P^T dO and dK += dS^T Q (issuing the 24 narrow MMAs of a block from one thread took a
//                microsecond).  The completion of both warps' products frees P / dS and the Q / dO ring slot and
//                publishes dQ_i.
//   compute:     read S_i / dP_i, build P_i / dS_i in registers while the previous block's products still read the
//                P / dS images, then store them.  The warps of chunks 2 and 3 own a staging block each: alternately
//                they move dQ_{i-1} from TMEM through it (in the 128-byte swizzle, no bank conflicts) into the fp32
//                accumulator with a TMA reduce-add, under the same proxy fence as P / dS, and at the end of an item
//                they write dK and dV.
//   TMA warp:    K / V (double-buffered for a padded head dim of 32) and the key bias of the next item, Q / dO blocks
//                through a ring of two.
// TMEM columns: S [0,128) dP [128,256) dV [256,..) dK [320,..) dQ [384,..) and [448,..) alternately.
// Trace codes (thread 256 of CTA 0, row 0): 1 block start, 2 scores there, 3 P / dS in registers, 31 previous products
// done, 32 P / dS stored, 33 dQ staged, 4 published, 5 last products done, 6 last dQ out, 7 dK / dV out; row 1 (MMA
// warp A): 10 item, 11 first scores issued, 12 block, 13 next scores issued, 14 P / dS ready, 15 dQ issued.
constexpr int kBwsThreads = 608;   // 16 compute warps, two MMA-issuing warps, one TMA warp
struct BwsBars {
  uint64_t kv_full[2], kv_empty[2];   // by K / V buffer
  uint64_t qdo_full[2], qdo_empty[2];
  uint64_t s_full, s_free, p_ready, pds_free, dkv_free;
  int item[2];               // work item by parity of its sequence number; -1: none left
  int bias_nz[2];            // the key bias of that item has a non-zero entry
};
template <int DP>
constexpr int bwd_ws_kv_bufs() { return DP == 32 ? 2 : 1; }
template <int DP>
constexpr int bwd_ws_smem() {
  return (4 + 2 * bwd_ws_kv_bufs<DP>()) * kBlk * 128 + 4 * kBlk * 128 + 2 * kBlk * DP * 4 + 2 * kBlk * 4 + 256 + 1024;
}
static_assert(bwd_ws_smem<32>() <= 232448 && bwd_ws_smem<64>() <= 232448, "shared memory of the persistent backward");

template <typename T, int DP>
__global__ void __launch_bounds__(kBwsThreads, 1)
attn_bwd_ws_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                   const __grid_constant__ CUtensorMap map_dq, AttnParams p) {
  static_assert(DP == 32 || DP == 64, "one 64-column image per operand");
  constexpr int kImg = kBlk * 128;                 // 16 KB: a [128 x 64] 16-bit image
  constexpr int kPImg = 2 * kBlk * 128;            // 32 KB: a [128 x 128] 16-bit image
  constexpr uint32_t kColDV = 256, kColDK = 320, kColDQ = 384;
  // K / V are double-buffered where shared memory allows: the next item's K / V and first scores are then under way
  // before this item's last products have been issued
  constexpr int KVB = bwd_ws_kv_bufs<DP>();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_img = smem;                           // [KVB]
  uint8_t* v_img = k_img + KVB * kImg;             // [KVB]
  uint8_t* q_img0 = v_img + KVB * kImg;            // [2]
  uint8_t* do_img0 = q_img0 + 2 * kImg;            // [2]
  uint8_t* p_img = do_img0 + 2 * kImg;
  uint8_t* ds_img = p_img + kPImg;
  float* dq_stage = reinterpret_cast<float*>(ds_img + kPImg);        // [8 compute warps][32][DP]
  float* s_bias = dq_stage + 2 * kBlk * DP;                          // [2][128], log2 domain
  BwsBars* bars = reinterpret_cast<BwsBars*>(s_bias + 2 * kBlk);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) { mbar_init(&bars->kv_full[i], 1); mbar_init(&bars->kv_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bars->qdo_full[i], 1); mbar_init(&bars->qdo_empty[i], 2); }
    mbar_init(&bars->s_full, 1); mbar_init(&bars->s_free, 16); mbar_init(&bars->p_ready, 16);
    mbar_init(&bars->pds_free, 2); mbar_init(&bars->dkv_free, 8);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 16) {
    __syncwarp();
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  const int n_q = (p.T + kBlk - 1) / kBlk;
  const int total = n_q * p.H * p.B;
  // item t: key block t % n_q (for a causal mask the block with the most query blocks first), head, batch
  auto n_it_of = [&](int kb) { return p.causal ? n_q - kb : n_q; };

  if (warp == 18) {
    // =========================================================================== TMA producer (+ key bias)
    int g = 0;
    for (int n = 0;; ++n) {
      int t = 0;
      bool ok = true;
      if (lane == 0) {
        t = atomicAdd(p.work_counter, 1);
        if (t >= total) t = -1;
      }
      t = __shfl_sync(0xffffffffu, t, 0);
      const int kb = t < 0 ? 0 : t % n_q, bh = t < 0 ? 0 : t / n_q, h = bh % p.H, b = bh / p.H;
      const int n_it = n_it_of(kb), i0 = n_q - n_it;
      // the bias values are requested before the wait below
      float bvals[4] = {0.f, 0.f, 0.f, 0.f};
      if (p.key_bias != nullptr && t >= 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int key = kb * kBlk + lane * 4 + i;
          if (key < p.T) bvals[i] = p.key_bias[static_cast<int64_t>(b) * p.T + key] * kLog2e;
        }
      }
      // the K / V buffer, the bias slot and the item slot that this item takes are no longer read
      if (lane == 0 && n >= KVB) ok = mbar_wait_ol(&bars->kv_empty[n % KVB], (n / KVB - 1) & 1, abort_flag, p.status, n);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (t < 0) {
        if (lane == 0) { bars->item[n & 1] = -1; mbar_arrive(&bars->kv_full[n % KVB]); }
        break;
      }
      if (p.key_bias != nullptr) {
        float* dst = s_bias + (n & 1) * kBlk;
        bool nz = false;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float bv = bvals[i];
          dst[lane * 4 + i] = bv;
          nz = nz || bv != 0.f;
        }
        // an all-zero bias (no padding among these keys) lets the compute warps skip it
        const bool any_nz = __any_sync(0xffffffffu, nz);
        if (lane == 0) bars->bias_nz[n & 1] = any_nz ? 1 : 0;
        __threadfence_block();
      }
      __syncwarp();
      if (lane == 0) {
        bars->item[n & 1] = t;
        mbar_expect_tx(&bars->kv_full[n % KVB], 2 * kImg);
        tma_load_4d(k_img + (n % KVB) * kImg, &map_k, &bars->kv_full[n % KVB], 0, kb * kBlk, h, b);
        tma_load_4d(v_img + (n % KVB) * kImg, &map_v, &bars->kv_full[n % KVB], 0, kb * kBlk, h, b);
        for (int it = 0; it < n_it; ++it) {
          const int gi = g + it, slot = gi & 1;
          if (gi >= 2) ok = mbar_wait_ol(&bars->qdo_empty[slot], ((gi >> 1) - 1) & 1, abort_flag, p.status, gi);
          if (!ok) break;
          mbar_expect_tx(&bars->qdo_full[slot], 2 * kImg);
          tma_load_4d(q_img0 + slot * kImg, &map_q, &bars->qdo_full[slot], 0, (i0 + it) * kBlk, h, b);
          tma_load_4d(do_img0 + slot * kImg, &map_do, &bars->qdo_full[slot], 0, (i0 + it) * kBlk, h, b);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      g += n_it;
      if (p.trace != nullptr && lane == 0) {
        // per-CTA totals in the third trace row: (items, blocks), (first item taken, last item taken)
        long long* e = p.trace + (static_cast<size_t>(2) * 4096 + 2 * blockIdx.x) * 2;
        const long long now = static_cast<long long>(globaltimer_ns());
        if (n == 0) e[2] = now;
        e[0] = n + 1; e[1] = g; e[3] = now;
      }
    }
  } else if (warp == 16) {
    // =========================================================================== MMA issuer A: S, dP and dQ
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_f16(kBlk, kBlk, false, false, p.is_bf16);     // Q K^T, dO V^T
      const uint32_t idesc_dq = make_idesc_f16(kBlk, DP, false, true, p.is_bf16);       // dS K
      const uint32_t dsa = smem_u32(ds_img);
      auto issue_scores = [&](int gi, int kvb) -> bool {
        const int slot = gi & 1;
        const uint32_t ka = smem_u32(k_img + kvb * kImg), va = smem_u32(v_img + kvb * kImg);
        if (gi > 0 && !mbar_wait_ol(&bars->s_free, (gi - 1) & 1, abort_flag, p.status, gi)) return false;
        if (!mbar_wait_ol(&bars->qdo_full[slot], (gi >> 1) & 1, abort_flag, p.status, gi)) return false;
        tc_fence_after();
        const uint32_t qa = smem_u32(q_img0 + slot * kImg), da = smem_u32(do_img0 + slot * kImg);
#pragma unroll
        for (int k16 = 0; k16 < DP / 16; ++k16) tc_mma_f16(tmem, kmajor_desc(qa, k16), kmajor_desc(ka, k16), idesc_s, k16 > 0);
#pragma unroll
        for (int k16 = 0; k16 < DP / 16; ++k16) tc_mma_f16(tmem + 128, kmajor_desc(da, k16), kmajor_desc(va, k16), idesc_s, k16 > 0);
        tc_commit(&bars->s_full);
        return true;
      };
      int g = 0, mtr = 0;
      bool ok = true, have_first = false;            // the scores of block g have been issued already
      for (int n = 0; ok; ++n) {
        if (!mbar_wait_ol(&bars->kv_full[n % KVB], (n / KVB) & 1, abort_flag, p.status, n)) break;
        const int t = bars->item[n & 1];
        if (t < 0) break;
        const int n_it = n_it_of(t % n_q);
        const int kvb = n % KVB;
        const uint32_t ka = smem_u32(k_img + kvb * kImg);
        attn_trace(p.trace, 1, mtr, 10);
        if (!have_first) ok = issue_scores(g, kvb);
        have_first = false;
        attn_trace(p.trace, 1, mtr, 11);
        for (int it = 0; it < n_it && ok; ++it) {
          const int gi = g + it, slot = gi & 1;
          attn_trace(p.trace, 1, mtr, 12);
          if (it + 1 < n_it) {
            ok = issue_scores(gi + 1, kvb);
            if (!ok) break;
          } else if (KVB == 2) {
            // the first scores of the next item, whose K / V sit in the other buffer
            if (!mbar_wait_ol(&bars->kv_full[(n + 1) % KVB], ((n + 1) / KVB) & 1, abort_flag, p.status, n)) { ok = false; break; }
            if (bars->item[(n + 1) & 1] >= 0) {
              ok = issue_scores(gi + 1, (n + 1) % KVB);
              if (!ok) break;
              have_first = true;
            }
          }
          attn_trace(p.trace, 1, mtr, 13);
          ok = mbar_wait_ol(&bars->p_ready, gi & 1, abort_flag, p.status, gi);
          if (!ok) break;
          tc_fence_after();
          attn_trace(p.trace, 1, mtr, 14);
#pragma unroll
          for (int k16 = 0; k16 < kBlk / 16; ++k16)   // dQ[q, d] = sum_key dS[q, key] K[key, d]
            tc_mma_f16(tmem + kColDQ + slot * 64, kmajor_desc(dsa, k16), mnmajor_desc(ka, k16), idesc_dq, k16 > 0);
          tc_commit(&bars->pds_free);
          tc_commit(&bars->qdo_empty[slot]);           // covers S / dP of this block as well
          if (it == n_it - 1) tc_commit(&bars->kv_empty[kvb]);
          attn_trace(p.trace, 1, mtr, 15);
        }
        g += n_it;
      }
    }
  } else if (warp == 17) {
    // =========================================================================== MMA issuer B: dV and dK
    if (lane == 0) {
      const uint32_t idesc_tt = make_idesc_f16(kBlk, DP, true, true, p.is_bf16);        // P^T dO, dS^T Q
      const uint32_t pa = smem_u32(p_img), dsa = smem_u32(ds_img);
      int g = 0;
      bool ok = true;
      for (int n = 0; ok; ++n) {
        if (!mbar_wait_ol(&bars->kv_full[n % KVB], (n / KVB) & 1, abort_flag, p.status, n)) break;
        const int t = bars->item[n & 1];
        if (t < 0) break;
        const int n_it = n_it_of(t % n_q);
        for (int it = 0; it < n_it && ok; ++it) {
          const int gi = g + it, slot = gi & 1;
          ok = mbar_wait_ol(&bars->qdo_full[slot], (gi >> 1) & 1, abort_flag, p.status, gi) &&
               mbar_wait_ol(&bars->p_ready, gi & 1, abort_flag, p.status, gi);
          // the compute warps have read the previous item's dK / dV out of TMEM
          if (ok && it == 0 && n > 0) ok = mbar_wait_ol(&bars->dkv_free, (n - 1) & 1, abort_flag, p.status, n);
          if (!ok) break;
          tc_fence_after();
          const uint32_t qa = smem_u32(q_img0 + slot * kImg), da = smem_u32(do_img0 + slot * kImg);
          const uint32_t acc = it > 0 ? 1u : 0u;
#pragma unroll
          for (int k16 = 0; k16 < kBlk / 16; ++k16)   // dV[key, d] += sum_q P[q, key] dO[q, d]
            tc_mma_f16(tmem + kColDV, mnmajor_desc(pa, k16), mnmajor_desc(da, k16), idesc_tt, (k16 > 0) ? 1u : acc);
#pragma unroll
          for (int k16 = 0; k16 < kBlk / 16; ++k16)   // dK[key, d] += sum_q dS[q, key] Q[q, d]
            tc_mma_f16(tmem + kColDK, mnmajor_desc(dsa, k16), mnmajor_desc(qa, k16), idesc_tt, (k16 > 0) ? 1u : acc);
          tc_commit(&bars->pds_free);
          tc_commit(&bars->qdo_empty[slot]);
        }
        g += n_it;
      }
    }
  } else {
    // =========================================================================== compute warps
    // Four threads per query row, one per 32-key chunk of the block (sixteen warps: four per scheduler, so that the
    // TMEM and exponential latencies of one warp are covered by the others).  The warps of chunks 2 and 3 also own a
    // staging block each: they write out dQ (alternately, block by block) and, at the end of an item, dK and dV.
    const int r = tid & 127;                         // query row inside a block == TMEM lane
    const int qt = tid >> 7;                         // this thread's 32-key chunk of the block
    const int wq = warp & 3;                         // this warp's 32-row block
    const bool owner = qt >= 2;
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    const float sc2 = p.scale * kLog2e;
    const int64_t ld = static_cast<int64_t>(p.H) * 3 * p.dh;
    float* stg = dq_stage + (((qt & 1) * 4 + wq) * 32) * DP;   // an owner warp's [32][DP] fp32 staging rows
    int g = 0, ntr = 0;
    bool ok = true;
    long long* tr = tid == 256 ? p.trace : nullptr;   // an owner thread

    // dQ of global block gi (TMEM column set gi & 1) -> this warp's staging rows: boxes of 32 rows x 128 bytes in the
    // 128-byte swizzle of the tensor map (16-byte chunk j of row l sits at chunk j ^ (l & 7): no bank conflicts)
    auto dq_ld = [&](int gi, int c, uint32_t (&raw)[32]) {
      tmem_ld_32x32(tmem + kColDQ + (gi & 1) * 64 + lane_base + c * 32, raw);
    };
    auto dq_st = [&](int c, uint32_t (&raw)[32]) {
      tmem_wait_ld_for(raw);
      uint8_t* row = reinterpret_cast<uint8_t*>(stg) + c * 4096 + lane * 128;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<uint4*>(row + ((j ^ (lane & 7)) << 4)) = make_uint4(raw[4 * j], raw[4 * j + 1], raw[4 * j + 2], raw[4 * j + 3]);
    };
    // staging rows -> fp32 accumulator by TMA reduce-add (lane 0, after the warp's proxy fences and __syncwarp)
    auto dq_reduce = [&](int h, int b, int q_first) {
      const int row0 = q_first + wq * 32;
      if (row0 < p.T) {
        // rows past the sequence end carry exact zeros (their dS is zero), so a box that overlaps them adds nothing
        const int grow = (b * p.H + h) * p.T + row0;
#pragma unroll
        for (int c = 0; c < DP / 32; ++c) tma_reduce_add_2d(&map_dq, reinterpret_cast<uint8_t*>(stg) + c * 4096, c * 32, grow);
      }
      bulk_commit_group();
    };

    for (int n = 0; ok; ++n) {
      if (!mbar_wait_ol(&bars->kv_full[n % KVB], (n / KVB) & 1, abort_flag, p.status, n)) { ok = false; break; }
      const int t = bars->item[n & 1];
      if (t < 0) break;
      const int kb = t % n_q, bh = t / n_q, h = bh % p.H, b = bh / p.H;
      const int k0 = kb * kBlk;
      const int n_it = n_it_of(kb), i0 = n_q - n_it;
      const bool has_bias = p.key_bias != nullptr && bars->bias_nz[n & 1] != 0;
      const float* sbias = s_bias + (n & 1) * kBlk + qt * 32;
      const int64_t stat0 = (static_cast<int64_t>(b) * p.H + h) * p.T;
      // row statistics of the first block; those of block it + 1 are requested while block it is processed
      float lse_nx = 0.f, dl_nx = 0.f;
      if (i0 * kBlk + r < p.T) { lse_nx = p.lse[stat0 + i0 * kBlk + r]; dl_nx = p.delta[stat0 + i0 * kBlk + r]; }
      for (int it = 0; it < n_it; ++it) {
        const int gi = g + it, i = i0 + it, q0 = i * kBlk;
        const int q_idx = q0 + r;
        const float lse2 = lse_nx;
        const float nds = -dl_nx * p.scale;
        lse_nx = 0.f; dl_nx = 0.f;
        if (it + 1 < n_it && q_idx + kBlk < p.T) { lse_nx = p.lse[stat0 + q_idx + kBlk]; dl_nx = p.delta[stat0 + q_idx + kBlk]; }
        // the owner warps of chunk 2 + ((gi - 1) & 1) write out the previous block's dQ
        const bool my_dq = it > 0 && owner && ((gi - 1) & 1) == (qt & 1);
        attn_trace(tr, 0, ntr, 1);
        if (!mbar_wait_ol(&bars->s_full, gi & 1, abort_flag, p.status, gi)) { ok = false; break; }
        tc_fence_after();
        attn_trace(tr, 0, ntr, 2);
        const bool tail = (k0 + kBlk > p.T) || (q0 + kBlk > p.T);
        const bool cdiag = p.causal && i == kb;
        // P / dS of this thread's chunk are computed into registers while the products of the previous block still
        // read the P / dS images; they are stored once those products are done.
        // Diagonal block of a causal mask: key chunks left of this warp's rows are plain, the chunk on the diagonal is
        // tested key by key, chunks to the right are zero.  Blocks that reach past the sequence end are tested everywhere.
        uint32_t pk[16], dk[16];
        if (!tail && cdiag && qt > wq) {
#pragma unroll
          for (int j = 0; j < 16; ++j) { pk[j] = 0u; dk[j] = 0u; }
        } else {
          const bool masked = tail || (cdiag && qt == wq);
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            uint32_t rs[16], rp[16];
            tmem_ld_32x16(tmem + lane_base + qt * 32 + hf * 16, rs);
            tmem_ld_32x16(tmem + 128 + lane_base + qt * 32 + hf * 16, rp);
            tmem_wait_ld_for(rs);
            tmem_wait_ld_for(rp);
            if (!masked) {
              if (has_bias) bwd_half_regs<false, true, T>(rs, rp, sbias + hf * 16, sc2, lse2, p.scale, nds, 0, 0, 0, false, pk + hf * 8, dk + hf * 8);
              else bwd_half_regs<false, false, T>(rs, rp, nullptr, sc2, lse2, p.scale, nds, 0, 0, 0, false, pk + hf * 8, dk + hf * 8);
            } else {
              if (has_bias) bwd_half_regs<true, true, T>(rs, rp, sbias + hf * 16, sc2, lse2, p.scale, nds, k0 + qt * 32 + hf * 16, q_idx, p.T, cdiag, pk + hf * 8, dk + hf * 8);
              else bwd_half_regs<true, false, T>(rs, rp, nullptr, sc2, lse2, p.scale, nds, k0 + qt * 32 + hf * 16, q_idx, p.T, cdiag, pk + hf * 8, dk + hf * 8);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->s_free);     // last read of S / dP: the next block's scores may overwrite them
        attn_trace(tr, 0, ntr, 3);
        // the products of the previous block have finished reading P / dS, and its dQ is complete
        if (gi > 0 && !mbar_wait_ol(&bars->pds_free, (gi - 1) & 1, abort_flag, p.status, gi)) ok = false;
        tc_fence_after();
        attn_trace(tr, 0, ntr, 31);
        const bool drain = my_dq && ok;
        store_packed_chunk(p_img, r, qt * 32, pk);
        store_packed_chunk(ds_img, r, qt * 32, dk);
        attn_trace(tr, 0, ntr, 32);
        if (drain) {
          uint32_t dq_raw[32];
          if (lane == 0) bulk_wait_group_read0();      // the previous reduction has read the staging rows
          __syncwarp();
          dq_ld(gi - 1, 0, dq_raw);
          dq_st(0, dq_raw);
          if constexpr (DP == 64) {
            dq_ld(gi - 1, 1, dq_raw);
            dq_st(1, dq_raw);
          }
          tc_fence_before();
        }
        attn_trace(tr, 0, ntr, 33);
        fence_proxy_async();                         // P / dS (and the staged dQ) become visible to the async proxy
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bars->p_ready);
          if (drain) dq_reduce(h, b, q0 - kBlk);
        }
        if (!ok) break;
        attn_trace(tr, 0, ntr, 4);
      }
      if (!ok) break;
      g += n_it;
      if (!owner) continue;
      // ---- owner warps: the item's last dQ, then its dK (chunk 2's warps) / dV (chunk 3's warps)
      const int g_last = g - 1;
      if (!mbar_wait_ol(&bars->pds_free, g_last & 1, abort_flag, p.status, g_last)) { ok = false; break; }
      tc_fence_after();
      attn_trace(tr, 0, ntr, 5);
      if ((g_last & 1) == (qt & 1)) {
        uint32_t dq_raw[32];
        if (lane == 0) bulk_wait_group_read0();
        __syncwarp();
#pragma unroll
        for (int c = 0; c < DP / 32; ++c) {
          dq_ld(g_last, c, dq_raw);
          dq_st(c, dq_raw);
        }
        tc_fence_before();
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) dq_reduce(h, b, (i0 + n_it - 1) * kBlk);
      }
      attn_trace(tr, 0, ntr, 6);
      {
        // rows go through the warp's staging block so that each global store instruction writes one row's contiguous
        // bytes instead of one column of 32 rows that lie kilobytes apart
        uint32_t raw[32];
        const uint32_t col = qt == 2 ? kColDK : kColDV;
        tmem_ld_32x32(tmem + col + lane_base, raw);
        if (lane == 0) bulk_wait_group_read0();      // the reduction that reads the staging block has done so
        __syncwarp();
        T* stage = reinterpret_cast<T*>(stg);        // [32][DP]
#pragma unroll
        for (int c = 0; c < DP / 32; ++c) {
          if (c > 0) tmem_ld_32x32(tmem + col + lane_base + c * 32, raw);
          tmem_wait_ld_for(raw);
          uint4* d4 = reinterpret_cast<uint4*>(stage + lane * DP + c * 32);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 u;
            u.x = pack_pair<T>(__uint_as_float(raw[q * 8 + 0]), __uint_as_float(raw[q * 8 + 1]));
            u.y = pack_pair<T>(__uint_as_float(raw[q * 8 + 2]), __uint_as_float(raw[q * 8 + 3]));
            u.z = pack_pair<T>(__uint_as_float(raw[q * 8 + 4]), __uint_as_float(raw[q * 8 + 5]));
            u.w = pack_pair<T>(__uint_as_float(raw[q * 8 + 6]), __uint_as_float(raw[q * 8 + 7]));
            d4[q] = u;
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->dkv_free);   // the next item's products may overwrite the accumulators
        const int row0 = k0 + wq * 32;
        const int rows = min(32, p.T - row0);
        T* dst = reinterpret_cast<T*>(p.dqkv) + (static_cast<int64_t>(b) * p.T + row0) * ld + h * 3 * p.dh + (qt == 2 ? p.dh : 2 * p.dh);
        for (int d = lane; d < p.dh; d += 32) {
          for (int r0 = 0; r0 < rows; r0 += 8) {
            T v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = stage[min(r0 + u, 31) * DP + d];
#pragma unroll
            for (int u = 0; u < 8; ++u)
              if (r0 + u < rows) dst[(r0 + u) * ld + d] = v[u];
          }
        }
        __syncwarp();                                // the rows have been read before the block is staged into again
      }
      attn_trace(tr, 0, ntr, 7);
    }
    if (lane == 0) bulk_wait_group0();
    if (!ok) *abort_flag = 1;
  }

  if (*abort_flag) {
    for (int i = 0; i < 32; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 16) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------------ host side
static int padded_dim(int dh) {
  TORCH_CHECK(dh >= 1 && dh <= 128, "head dimension must be in [1, 128]");
  return dh <= 32 ? 32 : dh <= 64 ? 64 : dh <= 96 ? 96 : 128;
}
template <int DP>
constexpr int fwd_smem() { return 3 * ((DP + 63) / 64) * kBlk * 128 + 2 * kBlk * 128 + 64 + 1024 + 1024; }
template <int DP>
constexpr int bwd_smem() {
  return (DP <= 64 ? 6 : 4) * ((DP + 63) / 64) * kBlk * 128 + 4 * kBlk * 128 + 64 + 1024 + 512 +
         (DP <= 64 ? kBlk * DP * 4 : 0);
}

struct AttnMaps {
  CUtensorMap q, k, v, d_out;
  CUtensorMap dq;   // fp32 dQ accumulator [B*H*T, DP] (persistent backward)
};

template <typename T, int DP>
static void launch_fwd_ws(const AttnMaps& m, const AttnParams& p, cudaStream_t s) {
  auto kern = attn_fwd_ws_kernel<T, DP>;
  static bool done = false;
  if (!done) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, fwd_ws_smem<DP>()));
    done = true;
  }
  const int tiles = ((p.T + kBlk - 1) / kBlk) * p.H * p.B;
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  kern<<<std::min(tiles, sms), kWsThreads, fwd_ws_smem<DP>(), s>>>(m.q, m.k, m.v, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

template <typename T, int DP>
static void launch_fwd(const AttnMaps& m, const AttnParams& p, cudaStream_t s) {
  if constexpr (DP <= 64) {
    launch_fwd_ws<T, DP>(m, p, s);
    return;
  }
  auto kern = attn_fwd_kernel<T, DP>;
  static bool done = false;
  if (!done) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, fwd_smem<DP>()));
    done = true;
  }
  dim3 grid((p.T + kBlk - 1) / kBlk, p.H, p.B);
  kern<<<grid, kAttnThreads, fwd_smem<DP>(), s>>>(m.q, m.k, m.v, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}
template <typename T, int DP>
static void launch_bwd(const AttnMaps& m, const AttnParams& p, cudaStream_t s) {
  if constexpr (DP <= 64) {
    auto kern = attn_bwd_ws_kernel<T, DP>;
    static bool done = false;
    if (!done) {
      C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bwd_ws_smem<DP>()));
      done = true;
    }
    const int items = ((p.T + kBlk - 1) / kBlk) * p.H * p.B;
    const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    kern<<<std::min(items, sms), kBwsThreads, bwd_ws_smem<DP>(), s>>>(m.q, m.k, m.v, m.d_out, m.dq, p);
  } else {
    auto kern = attn_bwd_kernel<T, DP>;
    static bool done = false;
    if (!done) {
      C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bwd_smem<DP>()));
      done = true;
    }
    dim3 grid((p.T + kBlk - 1) / kBlk, p.H, p.B);
    kern<<<grid, kBwdThreads, bwd_smem<DP>(), s>>>(m.q, m.k, m.v, m.d_out, p);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

#define DISPATCH_ATTN(FN, m, p, stream)                                                    \
  {                                                                                        \
    const int dp_ = padded_dim((p).dh);                                                    \
    if ((p).is_bf16) {                                                                     \
      if (dp_ == 32) FN<__nv_bfloat16, 32>(m, p, stream);                                  \
      else if (dp_ == 64) FN<__nv_bfloat16, 64>(m, p, stream);                             \
      else if (dp_ == 96) FN<__nv_bfloat16, 96>(m, p, stream);                             \
      else FN<__nv_bfloat16, 128>(m, p, stream);                                           \
    } else {                                                                               \
      if (dp_ == 32) FN<__half, 32>(m, p, stream);                                         \
      else if (dp_ == 64) FN<__half, 64>(m, p, stream);                                    \
      else if (dp_ == 96) FN<__half, 96>(m, p, stream);                                    \
      else FN<__half, 128>(m, p, stream);                                                  \
    }                                                                                      \
  }

static AttnParams base_params(const torch::Tensor& qkv, bool causal, const c10::optional<torch::Tensor>& key_bias,
                              double scale, int64_t status_ptr) {
  TORCH_CHECK(qkv.is_cuda() && qkv.dim() == 4 && qkv.is_contiguous() && qkv.size(3) % 3 == 0,
              "qkv must be a contiguous [B, T, heads, 3*dh] CUDA tensor");
  TORCH_CHECK(qkv.scalar_type() == torch::kBFloat16 || qkv.scalar_type() == torch::kFloat16);
  AttnParams p{};
  p.B = qkv.size(0); p.T = qkv.size(1); p.H = qkv.size(2); p.dh = qkv.size(3) / 3;
  p.scale = static_cast<float>(scale);
  TORCH_CHECK(scale > 0.0, "the softmax scale must be positive");
  p.causal = causal ? 1 : 0;
  p.is_bf16 = qkv.scalar_type() == torch::kBFloat16;
  p.status = reinterpret_cast<int*>(status_ptr);
  if (key_bias.has_value() && key_bias->defined()) {
    TORCH_CHECK(key_bias->scalar_type() == torch::kFloat32 && key_bias->is_contiguous() &&
                key_bias->numel() == static_cast<int64_t>(p.B) * p.T, "key_bias must be a contiguous fp32 [B, T]");
    p.key_bias = key_bias->data_ptr<float>();
  }
  return p;
}

// Row width of the padded copy: the TMA box is 64 columns wide whatever the tensor's extent (columns past the extent are
// zero-filled), so a narrow head only needs its rows 16-byte aligned.
static int pack_width(int dh) { return dh <= 32 ? 32 : dh <= 64 ? 64 : 128; }

// [parts][B, H, T, W] zero-padded copy of src [B, T, H, parts*dh].
static torch::Tensor pack_heads(const torch::Tensor& src, int B, int T, int H, int dh, int parts, cudaStream_t stream) {
  const int W = pack_width(dh);
  auto dst = torch::empty({parts, B, H, T, W}, src.options());
  const int64_t total = static_cast<int64_t>(B) * T * H * parts;
  if (src.scalar_type() == torch::kBFloat16) {
    attn_pack_kernel<__nv_bfloat16><<<(total + 127) / 128, 128, 128 * dh * 2, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(src.data_ptr()), reinterpret_cast<__nv_bfloat16*>(dst.data_ptr()), B, T, H, dh,
        parts, W);
  } else {
    attn_pack_kernel<__half><<<(total + 127) / 128, 128, 128 * dh * 2, stream>>>(reinterpret_cast<const __half*>(src.data_ptr()),
                                                                      reinterpret_cast<__half*>(dst.data_ptr()), B, T, H, dh,
                                                                      parts, W);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return dst;
}

// Tensor maps of the three QKV parts, either straight over the packed tensor (dh % 8 == 0) or over `packed`.
static void qkv_maps(AttnMaps& m, const torch::Tensor& qkv, const torch::Tensor& packed, const AttnParams& p) {
  const uint64_t B = p.B, T = p.T, H = p.H, dh = p.dh;
  if (packed.defined()) {
    const uint64_t W = packed.size(4);
    const char* base = reinterpret_cast<const char*>(packed.data_ptr());
    const uint64_t part = B * H * T * W * 2;
    m.q = make_tma_4d(base, W, T, H, B, W * 2, T * W * 2, H * T * W * 2);
    m.k = make_tma_4d(base + part, W, T, H, B, W * 2, T * W * 2, H * T * W * 2);
    m.v = make_tma_4d(base + 2 * part, W, T, H, B, W * 2, T * W * 2, H * T * W * 2);
  } else {
    const char* base = reinterpret_cast<const char*>(qkv.data_ptr());
    const uint64_t st = H * 3 * dh * 2, sh = 3 * dh * 2, sbt = T * H * 3 * dh * 2;
    m.q = make_tma_4d(base, dh, T, H, B, st, sh, sbt);
    m.k = make_tma_4d(base + dh * 2, dh, T, H, B, st, sh, sbt);
    m.v = make_tma_4d(base + 2 * dh * 2, dh, T, H, B, st, sh, sbt);
  }
}

bool attention_ready() { return true; }

// Returns (out, lse, packed): `packed` is the padded QKV copy when one was needed (undefined otherwise); the
// backward takes it back so the copy is made once.
std::vector<torch::Tensor> attention_fwd(torch::Tensor qkv, bool causal, c10::optional<torch::Tensor> key_bias,
                                         double scale, int64_t status_ptr, c10::optional<torch::Tensor> trace) {
  AttnParams p = base_params(qkv, causal, key_bias, scale, status_ptr);
  if (trace.has_value() && trace->defined()) {
    TORCH_CHECK(trace->scalar_type() == torch::kInt64 && trace->numel() >= 2 * 4096 * 2 && trace->is_cuda());
    p.trace = reinterpret_cast<long long*>(trace->data_ptr<int64_t>());
  }
  auto out = torch::empty({p.B, p.T, p.H, p.dh}, qkv.options());
  auto lse = torch::empty({p.B, p.H, p.T}, qkv.options().dtype(torch::kFloat32));
  torch::Tensor packed;
  if (qkv.numel() == 0) return {out, lse, packed};
  auto stream = at::cuda::getCurrentCUDAStream();
  if (p.dh % 8 != 0) packed = pack_heads(qkv, p.B, p.T, p.H, p.dh, 3, stream);
  AttnMaps m;
  qkv_maps(m, qkv, packed, p);
  p.out = out.data_ptr();
  p.lse = lse.data_ptr<float>();
  DISPATCH_ATTN(launch_fwd, m, p, stream)
  return {out, lse, packed};
}

torch::Tensor attention_bwd(torch::Tensor dout, torch::Tensor qkv, torch::Tensor out, torch::Tensor lse, bool causal,
                            c10::optional<torch::Tensor> key_bias, double scale, int64_t status_ptr,
                            c10::optional<torch::Tensor> packed_opt, c10::optional<torch::Tensor> trace) {
  AttnParams p = base_params(qkv, causal, key_bias, scale, status_ptr);
  if (trace.has_value() && trace->defined()) {
    TORCH_CHECK(trace->scalar_type() == torch::kInt64 && trace->numel() >= 2 * 4096 * 2 && trace->is_cuda());
    p.trace = reinterpret_cast<long long*>(trace->data_ptr<int64_t>());
  }
  TORCH_CHECK(p.trace == nullptr || trace->numel() >= 3 * 4096 * 2, "the backward trace has three rows");
  TORCH_CHECK(dout.is_contiguous() && dout.numel() == out.numel() && dout.scalar_type() == qkv.scalar_type());
  auto dqkv = torch::empty_like(qkv);
  if (qkv.numel() == 0) return dqkv;
  auto f32 = qkv.options().dtype(torch::kFloat32);
  auto delta = torch::empty({p.B, p.H, p.T}, f32);
  const int DPh = padded_dim(p.dh);
  // fp32 dQ accumulator [B, H, T, DPh], followed by the work counter of the persistent kernel (zeroed with it)
  const int64_t dq_elems = static_cast<int64_t>(p.B) * p.H * p.T * DPh;
  auto dq_acc = torch::zeros({dq_elems + 32}, f32);
  auto stream = at::cuda::getCurrentCUDAStream();
  const int64_t rows = static_cast<int64_t>(p.B) * p.T * p.H;
  const int dthreads = p.dh > 64 ? 64 : 128;       // 4 * dh bytes of shared memory per thread, 48 KB per CTA at most
  if (p.is_bf16) {
    attn_delta_kernel<__nv_bfloat16><<<(rows + dthreads - 1) / dthreads, dthreads, dthreads * p.dh * 4, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(dout.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(out.data_ptr()),
        delta.data_ptr<float>(), p.B, p.T, p.H, p.dh);
  } else {
    attn_delta_kernel<__half><<<(rows + dthreads - 1) / dthreads, dthreads, dthreads * p.dh * 4, stream>>>(
        reinterpret_cast<const __half*>(dout.data_ptr()), reinterpret_cast<const __half*>(out.data_ptr()),
        delta.data_ptr<float>(), p.B, p.T, p.H, p.dh);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  torch::Tensor packed, packed_do;
  if (p.dh % 8 != 0) {
    packed = (packed_opt.has_value() && packed_opt->defined()) ? *packed_opt : pack_heads(qkv, p.B, p.T, p.H, p.dh, 3, stream);
    packed_do = pack_heads(dout, p.B, p.T, p.H, p.dh, 1, stream);
  }
  AttnMaps m;
  qkv_maps(m, qkv, packed, p);
  {
    const uint64_t B = p.B, T = p.T, H = p.H, dh = p.dh;
    if (packed_do.defined()) {
      const uint64_t W = packed_do.size(4);
      m.d_out = make_tma_4d(packed_do.data_ptr(), W, T, H, B, W * 2, T * W * 2, H * T * W * 2);
    } else {
      m.d_out = make_tma_4d(dout.data_ptr(), dh, T, H, B, H * dh * 2, dh * 2, T * H * dh * 2);
    }
  }
  if (DPh <= 64)
    m.dq = make_tma_2d_store(dq_acc.data_ptr<float>(), static_cast<uint64_t>(p.B) * p.H * p.T, DPh, DPh, 4, false);
  p.lse = lse.data_ptr<float>();
  p.delta = delta.data_ptr<float>();
  p.dq_acc = dq_acc.data_ptr<float>();
  p.work_counter = reinterpret_cast<int*>(dq_acc.data_ptr<float>() + dq_elems);
  p.dqkv = dqkv.data_ptr();
  DISPATCH_ATTN(launch_bwd, m, p, stream)
  if (p.is_bf16) {
    attn_dq_store_kernel<__nv_bfloat16><<<(rows + 127) / 128, 128, 128 * DPh * 2, stream>>>(
        dq_acc.data_ptr<float>(), reinterpret_cast<__nv_bfloat16*>(dqkv.data_ptr()), p.B, p.T, p.H, p.dh, DPh);
  } else {
    attn_dq_store_kernel<__half><<<(rows + 127) / 128, 128, 128 * DPh * 2, stream>>>(
        dq_acc.data_ptr<float>(), reinterpret_cast<__half*>(dqkv.data_ptr()), p.B, p.T, p.H, p.dh, DPh);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return dqkv;
}

}  // namespace cw
