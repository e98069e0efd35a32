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
// Backward, one CTA per (128-key block, head, batch) looping over query blocks: S and dP = dO V^T in TMEM,
// P / dS written to shared memory, dV += P^T dO and dK += dS^T Q accumulate in TMEM across the loop,
// dQ = dS K is added to an fp32 scratch buffer with red.add (several key blocks contribute to one query block).
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
};

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

// Copy `parts` consecutive [dh] slices per (token, head) of src [B, T, H, parts*dh] into zero-padded rows
// dst [parts][B, H, T, W] (W a multiple of 64): makes every row 16-byte aligned for TMA.
template <typename T>
__global__ void attn_pack_kernel(const T* __restrict__ src, T* __restrict__ dst, int B, int Tn, int H, int dh, int parts,
                                 int W) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t total = static_cast<int64_t>(B) * Tn * H * parts;
  if (idx >= total) return;
  const int part = idx % parts;
  const int64_t bth = idx / parts;
  const int h = bth % H;
  const int64_t bt = bth / H;
  const int t = bt % Tn, b = bt / Tn;
  const T* s = src + bth * parts * dh + part * dh;
  T* d = dst + (((static_cast<int64_t>(part) * B + b) * H + h) * Tn + t) * W;
  for (int c0 = 0; c0 < W; c0 += 8) {
    T tmp[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) tmp[i] = (c0 + i < dh) ? s[c0 + i] : from_f<T>(0.f);
    *reinterpret_cast<uint4*>(d + c0) = *reinterpret_cast<const uint4*>(tmp);
  }
}

// delta[b, h, t] = sum_d dO[b,t,h,d] * O[b,t,h,d]
template <typename T>
__global__ void attn_delta_kernel(const T* __restrict__ dout, const T* __restrict__ out, float* __restrict__ delta, int B,
                                  int Tn, int H, int dh) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(B) * Tn * H) return;
  const int h = idx % H;
  const int64_t bt = idx / H;
  const int t = bt % Tn, b = bt / Tn;
  const T* a = dout + idx * dh;
  const T* o = out + idx * dh;
  float s = 0.f;
  for (int d = 0; d < dh; ++d) s += to_f(a[d]) * to_f(o[d]);
  delta[(static_cast<int64_t>(b) * H + h) * Tn + t] = s;
}

// dqkv[b, t, h, 0:dh] = dq_acc[b, h, t, 0:dh]   (fp32 accumulator, padded to DP columns, head-major)
template <typename T>
__global__ void attn_dq_store_kernel(const float* __restrict__ dq_acc, T* __restrict__ dqkv, int B, int Tn, int H, int dh,
                                     int DP) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(B) * Tn * H * dh) return;
  const int d = idx % dh;
  const int64_t bth = idx / dh;
  const int h = bth % H;
  const int64_t bt = bth / H;
  const int t = bt % Tn, b = bt / Tn;
  dqkv[bth * 3 * dh + d] = from_f<T>(dq_acc[((static_cast<int64_t>(b) * H + h) * Tn + t) * DP + d]);
}

template <typename T, int DP>
__global__ void __launch_bounds__(kAttnThreads)
attn_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do, AttnParams p) {
  constexpr int NB = (DP + 63) / 64;
  constexpr int kImg = NB * kBlk * 128;
  constexpr uint32_t kTmemCols = 512;   // S/dQ: [0,128)  dP: [128,256)  dV: [256,256+DP)  dK: [384,384+DP)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_img = smem;
  uint8_t* v_img = k_img + kImg;
  constexpr int kBufs = NB == 1 ? 2 : 1;          // Q and dO are double-buffered when shared memory allows
  uint8_t* q_img0 = v_img + kImg;
  uint8_t* do_img0 = q_img0 + kBufs * kImg;
  uint8_t* p_img = do_img0 + kBufs * kImg;
  uint8_t* ds_img = p_img + 2 * kBlk * 128;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ds_img + 2 * kBlk * 128);   // 0: S,dP  1: dV,dK,dQ  2: K,V  3,4: Q,dO
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_bias = reinterpret_cast<float*>(tmem_slot + 2);                 // [128] key bias (log2 domain) of this block
  float* dq_stage = reinterpret_cast<float*>(p_img);                       // [128][DP] fp32, aliases P / dS between uses

  const int r = threadIdx.x, warp = r >> 5;
  const int kb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int k0 = kb * kBlk;
  const int64_t ld = static_cast<int64_t>(p.H) * 3 * p.dh;
  const float* kbias = p.key_bias != nullptr ? p.key_bias + static_cast<int64_t>(b) * p.T : nullptr;
  if (kbias != nullptr) s_bias[r] = k0 + r < p.T ? kbias[k0 + r] * kLog2e : 0.f;
  const int n_q = (p.T + kBlk - 1) / kBlk;
  const int i0 = p.causal ? kb : 0;

  if (r == 0) {
    for (int i = 0; i < 5; ++i) mbar_init(&bars[i], 1);
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
  const uint32_t idesc_s = make_idesc_f16(kBlk, kBlk, false, false, p.is_bf16);     // Q K^T, dO V^T
  const uint32_t idesc_tt = make_idesc_f16(kBlk, DP, true, true, p.is_bf16);        // P^T dO, dS^T Q
  const uint32_t idesc_dq = make_idesc_f16(kBlk, DP, false, true, p.is_bf16);       // dS K
  const float sc2 = p.scale * kLog2e;

  bool ok = true;
  int it = 0;
  for (int i = i0; i < n_q && ok; ++i, ++it) {
    const int q0 = i * kBlk;
    const int sb = kBufs == 2 ? (it & 1) : 0;
    const uint32_t qdo_parity = kBufs == 2 ? ((it >> 1) & 1) : (it & 1);
    uint8_t* q_img = q_img0 + sb * kImg;
    uint8_t* do_img = do_img0 + sb * kImg;
    const int q_idx = q0 + r;
    const int64_t stat = (static_cast<int64_t>(b) * p.H + h) * p.T + q_idx;
    const float lse2 = q_idx < p.T ? p.lse[stat] : 0.f;
    const float dlt = q_idx < p.T ? p.delta[stat] : 0.f;
    // every thread has finished reading dQ (aliased with S) of the previous query block, and the bulk reduction
    // of that block has finished reading its staging area (aliased with P / dS)
    if (r == 0) bulk_wait_group_read0();
    tc_fence_before();
    __syncthreads();
    if (r == 0) {
      bool good = true;
      if (it == 0) good = mbar_wait(&bars[2], 0, abort_flag, p.status, kErrAttnBarrierTimeout, blockIdx.x);
      good = good && mbar_wait(&bars[3 + sb], qdo_parity, abort_flag, p.status, kErrAttnBarrierTimeout, blockIdx.x);
      if (good) {
        tc_fence_after();
#pragma unroll
        for (int k16 = 0; k16 < DP / 16; ++k16)
          tc_mma_f16(tmem, kmajor_desc(smem_u32(q_img), k16), kmajor_desc(smem_u32(k_img), k16), idesc_s, k16 > 0);
#pragma unroll
        for (int k16 = 0; k16 < DP / 16; ++k16)
          tc_mma_f16(tmem + 128, kmajor_desc(smem_u32(do_img), k16), kmajor_desc(smem_u32(v_img), k16), idesc_s, k16 > 0);
        tc_commit(&bars[0]);
        if (kBufs == 2 && i + 1 < n_q) {          // the other Q / dO buffer was released by the previous bars[1] wait
          mbar_expect_tx(&bars[3 + (sb ^ 1)], 2 * kImg);
          tma_tile<NB>(q_img0 + (sb ^ 1) * kImg, &map_q, &bars[3 + (sb ^ 1)], q0 + kBlk, h, b);
          tma_tile<NB>(do_img0 + (sb ^ 1) * kImg, &map_do, &bars[3 + (sb ^ 1)], q0 + kBlk, h, b);
        }
      }
    }
    if (!mbar_wait(&bars[0], it & 1, abort_flag, p.status, kErrAttnBarrierTimeout, blockIdx.x)) { ok = false; break; }
    tc_fence_after();
    const bool diag = (p.causal && i == kb) || (k0 + kBlk > p.T) || (q0 + kBlk > p.T);
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t rs[32], rp[32];
      tmem_ld_32x32(tmem + lane_base + c * 32, rs);
      tmem_ld_32x32(tmem + 128 + lane_base + c * 32, rp);
      tmem_wait_ld();
      float pv[32], dsv[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int key = k0 + c * 32 + j;
        float sx = __uint_as_float(rs[j]) * sc2;
        if (kbias != nullptr) sx += s_bias[c * 32 + j];
        const bool masked = diag && (key >= p.T || q_idx >= p.T || (p.causal && key > q_idx));
        const float pr = masked ? 0.f : exp2f(sx - lse2);
        pv[j] = pr;
        dsv[j] = pr * (__uint_as_float(rp[j]) - dlt) * p.scale;
      }
      store_p_chunk<T>(p_img, r, c * 32, pv);
      store_p_chunk<T>(ds_img, r, c * 32, dsv);
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (r == 0) {
      tc_fence_after();
      const uint32_t acc = it > 0 ? 1u : 0u;
#pragma unroll
      for (int k16 = 0; k16 < kBlk / 16; ++k16)   // dV[key, d] += sum_q P[q, key] dO[q, d]
        tc_mma_f16(tmem + 256, mnmajor_desc(smem_u32(p_img), k16), mnmajor_desc(smem_u32(do_img), k16), idesc_tt,
                   (k16 > 0) ? 1u : acc);
#pragma unroll
      for (int k16 = 0; k16 < kBlk / 16; ++k16)   // dK[key, d] += sum_q dS[q, key] Q[q, d]
        tc_mma_f16(tmem + 384, mnmajor_desc(smem_u32(ds_img), k16), mnmajor_desc(smem_u32(q_img), k16), idesc_tt,
                   (k16 > 0) ? 1u : acc);
#pragma unroll
      for (int k16 = 0; k16 < kBlk / 16; ++k16)   // dQ[q, d] = sum_key dS[q, key] K[key, d]
        tc_mma_f16(tmem, kmajor_desc(smem_u32(ds_img), k16), mnmajor_desc(smem_u32(k_img), k16), idesc_dq, k16 > 0);
      tc_commit(&bars[1]);
    }
    if (!mbar_wait(&bars[1], it & 1, abort_flag, p.status, kErrAttnBarrierTimeout, blockIdx.x)) { ok = false; break; }
    tc_fence_after();
    if (kBufs == 1 && r == 0 && i + 1 < n_q) {    // single buffer: refill it now that every MMA reading it is done
      mbar_expect_tx(&bars[3], 2 * kImg);
      tma_tile<NB>(q_img0, &map_q, &bars[3], q0 + kBlk, h, b);
      tma_tile<NB>(do_img0, &map_do, &bars[3], q0 + kBlk, h, b);
    }
    {
      // dQ of this (query block, key block) pair: TMEM -> registers -> shared staging -> one bulk fp32
      // reduction into the [B, H, T, DP] accumulator (several key blocks add into the same query rows)
#pragma unroll
      for (int c = 0; c < DP / 32; ++c) {
        uint32_t raw[32];
        tmem_ld_32x32(tmem + lane_base + c * 32, raw);
        tmem_wait_ld();
        float4* dst = reinterpret_cast<float4*>(dq_stage + r * DP + c * 32);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          dst[j] = make_float4(__uint_as_float(raw[4 * j]), __uint_as_float(raw[4 * j + 1]),
                               __uint_as_float(raw[4 * j + 2]), __uint_as_float(raw[4 * j + 3]));
      }
      fence_proxy_async();
      tc_fence_before();
      __syncthreads();
      if (r == 0) {
        const int qvalid = min(kBlk, p.T - q0);
        float* gdst = p.dq_acc + ((static_cast<int64_t>(b) * p.H + h) * p.T + q0) * DP;
        bulk_reduce_add_f32(gdst, dq_stage, static_cast<uint32_t>(qvalid) * DP * 4);
        bulk_commit_group();
      }
    }
  }
  if (r == 0) bulk_wait_group0();

  if (ok && it > 0) {
    const int key = k0 + r;
    T* dst = reinterpret_cast<T*>(p.dqkv) + (static_cast<int64_t>(b) * p.T + min(key, p.T - 1)) * ld + h * 3 * p.dh;
#pragma unroll
    for (int c = 0; c < DP / 32; ++c) {
      uint32_t rv[32], rk[32];
      tmem_ld_32x32(tmem + 256 + lane_base + c * 32, rv);
      tmem_ld_32x32(tmem + 384 + lane_base + c * 32, rk);
      tmem_wait_ld();
      if (key < p.T) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int d = c * 32 + j;
          if (d < p.dh) {
            dst[p.dh + d] = from_f<T>(__uint_as_float(rk[j]));
            dst[2 * p.dh + d] = from_f<T>(__uint_as_float(rv[j]));
          }
        }
      }
    }
  } else if (ok && k0 + r < p.T) {
    // no query block attends to this key block (cannot happen for causal / full attention, kept for safety)
    T* dst = reinterpret_cast<T*>(p.dqkv) + (static_cast<int64_t>(b) * p.T + k0 + r) * ld + h * 3 * p.dh;
    for (int d = 0; d < p.dh; ++d) { dst[p.dh + d] = from_f<T>(0.f); dst[2 * p.dh + d] = from_f<T>(0.f); }
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

// ------------------------------------------------------------------------------------------------ host side
static int padded_dim(int dh) {
  TORCH_CHECK(dh >= 1 && dh <= 128, "head dimension must be in [1, 128]");
  return dh <= 32 ? 32 : dh <= 64 ? 64 : dh <= 96 ? 96 : 128;
}
template <int DP>
constexpr int fwd_smem() { return 3 * ((DP + 63) / 64) * kBlk * 128 + 2 * kBlk * 128 + 64 + 1024 + 1024; }
template <int DP>
constexpr int bwd_smem() {
  return (DP <= 64 ? 6 : 4) * ((DP + 63) / 64) * kBlk * 128 + 4 * kBlk * 128 + 64 + 1024 + 512;
}

struct AttnMaps {
  CUtensorMap q, k, v, d_out;
};

template <typename T, int DP>
static void launch_fwd(const AttnMaps& m, const AttnParams& p, cudaStream_t s) {
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
  auto kern = attn_bwd_kernel<T, DP>;
  static bool done = false;
  if (!done) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bwd_smem<DP>()));
    done = true;
  }
  dim3 grid((p.T + kBlk - 1) / kBlk, p.H, p.B);
  kern<<<grid, kAttnThreads, bwd_smem<DP>(), s>>>(m.q, m.k, m.v, m.d_out, p);
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

static int pack_width(int dh) { return dh <= 64 ? 64 : 128; }

// [parts][B, H, T, W] zero-padded copy of src [B, T, H, parts*dh].
static torch::Tensor pack_heads(const torch::Tensor& src, int B, int T, int H, int dh, int parts, cudaStream_t stream) {
  const int W = pack_width(dh);
  auto dst = torch::empty({parts, B, H, T, W}, src.options());
  const int64_t total = static_cast<int64_t>(B) * T * H * parts;
  if (src.scalar_type() == torch::kBFloat16) {
    attn_pack_kernel<__nv_bfloat16><<<(total + 255) / 256, 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(src.data_ptr()), reinterpret_cast<__nv_bfloat16*>(dst.data_ptr()), B, T, H, dh,
        parts, W);
  } else {
    attn_pack_kernel<__half><<<(total + 255) / 256, 256, 0, stream>>>(reinterpret_cast<const __half*>(src.data_ptr()),
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
                                         double scale, int64_t status_ptr) {
  AttnParams p = base_params(qkv, causal, key_bias, scale, status_ptr);
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
                            c10::optional<torch::Tensor> packed_opt) {
  AttnParams p = base_params(qkv, causal, key_bias, scale, status_ptr);
  TORCH_CHECK(dout.is_contiguous() && dout.numel() == out.numel() && dout.scalar_type() == qkv.scalar_type());
  auto dqkv = torch::empty_like(qkv);
  if (qkv.numel() == 0) return dqkv;
  auto f32 = qkv.options().dtype(torch::kFloat32);
  auto delta = torch::empty({p.B, p.H, p.T}, f32);
  const int DPh = padded_dim(p.dh);
  auto dq_acc = torch::zeros({p.B, p.H, p.T, DPh}, f32);
  auto stream = at::cuda::getCurrentCUDAStream();
  const int64_t rows = static_cast<int64_t>(p.B) * p.T * p.H;
  if (p.is_bf16) {
    attn_delta_kernel<__nv_bfloat16><<<(rows + 255) / 256, 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(dout.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(out.data_ptr()),
        delta.data_ptr<float>(), p.B, p.T, p.H, p.dh);
  } else {
    attn_delta_kernel<__half><<<(rows + 255) / 256, 256, 0, stream>>>(
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
  p.lse = lse.data_ptr<float>();
  p.delta = delta.data_ptr<float>();
  p.dq_acc = dq_acc.data_ptr<float>();
  p.dqkv = dqkv.data_ptr();
  DISPATCH_ATTN(launch_bwd, m, p, stream)
  const int64_t n = rows * p.dh;
  if (p.is_bf16) {
    attn_dq_store_kernel<__nv_bfloat16><<<(n + 255) / 256, 256, 0, stream>>>(
        dq_acc.data_ptr<float>(), reinterpret_cast<__nv_bfloat16*>(dqkv.data_ptr()), p.B, p.T, p.H, p.dh, DPh);
  } else {
    attn_dq_store_kernel<__half><<<(n + 255) / 256, 256, 0, stream>>>(
        dq_acc.data_ptr<float>(), reinterpret_cast<__half*>(dqkv.data_ptr()), p.B, p.T, p.H, p.dh, DPh);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return dqkv;
}

}  // namespace cw
