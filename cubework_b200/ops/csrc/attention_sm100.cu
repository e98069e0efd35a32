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
// Head dims are zero-padded to DP in {32, 64, 96, 128}.  Rows of one head are not 16-byte aligned in general
// (dh = 25), so tiles are staged with ordinary loads instead of TMA.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAException.h>
#include <torch/extension.h>

#include "common.cuh"
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

// Stage `rows` x dh elements (row stride `ld` elements) into an image, zero-filling rows >= valid and the padding.
template <typename T, int DP>
__device__ __forceinline__ void stage_rows(uint8_t* img, const T* src, int64_t ld, int valid, int dh) {
  const int r = threadIdx.x;
  const bool vec = (dh % 8 == 0) && (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
  if (vec) {
    constexpr int CPR = DP / 8;
    for (int idx = threadIdx.x; idx < kBlk * CPR; idx += kAttnThreads) {
      const int row = idx / CPR, ch = idx % CPR;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (row < valid && ch * 8 < dh) v = *reinterpret_cast<const uint4*>(src + row * ld + ch * 8);
      *reinterpret_cast<uint4*>(img + img_off(row, ch * 8)) = v;
    }
  } else {
    const T* p = src + static_cast<int64_t>(r) * ld;
#pragma unroll
    for (int ch = 0; ch < DP / 8; ++ch) {
      T tmp[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int c = ch * 8 + i;
        tmp[i] = (r < valid && c < dh) ? p[c] : from_f<T>(0.f);
      }
      *reinterpret_cast<uint4*>(img + img_off(r, ch * 8)) = *reinterpret_cast<const uint4*>(tmp);
    }
  }
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
  const void* qkv;      // [B, T, H, 3*dh]
  void* out;            // [B, T, H, dh]
  float* lse;           // [B, H, T]   (log2 domain: m + log2(l))
  const float* key_bias;  // [B, T] or nullptr
  int B, T, H, dh;
  float scale;
  int causal;
  int is_bf16;
  int* status;
  // backward only
  const void* dout;     // [B, T, H, dh]
  const float* delta;   // [B, H, T]  rowsum(dO * O)
  float* dq_acc;        // [B, T, H, dh] fp32 scratch, zero-initialised
  void* dqkv;           // [B, T, H, 3*dh]
};

template <typename T, int DP>
__global__ void __launch_bounds__(kAttnThreads) attn_fwd_kernel(AttnParams p) {
  constexpr int NB = (DP + 63) / 64;
  constexpr int kImg = NB * kBlk * 128;          // bytes of a [128 x DP] image
  constexpr uint32_t kTmemCols = 256;             // S: [0,128)  O_blk: [128, 128+DP)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_img = smem;
  uint8_t* k_img = q_img + kImg;
  uint8_t* v_img = k_img + kImg;
  uint8_t* p_img = v_img + kImg;                  // [128 x 128] 16-bit = 32 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_img + 2 * kBlk * 128);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int r = threadIdx.x, warp = r >> 5;
  const int qb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q0 = qb * kBlk;
  const int64_t ld = static_cast<int64_t>(p.H) * 3 * p.dh;
  const T* base = reinterpret_cast<const T*>(p.qkv) + (static_cast<int64_t>(b) * p.T) * ld + h * 3 * p.dh;

  if (r == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    __syncwarp();   // lane 0 just left the barrier-init branch: the allocation is warp-collective
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  stage_rows<T, DP>(q_img, base + static_cast<int64_t>(q0) * ld, ld, min(kBlk, p.T - q0), p.dh);
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
    const int kvalid = min(kBlk, p.T - k0);
    stage_rows<T, DP>(k_img, base + static_cast<int64_t>(k0) * ld + p.dh, ld, kvalid, p.dh);
    stage_rows<T, DP>(v_img, base + static_cast<int64_t>(k0) * ld + 2 * p.dh, ld, kvalid, p.dh);
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (r == 0) {
      tc_fence_after();
#pragma unroll
      for (int k16 = 0; k16 < DP / 16; ++k16)
        tc_mma_f16(tmem, kmajor_desc(smem_u32(q_img), k16), kmajor_desc(smem_u32(k_img), k16), idesc_s, k16 > 0);
      tc_commit(&bars[0]);
    }
    if (!mbar_wait(&bars[0], j & 1, abort_flag, p.status, kErrAttnBarrierTimeout, blockIdx.x)) { ok = false; break; }
    tc_fence_after();

    // ---- pass 1: row maximum of the masked, scaled scores (log2 domain)
    float m_blk = -INFINITY;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t raw[32];
      tmem_ld_32x32(tmem + lane_base + c * 32, raw);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int key = k0 + c * 32 + i;
        float s = __uint_as_float(raw[i]) * sc2;
        if (p.key_bias != nullptr && key < p.T) s += p.key_bias[static_cast<int64_t>(b) * p.T + key] * kLog2e;
        const bool masked = key >= p.T || (p.causal && key > q_idx);
        m_blk = fmaxf(m_blk, masked ? -INFINITY : s);
      }
    }
    const float m_new = fmaxf(m_run, m_blk);
    const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
    const float alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_use);
    // ---- pass 2: probabilities -> shared memory, row sum
    float l_blk = 0.f;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t raw[32];
      tmem_ld_32x32(tmem + lane_base + c * 32, raw);
      tmem_wait_ld();
      float pv[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int key = k0 + c * 32 + i;
        float s = __uint_as_float(raw[i]) * sc2;
        if (p.key_bias != nullptr && key < p.T) s += p.key_bias[static_cast<int64_t>(b) * p.T + key] * kLog2e;
        const bool masked = key >= p.T || (p.causal && key > q_idx);
        const float e = masked ? 0.f : exp2f(s - m_use);
        pv[i] = e;
        l_blk += e;
      }
      store_p_chunk<T>(p_img, r, c * 32, pv);
    }
    l_run = l_run * alpha + l_blk;
    m_run = m_new;
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (r == 0) {
      tc_fence_after();
#pragma unroll
      for (int k16 = 0; k16 < kBlk / 16; ++k16)
        tc_mma_f16(tmem + 128, kmajor_desc(smem_u32(p_img), k16), mnmajor_desc(smem_u32(v_img), k16), idesc_o, k16 > 0);
      tc_commit(&bars[1]);
    }
    if (!mbar_wait(&bars[1], j & 1, abort_flag, p.status, kErrAttnBarrierTimeout, blockIdx.x)) { ok = false; break; }
    tc_fence_after();
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

template <typename T>
__global__ void attn_dq_store_kernel(const float* __restrict__ dq_acc, T* __restrict__ dqkv, int64_t rows, int dh) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= rows * dh) return;
  const int64_t row = idx / dh;
  const int d = idx % dh;
  dqkv[row * 3 * dh + d] = from_f<T>(dq_acc[idx]);
}

template <typename T, int DP>
__global__ void __launch_bounds__(kAttnThreads) attn_bwd_kernel(AttnParams p) {
  constexpr int NB = (DP + 63) / 64;
  constexpr int kImg = NB * kBlk * 128;
  constexpr uint32_t kTmemCols = 512;   // S/dQ: [0,128)  dP: [128,256)  dV: [256,256+DP)  dK: [384,384+DP)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_img = smem;
  uint8_t* v_img = k_img + kImg;
  uint8_t* q_img = v_img + kImg;
  uint8_t* do_img = q_img + kImg;
  uint8_t* p_img = do_img + kImg;
  uint8_t* ds_img = p_img + 2 * kBlk * 128;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ds_img + 2 * kBlk * 128);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int r = threadIdx.x, warp = r >> 5;
  const int kb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int k0 = kb * kBlk;
  const int kvalid = min(kBlk, p.T - k0);
  const int64_t ld = static_cast<int64_t>(p.H) * 3 * p.dh;
  const int64_t ldo = static_cast<int64_t>(p.H) * p.dh;
  const T* base = reinterpret_cast<const T*>(p.qkv) + (static_cast<int64_t>(b) * p.T) * ld + h * 3 * p.dh;
  const T* dobase = reinterpret_cast<const T*>(p.dout) + (static_cast<int64_t>(b) * p.T) * ldo + h * p.dh;

  if (r == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    __syncwarp();   // lane 0 just left the barrier-init branch: the allocation is warp-collective
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  stage_rows<T, DP>(k_img, base + static_cast<int64_t>(k0) * ld + p.dh, ld, kvalid, p.dh);
  stage_rows<T, DP>(v_img, base + static_cast<int64_t>(k0) * ld + 2 * p.dh, ld, kvalid, p.dh);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  const uint32_t idesc_s = make_idesc_f16(kBlk, kBlk, false, false, p.is_bf16);     // Q K^T, dO V^T
  const uint32_t idesc_tt = make_idesc_f16(kBlk, DP, true, true, p.is_bf16);        // P^T dO, dS^T Q
  const uint32_t idesc_dq = make_idesc_f16(kBlk, DP, false, true, p.is_bf16);       // dS K
  const float sc2 = p.scale * kLog2e;

  const int n_q = (p.T + kBlk - 1) / kBlk;
  const int i0 = p.causal ? kb : 0;
  bool ok = true;
  int it = 0;
  for (int i = i0; i < n_q && ok; ++i, ++it) {
    const int q0 = i * kBlk;
    const int qvalid = min(kBlk, p.T - q0);
    stage_rows<T, DP>(q_img, base + static_cast<int64_t>(q0) * ld, ld, qvalid, p.dh);
    stage_rows<T, DP>(do_img, dobase + static_cast<int64_t>(q0) * ldo, ldo, qvalid, p.dh);
    const int q_idx = q0 + r;
    const int64_t stat = (static_cast<int64_t>(b) * p.H + h) * p.T + q_idx;
    const float lse2 = q_idx < p.T ? p.lse[stat] : 0.f;
    const float dlt = q_idx < p.T ? p.delta[stat] : 0.f;
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (r == 0) {
      tc_fence_after();
#pragma unroll
      for (int k16 = 0; k16 < DP / 16; ++k16)
        tc_mma_f16(tmem, kmajor_desc(smem_u32(q_img), k16), kmajor_desc(smem_u32(k_img), k16), idesc_s, k16 > 0);
#pragma unroll
      for (int k16 = 0; k16 < DP / 16; ++k16)
        tc_mma_f16(tmem + 128, kmajor_desc(smem_u32(do_img), k16), kmajor_desc(smem_u32(v_img), k16), idesc_s, k16 > 0);
      tc_commit(&bars[0]);
    }
    if (!mbar_wait(&bars[0], it & 1, abort_flag, p.status, kErrAttnBarrierTimeout, blockIdx.x)) { ok = false; break; }
    tc_fence_after();
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
        float s = __uint_as_float(rs[j]) * sc2;
        if (p.key_bias != nullptr && key < p.T) s += p.key_bias[static_cast<int64_t>(b) * p.T + key] * kLog2e;
        const bool masked = key >= p.T || q_idx >= p.T || (p.causal && key > q_idx);
        const float pr = masked ? 0.f : exp2f(s - lse2);
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
    {
      // every lane executes the (warp-collective) TMEM loads; only the accumulation is predicated
      float* dq = p.dq_acc + ((static_cast<int64_t>(b) * p.T + min(q_idx, p.T - 1)) * p.H + h) * p.dh;
      const bool q_ok = q_idx < p.T;
#pragma unroll
      for (int c = 0; c < DP / 32; ++c) {
        uint32_t raw[32];
        tmem_ld_32x32(tmem + lane_base + c * 32, raw);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (q_ok && c * 32 + j < p.dh) atomicAdd(dq + c * 32 + j, __uint_as_float(raw[j]));
      }
    }
    tc_fence_before();
  }

  if (ok && it > 0) {
    const int key = k0 + r;
    T* dst = reinterpret_cast<T*>(p.dqkv) + (static_cast<int64_t>(b) * p.T + key) * ld + h * 3 * p.dh;
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
constexpr int fwd_smem() { return 3 * ((DP + 63) / 64) * kBlk * 128 + 2 * kBlk * 128 + 64 + 1024; }
template <int DP>
constexpr int bwd_smem() { return 4 * ((DP + 63) / 64) * kBlk * 128 + 4 * kBlk * 128 + 64 + 1024; }

template <typename T, int DP>
static void launch_fwd(const AttnParams& p, cudaStream_t s) {
  auto kern = attn_fwd_kernel<T, DP>;
  static bool done = false;
  if (!done) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, fwd_smem<DP>()));
    done = true;
  }
  dim3 grid((p.T + kBlk - 1) / kBlk, p.H, p.B);
  kern<<<grid, kAttnThreads, fwd_smem<DP>(), s>>>(p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}
template <typename T, int DP>
static void launch_bwd(const AttnParams& p, cudaStream_t s) {
  auto kern = attn_bwd_kernel<T, DP>;
  static bool done = false;
  if (!done) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bwd_smem<DP>()));
    done = true;
  }
  dim3 grid((p.T + kBlk - 1) / kBlk, p.H, p.B);
  kern<<<grid, kAttnThreads, bwd_smem<DP>(), s>>>(p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

#define DISPATCH_ATTN(FN, p, stream)                                                       \
  {                                                                                        \
    const int dp_ = padded_dim((p).dh);                                                    \
    if ((p).is_bf16) {                                                                     \
      if (dp_ == 32) FN<__nv_bfloat16, 32>(p, stream);                                     \
      else if (dp_ == 64) FN<__nv_bfloat16, 64>(p, stream);                                \
      else if (dp_ == 96) FN<__nv_bfloat16, 96>(p, stream);                                \
      else FN<__nv_bfloat16, 128>(p, stream);                                              \
    } else {                                                                               \
      if (dp_ == 32) FN<__half, 32>(p, stream);                                            \
      else if (dp_ == 64) FN<__half, 64>(p, stream);                                       \
      else if (dp_ == 96) FN<__half, 96>(p, stream);                                       \
      else FN<__half, 128>(p, stream);                                                     \
    }                                                                                      \
  }

static AttnParams base_params(const torch::Tensor& qkv, bool causal, const c10::optional<torch::Tensor>& key_bias,
                              double scale, int64_t status_ptr) {
  TORCH_CHECK(qkv.is_cuda() && qkv.dim() == 4 && qkv.is_contiguous() && qkv.size(3) % 3 == 0,
              "qkv must be a contiguous [B, T, heads, 3*dh] CUDA tensor");
  TORCH_CHECK(qkv.scalar_type() == torch::kBFloat16 || qkv.scalar_type() == torch::kFloat16);
  AttnParams p{};
  p.qkv = qkv.data_ptr();
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

bool attention_ready() { return true; }

std::vector<torch::Tensor> attention_fwd(torch::Tensor qkv, bool causal, c10::optional<torch::Tensor> key_bias,
                                         double scale, int64_t status_ptr) {
  AttnParams p = base_params(qkv, causal, key_bias, scale, status_ptr);
  auto out = torch::empty({p.B, p.T, p.H, p.dh}, qkv.options());
  auto lse = torch::empty({p.B, p.H, p.T}, qkv.options().dtype(torch::kFloat32));
  if (qkv.numel() == 0) return {out, lse};
  p.out = out.data_ptr();
  p.lse = lse.data_ptr<float>();
  auto stream = at::cuda::getCurrentCUDAStream();
  DISPATCH_ATTN(launch_fwd, p, stream)
  return {out, lse};
}

torch::Tensor attention_bwd(torch::Tensor dout, torch::Tensor qkv, torch::Tensor out, torch::Tensor lse, bool causal,
                            c10::optional<torch::Tensor> key_bias, double scale, int64_t status_ptr) {
  AttnParams p = base_params(qkv, causal, key_bias, scale, status_ptr);
  TORCH_CHECK(dout.is_contiguous() && dout.numel() == out.numel() && dout.scalar_type() == qkv.scalar_type());
  auto dqkv = torch::empty_like(qkv);
  if (qkv.numel() == 0) return dqkv;
  auto f32 = qkv.options().dtype(torch::kFloat32);
  auto delta = torch::empty({p.B, p.H, p.T}, f32);
  auto dq_acc = torch::zeros({p.B, p.T, p.H, p.dh}, f32);
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
  p.dout = dout.data_ptr();
  p.lse = lse.data_ptr<float>();
  p.delta = delta.data_ptr<float>();
  p.dq_acc = dq_acc.data_ptr<float>();
  p.dqkv = dqkv.data_ptr();
  DISPATCH_ATTN(launch_bwd, p, stream)
  const int64_t n = rows * p.dh;
  if (p.is_bf16) {
    attn_dq_store_kernel<__nv_bfloat16><<<(n + 255) / 256, 256, 0, stream>>>(
        dq_acc.data_ptr<float>(), reinterpret_cast<__nv_bfloat16*>(dqkv.data_ptr()), rows, p.dh);
  } else {
    attn_dq_store_kernel<__half><<<(n + 255) / 256, 256, 0, stream>>>(dq_acc.data_ptr<float>(),
                                                                      reinterpret_cast<__half*>(dqkv.data_ptr()), rows,
                                                                      p.dh);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return dqkv;
}

}  // namespace cw
