// mem_eff_attention for sm_100a: O = softmax(scale * Q K^T) V per (batch, head), with Q, K, V laid out
// [B, H, S, D] and O written as [B, Sq, H, Dv]; optional causal mask (key index <= query index).
//
// Replaces the reference's CUTLASS 2.x kernel
//   static/include/kernels/mem_eff_attention/kernel_forward.h:103-860
//   python/aitemplate/backend/cuda/attention/mem_eff_attention.py:40-188, 632-787
// and keeps its arithmetic: scores in fp32, online softmax in base 2 with a running row maximum and
// row sum (attention_scaling_coefs_updater.h:85-165), P rounded to 16 bits before P.V, O kept in fp32
// and divided by the row sum at the end. S is never written to global memory.
//
// Persistent CTAs walk work items of 128 query rows of one (batch, head):
//   warp 0      TMA producer: the item's Q tile, then K/V blocks of kBlockN keys into a 3-stage ring;
//               the next item's Q streams in while the current item drains
//   warp 1      MMA issuer:   S = Q K^T  (tcgen05.mma, fp32 accumulator in TMEM)
//                             T = P V    (P from shared memory, V as an MN-major B operand)
//               S, P and T are double-buffered: the MMAs of key block j+1 overlap the softmax of block j
//   warps 2-5   one thread per query row: TMEM -> registers, mask (skipped for full, unmasked blocks),
//               running max / sum, exp2, P -> swizzled shared memory, O (registers) = O * alpha + T
// Two CTAs share an SM (head dim <= 64) so one CTA's softmax also overlaps the other's MMAs.
// Head dims that are not a multiple of 8, or larger than 128, run on a CUDA-core kernel.
#include <cuda.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <type_traits>

#include "common.h"
#include "epilogue.cuh"
#include "ptx.cuh"

namespace b200ait {

// defined in gemm.cu
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_fn();

struct AttnParams {
  int B, H, Sq, Skv, D, Dv;
  int q_blocks;
  int num_items;  // B * H * q_blocks work items of 128 query rows
  float scale_log2;  // softmax scale * log2(e)
  int causal;
  void* out;  // [B, Sq, H, Dv]
  int* status;
};

constexpr int kAttnThreads = 192;
constexpr int kBlockM = 128;
constexpr int kBlockN = 64;     // keys per block
constexpr int kKvStages = 3;    // K/V ring: blocks j, j+1, j+2 are in flight

template <int DCH>
struct AttnCfg {
  static constexpr int kQBytes = DCH * kBlockM * 128;
  static constexpr int kKBytes = DCH * kBlockN * 128;  // one K (or V) block
  static constexpr int kPBytes = kBlockM * 128;        // one P block: 128 rows x 64 keys
  static constexpr int kDataBytes = kQBytes + kKvStages * 2 * kKBytes + 2 * kPBytes;
  // the dynamic shared-memory window is declared 1024-byte aligned, so no slack is reserved:
  // two CTAs of the 64-wide configuration (96 KB each) must fit one SM
  static constexpr int kSmemBytes = kDataBytes + 128;
  static constexpr int kTWidth = DCH * 64;                       // columns of one T = P V accumulator
  static constexpr int kTmemCols = (DCH == 1) ? 256 : 512;       // S x2 (64 each) then T x2
};

// Persistent CTAs: each walks work items (one item = 128 query rows of one (batch, head)) with stride
// gridDim.x, so barrier set-up, TMEM allocation and the load latency of the first tiles are paid once
// and the next item's Q / K / V stream in while the current item drains.
// Pipeline (key blocks numbered globally g = 0, 1, .. across items; everything double-buffered on g & 1):
//   MMA warp:      S(0), S(1); then for each j: wait P(j) -> T(j) = P(j) V(j) -> S(j+2)
//   softmax warps: wait S(j) -> max / exp2 / row sum -> P(j) -> signal; then fold T(j-1) into O
// so the tensor core computes S(j+1), S(j+2) and T(j-1) while the softmax threads work on block j,
// and the softmax threads never wait for an MMA that was not issued a whole block earlier.
// NOMASK: no causal mask and a key length that is a multiple of the block: every key block is "plain", and the
// kernel is compiled without the masked softmax body (the lean variant is measurably faster than a run-time test).
template <int DCH, bool BF16, bool NOMASK>
__global__ void __launch_bounds__(kAttnThreads, (DCH == 1) ? 2 : 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                    const __grid_constant__ CUtensorMap tma_v, const AttnParams p) {
  using Cfg = AttnCfg<DCH>;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0u) {  // swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, kDevBadSmemAlignment);
    return;
  }
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + Cfg::kQBytes;  // stage s: K at sKV + s*2*kKBytes, V right after K
  uint8_t* sP = sKV + kKvStages * 2 * Cfg::kKBytes;  // two P blocks
  uint64_t* q_full = reinterpret_cast<uint64_t*>(sP + 2 * Cfg::kPBytes);
  uint64_t* kv_full = q_full + 1;
  uint64_t* kv_empty = kv_full + kKvStages;
  uint64_t* s_full = kv_empty + kKvStages;  // [2]
  uint64_t* p_full = s_full + 2;            // [2]
  uint64_t* t_full = p_full + 2;            // [2]
  uint64_t* drain_bar = t_full + 2;
  uint64_t* q_empty = drain_bar + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // work item -> (batch*head index, first query row, visible key count, key blocks)
  auto decode_item = [&](int item, int& bh, int& q0, int& kv_len, int& n_blocks) {
    const int q_blk = item % p.q_blocks;
    bh = item / p.q_blocks;
    q0 = q_blk * kBlockM;
    kv_len = p.Skv;
    if (!NOMASK && p.causal) kv_len = min(kv_len, q0 + kBlockM);
    n_blocks = (kv_len + kBlockN - 1) / kBlockN;
  };
  const int dsteps = (p.D + 15) / 16;  // k-steps of Q K^T

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kKvStages; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 128);
      mbar_init(&t_full[i], 1);
    }
    mbar_init(drain_bar, 1);
    mbar_init(q_empty, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tma_q);
    tma_prefetch_desc(&tma_k);
    tma_prefetch_desc(&tma_v);
  }
  __syncthreads();
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;        // S(j) at + (j & 1) * 64
  const uint32_t tmem_t = tmem_base + 128;  // T(j) at + (j & 1) * kTWidth

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      int g = 0;  // global key-block counter (K/V ring position)
      int it = 0;
      for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++it) {
        int bh, q0, kv_len, n_blocks;
        decode_item(item, bh, q0, kv_len, n_blocks);
        // the Q tile is free once the previous item's last S = Q K^T has completed
        ok = mbar_wait(q_empty, (it & 1) ^ 1u, abort_flag, p.status, kDevWaitEmptyTimeout);
        if (!ok) break;
        mbar_arrive_expect_tx(q_full, Cfg::kQBytes);
#pragma unroll
        for (int c = 0; c < DCH; ++c) tma_load_3d(sQ + c * kBlockM * 128, &tma_q, q_full, c * 64, q0, bh);
        for (int j = 0; j < n_blocks; ++j, ++g) {
          const int st = g % kKvStages;
          const uint32_t ph = (g / kKvStages) & 1;
          ok = mbar_wait(&kv_empty[st], ph ^ 1u, abort_flag, p.status, kDevWaitEmptyTimeout);
          if (!ok) break;
          uint8_t* sK = sKV + st * 2 * Cfg::kKBytes;
          uint8_t* sV = sK + Cfg::kKBytes;
          mbar_arrive_expect_tx(&kv_full[st], 2 * Cfg::kKBytes);
#pragma unroll
          for (int c = 0; c < DCH; ++c) {
            tma_load_3d(sK + c * kBlockN * 128, &tma_k, &kv_full[st], c * 64, j * kBlockN, bh);
            tma_load_3d(sV + c * kBlockN * 128, &tma_v, &kv_full[st], c * 64, j * kBlockN, bh);
          }
        }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_f16(kBlockM, kBlockN, BF16, false, false);
      constexpr uint32_t idesc_t = umma_idesc_f16(kBlockM, Cfg::kTWidth, BF16, false, true);  // V is MN-major
      const uint32_t q_addr = smem_u32(sQ);
      bool ok = true;
      // S(g) = Q K(g)^T into S buffer g & 1 (g = global key-block index)
      auto issue_s = [&](int g) -> bool {
        const int st = g % kKvStages;
        if (!mbar_wait(&kv_full[st], (g / kKvStages) & 1, abort_flag, p.status, kDevWaitFullTimeout)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sKV + st * 2 * Cfg::kKBytes);
        for (int k = 0; k < dsteps; ++k) {
          const int c = k >> 2, kk = k & 3;
          const uint64_t adesc = umma_smem_desc_sw128(q_addr + c * kBlockM * 128 + kk * 32, 16, 1024);
          const uint64_t bdesc = umma_smem_desc_sw128(k_addr + c * kBlockN * 128 + kk * 32, 16, 1024);
          umma_f16_ss(tmem_s + static_cast<uint32_t>((g & 1) * kBlockN), adesc, bdesc, idesc_s, k != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[g & 1]);
        return true;
      };
      int gb = 0;  // global index of the item's first key block
      int it = 0;
      for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++it) {
        int bh, q0, kv_len, n_blocks;
        decode_item(item, bh, q0, kv_len, n_blocks);
        ok = mbar_wait(q_full, it & 1, abort_flag, p.status, kDevWaitFullTimeout);
        if (ok) ok = issue_s(gb);
        if (ok && n_blocks > 1) ok = issue_s(gb + 1);
        if (ok && n_blocks <= 2) umma_commit(q_empty);  // every S of this item has been issued
        for (int j = 0; ok && j < n_blocks; ++j) {
          const int g = gb + j;
          ok = mbar_wait(&p_full[g & 1], (g >> 1) & 1, abort_flag, p.status, kDevWaitOtherTimeout);
          if (!ok) break;
          tc_fence_after();
          const int st = g % kKvStages;
          const uint32_t p_addr = smem_u32(sP + (g & 1) * Cfg::kPBytes);
          const uint32_t v_addr = smem_u32(sKV + st * 2 * Cfg::kKBytes + Cfg::kKBytes);
#pragma unroll
          for (int k = 0; k < kBlockN / 16; ++k) {
            const uint64_t adesc = umma_smem_desc_sw128(p_addr + k * 32, 16, 1024);
            // V block rows are keys (128 B each): 16 keys per step = 2048 B; 64-wide d chunks are
            // kBlockN*128 B apart (leading byte offset), 8-key groups 1024 B apart (stride byte offset)
            const uint64_t bdesc = umma_smem_desc_sw128(v_addr + k * 2048, kBlockN * 128, 1024);
            umma_f16_ss(tmem_t + static_cast<uint32_t>((g & 1) * Cfg::kTWidth), adesc, bdesc, idesc_t, k != 0 ? 1u : 0u);
          }
          umma_commit(&t_full[g & 1]);
          umma_commit(&kv_empty[st]);
          if (j + 2 < n_blocks) {
            ok = issue_s(g + 2);
            if (ok && j + 3 == n_blocks) umma_commit(q_empty);
          }
        }
        gb += n_blocks;
      }
      if (!ok) {
        umma_commit(drain_bar);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(drain_bar, 0) && globaltimer_ns() - t0 < 1000000ull) {
        }
      }
    }
    __syncwarp();
  } else {
    using E = Elem16<BF16>;
    using T = typename E::T;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;  // row inside the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    float o[DCH * 64];
    bool ok = true;
    // O = O * alpha + T(g)
    auto fold_t = [&](int g, float alpha) -> bool {
      if (!mbar_wait(&t_full[g & 1], (g >> 1) & 1, abort_flag, p.status, kDevWaitAccFullTimeout)) return false;
      tc_fence_after();
      const uint32_t t_addr = tmem_t + lane_addr + static_cast<uint32_t>((g & 1) * Cfg::kTWidth);
#pragma unroll
      for (int c = 0; c < DCH * 2; ++c) {
        if (c * 32 < p.Dv) {  // warp-uniform
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_addr + c * 32, v);
          tmem_ld_wait();
          const uint64_t alpha2 = pack2(alpha, alpha);
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const uint64_t r2 = fma2(pack2(o[c * 32 + i], o[c * 32 + i + 1]), alpha2,
                                     pack2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])));
            unpack2(r2, o[c * 32 + i], o[c * 32 + i + 1]);
          }
        }
      }
      tc_fence_before();
      return true;
    };
    int gb = 0;  // global index of the item's first key block
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x) {
      int bh, q0, kv_len, n_blocks;
      decode_item(item, bh, q0, kv_len, n_blocks);
      const int q_idx = q0 + r;
#pragma unroll
      for (int i = 0; i < DCH * 64; ++i) o[i] = 0.f;
      float m_run = -INFINITY, l_run = 0.f, alpha_prev = 0.f;
      for (int j = 0; ok && j < n_blocks; ++j) {
        const int g = gb + j;
        ok = mbar_wait(&s_full[g & 1], (g >> 1) & 1, abort_flag, p.status, kDevWaitAccFullTimeout);
        if (!ok) break;
        tc_fence_after();
        const uint32_t s_addr = tmem_s + lane_addr + static_cast<uint32_t>((g & 1) * kBlockN);
      const int key0 = j * kBlockN;
      int limit = kv_len - key0;  // keys [0, limit) of this block are visible to this row
      if (!NOMASK && p.causal) limit = min(limit, q_idx - key0 + 1);
      // A key block is "plain" when every key of it is visible to every row of this warp: then both
      // passes run without per-element masks (only the last block of a ragged or causal sequence
      // needs them).
      const bool plain = NOMASK || __reduce_min_sync(0xffffffffu, limit) >= kBlockN;
      uint32_t s0[32], s1[32];
      tmem_ld_32x32b_x32(s_addr, s0);
      tmem_ld_32x32b_x32(s_addr + 32, s1);
      tmem_ld_wait();
      uint8_t* row_base = sP + (g & 1) * Cfg::kPBytes + r * 128;
      float alpha, m_new, l0 = 0.f, l1 = 0.f;
      // One body, compiled twice: kPlain drops every per-element mask.
      auto softmax_block = [&](auto plain_tag) {
        constexpr bool kPlain = decltype(plain_tag)::value;
        float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float a0 = __uint_as_float(s0[i]), a1 = __uint_as_float(s0[i + 1]);
          const float b0 = __uint_as_float(s1[i]), b1 = __uint_as_float(s1[i + 1]);
          if constexpr (kPlain) {
            m0 = max3(m0, a0, a1);
            m2 = max3(m2, b0, b1);
          } else {
            m0 = fmaxf(m0, (i < limit) ? a0 : -INFINITY);
            m1 = fmaxf(m1, (i + 1 < limit) ? a1 : -INFINITY);
            m2 = fmaxf(m2, (32 + i < limit) ? b0 : -INFINITY);
            m3 = fmaxf(m3, (33 + i < limit) ? b1 : -INFINITY);
          }
        }
        const float m_blk = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
        m_new = fmaxf(m_run, m_blk * p.scale_log2);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        alpha = exp2f(m_run - m_use);
        // p = exp2(s * scale - m), row sum, P -> swizzled shared memory (16-byte unit u of row r sits
        // at unit u ^ (r & 7))
        const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2), negm2 = pack2(-m_use, -m_use);
        uint64_t lsum2 = pack2(0.f, 0.f);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t(&sv)[32] = h == 0 ? s0 : s1;
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float x0, x1;
            unpack2(fma2(pack2(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])), scale2, negm2), x0, x1);
            float p0 = exp2f(x0);
            float p1 = exp2f(x1);
            if (!kPlain) {
              p0 = (h * 32 + i < limit) ? p0 : 0.f;
              p1 = (h * 32 + i + 1 < limit) ? p1 : 0.f;
            }
            lsum2 = add2(lsum2, pack2(p0, p1));
            packed[i >> 1] = E::from_float2(p0, p1);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int unit = (h * 4 + u) ^ (r & 7);
            *reinterpret_cast<uint4*>(row_base + unit * 16) =
                make_uint4(packed[u * 4], packed[u * 4 + 1], packed[u * 4 + 2], packed[u * 4 + 3]);
          }
        }
        unpack2(lsum2, l0, l1);
      };
      if constexpr (NOMASK) {
        softmax_block(std::true_type{});
      } else {
        if (plain)
          softmax_block(std::true_type{});
        else
          softmax_block(std::false_type{});
      }
      l_run = l_run * alpha + (l0 + l1);
      m_run = m_new;
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(&p_full[g & 1]);
      // fold the previous block's P V into O while the tensor core works on this block's
        if (j > 0) ok = fold_t(g - 1, alpha_prev);
        alpha_prev = alpha;
      }
      if (ok) ok = fold_t(gb + n_blocks - 1, alpha_prev);
      gb += n_blocks;
      if (ok && q_idx < p.Sq) {
        const float inv = (l_run > 0.f) ? 1.f / l_run : 0.f;
        const int b = bh / p.H, h = bh - b * p.H;
        T* out = static_cast<T*>(p.out) + ((static_cast<long long>(b) * p.Sq + q_idx) * p.H + h) * p.Dv;
#pragma unroll
        for (int c = 0; c < DCH * 8; ++c) {
          if (c * 8 < p.Dv) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = o[c * 8 + i] * inv;
            *reinterpret_cast<uint4*>(out + c * 8) = pack8<BF16>(f);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------------
// CUDA-core kernel for head dims the tensor-core kernel does not take: one warp per query row,
// lanes over keys for the scores and over channels for the output.
template <bool BF16>
__global__ void __launch_bounds__(128) attention_simt_kernel(const void* q_, const void* k_, const void* v_,
                                                             const AttnParams p) {
  using E = Elem16<BF16>;
  using T = typename E::T;
  extern __shared__ float sh[];  // per warp: D floats of q
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * 4 + warp;
  const long long total = static_cast<long long>(p.B) * p.H * p.Sq;
  if (row >= total) return;
  const int qi = static_cast<int>(row % p.Sq);
  const long long bh = row / p.Sq;
  const T* q = static_cast<const T*>(q_) + (bh * p.Sq + qi) * p.D;
  const T* k = static_cast<const T*>(k_) + bh * p.Skv * p.D;
  const T* v = static_cast<const T*>(v_) + bh * p.Skv * p.Dv;
  float* sq = sh + warp * p.D;
  for (int i = lane; i < p.D; i += 32) sq[i] = E::to_float(q[i]);
  __syncwarp();
  int kv_len = p.Skv;
  if (p.causal) kv_len = min(kv_len, qi + 1);
  constexpr int kMaxPerLane = 8;  // Dv <= 256
  float o[kMaxPerLane];
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) o[i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  for (int key0 = 0; key0 < kv_len; key0 += 32) {
    const int key = key0 + lane;
    float s = -INFINITY;
    if (key < kv_len) {
      float acc = 0.f;
      for (int d = 0; d < p.D; ++d) acc += sq[d] * E::to_float(k[static_cast<long long>(key) * p.D + d]);
      s = acc * p.scale_log2;
    }
    float m_blk = s;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m_blk = fmaxf(m_blk, __shfl_xor_sync(0xffffffffu, m_blk, off));
    const float m_new = fmaxf(m_run, m_blk);
    const float alpha = exp2f(m_run - m_new);
    float pr = (key < kv_len) ? exp2f(s - m_new) : 0.f;
    float l_blk = pr;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) l_blk += __shfl_xor_sync(0xffffffffu, l_blk, off);
    l_run = l_run * alpha + l_blk;
    m_run = m_new;
    pr = E::to_float(E::from_float(pr));  // the reference rounds P to the storage type before P.V
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) o[i] *= alpha;
    const int nk = min(32, kv_len - key0);
    for (int t = 0; t < nk; ++t) {
      const float pt = __shfl_sync(0xffffffffu, pr, t);
      const T* vr = v + static_cast<long long>(key0 + t) * p.Dv;
#pragma unroll
      for (int i = 0; i < kMaxPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < p.Dv) o[i] += pt * E::to_float(vr[d]);
      }
    }
  }
  const float inv = (l_run > 0.f) ? 1.f / l_run : 0.f;
  const long long b = bh / p.H, h = bh - b * p.H;
  T* out = static_cast<T*>(p.out) + ((b * p.Sq + qi) * p.H + h) * p.Dv;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int d = lane + 32 * i;
    if (d < p.Dv) out[d] = E::from_float(o[i] * inv);
  }
}

// [BH, S, D] map, box [1, box_rows, 64], 128-byte swizzle; a box wider than D zero-fills
static CUtensorMap make_attn_map(const void* base, bool bf16, int d, int s, long long bh, int box_rows) {
  CUtensorMap m;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(s), static_cast<cuuint64_t>(bh)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(d) * 2, static_cast<cuuint64_t>(d) * s * 2};
  cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = get_encode_fn()(&m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                               const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw Error("attention: cuTensorMapEncodeTiled failed with CUresult " + std::to_string(static_cast<int>(r)));
  return m;
}

template <int DCH, bool BF16, bool NOMASK>
void launch_attn_variant(const void* q, const void* k, const void* v, const AttnParams& p, cudaStream_t stream) {
  using Cfg = AttnCfg<DCH>;
  static std::atomic<uint64_t> configured{0};
  opt_in_smem_once(configured, reinterpret_cast<const void*>(&attention_tc_kernel<DCH, BF16, NOMASK>), Cfg::kSmemBytes);
  const long long bh = static_cast<long long>(p.B) * p.H;
  CUtensorMap tq = make_attn_map(q, BF16, p.D, p.Sq, bh, kBlockM);
  CUtensorMap tk = make_attn_map(k, BF16, p.D, p.Skv, bh, kBlockN);
  CUtensorMap tv = make_attn_map(v, BF16, p.Dv, p.Skv, bh, kBlockN);
  const long long items = bh * p.q_blocks;
  B200AIT_REQUIRE(items < (1ll << 31), "attention: too many work items");
  AttnParams pp = p;
  pp.num_items = static_cast<int>(items);
  const long long grid = std::min<long long>(items, static_cast<long long>(sm_count()) * (DCH == 1 ? 2 : 1));
  ::b200ait::count_launch(), attention_tc_kernel<DCH, BF16, NOMASK><<<static_cast<unsigned>(grid), kAttnThreads, Cfg::kSmemBytes, stream>>>(tq, tk, tv,
                                                                                                                 pp);
  B200AIT_CUDA_CHECK(cudaGetLastError());
}

template <int DCH, bool BF16>
void launch_attn(const void* q, const void* k, const void* v, const AttnParams& p, cudaStream_t stream) {
  if (!p.causal && p.Skv % kBlockN == 0)
    launch_attn_variant<DCH, BF16, true>(q, k, v, p, stream);
  else
    launch_attn_variant<DCH, BF16, false>(q, k, v, p, stream);
}

}  // namespace b200ait

using namespace b200ait;

// Argument order follows the reference's generated function
// (python/aitemplate/backend/cuda/attention/mem_eff_attention.py:632-654); variable-length inputs
// (lengths_kv / lengths_q) are not part of this path and must be null.
B200AIT_EXPORT int b200ait_mem_eff_attention(void* output, const void* query, const void* key, const void* value,
                                             int64_t batch_size, int64_t seq_len_kv, int64_t seq_len_q,
                                             int num_heads, int head_size, int head_size_v, float softmax_scale,
                                             int is_causal, const int32_t* lengths_kv, const int32_t* lengths_q,
                                             int dtype, cudaStream_t stream) {
  return guarded("b200ait_mem_eff_attention", [&] {
    B200AIT_REQUIRE(dtype == kDTypeHalf || dtype == kDTypeBFloat16, "attention: dtype must be float16 or bfloat16");
    B200AIT_REQUIRE(!lengths_kv && !lengths_q, "attention: variable sequence lengths are not supported");
    B200AIT_REQUIRE(batch_size >= 0 && seq_len_kv >= 0 && seq_len_q >= 0 && num_heads >= 0 && head_size >= 0 &&
                        head_size_v >= 0,
                    "attention: negative dimension");
    if (batch_size == 0 || seq_len_q == 0 || num_heads == 0 || head_size_v == 0) return;
    B200AIT_REQUIRE(output && query, "attention: null pointer with non-zero size");
    B200AIT_REQUIRE(seq_len_kv > 0 && head_size > 0, "attention: empty key sequence or head");
    B200AIT_REQUIRE(key && value, "attention: null pointer with non-zero size");
    B200AIT_REQUIRE(seq_len_q < (1 << 30) && seq_len_kv < (1 << 30), "attention: sequence too long");
    AttnParams p{};
    p.B = static_cast<int>(batch_size), p.H = num_heads;
    p.Sq = static_cast<int>(seq_len_q), p.Skv = static_cast<int>(seq_len_kv);
    p.D = head_size, p.Dv = head_size_v;
    p.q_blocks = (p.Sq + kBlockM - 1) / kBlockM;
    p.scale_log2 = softmax_scale * 1.4426950408889634f;
    p.causal = is_causal ? 1 : 0;
    p.out = output;
    p.status = device_status_word();
    const bool bf16 = dtype == kDTypeBFloat16;
    auto al = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15u) == 0; };
    const bool tc_ok = head_size % 8 == 0 && head_size_v % 8 == 0 && head_size <= 128 && head_size_v <= 128 &&
                       al(query) && al(key) && al(value) && al(output);
    if (tc_ok) {
      const bool two = head_size > 64 || head_size_v > 64;
      if (two) {
        if (bf16)
          launch_attn<2, true>(query, key, value, p, stream);
        else
          launch_attn<2, false>(query, key, value, p, stream);
      } else {
        if (bf16)
          launch_attn<1, true>(query, key, value, p, stream);
        else
          launch_attn<1, false>(query, key, value, p, stream);
      }
    } else {
      B200AIT_REQUIRE(head_size_v <= 256, "attention: head_size_v > 256 is not supported");
      const long long rows = static_cast<long long>(p.B) * p.H * p.Sq;
      const unsigned grid = static_cast<unsigned>((rows + 3) / 4);
      const size_t sh = 4 * static_cast<size_t>(p.D) * sizeof(float);
      if (bf16)
        ::b200ait::count_launch(), attention_simt_kernel<true><<<grid, 128, sh, stream>>>(query, key, value, p);
      else
        ::b200ait::count_launch(), attention_simt_kernel<false><<<grid, 128, sh, stream>>>(query, key, value, p);
      B200AIT_CUDA_CHECK(cudaGetLastError());
    }
  });
}
