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
// One CTA owns 128 query rows of one (batch, head):
//   warp 0      TMA producer: Q tile once, then K/V tiles of kBlockN keys into a 2-stage ring
//   warp 1      MMA issuer:   S = Q K^T  (tcgen05.mma, fp32 accumulator in TMEM)
//                             T = P V    (P from shared memory, V as an MN-major B operand)
//   warps 2-5   one thread per query row: TMEM -> registers, mask, running max / sum, exp2,
//               P -> swizzled shared memory, O (registers) = O * alpha + T
// Two CTAs share an SM (head dim <= 64) so one CTA's softmax overlaps the other's MMAs.
// Head dims that are not a multiple of 8, or larger than 128, run on a CUDA-core kernel.
#include <cuda.h>

#include <atomic>
#include <cmath>

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
  float scale_log2;  // softmax scale * log2(e)
  int causal;
  void* out;  // [B, Sq, H, Dv]
  int* status;
};

constexpr int kAttnThreads = 192;
constexpr int kBlockM = 128;

template <int BLOCK_N, int DCH>
struct AttnCfg {
  static constexpr int kQBytes = DCH * kBlockM * 128;
  static constexpr int kKBytes = DCH * BLOCK_N * 128;  // one K (or V) stage
  static constexpr int kPBytes = (BLOCK_N / 64) * kBlockM * 128;
  static constexpr int kStages = 2;
  static constexpr int kDataBytes = kQBytes + kStages * 2 * kKBytes + kPBytes;
  // the dynamic shared-memory window is declared 1024-byte aligned, so no slack is reserved:
  // two CTAs of the 64-wide configuration must fit one SM
  static constexpr int kSmemBytes = kDataBytes + 128;
  static constexpr int kTmemCols = (BLOCK_N + DCH * 64 <= 128) ? 128 : 256;  // S then T
};

template <int BLOCK_N, int DCH, bool BF16>
__global__ void __launch_bounds__(kAttnThreads, (DCH == 1) ? 2 : 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                    const __grid_constant__ CUtensorMap tma_v, const AttnParams p) {
  using Cfg = AttnCfg<BLOCK_N, DCH>;
  constexpr int kStages = Cfg::kStages;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0u) {  // swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, kDevBadSmemAlignment);
    return;
  }
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + Cfg::kQBytes;  // stage s: K at sKV + s*2*kKBytes, V right after K
  uint8_t* sP = sKV + kStages * 2 * Cfg::kKBytes;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(sP + Cfg::kPBytes);
  uint64_t* kv_full = q_full + 1;
  uint64_t* kv_empty = kv_full + kStages;
  uint64_t* s_full = kv_empty + kStages;
  uint64_t* p_full = s_full + 1;
  uint64_t* t_full = p_full + 1;
  uint64_t* drain_bar = t_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_blk = blockIdx.x % p.q_blocks;
  const int bh = blockIdx.x / p.q_blocks;
  const int q0 = q_blk * kBlockM;
  int kv_len = p.Skv;
  if (p.causal) kv_len = min(kv_len, q0 + kBlockM);
  const int n_blocks = (kv_len + BLOCK_N - 1) / BLOCK_N;
  const int dsteps = (p.D + 15) / 16;  // k-steps of Q K^T

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 128);
    mbar_init(t_full, 1);
    mbar_init(drain_bar, 1);
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
  const uint32_t tmem_s = tmem_base;            // BLOCK_N columns
  const uint32_t tmem_t = tmem_base + BLOCK_N;  // DCH*64 columns

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, Cfg::kQBytes);
#pragma unroll
      for (int c = 0; c < DCH; ++c) tma_load_3d(sQ + c * kBlockM * 128, &tma_q, q_full, c * 64, q0, bh);
      bool ok = true;
      for (int j = 0; ok && j < n_blocks; ++j) {
        const int st = j % kStages;
        const uint32_t ph = (j / kStages) & 1;
        ok = mbar_wait(&kv_empty[st], ph ^ 1u, abort_flag, p.status, kDevWaitEmptyTimeout);
        if (!ok) break;
        uint8_t* sK = sKV + st * 2 * Cfg::kKBytes;
        uint8_t* sV = sK + Cfg::kKBytes;
        mbar_arrive_expect_tx(&kv_full[st], 2 * Cfg::kKBytes);
#pragma unroll
        for (int c = 0; c < DCH; ++c) {
          tma_load_3d(sK + c * BLOCK_N * 128, &tma_k, &kv_full[st], c * 64, j * BLOCK_N, bh);
          tma_load_3d(sV + c * BLOCK_N * 128, &tma_v, &kv_full[st], c * 64, j * BLOCK_N, bh);
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
      constexpr uint32_t idesc_s = umma_idesc_f16(kBlockM, BLOCK_N, BF16, false, false);
      constexpr uint32_t idesc_t = umma_idesc_f16(kBlockM, DCH * 64, BF16, false, true);  // V is MN-major
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, kDevWaitFullTimeout);
      for (int j = 0; ok && j < n_blocks; ++j) {
        const int st = j % kStages;
        const uint32_t ph = (j / kStages) & 1;
        ok = mbar_wait(&kv_full[st], ph, abort_flag, p.status, kDevWaitFullTimeout);
        if (!ok) break;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQ);
        const uint32_t k_addr = smem_u32(sKV + st * 2 * Cfg::kKBytes);
        const uint32_t v_addr = k_addr + Cfg::kKBytes;
        for (int k = 0; k < dsteps; ++k) {
          const int c = k >> 2, kk = k & 3;
          const uint64_t adesc = umma_smem_desc_sw128(q_addr + c * kBlockM * 128 + kk * 32, 16, 1024);
          const uint64_t bdesc = umma_smem_desc_sw128(k_addr + c * BLOCK_N * 128 + kk * 32, 16, 1024);
          umma_f16_ss(tmem_s, adesc, bdesc, idesc_s, k != 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        ok = mbar_wait(p_full, j & 1, abort_flag, p.status, kDevWaitOtherTimeout);
        if (!ok) break;
        tc_fence_after();
        const uint32_t p_addr = smem_u32(sP);
#pragma unroll
        for (int k = 0; k < BLOCK_N / 16; ++k) {
          const int c = k >> 2, kk = k & 3;
          const uint64_t adesc = umma_smem_desc_sw128(p_addr + c * kBlockM * 128 + kk * 32, 16, 1024);
          // V tile rows are keys (128 B each): 16 keys per step = 2048 B; 64-wide d chunks are
          // BLOCK_N*128 B apart (leading byte offset), 8-key groups 1024 B apart (stride byte offset)
          const uint64_t bdesc = umma_smem_desc_sw128(v_addr + k * 2048, BLOCK_N * 128, 1024);
          umma_f16_ss(tmem_t, adesc, bdesc, idesc_t, k != 0 ? 1u : 0u);
        }
        umma_commit(t_full);
        umma_commit(&kv_empty[st]);
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
    const int q_idx = q0 + r;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    float o[DCH * 64];
#pragma unroll
    for (int i = 0; i < DCH * 64; ++i) o[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; ok && j < n_blocks; ++j) {
      ok = mbar_wait(s_full, j & 1, abort_flag, p.status, kDevWaitAccFullTimeout);
      if (!ok) break;
      tc_fence_after();
      const int key0 = j * BLOCK_N;
      int limit = kv_len - key0;  // keys [0, limit) of this block are valid
      if (p.causal) limit = min(limit, q_idx - key0 + 1);
      // A key block is "plain" when every key of it is visible to every row of this warp: then the two
      // passes run without per-element masks (the common case; only the last block of a ragged or
      // causal sequence needs them).
      const int limit_min = __reduce_min_sync(0xffffffffu, limit);
      const bool plain = limit_min >= BLOCK_N;
      // pass 1: row maximum
      float m_blk = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < BLOCK_N / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_s + lane_addr + c * 32, v);
        tmem_ld_wait();
        if (plain) {
          float m0 = __uint_as_float(v[0]), m1 = __uint_as_float(v[1]), m2 = __uint_as_float(v[2]),
                m3 = __uint_as_float(v[3]);
#pragma unroll
          for (int i = 4; i < 32; i += 4) {
            m0 = fmaxf(m0, __uint_as_float(v[i]));
            m1 = fmaxf(m1, __uint_as_float(v[i + 1]));
            m2 = fmaxf(m2, __uint_as_float(v[i + 2]));
            m3 = fmaxf(m3, __uint_as_float(v[i + 3]));
          }
          m_blk = fmaxf(m_blk, fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i < limit) m_blk = fmaxf(m_blk, __uint_as_float(v[i]));
        }
      }
      const float m_new = fmaxf(m_run, m_blk * p.scale_log2);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = exp2f(m_run - m_use);
      // pass 2: p = exp2(s*scale - m), row sum, P -> swizzled smem
      float l_blk = 0.f;
#pragma unroll 1
      for (int c = 0; c < BLOCK_N / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_s + lane_addr + c * 32, v);
        tmem_ld_wait();
        uint32_t packed[16];
        if (plain) {
          float l0 = 0.f, l1 = 0.f;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = exp2f(fmaf(__uint_as_float(v[i]), p.scale_log2, -m_use));
            const float p1 = exp2f(fmaf(__uint_as_float(v[i + 1]), p.scale_log2, -m_use));
            l0 += p0;
            l1 += p1;
            packed[i >> 1] = E::from_float2(p0, p1);
          }
          l_blk += l0 + l1;
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 =
                (c * 32 + i < limit) ? exp2f(fmaf(__uint_as_float(v[i]), p.scale_log2, -m_use)) : 0.f;
            const float p1 =
                (c * 32 + i + 1 < limit) ? exp2f(fmaf(__uint_as_float(v[i + 1]), p.scale_log2, -m_use)) : 0.f;
            l_blk += p0 + p1;
            packed[i >> 1] = E::from_float2(p0, p1);
          }
        }
        // keys c*32 .. c*32+31 live in 64-key chunk (c >> 1), 16-byte units (c & 1)*4 .. +3 of row r
        uint8_t* row_base = sP + (c >> 1) * kBlockM * 128 + r * 128;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int unit = ((c & 1) * 4 + u) ^ (r & 7);
          *reinterpret_cast<uint4*>(row_base + unit * 16) =
              make_uint4(packed[u * 4], packed[u * 4 + 1], packed[u * 4 + 2], packed[u * 4 + 3]);
        }
      }
      l_run = l_run * alpha + l_blk;
      m_run = m_new;
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(p_full);
      // O = O * alpha + P V
      ok = mbar_wait(t_full, j & 1, abort_flag, p.status, kDevWaitAccFullTimeout);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < DCH * 2; ++c) {
        if (c * 32 < p.Dv) {  // warp-uniform
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_t + lane_addr + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c * 32 + i] = o[c * 32 + i] * alpha + __uint_as_float(v[i]);
        }
      }
      tc_fence_before();
    }
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

template <int BLOCK_N, int DCH, bool BF16>
void launch_attn(const void* q, const void* k, const void* v, const AttnParams& p, cudaStream_t stream) {
  using Cfg = AttnCfg<BLOCK_N, DCH>;
  static std::atomic<uint64_t> configured{0};
  opt_in_smem_once(configured, reinterpret_cast<const void*>(&attention_tc_kernel<BLOCK_N, DCH, BF16>), Cfg::kSmemBytes);
  const long long bh = static_cast<long long>(p.B) * p.H;
  CUtensorMap tq = make_attn_map(q, BF16, p.D, p.Sq, bh, kBlockM);
  CUtensorMap tk = make_attn_map(k, BF16, p.D, p.Skv, bh, BLOCK_N);
  CUtensorMap tv = make_attn_map(v, BF16, p.Dv, p.Skv, bh, BLOCK_N);
  const long long grid = bh * p.q_blocks;
  B200AIT_REQUIRE(grid < (1ll << 31), "attention: grid too large");
  attention_tc_kernel<BLOCK_N, DCH, BF16><<<static_cast<unsigned>(grid), kAttnThreads, Cfg::kSmemBytes, stream>>>(tq, tk, tv, p);
  B200AIT_CUDA_CHECK(cudaGetLastError());
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
          launch_attn<128, 2, true>(query, key, value, p, stream);
        else
          launch_attn<128, 2, false>(query, key, value, p, stream);
      } else {
        if (bf16)
          launch_attn<128, 1, true>(query, key, value, p, stream);
        else
          launch_attn<128, 1, false>(query, key, value, p, stream);
      }
    } else {
      B200AIT_REQUIRE(head_size_v <= 256, "attention: head_size_v > 256 is not supported");
      const long long rows = static_cast<long long>(p.B) * p.H * p.Sq;
      const unsigned grid = static_cast<unsigned>((rows + 3) / 4);
      const size_t sh = 4 * static_cast<size_t>(p.D) * sizeof(float);
      if (bf16)
        attention_simt_kernel<true><<<grid, 128, sh, stream>>>(query, key, value, p);
      else
        attention_simt_kernel<false><<<grid, 128, sh, stream>>>(query, key, value, p);
      B200AIT_CUDA_CHECK(cudaGetLastError());
    }
  });
}
