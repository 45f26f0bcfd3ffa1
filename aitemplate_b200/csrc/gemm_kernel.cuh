// Device code of the tcgen05 GEMM (see gemm.cu for the design notes and the host side).
// Included by gemm.cu (parameters, scalar epilogue) and by the per-tile-width instantiation units
// gemm_bn64.cu / gemm_bn128.cu / gemm_bn256.cu.
#pragma once
#include <cuda.h>

#include <atomic>

#include "common.h"
#include "epilogue.cuh"
#include "ptx.cuh"

namespace b200ait {

struct GemmParams {
  int M, N, K, batch;
  int tiles_m, tiles_n, num_tiles;
  int splits, kb_per_split, num_units;  // split-K: unit = tile * splits + split
  float* partial;                       // [splits, batch, M, N] fp32 partial sums when splits > 1
  int a_batch_mul, b_batch_mul;  // 0 when that operand is broadcast over the batch
  int b_mn;                      // B is stored [K, N] (N contiguous, "row-major B") instead of [N, K]
  const void* bias;              // [N] or nullptr
  const void* d0;                // [M, N] residual operands (row stride ldd) or nullptr
  const void* d1;
  void* out;
  long long lda, ldb;            // only used by the CUDA-core kernel
  long long a_bs, b_bs;
  long long ldc, ldd, c_bs, d_bs;
  float alpha;
  int epilogue;
  // store_mode 0: out[b*c_bs + row*ldc + col]
  // store_mode 1: out[(row / t1)*rs_hi + (row % t1)*rs_lo + (col / (t3*d))*cs2 + ((col / d) % t3)*cs3 + col % d]
  int store_mode;
  int t1, t3, d;
  long long rs_hi, rs_lo, cs2, cs3;
  int vec_ok;  // 16-byte epilogue accesses are legal
  int tma_store;  // output goes through shared memory + TMA store (tensor maps `outs`)
  int num_out;    // destinations of the staged store (1 unless the caller passed several output buffers)
  int tma_d0;     // the residual d0 arrives by TMA in the output staging boxes (tensor map `tma_d0`)
  int* status;
  // batched "0213" store (bmm_*_permute): batch b = hi * c_bdiv + lo lands at hi * c_bs_hi + lo * c_bs, rows ldc
  // apart, i.e. [B / d1, d1, M, N] -> [B / d1, M, d1, N] with c_bdiv = d1, c_bs = N, ldc = d1 * N, c_bs_hi = M * d1 * N.
  // 0 = plain batch stride. Only the kernels with a run-time epilogue (EPI < 0) and the CUDA-core kernel honour it.
  int c_bdiv;
  long long c_bs_hi;
};

// Tensor maps of the output: one per destination buffer. More than one destination is how a rank that owns a
// column block of the result writes it straight into every rank's copy of the full matrix (peer pointers).
constexpr int kMaxOut = 8;
struct OutMaps {
  CUtensorMap m[kMaxOut];
};

constexpr int kBM = 128;
// Cycle probes for tuning (compiled only with -DB200AIT_GEMM_PROBE; never part of the shipped library): CTA 0's MMA
// thread and first epilogue warp add the clock64() time they spend in each phase to g_gemm_probe[slot].
#ifdef B200AIT_GEMM_PROBE
static __device__ long long g_gemm_probe[32];  // one copy per translation unit (no relocatable device code)
#define GEMM_PROBE_DECL(cond)            \
  const bool probe_on = (cond);          \
  long long probe_acc[4] = {0, 0, 0, 0}; \
  long long probe_t = clock64();
#define GEMM_PROBE(slot)                          \
  if (probe_on) {                                 \
    const long long probe_now = clock64();        \
    probe_acc[(slot) & 3] += probe_now - probe_t; \
    probe_t = probe_now;                          \
  }
#define GEMM_PROBE_FLUSH(base)                                                  \
  if (probe_on) {                                                               \
    for (int pi = 0; pi < 4; ++pi) g_gemm_probe[(base) + pi] += probe_acc[pi];  \
  }
#else
#define GEMM_PROBE_DECL(cond)
#define GEMM_PROBE(slot)
#define GEMM_PROBE_FLUSH(base)
#endif

constexpr int kBK = 64;
constexpr int kGroupM = 8;
constexpr int kEpiWarps = 8;                      // two per TMEM lane quarter, each takes half of the columns
constexpr int kGemmThreads = 64 + 32 * kEpiWarps;  // producer warp + MMA warp + epilogue warps

// PAIR: two CTAs of a cluster compute one 256 x BN tile with cta_group::2 MMAs. Each CTA loads its own 128
// rows of A and its own half (BN / 2 rows) of B, so a CTA moves 2/3 of the bytes per flop of the
// single-CTA 128 x 256 tile, and keeps its own 128 x BN half of the accumulator.
// D0BOX: the residual operand d0 is fetched by TMA into the output staging boxes (two boxes per epilogue
// warp, one ring stage fewer) and combined in place, instead of per-thread global loads.
template <int BN, bool PAIR = false, bool D0BOX = false>
struct TileCfg {
  static_assert(!D0BOX || PAIR, "staged residual boxes are only built for the CTA-pair tile");
  static constexpr int kBRows = PAIR ? BN / 2 : BN;  // B rows this CTA loads per stage
  static constexpr int kStageBytes = kBM * kBK * 2 + kBRows * kBK * 2;
  static constexpr int kStages = PAIR ? (D0BOX ? 5 : 6) : (BN == 256) ? 4 : (BN == 128) ? 6 : 8;
  static constexpr int kTmemCols = 2 * BN;  // two accumulators
  static constexpr int kBoxesPerWarp = D0BOX ? 2 : 1;  // 32 rows x 64 columns x 16 bit = 4 KB each
  static constexpr int kStagingBytes = (BN >= 128) ? kEpiWarps * kBoxesPerWarp * 4096 : 0;
  static constexpr int kBarrierBytes = 512;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + kBarrierBytes +
                                    2 * BN * 4 /*bias tile, fp32, one per accumulator*/;
};

// whether the compile-time epilogue code EPI takes its residual through staged boxes
template <int EPI, bool PAIR>
__host__ __device__ constexpr bool d0_box_of() {
  return PAIR && EPI >= 0 && epi_b1(EPI) != kBinaryNone && epi_b2(EPI) == kBinaryNone;
}

__device__ __forceinline__ void decode_tile(const GemmParams& p, int tile, int& b, int& m_blk, int& n_blk) {
  const int per_batch = p.tiles_m * p.tiles_n;
  b = tile / per_batch;
  const int t = tile - b * per_batch;
  const int group_size = kGroupM * p.tiles_n;
  const int g = t / group_size;
  const int first_m = g * kGroupM;
  const int gm = min(kGroupM, p.tiles_m - first_m);
  const int r = t - g * group_size;
  m_blk = first_m + r % gm;
  n_blk = r / gm;
}

// offset (in elements) of batch b of the output
__device__ __forceinline__ long long batch_offset(const GemmParams& p, int b) {
  if (p.c_bdiv == 0) return static_cast<long long>(b) * p.c_bs;
  const int hi = b / p.c_bdiv;
  return hi * p.c_bs_hi + (b - hi * p.c_bdiv) * p.c_bs;
}
// offset (in elements) of output element (row, col) relative to the batch base
__device__ __forceinline__ long long row_offset(const GemmParams& p, int row) {
  if (p.store_mode == 0) return static_cast<long long>(row) * p.ldc;
  const int hi = row / p.t1;
  return hi * p.rs_hi + (row - hi * p.t1) * p.rs_lo;
}
__device__ __forceinline__ long long col_offset(const GemmParams& p, int col) {
  if (p.store_mode == 0) return col;
  const int c = col / p.d;
  const int c2 = c / p.t3;
  return c2 * p.cs2 + (c - c2 * p.t3) * p.cs3 + (col - c * p.d);
}

// Applies the epilogue to 32 consecutive columns of one row and stores them.
template <bool BF16>
__device__ __forceinline__ void epilogue_chunk32(const GemmParams& p, float (&v)[32], int b, int row, int col0,
                                                 bool row_ok) {
  using E = Elem16<BF16>;
  using T = typename E::T;
  const int u1 = epi_u1(p.epilogue), b1 = epi_b1(p.epilogue), b2 = epi_b2(p.epilogue), u2 = epi_u2(p.epilogue);
  const bool full = p.vec_ok && (col0 + 32 <= p.N);
  if (p.alpha != 1.f) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] *= p.alpha;
  }
  if (p.bias != nullptr) {
    const T* bias = static_cast<const T*>(p.bias) + col0;
    if (full) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float f[8];
        unpack8<BF16>(__ldg(reinterpret_cast<const uint4*>(bias) + q), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[q * 8 + j] += f[j];
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) v[j] += E::to_float(bias[j]);
    }
  }
  apply_unary_vec(u1, v);
  if (!row_ok) return;
  const long long d_base = static_cast<long long>(b) * p.d_bs + static_cast<long long>(row) * p.ldd + col0;
  if (b1 != kBinaryNone) {
    const T* d0 = static_cast<const T*>(p.d0) + d_base;
    if (full) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float f[8];
        unpack8<BF16>(__ldg(reinterpret_cast<const uint4*>(d0) + q), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[q * 8 + j] = (b1 == kBinaryAdd) ? v[q * 8 + j] + f[j] : v[q * 8 + j] * f[j];
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) {
          const float f = E::to_float(d0[j]);
          v[j] = (b1 == kBinaryAdd) ? v[j] + f : v[j] * f;
        }
    }
  }
  if (b2 != kBinaryNone) {
    const T* d1 = static_cast<const T*>(p.d1) + d_base;
    if (full) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float f[8];
        unpack8<BF16>(__ldg(reinterpret_cast<const uint4*>(d1) + q), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[q * 8 + j] = (b2 == kBinaryAdd) ? v[q * 8 + j] + f[j] : v[q * 8 + j] * f[j];
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) {
          const float f = E::to_float(d1[j]);
          v[j] = (b2 == kBinaryAdd) ? v[j] + f : v[j] * f;
        }
    }
  }
  apply_unary_vec(u2, v);
  T* out = static_cast<T*>(p.out) + batch_offset(p, b) + row_offset(p, row);
  if (full) {
    if (p.store_mode == 0) {
#pragma unroll
      for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(out + col0 + q * 8) = pack8<BF16>(&v[q * 8]);
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q)
        *reinterpret_cast<uint4*>(out + col_offset(p, col0 + q * 8)) = pack8<BF16>(&v[q * 8]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < p.N) out[col_offset(p, col0 + j)] = E::from_float(v[j]);
  }
}


// EPI >= 0 fixes the epilogue code at compile time (straight-line code for the common epilogues);
// EPI == -1 reads it from the parameters.
template <int EPI>
__device__ __forceinline__ int epilogue_code_of(const GemmParams& p) {
  return EPI >= 0 ? EPI : p.epilogue;
}

// Fused epilogue math of the tensor-core kernel for 32 consecutive columns of one row. `v` already
// holds alpha * acc + bias. d0 is prefetched by the caller (d0v valid when the chunk is `full`).
template <bool BF16, int EPI>
__device__ __forceinline__ void epilogue_math32(const GemmParams& p, float (&v)[32], const uint4 (&d0v)[4], int b,
                                                int row, int col0, bool full, bool row_ok) {
  using E = Elem16<BF16>;
  using T = typename E::T;
  const int code = epilogue_code_of<EPI>(p);
  const int u1 = epi_u1(code), b1 = epi_b1(code), b2 = epi_b2(code), u2 = epi_u2(code);
  apply_unary_vec(u1, v);
  const long long d_base = static_cast<long long>(b) * p.d_bs + static_cast<long long>(row) * p.ldd + col0;
  if (b1 != kBinaryNone && row_ok) {
    if (full) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float f[8];
        unpack8<BF16>(d0v[q], f);
#pragma unroll
        for (int j = 0; j < 8; j += 2) {  // two elements per instruction
          const uint64_t x = pack2(v[q * 8 + j], v[q * 8 + j + 1]), y = pack2(f[j], f[j + 1]);
          unpack2((b1 == kBinaryAdd) ? add2(x, y) : mul2(x, y), v[q * 8 + j], v[q * 8 + j + 1]);
        }
      }
    } else {
      const T* d0 = static_cast<const T*>(p.d0) + d_base;
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) {
          const float f = E::to_float(d0[j]);
          v[j] = (b1 == kBinaryAdd) ? v[j] + f : v[j] * f;
        }
    }
  }
  if (b2 != kBinaryNone && row_ok) {
    const T* d1 = static_cast<const T*>(p.d1) + d_base;
    if (full) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float f[8];
        unpack8<BF16>(__ldg(reinterpret_cast<const uint4*>(d1) + q), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[q * 8 + j] = (b2 == kBinaryAdd) ? v[q * 8 + j] + f[j] : v[q * 8 + j] * f[j];
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) {
          const float f = E::to_float(d1[j]);
          v[j] = (b2 == kBinaryAdd) ? v[j] + f : v[j] * f;
        }
    }
  }
  apply_unary_vec(u2, v);
}

// Direct register -> global store of 32 consecutive columns of one row.
template <bool BF16>
__device__ __forceinline__ void epilogue_direct_store32(const GemmParams& p, const float (&v)[32], int b, int row,
                                                        int col0, bool full, bool chunk_contig) {
  using E = Elem16<BF16>;
  using T = typename E::T;
  T* out = static_cast<T*>(p.out) + batch_offset(p, b) + row_offset(p, row);
  if (full) {
    if (chunk_contig) {
      T* dst = out + col_offset(p, col0);
#pragma unroll
      for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(dst + q * 8) = pack8<BF16>(&v[q * 8]);
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q)
        *reinterpret_cast<uint4*>(out + col_offset(p, col0 + q * 8)) = pack8<BF16>(&v[q * 8]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < p.N) out[col_offset(p, col0 + j)] = E::from_float(v[j]);
  }
}

// BMN: B is stored [K, N]. MULTI: the staged store goes to p.num_out destinations. Both are compile-time, so that
// the plain [N, K] single-destination kernels carry no trace of them (a run-time flag cost the BERT-layer GEMMs
// 2-3 %), and both are only instantiated with the generic epilogue (EPI == -1).
template <int BN, bool BF16, int EPI, bool PAIR, bool BMN = false, bool MULTI = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
               const __grid_constant__ CUtensorMap tma_out, const __grid_constant__ CUtensorMap tma_d0,
               const GemmParams p, const __grid_constant__ OutMaps outs) {
  // `tma_out` is the (first) destination; `outs.m[1..]` are the extra destinations of a multi-destination store
  // and sit at the end of the parameter space, out of the way of what every launch reads.
  constexpr bool D0BOX = d0_box_of<EPI, PAIR>();
  using Cfg = TileCfg<BN, PAIR, D0BOX>;
  constexpr int kStages = Cfg::kStages;
  constexpr uint32_t kABytes = kBM * kBK * 2;
  constexpr uint32_t kStageBytes = Cfg::kStageBytes;

  extern __shared__ __align__(1024) uint8_t smem[];
  // Swizzled tiles need 1024-byte alignment. A misaligned CTA does no work but still walks through every
  // CTA-wide and cluster-wide barrier below.
  const bool misaligned = (smem_u32(smem) & 1023u) != 0u;
  if (misaligned && threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, kDevBadSmemAlignment);
  const int num_units = misaligned ? 0 : p.num_units;
  // Lean kernels: a compile-time epilogue on a tile wide enough for the staged TMA store, launched only for
  // alpha = 1, no split-K, the staged store and (with a residual: CTA pairs only) staged residual boxes. Their
  // code carries none of the other paths, which is worth several per cent on the short-K GEMMs.
  constexpr bool kLean = EPI >= 0 && BN >= 128 && (PAIR || epi_b1(EPI < 0 ? 0 : EPI) == kBinaryNone);
  const int splits = (PAIR || kLean) ? 1 : p.splits;  // CTA pairs never split K either
  // Work distribution: a single CTA, or a pair of CTAs (cluster ranks 0 and 1), walks the units.
  const int pair_rank = PAIR ? static_cast<int>(cluster_ctarank()) : 0;
  const int walker = PAIR ? (blockIdx.x >> 1) : blockIdx.x;
  const int num_walkers = PAIR ? (gridDim.x >> 1) : gridDim.x;
  uint8_t* staging = smem + kStages * kStageBytes;  // [kEpiWarps][32 rows][128 B], 128-byte swizzled
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(staging + Cfg::kStagingBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* acc_full = empty_bar + kStages;
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* drain_bar = acc_empty + 2;
  uint64_t* d0_bar = drain_bar + 1;  // [kEpiWarps][2]: a residual box has landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d0_bar + 2 * kEpiWarps);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  static_assert((2 * kStages + 5 + 2 * kEpiWarps) * 8 + 8 <= Cfg::kBarrierBytes, "barrier area too small");
  float* sbias = reinterpret_cast<float*>(staging + Cfg::kStagingBytes + Cfg::kBarrierBytes);  // [2][BN]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.K + kBK - 1) / kBK;
#ifdef B200AIT_GEMM_PROBE
  if (blockIdx.x == 0 && threadIdx.x == 0) g_gemm_probe[15] = clock64();  // kernel start
#endif

  // Set-up in parallel (a small problem's whole run is a few microseconds): lane 0 of warp 0 asks for the tensor maps,
  // the lanes of warp 0 initialise one barrier each, warp 1 allocates tensor memory meanwhile. The barriers lie in
  // shared memory as full[kStages], empty[kStages], acc_full[2], acc_empty[2], drain_bar, d0_bar[2 * kEpiWarps].
  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      if (p.tma_store) {
        tma_prefetch_desc(&tma_out);
        if (MULTI)
          for (int i = 1; i < p.num_out; ++i) tma_prefetch_desc(&outs.m[i]);
      }
      if (D0BOX && p.tma_d0) tma_prefetch_desc(&tma_d0);
      *abort_flag = 0;
    }
    constexpr int kBars = 2 * kStages + 5 + 2 * kEpiWarps;
    for (int i = lane; i < kBars; i += 32) {
      const int j = i - 2 * kStages;
      // acc_empty: the leader hears from both CTAs' epilogues
      mbar_init(&full_bar[i], (j == 2 || j == 3) ? static_cast<uint32_t>((PAIR ? 2 : 1) * 32 * kEpiWarps) : 1u);
    }
    fence_mbar_init();
  } else if (warp == 1) {
    if (PAIR) {  // the same warp of both CTAs, same result slot
      tmem_alloc_pair(tmem_slot, Cfg::kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, Cfg::kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  // the peer's barriers are initialised before anything signals them (no release needed on the arrive: the
  // initialisations are published by fence.mbarrier_init, and a releasing arrive costs about 0.5 us)
  if (PAIR) cluster_arrive_relaxed();
  __syncthreads();
  if (PAIR) cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = walker; ok && unit < num_units; unit += num_walkers) {
        int b, m_blk, n_blk;
        const int tile = unit / splits, split = unit - tile * splits;
        decode_tile(p, tile, b, m_blk, n_blk);
        if (PAIR) m_blk = 2 * m_blk + pair_rank;
        const int kb0 = split * p.kb_per_split, kb1 = min(num_kb, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, kDevWaitEmptyTimeout);
          if (!ok) break;
          uint8_t* sa = smem + stage * kStageBytes;
          if (PAIR) {
            // Both CTAs' copies are credited to the leader's barrier, which expects the bytes of both.
            const uint32_t leader_bar = mapa_shared(smem_u32(&full_bar[stage]), 0);
            if (pair_rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * kStageBytes);
            tma_load_3d_pair(sa, &tma_a, leader_bar, kb * kBK, m_blk * kBM, b * p.a_batch_mul);
            const int n0 = n_blk * BN + pair_rank * (BN / 2);
            if (BMN) {  // [K, N] storage: one box of 64 k-rows x 64 columns per 64-column chunk
#pragma unroll
              for (int ch = 0; ch < Cfg::kBRows / 64; ++ch)
                tma_load_3d_pair(sa + kABytes + ch * 8192, &tma_b, leader_bar, n0 + ch * 64, kb * kBK,
                                 b * p.b_batch_mul);
            } else {
              tma_load_3d_pair(sa + kABytes, &tma_b, leader_bar, kb * kBK, n0, b * p.b_batch_mul);
            }
          } else {
            mbar_arrive_expect_tx(&full_bar[stage], kStageBytes);
            tma_load_3d(sa, &tma_a, &full_bar[stage], kb * kBK, m_blk * kBM, b * p.a_batch_mul);
            if (BMN) {
#pragma unroll
              for (int ch = 0; ch < Cfg::kBRows / 64; ++ch)
                tma_load_3d(sa + kABytes + ch * 8192, &tma_b, &full_bar[stage], n_blk * BN + ch * 64, kb * kBK,
                            b * p.b_batch_mul);
            } else {
              tma_load_3d(sa + kABytes, &tma_b, &full_bar[stage], kb * kBK, n_blk * BN, b * p.b_batch_mul);
            }
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (PAIR) {
        // The leader's MMA commits release stages in BOTH CTAs: wait until every release addressed to this
        // CTA has landed, so that none arrives after the CTA has gone.
        for (int s = 0; ok && s < kStages; ++s) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, kDevWaitEmptyTimeout);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // give copies that are still in flight a bounded time to land before the CTA exits
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0 && pair_rank == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(PAIR ? 2 * kBM : kBM, BN, BF16, false, BMN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      GEMM_PROBE_DECL(blockIdx.x == 0)
      for (int unit = walker; ok && unit < num_units; unit += num_walkers) {
        GEMM_PROBE(3)  // other
        ok = mbar_wait(&acc_empty[acc], acc_phase ^ 1u, abort_flag, p.status, kDevWaitAccEmptyTimeout);
        if (!ok) break;
        tc_fence_after();
        GEMM_PROBE(0)  // waiting for a free accumulator
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        const int split = unit % splits;
        const int kb0 = split * p.kb_per_split, kb1 = min(num_kb, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          GEMM_PROBE(2)  // issuing MMAs and commits
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kDevWaitFullTimeout);
          if (!ok) break;
          tc_fence_after();
          GEMM_PROBE(1)  // waiting for operands
          const uint32_t a_addr = smem_u32(smem + stage * kStageBytes);
          const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t adesc = umma_smem_desc_sw128(a_addr + k * 32, 16, 1024);
            // [N, K] storage: K-major tile, 32 bytes per k-step. [K, N] storage: MN-major tile, rows are k (128 B
            // each): 16 k-rows = 2048 B per k-step, 64-column chunks 8192 B apart, 8-row groups 1024 B apart.
            const uint64_t bdesc = BMN ? umma_smem_desc_sw128(b_addr + k * 2048, 8192, 1024)
                                       : umma_smem_desc_sw128(b_addr + k * 32, 16, 1024);
            if (PAIR) {
              umma_f16_ss_pair(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k != 0) ? 1u : 0u);
            } else {
              umma_f16_ss(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k != 0) ? 1u : 0u);
            }
          }
          if (PAIR) {
            umma_commit_pair(&empty_bar[stage], 3);  // frees this stage in both CTAs
          } else {
            umma_commit(&empty_bar[stage]);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if (PAIR) {
          umma_commit_pair(&acc_full[acc], 3);  // both CTAs' epilogues read their half
        } else {
          umma_commit(&acc_full[acc]);
        }
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
        GEMM_PROBE(2)
      }
      GEMM_PROBE_FLUSH(0)
#ifdef B200AIT_GEMM_PROBE
      if (blockIdx.x == 0) g_gemm_probe[16] = clock64();  // end of the MMA thread's work
#endif
      if (!ok) {
        // let MMAs that were already issued finish before TMEM is released
        if (PAIR) {
          umma_commit_pair(drain_bar, 1);
        } else {
          umma_commit(drain_bar);
        }
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(drain_bar, 0) && globaltimer_ns() - t0 < 1000000ull) {
        }
      }
    }
    __syncwarp();
  } else {
    // ----------------------------------------------------------------- epilogue
    // Warp w of the eight reads TMEM lanes [32*(warp%4), +32) (a hardware rule) and the column half
    // w / 4 of the tile. Per tile: stage the bias slice in shared memory while the MMAs still run,
    // then walk the chunks with the next chunk's TMEM load and residual load already in flight.
    using E = Elem16<BF16>;
    using T = typename E::T;
    constexpr int kChunksPerWarp = BN / 64;  // 32-column chunks per warp
    const int ew = warp - 2;
    const int quarter = warp & 3;
    const int half = ew >> 2;
    const int et = threadIdx.x - 64;  // 0..255
    const int code = epilogue_code_of<EPI>(p);
    const bool has_d0 = epi_b1(code) != kBinaryNone;
    const bool has_bias = p.bias != nullptr && splits == 1;
    const bool chunk_contig = p.store_mode == 0 || (p.d % 32 == 0);
    const bool use_tma = kLean || ((BN >= 128) && p.tma_store != 0);
    // residual through staging boxes: needs the TMA store path and a tensor map over d0
    const bool box_d0 = D0BOX && (kLean || (use_tma && p.tma_d0 != 0));
    uint8_t* my_staging = staging + ew * (Cfg::kBoxesPerWarp * 4096);
    uint64_t* my_d0_bar = d0_bar + 2 * ew;
    uint32_t d0_phase_bits = 0;  // bit i: parity to wait for on my_d0_bar[i]
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const uint32_t acc_empty_leader[2] = {PAIR ? mapa_shared(smem_u32(&acc_empty[0]), 0) : 0u,
                                          PAIR ? mapa_shared(smem_u32(&acc_empty[1]), 0) : 0u};
    GEMM_PROBE_DECL(blockIdx.x == 0 && threadIdx.x == 64)
    for (int unit = walker; ok && unit < num_units; unit += num_walkers) {
      GEMM_PROBE(3)  // epilogue warp: other
      int b, m_blk, n_blk;
      const int tile = unit / splits, split = unit - tile * splits;
      decode_tile(p, tile, b, m_blk, n_blk);
      if (PAIR) m_blk = 2 * m_blk + pair_rank;
      const int colh = n_blk * BN + half * (BN / 2);  // first column of this warp's half
      const int row0 = m_blk * kBM + quarter * 32;    // first row of this warp
      if (box_d0) {
        // Fetch this warp's two 32 x 64 residual boxes into its staging buffers while the tile's MMAs run.
        // The previous tile's stores must have finished reading the buffers first.
        if (lane == 0) {
          bulk_wait_group_read0();
#pragma unroll
          for (int bx = 0; bx < 2; ++bx) {
            const int gcol = colh + bx * 64;
            if (row0 < p.M && gcol < p.N) {
              mbar_arrive_expect_tx(&my_d0_bar[bx], 4096);
              tma_load_3d(my_staging + bx * 4096, &tma_d0, &my_d0_bar[bx], gcol, row0, b);
            }
          }
        }
        __syncwarp();
      }
      float* bias_s = sbias + acc * BN;
      if (has_bias) {  // CTA-uniform
        if (et < BN) {
          const int col = n_blk * BN + et;
          bias_s[et] = col < p.N ? E::to_float(static_cast<const T*>(p.bias)[col]) : 0.f;
        }
        named_bar_sync(1, 32 * kEpiWarps);
      }
      const int row = m_blk * kBM + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const T* d0_row = static_cast<const T*>(p.d0) + static_cast<long long>(b) * p.d_bs + static_cast<long long>(row) * p.ldd;
      uint4 d0v[4];
      auto prefetch_d0 = [&](int col0) {
        if (has_d0 && row_ok && p.vec_ok && col0 + 32 <= p.N) {
#pragma unroll
          for (int q = 0; q < 4; ++q) d0v[q] = __ldg(reinterpret_cast<const uint4*>(d0_row + col0) + q);
        }
      };
      if (splits == 1 && !box_d0) prefetch_d0(colh);
      GEMM_PROBE(0)  // tile set-up: residual boxes issued, bias staged, epilogue barrier
      ok = mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.status, kDevWaitAccFullTimeout);
      if (!ok) break;
      tc_fence_after();
      GEMM_PROBE(1)  // waiting for the accumulator
      const uint32_t t_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                              static_cast<uint32_t>(acc * BN + half * (BN / 2));
      // Two register buffers alternate between "being read" and "being loaded", so that a chunk is used where
      // tcgen05.ld put it. The accumulator goes back to the MMA warp as soon as its last chunk is in registers.
      uint32_t ra[32], rb[32];
      bool released = false;
      tmem_ld_32x32b_x32(t_base, ra);
      auto chunk_step = [&](const int c, uint32_t (&cur)[32], uint32_t (&nxt)[32]) {
        if (!ok) return;
        const int col0 = colh + c * 32;
        tmem_ld_wait();
        uint4 d0c[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) d0c[q] = d0v[q];
        if (c + 1 < kChunksPerWarp && col0 + 32 < p.N) {  // next chunk's loads go out before this chunk's math
          tmem_ld_32x32b_x32(t_base + static_cast<uint32_t>((c + 1) * 32), nxt);
          if (splits == 1 && !box_d0) prefetch_d0(col0 + 32);
        } else if (!released) {
          released = true;
          tc_fence_before();
          if (PAIR) {
            // relaxed: the leader depends on this thread's TMEM reads (fenced above), not on its memory writes; a
            // release at cluster scope would wait here for the staged stores of the earlier chunks
            mbar_arrive_cluster_relaxed(acc_empty_leader[acc]);
          } else {
            mbar_arrive(&acc_empty[acc]);
          }
        }
        if (col0 >= p.N) return;  // warp-uniform
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(cur[j]);
        const bool full = p.vec_ok && (col0 + 32 <= p.N);
        if (splits > 1) {
          // split-K: raw fp32 partial sums; the reduce kernel applies the epilogue
          if (row_ok) {
            float* dst = p.partial + ((static_cast<long long>(split) * p.batch + b) * p.M + row) * p.N + col0;
            if (full) {
#pragma unroll
              for (int q = 0; q < 8; ++q)
                *reinterpret_cast<float4*>(dst + q * 4) = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) dst[j] = v[j];
            }
          }
          return;
        }
        if (!kLean && p.alpha != 1.f) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= p.alpha;
        }
        if (has_bias) {
          const float* bs = bias_s + half * (BN / 2) + c * 32;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 f = *reinterpret_cast<const float4*>(bs + q * 4);
            unpack2(add2(pack2(v[q * 4], v[q * 4 + 1]), pack2(f.x, f.y)), v[q * 4], v[q * 4 + 1]);
            unpack2(add2(pack2(v[q * 4 + 2], v[q * 4 + 3]), pack2(f.z, f.w)), v[q * 4 + 2], v[q * 4 + 3]);
          }
        }
        if (use_tma) {
          // Stage this warp's 32 rows x 64 columns (two chunks) in 128-byte-swizzled shared memory and
          // let TMA write the box: full 128-byte lines reach L2, rows / columns past M / N are clipped.
          uint8_t* box = my_staging + (box_d0 ? (c >> 1) * 4096 : 0);
          uint8_t* row_base = box + lane * 128;
          if (box_d0) {
            // the residual box sits where the output box will be written: combine in place
            if ((c & 1) == 0 && row0 < p.M) {
              const int bx = c >> 1;
              ok = mbar_wait(&my_d0_bar[bx], (d0_phase_bits >> bx) & 1u, abort_flag, p.status, kDevWaitOtherTimeout);
              d0_phase_bits ^= 1u << bx;
              if (!ok) return;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
              d0c[u] = *reinterpret_cast<const uint4*>(row_base + ((((c & 1) * 4 + u) ^ (lane & 7)) * 16));
          }
          epilogue_math32<BF16, EPI>(p, v, d0c, b, row, col0, full || box_d0, row_ok);
          if (!box_d0 && (c & 1) == 0) {  // the box buffer is about to be rewritten: its last store must have read it
            if (lane == 0) bulk_wait_group_read0();
            __syncwarp();
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int unit = ((c & 1) * 4 + u) ^ (lane & 7);
            *reinterpret_cast<uint4*>(row_base + unit * 16) = pack8<BF16>(&v[u * 8]);
          }
          if ((c & 1) != 0 || col0 + 32 >= p.N) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0 && row0 < p.M) {  // a box that starts past the last row has nothing to write
              const int gcol = colh + (c & ~1) * 32;
              if (p.store_mode == 0) {
                int b_lo = b, b_hi = 0;
                if (EPI < 0 && p.c_bdiv != 0) b_hi = b / p.c_bdiv, b_lo = b - b_hi * p.c_bdiv;
                tma_store_5d(&tma_out, box, gcol, row0, b_lo, b_hi, 0);
                if (MULTI)
                  for (int i = 1; i < p.num_out; ++i) tma_store_5d(&outs.m[i], box, gcol, row0, b, 0, 0);
              } else {
                const int cc = gcol / p.d, r_b = row0 / p.t1;
                tma_store_5d(&tma_out, box, gcol - cc * p.d, row0 - r_b * p.t1, cc % p.t3, r_b, cc / p.t3);
                if (MULTI)
                  for (int i = 1; i < p.num_out; ++i)
                    tma_store_5d(&outs.m[i], box, gcol - cc * p.d, row0 - r_b * p.t1, cc % p.t3, r_b, cc / p.t3);
              }
              bulk_commit_group();
            }
          }
        } else if (row_ok) {
          epilogue_math32<BF16, EPI>(p, v, d0c, b, row, col0, full, true);
          epilogue_direct_store32<BF16>(p, v, b, row, col0, full, chunk_contig);
        }
      };
#pragma unroll 1
      for (int c = 0; c < kChunksPerWarp; c += 2) {  // one copy of the two-chunk body: less code to fetch
        chunk_step(c, ra, rb);
        if (c + 1 < kChunksPerWarp) chunk_step(c + 1, rb, ra);
      }
      if (!ok) break;
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
      GEMM_PROBE(2)  // the tile's chunks: TMEM loads, residual, math, staging, stores
    }
    GEMM_PROBE_FLUSH(4)
#ifdef B200AIT_GEMM_PROBE
    if (blockIdx.x == 0 && threadIdx.x == 64) g_gemm_probe[17] = clock64();
#endif
    if (use_tma && lane == 0) bulk_wait_group0();  // shared memory must outlive the stores that read it
  }

  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // neither CTA leaves, or frees TMEM, while its peer can still signal or read it
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) {
      tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    } else {
      tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
  }
}

template <int BN, bool BF16, int EPI, bool BMN = false, bool MULTI = false>
void launch_tc(const CUtensorMap& ta, const CUtensorMap& tb, const OutMaps& tout, const GemmParams& p, int grid,
               cudaStream_t stream) {
  using Cfg = TileCfg<BN>;
  static std::atomic<uint64_t> configured{0};
  opt_in_smem_once(configured, reinterpret_cast<const void*>(&gemm_tc_kernel<BN, BF16, EPI, false, BMN, MULTI>),
                   Cfg::kSmemBytes);
  ::b200ait::count_launch(), gemm_tc_kernel<BN, BF16, EPI, false, BMN, MULTI><<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(
      ta, tb, tout.m[0], ta, p, tout);
  B200AIT_CUDA_CHECK(cudaGetLastError());
}

// CTA-pair variant: `grid` counts CTAs (twice the number of pairs); launched as clusters of two.
template <int BN, bool BF16, int EPI, bool BMN = false, bool MULTI = false>
void launch_tc_pair(const CUtensorMap& ta, const CUtensorMap& tb, const OutMaps& tout, const CUtensorMap& td0,
                    const GemmParams& p, int grid, cudaStream_t stream) {
  using Cfg = TileCfg<BN, true, d0_box_of<EPI, true>()>;
  static std::atomic<uint64_t> configured{0};
  auto* kernel = &gemm_tc_kernel<BN, BF16, EPI, true, BMN, MULTI>;
  opt_in_smem_once(configured, reinterpret_cast<const void*>(kernel), Cfg::kSmemBytes);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  ::b200ait::count_launch();
  B200AIT_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, ta, tb, tout.m[0], td0, p, tout));
}

// Epilogues that get their own straight-line instantiation (fp16): bias, relu, gelu, fast_gelu, add,
// add_relu, mul. Everything else, and bf16, runs the generic instantiation.
#define B200AIT_FOR_EACH_FAST_EPILOGUE(X)                                                  \
  X(make_epilogue(kUnaryIdentity, kBinaryNone, kBinaryNone, kUnaryIdentity))              \
  X(make_epilogue(kUnaryRelu, kBinaryNone, kBinaryNone, kUnaryIdentity))                  \
  X(make_epilogue(kUnaryGelu, kBinaryNone, kBinaryNone, kUnaryIdentity))                  \
  X(make_epilogue(kUnaryFastGelu, kBinaryNone, kBinaryNone, kUnaryIdentity))              \
  X(make_epilogue(kUnaryIdentity, kBinaryAdd, kBinaryNone, kUnaryIdentity))               \
  X(make_epilogue(kUnaryIdentity, kBinaryAdd, kBinaryNone, kUnaryRelu))                   \
  X(make_epilogue(kUnaryIdentity, kBinaryMul, kBinaryNone, kUnaryIdentity))

// Defined once per tile width in gemm_bn<BN>.cu.
template <int BN>
void launch_tc_width(bool bf16, const CUtensorMap& ta, const CUtensorMap& tb, const OutMaps& tout,
                     const GemmParams& p, int grid, cudaStream_t stream);

template <>
void launch_tc_width<64>(bool, const CUtensorMap&, const CUtensorMap&, const OutMaps&, const GemmParams&, int,
                          cudaStream_t);
template <>
void launch_tc_width<128>(bool, const CUtensorMap&, const CUtensorMap&, const OutMaps&, const GemmParams&, int,
                          cudaStream_t);
template <>
void launch_tc_width<256>(bool, const CUtensorMap&, const CUtensorMap&, const OutMaps&, const GemmParams&, int,
                          cudaStream_t);

// CTA-pair kernel, 256 x 256 tiles; defined in gemm_pair256.cu.
void launch_tc_pair256(bool bf16, const CUtensorMap& ta, const CUtensorMap& tb, const OutMaps& tout,
                       const CUtensorMap& td0, const GemmParams& p, int grid, cudaStream_t stream);

void launch_tc_pair256_bf16_lean(const CUtensorMap& ta, const CUtensorMap& tb, const OutMaps& tout,
                                 const CUtensorMap& td0, const GemmParams& p, int grid, cudaStream_t stream);

#define B200AIT_DEFINE_LAUNCH_TC_WIDTH(BN_)                                                                    \
  template <>                                                                                                  \
  void launch_tc_width<BN_>(bool bf16, const CUtensorMap& ta, const CUtensorMap& tb, const OutMaps& tout,  \
                            const GemmParams& p, int grid, cudaStream_t stream) {                              \
    if (p.c_bdiv != 0 && p.num_out == 1 && !p.b_mn) { /* batched 0213 store: generic epilogue only */          \
      if (bf16)                                                                                                \
        launch_tc<BN_, true, -1>(ta, tb, tout, p, grid, stream);                                               \
      else                                                                                                     \
        launch_tc<BN_, false, -1>(ta, tb, tout, p, grid, stream);                                              \
      return;                                                                                                  \
    }                                                                                                          \
    if (p.num_out > 1) { /* several destinations: generic epilogue instantiation only */                       \
      if (bf16)                                                                                                \
        launch_tc<BN_, true, -1, false, true>(ta, tb, tout, p, grid, stream);                                  \
      else                                                                                                     \
        launch_tc<BN_, false, -1, false, true>(ta, tb, tout, p, grid, stream);                                 \
      return;                                                                                                  \
    }                                                                                                          \
    if (p.b_mn) { /* B stored [K, N]: generic epilogue instantiation only */                                   \
      if (bf16)                                                                                                \
        launch_tc<BN_, true, -1, true>(ta, tb, tout, p, grid, stream);                                         \
      else                                                                                                     \
        launch_tc<BN_, false, -1, true>(ta, tb, tout, p, grid, stream);                                        \
      return;                                                                                                  \
    }                                                                                                          \
    if (bf16) {                                                                                                \
      launch_tc<BN_, true, -1>(ta, tb, tout, p, grid, stream);                                                 \
      return;                                                                                                  \
    }                                                                                                          \
    /* the compile-time-epilogue kernels of the wide tiles are lean (see the kernel): anything else is generic */ \
    const bool lean_ok = BN_ < 128 || epi_b1(p.epilogue) != kBinaryNone ||                                     \
                         (p.alpha == 1.f && p.tma_store != 0 && p.splits == 1);                                \
    if (!lean_ok) {                                                                                            \
      launch_tc<BN_, false, -1>(ta, tb, tout, p, grid, stream);                                                \
      return;                                                                                                  \
    }                                                                                                          \
    switch (p.epilogue) {                                                                                      \
      B200AIT_FOR_EACH_FAST_EPILOGUE(B200AIT_CASE_##BN_)                                                       \
      default:                                                                                                 \
        launch_tc<BN_, false, -1>(ta, tb, tout, p, grid, stream);                                              \
    }                                                                                                          \
  }

}  // namespace b200ait
