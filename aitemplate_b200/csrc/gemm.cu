// gemm_rcr / bmm_rcr family for sm_100a: Y[b] = epilogue(alpha * X[b] . W[b]^T + bias, D0, D1)
// with X [M,K] and W [N,K] both K-contiguous ("RCR": row-major A, column-major B, row-major C).
//
// Replaces the reference's CUTLASS / CuTe-DSL template instantiation for
//   gemm_rcr            python/aitemplate/backend/cuda/gemm_universal/gemm_rcr.py:148-315
//   gemm_rcr_bias*      .../gemm_rcr_bias.py:39-61, common_bias_activation.py, common_bias_broadcast.py:86-128
//   gemm_rcr_bias_permute  .../gemm_rcr_bias_permute.py:55-95, common_permute.py:88-107
//   bmm_rcr             .../bmm_xxx.py:30-155, bmm_common.py:200-434
// by one persistent, warp-specialised kernel:
//   warp 0      TMA producer: cp.async.bulk.tensor loads of 128x64 (A) and BNx64 (B) tiles into a
//               128-byte-swizzled shared-memory ring guarded by full/empty mbarriers
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16) into one of two TMEM
//               accumulators, tcgen05.commit releases smem stages / publishes the accumulator
//   warps 2-5   epilogue: tcgen05.ld of this warp's 32 TMEM lanes, bias / activation / residual in
//               fp32, one rounding, 16-byte global stores (row-major with stride, or permuted)
// The epilogue of tile i overlaps the main loop of tile i+1 (two accumulators).
// Shapes that TMA cannot address (K or a leading stride not a multiple of 8 elements, unaligned
// pointers) run on a plain tiled CUDA-core kernel in this file; there is no host fallback.
#include <cuda.h>

#include <algorithm>
#include <atomic>
#include <mutex>
#include <vector>

#include "gemm_kernel.cuh"

namespace b200ait {

// ------------------------------------------------------------------------------------------------
// split-K second pass: sums the fp32 partials of every split and applies the fused epilogue.
// One thread per (batch, row, 32-column chunk); a warp reads 4 KB of contiguous partials per split.
template <bool BF16>
__global__ void __launch_bounds__(256) gemm_splitk_reduce_kernel(const GemmParams p) {
  const int chunks = (p.N + 31) / 32;
  const long long total = static_cast<long long>(p.batch) * p.M * chunks;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int chunk = static_cast<int>(idx % chunks);
  const long long br = idx / chunks;
  const int row = static_cast<int>(br % p.M), b = static_cast<int>(br / p.M);
  const int col0 = chunk * 32;
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = 0.f;
  const bool full = p.vec_ok && col0 + 32 <= p.N;
  const long long split_stride = static_cast<long long>(p.batch) * p.M * p.N;
  int s0 = 0;
  if (full) {
    // two splits' 128 bytes per thread are requested before either is added: few threads run here when M is
    // small, so the pass is bound by how many loads each of them keeps in flight
    const float* base = p.partial + (static_cast<long long>(b) * p.M + row) * p.N + col0;
    for (; s0 + 1 < p.splits; s0 += 2) {
      float4 f[2][8];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int q = 0; q < 8; ++q) f[h][q] = __ldcs(reinterpret_cast<const float4*>(base + (s0 + h) * split_stride + q * 4));
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int q = 0; q < 8; ++q)
          v[q * 4] += f[h][q].x, v[q * 4 + 1] += f[h][q].y, v[q * 4 + 2] += f[h][q].z, v[q * 4 + 3] += f[h][q].w;
    }
  }
  for (int s = s0; s < p.splits; ++s) {
    const float* src = p.partial + ((static_cast<long long>(s) * p.batch + b) * p.M + row) * p.N + col0;
    if (full) {
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float4 f = *reinterpret_cast<const float4*>(src + q * 4);
        v[q * 4] += f.x, v[q * 4 + 1] += f.y, v[q * 4 + 2] += f.z, v[q * 4 + 3] += f.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) v[j] += src[j];
    }
  }
  epilogue_chunk32<BF16>(p, v, b, row, col0, true);
}

// The fused epilogue on one fp32 accumulator: alpha, bias, activation, residual(s), activation, one rounding.
template <bool BF16>
__device__ __forceinline__ void epilogue_scalar_store(const GemmParams& p, float acc, int b, int row, int col) {
  using E = Elem16<BF16>;
  using T = typename E::T;
  const int u1 = epi_u1(p.epilogue), b1 = epi_b1(p.epilogue), b2 = epi_b2(p.epilogue), u2 = epi_u2(p.epilogue);
  float v = acc * p.alpha;
  if (p.bias) v += E::to_float(static_cast<const T*>(p.bias)[col]);
  v = apply_unary(u1, v);
  const long long di = static_cast<long long>(b) * p.d_bs + static_cast<long long>(row) * p.ldd + col;
  if (b1 != kBinaryNone) {
    const float f = E::to_float(static_cast<const T*>(p.d0)[di]);
    v = (b1 == kBinaryAdd) ? v + f : v * f;
  }
  if (b2 != kBinaryNone) {
    const float f = E::to_float(static_cast<const T*>(p.d1)[di]);
    v = (b2 == kBinaryAdd) ? v + f : v * f;
  }
  v = apply_unary(u2, v);
  static_cast<T*>(p.out)[batch_offset(p, b) + row_offset(p, row) + col_offset(p, col)] = E::from_float(v);
}

// ------------------------------------------------------------------------------------------------
// CUDA-core kernel for shapes TMA cannot address. 32x32 output tile per block, K staged in smem.
template <bool BF16>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const void* a_, const void* b_, const GemmParams p) {
  using E = Elem16<BF16>;
  using T = typename E::T;
  __shared__ float sa[32][33];
  __shared__ float sb[32][33];
  const int b = blockIdx.z;
  const T* a = static_cast<const T*>(a_) + static_cast<long long>(b) * p.a_bs * p.a_batch_mul;
  const T* w = static_cast<const T*>(b_) + static_cast<long long>(b) * p.b_bs * p.b_batch_mul;
  const long long w_n = p.b_mn ? 1 : p.ldb, w_k = p.b_mn ? p.ldb : 1;  // element strides of B along n and k
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const int row0 = blockIdx.y * 32, col0 = blockIdx.x * 32;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < p.K; k0 += 32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = ty + i * 8;
      const int k = k0 + tx;
      sa[r][tx] = (row0 + r < p.M && k < p.K) ? E::to_float(a[static_cast<long long>(row0 + r) * p.lda + k]) : 0.f;
      sb[r][tx] = (col0 + r < p.N && k < p.K) ? E::to_float(w[static_cast<long long>(col0 + r) * w_n + k * w_k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 32; ++kk) {
      const float bv = sb[tx][kk];
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] = fmaf(sa[ty + i * 8][kk], bv, acc[i]);
    }
    __syncthreads();
  }
  const int col = col0 + tx;
  if (col >= p.N) return;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = row0 + ty + i * 8;
    if (row < p.M) epilogue_scalar_store<BF16>(p, acc[i], b, row, col);
  }
}

// ------------------------------------------------------------------------------------------------
// Weight-streaming kernel for M <= 4 (a GEMV per row of X): the run time is the time to read W once, and a
// handful of rows leaves nothing for the tensor core to amortise. One block of 32 warps per SM holds X in
// shared memory and owns a contiguous share of the rows of W; each warp streams one row at a time with
// 16-byte loads that do not allocate in L1 (8 in flight per lane), multiplies on the FMA pipe in fp32 and
// reduces across the lanes. No workspace, no second pass.
constexpr int kRowDotMaxM = 4;
constexpr int kRowDotThreads = 1024;
template <bool BF16, int MR>
__global__ void __launch_bounds__(kRowDotThreads, 1) gemm_rowdot_kernel(const void* a_, const void* b_,
                                                                         const GemmParams p) {
  using T = typename Elem16<BF16>::T;
  extern __shared__ __align__(16) uint8_t rowdot_smem[];
  uint4* xs = reinterpret_cast<uint4*>(rowdot_smem);  // [MR][K / 8]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int nvec = p.K >> 3;
  for (int i = threadIdx.x; i < MR * nvec; i += blockDim.x) {
    const int m = i / nvec, v = i - m * nvec;
    xs[i] = (m < p.M) ? __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(a_) + static_cast<long long>(m) * p.lda) + v)
                      : make_uint4(0, 0, 0, 0);
  }
  __syncthreads();
  // rows [n_begin, n_end) of W belong to this block
  const int per = (p.N + gridDim.x - 1) / gridDim.x;
  const int n_begin = blockIdx.x * per, n_end = min(p.N, n_begin + per);
  constexpr int kUnroll = 8;
  for (int n = n_begin + warp; n < n_end; n += nwarps) {
    const uint4* w = reinterpret_cast<const uint4*>(static_cast<const T*>(b_) + static_cast<long long>(n) * p.ldb);
    float acc[MR];
#pragma unroll
    for (int m = 0; m < MR; ++m) acc[m] = 0.f;
    for (int v0 = lane; v0 < nvec; v0 += 32 * kUnroll) {
      uint4 wq[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        wq[u] = (v0 + 32 * u < nvec) ? __ldcs(w + v0 + 32 * u) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int v = min(v0 + 32 * u, nvec - 1);  // past the end the weights above are zero
        float wf[8];
        unpack8<BF16>(wq[u], wf);
#pragma unroll
        for (int m = 0; m < MR; ++m) {
          float xf[8];
          unpack8<BF16>(xs[m * nvec + v], xf);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[m] = fmaf(xf[j], wf[j], acc[m]);
        }
      }
    }
#pragma unroll
    for (int m = 0; m < MR; ++m) {
      float t = acc[m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
      if (lane == m && m < p.M) epilogue_scalar_store<BF16>(p, t, 0, m, n);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Weight-streaming tensor-core kernel with the operands swapped: Y^T = W X^T.
// The run time of a GEMM with few rows of X is the time to read W once. Here the rows of W sit on the 128 MMA rows
// and the rows of X are the MMA's N (MX = 16 .. 256), so a CTA consumes 16 KB of weights per four MMAs, and W is
// partitioned so that every byte is read by exactly one CTA per group of MX rows of X: a cluster of R = 2, 4 or 8 CTAs
// owns a slab of 128 weight rows, rank r streams share r of K through a TMA ring, and the ranks hand each other
// their 128 x MX fp32 partial sums through the cluster's shared-memory window (a reduce-scatter: every rank finishes
// MX / R rows of X). No global workspace, no second pass (the 128 x 256 tiles + split-K + reduce kernel this
// replaces ran at 0.54 of the copy rate for M <= 32). More than 256 rows of X are taken in groups of 256.
//   warp 0: TMA producer   warp 1: MMA issuer   warps 2-5: epilogue (TMEM lane = weight row = output column)
constexpr int kSwapThreads = 192;
constexpr int kSwapMaxM = 256;
template <int MX, int R, int H>
struct SwapCfg {
  static_assert(R == 1 || R == 2 || R == 4 || R == 8, "cluster size");
  static constexpr int kPart = MX / R;              // rows of X each rank finishes ...
  static constexpr int kSub = kPart / H;            // ... in H passes of kSub rows (what bounds the exchange buffers)
  static_assert(H >= 1 && kSub * H == kPart && kSub >= 8, "a rank finishes at least 8 rows per pass");
  static constexpr int kWBytes = 128 * kBK * 2;     // 16 KB: 128 weight rows x 64 k
  static constexpr int kXBytes = MX * kBK * 2;      // MX rows of X x 64 k
  static constexpr int kStageBytes = kWBytes + kXBytes;
  static constexpr int kSlotBytes = 128 * kSub * 4;                // [kSub rows of X][128 weight rows] fp32
  static constexpr int kPartialBytes = (R - 1) * kSlotBytes;       // one slot per peer: its sums for this rank's rows
  static constexpr int kTileBytes = kSlotBytes;                    // the finished tile, [kSub][128]
  static constexpr int kFit = (227 * 1024 - 256 - kPartialBytes - kTileBytes) / kStageBytes;
  static constexpr int kStages = kFit < 8 ? kFit : 8;  // 144 to 192 KB in flight
  static constexpr int kAccCols = MX < 32 ? 32 : MX;  // TMEM columns of one accumulator
  static constexpr int kTmemCols = 2 * kAccCols;
  static constexpr int kSmemBytes = kStages * kStageBytes + kPartialBytes + kTileBytes + 256;
  static_assert(kStages >= 3 && kSmemBytes <= 227 * 1024, "swapped-operand kernel: shared memory");
};

template <int N>
__device__ __forceinline__ void tmem_ld_chunk(uint32_t taddr, uint32_t (&r)[N]) {
  static_assert(N == 8 || N == 16 || N == 32, "TMEM load width");
  if constexpr (N == 8) {
    tmem_ld_32x32b_x8(taddr, r);
  } else if constexpr (N == 16) {
    tmem_ld_32x32b_x16(taddr, r);
  } else {
    tmem_ld_32x32b_x32(taddr, r);
  }
}

template <bool BF16, int MX, int R, int H>
__global__ void __launch_bounds__(kSwapThreads, 1)
gemm_swapab_kernel(const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_x,
                   const GemmParams p, const int num_slabs, const int num_groups) {
  using Cfg = SwapCfg<MX, R, H>;
  extern __shared__ __align__(1024) uint8_t smem[];
  const bool misaligned = (smem_u32(smem) & 1023u) != 0u;
  if (misaligned && threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, kDevBadSmemAlignment);
  float* partial = reinterpret_cast<float*>(smem + Cfg::kStages * Cfg::kStageBytes);  // [R - 1][kSub / 4][128][4], a slot per peer
  float* tile = reinterpret_cast<float*>(smem + Cfg::kStages * Cfg::kStageBytes + Cfg::kPartialBytes);  // [kSub][128]
  uint64_t* full_bar =
      reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes + Cfg::kPartialBytes + Cfg::kTileBytes);
  uint64_t* empty_bar = full_bar + Cfg::kStages;
  uint64_t* acc_full = empty_bar + Cfg::kStages;   // [2]
  uint64_t* acc_empty = acc_full + 2;             // [2]
  uint64_t* partial_ready = acc_empty + 2;        // every peer's partial sums are in `partial` (counts their bytes)
  uint64_t* partial_taken = partial_ready + 1;    // [2] every peer has read the sums it was sent (even / odd passes)
  uint64_t* drain_bar = partial_taken + 2;
  uint64_t* tile_summed = drain_bar + 1;          // every thread has put its sums into `tile`
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tile_summed + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  static_assert((2 * Cfg::kStages + 9) * 8 + 8 <= 256, "barrier area too small");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster_ctarank());
  const int walker = blockIdx.x / R, num_walkers = gridDim.x / R;
  // a unit of work: one slab of 128 weight rows against one group of MX rows of X (consecutive units share the slab,
  // so the clusters that run them side by side fetch its weights from HBM once)
  const int my_units = misaligned ? 0 : num_slabs * num_groups;
  // this rank's share of the k-blocks (the host sends no problem with fewer k-blocks than ranks)
  const int kb_total = (p.K + kBK - 1) / kBK;
  // split evenly, so that no rank is left without a k-block (its accumulator would never be written)
  const int kb0 = rank * kb_total / R, kb1 = (rank + 1) * kb_total / R;

  // Set-up, kept short because a small problem's whole run is a few microseconds: the lanes of warp 0 initialise one
  // barrier each while warp 1 allocates tensor memory, and the opening cluster barrier is arrived at without a release
  // (the initialisations are published by fence.mbarrier_init; a releasing arrive alone was measured at 0.5 us):
  // 0.68 us from the CTA's start to its first instruction after the set-up, 1.26 us with everything done in turn.
  // (Letting the producer thread start streaming before the set-up barriers changed nothing: the first bytes land
  // 1.7 us after the CTA's start either way, a tensor-map fetch plus a trip to HBM after the first TMA instruction.)
  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tma_w);
      tma_prefetch_desc(&tma_x);
      *abort_flag = 0;
    }
    // barriers in the order they lie in shared memory: full[kStages], empty[kStages], acc_full[2], acc_empty[2],
    // partial_ready, partial_taken[2], drain_bar, tile_summed
    constexpr int kBars = 2 * Cfg::kStages + 9;
    for (int i = lane; i < kBars; i += 32) {
      const int j = i - 2 * Cfg::kStages;  // index among the barriers after the ring's
      // every epilogue thread arrives at acc_empty and tile_summed, every peer's at partial_taken, one thread elsewhere
      const uint32_t count = (j == 2 || j == 3 || j == 8) ? 128u : (j == 5 || j == 6) ? 128u * (R > 1 ? R - 1 : 1) : 1u;
      mbar_init(&full_bar[i], count);
    }
    fence_mbar_init();
  } else if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);  // two accumulators
    tmem_relinquish();
  }
  // The TMA producer (thread 0). Every CTA reads the same rows of X: walking the k-blocks from a different starting
  // point in every cluster keeps the CTAs from asking L2 for the same lines of X at the same moment.
  const int nkb = kb1 - kb0;
  int prod_stage = 0;
  uint32_t prod_phase = 0;
  auto produce = [&](int unit, int i0, int i1) -> bool {
    const int slab = unit / num_groups, grp = unit - slab * num_groups;
    // (by slab, not by unit: every group of X rows adds its k-blocks up in the same order, so a row's result does not
    // depend on the group it falls into)
    const int rot = nkb > 0 ? static_cast<int>((static_cast<unsigned>(slab) * 11u) % static_cast<unsigned>(nkb)) : 0;
    for (int i = i0; i < i1; ++i) {
      const int kb = kb0 + (i + rot >= nkb ? i + rot - nkb : i + rot);
      if (!mbar_wait(&empty_bar[prod_stage], prod_phase ^ 1u, abort_flag, p.status, kDevWaitEmptyTimeout)) return false;
      uint8_t* sw = smem + prod_stage * Cfg::kStageBytes;
      mbar_arrive_expect_tx(&full_bar[prod_stage], Cfg::kStageBytes);
      tma_load_3d(sw, &tma_w, &full_bar[prod_stage], kb * kBK, slab * 128, 0);
      tma_load_3d(sw + Cfg::kWBytes, &tma_x, &full_bar[prod_stage], kb * kBK, grp * MX, 0);
      if (++prod_stage == Cfg::kStages) {
        prod_stage = 0;
        prod_phase ^= 1u;
      }
    }
    return true;
  };
  tc_fence_before();
  cluster_arrive_relaxed();
  __syncthreads();
  cluster_wait();  // the peers' barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool epi_arrived = false;  // this thread has arrived at the closing cluster barrier

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      for (int unit = walker; ok && unit < my_units; unit += num_walkers)
        ok = produce(unit, 0, nkb);
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(128, MX, BF16, false, false);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int unit = walker; ok && unit < my_units; unit += num_walkers) {
        ok = mbar_wait(&acc_empty[acc], acc_phase ^ 1u, abort_flag, p.status, kDevWaitAccEmptyTimeout);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * Cfg::kAccCols);
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kDevWaitFullTimeout);
          if (!ok) break;
          tc_fence_after();
          const uint32_t w_addr = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t x_addr = w_addr + Cfg::kWBytes;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t adesc = umma_smem_desc_sw128(w_addr + k * 32, 16, 1024);
            const uint64_t bdesc = umma_smem_desc_sw128(x_addr + k * 32, 16, 1024);
            umma_f16_ss(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k != 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(&acc_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (!ok) {
        umma_commit(drain_bar);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(drain_bar, 0) && globaltimer_ns() - t0 < 1000000ull) {
        }
      }
    }
  } else {
    // The MX rows of X are cut into H x R blocks of kSub rows; in pass h rank r finishes block h * R + r: it keeps
    // that block of its own sums and sends each peer q the block h * R + q (slot "sender" of q's `partial`, four rows
    // of X per 16-byte store: a warp's store covers 512 consecutive bytes). The stores are asynchronous and credit their bytes to the receiver's
    // `partial_ready`: nobody waits for a store to land except the thread that needs the data. Then the rank adds
    // what its peers sent into `tile` and writes its rows out. (H > 1 only bounds the buffers: 256 rows of X would
    // otherwise need 128 KB of them.)
    constexpr int kSub = Cfg::kSub;
    constexpr int kChunk = kSub < 32 ? kSub : 32;  // TMEM columns per load
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // weight row inside the slab == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int et = static_cast<int>(threadIdx.x) - 64;  // 0..127 over the four epilogue warps
    int acc = 0;
    uint32_t acc_phase = 0;
    // Passes done so far: `tile_summed` changes phase once per pass. The peers' "taken" signals of pass s go to
    // partial_taken[s & 1]: a rank that has no rows in a pass runs through it without waiting for anybody's sums, so
    // its signals of pass s + 1 can be complete before a slow thread here has looked at those of pass s. With one
    // barrier that thread would then wait on a parity that has come round again; with two, a barrier is reused only
    // for pass s + 2, which no peer can finish before every thread here has signalled pass s + 1.
    int seq = 0;
    uint32_t ready_phase = 0;  // `partial_ready` only changes phase in the passes in which this rank has rows
    bool ok = true;
    for (int unit = walker; ok && unit < my_units; unit += num_walkers) {
      const bool last_slab = unit + num_walkers >= my_units;
      const int slab = unit / num_groups;
      const int row_base = (unit - slab * num_groups) * MX;  // first row of X of this unit's group
      const int m_here = p.M - row_base < MX ? p.M - row_base : MX;
      // The tile goes out row by row: a thread takes 8 consecutive columns (one 16-byte store), 16 threads one
      // row of the slab. A thread keeps the same columns for every row, so it fetches their bias once, early.
      const int col0 = slab * 128 + (et & 15) * 8;
      const bool vec = p.vec_ok && col0 + 8 <= p.N;
      float bias_v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (vec && p.bias != nullptr)
        unpack8<BF16>(__ldg(reinterpret_cast<const uint4*>(static_cast<const typename Elem16<BF16>::T*>(p.bias) + col0)),
                      bias_v);
      ok = mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.status, kDevWaitAccFullTimeout);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_addr = tmem_base + lane_addr + static_cast<uint32_t>(acc * Cfg::kAccCols);
#pragma unroll 1
      for (int pass = 0; ok && pass < H; ++pass, ++seq) {
      const bool last = last_slab && pass == H - 1;
      const int my_row0 = (pass * R + rank) * kSub;
      const int my_rows = m_here - my_row0 < 0 ? 0 : (m_here - my_row0 < kSub ? m_here - my_row0 : kSub);
      const int out_row0 = row_base + my_row0;  // where this rank's block starts in the output
      // what the peers will send for this pass (a rank with no valid row of X is sent nothing and waits for nothing)
      if (R > 1 && et == 0 && my_rows > 0) mbar_arrive_expect_tx(partial_ready, (R - 1) * Cfg::kSlotBytes);
      // the peers must have read what this CTA sent for the previous pass before it is overwritten
      if (R > 1 && seq > 0)
        ok = mbar_wait_cluster(&partial_taken[(seq - 1) & 1], ((seq - 1) >> 1) & 1, abort_flag, p.status,
                               kDevWaitOtherTimeout);
#pragma unroll
      for (int q = 0; q < R; ++q) {
        const int q_row0 = (pass * R + q) * kSub;
        if (q == rank || m_here <= q_row0) continue;
        const int slot = rank < q ? rank : rank - 1;  // where this rank's sums go in rank q's buffer
        const uint32_t dst = mapa_shared(smem_u32(partial), static_cast<uint32_t>(q)) +
                             static_cast<uint32_t>((slot * kSub * 128 + row * 4) * 4);
        const uint32_t dst_bar = mapa_shared(smem_u32(partial_ready), static_cast<uint32_t>(q));
#pragma unroll
        for (int c = 0; c < kSub / kChunk; ++c) {
          uint32_t v[kChunk];
          tmem_ld_chunk<kChunk>(t_addr + static_cast<uint32_t>(q_row0 + c * kChunk), v);
          tmem_ld_wait();
          if (ok) {
#pragma unroll
            for (int j = 0; j < kChunk; j += 4)
              st_async_cluster_v4(dst + static_cast<uint32_t>((c * kChunk + j) * 128 * 4), v[j], v[j + 1], v[j + 2], v[j + 3],
                                  dst_bar);
          }
        }
      }
      // After its last send a thread touches no peer again: the cluster-wide barrier that keeps every CTA alive
      // until then is arrived at here and waited for at the very end, when it has long completed.
      if (last) {
        cluster_arrive_relaxed();
        epi_arrived = true;
      }
      if (ok && my_rows > 0) {
        if constexpr (R > 1) {
          ok = mbar_wait_cluster(partial_ready, ready_phase, abort_flag, p.status, kDevWaitOtherTimeout);
          ready_phase ^= 1u;
        }
#pragma unroll
        for (int c = 0; c < kSub / kChunk; ++c) {
          uint32_t v[kChunk];
          tmem_ld_chunk<kChunk>(t_addr + static_cast<uint32_t>(my_row0 + c * kChunk), v);
          tmem_ld_wait();
          if (ok) {
            // The K shares are added in the order of their ranks whichever rank does the adding, so a row's result
            // does not depend on which rank finishes it (= on its position in X). All loads of the chunk come before
            // its first store: the compiler may not move a load of `partial` over a store to `tile` by itself.
            float sum[kChunk];
#pragma unroll
            for (int j = 0; j < kChunk; j += 4) {
#pragma unroll
              for (int q = 0; q < R; ++q) {
                const int slot = q < rank ? q : q - 1;  // where rank q's sums sit in this rank's buffer
                const float4 term =
                    q == rank ? make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]),
                                            __uint_as_float(v[j + 3]))
                              : *reinterpret_cast<const float4*>(partial + ((slot * kSub + c * kChunk + j) * 128 + row * 4));
                sum[j] = q == 0 ? term.x : sum[j] + term.x;
                sum[j + 1] = q == 0 ? term.y : sum[j + 1] + term.y;
                sum[j + 2] = q == 0 ? term.z : sum[j + 2] + term.z;
                sum[j + 3] = q == 0 ? term.w : sum[j + 3] + term.w;
              }
            }
#pragma unroll
            for (int j = 0; j < kChunk; ++j) tile[(c * kChunk + j) * 128 + row] = sum[j];
          }
        }
      }
      if (pass == H - 1) {  // the accumulator has been read for the last time
        tc_fence_before();
        mbar_arrive(&acc_empty[acc]);
      }
      if (ok) {
        mbar_arrive(tile_summed);
        ok = mbar_wait(tile_summed, seq & 1, abort_flag, p.status, kDevWaitOtherTimeout);
      }
      if (ok) {
        const int code = p.epilogue;
        // bias + one activation [+ one added residual [+ relu]] into a row-major output: the short store loop
        const bool add_d0 = epi_b1(code) == kBinaryAdd;
        const bool simple = vec && (epi_b1(code) == kBinaryNone || add_d0) && epi_b2(code) == kBinaryNone &&
                            (epi_u2(code) == kUnaryIdentity || (add_d0 && epi_u2(code) == kUnaryRelu)) &&
                            p.store_mode == 0;
        // An activation that is more than a max runs first, in place on this thread's own elements of the tile, a row
        // per trip of a rolled loop, so that the store loops below carry no activation code but relu. (This code runs
        // once or twice per launch, from a cold instruction cache: with the activations dispatched inside the 32-wide
        // store loop, 3072 x 768 at M = 128 with tanh took 4.7 us longer than with bias alone, 8192 x 8192 9.2 us.)
        const bool pre = vec && epi_u1(code) != kUnaryIdentity && epi_u1(code) != kUnaryRelu;
        if (pre) {
          const int u1 = epi_u1(code);
#pragma unroll 1
          for (int j = et >> 4; j < my_rows; j += 8) {
            float* src = tile + j * 128 + (et & 15) * 8;
            const float4 a0 = *reinterpret_cast<const float4*>(src), a1 = *reinterpret_cast<const float4*>(src + 4);
            float w[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) w[e] = w[e] * p.alpha + bias_v[e];
            apply_unary_vec(u1, w);
            *reinterpret_cast<float4*>(src) = make_float4(w[0], w[1], w[2], w[3]);
            *reinterpret_cast<float4*>(src + 4) = make_float4(w[4], w[5], w[6], w[7]);
          }
        }
        if (simple) {
          // four rows (j, j + 8, j + 16, j + 24) per trip, all of a trip's shared-memory loads first; no per-row
          // dispatch on the epilogue code
          using T = typename Elem16<BF16>::T;
          const bool relu = epi_u1(code) == kUnaryRelu, relu_after = epi_u2(code) == kUnaryRelu;
          T* out0 = static_cast<T*>(p.out) + col0;
          const T* res0 = static_cast<const T*>(p.d0) + col0;
          for (int j = et >> 4; j < my_rows; j += 32) {
            float o[4][8];
            uint4 r0[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const int jj = j + 8 * t < my_rows ? j + 8 * t : j;
              if (add_d0) r0[t] = __ldg(reinterpret_cast<const uint4*>(res0 + static_cast<long long>(out_row0 + jj) * p.ldd));
              const float* src = tile + jj * 128 + (et & 15) * 8;
              const float4 a0 = *reinterpret_cast<const float4*>(src), a1 = *reinterpret_cast<const float4*>(src + 4);
              o[t][0] = a0.x, o[t][1] = a0.y, o[t][2] = a0.z, o[t][3] = a0.w;
              o[t][4] = a1.x, o[t][5] = a1.y, o[t][6] = a1.z, o[t][7] = a1.w;
            }
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              if (j + 8 * t < my_rows) {
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  const float y = pre ? o[t][e] : o[t][e] * p.alpha + bias_v[e];
                  o[t][e] = relu ? fmaxf(y, 0.f) : y;  // identity keeps a NaN a NaN
                }
                if (add_d0) {
                  float f[8];
                  unpack8<BF16>(r0[t], f);
#pragma unroll
                  for (int e = 0; e < 8; ++e) o[t][e] = relu_after ? fmaxf(o[t][e] + f[e], 0.f) : o[t][e] + f[e];
                }
                *reinterpret_cast<uint4*>(out0 + static_cast<long long>(out_row0 + j + 8 * t) * p.ldc) = pack8<BF16>(o[t]);
              }
            }
          }
        }
        if (!simple && vec) {
          // Any epilogue: four rows per trip again. A trip's shared-memory loads and residual loads all go out
          // before the first is used, and each activation is dispatched once per trip, over the 32 values.
          using T = typename Elem16<BF16>::T;
          const int u1 = epi_u1(code), b1 = epi_b1(code), b2 = epi_b2(code), u2 = epi_u2(code);
          T* out0 = static_cast<T*>(p.out) + col_offset(p, col0);
          for (int j = et >> 4; j < my_rows; j += 32) {
            float o[32];
            uint4 r0[4], r1[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const int jj = j + 8 * t < my_rows ? j + 8 * t : j;
              const float* src = tile + jj * 128 + (et & 15) * 8;
              const float4 a0 = *reinterpret_cast<const float4*>(src), a1 = *reinterpret_cast<const float4*>(src + 4);
              o[t * 8 + 0] = a0.x, o[t * 8 + 1] = a0.y, o[t * 8 + 2] = a0.z, o[t * 8 + 3] = a0.w;
              o[t * 8 + 4] = a1.x, o[t * 8 + 5] = a1.y, o[t * 8 + 6] = a1.z, o[t * 8 + 7] = a1.w;
              const long long d_at = static_cast<long long>(out_row0 + jj) * p.ldd + col0;
              if (b1 != kBinaryNone) r0[t] = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(p.d0) + d_at));
              if (b2 != kBinaryNone) r1[t] = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(p.d1) + d_at));
            }
            if (!pre) {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const float y = o[i] * p.alpha + bias_v[i & 7];
                o[i] = u1 == kUnaryRelu ? fmaxf(y, 0.f) : y;
              }
            }
            if (b1 != kBinaryNone) {
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                float f[8];
                unpack8<BF16>(r0[t], f);
#pragma unroll
                for (int e = 0; e < 8; ++e) o[t * 8 + e] = (b1 == kBinaryAdd) ? o[t * 8 + e] + f[e] : o[t * 8 + e] * f[e];
              }
            }
            if (b2 != kBinaryNone) {
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                float f[8];
                unpack8<BF16>(r1[t], f);
#pragma unroll
                for (int e = 0; e < 8; ++e) o[t * 8 + e] = (b2 == kBinaryAdd) ? o[t * 8 + e] + f[e] : o[t * 8 + e] * f[e];
              }
            }
            apply_unary_vec(u2, o);
#pragma unroll
            for (int t = 0; t < 4; ++t)
              if (j + 8 * t < my_rows)
                *reinterpret_cast<uint4*>(out0 + row_offset(p, out_row0 + j + 8 * t)) = pack8<BF16>(&o[t * 8]);
          }
        }
        if (!vec) {
          // columns whose 16-byte accesses are not legal (a ragged last slab, an odd row pitch): element by element
          for (int j = et >> 4; j < my_rows; j += 8) {
            const float* src = tile + j * 128 + (et & 15) * 8;
#pragma unroll 1
            for (int e = 0; e < 8; ++e)
              if (col0 + e < p.N) epilogue_scalar_store<BF16>(p, src[e], 0, out_row0 + j, col0 + e);
          }
        }
        // This thread is done reading `partial`: the peers may send the next pass's sums. (Its reads have returned -
        // their values went into `tile` - so the signal needs no release. A rank without rows signals all the same:
        // the senders count every peer.)
        if (R > 1 && !last) {
#pragma unroll
          for (int q = 0; q < R; ++q)
            if (q != rank)
              mbar_arrive_cluster_relaxed(mapa_shared(smem_u32(&partial_taken[seq & 1]), static_cast<uint32_t>(q)));
        }
      }
      }  // passes
      if (last_slab) break;
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // Every thread arrives at the cluster-wide barrier exactly once: the epilogue threads did after their last send
  // (unless a wait ran out first), everybody else does here.
  if (!epi_arrived) cluster_arrive_relaxed();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  cluster_wait();  // no CTA leaves while a peer can still write to it or signal it
}

// One walker per cluster the GPU can hold at once (clusters do not straddle GPCs, so this can be fewer than SMs / R):
// a cluster left for a second wave would start when the first is already done streaming.
template <bool BF16, int MX, int R, int H>
static int swapab_resident_clusters() {
  using Cfg = SwapCfg<MX, R, H>;
  static std::atomic<uint64_t> configured{0};
  static std::atomic<int> resident{0};
  int clusters = resident.load(std::memory_order_relaxed);
  if (clusters == 0) {
    auto* kernel = &gemm_swapab_kernel<BF16, MX, R, H>;
    opt_in_smem_once(configured, reinterpret_cast<const void*>(kernel), Cfg::kSmemBytes);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(R * (sm_count() / R)));
    cfg.blockDim = dim3(kSwapThreads);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = R;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B200AIT_CUDA_CHECK(cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg));
    B200AIT_REQUIRE(clusters > 0, "gemm: the weight-streaming kernel's cluster does not fit this GPU");
    resident.store(clusters, std::memory_order_relaxed);
  }
  return clusters;
}

template <bool BF16, int MX, int R, int H>
static void launch_swapab(const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, int num_slabs,
                          int num_groups, cudaStream_t stream) {
  using Cfg = SwapCfg<MX, R, H>;
  const int walkers = swapab_resident_clusters<BF16, MX, R, H>();  // also opts the kernel in to its shared memory
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(R * std::min(num_slabs * num_groups, walkers)));
  cfg.blockDim = dim3(kSwapThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = R;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  ::b200ait::count_launch();
  B200AIT_CUDA_CHECK(cudaLaunchKernelEx(&cfg, &gemm_swapab_kernel<BF16, MX, R, H>, tw, tx, p, num_slabs, num_groups));
}

// The instantiations the planner chooses from: MX rows of X per group, K split R ways, exchange in H passes.
struct SwapKernel {
  int mx, r, stages;
  void (*launch)(bool bf16, const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, int num_slabs,
                 int num_groups, cudaStream_t stream);
  int (*resident)(bool bf16);
};
template <int MX, int R, int H>
static SwapKernel swap_kernel_entry() {
  return SwapKernel{MX, R, SwapCfg<MX, R, H>::kStages,
                    [](bool bf16, const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, int num_slabs,
                       int num_groups, cudaStream_t stream) {
                      if (bf16)
                        launch_swapab<true, MX, R, H>(tw, tx, p, num_slabs, num_groups, stream);
                      else
                        launch_swapab<false, MX, R, H>(tw, tx, p, num_slabs, num_groups, stream);
                    },
                    [](bool bf16) {
                      return bf16 ? swapab_resident_clusters<true, MX, R, H>() : swapab_resident_clusters<false, MX, R, H>();
                    }};
}
static const std::vector<SwapKernel>& swap_kernels() {
  static const std::vector<SwapKernel> table = {
      swap_kernel_entry<16, 2, 1>(),  swap_kernel_entry<32, 2, 1>(),  swap_kernel_entry<64, 2, 1>(),
      swap_kernel_entry<128, 2, 1>(), swap_kernel_entry<256, 2, 2>(), swap_kernel_entry<32, 4, 1>(),
      swap_kernel_entry<64, 4, 1>(),  swap_kernel_entry<128, 4, 1>(), swap_kernel_entry<256, 4, 2>(),
      swap_kernel_entry<64, 8, 1>(),  swap_kernel_entry<128, 8, 1>(), swap_kernel_entry<256, 8, 2>()};
  return table;
}

// Which weight-streaming kernel takes an unbatched problem (nullptr: the tile kernels do).
//
// Weights of more than 16 MB are bandwidth problems: W is read once at the HBM rate whatever the X tile, so the X
// tile is as wide as M needs (one group up to M = 256), K goes two ways, or four / eight ways while the slabs are too
// few to put most SMs to work. Bounds from sweeps against the tile kernels: M <= 128 from K = 512 on (M <= 32 from
// K = 256), M <= 256 from K = 2048 on (4096 x 4096 at M = 256: 19.9 against 24.9 us), larger M in groups of 256 while
// K >= 2048 and there are at most 32 units (beyond, the tile kernels are ahead again).
//
// Smaller problems are latency problems: a CTA's ring holds 150 - 190 KB, a trip to memory takes about 0.7 us, and a
// launch costs about 3 us before the first byte arrives, so the time is the number of ring-fulls a rank streams, plus
// the exchange (each CTA sends (R - 1) / R of its 128 x MX sums through the cluster's shared-memory window, measured
// at about 40 GB/s per CTA), plus a second wave's worth if the units outnumber the resident clusters. X is therefore
// cut into groups that are as small as it takes to fill one wave: 768 x 768 at M = 128 runs as 24 units of 32 rows,
// K four ways (5.7 us) rather than 6 units of 128 rows (7.5 us). The estimate below was fitted to a sweep of 84 shapes
// x 12 kernels (M = 32 .. 2048, N and K = 320 .. 4096) and picks within 2 % of the best kernel on average. Where the
// tile kernels win instead was read off the same sweep: more than 64 output tiles of 128 x 128 (128 with K >= 4096; 48
// with an added residual, 32 with any other epilogue beyond bias + relu), M > 1024 (2048 with K >= 4096), or K < 512
// with M > 256.
static const SwapKernel* plan_swapab(long long m, long long n, long long k, bool bf16, int epilogue_cost) {
  if (n < 128 || m < 5) return nullptr;
  const long long slabs = (n + 127) / 128, kb_total = (k + kBK - 1) / kBK;
  const auto& table = swap_kernels();
  auto find = [&](int mx, int r) -> const SwapKernel* {
    for (const SwapKernel& sk : table)
      if (sk.mx == mx && sk.r == r) return &sk;
    return nullptr;
  };
  if (n * k * 2 > (16ll << 20)) {
    const long long units = ((m + kSwapMaxM - 1) / kSwapMaxM) * slabs;
    const bool take = m <= 128   ? (k >= 512 || (k >= 256 && m <= 32))
                      : m <= 256 ? k >= 2048
                                 : (k >= 2048 && units <= 32);
    if (!take) return nullptr;
    const int r = (units <= sm_count() / 16 && kb_total >= 32) ? 8 : units <= sm_count() / 4 ? 4 : 2;
    const int mx = std::max(8 * r, m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : m <= 128 ? 128 : 256);
    return find(mx, r);
  }
  const long long tiles = ((m + 127) / 128) * slabs;
  const bool deep = kb_total >= 64;
  // (an activation other than relu costs this kernel a pre-pass over its tile, a second residual, a multiplied one or
  // a permuted store its long store loop, all of which the tile kernels compile away: 3072 x 768 + fast_gelu at
  // M = 256, 48 tiles, is 9.0 us here against 8.4)
  // (with an added residual, 1024 x 1024 at M = 1024, 64 tiles: 10.3 us here against 9.6; 768 x 768, 48 tiles: level)
  const long long max_tiles = epilogue_cost >= 2 ? 32 : epilogue_cost == 1 ? 48 : deep ? 128 : 64;
  if (k < 256 || (k < 512 && m > 256) || tiles > max_tiles || m > (deep ? 2048 : 1024)) return nullptr;
  const SwapKernel* best = nullptr;
  double best_us = 0.0;
  for (const SwapKernel& sk : table) {
    if (kb_total < sk.r) continue;                       // every rank needs a k-block
    const long long units = ((m + sk.mx - 1) / sk.mx) * slabs;
    const long long waves = (units + sk.resident(bf16) - 1) / sk.resident(bf16);
    const double kb_rank = static_cast<double>((kb_total + sk.r - 1) / sk.r);
    const double stream = std::max(0.7, kb_rank / sk.stages * 0.7) + kb_rank * 0.06;
    const double tail = 128.0 * sk.mx * 4.0 * (sk.r - 1) / sk.r / 40e3 + 0.005 * sk.mx / sk.r;
    const double us = 3.0 + stream + tail + (waves - 1) * (std::max(stream, tail) + 0.3);
    if (best == nullptr || us < best_us) best = &sk, best_us = us;
  }
  return best;
}

// ------------------------------------------------------------------------------------------------
// host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  if (!fn) throw Error("cuTensorMapEncodeTiled is not available from the CUDA driver");
  return fn;
}

// 3-D map over a [batch, rows, cols] 16-bit tensor, cols contiguous; box = [1, box_rows, 64], 128-byte swizzle
CUtensorMap make_tile_map(const void* base, bool bf16, long long cols, long long rows, long long batch,
                          long long row_stride_elems, long long batch_stride_elems, int box_rows) {
  CUtensorMap m;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(batch)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(row_stride_elems) * 2,
                           static_cast<cuuint64_t>(batch > 1 ? batch_stride_elems : rows * row_stride_elems) * 2};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = get_encode_fn()(&m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                               const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw Error("cuTensorMapEncodeTiled failed with CUresult " + std::to_string(static_cast<int>(r)));
  return m;
}

// 5-D map over the GEMM output for the shared-memory-staged store; box = 64 columns x 32 rows,
// 128-byte swizzle. dims / strides are innermost first; strides in elements.
CUtensorMap make_out_map(void* base, bool bf16, const long long (&dims)[5], const long long (&strides)[4]) {
  CUtensorMap m;
  cuuint64_t gd[5], gs[4];
  for (int i = 0; i < 5; ++i) gd[i] = static_cast<cuuint64_t>(dims[i]);
  for (int i = 0; i < 4; ++i) gs[i] = static_cast<cuuint64_t>(strides[i]) * 2;
  cuuint32_t box[5] = {64, 32, 1, 1, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = get_encode_fn()(&m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, base,
                               gd, gs, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw Error("cuTensorMapEncodeTiled (output) failed with CUresult " + std::to_string(static_cast<int>(r)));
  return m;
}

struct GemmArgs {
  const void *a, *b, *bias, *d0, *d1;
  void* c;
  long long batch, m, n, k;
  long long lda, ldb, ldc, ldd;
  long long a_bs, b_bs, c_bs, d_bs;
  int epilogue, dtype;
  float alpha;
  int store_mode;
  long long t1, t2, t3;
  int tile_n;  // 0 = choose
  cudaStream_t stream;
  int b_mn = 0;  // B is [K, N] with N contiguous (the reference's "rrr" layouts) instead of [N, K]
  int num_out = 1;                                // destinations: c, then extra_out[0 .. num_out - 2]
  void* extra_out[kMaxOut - 1] = {};              // same shape and strides as c (e.g. peers' copies of the result)
  void* workspace = nullptr;  // fp32 scratch for split-K partial sums (may be null: no split-K)
  long long workspace_bytes = 0;
  int split_k = 0;  // 0 = choose, 1 = off, n = at most n splits
  int* status = nullptr;  // device status word to use instead of the library's allocated one
};

constexpr int kTilePair = 512;  // tile_n value that asks for 256 x 256 tiles on CTA pairs

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Tile width by a cost model of the persistent kernel. A tcgen05 MMA of 128 rows takes ~128 cycles per 16
// of K whatever its N (the array is as wide as N = 256; narrower tiles leave columns idle), so a tile's main
// loop costs the same at every width and only the epilogue shrinks with it. Per CTA the run is
//   waves x max(main loop, epilogue) + one last epilogue,   waves = ceil(tiles / SMs),
// so narrow tiles pay only when they save a whole wave (or the problem is all epilogue).
int choose_tile_n(long long m, long long n, long long k, long long batch) {
  const long long sms = sm_count();
  const long long tm = (m + kBM - 1) / kBM;
  const long long mainloop = ((k + kBK - 1) / kBK) * 512;  // cycles
  // Result streamed to DRAM behind one or two k-blocks per tile (the attention-score shape of bmm_rcr): the run
  // is the drain of the staged stores. A 256-wide tile gives each epilogue warp two 64-column boxes to store
  // through its one staging buffer, the second waiting for the first to drain; 128-wide tiles store one box per
  // tile and overlap the drain with the next tile. Measured, 1024 x [512 x 512 x 64]: 119 us against 133 us;
  // K = 128: 131 against 159 us; from K = 256 on the wider tile wins again (89 against 105 us).
  // Measured later on wider results (us, 128- against 256-wide): K = 64 with N = 1024 .. 4096: 105 against 111 - 126;
  // K = 128 with N = 1024 / 2048: 128 against 118 / 107; K = 40 (rows of 80 bytes, padded to one k-block) with N = 2048 /
  // 4096: 141 against 125 (the wide tile fetches a quarter fewer operand rows, and TMA pays per row). So the narrow
  // tile is taken for one full k-block, and for two only on a narrow result.
  if (n >= 128 && batch * m * n * 2 > (96ll << 20) && ((k == kBK) || (k > kBK && k <= 2 * kBK && n <= 512))) return 128;
  int best = 256;
  long long best_cost = -1;
  for (int bn : {256, 128, 64}) {
    const long long tiles = tm * ((n + bn - 1) / bn) * batch;
    const long long waves = (tiles + sms - 1) / sms;
    const long long epilogue = 1500 + 8 * bn;  // measured: ~3.5 k cycles for a 128 x 256 tile, ~1.5 k of it fixed
    const long long cost = waves * std::max(mainloop, epilogue) + epilogue;
    if (best_cost < 0 || cost < best_cost) best = bn, best_cost = cost;
  }
  return best;
}

// Split-K plan: how many K-splits a problem gets and the fp32 workspace they need.
// Splitting pays when the output tiles cannot fill the SMs but K is deep enough to share out.
struct SplitPlan {
  int tile_n, splits, kb_per_split;
  long long bytes;
};
SplitPlan plan_split_k(long long batch, long long m, long long n, long long k, int tile_n, int max_splits,
                       long long workspace_bytes) {
  SplitPlan sp{tile_n ? tile_n : choose_tile_n(m, n, k, batch), 1, 0, 0};
  const long long num_kb = (k + kBK - 1) / kBK;
  sp.kb_per_split = static_cast<int>(num_kb);
  const long long sms = sm_count();
  if (max_splits == 1 || num_kb < 4) return sp;
  // One tile row (M <= 128): the run time is the time to stream the weights once. A tcgen05 MMA takes as long
  // as its M x K says, whatever N is, so a CTA consumes weight rows fastest through wide tiles: 128- and
  // 64-wide tiles cap a CTA at half and a quarter of the 256-wide rate, below its share of HBM bandwidth.
  // Take 256-wide tiles and split K to occupy the SMs, unless the fp32 partial sums that costs would add more
  // than ~5 % to the weight traffic (then 128-wide tiles, half the splits).
  if (tile_n == 0 && max_splits == 0 && batch == 1 && m <= kBM && num_kb >= 32) {
    for (int bn : {256, 128}) {
      const long long tiles_n = (n + bn - 1) / bn;
      const long long s = std::min<long long>(std::min<long long>(sms / tiles_n, num_kb / 8), 16);
      if (s < 2 || tiles_n * s * 2 < sms) continue;  // would leave most SMs idle anyway
      if (bn == 256 && s * m * 4 * 20 > k * 2) continue;  // partial sums: s * m * n * 4 bytes against n * k * 2
      if (s * m * n * 4 > workspace_bytes) continue;
      const long long per = (num_kb + s - 1) / s;
      return SplitPlan{bn, static_cast<int>((num_kb + per - 1) / per), static_cast<int>(per),
                       ((num_kb + per - 1) / per) * m * n * 4};
    }
  }
  const long long tiles = ((m + kBM - 1) / kBM) * ((n + sp.tile_n - 1) / sp.tile_n) * batch;
  long long s;
  if (max_splits > 1) {
    s = std::min<long long>(max_splits, num_kb / 2);  // the caller's choice
  } else {
    if (tiles * 2 > sms) return sp;
    // A split adds a second launch and a round trip of fp32 partial sums (4 - 5 us on a small problem): it pays only
    // when it takes that much off the main loop, i.e. from K = 2048 on and with at least 8 k-blocks left per split
    // (384 x 768 x 768: 8.3 us unsplit against 13.9 us in 6 splits; 256 x 768 x 3072: 16.7 us in 4 splits against 18.8).
    if (num_kb < 32) return sp;
    s = std::min<long long>(std::min<long long>(sms / tiles, num_kb / 8), 16);
  }
  while (s > 1 && s * batch * m * n * 4 > workspace_bytes) --s;
  if (s <= 1) return sp;
  const long long per = (num_kb + s - 1) / s;
  sp.splits = static_cast<int>((num_kb + per - 1) / per);  // no empty split
  sp.kb_per_split = static_cast<int>(per);
  sp.bytes = static_cast<long long>(sp.splits) * batch * m * n * 4;
  if (sp.splits <= 1) sp = SplitPlan{sp.tile_n, 1, static_cast<int>(num_kb), 0};
  return sp;
}

void gemm_run(const GemmArgs& g_in) {
  GemmArgs g = g_in;
  long long c_bdiv = 0, c_bs_hi = 0;
  if (g.store_mode == 3) {
    // Permute4DBMM "0213" of the batched GEMMs: [B / d1, d1, M, N] -> [B / d1, M, d1, N], d1 = t1
    // (python/aitemplate/compiler/ops/gemm_universal/bmm_rcr_permute.py, bmm_rrr_permute.py; functor
    // cutlass::layout::Tensor4DPermuteBMM0213 in the reference's CUTLASS fork). Batch b = hi * d1 + lo lands at
    // hi * M * d1 * N + lo * N and rows are d1 * N apart: a plain strided store with a two-level batch stride.
    B200AIT_REQUIRE(g.t1 > 0 && g.batch % g.t1 == 0, "bmm permute: the batch must be a multiple of shape[0]");
    B200AIT_REQUIRE(g.num_out == 1, "bmm permute: one output buffer only");
    c_bdiv = g.t1, c_bs_hi = g.m * g.t1 * g.n;
    g.ldc = g.t1 * g.n, g.c_bs = g.n, g.store_mode = 0;
    if (c_bdiv == 1) c_bdiv = 0, g.c_bs = g.m * g.n;  // d1 = 1: the identity permutation
  }
  B200AIT_REQUIRE(g.dtype == kDTypeHalf || g.dtype == kDTypeBFloat16, "gemm: dtype must be float16 or bfloat16");
  B200AIT_REQUIRE(g.batch >= 0 && g.m >= 0 && g.n >= 0 && g.k >= 0, "gemm: negative dimension");
  if (g.batch == 0 || g.m == 0 || g.n == 0 || g.k == 0) return;  // reference: zero-size problems launch nothing
  B200AIT_REQUIRE(g.a && g.b && g.c, "gemm: null operand pointer with non-zero size");
  B200AIT_REQUIRE(g.m < (1ll << 31) && g.n < (1ll << 31) && g.k < (1ll << 31), "gemm: dimension exceeds int32");
  const int b1 = epi_b1(g.epilogue), b2 = epi_b2(g.epilogue);
  B200AIT_REQUIRE(b1 == kBinaryNone || g.d0, "gemm: epilogue needs d0 but d0 is null");
  B200AIT_REQUIRE(b2 == kBinaryNone || g.d1, "gemm: epilogue needs d1 but d1 is null");
  const bool bf16 = g.dtype == kDTypeBFloat16;

  GemmParams p{};
  p.M = static_cast<int>(g.m), p.N = static_cast<int>(g.n), p.K = static_cast<int>(g.k);
  p.batch = static_cast<int>(g.batch);
  p.a_batch_mul = (g.batch > 1 && g.a_bs == 0) ? 0 : 1;
  p.b_batch_mul = (g.batch > 1 && g.b_bs == 0) ? 0 : 1;
  p.b_mn = g.b_mn;
  p.bias = g.bias, p.d0 = g.d0, p.d1 = g.d1, p.out = g.c;
  p.lda = g.lda, p.ldb = g.ldb, p.a_bs = g.a_bs, p.b_bs = g.b_bs;
  p.ldc = g.ldc, p.ldd = g.ldd, p.c_bs = g.c_bs, p.d_bs = g.d_bs;
  p.alpha = g.alpha, p.epilogue = g.epilogue;
  p.store_mode = 0;
  p.t1 = 1, p.t3 = 1, p.d = 1;
  p.c_bdiv = static_cast<int>(c_bdiv), p.c_bs_hi = c_bs_hi;
  bool vec = (g.n % 8 == 0) && aligned16(g.c) && (g.c_bs % 8 == 0);
  if (g.bias) vec = vec && aligned16(g.bias);
  B200AIT_REQUIRE(g.num_out >= 1 && g.num_out <= kMaxOut, "gemm: between 1 and 8 output buffers");
  B200AIT_REQUIRE(g.num_out == 1 || !g.b_mn, "gemm: several output buffers are not built for row-major B");
  for (int i = 1; i < g.num_out; ++i) {
    B200AIT_REQUIRE(g.extra_out[i - 1] != nullptr, "gemm: null extra output buffer");
    vec = vec && aligned16(g.extra_out[i - 1]);
  }
  if (b1 != kBinaryNone) vec = vec && aligned16(g.d0) && (g.ldd % 8 == 0) && (g.d_bs % 8 == 0);
  if (b2 != kBinaryNone) vec = vec && aligned16(g.d1) && (g.ldd % 8 == 0) && (g.d_bs % 8 == 0);
  if (g.store_mode == 0) {
    vec = vec && (g.ldc % 8 == 0);
  } else if (g.store_mode == 1) {
    // Permute5D "20314": [M/t1, t1, t2, t3, d] -> [t2, M/t1, t3, t1, d], d = N/(t2*t3)
    // (python/aitemplate/compiler/ops/gemm_universal/gemm_rcr_bias_permute.py:59-69)
    B200AIT_REQUIRE(g.t1 > 0 && g.t2 > 0 && g.t3 > 0, "gemm permute: shape entries must be positive");
    B200AIT_REQUIRE(g.m % g.t1 == 0 && g.n % (g.t2 * g.t3) == 0, "gemm permute: M %% t1 or N %% (t2*t3) != 0");
    B200AIT_REQUIRE(g.batch == 1, "gemm permute 20314 is not batched");
    const long long d = g.n / (g.t2 * g.t3);
    p.store_mode = 1;
    p.t1 = static_cast<int>(g.t1), p.t3 = static_cast<int>(g.t3), p.d = static_cast<int>(d);
    p.rs_hi = g.t3 * g.t1 * d, p.rs_lo = d;
    p.cs2 = (g.m / g.t1) * g.t3 * g.t1 * d, p.cs3 = g.t1 * d;
    vec = vec && (d % 8 == 0);
  } else if (g.store_mode == 2) {
    // Permute4D "0213": [M/t1, t1, t2, d] -> [M/t1, t2, t1, d], d = N/t2
    // (python/aitemplate/compiler/ops/gemm_universal/gemm_rcr_permute.py, bmm_rcr_permute.py layout "0213")
    B200AIT_REQUIRE(g.t1 > 0 && g.t2 > 0, "gemm permute: shape entries must be positive");
    B200AIT_REQUIRE(g.m % g.t1 == 0 && g.n % g.t2 == 0, "gemm permute: M %% t1 or N %% t2 != 0");
    const long long d = g.n / g.t2;
    p.store_mode = 1;
    p.t1 = static_cast<int>(g.t1), p.t3 = static_cast<int>(g.t2), p.d = static_cast<int>(d);
    p.rs_hi = g.t2 * g.t1 * d, p.rs_lo = d;
    p.cs2 = 0, p.cs3 = g.t1 * d;
    vec = vec && (d % 8 == 0);
  } else {
    throw Error("gemm: unknown store mode");
  }
  p.vec_ok = vec ? 1 : 0;
  p.status = g.status ? g.status : device_status_word();
  p.splits = 1;
  p.kb_per_split = static_cast<int>((g.k + kBK - 1) / kBK);
  p.partial = nullptr;

  const bool tma_ok = (g.k % 8 == 0) && (g.lda % 8 == 0) && (g.ldb % 8 == 0) && aligned16(g.a) && aligned16(g.b) &&
                      (g.a_bs % 8 == 0) && (g.b_bs % 8 == 0) && g.batch < 65536 * 32;
  B200AIT_REQUIRE(tma_ok || g.num_out == 1, "gemm: several output buffers need TMA-addressable operands");
  // M <= 4, deep K, the caller left tile width and split-K to the library: stream W once on the CUDA cores
  const long long rowdot_smem = (g.m <= 1 ? 1 : g.m <= 2 ? 2 : 4) * g.k * 2;
  if (tma_ok && g.batch == 1 && g.m <= kRowDotMaxM && !g.b_mn && g.num_out == 1 && g.tile_n == 0 && g.split_k == 0 &&
      g.k >= 1024 && g.n >= 64 && rowdot_smem <= 160 * 1024) {
    const unsigned grid = static_cast<unsigned>(std::min<long long>(sm_count(), (g.n + 3) / 4));
    const int smem = static_cast<int>(rowdot_smem);
#define B200AIT_ROWDOT(BF, MR)                                                                                 \
  do {                                                                                                         \
    static std::atomic<uint64_t> configured{0};                                                                \
    opt_in_smem_once(configured, reinterpret_cast<const void*>(&gemm_rowdot_kernel<BF, MR>), 160 * 1024);      \
    ::b200ait::count_launch(), gemm_rowdot_kernel<BF, MR><<<grid, kRowDotThreads, smem, g.stream>>>(g.a, g.b, p);                         \
  } while (0)
    if (bf16) {
      if (g.m <= 1) B200AIT_ROWDOT(true, 1); else if (g.m <= 2) B200AIT_ROWDOT(true, 2); else B200AIT_ROWDOT(true, 4);
    } else {
      if (g.m <= 1) B200AIT_ROWDOT(false, 1); else if (g.m <= 2) B200AIT_ROWDOT(false, 2); else B200AIT_ROWDOT(false, 4);
    }
#undef B200AIT_ROWDOT
    B200AIT_CUDA_CHECK(cudaGetLastError());
    return;
  }
  // few rows of X, or few output tiles: the weight-streaming kernel where its planner takes the problem
  if (tma_ok && g.batch == 1 && !g.b_mn && g.num_out == 1 && g.tile_n == 0 && g.split_k == 0) {
    const int code = p.epilogue;
    // what the weight-streaming kernel's short store loop does without an activation pre-pass: bias [+ relu]
    // [+ one added residual [+ relu]] into a row-major output
    const bool added = epi_b1(code) == kBinaryAdd;
    const bool plain = (epi_b1(code) == kBinaryNone || added) && epi_b2(code) == kBinaryNone &&
                       (epi_u2(code) == kUnaryIdentity || (added && epi_u2(code) == kUnaryRelu)) &&
                       (epi_u1(code) == kUnaryIdentity || epi_u1(code) == kUnaryRelu) && p.store_mode == 0;
    if (const SwapKernel* sk = plan_swapab(g.m, g.n, g.k, bf16, !plain ? 2 : added ? 1 : 0)) {
      const int num_groups = static_cast<int>((g.m + sk->mx - 1) / sk->mx);
      const int num_slabs = static_cast<int>((g.n + 127) / 128);
      CUtensorMap tw = make_tile_map(g.b, bf16, g.k, g.n, 1, g.ldb, 0, 128);
      CUtensorMap tx = make_tile_map(g.a, bf16, g.k, g.m, 1, g.lda, 0, sk->mx);
      sk->launch(bf16, tw, tx, p, num_slabs, num_groups, g.stream);
      return;
    }
  }
  if (!tma_ok) {
    dim3 grid(static_cast<unsigned>((g.n + 31) / 32), static_cast<unsigned>((g.m + 31) / 32),
              static_cast<unsigned>(g.batch));
    B200AIT_REQUIRE(grid.y < 65536 && grid.z < 65536, "gemm: unaligned problem too large for the CUDA-core kernel");
    if (bf16)
      ::b200ait::count_launch(), gemm_simt_kernel<true><<<grid, 256, 0, g.stream>>>(g.a, g.b, p);
    else
      ::b200ait::count_launch(), gemm_simt_kernel<false><<<grid, 256, 0, g.stream>>>(g.a, g.b, p);
    B200AIT_CUDA_CHECK(cudaGetLastError());
    return;
  }

  B200AIT_REQUIRE(g.tile_n == 0 || g.tile_n == 64 || g.tile_n == 128 || g.tile_n == 256 || g.tile_n == kTilePair,
                  "gemm: tile_n must be 64, 128, 256 or 512 (256 x 256 tiles on CTA pairs)");
  const bool ws_ok = g.workspace != nullptr && aligned16(g.workspace);
  const bool force_pair = g.tile_n == kTilePair;
  SplitPlan sp = force_pair ? SplitPlan{256, 1, static_cast<int>((g.k + kBK - 1) / kBK), 0}
                            : plan_split_k(g.batch, g.m, g.n, g.k, g.tile_n, g.num_out > 1 ? 1 : g.split_k,
                                           ws_ok ? g.workspace_bytes : 0);
  if (g.num_out > 1 && sp.tile_n == 64 && g.tile_n == 0) sp.tile_n = 128;  // several destinations need the staged store
  const int bn = sp.tile_n;
  // CTA pairs (256 x 256 tiles, cta_group::2): a third less operand traffic per flop into each SM. Chosen
  // when the 256-wide tile was picked automatically, the 256-row tiles still fill every pair once, and K is
  // deep enough for the main loop (not the per-tile epilogue and pair hand-shake) to set the pace.
  const long long pair_tiles = ((g.m + 2 * kBM - 1) / (2 * kBM)) * ((g.n + 255) / 256) * g.batch;
  B200AIT_REQUIRE(!(force_pair && p.c_bdiv != 0), "bmm permute: the CTA-pair tiles do not take the permuted store");
  // With one residual operand the pair kernel pays from K = 256 on: it fetches the residual by TMA into its
  // staging boxes where the single-CTA kernels load it per thread (8192 x 1280 x 320 "mul": 18.7 against 21.6 us).
  const bool staged_residual = b1 != kBinaryNone && b2 == kBinaryNone;
  // From K = 2048 on the pairs win even when only 3 in 5 of them get a tile: the operand traffic they save counts for
  // more than the idle SMs (768 x 4096 x 4096: 28.2 against 32.0 us with 48 tiles for 74 pairs).
  // (and with a residual, which only the pairs fetch by TMA: 3072 x 1280 x 320 + add: 11.3 against 12.3 us)
  const long long pair_tiles_min = (g.k >= 2048 || staged_residual) ? sm_count() * 3 / 10 : sm_count() / 2;
  const bool pair = force_pair || (g.tile_n == 0 && bn == 256 && sp.splits == 1 &&
                                   g.k >= (staged_residual ? 256 : 512) && pair_tiles >= pair_tiles_min &&
                                   p.c_bdiv == 0);
  p.splits = sp.splits;
  p.kb_per_split = sp.kb_per_split;
  p.partial = static_cast<float*>(g.workspace);
  const long long a_batch = p.a_batch_mul ? g.batch : 1, b_batch = p.b_batch_mul ? g.batch : 1;
  CUtensorMap ta = make_tile_map(g.a, bf16, g.k, g.m, a_batch, g.lda, g.a_bs, kBM);
  CUtensorMap tb = g.b_mn ? make_tile_map(g.b, bf16, g.n, g.k, b_batch, g.ldb, g.b_bs, kBK)  // 64 x 64 boxes
                          : make_tile_map(g.b, bf16, g.k, g.n, b_batch, g.ldb, g.b_bs, pair ? bn / 2 : bn);
  // Staged TMA store: row-major output with 16-byte aligned rows, or a permuted output whose 64-column
  // groups and 32-row groups each stay inside one contiguous run of the destination.
  OutMaps tout;
  for (int i = 0; i < kMaxOut; ++i) tout.m[i] = ta;  // placeholders: only the first num_out are ever read
  p.tma_store = 0;
  p.num_out = g.num_out;
  if (bn >= 128 && p.splits == 1 && p.vec_ok) {
    for (int i = 0; i < g.num_out; ++i) {
      void* dst = i == 0 ? g.c : g.extra_out[i - 1];
      if (p.store_mode == 0) {
        const long long bs = g.batch > 1 ? g.c_bs : g.m * g.ldc;
        if (p.c_bdiv != 0) {  // batch coordinate split into (lo, hi)
          const long long dims[5] = {g.n, g.m, p.c_bdiv, g.batch / p.c_bdiv, 1};
          const long long strides[4] = {g.ldc, g.c_bs, p.c_bs_hi, p.c_bs_hi};
          tout.m[i] = make_out_map(dst, bf16, dims, strides);
        } else {
          const long long dims[5] = {g.n, g.m, g.batch, 1, 1};
          const long long strides[4] = {g.ldc, bs, bs, bs};
          tout.m[i] = make_out_map(dst, bf16, dims, strides);
        }
        p.tma_store = 1;
      } else if (p.d % 64 == 0 && p.t1 % 32 == 0 && g.batch == 1) {
        // destination [c2][row / t1][c3][row % t1][d]: dims innermost first (d, t1, t3, M / t1, c2 extent)
        const long long c2_extent = g.n / (static_cast<long long>(p.d) * p.t3);
        const long long dims[5] = {p.d, p.t1, p.t3, g.m / p.t1, c2_extent};
        const long long strides[4] = {p.rs_lo, p.cs3, p.rs_hi, p.cs2 > 0 ? p.cs2 : p.rs_hi * (g.m / p.t1)};
        tout.m[i] = make_out_map(dst, bf16, dims, strides);
        p.tma_store = 1;
      }
    }
  }
  B200AIT_REQUIRE(g.num_out == 1 || p.tma_store,
                  "gemm: several output buffers need the staged TMA store (tile_n >= 128, no split-K, N and the "
                  "output strides multiples of 8, 16-byte aligned pointers)");
  p.tiles_m = pair ? (p.M + 2 * kBM - 1) / (2 * kBM) : (p.M + kBM - 1) / kBM;
  p.tiles_n = (p.N + bn - 1) / bn;
  p.num_tiles = p.tiles_m * p.tiles_n * p.batch;
  p.num_units = p.num_tiles * p.splits;
  const int grid = pair ? 2 * std::min(p.num_units, sm_count() / 2) : std::min(p.num_units, sm_count());
  CUtensorMap td0 = ta;
  p.tma_d0 = 0;
  if (pair && p.tma_store && b1 != kBinaryNone && b2 == kBinaryNone) {
    // residual boxes of 32 rows x 64 columns, fetched by the epilogue warps into their staging buffers
    td0 = make_tile_map(g.d0, bf16, g.n, g.m, g.batch, g.ldd, g.d_bs, 32);
    p.tma_d0 = 1;
  }
  if (pair)
    launch_tc_pair256(bf16, ta, tb, tout, td0, p, grid, g.stream);
  else if (bn == 256)
    launch_tc_width<256>(bf16, ta, tb, tout, p, grid, g.stream);
  else if (bn == 128)
    launch_tc_width<128>(bf16, ta, tb, tout, p, grid, g.stream);
  else
    launch_tc_width<64>(bf16, ta, tb, tout, p, grid, g.stream);
  if (p.splits > 1) {
    const long long total = static_cast<long long>(p.batch) * p.M * ((p.N + 31) / 32);
    const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
    if (bf16)
      ::b200ait::count_launch(), gemm_splitk_reduce_kernel<true><<<blocks, 256, 0, g.stream>>>(p);
    else
      ::b200ait::count_launch(), gemm_splitk_reduce_kernel<false><<<blocks, 256, 0, g.stream>>>(p);
    B200AIT_CUDA_CHECK(cudaGetLastError());
  }
}

}  // namespace b200ait

using namespace b200ait;

// Generic entry point: every gemm_rcr* / bmm_rcr* op of the path maps onto it.
// `workspace` (may be null) is fp32 scratch for split-K partial sums; split_k: 0 = library chooses,
// 1 = never split, n > 1 = at most n splits. Without a workspace the GEMM never splits.
B200AIT_EXPORT int b200ait_gemm_rcr(const void* a, const void* b, const void* bias, const void* d0, const void* d1,
                                    void* c, int64_t batch, int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb,
                                    int64_t ldc, int64_t ldd, int64_t a_batch_stride, int64_t b_batch_stride,
                                    int64_t c_batch_stride, int64_t d_batch_stride, int epilogue, int dtype,
                                    float alpha, int store_mode, int64_t t1, int64_t t2, int64_t t3, int tile_n,
                                    void* workspace, int64_t workspace_bytes, int split_k, cudaStream_t stream) {
  return guarded("b200ait_gemm_rcr", [&] {
    GemmArgs g{a,   b,   bias,           d0,             d1,             c,
               batch, m,   n,              k,              lda,            ldb,
               ldc, ldd, a_batch_stride, b_batch_stride, c_batch_stride, d_batch_stride,
               epilogue, dtype, alpha, store_mode, t1, t2, t3, tile_n, stream};
    g.workspace = workspace;
    g.workspace_bytes = workspace_bytes;
    g.split_k = split_k;
    gemm_run(g);
  });
}

// b200ait_gemm_rcr with B stored [batch, k, n] (n contiguous, row stride ldb): the reference's gemm_rrr / bmm_rrr
// layouts (python/aitemplate/compiler/ops/gemm_universal/gemm_rrr.py, bmm_xxx.py "rrr"). Same kernel, the B tile
// reaches the tensor core as an MN-major operand.
B200AIT_EXPORT int b200ait_gemm_rrr(const void* a, const void* b, const void* bias, const void* d0, const void* d1,
                                    void* c, int64_t batch, int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb,
                                    int64_t ldc, int64_t ldd, int64_t a_batch_stride, int64_t b_batch_stride,
                                    int64_t c_batch_stride, int64_t d_batch_stride, int epilogue, int dtype,
                                    float alpha, int tile_n, void* workspace, int64_t workspace_bytes, int split_k,
                                    cudaStream_t stream) {
  return guarded("b200ait_gemm_rrr", [&] {
    GemmArgs g{a,   b,   bias,           d0,             d1,             c,
               batch, m,   n,              k,              lda,            ldb,
               ldc, ldd, a_batch_stride, b_batch_stride, c_batch_stride, d_batch_stride,
               epilogue, dtype, alpha, 0, 1, 1, 1, tile_n, stream};
    g.b_mn = 1;
    g.workspace = workspace;
    g.workspace_bytes = workspace_bytes;
    g.split_k = split_k;
    gemm_run(g);
  });
}

// bmm_rcr_permute / bmm_rrr_permute (python/aitemplate/compiler/ops/gemm_universal/bmm_rcr_permute.py:28-116,
// bmm_rrr_permute.py; generated signature python/aitemplate/backend/cuda/gemm_universal/bmm_common.py:56-81 with the
// Permute4DBMM_0213 epilogue of bmm_permute_common.py): c[b] = alpha * a[b] @ op(b[b]) for a [batch, m, k] and
// b [batch, n, k] (b_row_major = 0) or [batch, k, n] (b_row_major = 1), stored as
// [batch / d1, d1, m, n].permute(0, 2, 1, 3), i.e. c has the shape [batch / d1, m, d1, n]. A batch stride of 0
// broadcasts that operand.
B200AIT_EXPORT int b200ait_bmm_permute0213(const void* a, const void* b, void* c, int64_t batch, int64_t m, int64_t n,
                                           int64_t k, int64_t a_batch_stride, int64_t b_batch_stride, int64_t d1,
                                           int b_row_major, int dtype, float alpha, int tile_n, cudaStream_t stream) {
  return guarded("b200ait_bmm_permute0213", [&] {
    B200AIT_REQUIRE(d1 > 0, "bmm permute: shape[0] must be positive");
    GemmArgs g{a, b, nullptr, nullptr, nullptr, c, batch, m, n, k, k, b_row_major ? n : k, n, n,
               a_batch_stride, b_batch_stride, m * n, m * n, 0, dtype, alpha, 3, d1, 1, 1, tile_n, stream};
    g.b_mn = b_row_major ? 1 : 0;
    g.split_k = 1;
    gemm_run(g);
  });
}

// The same GEMM with its result written to num_out buffers of identical shape and strides (1 <= num_out <= 8)
// by the epilogue's TMA stores: outs[0] is usually this GPU's buffer and the others are peer-mapped pointers
// to other GPUs' buffers, so that a rank that computes one column block of Y = X W^T places it in every
// rank's full Y while the next tile is being computed (no separate gather pass). Never splits K; needs the
// staged store (N and ldc multiples of 8, 16-byte aligned pointers).
B200AIT_EXPORT int b200ait_gemm_rcr_multi_out(const void* a, const void* b, const void* bias, const void* d0,
                                              void* const* outs, int num_out, int64_t m, int64_t n, int64_t k,
                                              int64_t lda, int64_t ldb, int64_t ldc, int64_t ldd, int epilogue,
                                              int dtype, float alpha, int tile_n, cudaStream_t stream) {
  return guarded("b200ait_gemm_rcr_multi_out", [&] {
    B200AIT_REQUIRE(outs != nullptr && num_out >= 1 && num_out <= kMaxOut, "outs: 1 to 8 output pointers");
    GemmArgs g{a, b, bias, d0, nullptr, outs[0], 1, m, n, k, lda, ldb, ldc, ldd, 0, 0, 0, 0,
               epilogue, dtype, alpha, 0, 1, 1, 1, tile_n, stream};
    g.num_out = num_out;
    for (int i = 1; i < num_out; ++i) g.extra_out[i - 1] = outs[i];
    g.split_k = 1;
    gemm_run(g);
  });
}

// Bytes of split-K workspace b200ait_gemm_rcr would use for this problem if given enough.
B200AIT_EXPORT int b200ait_gemm_rcr_workspace_bytes(int64_t batch, int64_t m, int64_t n, int64_t k, int tile_n,
                                                    int split_k, int64_t* bytes_out) {
  return guarded("b200ait_gemm_rcr_workspace_bytes", [&] {
    B200AIT_REQUIRE(bytes_out, "bytes_out is null");
    *bytes_out = 0;
    if (batch <= 0 || m <= 0 || n <= 0 || k <= 0) return;
    *bytes_out = tile_n == kTilePair ? 0 : plan_split_k(batch, m, n, k, tile_n, split_k, (1ll << 62)).bytes;
  });
}

// Entry points with the argument order of the reference's generated per-op functions
// (python/aitemplate/backend/cuda/gemm_universal/common_bias.py:77-97: a, b, bias, c, workspace, split_k,
//  pointers to the dims of a [M,K], b [N,K] and c [M,N], stream). *c_dim0/*c_dim1 are written.
static int gemm_rcr_bias_named(const char* name, int epilogue, void* a, void* b, void* bias, void* d0, void* d1,
                               void* c, int64_t* a_dim0, int64_t* a_dim1, int64_t* b_dim0, int64_t* b_dim1,
                               int64_t* c_dim0, int64_t* c_dim1, bool need_bias, cudaStream_t stream) {
  return guarded(name, [&] {
    B200AIT_REQUIRE(a_dim0 && a_dim1 && b_dim0 && b_dim1, "null dimension pointer");
    const int64_t m = *a_dim0, k = *a_dim1, n = *b_dim0;
    B200AIT_REQUIRE(*b_dim1 == k, "a and b disagree on K");
    if (c_dim0) *c_dim0 = m;
    if (c_dim1) *c_dim1 = n;
    if (m != 0 && n != 0 && k != 0) B200AIT_REQUIRE(!need_bias || bias, "bias_ptr is null!");
    GemmArgs g{a, b, bias, d0, d1, c, 1, m, n, k, k, k, n, n, 0, 0, 0, 0, epilogue, kDTypeHalf, 1.f, 0, 1, 1, 1, 0,
               stream};
    gemm_run(g);
  });
}

#define B200AIT_DEFINE_GEMM_BIAS(NAME, U1)                                                                         \
  B200AIT_EXPORT int b200ait_##NAME(void* a, void* b, void* bias, void* c, uint8_t* workspace, int split_k,        \
                                    int64_t* a_dim0, int64_t* a_dim1, int64_t* b_dim0, int64_t* b_dim1,            \
                                    int64_t* c_dim0, int64_t* c_dim1, cudaStream_t stream) {                       \
    (void)workspace;                                                                                               \
    (void)split_k;                                                                                                 \
    return gemm_rcr_bias_named("b200ait_" #NAME, make_epilogue(U1, kBinaryNone, kBinaryNone, kUnaryIdentity), a, b, \
                               bias, nullptr, nullptr, c, a_dim0, a_dim1, b_dim0, b_dim1, c_dim0, c_dim1, true,    \
                               stream);                                                                            \
  }
B200AIT_DEFINE_GEMM_BIAS(gemm_rcr_bias, kUnaryIdentity)
B200AIT_DEFINE_GEMM_BIAS(gemm_rcr_bias_relu, kUnaryRelu)
B200AIT_DEFINE_GEMM_BIAS(gemm_rcr_bias_gelu, kUnaryGelu)
B200AIT_DEFINE_GEMM_BIAS(gemm_rcr_bias_fast_gelu, kUnaryFastGelu)
B200AIT_DEFINE_GEMM_BIAS(gemm_rcr_bias_sigmoid, kUnarySigmoid)
B200AIT_DEFINE_GEMM_BIAS(gemm_rcr_bias_tanh, kUnaryTanh)
B200AIT_DEFINE_GEMM_BIAS(gemm_rcr_bias_swish, kUnarySwish)
B200AIT_DEFINE_GEMM_BIAS(gemm_rcr_bias_hardswish, kUnaryHardswish)
#undef B200AIT_DEFINE_GEMM_BIAS

// python/aitemplate/backend/cuda/gemm_universal/gemm_rcr.py (common.py:172-198): no bias operand
B200AIT_EXPORT int b200ait_gemm_rcr_plain(void* a, void* b, void* c, uint8_t* workspace, int split_k, int64_t* a_dim0,
                                          int64_t* a_dim1, int64_t* b_dim0, int64_t* b_dim1, int64_t* c_dim0,
                                          int64_t* c_dim1, cudaStream_t stream) {
  (void)workspace;
  (void)split_k;
  return gemm_rcr_bias_named("b200ait_gemm_rcr_plain", 0, a, b, nullptr, nullptr, nullptr, c, a_dim0, a_dim1, b_dim0,
                             b_dim1, c_dim0, c_dim1, false, stream);
}

// python/aitemplate/backend/cuda/gemm_universal/common_bias_broadcast.py:276-305: d0 (and d1) precede c
#define B200AIT_DEFINE_GEMM_BIAS_D0(NAME, U1, B1, U2)                                                                \
  B200AIT_EXPORT int b200ait_##NAME(void* a, void* b, void* bias, void* d0, void* c, uint8_t* workspace,             \
                                    int split_k, int64_t* a_dim0, int64_t* a_dim1, int64_t* b_dim0, int64_t* b_dim1, \
                                    int64_t* c_dim0, int64_t* c_dim1, cudaStream_t stream) {                         \
    (void)workspace;                                                                                                 \
    (void)split_k;                                                                                                   \
    return gemm_rcr_bias_named("b200ait_" #NAME, make_epilogue(U1, B1, kBinaryNone, U2), a, b, bias, d0, nullptr, c, \
                               a_dim0, a_dim1, b_dim0, b_dim1, c_dim0, c_dim1, true, stream);                        \
  }
#define B200AIT_DEFINE_GEMM_BIAS_D0_D1(NAME, U1, B1, B2, U2)                                                         \
  B200AIT_EXPORT int b200ait_##NAME(void* a, void* b, void* bias, void* d0, void* d1, void* c, uint8_t* workspace,   \
                                    int split_k, int64_t* a_dim0, int64_t* a_dim1, int64_t* b_dim0, int64_t* b_dim1, \
                                    int64_t* c_dim0, int64_t* c_dim1, cudaStream_t stream) {                         \
    (void)workspace;                                                                                                 \
    (void)split_k;                                                                                                   \
    return gemm_rcr_bias_named("b200ait_" #NAME, make_epilogue(U1, B1, B2, U2), a, b, bias, d0, d1, c, a_dim0,       \
                               a_dim1, b_dim0, b_dim1, c_dim0, c_dim1, true, stream);                                \
  }
B200AIT_DEFINE_GEMM_BIAS_D0(gemm_rcr_bias_add, kUnaryIdentity, kBinaryAdd, kUnaryIdentity)
B200AIT_DEFINE_GEMM_BIAS_D0(gemm_rcr_bias_add_relu, kUnaryIdentity, kBinaryAdd, kUnaryRelu)
B200AIT_DEFINE_GEMM_BIAS_D0(gemm_rcr_bias_mul, kUnaryIdentity, kBinaryMul, kUnaryIdentity)
B200AIT_DEFINE_GEMM_BIAS_D0(gemm_rcr_bias_mul_tanh, kUnaryIdentity, kBinaryMul, kUnaryTanh)
B200AIT_DEFINE_GEMM_BIAS_D0(gemm_rcr_bias_sigmoid_mul, kUnarySigmoid, kBinaryMul, kUnaryIdentity)
B200AIT_DEFINE_GEMM_BIAS_D0(gemm_rcr_bias_sigmoid_mul_tanh, kUnarySigmoid, kBinaryMul, kUnaryTanh)
B200AIT_DEFINE_GEMM_BIAS_D0_D1(gemm_rcr_bias_add_add, kUnaryIdentity, kBinaryAdd, kBinaryAdd, kUnaryIdentity)
B200AIT_DEFINE_GEMM_BIAS_D0_D1(gemm_rcr_bias_add_add_relu, kUnaryIdentity, kBinaryAdd, kBinaryAdd, kUnaryRelu)
B200AIT_DEFINE_GEMM_BIAS_D0_D1(gemm_rcr_bias_mul_add, kUnaryIdentity, kBinaryMul, kBinaryAdd, kUnaryIdentity)
#undef B200AIT_DEFINE_GEMM_BIAS_D0
#undef B200AIT_DEFINE_GEMM_BIAS_D0_D1

// python/aitemplate/backend/cuda/gemm_universal/gemm_rcr_bias_permute.py:55-95 (layout "20314", shape (t1,t2,t3))
B200AIT_EXPORT int b200ait_gemm_rcr_bias_permute(void* a, void* b, void* bias, void* c, uint8_t* workspace,
                                                 int split_k, int64_t* a_dim0, int64_t* a_dim1, int64_t* b_dim0,
                                                 int64_t* b_dim1, int64_t* c_dim0, int64_t* c_dim1, int64_t t1,
                                                 int64_t t2, int64_t t3, cudaStream_t stream) {
  (void)workspace;
  (void)split_k;
  return guarded("b200ait_gemm_rcr_bias_permute", [&] {
    B200AIT_REQUIRE(a_dim0 && a_dim1 && b_dim0 && b_dim1, "null dimension pointer");
    const int64_t m = *a_dim0, k = *a_dim1, n = *b_dim0;
    B200AIT_REQUIRE(*b_dim1 == k, "a and b disagree on K");
    if (c_dim0) *c_dim0 = m;
    if (c_dim1) *c_dim1 = n;
    if (m != 0 && n != 0 && k != 0) B200AIT_REQUIRE(bias, "bias_ptr is null!");
    GemmArgs g{a, b, bias, nullptr, nullptr, c, 1, m, n, k, k, k, n, n, 0, 0, 0, 0, 0, kDTypeHalf, 1.f, 1, t1, t2, t3,
               0, stream};
    gemm_run(g);
  });
}

// python/aitemplate/backend/cuda/gemm_universal/bmm_common.py:56-81: a [B,M,K], b [B,N,K], c [B,M,N]
B200AIT_EXPORT int b200ait_bmm_rcr(void* a, void* b, void* c, uint8_t* workspace, int64_t* a_dim0, int64_t* a_dim1,
                                   int64_t* a_dim2, int64_t* b_dim0, int64_t* b_dim1, int64_t* b_dim2,
                                   int64_t* c_dim0, int64_t* c_dim1, int64_t* c_dim2, cudaStream_t stream) {
  (void)workspace;
  return guarded("b200ait_bmm_rcr", [&] {
    B200AIT_REQUIRE(a_dim0 && a_dim1 && a_dim2 && b_dim0 && b_dim1 && b_dim2, "null dimension pointer");
    const int64_t ba = *a_dim0, m = *a_dim1, k = *a_dim2, bb = *b_dim0, n = *b_dim1;
    B200AIT_REQUIRE(*b_dim2 == k, "a and b disagree on K");
    B200AIT_REQUIRE(ba == bb || ba == 1 || bb == 1, "batch sizes are not broadcastable");
    const int64_t batch = ba > bb ? ba : bb;
    if (c_dim0) *c_dim0 = batch;
    if (c_dim1) *c_dim1 = m;
    if (c_dim2) *c_dim2 = n;
    GemmArgs g{a, b, nullptr, nullptr, nullptr, c, batch, m, n, k, k, k, n, n,
               (ba == 1 && batch > 1) ? 0 : m * k, (bb == 1 && batch > 1) ? 0 : n * k, m * n, m * n,
               0, kDTypeHalf, 1.f, 0, 1, 1, 1, 0, stream};
    gemm_run(g);
  });
}


// ------------------------------------------------------------------------------------------------
// Split-K GEMM for callers that must not allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: inside a serving process whose
// memory pool was sized and handed out at start-up, under a framework allocator that owns the whole
// device, or on a path that has to stay free of driver allocation calls because those serialise
// with other work. b200ait_gemm_rcr needs two pieces of device memory beyond its operands: the
// fp32 scratch for split-K partial sums (the caller's `workspace`) and the status word the kernels
// report into (allocated by the library on first use). This entry point needs neither from the
// caller and allocates neither: both live in the file-scope array below, which is part of the
// library image, so every GPU that loads the library holds these 16 MiB + 256 bytes until the
// process exits.
namespace b200ait {
constexpr long long kStaticScratchHeader = 256;               // status word, padded to the alignment
constexpr long long kStaticScratchBytes = 16ll << 20;         // split-K partial sums: at most 16 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchHeader + kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not an address a kernel can
// use; the device address comes from cudaGetSymbolAddress, asked once per device with that device
// current.
static unsigned char* static_scratch_device_ptr() {
  constexpr int kMaxDev = 64;
  static std::mutex mu;
  static unsigned char* ptrs[kMaxDev] = {};
  int dev = 0;
  B200AIT_CUDA_CHECK(cudaGetDevice(&dev));
  B200AIT_REQUIRE(dev >= 0 && dev < kMaxDev, "device ordinal out of range");
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    void* p = nullptr;
    B200AIT_CUDA_CHECK(cudaGetSymbolAddress(&p, g_static_scratch));
    B200AIT_REQUIRE(p != nullptr, "cudaGetSymbolAddress returned a null address for the static scratch");
    ptrs[dev] = static_cast<unsigned char*>(p);
  }
  return ptrs[dev];
}
}  // namespace b200ait

// Same computation and arguments as b200ait_gemm_rcr, minus the workspace: split-K partial sums go
// to the library's static scratch. Calls no cudaMalloc / cudaFree and no allocating library routine.
//   * Limit: the partial sums of two splits must fit, 2 * batch * m * n * 4 bytes <= 16 MiB;
//     larger problems are rejected with an error (use b200ait_gemm_rcr with your own workspace).
//     Within the limit the library may use fewer splits than b200ait_gemm_rcr would.
//   * The first call on each device looks up the scratch address (cudaGetSymbolAddress) and sets
//     kernel attributes; make that first call outside any stream capture.
//   * Every call on a device shares the one scratch area and it keeps whatever the last call left
//     there. Each call rewrites all partial sums it later reads and clears the status word first,
//     but two calls that overlap on the GPU (different streams) race on it: keep calls to this entry
//     point stream-ordered per device.
//   * status_out (device pointer, may be null) receives the kernel status word after the GEMM
//     (0 = clean), stream-ordered; read it after synchronising the stream.
B200AIT_EXPORT int b200ait_gemm_rcr_static_scratch(const void* a, const void* b, const void* bias, const void* d0,
                                                   const void* d1, void* c, int64_t batch, int64_t m, int64_t n,
                                                   int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldd,
                                                   int64_t a_batch_stride, int64_t b_batch_stride,
                                                   int64_t c_batch_stride, int64_t d_batch_stride, int epilogue,
                                                   int dtype, float alpha, int store_mode, int64_t t1, int64_t t2,
                                                   int64_t t3, int tile_n, int split_k, int* status_out,
                                                   cudaStream_t stream) {
  return guarded("b200ait_gemm_rcr_static_scratch", [&] {
    B200AIT_REQUIRE(batch >= 0 && m >= 0 && n >= 0 && k >= 0, "gemm: negative dimension");
    // limit check without forming the product first: 2 * batch * m * n * 4 can leave int64 for absurd
    // dimensions and would then slip under the limit
    const long long cap_elems = kStaticScratchBytes / 8;  // fp32 partial sums of two splits
    bool fits = true;
    long long elems = 1;
    for (long long d : {(long long)batch, (long long)m, (long long)n}) {
      if (d == 0) { elems = 0; break; }
      if (elems > cap_elems / d) { fits = false; break; }
      elems *= d;
    }
    if (!fits || elems > cap_elems) {
      const std::string need = fits ? std::to_string(elems * 8) : std::string("more than 2^40");
      throw Error("problem too large for the static scratch: two splits of " + std::to_string(batch) + " x " +
                  std::to_string(m) + " x " + std::to_string(n) + " fp32 partial sums need " + need +
                  " bytes, the limit is " + std::to_string(kStaticScratchBytes) +
                  "; call b200ait_gemm_rcr with a caller-provided workspace instead");
    }
    unsigned char* scratch = static_scratch_device_ptr();
    int* status = reinterpret_cast<int*>(scratch);
    B200AIT_CUDA_CHECK(cudaMemsetAsync(status, 0, sizeof(int), stream));  // must start at zero
    GemmArgs g{a,   b,   bias,           d0,             d1,             c,
               batch, m,   n,              k,              lda,            ldb,
               ldc, ldd, a_batch_stride, b_batch_stride, c_batch_stride, d_batch_stride,
               epilogue, dtype, alpha, store_mode, t1, t2, t3, tile_n, stream};
    g.workspace = scratch + kStaticScratchHeader;
    g.workspace_bytes = kStaticScratchBytes;
    g.split_k = split_k;
    g.status = status;
    gemm_run(g);
    if (status_out)
      B200AIT_CUDA_CHECK(cudaMemcpyAsync(status_out, status, sizeof(int), cudaMemcpyDeviceToDevice, stream));
  });
}

