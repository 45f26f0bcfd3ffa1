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
//   warp 6      MMA issuer:   S = Q K^T  (tcgen05.mma, fp32 accumulator in TMEM)
//   warp 1      MMA issuer:   O += P V   (P read from TMEM, where the softmax threads put it over the S columns
//                             they have consumed; V as an MN-major B operand from shared memory); O stays in
//                             TMEM for the whole item and every key block accumulates into it
//               S and P are double-buffered: the MMAs of key block j+1 overlap the softmax of block j; O is
//               double-buffered across items
//   warps 2-5   one thread per query row: TMEM -> registers, mask (skipped for full, unmasked blocks),
//               reference max / row sum, exp2, P (16-bit pairs) -> TMEM; O is touched only when a row's
//               maximum outgrows the reference by more than 2^8 (then O and the row sum are rescaled in
//               TMEM) and once at the end of the item (O / row sum -> global memory)
// Two CTAs share an SM (head dim <= 64) so one CTA's softmax also overlaps the other's MMAs.
// Shared-memory bandwidth is what the MMAs of this kernel run into (a 128 x 64 x 16 MMA with both operands in
// shared memory reads 6 KB and issues every 48 cycles = 128 B / clk, the whole bandwidth of an SM), which is why P
// never goes through shared memory: that removed a 16 KB write and a 16 KB read per key block.
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

// Cycle probes for tuning (compiled only with -DB200AIT_ATTN_PROBE; never part of the shipped library): CTA 0 adds
// the clock64() time its softmax warp 2 / its MMA thread spend in each phase to g_attn_probe[slot].
#ifdef B200AIT_ATTN_PROBE
__device__ long long g_attn_probe[32];
#define ATTN_PROBE_DECL(cond)                \
  const bool probe_on = (cond);              \
  long long probe_acc[4] = {0, 0, 0, 0};     \
  long long probe_t = clock64();
// phase times are kept in registers (slot & 3) and flushed once by ATTN_PROBE_FLUSH(base)
#define ATTN_PROBE(slot)                                   \
  if (probe_on) {                                          \
    const long long probe_now = clock64();                 \
    probe_acc[(slot) & 3] += probe_now - probe_t;          \
    probe_t = probe_now;                                   \
  }
#define ATTN_PROBE_SKIP() \
  if (probe_on) probe_t = clock64();
#define ATTN_PROBE_FLUSH(base)                                                  \
  if (probe_on) {                                                               \
    for (int pi = 0; pi < 4; ++pi) g_attn_probe[(base) + pi] += probe_acc[pi];  \
  }
#else
#define ATTN_PROBE_DECL(cond)
#define ATTN_PROBE(slot)
#define ATTN_PROBE_SKIP()
#define ATTN_PROBE_FLUSH(base)
#endif

// defined in gemm.cu
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_fn();

struct AttnParams {
  int B, H, Sq, Skv, D, Dv;
  int q_blocks;
  int num_items;  // B * H * q_blocks work items of 128 query rows
  // item -> (query tile, head, batch) runs at every item boundary on the critical path of every role: the two
  // divisions are multiplications by constants prepared on the host (FastDiv below)
  unsigned q_blocks_mul, q_blocks_shr, h_mul, h_shr;
  float scale_log2;  // softmax scale * log2(e)
  int causal;
  void* out;  // [B, Sq, H, Dv], or [total, H, Dv] with cu_seqlens
  int* status;
  // Variable-length ("packed") mode: sequence b owns rows cu_seqlens[b] .. cu_seqlens[b+1] of q, k, v and out, and
  // Sq = Skv = the longest sequence. Null: every sequence has Sq query and Skv key rows and its own batch coordinate.
  const int* cu_seqlens;
  // Padded variable-length mode (kernel_forward.h:183-197 in the reference): with lengths_kv, batch b attends to its
  // first lengths_kv[b] keys only; with lengths_q, only its first lengths_q[b] query rows are computed and written.
  // A row that sees no key comes out as NaN, as it does there (0 / 0).
  const int* lengths_kv;
  const int* lengths_q;
  // coordinate order of each tensor map: 0 = (channel, row, head, batch), 1 = (channel, head, row, batch); the host
  // picks whichever keeps the map's strides ascending
  int q_order, k_order, v_order;
};

// One operand (q, k or v) as the kernel addresses it: element strides of a [batch, head, row, channel] view with
// unit channel stride. [B, H, S, D] contiguous is {D, S*D, H*S*D}; the q part of a packed [total, 3, H, D] tensor
// is {3*H*D, D, -} with a single batch; a [B, S, H, D] tensor read in place is {H*D, D, S*H*D}.
struct AttnOperand {
  const void* ptr;
  long long row_stride, head_stride, batch_stride;
};

constexpr int kAttnThreads = 224;  // producer, P V issuer, 4 softmax warps, S issuer
constexpr int kBlockM = 128;
constexpr int kBlockN = 64;     // keys per block
constexpr float kRescaleLog2 = 8.f;  // a row's reference maximum may lag its true maximum by this much (log2 units)
// Of every eight pairs of scores, this many get their exp2 from the FMA pipe (exp2_poly2 below) instead of the
// special-function unit, which is the busiest unit of the kernel (64 exp2 per row and key block at 4 lanes per
// clock and scheduler).
#ifndef B200AIT_ATTN_POLY_OF8
#define B200AIT_ATTN_POLY_OF8 2
#endif
constexpr int kPolyOf8 = B200AIT_ATTN_POLY_OF8;

// exp2 of two values on the FMA pipe: x = n + f with n = round(x), f in [-0.5, 0.5]; 2^f by a cubic whose relative
// error stays below 7.5e-5 (P is rounded to 11 significant bits right after, 4.9e-4); n goes into the exponent
// field. x is clamped at -126, where the result is ~1e-38 (exp2f would return a denormal or 0).
__device__ __forceinline__ void exp2_poly2(float x0, float x1, float& p0, float& p1) {
  constexpr float kMagic = 12582912.f;  // 1.5 * 2^23: adding it leaves round(x) in the low mantissa bits
  const uint64_t t = pack2(fmaxf(x0, -126.f), fmaxf(x1, -126.f));
  const uint64_t r = add2(t, pack2(kMagic, kMagic));
  const uint64_t n = add2(r, pack2(-kMagic, -kMagic));          // round(x), exact
  const uint64_t f = fma2(n, pack2(-1.f, -1.f), t);             // x - round(x), exact
  uint64_t q = fma2(f, pack2(0.055171459913253784f, 0.055171459913253784f), pack2(0.2426108568906784f, 0.2426108568906784f));
  q = fma2(q, f, pack2(0.6932609677314758f, 0.6932609677314758f));
  q = fma2(q, f, pack2(0.9999281167984009f, 0.9999281167984009f));
  float q0, q1, r0, r1;
  unpack2(q, q0, q1);
  unpack2(r, r0, r1);
  p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(r0) << 23));
  p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(r1) << 23));
}

template <int DCH>
struct AttnCfg {
  static constexpr int kQBytes = DCH * kBlockM * 128;
  static constexpr int kKBytes = DCH * kBlockN * 128;  // one K (or V) block
  // K/V ring. A block's load is issued when the block kKvStages before it has been consumed and is needed two block
  // periods before its own P V, so the ring gives (kKvStages - 2) block periods of lead (six stages measured the
  // same as four, also on short sequences whose K / V come from DRAM).
  static constexpr int kKvStages = 4;
  static constexpr int kQBufs = (DCH == 1) ? 2 : 1;   // Q tiles in shared memory: the next item's Q loads an item ahead
  static constexpr int kDataBytes = kQBufs * kQBytes + kKvStages * 2 * kKBytes;
  // the dynamic shared-memory window is declared 1024-byte aligned, so no slack is reserved:
  // two CTAs of the 64-wide configuration (96 KB each) must fit one SM
  static constexpr int kBarrierBytes = 256;  // 19 mbarriers + the TMEM slot + the abort flag (160 bytes), padded
  static constexpr int kSmemBytes = kDataBytes + kBarrierBytes;
  static constexpr int kTWidth = DCH * 64;                       // columns of one O accumulator
  static constexpr int kTmemCols = (DCH == 1) ? 256 : 512;       // S x2 (64 each) then O x2 (item parity)
};

// Persistent CTAs: each walks work items (one item = 128 query rows of one (batch, head)) with stride
// gridDim.x, so barrier set-up, TMEM allocation and the load latency of the first tiles are paid once
// and the next item's Q / K / V stream in while the current item drains.
// Pipeline (key blocks numbered globally g = 0, 1, .. across items; S and P double-buffered on g & 1, O on the
// item's parity):
//   MMA warp:      S(0), S(1); then for each j: wait P(j) -> O += P(j) V(j) -> S(j+2)
//   softmax warps: wait S(j) -> max / exp2 / row sum -> P(j) -> signal; at the item's end O / row sum -> global
// so the tensor core computes S(j+1), S(j+2) and P(j-1) V(j-1) while the softmax threads work on block j.
// The softmax is "lazy" about the running maximum: a row keeps a reference maximum m_ref and evaluates
// p = exp2(s * scale - m_ref); m_ref is raised (and O and the row sum rescaled by exp2(m_ref_old - m_ref_new))
// only when the block's maximum exceeds it by more than kRescaleLog2, so p never exceeds 2^kRescaleLog2 and the
// final O / l is the same quotient the reference forms with the exact running maximum
// (attention_scaling_coefs_updater.h:85-165), up to the rounding of P at a different power-of-two-ish scale.
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
  uint8_t* sKV = sQ + Cfg::kQBufs * Cfg::kQBytes;  // stage s: K at sKV + s*2*kKBytes, V right after K
  uint64_t* q_full = reinterpret_cast<uint64_t*>(sKV + Cfg::kKvStages * 2 * Cfg::kKBytes);  // [2]
  uint64_t* kv_full = q_full + 2;
  uint64_t* kv_empty = kv_full + Cfg::kKvStages;
  uint64_t* s_full = kv_empty + Cfg::kKvStages;  // [2]
  uint64_t* p_full = s_full + 2;            // [2]
  // "P(g) V(g) has been accumulated into O" is the same event as "K/V stage g % Cfg::kKvStages is free": the softmax
  // threads wait on kv_empty for it (before a rescale of O, and for the item's last block before reading O out),
  // which spares two tcgen05.commit per key block; a commit costs the MMA thread as much as an MMA
  uint64_t* o_empty = p_full + 2;           // [2] the softmax threads have read the item's O out of TMEM
  uint64_t* drain_bar = o_empty + 2;         // [2] one per issuing thread, used only when a wait has given up
  uint64_t* q_empty = drain_bar + 2;          // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  static_assert((2 + 2 * Cfg::kKvStages + 2 * 3 + 4) * 8 + 8 <= Cfg::kBarrierBytes, "barrier block overflows its shared memory");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // work item -> where its rows live and how many key blocks it walks. n_blocks == 0 (a query tile past the end of
  // a short sequence in packed mode) means the item is skipped by every role alike.
  struct Item {
    int h, b4;      // head and batch coordinates of the tensor maps
    int row0;       // first row of the sequence in the maps' row dimension (0 unless packed)
    int q0;         // first query row of the tile inside its sequence
    int q_len;      // query rows of the sequence
    int kv_len;     // keys visible to this tile
    int n_blocks;
    long long out_row0;  // first output row of the sequence
  };
  auto decode_item = [&](int item) {
    Item w;
    const int bh = fast_div(item, p.q_blocks, p.q_blocks_mul, p.q_blocks_shr);
    int q_blk = item - bh * p.q_blocks;
    // causal: a tile's work grows with its position, so the items are handed out longest first (every CTA's last item
    // is then a short one, which evens out the end of the kernel)
    if (!NOMASK && p.causal) q_blk = p.q_blocks - 1 - q_blk;
    const int b = fast_div(bh, p.H, p.h_mul, p.h_shr);
    w.h = bh - b * p.H;
    w.q0 = q_blk * kBlockM;
    if (p.cu_seqlens) {
      const int lo = __ldg(p.cu_seqlens + b), hi = __ldg(p.cu_seqlens + b + 1);
      w.b4 = 0;
      w.row0 = lo;
      w.q_len = w.kv_len = max(hi - lo, 0);
      w.out_row0 = lo;
    } else {
      w.b4 = b;
      w.row0 = 0;
      w.q_len = p.Sq;
      w.kv_len = p.Skv;
      if constexpr (!NOMASK) {  // (the host sends problems with lengths to the masking variant)
        if (p.lengths_q) w.q_len = min(max(__ldg(p.lengths_q + b), 0), p.Sq);
        if (p.lengths_kv) w.kv_len = min(max(__ldg(p.lengths_kv + b), 0), p.Skv);
      }
      w.out_row0 = static_cast<long long>(b) * p.Sq;
    }
    if (!NOMASK && p.causal) w.kv_len = min(w.kv_len, w.q0 + kBlockM);
    w.n_blocks = (w.q0 < w.q_len) ? (w.kv_len + kBlockN - 1) / kBlockN : 0;
    return w;
  };
  auto load_rows = [&](void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int row, const Item& w, int order) {
    if (order == 0)
      tma_load_4d(dst, map, bar, c0, row, w.h, w.b4);
    else
      tma_load_4d(dst, map, bar, c0, w.h, row, w.b4);
  };
  const int dsteps = (p.D + 15) / 16;  // k-steps of Q K^T

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_full + 1, 1);
    for (int s = 0; s < Cfg::kKvStages; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 128);
      mbar_init(&o_empty[i], 128);
    }
    mbar_init(drain_bar, 1);
    mbar_init(drain_bar + 1, 1);
    mbar_init(q_empty, 1);
    mbar_init(q_empty + 1, 1);
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
  const uint32_t tmem_s = tmem_base;        // S(j) at + (j & 1) * 64; P(j) as 16-bit pairs over its first 32 columns
  const uint32_t tmem_o = tmem_base + 128;  // O of item it at + (it & 1) * kTWidth

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      int g = 0;  // global key-block counter (K/V ring position)
      int it = 0;
      for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x) {
        const Item w = decode_item(item);
        if (w.n_blocks == 0) continue;
        // Q buffer qb is free once the last S = Q K^T of the item that used it before has completed
        const int qb = it % Cfg::kQBufs;
        const uint32_t qph = static_cast<uint32_t>(it / Cfg::kQBufs) & 1u;
        ok = mbar_wait(&q_empty[qb], qph ^ 1u, abort_flag, p.status, kDevWaitEmptyTimeout);
        if (!ok) break;
        mbar_arrive_expect_tx(&q_full[qb], Cfg::kQBytes);
#pragma unroll
        for (int c = 0; c < DCH; ++c)
          load_rows(sQ + qb * Cfg::kQBytes + c * kBlockM * 128, &tma_q, &q_full[qb], c * 64, w.row0 + w.q0, w, p.q_order);
        for (int j = 0; j < w.n_blocks; ++j, ++g) {
          const int st = g % Cfg::kKvStages;
          const uint32_t ph = (g / Cfg::kKvStages) & 1;
          ok = mbar_wait(&kv_empty[st], ph ^ 1u, abort_flag, p.status, kDevWaitEmptyTimeout);
          if (!ok) break;
          uint8_t* sK = sKV + st * 2 * Cfg::kKBytes;
          uint8_t* sV = sK + Cfg::kKBytes;
          mbar_arrive_expect_tx(&kv_full[st], 2 * Cfg::kKBytes);
#pragma unroll
          for (int c = 0; c < DCH; ++c) {
            load_rows(sK + c * kBlockN * 128, &tma_k, &kv_full[st], c * 64, w.row0 + j * kBlockN, w, p.k_order);
            load_rows(sV + c * kBlockN * 128, &tma_v, &kv_full[st], c * 64, w.row0 + j * kBlockN, w, p.v_order);
          }
        }
        ++it;
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {
        }
      }
    }
#ifndef B200AIT_ATTN_NO_SYNCWARP
    __syncwarp();
#endif
  } else if (warp == 1) {
    // P V issuer: O(item) += P(g) V(g) as soon as the softmax threads have put P(g) into TMEM
    if (lane == 0) {
      constexpr uint32_t idesc_t = umma_idesc_f16(kBlockM, Cfg::kTWidth, BF16, false, true);  // V is MN-major
      bool ok = true;
      ATTN_PROBE_DECL(blockIdx.x == 0)
      int gb = 0;  // global index of the item's first key block
      int it = 0;
      for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x) {
        const Item w = decode_item(item);
        const int n_blocks = w.n_blocks;
        if (n_blocks == 0) continue;
        // this item's O buffer was last used by item it - 2: its rows must have been read out
        ok = mbar_wait(&o_empty[it & 1], ((it >> 1) & 1) ^ 1u, abort_flag, p.status, kDevWaitAccEmptyTimeout);
        const uint32_t o_addr = tmem_o + static_cast<uint32_t>((it & 1) * Cfg::kTWidth);
        for (int j = 0; ok && j < n_blocks; ++j) {
          const int g = gb + j;
          ATTN_PROBE(1)  // loop bookkeeping
          ok = mbar_wait(&p_full[g & 1], (g >> 1) & 1, abort_flag, p.status, kDevWaitOtherTimeout);
          if (!ok) break;
          tc_fence_after();
          ATTN_PROBE(2)  // wait for P
          const int st = g % Cfg::kKvStages;
          const uint32_t p_tmem = tmem_s + static_cast<uint32_t>((g & 1) * kBlockN);
          const uint32_t v_addr = smem_u32(sKV + st * 2 * Cfg::kKBytes + Cfg::kKBytes);
#pragma unroll
          for (int k = 0; k < kBlockN / 16; ++k) {
            // A = P from TMEM: 16 keys of a row are 8 columns of 16-bit pairs.
            // V block rows are keys (128 B each): 16 keys per step = 2048 B; 64-wide d chunks are
            // kBlockN*128 B apart (leading byte offset), 8-key groups 1024 B apart (stride byte offset)
            const uint64_t bdesc = umma_smem_desc_sw128(v_addr + k * 2048, kBlockN * 128, 1024);
            umma_f16_ts(o_addr, p_tmem + k * 8, bdesc, idesc_t, (j != 0 || k != 0) ? 1u : 0u);
          }
          umma_commit(&kv_empty[st]);  // K/V stage free; also "P(g) V(g) is in O" for the softmax threads and the S issuer
          ATTN_PROBE(0)  // issue of the 4 P V MMAs + commit
        }
        gb += n_blocks;
        ++it;
      }
      ATTN_PROBE_FLUSH(16)
      if (!ok) {
        umma_commit(drain_bar);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(drain_bar, 0) && globaltimer_ns() - t0 < 1000000ull) {
        }
      }
    }
#ifndef B200AIT_ATTN_NO_SYNCWARP
    __syncwarp();
#endif
  } else if (warp == 6) {
    // S issuer: S(g) = Q K(g)^T into S buffer g & 1 (g = global key-block index). A second issuing thread, so that
    // waiting for P and issuing P V never delays the scores of the blocks ahead (and the other way round): one
    // thread issuing both spent as long on its own waits and commits as the softmax threads on a block.
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_f16(kBlockM, kBlockN, BF16, false, false);
      bool ok = true;
      int gb = 0;
      int it = 0;
      for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x) {
        const Item w = decode_item(item);
        const int n_blocks = w.n_blocks;
        if (n_blocks == 0) continue;
        const int qb = it % Cfg::kQBufs;
        const uint32_t q_addr = smem_u32(sQ + qb * Cfg::kQBytes);
        ok = mbar_wait(&q_full[qb], static_cast<uint32_t>(it / Cfg::kQBufs) & 1u, abort_flag, p.status, kDevWaitFullTimeout);
        for (int j = 0; ok && j < n_blocks; ++j) {
          const int g = gb + j;
          const int st = g % Cfg::kKvStages;
          // S buffer g & 1 still holds P(g - 2) until P(g - 2) V(g - 2) has completed (un-aliasing P, so that the
          // scores only wait for the softmax threads to have loaded S(g - 2), was measured: no faster)
          if (g >= 2)
            ok = mbar_wait(&kv_empty[(g - 2) % Cfg::kKvStages], ((g - 2) / Cfg::kKvStages) & 1, abort_flag, p.status,
                           kDevWaitAccEmptyTimeout);
          if (ok) ok = mbar_wait(&kv_full[st], (g / Cfg::kKvStages) & 1, abort_flag, p.status, kDevWaitFullTimeout);
          if (!ok) break;
          tc_fence_after();
#ifdef B200AIT_ATTN_PROBE
          if (blockIdx.x == 0) g_attn_probe[20] += 1;  // S tiles issued
#endif
          const uint32_t k_addr = smem_u32(sKV + st * 2 * Cfg::kKBytes);
          for (int k = 0; k < dsteps; ++k) {
            const int c = k >> 2, kk = k & 3;
            const uint64_t adesc = umma_smem_desc_sw128(q_addr + c * kBlockM * 128 + kk * 32, 16, 1024);
            const uint64_t bdesc = umma_smem_desc_sw128(k_addr + c * kBlockN * 128 + kk * 32, 16, 1024);
            umma_f16_ss(tmem_s + static_cast<uint32_t>((g & 1) * kBlockN), adesc, bdesc, idesc_s, k != 0 ? 1u : 0u);
          }
          umma_commit(&s_full[g & 1]);
          if (j + 1 == n_blocks) umma_commit(&q_empty[qb]);  // every S of this item has been issued: its Q may be replaced
        }
        gb += n_blocks;
        ++it;
      }
      if (!ok) {
        umma_commit(drain_bar + 1);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(drain_bar + 1, 0) && globaltimer_ns() - t0 < 1000000ull) {
        }
      }
    }
#ifndef B200AIT_ATTN_NO_SYNCWARP
    __syncwarp();
#endif
  } else {
    using E = Elem16<BF16>;
    using T = typename E::T;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;  // row inside the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    bool ok = true;
    int gb = 0;  // global index of the item's first key block
    int it = 0;
    ATTN_PROBE_DECL(blockIdx.x == 0 && threadIdx.x == 64)
    // The read-out of an item's O (wait for its last P V, O / row sum -> global memory) is deferred until this thread
    // has handed the NEXT item's first P block to the tensor core: by then the last P V has long completed, so the
    // thread never waits for it, and its TMEM loads and stores overlap the other warps' exponentials. O is
    // double-buffered on the item's parity, which is what makes the deferral legal.
    struct Pending {
      bool valid = false;
      int it = 0, last_g = 0;   // item counter (selects the O buffer) and global index of its last key block
      float inv_l = 0.f;
      T* out = nullptr;         // this row's output; null when the row lies past the end of its sequence
    } pend;
    auto flush_pending = [&]() -> bool {
      if (!pend.valid) return true;
      pend.valid = false;
      // the item's O is complete once its last P V has been accumulated
      if (!mbar_wait(&kv_empty[pend.last_g % Cfg::kKvStages], (pend.last_g / Cfg::kKvStages) & 1, abort_flag, p.status,
                     kDevWaitAccFullTimeout))
        return false;
      tc_fence_after();
      const uint32_t o_prev = tmem_o + lane_addr + static_cast<uint32_t>((pend.it & 1) * Cfg::kTWidth);
#pragma unroll
      for (int c = 0; c < DCH * 2; ++c) {
        if (c * 32 < p.Dv) {  // warp-uniform
          uint32_t v[32];
          tmem_ld_32x32b_x32(o_prev + c * 32, v);
          tmem_ld_wait();
          if (pend.out != nullptr) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              if (c * 32 + u * 8 < p.Dv) {
                float f[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[u * 8 + i]) * pend.inv_l;
                *reinterpret_cast<uint4*>(pend.out + c * 32 + u * 8) = pack8<BF16>(f);
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&o_empty[pend.it & 1]);
      return true;
    };
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x) {
      const Item w = decode_item(item);
      const int n_blocks = w.n_blocks, kv_len = w.kv_len;
      if (n_blocks == 0) {
        // no key for this tile's rows (lengths_kv[b] == 0): softmax over nothing, NaN like the reference's 0 / 0
        if (!NOMASK && p.lengths_kv != nullptr && w.q0 + r < w.q_len) {
          T* row_out = static_cast<T*>(p.out) + ((w.out_row0 + w.q0 + r) * p.H + w.h) * p.Dv;
          const uint32_t nan2 = E::from_float2(__int_as_float(0x7fc00000), __int_as_float(0x7fc00000));
          for (int c = 0; c < p.Dv; c += 8) *reinterpret_cast<uint4*>(row_out + c) = make_uint4(nan2, nan2, nan2, nan2);
        }
        continue;
      }
      const int q_idx = w.q0 + r;
      const uint32_t o_addr = tmem_o + lane_addr + static_cast<uint32_t>((it & 1) * Cfg::kTWidth);
      float m_ref = -INFINITY, l_run = 0.f;
      for (int j = 0; ok && j < n_blocks; ++j) {
        const int g = gb + j;
        ok = mbar_wait(&s_full[g & 1], (g >> 1) & 1, abort_flag, p.status, kDevWaitAccFullTimeout);
        if (!ok) break;
        tc_fence_after();
        ATTN_PROBE(0)  // wait for S (and whatever the loop does before it)
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
        ATTN_PROBE(1)  // S from TMEM
        float l0 = 0.f, l1 = 0.f;
        // One body, compiled twice: kPlain drops every per-element mask.
        auto softmax_block = [&](auto plain_tag) {
          constexpr bool kPlain = decltype(plain_tag)::value;
          float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float a0 = __uint_as_float(s0[i]), a1 = __uint_as_float(s0[i + 1]);
            const float a2 = __uint_as_float(s0[i + 2]), a3 = __uint_as_float(s0[i + 3]);
            const float b0 = __uint_as_float(s1[i]), b1 = __uint_as_float(s1[i + 1]);
            const float b2 = __uint_as_float(s1[i + 2]), b3 = __uint_as_float(s1[i + 3]);
            if constexpr (kPlain) {
              m0 = max3(m0, a0, a1);
              m1 = max3(m1, a2, a3);
              m2 = max3(m2, b0, b1);
              m3 = max3(m3, b2, b3);
            } else {
              m0 = max3(m0, (i < limit) ? a0 : -INFINITY, (i + 1 < limit) ? a1 : -INFINITY);
              m1 = max3(m1, (i + 2 < limit) ? a2 : -INFINITY, (i + 3 < limit) ? a3 : -INFINITY);
              m2 = max3(m2, (32 + i < limit) ? b0 : -INFINITY, (33 + i < limit) ? b1 : -INFINITY);
              m3 = max3(m3, (34 + i < limit) ? b2 : -INFINITY, (35 + i < limit) ? b3 : -INFINITY);
            }
          }
          const float m_blk = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * p.scale_log2;
          // Raise the reference maximum only when some row of this warp outgrew it by more than the slack
          // (always on an item's first block, where nothing has been accumulated yet). The TMEM accesses of
          // the rescale are warp-wide, so the decision is too; rows that did not move get alpha = 1.
          if (__any_sync(0xffffffffu, m_blk > m_ref + kRescaleLog2)) {
            const float m_new = fmaxf(m_ref, m_blk);
            if (j > 0) {
              // O holds blocks 0 .. j-1 once P(j-1) V(j-1) is done; P(j) V(j) cannot start before this
              // thread's arrival on p_full below
              if (!mbar_wait(&kv_empty[(g - 1) % Cfg::kKvStages], ((g - 1) / Cfg::kKvStages) & 1, abort_flag, p.status,
                             kDevWaitAccFullTimeout)) {
                ok = false;
              } else {
                tc_fence_after();
                const float alpha = (m_new == -INFINITY) ? 1.f : exp2f(m_ref - m_new);  // m_ref = -inf: O is 0 anyway
                const uint64_t alpha2 = pack2(alpha, alpha);
#pragma unroll
                for (int c = 0; c < DCH * 4; ++c) {
                  if (c * 16 < p.Dv) {  // warp-uniform
                    uint32_t v[16];
                    tmem_ld_32x32b_x16(o_addr + c * 16, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
                      float x0, x1;
                      unpack2(mul2(pack2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])), alpha2), x0, x1);
                      v[i] = __float_as_uint(x0);
                      v[i + 1] = __float_as_uint(x1);
                    }
                    tmem_st_32x32b_x16(o_addr + c * 16, v);
                  }
                }
                tmem_st_wait();
                l_run *= alpha;
              }
            }
            m_ref = m_new;
          }
          ATTN_PROBE(2)  // row max (+ rescale when it happens)
          const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
          // p = exp2(s * scale - m_ref), row sum, P rounded to 16 bits (kernel_forward.h:785-824) and written as
          // pairs over the first 32 columns of this S buffer: every S value of the row is in registers by now
          const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2), negm2 = pack2(-m_use, -m_use);
          uint64_t lsum2 = pack2(0.f, 0.f);
          uint32_t packed[32];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t(&sv)[32] = h == 0 ? s0 : s1;
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              float x0, x1;
              unpack2(fma2(pack2(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])), scale2, negm2), x0, x1);
#ifdef B200AIT_ATTN_EXP_SKIP  // tuning experiment: no exponentials, to expose the MMA side's own pace
              float p0 = x0, p1 = x1;
#else
              float p0, p1;
              if (((i >> 1) & 7) < kPolyOf8) {  // compile-time: the loop is unrolled
                exp2_poly2(x0, x1, p0, p1);
              } else {
                p0 = exp2f(x0);
                p1 = exp2f(x1);
              }
#endif
              if (!kPlain) {
                p0 = (h * 32 + i < limit) ? p0 : 0.f;
                p1 = (h * 32 + i + 1 < limit) ? p1 : 0.f;
              }
              lsum2 = add2(lsum2, pack2(p0, p1));
              packed[h * 16 + (i >> 1)] = E::from_float2(p0, p1);
            }
          }
          tmem_st_32x32b_x32(s_addr, packed);
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
        l_run += l0 + l1;
        tmem_st_wait();  // P is in TMEM
        tc_fence_before();
        mbar_arrive(&p_full[g & 1]);
        ATTN_PROBE(3)  // exp2 pass, P to TMEM, fence, arrive
        if (j == 0 && ok) ok = flush_pending();  // the previous item's O, now that this item's first P is on its way
      }
      gb += n_blocks;
      if (ok) {
        pend.valid = true;
        pend.it = it;
        pend.last_g = gb - 1;
        pend.inv_l = (l_run > 0.f) ? 1.f / l_run : 0.f;
        pend.out = (q_idx < w.q_len) ? static_cast<T*>(p.out) + ((w.out_row0 + q_idx) * p.H + w.h) * p.Dv : nullptr;
      }
      ATTN_PROBE(0)  // item bookkeeping (booked with the wait for S)
      ++it;
    }
    if (ok) ok = flush_pending();  // the last item of this CTA
    ATTN_PROBE_FLUSH(0)
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
  const int batch = static_cast<int>(bh / p.H);
  if (p.lengths_q != nullptr && qi >= __ldg(p.lengths_q + batch)) return;  // (the whole warp: it owns one row)
  int kv_len = p.lengths_kv != nullptr ? min(max(__ldg(p.lengths_kv + batch), 0), p.Skv) : p.Skv;
  const bool no_keys = kv_len == 0;
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
  const float inv = (l_run > 0.f) ? 1.f / l_run : no_keys ? __int_as_float(0x7fc00000) : 0.f;  // no key at all: NaN
  const long long b = bh / p.H, h = bh - b * p.H;
  T* out = static_cast<T*>(p.out) + ((b * p.Sq + qi) * p.H + h) * p.Dv;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int d = lane + 32 * i;
    if (d < p.Dv) out[d] = E::from_float(o[i] * inv);
  }
}

// 4-D map over one operand with the operand's element strides, 128-byte swizzle, box = 64 channels x box_rows rows
// of one head of one batch; a box wider than D, or reaching past the last row, zero-fills. The row and head
// dimensions are emitted in ascending-stride order: order 0 = (channel, row, head, batch), 1 = (channel, head, row, batch).
static int attn_map_order(const AttnOperand& op) { return op.head_stride < op.row_stride ? 1 : 0; }
static CUtensorMap make_attn_map(const AttnOperand& op, bool bf16, int d, long long rows, int heads, int batches,
                                 int box_rows) {
  CUtensorMap m;
  const int order = attn_map_order(op);
  const cuuint64_t row_dim = static_cast<cuuint64_t>(rows), head_dim = static_cast<cuuint64_t>(heads);
  const cuuint64_t row_str = static_cast<cuuint64_t>(op.row_stride) * 2, head_str = static_cast<cuuint64_t>(op.head_stride) * 2;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(d), order ? head_dim : row_dim, order ? row_dim : head_dim,
                        static_cast<cuuint64_t>(batches)};
  cuuint64_t strides[3] = {order ? head_str : row_str, order ? row_str : head_str,
                           static_cast<cuuint64_t>(op.batch_stride) * 2};
  const cuuint32_t br = static_cast<cuuint32_t>(box_rows);
  cuuint32_t box[4] = {64, order ? 1u : br, order ? br : 1u, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = get_encode_fn()(&m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                               const_cast<void*>(op.ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw Error("attention: cuTensorMapEncodeTiled failed with CUresult " + std::to_string(static_cast<int>(r)));
  return m;
}

template <int DCH, bool BF16, bool NOMASK>
void launch_attn_variant(const AttnOperand& q, const AttnOperand& k, const AttnOperand& v, const AttnParams& p,
                         long long q_rows, long long kv_rows, cudaStream_t stream) {
  using Cfg = AttnCfg<DCH>;
  static std::atomic<uint64_t> configured{0};
  opt_in_smem_once(configured, reinterpret_cast<const void*>(&attention_tc_kernel<DCH, BF16, NOMASK>), Cfg::kSmemBytes);
  const int map_batches = p.cu_seqlens ? 1 : p.B;
  CUtensorMap tq = make_attn_map(q, BF16, p.D, q_rows, p.H, map_batches, kBlockM);
  CUtensorMap tk = make_attn_map(k, BF16, p.D, kv_rows, p.H, map_batches, kBlockN);
  CUtensorMap tv = make_attn_map(v, BF16, p.Dv, kv_rows, p.H, map_batches, kBlockN);
  const long long items = static_cast<long long>(p.B) * p.H * p.q_blocks;
  B200AIT_REQUIRE(items < (1ll << 31), "attention: too many work items");
  AttnParams pp = p;
  pp.num_items = static_cast<int>(items);
  pp.q_order = attn_map_order(q), pp.k_order = attn_map_order(k), pp.v_order = attn_map_order(v);
#ifdef B200AIT_ATTN_ONE_CTA  // tuning experiment: one CTA per SM
  const long long grid = std::min<long long>(items, static_cast<long long>(sm_count()));
#else
  const long long grid = std::min<long long>(items, static_cast<long long>(sm_count()) * (DCH == 1 ? 2 : 1));
#endif
  ::b200ait::count_launch(), attention_tc_kernel<DCH, BF16, NOMASK><<<static_cast<unsigned>(grid), kAttnThreads, Cfg::kSmemBytes, stream>>>(tq, tk, tv,
                                                                                                                 pp);
  B200AIT_CUDA_CHECK(cudaGetLastError());
}

template <int DCH, bool BF16>
void launch_attn(const AttnOperand& q, const AttnOperand& k, const AttnOperand& v, const AttnParams& p,
                 long long q_rows, long long kv_rows, cudaStream_t stream) {
  if (!p.causal && !p.cu_seqlens && !p.lengths_kv && !p.lengths_q && p.Skv % kBlockN == 0)
    launch_attn_variant<DCH, BF16, true>(q, k, v, p, q_rows, kv_rows, stream);
  else
    launch_attn_variant<DCH, BF16, false>(q, k, v, p, q_rows, kv_rows, stream);
}

static bool operand_ok_for_tma(const AttnOperand& o) {
  return (reinterpret_cast<uintptr_t>(o.ptr) & 15u) == 0 && o.row_stride % 8 == 0 && o.head_stride % 8 == 0 &&
         o.batch_stride % 8 == 0 && o.row_stride > 0 && o.head_stride > 0 && o.batch_stride > 0;
}

// Shared body of the attention entry points. q_rows / kv_rows: extent of the row dimension of the operands
// (Sq / Skv, or the packed total). The tensor-core kernel takes every layout whose strides are multiples of 8
// elements; the CUDA-core kernel needs contiguous [B, H, S, D] operands.
static void attention_run(void* output, const AttnOperand& q, const AttnOperand& k, const AttnOperand& v, AttnParams p,
                          long long q_rows, long long kv_rows, bool contiguous_bhsd, bool bf16, cudaStream_t stream) {
  p.q_blocks = (p.Sq + kBlockM - 1) / kBlockM;
  const FastDiv by_q_blocks(p.q_blocks), by_heads(p.H);
  p.q_blocks_mul = by_q_blocks.mul, p.q_blocks_shr = by_q_blocks.shr;
  p.h_mul = by_heads.mul, p.h_shr = by_heads.shr;
  p.out = output;
  p.status = device_status_word();
  const bool tc_ok = p.D % 8 == 0 && p.Dv % 8 == 0 && p.D <= 128 && p.Dv <= 128 && operand_ok_for_tma(q) &&
                     operand_ok_for_tma(k) && operand_ok_for_tma(v) &&
                     (reinterpret_cast<uintptr_t>(output) & 15u) == 0;
  if (tc_ok) {
    const bool two = p.D > 64 || p.Dv > 64;
    if (two) {
      if (bf16)
        launch_attn<2, true>(q, k, v, p, q_rows, kv_rows, stream);
      else
        launch_attn<2, false>(q, k, v, p, q_rows, kv_rows, stream);
    } else {
      if (bf16)
        launch_attn<1, true>(q, k, v, p, q_rows, kv_rows, stream);
      else
        launch_attn<1, false>(q, k, v, p, q_rows, kv_rows, stream);
    }
    return;
  }
  B200AIT_REQUIRE(contiguous_bhsd && !p.cu_seqlens,
                  "attention: this layout needs head sizes that are multiples of 8 (at most 128) and 16-byte aligned, "
                  "8-element-strided operands");
  B200AIT_REQUIRE(p.Dv <= 256, "attention: head_size_v > 256 is not supported");
  const long long rows = static_cast<long long>(p.B) * p.H * p.Sq;
  const unsigned grid = static_cast<unsigned>((rows + 3) / 4);
  const size_t sh = 4 * static_cast<size_t>(p.D) * sizeof(float);
  if (bf16)
    ::b200ait::count_launch(), attention_simt_kernel<true><<<grid, 128, sh, stream>>>(q.ptr, k.ptr, v.ptr, p);
  else
    ::b200ait::count_launch(), attention_simt_kernel<false><<<grid, 128, sh, stream>>>(q.ptr, k.ptr, v.ptr, p);
  B200AIT_CUDA_CHECK(cudaGetLastError());
}

}  // namespace b200ait

using namespace b200ait;

// Argument order follows the reference's generated function
// (python/aitemplate/backend/cuda/attention/mem_eff_attention.py:632-654). lengths_kv / lengths_q: null, or
// batch_size int32 values on the device (the op's variable_seq_length_kv / variable_seq_length_q inputs).
B200AIT_EXPORT int b200ait_mem_eff_attention(void* output, const void* query, const void* key, const void* value,
                                             int64_t batch_size, int64_t seq_len_kv, int64_t seq_len_q,
                                             int num_heads, int head_size, int head_size_v, float softmax_scale,
                                             int is_causal, const int32_t* lengths_kv, const int32_t* lengths_q,
                                             int dtype, cudaStream_t stream) {
  return guarded("b200ait_mem_eff_attention", [&] {
    B200AIT_REQUIRE(dtype == kDTypeHalf || dtype == kDTypeBFloat16, "attention: dtype must be float16 or bfloat16");
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
    p.scale_log2 = softmax_scale * 1.4426950408889634f;
    p.causal = is_causal ? 1 : 0;
    p.cu_seqlens = nullptr;
    p.lengths_kv = lengths_kv, p.lengths_q = lengths_q;
    const long long h = num_heads;
    const AttnOperand q{query, head_size, seq_len_q * head_size, h * seq_len_q * head_size};
    const AttnOperand k{key, head_size, seq_len_kv * head_size, h * seq_len_kv * head_size};
    const AttnOperand v{value, head_size_v, seq_len_kv * head_size_v, h * seq_len_kv * head_size_v};
    attention_run(output, q, k, v, p, seq_len_q, seq_len_kv, true, dtype == kDTypeBFloat16, stream);
  });
}

// mem_eff_attention over operands that are strided views: each of q, k, v is addressed as [batch, head, row, channel]
// with the element strides given (channel stride 1), e.g. a [B, S, H, D] projection output read in place
// ({H*D, D, S*H*D}) instead of through a permute copy. Output [B, Sq, H, Dv] contiguous. Strides must be positive
// multiples of 8 elements and head sizes multiples of 8 up to 128 (the tensor-core kernel is the only one that
// takes strided operands). Counterpart of the reference's input TensorAccessors on this op
// (python/aitemplate/backend/cuda/attention/mem_eff_attention.py:160-171 pass q/k/v strides to the kernel).
B200AIT_EXPORT int b200ait_mem_eff_attention_strided(void* output, const void* query, const void* key,
                                                     const void* value, int64_t batch_size, int64_t seq_len_kv,
                                                     int64_t seq_len_q, int num_heads, int head_size, int head_size_v,
                                                     const int64_t* q_strides, const int64_t* k_strides,
                                                     const int64_t* v_strides, float softmax_scale, int is_causal,
                                                     int dtype, cudaStream_t stream) {
  return guarded("b200ait_mem_eff_attention_strided", [&] {
    B200AIT_REQUIRE(dtype == kDTypeHalf || dtype == kDTypeBFloat16, "attention: dtype must be float16 or bfloat16");
    B200AIT_REQUIRE(q_strides && k_strides && v_strides, "attention: strides are null");
    B200AIT_REQUIRE(batch_size >= 0 && seq_len_kv >= 0 && seq_len_q >= 0 && num_heads >= 0 && head_size >= 0 &&
                        head_size_v >= 0,
                    "attention: negative dimension");
    if (batch_size == 0 || seq_len_q == 0 || num_heads == 0 || head_size_v == 0) return;
    B200AIT_REQUIRE(output && query && key && value, "attention: null pointer with non-zero size");
    B200AIT_REQUIRE(seq_len_kv > 0 && head_size > 0, "attention: empty key sequence or head");
    B200AIT_REQUIRE(seq_len_q < (1 << 30) && seq_len_kv < (1 << 30), "attention: sequence too long");
    AttnParams p{};
    p.B = static_cast<int>(batch_size), p.H = num_heads;
    p.Sq = static_cast<int>(seq_len_q), p.Skv = static_cast<int>(seq_len_kv);
    p.D = head_size, p.Dv = head_size_v;
    p.scale_log2 = softmax_scale * 1.4426950408889634f;
    p.causal = is_causal ? 1 : 0;
    p.cu_seqlens = nullptr;
    const AttnOperand q{query, q_strides[0], q_strides[1], q_strides[2]};
    const AttnOperand k{key, k_strides[0], k_strides[1], k_strides[2]};
    const AttnOperand v{value, v_strides[0], v_strides[1], v_strides[2]};
    attention_run(output, q, k, v, p, seq_len_q, seq_len_kv, false, dtype == kDTypeBFloat16, stream);
  });
}

// flash_attention: packed-QKV variable-length attention. qkv is [total, 3, num_heads, head_size]; cu_seqlens
// (device, int32, batch_size + 1 entries) gives each sequence's first row; output [total, num_heads, head_size].
// Argument order follows the reference's generated function
// (python/aitemplate/backend/cuda/attention/flash_attention.py:199-215); softmax_lse, o_tmp and loop are its
// kernel's scratch and scheduling arguments and are ignored here (may be null), p_dropout must be 0. `total` rows
// are read from cu_seqlens on the device, so the host only needs seq_len = the longest sequence's length (an upper
// bound is enough) and total_rows = the row extent of qkv.
B200AIT_EXPORT int b200ait_flash_attention(void* output, const void* qkv, const int* cu_seqlens, float* softmax_lse,
                                           float* o_tmp, int batch_size, int seq_len, int num_heads, int head_size,
                                           float p_dropout, float softmax_scale, int is_causal, int loop,
                                           int64_t total_rows, int dtype, cudaStream_t stream) {
  (void)softmax_lse, (void)o_tmp, (void)loop;
  return guarded("b200ait_flash_attention", [&] {
    B200AIT_REQUIRE(dtype == kDTypeHalf || dtype == kDTypeBFloat16, "attention: dtype must be float16 or bfloat16");
    B200AIT_REQUIRE(p_dropout == 0.f, "flash_attention: dropout is not supported (inference only)");
    B200AIT_REQUIRE(batch_size >= 0 && seq_len >= 0 && num_heads >= 0 && head_size >= 0 && total_rows >= 0,
                    "attention: negative dimension");
    if (batch_size == 0 || seq_len == 0 || num_heads == 0 || head_size == 0 || total_rows == 0) return;
    B200AIT_REQUIRE(output && qkv && cu_seqlens, "attention: null pointer with non-zero size");
    B200AIT_REQUIRE(head_size % 8 == 0 && head_size <= 128, "flash_attention: head size must be a multiple of 8, at most 128");
    B200AIT_REQUIRE(total_rows < (1ll << 30), "attention: too many rows");
    AttnParams p{};
    p.B = batch_size, p.H = num_heads;
    p.Sq = p.Skv = seq_len;
    p.D = p.Dv = head_size;
    p.scale_log2 = softmax_scale * 1.4426950408889634f;
    p.causal = is_causal ? 1 : 0;
    p.cu_seqlens = cu_seqlens;
    const long long hd = static_cast<long long>(num_heads) * head_size;
    const size_t esz = 2;
    const uint8_t* base = static_cast<const uint8_t*>(qkv);
    const AttnOperand q{base, 3 * hd, head_size, 3 * hd * total_rows};
    const AttnOperand k{base + hd * esz, 3 * hd, head_size, 3 * hd * total_rows};
    const AttnOperand v{base + 2 * hd * esz, 3 * hd, head_size, 3 * hd * total_rows};
    attention_run(output, q, k, v, p, total_rows, total_rows, false, dtype == kDTypeBFloat16, stream);
  });
}

#ifdef B200AIT_ATTN_PROBE
// tuning builds only: copies the probe counters to the host and clears them
B200AIT_EXPORT int b200ait_attn_probe_read(long long* out32) {
  return guarded("b200ait_attn_probe_read", [&] {
    B200AIT_CUDA_CHECK(cudaDeviceSynchronize());
    B200AIT_CUDA_CHECK(cudaMemcpyFromSymbol(out32, g_attn_probe, sizeof(long long) * 32));
    long long zero[32] = {};
    B200AIT_CUDA_CHECK(cudaMemcpyToSymbol(g_attn_probe, zero, sizeof(zero)));
  });
}
#endif
