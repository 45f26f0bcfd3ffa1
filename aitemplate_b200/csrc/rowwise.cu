// Row-wise memory-bound kernels: layernorm and softmax.
//
// layernorm replaces python/aitemplate/backend/cuda/layernorm_sigmoid_mul/layernorm_sigmoid_mul_kernel.cuh:108-806
// (two-pass fp32 mean / variance, y = (x - mean) * rsqrt(var + eps) * gamma + beta, one rounding).
// softmax replaces python/aitemplate/backend/cuda/softmax/softmax.cuh:204-520 (fp32 max, exp, sum, divide).
//
// Fast paths keep one row in the registers of one warp: each lane issues all of its 16-byte loads
// up front (streaming cache hint), reduces with warp shuffles and writes 16-byte vectors, so a row
// is read once and written once. Other shapes take a block-per-row kernel that re-reads the row
// from cache. All math is fp32.
#include "common.h"
#include "epilogue.cuh"

namespace b200ait {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ uint4 ld_stream(const uint4* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(uint4* p, const uint4& v) { __stcs(p, v); }

// block-wide reductions (result broadcast to every thread); `red` holds >= 33 floats
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

// ------------------------------------------------------------------------------------- layernorm
struct LayerNormParams {
  const void* x;
  const void* gamma;  // nullptr -> 1
  const void* beta;   // nullptr -> 0
  void* y;
  long long m;
  int n;
  long long x_stride, y_stride;  // elements between consecutive rows
  float eps;
};

// Blocks per SM are forced up by the launch bounds: a warp has one row (VPL x 512 bytes) in flight, so the bytes
// in flight per SM are set by how many warps fit, i.e. by the register count. Measured on N = 768: 6 blocks
// (40 registers) 13.8 us against 14.4 us unbounded (54 registers, 4 blocks); 8 blocks spill and lose (14.9 us).
template <int VPL, bool BF16>
__global__ void __launch_bounds__(256, (VPL >= 12) ? 2 : (VPL >= 6) ? 4 : (VPL >= 3) ? 6 : 8)
    layernorm_warp_kernel(const LayerNormParams p) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= p.m) return;
  using T = typename Elem16<BF16>::T;
  const int nvec = p.n >> 3;
  const uint4* xin = reinterpret_cast<const uint4*>(static_cast<const T*>(p.x) + row * p.x_stride);
  uint4 raw[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int v = lane + 32 * i;
    raw[i] = (v < nvec) ? ld_stream(xin + v) : make_uint4(0, 0, 0, 0);
  }
  // Only the packed row stays in registers (VPL x 16 bytes per lane); each pass unpacks on the fly,
  // which keeps wide rows (N = 4096: 16 vectors per lane) at full occupancy.
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    float f[8];
    unpack8<BF16>(raw[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += f[j];
  }
  const float inv_n = 1.f / static_cast<float>(p.n);
  const float mean = warp_sum(s) * inv_n;
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    if (lane + 32 * i < nvec) {
      float f[8];
      unpack8<BF16>(raw[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = f[j] - mean;
        q += d * d;
      }
    }
  }
  const float rstd = rsqrtf(warp_sum(q) * inv_n + p.eps);
  uint4* yout = reinterpret_cast<uint4*>(static_cast<T*>(p.y) + row * p.y_stride);
  const uint4* g4 = reinterpret_cast<const uint4*>(p.gamma);
  const uint4* b4 = reinterpret_cast<const uint4*>(p.beta);
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int v = lane + 32 * i;
    if (v < nvec) {
      float f[8], g[8], b[8], o[8];
      unpack8<BF16>(raw[i], f);
      if (g4) {
        unpack8<BF16>(__ldg(g4 + v), g);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = 1.f;
      }
      if (b4) {
        unpack8<BF16>(__ldg(b4 + v), b);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) b[j] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (f[j] - mean) * rstd * g[j] + b[j];
      st_stream(yout + v, pack8<BF16>(o));
    }
  }
}

// Short rows that the vector kernel cannot take (N or a stride not a multiple of 8, an unaligned pointer; N <= 1024):
// still one warp per row and one read of the row, element by element (a warp's load covers 64 consecutive bytes),
// instead of a block per row with shared-memory reductions.
template <int EPL, bool BF16>
__global__ void __launch_bounds__(256) layernorm_warp_scalar_kernel(const LayerNormParams p) {
  using E = Elem16<BF16>;
  using T = typename E::T;
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= p.m) return;
  const T* x = static_cast<const T*>(p.x) + row * p.x_stride;
  float f[EPL];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const int c = lane + 32 * i;
    f[i] = (c < p.n) ? E::to_float(x[c]) : 0.f;
    s += f[i];
  }
  const float inv_n = 1.f / static_cast<float>(p.n);
  const float mean = warp_sum(s) * inv_n;
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const float d = (lane + 32 * i < p.n) ? f[i] - mean : 0.f;
    q += d * d;
  }
  const float rstd = rsqrtf(warp_sum(q) * inv_n + p.eps);
  T* y = static_cast<T*>(p.y) + row * p.y_stride;
  const T* g = static_cast<const T*>(p.gamma);
  const T* b = static_cast<const T*>(p.beta);
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const int c = lane + 32 * i;
    if (c < p.n) {
      const float gv = g ? E::to_float(g[c]) : 1.f, bv = b ? E::to_float(b[c]) : 0.f;
      y[c] = E::from_float((f[i] - mean) * rstd * gv + bv);
    }
  }
}

// Rows wider than a warp can hold (4096 < N <= 32768, vector-aligned): one block of 512 threads per row, the packed
// row in registers (VPT x 16 bytes per thread), so the row is read once and written once like in the warp kernel;
// the two reductions go through shared memory.
template <int VPT, bool BF16>
__global__ void __launch_bounds__(512) layernorm_wide_kernel(const LayerNormParams p) {
  using T = typename Elem16<BF16>::T;
  __shared__ float red[33];
  const long long row = blockIdx.x;
  const int nvec = p.n >> 3;
  const uint4* xin = reinterpret_cast<const uint4*>(static_cast<const T*>(p.x) + row * p.x_stride);
  uint4 raw[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = static_cast<int>(threadIdx.x) + 512 * i;
    raw[i] = (v < nvec) ? ld_stream(xin + v) : make_uint4(0, 0, 0, 0);
  }
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    float f[8];
    unpack8<BF16>(raw[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += f[j];
  }
  const float inv_n = 1.f / static_cast<float>(p.n);
  const float mean = block_sum(s, red) * inv_n;
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    if (static_cast<int>(threadIdx.x) + 512 * i < nvec) {
      float f[8];
      unpack8<BF16>(raw[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = f[j] - mean;
        q += d * d;
      }
    }
  }
  const float rstd = rsqrtf(block_sum(q, red) * inv_n + p.eps);
  uint4* yout = reinterpret_cast<uint4*>(static_cast<T*>(p.y) + row * p.y_stride);
  const uint4* g4 = reinterpret_cast<const uint4*>(p.gamma);
  const uint4* b4 = reinterpret_cast<const uint4*>(p.beta);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = static_cast<int>(threadIdx.x) + 512 * i;
    if (v < nvec) {
      float f[8], g[8], b[8], o[8];
      unpack8<BF16>(raw[i], f);
      if (g4) {
        unpack8<BF16>(__ldg(g4 + v), g);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = 1.f;
      }
      if (b4) {
        unpack8<BF16>(__ldg(b4 + v), b);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) b[j] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (f[j] - mean) * rstd * g[j] + b[j];
      st_stream(yout + v, pack8<BF16>(o));
    }
  }
}

template <bool BF16>
__global__ void __launch_bounds__(512) layernorm_block_kernel(const LayerNormParams p) {
  using E = Elem16<BF16>;
  using T = typename E::T;
  __shared__ float red[33];
  const long long row = blockIdx.x;
  const T* x = static_cast<const T*>(p.x) + row * p.x_stride;
  T* y = static_cast<T*>(p.y) + row * p.y_stride;
  float s = 0.f;
  for (int i = threadIdx.x; i < p.n; i += blockDim.x) s += E::to_float(x[i]);
  const float mean = block_sum(s, red) / static_cast<float>(p.n);
  float q = 0.f;
  for (int i = threadIdx.x; i < p.n; i += blockDim.x) {
    const float d = E::to_float(x[i]) - mean;
    q += d * d;
  }
  const float rstd = rsqrtf(block_sum(q, red) / static_cast<float>(p.n) + p.eps);
  const T* g = static_cast<const T*>(p.gamma);
  const T* b = static_cast<const T*>(p.beta);
  for (int i = threadIdx.x; i < p.n; i += blockDim.x) {
    const float gv = g ? E::to_float(g[i]) : 1.f, bv = b ? E::to_float(b[i]) : 0.f;
    y[i] = E::from_float((E::to_float(x[i]) - mean) * rstd * gv + bv);
  }
}

// Rows the vector kernels cannot take (a length or a pitch that is not a multiple of 8 elements, or more than
// 32768 elements) but that fit in shared memory: a block stages its row there as it reads it, so the row crosses HBM
// once in and once out instead of three times in. W = elements per access: 8 when rows, gamma and beta are whole
// numbers of aligned 16-byte vectors (rows above 32768 elements), 2 for aligned 4-byte words, else 1.
constexpr int kStagedMaxElems = 100 * 1024;  // 200 KB of 16-bit elements
template <bool BF16, int W>
__global__ void __launch_bounds__(512) layernorm_block_staged_kernel(const LayerNormParams p) {
  constexpr bool W2 = W == 2;
  using E = Elem16<BF16>;
  using T = typename E::T;
  extern __shared__ __align__(16) unsigned char staged_row[];
  __shared__ float red[33];
  T* xs = reinterpret_cast<T*>(staged_row);
  const long long row = blockIdx.x;
  const T* x = static_cast<const T*>(p.x) + row * p.x_stride;
  T* y = static_cast<T*>(p.y) + row * p.y_stride;
  const int tid = threadIdx.x, nt = blockDim.x;
  float s = 0.f;
  if (W == 8) {
    const uint4* x8 = reinterpret_cast<const uint4*>(x);
    uint4* xs8 = reinterpret_cast<uint4*>(xs);
    for (int i = tid; i < (p.n >> 3); i += nt) {
      const uint4 w = ld_stream(x8 + i);
      xs8[i] = w;
      float f[8];
      unpack8<BF16>(w, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += f[j];
    }
  } else if (W2) {
    const uint32_t* x2 = reinterpret_cast<const uint32_t*>(x);
    uint32_t* xs2 = reinterpret_cast<uint32_t*>(xs);
    for (int i = tid; i < (p.n >> 1); i += nt) {
      const uint32_t w = __ldcs(x2 + i);
      xs2[i] = w;
      const float2 f = E::to_float2(w);
      s += f.x + f.y;
    }
  } else {
    for (int i = tid; i < p.n; i += nt) {
      const T v = x[i];
      xs[i] = v;
      s += E::to_float(v);
    }
  }
  const float inv_n = 1.f / static_cast<float>(p.n);
  const float mean = block_sum(s, red) * inv_n;  // (its barriers also publish the staged row)
  float q = 0.f;
  for (int i = tid; i < p.n; i += nt) {
    const float d = E::to_float(xs[i]) - mean;
    q += d * d;
  }
  const float rstd = rsqrtf(block_sum(q, red) * inv_n + p.eps);
  const T* g = static_cast<const T*>(p.gamma);
  const T* b = static_cast<const T*>(p.beta);
  if (W == 8) {
    uint4* y8 = reinterpret_cast<uint4*>(y);
    const uint4* g8 = reinterpret_cast<const uint4*>(g);
    const uint4* b8 = reinterpret_cast<const uint4*>(b);
    for (int i = tid; i < (p.n >> 3); i += nt) {
      float f[8], gv[8], bv[8], o[8];
      unpack8<BF16>(reinterpret_cast<const uint4*>(xs)[i], f);
      if (g) {
        unpack8<BF16>(__ldg(g8 + i), gv);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) gv[j] = 1.f;
      }
      if (b) {
        unpack8<BF16>(__ldg(b8 + i), bv);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) bv[j] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (f[j] - mean) * rstd * gv[j] + bv[j];
      st_stream(y8 + i, pack8<BF16>(o));
    }
  } else if (W2) {
    uint32_t* y2 = reinterpret_cast<uint32_t*>(y);
    for (int i = tid; i < (p.n >> 1); i += nt) {
      const float2 f = E::to_float2(reinterpret_cast<const uint32_t*>(xs)[i]);
      const float g0 = g ? E::to_float(g[2 * i]) : 1.f, g1 = g ? E::to_float(g[2 * i + 1]) : 1.f;
      const float b0 = b ? E::to_float(b[2 * i]) : 0.f, b1 = b ? E::to_float(b[2 * i + 1]) : 0.f;
      __stcs(y2 + i, E::from_float2((f.x - mean) * rstd * g0 + b0, (f.y - mean) * rstd * g1 + b1));
    }
  } else {
    for (int i = tid; i < p.n; i += nt) {
      const float gv = g ? E::to_float(g[i]) : 1.f, bv = b ? E::to_float(b[i]) : 0.f;
      y[i] = E::from_float((E::to_float(xs[i]) - mean) * rstd * gv + bv);
    }
  }
}

static bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static bool al4(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 3u) == 0; }

template <bool BF16>
void layernorm_launch(const LayerNormParams& p, cudaStream_t stream) {
  const bool aligned = (p.n % 8 == 0) && (p.x_stride % 8 == 0) && (p.y_stride % 8 == 0) && al16(p.x) && al16(p.y) &&
                       (!p.gamma || al16(p.gamma)) && (!p.beta || al16(p.beta));
  const bool vec = aligned && p.n <= 4096;
  if (aligned && p.n > 4096 && p.n <= 32768) {
    B200AIT_REQUIRE(p.m < (1ll << 31), "layernorm: too many rows");
    const unsigned grid = static_cast<unsigned>(p.m);
    const int vpt = (p.n / 8 + 511) / 512;
    if (vpt <= 2)
      ::b200ait::count_launch(), layernorm_wide_kernel<2, BF16><<<grid, 512, 0, stream>>>(p);
    else if (vpt <= 4)
      ::b200ait::count_launch(), layernorm_wide_kernel<4, BF16><<<grid, 512, 0, stream>>>(p);
    else
      ::b200ait::count_launch(), layernorm_wide_kernel<8, BF16><<<grid, 512, 0, stream>>>(p);
  } else if (vec) {
    const int nvec = p.n / 8;
    const int vpl = (nvec + 31) / 32;
    const int wpb = (vpl <= 4) ? 8 : 4;  // warps per block
    const unsigned grid = static_cast<unsigned>((p.m + wpb - 1) / wpb);
    const int threads = wpb * 32;
#define B200AIT_LN(V) ::b200ait::count_launch(), layernorm_warp_kernel<V, BF16><<<grid, threads, 0, stream>>>(p)
    if (vpl <= 1)
      B200AIT_LN(1);
    else if (vpl <= 2)
      B200AIT_LN(2);
    else if (vpl <= 3)
      B200AIT_LN(3);
    else if (vpl <= 4)
      B200AIT_LN(4);
    else if (vpl <= 6)
      B200AIT_LN(6);
    else if (vpl <= 8)
      B200AIT_LN(8);
    else if (vpl <= 12)
      B200AIT_LN(12);
    else
      B200AIT_LN(16);
#undef B200AIT_LN
  } else if (p.n <= 1024) {
    const unsigned grid = static_cast<unsigned>((p.m + 7) / 8);
    const int epl = (p.n + 31) / 32;
#define B200AIT_LNS(V) ::b200ait::count_launch(), layernorm_warp_scalar_kernel<V, BF16><<<grid, 256, 0, stream>>>(p)
    if (epl <= 1) B200AIT_LNS(1); else if (epl <= 2) B200AIT_LNS(2); else if (epl <= 4) B200AIT_LNS(4);
    else if (epl <= 8) B200AIT_LNS(8); else if (epl <= 16) B200AIT_LNS(16); else B200AIT_LNS(32);
#undef B200AIT_LNS
  } else if (p.n <= kStagedMaxElems) {
    B200AIT_REQUIRE(p.m < (1ll << 31), "layernorm: too many rows");
    const bool w2 = p.n % 2 == 0 && p.x_stride % 2 == 0 && p.y_stride % 2 == 0 && al4(p.x) && al4(p.y);
    const int bytes = ((p.n * 2 + 15) / 16) * 16;
    const unsigned grid = static_cast<unsigned>(p.m);
    const int threads = p.n >= 8192 ? 512 : p.n >= 2048 ? 256 : 128;  // short rows: more blocks per SM instead
    static std::atomic<uint64_t> configured[3] = {{0}, {0}, {0}};
    if (aligned) {
      opt_in_smem_once(configured[2], reinterpret_cast<const void*>(&layernorm_block_staged_kernel<BF16, 8>), 2 * kStagedMaxElems);
      ::b200ait::count_launch(), layernorm_block_staged_kernel<BF16, 8><<<grid, threads, bytes, stream>>>(p);
    } else if (w2) {
      opt_in_smem_once(configured[0], reinterpret_cast<const void*>(&layernorm_block_staged_kernel<BF16, 2>), 2 * kStagedMaxElems);
      ::b200ait::count_launch(), layernorm_block_staged_kernel<BF16, 2><<<grid, threads, bytes, stream>>>(p);
    } else {
      opt_in_smem_once(configured[1], reinterpret_cast<const void*>(&layernorm_block_staged_kernel<BF16, 1>), 2 * kStagedMaxElems);
      ::b200ait::count_launch(), layernorm_block_staged_kernel<BF16, 1><<<grid, threads, bytes, stream>>>(p);
    }
  } else {
    B200AIT_REQUIRE(p.m < (1ll << 31), "layernorm: too many rows");
    const int threads = p.n >= 2048 ? 512 : (p.n >= 512 ? 256 : 128);
    ::b200ait::count_launch(), layernorm_block_kernel<BF16><<<static_cast<unsigned>(p.m), threads, 0, stream>>>(p);
  }
  B200AIT_CUDA_CHECK(cudaGetLastError());
}

// --------------------------------------------------------------------------------------- softmax
struct SoftmaxParams {
  const void* x;
  void* y;
  long long outer;  // product of dims before the reduction dim
  int k;            // reduction length
  long long inner;  // product of dims after it
};

template <int VPL, bool BF16>
__global__ void __launch_bounds__(256) softmax_warp_kernel(const SoftmaxParams p) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= p.outer) return;
  using T = typename Elem16<BF16>::T;
  const int nvec = p.k >> 3;
  const uint4* xin = reinterpret_cast<const uint4*>(static_cast<const T*>(p.x) + row * p.k);
  uint4 raw[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int v = lane + 32 * i;
    raw[i] = (v < nvec) ? ld_stream(xin + v) : make_uint4(0, 0, 0, 0);
  }
  constexpr float kLog2e = 1.4426950408889634f;
  // Only the packed row stays in registers; exp2 is evaluated once for the sum and once for the output.
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    if (lane + 32 * i < nvec) {
      float f[8];
      unpack8<BF16>(raw[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) mx = fmaxf(mx, f[j]);
    }
  }
  mx = warp_max(mx);
  const float mb = (mx == -INFINITY) ? 0.f : mx * kLog2e;
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    if (lane + 32 * i < nvec) {
      float f[8];
      unpack8<BF16>(raw[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += exp2f(f[j] * kLog2e - mb);
    }
  }
  const float inv = 1.f / warp_sum(s);
  uint4* yout = reinterpret_cast<uint4*>(static_cast<T*>(p.y) + row * p.k);
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int v = lane + 32 * i;
    if (v < nvec) {
      float f[8], o[8];
      unpack8<BF16>(raw[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = exp2f(f[j] * kLog2e - mb) * inv;
      st_stream(yout + v, pack8<BF16>(o));
    }
  }
}

// one block per (outer, inner-chunk); blockDim.x threads walk the reduction dim when inner == 1,
// otherwise each thread owns one inner index and loops over k (coalesced along inner)
// short rows the vector kernel cannot take (K not a multiple of 8, e.g. the 77 keys of a text encoder; K <= 1024):
// see layernorm_warp_scalar_kernel
template <int EPL, bool BF16>
__global__ void __launch_bounds__(256) softmax_warp_scalar_kernel(const SoftmaxParams p) {
  using E = Elem16<BF16>;
  using T = typename E::T;
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= p.outer) return;
  const T* x = static_cast<const T*>(p.x) + row * p.k;
  constexpr float kLog2e = 1.4426950408889634f;
  float f[EPL];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const int c = lane + 32 * i;
    f[i] = (c < p.k) ? E::to_float(x[c]) : -INFINITY;
    mx = fmaxf(mx, f[i]);
  }
  mx = warp_max(mx);
  const float mb = (mx == -INFINITY) ? 0.f : mx * kLog2e;
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    f[i] = (lane + 32 * i < p.k) ? exp2f(f[i] * kLog2e - mb) : 0.f;
    s += f[i];
  }
  const float inv = 1.f / warp_sum(s);
  T* y = static_cast<T*>(p.y) + row * p.k;
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const int c = lane + 32 * i;
    if (c < p.k) y[c] = E::from_float(f[i] * inv);
  }
}

// softmax over the last dim of rows wider than a warp can hold (4096 < K <= 32768, vector-aligned): see
// layernorm_wide_kernel
template <int VPT, bool BF16>
__global__ void __launch_bounds__(512) softmax_wide_kernel(const SoftmaxParams p) {
  using T = typename Elem16<BF16>::T;
  __shared__ float red[33];
  const long long row = blockIdx.x;
  const int nvec = p.k >> 3;
  const uint4* xin = reinterpret_cast<const uint4*>(static_cast<const T*>(p.x) + row * p.k);
  uint4 raw[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = static_cast<int>(threadIdx.x) + 512 * i;
    raw[i] = (v < nvec) ? ld_stream(xin + v) : make_uint4(0, 0, 0, 0);
  }
  constexpr float kLog2e = 1.4426950408889634f;
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    if (static_cast<int>(threadIdx.x) + 512 * i < nvec) {
      float f[8];
      unpack8<BF16>(raw[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) mx = fmaxf(mx, f[j]);
    }
  }
  mx = block_max(mx, red);
  const float mb = (mx == -INFINITY) ? 0.f : mx * kLog2e;
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    if (static_cast<int>(threadIdx.x) + 512 * i < nvec) {
      float f[8];
      unpack8<BF16>(raw[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += exp2f(f[j] * kLog2e - mb);
    }
  }
  const float inv = 1.f / block_sum(s, red);
  uint4* yout = reinterpret_cast<uint4*>(static_cast<T*>(p.y) + row * p.k);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = static_cast<int>(threadIdx.x) + 512 * i;
    if (v < nvec) {
      float f[8], o[8];
      unpack8<BF16>(raw[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = exp2f(f[j] * kLog2e - mb) * inv;
      st_stream(yout + v, pack8<BF16>(o));
    }
  }
}

template <bool BF16>
__global__ void __launch_bounds__(512) softmax_block_kernel(const SoftmaxParams p) {
  using E = Elem16<BF16>;
  using T = typename E::T;
  __shared__ float red[33];
  const long long row = blockIdx.x;
  const T* x = static_cast<const T*>(p.x) + row * p.k;
  T* y = static_cast<T*>(p.y) + row * p.k;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < p.k; i += blockDim.x) mx = fmaxf(mx, E::to_float(x[i]));
  mx = block_max(mx, red);
  if (mx == -INFINITY) mx = 0.f;
  float s = 0.f;
  for (int i = threadIdx.x; i < p.k; i += blockDim.x) s += __expf(E::to_float(x[i]) - mx);
  const float inv = 1.f / block_sum(s, red);
  for (int i = threadIdx.x; i < p.k; i += blockDim.x) y[i] = E::from_float(__expf(E::to_float(x[i]) - mx) * inv);
}

// The same for softmax rows (see layernorm_block_staged_kernel): one read, one write.
template <bool BF16, int W>
__global__ void __launch_bounds__(512) softmax_block_staged_kernel(const SoftmaxParams p) {
  constexpr bool W2 = W == 2;
  using E = Elem16<BF16>;
  using T = typename E::T;
  extern __shared__ __align__(16) unsigned char staged_row[];
  __shared__ float red[33];
  T* xs = reinterpret_cast<T*>(staged_row);
  const long long row = blockIdx.x;
  const T* x = static_cast<const T*>(p.x) + row * p.k;
  T* y = static_cast<T*>(p.y) + row * p.k;
  const int tid = threadIdx.x, nt = blockDim.x;
  float mx = -INFINITY;
  if (W == 8) {
    const uint4* x8 = reinterpret_cast<const uint4*>(x);
    uint4* xs8 = reinterpret_cast<uint4*>(xs);
    for (int i = tid; i < (p.k >> 3); i += nt) {
      const uint4 w = ld_stream(x8 + i);
      xs8[i] = w;
      float f[8];
      unpack8<BF16>(w, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) mx = fmaxf(mx, f[j]);
    }
  } else if (W2) {
    const uint32_t* x2 = reinterpret_cast<const uint32_t*>(x);
    uint32_t* xs2 = reinterpret_cast<uint32_t*>(xs);
    for (int i = tid; i < (p.k >> 1); i += nt) {
      const uint32_t w = __ldcs(x2 + i);
      xs2[i] = w;
      const float2 f = E::to_float2(w);
      mx = fmaxf(mx, fmaxf(f.x, f.y));
    }
  } else {
    for (int i = tid; i < p.k; i += nt) {
      const T v = x[i];
      xs[i] = v;
      mx = fmaxf(mx, E::to_float(v));
    }
  }
  mx = block_max(mx, red);  // (its barriers also publish the staged row)
  if (mx == -INFINITY) mx = 0.f;
  float s = 0.f;
  for (int i = tid; i < p.k; i += nt) s += __expf(E::to_float(xs[i]) - mx);
  const float inv = 1.f / block_sum(s, red);
  if (W == 8) {
    uint4* y8 = reinterpret_cast<uint4*>(y);
    for (int i = tid; i < (p.k >> 3); i += nt) {
      float f[8];
      unpack8<BF16>(reinterpret_cast<const uint4*>(xs)[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = __expf(f[j] - mx) * inv;
      st_stream(y8 + i, pack8<BF16>(f));
    }
  } else if (W2) {
    uint32_t* y2 = reinterpret_cast<uint32_t*>(y);
    for (int i = tid; i < (p.k >> 1); i += nt) {
      const float2 f = E::to_float2(reinterpret_cast<const uint32_t*>(xs)[i]);
      __stcs(y2 + i, E::from_float2(__expf(f.x - mx) * inv, __expf(f.y - mx) * inv));
    }
  } else {
    for (int i = tid; i < p.k; i += nt) y[i] = E::from_float(__expf(E::to_float(xs[i]) - mx) * inv);
  }
}

template <bool BF16>
__global__ void __launch_bounds__(256) softmax_strided_kernel(const SoftmaxParams p) {
  using E = Elem16<BF16>;
  using T = typename E::T;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= p.outer * p.inner) return;
  const long long o = idx / p.inner, in = idx - o * p.inner;
  const T* x = static_cast<const T*>(p.x) + o * p.k * p.inner + in;
  T* y = static_cast<T*>(p.y) + o * p.k * p.inner + in;
  float mx = -INFINITY;
  for (int i = 0; i < p.k; ++i) mx = fmaxf(mx, E::to_float(x[i * p.inner]));
  if (mx == -INFINITY) mx = 0.f;
  float s = 0.f;
  for (int i = 0; i < p.k; ++i) s += __expf(E::to_float(x[i * p.inner]) - mx);
  const float inv = 1.f / s;
  for (int i = 0; i < p.k; ++i) y[i * p.inner] = E::from_float(__expf(E::to_float(x[i * p.inner]) - mx) * inv);
}

// softmax over a non-innermost dim with a long reduction: a block (256 threads, 1024 when there are few blocks) takes
// one outer index and `ti` consecutive inner indices (coalesced), and splits the reduction dim over its thread rows, which meet in
// shared memory for the maximum and for the sum. (One thread per (outer, inner) pair, as in softmax_strided_kernel,
// leaves a [16, 16384, 8] problem with 128 threads.)
template <bool BF16>
__global__ void __launch_bounds__(1024) softmax_inner_kernel(const SoftmaxParams p, const int ti) {
  using E = Elem16<BF16>;
  using T = typename E::T;
  __shared__ float red[1024];
  const int tks = static_cast<int>(blockDim.x) / ti;
  const int tx = static_cast<int>(threadIdx.x) % ti, ty = static_cast<int>(threadIdx.x) / ti;
  const long long tiles = (p.inner + ti - 1) / ti;
  const long long o = blockIdx.x / tiles;
  const long long in = (blockIdx.x - o * tiles) * ti + tx;
  const bool valid = in < p.inner;
  const T* x = static_cast<const T*>(p.x) + o * p.k * p.inner + (valid ? in : 0);
  T* y = static_cast<T*>(p.y) + o * p.k * p.inner + (valid ? in : 0);
  constexpr float kLog2e = 1.4426950408889634f;
  float mx = -INFINITY;
  for (long long i = ty; i < p.k; i += tks) mx = fmaxf(mx, E::to_float(x[i * p.inner]));
  red[threadIdx.x] = mx;
  __syncthreads();
  for (int j = 0; j < tks; ++j) mx = fmaxf(mx, red[j * ti + tx]);
  __syncthreads();
  const float mb = (mx == -INFINITY) ? 0.f : mx * kLog2e;
  float sum = 0.f;
  for (long long i = ty; i < p.k; i += tks) sum += exp2f(E::to_float(x[i * p.inner]) * kLog2e - mb);
  red[threadIdx.x] = sum;
  __syncthreads();
  sum = 0.f;
  for (int j = 0; j < tks; ++j) sum += red[j * ti + tx];
  const float inv = 1.f / sum;
  if (!valid) return;
  for (long long i = ty; i < p.k; i += tks) y[i * p.inner] = E::from_float(exp2f(E::to_float(x[i * p.inner]) * kLog2e - mb) * inv);
}

template <bool BF16>
void softmax_launch(const SoftmaxParams& p, cudaStream_t stream) {
  if (p.inner > 1 && p.k >= 128) {
    int ti = 32;
    while (ti > 1 && ti / 2 >= p.inner) ti /= 2;  // the smallest power of two covering a narrow inner extent
    const long long blocks = p.outer * ((p.inner + ti - 1) / ti);
    B200AIT_REQUIRE(blocks < (1ll << 31), "softmax: too many blocks");
    const int threads = blocks < 2 * sm_count() ? 1024 : 256;
    ::b200ait::count_launch(), softmax_inner_kernel<BF16><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(p, ti);
  } else if (p.inner > 1) {
    const long long total = p.outer * p.inner;
    ::b200ait::count_launch(), softmax_strided_kernel<BF16><<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(p);
  } else if (p.k % 8 == 0 && p.k > 4096 && p.k <= 32768 && al16(p.x) && al16(p.y)) {
    B200AIT_REQUIRE(p.outer < (1ll << 31), "softmax: too many rows");
    const unsigned grid = static_cast<unsigned>(p.outer);
    const int vpt = (p.k / 8 + 511) / 512;
    if (vpt <= 2)
      ::b200ait::count_launch(), softmax_wide_kernel<2, BF16><<<grid, 512, 0, stream>>>(p);
    else if (vpt <= 4)
      ::b200ait::count_launch(), softmax_wide_kernel<4, BF16><<<grid, 512, 0, stream>>>(p);
    else
      ::b200ait::count_launch(), softmax_wide_kernel<8, BF16><<<grid, 512, 0, stream>>>(p);
  } else if (p.k % 8 == 0 && p.k <= 4096 && al16(p.x) && al16(p.y)) {
    const int vpl = (p.k / 8 + 31) / 32;
    const int wpb = (vpl <= 4) ? 8 : 4;
    const unsigned grid = static_cast<unsigned>((p.outer + wpb - 1) / wpb);
    const int threads = wpb * 32;
#define B200AIT_SM(V) ::b200ait::count_launch(), softmax_warp_kernel<V, BF16><<<grid, threads, 0, stream>>>(p)
    if (vpl <= 1)
      B200AIT_SM(1);
    else if (vpl <= 2)
      B200AIT_SM(2);
    else if (vpl <= 4)
      B200AIT_SM(4);
    else if (vpl <= 8)
      B200AIT_SM(8);
    else
      B200AIT_SM(16);
#undef B200AIT_SM
  } else if (p.k <= 1024) {
    const unsigned grid = static_cast<unsigned>((p.outer + 7) / 8);
    const int epl = (p.k + 31) / 32;
#define B200AIT_SMS(V) ::b200ait::count_launch(), softmax_warp_scalar_kernel<V, BF16><<<grid, 256, 0, stream>>>(p)
    if (epl <= 1) B200AIT_SMS(1); else if (epl <= 2) B200AIT_SMS(2); else if (epl <= 4) B200AIT_SMS(4);
    else if (epl <= 8) B200AIT_SMS(8); else if (epl <= 16) B200AIT_SMS(16); else B200AIT_SMS(32);
#undef B200AIT_SMS
  } else if (p.k <= kStagedMaxElems) {
    B200AIT_REQUIRE(p.outer < (1ll << 31), "softmax: too many rows");
    const bool w8 = p.k % 8 == 0 && al16(p.x) && al16(p.y), w2 = p.k % 2 == 0 && al4(p.x) && al4(p.y);
    const int bytes = ((p.k * 2 + 15) / 16) * 16;
    const unsigned grid = static_cast<unsigned>(p.outer);
    const int threads = p.k >= 8192 ? 512 : p.k >= 2048 ? 256 : 128;  // short rows: more blocks per SM instead
    static std::atomic<uint64_t> configured[3] = {{0}, {0}, {0}};
    if (w8) {
      opt_in_smem_once(configured[2], reinterpret_cast<const void*>(&softmax_block_staged_kernel<BF16, 8>), 2 * kStagedMaxElems);
      ::b200ait::count_launch(), softmax_block_staged_kernel<BF16, 8><<<grid, threads, bytes, stream>>>(p);
    } else if (w2) {
      opt_in_smem_once(configured[0], reinterpret_cast<const void*>(&softmax_block_staged_kernel<BF16, 2>), 2 * kStagedMaxElems);
      ::b200ait::count_launch(), softmax_block_staged_kernel<BF16, 2><<<grid, threads, bytes, stream>>>(p);
    } else {
      opt_in_smem_once(configured[1], reinterpret_cast<const void*>(&softmax_block_staged_kernel<BF16, 1>), 2 * kStagedMaxElems);
      ::b200ait::count_launch(), softmax_block_staged_kernel<BF16, 1><<<grid, threads, bytes, stream>>>(p);
    }
  } else {
    B200AIT_REQUIRE(p.outer < (1ll << 31), "softmax: too many rows");
    const int threads = p.k >= 2048 ? 512 : (p.k >= 256 ? 256 : (p.k >= 64 ? 64 : 32));
    ::b200ait::count_launch(), softmax_block_kernel<BF16><<<static_cast<unsigned>(p.outer), threads, 0, stream>>>(p);
  }
  B200AIT_CUDA_CHECK(cudaGetLastError());
}

}  // namespace b200ait

using namespace b200ait;

// Argument order of the reference's generated function
// (python/aitemplate/backend/cuda/layernorm_sigmoid_mul/layernorm_sigmoid_mul.py:72-83:
//  out, in, gamma, beta, m, n, eps, stream), plus row strides for strided accessors and the dtype.
B200AIT_EXPORT int b200ait_layernorm(void* out, const void* in, const void* gamma, const void* beta, int64_t m,
                                     int64_t n, float eps, int64_t in_row_stride, int64_t out_row_stride, int dtype,
                                     cudaStream_t stream) {
  return guarded("b200ait_layernorm", [&] {
    B200AIT_REQUIRE(dtype == kDTypeHalf || dtype == kDTypeBFloat16, "layernorm: dtype must be float16 or bfloat16");
    B200AIT_REQUIRE(m >= 0 && n >= 0, "layernorm: negative dimension");
    if (m == 0 || n == 0) return;
    B200AIT_REQUIRE(in && out, "layernorm: null pointer with non-zero size");
    B200AIT_REQUIRE(n < (1ll << 31), "layernorm: n exceeds int32");
    LayerNormParams p{in, gamma, beta, out, m, static_cast<int>(n), in_row_stride ? in_row_stride : n,
                      out_row_stride ? out_row_stride : n, eps};
    if (dtype == kDTypeBFloat16)
      layernorm_launch<true>(p, stream);
    else
      layernorm_launch<false>(p, stream);
  });
}

// Reference: python/aitemplate/backend/cuda/softmax/softmax.py:142-153 (in, out, dims, sm count, stream).
// The tensor is viewed as [outer, k, inner] with the reduction over k.
B200AIT_EXPORT int b200ait_softmax(const void* in, void* out, int64_t outer, int64_t k, int64_t inner, int dtype,
                                   cudaStream_t stream) {
  return guarded("b200ait_softmax", [&] {
    B200AIT_REQUIRE(dtype == kDTypeHalf || dtype == kDTypeBFloat16, "softmax: dtype must be float16 or bfloat16");
    B200AIT_REQUIRE(outer >= 0 && k >= 0 && inner >= 0, "softmax: negative dimension");
    if (outer == 0 || k == 0 || inner == 0) return;
    B200AIT_REQUIRE(in && out, "softmax: null pointer with non-zero size");
    B200AIT_REQUIRE(k < (1ll << 31), "softmax: k exceeds int32");
    SoftmaxParams p{in, out, outer, static_cast<int>(k), inner};
    if (dtype == kDTypeBFloat16)
      softmax_launch<true>(p, stream);
    else
      softmax_launch<false>(p, stream);
  });
}
