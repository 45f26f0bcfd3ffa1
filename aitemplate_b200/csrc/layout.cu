// Bit-exact data-movement kernels (concatenate, split, permute) and the element-wise chain kernel.
//
// concatenate / split replace python/aitemplate/backend/common/concatenate_common.py:147-310 and
// split_common.py:111-168: both are batches of strided 2-D copies whose vector width is the widest
// of 16/8/4/2 bytes that every pointer, row length and offset allows.
// permute replaces python/aitemplate/backend/cuda/tensor/permute.cuh:227-389 and the permute021 /
// 102 / 210 / 0213 tiled transposes (python/aitemplate/backend/common/tensor/permute*_common.py).
// elementwise replaces the generated fused_elementwise kernel
// (python/aitemplate/backend/common/elementwise_common.py:201-258) for chains of FuncEnum ops.
#include <algorithm>
#include <vector>

#include "common.h"
#include "epilogue.cuh"

namespace b200ait {

// ------------------------------------------------------------------------- strided 2-D copy batch
constexpr int kMaxCopyJobs = 32;
struct CopyJob {
  const uint8_t* src;
  uint8_t* dst;
  long long row_vecs;        // vectors per row
  long long src_row_stride;  // bytes
  long long dst_row_stride;  // bytes
};
struct CopyBatch {
  CopyJob job[kMaxCopyJobs];
  long long rows;
};

template <typename V>
__global__ void __launch_bounds__(256) copy2d_kernel(const CopyBatch batch) {
  const CopyJob j = batch.job[blockIdx.y];
  const long long total = batch.rows * j.row_vecs;
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
  // four independent loads go out before the first store: the copy is bound by the bytes in flight per SM
  constexpr int kUnroll = 4;
  for (long long i0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total; i0 += kUnroll * step) {
    V v[kUnroll];
    long long dst_off[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long long i = i0 + u * step;
      if (i < total) {
        const long long r = i / j.row_vecs, c = i - r * j.row_vecs;
        v[u] = __ldcs(reinterpret_cast<const V*>(j.src + r * j.src_row_stride + c * sizeof(V)));
        dst_off[u] = r * j.dst_row_stride + c * sizeof(V);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      if (i0 + u * step < total) *reinterpret_cast<V*>(j.dst + dst_off[u]) = v[u];
  }
}

struct HostCopy {
  const void* src;
  void* dst;
  long long row_bytes, src_row_stride, dst_row_stride;
};

void run_copies(const std::vector<HostCopy>& copies, long long rows, cudaStream_t stream) {
  if (rows == 0) return;
  int vec = 16;
  for (const auto& c : copies) {
    if (c.row_bytes == 0) continue;
    const unsigned long long bits = reinterpret_cast<uintptr_t>(c.src) | reinterpret_cast<uintptr_t>(c.dst) |
                                    static_cast<unsigned long long>(c.row_bytes) |
                                    static_cast<unsigned long long>(c.src_row_stride) |
                                    static_cast<unsigned long long>(c.dst_row_stride);
    while (vec > 1 && (bits & (vec - 1))) vec >>= 1;
  }
  size_t i = 0;
  while (i < copies.size()) {
    CopyBatch b{};
    b.rows = rows;
    int n = 0;
    long long max_vecs = 0;
    for (; i < copies.size() && n < kMaxCopyJobs; ++i) {
      const auto& c = copies[i];
      if (c.row_bytes == 0) continue;
      b.job[n].src = static_cast<const uint8_t*>(c.src);
      b.job[n].dst = static_cast<uint8_t*>(c.dst);
      b.job[n].row_vecs = c.row_bytes / vec;
      b.job[n].src_row_stride = c.src_row_stride;
      b.job[n].dst_row_stride = c.dst_row_stride;
      max_vecs = std::max(max_vecs, b.job[n].row_vecs * rows);
      ++n;
    }
    if (n == 0) break;
    const long long per_block = 256 * 8;
    const unsigned gx = static_cast<unsigned>(std::min<long long>((max_vecs + per_block - 1) / per_block, 148 * 16));
    dim3 grid(std::max(gx, 1u), n);
    switch (vec) {
      case 16: ::b200ait::count_launch(), copy2d_kernel<uint4><<<grid, 256, 0, stream>>>(b); break;
      case 8: ::b200ait::count_launch(), copy2d_kernel<uint2><<<grid, 256, 0, stream>>>(b); break;
      case 4: ::b200ait::count_launch(), copy2d_kernel<uint32_t><<<grid, 256, 0, stream>>>(b); break;
      case 2: ::b200ait::count_launch(), copy2d_kernel<uint16_t><<<grid, 256, 0, stream>>>(b); break;
      default: ::b200ait::count_launch(), copy2d_kernel<uint8_t><<<grid, 256, 0, stream>>>(b); break;
    }
    B200AIT_CUDA_CHECK(cudaGetLastError());
  }
}

// ----------------------------------------------------------------------------------------- permute
constexpr int kMaxRank = 8;
struct PermuteParams {
  const uint8_t* src;
  uint8_t* dst;
  int rank;                       // of the simplified problem (in units of vectors on the last dim)
  long long out_dims[kMaxRank];   // output extents
  long long in_strides[kMaxRank]; // input stride (in vectors / elements) of each output dim
  long long total;
};

// I: type of the index arithmetic. 32-bit when every index fits (a 64-bit division costs several times a 32-bit
// one, and a thread does one per dimension for each 16-byte vector it moves).
template <typename V, typename I>
__global__ void __launch_bounds__(256) permute_gather_kernel(const PermuteParams p) {
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.total; i += step) {
    I rem = static_cast<I>(i), off = 0;
#pragma unroll
    for (int d = kMaxRank - 1; d >= 0; --d) {
      if (d < p.rank) {
        const I dim = static_cast<I>(p.out_dims[d]);
        const I q = rem / dim;
        off += (rem - q * dim) * static_cast<I>(p.in_strides[d]);
        rem = q;
      }
    }
    reinterpret_cast<V*>(p.dst)[i] = reinterpret_cast<const V*>(p.src)[off];
  }
}

// batched [R, C] -> [C, R] transpose of 16-bit or 32-bit elements through shared memory
template <typename V>
__global__ void __launch_bounds__(256) transpose_kernel(const V* __restrict__ src, V* __restrict__ dst, long long R,
                                                        long long C) {
  __shared__ V tile[32][33];
  const long long b = blockIdx.z;
  const V* s = src + b * R * C;
  V* d = dst + b * R * C;
  const long long r0 = static_cast<long long>(blockIdx.y) * 32, c0 = static_cast<long long>(blockIdx.x) * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long r = r0 + ty + i * 8, c = c0 + tx;
    if (r < R && c < C) tile[ty + i * 8][tx] = s[r * C + c];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long c = c0 + ty + i * 8, r = r0 + tx;
    if (r < R && c < C) d[c * R + r] = tile[tx][ty + i * 8];
  }
}

// The same transpose for 16-bit elements with even R and C: 64 x 64 tiles moved with 32-bit accesses, so that a
// warp reads and writes full 128-byte lines (the 32 x 32 kernel above moves 64-byte half lines of 16-bit data).
__global__ void __launch_bounds__(256) transpose16_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst,
                                                          long long R, long long C) {
  __shared__ __align__(4) uint16_t tile[64][66];
  const long long b = blockIdx.z;
  const uint16_t* s = src + b * R * C;
  uint16_t* d = dst + b * R * C;
  const long long r0 = static_cast<long long>(blockIdx.y) * 64, c0 = static_cast<long long>(blockIdx.x) * 64;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = ty + i * 8;
    const long long r = r0 + row, c = c0 + 2 * tx;
    if (r < R && c < C)
      *reinterpret_cast<uint32_t*>(&tile[row][2 * tx]) = __ldcs(reinterpret_cast<const uint32_t*>(s + r * C + c));
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int oc = ty + i * 8;  // column of the tile = row of the output
    const long long c = c0 + oc, r = r0 + 2 * tx;
    if (c < C && r < R) {
      const uint32_t w = static_cast<uint32_t>(tile[2 * tx][oc]) | (static_cast<uint32_t>(tile[2 * tx + 1][oc]) << 16);
      *reinterpret_cast<uint32_t*>(d + c * R + r) = w;
    }
  }
}

void permute_run(const void* src, void* dst, const int64_t* in_shape, const int64_t* perm, int rank, int elem_size,
                 cudaStream_t stream) {
  B200AIT_REQUIRE(rank >= 1 && rank <= kMaxRank, "permute: rank must be in [1, 8]");
  B200AIT_REQUIRE(elem_size == 1 || elem_size == 2 || elem_size == 4 || elem_size == 8, "permute: bad element size");
  bool seen[kMaxRank] = {};
  long long total = 1;
  for (int i = 0; i < rank; ++i) {
    B200AIT_REQUIRE(perm[i] >= 0 && perm[i] < rank && !seen[perm[i]], "permute: dims is not a permutation");
    seen[perm[i]] = true;
    B200AIT_REQUIRE(in_shape[i] >= 0, "permute: negative dimension");
    total *= in_shape[i];
  }
  if (total == 0) return;
  B200AIT_REQUIRE(src && dst, "permute: null pointer with non-zero size");
  // input strides in elements
  long long in_stride[kMaxRank];
  long long s = 1;
  for (int i = rank - 1; i >= 0; --i) {
    in_stride[i] = s;
    s *= in_shape[i];
  }
  // output dims with their input strides; drop size-1 dims, merge dims that stay adjacent
  std::vector<long long> od, os;
  for (int i = 0; i < rank; ++i) {
    const long long ext = in_shape[perm[i]], str = in_stride[perm[i]];
    if (ext == 1) continue;
    if (!od.empty() && os.back() == str * ext) {
      od.back() *= ext;
      os.back() = str;
    } else {
      od.push_back(ext);
      os.push_back(str);
    }
  }
  if (od.empty()) {
    od.push_back(1);
    os.push_back(1);
  }
  const int r = static_cast<int>(od.size());
  if (r == 1) {  // identity
    B200AIT_CUDA_CHECK(cudaMemcpyAsync(dst, src, static_cast<size_t>(total) * elem_size, cudaMemcpyDeviceToDevice, stream));
    return;
  }
  // batched 2-D transpose: [B, R, C] -> [B, C, R]
  if ((elem_size == 2 || elem_size == 4) && ((r == 2 && os[0] == 1 && os[1] == od[0]) ||
                                            (r == 3 && os[1] == 1 && os[2] == od[1] && os[0] == od[1] * od[2]))) {
    const long long B = (r == 3) ? od[0] : 1, C = od[r - 2], R = od[r - 1];
    if (B < 65536 && (R + 31) / 32 < 65536) {
      dim3 grid(static_cast<unsigned>((C + 31) / 32), static_cast<unsigned>((R + 31) / 32), static_cast<unsigned>(B));
      if (elem_size == 2 && R % 2 == 0 && C % 2 == 0 && R >= 64 && C >= 64 &&
          (reinterpret_cast<uintptr_t>(src) & 3) == 0 && (reinterpret_cast<uintptr_t>(dst) & 3) == 0) {
        dim3 grid64(static_cast<unsigned>((C + 63) / 64), static_cast<unsigned>((R + 63) / 64), static_cast<unsigned>(B));
        ::b200ait::count_launch(), transpose16_kernel<<<grid64, 256, 0, stream>>>(static_cast<const uint16_t*>(src), static_cast<uint16_t*>(dst), R, C);
      } else if (elem_size == 2)
        ::b200ait::count_launch(), transpose_kernel<uint16_t><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(src), static_cast<uint16_t*>(dst), R, C);
      else
        ::b200ait::count_launch(), transpose_kernel<uint32_t><<<grid, 256, 0, stream>>>(static_cast<const uint32_t*>(src), static_cast<uint32_t*>(dst), R, C);
      B200AIT_CUDA_CHECK(cudaGetLastError());
      return;
    }
  }
  // gather with the widest vector the preserved innermost run allows
  int vec = elem_size;
  if (os[r - 1] == 1) {
    const long long run_bytes = od[r - 1] * elem_size;
    unsigned long long bits = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) |
                              static_cast<unsigned long long>(run_bytes);
    for (int i = 0; i < r - 1; ++i) bits |= static_cast<unsigned long long>(os[i] * elem_size);
    vec = 16;
    while (vec > elem_size && (bits & (vec - 1))) vec >>= 1;
  }
  const int epv = vec / elem_size;  // elements per vector
  PermuteParams p{};
  p.src = static_cast<const uint8_t*>(src);
  p.dst = static_cast<uint8_t*>(dst);
  p.rank = r;
  for (int i = 0; i < r; ++i) {
    p.out_dims[i] = od[i];
    p.in_strides[i] = (epv > 1 && i < r - 1) ? os[i] / epv : os[i];
  }
  if (epv > 1) p.out_dims[r - 1] = od[r - 1] / epv;
  p.total = total / epv;
  const unsigned grid = static_cast<unsigned>(std::min<long long>((p.total + 255) / 256, 148 * 32));
  const bool small = total < (1ll << 31);  // element count bounds every index and every input offset
#define B200AIT_GATHER(V)                                                   \
  do {                                                                      \
    if (small)                                                              \
      ::b200ait::count_launch(), permute_gather_kernel<V, uint32_t><<<grid, 256, 0, stream>>>(p);      \
    else                                                                    \
      ::b200ait::count_launch(), permute_gather_kernel<V, long long><<<grid, 256, 0, stream>>>(p);     \
  } while (0)
  switch (vec) {
    case 16: B200AIT_GATHER(uint4); break;
    case 8: B200AIT_GATHER(uint2); break;
    case 4: B200AIT_GATHER(uint32_t); break;
    case 2: B200AIT_GATHER(uint16_t); break;
    default: B200AIT_GATHER(uint8_t); break;
  }
#undef B200AIT_GATHER
  B200AIT_CUDA_CHECK(cudaGetLastError());
}

// ------------------------------------------------------------------------------ element-wise chain
// acc = in[0]; for each step: acc = op(acc, operand) where the operand is another input tensor,
// a scalar constant, or absent (unary). Inputs broadcast against the output shape.
constexpr int kMaxEwInputs = 6;
constexpr int kMaxEwSteps = 12;
enum EwOp : int {
  kEwAdd = 1, kEwSub = 2, kEwMul = 3, kEwDiv = 4, kEwRsub = 5, kEwRdiv = 6, kEwMax = 7, kEwMin = 8,
  kEwRelu = 16, kEwGelu = 17, kEwFastGelu = 18, kEwSigmoid = 19, kEwTanh = 20, kEwSilu = 21, kEwNeg = 22,
  kEwAbs = 23, kEwExp = 24, kEwSqrt = 25, kEwHardswish = 26,
};
struct EwParams {
  const void* in[kMaxEwInputs];
  // input addressing: kind 0 = same linear index as the output, 1 = single element,
  // 2 = periodic (linear index % period), 3 = general strides over out_dims
  int kind[kMaxEwInputs];
  long long period[kMaxEwInputs];
  long long strides[kMaxEwInputs][kMaxRank];
  int rank;
  long long out_dims[kMaxRank];
  void* out;
  long long total;
  int nsteps;
  int op[kMaxEwSteps];
  int operand[kMaxEwSteps];  // input index, -1 = constant, -2 = none
  float constant[kMaxEwSteps];
  int vec_ok;
};

__device__ __forceinline__ float ew_apply(int op, float a, float b) {
  switch (op) {
    case kEwAdd: return a + b;
    case kEwSub: return a - b;
    case kEwMul: return a * b;
    case kEwDiv: return a / b;
    case kEwRsub: return b - a;
    case kEwRdiv: return b / a;
    case kEwMax: return fmaxf(a, b);
    case kEwMin: return fminf(a, b);
    case kEwRelu: return fmaxf(a, 0.f);
    case kEwGelu: return apply_unary(kUnaryGelu, a);
    case kEwFastGelu: return apply_unary(kUnaryFastGelu, a);
    case kEwSigmoid: return apply_unary(kUnarySigmoid, a);
    case kEwTanh: return tanhf(a);
    case kEwSilu: return apply_unary(kUnarySwish, a);
    case kEwNeg: return -a;
    case kEwAbs: return fabsf(a);
    case kEwExp: return __expf(a);
    case kEwSqrt: return sqrtf(a);
    case kEwHardswish: return apply_unary(kUnaryHardswish, a);
    default: return a;
  }
}

__device__ __forceinline__ long long ew_index(const EwParams& p, int i, long long lin) {
  switch (p.kind[i]) {
    case 0: return lin;
    case 1: return 0;
    case 2: return lin % p.period[i];
    default: {
      long long rem = lin, off = 0;
      for (int d = p.rank - 1; d >= 0; --d) {
        const long long q = rem / p.out_dims[d];
        off += (rem - q * p.out_dims[d]) * p.strides[i][d];
        rem = q;
      }
      return off;
    }
  }
}

template <bool BF16>
__global__ void __launch_bounds__(256) elementwise_kernel(const EwParams p) {
  using E = Elem16<BF16>;
  using T = typename E::T;
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
  if (p.vec_ok) {
    const long long nvec = p.total >> 3;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += step) {
      const long long lin = i << 3;
      float acc[8];
      {
        const T* src = static_cast<const T*>(p.in[0]);
        if (p.kind[0] == 1) {
          const float s = E::to_float(src[0]);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = s;
        } else {
          unpack8<BF16>(*reinterpret_cast<const uint4*>(src + ew_index(p, 0, lin)), acc);
        }
      }
      for (int s = 0; s < p.nsteps; ++s) {
        float b[8];
        const int o = p.operand[s];
        if (o >= 0) {
          const T* src = static_cast<const T*>(p.in[o]);
          if (p.kind[o] == 1) {
            const float c = E::to_float(src[0]);
#pragma unroll
            for (int j = 0; j < 8; ++j) b[j] = c;
          } else {
            unpack8<BF16>(*reinterpret_cast<const uint4*>(src + ew_index(p, o, lin)), b);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) b[j] = p.constant[s];
        }
        const int op = p.op[s];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = ew_apply(op, acc[j], b[j]);
      }
      *reinterpret_cast<uint4*>(static_cast<T*>(p.out) + lin) = pack8<BF16>(acc);
    }
  } else {
    for (long long lin = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; lin < p.total; lin += step) {
      float acc = E::to_float(static_cast<const T*>(p.in[0])[ew_index(p, 0, lin)]);
      for (int s = 0; s < p.nsteps; ++s) {
        const int o = p.operand[s];
        const float b = (o >= 0) ? E::to_float(static_cast<const T*>(p.in[o])[ew_index(p, o, lin)]) : p.constant[s];
        acc = ew_apply(p.op[s], acc, b);
      }
      static_cast<T*>(p.out)[lin] = E::from_float(acc);
    }
  }
}

}  // namespace b200ait

using namespace b200ait;

// Concatenate along `concat_dim`. `inputs` / `input_shapes` list ALL inputs; an input whose mask is
// false is assumed to be in place already (written there by a strided producer) and is skipped,
// but still occupies its slice of the output. output_shape[rank] is written.
// Reference: python/aitemplate/backend/common/concatenate_common.py:29-48.
B200AIT_EXPORT int b200ait_concatenate(void* output, int64_t* output_shape, const void* const* inputs,
                                       const int64_t* const* input_shapes, const uint8_t* input_masks,
                                       int64_t concat_dim, int64_t rank, int64_t num_inputs, int64_t elem_size,
                                       cudaStream_t stream) {
  return guarded("b200ait_concatenate", [&] {
    B200AIT_REQUIRE(rank >= 1 && rank <= 16 && concat_dim >= 0 && concat_dim < rank, "concatenate: bad rank or dim");
    B200AIT_REQUIRE(num_inputs >= 1 && inputs && input_shapes, "concatenate: needs at least one input");
    long long outer = 1, inner = 1, cat = 0;
    for (int64_t d = 0; d < concat_dim; ++d) outer *= input_shapes[0][d];
    for (int64_t d = concat_dim + 1; d < rank; ++d) inner *= input_shapes[0][d];
    for (int64_t i = 0; i < num_inputs; ++i) {
      for (int64_t d = 0; d < rank; ++d)
        if (d != concat_dim)
          B200AIT_REQUIRE(input_shapes[i][d] == input_shapes[0][d], "concatenate: inputs disagree outside the concat dim");
      B200AIT_REQUIRE(input_shapes[i][concat_dim] >= 0, "concatenate: negative dimension");
      cat += input_shapes[i][concat_dim];
    }
    if (output_shape) {
      for (int64_t d = 0; d < rank; ++d) output_shape[d] = (d == concat_dim) ? cat : input_shapes[0][d];
    }
    if (outer * inner * cat == 0) return;
    B200AIT_REQUIRE(output, "concatenate: null output with non-zero size");
    const long long out_row = cat * inner * elem_size;
    std::vector<HostCopy> copies;
    long long off = 0;
    for (int64_t i = 0; i < num_inputs; ++i) {
      const long long row = input_shapes[i][concat_dim] * inner * elem_size;
      if ((!input_masks || input_masks[i]) && row > 0) {
        B200AIT_REQUIRE(inputs[i], "concatenate: null input with non-zero size");
        copies.push_back({inputs[i], static_cast<uint8_t*>(output) + off, row, row, out_row});
      }
      off += row;
    }
    run_copies(copies, outer, stream);
  });
}

// Split along `split_dim` into pieces of `split_sizes`. An output whose mask is false is skipped.
// Reference: python/aitemplate/backend/common/split_common.py:21-40.
B200AIT_EXPORT int b200ait_split(void* const* outputs, const uint8_t* output_masks, const void* input,
                                 const int64_t* input_shape, int64_t num_splits, const int64_t* split_sizes,
                                 int64_t split_dim, int64_t rank, int64_t elem_size, cudaStream_t stream) {
  return guarded("b200ait_split", [&] {
    B200AIT_REQUIRE(rank >= 1 && rank <= 16 && split_dim >= 0 && split_dim < rank, "split: bad rank or dim");
    B200AIT_REQUIRE(num_splits >= 1 && outputs && split_sizes && input_shape, "split: needs at least one output");
    long long outer = 1, inner = 1, sum = 0;
    for (int64_t d = 0; d < split_dim; ++d) outer *= input_shape[d];
    for (int64_t d = split_dim + 1; d < rank; ++d) inner *= input_shape[d];
    for (int64_t i = 0; i < num_splits; ++i) {
      B200AIT_REQUIRE(split_sizes[i] >= 0, "split: negative split size");
      sum += split_sizes[i];
    }
    B200AIT_REQUIRE(sum == input_shape[split_dim], "split: sizes do not add up to the split dimension");
    if (outer * inner * sum == 0) return;
    B200AIT_REQUIRE(input, "split: null input with non-zero size");
    const long long in_row = sum * inner * elem_size;
    std::vector<HostCopy> copies;
    long long off = 0;
    for (int64_t i = 0; i < num_splits; ++i) {
      const long long row = split_sizes[i] * inner * elem_size;
      if ((!output_masks || output_masks[i]) && row > 0) {
        B200AIT_REQUIRE(outputs[i], "split: null output with non-zero size");
        copies.push_back({static_cast<const uint8_t*>(input) + off, outputs[i], row, in_row, row});
      }
      off += row;
    }
    run_copies(copies, outer, stream);
  });
}

// out = in.permute(dims).contiguous(). Reference: python/aitemplate/backend/cuda/tensor/permute.cuh:227-389.
B200AIT_EXPORT int b200ait_permute(const void* input, void* output, const int64_t* input_shape, const int64_t* dims,
                                   int64_t rank, int64_t elem_size, cudaStream_t stream) {
  return guarded("b200ait_permute", [&] {
    B200AIT_REQUIRE(input_shape && dims, "permute: null shape or dims");
    permute_run(input, output, input_shape, dims, static_cast<int>(rank), static_cast<int>(elem_size), stream);
  });
}

// Element-wise chain with broadcasting: acc = inputs[0]; acc = ops[s](acc, operand[s]) for each step.
// input_shapes are right-aligned against out_shape (each has `rank` entries, 1 where broadcast).
// operand_index[s]: >= 0 input tensor, -1 the scalar constants[s], -2 none (unary op).
// Reference: python/aitemplate/backend/common/elementwise_common.py:201-264.
B200AIT_EXPORT int b200ait_elementwise(void* output, const int64_t* out_shape, int64_t rank,
                                       const void* const* inputs, const int64_t* const* input_shapes,
                                       int64_t num_inputs, const int* ops, const int* operand_index,
                                       const float* constants, int64_t num_steps, int dtype, cudaStream_t stream) {
  return guarded("b200ait_elementwise", [&] {
    B200AIT_REQUIRE(dtype == kDTypeHalf || dtype == kDTypeBFloat16, "elementwise: dtype must be float16 or bfloat16");
    B200AIT_REQUIRE(rank >= 0 && rank <= kMaxRank, "elementwise: rank must be <= 8");
    B200AIT_REQUIRE(num_inputs >= 1 && num_inputs <= kMaxEwInputs, "elementwise: 1..6 inputs");
    B200AIT_REQUIRE(num_steps >= 0 && num_steps <= kMaxEwSteps, "elementwise: at most 12 steps");
    EwParams p{};
    p.rank = static_cast<int>(rank);
    p.total = 1;
    for (int d = 0; d < rank; ++d) {
      B200AIT_REQUIRE(out_shape[d] >= 0, "elementwise: negative dimension");
      p.out_dims[d] = out_shape[d];
      p.total *= out_shape[d];
    }
    if (p.total == 0) return;
    B200AIT_REQUIRE(output, "elementwise: null output");
    bool vec = (p.total % 8 == 0) && ((reinterpret_cast<uintptr_t>(output) & 15) == 0);
    for (int i = 0; i < num_inputs; ++i) {
      B200AIT_REQUIRE(inputs[i], "elementwise: null input");
      p.in[i] = inputs[i];
      long long numel = 1, s = 1;
      long long strides[kMaxRank];
      for (int d = static_cast<int>(rank) - 1; d >= 0; --d) {
        const long long e = input_shapes[i][d];
        B200AIT_REQUIRE(e == out_shape[d] || e == 1, "elementwise: input is not broadcastable to the output");
        strides[d] = (e == 1 && out_shape[d] != 1) ? 0 : s;
        s *= e;
        numel *= e;
      }
      for (int d = 0; d < rank; ++d) p.strides[i][d] = strides[d];
      // classify
      if (numel == p.total) {
        p.kind[i] = 0;
      } else if (numel == 1) {
        p.kind[i] = 1;
      } else {
        // periodic when the input covers exactly the trailing dims
        int first = 0;
        while (first < rank && input_shapes[i][first] == 1) ++first;
        bool trailing = true;
        for (int d = first; d < rank; ++d) trailing = trailing && (input_shapes[i][d] == out_shape[d]);
        if (trailing) {
          p.kind[i] = 2;
          p.period[i] = numel;
          vec = vec && (numel % 8 == 0);
        } else {
          p.kind[i] = 3;
          // a vector of 8 must stay inside one contiguous, non-broadcast innermost run
          vec = vec && rank > 0 && (out_shape[rank - 1] % 8 == 0) && strides[rank - 1] == 1;
          for (int d = 0; d < rank - 1; ++d) vec = vec && (strides[d] % 8 == 0);
        }
      }
      if (p.kind[i] != 1) vec = vec && ((reinterpret_cast<uintptr_t>(inputs[i]) & 15) == 0);
    }
    p.out = output;
    p.nsteps = static_cast<int>(num_steps);
    for (int s = 0; s < num_steps; ++s) {
      p.op[s] = ops[s];
      p.operand[s] = operand_index[s];
      p.constant[s] = constants ? constants[s] : 0.f;
      B200AIT_REQUIRE(p.operand[s] < num_inputs, "elementwise: operand index out of range");
      B200AIT_REQUIRE(!(ops[s] < 16 && p.operand[s] == -2), "elementwise: binary op without an operand");
    }
    p.vec_ok = vec ? 1 : 0;
    const long long work = vec ? p.total / 8 : p.total;
    const unsigned grid = static_cast<unsigned>(std::min<long long>((work + 255) / 256, 148 * 32));
    if (dtype == kDTypeBFloat16)
      ::b200ait::count_launch(), elementwise_kernel<true><<<grid, 256, 0, stream>>>(p);
    else
      ::b200ait::count_launch(), elementwise_kernel<false><<<grid, 256, 0, stream>>>(p);
    B200AIT_CUDA_CHECK(cudaGetLastError());
  });
}
