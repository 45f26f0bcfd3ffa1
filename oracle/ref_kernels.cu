// TEST INFRASTRUCTURE ONLY: C entry points over the REFERENCE's own dependency-free CUDA kernels.
//
// This file holds no kernel code. It includes, from the reference checkout given to nvcc with -I
// (<reference>/python/aitemplate/backend/cuda), the headers
//   softmax/softmax.cuh   (the softmax kernels and their launchers)
//   tensor/permute.cuh    (invokePermute)
// and exports plain C functions that call them the way the reference's generated code does:
// the softmax launcher for a row length K is the branch that
// python/aitemplate/backend/cuda/softmax/softmax.py:53-114 renders for that K (inner size 1,
// dtype half); permute is python/aitemplate/backend/cuda/tensor/permute.py:99
// (invokePermute<rank, half>). oracle/build_ref.py compiles it for sm_100a into
// oracle/_ref/libref_kernels.so. The GPU parity tests load that library, when it is present, and
// compare this repository's softmax / permute kernels with the reference's on the same device
// buffers. Nothing in the product path links or loads it.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

// permute.cuh expects what the reference's generated translation unit sets up before it
// (python/aitemplate/backend/cuda/tensor/permute.py:60-66): the CHECK_* macros of the reference's
// static/include/logging.h and, from CUTLASS (not part of the checkout), the single macro below.
#include "logging.h"
#ifndef CUTLASS_HOST_DEVICE
#define CUTLASS_HOST_DEVICE __forceinline__ __device__ __host__
#endif

#include "softmax/softmax.cuh"
#include "tensor/permute.cuh"

#define REF_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

template <int K>
int softmax_k8_small(const void* in, void* out, int64_t m, cudaStream_t s) {
  LaunchSoftmaxK8Small<half, K>(static_cast<const half*>(in), static_cast<half*>(out), (size_t)m, s);
  return 0;
}
template <int K>
int softmax_k8_middle(const void* in, void* out, int64_t m, cudaStream_t s) {
  LaunchSoftmaxK8Middle<half, K>(static_cast<const half*>(in), static_cast<half*>(out), (size_t)m, s);
  return 0;
}
template <int K>
int softmax_k1_middle(const void* in, void* out, int64_t m, cudaStream_t s) {
  LaunchSoftmaxK1Middle<half, K>(static_cast<const half*>(in), static_cast<half*>(out), (size_t)m, s);
  return 0;
}
template <int K>
int softmax_block_all_vec8(const void* in, void* out, int64_t m, cudaStream_t s) {
  using vec8 = VecTFor<half>::vec8;
  bool success = true;
  cudaError_t e = LaunchSoftmaxBlockAll<vec8, half, K>(
      reinterpret_cast<const vec8*>(in), reinterpret_cast<vec8*>(out), (size_t)m, s, &success);
  if (e != cudaSuccess) return 2;
  if (!success) {  // the fallback of softmax.py:112-114
    softmaxBlockNocache<half><<<m, 1024, 0, s>>>((half*)in, (half*)out, m, K);
  }
  return 0;
}

}  // namespace

// Row softmax over the last dim of a contiguous [m, k] fp16 matrix with the reference's kernels.
// Returns 0 on success, 1 when k is not one of the instantiated row lengths, 2 on a CUDA error.
REF_EXPORT int ref_softmax_half(const void* in, void* out, int64_t m, int k, cudaStream_t stream) {
  try {
    switch (k) {
      case 64: return softmax_k8_small<64>(in, out, m, stream);        // K % 8 == 0, K/8 <= 32
      case 128: return softmax_k8_small<128>(in, out, m, stream);
      case 384: return softmax_k8_middle<384>(in, out, m, stream);     // 32 < K/8, K <= 3840
      case 1024: return softmax_k8_middle<1024>(in, out, m, stream);
      case 4096: return softmax_block_all_vec8<4096>(in, out, m, stream);  // K > 3840
      case 77: return softmax_k1_middle<77>(in, out, m, stream);       // odd K, 32 < K <= 1408
      default: return 1;
    }
  } catch (...) {
    return 2;
  }
}

// N-D permute of a contiguous fp16 tensor with the reference's invokePermute. rank in {3, 4, 5}.
REF_EXPORT int ref_permute_half(void* dst, const void* src, int rank, const int64_t* dims, const int* perm,
                                cudaStream_t stream) {
  try {
    int64_t d[5];
    for (int i = 0; i < rank && i < 5; ++i) d[i] = dims[i];
    switch (rank) {
      case 3: invokePermute<3, half>(dst, src, d, perm, stream); return 0;
      case 4: invokePermute<4, half>(dst, src, d, perm, stream); return 0;
      case 5: invokePermute<5, half>(dst, src, d, perm, stream); return 0;
      default: return 1;
    }
  } catch (...) {
    return 2;
  }
}
