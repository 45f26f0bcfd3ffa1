// Fused GEMM epilogue: y = U2(B2(B1(U1(alpha*acc + bias), D0), D1)) computed in
// fp32 and rounded once to the 16-bit output type. The (U1, B1, B2, U2) tuple
// follows the reference's table of bias-elementwise GEMMs
// (python/aitemplate/backend/cuda/gemm_universal/gemm_rcr_bias_elementwise.py:34-53)
// and its activation epilogues (gemm_rcr_bias_relu.py:39-43, gemm_rcr_bias_gelu.py:39-43,
// gemm_rcr_bias_fast_gelu.py:39-43, gemm_rcr_bias_sigmoid/tanh/swish/hardswish.py).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "ptx.cuh"

namespace b200ait {

enum Unary : int {
  kUnaryIdentity = 0,
  kUnaryRelu = 1,
  kUnaryGelu = 2,      // 0.5 x (1 + erf(x / sqrt 2))
  kUnaryFastGelu = 3,  // 0.5 x (1 + tanh(sqrt(2/pi) x (1 + 0.044715 x^2)))
  kUnarySigmoid = 4,
  kUnaryTanh = 5,
  kUnarySwish = 6,      // x * sigmoid(x)
  kUnaryHardswish = 7,  // x * relu6(x + 3) / 6
};
enum Binary : int { kBinaryNone = 0, kBinaryAdd = 1, kBinaryMul = 2 };

// epilogue code = u1 | b1 << 4 | b2 << 6 | u2 << 8
__host__ __device__ constexpr int make_epilogue(int u1, int b1, int b2, int u2) {
  return u1 | (b1 << 4) | (b2 << 6) | (u2 << 8);
}
__host__ __device__ constexpr int epi_u1(int e) { return e & 15; }
__host__ __device__ constexpr int epi_b1(int e) { return (e >> 4) & 3; }
__host__ __device__ constexpr int epi_b2(int e) { return (e >> 6) & 3; }
__host__ __device__ constexpr int epi_u2(int e) { return (e >> 8) & 15; }

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float apply_unary(int u, float x) {
  switch (u) {
    case kUnaryRelu:
      return fmaxf(x, 0.f);
    case kUnaryGelu:
      return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
    case kUnaryFastGelu: {
      // 0.5 x (1 + tanh(k0 x (1 + k1 x^2))) in five floating-point instructions and one MUFU
      const float k0 = 0.7978845608028654f, k0k1 = 0.7978845608028654f * 0.044715f;
      const float u = x * fmaf(x * x, k0k1, k0);
      const float hx = 0.5f * x;
      return fmaf(hx, tanh_approx(u), hx);
    }
    case kUnarySigmoid:
      return 1.f / (1.f + __expf(-x));
    case kUnaryTanh:
      return tanh_approx(x);
    case kUnarySwish:
      return x / (1.f + __expf(-x));
    case kUnaryHardswish:
      return x * fminf(fmaxf(x + 3.f, 0.f), 6.f) * (1.f / 6.f);
    default:
      return x;
  }
}

// In-place unary over a register array; the switch is outside the loop so every
// branch is a straight unrolled loop (the code is warp-uniform).
template <int N>
__device__ __forceinline__ void apply_unary_vec(int u, float (&v)[N]) {
  switch (u) {
    case kUnaryIdentity:
      break;
    case kUnaryRelu:
#pragma unroll
      for (int i = 0; i < N; ++i) v[i] = fmaxf(v[i], 0.f);
      break;
    case kUnaryFastGelu: {
      // two elements per instruction: x^2, k0k1 x^2 + k0, times x, (MUFU tanh per element), 0.5 x, 0.5 x t + 0.5 x
      static_assert(N % 2 == 0, "packed path wants an even count");
      const uint64_t k0 = pack2(0.7978845608028654f, 0.7978845608028654f);
      const uint64_t k0k1 = pack2(0.7978845608028654f * 0.044715f, 0.7978845608028654f * 0.044715f);
      const uint64_t half2 = pack2(0.5f, 0.5f);
#pragma unroll
      for (int i = 0; i < N; i += 2) {
        const uint64_t x = pack2(v[i], v[i + 1]);
        float u0, u1;
        unpack2(mul2(x, fma2(mul2(x, x), k0k1, k0)), u0, u1);
        const uint64_t hx = mul2(x, half2);
        unpack2(fma2(hx, pack2(tanh_approx(u0), tanh_approx(u1)), hx), v[i], v[i + 1]);
      }
      break;
    }
#define B200AIT_UNARY_CASE(U)                                      \
  case U:                                                          \
    _Pragma("unroll") for (int i = 0; i < N; ++i) v[i] = apply_unary(U, v[i]); \
    break;
      // one straight loop per activation: with the code as a constant the per-element switch folds away
      B200AIT_UNARY_CASE(kUnaryGelu)
      B200AIT_UNARY_CASE(kUnarySigmoid)
      B200AIT_UNARY_CASE(kUnaryTanh)
      B200AIT_UNARY_CASE(kUnarySwish)
      B200AIT_UNARY_CASE(kUnaryHardswish)
#undef B200AIT_UNARY_CASE
    default:
      break;
  }
}

template <bool BF16>
struct Elem16;
template <>
struct Elem16<false> {
  using T = __half;
  using T2 = __half2;
  static __device__ __forceinline__ float2 to_float2(uint32_t w) {
    return __half22float2(*reinterpret_cast<const __half2*>(&w));
  }
  static __device__ __forceinline__ uint32_t from_float2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float to_float(T x) { return __half2float(x); }
  static __device__ __forceinline__ T from_float(float x) { return __float2half_rn(x); }
};
template <>
struct Elem16<true> {
  using T = __nv_bfloat16;
  using T2 = __nv_bfloat162;
  static __device__ __forceinline__ float2 to_float2(uint32_t w) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
  }
  static __device__ __forceinline__ uint32_t from_float2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float to_float(T x) { return __bfloat162float(x); }
  static __device__ __forceinline__ T from_float(float x) { return __float2bfloat16_rn(x); }
};

template <bool BF16>
__device__ __forceinline__ void unpack8(const uint4& q, float* f) {
  float2 a = Elem16<BF16>::to_float2(q.x), b = Elem16<BF16>::to_float2(q.y), c = Elem16<BF16>::to_float2(q.z),
         d = Elem16<BF16>::to_float2(q.w);
  f[0] = a.x, f[1] = a.y, f[2] = b.x, f[3] = b.y, f[4] = c.x, f[5] = c.y, f[6] = d.x, f[7] = d.y;
}
template <bool BF16>
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 q;
  q.x = Elem16<BF16>::from_float2(f[0], f[1]);
  q.y = Elem16<BF16>::from_float2(f[2], f[3]);
  q.z = Elem16<BF16>::from_float2(f[4], f[5]);
  q.w = Elem16<BF16>::from_float2(f[6], f[7]);
  return q;
}

}  // namespace b200ait
