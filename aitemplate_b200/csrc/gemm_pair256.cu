// Instantiations of the tcgen05 GEMM kernel for 256 x 256 output tiles computed by CTA pairs
// (cta_group::2, see gemm_kernel.cuh).
#include "gemm_kernel.cuh"

namespace b200ait {
#define B200AIT_CASE_PAIR(CODE)                                          \
  case (CODE):                                                           \
    launch_tc_pair<256, false, (CODE)>(ta, tb, tout, td0, p, grid, stream);   \
    break;

void launch_tc_pair256(bool bf16, const CUtensorMap& ta, const CUtensorMap& tb, const OutMaps& tout,
                       const CUtensorMap& td0, const GemmParams& p, int grid, cudaStream_t stream) {
  if (p.num_out > 1) {  // several destinations: generic epilogue instantiation only
    if (bf16)
      launch_tc_pair<256, true, -1, false, true>(ta, tb, tout, td0, p, grid, stream);
    else
      launch_tc_pair<256, false, -1, false, true>(ta, tb, tout, td0, p, grid, stream);
    return;
  }
  if (p.b_mn) {  // B stored [K, N]: generic epilogue instantiation only
    if (bf16)
      launch_tc_pair<256, true, -1, true>(ta, tb, tout, td0, p, grid, stream);
    else
      launch_tc_pair<256, false, -1, true>(ta, tb, tout, td0, p, grid, stream);
    return;
  }
  // the compile-time-epilogue kernels are lean: alpha = 1, staged TMA store, residual (if any) through staged boxes
  const bool lean_ok = p.alpha == 1.f && p.tma_store != 0 && (epi_b1(p.epilogue) == kBinaryNone || p.tma_d0 != 0);
  if (!lean_ok) {
    if (bf16)
      launch_tc_pair<256, true, -1>(ta, tb, tout, td0, p, grid, stream);
    else
      launch_tc_pair<256, false, -1>(ta, tb, tout, td0, p, grid, stream);
    return;
  }
  if (bf16) {  // the bfloat16 lean instantiations live in their own translation unit
    launch_tc_pair256_bf16_lean(ta, tb, tout, td0, p, grid, stream);
    return;
  }
  switch (p.epilogue) {
    B200AIT_FOR_EACH_FAST_EPILOGUE(B200AIT_CASE_PAIR)
    default:
      launch_tc_pair<256, false, -1>(ta, tb, tout, td0, p, grid, stream);
  }
}
#undef B200AIT_CASE_PAIR
}  // namespace b200ait

#ifdef B200AIT_GEMM_PROBE
// tuning builds only: the probe counters of the CTA-pair kernels of this translation unit
extern "C" __attribute__((visibility("default"))) int b200ait_gemm_probe_read(long long* out32) {
  if (cudaDeviceSynchronize() != cudaSuccess) return 1;
  if (cudaMemcpyFromSymbol(out32, b200ait::g_gemm_probe, sizeof(long long) * 32) != cudaSuccess) return 1;
  long long zero[32] = {};
  return cudaMemcpyToSymbol(b200ait::g_gemm_probe, zero, sizeof(zero)) == cudaSuccess ? 0 : 1;
}
#endif
