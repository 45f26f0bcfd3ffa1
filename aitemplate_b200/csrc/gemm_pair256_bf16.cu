// bfloat16 instantiations of the lean CTA-pair kernels (compile-time epilogues, see gemm_kernel.cuh).
#include "gemm_kernel.cuh"

namespace b200ait {
#define B200AIT_CASE_PAIR_BF16(CODE)                                        \
  case (CODE):                                                              \
    launch_tc_pair<256, true, (CODE)>(ta, tb, tout, td0, p, grid, stream);  \
    break;

// caller has checked the lean conditions (alpha = 1, staged store, staged residual boxes)
void launch_tc_pair256_bf16_lean(const CUtensorMap& ta, const CUtensorMap& tb, const OutMaps& tout,
                                 const CUtensorMap& td0, const GemmParams& p, int grid, cudaStream_t stream) {
  switch (p.epilogue) {
    B200AIT_FOR_EACH_FAST_EPILOGUE(B200AIT_CASE_PAIR_BF16)
    default:
      launch_tc_pair<256, true, -1>(ta, tb, tout, td0, p, grid, stream);
  }
}
#undef B200AIT_CASE_PAIR_BF16
}  // namespace b200ait
