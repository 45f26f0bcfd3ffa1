// Instantiations of the tcgen05 GEMM kernel for 128-column output tiles (see gemm_kernel.cuh).
#include "gemm_kernel.cuh"

namespace b200ait {
#define B200AIT_CASE_128(CODE)                                 \
  case (CODE):                                                  \
    launch_tc<128, false, (CODE)>(ta, tb, tout, p, grid, stream);     \
    break;
B200AIT_DEFINE_LAUNCH_TC_WIDTH(128)
#undef B200AIT_CASE_128
}  // namespace b200ait
