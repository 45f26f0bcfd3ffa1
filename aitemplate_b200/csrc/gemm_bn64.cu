// Instantiations of the tcgen05 GEMM kernel for 64-column output tiles (see gemm_kernel.cuh).
#include "gemm_kernel.cuh"

namespace b200ait {
#define B200AIT_CASE_64(CODE)                                 \
  case (CODE):                                                  \
    launch_tc<64, false, (CODE)>(ta, tb, tout, p, grid, stream);     \
    break;
B200AIT_DEFINE_LAUNCH_TC_WIDTH(64)
#undef B200AIT_CASE_64
}  // namespace b200ait
