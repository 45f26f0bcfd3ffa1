// Instantiations of the tcgen05 GEMM kernel for 256-column output tiles (see gemm_kernel.cuh).
#include "gemm_kernel.cuh"

namespace b200ait {
#define B200AIT_CASE_256(CODE)                                 \
  case (CODE):                                                  \
    launch_tc<256, false, (CODE)>(ta, tb, tout, p, grid, stream);     \
    break;
B200AIT_DEFINE_LAUNCH_TC_WIDTH(256)
#undef B200AIT_CASE_256
}  // namespace b200ait
