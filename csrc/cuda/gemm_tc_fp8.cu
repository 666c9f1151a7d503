// Block-scaled e4m3 instantiations of the tcgen05 GEMM template.
#include "gemm_api.h"
#include "gemm_tc.cuh"

namespace plow {
GemmArgs to_args(const PlowGemmDesc& d);

int gemm_dispatch_fp8(const PlowGemmDesc& d, cudaStream_t s) {
  const GemmArgs a = to_args(d);
#define PLOW_CASE(BN_, DUAL_, SWAP_)                                     \
  if (d.bn == BN_ && (d.dual != 0) == DUAL_ && (d.swap != 0) == SWAP_)   \
    return launch_gemm_tc<BN_, true, DUAL_, SWAP_>(a, d.ldx, d.ldw, d.w_rows, s);
  PLOW_CASE(32, false, true)
  PLOW_CASE(64, false, true)
  PLOW_CASE(128, false, true)
  PLOW_CASE(32, true, true)
  PLOW_CASE(64, true, true)
  PLOW_CASE(128, false, false)
  PLOW_CASE(64, true, false)
  PLOW_CASE(256, false, false)
  PLOW_CASE(128, true, false)
#undef PLOW_CASE
  return -2;
}
}  // namespace plow
