// Instantiates the fused kernel for one occupancy: compile with -DEB_OCC=<1..8>.
#include "eb_fused.cuh"
#include "eb_launch.h"

#ifndef EB_OCC
#error "define EB_OCC (1..8)"
#endif

#define EB_CAT2(a, b) a##b
#define EB_CAT(a, b) EB_CAT2(a, b)

namespace ebk {

#define EB_FLAVOR(K, U) \
  if (kind == K && unroll == U) return static_cast<FusedKernel>(eb_fused_kernel<EB_OCC, false, K, U>);

FusedKernel EB_CAT(fused_kernel_occ, EB_OCC)(bool timing, int kind, int unroll) {
  if (timing) return static_cast<FusedKernel>(eb_fused_kernel<EB_OCC, true>);
  EB_FLAVOR(5, 0) EB_FLAVOR(5, 2) EB_FLAVOR(5, 4) EB_FLAVOR(5, 6) EB_FLAVOR(5, 8)
  EB_FLAVOR(4, 0) EB_FLAVOR(4, 2) EB_FLAVOR(4, 4) EB_FLAVOR(4, 8)
  return static_cast<FusedKernel>(eb_fused_kernel<EB_OCC, false>);
}

}  // namespace ebk
