// Instantiates the fused kernel for one occupancy: compile with -DEB_OCC=<1..8>.
#include "eb_fused.cuh"
#include "eb_launch.h"

#ifndef EB_OCC
#error "define EB_OCC (1..8)"
#endif

#define EB_CAT2(a, b) a##b
#define EB_CAT(a, b) EB_CAT2(a, b)

namespace ebk {

FusedKernel EB_CAT(fused_kernel_occ, EB_OCC)(bool timing) {
  return timing ? static_cast<FusedKernel>(eb_fused_kernel<EB_OCC, true>)
                : static_cast<FusedKernel>(eb_fused_kernel<EB_OCC, false>);
}

}  // namespace ebk
